"""Training protocols (``python -m stacr reproduce ...``): named profiles in ``configs/protocols.json``."""
