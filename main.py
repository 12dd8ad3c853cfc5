"""``python main.py ...`` is ``python -m stacr train ...``."""

import sys

from stacr_b200.cli import main

if __name__ == "__main__":
    main(["train", *sys.argv[1:]])
