"""INSTANT comparator: activations and output gradients of a linear layer projected on calibrated token subspaces.

For a linear layer with input ``X [batch, tokens, features]`` the method keeps ``Pᵀ X`` (``k`` rows per sample
instead of ``tokens``), where ``P [tokens, k]`` spans the leading eigenvectors of the batch-averaged ``X Xᵀ``
measured during a short calibration, and propagates the input gradient through ``Q Qᵀ dY`` with ``Q`` calibrated
the same way on ``dY dYᵀ``.  Both subspaces are re-calibrated every ``calib_iter`` steps.

Parity: comparators/instant/ (``custom_op.py``, ``svd.py``, ``model.py``, ``callback.py``, ``dataset_prep.py``,
``utils.py``, ``train_language.py``, ``train_classification.py``).  The method is that of the public INSTANT
release named below; the implementation here is this framework's own and drives the in-tree models with a plain
training loop instead of a ``transformers.Trainer``.
"""

UPSTREAM = "https://github.com/hieu-trannn/INSTANT"
REVISION = "8a04bd43c19cc52984a49fb1b7fd1dae14fb2ffc"

from .callback import Calibrator  # noqa: E402
from .custom_op import InstantLinear, LinearSVDOp, register_filter, wrap_linear_compression_layer  # noqa: E402
from .model import (  # noqa: E402
    convert_conv1d_to_linear, disable_compression, enable_compression, freeze_layers, get_svd_layers, update_compression,
)
from .svd import SVD_expected_value, energy_basis  # noqa: E402

__all__ = [
    "UPSTREAM", "REVISION", "Calibrator", "InstantLinear", "LinearSVDOp", "register_filter", "wrap_linear_compression_layer",
    "convert_conv1d_to_linear", "disable_compression", "enable_compression", "freeze_layers", "get_svd_layers",
    "update_compression", "SVD_expected_value", "energy_basis",
]
