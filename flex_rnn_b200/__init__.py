"""flex_rnn_b200: B200 (sm_100a) backend for flex_rnn step functions."""
from .jit import jit, simplified_naive  # noqa: F401
from .check_grad import check_grad, benchmark  # noqa: F401

__version__ = "0.1"
