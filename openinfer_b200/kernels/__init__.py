"""Hand-written CUDA kernels for sm_100a and their Python wrappers."""
from .lib import KernelError, load  # noqa: F401
