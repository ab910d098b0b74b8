"""Hand-written sm_100a kernels (through a C ABI) and their autograd wrappers."""
from . import _lib
from ._lib import NativeError, available, check_status, launch_count, poll_status
from .gemm import gemm, linear
