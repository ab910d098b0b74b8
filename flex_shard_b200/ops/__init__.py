"""Hand-written sm_100a kernels (through a C ABI) and their autograd wrappers."""
from . import _lib
from ._lib import NativeError, available, check_status, launch_count
from .gemm import gemm, linear
