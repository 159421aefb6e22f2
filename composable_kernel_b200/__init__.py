"""B200 (sm_100a) dense-contraction kernels behind Composable Kernel's device-operation API.

``composable_kernel_b200.capi`` binds the C ABI of include/ckb200.h; ``device_op`` mirrors the
reference's DeviceGemm / DeviceGemmMultipleD / DeviceGroupedGemm / DeviceConvFwd call sequence.
The compiled library (lib/libckb200.so) is built by ``python -m composable_kernel_b200.build``.
"""
from . import capi  # noqa: F401
from .device_op import *  # noqa: F401,F403

__version__ = "0.1.0"
