"""aussm_b200: B200 (sm_100a) implementation of the AUSSM selective-scan operators.

``aussm_b200.ops`` mirrors the reference's ``extension_cpp.ops`` front end and
calls hand-written CUDA kernels through the C ABI of ``libaussm_b200.so``
(``include/aussm_b200.h``).  Build the library with ``python -m aussm_b200.build``.
"""
from . import _lib, ops, s6, variants
from .ops import (device_status, install_as_extension_cpp, scan_unitary, ssm_adaptive_interface,
                  ssm_adaptive_unitary)

__version__ = "0.1.0"
from .s6 import selective_scan_fn
from .variants import project, scan_complex, ssm_adaptive_complex, ssm_adaptive_preal
from .host import HostBatchStep, bind_process_to_gpu_cpus
from .linear import SplitLinear, split_linear

__all__ = ["ops", "HostBatchStep", "SplitLinear", "split_linear", "selective_scan_fn", "scan_complex", "project", "ssm_adaptive_complex", "ssm_adaptive_preal", "ssm_adaptive_interface", "ssm_adaptive_unitary", "scan_unitary", "install_as_extension_cpp",
           "device_status"]
