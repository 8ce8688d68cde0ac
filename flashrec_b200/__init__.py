"""flashrec_b200 — sm_100a kernels for the quantized SID decode step.

The package mirrors, name for name, the kernel- and layer-level Python
interface of the reference engine's decode hot path (its ``flashrec.kernel``,
``flashrec.layers``, ``flashrec.attention`` and ``flashrec.logits`` modules) on
top of one C-ABI shared library (``libflashrec_b200.so``, declared in
``include/flashrec_b200.h``). There is no CPU path: tensors must live on a CUDA
device and a missing library raises.
"""

from flashrec_b200._lib import FlashRecKernelError, device_status, lib_path, load  # noqa: F401

__all__ = ["FlashRecKernelError", "device_status", "lib_path", "load"]
__version__ = "0.1.0"
