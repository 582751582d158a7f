"""B200 (sm_100a) implementation of the Marlin weight-only GEMM / fused-MoE operator path.

``marlin_v100_b200.ops`` mirrors the reference's thin operator wrappers (``vllm/_custom_ops.py``) over
``ctypes``; the extension modules ``marlin_v100_b200/_C.abi3.so`` and ``_moe_C.abi3.so`` (built by
``python -m marlin_v100_b200.build --torch-ops``) register the same operator schemas under
``torch.ops._C`` / ``torch.ops._moe_C`` when they are imported.  ``fused_moe`` is the two-GEMM expert
layer, ``parallel`` the column-parallel and expert-parallel layers.  All compute goes through the C ABI
of ``include/marlin_b200.h``; there is no CPU path."""
from .scalar_type import ScalarType, scalar_types  # noqa: F401

__version__ = "0.1"
