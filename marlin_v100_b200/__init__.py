"""B200 (sm_100a) implementation of the Marlin weight-only GEMM / fused-MoE operator path.

``marlin_v100_b200.ops`` mirrors the reference's thin operator wrappers (``vllm/_custom_ops.py``);
``marlin_v100_b200.torch_ops`` registers the same operator schemas under ``torch.ops._C`` /
``torch.ops._moe_C``.  All compute goes through the C ABI of ``include/marlin_b200.h``."""
from .scalar_type import ScalarType, scalar_types  # noqa: F401

__version__ = "0.1"
