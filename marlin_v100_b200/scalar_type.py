"""Weight element types and their 58-bit ids, as the op boundary passes them
(reference: vllm/scalar_type.py:26-43,83-90; C++ twin csrc/core/scalar_type.hpp:124-157)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ScalarType:
    exponent: int
    mantissa: int
    signed: bool
    bias: int = 0
    finite_values_only: bool = False
    nan_repr: int = 1  # 0 none, 1 IEEE, 2 extended range

    @property
    def id(self) -> int:
        val, off = 0, 0
        for member, width in ((self.exponent, 8), (self.mantissa, 8), (int(self.signed), 1),
                              (self.bias, 32), (int(self.finite_values_only), 1), (self.nan_repr, 8)):
            val |= (int(member) & ((1 << width) - 1)) << off
            off += width
        return val

    @property
    def size_bits(self) -> int:
        return self.exponent + self.mantissa + int(self.signed)


class scalar_types:
    uint4 = ScalarType(0, 4, False, 0)
    uint4b8 = ScalarType(0, 4, False, 8)
    uint8 = ScalarType(0, 8, False, 0)
    uint8b128 = ScalarType(0, 8, False, 128)
    float4_e2m1f = ScalarType(2, 1, True, 0, True, 0)
    float8_e4m3fn = ScalarType(4, 3, True, 0, True, 2)
