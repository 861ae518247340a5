"""GGML dtype tags and block geometry (mirrors ``GgmlDType``, xn-core/src/quantized/mod.rs:77-196)."""
from __future__ import annotations

import enum


class GgmlDType(enum.IntEnum):
    """GGUF type tags; the integer values are the on-disk ids (mod.rs:97-137)."""
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q4_1 = 3
    Q5_0 = 6
    Q5_1 = 7
    Q8_0 = 8
    Q8_1 = 9
    Q2K = 10
    Q3K = 11
    Q4K = 12
    Q5K = 13
    Q6K = 14
    Q8K = 15
    BF16 = 30

    @property
    def type_size(self) -> int:
        """Bytes per block (mod.rs:160-179)."""
        return _TYPE_SIZE[self]

    @property
    def block_size(self) -> int:
        """Elements per block (mod.rs:182-195)."""
        return _BLOCK_SIZE[self]

    def row_bytes(self, k: int) -> int:
        """Bytes of one ``k``-element row in canonical GGUF layout."""
        if k % self.block_size:
            raise ValueError(f"k={k} is not a multiple of the {self.block_size}-element block of {self.name}")
        return k // self.block_size * self.type_size

    @property
    def is_quantized_weight(self) -> bool:
        return self in _VEC_DOT and self not in (GgmlDType.Q8_1, GgmlDType.Q8K)

    @property
    def vec_dot_type(self) -> "GgmlDType":
        """The activation block format this weight format is dotted against
        (``GgmlType::VecDotType``, k_quants.rs:210,310,405,511,615,883,1046,1321,1510,1727)."""
        return _VEC_DOT[self]

    @property
    def has_fast_kernels(self) -> bool:
        """The four formats of the benchmark configurations have their own device layouts and streaming / tensor-core
        kernels; the others are kept in canonical GGUF layout and served by one generic kernel."""
        return self in (GgmlDType.Q4_0, GgmlDType.Q8_0, GgmlDType.Q4K, GgmlDType.Q6K)


_TYPE_SIZE = {GgmlDType.F32: 4, GgmlDType.F16: 2, GgmlDType.BF16: 2, GgmlDType.Q4_0: 18, GgmlDType.Q4_1: 20, GgmlDType.Q5_0: 22,
              GgmlDType.Q5_1: 24, GgmlDType.Q8_0: 34, GgmlDType.Q8_1: 36, GgmlDType.Q2K: 84, GgmlDType.Q3K: 110, GgmlDType.Q4K: 144,
              GgmlDType.Q5K: 176, GgmlDType.Q6K: 210, GgmlDType.Q8K: 292}
_BLOCK_SIZE = {GgmlDType.F32: 1, GgmlDType.F16: 1, GgmlDType.BF16: 1, GgmlDType.Q4_0: 32, GgmlDType.Q4_1: 32, GgmlDType.Q5_0: 32,
               GgmlDType.Q5_1: 32, GgmlDType.Q8_0: 32, GgmlDType.Q8_1: 32, GgmlDType.Q2K: 256, GgmlDType.Q3K: 256, GgmlDType.Q4K: 256,
               GgmlDType.Q5K: 256, GgmlDType.Q6K: 256, GgmlDType.Q8K: 256}
_VEC_DOT = {GgmlDType.Q4_0: GgmlDType.Q8_0, GgmlDType.Q5_0: GgmlDType.Q8_0, GgmlDType.Q8_0: GgmlDType.Q8_0,
            GgmlDType.Q4_1: GgmlDType.Q8_1, GgmlDType.Q5_1: GgmlDType.Q8_1, GgmlDType.Q8_1: GgmlDType.Q8_1,
            GgmlDType.Q2K: GgmlDType.Q8K, GgmlDType.Q3K: GgmlDType.Q8K, GgmlDType.Q4K: GgmlDType.Q8K, GgmlDType.Q5K: GgmlDType.Q8K,
            GgmlDType.Q6K: GgmlDType.Q8K, GgmlDType.Q8K: GgmlDType.Q8K}
