"""The reference's block structs as numpy record dtypes, and PackedTensor.

Byte-for-byte the structs of include/lutmac/types.hpp:126-465 (all of them have alignment 4
and no padding), i.e. the bytes a .lutmac file stores (src/format.cpp:463-496).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np

TERNARY, BINARY, INT2, INT3, INT4, INT5, INT6, INT8 = 0, 1, 2, 3, 4, 5, 6, 8
BLOCK_SIZE = 256

BLOCK_DTYPES = {
    TERNARY: np.dtype([("sign_plane", "u1", 32), ("zero_plane", "u1", 32), ("scale", "<f4")]),  # types.hpp:126-137
    BINARY: np.dtype([("data", "u1", 32), ("scale", "<f4")]),                                     # types.hpp:394-401
    INT2: np.dtype([("data", "u1", 64), ("scale", "<f4"), ("scale2", "<f4")]),                     # types.hpp:209-215
    INT3: np.dtype([("data", "u1", 96), ("scale", "<f4")]),                                        # types.hpp:249-254
    INT4: np.dtype([("data", "u1", 128), ("scale", "<f4")]),                                       # types.hpp:174-181
    INT5: np.dtype([("data", "u1", 160), ("scale", "<f4")]),                                       # types.hpp:296-301
    INT6: np.dtype([("data", "u1", 192), ("scale", "<f4")]),                                       # types.hpp:344-349
    INT8: np.dtype([("scale", "<f4"), ("data", "i1", 256)]),                                       # types.hpp:434-438
}
BLOCK_BYTES = {k: d.itemsize for k, d in BLOCK_DTYPES.items()}
assert BLOCK_BYTES == {TERNARY: 68, BINARY: 36, INT2: 72, INT3: 100, INT4: 132, INT5: 164, INT6: 196, INT8: 260}

KIND_NAMES = {TERNARY: "ternary", BINARY: "binary", INT2: "int2", INT3: "int3", INT4: "int4", INT5: "int5",
              INT6: "int6", INT8: "int8"}
# PackedTensor::quant_bits as the reference's quantizers leave it: quantize_tensor never sets it,
# so ternary tensors carry the default 2 (types.hpp:483, quantize.hpp:196-198).
DEFAULT_QUANT_BITS = {TERNARY: 2, BINARY: 1, INT2: 2, INT3: 3, INT4: 4, INT5: 5, INT6: 6, INT8: 8}


def blocks_per_row(K: int) -> int:
    return (K + BLOCK_SIZE - 1) // BLOCK_SIZE


def algorithmic_bytes(kind: int, M: int, K: int, batch: int = 1, bias: bool = False) -> int:
    """Bytes one GEMV call must move: the reference's block bytes plus padded activations in
    and outputs out."""
    bpr = blocks_per_row(K)
    return M * bpr * BLOCK_BYTES[kind] + 4 * bpr * BLOCK_SIZE * batch + 4 * M * batch + (4 * M if bias else 0)


@dataclass
class PackedTensor:
    """Host-side weight tensor: the reference's PackedTensor (types.hpp:470-492) reduced to the
    one block vector that is in use.  `blocks` is a record array of M*ceil(K/256) blocks, row
    r starting at r*ceil(K/256)."""
    kind: int
    blocks: np.ndarray
    M: int
    K: int
    quant_bits: int = -1
    name: str = ""
    _device: Optional[object] = field(default=None, repr=False, compare=False)

    def __post_init__(self):
        if self.quant_bits < 0:
            self.quant_bits = DEFAULT_QUANT_BITS[self.kind]
        b = np.ascontiguousarray(self.blocks)
        if b.dtype != BLOCK_DTYPES[self.kind]:
            b = b.view(np.uint8).reshape(-1).view(BLOCK_DTYPES[self.kind])
        assert b.size == self.M * blocks_per_row(self.K), "block count does not match the shape"
        self.blocks = b

    @property
    def shape(self):
        return (self.M, self.K)

    @property
    def nbytes(self) -> int:
        return self.blocks.nbytes

    def needs_rotation(self) -> bool:
        """lut_linear rotates iff 0 < quant_bits <= 2 or the ternary vector is non-empty
        (src/kernels/lut_gemm_scalar.cpp:92-93)."""
        return (0 < self.quant_bits <= 2) or self.kind == TERNARY

    def rows(self, r0: int, r1: int) -> "PackedTensor":
        """A contiguous slice of the block array: rows [r0, r1)."""
        bpr = blocks_per_row(self.K)
        return PackedTensor(self.kind, self.blocks[r0 * bpr:r1 * bpr], r1 - r0, self.K, self.quant_bits, self.name)
