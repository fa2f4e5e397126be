"""lutmac_b200: B200 (sm_100a) implementation of LutMac's LUT-GEMV decode hot path.

Host-side mirror of the reference's kernel / layer API over the C ABI of
include/lutmac_b200.h.  The CUDA library must be built in-tree first
(`python -m lutmac_b200.build`); there is no CPU fallback.
"""
from .blocks import (BINARY, BLOCK_BYTES, BLOCK_DTYPES, INT2, INT3, INT4, INT5, INT6, INT8, TERNARY, PackedTensor,
                     algorithmic_bytes, blocks_per_row)

__all__ = ["BINARY", "BLOCK_BYTES", "BLOCK_DTYPES", "INT2", "INT3", "INT4", "INT5", "INT6", "INT8", "TERNARY",
           "PackedTensor", "algorithmic_bytes", "blocks_per_row"]
