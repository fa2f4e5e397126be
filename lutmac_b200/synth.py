"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

Weights are written directly into the reference's block structs (random-init stand-ins for
real checkpoints); activations are N(0,1) with 1 % of the positions multiplied by 10.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List

import numpy as np

from .blocks import (BINARY, BLOCK_DTYPES, BLOCK_SIZE, INT2, INT3, INT4, INT5, INT6, INT8, TERNARY, PackedTensor,
                     blocks_per_row)


def activations(rng: np.random.Generator, n: int, outlier_frac: float = 0.01, outlier_gain: float = 10.0) -> np.ndarray:
    x = rng.standard_normal(n).astype(np.float32)
    k = max(1, int(round(n * outlier_frac)))
    idx = rng.choice(n, size=k, replace=False)
    x[idx] *= outlier_gain
    return x


def _row_scales(rng, M, bpr, lo=0.01, hi=0.05, per_row=True):
    if per_row:
        return np.repeat(rng.uniform(lo, hi, size=(M, 1)).astype(np.float32), bpr, axis=1)
    return rng.uniform(lo, hi, size=(M, bpr)).astype(np.float32)


def _pad_mask(K: int) -> np.ndarray:
    """Boolean [bpr*256]: True for real columns, False for the zero padding of the last block."""
    bpr = blocks_per_row(K)
    m = np.zeros(bpr * BLOCK_SIZE, bool)
    m[:K] = True
    return m


def ternary_tensor(rng, M, K, per_row_scale=True, name="") -> PackedTensor:
    """i.i.d. {-1,0,+1} with p = 1/3 each, bit-planes packed MSB first (quantize.hpp:135-154);
    columns beyond K are zero weights, as quantize_tensor pads (quantize.hpp:262-273)."""
    bpr = blocks_per_row(K)
    t = rng.integers(-1, 2, size=(M, bpr * BLOCK_SIZE), dtype=np.int8)
    t[:, ~_pad_mask(K)] = 0
    blocks = np.zeros(M * bpr, BLOCK_DTYPES[TERNARY])
    blocks["sign_plane"] = np.packbits(t < 0, axis=1).reshape(M * bpr, 32)
    blocks["zero_plane"] = np.packbits(t == 0, axis=1).reshape(M * bpr, 32)
    blocks["scale"] = _row_scales(rng, M, bpr, per_row=per_row_scale).reshape(-1)
    return PackedTensor(TERNARY, blocks, M, K, name=name)


def _random_bytes(rng, shape):
    return rng.integers(0, 256, size=shape, dtype=np.uint8)


def int4_tensor(rng, M, K, name="") -> PackedTensor:
    """Uniform 4-bit codes 0..15 (including 0, which the reference quantizer never emits),
    one scale ~U(0.01,0.05)/8 per block; padding columns carry code 8 (= 0.0)."""
    bpr = blocks_per_row(K)
    data = _random_bytes(rng, (M, bpr * 128))
    if K % BLOCK_SIZE:
        codes = np.stack([data >> 4, data & 15], axis=2).reshape(M, bpr * BLOCK_SIZE)
        codes[:, ~_pad_mask(K)] = 8
        codes = codes.reshape(M, bpr * 128, 2)
        data = ((codes[:, :, 0] << 4) | codes[:, :, 1]).astype(np.uint8)
    blocks = np.zeros(M * bpr, BLOCK_DTYPES[INT4])
    blocks["data"] = data.reshape(M * bpr, 128)
    blocks["scale"] = (_row_scales(rng, M, bpr, per_row=False) / 8.0).reshape(-1)
    return PackedTensor(INT4, blocks, M, K, name=name)


def int2_tensor(rng, M, K, name="") -> PackedTensor:
    """RRQ 2-bit: uniform (b1,b2) pairs, scale ~U(0.01,0.05) and scale2 = scale*U(0.2,0.5),
    equal across the blocks of a row."""
    bpr = blocks_per_row(K)
    blocks = np.zeros(M * bpr, BLOCK_DTYPES[INT2])
    blocks["data"] = _random_bytes(rng, (M * bpr, 64))
    s = _row_scales(rng, M, bpr)
    blocks["scale"] = s.reshape(-1)
    blocks["scale2"] = (s * np.repeat(rng.uniform(0.2, 0.5, size=(M, 1)).astype(np.float32), bpr, axis=1)).reshape(-1)
    return PackedTensor(INT2, blocks, M, K, name=name)


def binary_tensor(rng, M, K, name="") -> PackedTensor:
    bpr = blocks_per_row(K)
    blocks = np.zeros(M * bpr, BLOCK_DTYPES[BINARY])
    blocks["data"] = _random_bytes(rng, (M * bpr, 32))
    blocks["scale"] = _row_scales(rng, M, bpr).reshape(-1)
    return PackedTensor(BINARY, blocks, M, K, name=name)


def bitstream_tensor(rng, kind, M, K, name="") -> PackedTensor:
    """3/5/6-bit kinds: uniform random bit streams, per-block scales."""
    assert kind in (INT3, INT5, INT6)
    bpr = blocks_per_row(K)
    blocks = np.zeros(M * bpr, BLOCK_DTYPES[kind])
    blocks["data"] = _random_bytes(rng, (M * bpr, 32 * kind))
    blocks["scale"] = (_row_scales(rng, M, bpr, per_row=False) / float(1 << (kind - 1))).reshape(-1)
    return PackedTensor(kind, blocks, M, K, name=name)


def int8_tensor(rng, M, K, scale_lo=0.01, scale_hi=0.05, name="") -> PackedTensor:
    bpr = blocks_per_row(K)
    blocks = np.zeros(M * bpr, BLOCK_DTYPES[INT8])
    d = rng.integers(-127, 128, size=(M, bpr * BLOCK_SIZE), dtype=np.int8)
    d[:, ~_pad_mask(K)] = 0
    blocks["data"] = d.reshape(M * bpr, 256)
    blocks["scale"] = (_row_scales(rng, M, bpr, scale_lo, scale_hi, per_row=False) / 127.0).reshape(-1)
    return PackedTensor(INT8, blocks, M, K, name=name)


def tensor(rng, kind, M, K, name="") -> PackedTensor:
    if kind == TERNARY:
        return ternary_tensor(rng, M, K, name=name)
    if kind == BINARY:
        return binary_tensor(rng, M, K, name=name)
    if kind == INT2:
        return int2_tensor(rng, M, K, name=name)
    if kind == INT4:
        return int4_tensor(rng, M, K, name=name)
    if kind == INT8:
        return int8_tensor(rng, M, K, name=name)
    return bitstream_tensor(rng, kind, M, K, name=name)


# ---- benchmark configurations ------------------------------------------------------------------------

LLAMA32_1B_SHAPES = [("q", 2048, 2048), ("k", 512, 2048), ("v", 512, 2048), ("o", 2048, 2048),
                     ("gate", 8192, 2048), ("up", 8192, 2048), ("down", 2048, 8192)]


def config1(seed: int = 0):
    """Single ternary LUT GEMV, 2048 x 2048, per-row scales, outlier activations."""
    rng = np.random.default_rng(seed)
    return ternary_tensor(rng, 2048, 2048, name="q_proj"), activations(rng, 2048)


def config2_layer(rng) -> Dict[str, PackedTensor]:
    """The seven 4-bit projections of one Llama-3.2-1B layer."""
    return {n: int4_tensor(rng, M, K, name=n) for n, M, K in LLAMA32_1B_SHAPES}


@dataclass
class ModelSpec:
    cfg: Dict
    embed: PackedTensor
    lm_head: PackedTensor
    final_norm: np.ndarray
    layers: List[Dict] = field(default_factory=list)

    def weight_bytes(self) -> int:
        n = self.lm_head.nbytes
        for L in self.layers:
            n += sum(L[k].nbytes for k in ("q", "k", "v", "o", "gate", "up", "down"))
        return n


MODEL_SHAPES = {
    # name: vocab, hidden, inter, layers, heads, kv_heads, head_dim, rope_theta, rope_factor, eps, qkv_bias
    "llama-3.2-1b": dict(vocab=128256, hidden=2048, inter=8192, n_layers=16, n_heads=32, n_kv_heads=8, head_dim=64,
                         rope_theta=500000.0, rope_factor=32.0, eps=1e-5, qkv_bias=False),
    "qwen-2.5-1.5b": dict(vocab=151936, hidden=1536, inter=8960, n_layers=28, n_heads=12, n_kv_heads=2, head_dim=128,
                          rope_theta=1000000.0, rope_factor=1.0, eps=1e-6, qkv_bias=True),
    "llama-3-70b": dict(vocab=128256, hidden=8192, inter=28672, n_layers=80, n_heads=64, n_kv_heads=8, head_dim=128,
                        rope_theta=500000.0, rope_factor=1.0, eps=1e-5, qkv_bias=False),
}


def model_spec(shape: Dict, kind: int, seed: int = 0, max_seq: int = 2048, shared_layers: int = 0,
               untied_head: bool = False) -> ModelSpec:
    """Random-init decoder of the given shape.  Projections use block kind `kind`; the embedding
    and the tied lm_head are int8, which is what the reference's quantizer produces for every
    bit width below 7.5 (tools/lutmac-quantize.cpp:385-389, src/model.cpp:667-689).

    shared_layers > 0 generates that many distinct layers and repeats them (keeps host memory
    and generation time bounded for the 80-layer stack; device copies are still distinct).
    untied_head gives lm_head its own int8 tensor (drawn after everything else, so the other
    tensors of a seed do not change) instead of sharing the embedding's block array."""
    rng = np.random.default_rng(seed)
    c = dict(shape)
    c["max_seq"] = max_seq
    h, inter, nh, nkv, hd = c["hidden"], c["inter"], c["n_heads"], c["n_kv_heads"], c["head_dim"]
    embed = int8_tensor(rng, c["vocab"], h, 0.5, 1.5, name="model.embed_tokens.weight")
    lm_head = PackedTensor(INT8, embed.blocks, embed.M, embed.K, embed.quant_bits, "lm_head.weight")
    final_norm = (1.0 + 0.1 * rng.standard_normal(h)).astype(np.float32)
    spec = ModelSpec(c, embed, lm_head, final_norm)
    n_gen = c["n_layers"] if shared_layers <= 0 else min(shared_layers, c["n_layers"])
    gen = []
    for i in range(n_gen):
        L = {
            "input_norm": (1.0 + 0.1 * rng.standard_normal(h)).astype(np.float32),
            "post_norm": (1.0 + 0.1 * rng.standard_normal(h)).astype(np.float32),
            "q": tensor(rng, kind, nh * hd, h, f"model.layers.{i}.self_attn.q_proj.weight"),
            "k": tensor(rng, kind, nkv * hd, h, f"model.layers.{i}.self_attn.k_proj.weight"),
            "v": tensor(rng, kind, nkv * hd, h, f"model.layers.{i}.self_attn.v_proj.weight"),
            "o": tensor(rng, kind, h, nh * hd, f"model.layers.{i}.self_attn.o_proj.weight"),
            "gate": tensor(rng, kind, inter, h, f"model.layers.{i}.mlp.gate_proj.weight"),
            "up": tensor(rng, kind, inter, h, f"model.layers.{i}.mlp.up_proj.weight"),
            "down": tensor(rng, kind, h, inter, f"model.layers.{i}.mlp.down_proj.weight"),
        }
        if c.get("qkv_bias"):
            L["q_bias"] = (0.02 * rng.standard_normal(nh * hd)).astype(np.float32)
            L["k_bias"] = (0.02 * rng.standard_normal(nkv * hd)).astype(np.float32)
            L["v_bias"] = (0.02 * rng.standard_normal(nkv * hd)).astype(np.float32)
        gen.append(L)
    spec.layers = [gen[i % n_gen] for i in range(c["n_layers"])]
    if untied_head:
        spec.lm_head = int8_tensor(rng, c["vocab"], h, 0.5, 1.5, name="lm_head.weight")
    return spec


def tiny_model_shape(**over) -> Dict:
    """A few-layer decoder small enough for the CPU oracle to run in well under a second."""
    s = dict(vocab=512, hidden=256, inter=512, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=64,
             rope_theta=10000.0, rope_factor=1.0, eps=1e-5, qkv_bias=False)
    s.update(over)
    return s
