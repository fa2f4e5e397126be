"""Generates tests/golden/*.npz by running the UNMODIFIED reference (compiled from its own
sources by oracle/Makefile into oracle/_ref/libref_lutmac.so) on seeded inputs.

Run where the reference checkout is available:   python tests/golden/make_golden.py
The fixtures travel with the repository; the reference does not.
"""
from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from lutmac_b200 import synth  # noqa: E402
from lutmac_b200.blocks import (BINARY, INT2, INT3, INT4, INT5, INT6, INT8, KIND_NAMES, TERNARY, PackedTensor,  # noqa: E402
                                blocks_per_row)
from oracle.oracle import Reference, ReferenceModel  # noqa: E402

ALL_KINDS = (TERNARY, BINARY, INT2, INT3, INT4, INT5, INT6, INT8)
GEMV_SHAPES = ((1, 4), (3, 256), (16, 256), (33, 300), (40, 768), (64, 2048))


def gemv_cases(ref: Reference):
    out = {}
    rng = np.random.default_rng(1234)
    for kind in ALL_KINDS:
        for (M, K) in GEMV_SHAPES:
            t = synth.tensor(rng, kind, M, K)
            x = synth.activations(rng, blocks_per_row(K) * 256)
            key = f"{KIND_NAMES[kind]}_{M}x{K}"
            out[key + "_blocks"] = t.blocks.view(np.uint8).reshape(-1)
            out[key + "_x"] = x
            out[key + "_y"] = ref.gemv(kind, t.blocks, x, M, K)
    return out


def linear_cases(ref: Reference):
    """lut_linear: padding, rotation rule, bias, batch."""
    out = {}
    rng = np.random.default_rng(4321)
    cases = [(TERNARY, 2, 48, 512, 2, True), (TERNARY, 2, 20, 300, 1, False), (BINARY, 1, 32, 256, 3, True),
             (INT2, 2, 33, 768, 2, True), (INT3, 3, 16, 512, 1, False), (INT4, 4, 40, 700, 2, True),
             (INT8, 8, 24, 260, 1, True), (INT5, 5, 8, 256, 1, False), (INT6, 6, 8, 512, 2, False)]
    for i, (kind, qb, M, K, batch, with_bias) in enumerate(cases):
        t = synth.tensor(rng, kind, M, K)
        x = np.concatenate([synth.activations(rng, K) for _ in range(batch)])
        bias = rng.standard_normal(M).astype(np.float32) if with_bias else None
        y = ref.lut_linear(kind, qb, t.blocks, M, K, bias, x, batch)
        key = f"lin{i}"
        out[key + "_meta"] = np.array([kind, qb, M, K, batch, int(with_bias)], np.int64)
        out[key + "_blocks"] = t.blocks.view(np.uint8).reshape(-1)
        out[key + "_x"] = x
        out[key + "_bias"] = bias if bias is not None else np.zeros(0, np.float32)
        out[key + "_y"] = y.reshape(-1)
    out["n_cases"] = np.array([len(cases)])
    return out


def transform_cases(ref: Reference):
    rng = np.random.default_rng(77)
    x = synth.activations(rng, 1024 + 100)  # trailing partial block stays untouched
    a4 = np.array([1.0, 2.0, 3.0, 4.0], np.float32)
    xl = synth.activations(rng, 512)
    return {"fwht_in": x, "fwht_out": ref.apply_hadamard_rotation(x), "fwht256_out": ref.fwht_256(x[:256]),
            "lut_in": a4, "lut_out": ref.precompute_lut(a4), "luts_in": xl, "luts_out": ref.precompute_luts(xl).reshape(-1)}


def quantizer_cases(ref: Reference):
    out = {}
    rng = np.random.default_rng(99)
    for kind in (TERNARY, BINARY, INT2, INT3, INT4, INT8):
        for (M, K) in ((4, 16), (3, 300), (16, 512)):
            w = (rng.standard_normal((M, K)) * 0.05).astype(np.float32)
            blocks, qb = ref.quantize(kind, w)
            key = f"{KIND_NAMES[kind]}_{M}x{K}"
            out[key + "_w"] = w
            out[key + "_blocks"] = blocks
            out[key + "_qb"] = np.array([qb])
    t = rng.integers(-1, 2, size=64).astype(np.int8)
    s, z = ref.pack_to_bitplanes(t)
    out["pack_t"], out["pack_s"], out["pack_z"] = t, s, z
    out["unpack_t"] = ref.unpack_from_bitplanes(s, z, 64)
    return out


def glue_cases(ref: Reference):
    rng = np.random.default_rng(5)
    x = rng.standard_normal(256).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(256)).astype(np.float32)
    q = rng.standard_normal(4 * 64).astype(np.float32)
    k = rng.standard_normal(2 * 64).astype(np.float32)
    q2, k2 = ref.apply_rope(q, k, 37, 4, 2, 64, 500000.0, 32.0)
    s = (rng.standard_normal(100) * 3).astype(np.float32)
    return {"rms_x": x, "rms_w": w, "rms_y": ref.rms_norm(x, w, 1e-5), "rope_q": q, "rope_k": k, "rope_q_out": q2,
            "rope_k_out": k2, "softmax_x": s, "softmax_y": ref.softmax(s)}


def model_cases(ref: Reference):
    """Logits of a few decode steps of tiny random decoders (one per projection kind)."""
    out = {}
    tokens = [3, 100, 7, 511]
    for name, kind, over in (("int4", INT4, {}), ("ternary", TERNARY, {}), ("int2_bias", INT2, {"qkv_bias": True}),
                             ("int8", INT8, {"n_kv_heads": 1})):
        spec = synth.model_spec(synth.tiny_model_shape(**over), kind, seed=11, max_seq=2048)
        m = ReferenceModel(ref, spec)
        logits = [m.forward(t, p) for p, t in enumerate(tokens)]
        out[name + "_logits"] = np.stack(logits)
        m.close()
    out["tokens"] = np.array(tokens)
    return out


FILE_CASES = (("tiny_int4", INT4, {}), ("tiny_ternary_bias", TERNARY, {"qkv_bias": True}),
              ("tiny_untied_head", INT4, {"untied_head": True}))
FILE_SHAPE = dict(vocab=256, hidden=256, inter=256, n_layers=1, n_heads=4, n_kv_heads=1, head_dim=64)
FILE_TOKENS = [5, 200, 17]


def file_cases(ref: Reference):
    """.lutmac files written by the reference's save_lutmac, and the logits its load_model +
    Model::forward produce from them."""
    out = {"tokens": np.array(FILE_TOKENS)}
    for name, kind, over in FILE_CASES:
        over = dict(over)
        untied = over.pop("untied_head", False)
        spec = synth.model_spec(synth.tiny_model_shape(**dict(FILE_SHAPE, **over)), kind, seed=21, max_seq=2048,
                                untied_head=untied)
        path = os.path.join(HERE, name + ".lutmac")
        ref.save_lutmac(path, spec)
        out[name + "_logits"] = ref.load_model_logits(path, FILE_TOKENS, spec.cfg["vocab"])
        print(name + ".lutmac", os.path.getsize(path) // 1024, "KiB")
    return out


def main():
    ref = Reference()
    for name, fn in (("gemv", gemv_cases), ("linear", linear_cases), ("transform", transform_cases),
                     ("quantize", quantizer_cases), ("glue", glue_cases), ("model", model_cases),
                     ("files", file_cases)):
        data = fn(ref)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **data)
        print(name, len(data), "arrays,", os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
