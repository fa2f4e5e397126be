"""Decode-step timing helper: random-init decoder of a named shape, KV cache filled with `ctx_len`
positions of uniform-random token ids, then `steps` timed single-token steps at that context."""
from __future__ import annotations

import time

import numpy as np

from . import synth
from .model import Model


def run_decode(ctx, shape_name: str, kind: int, ctx_len: int, batch: int = 1, steps: int = 20, warmup: int = 3,
               seed: int = 0, shared_layers: int = 0, max_seq: int = 2048, tp_rank: int = 0, tp_size: int = 1,
               spec=None, random_kv: bool = False):
    spec = spec or synth.model_spec(synth.MODEL_SHAPES[shape_name], kind, seed=seed, max_seq=max_seq,
                                    shared_layers=shared_layers)
    m = Model(spec, ctx, max_batch=batch, tp_rank=tp_rank, tp_size=tp_size)
    rng = np.random.default_rng(seed + 1)
    vocab = spec.cfg["vocab"]
    if random_kv and tp_size == 1:
        # a cache of random keys and values instead of ctx_len prefill steps (profiling runs)
        c = spec.cfg
        n = c["n_layers"] * 2 * c["max_seq"] * c["n_kv_heads"] * c["head_dim"]
        kv = (rng.standard_normal(n) * 0.1).astype(np.float32)
        for b in range(batch):
            m.kv_import(kv, seq=b)
    else:
        for p in range(ctx_len):  # prefill by decode, like the reference (src/inference.cpp:275-278)
            m.forward(rng.integers(0, vocab, size=batch), [p] * batch, fetch=False)
    toks = rng.integers(0, vocab, size=batch)
    pos = [ctx_len] * batch
    for _ in range(warmup):
        m.forward(toks, pos, fetch=False)
    ctx.sync()
    # device time of the step (kernels only, logits stay on the device)
    ctx.timer_start()
    for _ in range(steps):
        m.forward(toks, pos, fetch=False)
    dev_ms = ctx.timer_stop() / steps
    # end to end: token ids in, logits out on the host
    t0 = time.perf_counter()
    for _ in range(steps):
        logits = m.forward(toks, pos)
    e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
    step_bytes = m.step_bytes(ctx_len) if batch == 1 else None
    out = {"model": shape_name, "batch": batch, "context": ctx_len, "ms_per_step_device": dev_ms,
           "tokens_per_s_device": batch * 1e3 / dev_ms, "ms_per_step_e2e": e2e_ms,
           "tokens_per_s_e2e": batch * 1e3 / e2e_ms, "finite_logits": bool(np.isfinite(logits).all())}
    if step_bytes:
        out["algorithmic_bytes_per_step"] = step_bytes
        out["hbm_gbs"] = step_bytes / (dev_ms * 1e-3) / 1e9
    m.close()
    return out
