"""Decode-step timing helpers: a random-init decoder of a named shape on one context (or one
tensor-parallel rank), a KV cache holding `ctx_len` prior positions, then timed single-token
steps at that context.  Used by bench.py and by `python -m benchmarks.shape_bench --decode`."""
from __future__ import annotations

import time

import numpy as np

from lutmac_b200 import synth
from lutmac_b200.model import Model


class DecodeCase:
    """One model, built once, timed at several batch sizes."""

    def __init__(self, ctx, shape_name: str, kind: int, max_batch: int = 1, max_seq: int = 2048, seed: int = 0,
                 shared_layers: int = 0, tp_rank: int = 0, tp_size: int = 1, n_layers: int = 0, spec=None):
        shape = dict(synth.MODEL_SHAPES[shape_name])
        if n_layers:
            shape["n_layers"] = n_layers
        t0 = time.perf_counter()
        self.spec = spec or synth.model_spec(shape, kind, seed=seed, max_seq=max_seq, shared_layers=shared_layers)
        self.ctx, self.shape_name, self.seed = ctx, shape_name, seed
        self.shared_layers = shared_layers
        self.tp_size = tp_size
        self.model = Model(self.spec, ctx, max_batch=max_batch, tp_rank=tp_rank, tp_size=tp_size)
        ctx.sync()
        self.build_s = time.perf_counter() - t0
        self.rng = np.random.default_rng(seed + 1)

    def fill_cache(self, ctx_len: int, batch: int, random_kv: bool):
        """random_kv: every sequence's cache is one seeded array of N(0, 0.1) keys and values
        (what a timing run needs: 2048 prefill steps of an 80-layer stack take longer than the
        measurement); otherwise prefill by decode over uniform-random token ids, like the reference
        (src/inference.cpp:275-278)."""
        c = self.spec.cfg
        if random_kv:
            n = c["n_layers"] * 2 * c["max_seq"] * c["n_kv_heads"] * c["head_dim"]
            kv = np.random.default_rng(self.seed + 2).standard_normal(n, dtype=np.float32)
            kv *= np.float32(0.1)
            for b in range(batch):
                self.model.kv_import(kv, seq=b)
        else:
            for p in range(ctx_len):
                self.model.forward(self.rng.integers(0, c["vocab"], size=batch), [p] * batch, fetch=False)

    def time(self, ctx_len: int, batch: int = 1, steps: int = 20, warmup: int = 3, random_kv: bool = False, barrier=None,
             e2e_steps: int = 0, reduce_max=None, window=None):
        """Device time per step (CUDA events on the context's stream, between barriers) and the end
        to end time per step (token ids in, logits out on the host).  `window`, if given, receives
        the wall-clock interval of the two timed regions."""
        ctx, m, vocab = self.ctx, self.model, self.spec.cfg["vocab"]
        self.fill_cache(ctx_len, batch, random_kv)
        toks = self.rng.integers(0, vocab, size=batch)
        pos = [ctx_len] * batch
        if barrier:
            barrier()  # ranks finish building at different times: the device-side waits for other ranks are bounded (about a second)
        for _ in range(warmup):
            m.forward(toks, pos, fetch=False)
        ctx.sync()
        if barrier:
            barrier()
        launches0 = ctx.launch_count()
        w0 = time.time()
        ctx.timer_start()
        for _ in range(steps):
            m.forward(toks, pos, fetch=False)
        dev_ms = ctx.timer_stop() / steps
        launches = ctx.launch_count() - launches0
        if barrier:
            barrier()
        e2e_steps = e2e_steps or steps
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            logits = m.forward(toks, pos)
        e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
        w1 = time.time()
        if window is not None:
            window.extend([w0, w1])
        if reduce_max:
            dev_ms, e2e_ms = reduce_max(dev_ms), reduce_max(e2e_ms)
        out = {"model": self.shape_name, "layers": self.spec.cfg["n_layers"], "batch": batch, "context": ctx_len,
               "ms_per_step_device": dev_ms, "tokens_per_s_device": batch * 1e3 / dev_ms, "ms_per_step_e2e": e2e_ms,
               "tokens_per_s_e2e": batch * 1e3 / e2e_ms, "finite_logits": bool(np.isfinite(logits).all()),
               "kernel_launches_per_step": launches / steps, "tp": self.tp_size,
               "distinct_random_layers": self.shared_layers or self.spec.cfg["n_layers"],
               "kv_fill": "seeded random keys/values" if random_kv else "prefill by decode"}
        return out

    def step_bytes(self, ctx_len: int) -> int:
        """Algorithmic bytes of one batch-1 step of THIS rank's shard."""
        return self.model.step_bytes(ctx_len)

    def close(self):
        self.model.close()


def step_bytes_unsharded(spec, ctx_len: int, batch: int = 1) -> int:
    """Algorithmic bytes of one decode step of the whole model: reference block bytes of the 7L + 1
    projections (read once per step whatever the batch), padded activations in and outputs out of
    every GEMV per sequence, the KV cache of the attended positions per sequence, the embedding
    rows."""
    from lutmac_b200.blocks import BLOCK_BYTES, blocks_per_row
    c = spec.cfg

    def gemv(t):
        bpr = blocks_per_row(t.K)
        return t.M * bpr * BLOCK_BYTES[t.kind] + batch * (4 * bpr * 256 + 4 * t.M)

    n = gemv(spec.lm_head) + batch * 4 * c["hidden"]
    for L in spec.layers:
        n += sum(gemv(L[k]) for k in ("q", "k", "v", "o", "gate", "up", "down"))
    n += batch * 2 * c["n_layers"] * (ctx_len + 1) * c["n_kv_heads"] * c["head_dim"] * 4
    return n


def run_decode(ctx, shape_name: str, kind: int, ctx_len: int, batch: int = 1, steps: int = 20, warmup: int = 3,
               seed: int = 0, shared_layers: int = 0, max_seq: int = 2048, tp_rank: int = 0, tp_size: int = 1,
               random_kv: bool = False, n_layers: int = 0):
    case = DecodeCase(ctx, shape_name, kind, max_batch=batch, max_seq=max_seq, seed=seed, shared_layers=shared_layers,
                      tp_rank=tp_rank, tp_size=tp_size, n_layers=n_layers)
    out = case.time(ctx_len, batch, steps, warmup, random_kv)
    nbytes = step_bytes_unsharded(case.spec, ctx_len, batch)
    out["algorithmic_bytes_per_step"] = nbytes
    out["hbm_gbs"] = nbytes / (out["ms_per_step_device"] * 1e-3) / 1e9
    case.close()
    return out
