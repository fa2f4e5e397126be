"""Where one decode step spends its time, kernel by kernel, measured on the device:
`python -m benchmarks.step_timeline --model llama-3-70b --kind ternary --layers 8 --context 2047`.

Every GEMV and attention launch of the step records device time stamps (lmb_debug_launch_timeline:
first CTA started, first / last CTA past the wait for the preceding kernel, last CTA with its
activations ready, last CTA through its main loop, last / first CTA done).  The table gives, per
kind of launch and averaged over the layers after the first and over `--steps` steps:

    early     how long before the preceding kernel ended this one's first CTA was already resident
    gap       end of the preceding kernel -> first CTA past the wait
    skew      first -> last CTA past the wait
    prologue  -> last CTA has its activations in shared memory
    main      -> last CTA has streamed its weights
    tail      -> last CTA done (split-K arrival, final sums, hand-off / merge)
    period    end of the preceding kernel -> end of this one (these add up to the step)
    ideal     algorithmic bytes of the launch / the measured copy bandwidth

The stamps are atomics on a few words per launch; the step with them is within 1 % of the step without.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os

import numpy as np

from lutmac_b200 import _lib, synth
from lutmac_b200.api import Context
from lutmac_b200.blocks import BLOCK_BYTES, KIND_NAMES
from benchmarks.decode_bench import DecodeCase, step_bytes_unsharded

KIND_BY_NAME = {v: k for k, v in KIND_NAMES.items()}
NAMES = ("q/k/v", "attention", "o_proj", "gate/up", "down_proj")


def peak_gbs() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"])
    except Exception:
        return 6650.0  # earlier measurement on the same kind of GPU


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--model", default="llama-3-70b", choices=sorted(synth.MODEL_SHAPES))
    ap.add_argument("--kind", default="ternary", choices=sorted(KIND_BY_NAME))
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--context", type=int, default=2047)
    ap.add_argument("--steps", type=int, default=5)
    a = ap.parse_args(argv)
    kind = KIND_BY_NAME[a.kind]
    ctx = Context(0)
    L = _lib.lib()
    n = C.c_size_t()
    cap = 4096
    _lib.check(L.lmb_debug_launch_timeline(ctx.h, cap, None, C.byref(n)))  # before the step is captured into a graph
    shape = dict(synth.MODEL_SHAPES[a.model], n_layers=a.layers)
    spec = synth.model_spec(shape, kind, seed=0, max_seq=a.context + 1, shared_layers=2)
    case = DecodeCase(ctx, a.model, kind, max_batch=1, max_seq=a.context + 1, seed=0, shared_layers=2, n_layers=a.layers, spec=spec)
    r = case.time(a.context, 1, steps=20, warmup=3, random_kv=True)
    nb = step_bytes_unsharded(spec, a.context, 1)
    print("%s %s, %d layers + head, context %d: %.3f ms per step (CUDA events), %.0f GB/s algorithmic" %
          (a.model, a.kind, a.layers, a.context, r["ms_per_step_device"], nb / r["ms_per_step_device"] / 1e6))
    toks = np.array([5], np.int32)
    N = 5 * a.layers + 1
    runs = []
    for _ in range(a.steps):
        _lib.check(L.lmb_debug_launch_timeline(ctx.h, 0, None, C.byref(n)))  # clears the slots
        case.model.forward(toks, [a.context], fetch=True)
        out = (C.c_uint64 * (8 * cap))()
        _lib.check(L.lmb_debug_launch_timeline(ctx.h, 0, out, C.byref(n)))
        if n.value != N:
            raise SystemExit("expected %d recorded launches per step (5 per layer + head), got %d: not the default batch-1 step" % (N, n.value))
        runs.append(np.array(list(out)[:8 * N], np.float64).reshape(N, 8))
    c = spec.cfg
    h, inter, hd = c["hidden"], c["inter"], c["head_dim"]
    bb = BLOCK_BYTES[kind] / 256.0
    ideal_bytes = (
        (c["n_heads"] + 2 * c["n_kv_heads"]) * hd * h * bb, 2.0 * (a.context + 1) * c["n_kv_heads"] * hd * 4,
        h * c["n_heads"] * hd * bb, 2.0 * inter * h * bb, h * inter * bb)
    pk = peak_gbs()
    print("%-10s %6s %5s %5s %8s %6s %5s %7s %6s" % ("launch", "early", "gap", "skew", "prologue", "main", "tail", "period", "ideal"))
    total = 0.0
    for k, name in enumerate(NAMES):
        rows = []
        for t in runs:
            for l in range(1, a.layers):
                i = 5 * l + k
                prev = t[i - 1][5]
                rows.append([prev - t[i][0], t[i][1] - prev, t[i][2] - t[i][1], t[i][3] - t[i][2], t[i][4] - t[i][3], t[i][5] - t[i][4],
                             t[i][5] - prev])
        m = np.mean(np.array(rows), axis=0) / 1e3
        total += m[6]
        print("%-10s %6.1f %5.1f %5.1f %8.1f %6.1f %5.1f %7.1f %6.1f" % ((name,) + tuple(m) + (ideal_bytes[k] / pk / 1e3,)))
    t = runs[-1]
    print("per layer %.1f us (ideal %.1f); head %.1f us; step %.1f us from the first launch's start to the last one's end" %
          (total, sum(ideal_bytes) / pk / 1e3, (t[-1][5] - t[-2][5]) / 1e3, (t[-1][5] - t[0][0]) / 1e3))
    case.close()


if __name__ == "__main__":
    main()
