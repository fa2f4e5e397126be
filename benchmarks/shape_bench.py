"""Per-shape GEMV timing: `python -m benchmarks.shape_bench --kind ternary --M 28672 --K 8192`.

Uploads enough copies of one synthetic matrix that a pass over all of them exceeds L2, issues one
`lmb_linear` per copy (captured once as a CUDA graph unless --no-graph) and reports the time per
launch and the algorithmic bytes per second.  `--decode MODEL` times single-token decode steps of
a random-init decoder of a named shape instead.
"""
from __future__ import annotations

import argparse
import json

import numpy as np

from lutmac_b200 import _lib, synth
from lutmac_b200.api import Context
from lutmac_b200.blocks import KIND_NAMES, algorithmic_bytes

KIND_BY_NAME = {v: k for k, v in KIND_NAMES.items()}
L2_BYTES = 126e6


def run_shape(ctx: Context, kind: int, M: int, K: int, copies: int = 0, reps: int = 3, graph: bool = True,
              flags: int = _lib.AUTO_ROTATE, seed: int = 0) -> dict:
    rng = np.random.default_rng(seed)
    nbytes = algorithmic_bytes(kind, M, K)
    ncopies = copies or max(2, min(64, int(3 * L2_BYTES // nbytes) + 1))
    t = synth.tensor(rng, kind, M, K)
    ws = [ctx.upload(t) for _ in range(ncopies)]
    x = ctx.to_device(synth.activations(rng, K))
    y = ctx.malloc(M * 4)
    inner = max(1, 64 // ncopies)

    def issue():
        for _ in range(inner):
            for w in ws:
                ctx.linear(w, x, y, flags=flags)

    if graph:
        ctx.graph_begin()
        issue()
        g = ctx.graph_end()
        run = g.launch
    else:
        run = issue
    run()
    ctx.sync()
    ctx.timer_start()
    for _ in range(reps):
        run()
    ms = ctx.timer_stop()
    us = ms * 1e3 / (reps * inner * ncopies)
    for w in ws:
        w.free()
    return {"kind": KIND_NAMES[kind], "M": M, "K": K, "copies": ncopies, "us_per_launch": us,
            "algorithmic_bytes": nbytes, "gbs": nbytes / us / 1e3}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--kind", default="int4", choices=sorted(KIND_BY_NAME))
    ap.add_argument("--M", type=int, default=2048)
    ap.add_argument("--K", type=int, default=2048)
    ap.add_argument("--copies", type=int, default=0, help="weight copies (0: enough to exceed L2 three times)")
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-rotate", action="store_true")
    ap.add_argument("--lut", action="store_true", help="table-lookup layout for ternary / int2 / binary")
    ap.add_argument("--decode", default="", help="model shape name: time decode steps instead of one GEMV")
    ap.add_argument("--context", type=int, default=512)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--random-kv", action="store_true", help="fill the KV cache with random values instead of prefilling")
    ap.add_argument("--shared-layers", type=int, default=0, help="generate this many distinct layers and repeat them")
    ap.add_argument("--layers", type=int, default=0, help="with --decode: keep only this many layers of the named shape")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tp", action="store_true", help="tensor parallel over the ranks of a torch.distributed.run launch")
    a = ap.parse_args(argv)
    rank, world = 0, 1
    if a.tp:
        import os

        import torch.distributed as dist

        from lutmac_b200 import tp
        rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        dist.init_process_group("gloo")  # rendezvous only; the data path is NCCL inside the library
        ctx = Context(int(os.environ.get("LOCAL_RANK", rank)))
        tp.init_tp(ctx, dist)
    else:
        ctx = Context(0)
    if a.lut:
        ctx.set_option(_lib.OPT_TERNARY_LUT, 1)
    if a.decode:
        from .decode_bench import run_decode
        out = run_decode(ctx, a.decode, KIND_BY_NAME[a.kind], a.context, a.batch, steps=a.steps, random_kv=a.random_kv,
                         warmup=a.warmup, shared_layers=a.shared_layers, tp_rank=rank, tp_size=world, n_layers=a.layers)
    else:
        out = run_shape(ctx, KIND_BY_NAME[a.kind], a.M, a.K, a.copies, a.reps, not a.no_graph,
                        0 if a.no_rotate else _lib.AUTO_ROTATE)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if a.tp:
        dist.barrier()
        _lib.lib().lmb_tp_destroy(ctx.h)
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
