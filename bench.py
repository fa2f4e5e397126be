"""Benchmark of the LUT-GEMV decode hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
  python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...     (N > 1)

Workload (config.workload): one single-token decode step of the random-init Llama-3-70B-shaped
ternary stack -- 80 layers, hidden 8192, 64/8 heads of 128, FFN 28672, int8 head over a 128256
vocabulary, FWHT-rotated activations -- at batch 1 over a 2048-token KV cache.  With N ranks the
stack is tensor-parallel: q/k/v/gate/up and the head sharded by output rows, o/down by 256-column
blocks, the partial vectors exchanged over NVLink peer memory; the work is fixed as N grows
(strong scaling).  One step = one call of lmb_model_forward.  Metric: algorithmic bytes of the
UNSHARDED step / step time in GB/s (bytes = reference block bytes of the 7 x 80 + 1 projections
+ padded activations in and outputs out of every GEMV + the KV cache read), with tokens/s beside
it.  Every step streams 20 GB of weights, far more than the 126 MB L2.

Side keys (1 GPU only; they are the GEMV half of the metric): the 4-bit GEMV suite of the
Llama-3.2-1B layer shapes as one group launch and as a dependent chain, a per-shape table, the
Llama-3.2-1B decode step, the batch-16 step of the headline stack, the CPU baseline.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from lutmac_b200 import synth  # noqa: E402
from lutmac_b200.blocks import INT4, INT8, TERNARY, algorithmic_bytes  # noqa: E402

METRIC = "lut_gemv_decode_hbm_gbs"
UNIT = "GB/s"
MODEL = "llama-3-70b"
CONTEXT = 2047  # the step attends over 2048 positions: 2047 cached ones and its own
DISTINCT_LAYERS = 2  # random layers drawn on the host; the 80 layers are 80 separate device copies of them
WORKLOAD = ("config[4]: decode step, Llama-3-70B-shaped ternary stack (80 layers, hidden 8192, FFN 28672, int8 head), "
            "batch 1, 2048-token KV, tensor-parallel over the ranks")


def env_int(name, default):
    return int(os.environ.get(name, default))


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed regions run; only samples
    whose timestamp falls inside a timed region's wall-clock window are used."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.p = device, None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(self.device), "--query-gpu=" + self.Q,
                                       "--format=csv,noheader,nounits", "-lms", "50"],
                                      stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.p = None

    @staticmethod
    def _epoch(stamp):
        # "2026/11/25 10:00:00.123", local time of the box
        try:
            date, frac = stamp.strip().split(".")
            return time.mktime(time.strptime(date, "%Y/%m/%d %H:%M:%S")) + float("0." + frac)
        except ValueError:
            return None

    def stop(self, windows):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.p.terminate()
        out = self.p.communicate()[0]
        sm, mx, reasons, total = [], [], set(), 0
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            total += 1
            t = self._epoch(f[0])
            if t is None or not any(a - 0.03 <= t <= b + 0.03 for a, b in windows):
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_outside_timed_regions": total - len(sm)}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def headline_spec():
    shape = synth.MODEL_SHAPES[MODEL]
    return synth.model_spec(shape, TERNARY, seed=0, max_seq=2048, shared_layers=DISTINCT_LAYERS)


# ---- CPU baseline / reference arm (the only places that touch oracle/) -------------------------------

def cpu_backend():
    from oracle.oracle import Oracle, Reference
    if Reference.available():
        return Reference(), "reference"
    return Oracle(), "port"


LAYER_SHAPES = [("q", 8192, 8192), ("k", 1024, 8192), ("v", 1024, 8192), ("o", 8192, 8192), ("gate", 28672, 8192),
                ("up", 28672, 8192), ("down", 8192, 28672)]


def cpu_layer_inputs(seed=0):
    rng = np.random.default_rng(seed)
    layer = {n: synth.ternary_tensor(rng, M, K, name=n) for n, M, K in LAYER_SHAPES}
    acts = {n: synth.activations(rng, K) for n, M, K in LAYER_SHAPES}
    return layer, acts


def cpu_layer_pass(backend, layer, acts, threads):
    """The seven projections of ONE layer of the stack through the reference's CPU kernel
    (lut_linear's arithmetic: block-wise FWHT of the input, then lut_gemv); the rows of each GEMV
    are split over `threads` host threads (1 = the kernel exactly as shipped)."""
    t0 = time.perf_counter()
    nbytes = 0
    for name, M, K in LAYER_SHAPES:
        x = backend.apply_hadamard_rotation(acts[name])
        if threads > 1:
            backend.gemv_rows_parallel(TERNARY, layer[name].blocks, x, M, K, threads)
        else:
            backend.gemv(TERNARY, layer[name].blocks, x, M, K)
        nbytes += algorithmic_bytes(TERNARY, M, K)
    return nbytes, time.perf_counter() - t0


def run_reference(args):
    rank = env_int("RANK", 0)
    if rank != 0:
        return
    backend, kind = cpu_backend()
    cores = os.cpu_count() or 1
    layer, acts = cpu_layer_inputs()
    # the row-parallel wrapper does not scale linearly: take the best of a few thread counts
    best, best_t = 1, None
    for th in sorted({max(1, cores // 4), max(1, cores // 2), cores}):
        _, t = cpu_layer_pass(backend, layer, acts, th)
        if best_t is None or t < best_t:
            best, best_t = th, t
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_layer_pass(backend, layer, acts, best)
    steps = max(1, min(args.steps, int(150.0 / max(best_t, 1e-3))))  # K steps, fewer only if they would take over ~2.5 min
    tot_b, tot_t = 0, 0.0
    for _ in range(steps):
        b, t = cpu_layer_pass(backend, layer, acts, best)
        tot_b += b
        tot_t += t
    val = tot_b / tot_t / 1e9
    sample = (f"per step: the 7 ternary projections of 1 of the 80 layers (the reference spends > 99 % of a decode step "
              f"in them), rows of each GEMV split over {best} host threads (best of the thread counts tried); "
              f"{steps} steps timed")
    spec_bytes = 80 * tot_b / steps
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": args.warmup, "ms_per_step": tot_t / steps * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD},
            "tokens_per_s": 1.0 / (80 * tot_t / steps), "projected_step_bytes": spec_bytes,
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": best, "kind": kind, "sample": sample},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---- side measurements (1 GPU) ---------------------------------------------------------------------------

N_SUITE_LAYERS = 16
# dram__bytes_read.sum + dram__bytes_write.sum of one group launch of the 4-bit suite (one ncu capture)
NCU_DRAM_BYTES_PER_SUITE_LAUNCH = 508589056
# (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes of one decode step of the headline stack,
# from one ncu capture of a 4-layer + head step (2060.95 MB against 2046.48 MB); every layer streams its
# own weights once, so the ratio carries over to the 80-layer step
NCU_DRAM_TO_ALGORITHMIC_BYTES = 1.0071


def side_gemv_suite(ctx, peak):
    """The 4-bit GEMV suite over the Llama-3.2-1B per-layer shapes (16 layers x 7 GEMVs, every layer
    with its own weights, 501.7 MB): the 112 independent GEMVs as one prepared group launch, and
    as a dependent chain of single launches."""
    from lutmac_b200 import _lib
    from lutmac_b200.api import Group
    rng = np.random.default_rng(0)
    dev = []
    for _ in range(N_SUITE_LAYERS):
        for name, M, K in synth.LLAMA32_1B_SHAPES:
            w = ctx.upload(synth.int4_tensor(rng, M, K, name=name))
            x = ctx.to_device(synth.activations(rng, K))
            _lib.check(_lib.lib().lmb_fwht256(ctx.h, x.ptr, K))  # rotated activations (input generation)
            dev.append((w, x, ctx.malloc(M * 4), K))
    nbytes = N_SUITE_LAYERS * sum(algorithmic_bytes(INT4, M, K) for _, M, K in synth.LLAMA32_1B_SHAPES)
    group = Group(ctx, [e[0] for e in dev], [e[1] for e in dev], [e[2] for e in dev], flags=0)

    def chain():
        for w, x, y, K in dev:
            ctx.linear(w, x, y, flags=0, x_len=K, x_stride=K)

    chain()
    ctx.sync()
    ctx.graph_begin()
    chain()
    g = ctx.graph_end()
    out = {}
    for name, run, reps in (("one_group_launch", group.launch, 50), ("chain_of_112_launches", g.launch, 10)):
        for _ in range(3):
            run()
        ctx.sync()
        ctx.timer_start()
        for _ in range(reps):
            run()
        ms = ctx.timer_stop() / reps
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": ms, "gbs": gbs, "frac": gbs / peak}
    out["algorithmic_bytes"] = nbytes
    out["ncu_dram_bytes_per_group_launch"] = NCU_DRAM_BYTES_PER_SUITE_LAUNCH
    out["workload"] = "config[1]: int4 GEMV suite, Llama-3.2-1B shapes (q,k,v,o,gate,up,down) x 16 layers, batch 1"
    return out


def side_shapes(ctx, peak):
    """Every GEMV shape of the configurations on its own: a dependent chain of launches over distinct
    weight copies (cold weights, CUDA graph), GB/s of algorithmic bytes and the fraction of peak."""
    from benchmarks.shape_bench import run_shape
    shapes = [("config[0]", TERNARY, 2048, 2048)]
    shapes += [("config[1] " + n, INT4, M, K) for n, M, K in
               (("q/o", 2048, 2048), ("k/v", 512, 2048), ("gate/up", 8192, 2048), ("down", 2048, 8192))]
    shapes += [("config[4] " + n, TERNARY, M, K) for n, M, K in
               (("q/o", 8192, 8192), ("k/v", 1024, 8192), ("gate/up", 28672, 8192), ("down", 8192, 28672))]
    shapes += [("config[3] gate/up", 2, 8960, 1536), ("config[3] down", 2, 1536, 8960), ("lm_head", INT8, 128256, 2048)]
    rows = []
    for label, kind, M, K in shapes:
        r = run_shape(ctx, kind, M, K)
        rows.append({"shape": label, "kind": r["kind"], "M": M, "K": K, "us": round(r["us_per_launch"], 2),
                     "gbs": round(r["gbs"], 1), "frac": round(r["gbs"] / peak, 3)})
    return rows


# ---- our arm -------------------------------------------------------------------------------------------------

def run_ours(args):
    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from benchmarks.decode_bench import DecodeCase, step_bytes_unsharded
    from lutmac_b200 import tp
    from lutmac_b200.api import Context

    ctx = Context(local)
    if dist is not None:
        tp.init_tp(ctx, dist, peer_floats=16 * 8192)

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()
        ctx.sync()

    def reduce_max(v):
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    peak, peak_src = load_peaks()
    max_batch = 1 if args.no_batch16 else 16
    case = DecodeCase(ctx, MODEL, TERNARY, max_batch=max_batch, max_seq=2048, seed=0, shared_layers=DISTINCT_LAYERS,
                      tp_rank=rank, tp_size=world)
    sampler = ClockSampler(local)
    sampler.start()
    windows = []
    win = []
    head = case.time(CONTEXT, 1, steps=args.steps, warmup=max(args.warmup, 3), random_kv=True, barrier=barrier,
                     e2e_steps=max(3, min(args.steps, 30)), reduce_max=reduce_max, window=win)
    windows.append(tuple(win))
    clocks = sampler.stop(windows)
    ms = head["ms_per_step_device"]
    step_bytes = step_bytes_unsharded(case.spec, CONTEXT, 1)
    rank_bytes = case.step_bytes(CONTEXT)
    value = step_bytes / (ms * 1e-3) / 1e9
    e2e_val = step_bytes / (head["ms_per_step_e2e"] * 1e-3) / 1e9
    vocab = case.spec.cfg["vocab"]
    batch16 = None
    if not args.no_batch16:
        b16 = case.time(CONTEXT, 16, steps=max(5, args.steps // 4), warmup=3, random_kv=True, barrier=barrier,
                        reduce_max=reduce_max)
        b16_bytes = step_bytes_unsharded(case.spec, CONTEXT, 16)
        batch16 = {"ms_per_step": b16["ms_per_step_device"], "tokens_per_s": b16["tokens_per_s_device"],
                   "tokens_per_s_e2e": b16["tokens_per_s_e2e"], "algorithmic_bytes_per_step": b16_bytes,
                   "gbs": b16_bytes / (b16["ms_per_step_device"] * 1e-3) / 1e9, "finite_logits": b16["finite_logits"]}
    timed_out = tp.peer_timed_out(ctx) if world > 1 else False
    case.close()
    if rank != 0:
        from lutmac_b200._lib import lib
        barrier()
        lib().lmb_tp_destroy(ctx.h)
        dist.destroy_process_group()
        return
    achieved = rank_bytes / (ms * 1e-3) / 1e9  # this rank's shard: what its HBM has to deliver per step
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "tokens_per_s": 1e3 / ms,
            "config": {"workload": WORKLOAD, "context": CONTEXT + 1, "batch": 1, "tp": world,
                       "l2_policy": "inputs larger than L2 (every step streams all weights: 19.3 GB / N per rank)",
                       "weights": f"80 layers in 80 separate device allocations; values drawn for {DISTINCT_LAYERS} distinct "
                                  "random layers and repeated (host generation time); int8 head of its own",
                       "kv_cache": head["kv_fill"], "finite_logits": head["finite_logits"],
                       "peer_wait_timed_out": bool(timed_out), "model_build_s": round(case.build_s, 1)},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
                         "frac_of_nominal_8000_gbs": achieved / 8000.0,
                         "peak_source": peak_src, "kernel": "decode step of one rank (all kernels of lmb_model_forward)",
                         "algorithmic_bytes_per_launch": rank_bytes,
                         "traffic": int(rank_bytes * NCU_DRAM_TO_ALGORITHMIC_BYTES) if world == 1 else None,
                         "traffic_source": "ncu dram bytes of a 4-layer + head step, scaled by the algorithmic bytes"},
            "e2e": {"value": e2e_val, "unit": UNIT, "tokens_per_s": 1e3 / head["ms_per_step_e2e"],
                    "h2d_bytes_per_step": 4 + 8, "d2h_bytes_per_step": 4 * vocab,
                    "call": "lmb_model_forward: token id and position in from host memory, logits out to host memory"},
            "gpu_launches": int(round(head["kernel_launches_per_step"] * args.steps)), "clocks": clocks}
    if batch16:
        line["batch16"] = batch16
    if world == 1 and not args.no_sides:
        line["gemv_suite"] = side_gemv_suite(ctx, peak)
        line["gemv_shapes"] = side_shapes(ctx, peak)
        from benchmarks.decode_bench import run_decode
        d3 = run_decode(ctx, "llama-3.2-1b", INT4, 512, 1, steps=30)
        d3["frac"] = d3["hbm_gbs"] / peak
        line["decode_llama_1b_int4"] = d3
    if world == 1 and not args.no_cpu:
        backend, kind = cpu_backend()
        layer, acts = cpu_layer_inputs()
        b, t = cpu_layer_pass(backend, layer, acts, 1)
        line["cpu_baseline"] = {"value": b / t / 1e9, "unit": UNIT, "cores": 1, "kind": kind,
                                "sample": "the 7 ternary projections of 1 of the 80 layers (one pass), reference kernel as "
                                          "shipped (1 thread); projected tokens/s = 1 / (80 x that time)",
                                "projected_tokens_per_s": 1.0 / (80 * t)}
    print(json.dumps(line), flush=True)
    if dist is not None:
        from lutmac_b200._lib import lib
        barrier()
        lib().lmb_tp_destroy(ctx.h)
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-sides", action="store_true", help="skip the GEMV-suite, per-shape and 1B-decode side measurements")
    ap.add_argument("--no-batch16", action="store_true", help="skip the batch-16 step of the headline stack")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
