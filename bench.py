"""Benchmark of the LUT-GEMV hot path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config.workload): the 4-bit bit-plane GEMV suite over the Llama-3.2-1B per-layer
shapes at batch 1 -- q, k, v, o, gate, up, down for 16 layers, every layer with its own weights
(501.7 MB of blocks, four times the L2, so every step streams from HBM).  One step = one pass
over the 112 GEMVs.  Metric: algorithmic bytes / time in GB/s (bytes = reference block bytes +
padded activations in + outputs out, per GEMV).  With N > 1 every rank runs the suite on its
own weights (no data-path collective): weak scaling, value = bytes of all ranks / max time.

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
from lutmac_b200.blocks import INT4, algorithmic_bytes, blocks_per_row  # noqa: E402

N_LAYERS = 16
METRIC = "lut_gemv_hbm_gbs"
UNIT = "GB/s"
WORKLOAD = "config[1]: int4 GEMV suite, Llama-3.2-1B shapes (q,k,v,o,gate,up,down) x 16 layers, batch 1"


def env_int(name, default):
    return int(os.environ.get(name, default))


def suite_bytes():
    return N_LAYERS * sum(algorithmic_bytes(INT4, M, K) for _, M, K in synth.LLAMA32_1B_SHAPES)


def make_suite(seed):
    """16 layers x 7 tensors and one rotated activation vector per GEMV (the suite's inputs are
    FWHT-rotated activations; the rotation is part of input generation, not of the 4-bit path)."""
    rng = np.random.default_rng(seed)
    layers = [synth.config2_layer(rng) for _ in range(N_LAYERS)]
    acts = [{n: synth.activations(rng, K) for n, _, K in synth.LLAMA32_1B_SHAPES} for _ in range(N_LAYERS)]
    return layers, acts


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.p = device, None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(self.device), "--query-gpu=" + self.Q,
                                       "--format=csv,noheader,nounits", "-lms", "100"],
                                      stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        out = self.p.communicate()[0]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# dram__bytes_read.sum + dram__bytes_write.sum of one group launch of the suite, from the ncu
# capture summarised in profiles/k_gemv_int4_suite_group.md
NCU_DRAM_BYTES_PER_GROUP_LAUNCH = 508589056


def load_traffic():
    return NCU_DRAM_BYTES_PER_GROUP_LAUNCH


# ---- CPU baseline / reference arm (the only places that touch oracle/) -------------------------------

def cpu_backend():
    from oracle.oracle import Oracle, Reference
    if Reference.available():
        return Reference(), "reference"
    return Oracle(), "port"


def cpu_suite_pass(backend, layers, acts, n_layers, threads):
    """One pass of the reference's CPU kernel over the first n_layers layers; rows of each GEMV
    are split over `threads` host threads (1 = the kernel exactly as shipped)."""
    t0 = time.perf_counter()
    nbytes = 0
    for li in range(n_layers):
        for name, M, K in synth.LLAMA32_1B_SHAPES:
            t = layers[li][name]
            x = np.zeros(blocks_per_row(K) * 256, np.float32)
            x[:K] = acts[li][name]
            if threads > 1:
                backend.gemv_rows_parallel(INT4, t.blocks, x, M, K, threads)
            else:
                backend.gemv(INT4, t.blocks, x, M, K)
            nbytes += algorithmic_bytes(INT4, M, K)
    return nbytes, time.perf_counter() - t0


def run_reference(args):
    rank = env_int("RANK", 0)
    if rank != 0:
        return
    backend, kind = cpu_backend()
    cores = os.cpu_count() or 1
    layers, acts = make_suite(0)
    for _ in range(min(args.warmup, 1)):
        cpu_suite_pass(backend, layers, acts, 1, cores)
    tot_b, tot_t = 0, 0.0
    for _ in range(args.steps):
        b, t = cpu_suite_pass(backend, layers, acts, N_LAYERS, cores)
        tot_b += b
        tot_t += t
    val = tot_b / tot_t / 1e9
    sample = f"full suite pass ({N_LAYERS} layers) per step, rows of each GEMV split over {cores} threads"
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": tot_t / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---- our arm -------------------------------------------------------------------------------------------------

def run_ours(args):
    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from lutmac_b200 import _lib
    from lutmac_b200.api import Context, lut_linear_multi

    ctx = Context(local)
    layers, acts = make_suite(rank)
    dev = []  # per layer: list of (weight, x, y, K)
    for li in range(N_LAYERS):
        row = []
        for name, M, K in synth.LLAMA32_1B_SHAPES:
            w = ctx.upload(layers[li][name])
            x = ctx.to_device(acts[li][name])
            _lib.check(_lib.lib().lmb_fwht256(ctx.h, x.ptr, K))  # rotated activations (input generation)
            y = ctx.malloc(M * 4)
            row.append((w, x, y, K))
        dev.append(row)
    ctx.sync()

    def issue_suite():
        for row in dev:
            for w, x, y, K in row:
                ctx.linear(w, x, y, flags=0, x_len=K, x_stride=K)

    # throughput form: the 112 independent GEMVs of a pass as one prepared group (one launch);
    # latency form (reported beside it): the same 112 GEMVs as a chain of single launches.
    from lutmac_b200.api import Group
    flat = [e for row in dev for e in row]
    group = Group(ctx, [e[0] for e in flat], [e[1] for e in flat], [e[2] for e in flat], flags=0)
    chain_ms = None
    if not args.no_chain:
        issue_suite()  # sizes the split-K scratch before capture
        ctx.sync()
        ctx.graph_begin()
        issue_suite()
        chain = ctx.graph_end()
        for _ in range(3):
            chain.launch()
        ctx.sync()
        ctx.timer_start()
        for _ in range(10):
            chain.launch()
        chain_ms = ctx.timer_stop() / 10

    class graph:  # the timed step
        launch = staticmethod(group.launch)

    def barrier():
        ctx.sync()
        if dist is not None:
            dist.barrier()
        ctx.sync()

    for _ in range(args.warmup):
        graph.launch()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = ctx.launch_count()
    ctx.timer_start()
    for _ in range(args.steps):
        graph.launch()
    ms = ctx.timer_stop()
    gpu_launches = ctx.launch_count() - launches0
    barrier()
    # keep the device busy a little longer so the clock sampler sees the loaded state
    t_end = time.time() + 0.5
    while time.time() < t_end:
        graph.launch()
        ctx.sync()
    clocks = sampler.stop()
    if dist is not None:
        import torch
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    step_bytes = suite_bytes()
    value = world * step_bytes * args.steps / (ms * 1e-3) / 1e9

    # end to end: host buffers through the layer API, one call per layer (7 lut_linear each)
    h2d = N_LAYERS * sum(4 * K for _, _, K in synth.LLAMA32_1B_SHAPES)
    d2h = N_LAYERS * sum(4 * M for _, M, _ in synth.LLAMA32_1B_SHAPES)
    e2e_val = None
    hgroup = None
    if not args.no_e2e:
        from lutmac_b200.api import HostGroup
        host_in = [np.ascontiguousarray(acts[li][n]) for li in range(N_LAYERS) for n, _, _ in synth.LLAMA32_1B_SHAPES]
        hgroup = HostGroup(ctx, [e[0] for e in flat], flags=0)
        e2e_steps = max(3, min(args.steps, 20))
        for dst, src in zip(hgroup.ins, host_in):
            dst[:] = src  # the step's inputs sit in pinned host memory (the group's own buffers)
        for _ in range(2):
            hgroup.run()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            outs = hgroup.run()  # one H2D from pinned memory, one launch, one D2H of the step's results, one sync
        e2e_s = time.perf_counter() - t0
        assert all(np.isfinite(o[:4]).all() for o in outs)
        if dist is not None:
            import torch
            t = torch.tensor([e2e_s], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_s = float(t.item())
        e2e_val = world * step_bytes * e2e_steps / e2e_s / 1e9

    if rank != 0:
        dist.destroy_process_group()
        return
    peak, peak_src = load_peaks()
    per_launch_bytes = step_bytes  # one launch per step
    achieved = step_bytes * args.steps / (ms * 1e-3) / 1e9  # this rank: all launches are the same kernel
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "l2_policy": "inputs larger than L2 (501.7 MB of weights per step)",
                       "launch": "112 GEMVs per step as one prepared group launch (lmb_group_launch)",
                       "chain_of_112_single_launches_gbs": (step_bytes / (chain_ms * 1e-3) / 1e9) if chain_ms else None},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
                         "peak_source": peak_src, "kernel": "k_gemv<int4>",
                         "algorithmic_bytes_per_launch": per_launch_bytes, "traffic": load_traffic()},
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "call": "lmb_group_run_host: the step's 112 lut_linear calls, inputs read from and outputs written to pinned host memory"},
            "gpu_launches": int(gpu_launches), "clocks": clocks}
    if world == 1 and not args.no_decode:
        # side measurement: config[2], one decode step of the random-init Llama-3.2-1B shape (4-bit
        # projections, int8 tied head, 512 cached positions, batch 1); not the headline metric
        from lutmac_b200.decode_bench import run_decode
        del group, hgroup, dev, flat  # free the suite's device memory first
        line["decode"] = run_decode(ctx, "llama-3.2-1b", INT4, 512, 1, steps=30)
    if world == 1 and not args.no_cpu:
        backend, kind = cpu_backend()
        b, t = cpu_suite_pass(backend, layers, acts, N_LAYERS, 1)
        line["cpu_baseline"] = {"value": b / t / 1e9, "unit": UNIT, "cores": 1, "kind": kind,
                                "sample": f"one full suite pass ({N_LAYERS} layers), reference kernel as shipped (1 thread)"}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-chain", action="store_true", help="skip the chain-of-single-launches side measurement")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode-step side measurement")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
