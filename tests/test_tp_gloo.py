"""CPU, world_size 2 over gloo: the tensor-parallel sharding rule (row shards for gate/up,
256-column block shards for down, one all-reduce) reproduces the unsharded result when every
rank runs the oracle on its own shard."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from lutmac_b200 import synth, tp
    from lutmac_b200.blocks import TERNARY
    from oracle.oracle import Oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    o = Oracle()
    rng = np.random.default_rng(42)  # same weights on every rank; each keeps its shard
    h, inter = 512, 1024
    gate = synth.ternary_tensor(rng, inter, h)
    up = synth.ternary_tensor(rng, inter, h)
    down = synth.ternary_tensor(rng, h, inter)
    x = synth.activations(rng, h)
    # column-parallel gate/up on the replicated input
    g = o.lut_linear(TERNARY, 2, tp.shard("gate", gate, rank, world).blocks, inter // world, h, None, x)[0]
    u = o.lut_linear(TERNARY, 2, tp.shard("up", up, rank, world).blocks, inter // world, h, None, x)[0]
    act = (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
    # row-parallel down on the rank's own slice of the activation, then all-reduce
    part = o.lut_linear(TERNARY, 2, tp.shard("down", down, rank, world).blocks, h, inter // world, None, act)[0]
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t)
    if rank == 0:
        gf = o.lut_linear(TERNARY, 2, gate.blocks, inter, h, None, x)[0]
        uf = o.lut_linear(TERNARY, 2, up.blocks, inter, h, None, x)[0]
        af = (gf / (1.0 + np.exp(-gf)) * uf).astype(np.float32)
        want = o.lut_linear(TERNARY, 2, down.blocks, h, inter, None, af)[0]
        np.save(os.path.join(out_dir, "got.npy"), t.numpy())
        np.save(os.path.join(out_dir, "want.npy"), want)
    dist.barrier()
    dist.destroy_process_group()


def test_tp2_gate_up_down_over_gloo(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    got, want = np.load(tmp_path / "got.npy"), np.load(tmp_path / "want.npy")
    err = np.linalg.norm(got - want) / np.linalg.norm(want)
    assert err < 1e-5, err
