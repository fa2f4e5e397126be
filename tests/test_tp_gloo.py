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


def _leaver(rank, world, port, out_dir):
    """Rank 1 takes part in the first exchange and then leaves, between steps and with nothing in
    flight; rank 0's next exchange must end with RankLost within the group's timeout, not hang."""
    sys.path.insert(0, ROOT)
    import datetime
    import time
    import torch.distributed as dist
    from lutmac_b200 import tp
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    first = tp.exchange(dist, bytes([rank]) * 4, "step 0")
    assert first == [bytes([r]) * 4 for r in range(world)]
    if rank == 1:
        os._exit(0)  # gone: no destroy, no further collective
    t0 = time.time()
    try:
        tp.exchange(dist, b"step-1", "step 1")
        outcome = "no error"
    except tp.RankLost as e:
        outcome = "RankLost: " + str(e)
    with open(os.path.join(out_dir, "outcome.txt"), "w") as f:
        f.write("%.1f\n%s\n" % (time.time() - t0, outcome))
    os._exit(0)


def test_a_rank_that_leaves_is_reported_on_the_host(tmp_path):
    import torch.multiprocessing as mp
    port = 31500 + os.getpid() % 2000
    mp.spawn(_leaver, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    took, outcome = (tmp_path / "outcome.txt").read_text().splitlines()[:2]
    assert outcome.startswith("RankLost"), outcome
    assert float(took) < 30.0
