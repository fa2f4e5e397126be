"""Worker of tests/test_gpu_tp.py: one process per GPU (launched by torch.distributed.run).
Every rank builds the same random decoder, keeps its tensor-parallel shard, decodes a few
tokens; rank 0 checks the logits against the CPU oracle of the unsharded model."""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch.distributed as dist
    from lutmac_b200 import synth, tp
    from lutmac_b200.api import Context
    from lutmac_b200.blocks import INT4, TERNARY
    from lutmac_b200.model import Model
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dist.init_process_group("gloo")  # rendezvous only; the data path is NCCL inside the library
    ctx = Context(local)
    tp.init_tp(ctx, dist)
    out = {}
    for name, kind, peers in (("int4", INT4, "1"), ("ternary", TERNARY, "1"), ("int4_nccl", INT4, "0")):
        os.environ["LMB_TP_PEERS"] = peers  # read when the model is created
        shape = synth.tiny_model_shape(hidden=512, inter=1024, n_heads=8, n_kv_heads=2, head_dim=64, n_layers=3)
        spec = synth.model_spec(shape, kind, seed=7, max_seq=32)
        m = Model(spec, ctx, max_batch=2, tp_rank=rank, tp_size=world)
        logits = []
        for p, t in enumerate(((3, 9), (100, 4), (7, 7), (500, 1))):
            logits.append(m.forward(np.array(t), [p, p]).copy())
        m.close()
        assert not tp.peer_timed_out(ctx), "a rank gave up waiting for a partial vector"
        if rank == 0:
            from oracle.oracle import Oracle, OracleModel
            orc = Oracle()
            worst = 0.0
            for b in range(2):
                om = OracleModel(orc, spec)
                for p, t in enumerate(((3, 9), (100, 4), (7, 7), (500, 1))):
                    want = om.forward(t[b], p)
                    got = logits[p][b]
                    worst = max(worst, float(np.linalg.norm(got - want) / np.linalg.norm(want)))
            out[name] = worst
    dist.barrier()
    if rank == 0:
        print("TP_RESULT " + json.dumps(out), flush=True)
    from lutmac_b200._lib import lib
    lib().lmb_tp_destroy(ctx.h)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
