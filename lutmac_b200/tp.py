"""Tensor-parallel plumbing: one process per GPU, torch.distributed for the rendezvous.

Sharding rule (no counterpart in the single-process reference): q/k/v/gate/up and lm_head are
split by output rows (whole heads), o/down by 256-column blocks; the 256-point rotation is
local to a block, so a K-shard needs no exchange before its GEMV, only a sum after it.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from .blocks import PackedTensor, blocks_per_row

ROW_SHARDED = ("q", "k", "v", "gate", "up", "lm_head")
BLOCK_SHARDED = ("o", "down")


def shard_rows(t: PackedTensor, rank: int, size: int) -> PackedTensor:
    """Rows [M*rank/size, M*(rank+1)/size): a contiguous slice of the block array."""
    r0, r1 = t.M * rank // size, t.M * (rank + 1) // size
    return t.rows(r0, r1)


def shard_blocks(t: PackedTensor, rank: int, size: int) -> PackedTensor:
    """256-column blocks [bpr*rank/size, bpr*(rank+1)/size) of every row."""
    bpr = blocks_per_row(t.K)
    b0, b1 = bpr * rank // size, bpr * (rank + 1) // size
    blk = np.ascontiguousarray(t.blocks.reshape(t.M, bpr)[:, b0:b1]).reshape(-1)
    K = (t.K - b0 * 256) if b1 == bpr else (b1 - b0) * 256
    return PackedTensor(t.kind, blk, t.M, K, t.quant_bits, t.name)


def shard(name: str, t: PackedTensor, rank: int, size: int) -> PackedTensor:
    return shard_rows(t, rank, size) if name in ROW_SHARDED else shard_blocks(t, rank, size)


class RankLost(RuntimeError):
    """A rank of the tensor-parallel group did not take part in a host-side exchange."""


def exchange(dist, payload: bytes, what: str) -> list:
    """All ranks' payloads, in rank order.  A rank that has left (or never joins) ends the
    collective with the process group's timeout; that is reported as RankLost, so that the
    caller stops before launching kernels that would wait for the missing rank."""
    out = [None] * dist.get_world_size()
    try:
        dist.all_gather_object(out, payload)
    except Exception as e:  # torch raises RuntimeError / DistBackendError, depending on the backend
        raise RankLost(f"tensor-parallel {what}: a rank did not answer ({type(e).__name__}: {str(e)[:200]})") from e
    return out


def init_tp(ctx, dist, peer_floats: int = 32 * 8192) -> None:
    """Create the context's NCCL communicator: rank 0 makes the unique id, torch.distributed
    (any backend) carries it to the others.  peer_floats > 0 also sets up the exchange blocks of
    the peer-memory all-reduce (max batch x hidden size floats per vector)."""
    from ._lib import check, lib
    rank, size = dist.get_rank(), dist.get_world_size()
    ident = (C.c_char * 128)()
    if rank == 0:
        check(lib().lmb_tp_unique_id(ident))
    obj = [bytes(ident)]
    dist.broadcast_object_list(obj, src=0)
    buf = (C.c_char * 128).from_buffer_copy(obj[0])
    check(lib().lmb_tp_init(ctx.h, buf, rank, size))
    if size > 1 and peer_floats > 0:
        # exchange blocks for the all-reduce over peer memory: gather the IPC handles of all ranks
        handle = (C.c_char * 64)()
        check(lib().lmb_tp_peer_create(ctx.h, peer_floats, handle))
        handles = exchange(dist, bytes(handle), "peer-memory set-up")
        allh = (C.c_char * (64 * size)).from_buffer_copy(b"".join(handles))
        check(lib().lmb_tp_peer_open(ctx.h, allh))
        dist.barrier()


def peer_timed_out(ctx) -> bool:
    """True when a tensor-parallel kernel gave up waiting for another rank's partial vector."""
    from ._lib import check, lib
    v = C.c_int(0)
    check(lib().lmb_tp_peer_status(ctx.h, C.byref(v)))
    return bool(v.value)
