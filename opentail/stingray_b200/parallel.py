"""Multi-GPU plumbing: one process per GPU, ``torch.distributed`` for rendezvous only.

Two ways to split a sampling step over the GPUs of one box:

* row-sharded (default): rows are independent, rank r takes a contiguous block of rows and no
  data-path collective is needed;
* vocabulary-sharded: every rank holds a column slice of every row (what a tensor-parallel
  lm-head leaves behind); each rank selects its local candidates, one NCCL all-gather (issued by
  the C library on its own communicator) exchanges them, and every rank merges and finishes.

The reference is single-device (``src/OpenTail.Stingray.Cli/RunCommand.cs:100``); nothing here has
a counterpart there.
"""
from __future__ import annotations

from typing import List, Tuple

import numpy as np


def row_block(rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous block [lo, hi) of rows owned by `rank`; sizes differ by at most one."""
    base, extra = divmod(rows, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def vocab_slices(vocab: int, world: int, align: int = 32) -> List[Tuple[int, int]]:
    """Column slices [lo, hi) per rank, boundaries aligned to mask words / vector loads."""
    per = -(-vocab // world)
    per = -(-per // align) * align
    out = []
    for r in range(world):
        lo = min(r * per, vocab)
        out.append((lo, min(lo + per, vocab)))
    return out


def broadcast_bytes(payload: bytes, src: int = 0) -> bytes:
    """Broadcasts a fixed-length byte string from `src` over the default process group (any
    backend); used to hand the NCCL unique id to every rank."""
    import torch
    import torch.distributed as dist

    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.zeros(len(payload), dtype=torch.uint8, device=dev)
    if dist.get_rank() == src:
        t.copy_(torch.frombuffer(bytearray(payload), dtype=torch.uint8))
    dist.broadcast(t, src)
    return bytes(t.cpu().numpy().tobytes())


def slice_history_csr(ids: np.ndarray, offsets: np.ndarray, lo: int, hi: int):
    """CSR arrays of rows [lo, hi) re-based to start at 0."""
    o = offsets[lo:hi + 1]
    return ids[o[0]:o[-1]], (o - o[0]).astype(np.int32)


class VocabShardedSampler:
    """select -> all-gather -> finish over a communicator owned by the C library."""

    def __init__(self, sampler, rank: int, world: int, global_vocab: int):
        import torch.distributed as dist

        self.bs, self.rank, self.world, self.global_vocab = sampler, rank, world, global_vocab
        self.slices = vocab_slices(global_vocab, world)
        uid = sampler.comm_unique_id() if rank == 0 else bytes(128)
        if world > 1:
            uid = broadcast_bytes(uid, 0)
            dist.barrier()
        sampler.comm_init(uid, rank, world)

    def sample(self, local_logits, params, *, history_ids=None, history_offsets=None, uniforms=None,
               **want):
        lo, hi = self.slices[self.rank]
        assert local_logits.shape[1] == hi - lo
        self.bs.shard_select(local_logits, params, lo, self.global_vocab, history_ids=history_ids,
                             history_offsets=history_offsets, uniforms=uniforms)
        self.bs.shard_allgather()
        return self.bs.shard_finish(local_logits.shape[0], hi - lo, params, self.global_vocab,
                                    history_ids=history_ids, history_offsets=history_offsets,
                                    uniforms=uniforms, **want)
