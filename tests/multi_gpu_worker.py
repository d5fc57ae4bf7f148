"""Worker of the multi-GPU test (one process per GPU, launched by torchrun): the vocabulary-sharded
path with a real NCCL all-gather must reproduce the unsharded result, and row-sharding must
reproduce the corresponding rows."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import numpy as np
import torch
import torch.distributed as dist

from opentail.stingray_b200 import BatchSampler, parallel as P, workloads as W
from tests import parity


def main():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    rank, world = dist.get_rank(), dist.get_world_size()
    w = W.config5(rows=64, vocab=64000)
    mk = lambda: BatchSampler(max_rows=w.rows, max_vocab=w.vocab, max_history=256, max_top_k=64, device=local)
    full = mk()
    ref = parity.run_gpu(full, w, want_topk=50)
    if rank == 0:
        parity.compare(w, ref)
    # vocabulary-sharded
    bs = mk()
    vs = P.VocabShardedSampler(bs, rank, world, w.vocab)
    lo, hi = vs.slices[rank]
    sl = torch.from_numpy(np.ascontiguousarray(w.logits[:, lo:hi])).cuda()
    hist = torch.from_numpy(w.history_ids).cuda()
    uni = torch.from_numpy(w.uniforms).cuda()
    out = vs.sample(sl, w.params, history_ids=hist, history_offsets=w.history_offsets, uniforms=uni, want_topk=50)
    torch.cuda.synchronize()
    assert np.array_equal(out["tokens"].cpu().numpy(), ref["tokens"]), f"rank {rank}: sharded tokens differ"
    assert np.array_equal(out["topk_ids"].cpu().numpy(), ref["topk_ids"])
    assert np.array_equal(out["topk_probs"].cpu().numpy(), ref["topk_probs"])
    # row-sharded: this rank's block of rows, no collective on the data path
    rlo, rhi = P.row_block(w.rows, rank, world)
    ids, off = P.slice_history_csr(w.history_ids, w.history_offsets, rlo, rhi)
    part = full.sample_rows(torch.from_numpy(w.logits[rlo:rhi]).cuda(), w.params[rlo:rhi], history_ids=ids,
                            history_offsets=off, uniforms=w.uniforms[rlo:rhi])
    torch.cuda.synchronize()
    assert np.array_equal(part["tokens"].cpu().numpy(), ref["tokens"][rlo:rhi])
    gathered = [torch.empty_like(part["tokens"]) for _ in range(world)] if (rhi - rlo) * world == w.rows else None
    if gathered is not None:
        dist.all_gather(gathered, part["tokens"])
        assert np.array_equal(torch.cat(gathered).cpu().numpy(), ref["tokens"])
    dist.barrier()
    bs.close()
    full.close()
    dist.destroy_process_group()
    print(f"rank {rank}/{world} ok", flush=True)


if __name__ == "__main__":
    main()
