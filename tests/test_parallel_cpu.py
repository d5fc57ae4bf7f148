"""Host-side logic of the multi-GPU paths, on CPU: partitioning, CSR slicing, and the rendezvous
helper over a world_size-2 gloo group."""
import os
import socket
import subprocess
import sys

import numpy as np

from opentail.stingray_b200 import parallel as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_row_blocks_cover_all_rows_once():
    for rows in (0, 1, 7, 256, 4096, 4099):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                lo, hi = P.row_block(rows, r, world)
                assert 0 <= lo <= hi <= rows
                seen += list(range(lo, hi))
            assert seen == list(range(rows))
            sizes = [P.row_block(rows, r, world)[1] - P.row_block(rows, r, world)[0] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1


def test_vocab_slices_are_aligned_and_cover():
    for vocab in (32, 1000, 151936, 256000, 262144):
        for world in (1, 2, 4, 8):
            sl = P.vocab_slices(vocab, world)
            assert sl[0][0] == 0 and sl[-1][1] == vocab
            for (a, b), (c, d) in zip(sl, sl[1:]):
                assert b == c and a % 32 == 0 and c % 32 == 0


def test_history_csr_slice():
    ids = np.arange(20, dtype=np.int32)
    off = np.array([0, 3, 3, 10, 20], np.int32)
    sub, so = P.slice_history_csr(ids, off, 1, 3)
    assert list(so) == [0, 0, 7] and list(sub) == list(range(3, 10))


_WORKER = r"""
import os, sys
sys.path.insert(0, os.environ["STG_ROOT"])
import torch.distributed as dist
from opentail.stingray_b200 import parallel as P
dist.init_process_group("gloo")
rank = dist.get_rank()
payload = bytes(range(128)) if rank == 0 else bytes(128)
got = P.broadcast_bytes(payload, 0)
assert got == bytes(range(128)), got[:8]
lo, hi = P.row_block(4097, rank, dist.get_world_size())
import torch
t = torch.tensor([hi - lo])
dist.all_reduce(t)
assert int(t) == 4097
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
"""


def test_unique_id_broadcast_over_gloo_world_size_2(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, STG_ROOT=ROOT)
    res = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
         "--master-port", str(port), str(script)], env=env, capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.count("ok") == 2
