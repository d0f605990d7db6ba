"""(batch, head) sharding across two ranks over gloo on CPU: every rank computes
its shard, the all-gather reassembles the full result.  The per-shard compute
is the CPU oracle here (the test is about the split / gather plumbing; the CUDA
kernels are checked by the -m gpu tests)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import dense_masked as dm
from torch_blocksparse_b200 import layouts, shard


def _free_port():
    s = socket.socket()
    s.bind(('127.0.0.1', 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _problem(Z):
    g = torch.Generator().manual_seed(0)
    H, nb, block, D = 4, 4, 16, 32
    layout = layouts.fixed(H, nb, 2, 'unidirectional')
    layout[1, 3, 0] = 1                        # heads own different numbers of blocks
    q, k, v = (torch.randn((Z, H, nb * block, D), generator=g) for _ in range(3))
    return layout, block, q, k, v


def _worker(rank, world, port, Z, out):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        layout, block, q, k, v = _problem(Z)
        H = layout.size(0)
        shards = shard.plan(Z, H, world)
        s = shards[rank]
        lay = shard.slice_layout(layout, s)
        ql, kl, vl = (shard.slice_dense(t, s) for t in (q, k, v))
        scores, _, _ = dm.matmul_reference(ql, kl, 'sdd', False, True, lay, block)       # block format
        probs, _ = dm.softmax_reference(scores, lay, block, scale=0.25)
        o_local, _, _ = dm.matmul_reference(probs, vl, 'dsd', False, False, lay, block)  # dense
        o = shard.gather_dense(o_local, shards, Z, H)
        p = shard.gather_sparse(probs, layout, shards, Z)
        if rank == 0:
            torch.save({'o': o, 'p': p}, out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('Z', [2, 1])      # Z=2: split over the batch; Z=1: split over heads
def test_two_rank_shards_reassemble_to_the_unsharded_result(tmp_path, Z):
    out = str(tmp_path / 'gathered.pt')
    mp.spawn(_worker, args=(2, _free_port(), Z, out), nprocs=2, join=True)
    got = torch.load(out)
    layout, block, q, k, v = _problem(Z)
    scores, _, _ = dm.matmul_reference(q, k, 'sdd', False, True, layout, block)
    probs, _ = dm.softmax_reference(scores, layout, block, scale=0.25)
    o, _, _ = dm.matmul_reference(probs, v, 'dsd', False, False, layout, block)
    assert torch.allclose(got['o'], o, rtol=1e-5, atol=1e-6)
    assert torch.allclose(got['p'], probs, rtol=1e-5, atol=1e-6)
