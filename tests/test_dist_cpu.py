"""Host logic of the multi-GPU split-KV decode, on CPU with the gloo backend (world_size 2 and 4).

Each rank owns a contiguous slice of the KV rows (orin_llm_b200.dist.slice_bounds), produces the (m, l, O)
record for its slice -- here with the CPU oracle standing in for the GPU kernel, since this test has no
GPU --, the records are exchanged with the same gather_records() the GPU path uses, and the merged
result is compared with the oracle over the whole sequence."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _record_from_oracle(orc, q, K, V, lo, hi, scale):
    """(m, l, O) of attention restricted to rows [lo, hi): computed from two oracle calls."""
    n_head, hd = q.shape
    rec = np.zeros((n_head, hd + 4), np.float32)
    if hi <= lo:
        rec[:, hd] = -np.inf
        return rec
    Ks, Vs = np.ascontiguousarray(K[:, lo:hi]), np.ascontiguousarray(V[:, lo:hi])
    out = orc.attend(q, Ks, Vs, hi - lo, scale)                      # normalised
    n_kv = K.shape[0]
    for h in range(n_head):
        kv = h * n_kv // n_head
        s = (Ks[kv] @ q[h]) * scale
        m = s.max()
        l = np.exp(s - m).sum(dtype=np.float64)
        rec[h, :hd] = out[h] * l
        rec[h, hd], rec[h, hd + 1] = m, l
    return rec


def _worker(rank, world, port, L, fail_rank):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from helpers import assert_close, lse_merge, make_qkv
        from oracle.oracle import Oracle
        from orin_llm_b200.dist import gather_records, slice_bounds
        orc = Oracle()
        n_head, n_kv, hd = 16, 2, 128
        scale = np.float32(1.0 / np.sqrt(hd))
        q, K, V = make_qkv(77, n_head, n_kv, hd, L)          # same seed on every rank
        K32, V32 = K.astype(np.float32), V.astype(np.float32)
        bounds = slice_bounds(L, world)
        assert bounds[0] == 0 and bounds[-1] == L and all(b % 64 == 0 for b in bounds[:-1])
        lo, hi = bounds[rank], bounds[rank + 1]
        local = torch.from_numpy(_record_from_oracle(orc, q[0], K32, V32, lo, hi, scale))
        if rank == fail_rank:
            # a rank that has nothing to contribute (its slice was lost) sends the neutral record m = -inf, l = 0
            local = torch.from_numpy(_record_from_oracle(orc, q[0], K32, V32, 0, 0, scale))
        parts = torch.zeros(world, n_head, hd + 4)
        gather_records(local, parts)
        p = parts.numpy()
        merged = lse_merge([(p[r, :, hd], p[r, :, hd + 1], p[r, :, :hd]) for r in range(world)])
        if fail_rank < 0:
            want = orc.attend(q[0], K32, V32, L, scale)
        else:
            # the merge must equal attention over the rows of the remaining ranks
            keep = np.concatenate([np.arange(bounds[r], bounds[r + 1]) for r in range(world) if r != fail_rank])
            want = orc.attend(q[0], np.ascontiguousarray(K32[:, keep]), np.ascontiguousarray(V32[:, keep]), len(keep), scale)
        assert_close(merged, want, "rank %d merged" % rank)
        # a buffer sized for another world size is refused before any communication
        with pytest.raises(ValueError):
            gather_records(local, torch.zeros(world + 1, n_head, hd + 4))
        with pytest.raises(ValueError):
            gather_records(local[:, :-1], parts)
        # every rank holds the same gathered records
        chk = [torch.zeros_like(parts) for _ in range(world)]
        dist.all_gather(chk, parts)
        assert all(torch.equal(c, parts) for c in chk)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,L", [(2, 1000), (4, 130), (2, 64)])
def test_split_kv_exchange_gloo(world, L):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, L, -1), nprocs=world, join=True)


@pytest.mark.parametrize("world,fail_rank", [(2, 1), (4, 2)])
def test_a_rank_with_a_neutral_record_drops_out_of_the_merge(world, fail_rank):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, 1000, fail_rank), nprocs=world, join=True)


def test_slice_bounds_properties():
    from orin_llm_b200.dist import slice_bounds
    for L in (1, 63, 64, 65, 1000, 131072, 1048576):
        for world in (1, 2, 4, 8):
            b = slice_bounds(L, world)
            assert len(b) == world + 1 and b[0] == 0 and b[-1] == L
            assert all(b[i] <= b[i + 1] for i in range(world))
            assert all(x % 64 == 0 for x in b[:-1])
            sizes = [b[i + 1] - b[i] for i in range(world)]
            assert max(sizes) - min(sizes) <= 64 or L < 64 * world
