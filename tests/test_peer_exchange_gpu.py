"""The kernel-driven record exchange of multi-GPU split-KV decode, emulated on ONE GPU.

Two (or four) "ranks" live in one process on one device, each with its own exchange buffer, state block and KV
slice; the device array of buffer pointers is the same for all of them.  Every rank first runs its push call, then
every rank runs its wait/merge call, all on one stream: by the time a wait kernel starts, all records and flags are
in place, so no kernel ever waits on another (kernels that wait on one another must not share a GPU).  This checks
the buffer layout, generation counters, double buffering across repeated steps, and the merge."""
import numpy as np
import pytest
import torch

from helpers import assert_close, make_qkv

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("world", [2, 4])
def test_push_then_wait_on_one_device(ops, oracle, world):
    from orin_llm_b200.dist import slice_bounds
    n_head, n_kv, hd, L = 16, 2, 128, 5000
    scale = np.float32(1.0 / np.sqrt(hd))
    nbytes = ops.peer_buffer_bytes(world, n_head, hd)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    states = [torch.zeros(ops.peer_state_bytes(n_head), dtype=torch.uint8, device="cuda") for _ in range(world)]
    ptrs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device="cuda")
    bounds = slice_bounds(L, world)
    for step in range(3):            # three steps: both record slots get reused
        q, K, V = make_qkv(500 + step, n_head, n_kv, hd, L)
        want = oracle.attend(q[0], K.astype(np.float32), V.astype(np.float32), L, scale)
        dq = dev(q[0])
        slices = []
        for r in range(world):
            lo, hi = bounds[r], bounds[r + 1]
            slices.append((dev(K[:, lo:hi]), dev(V[:, lo:hi]), torch.tensor([hi - lo], dtype=torch.int32, device="cuda"), hi - lo))
        for r in range(world):
            Kl, Vl, d_len, n_loc = slices[r]
            ops.attn_decode_partial_push(dq, Kl, Vl, n_head, n_kv, hd, n_loc, d_len, float(scale), ptrs.data_ptr(), r, world,
                                         states[r])
        outs = [torch.empty(n_head, hd, device="cuda") for _ in range(world)]
        for r in range(world):
            ops.attn_peer_wait_combine(bufs[r], world, outs[r], n_head, hd, states[r])
        torch.cuda.synchronize()
        for r in range(world):
            assert ops.peer_status(states[r], n_head) == 0
            assert_close(outs[r].cpu().numpy(), want, "step %d rank %d" % (step, r))
            assert torch.equal(outs[r], outs[0])
