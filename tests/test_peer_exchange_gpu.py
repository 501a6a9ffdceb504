"""The kernel-driven record exchange of multi-GPU split-KV decode, emulated on ONE GPU.

Two (or four) "ranks" live in one process on one device, each with its own exchange buffer, state block and KV
slice; the device array of buffer pointers is the same for all of them.  Every rank first runs its push call, then
every rank runs its wait/merge call, all on one stream: by the time a wait kernel starts, all records and flags are
in place, so no kernel ever waits on another (kernels that wait on one another must not share a GPU).  This checks
the buffer layout, generation counters, double buffering across repeated steps, and the merge."""
import numpy as np
import pytest
import torch

from helpers import assert_close, assert_f16_rows_match, make_qkv

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("L", [5000, 40000])      # per rank: one merge level in the decode launch / several group results
@pytest.mark.parametrize("world", [2, 4])
def test_push_then_wait_on_one_device(ops, oracle, world, L):
    from orin_llm_b200.dist import slice_bounds
    n_head, n_kv, hd = 16, 2, 128
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


@pytest.mark.parametrize("L", [3000, 150, 30000])      # 47 tiles; one CTA per kv head; ten group results per kv head
def test_fused_exchange_world_one(ops, oracle, L):
    """oattn_decode_peer (push, wait and merge in one launch) with a single rank: the launch waits only for its own
    flag, so it can run alone on one GPU.  Covers the fused code path, its generation counter over repeated calls
    (both record slots) and the status word; equal to the plain decode call."""
    n_head, n_kv, hd = 16, 2, 128
    scale = np.float32(1.0 / np.sqrt(hd))
    buf = torch.zeros(ops.peer_buffer_bytes(1, n_head, hd), dtype=torch.uint8, device="cuda")
    state = torch.zeros(ops.peer_state_bytes(n_head), dtype=torch.uint8, device="cuda")
    ptrs = torch.tensor([buf.data_ptr()], dtype=torch.int64, device="cuda")
    for step in range(3):
        q, K, V = make_qkv(900 + step, n_head, n_kv, hd, L)
        want = oracle.attend(q[0], K.astype(np.float32), V.astype(np.float32), L, scale)
        dq, dK, dV = dev(q[0]), dev(K), dev(V)
        d_len = torch.tensor([L], dtype=torch.int32, device="cuda")
        out = torch.empty(n_head, hd, device="cuda")
        ops.attn_decode_peer(dq, dK, dV, out, n_head, n_kv, hd, L, d_len, float(scale), ptrs.data_ptr(), 0, 1, state)
        torch.cuda.synchronize()
        assert ops.peer_status(state, n_head) == 0
        assert_close(out.cpu().numpy(), want, "fused exchange step %d" % step)
        ref = torch.empty(n_head, hd, device="cuda")
        d_pos = torch.tensor([L - 1], dtype=torch.int32, device="cuda")
        ops.attn_decode(dq, None, None, dK, dV, ref, n_head, n_kv, hd, L, d_pos, float(scale), fuse=ops.FUSE_NONE)
        torch.cuda.synchronize()
        assert torch.allclose(out, ref, rtol=1e-5, atol=1e-6)


def test_rank_without_rows_contributes_the_neutral_record(ops, oracle):
    """A context shorter than the number of tiles the ranks could share: rank 1 of 2 owns no row at all (length 0).  Its
    decode launch leaves the empty state (m = -inf, l = 0), the exchange launch turns it into the neutral record, and
    both ranks' outputs equal the oracle over rank 0's rows."""
    n_head, n_kv, hd, L, world = 16, 2, 128, 50, 2
    scale = np.float32(1.0 / np.sqrt(hd))
    nbytes = ops.peer_buffer_bytes(world, n_head, hd)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    states = [torch.zeros(ops.peer_state_bytes(n_head), dtype=torch.uint8, device="cuda") for _ in range(world)]
    ptrs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device="cuda")
    q, K, V = make_qkv(321, n_head, n_kv, hd, L, 64)
    want = oracle.attend(q[0], K.astype(np.float32), V.astype(np.float32), L, scale)
    dq, dK, dV = dev(q[0]), dev(K), dev(V)
    lens = [torch.tensor([L], dtype=torch.int32, device="cuda"), torch.tensor([0], dtype=torch.int32, device="cuda")]
    for r in range(world):
        ops.attn_decode_partial_push(dq, dK, dV, n_head, n_kv, hd, 64, lens[r], float(scale), ptrs.data_ptr(), r, world, states[r])
    outs = [torch.empty(n_head, hd, device="cuda") for _ in range(world)]
    for r in range(world):
        ops.attn_peer_wait_combine(bufs[r], world, outs[r], n_head, hd, states[r])
    torch.cuda.synchronize()
    for r in range(world):
        assert ops.peer_status(states[r], n_head) == 0
        assert_close(outs[r].cpu().numpy(), want, "rank %d" % r)
    assert torch.equal(outs[0], outs[1])


def test_fused_exchange_more_group_results_than_one_round(ops, oracle):
    """One kv head gets all 2 x SM-count splits: at 100,000 rows the decode launch leaves 17 group results, which the
    exchange launch merges in two rounds of loads."""
    n_head, n_kv, hd, L = 8, 1, 128, 100000
    scale = np.float32(1.0 / np.sqrt(hd))
    buf = torch.zeros(ops.peer_buffer_bytes(1, n_head, hd), dtype=torch.uint8, device="cuda")
    state = torch.zeros(ops.peer_state_bytes(n_head), dtype=torch.uint8, device="cuda")
    ptrs = torch.tensor([buf.data_ptr()], dtype=torch.int64, device="cuda")
    q, K, V = make_qkv(77, n_head, n_kv, hd, L)
    want = oracle.attend(q[0], K.astype(np.float32), V.astype(np.float32), L, scale)
    d_len = torch.tensor([L], dtype=torch.int32, device="cuda")
    out = torch.empty(n_head, hd, device="cuda")
    ops.attn_decode_peer(dev(q[0]), dev(K), dev(V), out, n_head, n_kv, hd, L, d_len, float(scale), ptrs.data_ptr(), 0, 1, state)
    torch.cuda.synchronize()
    assert ops.peer_status(state, n_head) == 0
    assert_close(out.cpu().numpy(), want, "17 group results")


def test_fused_prologue_on_a_sharded_cache(ops, oracle):
    """oattn_decode_peer_fused on the rank that owns the newest rows of a longer sequence: its local cache holds rows
    [lo, pos) of the sequence as local rows 0..pos-lo-1, the new token is rotated at its GLOBAL position `pos` and
    appended at local row pos-lo.  One rank (waits only for itself), checked against the oracle run on the slice."""
    n_head, n_kv, hd, lo, pos = 16, 2, 128, 1000, 3000
    n_loc = pos - lo
    n_ctx = n_loc + 64
    scale = np.float32(1.0 / np.sqrt(hd))
    rng = np.random.default_rng(123)
    _, K, V = make_qkv(124, n_head, n_kv, hd, n_loc, n_ctx)
    q = rng.standard_normal((n_head, hd)).astype(np.float32)
    k = rng.standard_normal((n_kv, hd)).astype(np.float32)
    v = rng.standard_normal((n_kv, hd)).astype(np.float16).astype(np.float32)
    # oracle: rotate at the global position, append at the local row, attend over the slice
    qo, ko = q.copy(), k.copy()
    for h in range(n_head):
        oracle.rope(qo[h], 1, hd, 1e6, pos)
    for h in range(n_kv):
        oracle.rope(ko[h], 1, hd, 1e6, pos)
    kc32, vc32 = K.astype(np.float32), V.astype(np.float32)
    kc32[:, n_loc] = ko
    vc32[:, n_loc] = v
    want = oracle.attend(qo, kc32, vc32, n_loc + 1, scale)

    buf = torch.zeros(ops.peer_buffer_bytes(1, n_head, hd), dtype=torch.uint8, device="cuda")
    state = torch.zeros(ops.peer_state_bytes(n_head), dtype=torch.uint8, device="cuda")
    ptrs = torch.tensor([buf.data_ptr()], dtype=torch.int64, device="cuda")
    dK, dV = dev(K), dev(V)
    out = torch.empty(n_head, hd, device="cuda")
    d_len = torch.tensor([n_loc + 1], dtype=torch.int32, device="cuda")
    d_rope = torch.tensor([pos], dtype=torch.int32, device="cuda")
    ops.attn_decode_peer_fused(dev(q), dev(k), dev(v), dK, dV, out, n_head, n_kv, hd, n_ctx, d_len, d_rope, float(scale),
                               ops.FUSE_ALL, (1, hd, 1e6, None), ptrs.data_ptr(), 0, 1, state)
    torch.cuda.synchronize()
    assert ops.peer_status(state, n_head) == 0
    assert_close(out.cpu().numpy(), want, "fused prologue on a slice")
    assert_f16_rows_match(dK[:, n_loc].cpu().numpy(), ko, "appended K row at the local index")
    assert np.array_equal(dV[:, n_loc].cpu().numpy(), v.astype(np.float16))
    # a rank that does not receive the token only rotates q: same q rotation, cache untouched
    dK2, dV2 = dev(K), dev(V)
    out2 = torch.empty(n_head, hd, device="cuda")
    d_len2 = torch.tensor([n_loc], dtype=torch.int32, device="cuda")
    ops.attn_decode_peer_fused(dev(q), None, None, dK2, dV2, out2, n_head, n_kv, hd, n_ctx, d_len2, d_rope, float(scale),
                               ops.FUSE_ROPE_Q, (1, hd, 1e6, None), ptrs.data_ptr(), 0, 1, state)
    torch.cuda.synchronize()
    want2 = oracle.attend(qo, K.astype(np.float32), V.astype(np.float32), n_loc, scale)
    assert_close(out2.cpu().numpy(), want2, "q-only rotation on a slice")
    assert torch.equal(dK2.view(torch.int16), dev(K).view(torch.int16))


def test_a_wait_that_runs_out_returns_a_status(ops, oracle):
    """A rank whose peer is late: the bounded wait runs out after about a millisecond, raises the status word, leaves the
    output untouched and returns, so the context stays usable.  Once the late record has arrived the same exchange
    completes, and so does the next one.  (Two emulated ranks on one GPU; nothing waits for a kernel that is not
    already finished, and no wait is unbounded.)"""
    from orin_llm_b200.dist import slice_bounds
    n_head, n_kv, hd, L, world = 16, 2, 128, 4000, 2
    scale = np.float32(1.0 / np.sqrt(hd))
    nbytes = ops.peer_buffer_bytes(world, n_head, hd)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    states = [torch.zeros(ops.peer_state_bytes(n_head), dtype=torch.uint8, device="cuda") for _ in range(world)]
    ptrs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device="cuda")
    bounds = slice_bounds(L, world)
    ops.set_wait_limit_cycles(2_000_000)          # about a millisecond
    try:
        for step in range(2):
            q, K, V = make_qkv(640 + step, n_head, n_kv, hd, L)
            want = oracle.attend(q[0], K.astype(np.float32), V.astype(np.float32), L, scale)
            dq = dev(q[0])
            sl = [(dev(K[:, bounds[r]:bounds[r + 1]]), dev(V[:, bounds[r]:bounds[r + 1]]),
                   torch.tensor([bounds[r + 1] - bounds[r]], dtype=torch.int32, device="cuda"), bounds[r + 1] - bounds[r])
                  for r in range(world)]

            def push(r):
                Kl, Vl, d_len, n_loc = sl[r]
                ops.attn_decode_partial_push(dq, Kl, Vl, n_head, n_kv, hd, n_loc, d_len, float(scale), ptrs.data_ptr(), r, world,
                                             states[r])
            outs = [torch.full((n_head, hd), 123.0, device="cuda") for _ in range(world)]
            push(0)
            if step == 0:
                # rank 1 has not pushed yet: rank 0's wait must give up
                ops.attn_peer_wait_combine(bufs[0], world, outs[0], n_head, hd, states[0])
                torch.cuda.synchronize()
                assert ops.peer_status(states[0], n_head) == 1
                assert (outs[0] == 123.0).all()
                # the late rank arrives; its own wait finds both records
                push(1)
                ops.attn_peer_wait_combine(bufs[1], world, outs[1], n_head, hd, states[1])
                torch.cuda.synchronize()
                assert ops.peer_status(states[1], n_head) == 0
                assert_close(outs[1].cpu().numpy(), want, "late rank")
                states[0].view(torch.int32)[2 * n_head] = 0      # the host clears the status word it has handled
            else:
                push(1)
                for r in range(world):
                    ops.attn_peer_wait_combine(bufs[r], world, outs[r], n_head, hd, states[r])
                torch.cuda.synchronize()
                for r in range(world):
                    assert ops.peer_status(states[r], n_head) == 0
                    assert_close(outs[r].cpu().numpy(), want, "exchange after a timed-out one, rank %d" % r)
    finally:
        ops.set_wait_limit_cycles(4_000_000_000)
