"""GPU parity tests of the decode path (through the C ABI) against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from helpers import assert_close, assert_f16_rows_match, f16_round, lse_merge, make_qkv

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def run_decode(ops, q, K, V, npos, scale, **kw):
    n_head, hd = q.shape
    n_kv, n_ctx, _ = K.shape
    dq, dK, dV = dev(q), dev(K), dev(V)
    out = torch.empty(n_head, hd, device="cuda")
    d_pos = torch.tensor([npos - 1], dtype=torch.int32, device="cuda")
    ops.flash_attention_decode_ind(dq, dK, dV, out, n_head, n_kv, hd, n_ctx, d_pos, scale, **kw)
    torch.cuda.synchronize()
    return out.cpu().numpy()


# (n_head, n_kv, hd, npos, n_ctx): ratios 1/4/6/7/8/16, both head dims, lengths around tile (64) and
# split boundaries, a single position, a full cache.
SHAPES = [
    (28, 4, 128, 1, 64), (28, 4, 128, 63, 64), (28, 4, 128, 64, 64), (28, 4, 128, 65, 256),
    (28, 4, 128, 1000, 1024), (12, 2, 128, 173, 4096), (32, 8, 128, 640, 8192), (16, 2, 128, 4097, 8192),
    (4, 4, 128, 129, 256), (8, 2, 64, 200, 256), (16, 1, 64, 333, 512), (32, 2, 128, 515, 1024),
    (6, 2, 64, 9000, 16384),
]


@pytest.mark.parametrize("n_head,n_kv,hd,npos,n_ctx", SHAPES)
def test_decode_matches_oracle(ops, oracle, n_head, n_kv, hd, npos, n_ctx):
    q, K, V = make_qkv(1000 + npos, n_head, n_kv, hd, npos, n_ctx)
    scale = np.float32(1.0 / np.sqrt(hd))
    got = run_decode(ops, q[0], K, V, npos, float(scale))
    want = oracle.attend(q[0], K.astype(np.float32), V.astype(np.float32), npos, scale)
    assert_close(got, want, "decode %s" % ((n_head, n_kv, hd, npos),))


@pytest.mark.parametrize("L", [1024, 4096, 16384, 32768])
def test_decode_isolated_7b_shape(ops, oracle, L):
    """28 query / 4 kv heads, head_dim 128, one query token, scale 1/sqrt(128), N(0,1) fp16 inputs."""
    q, K, V = make_qkv(20 + L, 28, 4, 128, L)
    scale = np.float32(1.0 / np.sqrt(128))
    got = run_decode(ops, q[0], K, V, L, float(scale))
    want = oracle.attend(q[0], K.astype(np.float32), V.astype(np.float32), L, scale)
    assert_close(got, want, "decode L=%d" % L)


def test_rows_past_the_position_are_never_used(ops, oracle):
    """Cache rows beyond *d_pos hold NaN/Inf (the reference never clears its cache): the result must
    not depend on them."""
    n_head, n_kv, hd, npos, n_ctx = 28, 4, 128, 300, 1024
    q, K, V = make_qkv(31, n_head, n_kv, hd, npos, n_ctx)
    K[:, npos:] = np.float16(np.nan)
    V[:, npos:] = np.float16(np.inf)
    V[:, npos + 5:] = np.float16(np.nan)
    scale = np.float32(1.0 / np.sqrt(hd))
    got = run_decode(ops, q[0], K, V, npos, float(scale))
    want = oracle.attend(q[0], K.astype(np.float32)[:, :npos].copy(), V.astype(np.float32)[:, :npos].copy(), npos, scale)
    assert_close(got, want, "poisoned tail")


def test_split_count_invariance(ops):
    """Cutting the sequence into more or fewer slices changes only fp32 rounding."""
    n_head, n_kv, hd, npos = 16, 2, 128, 20000
    q, K, V = make_qkv(32, n_head, n_kv, hd, npos)
    scale = float(1.0 / np.sqrt(hd))
    outs = []
    try:
        for mt in (1, 2, 16, 512):
            ops.set_decode_min_tiles(mt)
            outs.append(run_decode(ops, q[0], K, V, npos, scale))
    finally:
        ops.set_decode_min_tiles(1)
    for o in outs[1:]:
        assert np.abs(o - outs[0]).max() < 2e-5


def test_fused_decode_matches_reference_fixture(ops, oracle):
    """Token-by-token fused decode (RoPE q, RoPE k, append, attend) on the inputs the reference's own
    forward() consumed; compared with the attention output it produced."""
    for name in ("probe_neox", "probe_normal", "probe_partial"):
        g = np.load(os.path.join(GOLD, name + ".npz"))
        n_head, n_kv, d, n_ctx = int(g["n_head"]), int(g["n_kv"]), int(g["d"]), int(g["n_ctx"])
        ff = dev(g["freq_factors"]) if g["freq_factors"].size else None
        rope = (int(g["rope_type"]), int(g["n_rot"]), float(g["theta"]), ff)
        kc = torch.zeros(n_kv, n_ctx, d, dtype=torch.float16, device="cuda")
        vc = torch.zeros_like(kc)
        out = torch.empty(n_head, d, device="cuda")
        d_pos = torch.zeros(1, dtype=torch.int32, device="cuda")
        n_tok = g["q_pre"].shape[0]
        for t in range(n_tok):
            d_pos.fill_(t)
            ops.attn_decode(dev(g["q_pre"][t]), dev(g["k_pre"][t]), dev(g["v_pre"][t]), kc, vc, out, n_head, n_kv, d,
                            n_ctx, d_pos, float(1.0 / np.sqrt(d)), ops.FUSE_ALL, rope)
            torch.cuda.synchronize()
            assert_close(out.cpu().numpy(), g["attn"][t], "%s token %d" % (name, t))
        # the cache now holds fp16(rotated k) and fp16(v), exactly
        want_k = np.transpose(g["k_rot"], (1, 0, 2)).astype(np.float16)
        want_v = np.transpose(g["v_pre"], (1, 0, 2)).astype(np.float16)
        got_k = kc.cpu().numpy()[:, :n_tok]
        assert np.array_equal(got_k.view(np.uint16), want_k.view(np.uint16)), name
        assert np.array_equal(vc.cpu().numpy()[:, :n_tok].view(np.uint16), want_v.view(np.uint16)), name


def test_fused_decode_long_context(ops, oracle):
    """Fused step far into a context: position 5000, normal and neox pairing, frequency factors."""
    rng = np.random.default_rng(33)
    n_head, n_kv, hd, n_ctx, pos = 32, 8, 128, 8192, 5000
    scale = np.float32(1.0 / np.sqrt(hd))
    for rope_type in (0, 1):
        ff = (1.0 + rng.random(hd // 2)).astype(np.float32)
        _, K, V = make_qkv(34 + rope_type, n_head, n_kv, hd, pos, n_ctx)
        q = rng.standard_normal((n_head, hd)).astype(np.float32)
        k = rng.standard_normal((n_kv, hd)).astype(np.float32)
        v = rng.standard_normal((n_kv, hd)).astype(np.float32)
        # oracle: fp32 cache holding the fp16 history, then the reference's step
        kc32, vc32 = K.astype(np.float32), V.astype(np.float32)
        qo, ko = q.copy()[None], k.copy()[None]
        want = oracle.attn_batch(qo, ko, v[None].copy(), kc32, vc32, pos, scale, True, rope_type, hd, 5e5, ff)[0]
        dK, dV = dev(K), dev(V)
        out = torch.empty(n_head, hd, device="cuda")
        d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
        ops.attn_decode(dev(q), dev(k), dev(v), dK, dV, out, n_head, n_kv, hd, n_ctx, d_pos, float(scale), ops.FUSE_ALL,
                        (rope_type, hd, 5e5, dev(ff)))
        torch.cuda.synchronize()
        assert_close(out.cpu().numpy(), want, "fused decode rope_type %d" % rope_type)
        assert_f16_rows_match(dK.cpu().numpy()[:, pos], ko[0], "appended K row")
        assert np.array_equal(dV.cpu().numpy()[:, pos].view(np.uint16), v.astype(np.float16).view(np.uint16))
        # history untouched
        assert np.array_equal(dK.cpu().numpy()[:, :pos], K[:, :pos])


def test_decode_replays_from_a_cuda_graph(ops, oracle):
    """The decode call is captured once and replayed with only the device-side position changing
    (src/model_gpu.cu:295-344)."""
    n_head, n_kv, hd, n_ctx = 12, 2, 128, 4096
    scale = np.float32(1.0 / np.sqrt(hd))
    rng = np.random.default_rng(35)
    n0 = 45
    _, K, V = make_qkv(36, n_head, n_kv, hd, n0, n_ctx)
    kc32, vc32 = K.astype(np.float32), V.astype(np.float32)
    dK, dV = dev(K), dev(V)
    dq = torch.empty(n_head, hd, device="cuda")
    dk = torch.empty(n_kv, hd, device="cuda")
    dv = torch.empty(n_kv, hd, device="cuda")
    out = torch.empty(n_head, hd, device="cuda")
    d_pos = torch.tensor([n0], dtype=torch.int32, device="cuda")
    rope = (1, hd, 1e6, None)
    ws = ops.decode_workspace(n_head, n_kv, hd)
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        ops.set_stream(stream)
        try:
            graph.capture_begin()
            ops.attn_decode(dq, dk, dv, dK, dV, out, n_head, n_kv, hd, n_ctx, d_pos, float(scale), ops.FUSE_ALL, rope, ws)
            graph.capture_end()
        finally:
            ops.set_stream(None)
    for step in range(70):       # crosses the 64-row tile boundary and a split boundary
        pos = n0 + step
        q = rng.standard_normal((n_head, hd)).astype(np.float32)
        k = rng.standard_normal((n_kv, hd)).astype(np.float32)
        v = f16_round(rng.standard_normal((n_kv, hd)).astype(np.float32))
        dq.copy_(dev(q)); dk.copy_(dev(k)); dv.copy_(dev(v)); d_pos.fill_(pos)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        qo, ko = q.copy()[None], k.copy()[None]
        want = oracle.attn_batch(qo, ko, v[None].copy(), kc32, vc32, pos, scale, True, 1, hd, 1e6, None)[0]
        # the device cache holds fp16(k); keep the oracle's history identical to it
        kc32[:, pos] = f16_round(ko[0])
        if step % 9 == 0 or step > 60:
            assert_close(out.cpu().numpy(), want, "graph replay step %d" % step)


def test_partial_and_combine(ops, oracle):
    """KV slices -> (m, l, O) partials -> combine == attention over the whole sequence."""
    n_head, n_kv, hd, L = 16, 2, 128, 6000
    scale = np.float32(1.0 / np.sqrt(hd))
    q, K, V = make_qkv(37, n_head, n_kv, hd, L)
    want = oracle.attend(q[0], K.astype(np.float32), V.astype(np.float32), L, scale)
    bounds = [0, 1500, 1500, 4321, 6000]       # includes an empty slice
    n_parts = len(bounds) - 1
    parts = torch.zeros(n_parts, n_head, hd + ops.PART_PAD, device="cuda")
    dq = dev(q[0])
    for i in range(n_parts):
        lo, hi = bounds[i], bounds[i + 1]
        n_loc = max(hi - lo, 1)
        Kl = np.zeros((n_kv, n_loc, hd), np.float16); Vl = np.zeros_like(Kl)
        Kl[:, :hi - lo] = K[:, lo:hi]; Vl[:, :hi - lo] = V[:, lo:hi]
        d_len = torch.tensor([hi - lo], dtype=torch.int32, device="cuda")
        ops.attn_decode_partial(dq, dev(Kl), dev(Vl), parts[i], n_head, n_kv, hd, n_loc, d_len, float(scale))
    out = torch.empty(n_head, hd, device="cuda")
    ops.attn_combine(parts, n_parts, out, n_head, hd)
    torch.cuda.synchronize()
    assert_close(out.cpu().numpy(), want, "partial+combine")
    p = parts.cpu().numpy()
    assert np.isneginf(p[1, :, hd]).all() and (p[1, :, hd + 1] == 0).all() and (p[1, :, :hd] == 0).all()
    # the records themselves merge to the same answer in float64 on the host
    host = lse_merge([(p[i, :, hd], p[i, :, hd + 1], p[i, :, :hd]) for i in range(n_parts)])
    assert_close(host, want, "host merge of device partials")


def test_long_context_3b_shape_properties(ops, oracle):
    """16 query / 2 kv heads at KV length 131072: oracle on two heads; and at 1048576: split invariance
    plus the oracle on one head."""
    n_head, n_kv, hd = 16, 2, 128
    scale = np.float32(1.0 / np.sqrt(hd))
    for L, heads in ((131072, (0, 15)), (1048576, (9,))):
        rng = np.random.default_rng(38)
        q = f16_round(rng.standard_normal((n_head, hd), dtype=np.float32))
        dK = torch.randn(n_kv, L, hd, device="cuda", dtype=torch.float16, generator=torch.Generator("cuda").manual_seed(L))
        dV = torch.randn(n_kv, L, hd, device="cuda", dtype=torch.float16, generator=torch.Generator("cuda").manual_seed(L + 1))
        out = torch.empty(n_head, hd, device="cuda")
        d_pos = torch.tensor([L - 1], dtype=torch.int32, device="cuda")
        ops.flash_attention_decode_ind(dev(q), dK, dV, out, n_head, n_kv, hd, L, d_pos, float(scale))
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        for h in heads:
            kv = h * n_kv // n_head
            Kh = dK[kv].float().cpu().numpy()[None]
            Vh = dV[kv].float().cpu().numpy()[None]
            want = oracle.attend(q[h:h + 1], Kh, Vh, L, scale)
            assert_close(got[h:h + 1], want, "L=%d head %d" % (L, h))
        try:
            ops.set_decode_min_tiles(512)
            out2 = torch.empty_like(out)
            ops.flash_attention_decode_ind(dev(q), dK, dV, out2, n_head, n_kv, hd, L, d_pos, float(scale))
            torch.cuda.synchronize()
        finally:
            ops.set_decode_min_tiles(1)
        assert (out2 - out).abs().max().item() < 2e-5
        del dK, dV


def test_argument_errors(ops):
    from orin_llm_b200 import capi
    L = capi.lib()
    t = torch.zeros(4096, device="cuda")
    p = t.data_ptr()
    ws = ops.decode_workspace(28, 4, 128)
    assert L.oattn_decode(p, None, None, p, p, p, 28, 4, 96, 64, p, 0.1, 0, None, ws.data_ptr(), ws.numel(), None) == capi.ERR_UNSUPPORTED
    assert L.oattn_decode(p, None, None, p, p, p, 28, 5, 128, 64, p, 0.1, 0, None, ws.data_ptr(), ws.numel(), None) == capi.ERR_UNSUPPORTED
    assert L.oattn_decode(p, None, None, p, p, p, 28, 4, 128, 64, p, 0.1, 0, None, ws.data_ptr(), 16, None) == capi.ERR_WORKSPACE
    assert L.oattn_decode(p, None, None, p, p, p, 28, 4, 128, 64, None, 0.1, 0, None, ws.data_ptr(), ws.numel(), None) == capi.ERR_ARG
    assert L.oattn_decode(p, None, None, p, p, p, 28, 4, 128, 64, p, 0.1, 7, None, ws.data_ptr(), ws.numel(), None) == capi.ERR_ARG
    assert L.oattn_prefill(p, None, None, p, p, p, 28, 4, 128, 64, 60, 8, 0.1, 0, None, ws.data_ptr(), ws.numel(), None) == capi.ERR_ARG


@pytest.mark.parametrize("mode", [1, 2])
def test_launch_overlap_modes_give_the_same_output(ops, oracle, mode):
    """A chain of layer calls, each on its own cache (as a decode step runs them), captured in a CUDA graph under
    launch-ordering modes 1 (dependent launches) and 2 (dependent launches with K/V prefetch before the wait): same
    bits as the default mode 0, and equal to the oracle."""
    n_head, n_kv, hd, n_ctx, layers = 16, 2, 128, 3000, 6
    scale = np.float32(1.0 / np.sqrt(hd))
    rope = (1, hd, 1e6, None)
    pos = 2500
    rng = np.random.default_rng(77)
    caches, qs, ks, vs = [], [], [], []
    for l in range(layers):
        _, K, V = make_qkv(700 + l, n_head, n_kv, hd, pos, n_ctx)
        caches.append((K, V))
        qs.append(rng.standard_normal((n_head, hd)).astype(np.float32))
        ks.append(rng.standard_normal((n_kv, hd)).astype(np.float32))
        vs.append(f16_round(rng.standard_normal((n_kv, hd)).astype(np.float32)))
    d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    dq, dk, dv = dev(np.stack(qs)), dev(np.stack(ks)), dev(np.stack(vs))
    ws = ops.decode_workspace(n_head, n_kv, hd)

    def run(m):
        ops.set_decode_overlap(m)
        try:
            dK = [dev(K) for K, _ in caches]
            dV = [dev(V) for _, V in caches]
            out = torch.zeros(layers, n_head, hd, device="cuda")
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                ops.set_stream(stream)
                try:
                    graph.capture_begin()
                    for l in range(layers):
                        ops.attn_decode(dq[l], dk[l], dv[l], dK[l], dV[l], out[l], n_head, n_kv, hd, n_ctx, d_pos, float(scale),
                                        ops.FUSE_ALL, rope, ws)
                    graph.capture_end()
                finally:
                    ops.set_stream(None)
            graph.replay()
            torch.cuda.synchronize()
            eager = torch.zeros_like(out)
            dK2 = [dev(K) for K, _ in caches]
            dV2 = [dev(V) for _, V in caches]
            for l in range(layers):
                ops.attn_decode(dq[l], dk[l], dv[l], dK2[l], dV2[l], eager[l], n_head, n_kv, hd, n_ctx, d_pos, float(scale),
                                ops.FUSE_ALL, rope, ws)
            torch.cuda.synchronize()
            assert torch.equal(out, eager)
            return out.cpu().numpy()
        finally:
            ops.set_decode_overlap(0)

    base = run(0)
    got = run(mode)
    assert np.array_equal(got, base)
    for l in (0, layers - 1):
        K, V = caches[l]
        want = oracle.attn_batch(qs[l][None].copy(), ks[l][None].copy(), vs[l][None].copy(), K.astype(np.float32),
                                 V.astype(np.float32), pos, scale, True, 1, hd, 1e6, None)[0]
        assert_close(got[l], want, "mode %d layer %d" % (mode, l))


def test_unfused_store_then_decode_under_early_fetch(ops, oracle):
    """The reference's unfused decode sequence (src/model_gpu.cu:281-282): kv_store_ind writes row *d_pos, the decode call
    right behind it reads it.  Under launch ordering 2 the decode kernel fetches cache tiles before it waits for the
    store kernel; the newest row must still be the stored one.  Several layers captured in one graph, compared bit
    for bit with ordinary launches and with the oracle."""
    n_head, n_kv, hd, n_ctx, layers, pos = 28, 4, 128, 2048, 5, 1500
    scale = np.float32(1.0 / np.sqrt(hd))
    rng = np.random.default_rng(91)
    caches, qs, ks, vs = [], [], [], []
    for l in range(layers):
        q, K, V = make_qkv(910 + l, n_head, n_kv, hd, pos, n_ctx)
        # the row that the store will overwrite holds a decoy: a stale read would change the result visibly
        K[:, pos] = np.float16(3.0)
        V[:, pos] = np.float16(-7.0)
        caches.append((K, V))
        qs.append(q[0])
        ks.append(f16_round(rng.standard_normal((n_kv, hd)).astype(np.float32)))
        vs.append(f16_round(rng.standard_normal((n_kv, hd)).astype(np.float32)))
    d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    dq, dk, dv = dev(np.stack(qs)), dev(np.stack(ks)), dev(np.stack(vs))
    ws = ops.decode_workspace(n_head, n_kv, hd)

    def run(mode):
        ops.set_decode_overlap(mode)
        try:
            dK = [dev(K) for K, _ in caches]
            dV = [dev(V) for _, V in caches]
            out = torch.zeros(layers, n_head, hd, device="cuda")
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                ops.set_stream(stream)
                try:
                    graph.capture_begin()
                    for l in range(layers):
                        ops.kv_store_ind(dK[l], dV[l], dk[l], dv[l], n_kv, hd, n_ctx, d_pos)
                        ops.flash_attention_decode_ind(dq[l], dK[l], dV[l], out[l], n_head, n_kv, hd, n_ctx, d_pos, float(scale), ws)
                    graph.capture_end()
                finally:
                    ops.set_stream(None)
            graph.replay()
            torch.cuda.synchronize()
            return out.cpu().numpy()
        finally:
            ops.set_decode_overlap(0)

    base = run(0)
    got = run(2)
    assert np.array_equal(got, base)
    for l in (0, layers - 1):
        K, V = caches[l]
        kc32, vc32 = K.astype(np.float32), V.astype(np.float32)
        kc32[:, pos] = ks[l]
        vc32[:, pos] = vs[l]
        want = oracle.attend(qs[l], kc32, vc32, pos + 1, scale)
        assert_close(got[l], want, "unfused sequence, early fetch, layer %d" % l)


def test_many_workspaces_do_not_share_arrival_counters(ops, oracle):
    """More distinct workspaces than the library has counter slots, used one after the other and then again: every call
    must still merge completely (a slot is recycled only when its previous user is at rest)."""
    n_head, n_kv, hd, npos = 16, 2, 128, 9000
    q, K, V = make_qkv(77, n_head, n_kv, hd, npos)
    scale = np.float32(1.0 / np.sqrt(hd))
    want = oracle.attend(q[0], K.astype(np.float32), V.astype(np.float32), npos, scale)
    nbytes = ops.decode_workspace(n_head, n_kv, hd).numel()
    spaces = [torch.empty(nbytes, dtype=torch.uint8, device="cuda") for _ in range(70)]
    first = None
    for rnd in range(2):
        for ws in spaces[:: 1 if rnd == 0 else 7]:
            got = run_decode(ops, q[0], K, V, npos, float(scale), workspace=ws)
            if first is None:
                first = got
                assert_close(got, want, "first workspace")
            assert np.array_equal(got, first)
