"""GPU parity tests of the chunked-prefill path (through the C ABI) against the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from helpers import assert_close, assert_f16_rows_match, f16_round, make_qkv

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
IMPLS = [0, 1]   # 0 = tcgen05 kernel (falls back to the mma kernel for shapes it does not cover), 1 = mma.sync kernel


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def oracle_prefill(oracle, q, K, V, n_past, scale):
    """q [batch][n_head][hd]; K,V hold rows [0, n_past+batch) already (fp16 values)."""
    batch = q.shape[0]
    kc, vc = K.astype(np.float32), V.astype(np.float32)
    out = np.empty_like(q)
    for b in range(batch):
        out[b] = oracle.attend(q[b], kc, vc, n_past + b + 1, scale)
    return out


SHAPES = [  # n_head, n_kv, hd, n_past, batch
    (32, 8, 128, 0, 1), (32, 8, 128, 0, 45), (12, 2, 128, 0, 45), (28, 4, 128, 100, 33), (32, 8, 128, 64, 64),
    (32, 8, 128, 127, 130), (4, 4, 128, 5, 70), (8, 1, 128, 0, 40), (8, 2, 64, 17, 50), (16, 1, 64, 3, 21),
    (32, 8, 128, 1000, 512),
]


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("n_head,n_kv,hd,n_past,batch", SHAPES)
def test_prefill_matches_oracle(ops, oracle, impl, n_head, n_kv, hd, n_past, batch):
    n_rows = n_past + batch
    n_ctx = ((n_rows + 63) // 64) * 64 + 64
    q, K, V = make_qkv(2000 + n_rows, n_head, n_kv, hd, n_rows, n_ctx, batch)
    # rows after the chunk are poison: the causal mask must hide them
    K[:, n_rows:] = np.float16(np.nan); V[:, n_rows:] = np.float16(np.nan)
    scale = np.float32(1.0 / np.sqrt(hd))
    out = torch.empty(batch, n_head, hd, device="cuda")
    ops.set_prefill_impl(impl)
    try:
        ops.flash_attention(dev(q), dev(K), dev(V), out, n_head, n_kv, hd, n_ctx, n_past, batch, float(scale))
        torch.cuda.synchronize()
        assert ops.prefill_status(n_head, n_kv, hd, batch) == 0, "kernel reported a timed-out wait"
    finally:
        ops.set_prefill_impl(0)
    want = oracle_prefill(oracle, q, K[:, :n_rows], V[:, :n_rows], n_past, scale)
    assert_close(out.cpu().numpy(), want, "prefill impl %d %s" % (impl, (n_head, n_kv, hd, n_past, batch)))


@pytest.mark.parametrize("impl", IMPLS)
def test_prefill_causal_mask_is_exact(ops, impl):
    """Token t's output must not change when K/V rows after n_past+t change."""
    n_head, n_kv, hd, n_past, batch = 32, 8, 128, 70, 96
    n_rows = n_past + batch
    q, K, V = make_qkv(41, n_head, n_kv, hd, n_rows, 256, batch)
    scale = float(1.0 / np.sqrt(hd))
    ops.set_prefill_impl(impl)
    try:
        out_a = torch.empty(batch, n_head, hd, device="cuda")
        ops.flash_attention(dev(q), dev(K), dev(V), out_a, n_head, n_kv, hd, 256, n_past, batch, scale)
        cut = 40
        K2, V2 = K.copy(), V.copy()
        K2[:, n_past + cut + 1:] *= np.float16(-3); V2[:, n_past + cut + 1:] += np.float16(7)
        out_b = torch.empty_like(out_a)
        ops.flash_attention(dev(q), dev(K2), dev(V2), out_b, n_head, n_kv, hd, 256, n_past, batch, scale)
        torch.cuda.synchronize()
    finally:
        ops.set_prefill_impl(0)
    assert torch.equal(out_a[:cut + 1], out_b[:cut + 1])
    assert not torch.equal(out_a[cut + 1:], out_b[cut + 1:])


@pytest.mark.parametrize("impl", IMPLS)
def test_fused_prefill_matches_reference_fixture(ops, impl):
    """One fused prefill call (RoPE q, RoPE k, append, causal attention) over the tokens the reference's
    forward() processed one by one; outputs compared with what the reference produced."""
    ops.set_prefill_impl(impl)
    try:
        for name in ("probe_neox", "probe_normal", "probe_partial"):
            g = np.load(os.path.join(GOLD, name + ".npz"))
            n_head, n_kv, d, n_ctx = int(g["n_head"]), int(g["n_kv"]), int(g["d"]), int(g["n_ctx"])
            ff = dev(g["freq_factors"]) if g["freq_factors"].size else None
            rope = (int(g["rope_type"]), int(g["n_rot"]), float(g["theta"]), ff)
            n_tok = g["q_pre"].shape[0]
            kc = torch.zeros(n_kv, n_ctx, d, dtype=torch.float16, device="cuda")
            vc = torch.zeros_like(kc)
            out = torch.empty(n_tok, n_head, d, device="cuda")
            # two chunks, to cover n_past > 0 with the fused append
            first = n_tok // 2
            for (a, b) in ((0, first), (first, n_tok)):
                ops.attn_prefill(dev(g["q_pre"][a:b]), dev(g["k_pre"][a:b]), dev(g["v_pre"][a:b]), kc, vc, out[a:b],
                                 n_head, n_kv, d, n_ctx, a, b - a, float(1.0 / np.sqrt(d)), ops.FUSE_ALL, rope)
            torch.cuda.synchronize()
            assert_close(out.cpu().numpy(), g["attn"], name)
            want_k = np.transpose(g["k_rot"], (1, 0, 2)).astype(np.float16)
            assert np.array_equal(kc.cpu().numpy()[:, :n_tok].view(np.uint16), want_k.view(np.uint16)), name
    finally:
        ops.set_prefill_impl(0)


@pytest.mark.parametrize("n_past", [0, 4096, 8192])
def test_prefill_isolated_llama3_8b_shape(ops, oracle, n_past):
    """32 query / 8 kv heads, head_dim 128, chunk of 512 queries at KV offset n_past, RoPE theta 5e5 (normal
    pairing) applied to Q and K, N(0,1) inputs.  The oracle runs on a subset of (token, head) rows."""
    n_head, n_kv, hd, batch, theta = 32, 8, 128, 512, 5e5
    n_ctx = n_past + batch
    scale = np.float32(1.0 / np.sqrt(hd))
    rng = np.random.default_rng(50 + n_past)
    q = rng.standard_normal((batch, n_head, hd), dtype=np.float32)
    k_new = rng.standard_normal((batch, n_kv, hd), dtype=np.float32)
    v_new = f16_round(rng.standard_normal((batch, n_kv, hd), dtype=np.float32))
    # history: already-rotated fp16 rows
    K = np.zeros((n_kv, n_ctx, hd), np.float16); V = np.zeros_like(K)
    K[:, :n_past] = rng.standard_normal((n_kv, n_past, hd), dtype=np.float32).astype(np.float16)
    V[:, :n_past] = rng.standard_normal((n_kv, n_past, hd), dtype=np.float32).astype(np.float16)
    dK, dV = dev(K), dev(V)
    out = torch.empty(batch, n_head, hd, device="cuda")
    ops.attn_prefill(dev(q), dev(k_new), dev(v_new), dK, dV, out, n_head, n_kv, hd, n_ctx, n_past, batch, float(scale),
                     ops.FUSE_ALL, (0, hd, theta, None))
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    # oracle: rotate with the reference arithmetic, fp16 cache image, then attend for sampled rows
    kr = k_new.copy()
    for b in range(batch):
        oracle.rope_rows(kr[b], 0, hd, theta, [n_past + b] * n_kv)
    kc32, vc32 = K.astype(np.float32), V.astype(np.float32)
    kc32[:, n_past:] = f16_round(np.transpose(kr, (1, 0, 2)))
    vc32[:, n_past:] = np.transpose(v_new, (1, 0, 2))
    assert_f16_rows_match(dK.cpu().numpy()[:, n_past:], np.transpose(kr, (1, 0, 2)), "appended K rows")
    for b in (0, 1, 63, 64, 200, 511):
        qb = q[b].copy()
        oracle.rope_rows(qb, 0, hd, theta, [n_past + b] * n_head)
        want = oracle.attend(qb, kc32, vc32, n_past + b + 1, scale)
        assert_close(got[b], want, "prefill n_past=%d token %d" % (n_past, b))
