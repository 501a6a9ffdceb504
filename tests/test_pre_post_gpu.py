"""The steps on either side of attention folded into the attention launches: q/k/v bias add and per-head q/k RMSNorm in
front (src/model_gpu.cu:372-377, src/model_cpu.cpp:258-274), the q8_1 activation form of the decode output behind
(src/model_gpu.cu:284, src/kernels.cu:136-145).  Checked against fixtures produced by the reference's forward() on
layers that carry biases and norm weights, against the CPU oracle on larger random cases, and against the reference's
own CUDA kernels for the same steps."""
import os

import numpy as np
import pytest
import torch

from helpers import assert_close, assert_f16_rows_match, f16_round, make_qkv

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def load_pre_probe(name):
    g = np.load(os.path.join(GOLD, name + ".npz"))
    opt = {k: (g[k] if g[k].size else None) for k in ("bias_q", "bias_k", "bias_v", "norm_q", "norm_k")}
    return g, opt


def dev_ext(opt, eps):
    ext = {k: dev(v) for k, v in opt.items() if v is not None}
    ext["norm_eps"] = float(eps)
    return ext


@pytest.mark.parametrize("name", ["probe_pre_qwen2", "probe_pre_qwen3"])
def test_fused_bias_and_norm_match_reference_fixture(ops, name):
    """Decode token by token, and the same tokens as one prefill chunk, from the projections the reference computed."""
    g, opt = load_pre_probe(name)
    n_head, n_kv, d, n_ctx = int(g["n_head"]), int(g["n_kv"]), int(g["d"]), int(g["n_ctx"])
    rope = (int(g["rope_type"]), int(g["n_rot"]), float(g["theta"]), None)
    scale = float(1.0 / np.sqrt(d))
    ext = dev_ext(opt, g["eps"])
    n_tok = g["q_pre"].shape[0]
    # decode
    kc = torch.zeros(n_kv, n_ctx, d, dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    for t in range(n_tok):
        out = torch.empty(n_head, d, device="cuda")
        d_pos = torch.tensor([t], dtype=torch.int32, device="cuda")
        ops.attn_decode(dev(g["q_pre"][t]), dev(g["k_pre"][t]), dev(g["v_pre"][t]), kc, vc, out, n_head, n_kv, d, n_ctx, d_pos,
                        scale, ops.FUSE_ALL, rope, ext=ext)
        torch.cuda.synchronize()
        assert_close(out.cpu().numpy(), g["attn"][t], "%s decode token %d" % (name, t))
    assert_f16_rows_match(kc[:, :n_tok].cpu().numpy(), np.transpose(g["k_rot"], (1, 0, 2)), name + " K rows")
    v_want = g["v_pre"] + (opt["bias_v"].reshape(n_kv, d) if opt["bias_v"] is not None else 0.0)
    assert np.array_equal(vc[:, :n_tok].cpu().numpy(), np.transpose(v_want, (1, 0, 2)).astype(np.float16))
    # prefill, both kernels
    for impl in (0, 1):
        ops.set_prefill_impl(impl)
        try:
            kc2 = torch.zeros_like(kc)
            vc2 = torch.zeros_like(kc)
            out = torch.empty(n_tok, n_head, d, device="cuda")
            ops.attn_prefill(dev(g["q_pre"]), dev(g["k_pre"]), dev(g["v_pre"]), kc2, vc2, out, n_head, n_kv, d, n_ctx, 0, n_tok,
                             scale, ops.FUSE_ALL, rope, ext=ext)
            torch.cuda.synchronize()
        finally:
            ops.set_prefill_impl(0)
        assert_close(out.cpu().numpy(), g["attn"], "%s prefill impl %d" % (name, impl))
        assert torch.equal(kc2.view(torch.int16), kc.view(torch.int16))
        assert torch.equal(vc2.view(torch.int16), vc.view(torch.int16))


def random_ext(rng, n_head, n_kv, hd, bias=True, norm=True):
    opt = dict(bias_q=None, bias_k=None, bias_v=None, norm_q=None, norm_k=None)
    if bias:
        opt["bias_q"] = (0.5 * rng.standard_normal(n_head * hd)).astype(np.float32)
        opt["bias_k"] = (0.5 * rng.standard_normal(n_kv * hd)).astype(np.float32)
        opt["bias_v"] = (0.5 * rng.standard_normal(n_kv * hd)).astype(np.float32)
    if norm:
        opt["norm_q"] = (1.0 + 0.3 * rng.standard_normal(hd)).astype(np.float32)
        opt["norm_k"] = (1.0 + 0.3 * rng.standard_normal(hd)).astype(np.float32)
    return opt


@pytest.mark.parametrize("bias,norm", [(True, False), (False, True), (True, True)])
def test_fused_pre_attention_long_context_vs_oracle(ops, oracle, bias, norm):
    n_head, n_kv, hd, n_ctx, pos = 28, 4, 128, 3072, 3000
    scale = np.float32(1.0 / np.sqrt(hd))
    rng = np.random.default_rng(40 + 2 * bias + norm)
    _, K, V = make_qkv(41, n_head, n_kv, hd, pos, n_ctx)
    opt = random_ext(rng, n_head, n_kv, hd, bias, norm)
    q = rng.standard_normal((1, n_head, hd)).astype(np.float32)
    k = rng.standard_normal((1, n_kv, hd)).astype(np.float32)
    v = rng.standard_normal((1, n_kv, hd)).astype(np.float32)
    qo, ko, vo = q.copy(), k.copy(), v.copy()
    oracle.pre_attention(qo, ko, vo, eps=1e-6, **opt)
    vo = f16_round(vo)       # the device cache holds fp16(v + bias)
    kc32, vc32 = K.astype(np.float32), V.astype(np.float32)
    want = oracle.attn_batch(qo, ko, vo, kc32, vc32, pos, scale, True, 1, hd, 1e6, None)[0]
    dK, dV = dev(K), dev(V)
    out = torch.empty(n_head, hd, device="cuda")
    d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    ops.attn_decode(dev(q[0]), dev(k[0]), dev(v[0]), dK, dV, out, n_head, n_kv, hd, n_ctx, d_pos, float(scale), ops.FUSE_ALL,
                    (1, hd, 1e6, None), ext=dev_ext(opt, 1e-6))
    torch.cuda.synchronize()
    assert_close(out.cpu().numpy(), want, "decode with bias=%s norm=%s" % (bias, norm))
    assert_f16_rows_match(dK[:, pos].cpu().numpy(), ko[0], "appended K row")


def test_fused_pre_attention_prefill_chunk_vs_oracle(ops, oracle):
    n_head, n_kv, hd, n_ctx, n_past, batch = 32, 8, 128, 512, 200, 96
    scale = np.float32(1.0 / np.sqrt(hd))
    rng = np.random.default_rng(50)
    _, K, V = make_qkv(51, n_head, n_kv, hd, n_past, n_ctx)
    opt = random_ext(rng, n_head, n_kv, hd)
    q = rng.standard_normal((batch, n_head, hd)).astype(np.float32)
    k = rng.standard_normal((batch, n_kv, hd)).astype(np.float32)
    v = rng.standard_normal((batch, n_kv, hd)).astype(np.float32)
    qo, ko, vo = q.copy(), k.copy(), v.copy()
    oracle.pre_attention(qo, ko, vo, eps=1e-5, **opt)
    vo = f16_round(vo)
    want = oracle.attn_batch(qo, ko, vo, K.astype(np.float32), V.astype(np.float32), n_past, scale, True, 0, hd, 5e5, None)
    dK, dV = dev(K), dev(V)
    out = torch.empty(batch, n_head, hd, device="cuda")
    ops.attn_prefill(dev(q), dev(k), dev(v), dK, dV, out, n_head, n_kv, hd, n_ctx, n_past, batch, float(scale), ops.FUSE_ALL,
                     (0, hd, 5e5, None), ext=dev_ext(opt, 1e-5))
    torch.cuda.synchronize()
    assert ops.prefill_status(n_head, n_kv, hd, batch) == 0
    assert_close(out.cpu().numpy(), want, "prefill with bias and norm")


def test_pre_attention_against_reference_cuda_kernels(ops, refcuda):
    """add_inplace_broadcast x3, rms_norm_rows x2, rope x2, kv_store, attention of the reference (src/model_gpu.cu:372-384)
    against the one fused call."""
    n_head, n_kv, hd, n_ctx, n_past, batch = 16, 2, 128, 256, 40, 24
    scale = float(1.0 / np.sqrt(hd))
    rng = np.random.default_rng(60)
    _, K, V = make_qkv(61, n_head, n_kv, hd, n_past, n_ctx)
    opt = random_ext(rng, n_head, n_kv, hd)
    q = rng.standard_normal((batch, n_head, hd)).astype(np.float32)
    k = rng.standard_normal((batch, n_kv, hd)).astype(np.float32)
    v = rng.standard_normal((batch, n_kv, hd)).astype(np.float32)
    ext = dev_ext(opt, 1e-6)
    rq, rk, rv, rK, rV = dev(q), dev(k), dev(v), dev(K), dev(V)
    refcuda.add_inplace_broadcast(rq, ext["bias_q"], n_head * hd, batch)
    refcuda.add_inplace_broadcast(rk, ext["bias_k"], n_kv * hd, batch)
    refcuda.add_inplace_broadcast(rv, ext["bias_v"], n_kv * hd, batch)
    refcuda.rms_norm_rows(rq, ext["norm_q"], batch * n_head, hd, 1e-6, rq)
    refcuda.rms_norm_rows(rk, ext["norm_k"], batch * n_kv, hd, 1e-6, rk)
    refcuda.rope_batch(rq, 1, batch * n_head, hd, hd, 1e6, n_past, n_head)
    refcuda.rope_batch(rk, 1, batch * n_kv, hd, hd, 1e6, n_past, n_kv)
    refcuda.kv_store_batch(rK, rV, rk, rv, n_kv, hd, n_ctx, n_past, batch)
    r_out = torch.empty(batch, n_head, hd, device="cuda")
    refcuda.flash_attention(rq, rK, rV, r_out, n_head, n_kv, hd, n_ctx, n_past, batch, scale)
    mK, mV = dev(K), dev(V)
    m_out = torch.empty(batch, n_head, hd, device="cuda")
    ops.attn_prefill(dev(q), dev(k), dev(v), mK, mV, m_out, n_head, n_kv, hd, n_ctx, n_past, batch, scale, ops.FUSE_ALL,
                     (1, hd, 1e6, None), ext=ext)
    torch.cuda.synchronize()
    assert_close(m_out.cpu().numpy(), r_out.cpu().numpy(), "fused pre-attention vs reference kernels")
    assert torch.equal(mV.view(torch.int16), rV.view(torch.int16))


@pytest.mark.parametrize("n_head,n_kv,hd,npos", [(16, 2, 128, 5000), (28, 4, 128, 40), (12, 2, 64, 700), (8, 8, 128, 1)])
def test_q8_1_output_is_the_quantised_fp32_output(ops, oracle, n_head, n_kv, hd, npos):
    """The int8/scale pair written by the decode call equals the reference quantiser's formula applied to the fp32
    output of the same call, bit for bit; with `out` omitted the pair is unchanged.  Covers the merge-kernel path and
    the single-split path (short contexts) that writes the output from the split kernel."""
    scale = float(1.0 / np.sqrt(hd))
    q, K, V = make_qkv(70 + npos, n_head, n_kv, hd, npos)
    dq, dK, dV = dev(q[0]), dev(K), dev(V)
    d_pos = torch.tensor([npos - 1], dtype=torch.int32, device="cuda")
    n = n_head * hd
    out = torch.empty(n_head, hd, device="cuda")
    qs = torch.full((n,), 99, dtype=torch.int8, device="cuda")
    sc = torch.full((n // 32,), -1.0, device="cuda")
    ops.attn_decode(dq, None, None, dK, dV, out, n_head, n_kv, hd, npos, d_pos, scale, ops.FUSE_NONE,
                    ext=dict(out_qs=qs, out_scales=sc))
    torch.cuda.synchronize()
    want_q, want_s = oracle.quantize_q8_1(out.cpu().numpy())
    assert np.array_equal(qs.cpu().numpy(), want_q)
    assert np.array_equal(sc.cpu().numpy(), want_s)
    plain = torch.empty(n_head, hd, device="cuda")
    ops.attn_decode(dq, None, None, dK, dV, plain, n_head, n_kv, hd, npos, d_pos, scale, ops.FUSE_NONE)
    qs2, sc2 = torch.zeros_like(qs), torch.zeros_like(sc)
    ops.attn_decode(dq, None, None, dK, dV, None, n_head, n_kv, hd, npos, d_pos, scale, ops.FUSE_NONE,
                    ext=dict(out_qs=qs2, out_scales=sc2))
    torch.cuda.synchronize()
    assert torch.equal(plain, out) and torch.equal(qs2, qs) and torch.equal(sc2, sc)


def test_q8_1_output_against_reference_quantise_kernel(ops, refcuda):
    """quantize_activation of the reference (fast-math build) on the fp32 output: same scales to an ulp, values equal
    except where fast division lands on the other side of a rounding boundary (at most one step, rarely)."""
    n_head, n_kv, hd, npos = 28, 4, 128, 2000
    scale = float(1.0 / np.sqrt(hd))
    q, K, V = make_qkv(80, n_head, n_kv, hd, npos, 2048)
    d_pos = torch.tensor([npos - 1], dtype=torch.int32, device="cuda")
    n = n_head * hd
    out = torch.empty(n_head, hd, device="cuda")
    qs = torch.empty(n, dtype=torch.int8, device="cuda")
    sc = torch.empty(n // 32, device="cuda")
    ops.attn_decode(dev(q[0]), None, None, dev(K), dev(V), out, n_head, n_kv, hd, 2048, d_pos, scale, ops.FUSE_NONE,
                    ext=dict(out_qs=qs, out_scales=sc))
    torch.cuda.synchronize()
    r_qs, r_sc = refcuda.quantize_activation(out, n)
    assert torch.allclose(sc, r_sc, rtol=1e-6, atol=0)
    diff = (qs.int() - r_qs.int()).abs()
    assert int(diff.max()) <= 1 and float((diff != 0).float().mean()) < 5e-3


def test_extension_argument_errors(ops):
    from orin_llm_b200 import capi
    n_head, n_kv, hd, n_ctx = 8, 2, 128, 128
    q = torch.zeros(n_head, hd, device="cuda")
    kc = torch.zeros(n_kv, n_ctx, hd, dtype=torch.float16, device="cuda")
    out = torch.zeros(n_head, hd, device="cuda")
    d_pos = torch.tensor([5], dtype=torch.int32, device="cuda")
    bias_k = torch.zeros(n_kv * hd, device="cuda")
    qs = torch.zeros(n_head * hd, dtype=torch.int8, device="cuda")
    sc = torch.zeros(n_head * hd // 32, device="cuda")
    with pytest.raises(capi.AttnError) as e:     # k bias without the fused append
        ops.attn_decode(q, None, None, kc, kc, out, n_head, n_kv, hd, n_ctx, d_pos, 0.1, ops.FUSE_NONE, ext=dict(bias_k=bias_k))
    assert e.value.code == capi.ERR_ARG
    with pytest.raises(capi.AttnError) as e:     # values without scales
        ops.attn_decode(q, None, None, kc, kc, out, n_head, n_kv, hd, n_ctx, d_pos, 0.1, ops.FUSE_NONE, ext=dict(out_qs=qs))
    assert e.value.code == capi.ERR_ARG
    with pytest.raises(capi.AttnError) as e:     # no output at all
        ops.attn_decode(q, None, None, kc, kc, None, n_head, n_kv, hd, n_ctx, d_pos, 0.1, ops.FUSE_NONE)
    assert e.value.code == capi.ERR_ARG
    qb = torch.zeros(4, n_head, hd, device="cuda")
    ob = torch.zeros(4, n_head, hd, device="cuda")
    with pytest.raises(capi.AttnError) as e:     # q8_1 output is a decode-only extra
        ops.attn_prefill(qb, None, None, kc, kc, ob, n_head, n_kv, hd, n_ctx, 0, 4, 0.1, ops.FUSE_NONE,
                         ext=dict(out_qs=qs, out_scales=sc))
    assert e.value.code == capi.ERR_UNSUPPORTED


def _mmq_fields(blocks, ds4):
    """uint8 [..., 144] -> (scales fp32 [..., 4], sums fp32 [..., 4] or None, int8 values [..., 128])."""
    b = np.ascontiguousarray(blocks)
    head = b[..., :16]
    qs = b[..., 16:].copy().view(np.int8)
    if ds4:
        h = head.copy().view(np.float16).astype(np.float32).reshape(b.shape[:-1] + (4, 2))
        return h[..., 0], h[..., 1], qs
    return head.copy().view(np.float32).reshape(b.shape[:-1] + (4,)), None, qs


@pytest.mark.parametrize("ds4", [False, True])
@pytest.mark.parametrize("n_head,n_kv,n_past,batch", [(32, 8, 4096, 512), (12, 2, 0, 45), (28, 4, 100, 37)])
def test_prefill_mmq_output_is_the_quantised_fp32_output(ops, oracle, ds4, n_head, n_kv, n_past, batch):
    """The block_q8_1_mmq blocks written by the prefill call equal the restated quantiser (src/kernels.cu:160-205)
    applied to the fp32 output of the same call: values and fp32 scales bit for bit, the fp16 group sums to fp16
    rounding (the kernel adds a group's 32 values in another order); with `out` omitted the blocks are unchanged."""
    hd = 128
    n_ctx = n_past + batch
    scale = float(1.0 / np.sqrt(hd))
    gen = torch.Generator("cuda").manual_seed(5 + n_past)
    K = torch.randn(n_kv, n_ctx, hd, device="cuda", dtype=torch.float16, generator=gen)
    V = torch.randn(n_kv, n_ctx, hd, device="cuda", dtype=torch.float16, generator=gen)
    q = torch.randn(batch, n_head, hd, device="cuda", generator=gen).half().float()
    out = torch.empty(batch, n_head, hd, device="cuda")
    blk = torch.full((n_head, batch, 144), 0x5A, dtype=torch.uint8, device="cuda")
    ops.attn_prefill(q, None, None, K, V, out, n_head, n_kv, hd, n_ctx, n_past, batch, scale, ops.FUSE_NONE,
                     ext=dict(out_mmq=blk, out_mmq_ds4=ds4))
    torch.cuda.synchronize()
    assert ops.prefill_status(n_head, n_kv, hd, batch) == 0
    want = oracle.quantize_mmq_q8_1(out.cpu().numpy().reshape(batch, n_head * hd), ds4)
    gd, gs, gq = _mmq_fields(blk.cpu().numpy(), ds4)
    wd, ws, wq = _mmq_fields(want, ds4)
    assert np.array_equal(gq, wq)
    assert np.array_equal(gd, wd)
    if ds4:
        assert np.allclose(gs, ws, rtol=2e-3, atol=2e-3)
    plain = torch.empty_like(out)
    ops.attn_prefill(q, None, None, K, V, plain, n_head, n_kv, hd, n_ctx, n_past, batch, scale, ops.FUSE_NONE)
    blk2 = torch.zeros_like(blk)
    ops.attn_prefill(q, None, None, K, V, None, n_head, n_kv, hd, n_ctx, n_past, batch, scale, ops.FUSE_NONE,
                     ext=dict(out_mmq=blk2, out_mmq_ds4=ds4))
    torch.cuda.synchronize()
    assert torch.equal(plain, out) and torch.equal(blk2, blk)


@pytest.mark.parametrize("ggml_type,ds4", [(12, True), (14, False)])
def test_prefill_mmq_output_against_the_reference_quantise_pass(ops, oracle, refcuda, ggml_type, ds4):
    """The reference's own quantize_mmq_q8_1_k, run the way its batched GEMM runs it (gemv_batch on a Q4_K / Q6_K weight,
    src/kernels.cu:1842-1850), on the fp32 output of the prefill call: same block layout and scales (to an ulp of its
    fast-math division), values equal except for a rare one-step difference on a rounding boundary."""
    import sys
    import os
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "e2e"))
    import make_gguf
    if not hasattr(refcuda.L, "refcuda_gemv_batch"):
        pytest.skip("oracle/_ref/libref_cuda.so predates refcuda_gemv_batch")
    n_head, n_kv, hd, n_past, batch = 32, 8, 128, 512, 64
    n_ctx = n_past + batch
    scale = float(1.0 / np.sqrt(hd))
    gen = torch.Generator("cuda").manual_seed(17)
    K = torch.randn(n_kv, n_ctx, hd, device="cuda", dtype=torch.float16, generator=gen)
    V = torch.randn(n_kv, n_ctx, hd, device="cuda", dtype=torch.float16, generator=gen)
    q = torch.randn(batch, n_head, hd, device="cuda", generator=gen).half().float()
    out = torch.empty(batch, n_head, hd, device="cuda")
    blk = torch.zeros(n_head, batch, 144, dtype=torch.uint8, device="cuda")
    ops.attn_prefill(q, None, None, K, V, out, n_head, n_kv, hd, n_ctx, n_past, batch, scale, ops.FUSE_NONE,
                     ext=dict(out_mmq=blk, out_mmq_ds4=ds4))
    torch.cuda.synchronize()
    n_in, n_out = n_head * hd, 128
    rng = np.random.default_rng(3)
    w = make_gguf.q4_k_bytes(rng, n_out, n_in) if ggml_type == 12 else make_gguf.q6_k_bytes(rng, n_out, n_in)
    r_blk, _ = refcuda.quantize_mmq(out.view(batch, n_in), ggml_type, dev(w.reshape(-1)), n_out)
    assert r_blk.shape == blk.shape
    gd, gs, gq = _mmq_fields(blk.cpu().numpy(), ds4)
    rd, rs, rq = _mmq_fields(r_blk.cpu().numpy(), ds4)
    assert np.allclose(gd, rd, rtol=2e-3 if ds4 else 1e-6, atol=0)
    diff = np.abs(gq.astype(np.int32) - rq.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 5e-3
    if ds4:
        assert np.allclose(gs, rs, rtol=2e-3, atol=2e-3)
