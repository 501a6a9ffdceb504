"""GPU against GPU: this repository's kernels next to the reference's own CUDA kernels (src/kernels.cu, compiled
unmodified for sm_100a) on the same device buffers.  The CPU oracle stays the parity gate; this second check shows
that the replacement and the replaced code agree on the reference's own data layout and call sequence
(src/model_gpu.cu:277-282 and :379-384).  Shapes respect the reference kernels' limits: group <= 8, n_ctx % 128 == 0."""
import numpy as np
import pytest
import torch

from helpers import assert_close, make_qkv

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("n_head,n_kv,L,n_ctx", [(12, 2, 173, 256), (28, 4, 1024, 1024), (28, 4, 4000, 4096),
                                                  (16, 2, 32768, 32768), (32, 8, 640, 1024)])
def test_decode_against_reference_kernel(ops, refcuda, oracle, n_head, n_kv, L, n_ctx):
    hd = 128
    scale = float(1.0 / np.sqrt(hd))
    q, K, V = make_qkv(1000 + L, n_head, n_kv, hd, L, n_ctx)
    dq, dK, dV = dev(q[0]), dev(K), dev(V)
    d_pos = torch.tensor([L - 1], dtype=torch.int32, device="cuda")
    mine = torch.empty(n_head, hd, device="cuda")
    ref = torch.empty(n_head, hd, device="cuda")
    ops.flash_attention_decode_ind(dq, dK, dV, mine, n_head, n_kv, hd, n_ctx, d_pos, scale)
    refcuda.flash_attention_decode_ind(dq, dK, dV, ref, n_head, n_kv, hd, n_ctx, d_pos, scale)
    torch.cuda.synchronize()
    assert_close(mine.cpu().numpy(), ref.cpu().numpy(), "decode vs reference kernel L=%d" % L)
    if L <= 4096:
        want = oracle.attend(q[0], K.astype(np.float32), V.astype(np.float32), L, np.float32(scale))
        e_mine = np.abs(mine.cpu().numpy() - want).max()
        e_ref = np.abs(ref.cpu().numpy() - want).max()
        # the replacement is at least as close to the fp32 oracle as the kernel it replaces (fp16 scale and fp16
        # q*scale in the reference cost it a little), with a small allowance
        assert e_mine <= max(2 * e_ref, 2e-3), (e_mine, e_ref)


@pytest.mark.parametrize("n_head,n_kv,n_past,batch,n_ctx", [(32, 8, 0, 64, 128), (32, 8, 300, 128, 512),
                                                           (12, 2, 0, 45, 128), (28, 4, 1000, 24, 1024)])
def test_prefill_sequence_against_reference_kernels(ops, refcuda, n_head, n_kv, n_past, batch, n_ctx):
    """The reference's prefill sequence rope(q), rope(k), kv_store_batch, flash_attention on one set of buffers and
    the fused call on another: same cache rows (to fp16 rounding of slightly different sin/cos), same output."""
    hd, theta, rope_type = 128, 5e5, 0
    scale = float(1.0 / np.sqrt(hd))
    rng = np.random.default_rng(2000 + n_past + batch)
    _, K, V = make_qkv(2100 + batch, n_head, n_kv, hd, n_past, n_ctx)
    q = rng.standard_normal((batch, n_head, hd)).astype(np.float32)
    k = rng.standard_normal((batch, n_kv, hd)).astype(np.float32)
    v = rng.standard_normal((batch, n_kv, hd)).astype(np.float32)
    # reference sequence (in place on q and k)
    rq, rk, rv = dev(q), dev(k), dev(v)
    rK, rV = dev(K), dev(V)
    r_out = torch.empty(batch, n_head, hd, device="cuda")
    refcuda.rope_batch(rq, rope_type, batch * n_head, hd, hd, theta, n_past, n_head)
    refcuda.rope_batch(rk, rope_type, batch * n_kv, hd, hd, theta, n_past, n_kv)
    refcuda.kv_store_batch(rK, rV, rk, rv, n_kv, hd, n_ctx, n_past, batch)
    refcuda.flash_attention(rq, rK, rV, r_out, n_head, n_kv, hd, n_ctx, n_past, batch, scale)
    # fused call
    mK, mV = dev(K), dev(V)
    m_out = torch.empty(batch, n_head, hd, device="cuda")
    ops.attn_prefill(dev(q), dev(k), dev(v), mK, mV, m_out, n_head, n_kv, hd, n_ctx, n_past, batch, scale, ops.FUSE_ALL,
                     (rope_type, hd, theta, None))
    torch.cuda.synchronize()
    assert ops.prefill_status(n_head, n_kv, hd, batch) == 0
    assert_close(m_out.cpu().numpy(), r_out.cpu().numpy(), "prefill vs reference kernels")
    # V rows are a plain fp32 -> fp16 conversion: identical bits
    assert torch.equal(mV.view(torch.int16), rV.view(torch.int16))
    # K rows differ only through the rotation's sin/cos (fast-math in the reference)
    dk = (mK.float() - rK.float()).abs().max().item()
    assert dk <= 2e-2, dk


def test_decode_sequence_against_reference_kernels(ops, refcuda):
    """rope_ind(q), rope_ind(k), kv_store_ind, flash_attention_decode_ind (src/model_gpu.cu:277-282) against the
    fused decode call, over a few consecutive positions."""
    n_head, n_kv, hd, n_ctx, theta, rope_type = 12, 2, 128, 256, 1e6, 1
    scale = float(1.0 / np.sqrt(hd))
    rng = np.random.default_rng(31)
    n0 = 60
    _, K, V = make_qkv(32, n_head, n_kv, hd, n0, n_ctx)
    rK, rV, mK, mV = dev(K), dev(V), dev(K), dev(V)
    for pos in range(n0, n0 + 6):
        q = rng.standard_normal((n_head, hd)).astype(np.float32)
        k = rng.standard_normal((n_kv, hd)).astype(np.float32)
        v = rng.standard_normal((n_kv, hd)).astype(np.float32)
        d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
        rq, rk, rv = dev(q), dev(k), dev(v)
        r_out = torch.empty(n_head, hd, device="cuda")
        refcuda.rope_ind(rq, rope_type, n_head, hd, hd, theta, d_pos)
        refcuda.rope_ind(rk, rope_type, n_kv, hd, hd, theta, d_pos)
        refcuda.kv_store_ind(rK, rV, rk, rv, n_kv, hd, n_ctx, d_pos)
        refcuda.flash_attention_decode_ind(rq, rK, rV, r_out, n_head, n_kv, hd, n_ctx, d_pos, scale)
        m_out = torch.empty(n_head, hd, device="cuda")
        ops.attn_decode(dev(q), dev(k), dev(v), mK, mV, m_out, n_head, n_kv, hd, n_ctx, d_pos, scale, ops.FUSE_ALL,
                        (rope_type, hd, theta, None))
        torch.cuda.synchronize()
        assert_close(m_out.cpu().numpy(), r_out.cpu().numpy(), "decode sequence pos %d" % pos)
    assert torch.equal(mV.view(torch.int16), rV.view(torch.int16))


def test_kv_store_and_shift_bit_exact_against_reference_kernels(ops, refcuda):
    n_layer, n_kv, hd, n_ctx = 2, 2, 128, 256
    rng = np.random.default_rng(5)
    cache = rng.standard_normal((2, n_layer, n_kv, n_ctx, hd)).astype(np.float16)
    rC, mC = dev(cache), dev(cache)
    k = dev(rng.standard_normal((7, n_kv, hd)).astype(np.float32))
    v = dev(rng.standard_normal((7, n_kv, hd)).astype(np.float32))
    refcuda.kv_store_batch(rC[0, 1], rC[1, 1], k, v, n_kv, hd, n_ctx, 33, 7)
    ops.kv_store_batch(mC[0, 1], mC[1, 1], k, v, n_kv, hd, n_ctx, 33, 7)
    torch.cuda.synchronize()
    assert torch.equal(rC.view(torch.int16), mC.view(torch.int16))
    refcuda.kv_shift(rC[0], rC[1], n_layer, n_kv, hd, n_ctx, 16, 100)
    ops.kv_shift(mC[0], mC[1], n_layer, n_kv, hd, n_ctx, 16, 100)
    torch.cuda.synchronize()
    assert torch.equal(rC.view(torch.int16), mC.view(torch.int16))
