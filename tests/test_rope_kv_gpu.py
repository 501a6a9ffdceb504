"""GPU parity tests of the unfused building blocks (RoPE, KV store, KV shift) against the oracle."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("rope_type,hd,n_rot,theta,use_ff", [(1, 128, 128, 1e6, False), (0, 128, 128, 5e5, True),
                                                             (0, 64, 32, 1e4, False), (1, 64, 64, 1e4, True)])
def test_rope_batch_and_indirect(ops, oracle, rope_type, hd, n_rot, theta, use_ff):
    rng = np.random.default_rng(60)
    heads, batch, n_past = 6, 37, 8100
    x = rng.standard_normal((batch * heads, hd)).astype(np.float32)
    ff = (1.0 + 3 * rng.random(n_rot // 2)).astype(np.float32) if use_ff else None
    want = x.copy()
    oracle.rope_rows(want, rope_type, n_rot, theta, [n_past + r // heads for r in range(batch * heads)], ff)
    dx = dev(x)
    fn = ops.rope_neox_batch if rope_type == 1 else ops.rope_normal_batch
    fn(dx, batch * heads, hd, n_rot, theta, n_past, heads, dev(ff) if use_ff else None)
    torch.cuda.synchronize()
    # angles reach ~8e3 rad; device sincosf/pow are within a few ulp of the host libm
    assert np.abs(dx.cpu().numpy() - want).max() < 2e-4
    # indirect position
    pos = 123456
    want = x[:heads].copy()
    oracle.rope_rows(want, rope_type, n_rot, theta, [pos] * heads, ff)
    dx = dev(x[:heads])
    d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    fn = ops.rope_neox_ind if rope_type == 1 else ops.rope_normal_ind
    fn(dx, heads, hd, n_rot, theta, d_pos, dev(ff) if use_ff else None)
    torch.cuda.synchronize()
    assert np.abs(dx.cpu().numpy() - want).max() < 2e-3


def test_rope_zero_rows_and_position_zero(ops):
    x = torch.randn(4, 128, device="cuda")
    y = x.clone()
    ops.rope_neox_batch(y, 0, 128, 128, 1e6, 0, 2)          # rows = 0: nothing to do
    ops.rope_neox_batch(y, 2, 128, 128, 1e6, 0, 2)          # rows 0,1 are token 0 at position 0: identity
    torch.cuda.synchronize()
    assert torch.equal(x, y)


def test_kv_store_batch_and_indirect(ops):
    rng = np.random.default_rng(61)
    heads, hd, n_ctx, batch, base = 4, 128, 64, 9, 50
    k = rng.standard_normal((batch, heads, hd)).astype(np.float32) * 100
    v = rng.standard_normal((batch, heads, hd)).astype(np.float32) * 1e-3
    kc = torch.zeros(heads, n_ctx, hd, dtype=torch.float16, device="cuda"); vc = torch.zeros_like(kc)
    ops.kv_store_batch(kc, vc, dev(k), dev(v), heads, hd, n_ctx, base, batch)
    d_pos = torch.tensor([7], dtype=torch.int32, device="cuda")
    ops.kv_store_ind(kc, vc, dev(k[3]), dev(v[3]), heads, hd, n_ctx, d_pos)
    torch.cuda.synchronize()
    K, V = kc.cpu().numpy(), vc.cpu().numpy()
    want_k = np.transpose(k, (1, 0, 2)).astype(np.float16)
    assert np.array_equal(K[:, base:base + batch].view(np.uint16), want_k.view(np.uint16))
    assert np.array_equal(V[:, base:base + batch], np.transpose(v, (1, 0, 2)).astype(np.float16))
    assert np.array_equal(K[:, 7], k[3].astype(np.float16)) and np.array_equal(V[:, 7], v[3].astype(np.float16))
    untouched = np.ones(n_ctx, bool); untouched[base:base + batch] = False; untouched[7] = False
    assert not K[:, untouched].any() and not V[:, untouched].any()
    from orin_llm_b200 import capi
    with pytest.raises(capi.AttnError):
        ops.kv_store_batch(kc, vc, dev(k), dev(v), heads, hd, n_ctx, n_ctx - 3, batch)   # would run past n_ctx


@pytest.mark.parametrize("n_layer,n_kv,hd,n_ctx,n_keep,shift", [(2, 3, 128, 1000, 4, 498), (3, 2, 64, 513, 0, 1),
                                                                (1, 1, 128, 300, 10, 290), (2, 2, 128, 4096, 16, 2040)])
def test_kv_shift_matches_oracle_bitwise(ops, oracle, n_layer, n_kv, hd, n_ctx, n_keep, shift):
    rng = np.random.default_rng(62)
    k = rng.standard_normal((n_layer, n_kv, n_ctx, hd)).astype(np.float16)
    v = rng.standard_normal((n_layer, n_kv, n_ctx, hd)).astype(np.float16)
    dk, dv = dev(k), dev(v)
    ops.kv_shift(dk, dv, n_layer, n_kv, hd, n_ctx, n_keep, shift)
    torch.cuda.synchronize()
    oracle.kv_shift(k, v, n_layer, n_kv, hd, n_ctx, n_keep, shift)
    assert np.array_equal(dk.cpu().numpy().view(np.uint16), k.view(np.uint16))
    assert np.array_equal(dv.cpu().numpy().view(np.uint16), v.view(np.uint16))


def test_kv_shift_golden_fixture(ops):
    g = np.load(os.path.join(GOLD, "kvshift.npz"))
    k0 = np.repeat(g["k0"], 2, axis=3).astype(np.float16)     # d=8 -> 16 so that rows are 32 bytes
    v0 = np.repeat(g["v0"], 2, axis=3).astype(np.float16)
    n_layer, n_kv, n_ctx, d = k0.shape
    dk, dv = dev(k0), dev(v0)
    ops.kv_shift(dk, dv, n_layer, n_kv, d, n_ctx, int(g["n_keep"]), int(g["shift"]))
    torch.cuda.synchronize()
    assert np.array_equal(dk.cpu().numpy(), np.repeat(g["k1"], 2, axis=3).astype(np.float16))
    assert np.array_equal(dv.cpu().numpy(), np.repeat(g["v1"], 2, axis=3).astype(np.float16))


def test_kv_cache_layout(ops):
    """K of all layers first, then V, per layer [n_kv][n_ctx][hd] (src/model_gpu.cu:229-235, 255-260)."""
    c = ops.KVCache(3, 2, 128, 64)
    assert c.k.data_ptr() == c.buf.data_ptr()
    assert c.v.data_ptr() == c.buf.data_ptr() + 3 * 2 * 128 * 64 * 2
    kl, vl = c.layer(2)
    assert kl.data_ptr() == c.buf.data_ptr() + 2 * c.per_layer * 2 and kl.shape == (2, 128, 64)
    assert not c.buf.any()
