"""The C++ wrappers with the reference's names (orin_llm_b200/host/kernels.h), driven through a small C shim:
the reference's own per-layer call sequences (src/model_gpu.cu:277-282 and 379-384), unfused and fused,
against the CPU oracle."""
import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

from helpers import assert_close

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def shim(ops):
    from orin_llm_b200 import build
    host = build.build_host()
    out = os.path.join(build.LIBDIR, "libhost_shim_test.so")
    src = os.path.join(HERE, "host_shim.cpp")
    if not os.path.exists(out) or os.path.getmtime(out) < max(os.path.getmtime(src), os.path.getmtime(host)):
        subprocess.check_call(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-o", out, src, "-L" + build.LIBDIR,
                               "-lorin_attn_host", "-lorin_attn_b200", "-Wl,-rpath," + build.LIBDIR])
    L = ctypes.CDLL(out)
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    L.shim_scratch_size.restype = ctypes.c_size_t
    L.shim_scratch_size.argtypes = [i, i, i, i]
    L.shim_scratch_assign.argtypes = [vp, i, i, i, i]
    L.shim_set_stream.argtypes = [vp]
    for name in ("shim_decode_layer_unfused", "shim_decode_layer_fused"):
        getattr(L, name).argtypes = [vp] * 6 + [i] * 4 + [vp, f, i, i, f]
    for name in ("shim_prefill_layer_unfused", "shim_prefill_layer_fused"):
        getattr(L, name).argtypes = [vp] * 6 + [i] * 6 + [f, i, i, f]
    L.shim_fuse_call_sequence.argtypes = [i]
    L.shim_decode_layer_mismatched.argtypes = [vp] * 7 + [i] * 4 + [vp, f, i, i, f]
    L.shim_decode_layer_fused_extras.argtypes = [vp] * 6 + [i] * 4 + [vp, f, i, i, f] + [vp] * 5 + [f, vp, vp]
    assert L.shim_init(0) == 0
    return L


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("rope_type,n_head,n_kv,theta", [(1, 12, 2, 1e6), (0, 32, 8, 5e5)])
def test_reference_call_sequences(shim, oracle, rope_type, n_head, n_kv, theta):
    hd, n_ctx, n_prompt, n_dec = 128, 512, 45, 3
    scale = np.float32(1.0 / np.sqrt(hd))
    rng = np.random.default_rng(90 + rope_type)
    n_tok = n_prompt + n_dec
    q = rng.standard_normal((n_tok, n_head, hd), dtype=np.float32)
    k = rng.standard_normal((n_tok, n_kv, hd), dtype=np.float32)
    v = rng.standard_normal((n_tok, n_kv, hd), dtype=np.float32).astype(np.float16).astype(np.float32)
    kc32 = np.zeros((n_kv, n_ctx, hd), np.float32); vc32 = np.zeros_like(kc32)
    want = oracle.attn_batch(q.copy(), k.copy(), v.copy(), kc32, vc32, 0, scale, True, rope_type, hd, theta, None)

    nbytes = shim.shim_scratch_size(n_head, n_kv, hd, n_prompt)
    assert nbytes > 0
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    shim.shim_scratch_assign(scratch.data_ptr(), n_head, n_kv, hd, n_prompt)
    shim.shim_set_stream(torch.cuda.current_stream().cuda_stream)

    for fused in (False, True):
        kc = torch.zeros(n_kv, n_ctx, hd, dtype=torch.float16, device="cuda"); vc = torch.zeros_like(kc)
        out = torch.empty(n_tok, n_head, hd, device="cuda")
        dq, dk, dv = dev(q), dev(k), dev(v)     # the unfused sequence rotates q and k in place, like the reference
        pf = shim.shim_prefill_layer_fused if fused else shim.shim_prefill_layer_unfused
        df = shim.shim_decode_layer_fused if fused else shim.shim_decode_layer_unfused
        pf(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), n_head, n_kv, hd, n_ctx,
           0, n_prompt, float(scale), rope_type, hd, theta)
        d_pos = torch.zeros(1, dtype=torch.int32, device="cuda")
        for t in range(n_prompt, n_tok):
            d_pos.fill_(t)
            df(dq[t].data_ptr(), dk[t].data_ptr(), dv[t].data_ptr(), kc.data_ptr(), vc.data_ptr(), out[t].data_ptr(), n_head,
               n_kv, hd, n_ctx, d_pos.data_ptr(), float(scale), rope_type, hd, theta)
        torch.cuda.synchronize()
        assert_close(out.cpu().numpy(), want, "C++ wrappers, fused=%s" % fused)


def test_fused_decode_with_extras_through_the_cpp_wrapper(shim, oracle):
    """attention_decode_fused with AttnExtras: biases, q/k norm and the q8_1 output in one call."""
    n_head, n_kv, hd, n_ctx, pos = 16, 2, 128, 512, 300
    scale = np.float32(1.0 / np.sqrt(hd))
    rng = np.random.default_rng(95)
    K = rng.standard_normal((n_kv, n_ctx, hd)).astype(np.float16)
    V = rng.standard_normal((n_kv, n_ctx, hd)).astype(np.float16)
    K[:, pos:] = 0
    V[:, pos:] = 0
    q = rng.standard_normal((1, n_head, hd)).astype(np.float32)
    k = rng.standard_normal((1, n_kv, hd)).astype(np.float32)
    v = rng.standard_normal((1, n_kv, hd)).astype(np.float32)
    opt = dict(bias_q=(0.3 * rng.standard_normal(n_head * hd)).astype(np.float32),
               bias_k=(0.3 * rng.standard_normal(n_kv * hd)).astype(np.float32),
               bias_v=(0.3 * rng.standard_normal(n_kv * hd)).astype(np.float32),
               norm_q=(1 + 0.2 * rng.standard_normal(hd)).astype(np.float32),
               norm_k=(1 + 0.2 * rng.standard_normal(hd)).astype(np.float32))
    qo, ko, vo = q.copy(), k.copy(), v.copy()
    oracle.pre_attention(qo, ko, vo, eps=1e-6, **opt)
    vo = vo.astype(np.float16).astype(np.float32)
    want = oracle.attn_batch(qo, ko, vo, K.astype(np.float32), V.astype(np.float32), pos, scale, True, 1, hd, 1e6, None)[0]

    nbytes = shim.shim_scratch_size(n_head, n_kv, hd, 1)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    shim.shim_scratch_assign(scratch.data_ptr(), n_head, n_kv, hd, 1)
    shim.shim_set_stream(torch.cuda.current_stream().cuda_stream)
    dK, dV = dev(K), dev(V)
    d = {name: dev(a) for name, a in opt.items()}
    out = torch.empty(n_head, hd, device="cuda")
    qs = torch.empty(n_head * hd, dtype=torch.int8, device="cuda")
    sc = torch.empty(n_head * hd // 32, device="cuda")
    d_pos = torch.tensor([pos], dtype=torch.int32, device="cuda")
    dq0, dk0, dv0 = dev(q[0]), dev(k[0]), dev(v[0])      # named, so that they outlive the call
    shim.shim_decode_layer_fused_extras(dq0.data_ptr(), dk0.data_ptr(), dv0.data_ptr(), dK.data_ptr(),
                                        dV.data_ptr(), out.data_ptr(), n_head, n_kv, hd, n_ctx, d_pos.data_ptr(), float(scale),
                                        1, hd, 1e6, d["bias_q"].data_ptr(), d["bias_k"].data_ptr(), d["bias_v"].data_ptr(),
                                        d["norm_q"].data_ptr(), d["norm_k"].data_ptr(), 1e-6, qs.data_ptr(), sc.data_ptr())
    torch.cuda.synchronize()
    assert_close(out.cpu().numpy(), want, "C++ wrapper with extras")
    want_q, want_s = oracle.quantize_q8_1(out.cpu().numpy())
    assert np.array_equal(qs.cpu().numpy(), want_q) and np.array_equal(sc.cpu().numpy(), want_s)


def test_call_sequence_fusion(shim, ops, oracle):
    """With call-sequence fusion on, the reference's four-call sequences run as the fused launches: same results as
    the oracle, two launches per decode layer (split + merge) and two per prefill chunk (prologue + attention) instead
    of five, q left unrotated; a sequence that does not match (another k buffer stored) is issued call by call."""
    rope_type, n_head, n_kv, theta = 1, 12, 2, 1e6
    hd, n_ctx, n_prompt, n_dec = 128, 512, 45, 3
    scale = np.float32(1.0 / np.sqrt(hd))
    rng = np.random.default_rng(97)
    n_tok = n_prompt + n_dec
    q = rng.standard_normal((n_tok, n_head, hd), dtype=np.float32)
    k = rng.standard_normal((n_tok, n_kv, hd), dtype=np.float32)
    v = rng.standard_normal((n_tok, n_kv, hd), dtype=np.float32).astype(np.float16).astype(np.float32)
    kc32 = np.zeros((n_kv, n_ctx, hd), np.float32); vc32 = np.zeros_like(kc32)
    want = oracle.attn_batch(q.copy(), k.copy(), v.copy(), kc32, vc32, 0, scale, True, rope_type, hd, theta, None)

    nbytes = shim.shim_scratch_size(n_head, n_kv, hd, n_prompt)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    shim.shim_scratch_assign(scratch.data_ptr(), n_head, n_kv, hd, n_prompt)
    shim.shim_set_stream(torch.cuda.current_stream().cuda_stream)
    shim.shim_fuse_call_sequence(1)
    try:
        kc = torch.zeros(n_kv, n_ctx, hd, dtype=torch.float16, device="cuda"); vc = torch.zeros_like(kc)
        out = torch.empty(n_tok, n_head, hd, device="cuda")
        dq, dk, dv = dev(q), dev(k), dev(v)
        l0 = ops.launch_count()
        shim.shim_prefill_layer_unfused(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(),
                                        n_head, n_kv, hd, n_ctx, 0, n_prompt, float(scale), rope_type, hd, theta)
        assert ops.launch_count() - l0 == 2
        d_pos = torch.zeros(1, dtype=torch.int32, device="cuda")
        for t in range(n_prompt, n_tok):
            d_pos.fill_(t)
            l0 = ops.launch_count()
            shim.shim_decode_layer_unfused(dq[t].data_ptr(), dk[t].data_ptr(), dv[t].data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                           out[t].data_ptr(), n_head, n_kv, hd, n_ctx, d_pos.data_ptr(), float(scale), rope_type,
                                           hd, theta)
            assert ops.launch_count() - l0 == 1
        torch.cuda.synchronize()
        assert_close(out.cpu().numpy(), want, "call-sequence fusion")
        assert torch.equal(dq.cpu(), torch.from_numpy(q)), "q must be left as it was"
        # a sequence whose stored k is not the k that was rotated does not fuse: four launches, q rotated in place
        q0, k0, k_other = dev(q[0]), dev(k[0]), dev(k[1])
        kc2 = torch.zeros_like(kc); vc2 = torch.zeros_like(kc)
        o0 = torch.empty(n_head, hd, device="cuda")
        d_pos.fill_(7)
        l0 = ops.launch_count()
        shim.shim_decode_layer_mismatched(q0.data_ptr(), k0.data_ptr(), k_other.data_ptr(), dv[0].data_ptr(), kc2.data_ptr(),
                                          vc2.data_ptr(), o0.data_ptr(), n_head, n_kv, hd, n_ctx, d_pos.data_ptr(), float(scale),
                                          rope_type, hd, theta)
        torch.cuda.synchronize()
        assert ops.launch_count() - l0 == 4
        assert not torch.equal(q0.cpu(), torch.from_numpy(q[0]))
        assert torch.equal(kc2[:, 7].cpu(), torch.from_numpy(k[1]).half())      # the unrotated other k, as asked
    finally:
        shim.shim_fuse_call_sequence(0)


def test_fused_decode_captured_without_assigned_scratch(shim, tmp_path):
    """attention_decode_fused as the FIRST call a host makes, under stream capture, with no attn_scratch_assign() before
    it (what the reference's forward_capture would do, src/model_gpu.cu:295-316): the wrapper must not allocate during
    the capture -- it runs on the library's built-in scratch block -- and the replayed graph must give the oracle's
    result at several positions.  A fresh process, because the wrappers keep process-global state."""
    from orin_llm_b200 import build
    code = r'''
import ctypes, os, sys
import numpy as np, torch
sys.path.insert(0, sys.argv[2]); sys.path.insert(0, os.path.join(sys.argv[2], "tests"))
from oracle.oracle import Oracle
from helpers import assert_close, f16_round, make_qkv
L = ctypes.CDLL(sys.argv[1])
vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
L.shim_set_stream.argtypes = [vp]
L.shim_decode_layer_fused.argtypes = [vp] * 6 + [i] * 4 + [vp, f, i, i, f]
torch.cuda.set_device(0); torch.zeros(1, device="cuda")
n_head, n_kv, hd, n_ctx, n0 = 12, 2, 128, 1024, 300
scale = np.float32(1.0 / np.sqrt(hd))
rng = np.random.default_rng(5)
_, K, V = make_qkv(6, n_head, n_kv, hd, n0, n_ctx)
kc32, vc32 = K.astype(np.float32), V.astype(np.float32)
dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
dK, dV = dev(K), dev(V)
dq = torch.empty(n_head, hd, device="cuda"); dk = torch.empty(n_kv, hd, device="cuda"); dv = torch.empty(n_kv, hd, device="cuda")
out = torch.empty(n_head, hd, device="cuda")
d_pos = torch.tensor([n0], dtype=torch.int32, device="cuda")
stream = torch.cuda.Stream(); graph = torch.cuda.CUDAGraph()
stream.wait_stream(torch.cuda.current_stream())
before = torch.cuda.memory_allocated()
free0 = torch.cuda.mem_get_info()[0]
with torch.cuda.stream(stream):
    L.shim_set_stream(stream.cuda_stream)
    graph.capture_begin(capture_error_mode="relaxed")       # the reference captures in relaxed mode too
    L.shim_decode_layer_fused(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dK.data_ptr(), dV.data_ptr(), out.data_ptr(), n_head,
                              n_kv, hd, n_ctx, d_pos.data_ptr(), float(scale), 1, hd, 1e6)
    graph.capture_end()
    L.shim_set_stream(None)
assert torch.cuda.mem_get_info()[0] >= free0 - (8 << 20), "the captured call allocated device memory"
orc = Oracle()
for step in range(3):
    pos = n0 + step
    q = rng.standard_normal((n_head, hd)).astype(np.float32); k = rng.standard_normal((n_kv, hd)).astype(np.float32)
    v = f16_round(rng.standard_normal((n_kv, hd)).astype(np.float32))
    dq.copy_(dev(q)); dk.copy_(dev(k)); dv.copy_(dev(v)); d_pos.fill_(pos)
    torch.cuda.synchronize(); graph.replay(); torch.cuda.synchronize()
    qo, ko = q.copy()[None], k.copy()[None]
    want = orc.attn_batch(qo, ko, v[None].copy(), kc32, vc32, pos, scale, True, 1, hd, 1e6, None)[0]
    kc32[:, pos] = f16_round(ko[0])
    assert_close(out.cpu().numpy(), want, "captured fused decode, step %d" % step)
print("ok")
'''
    root = os.path.dirname(HERE)
    r = subprocess.run(["python", "-c", code, os.path.join(build.LIBDIR, "libhost_shim_test.so"), root], capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stderr[-1500:]
