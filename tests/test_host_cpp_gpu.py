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
