"""The no-allocation decode entry point (oattn_decode_noalloc), called through the C ABI.

Some hosts of this library cannot give it a workspace: a plugin whose host application owns all device memory,
a callback that is not allowed to call cudaMalloc, a process whose memory is already fully committed.  For them
the library carries its own fixed scratch block in device memory.  This test checks that the entry point gives
the same result as the regular one (which gets a caller-allocated workspace), twice in a row -- the block is
shared by all calls and keeps the previous call's contents --, and that a shape whose partial results do not
fit is refused instead of overrunning the block.

Collected last (file name), so that a failure here cannot hide the other tests in a stop-at-first-failure run.
"""
import ctypes

import numpy as np
import pytest
import torch

from helpers import make_qkv

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_noalloc_matches_regular_entry_point_twice(ops, oracle):
    from orin_llm_b200 import capi
    L = capi.lib()
    assert L.oattn_decode_noalloc_max_bytes() == 2 << 20
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # two different shapes and lengths back to back: the second call finds the first call's partials in the block
    for (n_head, n_kv, hd, npos, seed) in [(28, 4, 128, 5000, 1), (16, 2, 128, 20000, 2), (28, 4, 128, 777, 3)]:
        q, K, V = make_qkv(9000 + seed, n_head, n_kv, hd, npos)
        dq, dK, dV = dev(q[0]), dev(K), dev(V)
        scale = float(1.0 / np.sqrt(hd))
        d_pos = torch.tensor([npos - 1], dtype=torch.int32, device="cuda")
        ref = torch.empty(n_head, hd, device="cuda")
        ws = ops.decode_workspace(n_head, n_kv, hd)
        capi.check(L.oattn_decode(dq.data_ptr(), None, None, dK.data_ptr(), dV.data_ptr(), ref.data_ptr(), n_head, n_kv, hd,
                                  npos, d_pos.data_ptr(), scale, capi.FUSE_NONE, None, ws.data_ptr(), ws.numel(), stream))
        outs = []
        for _ in range(2):
            out = torch.full((n_head, hd), float("nan"), device="cuda")
            before = torch.cuda.memory_allocated()
            capi.check(L.oattn_decode_noalloc(dq.data_ptr(), dK.data_ptr(), dV.data_ptr(), out.data_ptr(), n_head, n_kv, hd,
                                              npos, d_pos.data_ptr(), scale, stream))
            assert torch.cuda.memory_allocated() == before
            outs.append(out)
        torch.cuda.synchronize()
        # same kernel, same split plan, only the scratch address differs: within the tolerance the parity tests
        # use (in fact bit-identical)
        for out in outs:
            err = (out - ref).abs()
            assert torch.isfinite(out).all()
            assert err.max().item() <= 1e-2 and err.mean().item() <= 1e-3
            assert torch.equal(out, ref)
        # and against the CPU oracle itself, not only against the other entry point
        want = oracle.attend(q[0], K.astype(np.float32), V.astype(np.float32), npos, np.float32(scale))
        oerr = np.abs(outs[1].cpu().numpy() - want)
        assert oerr.max() <= 1e-2 and oerr.mean() <= 1e-3


def test_noalloc_refuses_shapes_beyond_the_block(ops):
    from orin_llm_b200 import capi
    L = capi.lib()
    t = torch.zeros(64, device="cuda")
    p = t.data_ptr()
    # 64 query heads over 4 kv heads: 64 heads * 74 splits * 130 floats * 4 bytes = 2.5 MB of partials (plus the group
    # partials), more than the 2 MiB block
    n_head, n_kv, hd = 16 * 4, 4, 128
    need = L.oattn_decode_workspace_bytes(n_head, n_kv, hd)
    if need <= L.oattn_decode_noalloc_max_bytes():
        pytest.skip("shape fits on this device")
    rc = L.oattn_decode_noalloc(p, p, p, p, n_head, n_kv, hd, 64, p, 0.1, None)
    assert rc == capi.ERR_WORKSPACE
    assert b"built-in block" in L.oattn_last_cuda_error()
