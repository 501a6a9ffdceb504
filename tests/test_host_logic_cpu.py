"""Host logic of the C++ wrappers (orin_llm_b200/host/kernels.cpp) on CPU: the wrappers are linked against a recording
stand-in for the CUDA library (tests/fake_capi.cpp) and driven through the same C shim the GPU tests use.  Checks the
first-use initialisation, the scratch fall-backs and the call-sequence fusion, call by call."""
import ctypes
import os
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


@pytest.fixture()
def host(tmp_path):
    """A fresh copy of the library per test: the wrappers keep process-global state, as the reference's do."""
    out = str(tmp_path / "libhost_fake.so")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-fPIC", "-shared", "-o", out,
                           os.path.join(ROOT, "orin_llm_b200", "host", "kernels.cpp"), os.path.join(HERE, "host_shim.cpp"),
                           os.path.join(HERE, "fake_capi.cpp")])
    L = ctypes.CDLL(out)
    L.fake_log.restype = ctypes.c_char_p
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    L.shim_scratch_size.restype = ctypes.c_size_t
    L.shim_scratch_size.argtypes = [i, i, i, i]
    L.shim_scratch_assign.argtypes = [vp, i, i, i, i]
    L.shim_set_stream.argtypes = [vp]
    L.shim_fuse_call_sequence.argtypes = [i]
    for name in ("shim_decode_layer_unfused", "shim_decode_layer_fused"):
        getattr(L, name).argtypes = [vp] * 6 + [i] * 4 + [vp, f, i, i, f]
    for name in ("shim_prefill_layer_unfused", "shim_prefill_layer_fused"):
        getattr(L, name).argtypes = [vp] * 6 + [i] * 6 + [f, i, i, f]
    L.shim_decode_layer_mismatched.argtypes = [vp] * 7 + [i] * 4 + [vp, f, i, i, f]
    L.shim_kv_shift.argtypes = [vp, vp, i, i, i, i, i, i]
    L.shim_decode_producers_only.argtypes = [vp] * 5 + [i] * 4 + [vp, i, i, f]
    return L


def log(L):
    s = L.fake_log().decode().strip(";")
    L.fake_log_clear()
    return s.split(";") if s else []


# distinct fake addresses; nothing is dereferenced by the stand-in
Q, K, V, KC, VC, OUT, DPOS, K2 = (0x1000 * n for n in range(1, 9))
DEC = (12, 2, 128, 4096)            # n_head, n_kv, head_dim, n_ctx


def decode_unfused(L):
    L.shim_decode_layer_unfused(Q, K, V, KC, VC, OUT, *DEC, DPOS, 0.1, 1, 128, 1e6)


def prefill_unfused(L, n_past=0, batch=45):
    L.shim_prefill_layer_unfused(Q, K, V, KC, VC, OUT, *DEC, n_past, batch, 0.1, 1, 128, 1e6)


def test_first_use_initialises_and_decode_falls_back_to_builtin_scratch(host):
    decode_unfused(host)
    assert log(host) == ["init/-1", "rope", "rope", "kv_store", "decode_noalloc"]
    decode_unfused(host)
    assert log(host) == ["rope", "rope", "kv_store", "decode_noalloc"]          # initialised once


def test_prefill_allocates_scratch_on_demand_and_grows(host):
    prefill_unfused(host, batch=8)
    assert log(host) == ["init/-1", "rope", "rope", "kv_store", "scratch_alloc", "prefill/0"]
    prefill_unfused(host, batch=8)
    assert log(host) == ["rope", "rope", "kv_store", "prefill/0"]
    prefill_unfused(host, batch=64)                                               # larger chunk: a larger block
    assert log(host) == ["rope", "rope", "kv_store", "scratch_alloc", "scratch_free", "prefill/0"]   # the old one is returned


def test_fused_decode_never_allocates(host):
    """attention_decode_fused may be the first call a host makes, under stream capture (src/model_gpu.cu:295-316):
    without an assigned block it must run on the built-in scratch block, not allocate."""
    host.shim_decode_layer_fused(Q, K, V, KC, VC, OUT, *DEC, DPOS, 0.1, 1, 128, 1e6)
    assert log(host) == ["init/-1", "builtin_scratch", "decode/7"]
    n = host.shim_scratch_size(12, 2, 128, 64)
    buf = ctypes.create_string_buffer(n)
    host.shim_scratch_assign(ctypes.addressof(buf), 12, 2, 128, 64)
    host.shim_decode_layer_fused(Q, K, V, KC, VC, OUT, *DEC, DPOS, 0.1, 1, 128, 1e6)
    assert log(host) == ["decode/7"]


def test_recorded_calls_without_an_attention_call_are_issued_by_flush(host):
    host.shim_fuse_call_sequence(1)
    host.shim_decode_producers_only(Q, K, V, KC, VC, 12, 2, 128, 4096, DPOS, 1, 128, 1e6)
    assert log(host) == ["init/-1"]                  # recorded, nothing issued yet
    host.shim_flush()
    assert log(host) == ["rope", "rope", "kv_store"]
    host.shim_flush()
    assert log(host) == []


def test_assigned_scratch_is_used(host):
    n = host.shim_scratch_size(12, 2, 128, 64)
    assert n >= 4096 + 64 * 1024
    buf = ctypes.create_string_buffer(n)
    host.shim_scratch_assign(ctypes.addressof(buf), 12, 2, 128, 64)
    prefill_unfused(host, batch=64)
    decode_unfused(host)
    assert log(host) == ["init/-1", "rope", "rope", "kv_store", "prefill/0", "rope", "rope", "kv_store", "decode/0"]


def test_call_sequence_fusion(host):
    host.shim_fuse_call_sequence(1)
    prefill_unfused(host)                    # allocates prefill and decode scratch here (never captured)
    assert log(host) == ["init/-1", "scratch_alloc", "scratch_alloc", "prefill/7"]
    decode_unfused(host)
    assert log(host) == ["decode/7"]
    # the stored k is not the rotated k: issued call by call, in order
    host.shim_decode_layer_mismatched(Q, K, K2, V, KC, VC, OUT, *DEC, DPOS, 0.1, 1, 128, 1e6)
    assert log(host) == ["rope", "rope", "kv_store", "decode/0"]
    # anything else in between flushes what was recorded
    host.shim_fuse_call_sequence(0)
    assert log(host) == []
    decode_unfused(host)
    assert log(host) == ["rope", "rope", "kv_store", "decode/0"]


def test_pending_calls_are_flushed_by_other_calls(host):
    host.shim_fuse_call_sequence(1)
    prefill_unfused(host)
    log(host)
    # a fused sequence followed by a call that is not part of any sequence
    decode_unfused(host)
    host.shim_kv_shift(KC, VC, 1, 2, 128, 4096, 4, 16)
    assert log(host) == ["decode/7", "kv_shift"]


def test_environment_switches(tmp_path):
    """OATTN_FUSE_CALL_SEQUENCE and OATTN_DECODE_OVERLAP are read on first use (fresh process)."""
    code = r'''
import ctypes, sys
L = ctypes.CDLL(sys.argv[1])
L.fake_log.restype = ctypes.c_char_p
vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
L.shim_prefill_layer_unfused.argtypes = [vp] * 6 + [i] * 6 + [f, i, i, f]
L.shim_prefill_layer_unfused(0x1000, 0x2000, 0x3000, 0x4000, 0x5000, 0x6000, 12, 2, 128, 4096, 0, 8, 0.1, 1, 128, 1e6)
print(L.fake_log().decode())
'''
    out = str(tmp_path / "libhost_fake.so")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-fPIC", "-shared", "-o", out,
                           os.path.join(ROOT, "orin_llm_b200", "host", "kernels.cpp"), os.path.join(HERE, "host_shim.cpp"),
                           os.path.join(HERE, "fake_capi.cpp")])
    env = dict(os.environ, OATTN_FUSE_CALL_SEQUENCE="1", OATTN_DECODE_OVERLAP="1")
    r = subprocess.run(["python", "-c", code, out], capture_output=True, text=True, env=env, timeout=60)
    assert r.returncode == 0, r.stderr
    assert r.stdout.strip().strip(";").split(";") == ["init/-1", "overlap/1", "scratch_alloc", "scratch_alloc", "prefill/7"]
