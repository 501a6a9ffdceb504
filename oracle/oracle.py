"""ctypes loader for the CPU oracle  --  TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may import this
module.  The product package (orin_llm_b200) never does: it has no CPU path.

`Oracle()` loads oracle/liboracle_attn.so, the plain-C restatement of the reference's scalar
fp32 attention (src/model_cpu.cpp:20-36, 179-203, 264-295, 321-340).
`RefLib()` loads oracle/_ref/libref_attn.so, the reference's own code compiled from its
sources, when that file has been built (it cannot be built where the reference tree is absent).
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle_attn.so")
REF_SO = os.path.join(HERE, "_ref", "libref_attn.so")

_f32p = ctypes.POINTER(ctypes.c_float)
_i = ctypes.c_int
_f = ctypes.c_float


def _fp(a):
    if a is None:
        return ctypes.cast(None, _f32p)
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_f32p)


def build(ref_root="/root/reference"):
    """Compile the C restatement, and the reference harness when the reference tree is present."""
    subprocess.check_call(["make", "-s", "-C", HERE, "all"])
    if os.path.isdir(os.path.join(ref_root, "src")):
        subprocess.check_call(["make", "-s", "-C", HERE, "ref", "REF=" + ref_root])


class Oracle:
    """Plain-C restatement.  All arrays are float32 numpy, C-contiguous."""

    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build()
        L = ctypes.CDLL(ORACLE_SO)
        L.oracle_rope.argtypes = [_f32p, _i, _i, _f, _i, _f32p]
        L.oracle_kv_append.argtypes = [_f32p, _f32p, _f32p, _f32p, _i, _i, _i, _i]
        L.oracle_attend.argtypes = [_f32p, _f32p, _f32p, _f32p, _i, _i, _i, _i, _i, _f, _f32p]
        L.oracle_attn_step.argtypes = [_f32p] * 6 + [_i] * 5 + [_f, _i, _i, _f, _f32p, _f32p]
        L.oracle_attn_batch.argtypes = [_f32p] * 6 + [_i] * 6 + [_f, _i, _i, _i, _f, _f32p, _f32p]
        L.oracle_kv_shift.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [_i] * 7
        L.oracle_softmax.argtypes = [_f32p, _i]
        self.L = L

    def rope(self, x, rope_type, n_rot, theta, pos, freq_factors=None):
        """In-place rotation of ONE head row x[head_dim] (model_cpu.cpp:179-203)."""
        self.L.oracle_rope(_fp(x), rope_type, n_rot, theta, pos, _fp(freq_factors))
        return x

    def rope_rows(self, x, rope_type, n_rot, theta, positions, freq_factors=None):
        """x [rows][head_dim] rotated in place, row r at positions[r]."""
        for r in range(x.shape[0]):
            self.L.oracle_rope(_fp(x[r]), rope_type, n_rot, theta, int(positions[r]), _fp(freq_factors))
        return x

    def kv_append(self, kcache, vcache, k, v, pos):
        n_kv, n_ctx, d = kcache.shape
        self.L.oracle_kv_append(_fp(kcache), _fp(vcache), _fp(k), _fp(v), n_kv, d, n_ctx, pos)

    def attend(self, q, kcache, vcache, npos, scale):
        """q [n_head][d]; caches [n_kv][n_ctx][d]; positions [0, npos). Returns [n_head][d]."""
        n_head, d = q.shape
        n_kv, n_ctx, _ = kcache.shape
        out = np.empty_like(q)
        score = np.empty(npos, np.float32)
        self.L.oracle_attend(_fp(q), _fp(kcache), _fp(vcache), _fp(out), n_head, n_kv, d, n_ctx, npos,
                             scale, _fp(score))
        return out

    def attn_batch(self, q, k, v, kcache, vcache, n_past, scale, apply_rope, rope_type=0, n_rot=0,
                   theta=10000.0, freq_factors=None):
        """forward_batch semantics (model_cpu.cpp:314-319).  q [batch][n_head][d], k,v [batch][n_kv][d].
        q and k are rotated in place when apply_rope; the caches are appended to."""
        batch, n_head, d = q.shape
        n_kv, n_ctx, _ = kcache.shape
        out = np.empty_like(q)
        score = np.empty(n_past + batch, np.float32)
        self.L.oracle_attn_batch(_fp(q), _fp(k), _fp(v), _fp(kcache), _fp(vcache), _fp(out), n_head, n_kv,
                                 d, n_ctx, n_past, batch, scale, int(apply_rope), rope_type, n_rot, theta,
                                 _fp(freq_factors), _fp(score))
        return out

    def kv_shift(self, kcache, vcache, n_layer, n_kv, d, n_ctx, n_keep, shift):
        """In place on arrays of any element width (fp32 oracle cache or the uint16 device image)."""
        assert kcache.flags["C_CONTIGUOUS"] and vcache.flags["C_CONTIGUOUS"]
        self.L.oracle_kv_shift(kcache.ctypes.data, vcache.ctypes.data, n_layer, n_kv, d, n_ctx, n_keep,
                               shift, kcache.dtype.itemsize)


class RefLib:
    """The reference's own CPU code (built from its sources into oracle/_ref/)."""

    @staticmethod
    def available():
        return os.path.exists(REF_SO)

    def __init__(self):
        L = ctypes.CDLL(REF_SO)
        L.ref_rope.argtypes = [_f32p, _i, _i, _f, _i, _f32p]
        L.ref_attend.argtypes = [_f32p, _f32p, _f32p, _f32p, _i, _i, _i, _i, _i, _f, _f32p]
        L.ref_attend_mt.argtypes = [_f32p, _f32p, _f32p, _f32p, _i, _i, _i, _i, _i, _f, _i]
        L.ref_attend_mt.restype = _i
        L.ref_attend_chunk_mt.argtypes = [_f32p, _f32p, _f32p, _f32p, _i, _i, _i, _i, _i, _i, _f, _i]
        L.ref_attend_chunk_mt.restype = _i
        L.ref_forward_probe.argtypes = [_f32p, _i, _i, _i, _i, _i, _i, _i, _f, _f32p] + [_f32p] * 6
        L.ref_forward_probe.restype = _i
        L.ref_kv_shift.argtypes = [_f32p, _f32p] + [_i] * 6
        self.L = L

    def rope(self, x, rope_type, n_rot, theta, pos, freq_factors=None):
        self.L.ref_rope(_fp(x), rope_type, n_rot, theta, pos, _fp(freq_factors))
        return x

    def attend(self, q, kcache, vcache, npos, scale):
        n_head, d = q.shape
        n_kv, n_ctx, _ = kcache.shape
        out = np.empty_like(q)
        score = np.empty(npos, np.float32)
        self.L.ref_attend(_fp(q), _fp(kcache), _fp(vcache), _fp(out), n_head, n_kv, d, n_ctx, npos, scale,
                          _fp(score))
        return out

    def attend_mt(self, q, kcache, vcache, npos, scale, max_threads):
        n_head, d = q.shape
        n_kv, n_ctx, _ = kcache.shape
        out = np.empty_like(q)
        nt = self.L.ref_attend_mt(_fp(q), _fp(kcache), _fp(vcache), _fp(out), n_head, n_kv, d, n_ctx, npos,
                                  scale, max_threads)
        return out, nt

    def attend_chunk_mt(self, q, kcache, vcache, n_past, scale, max_threads):
        batch, n_head, d = q.shape
        n_kv, n_ctx, _ = kcache.shape
        out = np.empty_like(q)
        nt = self.L.ref_attend_chunk_mt(_fp(q), _fp(kcache), _fp(vcache), _fp(out), n_head, n_kv, d, n_ctx,
                                        n_past, batch, scale, max_threads)
        return out, nt

    def forward_probe(self, x_in, n_head, n_kv, d, n_ctx, rope_type, n_rot, theta, freq_factors=None):
        """Runs the reference's real forward() token by token; see ref_harness.cpp."""
        n_tok, ne = x_in.shape
        assert ne == n_head * d
        nk = n_kv * d
        q_pre = np.empty((n_tok, n_head, d), np.float32)
        k_pre = np.empty((n_tok, n_kv, d), np.float32)
        v_pre = np.empty((n_tok, n_kv, d), np.float32)
        q_rot = np.empty((n_tok, n_head, d), np.float32)
        k_rot = np.empty((n_tok, n_kv, d), np.float32)
        attn = np.empty((n_tok, n_head, d), np.float32)
        rc = self.L.ref_forward_probe(_fp(x_in), n_tok, n_head, n_kv, d, n_ctx, rope_type, n_rot, theta,
                                      _fp(freq_factors), _fp(q_pre), _fp(k_pre), _fp(v_pre), _fp(q_rot),
                                      _fp(k_rot), _fp(attn))
        assert rc == 0, "probe self-check failed"
        del nk
        return dict(q_pre=q_pre, k_pre=k_pre, v_pre=v_pre, q_rot=q_rot, k_rot=k_rot, attn=attn)

    def kv_shift(self, kcache, vcache, n_layer, n_kv, d, n_ctx, n_keep, shift):
        self.L.ref_kv_shift(_fp(kcache), _fp(vcache), n_layer, n_kv, d, n_ctx, n_keep, shift)
