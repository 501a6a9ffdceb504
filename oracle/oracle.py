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
REF_CUDA_SO = os.path.join(HERE, "_ref", "libref_cuda.so")

_f32p = ctypes.POINTER(ctypes.c_float)
_i = ctypes.c_int
_f = ctypes.c_float


def _fp(a):
    if a is None:
        return ctypes.cast(None, _f32p)
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_f32p)


def reference_root():
    """Where the reference checkout lies: $ORIN_LLM_REFERENCE, else a directory `reference` beside this repository.
    None when neither holds its sources."""
    cands = [os.environ.get("ORIN_LLM_REFERENCE"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "src", "model_cpu.cpp")):
            return os.path.abspath(c)
    return None


def build(ref_root=None):
    """Compile the C restatement, and the reference harness when the reference tree is present."""
    subprocess.check_call(["make", "-s", "-C", HERE, "all"])
    ref_root = ref_root or reference_root()
    if ref_root:
        subprocess.check_call(["make", "-s", "-C", HERE, "ref", "REF=" + ref_root])
        try:     # optional: the GPU-side cross-check needs nvcc and a minute of compile time
            subprocess.check_call(["make", "-s", "-C", HERE, "refcuda", "REF=" + ref_root])
            if os.path.exists(os.path.join(os.path.dirname(HERE), "orin_llm_b200", "lib", "liborin_attn_host.so")):
                subprocess.check_call(["make", "-s", "-C", HERE, "e2e", "REF=" + ref_root])
        except (subprocess.CalledProcessError, OSError) as e:
            print("oracle: reference CUDA kernels / end-to-end binaries not built (%s)" % e)


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
        L.oracle_rms_norm.argtypes = [_f32p, _f32p, _i, _f, _f32p]
        L.oracle_pre_attention.argtypes = [_f32p, _f32p, _f32p, _i, _i, _i] + [_f32p] * 5 + [_f]
        L.oracle_quantize_q8_1.argtypes = [_f32p, _i, ctypes.c_void_p, _f32p]
        L.oracle_quantize_mmq_q8_1.argtypes = [_f32p, _i, _i, _i, ctypes.c_void_p]
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

    def pre_attention(self, q, k, v, bias_q=None, bias_k=None, bias_v=None, norm_q=None, norm_k=None, eps=1e-6):
        """Bias add and per-head RMSNorm of one token's (or a batch of tokens') q, k, v, in place
        (model_cpu.cpp:258-274).  q [..., n_head, d], k and v [..., n_kv, d]."""
        d = q.shape[-1]
        n_head, n_kv = q.shape[-2], k.shape[-2]
        q2, k2, v2 = q.reshape(-1, n_head, d), k.reshape(-1, n_kv, d), v.reshape(-1, n_kv, d)
        for t in range(q2.shape[0]):
            self.L.oracle_pre_attention(_fp(q2[t]), _fp(k2[t]), _fp(v2[t]), n_head, n_kv, d, _fp(bias_q), _fp(bias_k),
                                        _fp(bias_v), _fp(norm_q), _fp(norm_k), eps)
        return q, k, v

    def quantize_q8_1(self, x):
        """(int8 values, fp32 scales) of a flat fp32 vector in the reference's q8_1 activation form
        (kernels.cu:136-145)."""
        x = np.ascontiguousarray(x, np.float32).reshape(-1)
        qs = np.empty(x.size, np.int8)
        scales = np.empty((x.size + 31) // 32, np.float32)
        self.L.oracle_quantize_q8_1(_fp(x), x.size, qs.ctypes.data, _fp(scales))
        return qs, scales

    def quantize_mmq_q8_1(self, x, ds4):
        """x [batch][ne00] fp32 -> uint8 [ne00/128][batch][144]: the reference's block_q8_1_mmq activation form
        (kernels.cu:147-205)."""
        x = np.ascontiguousarray(x, np.float32)
        batch, ne00 = x.shape
        assert ne00 % 128 == 0
        y = np.zeros((ne00 // 128, batch, 144), np.uint8)
        self.L.oracle_quantize_mmq_q8_1(_fp(x), ne00, batch, 1 if ds4 else 0, y.ctypes.data)
        return y

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
        if hasattr(L, "ref_dequantize_row"):
            L.ref_dequantize_row.argtypes = [_i, ctypes.c_void_p, _f32p, ctypes.c_longlong]
        L.ref_attend_chunk_mt.argtypes = [_f32p, _f32p, _f32p, _f32p, _i, _i, _i, _i, _i, _i, _f, _i]
        L.ref_attend_chunk_mt.restype = _i
        L.ref_forward_probe.argtypes = [_f32p, _i, _i, _i, _i, _i, _i, _i, _f, _f32p] + [_f32p] * 6
        L.ref_forward_probe.restype = _i
        L.ref_kv_shift.argtypes = [_f32p, _f32p] + [_i] * 6
        L.ref_forward_probe_pre.argtypes = [_f32p, _i, _i, _i, _i, _i, _i, _i, _f, _f32p] + [_f32p] * 5 + [_f] + [_f32p] * 6
        L.ref_forward_probe_pre.restype = _i
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

    def dequantize_row(self, ggml_type, raw, n_elems):
        """The reference's dequantize_row on a buffer of quantised blocks (uint8 array) -> fp32 [n_elems]."""
        raw = np.ascontiguousarray(raw, np.uint8)
        y = np.empty(n_elems, np.float32)
        self.L.ref_dequantize_row(int(ggml_type), raw.ctypes.data_as(ctypes.c_void_p), _fp(y), n_elems)
        return y

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

    def forward_probe_pre(self, x_in, n_head, n_kv, d, n_ctx, rope_type, n_rot, theta, bias_q, bias_k, bias_v, norm_q,
                          norm_k, eps, freq_factors=None):
        """forward_probe on a layer that also has q/k/v biases and per-head q/k norm weights."""
        n_tok, ne = x_in.shape
        assert ne == n_head * d
        q_pre = np.empty((n_tok, n_head, d), np.float32)
        k_pre = np.empty((n_tok, n_kv, d), np.float32)
        v_pre = np.empty((n_tok, n_kv, d), np.float32)
        q_rot = np.empty((n_tok, n_head, d), np.float32)
        k_rot = np.empty((n_tok, n_kv, d), np.float32)
        attn = np.empty((n_tok, n_head, d), np.float32)
        rc = self.L.ref_forward_probe_pre(_fp(x_in), n_tok, n_head, n_kv, d, n_ctx, rope_type, n_rot, theta,
                                          _fp(freq_factors), _fp(bias_q), _fp(bias_k), _fp(bias_v), _fp(norm_q),
                                          _fp(norm_k), eps, _fp(q_pre), _fp(k_pre), _fp(v_pre), _fp(q_rot), _fp(k_rot),
                                          _fp(attn))
        assert rc == 0, "probe self-check failed"
        return dict(q_pre=q_pre, k_pre=k_pre, v_pre=v_pre, q_rot=q_rot, k_rot=k_rot, attn=attn)

    def kv_shift(self, kcache, vcache, n_layer, n_kv, d, n_ctx, n_keep, shift):
        self.L.ref_kv_shift(_fp(kcache), _fp(vcache), n_layer, n_kv, d, n_ctx, n_keep, shift)


class RefCuda:
    """The reference's own CUDA wrappers (src/kernels.h), recompiled for sm_100a into oracle/_ref/libref_cuda.so.
    Arguments are torch CUDA tensors on device 0 (the reference is device-0 only); calls run on torch's current
    stream.  Test infrastructure: a second parity check and the comparison leg of the benchmark.

    Limits of the reference kernels (src/kernels.cu:1117,1183-1196,1361,1430-1445): n_head / n_kv <= 8; n_ctx a
    multiple of 128 with the cache initialised up to the next multiple of 128 past the last position."""

    @staticmethod
    def available():
        return os.path.exists(REF_CUDA_SO)

    def __init__(self):
        import torch
        self.torch = torch
        L = ctypes.CDLL(REF_CUDA_SO)
        vp, sz = ctypes.c_void_p, ctypes.c_size_t
        L.refcuda_init.restype = _i
        L.refcuda_set_stream.argtypes = [vp]
        L.refcuda_scratch_size.restype = sz
        L.refcuda_scratch_size.argtypes = [_i, _i]
        L.refcuda_scratch_assign.argtypes = [vp, _i, _i]
        L.refcuda_quantize_activation.argtypes = [vp, _i]
        if hasattr(L, "refcuda_gemv_batch"):
            L.refcuda_gemv_batch.argtypes = [_i, vp, vp, vp, _i, _i, _i]
        L.refcuda_rms_norm_rows.argtypes = [vp, vp, _i, _i, _f, vp]
        L.refcuda_add_inplace_broadcast.argtypes = [vp, vp, _i, _i]
        L.refcuda_rope_batch.argtypes = [vp, _i, _i, _i, _i, _f, _i, _i, vp]
        L.refcuda_rope_ind.argtypes = [vp, _i, _i, _i, _i, _f, vp, vp]
        L.refcuda_kv_store_batch.argtypes = [vp, vp, vp, vp, _i, _i, _i, _i, _i]
        L.refcuda_kv_store_ind.argtypes = [vp, vp, vp, vp, _i, _i, _i, vp]
        L.refcuda_kv_shift.argtypes = [vp, vp, _i, _i, _i, _i, _i, _i]
        L.refcuda_flash_attention.argtypes = [vp, vp, vp, vp, _i, _i, _i, _i, _i, _i, _f]
        L.refcuda_flash_attention_decode_ind.argtypes = [vp, vp, vp, vp, _i, _i, _i, _i, vp, _f]
        self.L = L
        if L.refcuda_init() != 0:
            raise RuntimeError("reference cuda::init failed")

    def _sync_stream(self):
        self.L.refcuda_set_stream(ctypes.c_void_p(self.torch.cuda.current_stream().cuda_stream))

    @staticmethod
    def _p(t):
        return ctypes.c_void_p(t.data_ptr()) if t is not None else None

    @staticmethod
    def check_shape(n_head, n_kv, n_ctx):
        if n_head // n_kv > 8 or n_ctx % 128:
            raise ValueError("outside the reference kernels' limits (group <= 8, n_ctx % 128 == 0)")

    def flash_attention_decode_ind(self, q, kc, vc, out, n_head, n_kv, head_dim, n_ctx, d_pos, scale):
        self.check_shape(n_head, n_kv, n_ctx)
        self._sync_stream()
        self.L.refcuda_flash_attention_decode_ind(self._p(q), self._p(kc), self._p(vc), self._p(out), n_head, n_kv, head_dim,
                                                  n_ctx, self._p(d_pos), scale)

    def flash_attention(self, q, kc, vc, out, n_head, n_kv, head_dim, n_ctx, n_past, batch, scale):
        self.check_shape(n_head, n_kv, n_ctx)
        self._sync_stream()
        self.L.refcuda_flash_attention(self._p(q), self._p(kc), self._p(vc), self._p(out), n_head, n_kv, head_dim, n_ctx,
                                       n_past, batch, scale)

    def rope_batch(self, x, rope_type, rows, head_dim, n_rot, theta, n_past, heads, freq_factors=None):
        self._sync_stream()
        self.L.refcuda_rope_batch(self._p(x), rope_type, rows, head_dim, n_rot, theta, n_past, heads, self._p(freq_factors))

    def rope_ind(self, x, rope_type, rows, head_dim, n_rot, theta, d_pos, freq_factors=None):
        self._sync_stream()
        self.L.refcuda_rope_ind(self._p(x), rope_type, rows, head_dim, n_rot, theta, self._p(d_pos), self._p(freq_factors))

    def kv_store_batch(self, kc, vc, k, v, heads, head_dim, n_ctx, pos_base, batch):
        self._sync_stream()
        self.L.refcuda_kv_store_batch(self._p(kc), self._p(vc), self._p(k), self._p(v), heads, head_dim, n_ctx, pos_base, batch)

    def kv_store_ind(self, kc, vc, k, v, heads, head_dim, n_ctx, d_pos):
        self._sync_stream()
        self.L.refcuda_kv_store_ind(self._p(kc), self._p(vc), self._p(k), self._p(v), heads, head_dim, n_ctx, self._p(d_pos))

    def kv_shift(self, kc, vc, n_layer, n_kv, head_dim, n_ctx, n_keep, shift):
        self._sync_stream()
        self.L.refcuda_kv_shift(self._p(kc), self._p(vc), n_layer, n_kv, head_dim, n_ctx, n_keep, shift)

    def quantize_mmq(self, x, ggml_type, w_blocks, n_out):
        """The reference's quantize_mmq_q8_1_k pass (src/kernels.cu:160-205) as its batched GEMM runs it
        (mmq_batch_launch, :1842-1850): x [batch][n_in] fp32 and a [n_out][n_in] weight of K-quant blocks (uint8
        tensor) go through gemv_batch; returns the activation blocks it left in the scratch block,
        uint8 [n_in/128][batch][144], and the GEMM result [batch][n_out]."""
        torch = self.torch
        self._sync_stream()
        batch, n_in = x.shape
        nbytes = int(self.L.refcuda_scratch_size(n_in, batch))
        arena = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        self.L.refcuda_scratch_assign(self._p(arena), n_in, batch)
        y = torch.empty(batch, n_out, device="cuda")
        self.L.refcuda_gemv_batch(int(ggml_type), self._p(w_blocks), self._p(x), self._p(y), n_in, n_out, batch)
        torch.cuda.current_stream().synchronize()
        n_al = (n_in + 255) // 256 * 256
        off = n_al + (n_al // 32 * 4 + 255) // 256 * 256
        nblk = (n_in + 127) // 128 * batch
        return arena[off:off + nblk * 144].view(-1, batch, 144).clone(), y

    def rms_norm_rows(self, x, w, rows, cols, eps, y):
        self._sync_stream()
        self.L.refcuda_rms_norm_rows(self._p(x), self._p(w), rows, cols, eps, self._p(y))

    def add_inplace_broadcast(self, a, b, stride, batch):
        self._sync_stream()
        self.L.refcuda_add_inplace_broadcast(self._p(a), self._p(b), stride, batch)

    def quantize_activation(self, x, n_in):
        """Returns (int8 values [n_in], fp32 scales [ceil(n_in/32)]) as the reference's GEMV kernels read them."""
        torch = self.torch
        self._sync_stream()
        nbytes = int(self.L.refcuda_scratch_size(n_in, 1))
        arena = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        self.L.refcuda_scratch_assign(self._p(arena), n_in, 1)
        self.L.refcuda_quantize_activation(self._p(x), n_in)
        torch.cuda.current_stream().synchronize()
        n_al = (n_in + 255) // 256 * 256
        qs = arena[:n_in].view(torch.int8).clone()
        scales = arena[n_al:n_al + 4 * ((n_in + 31) // 32)].view(torch.float32).clone()
        return qs, scales
