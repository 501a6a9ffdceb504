"""ctypes binding of include/orin_attn_b200.h.

The shared library is the product; this module only loads it and declares the prototypes.
There is no CPU path: if the library is missing or cannot be loaded, importing this module's
`lib()` raises.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "liborin_attn_b200.so")

OK = 0
ERR_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_CUDA, ERR_DEVICE = 1, 2, 3, 4, 5
ROPE_NORMAL, ROPE_NEOX = 0, 1
FUSE_NONE, FUSE_ROPE_Q, FUSE_ROPE_K, FUSE_KV_APPEND, FUSE_ALL = 0, 1, 2, 4, 7
PART_PAD = 4

# Every symbol include/orin_attn_b200.h declares.
EXPORTS = [
    "oattn_strerror", "oattn_last_cuda_error", "oattn_init", "oattn_scratch_alloc", "oattn_scratch_free", "oattn_builtin_scratch", "oattn_weights_place", "oattn_logits_alloc", "oattn_logits_free",
    "oattn_copy_to_host_async", "oattn_device_clear", "oattn_sm_count", "oattn_rope",
    "oattn_kv_store", "oattn_kv_shift", "oattn_decode_workspace_bytes", "oattn_decode",
    "oattn_decode_ex", "oattn_prefill_ex", "oattn_decode_noalloc_max_bytes", "oattn_decode_noalloc",
    "oattn_decode_partial", "oattn_combine", "oattn_peer_buffer_bytes", "oattn_peer_state_bytes",
    "oattn_decode_partial_push", "oattn_peer_wait_combine", "oattn_decode_peer", "oattn_decode_peer_fused", "oattn_peer_status", "oattn_prefill_workspace_bytes", "oattn_prefill",
    "oattn_prefill_status",
    "oattn_set_prefill_impl", "oattn_set_decode_min_tiles", "oattn_set_decode_overlap", "oattn_set_wait_limit_cycles", "oattn_profile_enable", "oattn_profile_collect",
    "oattn_launch_count",
]


class RopeParams(ctypes.Structure):
    _fields_ = [("rope_type", ctypes.c_int), ("n_rot", ctypes.c_int), ("theta", ctypes.c_float),
                ("freq_factors", ctypes.c_void_p)]


class Ext(ctypes.Structure):
    _fields_ = [("bias_q", ctypes.c_void_p), ("bias_k", ctypes.c_void_p), ("bias_v", ctypes.c_void_p),
                ("norm_q", ctypes.c_void_p), ("norm_k", ctypes.c_void_p), ("norm_eps", ctypes.c_float),
                ("out_qs", ctypes.c_void_p), ("out_scales", ctypes.c_void_p), ("out_mmq", ctypes.c_void_p),
                ("out_mmq_ds4", ctypes.c_int)]


class AttnError(RuntimeError):
    def __init__(self, code, text):
        super().__init__("orin_attn_b200 error %d: %s" % (code, text))
        self.code = code


_lib = None


def lib():
    """Load liborin_attn_b200.so (once) and declare prototypes.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "CUDA library %s is not built; run `python -m orin_llm_b200.build`. "
            "There is no CPU fallback." % LIB_PATH)
    L = ctypes.CDLL(LIB_PATH)
    vp, i, f, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
    rp = ctypes.POINTER(RopeParams)
    L.oattn_strerror.restype = ctypes.c_char_p
    L.oattn_strerror.argtypes = [i]
    L.oattn_last_cuda_error.restype = ctypes.c_char_p
    L.oattn_last_cuda_error.argtypes = []
    L.oattn_init.argtypes = [i]
    L.oattn_sm_count.argtypes = []
    L.oattn_scratch_alloc.argtypes = [sz, ctypes.POINTER(ctypes.c_void_p)]
    L.oattn_scratch_free.argtypes = [vp]
    L.oattn_builtin_scratch.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(sz)]
    pvp = ctypes.POINTER(ctypes.c_void_p)
    L.oattn_weights_place.argtypes = [vp, sz, pvp]
    L.oattn_logits_alloc.argtypes = [sz, pvp, pvp]
    L.oattn_logits_free.argtypes = [vp, vp]
    L.oattn_copy_to_host_async.argtypes = [vp, vp, sz, vp]
    L.oattn_device_clear.argtypes = [vp, sz]
    L.oattn_rope.argtypes = [vp, i, i, i, i, f, i, i, vp, vp, vp]
    L.oattn_kv_store.argtypes = [vp, vp, vp, vp, i, i, i, i, i, vp, vp]
    L.oattn_kv_shift.argtypes = [vp, vp, i, i, i, i, i, i, vp]
    L.oattn_decode_workspace_bytes.restype = sz
    L.oattn_decode_workspace_bytes.argtypes = [i, i, i]
    L.oattn_decode.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, vp, f, i, rp, vp, sz, vp]
    ep = ctypes.POINTER(Ext)
    L.oattn_decode_ex.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, vp, f, i, rp, ep, vp, sz, vp]
    L.oattn_prefill_ex.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, f, i, rp, ep, vp, sz, vp]
    L.oattn_decode_noalloc_max_bytes.restype = sz
    L.oattn_decode_noalloc_max_bytes.argtypes = []
    L.oattn_decode_noalloc.argtypes = [vp, vp, vp, vp, i, i, i, i, vp, f, vp]
    L.oattn_decode_partial.argtypes = [vp, vp, vp, vp, i, i, i, i, vp, f, vp, sz, vp]
    L.oattn_combine.argtypes = [vp, i, vp, i, i, vp]
    L.oattn_peer_buffer_bytes.restype = sz
    L.oattn_peer_buffer_bytes.argtypes = [i, i, i]
    L.oattn_peer_state_bytes.restype = sz
    L.oattn_peer_state_bytes.argtypes = [i]
    L.oattn_decode_partial_push.argtypes = [vp, vp, vp, i, i, i, i, vp, f, vp, sz, vp, i, i, vp, vp]
    L.oattn_peer_wait_combine.argtypes = [vp, i, vp, i, i, vp, vp]
    L.oattn_decode_peer.argtypes = [vp, vp, vp, vp, i, i, i, i, vp, f, vp, sz, vp, i, i, vp, vp]
    L.oattn_decode_peer_fused.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, vp, vp, f, i, rp, vp, sz, vp, i, i, vp, vp]
    L.oattn_peer_status.argtypes = [vp, i, ctypes.POINTER(ctypes.c_int)]
    L.oattn_prefill_workspace_bytes.restype = sz
    L.oattn_prefill_workspace_bytes.argtypes = [i, i, i, i]
    L.oattn_prefill.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, f, i, rp, vp, sz, vp]
    L.oattn_prefill_status.argtypes = [vp, i, i, i, ctypes.POINTER(ctypes.c_int)]
    L.oattn_set_prefill_impl.argtypes = [i]
    L.oattn_set_decode_min_tiles.argtypes = [i]
    L.oattn_set_decode_overlap.argtypes = [i]
    L.oattn_set_wait_limit_cycles.argtypes = [ctypes.c_longlong]
    L.oattn_profile_enable.argtypes = [i]
    L.oattn_profile_collect.argtypes = [ctypes.POINTER(ctypes.c_float), i, ctypes.POINTER(ctypes.c_int)]
    L.oattn_launch_count.restype = ctypes.c_ulonglong
    L.oattn_launch_count.argtypes = []
    _lib = L
    return L


def check(code):
    if code != OK:
        L = lib()
        text = L.oattn_strerror(code).decode()
        if code == ERR_CUDA:
            text += " (" + L.oattn_last_cuda_error().decode() + ")"
        raise AttnError(code, text)
