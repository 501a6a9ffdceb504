"""Host-side mirror of the reference's kernel wrappers for the attention path.

Function names, argument order and meaning follow `namespace llm::cuda` in the reference
(src/kernels.h:53-81); tensors are torch CUDA tensors where the reference takes raw device
pointers.  Everything is forwarded to the C ABI (include/orin_attn_b200.h) through ctypes --
torch is used only for device memory and streams.  There is no CPU implementation here.
"""
import ctypes
import math

import torch

from . import capi
from .capi import (FUSE_ALL, FUSE_KV_APPEND, FUSE_NONE, FUSE_ROPE_K, FUSE_ROPE_Q, PART_PAD, ROPE_NEOX,  # noqa: F401
                   ROPE_NORMAL)

_state = {"device": None, "stream": None, "decode_ws": {}, "prefill_ws": {}}


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    s = _state["stream"]
    if s is None:
        s = torch.cuda.current_stream().cuda_stream
    return ctypes.c_void_p(s)


def init(device=0):
    """cuda::init (src/kernels.cu:1730-1737) for `device`; must precede every other call."""
    if not torch.cuda.is_available():
        raise RuntimeError("orin_llm_b200 needs a CUDA device (B200, sm_100a); there is no CPU path")
    torch.cuda.set_device(device)
    torch.cuda.current_stream()  # make sure the primary context exists
    capi.check(capi.lib().oattn_init(device))
    _state["device"] = device
    return 0


def set_stream(stream):
    """cuda::set_stream (src/kernels.cu:1726-1728).  `stream`: torch.cuda.Stream, raw handle or None."""
    if stream is None:
        _state["stream"] = None
    elif isinstance(stream, torch.cuda.Stream):
        _state["stream"] = stream.cuda_stream
    else:
        _state["stream"] = int(stream)


def sm_count():
    return capi.lib().oattn_sm_count()


def launch_count():
    return int(capi.lib().oattn_launch_count())


def _rope(x, rows, head_dim, rope_type, n_rot, theta, n_past, heads, d_pos, freq_factors):
    assert x.dtype == torch.float32 and x.is_contiguous()
    capi.check(capi.lib().oattn_rope(_ptr(x), rows, head_dim, rope_type, n_rot, theta, n_past, heads, _ptr(d_pos),
                                     _ptr(freq_factors), _stream()))


def rope_neox_batch(x, rows, head_dim, n_rot, theta, n_past, heads, freq_factors=None):
    _rope(x, rows, head_dim, ROPE_NEOX, n_rot, theta, n_past, heads, None, freq_factors)


def rope_normal_batch(x, rows, head_dim, n_rot, theta, n_past, heads, freq_factors=None):
    _rope(x, rows, head_dim, ROPE_NORMAL, n_rot, theta, n_past, heads, None, freq_factors)


def rope_neox_ind(x, rows, head_dim, n_rot, theta, d_pos, freq_factors=None):
    _rope(x, rows, head_dim, ROPE_NEOX, n_rot, theta, 0, 1, d_pos, freq_factors)


def rope_normal_ind(x, rows, head_dim, n_rot, theta, d_pos, freq_factors=None):
    _rope(x, rows, head_dim, ROPE_NORMAL, n_rot, theta, 0, 1, d_pos, freq_factors)


def kv_store_batch(kc, vc, k, v, heads, head_dim, n_ctx, pos_base, batch):
    capi.check(capi.lib().oattn_kv_store(_ptr(kc), _ptr(vc), _ptr(k), _ptr(v), heads, head_dim, n_ctx, pos_base, batch,
                                         None, _stream()))


def kv_store_ind(kc, vc, k, v, heads, head_dim, n_ctx, d_pos):
    capi.check(capi.lib().oattn_kv_store(_ptr(kc), _ptr(vc), _ptr(k), _ptr(v), heads, head_dim, n_ctx, 0, 1, _ptr(d_pos),
                                         _stream()))


def kv_shift(kc, vc, n_layer, n_kv, head_dim, n_ctx, n_keep, shift):
    capi.check(capi.lib().oattn_kv_shift(_ptr(kc), _ptr(vc), n_layer, n_kv, head_dim, n_ctx, n_keep, shift, _stream()))


def decode_workspace(n_head, n_kv, head_dim, device=None):
    """Scratch for the decode calls, allocated once per shape (scratch_size/scratch_assign pattern,
    src/kernels.cu:1753-1776)."""
    key = (n_head, n_kv, head_dim, torch.cuda.current_device())
    ws = _state["decode_ws"].get(key)
    if ws is None:
        nbytes = capi.lib().oattn_decode_workspace_bytes(n_head, n_kv, head_dim)
        if nbytes == 0:
            raise capi.AttnError(capi.ERR_UNSUPPORTED, "decode shape not supported or init() not called")
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        _state["decode_ws"][key] = ws
    return ws


def prefill_workspace(n_head, n_kv, head_dim, batch):
    key = (n_head, n_kv, head_dim, torch.cuda.current_device())
    ws = _state["prefill_ws"].get(key)
    nbytes = capi.lib().oattn_prefill_workspace_bytes(n_head, n_kv, head_dim, batch)
    if nbytes == 0:
        raise capi.AttnError(capi.ERR_UNSUPPORTED, "prefill shape not supported")
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        _state["prefill_ws"][key] = ws
    return ws


def _rope_params(rope):
    if rope is None:
        return None, None
    rope_type, n_rot, theta, ff = rope
    p = capi.RopeParams(rope_type, n_rot, theta, 0 if ff is None else ff.data_ptr())
    return ctypes.byref(p), p


def flash_attention(q, kc, vc, out, n_head, n_kv, head_dim, n_ctx, n_past, batch, scale, workspace=None):
    """cuda::flash_attention (src/kernels.cu:1974-1981): q already rotated, cache already written."""
    attn_prefill(q, None, None, kc, vc, out, n_head, n_kv, head_dim, n_ctx, n_past, batch, scale, FUSE_NONE, None,
                 workspace)


def flash_attention_decode_ind(q, kc, vc, out, n_head, n_kv, head_dim, n_ctx, d_pos, scale, workspace=None):
    """cuda::flash_attention_decode_ind (src/kernels.cu:1993-2000)."""
    attn_decode(q, None, None, kc, vc, out, n_head, n_kv, head_dim, n_ctx, d_pos, scale, FUSE_NONE, None, workspace)


def _ext_params(ext):
    """ext: dict with any of bias_q, bias_k, bias_v, norm_q, norm_k (fp32 CUDA tensors), norm_eps (float), out_qs (int8
    tensor), out_scales (fp32 tensor), out_mmq (uint8 tensor of 144-byte blocks, prefill only), out_mmq_ds4 (bool)
    -> (pointer to capi.Ext or None, object to keep alive)."""
    if not ext:
        return None, None
    unknown = set(ext) - {"bias_q", "bias_k", "bias_v", "norm_q", "norm_k", "norm_eps", "out_qs", "out_scales", "out_mmq",
                           "out_mmq_ds4"}
    if unknown:
        raise ValueError("unknown extension keys: %s" % sorted(unknown))
    e = capi.Ext()
    for name in ("bias_q", "bias_k", "bias_v", "norm_q", "norm_k", "out_qs", "out_scales", "out_mmq"):
        t = ext.get(name)
        setattr(e, name, t.data_ptr() if t is not None else None)
    e.norm_eps = float(ext.get("norm_eps", 0.0))
    e.out_mmq_ds4 = 1 if ext.get("out_mmq_ds4") else 0
    return ctypes.byref(e), e


def attn_decode(q, k_new, v_new, kc, vc, out, n_head, n_kv, head_dim, n_ctx, d_pos, scale, fuse=FUSE_ALL, rope=None,
                workspace=None, ext=None):
    """Fused decode step of one layer (src/model_gpu.cu:277-282).  rope = (rope_type, n_rot, theta, freq_factors);
    ext: optional bias / per-head norm in front and q8_1 output behind (see _ext_params)."""
    ws = workspace if workspace is not None else decode_workspace(n_head, n_kv, head_dim)
    ref, keep = _rope_params(rope)
    if ext:
        eref, ekeep = _ext_params(ext)
        capi.check(capi.lib().oattn_decode_ex(_ptr(q), _ptr(k_new), _ptr(v_new), _ptr(kc), _ptr(vc), _ptr(out), n_head, n_kv,
                                              head_dim, n_ctx, _ptr(d_pos), scale, fuse, ref, eref, _ptr(ws), ws.numel(),
                                              _stream()))
        del ekeep
    else:
        capi.check(capi.lib().oattn_decode(_ptr(q), _ptr(k_new), _ptr(v_new), _ptr(kc), _ptr(vc), _ptr(out), n_head, n_kv,
                                           head_dim, n_ctx, _ptr(d_pos), scale, fuse, ref, _ptr(ws), ws.numel(), _stream()))
    del keep


def attn_decode_partial(q, kc, vc, part, n_head, n_kv, head_dim, n_ctx, d_len, scale, workspace=None):
    """Partial (m, l, O) over the local cache rows [0, *d_len); part [n_head][head_dim+4] fp32."""
    ws = workspace if workspace is not None else decode_workspace(n_head, n_kv, head_dim)
    capi.check(capi.lib().oattn_decode_partial(_ptr(q), _ptr(kc), _ptr(vc), _ptr(part), n_head, n_kv, head_dim, n_ctx,
                                               _ptr(d_len), scale, _ptr(ws), ws.numel(), _stream()))


def peer_buffer_bytes(world, n_head, head_dim):
    return int(capi.lib().oattn_peer_buffer_bytes(world, n_head, head_dim))


def peer_state_bytes(n_head):
    return int(capi.lib().oattn_peer_state_bytes(n_head))


def attn_decode_partial_push(q, kc, vc, n_head, n_kv, head_dim, n_ctx, d_len, scale, peer_bufs_dev, rank, world, state,
                             workspace=None):
    """Partial (m, l, O) over the local rows, stored straight into every rank's exchange buffer (peer stores).
    peer_bufs_dev: address of a device array holding `world` buffer pointers; state: uint8 tensor of
    peer_state_bytes(n_head), zero-filled once."""
    ws = workspace if workspace is not None else decode_workspace(n_head, n_kv, head_dim)
    capi.check(capi.lib().oattn_decode_partial_push(_ptr(q), _ptr(kc), _ptr(vc), n_head, n_kv, head_dim, n_ctx, _ptr(d_len),
                                                    scale, _ptr(ws), ws.numel(), ctypes.c_void_p(int(peer_bufs_dev)), rank,
                                                    world, _ptr(state), _stream()))


def attn_decode_peer(q, kc, vc, out, n_head, n_kv, head_dim, n_ctx, d_len, scale, peer_bufs_dev, rank, world, state,
                     workspace=None):
    """Split-KV decode over this rank's rows with the record exchange and the final merge inside the merge launch
    (every rank on a GPU of its own).  out [n_head][head_dim] is written on every rank."""
    ws = workspace if workspace is not None else decode_workspace(n_head, n_kv, head_dim)
    capi.check(capi.lib().oattn_decode_peer(_ptr(q), _ptr(kc), _ptr(vc), _ptr(out), n_head, n_kv, head_dim, n_ctx, _ptr(d_len),
                                            scale, _ptr(ws), ws.numel(), ctypes.c_void_p(int(peer_bufs_dev)), rank, world,
                                            _ptr(state), _stream()))


def attn_decode_peer_fused(q, k_new, v_new, kc, vc, out, n_head, n_kv, head_dim, n_ctx, d_len, d_rope_pos, scale, fuse, rope,
                           peer_bufs_dev, rank, world, state, workspace=None):
    """attn_decode_peer with the fused prologue on a row-sharded cache: RoPE(q) on every rank at the global position
    *d_rope_pos; the rank that receives the new token also rotates and appends k_new / v_new (local row *d_len - 1)."""
    ws = workspace if workspace is not None else decode_workspace(n_head, n_kv, head_dim)
    ref, keep = _rope_params(rope)
    capi.check(capi.lib().oattn_decode_peer_fused(_ptr(q), _ptr(k_new), _ptr(v_new), _ptr(kc), _ptr(vc), _ptr(out), n_head, n_kv,
                                                  head_dim, n_ctx, _ptr(d_len), _ptr(d_rope_pos), scale, fuse, ref, _ptr(ws),
                                                  ws.numel(), ctypes.c_void_p(int(peer_bufs_dev)), rank, world, _ptr(state),
                                                  _stream()))
    del keep


def attn_peer_wait_combine(my_buf, world, out, n_head, head_dim, state):
    """Wait (bounded) until every rank's record of this step has landed in `my_buf`, then merge them into out."""
    capi.check(capi.lib().oattn_peer_wait_combine(_ptr(my_buf), world, _ptr(out), n_head, head_dim, _ptr(state), _stream()))


def peer_status(state, n_head):
    st = ctypes.c_int(-1)
    capi.check(capi.lib().oattn_peer_status(_ptr(state), n_head, ctypes.byref(st)))
    return st.value


def attn_combine(parts, n_parts, out, n_head, head_dim):
    capi.check(capi.lib().oattn_combine(_ptr(parts), n_parts, _ptr(out), n_head, head_dim, _stream()))


def attn_prefill(q, k_new, v_new, kc, vc, out, n_head, n_kv, head_dim, n_ctx, n_past, batch, scale, fuse=FUSE_ALL,
                 rope=None, workspace=None, ext=None):
    """Fused prefill step of one layer (src/model_gpu.cu:372-384).  ext: optional bias / per-head norm (_ext_params)."""
    ws = workspace if workspace is not None else prefill_workspace(n_head, n_kv, head_dim, batch)
    ref, keep = _rope_params(rope)
    eref, ekeep = _ext_params(ext)
    capi.check(capi.lib().oattn_prefill_ex(_ptr(q), _ptr(k_new), _ptr(v_new), _ptr(kc), _ptr(vc), _ptr(out), n_head, n_kv,
                                           head_dim, n_ctx, n_past, batch, scale, fuse, ref, eref, _ptr(ws), ws.numel(),
                                           _stream()))
    del keep, ekeep


def prefill_status(n_head, n_kv, head_dim, batch, workspace=None):
    """Status word of the last attn_prefill call with this shape (blocking read; 0 = completed)."""
    ws = workspace if workspace is not None else prefill_workspace(n_head, n_kv, head_dim, batch)
    st = ctypes.c_int(-1)
    capi.check(capi.lib().oattn_prefill_status(_ptr(ws), n_head, head_dim, batch, ctypes.byref(st)))
    return st.value


def set_prefill_impl(impl):
    capi.check(capi.lib().oattn_set_prefill_impl(impl))


def set_decode_overlap(mode):
    """0 ordinary launches (default), 1 dependent launches, 2 also prefetch K/V before waiting for the preceding kernel
    (the caller vouches for the position word and the cache rows below the newest one; see the C header)."""
    capi.check(capi.lib().oattn_set_decode_overlap(mode))


def set_wait_limit_cycles(cycles):
    """Bound of the device-side waits for the peers' records, in SM clock cycles (default 4e9)."""
    capi.check(capi.lib().oattn_set_wait_limit_cycles(int(cycles)))


def set_decode_min_tiles(tiles):
    capi.check(capi.lib().oattn_set_decode_min_tiles(tiles))


def profile_enable(max_records):
    """Time the decode kernel of the next `max_records` decode calls (0 switches it off)."""
    capi.check(capi.lib().oattn_profile_enable(max_records))


def profile_collect(capacity=65536):
    """Milliseconds of the decode kernel for each decode call recorded since the last collect."""
    buf = (ctypes.c_float * capacity)()
    n = ctypes.c_int(0)
    capi.check(capi.lib().oattn_profile_collect(buf, capacity, ctypes.byref(n)))
    return [buf[i] for i in range(n.value)]


class KVCache:
    """Device KV cache with the reference's layout (src/model_gpu.cu:229-235, 255-260): one
    allocation, K of all layers first, then V; per layer [n_kv][n_ctx][head_dim] fp16.  Unlike the
    reference it is zero-filled once, so rows that were never written are finite."""

    def __init__(self, n_layer, n_kv, n_ctx, head_dim, device="cuda"):
        self.n_layer, self.n_kv, self.n_ctx, self.head_dim = n_layer, n_kv, n_ctx, head_dim
        self.per_layer = n_kv * n_ctx * head_dim
        self.buf = torch.zeros(2 * n_layer * self.per_layer, dtype=torch.float16, device=device)
        self.k = self.buf[: n_layer * self.per_layer].view(n_layer, n_kv, n_ctx, head_dim)
        self.v = self.buf[n_layer * self.per_layer:].view(n_layer, n_kv, n_ctx, head_dim)

    def layer(self, l):
        return self.k[l], self.v[l]

    def shift(self, n_keep, shift):
        """Model::kv_shift (src/model_gpu.cu:413-416)."""
        if shift <= 0 or shift > self.n_ctx:
            return
        kv_shift(self.k, self.v, self.n_layer, self.n_kv, self.head_dim, self.n_ctx, n_keep, shift)


def default_scale(head_dim):
    return 1.0 / math.sqrt(head_dim)
