// Host-side C++ interface of the attention path, with the reference's names and signatures.
//
// This header mirrors the attention-path part of the reference's src/kernels.h (lines 53-81):
// same namespace, same function names, same argument order and meaning, raw device pointers.  A
// maintainer of the reference keeps calling these from src/model_gpu.cu; the definitions
// (kernels.cpp next to this file) forward to the C ABI in include/orin_attn_b200.h instead of
// launching the sm_87 kernels of src/kernels.cu.
//
// Differences from the reference, all additive:
//   - attn_scratch_size()/attn_scratch_assign(): the split-KV decode kernel and the tcgen05 prefill
//     kernel need scratch (partial results, fp16 query staging).  It follows the reference's own
//     scratch_size()/scratch_assign() pattern (src/kernels.cu:1753-1776): sized once, carved out
//     of the caller's arena, handed over once.
//   - attention_decode_fused()/attention_prefill_fused(): one call for the sequences
//     rope(q), rope(k), kv_store, flash_attention* at src/model_gpu.cu:277-282 and 379-384.
//   - AttnExtras: the steps on either side of attention that the fused calls can absorb -- q/k/v bias add and
//     per-head q/k RMSNorm (src/model_gpu.cu:372-377, 274-275) in front, the q8_1 activation form that
//     quantize_activation(d_attn_) produces for the Wo GEMV (src/model_gpu.cu:284) behind (decode only).
// Error convention as in the reference (src/common.h:10-22): a failed call prints and aborts.
#pragma once

#include <stddef.h>
#include <stdint.h>

namespace llm::cuda {

int init();                       // src/kernels.cu:1730-1737 (device 0)
int init_device(int device);      // same, for one process per GPU
void set_stream(void* stream);    // src/kernels.cu:1726-1728
// Same effect under a name of its own, for a host that links this library NEXT TO the reference's kernels.cu (whose own
// set_stream then keeps serving its GEMV kernels): call both, or wrap the reference's at link time.
void attn_set_stream(void* stream);

// Call-sequence fusion, off by default (on with attn_fuse_call_sequence(true) or OATTN_FUSE_CALL_SEQUENCE=1 in the
// environment): rope(q), rope(k), kv_store are recorded instead of launched, and when the attention call that follows
// consumes exactly them, the four become the one fused launch -- the reference's unmodified call sites
// (src/model_gpu.cu:277-282, 379-384) then cost what attention_*_fused costs.  Any other call first issues what is
// recorded, in order.  Visible difference: q and k are not rotated in place any more; turn it on only for a host that,
// like the reference, does not read them after attention.
void attn_fuse_call_sequence(bool on);
// Issues whatever rope / kv_store calls are still recorded, in order.  With fusion on, a host must call this before it
// launches a kernel of its own that reads q, k or the cache, before it synchronises or ends a stream capture, and
// before it frees a buffer a recorded call names -- recorded calls are otherwise only issued by the next call
// through these wrappers.  (The reference's own sequence, where the attention call directly follows, never needs it.)
void attn_flush();

// Optional.  Without them the first wrapper call initialises the current device, prefill scratch is allocated on
// demand and decode (fused or not) runs on the library's built-in 2 MiB scratch block: no decode call ever allocates,
// so all of them may be captured in a CUDA graph as src/model_gpu.cu:295-316 does.  A shape whose decode scratch does
// not fit the built-in block aborts with a message that asks for attn_scratch_assign().
size_t attn_scratch_size(int n_head, int n_kv, int head_dim, int max_batch);
void attn_scratch_assign(void* base, int n_head, int n_kv, int head_dim, int max_batch);

// --- RoPE (src/kernels.h:55-62) ---
void rope_neox_batch(float* x, int rows, int head_dim, int n_rot, float theta, int n_past, int heads, const float* freq_factors = nullptr);
void rope_normal_batch(float* x, int rows, int head_dim, int n_rot, float theta, int n_past, int heads, const float* freq_factors = nullptr);
void rope_neox_ind(float* x, int rows, int head_dim, int n_rot, float theta, const int* d_pos, const float* freq_factors = nullptr);
void rope_normal_ind(float* x, int rows, int head_dim, int n_rot, float theta, const int* d_pos, const float* freq_factors = nullptr);

// --- KV cache (src/kernels.h:66-73) ---
void kv_store_batch(uint16_t* kc, uint16_t* vc, const float* k, const float* v,
                    int heads, int head_dim, int n_ctx, int pos_base, int batch);
void kv_store_ind(uint16_t* kc, uint16_t* vc, const float* k, const float* v,
                  int heads, int head_dim, int n_ctx, const int* d_pos);
void kv_shift(uint16_t* kc, uint16_t* vc, int n_layer, int n_kv, int head_dim, int n_ctx, int n_keep, int shift);

// --- Flash attention (src/kernels.h:77-81) ---
void flash_attention(const float* q, const uint16_t* kc, const uint16_t* vc, float* out,
                    int n_head, int n_kv, int head_dim, int n_ctx, int n_past, int batch, float scale);
void flash_attention_decode_ind(const float* q, const uint16_t* kc, const uint16_t* vc, float* out,
                                int n_head, int n_kv, int head_dim, int n_ctx, const int* d_pos, float scale);

// --- fused call-site replacements ---
// rope_type: 0 = normal, 1 = neox (HParams::rope_type, src/model.h:27-28).  q and k are NOT modified
// (the reference rotates them in place; nothing downstream reads them after attention).
void attention_decode_fused(const float* q, const float* k, const float* v, uint16_t* kc, uint16_t* vc, float* out,
                            int n_head, int n_kv, int head_dim, int n_ctx, const int* d_pos, float scale,
                            int rope_type, int n_rot, float theta, const float* freq_factors = nullptr);
void attention_prefill_fused(const float* q, const float* k, const float* v, uint16_t* kc, uint16_t* vc, float* out,
                             int n_head, int n_kv, int head_dim, int n_ctx, int n_past, int batch, float scale,
                             int rope_type, int n_rot, float theta, const float* freq_factors = nullptr);

// Optional extras of the fused calls; device pointers, nullptr = step absent.
struct AttnExtras {
    const float* bq = nullptr;        // [n_head*head_dim]   Layer::bq
    const float* bk = nullptr;        // [n_kv*head_dim]     Layer::bk
    const float* bv = nullptr;        // [n_kv*head_dim]     Layer::bv
    const float* q_norm = nullptr;    // [head_dim]          Layer::wq_norm
    const float* k_norm = nullptr;    // [head_dim]          Layer::wk_norm
    float rms_eps = 0.0f;             // HParams::rms_eps
    int8_t* q8 = nullptr;             // decode only: int8 [n_head*head_dim], as g_q8 (src/kernels.cu:1748)
    float* q8_scale = nullptr;        //              fp32 [n_head*head_dim/32], as g_q8_scale (src/kernels.cu:1749)
    void* q8_mmq = nullptr;           // prefill only: block_q8_1_mmq blocks [n_head][batch], as g_q8_mmq (src/kernels.cu:1750)
    bool q8_mmq_ds4 = false;          //               true when Wo is Q4_K (scales as fp16 (d, sum)), false for Q6_K
};
void attention_decode_fused(const float* q, const float* k, const float* v, uint16_t* kc, uint16_t* vc, float* out,
                            int n_head, int n_kv, int head_dim, int n_ctx, const int* d_pos, float scale,
                            int rope_type, int n_rot, float theta, const float* freq_factors, const AttnExtras& extras);
void attention_prefill_fused(const float* q, const float* k, const float* v, uint16_t* kc, uint16_t* vc, float* out,
                             int n_head, int n_kv, int head_dim, int n_ctx, int n_past, int batch, float scale,
                             int rope_type, int n_rot, float theta, const float* freq_factors, const AttnExtras& extras);

} // namespace llm::cuda
