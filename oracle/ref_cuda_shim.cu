// TEST INFRASTRUCTURE ONLY -- never linked into or called by the product.
//
// C entry points over the reference's own CUDA wrappers (namespace llm::cuda, src/kernels.h:8-81), so that the
// GPU tests and the benchmark can run the reference's unmodified attention-path kernels, recompiled for
// sm_100a, next to this repository's kernels: a second parity check (GPU against GPU) and the "recompiled
// reference kernel" timing.  This file only forwards; the kernels come from the reference's src/kernels.cu,
// compiled from where it lies by oracle/Makefile (target refcuda) into oracle/_ref/libref_cuda.so.
//
// Limits of the reference kernels that callers of this shim must respect (read from src/kernels.cu):
//   * flash_attention_decode_ind loads whole 128-row tiles (:1183-1196): n_ctx must be a multiple of 128 and
//     the cache must be initialised up to the next multiple of 128 past the position;
//   * flash_attention loads whole 64-row tiles (:1430-1445): n_ctx a multiple of 64, same initialisation;
//   * both pad the GQA group to 8 columns (:1117, :1361): n_head / n_kv <= 8;
//   * everything runs on device 0 and on the stream given to set_stream (:1726-1735).
#include <cuda_runtime.h>

#include "kernels.h"

extern "C" {

int refcuda_init(void) { return llm::cuda::init(); }
void refcuda_set_stream(void* stream) { llm::cuda::set_stream(stream); }
size_t refcuda_scratch_size(int max_in, int max_batch) { return llm::cuda::scratch_size(max_in, max_batch); }
void refcuda_scratch_assign(void* base, int max_in, int max_batch) { llm::cuda::scratch_assign(base, max_in, max_batch); }

// src/kernels.h:15 -- writes int8 values at the scratch base and one fp32 scale per 32 values after them
// (layout fixed by scratch_assign, src/kernels.cu:1763-1776).
void refcuda_quantize_activation(const float* x, int n_in) { llm::cuda::quantize_activation(x, n_in); }

// src/kernels.h: gemv_batch.  For Q4_K / Q6_K weights (ggml types 12 / 14) it first writes X as block_q8_1_mmq blocks
// into the scratch block, behind the q8_1 values and scales (layout fixed by scratch_assign, src/kernels.cu:1763-1776).
void refcuda_gemv_batch(int type, const void* W, const float* X, float* Y, int n_in, int n_out, int batch) {
    llm::cuda::gemv_batch((llm::DType)type, W, X, Y, n_in, n_out, batch);
}

void refcuda_rms_norm_rows(const float* x, const float* w, int rows, int cols, float eps, float* y) {
    llm::cuda::rms_norm_rows(x, w, rows, cols, eps, y);
}
void refcuda_add_inplace_broadcast(float* a, const float* b, int stride, int batch) {
    llm::cuda::add_inplace_broadcast(a, b, stride, batch);
}

void refcuda_rope_batch(float* x, int rope_type, int rows, int head_dim, int n_rot, float theta, int n_past, int heads,
                        const float* freq_factors) {
    if (rope_type == 1) llm::cuda::rope_neox_batch(x, rows, head_dim, n_rot, theta, n_past, heads, freq_factors);
    else                llm::cuda::rope_normal_batch(x, rows, head_dim, n_rot, theta, n_past, heads, freq_factors);
}
void refcuda_rope_ind(float* x, int rope_type, int rows, int head_dim, int n_rot, float theta, const int* d_pos,
                      const float* freq_factors) {
    if (rope_type == 1) llm::cuda::rope_neox_ind(x, rows, head_dim, n_rot, theta, d_pos, freq_factors);
    else                llm::cuda::rope_normal_ind(x, rows, head_dim, n_rot, theta, d_pos, freq_factors);
}

void refcuda_kv_store_batch(uint16_t* kc, uint16_t* vc, const float* k, const float* v, int heads, int head_dim, int n_ctx,
                            int pos_base, int batch) {
    llm::cuda::kv_store_batch(kc, vc, k, v, heads, head_dim, n_ctx, pos_base, batch);
}
void refcuda_kv_store_ind(uint16_t* kc, uint16_t* vc, const float* k, const float* v, int heads, int head_dim, int n_ctx,
                          const int* d_pos) {
    llm::cuda::kv_store_ind(kc, vc, k, v, heads, head_dim, n_ctx, d_pos);
}
void refcuda_kv_shift(uint16_t* kc, uint16_t* vc, int n_layer, int n_kv, int head_dim, int n_ctx, int n_keep, int shift) {
    llm::cuda::kv_shift(kc, vc, n_layer, n_kv, head_dim, n_ctx, n_keep, shift);
}

void refcuda_flash_attention(const float* q, const uint16_t* kc, const uint16_t* vc, float* out, int n_head, int n_kv,
                             int head_dim, int n_ctx, int n_past, int batch, float scale) {
    llm::cuda::flash_attention(q, kc, vc, out, n_head, n_kv, head_dim, n_ctx, n_past, batch, scale);
}
void refcuda_flash_attention_decode_ind(const float* q, const uint16_t* kc, const uint16_t* vc, float* out, int n_head,
                                        int n_kv, int head_dim, int n_ctx, const int* d_pos, float scale) {
    llm::cuda::flash_attention_decode_ind(q, kc, vc, out, n_head, n_kv, head_dim, n_ctx, d_pos, scale);
}

}  // extern "C"
