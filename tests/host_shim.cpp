// Test-only shim: plain-C entry points that call the C++ wrappers of orin_llm_b200/host/kernels.h, so
// that pytest can drive the reference-named C++ interface through ctypes.
#include "../orin_llm_b200/host/kernels.h"

using namespace llm;

extern "C" {
int shim_init(int device) { return cuda::init_device(device); }
void shim_set_stream(void* s) { cuda::set_stream(s); }
size_t shim_scratch_size(int n_head, int n_kv, int hd, int max_batch) { return cuda::attn_scratch_size(n_head, n_kv, hd, max_batch); }
void shim_scratch_assign(void* base, int n_head, int n_kv, int hd, int max_batch) { cuda::attn_scratch_assign(base, n_head, n_kv, hd, max_batch); }
// The reference's decode sequence of one layer (src/model_gpu.cu:277-282), unfused.
void shim_decode_layer_unfused(float* q, float* k, const float* v, uint16_t* kc, uint16_t* vc, float* out, int n_head,
                               int n_kv, int hd, int n_ctx, const int* d_pos, float scale, int rope_type, int n_rot,
                               float theta) {
    auto rope_ind = rope_type == 1 ? cuda::rope_neox_ind : cuda::rope_normal_ind;
    rope_ind(q, n_head, hd, n_rot, theta, d_pos, nullptr);
    rope_ind(k, n_kv, hd, n_rot, theta, d_pos, nullptr);
    cuda::kv_store_ind(kc, vc, k, v, n_kv, hd, n_ctx, d_pos);
    cuda::flash_attention_decode_ind(q, kc, vc, out, n_head, n_kv, hd, n_ctx, d_pos, scale);
}
// The reference's prefill sequence of one layer (src/model_gpu.cu:379-384), unfused.
void shim_prefill_layer_unfused(float* q, float* k, const float* v, uint16_t* kc, uint16_t* vc, float* out, int n_head,
                                int n_kv, int hd, int n_ctx, int n_past, int batch, float scale, int rope_type, int n_rot,
                                float theta) {
    auto rope_batch = rope_type == 1 ? cuda::rope_neox_batch : cuda::rope_normal_batch;
    rope_batch(q, batch * n_head, hd, n_rot, theta, n_past, n_head, nullptr);
    rope_batch(k, batch * n_kv, hd, n_rot, theta, n_past, n_kv, nullptr);
    cuda::kv_store_batch(kc, vc, k, v, n_kv, hd, n_ctx, n_past, batch);
    cuda::flash_attention(q, kc, vc, out, n_head, n_kv, hd, n_ctx, n_past, batch, scale);
}
void shim_decode_layer_fused(const float* q, const float* k, const float* v, uint16_t* kc, uint16_t* vc, float* out,
                             int n_head, int n_kv, int hd, int n_ctx, const int* d_pos, float scale, int rope_type,
                             int n_rot, float theta) {
    cuda::attention_decode_fused(q, k, v, kc, vc, out, n_head, n_kv, hd, n_ctx, d_pos, scale, rope_type, n_rot, theta, nullptr);
}
void shim_prefill_layer_fused(const float* q, const float* k, const float* v, uint16_t* kc, uint16_t* vc, float* out,
                              int n_head, int n_kv, int hd, int n_ctx, int n_past, int batch, float scale, int rope_type,
                              int n_rot, float theta) {
    cuda::attention_prefill_fused(q, k, v, kc, vc, out, n_head, n_kv, hd, n_ctx, n_past, batch, scale, rope_type, n_rot, theta, nullptr);
}
// Fused decode call of a layer with biases, q/k norm and the q8_1 output (src/model_gpu.cu:268-284 in one call).
void shim_decode_layer_fused_extras(const float* q, const float* k, const float* v, uint16_t* kc, uint16_t* vc, float* out,
                                    int n_head, int n_kv, int hd, int n_ctx, const int* d_pos, float scale, int rope_type,
                                    int n_rot, float theta, const float* bq, const float* bk, const float* bv,
                                    const float* q_norm, const float* k_norm, float eps, int8_t* q8, float* q8_scale) {
    cuda::AttnExtras x;
    x.bq = bq; x.bk = bk; x.bv = bv; x.q_norm = q_norm; x.k_norm = k_norm; x.rms_eps = eps; x.q8 = q8; x.q8_scale = q8_scale;
    cuda::attention_decode_fused(q, k, v, kc, vc, out, n_head, n_kv, hd, n_ctx, d_pos, scale, rope_type, n_rot, theta, nullptr, x);
}
// A decode sequence that must NOT fuse: the k that is stored is not the k that was rotated.
void shim_decode_layer_mismatched(float* q, float* k, const float* k_stored, const float* v, uint16_t* kc, uint16_t* vc,
                                  float* out, int n_head, int n_kv, int hd, int n_ctx, const int* d_pos, float scale,
                                  int rope_type, int n_rot, float theta) {
    auto rope_ind = rope_type == 1 ? cuda::rope_neox_ind : cuda::rope_normal_ind;
    rope_ind(q, n_head, hd, n_rot, theta, d_pos, nullptr);
    rope_ind(k, n_kv, hd, n_rot, theta, d_pos, nullptr);
    cuda::kv_store_ind(kc, vc, k_stored, v, n_kv, hd, n_ctx, d_pos);
    cuda::flash_attention_decode_ind(q, kc, vc, out, n_head, n_kv, hd, n_ctx, d_pos, scale);
}
void shim_fuse_call_sequence(int on) { cuda::attn_fuse_call_sequence(on != 0); }
void shim_flush() { cuda::attn_flush(); }
// rope(q), rope(k), kv_store of a decode step with no attention call behind them
void shim_decode_producers_only(float* q, float* k, const float* v, uint16_t* kc, uint16_t* vc, int n_head, int n_kv, int hd,
                                int n_ctx, const int* d_pos, int rope_type, int n_rot, float theta) {
    auto rope_ind = rope_type == 1 ? cuda::rope_neox_ind : cuda::rope_normal_ind;
    rope_ind(q, n_head, hd, n_rot, theta, d_pos, nullptr);
    rope_ind(k, n_kv, hd, n_rot, theta, d_pos, nullptr);
    cuda::kv_store_ind(kc, vc, k, v, n_kv, hd, n_ctx, d_pos);
}
void shim_kv_shift(uint16_t* kc, uint16_t* vc, int n_layer, int n_kv, int hd, int n_ctx, int n_keep, int shift) {
    cuda::kv_shift(kc, vc, n_layer, n_kv, hd, n_ctx, n_keep, shift);
}
}
