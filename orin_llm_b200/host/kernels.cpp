// Definitions of the reference-named wrappers on top of the C ABI.  Plain C++ (no CUDA headers):
// everything device-side lives behind include/orin_attn_b200.h.
#include "kernels.h"
#include "placement.h"

#include <stdio.h>
#include <stdlib.h>

#include "../../include/orin_attn_b200.h"

namespace llm::cuda {

namespace {

void* s_stream = nullptr;            // process-global stream, as in src/kernels.cu:1726
void* g_decode_ws = nullptr;         // scratch handed over by attn_scratch_assign
size_t g_decode_ws_bytes = 0;
void* g_prefill_ws = nullptr;
size_t g_prefill_ws_bytes = 0;
bool g_prefill_ws_owned = false;     // allocated here (on demand), not handed over by attn_scratch_assign

inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

bool g_ready = false;                // a device was initialised through this library

void check(int rc, const char* what);

// Hosts that never call init()/attn_scratch_assign() (the reference's model_gpu.cu linked as it is) still work: the
// first wrapper call initialises the current device; prefill scratch is allocated on demand (prefill is never
// captured in a graph); decode, which the reference captures in a graph (src/model_gpu.cu:295-316), never allocates:
// without an assigned block it runs on the library's built-in scratch block.
// OATTN_DECODE_OVERLAP=0|1|2 in the environment selects the decode launch ordering (oattn_set_decode_overlap).
void apply_environment() {
    const char* e = getenv("OATTN_DECODE_OVERLAP");
    if (e && e[0] >= '0' && e[0] <= '2' && e[1] == 0) check(oattn_set_decode_overlap(e[0] - '0'), "OATTN_DECODE_OVERLAP");
}

void ensure_ready() {
    if (g_ready) return;
    check(oattn_init(-1), "init (on first use)");
    apply_environment();
    g_ready = true;
}

void ensure_prefill_scratch(int n_head, int n_kv, int head_dim, int batch) {
    const size_t need = oattn_prefill_workspace_bytes(n_head, n_kv, head_dim, batch);
    if (g_prefill_ws && g_prefill_ws_bytes >= need) return;
    void* p = nullptr;
    check(oattn_scratch_alloc(need, &p), "prefill scratch");
    // a smaller block allocated here earlier is returned; one handed over by the host stays with its owner
    if (g_prefill_ws_owned) check(oattn_scratch_free(g_prefill_ws), "prefill scratch (release)");
    g_prefill_ws = p;
    g_prefill_ws_bytes = need;
    g_prefill_ws_owned = true;
}

// Decode scratch allocated at a point that is never under stream capture (a prefill call).
void alloc_decode_scratch_outside_capture(int n_head, int n_kv, int head_dim) {
    if (g_decode_ws) return;
    const size_t need = oattn_decode_workspace_bytes(n_head, n_kv, head_dim);
    void* p = nullptr;
    check(oattn_scratch_alloc(need, &p), "decode scratch");
    g_decode_ws = p;
    g_decode_ws_bytes = need;
}

// Scratch of a decode call that may be running under stream capture: the assigned block, else the library's built-in
// block.  Never allocates; a shape too large for the built-in block is a usage error with a clear message.
void decode_scratch(int n_head, int n_kv, int head_dim, void** ws, size_t* bytes) {
    if (g_decode_ws) { *ws = g_decode_ws; *bytes = g_decode_ws_bytes; return; }
    check(oattn_builtin_scratch(ws, bytes), "built-in decode scratch");
    const size_t need = oattn_decode_workspace_bytes(n_head, n_kv, head_dim);
    if (need > *bytes) {
        fprintf(stderr, "[cuda::attention_decode_fused] this shape needs %zu bytes of decode scratch, the built-in block holds %zu: "
                        "call attn_scratch_assign() once before the first decode call\n", need, *bytes);
        abort();
    }
}

void check(int rc, const char* what) {
    if (rc == OATTN_OK) return;
    fprintf(stderr, "[cuda::%s] %s%s%s\n", what, oattn_strerror(rc), rc == OATTN_ERR_CUDA ? ": " : "",
            rc == OATTN_ERR_CUDA ? oattn_last_cuda_error() : "");
    abort();
}

// ---- call-sequence fusion (opt-in) ------------------------------------------------------------------------------
// The reference issues rope(q), rope(k), kv_store, attention as four calls (src/model_gpu.cu:277-282, 379-384).  With
// fusion on, the first three are only recorded; when the attention call that follows is their consumer (same q, the k
// that was rotated is the k that was stored, same cache, same position), all four become the one fused launch.  Any
// other call first issues what is pending, in order, so that the wrappers keep their meaning call by call.  What
// changes for the host: q and k are no longer rotated in place (nothing in the reference reads them afterwards).
struct PendingRope {
    float* x; int rows, head_dim, rope_type, n_rot; float theta; int n_past, heads; const int* d_pos; const float* ff;
};
struct PendingStore {
    uint16_t* kc; uint16_t* vc; const float* k; const float* v; int heads, head_dim, n_ctx, pos_base, batch; const int* d_pos;
};
int g_fuse_sequence = -1;            // -1: not decided yet (environment OATTN_FUSE_CALL_SEQUENCE), 0 off, 1 on
PendingRope g_rope[2];
int g_n_rope = 0;
PendingStore g_store;
bool g_store_on = false;

bool fuse_sequence() {
    if (g_fuse_sequence < 0) {
        const char* e = getenv("OATTN_FUSE_CALL_SEQUENCE");
        g_fuse_sequence = (e && e[0] == '1') ? 1 : 0;
    }
    return g_fuse_sequence == 1;
}

void issue_rope(const PendingRope& r) {
    check(oattn_rope(r.x, r.rows, r.head_dim, r.rope_type, r.n_rot, r.theta, r.n_past, r.heads, r.d_pos, r.ff, s_stream), "rope");
}
void issue_store(const PendingStore& t) {
    check(oattn_kv_store(t.kc, t.vc, t.k, t.v, t.heads, t.head_dim, t.n_ctx, t.pos_base, t.batch, t.d_pos, s_stream), "kv_store");
}

// Issue whatever is recorded, in the order it was called.
void flush_pending() {
    for (int i = 0; i < g_n_rope; ++i) issue_rope(g_rope[i]);
    g_n_rope = 0;
    if (g_store_on) issue_store(g_store);
    g_store_on = false;
}

void rope_call(const PendingRope& r) {
    ensure_ready();
    if (!fuse_sequence()) { issue_rope(r); return; }
    if (g_store_on || g_n_rope == 2) flush_pending();
    g_rope[g_n_rope++] = r;
}
void store_call(const PendingStore& t) {
    ensure_ready();
    if (!fuse_sequence()) { issue_store(t); return; }
    if (g_store_on) flush_pending();
    g_store = t;
    g_store_on = true;
}

// Are the recorded calls exactly the producers of this attention call?
bool sequence_matches(const float* q, const uint16_t* kc, const uint16_t* vc, int n_head, int n_kv, int head_dim, int n_ctx,
                      int n_past, int batch, const int* d_pos) {
    if (g_n_rope != 2 || !g_store_on) return false;
    const PendingRope& a = g_rope[0];
    const PendingRope& b = g_rope[1];
    const PendingStore& t = g_store;
    return a.x == q && a.rows == batch * n_head && a.head_dim == head_dim && a.d_pos == d_pos && a.n_past == n_past &&
           (d_pos || a.heads == n_head) &&
           b.x == t.k && b.rows == batch * n_kv && b.head_dim == head_dim && b.d_pos == d_pos && b.n_past == n_past &&
           (d_pos || b.heads == n_kv) &&
           a.rope_type == b.rope_type && a.n_rot == b.n_rot && a.theta == b.theta && a.ff == b.ff &&
           t.kc == kc && t.vc == vc && t.heads == n_kv && t.head_dim == head_dim && t.n_ctx == n_ctx && t.d_pos == d_pos &&
           t.batch == batch && (d_pos || t.pos_base == n_past);
}

} // namespace

int init() { return init_device(0); }

int init_device(int device) {
    const int rc = oattn_init(device);
    if (rc != OATTN_OK) {
        fprintf(stderr, "[cuda::init] %s %s\n", oattn_strerror(rc), oattn_last_cuda_error());
        return -1;
    }
    apply_environment();
    g_ready = true;
    return 0;
}

void attn_flush() { flush_pending(); }
void set_stream(void* stream) { flush_pending(); s_stream = stream; }
void attn_set_stream(void* stream) { flush_pending(); s_stream = stream; }
void attn_fuse_call_sequence(bool on) { flush_pending(); g_fuse_sequence = on ? 1 : 0; }

size_t attn_scratch_size(int n_head, int n_kv, int head_dim, int max_batch) {
    return align256(oattn_decode_workspace_bytes(n_head, n_kv, head_dim)) +
           align256(oattn_prefill_workspace_bytes(n_head, n_kv, head_dim, max_batch));
}

void attn_scratch_assign(void* base, int n_head, int n_kv, int head_dim, int max_batch) {
    flush_pending();
    g_decode_ws = base;
    g_decode_ws_bytes = oattn_decode_workspace_bytes(n_head, n_kv, head_dim);
    if (g_prefill_ws_owned) check(oattn_scratch_free(g_prefill_ws), "prefill scratch (release)");
    g_prefill_ws_owned = false;
    g_prefill_ws = static_cast<uint8_t*>(base) + align256(g_decode_ws_bytes);
    g_prefill_ws_bytes = oattn_prefill_workspace_bytes(n_head, n_kv, head_dim, max_batch);
}

void rope_neox_batch(float* x, int rows, int head_dim, int n_rot, float theta, int n_past, int heads, const float* ff) {
    rope_call({x, rows, head_dim, OATTN_ROPE_NEOX, n_rot, theta, n_past, heads, nullptr, ff});
}
void rope_normal_batch(float* x, int rows, int head_dim, int n_rot, float theta, int n_past, int heads, const float* ff) {
    rope_call({x, rows, head_dim, OATTN_ROPE_NORMAL, n_rot, theta, n_past, heads, nullptr, ff});
}
void rope_neox_ind(float* x, int rows, int head_dim, int n_rot, float theta, const int* d_pos, const float* ff) {
    rope_call({x, rows, head_dim, OATTN_ROPE_NEOX, n_rot, theta, 0, 1, d_pos, ff});
}
void rope_normal_ind(float* x, int rows, int head_dim, int n_rot, float theta, const int* d_pos, const float* ff) {
    rope_call({x, rows, head_dim, OATTN_ROPE_NORMAL, n_rot, theta, 0, 1, d_pos, ff});
}

void kv_store_batch(uint16_t* kc, uint16_t* vc, const float* k, const float* v, int heads, int head_dim, int n_ctx,
                    int pos_base, int batch) {
    store_call({kc, vc, k, v, heads, head_dim, n_ctx, pos_base, batch, nullptr});
}
void kv_store_ind(uint16_t* kc, uint16_t* vc, const float* k, const float* v, int heads, int head_dim, int n_ctx,
                  const int* d_pos) {
    store_call({kc, vc, k, v, heads, head_dim, n_ctx, 0, 1, d_pos});
}
void kv_shift(uint16_t* kc, uint16_t* vc, int n_layer, int n_kv, int head_dim, int n_ctx, int n_keep, int shift) {
    ensure_ready();
    flush_pending();
    check(oattn_kv_shift(kc, vc, n_layer, n_kv, head_dim, n_ctx, n_keep, shift, s_stream), "kv_shift");
}

void flash_attention(const float* q, const uint16_t* kc, const uint16_t* vc, float* out, int n_head, int n_kv,
                     int head_dim, int n_ctx, int n_past, int batch, float scale) {
    ensure_ready();
    ensure_prefill_scratch(n_head, n_kv, head_dim, batch);
    if (fuse_sequence()) {
        alloc_decode_scratch_outside_capture(n_head, n_kv, head_dim);       // prefill is never captured: a safe place
        if (sequence_matches(q, kc, vc, n_head, n_kv, head_dim, n_ctx, n_past, batch, nullptr)) {
            const oattn_rope_params rp = {g_rope[0].rope_type, g_rope[0].n_rot, g_rope[0].theta, g_rope[0].ff};
            const PendingStore t = g_store;
            g_n_rope = 0;
            g_store_on = false;
            check(oattn_prefill(q, t.k, t.v, t.kc, t.vc, out, n_head, n_kv, head_dim, n_ctx, n_past, batch, scale, OATTN_FUSE_ALL,
                                &rp, g_prefill_ws, g_prefill_ws_bytes, s_stream), "flash_attention (fused sequence)");
            return;
        }
        flush_pending();
    }
    check(oattn_prefill(q, nullptr, nullptr, const_cast<uint16_t*>(kc), const_cast<uint16_t*>(vc), out, n_head, n_kv,
                        head_dim, n_ctx, n_past, batch, scale, OATTN_FUSE_NONE, nullptr, g_prefill_ws, g_prefill_ws_bytes,
                        s_stream), "flash_attention");
}
void flash_attention_decode_ind(const float* q, const uint16_t* kc, const uint16_t* vc, float* out, int n_head, int n_kv,
                                int head_dim, int n_ctx, const int* d_pos, float scale) {
    ensure_ready();
    if (fuse_sequence()) {
        if (g_decode_ws && sequence_matches(q, kc, vc, n_head, n_kv, head_dim, n_ctx, 0, 1, d_pos)) {
            const oattn_rope_params rp = {g_rope[0].rope_type, g_rope[0].n_rot, g_rope[0].theta, g_rope[0].ff};
            const PendingStore t = g_store;
            g_n_rope = 0;
            g_store_on = false;
            check(oattn_decode(q, t.k, t.v, t.kc, t.vc, out, n_head, n_kv, head_dim, n_ctx, d_pos, scale, OATTN_FUSE_ALL, &rp,
                               g_decode_ws, g_decode_ws_bytes, s_stream), "flash_attention_decode_ind (fused sequence)");
            return;
        }
        flush_pending();
    }
    if (!g_decode_ws) {      // no scratch was handed over: the built-in block (graph-capturable, no allocation)
        check(oattn_decode_noalloc(q, kc, vc, out, n_head, n_kv, head_dim, n_ctx, d_pos, scale, s_stream),
              "flash_attention_decode_ind");
        return;
    }
    check(oattn_decode(q, nullptr, nullptr, const_cast<uint16_t*>(kc), const_cast<uint16_t*>(vc), out, n_head, n_kv,
                       head_dim, n_ctx, d_pos, scale, OATTN_FUSE_NONE, nullptr, g_decode_ws, g_decode_ws_bytes, s_stream),
          "flash_attention_decode_ind");
}

void attention_decode_fused(const float* q, const float* k, const float* v, uint16_t* kc, uint16_t* vc, float* out,
                            int n_head, int n_kv, int head_dim, int n_ctx, const int* d_pos, float scale, int rope_type,
                            int n_rot, float theta, const float* freq_factors) {
    const oattn_rope_params rp = {rope_type, n_rot, theta, freq_factors};
    ensure_ready();
    flush_pending();
    void* ws = nullptr;
    size_t ws_bytes = 0;
    decode_scratch(n_head, n_kv, head_dim, &ws, &ws_bytes);
    check(oattn_decode(q, k, v, kc, vc, out, n_head, n_kv, head_dim, n_ctx, d_pos, scale, OATTN_FUSE_ALL, &rp, ws, ws_bytes,
                       s_stream), "attention_decode_fused");
}
void attention_prefill_fused(const float* q, const float* k, const float* v, uint16_t* kc, uint16_t* vc, float* out,
                             int n_head, int n_kv, int head_dim, int n_ctx, int n_past, int batch, float scale,
                             int rope_type, int n_rot, float theta, const float* freq_factors) {
    const oattn_rope_params rp = {rope_type, n_rot, theta, freq_factors};
    ensure_ready();
    flush_pending();
    ensure_prefill_scratch(n_head, n_kv, head_dim, batch);
    check(oattn_prefill(q, k, v, kc, vc, out, n_head, n_kv, head_dim, n_ctx, n_past, batch, scale, OATTN_FUSE_ALL, &rp,
                        g_prefill_ws, g_prefill_ws_bytes, s_stream), "attention_prefill_fused");
}

static oattn_ext to_ext(const AttnExtras& x) {
    oattn_ext e;
    e.bias_q = x.bq; e.bias_k = x.bk; e.bias_v = x.bv;
    e.norm_q = x.q_norm; e.norm_k = x.k_norm; e.norm_eps = x.rms_eps;
    e.out_qs = x.q8; e.out_scales = x.q8_scale;
    e.out_mmq = x.q8_mmq; e.out_mmq_ds4 = x.q8_mmq_ds4 ? 1 : 0;
    return e;
}
void attention_decode_fused(const float* q, const float* k, const float* v, uint16_t* kc, uint16_t* vc, float* out,
                            int n_head, int n_kv, int head_dim, int n_ctx, const int* d_pos, float scale, int rope_type,
                            int n_rot, float theta, const float* freq_factors, const AttnExtras& extras) {
    const oattn_rope_params rp = {rope_type, n_rot, theta, freq_factors};
    const oattn_ext ext = to_ext(extras);
    ensure_ready();
    flush_pending();
    void* ws = nullptr;
    size_t ws_bytes = 0;
    decode_scratch(n_head, n_kv, head_dim, &ws, &ws_bytes);
    check(oattn_decode_ex(q, k, v, kc, vc, out, n_head, n_kv, head_dim, n_ctx, d_pos, scale, OATTN_FUSE_ALL, &rp, &ext,
                          ws, ws_bytes, s_stream), "attention_decode_fused");
}
void attention_prefill_fused(const float* q, const float* k, const float* v, uint16_t* kc, uint16_t* vc, float* out,
                             int n_head, int n_kv, int head_dim, int n_ctx, int n_past, int batch, float scale,
                             int rope_type, int n_rot, float theta, const float* freq_factors, const AttnExtras& extras) {
    const oattn_rope_params rp = {rope_type, n_rot, theta, freq_factors};
    const oattn_ext ext = to_ext(extras);
    ensure_ready();
    flush_pending();
    ensure_prefill_scratch(n_head, n_kv, head_dim, batch);
    check(oattn_prefill_ex(q, k, v, kc, vc, out, n_head, n_kv, head_dim, n_ctx, n_past, batch, scale, OATTN_FUSE_ALL, &rp, &ext,
                           g_prefill_ws, g_prefill_ws_bytes, s_stream), "attention_prefill_fused");
}

// ---- memory placement (placement.h) ------------------------------------------------------------------------------
namespace {
const unsigned char* g_w_host = nullptr;
unsigned char* g_w_dev = nullptr;
size_t g_w_bytes = 0;
}

void place_weights(const void* host_base, size_t bytes) {
    ensure_ready();
    if (g_w_dev) release_weights();
    void* d = nullptr;
    check(oattn_weights_place(host_base, bytes, &d), "place_weights");
    g_w_host = static_cast<const unsigned char*>(host_base);
    g_w_dev = static_cast<unsigned char*>(d);
    g_w_bytes = bytes;
}

void* placed_weight(const void* host_ptr) {
    const unsigned char* h = static_cast<const unsigned char*>(host_ptr);
    if (!g_w_dev || h < g_w_host || h >= g_w_host + g_w_bytes) {
        fprintf(stderr, "[cuda::placed_weight] %p lies outside the placed range\n", host_ptr);
        abort();
    }
    return g_w_dev + (h - g_w_host);
}

void release_weights() {
    if (g_w_dev) check(oattn_scratch_free(g_w_dev), "release_weights");
    g_w_dev = nullptr;
    g_w_host = nullptr;
    g_w_bytes = 0;
}

void logits_alloc(size_t bytes, float** d_logits, float** h_logits) {
    ensure_ready();
    void* d = nullptr;
    void* h = nullptr;
    check(oattn_logits_alloc(bytes, &d, &h), "logits_alloc");
    *d_logits = static_cast<float*>(d);
    *h_logits = static_cast<float*>(h);
}

void logits_fetch(float* h_logits, const float* d_logits, size_t bytes) {
    check(oattn_copy_to_host_async(h_logits, d_logits, bytes, s_stream), "logits_fetch");
}

void logits_free(float* d_logits, float* h_logits) { check(oattn_logits_free(d_logits, h_logits), "logits_free"); }

void kv_cache_clear(void* base, size_t bytes) {
    ensure_ready();
    check(oattn_device_clear(base, bytes), "kv_cache_clear");
}

} // namespace llm::cuda
