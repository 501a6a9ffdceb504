// Reference-side harness  --  TEST INFRASTRUCTURE ONLY, never part of the product library.
//
// Compiles the reference's own CPU backend (src/model_cpu.cpp) from where it lies, by
// textual inclusion, so that its file-local helpers (dot, softmax, rope_neox, rope_normal,
// rms_norm) and its unmodified Model::impl::forward are reachable from C.  Built only when
// the reference tree is present (see oracle/Makefile, target `ref`); output goes to
// oracle/_ref/libref_attn.so.  No reference source is copied into this repository.
//
// Exports:
//   ref_rope            the reference's rope_neox / rope_normal          (model_cpu.cpp:179-203)
//   ref_attend          scores/softmax/weighted sum with the reference's own dot() and
//                       softmax(); the loop nest around them follows model_cpu.cpp:281-295
//   ref_attend_mt       the same, one std::thread per query head (timed CPU baseline)
//   ref_forward_probe   runs the reference's real forward() on a one-layer fp32 model whose
//                       Wq/Wk/Wv are exact selection matrices, and returns the q/k/v it fed
//                       to attention together with the attention output it produced -- this
//                       is what pins oracle/attn_oracle.c to the reference bit-for-bit.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <thread>
#include <vector>

// The probe reads Model::impl's buffers (q_, k_, v_, attn_, k_cache_, v_cache_).
#define private public
#include "model_cpu.cpp"
#undef private

namespace {

struct ProbeModel {
    std::vector<float> embd, eye_q, sel_k, sel_v, wo, gate, up, down, norm1, norm2, onorm;
    llm::Tensor t_embd, t_q, t_k, t_v, t_o, t_gate, t_up, t_down, t_n1, t_n2, t_on;
};

llm::Tensor make_f32(std::vector<float>& buf, int ne0, int ne1) {
    llm::Tensor t;
    t.type = llm::DType::F32;
    t.ne0 = ne0;
    t.ne1 = ne1;
    t.data = (const uint8_t*)buf.data();
    return t;
}

} // namespace

// Runs the reference's forward() on the one-layer probe model; optional q/k/v biases and per-head q/k norm weights
// are attached to the layer the way the loader would (Layer::bq/bk/bv/wq_norm/wk_norm, model_cpu.cpp:258-274).
static int probe_impl(const float* x_in, int n_tok, int n_head, int n_kv, int d, int n_ctx,
                      int rope_type, int n_rot, float theta, const float* freq_factors,
                      const float* bias_q, const float* bias_k, const float* bias_v,
                      const float* norm_q, const float* norm_k, float eps,
                      float* q_pre, float* k_pre, float* v_pre, float* q_rot, float* k_rot, float* attn);

extern "C" {

// The reference's own weight dequantisation (src/model_cpu.cpp:142-158): `type` is the ggml type number.  Used to check
// the synthetic GGUF writer's K-quant blocks.
void ref_dequantize_row(int type, const void* x, float* y, long long k) {
    llm::dequantize_row((llm::DType)type, x, y, (int64_t)k);
}

void ref_rope(float* x, int rope_type, int n_rot, float theta, int pos, const float* freq_factors) {
    if (rope_type == 1) llm::rope_neox(x, n_rot, theta, pos, freq_factors);
    else                llm::rope_normal(x, n_rot, theta, pos, freq_factors);
}

void ref_attend_head(const float* q, const float* kcache, const float* vcache, float* out,
                     int h, int n_head, int n_kv, int d, int n_ctx, int npos, float scale, float* score) {
    const int kv = h * n_kv / n_head;
    const float* qh = q + (size_t)h * d;
    const float* kb = kcache + (size_t)kv * n_ctx * d;
    const float* vb = vcache + (size_t)kv * n_ctx * d;
    for (int j = 0; j < npos; ++j) score[j] = scale * llm::dot(qh, kb + (size_t)j * d, d);
    llm::softmax(score, npos);
    float* ah = out + (size_t)h * d;
    for (int jd = 0; jd < d; ++jd) {
        float s = 0.0f;
        for (int j = 0; j < npos; ++j) s += score[j] * vb[(size_t)j * d + jd];
        ah[jd] = s;
    }
}

void ref_attend(const float* q, const float* kcache, const float* vcache, float* out,
                int n_head, int n_kv, int d, int n_ctx, int npos, float scale, float* score) {
    for (int h = 0; h < n_head; ++h)
        ref_attend_head(q, kcache, vcache, out, h, n_head, n_kv, d, n_ctx, npos, scale, score);
}

// One thread per query head (the reference itself is single-threaded; heads are independent,
// so this is the reference's arithmetic on every core it can use).  Returns threads used.
int ref_attend_mt(const float* q, const float* kcache, const float* vcache, float* out,
                  int n_head, int n_kv, int d, int n_ctx, int npos, float scale, int max_threads) {
    int nt = std::min(n_head, std::max(1, max_threads));
    std::vector<std::thread> th;
    for (int t = 0; t < nt; ++t) {
        th.emplace_back([=]() {
            std::vector<float> score((size_t)npos);
            for (int h = t; h < n_head; h += nt)
                ref_attend_head(q, kcache, vcache, out, h, n_head, n_kv, d, n_ctx, npos, scale, score.data());
        });
    }
    for (auto& x : th) x.join();
    return nt;
}

// Causal chunk (forward_batch semantics, model_cpu.cpp:314-319: token b attends [0, n_past+b]),
// threads over (token, head) pairs.  K/V must already be in the fp32 cache.
int ref_attend_chunk_mt(const float* q, const float* kcache, const float* vcache, float* out,
                        int n_head, int n_kv, int d, int n_ctx, int n_past, int batch, float scale,
                        int max_threads) {
    int nt = std::max(1, max_threads);
    std::vector<std::thread> th;
    for (int t = 0; t < nt; ++t) {
        th.emplace_back([=]() {
            std::vector<float> score((size_t)n_past + batch);
            for (int item = t; item < batch * n_head; item += nt) {
                const int b = item / n_head, h = item % n_head;
                ref_attend_head(q + (size_t)b * n_head * d, kcache, vcache, out + (size_t)b * n_head * d,
                                h, n_head, n_kv, d, n_ctx, n_past + b + 1, scale, score.data());
            }
        });
    }
    for (auto& x : th) x.join();
    return nt;
}

// Runs the reference's unmodified forward() for `n_tok` tokens (positions 0..n_tok-1) on a
// one-layer fp32 model.  n_embd = n_head*d.  Token t's embedding row is x_in[t][n_embd].
// attn_norm = ones, so the normalised activation xn = rms_norm(x) feeds q = xn (identity Wq),
// k[i] = xn[(7*i+3) % n_embd], v[i] = -0.5 * xn[(5*i+1) % n_embd] (one non-zero per row: exact).
// Outputs per token: q_pre/k_pre/v_pre (before RoPE, i.e. what attention receives),
// q_rot/k_rot (after the reference's RoPE), attn (attention output, [n_head*d]).
int ref_forward_probe(const float* x_in, int n_tok, int n_head, int n_kv, int d, int n_ctx,
                      int rope_type, int n_rot, float theta, const float* freq_factors,
                      float* q_pre, float* k_pre, float* v_pre, float* q_rot, float* k_rot, float* attn) {
    return probe_impl(x_in, n_tok, n_head, n_kv, d, n_ctx, rope_type, n_rot, theta, freq_factors,
                      nullptr, nullptr, nullptr, nullptr, nullptr, 1e-6f, q_pre, k_pre, v_pre, q_rot, k_rot, attn);
}

// As ref_forward_probe, with q/k/v biases and per-head q/k RMSNorm weights on the layer.  q_pre/k_pre/v_pre are the
// projections BEFORE bias and norm (what a fused prologue receives); q_rot/k_rot what forward() fed to attention.
int ref_forward_probe_pre(const float* x_in, int n_tok, int n_head, int n_kv, int d, int n_ctx,
                          int rope_type, int n_rot, float theta, const float* freq_factors,
                          const float* bias_q, const float* bias_k, const float* bias_v,
                          const float* norm_q, const float* norm_k, float eps,
                          float* q_pre, float* k_pre, float* v_pre, float* q_rot, float* k_rot, float* attn) {
    return probe_impl(x_in, n_tok, n_head, n_kv, d, n_ctx, rope_type, n_rot, theta, freq_factors,
                      bias_q, bias_k, bias_v, norm_q, norm_k, eps, q_pre, k_pre, v_pre, q_rot, k_rot, attn);
}

// The reference's kv_shift on an fp32 cache (model_cpu.cpp:321-340), via its own member function.
void ref_kv_shift(float* kcache, float* vcache, int n_layer, int n_kv, int d, int n_ctx, int n_keep, int shift) {
    llm::HParams hp;
    hp.n_layer = n_layer; hp.n_head_kv = n_kv; hp.head_dim = d; hp.n_ctx = n_ctx;
    llm::Model::impl m;
    const size_t n = (size_t)n_layer * n_kv * n_ctx * d;
    m.k_cache_.assign(kcache, kcache + n);
    m.v_cache_.assign(vcache, vcache + n);
    m.kv_shift(hp, n_keep, shift);
    memcpy(kcache, m.k_cache_.data(), n * sizeof(float));
    memcpy(vcache, m.v_cache_.data(), n * sizeof(float));
}

} // extern "C"

static int probe_impl(const float* x_in, int n_tok, int n_head, int n_kv, int d, int n_ctx,
                      int rope_type, int n_rot, float theta, const float* freq_factors,
                      const float* bias_q, const float* bias_k, const float* bias_v,
                      const float* norm_q, const float* norm_k, float eps,
                      float* q_pre, float* k_pre, float* v_pre, float* q_rot, float* k_rot, float* attn) {
    const int ne = n_head * d, nk = n_kv * d;
    ProbeModel pm;
    pm.embd.assign(x_in, x_in + (size_t)n_tok * ne);
    pm.eye_q.assign((size_t)ne * ne, 0.0f);
    for (int i = 0; i < ne; ++i) pm.eye_q[(size_t)i * ne + i] = 1.0f;
    pm.sel_k.assign((size_t)nk * ne, 0.0f);
    pm.sel_v.assign((size_t)nk * ne, 0.0f);
    for (int i = 0; i < nk; ++i) {
        pm.sel_k[(size_t)i * ne + (7 * i + 3) % ne] = 1.0f;
        pm.sel_v[(size_t)i * ne + (5 * i + 1) % ne] = -0.5f;
    }
    pm.wo.assign((size_t)ne * ne, 0.0f);
    pm.gate.assign(ne, 0.0f); pm.up.assign(ne, 0.0f); pm.down.assign(ne, 0.0f);
    pm.norm1.assign(ne, 1.0f); pm.norm2.assign(ne, 1.0f); pm.onorm.assign(ne, 1.0f);

    pm.t_embd = make_f32(pm.embd, ne, n_tok);
    pm.t_q = make_f32(pm.eye_q, ne, ne);
    pm.t_k = make_f32(pm.sel_k, ne, nk);
    pm.t_v = make_f32(pm.sel_v, ne, nk);
    pm.t_o = make_f32(pm.wo, ne, ne);
    pm.t_gate = make_f32(pm.gate, ne, 1);
    pm.t_up = make_f32(pm.up, ne, 1);
    pm.t_down = make_f32(pm.down, 1, ne);
    pm.t_n1 = make_f32(pm.norm1, ne, 1);
    pm.t_n2 = make_f32(pm.norm2, ne, 1);
    pm.t_on = make_f32(pm.onorm, ne, 1);

    llm::HParams hp;
    hp.arch = "probe";
    hp.n_vocab = n_tok; hp.n_embd = ne; hp.n_layer = 1; hp.n_head = n_head; hp.n_head_kv = n_kv;
    hp.head_dim = d; hp.n_ff = 1; hp.n_rot = n_rot; hp.n_ctx = n_ctx;
    hp.rms_eps = eps; hp.rope_theta = theta; hp.rope_type = rope_type;
    hp.rope_freq_factors = freq_factors;

    llm::Model::impl m;
    m.w_.token_embd = &pm.t_embd;
    m.w_.output = &pm.t_embd;
    m.w_.output_norm = &pm.t_on;
    m.w_.layers.assign(1, llm::Layer{});
    llm::Layer& L = m.w_.layers[0];
    L.wq = &pm.t_q; L.wk = &pm.t_k; L.wv = &pm.t_v; L.wo = &pm.t_o;
    L.ffn_gate = &pm.t_gate; L.ffn_up = &pm.t_up; L.ffn_down = &pm.t_down;
    L.attn_norm = &pm.t_n1; L.ffn_norm = &pm.t_n2;
    std::vector<float> bq, bk, bv, nq, nkw;
    llm::Tensor t_bq, t_bk, t_bv, t_nq, t_nk;
    if (bias_q) { bq.assign(bias_q, bias_q + ne); t_bq = make_f32(bq, ne, 1); L.bq = &t_bq; }
    if (bias_k) { bk.assign(bias_k, bias_k + nk); t_bk = make_f32(bk, nk, 1); L.bk = &t_bk; }
    if (bias_v) { bv.assign(bias_v, bias_v + nk); t_bv = make_f32(bv, nk, 1); L.bv = &t_bv; }
    if (norm_q) { nq.assign(norm_q, norm_q + d); t_nq = make_f32(nq, d, 1); L.wq_norm = &t_nq; }
    if (norm_k) { nkw.assign(norm_k, norm_k + d); t_nk = make_f32(nkw, d, 1); L.wk_norm = &t_nk; }
    m.init_buffers(hp);

    std::vector<float> xn(ne);
    for (int t = 0; t < n_tok; ++t) {
        // what the reference will feed to attention, recomputed with its own helpers
        llm::rms_norm(x_in + (size_t)t * ne, pm.norm1.data(), ne, hp.rms_eps, xn.data());
        for (int i = 0; i < ne; ++i) q_pre[(size_t)t * ne + i] = llm::dot(pm.eye_q.data() + (size_t)i * ne, xn.data(), ne);
        for (int i = 0; i < nk; ++i) {
            k_pre[(size_t)t * nk + i] = llm::dot(pm.sel_k.data() + (size_t)i * ne, xn.data(), ne);
            v_pre[(size_t)t * nk + i] = llm::dot(pm.sel_v.data() + (size_t)i * ne, xn.data(), ne);
        }
        m.forward(hp, t, t);   // the reference's own forward, untouched
        memcpy(q_rot + (size_t)t * ne, m.q_.data(), ne * sizeof(float));
        memcpy(k_rot + (size_t)t * nk, m.k_.data(), nk * sizeof(float));
        memcpy(attn + (size_t)t * ne, m.attn_.data(), ne * sizeof(float));
        // v is stored untouched in the cache; check the probe's own claim about it
        for (int h = 0; h < n_kv; ++h)
            for (int i = 0; i < d; ++i)
                if (m.v_cache_[((size_t)h * n_ctx + t) * d + i] !=
                    v_pre[(size_t)t * nk + h * d + i] + (bias_v ? bias_v[h * d + i] : 0.0f)) return -1;
    }
    return 0;
}
