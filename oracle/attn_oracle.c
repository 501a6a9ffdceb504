/*
 * CPU oracle for the attention path of Heng-W/orin_llm  --  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement of the reference's scalar fp32 attention
 * (src/model_cpu.cpp, the USE_CPU_ONLY backend).  It exists so that tests, the
 * smoke check and the timed CPU baseline have something to compare the CUDA
 * kernels with.  It is never linked into, imported by, or called from the product
 * library: the product has no CPU fallback.
 *
 * Parity pin: every function here is checked bit-for-bit against the reference's
 * own code compiled from its own sources (oracle/ref_harness.cpp, which runs the
 * reference's unmodified Model::impl::forward on an in-memory one-layer model),
 * and against the committed fixtures under tests/golden/ that were produced by
 * that same reference build.  The reference ships no golden vectors of its own.
 *
 * Arithmetic is fp32 throughout, evaluated in the same order as the reference so
 * that results agree bit-for-bit when both are built with the reference's flags
 * (-O3, no -ffast-math).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

/* src/model_cpu.cpp:32-36  dot(): sequential fp32 accumulation. */
static float oracle_dot(const float *a, const float *b, int n) {
    float s = 0.0f;
    for (int i = 0; i < n; ++i) s += a[i] * b[i];
    return s;
}

/* src/model_cpu.cpp:20-30  softmax(): max, exp(x-m) summed in index order, then
 * multiplication by the reciprocal of the sum. */
void oracle_softmax(float *x, int n) {
    float m = x[0];
    for (int i = 1; i < n; ++i) m = (m < x[i]) ? x[i] : m;
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) {
        x[i] = expf(x[i] - m);
        sum += x[i];
    }
    const float inv = 1.0f / sum;
    for (int i = 0; i < n; ++i) x[i] *= inv;
}

/* src/model_cpu.cpp:179-190  rope_neox(): pair (i, i + n_rot/2),
 * freq = theta^(-2i/n_rot) [/ freq_factors[i]], angle = pos * freq, all fp32. */
void oracle_rope_neox(float *x, int n_rot, float theta, int pos, const float *freq_factors) {
    const int half = n_rot / 2;
    for (int i = 0; i < half; ++i) {
        float freq = powf(theta, -2.0f * i / n_rot);
        if (freq_factors) freq /= freq_factors[i];
        const float ang = (float)pos * freq;
        const float c = cosf(ang), s = sinf(ang);
        const float x0 = x[i], x1 = x[i + half];
        x[i] = x0 * c - x1 * s;
        x[i + half] = x0 * s + x1 * c;
    }
}

/* src/model_cpu.cpp:193-203  rope_normal(): pair (i, i+1) for even i,
 * freq = theta^(-i/n_rot) [/ freq_factors[i/2]]. */
void oracle_rope_normal(float *x, int n_rot, float theta, int pos, const float *freq_factors) {
    for (int i = 0; i < n_rot; i += 2) {
        float freq = powf(theta, -1.0f * i / n_rot);
        if (freq_factors) freq /= freq_factors[i / 2];
        const float ang = (float)pos * freq;
        const float c = cosf(ang), s = sinf(ang);
        const float x0 = x[i], x1 = x[i + 1];
        x[i] = x0 * c - x1 * s;
        x[i + 1] = x0 * s + x1 * c;
    }
}

/* rope_type follows HParams::rope_type (src/model.h:27-28): 0 = normal, 1 = neox. */
void oracle_rope(float *x, int rope_type, int n_rot, float theta, int pos, const float *freq_factors) {
    if (rope_type == 1) oracle_rope_neox(x, n_rot, theta, pos, freq_factors);
    else                oracle_rope_normal(x, n_rot, theta, pos, freq_factors);
}

/* src/model_cpu.cpp:276-279  append one token's K and V rows (fp32) at position pos.
 * Cache layout per layer: [n_kv][n_ctx][d]. */
void oracle_kv_append(float *kcache, float *vcache, const float *k, const float *v,
                      int n_kv, int d, int n_ctx, int pos) {
    for (int h = 0; h < n_kv; ++h) {
        memcpy(kcache + ((size_t)h * n_ctx + pos) * d, k + (size_t)h * d, (size_t)d * sizeof(float));
        memcpy(vcache + ((size_t)h * n_ctx + pos) * d, v + (size_t)h * d, (size_t)d * sizeof(float));
    }
}

/* src/model_cpu.cpp:281-295  one query token over positions [0, npos):
 * kv head = h*n_kv/n_head; scores = scale*dot(q,k_j); softmax; out[jd] = sum_j p_j*v_j[jd]
 * accumulated in j order.  score must hold npos floats. */
void oracle_attend(const float *q, const float *kcache, const float *vcache, float *out,
                   int n_head, int n_kv, int d, int n_ctx, int npos, float scale, float *score) {
    for (int h = 0; h < n_head; ++h) {
        const int kv = h * n_kv / n_head;
        const float *qh = q + (size_t)h * d;
        const float *kb = kcache + (size_t)kv * n_ctx * d;
        const float *vb = vcache + (size_t)kv * n_ctx * d;
        for (int j = 0; j < npos; ++j) score[j] = scale * oracle_dot(qh, kb + (size_t)j * d, d);
        oracle_softmax(score, npos);
        float *ah = out + (size_t)h * d;
        for (int jd = 0; jd < d; ++jd) {
            float s = 0.0f;
            for (int j = 0; j < npos; ++j) s += score[j] * vb[(size_t)j * d + jd];
            ah[jd] = s;
        }
    }
}

/* One head only (used by the threaded timing harness; same arithmetic as oracle_attend). */
void oracle_attend_head(const float *q, const float *kcache, const float *vcache, float *out,
                        int h, int n_head, int n_kv, int d, int n_ctx, int npos, float scale,
                        float *score) {
    const int kv = h * n_kv / n_head;
    const float *qh = q + (size_t)h * d;
    const float *kb = kcache + (size_t)kv * n_ctx * d;
    const float *vb = vcache + (size_t)kv * n_ctx * d;
    for (int j = 0; j < npos; ++j) score[j] = scale * oracle_dot(qh, kb + (size_t)j * d, d);
    oracle_softmax(score, npos);
    float *ah = out + (size_t)h * d;
    for (int jd = 0; jd < d; ++jd) {
        float s = 0.0f;
        for (int j = 0; j < npos; ++j) s += score[j] * vb[(size_t)j * d + jd];
        ah[jd] = s;
    }
}

/* src/model_cpu.cpp:264-295  the attention step for ONE token at position n_past:
 * RoPE on every q head and k head (in place), append k,v to the cache, attend over
 * [0, n_past].  q [n_head*d], k,v [n_kv*d] are modified/consumed exactly as the
 * reference does (q and k come back rotated). */
void oracle_attn_step(float *q, float *k, const float *v, float *kcache, float *vcache, float *out,
                      int n_head, int n_kv, int d, int n_ctx, int n_past, float scale,
                      int rope_type, int n_rot, float theta, const float *freq_factors,
                      float *score) {
    for (int h = 0; h < n_head; ++h) oracle_rope(q + (size_t)h * d, rope_type, n_rot, theta, n_past, freq_factors);
    for (int h = 0; h < n_kv; ++h)   oracle_rope(k + (size_t)h * d, rope_type, n_rot, theta, n_past, freq_factors);
    oracle_kv_append(kcache, vcache, k, v, n_kv, d, n_ctx, n_past);
    oracle_attend(q, kcache, vcache, out, n_head, n_kv, d, n_ctx, n_past + 1, scale, score);
}

/* src/model_cpu.cpp:314-319  forward_batch is a token loop: token b sits at n_past+b.
 * q [batch][n_head*d], k,v [batch][n_kv*d], out [batch][n_head*d].
 * apply_rope=0 skips the rotation (inputs already rotated). */
void oracle_attn_batch(float *q, float *k, const float *v, float *kcache, float *vcache, float *out,
                       int n_head, int n_kv, int d, int n_ctx, int n_past, int batch, float scale,
                       int apply_rope, int rope_type, int n_rot, float theta,
                       const float *freq_factors, float *score) {
    for (int b = 0; b < batch; ++b) {
        float *qb = q + (size_t)b * n_head * d;
        float *kb = k + (size_t)b * n_kv * d;
        const float *vb = v + (size_t)b * n_kv * d;
        float *ob = out + (size_t)b * n_head * d;
        if (apply_rope) {
            oracle_attn_step(qb, kb, vb, kcache, vcache, ob, n_head, n_kv, d, n_ctx, n_past + b, scale,
                             rope_type, n_rot, theta, freq_factors, score);
        } else {
            oracle_kv_append(kcache, vcache, kb, vb, n_kv, d, n_ctx, n_past + b);
            oracle_attend(qb, kcache, vcache, ob, n_head, n_kv, d, n_ctx, n_past + b + 1, scale, score);
        }
    }
}

/* src/model_cpu.cpp:321-340  kv_shift for one layer: drop [n_keep, n_keep+shift), slide
 * the remainder left, zero the last `shift` rows.  Element type is generic (elem bytes)
 * so the same routine checks the fp16 device cache. */
void oracle_kv_shift(void *kcache, void *vcache, int n_layer, int n_kv, int d, int n_ctx,
                     int n_keep, int shift, int elem) {
    const size_t row = (size_t)d * elem;
    const size_t per_layer = (size_t)n_kv * n_ctx * row;
    for (int l = 0; l < n_layer; ++l) {
        for (int h = 0; h < n_kv; ++h) {
            uint8_t *kh = (uint8_t *)kcache + l * per_layer + (size_t)h * n_ctx * row;
            uint8_t *vh = (uint8_t *)vcache + l * per_layer + (size_t)h * n_ctx * row;
            memmove(kh + n_keep * row, kh + (size_t)(n_keep + shift) * row, (size_t)(n_ctx - n_keep - shift) * row);
            memmove(vh + n_keep * row, vh + (size_t)(n_keep + shift) * row, (size_t)(n_ctx - n_keep - shift) * row);
            memset(kh + (size_t)(n_ctx - shift) * row, 0, (size_t)shift * row);
            memset(vh + (size_t)(n_ctx - shift) * row, 0, (size_t)shift * row);
        }
    }
}

/* src/model_cpu.cpp:13-18  rms_norm(): sum of squares in double, r = 1/sqrt(ss/n + eps) in double,
 * y[i] = (float)(x[i] * r * w[i]) with the product formed in double, left to right.  y may alias x. */
void oracle_rms_norm(const float *x, const float *w, int n, float eps, float *y) {
    double ss = 0.0;
    for (int i = 0; i < n; ++i) ss += (double)x[i] * x[i];
    double r = 1.0 / sqrt(ss / n + eps);
    for (int i = 0; i < n; ++i) y[i] = (float)(x[i] * r * w[i]);
}

/* src/model_cpu.cpp:258-274  what one token's q, k, v go through between the projections and RoPE:
 * bias add on all of q, k, v (:258-260), then the per-head RMSNorm of every q head (:266) and every k head
 * (:271) with a [d] weight.  In place; any pointer of the last five may be NULL (step absent). */
void oracle_pre_attention(float *q, float *k, float *v, int n_head, int n_kv, int d,
                          const float *bias_q, const float *bias_k, const float *bias_v,
                          const float *norm_q, const float *norm_k, float eps) {
    if (bias_q) for (int i = 0; i < n_head * d; ++i) q[i] += bias_q[i];
    if (bias_k) for (int i = 0; i < n_kv * d; ++i) k[i] += bias_k[i];
    if (bias_v) for (int i = 0; i < n_kv * d; ++i) v[i] += bias_v[i];
    if (norm_q) for (int h = 0; h < n_head; ++h) oracle_rms_norm(q + h * d, norm_q, d, eps, q + h * d);
    if (norm_k) for (int h = 0; h < n_kv; ++h) oracle_rms_norm(k + h * d, norm_k, d, eps, k + h * d);
}

/* src/kernels.cu:136-145  quantize_q8_1_k, the form in which the reference's GPU decode path hands the attention
 * output to the next GEMV (src/model_gpu.cu:284): per group of 32 consecutive values d = max|x| / 127 and
 * q = roundf(x / d), q = 0 when the group is all zero; a ragged last group is padded with zeros.  The reference
 * builds this kernel with fast-math division; this restatement uses IEEE fp32 division (what the replacement
 * kernel uses), so against the reference kernel itself a value on a rounding boundary may differ by one. */
void oracle_quantize_q8_1(const float *x, int n, signed char *qs, float *scales) {
    for (int g = 0; g * 32 < n; ++g) {
        float amax = 0.0f;
        for (int i = g * 32; i < g * 32 + 32 && i < n; ++i) {
            float a = fabsf(x[i]);
            if (a > amax) amax = a;
        }
        const float d = amax / 127.0f;
        for (int i = g * 32; i < g * 32 + 32 && i < n; ++i)
            qs[i] = amax == 0.0f ? 0 : (signed char)roundf(x[i] / d);
        scales[g] = d;
    }
}

/* src/kernels.cu:147-205  quantize_mmq_q8_1_k, the form in which the reference's GPU prefill path hands an activation
 * matrix X [batch][ne00] (ne00 a multiple of 128 here) to its batched int8 GEMM.  Output: 144-byte blocks of 128
 * values, block (chunk c, token t) at index c * batch + t (:172); inside a block four scale slots, then 128 int8.  Per
 * group of 32 values: d_inv = 127 / max|x|, q = roundf(x * d_inv) (:184-189); slot = fp32 d = 1 / d_inv (:203), or for
 * ds4 the fp16 pair (d, sum of the 32 values) (:194-201), the sum taken as the kernel takes it: four values per
 * thread, then a butterfly over eight threads.  An all-zero group gives q = 0, d = 0.  IEEE division here, fast-math
 * in the reference's build. */
static unsigned short half_bits(float f) {
    _Float16 h = (_Float16)f;
    unsigned short b;
    memcpy(&b, &h, 2);
    return b;
}

void oracle_quantize_mmq_q8_1(const float *x, int ne00, int batch, int ds4, unsigned char *y) {
    for (int t = 0; t < batch; ++t) {
        for (int c = 0; c * 128 < ne00; ++c) {
            unsigned char *blk = y + ((size_t)c * batch + t) * 144;
            for (int g = 0; g < 4; ++g) {
                const float *v = x + (size_t)t * ne00 + c * 128 + g * 32;
                float amax = 0.0f, part[8];
                for (int i = 0; i < 32; ++i) {
                    float a = fabsf(v[i]);
                    if (a > amax) amax = a;
                }
                for (int l = 0; l < 8; ++l) part[l] = ((v[4 * l] + v[4 * l + 1]) + v[4 * l + 2]) + v[4 * l + 3];
                const float sum = ((part[0] + part[4]) + (part[2] + part[6])) + ((part[1] + part[5]) + (part[3] + part[7]));
                const float d_inv = amax > 0.0f ? 127.0f / amax : 0.0f;
                const float d = amax > 0.0f ? 1.0f / d_inv : 0.0f;
                for (int i = 0; i < 32; ++i) blk[16 + g * 32 + i] = (unsigned char)(signed char)roundf(v[i] * d_inv);
                if (ds4) {
                    unsigned short pair[2] = {half_bits(d), half_bits(sum)};
                    memcpy(blk + 4 * g, pair, 4);
                } else {
                    memcpy(blk + 4 * g, &d, 4);
                }
            }
        }
    }
}
