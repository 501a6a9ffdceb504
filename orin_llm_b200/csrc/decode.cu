// Single-token decode attention over the fp16 KV cache: split-KV flash decoding.
//
// Stands in for flash_attention_decode_mma_k (src/kernels.cu:1107-1345), which walks the whole
// sequence with one CTA per kv head.  Here the sequence of every kv head is cut into
// `n_splits` contiguous slices, one CTA each (grid = n_splits x n_kv, about two CTAs per SM), so
// that every SM streams cache rows.  The grid never depends on the position: each CTA derives
// its slice from *d_pos, and CTAs whose slice is empty return at once, which keeps the launch
// replayable from a CUDA graph (src/model_gpu.cu:295-344).
//
// Data path of one CTA (4 warps): 64-row K and V tiles are brought to shared memory with 16-byte
// cp.async copies, three stages deep; rows at or past the valid length are zero-filled by the
// copy itself.  Warp w owns rows 16w..16w+15 of every tile: S = Q K^T with the (padded to 16)
// query heads of the group as the M dimension of mma.m16n8k16, online softmax in fp32 with
// quad shuffles for max and sum, O += P V with V fragments taken by ldmatrix.trans.  The four
// warps' (m, l, O) are merged through shared memory, and the CTA writes one partial per head.
// A second small kernel merges the partials of all slices (log-sum-exp combine).
//
// Optional fused prologue: RoPE of q, RoPE + fp16 conversion + cache store of the new token's
// k/v row (rope_*_ind, kv_store_ind of src/model_gpu.cu:277-281).  The CTA whose slice contains
// the new row stores it and patches it into its own shared-memory tile, so no CTA ever reads a
// row another CTA is writing.
#include "attn_internal.h"

namespace oattn {

namespace {

constexpr int kThreads = 128;
constexpr int kStages = 3;

template <int HD>
struct DecodeSmem {
    static constexpr int ROWB = HD * 2;
    static constexpr int CHUNKS = ROWB / 16;
    static constexpr int TILE_BYTES = DECODE_TILE * ROWB;
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int Q_OFF = kStages * STAGE_BYTES;
    static constexpr int Q_BYTES = 16 * ROWB;
    static constexpr int KNEW_OFF = Q_OFF + Q_BYTES;
    static constexpr int VNEW_OFF = KNEW_OFF + ROWB;
    static constexpr int CS_OFF = VNEW_OFF + ROWB;        // cos[HD/2], sin[HD/2] fp32
    static constexpr int TOTAL = CS_OFF + HD * 4;
    // merge buffers alias the stage area once the pipeline has drained
    static constexpr int MERGE_O_BYTES = 4 * 16 * HD * 4;
    static constexpr int MERGE_ML_OFF = MERGE_O_BYTES;
    static_assert(MERGE_O_BYTES + 4 * 16 * 2 * 4 <= kStages * STAGE_BYTES, "merge area must fit in the stage area");
};

struct SplitPlan {
    int n_tiles, tiles_per_split, active;
};

__host__ __device__ inline SplitPlan plan_splits(int npos, int n_splits, int min_tiles) {
    SplitPlan s;
    s.n_tiles = (npos + DECODE_TILE - 1) / DECODE_TILE;
    int tps = (s.n_tiles + n_splits - 1) / n_splits;
    if (tps < min_tiles) tps = min_tiles;
    if (tps < 1) tps = 1;
    s.tiles_per_split = tps;
    s.active = (s.n_tiles + tps - 1) / tps;
    return s;
}

__device__ __forceinline__ int clamp_len(int v, int n_ctx) { return v < 0 ? 0 : (v > n_ctx ? n_ctx : v); }

template <int HD, bool WIDE>
__global__ void __launch_bounds__(kThreads, 2) decode_split_kernel(const DecodeArgs p) {
    using L = DecodeSmem<HD>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int split = blockIdx.x, kvh = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = lane >> 2, t = lane & 3;
    const int G = p.n_head / p.n_kv;

    // The merge kernel of this call may start launching now; it waits for this grid to complete before it reads.
    pdl_trigger();
    // Unless the caller vouched for the position word and the cache rows below the valid length (overlap 2), nothing
    // is read before every preceding kernel of the stream has completed.
    if (p.overlap != 2) pdl_wait();

    const int npos = clamp_len(*p.d_pos + p.pos_bias, p.n_ctx);
    const SplitPlan plan = plan_splits(npos, p.n_splits, p.min_tiles);
    if (split >= plan.active) return;
    const int tile0 = split * plan.tiles_per_split;
    const int tile1 = min(tile0 + plan.tiles_per_split, plan.n_tiles);
    const int nt = tile1 - tile0;

    const bool append = (p.fuse & 4) != 0;
    const bool owner = append && split == plan.active - 1;   // this CTA's last tile holds row npos-1
    const int new_pos = npos - 1;
    // rows the async copies may read: the new row is not in the cache yet when it is fused
    const int nload = owner ? new_pos : npos;

    const __half* Kg = reinterpret_cast<const __half*>(p.kc) + (size_t)kvh * p.n_ctx * HD;
    const __half* Vg = reinterpret_cast<const __half*>(p.vc) + (size_t)kvh * p.n_ctx * HD;
    const uint32_t smem_base = smem_u32(smem);

    auto load_tile = [&](int rel, int stage) {
        const int row0 = (tile0 + rel) * DECODE_TILE;
        const uint32_t sb = smem_base + stage * L::STAGE_BYTES;
        constexpr int PER_MAT = DECODE_TILE * L::CHUNKS;
#pragma unroll
        for (int i = 0; i < 2 * PER_MAT / kThreads; ++i) {
            const int idx = tid + i * kThreads;
            const int which = idx / PER_MAT;
            const int rem = idx % PER_MAT;
            const int row = rem / L::CHUNKS, chunk = rem % L::CHUNKS;
            const int grow = row0 + row;
            const bool ok = grow < nload;
            const __half* src = (which ? Vg : Kg) + (size_t)(ok ? grow : 0) * HD + chunk * 8;
            cp_async_16(sb + which * L::TILE_BYTES + swz<L::ROWB>(row, chunk), src, ok ? 16 : 0);
        }
    };

#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) {
        if (s < nt) load_tile(s, s);
        cp_async_commit();
    }

    // the first tiles are in flight; q, the new K/V row and the scratch block belong to preceding kernels
    if (p.overlap == 2) pdl_wait();

    // ---- prologue: RoPE table, Q -> fp16 fragments, new K/V row ------------------------------
    float* s_cos = reinterpret_cast<float*>(smem + L::CS_OFF);
    float* s_sin = s_cos + HD / 2;
    const bool rope_q = (p.fuse & 1) != 0, rope_k = (p.fuse & 2) != 0;
    if (rope_q || (rope_k && owner)) {
        for (int i = tid; i < p.rope.n_rot / 2; i += kThreads) {
            const float f = rope_freq(i, p.rope.n_rot, p.rope.theta, p.rope.freq_factors);
            // the rotation angle follows the token's position in the whole sequence, which differs from the local row
            // index when the cache holds only a slice of the sequence
            rope_cs(p.d_rope_pos ? *p.d_rope_pos : new_pos, f, s_cos[i], s_sin[i]);
        }
        __syncthreads();
    }
    {
        // rows >= G of the 16-row query tile are zero
        for (int i = tid; i < 16 * L::CHUNKS; i += kThreads) {
            const int row = i / L::CHUNKS;
            if (row >= G) *reinterpret_cast<uint4*>(smem + L::Q_OFF + swz<L::ROWB>(row, i % L::CHUNKS)) = make_uint4(0, 0, 0, 0);
        }
        // one warp per head row, round-robin
        for (int h = warp; h < G; h += kThreads / 32) {
            const float* src = p.q + (size_t)(kvh * G + h) * HD;
            const float* bq = p.pre.bias_q ? p.pre.bias_q + (size_t)(kvh * G + h) * HD : nullptr;
            const float rn = p.pre.norm_q ? warp_row_rnorm(src, bq, HD, p.pre.eps, lane) : 1.f;
            rope_row_to_half(src, bq, p.pre.norm_q, rn, HD, rope_q, p.rope, s_cos, s_sin, lane, 32, [&](int e, float v) {
                *reinterpret_cast<__half*>(smem + L::Q_OFF + swz<L::ROWB>(h, e >> 3) + (e & 7) * 2) = __float2half_rn(v);
            });
        }
        if (owner) {
            __half* s_k = reinterpret_cast<__half*>(smem + L::KNEW_OFF);
            __half* s_v = reinterpret_cast<__half*>(smem + L::VNEW_OFF);
            if (warp == 0) {
                const float* src = p.k_new + (size_t)kvh * HD;
                const float* bk = p.pre.bias_k ? p.pre.bias_k + (size_t)kvh * HD : nullptr;
                const float rn = p.pre.norm_k ? warp_row_rnorm(src, bk, HD, p.pre.eps, lane) : 1.f;
                rope_row_to_half(src, bk, p.pre.norm_k, rn, HD, rope_k, p.rope, s_cos, s_sin, lane, 32,
                                 [&](int e, float v) { s_k[e] = __float2half_rn(v); });
            } else if (warp == 1) {
                const float* bv = p.pre.bias_v ? p.pre.bias_v + (size_t)kvh * HD : nullptr;
                for (int e = lane; e < HD; e += 32)
                    s_v[e] = __float2half_rn(pre_value(p.v_new + (size_t)kvh * HD, bv, nullptr, 1.f, e));
            }
        }
    }
    __syncthreads();
    if (owner && tid < 2 * L::CHUNKS) {
        // store the new row into the cache (kv_store_k, src/kernels.cu:1660-1678)
        const int which = tid / L::CHUNKS, chunk = tid % L::CHUNKS;
        const uint4 v = *reinterpret_cast<const uint4*>(smem + (which ? L::VNEW_OFF : L::KNEW_OFF) + chunk * 16);
        __half* dst = const_cast<__half*>(which ? Vg : Kg) + (size_t)new_pos * HD + chunk * 8;
        *reinterpret_cast<uint4*>(dst) = v;
    }

    uint32_t qa[HD / 16][4];
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
        const int row = (lane & 7) + 8 * ((lane >> 3) & 1);
        const int chunk = 2 * kk + (lane >> 4);
        ldmatrix_x4(smem_base + L::Q_OFF + swz<L::ROWB>(row, chunk), qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3]);
        if (!WIDE) { qa[kk][1] = 0u; qa[kk][3] = 0u; }
    }

    constexpr int NH = WIDE ? 2 : 1;           // row halves that carry real heads
    float o[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F};
    float l_run[2] = {0.f, 0.f};
    const float c = p.scale * LOG2E;
    const int wr0 = warp * 16;

    for (int it = 0; it < nt; ++it) {
        cp_async_wait<kStages - 2>();
        __syncthreads();
        {
            const int nxt = it + kStages - 1;
            if (nxt < nt) load_tile(nxt, nxt % kStages);
            cp_async_commit();
        }
        const int stage = it % kStages;
        const int row0 = (tile0 + it) * DECODE_TILE;
        const uint32_t sK = smem_base + stage * L::STAGE_BYTES;
        const uint32_t sV = sK + L::TILE_BYTES;

        if (owner && it == nt - 1) {
            // patch the new token's row into this CTA's copy of the tile
            const int prow = new_pos - row0;
            if (tid < 2 * L::CHUNKS) {
                const int which = tid / L::CHUNKS, chunk = tid % L::CHUNKS;
                const uint4 v = *reinterpret_cast<const uint4*>(smem + (which ? L::VNEW_OFF : L::KNEW_OFF) + chunk * 16);
                *reinterpret_cast<uint4*>(smem + stage * L::STAGE_BYTES + which * L::TILE_BYTES + swz<L::ROWB>(prow, chunk)) = v;
            }
            __syncthreads();
        }
        if (row0 + wr0 >= npos) continue;   // this warp's 16 rows are all past the end (warp-uniform)

        // ---- S = Q K^T for 16 rows: two 8-row n-tiles ----------------------------------------
        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            uint32_t b0, b1, b2, b3;
            const int row = wr0 + 8 * (lane >> 4) + (lane & 7);
            const int chunk = 2 * kk + ((lane >> 3) & 1);
            ldmatrix_x4(sK + swz<L::ROWB>(row, chunk), b0, b1, b2, b3);
            mma_16816(s[0], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b0, b1);
            mma_16816(s[1], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b2, b3);
        }
        if (row0 + DECODE_TILE > npos) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (row0 + wr0 + 8 * j + 2 * t + (e & 1) >= npos) s[j][e] = -CUDART_INF_F;
        }

        // ---- online softmax ------------------------------------------------------------------
        float alpha[2] = {1.f, 1.f};
#pragma unroll
        for (int hh = 0; hh < NH; ++hh) {
            float mx = fmaxf(fmaxf(s[0][2 * hh], s[0][2 * hh + 1]), fmaxf(s[1][2 * hh], s[1][2 * hh + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[hh], mx);
            const float m_safe = (m_new == -CUDART_INF_F) ? 0.f : m_new;
            alpha[hh] = fast_exp2((m_run[hh] - m_safe) * c);
            const float mc = m_safe * c;
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                s[j][2 * hh] = fast_exp2(fmaf(s[j][2 * hh], c, -mc));
                s[j][2 * hh + 1] = fast_exp2(fmaf(s[j][2 * hh + 1], c, -mc));
                sum += s[j][2 * hh] + s[j][2 * hh + 1];
            }
            l_run[hh] = l_run[hh] * alpha[hh] + sum;
            m_run[hh] = m_new;
        }
        const bool rescale = WIDE ? (alpha[0] != 1.f || alpha[1] != 1.f) : (alpha[0] != 1.f);
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
            for (int j = 0; j < HD / 8; ++j) {
                o[j][0] *= alpha[0];
                o[j][1] *= alpha[0];
                if (WIDE) { o[j][2] *= alpha[1]; o[j][3] *= alpha[1]; }
            }
        }
        const uint32_t pa0 = pack_half2(s[0][0], s[0][1]);
        const uint32_t pa2 = pack_half2(s[1][0], s[1][1]);
        const uint32_t pa1 = WIDE ? pack_half2(s[0][2], s[0][3]) : 0u;
        const uint32_t pa3 = WIDE ? pack_half2(s[1][2], s[1][3]) : 0u;

        // ---- O += P V ------------------------------------------------------------------------
#pragma unroll
        for (int jp = 0; jp < HD / 16; ++jp) {
            uint32_t b0, b1, b2, b3;
            const int row = wr0 + (lane & 7) + 8 * ((lane >> 3) & 1);
            const int chunk = 2 * jp + (lane >> 4);
            ldmatrix_x4_trans(sV + swz<L::ROWB>(row, chunk), b0, b1, b2, b3);
            mma_16816(o[2 * jp], pa0, pa1, pa2, pa3, b0, b1);
            mma_16816(o[2 * jp + 1], pa0, pa1, pa2, pa3, b2, b3);
        }
    }

    // ---- merge the four warps ------------------------------------------------------------------
    cp_async_wait<0>();
    __syncthreads();
    float* mO = reinterpret_cast<float*>(smem);                        // [4][16][HD]
    float* mML = reinterpret_cast<float*>(smem + L::MERGE_ML_OFF);     // [4][16][2]
#pragma unroll
    for (int hh = 0; hh < NH; ++hh) {
        float l = l_run[hh];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int row = r + 8 * hh;
        if (t == 0) {
            mML[(warp * 16 + row) * 2 + 0] = m_run[hh];
            mML[(warp * 16 + row) * 2 + 1] = l;
        }
#pragma unroll
        for (int j = 0; j < HD / 8; ++j) {
            float2 v = make_float2(o[j][2 * hh], o[j][2 * hh + 1]);
            *reinterpret_cast<float2*>(&mO[(warp * 16 + row) * HD + 8 * j + 2 * t]) = v;
        }
    }
    __syncthreads();
    const bool direct = (plan.active == 1) && !p.emit_partial;
    for (int idx = tid; idx < G * HD; idx += kThreads) {
        const int row = idx / HD, d = idx % HD;
        float M = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mML[(w * 16 + row) * 2]);
        float Lsum = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = mML[(w * 16 + row) * 2];
            const float wgt = (mw == -CUDART_INF_F) ? 0.f : fast_exp2((mw - M) * c);
            Lsum += wgt * mML[(w * 16 + row) * 2 + 1];
            O += wgt * mO[(w * 16 + row) * HD + d];
        }
        const int head = kvh * G + row;
        if (direct) {
            const float val = O / Lsum;
            if (p.out) p.out[(size_t)head * HD + d] = val;
            if (p.out_qs) store_q8_group(val, (size_t)head * HD + d, p.out_qs, p.out_scales);
        } else {
            p.ws_o[((size_t)head * p.n_splits + split) * HD + d] = O;
            if (d == 0) {
                p.ws_ml[((size_t)head * p.n_splits + split) * 2 + 0] = M * p.scale;
                p.ws_ml[((size_t)head * p.n_splits + split) * 2 + 1] = Lsum;
            }
        }
    }
}

// ---- log-sum-exp combine -----------------------------------------------------------------------
// One CTA per head, 8 warps.  Part s of head h: O at o_base + h*o_hs + s*o_ss (hd floats), (m, l)
// at ml_base + h*ml_hs + s*ml_ss.  n_parts < 0: derive the number of parts from *d_pos with the
// same plan as the split kernel (and do nothing when that kernel already wrote the result).
struct CombineArgs {
    const float* o_base;
    const float* ml_base;
    long long o_hs, o_ss, ml_hs, ml_ss;
    float* out;
    int head_dim;
    int n_parts;
    const int* d_pos;
    int pos_bias, n_ctx, n_splits, min_tiles;
    int emit_partial;
    // peer exchange (multi-GPU): when peer_bufs is set the un-normalised record of head h is stored straight into
    // every rank's exchange buffer (plain stores over NVLink), each value tagged with the generation of the call
    const unsigned long long* peer_bufs;   // device array of `world` pointers (this rank's own buffer included)
    int* gen_push;                          // [n_head] private generation counters of this rank
    int rank, world, n_head;
    int8_t* out_qs;                         // optional q8_1 form of the final output (see store_q8_group)
    float* out_scales;
    int fused_wait;                         // also wait for all ranks' records and write the final output to `out`
    int* status;                            // raised when that wait ran out
};

constexpr int kCombineThreads = 512;
constexpr int kPeerWaitThreads = 128 + 32;   // head_dim (at most 128) value pollers + up to DECODE_MAX_RANKS (m, l) pollers
constexpr int kCombineWarps = kCombineThreads / 32;

// ---- record exchange between ranks: tagged 8-byte words ---------------------------------------------------------
__device__ __forceinline__ void peer_store_word(unsigned long long* dst, float v, unsigned tag) {
    const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;\n" ::"l"(dst), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long peer_load_word(const unsigned long long* src) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];\n" : "=l"(w) : "l"(src) : "memory");
    return w;
}

// Wait for every rank's record of generation g for head h in this rank's exchange buffer and merge them.
// Called by all threads of a CTA of at least head_dim + world threads.  Thread d < head_dim polls the words that carry
// O[d] of every source rank (all polls of one round are independent loads); thread head_dim + r polls m and l of
// rank r.  A word is taken once its tag equals g.  The wait is bounded (about two seconds), after which a status
// word is raised and the output is left untouched.
__device__ __forceinline__ void peer_wait_merge(const unsigned char* my_buf, int g, int h, int world, int n_head, int hd,
                                                float* out, int* status) {
    __shared__ int s_fail;
    __shared__ float s_m[DECODE_MAX_RANKS], s_l[DECODE_MAX_RANKS];
    const int tid = threadIdx.x;
    __syncthreads();
    if (tid == 0) s_fail = 0;
    __syncthreads();
    const size_t rec_sz = hd + PART_PAD;
    const unsigned long long* recs = reinterpret_cast<const unsigned long long*>(my_buf) +
                                     ((size_t)(g & 1) * world * n_head + h) * rec_sz;
    const size_t rank_stride = (size_t)n_head * rec_sz;
    float o[DECODE_MAX_RANKS];
    const long long t0 = clock64();
    if (tid < hd) {
        unsigned pending = (1u << world) - 1u;      // world <= DECODE_MAX_RANKS = 16
        while (pending) {
            unsigned long long w[DECODE_MAX_RANKS];
#pragma unroll
            for (int r = 0; r < DECODE_MAX_RANKS; ++r)
                if (pending >> r & 1u) w[r] = peer_load_word(recs + r * rank_stride + tid);
#pragma unroll
            for (int r = 0; r < DECODE_MAX_RANKS; ++r) {
                if ((pending >> r & 1u) && (unsigned)(w[r] >> 32) == (unsigned)g) {
                    o[r] = __uint_as_float((unsigned)w[r]);
                    pending &= ~(1u << r);
                }
            }
            if (pending && clock64() - t0 > 4000000000LL) { s_fail = 1; break; }
        }
    } else if (tid < hd + world) {
        const int r = tid - hd;
        const unsigned long long* rec = recs + r * rank_stride + hd;
        for (;;) {
            const unsigned long long wm = peer_load_word(rec), wl = peer_load_word(rec + 1);
            if ((unsigned)(wm >> 32) == (unsigned)g && (unsigned)(wl >> 32) == (unsigned)g) {
                s_m[r] = __uint_as_float((unsigned)wm);
                s_l[r] = __uint_as_float((unsigned)wl);
                break;
            }
            if (clock64() - t0 > 4000000000LL) { s_fail = 1; break; }
        }
    }
    __syncthreads();
    if (s_fail) {
        if (tid == 0 && status) atomicExch(status, 1);
        return;
    }
    if (tid < hd) {
        float M = -CUDART_INF_F;
        for (int r = 0; r < world; ++r) M = fmaxf(M, s_m[r]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int r = 0; r < DECODE_MAX_RANKS; ++r) {
            if (r < world) {
                const float w = (s_m[r] == -CUDART_INF_F) ? 0.f : __expf(s_m[r] - M);
                L = fmaf(w, s_l[r], L);
                acc = fmaf(w, o[r], acc);
            }
        }
        out[(size_t)h * hd + tid] = L > 0.f ? acc / L : 0.f;
    }
}

__global__ void __launch_bounds__(kCombineThreads) combine_kernel(const CombineArgs p) {
    __shared__ float s_w[DECODE_MAX_SPLITS];
    __shared__ float s_red[kCombineWarps];
    __shared__ float4 s_acc[kCombineWarps][32];
    const int h = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hd = p.head_dim;

    pdl_trigger();
    pdl_wait();      // the split kernel's partials (or the gathered records) must be complete

    int n = p.n_parts;
    if (n < 0) {
        const int npos = clamp_len(*p.d_pos + p.pos_bias, p.n_ctx);
        const SplitPlan plan = plan_splits(npos, p.n_splits, p.min_tiles);
        n = plan.active;
        if (n == 1 && !p.emit_partial) return;   // the split kernel wrote the output itself
    }
    const float* ml = p.ml_base + (size_t)h * p.ml_hs;
    const float* ob = p.o_base + (size_t)h * p.o_hs;

    // The partials were written a moment ago and sit in L2; the kernel is a chain of L2 round trips, so every
    // phase issues all of its loads before it uses any of them.  (m, l) of part tid: one load per thread
    // (n <= DECODE_MAX_SPLITS = kCombineThreads).
    float2 my = make_float2(-CUDART_INF_F, 0.f);
    if (tid < n) my = make_float2(ml[(size_t)tid * p.ml_ss], ml[(size_t)tid * p.ml_ss + 1]);
    // prefetch this warp's O rows (up to 4 parts in flight per lane) while the weights are being computed
    constexpr int U = 4;
    float4 pre[U];
    const bool lane_ok = lane * 4 < hd;
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int s = warp + u * kCombineWarps;
        pre[u] = (lane_ok && s < n) ? *reinterpret_cast<const float4*>(ob + (size_t)s * p.o_ss + lane * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }

    float mx = my.x;
#pragma unroll
    for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if (lane == 0) s_red[warp] = mx;
    __syncthreads();
    float M = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < kCombineWarps; ++w) M = fmaxf(M, s_red[w]);
    __syncthreads();

    const float wgt = (my.x == -CUDART_INF_F) ? 0.f : __expf(my.x - M);
    if (tid < n) s_w[tid] = wgt;
    float lsum = wgt * my.y;
#pragma unroll
    for (int off = 16; off; off >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, off);
    if (lane == 0) s_red[warp] = lsum;
    __syncthreads();
    float Lsum = 0.f;
#pragma unroll
    for (int w = 0; w < kCombineWarps; ++w) Lsum += s_red[w];

    // O: warp w takes parts w, w+16, ...; lane takes 4 consecutive dims
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int s = warp + u * kCombineWarps;
        const float w = s < n ? s_w[s] : 0.f;
        acc.x = fmaf(w, pre[u].x, acc.x);
        acc.y = fmaf(w, pre[u].y, acc.y);
        acc.z = fmaf(w, pre[u].z, acc.z);
        acc.w = fmaf(w, pre[u].w, acc.w);
    }
    if (lane_ok) {
        for (int s0 = warp + U * kCombineWarps; s0 < n; s0 += U * kCombineWarps) {
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int s = s0 + u * kCombineWarps;
                v[u] = s < n ? *reinterpret_cast<const float4*>(ob + (size_t)s * p.o_ss + lane * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int s = s0 + u * kCombineWarps;
                const float w = s < n ? s_w[s] : 0.f;
                acc.x = fmaf(w, v[u].x, acc.x);
                acc.y = fmaf(w, v[u].y, acc.y);
                acc.z = fmaf(w, v[u].z, acc.z);
                acc.w = fmaf(w, v[u].w, acc.w);
            }
        }
    }
    s_acc[warp][lane] = acc;
    __syncthreads();
    if (tid < hd) {
        const int l4 = tid >> 2, e = tid & 3;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kCombineWarps; ++w) {
            const float4 a = s_acc[w][l4];
            v += (e == 0) ? a.x : (e == 1) ? a.y : (e == 2) ? a.z : a.w;
        }
        if (p.emit_partial && p.peer_bufs) {
            const unsigned g = (unsigned)(p.gen_push[h] + 1);   // generation of this call; only this CTA touches gen_push[h]
            const size_t rec_sz = hd + PART_PAD;
            for (int r = 0; r < p.world; ++r) {
                unsigned long long* rec = reinterpret_cast<unsigned long long*>(p.peer_bufs[r]) +
                                          ((size_t)((g & 1) * p.world + p.rank) * p.n_head + h) * rec_sz;
                peer_store_word(rec + tid, v, g);
                if (tid == 0) {
                    peer_store_word(rec + hd + 0, M, g);
                    peer_store_word(rec + hd + 1, Lsum, g);
                }
            }
        } else if (p.emit_partial) {
            float* rec = p.out + (size_t)h * (hd + PART_PAD);
            rec[tid] = v;
            if (tid == 0) {
                rec[hd + 0] = M;
                rec[hd + 1] = Lsum;
                rec[hd + 2] = 0.f;
                rec[hd + 3] = 0.f;
            }
        } else {
            const float val = Lsum > 0.f ? v / Lsum : 0.f;
            if (p.out) p.out[(size_t)h * hd + tid] = val;
            if (p.out_qs) store_q8_group(val, (size_t)h * hd + tid, p.out_qs, p.out_scales);
        }
    }
    if (p.emit_partial && p.peer_bufs) {
        const int g = p.gen_push[h] + 1;
        if (p.fused_wait) {
            // same launch also waits for the other ranks' records of this generation and writes the final output
            peer_wait_merge(reinterpret_cast<const unsigned char*>(p.peer_bufs[p.rank]), g, h, p.world, p.n_head, hd,
                            p.out, p.status);
        }
        __syncthreads();
        if (tid == 0) p.gen_push[h] = g;
    }
}

// ---- wait for every rank's record of this generation and merge them -------------------------------------------
// One CTA per head, in a launch of its own (the form that can run after all pushes on a single GPU); the work is
// peer_wait_merge above.
struct PeerWaitArgs {
    const unsigned char* my_buf;
    float* out;
    int* gen_wait;      // [n_head]
    int* status;
    int world, n_head, head_dim;
};

__global__ void __launch_bounds__(kPeerWaitThreads) peer_wait_combine_kernel(const PeerWaitArgs p) {
    const int h = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    const int g = p.gen_wait[h] + 1;
    peer_wait_merge(p.my_buf, g, h, p.world, p.n_head, p.head_dim, p.out, p.status);
    __syncthreads();
    if (threadIdx.x == 0) p.gen_wait[h] = g;
}

template <int HD, bool WIDE>
cudaError_t launch_split(const DecodeArgs& a, cudaStream_t stream) {
    return launch_dependent(decode_split_kernel<HD, WIDE>, dim3(a.n_splits, a.n_kv), kThreads, DecodeSmem<HD>::TOTAL, stream,
                            a.overlap, a);
}

} // namespace

// ---- built-in scratch for callers that cannot allocate --------------------------------------------------
// A fixed block of device memory that is part of the library image: every GPU that loads the library
// carries it until the process exits.  In host code the name below is only a handle for the runtime, not a
// device address; the address a kernel can use comes from cudaGetSymbolAddress, asked once per device with
// that device current.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static void* g_static_scratch_addr[64] = {};

cudaError_t decode_static_scratch(void** ptr) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!g_static_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return e;
        g_static_scratch_addr[dev] = p;
    }
    *ptr = g_static_scratch_addr[dev];
    return cudaSuccess;
}

int decode_num_splits(int n_kv, int sm_count) {
    int s = (2 * sm_count) / (n_kv > 0 ? n_kv : 1);
    if (s < 1) s = 1;
    if (s > DECODE_MAX_SPLITS) s = DECODE_MAX_SPLITS;
    return s;
}

cudaError_t decode_set_attributes() {
    cudaError_t e;
    e = cudaFuncSetAttribute(decode_split_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeSmem<128>::TOTAL);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(decode_split_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeSmem<128>::TOTAL);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(decode_split_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeSmem<64>::TOTAL);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(decode_split_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DecodeSmem<64>::TOTAL);
    return e;
}

cudaError_t launch_decode(const DecodeArgs& a, cudaStream_t stream, unsigned long long* launches,
                          cudaEvent_t ev_start, cudaEvent_t ev_stop) {
    const int G = a.n_head / a.n_kv;
    const bool wide = G > 8;
    cudaError_t e;
    // inside a stream capture the timing events become external event-record nodes of the graph
    unsigned ev_flags = cudaEventRecordDefault;
    if (ev_start || ev_stop) {
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &cs) == cudaSuccess && cs == cudaStreamCaptureStatusActive) ev_flags = cudaEventRecordExternal;
    }
    if (ev_start) cudaEventRecordWithFlags(ev_start, stream, ev_flags);
    if (a.head_dim == 128) e = wide ? launch_split<128, true>(a, stream) : launch_split<128, false>(a, stream);
    else                   e = wide ? launch_split<64, true>(a, stream) : launch_split<64, false>(a, stream);
    if (ev_stop) cudaEventRecordWithFlags(ev_stop, stream, ev_flags);
    if (e != cudaSuccess) return e;
    CombineArgs c;
    c.o_base = a.ws_o;
    c.ml_base = a.ws_ml;
    c.o_hs = (long long)a.n_splits * a.head_dim;
    c.o_ss = a.head_dim;
    c.ml_hs = (long long)a.n_splits * 2;
    c.ml_ss = 2;
    c.out = a.out;
    c.head_dim = a.head_dim;
    c.n_parts = -1;
    c.d_pos = a.d_pos;
    c.pos_bias = a.pos_bias;
    c.n_ctx = a.n_ctx;
    c.n_splits = a.n_splits;
    c.min_tiles = a.min_tiles;
    c.emit_partial = a.emit_partial;
    c.peer_bufs = a.peer_bufs;
    c.gen_push = a.gen_push;
    c.rank = a.rank;
    c.world = a.world;
    c.n_head = a.n_head;
    c.fused_wait = a.fused_wait;
    c.status = a.peer_status;
    c.out_qs = a.out_qs;
    c.out_scales = a.out_scales;
    e = launch_dependent(combine_kernel, dim3(a.n_head), kCombineThreads, 0, stream, a.overlap, c);
    if (launches) *launches += 2;
    return e;
}

cudaError_t launch_combine_records(const float* parts, int n_parts, float* out, int n_head, int head_dim,
                                   cudaStream_t stream, unsigned long long* launches) {
    CombineArgs c;
    const long long rec = head_dim + PART_PAD;
    c.o_base = parts;
    c.ml_base = parts + head_dim;
    c.o_hs = rec;
    c.o_ss = rec * n_head;
    c.ml_hs = rec;
    c.ml_ss = rec * n_head;
    c.out = out;
    c.head_dim = head_dim;
    c.n_parts = n_parts;
    c.d_pos = nullptr;
    c.pos_bias = 0;
    c.n_ctx = 0;
    c.n_splits = 0;
    c.min_tiles = 1;
    c.emit_partial = 0;
    c.peer_bufs = nullptr;
    c.gen_push = nullptr;
    c.rank = 0;
    c.world = 1;
    c.n_head = n_head;
    c.fused_wait = 0;
    c.status = nullptr;
    c.out_qs = nullptr;
    c.out_scales = nullptr;
    combine_kernel<<<n_head, kCombineThreads, 0, stream>>>(c);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

cudaError_t launch_peer_wait_combine(const void* my_buf, int world, float* out, int n_head, int head_dim, int* gen_wait,
                                     int* status, int overlap, cudaStream_t stream, unsigned long long* launches) {
    PeerWaitArgs w;
    w.my_buf = reinterpret_cast<const unsigned char*>(my_buf);
    w.out = out;
    w.gen_wait = gen_wait;
    w.status = status;
    w.world = world;
    w.n_head = n_head;
    w.head_dim = head_dim;
    cudaError_t e = launch_dependent(peer_wait_combine_kernel, dim3(n_head), kPeerWaitThreads, 0, stream, overlap, w);
    if (launches) *launches += 1;
    return e;
}

} // namespace oattn
