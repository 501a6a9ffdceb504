// Single-token decode attention over the fp16 KV cache: split-KV flash decoding in ONE launch.
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
// quad shuffles for max and sum, O += P V with V fragments taken by ldmatrix.trans.
//
// Merge, all inside the launch (the reference merges its four warps the same way,
// src/kernels.cu:1280-1344; here the tree has two more levels): the four warps' (m, l, O) are
// merged through shared memory into the CTA's partial; the CTA stores it and draws an arrival
// ticket for its group of about sqrt(n_splits) neighbouring splits; whoever draws a group's last ticket merges the
// group's partials, stores the result and draws a ticket of the kv head; the last of those
// merges the groups and writes the output (or the per-rank record of the multi-GPU path, which
// it can also push to the peers and merge with theirs).  Nobody waits for anybody: a CTA that is
// not last simply leaves.  Partials are always merged in index order, so the result does not
// depend on who arrives last.  The counters wrap to zero on the last ticket (atomicInc), which
// keeps a captured launch replayable.
//
// Optional fused prologue: RoPE of q, RoPE + fp16 conversion + cache store of the new token's
// k/v row (rope_*_ind, kv_store_ind of src/model_gpu.cu:277-281).  The CTA whose slice contains
// the new row stores it and patches it into its own shared-memory tile, so no CTA ever reads a
// row another CTA is writing.
#include <mutex>

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
    static constexpr int IN_OFF = CS_OFF + HD * 4;        // fp32 staging of q (16 rows), k_new, v_new (+ their biases)
    static constexpr int IN_ROWS = 18;
    static constexpr int TOTAL = IN_OFF + IN_ROWS * HD * 4;
    // merge buffers alias the stage area once the pipeline has drained: [4 warps][16 rows][HD + 8] fp32 (the 8
    // floats of padding spread the rows over the banks) and [4][16][2] for (m, l)
    static constexpr int MERGE_STRIDE = HD + 8;
    static constexpr int MERGE_O_BYTES = 4 * 16 * MERGE_STRIDE * 4;
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
    // short contexts are latency-bound: up to 4 tiles stay in one CTA (no merge across CTAs at all), up to 64 tiles
    // use at most 16 CTAs per kv head (one merge level instead of two)
    if (s.n_tiles <= 4) { if (tps < s.n_tiles) tps = s.n_tiles; }
    else if (s.n_tiles <= 64) { if (tps < (s.n_tiles + 15) / 16) tps = (s.n_tiles + 15) / 16; }
    if (tps < 1) tps = 1;
    s.tiles_per_split = tps;
    s.active = (s.n_tiles + tps - 1) / tps;
    return s;
}

__device__ __forceinline__ int clamp_len(int v, int n_ctx) { return v < 0 ? 0 : (v > n_ctx ? n_ctx : v); }

// ---- how the threads of a CTA share one kv head's [G][HD] block of fp32 values ------------------------------------
// The block is cut into float4 pieces; thread `tid` owns pieces tid, tid + 128, ... (piece -> row = head in the group,
// col4 = which four dims).  With HD = 128 a warp owns whole rows (rows warp, warp + 4, ...), a lane four dims.
template <int HD, bool WIDE>
struct Slots {
    static constexpr int F4_PER_ROW = HD / 4;
    static constexpr int ROWS = WIDE ? 16 : 8;
    static constexpr int N = ROWS * F4_PER_ROW / kThreads;
    static_assert(N >= 1, "at least one piece per thread");
    __device__ static __forceinline__ int row(int tid, int k) { return (tid + k * kThreads) / F4_PER_ROW; }
    __device__ static __forceinline__ int col4(int tid, int k) { return (tid + k * kThreads) % F4_PER_ROW; }
};

// Running log-sum-exp merge of one piece: acc = sum_i e^(m_i - M) O_i, L = sum_i e^(m_i - M) l_i, M = max m_i.
struct RunState {
    float M, L;
    float4 acc;
};
__device__ __forceinline__ RunState run_empty() { return RunState{-CUDART_INF_F, 0.f, make_float4(0.f, 0.f, 0.f, 0.f)}; }

// Adds n <= 8 parts; c turns a difference of m values into a base-2 exponent.
__device__ __forceinline__ void run_add(RunState& s, const float (&m)[8], const float (&l)[8], const float4 (&o)[8], int n, float c) {
    float mx = s.M;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        if (i < n) mx = fmaxf(mx, m[i]);
    if (mx == -CUDART_INF_F) return;           // only empty parts so far
    const float a = (s.M == -CUDART_INF_F) ? 0.f : fast_exp2((s.M - mx) * c);
    s.L *= a;
    s.acc.x *= a; s.acc.y *= a; s.acc.z *= a; s.acc.w *= a;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (i < n) {
            const float w = (m[i] == -CUDART_INF_F) ? 0.f : fast_exp2((m[i] - mx) * c);
            s.L = fmaf(w, l[i], s.L);
            s.acc.x = fmaf(w, o[i].x, s.acc.x);
            s.acc.y = fmaf(w, o[i].y, s.acc.y);
            s.acc.z = fmaf(w, o[i].z, s.acc.z);
            s.acc.w = fmaf(w, o[i].w, s.acc.w);
        }
    }
    s.M = mx;
}

// Merges parts 0..n-1 of one kv head, stored [part][G][HD] and [part][G][2], in index order.  The parts were written by
// other SMs a moment ago: read them from L2 (ld.cg), never through this SM's L1.  This runs on the critical path of the
// launch as a chain of L2 round trips, so a pass issues every load it needs before it uses any of them: the lanes that
// share a row (HD/4 of them) each fetch the (m, l) of one part and exchange the weights by shuffle, and every lane keeps
// its O pieces of up to 16 parts in flight.  Called by all threads of the CTA.
template <int HD, bool WIDE>
__device__ __forceinline__ void merge_parts(const float* o_base, const float* ml_base, int n, int G, float c,
                                            RunState (&st)[Slots<HD, WIDE>::N]) {
    using S = Slots<HD, WIDE>;
    constexpr int LPR = S::F4_PER_ROW;            // lanes per row: 32 or 16
    constexpr int PASS = 16;                      // parts per pass
    constexpr int KB = S::N < 2 ? S::N : 2;       // pieces per thread handled together
    const int tid = threadIdx.x;
    const int j = tid % LPR;
#pragma unroll
    for (int k = 0; k < S::N; ++k) st[k] = run_empty();
    for (int i0 = 0; i0 < n; i0 += PASS) {
        const int nn = min(PASS, n - i0);
#pragma unroll
        for (int k0 = 0; k0 < S::N; k0 += KB) {
            float2 ml[KB];
            float4 o[KB][PASS];
#pragma unroll
            for (int kk = 0; kk < KB; ++kk) {
                const int row = S::row(tid, k0 + kk), c4 = S::col4(tid, k0 + kk);
                const bool valid = row < G;
                ml[kk] = make_float2(-CUDART_INF_F, 0.f);
                if (valid && j < nn) ml[kk] = __ldcg(reinterpret_cast<const float2*>(ml_base + ((size_t)(i0 + j) * G + row) * 2));
#pragma unroll
                for (int i = 0; i < PASS; ++i) {
                    o[kk][i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (valid && i < nn) o[kk][i] = __ldcg(reinterpret_cast<const float4*>(o_base + ((size_t)(i0 + i) * G + row) * HD + c4 * 4));
                }
            }
#pragma unroll
            for (int kk = 0; kk < KB; ++kk) {
                RunState& r = st[k0 + kk];
                float mx = ml[kk].x;
#pragma unroll
                for (int off = PASS / 2; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off, LPR));
                const float m_new = fmaxf(r.M, mx);
                const bool empty = m_new == -CUDART_INF_F;
                const float a = (empty || r.M == -CUDART_INF_F) ? 0.f : fast_exp2((r.M - m_new) * c);
                const float w = (empty || ml[kk].x == -CUDART_INF_F) ? 0.f : fast_exp2((ml[kk].x - m_new) * c);
                r.L *= a;
                r.acc.x *= a; r.acc.y *= a; r.acc.z *= a; r.acc.w *= a;
#pragma unroll
                for (int i = 0; i < PASS; ++i) {
                    // parts are added in index order; lanes >= nn hold w = 0 and o = 0
                    const float wi = __shfl_sync(0xffffffffu, w, i, LPR);
                    const float li = __shfl_sync(0xffffffffu, ml[kk].y, i, LPR);
                    r.L = fmaf(wi, li, r.L);
                    r.acc.x = fmaf(wi, o[kk][i].x, r.acc.x);
                    r.acc.y = fmaf(wi, o[kk][i].y, r.acc.y);
                    r.acc.z = fmaf(wi, o[kk][i].z, r.acc.z);
                    r.acc.w = fmaf(wi, o[kk][i].w, r.acc.w);
                }
                r.M = m_new;
            }
        }
    }
}

template <int HD, bool WIDE>
__device__ __forceinline__ void store_part(float* o_base, float* ml_base, int G, const RunState (&st)[Slots<HD, WIDE>::N]) {
    using S = Slots<HD, WIDE>;
    const int tid = threadIdx.x;
#pragma unroll
    for (int k = 0; k < S::N; ++k) {
        const int row = S::row(tid, k), c4 = S::col4(tid, k);
        if (row < G) {
            *reinterpret_cast<float4*>(o_base + (size_t)row * HD + c4 * 4) = st[k].acc;
            if (c4 == 0) *reinterpret_cast<float2*>(ml_base + (size_t)row * 2) = make_float2(st[k].M, st[k].L);
        }
    }
}

// All threads of the CTA store their share of a partial, then one ticket is drawn from `counter`, which counts
// 0..n-1 and wraps to zero.  Returns true in every thread of the CTA that drew the last ticket.  Its later reads of
// the other arrivals' partials go to L2 (ld.cg), where those stores were made visible before their tickets were drawn,
// and cannot start before the ticket is known (barrier + branch).
__device__ __forceinline__ bool arrive_last(unsigned* counter, int n) {
    __shared__ unsigned s_ticket;
    if (n <= 1) return true;
    __syncthreads();                 // every thread's stores precede thread 0's fence (the fence is cumulative)
    if (threadIdx.x == 0) {
        __threadfence();
        s_ticket = atomicInc(counter, (unsigned)(n - 1));
    }
    __syncthreads();
    return s_ticket == (unsigned)(n - 1);
}

// ---- record exchange between ranks: tagged 8-byte words ---------------------------------------------------------
__device__ __forceinline__ unsigned long long tag_word(float v, unsigned tag) {
    return ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
}
__device__ __forceinline__ void peer_store_pair(unsigned long long* dst, float v0, float v1, unsigned tag) {
    asm volatile("st.relaxed.sys.global.v2.u64 [%0], {%1, %2};\n" ::"l"(dst), "l"(tag_word(v0, tag)), "l"(tag_word(v1, tag)) : "memory");
}
__device__ __forceinline__ void peer_load_pair(const unsigned long long* src, unsigned long long& w0, unsigned long long& w1) {
    asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];\n" : "=l"(w0), "=l"(w1) : "l"(src) : "memory");
}
__device__ __forceinline__ bool tagged(unsigned long long w, unsigned g) { return (unsigned)(w >> 32) == g; }

// Waits until the records of generation g of every rank have landed for one head and merges dims 4*c4..4*c4+3 of them.
// `recs`: rank 0's record of that head in this rank's exchange buffer, records of consecutive ranks `rank_stride` words
// apart.  A word is taken once its tag equals g; all polls of a round are independent loads.  The wait is bounded by
// `limit` SM clock cycles; false = it ran out (nothing merged).
__device__ __forceinline__ bool wait_records(const unsigned long long* recs, size_t rank_stride, int world, int hd, int c4,
                                             unsigned g, long long limit, RunState& fin) {
    const long long t0 = clock64();
    fin = run_empty();
    for (int r0 = 0; r0 < world; r0 += 8) {
        const int nn = min(8, world - r0);
        unsigned pending = (1u << nn) - 1u;
        float m[8], l[8];
        float4 o[8];
        while (pending) {
            unsigned long long w[8][6];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (pending >> i & 1u) {
                    const unsigned long long* rec = recs + (size_t)(r0 + i) * rank_stride;
                    peer_load_pair(rec + c4 * 4, w[i][0], w[i][1]);
                    peer_load_pair(rec + c4 * 4 + 2, w[i][2], w[i][3]);
                    peer_load_pair(rec + hd, w[i][4], w[i][5]);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if ((pending >> i & 1u) && tagged(w[i][0], g) && tagged(w[i][1], g) && tagged(w[i][2], g) && tagged(w[i][3], g) &&
                    tagged(w[i][4], g) && tagged(w[i][5], g)) {
                    o[i] = make_float4(__uint_as_float((unsigned)w[i][0]), __uint_as_float((unsigned)w[i][1]),
                                       __uint_as_float((unsigned)w[i][2]), __uint_as_float((unsigned)w[i][3]));
                    m[i] = __uint_as_float((unsigned)w[i][4]);
                    l[i] = __uint_as_float((unsigned)w[i][5]);
                    pending &= ~(1u << i);
                }
            }
            if (pending && clock64() - t0 > limit) return false;
        }
        run_add(fin, m, l, o, nn, LOG2E);      // records carry m in natural-log units of the scaled score
    }
    return true;
}

// q8_1 form of four consecutive output values per lane (see store_q8_group): a group of 32 values sits in 8 neighbouring
// lanes.  Called by all 32 lanes; `valid` only guards the stores.
__device__ __forceinline__ void store_q8_group4(float4 x, bool valid, size_t flat, int8_t* qs, float* scales) {
    float amax = fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));
#pragma unroll
    for (int off = 4; off; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const float d = __fdiv_rn(amax, 127.0f);
    if (!valid) return;
    char4 q = make_char4(0, 0, 0, 0);
    if (amax != 0.0f) {
        q.x = (signed char)roundf(__fdiv_rn(x.x, d));
        q.y = (signed char)roundf(__fdiv_rn(x.y, d));
        q.z = (signed char)roundf(__fdiv_rn(x.z, d));
        q.w = (signed char)roundf(__fdiv_rn(x.w, d));
    }
    *reinterpret_cast<char4*>(qs + flat) = q;
    if ((flat & 31) == 0) scales[flat >> 5] = d;
}

__device__ __forceinline__ float4 normalised(const RunState& s) {
    if (!(s.L > 0.f)) return make_float4(0.f, 0.f, 0.f, 0.f);
    return make_float4(s.acc.x / s.L, s.acc.y / s.L, s.acc.z / s.L, s.acc.w / s.L);
}

// What the CTA that holds a kv head's merged (M, L, O) does with it.  Called by all threads of that CTA.
template <int HD, bool WIDE, typename Args>
__device__ __forceinline__ void emit_final(const Args& p, int kvh, int G, const RunState (&st)[Slots<HD, WIDE>::N]) {
    using S = Slots<HD, WIDE>;
    const int tid = threadIdx.x;
    if (!p.emit_partial) {
#pragma unroll
        for (int k = 0; k < S::N; ++k) {
            const int row = S::row(tid, k), c4 = S::col4(tid, k);
            const bool valid = row < G;
            const size_t flat = (size_t)(kvh * G + row) * HD + c4 * 4;
            const float4 v = valid ? normalised(st[k]) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (valid && p.out) *reinterpret_cast<float4*>(p.out + flat) = v;
            if (p.out_qs) store_q8_group4(v, valid, flat, p.out_qs, p.out_scales);
        }
        return;
    }
    // per-rank record {O, m, l, 0, 0}, m in natural-log units of the scaled score
#pragma unroll
    for (int k = 0; k < S::N; ++k) {
        const int row = S::row(tid, k), c4 = S::col4(tid, k);
        if (row < G) {
            float* rec = p.out + (size_t)(kvh * G + row) * (HD + PART_PAD);
            *reinterpret_cast<float4*>(rec + c4 * 4) = st[k].acc;
            if (c4 == 0) *reinterpret_cast<float4*>(rec + HD) = make_float4(st[k].M * p.scale, st[k].L, 0.f, 0.f);
        }
    }
}

template <int HD, bool WIDE>
__global__ void __launch_bounds__(kThreads, 2) decode_split_kernel(const DecodeArgs p) {
    using L = DecodeSmem<HD>;
    using S = Slots<HD, WIDE>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int split = blockIdx.x, kvh = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = lane >> 2, t = lane & 3;
    const int G = p.n_head / p.n_kv;

    // The next kernel of the stream may start launching now; it waits for this grid to complete before it reads
    // anything this grid writes.
    pdl_trigger();
    // Unless the caller vouched for the position word and the cache rows below the newest one (overlap 2), nothing
    // is read before every preceding kernel of the stream has completed.
    if (p.overlap != 2) pdl_wait();

    const int npos = clamp_len(*p.d_pos + p.pos_bias, p.n_ctx);
    const SplitPlan plan = plan_splits(npos, p.n_splits, p.min_tiles);
    if (split >= max(plan.active, 1)) return;
    if (plan.active == 0) {
        // no valid row at all: the empty result (zero output, or a record with m = -inf, l = 0)
        if (p.overlap == 2) pdl_wait();
        RunState st[S::N];
#pragma unroll
        for (int k = 0; k < S::N; ++k) st[k] = run_empty();
        if (p.defer_final) store_part<HD, WIDE>(p.grp_o + (size_t)kvh * p.n_groups * G * HD, p.grp_ml + (size_t)kvh * p.n_groups * G * 2, G, st);
        else emit_final<HD, WIDE>(p, kvh, G, st);
        return;
    }
    const int tile0 = split * plan.tiles_per_split;
    const int tile1 = min(tile0 + plan.tiles_per_split, plan.n_tiles);
    const int nt = tile1 - tile0;

    const bool append = (p.fuse & 4) != 0;
    // The CTA whose last tile holds row npos-1 takes that row from the caller's k_new / v_new (fused append) or, when
    // tiles are fetched ahead of the dependency wait, re-reads it after the wait: the kernel just before this one
    // may be the one that stores it (kv_store_ind, src/model_gpu.cu:281).  Either way it is patched into this CTA's
    // shared-memory tile and left out of the asynchronous copies.
    const bool owner = (append || p.overlap == 2) && split == plan.active - 1;
    const int new_pos = npos - 1;
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

    // all stages are filled before anything else happens: tile s is copy group s
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
        if (s < nt) load_tile(s, s);
        cp_async_commit();
    }

    // RoPE table while the first tiles are in flight: it needs only the position word(s) and the model's constants
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
    }

    // q, the new K/V row and the scratch block belong to preceding kernels.  Their values may not be read yet, but L2 can be
    // asked to fetch the lines (a hint without a destination: whatever the preceding kernel still writes lands in the same
    // L2 lines), which takes the HBM latency of the first read after the wait off the critical path.
    if (p.overlap == 2) {
        const int q_lines = (G * HD * 4 + 127) / 128;
        if (tid < q_lines) l2_prefetch_line(reinterpret_cast<const char*>(p.q + (size_t)kvh * G * HD) + 128 * tid);
        if (owner && append && tid >= 64 && tid < 64 + 2 * (HD * 4 / 128)) {
            const int t2 = tid - 64, which = t2 / (HD * 4 / 128), ln = t2 % (HD * 4 / 128);
            l2_prefetch_line(reinterpret_cast<const char*>((which ? p.v_new : p.k_new) + (size_t)kvh * HD) + 128 * ln);
        }
        pdl_wait();
    }

    // ---- prologue: Q -> fp16 fragments, new K/V row ------------------------------------------
    // All global reads of the inputs are issued together (one round trip): q rows, then k_new and v_new, with their
    // biases added, land in a small fp32 staging area; the per-row work below reads shared memory only.
    float* s_in = reinterpret_cast<float*>(smem + L::IN_OFF);
    {
        const int rows = G + ((owner && append) ? 2 : 0);
        for (int idx = tid; idx < rows * (HD / 4); idx += kThreads) {
            const int row = idx / (HD / 4), c4 = idx % (HD / 4);
            const float* src;
            const float* bias;
            if (row < G) {
                src = p.q + (size_t)(kvh * G + row) * HD;
                bias = p.pre.bias_q ? p.pre.bias_q + (size_t)(kvh * G + row) * HD : nullptr;
            } else if (row == G) {
                src = p.k_new + (size_t)kvh * HD;
                bias = p.pre.bias_k ? p.pre.bias_k + (size_t)kvh * HD : nullptr;
            } else {
                src = p.v_new + (size_t)kvh * HD;
                bias = p.pre.bias_v ? p.pre.bias_v + (size_t)kvh * HD : nullptr;
            }
            float4 v = *reinterpret_cast<const float4*>(src + c4 * 4);
            if (bias) {
                const float4 bv = *reinterpret_cast<const float4*>(bias + c4 * 4);
                v.x += bv.x; v.y += bv.y; v.z += bv.z; v.w += bv.w;
            }
            const int srow = row < G ? row : 16 + (row - G);
            *reinterpret_cast<float4*>(s_in + srow * HD + c4 * 4) = v;
        }
        // rows >= G of the 16-row query tile are zero
        for (int i = tid; i < 16 * L::CHUNKS; i += kThreads) {
            const int row = i / L::CHUNKS;
            if (row >= G) *reinterpret_cast<uint4*>(smem + L::Q_OFF + swz<L::ROWB>(row, i % L::CHUNKS)) = make_uint4(0, 0, 0, 0);
        }
        if (owner && !append && tid < 2 * L::CHUNKS) {
            // the newest row as the cache holds it now that every preceding kernel has completed
            const int which = tid / L::CHUNKS, chunk = tid % L::CHUNKS;
            const uint4 v = __ldcg(reinterpret_cast<const uint4*>((which ? Vg : Kg) + (size_t)new_pos * HD + chunk * 8));
            *reinterpret_cast<uint4*>(smem + (which ? L::VNEW_OFF : L::KNEW_OFF) + chunk * 16) = v;
        }
    }
    __syncthreads();
    {
        // one warp per head row, round-robin
        for (int h = warp; h < G; h += kThreads / 32) {
            const float* src = s_in + h * HD;
            const float rn = p.pre.norm_q ? warp_row_rnorm(src, nullptr, HD, p.pre.eps, lane) : 1.f;
            rope_row_to_half(src, nullptr, p.pre.norm_q, rn, HD, rope_q, p.rope, s_cos, s_sin, lane, 32, [&](int e, float v) {
                *reinterpret_cast<__half*>(smem + L::Q_OFF + swz<L::ROWB>(h, e >> 3) + (e & 7) * 2) = __float2half_rn(v);
            });
        }
        if (owner && append) {
            __half* s_k = reinterpret_cast<__half*>(smem + L::KNEW_OFF);
            __half* s_v = reinterpret_cast<__half*>(smem + L::VNEW_OFF);
            if (warp == 0) {
                const float* src = s_in + 16 * HD;
                const float rn = p.pre.norm_k ? warp_row_rnorm(src, nullptr, HD, p.pre.eps, lane) : 1.f;
                rope_row_to_half(src, nullptr, p.pre.norm_k, rn, HD, rope_k, p.rope, s_cos, s_sin, lane, 32,
                                 [&](int e, float v) { s_k[e] = __float2half_rn(v); });
            } else if (warp == 1) {
                for (int e = lane; e < HD; e += 32) s_v[e] = __float2half_rn(s_in[17 * HD + e]);
            }
        }
    }
    __syncthreads();
    if (owner && append && tid < 2 * L::CHUNKS) {
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
        // tile t is copy group t; kStages groups were committed up front and one more per iteration from it = 1 on, so
        // at most kStages-1 (first iteration) or kStages-2 groups may still be in flight once tile `it` has landed
        if (it == 0) cp_async_wait<kStages - 1>(); else cp_async_wait<kStages - 2>();
        __syncthreads();                       // landed for every thread, and everybody is done with tile it-1
        if (it >= 1) {
            const int nxt = it - 1 + kStages;  // refill the stage tile it-1 used
            if (nxt < nt) load_tile(nxt, nxt % kStages);
            cp_async_commit();
        }
        const int stage = it % kStages;
        const int row0 = (tile0 + it) * DECODE_TILE;
        const uint32_t sK = smem_base + stage * L::STAGE_BYTES;
        const uint32_t sV = sK + L::TILE_BYTES;

        if (owner && it == nt - 1) {
            // patch the newest row into this CTA's copy of the tile
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

    // ---- merge the four warps: every warp scales its O by e^(m_w - M) and the sums are taken in warp order ---------
    cp_async_wait<0>();
    __syncthreads();
    float* mO = reinterpret_cast<float*>(smem);                        // [4][16][MERGE_STRIDE]
    float* mML = reinterpret_cast<float*>(smem + L::MERGE_ML_OFF);     // [4][16][2]
#pragma unroll
    for (int hh = 0; hh < NH; ++hh) {
        float l = l_run[hh];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (t == 0) *reinterpret_cast<float2*>(&mML[(warp * 16 + r + 8 * hh) * 2]) = make_float2(m_run[hh], l);
    }
    __syncthreads();
#pragma unroll
    for (int hh = 0; hh < NH; ++hh) {
        const int row = r + 8 * hh;
        float M = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, mML[(w * 16 + row) * 2]);
        const float wgt = (m_run[hh] == -CUDART_INF_F) ? 0.f : fast_exp2((m_run[hh] - M) * c);
        float* dst = mO + (size_t)(warp * 16 + row) * L::MERGE_STRIDE + 2 * t;
#pragma unroll
        for (int j = 0; j < HD / 8; ++j)
            *reinterpret_cast<float2*>(dst + 8 * j) = make_float2(o[j][2 * hh] * wgt, o[j][2 * hh + 1] * wgt);
    }
    __syncthreads();
    RunState st[S::N];
#pragma unroll
    for (int k = 0; k < S::N; ++k) {
        const int row = S::row(tid, k), c4 = S::col4(tid, k);
        st[k] = run_empty();
        if (row < G) {
            float mw[4], lw[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float2 ml = *reinterpret_cast<const float2*>(&mML[(w * 16 + row) * 2]);
                mw[w] = ml.x;
                lw[w] = ml.y;
                st[k].M = fmaxf(st[k].M, ml.x);
            }
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float wgt = (mw[w] == -CUDART_INF_F) ? 0.f : fast_exp2((mw[w] - st[k].M) * c);
                st[k].L = fmaf(wgt, lw[w], st[k].L);
                const float4 v = *reinterpret_cast<const float4*>(mO + (size_t)(w * 16 + row) * L::MERGE_STRIDE + c4 * 4);
                st[k].acc.x += v.x; st[k].acc.y += v.y; st[k].acc.z += v.z; st[k].acc.w += v.w;
            }
        }
    }

    // ---- merge across the CTAs of this kv head -------------------------------------------------------------------
    const size_t blk = (size_t)G * HD;       // floats of one partial
    if (plan.active == 1) {
        if (p.defer_final) store_part<HD, WIDE>(p.grp_o + (size_t)kvh * p.n_groups * blk, p.grp_ml + (size_t)kvh * p.n_groups * G * 2, G, st);
        else emit_final<HD, WIDE>(p, kvh, G, st);
        return;
    }
    {
        const size_t part = (size_t)kvh * p.n_splits + split;
        store_part<HD, WIDE>(p.ws_o + part * blk, p.ws_ml + part * G * 2, G, st);
    }
    // few partials merge in one level (one pass of merge_parts); more go through groups of p.group neighbours
    const int group = plan.active <= 16 ? plan.active : p.group;
    const int grp = split / group;
    const int grp_n = min(group, plan.active - grp * group);
    if (!arrive_last(p.tickets + kvh * p.n_groups + grp, grp_n)) return;
    {
        const size_t part0 = (size_t)kvh * p.n_splits + (size_t)grp * group;
        merge_parts<HD, WIDE>(p.ws_o + part0 * blk, p.ws_ml + part0 * G * 2, grp_n, G, c, st);
    }
    const int n_grp = (plan.active + group - 1) / group;
    if (p.defer_final) {
        // the exchange launch behind this one merges the kv head's group results (same plan, same order)
        const size_t gpart = (size_t)kvh * p.n_groups + grp;
        store_part<HD, WIDE>(p.grp_o + gpart * blk, p.grp_ml + gpart * G * 2, G, st);
        return;
    }
    if (n_grp > 1) {
        const size_t gpart = (size_t)kvh * p.n_groups + grp;
        store_part<HD, WIDE>(p.grp_o + gpart * blk, p.grp_ml + gpart * G * 2, G, st);
        if (!arrive_last(p.tickets + p.n_kv * p.n_groups + kvh, n_grp)) return;
        const size_t g0 = (size_t)kvh * p.n_groups;
        merge_parts<HD, WIDE>(p.grp_o + g0 * blk, p.grp_ml + g0 * G * 2, n_grp, G, c, st);
    }
    emit_final<HD, WIDE>(p, kvh, G, st);
}

// ---- log-sum-exp combine of gathered records -----------------------------------------------------------------
// One CTA per head, one thread per four dims: records [n_parts][n_head][hd + PART_PAD] -> out [n_head][hd].
__global__ void combine_records_kernel(const float* parts, int n_parts, float* out, int n_head, int hd) {
    const int h = blockIdx.x, c4 = threadIdx.x;
    if (c4 * 4 >= hd) return;
    const size_t rec = hd + PART_PAD;
    RunState fin = run_empty();
    for (int i0 = 0; i0 < n_parts; i0 += 8) {
        const int nn = min(8, n_parts - i0);
        float m[8], l[8];
        float4 o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (i < nn) {
                const float* r = parts + ((size_t)(i0 + i) * n_head + h) * rec;
                o[i] = *reinterpret_cast<const float4*>(r + c4 * 4);
                m[i] = r[hd];
                l[i] = r[hd + 1];
            }
        }
        run_add(fin, m, l, o, nn, LOG2E);
    }
    *reinterpret_cast<float4*>(out + (size_t)h * hd + c4 * 4) = normalised(fin);
}

// ---- record exchange between ranks, one CTA per head ----------------------------------------------------------
// The decode launch (defer_final) stops after its first merge level and leaves, per kv head, up to 16-odd group results
// (M, L, O) in the workspace.  CTA h of this launch merges head h's column of them into this rank's record -- one round
// of loads, every thread one dim -- and stores the record straight into every rank's exchange buffer (plain stores over
// NVLink, one tagged word per thread and rank); then, with fused_wait, it waits for every rank's record of the same
// generation in its own buffer and writes the merged output.  That takes the second ticket and the second merge pass of
// the decode launch off the path between the last K/V byte and the first peer store, and one CTA per head keeps the
// stores of a call spread over n_head SMs: from one or two SMs the same stores take several times as long (measured on
// 8 GPUs).  Only CTA h touches gen_push[h].
struct PeerExchangeArgs {
    const float* grp_o;                     // group results of the decode launch: [n_kv][n_groups][G][hd]
    const float* grp_ml;                    //                                     [n_kv][n_groups][G][2]  (M, L)
    const int* d_pos;
    int pos_bias, n_ctx, n_splits, min_tiles, group, n_groups, n_kv;
    float scale;
    const unsigned long long* peer_bufs;    // device array of `world` buffer pointers (this rank's own included)
    int* gen_push;                          // [n_head]
    float* out;
    int* status;
    int rank, world, n_head, head_dim, fused_wait, overlap;
    long long wait_cycles;
};

__global__ void __launch_bounds__(160) peer_exchange_kernel(const PeerExchangeArgs p) {
    const int h = blockIdx.x, tid = threadIdx.x, hd = p.head_dim;
    pdl_trigger();
    // how many group results the decode launch left for this kv head: its own plan, from the same position word
    const int G = p.n_head / p.n_kv, kvh = h / G, row = h - kvh * G;
    // What does not depend on the decode launch is fetched while that launch still runs: the ranks' buffer addresses, and
    // the position word where the caller vouched for it (overlap 2) -- the plan decides which loads follow the wait.
    unsigned long long* peer[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) peer[r] = r < p.world ? reinterpret_cast<unsigned long long*>(p.peer_bufs[r]) : nullptr;
    int pos_word = 0;
    if (p.overlap == 2) pos_word = __ldcg(p.d_pos);
    pdl_wait();                    // the decode launch's group results must be complete
    if (p.overlap != 2) pos_word = __ldcg(p.d_pos);
    const unsigned g = (unsigned)(__ldcg(p.gen_push + h) + 1);
    const size_t rec_sz = hd + PART_PAD;
    if (tid < hd + 2) {
        const int npos = clamp_len(pos_word + p.pos_bias, p.n_ctx);
        const SplitPlan plan = plan_splits(npos, p.n_splits, p.min_tiles);
        const int group = plan.active <= 16 ? max(plan.active, 1) : p.group;
        const int n_grp = plan.active <= 1 ? 1 : (plan.active + group - 1) / group;
        // thread d < hd carries O[d], threads hd and hd + 1 carry m and l (two neighbouring words of the record).  Every
        // thread reads all (M, L) pairs (a broadcast from L2) and its own column of every group: one round of loads.
        const float c = p.scale * LOG2E;
        const float* go = p.grp_o + ((size_t)kvh * p.n_groups * G + row) * hd;
        const float* gml = p.grp_ml + ((size_t)kvh * p.n_groups * G + row) * 2;
        float M = -CUDART_INF_F, L = 0.f, acc = 0.f;
        for (int i0 = 0; i0 < n_grp; i0 += 16) {
            float2 ml[16];
            float o[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                ml[i] = make_float2(-CUDART_INF_F, 0.f);
                o[i] = 0.f;
                if (i0 + i < n_grp) {
                    ml[i] = __ldcg(reinterpret_cast<const float2*>(gml + (size_t)(i0 + i) * G * 2));
                    if (tid < hd) o[i] = __ldcg(go + (size_t)(i0 + i) * G * hd + tid);
                }
            }
            float m_new = M;
#pragma unroll
            for (int i = 0; i < 16; ++i) m_new = fmaxf(m_new, ml[i].x);
            const float a = (m_new == -CUDART_INF_F || M == -CUDART_INF_F) ? 0.f : fast_exp2((M - m_new) * c);
            L *= a; acc *= a;
#pragma unroll
            for (int i = 0; i < 16; ++i) {          // groups are added in index order
                const float w = (m_new == -CUDART_INF_F || ml[i].x == -CUDART_INF_F) ? 0.f : fast_exp2((ml[i].x - m_new) * c);
                L = fmaf(w, ml[i].y, L);
                acc = fmaf(w, o[i], acc);
            }
            M = m_new;
        }
        // the record carries m in natural-log units of the scaled score
        const float v = tid < hd ? acc : (tid == hd ? M * p.scale : L);
        const size_t off = ((size_t)((g & 1) * p.world + p.rank) * p.n_head + h) * rec_sz + tid;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r < p.world) asm volatile("st.relaxed.sys.global.u64 [%0], %1;\n" ::"l"(peer[r] + off), "l"(tag_word(v, g)) : "memory");
        }
        for (int r = 8; r < p.world; ++r) {
            unsigned long long* dst = reinterpret_cast<unsigned long long*>(p.peer_bufs[r]) + off;
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;\n" ::"l"(dst), "l"(tag_word(v, g)) : "memory");
        }
    }
    if (p.fused_wait && tid * 4 < hd) {
        const unsigned long long* recs = reinterpret_cast<const unsigned long long*>(p.peer_bufs[p.rank]) +
                                         ((size_t)(g & 1) * p.world * p.n_head + h) * rec_sz;
        RunState fin;
        if (wait_records(recs, (size_t)p.n_head * rec_sz, p.world, hd, tid, g, p.wait_cycles, fin))
            *reinterpret_cast<float4*>(p.out + (size_t)h * hd + tid * 4) = normalised(fin);
        else if (p.status)
            atomicExch(p.status, 1);
    }
    __syncthreads();
    if (tid == 0) p.gen_push[h] = (int)g;
}

// ---- wait for every rank's record of this generation and merge them -------------------------------------------
// One CTA per head, one thread per four dims, in a launch of its own: the form that can run after all pushes on a
// single GPU.
struct PeerWaitArgs {
    const unsigned char* my_buf;
    float* out;
    int* gen_wait;      // [n_head]
    int* status;
    int world, n_head, head_dim;
    long long wait_cycles;
};

__global__ void peer_wait_combine_kernel(const PeerWaitArgs p) {
    const int h = blockIdx.x, c4 = threadIdx.x;
    pdl_trigger();
    pdl_wait();
    const unsigned g = (unsigned)(__ldcg(p.gen_wait + h) + 1);
    __syncthreads();
    if (c4 * 4 < p.head_dim) {
        const size_t rec_sz = p.head_dim + PART_PAD;
        const unsigned long long* recs = reinterpret_cast<const unsigned long long*>(p.my_buf) +
                                         ((size_t)(g & 1) * p.world * p.n_head + h) * rec_sz;
        RunState fin;
        if (wait_records(recs, (size_t)p.n_head * rec_sz, p.world, p.head_dim, c4, g, p.wait_cycles, fin))
            *reinterpret_cast<float4*>(p.out + (size_t)h * p.head_dim + c4 * 4) = normalised(fin);
        else if (p.status)
            atomicExch(p.status, 1);
    }
    __syncthreads();
    if (c4 == 0) p.gen_wait[h] = (int)g;
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

// ---- arrival counters ----------------------------------------------------------------------------------
// The counters of the in-launch merge must be zero when a launch starts and are zero again when it ends.  They live
// in the library image (zero-initialised when the module is loaded) rather than in the caller's workspace, which
// nobody promises to clear.  A slot is bound to a workspace address on first use; launches that use different
// workspaces therefore never share counters, and launches that share a workspace must not overlap anyway.
static __device__ unsigned g_tickets[kTicketSlots * kTicketWords];
namespace {
struct TicketTable {
    unsigned* base = nullptr;
    const void* owner[kTicketSlots] = {};
    unsigned long long stamp[kTicketSlots] = {};
    unsigned long long clock = 0;
};
TicketTable g_ticket_tab[64];
std::mutex g_ticket_mutex;
} // namespace

cudaError_t decode_ticket_slot(const void* workspace, unsigned** tickets) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_ticket_mutex);
    TicketTable& tab = g_ticket_tab[dev];
    if (!tab.base) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_tickets);
        if (e != cudaSuccess) return e;
        tab.base = reinterpret_cast<unsigned*>(p);
    }
    if (!workspace) { *tickets = tab.base; return cudaSuccess; }      // set-up call: only the address look-up
    int pick = -1, oldest = 0;
    for (int i = 0; i < kTicketSlots; ++i) {
        if (tab.owner[i] == workspace) { pick = i; break; }
        if (tab.stamp[i] < tab.stamp[oldest]) oldest = i;
    }
    if (pick < 0) {
        pick = oldest;                    // never used (stamp 0) or least recently used
        tab.owner[pick] = workspace;
    }
    tab.stamp[pick] = ++tab.clock;
    *tickets = tab.base + (size_t)pick * kTicketWords;
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
    if (launches) *launches += 1;
    return e;
}

cudaError_t launch_combine_records(const float* parts, int n_parts, float* out, int n_head, int head_dim,
                                   cudaStream_t stream, unsigned long long* launches) {
    combine_records_kernel<<<n_head, 32, 0, stream>>>(parts, n_parts, out, n_head, head_dim);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

cudaError_t launch_peer_exchange(const DecodeArgs& d, const unsigned long long* peer_bufs, int* gen_push, int rank, int world,
                                 int fused_wait, float* out, int* status, long long wait_cycles, int overlap,
                                 cudaStream_t stream, unsigned long long* launches) {
    PeerExchangeArgs x;
    x.grp_o = d.grp_o; x.grp_ml = d.grp_ml; x.d_pos = d.d_pos; x.pos_bias = d.pos_bias; x.n_ctx = d.n_ctx;
    x.n_splits = d.n_splits; x.min_tiles = d.min_tiles; x.group = d.group; x.n_groups = d.n_groups; x.n_kv = d.n_kv;
    x.scale = d.scale;
    x.peer_bufs = peer_bufs; x.gen_push = gen_push; x.out = out; x.status = status;
    x.rank = rank; x.world = world; x.n_head = d.n_head; x.head_dim = d.head_dim; x.fused_wait = fused_wait;
    x.wait_cycles = wait_cycles;
    x.overlap = overlap;
    cudaError_t e = launch_dependent(peer_exchange_kernel, dim3(d.n_head), 128 + 32, 0, stream, overlap, x);
    if (launches) *launches += 1;
    return e;
}

cudaError_t launch_peer_wait_combine(const void* my_buf, int world, float* out, int n_head, int head_dim, int* gen_wait,
                                     int* status, long long wait_cycles, int overlap, cudaStream_t stream,
                                     unsigned long long* launches) {
    PeerWaitArgs w;
    w.my_buf = reinterpret_cast<const unsigned char*>(my_buf);
    w.out = out;
    w.gen_wait = gen_wait;
    w.status = status;
    w.world = world;
    w.n_head = n_head;
    w.head_dim = head_dim;
    w.wait_cycles = wait_cycles;
    cudaError_t e = launch_dependent(peer_wait_combine_kernel, dim3(n_head), 32, 0, stream, overlap, w);
    if (launches) *launches += 1;
    return e;
}

} // namespace oattn
