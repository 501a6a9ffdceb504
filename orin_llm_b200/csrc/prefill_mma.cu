// Chunked-prefill causal GQA attention, warp-level mma.sync version.
//
// Same contract as flash_attention_prefill_mma_k (src/kernels.cu:1351-1568): query token t of
// the chunk sees cache rows 0..n_past+t.  This kernel is the in-library cross-check and the
// fall-back shape coverage for the tcgen05 kernel (prefill_tc.cu); it shares that kernel's
// prologue (q already rotated, scaled by scale*log2(e) and converted to fp16 in q16).
//
// One CTA = 4 warps = 64 query rows of ONE kv head, a row being a (token, head-in-group) pair:
// row R -> token t0 + R/G, head kvh*G + R%G, so one pass over the K/V rows of the kv head serves
// all G heads of floor(64/G) tokens.  K/V tiles of 64 rows are staged with cp.async (2 stages in
// flight); each warp computes S (16 x 64), the causal mask, online softmax and O += P V for its
// 16 rows.
#include "attn_internal.h"

namespace oattn {

namespace {

constexpr int kThreads = 128;
constexpr int kTile = 64;
constexpr int kStages = 3;

template <int HD>
struct PrefillSmem {
    static constexpr int ROWB = HD * 2;
    static constexpr int CHUNKS = ROWB / 16;
    static constexpr int TILE_BYTES = kTile * ROWB;
    static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
    static constexpr int Q_OFF = kStages * STAGE_BYTES;
    static constexpr int TOTAL = Q_OFF + 64 * ROWB;
};

template <int HD>
__global__ void __launch_bounds__(kThreads, 2) prefill_mma_kernel(const PrefillArgs p) {
    using L = PrefillSmem<HD>;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int r = lane >> 2, t = lane & 3;
    const int G = p.n_head / p.n_kv;
    const int TB = 64 / G;                       // tokens per CTA
    const int kvh = blockIdx.y;
    // heaviest blocks (latest tokens) first
    const int tb = gridDim.x - 1 - blockIdx.x;
    const int t0 = tb * TB;
    const int ntok = min(TB, p.batch - t0);
    const int kv_end = p.n_past + t0 + ntok;     // rows any query of this CTA may see
    const int nt = (kv_end + kTile - 1) / kTile;

    const __half* Kg = reinterpret_cast<const __half*>(p.kc) + (size_t)kvh * p.n_ctx * HD;
    const __half* Vg = reinterpret_cast<const __half*>(p.vc) + (size_t)kvh * p.n_ctx * HD;
    const uint32_t smem_base = smem_u32(smem);

    auto load_tile = [&](int tile, int stage) {
        const int row0 = tile * kTile;
        const uint32_t sb = smem_base + stage * L::STAGE_BYTES;
        constexpr int PER_MAT = kTile * L::CHUNKS;
#pragma unroll
        for (int i = 0; i < 2 * PER_MAT / kThreads; ++i) {
            const int idx = tid + i * kThreads;
            const int which = idx / PER_MAT;
            const int rem = idx % PER_MAT;
            const int row = rem / L::CHUNKS, chunk = rem % L::CHUNKS;
            const int grow = row0 + row;
            const bool ok = grow < kv_end;
            const __half* src = (which ? Vg : Kg) + (size_t)(ok ? grow : 0) * HD + chunk * 8;
            cp_async_16(sb + which * L::TILE_BYTES + swz<L::ROWB>(row, chunk), src, ok ? 16 : 0);
        }
    };
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) {
        if (s < nt) load_tile(s, s);
        cp_async_commit();
    }

    // Q rows -> shared (zero for rows that map to no token)
    for (int i = tid; i < 64 * L::CHUNKS; i += kThreads) {
        const int R = i / L::CHUNKS, chunk = i % L::CHUNKS;
        const int tok = R / G, hg = R % G;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tok < ntok) v = *reinterpret_cast<const uint4*>(p.q16 + ((size_t)(t0 + tok) * p.n_head + kvh * G + hg) * HD + chunk * 8);
        *reinterpret_cast<uint4*>(smem + L::Q_OFF + swz<L::ROWB>(R, chunk)) = v;
    }
    __syncthreads();
    uint32_t qa[HD / 16][4];
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
        const int row = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
        ldmatrix_x4(smem_base + L::Q_OFF + swz<L::ROWB>(row, 2 * kk + (lane >> 4)), qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3]);
    }

    // last visible cache row of this thread's two query rows
    int vis[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int R = warp * 16 + r + 8 * hh;
        const int tok = R / G;
        vis[hh] = (tok < ntok) ? p.n_past + t0 + tok : -1;
    }

    float o[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F};
    float l_run[2] = {0.f, 0.f};

    for (int it = 0; it < nt; ++it) {
        cp_async_wait<kStages - 2>();
        __syncthreads();
        {
            const int nxt = it + kStages - 1;
            if (nxt < nt) load_tile(nxt, nxt % kStages);
            cp_async_commit();
        }
        const int stage = it % kStages;
        const int row0 = it * kTile;
        const uint32_t sK = smem_base + stage * L::STAGE_BYTES;
        const uint32_t sV = sK + L::TILE_BYTES;

        float s[kTile / 8][4];
#pragma unroll
        for (int j = 0; j < kTile / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
            for (int jp = 0; jp < kTile / 16; ++jp) {
                uint32_t b0, b1, b2, b3;
                const int row = 16 * jp + 8 * (lane >> 4) + (lane & 7);
                ldmatrix_x4(sK + swz<L::ROWB>(row, 2 * kk + ((lane >> 3) & 1)), b0, b1, b2, b3);
                mma_16816(s[2 * jp], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b0, b1);
                mma_16816(s[2 * jp + 1], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b2, b3);
            }
        }
        // causal mask (also hides zero-filled rows >= kv_end, which are > vis for every row)
        if (row0 + kTile - 1 > p.n_past + t0) {
#pragma unroll
            for (int j = 0; j < kTile / 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (row0 + 8 * j + 2 * t + (e & 1) > vis[e >> 1]) s[j][e] = -CUDART_INF_F;
        }
        float alpha[2];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            float mx = -CUDART_INF_F;
#pragma unroll
            for (int j = 0; j < kTile / 8; ++j) mx = fmaxf(mx, fmaxf(s[j][2 * hh], s[j][2 * hh + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[hh], mx);
            const float m_safe = (m_new == -CUDART_INF_F) ? 0.f : m_new;
            alpha[hh] = fast_exp2(m_run[hh] - m_safe);
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < kTile / 8; ++j) {
                s[j][2 * hh] = fast_exp2(s[j][2 * hh] - m_safe);
                s[j][2 * hh + 1] = fast_exp2(s[j][2 * hh + 1] - m_safe);
                sum += s[j][2 * hh] + s[j][2 * hh + 1];
            }
            l_run[hh] = l_run[hh] * alpha[hh] + sum;
            m_run[hh] = m_new;
        }
        if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
            for (int j = 0; j < HD / 8; ++j) {
                o[j][0] *= alpha[0]; o[j][1] *= alpha[0];
                o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
            }
        }
#pragma unroll
        for (int ks = 0; ks < kTile / 16; ++ks) {
            const uint32_t pa0 = pack_half2(s[2 * ks][0], s[2 * ks][1]);
            const uint32_t pa1 = pack_half2(s[2 * ks][2], s[2 * ks][3]);
            const uint32_t pa2 = pack_half2(s[2 * ks + 1][0], s[2 * ks + 1][1]);
            const uint32_t pa3 = pack_half2(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
            for (int jp = 0; jp < HD / 16; ++jp) {
                uint32_t b0, b1, b2, b3;
                const int row = 16 * ks + (lane & 7) + 8 * ((lane >> 3) & 1);
                ldmatrix_x4_trans(sV + swz<L::ROWB>(row, 2 * jp + (lane >> 4)), b0, b1, b2, b3);
                mma_16816(o[2 * jp], pa0, pa1, pa2, pa3, b0, b1);
                mma_16816(o[2 * jp + 1], pa0, pa1, pa2, pa3, b2, b3);
            }
        }
    }
    cp_async_wait<0>();

#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        float l = l_run[hh];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int R = warp * 16 + r + 8 * hh;
        const int tok = R / G, hg = R % G;
        if (tok < ntok) {
            const float inv = 1.f / l;
            float* dst = p.out + ((size_t)(t0 + tok) * p.n_head + kvh * G + hg) * HD;
#pragma unroll
            for (int j = 0; j < HD / 8; ++j)
                *reinterpret_cast<float2*>(dst + 8 * j + 2 * t) = make_float2(o[j][2 * hh] * inv, o[j][2 * hh + 1] * inv);
        }
    }
}

} // namespace

cudaError_t prefill_mma_set_attributes() {
    cudaError_t e = cudaFuncSetAttribute(prefill_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, PrefillSmem<128>::TOTAL);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(prefill_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, PrefillSmem<64>::TOTAL);
}

cudaError_t launch_prefill_mma(const PrefillArgs& a, cudaStream_t stream, unsigned long long* launches) {
    const int G = a.n_head / a.n_kv;
    const int TB = 64 / G;
    dim3 grid((a.batch + TB - 1) / TB, a.n_kv);
    if (a.head_dim == 128) prefill_mma_kernel<128><<<grid, kThreads, PrefillSmem<128>::TOTAL, stream>>>(a);
    else                   prefill_mma_kernel<64><<<grid, kThreads, PrefillSmem<64>::TOTAL, stream>>>(a);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

} // namespace oattn
