// RoPE, KV-cache store, KV-cache shift, and the prefill prologue (RoPE + fp16 conversion of a
// chunk's q, k, v in one launch).
#include "attn_internal.h"

namespace oattn {

namespace {

// ---- standalone RoPE: rope_neox_k / rope_normal_k (src/kernels.cu:1622-1657) --------------------
// One CTA rotates ROWS_PER_CTA consecutive rows; the n_rot/2 frequencies are computed once per
// CTA.  Position of row r: *d_pos when given, else n_past + r/heads (src/kernels.cu:1627-1629).
constexpr int kRopeThreads = 256;
constexpr int kRopeRows = 32;

__global__ void __launch_bounds__(kRopeThreads) rope_kernel(float* x, int rows, int head_dim, RopeArgs r, int n_past,
                                                            int heads, const int* d_pos) {
    __shared__ float s_freq[128];
    const int half = r.n_rot / 2;
    for (int i = threadIdx.x; i < half; i += kRopeThreads) s_freq[i] = rope_freq(i, r.n_rot, r.theta, r.freq_factors);
    __syncthreads();
    const int row0 = blockIdx.x * kRopeRows;
    const int nrow = min(kRopeRows, rows - row0);
    const int pos_ind = d_pos ? *d_pos : 0;
    for (int idx = threadIdx.x; idx < nrow * half; idx += kRopeThreads) {
        const int row = row0 + idx / half, pair = idx % half;
        const int pos = d_pos ? pos_ind : n_past + row / heads;
        float c, s;
        rope_cs(pos, s_freq[pair], c, s);
        int i0, i1;
        rope_pair_index(r.rope_type, pair, r.n_rot, i0, i1);
        float* xr = x + (size_t)row * head_dim;
        const float x0 = xr[i0], x1 = xr[i1];
        xr[i0] = x0 * c - x1 * s;
        xr[i1] = x0 * s + x1 * c;
    }
}

// ---- standalone KV store: kv_store_k (src/kernels.cu:1660-1678) ---------------------------------
// One CTA per (token, head) row; fp32 -> fp16 round-to-nearest, cache layout [head][pos][hd].
__global__ void __launch_bounds__(128) kv_store_kernel(uint16_t* kc, uint16_t* vc, const float* k, const float* v,
                                                       int heads, int head_dim, int n_ctx, int pos_base,
                                                       const int* d_pos) {
    const int head = blockIdx.x % heads, b = blockIdx.x / heads;
    const int pos = d_pos ? *d_pos : pos_base + b;
    if (pos < 0 || pos >= n_ctx) return;
    const size_t src = (size_t)blockIdx.x * head_dim;
    const size_t dst = ((size_t)head * n_ctx + pos) * head_dim;
    for (int i = threadIdx.x; i < head_dim; i += blockDim.x) {
        kc[dst + i] = __half_as_ushort(__float2half_rn(k[src + i]));
        vc[dst + i] = __half_as_ushort(__float2half_rn(v[src + i]));
    }
}

// ---- KV shift: kv_shift_k (src/kernels.cu:1682-1700) --------------------------------------------
// The reference moves one element per thread per position in a serial loop.  Here one CTA slides the rows of one
// (layer, kv head) of K or of V: grid = (2, n_kv, n_layer), 512 threads.  The rows of a head are contiguous, so a step
// reads a contiguous block of 128 rows (every load issued, 64 bytes in flight per thread), passes a barrier and
// writes the block `shift` rows lower; a step's sources overlap only its own destinations, never those of another
// step.  Then the tail is zeroed.  All accesses are 16-byte pieces of consecutive addresses.
constexpr int kShiftThreads = 512;
constexpr int kShiftPieces = 4;        // 16-byte pieces per thread and step

__global__ void __launch_bounds__(kShiftThreads) kv_shift_kernel(uint16_t* kc, uint16_t* vc, int n_kv, int head_dim,
                                                                 int n_ctx, int n_keep, int shift) {
    const int head = blockIdx.y, layer = blockIdx.z;
    const size_t row_bytes = (size_t)head_dim * 2;
    uint8_t* base = reinterpret_cast<uint8_t*>(blockIdx.x ? vc : kc) + ((size_t)layer * n_kv + head) * n_ctx * row_bytes;
    const int last = n_ctx - shift;                        // first row of the zeroed tail
    const size_t p16 = row_bytes / 16;                     // pieces per row
    const size_t first = (size_t)n_keep * p16, end = (size_t)max(last, n_keep) * p16, off = (size_t)shift * p16;
    uint4* c = reinterpret_cast<uint4*>(base);
    constexpr size_t STEP = (size_t)kShiftThreads * kShiftPieces;
    for (size_t i0 = first; i0 < end; i0 += STEP) {
        uint4 t[kShiftPieces];
#pragma unroll
        for (int u = 0; u < kShiftPieces; ++u) {
            const size_t i = i0 + (size_t)u * kShiftThreads + threadIdx.x;
            if (i < end) t[u] = c[i + off];
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < kShiftPieces; ++u) {
            const size_t i = i0 + (size_t)u * kShiftThreads + threadIdx.x;
            if (i < end) c[i] = t[u];
        }
    }
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (size_t i = (size_t)max(last, 0) * p16 + threadIdx.x; i < (size_t)n_ctx * p16; i += kShiftThreads) c[i] = z;
}

// ---- prefill prologue ---------------------------------------------------------------------------
// One CTA per chunk token b (position n_past + b).  cos/sin of the n_rot/2 angles are computed
// once and reused by all query heads and kv heads of the token:
//   q  -> [RoPE] -> * scale*log2(e) -> fp16 -> q16[b][head][hd]
//   k  -> [RoPE] -> fp16 -> kc[head][n_past+b][hd]         (when appending)
//   v  ->           fp16 -> vc[head][n_past+b][hd]
// This is rope_*_batch(q), rope_*_batch(k), kv_store_batch of src/model_gpu.cu:379-383 plus the
// fp16 conversion of Q that the reference does inside its attention kernel (src/kernels.cu:1393-1410).
constexpr int kPrologueThreads = 256;
constexpr int kPrologueMaxRows = 160;     // q and k head rows of one token whose 1/rms the norm step keeps in shared memory

__global__ void __launch_bounds__(kPrologueThreads) prefill_prologue_kernel(const PrefillArgs p) {
    __shared__ float s_cos[64], s_sin[64];
    const int b = blockIdx.x, tid = threadIdx.x;
    const int hd = p.head_dim, pos = p.n_past + b;
    const bool rope_q = (p.fuse & 1) != 0, rope_k = (p.fuse & 2) != 0, append = (p.fuse & 4) != 0;
    // Programmatic dependent launch: the attention kernel of this call may start its set-up now, and the cos/sin table
    // (arguments only) is made while the kernel before this one drains; inputs, scratch and cache are touched after
    // the wait.
    pdl_trigger();
    if (rope_q || rope_k) {
        for (int i = tid; i < p.rope.n_rot / 2; i += kPrologueThreads) {
            const float f = rope_freq(i, p.rope.n_rot, p.rope.theta, p.rope.freq_factors);
            rope_cs(pos, f, s_cos[i], s_sin[i]);
        }
    }
    pdl_wait();
    __syncthreads();
    if (b == 0 && tid == 0 && p.status) *p.status = 0;
    // bias and per-head RMSNorm in front of the rotation (src/model_gpu.cu:372-377): 1/rms of every q and k head row
    __shared__ float s_rn[kPrologueMaxRows];
    if (p.pre.norm_q || p.pre.norm_k) {
        const int warp = tid >> 5, lane = tid & 31;
        const int rows = p.n_head + (append ? p.n_kv : 0);
        for (int row = warp; row < rows; row += kPrologueThreads / 32) {
            const bool is_q = row < p.n_head;
            const int head = is_q ? row : row - p.n_head;
            const float* src = is_q ? p.q + ((size_t)b * p.n_head + head) * hd : p.k_new + ((size_t)b * p.n_kv + head) * hd;
            const float* bias = is_q ? p.pre.bias_q : p.pre.bias_k;
            const float* nw = is_q ? p.pre.norm_q : p.pre.norm_k;
            const float rn = nw ? warp_row_rnorm(src, bias ? bias + (size_t)head * hd : nullptr, hd, p.pre.eps, lane) : 1.f;
            if (lane == 0) s_rn[row] = rn;
        }
        __syncthreads();
    }
    // Fast path (no per-head norm, whole-row rotation or none, head_dim a multiple of 16 and at most 128): a thread
    // takes 8 consecutive dims of one head row -- two float4 loads, one 16-byte store; for the (i, i + n_rot/2)
    // pairing it takes the partner 8 dims as well.  All loads of a thread are issued before its stores.
    const uintptr_t ptr_bits = (uintptr_t)p.q | (uintptr_t)p.k_new | (uintptr_t)p.v_new | (uintptr_t)p.pre.bias_q |
                               (uintptr_t)p.pre.bias_k | (uintptr_t)p.pre.bias_v;
    if (!p.pre.norm_q && !p.pre.norm_k && (hd & 15) == 0 && hd <= 128 && (ptr_bits & 15) == 0 &&
        ((!rope_q && !rope_k) || p.rope.n_rot == hd)) {
        const float qscale = p.scale * LOG2E;
        const bool neox = p.rope.rope_type == 1;
        const int cpr = hd / 8;                                  // 8-dim chunks per row
        const int upr = neox ? cpr / 2 : cpr;                    // work units per row (a neox unit is two chunks)
        const int n_rows = p.n_head + (append ? 2 * p.n_kv : 0);
        const int units = n_rows * upr;
        constexpr int MAXU = 3;                                  // (32 + 8 + 8 rows) * 16 chunks / 256 threads
        if (units <= MAXU * kPrologueThreads) {
            float4 x[MAXU][4];
#pragma unroll
            for (int u = 0; u < MAXU; ++u) {
                const int unit = tid + u * kPrologueThreads;
                if (unit >= units) continue;
                const int row = unit / upr, c = unit % upr;
                const int kind = row < p.n_head ? 0 : (row < p.n_head + p.n_kv ? 1 : 2);
                const int head = kind == 0 ? row : (kind == 1 ? row - p.n_head : row - p.n_head - p.n_kv);
                const float* src = (kind == 0 ? p.q + ((size_t)b * p.n_head + head) * hd
                                              : (kind == 1 ? p.k_new : p.v_new) + ((size_t)b * p.n_kv + head) * hd);
                const float* bias0 = kind == 0 ? p.pre.bias_q : (kind == 1 ? p.pre.bias_k : p.pre.bias_v);
                const int d0 = 8 * c, d1 = neox ? d0 + hd / 2 : d0;
                x[u][0] = *reinterpret_cast<const float4*>(src + d0);
                x[u][1] = *reinterpret_cast<const float4*>(src + d0 + 4);
                if (neox) {
                    x[u][2] = *reinterpret_cast<const float4*>(src + d1);
                    x[u][3] = *reinterpret_cast<const float4*>(src + d1 + 4);
                }
                if (bias0) {
                    const float* bs = bias0 + (size_t)head * hd;
#pragma unroll
                    for (int v4 = 0; v4 < 4; ++v4) {
                        if (v4 >= 2 && !neox) continue;
                        const float4 bv = *reinterpret_cast<const float4*>(bs + (v4 < 2 ? d0 : d1) + 4 * (v4 & 1));
                        x[u][v4].x += bv.x; x[u][v4].y += bv.y; x[u][v4].z += bv.z; x[u][v4].w += bv.w;
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < MAXU; ++u) {
                const int unit = tid + u * kPrologueThreads;
                if (unit >= units) continue;
                const int row = unit / upr, c = unit % upr;
                const int kind = row < p.n_head ? 0 : (row < p.n_head + p.n_kv ? 1 : 2);
                const int head = kind == 0 ? row : (kind == 1 ? row - p.n_head : row - p.n_head - p.n_kv);
                const bool rot = kind == 0 ? rope_q : (kind == 1 ? rope_k : false);
                const int d0 = 8 * c;
                float a[8], bb[8];
                a[0] = x[u][0].x; a[1] = x[u][0].y; a[2] = x[u][0].z; a[3] = x[u][0].w;
                a[4] = x[u][1].x; a[5] = x[u][1].y; a[6] = x[u][1].z; a[7] = x[u][1].w;
                if (neox) {
                    bb[0] = x[u][2].x; bb[1] = x[u][2].y; bb[2] = x[u][2].z; bb[3] = x[u][2].w;
                    bb[4] = x[u][3].x; bb[5] = x[u][3].y; bb[6] = x[u][3].z; bb[7] = x[u][3].w;
                }
                if (rot) {
                    if (neox) {            // pair (d0 + i, d0 + i + hd/2), angle index d0 + i
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float cs = s_cos[d0 + i], sn = s_sin[d0 + i];
                            const float x0 = a[i] * cs - bb[i] * sn, x1 = a[i] * sn + bb[i] * cs;
                            a[i] = x0; bb[i] = x1;
                        }
                    } else {               // pair (d0 + 2i, d0 + 2i + 1), angle index d0/2 + i
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float cs = s_cos[d0 / 2 + i], sn = s_sin[d0 / 2 + i];
                            const float x0 = a[2 * i] * cs - a[2 * i + 1] * sn, x1 = a[2 * i] * sn + a[2 * i + 1] * cs;
                            a[2 * i] = x0; a[2 * i + 1] = x1;
                        }
                    }
                }
                const float mul = kind == 0 ? qscale : 1.f;
                __half* dst = kind == 0 ? p.q16 + ((size_t)b * p.n_head + head) * hd
                                        : reinterpret_cast<__half*>(kind == 1 ? p.kc : p.vc) + ((size_t)head * p.n_ctx + pos) * hd;
                uint4 o;
                o.x = pack_half2(a[0] * mul, a[1] * mul); o.y = pack_half2(a[2] * mul, a[3] * mul);
                o.z = pack_half2(a[4] * mul, a[5] * mul); o.w = pack_half2(a[6] * mul, a[7] * mul);
                *reinterpret_cast<uint4*>(dst + d0) = o;
                if (neox) {
                    o.x = pack_half2(bb[0] * mul, bb[1] * mul); o.y = pack_half2(bb[2] * mul, bb[3] * mul);
                    o.z = pack_half2(bb[4] * mul, bb[5] * mul); o.w = pack_half2(bb[6] * mul, bb[7] * mul);
                    *reinterpret_cast<uint4*>(dst + d0 + hd / 2) = o;
                }
            }
            return;
        }
    }
    // One warp per head row: the q rows, then (with the append) the k rows and the v rows.  The lanes walk the row's
    // pairs, so consecutive lanes touch consecutive addresses.  A warp first loads the values of all its rows of a batch
    // and only then rotates and stores them: sources and destinations may alias as far as the compiler can tell, so
    // row-by-row code would pay one global round trip per row.
    const float qs = p.scale * LOG2E;
    const int warp = tid >> 5, lane = tid & 31;
    const int half = hd / 2;
    const int rows = p.n_head + (append ? 2 * p.n_kv : 0);
    struct Row {
        int kind, head, n_rot;          // kind 0 = q, 1 = k, 2 = v
        const float* src; const float* bias; const float* nw; float rn;
    };
    auto describe = [&](int row) {
        Row r;
        r.kind = row < p.n_head ? 0 : (row < p.n_head + p.n_kv ? 1 : 2);
        r.head = r.kind == 0 ? row : (r.kind == 1 ? row - p.n_head : row - p.n_head - p.n_kv);
        const float* base = r.kind == 0 ? p.q : (r.kind == 1 ? p.k_new : p.v_new);
        const int heads = r.kind == 0 ? p.n_head : p.n_kv;
        r.src = base + ((size_t)b * heads + r.head) * hd;
        const float* bias0 = r.kind == 0 ? p.pre.bias_q : (r.kind == 1 ? p.pre.bias_k : p.pre.bias_v);
        r.bias = bias0 ? bias0 + (size_t)r.head * hd : nullptr;
        r.nw = r.kind == 0 ? p.pre.norm_q : (r.kind == 1 ? p.pre.norm_k : nullptr);
        r.rn = r.nw ? s_rn[row] : 1.f;
        const bool rot = r.kind == 0 ? rope_q : (r.kind == 1 ? rope_k : false);
        r.n_rot = rot ? p.rope.n_rot : 0;
        return r;
    };
    auto pair_of = [&](const Row& r, int pp, int& i0, int& i1) {
        if (pp < r.n_rot / 2) {
            rope_pair_index(p.rope.rope_type, pp, r.n_rot, i0, i1);
        } else {
            i0 = r.n_rot + 2 * (pp - r.n_rot / 2);
            i1 = i0 + 1;
        }
    };
    constexpr int RB = 6;            // rows in flight per warp (32 + 8 + 8 head rows over 8 warps)
    constexpr int NW = kPrologueThreads / 32;
    for (int r0 = warp; r0 < rows; r0 += NW * RB) {
        float xa[RB][2], xb[RB][2];
#pragma unroll
        for (int u = 0; u < RB; ++u) {
            const int row = r0 + u * NW;
            if (row >= rows) continue;
            const Row r = describe(row);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int pp = lane + 32 * j;
                if (pp >= half) continue;
                int i0, i1;
                pair_of(r, pp, i0, i1);
                xa[u][j] = pre_value(r.src, r.bias, r.nw, r.rn, i0);
                xb[u][j] = pre_value(r.src, r.bias, r.nw, r.rn, i1);
            }
        }
#pragma unroll
        for (int u = 0; u < RB; ++u) {
            const int row = r0 + u * NW;
            if (row >= rows) continue;
            const Row r = describe(row);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int pp = lane + 32 * j;
                if (pp >= half) continue;
                int i0, i1;
                pair_of(r, pp, i0, i1);
                float x0 = xa[u][j], x1 = xb[u][j];
                if (pp < r.n_rot / 2) {
                    x0 = xa[u][j] * s_cos[pp] - xb[u][j] * s_sin[pp];
                    x1 = xa[u][j] * s_sin[pp] + xb[u][j] * s_cos[pp];
                }
                if (r.kind == 0) {
                    __half* dst = p.q16 + ((size_t)b * p.n_head + r.head) * hd;
                    dst[i0] = __float2half_rn(x0 * qs);
                    dst[i1] = __float2half_rn(x1 * qs);
                } else {
                    uint16_t* dst = (r.kind == 1 ? p.kc : p.vc) + ((size_t)r.head * p.n_ctx + pos) * hd;
                    dst[i0] = __half_as_ushort(__float2half_rn(x0));
                    dst[i1] = __half_as_ushort(__float2half_rn(x1));
                }
            }
        }
    }
}

} // namespace

cudaError_t launch_rope(float* x, int rows, int head_dim, const RopeArgs& r, int n_past, int heads,
                        const int* d_pos, cudaStream_t stream, unsigned long long* launches) {
    if (rows <= 0) return cudaSuccess;
    const int grid = (rows + kRopeRows - 1) / kRopeRows;
    rope_kernel<<<grid, kRopeThreads, 0, stream>>>(x, rows, head_dim, r, n_past, heads > 0 ? heads : 1, d_pos);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

cudaError_t launch_kv_store(uint16_t* kc, uint16_t* vc, const float* k, const float* v, int heads, int head_dim,
                            int n_ctx, int pos_base, int batch, const int* d_pos, cudaStream_t stream,
                            unsigned long long* launches) {
    kv_store_kernel<<<batch * heads, 128, 0, stream>>>(kc, vc, k, v, heads, head_dim, n_ctx, pos_base, d_pos);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

cudaError_t launch_kv_shift(uint16_t* kc, uint16_t* vc, int n_layer, int n_kv, int head_dim, int n_ctx, int n_keep,
                            int shift, cudaStream_t stream, unsigned long long* launches) {
    dim3 grid(2, n_kv, n_layer);
    kv_shift_kernel<<<grid, kShiftThreads, 0, stream>>>(kc, vc, n_kv, head_dim, n_ctx, n_keep, shift);
    if (launches) *launches += 1;
    return cudaGetLastError();
}

cudaError_t launch_prefill_prologue(const PrefillArgs& a, cudaStream_t stream, unsigned long long* launches) {
    const cudaError_t e = launch_dependent(prefill_prologue_kernel, dim3(a.batch), kPrologueThreads, 0, stream, 1, a);
    if (launches) *launches += 1;
    return e;
}

} // namespace oattn
