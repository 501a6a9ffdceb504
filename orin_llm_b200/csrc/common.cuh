// Shared device helpers of the sm_100a attention kernels.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

namespace oattn {

constexpr float LOG2E = 1.4426950408889634f;

struct RopeArgs {
    int rope_type;              // 0 = normal pairs (2i, 2i+1), 1 = neox pairs (i, i + n_rot/2)
    int n_rot;
    float theta;
    const float* freq_factors;  // device, n_rot/2 floats or nullptr
};

// Optional step in front of RoPE (src/model_cpu.cpp:258-274, src/model_gpu.cu:372-377): bias add on q/k/v, then a
// per-head RMSNorm of q and k rows with a [head_dim] weight.  All pointers device, any of them may be nullptr.
struct PreArgs {
    const float* bias_q = nullptr;   // [n_head * head_dim]
    const float* bias_k = nullptr;   // [n_kv * head_dim]
    const float* bias_v = nullptr;   // [n_kv * head_dim]
    const float* norm_q = nullptr;   // [head_dim]
    const float* norm_k = nullptr;   // [head_dim]
    float eps = 0.f;
};

// 1 / sqrt(mean((x + bias)^2) + eps) of one head row, computed by a full warp (rms_norm, src/model_cpu.cpp:13-18;
// fp32 here, the CPU code accumulates in double).
__device__ __forceinline__ float warp_row_rnorm(const float* x, const float* bias, int hd, float eps, int lane) {
    float ss = 0.f;
    for (int i = lane; i < hd; i += 32) {
        const float v = x[i] + (bias ? bias[i] : 0.f);
        ss = fmaf(v, v, ss);
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    return 1.0f / sqrtf(ss / (float)hd + eps);
}

// Element i of a head row after bias and norm: (x[i] + bias[i]) * r * w[i].
__device__ __forceinline__ float pre_value(const float* x, const float* bias, const float* w, float r, int i) {
    float v = x[i];
    if (bias) v += bias[i];
    if (w) v = v * r * w[i];
    return v;
}

// ---- RoPE arithmetic -----------------------------------------------------------------------
// Frequency of pair i exactly as the reference's CPU backend evaluates it
// (src/model_cpu.cpp:182-183, 195-196): exponent -2i/n_rot rounded to fp32, theta^e rounded to
// fp32, then an fp32 divide by the optional factor.  The power goes through double so that the
// fp32 result is correctly rounded, which is what the host libm delivers; fast-math __powf
// (src/kernels.cu:1631) drifts by several ulp and the error is multiplied by the position.
__device__ __forceinline__ float rope_freq(int pair, int n_rot, float theta, const float* freq_factors) {
    const float e = (-2.0f * (float)pair) / (float)n_rot;
    // theta^e = 2^(e * log2(theta)) in double: cheaper than a double pow, and the double result is within ~1e-15
    // relative, so its fp32 rounding is the correctly rounded power (as the host powf gives) in all but a
    // vanishing fraction of cases
    float freq = (float)exp2((double)e * log2((double)theta));
    if (freq_factors) freq = __fdiv_rn(freq, freq_factors[pair]);
    return freq;
}

// cos/sin of pos*freq with the accurate (range-reduced) single-precision routines.
__device__ __forceinline__ void rope_cs(int pos, float freq, float& c, float& s) {
    const float ang = __fmul_rn((float)pos, freq);
    sincosf(ang, &s, &c);
}

// The two element indices that pair `pair` touches inside a head row.
__device__ __forceinline__ void rope_pair_index(int rope_type, int pair, int n_rot, int& i0, int& i1) {
    if (rope_type == 1) { i0 = pair; i1 = pair + n_rot / 2; }
    else                { i0 = 2 * pair; i1 = 2 * pair + 1; }
}

// Rotates (optionally) one fp32 head row and writes it as fp16 through `store(elem, value)`.  Before the rotation
// the row gets its bias and per-head RMSNorm (`bias`, `nw` may be nullptr; `rn` is the row's 1/rms from
// warp_row_rnorm when nw is set).
template <typename Store>
__device__ __forceinline__ void rope_row_to_half(const float* src, const float* bias, const float* nw, float rn, int hd,
                                                 bool rotate, const RopeArgs& r, const float* s_cos, const float* s_sin,
                                                 int lane_id, int lanes, Store store) {
    const int n_rot = rotate ? r.n_rot : 0;
    for (int pp = lane_id; pp < hd / 2; pp += lanes) {
        int i0, i1;
        float x0, x1;
        if (pp < n_rot / 2) {
            rope_pair_index(r.rope_type, pp, n_rot, i0, i1);
            const float a = pre_value(src, bias, nw, rn, i0), b = pre_value(src, bias, nw, rn, i1);
            const float c = s_cos[pp], s = s_sin[pp];
            x0 = a * c - b * s;
            x1 = a * s + b * c;
        } else {
            i0 = n_rot + 2 * (pp - n_rot / 2);
            i1 = i0 + 1;
            x0 = pre_value(src, bias, nw, rn, i0);
            x1 = pre_value(src, bias, nw, rn, i1);
        }
        store(i0, x0);
        store(i1, x1);
    }
}

// ---- async copy / ldmatrix / mma -----------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// 16-byte global->shared copy; src_bytes = 0 writes zeros instead (used for rows past the
// valid length so that never-written cache rows cannot inject NaN into P*V).
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
// Hint: bring the 128-byte line at `p` into L2.  No destination, nothing to wait for.
__device__ __forceinline__ void l2_prefetch_line(const void* p) { asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p)); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

// D(16x8, fp32) += A(16x16, fp16, row) * B(16x8, fp16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// ---- programmatic dependent launch -----------------------------------------------------------
// A kernel launched with the programmatic-stream-serialization attribute may start while the preceding kernel of the
// stream is still running.  pdl_wait() blocks until every preceding kernel has completed and its writes are
// visible (a no-op for an ordinary launch); pdl_trigger() lets the next kernel of the stream begin launching.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

// ---- q8_1 activation form of the attention output --------------------------------------------------------
// What the reference's quantize_q8_1_k (src/kernels.cu:136-145) makes of a vector: per group of 32 consecutive
// values d = max|x| / 127 and q = round-half-away(x / d), q = 0 for an all-zero group; int8 values in `qs`, one fp32
// d per group in `scales` (the layout its GEMV kernels read, src/kernels.cu:1763-1776).  Called by a full warp whose
// lanes hold the 32 values of one group; `flat` is the value's index in the whole vector.  IEEE division.
__device__ __forceinline__ void store_q8_group(float x, size_t flat, int8_t* qs, float* scales) {
    float amax = fabsf(x);
#pragma unroll
    for (int off = 16; off; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const float d = __fdiv_rn(amax, 127.0f);
    qs[flat] = amax == 0.0f ? (int8_t)0 : (int8_t)roundf(__fdiv_rn(x, d));
    if ((threadIdx.x & 31) == 0) scales[flat >> 5] = d;
}

// Byte offset of (row, 16-byte chunk) inside a tile whose rows are ROW_BYTES wide, with the
// chunk index XOR-ed by the row so that the 8 rows one ldmatrix phase touches fall in 8
// different bank groups.
template <int ROW_BYTES>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
    return (uint32_t)(row * ROW_BYTES + ((chunk ^ (row & 7)) << 4));
}

} // namespace oattn
