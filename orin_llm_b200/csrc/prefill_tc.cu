// Chunked-prefill causal GQA attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// Stands in for flash_attention_prefill_mma_k (src/kernels.cu:1351-1568).  Query token t of the
// chunk sees cache rows 0..n_past+t.  q16 holds the chunk's queries already rotated, multiplied by
// scale*log2(e) and converted to fp16 (prefill_prologue_kernel), so the score matrix is in the
// log2 domain and the softmax is exp2.
//
// One CTA = one 128-row query tile of ONE kv head; a row is a (token, head-in-group) pair, row
// R -> token t0 + R/G, head kvh*G + R%G (G = n_head/n_kv), so a single pass over the kv head's K/V rows
// serves all G query heads of floor(128/G) tokens (when G does not divide 128 the last few tile rows are
// zero and unused).  The KV sequence is walked in blocks of
// 128 rows.  384 threads = three warpgroups (warps 2 and 3 only hold the place that makes the softmax teams whole warpgroups,
// so that registers can be moved to them); three roles:
//   warp 0   (one lane)  TMA producer: Q tile once, then 128-row K blocks (three-stage ring) and V blocks
//                        (two-stage ring) with cp.async.bulk.tensor, 128-byte swizzle, no multicast; rows
//                        past the chunk are outside the tensor map and arrive as zeros
//   warp 1   (all lanes) tcgen05.mma issuer: S_j = Q K_j^T (M128 N128 K16 x8, both operands from shared
//                        memory) into one of THREE TMEM score buffers, so that the scores of blocks j+1 and
//                        j+2 are already there while block j is in the softmax; O += P_j V_j with P read
//                        straight from TMEM (it overwrites the first 64 columns of its own score buffer as
//                        packed fp16 pairs) and V as MN-major B operand from shared memory, into the one
//                        TMEM accumulator.  The warp walks its loop with all 32 lanes and one elected lane
//                        executes the tcgen05 instructions: eight MMAs and the commit of a group in one
//                        predicated block, descriptors built once.  The commit behind S_j also frees K ring
//                        stage j % 3, the commit behind P_j V_j also frees V ring stage j & 1.
//   warps 4-7, 8-11      two softmax teams, one thread per row each, taking alternate KV blocks.  Per block:
//                        tcgen05.ld of the 128-column score row, causal mask, row max; the reference max is a
//                        single chain over all blocks, handed from team to team through shared memory (block
//                        j continues from what the other team published for block j-1); lazy rescale of O
//                        (only when the max grows by more than 2^4, after the previous P V has completed);
//                        exp2; fp16 P stored back to TMEM (tcgen05.st).  Each thread keeps its own partial
//                        row sum; the two are added at the end and O/l goes to global memory.
// TMEM: 3 x 128 score columns + 128 accumulator columns = 512.
//
// What bounds the loop (measured with clock stamps and with a stand-alone issue-rate kernel): an M128 N128 K16 MMA
// takes the tensor pipe 64 cycles, 1024 per KV block, whether its A operand comes from shared memory or from TMEM and
// whatever TMA copies, TMEM loads/stores and exp2 work run beside it.  But the pipe's queue is shallow: the issuing warp
// sits inside an MMA group for about as long as the group runs, and every cycle it spends between two groups (barrier
// waits, fences, address arithmetic) is a cycle the pipe idles -- hence the warp-uniform issue, the single election per
// group and the non-blocking look at the next barriers before a group is issued.  With that the loop is bound by the
// softmax side: one KV block takes a team about 2500-3000 cycles from scores ready to P stored, two teams alternate,
// and the score buffer of block j is tied up from S_j until P_j V_j has run; about 1650 cycles per block result.
// (Scores two blocks ahead in buffers of their own, P in separate buffers: measured, slower -- the extra hand-over
// and the wait for the P buffer lengthen the softmax, which is the bound.)
//
// Every mbarrier wait is bounded: after about a second without progress the kernel raises an abort
// flag, every role leaves its loop, outstanding copies and MMAs are drained (bounded again), TMEM is
// released and a non-zero status word is left for the host.
#include <cuda.h>

#include "attn_internal.h"

namespace oattn {

namespace {

constexpr int kThreads = 384;                   // three warpgroups: {TMA, MMA, two idle warps}, softmax team 0, softmax team 1
constexpr int kFirstSoftmaxWarp = 4;
constexpr int kRegsService = 104, kRegsSoftmax = 200;   // per-thread register budgets after the set-up (setmaxnreg)
constexpr int BM = 128, BN = 128, HD = 128;
constexpr int SLAB = 128 * 128;                 // bytes of one 128-row x 64-element fp16 slab
constexpr int TILE = 2 * SLAB;                  // a 128 x 128 fp16 tile = two slabs
constexpr int OFF_Q = 0;
constexpr int NKS = 3, NVS = 2;                 // K and V ring depths
constexpr int NSB = 3;                          // score buffers in TMEM
constexpr int OFF_K = OFF_Q + TILE;
constexpr int OFF_V = OFF_K + NKS * TILE;
constexpr int OFF_BAR = OFF_V + NVS * TILE;
constexpr int OFF_MREF = OFF_BAR + 256;         // float [2][128]: reference max published per block parity
constexpr int OFF_MX = OFF_MREF + 1024;         // float2 [2 teams][128 rows]: (m, l) exchanged at the end
constexpr int SMEM_BYTES = OFF_MX + 2048 + 1024;   // + slack for 1024-byte alignment
static_assert(SMEM_BYTES <= 232448, "shared memory budget");
constexpr long long kWaitCycles = 2000000000LL;    // ~1 s
constexpr long long kDrainCycles = 200000000LL;    // ~0.1 s
constexpr float kRescaleThreshold = 4.0f;          // log2 units: P stays below 2^4 relative to the reference max

enum Bar { Q_FULL = 0, K_FULL = 1, V_FULL = K_FULL + NKS, S_FULL = V_FULL + NVS, P_FULL = S_FULL + NSB, PV_DONE = P_FULL + NSB,
           MREF = PV_DONE + 2, DRAIN = MREF + 2, XCH = DRAIN + 1, ALL_DONE = XCH + 1, NBAR = ALL_DONE + 1 };
// K block j lives in ring stage j % NKS and its scores in buffer j % NSB: with NKS == NSB the commit that publishes the
// scores (S_FULL) is also the moment the K stage is free again.  The same holds for V stage j % NVS and PV_DONE[j & 1].
static_assert(NKS == NSB && NVS == 2, "the producer waits on S_FULL / PV_DONE for free ring stages");
static_assert(NBAR * 8 + 16 <= 256, "barrier block");

#ifndef OATTN_TC_POLY
#define OATTN_TC_POLY 0
#endif
#ifndef OATTN_TC_FAST
#define OATTN_TC_FAST 0
#endif

#ifdef OATTN_TC_TRACE
// Debug build only: per-event clock stamps of CTA (0,0).  [role][event][block]
__device__ long long g_trace[3][8][128];
#define TRACE(role, ev, blk) do { if (blockIdx.x == 0 && blockIdx.y == 0 && (blk) < 128) g_trace[role][ev][blk] = clock64(); } while (0)
#else
#define TRACE(role, ev, blk) do { } while (0)
#endif

struct TcArgs {
    float* out;
    uint8_t* out_mmq;      // optional block_q8_1_mmq form of the output (src/kernels.cu:147-155), [head][batch] blocks
    int mmq_ds4;
    int* status;
    int n_head, n_kv, n_past, batch, G, TQ;   // TQ = floor(128 / G) tokens per tile
    int out_tma;           // the fp32 output leaves through shared memory and bulk tensor stores (tmO is valid)
};

// ---- PTX wrappers ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    // the third operand is a suspend-time hint: the thread sleeps in hardware until the phase completes
    // (or the hint runs out) instead of taking issue slots from the warps that have work
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(1000000u) : "memory");
    return ok != 0;
}
// Non-blocking look at a phase (no suspend): used to take a barrier's latency off the MMA warp's critical path.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the abort flag is up or the time limit passed (and raises the flag).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* s_abort) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    int spins = 0;
    while (!mbar_try(bar, parity)) {
        if ((++spins & 31) == 0) {
            if (*s_abort) return false;
            if (clock64() - t0 > kWaitCycles) { *s_abort = 1; return false; }
        }
    }
    return true;
}
// Teardown wait: ignores the abort flag, shorter limit.
__device__ __forceinline__ void mbar_drain(uint32_t bar, uint32_t parity) {
    const long long t0 = clock64();
    while (!mbar_try(bar, parity)) {
        if (clock64() - t0 > kDrainCycles) break;
    }
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, int c0, int c1, int c2, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];\n"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// The MMA warp runs its loop with all 32 lanes: warp-uniform control flow lets the compiler keep the descriptor arithmetic
// on the uniform datapath.  (Issued from one lane inside a divergent branch, every MMA cost the lane about twice the 64
// cycles the tensor pipe needs for it.)  The pipe's queue is shallow: it hides only about a hundred cycles between two
// groups of MMAs, so the instruction count of this warp is what decides whether the pipe starves.  Hence one election
// per group of eight MMAs, with the group's commits in the same predicated block.  With a full mask the election is the
// same lane every time, which tcgen05.commit relies on (it tracks the MMAs of the thread that executes it).
// S = Q K^T: eight K16 steps, D[tmem] = A[smem desc] * B[smem desc], fp16 in, fp32 out, M128 N128; the first step
// overwrites.  Then commit to bar_a.
__device__ __forceinline__ void tc_group_ss(uint32_t d_tmem, const uint64_t (&a)[8], const uint64_t (&b)[8], uint32_t idesc,
                                            uint32_t bar_a) {
    asm volatile("{\n.reg .pred e, pt, pf;\n"
                 "elect.sync _|e, 0xffffffff;\n"
                 "setp.eq.u32 pt, %2, 0;\n"
                 "setp.ne.u32 pf, %2, 0;\n"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %5, %13, %1, {%2, %2, %2, %2}, pf;\n"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %6, %14, %1, {%2, %2, %2, %2}, pt;\n"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %7, %15, %1, {%2, %2, %2, %2}, pt;\n"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %8, %16, %1, {%2, %2, %2, %2}, pt;\n"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %9, %17, %1, {%2, %2, %2, %2}, pt;\n"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %10, %18, %1, {%2, %2, %2, %2}, pt;\n"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %11, %19, %1, {%2, %2, %2, %2}, pt;\n"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %12, %20, %1, {%2, %2, %2, %2}, pt;\n"
                 "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%3];\n}\n"
                 ::"r"(d_tmem), "r"(idesc), "r"(0u), "r"(bar_a), "r"(0u),
                   "l"(a[0]), "l"(a[1]), "l"(a[2]), "l"(a[3]), "l"(a[4]), "l"(a[5]), "l"(a[6]), "l"(a[7]),
                   "l"(b[0]), "l"(b[1]), "l"(b[2]), "l"(b[3]), "l"(b[4]), "l"(b[5]), "l"(b[6]), "l"(b[7]) : "memory");
}
// O (+)= P V: eight K16 steps with A from TMEM (128 lanes x 8 columns of packed fp16 pairs per step) and B[smem desc];
// the first step accumulates only if `acc0`.  Then commit to bar_a.
__device__ __forceinline__ void tc_group_ts(uint32_t d_tmem, uint32_t a_tmem, const uint64_t (&b)[8], uint32_t idesc, uint32_t acc0,
                                            uint32_t bar_a) {
    asm volatile("{\n.reg .pred e, pt, p0;\n.reg .b32 t;\n"
                 "elect.sync _|e, 0xffffffff;\n"
                 "setp.eq.u32 pt, %2, 0;\n"
                 "setp.ne.u32 p0, %4, 0;\n"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%5], %6, %1, {%2, %2, %2, %2}, p0;\n"
                 "add.u32 t, %5, 8;\n"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [t], %7, %1, {%2, %2, %2, %2}, pt;\n"
                 "add.u32 t, %5, 16;\n"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [t], %8, %1, {%2, %2, %2, %2}, pt;\n"
                 "add.u32 t, %5, 24;\n"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [t], %9, %1, {%2, %2, %2, %2}, pt;\n"
                 "add.u32 t, %5, 32;\n"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [t], %10, %1, {%2, %2, %2, %2}, pt;\n"
                 "add.u32 t, %5, 40;\n"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [t], %11, %1, {%2, %2, %2, %2}, pt;\n"
                 "add.u32 t, %5, 48;\n"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [t], %12, %1, {%2, %2, %2, %2}, pt;\n"
                 "add.u32 t, %5, 56;\n"
                 "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [t], %13, %1, {%2, %2, %2, %2}, pt;\n"
                 "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%3];\n}\n"
                 ::"r"(d_tmem), "r"(idesc), "r"(0u), "r"(bar_a), "r"(acc0), "r"(a_tmem),
                   "l"(b[0]), "l"(b[1]), "l"(b[2]), "l"(b[3]), "l"(b[4]), "l"(b[5]), "l"(b[6]), "l"(b[7]) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("{\n.reg .pred e;\nelect.sync _|e, 0xffffffff;\n"
                 "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}\n" ::"r"(bar) : "memory");
}
// Wait of the MMA warp: every lane polls (one warp instruction), no vote.  A time-out raises the abort flag and returns;
// the warp's loop looks at the flag once per block, with a vote, so all lanes leave together.
__device__ __forceinline__ void mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* s_abort) {
    if (mbar_try(bar, parity)) return;
    const long long t0 = clock64();
    int spins = 0;
    while (!mbar_try(bar, parity)) {
        if ((++spins & 31) == 0) {
            if (*s_abort) return;
            if (clock64() - t0 > kWaitCycles) { *s_abort = 1; return; }
        }
    }
}
// TMEM -> registers.  The load and its wait sit in ONE asm statement: the destination registers are
// written asynchronously, and nothing (not even a compiler-generated register move) may touch them before
// tcgen05.wait::ld has returned.  The outputs are early-clobber so that the address register can never be
// allocated on top of a destination register.  One load per statement: a second load issued before the wait
// would read its address while the first is still writing registers.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                 "tcgen05.wait::ld.sync.aligned;\n"
                 : "=&f"(v[0]), "=&f"(v[1]), "=&f"(v[2]), "=&f"(v[3]), "=&f"(v[4]), "=&f"(v[5]), "=&f"(v[6]), "=&f"(v[7]), "=&f"(v[8]), "=&f"(v[9]), "=&f"(v[10]), "=&f"(v[11]), "=&f"(v[12]), "=&f"(v[13]), "=&f"(v[14]), "=&f"(v[15]), "=&f"(v[16]), "=&f"(v[17]), "=&f"(v[18]), "=&f"(v[19]), "=&f"(v[20]), "=&f"(v[21]), "=&f"(v[22]), "=&f"(v[23]), "=&f"(v[24]), "=&f"(v[25]), "=&f"(v[26]), "=&f"(v[27]), "=&f"(v[28]), "=&f"(v[29]), "=&f"(v[30]), "=&f"(v[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
                 ::"r"(taddr),
                   "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
                   "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
                   "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                   "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
                   "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
                   "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
                   "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
                   "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
                 : "memory");
}

__device__ __forceinline__ unsigned long long f32x2_pack(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f32x2_unpack(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long f32x2_add(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// 2^x without the special-function unit: x = n + f with n = round(x), f in [-0.5, 0.5]; 2^f from a
// degree-3 polynomial (relative error 7.7e-5, well below the fp16 rounding of P); 2^n by adding n to the
// exponent field.  Inputs below -125 (including -inf for masked scores) give ~2^-125, which becomes 0 in fp16.
__device__ __forceinline__ float exp2_poly(float x) {
    x = fmaxf(x, -125.f);
    const float fi = x + 12582912.f;        // 1.5 * 2^23: n lands in the low mantissa bits
    const float f = x - (fi - 12582912.f);
    const float q = fmaf(fmaf(fmaf(0.05508868f, f, 0.24260405f), f, 0.69327624f), f, 0.99992894f);
    return __int_as_float(__float_as_int(q) + (__float_as_int(fi) << 23));
}

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1 (sm_100).
// K-major operand (rows 128 B apart, 8-row groups 1024 B apart): LBO field 1, SBO 1024 B.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// MN-major operand: 64 elements contiguous along N, next 64 at LBO = one slab; 8-row K groups 1024 B apart.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(SLAB >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor: fp32 accumulate, fp16 A and B, A K-major, N = 128, M = 128; bit 16 = B is MN-major.
constexpr uint32_t IDESC_S = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
constexpr uint32_t IDESC_PV = IDESC_S | (1u << 16);

__global__ void __launch_bounds__(kThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const TcArgs p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t sbase = (raw + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (sbase - raw);
    const uint32_t bars = sbase + OFF_BAR;
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + OFF_BAR + NBAR * 8 + 8);
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + OFF_BAR + NBAR * 8);
    auto bar = [&](int i) { return bars + 8u * i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.y;
    const int tile = gridDim.x - 1 - blockIdx.x;          // latest (longest) tiles first
    const int t0 = tile * p.TQ;
    const int ntok = min(p.TQ, p.batch - t0);
    const int kv_end = p.n_past + t0 + ntok;              // rows any query of this tile may see
    const int nb = (kv_end + BN - 1) / BN;

    if (tid == 0) {
        mbar_init(bar(Q_FULL), 1);
        for (int s = 0; s < NKS; ++s) mbar_init(bar(K_FULL + s), 1);
        for (int s = 0; s < NVS; ++s) mbar_init(bar(V_FULL + s), 1);
        for (int s = 0; s < NSB; ++s) { mbar_init(bar(S_FULL + s), 1); mbar_init(bar(P_FULL + s), 4); }
        for (int s = 0; s < 2; ++s) { mbar_init(bar(PV_DONE + s), 1); mbar_init(bar(MREF + s), 4); }
        mbar_init(bar(XCH), 256);
        mbar_init(bar(DRAIN), 1);
        mbar_init(bar(ALL_DONE), 1);
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    // Tile rows the TMA box does not cover (G * TQ < 128) are zeroed once; inside a slab row r is the 128 bytes at
    // r * 128, whatever the swizzle.
    for (int i = tid; i < (BM - p.G * p.TQ) * 16; i += kThreads) {
        const int r = p.G * p.TQ + i / 16, c = i % 16;
        *reinterpret_cast<uint4*>(smem + OFF_Q + (c >> 3) * SLAB + r * 128 + (c & 7) * 16) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(s_tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;
    // Up to here only this CTA's shared memory and TMEM were touched, so with a programmatic dependent launch all of it
    // overlaps the tail of the prologue kernel.  From here on the kernel reads what that kernel wrote (the fp16 queries,
    // the appended K/V rows) and writes the output: wait for everything before it in the stream to complete.
    pdl_trigger();
    pdl_wait();
    const uint32_t TM_S = tmem, TM_O = tmem + NSB * BN;   // score buffer b at TM_S + 128 b, the accumulator behind them

    // The kernel is compiled for 384 threads x 168 registers.  The warpgroup of the TMA and MMA warps needs fewer and hands
    // the difference to the two softmax warpgroups, whose threads keep a 128-value score row in registers.  Each
    // setmaxnreg sits at the head of the code it governs.
    if (warp < kFirstSoftmaxWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(kRegsService));
    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            bool ok = true;
            int k_issued[NKS] = {}, v_issued[NVS] = {};
            mbar_expect_tx(bar(Q_FULL), 2 * 128 * p.G * p.TQ);       // two slabs of G*TQ rows of 128 bytes
            tma_load_3d(sbase + OFF_Q, &tmQ, 0, kvh * p.G, t0, bar(Q_FULL));
            tma_load_3d(sbase + OFF_Q + SLAB, &tmQ, 64, kvh * p.G, t0, bar(Q_FULL));
            auto load_k = [&](int j) {
                const int s = j % NKS;
                if (j >= NKS) ok = mbar_wait(bar(S_FULL + s), ((j / NKS) - 1) & 1, s_abort);     // S_(j-NKS) done: stage free
                if (!ok) return;
                mbar_expect_tx(bar(K_FULL + s), TILE);
                tma_load_3d(sbase + OFF_K + s * TILE, &tmK, 0, j * BN, kvh, bar(K_FULL + s));
                tma_load_3d(sbase + OFF_K + s * TILE + SLAB, &tmK, 64, j * BN, kvh, bar(K_FULL + s));
                ++k_issued[s];
            };
            auto load_v = [&](int j) {
                const int s = j % NVS;
                if (j >= NVS) ok = mbar_wait(bar(PV_DONE + s), ((j / NVS) - 1) & 1, s_abort);    // P V of block j-2 done: stage free
                if (!ok) return;
                mbar_expect_tx(bar(V_FULL + s), TILE);
                tma_load_3d(sbase + OFF_V + s * TILE, &tmV, 0, j * BN, kvh, bar(V_FULL + s));
                tma_load_3d(sbase + OFF_V + s * TILE + SLAB, &tmV, 64, j * BN, kvh, bar(V_FULL + s));
                ++v_issued[s];
            };
            // consumption order of the MMA warp: K_0..K_2, then V_j, K_(j+3)
            for (int j = 0; j < NSB && j < nb && ok; ++j) load_k(j);
            for (int j = 0; j < nb && ok; ++j) {
                load_v(j);
                if (ok && j + NSB < nb) load_k(j + NSB);
            }
            if (*s_abort) {
                // make sure no copy is still writing this CTA's shared memory when it exits
                mbar_drain(bar(Q_FULL), 0);
                for (int s = 0; s < NKS; ++s)
                    if (k_issued[s]) mbar_drain(bar(K_FULL + s), (k_issued[s] - 1) & 1);
                for (int s = 0; s < NVS; ++s)
                    if (v_issued[s]) mbar_drain(bar(V_FULL + s), (v_issued[s] - 1) & 1);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (all lanes walk the loop)
        mbar_wait_warp(bar(Q_FULL), 0, s_abort);
        // Descriptors are built once: per k-step for Q, per ring stage and k-step for K and V (the offsets are added to the
        // 14-bit address field, in 16-byte units; it cannot carry out of the field).
        uint64_t dQ[8], dK0[8], dV0[8];
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
            const uint32_t off = (uint32_t)((kk >> 2) * SLAB + (kk & 3) * 32);
            dQ[kk] = desc_kmajor(sbase + OFF_Q + off);
            dK0[kk] = desc_kmajor(sbase + OFF_K + off);
            dV0[kk] = desc_mnmajor(sbase + OFF_V + kk * 2048);       // V: 16 rows of 128 B per k-step
        }
        // S_j = Q K_j^T into score buffer s = j % NSB, K from ring stage s.  The commit publishes the scores and frees the
        // K stage.
        auto issue_s = [&](int j, int s) {
            if (lane == 0) TRACE(0, 0, j);
            uint64_t dKs[8];
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) dKs[kk] = dK0[kk] + (uint64_t)((s * TILE) >> 4);
            tc_group_ss(TM_S + s * BN, dQ, dKs, IDESC_S, bar(S_FULL + s));
        };
        tc_fence_after();
        for (int j = 0; j < NSB && j < nb; ++j) {
            mbar_wait_warp(bar(K_FULL + j), 0, s_abort);
            issue_s(j, j);
        }
        // An MMA group keeps this warp inside its issue for about as long as the group runs (the pipe's queue is shallow),
        // and whatever the warp does between two groups is time the tensor pipe idles.  So the barriers a group needs are
        // looked at (non-blocking) before the group in front of it is issued: their latency passes while that group
        // runs, and only a barrier that really is late costs a wait.
        int b = 0;                      // j % NSB
        uint32_t ph3 = 0, ph2 = 0;      // (j / NSB) & 1, (j / 2) & 1
        bool rdy_p = false, rdy_v = false;
        for (int j = 0; j < nb; ++j) {
            if ((j & 3) == 0 && __any_sync(0xffffffffu, *s_abort != 0)) break;      // all lanes leave together
            const int sv = j & 1;
            if (!rdy_p) mbar_wait_warp(bar(P_FULL + b), ph3, s_abort);
            if (lane == 0) TRACE(0, 1, j);
            if (!rdy_v) mbar_wait_warp(bar(V_FULL + sv), ph2, s_abort);
            if (lane == 0) TRACE(0, 2, j);
            tc_fence_after();
            // K block j + NSB arrives in the ring stage b, in that stage's next phase
            const bool do_s = j + NSB < nb;
            const bool rdy_k = do_s && mbar_test(bar(K_FULL + b), ph3 ^ 1u);
            uint64_t dVs[8];
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) dVs[kk] = dV0[kk] + (uint64_t)((sv * TILE) >> 4);
            // commit: accumulator complete up to block j; V stage sv free
            tc_group_ts(TM_O, TM_S + b * BN, dVs, IDESC_PV, j > 0 ? 1u : 0u, bar(PV_DONE + sv));
            if (lane == 0) TRACE(0, 3, j);
            // what the next block's P V needs, looked at before the S group below is issued
            const int bn = (b + 1 == NSB) ? 0 : b + 1;
            const uint32_t ph3n = (b + 1 == NSB) ? ph3 ^ 1u : ph3, ph2n = ph2 ^ (uint32_t)sv;
            rdy_p = rdy_v = false;
            if (j + 1 < nb) {
                rdy_p = mbar_test(bar(P_FULL + bn), ph3n);
                rdy_v = mbar_test(bar(V_FULL + (sv ^ 1)), ph2n);
            }
            // score buffer b is free again once P_j V_j has been issued (the tensor pipe runs in order)
            if (do_s) {
                if (!rdy_k) mbar_wait_warp(bar(K_FULL + b), ph3 ^ 1u, s_abort);
                issue_s(j + NSB, b);
            }
            b = bn; ph3 = ph3n; ph2 = ph2n;
        }
        const bool ok = !__any_sync(0xffffffffu, *s_abort != 0);
        if (ok) tc_commit(bar(ALL_DONE));
        if (!ok) {
            tc_commit(bar(DRAIN));
            mbar_drain(bar(DRAIN), 0);
        }
        __syncwarp();
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(kRegsSoftmax));
        // ---------------------------------------------------------------- softmax + epilogue
        const int quad = warp & 3;                          // TMEM lane quadrant this warp may access
        const int team = (warp - kFirstSoftmaxWarp) >> 2;   // 0: even KV blocks, 1: odd KV blocks
        const int row = quad * 32 + lane;
        const int tok = row / p.G, hg = row - tok * p.G;
        const int tglob = t0 + tok;
        const bool valid = tok < ntok;
        const int vis = p.n_past + tglob;                   // last visible cache row
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        const uint32_t to = TM_O + lane_addr;               // the accumulator row of this thread
        float* s_mref = reinterpret_cast<float*>(smem + OFF_MREF);
        float m_l = -CUDART_INF_F, l = 0.f;                 // this thread's partial row sum and the reference max it is relative to
        bool ok = true;

        for (int j = team; j < nb && ok; j += 2) {
            const int b = j % NSB;
            const uint32_t ts = TM_S + lane_addr + b * BN;  // score buffer of this block, this thread's lane
            if (tid == 128 || tid == 256) TRACE(1 + team, 0, j);
            // every give-up decision is made warp-uniform: the TMEM loads and stores below are warp-collective
            ok = __all_sync(0xffffffffu, mbar_wait(bar(S_FULL + b), (j / NSB) & 1, s_abort));
            if (!ok) break;
            if (tid == 128 || tid == 256) TRACE(1 + team, 1, j);
            tc_fence_after();
            float v[128];
            tmem_ld32(ts, v);
            tmem_ld32(ts + 32, v + 32);
            tmem_ld32(ts + 64, v + 64);
            tmem_ld32(ts + 96, v + 96);
            if (tid == 128 || tid == 256) TRACE(1 + team, 2, j);
            if (j * BN + BN - 1 > p.n_past + t0) {          // block reaches past the tile's first query: mask
                const int lim = vis - j * BN;               // columns <= lim are visible
#pragma unroll
                for (int i = 0; i < 128; ++i) if (i > lim) v[i] = -CUDART_INF_F;
            }
            float mxc[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
            for (int i = 0; i < 128; i += 8) {
#pragma unroll
                for (int c = 0; c < 4; ++c) mxc[c] = max3(mxc[c], v[i + 2 * c], v[i + 2 * c + 1]);
            }
            const float mx = fmaxf(fmaxf(mxc[0], mxc[1]), fmaxf(mxc[2], mxc[3]));
            // The reference max is one chain over all blocks: block j continues from what the other team
            // published for block j-1 (slot and barrier (j-1) & 1), and publishes its own before anything else.
            float m_prev = -CUDART_INF_F;
            if (j > 0) {
                ok = __all_sync(0xffffffffu, mbar_wait(bar(MREF + ((j - 1) & 1)), ((j - 1) >> 1) & 1, s_abort));
                if (!ok) break;
                m_prev = s_mref[((j - 1) & 1) * 128 + row];
            }
            const float m_new = (m_prev == -CUDART_INF_F || mx > m_prev + kRescaleThreshold) ? fmaxf(mx, m_prev) : m_prev;
            s_mref[(j & 1) * 128 + row] = m_new;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(MREF + (j & 1)));
            // a row that is fully masked so far keeps -inf; use 0 as the exponent base then (all p = 0)
            const float m_use = (m_new == -CUDART_INF_F) ? 0.f : m_new;
            const bool need = (m_new != m_prev) && (m_prev != -CUDART_INF_F);
            if (__any_sync(0xffffffffu, need)) {
                // O must be quiescent and complete up to block j-1.  PV_DONE alternates between two barriers by
                // block parity; the score block just received proves that every P V up to j-3 has completed, and
                // P_j V_j cannot start before this thread delivers P_j, so each barrier is at most one phase
                // away from the one waited for.
                if (j >= 2) ok = mbar_wait(bar(PV_DONE + (j & 1)), ((j - 2) >> 1) & 1, s_abort);
                if (ok) ok = mbar_wait(bar(PV_DONE + ((j - 1) & 1)), ((j - 1) >> 1) & 1, s_abort);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const float alpha = need ? fast_exp2(m_prev - m_new) : 1.f;
                float o[32];
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    tmem_ld32(to + 32 * c, o);
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] *= alpha;
                    tmem_st32(to + 32 * c, o);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            }
            if (m_l != m_new) {                             // bring this thread's partial sum to the current reference
                l *= (m_l == -CUDART_INF_F) ? 0.f : fast_exp2(m_l - m_new);
                m_l = m_new;
            }
            if (tid == 128 || tid == 256) TRACE(1 + team, 3, j);
            // P (fp16 pairs) goes over the first 64 columns of this thread's own score row.
            uint32_t pk[64];
            // two-wide fp32 adds (add.f32x2) for the subtraction of the reference max and for the row sum: the loop is
            // short of issue slots, not of arithmetic
            unsigned long long l2[4] = {0ull, 0ull, 0ull, 0ull};       // four accumulators of (even, odd) partial sums
            const unsigned long long negm = f32x2_pack(-m_use, -m_use);
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                float x0, x1;
                f32x2_unpack(f32x2_add(f32x2_pack(v[2 * i], v[2 * i + 1]), negm), x0, x1);
                float p0, p1;
                if (OATTN_TC_POLY && (i % (OATTN_TC_POLY ? OATTN_TC_POLY : 1)) == OATTN_TC_POLY - 1) { p0 = exp2_poly(x0); p1 = exp2_poly(x1); }
                else { p0 = fast_exp2(x0); p1 = fast_exp2(x1); }
                l2[i & 3] = f32x2_add(l2[i & 3], f32x2_pack(p0, p1));
                pk[i] = pack_half2(p0, p1);
            }
            {
                float a0, a1, b0, b1;
                f32x2_unpack(f32x2_add(f32x2_add(l2[0], l2[1]), f32x2_add(l2[2], l2[3])), a0, a1);
                (void)b0; (void)b1;
                l += a0 + a1;
            }
            if (tid == 128 || tid == 256) TRACE(1 + team, 4, j);
            tmem_st32(ts, reinterpret_cast<const float*>(pk));
            tmem_st32(ts + 32, reinterpret_cast<const float*>(pk + 32));
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(P_FULL + b));         // one arrival per warp (the barrier counts 4)
            if (tid == 128 || tid == 256) TRACE(1 + team, 5, j);
        }
        // ---- add the two teams' row sums and write the output -----------------------------------------
        float2* s_x = reinterpret_cast<float2*>(smem + OFF_MX);
        if (ok) {
            s_x[team * 128 + row] = make_float2(m_l, l);
            mbar_arrive(bar(XCH));
            ok = mbar_wait(bar(XCH), 0, s_abort);
        }
        // the accumulator is final once every MMA of this CTA has completed (single-phase barrier, committed by
        // the MMA warp after its last P V)
        if (ok) ok = mbar_wait(bar(ALL_DONE), 0, s_abort);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc_fence_after();
            const float2 other = s_x[(1 - team) * 128 + row];
            // the reference max never decreases, so the later block's value is the final one and O is relative to it
            const float M = fmaxf(m_l, other.x);
            const float w_me = (m_l == -CUDART_INF_F) ? 0.f : fast_exp2(m_l - M);
            const float w_ot = (other.x == -CUDART_INF_F) ? 0.f : fast_exp2(other.x - M);
            const float inv = 1.f / (w_me * l + w_ot * other.y);
            // this thread writes columns [64 team, 64 team + 64) of its row
            float* dst = p.out + ((size_t)tglob * p.n_head + kvh * p.G + hg) * HD + 64 * team;
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                float a[32];
                tmem_ld32(to + 64 * team + 32 * c, a);
#pragma unroll
                for (int i = 0; i < 32; ++i) a[i] *= inv;
                if (p.out_tma) {
                    // Straight from here a warp's store would touch 32 rows, 512 bytes apart, with 16 bytes each.  The
                    // tile goes through shared memory instead (the K ring is idle now): four slabs of 32 columns, a row's
                    // 128 bytes of a slab swizzled like a tensor-map tile, and leaves as four bulk tensor stores.
                    uint8_t* rowp = smem + OFF_K + (2 * team + c) * (BM * 128) + row * 128;
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        *reinterpret_cast<float4*>(rowp + ((i ^ (row & 7)) << 4)) = make_float4(a[4 * i], a[4 * i + 1], a[4 * i + 2], a[4 * i + 3]);
                } else if (valid && p.out) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        *reinterpret_cast<float4*>(dst + 32 * c + 4 * i) = make_float4(a[4 * i], a[4 * i + 1], a[4 * i + 2], a[4 * i + 3]);
                }
                if (valid && p.out_mmq) {
                    // The 32 values are one quantisation group of the 128-value block of (head, token): what
                    // quantize_mmq_q8_1_k (src/kernels.cu:160-205) computes with a shuffle over eight lanes is a
                    // reduction over this thread's registers here.
                    float amax = 0.f, sum = 0.f;
#pragma unroll
                    for (int i = 0; i < 32; ++i) { amax = fmaxf(amax, fabsf(a[i])); sum += a[i]; }
                    const float d_inv = amax > 0.f ? __fdiv_rn(127.0f, amax) : 0.f;
                    uint32_t w[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int q0 = (int)roundf(a[4 * i] * d_inv), q1 = (int)roundf(a[4 * i + 1] * d_inv);
                        const int q2 = (int)roundf(a[4 * i + 2] * d_inv), q3 = (int)roundf(a[4 * i + 3] * d_inv);
                        w[i] = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
                    }
                    uint8_t* blk = p.out_mmq + ((size_t)(kvh * p.G + hg) * p.batch + tglob) * 144;
                    const int g = 2 * team + c;
                    const float d = amax > 0.f ? __fdiv_rn(1.0f, d_inv) : 0.f;
                    if (p.mmq_ds4) reinterpret_cast<__half2*>(blk)[g] = __halves2half2(__float2half(d), __float2half(sum));
                    else           reinterpret_cast<float*>(blk)[g] = d;
                    uint4* qs = reinterpret_cast<uint4*>(blk + 16 + 32 * g);
                    qs[0] = make_uint4(w[0], w[1], w[2], w[3]);
                    qs[1] = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
        }
        if (p.out_tma) {
            // every softmax thread comes here, whatever its waits returned
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");       // generic-proxy stores -> the bulk copies' reads
            asm volatile("bar.sync 1, 256;\n" ::: "memory");
            if (tid == 32 * kFirstSoftmaxWarp && !*s_abort) {
                // rows past the batch (a ragged last tile) lie outside the tensor map and are not written
#pragma unroll
                for (int c = 0; c < 4; ++c) tma_store_3d(&tmO, 32 * c, kvh * p.G, t0, sbase + OFF_K + c * (BM * 128));
                asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
                asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory");  // shared memory stays valid until it has been read
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512u) : "memory");
    }
    if (tid == 0 && *s_abort && p.status) atomicExch(p.status, 1);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

// fp16 tensor [d2][d1][128] with the given strides (bytes); box = 64 x b1 x b2, 128-byte swizzle, zero fill.
// fp32 tensor [d2][d1][128] (the output): box = 32 x b1 x b2 (one 128-byte swizzle span of columns), for stores.
bool make_out_map(CUtensorMap* m, const void* base, uint64_t d1, uint64_t d2, uint64_t stride1, uint64_t stride2, uint32_t b1,
                  uint32_t b2) {
    cuuint64_t dims[3] = {(cuuint64_t)HD, d1, d2};
    cuuint64_t strides[2] = {stride1, stride2};
    cuuint32_t box[3] = {32, b1, b2};
    cuuint32_t estr[3] = {1, 1, 1};
    return g_encode(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_map(CUtensorMap* m, const void* base, uint64_t d1, uint64_t d2, uint64_t stride1, uint64_t stride2, uint32_t b1,
              uint32_t b2) {
    cuuint64_t dims[3] = {(cuuint64_t)HD, d1, d2};
    cuuint64_t strides[2] = {stride1, stride2};
    cuuint32_t box[3] = {64, b1, b2};
    cuuint32_t estr[3] = {1, 1, 1};
    return g_encode(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

} // namespace

#ifdef OATTN_TC_TRACE
extern "C" int oattn_debug_trace_read(long long* host) {
    return (int)cudaMemcpyFromSymbol(host, g_trace, sizeof(g_trace));
}
#endif

cudaError_t prefill_tc_set_attributes() {
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess) return e;
        if (qres != cudaDriverEntryPointSuccess || !fn) return cudaErrorNotSupported;
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    return cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
}

cudaError_t launch_prefill_tc(const PrefillArgs& a, int sm_count, cudaStream_t stream, unsigned long long* launches) {
    (void)sm_count;
    const int G = a.n_head / a.n_kv;
    if (a.head_dim != HD || G > 128 || !g_encode) return cudaErrorNotSupported;
    const int TQ = 128 / G;
    const uint64_t rows = (uint64_t)a.n_past + a.batch;          // rows past the chunk are never read (zero fill)
    CUtensorMap tmQ, tmK, tmV;
    const uint64_t rowb = HD * sizeof(__half);
    if (!make_map(&tmQ, a.q16, a.n_head, a.batch, rowb, rowb * a.n_head, G, TQ)) return cudaErrorInvalidValue;
    if (!make_map(&tmK, a.kc, rows, a.n_kv, rowb, rowb * a.n_ctx, BN, 1)) return cudaErrorInvalidValue;
    if (!make_map(&tmV, a.vc, rows, a.n_kv, rowb, rowb * a.n_ctx, BN, 1)) return cudaErrorInvalidValue;
    // the fp32 output as a tensor map for bulk stores (16-byte aligned base; else the kernel stores directly)
    CUtensorMap tmO = tmQ;
    const uint64_t orow = HD * sizeof(float);
    const bool out_tma = a.out && !((uintptr_t)a.out & 15) && make_out_map(&tmO, a.out, a.n_head, a.batch, orow, orow * a.n_head, G, TQ);
    TcArgs t;
    t.out_tma = out_tma ? 1 : 0;
    t.out = a.out;
    t.out_mmq = a.out_mmq;
    t.mmq_ds4 = a.mmq_ds4;
    t.status = a.status;
    t.n_head = a.n_head; t.n_kv = a.n_kv; t.n_past = a.n_past; t.batch = a.batch; t.G = G; t.TQ = TQ;
    dim3 grid((a.batch + TQ - 1) / TQ, a.n_kv);
    const cudaError_t e = launch_dependent(prefill_tc_kernel, grid, kThreads, SMEM_BYTES, stream, 1, tmQ, tmK, tmV, tmO, t);
    if (launches) *launches += 1;
    return e;
}

} // namespace oattn
