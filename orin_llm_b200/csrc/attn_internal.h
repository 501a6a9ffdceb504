// Internal launch interface between the C ABI (capi.cu) and the kernel translation units.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "common.cuh"

namespace oattn {

constexpr int DECODE_TILE = 64;        // cache rows per pipeline stage of the decode kernel
constexpr int DECODE_MAX_SPLITS = 512; // upper bound on KV splits per kv head (combine smem)
constexpr int PART_PAD = 4;            // floats after O in a partial record: m, l, 0, 0
constexpr int DECODE_MAX_RANKS = 16;   // ranks of one peer exchange

// Exchange buffer of one rank (the same layout on every rank): 8-byte words [2 slots][world][n_head][hd+PART_PAD],
// each word = {fp32 value, 32-bit generation tag}.  Value and tag travel in one aligned 8-byte store, so a reader
// that sees the tag of the generation it waits for has the value too: no fence and no separate flag.
__host__ __device__ inline size_t peer_buffer_bytes(int world, int n_head, int head_dim) {
    const size_t rec = (size_t)2 * world * n_head * (head_dim + PART_PAD) * sizeof(unsigned long long);
    return (rec + 255) & ~(size_t)255;
}

// Splits per first-level merge group of the decode kernel: about sqrt(n_splits), so that both levels of the merge
// tree are one pass (at most 16 partials) for up to 256 splits.
inline int decode_group_size(int n_splits) {
    int g = 2;
    while (g * g < n_splits && g < 16) ++g;
    return g;
}

// Decode scratch (caller-owned): the un-normalised partial of every split, [n_kv][n_splits][G][hd] fp32 and
// [n_kv][n_splits][G][2] (m in raw-score units, l), and the same for every group of `group` neighbouring splits.
struct DecodeWsLayout {
    size_t part_o, part_ml, grp_o, grp_ml, rec, total;   // byte offsets, 256-byte aligned; rec: this rank's record
    int n_splits, group, n_groups;
};
inline DecodeWsLayout decode_ws_layout(int n_head, int n_kv, int head_dim, int n_splits) {
    auto al = [](size_t v) { return (v + 255) & ~(size_t)255; };
    DecodeWsLayout w;
    w.n_splits = n_splits;
    w.group = decode_group_size(n_splits);
    w.n_groups = (n_splits + w.group - 1) / w.group;
    w.part_o = 0;
    w.part_ml = w.part_o + al((size_t)n_head * n_splits * head_dim * sizeof(float));
    w.grp_o = w.part_ml + al((size_t)n_head * n_splits * 2 * sizeof(float));
    w.grp_ml = w.grp_o + al((size_t)n_head * w.n_groups * head_dim * sizeof(float));
    w.rec = w.grp_ml + al((size_t)n_head * w.n_groups * 2 * sizeof(float));
    w.total = w.rec + al((size_t)n_head * (head_dim + PART_PAD) * sizeof(float));
    return w;
}

struct DecodeArgs {
    const float* q;        // [n_head][hd] fp32
    const float* k_new;    // [n_kv][hd] fp32 or nullptr
    const float* v_new;    // [n_kv][hd] fp32 or nullptr
    uint16_t* kc;          // [n_kv][n_ctx][hd] fp16 bits
    uint16_t* vc;
    float* out;            // [n_head][hd] (final) or [n_head][hd+PART_PAD] (partial record)
    float* ws_o;           // scratch, see DecodeWsLayout
    float* ws_ml;
    float* grp_o;
    float* grp_ml;
    unsigned* tickets;     // arrival counters: [n_kv][n_groups] first level, then [n_kv] second level; zero at rest
    const int* d_pos;      // device scalar
    int pos_bias;          // valid rows = *d_pos + pos_bias  (1: d_pos is the new token's position; 0: d_pos is a length)
    int n_head, n_kv, head_dim, n_ctx, n_splits, group, n_groups, min_tiles;
    float scale;
    int fuse;
    RopeArgs rope;
    int emit_partial;      // write the un-normalised record instead of the normalised output
    int defer_final = 0;   // with emit_partial: stop after the first merge level and leave the kv head's group results
                           // (grp_o / grp_ml, group 0 when there is only one) to the exchange launch, which merges them
    PreArgs pre;                   // optional bias / per-head RMSNorm in front of RoPE
    const int* d_rope_pos = nullptr;   // position used for RoPE when it is not the local row index (sharded cache)
    int8_t* out_qs = nullptr;      // optional q8_1 form of the output: int8 [n_head*hd] ...
    float* out_scales = nullptr;   // ... and one fp32 scale per 32 values; `out` may then be nullptr
    int overlap = 0;                                  // 0 plain launch, 1 dependent launch, 2 + K/V prefetch before the wait
};

// Size of the scratch block built into the library for oattn_decode_noalloc, and its device address on the
// current device (looked up once per device).
constexpr size_t kStaticScratchBytes = 2u << 20;
cudaError_t decode_static_scratch(void** ptr);
// Arrival counters for the decode launches that use `workspace` on the current device: a slot of a zero-initialised
// table inside the library image (one slot per distinct workspace address, least recently used slot recycled).
constexpr int kTicketSlots = 64;
constexpr int kTicketWords = 512;
cudaError_t decode_ticket_slot(const void* workspace, unsigned** tickets);

// Number of KV splits per kv head the decode launch uses on a device with `sm_count` SMs.
int decode_num_splits(int n_kv, int sm_count);
cudaError_t decode_set_attributes();
// One launch; ev_start / ev_stop (optional) are recorded around it.
cudaError_t launch_decode(const DecodeArgs& a, cudaStream_t stream, unsigned long long* launches,
                          cudaEvent_t ev_start = nullptr, cudaEvent_t ev_stop = nullptr);
// Merge n_parts records [n_parts][n_head][hd+PART_PAD] -> out [n_head][hd].
cudaError_t launch_combine_records(const float* parts, int n_parts, float* out, int n_head, int head_dim,
                                   cudaStream_t stream, unsigned long long* launches);

// Merges the group results a decode launch with defer_final left for each kv head into this rank's record, stores it into
// every rank's exchange buffer and, with fused_wait, waits for all records of the generation and writes the merged out.
cudaError_t launch_peer_exchange(const DecodeArgs& d, const unsigned long long* peer_bufs, int* gen_push, int rank, int world,
                                 int fused_wait, float* out, int* status, long long wait_cycles, int overlap,
                                 cudaStream_t stream, unsigned long long* launches);
cudaError_t launch_peer_wait_combine(const void* my_buf, int world, float* out, int n_head, int head_dim, int* gen_wait,
                                     int* status, long long wait_cycles, int overlap, cudaStream_t stream,
                                     unsigned long long* launches);

// Launch with (overlap != 0) or without the programmatic-stream-serialization attribute.
template <typename Kernel, typename... Args>
inline cudaError_t launch_dependent(Kernel kernel, dim3 grid, int threads, size_t smem, cudaStream_t stream, int overlap, const Args&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

struct PrefillArgs {
    const float* q;        // [batch][n_head][hd] fp32
    const float* k_new;    // [batch][n_kv][hd] fp32 or nullptr
    const float* v_new;
    uint16_t* kc;
    uint16_t* vc;
    float* out;            // [batch][n_head][hd] fp32
    __half* q16;           // workspace: [batch][n_head][hd] fp16, rotated and pre-scaled by scale*log2(e)
    int* status;           // workspace: 0 = ok, non-zero = the tcgen05 kernel gave up on a bounded wait
    int n_head, n_kv, head_dim, n_ctx, n_past, batch;
    float scale;
    int fuse;
    RopeArgs rope;
    PreArgs pre;           // optional bias / per-head RMSNorm in front of RoPE (k and v parts only with the append)
    uint8_t* out_mmq = nullptr;   // optional: the output as block_q8_1_mmq blocks [head][batch], 144 bytes each
    int mmq_ds4 = 0;              // scales as fp16 (d, sum) pairs instead of fp32 d
};

// Prologue shared by both prefill kernels: RoPE(q) -> q16, RoPE(k_new) + fp16 append of k_new, v_new.
cudaError_t launch_prefill_prologue(const PrefillArgs& a, cudaStream_t stream, unsigned long long* launches);
cudaError_t prefill_mma_set_attributes();
cudaError_t launch_prefill_mma(const PrefillArgs& a, cudaStream_t stream, unsigned long long* launches);
cudaError_t prefill_tc_set_attributes();
// Returns cudaErrorNotSupported when the tcgen05 kernel does not cover the shape.
cudaError_t launch_prefill_tc(const PrefillArgs& a, int sm_count, cudaStream_t stream, unsigned long long* launches);

cudaError_t launch_rope(float* x, int rows, int head_dim, const RopeArgs& r, int n_past, int heads,
                        const int* d_pos, cudaStream_t stream, unsigned long long* launches);
cudaError_t launch_kv_store(uint16_t* kc, uint16_t* vc, const float* k, const float* v, int heads, int head_dim,
                            int n_ctx, int pos_base, int batch, const int* d_pos, cudaStream_t stream,
                            unsigned long long* launches);
cudaError_t launch_kv_shift(uint16_t* kc, uint16_t* vc, int n_layer, int n_kv, int head_dim, int n_ctx, int n_keep,
                            int shift, cudaStream_t stream, unsigned long long* launches);

} // namespace oattn
