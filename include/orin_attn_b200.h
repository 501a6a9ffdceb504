/*
 * orin_attn_b200 -- C ABI of the B200 (sm_100a) attention path for Heng-W/orin_llm.
 *
 * This is the drop-in boundary: plain pointers and sizes, no C++ or framework types.  The
 * reference reaches its attention through free functions in `namespace llm::cuda`
 * (src/kernels.h); each entry point below names the reference function it stands in for.
 * The C++ wrappers with the reference's exact signatures are in
 * orin_llm_b200/host/kernels.h and are implemented on top of this header.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless the comment says "host".
 *   - The caller owns every buffer; the attention calls allocate nothing, free nothing and never synchronise
 *     (only the set-up helpers oattn_scratch_alloc/free and the memory-placement group do).
 *   - `stream` is a cudaStream_t passed as void* (the reference does the same in
 *     cuda::set_stream, src/kernels.h:10).  Every call is asynchronous on that stream and may
 *     be recorded into a CUDA graph: launch shapes never depend on the token position, which
 *     arrives through `d_pos` in device memory (src/kernels.h:59-62, 69-70, 80-81).
 *   - Return value: OATTN_OK or an OATTN_ERR_* code.  Nothing aborts (the reference aborts
 *     through CUDA_CHECK, src/common.h:14-22; a library must not).
 *   - KV cache of one layer: fp16 bit patterns as uint16_t, laid out [n_kv][n_ctx][head_dim]
 *     (src/kernels.cu:1675, src/model_gpu.cu:229-235, 259-260).
 *   - Activations q / k / v / out: fp32, [batch][heads][head_dim] (src/kernels.cu:1404, 1563).
 *   - head_dim must be 64 or 128 (same restriction as src/kernels.cu:1976-1980);
 *     n_head must be a multiple of n_kv with n_head/n_kv <= 16.
 */
#ifndef ORIN_ATTN_B200_H
#define ORIN_ATTN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    OATTN_OK = 0,
    OATTN_ERR_ARG = 1,         /* null pointer, non-positive size, batch/n_past outside n_ctx */
    OATTN_ERR_UNSUPPORTED = 2, /* head_dim, GQA ratio or n_rot outside what the kernels cover */
    OATTN_ERR_WORKSPACE = 3,   /* workspace missing, misaligned or smaller than *_workspace_bytes() */
    OATTN_ERR_CUDA = 4,        /* a CUDA runtime call or launch failed; see oattn_last_cuda_error() */
    OATTN_ERR_DEVICE = 5       /* not an sm_100 device, or oattn_init() not called on this device */
};

/* RoPE pairing, numbered like HParams::rope_type (src/model.h:27-28). */
enum { OATTN_ROPE_NORMAL = 0, OATTN_ROPE_NEOX = 1 };

/* What the fused attention calls do before attending (src/model_gpu.cu:277-282, 379-384). */
enum {
    OATTN_FUSE_NONE = 0,      /* q already rotated, cache already holds this step's K/V          */
    OATTN_FUSE_ROPE_Q = 1,    /* rotate q (not written back)                                     */
    OATTN_FUSE_ROPE_K = 2,    /* rotate k_new before it is appended (needs OATTN_FUSE_KV_APPEND) */
    OATTN_FUSE_KV_APPEND = 4, /* convert k_new, v_new to fp16 and store them in the cache         */
    OATTN_FUSE_ALL = 7
};

/* RoPE parameters of the fused calls (src/model.h:24-30).  freq_factors: device, n_rot/2 floats
 * or NULL (src/model_common.cpp:37-43). */
typedef struct oattn_rope_params {
    int rope_type;
    int n_rot;
    float theta;
    const float* freq_factors;
} oattn_rope_params;

const char* oattn_strerror(int code);
/* Text of the last CUDA error seen by this library on the calling thread's device (host string). */
const char* oattn_last_cuda_error(void);

/* Replaces cuda::init (src/kernels.cu:1730-1737), generalised from device 0 to `device`:
 * makes it current, checks for compute capability 10.x, raises the shared-memory limits of the
 * kernels once (the reference does that on every launch, src/kernels.cu:1968,1988). */
int oattn_init(int device);      /* device < 0: the calling thread's current device */
/* Convenience for hosts without an arena of their own: `bytes` of device memory on the current device (cudaMalloc),
 * never freed by the library.  The one allocating entry point; nothing else in this interface calls it. */
int oattn_scratch_alloc(size_t bytes, void** ptr);
/* Returns a block obtained from oattn_scratch_alloc (cudaFree; NULL is accepted).  Synchronises the device as cudaFree
 * does: never call it on a hot path or under stream capture. */
int oattn_scratch_free(void* ptr);
/* Address and size of the library's built-in scratch block on the current device (the block oattn_decode_noalloc
 * uses, see there): lets a host that may not allocate pass it as the `workspace` of oattn_decode / oattn_decode_ex
 * when oattn_decode_workspace_bytes() fits.  No allocation, no stream operation.  The same sharing rule applies: calls
 * that use the block must not overlap on the GPU.  No counterpart in the reference. */
int oattn_builtin_scratch(void** ptr, size_t* bytes);
/* ---- memory placement for a discrete GPU (set-up time only; these are the entry points that allocate) -------------
 * The reference was written for a unified-memory Orin: the GPU reads the weights through a zero-copy mapping of the
 * memory-mapped model file (src/model_gpu.cu:96-149), writes the logits into mapped host memory (:210-211) and never
 * clears its KV cache (:232-235).  On a B200 the first two put PCIe on the path of every token, the third leaves NaN
 * bit patterns in rows that whole-tile loads touch.  These helpers are what the three places call instead.
 *   oattn_weights_place      `bytes` of device memory holding a copy of host[0, bytes) (cudaMalloc + one blocking copy);
 *                            a tensor at host + off is then at *dev + off.  Replaces cudaHostRegister +
 *                            cudaHostGetDevicePointer.  Release with oattn_scratch_free.
 *   oattn_logits_alloc       a device buffer for the output head to write and a pinned host buffer of the same size;
 *   oattn_copy_to_host_async the copy between them on `stream` (a memcpy node when the stream is being captured: the
 *                            decode graph then ends with it), replacing the mapped-host write of every logit;
 *   oattn_logits_free        frees the pair.
 *   oattn_device_clear       zero-fills device memory and waits (once, for the KV cache right after its allocation). */
int oattn_weights_place(const void* host, size_t bytes, void** dev);
int oattn_logits_alloc(size_t bytes, void** dev, void** pinned_host);
int oattn_logits_free(void* dev, void* pinned_host);
int oattn_copy_to_host_async(void* pinned_host, const void* dev, size_t bytes, void* stream);
int oattn_device_clear(void* dev, size_t bytes);

/* Number of SMs of the initialised device (0 before oattn_init). */
int oattn_sm_count(void);

/* ---- unfused building blocks: same semantics as the reference wrappers -------------------- */

/* Replaces cuda::rope_neox_batch / rope_normal_batch (src/kernels.cu:2059-2067) when d_pos is
 * NULL: row r of x [rows][head_dim] is rotated in place at position n_past + r/heads.
 * Replaces cuda::rope_neox_ind / rope_normal_ind (src/kernels.cu:2069-2075) when d_pos is not
 * NULL: every row is rotated at position *d_pos (n_past, heads ignored).
 * Frequencies and angles are evaluated as the reference's CPU backend does
 * (src/model_cpu.cpp:179-203), not with the fast-math intrinsics of src/kernels.cu:1631-1634. */
int oattn_rope(float* x, int rows, int head_dim, int rope_type, int n_rot, float theta, int n_past,
               int heads, const int* d_pos, const float* freq_factors, void* stream);

/* Replaces cuda::kv_store_batch (src/kernels.cu:2079-2083) when d_pos is NULL: k, v
 * [batch][heads][head_dim] fp32 -> fp16 at cache rows pos_base + b.
 * Replaces cuda::kv_store_ind (src/kernels.cu:2085-2088) when d_pos is not NULL: one token at
 * row *d_pos (pos_base ignored, batch must be 1). */
int oattn_kv_store(uint16_t* kc, uint16_t* vc, const float* k, const float* v, int heads, int head_dim,
                   int n_ctx, int pos_base, int batch, const int* d_pos, void* stream);

/* Replaces cuda::kv_shift (src/kernels.cu:2090-2093): for every layer and kv head drop rows
 * [n_keep, n_keep+shift), slide the rest left, zero the last `shift` rows.  kc, vc point at
 * layer 0; layers are n_kv*n_ctx*head_dim elements apart.  In place, no scratch.
 * Requires 0 <= n_keep, 0 < shift, n_keep + shift <= n_ctx. */
int oattn_kv_shift(uint16_t* kc, uint16_t* vc, int n_layer, int n_kv, int head_dim, int n_ctx, int n_keep,
                   int shift, void* stream);

/* ---- decode: one query token, split-KV flash decoding + log-sum-exp combine --------------- */

/* Bytes of scratch the decode calls need for their per-split and per-group partial results (m, l, O).
 * Follows the reference's scratch_size()/scratch_assign() pattern (src/kernels.cu:1753-1776):
 * the caller allocates once and passes the block on every call.  256-byte aligned; it need not be
 * cleared (the arrival counters of the in-launch merge live inside the library, one set per
 * workspace address).  Two calls that run on the GPU at the same time need two workspaces. */
size_t oattn_decode_workspace_bytes(int n_head, int n_kv, int head_dim);

/* Replaces the decode sequence rope_*_ind(q), rope_*_ind(k), kv_store_ind,
 * flash_attention_decode_ind (src/model_gpu.cu:277-282; src/kernels.cu:1993-2000).
 * Attends q [n_head][head_dim] over cache rows 0..*d_pos.  With fuse == OATTN_FUSE_NONE it is
 * exactly flash_attention_decode_ind (k_new, v_new, rope may be NULL).  With fuse flags the new
 * token's K/V row (k_new, v_new: [n_kv][head_dim] fp32) is rotated, converted and stored at row
 * *d_pos inside the same launch.  ONE launch (grid fixed by n_kv and the SM count): the CTAs
 * that finish last merge the per-split partials themselves (the cross-warp merge of
 * src/kernels.cu:1280-1344 extended over CTAs).  q, k_new, v_new and out must be 16-byte aligned. */
int oattn_decode(const float* q, const float* k_new, const float* v_new, uint16_t* kc, uint16_t* vc,
                 float* out, int n_head, int n_kv, int head_dim, int n_ctx, const int* d_pos, float scale,
                 int fuse, const oattn_rope_params* rope, void* workspace, size_t workspace_bytes, void* stream);

/* No counterpart in the reference.  Same result as oattn_decode with OATTN_FUSE_NONE, for hosts that are not
 * able to give the library a workspace: code that runs where device allocation is forbidden or unavailable --
 * inside a plugin whose host owns all device memory and hands out none, in a callback that must not call
 * cudaMalloc, or late in a process whose memory is fully committed.  The per-split partial results go to a block
 * of oattn_decode_noalloc_max_bytes() (2 MiB) that is part of the library image in device memory; every GPU that
 * loads the library holds that block until the process ends.  Shapes whose partials do not fit
 * (n_head * splits * (head_dim + 2) * 4 bytes, splits = 2 * SMs / n_kv) are refused with OATTN_ERR_WORKSPACE and a
 * message in oattn_last_cuda_error(); nothing is allocated or freed, here or later.  The block's device address is
 * looked up by oattn_init; on a device that was never initialised the first call to this entry point runs
 * oattn_init(-1) itself, so make that first call outside any stream capture.  All calls on a device share the one
 * block and it keeps what the previous call wrote: nothing in it has to start at zero (each call overwrites the
 * slots it later reads), but two calls that run on the GPU at the same time -- different streams, or a graph replay
 * overlapping an eager call -- would overwrite each other's partials, so keep calls to this entry point ordered on
 * one stream. */
size_t oattn_decode_noalloc_max_bytes(void);
int oattn_decode_noalloc(const float* q, const uint16_t* kc, const uint16_t* vc, float* out, int n_head, int n_kv,
                         int head_dim, int n_ctx, const int* d_pos, float scale, void* stream);

/* Multi-GPU building block (no reference counterpart as a function; the arithmetic is the
 * cross-warp merge of src/kernels.cu:1300-1342 lifted to KV slices).  Attends q over the LOCAL
 * cache rows [0, *d_len) and writes one un-normalised partial per head:
 * part [n_head][head_dim + 4] = { O[head_dim], m, l, 0, 0 } with m = max score (scaled),
 * l = sum exp(score - m), O = sum exp(score - m) * v.  *d_len == 0 gives m = -inf, l = 0. */
int oattn_decode_partial(const float* q, const uint16_t* kc, const uint16_t* vc, float* part, int n_head,
                         int n_kv, int head_dim, int n_ctx, const int* d_len, float scale, void* workspace,
                         size_t workspace_bytes, void* stream);

/* Merges n_parts partials laid out [n_parts][n_head][head_dim + 4] (the all-gathered output of
 * oattn_decode_partial on every rank) into out [n_head][head_dim]:
 * M = max m_r, L = sum l_r e^(m_r - M), out = sum O_r e^(m_r - M) / L. */
int oattn_combine(const float* parts, int n_parts, float* out, int n_head, int head_dim, void* stream);

/* ---- multi-GPU exchange without a collective call (no reference counterpart) ----------------------------------
 * The record exchange of split-KV decode is 8 KB per rank: latency-bound.  Instead of all-gather + combine, a small
 * launch behind the decode launch (one CTA per head, so that the peer stores of a call leave from n_head SMs) finishes
 * this rank's record -- the decode launch stops after its first merge level and leaves a handful of group results per
 * kv head -- and stores it straight into every rank's exchange buffer over NVLink (plain peer stores).  Every fp32
 * value travels in one aligned 8-byte word together with the generation number of the call, so the receiver needs neither a fence nor a flag: it polls the words of its own buffer until they carry
 * the current generation (bounded, ~2 s by default, see oattn_set_wait_limit_cycles; then a status word is set and the
 * output is left untouched) and merges the `world` records.
 *   exchange buffer   oattn_peer_buffer_bytes(world, n_head, head_dim) bytes on every rank, peer-mapped (e.g. CUDA
 *                     VMM / torch symmetric memory), zero-filled before first use; `peer_bufs_dev` is a DEVICE array
 *                     of `world` pointers (entry r = rank r's buffer as seen from this GPU, own buffer included)
 *   state             oattn_peer_state_bytes(n_head) bytes of ordinary device memory per rank, zero-filled once
 * Records are double-buffered by generation parity; every rank must make the same sequence of calls.  Both calls
 * are graph-capturable.  world <= 16. */
size_t oattn_peer_buffer_bytes(int world, int n_head, int head_dim);
size_t oattn_peer_state_bytes(int n_head);
int oattn_decode_partial_push(const float* q, const uint16_t* kc, const uint16_t* vc, int n_head, int n_kv, int head_dim,
                              int n_ctx, const int* d_len, float scale, void* workspace, size_t workspace_bytes,
                              const void* peer_bufs_dev, int rank, int world, void* state, void* stream);
int oattn_peer_wait_combine(const void* my_buf, int world, float* out, int n_head, int head_dim, void* state, void* stream);
/* Both steps in two launches instead of three: the exchange launch that stores this rank's record into every exchange
 * buffer also waits for the other ranks' records and writes the merged out [n_head][head_dim].  Every rank must be running on a
 * GPU of its own (the launch waits for kernels of the other ranks); do not mix with the two calls above on the same
 * state block.  No counterpart in the reference. */
int oattn_decode_peer(const float* q, const uint16_t* kc, const uint16_t* vc, float* out, int n_head, int n_kv, int head_dim,
                      int n_ctx, const int* d_len, float scale, void* workspace, size_t workspace_bytes,
                      const void* peer_bufs_dev, int rank, int world, void* state, void* stream);
/* The same with the decode step's fused prologue, for a cache that is sharded by rows: every rank passes the unrotated q
 * with OATTN_FUSE_ROPE_Q; the rank whose slice receives the new token passes k_new, v_new and OATTN_FUSE_ALL as well.
 * `d_len` is the number of valid local rows INCLUDING the row being appended (it lands in local row *d_len - 1);
 * `d_rope_pos` is the token's position in the whole sequence, which sets the rotation angle (device scalars, so the
 * call replays from a graph).  No counterpart in the reference. */
int oattn_decode_peer_fused(const float* q, const float* k_new, const float* v_new, uint16_t* kc, uint16_t* vc, float* out,
                            int n_head, int n_kv, int head_dim, int n_ctx, const int* d_len, const int* d_rope_pos, float scale,
                            int fuse, const oattn_rope_params* rope, void* workspace, size_t workspace_bytes,
                            const void* peer_bufs_dev, int rank, int world, void* state, void* stream);
/* Blocking read of the status word (0 = every wait so far was satisfied). */
int oattn_peer_status(const void* state, int n_head, int* status);
/* Bound of the device-side waits for the peers' records, in SM clock cycles (default 4e9, about two seconds; at least
 * 1000).  When a wait runs out the kernel raises the status word, leaves the output untouched and returns, so the
 * context stays usable; the next complete exchange works again.  Process-wide; applies to launches made after the
 * call (a captured graph keeps the bound it was captured with). */
int oattn_set_wait_limit_cycles(long long cycles);

/* ---- the steps on either side of attention, folded into the same launches -------------------- */

/* Optional extras of oattn_decode_ex / oattn_prefill_ex.  Every pointer is a device pointer and may be NULL.
 *   bias_q/k/v   replace add_inplace_broadcast on q, k, v (src/model_gpu.cu:372-374; src/model_cpu.cpp:258-260):
 *                [n_head*head_dim], [n_kv*head_dim], [n_kv*head_dim], added before everything else.
 *   norm_q/k     replace rms_norm_rows over the head rows of q and k (src/model_gpu.cu:274-275, 376-377;
 *                src/model_cpu.cpp:266, 271): y = x / sqrt(mean(x^2) + norm_eps) * w, w of [head_dim], after the bias
 *                and before RoPE.
 *   out_qs, out_scales   (decode only) the output in the form the next GEMV reads, replacing
 *                quantize_activation(d_attn_) (src/model_gpu.cu:284; quantize_q8_1_k, src/kernels.cu:136-145): per
 *                32 consecutive values d = max|x| / 127, q = round-half-away(x / d) (0 for an all-zero group); int8
 *                [n_head*head_dim] and fp32 [n_head*head_dim/32], laid out as scratch_assign does
 *                (src/kernels.cu:1763-1776).  With these set, `out` may be NULL.
 *   out_mmq, out_mmq_ds4 (prefill only, head_dim 128) the output in the form the reference's batched int8 GEMM reads,
 *                replacing the quantize_mmq_q8_1_k pass in front of the Wo projection (src/kernels.cu:147-205, launched
 *                at :1842-1850): 144-byte blocks of 128 values = four groups of 32, each group d = max|x| / 127 and
 *                q = round-half-away(x * (127 / max|x|)); block (chunk c, token t) at index c * batch + t, which with
 *                head_dim 128 is (head, token).  out_mmq_ds4 != 0: the four scales are fp16 pairs (d, sum of the
 *                group's values), the form a Q4_K weight needs; 0: four fp32 d, the form a Q6_K weight needs
 *                (src/kernels.cu:1846).  With out_mmq set, `out` may be NULL.
 * bias_k, bias_v and norm_k act on the appended row and need OATTN_FUSE_KV_APPEND. */
typedef struct oattn_ext {
    const float* bias_q;
    const float* bias_k;
    const float* bias_v;
    const float* norm_q;
    const float* norm_k;
    float norm_eps;
    int8_t* out_qs;
    float* out_scales;
    void* out_mmq;
    int out_mmq_ds4;
} oattn_ext;

/* oattn_decode with the extras above (ext == NULL: identical to oattn_decode). */
int oattn_decode_ex(const float* q, const float* k_new, const float* v_new, uint16_t* kc, uint16_t* vc, float* out,
                    int n_head, int n_kv, int head_dim, int n_ctx, const int* d_pos, float scale, int fuse,
                    const oattn_rope_params* rope, const oattn_ext* ext, void* workspace, size_t workspace_bytes, void* stream);
/* oattn_prefill with bias / norm and, optionally, the output as block_q8_1_mmq blocks (out_mmq; out_qs is the decode
 * form and is refused here). */
int oattn_prefill_ex(const float* q, const float* k_new, const float* v_new, uint16_t* kc, uint16_t* vc, float* out,
                     int n_head, int n_kv, int head_dim, int n_ctx, int n_past, int batch, float scale, int fuse,
                     const oattn_rope_params* rope, const oattn_ext* ext, void* workspace, size_t workspace_bytes,
                     void* stream);

/* ---- prefill: a chunk of `batch` query tokens, causal ------------------------------------ */

/* Scratch for the prefill call (fp16 staging of the rotated, scaled queries). 256-byte aligned. */
size_t oattn_prefill_workspace_bytes(int n_head, int n_kv, int head_dim, int max_batch);

/* Replaces the prefill sequence rope_*_batch(q), rope_*_batch(k), kv_store_batch,
 * flash_attention (src/model_gpu.cu:379-384; src/kernels.cu:1974-1981).  Query token t of
 * q [batch][n_head][head_dim] sits at position n_past + t and sees cache rows 0..n_past+t.
 * With fuse == OATTN_FUSE_NONE it is exactly cuda::flash_attention.  `out` must be 16-byte aligned
 * (OATTN_ERR_ARG otherwise); q, k_new and v_new may have any float alignment. */
int oattn_prefill(const float* q, const float* k_new, const float* v_new, uint16_t* kc, uint16_t* vc,
                  float* out, int n_head, int n_kv, int head_dim, int n_ctx, int n_past, int batch,
                  float scale, int fuse, const oattn_rope_params* rope, void* workspace, size_t workspace_bytes,
                  void* stream);

/* Reads back the status word the last oattn_prefill call on `workspace` left (same n_head, head_dim,
 * batch as that call): 0 = completed; 1 = the tcgen05 kernel gave up on one of its bounded waits and
 * the output is not valid.  SYNCHRONOUS (a blocking device-to-host copy): for tests and diagnostics. */
int oattn_prefill_status(const void* workspace, int n_head, int head_dim, int batch, int* status);

/* Which prefill kernel oattn_prefill launches: 0 = tcgen05/TMEM kernel (default),
 * 1 = the warp-level mma.sync kernel kept as an in-library cross-check.  Process-wide. */
int oattn_set_prefill_impl(int impl);

/* How the decode launches are ordered against the preceding kernels of the stream (no counterpart in the reference).
 *   0  (default) ordinary launches.
 *   1  programmatic dependent launches: a decode kernel may be scheduled while the preceding kernel of the
 *      stream drains, and waits for it to complete before it reads or writes anything.  Same results as 0.
 *   2  as 1, and the kernel reads *d_pos and fetches its first cache tiles (rows below *d_pos) BEFORE that wait, so
 *      that consecutive calls stream back to back.  The newest row (row *d_pos) is never taken from that early
 *      fetch: it comes from k_new / v_new (fused append) or is re-read after the wait, so the reference's unfused
 *      sequence rope, rope, kv_store_ind, flash_attention_decode_ind (src/model_gpu.cu:277-282) is safe.  The caller
 *      vouches that the position word and the cache rows BELOW *d_pos are not written by the kernel launched just
 *      before the call (true for the reference's decode graph, src/model_gpu.cu:295-344: the position is copied in
 *      before the graph starts and every layer has its own cache).  Do not use for back-to-back calls on one
 *      cache, e.g. a decode call right behind the prefill call that filled it. */
int oattn_set_decode_overlap(int mode);

/* Lower bound on the 64-row tiles one decode split handles (default 1).  Independently of it, contexts of up to 4
 * tiles stay in one CTA per kv head and contexts of up to 64 tiles use at most 16 (one merge level).  Process-wide
 * tuning knob; must not change between the capture and
 * the replays of a CUDA graph. */
int oattn_set_decode_min_tiles(int tiles);

/* Opt-in kernel timing for benchmarks (off by default; the hot calls allocate nothing either way:
 * the events are created here).  After oattn_profile_enable(n) every oattn_decode /
 * oattn_decode_partial call brackets its kernel with a pair of
 * CUDA events on the call's stream, for the first n calls.  oattn_profile_collect waits for those
 * events, writes the elapsed milliseconds of each recorded call to ms (host, `capacity` floats),
 * stores the count in *n_written and rearms the counter.  oattn_profile_enable(0) destroys the
 * events.  When the call is being captured into a CUDA graph the events are recorded as external
 * event nodes: after a replay they hold the timings of that replay. */
int oattn_profile_enable(int max_records);
int oattn_profile_collect(float* ms, int capacity, int* n_written);

/* Number of kernels this library has launched since load (for launch accounting in benchmarks). */
unsigned long long oattn_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* ORIN_ATTN_B200_H */
