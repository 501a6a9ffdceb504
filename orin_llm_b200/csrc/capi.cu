// extern "C" layer: argument checking, workspace carving, launch.  See include/orin_attn_b200.h.
#include <stdio.h>
#include <string.h>

#include "../../include/orin_attn_b200.h"
#include "attn_internal.h"

using namespace oattn;

namespace {

constexpr int kMaxDevices = 64;
struct DeviceState {
    bool ready = false;
    int sm_count = 0;
};
DeviceState g_dev[kMaxDevices];
int g_prefill_impl = 0;               // 0 = tcgen05, 1 = mma.sync
int g_decode_min_tiles = 1;
int g_decode_overlap = 0;
long long g_wait_cycles = 4000000000LL;   // bound of the device-side waits for peers' records (about two seconds)
unsigned long long g_launches = 0;
thread_local char g_cuda_err[256] = "";

// opt-in timing of the split-KV kernel (oattn_profile_enable)
cudaEvent_t* g_prof_ev = nullptr;   // 2 * g_prof_cap events: start, stop per record
int g_prof_cap = 0, g_prof_n = 0;

int cuda_fail(cudaError_t e, const char* where) {
    snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", where, cudaGetErrorString(e));
    return OATTN_ERR_CUDA;
}

inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

int check_shape(int n_head, int n_kv, int head_dim) {
    if (n_head <= 0 || n_kv <= 0) return OATTN_ERR_ARG;
    if (head_dim != 64 && head_dim != 128) return OATTN_ERR_UNSUPPORTED;
    if (n_head % n_kv != 0 || n_head / n_kv > 16) return OATTN_ERR_UNSUPPORTED;
    return OATTN_OK;
}

int check_rope(int fuse, const oattn_rope_params* rope, int head_dim, RopeArgs& r) {
    r = RopeArgs{0, 0, 10000.0f, nullptr};
    if (fuse & (OATTN_FUSE_ROPE_Q | OATTN_FUSE_ROPE_K)) {
        if (!rope) return OATTN_ERR_ARG;
        if (rope->rope_type != OATTN_ROPE_NORMAL && rope->rope_type != OATTN_ROPE_NEOX) return OATTN_ERR_ARG;
        if (rope->n_rot <= 0 || rope->n_rot > head_dim || (rope->n_rot & 1)) return OATTN_ERR_UNSUPPORTED;
        if (!(rope->theta > 0.0f)) return OATTN_ERR_ARG;
        r.rope_type = rope->rope_type;
        r.n_rot = rope->n_rot;
        r.theta = rope->theta;
        r.freq_factors = rope->freq_factors;
    }
    return OATTN_OK;
}

// State of the calling thread's current device, or nullptr before oattn_init() succeeded on it.
const DeviceState* cur_dev() {
    int d = -1;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDevices) return nullptr;
    return g_dev[d].ready ? &g_dev[d] : nullptr;
}
bool device_ready() { return cur_dev() != nullptr; }

DecodeWsLayout decode_ws(int n_head, int n_kv, int head_dim, int sm_count) {
    return decode_ws_layout(n_head, n_kv, head_dim, decode_num_splits(n_kv, sm_count));
}

} // namespace

extern "C" {

const char* oattn_strerror(int code) {
    switch (code) {
        case OATTN_OK: return "ok";
        case OATTN_ERR_ARG: return "invalid argument";
        case OATTN_ERR_UNSUPPORTED: return "shape not supported (head_dim 64/128, n_head/n_kv <= 16, even n_rot <= head_dim)";
        case OATTN_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case OATTN_ERR_CUDA: return "CUDA error";
        case OATTN_ERR_DEVICE: return "device not initialised or not compute capability 10.x";
        default: return "unknown error";
    }
}

const char* oattn_last_cuda_error(void) { return g_cuda_err; }

int oattn_init(int device) {
    cudaError_t e;
    if (device < 0) {       // the calling thread's current device
        if ((e = cudaGetDevice(&device)) != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    }
    if (device >= kMaxDevices) return OATTN_ERR_ARG;
    e = cudaSetDevice(device);
    if (e != cudaSuccess) return cuda_fail(e, "cudaSetDevice");
    int major = 0, sms = 0;
    if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device)) != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
    if (major != 10) return OATTN_ERR_DEVICE;
    if (!g_dev[device].ready) {
        if ((e = decode_set_attributes()) != cudaSuccess) return cuda_fail(e, "decode attributes");
        if ((e = prefill_mma_set_attributes()) != cudaSuccess) return cuda_fail(e, "prefill (mma) attributes");
        if ((e = prefill_tc_set_attributes()) != cudaSuccess) return cuda_fail(e, "prefill (tcgen05) attributes");
        void* scratch = nullptr;      // look the built-in scratch block up now, so that oattn_decode_noalloc never has to
        if ((e = decode_static_scratch(&scratch)) != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(built-in scratch)");
        unsigned* tickets = nullptr;  // ... and the arrival counters of the decode launches
        if ((e = decode_ticket_slot(nullptr, &tickets)) != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(arrival counters)");
        g_dev[device].sm_count = sms;
        g_dev[device].ready = true;
    }
    return OATTN_OK;
}

int oattn_scratch_alloc(size_t bytes, void** ptr) {
    if (!ptr || bytes == 0) return OATTN_ERR_ARG;
    if (!device_ready()) return OATTN_ERR_DEVICE;
    cudaError_t e = cudaMalloc(ptr, bytes);
    return e == cudaSuccess ? OATTN_OK : cuda_fail(e, "cudaMalloc(scratch)");
}

int oattn_scratch_free(void* ptr) {
    if (!ptr) return OATTN_OK;
    cudaError_t e = cudaFree(ptr);
    return e == cudaSuccess ? OATTN_OK : cuda_fail(e, "cudaFree(scratch)");
}

int oattn_builtin_scratch(void** ptr, size_t* bytes) {
    if (!ptr || !bytes) return OATTN_ERR_ARG;
    if (!device_ready()) return OATTN_ERR_DEVICE;
    cudaError_t e = decode_static_scratch(ptr);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(built-in scratch)");
    *bytes = kStaticScratchBytes;
    return OATTN_OK;
}

// ---- memory placement for a discrete GPU ---------------------------------------------------------------------
int oattn_weights_place(const void* host, size_t bytes, void** dev) {
    if (!host || !dev || bytes == 0) return OATTN_ERR_ARG;
    if (!device_ready()) return OATTN_ERR_DEVICE;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(weights)");
    e = cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) { cudaFree(p); return cuda_fail(e, "cudaMemcpy(weights)"); }
    *dev = p;
    return OATTN_OK;
}

int oattn_logits_alloc(size_t bytes, void** dev, void** pinned_host) {
    if (!dev || !pinned_host || bytes == 0) return OATTN_ERR_ARG;
    if (!device_ready()) return OATTN_ERR_DEVICE;
    void* d = nullptr;
    void* h = nullptr;
    cudaError_t e = cudaMalloc(&d, bytes);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(logits)");
    e = cudaHostAlloc(&h, bytes, cudaHostAllocDefault);
    if (e != cudaSuccess) { cudaFree(d); return cuda_fail(e, "cudaHostAlloc(logits)"); }
    *dev = d;
    *pinned_host = h;
    return OATTN_OK;
}

int oattn_logits_free(void* dev, void* pinned_host) {
    cudaError_t e = cudaSuccess;
    if (dev) e = cudaFree(dev);
    if (pinned_host && e == cudaSuccess) e = cudaFreeHost(pinned_host);
    return e == cudaSuccess ? OATTN_OK : cuda_fail(e, "logits free");
}

int oattn_copy_to_host_async(void* pinned_host, const void* dev, size_t bytes, void* stream) {
    if (!pinned_host || !dev) return OATTN_ERR_ARG;
    cudaError_t e = cudaMemcpyAsync(pinned_host, dev, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    return e == cudaSuccess ? OATTN_OK : cuda_fail(e, "cudaMemcpyAsync(device to host)");
}

int oattn_device_clear(void* dev, size_t bytes) {
    if (!dev) return OATTN_ERR_ARG;
    cudaError_t e = cudaMemset(dev, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    return e == cudaSuccess ? OATTN_OK : cuda_fail(e, "cudaMemset");
}

int oattn_sm_count(void) { const DeviceState* d = cur_dev(); return d ? d->sm_count : 0; }

int oattn_rope(float* x, int rows, int head_dim, int rope_type, int n_rot, float theta, int n_past, int heads,
               const int* d_pos, const float* freq_factors, void* stream) {
    if (!device_ready()) return OATTN_ERR_DEVICE;
    if (!x || rows < 0 || head_dim <= 0) return OATTN_ERR_ARG;
    if (rope_type != OATTN_ROPE_NORMAL && rope_type != OATTN_ROPE_NEOX) return OATTN_ERR_ARG;
    if (n_rot <= 0 || n_rot > head_dim || (n_rot & 1) || n_rot > 256) return OATTN_ERR_UNSUPPORTED;
    if (!d_pos && heads <= 0) return OATTN_ERR_ARG;
    RopeArgs r{rope_type, n_rot, theta, freq_factors};
    cudaError_t e = launch_rope(x, rows, head_dim, r, n_past, heads, d_pos, (cudaStream_t)stream, &g_launches);
    return e == cudaSuccess ? OATTN_OK : cuda_fail(e, "rope launch");
}

int oattn_kv_store(uint16_t* kc, uint16_t* vc, const float* k, const float* v, int heads, int head_dim, int n_ctx,
                   int pos_base, int batch, const int* d_pos, void* stream) {
    if (!device_ready()) return OATTN_ERR_DEVICE;
    if (!kc || !vc || !k || !v || heads <= 0 || head_dim <= 0 || n_ctx <= 0 || batch <= 0) return OATTN_ERR_ARG;
    if (d_pos && batch != 1) return OATTN_ERR_ARG;
    if (!d_pos && (pos_base < 0 || pos_base + batch > n_ctx)) return OATTN_ERR_ARG;
    cudaError_t e = launch_kv_store(kc, vc, k, v, heads, head_dim, n_ctx, pos_base, batch, d_pos, (cudaStream_t)stream, &g_launches);
    return e == cudaSuccess ? OATTN_OK : cuda_fail(e, "kv_store launch");
}

int oattn_kv_shift(uint16_t* kc, uint16_t* vc, int n_layer, int n_kv, int head_dim, int n_ctx, int n_keep, int shift,
                   void* stream) {
    if (!device_ready()) return OATTN_ERR_DEVICE;
    if (!kc || !vc || n_layer <= 0 || n_kv <= 0 || n_ctx <= 0) return OATTN_ERR_ARG;
    if (head_dim <= 0 || (head_dim % 16) != 0) return OATTN_ERR_UNSUPPORTED;
    if (n_keep < 0 || shift <= 0 || n_keep + shift > n_ctx) return OATTN_ERR_ARG;
    cudaError_t e = launch_kv_shift(kc, vc, n_layer, n_kv, head_dim, n_ctx, n_keep, shift, (cudaStream_t)stream, &g_launches);
    return e == cudaSuccess ? OATTN_OK : cuda_fail(e, "kv_shift launch");
}

size_t oattn_decode_workspace_bytes(int n_head, int n_kv, int head_dim) {
    const DeviceState* d = cur_dev();
    if (!d || check_shape(n_head, n_kv, head_dim) != OATTN_OK) return 0;
    return decode_ws(n_head, n_kv, head_dim, d->sm_count).total;
}

struct PeerTarget {
    const unsigned long long* bufs = nullptr;
    int* gen_push = nullptr;
    int rank = 0, world = 1;
    int fused_wait = 0;
    int* status = nullptr;
    const int* rope_pos = nullptr;
};

// Checks an extension block and copies it into the kernel arguments.  k/v bias and k norm act on the appended row,
// so they need the fused append; the q8_1 output exists for the decode call only.
static int apply_ext(const oattn_ext* ext, int fuse, bool allow_q8, int n_head, int n_kv, PreArgs& pre, int8_t** out_qs,
                     float** out_scales) {
    if (!ext) return OATTN_OK;
    const bool append = (fuse & OATTN_FUSE_KV_APPEND) != 0;
    if ((ext->bias_k || ext->bias_v || ext->norm_k) && !append) return OATTN_ERR_ARG;
    if ((ext->norm_q || ext->norm_k) && !(ext->norm_eps >= 0.0f)) return OATTN_ERR_ARG;
    if ((ext->out_qs != nullptr) != (ext->out_scales != nullptr)) return OATTN_ERR_ARG;
    if (ext->out_qs && !allow_q8) return OATTN_ERR_UNSUPPORTED;
    if (ext->out_mmq && out_qs) return OATTN_ERR_UNSUPPORTED;           // the decode calls have the q8_1 form instead
    if ((ext->norm_q || ext->norm_k) && n_head + n_kv > 160) return OATTN_ERR_UNSUPPORTED;
    pre.bias_q = ext->bias_q; pre.bias_k = ext->bias_k; pre.bias_v = ext->bias_v;
    pre.norm_q = ext->norm_q; pre.norm_k = ext->norm_k; pre.eps = ext->norm_eps;
    if (out_qs) { *out_qs = ext->out_qs; *out_scales = ext->out_scales; }
    return OATTN_OK;
}

static int decode_common(const float* q, const float* k_new, const float* v_new, uint16_t* kc, uint16_t* vc, float* out,
                         int n_head, int n_kv, int head_dim, int n_ctx, const int* d_pos, int pos_bias, float scale,
                         int fuse, const oattn_rope_params* rope, int emit_partial, void* workspace, size_t workspace_bytes,
                         void* stream, const PeerTarget* peer = nullptr, const oattn_ext* ext = nullptr) {
    const DeviceState* dev = cur_dev();
    if (!dev) return OATTN_ERR_DEVICE;
    int rc = check_shape(n_head, n_kv, head_dim);
    if (rc != OATTN_OK) return rc;
    const bool q8_only = ext && ext->out_qs && !emit_partial;     // the fp32 output is optional next to the q8_1 one
    if (!q || !kc || !vc || (!out && !q8_only) || !d_pos || n_ctx <= 0 || !(scale > 0.0f)) return OATTN_ERR_ARG;
    // q, k_new, v_new and the biases are read, out is written, as float4
    if (((uintptr_t)out | (uintptr_t)q | (uintptr_t)k_new | (uintptr_t)v_new) & 15) return OATTN_ERR_ARG;
    if (ext && (((uintptr_t)ext->bias_q | (uintptr_t)ext->bias_k | (uintptr_t)ext->bias_v) & 15)) return OATTN_ERR_ARG;
    if (fuse & ~OATTN_FUSE_ALL) return OATTN_ERR_ARG;
    if ((fuse & OATTN_FUSE_ROPE_K) && !(fuse & OATTN_FUSE_KV_APPEND)) return OATTN_ERR_ARG;
    if ((fuse & OATTN_FUSE_KV_APPEND) && (!k_new || !v_new)) return OATTN_ERR_ARG;
    DecodeArgs a;
    if ((rc = check_rope(fuse, rope, head_dim, a.rope)) != OATTN_OK) return rc;
    if ((rc = apply_ext(ext, fuse, !emit_partial, n_head, n_kv, a.pre, &a.out_qs, &a.out_scales)) != OATTN_OK) return rc;
    const DecodeWsLayout w = decode_ws(n_head, n_kv, head_dim, dev->sm_count);
    if (!workspace || ((uintptr_t)workspace & 255) || workspace_bytes < w.total) return OATTN_ERR_WORKSPACE;
    if ((size_t)n_kv * (w.n_groups + 1) > (size_t)kTicketWords) return OATTN_ERR_UNSUPPORTED;
    a.q = q; a.k_new = k_new; a.v_new = v_new; a.kc = kc; a.vc = vc; a.out = out;
    uint8_t* wsb = reinterpret_cast<uint8_t*>(workspace);
    a.ws_o = reinterpret_cast<float*>(wsb + w.part_o);
    a.ws_ml = reinterpret_cast<float*>(wsb + w.part_ml);
    a.grp_o = reinterpret_cast<float*>(wsb + w.grp_o);
    a.grp_ml = reinterpret_cast<float*>(wsb + w.grp_ml);
    cudaError_t te = decode_ticket_slot(workspace, &a.tickets);
    if (te != cudaSuccess) return cuda_fail(te, "arrival counters");
    a.d_pos = d_pos; a.pos_bias = pos_bias;
    a.n_head = n_head; a.n_kv = n_kv; a.head_dim = head_dim; a.n_ctx = n_ctx;
    a.n_splits = w.n_splits; a.group = w.group; a.n_groups = w.n_groups; a.min_tiles = g_decode_min_tiles; a.overlap = g_decode_overlap;
    a.scale = scale; a.fuse = fuse; a.emit_partial = emit_partial;
    if (peer) {
        // the launch leaves this rank's record in the workspace; the exchange launch below sends it round
        a.d_rope_pos = peer->rope_pos;
        a.out = reinterpret_cast<float*>(wsb + w.rec);
        a.defer_final = 1;            // the kv heads' group results are merged by the exchange launch
    }
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    if (g_prof_ev && g_prof_n < g_prof_cap) {
        ev0 = g_prof_ev[2 * g_prof_n];
        ev1 = g_prof_ev[2 * g_prof_n + 1];
        ++g_prof_n;
    }
    cudaError_t e = launch_decode(a, (cudaStream_t)stream, &g_launches, ev0, ev1);
    if (e != cudaSuccess) return cuda_fail(e, "decode launch");
    if (peer) {
        e = launch_peer_exchange(a, peer->bufs, peer->gen_push, peer->rank, peer->world, peer->fused_wait, out, peer->status,
                                 g_wait_cycles, g_decode_overlap, (cudaStream_t)stream, &g_launches);
        if (e != cudaSuccess) return cuda_fail(e, "peer exchange launch");
    }
    return OATTN_OK;
}

int oattn_decode(const float* q, const float* k_new, const float* v_new, uint16_t* kc, uint16_t* vc, float* out,
                 int n_head, int n_kv, int head_dim, int n_ctx, const int* d_pos, float scale, int fuse,
                 const oattn_rope_params* rope, void* workspace, size_t workspace_bytes, void* stream) {
    return decode_common(q, k_new, v_new, kc, vc, out, n_head, n_kv, head_dim, n_ctx, d_pos, 1, scale, fuse, rope, 0,
                         workspace, workspace_bytes, stream);
}

int oattn_decode_ex(const float* q, const float* k_new, const float* v_new, uint16_t* kc, uint16_t* vc, float* out,
                    int n_head, int n_kv, int head_dim, int n_ctx, const int* d_pos, float scale, int fuse,
                    const oattn_rope_params* rope, const oattn_ext* ext, void* workspace, size_t workspace_bytes, void* stream) {
    return decode_common(q, k_new, v_new, kc, vc, out, n_head, n_kv, head_dim, n_ctx, d_pos, 1, scale, fuse, rope, 0,
                         workspace, workspace_bytes, stream, nullptr, ext);
}

size_t oattn_decode_noalloc_max_bytes(void) { return kStaticScratchBytes; }

int oattn_decode_noalloc(const float* q, const uint16_t* kc, const uint16_t* vc, float* out, int n_head, int n_kv,
                         int head_dim, int n_ctx, const int* d_pos, float scale, void* stream) {
    if (!device_ready()) {
        // first use on this device: set it up here (address look-ups, kernel attributes); keep it out of stream capture
        const int irc = oattn_init(-1);
        if (irc != OATTN_OK) return irc;
    }
    int rc = check_shape(n_head, n_kv, head_dim);
    if (rc != OATTN_OK) return rc;
    const DecodeWsLayout w = decode_ws(n_head, n_kv, head_dim, cur_dev()->sm_count);
    if (w.total > kStaticScratchBytes) {
        snprintf(g_cuda_err, sizeof(g_cuda_err),
                 "oattn_decode_noalloc: this shape needs %zu bytes of scratch, the built-in block holds %zu; use oattn_decode "
                 "with a caller-provided workspace", w.total, (size_t)kStaticScratchBytes);
        return OATTN_ERR_WORKSPACE;
    }
    void* scratch = nullptr;
    cudaError_t e = decode_static_scratch(&scratch);     // the address oattn_init looked up for this device
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(built-in scratch)");
    return decode_common(q, nullptr, nullptr, const_cast<uint16_t*>(kc), const_cast<uint16_t*>(vc), out, n_head, n_kv,
                         head_dim, n_ctx, d_pos, 1, scale, OATTN_FUSE_NONE, nullptr, 0, scratch, w.total, stream);
}

int oattn_decode_partial(const float* q, const uint16_t* kc, const uint16_t* vc, float* part, int n_head, int n_kv,
                         int head_dim, int n_ctx, const int* d_len, float scale, void* workspace, size_t workspace_bytes,
                         void* stream) {
    return decode_common(q, nullptr, nullptr, const_cast<uint16_t*>(kc), const_cast<uint16_t*>(vc), part, n_head, n_kv,
                         head_dim, n_ctx, d_len, 0, scale, OATTN_FUSE_NONE, nullptr, 1, workspace, workspace_bytes, stream);
}

size_t oattn_peer_buffer_bytes(int world, int n_head, int head_dim) {
    if (world < 1 || world > DECODE_MAX_RANKS || n_head <= 0 || (head_dim != 64 && head_dim != 128)) return 0;
    return peer_buffer_bytes(world, n_head, head_dim);
}

size_t oattn_peer_state_bytes(int n_head) { return n_head > 0 ? align256((size_t)(2 * n_head + 1) * sizeof(int)) : 0; }

int oattn_decode_partial_push(const float* q, const uint16_t* kc, const uint16_t* vc, int n_head, int n_kv, int head_dim,
                              int n_ctx, const int* d_len, float scale, void* workspace, size_t workspace_bytes,
                              const void* peer_bufs_dev, int rank, int world, void* state, void* stream) {
    if (!peer_bufs_dev || !state || world < 1 || world > DECODE_MAX_RANKS || rank < 0 || rank >= world) return OATTN_ERR_ARG;
    PeerTarget t;
    t.bufs = reinterpret_cast<const unsigned long long*>(peer_bufs_dev);
    t.gen_push = reinterpret_cast<int*>(state);
    t.rank = rank;
    t.world = world;
    // `out` is not written in this mode; pass the state block so that the common checks see a non-null pointer
    return decode_common(q, nullptr, nullptr, const_cast<uint16_t*>(kc), const_cast<uint16_t*>(vc),
                         reinterpret_cast<float*>(state), n_head, n_kv, head_dim, n_ctx, d_len, 0, scale, OATTN_FUSE_NONE, nullptr,
                         1, workspace, workspace_bytes, stream, &t);
}

int oattn_decode_peer(const float* q, const uint16_t* kc, const uint16_t* vc, float* out, int n_head, int n_kv, int head_dim,
                      int n_ctx, const int* d_len, float scale, void* workspace, size_t workspace_bytes,
                      const void* peer_bufs_dev, int rank, int world, void* state, void* stream) {
    if (!peer_bufs_dev || !state || !out || world < 1 || world > DECODE_MAX_RANKS || rank < 0 || rank >= world) return OATTN_ERR_ARG;
    PeerTarget t;
    t.bufs = reinterpret_cast<const unsigned long long*>(peer_bufs_dev);
    t.gen_push = reinterpret_cast<int*>(state);
    t.rank = rank;
    t.world = world;
    t.fused_wait = 1;
    t.status = reinterpret_cast<int*>(state) + 2 * n_head;
    return decode_common(q, nullptr, nullptr, const_cast<uint16_t*>(kc), const_cast<uint16_t*>(vc), out, n_head, n_kv,
                         head_dim, n_ctx, d_len, 0, scale, OATTN_FUSE_NONE, nullptr, 1, workspace, workspace_bytes, stream, &t);
}

int oattn_decode_peer_fused(const float* q, const float* k_new, const float* v_new, uint16_t* kc, uint16_t* vc, float* out,
                            int n_head, int n_kv, int head_dim, int n_ctx, const int* d_len, const int* d_rope_pos, float scale,
                            int fuse, const oattn_rope_params* rope, void* workspace, size_t workspace_bytes,
                            const void* peer_bufs_dev, int rank, int world, void* state, void* stream) {
    if (!peer_bufs_dev || !state || !out || world < 1 || world > DECODE_MAX_RANKS || rank < 0 || rank >= world) return OATTN_ERR_ARG;
    if ((fuse & (OATTN_FUSE_ROPE_Q | OATTN_FUSE_ROPE_K)) && !d_rope_pos) return OATTN_ERR_ARG;
    PeerTarget t;
    t.bufs = reinterpret_cast<const unsigned long long*>(peer_bufs_dev);
    t.gen_push = reinterpret_cast<int*>(state);
    t.rank = rank;
    t.world = world;
    t.fused_wait = 1;
    t.status = reinterpret_cast<int*>(state) + 2 * n_head;
    t.rope_pos = d_rope_pos;
    return decode_common(q, k_new, v_new, kc, vc, out, n_head, n_kv, head_dim, n_ctx, d_len, 0, scale, fuse, rope, 1,
                         workspace, workspace_bytes, stream, &t);
}

int oattn_peer_wait_combine(const void* my_buf, int world, float* out, int n_head, int head_dim, void* state, void* stream) {
    if (!device_ready()) return OATTN_ERR_DEVICE;
    if (!my_buf || !out || !state || n_head <= 0 || world < 1 || world > DECODE_MAX_RANKS) return OATTN_ERR_ARG;
    if (head_dim != 64 && head_dim != 128) return OATTN_ERR_UNSUPPORTED;
    int* st = reinterpret_cast<int*>(state);
    if ((uintptr_t)out & 15) return OATTN_ERR_ARG;
    cudaError_t e = launch_peer_wait_combine(my_buf, world, out, n_head, head_dim, st + n_head, st + 2 * n_head,
                                             g_wait_cycles, g_decode_overlap, (cudaStream_t)stream, &g_launches);
    return e == cudaSuccess ? OATTN_OK : cuda_fail(e, "peer wait/combine launch");
}

int oattn_peer_status(const void* state, int n_head, int* status) {
    if (!state || !status || n_head <= 0) return OATTN_ERR_ARG;
    cudaError_t e = cudaMemcpy(status, reinterpret_cast<const int*>(state) + 2 * n_head, sizeof(int), cudaMemcpyDeviceToHost);
    return e == cudaSuccess ? OATTN_OK : cuda_fail(e, "peer status read");
}

int oattn_combine(const float* parts, int n_parts, float* out, int n_head, int head_dim, void* stream) {
    if (!device_ready()) return OATTN_ERR_DEVICE;
    if (!parts || !out || n_head <= 0 || n_parts <= 0) return OATTN_ERR_ARG;
    if (head_dim != 64 && head_dim != 128) return OATTN_ERR_UNSUPPORTED;
    if (n_parts > DECODE_MAX_SPLITS) return OATTN_ERR_UNSUPPORTED;
    if (((uintptr_t)parts & 15) || ((uintptr_t)out & 15)) return OATTN_ERR_ARG;
    cudaError_t e = launch_combine_records(parts, n_parts, out, n_head, head_dim, (cudaStream_t)stream, &g_launches);
    return e == cudaSuccess ? OATTN_OK : cuda_fail(e, "combine launch");
}

size_t oattn_prefill_workspace_bytes(int n_head, int n_kv, int head_dim, int max_batch) {
    if (check_shape(n_head, n_kv, head_dim) != OATTN_OK || max_batch <= 0) return 0;
    return align256((size_t)max_batch * n_head * head_dim * sizeof(__half)) + 256;   // fp16 queries + status word
}

int oattn_prefill_status(const void* workspace, int n_head, int head_dim, int batch, int* status) {
    if (!workspace || !status || n_head <= 0 || head_dim <= 0 || batch <= 0) return OATTN_ERR_ARG;
    const size_t off = align256((size_t)batch * n_head * head_dim * sizeof(__half));
    cudaError_t e = cudaMemcpy(status, reinterpret_cast<const uint8_t*>(workspace) + off, sizeof(int), cudaMemcpyDeviceToHost);
    return e == cudaSuccess ? OATTN_OK : cuda_fail(e, "prefill status read");
}

int oattn_prefill(const float* q, const float* k_new, const float* v_new, uint16_t* kc, uint16_t* vc, float* out,
                  int n_head, int n_kv, int head_dim, int n_ctx, int n_past, int batch, float scale, int fuse,
                  const oattn_rope_params* rope, void* workspace, size_t workspace_bytes, void* stream) {
    return oattn_prefill_ex(q, k_new, v_new, kc, vc, out, n_head, n_kv, head_dim, n_ctx, n_past, batch, scale, fuse, rope,
                            nullptr, workspace, workspace_bytes, stream);
}

int oattn_prefill_ex(const float* q, const float* k_new, const float* v_new, uint16_t* kc, uint16_t* vc, float* out,
                     int n_head, int n_kv, int head_dim, int n_ctx, int n_past, int batch, float scale, int fuse,
                     const oattn_rope_params* rope, const oattn_ext* ext, void* workspace, size_t workspace_bytes,
                     void* stream) {
    const DeviceState* dev = cur_dev();
    if (!dev) return OATTN_ERR_DEVICE;
    int rc = check_shape(n_head, n_kv, head_dim);
    if (rc != OATTN_OK) return rc;
    const bool mmq_only = ext && ext->out_mmq;                         // the fp32 output is optional next to the block form
    if (!q || !kc || !vc || (!out && !mmq_only) || n_ctx <= 0 || !(scale > 0.0f)) return OATTN_ERR_ARG;
    if (mmq_only && (head_dim != 128 || g_prefill_impl != 0 || ((uintptr_t)ext->out_mmq & 15))) return OATTN_ERR_UNSUPPORTED;
    if (batch <= 0 || n_past < 0 || n_past + batch > n_ctx) return OATTN_ERR_ARG;
    if ((uintptr_t)out & 15) return OATTN_ERR_ARG;                     // the output is written in 16-byte pieces
    if (fuse & ~OATTN_FUSE_ALL) return OATTN_ERR_ARG;
    if ((fuse & OATTN_FUSE_ROPE_K) && !(fuse & OATTN_FUSE_KV_APPEND)) return OATTN_ERR_ARG;
    if ((fuse & OATTN_FUSE_KV_APPEND) && (!k_new || !v_new)) return OATTN_ERR_ARG;
    PrefillArgs a;
    if ((rc = check_rope(fuse, rope, head_dim, a.rope)) != OATTN_OK) return rc;
    if ((rc = apply_ext(ext, fuse, false, n_head, n_kv, a.pre, nullptr, nullptr)) != OATTN_OK) return rc;
    const size_t need = oattn_prefill_workspace_bytes(n_head, n_kv, head_dim, batch);
    if (!workspace || ((uintptr_t)workspace & 255) || workspace_bytes < need) return OATTN_ERR_WORKSPACE;
    a.q = q; a.k_new = k_new; a.v_new = v_new; a.kc = kc; a.vc = vc; a.out = out;
    a.q16 = reinterpret_cast<__half*>(workspace);
    a.status = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(workspace) + need - 256);
    a.n_head = n_head; a.n_kv = n_kv; a.head_dim = head_dim; a.n_ctx = n_ctx; a.n_past = n_past; a.batch = batch;
    a.scale = scale; a.fuse = fuse;
    if (mmq_only) { a.out_mmq = reinterpret_cast<uint8_t*>(ext->out_mmq); a.mmq_ds4 = ext->out_mmq_ds4; }
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = launch_prefill_prologue(a, s, &g_launches);
    if (e != cudaSuccess) return cuda_fail(e, "prefill prologue launch");
    if (g_prefill_impl == 0) {
        e = launch_prefill_tc(a, dev->sm_count, s, &g_launches);
        if (e == cudaSuccess) return OATTN_OK;
        if (e != cudaErrorNotSupported) return cuda_fail(e, "prefill (tcgen05) launch");
    }
    if (mmq_only) return OATTN_ERR_UNSUPPORTED;       // the block form is written by the tcgen05 kernel only
    e = launch_prefill_mma(a, s, &g_launches);
    return e == cudaSuccess ? OATTN_OK : cuda_fail(e, "prefill (mma) launch");
}

int oattn_set_prefill_impl(int impl) {
    if (impl != 0 && impl != 1) return OATTN_ERR_ARG;
    g_prefill_impl = impl;
    return OATTN_OK;
}

int oattn_set_decode_overlap(int mode) {
    if (mode < 0 || mode > 2) return OATTN_ERR_ARG;
    g_decode_overlap = mode;
    return OATTN_OK;
}

int oattn_set_wait_limit_cycles(long long cycles) {
    if (cycles < 1000) return OATTN_ERR_ARG;
    g_wait_cycles = cycles;
    return OATTN_OK;
}

int oattn_set_decode_min_tiles(int tiles) {
    if (tiles < 1 || tiles > 1024) return OATTN_ERR_ARG;
    g_decode_min_tiles = tiles;
    return OATTN_OK;
}

int oattn_profile_enable(int max_records) {
    if (max_records < 0 || max_records > (1 << 16)) return OATTN_ERR_ARG;
    if (g_prof_ev) {
        for (int i = 0; i < 2 * g_prof_cap; ++i) cudaEventDestroy(g_prof_ev[i]);
        delete[] g_prof_ev;
        g_prof_ev = nullptr;
    }
    g_prof_cap = g_prof_n = 0;
    if (max_records == 0) return OATTN_OK;
    g_prof_ev = new cudaEvent_t[2 * max_records];
    for (int i = 0; i < 2 * max_records; ++i) {
        cudaError_t e = cudaEventCreate(&g_prof_ev[i]);
        if (e != cudaSuccess) return cuda_fail(e, "cudaEventCreate");
    }
    g_prof_cap = max_records;
    return OATTN_OK;
}

int oattn_profile_collect(float* ms, int capacity, int* n_written) {
    if (!ms || !n_written || capacity < 0) return OATTN_ERR_ARG;
    int n = g_prof_n < capacity ? g_prof_n : capacity;
    for (int i = 0; i < n; ++i) {
        cudaError_t e = cudaEventSynchronize(g_prof_ev[2 * i + 1]);
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms[i], g_prof_ev[2 * i], g_prof_ev[2 * i + 1]);
        if (e != cudaSuccess) return cuda_fail(e, "profile collect");
    }
    *n_written = n;
    g_prof_n = 0;
    return OATTN_OK;
}

unsigned long long oattn_launch_count(void) { return g_launches; }

} // extern "C"
