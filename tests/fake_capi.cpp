// Test-only stand-in for liborin_attn_b200.so: the entry points the C++ wrappers call, recording every call instead of
// launching anything.  Linked with orin_llm_b200/host/kernels.cpp and tests/host_shim.cpp it lets the CPU tests check
// the wrappers' host logic (first-use initialisation, scratch fall-backs, call-sequence fusion) without a GPU.
#include <stdlib.h>
#include <string.h>

#include <string>

#include "../include/orin_attn_b200.h"

namespace {
std::string g_log;
void note(const char* what) { g_log += what; g_log += ';'; }
void note_fuse(const char* what, int fuse) { g_log += what; g_log += '/'; g_log += std::to_string(fuse); g_log += ';'; }
}

extern "C" {

const char* fake_log(void) { return g_log.c_str(); }
void fake_log_clear(void) { g_log.clear(); }

const char* oattn_strerror(int) { return "fake"; }
const char* oattn_last_cuda_error(void) { return ""; }
int oattn_init(int device) { g_log += "init/" + std::to_string(device) + ";"; return OATTN_OK; }
int oattn_scratch_alloc(size_t bytes, void** ptr) { note("scratch_alloc"); *ptr = malloc(bytes); return OATTN_OK; }
int oattn_scratch_free(void* ptr) { note("scratch_free"); free(ptr); return OATTN_OK; }
int oattn_builtin_scratch(void** ptr, size_t* bytes) {
    static char block[8192];
    note("builtin_scratch");
    *ptr = block;
    *bytes = sizeof(block);
    return OATTN_OK;
}
int oattn_weights_place(const void*, size_t bytes, void** dev) { note("weights_place"); *dev = malloc(bytes); return OATTN_OK; }
int oattn_logits_alloc(size_t bytes, void** dev, void** host) { note("logits_alloc"); *dev = malloc(bytes); *host = malloc(bytes); return OATTN_OK; }
int oattn_logits_free(void* dev, void* host) { note("logits_free"); free(dev); free(host); return OATTN_OK; }
int oattn_copy_to_host_async(void*, const void*, size_t, void*) { note("copy_to_host"); return OATTN_OK; }
int oattn_device_clear(void*, size_t) { note("device_clear"); return OATTN_OK; }
int oattn_set_decode_overlap(int mode) { g_log += "overlap/" + std::to_string(mode) + ";"; return OATTN_OK; }
size_t oattn_decode_workspace_bytes(int, int, int) { return 4096; }
size_t oattn_prefill_workspace_bytes(int, int, int, int max_batch) { return 1024 * (size_t)max_batch; }

int oattn_rope(float*, int, int, int, int, float, int, int, const int*, const float*, void*) { note("rope"); return OATTN_OK; }
int oattn_kv_store(uint16_t*, uint16_t*, const float*, const float*, int, int, int, int, int, const int*, void*) {
    note("kv_store");
    return OATTN_OK;
}
int oattn_kv_shift(uint16_t*, uint16_t*, int, int, int, int, int, int, void*) { note("kv_shift"); return OATTN_OK; }
int oattn_decode(const float*, const float*, const float*, uint16_t*, uint16_t*, float*, int, int, int, int, const int*, float,
                 int fuse, const oattn_rope_params*, void*, size_t, void*) {
    note_fuse("decode", fuse);
    return OATTN_OK;
}
int oattn_decode_ex(const float*, const float*, const float*, uint16_t*, uint16_t*, float*, int, int, int, int, const int*,
                    float, int fuse, const oattn_rope_params*, const oattn_ext*, void*, size_t, void*) {
    note_fuse("decode_ex", fuse);
    return OATTN_OK;
}
int oattn_decode_noalloc(const float*, const uint16_t*, const uint16_t*, float*, int, int, int, int, const int*, float, void*) {
    note("decode_noalloc");
    return OATTN_OK;
}
int oattn_prefill(const float*, const float*, const float*, uint16_t*, uint16_t*, float*, int, int, int, int, int, int, float,
                  int fuse, const oattn_rope_params*, void*, size_t, void*) {
    note_fuse("prefill", fuse);
    return OATTN_OK;
}
int oattn_prefill_ex(const float*, const float*, const float*, uint16_t*, uint16_t*, float*, int, int, int, int, int, int,
                     float, int fuse, const oattn_rope_params*, const oattn_ext*, void*, size_t, void*) {
    note_fuse("prefill_ex", fuse);
    return OATTN_OK;
}

}  // extern "C"
