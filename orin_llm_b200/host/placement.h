// Memory placement of the reference's GPU runtime on a discrete GPU (B200).
//
// The reference's src/model_gpu.cu was written for a unified-memory Orin: weights are read through a zero-copy mapping
// of the memory-mapped model file (cudaHostRegister + cudaHostGetDevicePointer, src/model_gpu.cu:96-149), logits are
// written into mapped host memory (:210-211), and the KV cache is allocated but never cleared (:232-235).  On a B200
// every weight byte and every logit would then cross PCIe per token.  The functions below are what those three places
// call instead; INTEGRATION.md shows the six edited lines.  Definitions: kernels.cpp next to this file, on top of the
// memory-placement group of include/orin_attn_b200.h.  Errors print and abort, like the reference's CUDA_CHECK.
#pragma once

#include <stddef.h>

namespace llm::cuda {

// Copies the model file's tensor data [host_base, host_base + bytes) into device memory, once.  Afterwards
// placed_weight(p) maps any pointer into that range to its device address.  One range per process (the reference loads
// one model).  Replaces cudaHostRegister(mapped_ptr_, mapped_size_, ...) at src/model_gpu.cu:101.
void place_weights(const void* host_base, size_t bytes);
// Replaces cudaHostGetDevicePointer(&dp, s.src, 0) at src/model_gpu.cu:147.  Aborts for a pointer outside the range.
void* placed_weight(const void* host_ptr);
// Replaces cudaHostUnregister(mapped_ptr_) at src/model_gpu.cu:419.
void release_weights();

// Device buffer for the output head + pinned host buffer the host reads.  Replaces cudaHostAlloc(..., Mapped) and
// cudaHostGetDevicePointer at src/model_gpu.cu:210-211.
void logits_alloc(size_t bytes, float** d_logits, float** h_logits);
// Enqueues the device-to-host copy on the wrappers' current stream (set_stream); to be called right after the gemv that
// writes d_logits (src/model_gpu.cu:305, 334, 407).  Under stream capture it becomes the last node of the decode graph.
void logits_fetch(float* h_logits, const float* d_logits, size_t bytes);
void logits_free(float* d_logits, float* h_logits);

// Zero-fills the freshly allocated KV cache (src/model_gpu.cu:232-235 leaves it as cudaMalloc returned it) and waits.
void kv_cache_clear(void* base, size_t bytes);

} // namespace llm::cuda
