// TEST INFRASTRUCTURE, force-included (-include) into the reference's model_gpu.cu for the e2e builds only.
// The reference keeps its weights in the memory-mapped file and lets the GPU read them through a zero-copy host
// mapping (src/model_gpu.cu:96-149), which suits a unified-memory Orin; on a discrete GPU every token would stream
// the weights over PCIe.  These three renames send the calls that set the mapping up to oracle/e2e/placement.cu,
// which puts the weights into device memory instead, without touching the reference's source.
#pragma once

#include <cuda_runtime.h>    // already seen by nvcc before this header, hence the explicit declarations
extern "C" cudaError_t e2e_host_register(void* ptr, size_t size, unsigned int flags);
extern "C" cudaError_t e2e_host_get_device_pointer(void** dev, void* host, unsigned int flags);
extern "C" cudaError_t e2e_host_unregister(void* ptr);

#define cudaHostRegister e2e_host_register
#define cudaHostGetDevicePointer e2e_host_get_device_pointer
#define cudaHostUnregister e2e_host_unregister
