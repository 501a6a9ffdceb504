// TEST INFRASTRUCTURE: device-memory placement of the reference's weights (see placement.h).
//   e2e_host_register(ptr, size)            allocates `size` bytes of device memory and copies the mapped file range in
//   e2e_host_get_device_pointer(&d, p)      p inside that range -> the matching device address; anything else (the
//                                           mapped logits buffer, src/model_gpu.cu:210-211) goes to the real call
//   e2e_host_unregister(ptr)                frees the device copy
#include <cuda_runtime.h>
#include <stdint.h>

namespace {
uint8_t* g_host = nullptr;
uint8_t* g_dev = nullptr;
size_t g_size = 0;
}

extern "C" cudaError_t e2e_host_register(void* ptr, size_t size, unsigned int) {
    cudaError_t e = cudaMalloc(&g_dev, size);
    if (e != cudaSuccess) return e;
    e = cudaMemcpy(g_dev, ptr, size, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return e;
    g_host = static_cast<uint8_t*>(ptr);
    g_size = size;
    return cudaSuccess;
}

extern "C" cudaError_t e2e_host_get_device_pointer(void** dev, void* host, unsigned int flags) {
    uint8_t* h = static_cast<uint8_t*>(host);
    if (g_host && h >= g_host && h < g_host + g_size) {
        *dev = g_dev + (h - g_host);
        return cudaSuccess;
    }
    return cudaHostGetDevicePointer(dev, host, flags);
}

extern "C" cudaError_t e2e_host_unregister(void* ptr) {
    if (ptr == g_host && g_dev) {
        cudaFree(g_dev);
        g_dev = nullptr;
        g_host = nullptr;
        g_size = 0;
    }
    return cudaSuccess;
}
