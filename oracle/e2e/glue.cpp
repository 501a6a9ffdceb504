// TEST INFRASTRUCTURE: link-time glue of the e2e_b200 build.  The reference's kernels.cu stays in the link for its
// GEMV/GEMM/elementwise kernels and keeps its own set_stream (src/kernels.cu:1726-1728); the replacement library has
// a stream of its own.  The linker option --wrap sends model_gpu.cu's calls of llm::cuda::set_stream here, and this
// forwards them to both, so the unmodified model_gpu.cu drives both sets of kernels onto the same stream.
namespace llm::cuda {
void attn_set_stream(void* stream);
}

extern "C" void __real__ZN3llm4cuda10set_streamEPv(void* stream);

extern "C" void __wrap__ZN3llm4cuda10set_streamEPv(void* stream) {
    __real__ZN3llm4cuda10set_streamEPv(stream);
    llm::cuda::attn_set_stream(stream);
}
