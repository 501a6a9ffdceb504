// placeholder until the tcgen05 kernel lands
#include "attn_internal.h"
namespace oattn {
cudaError_t prefill_tc_set_attributes() { return cudaSuccess; }
cudaError_t launch_prefill_tc(const PrefillArgs&, int, cudaStream_t, unsigned long long*) { return cudaErrorNotSupported; }
}
