// placeholder until the tcgen05 prefill kernel lands
#include "kriya_device.cuh"
bool kriya_prefill_supported(uint32_t, uint32_t, uint32_t, uint32_t) { return false; }
cudaError_t kriya_launch_prefill(const KriyaPrefillArgs&, uint32_t, uint32_t, uint32_t, int, cudaStream_t) {
    return cudaErrorNotSupported;
}
