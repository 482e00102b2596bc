// A C++ host written against include/kriya_executor.hpp and include/kriya_kv.h: builds a plan with the C++ manager, then
// creates an executor.  Without a GPU the constructor must throw CudaError{DeviceInitFailed} (no CPU fallback); with one
// it runs one fused append + decode launch and waits for it.  Prints one line and exits 0 in both cases.
#include <cstdio>
#include <vector>

#include "kriya_executor.hpp"
#include "kriya_kv.h"

int main() {
    kriya_kv_manager* mgr = kriya_kv_create(64, 0, 16);
    if (!mgr) return 2;
    std::vector<uint32_t> tokens(40);
    for (uint32_t i = 0; i < tokens.size(); ++i) tokens[i] = 100 + i;
    size_t matched = 0;
    if (kriya_kv_allocate_sequence(mgr, 7, tokens.data(), tokens.size(), &matched) != KRIYA_KV_OK) return 3;
    const uint64_t ids[1] = {7};
    kriya_kv_plan_view view{};
    if (kriya_kv_build_schedule_plan(mgr, ids, 1, 8, &view) != KRIYA_KV_OK) return 4;
    if (view.page_indptr_len != 2 || view.page_indices_len != 3 || view.last_page_len[0] != 8) return 5;

    kriya_cuda_config cfg{};
    cfg.device = 0;
    cfg.num_layers = 1;
    cfg.num_kv_blocks = 64;
    cfg.block_size_tokens = 16;
    cfg.num_q_heads = 16;
    cfg.num_kv_heads = 2;
    cfg.head_dim = 128;
    cfg.dtype = KRIYA_DTYPE_BF16;
    cfg.rope_theta = 1e6f;
    try {
        kriya::CudaExecutor ex(cfg);
        const std::vector<uint32_t> positions = {39};
        ex.upload_plan(kriya::PlanRef(view), positions);
        ex.wait_for_gpu(10000);
        std::printf("executor created, plan uploaded, layer stride %llu bytes\n",
                    static_cast<unsigned long long>(ex.layer_kv_byte_offset(0)));
        try {  // an over-long position list must come back as InvalidExecutionInput, not as a crash
            const std::vector<uint32_t> bad(5000, 1);
            ex.upload_plan(kriya::PlanRef(view), bad);
        } catch (const kriya::CudaError& e) {
            if (e.kind != kriya::CudaErrorKind::InvalidExecutionInput) return 7;
        }
    } catch (const kriya::CudaError& e) {
        if (e.kind != kriya::CudaErrorKind::DeviceInitFailed) {
            std::printf("unexpected error kind %d: %s\n", int(e.kind), e.what());
            return 6;
        }
        std::printf("no usable GPU: DeviceInitFailed (%s)\n", e.what());
    }
    kriya_kv_destroy(mgr);
    return 0;
}
