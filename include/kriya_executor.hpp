// C++ host side above the C ABI of libkriya_cuda: the attention / KV-cache half of the reference's executor
// (`MetalExecutor`, crates/kriya-backend-metal/src/encoder.rs, "enc:") with the same method names, argument meaning
// and error behaviour.  Header-only, C++17; link with -lkriya_cuda (and -lkriya_kv for plans built by the C++
// manager).  The reference's host code is Rust; a `kriya-backend-cuda` crate binds the same C entry points, this
// class is the equivalent for hosts written in C++.
//
// Error behaviour: every method throws kriya::CudaError, whose `kind` mirrors MetalError (enc:32-54); the runtime's
// reaction (abort the request, free its KV, crates/kriya-server/src/runtime.rs:372-376) is unchanged.  Nothing
// aborts or traps.  An executor is single-threaded like `&mut self` on the reference.
#ifndef KRIYA_EXECUTOR_HPP
#define KRIYA_EXECUTOR_HPP

#include <array>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "kriya_cuda.h"

namespace kriya {

// MetalError (enc:32-54)
enum class CudaErrorKind {
    DeviceInitFailed,
    InvalidExecutionInput,
    ExecutionError,
    UnsupportedProductionConfiguration,
    Timeout,
};

class CudaError : public std::runtime_error {
  public:
    CudaError(CudaErrorKind k, int32_t status_code, const std::string& msg) : std::runtime_error(msg), kind(k), status(status_code) {}
    CudaErrorKind kind;
    int32_t status;  // the kriya_cuda_status the C ABI returned
};

inline CudaErrorKind error_kind_of(int32_t status) {
    switch (status) {
        case KRIYA_CUDA_DEVICE_INIT_FAILED: return CudaErrorKind::DeviceInitFailed;
        case KRIYA_CUDA_INVALID_INPUT: return CudaErrorKind::InvalidExecutionInput;
        case KRIYA_CUDA_UNSUPPORTED: return CudaErrorKind::UnsupportedProductionConfiguration;
        case KRIYA_CUDA_TIMEOUT: return CudaErrorKind::Timeout;
        default: return CudaErrorKind::ExecutionError;
    }
}

// FlashInferSchedulePlan as the executor consumes it (crates/kriya-kv/src/bsr_paged.rs:299-321): borrowed arrays, e.g.
// a kriya_kv_plan_view of the C++ manager or the vectors of a Rust plan.
struct PlanRef {
    const int32_t* page_indptr = nullptr;
    size_t page_indptr_len = 0;
    const int32_t* page_indices = nullptr;
    size_t page_indices_len = 0;
    const int32_t* last_page_len = nullptr;
    size_t last_page_len_len = 0;
    const kriya_cta_work_tile* cta_work_tiles = nullptr;
    size_t cta_work_tiles_len = 0;

    PlanRef() = default;
    explicit PlanRef(const kriya_kv_plan_view& v)
        : page_indptr(v.page_indptr), page_indptr_len(v.page_indptr_len), page_indices(v.page_indices),
          page_indices_len(v.page_indices_len), last_page_len(v.last_page_len), last_page_len_len(v.last_page_len_len),
          cta_work_tiles(v.cta_work_tiles), cta_work_tiles_len(v.cta_work_tiles_len) {}
};

class CudaExecutor {
  public:
    // MetalExecutor::new (enc:1680-1696): pools for all layers, RoPE table, plan buffers, scratch.
    explicit CudaExecutor(const kriya_cuda_config& cfg) : cfg_(cfg) {
        const int32_t rc = kriya_cuda_ctx_create(&cfg, &ctx_);
        if (rc != KRIYA_CUDA_OK) {
            const char* msg = kriya_cuda_last_error(nullptr);
            throw CudaError(error_kind_of(rc), rc, msg ? msg : "kriya_cuda_ctx_create failed");
        }
    }
    ~CudaExecutor() {
        if (ctx_) kriya_cuda_ctx_destroy(ctx_);
    }
    CudaExecutor(const CudaExecutor&) = delete;
    CudaExecutor& operator=(const CudaExecutor&) = delete;
    CudaExecutor(CudaExecutor&& o) noexcept : ctx_(o.ctx_), cfg_(o.cfg_) { o.ctx_ = nullptr; }
    CudaExecutor& operator=(CudaExecutor&& o) noexcept {
        if (this != &o) {
            if (ctx_) kriya_cuda_ctx_destroy(ctx_);
            ctx_ = o.ctx_;
            cfg_ = o.cfg_;
            o.ctx_ = nullptr;
        }
        return *this;
    }

    kriya_cuda_ctx* handle() const { return ctx_; }
    const kriya_cuda_config& config() const { return cfg_; }

    // layer_kv_byte_offset (enc:2059-2063)
    uint64_t layer_kv_byte_offset(uint32_t layer) const { return kriya_cuda_layer_kv_byte_offset(ctx_, layer); }
    // wait_for_gpu (enc:2070-2109)
    void wait_for_gpu(uint32_t timeout_ms = 0) { check(kriya_cuda_sync(ctx_, timeout_ms)); }
    void* stream() const { return kriya_cuda_stream(ctx_); }
    std::pair<void*, void*> kv_pool(uint32_t layer) {
        void *k = nullptr, *v = nullptr;
        check(kriya_cuda_kv_pool_ptrs(ctx_, layer, &k, &v));
        return {k, v};
    }

    // the parameter blocks the reference fills at its dispatch sites (enc:4945-4960, 4986-4996)
    kriya_rope_kv_write_params rope_params(bool apply_qk_norm = false, float rms_eps = 1e-6f) const {
        kriya_rope_kv_write_params p{};
        p.num_q_heads = cfg_.num_q_heads;
        p.num_kv_heads = cfg_.num_kv_heads;
        p.head_dim = cfg_.head_dim;
        p.rotary_dim = cfg_.rotary_dim ? cfg_.rotary_dim : cfg_.head_dim;
        p.block_size_tokens = cfg_.block_size_tokens;
        p.apply_qk_norm = apply_qk_norm ? 1u : 0u;
        p.rms_eps = rms_eps;
        p.rope_theta = cfg_.rope_theta;
        p.max_seq_len = cfg_.rope_max_seq_len ? cfg_.rope_max_seq_len : 4096u;
        p.has_table = 1u;
        return p;
    }
    kriya_bsr_gqa_params gqa_params(float sm_scale, uint32_t max_query_tokens = 1, float logit_softcap = 0.0f) const {
        kriya_bsr_gqa_params p{};
        p.num_q_heads = cfg_.num_q_heads;
        p.num_kv_heads = cfg_.num_kv_heads;
        p.head_dim = cfg_.head_dim;
        p.block_size_tokens = cfg_.block_size_tokens;
        p.max_split_k_tiles = 16;
        p.max_query_tokens = max_query_tokens;
        p.sm_scale = sm_scale;
        p.logit_softcap = logit_softcap;
        return p;
    }

    // ---- per-step plan: the copy of the plan into the executor's buffers (enc:4803-4846), once per step ----------
    void upload_plan(const PlanRef& plan, const uint32_t* seq_positions, size_t n_positions) {
        check(kriya_cuda_plan_upload(ctx_, plan.page_indptr, plan.page_indptr_len, plan.page_indices, plan.page_indices_len,
                                     plan.last_page_len, plan.last_page_len_len, plan.cta_work_tiles, plan.cta_work_tiles_len,
                                     seq_positions, n_positions));
    }
    void upload_plan(const PlanRef& plan, const std::vector<uint32_t>& seq_positions) {
        upload_plan(plan, seq_positions.data(), seq_positions.size());
    }

    // ---- decode: the three dispatches of enc:4945-5053 (append, decode stage 1, split-K reduce) ----------------------
    void rope_kv_append(uint32_t layer, void* q_inout, const void* k, const void* v, uint32_t num_tokens,
                        const kriya_rope_kv_write_params& p, const void* q_norm_w = nullptr, const void* k_norm_w = nullptr) {
        check(kriya_cuda_rope_kv_append(ctx_, layer, q_inout, k, v, q_norm_w, k_norm_w, num_tokens, &p));
    }
    void paged_gqa_decode(uint32_t layer, const void* q, void* out, const kriya_bsr_gqa_params& p) {
        check(kriya_cuda_paged_gqa_decode(ctx_, layer, q, out, &p));
    }
    // one launch per layer: RoPE + append + decode (q stays un-rotated; pass q_rope_out to receive the rotated queries)
    void attention_decode(uint32_t layer, const void* q, const void* k, const void* v, void* out,
                          const kriya_rope_kv_write_params& rope, const kriya_bsr_gqa_params& gqa, void* q_rope_out = nullptr) {
        check(kriya_cuda_append_decode(ctx_, layer, q, k, v, out, q_rope_out, &rope, &gqa));
    }
    // all layers of a step, activations [layers][rows][heads][D] back to back, on the device or in (pinned) host memory
    void decode_step(void* q_inout, const void* k, const void* v, void* out, uint32_t rows, const kriya_rope_kv_write_params& rope,
                     const kriya_bsr_gqa_params& gqa) {
        check(kriya_cuda_decode_step(ctx_, q_inout, k, v, out, rows, &rope, &gqa));
    }
    void decode_step_host_begin(const void* q, const void* k, const void* v, void* out, uint32_t rows,
                                const kriya_rope_kv_write_params& rope, const kriya_bsr_gqa_params& gqa) {
        check(kriya_cuda_decode_step_host_begin(ctx_, q, k, v, out, rows, &rope, &gqa));
    }
    void decode_step_host_end(uint32_t timeout_ms = 0) { check(kriya_cuda_decode_step_host_end(ctx_, timeout_ms)); }

    // ---- prefill: forward_prefill_batch's attention (enc:4218-4311) --------------------------------------------------
    // chunk of one sequence: plan = build_prefix_schedule_plan(seq, prefix_tokens + num_tokens)
    void prefill_chunk(uint32_t layer, void* q_inout, const void* k, const void* v, void* out, uint32_t prefix_tokens,
                       uint32_t num_tokens, const kriya_rope_kv_write_params& rope, const kriya_bsr_gqa_params& gqa,
                       const void* q_norm_w = nullptr, const void* k_norm_w = nullptr) {
        check(kriya_cuda_rope_kv_append_chunk(ctx_, layer, q_inout, k, v, q_norm_w, k_norm_w, prefix_tokens, num_tokens, &rope));
        check(kriya_cuda_paged_gqa_prefill(ctx_, layer, q_inout, out, prefix_tokens, num_tokens, &gqa));
    }
    // the chunks of several sequences in one launch (plan row r = sequence r); q already rotated and K/V appended
    void prefill_batch(uint32_t layer, const void* q, void* out, const std::vector<uint32_t>& q_start,
                       const std::vector<uint32_t>& prefix, const std::vector<uint32_t>& count, const kriya_bsr_gqa_params& gqa) {
        if (q_start.size() != prefix.size() || q_start.size() != count.size())
            throw CudaError(CudaErrorKind::InvalidExecutionInput, KRIYA_CUDA_INVALID_INPUT, "q_start, prefix and count differ in length");
        check(kriya_cuda_paged_gqa_prefill_batch(ctx_, layer, q, out, uint32_t(q_start.size()), q_start.data(), prefix.data(),
                                                 count.data(), &gqa));
    }

    // ---- prefix sharing and speculation ---------------------------------------------------------------------------
    // ScheduledIterationBatch.cow_block_copies (crates/kriya-scheduler/src/orca_engine.rs:172): before the step's appends
    void apply_cow_block_copies(const std::vector<std::pair<uint32_t, uint32_t>>& src_dst) {
        if (src_dst.empty()) return;
        static_assert(sizeof(std::pair<uint32_t, uint32_t>) == 8, "pairs are two packed u32");
        check(kriya_cuda_kv_block_copy(ctx_, reinterpret_cast<const uint32_t*>(src_dst.data()), uint32_t(src_dst.size())));
    }
    // commit_speculative_kv (enc:3591-3664): (node, block, slot) triples
    void commit_speculative_kv(uint32_t layer, const void* stage_k, const void* stage_v, const uint32_t* triples, uint32_t n) {
        check(kriya_cuda_kv_slot_write(ctx_, layer, stage_k, stage_v, triples, n));
    }
    // apply_rope_inplace + bsr_paged_gqa_tree_verify (enc:3258-3345); plan = one row per tree node over the prefix
    void rope_inplace(void* q_inout, void* k_inout, uint32_t num_tokens, const kriya_rope_kv_write_params& p,
                      const void* q_norm_w = nullptr, const void* k_norm_w = nullptr) {
        check(kriya_cuda_rope_inplace(ctx_, q_inout, k_inout, q_norm_w, k_norm_w, num_tokens, &p));
    }
    void tree_verify(uint32_t layer, const void* tree_q, const void* tree_k, const void* tree_v, const uint8_t* tree_mask_host,
                     void* tree_out, const kriya_tree_verify_params& p) {
        check(kriya_cuda_tree_verify(ctx_, layer, tree_q, tree_k, tree_v, tree_mask_host, tree_out, &p));
    }

    // the RoPE + append half of prefill_batch: the chunks of several sequences in one launch
    void append_chunk_batch(uint32_t layer, void* q_inout, const void* k, const void* v, const std::vector<uint32_t>& q_start,
                            const std::vector<uint32_t>& prefix, const std::vector<uint32_t>& count,
                            const kriya_rope_kv_write_params& rope, const void* q_norm_w = nullptr, const void* k_norm_w = nullptr) {
        if (q_start.size() != prefix.size() || q_start.size() != count.size())
            throw CudaError(CudaErrorKind::InvalidExecutionInput, KRIYA_CUDA_INVALID_INPUT, "q_start, prefix and count differ in length");
        check(kriya_cuda_rope_kv_append_chunk_batch(ctx_, layer, q_inout, k, v, q_norm_w, k_norm_w, uint32_t(q_start.size()),
                                                    q_start.data(), prefix.data(), count.data(), &rope));
    }

    // ---- AttentionMaskKind::SlidingWindowCausal { window_size } (crates/kriya-core/src/descriptor.rs:63-70); 0 = plain causal
    void set_attention_window(uint32_t window_size) { check(kriya_cuda_set_attention_window(ctx_, window_size)); }
    // bound of every wait inside a kernel (barriers, other CTAs' or GPUs' data); expiry surfaces as ExecutionError
    void set_wait_limit_us(uint64_t limit_us) { check(kriya_cuda_set_wait_limit_us(ctx_, limit_us)); }

    // ---- one sequence split along the KV axis over several GPUs (one executor per GPU) ---------------------------------
    // set-up: every rank exports the handle of its exchange buffer, the host passes all handles to every rank (rank order)
    std::array<uint8_t, KRIYA_COMM_HANDLE_BYTES> comm_export(uint32_t max_rows) {
        std::array<uint8_t, KRIYA_COMM_HANDLE_BYTES> h{};
        check(kriya_cuda_comm_export(ctx_, max_rows, h.data()));
        return h;
    }
    void comm_init(uint32_t rank, const std::vector<std::array<uint8_t, KRIYA_COMM_HANDLE_BYTES>>& handles) {
        check(kriya_cuda_comm_init(ctx_, uint32_t(handles.size()), rank, handles.data()));
    }
    // per plan: this rank's block range of every row; per layer (or per step): partial decode, exchange over NVLink, merge
    void set_kv_ranges(const uint32_t* blk_begin, const uint32_t* blk_end) { check(kriya_cuda_plan_set_ranges(ctx_, blk_begin, blk_end)); }
    void kvsplit_decode(uint32_t layer, const void* q, void* out, const kriya_bsr_gqa_params& gqa) {
        check(kriya_cuda_kvsplit_decode(ctx_, layer, q, out, &gqa));
    }
    void kvsplit_decode_step(const void* q, void* out, const kriya_bsr_gqa_params& gqa) {
        check(kriya_cuda_kvsplit_decode_step(ctx_, q, out, &gqa));
    }

    uint64_t launch_count() const { return kriya_cuda_launch_count(ctx_); }

  private:
    void check(int32_t rc) const {
        if (rc == KRIYA_CUDA_OK) return;
        const char* msg = kriya_cuda_last_error(ctx_);
        throw CudaError(error_kind_of(rc), rc, msg ? msg : "libkriya_cuda call failed");
    }

    kriya_cuda_ctx* ctx_ = nullptr;
    kriya_cuda_config cfg_{};
};

}  // namespace kriya

#endif  // KRIYA_EXECUTOR_HPP
