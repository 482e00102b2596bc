/*
 * C ABI of libkriya_cuda: the B200 (sm_100a) backend for KriyaRT's paged KV-cache hot path.
 *
 * These entry points are what a `kriya-backend-cuda` crate binds in place of the attention /
 * KV dispatch sites of `MetalExecutor` (crates/kriya-backend-metal/src/encoder.rs, "enc:").
 * Each declaration cites the reference interface it replaces.  There is no CPU fallback: every
 * compute entry point launches CUDA kernels on the context's device or returns an error code.
 *
 * Conventions
 *   - All functions return 0 on success or a negative kriya_cuda_status; the message of the most
 *     recent failure on a context is available from kriya_cuda_last_error().
 *   - A context is single-threaded and non-re-entrant, like `&mut self` on the reference executor
 *     (enc:4756, crates/kriya-server/src/runtime.rs:19-27).
 *   - Pointers named *_dev are device pointers on the context's device; *_host are host pointers.
 *     Activations and the cache are 16-bit (bf16 or fp16 bit patterns, chosen at create time);
 *     plan arrays are int32; positions are uint32; partial softmax states are fp32.
 *   - Work is enqueued on the context's stream; host-pointer variants and kriya_cuda_sync()
 *     wait for completion, everything else returns as soon as the launch is queued.
 *   - The step path allocates nothing: pool, plan buffers, work list and scratch are sized at
 *     create time (enc:7,1957-2035) and an over-capacity plan is rejected with
 *     KRIYA_CUDA_INVALID_INPUT (enc:2159-2218).
 */
#ifndef KRIYA_CUDA_H
#define KRIYA_CUDA_H

#include <stddef.h>
#include <stdint.h>

#include "kriya_kv.h" /* kriya_cta_work_tile */

#ifdef __cplusplus
extern "C" {
#endif

typedef struct kriya_cuda_ctx kriya_cuda_ctx;

/* MetalError (enc:32-54) as status codes. */
typedef enum kriya_cuda_status {
    KRIYA_CUDA_OK = 0,
    KRIYA_CUDA_DEVICE_INIT_FAILED = -1, /* DeviceInitFailed */
    KRIYA_CUDA_INVALID_INPUT = -2,      /* InvalidExecutionInput */
    KRIYA_CUDA_EXECUTION_ERROR = -3,    /* ExecutionError: a CUDA call failed or a kernel reported a bad index / timeout */
    KRIYA_CUDA_UNSUPPORTED = -4,        /* UnsupportedProductionConfiguration: shape the kernels are not built for */
    KRIYA_CUDA_TIMEOUT = -5             /* kriya_cuda_sync() gave up waiting */
} kriya_cuda_status;

enum { KRIYA_DTYPE_BF16 = 0, KRIYA_DTYPE_FP16 = 1 };
/* Storage of the KV cache.  KRIYA_KV_Q4_GROUP32 is DType::Q4KvGroup32 (crates/kriya-core/src/tensor.rs:50-51,77,91; switched
 * on by compress_kv_cache_q4, crates/kriya-core/src/hardware.rs:57,159-165): every 32 values of a cached K or V row are 16
 * bytes of 4-bit codes + f16 scale + f16 min = 20 bytes, value = code * scale + min.  Activations stay 16-bit. */
enum { KRIYA_KV_16BIT = 0, KRIYA_KV_Q4_GROUP32 = 1 };

/* RopeKvWriteParams, 48 bytes, byte-identical to enc:159-174 / paged_gqa_and_deltanet.metal:72-85. */
typedef struct kriya_rope_kv_write_params {
    uint32_t num_q_heads;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    uint32_t rotary_dim;
    uint32_t block_size_tokens;
    uint32_t apply_qk_norm;
    float rms_eps;
    float rope_theta;
    uint32_t max_seq_len;
    uint32_t has_table;
    uint32_t _pad0;
    uint32_t _pad1;
} kriya_rope_kv_write_params;

/* BsrGqaParams, 32 bytes, byte-identical to enc:176-187 / paged_gqa_and_deltanet.metal:60-69. */
typedef struct kriya_bsr_gqa_params {
    uint32_t num_q_heads;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    uint32_t block_size_tokens;
    uint32_t max_split_k_tiles;
    uint32_t max_query_tokens;
    float sm_scale;
    float logit_softcap;
} kriya_bsr_gqa_params;

/* What `MetalExecutor::new(desc, shader_dir, ckpt, num_kv_blocks, block_size_tokens)` (enc:1680-1696)
 * derives from the model descriptor for this path, plus capacities.  Zero capacities pick defaults
 * derived from num_kv_blocks (the reference's fixed 1024 / 16384 / 4096 entries, enc:1964-1967, are
 * too small for long contexts). */
typedef struct kriya_cuda_config {
    int32_t device;              /* CUDA device ordinal */
    uint32_t num_layers;         /* layers sharing the pool; layer l starts at l * layer stride (enc:2061) */
    uint32_t num_kv_blocks;      /* physical blocks per layer */
    uint32_t block_size_tokens;  /* tokens per block (kernels are built for 16) */
    uint32_t num_q_heads;
    uint32_t num_kv_heads;
    uint32_t head_dim;           /* 64 or 128 */
    uint32_t dtype;              /* KRIYA_DTYPE_* storage of activations and cache */
    uint32_t rotary_dim;         /* 0 -> head_dim (enc:1929-1933) */
    float rope_theta;
    uint32_t rope_max_seq_len;   /* rows of the fp32 cos/sin table; 0 -> 4096 (enc:1939) */
    uint32_t max_batch_rows;     /* plan rows (sequences) per step; 0 -> 1024 */
    uint32_t max_page_indices;   /* page_indices entries per plan; 0 -> max(16384, num_kv_blocks) */
    uint32_t max_tiles;          /* cta_work_tiles entries per plan; 0 -> 4096 */
    uint32_t max_query_tokens;   /* tokens per append / prefill call; 0 -> 8192 */
    uint32_t kv_format;          /* KRIYA_KV_*: 16-bit cache (default) or Q4KvGroup32 */
} kriya_cuda_config;

/* ---- context ------------------------------------------------------------------------------- */

/* MetalExecutor::new / new_internal (enc:1680-1696,1740-2035): selects the device, allocates the K
 * and V pools for all layers, the RoPE cos/sin table (enc:1939-1955), plan buffers and scratch. */
int32_t kriya_cuda_ctx_create(const kriya_cuda_config* cfg, kriya_cuda_ctx** out_ctx);
void kriya_cuda_ctx_destroy(kriya_cuda_ctx* ctx);
/* Message of the last failure on `ctx`; with ctx == NULL, of the last failed kriya_cuda_ctx_create on
 * this thread.  The string stays valid until the next call on the same context / thread. */
const char* kriya_cuda_last_error(const kriya_cuda_ctx* ctx);
/* MetalExecutor::layer_kv_byte_offset (enc:2059-2063). */
uint64_t kriya_cuda_layer_kv_byte_offset(const kriya_cuda_ctx* ctx, uint32_t layer);
/* Device base pointers of one layer's K and V pools, laid out [num_kv_blocks][block][Hkv][D] 16-bit
 * (kv_cache_k_buf / kv_cache_v_buf + layer offset, enc:1890-1894,4969-4970).  For tests and for hosts
 * that fill the cache themselves. */
int32_t kriya_cuda_kv_pool_ptrs(kriya_cuda_ctx* ctx, uint32_t layer, void** out_k_dev, void** out_v_dev);
/* The CUDA stream (cudaStream_t) all work of this context is queued on. */
void* kriya_cuda_stream(kriya_cuda_ctx* ctx);
/* wait_for_gpu (enc:2070-2109): waits until queued work has finished, polling; timeout_ms == 0 waits
 * without limit.  Also surfaces errors reported by kernels (bad block index, bounded wait expired). */
int32_t kriya_cuda_sync(kriya_cuda_ctx* ctx, uint32_t timeout_ms);

/* ---- per-step plan ("plan once, run per layer", crates/kriya-kv/src/bsr_paged.rs:299-301) -------- */

/* The copy of tokens/positions/indptr/indices/last_len/tiles into the executor's buffers
 * (enc:4803-4846) preceded by validate_batch_inputs (enc:2159-2218).  All pointers are host memory
 * and may be dropped when the call returns.  Besides capacities this checks what the kernels rely on:
 * indptr monotone from 0, 0 <= page_indices < num_kv_blocks, 1 <= last_page_len <= block size, tiles
 * inside their row.  The plan stays current for every following append / decode / prefill call on
 * any layer until the next upload.  `seq_positions` has one entry per row for decode, one per token
 * for prefill (n_positions says how many). */
int32_t kriya_cuda_plan_upload(kriya_cuda_ctx* ctx, const int32_t* page_indptr_host, size_t indptr_len,
                               const int32_t* page_indices_host, size_t indices_len,
                               const int32_t* last_page_len_host, size_t last_len_len,
                               const kriya_cta_work_tile* tiles_host, size_t tiles_len,
                               const uint32_t* seq_positions_host, size_t n_positions);

/* ---- the hot path ----------------------------------------------------------------------------- */

/* fused_qknorm_rope_and_kv_append (paged_gqa_and_deltanet.metal:115-226; dispatch enc:4945-4983 and
 * enc:4218-4256).  Row r of q/k/v is token r of the current plan: q is rotated in place, K is rotated
 * into slot (page_indices[indptr[r+1]-1], last_page_len[r]-1) of `layer`, V is copied bit for bit.
 * Uses the context's cos/sin table when params->has_table != 0 and the position is inside it,
 * otherwise pow/cos/sin on the device.  q_norm_w / k_norm_w may be NULL when apply_qk_norm == 0. */
int32_t kriya_cuda_rope_kv_append(kriya_cuda_ctx* ctx, uint32_t layer, void* q_inout_dev, const void* k_in_dev,
                                  const void* v_in_dev, const void* q_norm_w_dev, const void* k_norm_w_dev,
                                  uint32_t num_tokens, const kriya_rope_kv_write_params* params);

/* Chunked-prefill append: the same kernel for a chunk of `num_tokens` tokens of ONE sequence whose
 * block table is row 0 of the current plan; token i lands at absolute position prefix_tokens + i.
 * Replaces the per-token BSR rows of build_parallel_prefill_layout (bsr_paged.rs:607-667), which grow
 * as O(tokens x blocks), by (table, prefix, count).  Positions for RoPE are prefix_tokens + i. */
int32_t kriya_cuda_rope_kv_append_chunk(kriya_cuda_ctx* ctx, uint32_t layer, void* q_inout_dev, const void* k_in_dev,
                                        const void* v_in_dev, const void* q_norm_w_dev, const void* k_norm_w_dev,
                                        uint32_t prefix_tokens, uint32_t num_tokens,
                                        const kriya_rope_kv_write_params* params);

/* The same for the chunks of several sequences in ONE launch, with the arguments of kriya_cuda_paged_gqa_prefill_batch:
 * plan row r is sequence r's block table, its count_host[r] tokens are rows q_start_host[r] .. of q / k / v and land at
 * absolute positions prefix_host[r] + i.  (The reference appends per request, enc:4218-4256, one forward_prefill_batch
 * call each, crates/kriya-server/src/runtime.rs:315-377.) */
int32_t kriya_cuda_rope_kv_append_chunk_batch(kriya_cuda_ctx* ctx, uint32_t layer, void* q_inout_dev, const void* k_in_dev,
                                              const void* v_in_dev, const void* q_norm_w_dev, const void* k_norm_w_dev,
                                              uint32_t n_seqs, const uint32_t* q_start_host, const uint32_t* prefix_host,
                                              const uint32_t* count_host, const kriya_rope_kv_write_params* params);

/* bsr_paged_gqa_decode_stage1 + bsr_paged_gqa_split_k_reduce (paged_gqa_and_deltanet.metal:242-495,
 * 1474-1525; dispatch enc:4986-5053) behind one call.  For every row r of the current plan, query
 * heads q[r] attend over all blocks of the row (last block limited to last_page_len[r]); out[r] gets
 * the normalised result in the storage dtype.  The query heads of one KV head are processed together
 * so each cached K/V element is read once; long rows are split along the KV axis by the library's own
 * balanced work list and merged by the last work item to finish (the caller's cta_work_tiles are
 * validated but do not constrain the split).  q and out are [rows][Hq][D]. */
int32_t kriya_cuda_paged_gqa_decode(kriya_cuda_ctx* ctx, uint32_t layer, const void* q_dev, void* out_dev,
                                    const kriya_bsr_gqa_params* params);

/* Decode restricted to a block range of every row, returning the un-normalised softmax state instead
 * of the output: m [rows][Hq] (running maximum, natural-log units, -inf for an empty range),
 * l [rows][Hq] and o [rows][Hq][D], all fp32.  Row r covers logical blocks
 * [blk_begin_host[r], blk_end_host[r]) (both NULL: the ranges of the last
 * kriya_cuda_plan_set_ranges on this plan, else the whole row).  This is the per-GPU half of splitting
 * one long sequence along the KV axis; kriya_cuda_merge_states() finishes it.  The reference has no
 * multi-GPU path; the state is the (max, sum, output) triple of its split-K design
 * (paged_gqa_and_deltanet.metal:328-342). */
int32_t kriya_cuda_paged_gqa_decode_partial(kriya_cuda_ctx* ctx, uint32_t layer, const void* q_dev,
                                            const uint32_t* blk_begin_host, const uint32_t* blk_end_host,
                                            float* out_m_dev, float* out_l_dev, float* out_o_dev,
                                            const kriya_bsr_gqa_params* params);

/* Sets the block ranges once for the current plan (they stay until the next plan upload): the partial-state decode of
 * every following layer can then pass NULL ranges and re-uses the work split instead of rebuilding it per call. */
int32_t kriya_cuda_plan_set_ranges(kriya_cuda_ctx* ctx, const uint32_t* blk_begin_host, const uint32_t* blk_end_host);

/* Merge `parts` partial states laid out [parts][rows*Hq] (m, l) and [parts][rows*Hq][D] (o), e.g.
 * gathered from all ranks, into the normalised 16-bit output [rows*Hq][D]: the split-K reduce
 * (paged_gqa_and_deltanet.metal:1493-1524) on (m, l, o). */
int32_t kriya_cuda_merge_states(kriya_cuda_ctx* ctx, const float* m_dev, const float* l_dev, const float* o_dev,
                                uint32_t parts, uint32_t rows_times_heads, void* out_dev);

/* The same merge for states that were gathered as ONE buffer per part: part s occupies
 * packed[s * R * (D + 2) ...] as [m (R) | l (R) | o (R * D)], R = rows_times_heads.  A rank points the m / l / o outputs of
 * kriya_cuda_paged_gqa_decode_partial into such a buffer and needs a single all-gather per layer. */
int32_t kriya_cuda_merge_packed_states(kriya_cuda_ctx* ctx, const float* packed_dev, uint32_t parts,
                                       uint32_t rows_times_heads, void* out_dev);

/* ---- one long sequence split along the KV axis over the GPUs of one box ----------------------------------------
 * The reference is single-GPU (crates/kriya-scheduler/src/orca_engine.rs:21-24: one ColocatedHybrid role); these entry
 * points carry its split-K design (paged_gqa_and_deltanet.metal:328-342,1493-1524) across devices.  Every rank (one
 * context per GPU, in one process or in several) holds a contiguous block range of each row in its own pool.  Set-up, once:
 *   1. every rank calls kriya_cuda_comm_export() and hands the 128-byte handle to all other ranks by whatever channel
 *      the host has (the handle is plain bytes);
 *   2. every rank calls kriya_cuda_comm_init() with the handles of all ranks, ordered by rank.
 * Per step: kriya_cuda_plan_upload(), kriya_cuda_plan_set_ranges() with the rank's block range, then
 * kriya_cuda_kvsplit_decode() per layer (or kriya_cuda_kvsplit_decode_step() for all layers).  All ranks must make the
 * same sequence of kvsplit calls: the exchange pairs the n-th call of every rank.  The new token of a step is appended by
 * the rank that owns the row's last block, with kriya_cuda_rope_kv_append, before the call.
 * Data plane: no collective library.  After the partial-state decode one kernel stores the rank's (max, sum, output)
 * states into its slot of an exchange buffer in every peer's own memory (plain peer stores over NVLink), then waits, with a
 * bound of about a second, until the slots of all ranks in its OWN buffer carry this call's stamp, merges them and writes
 * the normalised output.  A peer that never delivers ends the wait with KRIYA_CUDA_EXECUTION_ERROR from the next
 * kriya_cuda_sync(); the context stays usable. */
#define KRIYA_COMM_MAX_RANKS 8
#define KRIYA_COMM_HANDLE_BYTES 128
/* Allocates this context's exchange buffer for plans of up to `max_rows` rows (set-up path: this allocates) and writes its
 * handle (KRIYA_COMM_HANDLE_BYTES bytes) to handle_out. */
int32_t kriya_cuda_comm_export(kriya_cuda_ctx* ctx, uint32_t max_rows, void* handle_out);
/* Maps the exchange buffers of all ranks: `handles` holds nranks handles of KRIYA_COMM_HANDLE_BYTES bytes each, ordered
 * by rank; handles[rank] must be this context's own.  Contexts of other processes are opened through CUDA IPC, contexts
 * of this process through peer access. */
int32_t kriya_cuda_comm_init(kriya_cuda_ctx* ctx, uint32_t nranks, uint32_t rank, const void* handles);
/* Partial-state decode over the rank's block ranges of the current plan, exchange, merge: out [rows][Hq][D] holds the
 * attention over the WHOLE rows on every rank.  Queued on the context's stream; the call does not wait. */
int32_t kriya_cuda_kvsplit_decode(kriya_cuda_ctx* ctx, uint32_t layer, const void* q_dev, void* out_dev,
                                  const kriya_bsr_gqa_params* params);
/* The same for every layer of the context in one call: q and out are [layers][rows][Hq][D]. */
int32_t kriya_cuda_kvsplit_decode_step(kriya_cuda_ctx* ctx, const void* q_dev, void* out_dev,
                                       const kriya_bsr_gqa_params* params);

/* bsr_paged_gqa_prefill_stage1 / _bq8 / bsr_paged_gqa_tiled_mma_prefill
 * (paged_gqa_and_deltanet.metal:508-847,851-1192,1206-1468; selection and dispatch enc:4262-4311).
 * Causal attention of a chunk of `num_tokens` queries of ONE sequence (row 0 of the current plan is
 * its block table, already holding the chunk's K/V) at absolute positions prefix_tokens + i over
 * cache positions 0..=prefix_tokens + i.  q and out are [num_tokens][Hq][D]. */
int32_t kriya_cuda_paged_gqa_prefill(kriya_cuda_ctx* ctx, uint32_t layer, const void* q_dev, void* out_dev,
                                     uint32_t prefix_tokens, uint32_t num_tokens, const kriya_bsr_gqa_params* params);

/* The same for the chunks of several sequences in ONE launch (the reference loops over requests on the host, one
 * forward_prefill_batch call each, crates/kriya-server/src/runtime.rs:315-377): plan row r is sequence r's block table;
 * its `count_host[r]` queries start at row `q_start_host[r]` of q / out and sit at absolute positions
 * `prefix_host[r] + i`.  All arrays are host memory with n_seqs entries. */
int32_t kriya_cuda_paged_gqa_prefill_batch(kriya_cuda_ctx* ctx, uint32_t layer, const void* q_dev, void* out_dev,
                                           uint32_t n_seqs, const uint32_t* q_start_host, const uint32_t* prefix_host,
                                           const uint32_t* count_host, const kriya_bsr_gqa_params* params);

/* Copy-on-write block copy: for every (src, dst) pair, in order, block dst := block src in every
 * layer, K and V.  Consumes the pairs produced by append_token_slot (bsr_paged.rs:412-420) and
 * collected in ScheduledIterationBatch.cow_block_copies (crates/kriya-scheduler/src/orca_engine.rs:
 * 267-278,359); the reference backend ships no consumer.  `pairs_host` is [n_pairs][2] uint32. */
int32_t kriya_cuda_kv_block_copy(kriya_cuda_ctx* ctx, const uint32_t* pairs_host, uint32_t n_pairs);

/* commit_speculative_kv (enc:3591-3664): row `node` of a staging buffer [nodes][Hkv*D] is copied bit
 * for bit into (block, slot) of `layer`'s K and V pools.  `triples_host` is [n][3] = (node, block, slot). */
int32_t kriya_cuda_kv_slot_write(kriya_cuda_ctx* ctx, uint32_t layer, const void* stage_k_dev, const void* stage_v_dev,
                                 const uint32_t* triples_host, uint32_t n);

/* ---- host-buffer step (end-to-end form) --------------------------------------------------------- */

/* One decode layer with HOST activations: copies q/k/v [rows][..] to the device, runs append then
 * decode on `layer` with the current plan, copies out [rows][Hq][D] back and waits.  This is the shape
 * of a forward_and_sample_batch call (enc:4756-4773) reduced to its attention ops: host inputs in,
 * host result out. */
int32_t kriya_cuda_decode_layer_host(kriya_cuda_ctx* ctx, uint32_t layer, const void* q_host, const void* k_host,
                                     const void* v_host, void* out_host, uint32_t rows,
                                     const kriya_rope_kv_write_params* rope, const kriya_bsr_gqa_params* gqa);

/* The append and the decode of one layer in ONE launch (head_dim 128, group size <= 8, no QK norm): queries are
 * rotated on their way into the attention kernel, and for every row the rotated new key and the new value are
 * written to their cache slot by the same kernel before it reads that page.  Cache contents and attention output
 * equal kriya_cuda_rope_kv_append followed by kriya_cuda_paged_gqa_decode (enc:4945-5053); q itself is NOT modified:
 * the rotated queries are written to q_rope_out [rows][Hq][D] when it is not NULL (it must not alias q). */
int32_t kriya_cuda_append_decode(kriya_cuda_ctx* ctx, uint32_t layer, const void* q_dev, const void* k_in_dev,
                                 const void* v_in_dev, void* out_dev, void* q_rope_out_dev,
                                 const kriya_rope_kv_write_params* rope, const kriya_bsr_gqa_params* gqa);
/* How kriya_cuda_decode_step / _host run a step.  Bit 0 (default set): use the fused launch where it applies; the step
 * then leaves q un-rotated, while with bit 0 clear q is rotated in place by the separate append kernel.  Bits 1-2 say how
 * the fused launch of layer l+1 relates to that of layer l (the first layer of a call is always an ordinary launch):
 *   0 (default)  the layers' inputs are independent and complete when the call is made, so a launch may begin while the
 *                previous layer's last thread blocks drain (programmatic dependent launch) and waits for nothing;
 *   1 (value 3)  serialised: a launch may be set up early (barriers, tensor memory) but reads and writes nothing before
 *                the previous layer has completed;
 *   2 (value 5)  layer l+1's activations depend on layer l (as in a model, where a projection sits between two attention
 *                layers): queries, the new K/V rows and outputs wait for the previous launch, the stream of cached K/V,
 *                which is older, starts at once;
 *   3 (value 7)  ordinary launches, one after the other.
 * Pass 1 for the default, 0 for separate kernels. */
int32_t kriya_cuda_set_fused_append(kriya_cuda_ctx* ctx, int32_t enable);

/* One decode step over ALL layers with device activations: for layer l = 0..num_layers-1, append then
 * decode with the current plan.  q/k/v/out hold the layers back to back: q and out [layers][rows][Hq][D],
 * k and v [layers][rows][Hkv][D].  One host call per step instead of two per layer; the per-layer loop of
 * forward_and_sample_impl (enc:4880-5053) reduced to its attention ops. */
int32_t kriya_cuda_decode_step(kriya_cuda_ctx* ctx, void* q_inout_dev, const void* k_dev, const void* v_dev,
                               void* out_dev, uint32_t rows, const kriya_rope_kv_write_params* rope,
                               const kriya_bsr_gqa_params* gqa);

/* The same step with HOST activations (pinned memory recommended): inputs are copied to the device, every
 * layer runs, out is copied back and the call waits.  The first call (and any call with more rows than
 * before) allocates the staging buffers; later calls allocate nothing. */
int32_t kriya_cuda_decode_step_host(kriya_cuda_ctx* ctx, const void* q_host, const void* k_host, const void* v_host,
                                    void* out_host, uint32_t rows, const kriya_rope_kv_write_params* rope,
                                    const kriya_bsr_gqa_params* gqa);

/* The same step in two halves, so that the host can prepare the next step (block allocation, next plan, even its upload,
 * which queues behind this step) while the GPU works: _begin queues the copies in, the layers and the copies back and
 * returns; _end waits until out_host is complete (timeout_ms as for kriya_cuda_sync).  The host buffers must stay
 * valid and untouched in between. */
int32_t kriya_cuda_decode_step_host_begin(kriya_cuda_ctx* ctx, const void* q_host, const void* k_host, const void* v_host,
                                          void* out_host, uint32_t rows, const kriya_rope_kv_write_params* rope,
                                          const kriya_bsr_gqa_params* gqa);
int32_t kriya_cuda_decode_step_host_end(kriya_cuda_ctx* ctx, uint32_t timeout_ms);

/* Chooses between the decode kernels, which compute the same result: 0 = by shape (for head_dim 128 a tensor-core kernel:
 * the one that moves whole pages of both KV heads with one copy where the shape is 2 KV heads, the one that moves one KV
 * head per copy otherwise; the CUDA-core kernel for head_dim 64), 1 = CUDA-core kernel, 2 = a tensor-core kernel (as 0,
 * refused where there is none), 3 = the one-KV-head-per-copy tensor-core kernel.  The reference picks kernels by shape in
 * the same way (enc:4262-4281); this switch exists so that tests can hold every kernel to the oracle.  The current plan's
 * work lists are cut for one kernel: upload the plan again after changing the path. */
int32_t kriya_cuda_set_decode_path(kriya_cuda_ctx* ctx, int32_t path);

/* Every wait inside a kernel of this library (on a copy, on another warp, on another thread block's partial state) is
 * bounded: when the limit passes, the kernel records a status word and returns, and the next kriya_cuda_sync() reports
 * KRIYA_CUDA_EXECUTION_ERROR ("a bounded wait inside a kernel expired") with the context still usable - the CUDA
 * counterpart of wait_for_gpu's bounded polling (enc:2070-2109).  The limit is 2 s unless set here (tensor-core decode
 * kernels; the other kernels keep 2 s). */
int32_t kriya_cuda_set_wait_limit_us(kriya_cuda_ctx* ctx, uint32_t limit_us);
/* Queues a one-block kernel that waits, with the context's limit, on a barrier nobody arrives at: the expiry path
 * exercised on purpose and without any fault.  The next kriya_cuda_sync() must return KRIYA_CUDA_EXECUTION_ERROR. */
int32_t kriya_cuda_selftest_wait_expiry(kriya_cuda_ctx* ctx);

/* Host only, no device needed: how a plan's rows are cut into pieces for the persistent tensor-core decode kernels (the
 * stream-K counterpart of the reference's split-K tile list, bsr_paged.rs:285-297, build_cta_work_tiles
 * kv_manager.rs:716-757).  `runs_per_row` is 1 for the whole-page kernel (a run = a plan row, both KV heads) and the number
 * of KV heads for the one-head-per-copy kernels; a tile is `pages_per_tile` blocks; a CTA is given at least `min_tiles`
 * tiles before another one is brought in; `window` as in kriya_cuda_set_attention_window (0 = none).  Writes one record of
 * 12 words per piece - row, KV head, first block, end block, scratch slot, the run's first slot, the run's piece count,
 * the row's offset in the page indices, its tokens, its first attended token, two zero words - in the order the CTAs
 * take them, and ctas + 1 offsets into that list.  Returns the number of records, or -1 when `cap` records do not suffice. */
int64_t kriya_cuda_debug_work_split(const int32_t* page_indptr, const int32_t* last_page_len, uint32_t rows,
                                    uint32_t block_size_tokens, uint32_t runs_per_row, uint32_t ctas, uint32_t pages_per_tile,
                                    uint32_t min_tiles, uint32_t window, uint32_t* out_records, uint32_t cap,
                                    uint32_t* out_cta_offsets);

/* AttentionMaskVariant::SlidingWindowCausal { window_size } (crates/kriya-core/src/descriptor.rs:63-70; declared by the
 * reference, read by none of its kernels).  With window_size > 0 a query at position p attends keys p + 1 - window_size
 * ..= p (itself included) in every following decode and prefill call; 0 (the default) is the plain causal mask.  Decode
 * rows then start at the window's first block, so the blocks in front of it are not read.  The setting takes part in
 * the work split: upload the plan again after changing it. */
int32_t kriya_cuda_set_attention_window(kriya_cuda_ctx* ctx, uint32_t window_size);

/* Per-kernel device timing.  While enabled, every decode (kind 0) and append (kind 1) launch is bracketed
 * by CUDA events on the context's stream; kriya_cuda_timing_read() waits for the stream, adds up the
 * finished brackets since the last read and returns launch count and total milliseconds per kind. */
int32_t kriya_cuda_timing_enable(kriya_cuda_ctx* ctx, int32_t enable);
int32_t kriya_cuda_timing_read(kriya_cuda_ctx* ctx, uint32_t kind, uint64_t* out_launches, double* out_total_ms);

/* Paged GQA decode without a context and without any allocation.  No counterpart in the reference: it exists for
 * hosts that may not call cudaMalloc (a process whose device memory is handed out up front by its own arena, or a plugin
 * inside such a process), and which therefore cannot own a kriya_cuda_ctx.
 * The caller passes every input and the output; the split-KV scratch (partial states, tickets, work list, status
 * word) lives in a fixed array of about 4.3 MB inside the library image, present on every GPU that loads the library
 * until the process exits.  Limits, rejected with KRIYA_CUDA_INVALID_INPUT and a message in `err`: at most 256 plan
 * rows, num_q_heads * head_dim <= 2048, at most 512 work items (long batches are cut coarser to fit).
 *   - q_dev / out_dev [rows][Hq][D], cache_*_dev one layer's pools [num_kv_blocks][16][Hkv][D], plan arrays as for
 *     kriya_cuda_plan_upload but already on the device; page_indptr_host is the same indptr on the host: the number of
 *     work items (the launch's grid) is computed from it, the items themselves are written on the device from
 *     page_indptr_dev, so the two must hold the same values.  Work is queued on `stream` (a cudaStream_t, may be 0);
 *     the call does not wait and nothing it queues reads host memory.  The caller's current device is left as it was.
 *   - The first call on a device looks up the array's device address; make that first call outside any stream
 *     capture.  Every call shares the array and starts by clearing its tickets and status word, so two calls whose
 *     kernels can overlap on the GPU (different streams, or different host threads) race: serialise them.
 *   - Page indices outside [0, num_kv_blocks) are not dereferenced (block 0 is read instead); there is no context
 *     to report them through, so validate tables on the host. */
int32_t kriya_cuda_paged_gqa_decode_static(int32_t device, void* stream, uint32_t dtype, const void* q_dev,
                                           const void* cache_k_dev, const void* cache_v_dev, uint32_t num_kv_blocks,
                                           const int32_t* page_indptr_host, const int32_t* page_indptr_dev,
                                           const int32_t* page_indices_dev, const int32_t* last_page_len_dev,
                                           uint32_t rows, void* out_dev, const kriya_bsr_gqa_params* params, char* err,
                                           size_t err_len);

/* TreeVerifyGqaParams (crates/kriya-backend-metal/src/encoder.rs:189-200; kernels/metal/paged_gqa_and_deltanet.metal:1604-1613),
 * byte-identical, 32 bytes. */
typedef struct kriya_tree_verify_params {
    uint32_t num_tree_nodes;    /* e.g. 11: the root and ten drafted nodes */
    uint32_t num_q_heads;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    uint32_t block_size_tokens;
    uint32_t prefix_kv_blocks;  /* blocks of cached context before the draft tree */
    uint32_t prefix_last_len;   /* valid tokens in the last of them */
    float sm_scale;
} kriya_tree_verify_params;

/* apply_rope_inplace (paged_gqa_and_deltanet.metal:1738-1829; dispatch enc:3258-3306): optional QK RMS norm and RoPE of
 * q [num_tokens][Hq][D] and k [num_tokens][Hkv][D] where they are; nothing is written to the cache.  Positions are the
 * ones uploaded with the current plan (num_tokens of them). */
int32_t kriya_cuda_rope_inplace(kriya_cuda_ctx* ctx, void* q_inout_dev, void* k_inout_dev, const void* q_norm_w_dev,
                                const void* k_norm_w_dev, uint32_t num_tokens, const kriya_rope_kv_write_params* params);

/* bsr_paged_gqa_tree_verify (paged_gqa_and_deltanet.metal:1620-1729; dispatch enc:3308-3345): every node i of a draft tree
 * attends the cached prefix and the in-flight K/V of the tree nodes j with tree_mask[i * n + j] != 0, in one call.
 * tree_q / tree_out are [n][Hq][D], tree_k / tree_v [n][Hkv][D] (q and k already rotated), tree_mask_host is n * n bytes
 * of host memory.  The prefix comes from the current plan: it must have exactly n rows, every row the sequence's
 * prefix table (prefix_kv_blocks blocks, last_page_len = prefix_last_len; build_schedule_plan with the sequence id
 * repeated n times) - the reference reads one table for all nodes, here each node is a decode row over the same
 * blocks.  prefix_kv_blocks = 0 verifies a tree without cached context.  At most 128 nodes. */
int32_t kriya_cuda_tree_verify(kriya_cuda_ctx* ctx, uint32_t layer, const void* tree_q_dev, const void* tree_k_dev,
                               const void* tree_v_dev, const uint8_t* tree_mask_host, void* tree_out_dev,
                               const kriya_tree_verify_params* params);

/* Number of kernels this library has launched on `ctx` since creation (for launch accounting). */
uint64_t kriya_cuda_launch_count(const kriya_cuda_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* KRIYA_CUDA_H */
