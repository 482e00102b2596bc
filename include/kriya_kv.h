/*
 * C ABI of the host-side paged KV bookkeeping (block allocator, radix prefix cache,
 * copy-on-write, BSR plan builders).
 *
 * In a KriyaRT build the Rust crate `kriya-kv` keeps this job unchanged; this library is
 * the compiled host side used where no Rust toolchain exists (tests, benchmark, C/C++
 * hosts).  Every entry point names the Rust method it mirrors, by file:line in
 * crates/kriya-kv/src/bsr_paged.rs, and must return bit-identical block ids, refcounts,
 * generations, CoW pairs and plan arrays.
 */
#ifndef KRIYA_KV_H
#define KRIYA_KV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct kriya_kv_manager kriya_kv_manager;

/* KvCacheError, bsr_paged.rs:12-24 */
enum {
    KRIYA_KV_OK = 0,
    KRIYA_KV_OUT_OF_BLOCKS = -1,       /* OutOfBlocks { requested, available } */
    KRIYA_KV_INVALID_SEQUENCE_ID = -2, /* InvalidSequenceId(u64) */
    KRIYA_KV_INVALID_BLOCK_ID = -3,    /* InvalidBlockId(u32) */
    KRIYA_KV_BAD_ARGUMENT = -4         /* null handle / null output pointer (no Rust counterpart) */
};

/* CtaWorkTile, #[repr(C)] 4 x u32, bsr_paged.rs:285-297 */
typedef struct kriya_cta_work_tile {
    uint32_t request_idx;
    uint32_t kv_block_start;
    uint32_t kv_block_count;
    uint32_t is_split_k;
} kriya_cta_work_tile;

/* FlashInferSchedulePlan + BsrKvLayout, bsr_paged.rs:274-321.  The arrays belong to the
 * manager and stay valid until the next plan is built on the same manager. */
typedef struct kriya_kv_plan_view {
    const int32_t* page_indptr;
    size_t page_indptr_len;
    const int32_t* page_indices;
    size_t page_indices_len;
    const int32_t* last_page_len;
    size_t last_page_len_len;
    const kriya_cta_work_tile* cta_work_tiles;
    size_t cta_work_tiles_len;
    uint32_t max_blocks_per_cta;
} kriya_kv_plan_view;

/* Details of the most recent error on this manager. */
typedef struct kriya_kv_error_info {
    int32_t code;
    uint64_t requested; /* OutOfBlocks.requested */
    uint64_t available; /* OutOfBlocks.available */
    uint64_t id;        /* offending sequence or block id */
} kriya_kv_error_info;

/* PagedKvCacheManager::new(num_gpu_blocks, _num_cpu_swap_blocks, block_size_tokens), bsr_paged.rs:332-338 */
kriya_kv_manager* kriya_kv_create(uint32_t num_gpu_blocks, uint32_t num_cpu_swap_blocks, uint32_t block_size_tokens);
void kriya_kv_destroy(kriya_kv_manager* m);
void kriya_kv_last_error(const kriya_kv_manager* m, kriya_kv_error_info* out);

/* BlockAllocator accessors, bsr_paged.rs:69-82,103-111,145-152 */
size_t kriya_kv_num_free_blocks(const kriya_kv_manager* m);
size_t kriya_kv_total_blocks(const kriya_kv_manager* m);
uint32_t kriya_kv_block_size_tokens(const kriya_kv_manager* m);
int32_t kriya_kv_ref_count(kriya_kv_manager* m, uint32_t block_id, uint32_t* out);
int32_t kriya_kv_generation(kriya_kv_manager* m, uint32_t block_id, uint64_t* out);
/* BlockAllocator::{allocate_block,inc_ref,free_block}, bsr_paged.rs:85-143 */
int32_t kriya_kv_allocate_block(kriya_kv_manager* m, uint32_t* out_block);
int32_t kriya_kv_inc_ref(kriya_kv_manager* m, uint32_t block_id);
int32_t kriya_kv_free_block(kriya_kv_manager* m, uint32_t block_id, int32_t* out_returned_to_pool);

/* PagedKvCacheManager::allocate_sequence, bsr_paged.rs:342-385 */
int32_t kriya_kv_allocate_sequence(kriya_kv_manager* m, uint64_t seq_id, const uint32_t* prompt_tokens, size_t len,
                                   size_t* out_matched_tokens);
/* append_token_slot, bsr_paged.rs:389-426.  *out_has_cow is 1 when a (src,dst) pair is returned. */
int32_t kriya_kv_append_token_slot(kriya_kv_manager* m, uint64_t seq_id, uint32_t* out_block, int32_t* out_has_cow,
                                   uint32_t* out_cow_src, uint32_t* out_cow_dst);
/* The scheduler's per-iteration loop over the running sequences (crates/kriya-scheduler/src/orca_engine.rs:267-278): one
 * append_token_slot per sequence, in order, collecting the copy-on-write pairs.  out_blocks holds n entries, out_cow_pairs
 * up to n (src, dst) pairs, *out_n_cow how many were emitted.  Stops at the first failing sequence (the error of
 * append_token_slot; *out_done says how many sequences were appended before it). */
int32_t kriya_kv_append_token_slots(kriya_kv_manager* m, const uint64_t* seq_ids, size_t n, uint32_t* out_blocks,
                                    uint32_t* out_cow_pairs, size_t* out_n_cow, size_t* out_done);
/* fork_sequence bsr_paged.rs:430-454, free_sequence :457-467, contains_sequence :471-473 */
int32_t kriya_kv_fork_sequence(kriya_kv_manager* m, uint64_t parent_seq_id, uint64_t child_seq_id);
int32_t kriya_kv_free_sequence(kriya_kv_manager* m, uint64_t seq_id);
int32_t kriya_kv_contains_sequence(const kriya_kv_manager* m, uint64_t seq_id);
/* block_for_position, bsr_paged.rs:477-493 */
int32_t kriya_kv_block_for_position(kriya_kv_manager* m, uint64_t seq_id, uint32_t position, uint32_t* out_block,
                                    uint32_t* out_slot);
/* Read-only view of one sequence's table (SequenceBlockTable, bsr_paged.rs:256-261). */
int32_t kriya_kv_sequence_table(kriya_kv_manager* m, uint64_t seq_id, const uint32_t** out_blocks, size_t* out_len,
                                uint32_t* out_total_tokens);

/* build_schedule_plan, bsr_paged.rs:497-544 */
int32_t kriya_kv_build_schedule_plan(kriya_kv_manager* m, const uint64_t* active_seq_ids, size_t n,
                                     uint32_t max_blocks_per_cta, kriya_kv_plan_view* out);
/* build_prefix_schedule_plan, bsr_paged.rs:550-594 */
int32_t kriya_kv_build_prefix_schedule_plan(kriya_kv_manager* m, uint64_t seq_id, uint32_t prefix_tokens,
                                            uint32_t max_blocks_per_cta, kriya_kv_plan_view* out);
/* build_parallel_prefill_layout, bsr_paged.rs:607-667 */
int32_t kriya_kv_build_parallel_prefill_layout(kriya_kv_manager* m, uint64_t seq_id, uint32_t prefix_tokens,
                                               uint32_t num_tokens, uint32_t max_blocks_per_cta,
                                               kriya_kv_plan_view* out);
/* build_deduplicated_prefill_layout, bsr_paged.rs:671-733 */
int32_t kriya_kv_build_deduplicated_prefill_layout(kriya_kv_manager* m, uint64_t seq_id, uint32_t prefix_tokens,
                                                   uint32_t num_tokens, uint32_t max_blocks_per_cta,
                                                   kriya_kv_plan_view* out);

#ifdef __cplusplus
}
#endif
#endif /* KRIYA_KV_H */
