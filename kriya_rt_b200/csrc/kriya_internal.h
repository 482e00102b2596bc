// Internal declarations shared by the translation units of libkriya_cuda.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <utility>
#include <vector>

#include "kriya_cuda.h"

// One unit of decode work: logical blocks [blk_begin, blk_end) of plan row `req`.
// `slot` is the index of this unit's partial state in the scratch arrays; the units of one row
// occupy slots [first_slot, first_slot + n_parts).
struct KriyaDecodeWork {
    uint32_t req;
    uint32_t blk_begin;
    uint32_t blk_end;
    uint32_t slot;
    uint32_t first_slot;
    uint32_t n_parts;
    uint32_t tok_first;  // first token of the row that may be attended (sliding window); 0 without a window
    uint32_t _pad1;
};
static_assert(sizeof(KriyaDecodeWork) == 32, "work item is 32 bytes");

// One piece of a (plan row, KV head) run for the tensor-core decode kernel: logical blocks [blk_lo, blk_hi).
// Pieces of one run occupy scratch slots [first_slot, first_slot + n_parts).
struct KriyaTcSeg {
    uint32_t req;
    uint32_t kv_head;
    uint32_t blk_lo;
    uint32_t blk_hi;
    uint32_t slot;
    uint32_t first_slot;
    uint32_t n_parts;
    uint32_t tbl_off;     // page_indptr[req]: where the row's block table starts
    uint32_t row_tokens;  // tokens in the whole row: (blocks - 1) * block size + last_page_len
    uint32_t tok_first;   // first token of the row that may be attended (sliding window); 0 without a window
    uint32_t _pad[2];
};
static_assert(sizeof(KriyaTcSeg) == 48, "segment record is 48 bytes");

// Device status word values written by kernels instead of trapping.
enum : uint32_t {
    KRIYA_DEV_OK = 0,
    KRIYA_DEV_BAD_BLOCK_INDEX = 1,  // a page index outside the pool reached a kernel
    KRIYA_DEV_WAIT_EXPIRED = 2,     // a bounded mbarrier wait gave up
    KRIYA_DEV_BAD_SLOT = 3          // append slot outside its block
};

struct kriya_comm_state;  // exchange buffers of the KV-axis split (kriya_comm.cu)
void kriya_comm_destroy(struct kriya_cuda_ctx* c);

struct kriya_cuda_ctx {
    kriya_cuda_config cfg{};
    kriya_comm_state* comm = nullptr;
    cudaStream_t stream = nullptr;
    cudaStream_t copy_stream = nullptr;      // host -> device inputs of whole-step host calls
    cudaStream_t copy_stream_out = nullptr;  // device -> host results
    cudaEvent_t ev_step_begin = nullptr, ev_step_end = nullptr;
    std::vector<cudaEvent_t> ev_in, ev_done;  // per input / output group of the host-buffer step
    int sm_count = 0;
    uint32_t tc_ctas = 0;  // largest grid of the tensor-core decode kernel variants: resident CTAs per SM x SMs
    // which tensor-core decode kernel the current plan's (range) lists are cut for: 0 = 128-token tiles of one KV head,
    // 1 = 64-token tiles of one KV head (two CTAs per SM), 2 = whole pages of both KV heads
    int tc_variant = 0, tc_variant_ranges = 0;
    int tc_force = 0;                            // KRIYA_TC_VARIANT: 128, 64 or 2 (whole pages)
    uint32_t tc64_min_tiles = 96;                // 128-token tiles per SM from which the 64-token-tile build is used
    int max_smem_optin = 0;
    // prefill launches with few query tiles are cut along the KV axis (KRIYA_PREFILL_SPLIT=0 switches that off, 2..8 forces that many pieces): states of
    // the pieces, one slot per (piece, head pair CTA)
    float* pf_part_o = nullptr;
    float* pf_part_ml = nullptr;
    uint32_t pf_part_slots = 0;
    bool pf_split_enable = true;
    uint32_t pf_split_force = 0;
    // Q4KvGroup32 cache: the chunked prefill reads K/V through tensor maps, so the blocks a plan names are expanded into
    // 16-bit staging pools (max_page_indices blocks each, plan order) in front of the attention launch; tmap_k / tmap_v then
    // cover the staging pools and the kernel walks them with the identity block table.
    uint8_t* q4_stage_k = nullptr;
    uint8_t* q4_stage_v = nullptr;
    int32_t* q4_identity = nullptr;
    bool q4_prefill_ok = false;

    // KV pools, all layers: layer l at l * layer_stride_bytes
    uint8_t* pool_k = nullptr;
    uint8_t* pool_v = nullptr;
    size_t layer_stride_bytes = 0;
    size_t block_bytes = 0;  // block_size * Hkv * D * 2

    // TMA tensor maps over the K and V pools (128-byte opaque blobs), valid when tmaps_ok
    alignas(64) unsigned char tmap_k[128];
    alignas(64) unsigned char tmap_v[128];
    bool tmaps_ok = false;
    // 5-D maps with one page (both KV heads) per box, valid when tcp_ok
    alignas(64) unsigned char tmap_kp[128];
    alignas(64) unsigned char tmap_vp[128];
    bool tcp_ok = false;

    float* rope_table = nullptr;  // [rope_max_seq_len][rotary_dim/2][2]
    uint32_t rope_rotary_dim = 0;

    // plan: one pinned host staging area, one device image, sub-arrays at fixed offsets
    uint8_t* h_plan[2] = {nullptr, nullptr};
    cudaEvent_t h_plan_free[2] = {nullptr, nullptr};
    int h_plan_cur = 0;
    uint8_t* d_plan = nullptr;
    size_t plan_bytes = 0;
    size_t off_indptr = 0, off_indices = 0, off_last_len = 0, off_tiles = 0, off_positions = 0, off_work = 0,
           off_range = 0, off_tcseg = 0, off_tcptr = 0, off_tcseg2 = 0, off_tcptr2 = 0, dyn_base = 0;
    uint32_t cap_seg = 0, n_seg = 0, n_seg_ranges = 0;
    uint32_t tc_max_parts = 0, tc_max_parts_ranges = 0;  // most pieces any run of the current (range) lists is cut into
    // Third work list of the whole-page decode kernel, for the launches of a whole-step call whose layers are declared
    // independent (layer_chain_mode 2): those launches overlap, so a CTA is given more tiles before another one is
    // brought in (fewer, longer streams per launch; a launch alone takes longer).  Built with every plan upload.
    size_t off_tcptr3 = 0, off_tcseg3 = 0;
    uint32_t n_seg_chain = 0, tc_max_parts_chain = 0, tc_chain_min_tiles = 14;
    bool chain_list_valid = false, use_chain_list = false;
    uint32_t layer_chain_mode = 2;  // KriyaFusedAppend::overlap_previous for the second and later layers of a whole-step call
    bool fuse_append = true;  // whole-step calls use the fused append + decode launch where it applies
    uint64_t wait_ns = 2000000000ull;  // limit of the bounded waits inside kernels (kriya_cuda_set_wait_limit_us)
    uint32_t attention_window = 0;  // SlidingWindowCausal window_size; 0 = plain causal
    int decode_path = 0;  // 0: pick per shape, 1: CUDA-core kernel, 2: tensor-core kernel, 3: tensor-core kernel with one KV head per copy
    uint32_t cap_rows = 0, cap_indices = 0, cap_tiles = 0, cap_tokens = 0, cap_work = 0;
    // current plan (host copy of the sizes and of what later calls need)
    bool plan_valid = false;
    uint32_t n_rows = 0, n_indices = 0, n_tiles = 0, n_positions = 0, n_work = 0;
    uint32_t row0_blocks = 0, row0_last_len = 0;
    uint64_t total_row_tokens = 0;
    uint8_t* h_plan_last = nullptr;  // staging buffer holding the current plan (for partial-range rebuilds)

    // split-KV scratch of the CUDA-core decode kernel
    float* part_o = nullptr;        // [cap_work][Hq][D]
    float* part_ml = nullptr;       // [cap_work][Hq][2]
    uint32_t* part_counter = nullptr;  // [cap_rows]
    // split-run scratch of the tensor-core decode kernel: kTcScratchSets sets, taken in turn by successive launches
    uint8_t* tc_ll_o = nullptr;     // per set: uint2 [cap_seg][G][128]
    uint8_t* tc_ll_ml = nullptr;    // per set: uint2 [cap_seg][G][2]
    uint32_t* tc_set_done = nullptr;  // per set, 64 bytes apart
    size_t tc_set_o_bytes = 0, tc_set_ml_bytes = 0;
    uint32_t tc_epoch = 0;
    uint32_t tc_done_expect[4] = {0, 0, 0, 0};
    bool ranges_valid = false;      // block ranges set for the current plan (kriya_cuda_plan_set_ranges)
    uint32_t n_work_ranges = 0;
    bool positions_are_context = false;  // current plan: seq_positions[r] == tokens in row r - 1 for every row
    uint32_t* d_status = nullptr;   // device status word
    uint32_t* h_status = nullptr;   // pinned mirror

    // staging for host-buffer entry points
    uint8_t* h_act = nullptr;  // pinned
    uint8_t* d_act = nullptr;
    size_t act_bytes = 0;
    uint32_t* d_pairs = nullptr;  // copy pairs / slot triples
    uint32_t* h_pairs = nullptr;
    uint32_t cap_pairs = 0;
    float* d_tree_state = nullptr;  // [kTreeMaxNodes * Hq * (D + 2)] prefix states of a tree verification
    uint8_t* d_tree_mask = nullptr;  // [kTreeMaxNodes^2] the tree mask of the last verification
    std::vector<uint8_t> tree_mask_last;  // its host copy: the layers of one verification pass the same mask
    cudaEvent_t h_pairs_free = nullptr;

    // staging for whole-step host calls (grown on demand by kriya_cuda_decode_step_host)
    uint8_t* d_step = nullptr;
    size_t step_bytes = 0;

    // optional per-kernel timing: event pairs around decode (kind 0) and append (kind 1) launches
    bool timing = false;
    std::vector<cudaEvent_t> ev_pool;
    std::vector<std::pair<uint32_t, uint32_t>> ev_open[2];  // indices into ev_pool: (start, stop)
    size_t ev_next = 0;
    uint64_t t_launches[2] = {0, 0};
    double t_ms[2] = {0.0, 0.0};

    uint64_t launches = 0;
    std::string last_error;

    int32_t fail(int32_t code, const std::string& msg) {
        last_error = msg;
        return code;
    }
    template <typename T>
    T* plan_dev(size_t off) const {
        return reinterpret_cast<T*>(d_plan + off);
    }
    uint8_t* layer_k(uint32_t layer) const { return pool_k + size_t(layer) * layer_stride_bytes; }
    uint8_t* layer_v(uint32_t layer) const { return pool_v + size_t(layer) * layer_stride_bytes; }
};

// ---- kernel launchers (one per translation unit) ---------------------------------------------

constexpr uint32_t kTreeMaxNodes = 128;

struct KriyaAppendArgs {
    void* q_inout;
    const void* k_in;
    const void* v_in;
    const void* q_norm_w;
    const void* k_norm_w;
    void* cache_k;
    void* cache_v;
    const int32_t* indptr;
    const int32_t* indices;
    const int32_t* last_len;
    const uint32_t* positions;
    const float* table;  // may be null
    uint32_t* status;
    uint32_t num_tokens;
    uint32_t num_blocks;
    // chunk mode: token i of row 0 at absolute position prefix + i (plan rows are not per token)
    uint32_t chunk_mode;
    uint32_t prefix_tokens;
    uint32_t inplace;  // rotate q and k where they are (k_in is written); v and the cache are not touched
    uint32_t kv_q4 = 0;  // the cache is Q4KvGroup32: keys and values are quantised on their way in
    // chunk_mode 2: chunks of several sequences; sequence s owns rows [seq_q_start[s], + seq_count[s]) of q / k / v, its
    // token i sits at position seq_prefix[s] + i and its block table is plan row s
    const uint32_t* seq_q_start = nullptr;
    const uint32_t* seq_prefix = nullptr;
    const uint32_t* seq_count = nullptr;
    uint32_t n_seqs = 0;
    kriya_rope_kv_write_params p;
};
cudaError_t kriya_launch_append(const KriyaAppendArgs& a, uint32_t dtype, cudaStream_t s);

struct KriyaDecodeArgs {
    const void* q;          // [rows][Hq][D]
    const void* cache_k;    // layer base
    const void* cache_v;
    const int32_t* indptr;
    const int32_t* indices;
    const int32_t* last_len;
    const KriyaDecodeWork* work;
    void* out;              // [rows][Hq][D] 16-bit (normal mode)
    float* part_o;          // scratch
    float* part_ml;
    uint32_t* counters;
    // partial mode: write merged (m, l, o) per row instead of the normalised output
    float* state_m;
    float* state_l;
    float* state_o;
    uint32_t* status;
    uint32_t n_work;
    uint32_t num_blocks;
    uint32_t num_q_heads;
    uint32_t num_kv_heads;
    float sm_scale;
    float logit_softcap;
    uint64_t wait_ns;  // limit of every bounded wait inside the kernel
};
// Returns cudaErrorInvalidValue for shapes the kernels are not instantiated for.
cudaError_t kriya_launch_decode(const KriyaDecodeArgs& a, uint32_t head_dim, uint32_t block_size, uint32_t dtype,
                                int max_smem_optin, cudaStream_t s, uint32_t kv_q4 = 0);
bool kriya_decode_supported(uint32_t head_dim, uint32_t group, uint32_t num_kv_heads, uint32_t block_size);

// Optional fused RoPE + KV append inside the tensor-core decode launch (null k_in: plain decode).
struct KriyaFusedAppend {
    const void* k_in = nullptr;     // [rows][Hkv][D] new keys (un-rotated)
    const void* v_in = nullptr;     // [rows][Hkv][D] new values
    void* q_rope_out = nullptr;     // optional [rows][Hq][D]: rotated queries (must not alias q)
    const uint32_t* positions = nullptr;
    const float* table = nullptr;   // cos/sin table or null
    void* cache_k_w = nullptr;      // writable layer bases
    void* cache_v_w = nullptr;
    uint32_t rotary_dim = 0;
    uint32_t max_seq_len = 0;
    uint32_t has_table = 0;
    float rope_theta = 0.0f;
    uint32_t positions_are_context = 0;  // every row's position equals its token count - 1 (checked on the host)
    // Launch option: 0 = ordinary launch; otherwise the launch may begin while the previous kernel of the stream drains
    // (programmatic dependent launch) and the kernel waits for that kernel's completion as far as the mode says:
    // 1 = before anything but its own set-up, 3 = before it touches activations (queries, new K/V, outputs) while the K/V
    // stream of the cache starts at once, 2 = never (every input is known to be complete).
    uint32_t overlap_previous = 0;
};
// Scratch of one tensor-core decode launch: the partial states of runs that are cut across CTAs, stored as (value, stamp)
// pairs, the counter the CTAs of the launch count themselves off in, and what that counter reads once every earlier
// launch on the same set has finished with it.
struct KriyaTcScratch {
    void* ll_o = nullptr;          // uint2 [segments][G][128]
    void* ll_ml = nullptr;         // uint2 [segments][G][2]
    uint32_t* set_done = nullptr;
    uint32_t done_expect = 0;
    uint32_t epoch = 1;            // stamp of the launch, never zero
};
bool kriya_decode_tc_supported(uint32_t head_dim, uint32_t group, uint32_t block_size);
uint32_t kriya_decode_tc_ctas_per_sm();
uint32_t kriya_decode_tc_pages_per_tile();
// the same kernel built with 64-token tiles and two resident CTAs per SM (kriya_decode_tc64.cu)
uint32_t kriya_decode_tc_ctas_per_sm_t64();
uint32_t kriya_decode_tc_pages_per_tile_t64();
cudaError_t kriya_launch_decode_tc_t64(const KriyaDecodeArgs& a, const KriyaTcSeg* segs, const uint32_t* cta_seg_ptr, uint32_t grid,
                                       const void* map_k, const void* map_v, uint32_t layer_row0, uint32_t dtype,
                                       int max_smem_optin, const KriyaFusedAppend& fused, uint32_t late_parts, uint32_t n_seg,
                                       const KriyaTcScratch& scratch, cudaStream_t s);
cudaError_t kriya_launch_decode_tc(const KriyaDecodeArgs& a, const KriyaTcSeg* segs, const uint32_t* cta_seg_ptr, uint32_t grid,
                                   const void* map_k, const void* map_v, uint32_t layer_row0, uint32_t dtype,
                                   int max_smem_optin, const KriyaFusedAppend& fused, uint32_t late_parts, uint32_t n_seg,
                                   const KriyaTcScratch& scratch, cudaStream_t s);

// The tensor-core decode kernel that moves whole pages (both KV heads) with one copy: head_dim 128, 2 KV heads, 16-token pages.
bool kriya_decode_tcp_supported(uint32_t head_dim, uint32_t num_kv_heads, uint32_t group, uint32_t block_size);
uint32_t kriya_decode_tcp_pages_per_tile();
cudaError_t kriya_decode_tcp_encode_maps(void* pool_k, void* pool_v, uint64_t total_pages, void* out_map_k, void* out_map_v);
cudaError_t kriya_launch_decode_tcp(const KriyaDecodeArgs& a, const KriyaTcSeg* segs, const uint32_t* cta_seg_ptr, uint32_t grid,
                                    const void* map_k, const void* map_v, uint32_t page0, uint32_t dtype, int max_smem_optin,
                                    const KriyaFusedAppend& fused, uint32_t late_parts, uint32_t n_seg, const KriyaTcScratch& scratch,
                                    cudaStream_t s);

// A one-block kernel that waits, with the given limit, on a barrier nobody arrives at and reports the expiry in `status`.
cudaError_t kriya_launch_wait_selftest(uint32_t* status, uint64_t wait_ns, cudaStream_t s);

cudaError_t kriya_launch_merge_states(const float* m, const float* l, const float* o, uint32_t parts, uint32_t rows,
                                      uint32_t D, size_t stride_ml, size_t stride_o, void* out, uint32_t dtype,
                                      cudaStream_t s);

cudaError_t kriya_launch_block_copy(uint8_t* pool_k, uint8_t* pool_v, size_t layer_stride_bytes, uint32_t num_layers,
                                    size_t block_bytes, const uint32_t* pairs_dev, uint32_t n_pairs, int sm_count,
                                    cudaStream_t s);
cudaError_t kriya_launch_slot_write(uint8_t* cache_k, uint8_t* cache_v, const void* stage_k, const void* stage_v,
                                    size_t row_bytes, uint32_t block_size, const uint32_t* triples_dev, uint32_t n,
                                    uint32_t num_blocks, uint32_t* status, cudaStream_t s);

// One 128-query tile of a prefill launch.
struct KriyaPrefillTile {
    uint32_t tbl_off;  // where the sequence's block table starts inside page_indices
    uint32_t q_row0;   // first row of the tile in q / out
    uint32_t rows;     // 1..128
    uint32_t pos0;     // absolute position of the tile's first query (prefix + offset inside the chunk)
    uint32_t seq_end;  // tokens of the sequence present in the cache (prefix + chunk length)
    // A tile with few companions is cut along the KV axis into pieces (one record each) so that the launch fills the
    // machine: the piece covers the 128-key tiles kv_t0 .. kv_t1 - 1 (kv_t1 = 0: to the causal end) and, when `slot` is
    // not UINT32_MAX, leaves its un-normalised state in scratch slot `slot` for prefill_merge_kernel instead of rows of out.
    uint32_t kv_t0;
    uint32_t kv_t1;
    uint32_t slot;
};
static_assert(sizeof(KriyaPrefillTile) == 32, "tile record is 32 bytes");

// One query tile whose pieces prefill_merge_kernel combines: pieces slot0 .. slot0 + n_parts - 1.
struct KriyaPrefillMerge {
    uint32_t q_row0;
    uint32_t rows;
    uint32_t slot0;
    uint32_t n_parts;
};
struct KriyaPrefillArgs {
    const void* q;        // [T][Hq][D]
    const void* cache_k;  // layer base
    const void* cache_v;
    const void* map_k;    // CUtensorMap over the K pool (host copy)
    const void* map_v;
    const int32_t* table; // page_indices of the plan
    const KriyaPrefillTile* tiles;
    void* out;            // [T][Hq][D]
    uint32_t* status;
    uint32_t n_tiles;
    uint32_t q_rows;      // rows of q / out that the launch may touch (extent of the query tensor map)
    uint32_t num_blocks;
    uint32_t num_q_heads;
    uint32_t num_kv_heads;
    uint32_t layer_row0;  // first row of this layer inside the all-layer tensor map
    uint32_t window;      // sliding-window size in tokens, 0 = plain causal
    float sm_scale;
    float logit_softcap;
    float* part_o;        // piece states: per (slot, head pair CTA) [2 heads][D / 4][128 rows] float4, un-normalised
    float* part_ml;       // and [2 heads][128 rows][2]: exponent reference (log2 units) and sum
    const KriyaPrefillMerge* merge_items;  // query tiles that were cut (device), n_merge of them
    uint32_t n_merge;
};
// Tree verification: attention of every draft-tree node over its ancestors in the tree (in-flight K/V, `mask`), started
// from the state (m, l, o) of the node's attention over the cached prefix.
struct KriyaTreeArgs {
    const void* q;        // [nodes][Hq][D], rotated
    const void* k;        // [nodes][Hkv][D], rotated
    const void* v;        // [nodes][Hkv][D]
    const uint8_t* mask;  // [nodes][nodes], 1 = node j is visible to node i
    const float* st_m;    // [nodes * Hq] prefix state, ignored when has_prefix == 0
    const float* st_l;
    const float* st_o;    // [nodes * Hq][D]
    void* out;            // [nodes][Hq][D]
    uint32_t n_nodes;
    uint32_t num_q_heads;
    uint32_t num_kv_heads;
    uint32_t has_prefix;
    float sm_scale;
};
cudaError_t kriya_launch_tree_finish(const KriyaTreeArgs& a, uint32_t head_dim, uint32_t dtype, cudaStream_t s);

cudaError_t kriya_launch_prefill(const KriyaPrefillArgs& a, uint32_t head_dim, uint32_t block_size, uint32_t dtype,
                                 int max_smem_optin, cudaStream_t s);
bool kriya_prefill_supported(uint32_t head_dim, uint32_t group, uint32_t block_size, uint32_t dtype);
cudaError_t kriya_launch_q4_expand_blocks(const void* pool_k, const void* pool_v, void* dst_k, void* dst_v, const int32_t* indices,
                                          uint32_t n_indices, uint32_t block_tokens, uint32_t hkv, uint32_t head_dim, uint32_t num_blocks,
                                          uint32_t dtype, uint32_t* status, cudaStream_t s);
cudaError_t kriya_prefill_encode_maps(void* pool_k, void* pool_v, uint64_t total_rows, uint32_t row_elems,
                                      void* out_map_k, void* out_map_v);
