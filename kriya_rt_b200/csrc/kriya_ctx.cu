// Context, plan upload and the C ABI of libkriya_cuda (see include/kriya_cuda.h).
//
// The context plays the part of MetalExecutor for this path
// (crates/kriya-backend-metal/src/encoder.rs:1740-2035): it owns the KV pools of all layers, the RoPE
// cos/sin table, the per-step plan buffers and all scratch, allocated once.  Nothing on the step path
// allocates.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <chrono>
#include <string>
#include <thread>
#include <vector>

#include "kriya_internal.h"

namespace {

thread_local std::string g_create_error;
constexpr uint32_t kTcScratchSets = 4;  // split-run scratch sets of the tensor-core decode kernel (see launch_decode)

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

#define KRIYA_CUDA_TRY(ctx, expr)                                                                          \
    do {                                                                                                   \
        cudaError_t _e = (expr);                                                                           \
        if (_e != cudaSuccess)                                                                             \
            return (ctx)->fail(KRIYA_CUDA_EXECUTION_ERROR, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
    } while (0)

void destroy(kriya_cuda_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->cfg.device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    if (c->copy_stream) cudaStreamSynchronize(c->copy_stream);
    if (c->copy_stream_out) cudaStreamSynchronize(c->copy_stream_out);
    kriya_comm_destroy(c);
    cudaFree(c->pool_k);
    cudaFree(c->pool_v);
    cudaFree(c->rope_table);
    cudaFree(c->d_plan);
    cudaFree(c->part_o);
    cudaFree(c->part_ml);
    cudaFree(c->part_counter);
    cudaFree(c->tc_ll_o);
    cudaFree(c->tc_ll_ml);
    cudaFree(c->tc_set_done);
    cudaFree(c->d_status);
    cudaFree(c->d_act);
    cudaFree(c->d_pairs);
    cudaFree(c->pf_part_o);
    cudaFree(c->pf_part_ml);
    cudaFree(c->q4_stage_k);
    cudaFree(c->q4_stage_v);
    cudaFree(c->q4_identity);
    cudaFree(c->d_tree_state);
    cudaFree(c->d_tree_mask);
    cudaFree(c->d_step);
    for (cudaEvent_t e : c->ev_pool) cudaEventDestroy(e);
    for (int i = 0; i < 2; ++i) {
        if (c->h_plan[i]) cudaFreeHost(c->h_plan[i]);
        if (c->h_plan_free[i]) cudaEventDestroy(c->h_plan_free[i]);
    }
    if (c->h_status) cudaFreeHost(c->h_status);
    if (c->h_act) cudaFreeHost(c->h_act);
    if (c->h_pairs) cudaFreeHost(c->h_pairs);
    if (c->h_pairs_free) cudaEventDestroy(c->h_pairs_free);
    for (cudaEvent_t e : c->ev_in) cudaEventDestroy(e);
    for (cudaEvent_t e : c->ev_done) cudaEventDestroy(e);
    if (c->ev_step_begin) cudaEventDestroy(c->ev_step_begin);
    if (c->ev_step_end) cudaEventDestroy(c->ev_step_end);
    if (c->stream) cudaStreamDestroy(c->stream);
    if (c->copy_stream) cudaStreamDestroy(c->copy_stream);
    if (c->copy_stream_out) cudaStreamDestroy(c->copy_stream_out);
    delete c;
}

// Splits every plan row into near-equal contiguous block ranges so that about `target` work items of
// similar size exist, largest first.  `begin`/`end` (optional) restrict each row to a block range.
// First token of row r inside a sliding window of `window` tokens that ends at the row's last token (0 = no window).
inline uint32_t window_first_token(const int32_t* indptr, const int32_t* last_len, uint32_t block_size, uint32_t r, uint32_t window) {
    if (window == 0u) return 0u;
    const uint32_t nb = uint32_t(indptr[r + 1] - indptr[r]);
    if (nb == 0u) return 0u;
    const uint64_t tokens = uint64_t(nb - 1u) * block_size + uint32_t(std::max(last_len[r], 1));
    return tokens > window ? uint32_t(tokens - window) : 0u;
}

uint32_t build_work(const int32_t* indptr, const int32_t* last_len, uint32_t block_size, uint32_t window, uint32_t rows,
                    const uint32_t* begin, const uint32_t* end, uint32_t target, uint32_t min_chunk, KriyaDecodeWork* out,
                    uint32_t cap) {
    uint64_t total = 0;
    auto first_block = [&](uint32_t r, uint32_t nb) {  // the row's range begins no earlier than the window does
        const uint32_t wb = window_first_token(indptr, last_len, block_size, r, window) / block_size;
        return std::min(std::max(begin ? begin[r] : 0u, wb), nb);
    };
    for (uint32_t r = 0; r < rows; ++r) {
        const uint32_t nb = uint32_t(indptr[r + 1] - indptr[r]);
        const uint32_t b = first_block(r, nb);
        const uint32_t e = end ? std::min(end[r], nb) : nb;
        total += e > b ? e - b : 0u;
    }
    uint32_t chunk = uint32_t((total + target - 1) / std::max(target, 1u));
    chunk = std::max(chunk, min_chunk);
    uint32_t n = 0, slot = 0;
    for (uint32_t r = 0; r < rows; ++r) {
        const uint32_t nb = uint32_t(indptr[r + 1] - indptr[r]);
        const uint32_t b = first_block(r, nb);
        const uint32_t e = end ? std::min(end[r], nb) : nb;
        const uint32_t len = e > b ? e - b : 0u;
        const uint32_t parts = std::max(1u, (len + chunk - 1) / chunk);
        const uint32_t size = (len + parts - 1) / parts;
        if (n + parts > cap) return UINT32_MAX;
        for (uint32_t k = 0; k < parts; ++k) {
            KriyaDecodeWork w{};
            w.req = r;
            w.tok_first = window_first_token(indptr, last_len, block_size, r, window);
            w.blk_begin = b + std::min(k * size, len);
            w.blk_end = b + std::min((k + 1) * size, len);
            w.slot = slot + k;
            w.first_slot = slot;
            w.n_parts = parts;
            out[n++] = w;
        }
        slot += parts;
    }
    std::stable_sort(out, out + n, [](const KriyaDecodeWork& x, const KriyaDecodeWork& y) {
        return (x.blk_end - x.blk_begin) > (y.blk_end - y.blk_begin);
    });
    return n;
}

// Tensor-core decode work: every (row, KV head) is a run of 128-token tiles; the runs laid end to end are cut
// into `ctas` contiguous pieces of equal weight.  A run's first tile can be given kRunStartWeight extra tiles of
// weight (a CTA that finishes one run and starts another pays an epilogue and a pipeline restart); measured on the
// benchmark shape, weights of 2 and 4 made the launch about a third slower than 0 because they multiply short
// leftover pieces, so plain tile counts are used.  Returns the number of segment records, or UINT32_MAX when `cap`
// is too small.  `ptr` receives ctas + 1 offsets into `out`.
constexpr uint32_t kRunStartWeight = 0;
// Fewest 128-token tiles a CTA of the tensor-core decode kernel is given before another CTA is brought in.
uint32_t tc_min_tiles_per_cta() {
    static const uint32_t v = [] {
        const char* e = getenv("KRIYA_TC_MIN_TILES");
        const int x = e ? atoi(e) : 8;  // 1024 tokens at 128-token tiles, 512 at 64-token tiles
        return uint32_t(x < 1 ? 1 : x);
    }();
    return v;
}

uint32_t build_tc_segments(const int32_t* indptr, const int32_t* last_len, uint32_t block_size, uint32_t rows, uint32_t hkv,
                           const uint32_t* begin, const uint32_t* end, uint32_t ctas, uint32_t TP, KriyaTcSeg* out, uint32_t cap,
                           uint32_t* ptr, uint32_t min_tiles, uint32_t window) {  // TP = pages per tile of the kernel variant the list is for
    uint64_t total = 0;
    auto first_block = [&](uint32_t r, uint32_t nb) {  // the row's range begins no earlier than the sliding window does
        const uint32_t wb = window_first_token(indptr, last_len, block_size, r, window) / block_size;
        return std::min(std::max(begin ? begin[r] : 0u, wb), nb);
    };
    for (uint32_t r = 0; r < rows; ++r) {
        const uint32_t nb = uint32_t(indptr[r + 1] - indptr[r]);
        const uint32_t b = first_block(r, nb);
        const uint32_t e = end ? std::min(end[r], nb) : nb;
        if (e > b) total += uint64_t((e + TP - 1) / TP - b / TP + kRunStartWeight) * hkv;
    }
    // A short plan is not spread over every CTA: a CTA that streams only a tile or two costs its start-up latency all
    // the same, and every extra piece of a run is one more partial state for the run's merge to read.
    const uint32_t all_ctas = ctas;
    ctas = uint32_t(std::min<uint64_t>(ctas, std::max<uint64_t>(1, (total + min_tiles - 1) / min_tiles)));
    uint32_t n = 0, slot = 0, cta = 0;
    uint64_t unit = 0;  // weight consumed so far
    auto cta_end = [&](uint32_t c) { return total * (c + 1) / ctas; };  // first unit NOT owned by cta c
    ptr[0] = 0;
    for (uint32_t r = 0; r < rows; ++r) {
        const uint32_t nb = uint32_t(indptr[r + 1] - indptr[r]);
        const uint32_t b = first_block(r, nb);
        const uint32_t e = end ? std::min(end[r], nb) : nb;
        const uint32_t tbl = uint32_t(indptr[r]);
        const uint32_t row_tokens = nb ? (nb - 1u) * block_size + uint32_t(std::max(last_len[r], 1)) : 0u;
        const uint32_t tok_first = window_first_token(indptr, last_len, block_size, r, window);
        for (uint32_t h = 0; h < hkv; ++h) {
            if (e <= b) {  // empty run: one zero-length record so that its output is still written
                if (n + 1 > cap) return UINT32_MAX;
                out[n++] = KriyaTcSeg{r, h, b, b, slot, slot, 1u, tbl, row_tokens, tok_first, {0u, 0u}};
                slot += 1;
                continue;
            }
            const uint32_t t0 = b / TP, t1 = (e + TP - 1) / TP;
            const uint32_t first = n, first_slot = slot;
            uint32_t t = t0;
            uint64_t lead = kRunStartWeight;  // weight carried by the run's first tile
            while (t < t1) {
                while (cta + 1 < ctas && unit >= cta_end(cta)) ptr[++cta] = n;
                uint32_t take;
                if (cta + 1 < ctas) {
                    const uint64_t room = cta_end(cta) - unit;  // > 0
                    // the first tile goes with its lead weight even when that overshoots the boundary a little
                    take = uint32_t(std::min<uint64_t>(room > lead ? room - lead : 1u, t1 - t));
                    take = std::max(take, 1u);
                } else {
                    take = t1 - t;
                }
                if (n + 1 > cap) return UINT32_MAX;
                out[n++] = KriyaTcSeg{r, h, std::max(b, t * TP), std::min(e, (t + take) * TP), slot++, first_slot, 0u, tbl,
                                      row_tokens, tok_first, {0u, 0u}};
                t += take;
                unit += take + lead;
                lead = 0;
            }
            for (uint32_t i = first; i < n; ++i) out[i].n_parts = n - first;
        }
    }
    while (cta < all_ctas) ptr[++cta] = n;
    // A CTA whose list begins with the continuation of a run that started in an earlier CTA takes that piece last.  The
    // run's last piece finishes the run (it gathers the other pieces' states): taken last, it finds them published.  It
    // is also the piece that reads the token the same launch appends, which is then in the cache long before.
    for (uint32_t k = 0; k < all_ctas; ++k)
        if (ptr[k + 1] - ptr[k] > 1u && out[ptr[k]].slot != out[ptr[k]].first_slot)
            std::rotate(out + ptr[k], out + ptr[k] + 1, out + ptr[k + 1]);
    return n;
}

// The whole-page kernel reads one 144-byte record per CTA instead of two entries of the segment-range list: word 0 the
// CTA's first segment (the next record's word 0 is its end), word 1 the pages of the CTA's first tile that may be fetched
// before anything else is known (0 = none: the tile holds the end of its row, which a fused append still has to write),
// word 2 the place of the first of them inside the tile, word 3 the row of the first piece the CTA works on (UINT32_MAX:
// none), words 4-7 the pool blocks of those pages, word 8 the position of that row's new token.  With it the first K/V
// bytes and the first query rows are asked for one memory round trip after the CTA starts instead of three or four
// (range list, segment, block table or position, data).  Words 12-35 are copies of the CTA's first two segment records, which
// is all most CTAs have: nothing but this record has to arrive before the CTA is set up.
constexpr uint32_t kTcpHdrWords = 36;  // 12 words of its own + copies of the CTA's first two segment records
void expand_tcp_headers(uint32_t* ptr, uint32_t ctas, const KriyaTcSeg* segs, const int32_t* indices, uint32_t TP, uint32_t block_size,
                        const uint32_t* positions, uint32_t n_positions) {
    for (uint32_t k = ctas + 1; k-- > 0;) {
        const uint32_t v = ptr[k];
        uint32_t* h = ptr + size_t(k) * kTcpHdrWords;
        for (uint32_t i = 1; i < kTcpHdrWords; ++i) h[i] = 0u;
        h[0] = v;
        h[3] = UINT32_MAX;
    }
    static_assert(sizeof(KriyaTcSeg) == 48, "two records fill words 12..35");
    for (uint32_t k = 0; k < ctas; ++k) {
        uint32_t* h = ptr + size_t(k) * kTcpHdrWords;
        for (uint32_t i = 0; i < 2u && h[0] + i < h[kTcpHdrWords]; ++i) memcpy(h + 12u + 12u * i, &segs[h[0] + i], sizeof(KriyaTcSeg));
        for (uint32_t si = h[0]; si < h[kTcpHdrWords]; ++si) {
            const KriyaTcSeg& s = segs[si];
            if (s.blk_hi <= s.blk_lo) continue;
            h[3] = s.req;
            h[8] = s.req < n_positions ? positions[s.req] : (s.row_tokens ? s.row_tokens - 1u : 0u);
            const uint32_t t0 = s.blk_lo / TP, t1 = (s.blk_hi + TP - 1) / TP;
            const bool row_end = uint64_t(s.blk_hi) * block_size >= s.row_tokens;
            if (!(t0 + 1 == t1 && row_end)) {
                const uint32_t p_lo = std::max(t0 * TP, s.blk_lo), p_hi = std::min((t0 + 1) * TP, s.blk_hi);
                h[1] = p_hi - p_lo;
                h[2] = p_lo - t0 * TP;
                for (uint32_t i = 0; i < p_hi - p_lo && i < 4u; ++i) h[4 + i] = uint32_t(indices[s.tbl_off + p_lo + i]);
            }
            break;
        }
    }
}

// Which build of the tensor-core decode kernel serves a plan: the 64-token-tile build (two CTAs per SM) streams faster
// but pays its per-CTA costs twice as often, so it is taken when every SM has a long stream ahead of it.
constexpr uint32_t kLateMergeParts = 12;  // runs cut into more pieces are merged by late_merge_kernel

uint32_t max_parts_of(const KriyaTcSeg* segs, uint32_t n) {
    uint32_t m = 0;
    for (uint32_t i = 0; i < n; ++i) m = std::max(m, segs[i].n_parts);
    return m;
}

// Which tensor-core decode kernel serves a plan (see kriya_cuda_ctx::tc_variant).  The whole-page kernel is taken wherever
// the shape allows it.  Between the two one-head-per-copy builds, the 64-token-tile build (two CTAs per SM) streams faster
// but pays its per-CTA costs twice as often, so it is taken when every SM has a long stream ahead of it.
int choose_tc_variant(const kriya_cuda_ctx* c, const int32_t* indptr, uint32_t rows, const uint32_t* begin, const uint32_t* end) {
    if (c->tc_force == 64) return 1;
    if (c->tc_force == 128) return 0;
    if (c->tcp_ok && c->decode_path != 3) return 2;
    uint64_t tiles = 0;  // 128-token tiles of the whole launch
    for (uint32_t r = 0; r < rows; ++r) {
        const uint32_t nb = uint32_t(indptr[r + 1] - indptr[r]);
        const uint32_t b = begin ? std::min(begin[r], nb) : 0u, e = end ? std::min(end[r], nb) : nb;
        if (e > b) tiles += uint64_t((e - b + 7) / 8) * c->cfg.num_kv_heads;
    }
    return tiles >= uint64_t(c->tc64_min_tiles) * uint64_t(c->sm_count) ? 1 : 0;
}
struct TcVariantGeometry {
    uint32_t ctas, pages_per_tile, runs_per_row, min_tiles;
};
TcVariantGeometry tc_geometry(const kriya_cuda_ctx* c, int variant) {
    const uint32_t sms = uint32_t(c->sm_count);
    if (variant == 2) return {sms, kriya_decode_tcp_pages_per_tile(), 1u, tc_min_tiles_per_cta()};
    if (variant == 1) return {sms * kriya_decode_tc_ctas_per_sm_t64(), kriya_decode_tc_pages_per_tile_t64(), c->cfg.num_kv_heads, tc_min_tiles_per_cta()};
    return {sms * kriya_decode_tc_ctas_per_sm(), kriya_decode_tc_pages_per_tile(), c->cfg.num_kv_heads, tc_min_tiles_per_cta()};
}

int32_t check_layer(kriya_cuda_ctx* c, uint32_t layer) {
    if (layer >= c->cfg.num_layers)
        return c->fail(KRIYA_CUDA_INVALID_INPUT, "layer " + std::to_string(layer) + " out of range (context has " +
                                                     std::to_string(c->cfg.num_layers) + ")");
    return KRIYA_CUDA_OK;
}

int32_t check_gqa(kriya_cuda_ctx* c, const kriya_bsr_gqa_params* p) {
    if (!p) return c->fail(KRIYA_CUDA_INVALID_INPUT, "params must not be null");
    if (p->num_q_heads != c->cfg.num_q_heads || p->num_kv_heads != c->cfg.num_kv_heads ||
        p->head_dim != c->cfg.head_dim || p->block_size_tokens != c->cfg.block_size_tokens)
        return c->fail(KRIYA_CUDA_INVALID_INPUT, "BsrGqaParams shape differs from the context's configuration");
    return KRIYA_CUDA_OK;
}

int32_t check_rope(kriya_cuda_ctx* c, const kriya_rope_kv_write_params* p) {
    if (!p) return c->fail(KRIYA_CUDA_INVALID_INPUT, "params must not be null");
    if (p->num_q_heads != c->cfg.num_q_heads || p->num_kv_heads != c->cfg.num_kv_heads ||
        p->head_dim != c->cfg.head_dim || p->block_size_tokens != c->cfg.block_size_tokens)
        return c->fail(KRIYA_CUDA_INVALID_INPUT, "RopeKvWriteParams shape differs from the context's configuration");
    if (p->rotary_dim > p->head_dim || (p->rotary_dim & 1u))
        return c->fail(KRIYA_CUDA_INVALID_INPUT, "rotary_dim must be even and <= head_dim");
    return KRIYA_CUDA_OK;
}

// The table is only usable when it was built for the same theta / rotary_dim the call asks for.
const float* table_for(const kriya_cuda_ctx* c, const kriya_rope_kv_write_params* p) {
    if (!p->has_table || !c->rope_table) return nullptr;
    if (p->rotary_dim != c->rope_rotary_dim || p->rope_theta != c->cfg.rope_theta) return nullptr;
    if (p->max_seq_len > c->cfg.rope_max_seq_len) return nullptr;
    return c->rope_table;
}

// Timing brackets: events come from a pool that grows while timing is on; closed brackets are summed by
// timing_collect() once the stream has drained.
struct TimingScope {
    kriya_cuda_ctx* c;
    uint32_t kind;
    uint32_t start = 0, stop = 0;
    bool on;
    TimingScope(kriya_cuda_ctx* ctx, uint32_t k) : c(ctx), kind(k), on(ctx->timing) {
        if (!on) return;
        while (c->ev_next + 2 > c->ev_pool.size()) {
            cudaEvent_t e;
            if (cudaEventCreate(&e) != cudaSuccess) {
                on = false;
                return;
            }
            c->ev_pool.push_back(e);
        }
        start = uint32_t(c->ev_next++);
        stop = uint32_t(c->ev_next++);
        cudaEventRecord(c->ev_pool[start], c->stream);
    }
    ~TimingScope() {
        if (!on) return;
        cudaEventRecord(c->ev_pool[stop], c->stream);
        c->ev_open[kind].emplace_back(start, stop);
    }
};

void timing_collect(kriya_cuda_ctx* c) {
    for (int k = 0; k < 2; ++k) {
        for (auto& pr : c->ev_open[k]) {
            float ms = 0.0f;
            if (cudaEventElapsedTime(&ms, c->ev_pool[pr.first], c->ev_pool[pr.second]) == cudaSuccess) {
                c->t_ms[k] += ms;
                c->t_launches[k] += 1;
            }
        }
        c->ev_open[k].clear();
    }
    c->ev_next = 0;
}

int32_t launch_append(kriya_cuda_ctx* c, uint32_t layer, void* q, const void* k, const void* v, const void* qw,
                      const void* kw, uint32_t num_tokens, uint32_t chunk_mode, uint32_t prefix,
                      const kriya_rope_kv_write_params* p) {
    KriyaAppendArgs a{};
    a.q_inout = q;
    a.k_in = k;
    a.v_in = v;
    a.q_norm_w = qw;
    a.k_norm_w = kw;
    a.cache_k = c->layer_k(layer);
    a.cache_v = c->layer_v(layer);
    a.indptr = c->plan_dev<int32_t>(c->off_indptr);
    a.indices = c->plan_dev<int32_t>(c->off_indices);
    a.last_len = c->plan_dev<int32_t>(c->off_last_len);
    a.positions = c->plan_dev<uint32_t>(c->off_positions);
    a.table = table_for(c, p);
    a.status = c->d_status;
    a.num_tokens = num_tokens;
    a.num_blocks = c->cfg.num_kv_blocks;
    a.chunk_mode = chunk_mode;
    a.prefix_tokens = prefix;
    a.kv_q4 = c->cfg.kv_format == KRIYA_KV_Q4_GROUP32 ? 1u : 0u;
    a.p = *p;
    TimingScope ts(c, 1);
    KRIYA_CUDA_TRY(c, kriya_launch_append(a, c->cfg.dtype, c->stream));
    c->launches += 1;
    return KRIYA_CUDA_OK;
}

bool use_tc_decode(const kriya_cuda_ctx* c) {
    if (c->decode_path == 1) return false;
    return c->tmaps_ok && kriya_decode_tc_supported(c->cfg.head_dim, c->cfg.num_q_heads / c->cfg.num_kv_heads,
                                                    c->cfg.block_size_tokens);
}

int32_t launch_decode(kriya_cuda_ctx* c, uint32_t layer, const void* q, void* out, float* sm, float* sl, float* so,
                      bool range_list, uint32_t n_work, const kriya_bsr_gqa_params* p,
                      const KriyaFusedAppend& fused = KriyaFusedAppend()) {
    KriyaDecodeArgs a{};
    a.q = q;
    a.cache_k = c->layer_k(layer);
    a.cache_v = c->layer_v(layer);
    a.indptr = c->plan_dev<int32_t>(c->off_indptr);
    a.indices = c->plan_dev<int32_t>(c->off_indices);
    a.last_len = c->plan_dev<int32_t>(c->off_last_len);
    a.work = c->plan_dev<KriyaDecodeWork>(range_list ? c->off_range : c->off_work);
    a.out = out;
    a.part_o = c->part_o;
    a.part_ml = c->part_ml;
    a.counters = c->part_counter;
    a.state_m = sm;
    a.state_l = sl;
    a.state_o = so;
    a.status = c->d_status;
    a.n_work = n_work;
    a.num_blocks = c->cfg.num_kv_blocks;
    a.num_q_heads = c->cfg.num_q_heads;
    a.num_kv_heads = c->cfg.num_kv_heads;
    a.sm_scale = p->sm_scale;
    a.logit_softcap = p->logit_softcap;
    a.wait_ns = c->wait_ns;
    TimingScope ts(c, 0);
    if (use_tc_decode(c)) {
        const uint32_t layer_row0 =
            uint32_t(size_t(layer) * c->layer_stride_bytes / (size_t(c->cfg.num_kv_heads) * c->cfg.head_dim * 2));
        const int variant = range_list ? c->tc_variant_ranges : c->tc_variant;
        const uint32_t grid = tc_geometry(c, variant).ctas;
        // A run spread over many CTAs (one long row) is merged by a kernel of its own behind the launch; launches that
        // overlap with their neighbours keep the merge inside, the scratch-set rotation relies on it.
        const bool chain_list = !range_list && c->use_chain_list && c->chain_list_valid && variant == 2;
        const uint32_t max_parts = range_list ? c->tc_max_parts_ranges : chain_list ? c->tc_max_parts_chain : c->tc_max_parts;
        const bool late = fused.overlap_previous == 0u && max_parts > kLateMergeParts;
        // Successive launches take the scratch sets in turn and stamp what they publish with their own number.  The launches
        // of one step may overlap at their edges; a set comes round again kTcScratchSets launches later, and the kernel
        // then checks the set's counter (every CTA of every earlier user has counted itself off) before it publishes.
        if (++c->tc_epoch == 0u) c->tc_epoch = 1u;
        const uint32_t set = c->tc_epoch % kTcScratchSets;
        KriyaTcScratch sc;
        sc.ll_o = c->tc_ll_o + size_t(set) * c->tc_set_o_bytes;
        sc.ll_ml = c->tc_ll_ml + size_t(set) * c->tc_set_ml_bytes;
        sc.set_done = c->tc_set_done + set * 16u;
        sc.done_expect = c->tc_done_expect[set];
        sc.epoch = c->tc_epoch;
        const KriyaTcSeg* segs = c->plan_dev<KriyaTcSeg>(range_list ? c->off_tcseg2 : chain_list ? c->off_tcseg3 : c->off_tcseg);
        const uint32_t* seg_ptr = c->plan_dev<uint32_t>(range_list ? c->off_tcptr2 : chain_list ? c->off_tcptr3 : c->off_tcptr);
        const uint32_t n_seg = range_list ? c->n_seg_ranges : chain_list ? c->n_seg_chain : c->n_seg;
        const uint32_t late_parts = late ? kLateMergeParts : UINT32_MAX;
        if (variant == 2) {
            KRIYA_CUDA_TRY(c, kriya_launch_decode_tcp(a, segs, seg_ptr, grid, c->tmap_kp, c->tmap_vp, layer * c->cfg.num_kv_blocks,
                                                      c->cfg.dtype, c->max_smem_optin, fused, late_parts, n_seg, sc, c->stream));
        } else {
            const auto launch = variant == 1 ? kriya_launch_decode_tc_t64 : kriya_launch_decode_tc;
            KRIYA_CUDA_TRY(c, launch(a, segs, seg_ptr, grid, c->tmap_k, c->tmap_v, layer_row0, c->cfg.dtype, c->max_smem_optin, fused,
                                     late_parts, n_seg, sc, c->stream));
        }
        c->tc_done_expect[set] += grid;  // every CTA of the grid counts itself off, idle ones included
        if (late) c->launches += 1;
    } else {
        KRIYA_CUDA_TRY(c, kriya_launch_decode(a, c->cfg.head_dim, c->cfg.block_size_tokens, c->cfg.dtype, c->max_smem_optin,
                                              c->stream, c->cfg.kv_format == KRIYA_KV_Q4_GROUP32 ? 1u : 0u));
    }
    c->launches += 1;
    return KRIYA_CUDA_OK;
}

// Into how many pieces (at most) the query tiles of a prefill launch are cut along the KV axis.  Only launches that do
// not fill the machine are cut, and only so far that the pieces still run as one wave: a tile of L 128-key tiles is cut
// into min(s, L / 2) pieces, every piece runs on `hp` CTAs (one per head pair), and the launch then takes as long as its
// longest CTA.  Costs in units of one KV tile (about 1.7 us), from measurements at the Qwen2.5-1.5B shape: a CTA costs
// its KV tiles plus 1.5 for its start-up (query tile, first K/V round trip) and its output; a piece costs 3 instead (its
// state is 128 KB of fp32 stores), and a launch with pieces pays about 4 more for the merge kernel behind it.  1 (no
// cut) stays unless a cut is at least 10 % shorter.  (Two pieces per tile at 8 prompts, 1.3 waves, measured 72 against
// 50 us per launch: cutting does not pay once the machine is full.)
uint32_t choose_prefill_split(const KriyaPrefillTile* tiles, uint32_t n, uint32_t hp, uint32_t sms, uint32_t max_cta_slots,
                              uint32_t max_records) {
    if (n == 0 || uint64_t(n) * hp >= sms) return 1u;
    uint32_t longest = 0;
    for (uint32_t i = 0; i < n; ++i) longest = std::max(longest, (tiles[i].pos0 + tiles[i].rows + 127u) / 128u);
    uint32_t best_s = 1u;
    float best = float(longest) + 1.5f;
    for (uint32_t s : {2u, 3u, 4u, 6u, 8u}) {
        uint64_t ctas = 0, records = 0;
        uint32_t longest_piece = 0;
        bool any = false;
        for (uint32_t i = 0; i < n; ++i) {
            const uint32_t L = (tiles[i].pos0 + tiles[i].rows + 127u) / 128u;
            const uint32_t parts = std::max(1u, std::min(s, L / 2u));
            any = any || parts > 1u;
            ctas += uint64_t(parts) * hp;
            records += parts + 1u;
            longest_piece = std::max(longest_piece, (L + parts - 1u) / parts);
        }
        if (!any || ctas > sms || ctas > max_cta_slots || records > max_records) continue;
        const float t = float(longest_piece) + 3.0f + 4.0f;
        if (t < best * 0.90f) {
            best = t;
            best_s = s;
        }
    }
    return best_s;
}

}  // namespace

extern "C" {

int32_t kriya_cuda_ctx_create(const kriya_cuda_config* cfg_in, kriya_cuda_ctx** out_ctx) {
    auto bad = [&](int32_t code, const std::string& msg) {
        g_create_error = msg;
        return code;
    };
    if (!cfg_in || !out_ctx) return bad(KRIYA_CUDA_INVALID_INPUT, "config and out_ctx must not be null");
    *out_ctx = nullptr;
    kriya_cuda_config cfg = *cfg_in;
    if (cfg.num_layers == 0 || cfg.num_kv_blocks == 0 || cfg.block_size_tokens == 0 || cfg.num_q_heads == 0 ||
        cfg.num_kv_heads == 0 || cfg.head_dim == 0)
        return bad(KRIYA_CUDA_INVALID_INPUT, "layers, blocks, block size, heads and head_dim must be non-zero");
    if (cfg.num_q_heads % cfg.num_kv_heads != 0)
        return bad(KRIYA_CUDA_INVALID_INPUT, "num_q_heads must be a multiple of num_kv_heads");
    if (cfg.dtype != KRIYA_DTYPE_BF16 && cfg.dtype != KRIYA_DTYPE_FP16)
        return bad(KRIYA_CUDA_INVALID_INPUT, "dtype must be KRIYA_DTYPE_BF16 or KRIYA_DTYPE_FP16");
    if ((cfg.head_dim * 2u) % 16u != 0)
        return bad(KRIYA_CUDA_UNSUPPORTED, "head_dim must make head rows a multiple of 16 bytes");
    if (cfg.kv_format != KRIYA_KV_16BIT && cfg.kv_format != KRIYA_KV_Q4_GROUP32)
        return bad(KRIYA_CUDA_INVALID_INPUT, "kv_format must be KRIYA_KV_16BIT or KRIYA_KV_Q4_GROUP32");
    if (cfg.kv_format == KRIYA_KV_Q4_GROUP32 && cfg.head_dim != 64 && cfg.head_dim != 128)
        return bad(KRIYA_CUDA_UNSUPPORTED, "the Q4KvGroup32 cache covers head_dim 64 and 128");
    if (cfg.rotary_dim == 0) cfg.rotary_dim = cfg.head_dim;  // enc:1929-1933
    if (cfg.rope_theta == 0.0f) cfg.rope_theta = 10000.0f;
    if (cfg.rope_max_seq_len == 0) cfg.rope_max_seq_len = 4096;  // enc:1939
    if (cfg.max_batch_rows == 0) cfg.max_batch_rows = 1024;
    if (cfg.max_page_indices == 0) cfg.max_page_indices = std::max(16384u, cfg.num_kv_blocks);
    if (cfg.max_tiles == 0) cfg.max_tiles = 4096;
    if (cfg.max_query_tokens == 0) cfg.max_query_tokens = 8192;

    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0)
        return bad(KRIYA_CUDA_DEVICE_INIT_FAILED,
                   std::string("no CUDA device available: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "count is 0"));
    if (cfg.device < 0 || cfg.device >= ndev)
        return bad(KRIYA_CUDA_DEVICE_INIT_FAILED, "device ordinal " + std::to_string(cfg.device) + " out of range");
    if ((e = cudaSetDevice(cfg.device)) != cudaSuccess)
        return bad(KRIYA_CUDA_DEVICE_INIT_FAILED, std::string("cudaSetDevice: ") + cudaGetErrorString(e));
    cudaDeviceProp prop{};
    if ((e = cudaGetDeviceProperties(&prop, cfg.device)) != cudaSuccess)
        return bad(KRIYA_CUDA_DEVICE_INIT_FAILED, std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(e));
    if (prop.major != 10)
        return bad(KRIYA_CUDA_DEVICE_INIT_FAILED, "this library holds sm_100a code only; device is sm_" +
                                                      std::to_string(prop.major) + std::to_string(prop.minor));

    auto* c = new kriya_cuda_ctx();
    c->cfg = cfg;
    c->sm_count = prop.multiProcessorCount;
    // the plan arrays hold the larger of the two kernel variants' grids
    c->tc_ctas = uint32_t(c->sm_count) * std::max(kriya_decode_tc_ctas_per_sm(), kriya_decode_tc_ctas_per_sm_t64());
    {
        const char* e = getenv("KRIYA_TC_VARIANT");  // 128 or 64: force one kernel variant (default: by plan)
        c->tc_force = e ? atoi(e) : 0;  // 128 / 64: one KV head per copy, 128- or 64-token tiles; default: by shape and plan
        const char* cm = getenv("KRIYA_TC_CHAIN_MIN_TILES");  // tiles per CTA for overlapping launches of a step (0: as for any launch)
        if (cm) c->tc_chain_min_tiles = uint32_t(std::max(0, atoi(cm)));
        const char* m = getenv("KRIYA_TC64_MIN_TILES");
        c->tc64_min_tiles = m ? uint32_t(std::max(1, atoi(m))) : 96u;
    }
    c->max_smem_optin = int(prop.sharedMemPerBlockOptin);
    c->block_bytes = cfg.kv_format == KRIYA_KV_Q4_GROUP32
                         ? size_t(cfg.block_size_tokens) * cfg.num_kv_heads * (cfg.head_dim / 32) * 20  // 20 bytes per 32 values
                         : size_t(cfg.block_size_tokens) * cfg.num_kv_heads * cfg.head_dim * 2;
    c->layer_stride_bytes = align_up(size_t(cfg.num_kv_blocks) * c->block_bytes, 256);  // enc:1890-1894
    c->cap_rows = cfg.max_batch_rows;
    c->cap_indices = cfg.max_page_indices;
    c->cap_tiles = cfg.max_tiles;
    c->cap_tokens = std::max(cfg.max_query_tokens, cfg.max_batch_rows);
    c->cap_work = c->cap_rows + 8u * uint32_t(c->sm_count);
    c->cap_pairs = std::max(4096u, c->cap_rows);

    auto fail_create = [&](const char* what, cudaError_t err) {
        g_create_error = std::string(what) + ": " + cudaGetErrorString(err);
        destroy(c);
        return int32_t(KRIYA_CUDA_DEVICE_INIT_FAILED);
    };
#define CREATE_TRY(expr)                                     \
    do {                                                     \
        cudaError_t _e = (expr);                             \
        if (_e != cudaSuccess) return fail_create(#expr, _e); \
    } while (0)

    CREATE_TRY(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    CREATE_TRY(cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking));
    CREATE_TRY(cudaStreamCreateWithFlags(&c->copy_stream_out, cudaStreamNonBlocking));
    CREATE_TRY(cudaEventCreateWithFlags(&c->ev_step_begin, cudaEventDisableTiming));
    CREATE_TRY(cudaEventCreateWithFlags(&c->ev_step_end, cudaEventDisableTiming));
    c->ev_in.resize(4);
    c->ev_done.resize(4);
    for (size_t i = 0; i < c->ev_in.size(); ++i) {
        CREATE_TRY(cudaEventCreateWithFlags(&c->ev_in[i], cudaEventDisableTiming));
        CREATE_TRY(cudaEventCreateWithFlags(&c->ev_done[i], cudaEventDisableTiming));
    }
    const size_t pool_bytes = c->layer_stride_bytes * cfg.num_layers;
    CREATE_TRY(cudaMalloc(&c->pool_k, pool_bytes));
    CREATE_TRY(cudaMalloc(&c->pool_v, pool_bytes));
    CREATE_TRY(cudaMemsetAsync(c->pool_k, 0, pool_bytes, c->stream));
    CREATE_TRY(cudaMemsetAsync(c->pool_v, 0, pool_bytes, c->stream));

    // tensor maps for the prefill kernel's paged gather (rows of all layers back to back)
    if (cfg.kv_format == KRIYA_KV_16BIT &&
        kriya_prefill_supported(cfg.head_dim, cfg.num_q_heads / cfg.num_kv_heads, cfg.block_size_tokens, cfg.dtype) &&
        c->layer_stride_bytes % (size_t(cfg.num_kv_heads) * cfg.head_dim * 2) == 0 &&
        (size_t(cfg.num_kv_heads) * cfg.head_dim * 2) % 16 == 0) {
        const uint32_t row_elems = cfg.num_kv_heads * cfg.head_dim;
        const uint64_t total_rows = pool_bytes / (size_t(row_elems) * 2);
        c->tmaps_ok = kriya_prefill_encode_maps(c->pool_k, c->pool_v, total_rows, row_elems, c->tmap_k, c->tmap_v) == cudaSuccess;
    }

    // Q4 cache: 16-bit staging pools for the prefill (see kriya_cuda_ctx::q4_stage_k), their maps and the identity table
    if (cfg.kv_format == KRIYA_KV_Q4_GROUP32 &&
        kriya_prefill_supported(cfg.head_dim, cfg.num_q_heads / cfg.num_kv_heads, cfg.block_size_tokens, cfg.dtype)) {
        const uint32_t row_elems = cfg.num_kv_heads * cfg.head_dim;
        const size_t stage_bytes = size_t(c->cap_indices) * cfg.block_size_tokens * row_elems * 2;
        CREATE_TRY(cudaMalloc(&c->q4_stage_k, stage_bytes));
        CREATE_TRY(cudaMalloc(&c->q4_stage_v, stage_bytes));
        CREATE_TRY(cudaMalloc(&c->q4_identity, size_t(c->cap_indices) * sizeof(int32_t)));
        std::vector<int32_t> iota(c->cap_indices);
        for (uint32_t i = 0; i < c->cap_indices; ++i) iota[i] = int32_t(i);
        CREATE_TRY(cudaMemcpy(c->q4_identity, iota.data(), iota.size() * sizeof(int32_t), cudaMemcpyHostToDevice));
        c->q4_prefill_ok = kriya_prefill_encode_maps(c->q4_stage_k, c->q4_stage_v, uint64_t(c->cap_indices) * cfg.block_size_tokens, row_elems,
                                                     c->tmap_k, c->tmap_v) == cudaSuccess;
        (void)cudaGetLastError();
    }

    // one-page-per-copy maps of the whole-page decode kernel
    if (c->tmaps_ok && kriya_decode_tcp_supported(cfg.head_dim, cfg.num_kv_heads, cfg.num_q_heads / cfg.num_kv_heads, cfg.block_size_tokens) &&
        c->layer_stride_bytes == size_t(cfg.num_kv_blocks) * c->block_bytes) {
        c->tcp_ok = kriya_decode_tcp_encode_maps(c->pool_k, c->pool_v, uint64_t(cfg.num_kv_blocks) * cfg.num_layers, c->tmap_kp,
                                                 c->tmap_vp) == cudaSuccess;
        (void)cudaGetLastError();
    }

    // RoPE table, enc:1939-1955: f32 cos/sin of pos * theta^-(2i/rot)
    {
        const uint32_t half_rot = std::max(cfg.rotary_dim / 2u, 1u);
        std::vector<float> inv_freq(half_rot);
        for (uint32_t i = 0; i < half_rot; ++i) {
            const float freq_exp = (2.0f * float(i)) / float(cfg.rotary_dim);
            inv_freq[i] = powf(cfg.rope_theta, -freq_exp);
        }
        std::vector<float> table(size_t(cfg.rope_max_seq_len) * half_rot * 2);
        for (uint32_t pos = 0; pos < cfg.rope_max_seq_len; ++pos)
            for (uint32_t i = 0; i < half_rot; ++i) {
                const float angle = float(pos) * inv_freq[i];
                table[(size_t(pos) * half_rot + i) * 2 + 0] = cosf(angle);
                table[(size_t(pos) * half_rot + i) * 2 + 1] = sinf(angle);
            }
        CREATE_TRY(cudaMalloc(&c->rope_table, table.size() * sizeof(float)));
        CREATE_TRY(cudaMemcpy(c->rope_table, table.data(), table.size() * sizeof(float), cudaMemcpyHostToDevice));
        c->rope_rotary_dim = cfg.rotary_dim;
    }

    // Plan image.  First, at fixed offsets, the lists of the block-range decode, which are built and copied on their own
    // (kriya_cuda_plan_set_ranges).  Behind them the arrays of a plan upload, packed anew for every plan so that one
    // copy moves just the bytes the plan uses (at the benchmark shape about 50 KB instead of the 470 KB the capacities
    // add up to; the copy sits in the stream in front of the step's first launch).
    size_t off = 0;
    c->cap_seg = c->cap_rows * cfg.num_kv_heads + c->tc_ctas + 8u;
    c->off_range = off;  // second work list, used by the block-range (partial state) decode
    off = align_up(off + size_t(c->cap_work) * sizeof(KriyaDecodeWork), 256);
    c->off_tcptr2 = off;
    off = align_up(off + (size_t(c->tc_ctas) + 1) * 4 * kTcpHdrWords, 256);
    c->off_tcseg2 = off;
    off = align_up(off + size_t(c->cap_seg) * sizeof(KriyaTcSeg), 256);
    c->dyn_base = off;
    off = align_up(off + (size_t(c->cap_rows) + 1) * 4, 256);                      // indptr
    off = align_up(off + size_t(c->cap_rows) * 4, 256);                            // last_page_len
    off = align_up(off + size_t(c->cap_tokens) * 4, 256);                          // positions
    off = align_up(off + size_t(c->cap_work) * sizeof(KriyaDecodeWork), 256);      // work list
    off = align_up(off + (size_t(c->tc_ctas) + 1) * 4 * kTcpHdrWords, 256);        // per-CTA segment ranges / records
    off = align_up(off + size_t(c->cap_seg) * sizeof(KriyaTcSeg), 256);            // segments
    off = align_up(off + (size_t(c->tc_ctas) + 1) * 4 * kTcpHdrWords, 256);        // the same two for the list of overlapping launches
    off = align_up(off + size_t(c->cap_seg) * sizeof(KriyaTcSeg), 256);
    off = align_up(off + size_t(c->cap_tiles) * sizeof(kriya_cta_work_tile), 256); // caller tiles
    off = align_up(off + size_t(c->cap_indices) * 4, 256);                         // page indices
    c->plan_bytes = off;
    CREATE_TRY(cudaMalloc(&c->d_plan, c->plan_bytes));
    CREATE_TRY(cudaMemsetAsync(c->d_plan, 0, c->plan_bytes, c->stream));
    {
        // Every layer of a step reads the same plan (records, segments, page indices) while the
        // pools stream through L2 between two layers; a persisting window over the plan keeps
        // those first loads of a launch out of DRAM.  A limit of this process's context only.
        const char* e = getenv("KRIYA_PLAN_L2_PERSIST");
        if ((!e || atoi(e) != 0) && prop.persistingL2CacheMaxSize > 0 && prop.accessPolicyMaxWindowSize > 0) {
            const size_t want = std::min<size_t>(c->plan_bytes, size_t(prop.accessPolicyMaxWindowSize));
            const size_t carve = std::min<size_t>(size_t(prop.persistingL2CacheMaxSize), std::max<size_t>(want, size_t(1) << 20));
            if (cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, carve) == cudaSuccess) {
                cudaStreamAttrValue av{};
                av.accessPolicyWindow.base_ptr = c->d_plan;
                av.accessPolicyWindow.num_bytes = want;
                av.accessPolicyWindow.hitRatio = carve >= want ? 1.0f : float(double(carve) / double(want));
                av.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
                av.accessPolicyWindow.missProp = cudaAccessPropertyNormal;
                if (cudaStreamSetAttribute(c->stream, cudaStreamAttributeAccessPolicyWindow, &av) != cudaSuccess)
                    (void)cudaGetLastError();
            } else {
                (void)cudaGetLastError();
            }
        }
    }
    for (int i = 0; i < 2; ++i) {
        CREATE_TRY(cudaMallocHost(&c->h_plan[i], c->plan_bytes));
        memset(c->h_plan[i], 0, c->plan_bytes);
        CREATE_TRY(cudaEventCreateWithFlags(&c->h_plan_free[i], cudaEventDisableTiming));
    }

    // split-row scratch of the CUDA-core decode kernel (its launches never overlap: one set)
    const size_t rows_hq = size_t(c->cap_work) * cfg.num_q_heads;
    CREATE_TRY(cudaMalloc(&c->part_o, rows_hq * cfg.head_dim * sizeof(float)));
    CREATE_TRY(cudaMalloc(&c->part_ml, rows_hq * 2 * sizeof(float)));
    CREATE_TRY(cudaMalloc(&c->part_counter, size_t(c->cap_rows) * sizeof(uint32_t)));
    CREATE_TRY(cudaMemsetAsync(c->part_counter, 0, size_t(c->cap_rows) * sizeof(uint32_t), c->stream));
    // split-run scratch of the tensor-core decode kernel: (value, stamp) pairs, zero stamps to begin with
    if (kriya_decode_tc_supported(cfg.head_dim, cfg.num_q_heads / cfg.num_kv_heads, cfg.block_size_tokens)) {
        // a slot holds the state of one run piece: one KV head's query heads, or all of the row's in the whole-page kernel
        const size_t heads = cfg.num_q_heads;
        c->tc_set_o_bytes = align_up(size_t(c->cap_seg) * heads * cfg.head_dim * 8, 256);
        c->tc_set_ml_bytes = align_up(size_t(c->cap_seg) * heads * 2 * 8, 256);
        CREATE_TRY(cudaMalloc(&c->tc_ll_o, kTcScratchSets * c->tc_set_o_bytes));
        CREATE_TRY(cudaMalloc(&c->tc_ll_ml, kTcScratchSets * c->tc_set_ml_bytes));
        CREATE_TRY(cudaMalloc(&c->tc_set_done, kTcScratchSets * 64));
        CREATE_TRY(cudaMemsetAsync(c->tc_ll_o, 0, kTcScratchSets * c->tc_set_o_bytes, c->stream));
        CREATE_TRY(cudaMemsetAsync(c->tc_ll_ml, 0, kTcScratchSets * c->tc_set_ml_bytes, c->stream));
        CREATE_TRY(cudaMemsetAsync(c->tc_set_done, 0, kTcScratchSets * 64, c->stream));
    }
    CREATE_TRY(cudaMalloc(&c->d_status, 256));
    CREATE_TRY(cudaMemsetAsync(c->d_status, 0, 256, c->stream));
    CREATE_TRY(cudaMallocHost(&c->h_status, 256));
    *c->h_status = 0;

    // staging for host-buffer calls: q, k, v in and out, for up to cap_tokens rows
    c->act_bytes = size_t(c->cap_tokens) * (2 * cfg.num_q_heads + 2 * cfg.num_kv_heads) * cfg.head_dim * 2;
    CREATE_TRY(cudaMalloc(&c->d_act, c->act_bytes));
    CREATE_TRY(cudaMallocHost(&c->h_act, c->act_bytes));
    CREATE_TRY(cudaMalloc(&c->d_pairs, size_t(c->cap_pairs) * 3 * sizeof(uint32_t)));
    // device staging of the host-buffer decode step (q, k, v, out of every layer for max_batch_rows rows): nothing is
    // allocated once the context exists
    c->step_bytes = 2 * size_t(c->cap_rows) * (cfg.num_q_heads + cfg.num_kv_heads) * cfg.head_dim * 2 * cfg.num_layers;
    CREATE_TRY(cudaMalloc(&c->d_step, c->step_bytes));
    if ((c->tmaps_ok || c->q4_prefill_ok) &&
        kriya_prefill_supported(cfg.head_dim, cfg.num_q_heads / cfg.num_kv_heads, cfg.block_size_tokens, cfg.dtype)) {
        const char* e = getenv("KRIYA_PREFILL_SPLIT");
        c->pf_split_enable = !(e && atoi(e) == 0);
        c->pf_split_force = (e && atoi(e) >= 2) ? uint32_t(std::min(atoi(e), 8)) : 0u;  // for tests: that many pieces whatever the policy says
        c->pf_part_slots = 4u * uint32_t(c->sm_count);
        CREATE_TRY(cudaMalloc(&c->pf_part_o, size_t(c->pf_part_slots) * 2 * cfg.head_dim * 128 * sizeof(float)));
        CREATE_TRY(cudaMalloc(&c->pf_part_ml, size_t(c->pf_part_slots) * 2 * 128 * 2 * sizeof(float)));
    }
    CREATE_TRY(cudaMalloc(&c->d_tree_state, size_t(kTreeMaxNodes) * c->cfg.num_q_heads * (c->cfg.head_dim + 2) * sizeof(float)));
    CREATE_TRY(cudaMalloc(&c->d_tree_mask, size_t(kTreeMaxNodes) * kTreeMaxNodes));
    CREATE_TRY(cudaMallocHost(&c->h_pairs, size_t(c->cap_pairs) * 3 * sizeof(uint32_t)));
    CREATE_TRY(cudaEventCreateWithFlags(&c->h_pairs_free, cudaEventDisableTiming));
    CREATE_TRY(cudaStreamSynchronize(c->stream));
#undef CREATE_TRY
    *out_ctx = c;
    return KRIYA_CUDA_OK;
}

void kriya_cuda_ctx_destroy(kriya_cuda_ctx* ctx) { destroy(ctx); }

const char* kriya_cuda_last_error(const kriya_cuda_ctx* ctx) {
    return ctx ? ctx->last_error.c_str() : g_create_error.c_str();
}

uint64_t kriya_cuda_layer_kv_byte_offset(const kriya_cuda_ctx* ctx, uint32_t layer) {
    return ctx ? uint64_t(layer) * ctx->layer_stride_bytes : 0;
}

int32_t kriya_cuda_kv_pool_ptrs(kriya_cuda_ctx* ctx, uint32_t layer, void** out_k_dev, void** out_v_dev) {
    if (!ctx) return KRIYA_CUDA_INVALID_INPUT;
    if (int32_t rc = check_layer(ctx, layer)) return rc;
    if (out_k_dev) *out_k_dev = ctx->layer_k(layer);
    if (out_v_dev) *out_v_dev = ctx->layer_v(layer);
    return KRIYA_CUDA_OK;
}

void* kriya_cuda_stream(kriya_cuda_ctx* ctx) { return ctx ? static_cast<void*>(ctx->stream) : nullptr; }

uint64_t kriya_cuda_launch_count(const kriya_cuda_ctx* ctx) { return ctx ? ctx->launches : 0; }

int32_t kriya_cuda_sync(kriya_cuda_ctx* ctx, uint32_t timeout_ms) {
    if (!ctx) return KRIYA_CUDA_INVALID_INPUT;
    cudaSetDevice(ctx->cfg.device);
    KRIYA_CUDA_TRY(ctx, cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(uint32_t), cudaMemcpyDeviceToHost,
                                        ctx->stream));
    if (timeout_ms == 0) {
        KRIYA_CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    } else {
        const auto t0 = std::chrono::steady_clock::now();
        for (;;) {
            const cudaError_t q = cudaStreamQuery(ctx->stream);
            if (q == cudaSuccess) break;
            if (q != cudaErrorNotReady)
                return ctx->fail(KRIYA_CUDA_EXECUTION_ERROR, std::string("stream query: ") + cudaGetErrorString(q));
            const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0);
            if (ms.count() > int64_t(timeout_ms))
                return ctx->fail(KRIYA_CUDA_TIMEOUT, "queued work did not finish within " + std::to_string(timeout_ms) + " ms");
            std::this_thread::yield();
        }
    }
    const uint32_t st = *ctx->h_status;
    if (st != KRIYA_DEV_OK) {
        cudaMemsetAsync(ctx->d_status, 0, sizeof(uint32_t), ctx->stream);
        *ctx->h_status = 0;
        const char* what = st == KRIYA_DEV_BAD_BLOCK_INDEX ? "a page index outside the pool reached a kernel"
                           : st == KRIYA_DEV_WAIT_EXPIRED  ? "a bounded wait inside a kernel expired"
                           : st == KRIYA_DEV_BAD_SLOT      ? "a slot index outside its block reached a kernel"
                                                           : "unknown kernel status";
        return ctx->fail(KRIYA_CUDA_EXECUTION_ERROR, what);
    }
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_plan_upload(kriya_cuda_ctx* c, const int32_t* indptr, size_t indptr_len, const int32_t* indices,
                               size_t indices_len, const int32_t* last_len, size_t last_len_len,
                               const kriya_cta_work_tile* tiles, size_t tiles_len, const uint32_t* positions,
                               size_t n_positions) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    c->plan_valid = false;
    c->ranges_valid = false;
    auto invalid = [&](const std::string& m) { return c->fail(KRIYA_CUDA_INVALID_INPUT, m); };
    // validate_batch_inputs, enc:2159-2218
    if (!indptr || indptr_len < 2) return invalid("page_indptr must hold at least one row");
    const size_t rows = indptr_len - 1;
    if (!last_len || last_len_len != rows)
        return invalid("last_page_len has " + std::to_string(last_len_len) + " entries but page_indptr describes " +
                       std::to_string(rows) + " rows");
    if (indices_len > 0 && !indices) return invalid("page_indices must not be null");
    if (tiles_len > 0 && !tiles) return invalid("cta_work_tiles must not be null");
    if (n_positions > 0 && !positions) return invalid("seq_positions must not be null");
    auto over = [&](const char* name, size_t len, size_t cap) {
        return invalid(std::string(name) + " has " + std::to_string(len) + " entries but its GPU buffer holds " +
                       std::to_string(cap));
    };
    if (rows > c->cap_rows) return over("page_indptr", indptr_len, size_t(c->cap_rows) + 1);
    if (indices_len > c->cap_indices) return over("page_indices", indices_len, c->cap_indices);
    if (tiles_len > c->cap_tiles) return over("cta_work_tiles", tiles_len, c->cap_tiles);
    if (n_positions > c->cap_tokens) return over("seq_positions", n_positions, c->cap_tokens);
    // what the kernels rely on
    if (indptr[0] != 0) return invalid("page_indptr must start at 0");
    for (size_t r = 0; r < rows; ++r) {
        if (indptr[r + 1] < indptr[r]) return invalid("page_indptr must be non-decreasing (row " + std::to_string(r) + ")");
        if (last_len[r] < 1 || uint32_t(last_len[r]) > c->cfg.block_size_tokens)
            return invalid("last_page_len[" + std::to_string(r) + "] = " + std::to_string(last_len[r]) +
                           " outside 1..=" + std::to_string(c->cfg.block_size_tokens));
        if (indptr[r + 1] == indptr[r]) return invalid("row " + std::to_string(r) + " has no KV blocks");
    }
    if (size_t(indptr[rows]) != indices_len)
        return invalid("page_indptr ends at " + std::to_string(indptr[rows]) + " but page_indices has " +
                       std::to_string(indices_len) + " entries");
    for (size_t i = 0; i < indices_len; ++i)
        if (indices[i] < 0 || uint32_t(indices[i]) >= c->cfg.num_kv_blocks)
            return invalid("page_indices[" + std::to_string(i) + "] = " + std::to_string(indices[i]) +
                           " outside the pool of " + std::to_string(c->cfg.num_kv_blocks) + " blocks");
    for (size_t t = 0; t < tiles_len; ++t) {
        const kriya_cta_work_tile& w = tiles[t];
        if (w.request_idx >= rows) return invalid("cta_work_tiles[" + std::to_string(t) + "].request_idx out of range");
        const uint32_t nb = uint32_t(indptr[w.request_idx + 1] - indptr[w.request_idx]);
        if (w.kv_block_start > nb || w.kv_block_count > nb - w.kv_block_start)
            return invalid("cta_work_tiles[" + std::to_string(t) + "] reaches outside its row");
    }

    cudaSetDevice(c->cfg.device);
    const int cur = c->h_plan_cur;
    c->h_plan_cur ^= 1;
    KRIYA_CUDA_TRY(c, cudaEventSynchronize(c->h_plan_free[cur]));  // the copy that last read this buffer is done
    uint8_t* h = c->h_plan[cur];
    // pack the plan's arrays behind one another; the context's offsets change only once everything has been built
    size_t off = c->dyn_base;
    auto place = [&](size_t bytes) {
        const size_t o = off;
        off = align_up(off + bytes, 256);
        return o;
    };
    const size_t o_indptr = place(indptr_len * 4), o_last = place(rows * 4), o_pos = place(std::max<size_t>(n_positions, 1) * 4);
    memcpy(h + o_indptr, indptr, indptr_len * 4);
    memcpy(h + o_last, last_len, rows * 4);
    if (n_positions) memcpy(h + o_pos, positions, n_positions * 4);
    const size_t o_work = off;
    auto* work = reinterpret_cast<KriyaDecodeWork*>(h + o_work);
    const uint32_t n_work =
        build_work(indptr, last_len, c->cfg.block_size_tokens, c->attention_window, uint32_t(rows), nullptr, nullptr,
                   2u * uint32_t(c->sm_count), 2u, work, c->cap_work);
    if (n_work == UINT32_MAX) return invalid("plan needs more decode work items than the context holds");
    place(size_t(n_work) * sizeof(KriyaDecodeWork));
    const int variant = choose_tc_variant(c, indptr, uint32_t(rows), nullptr, nullptr);
    const TcVariantGeometry geo = tc_geometry(c, variant);
    const uint32_t plan_ctas = geo.ctas;
    const size_t o_ptr = place((size_t(plan_ctas) + 1) * 4 * (variant == 2 ? kTcpHdrWords : 1u));
    const size_t o_seg = off;
    const uint32_t n_seg = build_tc_segments(indptr, last_len, c->cfg.block_size_tokens, uint32_t(rows), geo.runs_per_row, nullptr,
                                             nullptr, plan_ctas, geo.pages_per_tile, reinterpret_cast<KriyaTcSeg*>(h + o_seg),
                                             c->cap_seg, reinterpret_cast<uint32_t*>(h + o_ptr), geo.min_tiles, c->attention_window);
    if (n_seg == UINT32_MAX) return invalid("plan needs more decode segments than the context holds");
    if (variant == 2)
        expand_tcp_headers(reinterpret_cast<uint32_t*>(h + o_ptr), plan_ctas, reinterpret_cast<const KriyaTcSeg*>(h + o_seg), indices,
                           geo.pages_per_tile, c->cfg.block_size_tokens, positions, uint32_t(n_positions));
    place(size_t(n_seg) * sizeof(KriyaTcSeg));
    // the list for the overlapping launches of a whole-step call: the same rows, more tiles per CTA
    size_t o_ptr3 = 0, o_seg3 = 0;
    uint32_t n_seg3 = 0;
    bool chain_list = variant == 2 && c->tc_chain_min_tiles > geo.min_tiles;
    if (chain_list) {
        o_ptr3 = place((size_t(plan_ctas) + 1) * 4 * kTcpHdrWords);
        o_seg3 = off;
        n_seg3 = build_tc_segments(indptr, last_len, c->cfg.block_size_tokens, uint32_t(rows), geo.runs_per_row, nullptr, nullptr, plan_ctas,
                                   geo.pages_per_tile, reinterpret_cast<KriyaTcSeg*>(h + o_seg3), c->cap_seg,
                                   reinterpret_cast<uint32_t*>(h + o_ptr3), c->tc_chain_min_tiles, c->attention_window);
        if (n_seg3 == UINT32_MAX) {  // (it has no more pieces than the ordinary list; should it not fit, that list serves)
            chain_list = false;
            n_seg3 = 0;
        } else {
            expand_tcp_headers(reinterpret_cast<uint32_t*>(h + o_ptr3), plan_ctas, reinterpret_cast<const KriyaTcSeg*>(h + o_seg3), indices,
                               geo.pages_per_tile, c->cfg.block_size_tokens, positions, uint32_t(n_positions));
            place(size_t(n_seg3) * sizeof(KriyaTcSeg));
        }
    }
    const size_t o_tiles = place(std::max<size_t>(tiles_len, 1) * sizeof(kriya_cta_work_tile));
    if (tiles_len) memcpy(h + o_tiles, tiles, tiles_len * sizeof(kriya_cta_work_tile));
    const size_t o_indices = place(std::max<size_t>(indices_len, 1) * 4);
    if (indices_len) memcpy(h + o_indices, indices, indices_len * 4);
    KRIYA_CUDA_TRY(c, cudaMemcpyAsync(c->d_plan + c->dyn_base, h + c->dyn_base, off - c->dyn_base, cudaMemcpyHostToDevice, c->stream));
    KRIYA_CUDA_TRY(c, cudaEventRecord(c->h_plan_free[cur], c->stream));
    c->off_indptr = o_indptr;
    c->off_last_len = o_last;
    c->off_positions = o_pos;
    c->off_work = o_work;
    c->off_tcptr = o_ptr;
    c->off_tcseg = o_seg;
    c->off_tiles = o_tiles;
    c->off_indices = o_indices;
    c->tc_variant = variant;
    c->n_seg = n_seg;
    c->tc_max_parts = max_parts_of(reinterpret_cast<const KriyaTcSeg*>(h + o_seg), n_seg);
    c->chain_list_valid = chain_list;
    c->off_tcptr3 = o_ptr3;
    c->off_tcseg3 = o_seg3;
    c->n_seg_chain = n_seg3;
    c->tc_max_parts_chain = chain_list ? max_parts_of(reinterpret_cast<const KriyaTcSeg*>(h + o_seg3), n_seg3) : 0u;

    c->n_rows = uint32_t(rows);
    c->n_indices = uint32_t(indices_len);
    c->n_tiles = uint32_t(tiles_len);
    c->n_positions = uint32_t(n_positions);
    c->n_work = n_work;
    c->row0_blocks = uint32_t(indptr[1] - indptr[0]);
    c->row0_last_len = uint32_t(last_len[0]);
    c->h_plan_last = h;
    uint64_t tokens = 0;
    for (size_t r = 0; r < rows; ++r)
        tokens += uint64_t(indptr[r + 1] - indptr[r] - 1) * c->cfg.block_size_tokens + uint32_t(last_len[r]);
    c->total_row_tokens = tokens;
    c->positions_are_context = n_positions == rows;
    for (size_t r = 0; r < rows && c->positions_are_context; ++r) {
        const uint64_t row_tokens = uint64_t(indptr[r + 1] - indptr[r] - 1) * c->cfg.block_size_tokens + uint32_t(last_len[r]);
        c->positions_are_context = uint64_t(positions[r]) + 1u == row_tokens;
    }
    c->plan_valid = true;
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_rope_kv_append(kriya_cuda_ctx* c, uint32_t layer, void* q, const void* k, const void* v,
                                  const void* qw, const void* kw, uint32_t num_tokens,
                                  const kriya_rope_kv_write_params* p) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (int32_t rc = check_layer(c, layer)) return rc;
    if (int32_t rc = check_rope(c, p)) return rc;
    if (!c->plan_valid) return c->fail(KRIYA_CUDA_INVALID_INPUT, "no plan uploaded");
    if (num_tokens == 0) return c->fail(KRIYA_CUDA_INVALID_INPUT, "input_tokens must not be empty");  // enc:2165-2169
    if (!q || !k || !v) return c->fail(KRIYA_CUDA_INVALID_INPUT, "q, k and v must not be null");
    if (p->apply_qk_norm && (!qw || !kw)) return c->fail(KRIYA_CUDA_INVALID_INPUT, "apply_qk_norm needs both norm weights");
    if (num_tokens > c->n_rows)
        return c->fail(KRIYA_CUDA_INVALID_INPUT, "append of " + std::to_string(num_tokens) + " tokens but the plan has " +
                                                     std::to_string(c->n_rows) + " rows");
    if (num_tokens != c->n_positions)  // enc:2170-2176
        return c->fail(KRIYA_CUDA_INVALID_INPUT, "input_tokens has " + std::to_string(num_tokens) +
                                                     " entries but seq_positions has " + std::to_string(c->n_positions));
    cudaSetDevice(c->cfg.device);
    return launch_append(c, layer, q, k, v, qw, kw, num_tokens, 0, 0, p);
}

int32_t kriya_cuda_rope_kv_append_chunk(kriya_cuda_ctx* c, uint32_t layer, void* q, const void* k, const void* v,
                                        const void* qw, const void* kw, uint32_t prefix_tokens, uint32_t num_tokens,
                                        const kriya_rope_kv_write_params* p) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (int32_t rc = check_layer(c, layer)) return rc;
    if (int32_t rc = check_rope(c, p)) return rc;
    if (!c->plan_valid) return c->fail(KRIYA_CUDA_INVALID_INPUT, "no plan uploaded");
    if (num_tokens == 0) return c->fail(KRIYA_CUDA_INVALID_INPUT, "input_tokens must not be empty");
    if (!q || !k || !v) return c->fail(KRIYA_CUDA_INVALID_INPUT, "q, k and v must not be null");
    if (p->apply_qk_norm && (!qw || !kw)) return c->fail(KRIYA_CUDA_INVALID_INPUT, "apply_qk_norm needs both norm weights");
    if (num_tokens > c->cap_tokens) return c->fail(KRIYA_CUDA_INVALID_INPUT, "chunk exceeds max_query_tokens");
    const uint64_t end = uint64_t(prefix_tokens) + num_tokens;
    if (end > uint64_t(c->row0_blocks) * c->cfg.block_size_tokens)
        return c->fail(KRIYA_CUDA_INVALID_INPUT, "chunk ends at token " + std::to_string(end) + " but row 0 of the plan holds " +
                                                     std::to_string(c->row0_blocks) + " blocks");
    cudaSetDevice(c->cfg.device);
    return launch_append(c, layer, q, k, v, qw, kw, num_tokens, 1, prefix_tokens, p);
}

int32_t kriya_cuda_rope_kv_append_chunk_batch(kriya_cuda_ctx* c, uint32_t layer, void* q, const void* k, const void* v,
                                              const void* qw, const void* kw, uint32_t n_seqs, const uint32_t* q_start,
                                              const uint32_t* prefix, const uint32_t* count, const kriya_rope_kv_write_params* p) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (int32_t rc = check_layer(c, layer)) return rc;
    if (int32_t rc = check_rope(c, p)) return rc;
    if (!c->plan_valid) return c->fail(KRIYA_CUDA_INVALID_INPUT, "no plan uploaded");
    if (!q || !k || !v || !q_start || !prefix || !count) return c->fail(KRIYA_CUDA_INVALID_INPUT, "q, k, v and the per-sequence arrays must not be null");
    if (p->apply_qk_norm && (!qw || !kw)) return c->fail(KRIYA_CUDA_INVALID_INPUT, "apply_qk_norm needs both norm weights");
    if (n_seqs == 0) return c->fail(KRIYA_CUDA_INVALID_INPUT, "input_tokens must not be empty");
    if (n_seqs > c->n_rows) return c->fail(KRIYA_CUDA_INVALID_INPUT, "more sequences than plan rows");
    if (size_t(n_seqs) * 3 > size_t(c->cap_pairs) * 3) return c->fail(KRIYA_CUDA_INVALID_INPUT, "more sequences than the context holds");
    const int32_t* indptr = reinterpret_cast<const int32_t*>(c->h_plan_last + c->off_indptr);
    uint32_t rows = 0;
    for (uint32_t r = 0; r < n_seqs; ++r) {
        if (count[r] == 0) return c->fail(KRIYA_CUDA_INVALID_INPUT, "input_tokens must not be empty");
        const uint64_t end = uint64_t(prefix[r]) + count[r];
        if (end > uint64_t(indptr[r + 1] - indptr[r]) * c->cfg.block_size_tokens)
            return c->fail(KRIYA_CUDA_INVALID_INPUT, "chunk of sequence " + std::to_string(r) + " ends at token " + std::to_string(end) +
                                                         " but its plan row holds " + std::to_string(indptr[r + 1] - indptr[r]) + " blocks");
        if (uint64_t(q_start[r]) + count[r] > c->cap_tokens) return c->fail(KRIYA_CUDA_INVALID_INPUT, "chunk exceeds max_query_tokens");
        rows = std::max(rows, q_start[r] + count[r]);
    }
    cudaSetDevice(c->cfg.device);
    KRIYA_CUDA_TRY(c, cudaEventSynchronize(c->h_pairs_free));
    memcpy(c->h_pairs, q_start, size_t(n_seqs) * 4);
    memcpy(c->h_pairs + n_seqs, prefix, size_t(n_seqs) * 4);
    memcpy(c->h_pairs + 2 * size_t(n_seqs), count, size_t(n_seqs) * 4);
    KRIYA_CUDA_TRY(c, cudaMemcpyAsync(c->d_pairs, c->h_pairs, size_t(n_seqs) * 12, cudaMemcpyHostToDevice, c->stream));
    KRIYA_CUDA_TRY(c, cudaEventRecord(c->h_pairs_free, c->stream));
    KriyaAppendArgs a{};
    a.q_inout = q;
    a.k_in = k;
    a.v_in = v;
    a.q_norm_w = qw;
    a.k_norm_w = kw;
    a.cache_k = c->layer_k(layer);
    a.cache_v = c->layer_v(layer);
    a.indptr = c->plan_dev<int32_t>(c->off_indptr);
    a.indices = c->plan_dev<int32_t>(c->off_indices);
    a.last_len = c->plan_dev<int32_t>(c->off_last_len);
    a.positions = c->plan_dev<uint32_t>(c->off_positions);
    a.table = table_for(c, p);
    a.status = c->d_status;
    a.num_tokens = rows;
    a.num_blocks = c->cfg.num_kv_blocks;
    a.chunk_mode = 2;
    a.kv_q4 = c->cfg.kv_format == KRIYA_KV_Q4_GROUP32 ? 1u : 0u;
    a.seq_q_start = c->d_pairs;
    a.seq_prefix = c->d_pairs + n_seqs;
    a.seq_count = c->d_pairs + 2 * size_t(n_seqs);
    a.n_seqs = n_seqs;
    a.p = *p;
    TimingScope ts(c, 1);
    KRIYA_CUDA_TRY(c, kriya_launch_append(a, c->cfg.dtype, c->stream));
    c->launches += 1;
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_rope_inplace(kriya_cuda_ctx* c, void* q, void* k, const void* qw, const void* kw, uint32_t num_tokens,
                                const kriya_rope_kv_write_params* p) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (int32_t rc = check_rope(c, p)) return rc;
    if (!c->plan_valid) return c->fail(KRIYA_CUDA_INVALID_INPUT, "no plan uploaded");
    if (num_tokens == 0) return c->fail(KRIYA_CUDA_INVALID_INPUT, "input_tokens must not be empty");
    if (!q || !k) return c->fail(KRIYA_CUDA_INVALID_INPUT, "q and k must not be null");
    if (p->apply_qk_norm && (!qw || !kw)) return c->fail(KRIYA_CUDA_INVALID_INPUT, "apply_qk_norm needs both norm weights");
    if (num_tokens != c->n_positions)
        return c->fail(KRIYA_CUDA_INVALID_INPUT, "input_tokens has " + std::to_string(num_tokens) +
                                                     " entries but seq_positions has " + std::to_string(c->n_positions));
    cudaSetDevice(c->cfg.device);
    KriyaAppendArgs a{};
    a.q_inout = q;
    a.k_in = k;
    a.q_norm_w = qw;
    a.k_norm_w = kw;
    a.positions = c->plan_dev<uint32_t>(c->off_positions);
    a.table = table_for(c, p);
    a.status = c->d_status;
    a.num_tokens = num_tokens;
    a.num_blocks = c->cfg.num_kv_blocks;
    a.inplace = 1;
    a.p = *p;
    KRIYA_CUDA_TRY(c, kriya_launch_append(a, c->cfg.dtype, c->stream));
    c->launches += 1;
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_tree_verify(kriya_cuda_ctx* c, uint32_t layer, const void* tq, const void* tk, const void* tv,
                               const uint8_t* mask, void* out, const kriya_tree_verify_params* p) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (int32_t rc = check_layer(c, layer)) return rc;
    if (!p) return c->fail(KRIYA_CUDA_INVALID_INPUT, "params must not be null");
    if (p->num_q_heads != c->cfg.num_q_heads || p->num_kv_heads != c->cfg.num_kv_heads || p->head_dim != c->cfg.head_dim ||
        p->block_size_tokens != c->cfg.block_size_tokens)
        return c->fail(KRIYA_CUDA_INVALID_INPUT, "tree-verify params do not match the context's attention shape");
    if (!tq || !tk || !tv || !mask || !out) return c->fail(KRIYA_CUDA_INVALID_INPUT, "tree q, k, v, mask and out must not be null");
    const uint32_t n = p->num_tree_nodes;
    if (n == 0) return c->fail(KRIYA_CUDA_INVALID_INPUT, "input_tokens must not be empty");
    if (n > kTreeMaxNodes) return c->fail(KRIYA_CUDA_INVALID_INPUT, "a draft tree may hold at most 128 nodes");
    if (c->cfg.head_dim != 64 && c->cfg.head_dim != 128)
        return c->fail(KRIYA_CUDA_UNSUPPORTED, "tree verification covers head_dim 64/128");
    if (c->cfg.kv_format != KRIYA_KV_16BIT) return c->fail(KRIYA_CUDA_UNSUPPORTED, "tree verification covers the 16-bit cache");
    const bool has_prefix = p->prefix_kv_blocks > 0;
    if (has_prefix) {
        if (p->prefix_last_len == 0 || p->prefix_last_len > p->block_size_tokens)
            return c->fail(KRIYA_CUDA_INVALID_INPUT, "prefix_last_len must be in 1..=block_size_tokens");
        if (!c->plan_valid || c->n_rows != n)
            return c->fail(KRIYA_CUDA_INVALID_INPUT, "tree verification over a cached prefix needs a plan with one row per tree node");
        const int32_t* indptr = reinterpret_cast<const int32_t*>(c->h_plan_last + c->off_indptr);
        const int32_t* last = reinterpret_cast<const int32_t*>(c->h_plan_last + c->off_last_len);
        for (uint32_t r = 0; r < n; ++r)
            if (uint32_t(indptr[r + 1] - indptr[r]) != p->prefix_kv_blocks || uint32_t(last[r]) != p->prefix_last_len)
                return c->fail(KRIYA_CUDA_INVALID_INPUT, "plan row " + std::to_string(r) + " does not describe the prefix (" +
                                                             std::to_string(p->prefix_kv_blocks) + " blocks, last length " +
                                                             std::to_string(p->prefix_last_len) + ")");
        if (!use_tc_decode(c) && !kriya_decode_supported(c->cfg.head_dim, c->cfg.num_q_heads / c->cfg.num_kv_heads,
                                                         c->cfg.num_kv_heads, c->cfg.block_size_tokens))
            return c->fail(KRIYA_CUDA_UNSUPPORTED,
                           "decode kernels cover head_dim 64/128, group size 1..8, 16-token blocks (head_dim 64: up to 8 KV heads)");
    }
    cudaSetDevice(c->cfg.device);
    // The layers of one verification pass the same mask: it is copied (through the pinned staging buffer the copy lists
    // use) only when it differs from the one already on the device.
    if (c->tree_mask_last.size() != size_t(n) * n || memcmp(c->tree_mask_last.data(), mask, size_t(n) * n) != 0) {
        KRIYA_CUDA_TRY(c, cudaEventSynchronize(c->h_pairs_free));
        memcpy(c->h_pairs, mask, size_t(n) * n);
        KRIYA_CUDA_TRY(c, cudaMemcpyAsync(c->d_tree_mask, c->h_pairs, size_t(n) * n, cudaMemcpyHostToDevice, c->stream));
        KRIYA_CUDA_TRY(c, cudaEventRecord(c->h_pairs_free, c->stream));
        c->tree_mask_last.assign(mask, mask + size_t(n) * n);
    }
    const size_t R = size_t(n) * c->cfg.num_q_heads;
    float* st_m = c->d_tree_state;
    float* st_l = st_m + R;
    float* st_o = st_l + R;
    if (has_prefix) {
        // part A: every node is a decode row over the same prefix blocks; the state is left un-normalised
        kriya_bsr_gqa_params g{};
        g.num_q_heads = p->num_q_heads;
        g.num_kv_heads = p->num_kv_heads;
        g.head_dim = p->head_dim;
        g.block_size_tokens = p->block_size_tokens;
        g.max_split_k_tiles = 1;
        g.max_query_tokens = n;
        g.sm_scale = p->sm_scale;
        g.logit_softcap = 0.0f;
        if (int32_t rc = launch_decode(c, layer, tq, nullptr, st_m, st_l, st_o, false, c->n_work, &g)) return rc;
    }
    KriyaTreeArgs a{};
    a.q = tq;
    a.k = tk;
    a.v = tv;
    a.mask = c->d_tree_mask;
    a.st_m = st_m;
    a.st_l = st_l;
    a.st_o = st_o;
    a.out = out;
    a.n_nodes = n;
    a.num_q_heads = c->cfg.num_q_heads;
    a.num_kv_heads = c->cfg.num_kv_heads;
    a.has_prefix = has_prefix ? 1u : 0u;
    a.sm_scale = p->sm_scale;
    KRIYA_CUDA_TRY(c, kriya_launch_tree_finish(a, c->cfg.head_dim, c->cfg.dtype, c->stream));
    c->launches += 1;
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_paged_gqa_decode(kriya_cuda_ctx* c, uint32_t layer, const void* q, void* out,
                                    const kriya_bsr_gqa_params* p) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (int32_t rc = check_layer(c, layer)) return rc;
    if (int32_t rc = check_gqa(c, p)) return rc;
    if (!c->plan_valid) return c->fail(KRIYA_CUDA_INVALID_INPUT, "no plan uploaded");
    if (!q || !out) return c->fail(KRIYA_CUDA_INVALID_INPUT, "q and out must not be null");
    if (!use_tc_decode(c) && !kriya_decode_supported(c->cfg.head_dim, c->cfg.num_q_heads / c->cfg.num_kv_heads,
                                                     c->cfg.num_kv_heads, c->cfg.block_size_tokens))
        return c->fail(KRIYA_CUDA_UNSUPPORTED,
                       "decode kernels cover head_dim 64/128, group size 1..8, 16-token blocks (head_dim 64: up to 8 KV heads)");
    cudaSetDevice(c->cfg.device);
    return launch_decode(c, layer, q, out, nullptr, nullptr, nullptr, false, c->n_work, p);
}

int32_t kriya_cuda_plan_set_ranges(kriya_cuda_ctx* c, const uint32_t* blk_begin, const uint32_t* blk_end) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (!c->plan_valid) return c->fail(KRIYA_CUDA_INVALID_INPUT, "no plan uploaded");
    cudaSetDevice(c->cfg.device);
    // work lists for the requested ranges, staged behind the plan's own lists
    KRIYA_CUDA_TRY(c, cudaEventSynchronize(c->h_pairs_free));
    const int32_t* indptr = reinterpret_cast<const int32_t*>(c->h_plan_last + c->off_indptr);
    auto* work = reinterpret_cast<KriyaDecodeWork*>(c->h_plan_last + c->off_range);
    const int32_t* last_len_h = reinterpret_cast<const int32_t*>(c->h_plan_last + c->off_last_len);
    const uint32_t n_work = build_work(indptr, last_len_h, c->cfg.block_size_tokens, c->attention_window, c->n_rows, blk_begin,
                                       blk_end, 2u * uint32_t(c->sm_count), 2u, work, c->cap_work);
    if (n_work == UINT32_MAX) return c->fail(KRIYA_CUDA_INVALID_INPUT, "ranges need more work items than the context holds");
    KRIYA_CUDA_TRY(c, cudaMemcpyAsync(c->d_plan + c->off_range, work, size_t(n_work) * sizeof(KriyaDecodeWork),
                                      cudaMemcpyHostToDevice, c->stream));
    auto* segs = reinterpret_cast<KriyaTcSeg*>(c->h_plan_last + c->off_tcseg2);
    auto* sptr = reinterpret_cast<uint32_t*>(c->h_plan_last + c->off_tcptr2);
    c->tc_variant_ranges = choose_tc_variant(c, indptr, c->n_rows, blk_begin, blk_end);
    const TcVariantGeometry geo = tc_geometry(c, c->tc_variant_ranges);
    const uint32_t n_seg = build_tc_segments(
        indptr, reinterpret_cast<const int32_t*>(c->h_plan_last + c->off_last_len), c->cfg.block_size_tokens, c->n_rows,
        geo.runs_per_row, blk_begin, blk_end, geo.ctas, geo.pages_per_tile, segs, c->cap_seg, sptr, geo.min_tiles,
        c->attention_window);
    if (n_seg == UINT32_MAX) return c->fail(KRIYA_CUDA_INVALID_INPUT, "ranges need more segments than the context holds");
    if (c->tc_variant_ranges == 2)
        expand_tcp_headers(sptr, geo.ctas, segs, reinterpret_cast<const int32_t*>(c->h_plan_last + c->off_indices), geo.pages_per_tile,
                           c->cfg.block_size_tokens, reinterpret_cast<const uint32_t*>(c->h_plan_last + c->off_positions), c->n_positions);
    c->n_seg_ranges = n_seg;
    c->tc_max_parts_ranges = max_parts_of(segs, n_seg);
    KRIYA_CUDA_TRY(c, cudaMemcpyAsync(c->d_plan + c->off_tcptr2, sptr, c->off_tcseg2 - c->off_tcptr2 + size_t(n_seg) * sizeof(KriyaTcSeg),
                                      cudaMemcpyHostToDevice, c->stream));
    KRIYA_CUDA_TRY(c, cudaEventRecord(c->h_pairs_free, c->stream));
    c->n_work_ranges = n_work;
    c->ranges_valid = true;
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_paged_gqa_decode_partial(kriya_cuda_ctx* c, uint32_t layer, const void* q, const uint32_t* blk_begin,
                                            const uint32_t* blk_end, float* out_m, float* out_l, float* out_o,
                                            const kriya_bsr_gqa_params* p) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (int32_t rc = check_layer(c, layer)) return rc;
    if (int32_t rc = check_gqa(c, p)) return rc;
    if (!c->plan_valid) return c->fail(KRIYA_CUDA_INVALID_INPUT, "no plan uploaded");
    if (!q || !out_m || !out_l || !out_o) return c->fail(KRIYA_CUDA_INVALID_INPUT, "q and state outputs must not be null");
    if (!use_tc_decode(c) && !kriya_decode_supported(c->cfg.head_dim, c->cfg.num_q_heads / c->cfg.num_kv_heads,
                                                     c->cfg.num_kv_heads, c->cfg.block_size_tokens))
        return c->fail(KRIYA_CUDA_UNSUPPORTED,
                       "decode kernels cover head_dim 64/128, group size 1..8, 16-token blocks (head_dim 64: up to 8 KV heads)");
    cudaSetDevice(c->cfg.device);
    if (blk_begin != nullptr || blk_end != nullptr) {
        if (int32_t rc = kriya_cuda_plan_set_ranges(c, blk_begin, blk_end)) return rc;
    } else if (!c->ranges_valid) {
        // whole rows: the lists built by the plan upload serve
        return launch_decode(c, layer, q, nullptr, out_m, out_l, out_o, false, c->n_work, p);
    }
    const uint32_t n_work = c->n_work_ranges;
    return launch_decode(c, layer, q, nullptr, out_m, out_l, out_o, true, n_work, p);
}

int32_t kriya_cuda_merge_states(kriya_cuda_ctx* c, const float* m, const float* l, const float* o, uint32_t parts,
                                uint32_t rows_times_heads, void* out) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (!m || !l || !o || !out || parts == 0) return c->fail(KRIYA_CUDA_INVALID_INPUT, "merge needs states, an output and parts >= 1");
    cudaSetDevice(c->cfg.device);
    KRIYA_CUDA_TRY(c, kriya_launch_merge_states(m, l, o, parts, rows_times_heads, c->cfg.head_dim, rows_times_heads,
                                                size_t(rows_times_heads) * c->cfg.head_dim, out, c->cfg.dtype, c->stream));
    c->launches += 1;
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_merge_packed_states(kriya_cuda_ctx* c, const float* packed, uint32_t parts, uint32_t rows_times_heads,
                                       void* out) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (!packed || !out || parts == 0) return c->fail(KRIYA_CUDA_INVALID_INPUT, "merge needs states, an output and parts >= 1");
    cudaSetDevice(c->cfg.device);
    const size_t R = rows_times_heads, stride = R * (size_t(c->cfg.head_dim) + 2);
    KRIYA_CUDA_TRY(c, kriya_launch_merge_states(packed, packed + R, packed + 2 * R, parts, rows_times_heads, c->cfg.head_dim,
                                                stride, stride, out, c->cfg.dtype, c->stream));
    c->launches += 1;
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_paged_gqa_prefill_batch(kriya_cuda_ctx* c, uint32_t layer, const void* q, void* out, uint32_t n_seqs,
                                           const uint32_t* q_start, const uint32_t* prefix, const uint32_t* count,
                                           const kriya_bsr_gqa_params* p) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (int32_t rc = check_layer(c, layer)) return rc;
    if (int32_t rc = check_gqa(c, p)) return rc;
    if (!c->plan_valid) return c->fail(KRIYA_CUDA_INVALID_INPUT, "no plan uploaded");
    if (!q || !out || !q_start || !prefix || !count) return c->fail(KRIYA_CUDA_INVALID_INPUT, "q, out and the per-sequence arrays must not be null");
    if (n_seqs == 0) return c->fail(KRIYA_CUDA_INVALID_INPUT, "input_tokens must not be empty");
    if (n_seqs > c->n_rows) return c->fail(KRIYA_CUDA_INVALID_INPUT, "more sequences than plan rows");
    if (!kriya_prefill_supported(c->cfg.head_dim, c->cfg.num_q_heads / c->cfg.num_kv_heads, c->cfg.block_size_tokens,
                                 c->cfg.dtype) || !(c->tmaps_ok || c->q4_prefill_ok))
        return c->fail(KRIYA_CUDA_UNSUPPORTED, "prefill kernels cover head_dim 64/128 and 16-token blocks");
    const bool q4 = c->cfg.kv_format == KRIYA_KV_Q4_GROUP32;
    cudaSetDevice(c->cfg.device);
    KRIYA_CUDA_TRY(c, cudaEventSynchronize(c->h_pairs_free));
    const int32_t* indptr = reinterpret_cast<const int32_t*>(c->h_plan_last + c->off_indptr);
    auto* tiles = reinterpret_cast<KriyaPrefillTile*>(c->h_pairs);
    const uint32_t cap_tiles = uint32_t(size_t(c->cap_pairs) * 3 * sizeof(uint32_t) / sizeof(KriyaPrefillTile));
    uint32_t n = 0, q_rows = 0;
    for (uint32_t r = 0; r < n_seqs; ++r) {
        if (count[r] == 0) return c->fail(KRIYA_CUDA_INVALID_INPUT, "input_tokens must not be empty");
        q_rows = std::max(q_rows, q_start[r] + count[r]);
        const uint64_t end = uint64_t(prefix[r]) + count[r];
        const uint64_t row_cap = uint64_t(indptr[r + 1] - indptr[r]) * c->cfg.block_size_tokens;
        if (end > row_cap)
            return c->fail(KRIYA_CUDA_INVALID_INPUT, "chunk of sequence " + std::to_string(r) + " ends at token " + std::to_string(end) +
                                                         " but its plan row holds " + std::to_string(row_cap / c->cfg.block_size_tokens) + " blocks");
        if (uint64_t(q_start[r]) + count[r] > c->cap_tokens) return c->fail(KRIYA_CUDA_INVALID_INPUT, "chunk exceeds max_query_tokens");
        for (uint32_t t0 = 0; t0 < count[r]; t0 += 128u) {
            if (n >= cap_tiles) return c->fail(KRIYA_CUDA_INVALID_INPUT, "more query tiles than the context holds");
            tiles[n++] = KriyaPrefillTile{uint32_t(indptr[r]), q_start[r] + t0, std::min(128u, count[r] - t0), prefix[r] + t0,
                                          uint32_t(end), 0u, 0u, UINT32_MAX};
        }
    }
    // A launch with few tiles (one request's chunk is 24 CTAs at the Qwen2.5-1.5B shape) is cut along the KV axis so that
    // it fills the machine; the pieces of a tile leave their states in scratch and a merge kernel combines them.
    const uint32_t group = c->cfg.num_q_heads / c->cfg.num_kv_heads;
    const uint32_t hp_count = c->cfg.num_kv_heads * ((group + 1u) / 2u);
    auto kv_tiles_of = [](const KriyaPrefillTile& t) { return (t.pos0 + t.rows + 127u) / 128u; };
    uint32_t n_merge = 0;
    uint32_t split = 1u;
    if (c->pf_split_enable && c->attention_window == 0u && c->pf_part_o != nullptr) {
        split = choose_prefill_split(tiles, n, hp_count, uint32_t(c->sm_count), c->pf_part_slots, cap_tiles);
        if (c->pf_split_force != 0u && uint64_t(n) * c->pf_split_force * hp_count <= c->pf_part_slots &&
            uint64_t(n) * (c->pf_split_force + 1u) <= cap_tiles)
            split = c->pf_split_force;
    }
    if (split > 1u) {
        std::vector<KriyaPrefillTile> whole(tiles, tiles + n);
        std::vector<KriyaPrefillMerge> merges;
        uint32_t m = 0, slot = 0;
        for (const KriyaPrefillTile& t : whole) {
            const uint32_t L = kv_tiles_of(t), parts = std::max(1u, std::min(split, L / 2u));
            if (parts == 1u) {
                tiles[m++] = t;
                continue;
            }
            merges.push_back(KriyaPrefillMerge{t.q_row0, t.rows, slot, parts});
            uint32_t t0 = 0;
            for (uint32_t pc = 0; pc < parts; ++pc) {
                const uint32_t len = L / parts + (pc < L % parts ? 1u : 0u);
                KriyaPrefillTile piece = t;
                piece.kv_t0 = t0;
                piece.kv_t1 = t0 + len;
                piece.slot = slot++;
                tiles[m++] = piece;
                t0 += len;
            }
        }
        n = m;
        n_merge = uint32_t(merges.size());
        memcpy(tiles + n, merges.data(), merges.size() * sizeof(KriyaPrefillMerge));
    }
    auto piece_len = [&](const KriyaPrefillTile& t) { return t.kv_t1 != 0u ? t.kv_t1 - t.kv_t0 : kv_tiles_of(t); };
    std::stable_sort(tiles, tiles + n, [&](const KriyaPrefillTile& x, const KriyaPrefillTile& y) { return piece_len(x) > piece_len(y); });
    KRIYA_CUDA_TRY(c, cudaMemcpyAsync(c->d_pairs, tiles, size_t(n) * sizeof(KriyaPrefillTile) + size_t(n_merge) * sizeof(KriyaPrefillMerge),
                                      cudaMemcpyHostToDevice, c->stream));
    KRIYA_CUDA_TRY(c, cudaEventRecord(c->h_pairs_free, c->stream));
    KriyaPrefillArgs a{};
    a.q = q;
    a.cache_k = c->layer_k(layer);
    a.cache_v = c->layer_v(layer);
    a.layer_row0 = uint32_t(size_t(layer) * c->layer_stride_bytes / (size_t(c->cfg.num_kv_heads) * c->cfg.head_dim * 2));
    a.table = c->plan_dev<int32_t>(c->off_indices);
    a.tiles = reinterpret_cast<const KriyaPrefillTile*>(c->d_pairs);
    a.map_k = c->tmap_k;
    a.map_v = c->tmap_v;
    a.out = out;
    a.status = c->d_status;
    a.n_tiles = n;
    a.q_rows = q_rows;
    a.num_blocks = c->cfg.num_kv_blocks;
    a.num_q_heads = c->cfg.num_q_heads;
    a.num_kv_heads = c->cfg.num_kv_heads;
    a.window = c->attention_window;
    a.sm_scale = p->sm_scale;
    a.logit_softcap = p->logit_softcap;
    if (q4) {
        // the plan's blocks of this layer, expanded to 16 bits in plan order; the kernel reads them with the identity table
        KRIYA_CUDA_TRY(c, kriya_launch_q4_expand_blocks(c->layer_k(layer), c->layer_v(layer), c->q4_stage_k, c->q4_stage_v,
                                                        c->plan_dev<int32_t>(c->off_indices), c->n_indices, c->cfg.block_size_tokens,
                                                        c->cfg.num_kv_heads, c->cfg.head_dim, c->cfg.num_kv_blocks, c->cfg.dtype,
                                                        c->d_status, c->stream));
        c->launches += 1;
        a.cache_k = c->q4_stage_k;
        a.cache_v = c->q4_stage_v;
        a.layer_row0 = 0;
        a.table = c->q4_identity;
        a.num_blocks = c->cap_indices;
    }
    a.part_o = c->pf_part_o;
    a.part_ml = c->pf_part_ml;
    a.merge_items = reinterpret_cast<const KriyaPrefillMerge*>(reinterpret_cast<const KriyaPrefillTile*>(c->d_pairs) + n);
    a.n_merge = n_merge;
    KRIYA_CUDA_TRY(c, kriya_launch_prefill(a, c->cfg.head_dim, c->cfg.block_size_tokens, c->cfg.dtype, c->max_smem_optin,
                                           c->stream));
    c->launches += n_merge ? 2 : 1;
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_paged_gqa_prefill(kriya_cuda_ctx* c, uint32_t layer, const void* q, void* out, uint32_t prefix_tokens,
                                     uint32_t num_tokens, const kriya_bsr_gqa_params* p) {
    const uint32_t zero = 0;
    return kriya_cuda_paged_gqa_prefill_batch(c, layer, q, out, 1, &zero, &prefix_tokens, &num_tokens, p);
}

int32_t kriya_cuda_kv_block_copy(kriya_cuda_ctx* c, const uint32_t* pairs, uint32_t n_pairs) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (n_pairs == 0) return KRIYA_CUDA_OK;
    if (!pairs) return c->fail(KRIYA_CUDA_INVALID_INPUT, "pairs must not be null");
    if (n_pairs > c->cap_pairs) return c->fail(KRIYA_CUDA_INVALID_INPUT, "more copy pairs than the context holds");
    for (uint32_t i = 0; i < 2 * n_pairs; ++i)
        if (pairs[i] >= c->cfg.num_kv_blocks)
            return c->fail(KRIYA_CUDA_INVALID_INPUT, "copy pair " + std::to_string(i / 2) + " names block " +
                                                         std::to_string(pairs[i]) + " outside the pool");
    cudaSetDevice(c->cfg.device);
    KRIYA_CUDA_TRY(c, cudaEventSynchronize(c->h_pairs_free));
    memcpy(c->h_pairs, pairs, size_t(n_pairs) * 2 * sizeof(uint32_t));
    KRIYA_CUDA_TRY(c, cudaMemcpyAsync(c->d_pairs, c->h_pairs, size_t(n_pairs) * 2 * sizeof(uint32_t),
                                      cudaMemcpyHostToDevice, c->stream));
    KRIYA_CUDA_TRY(c, cudaEventRecord(c->h_pairs_free, c->stream));
    // Pairs apply in order.  A launch copies its pairs concurrently, so a batch ends where a pair reads a block an earlier
    // pair of the batch wrote, or writes a block an earlier pair of the batch read or wrote.
    uint32_t start = 0;
    std::vector<uint32_t> written, read;
    for (uint32_t i = 0; i <= n_pairs; ++i) {
        bool cut = i == n_pairs;
        if (!cut) {
            const uint32_t src = pairs[2 * i], dst = pairs[2 * i + 1];
            for (uint32_t wv : written)
                if (wv == src || wv == dst) {
                    cut = true;
                    break;
                }
            for (uint32_t rv : read)
                if (rv == dst && src != dst) {
                    cut = true;
                    break;
                }
        }
        if (cut && i > start) {
            KRIYA_CUDA_TRY(c, kriya_launch_block_copy(c->pool_k, c->pool_v, c->layer_stride_bytes, c->cfg.num_layers,
                                                      c->block_bytes, c->d_pairs + 2 * size_t(start), i - start,
                                                      c->sm_count, c->stream));
            c->launches += 1;
            start = i;
            written.clear();
            read.clear();
        }
        if (i < n_pairs) {
            written.push_back(pairs[2 * i + 1]);
            read.push_back(pairs[2 * i]);
        }
    }
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_kv_slot_write(kriya_cuda_ctx* c, uint32_t layer, const void* stage_k, const void* stage_v,
                                 const uint32_t* triples, uint32_t n) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (int32_t rc = check_layer(c, layer)) return rc;
    if (n == 0) return KRIYA_CUDA_OK;
    if (!stage_k || !stage_v || !triples) return c->fail(KRIYA_CUDA_INVALID_INPUT, "staging buffers and triples must not be null");
    if (n > c->cap_pairs) return c->fail(KRIYA_CUDA_INVALID_INPUT, "more slot writes than the context holds");
    for (uint32_t i = 0; i < n; ++i)
        if (triples[3 * i + 1] >= c->cfg.num_kv_blocks || triples[3 * i + 2] >= c->cfg.block_size_tokens)
            return c->fail(KRIYA_CUDA_INVALID_INPUT, "slot write " + std::to_string(i) + " is outside the pool");
    cudaSetDevice(c->cfg.device);
    KRIYA_CUDA_TRY(c, cudaEventSynchronize(c->h_pairs_free));
    memcpy(c->h_pairs, triples, size_t(n) * 3 * sizeof(uint32_t));
    KRIYA_CUDA_TRY(c, cudaMemcpyAsync(c->d_pairs, c->h_pairs, size_t(n) * 3 * sizeof(uint32_t), cudaMemcpyHostToDevice,
                                      c->stream));
    KRIYA_CUDA_TRY(c, cudaEventRecord(c->h_pairs_free, c->stream));
    KRIYA_CUDA_TRY(c, kriya_launch_slot_write(c->layer_k(layer), c->layer_v(layer), stage_k, stage_v,
                                              c->block_bytes / c->cfg.block_size_tokens, c->cfg.block_size_tokens,
                                              c->d_pairs, n, c->cfg.num_kv_blocks, c->d_status, c->stream));
    c->launches += 1;
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_decode_layer_host(kriya_cuda_ctx* c, uint32_t layer, const void* q_host, const void* k_host,
                                     const void* v_host, void* out_host, uint32_t rows,
                                     const kriya_rope_kv_write_params* rope, const kriya_bsr_gqa_params* gqa) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (!q_host || !k_host || !v_host || !out_host) return c->fail(KRIYA_CUDA_INVALID_INPUT, "host buffers must not be null");
    if (!c->plan_valid) return c->fail(KRIYA_CUDA_INVALID_INPUT, "no plan uploaded");
    if (rows == 0 || rows != c->n_rows) return c->fail(KRIYA_CUDA_INVALID_INPUT, "rows must equal the plan's row count");
    cudaSetDevice(c->cfg.device);
    const size_t qb = size_t(rows) * c->cfg.num_q_heads * c->cfg.head_dim * 2;
    const size_t kb = size_t(rows) * c->cfg.num_kv_heads * c->cfg.head_dim * 2;
    uint8_t* dq = c->d_act;
    uint8_t* dk = dq + qb;
    uint8_t* dv = dk + kb;
    uint8_t* dout = dv + kb;
    KRIYA_CUDA_TRY(c, cudaMemcpyAsync(dq, q_host, qb, cudaMemcpyHostToDevice, c->stream));
    KRIYA_CUDA_TRY(c, cudaMemcpyAsync(dk, k_host, kb, cudaMemcpyHostToDevice, c->stream));
    KRIYA_CUDA_TRY(c, cudaMemcpyAsync(dv, v_host, kb, cudaMemcpyHostToDevice, c->stream));
    if (int32_t rc = kriya_cuda_rope_kv_append(c, layer, dq, dk, dv, nullptr, nullptr, rows, rope)) return rc;
    if (int32_t rc = kriya_cuda_paged_gqa_decode(c, layer, dq, dout, gqa)) return rc;
    KRIYA_CUDA_TRY(c, cudaMemcpyAsync(out_host, dout, qb, cudaMemcpyDeviceToHost, c->stream));
    return kriya_cuda_sync(c, 0);
}

static int32_t append_decode_impl(kriya_cuda_ctx* c, uint32_t layer, const void* q, const void* k, const void* v, void* out,
                                  void* q_rope_out, const kriya_rope_kv_write_params* rope, const kriya_bsr_gqa_params* gqa,
                                  uint32_t overlap_previous) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (int32_t rc = check_layer(c, layer)) return rc;
    if (int32_t rc = check_rope(c, rope)) return rc;
    if (int32_t rc = check_gqa(c, gqa)) return rc;
    if (!c->plan_valid) return c->fail(KRIYA_CUDA_INVALID_INPUT, "no plan uploaded");
    if (!q || !k || !v || !out) return c->fail(KRIYA_CUDA_INVALID_INPUT, "q, k, v and out must not be null");
    if (q_rope_out == q) return c->fail(KRIYA_CUDA_INVALID_INPUT, "q_rope_out must not alias q");
    if (c->n_positions != c->n_rows)
        return c->fail(KRIYA_CUDA_INVALID_INPUT, "input_tokens has " + std::to_string(c->n_rows) + " entries but seq_positions has " +
                                                     std::to_string(c->n_positions));
    if (rope->apply_qk_norm || !use_tc_decode(c))
        return c->fail(KRIYA_CUDA_UNSUPPORTED, "the fused append + decode launch covers head_dim 128, group size 1..8, no QK norm");
    cudaSetDevice(c->cfg.device);
    KriyaFusedAppend f;
    f.k_in = k;
    f.v_in = v;
    f.q_rope_out = q_rope_out;
    f.positions = c->plan_dev<uint32_t>(c->off_positions);
    f.table = table_for(c, rope);
    f.cache_k_w = c->layer_k(layer);
    f.cache_v_w = c->layer_v(layer);
    f.rotary_dim = rope->rotary_dim;
    f.max_seq_len = rope->max_seq_len;
    f.has_table = rope->has_table;
    f.rope_theta = rope->rope_theta;
    f.positions_are_context = c->positions_are_context ? 1u : 0u;
    // how the launch relates to the kernel before it (KriyaFusedAppend::overlap_previous); event brackets forbid any overlap
    f.overlap_previous = c->timing ? 0u : overlap_previous;
    return launch_decode(c, layer, q, out, nullptr, nullptr, nullptr, false, c->n_work, gqa, f);
}

int32_t kriya_cuda_append_decode(kriya_cuda_ctx* c, uint32_t layer, const void* q, const void* k, const void* v, void* out,
                                 void* q_rope_out, const kriya_rope_kv_write_params* rope, const kriya_bsr_gqa_params* gqa) {
    return append_decode_impl(c, layer, q, k, v, out, q_rope_out, rope, gqa, 0u);
}

// Layers [l0, l1) of one step; `first_of_chain` says that the launch for l0 must not overlap what precedes it.
static int32_t decode_layers(kriya_cuda_ctx* c, uint32_t l0, uint32_t l1, bool first_of_chain, void* q, const void* k,
                             const void* v, void* out, uint32_t rows, const kriya_rope_kv_write_params* rope,
                             const kriya_bsr_gqa_params* gqa) {
    const size_t qb = size_t(rows) * c->cfg.num_q_heads * c->cfg.head_dim * 2;
    const size_t kb = size_t(rows) * c->cfg.num_kv_heads * c->cfg.head_dim * 2;
    // launches that are declared independent overlap: they take the work list with the longer streams (see chain_list_valid)
    struct ChainScope {
        kriya_cuda_ctx* c;
        ~ChainScope() { c->use_chain_list = false; }
    } chain_scope{c};
    c->use_chain_list = c->layer_chain_mode == 2u && !c->timing && c->fuse_append && use_tc_decode(c) && !rope->apply_qk_norm;
    for (uint32_t layer = l0; layer < l1; ++layer) {
        uint8_t* ql = static_cast<uint8_t*>(q) + layer * qb;
        const uint8_t* kl = static_cast<const uint8_t*>(k) + layer * kb;
        const uint8_t* vl = static_cast<const uint8_t*>(v) + layer * kb;
        uint8_t* ol = static_cast<uint8_t*>(out) + layer * qb;
        if (c->fuse_append && use_tc_decode(c) && !rope->apply_qk_norm) {
            // Layers of one step share nothing but the split-run scratch, which the kernel guards itself: from the
            // second layer on, a launch may start while the previous layer's last CTAs drain (by default).
            const uint32_t mode = (first_of_chain && layer == l0) ? 0u : c->layer_chain_mode;
            if (int32_t rc = append_decode_impl(c, layer, ql, kl, vl, ol, nullptr, rope, gqa, mode)) return rc;
        } else {
            if (int32_t rc = kriya_cuda_rope_kv_append(c, layer, ql, kl, vl, nullptr, nullptr, rows, rope)) return rc;
            if (int32_t rc = kriya_cuda_paged_gqa_decode(c, layer, ql, ol, gqa)) return rc;
        }
    }
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_decode_step(kriya_cuda_ctx* c, void* q, const void* k, const void* v, void* out, uint32_t rows,
                               const kriya_rope_kv_write_params* rope, const kriya_bsr_gqa_params* gqa) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (!q || !k || !v || !out) return c->fail(KRIYA_CUDA_INVALID_INPUT, "q, k, v and out must not be null");
    if (!c->plan_valid) return c->fail(KRIYA_CUDA_INVALID_INPUT, "no plan uploaded");
    if (rows == 0 || rows != c->n_rows) return c->fail(KRIYA_CUDA_INVALID_INPUT, "rows must equal the plan's row count");
    cudaSetDevice(c->cfg.device);
    return decode_layers(c, 0, c->cfg.num_layers, true, q, k, v, out, rows, rope, gqa);
}

int32_t kriya_cuda_decode_step_host_begin(kriya_cuda_ctx* c, const void* q_host, const void* k_host, const void* v_host,
                                          void* out_host, uint32_t rows, const kriya_rope_kv_write_params* rope,
                                          const kriya_bsr_gqa_params* gqa) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (!q_host || !k_host || !v_host || !out_host) return c->fail(KRIYA_CUDA_INVALID_INPUT, "host buffers must not be null");
    if (!c->plan_valid) return c->fail(KRIYA_CUDA_INVALID_INPUT, "no plan uploaded");
    if (rows == 0 || rows != c->n_rows) return c->fail(KRIYA_CUDA_INVALID_INPUT, "rows must equal the plan's row count");
    cudaSetDevice(c->cfg.device);
    const size_t L = c->cfg.num_layers;
    const size_t qb = size_t(rows) * c->cfg.num_q_heads * c->cfg.head_dim * 2 * L;
    const size_t kb = size_t(rows) * c->cfg.num_kv_heads * c->cfg.head_dim * 2 * L;
    const size_t need = 2 * qb + 2 * kb;
    if (need > c->step_bytes)  // the staging is sized for max_batch_rows when the context is created
        return c->fail(KRIYA_CUDA_INVALID_INPUT, "step of " + std::to_string(rows) + " rows exceeds the context's staging");
    uint8_t* dq = c->d_step;
    uint8_t* dk = dq + qb;
    uint8_t* dv = dk + kb;
    uint8_t* dout = dv + kb;
    // Three-way pipeline: inputs travel host->device on one copy stream and results travel back on another while the
    // layers compute.  A layer's inputs cross PCIe several times faster than the layer computes, so the input groups
    // grow (1, 3, 9, rest: only the first layer's copy is exposed) and the output groups shrink (rest, 9, 3, 1: only the
    // last layer's copy is exposed).  Every group boundary is an event between two launches, which costs the overlap
    // of those two layers, hence few groups.
    const uint32_t Lu = uint32_t(L);
    const size_t qbl = qb / L, kbl = kb / L;
    uint32_t in_start[5], out_end[5], n_in = 0, n_out = 0;
    for (uint32_t b : {0u, 1u, 4u, 13u})
        if (b < Lu && (n_in == 0 || b > in_start[n_in - 1])) in_start[n_in++] = b;
    in_start[n_in] = Lu;
    for (uint32_t back : {13u, 4u, 1u, 0u}) {
        const uint32_t e = Lu - std::min(back, Lu);
        if (e > 0 && (n_out == 0 || e > out_end[n_out - 1])) out_end[n_out++] = e;
    }
    KRIYA_CUDA_TRY(c, cudaEventRecord(c->ev_step_begin, c->stream));  // the plan upload and earlier work come first
    KRIYA_CUDA_TRY(c, cudaStreamWaitEvent(c->copy_stream, c->ev_step_begin, 0));
    KRIYA_CUDA_TRY(c, cudaStreamWaitEvent(c->copy_stream_out, c->ev_step_begin, 0));
    // The first group's copies are queued, then its launches, then the next group's copies and so on: a group's copies go
    // out as soon as the launches of the group in front of it have been issued (they run under that group's compute),
    // so the first launch is not held up by the host queuing a dozen copies.
    auto queue_in = [&](uint32_t g) -> cudaError_t {
        const uint32_t l0 = in_start[g], l1 = in_start[g + 1];
        const size_t nq = size_t(l1 - l0) * qbl, nk = size_t(l1 - l0) * kbl;
        cudaError_t e = cudaMemcpyAsync(dq + l0 * qbl, static_cast<const uint8_t*>(q_host) + l0 * qbl, nq, cudaMemcpyHostToDevice, c->copy_stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(dk + l0 * kbl, static_cast<const uint8_t*>(k_host) + l0 * kbl, nk, cudaMemcpyHostToDevice, c->copy_stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(dv + l0 * kbl, static_cast<const uint8_t*>(v_host) + l0 * kbl, nk, cudaMemcpyHostToDevice, c->copy_stream);
        if (e == cudaSuccess) e = cudaEventRecord(c->ev_in[g], c->copy_stream);
        return e;
    };
    KRIYA_CUDA_TRY(c, queue_in(0));
    uint32_t gi = 0, go = 0, layer = 0, out_from = 0, queued = 1;
    while (layer < Lu) {
        const bool group_start = gi < n_in && in_start[gi] == layer;
        if (group_start) KRIYA_CUDA_TRY(c, cudaStreamWaitEvent(c->stream, c->ev_in[gi++], 0));
        uint32_t stop = out_end[go];                                  // next boundary of either kind
        if (gi < n_in && in_start[gi] < stop) stop = in_start[gi];
        if (int32_t rc = decode_layers(c, layer, stop, true, dq, dk, dv, dout, rows, rope, gqa)) return rc;
        if (group_start && queued < n_in) KRIYA_CUDA_TRY(c, queue_in(queued++));
        layer = stop;
        if (layer == out_end[go]) {
            KRIYA_CUDA_TRY(c, cudaEventRecord(c->ev_done[go], c->stream));
            KRIYA_CUDA_TRY(c, cudaStreamWaitEvent(c->copy_stream_out, c->ev_done[go], 0));
            KRIYA_CUDA_TRY(c, cudaMemcpyAsync(static_cast<uint8_t*>(out_host) + out_from * qbl, dout + out_from * qbl,
                                              size_t(layer - out_from) * qbl, cudaMemcpyDeviceToHost, c->copy_stream_out));
            out_from = layer;
            ++go;
        }
    }
    KRIYA_CUDA_TRY(c, cudaEventRecord(c->ev_step_end, c->copy_stream_out));
    KRIYA_CUDA_TRY(c, cudaStreamWaitEvent(c->stream, c->ev_step_end, 0));  // later work on the context's stream follows the step
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_decode_step_host_end(kriya_cuda_ctx* c, uint32_t timeout_ms) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    return kriya_cuda_sync(c, timeout_ms);  // the context's stream waits for the last copy back: one wait covers the step
}

int32_t kriya_cuda_decode_step_host(kriya_cuda_ctx* c, const void* q_host, const void* k_host, const void* v_host,
                                    void* out_host, uint32_t rows, const kriya_rope_kv_write_params* rope,
                                    const kriya_bsr_gqa_params* gqa) {
    if (int32_t rc = kriya_cuda_decode_step_host_begin(c, q_host, k_host, v_host, out_host, rows, rope, gqa)) return rc;
    return kriya_cuda_decode_step_host_end(c, 0);
}

int32_t kriya_cuda_set_decode_path(kriya_cuda_ctx* c, int32_t path) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (path < 0 || path > 3)
        return c->fail(KRIYA_CUDA_INVALID_INPUT, "decode path must be 0 (auto), 1 (CUDA-core), 2 (tensor-core) or 3 (tensor-core, one KV head per copy)");
    if (path >= 2 && !(c->tmaps_ok && kriya_decode_tc_supported(c->cfg.head_dim, c->cfg.num_q_heads / c->cfg.num_kv_heads,
                                                                 c->cfg.block_size_tokens)))
        return c->fail(KRIYA_CUDA_UNSUPPORTED, "the tensor-core decode kernel covers head_dim 128, group size 1..8, 16-token blocks");
    c->decode_path = path;
    c->plan_valid = false;  // the work lists of an uploaded plan were cut for the kernel chosen before
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_set_wait_limit_us(kriya_cuda_ctx* c, uint32_t limit_us) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (limit_us == 0) return c->fail(KRIYA_CUDA_INVALID_INPUT, "the wait limit must be positive");
    c->wait_ns = uint64_t(limit_us) * 1000ull;
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_selftest_wait_expiry(kriya_cuda_ctx* c) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    cudaSetDevice(c->cfg.device);
    KRIYA_CUDA_TRY(c, kriya_launch_wait_selftest(c->d_status, c->wait_ns, c->stream));
    c->launches += 1;
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_set_attention_window(kriya_cuda_ctx* c, uint32_t window_size) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    c->attention_window = window_size;
    c->plan_valid = false;  // the work lists of an uploaded plan were cut for the mask set before
    return KRIYA_CUDA_OK;
}

int64_t kriya_cuda_debug_work_split(const int32_t* page_indptr, const int32_t* last_page_len, uint32_t rows,
                                    uint32_t block_size_tokens, uint32_t runs_per_row, uint32_t ctas, uint32_t pages_per_tile,
                                    uint32_t min_tiles, uint32_t window, uint32_t* out_records, uint32_t cap,
                                    uint32_t* out_cta_offsets) {
    if (!page_indptr || !last_page_len || !out_records || !out_cta_offsets || block_size_tokens == 0 || runs_per_row == 0 ||
        ctas == 0 || pages_per_tile == 0 || min_tiles == 0)
        return -1;
    static_assert(sizeof(KriyaTcSeg) == 12 * sizeof(uint32_t), "a record is twelve words");
    const uint32_t n = build_tc_segments(page_indptr, last_page_len, block_size_tokens, rows, runs_per_row, nullptr, nullptr, ctas,
                                         pages_per_tile, reinterpret_cast<KriyaTcSeg*>(out_records), cap, out_cta_offsets, min_tiles, window);
    return n == UINT32_MAX ? -1 : int64_t(n);
}

int32_t kriya_cuda_set_fused_append(kriya_cuda_ctx* c, int32_t enable) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    c->fuse_append = (enable & 1) != 0;
    static const uint32_t modes[4] = {2u, 1u, 3u, 0u};  // bits 1-2: free, serialised, dependent activations, ordinary launches
    c->layer_chain_mode = modes[(enable >> 1) & 3];
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_timing_enable(kriya_cuda_ctx* c, int32_t enable) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    cudaSetDevice(c->cfg.device);
    KRIYA_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    timing_collect(c);
    c->timing = enable != 0;
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_timing_read(kriya_cuda_ctx* c, uint32_t kind, uint64_t* out_launches, double* out_total_ms) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (kind > 1) return c->fail(KRIYA_CUDA_INVALID_INPUT, "timing kind must be 0 (decode) or 1 (append)");
    cudaSetDevice(c->cfg.device);
    KRIYA_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    timing_collect(c);
    if (out_launches) *out_launches = c->t_launches[kind];
    if (out_total_ms) *out_total_ms = c->t_ms[kind];
    c->t_launches[kind] = 0;
    c->t_ms[kind] = 0.0;
    return KRIYA_CUDA_OK;
}

}  // extern "C"
