// Host-side paged KV bookkeeping: block allocator, radix prefix cache, copy-on-write and the
// BSR plan builders, behind the C ABI of include/kriya_kv.h.
//
// Behaviour mirrors crates/kriya-kv/src/bsr_paged.rs exactly where it is observable: which
// block id an allocation returns (FIFO reuse), refcounts, generation counters, the
// allocate-then-free order of a copy-on-write, radix matching rules and every plan array.
// The data structures are this library's own: a ring-buffer free list over flat arrays,
// radix nodes in an arena with a single (parent, first token) -> child index map, and plan
// storage that is reused between calls so that the per-step path does not allocate once the
// vectors have grown to their working size.
#include "kriya_kv.h"

#include <algorithm>
#include <cstring>
#include <unordered_map>
#include <vector>

namespace {

struct RadixNode {
    size_t tok_off = 0;        // offset of this node's block_size tokens inside token_pool
    uint32_t phys = 0;         // physical block id holding these tokens' KV
    uint64_t generation = 0;   // generation of `phys` when the node was (re)bound
};

struct SeqTable {
    std::vector<uint32_t> blocks;
    uint32_t total_tokens = 0;
};

struct PlanStorage {
    std::vector<int32_t> indptr, indices, last_len;
    std::vector<kriya_cta_work_tile> tiles;
    uint32_t max_blocks_per_cta = 1;
    void clear() {
        indptr.clear();
        indices.clear();
        last_len.clear();
        tiles.clear();
    }
};

inline uint32_t div_ceil(uint32_t a, uint32_t b) { return (a + b - 1u) / b; }

}  // namespace

struct kriya_kv_manager {
    uint32_t block_size = 16;
    // allocator (bsr_paged.rs:41-153)
    std::vector<uint32_t> ref_count;
    std::vector<uint64_t> generation;
    std::vector<uint32_t> ring;  // FIFO free list: pop at head, push at (head+count)%cap
    size_t ring_head = 0, ring_count = 0;
    // radix cache (bsr_paged.rs:155-253); node 0 is the root
    std::vector<RadixNode> nodes;
    std::vector<uint32_t> token_pool;
    std::unordered_map<uint64_t, uint32_t> child_of;  // (parent index << 32 | first token) -> node index
    // sequences
    std::unordered_map<uint64_t, SeqTable> sequences;
    PlanStorage plan;
    std::vector<uint32_t> scratch_blocks;
    kriya_kv_error_info err{};

    int32_t fail(int32_t code, uint64_t id, uint64_t requested = 0, uint64_t available = 0) {
        err.code = code;
        err.id = id;
        err.requested = requested;
        err.available = available;
        return code;
    }

    size_t num_free() const { return ring_count; }

    // allocate_block, bsr_paged.rs:85-101
    int32_t allocate_block(uint32_t* out) {
        if (ring_count == 0) return fail(KRIYA_KV_OUT_OF_BLOCKS, 0, 1, 0);
        const uint32_t id = ring[ring_head];
        ring_head = (ring_head + 1) % ring.size();
        --ring_count;
        ref_count[id] = 1;
        generation[id] += 1;
        *out = id;
        return KRIYA_KV_OK;
    }

    // free_block, bsr_paged.rs:124-143
    int32_t free_block(uint32_t id, bool* returned) {
        if (id >= ref_count.size() || ref_count[id] == 0) return fail(KRIYA_KV_INVALID_BLOCK_ID, id);
        const bool last = --ref_count[id] == 0;
        if (last) {
            ring[(ring_head + ring_count) % ring.size()] = id;
            ++ring_count;
        }
        if (returned) *returned = last;
        return KRIYA_KV_OK;
    }

    static uint64_t child_key(uint32_t parent, uint32_t first_tok) { return (uint64_t(parent) << 32) | first_tok; }

    bool node_tokens_equal(const RadixNode& n, const uint32_t* chunk) const {
        return std::memcmp(token_pool.data() + n.tok_off, chunk, size_t(block_size) * 4) == 0;
    }

    // match_prefix, bsr_paged.rs:185-215
    size_t match_prefix(const uint32_t* tokens, size_t len, std::vector<uint32_t>& matched) {
        const size_t bs = block_size;
        uint32_t current = 0;
        size_t offset = 0;
        while (offset + bs <= len) {
            const uint32_t* chunk = tokens + offset;
            auto it = child_of.find(child_key(current, chunk[0]));
            if (it == child_of.end()) break;
            const RadixNode& child = nodes[it->second];
            if (!node_tokens_equal(child, chunk)) break;
            const uint32_t phys = child.phys;
            const uint64_t gen = phys < generation.size() ? generation[phys] : 0;
            const uint32_t rc = phys < ref_count.size() ? ref_count[phys] : 0;
            if (gen != child.generation || rc == 0) break;
            ref_count[phys] += 1;
            matched.push_back(phys);
            current = it->second;
            offset += bs;
        }
        return offset;
    }

    // insert_prefix, bsr_paged.rs:218-252
    void insert_prefix(const uint32_t* tokens, size_t len, const std::vector<uint32_t>& phys_blocks) {
        const size_t bs = block_size;
        const size_t full = std::min(len / bs, phys_blocks.size());
        uint32_t current = 0;
        for (size_t i = 0; i < full; ++i) {
            const uint32_t* chunk = tokens + i * bs;
            const uint32_t phys = phys_blocks[i];
            const uint64_t gen = phys < generation.size() ? generation[phys] : 0;
            const uint64_t key = child_key(current, chunk[0]);
            auto it = child_of.find(key);
            uint32_t idx;
            if (it == child_of.end()) {
                RadixNode n;
                n.tok_off = token_pool.size();
                token_pool.insert(token_pool.end(), chunk, chunk + bs);
                n.phys = phys;
                n.generation = gen;
                idx = uint32_t(nodes.size());
                nodes.push_back(n);
                child_of.emplace(key, idx);
            } else {
                idx = it->second;
            }
            RadixNode& node = nodes[idx];
            if (!node_tokens_equal(node, chunk)) break;  // another chunk owns this first token: stop
            node.phys = phys;
            node.generation = gen;
            current = idx;
        }
    }

    void fill_view(kriya_kv_plan_view* out) const {
        out->page_indptr = plan.indptr.data();
        out->page_indptr_len = plan.indptr.size();
        out->page_indices = plan.indices.data();
        out->page_indices_len = plan.indices.size();
        out->last_page_len = plan.last_len.data();
        out->last_page_len_len = plan.last_len.size();
        out->cta_work_tiles = plan.tiles.data();
        out->cta_work_tiles_len = plan.tiles.size();
        out->max_blocks_per_cta = plan.max_blocks_per_cta;
    }

    uint32_t last_page_len(const SeqTable& s) const {  // bsr_paged.rs:266-271
        const uint32_t rem = s.total_tokens % block_size;
        return (rem == 0 && s.total_tokens > 0) ? block_size : rem;
    }
};

extern "C" {

kriya_kv_manager* kriya_kv_create(uint32_t num_gpu_blocks, uint32_t /*num_cpu_swap_blocks*/, uint32_t block_size) {
    if (block_size == 0) return nullptr;
    auto* m = new kriya_kv_manager();
    m->block_size = block_size;
    m->ref_count.assign(num_gpu_blocks, 0);
    m->generation.assign(num_gpu_blocks, 0);
    m->ring.resize(std::max<uint32_t>(num_gpu_blocks, 1));
    for (uint32_t i = 0; i < num_gpu_blocks; ++i) m->ring[i] = i;
    m->ring_count = num_gpu_blocks;
    m->nodes.emplace_back();  // root
    return m;
}

void kriya_kv_destroy(kriya_kv_manager* m) { delete m; }

void kriya_kv_last_error(const kriya_kv_manager* m, kriya_kv_error_info* out) {
    if (m && out) *out = m->err;
}

size_t kriya_kv_num_free_blocks(const kriya_kv_manager* m) { return m ? m->num_free() : 0; }
size_t kriya_kv_total_blocks(const kriya_kv_manager* m) { return m ? m->ref_count.size() : 0; }
uint32_t kriya_kv_block_size_tokens(const kriya_kv_manager* m) { return m ? m->block_size : 0; }

int32_t kriya_kv_ref_count(kriya_kv_manager* m, uint32_t block_id, uint32_t* out) {
    if (!m || !out) return KRIYA_KV_BAD_ARGUMENT;
    if (block_id >= m->ref_count.size()) return m->fail(KRIYA_KV_INVALID_BLOCK_ID, block_id);
    *out = m->ref_count[block_id];
    return KRIYA_KV_OK;
}

int32_t kriya_kv_generation(kriya_kv_manager* m, uint32_t block_id, uint64_t* out) {
    if (!m || !out) return KRIYA_KV_BAD_ARGUMENT;
    if (block_id >= m->generation.size()) return m->fail(KRIYA_KV_INVALID_BLOCK_ID, block_id);
    *out = m->generation[block_id];
    return KRIYA_KV_OK;
}

int32_t kriya_kv_allocate_block(kriya_kv_manager* m, uint32_t* out_block) {
    if (!m || !out_block) return KRIYA_KV_BAD_ARGUMENT;
    return m->allocate_block(out_block);
}

int32_t kriya_kv_inc_ref(kriya_kv_manager* m, uint32_t block_id) {
    if (!m) return KRIYA_KV_BAD_ARGUMENT;
    if (block_id >= m->ref_count.size()) return m->fail(KRIYA_KV_INVALID_BLOCK_ID, block_id);
    m->ref_count[block_id] += 1;  // bsr_paged.rs:114-121 (no liveness check there either)
    return KRIYA_KV_OK;
}

int32_t kriya_kv_free_block(kriya_kv_manager* m, uint32_t block_id, int32_t* out_returned_to_pool) {
    if (!m) return KRIYA_KV_BAD_ARGUMENT;
    bool returned = false;
    const int32_t rc = m->free_block(block_id, &returned);
    if (rc == KRIYA_KV_OK && out_returned_to_pool) *out_returned_to_pool = returned ? 1 : 0;
    return rc;
}

int32_t kriya_kv_allocate_sequence(kriya_kv_manager* m, uint64_t seq_id, const uint32_t* prompt_tokens, size_t len,
                                   size_t* out_matched_tokens) {
    if (!m || (!prompt_tokens && len > 0)) return KRIYA_KV_BAD_ARGUMENT;
    std::vector<uint32_t> blocks;
    const size_t matched = m->match_prefix(prompt_tokens, len, blocks);
    const size_t needed = (len + m->block_size - 1) / m->block_size;
    const size_t additional = needed > blocks.size() ? needed - blocks.size() : 0;
    if (m->num_free() < additional) {
        for (uint32_t b : blocks) m->free_block(b, nullptr);  // roll back the prefix refcounts, bsr_paged.rs:355-359
        return m->fail(KRIYA_KV_OUT_OF_BLOCKS, seq_id, additional, m->num_free());
    }
    for (size_t i = 0; i < additional; ++i) {
        uint32_t id = 0;
        const int32_t rc = m->allocate_block(&id);
        if (rc != KRIYA_KV_OK) return rc;
        blocks.push_back(id);
    }
    m->insert_prefix(prompt_tokens, len, blocks);
    SeqTable& t = m->sequences[seq_id];  // insert or replace, like HashMap::insert
    t.blocks = std::move(blocks);
    t.total_tokens = uint32_t(len);
    if (out_matched_tokens) *out_matched_tokens = matched;
    return KRIYA_KV_OK;
}

int32_t kriya_kv_append_token_slots(kriya_kv_manager* m, const uint64_t* seq_ids, size_t n, uint32_t* out_blocks,
                                    uint32_t* out_cow_pairs, size_t* out_n_cow, size_t* out_done) {
    if (!m || (n && (!seq_ids || !out_blocks || !out_cow_pairs)) || !out_n_cow || !out_done) return KRIYA_KV_BAD_ARGUMENT;
    *out_n_cow = 0;
    *out_done = 0;
    for (size_t i = 0; i < n; ++i) {
        int32_t has = 0;
        uint32_t src = 0, dst = 0;
        const int32_t rc = kriya_kv_append_token_slot(m, seq_ids[i], &out_blocks[i], &has, &src, &dst);
        if (rc != KRIYA_KV_OK) return rc;
        if (has) {
            out_cow_pairs[2 * *out_n_cow] = src;
            out_cow_pairs[2 * *out_n_cow + 1] = dst;
            *out_n_cow += 1;
        }
        *out_done = i + 1;
    }
    return KRIYA_KV_OK;
}

int32_t kriya_kv_append_token_slot(kriya_kv_manager* m, uint64_t seq_id, uint32_t* out_block, int32_t* out_has_cow,
                                   uint32_t* out_cow_src, uint32_t* out_cow_dst) {
    if (!m || !out_block || !out_has_cow) return KRIYA_KV_BAD_ARGUMENT;
    auto it = m->sequences.find(seq_id);
    if (it == m->sequences.end()) return m->fail(KRIYA_KV_INVALID_SEQUENCE_ID, seq_id);
    SeqTable& seq = it->second;
    *out_has_cow = 0;
    if (seq.total_tokens % m->block_size == 0) {  // tail full (or empty sequence): fresh block
        uint32_t id = 0;
        const int32_t rc = m->allocate_block(&id);
        if (rc != KRIYA_KV_OK) return rc;
        seq.blocks.push_back(id);
        seq.total_tokens += 1;
        *out_block = id;
        return KRIYA_KV_OK;
    }
    if (seq.blocks.empty()) return m->fail(KRIYA_KV_INVALID_SEQUENCE_ID, seq_id);
    const uint32_t tail = seq.blocks.back();
    if (tail >= m->ref_count.size()) return m->fail(KRIYA_KV_INVALID_BLOCK_ID, tail);
    if (m->ref_count[tail] > 1) {
        uint32_t fresh = 0;
        int32_t rc = m->allocate_block(&fresh);  // allocate first ...
        if (rc != KRIYA_KV_OK) return rc;
        rc = m->free_block(tail, nullptr);       // ... then release the shared tail (bsr_paged.rs:413-414)
        if (rc != KRIYA_KV_OK) return rc;
        seq.blocks.back() = fresh;
        seq.total_tokens += 1;
        *out_block = fresh;
        *out_has_cow = 1;
        if (out_cow_src) *out_cow_src = tail;
        if (out_cow_dst) *out_cow_dst = fresh;
        return KRIYA_KV_OK;
    }
    seq.total_tokens += 1;
    *out_block = tail;
    return KRIYA_KV_OK;
}

int32_t kriya_kv_fork_sequence(kriya_kv_manager* m, uint64_t parent_seq_id, uint64_t child_seq_id) {
    if (!m) return KRIYA_KV_BAD_ARGUMENT;
    auto it = m->sequences.find(parent_seq_id);
    if (it == m->sequences.end()) return m->fail(KRIYA_KV_INVALID_SEQUENCE_ID, parent_seq_id);
    SeqTable copy = it->second;
    for (uint32_t b : copy.blocks) {
        if (b >= m->ref_count.size()) return m->fail(KRIYA_KV_INVALID_BLOCK_ID, b);
        m->ref_count[b] += 1;
    }
    m->sequences[child_seq_id] = std::move(copy);
    return KRIYA_KV_OK;
}

int32_t kriya_kv_free_sequence(kriya_kv_manager* m, uint64_t seq_id) {
    if (!m) return KRIYA_KV_BAD_ARGUMENT;
    auto it = m->sequences.find(seq_id);
    if (it == m->sequences.end()) return m->fail(KRIYA_KV_INVALID_SEQUENCE_ID, seq_id);
    SeqTable seq = std::move(it->second);
    m->sequences.erase(it);  // removed before the blocks are released, like HashMap::remove (bsr_paged.rs:458-461)
    for (uint32_t b : seq.blocks) {
        const int32_t rc = m->free_block(b, nullptr);
        if (rc != KRIYA_KV_OK) return rc;
    }
    return KRIYA_KV_OK;
}

int32_t kriya_kv_contains_sequence(const kriya_kv_manager* m, uint64_t seq_id) {
    return (m && m->sequences.count(seq_id)) ? 1 : 0;
}

int32_t kriya_kv_block_for_position(kriya_kv_manager* m, uint64_t seq_id, uint32_t position, uint32_t* out_block,
                                    uint32_t* out_slot) {
    if (!m || !out_block || !out_slot) return KRIYA_KV_BAD_ARGUMENT;
    auto it = m->sequences.find(seq_id);
    if (it == m->sequences.end()) return m->fail(KRIYA_KV_INVALID_SEQUENCE_ID, seq_id);
    const size_t idx = position / m->block_size;
    if (idx >= it->second.blocks.size()) return m->fail(KRIYA_KV_INVALID_SEQUENCE_ID, seq_id);
    *out_block = it->second.blocks[idx];
    *out_slot = position % m->block_size;
    return KRIYA_KV_OK;
}

int32_t kriya_kv_sequence_table(kriya_kv_manager* m, uint64_t seq_id, const uint32_t** out_blocks, size_t* out_len,
                                uint32_t* out_total_tokens) {
    if (!m) return KRIYA_KV_BAD_ARGUMENT;
    auto it = m->sequences.find(seq_id);
    if (it == m->sequences.end()) return m->fail(KRIYA_KV_INVALID_SEQUENCE_ID, seq_id);
    if (out_blocks) *out_blocks = it->second.blocks.data();
    if (out_len) *out_len = it->second.blocks.size();
    if (out_total_tokens) *out_total_tokens = it->second.total_tokens;
    return KRIYA_KV_OK;
}

int32_t kriya_kv_build_schedule_plan(kriya_kv_manager* m, const uint64_t* active_seq_ids, size_t n,
                                     uint32_t max_blocks_per_cta, kriya_kv_plan_view* out) {
    if (!m || !out || (!active_seq_ids && n > 0)) return KRIYA_KV_BAD_ARGUMENT;
    const uint32_t cap = std::max(max_blocks_per_cta, 1u);
    PlanStorage& p = m->plan;
    p.clear();
    p.max_blocks_per_cta = cap;
    p.indptr.push_back(0);
    for (size_t r = 0; r < n; ++r) {
        auto it = m->sequences.find(active_seq_ids[r]);
        if (it == m->sequences.end()) return m->fail(KRIYA_KV_INVALID_SEQUENCE_ID, active_seq_ids[r]);
        const SeqTable& s = it->second;
        for (uint32_t b : s.blocks) p.indices.push_back(int32_t(b));
        p.indptr.push_back(int32_t(p.indices.size()));
        p.last_len.push_back(int32_t(m->last_page_len(s)));
        const uint32_t nb = uint32_t(s.blocks.size());
        const uint32_t split = nb > cap ? 1u : 0u;
        for (uint32_t start = 0; start < nb; start += cap)
            p.tiles.push_back({uint32_t(r), start, std::min(nb - start, cap), split});
    }
    m->fill_view(out);
    return KRIYA_KV_OK;
}

int32_t kriya_kv_build_prefix_schedule_plan(kriya_kv_manager* m, uint64_t seq_id, uint32_t prefix_tokens,
                                            uint32_t max_blocks_per_cta, kriya_kv_plan_view* out) {
    if (!m || !out) return KRIYA_KV_BAD_ARGUMENT;
    auto it = m->sequences.find(seq_id);
    if (it == m->sequences.end()) return m->fail(KRIYA_KV_INVALID_SEQUENCE_ID, seq_id);
    const SeqTable& s = it->second;
    if (prefix_tokens == 0 || prefix_tokens > s.total_tokens) return m->fail(KRIYA_KV_INVALID_SEQUENCE_ID, seq_id);
    const uint32_t nb = div_ceil(prefix_tokens, m->block_size);
    if (nb > s.blocks.size()) return m->fail(KRIYA_KV_INVALID_SEQUENCE_ID, seq_id);
    const uint32_t cap = std::max(max_blocks_per_cta, 1u);
    PlanStorage& p = m->plan;
    p.clear();
    p.max_blocks_per_cta = cap;
    p.indptr = {0, int32_t(nb)};
    for (uint32_t i = 0; i < nb; ++i) p.indices.push_back(int32_t(s.blocks[i]));
    const uint32_t rem = prefix_tokens % m->block_size;
    p.last_len.push_back(int32_t(rem == 0 ? m->block_size : rem));
    const uint32_t split = nb > cap ? 1u : 0u;
    for (uint32_t start = 0; start < nb; start += cap) p.tiles.push_back({0u, start, std::min(nb - start, cap), split});
    m->fill_view(out);
    return KRIYA_KV_OK;
}

static int32_t prefill_common(kriya_kv_manager* m, uint64_t seq_id, uint32_t prefix_tokens, uint32_t num_tokens,
                              const SeqTable** out_seq) {
    auto it = m->sequences.find(seq_id);
    if (it == m->sequences.end()) return m->fail(KRIYA_KV_INVALID_SEQUENCE_ID, seq_id);
    const uint64_t end = uint64_t(prefix_tokens) + num_tokens;  // saturating_add in the Rust
    if (num_tokens == 0 || std::min<uint64_t>(end, 0xFFFFFFFFull) > it->second.total_tokens)
        return m->fail(KRIYA_KV_INVALID_SEQUENCE_ID, seq_id);
    *out_seq = &it->second;
    return KRIYA_KV_OK;
}

int32_t kriya_kv_build_parallel_prefill_layout(kriya_kv_manager* m, uint64_t seq_id, uint32_t prefix_tokens,
                                               uint32_t num_tokens, uint32_t max_blocks_per_cta,
                                               kriya_kv_plan_view* out) {
    if (!m || !out) return KRIYA_KV_BAD_ARGUMENT;
    const SeqTable* s = nullptr;
    const int32_t rc = prefill_common(m, seq_id, prefix_tokens, num_tokens, &s);
    if (rc != KRIYA_KV_OK) return rc;
    const uint32_t bs = m->block_size;
    PlanStorage& p = m->plan;
    p.clear();
    p.max_blocks_per_cta = max_blocks_per_cta;  // not clamped here (bsr_paged.rs:665)
    p.indptr.push_back(0);
    for (uint32_t i = 0; i < num_tokens; ++i) {
        const uint32_t need = div_ceil(prefix_tokens + i + 1, bs);
        if (need > s->blocks.size()) return m->fail(KRIYA_KV_INVALID_SEQUENCE_ID, seq_id);
        for (uint32_t b = 0; b < need; ++b) p.indices.push_back(int32_t(s->blocks[b]));
        p.indptr.push_back(int32_t(p.indices.size()));
        p.last_len.push_back(int32_t(((prefix_tokens + i) % bs) + 1));
        p.tiles.push_back({0u, 0u, need, need > max_blocks_per_cta ? 1u : 0u});
    }
    m->fill_view(out);
    return KRIYA_KV_OK;
}

int32_t kriya_kv_build_deduplicated_prefill_layout(kriya_kv_manager* m, uint64_t seq_id, uint32_t prefix_tokens,
                                                   uint32_t num_tokens, uint32_t max_blocks_per_cta,
                                                   kriya_kv_plan_view* out) {
    if (!m || !out) return KRIYA_KV_BAD_ARGUMENT;
    const SeqTable* s = nullptr;
    const int32_t rc = prefill_common(m, seq_id, prefix_tokens, num_tokens, &s);
    if (rc != KRIYA_KV_OK) return rc;
    const uint32_t bs = m->block_size;
    PlanStorage& p = m->plan;
    p.clear();
    p.max_blocks_per_cta = max_blocks_per_cta;
    const size_t max_need = std::min<size_t>(div_ceil(prefix_tokens + num_tokens, bs), s->blocks.size());
    for (size_t b = 0; b < max_need; ++b) p.indices.push_back(int32_t(s->blocks[b]));
    p.indptr.push_back(0);
    for (uint32_t i = 0; i < num_tokens; ++i) {
        const uint32_t need = div_ceil(prefix_tokens + i + 1, bs);
        p.indptr.push_back(int32_t(need));  // per-row block COUNT, not an offset (bsr_paged.rs:698-705)
        p.last_len.push_back(int32_t(((prefix_tokens + i) % bs) + 1));
        p.tiles.push_back({0u, 0u, need, need > max_blocks_per_cta ? 1u : 0u});
    }
    m->fill_view(out);
    return KRIYA_KV_OK;
}

}  // extern "C"
