// Chunked causal prefill attention over the paged cache on the 5th-generation tensor cores (the job of
// bsr_paged_gqa_prefill_stage1 / _bq8 / bsr_paged_gqa_tiled_mma_prefill,
// kernels/metal/paged_gqa_and_deltanet.metal:508-847,851-1192,1206-1468).
//
// One CTA owns a tile of 128 query tokens of one sequence for TWO query heads of the same KV head (heads A and B;
// an odd group size leaves the last CTA of a group with one head).  The two heads share every K/V tile the CTA
// loads and are processed by two independent softmax warpgroups, so that while one head's softmax runs the
// tensor pipe works on the other head:
//   - warp 8 (producer) loads the two query tiles with TMA (a 2-D map over q encoded per launch) and gathers the KV
//     pages 128 tokens (8 pages) at a time through the block table with TMA tensor loads (2-D map over the pool
//     [rows = block*16 + token][cols = kv_head*D + d], box 64 x 16, 128-byte swizzle, no multicast) into
//     shared-memory rings (K two deep, V three deep), completion on mbarriers;
//   - warp 9 issues tcgen05.mma in the order P_A.V(j), S_A(j+1), P_B.V(j), S_B(j+1): S_x = Q_x.K^T (128 x 128 x D) into head x's TMEM score tile and
//     O_x += P_x.V (128 x D x 128) into its TMEM accumulator.  P_x is read from TMEM (it is written in place over
//     the first half of S_x), V straight from its [token][d] layout as an MN-major operand: nothing is transposed
//     and P never touches shared memory;
//   - warps 0-3 (head A) and 4-7 (head B): one thread per query row = one TMEM lane.  A thread reads its 128 scores
//     once into registers, applies scale and the causal mask (key position <= prefix + query index), keeps the
//     running max / sum, writes P in the storage dtype back to TMEM and rescales O only when the running max moved
//     by more than 2^8 (the exponent reference is otherwise kept, which is exact in fp32).  The softmax warpgroups
//     take registers from the third warpgroup (setmaxnreg) so that the score row does not spill.
// Every mbarrier wait is bounded; on expiry the kernel records a status word, skips the remaining work, frees its
// TMEM and returns.
//
// Roofline: 4 * Hq * D * sum_q (prefix + q + 1) FLOP per chunk against the dense bf16 tensor peak.
#include <algorithm>
#include <cstdio>
#include <cstdlib>

#define KRIYA_INLINE_WAITS 1
#include "kriya_tc.cuh"

namespace kriya {

constexpr int kQTile = 128;   // query rows per CTA (= TMEM lanes)
constexpr int kKvTile = 128;  // keys per iteration (8 pages)
constexpr int kPagePf = 16;
constexpr int kPagesPerTile = kKvTile / kPagePf;
constexpr int kKStages = 2;  // K tile ring: a K tile is free again once both heads' S MMAs of its KV tile are done
constexpr int kVStages = 3;  // V tile ring: freed one softmax later, so it is one deeper
// Three warpgroups: warps 0-3 softmax A, 4-7 softmax B, 8 producer, 9 MMA issuer, 10-11 idle.  The kernel starts with
// 168 registers per thread; the third warpgroup hands most of its registers back and the softmax warpgroups take
// them (128 x 72 + 256 x 216 = 384 x 168), so a thread can hold a whole score row without spilling.
constexpr int kPrefillThreads = 384;
constexpr int kRegsWorkers = 72;
constexpr int kRegsSoftmax = 216;
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
constexpr float kLog2ePf = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;

struct PrefillParams {
    KriyaPrefillArgs a;
    uint32_t q_tiles;  // query tiles of the whole launch (all sequences)
    uint32_t pairs;    // head pairs per KV head = ceil(group / 2)
};

// Closes the thread's bulk group (tensor stores) and waits until their source has been read.
__device__ __forceinline__ void bulk_commit_wait_read() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// Shared memory (all tiles 1024-byte aligned):
//   Q_A, Q_B: D/64 panels x [128 rows][128 B] each
//   K ring  : 2 stages x D/64 panels x [128 tokens][128 B]
//   V ring  : 3 stages of the same size, each ring with its own full / empty barriers
// Tensor memory (512 columns): head A: S/P at 0, O at 128; head B: S/P at 256, O at 384.
template <int D, typename T>
__global__ void __launch_bounds__(kPrefillThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
               const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_o, PrefillParams pp) {
    constexpr int PANELS = D / 64;
    constexpr uint32_t PANEL_BYTES = 128 * 128;  // 128 rows x 128 B
    constexpr uint32_t Q_BYTES = PANELS * PANEL_BYTES;
    constexpr uint32_t KV_BYTES = PANELS * PANEL_BYTES;  // one of K or V, one stage
    constexpr uint32_t FMT = (T::kDtype == KRIYA_DTYPE_BF16) ? 1u : 0u;
    constexpr uint32_t IDESC_S = make_idesc(FMT, 128, 128, 0, 0);
    constexpr uint32_t IDESC_O = make_idesc(FMT, 128, D, 0, 1);
    constexpr uint32_t TMEM_COLS = 512;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
    uint8_t* sQ = sm;                      // [2 heads][Q_BYTES]
    uint8_t* sK = sQ + 2 * Q_BYTES;        // [kKStages][KV_BYTES]
    uint8_t* sV = sK + kKStages * KV_BYTES;  // [kVStages][KV_BYTES]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + kVStages * KV_BYTES);
    uint64_t* k_full = bars;         // [2]
    uint64_t* k_empty = bars + 2;    // [2]
    uint64_t* v_full = bars + 4;     // [3]
    uint64_t* v_empty = bars + 7;    // [3]
    uint64_t* s_full = bars + 10;    // [2 heads]
    uint64_t* p_ready = bars + 12;   // [2 heads], one arrival per softmax warp
    uint64_t* pv_done = bars + 14;   // [2 heads]
    uint64_t* q_full = bars + 16;
    uint64_t* o_staged = bars + 17;  // [2 heads], one arrival per softmax warp: the output tile is in shared memory
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const KriyaPrefillArgs& a = pp.a;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    // tiles arrive sorted, most keys first; blockIdx = (kv head, pair, tile) with the tile fastest
    const KriyaPrefillTile qt = a.tiles[blockIdx.x % pp.q_tiles];
    const uint32_t hp = blockIdx.x / pp.q_tiles;
    const uint32_t group = a.num_q_heads / a.num_kv_heads;
    const uint32_t kv_head = hp / pp.pairs, pair = hp % pp.pairs;
    const uint32_t head0 = kv_head * group + pair * 2u;
    const uint32_t n_heads = min(2u, group - pair * 2u);
    const uint32_t tile_start = qt.q_row0;  // first row of this tile in q / out
    const uint32_t tile_rows = qt.rows;
    const uint32_t kv_limit = qt.pos0 + tile_rows;  // keys [0, kv_limit) of the sequence can be seen by this tile
    // Sliding window (0 = none): query row r at position pos0 + r attends keys pos0 + r + 1 - window ..= pos0 + r.  The
    // earliest window start of the tile is row 0's, so KV tiles in front of it are skipped altogether: the loops below
    // count j = 0 .. n_tiles over the tiles tile0 + j.
    const uint32_t window = a.window;
    const uint32_t wtile0 = (window != 0u && qt.pos0 + 1u > window) ? (qt.pos0 + 1u - window) / uint32_t(kKvTile) : 0u;
    // a piece of a tile that was cut along the KV axis covers the KV tiles kv_t0 .. kv_t1 - 1 only
    const uint32_t tile_end = (kv_limit + kKvTile - 1) / kKvTile;
    const uint32_t tile0 = max(wtile0, qt.kv_t0);
    const uint32_t tile1 = qt.kv_t1 != 0u ? min(qt.kv_t1, tile_end) : tile_end;
    const uint32_t n_tiles = tile1 > tile0 ? tile1 - tile0 : 0u;
    const bool partial = qt.slot != UINT32_MAX;
    const uint32_t seq_end = qt.seq_end;  // tokens of the sequence that exist in the cache

    // ---- setup -------------------------------------------------------------------------------------------
    if (tid == 8 * 32) {  // the producer's first lane: the descriptors are on their way while the barriers are set up
        tma_prefetch_map(&map_q);
        tma_prefetch_map(&map_k);
        tma_prefetch_map(&map_v);
    }
    if (tid == 0) {
        for (int i = 0; i < kKStages; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
        }
        for (int i = 0; i < kVStages; ++i) {
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_ready[i], 4);
            mbar_init(&pv_done[i], 1);
            mbar_init(&o_staged[i], 4);
        }
        mbar_init(q_full, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 9) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp >= 8) {
    setmaxnreg_dec<kRegsWorkers>();
    if (warp == 8) {
        // ---- producer: gather the tile's pages through the block table --------------------------------
        const int32_t* table = a.table + qt.tbl_off;
        // the query tiles of the CTA's heads: one 64-column x 128-row box per panel (rows past the end of q read as zero;
        // rows past the tile but inside q belong to another sequence and only feed output rows that are never stored)
        if (lane == 0) {
            mbar_arrive_expect_tx(q_full, n_heads * Q_BYTES);
            for (uint32_t x = 0; x < n_heads; ++x)
#pragma unroll
                for (int p = 0; p < PANELS; ++p)
                    tma_load_2d(sQ + x * Q_BYTES + p * PANEL_BYTES, &map_q, int32_t(head0 + x) * D + p * 64, int32_t(tile_start), q_full);
        }
        __syncwarp();
        uint32_t vs = 0, v_round = 0;  // V stage of tile j = j % kVStages, round = j / kVStages
        for (uint32_t j = 0; j < n_tiles; ++j) {
            if (*abort_flag) break;
            const uint32_t ks = j & 1u;
            const uint32_t first_page = (tile0 + j) * kPagesPerTile;
            const uint32_t last_needed = (min(kv_limit, (tile0 + j + 1) * uint32_t(kKvTile)) + kPagePf - 1) / kPagePf;  // exclusive
            const uint32_t npages = last_needed - first_page;
            int32_t blk = 0;
            if (lane < npages) {
                blk = table[first_page + lane];
                if (uint32_t(blk) >= a.num_blocks) {
                    atomicMax(a.status, uint32_t(KRIYA_DEV_BAD_BLOCK_INDEX));
                    blk = 0;
                }
            }
            const int32_t y = int32_t(a.layer_row0) + blk * kPagePf;
            bool ok = j < uint32_t(kKStages) || warp_wait(&k_empty[ks], ((j >> 1) - 1u) & 1u);
            if (ok) {
                if (lane == 0) mbar_arrive_expect_tx(&k_full[ks], npages * uint32_t(PANELS * kPagePf * 128));
                __syncwarp();
                if (lane < npages) {
#pragma unroll
                    for (int p = 0; p < PANELS; ++p)
                        tma_load_2d(sK + ks * KV_BYTES + p * PANEL_BYTES + lane * (kPagePf * 128), &map_k, int32_t(kv_head) * D + p * 64, y, &k_full[ks]);
                }
                ok = j < uint32_t(kVStages) || warp_wait(&v_empty[vs], (v_round - 1u) & 1u);
            }
            if (!ok) {
                if (lane == 0) {
                    atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
                    *abort_flag = 1;
                }
                break;
            }
            if (lane == 0) mbar_arrive_expect_tx(&v_full[vs], npages * uint32_t(PANELS * kPagePf * 128));
            __syncwarp();
            if (lane < npages) {
#pragma unroll
                for (int p = 0; p < PANELS; ++p)
                    tma_load_2d(sV + vs * KV_BYTES + p * PANEL_BYTES + lane * (kPagePf * 128), &map_v, int32_t(kv_head) * D + p * 64, y, &v_full[vs]);
            }
            if (++vs == uint32_t(kVStages)) { vs = 0; ++v_round; }
        }
    } else if (warp == 9) {
        // ---- MMA issuer ------------------------------------------------------------------------------------
        // Issue order: S_A(0), S_B(0), then per KV tile j: P_A.V(j), S_A(j+1), P_B.V(j), S_B(j+1).  The tensor pipe runs
        // one thread's MMAs in issue order, so S_x(j+1) may overwrite the score tile that holds P_x(j) as soon as
        // P_x.V(j) has been issued, and the commit behind S_x(j+1) also covers P_x.V(j): a softmax group that sees
        // s_full[x] may rescale O_x.  While one head is in its softmax the pipe works on the other head.
        // Every lane runs this code; only the tensor-core instructions themselves are predicated on the elected lane.
        const uint32_t el = (lane == 0) ? 1u : 0u;
        const uint64_t q_desc = smem_desc_sw128(smem_u32(sQ), 16, 1024);
        const uint64_t k_desc = smem_desc_sw128(smem_u32(sK), 16, 1024);
        const uint64_t v_desc = smem_desc_sw128(smem_u32(sV), PANEL_BYTES, 1024);
        auto issue_s = [&](uint32_t x, uint32_t stage, bool last_head) {
            const uint32_t d_tmem = tmem_base + x * 256u;
            const uint64_t qd = q_desc + uint64_t((x * Q_BYTES) >> 4), kd = k_desc + uint64_t((stage * KV_BYTES) >> 4);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const uint64_t off = uint64_t((uint32_t(ks / 4) * PANEL_BYTES + uint32_t(ks % 4) * 32u) >> 4);
                umma_ss_pred(d_tmem, qd + off, kd + off, IDESC_S, ks > 0 ? 1u : 0u, el);
            }
            umma_commit_pred(&s_full[x], el);
            if (last_head) umma_commit_pred(&k_empty[stage], el);
        };
        bool ok = n_tiles > 0 && warp_wait(q_full, 0u);
        ok = ok && warp_wait(&k_full[0], 0u);
        if (ok) {
            tc_fence_after();
            for (uint32_t x = 0; x < n_heads; ++x) issue_s(x, 0u, x + 1u == n_heads);
        }
        uint32_t vs = 0, v_round = 0;
        for (uint32_t j = 0; j < n_tiles && ok; ++j) {
            if (*abort_flag) break;
            const uint32_t stage = j & 1u;
            const bool more = j + 1u < n_tiles;
            const uint64_t vd = v_desc + uint64_t((vs * KV_BYTES) >> 4);
            for (uint32_t x = 0; x < n_heads && ok; ++x) {
                if (x == 0u) {  // the tiles land long before the probabilities are ready: take these waits first
                    ok = warp_wait(&v_full[vs], v_round & 1u);
                    if (ok && more) ok = warp_wait(&k_full[stage ^ 1u], ((j + 1u) >> 1) & 1u);
                    if (!ok) break;
                }
                ok = warp_wait(&p_ready[x], j & 1u);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < kKvTile / 16; ++ks) {
                    // A = P_x from tensor memory (16 keys = 8 columns), B = V page ks (MN-major)
                    umma_ts_pred(tmem_base + x * 256u + 128u, tmem_base + x * 256u + uint32_t(ks) * 8u,
                                 vd + uint64_t((uint32_t(ks) * (kPagePf * 128)) >> 4), IDESC_O, (j > 0 || ks > 0) ? 1u : 0u, el);
                }
                if (x + 1u == n_heads) umma_commit_pred(&v_empty[vs], el);
                if (more) issue_s(x, stage ^ 1u, x + 1u == n_heads);
                else umma_commit_pred(&pv_done[x], el);
            }
            if (++vs == uint32_t(kVStages)) { vs = 0; ++v_round; }
        }
        if (!ok && n_tiles > 0 && lane == 0) {
            atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            *abort_flag = 1;
        }
    }
    } else {
    setmaxnreg_inc<kRegsSoftmax>();
    if ((warp >> 2) < n_heads) {
        // ---- softmax warpgroups: x = 0 (warps 0-3) / 1 (warps 4-7); thread = query row = TMEM lane -------------
        const uint32_t x = warp >> 2;
        const uint32_t row = tid & 127u;
        const uint32_t lane_addr = ((warp & 3u) * 32u) << 16;
        const uint32_t s_addr = tmem_base + lane_addr + x * 256u;
        const uint32_t o_addr = s_addr + 128u;
        const bool softcap = a.logit_softcap > 0.0f;
        const float scale2 = softcap ? kLog2ePf : a.sm_scale * kLog2ePf;
        const uint32_t q_pos = qt.pos0 + min(row, tile_rows - 1u);  // absolute position
        float m_used = -INFINITY, l_run = 0.0f;
        bool ok = true;
        uint32_t vs = 0, v_round = 0;
        for (uint32_t j = 0; j < n_tiles; ++j, vs = (vs + 1u == uint32_t(kVStages)) ? 0u : vs + 1u, v_round += (vs == 0u)) {
            if (*abort_flag) { ok = false; break; }
            ok = warp_wait(&s_full[x], j & 1u);
            if (!ok) break;
            tc_fence_after();
            const uint32_t key0 = (tile0 + j) * kKvTile;
            const bool diag = key0 + kKvTile - 1u > qt.pos0;  // some row of the tile masks some key
            // some key of the tile lies in front of some row's window (the last row's window starts latest)
            const bool wdiag = window != 0u && key0 + window < qt.pos0 + tile_rows;
            // The whole score row goes into registers, once.  A tile that needs no mask and comes behind the first one is
            // taken a quarter at a time against the exponent reference the row already has: the next quarter's load runs
            // under this quarter's maxima, exponentials and probability stores (P quarter c lies over score columns that
            // have been read: 16c .. 16c+15 against 32c ..).  The tile's own maximum is known at the end; if it is above
            // the reference by more than the threshold for some row of the warp, the tile is done again from the
            // registers, the ordinary way.
            uint32_t sr[4][32];
            const bool fast = j > 0 && !softcap && !diag && !wdiag && !__any_sync(0xFFFFFFFFu, m_used == -INFINITY);
            bool redo = false;
            if (fast) {
                const float2 sc2f = make_float2(scale2, scale2), neg_m2f = make_float2(-m_used, -m_used);
                float2 psum2f = make_float2(0.0f, 0.0f);
                float mq[4];
                tmem_ld32(s_addr, sr[0]);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if (c + 1 < 4) tmem_ld32(s_addr + (c + 1) * 32, sr[c + 1]);
                    float ma = -INFINITY, mb = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        ma = max3(ma, __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
                        mb = max3(mb, __uint_as_float(sr[c][i + 2]), __uint_as_float(sr[c][i + 3]));
                    }
                    mq[c] = fmaxf(ma, mb);
                    uint32_t packed[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float2 e = __ffma2_rn(make_float2(__uint_as_float(sr[c][2 * i]), __uint_as_float(sr[c][2 * i + 1])), sc2f, neg_m2f);
                        const float2 pr = make_float2(fast_exp2(e.x), fast_exp2(e.y));
                        psum2f = __fadd2_rn(psum2f, pr);
                        packed[i] = T::pack2(pr.x, pr.y);
                    }
                    tmem_st16(s_addr + c * 16, packed);
                    if (c + 1 < 4) tmem_wait_ld();
                }
                const float m_tile_f = fmaxf(max3(mq[0], mq[1], mq[2]), mq[3]) * scale2;
                redo = __any_sync(0xFFFFFFFFu, m_tile_f > m_used + kRescaleThreshold);
                if (!redo) {
                    tmem_wait_st();
                    l_run += psum2f.x + psum2f.y;
                }
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_ld32(s_addr + c * 32, sr[c]);
                tmem_wait_ld();
            }
            if (!fast || redo) {
            // the scores stay raw in registers; scale and exponent reference are folded into one fma per pair below
            if (softcap) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float s = __uint_as_float(sr[c][i]) * a.sm_scale;
                        sr[c][i] = __float_as_uint(tanhf(fminf(fmaxf(s / a.logit_softcap, -15.0f), 15.0f)) * a.logit_softcap);
                    }
            }
            if (diag) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (key0 + uint32_t(c * 32 + i) > q_pos) sr[c][i] = 0xFF800000u;  // -inf
            }
            if (wdiag) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (key0 + uint32_t(c * 32 + i) + window <= q_pos) sr[c][i] = 0xFF800000u;  // in front of the window
            }
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four independent chains
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int i = 0; i < 32; i += 2) m4[c] = max3(m4[c], __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
            const float m_tile = fmaxf(max3(m4[0], m4[1], m4[2]), m4[3]) * scale2;  // scale2 > 0
            // the commit behind S_x(j) covers P_x.V(j-1): O_x may be rescaled and the score tile rewritten
            float alpha = 1.0f;
            bool need = false;
            if (j == 0) {
                m_used = m_tile;
            } else if (m_tile > m_used + kRescaleThreshold) {
                alpha = exp2f(m_used - m_tile);
                m_used = m_tile;
                need = true;
            }
            if (__any_sync(0xFFFFFFFFu, need)) {
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(o_addr + c * 32, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                    tmem_st32(o_addr + c * 32, r);
                }
            }
            // probabilities in the storage dtype, two keys per 32-bit column, over the first 64 columns of the score tile
            float2 psum2 = make_float2(0.0f, 0.0f);
            // a row that has seen no key yet (its window begins behind this tile) has m_used = -inf: its exponents must
            // come out as -inf, not as inf - inf
            const float neg_m = (m_used == -INFINITY) ? 0.0f : -m_used;
            const float2 sc2 = make_float2(scale2, scale2), neg_m2 = make_float2(neg_m, neg_m);
#pragma unroll
            for (int c = 0; c < 4; ++c) {  // 32 keys = 16 columns at a time, each stored as soon as it is ready
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float2 e = __ffma2_rn(make_float2(__uint_as_float(sr[c][2 * i]), __uint_as_float(sr[c][2 * i + 1])), sc2, neg_m2);
                    const float2 pr = make_float2(fast_exp2(e.x), fast_exp2(e.y));
                    psum2 = __fadd2_rn(psum2, pr);
                    packed[i] = T::pack2(pr.x, pr.y);
                }
                tmem_st16(s_addr + c * 16, packed);
            }
            const float psum = psum2.x + psum2.y;
            tmem_wait_st();
            l_run = l_run * alpha + psum;
            }
            // Only the last tile can hold rows that are not valid V data: slots past the end of the sequence (loaded, but
            // they may hold anything) and pages the producer did not load (shared memory as the previous kernel left
            // it).  Their probabilities are zero, but 0 x NaN is NaN, so head A's warpgroup clears those rows; P.V of
            // head B is issued after P.V of head A and sees the cleared rows too.
            if (x == 0u && j + 1u == n_tiles) {
                const uint32_t loaded_end = ((kv_limit + kPagePf - 1) / kPagePf) * kPagePf;
                const uint32_t first_bad = min(seq_end, loaded_end) - key0;  // seq_end >= kv_limit > key0
                if (first_bad < uint32_t(kKvTile)) {
                    ok = warp_wait(&v_full[vs], v_round & 1u);  // the tile must have landed before rows of it are cleared
                    if (!ok) break;
                    for (uint32_t i = first_bad * 8u + row; i < uint32_t(kKvTile) * 8u; i += 128u) {
                        const uint32_t rr = i >> 3, ch = i & 7u;
#pragma unroll
                        for (int p = 0; p < PANELS; ++p)
                            *reinterpret_cast<uint4*>(sV + vs * KV_BYTES + p * PANEL_BYTES + rr * 128u + (ch << 4)) =
                                make_uint4(0u, 0u, 0u, 0u);
                    }
                    fence_async_smem();
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[x]);
        }
        if (ok && n_tiles > 0) {
            ok = warp_wait(&pv_done[x], 0u);
            if (ok && partial) {
                // A piece of a tile cut along the KV axis: its state (exponent reference, sum, un-normalised accumulator)
                // goes to the piece's scratch slot, accumulator as [d / 4][row] float4 so that a warp's stores are contiguous.
                tc_fence_after();
                const uint32_t hp_count = gridDim.x / pp.q_tiles;
                const size_t cta_slot = size_t(qt.slot) * hp_count + hp;
                float4* po = reinterpret_cast<float4*>(a.part_o) + (cta_slot * 2u + x) * size_t(D / 4) * kQTile;
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(o_addr + c * 32, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int q4 = 0; q4 < 8; ++q4)
                        po[size_t(c * 8 + q4) * kQTile + row] = make_float4(__uint_as_float(r[q4 * 4]), __uint_as_float(r[q4 * 4 + 1]),
                                                                            __uint_as_float(r[q4 * 4 + 2]), __uint_as_float(r[q4 * 4 + 3]));
                }
                reinterpret_cast<float2*>(a.part_ml)[(cta_slot * 2u + x) * kQTile + row] = make_float2(m_used, l_run);
            } else if (ok) {
                tc_fence_after();
                const float inv_l = 1.0f / fmaxf(l_run, 1e-12f);
                // A full tile goes through shared memory in the layout of the query tile it replaces (every S MMA is
                // complete once pv_done[x] has fired) and leaves with one tensor store per 64-column panel.  A partial
                // tile is written row by row from registers: a tensor store would also write the next sequence's rows.
                const bool full = tile_rows == uint32_t(kQTile);
                uint8_t* stage = sQ + x * Q_BYTES;
                uint16_t* og = reinterpret_cast<uint16_t*>(a.out) + (size_t(tile_start + row) * a.num_q_heads + head0 + x) * D;
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(o_addr + c * 32, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            w[i] = T::pack2(__uint_as_float(r[q4 * 8 + 2 * i]) * inv_l, __uint_as_float(r[q4 * 8 + 2 * i + 1]) * inv_l);
                        const uint4 val = make_uint4(w[0], w[1], w[2], w[3]);
                        const uint32_t chunk = uint32_t(c & 1) * 4u + uint32_t(q4);  // 16-byte chunk inside the 64-column panel
                        if (full)
                            *reinterpret_cast<uint4*>(stage + uint32_t(c >> 1) * PANEL_BYTES + row * 128u + ((chunk ^ (row & 7u)) << 4)) = val;
                        else if (row < tile_rows)
                            *reinterpret_cast<uint4*>(og + c * 32 + q4 * 8) = val;
                    }
                }
                if (full) {
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&o_staged[x]);
                    if (row == 0 && mbar_wait(&o_staged[x], 0u)) {  // bounded: the group's 128 rows are in place
#pragma unroll
                        for (int p = 0; p < PANELS; ++p)
                            tma_store_2d(&map_o, stage + p * PANEL_BYTES, int32_t(head0 + x) * D + p * 64, int32_t(tile_start));
                    }
                }
                bulk_commit_wait_read();  // the tile must have been read before the CTA gives its shared memory back
            }
        }
        if (!ok && lane == 0) {
            atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            *abort_flag = 1;
        }
    }

    }
    // ---- teardown: every thread gets here; TMEM is returned by the warp that took it ------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Combines the pieces of the query tiles that were cut along the KV axis: block = (tile, head pair, eight (head, row)
// jobs), a warp per job, a lane per four output dimensions.  Everything a job reads is asked for before any of it is
// used (at most kPfMaxParts pieces): the kernel is a few dependent memory round trips long, so it needs many warps and
// no chains.
constexpr uint32_t kPfMaxParts = 8;
template <int D, typename T>
__global__ void __launch_bounds__(256) prefill_merge_kernel(KriyaPrefillArgs a, const KriyaPrefillMerge* items, uint32_t pairs) {
    // launched with programmatic stream serialisation: the blocks are resident before the attention kernel has finished
    // and wait here for its completion (and with it for the pieces' states)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const KriyaPrefillMerge it = items[blockIdx.x];
    const uint32_t hp = blockIdx.y, hp_count = gridDim.y;
    const uint32_t group = a.num_q_heads / a.num_kv_heads;
    const uint32_t kv_head = hp / pairs, pair = hp % pairs;
    const uint32_t head0 = kv_head * group + pair * 2u;
    const uint32_t n_heads = min(2u, group - pair * 2u);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t job = blockIdx.z * 8u + warp;
    if (job >= n_heads * it.rows) return;
    const uint32_t x = job / it.rows, row = job % it.rows;
    const float4* po = reinterpret_cast<const float4*>(a.part_o);
    const float2* pml = reinterpret_cast<const float2*>(a.part_ml);
    const bool active = lane < uint32_t(D / 4);
    float2 ml[kPfMaxParts];
    float4 v[kPfMaxParts];
#pragma unroll
    for (uint32_t p = 0; p < kPfMaxParts; ++p) {
        const size_t cs = (size_t(it.slot0 + min(p, it.n_parts - 1u)) * hp_count + hp) * 2u + x;
        ml[p] = pml[cs * kQTile + row];
        v[p] = active ? po[(cs * uint32_t(D / 4) + lane) * kQTile + row] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    float m = -INFINITY;
#pragma unroll
    for (uint32_t p = 0; p < kPfMaxParts; ++p) m = (p < it.n_parts) ? fmaxf(m, ml[p].x) : m;
    float l = 0.0f;
    float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
    for (uint32_t p = 0; p < kPfMaxParts; ++p) {
        const float w = (p < it.n_parts && ml[p].x != -INFINITY) ? exp2f(ml[p].x - m) : 0.0f;
        l = fmaf(w, ml[p].y, l);
        o.x = fmaf(w, v[p].x, o.x);
        o.y = fmaf(w, v[p].y, o.y);
        o.z = fmaf(w, v[p].z, o.z);
        o.w = fmaf(w, v[p].w, o.w);
    }
    if (active) {
        const float inv_l = 1.0f / fmaxf(l, 1e-12f);
        uint16_t* og = reinterpret_cast<uint16_t*>(a.out) + (size_t(it.q_row0 + row) * a.num_q_heads + head0 + x) * D + lane * 4u;
        *reinterpret_cast<uint2*>(og) = make_uint2(T::pack2(o.x * inv_l, o.y * inv_l), T::pack2(o.z * inv_l, o.w * inv_l));
    }
}

template <int D, typename T>
cudaError_t launch_prefill_t(const KriyaPrefillArgs& a, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mq,
                             const CUtensorMap& mo, int max_smem_optin, cudaStream_t s) {
    constexpr int PANELS = D / 64;
    const size_t smem = size_t(PANELS) * 128 * 128 * (2 + kKStages + kVStages) + 256 + 1024;  // Q x 2 heads, K ring, V ring
    if (smem > size_t(max_smem_optin)) return cudaErrorInvalidValue;
    auto kern = prefill_kernel<D, T>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    PrefillParams pp;
    pp.a = a;
    pp.q_tiles = a.n_tiles;
    const uint32_t group = a.num_q_heads / a.num_kv_heads;
    pp.pairs = (group + 1u) / 2u;
    kern<<<pp.q_tiles * pp.pairs * a.num_kv_heads, kPrefillThreads, smem, s>>>(mk, mv, mq, mo, pp);
    if (a.n_merge != 0u) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(a.n_merge, pp.pairs * a.num_kv_heads, 2 * kQTile / 8);
        cfg.blockDim = dim3(256);
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        e = cudaLaunchKernelEx(&cfg, prefill_merge_kernel<D, T>, a, a.merge_items, pp.pairs);
        if (e != cudaSuccess) return e;
    }
    return cudaGetLastError();
}

}  // namespace kriya

bool kriya_prefill_supported(uint32_t head_dim, uint32_t group, uint32_t block_size, uint32_t dtype) {
    (void)dtype;
    return (head_dim == 64 || head_dim == 128) && group >= 1 && block_size == uint32_t(kriya::kPagePf);
}

namespace {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up once per process through the runtime.
cudaError_t tensor_map_encoder(EncodeFn* out) {
    static EncodeFn cached = nullptr;
    if (cached == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess) return e;
        if (fn == nullptr || qres != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
        cached = reinterpret_cast<EncodeFn>(fn);
    }
    *out = cached;
    return cudaSuccess;
}

// 2-D map over a row-major 16-bit matrix [rows][row_elems]; box = 64 columns x box_rows rows, 128-byte swizzle, zero
// fill outside the matrix.
cudaError_t encode_rows_map(void* base, uint64_t rows, uint32_t row_elems, uint32_t box_rows, CUtensorMap* out) {
    EncodeFn enc = nullptr;
    const cudaError_t e = tensor_map_encoder(&enc);
    if (e != cudaSuccess) return e;
    const cuuint64_t dims[2] = {row_elems, rows};
    const cuuint64_t strides[1] = {cuuint64_t(row_elems) * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}
}  // namespace

// Encodes the 2-D tensor maps over the K and V pools (all layers): rows = (layer, block, token), columns =
// (kv head, d); box = 64 columns x 16 rows with the 128-byte swizzle the MMA descriptors expect.
cudaError_t kriya_prefill_encode_maps(void* pool_k, void* pool_v, uint64_t total_rows, uint32_t row_elems,
                                      void* out_map_k, void* out_map_v) {
    cudaError_t e = encode_rows_map(pool_k, total_rows, row_elems, uint32_t(kriya::kPagePf), static_cast<CUtensorMap*>(out_map_k));
    if (e != cudaSuccess) return e;
    return encode_rows_map(pool_v, total_rows, row_elems, uint32_t(kriya::kPagePf), static_cast<CUtensorMap*>(out_map_v));
}

cudaError_t kriya_launch_prefill(const KriyaPrefillArgs& a, uint32_t head_dim, uint32_t block_size, uint32_t dtype,
                                 int max_smem_optin, cudaStream_t s) {
    if (a.n_tiles == 0) return cudaSuccess;
    if (!kriya_prefill_supported(head_dim, a.num_q_heads / a.num_kv_heads, block_size, dtype) || !a.map_k || !a.map_v)
        return cudaErrorInvalidValue;
    const CUtensorMap& mk = *static_cast<const CUtensorMap*>(a.map_k);
    const CUtensorMap& mv = *static_cast<const CUtensorMap*>(a.map_v);
    // the query and output matrices change with every call: their maps ([q_rows][Hq * D], one box = 64 columns x 128 rows) is encoded here
    // and travels to the kernel by value
    if ((reinterpret_cast<uintptr_t>(a.q) & 15u) != 0 || (reinterpret_cast<uintptr_t>(a.out) & 15u) != 0 || a.q_rows == 0)
        return cudaErrorInvalidValue;
    alignas(64) CUtensorMap mq, mo;
    cudaError_t e = encode_rows_map(const_cast<void*>(a.q), a.q_rows, a.num_q_heads * head_dim, uint32_t(kriya::kQTile), &mq);
    if (e == cudaSuccess) e = encode_rows_map(a.out, a.q_rows, a.num_q_heads * head_dim, uint32_t(kriya::kQTile), &mo);
    if (e != cudaSuccess) return e;
    using namespace kriya;
    if (head_dim == 128)
        return dtype == KRIYA_DTYPE_FP16 ? launch_prefill_t<128, Fp16>(a, mk, mv, mq, mo, max_smem_optin, s)
                                         : launch_prefill_t<128, Bf16>(a, mk, mv, mq, mo, max_smem_optin, s);
    return dtype == KRIYA_DTYPE_FP16 ? launch_prefill_t<64, Fp16>(a, mk, mv, mq, mo, max_smem_optin, s)
                                     : launch_prefill_t<64, Bf16>(a, mk, mv, mq, mo, max_smem_optin, s);
}
