// Chunked causal prefill attention over the paged cache on the 5th-generation tensor cores (the job of
// bsr_paged_gqa_prefill_stage1 / _bq8 / bsr_paged_gqa_tiled_mma_prefill,
// kernels/metal/paged_gqa_and_deltanet.metal:508-847,851-1192,1206-1468).
//
// One CTA owns a tile of 128 query tokens of one query head and walks the sequence's KV pages 128 tokens
// (8 pages) at a time:
//   - a producer thread gathers the tile's K and V pages through the block table with TMA tensor loads
//     (2-D map over the pool [rows = block*16 + token][cols = kv_head*D + d], box 64 x 16, 128-byte swizzle)
//     into a two-stage shared-memory ring, completion on mbarriers;
//   - one thread issues tcgen05.mma: S = Q.K^T (128 x 128 x D) into one of two TMEM score buffers, and
//     O += P.V (128 x D x 128) into a TMEM accumulator; V is consumed straight from its [token][d] layout as
//     an MN-major operand, so no transpose is ever materialised;
//   - four softmax warps (one thread per query row = one TMEM lane) read S with tcgen05.ld, apply scale and
//     the causal mask (key position <= prefix + query index), keep the running max / sum in registers,
//     write P in the storage dtype into a swizzled shared-memory tile and rescale O in TMEM only when the
//     running max moved by more than 2^8 (the exponent reference is otherwise kept, which is exact in fp32);
//   - S(j+1) is issued before P.V(j), so the tensor pipe works on the next scores while the softmax of the
//     current tile runs.
// Every mbarrier wait is bounded; on expiry the kernel records a status word, skips the remaining work,
// frees its TMEM and returns.
//
// Roofline: 4 * Hq * D * sum_q (prefix + q + 1) FLOP per chunk against the dense bf16 tensor peak.
#include <algorithm>

#include "kriya_tc.cuh"

namespace kriya {

constexpr int kQTile = 128;   // query rows per CTA (= TMEM lanes)
constexpr int kKvTile = 128;  // keys per iteration (8 pages)
constexpr int kPagePf = 16;
constexpr int kPagesPerTile = kKvTile / kPagePf;
constexpr int kPrefillThreads = 192;  // warps 0-3 softmax, warp 4 producer, warp 5 MMA issuer
constexpr float kLog2ePf = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;

struct PrefillParams {
    KriyaPrefillArgs a;
    uint32_t q_tiles;  // query tiles of the whole launch (all sequences)
    uint32_t dtype;
};

// Shared memory (all tiles 1024-byte aligned):
//   Q  : D/64 panels x [128 rows][128 B]
//   K,V: 2 stages x D/64 panels x [128 tokens][128 B] each
//   P  : 2 panels x [128 rows][128 B]
template <int D, typename T>
__global__ void __launch_bounds__(kPrefillThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, PrefillParams pp) {
    constexpr int PANELS = D / 64;
    constexpr uint32_t PANEL_BYTES = 128 * 128;  // 128 rows x 128 B
    constexpr uint32_t Q_BYTES = PANELS * PANEL_BYTES;
    constexpr uint32_t KV_BYTES = PANELS * PANEL_BYTES;  // one of K or V, one stage
    constexpr uint32_t P_BYTES = 2 * PANEL_BYTES;
    constexpr uint32_t FMT = (T::kDtype == KRIYA_DTYPE_BF16) ? 1u : 0u;
    constexpr uint32_t IDESC_S = make_idesc(FMT, 128, 128, 0, 0);
    constexpr uint32_t IDESC_O = make_idesc(FMT, 128, D, 0, 1);
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t COL_S0 = 0, COL_S1 = 128, COL_O = 256;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
    uint8_t* sQ = sm;
    uint8_t* sK = sQ + Q_BYTES;            // [2][KV_BYTES]
    uint8_t* sV = sK + 2 * KV_BYTES;       // [2][KV_BYTES]
    uint8_t* sP = sV + 2 * KV_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
    uint64_t* kv_full = bars;        // [2]
    uint64_t* kv_empty = bars + 2;   // [2]
    uint64_t* s_full = bars + 4;     // [2]
    uint64_t* p_ready = bars + 6;    // 128 arrivals
    uint64_t* pv_done = bars + 7;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const KriyaPrefillArgs& a = pp.a;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    // heavy tiles (late queries see more keys) first
    // tiles arrive sorted, most keys first
    const KriyaPrefillTile qt = a.tiles[blockIdx.x % pp.q_tiles];
    const uint32_t q_head = blockIdx.x / pp.q_tiles;
    const uint32_t group = a.num_q_heads / a.num_kv_heads;
    const uint32_t kv_head = q_head / group;
    const uint32_t tile_start = qt.q_row0;  // first row of this tile in q / out
    const uint32_t tile_rows = qt.rows;
    const uint32_t kv_limit = qt.pos0 + tile_rows;  // keys [0, kv_limit) of the sequence can be seen by this tile
    const uint32_t n_tiles = (kv_limit + kKvTile - 1) / kKvTile;
    const uint32_t seq_end = qt.seq_end;  // tokens of the sequence that exist in the cache

    // ---- setup -------------------------------------------------------------------------------------------
    if (tid == 0) {
        mbar_init(&kv_full[0], 1);
        mbar_init(&kv_full[1], 1);
        mbar_init(&kv_empty[0], 1);
        mbar_init(&kv_empty[1], 1);
        mbar_init(&s_full[0], 1);
        mbar_init(&s_full[1], 1);
        mbar_init(p_ready, 128);
        mbar_init(pv_done, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 5) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    // zero the K/V ring once: pages a tile does not load must read as finite values
    for (uint32_t i = tid; i < (4 * KV_BYTES) / 16; i += kPrefillThreads)
        reinterpret_cast<uint4*>(sK)[i] = make_uint4(0u, 0u, 0u, 0u);
    // Q tile -> swizzled K-major panels (rows past the chunk are zero)
    {
        const uint16_t* qg = reinterpret_cast<const uint16_t*>(a.q);
        constexpr int CHUNKS = D / 8;  // 16-byte chunks per row
        for (uint32_t i = tid; i < uint32_t(kQTile * CHUNKS); i += kPrefillThreads) {
            const uint32_t r = i / CHUNKS, c = i % CHUNKS;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (r < tile_rows)
                val = *reinterpret_cast<const uint4*>(qg + (size_t(tile_start + r) * a.num_q_heads + q_head) * D + c * 8);
            const uint32_t panel = c >> 3, cc = c & 7u;
            *reinterpret_cast<uint4*>(sQ + panel * PANEL_BYTES + r * 128u + ((cc ^ (r & 7u)) << 4)) = val;
        }
    }
    fence_async_smem();  // generic-proxy writes (zero fill, Q) visible to the tensor core / TMA proxy
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 4) {
        // ---- producer: gather the tile's pages through the block table --------------------------------
        const int32_t* table = a.table + qt.tbl_off;
        for (uint32_t j = 0; j < n_tiles; ++j) {
            if (*abort_flag) break;
            const uint32_t stage = j & 1u;
            if (j >= 2 && !warp_wait(&kv_empty[stage], ((j >> 1) - 1u) & 1u)) {
                if (lane == 0) {
                    atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
                    *abort_flag = 1;
                }
                break;
            }
            const uint32_t first_page = j * kPagesPerTile;
            const uint32_t last_needed = (min(kv_limit, (j + 1) * uint32_t(kKvTile)) + kPagePf - 1) / kPagePf;  // exclusive
            const uint32_t npages = last_needed - first_page;
            int32_t blk = 0;
            if (lane < npages) {
                blk = table[first_page + lane];
                if (uint32_t(blk) >= a.num_blocks) {
                    atomicMax(a.status, uint32_t(KRIYA_DEV_BAD_BLOCK_INDEX));
                    blk = 0;
                }
            }
            if (lane == 0) mbar_arrive_expect_tx(&kv_full[stage], npages * uint32_t(2 * PANELS * kPagePf * 128));
            __syncwarp();
            if (lane < npages) {
                const int32_t y = int32_t(a.layer_row0) + blk * kPagePf;
#pragma unroll
                for (int p = 0; p < PANELS; ++p) {
                    const int32_t x = int32_t(kv_head) * D + p * 64;
                    tma_load_2d(sK + stage * KV_BYTES + p * PANEL_BYTES + lane * (kPagePf * 128), &map_k, x, y, &kv_full[stage]);
                    tma_load_2d(sV + stage * KV_BYTES + p * PANEL_BYTES + lane * (kPagePf * 128), &map_v, x, y, &kv_full[stage]);
                }
            }
        }
    } else if (warp == 5) {
        // ---- MMA issuer ------------------------------------------------------------------------------------
        const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV), p_addr = smem_u32(sP);
        auto issue_s = [&](uint32_t j) {
            const uint32_t stage = j & 1u;
            const uint32_t d_tmem = tmem_base + ((j & 1u) ? COL_S1 : COL_S0);
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                const uint32_t off = uint32_t(ks / 4) * PANEL_BYTES + uint32_t(ks % 4) * 32u;
                umma_f16(d_tmem, smem_desc_sw128(q_addr + off, 16, 1024), smem_desc_sw128(k_addr + stage * KV_BYTES + off, 16, 1024),
                         IDESC_S, ks > 0 ? 1u : 0u);
            }
            umma_commit(&s_full[j & 1u]);
        };
        bool ok = true;
        for (uint32_t j = 0; j < n_tiles && ok; ++j) {
            if (*abort_flag) break;
            if (j == 0) {
                ok = warp_wait(&kv_full[0], 0);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) issue_s(0);
            }
            if (j + 1 < n_tiles) {
                ok = warp_wait(&kv_full[(j + 1) & 1u], ((j + 1) >> 1) & 1u);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) issue_s(j + 1);
            }
            ok = warp_wait(p_ready, j & 1u);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t stage = j & 1u;
#pragma unroll
                for (int ks = 0; ks < kKvTile / 16; ++ks) {
                    // A = P (K-major, 16 keys = 32 B inside a 64-key panel), B = V page ks (MN-major)
                    const uint32_t a_off = uint32_t(ks / 4) * PANEL_BYTES + uint32_t(ks % 4) * 32u;
                    const uint32_t b_off = stage * KV_BYTES + uint32_t(ks) * (kPagePf * 128);
                    umma_f16(tmem_base + COL_O, smem_desc_sw128(p_addr + a_off, 16, 1024),
                             smem_desc_sw128(v_addr + b_off, PANEL_BYTES, 1024), IDESC_O, (j > 0 || ks > 0) ? 1u : 0u);
                }
                umma_commit(&kv_empty[stage]);
                umma_commit(pv_done);
            }
            __syncwarp();
        }
        if (!ok && lane == 0) {
            atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            *abort_flag = 1;
        }
    } else {
        // ---- softmax warps: thread = query row = TMEM lane ---------------------------------------------------
        const uint32_t row = tid;  // 0..127
        const uint32_t lane_addr = (warp * 32u) << 16;
        const bool softcap = a.logit_softcap > 0.0f;
        const float scale2 = softcap ? a.sm_scale : a.sm_scale * kLog2ePf;
        const uint32_t q_pos = qt.pos0 + min(row, tile_rows - 1u);  // absolute position
        float m_used = -INFINITY, l_run = 0.0f;
        bool ok = true;
        for (uint32_t j = 0; j < n_tiles; ++j) {
            if (*abort_flag) { ok = false; break; }
            ok = warp_wait(&s_full[j & 1u], (j >> 1) & 1u);
            if (!ok) break;
            tc_fence_after();
            const uint32_t s_addr = tmem_base + lane_addr + ((j & 1u) ? COL_S1 : COL_S0);
            const uint32_t key0 = j * kKvTile;
            const bool diag = key0 + kKvTile - 1u > qt.pos0;  // some row of the tile masks some key
            // pass 1: row maximum
            float m_tile = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld32(s_addr + c * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    float s = __uint_as_float(r[i]) * scale2;
                    if (softcap) s = tanhf(fminf(fmaxf(s / a.logit_softcap, -15.0f), 15.0f)) * a.logit_softcap * kLog2ePf;
                    const uint32_t key = key0 + c * 32 + i;
                    if (diag && key > q_pos) s = -INFINITY;
                    m_tile = fmaxf(m_tile, s);
                }
            }
            // the previous P.V must be complete before P is overwritten or O rescaled
            if (j > 0) {
                ok = warp_wait(pv_done, (j - 1u) & 1u);
                if (!ok) break;
                tc_fence_after();
            }
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
                    tmem_ld32(tmem_base + lane_addr + COL_O + c * 32, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                    tmem_st32(tmem_base + lane_addr + COL_O + c * 32, r);
                }
                tmem_wait_st();
            }
            // pass 2: probabilities -> P tile (storage dtype, swizzled K-major), row sum
            float psum = 0.0f;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld32(s_addr + c * 32, r);
                tmem_wait_ld();
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float s0 = __uint_as_float(r[i]) * scale2, s1 = __uint_as_float(r[i + 1]) * scale2;
                    if (softcap) {
                        s0 = tanhf(fminf(fmaxf(s0 / a.logit_softcap, -15.0f), 15.0f)) * a.logit_softcap * kLog2ePf;
                        s1 = tanhf(fminf(fmaxf(s1 / a.logit_softcap, -15.0f), 15.0f)) * a.logit_softcap * kLog2ePf;
                    }
                    const uint32_t key = key0 + c * 32 + i;
                    float p0 = fast_exp2(s0 - m_used), p1 = fast_exp2(s1 - m_used);
                    if (diag && key > q_pos) p0 = 0.0f;
                    if (diag && key + 1u > q_pos) p1 = 0.0f;
                    const uint16_t b0 = T::store(p0), b1 = T::store(p1);
                    // the sum uses the rounded probabilities, so that numerator and denominator agree
                    psum += T::load(b0) + T::load(b1);
                    packed[i >> 1] = uint32_t(b0) | (uint32_t(b1) << 16);
                }
                // 32 keys = 64 B = four 16-byte chunks of this row; chunk index inside the 64-key panel
                const uint32_t panel = uint32_t(c) >> 1;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const uint32_t cc = (uint32_t(c) & 1u) * 4u + q4;
                    *reinterpret_cast<uint4*>(sP + panel * PANEL_BYTES + row * 128u + ((cc ^ (row & 7u)) << 4)) =
                        make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
                }
            }
            l_run = l_run * alpha + psum;
            // slots past the end of the sequence may hold anything: their V rows must not reach the MMA
            if ((j + 1u) * kKvTile > seq_end) {
                const uint32_t stage = j & 1u;
                const uint32_t first_bad = seq_end > key0 ? seq_end - key0 : 0u;
                const uint32_t end_row = min(uint32_t(kKvTile), ((seq_end + kPagePf - 1) / kPagePf) * kPagePf - min(key0, ((seq_end + kPagePf - 1) / kPagePf) * kPagePf));
                for (uint32_t i = first_bad * 8u + row; i < end_row * 8u; i += 128u) {
                    const uint32_t rr = i >> 3, ch = i & 7u;
#pragma unroll
                    for (int p = 0; p < PANELS; ++p)
                        *reinterpret_cast<uint4*>(sV + stage * KV_BYTES + p * PANEL_BYTES + rr * 128u + (ch << 4)) =
                            make_uint4(0u, 0u, 0u, 0u);
                }
            }
            tc_fence_before();
            fence_async_smem();
            mbar_arrive(p_ready);
        }
        if (ok && n_tiles > 0) {
            ok = warp_wait(pv_done, (n_tiles - 1u) & 1u);
            if (ok) {
                tc_fence_after();
                const float inv_l = 1.0f / fmaxf(l_run, 1e-12f);
                uint16_t* og = reinterpret_cast<uint16_t*>(a.out) + (size_t(tile_start + row) * a.num_q_heads + q_head) * D;
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + lane_addr + COL_O + c * 32, r);
                    tmem_wait_ld();
                    if (row < tile_rows) {
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            uint32_t w[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float x0 = __uint_as_float(r[q4 * 8 + 2 * i]) * inv_l;
                                const float x1 = __uint_as_float(r[q4 * 8 + 2 * i + 1]) * inv_l;
                                w[i] = uint32_t(T::store(x0)) | (uint32_t(T::store(x1)) << 16);
                            }
                            *reinterpret_cast<uint4*>(og + c * 32 + q4 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
        }
        if (!ok && lane == 0) {
            atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            *abort_flag = 1;
        }
    }

    // ---- teardown: every thread gets here; TMEM is returned by the warp that took it ------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int D, typename T>
cudaError_t launch_prefill_t(const KriyaPrefillArgs& a, const CUtensorMap& mk, const CUtensorMap& mv, int max_smem_optin,
                             cudaStream_t s) {
    constexpr int PANELS = D / 64;
    const size_t smem = size_t(PANELS) * 128 * 128 * 5 + 2 * 128 * 128 + 256 + 1024;
    if (smem > size_t(max_smem_optin)) return cudaErrorInvalidValue;
    auto kern = prefill_kernel<D, T>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    PrefillParams pp;
    pp.a = a;
    pp.q_tiles = a.n_tiles;
    pp.dtype = T::kDtype;
    kern<<<pp.q_tiles * a.num_q_heads, kPrefillThreads, smem, s>>>(mk, mv, pp);
    return cudaGetLastError();
}

}  // namespace kriya

bool kriya_prefill_supported(uint32_t head_dim, uint32_t group, uint32_t block_size, uint32_t dtype) {
    (void)dtype;
    return (head_dim == 64 || head_dim == 128) && group >= 1 && block_size == uint32_t(kriya::kPagePf);
}

// Encodes the 2-D tensor maps over the K and V pools (all layers): rows = (layer, block, token), columns =
// (kv head, d); box = 64 columns x 16 rows with the 128-byte swizzle the MMA descriptors expect.
cudaError_t kriya_prefill_encode_maps(void* pool_k, void* pool_v, uint64_t total_rows, uint32_t row_elems,
                                      void* out_map_k, void* out_map_v) {
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess) return e;
    if (fn == nullptr || qres != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
    const cuuint64_t dims[2] = {row_elems, total_rows};
    const cuuint64_t strides[1] = {cuuint64_t(row_elems) * 2};
    const cuuint32_t box[2] = {64, uint32_t(kriya::kPagePf)};
    const cuuint32_t estr[2] = {1, 1};
    void* pools[2] = {pool_k, pool_v};
    void* outs[2] = {out_map_k, out_map_v};
    for (int i = 0; i < 2; ++i) {
        const CUresult r = reinterpret_cast<EncodeFn>(fn)(
            static_cast<CUtensorMap*>(outs[i]), CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, pools[i], dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    return cudaSuccess;
}

cudaError_t kriya_launch_prefill(const KriyaPrefillArgs& a, uint32_t head_dim, uint32_t block_size, uint32_t dtype,
                                 int max_smem_optin, cudaStream_t s) {
    if (a.n_tiles == 0) return cudaSuccess;
    if (!kriya_prefill_supported(head_dim, a.num_q_heads / a.num_kv_heads, block_size, dtype) || !a.map_k || !a.map_v)
        return cudaErrorInvalidValue;
    const CUtensorMap& mk = *static_cast<const CUtensorMap*>(a.map_k);
    const CUtensorMap& mv = *static_cast<const CUtensorMap*>(a.map_v);
    using namespace kriya;
    if (head_dim == 128)
        return dtype == KRIYA_DTYPE_FP16 ? launch_prefill_t<128, Fp16>(a, mk, mv, max_smem_optin, s)
                                         : launch_prefill_t<128, Bf16>(a, mk, mv, max_smem_optin, s);
    return dtype == KRIYA_DTYPE_FP16 ? launch_prefill_t<64, Fp16>(a, mk, mv, max_smem_optin, s)
                                     : launch_prefill_t<64, Bf16>(a, mk, mv, max_smem_optin, s);
}
