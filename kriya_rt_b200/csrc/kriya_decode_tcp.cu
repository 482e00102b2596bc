// Paged GQA decode attention on the tensor cores, whole pages per copy: head_dim 128, two KV heads, 16-token pages (the job
// of bsr_paged_gqa_decode_stage1 and bsr_paged_gqa_split_k_reduce, kernels/metal/paged_gqa_and_deltanet.metal:242-495,
// 1474-1525; the shape of the Qwen2.5 family this path is measured on).
//
// Why a second tensor-core kernel.  The kernel of kriya_decode_tc.cu gathers one KV head of one page with four tensor
// copies of 2 KB; a B200 SM sustains about 50 GB/s of such copies however few SMs are streaming, and copies of 8 KB
// about twice that.  One page of this cache, [16 tokens][2 heads][128 d], is 8 KB of contiguous memory, so this kernel
// moves a page - both heads - with ONE copy and lets one CTA process both KV heads of a row together.
//
// Layout trick.  The copy goes through a 5-D tensor map over the pool with the dimensions permuted,
//   {64 d_lo, 16 tokens (512 B apart), 2 halves of d (128 B), 2 heads (256 B), pages (8 KB)},  box = one page,
// so a page lands in shared memory as four planes (head, half) of [16 tokens][128 B], 64 rows of 128 bytes with the
// 128-byte swizzle: a valid K-major MMA operand whose rows are (head, half, token) triples.  Two pages are 128 such
// rows = one M = 128 MMA.  The query operand has N = 32 rows (half', query head j), so the accumulator entry
//   S'[(h, p, t)][(p', j)] = sum over the 64 d of half p of  K[t][h][.] * Q[j][half p'][.]
// is a useful partial score when p' = p and j belongs to KV head h; the score of (t, j) is the sum of the entries of rows
// (h, 0, t) and (h, 1, t), which sit in lanes l and l + 16 of one warp: one shuffle.  The same rows are the K dimension
// of the second MMA:  O'[d_lo][(p', j)] += sum over rows of V[row][d_lo] * P[(p', j)][row], where the probability
// operand P holds p(t, j) at rows (h(j), p', t) and zeros elsewhere - the zero pattern never changes, every thread
// rewrites only its own eight entries per tile.  O' has M = 64 (d_lo) and N = 32: O[j][64 p' + d_lo].
//
// Roles (256 threads, one CTA per SM, persistent over a list of run pieces exactly as in kriya_decode_tc.cu):
//   warps 0-3 softmax (warp w: page w / 2 of the tile, KV head w % 2; lane: half = lane / 16, token = lane % 16),
//   warp 4 producer (page indices, tensor copies into a 6-deep ring of 32 KB tiles: 2 pages of K, 2 pages of V),
//   warp 5 MMA issuer, warp 6 scratch-set guard, warp 7 stager (queries, rotated in flight; the new token's K/V row).
// Split runs, the finishing piece, stamps and the set guard work as described in kriya_decode_tc.cu; a run here is a
// whole plan row (both KV heads).  Every wait is bounded.
#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>

#include "kriya_tc.cuh"

namespace kriya {
namespace tcp {

constexpr int kD = 128;
constexpr int kPage = 16;
constexpr int kHkv = 2;
constexpr int kHqMax = 16;                       // query heads of a row: up to 8 per KV head
constexpr int kPagesPerTile = 2;                 // 2 pages x 64 rows = 128 operand rows
constexpr int kTileTokens = kPagesPerTile * kPage;
constexpr uint32_t kPageBytes = 8192;            // one page of K (or V), both heads
constexpr uint32_t kTileKBytes = kPagesPerTile * kPageBytes;  // 16 KB
constexpr uint32_t kStageBytes = 2 * kTileKBytes;             // K tile + V tile
constexpr int kStages = 6;
constexpr int kQBufs = 3;
constexpr uint32_t kQBytes = 32 * 128;           // 32 operand rows (half', head) x 128 B
constexpr uint32_t kPBytes = 2 * 32 * 128;       // two 64-row K blocks x 32 operand rows x 128 B
constexpr int kThreads = 256;
constexpr int kN = 32;
constexpr uint32_t kTmemCols = 128;
constexpr uint32_t kColS0 = 0, kColS1 = 32, kColO = 64;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescale = 8.0f;

struct Params {
    KriyaDecodeArgs a;
    const KriyaTcSeg* segs;
    const uint32_t* cta_seg_ptr;  // [grid + 1]
    uint32_t page0;               // index of the layer's first page inside the all-layer tensor map
    uint32_t late_parts;
    uint32_t n_seg;
    uint2* ll_o;                  // [slot][Hq][128] (value, stamp)
    uint2* ll_ml;                 // [slot][Hq][2]
    uint32_t* set_done;
    uint32_t done_expect;
    uint32_t epoch;
    KriyaFusedAppend f;
};

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_previous_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void named_bar_sync_128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ bool bar_or_128(bool pred) {
    uint32_t res;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.or.pred p, 1, 128, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(res)
        : "r"(uint32_t(pred))
        : "memory");
    return res != 0;
}
__device__ __forceinline__ void ll_store(uint2* p, float v, uint32_t epoch) {
    asm volatile("st.global.cg.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(epoch) : "memory");
}
__device__ __forceinline__ uint2 ll_load(const uint2* p) {
    uint2 r;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p) : "memory");
    return r;
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
    uint32_t r;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(r) : "l"(p) : "memory");
    return r;
}
__device__ __forceinline__ bool warp_wait_l(uint64_t limit_ns, uint64_t* bar, uint32_t parity) { return warp_wait(bar, parity, limit_ns); }
__device__ __forceinline__ bool wait_set_free(const uint32_t* set_done, uint32_t done_expect, uint64_t wait_ns) {
    const uint64_t t_start = global_timer_ns();
    for (uint32_t spin = 0;; ++spin) {
        if (int32_t(ld_volatile_u32(set_done) - done_expect) >= 0) return true;
        if ((spin & 63u) == 63u && global_timer_ns() - t_start > wait_ns) return false;
    }
}
// One whole page through the permuted 5-D map: coordinates (d_lo, token, half, head, page) = (0, 0, 0, 0, page).
__device__ __forceinline__ void tma_load_page(void* dst_smem, const CUtensorMap* map, int32_t page, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %2, %2, %2, %3}], [%4];" ::"r"(
            smem_u32(dst_smem)),
        "l"(map), "r"(0), "r"(page), "r"(smem_u32(bar))
        : "memory");
}
// 8 consecutive TMEM columns of this thread's lane.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

// RoPE of eight (x[i], x[i + 64]) pairs held as two 16-byte chunks, in the operation order of the append kernel
// (fma(x0, c, -(x1 * s)), fma(x0, s, x1 * c), round to nearest even), so both paths write identical bits.
__device__ __forceinline__ void rope8_coeffs(float2 (&cs)[8], uint32_t first_pair, uint32_t position, const KriyaFusedAppend& f) {
    const uint32_t half_rot = f.rotary_dim / 2u;
    const bool use_table = f.has_table != 0u && position < f.max_seq_len && f.table != nullptr;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t i = first_pair + j;
        cs[j] = make_float2(1.0f, 0.0f);
        if (i < half_rot) {
            if (use_table) {
                cs[j] = reinterpret_cast<const float2*>(f.table)[size_t(position) * half_rot + i];
            } else {
                const float freq_exp = float(2u * i) / float(f.rotary_dim);
                const float inv_freq = powf(f.rope_theta, -freq_exp);
                const float angle = __fmul_rn(float(position), inv_freq);
                cs[j] = make_float2(cosf(angle), sinf(angle));
            }
        }
    }
}
template <typename T>
__device__ __forceinline__ void rope8_apply(uint4& lo, uint4& hi, uint32_t first_pair, const float2 (&cs)[8], uint32_t half_rot) {
    uint32_t* lw = reinterpret_cast<uint32_t*>(&lo);
    uint32_t* hw = reinterpret_cast<uint32_t*>(&hi);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint16_t l2[2] = {uint16_t(lw[j] & 0xFFFFu), uint16_t(lw[j] >> 16)};
        uint16_t h2[2] = {uint16_t(hw[j] & 0xFFFFu), uint16_t(hw[j] >> 16)};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            if (first_pair + 2 * j + e < half_rot) {
                const float c = cs[2 * j + e].x, sn = cs[2 * j + e].y;
                const float x0 = T::load(l2[e]), x1 = T::load(h2[e]);
                l2[e] = T::store(__fmaf_rn(x0, c, -__fmul_rn(x1, sn)));
                h2[e] = T::store(__fmaf_rn(x0, sn, __fmul_rn(x1, c)));
            }
        }
        lw[j] = uint32_t(l2[0]) | (uint32_t(l2[1]) << 16);
        hw[j] = uint32_t(h2[0]) | (uint32_t(h2[1]) << 16);
    }
}

// The run's last piece gathers the other pieces' states (two at a time) and finishes the run.  Thread t owns output
// dimension t of all HQ query heads.
template <int HQ>
__device__ __forceinline__ bool gather_merge(const uint2* __restrict__ ll_o, const uint2* __restrict__ ll_ml, const KriyaTcSeg& seg,
                                             uint32_t epoch, uint64_t wait_ns, float* stage, uint32_t t, float (&M)[HQ], float (&L)[HQ], float (&O)[HQ]) {
    const uint32_t others = seg.n_parts - 1u;
    for (uint32_t c0 = 0; c0 < others; c0 += 2u) {
        const uint32_t cnt = min(2u, others - c0);
        const size_t slot0 = size_t(seg.first_slot) + c0;
        uint2 w[2][HQ];
        uint2 mlw = make_uint2(0u, epoch);
        const bool has_ml = t < cnt * uint32_t(HQ) * 2u;  // (m, l) words of the chunk: [part][head][2], one per thread
        const uint2* mlp = &ll_ml[slot0 * HQ * 2 + (has_ml ? t : 0u)];
        bool got = false;
        const uint64_t t_start = global_timer_ns();
        for (uint32_t spin = 0; !got; ++spin) {
#pragma unroll
            for (int s2 = 0; s2 < 2; ++s2)
#pragma unroll
                for (int h = 0; h < HQ; ++h) w[s2][h] = ll_load(&ll_o[((slot0 + min(uint32_t(s2), cnt - 1u)) * HQ + h) * kD + t]);
            mlw = ll_load(mlp);
            uint32_t bad = mlw.y ^ epoch;
#pragma unroll
            for (int s2 = 0; s2 < 2; ++s2)
#pragma unroll
                for (int h = 0; h < HQ; ++h) bad |= w[s2][h].y ^ epoch;
            got = bad == 0u;
            if (!got && (spin & 63u) == 63u && global_timer_ns() - t_start > wait_ns) break;
        }
        if (has_ml) stage[t] = __uint_as_float(mlw.x);
        if (bar_or_128(!got)) return false;
#pragma unroll
        for (int h = 0; h < HQ; ++h) {
            float mc = M[h];
#pragma unroll
            for (int s2 = 0; s2 < 2; ++s2)
                if (uint32_t(s2) < cnt) mc = fmaxf(mc, stage[(s2 * HQ + h) * 2]);
            if (mc == -INFINITY) continue;
            const float keep = (M[h] == -INFINITY) ? 0.0f : exp2f(M[h] - mc);
            float lacc = L[h] * keep, oacc = O[h] * keep;
#pragma unroll
            for (int s2 = 0; s2 < 2; ++s2) {
                if (uint32_t(s2) < cnt) {
                    const float ms = stage[(s2 * HQ + h) * 2];
                    const float wgt = (ms == -INFINITY) ? 0.0f : exp2f(ms - mc);
                    lacc = fmaf(wgt, stage[(s2 * HQ + h) * 2 + 1], lacc);
                    oacc = fmaf(wgt, __uint_as_float(w[s2][h].x), oacc);
                }
            }
            M[h] = mc;
            L[h] = lacc;
            O[h] = oacc;
        }
        named_bar_sync_128();
    }
    return true;
}

// G = query heads per KV head (1..8); the row has HQ = 2 G query heads.
template <int G, typename T>
__global__ void __launch_bounds__(kThreads, 1)
decode_tcp_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, Params pp) {
    constexpr int HQ = kHkv * G;
    constexpr uint32_t FMT = (T::kDtype == KRIYA_DTYPE_BF16) ? 1u : 0u;
    constexpr uint32_t IDESC_S = make_idesc(FMT, 128, kN, 0, 0);  // A = K tile rows (K-major), B = Q rows (K-major)
    constexpr uint32_t IDESC_O = make_idesc(FMT, 64, kN, 1, 0);   // A = V tile (MN-major: M = d_lo), B = P (K-major)

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
    uint8_t* sKV = sm;                                  // [stages][K tile 16 KB | V tile 16 KB]
    uint8_t* sQ = sKV + kStages * kStageBytes;          // [3][4 KB]
    uint8_t* sP = sQ + kQBufs * kQBytes;                // [2][8 KB]; at the end of a piece also the [HQ][128] fp32 output staging
    float* red = reinterpret_cast<float*>(sP + 2 * kPBytes);  // [4 warps][8] maxima / sums, merge staging [2][HQ][2]
    float* alpha_s = red + 128;                         // [16] rescale factors per query head
    float* ml_s = alpha_s + 16;                         // [16][2] (m, l) of the piece per query head
    uint64_t* bars = reinterpret_cast<uint64_t*>(ml_s + 32);
    uint64_t* kv_full = bars;                     // [stages]
    uint64_t* kv_empty = bars + kStages;          // [stages]
    uint64_t* s_full = bars + 2 * kStages;        // [2]
    uint64_t* p_ready = bars + 2 * kStages + 2;   // [2], 128 arrivals
    uint64_t* pv_done = bars + 2 * kStages + 4;   // [2]
    uint64_t* q_ready = bars + 2 * kStages + 6;   // [3]
    uint64_t* q_free = bars + 2 * kStages + 9;    // [3]
    uint64_t* kv_ready = bars + 2 * kStages + 12; // [3]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 15);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* set_free_s = tmem_slot + 2;
    KriyaTcSeg* segs_s = reinterpret_cast<KriyaTcSeg*>(tmem_slot + 4);  // first 8 segment records of this CTA

    const KriyaDecodeArgs& a = pp.a;
    const uint64_t wait_ns = a.wait_ns;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t seg_begin = pp.cta_seg_ptr[blockIdx.x], seg_end = pp.cta_seg_ptr[blockIdx.x + 1];
    if (threadIdx.x == 0) pdl_launch_dependents();
    if (seg_begin == seg_end) {
        if (threadIdx.x == 0) {
            if (!wait_set_free(pp.set_done, pp.done_expect, pp.a.wait_ns)) atomicMax(pp.a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            atomicAdd(pp.set_done, 1u);
        }
        return;
    }
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&kv_full[s], 1);
            mbar_init(&kv_empty[s], 1);
        }
        mbar_init(&s_full[0], 1);
        mbar_init(&s_full[1], 1);
        mbar_init(&p_ready[0], 128);
        mbar_init(&p_ready[1], 128);
        mbar_init(&pv_done[0], 1);
        mbar_init(&pv_done[1], 1);
        for (int b = 0; b < 3; ++b) {
            mbar_init(&q_ready[b], 1);
            mbar_init(&q_free[b], 1);
            mbar_init(&kv_ready[b], 1);
        }
        *abort_flag = 0;
        *set_free_s = 0;
        mbar_fence_init();
    }
    if (warp == 5) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    {
        const uint32_t nstage = min(seg_end - seg_begin, 8u) * uint32_t(sizeof(KriyaTcSeg) / 4);
        const uint32_t* src = reinterpret_cast<const uint32_t*>(pp.segs + seg_begin);
        for (uint32_t i = tid; i < nstage; i += kThreads) reinterpret_cast<uint32_t*>(segs_s)[i] = src[i];
    }
    auto seg_at = [&](uint32_t si) -> KriyaTcSeg { return (si - seg_begin < 8u) ? segs_s[si - seg_begin] : pp.segs[si]; };
    // Query rows of heads that do not exist (G < 8) and every probability entry outside a thread's own eight stay zero.
    for (uint32_t i = tid; i < (kQBufs * kQBytes + 2 * kPBytes) / 16; i += kThreads)
        reinterpret_cast<uint4*>(sQ)[i] = make_uint4(0u, 0u, 0u, 0u);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t Hq = a.num_q_heads;
    const uint32_t pdl = pp.f.overlap_previous;  // see kriya_decode_tc.cu
    if (pdl == 1u) pdl_wait_previous_grid();

    if (warp == 4) {
        // ---- producer ------------------------------------------------------------------------------------
        uint32_t g = 0, runs = 0;
        bool ok = true;
        const bool fused = pp.f.k_in != nullptr;
        for (uint32_t si = seg_begin; si < seg_end && ok; ++si) {
            const KriyaTcSeg seg = seg_at(si);
            if (seg.blk_hi <= seg.blk_lo) continue;
            const uint32_t t0 = seg.blk_lo / kPagesPerTile, t1 = (seg.blk_hi + kPagesPerTile - 1) / kPagesPerTile;
            const int32_t* table = a.indices + seg.tbl_off;
            const bool owns_last = fused && seg.row_tokens > 0u && uint64_t(seg.blk_hi) * kPage >= seg.row_tokens;
            int32_t pf_blk = 0;
            bool pf_valid = false;
            for (uint32_t t = t0; t < t1; ++t, ++g) {
                if (*abort_flag) { ok = false; break; }
                const uint32_t stage = g % kStages;
                const uint32_t p_lo = max(t * kPagesPerTile, seg.blk_lo), p_hi = min((t + 1) * kPagesPerTile, seg.blk_hi);
                const uint32_t npages = p_hi - p_lo;
                const uint32_t my_page = p_lo + lane;
                int32_t blk = pf_blk;
                if (!pf_valid && lane < npages) blk = table[my_page];
                if (g >= kStages && !warp_wait_l(wait_ns, &kv_empty[stage], ((g / kStages) - 1u) & 1u)) { ok = false; break; }
                if (owns_last && t + 1u == t1 && !warp_wait_l(wait_ns, &kv_ready[runs % uint32_t(kQBufs)], (runs / uint32_t(kQBufs)) & 1u)) {
                    ok = false;
                    break;
                }
                if (lane < npages && uint32_t(blk) >= a.num_blocks) {
                    atomicMax(a.status, uint32_t(KRIYA_DEV_BAD_BLOCK_INDEX));
                    blk = 0;
                }
                if (lane == 0) mbar_arrive_expect_tx(&kv_full[stage], npages * 2u * kPageBytes);
                __syncwarp();
                if (lane < npages) {
                    uint8_t* dst = sKV + stage * kStageBytes + (my_page - t * kPagesPerTile) * kPageBytes;
                    const int32_t page = int32_t(pp.page0) + blk;
                    tma_load_page(dst, &map_k, page, &kv_full[stage]);
                    tma_load_page(dst + kTileKBytes, &map_v, page, &kv_full[stage]);
                }
                pf_valid = t + 1u < t1;
                if (pf_valid) {
                    const uint32_t n_lo = (t + 1u) * kPagesPerTile, n_hi = min((t + 2u) * kPagesPerTile, seg.blk_hi);
                    pf_blk = (n_lo + lane < n_hi) ? table[n_lo + lane] : 0;
                }
            }
            ++runs;
        }
        if (!ok && lane == 0) {
            atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            *abort_flag = 1;
        }
    } else if (warp == 7) {
        // ---- stager: per run piece the query operand (32 rows: (half, head)) and the new token's K/V row -----------
        uint32_t runs = 0;
        bool ok = true;
        const bool fused = pp.f.k_in != nullptr;
        if (pdl == 3u) pdl_wait_previous_grid();
        for (uint32_t si = seg_begin; si < seg_end && ok; ++si) {
            const KriyaTcSeg seg = seg_at(si);
            if (seg.blk_hi <= seg.blk_lo) continue;
            if (*abort_flag) break;
            if (runs >= uint32_t(kQBufs) && !warp_wait_l(wait_ns, &q_free[runs % uint32_t(kQBufs)], ((runs / uint32_t(kQBufs)) - 1u) & 1u)) {
                ok = false;
                break;
            }
            const int32_t* table = a.indices + seg.tbl_off;
            const bool owns_last = fused && seg.row_tokens > 0u && uint64_t(seg.blk_hi) * kPage >= seg.row_tokens;
            uint8_t* qb = sQ + (runs % uint32_t(kQBufs)) * kQBytes;
            const uint16_t* qg = reinterpret_cast<const uint16_t*>(a.q) + size_t(seg.req) * Hq * kD;
            // item i = (query head i / 8, 16-byte chunk c = i % 8 of the first half of d; its partner chunk is c + 8); a
            // lane's items all share c = lane % 8.  Head j of the row sits in operand row 8 * (j / G) + j % G.
            constexpr int ITEMS = (HQ * 8 + 31) / 32;
            const uint32_t c = lane & 7u;
            float2 cs[8];
            if (fused) {
                const uint32_t position = pp.f.positions_are_context ? seg.row_tokens - 1u : pp.f.positions[seg.req];
                rope8_coeffs(cs, c * 8u, position, pp.f);
            }
            uint4 lo[ITEMS], hi[ITEMS];
#pragma unroll
            for (int it = 0; it < ITEMS; ++it) {
                const uint32_t j = (lane + 32u * it) >> 3;
                if (j < uint32_t(HQ)) {
                    lo[it] = *reinterpret_cast<const uint4*>(qg + j * kD + c * 8);
                    hi[it] = *reinterpret_cast<const uint4*>(qg + j * kD + 64 + c * 8);
                }
            }
#pragma unroll
            for (int it = 0; it < ITEMS; ++it) {
                const uint32_t j = (lane + 32u * it) >> 3;
                if (j < uint32_t(HQ)) {
                    if (fused) rope8_apply<T>(lo[it], hi[it], c * 8u, cs, pp.f.rotary_dim / 2u);
                    const uint32_t row = 8u * (j / uint32_t(G)) + j % uint32_t(G);
                    *reinterpret_cast<uint4*>(qb + row * 128u + ((c ^ (row & 7u)) << 4)) = lo[it];
                    *reinterpret_cast<uint4*>(qb + 2048u + row * 128u + ((c ^ (row & 7u)) << 4)) = hi[it];
                    if (fused && owns_last && pp.f.q_rope_out != nullptr) {
                        uint16_t* qo = reinterpret_cast<uint16_t*>(pp.f.q_rope_out) + (size_t(seg.req) * Hq + j) * kD;
                        *reinterpret_cast<uint4*>(qo + c * 8) = lo[it];
                        *reinterpret_cast<uint4*>(qo + 64 + c * 8) = hi[it];
                    }
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&q_ready[runs % uint32_t(kQBufs)]);
            if (owns_last) {
                const uint32_t tok = seg.row_tokens - 1u;
                const uint32_t blk = uint32_t(table[tok / kPage]);
                if (blk >= a.num_blocks) {
                    if (lane == 0) atomicMax(a.status, uint32_t(KRIYA_DEV_BAD_BLOCK_INDEX));
                } else {
                    const size_t off = (size_t(blk) * kPage + tok % kPage) * kHkv * kD;  // the token's row: [head][d]
                    const size_t src = size_t(seg.req) * kHkv * kD;
                    uint16_t* kd = reinterpret_cast<uint16_t*>(pp.f.cache_k_w) + off;
                    uint16_t* vd = reinterpret_cast<uint16_t*>(pp.f.cache_v_w) + off;
                    const uint16_t* ks = reinterpret_cast<const uint16_t*>(pp.f.k_in) + src;
                    const uint16_t* vs = reinterpret_cast<const uint16_t*>(pp.f.v_in) + src;
                    if (lane < 16u) {  // key: head lane / 8, chunk lane % 8 and its partner; the coefficients above apply
                        const uint32_t hd = lane >> 3;
                        uint4 klo = *reinterpret_cast<const uint4*>(ks + hd * kD + c * 8);
                        uint4 khi = *reinterpret_cast<const uint4*>(ks + hd * kD + 64 + c * 8);
                        rope8_apply<T>(klo, khi, c * 8u, cs, pp.f.rotary_dim / 2u);
                        *reinterpret_cast<uint4*>(kd + hd * kD + c * 8) = klo;
                        *reinterpret_cast<uint4*>(kd + hd * kD + 64 + c * 8) = khi;
                    }
                    // value: 2 heads x 16 chunks, one per lane, bit for bit
                    *reinterpret_cast<uint4*>(vd + lane * 8) = *reinterpret_cast<const uint4*>(vs + lane * 8);
                }
                __threadfence();
                asm volatile("fence.proxy.async.global;" ::: "memory");
                __syncwarp();
            }
            if (lane == 0) mbar_arrive(&kv_ready[runs % uint32_t(kQBufs)]);
            ++runs;
        }
        if (!ok && lane == 0) {
            atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            *abort_flag = 1;
        }
    } else if (warp == 5) {
        // ---- MMA issuer ---------------------------------------------------------------------------------
        const uint32_t kv_addr = smem_u32(sKV), q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
        auto issue_s = [&](uint32_t gg, uint32_t qbuf) {
            const uint32_t stage = gg % kStages;
            const uint32_t d_tmem = tmem_base + ((gg & 1u) ? kColS1 : kColS0);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {  // 64 d of a half = 4 steps of 16
                const uint32_t a_off = stage * kStageBytes + uint32_t(ks) * 32u;
                const uint32_t b_off = qbuf * kQBytes + uint32_t(ks) * 32u;
                umma_f16(d_tmem, smem_desc_sw128(kv_addr + a_off, 16, 1024), smem_desc_sw128(q_addr + b_off, 16, 1024), IDESC_S,
                         ks > 0 ? 1u : 0u);
            }
            umma_commit(&s_full[gg & 1u]);
        };
        uint32_t g = 0;
        bool ok = true;
        uint32_t la_si = seg_begin, la_t = 0, la_t1 = 0, la_g = 0, la_run = 0;
        bool la_first = true;
        auto la_load = [&]() {
            while (la_si < seg_end) {
                const KriyaTcSeg s2 = seg_at(la_si);
                if (s2.blk_hi > s2.blk_lo) {
                    la_t = s2.blk_lo / kPagesPerTile;
                    la_t1 = (s2.blk_hi + kPagesPerTile - 1) / kPagesPerTile;
                    la_first = true;
                    return true;
                }
                ++la_si;
            }
            return false;
        };
        bool la_valid = la_load();
        auto la_issue = [&]() -> bool {
            if (!la_valid) return true;
            if (!warp_wait_l(wait_ns, &kv_full[la_g % kStages], (la_g / kStages) & 1u)) return false;
            if (la_first) {
                if (!warp_wait_l(wait_ns, &q_ready[la_run % uint32_t(kQBufs)], (la_run / uint32_t(kQBufs)) & 1u)) return false;
                la_first = false;
            }
            tc_fence_after();
            if (lane == 0) issue_s(la_g, la_run % uint32_t(kQBufs));
            __syncwarp();
            ++la_g;
            if (++la_t >= la_t1) {
                if (lane == 0) umma_commit(&q_free[la_run % uint32_t(kQBufs)]);
                __syncwarp();
                ++la_si;
                ++la_run;
                la_valid = la_load();
            }
            return true;
        };
        ok = la_issue();
        for (uint32_t si = seg_begin; si < seg_end && ok; ++si) {
            const KriyaTcSeg seg = seg_at(si);
            if (seg.blk_hi <= seg.blk_lo) continue;
            const uint32_t t0 = seg.blk_lo / kPagesPerTile, t1 = (seg.blk_hi + kPagesPerTile - 1) / kPagesPerTile;
            for (uint32_t t = t0; t < t1 && ok; ++t, ++g) {
                if (*abort_flag) { ok = false; break; }
                ok = la_issue();
                if (!ok) break;
                ok = warp_wait_l(wait_ns, &p_ready[g & 1u], (g >> 1) & 1u);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t stage = g % kStages;
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {  // 128 operand rows = 8 steps of 16
                        const uint32_t a_off = stage * kStageBytes + kTileKBytes + uint32_t(ks) * 2048u;
                        const uint32_t b_off = (g & 1u) * kPBytes + uint32_t(ks / 4) * 4096u + uint32_t(ks % 4) * 32u;
                        umma_f16(tmem_base + kColO, smem_desc_sw128(kv_addr + a_off, 8192, 1024), smem_desc_sw128(p_addr + b_off, 16, 1024),
                                 IDESC_O, (t > t0 || ks > 0) ? 1u : 0u);
                    }
                    umma_commit(&kv_empty[stage]);
                    umma_commit(&pv_done[g & 1u]);
                }
                __syncwarp();
            }
        }
        if (!ok && lane == 0) {
            atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            *abort_flag = 1;
        }
    } else if (warp == 6) {
        // ---- scratch-set guard (see kriya_decode_tc.cu) -------------------------------------------------------
        if (lane == 0) {
            const bool free_now = wait_set_free(pp.set_done, pp.done_expect, pp.a.wait_ns);
            if (!free_now) atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            __threadfence_block();
            *set_free_s = free_now ? 1u : 2u;
        }
    } else {
        // ---- softmax warps: warp w = (page w / 2 of the tile, KV head w % 2); lane = (half lane / 16, token lane % 16) -----
        const uint32_t lane_addr = (warp * 32u) << 16;
        const uint32_t hd = warp & 1u, pg = warp >> 1, half = lane >> 4, tk = lane & 15u;
        const bool softcap = a.logit_softcap > 0.0f;
        const float scale2 = softcap ? a.sm_scale : a.sm_scale * kLog2e;
        const bool state_mode = a.state_o != nullptr;
        // this thread's eight probability entries of a tile: operand row n = 16 half + 8 hd + jj, element k = 32 warp + lane
        const uint32_t k_in = (warp & 1u) * 32u + lane;  // position inside the 64-row K block (block = page of the tile)
        uint32_t p_off[G];
#pragma unroll
        for (int jj = 0; jj < G; ++jj) {
            const uint32_t n = 16u * half + 8u * hd + uint32_t(jj);
            p_off[jj] = pg * 4096u + n * 128u + ((((k_in >> 3) ^ (n & 7u)) << 4) | ((k_in & 7u) << 1));
        }
        uint32_t g = 0;
        bool ok = true;
        bool set_known = false;
        for (uint32_t si = seg_begin; si < seg_end && ok; ++si) {
            const KriyaTcSeg seg = seg_at(si);
            const uint32_t req = seg.req;
            const uint32_t row_tokens = seg.row_tokens;
            const uint32_t tok_lo = max(seg.blk_lo * kPage, seg.tok_first), tok_hi = min(seg.blk_hi * kPage, row_tokens);
            const uint32_t t0 = seg.blk_lo / kPagesPerTile, t1 = (seg.blk_hi + kPagesPerTile - 1) / kPagesPerTile;
            const bool empty = seg.blk_hi <= seg.blk_lo;
            float m_used[G], l_lane[G];
#pragma unroll
            for (int jj = 0; jj < G; ++jj) {
                m_used[jj] = -INFINITY;
                l_lane[jj] = 0.0f;
            }
            for (uint32_t t = empty ? t1 : t0; t < t1; ++t, ++g) {
                if (*abort_flag) { ok = false; break; }
                ok = warp_wait_l(wait_ns, &s_full[g & 1u], (g >> 1) & 1u);
                if (!ok) break;
                tc_fence_after();
                // partial scores of this row: columns 16 half' + 8 hd + jj; this lane's half is the useful one
                uint32_t r0[8], r1[8];
                const uint32_t s_col = tmem_base + lane_addr + ((g & 1u) ? kColS1 : kColS0) + 8u * hd;
                tmem_ld8(s_col, r0);
                tmem_ld8(s_col + 16u, r1);
                tmem_wait_ld();
                const uint32_t tok = t * kTileTokens + pg * kPage + tk;
                const bool valid = tok >= tok_lo && tok < tok_hi;
                float s[G];
                bool over = false;
#pragma unroll
                for (int jj = 0; jj < G; ++jj) {
                    float x = __uint_as_float(half ? r1[jj] : r0[jj]);
                    x += __shfl_xor_sync(0xFFFFFFFFu, x, 16);  // the other half of d: the same token and head, lane +- 16
                    x *= scale2;
                    if (softcap) x = tanhf(fminf(fmaxf(x / a.logit_softcap, -15.0f), 15.0f)) * a.logit_softcap * kLog2e;
                    s[jj] = valid ? x : -INFINITY;
                    over = over || (s[jj] > m_used[jj] + kRescale);
                }
                float alpha[G];
#pragma unroll
                for (int jj = 0; jj < G; ++jj) alpha[jj] = 1.0f;
                if (bar_or_128(over)) {
                    // per-head maximum over the tile: 16 tokens of this warp, then the other page's warp of the same head
                    float mx[G];
#pragma unroll
                    for (int jj = 0; jj < G; ++jj) mx[jj] = s[jj];
#pragma unroll
                    for (int off = 8; off >= 1; off >>= 1)
#pragma unroll
                        for (int jj = 0; jj < G; ++jj) mx[jj] = fmaxf(mx[jj], __shfl_xor_sync(0xFFFFFFFFu, mx[jj], off));
                    if (lane == 0) {
#pragma unroll
                        for (int jj = 0; jj < G; ++jj) red[warp * 8 + jj] = mx[jj];
                    }
                    named_bar_sync_128();
#pragma unroll
                    for (int jj = 0; jj < G; ++jj) {
                        const float m_tile = fmaxf(red[hd * 8 + jj], red[(hd + 2u) * 8 + jj]);
                        if (m_tile > m_used[jj]) {
                            alpha[jj] = (m_used[jj] == -INFINITY) ? 0.0f : exp2f(m_used[jj] - m_tile);
                            m_used[jj] = m_tile;
                        }
                    }
                    // the accumulator's columns belong to all query heads of the row: publish the factors
                    if (lane == 0 && pg == 0u) {
#pragma unroll
                        for (int jj = 0; jj < 8; ++jj) alpha_s[hd * 8 + jj] = (jj < G) ? alpha[jj < G ? jj : 0] : 1.0f;
                    }
                    named_bar_sync_128();
                    if (t > t0) {
                        ok = warp_wait_l(wait_ns, &pv_done[(g - 1u) & 1u], ((g - 1u) >> 1) & 1u);
                        if (!ok) break;
                        tc_fence_after();
                        // O' rows (d_lo) live in lanes 0-15 of every warp; the other lanes go through the motions
                        uint32_t o[32];
                        tmem_ld32(tmem_base + lane_addr + kColO, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int cI = 0; cI < 32; ++cI) o[cI] = __float_as_uint(__uint_as_float(o[cI]) * alpha_s[cI & 15]);
                        tmem_st32(tmem_base + lane_addr + kColO, o);
                        tmem_wait_st();
                    }
#pragma unroll
                    for (int jj = 0; jj < G; ++jj) l_lane[jj] *= alpha[jj];
                    named_bar_sync_128();  // alpha_s and red may be rewritten by the next tile
                }
                if (g >= 2) {
                    ok = warp_wait_l(wait_ns, &pv_done[g & 1u], ((g >> 1) - 1u) & 1u);
                    if (!ok) break;
                }
                {
                    uint8_t* pbuf = sP + (g & 1u) * kPBytes;
#pragma unroll
                    for (int jj = 0; jj < G; ++jj) {
                        const float p = (s[jj] == -INFINITY) ? 0.0f : fast_exp2(s[jj] - m_used[jj]);
                        l_lane[jj] += half ? 0.0f : p;  // both halves hold the same probability: count it once
                        *reinterpret_cast<uint16_t*>(pbuf + p_off[jj]) = T::store(p);
                    }
                }
                if (!valid) {  // this thread's V row must contribute nothing: clear it (0 * garbage must not appear)
                    const uint32_t stage = g % kStages;
                    uint4* vrow = reinterpret_cast<uint4*>(sKV + stage * kStageBytes + kTileKBytes + tid * 128u);
#pragma unroll
                    for (int cI = 0; cI < 8; ++cI) vrow[cI] = make_uint4(0u, 0u, 0u, 0u);
                }
                tc_fence_before();
                fence_async_smem();
                mbar_arrive(&p_ready[g & 1u]);
            }
            if (!ok) break;
            // ---- end of the run piece ---------------------------------------------------------------------------
            // sums per head: 16 tokens of the warp (the lanes of the second half hold zeros), then the two pages' warps
            float l_tot[G];
#pragma unroll
            for (int jj = 0; jj < G; ++jj) l_tot[jj] = l_lane[jj];
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1)
#pragma unroll
                for (int jj = 0; jj < G; ++jj) l_tot[jj] += __shfl_xor_sync(0xFFFFFFFFu, l_tot[jj], off);
            if (lane == 0) {
#pragma unroll
                for (int jj = 0; jj < G; ++jj) red[warp * 8 + jj] = l_tot[jj];
            }
            named_bar_sync_128();
            if (lane == 0 && pg == 0u) {  // (m, l) of the piece for the G heads of this KV head, row order j = hd * G + jj
#pragma unroll
                for (int jj = 0; jj < G; ++jj) {
                    ml_s[(hd * G + jj) * 2 + 0] = m_used[jj];
                    ml_s[(hd * G + jj) * 2 + 1] = red[hd * 8 + jj] + red[(hd + 2u) * 8 + jj];
                }
            }
            // the accumulator goes through shared memory so that thread t ends up with dimension t of every head
            float* ostage = reinterpret_cast<float*>(sP);  // [HQ][128]; the P buffers are idle here
            if (!empty) {
                ok = warp_wait_l(wait_ns, &pv_done[(g - 1u) & 1u], ((g - 1u) >> 1) & 1u);
                if (!ok) break;
                tc_fence_after();
                uint32_t o[32];
                tmem_ld32(tmem_base + lane_addr + kColO, o);
                tmem_wait_ld();
                tc_fence_before();
                if (lane < 16u) {
#pragma unroll
                    for (int cI = 0; cI < 32; ++cI) {
                        const uint32_t hh = (uint32_t(cI) & 15u) >> 3, jj = uint32_t(cI) & 7u;  // column = 16 half' + 8 head + jj
                        if (jj < uint32_t(G)) ostage[(hh * G + jj) * kD + (uint32_t(cI) >> 4) * 64u + warp * 16u + lane] = __uint_as_float(o[cI]);
                    }
                }
            }
            named_bar_sync_128();
            const uint32_t d = tid;
            float Mh[HQ], Lh[HQ], Oh[HQ];
#pragma unroll
            for (int j = 0; j < HQ; ++j) {
                Mh[j] = empty ? -INFINITY : ml_s[j * 2];
                Lh[j] = empty ? 0.0f : ml_s[j * 2 + 1];
                Oh[j] = empty ? 0.0f : ostage[j * kD + d];
            }
            named_bar_sync_128();  // ostage (the P buffers) and ml_s are free again
            if (pdl == 3u) pdl_wait_previous_grid();
            const size_t row0 = size_t(req) * Hq;
            const bool split = seg.n_parts > 1u;
            const bool finisher = !split || (seg.n_parts <= pp.late_parts && seg.slot + 1u == seg.first_slot + seg.n_parts);
            if (finisher) {
                if (split) {
                    ok = gather_merge<HQ>(pp.ll_o, pp.ll_ml, seg, pp.epoch, wait_ns, red, tid, Mh, Lh, Oh);
                    if (!ok) break;
                }
#pragma unroll
                for (int j = 0; j < HQ; ++j) {
                    if (state_mode) {
                        a.state_o[(row0 + j) * kD + d] = Oh[j];
                        if (d == 0) {
                            a.state_m[row0 + j] = Mh[j] / kLog2e;
                            a.state_l[row0 + j] = Lh[j];
                        }
                    } else {
                        reinterpret_cast<uint16_t*>(a.out)[(row0 + j) * kD + d] = T::store(Oh[j] / fmaxf(Lh[j], 1e-12f));
                    }
                }
            } else {
                if (!set_known) {
                    uint32_t st = *set_free_s;
                    const uint64_t t_start = global_timer_ns();
                    for (uint32_t spin = 0; st == 0u; ++spin) {
                        st = *set_free_s;
                        if (st == 0u && (spin & 63u) == 63u && global_timer_ns() - t_start > 2u * wait_ns) break;
                    }
                    ok = !bar_or_128(st != 1u);
                    if (!ok) break;
                    set_known = true;
                }
                const size_t prow = size_t(seg.slot) * HQ;
#pragma unroll
                for (int j = 0; j < HQ; ++j) {
                    ll_store(&pp.ll_o[(prow + j) * kD + d], Oh[j], pp.epoch);
                    if (tid == uint32_t(2 * j)) ll_store(&pp.ll_ml[(prow + j) * 2 + 0], Mh[j], pp.epoch);
                    if (tid == uint32_t(2 * j + 1)) ll_store(&pp.ll_ml[(prow + j) * 2 + 1], Lh[j], pp.epoch);
                }
            }
            // the probability buffers served as output staging: their fixed zero pattern must be back before the next piece
            if (si + 1 < seg_end) {
                for (uint32_t i = tid; i < 2 * kPBytes / 16; i += 128u) reinterpret_cast<uint4*>(sP)[i] = make_uint4(0u, 0u, 0u, 0u);
                named_bar_sync_128();
            }
        }
        if (!ok && lane == 0) {
            atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            *abort_flag = 1;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (tid == 0) atomicAdd(pp.set_done, 1u);
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// Runs cut into very many pieces (one long row spread over the machine): one CTA per (run, query head).
template <int G, typename T>
__global__ void __launch_bounds__(kD) late_merge_kernel(KriyaDecodeArgs a, const KriyaTcSeg* segs, uint32_t late_parts,
                                                        const uint2* __restrict__ ll_o, const uint2* __restrict__ ll_ml) {
    constexpr int HQ = kHkv * G;
    const KriyaTcSeg seg = segs[blockIdx.x];
    if (seg.slot != seg.first_slot || seg.n_parts <= late_parts) return;
    const uint32_t h = blockIdx.y, d = threadIdx.x;
    float M = -INFINITY, L = 0.0f, O = 0.0f;
    for (uint32_t c0 = 0; c0 < seg.n_parts; c0 += 8u) {
        const uint32_t cnt = min(8u, seg.n_parts - c0);
        float ms[8], ls[8], ov[8];
#pragma unroll
        for (int s2 = 0; s2 < 8; ++s2) {
            const size_t row = size_t(seg.first_slot + c0 + min(uint32_t(s2), cnt - 1u)) * HQ + h;
            ms[s2] = uint32_t(s2) < cnt ? __uint_as_float(ll_ml[row * 2 + 0].x) : -INFINITY;
            ls[s2] = __uint_as_float(ll_ml[row * 2 + 1].x);
            ov[s2] = __uint_as_float(ll_o[row * kD + d].x);
        }
        float mc = M;
#pragma unroll
        for (int s2 = 0; s2 < 8; ++s2) mc = fmaxf(mc, ms[s2]);
        if (mc == -INFINITY) continue;
        const float keep = (M == -INFINITY) ? 0.0f : exp2f(M - mc);
        L *= keep;
        O *= keep;
#pragma unroll
        for (int s2 = 0; s2 < 8; ++s2) {
            const float w = (ms[s2] == -INFINITY) ? 0.0f : exp2f(ms[s2] - mc);
            L = fmaf(w, ls[s2], L);
            O = fmaf(w, ov[s2], O);
        }
        M = mc;
    }
    const size_t row0 = size_t(seg.req) * a.num_q_heads + h;
    if (a.state_o != nullptr) {
        a.state_o[row0 * kD + d] = O;
        if (d == 0) {
            a.state_m[row0] = M / kLog2e;
            a.state_l[row0] = L;
        }
    } else {
        reinterpret_cast<uint16_t*>(a.out)[row0 * kD + d] = T::store(O / fmaxf(L, 1e-12f));
    }
}

template <int G, typename T>
cudaError_t launch_t(const Params& pp, const CUtensorMap& mk, const CUtensorMap& mv, uint32_t grid, int max_smem_optin,
                     bool programmatic, cudaStream_t s) {
    const size_t smem = size_t(kStages) * kStageBytes + kQBufs * kQBytes + 2 * kPBytes + 512 + 64 + 128 + 320 + 8 * sizeof(KriyaTcSeg) + 1024;
    if (smem > size_t(max_smem_optin)) return cudaErrorInvalidValue;
    auto kern = decode_tcp_kernel<G, T>;
    {
        static std::atomic<uint64_t> attr_set{0};
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        const uint64_t bit = uint64_t(1) << (dev & 63);
        if (!(attr_set.load(std::memory_order_acquire) & bit)) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
            if (e != cudaSuccess) return e;
            attr_set.fetch_or(bit, std::memory_order_release);
        }
    }
    if (programmatic) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, kern, mk, mv, pp);
        if (e != cudaSuccess) return e;
    } else {
        kern<<<grid, kThreads, smem, s>>>(mk, mv, pp);
    }
    if (pp.late_parts != UINT32_MAX && pp.n_seg != 0u)
        late_merge_kernel<G, T><<<dim3(pp.n_seg, kHkv * G), kD, 0, s>>>(pp.a, pp.segs, pp.late_parts, pp.ll_o, pp.ll_ml);
    return cudaGetLastError();
}

template <typename T>
cudaError_t launch_g(uint32_t group, const Params& pp, const CUtensorMap& mk, const CUtensorMap& mv, uint32_t grid,
                     int max_smem_optin, bool ov, cudaStream_t s) {
    switch (group) {
        case 1: return launch_t<1, T>(pp, mk, mv, grid, max_smem_optin, ov, s);
        case 2: return launch_t<2, T>(pp, mk, mv, grid, max_smem_optin, ov, s);
        case 3: return launch_t<3, T>(pp, mk, mv, grid, max_smem_optin, ov, s);
        case 4: return launch_t<4, T>(pp, mk, mv, grid, max_smem_optin, ov, s);
        case 5: return launch_t<5, T>(pp, mk, mv, grid, max_smem_optin, ov, s);
        case 6: return launch_t<6, T>(pp, mk, mv, grid, max_smem_optin, ov, s);
        case 7: return launch_t<7, T>(pp, mk, mv, grid, max_smem_optin, ov, s);
        case 8: return launch_t<8, T>(pp, mk, mv, grid, max_smem_optin, ov, s);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace tcp
}  // namespace kriya

bool kriya_decode_tcp_supported(uint32_t head_dim, uint32_t num_kv_heads, uint32_t group, uint32_t block_size) {
    return head_dim == uint32_t(kriya::tcp::kD) && num_kv_heads == uint32_t(kriya::tcp::kHkv) && group >= 1 && group <= 8 &&
           block_size == uint32_t(kriya::tcp::kPage);
}
uint32_t kriya_decode_tcp_pages_per_tile() { return uint32_t(kriya::tcp::kPagesPerTile); }

namespace {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
}

// 5-D maps over the K and V pools of all layers with one page per box: dimensions (d_lo 64, token 16, half of d 2, head 2,
// page), strides (512, 128, 256, 8192) bytes.
cudaError_t kriya_decode_tcp_encode_maps(void* pool_k, void* pool_v, uint64_t total_pages, void* out_map_k, void* out_map_v) {
    static EncodeFn enc = nullptr;
    if (enc == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess) return e;
        if (fn == nullptr || qres != cudaDriverEntryPointSuccess) return cudaErrorNotSupported;
        enc = reinterpret_cast<EncodeFn>(fn);
    }
    const cuuint64_t dims[5] = {64, 16, 2, 2, total_pages};
    const cuuint64_t strides[4] = {512, 128, 256, 8192};
    const cuuint32_t box[5] = {64, 16, 2, 2, 1};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    void* pools[2] = {pool_k, pool_v};
    void* outs[2] = {out_map_k, out_map_v};
    for (int i = 0; i < 2; ++i) {
        const CUresult r = enc(static_cast<CUtensorMap*>(outs[i]), CU_TENSOR_MAP_DATA_TYPE_UINT16, 5, pools[i], dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    return cudaSuccess;
}

cudaError_t kriya_launch_decode_tcp(const KriyaDecodeArgs& a, const KriyaTcSeg* segs, const uint32_t* cta_seg_ptr, uint32_t grid,
                                    const void* map_k, const void* map_v, uint32_t page0, uint32_t dtype, int max_smem_optin,
                                    const KriyaFusedAppend& fused, uint32_t late_parts, uint32_t n_seg, const KriyaTcScratch& scratch,
                                    cudaStream_t s) {
    if (grid == 0) return cudaSuccess;
    if (a.num_kv_heads != uint32_t(kriya::tcp::kHkv) || !map_k || !map_v) return cudaErrorInvalidValue;
    const uint32_t group = a.num_q_heads / a.num_kv_heads;
    kriya::tcp::Params pp;
    pp.a = a;
    pp.segs = segs;
    pp.cta_seg_ptr = cta_seg_ptr;
    pp.page0 = page0;
    pp.late_parts = late_parts;
    pp.n_seg = n_seg;
    pp.ll_o = static_cast<uint2*>(scratch.ll_o);
    pp.ll_ml = static_cast<uint2*>(scratch.ll_ml);
    pp.set_done = scratch.set_done;
    pp.done_expect = scratch.done_expect;
    pp.epoch = scratch.epoch;
    pp.f = fused;
    const CUtensorMap& mk = *static_cast<const CUtensorMap*>(map_k);
    const CUtensorMap& mv = *static_cast<const CUtensorMap*>(map_v);
    const bool ov = fused.overlap_previous != 0;
    return dtype == KRIYA_DTYPE_FP16 ? kriya::tcp::launch_g<kriya::Fp16>(group, pp, mk, mv, grid, max_smem_optin, ov, s)
                                     : kriya::tcp::launch_g<kriya::Bf16>(group, pp, mk, mv, grid, max_smem_optin, ov, s);
}
