// Paged GQA decode attention on the tensor cores, whole pages per copy: head_dim 128, two KV heads, 16-token pages (the job
// of bsr_paged_gqa_decode_stage1 and bsr_paged_gqa_split_k_reduce, kernels/metal/paged_gqa_and_deltanet.metal:242-495,
// 1474-1525; the shape of the Qwen2.5 family this path is measured on).
//
// Why a second tensor-core kernel.  The kernel of kriya_decode_tc.cu gathers one KV head of one page with four tensor
// copies of 2 KB; a B200 SM sustains about 50 GB/s of such copies however few SMs are streaming, and copies of 8 KB
// about twice that.  One page of this cache, [16 tokens][2 heads][128 d], is 8 KB of contiguous memory, so this kernel
// moves a page - both heads - with ONE copy and lets one CTA process both KV heads of a row together.
//
// Layout.  Both pools are read through 5-D tensor maps with the dimensions permuted, one copy per page, 128-byte swizzle.
//   V: {64 d_lo, 16 tokens (512 B apart), 2 halves of d (128 B), 2 heads (256 B), pages (8 KB)}, box = one page: a page
//      lands as four planes [head][half] of [16 tokens][128 B].  The two planes of a head are the MN-major A operand
//      (M = 128 d as two groups of 64, K = the page's 16 tokens) of  O^T[d][jj] += V_page_head^T . P[jj][tokens].
//   K: {64 d_lo, 8 tokens, 2 halves, 2 heads, (page, eight-token group) (4 KB apart)}, box {64, 8, 2, 2, 2} = one page: a
//      page lands as sixteen 1 KB blocks of eight rows, [group][head][half][token][64].  For one half of d the blocks of
//      a whole tile are 2 KB apart, all of them, so the tile's 128 rows (page, group, head, token) are ONE K-major A
//      operand per half (8-row groups 2 KB apart) and the two halves are K steps of one accumulation:
//        S[(page, group, head, token)][8 h' + jj] = sum over d of K[token][head][d] * Q[h' G + jj][d]     (M128 N16 K16 x 8)
//      whose entry is a score where h' is the row's own KV head.
// The probability operand of P.V is a K-major [query head][token] tile per pair of pages that every softmax thread fills at
// its own token; M = 128 allows no N below 16, so its upper eight rows are zero and their result columns are not read.
//
// Roles (384 threads, one CTA per SM, persistent over a list of run pieces exactly as in kriya_decode_tc.cu); a tile is
// four pages: 64 tokens of both heads, 32 KB of K and 32 KB of V:
//   warps 0-7 softmax: a thread owns one score row; warps w and w + 4 both read the TMEM lanes of page w % 4 (lane = (group,
//     head, token)) and share the row's query heads (warps 0-3 the first half of the group, warps 4-7 the second),
//   warp 8 producer (page indices, one tensor copy per page of K and one of V into a 3-deep ring of 64 KB stages; the K
//     half of a stage is loaded again as soon as its score MMAs are complete, the V half when the tile is done),
//   warp 9 MMA issuer (scores two tiles ahead of P.V), warp 10 scratch-set guard, warp 11 stager (queries, rotated in
//     flight; the new token's K/V row).
// Split runs, the finishing piece, stamps and the set guard work as described in kriya_decode_tc.cu; a run here is a
// whole plan row (both KV heads).  At the end of a piece threads 0-127 finish the query heads of KV head 0 and threads
// 128-255 those of KV head 1, one output dimension each.  Every wait is bounded.
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
constexpr int kPagesPerTile = 4;                 // 4 pages x 2 heads x 16 tokens = the 128 rows of a score MMA
constexpr int kTileTokens = kPagesPerTile * kPage;
constexpr uint32_t kPageBytes = 8192;            // one page of K (or V), both heads
constexpr uint32_t kTileKBytes = kPagesPerTile * kPageBytes;  // 32 KB
constexpr uint32_t kStageBytes = 2 * kTileKBytes;             // K tile + V tile
// A K page lands as sixteen 1 KB blocks of eight rows, [eight-token group][head][half of d][token][64]: for one half of d the
// blocks of a whole tile are 2 KB apart, all of them, so the tile's 128 (page, group, head, token) rows are one K-major MMA
// operand per half (8-row groups 2 KB apart) although every page arrived as a single copy.
constexpr uint32_t kKBlock = 1024;
constexpr int kStages = 3;
constexpr int kQBufs = 3;
constexpr uint32_t kQBytes = 32 * 128;           // 32 operand rows (half', head) x 128 B
constexpr uint32_t kPBytes = (kPagesPerTile / 2) * 8 * 128;  // per pair of pages 8 operand rows (query heads of a KV head) x 128 B
constexpr int kSoftmaxThreads = 256;
constexpr int kThreads = 384;  // warps 0-7 softmax, 8 producer, 9 MMA issuer, 10 scratch-set guard, 11 stager
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS0 = 0, kColS1 = 64, kColO = 128;  // score tiles: 16 columns each; accumulator 32 columns
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
// Named barriers: id 1 joins the 256 softmax threads; ids 2 and 3 join the 128 threads that finish KV head 0 / 1.
__device__ __forceinline__ void bar_sync(uint32_t id, uint32_t nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ bool bar_or(uint32_t id, uint32_t nthreads, bool pred) {
    uint32_t res;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %3, 0;\n\t"
        "bar.red.or.pred p, %1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(res)
        : "r"(id), "r"(nthreads), "r"(uint32_t(pred))
        : "memory");
    return res != 0;
}
__device__ __forceinline__ void softmax_sync() { bar_sync(1u, kSoftmaxThreads); }
__device__ __forceinline__ bool softmax_or(bool pred) { return bar_or(1u, kSoftmaxThreads, pred); }
__device__ __forceinline__ void ll_store(uint2* p, float v, uint32_t epoch) {
    asm volatile("st.global.cg.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(epoch) : "memory");
}
__device__ __forceinline__ uint2 ll_load(const uint2* p) {
    uint2 r;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p) : "memory");
    return r;
}
// The same word by an ordinary load that bypasses L1.  Many of these may be in flight at once, which the ordered loads
// above are not; a loop that polls with them must put a fence between two rounds, or the second round may be served from
// the first round's registers.
__device__ __forceinline__ uint2 ll_load_weak(const uint2* p) {
    uint2 r;
    asm volatile("ld.global.cg.v2.u32 {%0, %1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
    uint32_t r;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(r) : "l"(p) : "memory");
    return r;
}
__device__ __forceinline__ bool warp_wait_l(uint64_t limit_ns, uint64_t* bar, uint32_t parity) { return warp_wait(bar, parity, limit_ns); }
static __device__ __noinline__ bool wait_set_free(const uint32_t* set_done, uint32_t done_expect, uint64_t wait_ns) {
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
// A whole K page through the K map, whose outermost dimension counts (page, eight-token group): coordinates (0, 0, 0, 0, 2 page).
__device__ __forceinline__ void tma_load_kpage(void* dst_smem, const CUtensorMap* map, int32_t page, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %2, %2, %2, %3}], [%4];" ::"r"(
            smem_u32(dst_smem)),
        "l"(map), "r"(0), "r"(2 * page), "r"(smem_u32(bar))
        : "memory");
}
// 4 consecutive TMEM columns of this thread's lane.
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
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
// Soft-capped score in the exponent's base: a function of its own (tanhf is long and the call sits in an unrolled loop).
static __device__ __noinline__ float softcap_log2(float x, float cap) {
    return tanhf(fminf(fmaxf(x / cap, -15.0f), 15.0f)) * cap * kLog2e;
}
// (cos, sin) of one pair without the table: a function of its own, the inlined powf / cosf / sinf are kilobytes of code.
static __device__ __noinline__ float2 rope_pair_coeff(uint32_t i, uint32_t position, uint32_t rotary_dim, float theta) {
    const float freq_exp = float(2u * i) / float(rotary_dim);
    const float inv_freq = powf(theta, -freq_exp);
    const float angle = __fmul_rn(float(position), inv_freq);
    return make_float2(cosf(angle), sinf(angle));
}
__device__ __forceinline__ void rope8_coeffs(float2 (&cs)[8], uint32_t first_pair, uint32_t position, const KriyaFusedAppend& f) {
    const uint32_t half_rot = f.rotary_dim / 2u;
    const bool use_table = f.has_table != 0u && position < f.max_seq_len && f.table != nullptr;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const uint32_t i = first_pair + j;
        cs[j] = make_float2(1.0f, 0.0f);
        if (i < half_rot) {
            if (use_table)
                cs[j] = reinterpret_cast<const float2*>(f.table)[size_t(position) * half_rot + i];
            else
                cs[j] = rope_pair_coeff(i, position, f.rotary_dim, f.rope_theta);
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

// The run's last piece gathers the other pieces' states and finishes the run.  Called by the 128 threads that finish one
// KV head (barrier `bar_id`, staging area `stage` of their own): thread t owns output dimension t of the head's G query
// heads, which are heads head0 .. head0 + G - 1 of the row's HQ.  Other pieces are taken four at a time; every load of a
// chunk is issued before any is examined and repeated until it carries this launch's stamp (bounded).
template <int G>
__device__ __forceinline__ bool gather_merge(const uint2* __restrict__ ll_o, const uint2* __restrict__ ll_ml, const KriyaTcSeg& seg,
                                             uint32_t epoch, uint64_t wait_ns, float* stage, uint32_t bar_id, uint32_t t, uint32_t HQ,
                                             uint32_t head0, float (&M)[G], float (&L)[G], float (&O)[G]) {
    const uint32_t others = seg.n_parts - 1u;
    for (uint32_t c0 = 0; c0 < others; c0 += 4u) {
        const uint32_t cnt = min(4u, others - c0);
        const size_t slot0 = size_t(seg.first_slot) + c0;
        uint2 w[4][G];
        uint2 mlw = make_uint2(0u, epoch);
        // (m, l) words of the chunk, one per thread: t = (part * G + head) * 2 + which
        const bool has_ml = t < cnt * uint32_t(G) * 2u;
        const uint32_t ml_part = has_ml ? t / (2u * G) : 0u, ml_rest = has_ml ? t % (2u * G) : 0u;
        const uint2* mlp = &ll_ml[((slot0 + ml_part) * HQ + head0) * 2 + ml_rest];
        bool got = false;
        const uint64_t t_start = global_timer_ns();
        for (uint32_t spin = 0; !got; ++spin) {
#pragma unroll
            for (int s2 = 0; s2 < 4; ++s2)
#pragma unroll
                for (int h = 0; h < G; ++h)
                    w[s2][h] = ll_load_weak(&ll_o[((slot0 + min(uint32_t(s2), cnt - 1u)) * HQ + head0 + h) * kD + t]);
            mlw = ll_load_weak(mlp);
            uint32_t bad = mlw.y ^ epoch;
#pragma unroll
            for (int s2 = 0; s2 < 4; ++s2)
#pragma unroll
                for (int h = 0; h < G; ++h) bad |= w[s2][h].y ^ epoch;
            got = bad == 0u;
            if (!got) {
                __threadfence();  // the next round reads memory again
                if ((spin & 63u) == 63u && global_timer_ns() - t_start > wait_ns) break;
            }
        }
        if (has_ml) stage[t] = __uint_as_float(mlw.x);
        if (bar_or(bar_id, 128u, !got)) return false;
        // the weights depend on (piece, head) only: thread h works them out for head h, the others just accumulate
        float* wsm = stage + 64;            // [4][G] weights
        float* hsm = stage + 64 + 32;       // [3][8]: new maximum, new sum, factor on what was there
        if (t < uint32_t(G)) {
            float mh = M[0], lh = L[0];
#pragma unroll
            for (int h = 1; h < G; ++h) {
                mh = (t == uint32_t(h)) ? M[h] : mh;
                lh = (t == uint32_t(h)) ? L[h] : lh;
            }
            float mc = mh;
            for (uint32_t s2 = 0; s2 < cnt; ++s2) mc = fmaxf(mc, stage[(s2 * G + t) * 2]);
            const float keep = (mh == -INFINITY) ? 0.0f : fast_exp2(mh - mc);
            float lacc = lh * keep;
            for (uint32_t s2 = 0; s2 < 4u; ++s2) {
                float wgt = 0.0f;
                if (s2 < cnt) {
                    const float ms = stage[(s2 * G + t) * 2];
                    wgt = (ms == -INFINITY) ? 0.0f : fast_exp2(ms - mc);
                    lacc = fmaf(wgt, stage[(s2 * G + t) * 2 + 1], lacc);
                }
                wsm[s2 * G + t] = wgt;
            }
            hsm[t] = mc;
            hsm[8 + t] = lacc;
            hsm[16 + t] = keep;
        }
        bar_sync(bar_id, 128u);
#pragma unroll
        for (int h = 0; h < G; ++h) {
            float oacc = O[h] * hsm[16 + h];
#pragma unroll
            for (int s2 = 0; s2 < 4; ++s2) oacc = fmaf(wsm[s2 * G + h], __uint_as_float(w[s2][h].x), oacc);
            O[h] = oacc;
            M[h] = hsm[h];
            L[h] = hsm[8 + h];
        }
        bar_sync(bar_id, 128u);
    }
    return true;
}

// G = query heads per KV head (1..8); the row has HQ = 2 G query heads.
template <int G, typename T>
__global__ void __launch_bounds__(kThreads, 1)
decode_tcp_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, Params pp) {
    constexpr int HQ = kHkv * G;
    constexpr uint32_t FMT = (T::kDtype == KRIYA_DTYPE_BF16) ? 1u : 0u;
    constexpr uint32_t IDESC_S = make_idesc(FMT, 128, 16, 0, 0);  // A = the tile's 128 K rows (K-major), B = 16 query rows (K-major)
    // A = a page's two V planes of one head (MN-major: M = d), B = 16 x 16: rows 0-7 the probabilities of the head's query heads;
    // M = 128 allows no N below 16, so rows 8-15 are whatever follows in shared memory and their 8 result columns are never read
    constexpr uint32_t IDESC_O = make_idesc(FMT, 128, 16, 1, 0);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
    uint8_t* sKV = sm;                                  // [stages][K tile 32 KB | V tile 32 KB]
    uint8_t* sQ = sKV + kStages * kStageBytes;          // [3][4 KB]
    uint8_t* sP = sQ + kQBufs * kQBytes;                // [2][2 KB]
    float* red = reinterpret_cast<float*>(sP + 2 * kPBytes);  // [8 warps][8] maxima / sums; [64 ..): merge staging of the two KV heads
    float* alpha_s = red + 512;                         // [16] rescale factors per query head
    float* ml_s = alpha_s + 16;                         // [16][2] (m, l) of the piece per query head
    uint64_t* bars = reinterpret_cast<uint64_t*>(ml_s + 32);
    uint64_t* kv_full = bars;                     // [stages]: the K half of a stage has landed
    uint64_t* k_empty = bars + kStages;           // [stages]: the score MMAs of the stage's tile are complete, its K half may be
                                                  // loaded again (the V half and the rest of the stage wait for tile_done)
    uint64_t* s_full = bars + 2 * kStages;        // [2]
    uint64_t* p_ready = bars + 2 * kStages + 2;   // [2], 256 arrivals
                                                  // (bars + 2 * kStages + 4 .. + 5 are spare)
    uint64_t* q_ready = bars + 2 * kStages + 6;   // [3]
    uint64_t* q_free = bars + 2 * kStages + 9;    // [3]
    uint64_t* kv_ready = bars + 2 * kStages + 12; // [3]
    uint64_t* v_full = bars + 2 * kStages + 15;   // [stages]: the V half
    uint64_t* aux_full = bars + 3 * kStages + 15; // [0]: the segment records below have landed; [1]: the first piece's raw query rows;
                                                  // [2]: the other pieces' states (gather_merge_smem); [3] unused
    uint64_t* tile_done = bars + 3 * kStages + 19;  // [6]: the P.V of tile g is complete: entry g % 6, completion g / 6.  It frees
                                                    // the tile's stage (the producer waits for tile g - 3), its probability buffer
                                                    // (tile g - 2) and lets the accumulator be read.
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * kStages + 25);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* set_free_s = tmem_slot + 2;
    KriyaTcSeg* segs_s = reinterpret_cast<KriyaTcSeg*>(tmem_slot + 4);  // first 8 segment records of this CTA
    uint8_t* sQraw = reinterpret_cast<uint8_t*>(segs_s + 8);            // [HQ][256 B]: the first piece's query rows as they are in memory
    float2* sCs = reinterpret_cast<float2*>(sQraw + 16 * 256);          // [64]: the rotation table's row of its position

    const KriyaDecodeArgs& a = pp.a;
    const uint64_t wait_ns = a.wait_ns;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    // this CTA's record: first segment, pages of the first tile that may be fetched at once, their place, their blocks
    // and the row and the position of the first piece
    // followed by copies of the CTA's first two segment records (most CTAs have no more)
    constexpr uint32_t kHdrVec = 9;  // 144 bytes per record
    const uint4* hdr = reinterpret_cast<const uint4*>(pp.cta_seg_ptr) + size_t(blockIdx.x) * kHdrVec;
    const uint4 hdr0 = hdr[0], hdr1 = hdr[1];
    const uint32_t hdr_position = reinterpret_cast<const uint32_t*>(hdr + 2)[0];
    const uint32_t seg_begin = hdr0.x;
    const uint32_t seg_end = reinterpret_cast<const uint32_t*>(hdr + kHdrVec)[0];
    // the two segment records go to shared memory by plain stores (visible after the set-up barrier); further ones come by
    // a copy that is waited for only by whoever reads them
    if (tid < 24u) reinterpret_cast<uint32_t*>(segs_s)[tid] = reinterpret_cast<const uint32_t*>(hdr + 3)[tid];
    if (threadIdx.x == 0) pdl_launch_dependents();
    if (seg_begin == seg_end) {
        if (threadIdx.x == 0) {
            if (!wait_set_free(pp.set_done, pp.done_expect, pp.a.wait_ns)) atomicMax(pp.a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            atomicAdd(pp.set_done, 1u);
        }
        return;
    }
    const uint32_t pdl = pp.f.overlap_previous;  // see kriya_decode_tc.cu
    // What the CTA needs first is asked for before it is set up, by copies that complete on barriers of their own (a load
    // into registers would hold up the CTA-wide barrier below until it has returned): the segment records, the K/V pages
    // of the first tile, the query rows of the first piece and the rotation table's row of its position.  The K/V pages
    // not when this launch has to wait for the whole of the previous one (it may still be writing the cache); the query
    // rows not when the previous launch writes them.
    const uint32_t early_pages = (pdl == 1u) ? 0u : min(hdr0.y, uint32_t(kPagesPerTile));
    const bool stager_fused = pp.f.k_in != nullptr;
    const uint32_t half_rot0 = pp.f.rotary_dim / 2u;
    bool first_q = hdr0.w != UINT32_MAX;  // the CTA has a piece to work on
    const bool q_bulk = first_q && (reinterpret_cast<uintptr_t>(a.q) & 15u) == 0u;
    const bool cs_bulk = q_bulk && stager_fused && pp.f.has_table != 0u && hdr_position < pp.f.max_seq_len && pp.f.table != nullptr &&
                         (half_rot0 & 1u) == 0u && half_rot0 <= 64u;
    auto issue_q0 = [&]() {  // one thread
        const uint32_t q_bytes = uint32_t(HQ) * kD * 2u;
        mbar_arrive_expect_tx(&aux_full[1], q_bytes + (cs_bulk ? half_rot0 * 8u : 0u));
        bulk_g2s(sQraw, reinterpret_cast<const uint16_t*>(a.q) + size_t(hdr0.w) * a.num_q_heads * kD, q_bytes, &aux_full[1]);
        if (cs_bulk) bulk_g2s(sCs, reinterpret_cast<const float2*>(pp.f.table) + size_t(hdr_position) * half_rot0, half_rot0 * 8u, &aux_full[1]);
    };
    if (warp == 8) {
        if (lane == 0) {
            for (int s = 0; s < kStages; ++s) {
                mbar_init(&kv_full[s], 1);
                mbar_init(&k_empty[s], 1);
                mbar_init(&v_full[s], 1);
                mbar_init(&tile_done[s], 1);
                mbar_init(&tile_done[kStages + s], 1);
            }
            mbar_init(&aux_full[0], 1);
            mbar_init(&aux_full[1], 1);
            mbar_init(&aux_full[2], 1);
            mbar_fence_init();
            if (seg_end - seg_begin > 2u) {
                const uint32_t seg_bytes = (min(seg_end - seg_begin, 8u) - 2u) * uint32_t(sizeof(KriyaTcSeg));
                mbar_arrive_expect_tx(&aux_full[0], seg_bytes);
                bulk_g2s(segs_s + 2, pp.segs + seg_begin + 2u, seg_bytes, &aux_full[0]);
            }
            // the few KB of query rows go ahead of the tile: the copy engine takes its requests in order
            if (q_bulk && (pdl == 0u || pdl == 2u)) issue_q0();
            if (early_pages) {
                mbar_arrive_expect_tx(&kv_full[0], early_pages * kPageBytes);
                mbar_arrive_expect_tx(&v_full[0], early_pages * kPageBytes);
            }
        }
        __syncwarp();
        if (lane < early_pages) {
            uint32_t blk = lane == 0 ? hdr1.x : lane == 1 ? hdr1.y : lane == 2 ? hdr1.z : hdr1.w;
            if (blk >= a.num_blocks) {
                atomicMax(a.status, uint32_t(KRIYA_DEV_BAD_BLOCK_INDEX));
                blk = 0;
            }
            const uint32_t slot = hdr0.z + lane;  // the page's place in the tile
            const int32_t page = int32_t(pp.page0 + blk);
            tma_load_kpage(sKV + slot * kPageBytes, &map_k, page, &kv_full[0]);
            tma_load_page(sKV + kTileKBytes + slot * kPageBytes, &map_v, page, &v_full[0]);
        }
    }
    if (tid == 0) {
        mbar_init(&s_full[0], 1);
        mbar_init(&s_full[1], 1);
        mbar_init(&p_ready[0], kSoftmaxThreads);
        mbar_init(&p_ready[1], kSoftmaxThreads);
        for (int b = 0; b < 3; ++b) {
            mbar_init(&q_ready[b], 1);
            mbar_init(&q_free[b], 1);
            mbar_init(&kv_ready[b], 1);
        }
        *abort_flag = 0;
        *set_free_s = 0;
        mbar_fence_init();
    }
    if (warp == 9) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    auto seg_at = [&](uint32_t si) -> KriyaTcSeg {
        const uint32_t i = si - seg_begin;
        if (i < 2u) return segs_s[i];
        if (i >= 8u) return pp.segs[si];
        if (!mbar_wait(&aux_full[0], 0u, wait_ns)) {  // records 2 .. 7 come by a copy; one that never lands reads as an empty piece
            atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            *abort_flag = 1;
            return KriyaTcSeg{};
        }
        return segs_s[i];
    };
    // Query and probability rows of heads that do not exist (G < 8) stay zero (they feed unused columns only); with
    // G = 8 every row is written before it is read.
    if (G < 8) {
        for (uint32_t i = tid; i < (kQBufs * kQBytes + 2 * kPBytes) / 16; i += kThreads)
            reinterpret_cast<uint4*>(sQ)[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();  // every barrier is set up, the first two segment records are in place
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t Hq = a.num_q_heads;
    if (pdl == 1u) {
        pdl_wait_previous_grid();
        if (warp == 8 && lane == 0 && q_bulk && first_q) issue_q0();
    }

    if (warp == 8) {
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
                if (g > 0u || early_pages == 0u) {  // the CTA's first tile may be on its way already
                    int32_t blk = pf_blk;
                    if (!pf_valid && lane < npages) blk = table[my_page];
                    // the K half is free as soon as the scores of the tile it held are complete, a tile-time before the rest
                    if (g >= kStages && !warp_wait_l(wait_ns, &k_empty[stage], ((g / kStages) - 1u) & 1u)) { ok = false; break; }
                    if (owns_last && t + 1u == t1 && !warp_wait_l(wait_ns, &kv_ready[runs % uint32_t(kQBufs)], (runs / uint32_t(kQBufs)) & 1u)) {
                        ok = false;
                        break;
                    }
                    if (lane < npages && uint32_t(blk) >= a.num_blocks) {
                        atomicMax(a.status, uint32_t(KRIYA_DEV_BAD_BLOCK_INDEX));
                        blk = 0;
                    }
                    uint8_t* st = sKV + stage * kStageBytes;
                    const uint32_t slot = my_page - t * kPagesPerTile;
                    const int32_t page = int32_t(pp.page0) + blk;
                    if (lane == 0) mbar_arrive_expect_tx(&kv_full[stage], npages * kPageBytes);
                    __syncwarp();
                    if (lane < npages) tma_load_kpage(st + slot * kPageBytes, &map_k, page, &kv_full[stage]);
                    if (g >= kStages && !warp_wait_l(wait_ns, &tile_done[(g - kStages) % 6u], ((g - kStages) / 6u) & 1u)) { ok = false; break; }
                    if (lane == 0) mbar_arrive_expect_tx(&v_full[stage], npages * kPageBytes);
                    __syncwarp();
                    if (lane < npages) tma_load_page(st + kTileKBytes + slot * kPageBytes, &map_v, page, &v_full[stage]);
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
    } else if (warp == 11) {
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
            const bool stage_q = runs > 0u;  // the first piece's query rows are staged by warps 0-3
            // one item at a time, not unrolled: this warp runs a whole piece ahead of the tensor cores, and code that is
            // executed a few times per launch is paid for in instruction-cache misses
#pragma unroll 1
            for (int it = 0; it < ITEMS; ++it) {
                const uint32_t j = (lane + 32u * it) >> 3;
                if (stage_q && j < uint32_t(HQ)) {
                    uint4 lo = *reinterpret_cast<const uint4*>(qg + j * kD + c * 8);
                    uint4 hi = *reinterpret_cast<const uint4*>(qg + j * kD + 64 + c * 8);
                    if (fused) rope8_apply<T>(lo, hi, c * 8u, cs, pp.f.rotary_dim / 2u);
                    const uint32_t row = 8u * (j / uint32_t(G)) + j % uint32_t(G);
                    *reinterpret_cast<uint4*>(qb + row * 128u + ((c ^ (row & 7u)) << 4)) = lo;
                    *reinterpret_cast<uint4*>(qb + 2048u + row * 128u + ((c ^ (row & 7u)) << 4)) = hi;
                    if (fused && owns_last && pp.f.q_rope_out != nullptr) {
                        uint16_t* qo = reinterpret_cast<uint16_t*>(pp.f.q_rope_out) + (size_t(seg.req) * Hq + j) * kD;
                        *reinterpret_cast<uint4*>(qo + c * 8) = lo;
                        *reinterpret_cast<uint4*>(qo + 64 + c * 8) = hi;
                    }
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0 && stage_q) mbar_arrive(&q_ready[runs % uint32_t(kQBufs)]);
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
    } else if (warp == 9) {
        // ---- MMA issuer ---------------------------------------------------------------------------------
        // Every lane runs this code, descriptor arithmetic included; only the tensor-core instructions themselves are
        // predicated on the elected lane.  That keeps their operands in uniform registers: issued from inside a
        // one-lane branch every instruction costs about a hundred cycles and the issue rate, not the memory stream,
        // bounds the kernel.
        const uint32_t el = (lane == 0) ? 1u : 0u;
        const uint64_t kv_desc = smem_desc_sw128(smem_u32(sKV), 16, 2 * kKBlock);  // K rows of one half of d: K-major, 8-row groups 2 KB apart
        // V: MN-major, M = 128 d as two groups of 64 (the head's two planes, 2 KB apart), 8-token groups 1 KB apart
        const uint64_t v_desc = smem_desc_sw128(smem_u32(sKV), 2048, 1024);
        const uint64_t q_desc = smem_desc_sw128(smem_u32(sQ), 16, 1024);
        const uint64_t p_desc = smem_desc_sw128(smem_u32(sP), 16, 1024);
        auto issue_s = [&](uint32_t gg, uint32_t qbuf) {
            const uint32_t stage = gg % kStages;
            const uint32_t d_tmem = tmem_base + ((gg & 1u) ? kColS1 : kColS0);
            const uint64_t ad = kv_desc + uint64_t((stage * kStageBytes) >> 4), bd = q_desc + uint64_t((qbuf * kQBytes) >> 4);
            // scores[(page, head, token)][query head] over d = 128: eight steps of 16, four in each half of d
#pragma unroll
            for (int hf = 0; hf < 2; ++hf)
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    umma_ss_pred(d_tmem, ad + uint64_t((uint32_t(hf) * kKBlock + uint32_t(ks) * 32u) >> 4),
                                 bd + uint64_t((uint32_t(hf) * 2048u + uint32_t(ks) * 32u) >> 4), IDESC_S, (hf | ks) ? 1u : 0u, el);
            umma_commit_pred(&s_full[gg & 1u], el);
            umma_commit_pred(&k_empty[stage], el);
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
            issue_s(la_g, la_run % uint32_t(kQBufs));
            ++la_g;
            if (++la_t >= la_t1) {
                umma_commit_pred(&q_free[la_run % uint32_t(kQBufs)], el);
                ++la_si;
                ++la_run;
                la_valid = la_load();
            }
            return true;
        };
        bool primed = false;  // the very first tile's scores are issued together with the second's (one copy of the code)
        for (uint32_t si = seg_begin; si < seg_end && ok; ++si) {
            const KriyaTcSeg seg = seg_at(si);
            if (seg.blk_hi <= seg.blk_lo) continue;
            const uint32_t t0 = seg.blk_lo / kPagesPerTile, t1 = (seg.blk_hi + kPagesPerTile - 1) / kPagesPerTile;
            for (uint32_t t = t0; t < t1 && ok; ++t, ++g) {
                if (*abort_flag) { ok = false; break; }
#pragma unroll 1
                for (int k = primed ? 1 : 0; k < 2 && ok; ++k) ok = la_issue();
                primed = true;
                if (!ok) break;
                const uint32_t stage = g % kStages;
                ok = warp_wait_l(wait_ns, &p_ready[g & 1u], (g >> 1) & 1u);  // (its arrivals have seen the V half land)
                if (!ok) break;
                tc_fence_after();
                const uint64_t ad = v_desc + uint64_t((stage * kStageBytes + kTileKBytes) >> 4);
                const uint64_t bd = p_desc + uint64_t(((g & 1u) * kPBytes) >> 4);
                const uint32_t first = (t > t0) ? 1u : 0u;
#pragma unroll
                for (int pgi = 0; pgi < kPagesPerTile; ++pgi)
#pragma unroll
                    for (int h = 0; h < kHkv; ++h)  // the 16 tokens of head h of the page are one K step; its d halves the two M groups
                        umma_ss_pred(tmem_base + kColO + 16u * uint32_t(h),
                                     ad + uint64_t((uint32_t(pgi) * kPageBytes + uint32_t(h) * 4096u) >> 4),
                                     bd + uint64_t((uint32_t(pgi >> 1) * 1024u + uint32_t(pgi & 1) * 64u + uint32_t(h) * 32u) >> 4), IDESC_O,
                                     (pgi > 0) ? 1u : first, el);
                umma_commit_pred(&tile_done[g % 6u], el);
            }
        }
        if (!ok && lane == 0) {
            atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            *abort_flag = 1;
        }
    } else if (warp == 10) {
        // ---- scratch-set guard (see kriya_decode_tc.cu) -------------------------------------------------------
        if (lane == 0) {
            const bool free_now = wait_set_free(pp.set_done, pp.done_expect, pp.a.wait_ns);
            if (!free_now) atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            __threadfence_block();
            *set_free_s = free_now ? 1u : 2u;
        }
    } else {
        // ---- softmax warps 0-7: the tile's 128 score rows are (page, KV head, token) = TMEM lanes; warps w and w + 4 both
        // read lanes 32 (w % 4) .. (page w % 4; lane = (KV head lane / 16, token lane % 16)) and share the row's query
        // heads: warps 0-3 take heads 0 .. GH - 1 of the row's KV head, warps 4-7 heads GH .. G - 1.
        constexpr int GH = (G + 1) / 2;
        const uint32_t grp = warp >> 2, pg = warp & 3u;
        const uint32_t lane_addr = (pg * 32u) << 16;
        const uint32_t hd = (lane >> 3) & 1u, tk = ((lane >> 4) << 3) | (lane & 7u);  // rows of a page: (token group, head, token)
        const uint32_t jj0 = grp ? uint32_t(GH) : 0u;             // first query head (within the KV head) of this thread
        const uint32_t nj = grp ? uint32_t(G - GH) : uint32_t(GH);  // and how many
        const bool softcap = a.logit_softcap > 0.0f;
        const float scale2 = softcap ? a.sm_scale : a.sm_scale * kLog2e;
        const bool state_mode = a.state_o != nullptr;
        // a probability entry of this thread's token: pair of pages pg / 2, operand row jj, element k = 32 (pg % 2) + 16 hd + tk
        // of the pair's 64 (16-byte chunks swizzled with the row)
        const uint32_t k_in = 32u * (pg & 1u) + 16u * hd + tk;
        uint32_t p_off[GH];
#pragma unroll
        for (int i = 0; i < GH; ++i) {
            const uint32_t jj = jj0 + uint32_t(i);
            p_off[i] = (pg >> 1) * 1024u + jj * 128u + ((((k_in >> 3) ^ jj) << 4) | ((k_in & 7u) << 1));
        }
        // this thread's row of the tile's V half `grp` (cleared when its token lies outside the piece): [page][head][half][token]
        const uint32_t v_row_off = kTileKBytes + (((pg * 2u + hd) * 2u + grp) * 16u + tk) * 128u;
        // at the end of a piece threads 0-127 finish KV head 0 and threads 128-255 KV head 1, one output dimension each
        const uint32_t fin_hd = tid >> 7, d = tid & 127u;
        float* fin_stage = red + 64 + fin_hd * 128;
        bool ok = true;
        if (first_q && warp < 4u) {
            // ---- query rows of the first piece: warps 0-3 (idle until the first scores arrive), one 16-byte chunk pair per
            // thread; rotating sixteen heads is a few thousand instructions, microseconds for the single stager warp -----
            const uint32_t fq_j = tid >> 3, fq_c = tid & 7u;  // query head and chunk of this thread's item
            const bool fq_active = fq_j < uint32_t(HQ);
            if (pdl == 3u) {
                pdl_wait_previous_grid();
                if (tid == 0 && q_bulk) issue_q0();
            }
            uint32_t s0 = seg_begin;
            while (s0 + 1u < seg_end && seg_at(s0).blk_hi <= seg_at(s0).blk_lo) ++s0;
            const KriyaTcSeg seg0 = seg_at(s0);
            const bool owns_last0 = stager_fused && seg0.row_tokens > 0u && uint64_t(seg0.blk_hi) * kPage >= seg0.row_tokens;
            float2 fq_cs[8];
            if (stager_fused && !cs_bulk) rope8_coeffs(fq_cs, fq_c * 8u, hdr_position, pp.f);
            uint4 fq_lo = make_uint4(0u, 0u, 0u, 0u), fq_hi = make_uint4(0u, 0u, 0u, 0u);
            if (q_bulk) {
                ok = warp_wait_l(wait_ns, &aux_full[1], 0u);
                if (fq_active) {
                    fq_lo = *reinterpret_cast<const uint4*>(sQraw + fq_j * 256u + fq_c * 16u);
                    fq_hi = *reinterpret_cast<const uint4*>(sQraw + fq_j * 256u + 128u + fq_c * 16u);
                }
                if (cs_bulk) {
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        fq_cs[e] = (fq_c * 8u + uint32_t(e) < half_rot0) ? sCs[fq_c * 8u + uint32_t(e)] : make_float2(1.0f, 0.0f);
                }
            } else if (fq_active) {
                const uint16_t* qg = reinterpret_cast<const uint16_t*>(a.q) + (size_t(hdr0.w) * Hq + fq_j) * kD;
                fq_lo = *reinterpret_cast<const uint4*>(qg + fq_c * 8);
                fq_hi = *reinterpret_cast<const uint4*>(qg + 64 + fq_c * 8);
            }
            if (fq_active) {
                if (stager_fused) rope8_apply<T>(fq_lo, fq_hi, fq_c * 8u, fq_cs, half_rot0);
                const uint32_t row = 8u * (fq_j / uint32_t(G)) + fq_j % uint32_t(G);
                *reinterpret_cast<uint4*>(sQ + row * 128u + ((fq_c ^ (row & 7u)) << 4)) = fq_lo;
                *reinterpret_cast<uint4*>(sQ + 2048u + row * 128u + ((fq_c ^ (row & 7u)) << 4)) = fq_hi;
                if (owns_last0 && pp.f.q_rope_out != nullptr) {
                    uint16_t* qo = reinterpret_cast<uint16_t*>(pp.f.q_rope_out) + (size_t(hdr0.w) * Hq + fq_j) * kD;
                    *reinterpret_cast<uint4*>(qo + fq_c * 8) = fq_lo;
                    *reinterpret_cast<uint4*>(qo + 64 + fq_c * 8) = fq_hi;
                }
            }
            fence_async_smem();
            bar_sync(4u, 128u);
            if (tid == 0) mbar_arrive(&q_ready[0]);
        }
        ok = !softmax_or(!ok);
        uint32_t g = 0;
        bool set_known = false;
        for (uint32_t si = seg_begin; si < seg_end && ok; ++si) {
            const KriyaTcSeg seg = seg_at(si);
            const uint32_t req = seg.req;
            const uint32_t row_tokens = seg.row_tokens;
            const uint32_t tok_lo = max(seg.blk_lo * kPage, seg.tok_first), tok_hi = min(seg.blk_hi * kPage, row_tokens);
            const uint32_t t0 = seg.blk_lo / kPagesPerTile, t1 = (seg.blk_hi + kPagesPerTile - 1) / kPagesPerTile;
            const bool empty = seg.blk_hi <= seg.blk_lo;
            float m_used[GH], m_thr[GH], l_own[GH];  // m_thr: the score above which the exponent reference moves
#pragma unroll
            for (int i = 0; i < GH; ++i) {
                m_used[i] = m_thr[i] = -INFINITY;
                l_own[i] = 0.0f;
            }
            for (uint32_t t = empty ? t1 : t0; t < t1; ++t, ++g) {
                if (*abort_flag) { ok = false; break; }
                ok = warp_wait_l(wait_ns, &s_full[g & 1u], (g >> 1) & 1u);
                if (!ok) break;
                tc_fence_after();
                // this row's scores: columns 8 hd' + jj of the tile's score accumulator; the columns of the row's own KV head count
                uint32_t ra[4], rb[4];
                const uint32_t s_col = tmem_base + lane_addr + ((g & 1u) ? kColS1 : kColS0) + jj0;
                tmem_ld4(s_col, ra);
                tmem_ld4(s_col + 8u, rb);
                tmem_wait_ld();
                const uint32_t tok = t * kTileTokens + pg * kPage + tk;
                // only a piece's first and last tile can hold tokens outside the piece
                const bool inner = t * kTileTokens >= tok_lo && (t + 1u) * kTileTokens <= tok_hi;
                const bool valid = inner || (tok >= tok_lo && tok < tok_hi);
                float s[GH];
                bool over = false;
#pragma unroll
                for (int i = 0; i < GH; ++i) {
                    float x = __uint_as_float(hd ? rb[i] : ra[i]) * scale2;
                    if (softcap) x = softcap_log2(x, a.logit_softcap);
                    s[i] = (valid && uint32_t(i) < nj) ? x : -INFINITY;
                    over = over || (s[i] > m_thr[i]);
                }
                if (softmax_or(over)) {
                    float alpha[GH];
#pragma unroll
                    for (int i = 0; i < GH; ++i) alpha[i] = 1.0f;
                    // per-head maximum over the tile: the 16 tokens of this half-warp, then the four pages
                    float mx[GH];
#pragma unroll
                    for (int i = 0; i < GH; ++i) mx[i] = s[i];
#pragma unroll
                    for (int oi = 0; oi < 4; ++oi)  // the head's 16 lanes differ in bits 4, 2, 1, 0
#pragma unroll
                        for (int i = 0; i < GH; ++i) mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xFFFFFFFFu, mx[i], oi == 0 ? 16 : (4 >> (oi - 1))));
                    if (tk == 0u) {
#pragma unroll
                        for (int i = 0; i < GH; ++i)
                            if (uint32_t(i) < nj) red[(pg * 2u + hd) * 8u + jj0 + uint32_t(i)] = mx[i];
                    }
                    softmax_sync();
#pragma unroll
                    for (int i = 0; i < GH; ++i) {
                        const uint32_t c = hd * 8u + jj0 + uint32_t(i);
                        const float m_tile = (uint32_t(i) < nj) ? fmaxf(fmaxf(red[c], red[16u + c]), fmaxf(red[32u + c], red[48u + c])) : -INFINITY;
                        if (m_tile > m_used[i]) {
                            alpha[i] = (m_used[i] == -INFINITY) ? 0.0f : exp2f(m_used[i] - m_tile);
                            m_used[i] = m_tile;
                            m_thr[i] = m_tile + kRescale;
                        }
                    }
                    if (t > t0) {  // (a piece's first tile has nothing to rescale)
                        // the accumulator's columns belong to all query heads of the row: publish the factors
                        if (pg == 0u && tk == 0u) {
#pragma unroll
                            for (int i = 0; i < GH; ++i)
                                if (uint32_t(i) < nj) alpha_s[hd * 8u + jj0 + uint32_t(i)] = alpha[i];
                        }
                        softmax_sync();
                        ok = warp_wait_l(wait_ns, &tile_done[(g - 1u) % 6u], ((g - 1u) / 6u) & 1u);
                        if (!ok) break;
                        if (warp < 4u) {
                            tc_fence_after();
                            // O^T: lane = d, column = 16 head + jj (columns 8-15 of each head unused)
                            uint32_t o[32];
                            tmem_ld32(tmem_base + lane_addr + kColO, o);
                            tmem_wait_ld();
#pragma unroll
                            for (int cI = 0; cI < 32; ++cI) {
                                const float f = ((cI & 7) < G && (cI & 8) == 0) ? alpha_s[((cI >> 4) << 3) | (cI & 7)] : 1.0f;
                                o[cI] = __float_as_uint(__uint_as_float(o[cI]) * f);
                            }
                            tmem_st32(tmem_base + lane_addr + kColO, o);
                            tmem_wait_st();
                        }
                    }
#pragma unroll
                    for (int i = 0; i < GH; ++i) l_own[i] *= alpha[i];
                    softmax_sync();  // alpha_s and red may be rewritten by the next tile
                }
                if (g >= 2) {
                    ok = warp_wait_l(wait_ns, &tile_done[(g - 2u) % 6u], ((g - 2u) / 6u) & 1u);
                    if (!ok) break;
                }
                {
                    uint8_t* pbuf = sP + (g & 1u) * kPBytes;
#pragma unroll
                    for (int i = 0; i < GH; ++i) {
                        if (uint32_t(i) < nj) {
                            const float p = (s[i] == -INFINITY) ? 0.0f : fast_exp2(s[i] - m_used[i]);
                            l_own[i] += p;
                            *reinterpret_cast<uint16_t*>(pbuf + p_off[i]) = T::store(p);
                        }
                    }
                }
                // The V half must have landed before rows of it are cleared - and before the tile's P.V is issued: the softmax
                // warps wait for it here (they have time to spare), so that the MMA warp, which sets the pace, waits for one
                // barrier per tile only.
                ok = warp_wait_l(wait_ns, &v_full[g % kStages], (g / kStages) & 1u);
                if (!ok) break;
                if (!valid) {  // this token's V rows must contribute nothing (0 * garbage must not appear): this thread clears one
                    uint4* vrow = reinterpret_cast<uint4*>(sKV + (g % kStages) * kStageBytes + v_row_off);
#pragma unroll
                    for (int cI = 0; cI < 8; ++cI) vrow[cI] = make_uint4(0u, 0u, 0u, 0u);
                }
                tc_fence_before();
                fence_async_smem();
                mbar_arrive(&p_ready[g & 1u]);
            }
            if (!ok) break;
            // ---- end of the run piece ---------------------------------------------------------------------------
            // sums per head: the 16 tokens of this half-warp, then the four pages
            float l_tot[GH];
#pragma unroll
            for (int i = 0; i < GH; ++i) l_tot[i] = l_own[i];
#pragma unroll
            for (int oi = 0; oi < 4; ++oi)
#pragma unroll
                for (int i = 0; i < GH; ++i) l_tot[i] += __shfl_xor_sync(0xFFFFFFFFu, l_tot[i], oi == 0 ? 16 : (4 >> (oi - 1)));
            if (tk == 0u) {
#pragma unroll
                for (int i = 0; i < GH; ++i)
                    if (uint32_t(i) < nj) red[(pg * 2u + hd) * 8u + jj0 + uint32_t(i)] = l_tot[i];
            }
            softmax_sync();
            if (pg == 0u && tk == 0u) {  // (m, l) of the piece for this thread's heads, row order j = hd * G + jj
#pragma unroll
                for (int i = 0; i < GH; ++i) {
                    if (uint32_t(i) < nj) {
                        const uint32_t c = hd * 8u + jj0 + uint32_t(i), j = hd * uint32_t(G) + jj0 + uint32_t(i);
                        ml_s[j * 2u + 0u] = m_used[i];
                        ml_s[j * 2u + 1u] = (red[c] + red[16u + c]) + (red[32u + c] + red[48u + c]);
                    }
                }
            }
            // the accumulator: lane = d, columns 16 head + jj; threads 0-127 take KV head 0's columns, threads 128-255 head 1's
            uint32_t o8[8];
#pragma unroll
            for (int cI = 0; cI < 8; ++cI) o8[cI] = 0u;
            if (!empty) {
                ok = warp_wait_l(wait_ns, &tile_done[(g - 1u) % 6u], ((g - 1u) / 6u) & 1u);
                if (!ok) break;
                tc_fence_after();
                tmem_ld8(tmem_base + lane_addr + kColO + 16u * fin_hd, o8);
                tmem_wait_ld();
                tc_fence_before();
            }
            softmax_sync();
            float Mh[G], Lh[G], Oh[G];
#pragma unroll
            for (int jj = 0; jj < G; ++jj) {
                Mh[jj] = empty ? -INFINITY : ml_s[(fin_hd * G + jj) * 2];
                Lh[jj] = empty ? 0.0f : ml_s[(fin_hd * G + jj) * 2 + 1];
                Oh[jj] = __uint_as_float(o8[jj]);
            }
            softmax_sync();  // ml_s is free again
            if (pdl == 3u) pdl_wait_previous_grid();
            const size_t row0 = size_t(req) * Hq + fin_hd * G;
            const bool split = seg.n_parts > 1u;
            const bool finisher = !split || (seg.n_parts <= pp.late_parts && seg.slot + 1u == seg.first_slot + seg.n_parts);
            if (finisher) {
                if (split) {
                    const bool mine = gather_merge<G>(pp.ll_o, pp.ll_ml, seg, pp.epoch, wait_ns, fin_stage, 2u + fin_hd, d, uint32_t(HQ),
                                                      fin_hd * G, Mh, Lh, Oh);
                    ok = !softmax_or(!mine);
                    if (!ok) break;
                }
#pragma unroll
                for (int jj = 0; jj < G; ++jj) {
                    if (state_mode) {
                        a.state_o[(row0 + jj) * kD + d] = Oh[jj];
                        if (d == 0) {
                            a.state_m[row0 + jj] = Mh[jj] / kLog2e;
                            a.state_l[row0 + jj] = Lh[jj];
                        }
                    } else {
                        reinterpret_cast<uint16_t*>(a.out)[(row0 + jj) * kD + d] = T::store(Oh[jj] / fmaxf(Lh[jj], 1e-12f));
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
                    ok = !softmax_or(st != 1u);
                    if (!ok) break;
                    set_known = true;
                }
                const size_t prow = size_t(seg.slot) * HQ + fin_hd * G;
#pragma unroll
                for (int jj = 0; jj < G; ++jj) {
                    ll_store(&pp.ll_o[(prow + jj) * kD + d], Oh[jj], pp.epoch);
                    if (d == uint32_t(2 * jj)) ll_store(&pp.ll_ml[(prow + jj) * 2 + 0], Mh[jj], pp.epoch);
                    if (d == uint32_t(2 * jj + 1)) ll_store(&pp.ll_ml[(prow + jj) * 2 + 1], Lh[jj], pp.epoch);
                }
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
    if (warp == 9) {
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
    const size_t smem = size_t(kStages) * kStageBytes + kQBufs * kQBytes + 2 * kPBytes + 2048 + 64 + 128 + 448 + 8 * sizeof(KriyaTcSeg) + 16 * 256 + 512 + 1024;
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

// 5-D maps over the K and V pools of all layers: dimensions (d_lo 64, token 16, half of d 2, head 2, page), strides (512,
// 128, 256, 8192) bytes for V: a V box is a whole page and lands as [head][half][token][64].  The K map splits the tokens:
// dimensions (d_lo 64, token 8, half 2, head 2, (page, eight-token group)), strides (512, 128, 256, 4096) bytes; its box
// {64, 8, 2, 2, 2} is a whole page as well and lands as [group][head][half][token][64] (see kKBlock).
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
    const cuuint64_t dims_v[5] = {64, 16, 2, 2, total_pages}, dims_k[5] = {64, 8, 2, 2, 2 * total_pages};
    const cuuint64_t strides_v[4] = {512, 128, 256, 8192}, strides_k[4] = {512, 128, 256, 4096};
    const cuuint32_t box_v[5] = {64, 16, 2, 2, 1}, box_k[5] = {64, 8, 2, 2, 2};
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    void* pools[2] = {pool_k, pool_v};
    void* outs[2] = {out_map_k, out_map_v};
    for (int i = 0; i < 2; ++i) {
        const CUresult r = enc(static_cast<CUtensorMap*>(outs[i]), CU_TENSOR_MAP_DATA_TYPE_UINT16, 5, pools[i], i == 0 ? dims_k : dims_v, i == 0 ? strides_k : strides_v, i == 0 ? box_k : box_v, estr,
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
