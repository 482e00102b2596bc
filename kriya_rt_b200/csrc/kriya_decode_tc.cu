// Paged GQA decode attention on the tensor cores, head_dim 128 (the job of bsr_paged_gqa_decode_stage1 and
// bsr_paged_gqa_split_k_reduce, kernels/metal/paged_gqa_and_deltanet.metal:242-495,1474-1525).
//
// Why tensor cores for a bandwidth-bound op: with G query heads packed per KV head the fp32 path needs
// 2*G FMA per cached element; at G = 8 the instruction stream alone takes longer than the HBM transfer
// (measured on the CUDA-core kernel).  Here the KV tile sits on the M axis of the MMA, so the arithmetic is
// a handful of tiny tcgen05.mma per 64 KB of cache and the kernel is left with the HBM stream.
//
// Shape of the kernel (persistent, one CTA per SM, 192 threads)
//   - Work: every (plan row, KV head) is a run of 128-token tiles (8 pages).  All runs laid end to end form
//     one tile stream that the host cuts into equal contiguous pieces, one per CTA, so every SM streams the
//     same number of bytes.  A run cut across CTAs leaves partial (m, l, o) states in scratch; the last
//     piece to finish (atomic ticket, no waiting) merges them.
//   - Warp 4 (producer) walks its piece: per tile it reads up to 8 page indices and issues TMA tensor loads
//     of K and V ([16 tokens] x [64 d] boxes, 128-byte swizzle, no multicast) into a 3-stage shared-memory
//     ring.
//   - Warp 5 (one thread) issues tcgen05.mma:  S^T[128 tokens x 16] = K_tile . Q^T   (K-major operands) and
//     O^T[128 d x 16] += V_tile^T . P^T  (V consumed in place as an MN-major operand), accumulators in TMEM.
//     S^T of tile g+1 is issued before P.V of tile g so the softmax overlaps the tensor pipe.
//   - Warps 0-3: thread t owns token t of the tile (TMEM lane t of S^T) and dimension t of the output (lane t
//     of O^T).  Per tile: read 16 scores, mask tokens past the row end, column max by warp shuffles plus a
//     4-warp exchange in shared memory, exp2, write P (storage dtype) into the swizzled operand tile, keep
//     the running sum per lane, rescale O^T in TMEM only when a head's max moved by more than 2^8.
//   - Warp 7 (stager) prepares each run piece ahead of time: the G query heads as a 16-row MMA operand (rotated in
//     flight when the append is fused) and, fused, the rotated new key and the new value written to their cache slot
//     before the producer loads that page.
//   - Warp 6 takes over the cross-CTA merge of a piece that is not the CTA's last one, so the softmax warps go
//     straight on to the next run while partial states are published, ticketed and (if last) merged.
//   - Every mbarrier wait is bounded; on expiry the kernel records a status word, abandons its piece,
//     frees its TMEM and returns.
//
// HBM roofline: algorithmic bytes per launch = attended tokens * 2 * Hkv * D * 2 B; every K/V byte is read
// from HBM once (one TMA load) and from shared memory once (one MMA operand read).
#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>

#include "kriya_tc.cuh"

// This file is compiled twice: as it is (128-token tiles, one CTA per SM) and through kriya_decode_tc64.cu with
// KRIYA_TC_TILE64 defined (64-token tiles, two CTAs per SM); the two builds live in different namespaces and export
// differently named launchers, and the context picks one per plan.
#ifdef KRIYA_TC_TILE64
#define KRIYA_TC_NS t64
#define KRIYA_TC_FN(name) name##_t64
#else
#define KRIYA_TC_NS t128
#define KRIYA_TC_FN(name) name
#endif

namespace kriya {
namespace KRIYA_TC_NS {

constexpr int kTcD = 128;
// Tile of the K/V stream.  The default is 128 tokens with one resident CTA per SM.  KRIYA_TC_TILE64 builds the variant
// with 64-token tiles (M = 64 score MMAs: accumulator row r lands in tensor-memory lane (r % 16) + 32 * (r / 16), so each
// softmax warp owns 16 tokens of a tile and its upper 16 lanes idle) whose rings fit twice into an SM.
#ifdef KRIYA_TC_TILE64
constexpr int kTcTile = 64;
constexpr int kTcCtasPerSm = 2;
constexpr int kTcQBufs = 2;
#else
constexpr int kTcTile = 128;          // tokens per tile
constexpr int kTcCtasPerSm = 1;
constexpr int kTcQBufs = 3;
#endif
constexpr int kTcPage = 16;
constexpr int kTcPagesPerTile = kTcTile / kTcPage;
constexpr int kTcStages = 3;
constexpr int kTcThreads = 256;  // warps 0-3 softmax, 4 producer, 5 MMA issuer, 6 deferred merge, 7 query/new-token stager
constexpr int kTcN = 16;              // MMA N: query heads of one KV head, zero padded
constexpr float kTcLog2e = 1.4426950408889634f;
constexpr float kTcRescale = 8.0f;
constexpr uint32_t kTcPanel = kTcTile * 128;       // one 64-d panel of a tile
constexpr uint32_t kTcKvBytes = 2 * kTcPanel;      // K (or V) tile, both panels: 32 KB at 128 tokens
constexpr uint32_t kTcQBytes = 2 * 16 * 128;       // 16 rows x 256 B as two panels: 4 KB
constexpr uint32_t kTcPBytes = (kTcTile / 64) * 16 * 128;  // [16 heads][tile tokens] as 64-token panels: 4 KB at 128 tokens
constexpr uint32_t kTcTmemCols = 64;
constexpr uint32_t kColS0 = 0, kColS1 = 16, kColO = 32;

struct TcParams {
    KriyaDecodeArgs a;
    const KriyaTcSeg* segs;
    const uint32_t* cta_seg_ptr;  // [grid + 1]
    uint32_t layer_row0;
    // runs cut into more pieces than this are not merged by their last piece but by late_merge_kernel after the launch
    uint32_t late_parts;
    uint32_t n_seg;  // host side only: segments of the list (grid of the late merge)
    // Partial states of split runs, written as (value, epoch) pairs so that a reader needs no fence and no flag of its own
    // (see ll_store): ll_o [slot][G][128], ll_ml [slot][G][2] = (running max in log2 units, sum).
    uint2* ll_o;
    uint2* ll_ml;
    uint32_t* set_done;    // CTAs that have finished with this scratch set, over all launches so far
    uint32_t done_expect;  // its value once every earlier launch that used the set has finished with it
    uint32_t epoch;        // this launch's stamp, never zero
    KriyaFusedAppend f;
};

// RoPE of eight (x[i], x[i + D/2]) pairs held as two 16-byte chunks, in the operation order of the append kernel
// (fma(x0, c, -(x1 * s)), fma(x0, s, x1 * c), round to nearest even), so both paths write identical bits.  The
// cos/sin pairs are fetched (or computed) separately: they depend on the position and the chunk only, so one fetch serves
// every head of a run and its loads go out together with the loads of the vectors they rotate.
// Long scalar routines are functions of their own: inlined into unrolled loops they are a large share of the kernel's
// code, and code that runs once per CTA is paid for in instruction-cache misses.
static __device__ __noinline__ float2 rope_pair_coeff(uint32_t i, uint32_t position, uint32_t rotary_dim, float theta) {
    const float freq_exp = float(2u * i) / float(rotary_dim);
    const float inv_freq = powf(theta, -freq_exp);
    const float angle = __fmul_rn(float(position), inv_freq);
    return make_float2(cosf(angle), sinf(angle));
}
static __device__ __noinline__ float softcap_log2(float x, float cap) {
    return tanhf(fminf(fmaxf(x / cap, -15.0f), 15.0f)) * cap * kTcLog2e;
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
            if (first_pair + 2 * j + e < half_rot) {  // pairs past the rotary dimension keep their bits
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

// Programmatic dependent launch: both are no-ops when the launch did not ask for it.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_previous_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void named_bar_sync_128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// Barrier over the 128 softmax threads that also ORs a predicate across them.
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

// A partial-state word travels with the stamp of the launch that wrote it: one 8-byte store, so a reader that sees the
// stamp of its own launch also sees the value, without a fence on the writer's side or a separate flag to wait for.
__device__ __forceinline__ void ll_store(uint2* p, float v, uint32_t epoch) {
    asm volatile("st.global.cg.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(epoch) : "memory");
}
// Loads of such words are volatile: they go to L2 (the writer may be any SM) and a polling loop really repeats them
// (an ordinary load may be moved out of the loop by the assembler).  A polling loop issues a whole batch of them before
// it looks at the first result, so that the batch is in flight together.
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

// Waits (bounded) until the counter of a scratch set says that every CTA of every earlier launch on the set is done.
__device__ __forceinline__ bool warp_wait_l(uint64_t limit_ns, uint64_t* bar, uint32_t parity) { return warp_wait(bar, parity, limit_ns); }
__device__ __forceinline__ bool wait_set_free(const uint32_t* set_done, uint32_t done_expect, uint64_t wait_ns) {
    const uint64_t t_start = global_timer_ns();
    for (uint32_t spin = 0;; ++spin) {
        if (int32_t(ld_volatile_u32(set_done) - done_expect) >= 0) return true;
        if ((spin & 63u) == 63u && global_timer_ns() - t_start > wait_ns) return false;
    }
}

// The run's last piece gathers the other pieces' partial states and finishes the run.  Called by the 128 softmax threads
// with their own piece's state in registers: thread t owns output dimension t; M / L are the piece's running maximum (log2
// units) and sum per head, O its accumulator values for dimension t.  Other pieces are taken four at a time; every load of
// a chunk is issued before any is examined and is repeated until it carries this launch's stamp (bounded).  Returns false
// when a stamp never arrived.
template <int G>
__device__ __forceinline__ bool gather_merge(const uint2* __restrict__ ll_o, const uint2* __restrict__ ll_ml, const KriyaTcSeg& seg,
                                             uint32_t epoch, uint64_t wait_ns, float* stage, uint32_t t, float (&M)[G], float (&L)[G], float (&O)[G]) {
    const uint32_t others = seg.n_parts - 1u;
    for (uint32_t c0 = 0; c0 < others; c0 += 4u) {
        const uint32_t cnt = min(4u, others - c0);
        const size_t slot0 = size_t(seg.first_slot) + c0;
        uint2 w[4][G];
        uint2 mlw = make_uint2(0u, epoch);
        const bool has_ml = t < cnt * uint32_t(G) * 2u;  // (m, l) words of the chunk: [part][head][2], one per thread
        const uint2* mlp = &ll_ml[slot0 * G * 2 + (has_ml ? t : 0u)];
        bool got = false;
        const uint64_t t_start = global_timer_ns();
        for (uint32_t spin = 0; !got; ++spin) {
            // all loads first (a part past the chunk re-reads the chunk's last part), then the stamps
#pragma unroll
            for (int s2 = 0; s2 < 4; ++s2)
#pragma unroll
                for (int h = 0; h < G; ++h)
                    w[s2][h] = ll_load(&ll_o[((slot0 + min(uint32_t(s2), cnt - 1u)) * G + h) * kTcD + t]);
            mlw = ll_load(mlp);
            uint32_t bad = mlw.y ^ epoch;
#pragma unroll
            for (int s2 = 0; s2 < 4; ++s2)
#pragma unroll
                for (int h = 0; h < G; ++h) bad |= w[s2][h].y ^ epoch;
            got = bad == 0u;
            if (!got && (spin & 63u) == 63u && global_timer_ns() - t_start > wait_ns) break;
        }
        if (has_ml) stage[t] = __uint_as_float(mlw.x);
        if (bar_or_128(!got)) return false;  // also orders the writes to `stage` before its readers
        // the weights depend on (piece, head) only: thread h works them out for head h, the others just accumulate
        float* wsm = stage + 64;       // [4][G] weights
        float* hsm = stage + 64 + 32;  // [3][8]: new maximum, new sum, factor on what was there
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
        named_bar_sync_128();
#pragma unroll
        for (int h = 0; h < G; ++h) {
            float oacc = O[h] * hsm[16 + h];
#pragma unroll
            for (int s2 = 0; s2 < 4; ++s2) oacc = fmaf(wsm[s2 * G + h], __uint_as_float(w[s2][h].x), oacc);
            O[h] = oacc;
            M[h] = hsm[h];
            L[h] = hsm[8 + h];
        }
        named_bar_sync_128();  // `stage` is rewritten by the next chunk
    }
    return true;
}

template <int G, typename T>
__global__ void __launch_bounds__(kTcThreads, kTcCtasPerSm)
decode_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, TcParams pp) {
    constexpr uint32_t FMT = (T::kDtype == KRIYA_DTYPE_BF16) ? 1u : 0u;
    constexpr uint32_t IDESC_S = make_idesc(FMT, kTcTile, kTcN, 0, 0);  // A = K tile (K-major), B = Q (K-major)
    constexpr uint32_t IDESC_O = make_idesc(FMT, 128, kTcN, 1, 0);  // A = V tile (MN-major), B = P (K-major)

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
    uint8_t* sK = sm;                                   // [stages][32 KB]
    uint8_t* sV = sK + kTcStages * kTcKvBytes;          // [stages][32 KB]
    uint8_t* sQ = sV + kTcStages * kTcKvBytes;          // [3][4 KB]
    uint8_t* sP = sQ + kTcQBufs * kTcQBytes;                   // [2][4 KB]
    float* red = reinterpret_cast<float*>(sP + 2 * kTcPBytes);  // [4 warps][16] / merge staging [8][G][2]
    uint64_t* bars = reinterpret_cast<uint64_t*>(red + 128);
    uint64_t* kv_full = bars;                     // [stages]
    uint64_t* kv_empty = bars + kTcStages;        // [stages]
    uint64_t* s_full = bars + 2 * kTcStages;      // [2]
    uint64_t* p_ready = bars + 2 * kTcStages + 2; // [2], 128 arrivals each; tile g uses p_ready[g & 1]
    uint64_t* pv_done = bars + 2 * kTcStages + 4; // [2]; P.V of tile g commits to pv_done[g & 1]
    uint64_t* q_ready = bars + 2 * kTcStages + 6;   // [3]; run r's query operand is staged in buffer r % 3
    uint64_t* q_free = bars + 2 * kTcStages + 9;    // [3]; all S^T MMAs of the run that used the buffer are complete
    uint64_t* kv_ready = bars + 2 * kTcStages + 12; // [3]; run r's new-token K/V row is in the cache (fused append)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kTcStages + 15);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    volatile uint32_t* set_free_s = tmem_slot + 2;  // 0: not known yet, 1: the scratch set may be written, 2: the wait for it gave up
    KriyaTcSeg* segs_s = reinterpret_cast<KriyaTcSeg*>(tmem_slot + 4 + 128);  // first 8 segment records of this CTA

    const KriyaDecodeArgs& a = pp.a;
    const uint64_t wait_ns = a.wait_ns;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    if (threadIdx.x == 0) {
    }
    const uint32_t seg_begin = pp.cta_seg_ptr[blockIdx.x], seg_end = pp.cta_seg_ptr[blockIdx.x + 1];
    // The next launch of the stream may start as SMs free up (it decides itself what it must wait for, see `pdl` below).
    if (threadIdx.x == 0) pdl_launch_dependents();
    if (seg_begin == seg_end) {  // whole CTA idle: nothing allocated yet
        // Every CTA counts itself off in the scratch set's counter, and only once the set's earlier launches are complete:
        // the counter then never runs ahead of them (see the guard in warp 6 below).
        if (threadIdx.x == 0) {
            if (!wait_set_free(pp.set_done, pp.done_expect, pp.a.wait_ns)) atomicMax(pp.a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            atomicAdd(pp.set_done, 1u);
        }
        return;
    }

    if (tid == 0) {
        for (int s = 0; s < kTcStages; ++s) {
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
        tmem_alloc(tmem_slot, kTcTmemCols);
        tmem_relinquish();
    }
    {   // every role walks the same segment list: keep the first records in shared memory
        const uint32_t nstage = min(seg_end - seg_begin, 8u) * uint32_t(sizeof(KriyaTcSeg) / 4);
        const uint32_t* src = reinterpret_cast<const uint32_t*>(pp.segs + seg_begin);
        for (uint32_t i = tid; i < nstage; i += kTcThreads) reinterpret_cast<uint32_t*>(segs_s)[i] = src[i];
    }
    auto seg_at = [&](uint32_t si) -> KriyaTcSeg { return (si - seg_begin < 8u) ? segs_s[si - seg_begin] : pp.segs[si]; };
    // The padding heads of the Q and P operand tiles must be zero.  The K/V ring needs no clearing: a K row
    // that is never loaded only produces a score that is masked by selection, and the V row of every masked
    // token is cleared by the softmax thread that owns it.
    for (uint32_t i = tid; i < (kTcQBufs * kTcQBytes + 2 * kTcPBytes) / 16; i += kTcThreads)
        reinterpret_cast<uint4*>(sQ)[i] = make_uint4(0u, 0u, 0u, 0u);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t Hq = a.num_q_heads, Hkv = a.num_kv_heads;
    // How this launch relates to the kernel before it in the stream when it was allowed to start early (programmatic
    // dependent launch): 1 = nothing but the set-up above may precede that kernel's completion; 3 = only the cache and the
    // plan are older than that kernel, so the K/V stream starts at once while everything that touches activations (queries,
    // the new token's K/V, outputs) waits; 2 = nothing to wait for; 0 = ordinary launch.
    const uint32_t pdl = pp.f.overlap_previous;
    if (pdl == 1u) pdl_wait_previous_grid();

    if (warp == 4) {
        // ---- producer: page indices one tile ahead, TMA loads into the ring -------------------------------
        uint32_t g = 0;     // tiles issued by this CTA so far
        uint32_t runs = 0;  // non-empty run pieces started so far
        bool ok = true;
        const bool fused = pp.f.k_in != nullptr;
        for (uint32_t si = seg_begin; si < seg_end && ok; ++si) {
            const KriyaTcSeg seg = seg_at(si);
            const uint32_t t0 = seg.blk_lo / kTcPagesPerTile, t1 = (seg.blk_hi + kTcPagesPerTile - 1) / kTcPagesPerTile;
            if (seg.blk_hi <= seg.blk_lo) continue;
            const int32_t* table = a.indices + seg.tbl_off;
            const bool owns_last = fused && seg.row_tokens > 0u && uint64_t(seg.blk_hi) * kTcPage >= seg.row_tokens;
            int32_t pf_blk = 0;
            bool pf_valid = false;
            for (uint32_t t = t0; t < t1; ++t, ++g) {
                if (*abort_flag) { ok = false; break; }
                const uint32_t stage = g % kTcStages;
                const uint32_t p_lo = max(t * kTcPagesPerTile, seg.blk_lo), p_hi = min((t + 1) * kTcPagesPerTile, seg.blk_hi);
                const uint32_t npages = p_hi - p_lo;
                const uint32_t my_page = p_lo + lane;
                int32_t blk = pf_blk;
                if (!pf_valid && lane < npages) blk = table[my_page];
                if (g >= kTcStages && !warp_wait_l(wait_ns, &kv_empty[stage], ((g / kTcStages) - 1u) & 1u)) {
                    ok = false;
                    break;
                }
                // the piece's last tile reads the slot the stager warp writes: wait until it is in the cache
                if (owns_last && t + 1u == t1 && !warp_wait_l(wait_ns, &kv_ready[runs % uint32_t(kTcQBufs)], (runs / uint32_t(kTcQBufs)) & 1u)) {
                    ok = false;
                    break;
                }
                if (lane < npages && uint32_t(blk) >= a.num_blocks) {
                    atomicMax(a.status, uint32_t(KRIYA_DEV_BAD_BLOCK_INDEX));
                    blk = 0;
                }
                if (lane == 0) mbar_arrive_expect_tx(&kv_full[stage], npages * uint32_t(4 * kTcPage * 128));
                __syncwarp();
                if (lane < npages) {
                    const int32_t y = int32_t(pp.layer_row0) + blk * kTcPage;
                    const uint32_t row_off = (my_page - t * kTcPagesPerTile) * (kTcPage * 128);
#pragma unroll
                    for (int p = 0; p < 2; ++p) {
                        const int32_t x = int32_t(seg.kv_head) * kTcD + p * 64;
                        tma_load_2d(sK + stage * kTcKvBytes + p * kTcPanel + row_off, &map_k, x, y, &kv_full[stage]);
                        tma_load_2d(sV + stage * kTcKvBytes + p * kTcPanel + row_off, &map_v, x, y, &kv_full[stage]);
                    }
                }
                pf_valid = t + 1u < t1;
                if (pf_valid) {
                    const uint32_t n_lo = (t + 1u) * kTcPagesPerTile, n_hi = min((t + 2u) * kTcPagesPerTile, seg.blk_hi);
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
        // ---- stager: per run piece, the query operand (rotated when fused) and the new token's K/V row ---------
        // Runs up to three pieces ahead of the MMA warp; a Q buffer is reused once q_free says that every S^T MMA
        // of its previous run has completed.
        uint32_t runs = 0;
        bool ok = true;
        const bool fused = pp.f.k_in != nullptr;
        if (pdl == 3u) pdl_wait_previous_grid();
        for (uint32_t si = seg_begin; si < seg_end && ok; ++si) {
            const KriyaTcSeg seg = seg_at(si);
            if (seg.blk_hi <= seg.blk_lo) continue;
            if (*abort_flag) break;
            if (runs >= uint32_t(kTcQBufs) && !warp_wait_l(wait_ns, &q_free[runs % uint32_t(kTcQBufs)], ((runs / uint32_t(kTcQBufs)) - 1u) & 1u)) {
                ok = false;
                break;
            }
            const int32_t* table = a.indices + seg.tbl_off;
            const bool owns_last = fused && seg.row_tokens > 0u && uint64_t(seg.blk_hi) * kTcPage >= seg.row_tokens;
            uint8_t* qb = sQ + (runs % uint32_t(kTcQBufs)) * kTcQBytes;
            const uint16_t* qg = reinterpret_cast<const uint16_t*>(a.q) + (size_t(seg.req) * Hq + seg.kv_head * G) * kTcD;
            uint32_t position = 0;
            float2 cs[8];  // cos/sin of the run's position for this lane's chunk (fused form)
            if (!fused) {
                // 16 rows x 256 B as two swizzled K-major panels; rows >= G stay zero
                for (uint32_t i = lane; i < uint32_t(G) * 16u; i += 32u) {
                    const uint32_t h = i >> 4, c = i & 15u;
                    const uint4 val = *reinterpret_cast<const uint4*>(qg + h * kTcD + c * 8);
                    *reinterpret_cast<uint4*>(qb + (c >> 3) * 2048u + h * 128u + (((c & 7u) ^ (h & 7u)) << 4)) = val;
                }
            } else {
                // the usual decode step appends at position = tokens already in the row; then the segment record
                // already holds it and the dependent global load is skipped
                position = pp.f.positions_are_context ? seg.row_tokens - 1u : pp.f.positions[seg.req];
                // item i = (head i / 8, 16-byte chunk i % 8); a lane's items all share the chunk lane % 8, hence the
                // coefficients; every load of the run goes out before the first result is needed
                constexpr int ITEMS = (G * 8 + 31) / 32;
                const uint32_t c = lane & 7u;
                rope8_coeffs(cs, c * 8u, position, pp.f);
                uint4 lo[ITEMS], hi[ITEMS];
#pragma unroll
                for (int it = 0; it < ITEMS; ++it) {
                    const uint32_t h = (lane + 32u * it) >> 3;
                    if (h < uint32_t(G)) {
                        lo[it] = *reinterpret_cast<const uint4*>(qg + h * kTcD + c * 8);
                        hi[it] = *reinterpret_cast<const uint4*>(qg + h * kTcD + 64 + c * 8);
                    }
                }
#pragma unroll
                for (int it = 0; it < ITEMS; ++it) {
                    const uint32_t h = (lane + 32u * it) >> 3;
                    if (h < uint32_t(G)) {
                        rope8_apply<T>(lo[it], hi[it], c * 8u, cs, pp.f.rotary_dim / 2u);
                        *reinterpret_cast<uint4*>(qb + h * 128u + ((c ^ (h & 7u)) << 4)) = lo[it];
                        *reinterpret_cast<uint4*>(qb + 2048u + h * 128u + ((c ^ (h & 7u)) << 4)) = hi[it];
                        if (owns_last && pp.f.q_rope_out != nullptr) {
                            uint16_t* qo = reinterpret_cast<uint16_t*>(pp.f.q_rope_out) + (size_t(seg.req) * Hq + seg.kv_head * G + h) * kTcD;
                            *reinterpret_cast<uint4*>(qo + c * 8) = lo[it];
                            *reinterpret_cast<uint4*>(qo + 64 + c * 8) = hi[it];
                        }
                    }
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&q_ready[runs % uint32_t(kTcQBufs)]);
            if (owns_last) {
                // the rotated new key and the new value go into their cache slot; the fences order these generic-proxy
                // writes before the TMA loads (async proxy) the producer issues after it has seen kv_ready
                const uint32_t tok = seg.row_tokens - 1u;
                const uint32_t blk = uint32_t(table[tok / kTcPage]);
                if (blk >= a.num_blocks) {
                    if (lane == 0) atomicMax(a.status, uint32_t(KRIYA_DEV_BAD_BLOCK_INDEX));
                } else {
                    const size_t off = ((size_t(blk) * kTcPage + tok % kTcPage) * Hkv + seg.kv_head) * kTcD;
                    const size_t src = (size_t(seg.req) * Hkv + seg.kv_head) * kTcD;
                    uint16_t* kd = reinterpret_cast<uint16_t*>(pp.f.cache_k_w) + off;
                    uint16_t* vd = reinterpret_cast<uint16_t*>(pp.f.cache_v_w) + off;
                    const uint16_t* ks = reinterpret_cast<const uint16_t*>(pp.f.k_in) + src;
                    const uint16_t* vs = reinterpret_cast<const uint16_t*>(pp.f.v_in) + src;
                    if (lane < 8u) {  // chunk = lane: the coefficients fetched for the queries apply
                        uint4 lo = *reinterpret_cast<const uint4*>(ks + lane * 8);
                        uint4 hi = *reinterpret_cast<const uint4*>(ks + 64 + lane * 8);
                        rope8_apply<T>(lo, hi, lane * 8u, cs, pp.f.rotary_dim / 2u);
                        *reinterpret_cast<uint4*>(kd + lane * 8) = lo;
                        *reinterpret_cast<uint4*>(kd + 64 + lane * 8) = hi;
                    } else if (lane < 24u) {
                        const uint32_t c = lane - 8u;
                        *reinterpret_cast<uint4*>(vd + c * 8) = *reinterpret_cast<const uint4*>(vs + c * 8);
                    }
                }
                __threadfence();
                asm volatile("fence.proxy.async.global;" ::: "memory");
                __syncwarp();
            }
            if (lane == 0) mbar_arrive(&kv_ready[runs % uint32_t(kTcQBufs)]);
            ++runs;
        }
        if (!ok && lane == 0) {
            atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            *abort_flag = 1;
        }
    } else if (warp == 5) {
        // ---- MMA issuer ---------------------------------------------------------------------------------
        // Every lane runs this code, descriptor arithmetic included; only the tensor-core instructions themselves are
        // predicated on the elected lane, which keeps their operands in uniform registers (issued from inside a one-lane
        // branch every instruction costs about a hundred cycles, and the issue rate then bounds the kernel).
        const uint32_t el = (lane == 0) ? 1u : 0u;
        const uint64_t k_desc = smem_desc_sw128(smem_u32(sK), 16, 1024), q_desc = smem_desc_sw128(smem_u32(sQ), 16, 1024);
        const uint64_t v_desc = smem_desc_sw128(smem_u32(sV), kTcPanel, 1024), p_desc = smem_desc_sw128(smem_u32(sP), 16, 1024);
        // (segment, tile) cursor for the look-ahead S^T issue
        auto issue_s = [&](uint32_t gg, uint32_t qbuf) {
            const uint32_t stage = gg % kTcStages;
            const uint32_t d_tmem = tmem_base + ((gg & 1u) ? kColS1 : kColS0);
            const uint64_t ad = k_desc + uint64_t((stage * kTcKvBytes) >> 4), bd = q_desc + uint64_t((qbuf * kTcQBytes) >> 4);
#pragma unroll
            for (int ks = 0; ks < kTcD / 16; ++ks)
                umma_ss_pred(d_tmem, ad + uint64_t((uint32_t(ks / 4) * kTcPanel + uint32_t(ks % 4) * 32u) >> 4),
                             bd + uint64_t((uint32_t(ks / 4) * 2048u + uint32_t(ks % 4) * 32u) >> 4), IDESC_S, ks > 0 ? 1u : 0u, el);
            umma_commit_pred(&s_full[gg & 1u], el);
        };
        // flatten the piece into (tile -> q buffer, first-of-run) on the fly with two cursors
        uint32_t g = 0;
        bool ok = true;
        // look-ahead cursor
        uint32_t la_si = seg_begin, la_t = 0, la_t1 = 0, la_g = 0, la_run = 0;
        bool la_first = true;  // the look-ahead tile is the first of its run: its query operand must be in place
        auto la_load = [&]() {
            while (la_si < seg_end) {
                const KriyaTcSeg s2 = seg_at(la_si);
                if (s2.blk_hi > s2.blk_lo) {
                    la_t = s2.blk_lo / kTcPagesPerTile;
                    la_t1 = (s2.blk_hi + kTcPagesPerTile - 1) / kTcPagesPerTile;
                    la_first = true;
                    return true;
                }
                ++la_si;
            }
            return false;
        };
        bool la_valid = la_load();
        auto la_issue = [&]() -> bool {  // issue S^T for the look-ahead tile and advance the cursor
            if (!la_valid) return true;
            if (!warp_wait_l(wait_ns, &kv_full[la_g % kTcStages], (la_g / kTcStages) & 1u)) return false;
            if (la_first) {
                if (!warp_wait_l(wait_ns, &q_ready[la_run % uint32_t(kTcQBufs)], (la_run / uint32_t(kTcQBufs)) & 1u)) return false;
                la_first = false;
            }
            tc_fence_after();
            issue_s(la_g, la_run % uint32_t(kTcQBufs));
            ++la_g;
            if (++la_t >= la_t1) {
                umma_commit_pred(&q_free[la_run % uint32_t(kTcQBufs)], el);  // the run's last S^T is issued: its Q buffer frees when it completes
                ++la_si;
                ++la_run;
                la_valid = la_load();
            }
            return true;
        };
        ok = la_issue();  // S^T of the first tile
        for (uint32_t si = seg_begin; si < seg_end && ok; ++si) {
            const KriyaTcSeg seg = seg_at(si);
            if (seg.blk_hi <= seg.blk_lo) continue;
            const uint32_t t0 = seg.blk_lo / kTcPagesPerTile, t1 = (seg.blk_hi + kTcPagesPerTile - 1) / kTcPagesPerTile;
            for (uint32_t t = t0; t < t1 && ok; ++t, ++g) {
                if (*abort_flag) { ok = false; break; }
                ok = la_issue();  // S^T of tile g+1 (possibly of the next run) before P.V of tile g
                if (!ok) break;
                ok = warp_wait_l(wait_ns, &p_ready[g & 1u], (g >> 1) & 1u);
                if (!ok) break;
                tc_fence_after();
                {
                    const uint32_t stage = g % kTcStages;
                    const uint64_t ad = v_desc + uint64_t((stage * kTcKvBytes) >> 4), bd = p_desc + uint64_t(((g & 1u) * kTcPBytes) >> 4);
                    const uint32_t first = (t > t0) ? 1u : 0u;
#pragma unroll
                    for (int ks = 0; ks < kTcTile / 16; ++ks)
                        umma_ss_pred(tmem_base + kColO, ad + uint64_t((uint32_t(ks) * (kTcPage * 128)) >> 4),
                                     bd + uint64_t((uint32_t(ks / 4) * 2048u + uint32_t(ks % 4) * 32u) >> 4), IDESC_O, ks > 0 ? 1u : first, el);
                    umma_commit_pred(&kv_empty[stage], el);
                    umma_commit_pred(&pv_done[g & 1u], el);
                }
            }
        }
        if (!ok && lane == 0) {
            atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            *abort_flag = 1;
        }
    } else if (warp == 6) {
        // ---- scratch-set guard ----------------------------------------------------------------------------
        // The set this launch publishes partial states into was last used a few launches ago.  Launches of one step may
        // overlap (deeply, when a plan leaves most CTAs idle), so before anything is published every CTA of the set's
        // earlier launches must have finished with it: they count themselves off in set_done on their way out.  A CTA
        // counts itself off only after this guard has passed, so the counter holds completions of earlier launches only
        // until they are all in.  One lane looks the counter up while the first piece streams; the softmax threads find
        // the answer in shared memory.
        if (lane == 0) {
            const bool free_now = wait_set_free(pp.set_done, pp.done_expect, pp.a.wait_ns);
            if (!free_now) atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
            __threadfence_block();
            *set_free_s = free_now ? 1u : 2u;
        }
    } else {
        // ---- softmax warps ----------------------------------------------------------------------------------
        const uint32_t lane_addr = (warp * 32u) << 16;
        const bool softcap = a.logit_softcap > 0.0f;
        const float scale2 = softcap ? a.sm_scale : a.sm_scale * kTcLog2e;
        const bool state_mode = a.state_o != nullptr;
        uint32_t g = 0;
        bool ok = true;
        bool set_known = false;  // the scratch-set guard has been consulted
        for (uint32_t si = seg_begin; si < seg_end && ok; ++si) {
            const KriyaTcSeg seg = seg_at(si);
            const uint32_t req = seg.req;
            const uint32_t row_tokens = seg.row_tokens;
            const uint32_t tok_lo = max(seg.blk_lo * kTcPage, seg.tok_first), tok_hi = min(seg.blk_hi * kTcPage, row_tokens);
            const uint32_t t0 = seg.blk_lo / kTcPagesPerTile, t1 = (seg.blk_hi + kTcPagesPerTile - 1) / kTcPagesPerTile;
            const bool empty = seg.blk_hi <= seg.blk_lo;
            float m_used[G], l_lane[G];
#pragma unroll
            for (int h = 0; h < G; ++h) {
                m_used[h] = -INFINITY;
                l_lane[h] = 0.0f;
            }
            for (uint32_t t = empty ? t1 : t0; t < t1; ++t, ++g) {
                if (*abort_flag) { ok = false; break; }
                ok = warp_wait_l(wait_ns, &s_full[g & 1u], (g >> 1) & 1u);
                if (!ok) break;
                tc_fence_after();
                uint32_t r[16];
                tmem_ld16(tmem_base + lane_addr + ((g & 1u) ? kColS1 : kColS0), r);
                tmem_wait_ld();
                // the token (= accumulator row) this thread owns in the tile, and whether it owns one at all
                const uint32_t tile_row = (kTcTile == 128) ? tid : warp * 16u + lane;
                const bool has_row = (kTcTile == 128) || lane < 16u;
                const uint32_t tok = t * kTcTile + tile_row;
                const bool valid = has_row && tok >= tok_lo && tok < tok_hi;
                float s[G];
                bool over = false;  // does this token push some head's score past the exponent reference?
#pragma unroll
                for (int h = 0; h < G; ++h) {
                    float x = __uint_as_float(r[h]) * scale2;
                    if (softcap) x = softcap_log2(x, a.logit_softcap);
                    s[h] = valid ? x : -INFINITY;
                    over = over || (s[h] > m_used[h] + kTcRescale);
                }
                // One barrier-with-OR tells all 128 threads whether any score in the tile outgrew its reference.
                // Only then (first tile of a run, or a jump of more than 2^8) is the per-head column maximum
                // reduced and the accumulator rescaled; otherwise the reference is kept, which is exact.
                float alpha[G];
#pragma unroll
                for (int h = 0; h < G; ++h) alpha[h] = 1.0f;
                if (bar_or_128(over)) {
                    float mx[G];
#pragma unroll
                    for (int h = 0; h < G; ++h) mx[h] = s[h];
#pragma unroll
                    for (int off = 16; off >= 1; off >>= 1)
#pragma unroll
                        for (int h = 0; h < G; ++h) mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xFFFFFFFFu, mx[h], off));
                    if (lane == 0) {
#pragma unroll
                        for (int h = 0; h < G; ++h) red[warp * 16 + h] = mx[h];
                    }
                    named_bar_sync_128();
#pragma unroll
                    for (int h = 0; h < G; ++h) {
                        const float m_tile = fmaxf(fmaxf(red[h], red[16 + h]), fmaxf(red[32 + h], red[48 + h]));
                        if (m_tile > m_used[h]) {
                            alpha[h] = (m_used[h] == -INFINITY) ? 0.0f : exp2f(m_used[h] - m_tile);
                            m_used[h] = m_tile;
                        }
                    }
                    named_bar_sync_128();  // everyone has read `red`
                    if (t > t0) {
                        // O^T holds earlier tiles: the previous P.V must be complete before it is rescaled
                        ok = warp_wait_l(wait_ns, &pv_done[(g - 1u) & 1u], ((g - 1u) >> 1) & 1u);
                        if (!ok) break;
                        tc_fence_after();
                        uint32_t o[16];
                        tmem_ld16(tmem_base + lane_addr + kColO, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int h = 0; h < G; ++h) o[h] = __float_as_uint(__uint_as_float(o[h]) * alpha[h]);
                        tmem_st16(tmem_base + lane_addr + kColO, o);
                        tmem_wait_st();
                    }
#pragma unroll
                    for (int h = 0; h < G; ++h) l_lane[h] *= alpha[h];
                }
                // P buffer g&1 was last read by P.V of tile g-2
                if (g >= 2) {
                    ok = warp_wait_l(wait_ns, &pv_done[g & 1u], ((g >> 1) - 1u) & 1u);
                    if (!ok) break;
                }
                // probabilities of this token for the G heads -> P[h][token] (K-major, swizzled)
                {
                    uint8_t* pbuf = sP + (g & 1u) * kTcPBytes;
                    const uint32_t panel = tile_row >> 6, col = tile_row & 63u;
#pragma unroll
                    for (int h = 0; h < G; ++h) {
                        const float p = (s[h] == -INFINITY) ? 0.0f : fast_exp2(s[h] - m_used[h]);
                        l_lane[h] += p;
                        if (has_row)
                            *reinterpret_cast<uint16_t*>(pbuf + panel * 2048u + uint32_t(h) * 128u +
                                                         ((((col >> 3) ^ (uint32_t(h) & 7u)) << 4) | ((col & 7u) << 1))) = T::store(p);
                    }
                }
                // a token outside the run (past the row end, outside the block range, or a page that was not
                // loaded) must contribute nothing: its V row is cleared so that 0 * garbage cannot appear
                if (!valid && has_row) {
                    const uint32_t stage = g % kTcStages;
#pragma unroll
                    for (int p = 0; p < 2; ++p)
#pragma unroll
                        for (int c = 0; c < 8; ++c)
                            *reinterpret_cast<uint4*>(sV + stage * kTcKvBytes + p * kTcPanel + tile_row * 128u + (c << 4)) =
                                make_uint4(0u, 0u, 0u, 0u);
                }
                tc_fence_before();
                fence_async_smem();
                mbar_arrive(&p_ready[g & 1u]);
            }
            if (!ok) break;
            // ---- end of the run piece: total l per head, then O^T / l or the partial state ----------------
            float l_tot[G];
#pragma unroll
            for (int h = 0; h < G; ++h) l_tot[h] = l_lane[h];
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1)
#pragma unroll
                for (int h = 0; h < G; ++h) l_tot[h] += __shfl_xor_sync(0xFFFFFFFFu, l_tot[h], off);
            if (lane == 0) {
#pragma unroll
                for (int h = 0; h < G; ++h) red[warp * 16 + h] = l_tot[h];
            }
            named_bar_sync_128();
#pragma unroll
            for (int h = 0; h < G; ++h) l_tot[h] = (red[h] + red[16 + h]) + (red[32 + h] + red[48 + h]);
            named_bar_sync_128();
            uint32_t o[16];
#pragma unroll
            for (int h = 0; h < 16; ++h) o[h] = 0u;
            if (!empty) {
                ok = warp_wait_l(wait_ns, &pv_done[(g - 1u) & 1u], ((g - 1u) >> 1) & 1u);
                if (!ok) break;
                tc_fence_after();
                tmem_ld16(tmem_base + lane_addr + kColO, o);
                tmem_wait_ld();
                tc_fence_before();
            }
            const uint32_t d = tid;  // output dimension owned by this thread
            const size_t row0 = size_t(req) * Hq + seg.kv_head * G;
            // A run cut into pieces: every piece but the last publishes its partial state; the last piece (which its CTA
            // processes last, see the host's segment order) gathers them and finishes the run.  Runs in very many pieces
            // are finished by late_merge_kernel behind the launch instead; then every piece publishes.
            if (pdl == 3u) pdl_wait_previous_grid();  // outputs follow; returns at once when the wait is over already
            const bool split = seg.n_parts > 1u;
            const bool finisher = !split || (seg.n_parts <= pp.late_parts && seg.slot + 1u == seg.first_slot + seg.n_parts);
            if (finisher) {
                float Mh[G], Lh[G], Oh[G];
#pragma unroll
                for (int h = 0; h < G; ++h) {
                    Mh[h] = m_used[h];
                    Lh[h] = l_tot[h];
                    Oh[h] = __uint_as_float(o[h]);
                }
                if (split) {
                    ok = gather_merge<G>(pp.ll_o, pp.ll_ml, seg, pp.epoch, wait_ns, red, tid, Mh, Lh, Oh);
                    if (!ok) break;
                }
#pragma unroll
                for (int h = 0; h < G; ++h) {
                    if (state_mode) {
                        a.state_o[(row0 + h) * kTcD + d] = Oh[h];
                        if (d == 0) {
                            a.state_m[row0 + h] = Mh[h] / kTcLog2e;
                            a.state_l[row0 + h] = Lh[h];
                        }
                    } else {
                        reinterpret_cast<uint16_t*>(a.out)[(row0 + h) * kTcD + d] = T::store(Oh[h] / fmaxf(Lh[h], 1e-12f));
                    }
                }
            } else {
                // the scratch set must be free of its previous user (warp 6 looks that up at the start of the CTA)
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
                const size_t prow = size_t(seg.slot) * G;
#pragma unroll
                for (int h = 0; h < G; ++h) {
                    ll_store(&pp.ll_o[(prow + h) * kTcD + d], __uint_as_float(o[h]), pp.epoch);
                    if (tid == uint32_t(2 * h)) ll_store(&pp.ll_ml[(prow + h) * 2 + 0], m_used[h], pp.epoch);
                    if (tid == uint32_t(2 * h + 1)) ll_store(&pp.ll_ml[(prow + h) * 2 + 1], l_tot[h], pp.epoch);
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
    if (tid == 0) {
        atomicAdd(pp.set_done, 1u);  // every read of the scratch set by this CTA is complete, and warp 6 has seen the guard
    }
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTcTmemCols);
    }
}

// Merge of the runs that were cut into many pieces (one long row spread over the whole machine): one CTA per
// (run, query head), one thread per output dimension, eight partial states in flight per thread.  With dozens of
// pieces this is several times faster than the single warp or warpgroup that would otherwise do it at the tail of the
// decode launch.
template <int G, typename T>
__global__ void __launch_bounds__(kTcD) late_merge_kernel(KriyaDecodeArgs a, const KriyaTcSeg* segs, uint32_t late_parts,
                                                          const uint2* __restrict__ ll_o, const uint2* __restrict__ ll_ml) {
    const KriyaTcSeg seg = segs[blockIdx.x];
    if (seg.slot != seg.first_slot || seg.n_parts <= late_parts) return;  // not the first piece of a late-merged run
    const uint32_t h = blockIdx.y, d = threadIdx.x;
    float M = -INFINITY, L = 0.0f, O = 0.0f;
    for (uint32_t c0 = 0; c0 < seg.n_parts; c0 += 8u) {
        const uint32_t cnt = min(8u, seg.n_parts - c0);
        float ms[8], ls[8], ov[8];
#pragma unroll
        for (int s2 = 0; s2 < 8; ++s2) {
            const size_t row = size_t(seg.first_slot + c0 + min(uint32_t(s2), cnt - 1u)) * G + h;
            ms[s2] = uint32_t(s2) < cnt ? __uint_as_float(ll_ml[row * 2 + 0].x) : -INFINITY;
            ls[s2] = __uint_as_float(ll_ml[row * 2 + 1].x);
            ov[s2] = __uint_as_float(ll_o[row * kTcD + d].x);
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
    const size_t row0 = size_t(seg.req) * a.num_q_heads + seg.kv_head * G + h;
    if (a.state_o != nullptr) {
        a.state_o[row0 * kTcD + d] = O;
        if (d == 0) {
            a.state_m[row0] = M / kTcLog2e;
            a.state_l[row0] = L;
        }
    } else {
        reinterpret_cast<uint16_t*>(a.out)[row0 * kTcD + d] = T::store(O / fmaxf(L, 1e-12f));
    }
}

template <int G, typename T>
cudaError_t launch_tc_t(const TcParams& pp, const CUtensorMap& mk, const CUtensorMap& mv, uint32_t grid, int max_smem_optin,
                        bool overlap_previous, cudaStream_t s) {
    const size_t smem = size_t(2 * kTcStages) * kTcKvBytes + kTcQBufs * kTcQBytes + 2 * kTcPBytes + 512 + 320 + 512 + 8 * sizeof(KriyaTcSeg) + 1024;
    if (smem > size_t(max_smem_optin)) return cudaErrorInvalidValue;
    auto kern = decode_tc_kernel<G, T>;
    {   // the attribute belongs to the device: set it once on every device this process launches the kernel on
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
    if (overlap_previous) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(kTcThreads);
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
        kern<<<grid, kTcThreads, smem, s>>>(mk, mv, pp);
    }
    if (pp.late_parts != UINT32_MAX && pp.n_seg != 0u)
        late_merge_kernel<G, T><<<dim3(pp.n_seg, G), kTcD, 0, s>>>(pp.a, pp.segs, pp.late_parts, pp.ll_o, pp.ll_ml);
    return cudaGetLastError();
}

template <typename T>
cudaError_t launch_tc_g(uint32_t group, const TcParams& pp, const CUtensorMap& mk, const CUtensorMap& mv, uint32_t grid,
                        int max_smem_optin, bool ov, cudaStream_t s) {
    switch (group) {
        case 1: return launch_tc_t<1, T>(pp, mk, mv, grid, max_smem_optin, ov, s);
        case 2: return launch_tc_t<2, T>(pp, mk, mv, grid, max_smem_optin, ov, s);
        case 3: return launch_tc_t<3, T>(pp, mk, mv, grid, max_smem_optin, ov, s);
        case 4: return launch_tc_t<4, T>(pp, mk, mv, grid, max_smem_optin, ov, s);
        case 5: return launch_tc_t<5, T>(pp, mk, mv, grid, max_smem_optin, ov, s);
        case 6: return launch_tc_t<6, T>(pp, mk, mv, grid, max_smem_optin, ov, s);
        case 7: return launch_tc_t<7, T>(pp, mk, mv, grid, max_smem_optin, ov, s);
        case 8: return launch_tc_t<8, T>(pp, mk, mv, grid, max_smem_optin, ov, s);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace KRIYA_TC_NS
}  // namespace kriya

namespace ktc = kriya::KRIYA_TC_NS;


uint32_t KRIYA_TC_FN(kriya_decode_tc_ctas_per_sm)() { return uint32_t(ktc::kTcCtasPerSm); }
uint32_t KRIYA_TC_FN(kriya_decode_tc_pages_per_tile)() { return uint32_t(ktc::kTcPagesPerTile); }

bool KRIYA_TC_FN(kriya_decode_tc_supported)(uint32_t head_dim, uint32_t group, uint32_t block_size) {
    return head_dim == uint32_t(ktc::kTcD) && group >= 1 && group <= 8 && block_size == uint32_t(ktc::kTcPage);
}

cudaError_t KRIYA_TC_FN(kriya_launch_decode_tc)(const KriyaDecodeArgs& a, const KriyaTcSeg* segs, const uint32_t* cta_seg_ptr, uint32_t grid,
                                   const void* map_k, const void* map_v, uint32_t layer_row0, uint32_t dtype,
                                   int max_smem_optin, const KriyaFusedAppend& fused, uint32_t late_parts, uint32_t n_seg,
                                   const KriyaTcScratch& scratch, cudaStream_t s) {
    if (grid == 0) return cudaSuccess;
    const uint32_t group = a.num_q_heads / a.num_kv_heads;
    if (!KRIYA_TC_FN(kriya_decode_tc_supported)(ktc::kTcD, group, ktc::kTcPage) || !map_k || !map_v) return cudaErrorInvalidValue;
    ktc::TcParams pp;
    pp.a = a;
    pp.segs = segs;
    pp.cta_seg_ptr = cta_seg_ptr;
    pp.layer_row0 = layer_row0;
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
    return dtype == KRIYA_DTYPE_FP16 ? ktc::launch_tc_g<kriya::Fp16>(group, pp, mk, mv, grid, max_smem_optin, ov, s)
                                     : ktc::launch_tc_g<kriya::Bf16>(group, pp, mk, mv, grid, max_smem_optin, ov, s);
}
