// Paged GQA decode attention over the BSR block table (the job of bsr_paged_gqa_decode_stage1 and
// bsr_paged_gqa_split_k_reduce, kernels/metal/paged_gqa_and_deltanet.metal:242-495,1474-1525).
//
// Shape of the kernel
//   - One CTA per work item = a contiguous range of KV pages of one plan row, ALL KV heads of the row.
//     A page of K for all heads is one contiguous page*Hkv*D*2-byte span of the pool, so the producer
//     warp moves each page with two bulk async copies (K, V) into a shared-memory ring; completion is
//     signalled on an mbarrier per stage, stages are handed back on a second mbarrier.  Page indices are
//     fetched 32 at a time ahead of the copies, so the indirect address is never on the critical path.
//   - Compute warps are arranged as rows x kv_heads.  Warp (row r, kv head h) consumes pages r, r+rows,
//     ... for head h and carries the G query heads of that KV head together, so every cached element is
//     read from HBM once and from shared memory once.  Within a warp, D/8 lanes share one token (16-byte
//     K/V loads) and 32/(D/8) tokens are processed per step.
//   - Scores are reduced across the D/8 lanes by recursive halving (G partial sums shrink to one per
//     lane), the online softmax runs once per page (one rescale per 16 tokens), probabilities go through
//     a per-warp shared-memory scratch to all lanes of the token, and the PV accumulation uses packed
//     f32x2 FMAs.  State (m, l, o) is fp32 in registers.
//   - The CTA merges its warps' states; a row split over several work items parks its (m, l, o) in
//     global scratch and the LAST item of the row to finish (atomic ticket, no waiting) merges them and
//     writes the output, so split-KV costs no second launch.
//
// HBM roofline: algorithmic bytes per launch = sum over rows of tokens * 2 * Hkv * D * 2 B (+ q, out,
// tables); the kernel is bound by HBM bandwidth as long as the fp32 pipes keep up
// (4 FMA per KV byte at G = 8).
#include <algorithm>

#include "kriya_device.cuh"

namespace kriya {

constexpr int kPage = 16;            // tokens per KV page the kernel is built for
constexpr int kMaxComputeWarps = 8;  // rows * kv_heads
constexpr int kDecodeThreadsMax = (kMaxComputeWarps + 1) * 32;
constexpr float kLog2e = 1.4426950408889634f;

constexpr int next_pow2(int x) { return x <= 1 ? 1 : 2 * next_pow2((x + 1) / 2); }

// Recursive-halving reduction of N per-lane values across a group of LANES lanes.  On return v[0] holds
// the group total of the value with index `owned` (returned), where `owned` depends on the lane.
template <int N, int LANES>
__device__ __forceinline__ int group_reduce(float (&v)[N], uint32_t lane) {
    int owned = 0;
    int n = N;
    int off = LANES / 2;
#pragma unroll
    for (; n > 1 && off >= 1; n >>= 1, off >>= 1) {
        const bool upper = (lane & off) != 0;
        const int h = n >> 1;
#pragma unroll
        for (int i = 0; i < N / 2; ++i) {
            if (i < h) {
                const float send = upper ? v[i] : v[i + h];
                const float keep = upper ? v[i + h] : v[i];
                v[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, off);
            }
        }
        if (upper) owned += h;
    }
#pragma unroll
    for (; off >= 1; off >>= 1) v[0] += __shfl_xor_sync(0xFFFFFFFFu, v[0], off);
    return owned;
}

struct DecodeLaunch {
    int rows;      // page rows computed concurrently
    int nstages;   // ring depth, multiple of rows
    uint32_t stage_bytes;
    uint32_t page_bytes;  // one page of K (or V) for all heads
};

// Eight consecutive values of a Q4KvGroup32 row (DType::Q4KvGroup32, crates/kriya-core/src/tensor.rs:50-51,77,91: per 32
// values 16 bytes of 4-bit codes + f16 scale + f16 min; value = fma(code, scale, min) as in the reference's
// dequantize_q4_group64_to_f32, crates/kriya-core/src/quantizer.rs:112-127).  `row` is the (token, head) row of D / 32
// blocks of 20 bytes, `dl` the index of the eight values inside the row.
__device__ __forceinline__ void q4kv_load8(const uint8_t* row, uint32_t dl, float2 (&out)[4]) {
    const uint8_t* blk = row + (dl >> 2) * 20u;
    const uint32_t codes = *reinterpret_cast<const uint32_t*>(blk + (dl & 3u) * 4u);
    const uint32_t hdr = *reinterpret_cast<const uint32_t*>(blk + 16u);
    const float scale = __half2float(__ushort_as_half(uint16_t(hdr & 0xFFFFu)));
    const float mn = __half2float(__ushort_as_half(uint16_t(hdr >> 16)));
#pragma unroll
    for (int j = 0; j < 4; ++j)
        out[j] = make_float2(__fmaf_rn(float((codes >> (8 * j)) & 15u), scale, mn), __fmaf_rn(float((codes >> (8 * j + 4)) & 15u), scale, mn));
}

template <int D, int G, typename T, bool Q4>
__global__ void __launch_bounds__(kDecodeThreadsMax, 1) decode_kernel(KriyaDecodeArgs a, DecodeLaunch L) {
    constexpr int LPT = D / 8;        // lanes per token
    constexpr int TPW = 32 / LPT;     // tokens per warp step
    constexpr int NSTEP = kPage / TPW;
    constexpr int GP = next_pow2(G);
    static_assert(GP <= LPT, "group size must not exceed lanes per token");

    extern __shared__ __align__(128) uint8_t smem[];
    const int HPC = int(a.num_kv_heads);
    const int R = L.rows;
    const int NWC = R * HPC;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;

    // shared memory carve-up: [ring | barriers | per-warp p/alpha scratch | ticket]
    uint8_t* ring = smem;
    const size_t ring_bytes = size_t(L.nstages) * L.stage_bytes;
    const size_t merge_bytes = size_t(NWC) * (TPW * G * D + GP + TPW * GP) * sizeof(float);
    const size_t area = ring_bytes > merge_bytes ? ring_bytes : merge_bytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + ((area + 15) & ~size_t(15)));
    uint64_t* empty_bar = full_bar + L.nstages;
    float* p_all = reinterpret_cast<float*>(empty_bar + L.nstages);
    uint32_t* ticket_s = reinterpret_cast<uint32_t*>(p_all + size_t(NWC) * (kPage * GP + GP));

    const KriyaDecodeWork w = a.work[blockIdx.x];
    const uint32_t req = w.req;
    const int32_t row0 = a.indptr[req];
    const uint32_t total_blocks = uint32_t(max(a.indptr[req + 1] - row0, 0));
    const uint32_t blk_end = min(w.blk_end, total_blocks);
    const int n = blk_end > w.blk_begin ? int(blk_end - w.blk_begin) : 0;

    if (tid == 0) {
        for (int s = 0; s < L.nstages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], uint32_t(HPC));
        }
        mbar_fence_init();
    }
    __syncthreads();

    const bool is_producer = int(warp) == NWC;
    const int r = int(warp) / HPC, hh = int(warp) % HPC;  // compute warps: row, kv head
    const uint32_t slot = lane / LPT, dl = lane % LPT;

    float2 o2[G][4];
    float m_run = -INFINITY, l_run = 0.0f;
    int my_g = 0;
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int j = 0; j < 4; ++j) o2[g][j] = make_float2(0.0f, 0.0f);

    if (is_producer) {
        // ---- producer warp: page indices 32 at a time, two bulk copies per page ----------------------
        const int32_t* idx = a.indices + row0 + int32_t(w.blk_begin);
        const uint8_t* pool_k = reinterpret_cast<const uint8_t*>(a.cache_k);
        const uint8_t* pool_v = reinterpret_cast<const uint8_t*>(a.cache_v);
        bool ok = true;
        for (int i0 = 0; i0 < n && ok; i0 += 32) {
            const int32_t mine = (i0 + int(lane) < n) ? idx[i0 + int(lane)] : 0;
            const int cnt = min(32, n - i0);
            for (int j = 0; j < cnt; ++j) {
                const int i = i0 + j;
                const int stage = i % L.nstages;
                const int use = i / L.nstages;
                if (use > 0 && !warp_wait(&empty_bar[stage], uint32_t(use - 1) & 1u)) {
                    ok = false;
                    break;
                }
                uint32_t blk = uint32_t(__shfl_sync(0xFFFFFFFFu, mine, j));
                if (blk >= a.num_blocks) {  // never dereference an index outside the pool
                    if (lane == 0) atomicMax(a.status, uint32_t(KRIYA_DEV_BAD_BLOCK_INDEX));
                    blk = 0;
                }
                if (lane == 0) {
                    uint8_t* dst = ring + size_t(stage) * L.stage_bytes;
                    mbar_arrive_expect_tx(&full_bar[stage], 2u * L.page_bytes);
                    bulk_g2s(dst, pool_k + size_t(blk) * L.page_bytes, L.page_bytes, &full_bar[stage]);
                    bulk_g2s(dst + L.page_bytes, pool_v + size_t(blk) * L.page_bytes, L.page_bytes, &full_bar[stage]);
                }
            }
        }
        if (!ok && lane == 0) atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
    } else {
        // ---- compute warps ---------------------------------------------------------------------------
        const bool softcap = a.logit_softcap > 0.0f;
        const float qscale = softcap ? a.sm_scale : a.sm_scale * kLog2e;
        float2 q2[G][4];
        {
            const uint16_t* qrow = reinterpret_cast<const uint16_t*>(a.q) + (size_t(req) * a.num_q_heads + hh * G) * D;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const uint4 raw = *reinterpret_cast<const uint4*>(qrow + g * D + dl * 8);
                const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = T::load2(wds[j]);
                    q2[g][j] = make_float2(f.x * qscale, f.y * qscale);
                }
            }
        }
        float* p_s = p_all + size_t(warp) * (kPage * GP + GP);
        float* alpha_s = p_s + kPage * GP;
        const int32_t last_len = max(a.last_len[req], 1);

        for (int i = r; i < n; i += R) {
            const int stage = i % L.nstages;
            const int use = i / L.nstages;
            if (!warp_wait(&full_bar[stage], uint32_t(use) & 1u)) {
                if (lane == 0) atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
                break;
            }
            const uint8_t* Ks = ring + size_t(stage) * L.stage_bytes;
            const uint8_t* Vs = Ks + L.page_bytes;
            const uint32_t valid = (w.blk_begin + uint32_t(i) + 1u == total_blocks) ? uint32_t(last_len) : uint32_t(kPage);
            // tokens of this page in front of the sliding window (only the window's first page has any)
            const uint32_t page_tok0 = (w.blk_begin + uint32_t(i)) * uint32_t(kPage);
            const uint32_t first = w.tok_first > page_tok0 ? min(w.tok_first - page_tok0, uint32_t(kPage)) : 0u;

            // phase A: scores of the page's tokens for the G query heads
            float s[NSTEP];
#pragma unroll
            for (int st = 0; st < NSTEP; ++st) {
                const uint32_t tok = uint32_t(st) * TPW + slot;
                float2 k0, k1, k2, k3;
                if (Q4) {
                    float2 kq[4];
                    q4kv_load8(Ks + (size_t(tok) * HPC + hh) * (D / 32) * 20, dl, kq);
                    k0 = kq[0]; k1 = kq[1]; k2 = kq[2]; k3 = kq[3];
                } else {
                    const uint4 raw = *reinterpret_cast<const uint4*>(Ks + ((size_t(tok) * HPC + hh) * D + dl * 8) * 2);
                    k0 = T::load2(raw.x); k1 = T::load2(raw.y); k2 = T::load2(raw.z); k3 = T::load2(raw.w);
                }
                float part[GP];
#pragma unroll
                for (int g = 0; g < GP; ++g) {
                    if (g < G) {
                        float2 acc = __fmul2_rn(q2[g][0], k0);
                        acc = __ffma2_rn(q2[g][1], k1, acc);
                        acc = __ffma2_rn(q2[g][2], k2, acc);
                        acc = __ffma2_rn(q2[g][3], k3, acc);
                        part[g] = acc.x + acc.y;
                    } else {
                        part[g] = 0.0f;
                    }
                }
                my_g = group_reduce<GP, LPT>(part, dl);
                float sc = part[0];
                if (softcap) sc = tanhf(fminf(fmaxf(sc / a.logit_softcap, -15.0f), 15.0f)) * a.logit_softcap * kLog2e;
                s[st] = (tok < valid && tok >= first) ? sc : -INFINITY;
            }
            // phase B: one online-softmax update per page
            float m_loc = s[0];
#pragma unroll
            for (int st = 1; st < NSTEP; ++st) m_loc = fmaxf(m_loc, s[st]);
#pragma unroll
            for (int off = LPT; off < 32; off <<= 1) m_loc = fmaxf(m_loc, __shfl_xor_sync(0xFFFFFFFFu, m_loc, off));
            const float m_new = fmaxf(m_run, m_loc);
            const float alpha = fast_exp2(m_run - m_new);
            float psum = 0.0f;
#pragma unroll
            for (int st = 0; st < NSTEP; ++st) {
                const float p = fast_exp2(s[st] - m_new);
                psum += p;
                p_s[(st * TPW + int(slot)) * GP + my_g] = p;
            }
            l_run = fmaf(l_run, alpha, psum);
            m_run = m_new;
            alpha_s[my_g] = alpha;
            __syncwarp();
            // phase C: rescale once, then accumulate P.V
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float al = alpha_s[g];
                const float2 al2 = make_float2(al, al);
#pragma unroll
                for (int j = 0; j < 4; ++j) o2[g][j] = __fmul2_rn(o2[g][j], al2);
            }
#pragma unroll
            for (int st = 0; st < NSTEP; ++st) {
                const uint32_t tok = uint32_t(st) * TPW + slot;
                float2 v0, v1, v2, v3;
                if (Q4) {
                    float2 vq[4];
                    q4kv_load8(Vs + (size_t(tok) * HPC + hh) * (D / 32) * 20, dl, vq);
                    v0 = vq[0]; v1 = vq[1]; v2 = vq[2]; v3 = vq[3];
                } else {
                    const uint4 raw = *reinterpret_cast<const uint4*>(Vs + ((size_t(tok) * HPC + hh) * D + dl * 8) * 2);
                    v0 = T::load2(raw.x); v1 = T::load2(raw.y); v2 = T::load2(raw.z); v3 = T::load2(raw.w);
                }
                if (tok >= valid || tok < first) {  // slots no token of the row's window occupies may hold anything
                    v0 = v1 = v2 = v3 = make_float2(0.0f, 0.0f);
                }
                const float* pg = p_s + (st * TPW + int(slot)) * GP;
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float p = pg[g];
                    const float2 pp = make_float2(p, p);
                    o2[g][0] = __ffma2_rn(pp, v0, o2[g][0]);
                    o2[g][1] = __ffma2_rn(pp, v1, o2[g][1]);
                    o2[g][2] = __ffma2_rn(pp, v2, o2[g][2]);
                    o2[g][3] = __ffma2_rn(pp, v3, o2[g][3]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);
        }
    }

    // ---- merge the warps of this CTA (ring memory is free once every warp is past its loop) -----------
    __syncthreads();
    float* o_m = reinterpret_cast<float*>(smem);                  // [NWC][TPW][G][D]
    float* m_m = o_m + size_t(NWC) * TPW * G * D;                 // [NWC][GP]
    float* l_m = m_m + size_t(NWC) * GP;                          // [NWC][TPW][GP]
    if (!is_producer) {
        float* dst = o_m + (size_t(warp) * TPW + slot) * G * D + dl * 8;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            *reinterpret_cast<float4*>(dst + g * D) = make_float4(o2[g][0].x, o2[g][0].y, o2[g][1].x, o2[g][1].y);
            *reinterpret_cast<float4*>(dst + g * D + 4) = make_float4(o2[g][2].x, o2[g][2].y, o2[g][3].x, o2[g][3].y);
        }
        // my_g is only meaningful after at least one page; recompute it so idle warps publish -inf too
        {
            int owned = 0, nn = GP, off = LPT / 2;
            for (; nn > 1 && off >= 1; nn >>= 1, off >>= 1)
                if (dl & off) owned += nn >> 1;
            my_g = owned;
        }
        m_m[warp * GP + my_g] = m_run;
        l_m[(warp * TPW + slot) * GP + my_g] = l_run;
    }
    __syncthreads();

    const int HQC = HPC * G;  // query heads handled by this CTA (all of them)
    const bool single = w.n_parts == 1u;
    const bool state_mode = a.state_o != nullptr;
    for (int e = int(tid); e < HQC * D; e += int(blockDim.x)) {
        const int hq = e / D, d = e % D;
        const int h = hq / G, g = hq % G;
        float M = -INFINITY;
        for (int rr = 0; rr < R; ++rr) M = fmaxf(M, m_m[(rr * HPC + h) * GP + g]);
        float Ls = 0.0f, Os = 0.0f;
        for (int rr = 0; rr < R; ++rr) {
            const int ww = rr * HPC + h;
            const float mw = m_m[ww * GP + g];
            if (mw == -INFINITY) continue;
            const float sc = exp2f(mw - M);
            for (int sl = 0; sl < TPW; ++sl) {
                Ls = fmaf(sc, l_m[(ww * TPW + sl) * GP + g], Ls);
                Os = fmaf(sc, o_m[((size_t(ww) * TPW + sl) * G + g) * D + d], Os);
            }
        }
        const size_t row = size_t(req) * a.num_q_heads + hq;
        if (single) {
            if (state_mode) {
                a.state_o[row * D + d] = Os;
                if (d == 0) {
                    a.state_m[row] = M / kLog2e;
                    a.state_l[row] = Ls;
                }
            } else {
                reinterpret_cast<uint16_t*>(a.out)[row * D + d] = T::store(Os / fmaxf(Ls, 1e-12f));
            }
        } else {
            const size_t prow = size_t(w.slot) * a.num_q_heads + hq;
            a.part_o[prow * D + d] = Os;
            if (d == 0) {
                a.part_ml[prow * 2 + 0] = M;
                a.part_ml[prow * 2 + 1] = Ls;
            }
        }
    }
    if (single) return;

    // ---- split row: the last work item to arrive merges all parts (ticket, no waiting) -----------------
    __threadfence();
    __syncthreads();
    if (tid == 0) *ticket_s = atomicAdd(&a.counters[req], 1u);
    __syncthreads();
    if (*ticket_s != w.n_parts - 1u) return;
    __threadfence();
    // Parts are merged eight at a time with all of a chunk's loads issued before any is used, so the merge costs
    // about one memory round trip per chunk rather than one per part.
    for (int e = int(tid); e < HQC * D; e += int(blockDim.x)) {
        const int hq = e / D, d = e % D;
        float M = -INFINITY, Ls = 0.0f, Os = 0.0f;
        for (uint32_t c0 = 0; c0 < w.n_parts; c0 += 8u) {
            const uint32_t cnt = min(8u, w.n_parts - c0);
            float mv[8], lv[8], ov[8];
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const bool on = uint32_t(s) < cnt;
                const size_t prow = size_t(w.first_slot + c0 + (on ? s : 0)) * a.num_q_heads + hq;
                mv[s] = on ? __ldcg(&a.part_ml[prow * 2]) : -INFINITY;
                lv[s] = on ? __ldcg(&a.part_ml[prow * 2 + 1]) : 0.0f;
                ov[s] = on ? __ldcg(&a.part_o[prow * D + d]) : 0.0f;
            }
            float mc = M;
#pragma unroll
            for (int s = 0; s < 8; ++s) mc = fmaxf(mc, mv[s]);
            if (mc == -INFINITY) continue;
            const float keep = (M == -INFINITY) ? 0.0f : exp2f(M - mc);
            Ls *= keep;
            Os *= keep;
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const float wgt = (mv[s] == -INFINITY) ? 0.0f : exp2f(mv[s] - mc);
                Ls = fmaf(wgt, lv[s], Ls);
                Os = fmaf(wgt, ov[s], Os);
            }
            M = mc;
        }
        const size_t row = size_t(req) * a.num_q_heads + hq;
        if (state_mode) {
            a.state_o[row * D + d] = Os;
            if (d == 0) {
                a.state_m[row] = M / kLog2e;
                a.state_l[row] = Ls;
            }
        } else {
            reinterpret_cast<uint16_t*>(a.out)[row * D + d] = T::store(Os / fmaxf(Ls, 1e-12f));
        }
    }
    if (tid == 0) a.counters[req] = 0u;  // ready for the next launch on this stream
}

// Merge of partial states gathered from several ranks: [parts][rows] (m natural-log units, l) and
// [parts][rows][D] (o)  ->  normalised 16-bit [rows][D].
// `stride_ml` / `stride_o` are the distances, in floats, between consecutive parts of m, l and of o.
template <typename T>
__global__ void merge_states_kernel(const float* __restrict__ m, const float* __restrict__ l,
                                    const float* __restrict__ o, uint32_t parts, uint32_t rows, uint32_t D,
                                    size_t stride_ml, size_t stride_o, uint16_t* __restrict__ out) {
    const uint32_t row = blockIdx.x;
    if (row >= rows) return;
    float M = -INFINITY;
    for (uint32_t s = 0; s < parts; ++s) M = fmaxf(M, m[s * stride_ml + row]);
    float den = 0.0f;
    for (uint32_t s = 0; s < parts; ++s) {
        const float ms = m[s * stride_ml + row];
        if (ms > -INFINITY) den = fmaf(expf(ms - M), l[s * stride_ml + row], den);
    }
    const float inv = 1.0f / fmaxf(den, 1e-12f);
    for (uint32_t d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f;
        for (uint32_t s = 0; s < parts; ++s) {
            const float ms = m[s * stride_ml + row];
            if (ms > -INFINITY) acc = fmaf(expf(ms - M), o[s * stride_o + size_t(row) * D + d], acc);
        }
        out[size_t(row) * D + d] = T::store(acc * inv);
    }
}

template <int D, int G, typename T, bool Q4>
cudaError_t launch_decode_t(const KriyaDecodeArgs& a, int max_smem_optin, cudaStream_t s) {
    constexpr int LPT = D / 8, TPW = 32 / LPT, GP = next_pow2(G);
    const int HPC = int(a.num_kv_heads);
    if (HPC < 1 || HPC > kMaxComputeWarps) return cudaErrorInvalidValue;
    DecodeLaunch L;
    L.rows = kMaxComputeWarps / HPC;
    L.page_bytes = Q4 ? uint32_t(kPage) * HPC * (D / 32) * 20u : uint32_t(kPage) * HPC * D * 2u;
    L.stage_bytes = 2u * L.page_bytes;
    const int NWC = L.rows * HPC;
    const size_t extra = 2 * 64 * sizeof(uint64_t) + size_t(NWC) * (kPage * GP + GP) * sizeof(float) + 64;
    const size_t budget = size_t(max_smem_optin) - extra - 1024;
    int nst = int(std::min<size_t>(budget / L.stage_bytes, 16));
    nst = (nst / L.rows) * L.rows;
    // two stages per row are enough to keep copies ahead of compute; more only deepens the prefetch
    nst = std::min(nst, std::max(2 * L.rows, int((128u * 1024u) / L.stage_bytes) / L.rows * L.rows));
    if (nst < L.rows || nst > 64) return cudaErrorInvalidValue;
    L.nstages = nst;
    const size_t ring_bytes = size_t(nst) * L.stage_bytes;
    const size_t merge_bytes = size_t(NWC) * (TPW * G * D + GP + TPW * GP) * sizeof(float);
    const size_t area = (std::max(ring_bytes, merge_bytes) + 15) & ~size_t(15);
    const size_t smem = area + 2 * size_t(nst) * sizeof(uint64_t) + size_t(NWC) * (kPage * GP + GP) * sizeof(float) + 16;
    if (smem > size_t(max_smem_optin)) return cudaErrorInvalidValue;
    auto kern = decode_kernel<D, G, T, Q4>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return e;
    kern<<<a.n_work, (NWC + 1) * 32, smem, s>>>(a, L);
    return cudaGetLastError();
}

template <int D, typename T, bool Q4>
cudaError_t launch_decode_g(const KriyaDecodeArgs& a, uint32_t group, int max_smem_optin, cudaStream_t s) {
    switch (group) {
        case 1: return launch_decode_t<D, 1, T, Q4>(a, max_smem_optin, s);
        case 2: return launch_decode_t<D, 2, T, Q4>(a, max_smem_optin, s);
        case 3: return launch_decode_t<D, 3, T, Q4>(a, max_smem_optin, s);
        case 4: return launch_decode_t<D, 4, T, Q4>(a, max_smem_optin, s);
        case 5: return launch_decode_t<D, 5, T, Q4>(a, max_smem_optin, s);
        case 6: return launch_decode_t<D, 6, T, Q4>(a, max_smem_optin, s);
        case 7: return launch_decode_t<D, 7, T, Q4>(a, max_smem_optin, s);
        case 8: return launch_decode_t<D, 8, T, Q4>(a, max_smem_optin, s);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace kriya

bool kriya_decode_supported(uint32_t head_dim, uint32_t group, uint32_t num_kv_heads, uint32_t block_size) {
    return (head_dim == 64 || head_dim == 128) && group >= 1 && group <= 8 && num_kv_heads >= 1 &&
           num_kv_heads <= uint32_t(kriya::kMaxComputeWarps) && block_size == uint32_t(kriya::kPage);
}

cudaError_t kriya_launch_decode(const KriyaDecodeArgs& a, uint32_t head_dim, uint32_t block_size, uint32_t dtype,
                                int max_smem_optin, cudaStream_t s, uint32_t kv_q4) {
    if (a.n_work == 0) return cudaSuccess;
    const uint32_t group = a.num_kv_heads ? a.num_q_heads / a.num_kv_heads : 0;
    if (!kriya_decode_supported(head_dim, group, a.num_kv_heads, block_size)) return cudaErrorInvalidValue;
    using namespace kriya;
    if (kv_q4) {  // the query / output type still follows `dtype`
        if (head_dim == 128)
            return dtype == KRIYA_DTYPE_FP16 ? launch_decode_g<128, Fp16, true>(a, group, max_smem_optin, s)
                                             : launch_decode_g<128, Bf16, true>(a, group, max_smem_optin, s);
        return dtype == KRIYA_DTYPE_FP16 ? launch_decode_g<64, Fp16, true>(a, group, max_smem_optin, s)
                                         : launch_decode_g<64, Bf16, true>(a, group, max_smem_optin, s);
    }
    if (head_dim == 128)
        return dtype == KRIYA_DTYPE_FP16 ? launch_decode_g<128, Fp16, false>(a, group, max_smem_optin, s)
                                         : launch_decode_g<128, Bf16, false>(a, group, max_smem_optin, s);
    return dtype == KRIYA_DTYPE_FP16 ? launch_decode_g<64, Fp16, false>(a, group, max_smem_optin, s)
                                     : launch_decode_g<64, Bf16, false>(a, group, max_smem_optin, s);
}

cudaError_t kriya_launch_merge_states(const float* m, const float* l, const float* o, uint32_t parts, uint32_t rows,
                                      uint32_t D, size_t stride_ml, size_t stride_o, void* out, uint32_t dtype,
                                      cudaStream_t s) {
    if (rows == 0) return cudaSuccess;
    if (dtype == KRIYA_DTYPE_FP16)
        kriya::merge_states_kernel<kriya::Fp16><<<rows, 128, 0, s>>>(m, l, o, parts, rows, D, stride_ml, stride_o,
                                                                     static_cast<uint16_t*>(out));
    else
        kriya::merge_states_kernel<kriya::Bf16><<<rows, 128, 0, s>>>(m, l, o, parts, rows, D, stride_ml, stride_o,
                                                                     static_cast<uint16_t*>(out));
    return cudaGetLastError();
}
