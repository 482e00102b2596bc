// Fused QK-RMSNorm + RoPE + paged KV append (the job of fused_qknorm_rope_and_kv_append,
// kernels/metal/paged_gqa_and_deltanet.metal:115-226).
//
// One warp per (token, head): query heads are rotated in place, key heads are rotated into their
// cache slot, value heads are copied bit for bit.  The in-place mode is apply_rope_inplace
// (paged_gqa_and_deltanet.metal:1738-1829): keys are rotated where they are and nothing touches the cache.  The arithmetic keeps the reference's operation
// order (fma(x0, c, -x1*s), fma(x0, s, x1*c), round-to-nearest-even on store) so that with the
// precomputed cos/sin table the cache contents are bit-identical to a host evaluation.
//
// HBM traffic per token: read (Hq + 2 Hkv) * D * 2 B, write the same; at decode batch sizes this is
// a few hundred KB per launch, so the kernel is launch-latency bound and is laid out for
// coalescing only (each warp reads and writes whole 128-256 B head rows).
#include "kriya_device.cuh"

#include <algorithm>

namespace kriya {

constexpr int kAppendWarps = 8;

// DType::Q4KvGroup32 (crates/kriya-core/src/tensor.rs:50-51,77,91): 32 values -> 16 bytes of 4-bit codes + f16 scale +
// f16 min.  One warp quantises one group, lane i holding value i: the arithmetic of the reference's own 4-bit affine
// group quantiser (crates/kriya-core/src/quantizer.rs:61-109) with this format's group size and f16 header - range =
// max(max - min, 1e-8), scale = range / 15, codes taken with the ROUNDED scale (floored at 1e-8) and min,
// q = clamp(round((v - min) / scale), 0, 15) rounding halves away from zero, value 2i in the low nibble of byte i.
__device__ __forceinline__ void q4kv_store_group(uint8_t* block, float v, uint32_t lane) {
    float mn = v, mx = v;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xFFFFFFFFu, mn, off));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
    }
    const float range = fmaxf(__fsub_rn(mx, mn), 1e-8f);
    const __half scale_h = __float2half_rn(__fdiv_rn(range, 15.0f)), min_h = __float2half_rn(mn);
    const float eff_scale = fmaxf(__half2float(scale_h), 1e-8f), eff_min = __half2float(min_h);
    const float qf = fminf(fmaxf(roundf(__fdiv_rn(__fsub_rn(v, eff_min), eff_scale)), 0.0f), 15.0f);
    uint32_t q = uint32_t(qf) & 0xFu;
    // nibble i of the group's 128 code bits belongs to lane i: gather eight lanes' codes into one 32-bit word
    uint32_t w = q << (4u * (lane & 7u));
    w |= __shfl_xor_sync(0xFFFFFFFFu, w, 1);
    w |= __shfl_xor_sync(0xFFFFFFFFu, w, 2);
    w |= __shfl_xor_sync(0xFFFFFFFFu, w, 4);
    if ((lane & 7u) == 0u) reinterpret_cast<uint32_t*>(block)[lane >> 3] = w;
    if (lane == 0u)
        reinterpret_cast<uint32_t*>(block)[4] = uint32_t(__half_as_ushort(scale_h)) | (uint32_t(__half_as_ushort(min_h)) << 16);
}

template <typename T>
__global__ void __launch_bounds__(kAppendWarps * 32) append_kernel(KriyaAppendArgs a) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t Hq = a.p.num_q_heads, Hkv = a.p.num_kv_heads, D = a.p.head_dim;
    const uint32_t heads = Hq + Hkv;
    const uint32_t job = blockIdx.x * kAppendWarps + (threadIdx.x >> 5);
    if (job >= a.num_tokens * heads) return;
    const uint32_t r = job / heads, head = job % heads;
    const bool is_q = head < Hq;
    const uint32_t lh = is_q ? head : head - Hq;

    uint16_t* q_row = reinterpret_cast<uint16_t*>(a.q_inout) + (size_t(r) * Hq + lh) * D;
    const uint16_t* k_row = reinterpret_cast<const uint16_t*>(a.k_in) + (size_t(r) * Hkv + lh) * D;
    const uint16_t* src = is_q ? q_row : k_row;

    uint32_t position, blk = 0, slot = 0;
    if (a.inplace) {
        position = a.positions[r];  // apply_rope_inplace: no cache slot, keys are rotated where they are
    } else if (a.chunk_mode == 2u) {
        // which sequence owns row r: the lanes look through the (few) sequences together
        uint32_t found = UINT32_MAX;
        for (uint32_t s0 = 0; s0 < a.n_seqs && found == UINT32_MAX; s0 += 32u) {
            const uint32_t sq = s0 + lane;
            const bool hit = sq < a.n_seqs && r >= a.seq_q_start[sq] && r - a.seq_q_start[sq] < a.seq_count[sq];
            const uint32_t m = __ballot_sync(0xFFFFFFFFu, hit);
            if (m) found = s0 + uint32_t(__ffs(int(m)) - 1);
        }
        if (found == UINT32_MAX) return;  // a row between two chunks: not part of this call
        position = a.seq_prefix[found] + (r - a.seq_q_start[found]);
        if (!is_q) {
            blk = uint32_t(a.indices[a.indptr[found] + int32_t(position / a.p.block_size_tokens)]);
            slot = position % a.p.block_size_tokens;
        }
    } else if (a.chunk_mode) {
        position = a.prefix_tokens + r;
        if (!is_q) {
            blk = uint32_t(a.indices[a.indptr[0] + int32_t(position / a.p.block_size_tokens)]);
            slot = position % a.p.block_size_tokens;
        }
    } else {
        position = a.positions[r];
        if (!is_q) {
            blk = uint32_t(a.indices[a.indptr[r + 1] - 1]);
            slot = uint32_t(a.last_len[r] - 1);
        }
    }
    if (!is_q && !a.inplace && (blk >= a.num_blocks || slot >= a.p.block_size_tokens)) {
        if (lane == 0) atomicMax(a.status, blk >= a.num_blocks ? KRIYA_DEV_BAD_BLOCK_INDEX : KRIYA_DEV_BAD_SLOT);
        return;
    }

    const bool do_norm = a.p.apply_qk_norm != 0u;
    float rms_scale = 1.0f;
    if (do_norm) {
        float s = 0.0f;
        for (uint32_t d = lane; d < D; d += 32u) {
            const float v = T::load(src[d]);
            s = __fmaf_rn(v, v, s);
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, off);
        rms_scale = rsqrtf(s / float(D) + a.p.rms_eps);
    }

    const uint32_t half_d = D / 2u, half_rot = a.p.rotary_dim / 2u;
    const float pos_f = float(position);
    const bool use_table = a.p.has_table != 0u && position < a.p.max_seq_len && a.table != nullptr;
    const uint16_t* norm_w = reinterpret_cast<const uint16_t*>(is_q ? a.q_norm_w : a.k_norm_w);
    uint16_t* dst_k = nullptr;
    uint16_t* dst_v = nullptr;
    const uint16_t* v_row = nullptr;
    if (!is_q && a.inplace) {
        dst_k = const_cast<uint16_t*>(k_row);
    } else if (!is_q) {
        const size_t off = ((size_t(blk) * a.p.block_size_tokens + slot) * Hkv + lh) * D;
        dst_k = reinterpret_cast<uint16_t*>(a.cache_k) + off;
        dst_v = reinterpret_cast<uint16_t*>(a.cache_v) + off;
        v_row = reinterpret_cast<const uint16_t*>(a.v_in) + (size_t(r) * Hkv + lh) * D;
    }
    // Q4KvGroup32 cache: the row's D / 32 groups of 20 bytes; lane i holds value i of the two groups each pass touches
    const bool q4 = a.kv_q4 != 0u && !is_q && !a.inplace;
    uint8_t* q4_k = nullptr;
    uint8_t* q4_v = nullptr;
    if (q4) {
        const size_t row = ((size_t(blk) * a.p.block_size_tokens + slot) * Hkv + lh) * (D / 32u) * 20u;
        q4_k = reinterpret_cast<uint8_t*>(a.cache_k) + row;
        q4_v = reinterpret_cast<uint8_t*>(a.cache_v) + row;
    }

    for (uint32_t i = lane; i < half_d; i += 32u) {
        const uint32_t d0 = i, d1 = i + half_d;
        float x0 = __fmul_rn(T::load(src[d0]), rms_scale);
        float x1 = __fmul_rn(T::load(src[d1]), rms_scale);
        if (do_norm && norm_w != nullptr) {
            x0 = __fmul_rn(x0, T::load(norm_w[d0]));
            x1 = __fmul_rn(x1, T::load(norm_w[d1]));
        }
        if (i < half_rot) {
            float c, s;
            if (use_table) {
                const float2 cs = reinterpret_cast<const float2*>(a.table)[size_t(position) * half_rot + i];
                c = cs.x;
                s = cs.y;
            } else {
                const float freq_exp = float(2u * i) / float(a.p.rotary_dim);
                const float inv_freq = powf(a.p.rope_theta, -freq_exp);
                const float angle = __fmul_rn(pos_f, inv_freq);
                c = cosf(angle);
                s = sinf(angle);
            }
            const float rot0 = __fmaf_rn(x0, c, -__fmul_rn(x1, s));
            const float rot1 = __fmaf_rn(x0, s, __fmul_rn(x1, c));
            x0 = rot0;
            x1 = rot1;
        }
        if (is_q) {
            q_row[d0] = T::store(x0);
            q_row[d1] = T::store(x1);
        } else if (q4) {
            // half_d is a multiple of 32 here, so this pass's 32 values d0 are one group and its 32 values d1 another;
            // keys are quantised from the un-rounded rotated values, values from the 16-bit values as given
            q4kv_store_group(q4_k + (d0 / 32u) * 20u, x0, lane);
            q4kv_store_group(q4_k + (d1 / 32u) * 20u, x1, lane);
            q4kv_store_group(q4_v + (d0 / 32u) * 20u, T::load(v_row[d0]), lane);
            q4kv_store_group(q4_v + (d1 / 32u) * 20u, T::load(v_row[d1]), lane);
        } else {
            dst_k[d0] = T::store(x0);
            dst_k[d1] = T::store(x1);
            if (dst_v != nullptr) {
                dst_v[d0] = v_row[d0];
                dst_v[d1] = v_row[d1];
            }
        }
    }
}


// The same job for 16-bit caches without QK-norm, laid out for bandwidth.  A thread has the eight values at
// [8 sub, 8 sub + 8) of the lower half of a row and their rotation partners in the upper half (two 16-byte loads, two
// 16-byte stores) for kAppendRows (= 2) consecutive rows of one token, the token's rows being its query heads, its key heads
// and its value heads (copied): the 64 bytes a thread asks for are in flight together and are asked for before anything
// else, the look-ups of where the token goes (sequence, position, block) and its eight cos / sin pairs are fetched once
// per thread under them.  A chunk of thousands of tokens moves (Hq + 2 Hkv) * D * 2 B per token in and out; with
// 2-byte accesses per lane the kernel above reaches a sixth of the HBM rate on it.  Arithmetic per element is the
// kernel above's, so the cache contents are the same bits.
constexpr int kAppendVecThreads = 128;  // about: a block is (row groups of a token * D / 16) threads wide and a few tokens deep

template <typename T, int kAppendRows>
__global__ void __launch_bounds__(512) append_vec_kernel(KriyaAppendArgs a, uint32_t tpr_log2, uint32_t bs_log2) {
    // threadIdx.x = (group of rows of the token, 16-byte piece of a row), threadIdx.y = token of the block
    const uint32_t lane = (threadIdx.y * blockDim.x + threadIdx.x) & 31u;
    const uint32_t Hq = a.p.num_q_heads, Hkv = a.p.num_kv_heads, D = a.p.head_dim;
    const uint32_t rows = Hq + 2u * Hkv;
    const uint32_t row0 = (threadIdx.x >> tpr_log2) * uint32_t(kAppendRows), sub = threadIdx.x & ((1u << tpr_log2) - 1u);
    const uint32_t token = blockIdx.x * blockDim.y + threadIdx.y;
    bool live = token < a.num_tokens;
    const uint32_t r = live ? token : a.num_tokens - 1u;
    const uint32_t bs = a.p.block_size_tokens;
    const uint32_t half_d = D / 2u, half_rot = a.p.rotary_dim / 2u;
    const uint32_t e0 = sub * 8u;
    uint16_t* q_tok = reinterpret_cast<uint16_t*>(a.q_inout) + size_t(r) * Hq * D;
    const uint16_t* k_tok = reinterpret_cast<const uint16_t*>(a.k_in) + size_t(r) * Hkv * D;
    const uint16_t* v_tok = reinterpret_cast<const uint16_t*>(a.v_in) + size_t(r) * Hkv * D;

    uint4 lo[kAppendRows], hi[kAppendRows];
#pragma unroll
    for (int j = 0; j < kAppendRows; ++j) {
        const uint32_t head = row0 + uint32_t(j);
        lo[j] = make_uint4(0u, 0u, 0u, 0u);
        hi[j] = lo[j];
        if (head < rows && !(a.inplace && head >= Hq + Hkv)) {
            const uint16_t* src = head < Hq ? q_tok + size_t(head) * D
                                  : head < Hq + Hkv ? k_tok + size_t(head - Hq) * D : v_tok + size_t(head - Hq - Hkv) * D;
            lo[j] = *reinterpret_cast<const uint4*>(src + e0);
            hi[j] = *reinterpret_cast<const uint4*>(src + half_d + e0);
        }
    }

    const bool has_kv = row0 + uint32_t(kAppendRows) > Hq;  // this thread has key or value rows: it needs the token's slot
    uint32_t position = 0, blk = 0, slot = 0, seq_row = 0;
    if (a.inplace) {
        position = a.positions[r];
    } else if (a.chunk_mode == 2u) {
        // a warp's tokens are few and consecutive; the lanes look each one's sequence up together
        const uint32_t r_lo = __shfl_sync(0xFFFFFFFFu, r, 0), r_hi = __shfl_sync(0xFFFFFFFFu, r, 31);
        uint32_t found = UINT32_MAX;
        for (uint32_t rr = r_lo; rr <= r_hi; ++rr) {
            uint32_t f = UINT32_MAX;
            for (uint32_t s0 = 0; s0 < a.n_seqs && f == UINT32_MAX; s0 += 32u) {
                const uint32_t sq = s0 + lane;
                const bool hit = sq < a.n_seqs && rr >= a.seq_q_start[sq] && rr - a.seq_q_start[sq] < a.seq_count[sq];
                const uint32_t m = __ballot_sync(0xFFFFFFFFu, hit);
                if (m) f = s0 + uint32_t(__ffs(int(m)) - 1);
            }
            if (r == rr) found = f;
        }
        if (found == UINT32_MAX) {
            live = false;  // a row between two chunks: not part of this call
        } else {
            position = a.seq_prefix[found] + (r - a.seq_q_start[found]);
            seq_row = found;
        }
    } else if (a.chunk_mode) {
        position = a.prefix_tokens + r;
    } else {
        position = a.positions[r];
    }
    if (!live) return;

    // the token's cos / sin pairs go out before the block look-up: they only need the position
    const bool rotated = e0 < half_rot;  // half_rot is a multiple of 8 here: the eight pairs are all rotated or none is
    float c[8], sn[8];
    if (rotated) {
        const bool use_table = a.p.has_table != 0u && position < a.p.max_seq_len && a.table != nullptr;
        if (use_table) {
            const float4* t4 = reinterpret_cast<const float4*>(reinterpret_cast<const float2*>(a.table) + size_t(position) * half_rot + e0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float4 t = t4[j];
                c[2 * j] = t.x;
                sn[2 * j] = t.y;
                c[2 * j + 1] = t.z;
                sn[2 * j + 1] = t.w;
            }
        } else {
            const float pos_f = float(position);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float freq_exp = float(2u * (e0 + uint32_t(j))) / float(a.p.rotary_dim);
                const float inv_freq = powf(a.p.rope_theta, -freq_exp);
                const float angle = __fmul_rn(pos_f, inv_freq);
                c[j] = cosf(angle);
                sn[j] = sinf(angle);
            }
        }
    }
    bool slot_ok = true;
    if (has_kv && !a.inplace) {
        if (a.chunk_mode) {
            blk = uint32_t(a.indices[a.indptr[seq_row] + int32_t(position >> bs_log2)]);
            slot = position & (bs - 1u);
        } else {
            blk = uint32_t(a.indices[a.indptr[r + 1] - 1]);
            slot = uint32_t(a.last_len[r] - 1);
        }
        if (blk >= a.num_blocks || slot >= bs) {
            if (sub == 0u) atomicMax(a.status, blk >= a.num_blocks ? KRIYA_DEV_BAD_BLOCK_INDEX : KRIYA_DEV_BAD_SLOT);
            slot_ok = false;  // the token's key and value rows are left out, its query rows are still rotated
        }
    }
    const size_t cache_tok = (size_t(blk) * bs + slot) * Hkv * D;

#pragma unroll
    for (int j = 0; j < kAppendRows; ++j) {
        const uint32_t head = row0 + uint32_t(j);
        if (head >= rows) break;
        if (head >= Hq + Hkv) {  // a value row: the bits as they came
            if (a.inplace || !slot_ok) continue;
            uint16_t* dst_v = reinterpret_cast<uint16_t*>(a.cache_v) + cache_tok + size_t(head - Hq - Hkv) * D;
            *reinterpret_cast<uint4*>(dst_v + e0) = lo[j];
            *reinterpret_cast<uint4*>(dst_v + half_d + e0) = hi[j];
            continue;
        }
        uint16_t* dst;
        if (head < Hq) {
            dst = q_tok + size_t(head) * D;
        } else if (a.inplace) {
            dst = const_cast<uint16_t*>(k_tok) + size_t(head - Hq) * D;
        } else {
            if (!slot_ok) continue;
            dst = reinterpret_cast<uint16_t*>(a.cache_k) + cache_tok + size_t(head - Hq) * D;
        }
        if (rotated) {
            uint32_t lw[4] = {lo[j].x, lo[j].y, lo[j].z, lo[j].w};
            uint32_t hw[4] = {hi[j].x, hi[j].y, hi[j].z, hi[j].w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float2 x0 = T::load2(lw[w]), x1 = T::load2(hw[w]);
                const float r0a = __fmaf_rn(x0.x, c[2 * w], -__fmul_rn(x1.x, sn[2 * w]));
                const float r1a = __fmaf_rn(x0.x, sn[2 * w], __fmul_rn(x1.x, c[2 * w]));
                const float r0b = __fmaf_rn(x0.y, c[2 * w + 1], -__fmul_rn(x1.y, sn[2 * w + 1]));
                const float r1b = __fmaf_rn(x0.y, sn[2 * w + 1], __fmul_rn(x1.y, c[2 * w + 1]));
                // the paired conversion leaves the bits of T::store on every value that is not a NaN
                if (r0a == r0a && r0b == r0b && r1a == r1a && r1b == r1b) {
                    lw[w] = T::pack2(r0a, r0b);
                    hw[w] = T::pack2(r1a, r1b);
                } else {
                    lw[w] = uint32_t(T::store(r0a)) | (uint32_t(T::store(r0b)) << 16);
                    hw[w] = uint32_t(T::store(r1a)) | (uint32_t(T::store(r1b)) << 16);
                }
            }
            lo[j] = make_uint4(lw[0], lw[1], lw[2], lw[3]);
            hi[j] = make_uint4(hw[0], hw[1], hw[2], hw[3]);
        }
        *reinterpret_cast<uint4*>(dst + e0) = lo[j];
        *reinterpret_cast<uint4*>(dst + half_d + e0) = hi[j];
    }
}

}  // namespace kriya

cudaError_t kriya_launch_append(const KriyaAppendArgs& a, uint32_t dtype, cudaStream_t s) {
    const uint32_t jobs = a.num_tokens * (a.p.num_q_heads + a.p.num_kv_heads);
    if (jobs == 0) return cudaSuccess;
    // the 16-byte form: rows of 64 / 128 / 256 values, whole chunks of eight inside or outside the rotated part, every
    // base on a 16-byte boundary, a 16-bit cache and no QK-norm (its row sum keeps the one-warp-per-row order)
    const uint32_t D = a.p.head_dim;
    const uint32_t tpr_log2 = D == 64u ? 2u : D == 128u ? 3u : D == 256u ? 4u : 0u;
    auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0u; };
    const uint32_t bs = a.p.block_size_tokens;
    uint32_t bs_log2 = 0;
    while ((1u << bs_log2) < bs) ++bs_log2;
    const uint32_t R = 2u;  // rows of a token per thread (four measured slower: 87 registers, 20 resident warps)
    const uint32_t bdx = ((a.p.num_q_heads + 2u * a.p.num_kv_heads + R - 1u) / R) << tpr_log2;  // threads of one token
    // whole warps only (the lanes of a warp look the sequence up together): the block's depth is a multiple of 32 / gcd(width, 32)
    uint32_t gcd32 = 32u;
    while (bdx % gcd32 != 0u) gcd32 >>= 1;
    const uint32_t ystep = 32u / gcd32;
    const uint32_t bdy = bdx == 0u ? 0u : ystep * std::max(1u, (uint32_t(kriya::kAppendVecThreads) + bdx * ystep - 1u) / (bdx * ystep));
    const bool vec = tpr_log2 != 0u && (1u << bs_log2) == bs && bdx * bdy <= 512u && a.kv_q4 == 0u && a.p.apply_qk_norm == 0u && (a.p.rotary_dim % 16u) == 0u &&
                     a.p.rotary_dim <= D && aligned16(a.q_inout) && aligned16(a.k_in) &&
                     (a.inplace || (aligned16(a.v_in) && aligned16(a.cache_k) && aligned16(a.cache_v))) &&
                     (a.table == nullptr || aligned16(a.table));
    if (vec) {
        const dim3 block(bdx, bdy);
        const uint32_t grid = (a.num_tokens + block.y - 1u) / block.y;
        if (dtype == KRIYA_DTYPE_FP16)
            kriya::append_vec_kernel<kriya::Fp16, 2><<<grid, block, 0, s>>>(a, tpr_log2, bs_log2);
        else
            kriya::append_vec_kernel<kriya::Bf16, 2><<<grid, block, 0, s>>>(a, tpr_log2, bs_log2);
        return cudaGetLastError();
    }
    const uint32_t grid = (jobs + kriya::kAppendWarps - 1) / kriya::kAppendWarps;
    if (dtype == KRIYA_DTYPE_FP16)
        kriya::append_kernel<kriya::Fp16><<<grid, kriya::kAppendWarps * 32, 0, s>>>(a);
    else
        kriya::append_kernel<kriya::Bf16><<<grid, kriya::kAppendWarps * 32, 0, s>>>(a);
    return cudaGetLastError();
}
