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

}  // namespace kriya

cudaError_t kriya_launch_append(const KriyaAppendArgs& a, uint32_t dtype, cudaStream_t s) {
    const uint32_t jobs = a.num_tokens * (a.p.num_q_heads + a.p.num_kv_heads);
    if (jobs == 0) return cudaSuccess;
    const uint32_t grid = (jobs + kriya::kAppendWarps - 1) / kriya::kAppendWarps;
    if (dtype == KRIYA_DTYPE_FP16)
        kriya::append_kernel<kriya::Fp16><<<grid, kriya::kAppendWarps * 32, 0, s>>>(a);
    else
        kriya::append_kernel<kriya::Bf16><<<grid, kriya::kAppendWarps * 32, 0, s>>>(a);
    return cudaGetLastError();
}
