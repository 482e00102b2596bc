// Q4KvGroup32 cache -> 16-bit staging blocks, for the kernels that read K/V through tensor maps (the chunked prefill).
// The format (crates/kriya-core/src/tensor.rs:50-91): 32 values -> 16 bytes of 4-bit codes + f16 scale + f16 min, value =
// fma(code, scale, min) (the reference's dequantize_q4_group64_to_f32, crates/kriya-core/src/quantizer.rs:112-127, with
// this format's group size and header type).  The blocks a plan names are expanded in plan order: staging block i holds
// the values of pool block page_indices[i], so the attention kernel reads the staging pool with the identity block table.
#include "kriya_device.cuh"
#include "kriya_internal.h"

namespace kriya {

// One warp per (plan index, token, KV head) row of D values; a lane per group's four bytes (eight values).
template <typename T>
__global__ void __launch_bounds__(256) q4_expand_blocks_kernel(const uint8_t* __restrict__ pool_k, const uint8_t* __restrict__ pool_v,
                                                               uint16_t* __restrict__ dst_k, uint16_t* __restrict__ dst_v,
                                                               const int32_t* __restrict__ indices, uint32_t n_indices, uint32_t block_tokens,
                                                               uint32_t hkv, uint32_t D, uint32_t num_blocks, uint32_t* status) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint64_t row = uint64_t(blockIdx.x) * 8u + (threadIdx.x >> 5);
    const uint64_t rows_per_block = uint64_t(block_tokens) * hkv;
    if (row >= uint64_t(n_indices) * rows_per_block) return;
    const uint32_t i = uint32_t(row / rows_per_block);
    const uint32_t in_block = uint32_t(row % rows_per_block);
    uint32_t blk = uint32_t(indices[i]);
    if (blk >= num_blocks) {
        if (lane == 0) atomicMax(status, uint32_t(KRIYA_DEV_BAD_BLOCK_INDEX));
        blk = 0;
    }
    const uint32_t groups = D / 32u;
    const size_t src_row = (size_t(blk) * rows_per_block + in_block) * groups * 20u;
    const size_t dst_row = (size_t(i) * rows_per_block + in_block) * D;
    for (uint32_t c = lane; c < groups * 4u; c += 32u) {  // chunk c: eight values of group c / 4
        const uint32_t g = c >> 2, part = c & 3u;
#pragma unroll
        for (int kv = 0; kv < 2; ++kv) {
            const uint8_t* grp = (kv ? pool_v : pool_k) + src_row + g * 20u;
            const uint32_t codes = *reinterpret_cast<const uint32_t*>(grp + part * 4u);
            const uint32_t hdr = *reinterpret_cast<const uint32_t*>(grp + 16u);
            const float scale = __half2float(__ushort_as_half(uint16_t(hdr & 0xFFFFu)));
            const float mn = __half2float(__ushort_as_half(uint16_t(hdr >> 16)));
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                w[j] = T::pack2(__fmaf_rn(float((codes >> (8 * j)) & 15u), scale, mn), __fmaf_rn(float((codes >> (8 * j + 4)) & 15u), scale, mn));
            *reinterpret_cast<uint4*>((kv ? dst_v : dst_k) + dst_row + g * 32u + part * 8u) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

}  // namespace kriya

cudaError_t kriya_launch_q4_expand_blocks(const void* pool_k, const void* pool_v, void* dst_k, void* dst_v, const int32_t* indices,
                                          uint32_t n_indices, uint32_t block_tokens, uint32_t hkv, uint32_t head_dim, uint32_t num_blocks,
                                          uint32_t dtype, uint32_t* status, cudaStream_t s) {
    if (n_indices == 0) return cudaSuccess;
    const uint64_t rows = uint64_t(n_indices) * block_tokens * hkv;
    const uint32_t grid = uint32_t((rows + 7u) / 8u);
    if (dtype == KRIYA_DTYPE_FP16)
        kriya::q4_expand_blocks_kernel<kriya::Fp16><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(pool_k), static_cast<const uint8_t*>(pool_v),
                                                                         static_cast<uint16_t*>(dst_k), static_cast<uint16_t*>(dst_v), indices,
                                                                         n_indices, block_tokens, hkv, head_dim, num_blocks, status);
    else
        kriya::q4_expand_blocks_kernel<kriya::Bf16><<<grid, 256, 0, s>>>(static_cast<const uint8_t*>(pool_k), static_cast<const uint8_t*>(pool_v),
                                                                         static_cast<uint16_t*>(dst_k), static_cast<uint16_t*>(dst_v), indices,
                                                                         n_indices, block_tokens, hkv, head_dim, num_blocks, status);
    return cudaGetLastError();
}
