// Byte movers of the paged cache: the copy-on-write block copy and the single-slot write.
//
// Block copy: the reference produces (src, dst) pairs (crates/kriya-kv/src/bsr_paged.rs:412-420) and
// ships no consumer; the intended effect is dst := src for every layer, K and V.  One CTA copies one
// (pair, layer, K|V) block with 16-byte loads and stores, so a launch moves
// n_pairs * layers * 2 * block_bytes in and the same out, bound by HBM bandwidth.
//
// Slot write: the speculative-KV commit of crates/kriya-backend-metal/src/encoder.rs:3591-3664, a
// bit-for-bit copy of one staged K row and V row into (block, slot).
#include "kriya_device.cuh"

namespace kriya {

__global__ void __launch_bounds__(256) block_copy_kernel(uint8_t* pool_k, uint8_t* pool_v, size_t layer_stride,
                                                         uint32_t num_layers, size_t block_bytes,
                                                         const uint32_t* __restrict__ pairs, uint32_t n_pairs) {
    // blockIdx.x enumerates (pair, layer, k|v); consecutive CTAs touch consecutive layers of one pair
    const uint32_t job = blockIdx.x;
    const uint32_t kv = job & 1u;
    const uint32_t layer = (job >> 1) % num_layers;
    const uint32_t pair = (job >> 1) / num_layers;
    if (pair >= n_pairs) return;
    const uint32_t src = pairs[2 * pair], dst = pairs[2 * pair + 1];
    if (src == dst) return;
    uint8_t* base = (kv ? pool_v : pool_k) + size_t(layer) * layer_stride;
    const uint4* s = reinterpret_cast<const uint4*>(base + size_t(src) * block_bytes);
    uint4* d = reinterpret_cast<uint4*>(base + size_t(dst) * block_bytes);
    const uint32_t n16 = uint32_t(block_bytes / 16);
    for (uint32_t i = threadIdx.x; i < n16; i += blockDim.x) d[i] = s[i];
}

__global__ void __launch_bounds__(128) slot_write_kernel(uint8_t* cache_k, uint8_t* cache_v, const uint8_t* stage_k,
                                                         const uint8_t* stage_v, size_t row_bytes, uint32_t block_size,
                                                         const uint32_t* __restrict__ triples, uint32_t n,
                                                         uint32_t num_blocks, uint32_t* status) {
    const uint32_t job = blockIdx.x;  // (triple, k|v)
    const uint32_t kv = job & 1u, t = job >> 1;
    if (t >= n) return;
    const uint32_t node = triples[3 * t], blk = triples[3 * t + 1], slot = triples[3 * t + 2];
    if (blk >= num_blocks || slot >= block_size) {
        if (threadIdx.x == 0) atomicMax(status, blk >= num_blocks ? KRIYA_DEV_BAD_BLOCK_INDEX : KRIYA_DEV_BAD_SLOT);
        return;
    }
    const uint8_t* s = (kv ? stage_v : stage_k) + size_t(node) * row_bytes;
    uint8_t* d = (kv ? cache_v : cache_k) + (size_t(blk) * block_size + slot) * row_bytes;
    const uint32_t n16 = uint32_t(row_bytes / 16);
    for (uint32_t i = threadIdx.x; i < n16; i += blockDim.x)
        reinterpret_cast<uint4*>(d)[i] = reinterpret_cast<const uint4*>(s)[i];
}

}  // namespace kriya

cudaError_t kriya_launch_block_copy(uint8_t* pool_k, uint8_t* pool_v, size_t layer_stride_bytes, uint32_t num_layers,
                                    size_t block_bytes, const uint32_t* pairs_dev, uint32_t n_pairs, int /*sm_count*/,
                                    cudaStream_t s) {
    if (n_pairs == 0) return cudaSuccess;
    const uint32_t grid = n_pairs * num_layers * 2u;
    kriya::block_copy_kernel<<<grid, 256, 0, s>>>(pool_k, pool_v, layer_stride_bytes, num_layers, block_bytes, pairs_dev,
                                                   n_pairs);
    return cudaGetLastError();
}

cudaError_t kriya_launch_slot_write(uint8_t* cache_k, uint8_t* cache_v, const void* stage_k, const void* stage_v,
                                    size_t row_bytes, uint32_t block_size, const uint32_t* triples_dev, uint32_t n,
                                    uint32_t num_blocks, uint32_t* status, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    kriya::slot_write_kernel<<<n * 2u, 128, 0, s>>>(cache_k, cache_v, static_cast<const uint8_t*>(stage_k),
                                                    static_cast<const uint8_t*>(stage_v), row_bytes, block_size,
                                                    triples_dev, n, num_blocks, status);
    return cudaGetLastError();
}

// ---- self-test of the bounded waits --------------------------------------------------------------------------------
// Every wait inside this library's kernels is bounded: when its limit passes, the kernel records a status word and
// returns instead of hanging.  This one-block kernel exercises exactly that path without any fault: it initialises a
// barrier that nobody ever arrives at, waits on it with the given limit and reports the expiry.
namespace kriya {
__global__ void wait_selftest_kernel(uint32_t* status, uint64_t wait_ns) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    const bool ok = warp_wait(&bar, 0u, wait_ns);
    if (!ok && threadIdx.x == 0) atomicMax(status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
}
}  // namespace kriya

cudaError_t kriya_launch_wait_selftest(uint32_t* status, uint64_t wait_ns, cudaStream_t s) {
    kriya::wait_selftest_kernel<<<1, 32, 0, s>>>(status, wait_ns);
    return cudaGetLastError();
}
