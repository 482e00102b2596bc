// Draft-tree part of speculative tree verification (the job of bsr_paged_gqa_tree_verify, part B,
// kernels/metal/paged_gqa_and_deltanet.metal:1694-1718, and its normalisation, :1720-1728).
//
// The prefix part (part A, :1656-1692) is a paged decode of every tree node over the same cached prefix and runs on the
// decode kernel, which leaves one un-normalised state (m, l, o) per (node, query head).  This kernel continues the same
// online-softmax recurrence over the in-flight K/V of the tree nodes that the mask makes visible and writes the
// normalised output: one warp per (node, query head), lanes over head_dim like the shader (lane holds D/32
// consecutive elements), score by a butterfly sum.  A tree has a few dozen nodes: the launch is latency-bound
// (it reads nodes * (Hq + 2 Hkv) * D * 2 B and writes nodes * Hq * D * 2 B).
#include "kriya_device.cuh"

namespace kriya {

constexpr int kTreeWarps = 4;

template <int D, typename T>
__global__ void __launch_bounds__(kTreeWarps * 32) tree_finish_kernel(KriyaTreeArgs a) {
    constexpr int VPT = D / 32;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t job = blockIdx.x * kTreeWarps + (threadIdx.x >> 5);
    const uint32_t Hq = a.num_q_heads, Hkv = a.num_kv_heads;
    if (job >= a.n_nodes * Hq) return;
    const uint32_t node = job / Hq, qh = job % Hq, kvh = qh / (Hq / Hkv);
    const uint16_t* q = reinterpret_cast<const uint16_t*>(a.q) + size_t(job) * D + lane * VPT;
    float qr[VPT], o[VPT];
    float m = -INFINITY, l = 0.0f;
#pragma unroll
    for (int t = 0; t < VPT; ++t) {
        qr[t] = __fmul_rn(T::load(q[t]), a.sm_scale);
        o[t] = 0.0f;
    }
    if (a.has_prefix) {
        m = a.st_m[job];
        l = a.st_l[job];
#pragma unroll
        for (int t = 0; t < VPT; ++t) o[t] = a.st_o[size_t(job) * D + lane * VPT + t];
    }
    const uint8_t* mrow = a.mask + size_t(node) * a.n_nodes;
    for (uint32_t j = 0; j < a.n_nodes; ++j) {
        if (mrow[j] == 0) continue;  // warp-uniform
        const uint16_t* k = reinterpret_cast<const uint16_t*>(a.k) + (size_t(j) * Hkv + kvh) * D + lane * VPT;
        const uint16_t* v = reinterpret_cast<const uint16_t*>(a.v) + (size_t(j) * Hkv + kvh) * D + lane * VPT;
        float dot = 0.0f;
#pragma unroll
        for (int t = 0; t < VPT; ++t) dot = __fmaf_rn(qr[t], T::load(k[t]), dot);
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) dot += __shfl_xor_sync(0xFFFFFFFFu, dot, off);
        const float m_new = fmaxf(m, dot);
        const float alpha = expf(m - m_new);  // m = -inf before the first visible key: alpha = 0
        const float beta = expf(dot - m_new);
        l = __fmaf_rn(l, alpha, beta);
#pragma unroll
        for (int t = 0; t < VPT; ++t) o[t] = __fmaf_rn(o[t], alpha, __fmul_rn(beta, T::load(v[t])));
        m = m_new;
    }
    const float inv_l = 1.0f / fmaxf(l, 1e-12f);
    uint16_t* out = reinterpret_cast<uint16_t*>(a.out) + size_t(job) * D + lane * VPT;
#pragma unroll
    for (int t = 0; t < VPT; ++t) out[t] = T::store(__fmul_rn(o[t], inv_l));
}

template <int D, typename T>
cudaError_t launch_tree_t(const KriyaTreeArgs& a, cudaStream_t s) {
    const uint32_t jobs = a.n_nodes * a.num_q_heads;
    tree_finish_kernel<D, T><<<(jobs + kTreeWarps - 1) / kTreeWarps, kTreeWarps * 32, 0, s>>>(a);
    return cudaGetLastError();
}

}  // namespace kriya

cudaError_t kriya_launch_tree_finish(const KriyaTreeArgs& a, uint32_t head_dim, uint32_t dtype, cudaStream_t s) {
    using namespace kriya;
    if (a.n_nodes == 0) return cudaSuccess;
    if (head_dim == 128) return dtype == KRIYA_DTYPE_FP16 ? launch_tree_t<128, Fp16>(a, s) : launch_tree_t<128, Bf16>(a, s);
    if (head_dim == 64) return dtype == KRIYA_DTYPE_FP16 ? launch_tree_t<64, Fp16>(a, s) : launch_tree_t<64, Bf16>(a, s);
    return cudaErrorInvalidValue;
}
