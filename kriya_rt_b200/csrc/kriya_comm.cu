// One long sequence split along the KV axis over the GPUs of one box: the exchange of the partial softmax states and
// their merge, behind the C ABI (kriya_cuda_comm_export / _init, kriya_cuda_kvsplit_decode).
//
// The reference is single-GPU (crates/kriya-scheduler/src/orca_engine.rs:21-24: one ColocatedHybrid role); what is split
// here is its split-K design (kernels/metal/paged_gqa_and_deltanet.metal:328-342,1493-1524) taken across devices: every
// rank holds a contiguous block range of the sequence in its own pool, runs the partial-state decode over it and ends
// with the (max, sum, output) state of every (row, query head).  The exchange is one kernel per rank and layer:
//   1. it stores the rank's state into its slot of an exchange buffer in EVERY peer's own memory (plain peer stores over
//      NVLink, 8-byte (value, stamp) pairs, so no fence and no separate flag are needed),
//   2. it then polls its own buffer until the slots of all ranks carry this call's stamp (bounded: after about a
//      second it gives up, records a status word and returns), merges them and writes the normalised output.
// No collective library is involved and nothing is read from a peer: a rank only writes to peers and reads its own
// memory.  Exchange buffers rotate over four generations; a rank can be at most one call ahead of a peer's merge, so a
// slot is never overwritten before it has been read.
#include <string.h>
#include <unistd.h>

#include <string>

#include "kriya_device.cuh"
#include "kriya_internal.h"

namespace kriya {

constexpr uint32_t kCommBufs = 4;
constexpr uint64_t kCommWaitNs = 1000000000ull;  // a peer that has not delivered after a second is given up on

__device__ __forceinline__ void comm_store(uint2* p, float v, uint32_t stamp) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(stamp) : "memory");
}
__device__ __forceinline__ uint2 comm_load(const uint2* p) {
    uint2 r;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p) : "memory");
    return r;
}

struct CommKernelArgs {
    uint2* stage[KRIYA_COMM_MAX_RANKS];  // every rank's exchange buffer (peer mappings; [rank] is this rank's own)
    const float* local;                  // this rank's packed state [m (R) | l (R) | o (R * D)]
    void* out;                           // [R][D] 16-bit
    uint32_t* status;
    uint32_t nranks, rank, R, D;
    uint32_t stamp;                      // never zero
    size_t slot_words;                   // uint2 words of one rank's slot: cap_R * (D + 2)
    size_t buf_off;                      // offset (uint2 words) of this call's generation inside a buffer
    uint32_t wait_previous;              // launched as a programmatic dependent of the kernel that writes `local`
    uint64_t wait_ns;                    // how long a peer's words are waited for: the context's wait limit, a second at most
};

// One block per (row, query head), one thread per output dimension (blockDim.x == D).
template <typename T>
__global__ void kvsplit_exchange_merge_kernel(CommKernelArgs a) {
    if (a.wait_previous) asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t rh = blockIdx.x, d = threadIdx.x;
    const float m_loc = a.local[rh], l_loc = a.local[a.R + rh], o_loc = a.local[2 * size_t(a.R) + size_t(rh) * a.D + d];
    // slot layout: [rh][D + 2] words: o[0..D), m, l
    const size_t word = a.buf_off + size_t(a.rank) * a.slot_words + size_t(rh) * (a.D + 2);
    for (uint32_t p = 0; p < a.nranks; ++p) {
        uint2* dst = a.stage[p] + word;
        comm_store(dst + d, o_loc, a.stamp);
        if (d == 0) comm_store(dst + a.D, m_loc, a.stamp);
        if (d == 1) comm_store(dst + a.D + 1, l_loc, a.stamp);
    }
    // gather: this rank's own buffer, all ranks' slots
    const uint2* mine = a.stage[a.rank] + a.buf_off + size_t(rh) * (a.D + 2);
    float M = -INFINITY, L = 0.0f, O = 0.0f;
    bool ok = true;
    const uint64_t t_start = global_timer_ns();
    for (uint32_t p = 0; p < a.nranks && ok; ++p) {
        const uint2* src = mine + size_t(p) * a.slot_words;
        uint2 wo, wm, wl;
        for (uint32_t spin = 0;; ++spin) {
            wo = comm_load(src + d);
            wm = comm_load(src + a.D);
            wl = comm_load(src + a.D + 1);
            if (wo.y == a.stamp && wm.y == a.stamp && wl.y == a.stamp) break;
            if ((spin & 63u) == 63u && global_timer_ns() - t_start > a.wait_ns) {
                ok = false;
                break;
            }
        }
        if (!ok) break;
        const float mp = __uint_as_float(wm.x);
        if (mp == -INFINITY) continue;  // that rank's range held nothing for this row
        const float mc = fmaxf(M, mp);
        const float keep = (M == -INFINITY) ? 0.0f : expf(M - mc);
        const float w = expf(mp - mc);
        L = fmaf(w, __uint_as_float(wl.x), L * keep);
        O = fmaf(w, __uint_as_float(wo.x), O * keep);
        M = mc;
    }
    if (!ok) {
        if (d == 0) atomicMax(a.status, uint32_t(KRIYA_DEV_WAIT_EXPIRED));
        return;
    }
    reinterpret_cast<uint16_t*>(a.out)[size_t(rh) * a.D + d] = T::store(O / fmaxf(L, 1e-12f));
}

}  // namespace kriya

struct kriya_comm_state {
    uint32_t nranks = 0, rank = 0, cap_R = 0;
    uint32_t stamp = 0;
    uint8_t* own = nullptr;  // this rank's exchange buffer
    size_t own_bytes = 0;
    void* peer[KRIYA_COMM_MAX_RANKS] = {};
    bool opened[KRIYA_COMM_MAX_RANKS] = {};  // mapping obtained through cudaIpcOpenMemHandle
    float* local = nullptr;                  // packed local state [cap_R * (D + 2)]
    bool ready = false;
};

namespace {

struct HandleBlob {  // KRIYA_COMM_HANDLE_BYTES
    uint32_t magic;
    uint32_t device;
    uint64_t pid;
    uint64_t ptr;
    uint64_t bytes;
    uint32_t cap_R;
    uint32_t D;
    cudaIpcMemHandle_t ipc;
    uint8_t pad[KRIYA_COMM_HANDLE_BYTES - 40 - sizeof(cudaIpcMemHandle_t)];
};
static_assert(sizeof(HandleBlob) == KRIYA_COMM_HANDLE_BYTES, "handle blob size");
constexpr uint32_t kHandleMagic = 0x4B52434Du;

void comm_release(kriya_cuda_ctx* c) {
    kriya_comm_state* s = c->comm;
    if (!s) return;
    for (uint32_t p = 0; p < KRIYA_COMM_MAX_RANKS; ++p)
        if (s->opened[p] && s->peer[p]) cudaIpcCloseMemHandle(s->peer[p]);
    cudaFree(s->own);
    cudaFree(s->local);
    delete s;
    c->comm = nullptr;
}

#define COMM_TRY(ctx, expr)                                                                                \
    do {                                                                                                   \
        cudaError_t _e = (expr);                                                                           \
        if (_e != cudaSuccess)                                                                             \
            return (ctx)->fail(KRIYA_CUDA_EXECUTION_ERROR, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
    } while (0)

}  // namespace

void kriya_comm_destroy(kriya_cuda_ctx* c) { comm_release(c); }

extern "C" {

int32_t kriya_cuda_comm_export(kriya_cuda_ctx* c, uint32_t max_rows, void* handle_out) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (!handle_out || max_rows == 0) return c->fail(KRIYA_CUDA_INVALID_INPUT, "handle_out must not be null and max_rows must be positive");
    if (c->cfg.head_dim > 1024) return c->fail(KRIYA_CUDA_UNSUPPORTED, "head_dim too large for the exchange kernel");
    cudaSetDevice(c->cfg.device);
    COMM_TRY(c, cudaStreamSynchronize(c->stream));
    comm_release(c);
    auto* s = new kriya_comm_state();
    c->comm = s;
    s->cap_R = max_rows * c->cfg.num_q_heads;
    const size_t slot_words = size_t(s->cap_R) * (c->cfg.head_dim + 2);
    s->own_bytes = size_t(kriya::kCommBufs) * KRIYA_COMM_MAX_RANKS * slot_words * sizeof(uint2);
    COMM_TRY(c, cudaMalloc(&s->own, s->own_bytes));
    COMM_TRY(c, cudaMemset(s->own, 0, s->own_bytes));  // stamps start at zero, which no call uses
    COMM_TRY(c, cudaMalloc(&s->local, slot_words * sizeof(float)));
    HandleBlob h;
    memset(&h, 0, sizeof h);
    h.magic = kHandleMagic;
    h.device = uint32_t(c->cfg.device);
    h.pid = uint64_t(getpid());
    h.ptr = reinterpret_cast<uint64_t>(s->own);
    h.bytes = s->own_bytes;
    h.cap_R = s->cap_R;
    h.D = c->cfg.head_dim;
    COMM_TRY(c, cudaIpcGetMemHandle(&h.ipc, s->own));
    memcpy(handle_out, &h, sizeof h);
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_comm_init(kriya_cuda_ctx* c, uint32_t nranks, uint32_t rank, const void* handles) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    kriya_comm_state* s = c->comm;
    if (!s || !s->own) return c->fail(KRIYA_CUDA_INVALID_INPUT, "kriya_cuda_comm_export must be called first");
    if (!handles || nranks == 0 || nranks > KRIYA_COMM_MAX_RANKS || rank >= nranks)
        return c->fail(KRIYA_CUDA_INVALID_INPUT, "comm_init needs 1..=" + std::to_string(KRIYA_COMM_MAX_RANKS) + " ranks, rank < nranks and all ranks' handles");
    cudaSetDevice(c->cfg.device);
    const auto* hs = static_cast<const HandleBlob*>(handles);
    for (uint32_t p = 0; p < nranks; ++p) {
        const HandleBlob& h = hs[p];
        if (h.magic != kHandleMagic) return c->fail(KRIYA_CUDA_INVALID_INPUT, "handle of rank " + std::to_string(p) + " is not an exchange-buffer handle");
        if (h.cap_R != s->cap_R || h.D != c->cfg.head_dim || h.bytes != s->own_bytes)
            return c->fail(KRIYA_CUDA_INVALID_INPUT, "rank " + std::to_string(p) + " exported a buffer of another shape");
        if (p == rank) {
            if (h.ptr != reinterpret_cast<uint64_t>(s->own) || h.pid != uint64_t(getpid()))
                return c->fail(KRIYA_CUDA_INVALID_INPUT, "handles[rank] is not this context's own handle");
            s->peer[p] = s->own;
        } else if (h.pid == uint64_t(getpid())) {
            // another context of this process: its pointer is valid here once peer access is on
            if (int(h.device) != c->cfg.device) {
                int can = 0;
                COMM_TRY(c, cudaDeviceCanAccessPeer(&can, c->cfg.device, int(h.device)));
                if (!can) return c->fail(KRIYA_CUDA_UNSUPPORTED, "no peer access between devices " + std::to_string(c->cfg.device) + " and " + std::to_string(h.device));
                const cudaError_t e = cudaDeviceEnablePeerAccess(int(h.device), 0);
                if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
                    return c->fail(KRIYA_CUDA_EXECUTION_ERROR, std::string("cudaDeviceEnablePeerAccess: ") + cudaGetErrorString(e));
                (void)cudaGetLastError();
            }
            s->peer[p] = reinterpret_cast<void*>(h.ptr);
        } else {
            void* mapped = nullptr;
            COMM_TRY(c, cudaIpcOpenMemHandle(&mapped, h.ipc, cudaIpcMemLazyEnablePeerAccess));
            s->peer[p] = mapped;
            s->opened[p] = true;
        }
    }
    s->nranks = nranks;
    s->rank = rank;
    s->stamp = 0;
    s->ready = true;
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_kvsplit_decode(kriya_cuda_ctx* c, uint32_t layer, const void* q_dev, void* out_dev,
                                  const kriya_bsr_gqa_params* params) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    kriya_comm_state* s = c->comm;
    if (!s || !s->ready) return c->fail(KRIYA_CUDA_INVALID_INPUT, "kriya_cuda_comm_init must be called first");
    if (!c->plan_valid) return c->fail(KRIYA_CUDA_INVALID_INPUT, "no plan uploaded");
    const uint32_t R = c->n_rows * c->cfg.num_q_heads, D = c->cfg.head_dim;
    if (R > s->cap_R) return c->fail(KRIYA_CUDA_INVALID_INPUT, "plan has " + std::to_string(c->n_rows) + " rows but the exchange buffer was exported for " + std::to_string(s->cap_R / c->cfg.num_q_heads));
    if (!out_dev) return c->fail(KRIYA_CUDA_INVALID_INPUT, "q and out must not be null");
    // partial state over the ranges of kriya_cuda_plan_set_ranges (the whole rows when none were set)
    if (int32_t rc = kriya_cuda_paged_gqa_decode_partial(c, layer, q_dev, nullptr, nullptr, s->local, s->local + R, s->local + 2 * size_t(R), params))
        return rc;
    if (++s->stamp == 0u) s->stamp = 1u;
    kriya::CommKernelArgs a{};
    for (uint32_t p = 0; p < s->nranks; ++p) a.stage[p] = static_cast<uint2*>(s->peer[p]);
    a.local = s->local;
    a.out = out_dev;
    a.status = c->d_status;
    a.nranks = s->nranks;
    a.rank = s->rank;
    a.R = R;
    a.D = D;
    a.stamp = s->stamp;
    a.slot_words = size_t(s->cap_R) * (D + 2);
    a.buf_off = size_t(s->stamp % kriya::kCommBufs) * KRIYA_COMM_MAX_RANKS * a.slot_words;
    a.wait_previous = 1u;
    a.wait_ns = std::min<uint64_t>(c->wait_ns, kriya::kCommWaitNs);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(R);
    cfg.blockDim = dim3(D);
    cfg.stream = c->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (c->cfg.dtype == KRIYA_DTYPE_FP16)
        COMM_TRY(c, cudaLaunchKernelEx(&cfg, kriya::kvsplit_exchange_merge_kernel<kriya::Fp16>, a));
    else
        COMM_TRY(c, cudaLaunchKernelEx(&cfg, kriya::kvsplit_exchange_merge_kernel<kriya::Bf16>, a));
    c->launches += 1;
    return KRIYA_CUDA_OK;
}

int32_t kriya_cuda_kvsplit_decode_step(kriya_cuda_ctx* c, const void* q_dev, void* out_dev, const kriya_bsr_gqa_params* params) {
    if (!c) return KRIYA_CUDA_INVALID_INPUT;
    if (!q_dev || !out_dev) return c->fail(KRIYA_CUDA_INVALID_INPUT, "q and out must not be null");
    if (!c->plan_valid) return c->fail(KRIYA_CUDA_INVALID_INPUT, "no plan uploaded");
    const size_t qb = size_t(c->n_rows) * c->cfg.num_q_heads * c->cfg.head_dim * 2;
    for (uint32_t layer = 0; layer < c->cfg.num_layers; ++layer)
        if (int32_t rc = kriya_cuda_kvsplit_decode(c, layer, static_cast<const uint8_t*>(q_dev) + layer * qb,
                                                   static_cast<uint8_t*>(out_dev) + layer * qb, params))
            return rc;
    return KRIYA_CUDA_OK;
}

}  // extern "C"
