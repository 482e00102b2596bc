// Paged GQA decode for callers that must not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: a serving process whose device memory is handed out
// up front by its own arena allocator, or a plugin loaded into such a process.  kriya_cuda_ctx_create allocates pools
// and scratch, so those callers cannot own a context.  For them this file offers one self-contained decode call that
// needs nothing but the caller's own buffers: the split-KV partial states, the ticket counters, the work list and the
// status word live in a file-scope __device__ array that every GPU loading the library carries until exit.
//
// The attention kernel is the CUDA-core decode kernel of kriya_decode.cu, unchanged; only where its scratch lives
// differs.  Its work list is written by a one-block kernel from the caller's device-side page_indptr, so nothing the
// launch reads lives in host memory.
#include <string.h>

#include <algorithm>
#include <cstdio>
#include <mutex>

#include "kriya_internal.h"

namespace {

// Limits of the static scratch (about 4.3 MB per GPU).
constexpr uint32_t kMaxRows = 256;                 // plan rows per call
constexpr uint32_t kMaxWork = 512;                 // work items per call
constexpr uint32_t kMaxHqD = 16 * 128;             // num_q_heads * head_dim
constexpr size_t kOffPartO = 0;                                            // float [kMaxWork][kMaxHqD]
constexpr size_t kOffPartMl = kOffPartO + size_t(kMaxWork) * kMaxHqD * 4;  // float [kMaxWork][Hq][2], Hq <= kMaxHqD / 64
constexpr size_t kOffCounters = kOffPartMl + size_t(kMaxWork) * (kMaxHqD / 64) * 2 * 4;  // uint32 [kMaxRows]
constexpr size_t kOffStatus = kOffCounters + size_t(kMaxRows) * 4;         // uint32 (padded to 256 B)
constexpr size_t kOffWork = kOffStatus + 256;                              // KriyaDecodeWork [kMaxWork]
constexpr size_t kScratchBytes = kOffWork + size_t(kMaxWork) * sizeof(KriyaDecodeWork);

static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

// In host code `g_static_scratch` is only a stand-in for the symbol; the device address comes from
// cudaGetSymbolAddress, once per device, with that device current.
constexpr int kMaxDevices = 64;
unsigned char* g_scratch_dev[kMaxDevices] = {};
int g_max_smem_optin[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};
std::mutex g_setup_mutex;

// Writes the work list into the scratch array: row r is cut into ceil(blocks / chunk) near-equal block ranges, rows in
// order, item index == scratch slot.  `n_expected` is the item count the host derived from its copy of page_indptr
// (it is the grid of the decode launch that follows); a device-side table that disagrees is reported through the status
// word and can never produce an item outside the scratch: surplus items are dropped, missing ones become empty ranges
// of row 0 that own the last slot.
__global__ void static_work_kernel(const int32_t* __restrict__ indptr, uint32_t rows, uint32_t chunk, uint32_t n_expected,
                                   KriyaDecodeWork* __restrict__ work, uint32_t* __restrict__ status) {
    __shared__ uint32_t base[kMaxRows + 1];
    const uint32_t r = threadIdx.x;
    uint32_t nb = 0, parts = 0;
    if (r < rows) {
        const int32_t d = indptr[r + 1] - indptr[r];
        nb = d > 0 ? uint32_t(d) : 0u;
        parts = nb ? (nb + chunk - 1) / chunk : 1u;
    }
    base[r + 1] = parts;
    if (r == 0) base[0] = 0;
    __syncthreads();
    if (r == 0)
        for (uint32_t i = 1; i <= kMaxRows; ++i) base[i] += base[i - 1];
    __syncthreads();
    const uint32_t total = base[kMaxRows];
    if (r == 0 && total != n_expected) atomicMax(status, uint32_t(KRIYA_DEV_BAD_SLOT));
    if (r < rows) {
        const uint32_t first = base[r];
        const uint32_t size = (nb + parts - 1) / parts;
        for (uint32_t k = 0; k < parts; ++k) {
            const uint32_t i = first + k;
            if (i >= n_expected || first + parts > n_expected) break;
            KriyaDecodeWork w{};
            w.req = r;
            w.blk_begin = min(k * size, nb);
            w.blk_end = min((k + 1) * size, nb);
            w.slot = i;
            w.first_slot = first;
            w.n_parts = parts;
            work[i] = w;
        }
    }
    for (uint32_t i = min(total, n_expected) + r; i < n_expected; i += blockDim.x) {
        KriyaDecodeWork w{};
        w.slot = w.first_slot = kMaxWork - 1u;
        w.n_parts = 1u;
        work[i] = w;
    }
}

int32_t fail(char* err, size_t err_len, int32_t code, const char* msg, const char* detail = nullptr) {
    if (err && err_len) snprintf(err, err_len, "%s%s%s", msg, detail ? ": " : "", detail ? detail : "");
    return code;
}

}  // namespace

extern "C" int32_t kriya_cuda_paged_gqa_decode_static(int32_t device, void* stream, uint32_t dtype, const void* q_dev,
                                                      const void* cache_k_dev, const void* cache_v_dev,
                                                      uint32_t num_kv_blocks, const int32_t* page_indptr_host,
                                                      const int32_t* page_indptr_dev, const int32_t* page_indices_dev,
                                                      const int32_t* last_page_len_dev, uint32_t rows, void* out_dev,
                                                      const kriya_bsr_gqa_params* params, char* err, size_t err_len) {
    if (!q_dev || !cache_k_dev || !cache_v_dev || !page_indptr_host || !page_indptr_dev || !page_indices_dev ||
        !last_page_len_dev || !out_dev || !params)
        return fail(err, err_len, KRIYA_CUDA_INVALID_INPUT, "null argument");
    if (device < 0 || device >= kMaxDevices) return fail(err, err_len, KRIYA_CUDA_INVALID_INPUT, "device ordinal out of range");
    if (dtype != KRIYA_DTYPE_BF16 && dtype != KRIYA_DTYPE_FP16) return fail(err, err_len, KRIYA_CUDA_INVALID_INPUT, "bad dtype");
    if (rows == 0) return fail(err, err_len, KRIYA_CUDA_INVALID_INPUT, "input_tokens must not be empty");
    const uint32_t Hq = params->num_q_heads, Hkv = params->num_kv_heads, D = params->head_dim;
    if (Hkv == 0 || Hq % Hkv != 0 || !kriya_decode_supported(D, Hq / Hkv, Hkv, params->block_size_tokens))
        return fail(err, err_len, KRIYA_CUDA_UNSUPPORTED,
                    "shape not covered: head_dim 64/128, group size 1..8, up to 8 KV heads, 16-token blocks");
    char buf[160];
    if (rows > kMaxRows) {
        snprintf(buf, sizeof buf, "%u rows, the static scratch holds %u", rows, kMaxRows);
        return fail(err, err_len, KRIYA_CUDA_INVALID_INPUT, "too many plan rows", buf);
    }
    if (Hq * D > kMaxHqD) {
        snprintf(buf, sizeof buf, "num_q_heads * head_dim = %u, the static scratch holds %u", Hq * D, kMaxHqD);
        return fail(err, err_len, KRIYA_CUDA_INVALID_INPUT, "query width too large", buf);
    }
    if (page_indptr_host[0] != 0) return fail(err, err_len, KRIYA_CUDA_INVALID_INPUT, "page_indptr must start at 0");
    for (uint32_t r = 0; r < rows; ++r)
        if (page_indptr_host[r + 1] <= page_indptr_host[r])
            return fail(err, err_len, KRIYA_CUDA_INVALID_INPUT, "every row needs at least one KV block and page_indptr must increase");

    // the caller's current device is put back before returning
    struct DeviceGuard {
        int prev = -1;
        ~DeviceGuard() {
            if (prev >= 0) cudaSetDevice(prev);
        }
    } guard;
    cudaError_t e = cudaGetDevice(&guard.prev);
    if (e != cudaSuccess) guard.prev = -1;
    if (guard.prev == device) guard.prev = -1;  // nothing to restore
    else if ((e = cudaSetDevice(device)) != cudaSuccess)
        return fail(err, err_len, KRIYA_CUDA_DEVICE_INIT_FAILED, "cudaSetDevice", cudaGetErrorString(e));
    {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (!g_scratch_dev[device]) {  // first call on this device: resolve the symbol's device address
            void* ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_static_scratch);
            if (e != cudaSuccess || !ptr)
                return fail(err, err_len, KRIYA_CUDA_DEVICE_INIT_FAILED, "cudaGetSymbolAddress", cudaGetErrorString(e));
            cudaDeviceProp prop{};
            e = cudaGetDeviceProperties(&prop, device);
            if (e != cudaSuccess) return fail(err, err_len, KRIYA_CUDA_DEVICE_INIT_FAILED, "cudaGetDeviceProperties", cudaGetErrorString(e));
            if (prop.major != 10) return fail(err, err_len, KRIYA_CUDA_DEVICE_INIT_FAILED, "this library holds sm_100a code only");
            g_max_smem_optin[device] = int(prop.sharedMemPerBlockOptin);
            g_sm_count[device] = prop.multiProcessorCount;
            g_scratch_dev[device] = static_cast<unsigned char*>(ptr);
        }
    }
    unsigned char* scratch = g_scratch_dev[device];
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    // Size of the work list: rows cut into near-equal block ranges of at most `chunk` blocks, about two items per SM;
    // a coarser cut when that overflows the list.  Only the count and the chunk are computed here; the list itself is
    // written on the device from page_indptr_dev.
    uint64_t total = 0;
    for (uint32_t r = 0; r < rows; ++r) total += uint32_t(page_indptr_host[r + 1] - page_indptr_host[r]);
    const uint32_t target = 2u * uint32_t(g_sm_count[device]);
    uint32_t chunk = std::max<uint32_t>(2u, uint32_t((total + target - 1) / target));
    uint32_t n = 0;
    for (int pass = 0; pass < 2; ++pass) {
        uint64_t items = 0;
        for (uint32_t r = 0; r < rows; ++r) {
            const uint32_t nb = uint32_t(page_indptr_host[r + 1] - page_indptr_host[r]);
            items += (nb + chunk - 1) / chunk;
        }
        if (items <= kMaxWork) {
            n = uint32_t(items);
            break;
        }
        if (pass == 1) return fail(err, err_len, KRIYA_CUDA_INVALID_INPUT, "plan needs more work items than the static scratch holds");
        chunk = uint32_t((total + (kMaxWork - rows) - 1) / std::max(1u, kMaxWork - rows)) + 1u;
    }

    // the array keeps whatever the last call left: the tickets and the status word must start at zero
    e = cudaMemsetAsync(scratch + kOffCounters, 0, size_t(kMaxRows) * 4 + 256, s);
    if (e != cudaSuccess) return fail(err, err_len, KRIYA_CUDA_EXECUTION_ERROR, "cudaMemsetAsync", cudaGetErrorString(e));
    static_work_kernel<<<1, kMaxRows, 0, s>>>(page_indptr_dev, rows, chunk, n, reinterpret_cast<KriyaDecodeWork*>(scratch + kOffWork),
                                              reinterpret_cast<uint32_t*>(scratch + kOffStatus));
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(err, err_len, KRIYA_CUDA_EXECUTION_ERROR, "work-list launch", cudaGetErrorString(e));

    KriyaDecodeArgs a{};
    a.q = q_dev;
    a.cache_k = cache_k_dev;
    a.cache_v = cache_v_dev;
    a.indptr = page_indptr_dev;
    a.indices = page_indices_dev;
    a.last_len = last_page_len_dev;
    a.work = reinterpret_cast<const KriyaDecodeWork*>(scratch + kOffWork);
    a.out = out_dev;
    a.part_o = reinterpret_cast<float*>(scratch + kOffPartO);
    a.part_ml = reinterpret_cast<float*>(scratch + kOffPartMl);
    a.counters = reinterpret_cast<uint32_t*>(scratch + kOffCounters);
    a.status = reinterpret_cast<uint32_t*>(scratch + kOffStatus);
    a.n_work = n;
    a.num_blocks = num_kv_blocks;
    a.num_q_heads = Hq;
    a.num_kv_heads = Hkv;
    a.sm_scale = params->sm_scale;
    a.logit_softcap = params->logit_softcap;
    a.wait_ns = 2000000000ull;
    e = kriya_launch_decode(a, D, params->block_size_tokens, dtype, g_max_smem_optin[device], s);
    if (e != cudaSuccess) return fail(err, err_len, KRIYA_CUDA_EXECUTION_ERROR, "decode launch", cudaGetErrorString(e));
    return KRIYA_CUDA_OK;
}
