// skv_decode_attn_static: paged decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc on the hot path or at all: a serving process whose
// memory is fully carved up by its own allocator at start-up, a plugin that runs inside someone
// else's pre-sized arena, a latency-critical loop in which an allocation would synchronise the device.  skv_decode_attn asks such a caller for a workspace it has no way to
// provide.  This variant keeps the split-K partials in a fixed array that is part of the loaded
// library image instead, so the caller passes only its inputs and its output.
//
// Limits and rules that follow from that:
//   * The array is kStaticScratchBytes (16 MiB) on every GPU that loads the library, for the life of
//     the process.  A call whose partials need more is rejected with SKV_ERR_UNSUPPORTED and a message
//     that names both sizes; nothing is launched.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress with that
//     device current).  Make that first call outside any stream capture.
//   * All calls on a device share the one array and it keeps whatever the previous call left.  Nothing
//     in it has to start at zero: every partial the merge kernel reads was written by the split kernel
//     of the same call.  Two calls whose kernels overlap on the GPU (different streams, no ordering
//     between them) race on it -- order them on one stream or with events.
//   * No cudaMalloc / cudaFree / allocating library routine is reached from this entry point; per-call
//     metadata goes through the pool's staging slots that were allocated by skv_create.
#include <cstdio>
#include <mutex>

#include "common.cuh"

namespace {

constexpr size_t kStaticScratchBytes = SKV_STATIC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

// Lives in device memory of every GPU that loads this module.  In host code this name is only a
// handle for cudaGetSymbolAddress, never an address to hand to a kernel.
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

std::mutex g_setup_mutex;
void* g_scratch_addr[kMaxDevices] = {};

// Device address of the array on the pool's device, looked up once per device with that device current.
cudaError_t scratch_address(int device, void** out) {
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_addr[device]) {
        int prev = -1;
        cudaError_t e = cudaGetDevice(&prev);
        if (e != cudaSuccess) return e;
        if (prev != device) {
            e = cudaSetDevice(device);
            if (e != cudaSuccess) return e;
        }
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_decode_scratch);
        if (prev != device) cudaSetDevice(prev);
        if (e != cudaSuccess) return e;
        if (!ptr) return cudaErrorInvalidSymbol;
        g_scratch_addr[device] = ptr;
    }
    *out = g_scratch_addr[device];
    return cudaSuccess;
}

}  // namespace

extern "C" SKV_API int32_t skv_decode_attn_static(skv_pool* pool, int32_t layer, const int32_t* seq_ids, int32_t n_seqs,
                                                  const void* q, void* out, const int32_t* q_pos, int32_t n_q_heads,
                                                  float eps, void* stream_) {
    using namespace skv;
    if (!pool) return SKV_ERR_BAD_ARG;
    cudaStream_t stream = (cudaStream_t)stream_;
    const int device = pool_device(pool);
    int prev = -1;
    const bool on_gpu = device >= 0;
    if (on_gpu) {
        if (cudaGetDevice(&prev) != cudaSuccess) return pool_fail(pool, SKV_ERR_CUDA, "cudaGetDevice failed");
        if (prev != device && cudaSetDevice(device) != cudaSuccess) return pool_fail(pool, SKV_ERR_CUDA, "cudaSetDevice failed");
    }
    int32_t status = [&]() -> int32_t {
        DecodeLaunch d{};
        int64_t total = 0;
        int32_t launchable = 0;
        int32_t st = prepare_decode(pool, layer, seq_ids, n_seqs, q_pos, n_q_heads, q, out, eps, stream, &d, &total, &launchable);
        if (st != SKV_OK || !launchable) return st;
        d.total_tokens = total;
        decode_plan(d.pool.page_size, d.pool.max_pages_per_seq, n_seqs, d.pool.num_kv_heads, total, d.longest, &d.chunk_tokens, &d.max_splits);
        const size_t rows = (size_t)n_seqs * n_q_heads * d.max_splits;
        const size_t need = rows * ((size_t)d.pool.head_dim + 2) * sizeof(float);
        if (need > kStaticScratchBytes) {
            char msg[200];
            snprintf(msg, sizeof msg,
                     "split-K partials need %zu bytes, the built-in scratch array holds %zu; use skv_decode_attn with a "
                     "caller workspace or a smaller batch", need, kStaticScratchBytes);
            return pool_fail(pool, SKV_ERR_UNSUPPORTED, msg);
        }
        void* base = nullptr;
        cudaError_t e = scratch_address(device, &base);
        if (e != cudaSuccess) return pool_fail(pool, SKV_ERR_CUDA, cudaGetErrorString(e));
        d.ws_acc = reinterpret_cast<float*>(base);
        d.ws_ml = d.ws_acc + rows * d.pool.head_dim;
        e = launch_decode(d, stream);
        if (e != cudaSuccess) return pool_fail(pool, SKV_ERR_CUDA, cudaGetErrorString(e));
        return SKV_OK;
    }();
    if (on_gpu && prev != device) cudaSetDevice(prev);
    return status;
}
