// Host side of the paged KV pool: allocator, page tables, lengths, replay rejection,
// staging of per-call metadata, and the C ABI entry points that launch the kernels.
//
// The reference keeps one growing tensor per layer and re-copies it on every append
// (src/ollm/mlx_kvcache.py:107-118).  Here a sequence owns a row of page ids; an append
// writes only the new tokens.  All validation that the reference does in Python
// (mlx_kvcache.py:127-158) happens here on the host before anything is launched.
#include <algorithm>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <thread>

#include "skv_internal.h"
#include "tma.cuh"

#include <atomic>
#include <mutex>

using namespace skv;

static std::atomic<long long> g_launches{0};
void skv::count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

namespace {
std::mutex g_switch_mutex;
skv::Switches g_switches;
std::atomic<bool> g_switches_ready{false};

int env_int(const char* name, int unset) {
    const char* e = getenv(name);
    return (e && *e) ? atoi(e) : unset;
}
bool env_is(const char* name, char c) {
    const char* e = getenv(name);
    return e && e[0] == c;
}
void read_switches() {
    skv::Switches w{};
    w.step_fused = !env_is("SKV_STEP_FUSED", '0');
    w.decode_generic = env_is("SKV_DECODE_GENERIC", '1');
    w.impl_reg = env_is("SKV_DECODE_IMPL", 'r');
    w.stages = env_int("SKV_DECODE_STAGES", 2);
    w.chunk = env_int("SKV_DECODE_CHUNK", 0);
    w.fuse = env_is("SKV_DECODE_FUSE", '0') ? 0 : (env_is("SKV_DECODE_FUSE", '1') ? 1 : -1);
    w.prefill_generic = env_is("SKV_PREFILL_GENERIC", '1');
    w.append_scalar = env_is("SKV_APPEND_SCALAR", '1');
    w.pdl = !env_is("SKV_PDL", '0');
    w.step_early = !env_is("SKV_STEP_EARLY", '0');
    {
        const char* e = getenv("SKV_DECODE_ORDER");
        w.order = (e && (e[0] == '0' || e[0] == '1')) ? e[0] - '0' : -1;
    }
    g_switches = w;
}
}  // namespace

const skv::Switches& skv::switches() {
    if (!g_switches_ready.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_switch_mutex);
        if (!g_switches_ready.load(std::memory_order_relaxed)) {
            read_switches();
            g_switches_ready.store(true, std::memory_order_release);
        }
    }
    return g_switches;
}
void skv::reload_switches() {
    std::lock_guard<std::mutex> lock(g_switch_mutex);
    read_switches();
    g_switches_ready.store(true, std::memory_order_release);
}

namespace {

struct TableUpdate {
    int32_t seq, slot, value;
};

// Pinned host slots with matching device slots.  A slot is reused only after the copy that
// read it has finished (one event per slot), so per-call metadata can be uploaded without
// blocking the host.  The event covers the upload, not the kernel that reads the device slot afterwards: that
// kernel is protected by stream order, so a ring must only ever be used with ONE stream (the pool keeps one
// ring for the compute stream and one for its copy stream; sharing one let 64 later uploads on the other stream
// overwrite a slot whose kernel had not run yet).
struct StagingRing {
    static constexpr int kSlots = 64;
    static constexpr size_t kSlotBytes = 64 * 1024;
    char* host = nullptr;
    char* dev = nullptr;
    cudaEvent_t ev[kSlots] = {};
    bool pending[kSlots] = {};
    int next = 0;
    int n_slots = kSlots;

    cudaError_t init(int slots = kSlots) {
        n_slots = slots < 1 ? 1 : (slots > kSlots ? kSlots : slots);
        cudaError_t e = cudaHostAlloc((void**)&host, n_slots * kSlotBytes, cudaHostAllocDefault);
        if (e != cudaSuccess) return e;
        e = cudaMalloc((void**)&dev, n_slots * kSlotBytes);
        if (e != cudaSuccess) return e;
        for (int i = 0; i < n_slots; ++i) {
            e = cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming);
            if (e != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    void destroy() {
        for (int i = 0; i < kSlots; ++i)
            if (ev[i]) cudaEventDestroy(ev[i]);
        if (dev) cudaFree(dev);
        if (host) cudaFreeHost(host);
    }
    // Copies `bytes` of `src` to the device through the next slot; *dev_out is valid on `stream`.
    cudaError_t upload(const void* src, size_t bytes, cudaStream_t stream, void** dev_out) {
        if (bytes > kSlotBytes) return cudaErrorInvalidValue;
        int s = next;
        next = (next + 1) % n_slots;
        if (pending[s]) {
            cudaError_t e = cudaEventSynchronize(ev[s]);
            if (e != cudaSuccess) return e;
            pending[s] = false;
        }
        char* h = host + (size_t)s * kSlotBytes;
        char* d = dev + (size_t)s * kSlotBytes;
        std::memcpy(h, src, bytes);
        cudaError_t e = cudaMemcpyAsync(d, h, bytes, cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) return e;
        e = cudaEventRecord(ev[s], stream);
        if (e != cudaSuccess) return e;
        pending[s] = true;
        *dev_out = d;
        return cudaSuccess;
    }
};

}  // namespace

struct skv_pool {
    skv_config cfg{};
    bool host_only = false;
    size_t esize = 2;
    size_t page_bytes = 0;          // one layer's K (or V) bytes of one page: heads * page_size * dim * esize
    size_t layer_stride = 0;        // bytes between layers inside the K (or V) allocation

    // host bookkeeping
    std::vector<int32_t> page_table;     // [max_seqs][max_pages_per_seq]
    std::vector<int32_t> n_seq_pages;    // [max_seqs]
    std::vector<int32_t> lengths;        // [num_layers][max_seqs]
    std::vector<uint8_t> live;           // [max_seqs]
    std::vector<int32_t> page_owner;     // [num_pages] owning sequence or -1
    std::vector<int32_t> free_pages, free_seqs, free_host;
    int64_t n_evicted = 0, n_prefetched = 0, bytes_d2h = 0, bytes_h2d = 0;

    // device state
    char* d_k = nullptr;
    char* d_v = nullptr;
    int32_t* d_page_table = nullptr;
    int32_t* d_lengths = nullptr;
    int32_t* d_status = nullptr;
    int32_t* d_tickets = nullptr;        // [max_seqs][num_kv_heads] + 2, zero between decode calls
    int32_t* d_stored_len = nullptr;     // [num_layers][max_seqs][num_kv_heads]: see DecodeLaunch::stored_len
    float* d_inv_freq = nullptr;
    // K and V pools as 2-D bf16 tensors [layers*pages*heads*page_size][head_dim] with [16][64] boxes
    alignas(64) CUtensorMap k_map;
    alignas(64) CUtensorMap v_map;
    bool has_maps = false;
    int sm_count = 148;                  // multiprocessors of the pool's device
    bool rope_set = false;
    float rope_scaling = 1.0f;
    StagingRing ring;                    // compute stream
    StagingRing ring_copy;               // copy stream

    // host tier
    char* h_tier = nullptr;              // pinned + mapped: [host_pages][num_layers][2][page_bytes]
    char* h_tier_dev = nullptr;          // device alias of h_tier
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t ev_compute = nullptr, ev_copy = nullptr;
    bool copy_pending = false;           // copies enqueued on copy_stream not yet ordered before compute
    std::vector<uint8_t> copy_busy;      // [max_seqs] 1: pages of this sequence are among those copies
    std::vector<int32_t> n_parked;       // [max_seqs] page-table entries of the sequence that point into the host tier:
                                         // the residency checks of the hot calls scan a row only when this is not 0
    std::vector<TableUpdate> deferred_updates;   // page-table entries to publish once prefetch copies are ordered

    // scratch of the one-call decode step, kept between calls so that a step allocates nothing on the host
    std::vector<TableUpdate> step_ups;
    std::vector<uint32_t> seen_stamp;            // [max_seqs] generation stamps for the duplicate check
    uint32_t stamp = 0;
    std::vector<int32_t> step_store;             // [n_seqs] 0/1: the row's token is stored by this pool
    StepRows rows{};
    // What this pool's last step wrote besides pages and partials (the rotated q rows, the output), on which stream,
    // and the library-wide launch count right after it: a following step may start early only when it comes
    // directly after it and reads none of that.
    bool last_step_valid = false;
    cudaStream_t last_step_stream = nullptr;
    long long last_step_mark = 0;
    // [num_layers][max_seqs]: the length a one-kernel step left behind when it stored the row's newest token, -1 once
    // anything else has changed the row.  A later step that may run beside that one waits for the device-side copy
    // (d_stored_len) only where this says that a step wrote it.
    std::vector<int32_t> step_len;
    const char* last_w_lo[2] = {nullptr, nullptr};
    const char* last_w_hi[2] = {nullptr, nullptr};

    std::string err;

    int32_t fail(int32_t code, const char* fmt, ...) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        err = buf;
        return code;
    }
    int32_t cuda_fail(cudaError_t e, const char* what) {
        return fail(SKV_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    }
    PoolView view() const {
        PoolView v;
        v.k_base = d_k;
        v.v_base = d_v;
        v.layer_stride_bytes = (int64_t)layer_stride;
        v.page_table = d_page_table;
        v.lengths = d_lengths;
        v.status = d_status;
        v.num_kv_heads = cfg.num_kv_heads;
        v.head_dim = cfg.head_dim;
        v.page_size = cfg.page_size;
        v.num_pages = cfg.num_pages;
        v.max_seqs = cfg.max_seqs;
        v.max_pages_per_seq = cfg.max_pages_per_seq;
        return v;
    }
    int32_t& pt(int32_t seq, int32_t slot) { return page_table[(size_t)seq * cfg.max_pages_per_seq + slot]; }
    int32_t& len(int32_t layer, int32_t seq) { return lengths[(size_t)layer * cfg.max_seqs + seq]; }
};

namespace {

#define CUDA_TRY(pool, call)                                   \
    do {                                                       \
        cudaError_t _e = (call);                               \
        if (_e != cudaSuccess) return (pool)->cuda_fail(_e, #call); \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    bool active = false;
    explicit DeviceGuard(const skv_pool* p) {
        if (!p->host_only && cudaGetDevice(&prev) == cudaSuccess && prev != p->cfg.device) {
            cudaSetDevice(p->cfg.device);
            active = true;
        }
    }
    ~DeviceGuard() {
        if (active) cudaSetDevice(prev);
    }
};

__global__ void apply_table_updates_kernel(int32_t* __restrict__ table, const TableUpdate* __restrict__ ups, int n,
                                           int max_seqs, int max_pages) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    TableUpdate u = ups[i];
    if (u.seq < 0 || u.seq >= max_seqs || u.slot < 0 || u.slot >= max_pages) return;
    table[(size_t)u.seq * max_pages + u.slot] = u.value;
}

struct LengthUpdate {
    int32_t index, value;
};
// Lengths set from the host (free, truncate, adopted page tables) may shrink a row: the per-head "stored length"
// words that steps publish are cleared with them, so that a stale larger value can never satisfy a later wait.
__global__ void apply_length_updates_kernel(int32_t* __restrict__ lengths, const LengthUpdate* __restrict__ ups, int n,
                                            int total, int32_t* __restrict__ stored_len, int heads) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    LengthUpdate u = ups[i];
    if (u.index >= 0 && u.index < total) {
        lengths[u.index] = u.value;
        for (int h = 0; h < heads; ++h) stored_len[(int64_t)u.index * heads + h] = 0;
    }
}

// 16-byte vector copy of whole pages between the device pools and the mapped host tier.
struct CopyItem {
    int32_t page, slot;
};
__global__ void __launch_bounds__(256) page_copy_kernel(char* __restrict__ k_base, char* __restrict__ v_base, char* __restrict__ tier,
                                                         const CopyItem* __restrict__ items, int n_items, int64_t layer_stride,
                                                         int64_t page_bytes, int num_layers, int to_host) {
    // One block moves several (layer, K|V) chunks of one page at a time; every thread keeps four 16-byte loads in
    // flight, which is what the host link needs (loads from mapped host memory are latency-bound otherwise).
    // The grid is small and strides over the pages: the link (about 52 GB/s measured, either direction) is
    // saturated by a few hundred blocks, and a grid that filled every SM would keep compute kernels from running
    // beside the copy.
    const int n = (int)(page_bytes / 16);
    const int n_chunks = num_layers * 2;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const CopyItem it = items[item];
    for (int c0 = blockIdx.y; c0 < n_chunks; c0 += 4 * gridDim.y) {
        const int4* src[4];
        int4* dst[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int chunk = c0 + u * gridDim.y;
            const int cc = chunk < n_chunks ? chunk : c0;
            const int layer = cc >> 1, is_v = cc & 1;
            char* dev = (is_v ? v_base : k_base) + (int64_t)layer * layer_stride + (int64_t)it.page * page_bytes;
            char* hst = tier + (((int64_t)it.slot * num_layers + layer) * 2 + is_v) * page_bytes;
            src[u] = reinterpret_cast<const int4*>(to_host ? dev : hst);
            dst[u] = reinterpret_cast<int4*>(to_host ? hst : dev);
        }
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            int4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = src[u][i];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (c0 + u * (int)gridDim.y < n_chunks) dst[u][i] = v[u];
        }
    }
    }
}

int32_t publish_table_updates(skv_pool* p, const std::vector<TableUpdate>& ups, cudaStream_t stream) {
    if (p->host_only || ups.empty()) return SKV_OK;
    const size_t per = StagingRing::kSlotBytes / sizeof(TableUpdate);
    for (size_t off = 0; off < ups.size(); off += per) {
        size_t n = std::min(per, ups.size() - off);
        void* dev = nullptr;
        CUDA_TRY(p, p->ring.upload(ups.data() + off, n * sizeof(TableUpdate), stream, &dev));
        apply_table_updates_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(
            p->d_page_table, (const TableUpdate*)dev, (int)n, p->cfg.max_seqs, p->cfg.max_pages_per_seq);
        CUDA_TRY(p, cudaGetLastError());
        count_launches(1);
    }
    return SKV_OK;
}

int32_t publish_length_updates(skv_pool* p, const std::vector<LengthUpdate>& ups, cudaStream_t stream) {
    if (p->host_only || ups.empty()) return SKV_OK;
    const size_t per = StagingRing::kSlotBytes / sizeof(LengthUpdate);
    for (size_t off = 0; off < ups.size(); off += per) {
        size_t n = std::min(per, ups.size() - off);
        void* dev = nullptr;
        CUDA_TRY(p, p->ring.upload(ups.data() + off, n * sizeof(LengthUpdate), stream, &dev));
        apply_length_updates_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(
            p->d_lengths, (const LengthUpdate*)dev, (int)n, p->cfg.num_layers * p->cfg.max_seqs, p->d_stored_len,
            p->cfg.num_kv_heads);
        CUDA_TRY(p, cudaGetLastError());
        count_launches(1);
    }
    return SKV_OK;
}

bool valid_seq(const skv_pool* p, int32_t seq) { return seq >= 0 && seq < p->cfg.max_seqs && p->live[seq]; }

// Orders everything enqueued on the copy stream before later work on `stream` and publishes
// page-table entries that were waiting for those copies.
int32_t order_transfers(skv_pool* p, cudaStream_t stream) {
    if (p->host_only) return SKV_OK;
    if (p->copy_pending) {
        CUDA_TRY(p, cudaEventRecord(p->ev_copy, p->copy_stream));
        CUDA_TRY(p, cudaStreamWaitEvent(stream, p->ev_copy, 0));
        p->copy_pending = false;
        std::fill(p->copy_busy.begin(), p->copy_busy.end(), (uint8_t)0);
    }
    if (!p->deferred_updates.empty()) {
        int32_t st = publish_table_updates(p, p->deferred_updates, stream);
        if (st != SKV_OK) return st;
        p->deferred_updates.clear();
    }
    return SKV_OK;
}

// A call that only reads (or appends inside pages it already owns) needs the pending copies ordered before it only
// when one of its sequences is among them: attention over other sequences runs beside an eviction or a copy back.
// A call that takes fresh pages always orders: a page freed by an eviction may still be read by its copy.
int32_t order_transfers_for(skv_pool* p, cudaStream_t stream, const int32_t* seq_ids, int32_t n_seqs, bool takes_pages) {
    if (p->host_only || !p->copy_pending) return order_transfers(p, stream);
    bool involved = takes_pages;
    for (int32_t i = 0; !involved && i < n_seqs; ++i) {
        const int32_t s = seq_ids ? seq_ids[i] : i;
        involved = s >= 0 && s < p->cfg.max_seqs && p->copy_busy[s];
    }
    return involved ? order_transfers(p, stream) : SKV_OK;
}

// Grows a sequence's page-table row to cover `total_tokens`; all-or-nothing.
int32_t grow(skv_pool* p, int32_t seq, int32_t total_tokens, std::vector<TableUpdate>* ups) {
    const int32_t P = p->cfg.page_size;
    int32_t need = (total_tokens + P - 1) / P;
    int32_t have = p->n_seq_pages[seq];
    if (need <= have) return SKV_OK;
    if (need > p->cfg.max_pages_per_seq)
        return p->fail(SKV_ERR_OUT_OF_PAGES, "sequence %d needs %d pages, row holds %d", seq, need,
                       p->cfg.max_pages_per_seq);
    if ((size_t)(need - have) > p->free_pages.size())
        return p->fail(SKV_ERR_OUT_OF_PAGES, "need %d pages, %zu free", need - have, p->free_pages.size());
    for (int32_t slot = have; slot < need; ++slot) {
        int32_t page = p->free_pages.back();
        p->free_pages.pop_back();
        p->pt(seq, slot) = page;
        p->page_owner[page] = seq;
        ups->push_back({seq, slot, page});
    }
    p->n_seq_pages[seq] = need;
    return SKV_OK;
}

}  // namespace

extern "C" {

int32_t skv_abi_version(void) { return SKV_ABI_VERSION; }

void skv_reload_env(void) { reload_switches(); }

int64_t skv_launch_count(void) { return (int64_t)g_launches.load(std::memory_order_relaxed); }

const char* skv_status_string(int32_t s) {
    switch (s) {
        case SKV_OK: return "ok";
        case SKV_ERR_BAD_ARG: return "bad argument";
        case SKV_ERR_REPLAY: return "append does not start exactly after the cached sequence";
        case SKV_ERR_OUT_OF_PAGES: return "out of pages";
        case SKV_ERR_NOT_RESIDENT: return "page not resident";
        case SKV_ERR_TIMEOUT: return "timeout";
        case SKV_ERR_CUDA: return "CUDA error";
        case SKV_ERR_UNSUPPORTED: return "unsupported shape or dtype";
        case SKV_ERR_DEVICE_FLAG: return "device status flag set";
        default: return "unknown status";
    }
}

const char* skv_last_error(const skv_pool* pool) { return pool ? pool->err.c_str() : "null pool"; }

int32_t skv_create(const skv_config* cfg, skv_pool** out) {
    if (!cfg || !out) return SKV_ERR_BAD_ARG;
    *out = nullptr;
    if (cfg->num_layers <= 0 || cfg->num_kv_heads <= 0 || cfg->head_dim <= 0 || cfg->page_size <= 0 ||
        cfg->num_pages <= 0 || cfg->max_seqs <= 0 || cfg->max_pages_per_seq <= 0 || cfg->host_pages < 0)
        return SKV_ERR_BAD_ARG;
    if (cfg->dtype != SKV_F32 && cfg->dtype != SKV_BF16) return SKV_ERR_BAD_ARG;
    if (cfg->head_dim % 2 != 0 || cfg->head_dim > 256) return SKV_ERR_UNSUPPORTED;
    skv_pool* p = new (std::nothrow) skv_pool();
    if (!p) return SKV_ERR_BAD_ARG;
    p->cfg = *cfg;
    if ((int64_t)cfg->max_pages_per_seq * cfg->page_size > SKV_MAX_TOKENS_PER_SEQ) {
        // the split-K plan gives one sequence at most 128 chunks of 2048 tokens (a warp keeps 32 tile page ids, the
        // merge kernel takes one chunk per thread); a longer row would make every decode call fail at launch
        *out = p;
        p->host_only = true;
        return p->fail(SKV_ERR_UNSUPPORTED, "max_pages_per_seq * page_size = %lld exceeds %d tokens per sequence",
                       (long long)cfg->max_pages_per_seq * cfg->page_size, SKV_MAX_TOKENS_PER_SEQ);
    }
    p->host_only = cfg->device < 0;
    p->esize = dtype_size(cfg->dtype);
    p->page_bytes = (size_t)cfg->num_kv_heads * cfg->page_size * cfg->head_dim * p->esize;
    p->layer_stride = p->page_bytes * (size_t)cfg->num_pages;
    p->page_table.assign((size_t)cfg->max_seqs * cfg->max_pages_per_seq, SKV_PAGE_UNASSIGNED);
    p->n_seq_pages.assign(cfg->max_seqs, 0);
    p->lengths.assign((size_t)cfg->num_layers * cfg->max_seqs, 0);
    p->live.assign(cfg->max_seqs, 0);
    p->page_owner.assign(cfg->num_pages, -1);
    p->seen_stamp.assign(cfg->max_seqs, 0);
    p->copy_busy.assign(cfg->max_seqs, 0);
    p->n_parked.assign(cfg->max_seqs, 0);
    p->step_len.assign((size_t)cfg->num_layers * cfg->max_seqs, -1);
    for (int32_t i = cfg->num_pages - 1; i >= 0; --i) p->free_pages.push_back(i);
    for (int32_t i = cfg->max_seqs - 1; i >= 0; --i) p->free_seqs.push_back(i);
    for (int32_t i = cfg->host_pages - 1; i >= 0; --i) p->free_host.push_back(i);
    *out = p;
    if (p->host_only) return SKV_OK;

    int32_t st = [&]() -> int32_t {
        DeviceGuard g(p);
        CUDA_TRY(p, cudaSetDevice(cfg->device));
        size_t total = p->layer_stride * (size_t)cfg->num_layers;
        CUDA_TRY(p, cudaMalloc((void**)&p->d_k, total));
        CUDA_TRY(p, cudaMalloc((void**)&p->d_v, total));
        CUDA_TRY(p, cudaMemset(p->d_k, 0, total));
        CUDA_TRY(p, cudaMemset(p->d_v, 0, total));
        CUDA_TRY(p, cudaMalloc((void**)&p->d_page_table, p->page_table.size() * sizeof(int32_t)));
        CUDA_TRY(p, cudaMemset(p->d_page_table, 0xFF, p->page_table.size() * sizeof(int32_t)));
        CUDA_TRY(p, cudaMalloc((void**)&p->d_lengths, p->lengths.size() * sizeof(int32_t)));
        CUDA_TRY(p, cudaMemset(p->d_lengths, 0, p->lengths.size() * sizeof(int32_t)));
        CUDA_TRY(p, cudaMalloc((void**)&p->d_status, sizeof(int32_t)));
        CUDA_TRY(p, cudaMemset(p->d_status, 0, sizeof(int32_t)));
        CUDA_TRY(p, cudaMalloc((void**)&p->d_tickets, ((size_t)cfg->max_seqs * cfg->num_kv_heads + 2) * sizeof(int32_t)));
        CUDA_TRY(p, cudaMemset(p->d_tickets, 0, ((size_t)cfg->max_seqs * cfg->num_kv_heads + 2) * sizeof(int32_t)));
        const size_t n_flags = (size_t)cfg->num_layers * cfg->max_seqs * cfg->num_kv_heads;
        CUDA_TRY(p, cudaMalloc((void**)&p->d_stored_len, n_flags * sizeof(int32_t)));
        CUDA_TRY(p, cudaMemset(p->d_stored_len, 0, n_flags * sizeof(int32_t)));
        CUDA_TRY(p, cudaMalloc((void**)&p->d_inv_freq, (size_t)cfg->head_dim / 2 * sizeof(float)));
        CUDA_TRY(p, p->ring.init());
        CUDA_TRY(p, p->ring_copy.init(16));
        CUDA_TRY(p, cudaStreamCreateWithFlags(&p->copy_stream, cudaStreamNonBlocking));
        CUDA_TRY(p, cudaEventCreateWithFlags(&p->ev_compute, cudaEventDisableTiming));
        CUDA_TRY(p, cudaEventCreateWithFlags(&p->ev_copy, cudaEventDisableTiming));
        if (cfg->host_pages > 0) {
            if (p->page_bytes % 16 != 0)
                return p->fail(SKV_ERR_UNSUPPORTED, "host tier needs page bytes to be a multiple of 16");
            size_t bytes = (size_t)cfg->host_pages * cfg->num_layers * 2 * p->page_bytes;
            CUDA_TRY(p, cudaHostAlloc((void**)&p->h_tier, bytes, cudaHostAllocMapped | cudaHostAllocPortable));
            CUDA_TRY(p, cudaHostGetDevicePointer((void**)&p->h_tier_dev, p->h_tier, 0));
        }
        {
            int sms = 0;
            if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, cfg->device) == cudaSuccess && sms > 0) p->sm_count = sms;
        }
        if (cfg->dtype == SKV_BF16 && cfg->head_dim == 128 && cfg->page_size % 16 == 0) {
            const uint64_t rows = (uint64_t)cfg->num_layers * cfg->num_pages * cfg->num_kv_heads * cfg->page_size;
            if (rows < (1ull << 31))
                p->has_maps = encode_bf16_2d(&p->k_map, p->d_k, rows, 128, 256, 16, 64) &&
                              encode_bf16_2d(&p->v_map, p->d_v, rows, 128, 256, 16, 64);
        }
        CUDA_TRY(p, cudaDeviceSynchronize());
        return SKV_OK;
    }();
    return st;   // on failure the caller still owns *out and may read skv_last_error before skv_destroy
}

int32_t skv_destroy(skv_pool* p) {
    if (!p) return SKV_OK;
    if (!p->host_only) {
        DeviceGuard g(p);
        cudaDeviceSynchronize();
        p->ring.destroy();
        p->ring_copy.destroy();
        if (p->copy_stream) cudaStreamDestroy(p->copy_stream);
        if (p->ev_compute) cudaEventDestroy(p->ev_compute);
        if (p->ev_copy) cudaEventDestroy(p->ev_copy);
        if (p->h_tier) cudaFreeHost(p->h_tier);
        cudaFree(p->d_k);
        cudaFree(p->d_v);
        cudaFree(p->d_page_table);
        cudaFree(p->d_lengths);
        cudaFree(p->d_status);
        cudaFree(p->d_tickets);
        cudaFree(p->d_stored_len);
        cudaFree(p->d_inv_freq);
    }
    delete p;
    return SKV_OK;
}

int32_t skv_alloc_sequence(skv_pool* p, int32_t* seq_out) {
    if (!p || !seq_out) return SKV_ERR_BAD_ARG;
    if (p->free_seqs.empty()) return p->fail(SKV_ERR_OUT_OF_PAGES, "no free sequence id (max_seqs %d)", p->cfg.max_seqs);
    int32_t s = p->free_seqs.back();
    p->free_seqs.pop_back();
    p->live[s] = 1;
    *seq_out = s;
    return SKV_OK;
}

int32_t skv_free_sequence(skv_pool* p, int32_t seq, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!p) return SKV_ERR_BAD_ARG;
    if (!valid_seq(p, seq)) return p->fail(SKV_ERR_BAD_ARG, "sequence %d is not live", seq);
    std::vector<TableUpdate> ups;
    std::vector<LengthUpdate> lups;
    for (int32_t slot = p->n_seq_pages[seq] - 1; slot >= 0; --slot) {
        int32_t e = p->pt(seq, slot);
        if (e >= 0) {
            p->free_pages.push_back(e);
            p->page_owner[e] = -1;
        } else if (e <= -2) {
            p->free_host.push_back(-2 - e);
        }
        p->pt(seq, slot) = SKV_PAGE_UNASSIGNED;
        ups.push_back({seq, slot, SKV_PAGE_UNASSIGNED});
    }
    p->n_seq_pages[seq] = 0;
    p->n_parked[seq] = 0;
    for (int32_t l = 0; l < p->cfg.num_layers; ++l) {
        p->len(l, seq) = 0;
        p->step_len[(size_t)l * p->cfg.max_seqs + seq] = -1;
        lups.push_back({l * p->cfg.max_seqs + seq, 0});
    }
    p->live[seq] = 0;
    p->free_seqs.push_back(seq);
    // drop deferred entries of this sequence
    p->deferred_updates.erase(std::remove_if(p->deferred_updates.begin(), p->deferred_updates.end(),
                                             [&](const TableUpdate& u) { return u.seq == seq; }),
                              p->deferred_updates.end());
    DeviceGuard g(p);
    int32_t st = publish_table_updates(p, ups, stream);
    if (st != SKV_OK) return st;
    return publish_length_updates(p, lups, stream);
}

int32_t skv_reserve(skv_pool* p, int32_t seq, int32_t total_tokens, void* stream_) {
    if (!p) return SKV_ERR_BAD_ARG;
    if (!valid_seq(p, seq)) return p->fail(SKV_ERR_BAD_ARG, "sequence %d is not live", seq);
    if (total_tokens < 0) return p->fail(SKV_ERR_BAD_ARG, "total_tokens must be non-negative");
    std::vector<TableUpdate> ups;
    int32_t st = grow(p, seq, total_tokens, &ups);
    if (st != SKV_OK) return st;
    DeviceGuard g(p);
    return publish_table_updates(p, ups, (cudaStream_t)stream_);
}

int32_t skv_set_page_table(skv_pool* p, int32_t seq, const int32_t* pages, int32_t n_pages, int32_t length, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!p || (!pages && n_pages > 0)) return SKV_ERR_BAD_ARG;
    if (!valid_seq(p, seq)) return p->fail(SKV_ERR_BAD_ARG, "sequence %d is not live", seq);
    if (n_pages < 0 || n_pages > p->cfg.max_pages_per_seq)
        return p->fail(SKV_ERR_BAD_ARG, "n_pages %d outside [0, %d]", n_pages, p->cfg.max_pages_per_seq);
    if (length < 0 || (int64_t)length > (int64_t)n_pages * p->cfg.page_size)
        return p->fail(SKV_ERR_BAD_ARG, "length %d does not fit %d pages", length, n_pages);
    if (p->n_seq_pages[seq] != 0) return p->fail(SKV_ERR_BAD_ARG, "sequence %d already owns pages", seq);
    // validate: in range, owned by nobody, no duplicates
    std::vector<int32_t> sorted(pages, pages + n_pages);
    std::sort(sorted.begin(), sorted.end());
    for (int32_t i = 0; i < n_pages; ++i) {
        int32_t pg = sorted[i];
        if (pg < 0 || pg >= p->cfg.num_pages) return p->fail(SKV_ERR_BAD_ARG, "page id %d outside the pool", pg);
        if (i > 0 && sorted[i - 1] == pg) return p->fail(SKV_ERR_BAD_ARG, "page id %d listed twice", pg);
        if (p->page_owner[pg] != -1) return p->fail(SKV_ERR_BAD_ARG, "page id %d belongs to sequence %d", pg, p->page_owner[pg]);
    }
    // take the pages out of the free stack, keeping the order of the rest
    std::vector<uint8_t> taken(p->cfg.num_pages, 0);
    for (int32_t i = 0; i < n_pages; ++i) taken[pages[i]] = 1;
    p->free_pages.erase(std::remove_if(p->free_pages.begin(), p->free_pages.end(), [&](int32_t pg) { return taken[pg] != 0; }),
                        p->free_pages.end());
    std::vector<TableUpdate> ups;
    std::vector<LengthUpdate> lups;
    for (int32_t i = 0; i < n_pages; ++i) {
        p->pt(seq, i) = pages[i];
        p->page_owner[pages[i]] = seq;
        ups.push_back({seq, i, pages[i]});
    }
    p->n_seq_pages[seq] = n_pages;
    for (int32_t l = 0; l < p->cfg.num_layers; ++l) {
        p->len(l, seq) = length;
        p->step_len[(size_t)l * p->cfg.max_seqs + seq] = -1;
        lups.push_back({l * p->cfg.max_seqs + seq, length});
    }
    DeviceGuard g(p);
    int32_t st = publish_table_updates(p, ups, stream);
    if (st != SKV_OK) return st;
    return publish_length_updates(p, lups, stream);
}

int32_t skv_truncate(skv_pool* p, int32_t layer, const int32_t* seq_ids, int32_t n_seqs, int32_t new_length, void* stream_) {
    if (!p) return SKV_ERR_BAD_ARG;
    if (layer < 0) return p->fail(SKV_ERR_BAD_ARG, "layer_idx must be a non-negative integer");
    if (layer >= p->cfg.num_layers)
        return p->fail(SKV_ERR_BAD_ARG, "layer_idx %d is outside configured layer count %d", layer, p->cfg.num_layers);
    if (n_seqs <= 0 || n_seqs > p->cfg.max_seqs || new_length < 0) return p->fail(SKV_ERR_BAD_ARG, "n_seqs %d / new_length %d out of range", n_seqs, new_length);
    for (int32_t i = 0; i < n_seqs; ++i) {
        int32_t s = seq_ids ? seq_ids[i] : i;
        if (!valid_seq(p, s)) return p->fail(SKV_ERR_BAD_ARG, "sequence %d is not live", s);
        if (new_length > p->len(layer, s)) return p->fail(SKV_ERR_BAD_ARG, "new_length %d exceeds sequence %d's length %d", new_length, s, p->len(layer, s));
    }
    std::vector<LengthUpdate> lups;
    for (int32_t i = 0; i < n_seqs; ++i) {
        int32_t s = seq_ids ? seq_ids[i] : i;
        p->len(layer, s) = new_length;
        p->step_len[(size_t)layer * p->cfg.max_seqs + s] = -1;
        lups.push_back({layer * p->cfg.max_seqs + s, new_length});
    }
    DeviceGuard g(p);
    return publish_length_updates(p, lups, (cudaStream_t)stream_);
}

int32_t skv_length(const skv_pool* p, int32_t layer, int32_t seq, int32_t* out) {
    if (!p || !out) return SKV_ERR_BAD_ARG;
    if (layer < 0 || layer >= p->cfg.num_layers || seq < 0 || seq >= p->cfg.max_seqs) return SKV_ERR_BAD_ARG;
    *out = p->lengths[(size_t)layer * p->cfg.max_seqs + seq];
    return SKV_OK;
}

int32_t skv_lengths(const skv_pool* p, int32_t layer, int32_t* out, int32_t n) {
    if (!p || !out || layer < 0 || layer >= p->cfg.num_layers || n < 0 || n > p->cfg.max_seqs) return SKV_ERR_BAD_ARG;
    std::memcpy(out, p->lengths.data() + (size_t)layer * p->cfg.max_seqs, (size_t)n * sizeof(int32_t));
    return SKV_OK;
}

int32_t skv_page_table(const skv_pool* p, int32_t seq, int32_t* out, int32_t capacity, int32_t* n_out) {
    if (!p || seq < 0 || seq >= p->cfg.max_seqs) return SKV_ERR_BAD_ARG;
    int32_t n = p->n_seq_pages[seq];
    if (n_out) *n_out = n;
    if (out) {
        if (capacity < n) return SKV_ERR_BAD_ARG;
        std::memcpy(out, p->page_table.data() + (size_t)seq * p->cfg.max_pages_per_seq, (size_t)n * sizeof(int32_t));
    }
    return SKV_OK;
}

int32_t skv_pool_counters(const skv_pool* p, int64_t out[8]) {
    if (!p || !out) return SKV_ERR_BAD_ARG;
    out[0] = (int64_t)p->free_pages.size();
    out[1] = (int64_t)p->cfg.num_pages - out[0];
    out[2] = (int64_t)p->free_host.size();
    out[3] = p->n_evicted;
    out[4] = p->n_prefetched;
    out[5] = p->bytes_d2h;
    out[6] = p->bytes_h2d;
    int64_t n = 0;
    for (uint8_t l : p->live) n += l;
    out[7] = n;
    return SKV_OK;
}

int32_t skv_pool_pointers(const skv_pool* p, int32_t layer, void** k, void** v) {
    if (!p || layer < 0 || layer >= p->cfg.num_layers) return SKV_ERR_BAD_ARG;
    if (k) *k = p->d_k ? p->d_k + (size_t)layer * p->layer_stride : nullptr;
    if (v) *v = p->d_v ? p->d_v + (size_t)layer * p->layer_stride : nullptr;
    return SKV_OK;
}

int32_t skv_device_tables(const skv_pool* p, int32_t** page_table, int32_t** lengths) {
    if (!p) return SKV_ERR_BAD_ARG;
    if (page_table) *page_table = p->d_page_table;
    if (lengths) *lengths = p->d_lengths;
    return SKV_OK;
}

int32_t skv_set_rope(skv_pool* p, const float* inv_freq, int32_t n, float scaling) {
    if (!p || !inv_freq) return SKV_ERR_BAD_ARG;
    if (n != p->cfg.head_dim / 2) return p->fail(SKV_ERR_BAD_ARG, "inv_freq has %d entries, head_dim/2 is %d", n, p->cfg.head_dim / 2);
    if (!(scaling > 0.0f)) return p->fail(SKV_ERR_BAD_ARG, "scaling_factor must be positive");
    p->rope_scaling = scaling;
    p->rope_set = true;
    if (p->host_only) return SKV_OK;
    DeviceGuard g(p);
    CUDA_TRY(p, cudaMemcpy(p->d_inv_freq, inv_freq, (size_t)n * sizeof(float), cudaMemcpyHostToDevice));
    return SKV_OK;
}

int32_t skv_append(skv_pool* p, const skv_append_args* a, void* stream_) {
    if (!p || !a) return SKV_ERR_BAD_ARG;
    cudaStream_t stream = (cudaStream_t)stream_;
    // -- validation, in the reference's order (mlx_kvcache.py:85-104) --
    if (a->layer < 0) return p->fail(SKV_ERR_BAD_ARG, "layer_idx must be a non-negative integer");
    if (a->layer >= p->cfg.num_layers)
        return p->fail(SKV_ERR_BAD_ARG, "layer_idx %d is outside configured layer count %d", a->layer, p->cfg.num_layers);
    if (a->n_seqs <= 0 || a->n_seqs > p->cfg.max_seqs || a->n_new < 0)
        return p->fail(SKV_ERR_BAD_ARG, "n_seqs %d / n_new %d out of range", a->n_seqs, a->n_new);
    if (!p->host_only && a->n_new > 0 && (!a->k || !a->v)) return p->fail(SKV_ERR_BAD_ARG, "k and v must be given");
    if ((a->rope_k || a->q_in) && !p->rope_set) return p->fail(SKV_ERR_BAD_ARG, "RoPE requested but skv_set_rope was not called");
    if (a->q_in && (!a->q_out || a->n_q_heads <= 0)) return p->fail(SKV_ERR_BAD_ARG, "q_out and n_q_heads must accompany q_in");
    std::vector<AppendMeta> meta(a->n_seqs);
    std::vector<uint8_t> seen(p->cfg.max_seqs, 0);
    for (int32_t i = 0; i < a->n_seqs; ++i) {
        int32_t s = a->seq_ids ? a->seq_ids[i] : i;
        if (!valid_seq(p, s)) return p->fail(SKV_ERR_BAD_ARG, "sequence %d is not live", s);
        if (seen[s]) return p->fail(SKV_ERR_BAD_ARG, "sequence %d listed twice", s);
        seen[s] = 1;
        int32_t cur = p->len(a->layer, s);
        int32_t start = a->start_pos ? a->start_pos[i] : cur;
        if (start != cur)
            return p->fail(SKV_ERR_REPLAY,
                           "cache_position must append exactly after the cached sequence; sequence %d layer %d expected start %d, got %d",
                           s, a->layer, cur, start);
        meta[i] = {s, start};
    }
    if (a->n_new == 0) return SKV_OK;
    // -- page allocation: all-or-nothing across the batch --
    {
        int64_t need_total = 0;
        const int32_t P = p->cfg.page_size;
        for (int32_t i = 0; i < a->n_seqs; ++i) {
            int32_t need = (meta[i].start + a->n_new + P - 1) / P;
            if (need > p->cfg.max_pages_per_seq)
                return p->fail(SKV_ERR_OUT_OF_PAGES, "sequence %d needs %d pages, row holds %d", meta[i].seq, need, p->cfg.max_pages_per_seq);
            need_total += std::max(0, need - p->n_seq_pages[meta[i].seq]);
        }
        if (need_total > (int64_t)p->free_pages.size())
            return p->fail(SKV_ERR_OUT_OF_PAGES, "need %lld pages, %zu free", (long long)need_total, p->free_pages.size());
    }
    // target pages must be resident
    for (int32_t i = 0; i < a->n_seqs; ++i) {
        int32_t first = meta[i].start / p->cfg.page_size;
        for (int32_t slot = first; p->n_parked[meta[i].seq] > 0 && slot < p->n_seq_pages[meta[i].seq]; ++slot)
            if (p->pt(meta[i].seq, slot) < 0)
                return p->fail(SKV_ERR_NOT_RESIDENT, "sequence %d slot %d is not resident", meta[i].seq, slot);
    }
    std::vector<TableUpdate> ups;
    for (int32_t i = 0; i < a->n_seqs; ++i) {
        int32_t st = grow(p, meta[i].seq, meta[i].start + a->n_new, &ups);
        if (st != SKV_OK) return st;   // cannot happen after the check above
    }
    for (int32_t i = 0; i < a->n_seqs; ++i) {
        p->len(a->layer, meta[i].seq) = meta[i].start + a->n_new;
        p->step_len[(size_t)a->layer * p->cfg.max_seqs + meta[i].seq] = -1;
    }
    if (p->host_only) return SKV_OK;

    DeviceGuard g(p);
    int32_t st = order_transfers(p, stream);
    if (st != SKV_OK) return st;
    st = publish_table_updates(p, ups, stream);
    if (st != SKV_OK) return st;
    AppendLaunch L{};
    L.pool = p->view();
    L.layer = a->layer;
    L.n_seqs = a->n_seqs;
    L.n_new = a->n_new;
    L.dtype = p->cfg.dtype;
    L.k = a->k;
    L.v = a->v;
    L.kv_stride_seq = a->kv_stride_seq;
    L.kv_stride_head = a->kv_stride_head;
    L.kv_stride_tok = a->kv_stride_tok;
    L.rope_k = a->rope_k;
    L.q_in = a->q_in;
    L.q_out = a->q_out;
    L.n_q_heads = a->q_in ? a->n_q_heads : 0;
    L.q_stride_seq = a->q_stride_seq;
    L.q_stride_head = a->q_stride_head;
    L.q_stride_tok = a->q_stride_tok;
    L.inv_freq = p->d_inv_freq;
    L.scaling = p->rope_scaling;
    const size_t per = StagingRing::kSlotBytes / sizeof(AppendMeta);
    for (size_t off = 0; off < meta.size(); off += per) {
        size_t n = std::min(per, meta.size() - off);
        void* dev = nullptr;
        CUDA_TRY(p, p->ring.upload(meta.data() + off, n * sizeof(AppendMeta), stream, &dev));
        L.meta = (const AppendMeta*)dev;
        L.n_seqs = (int32_t)n;
        // advance the tensor pointers to the first sequence of this slice
        L.k = (const char*)a->k + (int64_t)off * a->kv_stride_seq * (int64_t)p->esize;
        L.v = (const char*)a->v + (int64_t)off * a->kv_stride_seq * (int64_t)p->esize;
        if (a->q_in) {
            L.q_in = (const char*)a->q_in + (int64_t)off * a->q_stride_seq * (int64_t)p->esize;
            L.q_out = (char*)a->q_out + (int64_t)off * a->q_stride_seq * (int64_t)p->esize;
        }
        CUDA_TRY(p, launch_append(L, stream));
    }
    return SKV_OK;
}

static int32_t upload_ids(skv_pool* p, const int32_t* ids, int32_t n, cudaStream_t stream, const int32_t** dev_out) {
    *dev_out = nullptr;
    if (!ids) return SKV_OK;
    if ((size_t)n * sizeof(int32_t) > StagingRing::kSlotBytes) return p->fail(SKV_ERR_BAD_ARG, "too many entries (%d) for one call", n);
    void* dev = nullptr;
    CUDA_TRY(p, p->ring.upload(ids, (size_t)n * sizeof(int32_t), stream, &dev));
    *dev_out = (const int32_t*)dev;
    return SKV_OK;
}

// Validates a list of sequences for a read over the first `upto[i]` tokens (or the whole length).
static int32_t check_readable(skv_pool* p, int32_t layer, const int32_t* seq_ids, int32_t n_seqs, const int32_t* upto) {
    if (layer < 0) return p->fail(SKV_ERR_BAD_ARG, "layer_idx must be a non-negative integer");
    if (layer >= p->cfg.num_layers)
        return p->fail(SKV_ERR_BAD_ARG, "layer_idx %d is outside configured layer count %d", layer, p->cfg.num_layers);
    if (n_seqs <= 0 || n_seqs > p->cfg.max_seqs) return p->fail(SKV_ERR_BAD_ARG, "n_seqs %d out of range", n_seqs);
    for (int32_t i = 0; i < n_seqs; ++i) {
        int32_t s = seq_ids ? seq_ids[i] : i;
        if (!valid_seq(p, s)) return p->fail(SKV_ERR_BAD_ARG, "sequence %d is not live", s);
        int32_t T = p->len(layer, s);
        if (upto) T = std::min(T, upto[i]);
        int32_t pages = (T + p->cfg.page_size - 1) / p->cfg.page_size;
        for (int32_t slot = 0; p->n_parked[s] > 0 && slot < pages; ++slot)
            if (p->pt(s, slot) < 0) return p->fail(SKV_ERR_NOT_RESIDENT, "sequence %d slot %d is not resident", s, slot);
    }
    return SKV_OK;
}

int32_t skv_gather(skv_pool* p, int32_t layer, const int32_t* seq_ids, int32_t n_seqs, void* out_k, void* out_v,
                   int32_t max_len, void* stream_) {
    if (!p) return SKV_ERR_BAD_ARG;
    cudaStream_t stream = (cudaStream_t)stream_;
    int32_t st = check_readable(p, layer, seq_ids, n_seqs, nullptr);
    if (st != SKV_OK) return st;
    if (max_len < 0) return p->fail(SKV_ERR_BAD_ARG, "max_len must be non-negative");
    for (int32_t i = 0; i < n_seqs; ++i)
        if (p->len(layer, seq_ids ? seq_ids[i] : i) > max_len)
            return p->fail(SKV_ERR_BAD_ARG, "max_len %d is shorter than a sequence", max_len);
    if (p->host_only || max_len == 0) return SKV_OK;
    if (!out_k || !out_v) return p->fail(SKV_ERR_BAD_ARG, "output pointers must be given");
    DeviceGuard g(p);
    st = order_transfers(p, stream);
    if (st != SKV_OK) return st;
    GatherLaunch G{};
    G.pool = p->view();
    G.layer = layer;
    G.n_seqs = n_seqs;
    G.max_len = max_len;
    G.dtype = p->cfg.dtype;
    st = upload_ids(p, seq_ids, n_seqs, stream, &G.seq_ids);
    if (st != SKV_OK) return st;
    G.out_k = out_k;
    G.out_v = out_v;
    CUDA_TRY(p, launch_gather(G, stream));
    return SKV_OK;
}

}  // extern "C"

namespace skv {

int32_t pool_fail(skv_pool* p, int32_t code, const char* message) { return p->fail(code, "%s", message); }
int32_t pool_device(const skv_pool* p) { return p->cfg.device; }

int32_t prepare_decode(skv_pool* p, int32_t layer, const int32_t* seq_ids, int32_t n_seqs, const int32_t* q_pos,
                       int32_t n_q_heads, const void* q, void* out, float eps, cudaStream_t stream, DecodeLaunch* d,
                       int64_t* total_tokens, int32_t* launchable) {
    *launchable = 0;
    *total_tokens = 0;
    if (n_q_heads <= 0 || n_q_heads % p->cfg.num_kv_heads != 0)
        return p->fail(SKV_ERR_BAD_ARG, "query heads must be divisible by key/value heads");
    if (layer < 0) return p->fail(SKV_ERR_BAD_ARG, "layer_idx must be a non-negative integer");
    if (layer >= p->cfg.num_layers)
        return p->fail(SKV_ERR_BAD_ARG, "layer_idx %d is outside configured layer count %d", layer, p->cfg.num_layers);
    if (n_seqs <= 0 || n_seqs > p->cfg.max_seqs) return p->fail(SKV_ERR_BAD_ARG, "n_seqs %d out of range", n_seqs);
    if ((size_t)n_seqs * sizeof(int32_t) > StagingRing::kSlotBytes)
        return p->fail(SKV_ERR_BAD_ARG, "too many sequences (%d) for one call", n_seqs);
    for (int32_t i = 0; i < n_seqs; ++i) {
        const int32_t s = seq_ids ? seq_ids[i] : i;
        if (!valid_seq(p, s)) return p->fail(SKV_ERR_BAD_ARG, "sequence %d is not live", s);
        int32_t T = p->len(layer, s);
        *total_tokens += T;
        d->longest = i == 0 ? T : std::max(d->longest, T);
        if (q_pos) T = std::min(T, std::max(0, q_pos[i] + 1));
        const int32_t pages = (T + p->cfg.page_size - 1) / p->cfg.page_size;
        for (int32_t slot = 0; p->n_parked[s] > 0 && slot < pages; ++slot)
            if (p->pt(s, slot) < 0) return p->fail(SKV_ERR_NOT_RESIDENT, "sequence %d slot %d is not resident", s, slot);
    }
    if (p->host_only) return SKV_OK;
    if (!q || !out) return p->fail(SKV_ERR_BAD_ARG, "q and out must be given");
    int32_t st = order_transfers_for(p, stream, seq_ids, n_seqs, false);
    if (st != SKV_OK) return st;
    p->last_step_valid = false;
    d->pool = p->view();
    d->layer = layer;
    d->n_seqs = n_seqs;
    d->n_q_heads = n_q_heads;
    d->dtype = p->cfg.dtype;
    st = upload_ids(p, seq_ids, n_seqs, stream, &d->seq_ids);
    if (st != SKV_OK) return st;
    st = upload_ids(p, q_pos, n_seqs, stream, &d->q_pos);
    if (st != SKV_OK) return st;
    d->q = q;
    d->out = out;
    d->q_stride = d->out_stride = (int64_t)n_q_heads * p->cfg.head_dim;
    d->eps = eps;
    d->force_generic = switches().decode_generic;
    d->k_map = p->has_maps ? &p->k_map : nullptr;
    d->v_map = p->has_maps ? &p->v_map : nullptr;
    d->tickets = p->d_tickets;
    *launchable = 1;
    return SKV_OK;
}

}  // namespace skv

namespace {

// 16-byte words of one parity half of an exchange buffer (see ExchangeView).
size_t exchange_words(int32_t mode, int32_t world, int64_t n_rows, int32_t head_dim, size_t esize) {
    const size_t W = (size_t)head_dim * esize / 8;
    if (mode == SKV_XCHG_HEAD_GATHER) return (size_t)world * n_rows * W;
    const size_t Wp = ((size_t)head_dim + 2) / 2;
    const size_t rows_owned = ((size_t)n_rows + world - 1) / world;
    return (size_t)world * rows_owned * Wp + (size_t)n_rows * W;
}

int32_t fill_exchange(skv_pool* p, const skv_exchange* x, int32_t n_seqs, int32_t n_q_heads, ExchangeView* v) {
    if (x->mode != SKV_XCHG_HEAD_GATHER && x->mode != SKV_XCHG_SEQ_MERGE)
        return p->fail(SKV_ERR_BAD_ARG, "exchange mode %d is neither head gather nor sequence merge", x->mode);
    if (x->world < 1 || x->world > 8 || x->rank < 0 || x->rank >= x->world || !x->recv_ptrs || !x->out)
        return p->fail(SKV_ERR_BAD_ARG, "exchange needs 1 <= world <= 8, a rank inside it, the receive pointers and out");
    if (x->epoch == 0) return p->fail(SKV_ERR_BAD_ARG, "exchange epochs start at 1");
    if (((size_t)p->cfg.head_dim * p->esize) % 8 != 0)
        return p->fail(SKV_ERR_UNSUPPORTED, "the exchange needs head_dim * element size to be a multiple of 8 bytes");
    if ((uintptr_t)x->out % 16 != 0) return p->fail(SKV_ERR_BAD_ARG, "exchange out must be 16-byte aligned");
    const size_t half = exchange_words(x->mode, x->world, (int64_t)n_seqs * n_q_heads, p->cfg.head_dim, p->esize) * 16;
    v->mode = x->mode;
    v->world = x->world;
    v->rank = x->rank;
    v->epoch = x->epoch;
    v->out = x->out;
    for (int32_t r = 0; r < x->world; ++r) {
        if (!x->recv_ptrs[r] || (uintptr_t)x->recv_ptrs[r] % 16 != 0)
            return p->fail(SKV_ERR_BAD_ARG, "receive pointer %d is null or not 16-byte aligned", r);
        v->recv[r] = (char*)x->recv_ptrs[r] + (size_t)(x->epoch & 1u) * half;
    }
    return SKV_OK;
}

int32_t check_workspace(skv_pool* p, const void* workspace, size_t workspace_bytes, size_t need) {
    if (!workspace || workspace_bytes < need)
        return p->fail(SKV_ERR_BAD_ARG, "workspace holds %zu bytes, %zu needed", workspace_bytes, need);
    if ((uintptr_t)workspace % 16 != 0) return p->fail(SKV_ERR_BAD_ARG, "workspace must be 16-byte aligned");
    return SKV_OK;
}

// Decode attention over what the pool holds: the shared body of skv_decode_attn, skv_decode_attn_xchg and
// skv_decode_partial, and the second half of a step that cannot take the one-kernel form.
int32_t attn_impl(skv_pool* p, int32_t layer, const int32_t* seq_ids, int32_t n_seqs, const void* q, int64_t q_stride,
                  void* out, int64_t out_stride, const int32_t* q_pos, int32_t n_q_heads, float eps, void* workspace,
                  size_t workspace_bytes, const skv_exchange* xchg, float* partial_out, cudaStream_t stream) {
    // a misaligned workspace is refused whatever else the call would do (the merge kernel reads it with 8- and
    // 16-byte loads), bookkeeping-only pools included
    if (workspace && (uintptr_t)workspace % 16 != 0) return p->fail(SKV_ERR_BAD_ARG, "workspace must be 16-byte aligned");
    DeviceGuard guard(p);
    DecodeLaunch D{};
    int64_t total = 0;
    int32_t launchable = 0;
    // `q` doubles as the non-null output argument of the shared front half when the result goes elsewhere
    void* out_arg = out ? out : const_cast<void*>(q);
    if (!p->host_only && !out && !xchg && !partial_out) return p->fail(SKV_ERR_BAD_ARG, "q and out must be given");
    if (!p->host_only) {   // argument checks that must not depend on what the front half enqueues
        if (n_q_heads > 0 && n_seqs > 0 && n_seqs <= p->cfg.max_seqs) {
            int32_t chunk = 0, splits = 0;
            decode_plan(p->cfg.page_size, p->cfg.max_pages_per_seq, n_seqs, p->cfg.num_kv_heads, 0, 0, &chunk, &splits);
            const size_t least = (size_t)n_seqs * n_q_heads * 1 * ((size_t)p->cfg.head_dim + 2) * sizeof(float);
            int32_t st0 = check_workspace(p, workspace, workspace_bytes, least);
            if (st0 != SKV_OK) return st0;
        }
    }
    int32_t st = prepare_decode(p, layer, seq_ids, n_seqs, q_pos, n_q_heads, q, out_arg, eps, stream, &D, &total, &launchable);
    if (st != SKV_OK || !launchable) return st;
    decode_plan(p->cfg.page_size, p->cfg.max_pages_per_seq, n_seqs, p->cfg.num_kv_heads, total, D.longest, &D.chunk_tokens, &D.max_splits);
    D.grid_splits = std::max(1, (D.longest + D.chunk_tokens - 1) / D.chunk_tokens);
    const size_t need = (size_t)n_seqs * n_q_heads * D.max_splits * ((size_t)p->cfg.head_dim + 2) * sizeof(float);
    st = check_workspace(p, workspace, workspace_bytes, need);
    if (st != SKV_OK) return st;
    D.ws_acc = (float*)workspace;
    D.ws_ml = D.ws_acc + (size_t)n_seqs * n_q_heads * D.max_splits * p->cfg.head_dim;
    D.total_tokens = total;
    D.out = out;
    if (q_stride) D.q_stride = q_stride;
    if (out_stride) D.out_stride = out_stride;
    D.partial_out = partial_out;
    if (xchg) {
        st = fill_exchange(p, xchg, n_seqs, n_q_heads, &D.xchg);
        if (st != SKV_OK) return st;
    }
    CUDA_TRY(p, launch_decode(D, stream));
    return SKV_OK;
}

}  // namespace

extern "C" {

size_t skv_decode_workspace_bytes(const skv_pool* p, int32_t n_seqs, int32_t n_q_heads) {
    if (!p || n_seqs <= 0 || n_q_heads <= 0) return 0;
    int32_t chunk = 0, splits = 0;
    // the largest split count any plan can produce: the smallest chunk
    decode_plan(p->cfg.page_size, p->cfg.max_pages_per_seq, n_seqs, p->cfg.num_kv_heads, 0, 0, &chunk, &splits);
    return (size_t)n_seqs * n_q_heads * splits * ((size_t)p->cfg.head_dim + 2) * sizeof(float);
}

size_t skv_exchange_bytes(int32_t mode, int32_t world, int32_t n_seqs, int32_t n_q_heads, int32_t head_dim, int32_t dtype) {
    if ((mode != SKV_XCHG_HEAD_GATHER && mode != SKV_XCHG_SEQ_MERGE) || world < 1 || world > 8 || n_seqs <= 0 ||
        n_q_heads <= 0 || head_dim <= 0 || (dtype != SKV_F32 && dtype != SKV_BF16))
        return 0;
    return 2 * 16 * exchange_words(mode, world, (int64_t)n_seqs * n_q_heads, head_dim, dtype_size(dtype));
}

int32_t skv_decode_attn(skv_pool* p, int32_t layer, const int32_t* seq_ids, int32_t n_seqs, const void* q, void* out,
                        const int32_t* q_pos, int32_t n_q_heads, float eps, void* workspace, size_t workspace_bytes,
                        void* stream) {
    if (!p) return SKV_ERR_BAD_ARG;
    if (!p->host_only && (!q || !out)) return p->fail(SKV_ERR_BAD_ARG, "q and out must be given");
    return attn_impl(p, layer, seq_ids, n_seqs, q, 0, out, 0, q_pos, n_q_heads, eps, workspace, workspace_bytes, nullptr,
                     nullptr, (cudaStream_t)stream);
}

int32_t skv_decode_attn_xchg(skv_pool* p, int32_t layer, const int32_t* seq_ids, int32_t n_seqs, const void* q,
                             const int32_t* q_pos, int32_t n_q_heads, float eps, void* workspace, size_t workspace_bytes,
                             const skv_exchange* x, void* stream) {
    if (!p || !x) return SKV_ERR_BAD_ARG;
    return attn_impl(p, layer, seq_ids, n_seqs, q, 0, nullptr, 0, q_pos, n_q_heads, eps, workspace, workspace_bytes, x,
                     nullptr, (cudaStream_t)stream);
}

int32_t skv_decode_partial(skv_pool* p, int32_t layer, const int32_t* seq_ids, int32_t n_seqs, const void* q, const int32_t* q_pos,
                           int32_t n_q_heads, void* workspace, size_t workspace_bytes, float* partial_out, void* stream) {
    if (!p) return SKV_ERR_BAD_ARG;
    if (!partial_out && !p->host_only) return p->fail(SKV_ERR_BAD_ARG, "partial_out must be given");
    return attn_impl(p, layer, seq_ids, n_seqs, q, 0, nullptr, 0, q_pos, n_q_heads, 0.f, workspace, workspace_bytes, nullptr,
                     partial_out, (cudaStream_t)stream);
}

int32_t skv_merge_partials(const float* parts, int32_t n_parts, int64_t part_stride, int32_t n_rows, int32_t head_dim, float eps,
                           void* out, int32_t dtype, void* stream) {
    if (!parts || !out || n_parts < 1 || n_parts > 128 || n_rows < 0 || head_dim <= 0) return SKV_ERR_BAD_ARG;
    if (dtype != SKV_F32 && dtype != SKV_BF16) return SKV_ERR_BAD_ARG;
    if (n_rows == 0) return SKV_OK;
    return launch_merge_partials(parts, n_parts, part_stride, n_rows, head_dim, eps, out, dtype, (cudaStream_t)stream) == cudaSuccess
               ? SKV_OK : SKV_ERR_CUDA;
}

}  // extern "C"

namespace {

// Whether the one-kernel step (RoPE, store and attention inside the split-K kernel) covers this call; otherwise
// the caller takes the append + attention pair.
bool fused_step_applies(const skv_pool* p, const skv_step_args& a, int64_t q_stride) {
    const Switches& sw = switches();
    if (!sw.step_fused || p->host_only || !p->has_maps || !p->rope_set) return false;
    if (p->cfg.dtype != SKV_BF16 || p->cfg.head_dim != 128 || p->cfg.page_size % 16 != 0) return false;
    if (a.n_q_heads <= 0 || a.n_q_heads % p->cfg.num_kv_heads != 0 || a.n_q_heads / p->cfg.num_kv_heads > 8) return false;
    if (sw.decode_generic || sw.impl_reg) return false;
    return (uintptr_t)a.q % 16 == 0 && (q_stride * 2) % 16 == 0;
}

bool overlaps(const char* lo, const char* hi, const char* a, const char* b) { return lo && a < hi && lo < b; }

// Undo of grow(): the pages go back on the free stack in the order that restores it exactly.
void ungrow(skv_pool* p, const std::vector<TableUpdate>& ups) {
    for (auto it = ups.rbegin(); it != ups.rend(); ++it) {
        p->free_pages.push_back(it->value);
        p->page_owner[it->value] = -1;
        p->pt(it->seq, it->slot) = SKV_PAGE_UNASSIGNED;
        p->n_seq_pages[it->seq] -= 1;
    }
}

int32_t step_impl(skv_pool* p, const skv_step_args& a, cudaStream_t stream) {
    const int32_t layer = a.layer, n_seqs = a.n_seqs;
    if (layer < 0) return p->fail(SKV_ERR_BAD_ARG, "layer_idx must be a non-negative integer");
    if (layer >= p->cfg.num_layers)
        return p->fail(SKV_ERR_BAD_ARG, "layer_idx %d is outside configured layer count %d", layer, p->cfg.num_layers);
    if (n_seqs <= 0 || n_seqs > p->cfg.max_seqs) return p->fail(SKV_ERR_BAD_ARG, "n_seqs %d out of range", n_seqs);
    if (a.n_q_heads <= 0 || a.n_q_heads % p->cfg.num_kv_heads != 0)
        return p->fail(SKV_ERR_BAD_ARG, "query heads must be divisible by key/value heads");
    if (a.workspace && (uintptr_t)a.workspace % 16 != 0) return p->fail(SKV_ERR_BAD_ARG, "workspace must be 16-byte aligned");
    if (!p->host_only && (!a.q || !a.k || !a.v || (!a.out && !a.xchg && !a.partial_out)))
        return p->fail(SKV_ERR_BAD_ARG, "q, k, v and out must be given");
    if (a.partial_out && a.xchg) return p->fail(SKV_ERR_BAD_ARG, "partial_out and xchg exclude each other");
    if ((a.positions == nullptr) != (a.store == nullptr))
        return p->fail(SKV_ERR_BAD_ARG, "positions and store are given together or not at all");
    const int32_t P = p->cfg.page_size, Dh = p->cfg.head_dim, Hkv = p->cfg.num_kv_heads;
    const int64_t q_stride = a.q_row_stride ? a.q_row_stride : (int64_t)a.n_q_heads * Dh;
    const int64_t out_stride = a.out_row_stride ? a.out_row_stride : (int64_t)a.n_q_heads * Dh;
    const int64_t k_stride = a.k_row_stride ? a.k_row_stride : (int64_t)Hkv * Dh;
    const int64_t v_stride = a.v_row_stride ? a.v_row_stride : (int64_t)Hkv * Dh;
    if (q_stride < (int64_t)a.n_q_heads * Dh || out_stride < (int64_t)a.n_q_heads * Dh || k_stride < (int64_t)Hkv * Dh ||
        v_stride < (int64_t)Hkv * Dh)
        return p->fail(SKV_ERR_BAD_ARG, "a row stride is shorter than the row");

    if (!fused_step_applies(p, a, q_stride)) {
        // the append + attention pair (float32 pools, other head sizes, bookkeeping-only pools, SKV_STEP_FUSED=0)
        if (a.positions) return p->fail(SKV_ERR_UNSUPPORTED, "a sequence-sharded step needs the bf16 / head_dim 128 kernel");
        skv_append_args ap{};
        ap.layer = layer;
        ap.n_seqs = n_seqs;
        ap.seq_ids = a.seq_ids;
        ap.n_new = 1;
        ap.k = a.k;
        ap.v = a.v;
        ap.kv_stride_seq = k_stride;
        ap.kv_stride_head = Dh;
        ap.rope_k = 1;
        ap.q_in = a.q;
        ap.q_out = a.q;
        ap.n_q_heads = a.n_q_heads;
        ap.q_stride_seq = q_stride;
        ap.q_stride_head = Dh;
        if (k_stride != v_stride) return p->fail(SKV_ERR_UNSUPPORTED, "k and v need the same row stride outside the one-kernel step");
        // the attention half can still refuse (workspace): check what does not depend on the append first
        if (!p->host_only) {
            const size_t least = (size_t)n_seqs * a.n_q_heads * ((size_t)Dh + 2) * sizeof(float);
            int32_t st0 = check_workspace(p, a.workspace, a.workspace_bytes, least);
            if (st0 != SKV_OK) return st0;
        }
        int32_t st = skv_append(p, &ap, stream);
        if (st != SKV_OK) return st;
        return attn_impl(p, layer, a.seq_ids, n_seqs, a.q, q_stride, a.partial_out ? nullptr : a.out, out_stride, nullptr,
                         a.n_q_heads, a.eps, a.workspace, a.workspace_bytes, a.xchg, a.partial_out, stream);
    }

    // ---- validation: nothing is changed or enqueued before all of it has passed -------------------------------
    const bool inline_rows = n_seqs <= kInlineRows;
    if (!inline_rows && (size_t)n_seqs * 3 * sizeof(int32_t) > StagingRing::kSlotBytes)
        return p->fail(SKV_ERR_BAD_ARG, "too many sequences (%d) for one call", n_seqs);
    int64_t total = 0, need_total = 0;
    int32_t longest = 0;
    if (a.seq_ids && ++p->stamp == 0) {   // generation counter wrapped: start over
        std::fill(p->seen_stamp.begin(), p->seen_stamp.end(), 0u);
        p->stamp = 1;
    }
    for (int32_t i = 0; i < n_seqs; ++i) {
        const int32_t s = a.seq_ids ? a.seq_ids[i] : i;
        if (!valid_seq(p, s)) return p->fail(SKV_ERR_BAD_ARG, "sequence %d is not live", s);
        if (a.seq_ids) {
            if (p->seen_stamp[s] == p->stamp) return p->fail(SKV_ERR_BAD_ARG, "sequence %d listed twice", s);
            p->seen_stamp[s] = p->stamp;
        }
        const int32_t cur = p->len(layer, s);
        const int32_t stores = a.store ? (a.store[i] ? 1 : 0) : 1;
        if (a.positions && (a.positions[i] < 0 || (uint32_t)a.positions[i] > kRowPosMask))
            return p->fail(SKV_ERR_BAD_ARG, "position of row %d is outside [0, 2^30)", i);
        const int32_t need = (cur + stores + P - 1) / P;
        if (need > p->cfg.max_pages_per_seq)
            return p->fail(SKV_ERR_OUT_OF_PAGES, "sequence %d needs %d pages, row holds %d", s, need, p->cfg.max_pages_per_seq);
        need_total += std::max(0, need - p->n_seq_pages[s]);
        for (int32_t slot = 0; p->n_parked[s] > 0 && slot < std::min(need, p->n_seq_pages[s]); ++slot)
            if (p->pt(s, slot) < 0) return p->fail(SKV_ERR_NOT_RESIDENT, "sequence %d slot %d is not resident", s, slot);
        total += cur + stores;
        longest = std::max(longest, cur + stores);
    }
    if (need_total > (int64_t)p->free_pages.size())
        return p->fail(SKV_ERR_OUT_OF_PAGES, "need %lld pages, %zu free", (long long)need_total, p->free_pages.size());
    DecodeLaunch D{};
    D.longest = longest;
    decode_plan(P, p->cfg.max_pages_per_seq, n_seqs, Hkv, total, longest, &D.chunk_tokens, &D.max_splits);
    if (D.max_splits > 128) return p->fail(SKV_ERR_UNSUPPORTED, "a sequence would need %d split-K chunks, 128 is the limit", D.max_splits);
    D.grid_splits = std::max(1, (longest + D.chunk_tokens - 1) / D.chunk_tokens);
    const size_t need_ws = (size_t)n_seqs * a.n_q_heads * D.max_splits * ((size_t)Dh + 2) * sizeof(float);
    int32_t st = check_workspace(p, a.workspace, a.workspace_bytes, need_ws);
    if (st != SKV_OK) return st;
    if (a.xchg) {
        st = fill_exchange(p, a.xchg, n_seqs, a.n_q_heads, &D.xchg);
        if (st != SKV_OK) return st;
    }

    DeviceGuard guard(p);
    // May the split-K kernel run ahead of the previous kernel in the stream?  Only when the caller says that this
    // call directly follows this pool's previous step, when no other call of the library launched anything in
    // between, and when q, k, v do not overlap what that step's merge kernel wrote.
    const char* q_lo = (const char*)a.q;
    const char* q_hi = q_lo + ((int64_t)(n_seqs - 1) * q_stride + (int64_t)a.n_q_heads * Dh) * 2;
    const char* k_lo = (const char*)a.k;
    const char* k_hi = k_lo + ((int64_t)(n_seqs - 1) * k_stride + (int64_t)Hkv * Dh) * 2;
    const char* v_lo = (const char*)a.v;
    const char* v_hi = v_lo + ((int64_t)(n_seqs - 1) * v_stride + (int64_t)Hkv * Dh) * 2;
    bool early = (a.flags & SKV_STEP_CONSECUTIVE) && switches().step_early && p->last_step_valid && p->last_step_stream == stream &&
                 p->last_step_mark == g_launches.load(std::memory_order_relaxed) && inline_rows;
    for (int w = 0; early && w < 2; ++w)
        if (overlaps(p->last_w_lo[w], p->last_w_hi[w], q_lo, q_hi) || overlaps(p->last_w_lo[w], p->last_w_hi[w], k_lo, k_hi) ||
            overlaps(p->last_w_lo[w], p->last_w_hi[w], v_lo, v_hi))
            early = false;
    p->last_step_valid = false;

    // ---- fallible work that does not depend on the new state ------------------------------------------------
    const bool copies_were_pending = p->copy_pending;
    st = order_transfers_for(p, stream, a.seq_ids, n_seqs, need_total > 0);
    if (st != SKV_OK) return st;
    if (copies_were_pending && !p->copy_pending) early = false;   // a wait for the copy stream now sits ahead of the step
    // ---- mutate, then enqueue; a failure from here on puts the host state back -----------------------------------
    std::vector<TableUpdate>& ups = p->step_ups;
    ups.clear();
    p->step_store.resize(n_seqs);
    for (int32_t i = 0; i < n_seqs; ++i) {
        const int32_t s = a.seq_ids ? a.seq_ids[i] : i;
        const int32_t stores = a.store ? (a.store[i] ? 1 : 0) : 1;
        p->step_store[i] = stores;
        if (stores) grow(p, s, p->len(layer, s) + 1, &ups);   // cannot fail after the checks above
    }
    StepRows& R = p->rows;
    std::vector<int32_t> big;   // only for calls beyond the inline capacity
    if (!inline_rows) big.resize((size_t)3 * n_seqs);
    for (int32_t i = 0; i < n_seqs; ++i) {
        const int32_t s = a.seq_ids ? a.seq_ids[i] : i;
        const int32_t cur = p->len(layer, s);
        // the row's newest token came from a step (possibly still running when this one starts early): guarded
        const bool guarded = cur > 0 && p->step_len[(size_t)layer * p->cfg.max_seqs + s] == cur;
        const uint32_t pos = (uint32_t)(a.positions ? a.positions[i] : cur) | (p->step_store[i] ? 0u : kRowNoStore) |
                             (guarded ? kRowWaitPrev : 0u);
        if (inline_rows) {
            R.seq[i] = s;
            R.len[i] = cur;
            R.pos[i] = pos;
        } else {
            big[i] = s;
            big[(size_t)n_seqs + i] = cur;
            big[(size_t)2 * n_seqs + i] = (int32_t)pos;
        }
    }
    for (int32_t i = 0; i < n_seqs; ++i) {
        const int32_t s = a.seq_ids ? a.seq_ids[i] : i;
        if (p->step_store[i]) p->step_len[(size_t)layer * p->cfg.max_seqs + s] = (p->len(layer, s) += 1);
    }
    auto roll_back = [&]() {
        for (int32_t i = 0; i < n_seqs; ++i) {
            const int32_t s = a.seq_ids ? a.seq_ids[i] : i;
            if (p->step_store[i]) {
                p->len(layer, s) -= 1;
                p->step_len[(size_t)layer * p->cfg.max_seqs + s] = -1;
            }
        }
        ungrow(p, ups);
    };
    st = publish_table_updates(p, ups, stream);
    if (st != SKV_OK) {
        roll_back();
        return st;
    }
    // More live CTAs than the GPU holds at once (3 per SM) and rows of one or two chunks: hand the longest rows out
    // first, so that the CTAs that start late, in freed slots, are short ones.  64 ragged rows of 88..1024 tokens x 8
    // KV heads (a sequence-sharded rank's share): the split-K kernel's SMs were busy 65 % of its 47 us with the rows
    // in the caller's order; 49.5 -> 41.8 us per step (rows of up to 2048 tokens: 71.3 -> 62.6).  Rows of many chunks
    // do not gain (their CTAs are equal but for the last one; the 64-sequence workload of 6 chunks per row lost 3 %).
    R.ordered = 0;
    if (inline_rows && switches().order != 0) {
        int64_t live = 0;
        for (int32_t i = 0; i < n_seqs; ++i) live += (R.len[i] + D.chunk_tokens) / D.chunk_tokens;   // chunks of len + 1 tokens, at least one
        live *= Hkv;
        if (switches().order == 1 || (D.grid_splits <= 2 && live > 3 * (int64_t)p->sm_count)) {
            for (int32_t i = 0; i < n_seqs; ++i) R.order[i] = (uint8_t)i;
            std::sort(R.order, R.order + n_seqs,
                      [&](uint8_t x, uint8_t y) { return R.len[x] != R.len[y] ? R.len[x] > R.len[y] : x < y; });   // in place, no allocation
            R.ordered = 1;
        }
    }
    R.dev = nullptr;
    if (!inline_rows) {
        void* dev = nullptr;
        cudaError_t e = p->ring.upload(big.data(), big.size() * sizeof(int32_t), stream, &dev);
        if (e != cudaSuccess) {
            roll_back();
            return p->cuda_fail(e, "upload of the step's rows");
        }
        R.dev = (const int32_t*)dev;
        early = false;
    }
    if (!ups.empty()) early = false;   // the page-table update sits between the two kernels anyway
    D.pool = p->view();
    D.layer = layer;
    D.n_seqs = n_seqs;
    D.n_q_heads = a.n_q_heads;
    D.dtype = p->cfg.dtype;
    D.q = a.q;
    D.out = a.out;
    D.q_stride = q_stride;
    D.out_stride = out_stride;
    D.eps = a.eps;
    D.ws_acc = (float*)a.workspace;
    D.ws_ml = D.ws_acc + (size_t)n_seqs * a.n_q_heads * D.max_splits * Dh;
    D.k_map = &p->k_map;
    D.v_map = &p->v_map;
    D.tickets = p->d_tickets;
    D.total_tokens = total;
    D.fused_append = 1;
    D.new_k = a.k;
    D.new_v = a.v;
    D.k_stride = k_stride;
    D.v_stride = v_stride;
    D.inv_freq = p->d_inv_freq;
    D.rope_scaling = p->rope_scaling;
    D.early_start = early ? 1 : 0;
    D.stored_len = p->d_stored_len;
    D.rows = &R;
    if (a.xchg || a.partial_out) D.out = nullptr;
    D.partial_out = a.partial_out;
    cudaError_t e = launch_decode(D, stream);
    if (e != cudaSuccess) {
        roll_back();
        return p->cuda_fail(e, "launch of the decode step");
    }
    // what the merge kernel of this step writes besides pages and partials
    p->last_w_lo[0] = q_lo;
    p->last_w_hi[0] = q_hi;
    if (a.xchg) {
        const size_t rows_total = (size_t)n_seqs * a.n_q_heads * (a.xchg->mode == SKV_XCHG_HEAD_GATHER ? a.xchg->world : 1);
        p->last_w_lo[1] = (const char*)a.xchg->out;
        p->last_w_hi[1] = p->last_w_lo[1] + rows_total * Dh * 2;
    } else if (a.partial_out) {
        p->last_w_lo[1] = (const char*)a.partial_out;
        p->last_w_hi[1] = p->last_w_lo[1] + (size_t)n_seqs * a.n_q_heads * (Dh + 2) * sizeof(float);
    } else {
        p->last_w_lo[1] = (const char*)a.out;
        p->last_w_hi[1] = p->last_w_lo[1] + ((int64_t)(n_seqs - 1) * out_stride + (int64_t)a.n_q_heads * Dh) * 2;
    }
    p->last_step_stream = stream;
    p->last_step_mark = g_launches.load(std::memory_order_relaxed);
    p->last_step_valid = true;
    return SKV_OK;
}

}  // namespace

extern "C" {

int32_t skv_decode_step_ex(skv_pool* p, const skv_step_args* a, void* stream) {
    if (!p || !a) return SKV_ERR_BAD_ARG;
    return step_impl(p, *a, (cudaStream_t)stream);
}

int32_t skv_decode_step(skv_pool* p, int32_t layer, int32_t n_seqs, void* q, const void* k, const void* v, void* out,
                        int32_t n_q_heads, float eps, void* workspace, size_t workspace_bytes, void* stream) {
    return skv_decode_step_seqs(p, layer, nullptr, n_seqs, q, k, v, out, n_q_heads, eps, workspace, workspace_bytes, stream);
}

int32_t skv_decode_step_seqs(skv_pool* p, int32_t layer, const int32_t* seq_ids, int32_t n_seqs, void* q, const void* k,
                             const void* v, void* out, int32_t n_q_heads, float eps, void* workspace, size_t workspace_bytes,
                             void* stream) {
    if (!p) return SKV_ERR_BAD_ARG;
    skv_step_args a{};
    a.layer = layer;
    a.n_seqs = n_seqs;
    a.seq_ids = seq_ids;
    a.q = q;
    a.k = k;
    a.v = v;
    a.out = out;
    a.n_q_heads = n_q_heads;
    a.eps = eps;
    a.workspace = workspace;
    a.workspace_bytes = workspace_bytes;
    return step_impl(p, a, (cudaStream_t)stream);
}

int32_t skv_decode_step_xchg(skv_pool* p, int32_t layer, const int32_t* seq_ids, int32_t n_seqs, void* q, const void* k,
                             const void* v, int32_t n_q_heads, float eps, void* workspace, size_t workspace_bytes,
                             const skv_exchange* xchg, void* stream) {
    if (!p || !xchg) return SKV_ERR_BAD_ARG;
    skv_step_args a{};
    a.layer = layer;
    a.n_seqs = n_seqs;
    a.seq_ids = seq_ids;
    a.q = q;
    a.k = k;
    a.v = v;
    a.n_q_heads = n_q_heads;
    a.eps = eps;
    a.workspace = workspace;
    a.workspace_bytes = workspace_bytes;
    a.xchg = xchg;
    return step_impl(p, a, (cudaStream_t)stream);
}

int32_t skv_attn_dense(const void* q, const void* k, const void* v, void* out, const int32_t* positions, int32_t B,
                       int32_t Hq, int32_t Hkv, int32_t Lq, int32_t Lk, int32_t D, int32_t dtype, int32_t causal,
                       float eps, int32_t* status, void* stream_) {
    // shape rules of mlx_ops.py:51-67
    if (!q || !k || !v || !out) return SKV_ERR_BAD_ARG;
    if (B <= 0 || Hq <= 0 || Lq < 0 || Lk < 0 || D <= 0) return SKV_ERR_BAD_ARG;
    if (Hkv <= 0 || Hq % Hkv != 0) return SKV_ERR_BAD_ARG;
    if (causal && Lk < Lq) return SKV_ERR_BAD_ARG;
    if (dtype != SKV_F32 && dtype != SKV_BF16) return SKV_ERR_BAD_ARG;
    if (D > 256) return SKV_ERR_UNSUPPORTED;
    if (Lq == 0) return SKV_OK;
    DenseAttnLaunch A{};
    A.q = q; A.k = k; A.v = v; A.out = out; A.positions = positions;
    A.B = B; A.Hq = Hq; A.Hkv = Hkv; A.Lq = Lq; A.Lk = Lk; A.D = D; A.dtype = dtype; A.causal = causal;
    A.eps = eps;
    A.pool.k_base = nullptr;
    A.status = status;
    cudaStream_t stream = (cudaStream_t)stream_;
    cudaError_t e = cudaErrorNotSupported;
    if (!switches().prefill_generic) e = launch_attn_tc(A, stream);
    if (e == cudaErrorNotSupported) e = launch_attn_generic(A, stream);
    return e == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}

int32_t skv_prefill_attn_paged(skv_pool* p, int32_t layer, const int32_t* seq_ids, int32_t n_seqs, const void* q, void* out,
                               const int32_t* positions, int32_t n_q_heads, int32_t Lq, int32_t causal, float eps, void* stream_) {
    if (!p) return SKV_ERR_BAD_ARG;
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n_q_heads <= 0 || n_q_heads % p->cfg.num_kv_heads != 0)
        return p->fail(SKV_ERR_BAD_ARG, "query heads must be divisible by key/value heads");
    int32_t st = check_readable(p, layer, seq_ids, n_seqs, nullptr);
    if (st != SKV_OK) return st;
    if (Lq < 0) return p->fail(SKV_ERR_BAD_ARG, "Lq must be non-negative");
    if (causal && !positions)
        for (int32_t i = 0; i < n_seqs; ++i)
            if (p->len(layer, seq_ids ? seq_ids[i] : i) < Lq)
                return p->fail(SKV_ERR_BAD_ARG, "causal attention requires key length >= query length");
    if (p->host_only || Lq == 0) return SKV_OK;
    if (!q || !out) return p->fail(SKV_ERR_BAD_ARG, "q and out must be given");
    DeviceGuard g(p);
    st = order_transfers(p, stream);
    if (st != SKV_OK) return st;
    DenseAttnLaunch A{};
    A.q = q; A.out = out; A.positions = positions;
    A.B = n_seqs; A.Hq = n_q_heads; A.Hkv = p->cfg.num_kv_heads; A.Lq = Lq; A.Lk = 0; A.D = p->cfg.head_dim;
    A.dtype = p->cfg.dtype; A.causal = causal ? 1 : 0; A.eps = eps;
    A.pool = p->view();
    A.layer = layer;
    st = upload_ids(p, seq_ids, n_seqs, stream, &A.seq_ids);
    if (st != SKV_OK) return st;
    A.k_map = p->has_maps ? &p->k_map : nullptr;
    A.v_map = p->has_maps ? &p->v_map : nullptr;
    // bf16, head_dim 128, pages of a multiple of 16 tokens and at least 32 query rows: the tensor-core kernel reads the pages
    // directly through the pool's tensor maps; everything else takes the float32 CUDA-core kernel
    cudaError_t e = cudaErrorNotSupported;
    if (!switches().prefill_generic) e = launch_attn_tc(A, stream);
    if (e == cudaErrorNotSupported) e = launch_attn_generic(A, stream);
    CUDA_TRY(p, e);
    return SKV_OK;
}

int32_t skv_evict(skv_pool* p, int32_t seq, int32_t first_slot, int32_t n_slots, void* stream_) {
    if (!p) return SKV_ERR_BAD_ARG;
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!valid_seq(p, seq)) return p->fail(SKV_ERR_BAD_ARG, "sequence %d is not live", seq);
    if (first_slot < 0 || n_slots < 0 || first_slot + n_slots > p->n_seq_pages[seq])
        return p->fail(SKV_ERR_BAD_ARG, "slots [%d, %d) outside the sequence's %d pages", first_slot, first_slot + n_slots, p->n_seq_pages[seq]);
    if (p->cfg.host_pages == 0) return p->fail(SKV_ERR_BAD_ARG, "pool was created without a host tier");
    int32_t movable = 0;
    for (int32_t s = first_slot; s < first_slot + n_slots; ++s) movable += p->pt(seq, s) >= 0;
    if ((size_t)movable > p->free_host.size())
        return p->fail(SKV_ERR_OUT_OF_PAGES, "need %d host slots, %zu free", movable, p->free_host.size());
    std::vector<CopyItem> items;
    std::vector<TableUpdate> ups;
    for (int32_t s = first_slot; s < first_slot + n_slots; ++s) {
        int32_t e = p->pt(seq, s);
        if (e < 0) continue;
        int32_t h = p->free_host.back();
        p->free_host.pop_back();
        p->pt(seq, s) = -2 - h;
        p->n_parked[seq] += 1;
        p->page_owner[e] = -1;
        items.push_back({e, h});
        ups.push_back({seq, s, -2 - h});
    }
    for (auto it = items.rbegin(); it != items.rend(); ++it) p->free_pages.push_back(it->page);
    p->n_evicted += (int64_t)items.size();
    p->bytes_d2h += (int64_t)items.size() * p->cfg.num_layers * 2 * (int64_t)p->page_bytes;
    if (p->host_only || items.empty()) return SKV_OK;
    DeviceGuard g(p);
    // Page-table entries deferred by earlier prefetches must reach the device before this call's entries: flushed
    // later, they would overwrite them with stale page ids.
    if (!p->deferred_updates.empty()) {
        int32_t st0 = order_transfers(p, stream);
        if (st0 != SKV_OK) return st0;
    }
    // the copy must see everything already enqueued on the compute stream
    CUDA_TRY(p, cudaEventRecord(p->ev_compute, stream));
    CUDA_TRY(p, cudaStreamWaitEvent(p->copy_stream, p->ev_compute, 0));
    const size_t per = StagingRing::kSlotBytes / sizeof(CopyItem);
    for (size_t off = 0; off < items.size(); off += per) {
        size_t n = std::min(per, items.size() - off);
        void* dev = nullptr;
        CUDA_TRY(p, p->ring_copy.upload(items.data() + off, n * sizeof(CopyItem), p->copy_stream, &dev));
        dim3 grid((unsigned)std::min<size_t>(n, 32), (unsigned)std::min(p->cfg.num_layers * 2, 8));
        page_copy_kernel<<<grid, 256, 0, p->copy_stream>>>(p->d_k, p->d_v, p->h_tier_dev, (const CopyItem*)dev, (int)n,
                                                           (int64_t)p->layer_stride, (int64_t)p->page_bytes,
                                                           p->cfg.num_layers, 1);
        CUDA_TRY(p, cudaGetLastError());
        count_launches(1);
    }
    p->copy_pending = true;   // freed pages may be rewritten only after the copy: order_transfers enforces it
    p->copy_busy[seq] = 1;
    return publish_table_updates(p, ups, stream);
}

int32_t skv_prefetch(skv_pool* p, int32_t seq, int32_t first_slot, int32_t n_slots, void* stream_) {
    if (!p) return SKV_ERR_BAD_ARG;
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!valid_seq(p, seq)) return p->fail(SKV_ERR_BAD_ARG, "sequence %d is not live", seq);
    if (first_slot < 0 || n_slots < 0 || first_slot + n_slots > p->n_seq_pages[seq])
        return p->fail(SKV_ERR_BAD_ARG, "slots [%d, %d) outside the sequence's %d pages", first_slot, first_slot + n_slots, p->n_seq_pages[seq]);
    int32_t parked = 0;
    for (int32_t s = first_slot; s < first_slot + n_slots; ++s) parked += p->pt(seq, s) <= -2;
    if ((size_t)parked > p->free_pages.size())
        return p->fail(SKV_ERR_OUT_OF_PAGES, "need %d device pages, %zu free", parked, p->free_pages.size());
    std::vector<CopyItem> items;
    for (int32_t s = first_slot; s < first_slot + n_slots; ++s) {
        int32_t e = p->pt(seq, s);
        if (e > -2) continue;
        int32_t h = -2 - e;
        int32_t page = p->free_pages.back();
        p->free_pages.pop_back();
        p->pt(seq, s) = page;
        p->n_parked[seq] -= 1;
        p->page_owner[page] = seq;
        items.push_back({page, h});
        p->deferred_updates.push_back({seq, s, page});
    }
    for (auto it = items.rbegin(); it != items.rend(); ++it) p->free_host.push_back(it->slot);
    p->n_prefetched += (int64_t)items.size();
    p->bytes_h2d += (int64_t)items.size() * p->cfg.num_layers * 2 * (int64_t)p->page_bytes;
    if (p->host_only) {
        p->deferred_updates.clear();
        return SKV_OK;
    }
    if (items.empty()) return SKV_OK;
    DeviceGuard g(p);
    // target pages may still be read by kernels already enqueued on the compute stream
    CUDA_TRY(p, cudaEventRecord(p->ev_compute, stream));
    CUDA_TRY(p, cudaStreamWaitEvent(p->copy_stream, p->ev_compute, 0));
    const size_t per = StagingRing::kSlotBytes / sizeof(CopyItem);
    for (size_t off = 0; off < items.size(); off += per) {
        size_t n = std::min(per, items.size() - off);
        void* dev = nullptr;
        CUDA_TRY(p, p->ring_copy.upload(items.data() + off, n * sizeof(CopyItem), p->copy_stream, &dev));
        dim3 grid((unsigned)std::min<size_t>(n, 32), (unsigned)std::min(p->cfg.num_layers * 2, 8));
        page_copy_kernel<<<grid, 256, 0, p->copy_stream>>>(p->d_k, p->d_v, p->h_tier_dev, (const CopyItem*)dev, (int)n,
                                                           (int64_t)p->layer_stride, (int64_t)p->page_bytes,
                                                           p->cfg.num_layers, 0);
        CUDA_TRY(p, cudaGetLastError());
        count_launches(1);
    }
    p->copy_pending = true;
    p->copy_busy[seq] = 1;
    return SKV_OK;
}

int32_t skv_sync_transfers(skv_pool* p, void* stream_) {
    if (!p) return SKV_ERR_BAD_ARG;
    DeviceGuard g(p);
    return order_transfers(p, (cudaStream_t)stream_);
}

int32_t skv_wait_resident(skv_pool* p, int32_t timeout_ms) {
    if (!p) return SKV_ERR_BAD_ARG;
    if (p->host_only) return SKV_OK;
    DeviceGuard g(p);
    auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        cudaError_t e = cudaStreamQuery(p->copy_stream);
        if (e == cudaSuccess) return SKV_OK;
        if (e != cudaErrorNotReady) return p->cuda_fail(e, "cudaStreamQuery(copy_stream)");
        auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms >= timeout_ms) return p->fail(SKV_ERR_TIMEOUT, "transfers still running after %d ms", timeout_ms);
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

int32_t skv_check_device_status(skv_pool* p, void* stream_, int32_t* flag_out) {
    if (!p) return SKV_ERR_BAD_ARG;
    if (flag_out) *flag_out = 0;
    if (p->host_only) return SKV_OK;
    DeviceGuard g(p);
    cudaStream_t stream = (cudaStream_t)stream_;
    int32_t flag = 0;
    CUDA_TRY(p, cudaMemcpyAsync(&flag, p->d_status, sizeof flag, cudaMemcpyDeviceToHost, stream));
    CUDA_TRY(p, cudaStreamSynchronize(stream));
    if (flag_out) *flag_out = flag;
    if (flag != 0) {
        CUDA_TRY(p, cudaMemsetAsync(p->d_status, 0, sizeof flag, stream));
        // a kernel that gave up may have left arrival counters behind
        CUDA_TRY(p, cudaMemsetAsync(p->d_tickets, 0, ((size_t)p->cfg.max_seqs * p->cfg.num_kv_heads + 2) * sizeof(int32_t), stream));
        return p->fail(SKV_ERR_DEVICE_FLAG, "device status word 0x%x (1 bad page id, 2 bad length, 4 bad sequence id)", flag);
    }
    return SKV_OK;
}

int32_t skv_rope_rows(const void* x_in, void* x_out, const int32_t* positions, const float* inv_freq_dev, int32_t n_rows,
                      int32_t n_heads, int32_t head_dim, int64_t stride_row, int64_t stride_head, float scaling,
                      int32_t dtype, void* stream_) {
    if (!x_in || !x_out || !positions || !inv_freq_dev) return SKV_ERR_BAD_ARG;
    if (n_rows < 0 || n_heads <= 0 || head_dim <= 0 || head_dim % 2 != 0 || !(scaling > 0.0f)) return SKV_ERR_BAD_ARG;
    if (dtype != SKV_F32 && dtype != SKV_BF16) return SKV_ERR_BAD_ARG;
    if (n_rows == 0) return SKV_OK;
    RopeRowsLaunch R{x_in, x_out, positions, inv_freq_dev, n_rows, n_heads, head_dim, dtype, stride_row, stride_head, scaling};
    return launch_rope_rows(R, (cudaStream_t)stream_) == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}

}  // extern "C"
