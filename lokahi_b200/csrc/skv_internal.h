// Internal declarations shared by the host pool and the kernel translation units.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "strata_b200.h"

namespace skv {

// Device-visible description of one pool, passed to kernels by value.
struct PoolView {
    void* k_base;                 // layer 0 K pool; layers are layer_stride bytes apart
    void* v_base;
    int64_t layer_stride_bytes;
    const int32_t* page_table;    // [max_seqs][max_pages_per_seq]
    int32_t* lengths;             // [num_layers][max_seqs]
    int32_t* status;              // device status word (0 = fine)
    int32_t num_kv_heads, head_dim, page_size, num_pages, max_seqs, max_pages_per_seq;
};

// Bits recorded in the device status word.
enum : int32_t {
    FLAG_BAD_PAGE = 1,       // page-table entry outside [0, num_pages)
    FLAG_BAD_LENGTH = 2,     // length beyond the page-table row
    FLAG_BAD_SEQ = 4,        // sequence id outside [0, max_seqs)
    FLAG_WAIT_TIMEOUT = 8,   // a bounded wait (mbarrier, peer flag) ran out
};

// Per-call metadata uploaded through the staging ring.
struct AppendMeta {            // followed in memory by n_seqs x {seq, start}
    int32_t seq;
    int32_t start;
};

struct AppendLaunch {
    PoolView pool;
    int32_t layer, n_seqs, n_new, dtype;
    const AppendMeta* meta;      // device, n_seqs entries
    const void* k;
    const void* v;
    int64_t kv_stride_seq, kv_stride_head, kv_stride_tok;
    int32_t rope_k;
    const void* q_in;
    void* q_out;
    int32_t n_q_heads;
    int64_t q_stride_seq, q_stride_head, q_stride_tok;
    const float* inv_freq;       // device, head_dim/2
    float inv_scaling;           // 1 / scaling_factor applied as a division of the position
    float scaling;
};
cudaError_t launch_append(const AppendLaunch& a, cudaStream_t stream);

struct GatherLaunch {
    PoolView pool;
    int32_t layer, n_seqs, max_len, dtype;
    const int32_t* seq_ids;      // device or nullptr (identity)
    void* out_k;
    void* out_v;
};
cudaError_t launch_gather(const GatherLaunch& g, cudaStream_t stream);

// Exchange fused into the merge kernel.  Every 8-byte unit that crosses NVLink carries its own flag (4 bytes of
// payload + the call's epoch), so a receiver validates what it reads by itself: no fence, no ticket and no separate
// flag write sit between a peer store and the moment the peer may consume it.  Two units travel per 16-byte store.
//   mode 1 (KV-head sharding): a merge block stores its finished output row into slot `rank` of every rank's
//     receive buffer, then polls the same row of all `world` slots of its own buffer and unpacks them into the
//     plain gathered output `out` [world][n_seqs][q_heads][head_dim].
//   mode 2 (sequence sharding): a merge block sends its un-normalised partial row (acc[D], m, l) to the row's
//     owner (row % world); the owner's block merges the `world` partials with the chunk-merge rule
//     (mlx_ops.py:125-146) and broadcasts the finished row; every block unpacks it into `out`
//     [n_seqs][q_heads][head_dim].
struct ExchangeView {
    int32_t mode;                // 0: none, 1: head gather, 2: sequence-shard merge
    int32_t world, rank;
    uint32_t epoch;              // > 0, grows by one per call; receive buffers alternate by its parity
    void* recv[8];               // per rank: base of its receive buffer of THIS call's parity (peer-mapped)
    void* out;                   // local result buffer (plain layout)
};

// Per-row metadata of a one-call decode step, carried in the kernel parameters: the split-K kernel of a step
// reads nothing that the previous step's merge kernel wrote until it stores its partials, so its start-up and its
// K/V streaming overlap that merge kernel (and the exchange wait inside it).  Calls with more rows than fit here
// upload the same three arrays and pass them through `dev`.
#ifndef SKV_INLINE_ROWS
#define SKV_INLINE_ROWS 256
#endif
constexpr int kInlineRows = SKV_INLINE_ROWS;
constexpr uint32_t kRowNoStore = 0x80000000u;   // bit 31 of pos: this pool does not store the step's token
constexpr uint32_t kRowWaitPrev = 0x40000000u;  // bit 30 of pos: the row's newest token was stored by an earlier step that
                                                // may still be running: wait for its flag before reading that page row
constexpr uint32_t kRowPosMask = 0x3fffffffu;
struct StepRows {
    const int32_t* dev;           // nullptr, or device [3][n_seqs]: seq, len, pos
    int32_t seq[kInlineRows];     // sequence id of row i
    int32_t len[kInlineRows];     // tokens of row i held by this pool before the step
    uint32_t pos[kInlineRows];    // absolute position of the step's token (RoPE angle) | kRowNoStore
    uint8_t order[kInlineRows];   // when `ordered`: the split-K kernel's grid index z works on row order[z] (longest rows
    int32_t ordered;              // first, so that a grid of more CTAs than the GPU holds ends on short ones)
};
static_assert(kInlineRows <= 256, "row indices are stored in one byte");

struct DecodeLaunch {
    PoolView pool;
    int32_t layer, n_seqs, n_q_heads, dtype;
    const int32_t* seq_ids;      // device or nullptr (identity)
    const int32_t* q_pos;        // device or nullptr (length - 1)
    const void* q;
    void* out;
    int64_t q_stride, out_stride;   // elements between the rows of consecutive sequences (heads are contiguous)
    float eps;
    float* ws_acc;               // [n_seqs][n_q_heads][max_splits][head_dim]
    float* ws_ml;                // [n_seqs][n_q_heads][max_splits][2]
    int32_t max_splits, chunk_tokens;
    int32_t grid_splits;         // chunks of the longest sequence of this call (0: launch max_splits of them)
    int32_t force_generic;       // 1: take the CUDA-core kernel even where the tensor-core one applies
    // tensor maps (host pointers to CUtensorMap) of the K and V pools viewed as [rows][head_dim] bf16 with
    // [16][64] boxes; nullptr when the pool has none, and then the direct-load kernel runs
    const void* k_map;
    const void* v_map;
    // [n_seqs][kv_heads] arrival counters, zero between calls: the CTA that finishes last for a
    // (sequence, KV head) merges the partials itself, so no separate merge launch is needed
    int32_t* tickets;
    int32_t fuse_merge;          // 0: leave the merge to decode_reduce_kernel
    int64_t total_tokens;        // host's sum of the attended lengths (drives the plan and the merge choice)
    int32_t longest;             // host's longest attended length of the call (drives the plan)
    ExchangeView xchg;
    float* partial_out;          // when set, the merge kernel writes un-normalised [n_seqs][q_heads][head_dim + 2]
                                 // rows (acc..., m, l) instead of the output: the unit of sequence sharding
    // One-call decode step (bf16 TMA kernel only): per-row sequence id, stored length and token position come
    // from `rows`.  Every CTA rotates its own copy of q at the token's position; the CTA whose chunk contains
    // the row's length rotates the new K row, stores it and the V row into the page and attends the token from
    // shared memory; the merge kernel writes the rotated q back and sets the device lengths.
    int32_t fused_append;
    const void* new_k;           // row i at new_k + i * k_stride elements: [kv_heads][head_dim], un-rotated
    const void* new_v;
    int64_t k_stride, v_stride;
    const float* inv_freq;       // [head_dim / 2]
    float rope_scaling;
    int32_t early_start;         // 1: the split-K kernel of a step may run beside the previous step's kernels up to the
                                 // point where it stores its partials (the caller vouched for its inputs); rows marked
                                 // kRowWaitPrev wait until stored_len[layer][seq][head] has reached the row's length
                                 // before they read the page row of its newest token
    int32_t* stored_len;         // [layers][max_seqs][kv_heads]: tokens of (layer, seq, head) in place, as published by
                                 // the CTA of a step that stored the last of them
    const StepRows* rows;        // host pointer; copied into the kernel parameters at launch
};
cudaError_t launch_decode(const DecodeLaunch& d, cudaStream_t stream);
// chunk length (tokens handled by one CTA) and the number of splits that follow from it; the hints (0 = unknown)
// are the call's attended tokens in all and its longest sequence
void decode_plan(int32_t page_size, int32_t max_pages_per_seq, int32_t n_seqs, int32_t num_kv_heads,
                 int64_t total_tokens_hint, int32_t longest_hint, int32_t* chunk_tokens, int32_t* max_splits);

struct DenseAttnLaunch {
    const void *q, *k, *v;
    void* out;
    const int32_t* positions;    // device [B][Lq] or nullptr
    int32_t B, Hq, Hkv, Lq, Lk, D, dtype, causal;
    float eps;
    // paged K/V instead of dense (k, v ignored) when pool.k_base != nullptr
    PoolView pool;
    int32_t layer;
    const int32_t* seq_ids;      // device or nullptr
    // host pointers to the pool's CUtensorMaps ([rows][head_dim] bf16, [16][64] boxes); nullptr when it has none
    const void* k_map;
    const void* v_map;
    int32_t* status;             // dense calls: optional device word for FLAG_WAIT_TIMEOUT (paged calls use the pool's)
};
cudaError_t launch_attn_generic(const DenseAttnLaunch& a, cudaStream_t stream);
// Tensor-core (tcgen05) causal prefill; returns cudaErrorNotSupported when the shape is outside its cover.
cudaError_t launch_attn_tc(const DenseAttnLaunch& a, cudaStream_t stream);

struct RopeRowsLaunch {
    const void* x_in;
    void* x_out;
    const int32_t* positions;
    const float* inv_freq;
    int32_t n_rows, n_heads, head_dim, dtype;
    int64_t stride_row, stride_head;
    float scaling;
};
cudaError_t launch_rope_rows(const RopeRowsLaunch& r, cudaStream_t stream);

// Front half of a decode call without any allocation: validates the arguments against the pool's host
// state, orders the call after pending page transfers, uploads seq_ids / q_pos through the pool's
// staging ring and fills every field of *d except the split plan and the workspace pointers.
// *launchable is 0 for bookkeeping-only pools.
int32_t prepare_decode(skv_pool* pool, int32_t layer, const int32_t* seq_ids, int32_t n_seqs, const int32_t* q_pos,
                       int32_t n_q_heads, const void* q, void* out, float eps, cudaStream_t stream, DecodeLaunch* d,
                       int64_t* total_tokens, int32_t* launchable);
int32_t pool_fail(skv_pool* pool, int32_t code, const char* message);
int32_t pool_device(const skv_pool* pool);

cudaError_t launch_merge_partials(const float* parts, int32_t n_parts, int64_t part_stride, int32_t n_rows, int32_t head_dim,
                                  float eps, void* out, int32_t dtype, cudaStream_t stream);

// Process-wide A/B switches, read from the environment once (and again on skv_reload_env).
struct Switches {
    int step_fused;        // SKV_STEP_FUSED != "0"
    int decode_generic;    // SKV_DECODE_GENERIC == "1"
    int impl_reg;          // SKV_DECODE_IMPL starts with 'r'
    int stages;            // SKV_DECODE_STAGES (2 when unset)
    int chunk;             // SKV_DECODE_CHUNK (0 when unset)
    int fuse;              // SKV_DECODE_FUSE: -1 unset, 0, 1
    int prefill_generic;   // SKV_PREFILL_GENERIC == "1"
    int append_scalar;     // SKV_APPEND_SCALAR == "1"
    int pdl;               // SKV_PDL != "0"
    int step_early;        // SKV_STEP_EARLY != "0"
    int order;             // SKV_DECODE_ORDER: -1 unset (longest rows first when the grid exceeds the GPU), 0 never, 1 always
};
const Switches& switches();
void reload_switches();

// process-wide count of kernel launches issued by this library
void count_launches(int n);

inline size_t dtype_size(int32_t dtype) { return dtype == SKV_BF16 ? 2 : 4; }

}  // namespace skv
