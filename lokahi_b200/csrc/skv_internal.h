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

// Output gather fused into the merge kernel: every rank stores its output rows straight into all ranks'
// gathered buffers over NVLink (plain peer stores) and then raises its flag on each peer.
struct PeerGatherView {
    int32_t world;               // 0: no gather, the merge kernel writes `out`
    int32_t rank;
    int32_t epoch;               // value written to the flags when this call's rows have landed
    int32_t* ticket;             // device counter of finished merge blocks (zero between calls)
    void* out[8];                // per rank: base of its gathered buffer [world][n_seqs][q_heads][head_dim]
    int32_t* flags[8];           // per rank: its flag array [world]
    const int32_t* wait_flags;   // this rank's own flag array: when set, the merge kernel's last block also waits
                                 // (bounded) until every rank's slice of this epoch has landed here
};

struct DecodeLaunch {
    PoolView pool;
    int32_t layer, n_seqs, n_q_heads, dtype;
    const int32_t* seq_ids;      // device or nullptr (identity)
    const int32_t* q_pos;        // device or nullptr (length - 1)
    const void* q;
    void* out;
    float eps;
    float* ws_acc;               // [n_seqs][n_q_heads][max_splits][head_dim]
    float* ws_ml;                // [n_seqs][n_q_heads][max_splits][2]
    int32_t max_splits, chunk_tokens;
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
    PeerGatherView gather;
    float* partial_out;          // when set, the merge kernel writes un-normalised [n_seqs][q_heads][head_dim + 2]
                                 // rows (acc..., m, l) instead of the output: the unit of sequence sharding
    // Fused append (one decode step, identity batch, bf16 TMA kernel only): the device lengths still hold the
    // count BEFORE this step's token.  Every CTA rotates its own copy of q at position `length`; the CTA whose
    // chunk contains that position rotates the new K row, stores it and the V row into the page, and attends
    // the token from registers; the merge kernel writes the rotated q back and bumps the lengths.
    int32_t fused_append;
    const void* new_k;           // [n_seqs][kv_heads][head_dim], un-rotated
    const void* new_v;
    const float* inv_freq;       // [head_dim / 2]
    float rope_scaling;
    int32_t* append_ticket;      // one counter, zero between calls
};
cudaError_t launch_decode(const DecodeLaunch& d, cudaStream_t stream);
// chunk length (tokens handled by one CTA) and the number of splits that follow from it
void decode_plan(int32_t page_size, int32_t max_pages_per_seq, int32_t n_seqs, int32_t num_kv_heads,
                 int64_t total_tokens_hint, int32_t* chunk_tokens, int32_t* max_splits);

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
cudaError_t launch_gather_wait(const int32_t* flags, int32_t world, int32_t epoch, int32_t* status, cudaStream_t stream);

// process-wide count of kernel launches issued by this library
void count_launches(int n);

inline size_t dtype_size(int32_t dtype) { return dtype == SKV_BF16 ? 2 : 4; }

}  // namespace skv
