/*
 * strata_b200.h -- C ABI of the B200 (sm_100a) paged KV-cache / RoPE / grouped-query
 * attention library (libstrata_b200.so).
 *
 * Every entry point returns an int32 status (SKV_OK == 0, negatives are errors),
 * never throws and never aborts.  Host-side validation happens before any kernel
 * launch; skv_last_error() gives the message of the last failing call on a pool.
 * Device pointers are borrowed for the duration of the call on the given stream;
 * the library never frees caller memory.  `stream` is a cudaStream_t passed as
 * void* (NULL = the legacy default stream).  Calls that change page tables or lengths publish the
 * change to the device on the stream they are given; a pool is driven from one stream at a time
 * (hand it from one stream to another with an event, as with any buffer).
 *
 * Each declaration cites the interface of the reference project (Strata,
 * Python package `ollm`) that it stands in for, as  path:line  inside that project.
 */
#ifndef STRATA_B200_H
#define STRATA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define SKV_API __attribute__((visibility("default")))
#else
#define SKV_API
#endif

#define SKV_ABI_VERSION 2

/* status codes */
enum {
    SKV_OK = 0,
    SKV_ERR_BAD_ARG = -1,       /* shape / index / pointer validation failed (ValueError in the reference) */
    SKV_ERR_REPLAY = -2,        /* append does not start exactly after the cached sequence
                                   (src/ollm/mlx_kvcache.py:143-158, "append exactly") */
    SKV_ERR_OUT_OF_PAGES = -3,  /* page / sequence / host-slot allocator exhausted; nothing was changed */
    SKV_ERR_NOT_RESIDENT = -4,  /* a page needed by the call is parked in host memory */
    SKV_ERR_TIMEOUT = -5,       /* bounded wait ran out */
    SKV_ERR_CUDA = -6,          /* a CUDA runtime call failed; message holds cudaGetErrorString */
    SKV_ERR_UNSUPPORTED = -7,   /* shape or dtype outside what the kernels cover */
    SKV_ERR_DEVICE_FLAG = -8    /* a kernel recorded an error in the pool's device status word */
};

/* element types of stored K/V, queries and outputs */
enum { SKV_F32 = 0, SKV_BF16 = 1 };

/* page-table entry encoding (int32): >= 0 device page, -1 unassigned, -2 - s = parked in host slot s */
#define SKV_PAGE_UNASSIGNED (-1)

typedef struct skv_pool skv_pool;

typedef struct skv_config {
    int32_t device;            /* CUDA device ordinal; -1 = bookkeeping only (no device memory, no launches) */
    int32_t dtype;             /* SKV_F32 or SKV_BF16 */
    int32_t num_layers;        /* config.num_hidden_layers of the reference cache ctor (mlx_kvcache.py:31-63) */
    int32_t num_kv_heads;      /* KV heads held by THIS pool (the local heads under KV-head sharding) */
    int32_t head_dim;
    int32_t page_size;         /* tokens per page */
    int32_t num_pages;         /* device pages; one page id covers all layers and local KV heads */
    int32_t max_seqs;
    int32_t max_pages_per_seq;
    int32_t host_pages;        /* pinned host slots for parked pages (0 = no host tier) */
} skv_config;

/* Pool life cycle.  Stands in for MLXKVCache.__init__ / clear (mlx_kvcache.py:31-63, 271-284).
 * Device layout per layer: K[page][kv_head][page_size][head_dim], V likewise. */
/* A sequence may hold at most SKV_MAX_TOKENS_PER_SEQ tokens (the split-K plan gives a sequence at most 128
 * chunks of 2048 tokens): skv_create refuses a pool whose max_pages_per_seq * page_size exceeds it with
 * SKV_ERR_UNSUPPORTED (on failure *out still holds a handle for skv_last_error; destroy it). */
#define SKV_MAX_TOKENS_PER_SEQ 262144
SKV_API int32_t skv_abi_version(void);
SKV_API int32_t skv_create(const skv_config* cfg, skv_pool** out);
/* The SKV_* environment switches (A/B aids) are read once, at the first call that needs one; this reads them
 * again.  No reference counterpart. */
SKV_API void skv_reload_env(void);
SKV_API int32_t skv_destroy(skv_pool* pool);
SKV_API const char* skv_last_error(const skv_pool* pool);
SKV_API const char* skv_status_string(int32_t status);
/* Number of kernels this library has launched in this process so far (all pools, all streams).
 * No reference counterpart; lets a caller state how much work really ran on the GPU. */
SKV_API int64_t skv_launch_count(void);

/* Sequences.  The reference keeps one tensor per layer with a batch axis (mlx_kvcache.py:54);
 * here each batch row is a sequence with its own page-table row and per-layer lengths. */
SKV_API int32_t skv_alloc_sequence(skv_pool* pool, int32_t* seq_out);
/* The three calls below change the device copy of the page table / lengths on `stream`, in order with the
 * kernels enqueued there before and after them. */
SKV_API int32_t skv_free_sequence(skv_pool* pool, int32_t seq, void* stream);
SKV_API int32_t skv_reserve(skv_pool* pool, int32_t seq, int32_t total_tokens, void* stream);
/* Adopt an externally chosen page-table row (validated: range, no page shared with a live sequence)
 * and set every layer's length to `length`.  No reference counterpart. */
SKV_API int32_t skv_set_page_table(skv_pool* pool, int32_t seq, const int32_t* pages, int32_t n_pages, int32_t length,
                                   void* stream);

/* Shorten one layer's history of the listed sequences to `new_length` tokens; pages stay owned.
 * Used when a layer is dropped to a file and later re-appended from position 0
 * (the reference deletes the layer's tensors, mlx_kvcache.py:220-222). */
SKV_API int32_t skv_truncate(skv_pool* pool, int32_t layer, const int32_t* seq_ids, int32_t n_seqs,
                             int32_t new_length, void* stream);

/* Queries on host-side state: get_seq_length (mlx_kvcache.py:160-172). */
SKV_API int32_t skv_length(const skv_pool* pool, int32_t layer, int32_t seq, int32_t* length_out);
SKV_API int32_t skv_lengths(const skv_pool* pool, int32_t layer, int32_t* out, int32_t n);
SKV_API int32_t skv_page_table(const skv_pool* pool, int32_t seq, int32_t* out, int32_t capacity, int32_t* n_pages_out);
SKV_API int32_t skv_pool_counters(const skv_pool* pool, int64_t out[8]);
/*   out[0] free device pages, [1] used device pages, [2] free host slots, [3] pages evicted (total),
 *   [4] pages prefetched (total), [5] bytes device->host, [6] bytes host->device, [7] live sequences */

/* Raw device views, for tests and for host code that fills a pool directly. */
SKV_API int32_t skv_pool_pointers(const skv_pool* pool, int32_t layer, void** k_pool, void** v_pool);
SKV_API int32_t skv_device_tables(const skv_pool* pool, int32_t** page_table, int32_t** lengths);

/* RoPE table: inv_freq[head_dim/2] float32 exactly as MLXRotaryEmbedding builds it
 * (src/ollm/llama_mlx.py:111-114); positions are divided by `scaling_factor` first
 * (linear scaling; the reference has none, 1.0 reproduces it). */
SKV_API int32_t skv_set_rope(skv_pool* pool, const float* inv_freq, int32_t n, float scaling_factor);

/* K1: append `n_new` tokens per sequence to one layer (MLXKVCache.update, mlx_kvcache.py:65-125),
 * optionally rotating K (and a query tensor) on the way in
 * (apply_rotary_pos_emb_mlx, llama_mlx.py:149-182). */
typedef struct skv_append_args {
    int32_t layer;
    int32_t n_seqs;
    const int32_t* seq_ids;     /* host, n_seqs entries; NULL = sequences 0..n_seqs-1 */
    const int32_t* start_pos;   /* host, n_seqs entries; must equal each sequence's length in this layer.
                                   NULL = append at the current length (no replay check, as when the
                                   reference is called without cache_position) */
    int32_t n_new;              /* tokens appended per sequence */
    const void* k;              /* device, element strides below, head_dim contiguous */
    const void* v;
    int64_t kv_stride_seq, kv_stride_head, kv_stride_tok;   /* in elements */
    int32_t rope_k;             /* 1: rotate K with the pool's table at positions start..start+n_new */
    /* optional query rotation in the same launch (q_out may alias q_in) */
    const void* q_in;
    void* q_out;
    int32_t n_q_heads;
    int64_t q_stride_seq, q_stride_head, q_stride_tok;
} skv_append_args;
SKV_API int32_t skv_append(skv_pool* pool, const skv_append_args* args, void* stream);

/* K2: materialise the dense [n_seqs][kv_heads][max_len][head_dim] history of a layer
 * (what update returns / __getitem__ holds, mlx_kvcache.py:125, 290-303).  Rows beyond a
 * sequence's length are zero-filled. */
SKV_API int32_t skv_gather(skv_pool* pool, int32_t layer, const int32_t* seq_ids, int32_t n_seqs,
                   void* out_k, void* out_v, int32_t max_len, void* stream);

/* K3: one query token per sequence against its paged history
 * (online_chunked_grouped_attention_mx with Lq == 1, src/ollm/backends/mlx_ops.py:32-152;
 * call site llama_mlx.py:300-308).  q, out: [n_seqs][n_q_heads][head_dim], pool dtype.
 * q_pos (host, may be NULL = length-1) are absolute query positions: keys 0..q_pos are attended.
 * workspace holds the split-K partials: skv_decode_workspace_bytes bytes, 16-byte aligned (a pointer that is not
 * is refused with SKV_ERR_BAD_ARG before anything is launched). */
SKV_API size_t skv_decode_workspace_bytes(const skv_pool* pool, int32_t n_seqs, int32_t n_q_heads);
SKV_API int32_t skv_decode_attn(skv_pool* pool, int32_t layer, const int32_t* seq_ids, int32_t n_seqs,
                        const void* q, void* out, const int32_t* q_pos, int32_t n_q_heads,
                        float eps, void* workspace, size_t workspace_bytes, void* stream);

/* Exchange between GPUs fused into the merge kernel (no reference counterpart: the reference is single-device; it
 * loops over its KV heads and concatenates their results, mlx_ops.py:81-87, :152, and merges key chunks with the
 * rule of :125-146).  Every rank passes the same description with its own `rank`:
 *   SKV_XCHG_HEAD_GATHER  KV-head sharding: rank r holds KV heads [r*Hkv/N, (r+1)*Hkv/N) and their query heads; its
 *       merge kernel stores each finished row into slot r of every rank's receive buffer and unpacks all slots into
 *       `out` [world][n_seqs][n_q_heads][head_dim] (n_q_heads = this rank's heads).
 *   SKV_XCHG_SEQ_MERGE    sequence sharding: every rank holds all heads and a share of every sequence's tokens; the
 *       un-normalised partial row (acc, m, l) goes to the row's owner (row % world), which merges the `world`
 *       partials and sends the finished row to every rank; `out` is [n_seqs][n_q_heads][head_dim].
 * recv_ptrs[r] is rank r's receive buffer as seen from this rank (peer-mapped device memory: CUDA IPC, symmetric
 * memory ...), skv_exchange_bytes long, 16-byte aligned and zero-filled before the first call.  `epoch` starts at 1
 * and grows by one per call on every rank alike (the two halves of a buffer alternate by its parity).  Data crosses
 * NVLink as 16-byte stores whose 8-byte halves each carry the epoch, so the receiver needs no flag and no fence; the
 * merge kernel of a call waits (bounded, about a second; a timeout sets bit 8 of the pool's status word) for the
 * rows it unpacks, and work enqueued after the call sees the complete `out`.  head_dim * element size must be a
 * multiple of 8 and world at most 8. */
enum { SKV_XCHG_HEAD_GATHER = 1, SKV_XCHG_SEQ_MERGE = 2 };
typedef struct skv_exchange {
    int32_t mode, rank, world;
    uint32_t epoch;
    void* const* recv_ptrs;       /* host array, world entries */
    void* out;                    /* this rank's result buffer */
} skv_exchange;
SKV_API size_t skv_exchange_bytes(int32_t mode, int32_t world, int32_t n_seqs, int32_t n_q_heads, int32_t head_dim,
                                  int32_t dtype);
/* skv_decode_attn with the exchange in place of `out`. */
SKV_API int32_t skv_decode_attn_xchg(skv_pool* pool, int32_t layer, const int32_t* seq_ids, int32_t n_seqs,
                                     const void* q, const int32_t* q_pos, int32_t n_q_heads, float eps,
                                     void* workspace, size_t workspace_bytes, const skv_exchange* xchg, void* stream);

/* K1 + K3 in one call for the cached decode step of a layer: rotate q (in place) and the new k with the pool's
 * RoPE table, append k, v at each sequence's current length, then attend
 * (the sequence apply_rotary_pos_emb_mlx -> cache.update -> attention of src/ollm/llama_mlx.py:284-308 for L == 1).
 * For bf16, head_dim 128, page_size a multiple of 16 and at most 8 query heads per KV head the whole step is two
 * launches: the split-K kernel rotates q and the new k itself, stores the new rows into their page and attends
 * them from shared memory; the merge kernel writes the rotated q back, sets the device lengths and runs the
 * exchange.  The stored pages and the rotated q are bit-identical to the append + attention pair; the output
 * differs from it by rounding only (the new token's weight stays in float32).  SKV_STEP_FUSED=0 in the
 * environment selects the pair.  On any error nothing was launched and the pool's host state is unchanged. */
typedef struct skv_step_args {
    int32_t layer, n_seqs;
    const int32_t* seq_ids;       /* host, n_seqs live distinct sequences; NULL = 0..n_seqs-1.  Row i of q, k, v, out
                                     belongs to seq_ids[i] */
    void* q;                      /* row i at q + i * q_row_stride elements: [n_q_heads][head_dim]; rotated in place */
    const void* k;                /* row i at k + i * k_row_stride: [kv_heads][head_dim], un-rotated */
    const void* v;
    void* out;                    /* row i at out + i * out_row_stride: [n_q_heads][head_dim]; ignored with xchg */
    int64_t q_row_stride, k_row_stride, v_row_stride, out_row_stride;   /* elements; 0 = rows packed back to back.
                                     With strides q, k and v can be slices of one fused projection output
                                     [n_seqs][(n_q_heads + 2 * kv_heads) * head_dim] (llama_mlx.py:257-281) */
    int32_t n_q_heads;
    float eps;
    void* workspace;              /* as for skv_decode_attn */
    size_t workspace_bytes;
    const skv_exchange* xchg;     /* NULL: the result goes to `out` */
    float* partial_out;           /* when set (and xchg is NULL): un-normalised float32 rows [n_seqs][n_q_heads][head_dim + 2]
                                     as skv_decode_partial writes them, instead of `out` */
    /* Sequence sharding: this pool holds only a share of every sequence's tokens.  positions[i] is the absolute
     * position of the step's token (its RoPE angle) and store[i] != 0 says that this pool keeps it.  NULL, NULL:
     * the position is the row's length in this pool and every row is stored (the single-pool case). */
    const int32_t* positions;     /* host */
    const uint8_t* store;         /* host */
    /* SKV_STEP_CONSECUTIVE: the caller states that (1) nothing was enqueued on `stream` since this pool's previous
     * skv_decode_step* call on it, and (2) q, k, v and the pool's pages were complete before that call was made
     * (they are not outputs of it).  When that previous call was a step of the same layer over the same sequences in
     * the same order, the split-K kernel of this step then runs beside the previous step's kernels: it starts while
     * that step's last blocks drain, waits (bounded) for a per-(sequence, head) flag before it reads the one page row
     * that step stored, and waits for that step's merge kernel and exchange only where it stores its own partials.
     * The library drops the flag by itself when the previous call on this pool was not such a step on the same
     * stream, when a page-table update has to run between the two, or when q, k, v overlap what that step wrote
     * (its rotated q, its output).  SKV_STEP_EARLY=0 in the environment drops it always. */
    uint32_t flags;
} skv_step_args;
#define SKV_STEP_CONSECUTIVE 1u
SKV_API int32_t skv_decode_step_ex(skv_pool* pool, const skv_step_args* args, void* stream);
/* Short forms of skv_decode_step_ex: packed rows, sequences 0..n_seqs-1 (skv_decode_step), an explicit list
 * (skv_decode_step_seqs), and the list plus an exchange (skv_decode_step_xchg). */
SKV_API int32_t skv_decode_step(skv_pool* pool, int32_t layer, int32_t n_seqs, void* q, const void* k, const void* v,
                                void* out, int32_t n_q_heads, float eps, void* workspace, size_t workspace_bytes,
                                void* stream);
SKV_API int32_t skv_decode_step_seqs(skv_pool* pool, int32_t layer, const int32_t* seq_ids, int32_t n_seqs, void* q,
                                     const void* k, const void* v, void* out, int32_t n_q_heads, float eps,
                                     void* workspace, size_t workspace_bytes, void* stream);
SKV_API int32_t skv_decode_step_xchg(skv_pool* pool, int32_t layer, const int32_t* seq_ids, int32_t n_seqs, void* q,
                                     const void* k, const void* v, int32_t n_q_heads, float eps, void* workspace,
                                     size_t workspace_bytes, const skv_exchange* xchg, void* stream);

/* Sequence sharding without the fused exchange (no reference counterpart; the merge is the reference's own
 * chunk-merge rule, src/ollm/backends/mlx_ops.py:125-144, applied across ranks instead of across key blocks).
 * skv_decode_partial: K3 over the keys THIS pool holds, writing un-normalised float32 rows
 *   partial_out[n_seqs][n_q_heads][head_dim + 2] = (weighted V sum relative to m, m, l); q_pos are positions in this
 *   pool's own token numbering (a negative position means "none of my keys": l = 0).
 * skv_merge_partials: merges n_parts (<= 128) such buffers (part p at parts + p * part_stride floats) of n_rows =
 *   n_seqs * n_q_heads rows and writes out[n_rows][head_dim] = wv / max(s, eps) in `dtype`. */
SKV_API int32_t skv_decode_partial(skv_pool* pool, int32_t layer, const int32_t* seq_ids, int32_t n_seqs, const void* q,
                                   const int32_t* q_pos, int32_t n_q_heads, void* workspace, size_t workspace_bytes,
                                   float* partial_out, void* stream);
SKV_API int32_t skv_merge_partials(const float* parts, int32_t n_parts, int64_t part_stride, int32_t n_rows,
                                   int32_t head_dim, float eps, void* out, int32_t dtype, void* stream);

/* K3 without a caller workspace.  This entry point has no counterpart in the reference; it exists for
 * hosts that cannot allocate device memory (a process whose memory is handed out once at start-up,
 * a plugin inside a foreign arena, code that must not trigger a device-synchronising allocation).
 * Same arguments and result as skv_decode_attn, but the split-K partials live in an array of
 * SKV_STATIC_SCRATCH_BYTES that is part of the library image on every GPU that loads it.
 *   - a call whose partials need more than that returns SKV_ERR_UNSUPPORTED (message names both sizes);
 *   - no cudaMalloc / cudaFree / allocating library call is made;
 *   - the first call on a device resolves the array's address: make it outside stream capture;
 *   - all calls on a device share the array; calls that overlap on the GPU race, so order them. */
#define SKV_STATIC_SCRATCH_BYTES (16u << 20)
SKV_API int32_t skv_decode_attn_static(skv_pool* pool, int32_t layer, const int32_t* seq_ids, int32_t n_seqs,
                                       const void* q, void* out, const int32_t* q_pos, int32_t n_q_heads,
                                       float eps, void* stream);

/* K4: chunked grouped-query attention on dense tensors
 * (online_chunked_grouped_attention_mx, mlx_ops.py:32-152; unmasked twin :155-178).
 * q,out [B][Hq][Lq][D], k,v [B][Hkv][Lk][D], contiguous.  positions: device int32 [B][Lq]
 * absolute query positions, or NULL for bottom-right alignment arange(Lk-Lq, Lk) (:69-72).
 * Rows with no allowed key produce 0 (:118, :146).  status (device int32, may be NULL): the tensor-core kernel ORs
 * bit 8 into it when one of its bounded waits ran out (the result is then invalid); the caller zeroes and reads it. */
SKV_API int32_t skv_attn_dense(const void* q, const void* k, const void* v, void* out, const int32_t* positions,
                       int32_t B, int32_t Hq, int32_t Hkv, int32_t Lq, int32_t Lk, int32_t D,
                       int32_t dtype, int32_t causal, float eps, int32_t* status, void* stream);

/* K4 over pages: queries [n_seqs][Hq][Lq][D] against each sequence's first `lengths` tokens of a layer
 * (the attention call of a chunked prefill over the cache, src/ollm/llama_mlx.py:300-308 with L > 1).
 * bf16 pools with head_dim 128 and pages of a multiple of 16 tokens, Lq >= 32 and 16-byte aligned q/out run on the tensor cores and
 * read K/V straight from the pages; every other case takes the float32 CUDA-core kernel.  positions NULL means
 * the bottom-right default (length - Lq + i); SKV_PREFILL_GENERIC=1 forces the CUDA-core kernel. */
SKV_API int32_t skv_prefill_attn_paged(skv_pool* pool, int32_t layer, const int32_t* seq_ids, int32_t n_seqs,
                               const void* q, void* out, const int32_t* positions /* device [n_seqs][Lq] or NULL */,
                               int32_t n_q_heads, int32_t Lq, int32_t causal, float eps, void* stream);

/* K5: park pages in pinned host memory and bring them back
 * (stands in for save_to_disk / _load_layer_from_disk, mlx_kvcache.py:183-255).
 * Slots are page-table slots of one sequence; all layers of a page move together.  Copies run on the
 * pool's own copy streams; skv_wait_resident bounds the wait and returns SKV_ERR_TIMEOUT instead of
 * blocking forever.  Compute on `stream` issued after skv_sync_transfers(pool, stream) is ordered
 * after the copies. */
SKV_API int32_t skv_evict(skv_pool* pool, int32_t seq, int32_t first_slot, int32_t n_slots, void* stream);
SKV_API int32_t skv_prefetch(skv_pool* pool, int32_t seq, int32_t first_slot, int32_t n_slots, void* stream);
SKV_API int32_t skv_sync_transfers(skv_pool* pool, void* stream);
SKV_API int32_t skv_wait_resident(skv_pool* pool, int32_t timeout_ms);

/* Device status word: kernels record out-of-range page ids or lengths there and skip the access.
 * Reads it back (synchronises `stream`), clears it, returns SKV_ERR_DEVICE_FLAG if it was set. */
SKV_API int32_t skv_check_device_status(skv_pool* pool, void* stream, int32_t* flag_out);

/* Stand-alone RoPE on a [n_rows][n_heads][head_dim] tensor with one position per row
 * (apply_rotary_pos_emb_mlx, llama_mlx.py:149-182). positions: device int32 [n_rows]. */
SKV_API int32_t skv_rope_rows(const void* x_in, void* x_out, const int32_t* positions, const float* inv_freq_dev,
                      int32_t n_rows, int32_t n_heads, int32_t head_dim, int64_t stride_row, int64_t stride_head,
                      float scaling_factor, int32_t dtype, void* stream);

/* Decoder glue on either side of the hot path (the callers directly above it; float32 arithmetic, one rounding per
 * output element, storage dtype float32 or bfloat16).
 * skv_rmsnorm: out = weight * (h * rsqrt(mean(h^2) + eps)) per row of [n_rows][hidden]
 *   (MLXRMSNorm, src/ollm/llama_mlx.py:77-92; optimized_rmsnorm, src/ollm/metal_optimizations.py:75-97).
 *   delta == NULL: h = x.  Otherwise h = x + delta, rounded to the storage dtype, and h is also written to
 *   sum_out (may alias x): the residual add that precedes the norm, fused
 *   (optimized_rmsnorm_residual, metal_optimizations.py:100-117).
 * skv_swiglu: out = (gate * sigmoid(gate)) * up over n elements
 *   (MLXLlamaMLP, llama_mlx.py:345-408; optimized_swiglu, metal_optimizations.py:140-157). */
SKV_API int32_t skv_rmsnorm(const void* x, const void* delta, void* sum_out, const void* weight, void* out, int64_t n_rows,
                            int32_t hidden, float eps, int32_t dtype, void* stream);
SKV_API int32_t skv_swiglu(const void* gate, const void* up, void* out, int64_t n, int32_t dtype, void* stream);
/* skv_swiglu over [n_rows][cols] with a row stride (in elements) per operand: gate and up can be the two halves of one
 * fused gate/up projection output [n_rows][2 * cols] (the reference projects them separately, llama_mlx.py:398-406). */
SKV_API int32_t skv_swiglu_rows(const void* gate, const void* up, void* out, int64_t n_rows, int32_t cols,
                                int64_t gate_row_stride, int64_t up_row_stride, int64_t out_row_stride, int32_t dtype,
                                void* stream);

#ifdef __cplusplus
}
#endif
#endif /* STRATA_B200_H */
