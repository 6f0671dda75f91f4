// K4: causal chunked-prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Mathematics: online_chunked_grouped_attention_mx (src/ollm/backends/mlx_ops.py:32-152) for bf16
// tensors with head_dim 128: scores = q.k * D^-0.5, key t allowed for a query row iff t <= q_pos[row]
// (:107-112), online softmax across key tiles with the (max, sum, weighted V) merge of :125-144, and
// out = wv / max(s, eps) so that a row with no allowed key is exactly 0 (:118, :146).
//
// One CTA = 128 query rows of one query head: four softmax warps (thread r owns query row r, which is TMEM
// lane r) plus two warps that issue the MMAs, one for S = Q . K^T and one for O += P . V, so that instruction
// issue to the tensor cores never sits on a softmax warp's path and the two chains of MMAs issue side by side (one
// thread gets an MMA out every 90 to 104 clocks; with a single issuer the next pair's eight S instructions sat
// between a tile's P and its four O instructions).  The O warp also issues the TMA copies of dense K/V in its
// gaps; paged K/V needs four times as many copies and has a warp for them.  An issuing warp runs its loop in
// warp-uniform control flow with only lane 0 enabled on the copy / MMA / commit instructions: the descriptors
// then live in uniform registers.  Measured on B200 with back-to-back MMAs (M128, K16, operands in shared
// memory): 116 clocks per instruction when issued from inside a one-lane branch, 89 issued this way, the same for
// N = 64 and N = 128 (N = 256 runs at the pipe's full rate of 128).  Since N = 64 costs as much as N = 128, the
// scores of TWO 64-key tiles come from one set of N = 128 instructions.
// Per pair of 64-key tiles:
//   TMA   the pair's K tiles -> shared memory, laid out [dim box][tile][64 keys x 128 B] so that they form one
//         128-row K-major operand; V tile by tile (3-D tensor maps [batch*head][token][dim], 128-byte
//         swizzle, rows past the end of a head are zero-filled by the copy engine);
//   MMA 1 S[128x128] = Q[128x128] . K^T        eight tcgen05.mma kind::f16 (N = 128), both operands K-major
//                                              from smem, accumulator in TMEM columns [0, 128): tile 2m in
//                                              [0, 64), tile 2m+1 in [64, 128);
// then per tile:
//   soft  tcgen05.ld S -> registers, scale, mask by the row's absolute position, running max / sum,
//         P = exp2(...) rounded to bf16 and written to shared memory in the swizzled K-major layout;
//   MMA 2 O[128x128] += P[128x64] . V[64x128]  four MMAs, V is the MN-major B operand straight from the TMA box
//                                              (two-stage ring); the accumulator stays in TMEM columns
//                                              [128, 256) for the whole key loop.
//   As soon as the softmax threads hold the pair's second tile in registers they say so (bar_r) and the next
//   pair's MMA 1 is issued, so it overlaps that tile's softmax.
//   The running maximum that scales P and O is raised only when a tile's maximum exceeds it by more than
//   8 in the log2 domain; only then is O read, scaled and written back (tcgen05.ld / tcgen05.st).  The
//   final division by the row sum makes the stale maximum cancel exactly.
// Two CTAs fit on an SM (112 KB shared memory each, 256 TMEM columns each), so one CTA's softmax overlaps the
// other's MMAs.  Completion travels through mbarriers (tcgen05.commit), every wait is bounded, and on a
// timeout the CTA records FLAG_WAIT_TIMEOUT in the caller's status word (when given), stops issuing work,
// frees its TMEM and returns.  No cluster launch and no multicast anywhere.
//
// Paged K/V (the PAGED instantiation): the same kernel reads the history of a sequence straight from the pool's
// 16-token pages.  A 64-key tile is four pages; each page is two boxes [16 tokens][64 dims] of the pool's 2-D
// tensor map, placed 2 KB apart inside the tile's shared-memory region, which gives exactly the layout a
// [64][64] box would have (the 128-byte swizzle depends on the address only).  That is sixteen copies per tile
// instead of four, at 80 to 150 clocks of issue each, so they get a warp of their own; it reads each
// page-table entry once (K is fetched a pair of tiles ahead, V a tile ahead).  Slots past the sequence's pages
// are read from page 0 and masked.  Measured at 4096 tokens, pages in a random order: 0.159 ms against 0.147 ms
// for dense K/V.
#include <cstdlib>

#include "common.cuh"
#include "tma.cuh"

namespace skv {

namespace {

constexpr int kBM = 128;          // query rows per CTA
constexpr int kBN = 64;           // keys per tile
constexpr int kD = 128;           // head_dim
constexpr int kSoftmaxWarps = 4;   // one query row per thread
// Helper warps behind the softmax warps.  Dense K/V: one that issues the MMAs of S = Q . K^T and one that issues the
// MMAs of O += P . V and, in the gaps, the four TMA copies of a tile (six warps: 168 registers per thread at two CTAs
// per SM).  Paged K/V: sixteen copies per tile, which get a warp of their own in front of the two issuers.
constexpr int kThreadsDense = (kSoftmaxWarps + 2) * 32;
constexpr int kThreadsPaged = (kSoftmaxWarps + 3) * 32;
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0;     // S of a pair of tiles: 64 fp32 columns each, [0,64) and [64,128), written by one N = 128 MMA set
constexpr uint32_t kColO = 128;   // O accumulator: 128 fp32 columns
constexpr float kLog2eF = 1.4426950408889634f;

// shared memory map (offsets from a 1024-byte aligned base)
constexpr int kOffQ = 0;                       // 2 boxes [128 rows][64 dims]   = 32 KB
constexpr int kOffK = kOffQ + 2 * kBM * 128;   // [2 dim boxes][2 tiles of the pair][64 keys x 128 B] = 32 KB
constexpr int kVStage = 2 * kBN * 128;         // bytes of one K or V stage
constexpr int kOffV = kOffK + 2 * kVStage;     // 2 stages x 2 boxes [64 keys][64 dims] = 32 KB
constexpr int kOffP = kOffV + 2 * kVStage;     // [128 rows][64 keys] bf16      = 16 KB
constexpr int kOffBar = kOffP + kBM * 128;     // mbarriers + TMEM base + flags
constexpr int kSmemBytes = kOffBar + 128;       // the dynamic shared-memory base is 1024-byte aligned (checked in the kernel)

// ---- tcgen05 wrappers -------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float max3(float a, float b, float c) {
    float y;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
    return y;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// D[tmem] (+)= A[smem] . B[smem].  The whole issuer warp executes the call in uniform control flow, so that the
// descriptors live in uniform registers; only the lane with `lead` != 0 issues the instruction.  (Measured on
// B200 with a loop of back-to-back MMAs: issued from inside a one-lane branch an M128 N128 K16 MMA costs 116
// clocks, issued this way 89; N = 64 costs the same, N = 256 runs at the pipe's full rate of 128.)
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
                                        uint32_t lead) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(lead)
        : "memory");
}
// Arrive on `bar` once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
    uint32_t* r = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
    const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle (descriptor version 1).
//   K-major operand  (rows of 128 bytes, 8-row groups 1024 bytes apart):  lbo = 16 (unused), sbo = 1024
//   MN-major operand (64-element groups `lbo` bytes apart along MN, 8-row k-groups `sbo` bytes apart)
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;   // version
    d |= (uint64_t)2 << 61;   // SWIZZLE_128B
    return d;
}

// Instruction descriptor: bf16 x bf16 -> f32, M = 128, given N, A K-major, B K-major or MN-major.
__host__ __device__ constexpr uint32_t instr_desc(int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(kBM >> 4) << 24);
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int32_t x, int32_t y, int32_t z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}

struct TcParams {
    const int32_t* positions;   // device [B][Lq] or nullptr
    void* out;
    int32_t* status;            // device status word or nullptr
    int32_t B, Hq, Hkv, Lq, Lk, causal;
    float eps;
    // paged K/V (PAGED kernel only): keys and values come from the pool's pages through its 2-D tensor maps
    // ([rows][128] bf16, boxes of [16 tokens][64 dims]); Lk is then the per-sequence length of the layer
    PoolView pool;
    int32_t layer;
    const int32_t* seq_ids;     // device [B] or nullptr (identity)
};

template <bool PAGED>
__global__ void __launch_bounds__(PAGED ? kThreadsPaged : kThreadsDense, 2)
prefill_tc_kernel(TcParams p, const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                  const __grid_constant__ CUtensorMap vmap) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    uint64_t* bar_q = reinterpret_cast<uint64_t*>(smem + kOffBar);
    uint64_t* bar_k = bar_q + 1;       // two stages (the two tiles of a pair)
    uint64_t* bar_v = bar_q + 3;       // two stages
    uint64_t* bar_s = bar_q + 5;       // first MMA of a PAIR of tiles done: S of both tiles is in TMEM, both K stages are free
    uint64_t* bar_o = bar_q + 6;       // two, by tile parity: second MMA of the tile done (P buffer, O and the V stage are free)
    uint64_t* bar_p = bar_q + 8;       // softmax threads -> issuer: P of this tile is in shared memory
    uint64_t* bar_r = bar_q + 9;       // softmax threads -> issuer: S of the pair's second tile is in registers, S may be overwritten
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_q + 10);
    int32_t* sh_limit = reinterpret_cast<int32_t*>(bar_q + 11);   // max over the tile's rows of the allowed-key count
    int32_t* sh_abort = sh_limit + 1;
    if ((smem_u32(smem) & 1023u) != 0) {   // the swizzled layouts need a 1024-byte aligned base
        if (p.status && threadIdx.x == 0) atomicOr(p.status, FLAG_WAIT_TIMEOUT);
        return;
    }

    constexpr int kWarpCopy = PAGED ? kSoftmaxWarps : -1;
    constexpr int kWarpQK = kSoftmaxWarps + (PAGED ? 1 : 0);
    constexpr int kWarpPV = kWarpQK + 1;
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);   // provably warp-uniform for the compiler
    // heavy (late) query tiles first so that the causal triangle balances across SMs
    // (blocks are dispatched x-fastest: all heads' heaviest tiles start first)
    const int q_tile = (int)gridDim.y - 1 - (int)blockIdx.y;
    const int hq = blockIdx.x, b = blockIdx.z;
    const int G = p.Hq / p.Hkv;
    const int hkv = hq / G;
    const int row = q_tile * kBM + tid;
    const int zq = b * p.Hq + hq, zkv = b * p.Hkv + hkv;
    int seq = b, Lk = p.Lk;
    if constexpr (PAGED) {   // the layer's history of sequence `seq`, found through its page-table row
        seq = p.seq_ids ? p.seq_ids[b] : b;
        if (seq < 0 || seq >= p.pool.max_seqs) {   // uniform over the CTA: nothing has been set up yet
            if (tid == 0) atomicOr(p.pool.status, FLAG_BAD_SEQ);
            return;
        }
        Lk = p.pool.lengths[(int64_t)p.layer * p.pool.max_seqs + seq];
        const int cap = p.pool.max_pages_per_seq * p.pool.page_size;
        if (Lk < 0 || Lk > cap) {
            if (tid == 0) atomicOr(p.pool.status, FLAG_BAD_LENGTH);
            Lk = Lk < 0 ? 0 : cap;
        }
    }

    // number of keys this row may attend: keys 0 .. min(Lk, q_pos + 1)
    int limit = 0;
    if (row < p.Lq && warp < kSoftmaxWarps) {
        limit = Lk;
        if (p.causal) {
            const int qpos = p.positions ? p.positions[(int64_t)b * p.Lq + row] : (Lk - p.Lq + row);
            const int lim = qpos < 0 ? 0 : qpos + 1;
            limit = lim < Lk ? lim : Lk;
        }
    }
    if (tid == 0) {
        *sh_limit = 0;
        *sh_abort = 0;
        mbar_init(bar_q, 1);
        mbar_init(&bar_k[0], 1);
        mbar_init(&bar_k[1], 1);
        mbar_init(&bar_v[0], 1);
        mbar_init(&bar_v[1], 1);
        mbar_init(bar_s, 1);
        mbar_init(bar_r, kSoftmaxWarps);          // one arrival per softmax warp
        mbar_init(&bar_o[0], 1);
        mbar_init(&bar_o[1], 1);
        mbar_init(bar_p, kSoftmaxWarps);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    atomicMax(sh_limit, limit);
    __syncthreads();
    const uint32_t tmem_base = *tmem_slot;
    const int n_tiles = (*sh_limit + kBN - 1) / kBN;

    // K lives as [dim box][stage][64 keys x 128 B]: the two stages of a box are contiguous, so that the two tiles
    // of a pair form one 128-row K-major operand and their scores come from ONE set of N = 128 MMAs.
    // Paged K/V: row, in the pool map's row numbering, of a group of 16 tokens of this KV head (pages hold a multiple
    // of 16 tokens).  A slot the sequence does not have is read from page 0 instead: the bytes are finite (the pool starts zeroed and only
    // ever holds K/V values) and every key at or past the length is masked, so they never reach the output.
    auto group_row = [&](int t) -> int {   // t: first token of a group of 16 (a group never straddles a page)
        const PoolView& pv = p.pool;
        const int slot = t / pv.page_size;
        int page = 0;
        if (slot < pv.max_pages_per_seq) {
            const int id = __ldg(pv.page_table + (int64_t)seq * pv.max_pages_per_seq + slot);
            if (id >= 0 && id < pv.num_pages)
                page = id;
            else if (t < Lk)
                atomicOr(pv.status, FLAG_BAD_PAGE);   // a page inside the history is missing: flagged, not dereferenced
        }
        return (int)((int64_t)p.layer * (pv.layer_stride_bytes / (kD * 2))) + (page * pv.num_kv_heads + hkv) * pv.page_size +
               (t - slot * pv.page_size);
    };
    auto tile_rows = [&](int j, int* y) {   // the four 16-token groups of tile j: four independent loads in flight
#pragma unroll
        for (int sub = 0; sub < 4; ++sub) y[sub] = group_row(kBN * j + 16 * sub);
    };
    auto load_k = [&](int j, const int* y) {
        uint8_t* dst = smem + kOffK + (j & 1) * (kBN * 128);
        mbar_expect_tx(&bar_k[j & 1], 2 * kBN * 128);
        if constexpr (PAGED) {
#pragma unroll
            for (int sub = 0; sub < 4; ++sub) {
                tma_load_2d(dst + sub * 2048, &kmap, 0, y[sub], &bar_k[j & 1]);
                tma_load_2d(dst + 2 * kBN * 128 + sub * 2048, &kmap, 64, y[sub], &bar_k[j & 1]);
            }
        } else {
            tma_load_3d(dst, &kmap, 0, j * kBN, zkv, &bar_k[j & 1]);
            tma_load_3d(dst + 2 * kBN * 128, &kmap, 64, j * kBN, zkv, &bar_k[j & 1]);
        }
    };
    auto load_v = [&](int j, const int* y) {
        uint8_t* dst = smem + kOffV + (j & 1) * kVStage;
        mbar_expect_tx(&bar_v[j & 1], 2 * kBN * 128);
        if constexpr (PAGED) {
#pragma unroll
            for (int sub = 0; sub < 4; ++sub) {
                tma_load_2d(dst + sub * 2048, &vmap, 0, y[sub], &bar_v[j & 1]);
                tma_load_2d(dst + kBN * 128 + sub * 2048, &vmap, 64, y[sub], &bar_v[j & 1]);
            }
        } else {
            tma_load_3d(dst, &vmap, 0, j * kBN, zkv, &bar_v[j & 1]);
            tma_load_3d(dst + kBN * 128, &vmap, 64, j * kBN, zkv, &bar_v[j & 1]);
        }
    };
    // m_run is the maximum the stored numbers are scaled by.  It is only raised when a tile's maximum exceeds
    // it by more than 8 (log2 domain), so P stays below 2^8 and the accumulator in TMEM is rescaled rarely.
    float m_run = -INFINITY, l_run = 0.f;
    const float sc = rsqrtf((float)kD) * kLog2eF;
    const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t q_addr = smem_u32(smem + kOffQ), k_addr = smem_u32(smem + kOffK);
    const uint32_t v_addr = smem_u32(smem + kOffV), p_addr = smem_u32(smem + kOffP);
    constexpr uint32_t kIdescS = instr_desc(2 * kBN, 0);   // a pair of tiles per instruction
    constexpr uint32_t kIdescO = instr_desc(kD, 1);
    bool ok = true;

    if (PAGED && warp == kWarpCopy) {
        // =============================== producer warp (paged K/V): TMA copies ===============================
        // A tile of 16-token pages is eight copies for K and eight for V, and a copy costs its issuing thread 80
        // to 150 clocks.  The K stages are refilled for the next pair as soon as the pair's first MMA has
        // completed, a V stage as soon as the second MMA that read it has.
        if (lane == 0 && n_tiles > 0) {
            mbar_expect_tx(bar_q, 2 * kBM * 128);
            tma_load_3d(smem + kOffQ, &qmap, 0, q_tile * kBM, zq, bar_q);
            tma_load_3d(smem + kOffQ + kBM * 128, &qmap, 64, q_tile * kBM, zq, bar_q);
            // paged: page rows of the current pair of tiles and of the next one; K is fetched a pair ahead, V a
            // tile ahead, so every page-table entry is read once and serves both
            int y_cur[2][4], y_next[2][4];
            if constexpr (PAGED) {
                tile_rows(0, y_cur[0]);
                tile_rows(1, y_cur[1]);
            }
            load_k(0, y_cur[0]);
            load_k(1, y_cur[1]);      // always a whole pair: rows the sequence does not have are zero-filled (dense) or read from page 0, and masked
            load_v(0, y_cur[0]);
            if (n_tiles > 1) load_v(1, y_cur[1]);
            for (int m = 0; 2 * m < n_tiles && ok; ++m) {
                const int j0 = 2 * m, j1 = 2 * m + 1;
                const bool next_pair = 2 * (m + 1) < n_tiles;
                if (next_pair) {
                    if constexpr (PAGED) {
                        tile_rows(j0 + 2, y_next[0]);
                        tile_rows(j0 + 3, y_next[1]);
                    }
                    ok = mbar_wait(bar_s, (uint32_t)(m & 1));      // the pair's first MMA is done: both K stages are free
                    if (!ok) break;
                    load_k(j0 + 2, y_next[0]);
                    load_k(j0 + 3, y_next[1]);
                }
                if (j0 >= 1 && j0 + 1 < n_tiles) {     // V stage (j0+1)&1 was read by the second MMA of tile j0-1
                    ok = mbar_wait(&bar_o[(j0 - 1) & 1], (uint32_t)(((j0 - 1) >> 1) & 1));
                    if (!ok) break;
                    load_v(j0 + 1, y_cur[1]);
                }
                if (j1 + 1 < n_tiles) {                // V stage (j1+1)&1 was read by the second MMA of tile j1-1
                    ok = mbar_wait(&bar_o[(j1 - 1) & 1], (uint32_t)(((j1 - 1) >> 1) & 1));
                    if (!ok) break;
                    load_v(j1 + 1, y_next[0]);
                }
                if constexpr (PAGED) {
#pragma unroll
                    for (int sub = 0; sub < 4; ++sub) {
                        y_cur[0][sub] = y_next[0][sub];
                        y_cur[1][sub] = y_next[1][sub];
                    }
                }
            }
            if (!ok) *sh_abort = 1;
        }
    } else if (warp == kWarpQK) {
        // =============================== first issuer warp: S = Q . K^T ===============================
        // The whole warp runs the loop (uniform control flow keeps the MMA descriptors in uniform registers);
        // lane 0 alone issues the MMAs and the commits.  S of tiles 2m and 2m+1 in one go: eight N = 128 MMAs
        // into columns [0, 128), as soon as the softmax threads hold the previous pair's second tile in registers.
        if (n_tiles > 0) {
            const uint32_t lead = lane == 0 ? 1u : 0u;
            ok = mbar_wait_warp(bar_q, 0);
            for (int m = 0; 2 * m < n_tiles && ok; ++m) {
                ok = ok && mbar_wait_warp(&bar_k[0], (uint32_t)(m & 1));
                ok = ok && mbar_wait_warp(&bar_k[1], (uint32_t)(m & 1));
                if (m > 0) ok = ok && mbar_wait_warp(bar_r, (uint32_t)((m - 1) & 1));
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < kD / 16; ++ks) {
                    const uint32_t blk = (uint32_t)(ks >> 2), in = (uint32_t)(ks & 3) * 32;
                    umma_ss(tmem_base + kColS, smem_desc(q_addr + blk * (kBM * 128) + in, 16, 1024),
                            smem_desc(k_addr + blk * (2 * kBN * 128) + in, 16, 1024), kIdescS, ks > 0 ? 1u : 0u, lead);
                }
                if (lead) umma_commit(bar_s);
                __syncwarp();
            }
            if (!ok) *sh_abort = 1;
        }
    } else if (warp == kWarpPV) {
        // =============================== second issuer warp: O += P . V ===============================
        // One issuing thread gets an MMA out every 90 to 104 clocks, so with a single issuer the pair's eight
        // S instructions sat between a tile's P and its four O instructions; the two chains now issue side by side.
        if (n_tiles > 0) {
            const uint32_t lead = lane == 0 ? 1u : 0u;
            if constexpr (!PAGED) {
                if (lead) {
                    mbar_expect_tx(bar_q, 2 * kBM * 128);
                    tma_load_3d(smem + kOffQ, &qmap, 0, q_tile * kBM, zq, bar_q);
                    tma_load_3d(smem + kOffQ + kBM * 128, &qmap, 64, q_tile * kBM, zq, bar_q);
                    load_k(0, nullptr);
                    load_k(1, nullptr);      // always a whole pair: rows past the end are zero-filled, rows past the limit are masked
                    load_v(0, nullptr);
                    if (n_tiles > 1) load_v(1, nullptr);
                }
                __syncwarp();
            }
            for (int j = 0; j < n_tiles && ok; ++j) {
                // softmax of tile j done: P_j is in shared memory, O has been rescaled where needed
                ok = ok && mbar_wait_warp(bar_p, (uint32_t)(j & 1));
                ok = ok && mbar_wait_warp(&bar_v[j & 1], (uint32_t)((j >> 1) & 1));
                if (!ok) break;
                tc_fence_after();
                const uint32_t vs = v_addr + (uint32_t)(j & 1) * kVStage;
#pragma unroll
                for (int ks = 0; ks < kBN / 16; ++ks)
                    umma_ss(tmem_base + kColO, smem_desc(p_addr + (uint32_t)ks * 32, 16, 1024),
                            smem_desc(vs + (uint32_t)ks * 2048, kBN * 128, 1024), kIdescO, (j > 0 || ks > 0) ? 1u : 0u, lead);
                if (lead) umma_commit(&bar_o[j & 1]);
                __syncwarp();
                if constexpr (!PAGED) {
                    // Dense K/V: this warp also issues the copies, after the MMAs and without further waiting.  The
                    // softmax threads waited for the second MMA of tile j-1 before they wrote P_j, so V stage
                    // (j+1)&1 is free.  K for pair m+1 goes out after tile 2m-1 (pair 1: after tile 0), once the
                    // first MMA of pair m has completed, which frees both K stages: a tile's time before its use.
                    if (lead && j >= 1 && j + 1 < n_tiles) load_v(j + 1, nullptr);
                    const int m_next = j == 0 ? 1 : ((j & 1) ? (j + 3) / 2 : -1);
                    if (m_next > 0 && 2 * m_next < n_tiles) {
                        ok = mbar_wait_warp(bar_s, (uint32_t)((m_next - 1) & 1));
                        if (!ok) break;
                        if (lead) {
                            load_k(2 * m_next, nullptr);
                            load_k(2 * m_next + 1, nullptr);
                        }
                    }
                    __syncwarp();
                }
            }
            if (!ok) *sh_abort = 1;
        }
    } else if (warp < kSoftmaxWarps) {
        // =============================== softmax warps: one query row per thread ===============================
        for (int j = 0; j < n_tiles; ++j) {
            if ((j & 1) == 0) {   // one completion per pair of tiles: the second tile's scores are there already
                ok = mbar_wait_warp(bar_s, (uint32_t)((j >> 1) & 1));
                if (!ok) break;
                tc_fence_after();
            }
            const uint32_t s_col = kColS + (uint32_t)(j & 1) * kBN;
            float s[kBN];
            tmem_ld32(lane_addr + s_col, s);
            tmem_ld32(lane_addr + s_col + 32, s + 32);
            tc_wait_ld();
            if (j & 1) {   // the pair's scores have left tensor memory: the next pair's first MMA may overwrite them
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_r);
            }
            const int t0 = j * kBN;
            if (t0 + kBN > limit) {   // only tiles that cross the row's limit pay for the mask
#pragma unroll
                for (int t = 0; t < kBN; ++t)
                    if (t0 + t >= limit) s[t] = -INFINITY;
            }
            float mx8[8];                              // eight independent chains of three-input maxima
#pragma unroll
            for (int i = 0; i < 8; ++i) mx8[i] = fmaxf(s[i], s[i + 8]);
#pragma unroll
            for (int t = 16; t < kBN; t += 16)
#pragma unroll
                for (int i = 0; i < 8; ++i) mx8[i] = max3(mx8[i], s[t + i], s[t + i + 8]);
            const float mx = max3(max3(mx8[0], mx8[1], mx8[2]), max3(mx8[3], mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])) * sc;   // sc > 0: the scaled maximum
            const bool raise = mx > m_run + 8.0f;               // also true for the first allowed key (m_run = -inf)
            const float m_new = raise ? mx : m_run;
            const float alpha = raise ? ex2(m_run - m_new) : 1.0f;   // ex2(-inf) = 0 when nothing was accumulated yet
            const bool rescale = raise && j > 0 && m_run != -INFINITY;
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;  // row with no allowed key so far: P = 0
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};
            uint32_t pk[kBN / 2];
#pragma unroll
            for (int t = 0; t < kBN; t += 2) {
                const float p0 = ex2(fmaf(s[t], sc, -m_use)), p1 = ex2(fmaf(s[t + 1], sc, -m_use));
                rs4[(t >> 1) & 3] += p0 + p1;
                __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
                pk[t >> 1] = *reinterpret_cast<uint32_t*>(&h2);
            }
            l_run = l_run * alpha + ((rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));
            m_run = m_new;
            // P's buffer and the O accumulator are still in use by the previous tile's second MMA
            if (j > 0) {
                ok = mbar_wait_warp(&bar_o[(j - 1) & 1], (uint32_t)(((j - 1) >> 1) & 1));
                if (!ok) break;
                tc_fence_after();
            }
            if (__any_sync(0xffffffffu, rescale)) {   // warp-uniform: tcgen05.ld/st are warp-wide
                const float f = rescale ? alpha : 1.0f;
#pragma unroll
                for (int cc = 0; cc < kD / 32; ++cc) {
                    float t32[32];
                    tmem_ld32(lane_addr + kColO + cc * 32, t32);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) t32[i] *= f;
                    tmem_st32(lane_addr + kColO + cc * 32, t32);
                }
                tc_wait_st();
            }
            // P row -> shared memory, K-major with the 128-byte swizzle the MMA descriptor expects
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const uint32_t dst = p_addr + (uint32_t)tid * 128 + (((uint32_t)u ^ ((uint32_t)tid & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[4 * u]), "r"(pk[4 * u + 1]),
                             "r"(pk[4 * u + 2]), "r"(pk[4 * u + 3])
                             : "memory");
            }
            fence_proxy_async();          // every lane publishes its own stores to the async proxy,
            tc_fence_before();
            __syncwarp();                 // then one arrival stands for the warp
            if (lane == 0) mbar_arrive(bar_p);
        }
        // wait for the last accumulation
        if (n_tiles > 0 && ok) {
            ok = mbar_wait_warp(&bar_o[(n_tiles - 1) & 1], (uint32_t)(((n_tiles - 1) >> 1) & 1));
            tc_fence_after();
        }
        if (!ok) *sh_abort = 1;
        // ---- epilogue: normalise and store (a CTA whose rows attend nothing writes zeros) ----
        if (ok) {
            const float inv = 1.0f / fmaxf(l_run, p.eps);
            __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + (((int64_t)b * p.Hq + hq) * p.Lq + row) * kD;
#pragma unroll
            for (int cc = 0; cc < kD / 32; ++cc) {
                float t32[32];
                if (n_tiles > 0) {   // uniform over the CTA
                    tmem_ld32(lane_addr + kColO + cc * 32, t32);
                    tc_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) t32[i] = 0.f;
                }
                if (row < p.Lq) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            // a row with no allowed key has l = 0 and only zero-weight products: force an exact 0
                            const float a0 = l_run > 0.f ? t32[8 * u + 2 * i] * inv : 0.f;
                            const float a1 = l_run > 0.f ? t32[8 * u + 2 * i + 1] * inv : 0.f;
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(a0, a1);
                            w[i] = *reinterpret_cast<uint32_t*>(&h2);
                        }
                        *reinterpret_cast<uint4*>(orow + cc * 32 + 8 * u) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    // a wait that ran out anywhere in the CTA invalidates the result: tell the caller
    __syncthreads();
    if (tid == 0 && *sh_abort && p.status) atomicOr(p.status, FLAG_WAIT_TIMEOUT);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

// [batch*heads][tokens][128] bf16, contiguous; box = [1][box_rows][64], 128-byte swizzle.
bool encode_heads_3d(CUtensorMap* map, const void* base, uint64_t n_heads, uint64_t tokens, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[3] = {(cuuint64_t)kD, tokens, n_heads};
    cuuint64_t strides[2] = {(cuuint64_t)kD * 2, tokens * (cuuint64_t)kD * 2};
    cuuint32_t box[3] = {64, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

cudaError_t launch_attn_tc(const DenseAttnLaunch& a, cudaStream_t stream) {
    const bool paged = a.pool.k_base != nullptr;
    const bool aligned = paged ? ((((uintptr_t)a.q | (uintptr_t)a.out) & 15) == 0)
                               : ((((uintptr_t)a.q | (uintptr_t)a.k | (uintptr_t)a.v | (uintptr_t)a.out) & 15) == 0);
    if (a.dtype != SKV_BF16 || a.D != kD || !aligned || a.Lq < 32) return cudaErrorNotSupported;
    // paged K/V: the pool's own tensor maps with [16 tokens][64 dims] boxes, so pages of a multiple of 16 tokens
    if (paged && (a.pool.page_size % 16 != 0 || !a.k_map || !a.v_map || a.pool.head_dim != kD)) return cudaErrorNotSupported;
    if (!paged && a.Lk < 1) return cudaErrorNotSupported;
    alignas(64) CUtensorMap qmap, kmap, vmap;
    if (!encode_heads_3d(&qmap, a.q, (uint64_t)a.B * a.Hq, (uint64_t)a.Lq, kBM)) return cudaErrorNotSupported;
    if (paged) {
        kmap = *reinterpret_cast<const CUtensorMap*>(a.k_map);
        vmap = *reinterpret_cast<const CUtensorMap*>(a.v_map);
    } else if (!encode_heads_3d(&kmap, a.k, (uint64_t)a.B * a.Hkv, (uint64_t)a.Lk, kBN) ||
               !encode_heads_3d(&vmap, a.v, (uint64_t)a.B * a.Hkv, (uint64_t)a.Lk, kBN)) {
        return cudaErrorNotSupported;
    }
    static bool configured[64][2] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev][paged ? 1 : 0]) {
        cudaError_t e = paged ? cudaFuncSetAttribute(prefill_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes)
                              : cudaFuncSetAttribute(prefill_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev][paged ? 1 : 0] = true;
    }
    TcParams p{};
    p.positions = a.positions;
    p.out = a.out;
    p.status = paged ? a.pool.status : a.status;
    p.B = a.B; p.Hq = a.Hq; p.Hkv = a.Hkv; p.Lq = a.Lq; p.Lk = a.Lk; p.causal = a.causal;
    p.eps = a.eps;
    p.pool = a.pool;
    p.layer = a.layer;
    p.seq_ids = a.seq_ids;
    dim3 grid((unsigned)a.Hq, (unsigned)((a.Lq + kBM - 1) / kBM), (unsigned)a.B);
    if (paged)
        prefill_tc_kernel<true><<<grid, kThreadsPaged, kSmemBytes, stream>>>(p, qmap, kmap, vmap);
    else
        prefill_tc_kernel<false><<<grid, kThreadsDense, kSmemBytes, stream>>>(p, qmap, kmap, vmap);
    count_launches(1);
    return cudaGetLastError();
}

}  // namespace skv
