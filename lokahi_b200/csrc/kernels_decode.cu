// K3: split-K flash-decoding grouped-query attention through the page table, and K3r, the
// merge of the split partials.
//
// Mathematics: online_chunked_grouped_attention_mx with one query row
// (src/ollm/backends/mlx_ops.py:81-152): scores = q.k * D^-0.5 in float32, keys 0..q_pos
// allowed, running (max, sum, weighted V) merged across key chunks (:125-144), and
// out = wv / max(s, eps) so that a row with no allowed key is exactly 0 (:118, :146).
//
// Three kernels produce the same partials (m, l, acc[D]) per (sequence, query head, split); the third,
// decode_tma_kernel (described at its definition), is decode_mma_kernel with K/V staged through shared memory
// by TMA and is the default where it applies:
//   * decode_generic_kernel: CUDA cores, float32 or bf16 storage, any head_dim <= 256, any group
//     size; one CTA per query head, so K/V of a KV head are re-read by its G query heads (L2).
//   * decode_mma_kernel: bf16, head_dim 128, group size <= 8.  One CTA serves all G query heads of
//     a KV head, so every K/V byte is read from HBM once.  K and V go from global memory straight
//     into mma.sync fragments with 16-byte loads that cover whole 32-byte sectors: the
//     contraction index of Q.K^T and the column index of P.V are permuted so that each lane's
//     fragment registers are the 16-byte units it loaded (no shared-memory staging, no
//     transposes).  Row maxima and sums are reduced with warp shuffles inside the quad that
//     shares a query row; the four warps of a CTA combine through shared memory.
#include <cstdlib>

#include "common.cuh"
#include "tma.cuh"

namespace skv {

namespace {

constexpr int kDecodeWarps = 4;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ int attend_count(const DecodeLaunch& d, int i, int seq) {
    const PoolView& pv = d.pool;
    int len = pv.lengths[(int64_t)d.layer * pv.max_seqs + seq];
    const int cap = pv.max_pages_per_seq * pv.page_size;
    if (len < 0 || len > cap) {
        atomicOr(pv.status, FLAG_BAD_LENGTH);
        len = len < 0 ? 0 : cap;
    }
    if (d.q_pos) {
        const int qp = d.q_pos[i];
        const int lim = qp < 0 ? 0 : qp + 1;
        len = len < lim ? len : lim;
    }
    return len;
}

// ---------------------------------------------------------------------------------------------
// Generic CUDA-core kernel.  grid (max_splits, n_q_heads, n_seqs), 4 warps; warp w takes tokens
// t0 + w, t0 + w + 4, ...; lane l holds elements l, l + 32, ... of the head dimension.
// ---------------------------------------------------------------------------------------------
template <typename T, int DPL>
__global__ void __launch_bounds__(kDecodeThreads) decode_generic_kernel(DecodeLaunch d) {
    const PoolView& pv = d.pool;
    const int split = blockIdx.x, hq = blockIdx.y, i = blockIdx.z;
    const int seq = d.seq_ids ? d.seq_ids[i] : i;
    if (!checked_seq(pv, seq)) return;
    const int n_attend = attend_count(d, i, seq);
    const int t0 = split * d.chunk_tokens;
    if (t0 >= n_attend) return;
    const int t1 = min(n_attend, t0 + d.chunk_tokens);
    const int D = pv.head_dim;
    const int G = d.n_q_heads / pv.num_kv_heads;
    const int h = hq / G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float scale = rsqrtf((float)D);

    float q[DPL], acc[DPL];
    const T* qrow = reinterpret_cast<const T*>(d.q) + (int64_t)i * d.q_stride + (int64_t)hq * D;
#pragma unroll
    for (int e = 0; e < DPL; ++e) {
        const int dd = lane + 32 * e;
        q[e] = dd < D ? to_f32(qrow[dd]) : 0.f;
        acc[e] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const T* kl = reinterpret_cast<const T*>(reinterpret_cast<const char*>(pv.k_base) + (int64_t)d.layer * pv.layer_stride_bytes);
    const T* vl = reinterpret_cast<const T*>(reinterpret_cast<const char*>(pv.v_base) + (int64_t)d.layer * pv.layer_stride_bytes);
    for (int t = t0 + warp; t < t1; t += kDecodeWarps) {
        const int page = checked_page(pv, seq, t / pv.page_size);
        if (page < 0) continue;
        const int64_t off = row_offset(pv, page, h, t % pv.page_size);
        float part = 0.f, v[DPL];
#pragma unroll
        for (int e = 0; e < DPL; ++e) {
            const int dd = lane + 32 * e;
            const float kk = dd < D ? to_f32(kl[off + dd]) : 0.f;
            v[e] = dd < D ? to_f32(vl[off + dd]) : 0.f;
            part = fmaf(q[e], kk, part);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        const float s = part * scale;
        const float m_new = fmaxf(m, s);
        const float alpha = expf(m - m_new);   // m = -inf on the first token gives 0
        const float p = expf(s - m_new);
        l = l * alpha + p;
#pragma unroll
        for (int e = 0; e < DPL; ++e) acc[e] = acc[e] * alpha + p * v[e];
        m = m_new;
    }
    // combine the four warps
    __shared__ float sm_m[kDecodeWarps], sm_l[kDecodeWarps];
    __shared__ float sm_acc[kDecodeWarps][DPL * 32];
    if (lane == 0) {
        sm_m[warp] = m;
        sm_l[warp] = l;
    }
#pragma unroll
    for (int e = 0; e < DPL; ++e) sm_acc[warp][lane + 32 * e] = acc[e];
    __syncthreads();
    if (warp == 0) {
        float M = -INFINITY;
        for (int w = 0; w < kDecodeWarps; ++w)
            if (sm_l[w] > 0.f) M = fmaxf(M, sm_m[w]);
        float L = 0.f, wgt[kDecodeWarps];
        for (int w = 0; w < kDecodeWarps; ++w) {
            wgt[w] = sm_l[w] > 0.f ? expf(sm_m[w] - M) : 0.f;
            L += wgt[w] * sm_l[w];
        }
        const int64_t pidx = ((int64_t)i * d.n_q_heads + hq) * d.max_splits + split;
#pragma unroll
        for (int e = 0; e < DPL; ++e) {
            const int dd = lane + 32 * e;
            float a = 0.f;
            for (int w = 0; w < kDecodeWarps; ++w) a += wgt[w] * sm_acc[w][dd];
            if (dd < D) d.ws_acc[pidx * D + dd] = a;
        }
        if (lane == 0) {
            d.ws_ml[pidx * 2 + 0] = M;
            d.ws_ml[pidx * 2 + 1] = L;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Tensor-core kernel (mma.sync m16n8k16, bf16 in, f32 accumulate).  grid (max_splits, kv_heads,
// n_seqs), 4 warps; warp w takes the 16-token tiles w, w + 4, ... of the CTA's chunk.
// Only rows 0..7 of the 16-row A operand carry query heads (G <= 8); rows 8..15 are zero and
// their accumulators are discarded, which halves the live accumulator registers.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16_rows8(float& c0, float& c1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    float z0 = 0.f, z1 = 0.f;
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c0), "+f"(c1), "+f"(z0), "+f"(z1)
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 r;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

constexpr int kMmaD = 128;

__global__ void __launch_bounds__(kDecodeThreads) decode_mma_kernel(DecodeLaunch d) {
    const PoolView& pv = d.pool;
    const int split = blockIdx.x, h = blockIdx.y, i = blockIdx.z;
    const int seq = d.seq_ids ? d.seq_ids[i] : i;
    if (!checked_seq(pv, seq)) return;
    const int n_attend = attend_count(d, i, seq);
    const int t0 = split * d.chunk_tokens;
    if (t0 >= n_attend) return;
    const int t1 = min(n_attend, t0 + d.chunk_tokens);
    const int G = d.n_q_heads / pv.num_kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int P = pv.page_size;

    // Q fragments: row g of the group, 16-byte units c, 4+c, 8+c, 12+c of the head dimension.
    uint32_t qa[8][2];
    {
        const char* qrow = reinterpret_cast<const char*>(d.q) + ((int64_t)i * d.q_stride + (int64_t)(h * G + g) * kMmaD) * 2;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            uint4 r = make_uint4(0, 0, 0, 0);
            if (g < G) r = *reinterpret_cast<const uint4*>(qrow + (4 * u + c) * 16);
            qa[2 * u][0] = r.x;
            qa[2 * u][1] = r.y;
            qa[2 * u + 1][0] = r.z;
            qa[2 * u + 1][1] = r.w;
        }
    }
    const char* kl = reinterpret_cast<const char*>(pv.k_base) + (int64_t)d.layer * pv.layer_stride_bytes;
    const char* vl = reinterpret_cast<const char*>(pv.v_base) + (int64_t)d.layer * pv.layer_stride_bytes;
    const int n_tiles = (t1 - t0 + 15) >> 4;

    // page ids of this warp's tiles, one per lane, fetched up front (a warp owns at most 32 tiles)
    int my_page = -1;
    {
        const int tile = warp + kDecodeWarps * lane;
        if (tile < n_tiles) my_page = checked_page(pv, seq, (t0 + tile * 16) / P);
    }

    float o[2][8][2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
        for (int e = 0; e < 8; ++e) o[hh][e][0] = o[hh][e][1] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    const float sc = rsqrtf((float)kMmaD) * kLog2e;

    int it = 0;
    for (int tile = warp; tile < n_tiles; tile += kDecodeWarps, ++it) {
        const int page = __shfl_sync(0xffffffffu, my_page, it);
        if (page < 0) continue;   // flagged in the status word
        const int tb = t0 + tile * 16;
        const int64_t tile_off = ((((int64_t)page * pv.num_kv_heads + h) * P) + (tb % P)) * (kMmaD * 2);
        const char* kp = kl + tile_off;
        const char* vp = vl + tile_off;
        uint4 kr[2][4], vr[4][2];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int u = 0; u < 4; ++u) kr[j][u] = ld_stream(kp + (8 * j + g) * 256 + (4 * u + c) * 16);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int row = 2 * c + (r & 1) + 8 * (r >> 1);
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) vr[r][hh] = ld_stream(vp + row * 256 + (g + 8 * hh) * 16);
        }
        // S = Q K^T for the two 8-token halves
        float s[2][2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            s[j][0] = s[j][1] = 0.f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                mma_bf16_rows8(s[j][0], s[j][1], qa[2 * u][0], qa[2 * u][1], kr[j][u].x, kr[j][u].y);
                mma_bf16_rows8(s[j][0], s[j][1], qa[2 * u + 1][0], qa[2 * u + 1][1], kr[j][u].z, kr[j][u].w);
            }
        }
        // mask the tail of the last tile; zero V rows there so that stale bytes cannot leak through 0 * x
        const bool tail = tb + 16 > t1;
        if (tail) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int b = 0; b < 2; ++b)
                    if (tb + 8 * j + 2 * c + b >= t1) s[j][b] = -INFINITY;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int row = 2 * c + (r & 1) + 8 * (r >> 1);
                if (tb + row >= t1) vr[r][0] = vr[r][1] = make_uint4(0, 0, 0, 0);
            }
        }
        float mx = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx * sc);   // the tile holds at least one allowed key
        const float alpha = exp2f(m_run - m_new);
        float p[2][2];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int b = 0; b < 2; ++b) p[j][b] = exp2f(fmaf(s[j][b], sc, -m_new));
        l_run = l_run * alpha + (p[0][0] + p[0][1]) + (p[1][0] + p[1][1]);
        m_run = m_new;
        const uint32_t pa0 = pack_bf16(p[0][0], p[0][1]);
        const uint32_t pa2 = pack_bf16(p[1][0], p[1][1]);
        // O = alpha * O + P V
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const uint32_t* ra = reinterpret_cast<const uint32_t*>(&vr[0][hh]);   // token 2c
            const uint32_t* rb = reinterpret_cast<const uint32_t*>(&vr[1][hh]);   // token 2c+1
            const uint32_t* rc = reinterpret_cast<const uint32_t*>(&vr[2][hh]);   // token 2c+8
            const uint32_t* rd = reinterpret_cast<const uint32_t*>(&vr[3][hh]);   // token 2c+9
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
                const uint32_t b0 = __byte_perm(ra[e >> 1], rb[e >> 1], sel);
                const uint32_t b1 = __byte_perm(rc[e >> 1], rd[e >> 1], sel);
                o[hh][e][0] *= alpha;
                o[hh][e][1] *= alpha;
                mma_bf16_rows8(o[hh][e][0], o[hh][e][1], pa0, pa2, b0, b1);
            }
        }
    }
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);

    // combine the four warps: (m, l) per row and the 8 x 128 accumulator tile
    __shared__ float sm_m[kDecodeWarps][8], sm_l[kDecodeWarps][8];
    __shared__ __align__(16) float sm_o[kDecodeWarps][8][kMmaD];
    if (c == 0) {
        sm_m[warp][g] = m_run;
        sm_l[warp][g] = l_run;
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            float* dst = &sm_o[warp][g][64 * hh + 16 * c + 8 * b];
            *reinterpret_cast<float4*>(dst) = make_float4(o[hh][0][b], o[hh][1][b], o[hh][2][b], o[hh][3][b]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(o[hh][4][b], o[hh][5][b], o[hh][6][b], o[hh][7][b]);
        }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * kMmaD; idx += kDecodeThreads) {
        const int r = idx >> 7, dd = idx & 127;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w)
            if (sm_l[w][r] > 0.f) M = fmaxf(M, sm_m[w][r]);
        float L = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w) {
            const float wgt = sm_l[w][r] > 0.f ? exp2f(sm_m[w][r] - M) : 0.f;
            L += wgt * sm_l[w][r];
            a += wgt * sm_o[w][r][dd];
        }
        const int64_t pidx = ((int64_t)i * d.n_q_heads + h * G + r) * d.max_splits + split;
        d.ws_acc[pidx * kMmaD + dd] = a;
        if (dd == 0) {
            d.ws_ml[pidx * 2 + 0] = M * (1.0f / kLog2e);   // back to the natural-log domain
            d.ws_ml[pidx * 2 + 1] = L;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// TMA-staged variant of the tensor-core kernel.  Same work split, same fragments, same partials;
// the difference is how K/V reach the fragments.  Every warp owns a private ring of NS stages in
// shared memory; lane 0 fills a stage with four cp.async.bulk.tensor 2-D boxes ([16 tokens][64 dims]
// of K and of V, 128-byte swizzle) that complete on the stage's mbarrier, so the bytes in flight per
// SM are set by the ring depth (NS x 8 KB per warp) instead of by the register file.  Fragments are
// read back with 16-byte shared loads whose lane-to-unit mapping is conflict-free under the
// hardware swizzle: for K a lane takes units 2c and 2c+1 of each 128-byte half-row (rows g and g+1
// of a quarter-warp then fall into opposite bank parities), for V a lane takes unit g of rows
// 2c, 2c+1, 2c+8, 2c+9.  No cluster, no multicast; every mbarrier wait is bounded and a timeout sets
// FLAG_WAIT_TIMEOUT, drains the copies still in flight and writes an empty partial.
// ---------------------------------------------------------------------------------------------
constexpr int kStageBytes = 8192;   // one 16-token tile: K (2 boxes x 2 KB) + V (2 boxes x 2 KB)

// Per-row metadata of a one-call step: from the kernel parameters, or from the uploaded copy for large batches.
__device__ __forceinline__ int row_seq(const StepRows& r, int n, int i) { return r.dev ? r.dev[i] : r.seq[i]; }
__device__ __forceinline__ int row_len(const StepRows& r, int n, int i) { return r.dev ? r.dev[n + i] : r.len[i]; }
__device__ __forceinline__ uint32_t row_pos(const StepRows& r, int n, int i) {
    return r.dev ? (uint32_t)r.dev[2 * n + i] : r.pos[i];
}

// FA (the one-call decode step): sequence id, stored length and token position of a row come from `rows`, so the
// kernel depends on nothing that an earlier kernel of the stream wrote except q, the new K/V rows and the pages.
// With d.early_start the caller has vouched for those (see skv_step_args), the wait for the previous kernel moves
// from the top to just before the partials are stored, and the whole K/V stream of this step overlaps the previous
// step's merge kernel and its exchange.
template <int NS, bool FA>
__global__ void __launch_bounds__(kDecodeThreads) decode_tma_kernel(const __grid_constant__ DecodeLaunch d,
                                                                    const __grid_constant__ CUtensorMap kmap,
                                                                    const __grid_constant__ CUtensorMap vmap,
                                                                    const __grid_constant__ StepRows rows) {
    extern __shared__ uint8_t smem_raw[];
    const PoolView& pv = d.pool;
    const int split = blockIdx.x, h = blockIdx.y;
    const int i = (FA && rows.ordered) ? (int)rows.order[blockIdx.z] : (int)blockIdx.z;   // a step may hand its longest rows out first
    const bool late_wait = FA && d.early_start;
    if (threadIdx.x == 0) {
        prefetch_tensormap(&kmap);
        prefetch_tensormap(&vmap);
    }
    if (!late_wait) pdl_wait();
    int seq, len_old = 0;
    uint32_t pos_raw = 0;
    if constexpr (FA) {
        seq = row_seq(rows, d.n_seqs, i);
        len_old = row_len(rows, d.n_seqs, i);
        pos_raw = row_pos(rows, d.n_seqs, i);
    } else {
        seq = d.seq_ids ? d.seq_ids[i] : i;
    }
    if (!checked_seq(pv, seq)) return;
    const int t0 = split * d.chunk_tokens;
    // The page id of this lane's tile does not depend on the sequence length: fetch it now, next to the
    // length, instead of after it (one dependent memory round trip less in every CTA's start-up).
    int raw_page = -1;
    {
        const int slot = (t0 + ((int)(threadIdx.x >> 5) + kDecodeWarps * (int)(threadIdx.x & 31)) * 16) / pv.page_size;
        if (slot < pv.max_pages_per_seq) raw_page = pv.page_table[(int64_t)seq * pv.max_pages_per_seq + slot];
    }
    // In a step the row's length does not count this step's token yet: it sits at position len_old of the pages,
    // is attended from shared memory by the CTA whose chunk contains it, and t1 bounds the tokens read from pages.
    if constexpr (!FA) len_old = attend_count(d, i, seq);
    const bool stores = FA && !(pos_raw & kRowNoStore);
    const int n_attend = len_old + (stores ? 1 : 0);
    const int G = d.n_q_heads / pv.num_kv_heads;
    if (t0 >= n_attend) {
        if (split == 0 && d.fuse_merge) {   // nothing to attend: the output row is exactly 0 (mlx_ops.py:118, :146)
            __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(d.out) + (int64_t)i * d.out_stride + (int64_t)h * G * kMmaD;
            for (int idx = threadIdx.x; idx < G * kMmaD; idx += kDecodeThreads) orow[idx] = __float2bfloat16_rn(0.f);
        }
        return;
    }
    const int t1 = min(len_old, t0 + d.chunk_tokens);
    const bool owner = stores && len_old >= t0 && len_old < t0 + d.chunk_tokens;
    const int n_splits = (n_attend + d.chunk_tokens - 1) / d.chunk_tokens;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int P = pv.page_size;
    if constexpr (FA) {
        // The kernels of a step launch their dependents at once: the merge kernel's blocks are resident by the time
        // this grid drains, and a following step that may start early fills the SMs this grid's tail leaves idle.
        pdl_launch_dependents();
        // Started beside earlier steps: the newest token of this row (position len_old - 1) may still be on its
        // way into the page.  The CTA whose chunk holds it waits (bounded) until the step that stores it has
        // published the row's length, before any of its tiles are requested; every other CTA reads pages that were
        // complete long before.
        if (late_wait && (pos_raw & kRowWaitPrev) && len_old > 0 && len_old - 1 >= t0 && len_old - 1 < t0 + d.chunk_tokens) {
            if (threadIdx.x == 0) {
                const int32_t* flag = d.stored_len + ((int64_t)d.layer * pv.max_seqs + seq) * pv.num_kv_heads + h;
                const long long start = clock64();
                int32_t seen;
                for (;;) {
                    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
                    if (seen >= len_old) break;
                    if (clock64() - start > 2000000000LL) {
                        atomicOr(pv.status, FLAG_WAIT_TIMEOUT);
                        break;
                    }
                }
                asm volatile("fence.proxy.async;" ::: "memory");   // the row is read by the TMA unit (async proxy)
            }
            __syncthreads();
        }
    }

    // Q fragments: row g, 16-byte units 2c and 2c+1 of each 128-byte half (the K lane mapping).  The loads are
    // issued here, beside the page ids, and used after the first tiles have been requested.
    uint4 qr[4];
    {
        const char* qrow = reinterpret_cast<const char*>(d.q) + ((int64_t)i * d.q_stride + (int64_t)(h * G + g) * kMmaD) * 2;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            qr[u] = make_uint4(0, 0, 0, 0);
            if (g < G) qr[u] = *reinterpret_cast<const uint4*>(qrow + (8 * (u >> 1) + 2 * c + (u & 1)) * 16);
        }
    }
    float my_inv_freq = 0.f;
    if (FA && threadIdx.x < kMmaD / 2) my_inv_freq = d.inv_freq[threadIdx.x];

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint8_t* ring = smem + warp * NS * kStageBytes;
    uint64_t* wbar = reinterpret_cast<uint64_t*>(smem + kDecodeWarps * NS * kStageBytes) + warp * NS;
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < NS; ++s) mbar_init(&wbar[s], 1);
        fence_mbar_init();
    }
    __syncwarp();

    uint32_t qa[8][2];
    float* fa_cos = reinterpret_cast<float*>(smem + kDecodeWarps * NS * kStageBytes + 128);   // [64]
    float* fa_sin = fa_cos + 64;                                                             // [64]
    float* fa_k = fa_sin + 64;                                                               // [128] rotated new K row
    float* fa_v = fa_k + kMmaD;                                                              // [128] new V row
    auto finish_q = [&]() {
        if constexpr (FA) {
            // unit u (first half) pairs with unit u + 2 (second half): dims 8 * (2c + u) + e and 64 more
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                uint32_t* lo = reinterpret_cast<uint32_t*>(&qr[u]);
                uint32_t* hi = reinterpret_cast<uint32_t*>(&qr[u + 2]);
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&lo[w]));
                    const float2 x2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&hi[w]));
                    const int dd = 8 * (2 * c + u) + 2 * w;
                    const float c0 = fa_cos[dd], s0 = fa_sin[dd], c1 = fa_cos[dd + 1], s1 = fa_sin[dd + 1];
                    const float y1a = __fadd_rn(__fmul_rn(x1.x, c0), __fmul_rn(-x2.x, s0));
                    const float y2a = __fadd_rn(__fmul_rn(x2.x, c0), __fmul_rn(x1.x, s0));
                    const float y1b = __fadd_rn(__fmul_rn(x1.y, c1), __fmul_rn(-x2.y, s1));
                    const float y2b = __fadd_rn(__fmul_rn(x2.y, c1), __fmul_rn(x1.y, s1));
                    lo[w] = pack_bf16(y1a, y1b);
                    hi[w] = pack_bf16(y2a, y2b);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            qa[2 * u][0] = qr[u].x;
            qa[2 * u][1] = qr[u].y;
            qa[2 * u + 1][0] = qr[u].z;
            qa[2 * u + 1][1] = qr[u].w;
        }
    };
    const int n_tiles = (t1 - t0 + 15) >> 4;
    const int n_my = n_tiles > warp ? (n_tiles - warp + kDecodeWarps - 1) / kDecodeWarps : 0;
    int my_page = -1;
    {
        const int tile = warp + kDecodeWarps * lane;
        if (tile < n_tiles) {
            if (raw_page >= 0 && raw_page < pv.num_pages)
                my_page = raw_page;
            else
                atomicOr(pv.status, FLAG_BAD_PAGE);   // skipped, not dereferenced
        }
    }
    const int layer_rows = (int)((int64_t)d.layer * (pv.layer_stride_bytes / (kMmaD * 2)));

    auto issue = [&](int k) {   // called by the whole warp
        const int page = __shfl_sync(0xffffffffu, my_page, k);
        if (lane == 0) {
            uint64_t* bar = &wbar[k % NS];
            if (page >= 0) {
                const int tb = t0 + (warp + kDecodeWarps * k) * 16;
                const int y = layer_rows + (page * pv.num_kv_heads + h) * P + (tb % P);
                uint8_t* st = ring + (k % NS) * kStageBytes;
                mbar_expect_tx(bar, kStageBytes);
                tma_load_2d(st, &kmap, 0, y, bar);
                tma_load_2d(st + 2048, &kmap, 64, y, bar);
                tma_load_2d(st + 4096, &vmap, 0, y, bar);
                tma_load_2d(st + 6144, &vmap, 64, y, bar);
            } else {
                mbar_arrive(bar);   // keep the stage's phase in step for a skipped tile
            }
        }
    };

    float o[2][8][2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
        for (int e = 0; e < 8; ++e) o[hh][e][0] = o[hh][e][1] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    const float sc = rsqrtf((float)kMmaD) * kLog2e;

    for (int k = 0; k < NS && k < n_my; ++k) issue(k);
    if constexpr (FA) {
        // While the first tiles are in flight: cos/sin of the token's position (the append kernel's arithmetic,
        // llama_mlx.py:132-136, :172-182), and in the owning CTA the new token's rows.
        const int tid = threadIdx.x;
        if (tid < kMmaD / 2) {
            float fpos = (float)(pos_raw & kRowPosMask);
            if (d.rope_scaling != 1.0f) fpos = __fdiv_rn(fpos, d.rope_scaling);
            float sn, cs;
            sincosf(__fmul_rn(fpos, my_inv_freq), &sn, &cs);
            fa_cos[tid] = cs;
            fa_sin[tid] = sn;
            if (owner) {
                const __nv_bfloat16* ks = reinterpret_cast<const __nv_bfloat16*>(d.new_k) + (int64_t)i * d.k_stride + (int64_t)h * kMmaD;
                const __nv_bfloat16* vs = reinterpret_cast<const __nv_bfloat16*>(d.new_v) + (int64_t)i * d.v_stride + (int64_t)h * kMmaD;
                const float x1 = __bfloat162float(ks[tid]), x2 = __bfloat162float(ks[tid + 64]);
                const __nv_bfloat16 k1 = __float2bfloat16_rn(__fadd_rn(__fmul_rn(x1, cs), __fmul_rn(-x2, sn)));
                const __nv_bfloat16 k2 = __float2bfloat16_rn(__fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn)));
                const __nv_bfloat16 v1 = vs[tid], v2 = vs[tid + 64];
                fa_k[tid] = __bfloat162float(k1);
                fa_k[tid + 64] = __bfloat162float(k2);
                fa_v[tid] = __bfloat162float(v1);
                fa_v[tid + 64] = __bfloat162float(v2);
                const int page = checked_page(pv, seq, len_old / P);
                if (page >= 0) {
                    const int64_t off = (int64_t)d.layer * (pv.layer_stride_bytes / 2) + row_offset(pv, page, h, len_old % P);
                    __nv_bfloat16* kdst = reinterpret_cast<__nv_bfloat16*>(pv.k_base) + off;
                    __nv_bfloat16* vdst = reinterpret_cast<__nv_bfloat16*>(pv.v_base) + off;
                    kdst[tid] = k1;
                    kdst[tid + 64] = k2;
                    vdst[tid] = v1;
                    vdst[tid + 64] = v2;
                    __threadfence();   // ahead of the flag below, for a later step that runs beside this one
                }
            }
        }
        __syncthreads();
        if (owner && d.stored_len && tid == 0) {
            asm volatile("fence.proxy.async;" ::: "memory");
            asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(d.stored_len + ((int64_t)d.layer * pv.max_seqs + seq) * pv.num_kv_heads + h),
                         "r"(len_old + 1) : "memory");
        }
    }
    finish_q();
    bool dead = false;
    int k = 0;
    for (; k < n_my; ++k) {
        const int page = __shfl_sync(0xffffffffu, my_page, k);
        const int stage = k % NS;
        // every lane runs its own bounded wait; the verdict is made warp-uniform before anything branches on it
        if (!mbar_wait_warp(&wbar[stage], (k / NS) & 1)) {
            dead = true;
            break;
        }
        if (page >= 0) {
            const int tb = t0 + (warp + kDecodeWarps * k) * 16;
            const uint8_t* st = ring + stage * kStageBytes;
            uint4 kr[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    kr[j][u] = *reinterpret_cast<const uint4*>(st + (u >> 1) * 2048 + (8 * j + g) * 128 +
                                                               (((2 * c + (u & 1)) ^ g) << 4));
            float s[2][2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                s[j][0] = s[j][1] = 0.f;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    mma_bf16_rows8(s[j][0], s[j][1], qa[2 * u][0], qa[2 * u][1], kr[j][u].x, kr[j][u].y);
                    mma_bf16_rows8(s[j][0], s[j][1], qa[2 * u + 1][0], qa[2 * u + 1][1], kr[j][u].z, kr[j][u].w);
                }
            }
            uint4 vr[4][2];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int row = 2 * c + (r & 1) + 8 * (r >> 1);
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
                    vr[r][hh] = *reinterpret_cast<const uint4*>(st + 4096 + hh * 2048 + row * 128 + ((g ^ (row & 7)) << 4));
            }
            const bool tail = tb + 16 > t1;
            if (tail) {
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int b = 0; b < 2; ++b)
                        if (tb + 8 * j + 2 * c + b >= t1) s[j][b] = -INFINITY;
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int row = 2 * c + (r & 1) + 8 * (r >> 1);
                    if (tb + row >= t1) vr[r][0] = vr[r][1] = make_uint4(0, 0, 0, 0);
                }
            }
            float mx = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run, mx * sc);
            const float alpha = exp2f(m_run - m_new);
            float p[2][2];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int b = 0; b < 2; ++b) p[j][b] = exp2f(fmaf(s[j][b], sc, -m_new));
            l_run = l_run * alpha + (p[0][0] + p[0][1]) + (p[1][0] + p[1][1]);
            m_run = m_new;
            const uint32_t pa0 = pack_bf16(p[0][0], p[0][1]);
            const uint32_t pa2 = pack_bf16(p[1][0], p[1][1]);
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const uint32_t* ra = reinterpret_cast<const uint32_t*>(&vr[0][hh]);
                const uint32_t* rb = reinterpret_cast<const uint32_t*>(&vr[1][hh]);
                const uint32_t* rc = reinterpret_cast<const uint32_t*>(&vr[2][hh]);
                const uint32_t* rd = reinterpret_cast<const uint32_t*>(&vr[3][hh]);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
                    const uint32_t b0 = __byte_perm(ra[e >> 1], rb[e >> 1], sel);
                    const uint32_t b1 = __byte_perm(rc[e >> 1], rd[e >> 1], sel);
                    o[hh][e][0] *= alpha;
                    o[hh][e][1] *= alpha;
                    mma_bf16_rows8(o[hh][e][0], o[hh][e][1], pa0, pa2, b0, b1);
                }
            }
        }
        // the stage has been read into registers and consumed: hand it back to the copy engine
        if (k + NS < n_my) {
            __syncwarp();
            fence_proxy_async();
            issue(k + NS);
        }
    }
    if constexpr (!FA) pdl_launch_dependents();   // the merge kernel may begin launching while this CTA combines and stores
    if (dead) {
        if (lane == 0) atomicOr(pv.status, FLAG_WAIT_TIMEOUT);
        // copies already issued for later tiles still target this CTA's shared memory: wait for them (bounded)
        for (int kk = k + 1; kk < n_my && kk < k + NS; ++kk) mbar_wait(&wbar[kk % NS], (kk / NS) & 1);
        __syncwarp();
        l_run = 0.f;
        m_run = -INFINITY;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
#pragma unroll
            for (int e = 0; e < 8; ++e) o[hh][e][0] = o[hh][e][1] = 0.f;
    }
    if constexpr (FA) {
        if (owner && warp == 0 && !dead) {   // this step's token: one more key, taken from shared memory
            float part = 0.f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float* kk = fa_k + 64 * (u >> 1) + 8 * (2 * c + (u & 1));
                const uint32_t regs[4] = {qa[2 * u][0], qa[2 * u][1], qa[2 * u + 1][0], qa[2 * u + 1][1]};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const float2 qf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&regs[w]));
                    part = fmaf(qf.x, kk[2 * w], part);
                    part = fmaf(qf.y, kk[2 * w + 1], part);
                }
            }
            part += __shfl_xor_sync(0xffffffffu, part, 1);
            part += __shfl_xor_sync(0xffffffffu, part, 2);
            const float sl = part * sc;
            const float m_new = fmaxf(m_run, sl);
            const float alpha = exp2f(m_run - m_new);
            const float pn = exp2f(sl - m_new);
            l_run = l_run * alpha + (c == 0 ? pn : 0.f);   // l_run is a per-lane share of the row sum
            m_run = m_new;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh)
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    const float* vv = fa_v + 64 * hh + 16 * c + 8 * b;
#pragma unroll
                    for (int e = 0; e < 8; ++e) o[hh][e][b] = fmaf(pn, vv[e], o[hh][e][b] * alpha);
                }
        }
    }
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);

    // all rings are idle now: reuse the start of shared memory for the cross-warp combine
    __syncthreads();
    float* sm_m = reinterpret_cast<float*>(smem);                  // [warps][8]
    float* sm_l = sm_m + kDecodeWarps * 8;                          // [warps][8]
    float* sm_o = sm_l + kDecodeWarps * 8;                          // [warps][8][128]
    if (c == 0) {
        sm_m[warp * 8 + g] = m_run;
        sm_l[warp * 8 + g] = l_run;
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh)
#pragma unroll
        for (int b = 0; b < 2; ++b) {
            float* dst = sm_o + (warp * 8 + g) * kMmaD + 64 * hh + 16 * c + 8 * b;
            *reinterpret_cast<float4*>(dst) = make_float4(o[hh][0][b], o[hh][1][b], o[hh][2][b], o[hh][3][b]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(o[hh][4][b], o[hh][5][b], o[hh][6][b], o[hh][7][b]);
        }
    __syncthreads();
    // The partials go into the workspace that the previous step's merge kernel may still be reading: this is
    // the first point that has to wait for it.
    if (late_wait) pdl_wait();
    __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(d.out) + (int64_t)i * d.out_stride + (int64_t)h * G * kMmaD;
    for (int idx = threadIdx.x; idx < G * kMmaD; idx += kDecodeThreads) {
        const int r = idx >> 7, dd = idx & 127;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w)
            if (sm_l[w * 8 + r] > 0.f) M = fmaxf(M, sm_m[w * 8 + r]);
        float L = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w) {
            const float wgt = sm_l[w * 8 + r] > 0.f ? exp2f(sm_m[w * 8 + r] - M) : 0.f;
            L += wgt * sm_l[w * 8 + r];
            a += wgt * sm_o[(w * 8 + r) * kMmaD + dd];
        }
        if (n_splits == 1 && d.fuse_merge) {   // the only chunk of this sequence: finish here, no partial is written
            orow[idx] = __float2bfloat16_rn(a / fmaxf(L, d.eps));
        } else {
            const int64_t pidx = ((int64_t)i * d.n_q_heads + h * G + r) * d.max_splits + split;
            d.ws_acc[pidx * kMmaD + dd] = a;
            if (dd == 0) {
                d.ws_ml[pidx * 2 + 0] = M * (1.0f / kLog2e);
                d.ws_ml[pidx * 2 + 1] = L;
            }
        }
    }
    if (n_splits == 1 || !d.fuse_merge) return;
    // The CTA that arrives last for this (sequence, KV head) merges all partials (K3r fused in).
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int32_t* ticket = d.tickets + (int64_t)i * pv.num_kv_heads + h;
        const int t = atomicAdd(ticket, 1);
        s_last = (t == n_splits - 1);
        if (s_last) *ticket = 0;   // ready for the next call
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    float* w_s = reinterpret_cast<float*>(smem);   // [G][n_splits] merge weights, then 1 / max(s, eps) per row
    float* inv_s = w_s + 8 * 128;
    for (int r = warp; r < G; r += kDecodeWarps) {
        const int64_t base = ((int64_t)i * d.n_q_heads + h * G + r) * d.max_splits;
        float M = -INFINITY;
        for (int sp = lane; sp < n_splits; sp += 32)
            if (__ldcg(&d.ws_ml[(base + sp) * 2 + 1]) > 0.f) M = fmaxf(M, __ldcg(&d.ws_ml[(base + sp) * 2]));
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o2));
        float L = 0.f;
        for (int sp = lane; sp < n_splits; sp += 32) {
            const float l = __ldcg(&d.ws_ml[(base + sp) * 2 + 1]);
            const float wgt = l > 0.f ? expf(__ldcg(&d.ws_ml[(base + sp) * 2]) - M) : 0.f;
            w_s[r * 128 + sp] = wgt;
            L += wgt * l;
        }
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o2);
        if (lane == 0) inv_s[r] = 1.0f / fmaxf(L, d.eps);
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * kMmaD; idx += kDecodeThreads) {
        const int r = idx >> 7, dd = idx & 127;
        const int64_t base = ((int64_t)i * d.n_q_heads + h * G + r) * d.max_splits;
        float a = 0.f;
        for (int sp0 = 0; sp0 < n_splits; sp0 += 8) {   // eight independent loads in flight per thread
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = sp0 + j < n_splits ? __ldcg(&d.ws_acc[(base + sp0 + j) * kMmaD + dd]) : 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) a += (sp0 + j < n_splits ? w_s[r * 128 + sp0 + j] : 0.f) * v[j];
        }
        orow[idx] = __float2bfloat16_rn(a * inv_s[r]);
    }
}

const StepRows& empty_rows() {
    static const StepRows r{};
    return r;
}

template <int NS, bool FA>
cudaError_t launch_tma(const DecodeLaunch& d, cudaStream_t stream) {
    static bool configured[64] = {};
    // rings, mbarriers (padded to 128 bytes), the fused append's cos/sin and new-row staging, alignment slack
    const int smem = kDecodeWarps * NS * kStageBytes + 128 + (FA ? (64 + 64 + 2 * kMmaD) * 4 : 0) + 1024;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(decode_tma_kernel<NS, FA>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    // the grid covers the longest sequence of the call, the workspace stride (max_splits) the longest possible one
    dim3 grid((unsigned)(d.grid_splits > 0 ? d.grid_splits : d.max_splits), (unsigned)d.pool.num_kv_heads, (unsigned)d.n_seqs);
    return launch_pdl(decode_tma_kernel<NS, FA>, grid, dim3(kDecodeThreads), (size_t)smem, stream, d,
                      *reinterpret_cast<const CUtensorMap*>(d.k_map), *reinterpret_cast<const CUtensorMap*>(d.v_map),
                      d.rows ? *d.rows : empty_rows());
}

// ---------------------------------------------------------------------------------------------
// Self-validating 16-byte words for the exchange between GPUs: {payload0, epoch, payload1, epoch}.  Each 8-byte
// half is a naturally aligned unit that arrives whole, so a reader that sees the call's epoch beside a payload word
// has that word; nothing else (fence, ticket, flag) orders the two sides.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void st_word(void* p, uint32_t d0, uint32_t d1, uint32_t epoch) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d0), "r"(epoch), "r"(d1), "r"(epoch) : "memory");
}
// Bounded (about a second of SM clocks) wait for one word of this call's epoch.
__device__ __forceinline__ bool poll_word(const void* p, uint32_t epoch, uint32_t& d0, uint32_t& d1) {
    const long long start = clock64();
    for (;;) {
        uint32_t x, y, z, w;
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(x), "=r"(y), "=r"(z), "=r"(w) : "l"(p) : "memory");
        if (y == epoch && w == epoch) {
            d0 = x;
            d1 = z;
            return true;
        }
        if (clock64() - start > 2000000000LL) return false;
    }
}

// ---------------------------------------------------------------------------------------------
// K3r: merge the partials of one (sequence, query head) with the reference's chunk-merge rule and
// write out = wv / max(s, eps) in the storage dtype.  grid (n_q_heads, n_seqs).  The same block also runs the
// row's share of the exchange between GPUs (ExchangeView) and, for a one-call step, writes the rotated q back and
// sets the sequence's device length.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) decode_reduce_kernel(const __grid_constant__ DecodeLaunch d,
                                                            const __grid_constant__ StepRows rows) {
    const PoolView& pv = d.pool;
    const int hq = blockIdx.x, i = blockIdx.y;
    // The next kernel in the stream (the following step's split-K kernel) either waits for this grid at its top or
    // touches nothing this grid reads or writes until it does (and takes care of the one page row the split-K kernel
    // ahead of this grid may still be storing): letting it launch now hides its launch latency and, in the second
    // case, lets its K/V stream begin while that kernel's last blocks drain.
    pdl_launch_dependents();
    pdl_wait();
    const int D = pv.head_dim;
    int seq, n_attend = 0;
    uint32_t pos_raw = 0;
    if (d.fused_append) {
        seq = row_seq(rows, d.n_seqs, i);
        pos_raw = row_pos(rows, d.n_seqs, i);
        n_attend = row_len(rows, d.n_seqs, i) + ((pos_raw & kRowNoStore) ? 0 : 1);
    } else {
        seq = d.seq_ids ? d.seq_ids[i] : i;
        if (seq >= 0 && seq < pv.max_seqs) n_attend = attend_count(d, i, seq);
    }
    const int n_splits = (n_attend + d.chunk_tokens - 1) / d.chunk_tokens;   // <= 128 by the plan
    const int64_t base = ((int64_t)i * d.n_q_heads + hq) * d.max_splits;
    // one thread per split fetches (m, l): the loads of all splits are in flight together
    __shared__ float sm_w[128];
    __shared__ float sm_red[8];
    __shared__ __align__(16) uint32_t sm_row[260];   // the finished row (storage dtype) or the partial row (float bits)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float m = -INFINITY, l = 0.f;
    if (tid < n_splits) {
        const float2 ml = *reinterpret_cast<const float2*>(&d.ws_ml[(base + tid) * 2]);
        m = ml.y > 0.f ? ml.x : -INFINITY;
        l = ml.y;
    }
    float M = m;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    if (lane == 0) sm_red[warp] = M;
    __syncthreads();
    M = fmaxf(fmaxf(sm_red[0], sm_red[1]), fmaxf(sm_red[2], sm_red[3]));
    const float w = l > 0.f ? expf(m - M) : 0.f;
    sm_w[tid] = w;
    float L = w * l;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    if (lane == 0) sm_red[4 + warp] = L;
    __syncthreads();
    L = (sm_red[4] + sm_red[5]) + (sm_red[6] + sm_red[7]);
    const float inv = 1.0f / fmaxf(L, d.eps);
    const int mode = d.xchg.mode;
    T* out = reinterpret_cast<T*>(d.out) + (int64_t)i * d.out_stride + (int64_t)hq * D;
    for (int dd = tid; dd < D; dd += blockDim.x) {
        float a = 0.f;
        for (int s0 = 0; s0 < n_splits; s0 += 8) {   // eight independent loads per thread in flight
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = s0 + j < n_splits ? d.ws_acc[(base + s0 + j) * D + dd] : 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) a += (s0 + j < n_splits ? sm_w[s0 + j] : 0.f) * v[j];
        }
        if (d.partial_out) {   // un-normalised partial for a merge done elsewhere: (acc, m, l) relative to M
            float* prow = d.partial_out + ((int64_t)i * d.n_q_heads + hq) * (D + 2);
            prow[dd] = a;
            if (dd == 0) {
                prow[D] = M;
                prow[D + 1] = L;
            }
        } else if (mode == 0) {
            out[dd] = from_f32<T>(a * inv);
        } else if (mode == 1) {
            reinterpret_cast<T*>(sm_row)[dd] = from_f32<T>(a * inv);
        } else {
            sm_row[dd] = __float_as_uint(a);
            if (dd == 0) {
                sm_row[D] = __float_as_uint(M);
                sm_row[D + 1] = __float_as_uint(L);
            }
        }
    }
    if (d.fused_append && seq >= 0 && seq < pv.max_seqs) {
        // The decode CTAs worked on their own rotated copies of q: write the rotated row back (the step's
        // contract).  Every CTA of the split-K kernel has finished, and nothing reads the device length of a row
        // during a step (the kernels take it from `rows`), so one block per sequence can set it here.
        if (tid < D / 2) {
            T* qrow = reinterpret_cast<T*>(const_cast<void*>(d.q)) + (int64_t)i * d.q_stride + (int64_t)hq * D;
            float fpos = (float)(pos_raw & kRowPosMask);
            if (d.rope_scaling != 1.0f) fpos = __fdiv_rn(fpos, d.rope_scaling);
            float sn, cs;
            sincosf(__fmul_rn(fpos, d.inv_freq[tid]), &sn, &cs);
            const float x1 = to_f32(qrow[tid]), x2 = to_f32(qrow[tid + D / 2]);
            qrow[tid] = from_f32<T>(__fadd_rn(__fmul_rn(x1, cs), __fmul_rn(-x2, sn)));
            qrow[tid + D / 2] = from_f32<T>(__fadd_rn(__fmul_rn(x2, cs), __fmul_rn(x1, sn)));
        }
        if (hq == 0 && tid == 0 && !(pos_raw & kRowNoStore)) pv.lengths[(int64_t)d.layer * pv.max_seqs + seq] = n_attend;
    }
    if (mode == 0) return;

    // ---- exchange between GPUs --------------------------------------------------------------------------------
    const uint32_t ep = d.xchg.epoch;
    const int world = d.xchg.world, rank = d.xchg.rank;
    const int W = (D * (int)sizeof(T)) >> 3;                       // 16-byte words of a finished row
    const int64_t row = (int64_t)i * d.n_q_heads + hq;
    const int64_t n_rows = (int64_t)d.n_seqs * d.n_q_heads;
    bool ok = true;
    __syncthreads();                                               // sm_row is complete
    if (mode == 1) {
        // finished row -> slot `rank` of every rank's buffer [world][n_rows][W]
        for (int task = tid; task < W * world; task += 128) {
            const int wd = task % W, p = task / W;
            uint4* dst = reinterpret_cast<uint4*>(d.xchg.recv[p]) + ((int64_t)rank * n_rows + row) * W + wd;
            st_word(dst, sm_row[2 * wd], sm_row[2 * wd + 1], ep);
        }
        // the same row of every rank's slot in this rank's buffer -> out[world][n_seqs][q_heads][D]
        for (int task = tid; task < W * world && ok; task += 128) {
            const int wd = task % W, s = task / W;
            const uint4* src = reinterpret_cast<const uint4*>(d.xchg.recv[rank]) + ((int64_t)s * n_rows + row) * W + wd;
            uint32_t d0 = 0, d1 = 0;
            ok = poll_word(src, ep, d0, d1);
            uint2* o = reinterpret_cast<uint2*>(reinterpret_cast<T*>(d.xchg.out) + ((int64_t)s * n_rows + row) * D) + wd;
            *o = make_uint2(d0, d1);
        }
    } else {
        // Buffer of a rank: region A [world][rows_owned][Wp] receives the partial rows this rank owns (row % world
        // == rank, slot row / world); region B [n_rows][W] receives every finished row from its owner.
        const int Wp = (D + 2) >> 1;
        const int64_t rows_owned = (n_rows + world - 1) / world;
        const int owner = (int)(row % world);
        const int64_t slot = row / world;
        const int64_t b_off = (int64_t)world * rows_owned * Wp;    // in 16-byte words
        for (int wd = tid; wd < Wp; wd += 128) {
            uint4* dst = reinterpret_cast<uint4*>(d.xchg.recv[owner]) + ((int64_t)rank * rows_owned + slot) * Wp + wd;
            st_word(dst, sm_row[2 * wd], sm_row[2 * wd + 1], ep);
        }
        if (rank == owner) {
            __shared__ float sm_part[8][260];
            for (int task = tid; task < Wp * world && ok; task += 128) {
                const int wd = task % Wp, s = task / Wp;
                const uint4* src = reinterpret_cast<const uint4*>(d.xchg.recv[rank]) + ((int64_t)s * rows_owned + slot) * Wp + wd;
                uint32_t d0 = 0, d1 = 0;
                ok = poll_word(src, ep, d0, d1);
                sm_part[s][2 * wd] = __uint_as_float(d0);
                sm_part[s][2 * wd + 1] = __uint_as_float(d1);
            }
            __syncthreads();
            // the chunk-merge rule across ranks (mlx_ops.py:125-146), every thread on the same eight (m, l) pairs
            float Mx = -INFINITY;
            for (int s = 0; s < world; ++s)
                if (sm_part[s][D + 1] > 0.f) Mx = fmaxf(Mx, sm_part[s][D]);
            float Lx = 0.f, wr[8];
            for (int s = 0; s < world; ++s) {
                wr[s] = sm_part[s][D + 1] > 0.f ? expf(sm_part[s][D] - Mx) : 0.f;
                Lx += wr[s] * sm_part[s][D + 1];
            }
            const float invx = 1.0f / fmaxf(Lx, d.eps);
            for (int dd = tid; dd < D; dd += 128) {
                float a = 0.f;
                for (int s = 0; s < world; ++s) a += wr[s] * sm_part[s][dd];
                reinterpret_cast<T*>(sm_row)[dd] = from_f32<T>(a * invx);
            }
            __syncthreads();
            for (int task = tid; task < W * world; task += 128) {
                const int wd = task % W, p = task / W;
                uint4* dst = reinterpret_cast<uint4*>(d.xchg.recv[p]) + b_off + row * W + wd;
                st_word(dst, sm_row[2 * wd], sm_row[2 * wd + 1], ep);
            }
        }
        T* orow = reinterpret_cast<T*>(d.xchg.out) + row * D;
        for (int wd = tid; wd < W && ok; wd += 128) {
            const uint4* src = reinterpret_cast<const uint4*>(d.xchg.recv[rank]) + b_off + row * W + wd;
            uint32_t d0 = 0, d1 = 0;
            ok = poll_word(src, ep, d0, d1);
            reinterpret_cast<uint2*>(orow)[wd] = make_uint2(d0, d1);
        }
    }
    if (!ok) atomicOr(pv.status, FLAG_WAIT_TIMEOUT);
}

// Merge of partial rows (acc[D], m, l) from several key ranges of the same query rows (sequence sharding, or any
// split of the keys): the reference's chunk-merge rule (mlx_ops.py:125-144) and out = wv / max(s, eps).
// parts[p] starts at parts + p * part_stride; each holds [n_rows][D + 2] floats.  grid n_rows, 128 threads.
template <typename T>
__global__ void __launch_bounds__(128) merge_partials_kernel(const float* __restrict__ parts, int n_parts, int64_t part_stride,
                                                             int D, float eps, T* __restrict__ out) {
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __shared__ float sm_w[128];
    __shared__ float sm_red[8];
    float m = -INFINITY, l = 0.f;
    if (tid < n_parts) {
        const float* prow = parts + tid * part_stride + (int64_t)row * (D + 2);
        l = prow[D + 1];
        m = l > 0.f ? prow[D] : -INFINITY;
    }
    float M = m;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    if (lane == 0) sm_red[warp] = M;
    __syncthreads();
    M = fmaxf(fmaxf(sm_red[0], sm_red[1]), fmaxf(sm_red[2], sm_red[3]));
    const float w = l > 0.f ? expf(m - M) : 0.f;
    sm_w[tid] = w;
    float L = w * l;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    if (lane == 0) sm_red[4 + warp] = L;
    __syncthreads();
    L = (sm_red[4] + sm_red[5]) + (sm_red[6] + sm_red[7]);
    const float inv = 1.0f / fmaxf(L, eps);
    for (int dd = tid; dd < D; dd += 128) {
        float a = 0.f;
        for (int p = 0; p < n_parts; ++p) a += sm_w[p] * parts[p * part_stride + (int64_t)row * (D + 2) + dd];
        out[(int64_t)row * D + dd] = from_f32<T>(a * inv);
    }
}

template <typename T>
cudaError_t launch_generic(const DecodeLaunch& d, cudaStream_t stream) {
    dim3 grid((unsigned)(d.grid_splits > 0 ? d.grid_splits : d.max_splits), (unsigned)d.n_q_heads, (unsigned)d.n_seqs);
    const int dpl = (d.pool.head_dim + 31) / 32;
    switch (dpl) {
        case 1: decode_generic_kernel<T, 1><<<grid, kDecodeThreads, 0, stream>>>(d); break;
        case 2: decode_generic_kernel<T, 2><<<grid, kDecodeThreads, 0, stream>>>(d); break;
        case 3: decode_generic_kernel<T, 3><<<grid, kDecodeThreads, 0, stream>>>(d); break;
        case 4: decode_generic_kernel<T, 4><<<grid, kDecodeThreads, 0, stream>>>(d); break;
        case 5: case 6: decode_generic_kernel<T, 6><<<grid, kDecodeThreads, 0, stream>>>(d); break;
        default: decode_generic_kernel<T, 8><<<grid, kDecodeThreads, 0, stream>>>(d); break;
    }
    return cudaGetLastError();
}

}  // namespace

void decode_plan(int32_t page_size, int32_t max_pages_per_seq, int32_t n_seqs, int32_t num_kv_heads,
                 int64_t total_tokens_hint, int32_t longest_hint, int32_t* chunk_tokens, int32_t* max_splits) {
    // `splits` bounds the partials per sequence, and with them the workspace, independently of the lengths: a chunk
    // is never shorter than 256 tokens and a sequence never has more than 128 of them.
    const int64_t max_ctx = (int64_t)max_pages_per_seq * page_size;
    int64_t splits = (max_ctx + 255) / 256;
    splits = splits < 1 ? 1 : (splits > 128 ? 128 : splits);
    int64_t floor_chunk = (max_ctx + splits - 1) / splits;
    floor_chunk = ((floor_chunk + 63) / 64) * 64;         // 4 warps x 16-token tiles
    if (floor_chunk < 256) floor_chunk = 256;
    // Aim at about 192 CTAs of up to 1536 tokens.  Measured on B200 with steps enqueued back to back: at 3 CTAs per
    // SM the grid of a step then leaves room for the next step's CTAs beside it (its start-up hides behind this
    // step's tail), the merge kernel has few partials to read, and 192 CTAs x 64 KB in flight already saturate HBM.
    // Per-GPU shares of the 64-sequence workload: 1/8 33.9 -> 29.0 us per step, 1/4 54.9 -> 49.2; four sequences of
    // 96k tokens with one KV head: 52 -> 32 us per layer step (2048-token chunks: 30 us, but ragged batches lose
    // with them: their last, partly filled chunks leave SMs idle).
    const Switches& sw = switches();
    int64_t chunk = floor_chunk;
    if (total_tokens_hint > 0) {
        chunk = ((num_kv_heads * total_tokens_hint + 191) / 192 + 63) / 64 * 64;
        const int64_t cap = floor_chunk > 1536 ? floor_chunk : 1536;
        if (chunk > cap) chunk = cap;
        if (chunk < floor_chunk) chunk = floor_chunk;
        // A batch of about equal lengths (a decoder's: every sequence at the same position): cut the longest
        // sequence into equal chunks instead of full ones and a remainder.  Eight sequences of 2304 tokens with 16
        // KV heads: 1536 + 768 tokens per sequence took 41 us per layer step, 2 x 1152 takes 36 us.
        if (longest_hint > 0 && total_tokens_hint * 10 >= (int64_t)9 * longest_hint * n_seqs) {
            const int64_t n = (longest_hint + chunk - 1) / chunk;
            const int64_t even = (((int64_t)longest_hint + n - 1) / n + 63) / 64 * 64;
            if (even >= floor_chunk && even < chunk) chunk = even;
        }
        if (sw.chunk > 0 && sw.chunk >= floor_chunk) chunk = ((sw.chunk + 63) / 64) * 64;   // SKV_DECODE_CHUNK
    }
    if (chunk > 2048) chunk = 2048;                       // a warp holds at most 32 tile page ids
    *chunk_tokens = (int32_t)chunk;
    *max_splits = (int32_t)splits;                        // >= ceil(max_ctx / chunk) for every chunk chosen above
}

cudaError_t launch_decode(const DecodeLaunch& d_in, cudaStream_t stream) {
    DecodeLaunch d = d_in;
    const Switches& sw = switches();
    // Measured on B200: the in-kernel merge (last-arriving CTA) costs about 2 us more per call than the
    // separate merge launch at the full 64-sequence workload and at a quarter of it (device-wide fences in
    // every CTA plus a serial tail), but saves about 5 us at an eighth of it, where the call is latency-bound.
    // So it is chosen only for small calls; SKV_DECODE_FUSE=0/1 overrides.
    d.fuse_merge = d.total_tokens * d.pool.num_kv_heads < 400000 ? 1 : 0;
    // the gather, the partial output and the fused append's bookkeeping live in the merge kernel
    const bool needs_merge_kernel = d.xchg.mode != 0 || d.partial_out || d.fused_append;
    if (needs_merge_kernel) d.fuse_merge = 0;
    if (sw.fuse >= 0 && !needs_merge_kernel) d.fuse_merge = sw.fuse;
    const int G = d.n_q_heads / d.pool.num_kv_heads;
    const bool mma_ok = d.dtype == SKV_BF16 && d.pool.head_dim == kMmaD && d.pool.page_size % 16 == 0 && G <= 8 &&
                        !d.force_generic && ((uintptr_t)d.q % 16 == 0) && (d.q_stride * 2) % 16 == 0;
    if (d.max_splits > 128) return cudaErrorInvalidValue;   // the merge kernel handles one split per thread; skv_create rejects such pools
    cudaError_t e;
    // SKV_DECODE_IMPL=reg: direct-to-register loads; default: the TMA ring when the pool has tensor maps
    const bool tma_ok = mma_ok && d.k_map && d.v_map && (d.fused_append || !sw.impl_reg) && (d.q_stride * 2) % 16 == 0;
    if (d.fused_append && (!tma_ok || d.q_pos || !d.new_k || !d.new_v || !d.inv_freq || !d.rows))
        return cudaErrorInvalidValue;   // only the TMA kernel implements it; callers check the conditions first
    if (tma_ok) {
        const int ns = sw.stages;   // 2 stages -> 3 CTAs per SM (24 stages of 8 KB in flight), the measured best
        if (d.fused_append)
            e = launch_tma<2, true>(d, stream);
        else
            e = ns == 3 ? launch_tma<3, false>(d, stream) : ns == 4 ? launch_tma<4, false>(d, stream) : launch_tma<2, false>(d, stream);
    } else if (mma_ok) {
        dim3 grid((unsigned)(d.grid_splits > 0 ? d.grid_splits : d.max_splits), (unsigned)d.pool.num_kv_heads, (unsigned)d.n_seqs);
        decode_mma_kernel<<<grid, kDecodeThreads, 0, stream>>>(d);
        e = cudaGetLastError();
    } else if (d.dtype == SKV_BF16) {
        e = launch_generic<__nv_bfloat16>(d, stream);
    } else {
        e = launch_generic<float>(d, stream);
    }
    if (e != cudaSuccess) return e;
    if (tma_ok && d.fuse_merge) {   // merge is fused into the kernel
        count_launches(1);
        return cudaSuccess;
    }
    count_launches(2);
    dim3 rgrid((unsigned)d.n_q_heads, (unsigned)d.n_seqs);
    const int threads = 128;
    const StepRows& rows = d.rows ? *d.rows : empty_rows();
    return d.dtype == SKV_BF16 ? launch_pdl(decode_reduce_kernel<__nv_bfloat16>, rgrid, dim3(threads), 0, stream, d, rows)
                               : launch_pdl(decode_reduce_kernel<float>, rgrid, dim3(threads), 0, stream, d, rows);
}

cudaError_t launch_merge_partials(const float* parts, int32_t n_parts, int64_t part_stride, int32_t n_rows, int32_t head_dim,
                                  float eps, void* out, int32_t dtype, cudaStream_t stream) {
    if (dtype == SKV_BF16)
        merge_partials_kernel<__nv_bfloat16><<<n_rows, 128, 0, stream>>>(parts, n_parts, part_stride, head_dim, eps,
                                                                       reinterpret_cast<__nv_bfloat16*>(out));
    else
        merge_partials_kernel<float><<<n_rows, 128, 0, stream>>>(parts, n_parts, part_stride, head_dim, eps,
                                                               reinterpret_cast<float*>(out));
    count_launches(1);
    return cudaGetLastError();
}

}  // namespace skv
