// K1: append with optional RoPE-on-write (K and, in the same launch, Q); K2: paged -> dense gather;
// stand-alone RoPE over rows.
//
// RoPE follows the reference bit pattern as closely as a GPU can: the angle is
// float(position) * inv_freq[i] in float32 (src/ollm/llama_mlx.py:132-136), cos/sin come from
// the accurate sincosf (this file must not be built with fast-math), and the rotation is
// x*cos + rotate_half(x)*sin with separately rounded products (llama_mlx.py:172-182).
#include "common.cuh"

namespace skv {

__device__ __forceinline__ void rope_pair(float x1, float x2, float pos, float inv_freq, float& y1, float& y2) {
    float angle = __fmul_rn(pos, inv_freq);
    float s, c;
    sincosf(angle, &s, &c);
    // first half:  x1*cos + (-x2)*sin ; second half: x2*cos + x1*sin
    y1 = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(-x2, s));
    y2 = __fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s));
}

template <typename T>
__global__ void append_kernel(AppendLaunch a) {
    const PoolView& pv = a.pool;
    pdl_wait();
    const int half = pv.head_dim >> 1;
    const int tok = blockIdx.x;                 // i * n_new + j
    const int i = tok / a.n_new;
    const int j = tok - i * a.n_new;
    const int heads_per_block = blockDim.x / half;
    const int local_head = threadIdx.x / half;
    const int d = threadIdx.x - local_head * half;
    if (local_head >= heads_per_block) return;
    const int slot_head = blockIdx.y * heads_per_block + local_head;   // [0, Hkv) = K/V heads, then Q heads
    const int n_slots = pv.num_kv_heads + a.n_q_heads;
    if (slot_head >= n_slots) return;

    const AppendMeta m = a.meta[i];
    if (!checked_seq(pv, m.seq)) return;
    const int pos = m.start + j;
    float fpos = (float)pos;
    if (a.scaling != 1.0f) fpos = __fdiv_rn(fpos, a.scaling);

    if (slot_head < pv.num_kv_heads) {
        const int h = slot_head;
        const T* ksrc = reinterpret_cast<const T*>(a.k) + i * a.kv_stride_seq + h * a.kv_stride_head + j * a.kv_stride_tok;
        const T* vsrc = reinterpret_cast<const T*>(a.v) + i * a.kv_stride_seq + h * a.kv_stride_head + j * a.kv_stride_tok;
        const int page = checked_page(pv, m.seq, pos / pv.page_size);
        if (page >= 0) {
            const int64_t off = (int64_t)a.layer * (pv.layer_stride_bytes / (int64_t)sizeof(T)) +
                                row_offset(pv, page, h, pos % pv.page_size);
            T* kdst = reinterpret_cast<T*>(pv.k_base) + off;
            T* vdst = reinterpret_cast<T*>(pv.v_base) + off;
            T k1 = ksrc[d], k2 = ksrc[d + half];
            if (a.rope_k) {
                float y1, y2;
                rope_pair(to_f32(k1), to_f32(k2), fpos, a.inv_freq[d], y1, y2);
                k1 = from_f32<T>(y1);
                k2 = from_f32<T>(y2);
            }
            kdst[d] = k1;
            kdst[d + half] = k2;
            vdst[d] = vsrc[d];
            vdst[d + half] = vsrc[d + half];
        }
        if (h == 0 && j == 0 && d == 0) pv.lengths[(int64_t)a.layer * pv.max_seqs + m.seq] = m.start + a.n_new;
    } else {
        const int h = slot_head - pv.num_kv_heads;
        const int64_t qoff = i * a.q_stride_seq + h * a.q_stride_head + j * a.q_stride_tok;
        const T* qsrc = reinterpret_cast<const T*>(a.q_in) + qoff;
        T* qdst = reinterpret_cast<T*>(a.q_out) + qoff;
        float y1, y2;
        rope_pair(to_f32(qsrc[d]), to_f32(qsrc[d + half]), fpos, a.inv_freq[d], y1, y2);
        qdst[d] = from_f32<T>(y1);
        qdst[d + half] = from_f32<T>(y2);
    }
}

// Vectorised append: one block per new token, 16-byte accesses, cos/sin of the token's position computed once
// per block and shared by all heads (the scalar kernel above recomputes them per head and moves 2 or 4 bytes
// per access: measured 0.27 ms for 16 k tokens x 32 heads of bf16 where the bytes need about 0.07 ms).
// Work items: (head slot, 16-byte chunk c of the first half) for K and Q -- the thread loads chunk c of both
// halves, rotates the pairs and stores both -- and (KV head, 16-byte chunk of the whole row) for V.
// Same arithmetic per element as rope_pair, so the stored bytes are identical to the scalar kernel's.
template <typename T>
__global__ void __launch_bounds__(128) append_vec_kernel(AppendLaunch a) {
    constexpr int VEC = 16 / (int)sizeof(T);
    const PoolView& pv = a.pool;
    pdl_wait();
    extern __shared__ float cs[];                // [half] cos, [half] sin
    const int half = pv.head_dim >> 1;
    const int tok = blockIdx.x;                  // i * n_new + j
    const int i = tok / a.n_new;
    const int j = tok - i * a.n_new;
    const AppendMeta m = a.meta[i];
    if (!checked_seq(pv, m.seq)) return;
    const int pos = m.start + j;
    const bool need_rope = a.rope_k || a.n_q_heads > 0;
    if (need_rope) {
        float fpos = (float)pos;
        if (a.scaling != 1.0f) fpos = __fdiv_rn(fpos, a.scaling);
        for (int d = threadIdx.x; d < half; d += blockDim.x) {
            float sn, c;
            sincosf(__fmul_rn(fpos, a.inv_freq[d]), &sn, &c);
            cs[d] = c;
            cs[half + d] = sn;
        }
        __syncthreads();
    }
    const int page = checked_page(pv, m.seq, pos / pv.page_size);
    const int chunks = half / VEC;               // 16-byte chunks per half row
    const int n_rot = pv.num_kv_heads + a.n_q_heads;
    // K rows (rotated or copied) and Q rows (rotated)
    for (int item = threadIdx.x; item < n_rot * chunks; item += blockDim.x) {
        const int slot = item / chunks, c = item - slot * chunks;
        const T* src;
        T* dst;
        bool rotate;
        if (slot < pv.num_kv_heads) {
            if (page < 0) continue;
            src = reinterpret_cast<const T*>(a.k) + i * a.kv_stride_seq + slot * a.kv_stride_head + j * a.kv_stride_tok;
            dst = reinterpret_cast<T*>(pv.k_base) + (int64_t)a.layer * (pv.layer_stride_bytes / (int64_t)sizeof(T)) +
                  row_offset(pv, page, slot, pos % pv.page_size);
            rotate = a.rope_k != 0;
        } else {
            const int64_t qoff = i * a.q_stride_seq + (slot - pv.num_kv_heads) * a.q_stride_head + j * a.q_stride_tok;
            src = reinterpret_cast<const T*>(a.q_in) + qoff;
            dst = reinterpret_cast<T*>(a.q_out) + qoff;
            rotate = true;
        }
        uint4 lo = *reinterpret_cast<const uint4*>(src + c * VEC);
        uint4 hi = *reinterpret_cast<const uint4*>(src + half + c * VEC);
        if (rotate) {
            T* x1 = reinterpret_cast<T*>(&lo);
            T* x2 = reinterpret_cast<T*>(&hi);
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                const float f1 = to_f32(x1[e]), f2 = to_f32(x2[e]);
                const float co = cs[c * VEC + e], sn = cs[half + c * VEC + e];
                x1[e] = from_f32<T>(__fadd_rn(__fmul_rn(f1, co), __fmul_rn(-f2, sn)));
                x2[e] = from_f32<T>(__fadd_rn(__fmul_rn(f2, co), __fmul_rn(f1, sn)));
            }
        }
        *reinterpret_cast<uint4*>(dst + c * VEC) = lo;
        *reinterpret_cast<uint4*>(dst + half + c * VEC) = hi;
    }
    // V rows: plain copy
    if (page >= 0) {
        for (int item = threadIdx.x; item < pv.num_kv_heads * 2 * chunks; item += blockDim.x) {
            const int h = item / (2 * chunks), c = item - h * 2 * chunks;
            const T* src = reinterpret_cast<const T*>(a.v) + i * a.kv_stride_seq + h * a.kv_stride_head + j * a.kv_stride_tok;
            T* dst = reinterpret_cast<T*>(pv.v_base) + (int64_t)a.layer * (pv.layer_stride_bytes / (int64_t)sizeof(T)) +
                     row_offset(pv, page, h, pos % pv.page_size);
            *reinterpret_cast<uint4*>(dst + c * VEC) = *reinterpret_cast<const uint4*>(src + c * VEC);
        }
    }
    if (j == 0 && threadIdx.x == 0) pv.lengths[(int64_t)a.layer * pv.max_seqs + m.seq] = m.start + a.n_new;
}

// 16-byte accesses need 16-byte aligned rows on both sides.
static bool append_vectorisable(const AppendLaunch& a, size_t esize) {
    const int vec = (int)(16 / esize);
    if (a.pool.head_dim % (2 * vec) != 0) return false;
    auto ok_ptr = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    auto ok_stride = [vec](int64_t s) { return s % vec == 0; };
    if (!ok_ptr(a.k) || !ok_ptr(a.v) || !ok_stride(a.kv_stride_seq) || !ok_stride(a.kv_stride_head) || !ok_stride(a.kv_stride_tok))
        return false;
    if (a.n_q_heads > 0 && (!ok_ptr(a.q_in) || !ok_ptr(a.q_out) || !ok_stride(a.q_stride_seq) || !ok_stride(a.q_stride_head) ||
                            !ok_stride(a.q_stride_tok)))
        return false;
    return !switches().append_scalar;
}

cudaError_t launch_append(const AppendLaunch& a, cudaStream_t stream) {
    const size_t esize = a.dtype == SKV_BF16 ? 2 : 4;
    if (append_vectorisable(a, esize)) {
        dim3 grid((unsigned)(a.n_seqs * a.n_new));
        const size_t smem = (size_t)a.pool.head_dim * sizeof(float);
        cudaError_t e = a.dtype == SKV_BF16 ? launch_pdl(append_vec_kernel<__nv_bfloat16>, grid, dim3(128), smem, stream, a)
                                            : launch_pdl(append_vec_kernel<float>, grid, dim3(128), smem, stream, a);
        count_launches(1);
        return e;
    }
    const int half = a.pool.head_dim / 2;
    int heads_per_block = 128 / half;
    if (heads_per_block < 1) heads_per_block = 1;
    const int n_slots = a.pool.num_kv_heads + a.n_q_heads;
    if (heads_per_block > n_slots) heads_per_block = n_slots;
    dim3 grid((unsigned)(a.n_seqs * a.n_new), (unsigned)((n_slots + heads_per_block - 1) / heads_per_block));
    dim3 block((unsigned)(heads_per_block * half));
    cudaError_t e = a.dtype == SKV_BF16 ? launch_pdl(append_kernel<__nv_bfloat16>, grid, block, 0, stream, a)
                                        : launch_pdl(append_kernel<float>, grid, block, 0, stream, a);
    count_launches(1);
    return e;
}

template <typename T>
__global__ void rope_rows_kernel(RopeRowsLaunch r) {
    const int half = r.head_dim >> 1;
    const int row = blockIdx.x;
    for (int idx = threadIdx.x; idx < r.n_heads * half; idx += blockDim.x) {
        const int h = idx / half, d = idx - h * half;
        float fpos = (float)r.positions[row];
        if (r.scaling != 1.0f) fpos = __fdiv_rn(fpos, r.scaling);
        const int64_t off = row * r.stride_row + h * r.stride_head;
        const T* src = reinterpret_cast<const T*>(r.x_in) + off;
        T* dst = reinterpret_cast<T*>(r.x_out) + off;
        float y1, y2;
        rope_pair(to_f32(src[d]), to_f32(src[d + half]), fpos, r.inv_freq[d], y1, y2);
        dst[d] = from_f32<T>(y1);
        dst[d + half] = from_f32<T>(y2);
    }
}

cudaError_t launch_rope_rows(const RopeRowsLaunch& r, cudaStream_t stream) {
    int threads = r.n_heads * (r.head_dim / 2);
    threads = threads > 256 ? 256 : ((threads + 31) / 32) * 32;
    if (r.dtype == SKV_BF16)
        rope_rows_kernel<__nv_bfloat16><<<r.n_rows, threads, 0, stream>>>(r);
    else
        rope_rows_kernel<float><<<r.n_rows, threads, 0, stream>>>(r);
    count_launches(1);
    return cudaGetLastError();
}

// K2.  One block copies a tile of token rows of one (sequence, head); VEC is the copy width in bytes.
template <int VEC>
__global__ void gather_kernel(GatherLaunch g, int esize) {
    const PoolView& pv = g.pool;
    const int i = blockIdx.z, h = blockIdx.y;
    const int seq = g.seq_ids ? g.seq_ids[i] : i;
    if (!checked_seq(pv, seq)) return;
    const int len = pv.lengths[(int64_t)g.layer * pv.max_seqs + seq];
    const int row_bytes = pv.head_dim * esize;
    const int vec_per_row = row_bytes / VEC;
    const int rows_per_block = 16;
    const int t0 = blockIdx.x * rows_per_block;
    char* out_k = reinterpret_cast<char*>(g.out_k) + (((int64_t)i * pv.num_kv_heads + h) * g.max_len) * row_bytes;
    char* out_v = reinterpret_cast<char*>(g.out_v) + (((int64_t)i * pv.num_kv_heads + h) * g.max_len) * row_bytes;
    const char* kb = reinterpret_cast<const char*>(pv.k_base) + (int64_t)g.layer * pv.layer_stride_bytes;
    const char* vb = reinterpret_cast<const char*>(pv.v_base) + (int64_t)g.layer * pv.layer_stride_bytes;
    for (int idx = threadIdx.x; idx < rows_per_block * vec_per_row; idx += blockDim.x) {
        const int t = t0 + idx / vec_per_row;
        const int c = idx % vec_per_row;
        if (t >= g.max_len) break;
        const int64_t dst = (int64_t)t * row_bytes + (int64_t)c * VEC;
        if (t < len) {
            const int page = checked_page(pv, seq, t / pv.page_size);
            if (page < 0) continue;
            const int64_t src = row_offset(pv, page, h, t % pv.page_size) * esize + (int64_t)c * VEC;
            if (VEC == 16) {
                *reinterpret_cast<int4*>(out_k + dst) = *reinterpret_cast<const int4*>(kb + src);
                *reinterpret_cast<int4*>(out_v + dst) = *reinterpret_cast<const int4*>(vb + src);
            } else if (VEC == 4) {
                *reinterpret_cast<uint32_t*>(out_k + dst) = *reinterpret_cast<const uint32_t*>(kb + src);
                *reinterpret_cast<uint32_t*>(out_v + dst) = *reinterpret_cast<const uint32_t*>(vb + src);
            } else {
                *reinterpret_cast<uint16_t*>(out_k + dst) = *reinterpret_cast<const uint16_t*>(kb + src);
                *reinterpret_cast<uint16_t*>(out_v + dst) = *reinterpret_cast<const uint16_t*>(vb + src);
            }
        } else {
            if (VEC == 16) {
                *reinterpret_cast<int4*>(out_k + dst) = make_int4(0, 0, 0, 0);
                *reinterpret_cast<int4*>(out_v + dst) = make_int4(0, 0, 0, 0);
            } else if (VEC == 4) {
                *reinterpret_cast<uint32_t*>(out_k + dst) = 0u;
                *reinterpret_cast<uint32_t*>(out_v + dst) = 0u;
            } else {
                *reinterpret_cast<uint16_t*>(out_k + dst) = 0;
                *reinterpret_cast<uint16_t*>(out_v + dst) = 0;
            }
        }
    }
}

cudaError_t launch_gather(const GatherLaunch& g, cudaStream_t stream) {
    const int esize = (int)dtype_size(g.dtype);
    const int row_bytes = g.pool.head_dim * esize;
    dim3 grid((unsigned)((g.max_len + 15) / 16), (unsigned)g.pool.num_kv_heads, (unsigned)g.n_seqs);
    const bool aligned16 = row_bytes % 16 == 0 && ((uintptr_t)g.out_k % 16 == 0) && ((uintptr_t)g.out_v % 16 == 0);
    if (aligned16)
        gather_kernel<16><<<grid, 256, 0, stream>>>(g, esize);
    else if (row_bytes % 4 == 0 && ((uintptr_t)g.out_k % 4 == 0) && ((uintptr_t)g.out_v % 4 == 0))
        gather_kernel<4><<<grid, 256, 0, stream>>>(g, esize);
    else
        gather_kernel<2><<<grid, 256, 0, stream>>>(g, esize);
    count_launches(1);
    return cudaGetLastError();
}

}  // namespace skv
