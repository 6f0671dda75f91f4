// K4f: chunked grouped-query attention on CUDA cores in float32 arithmetic, for dense
// [B][H][L][D] tensors or for K/V read through a page table.  Covers every shape the reference
// function accepts (src/ollm/backends/mlx_ops.py:32-152): any head_dim <= 256, any group size,
// float32 or bf16 storage, causal with absolute query positions or unmasked.  It is the exact-
// arithmetic path (no tensor cores, so the 1e-4 float32 tolerance holds) and the cross-check of
// the tensor-core prefill kernel.
//
// The causal mask k_pos <= q_pos (:107-112) allows a prefix of the keys, so a query row simply
// attends keys 0 .. min(Lk, q_pos + 1); a row whose prefix is empty yields 0 (:118, :146).
#include "common.cuh"

namespace skv {

namespace {

constexpr int kRowsPerBlock = 4;   // one warp per query row

template <typename T, int DPL>
__global__ void __launch_bounds__(kRowsPerBlock * 32) attn_generic_kernel(DenseAttnLaunch a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * kRowsPerBlock + warp;
    const int hq = blockIdx.y, b = blockIdx.z;
    if (row >= a.Lq) return;
    const int D = a.D;
    const int G = a.Hq / a.Hkv;
    const int h = hq / G;
    const bool paged = a.pool.k_base != nullptr;
    const PoolView& pv = a.pool;
    int seq = b, Lk = a.Lk;
    if (paged) {
        seq = a.seq_ids ? a.seq_ids[b] : b;
        if (!checked_seq(pv, seq)) return;
        Lk = pv.lengths[(int64_t)a.layer * pv.max_seqs + seq];
        const int cap = pv.max_pages_per_seq * pv.page_size;
        if (Lk < 0 || Lk > cap) {
            atomicOr(pv.status, FLAG_BAD_LENGTH);
            Lk = Lk < 0 ? 0 : cap;
        }
    }
    int n_keys = Lk;
    if (a.causal) {
        const int qpos = a.positions ? a.positions[(int64_t)b * a.Lq + row] : (Lk - a.Lq + row);
        const int lim = qpos < 0 ? 0 : qpos + 1;
        n_keys = lim < Lk ? lim : Lk;
    }
    const T* qrow = reinterpret_cast<const T*>(a.q) + (((int64_t)b * a.Hq + hq) * a.Lq + row) * D;
    T* orow = reinterpret_cast<T*>(a.out) + (((int64_t)b * a.Hq + hq) * a.Lq + row) * D;
    float q[DPL], acc[DPL];
#pragma unroll
    for (int e = 0; e < DPL; ++e) {
        const int dd = lane + 32 * e;
        q[e] = dd < D ? to_f32(qrow[dd]) : 0.f;
        acc[e] = 0.f;
    }
    const float scale = rsqrtf((float)D);
    float m = -INFINITY, l = 0.f;
    const T* kd = reinterpret_cast<const T*>(a.k) + ((int64_t)b * a.Hkv + h) * (int64_t)a.Lk * D;
    const T* vd = reinterpret_cast<const T*>(a.v) + ((int64_t)b * a.Hkv + h) * (int64_t)a.Lk * D;
    const T* kl = nullptr;
    const T* vl = nullptr;
    if (paged) {
        kl = reinterpret_cast<const T*>(reinterpret_cast<const char*>(pv.k_base) + (int64_t)a.layer * pv.layer_stride_bytes);
        vl = reinterpret_cast<const T*>(reinterpret_cast<const char*>(pv.v_base) + (int64_t)a.layer * pv.layer_stride_bytes);
    }
    for (int t = 0; t < n_keys; ++t) {
        const T* kr;
        const T* vr;
        if (paged) {
            const int page = checked_page(pv, seq, t / pv.page_size);
            if (page < 0) continue;
            const int64_t off = row_offset(pv, page, h, t % pv.page_size);
            kr = kl + off;
            vr = vl + off;
        } else {
            kr = kd + (int64_t)t * D;
            vr = vd + (int64_t)t * D;
        }
        float part = 0.f, v[DPL];
#pragma unroll
        for (int e = 0; e < DPL; ++e) {
            const int dd = lane + 32 * e;
            const float kk = dd < D ? to_f32(kr[dd]) : 0.f;
            v[e] = dd < D ? to_f32(vr[dd]) : 0.f;
            part = fmaf(q[e], kk, part);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        const float s = part * scale;
        const float m_new = fmaxf(m, s);
        const float alpha = expf(m - m_new);
        const float p = expf(s - m_new);
        l = l * alpha + p;
#pragma unroll
        for (int e = 0; e < DPL; ++e) acc[e] = acc[e] * alpha + p * v[e];
        m = m_new;
    }
    const float inv = 1.0f / fmaxf(l, a.eps);
#pragma unroll
    for (int e = 0; e < DPL; ++e) {
        const int dd = lane + 32 * e;
        if (dd < D) orow[dd] = from_f32<T>(acc[e] * inv);
    }
}

template <typename T>
cudaError_t launch_t(const DenseAttnLaunch& a, cudaStream_t stream) {
    dim3 grid((unsigned)((a.Lq + kRowsPerBlock - 1) / kRowsPerBlock), (unsigned)a.Hq, (unsigned)a.B);
    const int dpl = (a.D + 31) / 32;
    switch (dpl) {
        case 1: attn_generic_kernel<T, 1><<<grid, kRowsPerBlock * 32, 0, stream>>>(a); break;
        case 2: attn_generic_kernel<T, 2><<<grid, kRowsPerBlock * 32, 0, stream>>>(a); break;
        case 3: attn_generic_kernel<T, 3><<<grid, kRowsPerBlock * 32, 0, stream>>>(a); break;
        case 4: attn_generic_kernel<T, 4><<<grid, kRowsPerBlock * 32, 0, stream>>>(a); break;
        case 5: case 6: attn_generic_kernel<T, 6><<<grid, kRowsPerBlock * 32, 0, stream>>>(a); break;
        default: attn_generic_kernel<T, 8><<<grid, kRowsPerBlock * 32, 0, stream>>>(a); break;
    }
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_attn_generic(const DenseAttnLaunch& a, cudaStream_t stream) {
    count_launches(1);
    return a.dtype == SKV_BF16 ? launch_t<__nv_bfloat16>(a, stream) : launch_t<float>(a, stream);
}

}  // namespace skv
