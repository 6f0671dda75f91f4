// Decoder glue on either side of the hot path: RMSNorm (optionally fused with the residual add that precedes it)
// and the SwiGLU activation product.  Both are bandwidth-bound element-wise passes; fusing them removes the chain
// of small launches (square, mean, add, rsqrt, two multiplies, cast; sigmoid, two multiplies) that keeps a cached
// decode step launch-bound.
//
// Arithmetic follows the reference's float32 formulation:
//   RMSNorm  w * (x * rsqrt(mean(x^2) + eps))          MLXRMSNorm, src/ollm/llama_mlx.py:77-92; fused twins
//                                                        optimized_rmsnorm / optimized_rmsnorm_residual,
//                                                        src/ollm/metal_optimizations.py:75-117
//   SwiGLU   (gate * sigmoid(gate)) * up                 MLXLlamaMLP, llama_mlx.py:345-408; optimized_swiglu,
//                                                        metal_optimizations.py:140-157
// Inputs and outputs are in the storage dtype (float32 or bfloat16), everything in between is float32, and each
// output element is rounded once.
#include "common.cuh"
#include "strata_b200.h"

namespace skv {

namespace {

constexpr int kNormThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = lane < (int)(blockDim.x >> 5) ? red[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;   // every thread holds the block total
}

// One block per row.  VEC elements (16 bytes) per access when `vec` is set (hidden a multiple of VEC and all
// rows 16-byte aligned), one element otherwise.  With `delta`, the row that is normalised is x + delta, and that
// sum is also written to `sum_out` (the updated residual stream); `sum_out` may alias x.
template <typename T>
__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(const T* x /* may alias sum_out */, const T* __restrict__ delta, T* sum_out,
                                                              const T* __restrict__ weight, T* __restrict__ out, int hidden,
                                                              float eps, int vec) {
    constexpr int VEC = 16 / (int)sizeof(T);
    __shared__ float red[kNormThreads / 32];
    extern __shared__ float row[];               // the row in float32, so that x (+ delta) is read from memory once
    const int64_t base = (int64_t)blockIdx.x * hidden;
    float ss = 0.f;
    if (vec) {
        for (int c = threadIdx.x; c < hidden / VEC; c += blockDim.x) {
            uint4 a = *reinterpret_cast<const uint4*>(x + base + (int64_t)c * VEC);
            T* ae = reinterpret_cast<T*>(&a);
            if (delta) {
                const uint4 b = *reinterpret_cast<const uint4*>(delta + base + (int64_t)c * VEC);
                const T* be = reinterpret_cast<const T*>(&b);
#pragma unroll
                for (int e = 0; e < VEC; ++e) ae[e] = from_f32<T>(__fadd_rn(to_f32(ae[e]), to_f32(be[e])));   // rounded like a stored sum
                *reinterpret_cast<uint4*>(sum_out + base + (int64_t)c * VEC) = a;
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                const float f = to_f32(ae[e]);
                row[c * VEC + e] = f;
                ss = fmaf(f, f, ss);
            }
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
            T a = x[base + i];
            if (delta) {
                a = from_f32<T>(__fadd_rn(to_f32(a), to_f32(delta[base + i])));
                sum_out[base + i] = a;
            }
            const float f = to_f32(a);
            row[i] = f;
            ss = fmaf(f, f, ss);
        }
    }
    const float total = block_sum(ss, red);      // also orders the writes to `row` before the reads below
    const float inv = rsqrtf(total / (float)hidden + eps);
    if (vec) {
        for (int c = threadIdx.x; c < hidden / VEC; c += blockDim.x) {
            const uint4 w = *reinterpret_cast<const uint4*>(weight + (int64_t)c * VEC);
            const T* we = reinterpret_cast<const T*>(&w);
            uint4 o;
            T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
            for (int e = 0; e < VEC; ++e) oe[e] = from_f32<T>(to_f32(we[e]) * (row[c * VEC + e] * inv));
            *reinterpret_cast<uint4*>(out + base + (int64_t)c * VEC) = o;
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[base + i] = from_f32<T>(to_f32(weight[i]) * (row[i] * inv));
    }
}

// Warp-per-row variant for rows of exactly 32 * CPL 16-byte chunks (hidden = 256 * CPL bf16 or 128 * CPL float32
// elements): the row lives in registers, the sum of squares is a warp reduction, and a block of eight warps
// covers eight rows, so short rows do not pay for a block barrier and a block launch each (measured at 16384 rows
// of 2048 bf16: 0.049 ms per call with one block per row).
template <typename T, int CPL>
__global__ void __launch_bounds__(256) rmsnorm_warp_kernel(const T* x /* may alias sum_out */, const T* __restrict__ delta, T* sum_out,
                                                           const T* __restrict__ weight, T* __restrict__ out, int64_t n_rows,
                                                           float eps) {
    constexpr int VEC = 16 / (int)sizeof(T);
    constexpr int hidden = 32 * CPL * VEC;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int64_t base = row * hidden;
    uint4 v[CPL];
#pragma unroll
    for (int k = 0; k < CPL; ++k) v[k] = *reinterpret_cast<const uint4*>(x + base + (int64_t)(k * 32 + lane) * VEC);
    if (delta) {
#pragma unroll
        for (int k = 0; k < CPL; ++k) {
            const uint4 b = *reinterpret_cast<const uint4*>(delta + base + (int64_t)(k * 32 + lane) * VEC);
            T* ae = reinterpret_cast<T*>(&v[k]);
            const T* be = reinterpret_cast<const T*>(&b);
#pragma unroll
            for (int e = 0; e < VEC; ++e) ae[e] = from_f32<T>(__fadd_rn(to_f32(ae[e]), to_f32(be[e])));
            *reinterpret_cast<uint4*>(sum_out + base + (int64_t)(k * 32 + lane) * VEC) = v[k];
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < CPL; ++k) {
        const T* ae = reinterpret_cast<const T*>(&v[k]);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const float f = to_f32(ae[e]);
            ss = fmaf(f, f, ss);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss / (float)hidden + eps);
#pragma unroll
    for (int k = 0; k < CPL; ++k) {
        const uint4 w = *reinterpret_cast<const uint4*>(weight + (int64_t)(k * 32 + lane) * VEC);
        const T* we = reinterpret_cast<const T*>(&w);
        const T* ae = reinterpret_cast<const T*>(&v[k]);
        uint4 o;
        T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int e = 0; e < VEC; ++e) oe[e] = from_f32<T>(to_f32(we[e]) * (to_f32(ae[e]) * inv));
        *reinterpret_cast<uint4*>(out + base + (int64_t)(k * 32 + lane) * VEC) = o;
    }
}

template <typename T>
__global__ void __launch_bounds__(256) swiglu_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out,
                                                     int64_t n, int vec) {
    constexpr int VEC = 16 / (int)sizeof(T);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < n / VEC; c += stride) {
            const uint4 g = *reinterpret_cast<const uint4*>(gate + c * VEC);
            const uint4 u = *reinterpret_cast<const uint4*>(up + c * VEC);
            const T* ge = reinterpret_cast<const T*>(&g);
            const T* ue = reinterpret_cast<const T*>(&u);
            uint4 o;
            T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                const float gf = to_f32(ge[e]);
                oe[e] = from_f32<T>((gf * (1.0f / (1.0f + expf(-gf)))) * to_f32(ue[e]));
            }
            *reinterpret_cast<uint4*>(out + c * VEC) = o;
        }
    } else {
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
            const float gf = to_f32(gate[i]);
            out[i] = from_f32<T>((gf * (1.0f / (1.0f + expf(-gf)))) * to_f32(up[i]));
        }
    }
}

// SwiGLU over rows with their own strides: gate and up may be the two halves of one fused projection output
// [n_rows][2 * cols] (row stride 2 * cols), out a packed [n_rows][cols].  One block walks rows; 16-byte accesses when
// everything is 16-byte aligned.
template <typename T>
__global__ void __launch_bounds__(256) swiglu_rows_kernel(const T* __restrict__ gate, const T* __restrict__ up, T* __restrict__ out,
                                                          int64_t n_rows, int cols, int64_t gate_stride, int64_t up_stride,
                                                          int64_t out_stride, int vec) {
    constexpr int VEC = 16 / (int)sizeof(T);
    const int per_row = vec ? cols / VEC : cols;
    const int64_t total = n_rows * per_row;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t r = idx / per_row;
        const int c = (int)(idx - r * per_row);
        if (vec) {
            const uint4 g = *reinterpret_cast<const uint4*>(gate + r * gate_stride + (int64_t)c * VEC);
            const uint4 u = *reinterpret_cast<const uint4*>(up + r * up_stride + (int64_t)c * VEC);
            const T* ge = reinterpret_cast<const T*>(&g);
            const T* ue = reinterpret_cast<const T*>(&u);
            uint4 o;
            T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                const float gf = to_f32(ge[e]);
                oe[e] = from_f32<T>((gf * (1.0f / (1.0f + expf(-gf)))) * to_f32(ue[e]));
            }
            *reinterpret_cast<uint4*>(out + r * out_stride + (int64_t)c * VEC) = o;
        } else {
            const float gf = to_f32(gate[r * gate_stride + c]);
            out[r * out_stride + c] = from_f32<T>((gf * (1.0f / (1.0f + expf(-gf)))) * to_f32(up[r * up_stride + c]));
        }
    }
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

template <typename T>
cudaError_t run_rmsnorm(const void* x, const void* delta, void* sum_out, const void* weight, void* out, int64_t n_rows,
                        int32_t hidden, float eps, cudaStream_t stream) {
    constexpr int VEC = 16 / (int)sizeof(T);
    const bool vec = hidden % VEC == 0 && aligned16(x) && aligned16(weight) && aligned16(out) &&
                     (!delta || (aligned16(delta) && aligned16(sum_out)));
    if (vec && hidden % (32 * VEC) == 0) {
        const int cpl = hidden / (32 * VEC);
        const unsigned blocks = (unsigned)((n_rows + 7) / 8);
        auto launch = [&](auto kernel) {
            kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const T*>(x), reinterpret_cast<const T*>(delta),
                                               reinterpret_cast<T*>(sum_out), reinterpret_cast<const T*>(weight),
                                               reinterpret_cast<T*>(out), n_rows, eps);
            count_launches(1);
            return cudaGetLastError();
        };
        switch (cpl) {
            case 1: return launch(rmsnorm_warp_kernel<T, 1>);
            case 2: return launch(rmsnorm_warp_kernel<T, 2>);
            case 4: return launch(rmsnorm_warp_kernel<T, 4>);
            case 8: return launch(rmsnorm_warp_kernel<T, 8>);
            case 16: return launch(rmsnorm_warp_kernel<T, 16>);
            default: break;   // other sizes: one block per row below
        }
    }
    const size_t smem = (size_t)hidden * sizeof(float);
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || !configured[dev])) {
        cudaError_t e = cudaFuncSetAttribute(rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    rmsnorm_kernel<T><<<(unsigned)n_rows, kNormThreads, smem, stream>>>(
        reinterpret_cast<const T*>(x), reinterpret_cast<const T*>(delta), reinterpret_cast<T*>(sum_out),
        reinterpret_cast<const T*>(weight), reinterpret_cast<T*>(out), hidden, eps, vec ? 1 : 0);
    count_launches(1);
    return cudaGetLastError();
}

template <typename T>
cudaError_t run_swiglu(const void* gate, const void* up, void* out, int64_t n, cudaStream_t stream) {
    constexpr int VEC = 16 / (int)sizeof(T);
    const bool vec = n % VEC == 0 && aligned16(gate) && aligned16(up) && aligned16(out);
    const int64_t items = vec ? n / VEC : n;
    int64_t blocks = (items + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;    // grid-stride beyond 16 blocks per SM
    if (blocks < 1) blocks = 1;
    swiglu_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<const T*>(gate), reinterpret_cast<const T*>(up),
                                                          reinterpret_cast<T*>(out), n, vec ? 1 : 0);
    count_launches(1);
    return cudaGetLastError();
}

template <typename T>
cudaError_t run_swiglu_rows(const void* gate, const void* up, void* out, int64_t n_rows, int32_t cols, int64_t gs, int64_t us,
                            int64_t os, cudaStream_t stream) {
    constexpr int VEC = 16 / (int)sizeof(T);
    const bool vec = cols % VEC == 0 && gs % VEC == 0 && us % VEC == 0 && os % VEC == 0 && aligned16(gate) && aligned16(up) &&
                     aligned16(out);
    const int64_t items = n_rows * (vec ? cols / VEC : cols);
    int64_t blocks = (items + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    swiglu_rows_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<const T*>(gate), reinterpret_cast<const T*>(up),
                                                               reinterpret_cast<T*>(out), n_rows, cols, gs, us, os, vec ? 1 : 0);
    count_launches(1);
    return cudaGetLastError();
}

}  // namespace

}  // namespace skv

extern "C" {

int32_t skv_swiglu_rows(const void* gate, const void* up, void* out, int64_t n_rows, int32_t cols, int64_t gate_row_stride,
                        int64_t up_row_stride, int64_t out_row_stride, int32_t dtype, void* stream) {
    if (!gate || !up || !out || n_rows < 0 || cols <= 0 || gate_row_stride < cols || up_row_stride < cols || out_row_stride < cols)
        return SKV_ERR_BAD_ARG;
    if (dtype != SKV_F32 && dtype != SKV_BF16) return SKV_ERR_BAD_ARG;
    if (n_rows == 0) return SKV_OK;
    cudaError_t e = dtype == SKV_BF16
                        ? skv::run_swiglu_rows<__nv_bfloat16>(gate, up, out, n_rows, cols, gate_row_stride, up_row_stride,
                                                              out_row_stride, (cudaStream_t)stream)
                        : skv::run_swiglu_rows<float>(gate, up, out, n_rows, cols, gate_row_stride, up_row_stride, out_row_stride,
                                                      (cudaStream_t)stream);
    return e == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}

int32_t skv_rmsnorm(const void* x, const void* delta, void* sum_out, const void* weight, void* out, int64_t n_rows, int32_t hidden,
                    float eps, int32_t dtype, void* stream) {
    if (!x || !weight || !out || n_rows < 0 || hidden <= 0 || hidden > 49152 || !(eps >= 0.0f)) return SKV_ERR_BAD_ARG;
    if (delta && !sum_out) return SKV_ERR_BAD_ARG;
    if (dtype != SKV_F32 && dtype != SKV_BF16) return SKV_ERR_BAD_ARG;
    if (n_rows == 0) return SKV_OK;
    cudaError_t e = dtype == SKV_BF16
                        ? skv::run_rmsnorm<__nv_bfloat16>(x, delta, sum_out, weight, out, n_rows, hidden, eps, (cudaStream_t)stream)
                        : skv::run_rmsnorm<float>(x, delta, sum_out, weight, out, n_rows, hidden, eps, (cudaStream_t)stream);
    return e == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}

int32_t skv_swiglu(const void* gate, const void* up, void* out, int64_t n, int32_t dtype, void* stream) {
    if (!gate || !up || !out || n < 0) return SKV_ERR_BAD_ARG;
    if (dtype != SKV_F32 && dtype != SKV_BF16) return SKV_ERR_BAD_ARG;
    if (n == 0) return SKV_OK;
    cudaError_t e = dtype == SKV_BF16 ? skv::run_swiglu<__nv_bfloat16>(gate, up, out, n, (cudaStream_t)stream)
                                      : skv::run_swiglu<float>(gate, up, out, n, (cudaStream_t)stream);
    return e == cudaSuccess ? SKV_OK : SKV_ERR_CUDA;
}

}  // extern "C"
