// Device helpers shared by the kernels.
#pragma once

#include <cuda_bf16.h>
#include <cstdlib>
#include <cuda_runtime.h>
#include <stdint.h>

#include "skv_internal.h"

namespace skv {

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// Programmatic dependent launch: a kernel launched with launch_pdl may start while the previous kernel in
// the stream is still draining; it must execute pdl_wait() before it reads anything that kernel wrote
// (the wait returns once the previous grid has completed and its writes are visible).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Page id of (sequence, slot) with range checks: a bad id sets a bit in the status word and the
// caller skips the access instead of faulting.
__device__ __forceinline__ int32_t checked_page(const PoolView& pv, int32_t seq, int32_t slot) {
    if (slot < 0 || slot >= pv.max_pages_per_seq) {
        atomicOr(pv.status, FLAG_BAD_LENGTH);
        return -1;
    }
    int32_t page = pv.page_table[(int64_t)seq * pv.max_pages_per_seq + slot];
    if (page < 0 || page >= pv.num_pages) {
        atomicOr(pv.status, FLAG_BAD_PAGE);
        return -1;
    }
    return page;
}

__device__ __forceinline__ bool checked_seq(const PoolView& pv, int32_t seq) {
    if (seq < 0 || seq >= pv.max_seqs) {
        atomicOr(pv.status, FLAG_BAD_SEQ);
        return false;
    }
    return true;
}

// Element offset of token row (page, head, row) inside one layer's K (or V) pool.
__device__ __forceinline__ int64_t row_offset(const PoolView& pv, int32_t page, int32_t head, int32_t row) {
    return (((int64_t)page * pv.num_kv_heads + head) * pv.page_size + row) * pv.head_dim;
}

#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    const bool enabled = switches().pdl != 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = enabled ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

}  // namespace skv
