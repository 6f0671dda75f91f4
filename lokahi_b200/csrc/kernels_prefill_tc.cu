// K4: causal chunked-prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM, TMA-fed).
#include "common.cuh"

namespace skv {

cudaError_t launch_attn_tc(const DenseAttnLaunch& a, cudaStream_t stream) {
    (void)a;
    (void)stream;
    return cudaErrorNotSupported;
}

}  // namespace skv
