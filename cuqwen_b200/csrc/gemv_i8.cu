// Instantiations of the GEMV kernel family for one weight format.
#include "gemv_kernel.cuh"
#include "launch.h"

namespace cq {

template <int EPI>
static int go(const GemvArgs& a, dim3 grid, dim3 block, size_t smem, const LaunchCfg& cfg) {
    cudaLaunchConfig_t lc = {};
    lc.gridDim = grid; lc.blockDim = block; lc.dynamicSmemBytes = smem; lc.stream = cfg.stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = cfg.pdl ? 1 : 0;
    {
        // Every kernel of the step asks for the largest shared-memory carveout: CTAs of two consecutive kernels can only
        // share an SM (the second one prefetching its weights while the first still runs) when both run under the same
        // L1 / shared-memory split.
        static bool once = false;
        if (!once) {
            cudaError_t e = cudaFuncSetAttribute(gemv_kernel<Q_I8, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_kernel<Q_I8, EPI>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            if (e != cudaSuccess) return (int)e;
            once = true;
        }
    }
    return (int)cudaLaunchKernelEx(&lc, gemv_kernel<Q_I8, EPI>, a);
}

int launch_gemv_i8(int epi, const GemvArgs& a, dim3 grid, dim3 block, size_t smem, const LaunchCfg& cfg) {
    switch (epi) {
        case EPI_F16: return go<EPI_F16>(a, grid, block, smem, cfg);
        case EPI_F32: return go<EPI_F32>(a, grid, block, smem, cfg);
        case EPI_RESID: return go<EPI_RESID>(a, grid, block, smem, cfg);
        case EPI_SWIGLU: return go<EPI_SWIGLU>(a, grid, block, smem, cfg);
        case EPI_QKV: return go<EPI_QKV>(a, grid, block, smem, cfg);
        case EPI_PUSH: return go<EPI_PUSH>(a, grid, block, smem, cfg);
    }
    return (int)cudaErrorInvalidValue;
}

}  // namespace cq
