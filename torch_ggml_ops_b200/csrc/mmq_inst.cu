// One translation unit per quant type (compile with -DTGO_QT=<ggml type id>): instantiates the
// forward and backward GEMM kernels for that type and their launch function.
#include "mmq_launch.h"

#ifndef TGO_QT
#error "compile with -DTGO_QT=<11|12|13|14|22>"
#endif

namespace tgo {

template <int QT, int MODE>
static int launch_one(const GemmArgs& args, int grid, cudaStream_t stream) {
    using Cfg = GemmCfg<QT, MODE>;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 64 && !configured[dev]) {
        e = cudaFuncSetAttribute(mmq_gemm_kernel<QT, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg::kSmemBytes);
        if (e != cudaSuccess) return static_cast<int>(e);
        configured[dev] = true;
    }
    mmq_gemm_kernel<QT, MODE><<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(args);
    return static_cast<int>(cudaGetLastError());
}

#define TGO_CAT2(a, b) a##b
#define TGO_CAT(a, b) TGO_CAT2(a, b)

int TGO_CAT(launch_gemm_, TGO_QT)(int mode, const GemmArgs& args, int grid, cudaStream_t stream) {
    return mode == kFwd ? launch_one<TGO_QT, kFwd>(args, grid, stream)
                        : launch_one<TGO_QT, kBwd>(args, grid, stream);
}

}  // namespace tgo
