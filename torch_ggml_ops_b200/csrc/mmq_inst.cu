// One translation unit per quant type (compile with -DTGO_QT=<ggml type id>): instantiates the
// forward and backward GEMM kernels for that type, as single-CTA kernels and as CTA-pair
// (cluster of two) kernels, and their launch functions.
#include <atomic>

#include "mmq_launch.h"

#ifndef TGO_QT
#error "compile with -DTGO_QT=<11|12|13|14|22>"
#endif

namespace tgo {

template <int QT, int MODE, int CG, int WIDE, int SPLIT>
static cudaError_t configure() {
    using Cfg = GemmCfg<QT, MODE, CG, WIDE>;
    // relaxed atomics: threads that race on a device's first call set the same attribute and flag
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 64 && configured[dev].load(std::memory_order_relaxed)) return cudaSuccess;
    e = cudaFuncSetAttribute(mmq_gemm_kernel<QT, MODE, CG, WIDE, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg::kSmemBytes);
    if (e != cudaSuccess) return e;
    if (dev < 64) configured[dev].store(true, std::memory_order_relaxed);
    return cudaSuccess;
}

template <int QT, int MODE, int CG, int WIDE, int SPLIT>
static void fill_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute& attr, int grid, cudaStream_t stream) {
    using Cfg = GemmCfg<QT, MODE, CG, WIDE>;
    cfg = cudaLaunchConfig_t{};
    cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = stream;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = CG;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
}

template <int QT, int MODE, int CG, int WIDE, int SPLIT>
static int launch_one(const GemmArgs& args, int grid, cudaStream_t stream) {
    cudaError_t e = configure<QT, MODE, CG, WIDE, SPLIT>();
    if (e != cudaSuccess) return static_cast<int>(e);
    if (CG == 1) {
        mmq_gemm_kernel<QT, MODE, CG, WIDE, SPLIT><<<grid, kGemmThreads, GemmCfg<QT, MODE, CG, WIDE>::kSmemBytes, stream>>>(args);
        return static_cast<int>(cudaGetLastError());
    }
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr;
    fill_config<QT, MODE, CG, WIDE, SPLIT>(cfg, attr, grid, stream);
    return static_cast<int>(cudaLaunchKernelEx(&cfg, mmq_gemm_kernel<QT, MODE, CG, WIDE, SPLIT>, args));
}

// the kernel variant for this launch: wide tiles, or (backward only) a split reduction, or neither
template <int QT, int MODE, int CG>
static int launch_width(int wide, const GemmArgs& args, int grid, cudaStream_t stream) {
    if (MODE == kBwd && args.nsplit > 1) return launch_one<QT, kBwd, CG, 0, 1>(args, grid, stream);
    return wide ? launch_one<QT, MODE, CG, 1, 0>(args, grid, stream) : launch_one<QT, MODE, CG, 0, 0>(args, grid, stream);
}

// Most CTA pairs of this kernel that can be resident at once on the current device (0: pairs
// cannot be launched here).
template <int QT, int MODE>
static int max_pairs_one() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (dev < 64) {
        const int c = cached[dev].load(std::memory_order_relaxed);
        if (c != 0) return c > 0 ? c : 0;
    }
    int n = 0;
    if (configure<QT, MODE, 2, 0, 0>() == cudaSuccess) {   // both tile widths use the same threads and shared memory
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr;
        int sms = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        fill_config<QT, MODE, 2, 0, 0>(cfg, attr, sms & ~1, nullptr);
        if (cudaOccupancyMaxActiveClusters(&n, mmq_gemm_kernel<QT, MODE, 2, 0, 0>, &cfg) != cudaSuccess) {
            (void)cudaGetLastError();
            n = 0;
        }
    } else {
        (void)cudaGetLastError();
    }
    if (dev < 64) cached[dev].store(n > 0 ? n : -1, std::memory_order_relaxed);
    return n;
}

#define TGO_CAT2(a, b) a##b
#define TGO_CAT(a, b) TGO_CAT2(a, b)

int TGO_CAT(launch_gemm_, TGO_QT)(int mode, int cta_group, int wide, const GemmArgs& args, int grid, cudaStream_t stream) {
    if (cta_group == 2)
        return mode == kFwd ? launch_width<TGO_QT, kFwd, 2>(wide, args, grid, stream)
                            : launch_width<TGO_QT, kBwd, 2>(wide, args, grid, stream);
    return mode == kFwd ? launch_width<TGO_QT, kFwd, 1>(wide, args, grid, stream)
                        : launch_width<TGO_QT, kBwd, 1>(wide, args, grid, stream);
}

int TGO_CAT(max_pairs_, TGO_QT)(int mode) {
    return mode == kFwd ? max_pairs_one<TGO_QT, kFwd>() : max_pairs_one<TGO_QT, kBwd>();
}

}  // namespace tgo
