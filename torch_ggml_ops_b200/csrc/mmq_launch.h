// Host-side launch interface between the C-ABI layer (tgo_api.cu) and the per-quant-type
// instantiations of the GEMM kernel (mmq_inst.cu, compiled once per type).
#pragma once

#include "mmq_gemm.cuh"

namespace tgo {

// launch_gemm_<QT>: launches mmq_gemm_kernel<QT, mode, cta_group, wide> with `grid` persistent CTAs
// (cta_group 2: `grid` is even, CTAs 2i and 2i+1 form a cluster).  Returns a cudaError_t.
// max_pairs_<QT>: how many CTA pairs of that kernel fit on the current device at once.
#define TGO_DECLARE_LAUNCH(QT)                                                                          \
    int launch_gemm_##QT(int mode, int cta_group, int wide, const GemmArgs& args, int grid, cudaStream_t stream); \
    int max_pairs_##QT(int mode);
TGO_DECLARE_LAUNCH(11)
TGO_DECLARE_LAUNCH(12)
TGO_DECLARE_LAUNCH(13)
TGO_DECLARE_LAUNCH(14)
TGO_DECLARE_LAUNCH(22)
#undef TGO_DECLARE_LAUNCH

}  // namespace tgo
