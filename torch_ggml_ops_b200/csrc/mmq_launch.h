// Host-side launch interface between the C-ABI layer (tgo_api.cu) and the per-quant-type
// instantiations of the GEMM kernel (mmq_inst.cu, compiled once per type).
#pragma once

#include "mmq_gemm.cuh"

namespace tgo {

// Launches mmq_gemm_kernel<QT, mode> with `grid` persistent CTAs.  Returns a cudaError_t.
#define TGO_DECLARE_LAUNCH(QT) int launch_gemm_##QT(int mode, const GemmArgs& args, int grid, cudaStream_t stream);
TGO_DECLARE_LAUNCH(11)
TGO_DECLARE_LAUNCH(12)
TGO_DECLARE_LAUNCH(13)
TGO_DECLARE_LAUNCH(14)
TGO_DECLARE_LAUNCH(22)
#undef TGO_DECLARE_LAUNCH

}  // namespace tgo
