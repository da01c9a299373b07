// Element-wise kernels of the MoE feed-forward block that sits between the grouped projections:
// h = silu(gate) * up (optionally scaled by a per-row routing weight) and its backward.  The
// reference leaves activation and combine to its caller (README.md:3 "fused MoE" is the matmul pair
// only; csrc/mmq_hip.cu:1054-1193 launches gate and up and returns both); these kernels are that
// caller-side step, run on the expert-major rows the grouped operators produce, so that a whole
// expert-parallel MLP step stays on the device.
//
// bf16 in and out, fp32 arithmetic, one rounding per output element.  16 bytes per thread access.
#include "../../include/tgo_mmq.h"

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace tgo {

int route_fail(int code, const char* msg);  // tgo_api.cu

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }

// rows that exist: *n_rows_device (clamped to rows) when given, else rows
__device__ __forceinline__ long long live_rows(const int32_t* n_rows_device, long long rows) {
    if (n_rows_device == nullptr) return rows;
    const long long n = *n_rows_device;
    return n < 0 ? 0 : (n > rows ? rows : n);
}

__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up,
                                                         const float* __restrict__ row_scale, uint4* __restrict__ out,
                                                         long long rows, int vec_per_row, const int32_t* __restrict__ n_rows_device) {
    const long long total = live_rows(n_rows_device, rows) * vec_per_row;
    for (long long v = blockIdx.x * 256LL + threadIdx.x; v < total; v += 256LL * gridDim.x) {
        const uint4 gv = gate[v], uv = up[v];
        const float s = row_scale != nullptr ? row_scale[v / vec_per_row] : 1.0f;
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
            o2[j] = __floats2bfloat162_rn(s * (g.x * sigmoidf_(g.x)) * u.x, s * (g.y * sigmoidf_(g.y)) * u.y);
        }
        out[v] = o;
    }
}

// dgate = dh * s * up * silu'(gate),  dup = dh * s * silu(gate);  silu'(x) = sig(x) * (1 + x * (1 - sig(x)))
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const uint4* __restrict__ dh, const uint4* __restrict__ gate,
                                                         const uint4* __restrict__ up, const float* __restrict__ row_scale,
                                                         uint4* __restrict__ dgate, uint4* __restrict__ dup, long long rows,
                                                         int vec_per_row, const int32_t* __restrict__ n_rows_device) {
    const long long total = live_rows(n_rows_device, rows) * vec_per_row;
    for (long long v = blockIdx.x * 256LL + threadIdx.x; v < total; v += 256LL * gridDim.x) {
        const uint4 dv = dh[v], gv = gate[v], uv = up[v];
        const float s = row_scale != nullptr ? row_scale[v / vec_per_row] : 1.0f;
        const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dv);
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
        uint4 og, ou;
        __nv_bfloat162* og2 = reinterpret_cast<__nv_bfloat162*>(&og);
        __nv_bfloat162* ou2 = reinterpret_cast<__nv_bfloat162*>(&ou);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 d = __bfloat1622float2(d2[j]), g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
            const float sx = sigmoidf_(g.x), sy = sigmoidf_(g.y);
            const float dx = d.x * s, dy = d.y * s;
            og2[j] = __floats2bfloat162_rn(dx * u.x * (sx * (1.0f + g.x * (1.0f - sx))), dy * u.y * (sy * (1.0f + g.y * (1.0f - sy))));
            ou2[j] = __floats2bfloat162_rn(dx * (g.x * sx), dy * (g.y * sy));
        }
        dgate[v] = og;
        dup[v] = ou;
    }
}

static int moe_grid(long long work_items) {
    long long blocks = (work_items + 255) / 256;
    if (blocks > 148LL * 16) blocks = 148LL * 16;
    return static_cast<int>(blocks < 1 ? 1 : blocks);
}
static bool a16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace tgo

using namespace tgo;

extern "C" {

int tgo_swiglu_fwd(const void* gate, const void* up, const float* row_scale, void* out, int64_t rows, int64_t width,
                   const int32_t* n_rows_device, void* stream) {
    if (gate == nullptr || up == nullptr || out == nullptr) return route_fail(TGO_E_ARG, "null pointer");
    if (rows <= 0 || width <= 0 || (width * 2) % 16 != 0)
        return route_fail(TGO_E_ARG, "swiglu needs rows > 0 and a row length that is a multiple of 8");
    if (!a16(gate) || !a16(up) || !a16(out)) return route_fail(TGO_E_ARG, "data pointers must be 16-byte aligned");
    const int vec = static_cast<int>(width / 8);
    swiglu_fwd_kernel<<<moe_grid(rows * vec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(gate), static_cast<const uint4*>(up), row_scale, static_cast<uint4*>(out), rows, vec,
        n_rows_device);
    return cudaGetLastError() == cudaSuccess ? TGO_OK : route_fail(TGO_E_CUDA, "swiglu_fwd_kernel launch failed");
}

int tgo_swiglu_bwd(const void* dh, const void* gate, const void* up, const float* row_scale, void* dgate, void* dup,
                   int64_t rows, int64_t width, const int32_t* n_rows_device, void* stream) {
    if (dh == nullptr || gate == nullptr || up == nullptr || dgate == nullptr || dup == nullptr)
        return route_fail(TGO_E_ARG, "null pointer");
    if (rows <= 0 || width <= 0 || (width * 2) % 16 != 0)
        return route_fail(TGO_E_ARG, "swiglu needs rows > 0 and a row length that is a multiple of 8");
    if (!a16(dh) || !a16(gate) || !a16(up) || !a16(dgate) || !a16(dup))
        return route_fail(TGO_E_ARG, "data pointers must be 16-byte aligned");
    const int vec = static_cast<int>(width / 8);
    swiglu_bwd_kernel<<<moe_grid(rows * vec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(dh), static_cast<const uint4*>(gate), static_cast<const uint4*>(up), row_scale,
        static_cast<uint4*>(dgate), static_cast<uint4*>(dup), rows, vec, n_rows_device);
    return cudaGetLastError() == cudaSuccess ? TGO_OK : route_fail(TGO_E_CUDA, "swiglu_bwd_kernel launch failed");
}

}  // extern "C"
