// Device-side routing helpers for the grouped operators: a stable counting sort of routed
// (token, slot) pairs by expert id that yields the row permutation and the cumulative end
// offsets the grouped kernels consume, plus the row gather and the weighted top-k combine that sit
// either side of the expert projections.
//
// The reference leaves this to its callers (rows must arrive pre-sorted with int64 expert ids and
// int32 cumulative end offsets: csrc/mmq_hip.cu:325-406, docs/grouped_mmq_fwd_optimization.md:41-47);
// its only device prefix sum is the row-task builder (csrc/mmq_core.cuh:516-571).  Nothing here
// reads routing data back to the host: every expert gets a group (empty ones included), so the
// group count is the static expert count.
#include "../../include/tgo_mmq.h"

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace tgo {

int route_fail(int code, const char* msg);  // defined in tgo_api.cu (sets the thread's error text)

constexpr int kRouteBlock = 256;   // routed pairs per block, one per thread
constexpr int kRouteMaxExperts = 4096;

// Pass 1: per-block histogram of expert ids -> block_counts[block][expert].
__global__ void __launch_bounds__(kRouteBlock) route_count_kernel(const int32_t* __restrict__ ids, int n, int num_experts,
                                                                  int32_t* __restrict__ block_counts) {
    extern __shared__ int32_t hist[];
    for (int e = threadIdx.x; e < num_experts; e += kRouteBlock) hist[e] = 0;
    __syncthreads();
    const int i = blockIdx.x * kRouteBlock + threadIdx.x;
    if (i < n) {
        const int e = ids[i];
        if (e >= 0 && e < num_experts) atomicAdd(&hist[e], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < num_experts; e += kRouteBlock)
        block_counts[static_cast<size_t>(blockIdx.x) * num_experts + e] = hist[e];
}

// Pass 2 (one block): per expert, exclusive prefix over the blocks; then the prefix over experts.
// block_counts[b][e] becomes the first row of block b's pairs for expert e inside that expert's
// run of sorted rows (the scatter pass adds the expert's first row, expert_offsets[e - 1]).
__global__ void __launch_bounds__(1024) route_scan_kernel(int32_t* __restrict__ block_counts, int num_blocks,
                                                          int num_experts, int64_t* __restrict__ expert_indices,
                                                          int32_t* __restrict__ expert_offsets,
                                                          int32_t* __restrict__ expert_counts) {
    __shared__ int32_t totals[kRouteMaxExperts];
    __shared__ int32_t warp_sums[32];
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
        int32_t run = 0;
        int b = 0;
        // sixteen independent loads in flight per round trip to L2, then the running sum
        for (; b + 16 <= num_blocks; b += 16) {
            int32_t v[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) v[u] = block_counts[static_cast<size_t>(b + u) * num_experts + e];
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                block_counts[static_cast<size_t>(b + u) * num_experts + e] = run;
                run += v[u];
            }
        }
        for (; b < num_blocks; ++b) {
            const size_t k = static_cast<size_t>(b) * num_experts + e;
            const int32_t v = block_counts[k];
            block_counts[k] = run;
            run += v;
        }
        totals[e] = run;
    }
    __syncthreads();
    // exclusive scan of totals[] in chunks of blockDim.x
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    int32_t carry = 0;
    for (int e0 = 0; e0 < num_experts; e0 += blockDim.x) {
        const int e = e0 + threadIdx.x;
        const int32_t v = e < num_experts ? totals[e] : 0;
        int32_t incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int32_t u = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= d) incl += u;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int32_t w = lane < nwarps ? warp_sums[lane] : 0;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int32_t u = __shfl_up_sync(0xFFFFFFFFu, w, d);
                if (lane >= d) w += u;
            }
            warp_sums[lane] = w;
        }
        __syncthreads();
        const int32_t before = carry + (warp > 0 ? warp_sums[warp - 1] : 0) + incl - v;
        if (e < num_experts) {
            totals[e] = before;                    // first sorted row of expert e
            expert_offsets[e] = before + v;        // cumulative end row
            expert_indices[e] = e;
            if (expert_counts != nullptr) expert_counts[e] = v;
        }
        carry += warp_sums[nwarps - 1];
        __syncthreads();
    }
}

// Pass 3: stable placement.  Warps of a block take turns so that earlier pairs get earlier rows.
__global__ void __launch_bounds__(kRouteBlock) route_scatter_kernel(const int32_t* __restrict__ ids, int n, int num_experts,
                                                                    const int32_t* __restrict__ block_starts,
                                                                    const int32_t* __restrict__ expert_offsets,
                                                                    int32_t* __restrict__ sorted_to_pair,
                                                                    int32_t* __restrict__ pair_to_sorted) {
    extern __shared__ int32_t cursor[];
    for (int e = threadIdx.x; e < num_experts; e += kRouteBlock)
        cursor[e] = block_starts[static_cast<size_t>(blockIdx.x) * num_experts + e] + (e > 0 ? expert_offsets[e - 1] : 0);
    __syncthreads();
    const int i = blockIdx.x * kRouteBlock + threadIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int e = -1;
    if (i < n) {
        e = ids[i];
        if (e < 0 || e >= num_experts) e = -1;
    }
    for (int w = 0; w < kRouteBlock / 32; ++w) {
        if (warp == w) {
            const unsigned peers = __match_any_sync(0xFFFFFFFFu, e);
            if (e >= 0) {
                const int rank = __popc(peers & ((1u << lane) - 1u));
                const int pos = cursor[e] + rank;
                sorted_to_pair[pos] = i;
                pair_to_sorted[i] = pos;
                __syncwarp(peers);
                if (rank == 0) cursor[e] += __popc(peers);
            } else if (i < n) {
                pair_to_sorted[i] = -1;  // invalid expert id: the pair is dropped
            }
        }
        __syncthreads();
    }
}

// dst[r][:] = src[index[r] / divisor][:], rows of `width` bf16 (width * 2 a multiple of 16); an
// index that is negative or names a row at or beyond src_rows gives a row of zeros.
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ src, long long src_rows,
                                                          const int32_t* __restrict__ index, int divisor,
                                                          uint4* __restrict__ dst, long long n_rows, int vec_per_row) {
    const long long total = n_rows * vec_per_row;
    for (long long v = blockIdx.x * 256LL + threadIdx.x; v < total; v += 256LL * gridDim.x) {
        const long long r = v / vec_per_row;
        const int c = static_cast<int>(v - r * vec_per_row);
        const int s = index[r];
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (s >= 0 && s / divisor < src_rows) val = src[static_cast<long long>(s / divisor) * vec_per_row + c];
        dst[v] = val;
    }
}

// out[t][:] = sum_slot weight[t][slot] * rows[pair_to_sorted[t*top_k+slot]][:] in fp32, rounded once.
__global__ void __launch_bounds__(256) combine_rows_kernel(const uint4* __restrict__ rows, const int32_t* __restrict__ pair_to_sorted,
                                                           const float* __restrict__ weights, uint4* __restrict__ out,
                                                           long long tokens, int top_k, int vec_per_row) {
    const long long total = tokens * vec_per_row;
    for (long long v = blockIdx.x * 256LL + threadIdx.x; v < total; v += 256LL * gridDim.x) {
        const long long t = v / vec_per_row;
        const int c = static_cast<int>(v - t * vec_per_row);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < top_k; ++s) {
            const int r = pair_to_sorted[t * top_k + s];
            if (r < 0) continue;
            const float w = weights != nullptr ? weights[t * top_k + s] : 1.0f;
            const uint4 val = rows[static_cast<long long>(r) * vec_per_row + c];
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&val);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h[j]);
                acc[2 * j] = fmaf(w, f.x, acc[2 * j]);
                acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]);
            }
        }
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        out[v] = o;
    }
}

// bf16 activations -> q8_1-style blocks of 32: int8 quants, fp32 scale d = amax / 127, fp32 sum of
// the unquantised values (reference: quantize_bf16_mmq_q8_1, csrc/mmq_core.cuh:151-209, which
// stores d and the sum in fp16 for the Q4_K / Q5_K layout; fp32 is kept here).
__global__ void __launch_bounds__(256) quantize_q8_kernel(const uint4* __restrict__ x, long long n_vec, int8_t* __restrict__ q,
                                                          float* __restrict__ d, float* __restrict__ sum) {
    // warp-uniform trip count: every lane takes part in the shuffles, out-of-range lanes hold zeros
    const int lane = threadIdx.x & 31;
    for (long long w = blockIdx.x * 256LL + (threadIdx.x - lane); w < n_vec; w += 256LL * gridDim.x) {
        const long long v = w + lane;
        const bool valid = v < n_vec;  // n_vec is a multiple of 4: the 4 lanes of a block agree
        const uint4 val = valid ? x[v] : make_uint4(0u, 0u, 0u, 0u);  // 8 consecutive values
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&val);
        float f[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 p = __bfloat1622float2(h[j]);
            f[2 * j] = p.x;
            f[2 * j + 1] = p.y;
        }
        float amax = 0.f, s = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            amax = fmaxf(amax, fabsf(f[j]));
            s += f[j];
        }
#pragma unroll
        for (int m = 1; m < 4; m <<= 1) {  // 4 neighbouring lanes hold one block of 32 values
            amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, m));
            s += __shfl_xor_sync(0xFFFFFFFFu, s, m);
        }
        const float scale = amax > 0.f ? 127.0f / amax : 0.f;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            lo |= (static_cast<uint32_t>(static_cast<int>(roundf(f[j] * scale))) & 0xFFu) << (8 * j);
            hi |= (static_cast<uint32_t>(static_cast<int>(roundf(f[4 + j] * scale))) & 0xFFu) << (8 * j);
        }
        if (valid) {
            reinterpret_cast<uint2*>(q)[v] = make_uint2(lo, hi);
            if ((v & 3) == 0) {
                d[v >> 2] = amax > 0.f ? amax / 127.0f : 0.f;
                sum[v >> 2] = s;
            }
        }
    }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int launch_check(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return route_fail(TGO_E_CUDA, what);
    return TGO_OK;
}

static int grid_for(long long work_items) {
    long long blocks = (work_items + 255) / 256;
    if (blocks > 148LL * 16) blocks = 148LL * 16;
    if (blocks < 1) blocks = 1;
    return static_cast<int>(blocks);
}

}  // namespace tgo

using namespace tgo;

extern "C" {

int64_t tgo_route_workspace_bytes(int64_t n_pairs, int64_t num_experts) {
    if (n_pairs < 0 || num_experts <= 0) return -1;
    const int64_t blocks = (n_pairs + kRouteBlock - 1) / kRouteBlock;
    return (blocks > 0 ? blocks : 1) * num_experts * 4;
}

int tgo_route_sort(const int32_t* expert_ids, int64_t n_pairs, int64_t num_experts, int32_t* sorted_to_pair,
                   int32_t* pair_to_sorted, int64_t* expert_indices, int32_t* expert_offsets, int32_t* expert_counts,
                   void* workspace, int64_t workspace_bytes, void* stream) {
    if (expert_ids == nullptr || sorted_to_pair == nullptr || pair_to_sorted == nullptr || expert_indices == nullptr ||
        expert_offsets == nullptr || workspace == nullptr)
        return route_fail(TGO_E_ARG, "null pointer");
    if (n_pairs <= 0 || n_pairs > INT32_MAX) return route_fail(TGO_E_ARG, "n_pairs must be in 1..2^31-1");
    if (num_experts <= 0 || num_experts > kRouteMaxExperts)
        return route_fail(TGO_E_ARG, "num_experts must be in 1..4096");
    if (workspace_bytes < tgo_route_workspace_bytes(n_pairs, num_experts))
        return route_fail(TGO_E_WORKSPACE, "routing workspace too small");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int n = static_cast<int>(n_pairs), E = static_cast<int>(num_experts);
    const int blocks = (n + kRouteBlock - 1) / kRouteBlock;
    int32_t* counts = static_cast<int32_t*>(workspace);
    route_count_kernel<<<blocks, kRouteBlock, E * sizeof(int32_t), s>>>(expert_ids, n, E, counts);
    route_scan_kernel<<<1, 1024, 0, s>>>(counts, blocks, E, expert_indices, expert_offsets, expert_counts);
    route_scatter_kernel<<<blocks, kRouteBlock, E * sizeof(int32_t), s>>>(expert_ids, n, E, counts, expert_offsets, sorted_to_pair,
                                                                         pair_to_sorted);
    return launch_check("routing kernel launch failed");
}

int tgo_gather_rows(const void* src, int64_t src_rows, const int32_t* index, int64_t divisor, void* dst, int64_t n_rows,
                    int64_t width, void* stream) {
    if (src == nullptr || index == nullptr || dst == nullptr) return route_fail(TGO_E_ARG, "null pointer");
    if (src_rows <= 0) return route_fail(TGO_E_ARG, "gather needs at least one source row");
    if (n_rows <= 0 || width <= 0 || (width * 2) % 16 != 0 || divisor <= 0 || divisor > INT32_MAX)
        return route_fail(TGO_E_ARG, "gather needs rows > 0, a row length that is a multiple of 8 and divisor > 0");
    if (!aligned16(src) || !aligned16(dst)) return route_fail(TGO_E_ARG, "data pointers must be 16-byte aligned");
    const int vec = static_cast<int>(width / 8);
    gather_rows_kernel<<<grid_for(n_rows * vec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), src_rows, index, static_cast<int>(divisor), static_cast<uint4*>(dst), n_rows, vec);
    return launch_check("gather_rows_kernel launch failed");
}

int tgo_combine_rows(const void* rows, const int32_t* pair_to_sorted, const float* weights, void* out, int64_t tokens,
                     int64_t top_k, int64_t width, void* stream) {
    if (rows == nullptr || pair_to_sorted == nullptr || out == nullptr) return route_fail(TGO_E_ARG, "null pointer");
    if (tokens <= 0 || top_k <= 0 || top_k > 1024 || width <= 0 || (width * 2) % 16 != 0)
        return route_fail(TGO_E_ARG, "combine needs tokens > 0, 1 <= top_k <= 1024 and a row length that is a multiple of 8");
    if (!aligned16(rows) || !aligned16(out)) return route_fail(TGO_E_ARG, "data pointers must be 16-byte aligned");
    const int vec = static_cast<int>(width / 8);
    combine_rows_kernel<<<grid_for(tokens * vec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(rows), pair_to_sorted, weights, static_cast<uint4*>(out), tokens,
        static_cast<int>(top_k), vec);
    return launch_check("combine_rows_kernel launch failed");
}

int tgo_quantize_q8(const void* x, int64_t rows, int64_t width, void* q, float* d, float* sum, void* stream) {
    if (x == nullptr || q == nullptr || d == nullptr || sum == nullptr) return route_fail(TGO_E_ARG, "null pointer");
    if (rows <= 0 || width <= 0 || width % 32 != 0)
        return route_fail(TGO_E_ARG, "quantize needs rows > 0 and a row length that is a multiple of 32");
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 7u) != 0)
        return route_fail(TGO_E_ARG, "x must be 16-byte aligned and q 8-byte aligned");
    const long long n_vec = rows * width / 8;
    int blocks = grid_for(n_vec);
    quantize_q8_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(x), n_vec, static_cast<int8_t*>(q), d, sum);
    return launch_check("quantize_q8_kernel launch failed");
}

}  // extern "C"
