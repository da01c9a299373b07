// C-ABI entry points of libtgo_mmq.so (declared in include/tgo_mmq.h) plus the small kernels
// that are not the GEMM itself: the tile-list builder and the stand-alone dequantiser.
//
// Host responsibilities mirrored from the reference's native layer (csrc/mmq_hip.cu): argument
// validation on host-visible sizes only, launch on the caller's stream, launch-error check; no
// host synchronisation and no device-to-host read on any path except tgo_device_status.
#include "../../include/tgo_mmq.h"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include "mmq_launch.h"

namespace tgo {

// ------------------------------------------------------------------ device globals
__device__ int g_status = 0;

__device__ const uint64_t g_iq2s_grid[1024] = {
#include "iq2s_grid.inc"
};

// ------------------------------------------------------------------ errors
static thread_local std::string t_error;

static int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    t_error = buf;
    return code;
}
static int cuda_fail(cudaError_t e, const char* what) {
    return fail(TGO_E_CUDA, "%s failed: %s", what, cudaGetErrorString(e));
}
static int check_status_if_asked(cudaStream_t stream);

// Error setter for the other translation units of the library.
int route_fail(int code, const char* msg) { return fail(code, "%s", msg); }

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Per-device caches below are relaxed atomics: two host threads that make their first call on a
// device at the same time both compute the same value and store it.
static int num_sms() {
    static std::atomic<int> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev < 64 && cached[dev].load(std::memory_order_relaxed) > 0) return cached[dev].load(std::memory_order_relaxed);
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (dev < 64) cached[dev].store(n, std::memory_order_relaxed);
    return n;
}

static int* status_ptr() {
    int* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_status) != cudaSuccess) return nullptr;
    return p;
}
static const uint64_t* grid_ptr() {
    const uint64_t* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(const_cast<uint64_t**>(&p)), g_iq2s_grid) != cudaSuccess)
        return nullptr;
    return p;
}

}  // namespace tgo
// the status word for the other translation units of the library (null if the lookup fails)
extern "C" int* tgo_status_word(void) { return tgo::status_ptr(); }
namespace tgo {

// ------------------------------------------------------------------ tensor maps
static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    }
    return fn;
}

// bf16 matrix [rows][inner], row-major; boxes of 64 columns x {256,128,64,32,16} rows with the
// 128-byte swizzle.  Out-of-range rows / columns read as zero.
static int encode_act_maps(ActMaps& maps, const void* base, int64_t rows, int64_t inner) {
    // The encoder is a driver entry point and needs a context bound to the calling thread; a
    // thread that has only inherited its device (an autograd worker, say) may not have one yet.
    int dev = 0;
    cudaError_t ce = cudaGetDevice(&dev);
    if (ce == cudaSuccess) ce = cudaSetDevice(dev);
    if (ce != cudaSuccess) return cuda_fail(ce, "cudaSetDevice");
    auto encode = encode_fn();
    if (encode == nullptr) return fail(TGO_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows)};
    const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(inner) * 2};
    const cuuint32_t estride[2] = {1, 1};
    for (int b = 0; b < kNumBoxes; ++b) {
        const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(256 >> b)};
        const CUresult r = encode(&maps.box[b], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim,
                                  gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(TGO_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
    }
    return TGO_OK;
}

// Packed weight tensor [total_rows][row_bytes] as up to 8 byte-typed 2-D maps, one per alignment
// class of its rows (see WgtMaps).  Box = one block window (copy_bytes) x box_rows / P rows.
static int encode_wgt_maps(WgtMaps& maps, const void* base, int64_t total_rows, int64_t row_bytes, int copy_bytes,
                           int box_rows, int& classes, int& classes_log2) {
    auto encode = encode_fn();
    if (encode == nullptr) return fail(TGO_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    int g = 16;
    while (row_bytes % g != 0) g >>= 1;  // gcd(row_bytes, 16); row_bytes is even
    const int P = 16 / g;
    classes = P;
    classes_log2 = P == 1 ? 0 : P == 2 ? 1 : P == 4 ? 2 : 3;
    const cuuint32_t estride[2] = {1, 1};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(copy_bytes), static_cast<cuuint32_t>(box_rows / P)};
    for (int c = 0; c < P; ++c) {
        const uint8_t* b = static_cast<const uint8_t*>(base);
        cuuint64_t gdim[2], gstride[1] = {static_cast<cuuint64_t>(row_bytes) * P};
        if (c < total_rows) {
            const int64_t off = c * row_bytes;
            b += off & ~15LL;
            gdim[0] = static_cast<cuuint64_t>((off & 15) + row_bytes);  // last byte of the row, nothing beyond
            gdim[1] = static_cast<cuuint64_t>((total_rows - c + P - 1) / P);
        } else {  // fewer rows than classes: an in-bounds dummy, its rows are never decoded
            gdim[0] = 16;
            gdim[1] = 1;
        }
        const CUresult r = encode(&maps.cls[c], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(b), gdim, gstride,
                                  box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
            return fail(TGO_E_CUDA, "cuTensorMapEncodeTiled (weights) failed with CUresult %d", static_cast<int>(r));
    }
    return TGO_OK;
}

// A tensor map only encodes (address, shape, box): it can be reused for as long as those are the
// same, whatever the buffer holds.  Encoding takes a few microseconds per map and a call needs up
// to 26 of them, so each thread remembers the last few (weights come back with every call,
// activations whenever the caller's allocator hands out the same block again).
template <typename Maps>
struct MapCache {
    struct Entry {
        const void* base = nullptr;
        int64_t a = 0, b = 0, c = 0;
        int dev = -1, classes = 0, classes_log2 = 0;
        Maps maps;
    };
    static constexpr int kEntries = 8;
    Entry e[kEntries];
    int next = 0;
    Entry* find(const void* base, int64_t a, int64_t b, int64_t c, int dev) {
        for (int i = 0; i < kEntries; ++i)
            if (e[i].base == base && e[i].a == a && e[i].b == b && e[i].c == c && e[i].dev == dev) return &e[i];
        return nullptr;
    }
    Entry* slot() {
        Entry* r = &e[next];
        next = (next + 1) % kEntries;
        return r;
    }
};

static int make_act_maps(ActMaps& maps, const void* base, int64_t rows, int64_t inner) {
    static thread_local MapCache<ActMaps> cache;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = -2;
    if (auto* hit = cache.find(base, rows, inner, 0, dev)) {
        maps = hit->maps;
        return TGO_OK;
    }
    const int rc = encode_act_maps(maps, base, rows, inner);
    if (rc != TGO_OK) return rc;
    auto* s = cache.slot();
    s->base = base; s->a = rows; s->b = inner; s->c = 0; s->dev = dev; s->maps = maps;
    return TGO_OK;
}

static int make_wgt_maps(WgtMaps& maps, const void* base, int64_t total_rows, int64_t row_bytes, int copy_bytes,
                         int box_rows, int& classes, int& classes_log2) {
    static thread_local MapCache<WgtMaps> cache;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = -2;
    const int64_t shape_key = (static_cast<int64_t>(copy_bytes) << 16) | box_rows;
    if (auto* hit = cache.find(base, total_rows, row_bytes, shape_key, dev)) {
        maps = hit->maps;
        classes = hit->classes;
        classes_log2 = hit->classes_log2;
        return TGO_OK;
    }
    const int rc = encode_wgt_maps(maps, base, total_rows, row_bytes, copy_bytes, box_rows, classes, classes_log2);
    if (rc != TGO_OK) return rc;
    auto* s = cache.slot();
    s->base = base; s->a = total_rows; s->b = row_bytes; s->c = shape_key; s->dev = dev;
    s->classes = classes; s->classes_log2 = classes_log2; s->maps = maps;
    return TGO_OK;
}

static int copy_bytes_of(int qt) {
    switch (qt) {
        case QT_Q3_K: return BlockFmt<QT_Q3_K>::kBox;
        case QT_Q4_K: return BlockFmt<QT_Q4_K>::kBox;
        case QT_Q5_K: return BlockFmt<QT_Q5_K>::kBox;
        case QT_Q6_K: return BlockFmt<QT_Q6_K>::kBox;
        default: return BlockFmt<QT_IQ2_S>::kBox;
    }
}

// ------------------------------------------------------------------ tile-list builder
// Workspace layout: int32 count at byte 0, int4 tasks from byte 16.
// One CTA: per group, the number of token tiles ceil(rows / max_tok); exclusive prefix sum; each
// group then writes its tiles, split evenly and rounded up to 16 tokens.  max_tok is 256 (one
// accumulator per tile) or 512 (wide tiles: both accumulators share every decoded weight step).
__global__ void __launch_bounds__(256) build_tiles_kernel(const int64_t* __restrict__ experts,
                                                          const int32_t* __restrict__ offsets, int num_groups,
                                                          int num_experts, int rows, int4* __restrict__ tasks,
                                                          int* __restrict__ count, int capacity, int max_tok) {
    __shared__ int warp_sums[8];
    __shared__ int chunk_total;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int base = 0;
    for (int g0 = 0; g0 < num_groups; g0 += 256) {
        const int g = g0 + tid;
        int nt = 0, beg = 0, end = 0;
        long long e = -1;
        if (g < num_groups) {
            e = experts[g];
            end = offsets[g];
            beg = g > 0 ? offsets[g - 1] : 0;
            const bool valid = e >= 0 && e < num_experts && beg >= 0 && beg < end && end <= rows;
            if (valid) nt = (end - beg + max_tok - 1) / max_tok;
        }
        int incl = nt;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= d) incl += v;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = lane < 8 ? warp_sums[lane] : 0;
#pragma unroll
            for (int d = 1; d < 8; d <<= 1) {
                const int v = __shfl_up_sync(0xFFFFFFFFu, w, d);
                if (lane >= d) w += v;
            }
            if (lane < 8) warp_sums[lane] = w;
            if (lane == 7) chunk_total = w;
        }
        __syncthreads();
        const int pos = base + (warp > 0 ? warp_sums[warp - 1] : 0) + incl - nt;
        if (nt > 0) {
            const int n = end - beg;
            const int per = (((n + nt - 1) / nt) + 15) & ~15;
            for (int j = 0; j < nt; ++j) {
                const int r0 = beg + j * per;
                const int cnt = min(per, end - r0);
                if (pos + j < capacity && cnt > 0) tasks[pos + j] = make_int4(static_cast<int>(e), r0, cnt, g);
                else if (pos + j < capacity) tasks[pos + j] = make_int4(0, 0, 0, g);
            }
        }
        base += chunk_total;
        __syncthreads();
    }
    if (tid == 0) *count = min(base, capacity);
}

static int64_t task_capacity(int64_t rows, int64_t groups) { return rows / kTileTok + groups; }

// ------------------------------------------------------------------ stand-alone dequantiser
// 32 blocks per CTA: their 16-byte-aligned windows are copied into shared memory exactly as the
// GEMM's raw-weight producer stages them, then decoded with the same decode32<>.
template <int QT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ packed, long long n_blocks,
                                                      long long total_bytes, const uint64_t* __restrict__ grid_g,
                                                      __nv_bfloat16* __restrict__ out) {
    using Fmt = BlockFmt<QT>;
    __shared__ __align__(16) uint8_t windows[32 * Fmt::kSlot];
    __shared__ uint64_t grid_s[QT == QT_IQ2_S ? 1024 : 1];
    if (QT == QT_IQ2_S)
        for (int i = threadIdx.x; i < 1024; i += 256) grid_s[i] = grid_g[i];
    const long long b0 = static_cast<long long>(blockIdx.x) * 32;
    constexpr int kChunks = Fmt::kCopy / 16;
    for (int i = threadIdx.x; i < 32 * kChunks; i += 256) {
        const int b = i / kChunks, c = i - b * kChunks;
        const long long blk = b0 + b;
        if (blk >= n_blocks) continue;
        const long long src = ((blk * Fmt::kBytes) & ~15LL) + c * 16;
        uint8_t* dst = windows + b * Fmt::kSlot + c * 16;
        if (src + 16 <= total_bytes) {
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(packed + src);
        } else {
            for (int j = 0; j < 16 && src + j + 2 <= total_bytes; j += 2)
                *reinterpret_cast<uint16_t*>(dst + j) = *reinterpret_cast<const uint16_t*>(packed + src + j);
        }
    }
    __syncthreads();
    const int b = threadIdx.x >> 3, g = threadIdx.x & 7;
    const long long blk = b0 + b;
    if (blk >= n_blocks) return;
    const int mis = static_cast<int>((blk * Fmt::kBytes) & 15);
    uint4 o[4];
    decode32<QT>(smem_u32(windows) + b * Fmt::kSlot + mis, g, smem_u32(grid_s), o);
    uint4* dst = reinterpret_cast<uint4*>(out + blk * 256 + g * 32);
#pragma unroll
    for (int c = 0; c < 4; ++c) dst[c] = o[c];
}

// ------------------------------------------------------------------ wait self-test
// One warp waits on an mbarrier that nobody ever arrives on, with a short limit: the wait gives up,
// sets the abort word, and the kernel records the code in the status word exactly as the GEMM
// kernel's exit path does.  No copy, no UMMA and no TMEM allocation is in flight.
__global__ void __launch_bounds__(64) wait_selftest_kernel(long long limit_cycles, int* status) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_word;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_word = 0;
        mbar_fence_init();
    }
    __syncthreads();
    bool ok = true;
    if ((threadIdx.x & 31) == 0)   // one lane per warp; the second warp leaves through the abort word or its own limit
        ok = mbar_wait(smem_u32(&bar), 0u, &abort_word, kAbortSelfTest, limit_cycles);
    __syncthreads();
    if (threadIdx.x == 0 && (!ok || abort_word != 0) && status != nullptr)
        atomicCAS(status, 0, abort_word | (static_cast<int>(blockIdx.x) << 8));
}

// ------------------------------------------------------------------ split-reduction epilogue
// out[i] = bf16(sum over splits s, in ascending order, of partial[s][i]); four elements per thread.
__global__ void __launch_bounds__(256) split_reduce_kernel(const float4* __restrict__ partial, int nsplit, long long n_vec,
                                                           uint2* __restrict__ out) {
    for (long long v = blockIdx.x * 256LL + threadIdx.x; v < n_vec; v += 256LL * gridDim.x) {
        float4 acc = partial[v];
        for (int s = 1; s < nsplit; ++s) {
            const float4 p = partial[s * n_vec + v];
            acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
        }
        const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        out[v] = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
}

// ------------------------------------------------------------------ GEMM dispatch
static int dispatch_gemm(int qt, int mode, int cta_group, int wide, const GemmArgs& args, int grid, cudaStream_t stream) {
    int e;
    switch (qt) {
        case QT_Q3_K: e = launch_gemm_11(mode, cta_group, wide, args, grid, stream); break;
        case QT_Q4_K: e = launch_gemm_12(mode, cta_group, wide, args, grid, stream); break;
        case QT_Q5_K: e = launch_gemm_13(mode, cta_group, wide, args, grid, stream); break;
        case QT_Q6_K: e = launch_gemm_14(mode, cta_group, wide, args, grid, stream); break;
        case QT_IQ2_S: e = launch_gemm_22(mode, cta_group, wide, args, grid, stream); break;
        default: return fail(TGO_E_ARG, "unsupported quant_type: %d", qt);
    }
    if (e != 0) return cuda_fail(static_cast<cudaError_t>(e), "mmq_gemm_kernel launch");
    return TGO_OK;
}

static int max_pairs(int qt, int mode) {
    switch (qt) {
        case QT_Q3_K: return max_pairs_11(mode);
        case QT_Q4_K: return max_pairs_12(mode);
        case QT_Q5_K: return max_pairs_13(mode);
        case QT_Q6_K: return max_pairs_14(mode);
        case QT_IQ2_S: return max_pairs_22(mode);
        default: return 0;
    }
}

// 2: tiles of 256 weight rows on CTA pairs (the default); 1: tiles of 128 rows on single CTAs
// (environment TGO_CTA_PAIR=0, or a device that cannot co-schedule a pair).
static int wanted_cta_group() {
    static const int v = [] {
        const char* e = getenv("TGO_CTA_PAIR");
        return (e != nullptr && e[0] == '0') ? 1 : 2;
    }();
    return v;
}

// TGO_WIDE_TILES=0 / 1 forces tiles of at most 256 / 512 tokens (read at every call so that a test
// can switch it); unset: chosen per call from the problem size.
static int wide_tiles_env() {
    const char* e = getenv("TGO_WIDE_TILES");
    if (e == nullptr || e[0] == '\0') return -1;
    return e[0] == '0' ? 0 : 1;
}

static int build_tiles(const int64_t* expert_indices, const int32_t* expert_offsets, int64_t num_groups,
                       int64_t num_experts, int64_t rows, void* workspace, int64_t workspace_bytes, int max_tok,
                       cudaStream_t stream);

// Debug aid (environment TGO_CHECK_STATUS=1): wait for the stream after every matmul launch and
// turn a recorded wait time-out into an error of that call.  Off by default: the operators never
// synchronise; a production caller polls tgo_device_status at a point where it synchronises anyway.
static int check_status_if_asked(cudaStream_t stream) {
    const char* e = getenv("TGO_CHECK_STATUS");
    if (e == nullptr || e[0] == '\0' || e[0] == '0') return TGO_OK;
    const cudaError_t ce = cudaStreamSynchronize(stream);
    if (ce != cudaSuccess) return cuda_fail(ce, "cudaStreamSynchronize");
    int v = 0;
    const int rc = tgo_device_status(&v);
    if (rc != TGO_OK) return rc;
    if (v != 0)
        return fail(TGO_E_DEVICE, "a kernel gave up a bounded wait: code %d in block %d (outputs of that launch are incomplete)",
                    v & 0xFF, v >> 8);
    return TGO_OK;
}

// Dense input gradient with few tiles and a long reduction (an LM head: 8 tiles of 3880 steps): the
// out-features are cut into ranges so that every CTA pair gets a tile; each range's fp32 partial
// sums go to a workspace and are added in a fixed order afterwards.  Returns the number of ranges
// (1: no split) and the 64-element steps per range.
static int plan_split(int64_t rows, int64_t N, int64_t K, int64_t tile_m, int64_t limit, int& split_steps) {
    const int64_t tiles = ((rows + kTileTok - 1) / kTileTok) * (K / tile_m);
    const int64_t steps = (N + kStepK - 1) / kStepK;
    split_steps = 0;
    if (tiles * 2 > limit || steps < 128) return 1;
    int64_t s = limit / tiles;
    if (s > steps / 32) s = steps / 32;          // at least 32 steps per range
    if (s < 2) return 1;
    int64_t per = (steps + s - 1) / s;
    per = (per + 1) & ~1LL;                        // whole pipeline stages
    split_steps = static_cast<int>(per);
    return static_cast<int>((steps + per - 1) / per);
}

struct Problem {
    const void* act[2];
    const void* wgt[2];
    void* out[2];
    int nsets;
    int64_t rows, N, K, E;
    int qt, mode;
    const int64_t* experts;   // null: dense
    const int32_t* offsets;
    int64_t groups;
    void* ws;
    int64_t ws_bytes;
    void* const* out_rows;    // forward, one weight set: per-row destinations instead of out[0]
};

static int check_common(const Problem& p) {
    const int64_t bb = tgo_block_bytes(p.qt);
    if (bb < 0) return fail(TGO_E_ARG, "unsupported quant_type: %d", p.qt);
    if (p.rows <= 0) return fail(TGO_E_ARG, "zero-row inputs are not supported");
    if (p.K <= 0 || p.K % 256 != 0) return fail(TGO_E_ARG, "in_features must be a positive multiple of 256; got %lld", (long long)p.K);
    if (p.N <= 0) return fail(TGO_E_ARG, "out_features must be positive; got %lld", (long long)p.N);
    if (p.rows > INT32_MAX || p.N > INT32_MAX || p.K > INT32_MAX || p.E > INT32_MAX || p.groups > INT32_MAX)
        return fail(TGO_E_ARG, "a dimension exceeds the kernel limit of 2^31-1");
    const int nacts = p.mode == kFwd ? 1 : p.nsets;
    for (int s = 0; s < nacts; ++s) {
        if (p.act[s] == nullptr) return fail(TGO_E_ARG, "null tensor pointer");
        if (!aligned16(p.act[s])) return fail(TGO_E_ARG, "activation data pointer must be 16-byte aligned");
    }
    for (int s = 0; s < p.nsets; ++s) {
        if (p.wgt[s] == nullptr) return fail(TGO_E_ARG, "null tensor pointer");
        if (!aligned16(p.wgt[s])) return fail(TGO_E_ARG, "packed_weight data pointer must be 16-byte aligned");
    }
    const int nouts = p.mode == kFwd ? p.nsets : 1;
    for (int s = 0; s < nouts; ++s) {
        if (p.out_rows != nullptr) break;   // the rows go where the table says
        if (p.out[s] == nullptr) return fail(TGO_E_ARG, "null output pointer");
        if (!aligned16(p.out[s])) return fail(TGO_E_ARG, "output data pointer must be 16-byte aligned");
    }
    return TGO_OK;
}

static int run_problem(const Problem& p, cudaStream_t stream) {
    int rc = check_common(p);
    if (rc != TGO_OK) return rc;
    if (p.experts != nullptr) {
        const int64_t need = tgo_grouped_workspace_bytes(p.rows, p.groups);
        if (p.ws == nullptr || p.ws_bytes < need)
            return fail(TGO_E_WORKSPACE, "workspace has %lld bytes, need %lld", (long long)p.ws_bytes, (long long)need);
        if (!aligned16(p.ws)) return fail(TGO_E_ARG, "workspace pointer must be 16-byte aligned");
    }
    GemmArgs a;
    memset(&a, 0, sizeof(a));
    const int64_t red = p.mode == kFwd ? p.K : p.N;  // activation row length
    a.use_tma = (red * 2) % 16 == 0 ? 1 : 0;
    const int nact = p.mode == kFwd ? 1 : p.nsets;
    for (int s = 0; s < 2; ++s) {
        const int src = s < nact ? s : 0;
        a.act[s] = static_cast<const __nv_bfloat16*>(p.act[src]);
        if (a.use_tma) {
            rc = make_act_maps(a.act_maps[s], p.act[src], p.rows, red);
            if (rc != TGO_OK) return rc;
        }
        a.out[s] = static_cast<__nv_bfloat16*>(p.out[(p.mode == kFwd && s < p.nsets) ? s : 0]);
    }
    const int64_t bb = tgo_block_bytes(p.qt);
    if (p.E * p.N > INT32_MAX) return fail(TGO_E_ARG, "experts * out_features exceeds the kernel limit of 2^31-1");
    for (int s = 0; s < p.nsets; ++s) {
        rc = make_wgt_maps(a.wgt_maps[s], p.wgt[s], p.E * p.N, (p.K / 256) * bb, copy_bytes_of(p.qt),
                           p.mode == kFwd ? 128 : 64, a.wgt_classes, a.wgt_classes_log2);
        if (rc != TGO_OK) return rc;
    }
    a.wgt_row_bytes = static_cast<int>((p.K / 256) * bb);
    a.status = status_ptr();
    a.out_rows = reinterpret_cast<__nv_bfloat16* const*>(p.out_rows);
    a.iq2s_grid = grid_ptr();
    if (a.status == nullptr || a.iq2s_grid == nullptr) return fail(TGO_E_CUDA, "cudaGetSymbolAddress failed");
    a.rows = static_cast<int>(p.rows);
    a.out_features = static_cast<int>(p.N);
    a.in_features = static_cast<int>(p.K);
    a.nsets = p.nsets;

    int cg = wanted_cta_group();
    int pairs = 0;
    if (cg == 2) {
        pairs = max_pairs(p.qt, p.mode);
        if (pairs < 1) cg = 1;
    }
    const int64_t tile_m = static_cast<int64_t>(kTileM) * cg;
    const int64_t mtiles = p.mode == kFwd ? ((p.N + tile_m - 1) / tile_m) * p.nsets : p.K / tile_m;
    const int64_t limit = cg == 2 ? pairs : num_sms();
    // Tiles of up to 512 tokens (two accumulators sharing each decoded weight step) halve the
    // decode work per output element and the number of tiles.  Measured on B200 (Q4_K): dense
    // M = 4096 gains 11 % forward and 20 % backward once the 256-token tiles no longer all run at
    // once; grouped inputs lose 3-10 % whatever the mean group size (256, 512 or 2048 rows), because
    // ragged groups leave the wide tiles part empty and the coarser tiles balance worse.  So: dense
    // inputs only.  TGO_WIDE_TILES overrides the choice (tests run every case both ways).
    const int wide_env = wide_tiles_env();
    bool wide = p.experts == nullptr && ((p.rows + kTileTok - 1) / kTileTok) * mtiles > limit;
    if (wide_env >= 0) wide = wide_env != 0;
    int max_tok = wide ? kWideTok : kTileTok;
    // split reduction: dense input gradient of a single weight with a workspace to hold the partial sums
    int nsplit = 1, split_steps = 0;
    if (p.experts == nullptr && p.mode == kBwd && p.nsets == 1 && p.ws != nullptr && wide_env < 0) {
        nsplit = plan_split(p.rows, p.N, p.K, tile_m, limit, split_steps);
        if (nsplit > 1) {
            const int64_t need = static_cast<int64_t>(nsplit) * p.rows * p.K * 4;
            if (p.ws_bytes < need) return fail(TGO_E_WORKSPACE, "workspace has %lld bytes, need %lld", (long long)p.ws_bytes, (long long)need);
            if (!aligned16(p.ws)) return fail(TGO_E_ARG, "workspace pointer must be 16-byte aligned");
            wide = false;
            max_tok = kTileTok;
        }
    }
    a.nsplit = nsplit;
    a.split_steps = split_steps;
    a.partial = nsplit > 1 ? static_cast<float*>(p.ws) : nullptr;
    int64_t max_tasks;
    if (p.experts == nullptr) {
        a.dense_tasks = static_cast<int>((p.rows + max_tok - 1) / max_tok);
        a.dense_tok = static_cast<int>((((p.rows + a.dense_tasks - 1) / a.dense_tasks) + 15) & ~15LL);
        max_tasks = a.dense_tasks;
    } else {
        const int64_t cap = task_capacity(p.rows, p.groups);
        rc = build_tiles(p.experts, p.offsets, p.groups, p.E, p.rows, p.ws, p.ws_bytes, max_tok, stream);
        if (rc != TGO_OK) return rc;
        a.task_count = static_cast<const int*>(p.ws);
        a.tasks = reinterpret_cast<const int4*>(static_cast<const uint8_t*>(p.ws) + 16);
        max_tasks = cap;
    }
    if (max_tasks * mtiles * nsplit > INT32_MAX) return fail(TGO_E_ARG, "the problem has more than 2^31-1 tiles");
    int64_t grid = max_tasks * mtiles * nsplit;  // persistent CTAs (pairs) never outnumber the tiles
    if (grid > limit) grid = limit;
    if (grid < 1) grid = 1;
    if (getenv("TGO_DEBUG_LAUNCH") != nullptr)
        fprintf(stderr, "tgo launch: mode %d cta_group %d pairs %d grid %lld tiles<=%lld\n", p.mode, cg, pairs,
                (long long)(grid * cg), (long long)(max_tasks * mtiles));
    rc = dispatch_gemm(p.qt, p.mode, cg, wide ? 1 : 0, a, static_cast<int>(grid * cg), stream);
    if (rc != TGO_OK) return rc;
    if (nsplit > 1) {
        const long long n_vec = p.rows * p.K / 4;   // K is a multiple of 256
        long long blocks = (n_vec + 255) / 256;
        if (blocks > num_sms() * 8LL) blocks = num_sms() * 8LL;
        split_reduce_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(static_cast<const float4*>(p.ws), nsplit, n_vec,
                                                                          static_cast<uint2*>(p.out[0]));
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "split_reduce_kernel launch");
    }
    return check_status_if_asked(stream);
}

static int build_tiles(const int64_t* expert_indices, const int32_t* expert_offsets, int64_t num_groups,
                       int64_t num_experts, int64_t rows, void* workspace, int64_t workspace_bytes, int max_tok,
                       cudaStream_t stream) {
    if (expert_indices == nullptr || expert_offsets == nullptr || workspace == nullptr)
        return fail(TGO_E_ARG, "null pointer");
    if (num_groups <= 0) return fail(TGO_E_ARG, "grouped MMQ requires at least one active expert");
    if (num_experts <= 0) return fail(TGO_E_ARG, "packed_weight must contain at least one expert");
    if (rows <= 0) return fail(TGO_E_ARG, "zero-row inputs are not supported");
    if (rows > INT32_MAX || num_groups > INT32_MAX || num_experts > INT32_MAX)
        return fail(TGO_E_ARG, "a dimension exceeds the kernel limit of 2^31-1");
    const int64_t need = tgo_grouped_workspace_bytes(rows, num_groups);
    if (workspace_bytes < need)
        return fail(TGO_E_WORKSPACE, "workspace has %lld bytes, need %lld", (long long)workspace_bytes, (long long)need);
    if (!aligned16(workspace)) return fail(TGO_E_ARG, "workspace pointer must be 16-byte aligned");
    int* count = static_cast<int*>(workspace);
    int4* tasks = reinterpret_cast<int4*>(static_cast<uint8_t*>(workspace) + 16);
    build_tiles_kernel<<<1, 256, 0, stream>>>(expert_indices, expert_offsets, static_cast<int>(num_groups),
                                              static_cast<int>(num_experts), static_cast<int>(rows), tasks, count,
                                              static_cast<int>(task_capacity(rows, num_groups)), max_tok);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "build_tiles_kernel launch");
    return TGO_OK;
}

// ------------------------------------------------------------------ built-in tile-list scratch
// Scratch for tgo_grouped_fwd_noalloc: the tile list lives in this fixed array instead of a
// caller-provided workspace.  Every GPU that loads the library holds these bytes until exit.
constexpr int64_t kStaticMaxTiles = TGO_NOALLOC_MAX_TILES;  // most (rows / 256 + groups) it can describe
constexpr int64_t kStaticScratchBytes = 16 + 16 * kStaticMaxTiles;
static __device__ __align__(256) unsigned char g_static_tile_scratch[kStaticScratchBytes];

// Device address of the array on the current device.  In host code the array's name is only a
// handle for the runtime, never an address a kernel may be given, so the address is looked up
// once per device (with that device current) and remembered.
static int static_scratch_ptr(void** out) {
    static std::atomic<void*> cached[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    if (dev < 0 || dev >= 64) return fail(TGO_E_ARG, "device index %d is outside the supported range 0..63", dev);
    void* p = cached[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        // two threads racing here both get the same address from the runtime and store it
        e = cudaGetSymbolAddress(&p, g_static_tile_scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(built-in tile scratch)");
        if (p == nullptr) return fail(TGO_E_CUDA, "cudaGetSymbolAddress returned a null address for the built-in tile scratch");
        cached[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return TGO_OK;
}

}  // namespace tgo

// ====================================================================== C ABI
using namespace tgo;

extern "C" {

int tgo_version(void) { return 100; }

const char* tgo_last_error(void) { return t_error.c_str(); }

int64_t tgo_block_bytes(int quant_type) { return block_bytes_of(quant_type); }

int tgo_device_status(int* status) {
    if (status == nullptr) return fail(TGO_E_ARG, "null status pointer");
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_status, sizeof(int));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyFromSymbol");
    if (v != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
        if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyToSymbol");
    }
    *status = v;
    return TGO_OK;
}

int tgo_selftest_wait_timeout(int64_t limit_cycles, void* stream) {
    if (limit_cycles < 1000 || limit_cycles > 200000000LL)
        return fail(TGO_E_ARG, "limit_cycles must be in 1000..200000000 (at most about a tenth of a second)");
    int* status = status_ptr();
    if (status == nullptr) return fail(TGO_E_CUDA, "cudaGetSymbolAddress failed");
    wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(limit_cycles, status);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "wait_selftest_kernel launch");
    return TGO_OK;
}

int tgo_dequantize_bf16(const void* packed, int64_t n_blocks, int quant_type, void* out_bf16, void* stream) {
    const int64_t bb = tgo_block_bytes(quant_type);
    if (bb < 0) return fail(TGO_E_ARG, "unsupported quant_type: %d", quant_type);
    if (n_blocks <= 0) return fail(TGO_E_ARG, "n_blocks must be positive");
    if (packed == nullptr || out_bf16 == nullptr) return fail(TGO_E_ARG, "null tensor pointer");
    if (!aligned16(packed) || !aligned16(out_bf16)) return fail(TGO_E_ARG, "data pointers must be 16-byte aligned");
    const uint64_t* grid = grid_ptr();
    if (grid == nullptr) return fail(TGO_E_CUDA, "cudaGetSymbolAddress failed");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned nb = static_cast<unsigned>((n_blocks + 31) / 32);
    const uint8_t* p = static_cast<const uint8_t*>(packed);
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out_bf16);
    const long long total = n_blocks * bb;
    switch (quant_type) {
        case QT_Q3_K: dequant_kernel<QT_Q3_K><<<nb, 256, 0, s>>>(p, n_blocks, total, grid, o); break;
        case QT_Q4_K: dequant_kernel<QT_Q4_K><<<nb, 256, 0, s>>>(p, n_blocks, total, grid, o); break;
        case QT_Q5_K: dequant_kernel<QT_Q5_K><<<nb, 256, 0, s>>>(p, n_blocks, total, grid, o); break;
        case QT_Q6_K: dequant_kernel<QT_Q6_K><<<nb, 256, 0, s>>>(p, n_blocks, total, grid, o); break;
        default: dequant_kernel<QT_IQ2_S><<<nb, 256, 0, s>>>(p, n_blocks, total, grid, o); break;
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "dequant_kernel launch");
    return TGO_OK;
}

int tgo_mmq_fwd(const void* x, const void* packed_weight, void* y, int64_t rows, int64_t out_features,
                int64_t in_features, int quant_type, void* stream) {
    Problem p = {};
    p.act[0] = x; p.wgt[0] = packed_weight; p.out[0] = y; p.nsets = 1;
    p.rows = rows; p.N = out_features; p.K = in_features; p.E = 1; p.qt = quant_type; p.mode = kFwd;
    return run_problem(p, static_cast<cudaStream_t>(stream));
}

int tgo_mmq_dx(const void* dy, const void* packed_weight, void* dx, int64_t rows, int64_t out_features,
               int64_t in_features, int quant_type, void* stream) {
    Problem p = {};
    p.act[0] = dy; p.wgt[0] = packed_weight; p.out[0] = dx; p.nsets = 1;
    p.rows = rows; p.N = out_features; p.K = in_features; p.E = 1; p.qt = quant_type; p.mode = kBwd;
    return run_problem(p, static_cast<cudaStream_t>(stream));
}

int64_t tgo_mmq_dx_workspace_bytes(int64_t rows, int64_t out_features, int64_t in_features, int quant_type) {
    if (rows <= 0 || out_features <= 0 || in_features <= 0 || in_features % 256 != 0 || tgo_block_bytes(quant_type) < 0) return 0;
    int cg = wanted_cta_group();
    int pairs = 0;
    if (cg == 2) {
        pairs = max_pairs(quant_type, kBwd);
        if (pairs < 1) cg = 1;
    }
    int split_steps = 0;
    const int n = plan_split(rows, out_features, in_features, static_cast<int64_t>(kTileM) * cg, cg == 2 ? pairs : num_sms(), split_steps);
    return n > 1 ? static_cast<int64_t>(n) * rows * in_features * 4 : 0;
}

int tgo_mmq_dx_ws(const void* dy, const void* packed_weight, void* dx, int64_t rows, int64_t out_features,
                  int64_t in_features, int quant_type, void* workspace, int64_t workspace_bytes, void* stream) {
    Problem p = {};
    p.act[0] = dy; p.wgt[0] = packed_weight; p.out[0] = dx; p.nsets = 1;
    p.rows = rows; p.N = out_features; p.K = in_features; p.E = 1; p.qt = quant_type; p.mode = kBwd;
    p.ws = workspace; p.ws_bytes = workspace_bytes;
    return run_problem(p, static_cast<cudaStream_t>(stream));
}

int tgo_mmq_fwd_multi(const void* x, const void* const* packed_weights, void* const* ys, int64_t num_weights, int64_t rows,
                      int64_t out_features, int64_t in_features, int quant_type, void* stream) {
    if (packed_weights == nullptr || ys == nullptr) return fail(TGO_E_ARG, "null pointer array");
    if (num_weights < 1 || num_weights > 4) return fail(TGO_E_ARG, "num_weights must be in 1..4; got %lld", (long long)num_weights);
    // one launch covers two weight sets (their tiles share the launch and the activation rows' L2 residency)
    for (int64_t s = 0; s < num_weights; s += 2) {
        Problem p = {};
        p.nsets = num_weights - s >= 2 ? 2 : 1;
        p.act[0] = x;
        for (int i = 0; i < p.nsets; ++i) { p.wgt[i] = packed_weights[s + i]; p.out[i] = ys[s + i]; }
        p.rows = rows; p.N = out_features; p.K = in_features; p.E = 1; p.qt = quant_type; p.mode = kFwd;
        const int rc = run_problem(p, static_cast<cudaStream_t>(stream));
        if (rc != TGO_OK) return rc;
    }
    return TGO_OK;
}

int64_t tgo_grouped_workspace_bytes(int64_t rows, int64_t num_groups) {
    if (rows < 0 || num_groups < 0) return -1;
    return 16 + 16 * task_capacity(rows, num_groups);
}

int tgo_build_tiles(const int64_t* expert_indices, const int32_t* expert_offsets, int64_t num_groups,
                    int64_t num_experts, int64_t rows, int64_t max_tile_tokens, void* workspace,
                    int64_t workspace_bytes, void* stream) {
    if (max_tile_tokens != kTileTok && max_tile_tokens != kWideTok)
        return fail(TGO_E_ARG, "max_tile_tokens must be %d or %d; got %lld", kTileTok, kWideTok, (long long)max_tile_tokens);
    return build_tiles(expert_indices, expert_offsets, num_groups, num_experts, rows, workspace, workspace_bytes,
                       static_cast<int>(max_tile_tokens), static_cast<cudaStream_t>(stream));
}

int tgo_grouped_fwd(const void* x, const void* w0, const void* w1, void* y0, void* y1,
                    const int64_t* expert_indices, const int32_t* expert_offsets, int64_t num_groups,
                    int64_t num_experts, int64_t rows, int64_t out_features, int64_t in_features, int quant_type,
                    void* workspace, int64_t workspace_bytes, void* stream) {
    if ((w1 == nullptr) != (y1 == nullptr)) return fail(TGO_E_ARG, "w1 and y1 must both be given or both be null");
    if (expert_indices == nullptr || expert_offsets == nullptr) return fail(TGO_E_ARG, "null routing pointer");
    if (num_groups > num_experts) return fail(TGO_E_ARG, "active expert count exceeds packed expert count");
    Problem p = {};
    p.act[0] = x; p.wgt[0] = w0; p.wgt[1] = w1; p.out[0] = y0; p.out[1] = y1; p.nsets = w1 ? 2 : 1;
    p.rows = rows; p.N = out_features; p.K = in_features; p.E = num_experts; p.qt = quant_type; p.mode = kFwd;
    p.experts = expert_indices; p.offsets = expert_offsets; p.groups = num_groups;
    p.ws = workspace; p.ws_bytes = workspace_bytes;
    return run_problem(p, static_cast<cudaStream_t>(stream));
}

int tgo_grouped_fwd_rows(const void* x, const void* w, void* const* y_rows, const int64_t* expert_indices,
                         const int32_t* expert_offsets, int64_t num_groups, int64_t num_experts, int64_t rows,
                         int64_t out_features, int64_t in_features, int quant_type, void* workspace,
                         int64_t workspace_bytes, void* stream) {
    if (y_rows == nullptr) return fail(TGO_E_ARG, "null row-pointer table");
    if (expert_indices == nullptr || expert_offsets == nullptr) return fail(TGO_E_ARG, "null routing pointer");
    if (num_groups > num_experts) return fail(TGO_E_ARG, "active expert count exceeds packed expert count");
    if ((out_features * 2) % 16 != 0) return fail(TGO_E_ARG, "scattered output rows need out_features to be a multiple of 8");
    Problem p = {};
    p.act[0] = x; p.wgt[0] = w; p.nsets = 1; p.out_rows = y_rows;
    p.rows = rows; p.N = out_features; p.K = in_features; p.E = num_experts; p.qt = quant_type; p.mode = kFwd;
    p.experts = expert_indices; p.offsets = expert_offsets; p.groups = num_groups;
    p.ws = workspace; p.ws_bytes = workspace_bytes;
    return run_problem(p, static_cast<cudaStream_t>(stream));
}

int tgo_grouped_dx(const void* dy0, const void* dy1, const void* w0, const void* w1, void* dx,
                   const int64_t* expert_indices, const int32_t* expert_offsets, int64_t num_groups,
                   int64_t num_experts, int64_t rows, int64_t out_features, int64_t in_features, int quant_type,
                   void* workspace, int64_t workspace_bytes, void* stream) {
    if ((w1 == nullptr) != (dy1 == nullptr)) return fail(TGO_E_ARG, "w1 and dy1 must both be given or both be null");
    if (expert_indices == nullptr || expert_offsets == nullptr) return fail(TGO_E_ARG, "null routing pointer");
    if (num_groups > num_experts) return fail(TGO_E_ARG, "active expert count exceeds packed expert count");
    Problem p = {};
    p.act[0] = dy0; p.act[1] = dy1; p.wgt[0] = w0; p.wgt[1] = w1; p.out[0] = dx; p.nsets = w1 ? 2 : 1;
    p.rows = rows; p.N = out_features; p.K = in_features; p.E = num_experts; p.qt = quant_type; p.mode = kBwd;
    p.experts = expert_indices; p.offsets = expert_offsets; p.groups = num_groups;
    p.ws = workspace; p.ws_bytes = workspace_bytes;
    return run_problem(p, static_cast<cudaStream_t>(stream));
}

int tgo_grouped_fwd_noalloc(const void* x, const void* w0, const void* w1, void* y0, void* y1,
                            const int64_t* expert_indices, const int32_t* expert_offsets, int64_t num_groups,
                            int64_t num_experts, int64_t rows, int64_t out_features, int64_t in_features,
                            int quant_type, void* stream) {
    if (rows > 0 && num_groups > 0 && task_capacity(rows, num_groups) > kStaticMaxTiles)
        return fail(TGO_E_WORKSPACE,
                    "tgo_grouped_fwd_noalloc: rows/256 + groups = %lld exceeds the built-in limit of %lld tiles; "
                    "use tgo_grouped_fwd with a caller-provided workspace",
                    (long long)task_capacity(rows, num_groups), (long long)kStaticMaxTiles);
    void* scratch = nullptr;
    const int rc = static_scratch_ptr(&scratch);
    if (rc != TGO_OK) return rc;
    return tgo_grouped_fwd(x, w0, w1, y0, y1, expert_indices, expert_offsets, num_groups, num_experts, rows,
                           out_features, in_features, quant_type, scratch, kStaticScratchBytes, stream);
}

}  // extern "C"
