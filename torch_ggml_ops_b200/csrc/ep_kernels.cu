// Expert-parallel row exchange over peer memory (NVLink / NVSwitch): routed rows are written
// straight into the expert-major receive buffer of the GPU that owns their expert, and results are
// read back from the owner's buffer, each in ONE pass of plain 16-byte peer stores / loads.  No
// multicast, no waits inside these kernels: ranks are ordered by stream-ordered collectives issued
// by the host layer between the phases.
//
// The reference is single-GPU; its contract "rows sorted by expert + cumulative end offsets"
// (csrc/mmq_hip.cu:325-406) is what tgo_ep_plan produces for the local experts of every rank.
#include "../../include/tgo_mmq.h"

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace tgo {

int route_fail(int code, const char* msg);  // tgo_api.cu

constexpr int kEpMaxRanks = 64;

// counts[s][e]: routed pairs of rank s for (global) expert e.  Expert e lives on rank e / EL, in
// whose buffer rows are ordered by (local expert, source rank, position in the source's sorted
// order).  One block.
__global__ void __launch_bounds__(1024) ep_offsets_kernel(const int32_t* __restrict__ counts, int W, int E, int EL, int me,
                                                          int capacity, int32_t* __restrict__ dst_base,
                                                          int32_t* __restrict__ seg_start,
                                                          int64_t* __restrict__ local_indices,
                                                          int32_t* __restrict__ local_offsets) {
    // per expert: rows from all sources, rows from the sources before this rank, this rank's rows
    __shared__ int32_t total[4096], earlier[4096], mine[4096];
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int t = 0, b = 0;
        for (int s = 0; s < W; ++s) {
            const int c = counts[s * E + e];
            if (s < me) b += c;
            t += c;
        }
        total[e] = t;
        earlier[e] = b;
        mine[e] = counts[me * E + e];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int first = (e / EL) * EL;
        int before_experts = 0;   // rows of earlier experts of the same owner, all sources
        for (int f = first; f < e; ++f) before_experts += total[f];
        int mine_before = 0;
        for (int f = 0; f < e; ++f) mine_before += mine[f];
        dst_base[e] = before_experts + earlier[e];
        seg_start[e] = mine_before;
        if (e / EL == me) {
            local_indices[e - first] = e - first;
            // rows at or beyond the capacity are dropped by ep_map_kernel (and flagged): the group
            // that straddles the capacity keeps the rows that fit, later groups become empty
            local_offsets[e - first] = min(before_experts + total[e], capacity);
        }
    }
}

// Destination (rank, row) of every routed pair of this rank.
__global__ void __launch_bounds__(256) ep_map_kernel(const int32_t* __restrict__ expert_ids, const int32_t* __restrict__ pair_to_sorted,
                                                     const int32_t* __restrict__ dst_base, const int32_t* __restrict__ seg_start,
                                                     int n_pairs, int E, int EL, int capacity, int32_t* __restrict__ dst_rank,
                                                     int32_t* __restrict__ dst_row, int* __restrict__ overflow) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= n_pairs) return;
    const int e = expert_ids[i];
    const int j = pair_to_sorted[i];
    if (e < 0 || e >= E || j < 0) {
        dst_rank[i] = -1;
        dst_row[i] = -1;
        return;
    }
    const int row = dst_base[e] + (j - seg_start[e]);
    if (row >= capacity) {  // receive buffer too small: drop the pair and say so
        dst_rank[i] = -1;
        dst_row[i] = -1;
        atomicExch(overflow, 1);
        return;
    }
    dst_rank[i] = e / EL;
    dst_row[i] = row;
}

struct PeerPtrs {
    void* p[kEpMaxRanks];
};

// Independent 16-byte peer loads per thread and loop iteration in ep_pull_kernel.  Measured at two
// GPUs: the per-pair pull 0.074 -> 0.064 ms; the same unrolling made the local expand / reduce
// kernels and the token-level pull slower (registers, occupancy), so they keep one access per thread.
constexpr int kEpUnroll = 4;

// peer[dst_rank[i]][dst_row[i]][:] = src[i / divisor][:]   (rows of vec_per_row 16-byte vectors)
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const uint4* __restrict__ src, int divisor, const int32_t* __restrict__ dst_rank,
                                                          const int32_t* __restrict__ dst_row, long long n_pairs, int vec_per_row,
                                                          const __grid_constant__ PeerPtrs peers) {
    const long long total = n_pairs * vec_per_row;
    for (long long v = blockIdx.x * 256LL + threadIdx.x; v < total; v += 256LL * gridDim.x) {
        const long long i = v / vec_per_row;
        const int c = static_cast<int>(v - i * vec_per_row);
        const int r = dst_rank[i];
        if (r < 0) continue;
        const uint4 val = src[(i / divisor) * vec_per_row + c];
        static_cast<uint4*>(peers.p[r])[static_cast<long long>(dst_row[i]) * vec_per_row + c] = val;
    }
}

// out[t][:] = sum over the `group` consecutive pairs of t of weight * peer[dst_rank][dst_row][:]
// (group = 1: one output row per pair; group = top_k: the per-token combine), fp32 accumulation.
__global__ void __launch_bounds__(256) ep_pull_kernel(const __grid_constant__ PeerPtrs peers, const int32_t* __restrict__ dst_rank,
                                                      const int32_t* __restrict__ dst_row, const float* __restrict__ weights,
                                                      uint4* __restrict__ out, long long n_out, int group, int vec_per_row) {
    const long long total = n_out * vec_per_row;
    if (group == 1) {
        // one row per pair: kEpUnroll independent peer loads in flight per thread
        const long long stride = 256LL * gridDim.x;
        for (long long v0 = blockIdx.x * 256LL + threadIdx.x; v0 < total; v0 += kEpUnroll * stride) {
            int r[kEpUnroll], row[kEpUnroll], c[kEpUnroll];
#pragma unroll
            for (int u = 0; u < kEpUnroll; ++u) {
                const long long v = v0 + u * stride;
                r[u] = -1;
                if (v < total) {
                    const long long t = v / vec_per_row;
                    c[u] = static_cast<int>(v - t * vec_per_row);
                    r[u] = dst_rank[t];
                    row[u] = dst_row[t];
                }
            }
            uint4 val[kEpUnroll];
#pragma unroll
            for (int u = 0; u < kEpUnroll; ++u) {
                val[u] = make_uint4(0u, 0u, 0u, 0u);
                if (r[u] >= 0) val[u] = static_cast<const uint4*>(peers.p[r[u]])[static_cast<long long>(row[u]) * vec_per_row + c[u]];
            }
#pragma unroll
            for (int u = 0; u < kEpUnroll; ++u)
                if (v0 + u * stride < total) out[v0 + u * stride] = val[u];
        }
        return;
    }
    for (long long v = blockIdx.x * 256LL + threadIdx.x; v < total; v += 256LL * gridDim.x) {
        const long long t = v / vec_per_row;
        const int c = static_cast<int>(v - t * vec_per_row);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < group; ++s) {
            const long long i = t * group + s;
            const int r = dst_rank[i];
            if (r < 0) continue;
            const float w = weights != nullptr ? weights[i] : 1.0f;
            const uint4 val = static_cast<const uint4*>(peers.p[r])[static_cast<long long>(dst_row[i]) * vec_per_row + c];
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

// ---------------------------------------------------------------- token-level exchange
// With top-k routing a token usually has several experts on the same GPU.  The kernels below move
// a token's row once per destination GPU instead of once per routed pair, and bring back one
// partial sum per GPU instead of one gradient row per pair: the owner replicates / reduces locally
// at HBM speed.  Token t of rank r has the fixed slot r * tokens_per_rank + t in every owner's
// token buffers, so no counting or extra collective is needed.

// Plan time, one thread per routed pair i = t * top_k + s of this rank: tell every owner g which
// of its rows belong to the token's slot (slot_rows[g][slot][s] = row or -1) and tell the pair's
// owner which slot feeds that row (row_slot[owner][row] = slot).
__global__ void __launch_bounds__(256) ep_token_maps_kernel(const int32_t* __restrict__ dst_rank, const int32_t* __restrict__ dst_row,
                                                            long long n_pairs, int top_k, int world, long long slot0,
                                                            const __grid_constant__ PeerPtrs row_slot,
                                                            const __grid_constant__ PeerPtrs slot_rows,
                                                            const float* __restrict__ pair_weights,
                                                            const __grid_constant__ PeerPtrs row_weight,
                                                            uint4* __restrict__ result, int result_vec) {
    const long long i = blockIdx.x * 256LL + threadIdx.x;
    if (i >= n_pairs) return;
    const long long t = i / top_k;
    const int s = static_cast<int>(i - t * top_k);
    const int r = dst_rank[i], row = dst_row[i];
    const long long slot = slot0 + t;
    for (int g = 0; g < world; ++g) static_cast<int32_t*>(slot_rows.p[g])[slot * top_k + s] = (r == g) ? row : -1;
    if (r >= 0) {
        static_cast<int32_t*>(row_slot.p[r])[row] = static_cast<int32_t>(slot);
        // the pair's routing weight travels with the map, so the owner can scale the row it computes
        if (pair_weights != nullptr) static_cast<float*>(row_weight.p[r])[row] = pair_weights[i];
    } else if (result != nullptr) {
        // a dropped pair (no room on its expert's GPU): nobody writes its result row, it reads as zeros
        for (int c = 0; c < result_vec; ++c) result[i * result_vec + c] = make_uint4(0u, 0u, 0u, 0u);
    }
}

// tok[g][slot][:] = src[t][:] for every GPU g that owns at least one of token t's experts.
__global__ void __launch_bounds__(256) ep_dispatch_tokens_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ dst_rank,
                                                                 long long tokens, int top_k, int vec_per_row, long long slot0,
                                                                 const __grid_constant__ PeerPtrs tok) {
    const long long total = tokens * vec_per_row;
    for (long long v = blockIdx.x * 256LL + threadIdx.x; v < total; v += 256LL * gridDim.x) {
        const long long t = v / vec_per_row;
        const int c = static_cast<int>(v - t * vec_per_row);
        const uint4 val = src[v];
        unsigned long long seen = 0ull;
        for (int s = 0; s < top_k; ++s) {
            const int r = dst_rank[t * top_k + s];
            if (r < 0 || ((seen >> r) & 1ull)) continue;
            seen |= 1ull << r;
            static_cast<uint4*>(tok.p[r])[(slot0 + t) * vec_per_row + c] = val;
        }
    }
}

// Owner side: rows[row][:] = tok[row_slot[row]][:] for the rows that exist (*n_rows, a device value).
// A row whose slot entry is not a slot of the token buffer (nobody announced that row through
// tgo_ep_token_maps) is left as it is.
__global__ void __launch_bounds__(256) ep_expand_kernel(const uint4* __restrict__ tok, const int32_t* __restrict__ row_slot,
                                                        const int32_t* __restrict__ n_rows, uint4* __restrict__ rows,
                                                        long long capacity, long long n_slots, int vec_per_row) {
    long long n = *n_rows;
    if (n > capacity) n = capacity;
    const long long total = n * vec_per_row;
    for (long long v = blockIdx.x * 256LL + threadIdx.x; v < total; v += 256LL * gridDim.x) {
        const long long row = v / vec_per_row;
        const int c = static_cast<int>(v - row * vec_per_row);
        const long long slot = row_slot[row];
        if (slot < 0 || slot >= n_slots) continue;
        rows[v] = tok[slot * vec_per_row + c];
    }
}

// Token owner's side of the same scheme: result rows of routed pairs that were dropped (no room
// in the expert's GPU) are never written by anybody; they are zeroed here, one warp per row.
__global__ void __launch_bounds__(256) ep_zero_dropped_kernel(const int32_t* __restrict__ dst_rank, long long n_pairs,
                                                              uint4* __restrict__ result, int vec_per_row) {
    const long long warp = (blockIdx.x * 256LL + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= n_pairs || dst_rank[warp] >= 0) return;
    for (int c = lane; c < vec_per_row; c += 32) result[warp * vec_per_row + c] = make_uint4(0u, 0u, 0u, 0u);
}

// Owner side, for a forward whose epilogue returns every row to the token's owner
// (tgo_grouped_fwd_rows): row_ptrs[row] = address, in this GPU's view of the owner's result buffer,
// of the routed pair the row belongs to.  Row -> slot comes from row_slot, the pair's position s in
// the token's top-k from slot_rows[slot][s] == row; slot = owner * tokens_per_rank + token, and the
// pair's result row at the owner is token * top_k + s.  A row nobody announced gets a null pointer.
__global__ void __launch_bounds__(256) ep_row_pointers_kernel(const int32_t* __restrict__ row_slot,
                                                              const int32_t* __restrict__ slot_rows,
                                                              const int32_t* __restrict__ n_rows, long long capacity,
                                                              long long n_slots, int top_k, long long tokens_per_rank,
                                                              const __grid_constant__ PeerPtrs result, long long row_bytes,
                                                              unsigned long long* __restrict__ row_ptrs) {
    long long n = *n_rows;
    if (n > capacity) n = capacity;
    for (long long row = blockIdx.x * 256LL + threadIdx.x; row < n; row += 256LL * gridDim.x) {
        const long long slot = row_slot[row];
        unsigned long long ptr = 0ull;
        if (slot >= 0 && slot < n_slots) {
            const long long owner = slot / tokens_per_rank, token = slot - owner * tokens_per_rank;
            for (int s = 0; s < top_k; ++s) {
                if (slot_rows[slot * top_k + s] == row) {
                    ptr = reinterpret_cast<unsigned long long>(result.p[owner]) +
                          static_cast<unsigned long long>((token * top_k + s) * row_bytes);
                    break;
                }
            }
        }
        row_ptrs[row] = ptr;
    }
}

// Owner side: part[slot][:] = sum over the slot's rows of rows[row][:] (fp32, rounded once); slots
// without a row on this GPU are left alone (nobody reads them).
__global__ void __launch_bounds__(256) ep_reduce_kernel(const uint4* __restrict__ rows, const int32_t* __restrict__ slot_rows,
                                                        long long n_slots, int top_k, uint4* __restrict__ part, int vec_per_row) {
    const long long total = n_slots * vec_per_row;
    for (long long v = blockIdx.x * 256LL + threadIdx.x; v < total; v += 256LL * gridDim.x) {
        const long long slot = v / vec_per_row;
        const int c = static_cast<int>(v - slot * vec_per_row);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        bool any = false;
        for (int s = 0; s < top_k; ++s) {
            const int row = slot_rows[slot * top_k + s];
            if (row < 0) continue;
            any = true;
            const uint4 val = rows[static_cast<long long>(row) * vec_per_row + c];
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&val);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h[j]);
                acc[2 * j] += f.x;
                acc[2 * j + 1] += f.y;
            }
        }
        if (!any) continue;
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        part[v] = o;
    }
}

// out[t][:] = sum over the GPUs g that own one of token t's experts of part[g][slot][:] (fp32).
__global__ void __launch_bounds__(256) ep_pull_tokens_kernel(const __grid_constant__ PeerPtrs part, const int32_t* __restrict__ dst_rank,
                                                             long long tokens, int top_k, int vec_per_row, long long slot0,
                                                             uint4* __restrict__ out) {
    const long long total = tokens * vec_per_row;
    for (long long v = blockIdx.x * 256LL + threadIdx.x; v < total; v += 256LL * gridDim.x) {
        const long long t = v / vec_per_row;
        const int c = static_cast<int>(v - t * vec_per_row);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        unsigned long long seen = 0ull;
        // eight pairs at a time: first which GPUs (each once, in the pairs' order), then all the peer
        // loads (independent, so up to eight are in flight per thread), then the sums in that order
        for (int s0 = 0; s0 < top_k; s0 += 8) {
            const uint4* src[8];
            uint4 val[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = s0 + i < top_k ? dst_rank[t * top_k + s0 + i] : -1;
                src[i] = nullptr;
                if (r >= 0 && !((seen >> r) & 1ull)) {
                    seen |= 1ull << r;
                    src[i] = static_cast<const uint4*>(part.p[r]) + (slot0 + t) * vec_per_row + c;
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) val[i] = src[i] != nullptr ? *src[i] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (src[i] == nullptr) continue;
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&val[i]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(h[j]);
                    acc[2 * j] += f.x;
                    acc[2 * j + 1] += f.y;
                }
            }
        }
        uint4 o;
        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        out[v] = o;
    }
}

// ---------------------------------------------------------------- rank barrier and count exchange
// Stream-ordered barrier between the ranks without a collective library: rank r stores `epoch`
// into slot r of every rank's flag array (system-scope release, after a system fence that makes
// this GPU's earlier peer stores visible), then waits until every slot of its own array has reached
// `epoch`.  The wait is bounded: after `limit_cycles` it records kAbortRankBarrier in the status
// word and returns, so a missing peer costs a wrong step, not a hung GPU.  One block of 64 threads.
constexpr int kAbortRankBarrier = 11;

__global__ void __launch_bounds__(64) ep_barrier_kernel(const __grid_constant__ PeerPtrs flags, int world, int me, int epoch,
                                                        long long limit_cycles, int* __restrict__ status) {
    const int r = threadIdx.x;
    __threadfence_system();
    if (r < world) {
        int* slot = static_cast<int*>(flags.p[r]) + me;
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(slot), "r"(epoch) : "memory");
        const int* mine = static_cast<const int*>(flags.p[me]) + r;
        const long long t0 = clock64();
        bool ok = false;
        for (unsigned polls = 0;; ++polls) {
            int v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if (v - epoch >= 0) { ok = true; break; }          // epochs only grow (wrap-safe comparison)
            if ((polls & 63u) == 63u && clock64() - t0 > limit_cycles) break;
        }
        if (!ok && status != nullptr) atomicCAS(status, 0, kAbortRankBarrier | (r << 8));
    }
    __syncthreads();
    __threadfence_system();
}

// counts_all[g][me][:] = counts[:] on every rank g (the all-gather of the per-expert pair counts,
// by plain peer stores; a rank barrier must follow before anybody reads its table).
__global__ void __launch_bounds__(256) ep_share_counts_kernel(const int32_t* __restrict__ counts, int E, int me, int world,
                                                              const __grid_constant__ PeerPtrs tables) {
    for (int i = blockIdx.x * 256 + threadIdx.x; i < E * world; i += 256 * gridDim.x) {
        const int g = i / E, e = i - g * E;
        static_cast<int32_t*>(tables.p[g])[static_cast<long long>(me) * E + e] = counts[e];
    }
}

static int ep_grid(long long work_items) {
    long long blocks = (work_items + 255) / 256;
    if (blocks > 148LL * 8) blocks = 148LL * 8;
    return static_cast<int>(blocks < 1 ? 1 : blocks);
}

static int ep_launch_check(const char* what) {
    return cudaGetLastError() == cudaSuccess ? TGO_OK : route_fail(TGO_E_CUDA, what);
}

static int fill_peers(PeerPtrs& pp, void* const* peer_ptrs, int64_t world) {
    if (peer_ptrs == nullptr || world <= 0 || world > kEpMaxRanks) return route_fail(TGO_E_ARG, "world size must be in 1..64");
    for (int r = 0; r < world; ++r) {
        if (peer_ptrs[r] == nullptr || (reinterpret_cast<uintptr_t>(peer_ptrs[r]) & 15u) != 0)
            return route_fail(TGO_E_ARG, "peer buffers must be non-null and 16-byte aligned");
        pp.p[r] = peer_ptrs[r];
    }
    return TGO_OK;
}

}  // namespace tgo

using namespace tgo;

extern "C" {

int tgo_ep_plan(const int32_t* counts_all, int64_t world, int64_t num_experts, int64_t my_rank, const int32_t* expert_ids,
                const int32_t* pair_to_sorted, int64_t n_pairs, int64_t capacity, int32_t* dst_rank, int32_t* dst_row,
                int64_t* local_indices, int32_t* local_offsets, int32_t* scratch, int32_t* overflow, void* stream) {
    if (counts_all == nullptr || expert_ids == nullptr || pair_to_sorted == nullptr || dst_rank == nullptr ||
        dst_row == nullptr || local_indices == nullptr || local_offsets == nullptr || scratch == nullptr || overflow == nullptr)
        return route_fail(TGO_E_ARG, "null pointer");
    if (world <= 0 || world > kEpMaxRanks || my_rank < 0 || my_rank >= world)
        return route_fail(TGO_E_ARG, "world size must be in 1..64 and the rank inside it");
    if (num_experts <= 0 || num_experts > 4096 || num_experts % world != 0)
        return route_fail(TGO_E_ARG, "num_experts must be in 1..4096 and divisible by the world size");
    if (n_pairs <= 0 || n_pairs > INT32_MAX || capacity <= 0 || capacity > INT32_MAX)
        return route_fail(TGO_E_ARG, "n_pairs and capacity must be in 1..2^31-1");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int E = static_cast<int>(num_experts), W = static_cast<int>(world), EL = E / W;
    ep_offsets_kernel<<<1, 1024, 0, s>>>(counts_all, W, E, EL, static_cast<int>(my_rank), static_cast<int>(capacity),
                                         scratch, scratch + E, local_indices, local_offsets);
    ep_map_kernel<<<static_cast<int>((n_pairs + 255) / 256), 256, 0, s>>>(
        expert_ids, pair_to_sorted, scratch, scratch + E, static_cast<int>(n_pairs), E, EL, static_cast<int>(capacity),
        dst_rank, dst_row, overflow);
    return ep_launch_check("expert-parallel plan kernel launch failed");
}

int* tgo_status_word(void);   // tgo_api.cu

int tgo_ep_barrier(void* const* flag_ptrs, int64_t world, int64_t my_rank, int64_t epoch, int64_t limit_cycles, void* stream) {
    if (world <= 0 || world > kEpMaxRanks || my_rank < 0 || my_rank >= world)
        return route_fail(TGO_E_ARG, "world size must be in 1..64 and the rank inside it");
    if (limit_cycles < 1000 || limit_cycles > 4000000000LL)
        return route_fail(TGO_E_ARG, "limit_cycles must be in 1000..4000000000 (about two seconds)");
    PeerPtrs pp = {};
    const int rc = fill_peers(pp, flag_ptrs, world);
    if (rc != TGO_OK) return rc;
    ep_barrier_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(pp, static_cast<int>(world), static_cast<int>(my_rank),
                                                                        static_cast<int>(epoch), limit_cycles, tgo_status_word());
    return ep_launch_check("ep_barrier_kernel launch failed");
}

int tgo_ep_share_counts(const int32_t* counts, int64_t num_experts, int64_t my_rank, void* const* table_ptrs, int64_t world,
                        void* stream) {
    if (counts == nullptr) return route_fail(TGO_E_ARG, "null pointer");
    if (num_experts <= 0 || num_experts > 4096 || world <= 0 || world > kEpMaxRanks || my_rank < 0 || my_rank >= world)
        return route_fail(TGO_E_ARG, "num_experts must be in 1..4096, the world size in 1..64 and the rank inside it");
    PeerPtrs pp = {};
    const int rc = fill_peers(pp, table_ptrs, world);
    if (rc != TGO_OK) return rc;
    const int n = static_cast<int>(num_experts * world);
    ep_share_counts_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        counts, static_cast<int>(num_experts), static_cast<int>(my_rank), static_cast<int>(world), pp);
    return ep_launch_check("ep_share_counts_kernel launch failed");
}

int tgo_ep_dispatch(const void* src, int64_t divisor, const int32_t* dst_rank, const int32_t* dst_row, int64_t n_pairs,
                    int64_t width, void* const* peer_ptrs, int64_t world, void* stream) {
    if (src == nullptr || dst_rank == nullptr || dst_row == nullptr) return route_fail(TGO_E_ARG, "null pointer");
    if (n_pairs <= 0 || width <= 0 || (width * 2) % 16 != 0 || divisor <= 0 || divisor > INT32_MAX)
        return route_fail(TGO_E_ARG, "dispatch needs pairs > 0, a row length that is a multiple of 8 and divisor > 0");
    if ((reinterpret_cast<uintptr_t>(src) & 15u) != 0) return route_fail(TGO_E_ARG, "src must be 16-byte aligned");
    PeerPtrs pp = {};
    const int rc = fill_peers(pp, peer_ptrs, world);
    if (rc != TGO_OK) return rc;
    const int vec = static_cast<int>(width / 8);
    ep_dispatch_kernel<<<ep_grid(n_pairs * vec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), static_cast<int>(divisor), dst_rank, dst_row, n_pairs, vec, pp);
    return ep_launch_check("ep_dispatch_kernel launch failed");
}

int tgo_ep_pull(void* const* peer_ptrs, int64_t world, const int32_t* dst_rank, const int32_t* dst_row, const float* weights,
                void* out, int64_t n_out, int64_t group, int64_t width, void* stream) {
    if (dst_rank == nullptr || dst_row == nullptr || out == nullptr) return route_fail(TGO_E_ARG, "null pointer");
    if (n_out <= 0 || group <= 0 || group > 1024 || width <= 0 || (width * 2) % 16 != 0)
        return route_fail(TGO_E_ARG, "pull needs rows > 0, 1 <= group <= 1024 and a row length that is a multiple of 8");
    if ((reinterpret_cast<uintptr_t>(out) & 15u) != 0) return route_fail(TGO_E_ARG, "out must be 16-byte aligned");
    PeerPtrs pp = {};
    const int rc = fill_peers(pp, peer_ptrs, world);
    if (rc != TGO_OK) return rc;
    const int vec = static_cast<int>(width / 8);
    ep_pull_kernel<<<ep_grid(n_out * vec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        pp, dst_rank, dst_row, weights, static_cast<uint4*>(out), n_out, static_cast<int>(group), vec);
    return ep_launch_check("ep_pull_kernel launch failed");
}

static int token_maps(const int32_t* dst_rank, const int32_t* dst_row, int64_t tokens, int64_t top_k, int64_t my_rank,
                      int64_t tokens_per_rank, void* const* row_slot_ptrs, void* const* slot_rows_ptrs,
                      const float* pair_weights, void* const* row_weight_ptrs, int64_t world, void* result,
                      int64_t result_width, void* stream) {
    if (dst_rank == nullptr || dst_row == nullptr) return route_fail(TGO_E_ARG, "null pointer");
    if (tokens <= 0 || top_k <= 0 || top_k > 1024 || tokens > tokens_per_rank || my_rank < 0 || my_rank >= world ||
        tokens_per_rank * world * top_k > INT32_MAX)
        return route_fail(TGO_E_ARG, "token maps need 0 < tokens <= tokens_per_rank, 0 < top_k <= 1024 and the rank inside the world");
    if ((pair_weights == nullptr) != (row_weight_ptrs == nullptr))
        return route_fail(TGO_E_ARG, "pair_weights and row_weight_ptrs must both be given or both be null");
    PeerPtrs rs = {}, sr = {}, rw = {};
    int rc = fill_peers(rs, row_slot_ptrs, world);
    if (rc == TGO_OK) rc = fill_peers(sr, slot_rows_ptrs, world);
    if (rc == TGO_OK && row_weight_ptrs != nullptr) rc = fill_peers(rw, row_weight_ptrs, world);
    if (rc != TGO_OK) return rc;
    const long long n_pairs = tokens * top_k;
    ep_token_maps_kernel<<<static_cast<int>((n_pairs + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        dst_rank, dst_row, n_pairs, static_cast<int>(top_k), static_cast<int>(world), my_rank * tokens_per_rank, rs, sr,
        pair_weights, rw, static_cast<uint4*>(result), static_cast<int>(result_width / 8));
    return ep_launch_check("ep_token_maps_kernel launch failed");
}

int tgo_ep_token_maps(const int32_t* dst_rank, const int32_t* dst_row, int64_t tokens, int64_t top_k, int64_t my_rank,
                      int64_t tokens_per_rank, void* const* row_slot_ptrs, void* const* slot_rows_ptrs,
                      const float* pair_weights, void* const* row_weight_ptrs, int64_t world, void* stream) {
    return token_maps(dst_rank, dst_row, tokens, top_k, my_rank, tokens_per_rank, row_slot_ptrs, slot_rows_ptrs, pair_weights,
                      row_weight_ptrs, world, nullptr, 0, stream);
}

int tgo_ep_token_maps_rows(const int32_t* dst_rank, const int32_t* dst_row, int64_t tokens, int64_t top_k, int64_t my_rank,
                           int64_t tokens_per_rank, void* const* row_slot_ptrs, void* const* slot_rows_ptrs,
                           int64_t world, void* result, int64_t result_width, void* stream) {
    if (result == nullptr || result_width <= 0 || (result_width * 2) % 16 != 0)
        return route_fail(TGO_E_ARG, "the result buffer needs a row length that is a multiple of 8");
    return token_maps(dst_rank, dst_row, tokens, top_k, my_rank, tokens_per_rank, row_slot_ptrs, slot_rows_ptrs, nullptr,
                      nullptr, world, result, result_width, stream);
}

int tgo_ep_dispatch_tokens(const void* src, const int32_t* dst_rank, int64_t tokens, int64_t top_k, int64_t width,
                           int64_t my_rank, int64_t tokens_per_rank, void* const* token_buffer_ptrs, int64_t world,
                           void* stream) {
    if (src == nullptr || dst_rank == nullptr) return route_fail(TGO_E_ARG, "null pointer");
    if (tokens <= 0 || top_k <= 0 || tokens > tokens_per_rank || width <= 0 || (width * 2) % 16 != 0 || my_rank < 0 ||
        my_rank >= world)
        return route_fail(TGO_E_ARG, "token dispatch needs 0 < tokens <= tokens_per_rank, a row length that is a multiple of 8 and the rank inside the world");
    if ((reinterpret_cast<uintptr_t>(src) & 15u) != 0) return route_fail(TGO_E_ARG, "src must be 16-byte aligned");
    PeerPtrs pp = {};
    const int rc = fill_peers(pp, token_buffer_ptrs, world);
    if (rc != TGO_OK) return rc;
    const int vec = static_cast<int>(width / 8);
    ep_dispatch_tokens_kernel<<<ep_grid(tokens * vec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), dst_rank, tokens, static_cast<int>(top_k), vec, my_rank * tokens_per_rank, pp);
    return ep_launch_check("ep_dispatch_tokens_kernel launch failed");
}

int tgo_ep_expand(const void* token_buffer, int64_t n_slots, const int32_t* row_slot, const int32_t* n_rows_device,
                  void* rows, int64_t capacity, int64_t width, void* stream) {
    if (token_buffer == nullptr || row_slot == nullptr || n_rows_device == nullptr || rows == nullptr)
        return route_fail(TGO_E_ARG, "null pointer");
    if (capacity <= 0 || n_slots <= 0 || width <= 0 || (width * 2) % 16 != 0)
        return route_fail(TGO_E_ARG, "expand needs capacity > 0, slots > 0 and a row length that is a multiple of 8");
    const int vec = static_cast<int>(width / 8);
    ep_expand_kernel<<<ep_grid(capacity * vec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(token_buffer), row_slot, n_rows_device, static_cast<uint4*>(rows), capacity, n_slots, vec);
    return ep_launch_check("ep_expand_kernel launch failed");
}

int tgo_ep_zero_dropped(const int32_t* dst_rank, int64_t n_pairs, void* result, int64_t width, void* stream) {
    if (dst_rank == nullptr || result == nullptr) return route_fail(TGO_E_ARG, "null pointer");
    if (n_pairs <= 0 || width <= 0 || (width * 2) % 16 != 0)
        return route_fail(TGO_E_ARG, "zeroing dropped rows needs pairs > 0 and a row length that is a multiple of 8");
    const long long blocks = (n_pairs * 32 + 255) / 256;
    if (blocks > INT32_MAX) return route_fail(TGO_E_ARG, "too many routed pairs");
    ep_zero_dropped_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        dst_rank, n_pairs, static_cast<uint4*>(result), static_cast<int>(width / 8));
    return ep_launch_check("ep_zero_dropped_kernel launch failed");
}

int tgo_ep_row_pointers(const int32_t* row_slot, const int32_t* slot_rows, const int32_t* n_rows_device, int64_t capacity,
                        int64_t n_slots, int64_t top_k, int64_t tokens_per_rank, void* const* result_ptrs, int64_t world,
                        int64_t width, void** row_ptrs, void* stream) {
    if (row_slot == nullptr || slot_rows == nullptr || n_rows_device == nullptr || row_ptrs == nullptr)
        return route_fail(TGO_E_ARG, "null pointer");
    if (capacity <= 0 || n_slots <= 0 || top_k <= 0 || tokens_per_rank <= 0 || width <= 0 || (width * 2) % 16 != 0 ||
        n_slots != world * tokens_per_rank)
        return route_fail(TGO_E_ARG, "row pointers need capacity > 0, slots = world * tokens_per_rank and a row length that is a multiple of 8");
    PeerPtrs res = {};
    const int rc = fill_peers(res, result_ptrs, world);
    if (rc != TGO_OK) return rc;
    ep_row_pointers_kernel<<<ep_grid(capacity), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        row_slot, slot_rows, n_rows_device, capacity, n_slots, static_cast<int>(top_k), tokens_per_rank, res, width * 2,
        reinterpret_cast<unsigned long long*>(row_ptrs));
    return ep_launch_check("ep_row_pointers_kernel launch failed");
}

int tgo_ep_reduce(const void* rows, const int32_t* slot_rows, int64_t n_slots, int64_t top_k, void* partial_sums,
                  int64_t width, void* stream) {
    if (rows == nullptr || slot_rows == nullptr || partial_sums == nullptr) return route_fail(TGO_E_ARG, "null pointer");
    if (n_slots <= 0 || top_k <= 0 || width <= 0 || (width * 2) % 16 != 0)
        return route_fail(TGO_E_ARG, "reduce needs slots > 0, top_k > 0 and a row length that is a multiple of 8");
    const int vec = static_cast<int>(width / 8);
    ep_reduce_kernel<<<ep_grid(n_slots * vec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(rows), slot_rows, n_slots, static_cast<int>(top_k), static_cast<uint4*>(partial_sums), vec);
    return ep_launch_check("ep_reduce_kernel launch failed");
}

int tgo_ep_pull_tokens(void* const* partial_sum_ptrs, int64_t world, const int32_t* dst_rank, int64_t tokens, int64_t top_k,
                       int64_t my_rank, int64_t tokens_per_rank, void* out, int64_t width, void* stream) {
    if (dst_rank == nullptr || out == nullptr) return route_fail(TGO_E_ARG, "null pointer");
    if (tokens <= 0 || top_k <= 0 || tokens > tokens_per_rank || width <= 0 || (width * 2) % 16 != 0 || my_rank < 0 ||
        my_rank >= world)
        return route_fail(TGO_E_ARG, "token pull needs 0 < tokens <= tokens_per_rank, a row length that is a multiple of 8 and the rank inside the world");
    if ((reinterpret_cast<uintptr_t>(out) & 15u) != 0) return route_fail(TGO_E_ARG, "out must be 16-byte aligned");
    PeerPtrs pp = {};
    const int rc = fill_peers(pp, partial_sum_ptrs, world);
    if (rc != TGO_OK) return rc;
    const int vec = static_cast<int>(width / 8);
    ep_pull_tokens_kernel<<<ep_grid(tokens * vec), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        pp, dst_rank, tokens, static_cast<int>(top_k), vec, my_rank * tokens_per_rank, static_cast<uint4*>(out));
    return ep_launch_check("ep_pull_tokens_kernel launch failed");
}

}  // extern "C"
