/*
 * tgo_mmq.h - C ABI of the sm_100a quantized-weight matmul library (libtgo_mmq.so).
 *
 * This is the boundary a host layer binds instead of the reference's ROCm extension
 * (csrc/mmq_hip.cu): one entry point per native operator body.  Plain pointers and sizes only;
 * every pointer is a device pointer on the current CUDA device unless stated otherwise; every
 * call is asynchronous on `stream` (a cudaStream_t passed as void*), performs no host
 * synchronisation and no device-to-host read, borrows its inputs and writes only its outputs
 * and workspace.  Return value: 0 on success, a negative TGO_E_* code otherwise, with a
 * human-readable message available from tgo_last_error() on the calling thread.
 *
 * Tensor conventions (reference: csrc/mmq_hip.cu:325-406, 587-631):
 *   activations / outputs / gradients: bf16, row-major, contiguous, 16-byte aligned;
 *   packed weights: raw GGUF super-blocks, uint8, row n = K/256 consecutive blocks, 16-byte
 *   aligned; grouped weights are [E][N][K/256 * block_bytes];
 *   quant types use the GGML ids (Q3_K 11, Q4_K 12, Q5_K 13, Q6_K 14, IQ2_S 22);
 *   K must be a positive multiple of 256;
 *   routing metadata: expert_indices int64[G], expert_offsets int32[G] = cumulative END row of
 *   each group (group g covers rows [offsets[g-1], offsets[g]), offsets[-1] = 0).  A group with
 *   an out-of-range expert id or an empty / out-of-range row span is skipped on the device and
 *   its output rows are left untouched (reference: csrc/mmq_core.cuh:468-476).
 */
#ifndef TGO_MMQ_H_
#define TGO_MMQ_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TGO_OK 0
#define TGO_E_ARG (-1)      /* bad argument (null pointer, size, alignment, type) */
#define TGO_E_CUDA (-2)     /* a CUDA runtime / driver call failed */
#define TGO_E_WORKSPACE (-3) /* workspace too small */
#define TGO_E_DEVICE (-4)   /* a kernel reported a timed-out wait (see tgo_device_status) */

#define TGO_Q3_K 11
#define TGO_Q4_K 12
#define TGO_Q5_K 13
#define TGO_Q6_K 14
#define TGO_IQ2_S 22

/* Most tiles (rows / 256 + groups) tgo_grouped_fwd_noalloc accepts. */
#define TGO_NOALLOC_MAX_TILES 4096

/* Library version (major*10000 + minor*100 + patch). */
int tgo_version(void);

/* Message of the last failing call on this thread ("" if none). */
const char* tgo_last_error(void);

/* Bytes of one 256-weight super-block of `quant_type`, or -1 if unsupported.
 * Replaces packed_block_bytes (csrc/mmq_hip.cu:38-48). */
int64_t tgo_block_bytes(int quant_type);

/* Reads (synchronously) and clears the device status word that kernels set when a bounded wait
 * gives up: *status = code | block << 8, 0 means no kernel gave up since the last read.  A kernel
 * that gave up returns with its outputs incomplete, and the asynchronous calls cannot report that
 * themselves: poll this where the host synchronises anyway (end of a step), or set the environment
 * variable TGO_CHECK_STATUS=1, which makes every matmul call wait for its stream and return
 * TGO_E_DEVICE if the word is set (a debugging aid: it serialises host and device).  No
 * counterpart in the reference (its kernels have no inter-warp waits). */
int tgo_device_status(int* status);

/* Test hook for the time-out path of the kernels' bounded waits: launches a one-block kernel in
 * which a warp waits, for at most limit_cycles SM cycles (1000..200000000), on a barrier nobody
 * arrives on.  The wait gives up and the kernel records code 10 in the status word, which
 * tgo_device_status then returns (and clears).  Nothing else is in flight in that kernel, the
 * context stays usable.  No counterpart in the reference. */
int tgo_selftest_wait_timeout(int64_t limit_cycles, void* stream);

/* Decode n_blocks consecutive super-blocks to bf16 (round-to-nearest-even), 256 values each.
 * The same device decoders feed the matmul kernels; exposed for bit-exact checks against
 * decode_gguf_value (csrc/ck/gguf_decode.cuh:54-149). */
int tgo_dequantize_bf16(const void* packed, int64_t n_blocks, int quant_type, void* out_bf16,
                        void* stream);

/* Dense forward  Y[M,N] = X[M,K] * W[N,K]^T.
 * Replaces the device work of mmq_cuda -> launch_dense_mmq (csrc/mmq_hip.cu:117-147, 587-678). */
int tgo_mmq_fwd(const void* x, const void* packed_weight, void* y, int64_t rows,
                int64_t out_features, int64_t in_features, int quant_type, void* stream);

/* Dense input gradient  dX[M,K] = dY[M,N] * W[N,K].
 * Replaces mmq_grad_input_cuda -> ck::launch_dense_mmq_grad_input
 * (csrc/mmq_hip.cu:680-774, csrc/ck/mmq_backward.cuh:1066-1241). */
int tgo_mmq_dx(const void* dy, const void* packed_weight, void* dx, int64_t rows,
               int64_t out_features, int64_t in_features, int quant_type, void* stream);

/* Dense input gradient with a workspace for the split reduction.  When the problem has few tiles
 * and a long reduction (few rows, very many out-features: an LM head of 248320 x 2048 gives 8 tiles
 * of 3880 steps) the out-features are cut into ranges, one tile each, whose fp32 partial sums go to
 * `workspace` and are added in ascending order by a second kernel; results then differ from
 * tgo_mmq_dx only by that summation order.  tgo_mmq_dx_workspace_bytes returns the bytes needed on
 * the current device (0: no split, and tgo_mmq_dx_ws is tgo_mmq_dx).  Replaces the small-M dispatch
 * of ck::launch_dense_mmq_grad_input (csrc/ck/mmq_backward.cuh:1066-1241), which picks narrower
 * tiles for the same reason; shapes: docs/mmq_bwd_optimization.md:442-446. */
int64_t tgo_mmq_dx_workspace_bytes(int64_t rows, int64_t out_features, int64_t in_features,
                                   int quant_type);
int tgo_mmq_dx_ws(const void* dy, const void* packed_weight, void* dx, int64_t rows,
                  int64_t out_features, int64_t in_features, int quant_type, void* workspace,
                  int64_t workspace_bytes, void* stream);

/* Several dense projections of the same activations in one call: ys[i] = X * W_i^T for
 * num_weights (1..4) packed weights of the same quant type and shape [out_features, in_features];
 * packed_weights and ys are HOST arrays of device pointers.  Two weight sets share a launch, as the
 * gate/up pair does in tgo_grouped_fwd; every ys[i] is bit-identical to tgo_mmq_fwd on W_i alone.
 * No counterpart in the reference, which lists a dense pair / multi-projection operator as its
 * remaining dense-forward work (docs/mmq_fwd_optimization.md:299-307: there the shared cost is the
 * q8_1 quantisation of the activations, which this library's bf16 path does not have at all). */
int tgo_mmq_fwd_multi(const void* x, const void* const* packed_weights, void* const* ys,
                      int64_t num_weights, int64_t rows, int64_t out_features, int64_t in_features,
                      int quant_type, void* stream);

/* Workspace bytes the grouped calls below need for `rows` routed rows in `num_groups` groups
 * (the device-built tile list; reference: new_grouped_row_task_workspace,
 * csrc/mmq_hip.cu:544-558). */
int64_t tgo_grouped_workspace_bytes(int64_t rows, int64_t num_groups);

/* Builds the tile list (device prefix sum over the groups) into `workspace`: int32 count at byte
 * 0, then from byte 16 one int32x4 (expert, first row, tokens, group) per tile; a group is cut
 * into ceil(size / max_tile_tokens) tiles of equal size rounded up to 16.  max_tile_tokens is
 * 256 or 512 (a tile of more than 256 tokens uses both accumulators of the matmul kernel and
 * shares each decoded weight step between them).  The grouped calls below do this themselves;
 * exposed for tests.  Replaces grouped_mmq_build_row_tasks (csrc/mmq_core.cuh:516-571). */
int tgo_build_tiles(const int64_t* expert_indices, const int32_t* expert_offsets,
                    int64_t num_groups, int64_t num_experts, int64_t rows,
                    int64_t max_tile_tokens, void* workspace, int64_t workspace_bytes,
                    void* stream);

/* Grouped forward over expert-sorted rows; with w1/y1 non-null also the second projection of a
 * gate/up pair from the same activations (y0 = X*W0[e]^T, y1 = X*W1[e]^T).
 * Replaces grouped_mmq_cuda and grouped_mmq_pair_cuda (csrc/mmq_hip.cu:954-1193). */
int tgo_grouped_fwd(const void* x, const void* w0, const void* w1, void* y0, void* y1,
                    const int64_t* expert_indices, const int32_t* expert_offsets,
                    int64_t num_groups, int64_t num_experts, int64_t rows, int64_t out_features,
                    int64_t in_features, int quant_type, void* workspace, int64_t workspace_bytes,
                    void* stream);

/* The same forward (one projection) with scattered output rows: row r of the result is stored at
 * y_rows[r] (a device array of `rows` addresses, each 16-byte aligned and writable by this GPU -
 * its own memory or a peer's; null drops the row) instead of a contiguous [rows][out_features]
 * tensor.  The matmul kernel's epilogue stores straight there, so an expert-parallel step can
 * return every routed pair's row to the GPU that owns the token from inside the matmul
 * (tgo_ep_row_pointers builds the table).  out_features must be a multiple of 8.  Values are
 * bit-identical to tgo_grouped_fwd.  No counterpart in the reference (it is single-GPU). */
int tgo_grouped_fwd_rows(const void* x, const void* w, void* const* y_rows,
                         const int64_t* expert_indices, const int32_t* expert_offsets,
                         int64_t num_groups, int64_t num_experts, int64_t rows,
                         int64_t out_features, int64_t in_features, int quant_type,
                         void* workspace, int64_t workspace_bytes, void* stream);

/* Grouped input gradient dX = dY0*W0[e] (+ dY1*W1[e] when dy1/w1 are non-null; both products
 * are summed in fp32 before the single bf16 rounding).
 * Replaces grouped_mmq_grad_input_cuda and grouped_mmq_pair_grad_input_cuda
 * (csrc/mmq_hip.cu:776-952, csrc/ck/grouped_mmq_backward.cuh:154-306, 460-568). */
int tgo_grouped_dx(const void* dy0, const void* dy1, const void* w0, const void* w1, void* dx,
                   const int64_t* expert_indices, const int32_t* expert_offsets,
                   int64_t num_groups, int64_t num_experts, int64_t rows, int64_t out_features,
                   int64_t in_features, int quant_type, void* workspace, int64_t workspace_bytes,
                   void* stream);

/* ---- routing helpers (the steps either side of the grouped projections) ------------------------
 * The reference takes rows that its caller already sorted by expert; these entry points do that
 * sort, the gather and the top-k combine on the device with no device-to-host read (every expert
 * gets a group, empty ones included, so the group count is the static expert count). */

/* Workspace bytes for tgo_route_sort. */
int64_t tgo_route_workspace_bytes(int64_t n_pairs, int64_t num_experts);

/* Stable counting sort of routed (token, slot) pairs by expert id.  expert_ids int32[n_pairs]
 * (pair index = token * top_k + slot); outputs: sorted_to_pair int32[n_pairs] (pair held by each
 * sorted row), pair_to_sorted int32[n_pairs] (its inverse; -1 for an out-of-range id),
 * expert_indices int64[E] = 0..E-1 and expert_offsets int32[E] = cumulative end rows: exactly the
 * metadata of validate_grouped_mmq (csrc/mmq_hip.cu:325-406); expert_counts int32[E] (may be null)
 * = pairs per expert.  Device prefix sum; counterpart of
 * the reference's only device scan, grouped_mmq_build_row_tasks (csrc/mmq_core.cuh:516-571). */
int tgo_route_sort(const int32_t* expert_ids, int64_t n_pairs, int64_t num_experts,
                   int32_t* sorted_to_pair, int32_t* pair_to_sorted, int64_t* expert_indices,
                   int32_t* expert_offsets, int32_t* expert_counts, void* workspace,
                   int64_t workspace_bytes, void* stream);

/* dst[r][:] = src[index[r] / divisor][:] for bf16 rows of `width` (a multiple of 8); with
 * index = sorted_to_pair and divisor = top_k this builds the expert-sorted activation rows.  An
 * index that is negative, or whose source row is not below src_rows, gives a row of zeros. */
int tgo_gather_rows(const void* src, int64_t src_rows, const int32_t* index, int64_t divisor,
                    void* dst, int64_t n_rows, int64_t width, void* stream);

/* out[t][:] = sum over slots of weights[t][slot] * rows[pair_to_sorted[t*top_k+slot]][:] (fp32
 * accumulation, one bf16 rounding; weights may be null = 1). */
int tgo_combine_rows(const void* rows, const int32_t* pair_to_sorted, const float* weights,
                     void* out, int64_t tokens, int64_t top_k, int64_t width, void* stream);

/* bf16 activations [rows][width] -> q8_1-style blocks of 32 values: int8 quants q[rows][width],
 * fp32 scales d[rows][width/32] = amax/127 and fp32 sums of the unquantised values
 * sum[rows][width/32].  Replaces quantize_bf16_mmq_q8_1 (csrc/mmq_core.cuh:151-209), with fp32
 * instead of fp16 scales.  Not used by the bf16-dequant matmul path; provided for the int8
 * variant of the forward. */
int tgo_quantize_q8(const void* x, int64_t rows, int64_t width, void* q, float* d, float* sum,
                    void* stream);

/* ---- expert-parallel row exchange over peer memory (no counterpart in the reference, which is
 * single-GPU).  One process per GPU; expert e lives on rank e / (num_experts / world).  Every rank
 * owns a receive buffer of `capacity` rows that its peers can address (peer_ptrs[r] = rank r's
 * buffer, e.g. from CUDA IPC / symmetric memory); rows are written into and read from those
 * buffers with plain 16-byte peer stores and loads.  None of these calls waits for another GPU:
 * the host layer orders the phases with stream-ordered collectives (dispatch | barrier | grouped
 * matmul | barrier | pull). */

/* Stream-ordered barrier between the ranks by peer memory alone (no collective library): rank r
 * stores `epoch` (which must grow by one with every barrier of a series) into slot r of every rank's
 * flag array (flag_ptrs[g] = rank g's int32[world] array, zero-initialised, peer-addressable) and
 * waits until all slots of its own array have reached `epoch`.  Everything this GPU wrote to peer
 * memory before the call is visible to a peer's kernels launched after that peer's call returns.
 * The wait is bounded by limit_cycles SM cycles (1000..4000000000); when it runs out, code 11 is
 * recorded in the status word (tgo_device_status) and the kernel returns. */
int tgo_ep_barrier(void* const* flag_ptrs, int64_t world, int64_t my_rank, int64_t epoch,
                   int64_t limit_cycles, void* stream);

/* counts_all[g][my_rank][:] = counts[:] for every rank g: the all-gather of the per-expert pair
 * counts (tgo_route_sort's expert_counts) by peer stores; table_ptrs[g] = rank g's
 * int32[world][num_experts] table.  Follow with tgo_ep_barrier before reading the table. */
int tgo_ep_share_counts(const int32_t* counts, int64_t num_experts, int64_t my_rank,
                        void* const* table_ptrs, int64_t world, void* stream);

/* From the per-expert pair counts of all ranks (counts_all int32[world][num_experts], identical
 * on every rank) and this rank's routing (expert_ids, pair_to_sorted from tgo_route_sort):
 * dst_rank / dst_row int32[n_pairs] = where each routed pair goes (-1 if dropped; *overflow is set
 * to 1 if a row would not fit in `capacity`), and the group metadata of the local experts in the
 * receive buffer (local_indices int64[E/world], local_offsets int32[E/world]: the contract of
 * validate_grouped_mmq, csrc/mmq_hip.cu:325-406).  scratch: int32[2 * num_experts]. */
int tgo_ep_plan(const int32_t* counts_all, int64_t world, int64_t num_experts, int64_t my_rank,
                const int32_t* expert_ids, const int32_t* pair_to_sorted, int64_t n_pairs,
                int64_t capacity, int32_t* dst_rank, int32_t* dst_row, int64_t* local_indices,
                int32_t* local_offsets, int32_t* scratch, int32_t* overflow, void* stream);

/* peer[dst_rank[i]][dst_row[i]][:] = src[i / divisor][:] for bf16 rows of `width` (multiple of 8).
 * peer_ptrs is a HOST array of `world` device pointers. */
int tgo_ep_dispatch(const void* src, int64_t divisor, const int32_t* dst_rank, const int32_t* dst_row,
                    int64_t n_pairs, int64_t width, void* const* peer_ptrs, int64_t world,
                    void* stream);

/* out[t][:] = sum over the `group` consecutive pairs of t of weights[pair] * peer[dst_rank][dst_row][:]
 * (group = 1: one row per pair; group = top_k: the per-token combine; fp32 accumulation, one bf16
 * rounding; weights may be null = 1). */
int tgo_ep_pull(void* const* peer_ptrs, int64_t world, const int32_t* dst_rank, const int32_t* dst_row,
                const float* weights, void* out, int64_t n_out, int64_t group, int64_t width,
                void* stream);

/* Token-level exchange: with top-k routing several of a token's experts usually sit on the same
 * GPU, so a token's row is sent once per destination GPU (not once per routed pair) and one
 * partial gradient sum per GPU comes back; the owner replicates rows into / reduces rows out of
 * its expert-major buffers locally.  Token t of rank r owns slot r * tokens_per_rank + t in every
 * GPU's token buffers ([world * tokens_per_rank][width] bf16).  No counterpart in the reference.
 *
 *  tgo_ep_token_maps      after tgo_ep_plan: writes, on every owner g, slot_rows[g][slot][s] (the row
 *                         of the slot's s-th routed pair on g, or -1; int32 [world*tokens_per_rank][top_k])
 *                         and, on the pair's owner, row_slot[owner][row] = slot (int32 [capacity]) and, when
 *                         pair_weights (fp32 [tokens * top_k]) is given, row_weight[owner][row] = the pair's
 *                         routing weight (fp32 [capacity]; both null otherwise);
 *  tgo_ep_dispatch_tokens writes src[t] into the token buffer of every GPU that owns one of t's experts;
 *  tgo_ep_expand          owner side: rows[row] = token_buffer[row_slot[row]] for row < *n_rows_device
 *                         (a device int32, e.g. the last cumulative offset of tgo_ep_plan); a row whose
 *                         entry is outside [0, n_slots) is left untouched;
 *  tgo_ep_row_pointers    owner side, for tgo_grouped_fwd_rows: row_ptrs[row] = result_ptrs[owner] + (token * top_k
 *                         + s) * width * 2 for the routed pair (slot = owner * tokens_per_rank + token, s) that row
 *                         belongs to (found through row_slot and slot_rows), null for a row nobody announced;
 *                         result_ptrs are this GPU's addresses of every rank's [tokens_per_rank * top_k][width]
 *                         result buffer;
 *  tgo_ep_zero_dropped    token owner's side of that scheme: zeroes result[i] for the routed pairs with
 *                         dst_rank[i] < 0 (dropped for lack of room), which nobody else writes;
 *  tgo_ep_reduce          owner side: partial_sums[slot] = sum of rows[slot_rows[slot][s]] (fp32, one rounding);
 *  tgo_ep_pull_tokens     out[t] = sum over the GPUs owning one of t's experts of their partial_sums[slot]. */
int tgo_ep_token_maps(const int32_t* dst_rank, const int32_t* dst_row, int64_t tokens, int64_t top_k,
                      int64_t my_rank, int64_t tokens_per_rank, void* const* row_slot_ptrs,
                      void* const* slot_rows_ptrs, const float* pair_weights,
                      void* const* row_weight_ptrs, int64_t world, void* stream);
int tgo_ep_dispatch_tokens(const void* src, const int32_t* dst_rank, int64_t tokens, int64_t top_k,
                           int64_t width, int64_t my_rank, int64_t tokens_per_rank,
                           void* const* token_buffer_ptrs, int64_t world, void* stream);
int tgo_ep_expand(const void* token_buffer, int64_t n_slots, const int32_t* row_slot,
                  const int32_t* n_rows_device, void* rows, int64_t capacity, int64_t width,
                  void* stream);
int tgo_ep_zero_dropped(const int32_t* dst_rank, int64_t n_pairs, void* result, int64_t width,
                        void* stream);
/* tgo_ep_token_maps + tgo_ep_zero_dropped as one launch (the same fusion of tgo_ep_expand with
 * tgo_ep_row_pointers was measured and is slower than the two launches: the pointer look-up
 * stalls the copy) */
int tgo_ep_token_maps_rows(const int32_t* dst_rank, const int32_t* dst_row, int64_t tokens, int64_t top_k,
                           int64_t my_rank, int64_t tokens_per_rank, void* const* row_slot_ptrs,
                           void* const* slot_rows_ptrs, int64_t world, void* result,
                           int64_t result_width, void* stream);
int tgo_ep_row_pointers(const int32_t* row_slot, const int32_t* slot_rows, const int32_t* n_rows_device,
                        int64_t capacity, int64_t n_slots, int64_t top_k, int64_t tokens_per_rank,
                        void* const* result_ptrs, int64_t world, int64_t width, void** row_ptrs,
                        void* stream);
int tgo_ep_reduce(const void* rows, const int32_t* slot_rows, int64_t n_slots, int64_t top_k,
                  void* partial_sums, int64_t width, void* stream);
int tgo_ep_pull_tokens(void* const* partial_sum_ptrs, int64_t world, const int32_t* dst_rank,
                       int64_t tokens, int64_t top_k, int64_t my_rank, int64_t tokens_per_rank,
                       void* out, int64_t width, void* stream);

/* ---- element-wise step of the MoE feed-forward block between the grouped projections (the
 * reference leaves activation and combine to its caller, README.md:3; csrc/mmq_hip.cu:1054-1193
 * returns gate and up separately).  bf16 rows of `width` (a multiple of 8), fp32 arithmetic.
 * row_scale (fp32 [rows], may be null = 1) is the routing weight of each expert-major row;
 * n_rows_device (device int32, may be null) limits the work to the rows that exist. */

/* out = row_scale * silu(gate) * up */
int tgo_swiglu_fwd(const void* gate, const void* up, const float* row_scale, void* out, int64_t rows,
                   int64_t width, const int32_t* n_rows_device, void* stream);

/* dgate = dh * row_scale * up * silu'(gate),  dup = dh * row_scale * silu(gate) */
int tgo_swiglu_bwd(const void* dh, const void* gate, const void* up, const float* row_scale,
                   void* dgate, void* dup, int64_t rows, int64_t width,
                   const int32_t* n_rows_device, void* stream);

/* Grouped forward for callers that cannot hand over a workspace and must not trigger a device
 * allocation: the same operation and results as tgo_grouped_fwd, with the tile list kept in a
 * fixed array inside the library instead of caller memory.  No counterpart in the reference.
 *
 * Who needs it: a host runtime that reserved all device memory for its own plan at start-up, an
 * inference loop that forbids cudaMalloc/cudaFree while serving because they stall every stream of
 * the device, or a foreign-function binding that only receives input and output buffers and has
 * no allocator to ask.  This call performs no cudaMalloc, no cudaFree and calls no allocating
 * library routine; the caller still passes every input and output.
 *
 * Limit: rows / 256 + num_groups must not exceed TGO_NOALLOC_MAX_TILES (4096, i.e.
 * 64 KiB + 16 B of device memory that every GPU loading the library holds until the process
 * exits); larger problems are rejected with TGO_E_WORKSPACE and must use tgo_grouped_fwd.
 * The first call on a device looks up the array's device address (the device must be current);
 * make that first call outside any stream capture.  All calls on a device share the one array,
 * which keeps whatever the previous call left in it: each call rewrites the count and every
 * entry it later reads, so nothing has to be cleared, but two calls whose kernels overlap on the
 * GPU (different streams without an ordering between them) race on it. */
int tgo_grouped_fwd_noalloc(const void* x, const void* w0, const void* w1, void* y0, void* y1,
                            const int64_t* expert_indices, const int32_t* expert_offsets,
                            int64_t num_groups, int64_t num_experts, int64_t rows,
                            int64_t out_features, int64_t in_features, int quant_type,
                            void* stream);

#ifdef __cplusplus
}
#endif

#endif /* TGO_MMQ_H_ */
