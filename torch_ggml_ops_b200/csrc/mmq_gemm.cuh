// The quantized-weight GEMM kernel for sm_100a: one persistent, warp-specialised kernel that
// serves dense, grouped and paired products in both directions.
//
//   forward  (kFwd):  Y[t, n]  = sum_k X[t, k]  * W[n, k]      (reference: csrc/mmq_core.cuh:211-267,
//                                                                450-514, 573-635)
//   backward (kBwd):  dX[t, k] = sum_n dY[t, n] * W[n, k]      (reference: csrc/ck/mmq_backward.cuh:496-1004,
//                                                                csrc/ck/grouped_mmq_backward.cuh:42-152, 308-458)
//
// The weight side sits on the UMMA M axis (128 TMEM lanes per CTA = 128 out-features forward, 128
// in-features backward) and the tokens on the UMMA N axis (16..256 TMEM columns), so a ragged
// expert group costs at most 15 (pair: 31) padded token columns and one decoded weight tile is
// reused by up to 256 tokens.  Raw GGUF super-blocks are staged into shared memory by TMA, decoded
// there to bf16 in the 128-byte-swizzled operand layout by sixteen decode warps, and consumed by
// tcgen05.mma (kind::f16, bf16 x bf16 -> fp32 in TMEM).  The same decoded image
// [weight row n][64 k] is a K-major operand forward and an MN-major operand backward, so neither
// direction transposes.  The reduction order of every output element is fixed (ascending
// reduction index, 16 per UMMA), independent of tiling, which makes grouped == dense and
// pair == two singles bit-exact.
//
// CG = 2 (the default): two CTAs of a cluster share a token tile and cover 256 weight rows with
// cta_group::2 UMMAs; each CTA decodes its own 128 rows and stages half of the tokens, the
// leader CTA (cluster rank 0) issues the UMMAs and owns the barriers both CTAs feed.
//
// Warp roles (768 threads; backward - forward places them differently, see the kernel): 0 activation
// producer (TMA), 1 UMMA issuer + TMEM owner, 2 and 3 raw weight producers (TMA, alternate stages),
// 4-19 decode (groups of warps on alternate 64-element steps: four groups of 4 for Q4_K / Q5_K, two
// groups of 8 otherwise), 20-23 epilogue (TMEM -> bf16 -> global, or to per-row destinations).
//
// Wide tiles.  A tile of more than 256 tokens (up to 512) is split into two halves that use both
// accumulators at once and share every decoded weight step: each decoded stage is consumed by two
// consecutive pipeline stages (half 0 -> accumulator a, half 1 -> accumulator a ^ 1), so the
// decode work per output element halves.  The epilogue sees the halves as two ordinary tiles.
//
// Synchronisation.  A stage is KS steps (1 for a single CTA, 2 for a pair; each step is decoded by
// one decode group); pipeline stages have running index j over all tiles of the CTA (a wide tile has two
// pipeline stages per decoded stage):
//   full[j % NB]  <- the activation TMA (expect_tx for the whole stage, announced by the leader)
//                    and the decode warps of the stage's steps (of both CTAs); the UMMA issuer
//                    waits on it once and issues the stage's 4 * KS UMMAs;
//   done[j % NB]  <- one tcgen05.commit after those UMMAs (one per CTA of a pair).  Operands live
//                    in rings of one-step slots (NBS activation slots, NAS decoded-weight slots):
//                    whoever refills the slot of step i waits for done of the stage that held step
//                    i - NBS (activation producer) or i - NAS (decode warps);
//   raw_full / raw_empty: TMA raw-block ring <-> decode;  acc_full / acc_empty: TMEM <-> epilogue.
// All waits are bounded (ptx.cuh); a wait that gives up unwinds every role to the common exit,
// which frees TMEM and records a status code.
#pragma once

#include "gguf_decode.cuh"
#include "ptx.cuh"

namespace tgo {

enum : int { kFwd = 0, kBwd = 1 };

constexpr int kTileM = 128;          // weight-side extent of one tile (TMEM lanes)
constexpr int kTileTok = 256;        // most tokens per accumulator (TMEM columns of one accumulator)
constexpr int kWideTok = 2 * kTileTok;   // most tokens of a wide tile (both accumulators at once)
constexpr int kStepK = 64;           // reduction elements per pipeline step (one swizzle row)
constexpr int kWgtTileBytes = kTileM * 128;
// Ring depths, in slots of one step (the barriers are per stage).  One CTA: 4 activation slots of
// 32 KB, up to 3 decoded-weight slots of 16 KB.  CTA pair: each CTA stages only its half of the
// tokens (16 KB per slot), which buys deeper rings from the same shared memory; measured on the
// grouped benchmark, six activation slots (a TMA round trip is ~1500-2000 cycles) and five
// decoded-weight slots beat 5/6, 7/4 and 4/7.
#ifndef TGO_ACT_STAGES
#define TGO_ACT_STAGES 4
#endif
#ifndef TGO_WGT_STAGES_MAX
#define TGO_WGT_STAGES_MAX 3
#endif
#ifndef TGO_PAIR_ACT_SLOTS
#define TGO_PAIR_ACT_SLOTS 6
#endif
#ifndef TGO_PAIR_WGT_SLOTS_MAX
#define TGO_PAIR_WGT_SLOTS_MAX 5
#endif
// 64-element steps per pipeline stage ("super-step").  The UMMA issuer pays one barrier wait and
// one commit per stage whatever its size, and every tcgen05 instruction costs that thread some
// 50-70 cycles, so with short UMMAs (few tokens) a stage of one step makes the issuer the limit.
#ifndef TGO_SUBSTEPS
#define TGO_SUBSTEPS 1
#endif
#ifndef TGO_PAIR_SUBSTEPS
#define TGO_PAIR_SUBSTEPS 2
#endif
#ifndef TGO_PAIR_RAW_STAGES_FWD
#define TGO_PAIR_RAW_STAGES_FWD 2
#endif
#ifndef TGO_PAIR_RAW_STAGES_BWD
#define TGO_PAIR_RAW_STAGES_BWD 4
#endif
// Sixteen decode warps in groups that take alternate steps.  Block types whose blocks start 16-byte
// aligned (Q4_K, Q5_K): four groups of four warps, a thread decodes the 64 weights of one row and
// step, which share their quant bytes and scales (one pass over the raw bytes; half the
// shared-memory loads).  The other types: two groups of eight warps, 32 weights per thread.
constexpr int kDecodeWarpsAll = 16;
constexpr int kFirstDecodeWarp = 4;
constexpr int kFirstEpilogueWarp = kFirstDecodeWarp + kDecodeWarpsAll;  // multiple of 4
#ifndef TGO_EPILOGUE_WARPS
#define TGO_EPILOGUE_WARPS 4
#endif
constexpr int kEpilogueWarps = TGO_EPILOGUE_WARPS;   // 4 or 8: one or two per TMEM lane quarter (two take alternate 16-token chunks)
static_assert(kEpilogueWarps == 4 || kEpilogueWarps == 8, "epilogue warps");
constexpr int kGemmThreads = (kFirstEpilogueWarp + kEpilogueWarps) * 32;
constexpr int kTmemCols = 512;       // two accumulators of 256 columns
constexpr int kNumBoxes = 5;         // activation TMA boxes of 256, 128, 64, 32, 16 rows
constexpr int kSmemLimit = 232448;   // 227 KB opt-in limit per CTA
constexpr int kEpiStageBytes = kEpilogueWarps * 16 * 64;  // per epilogue warp: 16 tokens x 32 outputs, bf16

struct ActMaps {
    CUtensorMap box[kNumBoxes];
};

// Packed weights as 2-D byte tensors for TMA.  Rows of 110 / 210 / 82-byte blocks start on 2-byte
// boundaries only, but the alignment of row g repeats with period P = 16 / gcd(row_bytes, 16)
// (at most 8): rows g = r (mod P) are mutually 16-byte aligned.  Map r therefore describes the
// rows of class r with row pitch P * row_bytes, based at the 16-byte boundary below row r, so a
// tile of 128 (or 64) weight rows is fetched with P box loads of rows / P rows each.
constexpr int kMaxWgtClasses = 8;
struct WgtMaps {
    CUtensorMap cls[kMaxWgtClasses];
};

struct GemmArgs {
    ActMaps act_maps[2];                 // per set: activations [rows][red] bf16, 128B swizzle
    WgtMaps wgt_maps[2];                 // per set: packed weight rows by alignment class
    const __nv_bfloat16* act[2];         // same tensors, for the non-TMA loader
    __nv_bfloat16* out[2];
    const int4* tasks;                   // (expert, first row, tokens <= 512, group) or null for dense
    const int* task_count;               // device count of tasks (grouped)
    int* status;                         // device status word (0 = ok)
    const uint64_t* iq2s_grid;           // IQ2_S codebook (1024 entries) in global memory
    int rows;                            // R
    int out_features;                    // N
    int in_features;                     // K
    int nsets;                           // 1, or 2 for the gate/up pair
    int dense_tasks;                     // dense: number of token tiles
    int dense_tok;                       // dense: tokens per tile (multiple of 16, at most 512)
    int use_tma;                         // 0: activation rows are not 16-byte multiples
    int wgt_classes;                     // P: alignment classes of the packed weight rows (1, 2, 4 or 8)
    int wgt_classes_log2;
    int wgt_row_bytes;                   // (K / 256) * block bytes
    // Split reduction (dense input gradient with few tiles and a long reduction): the out-features
    // are cut into nsplit ranges of split_steps 64-element steps, each tile reduces one range and
    // writes fp32 partial sums [split][row][k] to `partial`; a second kernel adds them in order.
    float* partial;                      // null: no split
    int nsplit;                          // 1: no split
    int split_steps;                     // steps per split (a multiple of the steps per stage)
    // Forward of one weight set with scattered output rows: out_rows[r] is where row r of the result
    // goes (any address this GPU can store to - its own memory or a peer's - 16-byte aligned, or null
    // to drop the row).  The epilogue then stores straight there, which lets an expert-parallel step
    // return every routed pair's row to the GPU that owns the token without a second pass.
    __nv_bfloat16* const* out_rows;      // null: rows are contiguous in out[set]
};

// CG = 1: one CTA per tile of 128 weight rows.  CG = 2: a cluster of two CTAs works on 256 weight
// rows and one token tile with cta_group::2 UMMAs (each CTA decodes its own 128 rows and stages
// half of the tokens; the leader CTA issues).
template <int QT, int MODE, int CG, int WIDE = 1>
struct GemmCfg {
    using Fmt = BlockFmt<QT>;
    static constexpr int kSub = CG == 2 ? TGO_PAIR_SUBSTEPS : TGO_SUBSTEPS;   // steps per stage
    static constexpr int kDecodeWarps = Fmt::kAligned ? 4 : 8;               // warps of one decode group (one step)
    static constexpr int kDecodeGroups = kDecodeWarpsAll / kDecodeWarps;
    static_assert(kDecodeGroups % kSub == 0 && 4 % kDecodeGroups == 0, "steps per stage / per block against decode groups");
    static constexpr int kActRows = kTileTok / CG;              // token rows staged by one CTA
    static constexpr int kActTileBytes = kActRows * 128;        // one step of activations
    static constexpr int kActSlots = CG == 2 ? TGO_PAIR_ACT_SLOTS : TGO_ACT_STAGES;          // steps of activations in flight
    static constexpr int kWgtSlotsMax = CG == 2 ? TGO_PAIR_WGT_SLOTS_MAX : TGO_WGT_STAGES_MAX;   // decoded steps in flight
    // full / done barrier pairs.  A barrier is reused every kBars pipeline stages; whoever waits
    // for stage q does so before stage q + kBars can complete, and whoever arrives for stage p
    // knows that stage p - kBars has completed.  The longest such distances occur in wide tiles
    // (a decoded slot is refilled up to 5 pipeline stages after its last reader, and the decode
    // warps arrive for two consecutive stages), which is why there are 8 and not 4.
    static constexpr int kBars = WIDE ? 8 : 4;
    static constexpr int kTokPad = CG == 2 ? 32 : 16;           // token padding of a tile (UMMA N granularity)
    static constexpr int kRawRows = MODE == kFwd ? 128 : 64;    // block windows per raw stage
    // pair: as many raw stages as fit in 60 KB (the raw ring has to cover an HBM round trip).
    // Backward, a raw stage is one step and the two decode groups take alternate steps: the ring
    // depth must be even, so that a stage always goes to the same group.  With an odd depth a group
    // could reach a stage one phase ahead of its barrier - before the other group's earlier load
    // into that stage has landed, when loads complete out of order - and a wait on a barrier that
    // is a whole phase behind passes at once.
    static constexpr int kRawFit = 61440 / (kRawRows * Fmt::kBox);
    static constexpr int kRawMaxPair = MODE == kFwd ? TGO_PAIR_RAW_STAGES_FWD : TGO_PAIR_RAW_STAGES_BWD;
    static constexpr int kRawWanted = kRawFit >= kRawMaxPair ? kRawMaxPair : (kRawFit < 2 ? 2 : kRawFit);
    static constexpr int kRawStages = CG == 2 ? (MODE == kBwd ? kRawWanted / kDecodeGroups * kDecodeGroups : kRawWanted)
                                              : (MODE == kFwd ? 2 : 4);
    static_assert(kRawStages >= 2 && kRawStages % 2 == 0, "raw ring: two producers take alternate stages");
    static_assert(MODE == kFwd || kRawStages % kDecodeGroups == 0, "backward raw ring depth must be a multiple of the decode groups");
    static constexpr int kRawStageBytes = kRawRows * Fmt::kBox;
    static constexpr int kRawBytes = kRawStages * kRawStageBytes;
    static constexpr int kGridBytes = QT == QT_IQ2_S ? 8192 : 0;
    static constexpr int kFixed = 1024 /*alignment slack*/ + 512 /*barriers etc.*/ + 128 /*read slack*/ + kEpiStageBytes +
                                  kActSlots * kActTileBytes + kRawBytes + kGridBytes;
    static constexpr int kWgtSlotsFit = (kSmemLimit - kFixed) / kWgtTileBytes;
    static constexpr int kWgtSlots = kWgtSlotsFit >= kWgtSlotsMax ? kWgtSlotsMax : kWgtSlotsFit;
    static_assert(kWgtSlots > kSub && kActSlots > kSub, "shared memory budget: more than one stage must fit");
    // a barrier is reused every kBars stages: nobody may still wait on its previous phase then
    static_assert((kWgtSlots + kSub - 1) / kSub <= kBars && (kActSlots + kSub - 1) / kSub <= kBars, "ring deeper than the barriers");
    // wide tiles: a decode group arrives for two pipeline stages per decoded stage, knowing only
    // that the last reader of the slot's previous step is done, up to 2 * ceil(slots / steps per
    // stage) - 1 pipeline stages back; the barrier it arrives on must not still be in the phase of
    // a stage older than that
    static_assert(!WIDE || 2 * ((kWgtSlots + kSub - 1) / kSub) <= kBars, "decoded-weight ring too deep for the barrier ring with wide tiles");
    static constexpr int kSmemBytes = kFixed + kWgtSlots * kWgtTileBytes;
};

struct TileInfo {
    int expert, row0, ntok, set, m0;
    int split;   // backward with a split reduction: which range of the out-features
    int nhalf;   // 1, or 2 for a wide tile (more than kTileTok tokens)
    int tok0;    // tokens of half 0; half 1 holds the other ntok - tok0
};

template <int CG>
__device__ __forceinline__ int pad_tokens(int n) {
    constexpr int kPad = CG == 2 ? 32 : 16;   // UMMA N granularity
    return (n + kPad - 1) & ~(kPad - 1);
}
__device__ __forceinline__ int half_tokens(const TileInfo& t, int half) { return half == 0 ? t.tok0 : t.ntok - t.tok0; }
__device__ __forceinline__ int half_row0(const TileInfo& t, int half) { return half == 0 ? t.row0 : t.row0 + t.tok0; }

// `mtiles` / `mtiles_set` count tiles of CG * 128 weight rows; `rank` is the CTA's rank in its pair.
template <int MODE, int CG, int WIDE, int SPLIT>
__device__ __forceinline__ bool load_tile(const GemmArgs& a, int tile, int mtiles, int mtiles_set,
                                          int rank, TileInfo& t) {
    const int task = tile / mtiles;
    const int mt = tile - task * mtiles;
    if (a.tasks != nullptr) {
        const int4 k = a.tasks[task];
        t.expert = k.x;
        t.row0 = k.y;
        t.ntok = min(k.z, WIDE ? kWideTok : kTileTok);
    } else {
        t.expert = 0;
        t.row0 = task * a.dense_tok;
        t.ntok = min(a.dense_tok, a.rows - t.row0);
    }
    if (WIDE && t.ntok > kTileTok) {
        t.nhalf = 2;
        t.tok0 = pad_tokens<CG>((t.ntok + 1) >> 1);
    } else {
        t.nhalf = 1;
        t.tok0 = t.ntok;
    }
    if (MODE == kFwd) {
        t.split = 0;
        t.set = mt / mtiles_set;
        t.m0 = ((mt - t.set * mtiles_set) * CG + rank) * kTileM;
    } else {
        t.set = 0;
        t.split = SPLIT ? mt / mtiles_set : 0;          // which range of a split reduction
        t.m0 = ((mt - t.split * mtiles_set) * CG + rank) * kTileM;
    }
    return t.ntok > 0;
}

// A role's walk over the tiles of its CTA (pair).  AHEAD: the task record of the next tile is
// requested one tile ahead - the record is a dependent global load of several hundred cycles, which
// the role would otherwise pay at each tile boundary.  Used by the decode and epilogue warps
// backward, where a tile has only eight steps (measured: dX +1-2 %; forward -0.6 %, so not there).
template <int MODE, int CG, int WIDE, int SPLIT, bool AHEAD>
struct TileWalk {
    long long tile, total;
    int ncta, mtiles, mtiles_set, rank;
    int4 rec;       // record of `tile`
    int task, mt;   // tile = task * mtiles + mt
    __device__ __forceinline__ void fetch(const GemmArgs& a) {
        task = static_cast<int>(tile) / mtiles;
        mt = static_cast<int>(tile) - task * mtiles;
        if (a.tasks != nullptr) {
            rec = a.tasks[task];
        } else {
            const int row0 = task * a.dense_tok;
            rec = make_int4(0, row0, min(a.dense_tok, a.rows - row0), 0);
        }
    }
    __device__ __forceinline__ TileWalk(const GemmArgs& a, int cta, int ncta_, long long total_, int mtiles_,
                                        int mtiles_set_, int rank_)
        : tile(cta), total(total_), ncta(ncta_), mtiles(mtiles_), mtiles_set(mtiles_set_), rank(rank_) {
        rec = make_int4(0, 0, 0, 0);
        task = mt = 0;
        if (AHEAD && tile < total) fetch(a);
    }
    // the next tile that has tokens; false when the walk is over
    __device__ __forceinline__ bool next(const GemmArgs& a, TileInfo& t) {
        while (tile < total) {
            if (!AHEAD) fetch(a);
            const int4 k = rec;
            const int cur_mt = mt;
            tile += ncta;
            if (AHEAD && tile < total) fetch(a);
            t.expert = k.x;
            t.row0 = k.y;
            t.ntok = min(k.z, WIDE ? kWideTok : kTileTok);
            if (WIDE && t.ntok > kTileTok) {
                t.nhalf = 2;
                t.tok0 = pad_tokens<CG>((t.ntok + 1) >> 1);
            } else {
                t.nhalf = 1;
                t.tok0 = t.ntok;
            }
            if (MODE == kFwd) {
                t.split = 0;
                t.set = cur_mt / mtiles_set;
                t.m0 = ((cur_mt - t.set * mtiles_set) * CG + rank) * kTileM;
            } else {
                t.set = 0;
                t.split = SPLIT ? cur_mt / mtiles_set : 0;
                t.m0 = ((cur_mt - t.split * mtiles_set) * CG + rank) * kTileM;
            }
            if (t.ntok > 0) return true;
        }
        return false;
    }
};

// One lane waits, the whole warp learns the outcome (keeps the warp converged).
__device__ __forceinline__ bool lane0_wait(uint32_t bar, uint32_t parity, volatile int* abort_word,
                                           int code, int lane) {
    int ok = 1;
    if (lane == 0) ok = mbar_wait(bar, parity, abort_word, code) ? 1 : 0;
    return __shfl_sync(0xFFFFFFFFu, ok, 0) != 0;
}
// Every lane waits (each needs the acquire), the warp agrees on the outcome.  The common case -
// the phase has already completed - costs one try_wait and one vote.
__device__ __forceinline__ bool all_wait(uint32_t bar, uint32_t parity, volatile int* abort_word,
                                         int code) {
    bool ok = mbar_try_wait(bar, parity);
    if (__all_sync(0xFFFFFFFFu, ok)) return true;
    if (!ok) ok = mbar_wait(bar, parity, abort_word, code);
    return __all_sync(0xFFFFFFFFu, ok) != 0;
}

// WIDE = 0: every tile has at most 256 tokens and one accumulator (the wide-tile paths compile
// out); WIDE = 1: tiles of up to 512 tokens.  SPLIT = 1 (backward, narrow tiles only): the
// reduction is cut into ranges with fp32 partial sums; compiled out otherwise (measured: carrying
// the split arithmetic in the ordinary backward kernel cost it 4 %).
template <int QT, int MODE, int CG, int WIDE, int SPLIT>
__global__ void __launch_bounds__(kGemmThreads, 1)
mmq_gemm_kernel(const __grid_constant__ GemmArgs args) {
    using Cfg = GemmCfg<QT, MODE, CG, WIDE>;
    using Fmt = BlockFmt<QT>;
    // NAS / NBS: decoded-weight and activation slots (one step each); NB: stage barriers
    constexpr int NAS = Cfg::kWgtSlots, NBS = Cfg::kActSlots, NB = Cfg::kBars, NR = Cfg::kRawStages;
    constexpr int kActTileBytes = Cfg::kActTileBytes, KS = Cfg::kSub;
    constexpr int kDecodeWarps = Cfg::kDecodeWarps, kDecodeGroups = Cfg::kDecodeGroups;
    constexpr bool k64 = kDecodeWarps == 4;   // a decode thread takes 64 weights (one row of a step)
    // CTA pair: rank 0 (the leader) owns the barriers both CTAs feed (full, acc_empty) and issues
    // the UMMAs; every CTA owns the barriers only it waits on (done, raw, acc_full).
    const int rank = CG == 2 ? static_cast<int>(cluster_ctarank()) : 0;
    const int cta = CG == 2 ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int ncta = CG == 2 ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

    extern __shared__ uint8_t smem_dyn[];
    const uint32_t smem_base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    uint8_t* smem = smem_dyn + (smem_base - smem_u32(smem_dyn));

    // carve-up (all operand tiles 1024-byte aligned)
    const uint32_t act_s = smem_base;
    const uint32_t wgt_s = act_s + NBS * kActTileBytes;
    const uint32_t raw_s = wgt_s + NAS * kWgtTileBytes;
    const uint32_t grid_s = raw_s + Cfg::kRawBytes + 128;
    const uint32_t epi_s = grid_s + Cfg::kGridBytes;
    const uint32_t misc_s = epi_s + kEpiStageBytes;
    uint8_t* act_g = smem;
    uint8_t* grid_g = smem + (grid_s - smem_base);
    uint8_t* epi_g = smem + (epi_s - smem_base);
    uint8_t* misc_g = smem + (misc_s - smem_base);
    // barriers (8 bytes each)
    const uint32_t bar_full = misc_s;                        // NB
    const uint32_t bar_done = bar_full + 8 * NB;             // NB
    const uint32_t bar_raw_full = bar_done + 8 * NB;         // NR
    const uint32_t bar_raw_empty = bar_raw_full + 8 * NR;    // NR
    const uint32_t bar_acc_full = bar_raw_empty + 8 * NR;    // 2
    const uint32_t bar_acc_empty = bar_acc_full + 16;        // 2
    constexpr int kBarBytes = 8 * (2 * NB + 2 * NR + 4);
    static_assert(kBarBytes + 16 <= 512, "misc region");
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc_g + kBarBytes);
    volatile int* abort_word = reinterpret_cast<volatile int*>(misc_g + kBarBytes + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int N = args.out_features, K = args.in_features;
    const int nkb = K >> 8;
    // tile space
    const int mtiles_set = MODE == kFwd ? (N + CG * kTileM - 1) / (CG * kTileM) : K / (CG * kTileM);
    static_assert(!SPLIT || (MODE == kBwd && !WIDE), "the split reduction exists for the narrow backward kernel only");
    const int nsplit = SPLIT ? args.nsplit : 1;
    const int mtiles = MODE == kFwd ? mtiles_set * args.nsets : mtiles_set * nsplit;
    const int steps_set = MODE == kFwd ? K / kStepK : (N + kStepK - 1) / kStepK;
    // 64-element steps of a tile: the whole reduction (both weight sets of a pair backward), or one
    // range of it when the reduction is split
    const int nsteps = MODE == kFwd ? steps_set : (nsplit > 1 ? args.split_steps : steps_set * args.nsets);
    const int steps_all = MODE == kFwd ? steps_set : steps_set * args.nsets;   // steps that hold data
    const int nstages = (nsteps + KS - 1) / KS;                              // decoded stages of a tile
    const int nsteps_pad = nstages * KS;   // a stage's missing steps are fed zeros
    const int ntasks = args.tasks != nullptr ? *args.task_count : args.dense_tasks;
    const long long total_tiles = static_cast<long long>(ntasks) * mtiles;

    if (threadIdx.x == 0) {
        // full: the leader's activation producer (with the byte count of both halves) - or both
        // producers when they copy with plain loads - and the decode warps of every CTA
        for (int i = 0; i < NB; ++i) {
            mbar_init(bar_full + 8 * i, (args.use_tma ? 1 : CG) + CG * kDecodeWarps * KS);
            mbar_init(bar_done + 8 * i, 1);
        }
        for (int i = 0; i < NR; ++i) {
            mbar_init(bar_raw_full + 8 * i, 1);
            mbar_init(bar_raw_empty + 8 * i, MODE == kFwd ? kDecodeWarps * kDecodeGroups : kDecodeWarps);
        }
        for (int i = 0; i < 2; ++i) { mbar_init(bar_acc_full + 8 * i, 1); mbar_init(bar_acc_empty + 8 * i, kEpilogueWarps * CG); }
        *abort_word = 0;
        mbar_fence_init();
    }
    if (QT == QT_IQ2_S) {
        uint64_t* gdst = reinterpret_cast<uint64_t*>(grid_g);
        for (int i = threadIdx.x; i < 1024; i += kGemmThreads) gdst[i] = args.iq2s_grid[i];
    }
    if (warp == 1) {
        if (CG == 2) {
            tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(smem_u32(tmem_slot), kTmemCols);
            tmem_relinquish();
        }
    }
    tc_fence_before_sync();
    if (CG == 2) cluster_sync_all(); else __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // barriers of the leader, as seen from this CTA
    const uint32_t lead_full = CG == 2 ? map_to_cta(bar_full, 0) : bar_full;
    const uint32_t lead_acc_empty = CG == 2 ? map_to_cta(bar_acc_empty, 0) : bar_acc_empty;

    // Warp roles.  Backward: warps 0 / 2 / 3 are the activation and the two raw-weight producers,
    // 4-19 decode.  Forward: the three single-thread roles whose serial instruction streams set the
    // pace there (UMMA issuer 1, activation producer 5, raw producers 9 and 13) share scheduler
    // partition 1 with one decode warp and one epilogue warp, so that they compete for issue slots
    // with two busy warps instead of five; the other partitions take five decode warps each.
    // Measured on the benchmark (Q4_K, 256 ragged groups): forward +3 %; backward, whose short
    // tiles keep the epilogue warps busy, loses with that placement and keeps the plain one.
    constexpr bool kRemap = MODE == kFwd;
    constexpr int kActWarp = kRemap ? 5 : 0, kRawWarp = kRemap ? 9 : 2, kRawWarp2 = kRemap ? 13 : 3;
    const bool light = kRemap ? ((warp & 3) == 1 && warp < 16) : warp < kFirstDecodeWarp;
    // decode warp index 0..15
    const int dwarp = kRemap ? warp - ((warp > 1) + (warp > 5) + (warp > 9) + (warp > 13)) : warp - kFirstDecodeWarp;
    if (warp == kActWarp) {
        // ------------------------------------------------------------ activation producer
        // One pipeline stage = KS one-step slots of the tokens of one half.  `it` is the running
        // pipeline-stage index; stage it uses slots it * KS .. it * KS + KS - 1 (mod NBS).
        if (args.use_tma) {
            if (lane == 0) {
                for (int s = 0; s < args.nsets; ++s)
                    for (int b = 0; b < kNumBoxes; ++b) prefetch_tmap(&args.act_maps[s].box[b]);
                // This thread's loop is one of the serial chains that set the pace, so everything
                // it needs per stage is a running value: the stage's barrier, the barrier of the
                // stage whose slots it refills (D stages back), the ring slot, and the position in
                // the reduction.  The token rows of a half are fetched with the boxes whose heights
                // are the binary digits of the row count (a multiple of 16).
                constexpr uint32_t D = NBS / KS;            // stage it refills the last slot of stage it - D
                uint32_t it = 0;                            // running pipeline stage
                uint32_t full_off = 0;                      // 8 * (it % NB)
                uint32_t wait_off = 0, wait_ph = 0;         // barrier and phase of stage it - D
                uint32_t slot = 0;                          // (it * KS) % NBS
                bool ok = true;
                for (long long tile = cta; ok && tile < total_tiles; tile += ncta) {
                    TileInfo t;
                    if (!load_tile<MODE, CG, WIDE, SPLIT>(args, static_cast<int>(tile), mtiles, mtiles_set, rank, t)) continue;
                    int rem_h[2], row_h[2];
#pragma unroll
                    for (int h = 0; h < (WIDE ? 2 : 1); ++h) {
                        rem_h[h] = pad_tokens<CG>(half_tokens(t, h)) / CG;
                        row_h[h] = half_row0(t, h) + rank * rem_h[h];
                    }
                    // position of the tile's next decoded stage in the reduction
                    int step = 0;
                    int astep = SPLIT ? t.split * nsteps : 0;
                    int set = 0, red0 = MODE == kFwd ? 0 : astep * kStepK;
                    if (MODE == kBwd && SPLIT) {
                        set = astep / steps_set;
                        red0 = (astep - set * steps_set) * kStepK;
                    }
                    const int npipe = nstages * t.nhalf;
                    for (int ps = 0; ps < npipe; ++ps, ++it) {
                        const int half = (WIDE && t.nhalf == 2) ? ps & 1 : 0;
                        const bool last_half = !(WIDE && t.nhalf == 2) || half == 1;
                        const int rem = rem_h[WIDE ? half : 0], row0 = row_h[WIDE ? half : 0];
                        if (it >= D) {
                            if (!mbar_wait(bar_done + wait_off, wait_ph, abort_word, kAbortActEmpty)) { ok = false; break; }
                            wait_off += 8;
                            if (wait_off == 8 * NB) { wait_off = 0; wait_ph ^= 1u; }
                        }
                        // the leader announces the bytes of the whole stage; each CTA copies its share
                        // of the token rows (all of them, or its half) and the bytes count on the
                        // leader's barrier
                        const uint32_t bar = lead_full + full_off;
                        if (rank == 0) mbar_arrive_expect_tx(bar_full + full_off, static_cast<uint32_t>(rem * CG) * 128u * KS);
                        int s_step = step, s_astep = astep, s_set = set, s_red = red0;
#pragma unroll
                        for (int ks = 0; ks < KS; ++ks) {
                            // a step past the end reads columns outside the matrix: TMA fills zeros
                            const bool past = s_step >= nsteps || s_astep >= steps_all;
                            const int use_set = past ? 0 : s_set;
                            const int col = past ? (steps_set + 1) * kStepK : s_red;
                            const uint32_t dst = act_s + slot * kActTileBytes;
#pragma unroll
                            for (int b = 0; b < kNumBoxes; ++b) {
                                constexpr int kAll = 2 * Cfg::kActRows - 1;
                                const int h = 256 >> b;
                                if (h <= Cfg::kActRows && (rem & h) != 0) {
                                    const int off = rem & (kAll & ~(2 * h - 1));   // rows taken by the taller boxes
                                    if (CG == 2) tma_load_2d_pair(dst + off * 128, &args.act_maps[use_set].box[b], bar, col, row0 + off);
                                    else tma_load_2d(dst + off * 128, &args.act_maps[use_set].box[b], bar, col, row0 + off);
                                }
                            }
                            if (++slot == NBS) slot = 0;
                            ++s_step;
                            ++s_astep;
                            s_red += kStepK;
                            if (MODE == kBwd && s_red >= steps_set * kStepK) { s_red = 0; ++s_set; }
                        }
                        if (last_half) { step = s_step; astep = s_astep; set = s_set; red0 = s_red; }
                        full_off += 8;
                        if (full_off == 8 * NB) full_off = 0;
                    }
                }
            }
        } else {
            // Rows whose byte length is not a multiple of 16 cannot be described to TMA: copy
            // with plain loads, zero-filling past the matrix edge, into the same swizzled image.
            uint32_t it = 0;
            bool ok = true;
            const int red_total = MODE == kFwd ? K : N;
            for (long long tile = cta; ok && tile < total_tiles; tile += ncta) {
                TileInfo t;
                if (!load_tile<MODE, CG, WIDE, SPLIT>(args, static_cast<int>(tile), mtiles, mtiles_set, rank, t)) continue;
                const int npipe = nstages * t.nhalf;
                for (int ps = 0; ps < npipe; ++ps, ++it) {
                    const int stage = t.nhalf == 2 ? ps >> 1 : ps;
                    const int half = t.nhalf == 2 ? ps & 1 : 0;
                    const int my_rows = pad_tokens<CG>(half_tokens(t, half)) / CG;
                    const long long first_row = static_cast<long long>(half_row0(t, half)) + rank * my_rows;
                    const uint32_t s = it % NB;
                    const uint32_t last = it * KS + (KS - 1);
                    if (last >= static_cast<uint32_t>(NBS)) {
                        const uint32_t jw = (last - NBS) / KS;
                        if (!lane0_wait(bar_done + 8 * (jw % NB), (jw / NB) & 1u, abort_word, kAbortActEmpty, lane)) { ok = false; break; }
                    }
                    for (int ks = 0; ks < KS; ++ks) {
                        const int step = stage * KS + ks;
                        const int astep = SPLIT ? t.split * nsteps + step : step;
                        int set = MODE == kFwd ? 0 : astep / steps_set;
                        int red0 = (MODE == kFwd ? step : astep - set * steps_set) * kStepK;
                        if (step >= nsteps || astep >= steps_all) { set = 0; red0 = red_total; }   // a step past the end: zeros
                        const __nv_bfloat16* src = args.act[set];
                        uint8_t* dst = act_g + ((it * KS + ks) % NBS) * kActTileBytes;
                        for (int idx = lane; idx < my_rows * 8; idx += 32) {
                            const int r = idx >> 3, c = idx & 7;
                            const long long grow = first_row + r;
                            alignas(16) __nv_bfloat16 v[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                const int col = red0 + c * 8 + e;
                                v[e] = (grow < args.rows && col < red_total) ? src[grow * red_total + col]
                                                                             : __float2bfloat16(0.0f);
                            }
                            *reinterpret_cast<uint4*>(dst + r * 128 + ((c ^ (r & 7)) << 4)) =
                                *reinterpret_cast<const uint4*>(v);
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (CG == 2) mbar_arrive_cluster(lead_full + 8 * s); else mbar_arrive(bar_full + 8 * s);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ UMMA issuer (one thread)
        // This thread's instruction stream is the serial spine of the kernel: per pipeline stage it
        // waits once, issues 4 * KS UMMAs and commits once (twice for a pair); every one of these
        // costs it 50-70 cycles whatever the UMMA's size.  The loop keeps stage counters, barrier
        // addresses and the low descriptor words as running values (one add per use), and the
        // narrow kernel's loop body carries nothing of the wide tiles (measured: 4 % of the
        // forward time).
        if (lane == 0 && rank == 0) {
            constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);   // SBO 1024, version, SWIZZLE_128B
            constexpr uint32_t kLboA = MODE == kFwd ? 16u : 8192u;                 // forward K-major, backward MN-major
            constexpr uint32_t kStepA = (MODE == kFwd ? 32u : 2048u) >> 4;         // next 16 reduction elements of A
            constexpr uint32_t kStepB = 32u >> 4;
            // descriptors hold the address inside the CTA's shared memory (the same in both CTAs of a pair)
            const uint32_t a_lo0 = ((wgt_s & 0x3FFFFu) >> 4) | ((kLboA >> 4) << 16);
            const uint32_t b_lo0 = ((act_s & 0x3FFFFu) >> 4) | ((16u >> 4) << 16);
            // the peer's copies of the barriers the commits signal
            const uint32_t peer_done = CG == 2 ? map_to_cta(bar_done, 1) : 0u;
            const uint32_t peer_acc_full = CG == 2 ? map_to_cta(bar_acc_full, 1) : 0u;
            uint32_t sa = 0, sb = 0, sbar = 0, ph = 0;   // next decoded-weight slot, activation slot, barrier pair
            uint32_t full_bar = bar_full, done_bar = bar_done;
            uint32_t tl = 0;   // running accumulator use (a wide tile takes two)
            bool ok = true, ready = false;
            for (long long tile = cta; ok && tile < total_tiles; tile += ncta) {
                TileInfo t;
                if (!load_tile<MODE, CG, WIDE, SPLIT>(args, static_cast<int>(tile), mtiles, mtiles_set, rank, t)) continue;
                const uint32_t acc0 = tl & 1u, acc1 = acc0 ^ 1u;
                if (!mbar_wait(bar_acc_empty + 8 * acc0, ((tl >> 1) & 1u) ^ 1u, abort_word, kAbortAccEmpty)) break;
                tc_fence_after_sync();
                const uint32_t d_tmem0 = tmem_base + acc0 * kTileTok;
                const uint32_t idesc0 = umma_idesc_bf16(static_cast<uint32_t>(pad_tokens<CG>(t.tok0)), MODE == kBwd ? 1u : 0u, 0u, 128u * CG);
                // second half of a wide tile: the other accumulator, its own token count
                const uint32_t d_tmem1 = tmem_base + acc1 * kTileTok;
                const uint32_t idesc1 = WIDE ? umma_idesc_bf16(static_cast<uint32_t>(pad_tokens<CG>(t.ntok - t.tok0)), MODE == kBwd ? 1u : 0u, 0u, 128u * CG) : 0u;
                const int nhalf = WIDE ? t.nhalf : 1;
                for (int stage = 0; ok && stage < nstages; ++stage) {
                    for (int half = 0; half < nhalf; ++half) {
                        if (WIDE && half == 1 && stage == 0) {   // first use of the second accumulator
                            if (!mbar_wait(bar_acc_empty + 8 * acc1, (((tl + 1u) >> 1) & 1u) ^ 1u, abort_word, kAbortAccEmpty)) { ok = false; break; }
                            tc_fence_after_sync();
                        }
                        const uint32_t d_tmem = (WIDE && half == 1) ? d_tmem1 : d_tmem0;
                        const uint32_t idesc = (WIDE && half == 1) ? idesc1 : idesc0;
                        if (!ready && !mbar_wait(full_bar, ph, abort_word, kAbortWgtFull)) { ok = false; break; }
                        const uint32_t cur_done = done_bar;
                        uint32_t slot_a[KS], slot_b[KS];
                        uint32_t sa_next = sa;
#pragma unroll
                        for (int ks = 0; ks < KS; ++ks) {
                            slot_a[ks] = a_lo0 + sa_next * (kWgtTileBytes >> 4);
                            slot_b[ks] = b_lo0 + sb * (kActTileBytes >> 4);
                            if (++sa_next == NAS) sa_next = 0;
                            if (++sb == NBS) sb = 0;
                        }
                        // the decoded steps stay in place until the last half has read them
                        if (half == nhalf - 1) sa = sa_next;
                        full_bar += 8;
                        done_bar += 8;
                        if (++sbar == NB) { sbar = 0; full_bar = bar_full; done_bar = bar_done; ph ^= 1u; }
                        // with short stages, test the next stage's barrier now: the answer arrives while
                        // the UMMAs issue; "no" only means "ask again, blocking"
                        ready = KS == 1 ? mbar_try_wait(full_bar, ph) : false;
#pragma unroll
                        for (uint32_t ks = 0; ks < static_cast<uint32_t>(KS); ++ks) {
                            const uint32_t sa_lo = slot_a[ks], sb_lo = slot_b[ks];
#pragma unroll
                            for (uint32_t kk = 0; kk < kStepK / 16; ++kk) {
                                const uint32_t accum = (ks | kk) != 0 ? 1u : (stage != 0 ? 1u : 0u);
                                if (CG == 2) umma_bf16_lohi_pair(d_tmem, sa_lo + kk * kStepA, sb_lo + kk * kStepB, kDescHi, idesc, accum);
                                else umma_bf16_lohi(d_tmem, sa_lo + kk * kStepA, sb_lo + kk * kStepB, kDescHi, idesc, accum);
                            }
                        }
                        if (CG == 2) {
                            umma_commit_pair(cur_done);
                            umma_commit_pair(peer_done + (cur_done - bar_done));
                        } else {
                            umma_commit(cur_done);
                        }
                    }
                }
                if (ok) {
                    // the accumulators are complete once everything issued so far has finished
                    for (int half = 0; half < nhalf; ++half) {
                        const uint32_t acc = half == 0 ? acc0 : acc1;
                        if (CG == 2) {
                            umma_commit_pair(bar_acc_full + 8 * acc);
                            umma_commit_pair(peer_acc_full + 8 * acc);
                        } else {
                            umma_commit(bar_acc_full + 8 * acc);
                        }
                    }
                }
                tl += static_cast<uint32_t>(nhalf);
            }
        }
    } else if (warp == kRawWarp || warp == kRawWarp2) {
        // ------------------------------------------------------------ raw weight producer
        // One box load per alignment class and stage: rows / P block windows of kBox bytes each.
        // Two producer threads (in different warps) take alternate raw stages: one thread needs
        // some 900 cycles per stage (a wait, an expect_tx, the copies, each a shared-memory or TMA
        // round trip under load), which backward - one raw stage per 64-element step - set the pace.
        const uint32_t my_parity = warp == kRawWarp ? 0u : 1u;
        if (lane == 0) {
            uint32_t itr = 0;
            bool ok = true;
            const int P = args.wgt_classes, lgP = args.wgt_classes_log2;
            constexpr int kRows = Cfg::kRawRows;
            for (int s = 0; s < args.nsets; ++s)
                for (int c = 0; c < P; ++c) prefetch_tmap(&args.wgt_maps[s].cls[c]);
            // Everything that does not change from one raw stage to the next is worked out once
            // per tile: this thread's loop is one of the serial chains that set the pace backward
            // (one raw stage per 64-element step).  Per alignment class c: the box's byte column x
            // (backward: fixed for the tile; forward: advances by one block per stage) and the row
            // index inside map c of the tile's first weight row.  A step is 64 rows and P divides
            // 64, so the class of a row and the rows' order inside a stage never change.
            const uint32_t tx_bytes = static_cast<uint32_t>(kRows) * Fmt::kBox;
            const int rows_per_class = kRows >> lgP;
            for (long long tile = cta; ok && tile < total_tiles; tile += ncta) {
                TileInfo t;
                if (!load_tile<MODE, CG, WIDE, SPLIT>(args, static_cast<int>(tile), mtiles, mtiles_set, rank, t)) continue;
                const int nraw = MODE == kFwd ? nkb : nsteps_pad;
                const long long gbase = static_cast<long long>(t.expert) * N + (MODE == kFwd ? t.m0 : 0);
                int y0[kMaxWgtClasses], x0[kMaxWgtClasses];
#pragma unroll
                for (int c = 0; c < kMaxWgtClasses; ++c) {
                    if (c < P) {
                        const long long first = gbase + ((c - gbase) & (P - 1));   // first row of class c at or after the base
                        y0[c] = static_cast<int>((first - c) >> lgP);
                        const int mis_c = (c * args.wgt_row_bytes) & 15;
                        x0[c] = mis_c + (MODE == kFwd ? 0 : (t.m0 >> 8) * Fmt::kBytes);
                    }
                }
                // backward: running position in the reduction (weight set, first out-feature of the step)
                int set = MODE == kFwd ? t.set : 0, n_first = 0;
                if (SPLIT) {
                    const int astep0 = t.split * nsteps;
                    set = astep0 / steps_set;
                    n_first = (astep0 - set * steps_set) * kStepK;
                }
                int astep = SPLIT ? t.split * nsteps : 0;
                for (int ri = 0; ri < nraw; ++ri, ++itr) {
                    if ((itr & 1u) != my_parity) {   // the other producer's stage
                        if (MODE == kBwd) {
                            ++astep;
                            n_first += kStepK;
                            if (n_first >= steps_set * kStepK) { n_first = 0; ++set; }
                        }
                        continue;
                    }
                    const uint32_t r = itr % NR, ph = (itr / NR) & 1u;
                    if (!mbar_wait(bar_raw_empty + 8 * r, ph ^ 1u, abort_word, kAbortRawEmpty)) { ok = false; break; }
                    int use_set = set, yoff = 0, xoff = 0;
                    if (MODE == kFwd) {
                        xoff = ri * Fmt::kBytes;
                    } else {
                        yoff = n_first >> lgP;
                        if (ri >= nsteps || astep >= steps_all) { use_set = 0; yoff = 0; }   // a step past the end: decoded as zeros
                    }
                    const uint32_t bar = bar_raw_full + 8 * r;
                    mbar_arrive_expect_tx(bar, tx_bytes);
                    const uint32_t stage_s = raw_s + r * Cfg::kRawStageBytes;
#pragma unroll
                    for (int c = 0; c < kMaxWgtClasses; ++c) {
                        if (c < P)
                            tma_load_2d(stage_s + c * rows_per_class * Fmt::kBox, &args.wgt_maps[use_set].cls[c], bar,
                                        (x0[c] + xoff) & ~15, y0[c] + yoff);
                    }
                    if (MODE == kBwd) {
                        ++astep;
                        n_first += kStepK;
                        if (n_first >= steps_set * kStepK) { n_first = 0; ++set; }
                    }
                }
            }
        }
    } else if (!light && warp < kFirstEpilogueWarp) {
        // ------------------------------------------------------------ decode warps
        // Group g decodes the steps whose running index is g (mod kDecodeGroups).  Forward: one raw
        // stage (a super-block column of 128 rows) serves four steps, shared out over the groups; a thread
        // keeps its row and 32-weight half for the whole tile.  Backward: one raw stage (64 rows)
        // per step; a thread keeps its row slot and 32-weight group.
        const int group = dwarp / kDecodeWarps;
        const int dt = (dwarp % kDecodeWarps) * 32 + lane;  // 0 .. 32 * kDecodeWarps - 1
        // Forward: 128 rows x 2 halves, (row, half) = (dt / 2, dt % 2).  Backward: 64 rows x 4
        // quarters.  For the 16-byte-aligned block types (128-bit loads) (row, quarter) =
        // (dt % 64, dt / 64): a quarter-warp, which shares one 128-bit store wavefront, then holds
        // eight different rows of the same quarter, whose swizzled chunks cover all banks; with the
        // quarter in the low bits two of every four lanes meet on the same banks (the two
        // 64-column halves of the image are 8 KB apart).  The other types read their blocks as
        // 32-bit words, many of them common to the four quarters of a row: there (dt / 4, dt % 4)
        // keeps those loads broadcasts and the eight rows of a warp on different banks.
        // 64 weights per thread (aligned types): forward 128 rows, thread = row; backward 64 rows x
        // the two 64-column halves of the CTA's 128 in-features, (row, half) = (dt % 64, dt / 64).
        // Either way a quarter-warp holds eight consecutive rows, whose raw blocks (128-bit loads)
        // and swizzled chunks (128-bit stores) cover all banks.
        constexpr bool kRowMajorLanes = MODE == kBwd && Fmt::kAligned;
        const int row = k64 ? (MODE == kFwd ? dt : dt & 63)
                            : (MODE == kFwd ? dt >> 1 : (kRowMajorLanes ? dt & 63 : dt >> 2));   // weight row inside the raw stage
        const int sub = k64 ? (MODE == kFwd ? 0 : 2 * (dt >> 6))
                            : (MODE == kFwd ? dt & 1 : (kRowMajorLanes ? dt >> 6 : dt & 3));     // first 32-weight group of the step's span
        // byte offsets of this thread's 16-byte chunks inside a decoded tile (128B swizzle)
        constexpr int kChunks = k64 ? 8 : 4;
        uint32_t coff[kChunks];
        {
            const uint32_t base = (MODE == kFwd ? 0u : static_cast<uint32_t>(sub >> 1) * 8192u) + row * 128u;
            const int cbase = 4 * (sub & 1);
#pragma unroll
            for (int c = 0; c < kChunks; ++c) coff[c] = base + (((cbase + c) ^ (row & 7)) << 4);
        }
        const int P = args.wgt_classes, lgP = args.wgt_classes_log2;
        // Running state of this group.  A decoded step is read by pipeline stage `stg` (and by
        // stg + 1 in a wide tile); its slot is free again once the last reader of the step that
        // held it before (NAS steps earlier) has finished, stage `jw`.  Both advance by a fixed
        // amount per step inside a tile, so they are kept as running values; only a tile's first
        // steps, whose slot was last used by an earlier tile, look the stage up.
        uint32_t it = static_cast<uint32_t>(group);                       // running index of this group's next step
        uint32_t slot_off = static_cast<uint32_t>(group % NAS) * kWgtTileBytes;   // (it % NAS) * slot bytes
        uint32_t raw_it = 0;   // forward: raw stages consumed
        // running decoded-step and pipeline-stage indices at the start of this tile, whether it is
        // wide, and how many pipeline stages per decoded stage the previous tile had (1 or 2)
        uint32_t d0 = 0, p0 = 0;
        bool wide = false;
        uint32_t prev_per = 1;
        uint32_t stg = 0, stg_inc = 0;
        int jw = 0;
        bool ok = true;
        constexpr uint32_t kSlotWrap = NAS * kWgtTileBytes;
        constexpr int kAdv = kDecodeGroups / KS;   // decoded stages a group advances per step it decodes

        // last pipeline stage that reads the decoded step with running index `o` (this tile or an earlier one)
        auto last_reader = [&](uint32_t o) -> uint32_t {
            if (o >= d0) { const uint32_t ds = (o - d0) / KS; return wide ? p0 + 2u * ds + 1u : p0 + ds; }
            // k steps before this tile: inside the previous tile (all tiles have nsteps_pad steps) its
            // decoded stage counts back from that tile's end, which is p0; older steps were read
            // before the previous tile began
            const uint32_t k = d0 - o;
            if (k <= static_cast<uint32_t>(nsteps_pad)) return p0 - 1u - prev_per * ((k + KS - 1) / KS - 1u);
            return p0 - static_cast<uint32_t>(nstages) * prev_per - 1u;
        };

        // waits until this step's decoded-weight slot is free, decodes into it and signals the step
        auto emit = [&](uint32_t blk, int g, bool valid, uint32_t raw_bar_to_release) -> bool {
            // Decode first, into registers: the arithmetic does not need the destination slot, so
            // it overlaps the wait for that slot, and what follows the wait (four stores, a fence,
            // an arrival) is short.  The slot's credit loop - the latency that sets the stage time -
            // no longer contains the decode.
            uint4 o[4];
            Pending32 rest;   // 64 weights per thread: the last 32 stay byte-sized quants until the first 32 are stored
            if constexpr (k64) {
                if (valid) {
                    decode64<QT>(blk, g >> 1, o, rest);
                } else {
                    o[0] = o[1] = o[2] = o[3] = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                    for (int i = 0; i < 8; ++i) rest.v[i] = 0u;
                    rest.ds = 0.0f;
                    rest.dm = 0.0f;
                }
            } else {
                if (valid) {
                    decode32<QT>(blk, g, grid_s, o);
                } else {
                    o[0] = o[1] = o[2] = o[3] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            if (raw_bar_to_release != 0) {   // the raw blocks are in registers now: hand the raw stage back early
                __syncwarp();
                if (lane == 0) mbar_arrive(raw_bar_to_release);
            }
            // Without wide tiles every pipeline stage is KS consecutive steps, so the stages and the
            // slot follow from the step index alone; with them they are the running values above.
            const uint32_t stg_now = WIDE ? stg : it / KS;
            if (it >= static_cast<uint32_t>(NAS)) {
                uint32_t j;
                if (WIDE) j = (it - d0 >= static_cast<uint32_t>(NAS)) ? static_cast<uint32_t>(jw) : last_reader(it - NAS);
                else j = (it - NAS) / KS;
                if (!all_wait(bar_done + 8 * (j % NB), (j / NB) & 1u, abort_word, kAbortWgtEmpty)) return false;
            }
            const uint32_t tile_s = wgt_s + (WIDE ? slot_off : (it % NAS) * kWgtTileBytes);
#pragma unroll
            for (int c = 0; c < 4; ++c) sts128(tile_s + coff[c], o[c]);
            if constexpr (k64) {
                finish32(rest, o);
#pragma unroll
                for (int c = 0; c < 4; ++c) sts128(tile_s + coff[4 + c], o[c]);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                if (CG == 2) mbar_arrive_cluster(lead_full + 8 * (stg_now % NB)); else mbar_arrive(bar_full + 8 * (stg_now % NB));
                if (WIDE && wide) {   // the second half reads this step in the next pipeline stage
                    if (CG == 2) mbar_arrive_cluster(lead_full + 8 * ((stg_now + 1u) % NB)); else mbar_arrive(bar_full + 8 * ((stg_now + 1u) % NB));
                }
            }
            it += kDecodeGroups;
            if (WIDE) {
                slot_off += (kDecodeGroups % NAS) * kWgtTileBytes;
                if (slot_off >= kSlotWrap) slot_off -= kSlotWrap;
                stg += stg_inc;
                jw += static_cast<int>(stg_inc);
            }
            return true;
        };

        TileWalk<MODE, CG, WIDE, SPLIT, MODE == kBwd> walk(args, cta, ncta, total_tiles, mtiles, mtiles_set, rank);
        TileInfo t;
        while (ok && walk.next(args, t)) {
            wide = t.nhalf == 2;
            if (WIDE) {
                // this group's first step of the tile (running index parity equals the group)
                const int first = static_cast<int>(it - d0);
                const int per_stage = wide ? 2 : 1;          // pipeline stages per decoded stage
                stg_inc = static_cast<uint32_t>(per_stage * kAdv);
                stg = p0 + static_cast<uint32_t>(per_stage * (first / KS));
                // floor((first - NAS) / KS): negative until the slot's previous step lies in this tile
                const int ds_old = KS == 2 ? ((first - NAS) >> 1) : (first - NAS);
                jw = static_cast<int>(p0) + per_stage * ds_old + (per_stage - 1);
            }
            const long long gexp = static_cast<long long>(t.expert) * N;
            if (MODE == kFwd) {
                const bool row_ok = t.m0 + row < N;
                int slot = row, cls = 0;
                if (!Fmt::kAligned) {
                    cls = static_cast<int>((gexp + t.m0 + row) & (P - 1));
                    slot = cls * (Cfg::kRawRows >> lgP) + (row >> lgP);
                }
                const uint32_t blk0 = raw_s + slot * Fmt::kBox;
                const int mis0 = Fmt::kAligned ? 0 : (cls * args.wgt_row_bytes) & 15;
                for (int kb = 0; kb < nkb && ok; ++kb, ++raw_it) {
                    const uint32_t r = raw_it % NR, rph = (raw_it / NR) & 1u;
                    if (!all_wait(bar_raw_full + 8 * r, rph, abort_word, kAbortRawFull)) { ok = false; break; }
                    const uint32_t blk = blk0 + r * Cfg::kRawStageBytes + (Fmt::kAligned ? 0 : (mis0 + kb * Fmt::kBytes) & 15);
                    constexpr int kPerBlock = 4 / kDecodeGroups;   // steps of a block column that one group decodes
#pragma unroll
                    for (int u = 0; u < kPerBlock; ++u) {
                        if (!emit(blk, 2 * (group + kDecodeGroups * u) + sub, row_ok, u == kPerBlock - 1 ? bar_raw_empty + 8 * r : 0u)) { ok = false; break; }
                    }
                }
            } else {
                const int g = ((t.m0 >> 7) & 1) * 4 + sub;
                const int kb = t.m0 >> 8;
                // The alignment class of a weight row repeats every P rows and a step is 64 rows,
                // so a thread's window slot and misalignment are the same in every step of a tile.
                int slot = row, mis = 0;
                if (!Fmt::kAligned) {
                    const int cls = static_cast<int>((gexp + row) & (P - 1));
                    slot = cls * (Cfg::kRawRows >> lgP) + (row >> lgP);
                    mis = (((cls * args.wgt_row_bytes) & 15) + kb * Fmt::kBytes) & 15;
                }
                const uint32_t blk0 = raw_s + slot * Fmt::kBox + mis;
                for (int step = static_cast<int>((it - d0) & 0x7FFFFFFFu); step < nsteps_pad; step += kDecodeGroups) {
                    const uint32_t ri = d0 + step;
                    const uint32_t r = ri % NR, rph = (ri / NR) & 1u;
                    if (!all_wait(bar_raw_full + 8 * r, rph, abort_word, kAbortRawFull)) { ok = false; break; }
                    const int astep = SPLIT ? t.split * nsteps + step : step;
                    const int n_first = (astep >= steps_set ? astep - steps_set : astep) * kStepK;
                    const bool valid = step < nsteps && astep < steps_all && n_first + row < N;
                    if (!emit(blk0 + r * Cfg::kRawStageBytes, g, valid, bar_raw_empty + 8 * r)) { ok = false; break; }
                }
            }
            d0 += static_cast<uint32_t>(nsteps_pad);
            if (WIDE) {
                prev_per = wide ? 2u : 1u;
                p0 += static_cast<uint32_t>(nstages * t.nhalf);
            }
        }
    } else if (warp >= kFirstEpilogueWarp) {
        // ------------------------------------------------------------ epilogue
        const int quad = warp & 3;                              // TMEM lanes 32 * quad .. + 31
        const int ehalf = (warp - kFirstEpilogueWarp) >> 2;     // which of the alternate 16-token chunks
        const int mdim = MODE == kFwd ? N : K;
        // drains accumulator use `u` (rows row0 .. row0 + ntok of the output) and hands it back
        auto drain = [&](uint32_t u, int m0, int set, int row0, int ntok, int split) -> bool {
            const uint32_t acc = u & 1u, aph = (u >> 1) & 1u;
            const int ntok_pad = pad_tokens<CG>(ntok);
            if (!all_wait(bar_acc_full + 8 * acc, aph, abort_word, kAbortAccFull)) return false;
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + acc * kTileTok + (static_cast<uint32_t>(quad * 32) << 16);
            const int mq = m0 + quad * 32;  // first output column of this warp
            __nv_bfloat16* out_base = args.out[MODE == kFwd ? set : 0] + static_cast<long long>(row0) * mdim;
            const bool scatter = MODE == kFwd && args.out_rows != nullptr;
            if (SPLIT && args.partial != nullptr) {
                // split reduction: fp32 partial sums, lane = output column (128 bytes per warp store)
                const int m = mq + lane;
                float* part = args.partial + (static_cast<long long>(split) * args.rows + row0) * mdim + m;
                for (int c0 = 16 * ehalf; c0 < ntok_pad; c0 += 4 * kEpilogueWarps) {
                    uint32_t v[16];
                    tmem_ld16(taddr + c0, v);
                    tmem_ld_wait();
                    if (m < mdim) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c0 + j < ntok) part[static_cast<long long>(c0 + j) * mdim] = __uint_as_float(v[j]);
                    }
                }
            } else if (MODE == kFwd && scatter) {
                // Scattered rows (tgo_grouped_fwd_rows): every result row has its own destination,
                // possibly in a peer GPU's memory.  A loop of its own, so that the ordinary epilogue
                // below carries none of it.  Same staging tile as the transposing path; where the
                // warp's 32 outputs do not all exist (last tile of weight rows) or rows are not
                // 16-byte multiples, element-wise stores.
                const bool vec_ok = (mdim & 7) == 0 && mq + 32 <= mdim;
                uint8_t* stage = epi_g + (warp - kFirstEpilogueWarp) * (16 * 64);
                const int wchunk = lane >> 2, wword = (lane & 3) << 2;
                const int p = lane >> 2, part = lane & 3;
                const uint8_t* rd0 = stage + p * 128 + (((2 * part) ^ (p & 1)) << 4);
                const uint8_t* rd1 = stage + p * 128 + (((2 * part + 1) ^ (p & 1)) << 4);
                for (int c0 = 16 * ehalf; c0 < ntok_pad; c0 += 4 * kEpilogueWarps) {
                    uint32_t v[16];
                    tmem_ld16(taddr + c0, v);
                    tmem_ld_wait();
                    if (vec_ok) {
                        __nv_bfloat16* const* rp = args.out_rows + row0 + c0 + 2 * p;
                        __nv_bfloat16* dst0 = c0 + 2 * p < ntok ? rp[0] : nullptr;
                        __nv_bfloat16* dst1 = c0 + 2 * p + 1 < ntok ? rp[1] : nullptr;
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            *reinterpret_cast<uint32_t*>(stage + q * 128 + (((wchunk ^ (q & 1)) << 4) | wword)) =
                                pack_bf16(__uint_as_float(v[2 * q]), __uint_as_float(v[2 * q + 1]));
                        __syncwarp();
                        const uint4 a = *reinterpret_cast<const uint4*>(rd0);
                        const uint4 b = *reinterpret_cast<const uint4*>(rd1);
                        if (dst0 != nullptr)
                            *reinterpret_cast<uint4*>(dst0 + mq + part * 8) =
                                make_uint4(__byte_perm(a.x, a.y, 0x5410), __byte_perm(a.z, a.w, 0x5410),
                                           __byte_perm(b.x, b.y, 0x5410), __byte_perm(b.z, b.w, 0x5410));
                        if (dst1 != nullptr)
                            *reinterpret_cast<uint4*>(dst1 + mq + part * 8) =
                                make_uint4(__byte_perm(a.x, a.y, 0x7632), __byte_perm(a.z, a.w, 0x7632),
                                           __byte_perm(b.x, b.y, 0x7632), __byte_perm(b.z, b.w, 0x7632));
                        __syncwarp();
                    } else if (mq + lane < mdim) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (c0 + j < ntok) {
                                __nv_bfloat16* row = args.out_rows[row0 + c0 + j];
                                if (row != nullptr) row[mq + lane] = __float2bfloat16(__uint_as_float(v[j]));
                            }
                        }
                    }
                }
            } else if ((mdim & 7) == 0 && mq + 32 <= mdim) {
                // Transposing path: the warp's 32 outputs x 16 tokens go through a private staging
                // tile so that global stores are 16 bytes per lane.  The tile holds token pairs:
                // row p = tokens 2p, 2p + 1, one 4-byte word per output (one conversion and one
                // conflict-free store per two accumulator values); the 16-byte chunks of a row are
                // XOR-swizzled with the row's parity so that the 128-bit reads of two rows at a
                // time are conflict-free as well.  A lane then unzips 8 outputs of both tokens.
                uint8_t* stage = epi_g + (warp - kFirstEpilogueWarp) * (16 * 64);
                const int wchunk = lane >> 2, wword = (lane & 3) << 2;
                const int p = lane >> 2, part = lane & 3;
                const uint8_t* rd0 = stage + p * 128 + (((2 * part) ^ (p & 1)) << 4);
                const uint8_t* rd1 = stage + p * 128 + (((2 * part + 1) ^ (p & 1)) << 4);
                for (int c0 = 16 * ehalf; c0 < ntok_pad; c0 += 4 * kEpilogueWarps) {
                    uint32_t v[16];
                    tmem_ld16(taddr + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        *reinterpret_cast<uint32_t*>(stage + q * 128 + (((wchunk ^ (q & 1)) << 4) | wword)) =
                            pack_bf16(__uint_as_float(v[2 * q]), __uint_as_float(v[2 * q + 1]));
                    __syncwarp();
                    const uint4 a = *reinterpret_cast<const uint4*>(rd0);
                    const uint4 b = *reinterpret_cast<const uint4*>(rd1);
                    __nv_bfloat16* dst = out_base + static_cast<long long>(c0 + 2 * p) * mdim + mq + part * 8;
                    if (c0 + 2 * p < ntok)
                        *reinterpret_cast<uint4*>(dst) = make_uint4(__byte_perm(a.x, a.y, 0x5410), __byte_perm(a.z, a.w, 0x5410),
                                                                    __byte_perm(b.x, b.y, 0x5410), __byte_perm(b.z, b.w, 0x5410));
                    if (c0 + 2 * p + 1 < ntok)
                        *reinterpret_cast<uint4*>(dst + mdim) = make_uint4(__byte_perm(a.x, a.y, 0x7632), __byte_perm(a.z, a.w, 0x7632),
                                                                           __byte_perm(b.x, b.y, 0x7632), __byte_perm(b.z, b.w, 0x7632));
                    __syncwarp();
                }
            } else {
                const int m = mq + lane;
                const bool m_ok = m < mdim;
                __nv_bfloat16* out = out_base + m;
                for (int c0 = 16 * ehalf; c0 < ntok_pad; c0 += 4 * kEpilogueWarps) {
                    uint32_t v[16];
                    tmem_ld16(taddr + c0, v);
                    tmem_ld_wait();
                    if (m_ok) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (c0 + j < ntok)
                                out[static_cast<long long>(c0 + j) * mdim] = __float2bfloat16(__uint_as_float(v[j]));
                        }
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (CG == 2) mbar_arrive_cluster(lead_acc_empty + 8 * acc); else mbar_arrive(bar_acc_empty + 8 * acc);
            }
            return true;
        };
        uint32_t tl = 0;
        TileWalk<MODE, CG, WIDE, SPLIT, MODE == kBwd> walk(args, cta, ncta, total_tiles, mtiles, mtiles_set, rank);
        TileInfo t;
        while (walk.next(args, t)) {
            if (!drain(tl, t.m0, t.set, t.row0, t.tok0, t.split)) break;
            ++tl;
            if (WIDE && t.nhalf == 2) {   // the second half of a wide tile is an accumulator of its own
                if (!drain(tl, t.m0, t.set, t.row0 + t.tok0, t.ntok - t.tok0, t.split)) break;
                ++tl;
            }
        }
    }

    // ------------------------------------------------------------ common exit
    __syncwarp();
    if (*abort_word != 0) {
        // Some wait gave up.  Give copies and UMMAs still in flight a bounded time to land before
        // shared memory and TMEM are released.
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    tc_fence_before_sync();
    // pair: neither CTA may leave (or free its TMEM) while the other can still signal its barriers
    // or have UMMAs reading its shared memory
    if (CG == 2) cluster_sync_all(); else __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        if (CG == 2) tmem_dealloc_pair(tmem_base, kTmemCols); else tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_word != 0 && args.status != nullptr)
        atomicCAS(args.status, 0, (*abort_word) | (static_cast<int>(blockIdx.x) << 8));
}

}  // namespace tgo
