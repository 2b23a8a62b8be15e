// The FP8 x NVFP4 GEMM kernel for sm_100a: dense (optionally with deterministic K splits) and grouped by expert
// (contiguous / masked / indexed routing), per-token or [1,128] activation scales.
//
// Orientation: weights are the UMMA A operand (M = 128 channels per instruction), tokens the B operand (N = token
// tile BM); the FP32 accumulator D^T[channel, token] lives in tensor memory (lanes = channels, columns = tokens).
// The bridged FP8 weights never touch shared memory: the bridge warps write them into tensor memory (tcgen05.st, a
// thread per channel row) and the MMA reads its A operand from there, so shared-memory bandwidth -- the unit this
// kernel saturates first -- carries only the raw NVFP4 codes and the activation tile.
//
// One persistent CTA per SM:
//   warps 0-3 (0-7)  epilogue  tcgen05.ld -> scale -> BF16 -> global (or tagged FP32 partials + ordered split-K reduction)
//   next 8 or 16     bridge    prepared NVFP4 codes + scales (shared) -> FP8 E4M3 A tiles (tensor memory)
//   next warp        weights   bulk / TMA copies of codes and scales into the weight ring (may start before the previous
//                              kernel on the stream has finished, see GemmParams::static_weights)
//   next warp        tokens    TMA tile loads of the activations into the token ring; per-row cp.async gather for indexed
//                              routing without a gather pass
//   last warp        MMA       one elected thread issues tcgen05.mma kind::f8f6f4 and the commits; owns the TMEM
//
// Three rings, one per hand-over, so that no stage waits for a consumer it does not need:
//   weight ring   {codes 8 KB + scales 1 KB} in shared memory: weight producer -> bridge teams (who release it)
//   bridged ring  {128 lanes x 32 columns of tensor memory = one 128 x 128 FP8 A tile}: bridge teams -> MMA (commit)
//   token ring    {activations BM x 128 B, 128-byte swizzled} in shared memory: activation producer -> MMA (commit)
// The depths of the weight and bridged rings are multiples of the number of bridge teams (the host sees to it), so
// that a stage always meets the same team: the mbarrier parity waits are only sound for a waiter that looks at every
// phase of its barrier.
// The remaining tensor-memory columns hold the accumulator sets, so the epilogue of one unit overlaps the main loop of
// the next.  Weights run ahead of the tokens: with static weights under programmatic dependent launch the weight
// producer and the bridge teams of a dense launch fill their rings while the previous kernel is still running.
// Every wait is bounded (tb_ptx.cuh); a wait that runs out makes the whole CTA unwind and the kernel writes a code to
// `status`.
#pragma once

#include <cuda_bf16.h>

#include "tb_bridge.cuh"

namespace tb {

constexpr int kMaxEpilogueWarps = 8;
constexpr int kMaxExperts = 1024;
constexpr int kMaxRawStages = 16;
constexpr int kMaxBridgedStages = 8;
constexpr int kTileCols = 32;  // tensor-memory columns of one bridged FP8 tile: 128 K values, four per column
constexpr int kTmemCols = 512;
constexpr int kMaxAccSets = 8;
constexpr int kEpochCells = 1024;  // 32-bit words at the head of the split-K workspace: [0] launch sequence, [1] CTAs arrived
constexpr int kBalancedFlag0 = 16;  // balanced launches: word kBalancedFlag0 + c is raised when CTA c has published its partial tile
constexpr int kMaxBalancedCtas = kEpochCells - kBalancedFlag0;
constexpr int kBalancedTileWords = 128 * 256;  // FP32 partial sums of one 128-channel x 256-token tile
constexpr int kMaxSharedParts = 4;  // CTAs that share one tile of the last round
constexpr int kMaxOutputPeers = 16;   // ranks whose buffers an epilogue can scatter to
constexpr int kMaxSplitTiles = 128;  // output tiles of a K-split launch: the tile index takes 7 bits of a tag
constexpr int kTransposeBytes = 16 * 32 * 2;  // an epilogue warp's 16-column chunk as BF16 [token][channel]
// Chunks of turned output an epilogue warp can park in shared memory.  The 256-token tile has one accumulator set, so
// its drain stands between two main loops: the warps move the accumulator out as fast as tensor memory gives it up --
// six of a warp's eight chunks into shared memory, two into registers as packed BF16 -- hand the accumulator back, and
// write the output while the next tile's main loop runs.  Smaller tiles have a second accumulator set instead.
__host__ __device__ constexpr int staged_chunks(int bm) { return bm == 256 ? 6 : 1; }
constexpr int kBarrierBytes = 832;     // 4 * 16 + 2 * 8 + 2 * 8 + 1 barriers of 8 bytes, padded

// Epilogue warps of a token tile: four cover the 128 tensor-memory lanes; from 64 tokens up a second set of four takes
// the other half of the columns (halves the accumulator registers per thread and the time to drain a tile).
__host__ __device__ constexpr int epilogue_warps(int bm) { return bm >= 64 ? 8 : 4; }
// Threads of a CTA: epilogue + bridge (8 or 16) + weight producer + activation producer + MMA warps.
__host__ __device__ constexpr int gemm_threads(int bm, int bridge_warps) { return (epilogue_warps(bm) + bridge_warps + 3) * 32; }

enum Layout : int { kDense = 0, kIndexed = 1, kContiguous = 2, kMasked = 3 };

// Wait-site codes written to status[0] (status[1] = block index) when a wait gives up.
enum WaitCode : int {
    kWaitWeightEmpty = 1, kWaitWeightFull = 2, kWaitBridgedEmpty = 3, kWaitTokenEmpty = 4, kWaitBridgedFull = 5, kWaitAccEmpty = 6,
    kWaitAccFull = 7, kWaitTokenFull = 8, kWaitSplit = 9
};

// Division of a non-negative int below 2^31 by an invariant positive divisor: one multiply-high and a shift, with the
// two constants worked out on the host.  The unit decode runs at the head of every role's serial instruction stream
// (a single thread issues one dependent instruction every few cycles), where five hardware-emulated divisions cost
// half a microsecond of a ten-microsecond launch.
struct FastDiv {
    uint32_t mul, shr, divisor, pad;
#ifndef __CUDACC_RTC__
    static FastDiv make(uint32_t d) {
        FastDiv f = {0, 0, d, 0};
        if (d > 1) {
            uint32_t log2_ceil = 0;
            while ((1ull << log2_ceil) < d) ++log2_ceil;
            const uint32_t bits = 31 + log2_ceil;
            f.mul = static_cast<uint32_t>(((1ull << bits) + d - 1) / d);
            f.shr = bits - 32;
        }
        return f;
    }
#endif
    __device__ __forceinline__ int div(int n) const {
        return divisor == 1 ? n : static_cast<int>(__umulhi(static_cast<uint32_t>(n), mul) >> shr);
    }
};

struct alignas(64) GemmParams {
    CUtensorMap map_a;   // activations uint8 [rows, k]: box 128 x BM, 128-byte swizzle (unused for indexed)
    CUtensorMap map_sf;  // scales uint8 [E * k_pad/16, n_pad]: box 128 x 8 (unused with group scales)
    const uint8_t* a;
    const float* a_scale;
    long long a_scale_stride_m, a_scale_stride_k;
    const uint8_t* weight;
    const uint8_t* scale;
    const float* global_scale;
    int* locks;
    float* workspace;  // split-K: kEpochCells header words (launch sequence, arrival count), then {value, tag} words
    __nv_bfloat16* d;
    long long rows;  // rows of `a`
    int n, k, n_pad, k_pad;
    int n_tiles, k_blocks;  // 128-channel tiles, 128-deep K blocks
    int layout, num_experts, top_k;
    int splits;    // dense: K splits (>= 1)
    // dense, 256-token tile: when shared_tiles > 0 every CTA runs whole_rounds whole tiles (tile = CTA + round x grid)
    // and then CTA c takes K blocks [j, j + 1) * k_blocks / shared_parts of left-over tile c / shared_parts,
    // j = c % shared_parts (CTAs from shared_tiles * shared_parts on are done).  The parts of a tile exchange FP32
    // partial sums through the workspace and each finishes a share of the tile's columns.
    int whole_rounds, shared_tiles, shared_parts;
    int a_gathered;  // indexed: `a` is already [padded routes, k] in sorted order (tb_gather_rows ran first)
    int static_weights;      // 1: no kernel in flight on the stream writes weight / scale: they may be read before
                             //    griddepcontrol.wait returns
    int m_blocks;  // dense: ceil(rows / BM)
    int w_stages, a_stages, bridged_stages;  // ring depths: weights, tokens (shared memory), bridged tiles (tensor memory)
    const long long* expert_offsets;
    const int* expert_counts;
    const int* sorted_ids;
    const int* expert_ids;
    const int* num_tokens_padded;
    long long sorted_capacity;
    int* status;
    // Grouped launches of an expert-parallel step: row r of `a` belongs to route row_target[r] & 0x3FFFFFF of rank
    // row_target[r] >> 26 (-1: nobody's), and its output row goes straight into that rank's buffer peer_out[rank] (plain
    // stores over NVLink, row stride n) instead of `d`.  Null for every other launch.
    const int* row_target;
    __nv_bfloat16* peer_out[kMaxOutputPeers];
    FastDiv div_splits, div_n_tiles;  // dense unit -> (tile, split); tile or token block -> (token block, channel tile)
    long long wait_cycles;  // budget of every bounded wait
    int only_split;         // test hook: s + 1 runs only the units of K split s (0 = all)
};

// One unit of work: one 128-channel tile x BM tokens over a K-block range.
struct Unit {
    int expert;
    int nt;          // 128-channel tile of the unit
    int row0;        // first row of `a` (contiguous / masked / dense) or first slot of sorted_ids (indexed)
    int rows_valid;  // rows of the tile that exist
    int kb0, kb1;    // K-block range
    int tile;        // dense tile index (slot of its partial sums in the split-K workspace)
    int split;
    int parts;       // shared tiles: number of CTAs that hold K-block ranges of this tile (0: the whole tile is this CTA's)
    int part;        // ... and which of them this CTA is
    bool skip;       // test hook (GemmParams::only_split): the unit is left out by every role
};

// Accumulator sets in tensor memory.  Per-token scales: two while they leave room for two bridged tiles (one set drains
// while the next tile accumulates; 192 tokens is the widest tile that can).  Group scales: every K block is its own accumulation that the epilogue must drain, so up to eight
// sets in three quarters of the columns keep the MMA from waiting on the drain latency.  The columns behind the
// accumulators hold the ring of bridged weight tiles.
__host__ __device__ constexpr int acc_sets(int bm, bool group_scales) {
    return group_scales ? (384 / bm > kMaxAccSets ? kMaxAccSets : 384 / bm) : (2 * bm + 2 * kTileCols <= kTmemCols ? 2 : 1);
}
__host__ __device__ constexpr int max_bridged_stages(int bm, bool group_scales) {
    return (kTmemCols - acc_sets(bm, group_scales) * bm) / kTileCols > kMaxBridgedStages
               ? kMaxBridgedStages : (kTmemCols - acc_sets(bm, group_scales) * bm) / kTileCols;
}

// Register shares with [1,128] activation scales on the 128-token tile: every epilogue lane keeps 64 FP32 totals live
// across the K loop, which does not fit the even share of the register file, while the bridge warps need little.  The
// two bridge warpgroups give registers back (setmaxnreg.dec) and the two epilogue warpgroups take them
// (setmaxnreg.inc).  inc waits until the pool holds enough, so the sum of the two targets must not exceed twice the
// kernel's own count: the host checks that count before it launches such an instance.
__host__ __device__ constexpr bool rebalances_registers(int bm, bool group_scales, int bridge_warps) {
    return (group_scales && bm == 128 && bridge_warps == 8) || (!group_scales && bm == 256 && bridge_warps == 16);
}
// The same on the 256-token tile with per-token scales: its epilogue warps hold part of the converted output in
// registers while they hand the accumulator back; sixteen bridge warps give eight registers each.
__host__ __device__ constexpr int rebalanced_bridge_regs(int bm) { return 64 + 0 * bm; }
__host__ __device__ constexpr int rebalanced_epilogue_regs(int bm) { return bm == 256 ? 88 : 128; }
// Registers per thread the kernel must have been built with for the pool to cover the epilogue's share.
__host__ __device__ constexpr int min_kernel_registers(int bm, bool group_scales, int bridge_warps) {
    return !rebalances_registers(bm, group_scales, bridge_warps) ? 0
           : (bridge_warps * rebalanced_bridge_regs(bm) + epilogue_warps(bm) * rebalanced_epilogue_regs(bm) +
              bridge_warps + epilogue_warps(bm) - 1) / (bridge_warps + epilogue_warps(bm));
}

template <int kValue> struct IntC { static constexpr int value = kValue; };

struct SmemLayout {
    uint32_t tokens, token_stage, weights, weight_stage, barriers, misc, ids, epi, transpose, group_scales, prefix, total;
};

// [1,128] activation scales are staged in shared memory for kScaleChunk K blocks at a time, per epilogue warp as
// [K block][token column of the warp], so that a K block costs the warp broadcast reads and no global load.
constexpr int kScaleChunk = 16;

__host__ __device__ inline SmemLayout smem_layout(int bm, int w_stages, int a_stages, int num_experts, bool group_scales = false) {
    SmemLayout l;
    l.tokens = 0;  // swizzled tiles first: every stage starts on a 1024-byte boundary
    l.token_stage = bm * 128;
    l.weights = a_stages * l.token_stage;
    l.weight_stage = kBlockBytes + kBlockScaleBytes;
    l.barriers = l.weights + w_stages * l.weight_stage;
    l.misc = l.barriers + kBarrierBytes;
    l.ids = l.misc + 64;
    l.epi = l.ids + 256 * 4;  // per epilogue warp: BM scales + BM output rows
    l.transpose = l.epi + 4 * bm * 8;  // per lane quadrant: bm scales + bm rows, split between its column groups
    l.group_scales = l.transpose + epilogue_warps(bm) * staged_chunks(bm) * kTransposeBytes;  // per warp: chunks of 16 tokens x 32 channels of BF16
    l.prefix = l.group_scales + (group_scales ? 4 * bm * kScaleChunk * 4 : 0);  // per lane quadrant: kScaleChunk x bm floats
    l.total = l.prefix + (num_experts > 0 ? (3 * num_experts + 4) * 4 : 0);
    return l;
}

#ifdef TB_TRACE
// Debug builds only.  Every block stamps the global nanosecond timer at 16 phases of its life into the words behind
// status[4 + 32768], and its producer, MMA and first bridge warp report the cycles they ran and waited (8 words per
// block behind status[4 + 40960]).
__device__ __forceinline__ uint32_t tb_clock() { uint32_t c; asm volatile("mov.u32 %0, %%clock;" : "=r"(c)); return c; }
__device__ __forceinline__ unsigned long long tb_globaltimer() {
    unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t;
}
#define TB_PHASE(idx) do { if (blockIdx.x < 256) \
    reinterpret_cast<unsigned long long*>(p.status + 4 + 32768)[blockIdx.x * 16 + (idx)] = tb_globaltimer(); } while (0)
#define TB_CLOCK() tb_clock()
#define TB_REPORT(slot, value) do { if (blockIdx.x < 256) p.status[4 + 40960 + blockIdx.x * 8 + (slot)] = static_cast<int>(value); } while (0)
#else
#define TB_PHASE(idx) do { } while (0)
#define TB_CLOCK() 0u
#define TB_REPORT(slot, value) do { } while (0)
#endif

// The whole kernel as a device function, so that a translation unit compiled at run time can wrap an instance of it in an
// entry point with a plain C name (see tensorbridge/jit/codegen.py); `p` must be the kernel's __grid_constant__ parameter
// itself (the tensor maps are handed to the TMA unit by their address in parameter space).
template <int BM, bool kExact, bool kGroupScales, int kBridgeWarps, int kBridgeGroups>
__device__ __forceinline__ void gemm_body(const GemmParams& p) {
    constexpr int kEpilogueWarps = epilogue_warps(BM);
    constexpr int kColumnGroups = kEpilogueWarps / 4;  // warp w drains lanes 32 * (w % 4) .. +31, columns of group w / 4
    constexpr int kCols = BM / kColumnGroups;          // token columns per epilogue warp
    static_assert(kCols % 16 == 0, "an epilogue warp drains whole 16-column chunks");
    constexpr int kWeightWarp = kEpilogueWarps + kBridgeWarps;
    constexpr int kActWarp = kWeightWarp + 1;
    constexpr int kMmaWarp = kActWarp + 1;
    // The bridge warps form kBridgeGroups teams.  Team g converts the K blocks g, g + kTurns, ...: the fixed latency
    // of one block's hand-over (waits, fences, arrive) overlaps the conversion of the next blocks by the other teams.
    // A team is a multiple of four warps because warp w reaches only tensor-memory lanes 32 * (w % 4) .. +31.
    constexpr int kGroupWarps = kBridgeWarps / kBridgeGroups;
    constexpr int kTeamThreads = kGroupWarps * 32;  // threads that share one 128 x 128 block
    constexpr int kTurns = kBridgeGroups;           // teams alternating over K blocks
    constexpr int kArrivals = kGroupWarps;          // bridge-warp arrivals per stage
    static_assert(kBridgeWarps == 8 || kBridgeWarps == 16, "8 or 16 bridge warps");
    static_assert(kGroupWarps == 4 || kGroupWarps == 8 || kGroupWarps == 16, "4, 8 or 16 warps per bridge team");
    static_assert(kEpilogueWarps % 4 == 0, "bridge warp w must sit on lane quadrant w % 4");
    constexpr int kAccSets = acc_sets(BM, kGroupScales);
    constexpr uint32_t kAccCols = kAccSets * BM;  // the bridged ring starts at this column
    static_assert(kAccCols + 2 * kTileCols <= kTmemCols, "no room for a bridged ring behind the accumulators");

    extern __shared__ uint8_t smem_unaligned[];
    // The swizzled tiles need 1024-byte alignment of their shared addresses.
    const uint32_t base_u32 = (smem_u32(smem_unaligned) + 1023u) & ~1023u;
    uint8_t* smem = smem_unaligned + (base_u32 - smem_u32(smem_unaligned));
    const SmemLayout L = smem_layout(BM, p.w_stages, p.a_stages, p.num_experts, kGroupScales);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int WS = p.w_stages, AS = p.a_stages, BS = p.bridged_stages;

    const uint32_t bar0 = base_u32 + L.barriers;
    auto w_full = [&](int s) { return bar0 + 8u * s; };
    auto w_empty = [&](int s) { return bar0 + 8u * (kMaxRawStages + s); };
    auto a_full = [&](int s) { return bar0 + 8u * (2 * kMaxRawStages + s); };
    auto a_empty = [&](int s) { return bar0 + 8u * (3 * kMaxRawStages + s); };
    auto br_full = [&](int s) { return bar0 + 8u * (4 * kMaxRawStages + s); };
    auto br_empty = [&](int s) { return bar0 + 8u * (4 * kMaxRawStages + kMaxBridgedStages + s); };
    auto acc_full = [&](int s) { return bar0 + 8u * (4 * kMaxRawStages + 2 * kMaxBridgedStages + s); };
    auto acc_empty = [&](int s) { return bar0 + 8u * (4 * kMaxRawStages + 2 * kMaxBridgedStages + kMaxAccSets + s); };
    const uint32_t drain_bar = bar0 + 8u * (4 * kMaxRawStages + 2 * kMaxBridgedStages + 2 * kMaxAccSets);

    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L.misc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.misc + 4);
    int* ids = reinterpret_cast<int*>(smem + L.ids);
    int* prefix = reinterpret_cast<int*>(smem + L.prefix);  // [E + 1] exclusive prefix of M blocks
    int* row_base = prefix + p.num_experts + 1;             // [E]
    int* row_count = row_base + p.num_experts;              // [E]

    const bool indexed = p.layout == kIndexed;
    const bool gather = indexed && p.a_gathered == 0;  // rows fetched one by one inside the kernel
    const bool routed = indexed || p.row_target != nullptr;  // output rows come from a table, not from the tile's position

    // ---- set-up (overlaps the previous kernel under PDL: no global reads yet) ----
    if (threadIdx.x == 0) TB_PHASE(0);
    if (warp == kWeightWarp) {
        if (lane == 0) {
            *abort_flag = 0;  // by the warp that does not wait at the set-up barrier, so that it never reads it unset
            prefetch_tensormap(&p.map_a);
            prefetch_tensormap(&p.map_sf);
        }
        // The weight ring's barriers (full, then empty), one per lane: all this warp needs before its first copy.
        static_assert(2 * kMaxRawStages <= 32, "one lane per barrier of the weight ring");
        if (lane < 2 * kMaxRawStages) mbar_init(bar0 + 8u * lane, lane < kMaxRawStages ? 1u : kArrivals);
        fence_barrier_init();
    } else if (warp == kActWarp) {
        // Every other barrier slot, used or not, one per lane and pass: arrival counts by slot range.
        constexpr int kSlots = 4 * kMaxRawStages + 2 * kMaxBridgedStages + 2 * kMaxAccSets + 1;
        for (int slot = 2 * kMaxRawStages + lane; slot < kSlots; slot += 32) {
            uint32_t count = 1u;  // a_empty, br_empty, acc_full, drain: one arrival (expect_tx or a commit)
            if (slot < 3 * kMaxRawStages) count = gather ? 32u : 1u;                                             // a_full
            else if (slot >= 4 * kMaxRawStages && slot < 4 * kMaxRawStages + kMaxBridgedStages) count = kArrivals;  // br_full
            else if (slot >= 4 * kMaxRawStages + 2 * kMaxBridgedStages + kMaxAccSets && slot < kSlots - 1) count = kEpilogueWarps;  // acc_empty
            mbar_init(bar0 + 8u * slot, count);
        }
        fence_barrier_init();
    }
    // Tensor-memory columns of this CTA: accumulators + bridged ring, rounded up to a power of two (at least 32).
    uint32_t tmem_cols = 32;
    while (tmem_cols < kAccCols + static_cast<uint32_t>(BS) * kTileCols) tmem_cols <<= 1;
    if (warp == kMmaWarp) {
        tmem_alloc(base_u32 + L.misc, tmem_cols);
        tmem_relinquish();
    }
    // The weight producer needs nothing of what the other warps set up (it made the barriers itself): it arrives at
    // the CTA barrier without waiting, so that its first copies are on their way while the tensor memory is still
    // being allocated.  (A barrier of its own: the one at the end of the kernel is the plain CTA barrier.)
    tc_fence_before_sync();
    if (warp == kWeightWarp) {
        asm volatile("barrier.arrive 2, %0;" ::"r"(static_cast<uint32_t>(blockDim.x)) : "memory");
    } else {
        asm volatile("barrier.sync 2, %0;" ::"r"(static_cast<uint32_t>(blockDim.x)) : "memory");
    }
    tc_fence_after_sync();
    const uint32_t tmem_base = warp == kWeightWarp ? 0u : *tmem_slot;

    // Let a kernel launched behind this one with programmatic dependent launch start its own set-up now: it waits for
    // this whole grid (griddepcontrol.wait) before it reads anything, so releasing it early costs nothing.
    if (threadIdx.x == 0) { TB_PHASE(1); pdl_launch_dependents(); }
    // Everything below may read memory the previous kernel on the stream wrote -- except, when the caller vouches that
    // no kernel still in flight writes the weights, the weight producer of a dense launch: it starts streaming at once.
    // ... and the bridge teams, which touch nothing but shared and tensor memory.  In a dense launch the MMA warp never
    // touches global memory either, and the activation producer waits right before its first load, after it has worked
    // out (and pulled into the instruction cache) everything the load needs.
    const bool dense = p.layout == kDense;
    const bool early = dense && ((p.static_weights != 0 && warp >= kEpilogueWarps && warp <= kWeightWarp) ||
                                 warp == kMmaWarp || (warp == kActWarp && !gather));
    if (!early) pdl_wait_prior_grid();
    if (threadIdx.x == 0) TB_PHASE(2);

    // ---- routing: per-expert row ranges and the prefix of their M blocks ----
    if (p.layout == kContiguous || p.layout == kMasked) {
        if (warp == 0) {
            const int E = p.num_experts;
            const int capacity = p.layout == kMasked ? static_cast<int>(p.rows / E) : 0;
            int carry = 0;
            for (int e0 = 0; e0 < E; e0 += 32) {
                const int e = e0 + lane;
                int base = 0, count = 0;
                if (e < E) {
                    if (p.layout == kContiguous) {
                        base = static_cast<int>(p.expert_offsets[e]);
                        count = static_cast<int>(p.expert_offsets[e + 1]) - base;
                    } else {
                        base = e * capacity;
                        count = min(p.expert_counts[e], capacity);
                    }
                    count = max(count, 0);
                    row_base[e] = base;
                    row_count[e] = count;
                }
                const int blocks = (count + BM - 1) / BM;
                int incl = blocks;
                for (int o = 1; o < 32; o <<= 1) {
                    const int v = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += v;
                }
                if (e < E) prefix[e] = carry + incl - blocks;
                carry += __shfl_sync(0xffffffffu, incl, 31);
            }
            if (lane == 0) prefix[E] = carry;
        }
        __syncthreads();
    }

    const int n_groups = p.n_tiles;  // units along the channel dimension
    int total_units;
    if (p.layout == kDense) {
        total_units = p.m_blocks * n_groups * p.splits;
    } else if (indexed) {
        long long padded = *p.num_tokens_padded;
        padded = padded < 0 ? 0 : (padded > p.sorted_capacity ? p.sorted_capacity : padded);
        total_units = static_cast<int>(padded / BM) * n_groups;
    } else {
        total_units = prefix[p.num_experts] * n_groups;
    }

    // Units of this CTA: every gridDim.x-th unit -- or, with shared tiles, an index into its whole rounds followed by
    // its part of a shared tile, if it has one.
    int u_begin = blockIdx.x, u_step = gridDim.x, u_end = total_units;
    if constexpr (kAccSets == 1) {
        if (p.shared_tiles > 0) {
            u_begin = 0;
            u_step = 1;
            u_end = p.whole_rounds + (static_cast<int>(blockIdx.x) < p.shared_tiles * p.shared_parts ? 1 : 0);
        }
    }

    auto decode = [&](int u) {
        Unit t;
        t.split = 0;
        t.parts = 0;
        t.part = 0;
        t.skip = false;
        t.kb0 = 0;
        t.kb1 = p.k_blocks;
        t.expert = 0;
        if (p.layout == kDense) {
            t.tile = p.div_splits.div(u);
            t.split = u - t.tile * p.splits;
            if constexpr (kAccSets == 1) {
                if (p.shared_tiles > 0) {
                    if (u < p.whole_rounds) {
                        t.tile = blockIdx.x + u * gridDim.x;
                    } else {
                        t.parts = p.shared_parts;
                        t.part = static_cast<int>(blockIdx.x) % p.shared_parts;
                        t.tile = p.whole_rounds * gridDim.x + static_cast<int>(blockIdx.x) / p.shared_parts;
                    }
                }
            }
            const int g = p.div_n_tiles.div(t.tile);
            t.nt = t.tile - g * n_groups;
            t.row0 = g * BM;
            t.rows_valid = min(BM, static_cast<int>(p.rows) - t.row0);
            // at most 16 splits of fewer than 2^27 blocks: the products stay below 2^31
            t.kb0 = p.div_splits.div(t.split * p.k_blocks);
            t.kb1 = p.div_splits.div((t.split + 1) * p.k_blocks);
            t.skip = p.only_split != 0 && t.split != p.only_split - 1;
            if (t.parts > 0) {
                t.kb0 = t.part * p.k_blocks / t.parts;
                t.kb1 = (t.part + 1) * p.k_blocks / t.parts;
            }
        } else {
            const int g = p.div_n_tiles.div(u);
            t.nt = u - g * n_groups;
            t.tile = u;
            if (indexed) {
                t.expert = p.expert_ids[g];
                t.row0 = g * BM;
                t.rows_valid = BM;
            } else {
                int lo = 0, hi = p.num_experts;  // last e with prefix[e] <= g
                while (hi - lo > 1) {
                    const int mid = (lo + hi) >> 1;
                    if (prefix[mid] <= g) lo = mid; else hi = mid;
                }
                t.expert = lo;
                const int mb = g - prefix[lo];
                t.row0 = row_base[lo] + mb * BM;
                t.rows_valid = min(BM, row_count[lo] - mb * BM);
            }
        }
        return t;
    };

    uint8_t* const weights0 = smem + L.weights;
    const uint32_t weights0_u32 = base_u32 + L.weights;
    const uint32_t tokens0_u32 = base_u32 + L.tokens;
    constexpr uint32_t kActBytes = BM * 128;
    constexpr uint32_t kWeightRawBytes = kBlockBytes + kBlockScaleBytes;  // codes, then scales

    if (warp == kWeightWarp) {
        // =========================== weight producer ===========================
        // One thread runs the whole loop: codes (one 8 KB bulk copy) and scales of every K block into the raw ring.
        bool ok = true;
        if (elect_one()) {
            TB_PHASE(13);
            uint32_t stage = weights0_u32, full = w_full(0), empty = w_empty(0);
            int rs = 0;
            uint32_t phase = 0;
            [[maybe_unused]] uint32_t waited = 0;
            [[maybe_unused]] const uint32_t loop_begin = TB_CLOCK();
            for (int u = u_begin; u < u_end && ok; u += u_step) {
                const Unit t = decode(u);
                if (t.skip) continue;
                if (u == u_begin) TB_PHASE(14);
                const uint8_t* codes =
                    p.weight + ((static_cast<long long>(t.expert) * p.n_tiles + t.nt) * p.k_blocks + t.kb0) * kBlockBytes;
                // group scales: [E, K/128, n_pad, 8] bytes, 1 KB per (K block, channel tile); else a TMA box of the
                // [E * K/16, n_pad] matrix at row sf_y
                const uint8_t* gscale = p.scale + ((static_cast<long long>(t.expert) * p.k_blocks + t.kb0) * p.n_pad + t.nt * 128) * 8;
                const long long gscale_step = static_cast<long long>(p.n_pad) * 8;
                int sf_y = t.expert * (p.k_pad / 16) + t.kb0 * 8;
                const int sf_x = t.nt * 128;
                for (int kb = t.kb0; kb < t.kb1; ++kb) {
                    [[maybe_unused]] const uint32_t w0 = TB_CLOCK();
                    if (!mbar_wait(empty, phase ^ 1u, abort_flag, kWaitWeightEmpty, 0, p.wait_cycles)) { ok = false; break; }
                    waited += TB_CLOCK() - w0;
                    if (kb == t.kb0 && u == u_begin) TB_PHASE(15);
                    mbar_arrive_expect_tx(full, kWeightRawBytes);
                    bulk_load(stage, codes, kBlockBytes, full);
                    if constexpr (kGroupScales) {
                        bulk_load(stage + kBlockBytes, gscale, kBlockScaleBytes, full);
                        gscale += gscale_step;
                    } else {
                        tma_load_2d(stage + kBlockBytes, &p.map_sf, sf_x, sf_y, full);
                        sf_y += 8;
                    }
                    if (kb == t.kb0 && u == static_cast<int>(blockIdx.x)) TB_PHASE(3);
                    codes += kBlockBytes;
                    stage += L.weight_stage; full += 8; empty += 8;
                    if (++rs == WS) { rs = 0; phase ^= 1u; stage = weights0_u32; full = w_full(0); empty = w_empty(0); }
                }
            }
            TB_REPORT(0, TB_CLOCK() - loop_begin);
            TB_REPORT(1, waited);
        }
        __syncwarp();
        // All loads were consumed unless the CTA is unwinding; then give the copies in flight a bounded chance to land.
        if (*abort_flag != 0) {
            for (int s = 0; s < WS; ++s) {
                const long long start = clock64();
                while (!mbar_try_wait(w_full(s), 0) && !mbar_try_wait(w_full(s), 1) && clock64() - start < (1ll << 24)) {}
            }
        }
    } else if (warp == kActWarp) {
        // =========================== activation producer ===========================
        // The BM x 128-byte activation tile of every K block: one TMA tile load by one thread, or (indexed routing
        // without a gather pass) per-row cp.async by the whole warp.
        if (!gather) {
            if (elect_one()) {
                uint32_t stage = tokens0_u32, full = a_full(0), empty = a_empty(0);
                int rs = 0;
                uint32_t phase = 0;
                bool ok = true;
                for (int u = u_begin; u < u_end && ok; u += u_step) {
                    const Unit t = decode(u);
                    if (t.skip) continue;
                    int x = t.kb0 * 128;
                    for (int kb = t.kb0; kb < t.kb1; ++kb) {
                        if (!mbar_wait(empty, phase ^ 1u, abort_flag, kWaitTokenEmpty, 0, p.wait_cycles)) { ok = false; break; }
                        if (dense && u == u_begin && kb == t.kb0) pdl_wait_prior_grid();
                        mbar_arrive_expect_tx(full, kActBytes);
                        tma_load_2d(stage, &p.map_a, x, t.row0, full);
                        x += 128;
                        stage += L.token_stage; full += 8; empty += 8;
                        if (++rs == AS) { rs = 0; phase ^= 1u; stage = tokens0_u32; full = a_full(0); empty = a_empty(0); }
                    }
                }
            }
            __syncwarp();
        } else {
            int rs = 0;
            uint32_t phase = 0;
            const long long route_limit = p.rows * p.top_k;
            bool ok = true;
            for (int u = u_begin; u < u_end && ok; u += u_step) {
                const Unit t = decode(u);
                if (t.skip) continue;
                // Source row of every tile row (-1 = padding), once per tile: route id / top_k.
                __syncwarp();
                for (int i = lane; i < BM; i += 32) {
                    const long long id = p.sorted_ids[t.row0 + i];
                    ids[i] = (id >= 0 && id < route_limit) ? static_cast<int>(id / p.top_k) : -1;
                }
                __syncwarp();
                for (int kb = t.kb0; kb < t.kb1; ++kb) {
                    if (!__all_sync(0xffffffffu, mbar_wait(a_empty(rs), phase ^ 1u, abort_flag, kWaitTokenEmpty, 0, p.wait_cycles))) { ok = false; break; }
                    const uint32_t stage = tokens0_u32 + rs * L.token_stage;
                    // Row gather: 8 chunks of 16 bytes per row, written through the 128-byte swizzle.
                    const int chunk = lane & 7;
                    const int col = kb * 128 + chunk * 16;
                    const bool col_ok = col < p.k;
#pragma unroll 4
                    for (int row = lane >> 3; row < BM; row += 4) {
                        const int src_row = ids[row];
                        const bool valid = src_row >= 0 && col_ok;
                        const uint8_t* src = p.a + (valid ? static_cast<long long>(src_row) * p.k + col : 0);
                        cp_async_16(stage + row * 128 + ((chunk ^ (row & 7)) << 4), src, valid);
                    }
                    cp_async_arrive_noinc(a_full(rs));
                    if (++rs == AS) { rs = 0; phase ^= 1u; }
                }
            }
            asm volatile("cp.async.wait_all;" ::: "memory");
        }
    } else if (warp == kMmaWarp) {
        // =========================== MMA issue ===========================
        // One thread runs the whole loop.  Descriptors advance by additions: the B operand (activation tile, K-major,
        // 128-byte swizzle) moves by the stage size, the A operand by 32 tensor-memory columns per bridged stage.
        constexpr uint32_t idesc = umma_idesc_e4m3(128, BM);
        bool ok = true;
        if (elect_one()) {
            const uint64_t b_desc0 = umma_desc_k_sw128(tokens0_u32);
            const uint64_t b_step = L.token_stage >> 4;
            const uint32_t a_addr0 = tmem_base + kAccCols;
            uint64_t b_desc = b_desc0;
            uint32_t a_addr = a_addr0;
            uint32_t t_full = a_full(0), t_empty = a_empty(0), b_full = br_full(0), b_empty = br_empty(0);
            int rs = 0, bs = 0, acc = 0;
            uint32_t bphase = 0, tphase = 0, aphase = 0;
            [[maybe_unused]] uint32_t waited = 0, blocks = 0, loop_begin = 0;
            for (int u = u_begin; u < u_end && ok; u += u_step) {
                const Unit t = decode(u);
                if (t.skip) continue;
                if constexpr (!kGroupScales) {
                    if (!mbar_wait(acc_empty(acc), aphase ^ 1u, abort_flag, kWaitAccEmpty, 0, p.wait_cycles)) { ok = false; break; }
                    tc_fence_after_sync();
                }
                for (int kb = t.kb0; kb < t.kb1; ++kb) {
                    if constexpr (kGroupScales) {
                        if (!mbar_wait(acc_empty(acc), aphase ^ 1u, abort_flag, kWaitAccEmpty, 0, p.wait_cycles)) { ok = false; break; }
                    }
                    [[maybe_unused]] const uint32_t w0 = TB_CLOCK();
                    {   // both polls in flight at once; the bounded waits only when one of them is not there yet
                        const bool tokens_in = mbar_try_wait(t_full, tphase), bridged_in = mbar_try_wait(b_full, bphase);
                        if (!tokens_in && !mbar_wait(t_full, tphase, abort_flag, kWaitTokenFull, 0, p.wait_cycles)) { ok = false; break; }
                        if (!bridged_in && !mbar_wait(b_full, bphase, abort_flag, kWaitBridgedFull, 0, p.wait_cycles)) { ok = false; break; }
                    }
                    if (blocks++ == 0) { loop_begin = TB_CLOCK(); TB_PHASE(5); } else { waited += TB_CLOCK() - w0; }
                    tc_fence_after_sync();
                    if (gather) fence_proxy_async_smem();
                    const uint32_t d_addr = tmem_base + acc * BM;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {  // 32 K values = 8 tensor-memory columns of A, 32 bytes of each B row
                        const uint32_t accumulate = kGroupScales ? (k > 0) : (kb > t.kb0 || k > 0);
                        umma_f8f6f4_ts(d_addr, a_addr + k * 8, b_desc + k * 2, idesc, accumulate);
                    }
                    umma_commit(b_empty);
                    umma_commit(t_empty);
                    if (kGroupScales || kb == t.kb1 - 1) umma_commit(acc_full(acc));
                    b_desc += b_step; t_full += 8; t_empty += 8;
                    if (++rs == AS) { rs = 0; tphase ^= 1u; b_desc = b_desc0; t_full = a_full(0); t_empty = a_empty(0); }
                    a_addr += kTileCols; b_full += 8; b_empty += 8;
                    if (++bs == BS) { bs = 0; bphase ^= 1u; a_addr = a_addr0; b_full = br_full(0); b_empty = br_empty(0); }
                    if constexpr (kGroupScales) {
                        if (++acc == kAccSets) { acc = 0; aphase ^= 1u; }
                    }
                }
                if constexpr (!kGroupScales) {
                    if (++acc == kAccSets) { acc = 0; aphase ^= 1u; }
                }
            }
            TB_PHASE(6);
            TB_REPORT(2, TB_CLOCK() - loop_begin);
            TB_REPORT(3, waited);
            TB_REPORT(7, blocks);
        }
        __syncwarp();
        // When unwinding, MMAs may still be running: wait (bounded) for them before the TMEM is released.
        if (*abort_flag != 0) {
            if (lane == 0) umma_commit(drain_bar);
            __syncwarp();
            const long long start = clock64();
            while (!mbar_try_wait(drain_bar, 0) && clock64() - start < (1ll << 26)) {}
        }
    } else if (warp >= kEpilogueWarps) {
        // =========================== bridge ===========================
        if constexpr (rebalances_registers(BM, kGroupScales, kBridgeWarps)) setmaxnreg_dec<rebalanced_bridge_regs(BM)>();
        // Thread bt of a team owns vectors bt, bt + kTeamThreads, ... of its 128 x 128 block (layout in tb_bridge.cuh).
        const int team = (warp - kEpilogueWarps) / kGroupWarps;
        const int first = team;  // its first K block; then every kTurns-th
        const int bt = ((warp - kEpilogueWarps) % kGroupWarps) * 32 + lane;
        constexpr int kVecsPerThread = 512 / kTeamThreads;  // 4, 2 or 1
        const int r = bt & 127;  // channel row = tensor-memory lane 32 * (warp % 4) + lane
        const uint32_t a_lane = tmem_base + kAccCols + (static_cast<uint32_t>(r & ~31) << 16);
        int rs = first % WS, bs = first % BS;
        uint32_t rphase = (first / WS) & 1, bphase = (first / BS) & 1;
        int turn = first;  // blocks of the coming unit that belong to the teams before this one's next block
        bool ok = true;
        [[maybe_unused]] uint32_t waited_raw = 0, waited_empty = 0, blocks = 0, loop_begin = 0;
        for (int u = u_begin; u < u_end && ok; u += u_step) {
            const Unit t = decode(u);
            if (t.skip) continue;
            int kb = t.kb0 + turn;
            for (; kb < t.kb1; kb += kTurns) {  // this team's blocks only
                // The tensor-memory stores below are warp-wide instructions: the warp must agree on every wait's outcome.
                [[maybe_unused]] const uint32_t w0 = TB_CLOCK();
                if (!__all_sync(0xffffffffu, mbar_wait(w_full(rs), rphase, abort_flag, kWaitWeightFull, 0, p.wait_cycles))) { ok = false; break; }
                if (blocks++ == 0) { loop_begin = TB_CLOCK(); if (warp == kEpilogueWarps && lane == 0) TB_PHASE(4); } else { waited_raw += TB_CLOCK() - w0; }
                const uint8_t* codes = weights0 + rs * L.weight_stage;
                const uint8_t* scales = codes + kBlockBytes;
                uint4 v[kVecsPerThread];
                uint32_t sc[kVecsPerThread][2];
#pragma unroll
                for (int i = 0; i < kVecsPerThread; ++i) {
                    const int vec = bt + i * kTeamThreads;
                    v[i] = *reinterpret_cast<const uint4*>(codes + vec * 16);
                    const int c0 = (vec >> 7) * 2;  // first of the vector's two 16-wide scale groups
                    if constexpr (kGroupScales) {
                        const uint32_t two = *reinterpret_cast<const uint16_t*>(scales + r * 8 + c0);
                        sc[i][0] = two & 0xFFu;
                        sc[i][1] = two >> 8;
                    } else {
                        sc[i][0] = scales[c0 * 128 + r];
                        sc[i][1] = scales[(c0 + 1) * 128 + r];
                    }
                }
                // Convert first, into registers: the stage of the bridged ring may still be feeding the tensor core, and
                // only the stores have to wait for it.
                uint4 fp8[kVecsPerThread][2];
#pragma unroll
                for (int i = 0; i < kVecsPerThread; ++i) {
                    const BridgeTables<kExact> t0(sc[i][0]), t1(sc[i][1]);
                    fp8[i][0] = t0.chunk(v[i].x, v[i].y);
                    fp8[i][1] = t1.chunk(v[i].z, v[i].w);
                }
                [[maybe_unused]] const uint32_t w1 = TB_CLOCK();
                if (!__all_sync(0xffffffffu, mbar_wait(br_empty(bs), bphase ^ 1u, abort_flag, kWaitBridgedEmpty, 0, p.wait_cycles))) { ok = false; break; }
                waited_empty += TB_CLOCK() - w1;
                tc_fence_after_sync();
#pragma unroll
                for (int i = 0; i < kVecsPerThread; ++i) {
                    const int vec = bt + i * kTeamThreads;
                    // 32 K values of this row: columns 8 * (vec / 128) .. +7 of the stage
                    tmem_st_8(a_lane + bs * kTileCols + (vec >> 7) * 8, fp8[i][0], fp8[i][1]);
                }
                tmem_st_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(br_full(bs));
                    mbar_arrive(w_empty(rs));
                }
                rs += kTurns;
                if (rs >= WS) { rs -= WS; rphase ^= 1u; }
                bs += kTurns;
                if (bs >= BS) { bs -= BS; bphase ^= 1u; }
            }
            turn = kb - t.kb1;  // what is left of the stride carries into the next unit
        }
        if (warp == kEpilogueWarps && lane == 0) { TB_REPORT(4, TB_CLOCK() - loop_begin); TB_REPORT(5, waited_raw); TB_REPORT(6, waited_empty); }
    } else {
        // =========================== epilogue ===========================
        if constexpr (rebalances_registers(BM, kGroupScales, kBridgeWarps)) setmaxnreg_inc<rebalanced_epilogue_regs(BM)>();
        const int quad = warp & 3, cgroup = warp >> 2;
        const int col0 = cgroup * kCols;          // first token column of this warp
        const int n_local = quad * 32 + lane;     // TMEM lane = channel within a 128-channel tile
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
        // This warp's staged row scales and output rows (-1 = none) for its kCols columns.
        float* my_scale = reinterpret_cast<float*>(smem + L.epi) + quad * 2 * BM + cgroup * 2 * kCols;
        int* my_row = reinterpret_cast<int*>(my_scale + kCols);
        // Output as 16-byte words: when eight channels of a row make an aligned word, the warp turns each 16-column
        // chunk around in shared memory ([token][channel] BF16) and writes it with two 16-byte stores per lane (four
        // lanes per row) instead of sixteen 2-byte stores, which the store path takes at a fraction of the rate.
        // (Worked out where they are used: nothing of this stays in registers across the main loop.)
        auto wide = [&]() { return (p.n & 7) == 0 && (reinterpret_cast<uintptr_t>(p.d) & 15) == 0; };
        auto turned_chunk = [&]() {
            return reinterpret_cast<__nv_bfloat16*>(smem + L.transpose + warp * (staged_chunks(BM) * kTransposeBytes));
        };
        // K-split launches number themselves on the device.  Word 0 of the workspace is the sequence of the last launch
        // that ran on it, word 1 counts the CTAs of this launch that have read it; the CTA that arrives last advances the
        // sequence.  By then every CTA of the grid holds its copy, and the next launch on the workspace starts after this
        // one has ended, so the tags of a launch differ from those of every earlier one -- under CUDA-graph replay and
        // after a launch that gave up as well.  (The arrival releases, so the read before it cannot slip behind it.)
        uint32_t launch_seq = 0;
        if (!kGroupScales && p.layout == kDense && (p.splits > 1 || p.shared_tiles > 0)) {
            volatile uint32_t* const seq_slot = reinterpret_cast<volatile uint32_t*>(smem + L.misc + 8);
            if (warp == 0 && lane == 0) {
                unsigned* const head = reinterpret_cast<unsigned*>(p.workspace);
                const unsigned seq = __ldcg(head) & 0x1FFFFFFu;
                unsigned arrived;
                asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(arrived) : "l"(head + 1) : "memory");
                if (arrived == gridDim.x - 1) {
                    __stcg(head + 1, 0u);
                    __stcg(head, (seq + 1u) & 0x1FFFFFFu);
                }
                *seq_slot = seq;
            }
            named_barrier_sync(1, kEpilogueWarps * 32);
            launch_seq = *seq_slot;
        }
        int acc = 0;
        uint32_t aphase = 0;
        bool ok = true;
        const long long route_limit = p.rows * p.top_k;
        for (int u = u_begin; u < u_end && ok; u += u_step) {
            const Unit t = decode(u);
            if (t.skip) continue;
            const float gs = p.global_scale[t.expert];
            const bool partial = !kGroupScales && p.layout == kDense && p.splits > 1;
            const uint32_t tag = (static_cast<uint32_t>(t.tile) << 25) | ((launch_seq + 1u) & 0x1FFFFFFu);
            const int cols_valid = indexed ? kCols : max(0, min(kCols, t.rows_valid - col0));  // live columns of this warp
            // First element of a staged output row: a row of `d`, or (expert-parallel scatter) of the owning rank's buffer.
            auto out_row_ptr = [&](int row) -> __nv_bfloat16* {
                if (p.row_target == nullptr) return p.d + static_cast<long long>(row) * p.n;
                return p.peer_out[row >> 26] + static_cast<long long>(row & 0x3FFFFFF) * p.n;
            };
            // Writes the turned chunk c to the staged output rows of its columns: lane -> row lane / 4 (and + 8) of the
            // chunk, 8-channel word lane % 4 of the row.
            // (`swapped`: the chunk was turned by stmatrix, which keeps the 16-byte words of a row swapped around by the
            // token index.)
            auto flush_turned = [&](int c, bool swapped = false) {
                const int tok = lane >> 2, part = lane & 3;
                const int nv = t.nt * 128 + quad * 32 + part * 8;
                const __nv_bfloat16* turned = turned_chunk();
                const int slot = swapped ? (part ^ ((tok >> 1) & 3)) : part;
                __syncwarp();
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = my_row[c * 16 + h * 8 + tok];
                    const uint4 word = *reinterpret_cast<const uint4*>(turned + (h * 8 + tok) * 32 + slot * 8);
                    if (nv < p.n && row >= 0) *reinterpret_cast<uint4*>(out_row_ptr(row) + nv) = word;
                }
                __syncwarp();
            };

            // Stage the output row of every column and (per-token scales) its scale times the global scale; this runs
            // while the main loop of the tile is still in flight.
            __syncwarp();
#pragma unroll
            for (int j = 0; j < (kCols + 31) / 32; ++j) {
                const int c = j * 32 + lane;
                if (c < kCols) {
                    const int i = col0 + c;
                    long long in_row = -1, out_row = -1;
                    if (indexed) {
                        const long long id = p.sorted_ids[t.row0 + i];
                        if (id >= 0 && id < route_limit) { in_row = id / p.top_k; out_row = id; }
                    } else if (i < t.rows_valid) {
                        in_row = out_row = t.row0 + i;
                        if (p.row_target != nullptr) out_row = p.row_target[in_row];
                    }
                    my_row[c] = static_cast<int>(out_row);
                    if constexpr (!kGroupScales) my_scale[c] = in_row >= 0 ? p.a_scale[in_row * p.a_scale_stride_m] * gs : 0.f;
                }
            }
            __syncwarp();

            if constexpr (kGroupScales) {
                // Promote each 128-deep partial with its [1,128] activation scale in registers.  The scales of
                // kScaleChunk K blocks at a time are staged in shared memory as [K block][column of this warp]: a
                // lane fetches them for its one or two columns (independent loads, one round trip per chunk), and a
                // K block then reads them with broadcast loads.
                const int n = t.nt * 128 + n_local;
                const bool n_ok = n < p.n;
                constexpr int kPer = (kCols + 31) / 32;
                float total[kCols];
#pragma unroll
                for (int c = 0; c < kCols; ++c) total[c] = 0.f;
                float* const staged = reinterpret_cast<float*>(smem + L.group_scales) + (quad * BM + cgroup * kCols) * kScaleChunk;
                const float* scale_row[kPer];  // first scale of this lane's columns (null: no such row)
#pragma unroll
                for (int j = 0; j < kPer; ++j) {
                    const int c = j * 32 + lane;
                    long long in_row = -1;
                    if (c < kCols) {
                        const int i = col0 + c;
                        if (indexed) {
                            const long long id = p.sorted_ids[t.row0 + i];
                            if (id >= 0 && id < route_limit) in_row = id / p.top_k;
                        } else if (i < t.rows_valid) {
                            in_row = t.row0 + i;
                        }
                    }
                    scale_row[j] = in_row >= 0 ? p.a_scale + in_row * p.a_scale_stride_m : nullptr;
                }
                auto stage_scales = [&](int kb) {  // K blocks kb .. kb + kScaleChunk - 1 of the tile
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < kPer; ++j) {
                        const int c = j * 32 + lane;
                        if (c < kCols) {
                            float sv[kScaleChunk];
#pragma unroll
                            for (int g = 0; g < kScaleChunk; ++g)
                                sv[g] = (scale_row[j] != nullptr && kb + g < t.kb1) ? scale_row[j][(kb + g) * p.a_scale_stride_k] : 0.f;
#pragma unroll
                            for (int g = 0; g < kScaleChunk; ++g) staged[g * kCols + c] = sv[g];
                        }
                    }
                    __syncwarp();
                };
                for (int kb = t.kb0; kb < t.kb1 && ok; ++kb) {
                    const int local = (kb - t.kb0) & (kScaleChunk - 1);
                    if (local == 0) stage_scales(kb);
                    const float* const block_scale = staged + local * kCols;
                    if (!mbar_wait(acc_full(acc), aphase, abort_flag, kWaitAccFull, 0, p.wait_cycles)) { ok = false; break; }
                    tc_fence_after_sync();
#pragma unroll
                    for (int c = 0; c < kCols / 32; ++c) {  // two 16-column loads in flight per wait
                        uint32_t v[2][16];
                        tmem_ld_16(lane_base + acc * BM + col0 + c * 32, v[0]);
                        tmem_ld_16(lane_base + acc * BM + col0 + c * 32 + 16, v[1]);
                        tmem_ld_wait();
#pragma unroll
                        for (int j4 = 0; j4 < 8; ++j4) {  // two packed FP32 multiply-adds per four columns
                            const float4 s4 = *reinterpret_cast<const float4*>(block_scale + c * 32 + j4 * 4);
                            const uint32_t* vv = &v[j4 >> 2][(j4 & 3) * 4];
                            float* tt = &total[c * 32 + j4 * 4];
                            fma2(tt[0], tt[1], __uint_as_float(vv[0]), __uint_as_float(vv[1]), s4.x, s4.y);
                            fma2(tt[2], tt[3], __uint_as_float(vv[2]), __uint_as_float(vv[3]), s4.z, s4.w);
                        }
                    }
                    if constexpr (kCols % 32 != 0) {  // a trailing 16-column chunk (token tile 16)
                        constexpr int c16 = kCols / 32 * 32;
                        uint32_t v[16];
                        tmem_ld_16(lane_base + acc * BM + col0 + c16, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int j4 = 0; j4 < 4; ++j4) {
                            const float4 s4 = *reinterpret_cast<const float4*>(block_scale + c16 + j4 * 4);
                            float* tt = &total[c16 + j4 * 4];
                            tt[0] = fmaf(__uint_as_float(v[j4 * 4 + 0]), s4.x, tt[0]);
                            tt[1] = fmaf(__uint_as_float(v[j4 * 4 + 1]), s4.y, tt[1]);
                            tt[2] = fmaf(__uint_as_float(v[j4 * 4 + 2]), s4.z, tt[2]);
                            tt[3] = fmaf(__uint_as_float(v[j4 * 4 + 3]), s4.w, tt[3]);
                        }
                    }
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty(acc));
                    if (++acc == kAccSets) { acc = 0; aphase ^= 1u; }
                }
                if (!ok) break;
                if (wide()) {
                    __nv_bfloat16* const turned = turned_chunk();
#pragma unroll
                    for (int c = 0; c < kCols / 16; ++c) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) turned[j * 32 + lane] = __float2bfloat16_rn(total[c * 16 + j] * gs);
                        flush_turned(c);
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < kCols; ++c) {
                        const int out_row = my_row[c];
                        if (out_row >= 0 && n_ok) out_row_ptr(out_row)[n] = __float2bfloat16_rn(total[c] * gs);
                    }
                }
            } else {
                if (!mbar_wait(acc_full(acc), aphase, abort_flag, kWaitAccFull, 100, p.wait_cycles)) { ok = false; break; }
                tc_fence_after_sync();
                if (warp == 0 && lane == 0) TB_PHASE(7);
                const int n = t.nt * 128 + n_local;
                const bool n_ok = n < p.n;
                const bool wide_stores = wide();
                // Chunk c (16 token columns) of this warp's accumulator -> BF16 [token][32 channels] in the warp's shared
                // buffer, scaled: two 16-lane loads in MMA-fragment layout, packed pairs, two stmatrix.trans (the
                // 16-byte words of a row end up swapped around by the token index: no bank conflicts either way).
                auto turn_chunk = [&](int c) {
                    uint32_t lo[8], hi[8];
                    const uint32_t addr = lane_base + acc * BM + col0 + c * 16;
                    tmem_ld_16x256b_x2(addr, lo);
                    tmem_ld_16x256b_x2(addr + (16u << 16), hi);
                    tmem_ld_wait_for(lo, hi);
                    const float2 s0 = *reinterpret_cast<const float2*>(my_scale + c * 16 + 2 * (lane & 3));
                    const float2 s1 = *reinterpret_cast<const float2*>(my_scale + c * 16 + 8 + 2 * (lane & 3));
                    auto pack = [](uint32_t x, uint32_t y, const float2& sc) {
                        const __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(x) * sc.x, __uint_as_float(y) * sc.y);
                        return *reinterpret_cast<const uint32_t*>(&pair);
                    };
                    const uint32_t st = smem_u32(turned_chunk()) + (lane & 7) * 64 + (((lane >> 3) ^ ((lane >> 1) & 3)) << 4);
                    stmatrix_x4_trans(st, pack(lo[0], lo[1], s0), pack(lo[2], lo[3], s0), pack(hi[0], hi[1], s0), pack(hi[2], hi[3], s0));
                    stmatrix_x4_trans(st + 512, pack(lo[4], lo[5], s1), pack(lo[6], lo[7], s1), pack(hi[4], hi[5], s1), pack(hi[6], hi[7], s1));
                };
                if constexpr (kAccSets == 1) if (t.parts > 0) {
                    // A tile of the last, partial round: `parts` CTAs hold K-block ranges of it (CTAs first ... first +
                    // parts - 1, this one is number `part`).  Every warp's eight 16-token chunks are dealt out among the
                    // parts (chunk c belongs to part c % parts).  A part first publishes the FP32 partial sums of the
                    // chunks it does not own -- as they come out of tensor memory, register for register, into its
                    // slot of the workspace -- and raises its flag with the launch's tag; then it waits (bounded) for
                    // the flags of the others and finishes its own chunks: partial sums added in part order 0, 1, ...
                    // whoever does the adding, so the result does not depend on timing.  Nobody waits before it has
                    // published, and all CTAs of the grid are resident: no part waits on one that waits on it.
                    const int first_cta = static_cast<int>(blockIdx.x) - t.part;
                    uint4* const slot0 = reinterpret_cast<uint4*>(p.workspace + kEpochCells) + warp * (8 * 4 * 32) + lane;
                    auto slot_of = [&](int cta) { return slot0 + (static_cast<long long>(cta) * kBalancedTileWords >> 2); };
                    const uint32_t balanced_tag = (launch_seq + 1u) & 0x1FFFFFFu;
                    const uint32_t acc_addr = lane_base + acc * BM + col0;
                    constexpr int kChunks = kCols / 16;
                    uint4* const mine = slot_of(blockIdx.x);
                    for (int c = 0; c < kChunks; ++c) {  // pass 1: publish
                        if (c * 16 >= cols_valid) break;
                        if (c % t.parts == t.part) continue;
                        uint32_t lo[8], hi[8];
                        tmem_ld_16x256b_x2(acc_addr + c * 16, lo);
                        tmem_ld_16x256b_x2(acc_addr + c * 16 + (16u << 16), hi);
                        tmem_ld_wait_for(lo, hi);
                        __stcg(mine + (c * 4 + 0) * 32, make_uint4(lo[0], lo[1], lo[2], lo[3]));
                        __stcg(mine + (c * 4 + 1) * 32, make_uint4(lo[4], lo[5], lo[6], lo[7]));
                        __stcg(mine + (c * 4 + 2) * 32, make_uint4(hi[0], hi[1], hi[2], hi[3]));
                        __stcg(mine + (c * 4 + 3) * 32, make_uint4(hi[4], hi[5], hi[6], hi[7]));
                    }
                    __threadfence();
                    named_barrier_sync(1, kEpilogueWarps * 32);
                    if (warp == 0 && lane == 0) {
                        unsigned* const flags = reinterpret_cast<unsigned*>(p.workspace) + kBalancedFlag0;
                        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flags + blockIdx.x), "r"(balanced_tag) : "memory");
                        const long long start = clock64();
                        for (int q = 0; q < t.parts && *abort_flag == 0; ++q) {
                            if (q == t.part) continue;
                            unsigned seen;
                            for (uint32_t spin = 0;; ++spin) {
                                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags + first_cta + q) : "memory");
                                if (seen == balanced_tag) break;
                                if ((spin & 15u) == 15u && (*abort_flag != 0 || clock64() - start > p.wait_cycles)) {
                                    atomicCAS(const_cast<int*>(abort_flag), 0, kWaitSplit);
                                    break;
                                }
                            }
                        }
                    }
                    named_barrier_sync(1, kEpilogueWarps * 32);
                    if (*abort_flag != 0) { ok = false; break; }
                    // pass 2: this part's chunks.  Sums in part order; the own partial sums come from tensor memory.
                    const uint32_t stage_u32 = smem_u32(turned_chunk());
                    const uint32_t st_addr = stage_u32 + (lane & 7) * 64 + (((lane >> 3) ^ ((lane >> 1) & 3)) << 4);
                    const float* const scale_pair = my_scale + 2 * (lane & 3);
                    int parked = 0;  // chunks of this warp turned into shared memory (at most three: parts >= 2, one slot each)
                    for (int c = t.part; c < kChunks; c += t.parts) {
                        if (c * 16 >= cols_valid) break;
                        uint32_t lo[8], hi[8];
                        tmem_ld_16x256b_x2(acc_addr + c * 16, lo);
                        tmem_ld_16x256b_x2(acc_addr + c * 16 + (16u << 16), hi);
                        tmem_ld_wait_for(lo, hi);
                        // The others' sums of the same registers, all loads in flight at once (another SM wrote them:
                        // not through L1); then the additions in part order, the own sums in their place.
                        constexpr int kOthers = kMaxSharedParts - 1;
                        uint4 theirs[kOthers][4];
#pragma unroll
                        for (int r = 0; r < kOthers; ++r) {
                            if (r < t.parts - 1) {
                                const uint4* const from = slot_of(first_cta + (r < t.part ? r : r + 1)) + c * 4 * 32;
#pragma unroll
                                for (int i = 0; i < 4; ++i) theirs[r][i] = __ldcg(from + i * 32);
                            }
                        }
                        float sum[16];
#pragma unroll
                        for (int q = 0; q < kMaxSharedParts; ++q) {
                            if (q < t.parts) {
                                float term[16];
                                if (q == t.part) {
#pragma unroll
                                    for (int i = 0; i < 8; ++i) { term[i] = __uint_as_float(lo[i]); term[8 + i] = __uint_as_float(hi[i]); }
                                } else {
#pragma unroll
                                    for (int r = 0; r < kOthers; ++r) {
                                        if (r == (q < t.part ? q : q - 1)) {
                                            const uint4* const w = theirs[r];
                                            const uint32_t words[16] = {w[0].x, w[0].y, w[0].z, w[0].w, w[1].x, w[1].y, w[1].z, w[1].w,
                                                                        w[2].x, w[2].y, w[2].z, w[2].w, w[3].x, w[3].y, w[3].z, w[3].w};
#pragma unroll
                                            for (int i = 0; i < 16; ++i) term[i] = __uint_as_float(words[i]);
                                        }
                                    }
                                }
#pragma unroll
                                for (int i = 0; i < 16; ++i) sum[i] = q == 0 ? term[i] : sum[i] + term[i];
                            }
                        }
                        const float2 s0 = *reinterpret_cast<const float2*>(scale_pair + c * 16);
                        const float2 s1 = *reinterpret_cast<const float2*>(scale_pair + c * 16 + 8);
                        auto pack = [](float x, float y, const float2& sc) {
                            const __nv_bfloat162 pair = __floats2bfloat162_rn(x * sc.x, y * sc.y);
                            return *reinterpret_cast<const uint32_t*>(&pair);
                        };
                        stmatrix_x4_trans(st_addr + parked * 1024, pack(sum[0], sum[1], s0), pack(sum[2], sum[3], s0),
                                          pack(sum[8], sum[9], s0), pack(sum[10], sum[11], s0));
                        stmatrix_x4_trans(st_addr + parked * 1024 + 512, pack(sum[4], sum[5], s1), pack(sum[6], sum[7], s1),
                                          pack(sum[12], sum[13], s1), pack(sum[14], sum[15], s1));
                        ++parked;
                    }
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty(acc));
                    {   // the output of this part's chunks: lane -> token lane / 4 (and + 8), 8-channel word lane % 4 of its row
                        const int tok = lane >> 2, part8 = lane & 3;
                        const int nv = t.nt * 128 + quad * 32 + part8 * 8;
                        const uint32_t ld_addr = stage_u32 + tok * 64 + ((part8 ^ ((tok >> 1) & 3)) << 4);
                        int slot = 0;
                        for (int c = t.part; c < kChunks && slot < parked; c += t.parts, ++slot) {
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const int col = c * 16 + h * 8 + tok;
                                const uint4 word = lds_128(ld_addr + slot * 1024 + h * 512);
                                if (nv < p.n && col < cols_valid)
                                    *reinterpret_cast<uint4*>(p.d + static_cast<long long>(t.row0 + col0 + col) * p.n + nv) = word;
                            }
                        }
                    }
                    __syncwarp();
                    if (++acc == kAccSets) { acc = 0; aphase ^= 1u; }
                    continue;
                }
                if constexpr (kAccSets == 1) if (!partial && wide_stores) {
                    // One accumulator set: everything out of tensor memory first, then the accumulator goes back to the
                    // MMA warp, then the output is written (while the next tile accumulates).
                    // A 16-token chunk comes out of tensor memory as two 16-lane loads in the layout of an MMA
                    // accumulator fragment (lane: channels lane / 4 and + 8, tokens 2 * (lane % 4) and + 1 of each
                    // 8-token half), is scaled, packed to BF16 pairs and turned around by stmatrix.trans: shared
                    // memory gets [token][32 channels], 64 bytes a token, the 16-byte words of a row swapped around by
                    // the token index so that neither the matrix stores nor the row reads collide on banks.
                    constexpr int kChunks = kCols / 16, kStaged = staged_chunks(BM) < kChunks ? staged_chunks(BM) : kChunks;
                    constexpr int kKept = kChunks - kStaged;
                    const uint32_t stage_u32 = smem_u32(turned_chunk());
                    // stmatrix: lane -> 8-channel group lane / 8, token lane % 8 of a half; the word's slot in its row
                    const uint32_t st_addr = stage_u32 + (lane & 7) * 64 + (((lane >> 3) ^ ((lane >> 1) & 3)) << 4);
                    uint32_t kept[kKept > 0 ? kKept * 8 : 1];
                    const uint32_t acc_addr = lane_base + acc * BM + col0;
                    const float* const scale_pair = my_scale + 2 * (lane & 3);
                    auto step = [&](auto chunk) {
                        constexpr int c = decltype(chunk)::value;
                        if (c * 16 < cols_valid) {  // warp-uniform
                            uint32_t lo[8], hi[8];  // channels 0-15 and 16-31 of the warp's 32
                            tmem_ld_16x256b_x2(acc_addr + c * 16, lo);
                            tmem_ld_16x256b_x2(acc_addr + c * 16 + (16u << 16), hi);
                            tmem_ld_wait_for(lo, hi);
                            const float2 s0 = *reinterpret_cast<const float2*>(scale_pair + c * 16);
                            const float2 s1 = *reinterpret_cast<const float2*>(scale_pair + c * 16 + 8);
                            auto pack = [](uint32_t x, uint32_t y, const float2& sc) {
                                const __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(x) * sc.x, __uint_as_float(y) * sc.y);
                                return *reinterpret_cast<const uint32_t*>(&pair);
                            };
                            // words of the first token half (channel groups 0-3), then of the second
                            const uint32_t w[8] = {pack(lo[0], lo[1], s0), pack(lo[2], lo[3], s0), pack(hi[0], hi[1], s0), pack(hi[2], hi[3], s0),
                                                   pack(lo[4], lo[5], s1), pack(lo[6], lo[7], s1), pack(hi[4], hi[5], s1), pack(hi[6], hi[7], s1)};
                            if constexpr (c < kStaged) {
                                stmatrix_x4_trans(st_addr + c * 1024, w[0], w[1], w[2], w[3]);
                                stmatrix_x4_trans(st_addr + c * 1024 + 512, w[4], w[5], w[6], w[7]);
                            } else {
#pragma unroll
                                for (int i = 0; i < 8; ++i) kept[(c - kStaged) * 8 + i] = w[i];
                            }
                        }
                    };
                    static_assert(kChunks == 8, "the drain is written out for eight chunks");
                    step(IntC<0>{}); step(IntC<1>{}); step(IntC<2>{}); step(IntC<3>{});
                    step(IntC<4>{}); step(IntC<5>{}); step(IntC<6>{}); step(IntC<7>{});
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty(acc));
                    // The output: lane -> token lane / 4 (and + 8) of a chunk, 8-channel word lane % 4 of its row.
                    const int tok = lane >> 2, part = lane & 3;
                    const int nv = t.nt * 128 + quad * 32 + part * 8;
                    const bool nv_ok = nv < p.n;
                    const uint32_t ld_addr = stage_u32 + tok * 64 + ((part ^ ((tok >> 1) & 3)) << 4);
                    auto write_chunk = [&](int c, int slot) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int col = c * 16 + h * 8 + tok;
                            const uint4 word = lds_128(ld_addr + slot * 1024 + h * 512);
                            if (!nv_ok || col >= cols_valid) continue;
                            if (routed) {
                                const int row = my_row[col];
                                if (row >= 0) *reinterpret_cast<uint4*>(out_row_ptr(row) + nv) = word;
                            } else {
                                *reinterpret_cast<uint4*>(p.d + static_cast<long long>(t.row0 + col0 + col) * p.n + nv) = word;
                            }
                        }
                    };
#pragma unroll
                    for (int c = 0; c < kStaged; ++c) {
                        if (c * 16 < cols_valid) write_chunk(c, c);
                    }
                    if constexpr (kKept > 0) {
                        __syncwarp();  // the parked chunks have been read: their room takes the chunks kept in registers
#pragma unroll
                        for (int c = kStaged; c < kChunks; ++c) {
                            if (c * 16 < cols_valid) {
                                const uint32_t* const w = &kept[(c - kStaged) * 8];
                                stmatrix_x4_trans(st_addr + (c - kStaged) * 1024, w[0], w[1], w[2], w[3]);
                                stmatrix_x4_trans(st_addr + (c - kStaged) * 1024 + 512, w[4], w[5], w[6], w[7]);
                            }
                        }
                        __syncwarp();
#pragma unroll
                        for (int c = kStaged; c < kChunks; ++c) {
                            if (c * 16 < cols_valid) write_chunk(c, c - kStaged);
                        }
                    }
                    __syncwarp();  // before the next tile parks its chunks
                    if (++acc == kAccSets) { acc = 0; aphase ^= 1u; }
                    continue;
                }
                if (!partial && !routed && wide_stores) {
                    // Rows of the tile are consecutive rows of the output: one pointer, a fixed step per column.
                    __nv_bfloat16* const turned = turned_chunk();
                    const int tok = lane >> 2, part = lane & 3;
                    const int nv = t.nt * 128 + quad * 32 + part * 8;
                    const bool nv_ok = nv < p.n;
                    const long long step = p.n;
                    __nv_bfloat16* const out0 = p.d + static_cast<long long>(t.row0 + col0 + tok) * step + nv;
                    const int slot = part ^ ((tok >> 1) & 3);
                    for (int c = 0; c < kCols / 16; ++c) {
                        if (c * 16 >= cols_valid) break;
                        turn_chunk(c);
                        __syncwarp();
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int col = c * 16 + h * 8 + tok;
                            const uint4 word = *reinterpret_cast<const uint4*>(turned + (h * 8 + tok) * 32 + slot * 8);
                            if (nv_ok && col < cols_valid) *reinterpret_cast<uint4*>(out0 + (c * 16 + h * 8) * step) = word;
                        }
                        __syncwarp();
                    }
                } else if (!partial && !routed) {
                    // The same rows, any channel count or alignment: one pointer, a fixed step per column.
                    __nv_bfloat16* const out0 = p.d + static_cast<long long>(t.row0 + col0) * p.n + n;
                    const long long step = p.n;
                    for (int c = 0; c < kCols / 16; ++c) {
                        if (c * 16 >= cols_valid) break;
                        uint32_t v[16];
                        tmem_ld_16(lane_base + acc * BM + col0 + c * 16, v);
                        tmem_ld_wait();
                        __nv_bfloat16* out = out0 + c * 16 * step;
                        const int live = n_ok ? cols_valid - c * 16 : 0;  // columns of this chunk to write
#pragma unroll
                        for (int j4 = 0; j4 < 4; ++j4) {
                            const float4 s4 = *reinterpret_cast<const float4*>(my_scale + c * 16 + j4 * 4);
                            const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                if (j4 * 4 + e < live) out[(j4 * 4 + e) * step] = __float2bfloat16_rn(__uint_as_float(v[j4 * 4 + e]) * sv[e]);
                            }
                        }
                    }
                } else if (!partial && wide_stores) {
                    // Routed rows, 16-byte words: the staged output row of every column.
                    for (int c = 0; c < kCols / 16; ++c) {
                        if (c * 16 >= cols_valid) break;
                        turn_chunk(c);
                        flush_turned(c, true);
                    }
                } else if (!partial) {
                    for (int c = 0; c < kCols / 16; ++c) {
                        if (c * 16 >= cols_valid) break;
                        uint32_t v[16];
                        tmem_ld_16(lane_base + acc * BM + col0 + c * 16, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int j4 = 0; j4 < 4; ++j4) {
                            const float4 s4 = *reinterpret_cast<const float4*>(my_scale + c * 16 + j4 * 4);
                            const int4 r4 = *reinterpret_cast<const int4*>(my_row + c * 16 + j4 * 4);
                            const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
                            const int rv[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                if (rv[e] >= 0 && n_ok)
                                    out_row_ptr(rv[e])[n] = __float2bfloat16_rn(__uint_as_float(v[j4 * 4 + e]) * sv[e]);
                            }
                        }
                    }
                } else {
                    // Ordered split-K reduction without fences.  The token columns of a tile are cut into batches of
                    // eight and every batch has one owner among the tile's splits.  A split first publishes the FP32
                    // partial sums of the batches it does not own as 8-byte {value, tag} words (single stores, so a
                    // reader sees both halves or neither) -- all of them before it reads anything, so that nobody
                    // waits on a peer that is itself waiting -- then, for each batch it owns, reads its peers' words
                    // until their tags match, adds the splits in the order 0, 1, ..., S-1 and writes the output.  The
                    // words of two peers are in flight at once, so three splits cost one round trip to the L2 per
                    // batch.  The thread that holds an element in one split holds it in all of them: no thread waits
                    // for anything but its own elements.
                    // Ownership: when every unit of the launch has its own CTA (and so all splits of a tile are
                    // running, or will be as soon as an SM is free), batch b belongs to split b % S; otherwise the
                    // last split owns them all -- it is the last of the tile's units in launch order, so its peers
                    // are running or done.  The order of the additions does not depend on the owner.  Every wait is
                    // bounded.
                    // tag = {tile, launch sequence + 1}: words left by earlier launches never match.
                    if (warp == 0 && lane == 0) TB_PHASE(8);
                    const int S = p.splits;
                    const bool shared = total_units <= static_cast<int>(gridDim.x);
                    uint2* const slots = reinterpret_cast<uint2*>(p.workspace + kEpochCells) +
                                         static_cast<long long>(t.tile) * S * (BM * 128) + col0 * 128 + n_local;
                    const int batches = (cols_valid + 7) >> 3;
                    const int first_batch = col0 >> 3;  // index of this warp's first batch within the tile
                    for (int b = 0; b < batches; ++b) {  // pass 1: publish
                        if ((shared ? (first_batch + b) % S : S - 1) == t.split) continue;
                        uint32_t v[8];
                        tmem_ld_8(lane_base + acc * BM + col0 + b * 8, v);
                        tmem_ld_wait();
                        uint2* out = slots + (t.split * BM + b * 8) * 128;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            if (b * 8 + j < cols_valid)
                                asm volatile("st.global.cg.v2.b32 [%0], {%1, %2};" ::"l"(out + j * 128), "r"(v[j]), "r"(tag) : "memory");
                        }
                    }
                    for (int b = 0; b < batches && ok; ++b) {  // pass 2: reduce the owned batches
                        if ((shared ? (first_batch + b) % S : S - 1) != t.split) continue;
                        const int live = min(8, cols_valid - b * 8);
                        const uint32_t want = (1u << live) - 1u;
                        float sum[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) sum[j] = 0.f;
                        // Every lane runs every step (the tensor-memory load of the own partial sums is warp-wide); a lane
                        // whose wait ran out stops polling and its warp leaves after the batch.
                        for (int sp = 0; sp < S; sp += 2) {  // splits sp and sp + 1, fixed order of additions
                            uint2 got[2][8];
                            uint32_t need0 = (ok && sp != t.split) ? want : 0u;
                            uint32_t need1 = (ok && sp + 1 < S && sp + 1 != t.split) ? want : 0u;
                            const uint2* in = slots + (sp * BM + b * 8) * 128;
                            long long start = 0;
                            for (uint32_t spin = 0; (need0 | need1) != 0u; ++spin) {
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    if ((need0 >> j) & 1u)
                                        asm volatile("ld.global.cg.v2.b32 {%0, %1}, [%2];" : "=r"(got[0][j].x), "=r"(got[0][j].y)
                                                     : "l"(in + j * 128) : "memory");
                                    if ((need1 >> j) & 1u)
                                        asm volatile("ld.global.cg.v2.b32 {%0, %1}, [%2];" : "=r"(got[1][j].x), "=r"(got[1][j].y)
                                                     : "l"(in + (BM + j) * 128) : "memory");
                                }
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    if (((need0 >> j) & 1u) && got[0][j].y == tag) need0 &= ~(1u << j);
                                    if (((need1 >> j) & 1u) && got[1][j].y == tag) need1 &= ~(1u << j);
                                }
                                if ((need0 | need1) == 0u) break;
                                if (spin == 0) {
                                    start = clock64();
                                } else if ((spin & 15u) == 0u && (*abort_flag != 0 || clock64() - start > p.wait_cycles)) {
                                    atomicCAS(const_cast<int*>(abort_flag), 0, kWaitSplit);
                                    ok = false;
                                    break;
                                }
                            }
#pragma unroll
                            for (int q = 0; q < 2; ++q) {
                                if (sp + q >= S) break;
                                if (sp + q == t.split) {  // warp-uniform
                                    uint32_t v[8];
                                    tmem_ld_8(lane_base + acc * BM + col0 + b * 8, v);
                                    tmem_ld_wait();
#pragma unroll
                                    for (int j = 0; j < 8; ++j) sum[j] += __uint_as_float(v[j]);
                                } else {
#pragma unroll
                                    for (int j = 0; j < 8; ++j) sum[j] += __uint_as_float(got[q][j].x);
                                }
                            }
                        }
                        ok = __all_sync(0xffffffffu, ok);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const int i = b * 8 + j;
                            if (((want >> j) & 1u) && n_ok && ok)
                                p.d[static_cast<long long>(my_row[i]) * p.n + n] = __float2bfloat16_rn(sum[j] * my_scale[i]);
                        }
                    }
                    if (warp == 0 && lane == 0) TB_PHASE(t.split == S - 1 ? 9 : 10);
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty(acc));
                if (++acc == kAccSets) { acc = 0; aphase ^= 1u; }
            }
        }
    }

    // ---- teardown ----
    if (warp == 0 && lane == 0) TB_PHASE(11);
    if (*abort_flag != 0) {
        // Unwinding after a wait gave up: copies into this CTA's shared memory may still be in flight, and they must
        // land before the CTA exits.  A couple of milliseconds cover any of them.
        const long long start = clock64();
        while (clock64() - start < (1ll << 22)) {}
    }
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0) TB_PHASE(12);
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, tmem_cols);
    }
    if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) {
        if (atomicCAS(p.status, 0, *abort_flag) == 0) {
            p.status[1] = blockIdx.x;
            p.status[2] = total_units;
        }
    }
}

template <int BM, bool kExact, bool kGroupScales, int kBridgeWarps, int kBridgeGroups>
__global__ void __launch_bounds__(gemm_threads(BM, kBridgeWarps), 1) gemm_kernel(const __grid_constant__ GemmParams p) {
    gemm_body<BM, kExact, kGroupScales, kBridgeWarps, kBridgeGroups>(p);
}

}  // namespace tb
