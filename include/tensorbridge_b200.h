/* C ABI of libtensorbridge_b200.so: FP8-activation x NVFP4-weight GEMMs for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers, sizes and a `cudaStream_t` passed as `void*`; none allocates,
 * frees, synchronises or throws (the four set-up helpers for peer memory at the end of this file excepted).  The return value is 0 on success or one of the TB_ERR_* codes below, with a
 * human-readable message available from tb_last_error() (thread-local).  The caller owns every buffer, the
 * output included, so a launch is allocation-free and can be captured in a CUDA graph.
 *
 * Each declaration names the interface of the reference library (revollllt/atc26-tensorbridge) that it
 * replaces, as `file:line` relative to that project's root.
 */
#ifndef TENSORBRIDGE_B200_H_
#define TENSORBRIDGE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    TB_OK = 0,
    TB_ERR_INVALID = 1,     /* bad argument (shape, alignment, null pointer, unknown enum) */
    TB_ERR_CUDA = 2,        /* a CUDA runtime / driver call failed                           */
    TB_ERR_UNSUPPORTED = 3, /* valid request the library has no kernel for                   */
    TB_ERR_DEVICE = 4       /* a kernel reported an error in its status word                 */
};

/* Expert layouts of the grouped GEMM; values follow tensorbridge/jit/codegen.py:18 (LAYOUT_IDS). */
enum { TB_LAYOUT_DENSE = 0, TB_LAYOUT_INDEXED = 1, TB_LAYOUT_CONTIGUOUS = 2, TB_LAYOUT_MASKED = 3 };

/* Bridge tables; tensorbridge/jit/codegen.py:15 (Bridge). */
enum { TB_BRIDGE_FPMA = 0, TB_BRIDGE_EXACT = 1 };

/* Input element types of tb_quantize_fp8. */
enum { TB_DTYPE_BF16 = 0, TB_DTYPE_F16 = 1, TB_DTYPE_F32 = 2 };

/* Activation scale granularity; tensorbridge/quant/fp8.py:9 (InputQuant). */
enum { TB_QUANT_PER_TOKEN = 0, TB_QUANT_GROUP_128 = 1 };

/* The nine-field kernel configuration, in the wire order of tensorbridge/jit/codegen.py:40-49 and
 * tensorbridge/csrc/heuristics/config.hpp:28-55.  On sm_100a the fields mean:
 *   block_m            token tile (UMMA N): 16, 32, 64, 128, 192 or 256 ahead of time; other multiples of 16 (of 32 from
 *                      64 up) once tb_register_kernel has a kernel for them
 *   num_stages         depth of the weight ring (codes + scales, 9 KB a stage), rounded down to a multiple of the
 *                      bridge teams; the token ring takes what is left of shared memory, at most 8 stages
 *   use_stream_k       dense GEMM: 0 = whole tiles; 1 = the tiles of the last, partial round are shared out, two
 *                      to four CTAs with a K-block range each per tile (256-token tiles, more tiles than SMs, a
 *                      last round that fills at most half of them: the parts exchange FP32 partial sums and add
 *                      them in a fixed order; launches it does not fit run whole tiles);
 *                      2..16 = that many deterministic K splits of every tile
 *   m_fast_tile_order  bridge teams that alternate K blocks: 0/1 = one team, 2 or 4
 *   block_k            128
 *   block_n            128 (channels per unit of work = UMMA M)
 *   ctas_per_sm        1
 *   stream_k_aligned   bridged FP8 weight tiles kept in tensor memory: 2..8, as far as the 512 columns hold them
 *                      next to the accumulators (0 = default 4), rounded down to a multiple of the bridge teams
 *   math_warpgroups    bridge warps / 4: 2 (8 warps; 1 or 2 teams) or 4 (16 warps; 2 or 4 teams)
 */
typedef struct tb_config {
    int32_t block_m;
    int32_t num_stages;
    int32_t use_stream_k;
    int32_t m_fast_tile_order;
    int32_t block_k;
    int32_t block_n;
    int32_t ctas_per_sm;
    int32_t stream_k_aligned;
    int32_t math_warpgroups;
} tb_config;

/* Shape handed to the selection rule; tensorbridge/csrc/heuristics/config.hpp:12-22 (GemmDesc). */
typedef struct tb_problem {
    int64_t m;             /* rows (routed rows of a grouped layout) */
    int64_t n;             /* weight channels, unpadded */
    int64_t k;             /* reduction size, unpadded */
    int32_t num_sms;       /* SMs the launch may use */
    int32_t num_experts;   /* 0 for dense */
    int32_t layout;        /* TB_LAYOUT_* */
    int32_t group_scales;  /* 1 for [1,128] activation scales */
    int32_t split_k_override; /* -1 = rule decides, 0 = off, >0 = this many splits (dense only) */
} tb_problem;

/* Message of the last failing call on this thread ("" if none). */
const char* tb_last_error(void);

/* Library version string. */
const char* tb_version(void);

/* SM count of `device`, capped by the TENSORBRIDGE_NUM_SMS environment variable.
 * Replaces get_num_sms, tensorbridge/csrc/launcher/launcher.cpp:70-89. */
int tb_num_sms(int device, int* num_sms);

/* Shape -> configuration for the B200 device class.
 * Replaces select_config, tensorbridge/csrc/launcher/launcher.cpp:139-206 and the rule in
 * tensorbridge/csrc/heuristics/sm90_rule.hpp:333-348. */
int tb_select_config(const tb_problem* problem, tb_config* config);

/* Bytes of scratch a dense launch with `config` needs (0 for whole-tile launches, or for a block_m the library does
 * not have).  K splits (use_stream_k >= 2): a 4 KB header and one 8-byte {partial sum, tag} word per element of every
 * split.  Shared last round (use_stream_k = 1): the header and one FP32 partial tile (128 KB) per CTA, counted for up
 * to 256 SMs.  Do not hand one workspace to launches of both kinds: a partial sum left by a shared-round launch could be
 * mistaken for the tag of a later K-split launch.
 * No counterpart in the reference, whose Stream-K tail adds into the BF16 output in place. */
int64_t tb_workspace_bytes(int64_t m, int64_t n, const tb_config* config);

/* Dynamic FP8 E4M3 quantisation of `x` [m, k] (row stride `x_stride` elements):
 *   scale = max(amax, 1e-30) / 448;  per token q = rne_sat(x * (1/scale)), group-128 q = rne_sat(x / scale).
 * `q` is [m, k] contiguous; scale element (row, group) is written at scale[row * scale_stride_m +
 * group * scale_stride_k].  The kernel releases programmatic dependents at entry.
 * Replaces quantize / quantize_group_128, tensorbridge/quant/fp8.py:298-320 and :197-222. */
int tb_quantize_fp8(void* stream, const void* x, int x_dtype, int64_t x_stride, int64_t m, int64_t k, int mode,
                    void* q, float* scale, int64_t scale_stride_m, int64_t scale_stride_k);

/* Fused MoE producers: quantise rows to FP8 E4M3 with optional gated activation, row validity and scatter.
 *   value  = x[row, :width], or bf16(bf16(silu(gate)) * up) when `activation` (x is BF16 [rows, 2 * width], gate first)
 *   scale  = max(amax, 1e-30) / 448 per row (TB_QUANT_PER_TOKEN) or per 128 columns (TB_QUANT_GROUP_128)
 *   q      = rne_sat(value / scale) when `use_division`, else rne_sat(value * (1 / scale))
 *   rows   : all; or with `expert_counts` (int32 [E], capacity = rows / E) only row % capacity < counts[row / capacity];
 *            or with `num_valid_rows` (int32 [1]) only rows below it; other rows are neither read nor written
 *   output : q [out_rows, width] and scale [out_rows, groups] contiguous; a row goes to itself, or with `scatter_idx`
 *            (int32 [rows, top_k]) to every target inside [0, out_rows)
 * width <= 8192.  The kernel releases programmatic dependents at entry.
 * Replaces quantize_moe, silu_mul_quantize and scatter_quantize, tensorbridge/quant/fp8.py:225-275, :347-369, :390-413. */
typedef struct tb_quant_moe_args {
    const void* x;
    int32_t x_dtype;         /* TB_DTYPE_* (BF16 with activation) */
    int32_t mode;            /* TB_QUANT_* */
    int64_t x_stride;        /* elements between input rows */
    int64_t rows;
    int64_t width;
    int32_t activation;
    int32_t use_division;
    const int32_t* expert_counts;
    int64_t num_experts;
    const void* num_valid_rows;   /* int32 [1], or int64 [1] when num_valid_rows_int64 */
    const int32_t* scatter_idx;
    int32_t top_k;
    int32_t num_valid_rows_int64;
    int64_t out_rows;
    void* q;
    float* scale;
} tb_quant_moe_args;

int tb_quantize_moe(void* stream, const tb_quant_moe_args* args);

/* Copy FP8 rows x [rows, width] (row stride x_stride bytes) and their FP32 scales (rows x groups, by strides) to every
 * scatter target inside [0, out_rows): out [out_rows, width], out_scale [out_rows, groups] contiguous.
 * Replaces scatter_fp8, tensorbridge/quant/fp8.py:36-59. */
int tb_scatter_fp8(void* stream, const void* x, int64_t x_stride, const float* scale, int64_t scale_stride_m,
                   int64_t scale_stride_k, const int32_t* scatter_idx, int64_t rows, int32_t top_k, int64_t width,
                   int64_t groups, int64_t out_rows, void* out, float* out_scale);

/* Checkpoint NVFP4 tensors -> kernel layout, in one pass on the device.
 *   packed  uint8 [rows, k/2]  (rows = n, or E*n for stacked experts), scale raw E4M3 bytes [rows, k/16]
 *   weight  int32 [rows_pad, k_pad/8] in 128x128 block order (8192 bytes per block, layout in csrc/tb_bridge.cuh), scale_out uint8 [E, k_pad/16, n_pad]
 * Zero-pads to multiples of 128, zeroes groups whose scale byte is below 0x1C, prefolds the scale for `bridge`,
 * clamps bytes above 0x7E when `clamp_scale`, else counts them in *too_large (device int32, must be zero on
 * entry; the caller reads it back and raises).
 * Replaces prepare / prepare_experts, tensorbridge/quant/nvfp4.py:83-144 and :169-209. */
int tb_prepare_weight(void* stream, const uint8_t* packed, const uint8_t* scale, int64_t num_experts, int64_t n,
                      int64_t k, int bridge, int clamp_scale, int32_t* weight, uint8_t* scale_out,
                      int32_t* too_large);

/* Test hook: the FP8 E4M3 operand bytes the GEMM feeds the tensor core, fp8_out uint8 [rows_pad, k_pad].
 * `group_scale_layout` selects the [E, k/128, n, 8] scale layout.  Follows the reference bridge,
 * tensorbridge/include/tensorbridge/dequant/fpma.cuh:28-53. */
int tb_bridge_dump(void* stream, const int32_t* weight, const uint8_t* scale, int64_t num_experts, int64_t n_pad,
                   int64_t k_pad, int bridge, int group_scale_layout, uint8_t* fp8_out);

/* A kernel compiled at run time (NVRTC) for a point of the kernel template the library has no ahead-of-time instance
 * of -- token tiles of 48, 96, 160, 224 ... tokens, other bridge arrangements.  `function` is a CUfunction of a loaded
 * module whose entry point wraps tb::gemm_body<block_m, exact, group_scales, bridge_warps, teams> (csrc/tb_gemm.cuh) and
 * whose maximum dynamic shared memory has been raised to 227 KB; it serves every later launch on `device` whose config
 * asks for that point.  Replaces register_device_kernel / get_kernel of the reference's launcher
 * (tensorbridge/csrc/launcher/launcher.cpp:208-239, tensorbridge/jit/runtime.py:162-244). */
typedef struct tb_kernel_key {
    int32_t device;
    int32_t block_m;       /* multiple of 16 up to 256 (of 32 from 64 up) */
    int32_t exact;         /* bridge: 1 exact, 0 fpma */
    int32_t group_scales;
    int32_t bridge_warps;  /* 8 or 16 */
    int32_t teams;         /* teams of 4, 8 or 16 warps */
} tb_kernel_key;

int tb_register_kernel(const tb_kernel_key* key, void* function);

/* Number of kernels registered so far. */
int tb_registered_kernels(void);

#define TB_PDL_STATIC_WEIGHTS 2

/* Arguments shared by the dense and grouped launches. */
typedef struct tb_gemm_args {
    const void* a;          /* FP8 E4M3 [rows, k], contiguous */
    const float* a_scale;   /* FP32; element (row, group) at a_scale[row * a_scale_stride_m + group * a_scale_stride_k] */
    int64_t a_scale_stride_m;
    int64_t a_scale_stride_k;
    const int32_t* weight;  /* prepared codes, [E,] n_pad x k_pad/8 */
    const uint8_t* scale;   /* prepared scales: [E,] k_pad/16 x n_pad, or [E,] k_pad/128 x n_pad x 8 with group scales */
    const float* global_scale; /* FP32 [max(E,1)], already times 6 */
    int32_t* locks;         /* the reference's int32 [1024] lock tensor; kept in the signature, not used on sm_100a
                             * (the K-split reduction needs no counters), may be NULL */
    float* workspace;       /* scratch of tb_workspace_bytes() for K splits, 8-byte aligned, or NULL when the config has
                             * none.  Zero it once after allocating it and leave its first 4 KB alone afterwards: they
                             * hold the launch sequence number that tells this launch's partial sums from older ones
                             * (kept on the device, so CUDA-graph replays number themselves too).  Launches that can
                             * overlap need separate workspaces. */
    int64_t workspace_bytes;
    void* d;                /* BF16 [out_rows, n] contiguous */
    int64_t rows;           /* rows of `a` */
    int64_t n;              /* unpadded channels */
    int64_t k;              /* unpadded reduction size */
    int32_t bridge;         /* TB_BRIDGE_* */
    int32_t group_scales;   /* 1: [1,128] activation scales */
    int32_t enable_pdl;     /* 0: plain launch; 1: programmatic stream serialisation; 2 (TB_PDL_STATIC_WEIGHTS): the same,
                             * and no kernel still in flight on the stream writes weight / scale, so a dense launch may
                             * stream them before the previous kernel has finished */
    int32_t num_sms;        /* 0 = all SMs of the device (after TENSORBRIDGE_NUM_SMS) */
    int32_t* status;        /* device int32 [4] the kernel writes on a timed-out wait, or NULL */
    int32_t wait_us;        /* budget of every wait inside the kernel in microseconds (counted at 2 GHz); 0 = about a
                             * second.  A wait that runs out makes the kernel return early and write `status`. */
    int32_t only_split;     /* test hook, dense K splits only: s + 1 runs just the units of split s, so that its peers'
                             * partial sums never arrive and its bounded wait runs out; 0 = all units (normal use) */
    const int32_t* row_target; /* grouped masked / contiguous launches of an expert-parallel step, else NULL: int32 [rows],
                             * row r of `a` belongs to route (row_target[r] & 0x3FFFFFF) of rank (row_target[r] >> 26), -1 =
                             * nobody's; the epilogue then stores the row's output straight into that rank's buffer
                             * peer_out[rank] (row stride n elements; plain stores over NVLink) instead of `d` */
    void* const* peer_out;  /* host array of peer_count device pointers (every rank's BF16 route buffer, as mapped here) */
    int32_t peer_count;     /* 1..16 */
    int32_t reserved;
} tb_gemm_args;

/* D[m, n] = bf16((A @ bridge(W).T) * a_scale * global_scale).
 * Replaces launch_kernel, tensorbridge/csrc/launcher/launcher.cpp:464-469 (body :241-462). */
int tb_gemm_dense(void* stream, const tb_gemm_args* args, const tb_config* config);

/* tb_gemm_dense for callers that have no way to provide split-K scratch: `args->workspace` is ignored and the FP32
 * partial sums go to an 8 MiB array that is part of the library's device image.  It exists for hosts that must not
 * touch the CUDA allocator once they are running -- a serving engine that has already handed all free HBM to its own
 * pools, a C or ctypes caller with no tensor library at hand, code inside a region where cudaMalloc would
 * synchronise the device -- and that still want the K-split kernel for small M.  This function and everything it
 * calls performs no cudaMalloc, cudaFree or other allocating call.
 *   - A launch whose K splits need more than 8 MiB (tb_workspace_bytes(rows, n, config) > 8 << 20) is rejected with
 *     TB_ERR_INVALID and a message that states both sizes.  The size is that of the splits the launch really makes
 *     (at most one per 128 of K, none with [1,128] scales): launches without a K split need no scratch and always pass.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current).  Make that first call outside any CUDA stream capture; later calls only launch.
 *   - All calls on a device share the one array and it keeps whatever the last launch left there: it starts zeroed
 *     (static storage), its first 4 KB hold the launch sequence number and every partial sum carries the tag of its launch.  Two
 *     launches that may run at the same time on one device (different streams) would overwrite each other's partial
 *     sums: serialise them, or use tb_gemm_dense with one workspace per stream.
 * The inputs, the output and `status` are still the caller's, exactly as for tb_gemm_dense.
 * It has no counterpart in the reference, whose Stream-K tail accumulates into the BF16 output itself. */
int tb_gemm_dense_static_scratch(void* stream, const tb_gemm_args* args, const tb_config* config);

/* Routing of a grouped launch (device pointers; unused ones NULL).  tensorbridge/gemm.py:46-73. */
typedef struct tb_routing {
    int32_t layout;                  /* TB_LAYOUT_INDEXED / CONTIGUOUS / MASKED */
    int32_t num_experts;
    const int64_t* expert_offsets;   /* contiguous: int64 [E + 1] */
    const int32_t* expert_counts;    /* masked: int32 [E]; capacity = rows / E */
    const int32_t* sorted_ids;       /* indexed: int32 [sorted_capacity] route ids, padding >= rows * top_k */
    const int32_t* expert_ids;       /* indexed: int32, one per block_m block */
    const int32_t* num_tokens_padded;/* indexed: int32 [1] */
    int64_t sorted_capacity;         /* indexed: numel of sorted_ids */
    int32_t top_k;                   /* indexed: route r reads row r / top_k and writes output row r */
    void* gather_scratch;            /* indexed, optional: caller-owned bytes [sorted_capacity * k]; when given, the rows
                                        are gathered into it by a first kernel and the GEMM loads whole tiles by TMA */
    int64_t gather_scratch_bytes;
} tb_routing;

/* One launch over all experts; no K split, static tile order, run-to-run bit-identical.
 * Replaces launch_grouped_kernel, tensorbridge/csrc/launcher/launcher.cpp:471-478. */
int tb_gemm_grouped(void* stream, const tb_gemm_args* args, const tb_routing* routing, const tb_config* config);

/* ---- Expert-parallel token dispatch around the masked grouped GEMM (one process per GPU) ------------------------
 * The reference has no counterpart for these five: it is handed expert-parallel shapes already dispatched by the
 * serving framework (tensorbridge/vllm_moe.py:130-132).  They are the integer bookkeeping and the row movement on
 * either side of the all-to-all exchange; the exchange itself (NCCL) stays with the caller.  World size W, E experts
 * in all, E / W per rank; "placed" expert index = owner rank * (E / W) + local index, with owner = e / (E / W)
 * (contiguous placement) or e % W (interleaved). */

/* Routes of this rank -> send plan.  `topk_ids` int32 or int64 [routes] (route = token * top_k + slot; ids outside
 * [0, E) are not sent); send_counts int32 [E] in placed order = [W][E / W]; send_pos int32 [routes] = row of the route
 * in the send buffer, ordered by destination rank, then local expert, then route id (-1 = not sent); route_rank int32
 * [routes] = rank of the route among this rank's routes to the same expert, in route order (either output may be
 * NULL).  E <= 1024. */
int tb_ep_plan(void* stream, const void* topk_ids, int ids_int64, int64_t routes, int32_t num_experts, int32_t world,
               int32_t interleaved, int32_t* send_counts, int32_t* send_pos, int32_t* route_rank);

/* send[send_pos[r]] = { x[r / top_k] (width bytes of FP8), scale[r / top_k] (groups floats) } in rows of `row_bytes`
 * (a multiple of 16, >= width + 4 * groups; width a multiple of 16): one exchange carries rows and scales. */
int tb_ep_pack(void* stream, const void* x, const float* scale, const int32_t* send_pos, int64_t routes, int32_t top_k,
               int64_t width, int64_t groups, int64_t row_bytes, void* send);

/* recv_counts int32 [W][E / W] (rows received from every source rank for every local expert) -> seg_start and seg_dest
 * int32 [W * E / W] (first row of every (source, expert) run in the receive buffer, and the masked-buffer row its
 * first row goes to: expert * capacity + rows of earlier sources), counts int32 [E / W] = min(capacity, rows). */
int tb_ep_layout(void* stream, const int32_t* recv_counts, int32_t world, int32_t experts_local, int32_t capacity,
                 int32_t* seg_start, int32_t* seg_dest, int32_t* counts);

/* Received packed rows -> masked activation buffer a [E / W * capacity, width] and a_scale [E / W * capacity, groups];
 * recv_rows int32 [rows] = destination row of every received row, -1 for rows past their expert's capacity. */
int tb_ep_place(void* stream, const void* recv, int64_t rows, int64_t row_bytes, int64_t width, int64_t groups,
                const int32_t* seg_start, const int32_t* seg_dest, int32_t world, int32_t experts_local, int32_t capacity,
                void* a, float* a_scale, int32_t* recv_rows);

/* dst[i] = index[i] >= 0 ? src[index[i]] : zeros, rows of `row_bytes` bytes (a multiple of 16). */
int tb_gather_rows(void* stream, const void* src, const int32_t* index, int64_t rows, int64_t row_bytes, void* dst);

/* out[t, :] = bf16(sum_j weights[t, j] * rows[index[t * top_k + j], :]) over BF16 rows of `width` channels (a multiple
 * of 8; FP32 sums in slot order, so the result repeats from run to run).  `index` NULL: route t * top_k + j reads row
 * t * top_k + j (the route-ordered output of an indexed grouped GEMM); a negative index adds nothing (a route whose
 * expert lives on another rank).  `weights` FP32 [tokens, top_k].
 * Stands in for the two vLLM helpers the reference calls after its down projection, moe_fused_mul_sum (indexed) and
 * moe_unpermute (contiguous): tensorbridge/vllm_moe.py:377-379 and :407. */
int tb_moe_combine(void* stream, const void* rows, const int32_t* index, const float* weights, int64_t tokens, int32_t top_k,
                   int64_t width, void* out);

/* ---- The same dispatch over peer memory: NVLink loads and stores between the GPUs of one node, no collective library,
 * no host read, no staging copy.  No counterpart in the reference (its overlap.py streams tokens into a masked buffer
 * from one producer on the same GPU, tensorbridge/overlap.py:110-180).  Every rank owns, in memory its peers have
 * mapped: the masked activation buffer a [E/W * capacity, width] and a_scale [E/W * capacity, groups], the output
 * buffer y [E/W * capacity, n], a count matrix int32 [W][E] and W arrival flags (uint32, zero at start).  One step:
 *   tb_ep_plan (route_rank, send_counts) -> tb_peer_barrier carrying send_counts into row `rank` of every peer's count
 *   matrix -> tb_ep_push -> tb_peer_barrier -> tb_gemm_grouped (masked) into y -> tb_peer_barrier -> tb_ep_pull;
 *   or, with the combine fused into the GEMM's epilogue: ... tb_ep_push (also fills the owners' row_target tables) ->
 *   tb_peer_barrier -> tb_gemm_grouped with row_target / peer_out (every output row is stored into the buffer of the rank
 *   its route came from) -> tb_peer_barrier.
 * Only plain loads and stores cross NVLink (no TMA on peer memory, no multicast). */

/* Set-up helpers for that memory.  These four are the only entry points of the library that allocate, free or map
 * memory; none of them belongs on a hot path.  tb_peer_alloc returns zeroed device memory from cudaMalloc (the kind
 * cudaIpcGetMemHandle accepts); a handle is 64 bytes; tb_ipc_open maps a peer's allocation into this process with the
 * current device as the accessing device (peer access is enabled on first use). */
int tb_peer_alloc(int64_t bytes, void** ptr);
int tb_peer_free(void* ptr);
int tb_ipc_export(const void* ptr, uint8_t* handle);
int tb_ipc_open(const uint8_t* handle, void** ptr);
int tb_ipc_close(void* ptr);

/* Barrier between the ranks' streams on the flags above (flags[p] = rank p's flag array, as mapped here), optionally
 * copying `count` ints from `payload` to row `rank` of every peer's [W][count] matrix payload_dst[p] first.  Every rank
 * calls it the same number of times; `local_epoch` (device uint32, zero at start, this rank's own) counts them.  A wait
 * that lasts longer than `wait_us` microseconds (0 = about a second) ends the kernel with 100 + the missing peer in
 * status[0].  Kernels of different ranks wait for one another here: every rank must run on a GPU of its own. */
int tb_peer_barrier(void* stream, void* const* flags, void* const* payload_dst, const int32_t* payload, int32_t count,
                    int32_t rank, int32_t world, uint32_t* local_epoch, int32_t wait_us, int32_t* status);

/* Writes every route's FP8 row and scales into the masked buffer of the rank that owns its expert: row = local expert
 * * capacity + routes of lower ranks for that expert + route_rank; routes past the capacity are not sent.  dest_row
 * int32 [routes] receives the row (-1 = not sent); counts int32 [E/W] the rows of this rank's own experts, clamped. */
typedef struct tb_ep_push_args {
    const void* topk_ids;      /* int32 or int64 [routes] */
    int32_t ids_int64;
    int32_t top_k;
    int64_t routes;
    const void* x;             /* FP8 [routes / top_k, width] */
    const float* scale;        /* FP32 [routes / top_k, groups] */
    int64_t width;
    int64_t groups;
    const int32_t* route_rank; /* from tb_ep_plan */
    const int32_t* all_counts; /* this rank's count matrix [W][E], filled by the barrier before */
    int32_t num_experts;
    int32_t world;
    int32_t rank;
    int32_t interleaved;
    int32_t capacity;
    int32_t reserved;
    void* const* peer_a;       /* host array of W device pointers: every rank's masked activation buffer */
    void* const* peer_a_scale; /* ... and scale buffer */
    int32_t* dest_row;
    int32_t* counts;
    void* const* peer_row_target; /* optional: every rank's int32 [E/W * capacity] table; the row a route lands in gets
                                   * (rank << 26 | route), which tb_gemm_grouped takes as row_target to return the row's
                                   * output to this rank without a combine pass */
    void* out;                 /* optional, with peer_row_target: this rank's route buffer [routes, out_row_bytes]; the
                                * rows of routes that were not sent are cleared here */
    int64_t out_row_bytes;     /* multiple of 16 */
} tb_ep_push_args;

int tb_ep_push(void* stream, const tb_ep_push_args* args);

/* out[r] = dest_row[r] >= 0 ? (owner of route r).y[dest_row[r]] : zeros; rows of `row_bytes` bytes (multiple of 16). */
int tb_ep_pull(void* stream, const void* topk_ids, int ids_int64, const int32_t* dest_row, int64_t routes, int32_t num_experts,
               int32_t world, int32_t interleaved, void* const* peer_y, int64_t row_bytes, void* out);

#ifdef __cplusplus
}
#endif
#endif /* TENSORBRIDGE_B200_H_ */
