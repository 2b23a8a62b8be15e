// Host side of libtensorbridge_b200.so: argument validation, tensor maps, the B200 selection rule and the launches.
// The C ABI is declared in include/tensorbridge_b200.h.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/tensorbridge_b200.h"
#include "tb_aux.cuh"
#include "tb_launch.cuh"

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

}  // namespace

namespace tb {
// For the other translation units of the library: records the message tb_last_error() returns on this thread.
int set_last_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}
}  // namespace tb

namespace {

#define TB_CUDA(expr)                                                                                  \
    do {                                                                                               \
        cudaError_t err__ = (expr);                                                                    \
        if (err__ != cudaSuccess) return fail(TB_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(err__)); \
    } while (0)

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) != cudaSuccess ||
            status != cudaDriverEntryPointSuccess) {
            return static_cast<EncodeTiled>(nullptr);
        }
        return reinterpret_cast<EncodeTiled>(ptr);
    }();
    return fn;
}

// uint8 matrix [rows, cols] with `row_stride` bytes between rows; box = box_cols x box_rows.
int make_map_u8(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint64_t row_stride, uint32_t box_cols,
                uint32_t box_rows, CUtensorMapSwizzle swizzle) {
    EncodeTiled fn = encode_tiled();
    if (fn == nullptr) return fail(TB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {row_stride};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult res = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) return fail(TB_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", static_cast<int>(res));
    return TB_OK;
}

// Encoding a tensor map costs a driver call of a microsecond or two, and a layer meets the same few (buffer, shape, tile)
// combinations over and over.  The encoded bytes are a pure function of the arguments, so a small direct-mapped cache
// per thread returns them without the call.
struct MapKey {
    const void* base;
    uint64_t cols, rows, row_stride;
    uint32_t box_cols, box_rows;
    int swizzle;
    bool operator==(const MapKey& o) const {
        return base == o.base && cols == o.cols && rows == o.rows && row_stride == o.row_stride && box_cols == o.box_cols &&
               box_rows == o.box_rows && swizzle == o.swizzle;
    }
};

int cached_map_u8(CUtensorMap* map, const void* base, uint64_t cols, uint64_t rows, uint64_t row_stride, uint32_t box_cols,
                  uint32_t box_rows, CUtensorMapSwizzle swizzle) {
    constexpr int kEntries = 256;
    struct Entry { MapKey key; CUtensorMap map; bool used; };
    thread_local Entry* table = nullptr;
    if (table == nullptr) table = new Entry[kEntries]();
    const MapKey key = {base, cols, rows, row_stride, box_cols, box_rows, static_cast<int>(swizzle)};
    uint64_t h = reinterpret_cast<uintptr_t>(base) >> 8;
    h = (h ^ (rows * 0x9E3779B97F4A7C15ull) ^ (cols << 17) ^ (static_cast<uint64_t>(box_rows) << 40) ^ static_cast<uint64_t>(swizzle)) * 0xD6E8FEB86659FD93ull;
    Entry& e = table[(h >> 32) % kEntries];
    if (e.used && e.key == key) {
        *map = e.map;
        return TB_OK;
    }
    if (int rc = make_map_u8(map, base, cols, rows, row_stride, box_cols, box_rows, swizzle)) return rc;
    e.key = key;
    e.map = *map;
    e.used = true;
    return TB_OK;
}

struct DeviceInfo {
    int num_sms = 0;
    int smem_optin = 0;
};

int device_info(int device, DeviceInfo* out) {
    static std::mutex mutex;
    static DeviceInfo cache[64];
    if (device < 0 || device >= 64) return fail(TB_ERR_INVALID, "device %d out of range", device);
    std::lock_guard<std::mutex> guard(mutex);
    if (cache[device].num_sms == 0) {
        TB_CUDA(cudaDeviceGetAttribute(&cache[device].num_sms, cudaDevAttrMultiProcessorCount, device));
        TB_CUDA(cudaDeviceGetAttribute(&cache[device].smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
    }
    *out = cache[device];
    return TB_OK;
}

int env_sm_cap() {
    const char* env = std::getenv("TENSORBRIDGE_NUM_SMS");
    if (env == nullptr || *env == '\0') return 0;
    const int value = std::atoi(env);
    return value > 0 ? value : 0;
}

constexpr int kB200Sms = 148;
constexpr int kSmemBudget = 227 * 1024;  // dynamic shared memory per CTA on sm_100

int ceil_div(long long a, long long b) { return static_cast<int>((a + b - 1) / b); }
int pad128(long long x) { return ceil_div(x, 128) * 128; }

bool valid_block_m(int bm) { return bm == 16 || bm == 32 || bm == 64 || bm == 128 || bm == 192 || bm == 256; }

// Bytes left for the two rings once barriers, staging and routing tables are placed.
int ring_room(int bm, int num_experts, bool group_scales) {
    return kSmemBudget - 1024 - static_cast<int>(tb::smem_layout(bm, 0, 0, num_experts, group_scales).total);
}

// Token ring depth that goes with a weight ring of `w_stages`: what is left, at most 8.
int token_stages_for(int bm, int w_stages, int num_experts, bool group_scales) {
    const int room = ring_room(bm, num_experts, group_scales) - w_stages * (tb::kBlockBytes + tb::kBlockScaleBytes);
    return std::min(room / (bm * 128), 8);
}

// Weight ring depth of the rule: leave the token ring 8 stages for small token tiles, 6 at 128 and 5 at 256 tokens.
int pick_weight_stages(int bm, int num_experts, bool group_scales) {
    const int token_stages = bm <= 64 ? 8 : (bm == 128 ? 6 : 5);
    const int room = ring_room(bm, num_experts, group_scales) - token_stages * bm * 128;
    const int fit = std::min(room / (tb::kBlockBytes + tb::kBlockScaleBytes), tb::kMaxRawStages);
    return std::max(4, fit / 4 * 4);  // a multiple of every team count (1, 2, 4): see the ring rule in run_gemm
}

// The B200 rule.  Small M is bound by the HBM weight stream: one token tile that covers M, and K splits until the
// 148 SMs all stream weights.  Large M takes the widest token tile (256), which amortises each bridged weight block
// over the most tensor-core work.  Grouped calls size the tile by the mean rows per expert and never split K.
int rule(const tb_problem& pr, tb_config* cfg) {
    if (pr.m < 0 || pr.n <= 0 || pr.k <= 0) return fail(TB_ERR_INVALID, "no config runs (M, N, K) = (%lld, %lld, %lld)",
                                                        (long long)pr.m, (long long)pr.n, (long long)pr.k);
    const int sms = pr.num_sms > 0 ? pr.num_sms : kB200Sms;
    const int n_tiles = pad128(pr.n) / 128, k_blocks = pad128(pr.k) / 128;
    // Group scales keep one FP32 total per column in registers: 64 a lane on the 128-token tile, which the instance
    // affords by moving registers from its bridge warps to its epilogue warps (tb_gemm.cuh, rebalances_registers).
    const int max_bm = pr.group_scales ? 128 : 256;
    int bm;
    int splits = 1;
    if (pr.layout == TB_LAYOUT_DENSE) {
        const long long m = std::max<long long>(pr.m, 1);
        const int one_tile_limit = pr.group_scales ? max_bm : 192;
        if (m <= one_tile_limit) {
            // One token tile that covers M (and K splits below); 192 tokens above 128.  With per-token scales a
            // 32-token tile gives way to the 64-token one, whose eight epilogue warps share the split-K reduction
            // (measured 13.5 against 15.0 us at M = 32).
            bm = 16;
            while (bm < m) bm *= 2;
            if (bm == 256) bm = 192;
            if (bm == 32 && !pr.group_scales && pr.split_k_override != 0 && pad128(pr.n) / 128 * 2 <= sms) bm = 64;
        } else if (pr.group_scales) {
            bm = max_bm;
        } else {
            // Above one tile every 128 x 128 weight block is bridged once per token tile, so wide tiles win; which of
            // 128 / 192 (two accumulator sets, the epilogue overlaps the next tile) / 256 tokens (one set, fewest
            // bridge passes) is decided by how evenly the tiles fill the SMs: waves x (tile width + fixed cost per
            // tile).  At N = 6144, K = 7168 this reproduces the measured winners: 128 up to M = 384, 192 at 512 and
            // 1024, 256 at 768, 1536 and from 2048 on.
            long long best = 0;
            bm = 256;
            for (int cand : {256, 192, 128}) {
                const long long waves = ceil_div(static_cast<long long>(ceil_div(m, cand)) * n_tiles, sms);
                const long long cost = waves * (cand + 64);
                if (best == 0 || cost < best) { best = cost; bm = cand; }
            }
        }
        const int tiles = ceil_div(m, bm) * n_tiles;
        if (pr.split_k_override > 0) {
            splits = pr.split_k_override;
        } else if (pr.split_k_override < 0 && !pr.group_scales && tiles * 2 <= sms) {
            // Splits until the SMs are full pay only while there are enough tiles: the reducing split polls its peers
            // one after the other, so with few tiles (narrow weights, e.g. column-parallel shards) about 48 CTAs in
            // all are the optimum (measured at K = 7168: 48 tiles -> 3 splits, 24 -> 3, 12 -> 4..6, 6 -> 8).
            splits = std::min(sms / tiles, std::max(3, 48 / tiles));
        }
        splits = std::max(1, std::min({splits, k_blocks / 2 > 0 ? k_blocks / 2 : 1, 16}));
        if (tiles > 128 || pr.group_scales) splits = 1;
        // Sharing the tiles of the last, partial round among the CTAs (use_stream_k = 1) is never picked: it measures
        // the same as whole tiles (N = 6144, K = 7168: 283 against 282 us at M = 8192, 148 against 147 at 4096, 46
        // against 45 at 1024).  These launches run under the power cap, where the few SMs of a partial last round clock
        // higher while the others idle, so filling the round buys no time.  The path stays for callers that ask for it.
    } else {
        // Routed rows are uneven across experts: a tile of twice the mean rows (at least 32) keeps the busy experts to
        // one or two token tiles, so their weights stream from HBM once; the extra columns cost next to nothing while
        // the call is weight bound.
        const int experts = std::max(pr.num_experts, 1);
        const long long mean = std::max<long long>((pr.m + experts - 1) / experts, 1);
        bm = 32;
        while (bm < 2 * mean && bm < max_bm) bm *= 2;
    }
    // Bridge warps, measured on B200 (dense N = 6144, K = 7168; the MoE shapes of DeepSeek-V3): 16 warps in four teams
    // where the bridge is the longest stage -- the smallest dense token tile, unsplit launches of 128 tokens and more and grouped
    // launches (masked decode: 116 against 138 us) -- and 8 warps in two teams for split-K tiles of 32 to 256 tokens
    // and for group scales, whose epilogues need the registers that 864 threads would not leave them (contiguous
    // group-scale prefill: 1.08 against 1.69 ms).  Four bridged tiles in tensor memory.
    const int dense_tiles = pr.layout == TB_LAYOUT_DENSE ? ceil_div(std::max<long long>(pr.m, 1), bm) * n_tiles : 0;
    const bool wide_bridge = !pr.group_scales && (pr.layout != TB_LAYOUT_DENSE || (bm <= 16 && dense_tiles >= 32) || (splits == 1 && bm >= 128));
    // Eight bridged tiles where two teams feed a split-K tile (measured better on the narrow shapes, equal elsewhere).
    const int bridged = std::min((!wide_bridge && splits > 1 && bm <= 128) ? 8 : 4, tb::max_bridged_stages(bm, pr.group_scales != 0));
    cfg->block_m = bm;
    cfg->num_stages = pick_weight_stages(bm, pr.layout == TB_LAYOUT_DENSE ? 0 : pr.num_experts, pr.group_scales != 0);
    cfg->use_stream_k = splits > 1 ? splits : 0;
    cfg->m_fast_tile_order = wide_bridge ? 4 : 2;
    cfg->block_k = 128;
    cfg->block_n = 128;
    cfg->ctas_per_sm = 1;
    cfg->stream_k_aligned = bridged;
    cfg->math_warpgroups = wide_bridge ? 4 : 2;
    return TB_OK;
}

// Bytes of K-split scratch: the header words, then one 8-byte {partial sum, tag} word per element of every split.
// Workspace of a balanced launch of `ctas` CTAs: the header, then one partial tile per CTA.
long long balanced_scratch_bytes(int ctas) {
    return tb::kEpochCells * 4 + static_cast<long long>(ctas) * tb::kBalancedTileWords * 4;
}

long long split_scratch_bytes(long long m, long long n, int block_m, int splits) {
    const long long tiles = static_cast<long long>(ceil_div(m, block_m)) * (pad128(n) / 128);
    return tb::kEpochCells * 4 + tiles * splits * block_m * 128 * 8;
}

// ---- kernels compiled at run time (tensorbridge/jit) ----------------------------------------------------------------
// The ahead-of-time instances cover six token tiles and three bridge arrangements.  Any other point of the template
// (token tiles of 48, 96, 160, 224 ... tokens, 16 bridge warps in two teams, ...) is compiled by NVRTC on the Python side
// and handed over as a CUfunction; a registered function takes precedence over an ahead-of-time instance of the same key.
struct KernelKey {
    int device, block_m, exact, group_scales, bridge_warps, teams;
    bool operator==(const KernelKey& o) const {
        return device == o.device && block_m == o.block_m && exact == o.exact && group_scales == o.group_scales &&
               bridge_warps == o.bridge_warps && teams == o.teams;
    }
};
struct RegisteredKernel { KernelKey key; CUfunction function; };
std::mutex g_registry_mutex;
RegisteredKernel g_registry[256];
int g_registered = 0;

CUfunction find_registered(const KernelKey& key) {
    std::lock_guard<std::mutex> guard(g_registry_mutex);
    for (int i = 0; i < g_registered; ++i)
        if (g_registry[i].key == key) return g_registry[i].function;
    return nullptr;
}

bool jit_block_m(int bm) { return bm >= 16 && bm <= 256 && bm % 16 == 0 && (bm < 64 || bm % 32 == 0); }

using LaunchKernelEx = CUresult (*)(const CUlaunchConfig*, CUfunction, void**, void**);
LaunchKernelEx launch_kernel_ex() {
    static LaunchKernelEx fn = [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuLaunchKernelEx", &ptr, cudaEnableDefault, &status) != cudaSuccess ||
            status != cudaDriverEntryPointSuccess) {
            return static_cast<LaunchKernelEx>(nullptr);
        }
        return reinterpret_cast<LaunchKernelEx>(ptr);
    }();
    return fn;
}

int launch_registered(CUfunction function, int threads, cudaStream_t stream, const tb::GemmParams& params, int grid, size_t smem,
                      bool pdl) {
    LaunchKernelEx fn = launch_kernel_ex();
    if (fn == nullptr) return fail(TB_ERR_CUDA, "cuLaunchKernelEx is not available from the driver");
    CUlaunchConfig cfg = {};
    cfg.gridDimX = static_cast<unsigned>(grid); cfg.gridDimY = 1; cfg.gridDimZ = 1;
    cfg.blockDimX = static_cast<unsigned>(threads); cfg.blockDimY = 1; cfg.blockDimZ = 1;
    cfg.sharedMemBytes = static_cast<unsigned>(smem);
    cfg.hStream = stream;
    CUlaunchAttribute attr[1];
    attr[0].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
    attr[0].value.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    void* args[1] = {const_cast<tb::GemmParams*>(&params)};
    const CUresult res = fn(&cfg, function, args, nullptr);
    if (res != CUDA_SUCCESS) return fail(TB_ERR_CUDA, "cuLaunchKernelEx of a run-time compiled kernel failed with %d", static_cast<int>(res));
    return TB_OK;
}

int run_gemm(cudaStream_t stream, const tb_gemm_args* a, const tb_routing* routing, const tb_config* cfg) {
    if (a == nullptr || cfg == nullptr) return fail(TB_ERR_INVALID, "null arguments");
    if (a->rows < 0 || a->n <= 0 || a->k <= 0) return fail(TB_ERR_INVALID, "bad shape rows=%lld n=%lld k=%lld",
                                                          (long long)a->rows, (long long)a->n, (long long)a->k);
    if (a->rows == 0) return TB_OK;  // nothing to do, as the reference returns before launching
    if (a->a == nullptr || a->a_scale == nullptr || a->weight == nullptr || a->scale == nullptr ||
        a->global_scale == nullptr || a->d == nullptr) return fail(TB_ERR_INVALID, "null tensor pointer");
    if (a->k % 16 != 0) return fail(TB_ERR_INVALID, "K must be a multiple of 16, got %lld", (long long)a->k);
    if (reinterpret_cast<uintptr_t>(a->a) % 16 != 0 || reinterpret_cast<uintptr_t>(a->weight) % 16 != 0 ||
        reinterpret_cast<uintptr_t>(a->scale) % 16 != 0) return fail(TB_ERR_INVALID, "a, weight and scale must be 16-byte aligned");
    if (a->rows > 0x7FFFFFFFll / 2) return fail(TB_ERR_INVALID, "too many rows");
    const int bm = cfg->block_m;
    if (!valid_block_m(bm) && !jit_block_m(bm))
        return fail(TB_ERR_INVALID, "block_m must be 16, 32, 64, 128, 192 or 256 (or, with a kernel compiled at run time, another "
                    "multiple of 16 up to 256: of 32 from 64 up), got %d", bm);
    if (cfg->block_n != 128 || cfg->block_k != 128) return fail(TB_ERR_INVALID, "block_n and block_k must be 128");
    if (cfg->ctas_per_sm != 0 && cfg->ctas_per_sm != 1) return fail(TB_ERR_INVALID, "ctas_per_sm must be 1, got %d", cfg->ctas_per_sm);

    const int layout = routing == nullptr ? TB_LAYOUT_DENSE : routing->layout;
    const int experts = routing == nullptr ? 0 : routing->num_experts;
    if (routing != nullptr) {
        if (experts <= 0 || experts > tb::kMaxExperts) return fail(TB_ERR_INVALID, "num_experts must be in 1..%d", tb::kMaxExperts);
        if (layout == TB_LAYOUT_CONTIGUOUS && routing->expert_offsets == nullptr) return fail(TB_ERR_INVALID, "contiguous routing needs expert_offsets");
        if (layout == TB_LAYOUT_MASKED) {
            if (routing->expert_counts == nullptr) return fail(TB_ERR_INVALID, "masked routing needs expert_counts");
            if (a->rows % experts != 0) return fail(TB_ERR_INVALID, "masked activation rows must divide into equal expert capacities");
        }
        if (layout == TB_LAYOUT_INDEXED) {
            if (routing->sorted_ids == nullptr || routing->expert_ids == nullptr || routing->num_tokens_padded == nullptr)
                return fail(TB_ERR_INVALID, "indexed routing needs IDs and padded count");
            if (routing->top_k < 1) return fail(TB_ERR_INVALID, "top_k must be positive");
            if (a->n % 128 != 0 || a->k % 128 != 0) return fail(TB_ERR_INVALID, "grouped N and K must be multiples of 128");
        }
        if (layout != TB_LAYOUT_INDEXED && layout != TB_LAYOUT_CONTIGUOUS && layout != TB_LAYOUT_MASKED)
            return fail(TB_ERR_INVALID, "unknown grouped layout %d", layout);
        if (cfg->use_stream_k > 1) return fail(TB_ERR_INVALID, "grouped GEMM does not split K");
    }

    int device = 0;
    TB_CUDA(cudaGetDevice(&device));
    DeviceInfo info;
    if (int rc = device_info(device, &info)) return rc;
    int sms = info.num_sms;
    if (int cap = env_sm_cap()) sms = std::min(sms, cap);
    if (a->num_sms > 0) sms = std::min(sms, static_cast<int>(a->num_sms));

    tb::GemmParams p;
    std::memset(&p, 0, sizeof(p));
    p.a = static_cast<const uint8_t*>(a->a);
    p.a_scale = a->a_scale;
    p.a_scale_stride_m = a->a_scale_stride_m;
    p.a_scale_stride_k = a->a_scale_stride_k;
    p.weight = reinterpret_cast<const uint8_t*>(a->weight);
    p.scale = a->scale;
    p.global_scale = a->global_scale;
    p.locks = a->locks;
    p.workspace = a->workspace;
    p.d = static_cast<__nv_bfloat16*>(a->d);
    p.rows = a->rows;
    p.n = static_cast<int>(a->n);
    p.k = static_cast<int>(a->k);
    p.n_pad = pad128(a->n);
    p.k_pad = pad128(a->k);
    p.n_tiles = p.n_pad / 128;
    p.k_blocks = p.k_pad / 128;
    p.layout = layout;
    p.num_experts = experts;
    p.top_k = routing != nullptr && layout == TB_LAYOUT_INDEXED ? routing->top_k : 1;
    p.status = a->status;
    if (a->row_target != nullptr) {
        if (layout != TB_LAYOUT_MASKED && layout != TB_LAYOUT_CONTIGUOUS)
            return fail(TB_ERR_INVALID, "row_target (output rows scattered to the ranks' buffers) goes with masked or contiguous routing");
        if (a->peer_out == nullptr || a->peer_count < 1 || a->peer_count > tb::kMaxOutputPeers)
            return fail(TB_ERR_INVALID, "row_target needs peer_out with 1..%d pointers", tb::kMaxOutputPeers);
        if (a->n % 8 != 0) return fail(TB_ERR_INVALID, "scattered output rows need N to be a multiple of 8");
        p.row_target = a->row_target;
        for (int i = 0; i < a->peer_count; ++i) {
            if (a->peer_out[i] == nullptr || reinterpret_cast<uintptr_t>(a->peer_out[i]) % 16 != 0)
                return fail(TB_ERR_INVALID, "peer_out[%d] must be a 16-byte aligned device pointer", i);
            p.peer_out[i] = static_cast<__nv_bfloat16*>(a->peer_out[i]);
        }
    }
    // Wait budget in SM cycles: the default is about a second; `wait_us` counts at 2 GHz (the clock tops out below).
    p.wait_cycles = a->wait_us > 0 ? static_cast<long long>(a->wait_us) * 2000 : tb::kWaitCycles;
    if (a->only_split < 0) return fail(TB_ERR_INVALID, "only_split must not be negative");
    const int max_bridged = tb::max_bridged_stages(bm, a->group_scales != 0);
    p.bridged_stages = cfg->stream_k_aligned > 0 ? cfg->stream_k_aligned : std::min(4, max_bridged);
    if (p.bridged_stages < 2 || p.bridged_stages > max_bridged)
        return fail(TB_ERR_INVALID, "stream_k_aligned (bridged tiles in tensor memory) must be in 2..%d for block_m %d, got %d",
                    max_bridged, bm, p.bridged_stages);
    p.w_stages = cfg->num_stages;
    if (p.w_stages < 2 || p.w_stages > tb::kMaxRawStages) return fail(TB_ERR_INVALID, "num_stages must be in 2..%d", tb::kMaxRawStages);
    // A stage of the weight ring and of the bridged ring must always meet the same bridge team: a team that visited a
    // stage only every other pass would be two mbarrier phases away from its last look, and a one-bit parity wait
    // cannot tell "two phases ago" from "now": it passes early, reads a stage that is being refilled and arrives once
    // too often.  (Seen as rare "unspecified launch failure"s of grouped launches with 6 weight stages and 4 teams.)
    // Ring depths are therefore rounded down to multiples of the team count.
    const int ring_teams = cfg->m_fast_tile_order <= 1 ? 1 : cfg->m_fast_tile_order;
    p.w_stages = p.w_stages / ring_teams * ring_teams;
    p.bridged_stages = p.bridged_stages / ring_teams * ring_teams;
    if (p.w_stages < ring_teams || p.bridged_stages < ring_teams || p.w_stages < 2 || p.bridged_stages < 2)
        return fail(TB_ERR_INVALID, "ring depths (num_stages %d, stream_k_aligned %d) must hold at least one stage per bridge team (%d) and two in all",
                    cfg->num_stages, cfg->stream_k_aligned, ring_teams);
    p.a_stages = token_stages_for(bm, p.w_stages, experts, a->group_scales != 0);
    if (p.a_stages < 2)
        return fail(TB_ERR_INVALID, "num_stages %d leaves no room for two %d-token stages in %d bytes of shared memory",
                    p.w_stages, bm, std::min(kSmemBudget, info.smem_optin));
    const tb::SmemLayout L = tb::smem_layout(bm, p.w_stages, p.a_stages, experts, a->group_scales != 0);
    // Slack for the 1024-byte alignment of the tiles; never less than half of an SM's shared memory, so that two
    // CTAs (of this launch, or of launches chained by PDL) cannot share an SM and wait for each other's tensor memory.
    const size_t smem = std::max<size_t>(L.total + 1024, 116 * 1024);
    if (smem > static_cast<size_t>(std::min(kSmemBudget, info.smem_optin)))
        return fail(TB_ERR_INVALID, "config needs %zu bytes of shared memory, the device offers %d", smem, info.smem_optin);

    p.splits = 1;
    p.div_n_tiles = tb::FastDiv::make(static_cast<uint32_t>(p.n_tiles));
    p.m_blocks = ceil_div(a->rows, bm);
    long long units;
    if (layout == TB_LAYOUT_DENSE) {
        p.splits = std::max(1, static_cast<int>(cfg->use_stream_k));
        p.splits = std::min(p.splits, p.k_blocks);
        if (a->group_scales) p.splits = 1;
        if (a->only_split > p.splits) return fail(TB_ERR_INVALID, "only_split %d exceeds the %d K splits", a->only_split, p.splits);
        p.only_split = p.splits > 1 ? a->only_split : 0;
        const long long tiles = static_cast<long long>(p.m_blocks) * p.n_tiles;
        if (p.splits > 1) {
            if (tiles > tb::kMaxSplitTiles) return fail(TB_ERR_INVALID, "K splits need at most %d output tiles, got %lld", tb::kMaxSplitTiles, tiles);
            if (a->workspace == nullptr) return fail(TB_ERR_INVALID, "K splits need a workspace");
            if (reinterpret_cast<uintptr_t>(a->workspace) % 8 != 0) return fail(TB_ERR_INVALID, "workspace must be 8-byte aligned");
            const long long need = split_scratch_bytes(a->rows, a->n, bm, p.splits);
            if (a->workspace_bytes < need) return fail(TB_ERR_INVALID, "workspace of %lld bytes is below the %lld needed", (long long)a->workspace_bytes, need);
        }
        units = tiles * p.splits;
    } else {
        p.expert_offsets = reinterpret_cast<const long long*>(routing->expert_offsets);
        p.expert_counts = routing->expert_counts;
        p.sorted_ids = routing->sorted_ids;
        p.expert_ids = routing->expert_ids;
        p.num_tokens_padded = routing->num_tokens_padded;
        p.sorted_capacity = routing->sorted_capacity;
        // Upper bound of the units the device-side schedule can produce; the real count is computed on the device.
        long long m_blocks_bound;
        if (layout == TB_LAYOUT_INDEXED) m_blocks_bound = routing->sorted_capacity / bm;
        else if (layout == TB_LAYOUT_MASKED) m_blocks_bound = static_cast<long long>(experts) * ceil_div(a->rows / experts, bm);
        else m_blocks_bound = a->rows / bm + experts;
        units = std::max<long long>(m_blocks_bound, 1) * p.n_tiles;
        if (units > 0x7FFFFFFFll) return fail(TB_ERR_INVALID, "too many tiles");
    }

    // Indexed routing with scratch: gather the routed rows into sorted order first, then treat them as a dense matrix.
    const void* act_base = a->a;
    uint64_t act_rows = static_cast<uint64_t>(a->rows);
    if (layout == TB_LAYOUT_INDEXED && routing->gather_scratch != nullptr && routing->sorted_capacity > 0) {
        const long long need = routing->sorted_capacity * a->k;
        if (routing->gather_scratch_bytes < need)
            return fail(TB_ERR_INVALID, "gather scratch of %lld bytes is below the %lld needed", (long long)routing->gather_scratch_bytes, need);
        if (reinterpret_cast<uintptr_t>(routing->gather_scratch) % 16 != 0) return fail(TB_ERR_INVALID, "gather scratch must be 16-byte aligned");
        cudaLaunchConfig_t gcfg = {};
        gcfg.gridDim = dim3(static_cast<unsigned>(std::min<long long>((routing->sorted_capacity + 7) / 8, 4 * sms)));
        gcfg.blockDim = dim3(256);
        gcfg.stream = stream;
        cudaLaunchAttribute gattr[1];
        gattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        gattr[0].val.programmaticStreamSerializationAllowed = 1;
        gcfg.attrs = gattr;
        gcfg.numAttrs = a->enable_pdl ? 1 : 0;
        TB_CUDA(cudaLaunchKernelEx(&gcfg, tb::gather_rows_kernel, static_cast<const uint8_t*>(a->a), routing->sorted_ids,
                                   routing->num_tokens_padded, static_cast<long long>(routing->sorted_capacity),
                                   static_cast<long long>(a->rows), static_cast<int>(routing->top_k), static_cast<int>(a->k),
                                   static_cast<uint8_t*>(routing->gather_scratch)));
        p.a_gathered = 1;
        act_base = routing->gather_scratch;
        act_rows = static_cast<uint64_t>(routing->sorted_capacity);
    }
    // Tensor maps: activations (128-byte swizzle, rows past the end read as zero) and weight scales.
    if (layout != TB_LAYOUT_INDEXED || p.a_gathered) {
        if (int rc = cached_map_u8(&p.map_a, act_base, static_cast<uint64_t>(a->k), act_rows,
                                 static_cast<uint64_t>(a->k), 128, static_cast<uint32_t>(bm), CU_TENSOR_MAP_SWIZZLE_128B))
            return rc;
    }
    if (!a->group_scales) {
        const uint64_t sf_rows = static_cast<uint64_t>(std::max(experts, 1)) * (p.k_pad / 16);
        if (int rc = cached_map_u8(&p.map_sf, a->scale, static_cast<uint64_t>(p.n_pad), sf_rows, static_cast<uint64_t>(p.n_pad),
                                 128, 8, CU_TENSOR_MAP_SWIZZLE_NONE))
            return rc;
    }

    p.div_splits = tb::FastDiv::make(static_cast<uint32_t>(p.splits));
    const int grid = static_cast<int>(std::min<long long>(units, sms));
    // use_stream_k = 1: the tiles of the last, partial round are shared out: with `left` tiles on `grid` CTAs, grid / left
    // CTAs (at most four) take a K-block range each of one tile and reduce it among themselves.  It applies where it can
    // pay and the kernel has the path: 256-token tiles with per-token scales, more tiles than CTAs, a last round that
    // fills at most half of them, at least four K blocks per part, 16-byte output words, a workspace for the partial
    // sums.  Otherwise the launch runs whole tiles.
    if (layout == TB_LAYOUT_DENSE && cfg->use_stream_k == 1 && bm == 256 && !a->group_scales && a->only_split == 0) {
        const long long tiles = units, left = tiles % grid;
        const int parts = left > 0 ? static_cast<int>(std::min<long long>({grid / left, tb::kMaxSharedParts, p.k_blocks / 4})) : 0;
        if (tiles > grid && parts >= 2 && grid <= tb::kMaxBalancedCtas && tiles < (1ll << 24) && a->n % 8 == 0 &&
            reinterpret_cast<uintptr_t>(a->d) % 16 == 0 && a->workspace != nullptr &&
            reinterpret_cast<uintptr_t>(a->workspace) % 16 == 0 && a->workspace_bytes >= balanced_scratch_bytes(grid)) {
            p.whole_rounds = static_cast<int>(tiles / grid);
            p.shared_tiles = static_cast<int>(left);
            p.shared_parts = parts;
        }
    }
    const bool exact = a->bridge == TB_BRIDGE_EXACT;
    if (a->bridge != TB_BRIDGE_EXACT && a->bridge != TB_BRIDGE_FPMA) return fail(TB_ERR_INVALID, "unknown bridge %d", a->bridge);
    const bool pdl = a->enable_pdl != 0 || p.a_gathered != 0;  // behind its own gather pass the GEMM always chains
    p.static_weights = a->enable_pdl == TB_PDL_STATIC_WEIGHTS ? 1 : 0;
    const int teams = cfg->m_fast_tile_order <= 1 ? 1 : cfg->m_fast_tile_order;
    const bool group = a->group_scales != 0;
    if (CUfunction jit = find_registered({device, bm, exact ? 1 : 0, group ? 1 : 0, cfg->math_warpgroups * 4, teams}))
        return launch_registered(jit, tb::gemm_threads(bm, cfg->math_warpgroups * 4), stream, p, grid, smem, pdl);
    if (!valid_block_m(bm))
        return fail(TB_ERR_UNSUPPORTED, "no kernel for block_m %d: compile one with tensorbridge.jit.runtime.get_kernel first", bm);
    tb::LaunchFn launch = nullptr;
    if (cfg->math_warpgroups == 2 && teams == 1) launch = tb::launch_w8_t1;
    if (cfg->math_warpgroups == 2 && teams == 2) launch = tb::launch_w8_t2;
    if (cfg->math_warpgroups == 4 && teams == 4) launch = tb::launch_w16_t4;
    if (launch == nullptr)
        return fail(TB_ERR_UNSUPPORTED, "no kernel for %d bridge warps in %d teams (math_warpgroups %d, m_fast_tile_order %d): the "
                    "library holds 8 warps in 1 or 2 teams and 16 in 4; compile one with tensorbridge.jit.runtime.get_kernel first",
                    cfg->math_warpgroups * 4, teams, cfg->math_warpgroups, cfg->m_fast_tile_order);
    const int rc = launch(bm, exact, group, stream, p, grid, smem, pdl);
    if (rc == tb::kLaunchUnsupported)
        return fail(TB_ERR_UNSUPPORTED, "no kernel for block_m %d%s", bm, group ? " with group scales" : "");
    if (rc != 0) return fail(TB_ERR_CUDA, "kernel launch: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
    return TB_OK;
}

template <typename T>
int launch_quantize(cudaStream_t stream, const void* x, long long x_stride, long long m, long long k, int mode, void* q,
                    float* scale, long long ssm, long long ssk) {
    cudaLaunchConfig_t cfg = {};
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (mode == TB_QUANT_PER_TOKEN) {
        cfg.gridDim = dim3(static_cast<unsigned>(m));
        cfg.blockDim = dim3(tb::kQuantThreads);
        TB_CUDA(cudaLaunchKernelEx(&cfg, tb::quantize_per_token_kernel<T>, static_cast<const T*>(x), x_stride,
                                   static_cast<int>(k), static_cast<uint8_t*>(q), scale, ssm));
    } else {
        const long long items = m * ((k + 127) / 128);
        cfg.gridDim = dim3(static_cast<unsigned>((items + 15) / 16));
        cfg.blockDim = dim3(256);
        TB_CUDA(cudaLaunchKernelEx(&cfg, tb::quantize_group128_kernel<T>, static_cast<const T*>(x), x_stride, m,
                                   static_cast<int>(k), static_cast<uint8_t*>(q), scale, ssm, ssk));
    }
    return TB_OK;
}

// ---- scratch that needs no allocation (tb_gemm_dense_static_scratch) -------------------------------------------
// 8 MiB of FP32 split-K partials reserved in the library's own device image: every GPU that loads the library holds
// it until the process exits.  In host code the array's name is only a handle for cudaGetSymbolAddress, never a
// device address.
constexpr long long kStaticScratchBytes = 8ll << 20;
static __device__ __align__(256) float g_static_scratch[kStaticScratchBytes / sizeof(float)];

// Device address of g_static_scratch on the current device, looked up once per device.
int static_scratch_address(float** out) {
    static std::mutex mutex;
    static float* address[64] = {};
    int device = 0;
    TB_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return fail(TB_ERR_INVALID, "device %d out of range", device);
    std::lock_guard<std::mutex> guard(mutex);
    if (address[device] == nullptr) {
        float* ptr = nullptr;
        const cudaError_t err = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
        if (err != cudaSuccess || ptr == nullptr)
            return fail(TB_ERR_CUDA, "cudaGetSymbolAddress(static scratch) on device %d: %s", device, cudaGetErrorString(err));
        address[device] = ptr;
    }
    *out = address[device];
    return TB_OK;
}

}  // namespace

extern "C" {

const char* tb_last_error(void) { return g_error; }

const char* tb_version(void) { return "tensorbridge_b200 0.1 (sm_100a)"; }

int tb_num_sms(int device, int* num_sms) {
    if (num_sms == nullptr) return fail(TB_ERR_INVALID, "null output");
    DeviceInfo info;
    if (int rc = device_info(device, &info)) return rc;
    int sms = info.num_sms;
    if (int cap = env_sm_cap()) sms = std::min(sms, cap);
    *num_sms = sms;
    return TB_OK;
}

int tb_select_config(const tb_problem* problem, tb_config* config) {
    if (problem == nullptr || config == nullptr) return fail(TB_ERR_INVALID, "null arguments");
    return rule(*problem, config);
}

int64_t tb_workspace_bytes(int64_t m, int64_t n, const tb_config* config) {
    if (config == nullptr || config->use_stream_k < 1 || m <= 0 || n <= 0 || !(valid_block_m(config->block_m) || jit_block_m(config->block_m))) return 0;
    if (config->use_stream_k == 1) {  // balanced shares: a partial tile per CTA, whatever the device (at most 256 SMs)
        const long long tiles = static_cast<long long>(ceil_div(m, config->block_m)) * (pad128(n) / 128);
        return config->block_m == 256 && tiles > 1 ? balanced_scratch_bytes(static_cast<int>(std::min<long long>(tiles, 256))) : 0;
    }
    return split_scratch_bytes(m, n, config->block_m, config->use_stream_k);
}

int tb_quantize_fp8(void* stream, const void* x, int x_dtype, int64_t x_stride, int64_t m, int64_t k, int mode, void* q,
                    float* scale, int64_t scale_stride_m, int64_t scale_stride_k) {
    if (m < 0 || k <= 0) return fail(TB_ERR_INVALID, "bad shape m=%lld k=%lld", (long long)m, (long long)k);
    if (m == 0) return TB_OK;
    if (x == nullptr || q == nullptr || scale == nullptr) return fail(TB_ERR_INVALID, "null tensor pointer");
    if (mode != TB_QUANT_PER_TOKEN && mode != TB_QUANT_GROUP_128) return fail(TB_ERR_INVALID, "unknown mode %d", mode);
    if (m > 0x7FFFFFFFll || k > 0x3FFFFFFFll) return fail(TB_ERR_INVALID, "shape too large");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (x_dtype) {
        case TB_DTYPE_BF16: return launch_quantize<__nv_bfloat16>(s, x, x_stride, m, k, mode, q, scale, scale_stride_m, scale_stride_k);
        case TB_DTYPE_F16: return launch_quantize<__half>(s, x, x_stride, m, k, mode, q, scale, scale_stride_m, scale_stride_k);
        case TB_DTYPE_F32: return launch_quantize<float>(s, x, x_stride, m, k, mode, q, scale, scale_stride_m, scale_stride_k);
        default: return fail(TB_ERR_INVALID, "unknown dtype %d", x_dtype);
    }
}

int tb_quantize_moe(void* stream, const tb_quant_moe_args* a) {
    if (a == nullptr) return fail(TB_ERR_INVALID, "null arguments");
    if (a->rows < 0 || a->width <= 0) return fail(TB_ERR_INVALID, "bad shape rows=%lld width=%lld", (long long)a->rows, (long long)a->width);
    if (a->rows == 0) return TB_OK;
    if (a->x == nullptr || a->q == nullptr || a->scale == nullptr) return fail(TB_ERR_INVALID, "null tensor pointer");
    if (a->width > tb::kQuantThreads * tb::kQuantVec * tb::kQuantMaxSteps) return fail(TB_ERR_UNSUPPORTED, "width %lld exceeds 8192", (long long)a->width);
    if (a->mode != TB_QUANT_PER_TOKEN && a->mode != TB_QUANT_GROUP_128) return fail(TB_ERR_INVALID, "unknown mode %d", a->mode);
    if (a->activation && a->x_dtype != TB_DTYPE_BF16) return fail(TB_ERR_INVALID, "the gated activation takes BF16 input");
    if (a->expert_counts != nullptr && (a->num_experts <= 0 || a->rows % a->num_experts != 0))
        return fail(TB_ERR_INVALID, "masked rows must divide into equal expert capacities");
    if (a->scatter_idx != nullptr && a->top_k < 1) return fail(TB_ERR_INVALID, "top_k must be positive");
    if (a->rows > 0x7FFFFFFFll) return fail(TB_ERR_INVALID, "too many rows");
    tb::QuantMoeParams p = {};
    p.x = a->x; p.x_stride = a->x_stride; p.rows = a->rows; p.width = static_cast<int>(a->width);
    p.group_128 = a->mode == TB_QUANT_GROUP_128; p.use_division = a->use_division;
    p.counts = a->expert_counts; p.capacity = a->expert_counts != nullptr ? a->rows / a->num_experts : 1;
    p.num_valid = a->num_valid_rows; p.num_valid_int64 = a->num_valid_rows_int64; p.scatter_idx = a->scatter_idx; p.top_k = a->top_k;
    p.out_rows = a->out_rows; p.q = static_cast<uint8_t*>(a->q); p.scale = a->scale;
    cudaLaunchConfig_t cfg = {};
    cfg.stream = static_cast<cudaStream_t>(stream);
    cfg.gridDim = dim3(static_cast<unsigned>(a->rows));
    cfg.blockDim = dim3(tb::kQuantThreads);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (a->activation) {
        TB_CUDA(cudaLaunchKernelEx(&cfg, tb::quantize_moe_kernel<__nv_bfloat16, true>, p));
    } else if (a->x_dtype == TB_DTYPE_BF16) {
        TB_CUDA(cudaLaunchKernelEx(&cfg, tb::quantize_moe_kernel<__nv_bfloat16, false>, p));
    } else if (a->x_dtype == TB_DTYPE_F16) {
        TB_CUDA(cudaLaunchKernelEx(&cfg, tb::quantize_moe_kernel<__half, false>, p));
    } else if (a->x_dtype == TB_DTYPE_F32) {
        TB_CUDA(cudaLaunchKernelEx(&cfg, tb::quantize_moe_kernel<float, false>, p));
    } else {
        return fail(TB_ERR_INVALID, "unknown dtype %d", a->x_dtype);
    }
    return TB_OK;
}

int tb_scatter_fp8(void* stream, const void* x, int64_t x_stride, const float* scale, int64_t scale_stride_m,
                   int64_t scale_stride_k, const int32_t* scatter_idx, int64_t rows, int32_t top_k, int64_t width,
                   int64_t groups, int64_t out_rows, void* out, float* out_scale) {
    if (rows < 0 || width <= 0 || groups <= 0 || top_k < 1) return fail(TB_ERR_INVALID, "bad shape");
    if (rows == 0) return TB_OK;
    if (x == nullptr || scale == nullptr || scatter_idx == nullptr || out == nullptr || out_scale == nullptr)
        return fail(TB_ERR_INVALID, "null tensor pointer");
    cudaLaunchConfig_t cfg = {};
    cfg.stream = static_cast<cudaStream_t>(stream);
    cfg.gridDim = dim3(static_cast<unsigned>(rows));
    cfg.blockDim = dim3(256);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    TB_CUDA(cudaLaunchKernelEx(&cfg, tb::scatter_fp8_kernel, static_cast<const uint8_t*>(x), static_cast<long long>(x_stride), scale,
                               static_cast<long long>(scale_stride_m), static_cast<long long>(scale_stride_k), scatter_idx,
                               static_cast<int>(top_k), static_cast<int>(width), static_cast<int>(groups),
                               static_cast<long long>(out_rows), static_cast<uint8_t*>(out), out_scale));
    return TB_OK;
}

int tb_prepare_weight(void* stream, const uint8_t* packed, const uint8_t* scale, int64_t num_experts, int64_t n, int64_t k,
                      int bridge, int clamp_scale, int32_t* weight, uint8_t* scale_out, int32_t* too_large) {
    if (packed == nullptr || scale == nullptr || weight == nullptr || scale_out == nullptr || too_large == nullptr)
        return fail(TB_ERR_INVALID, "null tensor pointer");
    if (num_experts < 1 || n <= 0 || k <= 0 || n % 8 || k % 16) return fail(TB_ERR_INVALID, "N must be a positive multiple of 8 and K of 16");
    if (num_experts > 1 && (n % 128 || k % 128)) return fail(TB_ERR_INVALID, "N and K of stacked experts must be multiples of 128");
    if (bridge != TB_BRIDGE_EXACT && bridge != TB_BRIDGE_FPMA) return fail(TB_ERR_INVALID, "unknown bridge %d", bridge);
    if (reinterpret_cast<uintptr_t>(packed) % 4 != 0) return fail(TB_ERR_INVALID, "packed must be 4-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int n_pad = pad128(n), k_pad = pad128(k);
    const long long rows = num_experts * n, rows_pad = num_experts * n_pad;
    const long long words = rows_pad * (k_pad / 8);
    tb::prepare_codes_kernel<<<static_cast<unsigned>((words + 255) / 256), 256, 0, s>>>(
        packed, scale, rows, static_cast<int>(k), rows_pad, k_pad, reinterpret_cast<uint32_t*>(weight));
    TB_CUDA(cudaGetLastError());
    const dim3 grid((n_pad + 31) / 32, (k_pad / 16 + 31) / 32, static_cast<unsigned>(num_experts));
    tb::prepare_scales_kernel<<<grid, dim3(32, 8), 0, s>>>(scale, static_cast<int>(num_experts), static_cast<int>(n),
                                                           static_cast<int>(k), n_pad, k_pad, bridge == TB_BRIDGE_EXACT,
                                                           clamp_scale, scale_out, too_large);
    TB_CUDA(cudaGetLastError());
    return TB_OK;
}

int tb_bridge_dump(void* stream, const int32_t* weight, const uint8_t* scale, int64_t num_experts, int64_t n_pad,
                   int64_t k_pad, int bridge, int group_scale_layout, uint8_t* fp8_out) {
    if (weight == nullptr || scale == nullptr || fp8_out == nullptr) return fail(TB_ERR_INVALID, "null tensor pointer");
    if (num_experts < 1 || n_pad <= 0 || k_pad <= 0 || n_pad % 128 || k_pad % 128) return fail(TB_ERR_INVALID, "padded sizes must be multiples of 128");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long rows_pad = num_experts * n_pad;
    const long long vecs = rows_pad * (k_pad / 32);
    const unsigned grid = static_cast<unsigned>((vecs + 255) / 256);
    if (bridge == TB_BRIDGE_EXACT) {
        tb::bridge_dump_kernel<true><<<grid, 256, 0, s>>>(reinterpret_cast<const uint4*>(weight), scale, rows_pad,
                                                          static_cast<int>(n_pad), static_cast<int>(k_pad), group_scale_layout, fp8_out);
    } else if (bridge == TB_BRIDGE_FPMA) {
        tb::bridge_dump_kernel<false><<<grid, 256, 0, s>>>(reinterpret_cast<const uint4*>(weight), scale, rows_pad,
                                                           static_cast<int>(n_pad), static_cast<int>(k_pad), group_scale_layout, fp8_out);
    } else {
        return fail(TB_ERR_INVALID, "unknown bridge %d", bridge);
    }
    TB_CUDA(cudaGetLastError());
    return TB_OK;
}

int tb_register_kernel(const tb_kernel_key* key, void* function) {
    if (key == nullptr || function == nullptr) return fail(TB_ERR_INVALID, "null arguments");
    if (!jit_block_m(key->block_m)) return fail(TB_ERR_INVALID, "block_m %d is no token tile the kernel template takes", key->block_m);
    if ((key->bridge_warps != 8 && key->bridge_warps != 16) || key->teams < 1 || key->bridge_warps % key->teams != 0 ||
        (key->bridge_warps / key->teams) % 4 != 0)
        return fail(TB_ERR_INVALID, "bridge warps %d in %d teams: 8 or 16 warps, teams of 4, 8 or 16 warps", key->bridge_warps, key->teams);
    if (key->device < 0 || key->device >= 64) return fail(TB_ERR_INVALID, "device %d out of range", key->device);
    const KernelKey k = {key->device, key->block_m, key->exact ? 1 : 0, key->group_scales ? 1 : 0, key->bridge_warps, key->teams};
    std::lock_guard<std::mutex> guard(g_registry_mutex);
    for (int i = 0; i < g_registered; ++i) {
        if (g_registry[i].key == k) {
            g_registry[i].function = static_cast<CUfunction>(function);
            return TB_OK;
        }
    }
    if (g_registered == 256) return fail(TB_ERR_UNSUPPORTED, "the kernel registry holds 256 kernels");
    g_registry[g_registered++] = {k, static_cast<CUfunction>(function)};
    return TB_OK;
}

int tb_registered_kernels(void) {
    std::lock_guard<std::mutex> guard(g_registry_mutex);
    return g_registered;
}

int tb_gemm_dense(void* stream, const tb_gemm_args* args, const tb_config* config) {
    return run_gemm(static_cast<cudaStream_t>(stream), args, nullptr, config);
}

int tb_gemm_dense_static_scratch(void* stream, const tb_gemm_args* args, const tb_config* config) {
    if (args == nullptr || config == nullptr) return fail(TB_ERR_INVALID, "null arguments");
    if (!valid_block_m(config->block_m) && !jit_block_m(config->block_m)) return fail(TB_ERR_INVALID, "block_m must be a multiple of 16 up to 256, got %d", config->block_m);
    // The splits the launch will really make: never more than K blocks, none with [1,128] scales.
    const int k_blocks = pad128(std::max<long long>(args->k, 1)) / 128;
    const int splits = args->group_scales ? 1 : std::min(std::max(1, static_cast<int>(config->use_stream_k)), k_blocks);
    const long long need = splits > 1 && args->rows > 0 && args->n > 0 ? split_scratch_bytes(args->rows, args->n, config->block_m, splits) : 0;
    if (need > kStaticScratchBytes)
        return fail(TB_ERR_INVALID, "this launch needs %lld bytes of split-K scratch; the library's static scratch holds %lld "
                    "(use fewer K splits, or tb_gemm_dense with a caller-owned workspace)", need, kStaticScratchBytes);
    float* scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    tb_gemm_args with_scratch = *args;
    with_scratch.workspace = scratch;
    with_scratch.workspace_bytes = kStaticScratchBytes;
    return run_gemm(static_cast<cudaStream_t>(stream), &with_scratch, nullptr, config);
}

int tb_gemm_grouped(void* stream, const tb_gemm_args* args, const tb_routing* routing, const tb_config* config) {
    if (routing == nullptr) return fail(TB_ERR_INVALID, "null routing");
    return run_gemm(static_cast<cudaStream_t>(stream), args, routing, config);
}

}  // extern "C"
