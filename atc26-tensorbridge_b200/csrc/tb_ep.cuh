// Expert-parallel token dispatch around the masked grouped GEMM: the integer bookkeeping and row movement on either
// side of the all-to-all, as kernels, so that a dispatch step reads nothing back to the host but the split sizes.
//
//   plan     routes (expert of every (token, slot)) -> routes per (destination rank, local expert) and the row of
//            every route in the send buffer, ordered by destination rank, then local expert, then route id
//   pack     FP8 rows + their FP32 scales -> one packed row per route, in send order (one exchange instead of two)
//   layout   received counts per (source rank, local expert) -> where each (source, expert) run starts in the receive
//            buffer and in the masked activation buffer; per-expert row counts clamped to the capacity
//   place    received packed rows -> masked buffer rows (+ scales); rows past an expert's capacity are dropped
//   gather   BF16 rows by index (-1 = zeros): results back into receive order, and returned rows into route order
//
// The reference has no counterpart: it is handed expert-parallel shapes already dispatched by the serving framework.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {

constexpr int kPlanThreads = 1024;
constexpr int kPlanWarps = kPlanThreads / 32;
constexpr int kEpMaxExperts = 1024;

// Global expert id -> owner rank * e_local + local index.
__device__ __forceinline__ int ep_placed(int expert, int e_local, int world, bool interleaved) {
    return interleaved ? (expert % world) * e_local + expert / world : expert;
}

__device__ __forceinline__ int ep_load_id(const void* ids, bool ids_int64, long long i) {
    return ids_int64 ? static_cast<int>(static_cast<const long long*>(ids)[i]) : static_cast<const int*>(ids)[i];
}

// Shared memory of the plan kernel, for E experts: int cursor[E], int first_row[E], unsigned short tile_total[E],
// unsigned short prefix[kPlanWarps][E], unsigned char count[kPlanWarps][E].
__host__ __device__ inline size_t ep_plan_smem(int experts) {
    return static_cast<size_t>(experts) * (4 + 4 + 2 + kPlanWarps * 3) + 64 * 4;
}

// One CTA.  Routes with an id outside [0, num_experts) are not sent: send_pos = -1.
__global__ void __launch_bounds__(kPlanThreads, 1)
ep_plan_kernel(const void* ids, int ids_int64, long long routes, int num_experts, int world, int interleaved,
               int* __restrict__ send_counts, int* __restrict__ send_pos, int* __restrict__ route_rank) {
    extern __shared__ __align__(16) unsigned char plan_smem[];
    const int E = num_experts, e_local = E / world;
    int* cursor = reinterpret_cast<int*>(plan_smem);
    int* first_row = cursor + E;      // first send row of every expert
    int* warp_totals = first_row + E;  // 64 ints
    unsigned short* tile_total = reinterpret_cast<unsigned short*>(warp_totals + 64);
    unsigned short* prefix = tile_total + E;                                    // [kPlanWarps][E]
    unsigned char* count = reinterpret_cast<unsigned char*>(prefix + kPlanWarps * E);  // [kPlanWarps][E]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // pass A: routes per placed expert, then their exclusive prefix = first send row of every expert
    for (int e = tid; e < E; e += kPlanThreads) cursor[e] = 0;
    __syncthreads();
    for (long long r = tid; r < routes; r += kPlanThreads) {
        const int e = ep_load_id(ids, ids_int64 != 0, r);
        if (e >= 0 && e < E) atomicAdd(&cursor[ep_placed(e, e_local, world, interleaved != 0)], 1);
    }
    __syncthreads();
    {
        const int mine = tid < E ? cursor[tid] : 0;  // E <= kPlanThreads
        if (tid < E) send_counts[tid] = mine;
        int incl = mine;
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) warp_totals[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            const int t = warp_totals[lane];
            int s = t;
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, s, o);
                if (lane >= o) s += v;
            }
            warp_totals[32 + lane] = s - t;
        }
        __syncthreads();
        if (tid < E) cursor[tid] = first_row[tid] = warp_totals[32 + warp] + incl - mine;
    }
    __syncthreads();

    // pass B: tiles of kPlanThreads routes in route order.  Within a tile a route's rank among the routes of its expert
    // is (routes of that expert in earlier warps) + (earlier lanes of its own warp), which keeps route order.
    for (long long tile0 = 0; tile0 < routes; tile0 += kPlanThreads) {
        for (int i = tid; i < kPlanWarps * E; i += kPlanThreads) count[i] = 0;
        __syncthreads();
        const long long r = tile0 + tid;
        int placed = -1;
        if (r < routes) {
            const int e = ep_load_id(ids, ids_int64 != 0, r);
            if (e >= 0 && e < E) placed = ep_placed(e, e_local, world, interleaved != 0);
        }
        const unsigned peers = __match_any_sync(0xffffffffu, placed);
        const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
        if (placed >= 0 && rank_in_warp == 0) count[warp * E + placed] = static_cast<unsigned char>(__popc(peers));
        __syncthreads();
        for (int e = tid; e < E; e += kPlanThreads) {
            int run = 0;
            for (int w = 0; w < kPlanWarps; ++w) {
                prefix[w * E + e] = static_cast<unsigned short>(run);
                run += count[w * E + e];
            }
            tile_total[e] = static_cast<unsigned short>(run);
        }
        __syncthreads();
        if (r < routes) {
            const int pos = placed >= 0 ? cursor[placed] + prefix[warp * E + placed] + rank_in_warp : -1;
            if (send_pos != nullptr) send_pos[r] = pos;
            // rank of the route among this rank's routes to the same expert, in route order
            if (route_rank != nullptr) route_rank[r] = placed >= 0 ? pos - first_row[placed] : -1;
        }
        __syncthreads();
        for (int e = tid; e < E; e += kPlanThreads) cursor[e] += tile_total[e];
        // the zeroing pass of the next tile is separated from these reads by its own barrier
        __syncthreads();
    }
}

// One warp per route: send[pos] = {x[row] (width bytes), scale[row] (groups floats)}, row = route / top_k.
// row_bytes (a multiple of 16) >= width + 4 * groups; width a multiple of 16.
__global__ void __launch_bounds__(256)
ep_pack_kernel(const uint8_t* __restrict__ x, const float* __restrict__ scale, const int* __restrict__ send_pos,
               long long routes, int top_k, int width, int groups, int row_bytes, uint8_t* __restrict__ send) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    for (long long r = warp0; r < routes; r += warps) {
        const int pos = send_pos[r];
        if (pos < 0) continue;
        const long long row = r / top_k;
        const uint4* src = reinterpret_cast<const uint4*>(x + row * width);
        uint4* dst = reinterpret_cast<uint4*>(send + static_cast<long long>(pos) * row_bytes);
        for (int i = lane; i < width / 16; i += 32) dst[i] = src[i];
        float* sdst = reinterpret_cast<float*>(send + static_cast<long long>(pos) * row_bytes + width);
        for (int g = lane; g < groups; g += 32) sdst[g] = scale[row * groups + g];
    }
}

// One CTA.  recv_counts [world][e_local] (source-major, as the count exchange delivers them).
//   seg_start [world * e_local]  first row of run (s, e) in the receive buffer (source-major order)
//   seg_dest  [world * e_local]  row of the masked buffer its first row goes to: e * capacity + rows of earlier sources
//   counts    [e_local]          min(capacity, rows received for e)
__global__ void __launch_bounds__(1024, 1)
ep_layout_kernel(const int* __restrict__ recv_counts, int world, int e_local, int capacity, int* __restrict__ seg_start,
                 int* __restrict__ seg_dest, int* __restrict__ counts) {
    __shared__ int warp_totals[64];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int segments = world * e_local;
    // exclusive prefix over the segments in source-major order, 1024 at a time
    int carry = 0;
    for (int base = 0; base < segments; base += 1024) {
        const int g = base + tid;
        const int mine = g < segments ? recv_counts[g] : 0;
        int incl = mine;
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) warp_totals[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            const int t = warp_totals[lane];
            int s = t;
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, s, o);
                if (lane >= o) s += v;
            }
            warp_totals[32 + lane] = s - t;
            if (lane == 31) warp_totals[31] = s;  // total of this pass (slot 31 is read only after the barrier)
        }
        __syncthreads();
        const int pass_total = warp_totals[31];
        if (g < segments) seg_start[g] = carry + warp_totals[32 + warp] + incl - mine;
        __syncthreads();
        carry += pass_total;
    }
    // rows of earlier sources per expert
    for (int e = tid; e < e_local; e += 1024) {
        int before = 0;
        for (int s = 0; s < world; ++s) {
            seg_dest[s * e_local + e] = e * capacity + before;
            before += recv_counts[s * e_local + e];
        }
        counts[e] = min(before, capacity);
    }
}

// One warp per received row.  recv_rows[i] = its row in the masked buffer, or -1 when it fell past the capacity.
__global__ void __launch_bounds__(256)
ep_place_kernel(const uint8_t* __restrict__ recv, long long rows, int row_bytes, int width, int groups,
                const int* __restrict__ seg_start, const int* __restrict__ seg_dest, int segments, int e_local, int capacity,
                uint8_t* __restrict__ a, float* __restrict__ a_scale, int* __restrict__ recv_rows) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    for (long long i = warp0; i < rows; i += warps) {
        int lo = 0, hi = segments;  // last segment with seg_start <= i (empty runs share a start: take the last)
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (seg_start[mid] <= i) lo = mid; else hi = mid;
        }
        const int e = lo % e_local;
        const int dest = seg_dest[lo] + static_cast<int>(i - seg_start[lo]);
        const bool keep = dest - e * capacity < capacity;
        if (lane == 0) recv_rows[i] = keep ? dest : -1;
        if (!keep) continue;
        const uint4* src = reinterpret_cast<const uint4*>(recv + i * row_bytes);
        uint4* dst = reinterpret_cast<uint4*>(a + static_cast<long long>(dest) * width);
        for (int v = lane; v < width / 16; v += 32) dst[v] = src[v];
        const float* ssrc = reinterpret_cast<const float*>(recv + i * row_bytes + width);
        for (int g = lane; g < groups; g += 32) a_scale[static_cast<long long>(dest) * groups + g] = ssrc[g];
    }
}

// dst[i, :] = index[i] >= 0 ? src[index[i], :] : 0, rows of `row_bytes` bytes (a multiple of 16); one warp per row.
__global__ void __launch_bounds__(256)
gather_rows16_kernel(const uint8_t* __restrict__ src, const int* __restrict__ index, long long rows, int row_bytes,
                     uint8_t* __restrict__ dst) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    for (long long i = warp0; i < rows; i += warps) {
        const int from = index[i];
        uint4* out = reinterpret_cast<uint4*>(dst + i * row_bytes);
        if (from < 0) {
            for (int v = lane; v < row_bytes / 16; v += 32) out[v] = make_uint4(0, 0, 0, 0);
        } else {
            const uint4* in = reinterpret_cast<const uint4*>(src + static_cast<long long>(from) * row_bytes);
            for (int v = lane; v < row_bytes / 16; v += 32) out[v] = in[v];
        }
    }
}

// out[t, :] = bf16(sum over j < top_k of weights[t, j] * rows[r(t, j), :]), r = index[t * top_k + j] (or t * top_k + j
// without an index); routes whose index is negative add nothing.  The sum runs in FP32 in slot order j = 0, 1, ...,
// so it is the same from run to run.  One warp per token, eight channels (16 bytes) per lane and step.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ rows, const int* __restrict__ index, const float* __restrict__ weights,
                   long long tokens, int top_k, int width, __nv_bfloat16* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    for (long long t = warp0; t < tokens; t += warps) {
        for (int v = lane; v < width / 8; v += 32) {
            float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int j = 0; j < top_k; ++j) {
                const long long route = t * top_k + j;
                const long long from = index != nullptr ? index[route] : route;
                if (from < 0) continue;
                const float w = weights[route];
                const uint4 word = *reinterpret_cast<const uint4*>(rows + from * width + v * 8);
                const __nv_bfloat162* pair = reinterpret_cast<const __nv_bfloat162*>(&word);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(pair[i]);
                    sum[2 * i] = fmaf(w, f.x, sum[2 * i]);
                    sum[2 * i + 1] = fmaf(w, f.y, sum[2 * i + 1]);
                }
            }
            uint4 word;
            __nv_bfloat162* pair = reinterpret_cast<__nv_bfloat162*>(&word);
#pragma unroll
            for (int i = 0; i < 4; ++i) pair[i] = __floats2bfloat162_rn(sum[2 * i], sum[2 * i + 1]);
            *reinterpret_cast<uint4*>(out + t * width + v * 8) = word;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// The same dispatch over peer memory (NVLink loads and stores between the GPUs of one node) instead of an all-to-all:
// every rank keeps its masked activation buffer, its output buffer, a [world][E] count matrix and a row of arrival flags
// in memory its peers have mapped, and
//   barrier  a rank-to-rank barrier on those flags, optionally carrying this rank's route counts to every peer first
//   push     writes each route's FP8 row and scales straight into the masked buffer of the rank that owns its expert, at
//            the row the layout rule gives it (expert block, then source rank, then route order); routes past an expert's
//            capacity are never sent
//   pull     reads each route's output row back from the owner's output buffer
// so a step needs no host read, no staging copy and no collective library.  Plain loads and stores only.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kMaxPeers = 16;

struct PeerPointers {
    void* ptr[kMaxPeers];
};

// One CTA of 256 threads per launch.  Copies `count` ints from `payload` to row `rank` of every peer's [world][count]
// matrix (when count > 0), then tells every peer "rank has arrived at barrier number e" and waits until every peer has
// told it the same.  e is this rank's own count of barriers so far, kept in `local_epoch`: all ranks call the barrier the
// same number of times.  The wait is bounded: when it runs out the kernel writes 100 + the peer it waited for to
// status[0] and returns.
__global__ void __launch_bounds__(256, 1)
peer_barrier_kernel(PeerPointers flags, PeerPointers payload_dst, const int* __restrict__ payload, int count, int rank,
                    int world, unsigned* local_epoch, long long wait_cycles, int* status) {
    if (count > 0) {
        for (int p = 0; p < world; ++p) {
            int* dst = static_cast<int*>(payload_dst.ptr[p]) + static_cast<long long>(rank) * count;
            for (int i = threadIdx.x; i < count; i += blockDim.x) dst[i] = payload[i];
        }
    }
    __threadfence_system();
    __syncthreads();
    __shared__ unsigned epoch;
    if (threadIdx.x == 0) {
        epoch = *local_epoch + 1u;
        *local_epoch = epoch;
    }
    __syncthreads();
    const unsigned e = epoch;
    if (threadIdx.x < world) {
        const int p = threadIdx.x;
        unsigned* theirs = static_cast<unsigned*>(flags.ptr[p]) + rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(e) : "memory");
        const unsigned* mine = static_cast<const unsigned*>(flags.ptr[rank]) + p;
        const long long start = clock64();
        for (unsigned spin = 0;; ++spin) {
            unsigned seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
            if (static_cast<int>(seen - e) >= 0) break;
            if ((spin & 63u) == 63u && clock64() - start > wait_cycles) {
                if (status != nullptr) atomicCAS(status, 0, 100 + p);
                break;
            }
        }
    }
    __threadfence_system();
}

struct PushParams {
    const void* ids;           // [routes] int32 or int64: global expert of every route
    const uint8_t* x;          // [tokens, width] FP8
    const float* scale;        // [tokens, groups]
    const int* route_rank;     // [routes] from the plan kernel
    const int* all_counts;     // [world][E] in placed order: routes of every source rank for every expert
    int* dest_row;             // [routes] out: row in the owner's masked buffer, -1 = not sent
    int* counts;               // [E / world] out: rows of this rank's own experts, clamped to the capacity
    PeerPointers a, a_scale;   // every rank's masked buffers
    PeerPointers row_target;   // optional (ptr[0] != nullptr): every rank's int32 [E / world * capacity] table
    uint8_t* out;              // optional: this rank's route buffer, rows of routes that are not sent are cleared
    int out_row_bytes;
    long long routes;
    int ids_int64, top_k, num_experts, world, rank, interleaved, capacity, width, groups;
};

__global__ void __launch_bounds__(256)
ep_push_kernel(const PushParams p) {
    const int lane = threadIdx.x & 31;
    const int e_local = p.num_experts / p.world;
    if (blockIdx.x == 0) {
        for (int e = threadIdx.x; e < e_local; e += blockDim.x) {
            int total = 0;
            for (int s = 0; s < p.world; ++s) total += p.all_counts[s * p.num_experts + p.rank * e_local + e];
            p.counts[e] = min(total, p.capacity);
        }
    }
    const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    for (long long r = warp0; r < p.routes; r += warps) {
        const int e = ep_load_id(p.ids, p.ids_int64 != 0, r);
        int row = -1, owner = 0;
        if (e >= 0 && e < p.num_experts) {
            const int placed = ep_placed(e, e_local, p.world, p.interleaved != 0);
            owner = placed / e_local;
            int slot = p.route_rank[r];
            for (int s = 0; s < p.rank; ++s) slot += p.all_counts[s * p.num_experts + placed];
            if (slot < p.capacity) row = (placed - owner * e_local) * p.capacity + slot;
        }
        if (lane == 0) p.dest_row[r] = row;
        if (row < 0) {
            if (p.out != nullptr) {
                uint4* cleared = reinterpret_cast<uint4*>(p.out + r * p.out_row_bytes);
                for (int v = lane; v < p.out_row_bytes / 16; v += 32) cleared[v] = make_uint4(0, 0, 0, 0);
            }
            continue;
        }
        if (lane == 0 && p.row_target.ptr[0] != nullptr)
            static_cast<int*>(p.row_target.ptr[owner])[row] = (p.rank << 26) | static_cast<int>(r);
        const long long token = r / p.top_k;
        const uint4* src = reinterpret_cast<const uint4*>(p.x + token * p.width);
        uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.a.ptr[owner]) + static_cast<long long>(row) * p.width);
        for (int i = lane; i < p.width / 16; i += 32) dst[i] = src[i];
        float* sdst = static_cast<float*>(p.a_scale.ptr[owner]) + static_cast<long long>(row) * p.groups;
        for (int g = lane; g < p.groups; g += 32) sdst[g] = p.scale[token * p.groups + g];
    }
}

struct PullParams {
    const void* ids;
    const int* dest_row;   // [routes] from the push kernel
    PeerPointers y;        // every rank's output buffer [E / world * capacity, row_bytes]
    uint8_t* out;          // [routes, row_bytes]
    long long routes;
    int ids_int64, num_experts, world, interleaved, row_bytes;
};

__global__ void __launch_bounds__(256)
ep_pull_kernel(const PullParams p) {
    const int lane = threadIdx.x & 31;
    const int e_local = p.num_experts / p.world;
    const long long warp0 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
    for (long long r = warp0; r < p.routes; r += warps) {
        const int row = p.dest_row[r];
        uint4* out = reinterpret_cast<uint4*>(p.out + r * p.row_bytes);
        if (row < 0) {
            for (int v = lane; v < p.row_bytes / 16; v += 32) out[v] = make_uint4(0, 0, 0, 0);
            continue;
        }
        const int e = ep_load_id(p.ids, p.ids_int64 != 0, r);
        const int owner = ep_placed(e, e_local, p.world, p.interleaved != 0) / e_local;
        const uint4* in = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.y.ptr[owner]) + static_cast<long long>(row) * p.row_bytes);
        for (int v = lane; v < p.row_bytes / 16; v += 32) out[v] = in[v];
    }
}

}  // namespace tb
