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

// Shared memory of the plan kernel, for E experts: int cursor[E], unsigned short tile_total[E],
// unsigned short prefix[kPlanWarps][E], unsigned char count[kPlanWarps][E].
__host__ __device__ inline size_t ep_plan_smem(int experts) {
    return static_cast<size_t>(experts) * (4 + 2 + kPlanWarps * 3) + 64 * 4;
}

// One CTA.  Routes with an id outside [0, num_experts) are not sent: send_pos = -1.
__global__ void __launch_bounds__(kPlanThreads, 1)
ep_plan_kernel(const void* ids, int ids_int64, long long routes, int num_experts, int world, int interleaved,
               int* __restrict__ send_counts, int* __restrict__ send_pos) {
    extern __shared__ __align__(16) unsigned char plan_smem[];
    const int E = num_experts, e_local = E / world;
    int* cursor = reinterpret_cast<int*>(plan_smem);
    int* warp_totals = cursor + E;  // 64 ints
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
        if (tid < E) cursor[tid] = warp_totals[32 + warp] + incl - mine;
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
        if (r < routes) send_pos[r] = placed >= 0 ? cursor[placed] + prefix[warp * E + placed] + rank_in_warp : -1;
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

}  // namespace tb
