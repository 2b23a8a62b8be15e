// C ABI of the expert-parallel dispatch kernels (tb_ep.cuh); declared in include/tensorbridge_b200.h.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "../../include/tensorbridge_b200.h"
#include "tb_ep.cuh"

namespace tb {
int set_last_error(int code, const char* fmt, ...);  // tb_api.cu
}

namespace {

#define TB_EP_CUDA(expr)                                                                                              \
    do {                                                                                                              \
        cudaError_t err__ = (expr);                                                                                   \
        if (err__ != cudaSuccess) return tb::set_last_error(TB_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(err__)); \
    } while (0)

int row_grid(long long rows) { return static_cast<int>(std::min<long long>(std::max<long long>((rows + 7) / 8, 1), 148 * 8)); }

}  // namespace

extern "C" {

int tb_ep_plan(void* stream, const void* topk_ids, int ids_int64, int64_t routes, int32_t num_experts, int32_t world,
               int32_t interleaved, int32_t* send_counts, int32_t* send_pos) {
    if (routes < 0 || num_experts <= 0 || world <= 0 || num_experts % world != 0)
        return tb::set_last_error(TB_ERR_INVALID, "bad dispatch shape: routes=%lld experts=%d world=%d", (long long)routes, num_experts, world);
    if (num_experts > tb::kEpMaxExperts) return tb::set_last_error(TB_ERR_UNSUPPORTED, "at most %d experts", tb::kEpMaxExperts);
    if (routes > 0x7FFFFFFFll) return tb::set_last_error(TB_ERR_INVALID, "too many routes");
    if (send_counts == nullptr || (routes > 0 && (topk_ids == nullptr || send_pos == nullptr)))
        return tb::set_last_error(TB_ERR_INVALID, "null tensor pointer");
    const size_t smem = tb::ep_plan_smem(num_experts);
    static std::mutex mutex;
    static bool configured[64] = {};
    int device = 0;
    TB_EP_CUDA(cudaGetDevice(&device));
    if (device >= 0 && device < 64) {
        std::lock_guard<std::mutex> guard(mutex);
        if (!configured[device]) {
            TB_EP_CUDA(cudaFuncSetAttribute(tb::ep_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            static_cast<int>(tb::ep_plan_smem(tb::kEpMaxExperts))));
            configured[device] = true;
        }
    }
    tb::ep_plan_kernel<<<1, tb::kPlanThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        topk_ids, ids_int64, routes, num_experts, world, interleaved, send_counts, send_pos);
    TB_EP_CUDA(cudaGetLastError());
    return TB_OK;
}

int tb_ep_pack(void* stream, const void* x, const float* scale, const int32_t* send_pos, int64_t routes, int32_t top_k,
               int64_t width, int64_t groups, int64_t row_bytes, void* send) {
    if (routes < 0 || top_k < 1 || width <= 0 || width % 16 != 0 || groups < 1 || row_bytes % 16 != 0 || row_bytes < width + 4 * groups)
        return tb::set_last_error(TB_ERR_INVALID, "bad pack shape: width=%lld groups=%lld row_bytes=%lld", (long long)width, (long long)groups, (long long)row_bytes);
    if (routes == 0) return TB_OK;
    if (x == nullptr || scale == nullptr || send_pos == nullptr || send == nullptr) return tb::set_last_error(TB_ERR_INVALID, "null tensor pointer");
    tb::ep_pack_kernel<<<row_grid(routes), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(x), scale, send_pos, routes, top_k, static_cast<int>(width), static_cast<int>(groups),
        static_cast<int>(row_bytes), static_cast<uint8_t*>(send));
    TB_EP_CUDA(cudaGetLastError());
    return TB_OK;
}

int tb_ep_layout(void* stream, const int32_t* recv_counts, int32_t world, int32_t experts_local, int32_t capacity,
                 int32_t* seg_start, int32_t* seg_dest, int32_t* counts) {
    if (world <= 0 || experts_local <= 0 || capacity <= 0) return tb::set_last_error(TB_ERR_INVALID, "bad layout shape");
    if (recv_counts == nullptr || seg_start == nullptr || seg_dest == nullptr || counts == nullptr)
        return tb::set_last_error(TB_ERR_INVALID, "null tensor pointer");
    tb::ep_layout_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(recv_counts, world, experts_local, capacity, seg_start,
                                                                           seg_dest, counts);
    TB_EP_CUDA(cudaGetLastError());
    return TB_OK;
}

int tb_ep_place(void* stream, const void* recv, int64_t rows, int64_t row_bytes, int64_t width, int64_t groups,
                const int32_t* seg_start, const int32_t* seg_dest, int32_t world, int32_t experts_local, int32_t capacity,
                void* a, float* a_scale, int32_t* recv_rows) {
    if (rows < 0 || width <= 0 || width % 16 != 0 || groups < 1 || row_bytes % 16 != 0 || row_bytes < width + 4 * groups ||
        world <= 0 || experts_local <= 0 || capacity <= 0)
        return tb::set_last_error(TB_ERR_INVALID, "bad place shape");
    if (rows == 0) return TB_OK;
    if (recv == nullptr || seg_start == nullptr || seg_dest == nullptr || a == nullptr || a_scale == nullptr || recv_rows == nullptr)
        return tb::set_last_error(TB_ERR_INVALID, "null tensor pointer");
    tb::ep_place_kernel<<<row_grid(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(recv), rows, static_cast<int>(row_bytes), static_cast<int>(width), static_cast<int>(groups),
        seg_start, seg_dest, world * experts_local, experts_local, capacity, static_cast<uint8_t*>(a), a_scale, recv_rows);
    TB_EP_CUDA(cudaGetLastError());
    return TB_OK;
}

int tb_gather_rows(void* stream, const void* src, const int32_t* index, int64_t rows, int64_t row_bytes, void* dst) {
    if (rows < 0 || row_bytes <= 0 || row_bytes % 16 != 0) return tb::set_last_error(TB_ERR_INVALID, "row_bytes must be a positive multiple of 16");
    if (rows == 0) return TB_OK;
    if (src == nullptr || index == nullptr || dst == nullptr) return tb::set_last_error(TB_ERR_INVALID, "null tensor pointer");
    tb::gather_rows16_kernel<<<row_grid(rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(src), index, rows, static_cast<int>(row_bytes), static_cast<uint8_t*>(dst));
    TB_EP_CUDA(cudaGetLastError());
    return TB_OK;
}

}  // extern "C"
