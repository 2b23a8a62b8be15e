// C ABI of the expert-parallel dispatch kernels (tb_ep.cuh); declared in include/tensorbridge_b200.h.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
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
               int32_t interleaved, int32_t* send_counts, int32_t* send_pos, int32_t* route_rank) {
    if (routes < 0 || num_experts <= 0 || world <= 0 || num_experts % world != 0)
        return tb::set_last_error(TB_ERR_INVALID, "bad dispatch shape: routes=%lld experts=%d world=%d", (long long)routes, num_experts, world);
    if (num_experts > tb::kEpMaxExperts) return tb::set_last_error(TB_ERR_UNSUPPORTED, "at most %d experts", tb::kEpMaxExperts);
    if (routes > 0x7FFFFFFFll) return tb::set_last_error(TB_ERR_INVALID, "too many routes");
    if (send_counts == nullptr || (routes > 0 && (topk_ids == nullptr || (send_pos == nullptr && route_rank == nullptr))))
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
        topk_ids, ids_int64, routes, num_experts, world, interleaved, send_counts, send_pos, route_rank);
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

int tb_moe_combine(void* stream, const void* rows, const int32_t* index, const float* weights, int64_t tokens, int32_t top_k,
                   int64_t width, void* out) {
    if (tokens < 0 || top_k <= 0 || width <= 0 || width % 8 != 0)
        return tb::set_last_error(TB_ERR_INVALID, "combine needs top_k > 0 and a width that is a positive multiple of 8");
    if (tokens == 0) return TB_OK;
    if (rows == nullptr || weights == nullptr || out == nullptr) return tb::set_last_error(TB_ERR_INVALID, "null tensor pointer");
    if (reinterpret_cast<uintptr_t>(rows) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0)
        return tb::set_last_error(TB_ERR_INVALID, "rows and out must be 16-byte aligned");
    tb::moe_combine_kernel<<<row_grid(tokens), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(rows), index, weights, tokens, top_k, static_cast<int>(width),
        static_cast<__nv_bfloat16*>(out));
    TB_EP_CUDA(cudaGetLastError());
    return TB_OK;
}

// ---- peer memory ----------------------------------------------------------------------------------------------------
int tb_peer_alloc(int64_t bytes, void** ptr) {
    if (bytes <= 0 || ptr == nullptr) return tb::set_last_error(TB_ERR_INVALID, "bad allocation request");
    TB_EP_CUDA(cudaMalloc(ptr, static_cast<size_t>(bytes)));
    TB_EP_CUDA(cudaMemset(*ptr, 0, static_cast<size_t>(bytes)));
    TB_EP_CUDA(cudaDeviceSynchronize());
    return TB_OK;
}

int tb_peer_free(void* ptr) {
    if (ptr != nullptr) TB_EP_CUDA(cudaFree(ptr));
    return TB_OK;
}

int tb_ipc_export(const void* ptr, uint8_t* handle) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the C ABI carries IPC handles as 64 bytes");
    if (ptr == nullptr || handle == nullptr) return tb::set_last_error(TB_ERR_INVALID, "null pointer");
    cudaIpcMemHandle_t h;
    TB_EP_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)));
    std::memcpy(handle, &h, sizeof(h));
    return TB_OK;
}

int tb_ipc_open(const uint8_t* handle, void** ptr) {
    if (ptr == nullptr || handle == nullptr) return tb::set_last_error(TB_ERR_INVALID, "null pointer");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    TB_EP_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return TB_OK;
}

int tb_ipc_close(void* ptr) {
    if (ptr != nullptr) TB_EP_CUDA(cudaIpcCloseMemHandle(ptr));
    return TB_OK;
}

namespace {
int fill_peers(tb::PeerPointers* out, void* const* ptrs, int world, const char* what) {
    if (world < 1 || world > tb::kMaxPeers) return tb::set_last_error(TB_ERR_INVALID, "world size must be in 1..%d", tb::kMaxPeers);
    if (ptrs == nullptr) return tb::set_last_error(TB_ERR_INVALID, "null %s pointers", what);
    for (int i = 0; i < tb::kMaxPeers; ++i) out->ptr[i] = nullptr;
    for (int i = 0; i < world; ++i) {
        if (ptrs[i] == nullptr) return tb::set_last_error(TB_ERR_INVALID, "%s pointer of rank %d is null", what, i);
        out->ptr[i] = ptrs[i];
    }
    return TB_OK;
}
}  // namespace

int tb_peer_barrier(void* stream, void* const* flags, void* const* payload_dst, const int32_t* payload, int32_t count,
                    int32_t rank, int32_t world, uint32_t* local_epoch, int32_t wait_us, int32_t* status) {
    tb::PeerPointers f, d;
    if (int rc = fill_peers(&f, flags, world, "flag")) return rc;
    if (rank < 0 || rank >= world || local_epoch == nullptr || count < 0) return tb::set_last_error(TB_ERR_INVALID, "bad barrier arguments");
    if (count > 0) {
        if (payload == nullptr) return tb::set_last_error(TB_ERR_INVALID, "null payload");
        if (int rc = fill_peers(&d, payload_dst, world, "payload")) return rc;
    } else {
        d = f;
    }
    const long long cycles = wait_us > 0 ? static_cast<long long>(wait_us) * 2000 : (1ll << 31);
    tb::peer_barrier_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(f, d, payload, count, rank, world, local_epoch, cycles, status);
    TB_EP_CUDA(cudaGetLastError());
    return TB_OK;
}

int tb_ep_push(void* stream, const tb_ep_push_args* a) {
    if (a == nullptr) return tb::set_last_error(TB_ERR_INVALID, "null arguments");
    if (a->routes < 0 || a->top_k < 1 || a->num_experts <= 0 || a->world <= 0 || a->num_experts % a->world != 0 || a->rank < 0 ||
        a->rank >= a->world || a->capacity <= 0 || a->width <= 0 || a->width % 16 != 0 || a->groups < 1)
        return tb::set_last_error(TB_ERR_INVALID, "bad push shape");
    if (a->all_counts == nullptr || a->counts == nullptr) return tb::set_last_error(TB_ERR_INVALID, "null tensor pointer");
    if (a->routes > 0 && (a->topk_ids == nullptr || a->x == nullptr || a->scale == nullptr || a->route_rank == nullptr || a->dest_row == nullptr))
        return tb::set_last_error(TB_ERR_INVALID, "null tensor pointer");
    tb::PushParams p = {};
    if (int rc = fill_peers(&p.a, a->peer_a, a->world, "activation")) return rc;
    if (int rc = fill_peers(&p.a_scale, a->peer_a_scale, a->world, "scale")) return rc;
    if (a->peer_row_target != nullptr) {
        if (a->routes >= (1 << 26) || a->world > 32) return tb::set_last_error(TB_ERR_INVALID, "row targets hold 26 bits of route and 5 of rank");
        if (int rc = fill_peers(&p.row_target, a->peer_row_target, a->world, "row target")) return rc;
        if (a->out != nullptr && (a->out_row_bytes <= 0 || a->out_row_bytes % 16 != 0))
            return tb::set_last_error(TB_ERR_INVALID, "out_row_bytes must be a positive multiple of 16");
        p.out = static_cast<uint8_t*>(a->out);
        p.out_row_bytes = static_cast<int>(a->out_row_bytes);
    }
    p.ids = a->topk_ids; p.x = static_cast<const uint8_t*>(a->x); p.scale = a->scale; p.route_rank = a->route_rank;
    p.all_counts = a->all_counts; p.dest_row = a->dest_row; p.counts = a->counts; p.routes = a->routes; p.ids_int64 = a->ids_int64;
    p.top_k = a->top_k; p.num_experts = a->num_experts; p.world = a->world; p.rank = a->rank; p.interleaved = a->interleaved;
    p.capacity = a->capacity; p.width = static_cast<int>(a->width); p.groups = static_cast<int>(a->groups);
    tb::ep_push_kernel<<<row_grid(a->routes), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    TB_EP_CUDA(cudaGetLastError());
    return TB_OK;
}

int tb_ep_pull(void* stream, const void* topk_ids, int ids_int64, const int32_t* dest_row, int64_t routes, int32_t num_experts,
               int32_t world, int32_t interleaved, void* const* peer_y, int64_t row_bytes, void* out) {
    if (routes < 0 || num_experts <= 0 || world <= 0 || num_experts % world != 0 || row_bytes <= 0 || row_bytes % 16 != 0)
        return tb::set_last_error(TB_ERR_INVALID, "bad pull shape");
    if (routes == 0) return TB_OK;
    if (topk_ids == nullptr || dest_row == nullptr || out == nullptr) return tb::set_last_error(TB_ERR_INVALID, "null tensor pointer");
    tb::PullParams p = {};
    if (int rc = fill_peers(&p.y, peer_y, world, "output")) return rc;
    p.ids = topk_ids; p.dest_row = dest_row; p.out = static_cast<uint8_t*>(out); p.routes = routes; p.ids_int64 = ids_int64;
    p.num_experts = num_experts; p.world = world; p.interleaved = interleaved; p.row_bytes = static_cast<int>(row_bytes);
    tb::ep_pull_kernel<<<row_grid(routes), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    TB_EP_CUDA(cudaGetLastError());
    return TB_OK;
}

}  // extern "C"
