// Body shared by the tb_inst_*.cu translation units: instantiate and launch one variant of gemm_kernel.
#pragma once

#include <mutex>

#include "tb_launch.cuh"

namespace tb {

constexpr int kSmemOptIn = 227 * 1024;

template <int BM, bool kExact, bool kGroupScales, int kWarps, int kTeams>
int launch_instance(cudaStream_t stream, const GemmParams& params, int grid, size_t smem, bool pdl) {
    auto kernel = gemm_kernel<BM, kExact, kGroupScales, kWarps, kTeams>;
    static std::mutex mutex;
    static bool configured[64] = {};
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return static_cast<int>(err);
    if (device >= 0 && device < 64) {
        std::lock_guard<std::mutex> guard(mutex);
        if (!configured[device]) {
            err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemOptIn);
            if (err != cudaSuccess) return static_cast<int>(err);
            // An instance whose warpgroups trade registers must own enough of them, or its epilogue would wait for ever.
            if (min_kernel_registers(BM, kGroupScales, kWarps) > 0) {
                cudaFuncAttributes attributes;
                err = cudaFuncGetAttributes(&attributes, kernel);
                if (err != cudaSuccess) return static_cast<int>(err);
                if (attributes.numRegs < min_kernel_registers(BM, kGroupScales, kWarps)) return kLaunchUnsupported;
            }
            configured[device] = true;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(gemm_threads(BM, kWarps));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, kernel, params));
}

template <bool kExact, bool kGroupScales, int kWarps, int kTeams>
int launch_by_tile(int bm, cudaStream_t stream, const GemmParams& params, int grid, size_t smem, bool pdl) {
    switch (bm) {
        case 16: return launch_instance<16, kExact, kGroupScales, kWarps, kTeams>(stream, params, grid, smem, pdl);
        case 32: return launch_instance<32, kExact, kGroupScales, kWarps, kTeams>(stream, params, grid, smem, pdl);
        case 64: return launch_instance<64, kExact, kGroupScales, kWarps, kTeams>(stream, params, grid, smem, pdl);
        case 128: return launch_instance<128, kExact, kGroupScales, kWarps, kTeams>(stream, params, grid, smem, pdl);
        default: break;
    }
    if constexpr (!kGroupScales) {
        if (bm == 192) return launch_instance<192, kExact, false, kWarps, kTeams>(stream, params, grid, smem, pdl);
        if (bm == 256) return launch_instance<256, kExact, false, kWarps, kTeams>(stream, params, grid, smem, pdl);
    }
    return kLaunchUnsupported;
}

template <int kWarps, int kTeams>
int launch_variant(int bm, bool exact, bool group_scales, cudaStream_t stream, const GemmParams& params, int grid,
                   size_t smem, bool pdl) {
    if (group_scales) {
        return exact ? launch_by_tile<true, true, kWarps, kTeams>(bm, stream, params, grid, smem, pdl)
                     : launch_by_tile<false, true, kWarps, kTeams>(bm, stream, params, grid, smem, pdl);
    }
    return exact ? launch_by_tile<true, false, kWarps, kTeams>(bm, stream, params, grid, smem, pdl)
                 : launch_by_tile<false, false, kWarps, kTeams>(bm, stream, params, grid, smem, pdl);
}

}  // namespace tb

#define TB_DEFINE_VARIANT(name, warps, teams)                                                                     \
    namespace tb {                                                                                            \
    int name(int bm, bool exact, bool group_scales, cudaStream_t stream, const GemmParams& params, int grid,  \
             size_t smem, bool pdl) {                                                                         \
        return launch_variant<warps, teams>(bm, exact, group_scales, stream, params, grid, smem, pdl);        \
    }                                                                                                         \
    }
