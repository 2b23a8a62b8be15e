// Thin inline-PTX wrappers for sm_100a: mbarrier, bulk/TMA copies, tcgen05 (UMMA + tensor memory), fences, PDL.
// Every wait is bounded: it gives up after a cycle budget, records a code and returns false, so a kernel can
// unwind and report an error instead of hanging.
#pragma once

#ifdef __CUDACC_RTC__
// Run-time compilation (NVRTC) has no host headers: the fixed-width integers and an opaque tensor map of the right size
// and alignment are all the kernels need from them.
typedef unsigned char uint8_t;
typedef unsigned short uint16_t;
typedef unsigned int uint32_t;
typedef unsigned long long uint64_t;
typedef unsigned long long uintptr_t;
struct alignas(64) CUtensorMap_st { unsigned long long opaque[16]; };
typedef CUtensorMap_st CUtensorMap;
#else
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#endif

namespace tb {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier --------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Default cycle budget of one wait: about a second at the B200's clocks.
constexpr long long kWaitCycles = 1ll << 31;

// Waits for the phase with `parity` of `bar` to complete.  Returns false when `budget` cycles run out or another
// thread of the CTA has already given up (`*abort_flag != 0`); the first thread to give up stores `code`.
// `sleep_ns` > 0 backs off between polls: for waits that last a whole main loop, so that the polling warps stay out of
// the way of the warps doing the work (they share the issue slots and the shared-memory pipe).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code,
                                          unsigned sleep_ns = 0, long long budget = kWaitCycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if (sleep_ns != 0) __nanosleep(sleep_ns);
        if ((spin & 63u) == 0u) {
            if (*abort_flag != 0) return false;
            if (clock64() - start > budget) {
                atomicCAS(const_cast<int*>(abort_flag), 0, code);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Makes generic-proxy shared-memory writes of this thread visible to the async proxy (TMA, UMMA).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- bulk copies -------------------------------------------------------------------------------------
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

// Tiled 2D TMA load; `x` is the innermost coordinate (x * element size must be a multiple of 16 bytes).
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst_smem), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// 16-byte asynchronous copy global -> shared (non-bulk), zero-filling when `valid` is false.
__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void* src, bool valid) {
    const uint32_t src_bytes = valid ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes) : "memory");
}

// Arrive on `bar` once all cp.async of this thread issued so far have landed (counts as a plain arrival).
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- programmatic dependent launch ---------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait_prior_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- tensor memory ----------------------------------------------------------------------------------
// Whole-warp calls.  `columns` is a power of two in [32, 512]; the base address lands in shared memory.
__device__ __forceinline__ void tmem_alloc(uint32_t result_smem, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_smem), "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// mbarrier arrival once every tcgen05.mma this thread issued before has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], FP8/FP6/FP4 kind, one CTA.  `accumulate` = 0 overwrites D.
__device__ __forceinline__ void umma_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Same product with the A operand in tensor memory: 128 lanes (rows of A) x 8 columns of 32 bits (32 FP8 values of K)
// starting at `a_tmem`.
__device__ __forceinline__ void umma_f8f6f4_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Shared-memory operand descriptor: K-major rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart.
// `addr` is the shared address of the first row (tile base 1024-byte aligned) plus the K offset in bytes.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t addr) {
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);  // start address
    desc |= static_cast<uint64_t>(1) << 16;                   // leading byte offset (unused with swizzle): 16 B
    desc |= static_cast<uint64_t>(1024 >> 4) << 32;           // stride byte offset between 8-row groups
    desc |= static_cast<uint64_t>(1) << 46;                   // descriptor version of sm_100
    desc |= static_cast<uint64_t>(2) << 61;                   // SWIZZLE_128B
    return desc;
}

// Instruction descriptor: E4M3 x E4M3 -> FP32, both operands K-major, M = 128 rows, N = `n` columns.
__host__ __device__ constexpr uint32_t umma_idesc_e4m3(uint32_t m, uint32_t n) {
    return (1u << 4)            // D format FP32
           | (0u << 7)          // A format E4M3
           | (0u << 10)         // B format E4M3
           | ((n >> 3) << 17)   // N / 8
           | ((m >> 4) << 24);  // M / 16
}

// 32 lanes x 16 consecutive 32-bit columns of tensor memory -> 16 registers per thread (lane = thread).
__device__ __forceinline__ void tmem_ld_16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// The same for 8 consecutive columns.
__device__ __forceinline__ void tmem_ld_8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
// 8 registers per thread -> 8 consecutive 32-bit columns of this thread's lane (lane = 32 * (warp % 4) + thread lane).
__device__ __forceinline__ void tmem_st_8(uint32_t taddr, const uint4& a, const uint4& b) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 16 lanes x 16 columns in the layout of an MMA accumulator fragment: thread t gets lanes t / 4 (r0, r1 and r4, r5)
// and t / 4 + 8 (r2, r3 and r6, r7) of the 16 lanes that start at the address's lane, columns 2 * (t % 4) and + 1 of
// the first eight columns (r0..r3) and of the second eight (r4..r7).
__device__ __forceinline__ void tmem_ld_16x256b_x2(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
// Waits for the loads in flight, tied to the registers of two of them: nothing that reads those moves above the wait.
__device__ __forceinline__ void tmem_ld_wait_for(uint32_t (&a)[8], uint32_t (&b)[8]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]),
                   "+r"(b[0]), "+r"(b[1]), "+r"(b[2]), "+r"(b[3]), "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7])
                 :
                 : "memory");
}
// Four 8 x 8 matrices of 16-bit elements, transposed on the way: thread t holds elements [t / 4][2 * (t % 4)] and
// [t / 4][2 * (t % 4) + 1] of each matrix (one register per matrix, first element in the low half); element [r][c]
// lands at position r of the 16-byte row whose address thread 8 * matrix + c passed.
__device__ __forceinline__ void stmatrix_x4_trans(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
                 : "memory");
}
__device__ __forceinline__ uint4 lds_128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}

// ---- register shares ----------------------------------------------------------------------------------
// Whole-warpgroup calls (four consecutive warps starting at a multiple of four, all of their threads).
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs)); }
template <int kRegs>
__device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs)); }

// (x, y) += (a, b) * (s, t) as one packed FP32 instruction.
__device__ __forceinline__ void fma2(float& x, float& y, float a, float b, float s, float t) {
    asm("{\n\t.reg .b64 acc, lhs, rhs;\n\t"
        "mov.b64 acc, {%0, %1};\n\tmov.b64 lhs, {%2, %3};\n\tmov.b64 rhs, {%4, %5};\n\t"
        "fma.rn.f32x2 acc, lhs, rhs, acc;\n\t"
        "mov.b64 {%0, %1}, acc;\n\t}\n"
        : "+f"(x), "+f"(y)
        : "f"(a), "f"(b), "f"(s), "f"(t));
}

// ---- misc --------------------------------------------------------------------------------------------
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ uint32_t prmt(uint32_t lo, uint32_t hi, uint32_t sel) {
    uint32_t out;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(lo), "r"(hi), "r"(sel));
    return out;
}

// (a & b) | c
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t out;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(out) : "r"(a), "r"(b), "r"(c));
    return out;
}

}  // namespace tb
