// Shared device helpers for the sm_100a kernels: mbarrier wrappers with bounded waits, warp-level
// MMA, programmatic dependent launch, and the device status word.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tmb {

// Bits of the device status word (one unsigned per handle).  A kernel that gives up on a
// bounded wait ORs its bit in and finishes without touching its output any further.
enum : unsigned {
    kStatusGemmPipeWait  = 1u << 2,  // tcgen05 GEMM: a pipeline barrier (copies, expanded weight, MMA completion)
    kStatusGemmTmemWait  = 1u << 3,  // tcgen05 GEMM: accumulator hand-over or the partners of a split tile
    kStatusCommWait      = 1u << 6,  // peer-memory all-reduce: a peer's slot did not become ready in time
    kStatusPrefillOverflow = 1u << 5,  // prefill: a sequence's history + new tokens exceed the cache (session_len) or
                                       // its new tokens exceed max_q_len: the surplus rows were dropped
};

// Upper bound, in SM clock cycles, on one mbarrier wait (about 0.15-0.3 s): far above any
// legitimate wait (microseconds), far below a host-side watchdog.
constexpr long long kMaxWaitCycles = 1ll << 29;

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Same test, but the hardware may park the thread for up to `ns` nanoseconds until the phase completes:
// a waiting thread then costs no issue slots (a bare try_wait loop takes them from the warps that work).
__device__ __forceinline__ bool mbar_try_wait_sleep(uint64_t* bar, uint32_t parity, uint32_t ns)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when the time budget ran out (caller records the status bit).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, long long max_cycles = kMaxWaitCycles)
{
    if (mbar_try_wait(bar, parity)) {
        return true;
    }
    const long long t0 = clock64();
    while (!mbar_try_wait_sleep(bar, parity, 20000u)) {
        if (clock64() - t0 > max_cycles) {
            return false;
        }
    }
    return true;
}

// Programmatic dependent launch.  A kernel launched with the programmatic-serialization attribute may
// start while its predecessor in the stream is still running; pdl_wait() returns once that predecessor
// has completed and its writes are visible (a no-op for a normal launch).  Everything before it may
// only read data that no kernel writes (weights).  pdl_launch_dependents() lets the successor start;
// the kernels here call it after their own wait, so at most two kernels overlap.
__device__ __forceinline__ void pdl_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// D(16x8,f32) = A * B (the accumulator starts at zero)
__device__ __forceinline__ void mma_m16n8k16_init(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

// One packed word of the runtime int4 layout -> the four half2 registers of an m16n8k16 A
// fragment holding the exact integers (nibble - zero):
//   out[0] = nibbles {0,4} (row r,   k pair low)     out[1] = nibbles {1,5} (row r+8, k pair low)
//   out[2] = nibbles {2,6} (row r,   k pair high)    out[3] = nibbles {3,7} (row r+8, k pair high)
// `z1024_lo` = half2{1024 + z(row r)} ; `nz64_hi` = half2{-(64 + z(row r+8))}.
// 1024 + nib and (1024 + 16 nib) / 16 - (64 + z) are exact in fp16, so the result equals the
// reference's (64 + nib) - (64 + z) (kernels/gemm_s_f16/common.h:115-156, 218-235) bit for bit.
__device__ __forceinline__ void unpack_s4_minus_zero(uint32_t w, uint32_t z1024_lo, uint32_t nz64_hi, uint32_t (&out)[4])
{
    constexpr uint32_t kLut   = (0xf0 & 0xcc) | 0xaa;  // (a & b) | c
    constexpr uint32_t kBot   = 0x000f000f;
    constexpr uint32_t kTop   = 0x00f000f0;
    constexpr uint32_t kMagic = 0x64006400;  // half2{1024, 1024}
    constexpr uint32_t kSixteenth = 0x2c002c00;  // half2{1/16, 1/16}
    const uint32_t     hi     = w >> 8;
    uint32_t           t0, t1, t2, t3;
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(t0) : "r"(w), "n"(kBot), "n"(kMagic), "n"(kLut));
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(t1) : "r"(w), "n"(kTop), "n"(kMagic), "n"(kLut));
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(t2) : "r"(hi), "n"(kBot), "n"(kMagic), "n"(kLut));
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(t3) : "r"(hi), "n"(kTop), "n"(kMagic), "n"(kLut));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(out[0]) : "r"(t0), "r"(z1024_lo));
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(out[1]) : "r"(t1), "r"(kSixteenth), "r"(nz64_hi));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(out[2]) : "r"(t2), "r"(z1024_lo));
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(out[3]) : "r"(t3), "r"(kSixteenth), "r"(nz64_hi));
}

// Kernel launch with or without the programmatic-serialization attribute
template<typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, Args&&... args)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim          = grid;
    cfg.blockDim         = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream           = st;
    cudaLaunchAttribute attr[1];
    attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs                                          = attr;
    cfg.numAttrs                                       = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace tmb
