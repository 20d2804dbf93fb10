// PTX wrappers shared by the tcgen05 kernels: mbarriers with bounded waits, TMA and bulk copies,
// tensor-memory allocation, MMA issue and commit, accumulator loads, shared-memory descriptors.
#pragma once

#include <cuda.h>

#include "oxq_common.cuh"

namespace oxq {

constexpr unsigned long long TC_WAIT_LIMIT_NS = 2000000000ull; // 2 s: every spin on an mbarrier gives up after this

// ---- PTX wrappers ---------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// One poll that lets the hardware park the thread for up to `ns` nanoseconds while the phase is incomplete
// (it resumes at once when the phase completes). Without the hint a failed poll returns almost immediately,
// and a dozen threads polling in a loop keep the shared-memory pipeline busy enough to slow every other warp.
__device__ __forceinline__ bool mbar_test_parked(uint32_t bar, uint32_t parity, uint32_t ns)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity), "r"(ns)
                 : "memory");
    return ok != 0;
}
// Bounded wait: false (and `code` recorded) when the barrier did not flip within the limit. The wall clock
// (slow to read) is only consulted after a good number of parked polls.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int *flag, int code,
                                          unsigned long long limit_ns = TC_WAIT_LIMIT_NS)
{
    if (mbar_test(bar, parity)) return true;
#ifndef OXQ_WAIT_MODE
#define OXQ_WAIT_MODE 0
#endif
#if OXQ_WAIT_MODE == 0
#define OXQ_POLL() mbar_test_parked(bar, parity, 20000u)
#elif OXQ_WAIT_MODE == 1
#define OXQ_POLL() (__nanosleep(64), mbar_test(bar, parity))
#else
#define OXQ_POLL() mbar_test(bar, parity)
#endif
#pragma unroll 1
    for (int i = 0; i < 64; i++)
        if (OXQ_POLL()) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; i++)
            if (OXQ_POLL()) return true;
        if (global_ns() - t0 > limit_ns) {
            atomicCAS(flag, 0, code);
            return false;
        }
    }
}
// The same for a whole warp: lane 0 waits, every lane gets the outcome (and is ordered after the wait).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, int *flag, int code)
{
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, flag, code) ? 1 : 0;
    return __shfl_sync(0xFFFFFFFFu, ok, 0) != 0;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
                 : "memory");
}

// Untiled bulk copy global -> shared: both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xFFFFFFFF;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 x bf16 -> f32.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// Arrive on an mbarrier once all tcgen05.mma issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row
// groups 1024 bytes apart (SBO), descriptor version 1 (Blackwell), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t kmajor_sw128_desc(uint32_t smem_addr)
{
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// Instruction descriptor: D f32, A and B bf16, both K-major, N and M of the instruction.
__host__ __device__ constexpr uint32_t tc_idesc(int m, int n)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---- host side: the driver's tensor-map encoder, looked up once ----
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}


// 2-D tiled tensor map through a small per-thread cache. A tensor map is a pure function of these arguments, and
// the driver call that encodes one costs several microseconds, which a decode call cannot afford on every launch.
inline CUresult encode_tiled_2d(CUtensorMap *out, CUtensorMapDataType dtype, const void *ptr, uint64_t dim0, uint64_t dim1,
                                uint64_t stride1_bytes, uint32_t box0, uint32_t box1, CUtensorMapSwizzle swizzle,
                                CUtensorMapL2promotion promo)
{
    struct Entry {
        const void *ptr;
        uint64_t dim0, dim1, stride;
        uint32_t box0, box1;
        int dtype, swizzle, promo, valid;
        CUtensorMap map;
    };
    constexpr int SLOTS = 256;
    static thread_local Entry cache[SLOTS];
    const uintptr_t a = reinterpret_cast<uintptr_t>(ptr);
    Entry &e = cache[((a >> 8) ^ (a >> 20) ^ box1 ^ (dim1 << 3)) & (SLOTS - 1)];
    if (e.valid && e.ptr == ptr && e.dim0 == dim0 && e.dim1 == dim1 && e.stride == stride1_bytes && e.box0 == box0 &&
        e.box1 == box1 && e.dtype == (int)dtype && e.swizzle == (int)swizzle && e.promo == (int)promo) {
        *out = e.map;
        return CUDA_SUCCESS;
    }
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return CUDA_ERROR_NOT_SUPPORTED;
    const cuuint64_t dims[2] = {dim0, dim1};
    const cuuint64_t strides[1] = {stride1_bytes};
    const cuuint32_t box[2] = {box0, box1};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(out, dtype, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                          promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) {
        e.ptr = ptr; e.dim0 = dim0; e.dim1 = dim1; e.stride = stride1_bytes; e.box0 = box0; e.box1 = box1;
        e.dtype = (int)dtype; e.swizzle = (int)swizzle; e.promo = (int)promo; e.map = *out; e.valid = 1;
    }
    return r;
}

} // namespace oxq
