// Prefill-sized matmuls on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   y[m, n] = x[m, k] . W[n, k]^T (+ bias),  x bf16, W bf16 (a dequantized slab), f32 accumulation
//
// A persistent CTA per SM walks 128 x BN output tiles (BN <= 256 picked per call). Warp-specialised:
//   warp 0     TMA producer: x tile [128 x 64] and W tile [BN x 64] per k block, both K-major,
//              128-byte swizzle, 4-stage ring guarded by full/empty mbarriers;
//   warp 1     MMA issuer: one elected lane issues tcgen05.mma (cta_group::1, kind::f16, M=128,
//              N=BN, K=16) on shared-memory descriptors into one of two TMEM accumulators, so the
//              epilogue of a tile overlaps the MMAs of the next;
//              tcgen05.commit releases ring slots and finally signals the epilogue;
//   warps 2-5  epilogue: tcgen05.ld 32 lanes x 32 columns at a time, bias, narrowing, stores.
// Every wait is bounded (wall-clock limit); on expiry the kernel records a code in the caller's
// flag word, all roles fall through, TMEM is released and the kernel returns.
// With more than one 128-row tile of x the dense GEMM runs as pairs of CTAs (tcgen05 cta_group::2):
// a pair shares a 256 x BN tile and each CTA stages only half of the W tile (see the two-CTA kernel).
//
// The quantized entry points dequantize W in slabs of rows into the caller's workspace with the
// bit-exact dequantization kernels and run this GEMM per slab: the B operand the tensor cores
// see is exactly the dense weight the reference materialises (awq.rs:325-440, linear.rs:96-141).
#include <cstdlib>

#include "tc_common.cuh"

namespace oxq {

constexpr int TC_BM = 128;
constexpr int TC_BN = 256;
constexpr int TC_BK = 64;
constexpr int TC_STAGES = 4;
constexpr int TC_UMMA_K = 16;
constexpr uint32_t TC_A_BYTES = TC_BM * TC_BK * 2;
constexpr uint32_t TC_B_BYTES = TC_BN * TC_BK * 2;
constexpr uint32_t TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;
constexpr size_t TC_SMEM_BYTES = 1024 /* alignment slack */ + (size_t)TC_STAGES * TC_STAGE_BYTES + 256 /* barriers */;
constexpr int TC_BN_CHOICES[] = {256, 224, 192, 160, 128};

struct GemmParams {
    const void *bias;
    void *y;
    int *flag;
    int bias_dtype, y_dtype;
    int m, n, k;      // n = rows of W in this call (a slab); y columns [n_off, n_off + n)
    int n_off, ldy;   // ldy = full out_features
    int tiles_m, tiles_n, bn; // tile grid of this call; bn = tile width (multiple of 32, <= 256)
    int test_skip_loads; // self-test only: the TMA producer issues nothing, so the waits of the other roles run out
    int epi; // 0: y = acc (+ bias). 1 / 2: W rows interleave (gate j, up j); y[:, j] = SiLU / GeLU-tanh(gate) * up, bf16 [m, n/2]
};

// Gated FFN activations on f32 (ffn.rs:385-470: act(gate) * up).
__device__ __forceinline__ float gated_act(float gate, float up, int epi)
{
    if (epi == 1) return gate * __fdividef(1.0f, 1.0f + __expf(-gate)) * up;
    const float t = tanhf(0.7978845608028654f * (gate + 0.044715f * gate * gate * gate));
    return 0.5f * gate * (1.0f + t) * up;
}

// One 32-column chunk of one accumulator row: bias, optional gated activation, narrowing, store.
__device__ __forceinline__ void gemm_store_chunk(const GemmParams &p, const uint32_t (&r)[32], int row, int col0, bool vec_ok)
{
    if (row < p.m && col0 < p.n && p.epi != 0) {
        // 32 accumulator columns = 16 (gate, up) pairs -> 16 outputs of this lane's row
        __nv_bfloat16 *yo = reinterpret_cast<__nv_bfloat16 *>(p.y) + (size_t)row * p.ldy + ((p.n_off + col0) >> 1);
        float act[16];
#pragma unroll
        for (int j = 0; j < 16; j++) {
            float gate = __uint_as_float(r[2 * j]), up = __uint_as_float(r[2 * j + 1]);
            if (p.bias) {
                gate += load_as_f32(p.bias, p.bias_dtype, p.n_off + col0 + 2 * j);
                up += load_as_f32(p.bias, p.bias_dtype, p.n_off + col0 + 2 * j + 1);
            }
            act[j] = gated_act(gate, up, p.epi);
        }
        if (vec_ok && col0 + 32 <= p.n) {
            uint32_t packed[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                __nv_bfloat162 h2 = __floats2bfloat162_rn(act[2 * j], act[2 * j + 1]);
                packed[j] = *reinterpret_cast<uint32_t *>(&h2);
            }
            uint4 *dst = reinterpret_cast<uint4 *>(yo);
            dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        } else {
#pragma unroll
            for (int j = 0; j < 16; j++)
                if (col0 + 2 * j < p.n) yo[j] = __float2bfloat16_rn(act[j]);
        }
    } else if (row < p.m && col0 < p.n) {
        const size_t out = (size_t)row * p.ldy + p.n_off + col0;
        if (vec_ok && col0 + 32 <= p.n) {
            uint32_t packed[16];
#pragma unroll
            for (int j = 0; j < 16; j++) {
                float v0 = __uint_as_float(r[2 * j]), v1 = __uint_as_float(r[2 * j + 1]);
                if (p.bias) {
                    v0 += load_as_f32(p.bias, p.bias_dtype, p.n_off + col0 + 2 * j);
                    v1 += load_as_f32(p.bias, p.bias_dtype, p.n_off + col0 + 2 * j + 1);
                }
                __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
                packed[j] = *reinterpret_cast<uint32_t *>(&h);
            }
            uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(p.y) + out);
#pragma unroll
            for (int q = 0; q < 4; q++)
                dst[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++) {
                if (col0 + j < p.n) {
                    float v = __uint_as_float(r[j]);
                    if (p.bias) v += load_as_f32(p.bias, p.bias_dtype, p.n_off + col0 + j);
                    store_as(p.y, p.y_dtype, out + j, v);
                }
            }
        }
    }
}

// Persistent kernel: CTA c handles tiles c, c + gridDim.x, ... (m fastest, so CTAs running together
// share W tiles through L2). Two TMEM accumulators (2 x 256 columns) let the epilogue of one tile
// overlap the MMAs of the next. `bn` (a multiple of 32, <= 256) is the tile width chosen by the host.
__global__ void __launch_bounds__(192, 1)
gemm_bf16_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmParams p)
{
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u; // swizzled tiles need 1024-byte alignment
    unsigned char *base_ptr = smem_raw + (base - raw);
    const uint32_t bars = base + TC_STAGES * TC_STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (TC_STAGES + s); };
    auto tmem_full_bar = [&](int b) { return bars + 8u * (2 * TC_STAGES + b); };
    auto tmem_empty_bar = [&](int b) { return bars + 8u * (2 * TC_STAGES + 2 + b); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(base_ptr + TC_STAGES * TC_STAGE_BYTES + 8 * (2 * TC_STAGES + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_iters = (p.k + TC_BK - 1) / TC_BK;
    const int num_tiles = p.tiles_m * p.tiles_n;
    const uint32_t stage_tx = TC_A_BYTES + (uint32_t)p.bn * TC_BK * 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(tmem_full_bar(b), 1);
            mbar_init(tmem_empty_bar(b), 4); // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) { // the allocating warp also frees
        tmem_alloc(smem_u32(tmem_slot), 2 * TC_BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (elect_one()) {
            uint32_t it = 0; // k blocks issued so far by this CTA, across tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok && !p.test_skip_loads; tile += gridDim.x) {
                const int m0 = (tile % p.tiles_m) * TC_BM, n0 = (tile / p.tiles_m) * p.bn;
                for (int kb = 0; kb < k_iters; kb++, it++) {
                    const int s = it % TC_STAGES;
                    ok = mbar_wait(empty_bar(s), ((it / TC_STAGES) & 1) ^ 1, p.flag, 1);
                    if (!ok) break;
                    mbar_arrive_expect_tx(full_bar(s), stage_tx);
                    const uint32_t sa = base + s * TC_STAGE_BYTES, sb = sa + TC_A_BYTES;
                    tma_load_2d(sa, &map_a, full_bar(s), kb * TC_BK, m0);
                    tma_load_2d(sb, &map_b, full_bar(s), kb * TC_BK, n0);
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            const uint32_t idesc = tc_idesc(TC_BM, p.bn);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, local++) {
                const int buf = local & 1;
                ok = mbar_wait(tmem_empty_bar(buf), ((local >> 1) & 1) ^ 1, p.flag, 4);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * TC_BN;
                for (int kb = 0; kb < k_iters; kb++, it++) {
                    const int s = it % TC_STAGES;
                    ok = mbar_wait(full_bar(s), (it / TC_STAGES) & 1, p.flag, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = base + s * TC_STAGE_BYTES, sb = sa + TC_A_BYTES;
                    const uint64_t da = kmajor_sw128_desc(sa), db = kmajor_sw128_desc(sb);
#pragma unroll
                    for (int kk = 0; kk < TC_BK / TC_UMMA_K; kk++) {
                        // 16 bf16 along k = 32 bytes inside the 128-byte swizzled row: +2 in the address field
                        umma_bf16(d_tmem, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0);
                    }
                    umma_commit(empty_bar(s)); // slot reusable once these MMAs have read it
                }
                umma_commit(tmem_full_bar(buf)); // accumulator complete (arrives even after an aborted loop)
            }
        }
    } else {
        // Epilogue: warp w may touch TMEM lanes 32*(w%4) .. +31 only.
        const int quad = warp & 3;
        const bool vec_ok = p.y_dtype == OXQ_BF16 && (p.ldy % 8 == 0) && (p.n_off % 8 == 0) &&
                            (reinterpret_cast<uintptr_t>(p.y) & 15) == 0;
        uint32_t local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, local++) {
            const int buf = local & 1;
            const int m0 = (tile % p.tiles_m) * TC_BM, n0 = (tile / p.tiles_m) * p.bn;
            const int row = m0 + quad * 32 + lane;
            ok = mbar_wait(tmem_full_bar(buf), (local >> 1) & 1, p.flag, 3);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tc_fence_after();
#pragma unroll 1
            for (int cb = 0; cb < p.bn / 32; cb++) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + buf * TC_BN + cb * 32, r);
                tmem_ld_wait();
                gemm_store_chunk(p, r, row, n0 + cb * 32, vec_ok);
            }
            // This warp has drained its quarter of the accumulator: hand the buffer back.
            tc_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tmem_empty_bar(buf)) : "memory");
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * TC_BN);
    }
}

// ---- two-CTA variant (tcgen05 cta_group::2) -----------------------------------------------------
// A cluster of two CTAs on neighbouring SMs computes one 256 x BN tile: CTA r of the pair owns rows
// 128 r .. 128 r + 127 of it (its own x tile, its own 128 TMEM lanes) and loads only HALF of the W
// tile (rows n0 + r BN/2 .. of W); the MMA, issued by the even CTA alone, reads both halves out of
// the two CTAs' shared memory. Per k block an SM stages 16 KB of x and BN/2 x 128 B of W instead of
// BN x 128 B, which is what the one-CTA kernel is short of (operand traffic per tensor-core cycle).
// Protocol: both CTAs issue their TMA loads with cta_group::2 so that the bytes are counted on the
// even CTA's full barrier; tcgen05.commit with a two-CTA multicast releases ring slots and
// accumulators in both CTAs; the epilogue warps of both CTAs arrive on the even CTA's
// accumulator-free barrier. All waits are bounded as in the one-CTA kernel.
constexpr int TC2_STAGES = 6;
constexpr uint32_t TC2_B_BYTES = (TC_BN / 2) * TC_BK * 2;
constexpr uint32_t TC2_STAGE_BYTES = TC_A_BYTES + TC2_B_BYTES;
constexpr size_t TC2_SMEM_BYTES = 1024 + (size_t)TC2_STAGES * TC2_STAGE_BYTES + 256;
constexpr uint32_t TC_PEER_BIT_MASK = 0xFEFFFFFFu; // clears the CTA-rank bit of a shared::cluster address: the even CTA's copy

__device__ __forceinline__ void tma_load_2d_2cta(uint32_t dst, const CUtensorMap *map, uint32_t bar_even, int c0, int c1)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar_even), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void umma_bf16_2cta(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    const uint32_t z = 0u;
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(z)
                 : "memory");
}
// Arrive on the barrier at the same offset in both CTAs once the MMAs issued so far have completed.
__device__ __forceinline__ void umma_commit_2cta(uint32_t bar)
{
    const unsigned short mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(mask)
                 : "memory");
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_cta_rank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__global__ void __launch_bounds__(192, 1)
gemm_bf16_tn_2cta_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const GemmParams p)
{
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u; // swizzled tiles need 1024-byte alignment
    unsigned char *base_ptr = smem_raw + (base - raw);
    const uint32_t bars = base + TC2_STAGES * TC2_STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (TC2_STAGES + s); };
    auto tmem_full_bar = [&](int b) { return bars + 8u * (2 * TC2_STAGES + b); };
    auto tmem_empty_bar = [&](int b) { return bars + 8u * (2 * TC2_STAGES + 2 + b); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(base_ptr + TC2_STAGES * TC2_STAGE_BYTES + 8 * (2 * TC2_STAGES + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank(); // 0: issues the MMAs, 1: its partner
    const int k_iters = (p.k + TC_BK - 1) / TC_BK;
    const int pair_m = (p.tiles_m + 1) / 2;             // 256-row tiles
    const int num_tiles = pair_m * p.tiles_n;
    const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
    const uint32_t half_b = (uint32_t)(p.bn / 2) * TC_BK * 2;
    const uint32_t stage_tx = 2u * (TC_A_BYTES + half_b); // both CTAs' copies land on the even CTA's barrier

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC2_STAGES; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(tmem_full_bar(b), 1);
            mbar_init(tmem_empty_bar(b), 8); // one arrival per epilogue warp of both CTAs (used in the even CTA only)
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) { // the allocating warp (the same warp index in both CTAs) also frees
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * TC_BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all(); // barriers of both CTAs exist before anything is signalled across the pair
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (elect_one()) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < num_tiles && ok && !p.test_skip_loads; tile += num_clusters) {
                const int m0 = ((tile % pair_m) * 2 + (int)rank) * TC_BM;                  // this CTA's 128 rows
                const int n0 = (tile / pair_m) * p.bn + (int)rank * (p.bn / 2);           // this CTA's half of the W rows
                for (int kb = 0; kb < k_iters; kb++, it++) {
                    const int s = it % TC2_STAGES;
                    ok = mbar_wait(empty_bar(s), ((it / TC2_STAGES) & 1) ^ 1, p.flag, 1);
                    if (!ok) break;
                    if (rank == 0) mbar_arrive_expect_tx(full_bar(s), stage_tx);
                    const uint32_t sa = base + s * TC2_STAGE_BYTES, sb = sa + TC_A_BYTES;
                    const uint32_t bar_even = full_bar(s) & TC_PEER_BIT_MASK;
                    tma_load_2d_2cta(sa, &map_a, bar_even, kb * TC_BK, m0);
                    tma_load_2d_2cta(sb, &map_b, bar_even, kb * TC_BK, n0);
                }
            }
        }
    } else if (warp == 1) {
        if (rank == 0 && elect_one()) {
            const uint32_t idesc = tc_idesc(2 * TC_BM, p.bn);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, local++) {
                const int buf = local & 1;
                ok = mbar_wait(tmem_empty_bar(buf), ((local >> 1) & 1) ^ 1, p.flag, 4);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * TC_BN;
                for (int kb = 0; kb < k_iters; kb++, it++) {
                    const int s = it % TC2_STAGES;
                    ok = mbar_wait(full_bar(s), (it / TC2_STAGES) & 1, p.flag, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = base + s * TC2_STAGE_BYTES, sb = sa + TC_A_BYTES;
                    const uint64_t da = kmajor_sw128_desc(sa), db = kmajor_sw128_desc(sb);
#pragma unroll
                    for (int kk = 0; kk < TC_BK / TC_UMMA_K; kk++)
                        umma_bf16_2cta(d_tmem, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0);
                    umma_commit_2cta(empty_bar(s)); // slot reusable in both CTAs once these MMAs have read it
                }
                umma_commit_2cta(tmem_full_bar(buf)); // accumulator complete in both CTAs
            }
        }
    } else {
        const int quad = warp & 3;
        const bool vec_ok = p.y_dtype == OXQ_BF16 && (p.ldy % 8 == 0) && (p.n_off % 8 == 0) &&
                            (reinterpret_cast<uintptr_t>(p.y) & 15) == 0;
        uint32_t local = 0;
        bool ok = true;
        for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters, local++) {
            const int buf = local & 1;
            const int m0 = ((tile % pair_m) * 2 + (int)rank) * TC_BM, n0 = (tile / pair_m) * p.bn;
            const int row = m0 + quad * 32 + lane;
            ok = mbar_wait(tmem_full_bar(buf), (local >> 1) & 1, p.flag, 3);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tc_fence_after();
#pragma unroll 1
            for (int cb = 0; cb < p.bn / 32; cb++) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + buf * TC_BN + cb * 32, r);
                tmem_ld_wait();
                gemm_store_chunk(p, r, row, n0 + cb * 32, vec_ok);
            }
            // This warp has drained its quarter of its CTA's accumulator: tell the MMA issuer (even CTA).
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(tmem_empty_bar(buf) & TC_PEER_BIT_MASK) : "memory");
        }
        tc_fence_before();
    }
    __syncthreads();
    cluster_sync_all(); // neither CTA frees tensor memory or leaves while its partner may still use the pair
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * TC_BN) : "memory");
    }
}

// ---- grouped (ragged-batch) variant for the MoE expert layer -----------------------------------
// Same pipeline; the tiles come from a device-side table built by the routing kernels, so no host
// round trip is needed: entry = {first row in the expert-sorted activation matrix, valid rows,
// expert id}. B rows of expert e start at (e - e_first) * nw in the dequantized slab.
// epi 0: out[row, col] = acc + bias[e, col]                      (bf16, [rows, nw])
// epi 1: GPT-OSS clamped SwiGLU on interleaved (gate, up) columns (bf16, [rows, nw / 2]):
//        gate = min(g, limit), up = clamp(u, +-limit), out = (up + 1) * gate * sigmoid(1.702 gate)
struct GroupedParams {
    const int4 *entries;
    const int *grp_beg;
    const void *bias;
    void *out;
    int *flag;
    int group, e_first, nw, k, tiles_n, bn, bias_dtype, ldo, epi, vec_ok;
    float limit;
};

__global__ void __launch_bounds__(192, 1)
gemm_grouped_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GroupedParams p)
{
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char *base_ptr = smem_raw + (base - raw);
    const uint32_t bars = base + TC_STAGES * TC_STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (TC_STAGES + s); };
    auto tmem_full_bar = [&](int b) { return bars + 8u * (2 * TC_STAGES + b); };
    auto tmem_empty_bar = [&](int b) { return bars + 8u * (2 * TC_STAGES + 2 + b); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(base_ptr + TC_STAGES * TC_STAGE_BYTES + 8 * (2 * TC_STAGES + 4));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_iters = (p.k + TC_BK - 1) / TC_BK;
    const int mt_beg = p.grp_beg[p.group];
    const int num_mt = p.grp_beg[p.group + 1] - mt_beg;
    const int num_tiles = num_mt * p.tiles_n;
    const uint32_t stage_tx = TC_A_BYTES + (uint32_t)p.bn * TC_BK * 2;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(tmem_full_bar(b), 1);
            mbar_init(tmem_empty_bar(b), 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 2 * TC_BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (elect_one()) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int4 en = p.entries[mt_beg + tile % num_mt];
                const int n0 = (tile / num_mt) * p.bn;
                const int brow = (en.z - p.e_first) * p.nw + n0;
                for (int kb = 0; kb < k_iters; kb++, it++) {
                    const int s = it % TC_STAGES;
                    ok = mbar_wait(empty_bar(s), ((it / TC_STAGES) & 1) ^ 1, p.flag, 1);
                    if (!ok) break;
                    mbar_arrive_expect_tx(full_bar(s), stage_tx);
                    const uint32_t sa = base + s * TC_STAGE_BYTES, sb = sa + TC_A_BYTES;
                    tma_load_2d(sa, &map_a, full_bar(s), kb * TC_BK, en.x);
                    tma_load_2d(sb, &map_b, full_bar(s), kb * TC_BK, brow);
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            const uint32_t idesc = tc_idesc(TC_BM, p.bn);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, local++) {
                const int buf = local & 1;
                ok = mbar_wait(tmem_empty_bar(buf), ((local >> 1) & 1) ^ 1, p.flag, 4);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * TC_BN;
                for (int kb = 0; kb < k_iters; kb++, it++) {
                    const int s = it % TC_STAGES;
                    ok = mbar_wait(full_bar(s), (it / TC_STAGES) & 1, p.flag, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = base + s * TC_STAGE_BYTES, sb = sa + TC_A_BYTES;
                    const uint64_t da = kmajor_sw128_desc(sa), db = kmajor_sw128_desc(sb);
#pragma unroll
                    for (int kk = 0; kk < TC_BK / TC_UMMA_K; kk++)
                        umma_bf16(d_tmem, da + 2 * kk, db + 2 * kk, idesc, (kb | kk) != 0);
                    umma_commit(empty_bar(s));
                }
                umma_commit(tmem_full_bar(buf));
            }
        }
    } else {
        const int quad = warp & 3;
        uint32_t local = 0;
        bool ok = true;
        __nv_bfloat16 *outp = reinterpret_cast<__nv_bfloat16 *>(p.out);
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, local++) {
            const int buf = local & 1;
            const int4 en = p.entries[mt_beg + tile % num_mt];
            const int n0 = (tile / num_mt) * p.bn;
            const int r_in = quad * 32 + lane;
            const size_t row = (size_t)en.x + r_in;
            ok = mbar_wait(tmem_full_bar(buf), (local >> 1) & 1, p.flag, 3);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tc_fence_after();
#pragma unroll 1
            for (int cb = 0; cb < p.bn / 32; cb++) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + buf * TC_BN + cb * 32, r);
                tmem_ld_wait();
                const int col0 = n0 + cb * 32;
                if (r_in < en.y && col0 < p.nw) {
                    const size_t bcol = (size_t)en.z * p.nw + col0;
                    const bool full = p.vec_ok && col0 + 32 <= p.nw;
                    float bv[32]; // bias of the 32 columns (the same for every lane: broadcast loads)
                    if (p.bias && full && p.bias_dtype == OXQ_BF16 && (bcol & 7) == 0) {
                        const uint4 *bp = reinterpret_cast<const uint4 *>(reinterpret_cast<const __nv_bfloat16 *>(p.bias) + bcol);
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const uint4 t = __ldg(bp + q);
                            const uint32_t tw[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                            for (int u = 0; u < 4; u++) {
                                bv[8 * q + 2 * u] = __uint_as_float(tw[u] << 16);
                                bv[8 * q + 2 * u + 1] = __uint_as_float(tw[u] & 0xFFFF0000u);
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            bv[j] = (p.bias && col0 + j < p.nw) ? load_as_f32(p.bias, p.bias_dtype, bcol + j) : 0.0f;
                    }
                    if (p.epi == 0) {
                        if (full) { // 32 columns = 64 bytes of this lane's row
                            uint32_t packed[16];
#pragma unroll
                            for (int j = 0; j < 16; j++) {
                                __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[2 * j]) + bv[2 * j],
                                                                          __uint_as_float(r[2 * j + 1]) + bv[2 * j + 1]);
                                packed[j] = *reinterpret_cast<uint32_t *>(&h2);
                            }
                            uint4 *dst = reinterpret_cast<uint4 *>(outp + row * p.ldo + col0);
#pragma unroll
                            for (int q = 0; q < 4; q++)
                                dst[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j += 2) {
                                if (col0 + j < p.nw) { // nw is even
                                    *reinterpret_cast<__nv_bfloat162 *>(outp + row * p.ldo + col0 + j) =
                                        __floats2bfloat162_rn(__uint_as_float(r[j]) + bv[j], __uint_as_float(r[j + 1]) + bv[j + 1]);
                                }
                            }
                        }
                    } else {
                        float act[16];
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            float gate = __uint_as_float(r[2 * j]) + bv[2 * j], up = __uint_as_float(r[2 * j + 1]) + bv[2 * j + 1];
                            gate = fminf(gate, p.limit);
                            up = fminf(fmaxf(up, -p.limit), p.limit);
                            const float sig = __fdividef(1.0f, __expf(-1.702f * gate) + 1.0f);
                            act[j] = (up + 1.0f) * (gate * sig);
                        }
                        if (full) { // 16 outputs = 32 bytes of this lane's row
                            uint32_t packed[8];
#pragma unroll
                            for (int j = 0; j < 8; j++) {
                                __nv_bfloat162 h2 = __floats2bfloat162_rn(act[2 * j], act[2 * j + 1]);
                                packed[j] = *reinterpret_cast<uint32_t *>(&h2);
                            }
                            uint4 *dst = reinterpret_cast<uint4 *>(outp + row * p.ldo + (col0 >> 1));
                            dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                            dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; j++)
                                if (col0 + 2 * j < p.nw) outp[row * p.ldo + ((col0 >> 1) + j)] = __float2bfloat16_rn(act[j]);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tmem_empty_bar(buf)) : "memory");
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * TC_BN);
    }
}

// ---- host side ---------------------------------------------------------------
// 2-D bf16 row-major [rows, cols] tensor, box [box_rows, 64 cols], 128-byte swizzle, zero fill.
static int make_map_bf16(CUtensorMap *map, const void *ptr, uint64_t rows, uint64_t cols, uint32_t box_rows)
{
    const CUresult r = encode_tiled_2d(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, ptr, cols, rows, cols * 2, (uint32_t)TC_BK, box_rows,
                                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    OXQ_REQUIRE(r == CUDA_SUCCESS, OXQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return OXQ_OK;
}

// Tile width that minimises (rounds of the persistent grid) x (time of one tile ~ bn + fixed cost).
int gemm_pick_bn(int m, int n)
{
    const int sms = sm_count(), tiles_m = ceil_div(m, TC_BM);
    long long best_cost = -1;
    int best = TC_BN;
    for (int bn : TC_BN_CHOICES) {
        const long long tiles = (long long)tiles_m * ceil_div(n, bn);
        const long long rounds = (tiles + sms - 1) / sms;
        const long long cost = rounds * (bn + 24);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
    }
    return best;
}

// The same for the two-CTA kernel: 256-row tiles, one cluster of two CTAs per tile, sm_count / 2 clusters.
int gemm_pick_bn_2cta(int m, int n)
{
    const int clusters = sm_count() / 2, pair_m = (ceil_div(m, TC_BM) + 1) / 2;
    long long best_cost = -1;
    int best = TC_BN;
    for (int bn : TC_BN_CHOICES) {
        const long long tiles = (long long)pair_m * ceil_div(n, bn);
        const long long rounds = (tiles + clusters - 1) / clusters;
        const long long cost = rounds * (bn + 24);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; }
    }
    return best;
}

// y[:, n_off : n_off + n] = x[m, k] . w[n, k]^T (+ bias) with x, w bf16 row-major.
static thread_local int g_selftest_skip_loads = 0; // set only inside oxq_selftest_gemm_wait_expiry

int gemm_bf16_tn(const void *x, const void *w, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int n,
                 int k, int n_off, int ldy, int *flag, cudaStream_t stream, int epi)
{
    OXQ_REQUIRE(epi == 0 || (y_dtype == OXQ_BF16 && n % 2 == 0 && n_off % 2 == 0), OXQ_ERR_UNSUPPORTED,
                "gated epilogue needs bf16 output and an even number of interleaved columns");
    OXQ_REQUIRE(aligned(x, 16) && aligned(w, 16), OXQ_ERR_BAD_ALIGN, "tensor-core GEMM operands must be 16-byte aligned");
    OXQ_REQUIRE(k % 8 == 0, OXQ_ERR_UNSUPPORTED, "tensor-core GEMM needs in_features %% 8 == 0 (got %d)", k);
    // More than one 128-row tile: pairs of CTAs share 256-row tiles (two-CTA kernel) unless switched off.
    const char *env2 = tuning_env("OXQ_GEMM_2CTA"); // bench-harness knob: "0" keeps the one-CTA kernel
    const bool two_cta = m > TC_BM && !(env2 && env2[0] == '0');
    const int bn = two_cta ? gemm_pick_bn_2cta(m, n) : gemm_pick_bn(m, n);
    CUtensorMap map_a, map_b;
    int rc = make_map_bf16(&map_a, x, (uint64_t)m, (uint64_t)k, TC_BM);
    if (rc) return rc;
    rc = make_map_bf16(&map_b, w, (uint64_t)n, (uint64_t)k, (uint32_t)bn);
    if (rc) return rc;
    static bool configured[64] = {};
    int device = 0;
    OXQ_CUDA(cudaGetDevice(&device));
    if (device >= 64 || !configured[device]) {
        OXQ_CUDA(cudaFuncSetAttribute(gemm_bf16_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_BYTES));
        if (device < 64) configured[device] = true;
    }
    GemmParams p;
    p.test_skip_loads = g_selftest_skip_loads;
    p.bias = bias; p.y = y; p.flag = flag; p.bias_dtype = bias_dtype; p.y_dtype = y_dtype;
    p.m = m; p.n = n; p.k = k; p.n_off = n_off; p.ldy = ldy; p.epi = epi;
    p.tiles_m = ceil_div(m, TC_BM); p.tiles_n = ceil_div(n, bn); p.bn = bn;
    const int tiles = p.tiles_m * p.tiles_n, sms = sm_count();
    if (two_cta) {
        // W box of half a tile per CTA; pairs of CTAs share a 256-row tile.
        rc = make_map_bf16(&map_b, w, (uint64_t)n, (uint64_t)k, (uint32_t)(bn / 2));
        if (rc) return rc;
        static bool configured2[64] = {};
        if (device >= 64 || !configured2[device]) {
            OXQ_CUDA(cudaFuncSetAttribute(gemm_bf16_tn_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC2_SMEM_BYTES));
            if (device < 64) configured2[device] = true;
        }
        const int pair_tiles = ((p.tiles_m + 1) / 2) * p.tiles_n;
        int clusters = sms / 2 < pair_tiles ? sms / 2 : pair_tiles;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * clusters, 1, 1);
        cfg.blockDim = dim3(192, 1, 1);
        cfg.dynamicSmemBytes = TC2_SMEM_BYTES;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        OXQ_CUDA(cudaLaunchKernelEx(&cfg, gemm_bf16_tn_2cta_kernel, map_a, map_b, p));
        return OXQ_OK;
    }
    gemm_bf16_tn_kernel<<<tiles < sms ? tiles : sms, 192, TC_SMEM_BYTES, stream>>>(map_a, map_b, p);
    OXQ_LAUNCH_CHECK("gemm_bf16_tn_kernel");
    return OXQ_OK;
}

// Grouped GEMM over the m tiles of expert group `group`: a = expert-sorted activations [a_rows, k],
// w = dequantized slab [slab_experts * nw, k]; out rows follow the sorted order.
int gemm_grouped(const void *a, int a_rows, const void *w, int slab_experts, int e_first, int nw, int k,
                 const int4 *entries, const int *grp_beg, int group, const void *bias, int bias_dtype, void *out,
                 int ldo, int epi, float limit, int *flag, cudaStream_t stream)
{
    OXQ_REQUIRE(aligned(a, 16) && aligned(w, 16), OXQ_ERR_BAD_ALIGN, "grouped GEMM operands must be 16-byte aligned");
    OXQ_REQUIRE(k % 8 == 0 && nw % 2 == 0, OXQ_ERR_UNSUPPORTED, "grouped GEMM needs in_features %% 8 == 0 and even out_features");
    int bn = TC_BN; // widest tile whose last column tile wastes the least
    {
        long long best = -1;
        for (int c : TC_BN_CHOICES) {
            const long long cost = (long long)ceil_div(nw, c) * (c + 24);
            if (best < 0 || cost < best) { best = cost; bn = c; }
        }
    }
    CUtensorMap map_a, map_b;
    int rc = make_map_bf16(&map_a, a, (uint64_t)a_rows, (uint64_t)k, TC_BM);
    if (rc) return rc;
    rc = make_map_bf16(&map_b, w, (uint64_t)slab_experts * nw, (uint64_t)k, (uint32_t)bn);
    if (rc) return rc;
    static bool configured[64] = {};
    int device = 0;
    OXQ_CUDA(cudaGetDevice(&device));
    if (device >= 64 || !configured[device]) {
        OXQ_CUDA(cudaFuncSetAttribute(gemm_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_BYTES));
        if (device < 64) configured[device] = true;
    }
    GroupedParams p;
    p.entries = entries; p.grp_beg = grp_beg; p.bias = bias; p.out = out; p.flag = flag;
    p.group = group; p.e_first = e_first; p.nw = nw; p.k = k; p.tiles_n = ceil_div(nw, bn); p.bn = bn;
    p.bias_dtype = bias_dtype; p.ldo = ldo; p.epi = epi; p.limit = limit;
    p.vec_ok = (ldo % 8 == 0 && aligned(out, 16)) ? 1 : 0;
    gemm_grouped_kernel<<<sm_count(), 192, TC_SMEM_BYTES, stream>>>(map_a, map_b, p);
    OXQ_LAUNCH_CHECK("gemm_grouped_kernel");
    return OXQ_OK;
}

} // namespace oxq

// One thread waits on an mbarrier that nothing ever arrives on, with a 50 ms limit: the wait must give up, record
// its code in the flag word and let the kernel end normally.
namespace oxq {
__global__ void wait_expiry_selftest_kernel(int *flag, int code)
{
    __shared__ __align__(8) unsigned long long bar;
    const uint32_t b = smem_u32(&bar);
    mbar_init(b, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_wait(b, 0, flag, code, 50000000ull);
}
} // namespace oxq

OXQ_EXPORT int oxq_selftest_wait_expiry(void *workspace, int code, void *stream)
{
    oxq::clear_error();
    OXQ_REQUIRE(workspace, OXQ_ERR_NULL, "oxq_selftest_wait_expiry: null workspace");
    OXQ_REQUIRE(code > 0, OXQ_ERR_BAD_SHAPE, "oxq_selftest_wait_expiry: code must be positive");
    oxq::wait_expiry_selftest_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(reinterpret_cast<int *>(workspace), code);
    OXQ_CUDA(cudaGetLastError());
    return OXQ_OK;
}

// The dense tensor-core GEMM (one-CTA kernel for m <= 128, two-CTA kernel above) with a producer that issues no
// loads: the MMA issuer's wait for the first tile data runs out (2 s), the roles fall through, tensor memory is freed
// and the kernel ends with code 2 in the flag word. Operands and output are scratch inside `workspace` (>= 1 MiB).
OXQ_EXPORT int oxq_selftest_gemm_wait_expiry(void *workspace, size_t workspace_bytes, int m, void *stream)
{
    oxq::clear_error();
    OXQ_REQUIRE(workspace && workspace_bytes >= (1u << 20) && oxq::aligned(workspace, 256), OXQ_ERR_WORKSPACE,
                "oxq_selftest_gemm_wait_expiry: 256-byte aligned workspace of at least 1 MiB needed");
    OXQ_REQUIRE(m >= 1 && m <= 256, OXQ_ERR_BAD_SHAPE, "oxq_selftest_gemm_wait_expiry: m in 1..256");
    unsigned char *b = reinterpret_cast<unsigned char *>(workspace);
    const int k = 64, n = 256;
    void *x = b + 4096, *w = b + 4096 + 256 * 64 * 2, *y = b + 4096 + 2 * 256 * 64 * 2; // x [256, 64], w [256, 64], y [256, 256] bf16
    oxq::g_selftest_skip_loads = 1;
    const int rc = oxq::gemm_bf16_tn(x, w, nullptr, 0, y, OXQ_BF16, m, n, k, 0, n, reinterpret_cast<int *>(workspace),
                                     (cudaStream_t)stream, 0);
    oxq::g_selftest_skip_loads = 0;
    return rc;
}
