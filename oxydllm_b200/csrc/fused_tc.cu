// AWQ W4A16 matmul for batches of up to 256 tokens with the dequantization fused into the tensor-core
// kernel: the packed words are read from HBM once and no dense copy of the weight is ever written.
//
// One CTA owns 128 out features and walks k in stages of 64 input rows:
//   warp 0 (one lane)   TMA: boxes of packed words (64 rows x 16 words, 4 KB) into a ring of up to 32 slots,
//                       as far ahead as the ring allows: this ring is what is in flight from HBM;
//   warp 2 (one lane)   TMA: the stage's tile of x ([tokens, 64] bf16, 128-byte swizzle) into one of the
//                       two or four operand slots;
//   warps 4..19         unpack, two teams of eight warps taking stages in turn: every thread turns four
//                       packed words into 4 x 8 bf16 weights, the same bits the dequantization kernel
//                       writes ((128 + q) - (128 + z) exactly in bf16, times the scale with one
//                       rounding: see split_scales), and stores each word's
//                       eight out features, which are neighbours in memory in the MN-major operand
//                       layout, with one 16-byte store;
//   warp 1 (one lane)   tcgen05.mma kind::f16, A = weights (bf16, MN-major, 128-byte swizzle: 64 out
//                       features x 8 input rows per 1 KB atom), B = x (bf16, K-major), D[128, tokens] f32
//                       in tensor memory for the whole of k; a commit per stage frees the slots;
//   warps 4..19         epilogue: accumulator rows (out features) -> registers -> + bias -> y[token, n].
// Every wait is bounded and reports through the workspace flag word.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "tc_common.cuh"

namespace oxq {

constexpr int FT_ROWS = 128;
constexpr int FT_BK = 64;
constexpr int FT_TEAM_WARPS = 8;                 // warps that unpack one stage together (256 threads x 4 words)
constexpr int FT_TEAMS = 2;                      // teams take stages in turn, so one team's store-fence-arrive tail overlaps the other's unpack
constexpr int FT_UNPACK_WARPS = FT_TEAM_WARPS * FT_TEAMS;
constexpr int FT_THREADS = (4 + FT_UNPACK_WARPS) * 32;
constexpr int FT_BOX_BYTES = FT_BK * 16 * 4;      // 64 input rows x 16 packed words
constexpr int FT_ZERO_BYTES = 64, FT_SCALE_BYTES = 256; // the box's group: 16 zero-point words, 128 16-bit scales
constexpr int FT_RAW_BYTES = FT_BOX_BYTES + 384;  // ring slot: box | zero points | scales | pad to 128 bytes
constexpr int FT_A_BYTES = FT_ROWS * FT_BK * 2;
constexpr int FT_MAX_STAGES = 4;                 // operand slots (A tile + x tile)
constexpr int FT_MAX_RAW = 32;                   // ring slots of packed boxes: what is in flight from HBM
constexpr int FT_NUM_BARS = 2 * FT_MAX_RAW + 3 * FT_MAX_STAGES + 1;
constexpr int FT_MAX_M = 256;
constexpr int FT_SMEM_BUDGET = 227 * 1024;

#ifdef OXQ_TUNING
__device__ long long g_ft_trace[12][64]; // clock stamps of CTA 0, per role and stage (tuning builds only)
#define FT_TRACE(role, it) do { if (blockIdx.x == 0 && (it) < 64) g_ft_trace[role][it] = clock64(); } while (0)
#else
#define FT_TRACE(role, it) do { } while (0)
#endif

struct FusedParams {
    const uint32_t *qzeros;
    const void *scales;
    int scales_dtype;
    const void *bias;
    void *y;
    int bias_dtype, y_dtype;
    int m, mpad, k, n, group_size, packed_out;
    int stages, raw_slots, stage_bytes, tmem_cols;
    int col_base, ldy; // y column of out feature 0 and the row pitch of y in elements
    int *flag;
};

// A operand: 16-bit, MN-major, 128-byte swizzle. An atom is 8 input rows x 64 out features (1 KB); atoms of
// later input rows follow at 1 KB (stride byte offset), the second 64 out features at 8 KB (leading byte offset).
__device__ __forceinline__ uint64_t ft_a_desc(uint32_t smem_addr)
{
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)(8192 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// D f32, A bf16 MN-major, B bf16 K-major.
__device__ __forceinline__ uint32_t ft_idesc(int n)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(FT_ROWS >> 4) << 24);
}

__global__ void __launch_bounds__(FT_THREADS, 1)
    awq_fused_tc_kernel(const FusedParams p, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap)
{
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u; // operand slots want 1 KB alignment
    unsigned char *base_ptr = smem_raw + (base - smem_u32(smem_raw));
    // operand slots (A tile + x tile) | ring of packed boxes | barriers | tensor-memory address
    const int S = p.stages, R = p.raw_slots;
    const uint32_t raw_base = (uint32_t)S * p.stage_bytes;
    const uint32_t bars = base + raw_base + (uint32_t)R * FT_RAW_BYTES;
    auto rawfull_bar = [&](int r) { return bars + 8u * r; };
    auto rawempty_bar = [&](int r) { return bars + 8u * (FT_MAX_RAW + r); };
    auto xfull_bar = [&](int s) { return bars + 8u * (2 * FT_MAX_RAW + s); };
    auto ready_bar = [&](int s) { return bars + 8u * (2 * FT_MAX_RAW + FT_MAX_STAGES + s); };
    auto empty_bar = [&](int s) { return bars + 8u * (2 * FT_MAX_RAW + 2 * FT_MAX_STAGES + s); };
    const uint32_t acc_bar = bars + 8u * (2 * FT_MAX_RAW + 3 * FT_MAX_STAGES);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(base_ptr + raw_base + (size_t)R * FT_RAW_BYTES + 8 * FT_NUM_BARS);
    const uint32_t b_off = FT_A_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * FT_ROWS;
    const int nk = p.k / FT_BK;

    if (threadIdx.x == 0) {
        for (int r = 0; r < R; r++) {
            mbar_init(rawfull_bar(r), 1);
            mbar_init(rawempty_bar(r), FT_TEAM_WARPS);
        }
        for (int s = 0; s < S; s++) {
            mbar_init(xfull_bar(s), 1);
            mbar_init(ready_bar(s), FT_TEAM_WARPS);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(acc_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) { // the allocating warp also frees
        tmem_alloc(smem_u32(tmem_slot), (uint32_t)p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA, packed words: runs as far ahead of the unpack teams as the ring of boxes allows ------------
        if (elect_one()) {
            int r = 0;
            uint32_t ph = 0;
            for (int it = 0; it < nk; it++) {
                if (it >= R && !mbar_wait(rawempty_bar(r), ph ^ 1u, p.flag, 1)) break;
                const uint32_t dst = base + raw_base + (uint32_t)r * FT_RAW_BYTES;
                const int qg = it * FT_BK / p.group_size;
                mbar_arrive_expect_tx(rawfull_bar(r), FT_BOX_BYTES + FT_ZERO_BYTES + FT_SCALE_BYTES);
                tma_load_2d(dst, &wmap, rawfull_bar(r), n0 / 8, it * FT_BK);
                // the group's zero points and scales travel with the box: a plain load issued by the unpack threads
                // would wait a full DRAM round trip per group
                bulk_copy_g2s(dst + FT_BOX_BYTES, p.qzeros + (size_t)qg * p.packed_out + n0 / 8, FT_ZERO_BYTES, rawfull_bar(r));
                bulk_copy_g2s(dst + FT_BOX_BYTES + FT_ZERO_BYTES,
                              reinterpret_cast<const uint16_t *>(p.scales) + (size_t)qg * p.n + n0, FT_SCALE_BYTES, rawfull_bar(r));
                FT_TRACE(0, it);
                if (++r == R) { r = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 2) {
        // ---- TMA, x tiles: one per operand slot, as soon as the MMAs that read the slot have completed --------
        if (elect_one()) {
            int s = 0;
            uint32_t ph = 0;
            for (int it = 0; it < nk; it++) {
                if (it >= S && !mbar_wait(empty_bar(s), ph ^ 1u, p.flag, 5)) break;
                mbar_arrive_expect_tx(xfull_bar(s), (uint32_t)p.mpad * 128u);
                tma_load_2d(base + (uint32_t)s * p.stage_bytes + b_off, &xmap, xfull_bar(s), it * FT_BK, 0);
                if (++s == S) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue -------------------------------------------------------------------------------
        if (elect_one()) {
            const uint32_t idesc = ft_idesc(p.mpad);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int it = 0; it < nk; it++) {
                ok = mbar_wait(ready_bar(s), ph, p.flag, 2) && mbar_wait(xfull_bar(s), ph, p.flag, 6);
                if (!ok) break;
                FT_TRACE(1, it);
                tc_fence_after();
                const uint32_t slot = base + (uint32_t)s * p.stage_bytes;
                const uint64_t da = ft_a_desc(slot), db = kmajor_sw128_desc(slot + b_off);
#pragma unroll
                for (int kk = 0; kk < FT_BK / 16; kk++) // 16 input rows: two 1 KB atoms of A, 32 bytes inside the swizzled row of B
                    umma_bf16(tmem_base, da + (uint64_t)kk * (2048 >> 4), db + 2 * kk, idesc, (it | kk) != 0);
                umma_commit(empty_bar(s));
                FT_TRACE(2, it);
                if (++s == S) { s = 0; ph ^= 1u; }
            }
            if (ok) umma_commit(acc_bar);
        }
    } else if (warp >= 4) {
        // ---- unpack ------------------------------------------------------------------------------------
        // S and R are multiples of the number of teams, so a slot always meets the same team: every waiter
        // of a barrier sees each of its phases.
        const int team = (warp - 4) / FT_TEAM_WARPS;
        const int ut = (threadIdx.x - 128) % (FT_TEAM_WARPS * 32); // 0..255 inside the team
        const int j = ut & 15, r0 = ut >> 4;  // word column (8 out features) and first of this thread's four rows
        const int gstages = p.group_size / FT_BK;
        // A scale s (f16: 11 significant bits) is used as s_hi + s_lo, two bf16 values that
        // add up to it exactly; for d = q - z (an integer of at most 4 bits) d * s_lo is exact in bf16 and
        // fma(d, s_hi, d * s_lo) rounds the exact d * s once: the bits of bf16(f32(d) * f32(s)).
        const bool sc_f16 = p.scales_dtype == OXQ_F16;
        auto split_scales = [&](const uint4 &raw, __nv_bfloat162 (&hi)[4], __nv_bfloat162 (&lo)[4]) {
            const uint32_t tv[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                if (sc_f16) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&tv[i]));
                    hi[i] = __floats2bfloat162_rn(f.x, f.y);
                    const float2 h = __bfloat1622float2(hi[i]);
                    lo[i] = __floats2bfloat162_rn(f.x - h.x, f.y - h.y); // exact: at most four significant bits
                } else {
                    hi[i] = *reinterpret_cast<const __nv_bfloat162 *>(&tv[i]);
                    lo[i] = __floats2bfloat162_rn(0.0f, 0.0f);
                }
            }
        };
        int cur_qg = -1;
        __nv_bfloat162 zp[4], shi[4], slo[4];
        // byte offset of this thread's first 16-byte chunk inside the A slot; rows r0 + 16 i are 2 KB apart
        const uint32_t a_off = (uint32_t)(j >> 3) * 8192u + (uint32_t)(r0 >> 3) * 1024u + (uint32_t)(r0 & 7) * 128u +
                               (uint32_t)(((j & 7) ^ (r0 & 7)) << 4);
        const uint32_t raw_idx = raw_base + (uint32_t)(r0 * 16 + j) * 4u;
        int s = team % S, r = team % R;
        uint32_t ph = (uint32_t)(team / S) & 1u, rph = (uint32_t)(team / R) & 1u;
        bool ok = true;
        for (int it = team; it < nk; it += FT_TEAMS) {
            // the box: four words into registers, then the ring slot goes back to the producer
            if (ut == 0) FT_TRACE(7, it);
            ok = mbar_wait(rawfull_bar(r), rph, p.flag, 3);
            if (!ok) break;
            if (ut == 0) FT_TRACE(3, it);
            const unsigned char *raw = base_ptr + raw_idx + (size_t)r * FT_RAW_BYTES;
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) w[i] = *reinterpret_cast<const uint32_t *>(raw + i * 16 * 64);
            if (ut == 0) FT_TRACE(8, it);
            const int qg = it / gstages;
            if (qg != cur_qg) { // a new quantization group: its zero points and scales sit behind the box
                cur_qg = qg;
                const unsigned char *aux = base_ptr + raw_base + (size_t)r * FT_RAW_BYTES + FT_BOX_BYTES;
                const uint32_t zw = *reinterpret_cast<const uint32_t *>(aux + 4 * j);
                split_scales(*reinterpret_cast<const uint4 *>(aux + FT_ZERO_BYTES + 16 * j), shi, slo);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t v = ((zw >> (4 * i)) & 0x000F000Fu) | 0x43004300u; // bf16 pair (128 + z, 128 + z')
                    zp[i] = *reinterpret_cast<const __nv_bfloat162 *>(&v);
                }
            }
            if (ut == 0) FT_TRACE(9, it);
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(rawempty_bar(r)) : "memory");
            if (ut == 0) FT_TRACE(10, it);
            // the operand slot is free once the MMAs of the stage that used it last have completed
            if (it >= S) {
                ok = mbar_wait(empty_bar(s), ph ^ 1u, p.flag, 7);
                if (!ok) break;
            }
            unsigned char *slot = base_ptr + (size_t)s * p.stage_bytes;
            if (ut == 0) FT_TRACE(6, it);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint4 o;
                uint32_t *ov = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
                for (int q = 0; q < 4; q++) { // nibbles q and q + 4 are out features 2q and 2q + 1 of the word
                    const uint32_t v = ((w[i] >> (4 * q)) & 0x000F000Fu) | 0x43004300u; // bf16 pair (128 + q, 128 + q')
                    const __nv_bfloat162 d = __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&v), zp[q]); // q - z, exact
                    const __nv_bfloat162 b2 = __hfma2(d, shi[q], __hmul2(d, slo[q]));
                    ov[q] = *reinterpret_cast<const uint32_t *>(&b2);
                }
                *reinterpret_cast<uint4 *>(slot + a_off + i * 2048) = o;
            }
            if (ut == 0) FT_TRACE(4, it);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic-proxy stores -> visible to the MMA
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ready_bar(s)) : "memory");
            if (ut == 0) FT_TRACE(5, it);
            s += FT_TEAMS;
            while (s >= S) { s -= S; ph ^= 1u; }
            r += FT_TEAMS;
            while (r >= R) { r -= R; rph ^= 1u; }
        }

        // ---- epilogue: lane = out feature inside this warp's quarter of the accumulator rows -----------------
        if (ok) ok = mbar_wait(acc_bar, 0, p.flag, 4);
        if (ok) {
            tc_fence_after();
            const int quad = warp & 3, turn = (warp - 4) >> 2; // the warps of a quarter take 32-token chunks in turn
            const int ncol = n0 + quad * 32 + lane;
            const float bv = p.bias ? load_as_f32(p.bias, p.bias_dtype, (size_t)p.col_base + ncol) : 0.0f;
            for (int c0 = 32 * turn; c0 < p.mpad; c0 += 32 * (FT_UNPACK_WARPS / 4)) {
                uint32_t rr[32];
                tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, rr);
                tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; c++)
                    if (c0 + c < p.m)
                        store_as(p.y, p.y_dtype, (size_t)(c0 + c) * p.ldy + p.col_base + ncol, __uint_as_float(rr[c]) + bv);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    }
}

// True when the fused kernel serves this call; otherwise the caller dequantizes into a slab.
bool awq_fused_supported(int m, int k, int n, int group_size, int scales_dtype, const void *x, const void *qweight,
                         const void *scales)
{
    if (const char *env = tuning_env("OXQ_AWQ_FUSED"))
        if (env[0] == '0') return false;
    return m >= 1 && m <= FT_MAX_M && n % FT_ROWS == 0 && k % FT_BK == 0 && group_size % FT_BK == 0 &&
           (scales_dtype == OXQ_F16 || scales_dtype == OXQ_BF16) && aligned(x, 16) && aligned(qweight, 16) && aligned(scales, 16);
}

int awq_fused_matmul(const void *x, const uint32_t *qweight, const uint32_t *qzeros, const void *scales, int scales_dtype, const void *bias,
                     int bias_dtype, void *y, int y_dtype, int m, int k, int n, int group_size, int col_base, int ldy,
                     int *flag, cudaStream_t st)
{
    EncodeTiledFn fn = encode_tiled_fn();
    OXQ_REQUIRE(fn != nullptr, OXQ_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    FusedParams p;
    p.qzeros = qzeros; p.scales = scales; p.scales_dtype = scales_dtype; p.bias = bias; p.y = y;
    p.bias_dtype = bias_dtype; p.y_dtype = y_dtype;
    p.m = m; p.mpad = (m + 15) / 16 * 16; p.k = k; p.n = n; p.group_size = group_size; p.packed_out = n / 8;
    p.col_base = col_base; p.ldy = ldy; p.flag = flag;
    p.stage_bytes = FT_A_BYTES + p.mpad * 128;
    const int fixed = 1024 + 8 * FT_NUM_BARS + 16;
    const int nk = k / FT_BK;
    // Operand slots: four when that still leaves eight boxes in flight, else two; the rest of shared memory is the
    // ring of packed boxes. Both counts are multiples of the number of unpack teams.
    p.stages = (FT_SMEM_BUDGET - fixed - 8 * FT_RAW_BYTES) / p.stage_bytes >= 4 ? 4 : 2;
    p.raw_slots = (FT_SMEM_BUDGET - fixed - p.stages * p.stage_bytes) / FT_RAW_BYTES / FT_TEAMS * FT_TEAMS;
    if (p.raw_slots > FT_MAX_RAW) p.raw_slots = FT_MAX_RAW;
    if (const char *env = tuning_env("OXQ_AWQ_FUSED_RAW")) p.raw_slots = atoi(env) < p.raw_slots ? atoi(env) : p.raw_slots;
    OXQ_REQUIRE(p.raw_slots >= FT_TEAMS && nk >= 1, OXQ_ERR_UNSUPPORTED, "awq_fused_matmul: no room for the ring of boxes");
    p.tmem_cols = 32;
    while (p.tmem_cols < p.mpad) p.tmem_cols *= 2;
    const size_t smem = (size_t)p.stages * p.stage_bytes + (size_t)p.raw_slots * FT_RAW_BYTES + fixed;

    CUtensorMap wmap, xmap;
    {
        const cuuint64_t dims[2] = {(cuuint64_t)p.packed_out, (cuuint64_t)k};
        const cuuint64_t strides[1] = {(cuuint64_t)p.packed_out * 4};
        const cuuint32_t box[2] = {16, FT_BK};
        const cuuint32_t estr[2] = {1, 1};
        CUresult r = fn(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<uint32_t *>(qweight), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        OXQ_REQUIRE(r == CUDA_SUCCESS, OXQ_ERR_CUDA, "cuTensorMapEncodeTiled (weights) failed with CUresult %d", (int)r);
    }
    {
        const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)m};
        const cuuint64_t strides[1] = {(cuuint64_t)k * 2};
        const cuuint32_t box[2] = {FT_BK, (cuuint32_t)p.mpad};
        const cuuint32_t estr[2] = {1, 1};
        CUresult r = fn(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(x), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        OXQ_REQUIRE(r == CUDA_SUCCESS, OXQ_ERR_CUDA, "cuTensorMapEncodeTiled (x) failed with CUresult %d", (int)r);
    }

    static size_t configured[64] = {};
    int device = 0;
    OXQ_CUDA(cudaGetDevice(&device));
    if (device >= 64 || configured[device] < smem) {
        OXQ_CUDA(cudaFuncSetAttribute(awq_fused_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (device < 64) configured[device] = smem;
    }
    awq_fused_tc_kernel<<<n / FT_ROWS, FT_THREADS, smem, st>>>(p, wmap, xmap);
    OXQ_CUDA(cudaGetLastError());
    return OXQ_OK;
}

} // namespace oxq

#ifdef OXQ_TUNING
OXQ_EXPORT int oxq_ft_trace_read(long long *host_out)
{
    return cudaMemcpyFromSymbol(host_out, oxq::g_ft_trace, sizeof(long long) * 12 * 64) == cudaSuccess ? 0 : -6;
}
#endif
