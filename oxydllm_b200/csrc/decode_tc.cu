// Batched decode matmul (1 <= m <= 32 tokens) of a packed 4-bit weight on the tcgen05 tensor cores.
//
//   y[m, n] = x[m, k] . W[n, k]^T (+ bias),   W = AWQ 4-bit, group scales and zero points
//
// The work is the stream of packed weights out of HBM, once; everything else is arranged so that the
// SM spends as few instructions and shared-memory bytes per weight as possible:
//
//  * Weights are the 128-row operand of the MMA (tcgen05.mma kind::f8f6f4, M = 128), tokens its columns,
//    so one unpack serves every token. The A operand is ONE BYTE per weight: the raw nibble q (0..15)
//    read as E4M3 is the subnormal/first-binade value q * 2^-9 exactly, so unpacking a packed word is two
//    masks and a shift, with no table, no conversion and no zero-point or scale arithmetic per weight.
//    A packed AWQ word holds 8 output columns of one input row; the bytes go to shared memory in the
//    MN-major (out-feature-contiguous) 128-byte-swizzled operand layout, which is the order they arrive
//    in. The interleaved column order of the AWQ word becomes a fixed permutation of accumulator rows
//    that the store undoes.
//  * Activations are bf16. Each value is written as the exact sum of three E5M2 numbers (3 + 3 + 2
//    significant bits) after a power-of-two scaling per (token, 128-wide k group) that places the
//    group's largest magnitude at the top of the E5M2 range; the three pieces are three neighbouring
//    columns of the B operand. Products of a 4-bit integer and a 3-bit significand are exact, the tensor
//    core adds them in f32. A small kernel launched in front (programmatic dependent launch: the main
//    kernel starts streaming weights while it runs) writes the pieces, per-group sums of x and the
//    scaling factors.
//  * Per 128-wide k group the accumulator [128 rows x tokens] is read from tensor memory by four warps
//    (one accumulator row per thread) and folded in f32:  tot += s * (512 * sum_pieces / 2^p - z * sum_x),
//    s and z being the group's scale and zero point of that row.
//  * One persistent CTA per SM. A unit of work is (H x 128 out features) x (one 128-wide k group); with
//    H = 2 a row of the packed tile is a whole 128-byte line of qweight. Units are dealt out in contiguous,
//    equal ranges, so every SM streams the same number of bytes whatever the shape. A tile that is shared
//    by several CTAs is summed through a workspace in a fixed order by the CTA that arrives last (fence +
//    counter, no spinning): same inputs, same bits.
//  * Roles: warps 0-3 issue the MMAs (warp i for stages i and i + 4); warps 4-7 fold; warps 8-15 each own
//    one stage of the ring: they load the packed words of their next half unit while they unpack and store
//    the current one, and copy the unit's token pieces (cp.async.bulk). Every wait on an mbarrier is bounded.
//    A single warp runs its instructions one after another, so what bounds the rate of the pipeline is the
//    length of the per-unit instruction path of its slowest role: the loops carry counters and pointers from
//    unit to unit instead of recomputing them.
#include <cuda_fp8.h>

#include <cstdlib>

#include "tc_common.cuh"

namespace oxq {

constexpr int DT_ROWS = 128;                        // out features per MMA = rows of one accumulator
constexpr int DT_UNIT_K = 128;                      // in features per unit = 4 MMAs of K = 32 per accumulator
constexpr uint32_t DT_A_BYTES = DT_ROWS * DT_UNIT_K; // one byte per weight
constexpr int DT_MMA_WARPS = 4;
constexpr int DT_FOLD_WARPS = 4;
constexpr int DT_UNPACK_WARPS = 8;
constexpr int DT_THREADS = 32 * (DT_MMA_WARPS + DT_FOLD_WARPS + DT_UNPACK_WARPS);
constexpr int DT_MAX_M = 32;
constexpr int DT_SZ_DEPTH = 8;                      // units of scales / zero points in flight per fold thread
constexpr size_t DT_WS_HEADER = 256;                // flag word
constexpr size_t DT_SMEM_BUDGET = 227 * 1024;

struct DecodeParams {
    const uint32_t *qweight, *qzeros;
    const void *scales, *bias;
    void *y;
    const unsigned char *xq; // [kgroups][np * 128] token pieces, operand layout, row 3 * token + piece
    const float2 *xs;        // [kgroups][q] {512 / 2^p, sum of x} per (k group, token)
    float *partials;         // [2 * ctas][H][q][128]
    int *counters;           // [tiles]
    int *flag;
    int scales_dtype, bias_dtype, y_dtype;
    int m, k, n, group_size, packed_out;
    int gshift;              // log2(group_size / 128): units per quantization group
    int q, np;               // token slots (power of two), rows of the B operand (multiple of 16)
    int tiles, kgroups, units;
    int stages, tmem_cols;   // stages (operands + accumulators), allocated tensor-memory columns
    uint32_t stage_bytes, x_bytes, xs_smem_bytes;
    int dbg;                 // experiments only (builds with OXQ_TUNING)
};

#ifdef OXQ_TUNING
__device__ long long g_dt_trace[16][64];
#define DT_TRACE(role, it) do { if (blockIdx.x == 0 && (it) < 64) g_dt_trace[role][it] = clock64(); } while (0)
__device__ unsigned long long g_dt_cta[160][8];
#define DT_CTA(slot) do { if (blockIdx.x < 160) g_dt_cta[blockIdx.x][slot] = global_ns(); } while (0)
#else
#define DT_TRACE(role, it) do { } while (0)
#define DT_CTA(slot) do { } while (0)
#endif

// Accumulator row r of a 128-row tile <-> out feature: 16-row chunks are two packed words, and inside a word the
// low-nibble bytes (slots 0, 2, 4, 6 = columns 0, 4, 1, 5) come before the high-nibble bytes (columns 2, 6, 3, 7).
__device__ __forceinline__ int row_to_col(int r)
{
    const int perm = (0x73625140u >> (4 * (r & 7))) & 7; // {0, 4, 1, 5, 2, 6, 3, 7}
    return (r & ~15) + ((r >> 3) & 1) * 8 + perm;
}

__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t *r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t *r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t *r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}

__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
}

// A operand: 8-bit, MN-major (128 out features contiguous = one 128-byte row per input row), 128-byte
// swizzle, groups of 8 input rows 1024 bytes apart.
__device__ __forceinline__ uint64_t mnmajor_sw128_desc(uint32_t smem_addr)
{
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// D f32, A E4M3 MN-major, B E5M2 K-major.
__host__ __device__ constexpr uint32_t decode_idesc(int n)
{
    return (1u << 4) | (0u << 7) | (1u << 10) | (1u << 15) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(DT_ROWS >> 4) << 24);
}

__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- token pieces ---------------------------------------------------------------------------------
// One warp per (token, 128-wide k group): lane l holds x[4 l .. 4 l + 3] of the group.
__global__ void __launch_bounds__(256)
decode_prep_kernel(const __nv_bfloat16 *__restrict__ x, unsigned char *__restrict__ xq, float2 *__restrict__ xs,
                   int *__restrict__ counters, int tiles, int m, int k, int q, int np)
{
    grid_launch_dependents(); // the matmul kernel may start now; it waits for this grid before touching xq / xs
    const int gthread = blockIdx.x * blockDim.x + threadIdx.x;
    if (gthread < tiles) counters[gthread] = 0;
    const int kgroups = k / DT_UNIT_K;
    const int gw = gthread >> 5, lane = threadIdx.x & 31;
    if (gw >= m * kgroups) return;
    const int tok = gw / kgroups, g = gw % kgroups;
    const uint2 raw = __ldg(reinterpret_cast<const uint2 *>(x + (size_t)tok * k + (size_t)g * DT_UNIT_K) + lane);
    float f[4] = {bf16_lo_f32(raw.x), bf16_hi_f32(raw.x), bf16_lo_f32(raw.y), bf16_hi_f32(raw.y)};
    float amax = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3])));
    float sum = (f[0] + f[1]) + (f[2] + f[3]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    }
    // 2^p puts the group's largest magnitude into [2^14, 2^15): the top binade of E5M2 below its maximum.
    int p = 0;
    if (amax > 0.0f) {
        p = 14 - ((int)((__float_as_uint(amax) >> 23) & 0xFFu) - 127);
        p = p > 126 ? 126 : (p < -112 ? -112 : p);
    }
    const float scale = __uint_as_float((uint32_t)(127 + p) << 23), inv = __uint_as_float((uint32_t)(127 - p) << 23);
    float r[4];
#pragma unroll
    for (int i = 0; i < 4; i++) r[i] = f[i] * scale;
    unsigned char *tile = xq + (size_t)g * np * 128;
#pragma unroll
    for (int piece = 0; piece < 3; piece++) {
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(r[0], r[1]), __NV_SATFINITE, __NV_E5M2);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(r[2], r[3]), __NV_SATFINITE, __NV_E5M2);
        const uint32_t word = lo | (hi << 16);
        // an E5M2 byte is the upper byte of the f16 of the same value
#pragma unroll
        for (int i = 0; i < 4; i++) r[i] -= __half2float(__ushort_as_half((unsigned short)(((word >> (8 * i)) & 0xFFu) << 8)));
        const int row = 3 * tok + piece; // the three pieces of a token are neighbouring accumulator columns
        const uint32_t off = (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u +
                             ((uint32_t)((lane >> 2) ^ (row & 7)) << 4) + (uint32_t)(lane & 3) * 4u;
        *reinterpret_cast<uint32_t *>(tile + off) = word;
    }
    if (lane == 0) xs[(size_t)g * q + tok] = make_float2(512.0f * inv, sum);
}

// ---- the matmul ------------------------------------------------------------------------------------
// Stage s of the ring = H operand tiles A (16 KB each) + token pieces X + H accumulators in tensor memory.
// Every barrier has one waiting party that sees each of its phases in turn (a parity wait cannot tell
// phase k from phase k - 2): unpack warp s fills stage s, MMA warp s % 4 issues for it, the fold warps take
// units in order.
template <int MT, int H>
__global__ void __launch_bounds__(DT_THREADS, 1) awq_decode_tc_kernel(const DecodeParams p)
{
    extern __shared__ unsigned char smem_raw[];
    if (threadIdx.x == 0) DT_CTA(0);
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u; // swizzled tiles need 1024-byte alignment
    unsigned char *base_ptr = smem_raw + (base - raw);
    const int S = p.stages;
    constexpr int TILE_N = DT_ROWS * H;
    constexpr uint32_t X_OFF = (uint32_t)H * DT_A_BYTES;
    // after the stages: per-(k group, token) factors, the fold threads' scale/zero ring, barriers
    unsigned char *tail = base_ptr + (size_t)S * p.stage_bytes;
    float2 *xs_s = reinterpret_cast<float2 *>(tail);
    uint2 *sz_ring = reinterpret_cast<uint2 *>(tail + p.xs_smem_bytes); // [DT_SZ_DEPTH][H][128]
    constexpr uint32_t RING_SLOT = H * DT_FOLD_WARPS * 32 * 8, RING_BYTES = DT_SZ_DEPTH * RING_SLOT;
    const uint32_t bars = base + (uint32_t)S * p.stage_bytes + p.xs_smem_bytes + RING_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };            // operands of the stage are in shared memory
    auto empty_bar = [&](int s) { return bars + 8u * (S + s); };     // the MMAs have read them AND the fold has read the accumulators
    auto dfull_bar = [&](int s) { return bars + 8u * (2 * S + s); }; // the accumulators of stage s are complete
    const uint32_t fsync_bar = bars + 8u * (3 * S);                  // meeting point of the four fold warps
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tail + p.xs_smem_bytes + RING_BYTES + 8 * (3 * S + 1));
    int *fin_slot = reinterpret_cast<int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x, ctas = gridDim.x;
    const int u0 = (int)((long long)cta * p.units / ctas), u1 = (int)((long long)(cta + 1) * p.units / ctas);
    const int nu = u1 - u0;
    const int G = p.kgroups;

    // ---- unpack warps: geometry, and the first packed words on their way before anything else ---------------
    // H = 1: a tile row is 16 words (64 bytes): 4 lanes per input row, 8 rows per load instruction, 16 tasks per unit.
    // H = 2: a tile row is 32 words (one 128-byte line): 8 lanes per row, 4 rows per instruction, 32 tasks per unit.
    constexpr int LPR = 4 * H;          // lanes per row
    constexpr int RPI = 32 / LPR;       // rows per instruction
    constexpr int TASKS = DT_UNIT_K / RPI;
    const int uw = warp - DT_MMA_WARPS - DT_FOLD_WARPS; // 0 .. 7 for unpack warps
    const bool unpacker = uw >= 0 && uw < S && u0 + uw < u1;
    const int piece16 = lane % LPR, kr0 = lane / LPR;   // 16-byte piece of the row, first input row
    const int words_per_row = 16 * H;
    const size_t rstep = (size_t)RPI * p.packed_out;                 // words between two tasks of a lane
    const size_t unit_words = (size_t)DT_UNIT_K * p.packed_out;      // words between two k groups
    uint4 buf[16];
    int ut = 0, ug = 0; // (tile, k group) of the unpack warp's current unit
    const uint32_t *lane_base = p.qweight;
    auto tile_word = [&](int t) { // first word of this lane's piece; tiles past the end re-read the last words (results never stored)
        const int w = t * words_per_row + piece16 * 4;
        return w + 4 <= p.packed_out ? w : p.packed_out - 4;
    };
    if (unpacker) {
        lane_base = p.qweight + (size_t)kr0 * p.packed_out;
        ut = (u0 + uw) / G;
        ug = (u0 + uw) - ut * G;
        const uint32_t *src = lane_base + (size_t)ug * unit_words + tile_word(ut);
#pragma unroll
        for (int j = 0; j < 16; j++) buf[j] = __ldcs(reinterpret_cast<const uint4 *>(src + j * rstep));
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; s++) {
            mbar_init(full_bar(s), 2);                   // the unpacking warp + its token-piece copy
            mbar_init(empty_bar(s), 1 + DT_FOLD_WARPS);  // tcgen05.commit + one arrival per fold warp
            mbar_init(dfull_bar(s), 1);
        }
        mbar_init(fsync_bar, DT_FOLD_WARPS);
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
    if (threadIdx.x == 0) DT_CTA(1);

    if (warp < DT_MMA_WARPS) {
        // ---- MMA issue: warp i serves stages i, i + 4 ----------------------------------------------------
        if (elect_one()) {
            const uint32_t idesc = decode_idesc(p.np);
            bool ok = true;
            int s = 0;
            uint32_t ph = 0;
            for (int it = 0; it < nu && ok; it++) {
                if ((s & (DT_MMA_WARPS - 1)) == warp) {
                    ok = mbar_wait(full_bar(s), ph, p.flag, 2);
                    if (!ok) break;
                    if (warp == 0) DT_TRACE(1, it);
                    tc_fence_after();
                    const uint32_t sa = base + (uint32_t)s * p.stage_bytes;
                    const uint64_t db = kmajor_sw128_desc(sa + X_OFF);
#pragma unroll
                    for (int h = 0; h < H; h++) {
                        const uint64_t da = mnmajor_sw128_desc(sa + (uint32_t)h * DT_A_BYTES);
                        const uint32_t d_tmem = tmem_base + (uint32_t)(s * H + h) * p.np;
#pragma unroll
                        for (int kk = 0; kk < DT_UNIT_K / 32; kk++) // 32 input rows = 4 KB of A, 32 bytes inside the swizzled row of B
                            umma_f8(d_tmem, da + (uint64_t)kk * (4096 >> 4), db + 2 * kk, idesc, kk != 0);
                    }
                    umma_commit(empty_bar(s));
                    umma_commit(dfull_bar(s));
                    if (warp == 0) DT_TRACE(2, it);
                }
                if (++s == S) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp < DT_MMA_WARPS + DT_FOLD_WARPS) {
        // ---- fold: one accumulator row (out feature) of each of the H tiles per thread -------------------------
        const int quad = warp & 3; // tensor-memory lanes this warp may read
        const int r = quad * 32 + lane;
        const int fold_tid = (warp - DT_MMA_WARPS) * 32 + lane;
        const int ncol = row_to_col(r);
        const int zshift = 4 * ((ncol & 1) ? 4 + ((ncol & 7) >> 1) : ((ncol & 7) >> 1));
        const bool sc32 = p.scales_dtype == OXQ_F32, sc16f = p.scales_dtype == OXQ_F16;
        const uint32_t hshift = 16u * (uint32_t)(ncol & 1); // which half of the copied word holds a 16-bit scale
        uint32_t fphase = 0;
        // All fold warps meet (bounded like every other wait): one arrival per warp, then everyone waits for the phase.
        auto fold_sync = [&]() {
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(fsync_bar) : "memory");
            const bool got = mbar_wait_warp(fsync_bar, fphase & 1, p.flag, 5);
            fphase++;
            return got;
        };
        // Scale and zero point of this thread's rows for a unit's quantization group travel to private
        // shared-memory slots with 4-byte cp.async copies issued DT_SZ_DEPTH - 1 units ahead (no registers held).
        // The copy stream has its own (tile, k group) counters; rows past the end read the last column.
        const uint32_t my_ring = smem_u32(sz_ring) + (uint32_t)fold_tid * 8u;
        const size_t sc_row_bytes = (size_t)p.n * (sc32 ? 4 : 2), z_row_bytes = (size_t)p.packed_out * 4;
        int tl = u0 / G, gl = u0 - tl * G, ul = u0;
        const unsigned char *scb[H], *zb[H];
        auto set_tile_l = [&]() {
#pragma unroll
            for (int h = 0; h < H; h++) {
                int nn = tl * TILE_N + h * DT_ROWS + ncol;
                nn = nn < p.n ? nn : p.n - 1;
                scb[h] = reinterpret_cast<const unsigned char *>(p.scales) + (sc32 ? (size_t)nn * 4 : (size_t)(nn >> 1) * 4);
                zb[h] = reinterpret_cast<const unsigned char *>(p.qzeros + (nn >> 3));
            }
        };
        set_tile_l();
        auto issue_sz = [&]() {
            if (ul < u1) {
                const int qg = gl >> p.gshift;
                const uint32_t dst = my_ring + (uint32_t)((ul - u0) & (DT_SZ_DEPTH - 1)) * RING_SLOT;
#pragma unroll
                for (int h = 0; h < H; h++) {
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + h * (DT_FOLD_WARPS * 32 * 8)), "l"(scb[h] + (size_t)qg * sc_row_bytes) : "memory");
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + h * (DT_FOLD_WARPS * 32 * 8) + 4), "l"(zb[h] + (size_t)qg * z_row_bytes) : "memory");
                }
                ul++;
                if (++gl == G) { gl = 0; tl++; set_tile_l(); }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
#pragma unroll 1
        for (int d = 0; d < DT_SZ_DEPTH - 1; d++) issue_sz();

        grid_dependency_wait();
        // {512 / 2^p, sum x} of every (k group, token) into shared memory once (when it fits)
        const bool xs_in_smem = p.xs_smem_bytes != 0;
        if (xs_in_smem) {
            const float2 *src = p.xs;
            for (int i = fold_tid; i < G * MT; i += DT_FOLD_WARPS * 32) xs_s[i] = __ldcg(src + i);
        }
        bool ok = fold_sync();
        if (fold_tid == 0) DT_CTA(2);

        float tot[H][MT];
#pragma unroll
        for (int h = 0; h < H; h++)
#pragma unroll
            for (int i = 0; i < MT; i++) tot[h][i] = 0.0f;
        int t = u0 / G, g = u0 - t * G;
        int s = 0;
        uint32_t ph = 0;
        for (int u = u0; u < u1 && ok; u++) {
            const int it = u - u0;
            issue_sz();
            asm volatile("cp.async.wait_group %0;" ::"n"(DT_SZ_DEPTH - 1) : "memory");
            float s_cur[H], sz_cur[H];
#pragma unroll
            for (int h = 0; h < H; h++) {
                const uint2 szw = sz_ring[((it & (DT_SZ_DEPTH - 1)) * H + h) * (DT_FOLD_WARPS * 32) + fold_tid];
                const uint32_t h16 = (szw.x >> hshift) & 0xFFFFu;
                s_cur[h] = sc32 ? __uint_as_float(szw.x)
                                : (sc16f ? __half2float(__ushort_as_half((unsigned short)h16)) : __uint_as_float(h16 << 16));
                sz_cur[h] = s_cur[h] * (float)((szw.y >> zshift) & 0xFu);
            }
            const float2 *xsg = xs_in_smem ? xs_s + g * MT : p.xs + (size_t)g * MT;

            ok = mbar_wait_warp(dfull_bar(s), ph, p.flag, 3);
            if (!ok) break;
            if (fold_tid == 0) DT_TRACE(3, it);
            if (fold_tid == 0 && it == 0) DT_CTA(5);
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(s * H) * p.np;
            if constexpr (MT <= 4) {
                constexpr int NC = MT == 1 ? 4 : (MT == 2 ? 8 : 16);
                uint32_t d[H][NC];
#pragma unroll
                for (int h = 0; h < H; h++) {
                    if constexpr (NC == 4) tmem_ld4(taddr + h * p.np, d[h]);
                    else if constexpr (NC == 8) tmem_ld8(taddr + h * p.np, d[h]);
                    else tmem_ld16(taddr + h * p.np, d[h]);
                }
                float2 xv[MT];
#pragma unroll
                for (int i = 0; i < MT; i++) xv[i] = xs_in_smem ? xsg[i] : __ldcg(xsg + i);
                tmem_ld_wait();
#pragma unroll
                for (int h = 0; h < H; h++)
#pragma unroll
                    for (int i = 0; i < MT; i++) {
                        const float dsum = (__uint_as_float(d[h][3 * i]) + __uint_as_float(d[h][3 * i + 1])) + __uint_as_float(d[h][3 * i + 2]);
                        if (i < p.m) tot[h][i] = fmaf(s_cur[h] * xv[i].x, dsum, fmaf(-sz_cur[h], xv[i].y, tot[h][i]));
                    }
            } else {
#pragma unroll
                for (int c = 0; c < MT / 8; c++) {
                    if (8 * c < p.m) {
                        float2 xv[8];
#pragma unroll
                        for (int i = 0; i < 8; i++) xv[i] = xs_in_smem ? xsg[8 * c + i] : __ldcg(xsg + 8 * c + i);
#pragma unroll
                        for (int h = 0; h < H; h++) {
                            uint32_t d[24]; // 8 tokens x 3 pieces, neighbouring columns
                            tmem_ld8(taddr + h * p.np + 24 * c, d);
                            tmem_ld8(taddr + h * p.np + 24 * c + 8, d + 8);
                            tmem_ld8(taddr + h * p.np + 24 * c + 16, d + 16);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                const float dsum = (__uint_as_float(d[3 * i]) + __uint_as_float(d[3 * i + 1])) + __uint_as_float(d[3 * i + 2]);
                                if (8 * c + i < p.m)
                                    tot[h][8 * c + i] = fmaf(s_cur[h] * xv[i].x, dsum, fmaf(-sz_cur[h], xv[i].y, tot[h][8 * c + i]));
                            }
                        }
                    }
                }
            }
            // this warp's quarter of the accumulators has been read: its share of the stage's release
            tc_fence_before();
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_bar(s)) : "memory");
            __syncwarp();
            if (fold_tid == 0) DT_TRACE(4, it);

            if (g == G - 1 || u == u1 - 1) {
                // The tile ends here, or this CTA's share of it does.
                const bool whole = (t * G >= u0) && (g == G - 1);
                bool last = whole;
                const long long U = p.units;
                if (!whole) {
                    // Partial sums meet in the workspace; the CTA that arrives last adds them in CTA order.
                    const int c_first = (int)((((long long)t * G + 1) * ctas - 1) / U);
                    const int c_last = (int)(((long long)(t + 1) * G * ctas - 1) / U);
                    float *mine = p.partials + ((size_t)2 * cta + (t == u0 / G ? 0 : 1)) * (H * MT * DT_ROWS);
#pragma unroll
                    for (int h = 0; h < H; h++)
#pragma unroll
                        for (int i = 0; i < MT; i++)
                            if (i < p.m) __stcg(mine + (h * MT + i) * DT_ROWS + r, tot[h][i]);
                    __threadfence();
                    ok = fold_sync();
                    if (!ok) break;
                    if (fold_tid == 0) *fin_slot = (atomicAdd(p.counters + t, 1) == c_last - c_first) ? 1 : 0;
                    ok = fold_sync();
                    if (!ok) break;
                    last = *fin_slot != 0; // rewritten only after everyone has passed the next meeting
                    if (last) {
                        __threadfence();
#pragma unroll
                        for (int h = 0; h < H; h++)
#pragma unroll
                            for (int i = 0; i < MT; i++) tot[h][i] = 0.0f;
                        for (int cc = c_first; cc <= c_last; cc++) {
                            const int cu0 = (int)((long long)cc * U / ctas);
                            const float *src = p.partials + ((size_t)2 * cc + (t == cu0 / G ? 0 : 1)) * (H * MT * DT_ROWS);
#pragma unroll
                            for (int h = 0; h < H; h++)
#pragma unroll
                                for (int i = 0; i < MT; i++)
                                    if (i < p.m) tot[h][i] += __ldcg(src + (h * MT + i) * DT_ROWS + r);
                        }
                    }
                }
                if (last) {
#pragma unroll
                    for (int h = 0; h < H; h++) {
                        const int n = t * TILE_N + h * DT_ROWS + ncol;
                        if (n < p.n) {
                            const float b = p.bias ? load_as_f32(p.bias, p.bias_dtype, n) : 0.0f;
#pragma unroll
                            for (int i = 0; i < MT; i++)
                                if (i < p.m) store_as(p.y, p.y_dtype, (size_t)i * p.n + n, tot[h][i] + b);
                        }
                    }
                }
#pragma unroll
                for (int h = 0; h < H; h++)
#pragma unroll
                    for (int i = 0; i < MT; i++) tot[h][i] = 0.0f;
            }
            if (++g == G) { g = 0; t++; }
            if (++s == S) { s = 0; ph ^= 1u; }
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        tc_fence_before();
        if (fold_tid == 0) DT_CTA(3);
    } else if (unpacker) {
        // ---- unpack: packed words -> one E4M3 byte per weight in the operand layout ---------------------------
        // Warp w owns stage w: it copies the unit's token pieces there, and holds 16 tasks (16 x 16 bytes per lane)
        // of packed words in registers: the rest of this unit (H = 2) or the next unit while it writes out the
        // current ones.
        uint32_t mask;
        asm volatile("mov.b32 %0, 0x0F0F0F0F;" : "=r"(mask));
        unsigned char *a = base_ptr + (size_t)uw * p.stage_bytes;
        // Lane constants of the swizzled destination. A task's row is kr0 + RPI * j; its 16-byte piece holds two
        // pairs of packed words (chunks c, c + 1 of the 128-byte operand row, XOR-swizzled with row & 7).
        // H = 1: row & 7 == kr0 for every task. H = 2: row & 7 == kr0 + 4 * (j & 1); the lanes of the second tile
        // store their two chunks in the opposite order so that a quarter warp never meets in a bank.
        const int half = piece16 >> 2, cq = piece16 & 3;
        unsigned char *abase = a + (uint32_t)half * DT_A_BYTES + (uint32_t)kr0 * 128u;
        uint32_t offA[H], offB[H]; // per parity of j (H = 2) the byte offsets of the two chunks inside the row
#pragma unroll
        for (int par = 0; par < H; par++) {
            const int r7 = kr0 + 4 * par;
            const uint32_t c0 = (uint32_t)(((2 * cq) ^ r7) << 4), c1 = (uint32_t)(((2 * cq + 1) ^ r7) << 4);
            offA[par] = half ? c1 : c0;
            offB[par] = half ? c0 : c1;
        }
        const uint32_t xdst = smem_u32(a) + X_OFF, fbar = full_bar(uw), ebar = empty_bar(uw);
        bool ok = true;
        uint32_t ph = 1; // parity of "the stage is free": passes at once on the first lap
        if (lane == 0) grid_dependency_wait(); // before the first copy of token pieces
        __syncwarp();
        for (int u = u0 + uw; u < u1 && ok; u += S) {
            const int it = u - u0;
            (void)it; // only the trace of tuning builds reads it
            ok = mbar_wait_warp(ebar, ph, p.flag, 1);
            ph ^= 1u;
            if (lane == 0 && uw == 0) DT_TRACE(5, it);
            if (!ok) break;
            if (lane == 0) {
                mbar_arrive_expect_tx(fbar, p.x_bytes);
                bulk_copy_g2s(xdst, p.xq + (size_t)ug * p.x_bytes, p.x_bytes, fbar);
            }
            __syncwarp(); // lane 0 rejoins before the vector work
            const uint32_t *cur = lane_base + (size_t)ug * unit_words + tile_word(ut);
            const bool more = u + S < u1;
            ug += S;
            while (ug >= G) { ug -= G; ut++; }
            const uint32_t *nxt = lane_base + (size_t)ug * unit_words + tile_word(ut);
#pragma unroll
            for (int pass = 0; pass < TASKS / 16; pass++) {
                unsigned char *dst = abase + (uint32_t)pass * 16u * RPI * 128u;
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const uint4 w = buf[j];
                    const int par = (H == 2) ? (j & 1) : 0;
                    unsigned char *rowp = dst + (uint32_t)j * RPI * 128u;
                    const uint4 lo = make_uint4(w.x & mask, (w.x >> 4) & mask, w.y & mask, (w.y >> 4) & mask);
                    const uint4 hi = make_uint4(w.z & mask, (w.z >> 4) & mask, w.w & mask, (w.w >> 4) & mask);
                    *reinterpret_cast<uint4 *>(rowp + offA[par]) = half ? hi : lo;
                    *reinterpret_cast<uint4 *>(rowp + offB[par]) = half ? lo : hi;
                }
                // refill: the second half of this unit (H = 2, first pass) or the first 16 tasks of the warp's next unit
                const bool second_half_next = (H == 2) && pass == 0;
                if (second_half_next || more) {
                    const uint32_t *src = second_half_next ? cur + 16 * rstep : nxt;
#pragma unroll
                    for (int j = 0; j < 16; j++) buf[j] = __ldcs(reinterpret_cast<const uint4 *>(src + j * rstep));
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic-proxy stores -> visible to the MMA
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(fbar) : "memory");
            __syncwarp();
            if (lane == 0 && uw == 0) DT_TRACE(6, it);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) DT_CTA(4);
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    }
}

struct DecodeLayout {
    int q, np, h, tiles, kgroups, ctas, tmem_cols, stages;
    size_t off_counters, off_xs, off_xq, off_partials, total;
};

static DecodeLayout decode_layout(int m, int k, int n)
{
    DecodeLayout L;
    L.q = 1;
    while (L.q < m) L.q *= 2; // token slots: 1, 2, 4, 8, 16, 32
    L.np = (3 * L.q + 15) / 16 * 16;
    L.h = L.q <= 16 ? 2 : 1;  // 256 out features per unit while two accumulators per stage leave room for enough stages
    L.tiles = (n + DT_ROWS * L.h - 1) / (DT_ROWS * L.h);
    L.kgroups = k / DT_UNIT_K;
    const long long units = (long long)L.tiles * L.kgroups;
    const int sms = sm_count();
    L.ctas = units < sms ? (int)units : sms;
    const int by_tmem = 512 / (L.h * L.np);
    L.stages = by_tmem < DT_UNPACK_WARPS ? by_tmem : DT_UNPACK_WARPS; // accumulators per stage, one unpack warp per stage
    L.tmem_cols = 32;
    while (L.tmem_cols < L.stages * L.h * L.np) L.tmem_cols *= 2;
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    L.off_counters = DT_WS_HEADER;
    L.off_xs = up(L.off_counters + (size_t)L.tiles * sizeof(int));
    L.off_xq = up(L.off_xs + (size_t)L.kgroups * L.q * sizeof(float2));
    L.off_partials = up(L.off_xq + (size_t)L.kgroups * L.np * 128);
    L.total = up(L.off_partials + (size_t)2 * sms * L.h * L.q * DT_ROWS * sizeof(float));
    return L;
}

} // namespace oxq

using namespace oxq;

#ifdef OXQ_TUNING
OXQ_EXPORT int oxq_dt_cta_read(unsigned long long *host_out)
{
    return cudaMemcpyFromSymbol(host_out, g_dt_cta, sizeof(unsigned long long) * 160 * 8) == cudaSuccess ? 0 : -6;
}
OXQ_EXPORT int oxq_dt_trace_read(long long *host_out)
{
    return cudaMemcpyFromSymbol(host_out, g_dt_trace, sizeof(long long) * 16 * 64) == cudaSuccess ? 0 : -6;
}
#endif

OXQ_EXPORT int oxq_decode_max_m(void) { return DT_MAX_M; }

OXQ_EXPORT size_t oxq_decode_workspace_bytes(int m, int k, int n)
{
    if (m < 1 || m > DT_MAX_M || k <= 0 || n <= 0) return 0;
    return decode_layout(m, k, n).total;
}

OXQ_EXPORT int oxq_awq_decode_matmul(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros,
                                     const void *scales, int scales_dtype, const void *bias, int bias_dtype, void *y,
                                     int y_dtype, int m, int k, int n, int group_size, void *workspace,
                                     size_t workspace_bytes, void *stream)
{
    clear_error();
    OXQ_REQUIRE(x && qweight && qzeros && scales && y, OXQ_ERR_NULL, "oxq_awq_decode_matmul: null pointer");
    OXQ_REQUIRE(x_dtype == OXQ_BF16, OXQ_ERR_UNSUPPORTED, "oxq_awq_decode_matmul: activations must be bf16");
    OXQ_REQUIRE(valid_dtype(scales_dtype) && valid_dtype(y_dtype) && (!bias || valid_dtype(bias_dtype)), OXQ_ERR_UNSUPPORTED,
                "oxq_awq_decode_matmul: unsupported dtype");
    OXQ_REQUIRE(m >= 1 && m <= DT_MAX_M, OXQ_ERR_BAD_SHAPE, "oxq_awq_decode_matmul: m=%d outside 1..%d (use the GEMM entry)", m, DT_MAX_M);
    OXQ_REQUIRE(k > 0 && n > 0 && group_size > 0, OXQ_ERR_BAD_SHAPE, "oxq_awq_decode_matmul: non-positive size");
    OXQ_REQUIRE(n % 8 == 0, OXQ_ERR_BAD_SHAPE, "AWQ out_features (%d) not divisible by pack factor 8", n);
    OXQ_REQUIRE(k % group_size == 0, OXQ_ERR_BAD_SHAPE, "quant in_features (%d) not divisible by group size (%d)", k, group_size);
    OXQ_REQUIRE((group_size & (group_size - 1)) == 0, OXQ_ERR_BAD_SHAPE, "group_size %d is not a power of two", group_size);
    OXQ_REQUIRE(n % 32 == 0 && k % DT_UNIT_K == 0 && group_size % DT_UNIT_K == 0, OXQ_ERR_UNSUPPORTED,
                "oxq_awq_decode_matmul: needs out_features %% 32 == 0, in_features and group size multiples of %d (got n=%d k=%d g=%d)",
                DT_UNIT_K, n, k, group_size);
    OXQ_REQUIRE(aligned(x, 8) && aligned(qweight, 16) && aligned(qzeros, 4) && aligned(scales, 4), OXQ_ERR_BAD_ALIGN,
                "oxq_awq_decode_matmul: x must be 8-byte and qweight 16-byte aligned");
    const DecodeLayout L = decode_layout(m, k, n);
    OXQ_REQUIRE(workspace != nullptr && workspace_bytes >= L.total, OXQ_ERR_WORKSPACE,
                "oxq_awq_decode_matmul: workspace of %zu bytes needed, got %zu", L.total, workspace_bytes);
    OXQ_REQUIRE(aligned(workspace, 256), OXQ_ERR_BAD_ALIGN, "oxq_awq_decode_matmul: workspace must be 256-byte aligned");
    unsigned char *ws = reinterpret_cast<unsigned char *>(workspace);
    cudaStream_t st = (cudaStream_t)stream;

    DecodeParams p;
    p.qweight = qweight; p.qzeros = qzeros; p.scales = scales; p.bias = bias; p.y = y;
    p.flag = reinterpret_cast<int *>(ws);
    p.counters = reinterpret_cast<int *>(ws + L.off_counters);
    p.xs = reinterpret_cast<const float2 *>(ws + L.off_xs);
    p.xq = ws + L.off_xq;
    p.partials = reinterpret_cast<float *>(ws + L.off_partials);
    p.scales_dtype = scales_dtype; p.bias_dtype = bias_dtype; p.y_dtype = y_dtype;
    p.m = m; p.k = k; p.n = n; p.group_size = group_size; p.packed_out = n / 8;
    p.gshift = 0;
    while ((DT_UNIT_K << p.gshift) < group_size) p.gshift++;
    p.q = L.q; p.np = L.np; p.tiles = L.tiles; p.kgroups = L.kgroups; p.units = L.tiles * L.kgroups;
    p.tmem_cols = L.tmem_cols;
    p.x_bytes = (uint32_t)L.np * 128u;
    p.stage_bytes = ((uint32_t)L.h * DT_A_BYTES + p.x_bytes + 1023u) & ~1023u;
    const size_t xs_bytes = (size_t)L.kgroups * L.q * sizeof(float2);
    p.xs_smem_bytes = xs_bytes <= 32 * 1024 ? (uint32_t)((xs_bytes + 15) / 16 * 16) : 0u; // else read from global memory
    const size_t fixed = 1024 + p.xs_smem_bytes + (size_t)DT_SZ_DEPTH * L.h * DT_FOLD_WARPS * 32 * 8 + 8 * (3 * DT_UNPACK_WARPS + 1) + 16;
    const int fit = (int)((DT_SMEM_BUDGET - fixed) / p.stage_bytes);
    p.stages = fit < L.stages ? fit : L.stages;
    OXQ_REQUIRE(p.stages >= 2, OXQ_ERR_UNSUPPORTED, "oxq_awq_decode_matmul: shape leaves fewer than two pipeline stages");
    bool use_pdl = true, run_prep = true;
    p.dbg = 0;
#ifdef OXQ_TUNING
    if (const char *e = tuning_env("OXQ_DT_DBG")) p.dbg = atoi(e);
    if (const char *e = tuning_env("OXQ_DT_PDL")) use_pdl = atoi(e) != 0;
    if (const char *e = tuning_env("OXQ_DT_PREP")) run_prep = atoi(e) != 0;
    if (const char *e = tuning_env("OXQ_DT_STAGES")) { const int v = atoi(e); if (v >= 2 && v <= p.stages) p.stages = v; }
#endif
    const size_t smem = fixed + (size_t)p.stages * p.stage_bytes;

    const int prep_threads = 32 * m * L.kgroups > L.tiles ? 32 * m * L.kgroups : L.tiles;
    if (run_prep)
        decode_prep_kernel<<<(prep_threads + 255) / 256, 256, 0, st>>>(
            reinterpret_cast<const __nv_bfloat16 *>(x), ws + L.off_xq, reinterpret_cast<float2 *>(ws + L.off_xs),
            p.counters, L.tiles, m, k, L.q, L.np);
    OXQ_LAUNCH_CHECK("decode_prep_kernel");

    void (*kern)(const DecodeParams) = nullptr;
    int qi = 0;
    switch (L.q) {
    case 1: kern = awq_decode_tc_kernel<1, 2>; qi = 0; break;
    case 2: kern = awq_decode_tc_kernel<2, 2>; qi = 1; break;
    case 4: kern = awq_decode_tc_kernel<4, 2>; qi = 2; break;
    case 8: kern = awq_decode_tc_kernel<8, 2>; qi = 3; break;
    case 16: kern = awq_decode_tc_kernel<16, 2>; qi = 4; break;
    default: kern = awq_decode_tc_kernel<32, 1>; qi = 5; break;
    }
    static size_t configured[64][6] = {};
    int device = 0;
    OXQ_CUDA(cudaGetDevice(&device));
    if (device >= 64 || configured[device][qi] < smem) {
        OXQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (device < 64) configured[device][qi] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(L.ctas, 1, 1);
    cfg.blockDim = dim3(DT_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; // may start while the piece kernel still runs
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl ? 1 : 0;
    OXQ_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
    return OXQ_OK;
}
