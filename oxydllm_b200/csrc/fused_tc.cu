// AWQ W4A16 matmul for batches of up to 256 tokens with the dequantization fused into the tensor-core
// kernel: the packed words are read from HBM once and no dense copy of the weight is ever written.
//
// One CTA owns 128 out features and walks k in stages of 64 input rows:
//   warp 0 (one lane)   TMA: boxes of packed words (64 rows x 16 words, 4 KB) into a ring of up to 32 slots,
//                       as far ahead as the ring allows: this ring is what is in flight from HBM;
//   warp 2 (one lane)   TMA: the stage's tile of x ([tokens, 64] bf16, 128-byte swizzle) into one of the
//                       two or four operand slots;
//   warps 4..19         unpack, two teams of eight warps taking rounds of two stages in turn: every thread
//                       turns four packed words per stage into 4 x 8 bf16 weights, the same bits the dequantization kernel
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
constexpr int FT_UNPACK_WARPS = 16;
constexpr int FT_TEAMS = 2;                      // teams of unpack warps take rounds in turn (measured: 29 us with two teams, 33 us with one)
constexpr int FT_TEAM_WARPS = FT_UNPACK_WARPS / FT_TEAMS;
constexpr int FT_WORDS = FT_BK * 16 / (FT_TEAM_WARPS * 32); // packed words per thread and stage
constexpr int FT_ROUND = 2;                      // stages per round: polls, proxy fence and arrivals are paid once per round
constexpr int FT_ROUND_SLOTS = 4;                // most rounds of operand slots (S = FT_ROUND * 2 or FT_ROUND * 4: multiples of the teams' rounds)
constexpr int FT_THREADS = (4 + FT_UNPACK_WARPS) * 32;
constexpr int FT_BOX_BYTES = FT_BK * 16 * 4;      // 64 input rows x 16 packed words
constexpr int FT_ZERO_BYTES = 64, FT_SCALE_BYTES = 256; // the box's group: 16 zero-point words, 128 16-bit scales
constexpr int FT_A_BYTES = FT_ROWS * FT_BK * 2;
constexpr int FT_MAX_STAGES = FT_ROUND * FT_ROUND_SLOTS; // operand slots (A tile + x tile)
constexpr int FT_MAX_RAW = 32;                   // ring slots of packed boxes: what is in flight from HBM
constexpr int FT_NUM_BARS = 2 * FT_MAX_RAW + 3 * FT_MAX_STAGES + 1;
static_assert(FT_ROUND_SLOTS % FT_TEAMS == 0 && FT_MAX_RAW % (FT_ROUND * FT_TEAMS) == 0, "a slot must always meet the same team");
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
    int gshift;        // log2(stages per quantization group)
    int sym;           // GPTQ: no stored zero points (zero + 1 = 8)
    const float *scale_inv; // FP8: scale grid [s_out, s_in] or null
    int s_in, block_out, block_in;
    int col_base, ldy; // y column of out feature 0 and the row pitch of y in elements
    int *flag;
    int sk;              // k splits per tile (grid y); > 1: partial tiles meet in `partials`, the last CTA of a tile adds them
    float *partials;     // [tile][split][mpad][128] f32
    unsigned int *tickets; // 16-bit arrival counters, two per word, zero between calls
};

// A operand: 16-bit, MN-major, 128-byte swizzle. An atom is 8 input rows x 64 out features (1 KB); atoms of
// later input rows follow at 1 KB (stride byte offset), the second 64 out features at 8 KB (leading byte offset).
__device__ __forceinline__ uint64_t ft_a_desc(uint32_t smem_addr)
{
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)(8192 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint32_t ft_and_or(uint32_t v, uint32_t mask, uint32_t magic) // (v & mask) | magic
{
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(v), "r"(mask), "r"(magic));
    return r;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4 &v)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// D f32, A bf16 MN-major, B bf16 K-major.
__device__ __forceinline__ uint32_t ft_idesc(int n)
{
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(FT_ROWS >> 4) << 24);
}

// GPTQ = false: AWQ layout (a word is eight out features of one input row; A operand MN-major).
// GPTQ = true:  GPTQ 4-bit layout (a word is eight input rows of one out feature, nibble i = row 8 r + i; A operand
//               K-major: the word becomes one 16-byte chunk of the out feature's 128-byte row). The box is 8 packed
//               rows x 128 words; the zero point is the stored nibble + 1, or 8 for symmetric weights (awq.rs:540-590).
// LAYOUT 2: FP8 E4M3 [n, k] row-major with an f32 scale grid (Fp8Linear, linear.rs:96-145). The box is 128 rows x
//               64 bytes, already K-major; every thread widens 32 bytes of one row (e4m3 -> f16 exactly in hardware,
//               -> f32, times the block's scale, one rounding to bf16: the bits of the dequantization kernel). The
//               tile's row of the scale grid is copied to shared memory once.
template <int LAYOUT>
__global__ void __launch_bounds__(FT_THREADS, 1)
    awq_fused_tc_kernel(const FusedParams p, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap)
{
    constexpr bool GPTQ = LAYOUT == 1, FP8 = LAYOUT == 2;
    constexpr int BOX_BYTES = FP8 ? FT_ROWS * FT_BK : FT_BOX_BYTES; // one stage of packed weights
    constexpr int RAW_BYTES = BOX_BYTES + (FP8 ? 0 : 384);          // ring slot: box | zero points | scales | pad
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u; // operand slots want 1 KB alignment
    unsigned char *base_ptr = smem_raw + (base - smem_u32(smem_raw));
    // operand slots (A tile + x tile) | ring of packed boxes | barriers | tensor-memory address
    const int S = p.stages, R = p.raw_slots;
    const uint32_t raw_base = (uint32_t)S * p.stage_bytes;
    const uint32_t bars = base + raw_base + (uint32_t)R * RAW_BYTES;
    auto rawfull_bar = [&](int r) { return bars + 8u * r; };
    auto rawempty_bar = [&](int r) { return bars + 8u * (FT_MAX_RAW + r); };
    auto xfull_bar = [&](int s) { return bars + 8u * (2 * FT_MAX_RAW + s); };
    auto ready_bar = [&](int s) { return bars + 8u * (2 * FT_MAX_RAW + FT_MAX_STAGES + s); };
    auto empty_bar = [&](int s) { return bars + 8u * (2 * FT_MAX_RAW + 2 * FT_MAX_STAGES + s); };
    const uint32_t acc_bar = bars + 8u * (2 * FT_MAX_RAW + 3 * FT_MAX_STAGES);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(base_ptr + raw_base + (size_t)R * RAW_BYTES + 8 * FT_NUM_BARS);
    float *fp8_scales = reinterpret_cast<float *>(tmem_slot + 4); // FP8: the tile's row of the scale grid, one float per k block
    const uint32_t b_off = FT_A_BYTES;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * FT_ROWS;
    const int nk = p.k / FT_BK / p.sk;        // stages of this CTA: split sk of the tile takes stages [sbase, sbase + nk)
    const int sbase = (int)blockIdx.y * nk;

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
    if (FP8 && warp == 3) {
        const int cnt = p.k / p.block_in;
        for (int i = lane; i < cnt; i += 32)
            fp8_scales[i] = p.scale_inv ? __ldg(p.scale_inv + (size_t)(n0 / p.block_out) * p.s_in + i) : 1.0f;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA, packed words: runs as far ahead of the unpack warps as the ring of boxes allows ------------
        if (elect_one()) {
            int r = 0;
            uint32_t ph = 0;
            for (int it = 0; it < nk; it++) {
                if (it >= R && !mbar_wait(rawempty_bar(r), ph ^ 1u, p.flag, 1)) break;
                const uint32_t dst = base + raw_base + (uint32_t)r * RAW_BYTES;
                const int qg = (sbase + it) * FT_BK / p.group_size;
                if (FP8) { // the box alone
                    mbar_arrive_expect_tx(rawfull_bar(r), BOX_BYTES);
                    tma_load_2d(dst, &wmap, rawfull_bar(r), (sbase + it) * FT_BK, n0);
                    FT_TRACE(0, it);
                    if (++r == R) { r = 0; ph ^= 1u; }
                    continue;
                }
                const bool with_zeros = !(GPTQ && p.sym);
                mbar_arrive_expect_tx(rawfull_bar(r), BOX_BYTES + (with_zeros ? FT_ZERO_BYTES : 0) + FT_SCALE_BYTES);
                if (GPTQ) tma_load_2d(dst, &wmap, rawfull_bar(r), n0, (sbase + it) * (FT_BK / 8));
                else tma_load_2d(dst, &wmap, rawfull_bar(r), n0 / 8, (sbase + it) * FT_BK);
                // the group's zero points and scales travel with the box: a plain load issued by the unpack threads
                // would wait a full DRAM round trip per group
                if (with_zeros)
                    bulk_copy_g2s(dst + BOX_BYTES, p.qzeros + (size_t)qg * p.packed_out + n0 / 8, FT_ZERO_BYTES, rawfull_bar(r));
                bulk_copy_g2s(dst + BOX_BYTES + FT_ZERO_BYTES,
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
                tma_load_2d(base + (uint32_t)s * p.stage_bytes + b_off, &xmap, xfull_bar(s), (sbase + it) * FT_BK, 0);
                if (++s == S) { s = 0; ph ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue -------------------------------------------------------------------------------
        if (elect_one()) {
            const uint32_t idesc = (GPTQ || FP8) ? tc_idesc(FT_ROWS, p.mpad) : ft_idesc(p.mpad);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int it = 0; it < nk; it++) {
                ok = mbar_wait(ready_bar(s), ph, p.flag, 2) && mbar_wait(xfull_bar(s), ph, p.flag, 6);
                if (!ok) break;
                FT_TRACE(1, it);
                tc_fence_after();
                const uint32_t slot = base + (uint32_t)s * p.stage_bytes;
                const uint64_t da = (GPTQ || FP8) ? kmajor_sw128_desc(slot) : ft_a_desc(slot), db = kmajor_sw128_desc(slot + b_off);
#pragma unroll
                for (int kk = 0; kk < FT_BK / 16; kk++) // 16 input rows: two 1 KB atoms of an MN-major A, 32 bytes inside a swizzled K-major row
                    umma_bf16(tmem_base, da + (uint64_t)kk * ((GPTQ || FP8) ? 2 : (2048 >> 4)), db + 2 * kk, idesc, (it | kk) != 0);
                umma_commit(empty_bar(s));
                FT_TRACE(2, it);
                if (++s == S) { s = 0; ph ^= 1u; }
            }
            if (ok) umma_commit(acc_bar);
        }
    } else if (warp >= 4) {
        // ---- unpack ------------------------------------------------------------------------------------
        // A slot always meets the same team (the slot counts are multiples of the teams' rounds), so every waiter of a
        // barrier sees each of its phases.
        const int team = (warp - 4) / FT_TEAM_WARPS;
        const int ut = (threadIdx.x - 128) % (FT_TEAM_WARPS * 32);
        constexpr int ROW_STEP = (GPTQ ? FT_BK / 8 : FT_BK) / FT_WORDS; // this thread's (packed) rows of a stage: r0, r0 + ROW_STEP, ...
        const int j = GPTQ ? (ut & 127) : (ut & 15); // AWQ: word column (8 out features); GPTQ: out feature of the tile
        const int r0 = GPTQ ? (ut >> 7) : (ut >> 4); // first (packed) row of this thread; the others follow ROW_STEP apart
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
        uint32_t nib_mask, nib_magic, nib_lo, nib_hi16; // in registers, opaque to constant propagation: one LOP3 per use
        asm volatile("mov.b32 %0, 0x000F000F;\n\tmov.b32 %1, 0x43004300;\n\tmov.b32 %2, 0x0000000F;\n\tmov.b32 %3, 0x000F0000;"
                     : "=r"(nib_mask), "=r"(nib_magic), "=r"(nib_lo), "=r"(nib_hi16));
        // byte offset of this thread's first 16-byte chunk inside the A slot; rows ROW_STEP apart are ROW_STEP * 128 bytes apart
        // (GPTQ: out feature j is a 128-byte row of a 1 KB atom of eight rows; packed row c is its 16-byte chunk c ^ (j & 7))
        const uint32_t a_off = GPTQ ? (uint32_t)(j >> 3) * 1024u + (uint32_t)(j & 7) * 128u
                                    : (uint32_t)(j >> 3) * 8192u + (uint32_t)(r0 >> 3) * 1024u + (uint32_t)(r0 & 7) * 128u +
                                          (uint32_t)(((j & 7) ^ (r0 & 7)) << 4);
        const uint32_t raw_idx = raw_base + (uint32_t)(GPTQ ? r0 * 128 + j : r0 * 16 + j) * 4u;
        // FT_ROUND consecutive stages per round: the barrier polls, the proxy fence and the arrivals, which
        // cost more than the arithmetic of one stage, are paid once per round. Shared memory
        // is addressed with 32-bit shared-space addresses throughout (no generic-pointer arithmetic in the loop).
        const uint32_t a_addr = base + a_off;                           // first 16-byte chunk in slot 0
        const uint32_t box_addr0 = base + raw_idx;                      // this thread's first word in ring slot 0
        const uint32_t aux_addr0 = base + raw_base + BOX_BYTES;      // zero points of ring slot 0
        int r = FT_ROUND * team;                                       // first ring slot of the round
        uint32_t my_s = (uint32_t)(FT_ROUND * team) % (uint32_t)S;      // first operand slot of the round
        uint32_t ph = ((uint32_t)(FT_ROUND * team) / (uint32_t)S) & 1u, rph = 0; // phases of the operand-slot and ring barriers
        bool ok = true;
        for (int it0 = FT_ROUND * team; it0 < nk; it0 += FT_ROUND * FT_TEAMS) {
            if (ut == 0) FT_TRACE(7, it0);
            // all polls of the round first (they do not depend on each other), the bounded waits only where one failed
            bool t0 = mbar_test(rawfull_bar(r), rph), t1 = mbar_test(rawfull_bar(r + 1), rph);
            bool t2 = true, t3 = true;
            if (it0 >= S) { // the operand slots are free once the MMAs of the stages that used them last have completed
                t2 = mbar_test(empty_bar(my_s), ph ^ 1u);
                t3 = mbar_test(empty_bar(my_s + 1), ph ^ 1u);
            }
            if (!t0) ok = mbar_wait(rawfull_bar(r), rph, p.flag, 3);
            if (ok && !t1) ok = mbar_wait(rawfull_bar(r + 1), rph, p.flag, 3);
            if (ok && !t2) ok = mbar_wait(empty_bar(my_s), ph ^ 1u, p.flag, 7);
            if (ok && !t3) ok = mbar_wait(empty_bar(my_s + 1), ph ^ 1u, p.flag, 7);
            if (!ok) break;
            if (ut == 0) FT_TRACE(3, it0);
#pragma unroll
            for (int h = 0; h < FT_ROUND; h++) {
                const uint32_t ring = (uint32_t)(r + h) * RAW_BYTES;
                if constexpr (FP8) {
                    // thread = (row, half): 32 bytes of the row -> 32 bf16 = four 16-byte chunks of the K-major row
                    const int row = ut >> 1, half = ut & 1;
                    const float sc = fp8_scales[((sbase + it0 + h) * FT_BK) / p.block_in];
                    const uint32_t src = base + raw_base + ring + (uint32_t)row * 64u + (uint32_t)half * 32u;
                    const uint4 lo = lds128(src), hi = lds128(src + 16);
                    const uint32_t wv[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
                    const uint32_t dst = base + (my_s + h) * p.stage_bytes + (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u;
#pragma unroll
                    for (int c4 = 0; c4 < 4; c4++) {
                        uint4 o;
                        uint32_t *ov = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
                        for (int q = 0; q < 2; q++) {
                            uint32_t h01, h23;
                            asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
                                "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t}"
                                : "=r"(h01), "=r"(h23)
                                : "r"(wv[2 * c4 + q]));
                            const float2 f01 = __half22float2(*reinterpret_cast<const __half2 *>(&h01));
                            const float2 f23 = __half22float2(*reinterpret_cast<const __half2 *>(&h23));
                            const __nv_bfloat162 b01 = __floats2bfloat162_rn(__fmul_rn(sc, f01.x), __fmul_rn(sc, f01.y));
                            const __nv_bfloat162 b23 = __floats2bfloat162_rn(__fmul_rn(sc, f23.x), __fmul_rn(sc, f23.y));
                            ov[2 * q] = *reinterpret_cast<const uint32_t *>(&b01);
                            ov[2 * q + 1] = *reinterpret_cast<const uint32_t *>(&b23);
                        }
                        sts128(dst + ((((uint32_t)(half * 4 + c4)) ^ (uint32_t)(row & 7)) << 4), o);
                    }
                } else {
                uint32_t w[FT_WORDS];
#pragma unroll
                for (int i = 0; i < FT_WORDS; i++) w[i] = lds32(box_addr0 + ring + i * ROW_STEP * (GPTQ ? 512 : 64));
                const int qg = (sbase + it0 + h) >> p.gshift;
                if (qg != cur_qg) { // a new quantization group: its zero points and scales sit behind the box
                    cur_qg = qg;
                    if (GPTQ) { // one out feature per thread: one zero point and one scale, both halves of the pairs alike
                        uint32_t z1 = 8u; // symmetric weights: zero 7, + 1
                        if (!p.sym) z1 = ((lds32(aux_addr0 + ring + 4 * (j >> 3)) >> (4 * (j & 7))) & 0xFu) + 1u;
                        const uint32_t zv = 0x43004300u | z1 | (z1 << 16); // bf16 pair (128 + z + 1, 128 + z + 1)
                        const uint32_t sw = lds32(aux_addr0 + ring + FT_ZERO_BYTES + 4 * (j >> 1));
                        const uint32_t s16 = (j & 1) ? (sw >> 16) : (sw & 0xFFFFu);
                        uint4 both;
                        both.x = both.y = both.z = both.w = s16 | (s16 << 16);
                        split_scales(both, shi, slo);
#pragma unroll
                        for (int i = 0; i < 4; i++) zp[i] = *reinterpret_cast<const __nv_bfloat162 *>(&zv);
                    } else {
                        const uint32_t zw = lds32(aux_addr0 + ring + 4 * j);
                        split_scales(lds128(aux_addr0 + ring + FT_ZERO_BYTES + 16 * j), shi, slo);
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const uint32_t v = ((zw >> (4 * i)) & 0x000F000Fu) | 0x43004300u; // bf16 pair (128 + z, 128 + z')
                            zp[i] = *reinterpret_cast<const __nv_bfloat162 *>(&v);
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < FT_WORDS; i++) {
                    uint4 o;
                    uint32_t *ov = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        uint32_t v;
                        if (GPTQ) { // byte q of the word: rows 2q (low nibble) and 2q + 1 (high nibble), neighbours in the K-major row
                            const uint32_t t = w[i] >> (8 * q);
                            v = ft_and_or(t << 12, nib_hi16, ft_and_or(t, nib_lo, nib_magic));
                        } else { // nibbles q and q + 4 are out features 2q and 2q + 1 of the word
                            v = ft_and_or(w[i] >> (4 * q), nib_mask, nib_magic); // bf16 pair (128 + q, 128 + q')
                        }
                        const __nv_bfloat162 d = __hsub2(*reinterpret_cast<const __nv_bfloat162 *>(&v), zp[q]); // q - z, exact
                        const __nv_bfloat162 b2 = __hfma2(d, shi[q], __hmul2(d, slo[q])); // s_lo is zero for bf16 scales
                        ov[q] = *reinterpret_cast<const uint32_t *>(&b2);
                    }
                    if (GPTQ) {
                        const uint32_t c = (uint32_t)(r0 + i * ROW_STEP);
                        sts128(a_addr + (my_s + h) * p.stage_bytes + ((c ^ (uint32_t)(j & 7)) << 4), o);
                    } else
                    sts128(a_addr + (my_s + h) * p.stage_bytes + i * ROW_STEP * 128, o);
                }
                } // layouts with packed words
            }
            if (ut == 0) FT_TRACE(4, it0);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic-proxy stores -> visible to the MMA
            __syncwarp();
            if (lane == 0) {
#pragma unroll
                for (int h = 0; h < FT_ROUND; h++) {
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ready_bar(my_s + h)) : "memory");
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(rawempty_bar(r + h)) : "memory");
                }
            }
            if (ut == 0) FT_TRACE(5, it0);
            my_s += FT_ROUND * FT_TEAMS;
            if (my_s >= (uint32_t)S) { my_s -= (uint32_t)S; ph ^= 1u; }
            r += FT_ROUND * FT_TEAMS;
            if (r >= R) { r -= R; rph ^= 1u; }
        }

        // ---- epilogue: lane = out feature inside this warp's quarter of the accumulator rows -----------------
        if (ok) ok = mbar_wait(acc_bar, 0, p.flag, 4);
        if (ok) tc_fence_after();
        const int quad = warp & 3, turn = (warp - 4) >> 2; // the warps of a quarter take 32-token chunks in turn
        const int ncol = n0 + quad * 32 + lane;
        if (p.sk == 1) {
            if (ok) {
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
        } else {
            // Split k: this CTA's partial tile goes to the scratch area; the CTA that arrives last at the tile's ticket
            // adds the partial tiles in split order (ascending k) and stores y. No CTA waits for another; the two
            // barriers below are among this CTA's unpack warps, which all get here whether or not a wait gave up
            // (in that case the flag word is set and the output is not to be trusted).
            if (ok) {
                float *part = p.partials + (size_t)(blockIdx.x * p.sk + blockIdx.y) * p.mpad * FT_ROWS;
                for (int c0 = 32 * turn; c0 < p.mpad; c0 += 32 * (FT_UNPACK_WARPS / 4)) {
                    uint32_t rr[32];
                    tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, rr);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; c++)
                        if (c0 + c < p.m) part[(size_t)(c0 + c) * FT_ROWS + quad * 32 + lane] = __uint_as_float(rr[c]);
                }
            }
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"n"(FT_UNPACK_WARPS * 32) : "memory");
            const int et = threadIdx.x - 128; // 0 .. 511
            const unsigned shift = (blockIdx.x & 1u) * 16u;
            if (et == 0) tmem_slot[1] = (atomicAdd(p.tickets + (blockIdx.x >> 1), 1u << shift) >> shift) & 0xFFFFu;
            asm volatile("bar.sync 1, %0;" ::"n"(FT_UNPACK_WARPS * 32) : "memory");
            if (tmem_slot[1] == (uint32_t)(p.sk - 1)) {
                __threadfence();
                const float *tile_parts = p.partials + (size_t)blockIdx.x * p.sk * p.mpad * FT_ROWS;
                // a thread keeps its out feature (512 threads = four tokens x 128 features per pass) and takes eight
                // tokens per batch: all loads of a batch are issued before the first sum is stored
                const int nn = et % FT_ROWS;
                const float bv = p.bias ? load_as_f32(p.bias, p.bias_dtype, (size_t)p.col_base + n0 + nn) : 0.0f;
                constexpr int TOK_STEP = FT_UNPACK_WARPS * 32 / FT_ROWS, BATCH = 8;
                for (int tok0 = et / FT_ROWS; tok0 < p.m; tok0 += TOK_STEP * BATCH) {
                    float sum[BATCH];
#pragma unroll
                    for (int b = 0; b < BATCH; b++) sum[b] = 0.0f;
                    for (int sp = 0; sp < p.sk; sp++) { // ascending k
#pragma unroll
                        for (int b = 0; b < BATCH; b++) {
                            const int tok = tok0 + b * TOK_STEP;
                            if (tok < p.m) sum[b] += __ldcg(tile_parts + ((size_t)sp * p.mpad + tok) * FT_ROWS + nn);
                        }
                    }
#pragma unroll
                    for (int b = 0; b < BATCH; b++) {
                        const int tok = tok0 + b * TOK_STEP;
                        if (tok < p.m) store_as(p.y, p.y_dtype, (size_t)tok * p.ldy + p.col_base + n0 + nn, sum[b] + bv);
                    }
                }
                if (et == 0) atomicAnd(p.tickets + (blockIdx.x >> 1), ~(0xFFFFu << shift)); // zero again for the next call
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
    return m >= 1 && m <= FT_MAX_M && n % FT_ROWS == 0 && k % (FT_BK * FT_ROUND) == 0 && group_size % FT_BK == 0 &&
           (group_size & (group_size - 1)) == 0 &&
           (scales_dtype == OXQ_F16 || scales_dtype == OXQ_BF16) && aligned(x, 16) && aligned(qweight, 16) && aligned(scales, 16);
}

// layout 0 = AWQ, 1 = GPTQ 4-bit (sym: no stored zero points), 2 = FP8 E4M3 (qweight = the bytes, scale_inv / s_in /
// block_out / block_in describe the scale grid; qzeros, scales unused).
static int fused_launch(int layout, FusedParams p, const void *x, const void *qweight, int m, int k, int n, cudaStream_t st,
                        void *scratch, size_t scratch_bytes)
{
    const int raw_bytes = layout == 2 ? FT_ROWS * FT_BK : FT_BOX_BYTES + 384;
    p.mpad = (m + 15) / 16 * 16;
    p.stage_bytes = FT_A_BYTES + p.mpad * 128;
    const int fixed = 1024 + 8 * FT_NUM_BARS + 16 + (layout == 2 ? (k / p.block_in) * 4 + 16 : 0);
    const int nk = k / FT_BK;
    // FP8: eight operand slots (each team two rounds ahead of the MMAs) when that leaves at least eight boxes in flight,
    // else four; the rest of shared memory is the ring of packed boxes, a multiple of four. (FP8, 32 tokens on a
    // 14336 x 4096 layer: 29.2 us with four slots, 24.3 us with eight; AWQ, bound by its unpack arithmetic: no change.)
    constexpr int UNIT = FT_ROUND * FT_TEAMS;
    p.stages = layout == 2 ? 2 * UNIT : UNIT; // the 4-bit layouts lose a little to the shallower ring (GPTQ, 64 tokens: 31.4 -> 33.3 us)
    if ((FT_SMEM_BUDGET - fixed - p.stages * p.stage_bytes) / raw_bytes < 8) p.stages = UNIT;
    if (const char *env = tuning_env("OXQ_AWQ_FUSED_STAGES")) p.stages = atoi(env) == UNIT ? UNIT : p.stages;
    p.raw_slots = (FT_SMEM_BUDGET - fixed - p.stages * p.stage_bytes) / raw_bytes / UNIT * UNIT;
    if (p.raw_slots > FT_MAX_RAW) p.raw_slots = FT_MAX_RAW;
    if (const char *env = tuning_env("OXQ_AWQ_FUSED_RAW")) p.raw_slots = atoi(env) < p.raw_slots ? atoi(env) : p.raw_slots;
    if (p.raw_slots < UNIT || nk < 1) return OXQ_ERR_UNSUPPORTED; // the caller takes the slab path
    p.tmem_cols = 32;
    while (p.tmem_cols < p.mpad) p.tmem_cols *= 2;
    // Few out-feature tiles (narrow layers: attention and down projections): split k over grid y so that about every SM has a
    // CTA. Splits are whole rounds, at least eight stages each; at most 126 tiles (the 16-bit tickets share the workspace header
    // with the flag word) and only while the partial tiles fit the scratch area.
    const int tiles = n / FT_ROWS, rounds = nk / FT_ROUND;
    p.sk = 1;
    p.partials = reinterpret_cast<float *>(scratch);
    p.tickets = reinterpret_cast<unsigned int *>(p.flag) + 1;
    if (tiles <= 126 && scratch != nullptr) {
        for (int cand = sm_count() / tiles; cand >= 2; cand--) {
            if (rounds % cand != 0 || nk / cand < 8) continue;
            if ((size_t)tiles * cand * p.mpad * FT_ROWS * sizeof(float) > scratch_bytes) continue;
            p.sk = cand;
            break;
        }
    }
    if (const char *env = tuning_env("OXQ_AWQ_FUSED_SK")) p.sk = atoi(env) >= 1 && rounds % atoi(env) == 0 && tiles <= 126 ? atoi(env) : p.sk;
    const size_t smem = (size_t)p.stages * p.stage_bytes + (size_t)p.raw_slots * raw_bytes + fixed;

    CUtensorMap wmap, xmap;
    CUresult r;
    if (layout == 1)
        r = encode_tiled_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, qweight, (uint64_t)n, (uint64_t)k / 8, (uint64_t)n * 4, 128, FT_BK / 8,
                            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    else if (layout == 2)
        r = encode_tiled_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, qweight, (uint64_t)k, (uint64_t)n, (uint64_t)k, FT_BK, FT_ROWS,
                            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    else
        r = encode_tiled_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, qweight, (uint64_t)p.packed_out, (uint64_t)k, (uint64_t)p.packed_out * 4,
                            16, FT_BK, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    OXQ_REQUIRE(r == CUDA_SUCCESS, OXQ_ERR_CUDA, "cuTensorMapEncodeTiled (weights) failed with CUresult %d", (int)r);
    r = encode_tiled_2d(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, (uint64_t)k, (uint64_t)m, (uint64_t)k * 2, FT_BK, (uint32_t)p.mpad,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    OXQ_REQUIRE(r == CUDA_SUCCESS, OXQ_ERR_CUDA, "cuTensorMapEncodeTiled (x) failed with CUresult %d", (int)r);

    static size_t configured[3][64] = {};
    int device = 0;
    OXQ_CUDA(cudaGetDevice(&device));
    if (device >= 64 || configured[layout][device] < smem) {
        if (layout == 1) OXQ_CUDA(cudaFuncSetAttribute(awq_fused_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        else if (layout == 2) OXQ_CUDA(cudaFuncSetAttribute(awq_fused_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        else OXQ_CUDA(cudaFuncSetAttribute(awq_fused_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (device < 64) configured[layout][device] = smem;
    }
    const dim3 grid(tiles, p.sk, 1);
    if (layout == 1) awq_fused_tc_kernel<1><<<grid, FT_THREADS, smem, st>>>(p, wmap, xmap);
    else if (layout == 2) awq_fused_tc_kernel<2><<<grid, FT_THREADS, smem, st>>>(p, wmap, xmap);
    else awq_fused_tc_kernel<0><<<grid, FT_THREADS, smem, st>>>(p, wmap, xmap);
    OXQ_CUDA(cudaGetLastError());
    return OXQ_OK;
}

int awq_fused_matmul(const void *x, const uint32_t *qweight, const uint32_t *qzeros, const void *scales, int scales_dtype, const void *bias,
                     int bias_dtype, void *y, int y_dtype, int m, int k, int n, int group_size, int col_base, int ldy,
                     int *flag, cudaStream_t st, int gptq, int sym, void *scratch, size_t scratch_bytes)
{
    FusedParams p = {};
    p.qzeros = qzeros; p.scales = scales; p.scales_dtype = scales_dtype; p.bias = bias; p.y = y;
    p.bias_dtype = bias_dtype; p.y_dtype = y_dtype;
    p.m = m; p.k = k; p.n = n; p.group_size = group_size; p.packed_out = n / 8;
    p.col_base = col_base; p.ldy = ldy; p.flag = flag;
    p.sym = (gptq && (sym || qzeros == nullptr)) ? 1 : 0;
    p.gshift = 0;
    while ((FT_BK << p.gshift) < group_size) p.gshift += 1;
    p.block_in = FT_BK; p.block_out = FT_ROWS; p.s_in = 1;
    return fused_launch(gptq ? 1 : 0, p, x, qweight, m, k, n, st, scratch, scratch_bytes);
}

bool fp8_fused_supported(int m, int k, int n, int block_out, int block_in, const void *x, const void *weight, const void *scale_inv)
{
    if (const char *env = tuning_env("OXQ_AWQ_FUSED"))
        if (env[0] == '0') return false;
    return m >= 1 && m <= FT_MAX_M && n % FT_ROWS == 0 && k % (FT_BK * FT_ROUND) == 0 && block_out % FT_ROWS == 0 &&
           block_in % FT_BK == 0 && k / block_in <= 1024 && aligned(x, 16) && aligned(weight, 16) && aligned(scale_inv, 4);
}

int fp8_fused_matmul(const void *x, const uint8_t *weight, const float *scale_inv, int s_in, int block_out, int block_in,
                     const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n, int *flag, cudaStream_t st,
                     void *scratch, size_t scratch_bytes)
{
    FusedParams p = {};
    p.bias = bias; p.y = y; p.bias_dtype = bias_dtype; p.y_dtype = y_dtype;
    p.m = m; p.k = k; p.n = n; p.group_size = FT_BK; p.packed_out = n / 8;
    p.col_base = 0; p.ldy = n; p.flag = flag;
    p.scale_inv = scale_inv; p.s_in = s_in; p.block_out = block_out; p.block_in = block_in;
    return fused_launch(2, p, x, weight, m, k, n, st, scratch, scratch_bytes);
}

} // namespace oxq
