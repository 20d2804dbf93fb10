// Grouped expert matmul of the GPT-OSS MoE layer on MXFP4 weights, with the dequantization inside the
// tensor-core kernel: the packed blocks are read once and no dense copy of the expert weights is written.
// Mirrors the expert half of MoeFeedForward::forward (moe.rs:466-499, dispatch_sparse 563-607) with the
// experts' Mxfp4Linear weights (linear.rs, [experts, out, in / 32, 16] blocks + [experts, out, in / 32] scales).
//
// A unit of work is (token block of one expert: up to 256 expert-sorted rows) x (128 out features). The grid is
// persistent: CTA b takes units b, b + grid, ... of a device-side table, feature tiles fastest, so that CTAs
// running at the same time share their token block in L2. Per CTA:
//   warp 0 (one lane)   TMA: boxes of packed nibbles (128 out features x 32 bytes = 64 input columns) into a
//                       ring of six slots;
//   warp 2 (one lane)   TMA: the stage's tile of the activations ([rows, 64] bf16 in boxes of 64 rows, 128-byte
//                       swizzle) into one of four slots;
//   warps 4..19         unpack, two teams of eight warps taking stages in turn: a thread turns one 16-byte block
//                       (32 weights; its E8M0 scale byte read through L1/L2) into 32 bf16 weights, the bits the
//                       dequantization kernel writes, as four 16-byte chunks of the K-major operand row (128-byte
//                       swizzle) in one of four slots;
//   warp 1 (one lane)   tcgen05.mma kind::f16, A = weights [128, 64], B = activations, D[128, rows] f32 in one of
//                       two tensor-memory buffers for the whole of k; one commit per stage frees the slot (weights and
//                       activations share a full / empty barrier pair per slot, so the issuer polls once per stage);
//   warps 20..23        epilogue of the previous unit while the next one accumulates: accumulator rows (out
//                       features) -> + bias -> bf16 out[row, feature], or the clamped SwiGLU of GPT-OSS on
//                       interleaved (gate, up) features -> out[row, feature / 2].
// Every wait is bounded and reports through the workspace flag word.
#include <cuda_bf16.h>

#include "tc_common.cuh"

namespace oxq {

#ifdef OXQ_TUNING
#define MF_DBG(bit) (p.dbg & (bit))
__device__ long long g_mf_trace[10][256]; // clock stamps of CTA 0, per role and stage (tuning builds only)
#define MF_TRACE(role, it) do { if (blockIdx.x == 0 && (it) < 256) g_mf_trace[role][it] = clock64(); } while (0)
#else
#define MF_DBG(bit) 0
#define MF_TRACE(role, it) do { } while (0)
#endif

constexpr int MF_ROWS = 128;                   // out features per unit
constexpr int MF_BK = 64;                      // input columns per stage
constexpr int MF_UNPACK_WARPS = 16, MF_TEAMS = 2, MF_TEAM_WARPS = 8, MF_ROUND = 1;
constexpr int MF_EPI_WARPS = 4;
constexpr int MF_THREADS = (4 + MF_UNPACK_WARPS + MF_EPI_WARPS) * 32;
constexpr int MF_SLOTS = 4;                    // operand slots: an unpacked weight tile and an activation tile each, one pair of barriers
constexpr int MF_A_SLOTS = MF_SLOTS, MF_X_SLOTS = MF_SLOTS;
constexpr int MF_RAW_SLOTS = 6;
constexpr int MF_MAX_TOK = 256;                // rows of a token block
constexpr int MF_TMEM_BUF = 256;               // accumulator columns per buffer
constexpr int MF_A_BYTES = MF_ROWS * MF_BK * 2;
constexpr int MF_XBOX_ROWS = 64, MF_XBOX_BYTES = MF_XBOX_ROWS * MF_BK * 2, MF_X_BYTES = MF_MAX_TOK * MF_BK * 2; // activation rows travel in boxes of 64
constexpr int MF_RAW_BYTES = MF_ROWS * MF_BK / 2;
constexpr int MF_NUM_BARS = 2 * MF_RAW_SLOTS + 2 * MF_SLOTS + 4;
static_assert(MF_RAW_SLOTS % MF_ROUND == 0 && MF_A_SLOTS % MF_ROUND == 0, "a round's slots are neighbours");
constexpr int MF_SMEM_BUDGET = 227 * 1024;

struct MoeFusedParams {
    const int4 *entries;   // token blocks: {first row in the expert-sorted matrix, rows (<= 256), expert, -}
    const int *n_blocks;   // how many
    const uint8_t *scales; // [experts, n, k / 32]
    const void *bias;      // [experts, n] or null
    void *out;
    int *flag;
    int n, k, nkb, nk2;    // out features per expert, in features, scale bytes per row, stages per unit (whole rounds)
    int tiles_n, bias_dtype, ldo, epi;
    float limit;
    int dbg;               // tuning builds: parts of the pipeline switched off for timing
    int test_skip_loads;   // self-test only: the weight producer issues nothing, so the waits of the other roles run out
};

__device__ __forceinline__ uint4 mf_lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void mf_sts128(uint32_t addr, const uint4 &v)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void mf_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__global__ void __launch_bounds__(MF_THREADS, 1)
    moe_mxfp4_fused_kernel(const MoeFusedParams p, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap)
{
    extern __shared__ unsigned char smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u; // operand slots want 1 KB alignment
    unsigned char *base_ptr = smem_raw + (base - smem_u32(smem_raw));
    // A slots | activation slots | ring of packed boxes | barriers | tensor-memory address
    const uint32_t x_base = base + MF_A_SLOTS * MF_A_BYTES;
    const uint32_t raw_base = x_base + MF_X_SLOTS * MF_X_BYTES;
    const uint32_t bars = raw_base + MF_RAW_SLOTS * MF_RAW_BYTES;
    auto rawfull_bar = [&](int r) { return bars + 8u * r; };
    auto rawempty_bar = [&](int r) { return bars + 8u * (MF_RAW_SLOTS + r); };
    // full: the slot's weight tile is unpacked (one arrival per warp of the team) and its activation tile has landed (the
    // producer's arrival with the byte count); empty: the MMAs that read the slot have completed (one commit)
    auto full_bar = [&](int s) { return bars + 8u * (2 * MF_RAW_SLOTS + s); };
    auto empty_bar = [&](int s) { return bars + 8u * (2 * MF_RAW_SLOTS + MF_SLOTS + s); };
    const uint32_t misc = bars + 8u * (2 * MF_RAW_SLOTS + 2 * MF_SLOTS);
    auto tfull_bar = [&](int b) { return misc + 8u * b; };
    auto tempty_bar = [&](int b) { return misc + 8u * (2 + b); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(base_ptr + (bars - base) + 8 * MF_NUM_BARS);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_units = __ldg(p.n_blocks) * p.tiles_n;
    const int nk2 = p.nk2;

    if (threadIdx.x == 0) {
        for (int r = 0; r < MF_RAW_SLOTS; r++) {
            mbar_init(rawfull_bar(r), 1);
            mbar_init(rawempty_bar(r), MF_TEAM_WARPS);
        }
        for (int s = 0; s < MF_SLOTS; s++) {
            mbar_init(full_bar(s), MF_TEAM_WARPS + 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(tfull_bar(b), 1);
            mbar_init(tempty_bar(b), MF_EPI_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) { // the allocating warp also frees
        tmem_alloc(smem_u32(tmem_slot), 512u);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- TMA, packed nibbles -----------------------------------------------------------------------
        if (elect_one()) {
            uint32_t gs = 0, ul = 0;
            bool ok = true;
            for (int u = blockIdx.x; ok && u < n_units && !p.test_skip_loads; u += gridDim.x, ul++) {
                const int tb = u / p.tiles_n, f = u - tb * p.tiles_n;
                const int4 en = __ldg(p.entries + tb);
                const int rowbase = en.z * p.n + f * MF_ROWS;
                for (int it = 0; it < nk2; it++, gs++) {
                    const uint32_t r = gs % MF_RAW_SLOTS;
                    if (gs >= MF_RAW_SLOTS && !mbar_wait(rawempty_bar(r), ((gs / MF_RAW_SLOTS) & 1u) ^ 1u, p.flag, 1)) { ok = false; break; }
                    MF_TRACE(0, gs);
                    if (MF_DBG(8)) { mf_arrive(rawfull_bar(r)); continue; }
                    mbar_arrive_expect_tx(rawfull_bar(r), MF_RAW_BYTES);
                    tma_load_2d(raw_base + r * MF_RAW_BYTES, &wmap, rawfull_bar(r), it * (MF_BK / 2), rowbase);
                }
            }
        }
    } else if (warp == 2) {
        // ---- TMA, activation tiles ----------------------------------------------------------------------
        if (elect_one()) {
            int xs = 0;
            uint32_t xph = 0, gx = 0;
            bool ok = true;
            for (int u = blockIdx.x; ok && u < n_units; u += gridDim.x) {
                const int4 en = __ldg(p.entries + u / p.tiles_n);
                const int boxes = (en.y + MF_XBOX_ROWS - 1) / MF_XBOX_ROWS;
                for (int it = 0; it < nk2; it++, gx++) {
                    if (gx >= MF_SLOTS && !mbar_wait(empty_bar(xs), xph ^ 1u, p.flag, 5)) { ok = false; break; }
                    const uint32_t dst = x_base + (uint32_t)xs * MF_X_BYTES;
                    MF_TRACE(1, gx);
                    if (MF_DBG(2)) mf_arrive(full_bar(xs));
                    else {
                    mbar_arrive_expect_tx(full_bar(xs), (uint32_t)boxes * MF_XBOX_BYTES);
                    for (int b = 0; b < boxes; b++)
                        tma_load_2d(dst + (uint32_t)b * MF_XBOX_BYTES, &xmap, full_bar(xs), it * MF_BK, en.x + b * MF_XBOX_ROWS);
                    }
                    if (++xs == MF_X_SLOTS) { xs = 0; xph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue ----------------------------------------------------------------------------------
        if (elect_one()) {
            // One thread issues every MMA of the CTA, so its instruction count per stage is on the critical path: the loop
            // runs over all stages of all this CTA's units, four at a time, so that slot, barrier and descriptor addresses are
            // constants of the unrolled body; one poll (full) and one commit (empty) per stage.
            int my_units = 0;
            if ((int)blockIdx.x < n_units) my_units = (n_units - 1 - (int)blockIdx.x) / (int)gridDim.x + 1;
            const uint32_t total = (uint32_t)my_units * (uint32_t)nk2;
            const uint64_t da0 = kmajor_sw128_desc(base), db0 = kmajor_sw128_desc(x_base);
            const uint32_t full0 = full_bar(0), empty0 = empty_bar(0);
            uint32_t ul = 0, idesc = 0, d_tmem = tmem_base, buf = 0;
            int it = 0;
            bool ok = true;
            auto stage = [&](const uint32_t gs, const int j) { // j = gs % MF_SLOTS, a constant after unrolling
                if (it == 0) { // first stage of a unit
                    const int u = (int)blockIdx.x + (int)ul * (int)gridDim.x;
                    const int rows = __ldg(p.entries + u / p.tiles_n).y;
                    idesc = tc_idesc(MF_ROWS, (rows + 15) & ~15);
                    buf = ul & 1u;
                    if (ul >= 2 && !mbar_wait(tempty_bar(buf), ((ul >> 1) & 1u) ^ 1u, p.flag, 8)) { ok = false; return; }
                    d_tmem = tmem_base + buf * MF_TMEM_BUF;
                }
                MF_TRACE(7, gs);
                if (!mbar_wait(full0 + 8u * j, (gs / MF_SLOTS) & 1u, p.flag, 2)) { ok = false; return; }
                MF_TRACE(2, gs);
                tc_fence_after();
                const uint64_t da = da0 + (uint64_t)(j * (MF_A_BYTES >> 4)), db = db0 + (uint64_t)(j * (MF_X_BYTES >> 4));
                if (!MF_DBG(4))
#pragma unroll
                for (int kk = 0; kk < MF_BK / 16; kk++) // 16 input columns: 32 bytes inside a swizzled K-major row
                    umma_bf16(d_tmem, da + 2 * kk, db + 2 * kk, idesc, (it | kk) != 0);
                umma_commit(empty0 + 8u * j);
                MF_TRACE(3, gs);
                if (++it == nk2) { // last stage of the unit: the accumulator is complete once these MMAs are
                    umma_commit(tfull_bar(buf));
                    it = 0;
                    ul += 1;
                }
            };
            for (uint32_t g = 0; ok && g < total; g += MF_SLOTS) {
#pragma unroll
                for (int j = 0; j < MF_SLOTS; j++)
                    if (ok && g + j < total) stage(g + j, j);
            }
        }
    } else if (warp >= 4 && warp < 4 + MF_UNPACK_WARPS) {
        // ---- unpack ---------------------------------------------------------------------------------------
        const int team = (warp - 4) / MF_TEAM_WARPS;
        const int ut = (threadIdx.x - 128) % (MF_TEAM_WARPS * 32);
        const int row = ut >> 1, half = ut & 1;                   // this thread: one 16-byte block of one out feature per stage
        const uint32_t raw_off = (uint32_t)row * 32u + (uint32_t)half * 16u;
        const uint32_t a_row = (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u;
        const uint32_t sw = (uint32_t)(row & 7);
        const int rpu = nk2 / MF_ROUND;                            // rounds per unit
        int my_units = 0;
        if ((int)blockIdx.x < n_units) my_units = (n_units - 1 - (int)blockIdx.x) / (int)gridDim.x + 1;
        const uint32_t total_rounds = (uint32_t)my_units * (uint32_t)rpu;
        uint32_t cur_ul = 0xFFFFFFFFu, r_in_unit = 0, ul = 0;
        const uint8_t *srow = nullptr;
        bool ok = true;
        // rounds are counted over all units of this CTA, so slots and teams keep alternating across unit boundaries
        for (uint32_t gr = (uint32_t)team; gr < total_rounds; gr += MF_TEAMS) {
            ul = gr / (uint32_t)rpu;
            r_in_unit = gr - ul * (uint32_t)rpu;
            if (ul != cur_ul) { // first round of this team in a new unit: this thread's row of the scale bytes
                cur_ul = ul;
                const int u = (int)blockIdx.x + (int)ul * (int)gridDim.x;
                const int tb = u / p.tiles_n, f = u - tb * p.tiles_n;
                const int e = __ldg(p.entries + tb).z;
                srow = (f * MF_ROWS + row < p.n) ? p.scales + ((size_t)e * p.n + f * MF_ROWS + row) * p.nkb : nullptr;
            }
            // the scale bytes of the round's two blocks come straight from L2 (the row's bytes are neighbours, so most loads
            // hit L1); they are asked for before the polls, which hide their latency. Past k (zero-filled boxes) and past the
            // expert's last out feature: 1.0
            const int kb0 = (int)r_in_unit * (2 * MF_ROUND) + half;
            uint32_t sbv[MF_ROUND];
#pragma unroll
            for (int h = 0; h < MF_ROUND; h++) sbv[h] = (srow != nullptr && kb0 + 2 * h < p.nkb) ? (uint32_t)__ldg(srow + kb0 + 2 * h) : 127u;
            const uint32_t gs0 = gr * MF_ROUND;
            const uint32_t r0 = gs0 % MF_RAW_SLOTS, rph = (gs0 / MF_RAW_SLOTS) & 1u;
            const uint32_t s0 = gs0 % MF_A_SLOTS, aph = (gs0 / MF_A_SLOTS) & 1u;
            // all polls of the round first (they do not depend on each other), the bounded waits only where one failed
            bool tr[MF_ROUND], ta[MF_ROUND];
#pragma unroll
            for (int h = 0; h < MF_ROUND; h++) {
                tr[h] = mbar_test(rawfull_bar(r0 + h), rph);
                ta[h] = gs0 < MF_SLOTS || mbar_test(empty_bar(s0 + h), aph ^ 1u);
            }
#pragma unroll
            for (int h = 0; h < MF_ROUND; h++) {
                if (ok && !tr[h]) ok = mbar_wait(rawfull_bar(r0 + h), rph, p.flag, 3);
                if (ok && !ta[h]) ok = mbar_wait(empty_bar(s0 + h), aph ^ 1u, p.flag, 7);
            }
            if (!ok) break;
            if (ut == 0) MF_TRACE(4, gs0);
            if (!MF_DBG(1))
#pragma unroll
            for (int h = 0; h < MF_ROUND; h++) {
                const uint32_t sb = sbv[h];
                const uint4 rawv = mf_lds128(raw_base + (r0 + h) * MF_RAW_BYTES + raw_off);
                const uint32_t v[4] = {rawv.x, rawv.y, rawv.z, rawv.w};
                const uint32_t dst = base + (s0 + h) * MF_A_BYTES + a_row;
                if (sb >= 4u && sb <= 250u) { // 2^(s-127) as a bf16 pair: the products are exact
                    // The block's eight magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 times its scale, as bf16 (four multiplies for
                    // 32 weights), split into a table of low bytes and a table of high bytes; the byte permute unit then looks
                    // up four nibbles at a time, and each nibble's sign bit is copied onto its element (prmt's sign-replicate
                    // mode turns bit 7 of a byte into a mask).
                    const uint32_t s2 = (sb << 7) | (sb << 23);
                    const __nv_bfloat162 sc = *reinterpret_cast<const __nv_bfloat162 *>(&s2);
                    const uint32_t mags[4] = {0x3F000000u, 0x3FC03F80u, 0x40404000u, 0x40C04080u}; // (0, .5) (1, 1.5) (2, 3) (4, 6)
                    uint32_t pm[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const __nv_bfloat162 t = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&mags[i]), sc);
                        pm[i] = *reinterpret_cast<const uint32_t *>(&t);
                    }
                    const uint32_t tlo_a = __byte_perm(pm[0], pm[1], 0x6420u), thi_a = __byte_perm(pm[0], pm[1], 0x7531u);
                    const uint32_t tlo_b = __byte_perm(pm[2], pm[3], 0x6420u), thi_b = __byte_perm(pm[2], pm[3], 0x7531u);
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const uint32_t w = v[q];
                        const uint32_t sel_l = w & 0x77777777u, sel_h = sel_l >> 16, wl = w << 4;
                        const uint32_t lo_a = __byte_perm(tlo_a, tlo_b, sel_l), hi_a = __byte_perm(thi_a, thi_b, sel_l);
                        const uint32_t lo_b = __byte_perm(tlo_a, tlo_b, sel_h), hi_b = __byte_perm(thi_a, thi_b, sel_h);
                        const uint32_t pr[4] = {__byte_perm(lo_a, hi_a, 0x5140u), __byte_perm(lo_a, hi_a, 0x7362u),
                                                __byte_perm(lo_b, hi_b, 0x5140u), __byte_perm(lo_b, hi_b, 0x7362u)};
                        uint4 o;
                        uint32_t *ov = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
                        for (int b = 0; b < 4; b++) {
                            // byte 1 <- sign of the low nibble of byte b (bit 7 of (w << 4)), byte 3 <- sign of the high nibble
                            const uint32_t sm = __byte_perm(wl, w, 0xC080u + 0x1010u * b);
                            asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(ov[b]) : "r"(sm), "r"(0x80008000u), "r"(pr[b])); // (sm & mask) ^ pr
                        }
                        mf_sts128(dst + ((((uint32_t)(half * 4 + q)) ^ sw) << 4), o);
                    }
                } else { // scales whose products leave the normal range (NaN, 2^-127 among them): f32 product, one rounding
                    const float s = e8m0_to_f32(sb);
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        uint4 o;
                        uint32_t *ov = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
                        for (int b = 0; b < 4; b++) {
                            const uint32_t by = (v[q] >> (8 * b)) & 0xFFu;
                            const __nv_bfloat162 hh = __halves2bfloat162(narrow<__nv_bfloat16>(__fmul_rn(e2m1_to_f32(by & 0xFu), s)),
                                                                         narrow<__nv_bfloat16>(__fmul_rn(e2m1_to_f32(by >> 4), s)));
                            ov[b] = *reinterpret_cast<const uint32_t *>(&hh);
                        }
                        mf_sts128(dst + ((((uint32_t)(half * 4 + q)) ^ sw) << 4), o);
                    }
                }
            }
            if (ut == 0) MF_TRACE(5, gs0);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // generic-proxy stores -> visible to the MMA
            __syncwarp();
            if (lane == 0) {
#pragma unroll
                for (int h = 0; h < MF_ROUND; h++) {
                    mf_arrive(full_bar(s0 + h));
                    mf_arrive(rawempty_bar(r0 + h));
                }
            }
            if (ut == 0) MF_TRACE(6, gs0);
        }
    } else if (warp >= 4 + MF_UNPACK_WARPS) {
        // ---- epilogue: lane = out feature inside this warp's quarter of the accumulator rows ---------------
        const int quad = warp & 3;
        uint32_t ul = 0;
        __nv_bfloat16 *outp = reinterpret_cast<__nv_bfloat16 *>(p.out);
        for (int u = blockIdx.x; u < n_units; u += gridDim.x, ul++) {
            const int tb = u / p.tiles_n, f = u - tb * p.tiles_n;
            const int4 en = __ldg(p.entries + tb);
            const int mpad = (en.y + 15) & ~15;
            const uint32_t buf = ul & 1u;
            if (!mbar_wait(tfull_bar(buf), (ul >> 1) & 1u, p.flag, 4)) break;
            tc_fence_after();
            const int feat = f * MF_ROWS + quad * 32 + lane;
            const bool fv = feat < p.n;
            const float bv = (p.bias && fv) ? load_as_f32(p.bias, p.bias_dtype, (size_t)en.z * p.n + feat) : 0.0f;
            for (int c0 = 0; c0 < mpad; c0 += 32) {
                uint32_t rr[32];
                tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + buf * MF_TMEM_BUF + (uint32_t)c0, rr);
                tmem_ld_wait();
                if (p.epi == 0) {
#pragma unroll
                    for (int c = 0; c < 32; c++)
                        if (fv && c0 + c < en.y)
                            outp[(size_t)(en.x + c0 + c) * p.ldo + feat] = __float2bfloat16_rn(__uint_as_float(rr[c]) + bv);
                } else {
                    // even lane = gate feature, odd lane = up feature of the same output column; the even lane takes the
                    // even row of a pair of rows and the odd lane the odd one, so one exchange serves two rows
                    const bool odd = lane & 1;
#pragma unroll
                    for (int c = 0; c < 32; c += 2) {
                        const float mine0 = __uint_as_float(rr[c]) + bv, mine1 = __uint_as_float(rr[c + 1]) + bv;
                        const float other = __shfl_xor_sync(0xFFFFFFFFu, odd ? mine0 : mine1, 1);
                        float gate = odd ? other : mine0, up = odd ? mine1 : other;
                        gate = fminf(gate, p.limit);
                        up = fminf(fmaxf(up, -p.limit), p.limit);
                        const float sig = __fdividef(1.0f, __expf(-1.702f * gate) + 1.0f);
                        const int rowi = c0 + c + (odd ? 1 : 0);
                        if (fv && rowi < en.y)
                            outp[(size_t)(en.x + rowi) * p.ldo + (feat >> 1)] = __float2bfloat16_rn((up + 1.0f) * (gate * sig));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mf_arrive(tempty_bar(buf));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512u);
    }
}

static thread_local int g_moe_selftest_skip_loads = 0; // set only inside oxq_selftest_moe_wait_expiry

// Rows of a token block (the plan kernel cuts every expert's rows into blocks of at most this many).
int moe_fused_block_rows() { return MF_MAX_TOK; }

// True when the fused grouped kernel serves these expert weights; otherwise the caller dequantizes expert groups.
bool moe_fused_supported(int n, int k, const void *blocks, const void *scales, const void *a, const void *out, int ldo)
{
    if (const char *env = tuning_env("OXQ_MOE_FUSED"))
        if (env[0] == '0') return false;
    // k % 32 == 0: whole MXFP4 blocks, and the packed rows (k / 2 bytes) keep the 16-byte pitch a tensor map needs
    if (n <= 0 || k <= 0 || k % 32 != 0 || n % 2 != 0 || scales == nullptr) return false;
    return aligned(blocks, 16) && aligned(a, 16) && aligned(out, 2) && ldo > 0;
}

// out = epilogue(a . W_e^T + bias_e) for every token block of the table: a = expert-sorted activations [a_rows, k] bf16,
// blocks / scales = the MXFP4 weights of all `experts` experts, n out features each. epi 0: bias; epi 1: clamped SwiGLU.
int moe_fused_grouped(const void *a, int a_rows, const uint8_t *blocks, const uint8_t *scales, int experts, int n, int k,
                      const int4 *entries, const int *n_blocks, const void *bias, int bias_dtype, void *out, int ldo, int epi,
                      float limit, int *flag, cudaStream_t st)
{
    MoeFusedParams p = {};
    p.entries = entries; p.n_blocks = n_blocks; p.scales = scales; p.bias = bias; p.out = out; p.flag = flag;
    p.n = n; p.k = k; p.nkb = k / 32;
    const int nk = (k + MF_BK - 1) / MF_BK;
    p.nk2 = (nk + MF_ROUND - 1) / MF_ROUND * MF_ROUND;
    p.tiles_n = (n + MF_ROWS - 1) / MF_ROWS;
    p.bias_dtype = bias_dtype; p.ldo = ldo; p.epi = epi; p.limit = limit;
    p.test_skip_loads = g_moe_selftest_skip_loads;
    if (const char *env = tuning_env("OXQ_MF_DBG")) p.dbg = atoi(env);
    constexpr size_t smem = 1024 + MF_A_SLOTS * MF_A_BYTES + MF_X_SLOTS * MF_X_BYTES + MF_RAW_SLOTS * MF_RAW_BYTES + 8 * MF_NUM_BARS + 16;
    static_assert(smem <= (size_t)MF_SMEM_BUDGET, "operand slots and the ring must fit one CTA's shared memory");
    CUtensorMap wmap, xmap;
    CUresult r = encode_tiled_2d(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, blocks, (uint64_t)k / 2, (uint64_t)experts * n, (uint64_t)k / 2,
                                 MF_BK / 2, MF_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    OXQ_REQUIRE(r == CUDA_SUCCESS, OXQ_ERR_CUDA, "cuTensorMapEncodeTiled (expert blocks) failed with CUresult %d", (int)r);
    r = encode_tiled_2d(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a, (uint64_t)k, (uint64_t)a_rows, (uint64_t)k * 2, MF_BK, MF_XBOX_ROWS,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    OXQ_REQUIRE(r == CUDA_SUCCESS, OXQ_ERR_CUDA, "cuTensorMapEncodeTiled (expert rows) failed with CUresult %d", (int)r);
    static size_t configured[64] = {};
    int device = 0;
    OXQ_CUDA(cudaGetDevice(&device));
    if (device >= 64 || configured[device] < smem) {
        OXQ_CUDA(cudaFuncSetAttribute(moe_mxfp4_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (device < 64) configured[device] = smem;
    }
    moe_mxfp4_fused_kernel<<<sm_count(), MF_THREADS, smem, st>>>(p, wmap, xmap);
    OXQ_LAUNCH_CHECK("moe_mxfp4_fused_kernel");
    return OXQ_OK;
}

} // namespace oxq

// Self-test of the grouped kernel's abort path: one unit (one expert, 128 out features, 64 in features, 16 rows) whose
// weight producer never loads. The unpack teams, the MMA issuer, the activation producer and the epilogue warps each give
// up on their bounded wait (about two seconds, side by side), the flag word of the workspace takes the first code,
// tensor memory is freed and the kernel returns; oxq_gemm_check(workspace) then reports it. Nothing faults or hangs.
OXQ_EXPORT int oxq_selftest_moe_wait_expiry(void *workspace, size_t workspace_bytes, void *stream)
{
    oxq::clear_error();
    OXQ_REQUIRE(workspace && workspace_bytes >= (1u << 20) && oxq::aligned(workspace, 256), OXQ_ERR_WORKSPACE,
                "oxq_selftest_moe_wait_expiry: 256-byte aligned workspace of at least 1 MiB needed");
    unsigned char *b = reinterpret_cast<unsigned char *>(workspace);
    cudaStream_t st = (cudaStream_t)stream;
    const int n = 128, k = 64, rows = 16;
    // table | rows [256 + 128, 64] bf16 | blocks [128, 32] | scales [128, 2] | out [256, 128] bf16
    int4 *entries = reinterpret_cast<int4 *>(b + 4096);
    int *n_blocks = reinterpret_cast<int *>(b + 4096 + 64);
    void *a = b + 8192;
    uint8_t *blocks = b + 8192 + 384 * 64 * 2, *scales = blocks + 128 * 32;
    void *out = b + 131072;
    const int4 en = make_int4(0, rows, 0, 0);
    const int one = 1;
    OXQ_CUDA(cudaMemcpyAsync(entries, &en, sizeof(en), cudaMemcpyHostToDevice, st));
    OXQ_CUDA(cudaMemcpyAsync(n_blocks, &one, sizeof(one), cudaMemcpyHostToDevice, st));
    OXQ_CUDA(cudaStreamSynchronize(st)); // the two host words above live on this stack frame
    oxq::g_moe_selftest_skip_loads = 1;
    const int rc = oxq::moe_fused_grouped(a, 384, blocks, scales, 1, n, k, entries, n_blocks, nullptr, 0, out, n, 0, 0.0f,
                                          reinterpret_cast<int *>(workspace), st);
    oxq::g_moe_selftest_skip_loads = 0;
    return rc;
}

#ifdef OXQ_TUNING
OXQ_EXPORT int oxq_mf_trace_read(long long *out)
{
    return cudaMemcpyFromSymbol(out, oxq::g_mf_trace, sizeof(oxq::g_mf_trace)) == cudaSuccess ? 0 : 1;
}
#endif
