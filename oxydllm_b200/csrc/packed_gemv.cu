// Decode GEMVs of the packed-int layouts that the tensor-core AWQ 4-bit kernels do not cover, on the
// packed weights as stored (nothing is dequantized to memory):
//
//   GPTQ 4/8-bit  qweight u32 [k / pf, n], pf = 32 / bits consecutive INPUT rows of one column per word,
//                 LSB first; qzeros u32 [k / g, n / pf] along n; w = (q - (zero + 1)) * scale, or with the
//                 symmetric zero 2^(bits-1) - 1 when `sym` or no qzeros (awq.rs:561-590)
//   W8A16         the AWQ layout at 8 bits: qweight u32 [k, n / 4], byte c of word j = out column 4 j + c
//                 (no interleave), qzeros u32 [k / g, n / 4]; w = (q - zero) * scale
//                 (quant_kernels.metal:1-16,40-48)
//
// One thread owns one output column (GPTQ) or the four columns of a word (W8A16), so a warp reads 128
// contiguous bytes per packed row; the 8 warps of a CTA split k by quantization groups and meet in shared
// memory in warp order (fixed order: same bits every run). Activations are staged once per CTA as f32
// together with their per-group sums, so the zero point costs two FMAs per (group, token):
//   y += s * (sum_k q x - zero * sum_k x).
// Integers become floats with the 2^23 trick (0x4B000000 | q is 2^23 + q exactly; one subtraction).
#include "oxq_common.cuh"

namespace oxq {

constexpr int PG_WARPS = 8;
constexpr int PG_MAX_MT = 4; // tokens per launch (bounded by the f32 copy of x in shared memory)

struct PackedGemvParams {
    const __nv_bfloat16 *x;
    const uint32_t *qweight, *qzeros;
    const void *scales, *bias;
    void *y;
    int scales_dtype, bias_dtype, y_dtype;
    int m, k, n, group_size, sym;
    int y_row0; // first token of this launch (rows of x and y)
};

__device__ __forceinline__ float magic_to_f32(uint32_t bits_with_magic) { return __uint_as_float(bits_with_magic) - 8388608.0f; }

// x rows [row0, row0 + MT) -> f32 in shared memory, then sums over each quantization group (fixed-order tree).
template <int MT>
__device__ __forceinline__ void stage_x(const PackedGemvParams &p, float *xs, float *gsum)
{
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int mloc = min(MT, p.m - p.y_row0);
    for (int idx = tid; idx < mloc * (p.k >> 1); idx += PG_WARPS * 32) {
        const int tok = idx / (p.k >> 1), i2 = idx - tok * (p.k >> 1);
        const uint32_t raw = __ldg(reinterpret_cast<const uint32_t *>(p.x + (size_t)(p.y_row0 + tok) * p.k) + i2);
        *reinterpret_cast<float2 *>(xs + (size_t)tok * p.k + 2 * i2) = make_float2(bf16_lo_f32(raw), bf16_hi_f32(raw));
    }
    __syncthreads();
    const int groups = p.k / p.group_size;
    for (int pair = warp; pair < mloc * groups; pair += PG_WARPS) {
        const int tok = pair / groups, g = pair - tok * groups;
        const float *src = xs + (size_t)tok * p.k + (size_t)g * p.group_size;
        float s = 0.0f;
        for (int i = lane; i < p.group_size; i += 32) s += src[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
        if (lane == 0) gsum[tok * groups + g] = s;
    }
    __syncthreads();
}

template <int BITS, int MT>
__global__ void __launch_bounds__(PG_WARPS * 32) gptq_gemv_kernel(const PackedGemvParams p)
{
    pdl_launch_dependents();
    pdl_wait(); // x is staged first: only the start-up of the kernel overlaps the previous one
    constexpr int PF = 32 / BITS;
    constexpr uint32_t QMASK = (1u << BITS) - 1u;
    extern __shared__ __align__(16) float smem_f[];
    const int groups = p.k / p.group_size;
    float *xs = smem_f, *gsum = xs + (size_t)MT * p.k, *red = gsum + MT * groups;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int col = blockIdx.x * 32 + lane;
    const bool valid = col < p.n;
    const int c = valid ? col : p.n - 1; // lanes past the end read the last column; nothing of theirs is stored
    const int mloc = min(MT, p.m - p.y_row0);
    stage_x<MT>(p, xs, gsum);

    const int gp = (groups + PG_WARPS - 1) / PG_WARPS;
    const int g0 = warp * gp, g1 = min(groups, g0 + gp);
    const int wpg = p.group_size / PF; // packed rows per group
    float tot[MT];
#pragma unroll
    for (int t = 0; t < MT; t++) tot[t] = 0.0f;
    for (int g = g0; g < g1; g++) {
        const float s = load_as_f32(p.scales, p.scales_dtype, (size_t)g * p.n + c);
        float zero;
        if (p.sym || p.qzeros == nullptr) zero = (float)(1u << (BITS - 1));
        else zero = (float)(((__ldg(p.qzeros + (size_t)g * (p.n / PF) + c / PF) >> (BITS * (c % PF))) & QMASK) + 1u);
        float acc[MT];
#pragma unroll
        for (int t = 0; t < MT; t++) acc[t] = 0.0f;
        const uint32_t *wp = p.qweight + (size_t)g * wpg * p.n + c;
        const float *xg = xs + (size_t)g * p.group_size;
#pragma unroll 4
        for (int wi = 0; wi < wpg; wi++) {
            const uint32_t w = __ldcs(wp + (size_t)wi * p.n);
            float q[PF];
#pragma unroll
            for (int i = 0; i < PF; i++) q[i] = magic_to_f32(((w >> (BITS * i)) & QMASK) | 0x4B000000u);
#pragma unroll
            for (int t = 0; t < MT; t++) {
                if (t < mloc) {
                    const float4 *xv = reinterpret_cast<const float4 *>(xg + (size_t)t * p.k + wi * PF);
#pragma unroll
                    for (int i4 = 0; i4 < PF / 4; i4++) {
                        const float4 v = xv[i4];
                        acc[t] = fmaf(q[4 * i4], v.x, acc[t]);
                        acc[t] = fmaf(q[4 * i4 + 1], v.y, acc[t]);
                        acc[t] = fmaf(q[4 * i4 + 2], v.z, acc[t]);
                        acc[t] = fmaf(q[4 * i4 + 3], v.w, acc[t]);
                    }
                }
            }
        }
#pragma unroll
        for (int t = 0; t < MT; t++)
            if (t < mloc) tot[t] = fmaf(s, fmaf(-zero, gsum[t * groups + g], acc[t]), tot[t]);
    }
#pragma unroll
    for (int t = 0; t < MT; t++) red[(warp * MT + t) * 32 + lane] = tot[t];
    __syncthreads();
    for (int o = tid; o < mloc * 32; o += PG_WARPS * 32) {
        const int t = o >> 5, l = o & 31, oc = blockIdx.x * 32 + l;
        if (oc < p.n) {
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < PG_WARPS; w++) sum += red[(w * MT + t) * 32 + l];
            if (p.bias) sum += load_as_f32(p.bias, p.bias_dtype, oc);
            store_as(p.y, p.y_dtype, (size_t)(p.y_row0 + t) * p.n + oc, sum);
        }
    }
}

template <int MT>
__global__ void __launch_bounds__(PG_WARPS * 32) w8a16_gemv_kernel(const PackedGemvParams p)
{
    pdl_launch_dependents();
    pdl_wait(); // x is staged first: only the start-up of the kernel overlaps the previous one
    extern __shared__ __align__(16) float smem_f[];
    const int groups = p.k / p.group_size;
    float *xs = smem_f, *gsum = xs + (size_t)MT * p.k, *red = gsum + MT * groups;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int packed_out = p.n / 4;
    const int word = blockIdx.x * 32 + lane;
    const bool valid = word < packed_out;
    const int j = valid ? word : packed_out - 1;
    const int mloc = min(MT, p.m - p.y_row0);
    stage_x<MT>(p, xs, gsum);

    const int gp = (groups + PG_WARPS - 1) / PG_WARPS;
    const int g0 = warp * gp, g1 = min(groups, g0 + gp);
    float tot[4][MT];
#pragma unroll
    for (int cc = 0; cc < 4; cc++)
#pragma unroll
        for (int t = 0; t < MT; t++) tot[cc][t] = 0.0f;
    for (int g = g0; g < g1; g++) {
        const uint32_t zw = __ldg(p.qzeros + (size_t)g * packed_out + j);
        float s[4], zero[4];
#pragma unroll
        for (int cc = 0; cc < 4; cc++) {
            s[cc] = load_as_f32(p.scales, p.scales_dtype, (size_t)g * p.n + 4 * j + cc);
            zero[cc] = (float)((zw >> (8 * cc)) & 0xFFu);
        }
        float acc[4][MT];
#pragma unroll
        for (int cc = 0; cc < 4; cc++)
#pragma unroll
            for (int t = 0; t < MT; t++) acc[cc][t] = 0.0f;
        const uint32_t *wp = p.qweight + (size_t)g * p.group_size * packed_out + j;
        const float *xg = xs + (size_t)g * p.group_size;
#pragma unroll 8
        for (int i = 0; i < p.group_size; i++) {
            const uint32_t w = __ldcs(wp + (size_t)i * packed_out);
            // byte c of w under the float 2^23: one byte permute per value
            const float q0 = magic_to_f32(__byte_perm(w, 0x4B000000u, 0x7440)), q1 = magic_to_f32(__byte_perm(w, 0x4B000000u, 0x7441));
            const float q2 = magic_to_f32(__byte_perm(w, 0x4B000000u, 0x7442)), q3 = magic_to_f32(__byte_perm(w, 0x4B000000u, 0x7443));
#pragma unroll
            for (int t = 0; t < MT; t++) {
                if (t < mloc) {
                    const float xv = xg[(size_t)t * p.k + i];
                    acc[0][t] = fmaf(q0, xv, acc[0][t]);
                    acc[1][t] = fmaf(q1, xv, acc[1][t]);
                    acc[2][t] = fmaf(q2, xv, acc[2][t]);
                    acc[3][t] = fmaf(q3, xv, acc[3][t]);
                }
            }
        }
#pragma unroll
        for (int cc = 0; cc < 4; cc++)
#pragma unroll
            for (int t = 0; t < MT; t++)
                if (t < mloc) tot[cc][t] = fmaf(s[cc], fmaf(-zero[cc], gsum[t * groups + g], acc[cc][t]), tot[cc][t]);
    }
    // red[warp][token][column of the CTA's 128]
#pragma unroll
    for (int cc = 0; cc < 4; cc++)
#pragma unroll
        for (int t = 0; t < MT; t++) red[(warp * MT + t) * 128 + 4 * lane + cc] = tot[cc][t];
    __syncthreads();
    for (int o = tid; o < mloc * 128; o += PG_WARPS * 32) {
        const int t = o >> 7, l = o & 127, oc = blockIdx.x * 128 + l;
        if (oc < p.n) {
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < PG_WARPS; w++) sum += red[(w * MT + t) * 128 + l];
            if (p.bias) sum += load_as_f32(p.bias, p.bias_dtype, oc);
            store_as(p.y, p.y_dtype, (size_t)(p.y_row0 + t) * p.n + oc, sum);
        }
    }
}


// ---- GPTQ 4-bit on the tensor cores (m <= 8 per launch) ------------------------------------------------------
// A GPTQ word is 8 consecutive input rows of ONE output column: exactly what a lane of mma.sync.m16n8k16 needs for
// its row of the weight operand, so there is no gather between words. The order of k inside an MMA is free as
// long as x follows it: lane (g, c) of a warp takes the word of column n0 + g (and n0 + g + 8) at packed row
// 4 * step + c and spreads its nibbles over two MMAs: nibbles (0, 4) and (2, 6) become f16 pairs 1024 + q with one
// LOP3 each ((w & 0x000F000F) | 0x64006400), nibbles (1, 5) and (3, 7) become 1024 + 16 q without a shift
// ((w & 0x00F000F0) | 0x64006400) and meet x / 16. x is staged per CTA as f16 in that order
// [x0, x4, x1/16, x5/16, x2, x6, x3/16, x7/16], so one 16-byte read feeds both MMAs, together with the two sums per
// (group, token) that take the offsets and the zero point out again in f32:
//   y += s * (acc - 1024 * S1 - (zero + 1) * S2),  S1 = sum of the staged values, S2 = the same with the /16 undone.
__device__ __forceinline__ void mma_f16_16816_gptq(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int GQ_TILES = 2; // 16-column tiles per warp: a CTA covers 32 output columns

__global__ void __launch_bounds__(PG_WARPS * 32) gptq4_gemv_mma_kernel(const PackedGemvParams p)
{
    pdl_launch_dependents();
    pdl_wait(); // x is staged first: only the start-up of the kernel overlaps the previous one
    extern __shared__ __align__(16) unsigned char smem_b[];
    const int groups = p.k / p.group_size;
    const int mloc = min(8, p.m - p.y_row0);
    // layout: x as permuted f16 [mloc][k], one 16-byte block of zeros, sums float2 {1024 S1, S2} [groups][8], reduction scratch
    __half *xs = reinterpret_cast<__half *>(smem_b);
    uint4 *zeros = reinterpret_cast<uint4 *>(smem_b + (size_t)mloc * p.k * 2);
    float2 *sums = reinterpret_cast<float2 *>(zeros + 1);
    float *red = reinterpret_cast<float *>(sums + (size_t)groups * 8);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, c = lane & 3;

    // ---- stage x (8 values per thread and step) and the per-group sums ---------------------------------------
    if (tid == 0) *zeros = make_uint4(0u, 0u, 0u, 0u);
    const int blocks_per_row = p.k >> 3;
    for (int idx = tid; idx < mloc * blocks_per_row; idx += PG_WARPS * 32) {
        const int tok = idx / blocks_per_row, b = idx - tok * blocks_per_row;
        const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(p.x + (size_t)(p.y_row0 + tok) * p.k) + b);
        const float v[8] = {bf16_lo_f32(raw.x), bf16_hi_f32(raw.x), bf16_lo_f32(raw.y), bf16_hi_f32(raw.y),
                            bf16_lo_f32(raw.z), bf16_hi_f32(raw.z), bf16_lo_f32(raw.w), bf16_hi_f32(raw.w)};
        uint4 o;
        o.x = f32x2_to_f16x2_sat(v[0], v[4]);
        o.y = f32x2_to_f16x2_sat(v[1] * 0.0625f, v[5] * 0.0625f);
        o.z = f32x2_to_f16x2_sat(v[2], v[6]);
        o.w = f32x2_to_f16x2_sat(v[3] * 0.0625f, v[7] * 0.0625f);
        reinterpret_cast<uint4 *>(xs + (size_t)tok * p.k)[b] = o;
    }
    __syncthreads();
    for (int pair = warp; pair < mloc * groups; pair += PG_WARPS) { // slots of tokens past the end stay unwritten: never stored
        const int tok = pair % mloc, gi = pair / mloc;
        float s1 = 0.0f, s2 = 0.0f;
        const __half2 *src = reinterpret_cast<const __half2 *>(xs + (size_t)tok * p.k + (size_t)gi * p.group_size);
        for (int i = lane; i < (p.group_size >> 1); i += 32) { // half2 i: odd pairs carry the /16
            const float2 f = __half22float2(src[i]);
            const float t = f.x + f.y;
            s1 += t;
            s2 += (i & 1) ? 16.0f * t : t;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, o);
            s2 += __shfl_xor_sync(0xFFFFFFFFu, s2, o);
        }
        if (lane == 0) sums[gi * 8 + tok] = make_float2(1024.0f * s1, s2);
    }
    __syncthreads();

    // ---- main loop: warp w takes a contiguous run of quantization groups ------------------------------------------
    const int n0 = blockIdx.x * (16 * GQ_TILES);
    int col[GQ_TILES][2];
#pragma unroll
    for (int t = 0; t < GQ_TILES; t++) {
        col[t][0] = min(n0 + 16 * t + g, p.n - 1); // columns past the end read the last one; nothing of theirs is stored
        col[t][1] = min(n0 + 16 * t + g + 8, p.n - 1);
    }
    const int gp = (groups + PG_WARPS - 1) / PG_WARPS;
    const int g0 = warp * gp, g1 = min(groups, g0 + gp);
    const int steps = p.group_size >> 5; // 32 input rows (4 packed rows) per step
    const bool has_tok = g < mloc;
    uint32_t mask_lo, mask_hi, kmagic;
    asm volatile("mov.b32 %0, 0x000F000F;\n\tmov.b32 %1, 0x00F000F0;\n\tmov.b32 %2, 0x64006400;" : "=r"(mask_lo), "=r"(mask_hi), "=r"(kmagic));
    float tot[GQ_TILES][4];
#pragma unroll
    for (int t = 0; t < GQ_TILES; t++)
#pragma unroll
        for (int e = 0; e < 4; e++) tot[t][e] = 0.0f;
    // The packed words of a whole group (up to GQ_STEPS steps) are requested before the previous group is folded,
    // and a group's scales and zero points before its MMAs, so no global load is waited for where it is issued.
    constexpr int GQ_STEPS = 4; // steps (32 input rows each) held in registers: group sizes up to 128 in one go
    uint32_t wbuf[GQ_STEPS][GQ_TILES][2];
    auto load_steps = [&](int gi, int st0) {
        const size_t prow0 = (size_t)gi * (p.group_size >> 3) + c; // this lane's packed row in step 0
#pragma unroll
        for (int u = 0; u < GQ_STEPS; u++)
            if (st0 + u < steps) {
#pragma unroll
                for (int t = 0; t < GQ_TILES; t++) {
                    wbuf[u][t][0] = __ldcs(p.qweight + (prow0 + (size_t)4 * (st0 + u)) * p.n + col[t][0]);
                    wbuf[u][t][1] = __ldcs(p.qweight + (prow0 + (size_t)4 * (st0 + u)) * p.n + col[t][1]);
                }
            }
    };
    if (g0 < g1) load_steps(g0, 0);
    for (int gi = g0; gi < g1; gi++) {
        float acc[GQ_TILES][4];
#pragma unroll
        for (int t = 0; t < GQ_TILES; t++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[t][e] = 0.0f;
        float sc[GQ_TILES][2], zr[GQ_TILES][2];
#pragma unroll
        for (int t = 0; t < GQ_TILES; t++)
#pragma unroll
            for (int hrow = 0; hrow < 2; hrow++) {
                const int cc = col[t][hrow];
                sc[t][hrow] = load_as_f32(p.scales, p.scales_dtype, (size_t)gi * p.n + cc);
                if (p.sym || p.qzeros == nullptr) zr[t][hrow] = 8.0f;
                else zr[t][hrow] = (float)(((__ldg(p.qzeros + (size_t)gi * (p.n >> 3) + (cc >> 3)) >> (4 * (cc & 7))) & 0xFu) + 1u);
            }
        const uint4 *xrow = has_tok ? reinterpret_cast<const uint4 *>(xs + (size_t)g * p.k + (size_t)gi * p.group_size) + c : zeros;
        const int xinc = has_tok ? 4 : 0;
        for (int st0 = 0; st0 < steps; st0 += GQ_STEPS) {
            uint32_t w[GQ_STEPS][GQ_TILES][2];
#pragma unroll
            for (int u = 0; u < GQ_STEPS; u++)
#pragma unroll
                for (int t = 0; t < GQ_TILES; t++) { w[u][t][0] = wbuf[u][t][0]; w[u][t][1] = wbuf[u][t][1]; }
            // next chunk of this group, or the first chunk of the next group
            if (st0 + GQ_STEPS < steps) load_steps(gi, st0 + GQ_STEPS);
            else if (gi + 1 < g1) load_steps(gi + 1, 0);
#pragma unroll
            for (int u = 0; u < GQ_STEPS; u++) {
                if (st0 + u < steps) {
                    const uint4 xv = xrow[(size_t)(st0 + u) * xinc];
#pragma unroll
                    for (int t = 0; t < GQ_TILES; t++) {
                        const uint32_t h0 = w[u][t][0] >> 8, h1 = w[u][t][1] >> 8;
                        const uint32_t a[4] = {(w[u][t][0] & mask_lo) | kmagic, (w[u][t][1] & mask_lo) | kmagic,
                                               (w[u][t][0] & mask_hi) | kmagic, (w[u][t][1] & mask_hi) | kmagic};
                        const uint32_t b[4] = {(h0 & mask_lo) | kmagic, (h1 & mask_lo) | kmagic, (h0 & mask_hi) | kmagic, (h1 & mask_hi) | kmagic};
                        mma_f16_16816_gptq(acc[t], a, xv.x, xv.y);
                        mma_f16_16816_gptq(acc[t], b, xv.z, xv.w);
                    }
                }
            }
        }
        // fold the group: rows g and g + 8 of each tile, tokens 2 c and 2 c + 1
        const float2 sa = sums[gi * 8 + 2 * c], sb = sums[gi * 8 + 2 * c + 1];
#pragma unroll
        for (int t = 0; t < GQ_TILES; t++) {
#pragma unroll
            for (int hrow = 0; hrow < 2; hrow++) {
                tot[t][2 * hrow] = fmaf(sc[t][hrow], acc[t][2 * hrow] - sa.x - zr[t][hrow] * sa.y, tot[t][2 * hrow]);
                tot[t][2 * hrow + 1] = fmaf(sc[t][hrow], acc[t][2 * hrow + 1] - sb.x - zr[t][hrow] * sb.y, tot[t][2 * hrow + 1]);
            }
        }
    }
    // ---- the 8 warps meet in shared memory in warp order ---------------------------------------------------------
#pragma unroll
    for (int t = 0; t < GQ_TILES; t++)
#pragma unroll
        for (int e = 0; e < 4; e++) red[((warp * GQ_TILES + t) * 4 + e) * 32 + lane] = tot[t][e];
    __syncthreads();
    for (int o = tid; o < GQ_TILES * 4 * 32; o += PG_WARPS * 32) {
        const int l = o & 31, e = (o >> 5) & 3, t = o >> 7;
        const int og = l >> 2, oc = l & 3;
        const int tok = 2 * oc + (e & 1), ncol = n0 + 16 * t + og + 8 * (e >> 1);
        if (tok < mloc && ncol < p.n) {
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < PG_WARPS; w++) sum += red[((w * GQ_TILES + t) * 4 + e) * 32 + l];
            if (p.bias) sum += load_as_f32(p.bias, p.bias_dtype, ncol);
            store_as(p.y, p.y_dtype, (size_t)(p.y_row0 + tok) * p.n + ncol, sum);
        }
    }
}

template <typename Kern>
static int launch_packed(Kern kern, const char *name, PackedGemvParams p, int mt, int cols_per_cta, int red_cols, cudaStream_t st,
                         size_t smem_override = 0)
{
    const int groups = p.k / p.group_size;
    const size_t smem = smem_override ? smem_override
                                      : ((size_t)mt * p.k + (size_t)mt * groups + (size_t)PG_WARPS * mt * red_cols) * sizeof(float);
    // per (kernel, device): raise the dynamic shared-memory limit when a larger size is first needed
    static struct { const void *fn; int device; size_t bytes; } seen[64];
    static int nseen = 0;
    int device = 0;
    OXQ_CUDA(cudaGetDevice(&device));
    int slot = -1;
    for (int i = 0; i < nseen; i++)
        if (seen[i].fn == (const void *)kern && seen[i].device == device) slot = i;
    if (slot < 0 || seen[slot].bytes < smem) {
        OXQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (slot < 0 && nseen < 64) slot = nseen++;
        if (slot >= 0) { seen[slot].fn = (const void *)kern; seen[slot].device = device; seen[slot].bytes = smem; }
    }
    const int ctas = ceil_div(p.n, cols_per_cta);
    for (int row0 = 0; row0 < p.m; row0 += mt) {
        p.y_row0 = row0;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(ctas, 1, 1);
        cfg.blockDim = dim3(PG_WARPS * 32, 1, 1);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        cfg.attrs = attr;
        cfg.numAttrs = 0;
        allow_early_start(attr, cfg.numAttrs);
        cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
        if (e != cudaSuccess) return fail(OXQ_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e));
    }
    return OXQ_OK;
}

// Tokens per launch: as many (4, 2, 1) as keep the f32 copy of x under 160 KB of shared memory.
static int tokens_per_launch(int m, int k)
{
    int mt = PG_MAX_MT;
    while (mt > 1 && ((size_t)mt * k * 4 > 160 * 1024 || mt / 2 >= m)) mt /= 2;
    return mt;
}

} // namespace oxq

using namespace oxq;

static int check_common(const char *who, const void *x, int x_dtype, const void *qweight, const void *scales, int scales_dtype,
                        const void *bias, int bias_dtype, const void *y, int y_dtype, int m, int k, int n, int group_size)
{
    OXQ_REQUIRE(x && qweight && scales && y, OXQ_ERR_NULL, "%s: null pointer", who);
    OXQ_REQUIRE(x_dtype == OXQ_BF16, OXQ_ERR_UNSUPPORTED, "%s: activations must be bf16", who);
    OXQ_REQUIRE(valid_dtype(scales_dtype) && valid_dtype(y_dtype) && (!bias || valid_dtype(bias_dtype)), OXQ_ERR_UNSUPPORTED,
                "%s: unsupported dtype", who);
    OXQ_REQUIRE(m >= 1 && m <= 32, OXQ_ERR_BAD_SHAPE, "%s: m=%d outside 1..32 (use the GEMM entry)", who, m);
    OXQ_REQUIRE(k > 0 && n > 0 && group_size > 0, OXQ_ERR_BAD_SHAPE, "%s: non-positive size", who);
    OXQ_REQUIRE(k % group_size == 0, OXQ_ERR_BAD_SHAPE, "quant in_features (%d) not divisible by group size (%d)", k, group_size);
    OXQ_REQUIRE(aligned(x, 4) && aligned(qweight, 4), OXQ_ERR_BAD_ALIGN, "%s: x and qweight must be 4-byte aligned", who);
    OXQ_REQUIRE((size_t)k * 4 <= 160 * 1024, OXQ_ERR_UNSUPPORTED, "%s: in_features %d exceeds the staged-activation limit (40960)", who, k);
    return OXQ_OK;
}

OXQ_EXPORT int oxq_gptq_gemv(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros, const void *scales,
                             int scales_dtype, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
                             int group_size, int bits, int sym, void *stream)
{
    clear_error();
    int rc = check_common("oxq_gptq_gemv", x, x_dtype, qweight, scales, scales_dtype, bias, bias_dtype, y, y_dtype, m, k, n, group_size);
    if (rc) return rc;
    OXQ_REQUIRE(bits == 4 || bits == 8, OXQ_ERR_UNSUPPORTED, "dequantize_gptq: only 4/8-bit supported, got %d", bits);
    const int pf = 32 / bits;
    OXQ_REQUIRE(n % pf == 0 && k % pf == 0 && group_size % pf == 0 && k % 2 == 0, OXQ_ERR_BAD_SHAPE,
                "oxq_gptq_gemv: shape [%d, %d] / group size %d incompatible with pack factor %d", n, k, group_size, pf);
    PackedGemvParams p;
    p.x = (const __nv_bfloat16 *)x; p.qweight = qweight; p.qzeros = qzeros; p.scales = scales; p.bias = bias; p.y = y;
    p.scales_dtype = scales_dtype; p.bias_dtype = bias_dtype; p.y_dtype = y_dtype;
    p.m = m; p.k = k; p.n = n; p.group_size = group_size; p.sym = (sym != 0 || qzeros == nullptr) ? 1 : 0; p.y_row0 = 0;
    const int mt = tokens_per_launch(m, k);
    cudaStream_t st = (cudaStream_t)stream;
    if (bits == 4 && group_size % 32 == 0 && aligned(x, 16) && (size_t)k * 16 <= 160 * 1024 && !tuning_env("OXQ_GPTQ_SIMT")) {
        // tensor-core kernel, 8 tokens per launch
        const size_t smem = (size_t)(m < 8 ? m : 8) * k * 2 + 16 + (size_t)(k / group_size) * 8 * sizeof(float2) +
                            (size_t)PG_WARPS * GQ_TILES * 4 * 32 * sizeof(float);
        return launch_packed(gptq4_gemv_mma_kernel, "gptq4_gemv_mma_kernel", p, 8, 16 * GQ_TILES, 0, st, smem);
    }
    if (bits == 4) {
        if (mt == 4) return launch_packed(gptq_gemv_kernel<4, 4>, "gptq_gemv_kernel", p, 4, 32, 32, st);
        if (mt == 2) return launch_packed(gptq_gemv_kernel<4, 2>, "gptq_gemv_kernel", p, 2, 32, 32, st);
        return launch_packed(gptq_gemv_kernel<4, 1>, "gptq_gemv_kernel", p, 1, 32, 32, st);
    }
    if (mt == 4) return launch_packed(gptq_gemv_kernel<8, 4>, "gptq_gemv_kernel", p, 4, 32, 32, st);
    if (mt == 2) return launch_packed(gptq_gemv_kernel<8, 2>, "gptq_gemv_kernel", p, 2, 32, 32, st);
    return launch_packed(gptq_gemv_kernel<8, 1>, "gptq_gemv_kernel", p, 1, 32, 32, st);
}

OXQ_EXPORT int oxq_w8a16_gemv(const void *x, int x_dtype, const uint32_t *qweight, const uint32_t *qzeros, const void *scales,
                              int scales_dtype, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
                              int group_size, void *stream)
{
    clear_error();
    int rc = check_common("oxq_w8a16_gemv", x, x_dtype, qweight, scales, scales_dtype, bias, bias_dtype, y, y_dtype, m, k, n, group_size);
    if (rc) return rc;
    OXQ_REQUIRE(qzeros != nullptr, OXQ_ERR_NULL, "oxq_w8a16_gemv: qzeros missing");
    OXQ_REQUIRE(n % 4 == 0 && k % 2 == 0, OXQ_ERR_BAD_SHAPE, "W8A16 out_features (%d) not divisible by pack factor 4", n);
    PackedGemvParams p;
    p.x = (const __nv_bfloat16 *)x; p.qweight = qweight; p.qzeros = qzeros; p.scales = scales; p.bias = bias; p.y = y;
    p.scales_dtype = scales_dtype; p.bias_dtype = bias_dtype; p.y_dtype = y_dtype;
    p.m = m; p.k = k; p.n = n; p.group_size = group_size; p.sym = 0; p.y_row0 = 0;
    int mt = tokens_per_launch(m, k);
    if (mt > 2) mt = 2; // four columns per thread: two tokens keep the accumulators in registers
    cudaStream_t st = (cudaStream_t)stream;
    if (mt == 2) return launch_packed(w8a16_gemv_kernel<2>, "w8a16_gemv_kernel", p, 2, 128, 128, st);
    return launch_packed(w8a16_gemv_kernel<1>, "w8a16_gemv_kernel", p, 1, 128, 128, st);
}
