// GGUF Q6_K decode GEMV (1 <= m <= 32), tuned variant.
//
// Q6_K super-block (210 B / 256 weights): u8 ql[128] (low 4 bits), u8 qh[64] (high 2 bits), i8
// scales[16] (one per 16 weights), f16 d. For half h (0, 1), quad q (0..3) and l (0..31), weight
// 128h + 32q + l has low bits in ql[64h + 32(q&1) + l] (low nibble for q < 2, high nibble else),
// high bits in qh[32h + l] >> 2q, scale scales[8h + 2q + l/16]; w = d * scale * (6-bit - 32).
//
// Same decomposition as the other row-format kernels: warps of a CTA = row tiles x k parts, a
// thread-block cluster adds further k slices, partial sums meet in (distributed) shared memory and
// are added in a fixed order; tokens beyond 8 per CTA go to neighbouring CTAs that stream the same
// weights. One mma.sync.m16n8k16 step covers the 16 consecutive weights that share a scale: lane c
// of the quad that feeds one operand row takes l = 16s + 4c .. 16s + 4c + 3, i.e. one 32-bit word of
// ql per quad parity and one of qh per (h, s), which serve the four quads. The 6-bit values are
// assembled four at a time with shifts and lop3, become f16 by byte permute (0x6400 | v = 1024 + v)
// and the offset 1024 + 32 comes out in f32 with the sums of x over each 16 weights when the step
// is folded with d * scale. Super-blocks are 210 bytes, so every other one starts 2 bytes off a
// word boundary: its words are read as two halfwords. Rows must hold an even number of
// super-blocks (4-byte aligned rows).
#include <cooperative_groups.h>

#include <cstdio>
#include <cstdlib>

#include "oxq_common.cuh"

namespace oxq {

namespace cg = cooperative_groups;

struct Q6kGemvParams {
    const __nv_bfloat16 *x;
    const uint8_t *blocks; // [n][k/256][210]
    const void *bias;
    void *y;
    int bias_dtype, y_dtype;
    int m, k, n;
    int row_tiles, k_warps; // warps of a CTA = row_tiles x k_warps
    int token_split;        // neighbouring CTAs that share their rows and take 8 tokens each (>= 1)
};

__device__ __forceinline__ void q6k_mma_f16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// 32-bit word at a 2-byte aligned address (warp-uniform alignment).
__device__ __forceinline__ uint32_t q6k_ld32(const uint8_t *p)
{
    if (reinterpret_cast<uintptr_t>(p) & 2) {
        const unsigned short *h = reinterpret_cast<const unsigned short *>(p);
        return (uint32_t)__ldg(h) | ((uint32_t)__ldg(h + 1) << 16);
    }
    return __ldg(reinterpret_cast<const uint32_t *>(p));
}

// The words of one (half h, sixteen s) combination for one row: ql of even quads, ql of odd quads, qh.
struct Q6kCombo {
    uint32_t ql_even, ql_odd, qh;
};

__device__ __forceinline__ void q6k_load_combo(Q6kCombo &w, const uint8_t *blk, int combo, int c)
{
    const int h = combo >> 1, s = combo & 1;
    const uint8_t *ql = blk + 64 * h + 16 * s + 4 * c;
    w.ql_even = q6k_ld32(ql);
    w.ql_odd = q6k_ld32(ql + 32);
    w.qh = q6k_ld32(blk + 128 + 32 * h + 16 * s + 4 * c);
}

// Exact float of a signed byte without the conversion unit.
__device__ __forceinline__ float q6k_i8_to_f32(uint32_t byte)
{
    return __uint_as_float(0x4B000000u | (byte ^ 0x80u)) - 8388736.0f; // 2^23 + 128
}

__global__ void __launch_bounds__(256, 3) q6k_gemv_kernel(const Q6kGemvParams p)
{
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_launch_dependents();
    cg::cluster_group cluster = cg::this_cluster();
    const int nrt = p.row_tiles, ks = (int)gridDim.y, rank = (int)blockIdx.y; // cluster = the y extent of the grid
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    const int rt = warp % nrt, kw = warp / nrt;
    const int zt = blockIdx.x % p.token_split, bx = blockIdx.x / p.token_split;
    const int m0 = zt * 8, m_loc = min(8, p.m - m0); // this CTA's tokens [m0, m0 + m_loc)
    const int n0 = (bx * nrt + rt) * 16;
    const int nsb = p.k >> 8;                        // super-blocks per row
    const int sl = nsb / ks, sb_cta = rank * sl;     // this CTA's super-blocks
    const int wsb = sl / p.k_warps, sb_off = kw * wsb; // this warp's part of them
    const int kl = sl << 8, k_cta = sb_cta << 8;
    const int xrow = kl + 16; // halves; 32 bytes of padding: the 8-byte fragment reads of a half warp hit distinct banks
    __half *xs = reinterpret_cast<__half *>(smem);
    float *sx = reinterpret_cast<float *>(smem + (size_t)m_loc * xrow * 2); // [kl/16][8]: sums of x per 16 k and token
    float *red = sx + (size_t)(kl >> 4) * 8;                                // [warp][4][lane]
    float *zeros = red + blockDim.x * 4; // 16 bytes of zeros: what lanes without a token read as x

    const int r0 = min(n0 + g, p.n - 1), r1 = min(n0 + g + 8, p.n - 1); // past-the-end rows re-read the last row
    const uint8_t *q0 = p.blocks + ((size_t)r0 * nsb + sb_cta + sb_off) * 210;
    const uint8_t *q1 = p.blocks + ((size_t)r1 * nsb + sb_cta + sb_off) * 210;

    Q6kCombo cur0, cur1;
    if (wsb > 0) {
        q6k_load_combo(cur0, q0, 0, c);
        q6k_load_combo(cur1, q1, 0, c);
    }

    // Stage the slice of x as f16 with the sums of the staged values over each 16 k: four neighbouring
    // threads hold one. Rows without a token keep zero sums.
    if (tid < 4) zeros[tid] = 0.0f;
    for (int idx = tid; idx < (kl >> 4) * 8; idx += blockDim.x) sx[idx] = 0.0f;
    __syncthreads();
    pdl_wait(); // x may come from the kernel before this one; the first weights are already on their way
    for (int row = 0; row < m_loc; row++) {
        const uint2 *src = reinterpret_cast<const uint2 *>(p.x + (size_t)(m0 + row) * p.k + k_cta);
        uint2 *dst = reinterpret_cast<uint2 *>(xs + (size_t)row * xrow);
        for (int q4 = tid; q4 < (kl >> 2); q4 += blockDim.x) { // kl / 4 is a multiple of 64: whole warps
            const uint2 raw = __ldg(src + q4);
            uint2 o;
            o.x = f32x2_to_f16x2_sat(bf16_lo_f32(raw.x), bf16_hi_f32(raw.x));
            o.y = f32x2_to_f16x2_sat(bf16_lo_f32(raw.y), bf16_hi_f32(raw.y));
            dst[q4] = o;
            const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&o.x));
            const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&o.y)); // sum what the tensor cores will see
            float sum = (a.x + a.y) + (b.x + b.y);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
            if ((lane & 3) == 0) sx[(q4 >> 2) * 8 + row] = sum;
        }
    }
    __syncthreads();

    // This lane's x for fragment column g (four halves per step), or the zeros (stride 0).
    const bool real = g < m_loc;
    const __half *xbase = real ? xs + (size_t)g * xrow + (sb_off << 8) + 4 * c : reinterpret_cast<const __half *>(zeros);
    const int xmul = real ? 1 : 0;
    const float *sxb = sx + (size_t)(sb_off << 4) * 8 + 2 * c; // sums of tokens 2c, 2c+1 (the accumulator's columns)

    float tot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int sb = 0; sb < wsb; sb++) {
        const uint8_t *blk0 = q0 + (size_t)sb * 210, *blk1 = q1 + (size_t)sb * 210;
        uint32_t sc0[4], sc1[4]; // the 16 signed scales of each row's super-block
#pragma unroll
        for (int i = 0; i < 4; i++) {
            sc0[i] = q6k_ld32(blk0 + 192 + 4 * i);
            sc1[i] = q6k_ld32(blk1 + 192 + 4 * i);
        }
        const float d0 = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short *>(blk0 + 208))));
        const float d1 = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short *>(blk1 + 208))));
#pragma unroll
        for (int combo = 0; combo < 4; combo++) {
            const Q6kCombo w0 = cur0, w1 = cur1;
            if (combo < 3) { // next combination on its way while this one is consumed
                q6k_load_combo(cur0, blk0, combo + 1, c);
                q6k_load_combo(cur1, blk1, combo + 1, c);
            } else if (sb + 1 < wsb) {
                q6k_load_combo(cur0, blk0 + 210, 0, c);
                q6k_load_combo(cur1, blk1 + 210, 0, c);
            }
            const int h = combo >> 1, s = combo & 1;
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const uint32_t l0 = (q & 1) ? w0.ql_odd : w0.ql_even, l1 = (q & 1) ? w1.ql_odd : w1.ql_even;
                const uint32_t v0 = ((q < 2 ? l0 : l0 >> 4) & 0x0F0F0F0Fu) | (((w0.qh >> (2 * q)) & 0x03030303u) << 4);
                const uint32_t v1 = ((q < 2 ? l1 : l1 >> 4) & 0x0F0F0F0Fu) | (((w1.qh >> (2 * q)) & 0x03030303u) << 4);
                // bytes of v = weights k0 + 4c .. k0 + 4c + 3 (0..63 each) -> f16 pairs 1024 + v
                const uint32_t a[4] = {__byte_perm(v0, 0x64646464u, 0x5140), __byte_perm(v1, 0x64646464u, 0x5140),
                                       __byte_perm(v0, 0x64646464u, 0x7362), __byte_perm(v1, 0x64646464u, 0x7362)};
                const int k0 = (sb << 8) + 128 * h + 32 * q + 16 * s; // first k of the step within the warp's range
                const uint2 xv = *reinterpret_cast<const uint2 *>(xbase + xmul * k0);
                const float2 sxv = *reinterpret_cast<const float2 *>(sxb + (size_t)(k0 >> 4) * 8);
                float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                const uint32_t b[2] = {xv.x, xv.y};
                q6k_mma_f16(acc, a, b);
                const int si = 8 * h + 2 * q + s; // scale index
                const float f0 = d0 * q6k_i8_to_f32((sc0[si >> 2] >> (8 * (si & 3))) & 0xFFu);
                const float f1 = d1 * q6k_i8_to_f32((sc1[si >> 2] >> (8 * (si & 3))) & 0xFFu);
                tot[0] = fmaf(f0, fmaf(-1056.0f, sxv.x, acc[0]), tot[0]);
                tot[1] = fmaf(f0, fmaf(-1056.0f, sxv.y, acc[1]), tot[1]);
                tot[2] = fmaf(f1, fmaf(-1056.0f, sxv.x, acc[2]), tot[2]);
                tot[3] = fmaf(f1, fmaf(-1056.0f, sxv.y, acc[3]), tot[3]);
            }
        }
    }

#pragma unroll
    for (int e = 0; e < 4; e++) red[(warp * 4 + e) * 32 + lane] = tot[e];
    if (ks > 1) cluster.sync(); else __syncthreads();

    // Every (row tile, accumulator slot, lane) is summed by one thread of the cluster, in ascending k.
    const int slots = nrt * 4 * 32;
    for (int o = rank * blockDim.x + tid; o < slots; o += ks * blockDim.x) {
        const int ln = o & 31, e = (o >> 5) & 3, wt = o >> 7;
        const int nn = (bx * nrt + wt) * 16 + (ln >> 2) + 8 * (e >> 1), row = 2 * (ln & 3) + (e & 1);
        if (nn < p.n && row < m_loc) {
            float sum = 0.0f;
            for (int q = 0; q < ks; q++) {
                const float *src = ks > 1 ? cluster.map_shared_rank(red, q) : red;
                for (int w = 0; w < p.k_warps; w++) sum += src[((w * nrt + wt) * 4 + e) * 32 + ln];
            }
            if (p.bias) sum += load_as_f32(p.bias, p.bias_dtype, nn);
            store_as(p.y, p.y_dtype, (size_t)(m0 + row) * p.n + nn, sum);
        }
    }
    if (ks > 1) cluster.sync(); // nobody leaves while a peer may still read its shared memory
}

static size_t q6k_smem(int m_cta, int kl, int warps)
{
    return (size_t)m_cta * (kl + 16) * 2 + (size_t)(kl / 16) * 8 * 4 + (size_t)warps * 4 * 32 * 4 + 16;
}

static int launch_q6k(const Q6kGemvParams &p, int ks, cudaStream_t st)
{
    const int nw = p.row_tiles * p.k_warps;
    const size_t smem = q6k_smem(p.m < 8 ? p.m : 8, p.k / ks, nw);
    auto kern = q6k_gemv_kernel;
    static size_t configured[64] = {};
    int device = 0;
    OXQ_CUDA(cudaGetDevice(&device));
    if (device >= 64 || configured[device] < smem) {
        OXQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (device < 64) configured[device] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ceil_div(p.n, 16 * p.row_tiles) * p.token_split, ks, 1);
    cfg.blockDim = dim3(nw * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = ks;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ks > 1 ? 1 : 0;
    allow_early_start(attr, cfg.numAttrs);
    OXQ_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
    return OXQ_OK;
}

// Picks warps-per-CTA x cluster so that the k split divides the super-blocks of a row evenly.
static bool q6k_pick(int m, int k, int &nrt, int &kw, int &ks)
{
    const int nsb = k / 256;
    static const int few[][3] = {{1, 8, 1}, {2, 4, 1}, {1, 6, 1}, {1, 5, 1}, {2, 3, 1}, {2, 2, 1}, {1, 7, 1}, {2, 1, 1}, {1, 1, 1}};
    static const int many[][3] = {{2, 4, 1}, {4, 2, 1}, {2, 3, 1}, {8, 1, 2}, {8, 1, 1}};
    const int(*cand)[3] = m <= 8 ? few : many;
    const int count = m <= 8 ? 9 : 5;
    for (int t = 0; t < count; t++)
        if (nsb % (cand[t][1] * cand[t][2]) == 0) { nrt = cand[t][0]; kw = cand[t][1]; ks = cand[t][2]; return true; }
    return false;
}

// True when the tuned kernel applies; otherwise the caller uses the generic row-format kernel.
bool q6k_gemv_supported(int m, int k, const void *blocks)
{
    int a, b, c;
    return m <= 32 && k % 512 == 0 && (reinterpret_cast<uintptr_t>(blocks) & 3) == 0 && q6k_pick(m, k, a, b, c) &&
           q6k_smem(m < 8 ? m : 8, k, 8) <= 160 * 1024;
}

int q6k_gemv(const void *x, const void *blocks, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
             cudaStream_t st)
{
    Q6kGemvParams p;
    p.x = (const __nv_bfloat16 *)x; p.blocks = (const uint8_t *)blocks; p.bias = bias; p.y = y;
    p.bias_dtype = bias_dtype; p.y_dtype = y_dtype; p.m = m; p.k = k; p.n = n;
    int nrt = 2, kw = 4, ks = 1;
    q6k_pick(m, k, nrt, kw, ks);
    if (const char *env = tuning_env("OXQ_Q6K_GEMV_TUNE")) { // bench-harness knob: "row_tiles,k_warps,cluster"
        int a = 0, b = 0, cc = 0;
        if (sscanf(env, "%d,%d,%d", &a, &b, &cc) == 3 && a >= 1 && b >= 1 && a * b <= 8 && cc >= 1 && cc <= 8 &&
            (cc & (cc - 1)) == 0 && (k / 256) % (b * cc) == 0) {
            nrt = a; kw = b; ks = cc;
        }
    }
    p.row_tiles = nrt; p.k_warps = kw;
    p.token_split = ceil_div(m, 8); // 8 tokens per CTA; more on neighbouring CTAs
    return launch_q6k(p, ks, st);
}

} // namespace oxq
