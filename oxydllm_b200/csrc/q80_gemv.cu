// GGUF Q8_0 ({f16 d; i8 qs[32]}, 34 bytes per 32 weights) decode GEMV (1 <= m <= 32), tuned variant.
//
// Same decomposition as the MXFP4 kernel: warps of a CTA = row tiles x k parts, a thread-block
// cluster adds further k slices, partial sums meet in (distributed) shared memory and are added in
// a fixed order; tokens beyond 8 per CTA go to neighbouring CTAs that stream the same weights.
// The four lanes that feed one row of the tensor-core operand work on the same block: lane c takes
// the block's weights k = 8c .. 8c+7 (two mma.sync.m16n8k16 steps per block). Blocks are 34 bytes,
// so a lane's 8 bytes start on a 2-byte boundary in every other block: it reads the three aligned
// words around them and funnel-shifts. int8 becomes f16 without a conversion: (b ^ 0x80) | 0x6400
// per byte is exactly 1024 + 128 + b, and the offset is taken out with the per-block sums of x when
// the block's accumulator is folded with its scale in f32:  y += d * (acc - 1152 * sum_x).
// x is staged as f16 (saturating) together with those sums. Rows must hold an even number of
// blocks (4-byte aligned rows).
#include <cooperative_groups.h>

#include <cstdio>
#include <cstdlib>

#include "oxq_common.cuh"

namespace oxq {

namespace cg = cooperative_groups;

struct Q80GemvParams {
    const __nv_bfloat16 *x;
    const uint8_t *blocks; // [n][k/32][34]
    const void *bias;
    void *y;
    int bias_dtype, y_dtype;
    int m, k, n;
    int row_tiles, k_warps; // warps of a CTA = row_tiles x k_warps
    int token_split;        // neighbouring CTAs that share their rows and take 8 tokens each (>= 1)
};

__device__ __forceinline__ void q80_mma_f16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Four int8 of one word -> two f16 pairs holding 1152 + b each.
__device__ __forceinline__ void i8x4_to_f16x4(uint32_t w, uint32_t &lo, uint32_t &hi)
{
    const uint32_t u = w ^ 0x80808080u;
    lo = __byte_perm(u, 0x64646464u, 0x5140); // (byte 0, 0x64), (byte 1, 0x64)
    hi = __byte_perm(u, 0x64646464u, 0x7362); // (byte 2, 0x64), (byte 3, 0x64)
}

// One lane's share of one block: the three aligned words around its 8 bytes, and the block's scale.
struct Q80Piece {
    uint32_t w0, w1, w2;
    unsigned short d;
};

__device__ __forceinline__ void q80_load(Q80Piece &q, const uint8_t *blk, int c)
{
    const uint8_t *p8 = blk + 2 + 8 * c;
    const uint32_t *al = reinterpret_cast<const uint32_t *>(reinterpret_cast<uintptr_t>(p8) & ~(uintptr_t)3);
    q.w0 = __ldg(al);
    q.w1 = __ldg(al + 1);
    // A piece that starts on a word boundary needs no third word (and the last block of the weight has
    // none after it); a shifted piece ends 2 bytes into a word whose other half is the next block's scale.
    q.w2 = (reinterpret_cast<uintptr_t>(p8) & 3) ? __ldg(al + 2) : 0u;
    q.d = __ldg(reinterpret_cast<const unsigned short *>(blk));
}

template <int D>
__global__ void __launch_bounds__(256, 3) q80_gemv_kernel(const Q80GemvParams p)
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
    const int nb = p.k >> 5;                        // blocks per row
    const int bl = nb / ks, b_cta = rank * bl;      // this CTA's blocks
    const int wb = bl / p.k_warps, b_off = kw * wb; // this warp's part of them
    const int kl = bl << 5, k_cta = b_cta << 5;
    const int xrow = kl + 8; // halves; 16 bytes of padding: the 16-byte reads of a quarter warp hit distinct banks
    __half *xs = reinterpret_cast<__half *>(smem);
    float *sx = reinterpret_cast<float *>(smem + (size_t)m_loc * xrow * 2); // [block][8]: sums of x per block and token
    float *red = sx + (size_t)bl * 8;                                       // [warp][4][lane]
    float *zeros = red + blockDim.x * 4; // 16 bytes of zeros: what lanes without a token read as x

    const int r0 = min(n0 + g, p.n - 1), r1 = min(n0 + g + 8, p.n - 1); // past-the-end rows re-read the last row
    const uint8_t *q0 = p.blocks + ((size_t)r0 * nb + b_cta + b_off) * 34;
    const uint8_t *q1 = p.blocks + ((size_t)r1 * nb + b_cta + b_off) * 34;

    Q80Piece buf0[D], buf1[D];
#pragma unroll
    for (int d = 0; d < D; d++)
        if (d < wb) {
            q80_load(buf0[d], q0 + 34 * d, c);
            q80_load(buf1[d], q1 + 34 * d, c);
        }

    // Stage the slice of x as f16 with the per-block sums of the staged values: eight neighbouring
    // threads hold one 32-element block. Rows without a token keep zero sums.
    if (tid < 4) zeros[tid] = 0.0f;
    for (int idx = tid; idx < bl * 8; idx += blockDim.x) sx[idx] = 0.0f;
    __syncthreads();
    pdl_wait(); // x may come from the kernel before this one; the first weights are already on their way
    for (int row = 0; row < m_loc; row++) {
        const uint2 *src = reinterpret_cast<const uint2 *>(p.x + (size_t)(m0 + row) * p.k + k_cta);
        uint2 *dst = reinterpret_cast<uint2 *>(xs + (size_t)row * xrow);
        // kl / 4 is a multiple of 8, so groups of 8 lanes are valid or not as a whole; the loop bound is
        // rounded up to whole warps because of the shuffles
        for (int q4 = tid; q4 < (((kl >> 2) + 31) & ~31); q4 += blockDim.x) {
            const bool valid = q4 < (kl >> 2);
            const uint2 raw = valid ? __ldg(src + q4) : make_uint2(0u, 0u);
            uint2 o;
            o.x = f32x2_to_f16x2_sat(bf16_lo_f32(raw.x), bf16_hi_f32(raw.x));
            o.y = f32x2_to_f16x2_sat(bf16_lo_f32(raw.y), bf16_hi_f32(raw.y));
            if (valid) dst[q4] = o;
            const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&o.x));
            const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&o.y)); // sum what the tensor cores will see
            float sum = (a.x + a.y) + (b.x + b.y);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
            if (valid && (lane & 7) == 0) sx[(q4 >> 3) * 8 + row] = sum;
        }
    }
    __syncthreads();

    // This lane's x for fragment column g: 8 halves per block, or the zeros (stride 0).
    const bool real = g < m_loc;
    const uint4 *xp = real ? reinterpret_cast<const uint4 *>(xs + (size_t)g * xrow + (b_off << 5) + 8 * c)
                           : reinterpret_cast<const uint4 *>(zeros);
    const int xstep = real ? 4 : 0; // 32 halves per block
    const float *sxp = sx + (size_t)b_off * 8 + 2 * c; // sums of tokens 2c, 2c+1 (the accumulator's columns)

    float tot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int b = 0; b < wb; b += D) {
#pragma unroll
        for (int d = 0; d < D; d++) {
            if (b + d < wb) {
                const Q80Piece p0 = buf0[d], p1 = buf1[d];
                if (b + D + d < wb) {
                    q80_load(buf0[d], q0 + 34 * (b + D + d), c);
                    q80_load(buf1[d], q1 + 34 * (b + D + d), c);
                }
                // even blocks of a row start 2 bytes after a word boundary, odd blocks on one
                const uint32_t sh0 = (uint32_t)(reinterpret_cast<uintptr_t>(q0 + 34 * (b + d) + 2) & 3) * 8;
                const uint32_t sh1 = (uint32_t)(reinterpret_cast<uintptr_t>(q1 + 34 * (b + d) + 2) & 3) * 8;
                const uint32_t w0a = __funnelshift_r(p0.w0, p0.w1, sh0), w0b = __funnelshift_r(p0.w1, p0.w2, sh0);
                const uint32_t w1a = __funnelshift_r(p1.w0, p1.w1, sh1), w1b = __funnelshift_r(p1.w1, p1.w2, sh1);
                uint32_t a_lo[4], a_hi[4]; // rows (g, g+8) x k (8c..8c+3) and (8c+4..8c+7)
                i8x4_to_f16x4(w0a, a_lo[0], a_lo[2]);
                i8x4_to_f16x4(w1a, a_lo[1], a_lo[3]);
                i8x4_to_f16x4(w0b, a_hi[0], a_hi[2]);
                i8x4_to_f16x4(w1b, a_hi[1], a_hi[3]);
                const uint4 xv = *xp;
                xp += xstep;
                const float2 sxv = *reinterpret_cast<const float2 *>(sxp + (size_t)(b + d) * 8);
                float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                const uint32_t b_lo[2] = {xv.x, xv.y}, b_hi[2] = {xv.z, xv.w};
                q80_mma_f16(acc, a_lo, b_lo);
                q80_mma_f16(acc, a_hi, b_hi);
                const float d0 = __half2float(__ushort_as_half(p0.d)), d1 = __half2float(__ushort_as_half(p1.d));
                tot[0] = fmaf(d0, fmaf(-1152.0f, sxv.x, acc[0]), tot[0]);
                tot[1] = fmaf(d0, fmaf(-1152.0f, sxv.y, acc[1]), tot[1]);
                tot[2] = fmaf(d1, fmaf(-1152.0f, sxv.x, acc[2]), tot[2]);
                tot[3] = fmaf(d1, fmaf(-1152.0f, sxv.y, acc[3]), tot[3]);
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

static size_t q80_smem(int m_cta, int kl, int warps)
{
    return (size_t)m_cta * (kl + 8) * 2 + (size_t)(kl / 32) * 8 * 4 + (size_t)warps * 4 * 32 * 4 + 16;
}

static int launch_q80(const Q80GemvParams &p, int ks, cudaStream_t st)
{
    const int nw = p.row_tiles * p.k_warps;
    const size_t smem = q80_smem(p.m < 8 ? p.m : 8, p.k / ks, nw);
    auto kern = q80_gemv_kernel<4>;
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
    cfg.numAttrs = ks > 1 ? 1 : 0; // no early start: measured 8 % slower with it on a 4096 x 4096 layer (14.4 -> 15.6 us)
    OXQ_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
    return OXQ_OK;
}

// Picks warps-per-CTA x cluster so that the k split divides the blocks of a row evenly.
static bool q80_pick(int m, int k, int &nrt, int &kw, int &ks)
{
    const int nb = k / 32;
    static const int few[][3] = {{1, 8, 1}, {2, 4, 1}, {1, 6, 1}, {1, 5, 1}, {2, 3, 1}, {2, 2, 1}, {1, 7, 1}, {2, 1, 1}, {1, 1, 1}};
    static const int many[][3] = {{8, 1, 2}, {4, 2, 2}, {4, 2, 1}, {2, 3, 1}, {8, 1, 1}};
    const int(*cand)[3] = m <= 8 ? few : many;
    const int count = m <= 8 ? 9 : 5;
    for (int t = 0; t < count; t++)
        if (nb % (cand[t][1] * cand[t][2]) == 0) { nrt = cand[t][0]; kw = cand[t][1]; ks = cand[t][2]; return true; }
    return false;
}

// True when the tuned kernel applies; otherwise the caller uses the generic row-format kernel.
bool q80_gemv_supported(int m, int k, const void *blocks)
{
    int a, b, c;
    return m <= 32 && k % 64 == 0 && (reinterpret_cast<uintptr_t>(blocks) & 3) == 0 && q80_pick(m, k, a, b, c) &&
           q80_smem(m < 8 ? m : 8, k, 8) <= 160 * 1024;
}

int q80_gemv(const void *x, const void *blocks, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
             cudaStream_t st)
{
    Q80GemvParams p;
    p.x = (const __nv_bfloat16 *)x; p.blocks = (const uint8_t *)blocks; p.bias = bias; p.y = y;
    p.bias_dtype = bias_dtype; p.y_dtype = y_dtype; p.m = m; p.k = k; p.n = n;
    int nrt = 2, kw = 4, ks = 1;
    q80_pick(m, k, nrt, kw, ks);
    if (const char *env = tuning_env("OXQ_Q80_GEMV_TUNE")) { // bench-harness knob: "row_tiles,k_warps,cluster"
        int a = 0, b = 0, cc = 0;
        if (sscanf(env, "%d,%d,%d", &a, &b, &cc) == 3 && a >= 1 && b >= 1 && a * b <= 8 && cc >= 1 && cc <= 8 &&
            (cc & (cc - 1)) == 0 && (k / 32) % (b * cc) == 0) {
            nrt = a; kw = b; ks = cc;
        }
    }
    p.row_tiles = nrt; p.k_warps = kw;
    p.token_split = ceil_div(m, 8); // 8 tokens per CTA; more on neighbouring CTAs
    return launch_q80(p, ks, st);
}

} // namespace oxq
