// FP8 E4M3 block-scaled decode GEMV (1 <= m <= 32), tuned variant.
//
// A thread-block cluster of KS CTAs owns 16 * NW output rows: CTA r of the cluster takes the r-th
// slice of k, warp w of every CTA the w-th 16-row tile, and the KS partial sums of an output are
// added in ascending k order by one thread of the cluster through distributed shared memory (no
// workspace, no atomics). Slicing k across CTAs rather than across the warps of one CTA means a
// CTA stages only its own slice of x, once for all its row tiles.
//
// Per 64-wide k chunk a lane streams 16 bytes of each of its two rows (lane/4 and lane/4 + 8)
// straight into registers -- bytes [16c, 16c+16), c = lane%4, so the four lanes of a row read 64
// contiguous bytes -- and uses them for four tensor-core steps; which k goes into which step is
// free as long as x follows, so no data is exchanged between lanes. E4M3 pairs are widened to f16
// pairs by the hardware conversion (exact) and contracted with mma.sync m16n8k16 (f16 x f16 ->
// f32); x is staged as f16 (saturated to +-65504). The f32 scale of a (row block, k block) is
// folded when the k block ends, so weights enter the tensor cores unrounded.
#include <cooperative_groups.h>
#include <cuda_fp8.h>

#include <cstdio>
#include <cstdlib>

#include "oxq_common.cuh"

namespace oxq {

struct Fp8GemvParams {
    const __nv_bfloat16 *x;
    const uint8_t *w;
    const float *scale_inv;
    const void *bias;
    void *y;
    int bias_dtype, y_dtype;
    int m, k, n;
    int s_in, block_out, block_in;
    int row_tiles, k_warps; // warps of a CTA = row_tiles x k_warps
    int token_split;        // neighbouring CTAs that share their rows and take 8*MT tokens each (>= 1)
};

namespace cg = cooperative_groups;

__device__ __forceinline__ void mma_f16_f8(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Four E4M3 bytes -> two f16 pairs (bytes 0,1 and bytes 2,3).
__device__ __forceinline__ void e4m3x4_to_f16x4(uint32_t v, uint32_t &lo2, uint32_t &hi2)
{
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, lo;\n\tcvt.rn.f16x2.e4m3x2 %1, hi;\n\t}"
        : "=r"(lo2), "=r"(hi2)
        : "r"(v));
}

// D = 64-wide k chunks in flight per warp.
template <int MT, int D>
__global__ void __launch_bounds__(256, MT == 1 ? 4 : MT == 2 ? 3 : 2) fp8_gemv_kernel(const Fp8GemvParams p)
{
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_launch_dependents();
    cg::cluster_group cluster = cg::this_cluster();
    const int nrt = p.row_tiles, ks = (int)gridDim.y, rank = (int)blockIdx.y; // cluster = the y extent of the grid
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    const int rt = warp % nrt, kw = warp / nrt;
    // Token tiles of one row group sit in neighbouring CTAs: they stream the same weights at the same
    // time, so all but the first reader hit in L2.
    const int zt = blockIdx.x % p.token_split, bx = blockIdx.x / p.token_split;
    const int m0 = zt * 8 * MT, m_loc = min(8 * MT, p.m - m0); // this CTA's tokens [m0, m0 + m_loc)
    const int n0 = (bx * nrt + rt) * 16;
    const int kl = p.k / ks, k_cta = rank * kl; // this CTA's k slice
    const int wl = kl / p.k_warps, k_off = kw * wl, k_beg = k_cta + k_off; // this warp's part of it
    const int xrow = kl + 8; // halves; 16 bytes of padding: the 16-byte reads of a quarter warp hit distinct banks
    __half *xs = reinterpret_cast<__half *>(smem);
    float *red = reinterpret_cast<float *>(smem + (size_t)m_loc * xrow * 2); // [warp][MT*4][lane]

    float *zeros = red + blockDim.x * MT * 4; // 32 bytes of zeros: what lanes without a token read as x

    const int chunks = wl >> 6; // a multiple of D
    const int r0 = min(n0 + g, p.n - 1), r1 = min(n0 + g + 8, p.n - 1); // past-the-end rows re-read the last row
    const uint8_t *row0 = p.w + (size_t)r0 * p.k + k_beg + 16 * c, *row1 = p.w + (size_t)r1 * p.k + k_beg + 16 * c;

    uint4 buf0[D], buf1[D];
#pragma unroll
    for (int d = 0; d < D; d++) {
        buf0[d] = __ldcs(reinterpret_cast<const uint4 *>(row0 + 64 * d));
        buf1[d] = __ldcs(reinterpret_cast<const uint4 *>(row1 + 64 * d));
    }
    // Scales of the first k block this warp meets; the next block's are fetched when a block ends.
    int si0 = 0, si1 = 0; // indices into the scale grid
    float s0 = 1.0f, s1 = 1.0f;
    if (p.scale_inv) {
        si0 = (r0 / p.block_out) * p.s_in + k_beg / p.block_in;
        si1 = (r1 / p.block_out) * p.s_in + k_beg / p.block_in;
        s0 = __ldg(p.scale_inv + si0);
        s1 = __ldg(p.scale_inv + si1);
    }

    if (tid < 8) zeros[tid] = 0.0f;
    pdl_wait(); // x may come from the kernel before this one; the first weights are already on their way
    for (int row = 0; row < m_loc; row++) {
        const uint2 *src = reinterpret_cast<const uint2 *>(p.x + (size_t)(m0 + row) * p.k + k_cta);
        uint2 *dst = reinterpret_cast<uint2 *>(xs + (size_t)row * xrow);
        for (int q4 = tid; q4 < (kl >> 2); q4 += blockDim.x) {
            const uint2 raw = __ldg(src + q4);
            dst[q4] = make_uint2(f32x2_to_f16x2_sat(bf16_lo_f32(raw.x), bf16_hi_f32(raw.x)),
                                 f32x2_to_f16x2_sat(bf16_lo_f32(raw.y), bf16_hi_f32(raw.y)));
        }
    }
    __syncthreads();

    // This lane's x for fragment column g of token tile mt: 16 halves per chunk, or the zeros (stride 0).
    const uint4 *xp[MT];
    int xstep[MT];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        const bool real = 8 * mt + g < m_loc;
        xp[mt] = real ? reinterpret_cast<const uint4 *>(xs + (size_t)(8 * mt + g) * xrow + k_off + 16 * c)
                      : reinterpret_cast<const uint4 *>(zeros);
        xstep[mt] = real ? 8 : 0; // 64 halves per chunk
    }

    float acc[MT][4], tot[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[mt][e] = tot[mt][e] = 0.0f;
    const int chunks_per_block = p.block_in >> 6; // k chunks that share one scale
    int left = chunks_per_block - ((k_beg >> 6) % chunks_per_block);

    for (int ch = 0; ch < chunks; ch += D) {
        const bool more = ch + D < chunks;
#pragma unroll
        for (int d = 0; d < D; d++) {
            const uint4 w0 = buf0[d], w1 = buf1[d];
            if (more) {
                buf0[d] = __ldcs(reinterpret_cast<const uint4 *>(row0 + 64 * (D + d)));
                buf1[d] = __ldcs(reinterpret_cast<const uint4 *>(row1 + 64 * (D + d)));
            }
            const uint32_t v0[4] = {w0.x, w0.y, w0.z, w0.w}, v1[4] = {w1.x, w1.y, w1.z, w1.w};
            if constexpr (MT == 1) { // convert step by step: fewer live registers
                const uint4 xa = xp[0][0], xb = xp[0][1];
                xp[0] += xstep[0];
                const uint32_t xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                for (int j = 0; j < 4; j++) { // step j: bytes 4j..4j+3 of the 16
                    uint32_t a[4];
                    e4m3x4_to_f16x4(v0[j], a[0], a[2]);
                    e4m3x4_to_f16x4(v1[j], a[1], a[3]);
                    const uint32_t b[2] = {xv[2 * j], xv[2 * j + 1]};
                    mma_f16_f8(acc[0], a, b);
                }
            } else {
                uint32_t a[4][4]; // a[j]: the A fragment of step j (bytes 4j..4j+3 of the 16)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    e4m3x4_to_f16x4(v0[j], a[j][0], a[j][2]);
                    e4m3x4_to_f16x4(v1[j], a[j][1], a[j][3]);
                }
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    const uint4 xa = xp[mt][0], xb = xp[mt][1];
                    xp[mt] += xstep[mt];
                    const uint32_t xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const uint32_t b[2] = {xv[2 * j], xv[2 * j + 1]};
                        mma_f16_f8(acc[mt], a[j], b);
                    }
                }
            }
            if (--left == 0) { // end of a scale block along k
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    tot[mt][0] = fmaf(s0, acc[mt][0], tot[mt][0]);
                    tot[mt][1] = fmaf(s0, acc[mt][1], tot[mt][1]);
                    tot[mt][2] = fmaf(s1, acc[mt][2], tot[mt][2]);
                    tot[mt][3] = fmaf(s1, acc[mt][3], tot[mt][3]);
                    acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.0f;
                }
                left = chunks_per_block;
                if (p.scale_inv && (more || d + 1 < D)) { // another block follows within this warp's range
                    s0 = __ldg(p.scale_inv + ++si0);
                    s1 = __ldg(p.scale_inv + ++si1);
                }
            }
        }
        row0 += 64 * D;
        row1 += 64 * D;
    }
    if (left != chunks_per_block) { // the range ended inside a scale block
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            tot[mt][0] = fmaf(s0, acc[mt][0], tot[mt][0]);
            tot[mt][1] = fmaf(s0, acc[mt][1], tot[mt][1]);
            tot[mt][2] = fmaf(s1, acc[mt][2], tot[mt][2]);
            tot[mt][3] = fmaf(s1, acc[mt][3], tot[mt][3]);
        }
    }

#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int e = 0; e < 4; e++) red[(warp * MT * 4 + mt * 4 + e) * 32 + lane] = tot[mt][e];
    if (ks > 1) cluster.sync(); else __syncthreads();

    // Every (row tile, accumulator slot, lane) is summed by one thread of the cluster, in ascending k.
    const int slots = nrt * MT * 4 * 32;
    for (int o = rank * blockDim.x + tid; o < slots; o += ks * blockDim.x) {
        const int ln = o & 31, e = (o >> 5) & 3, mt = (o >> 7) % MT, wt = (o >> 7) / MT;
        const int nn = (bx * nrt + wt) * 16 + (ln >> 2) + 8 * (e >> 1), row = 8 * mt + 2 * (ln & 3) + (e & 1);
        if (nn < p.n && row < m_loc) {
            float sum = 0.0f;
            for (int q = 0; q < ks; q++) {
                const float *src = ks > 1 ? cluster.map_shared_rank(red, q) : red;
                for (int w = 0; w < p.k_warps; w++) sum += src[((w * nrt + wt) * MT * 4 + mt * 4 + e) * 32 + ln];
            }
            if (p.bias) sum += load_as_f32(p.bias, p.bias_dtype, nn);
            store_as(p.y, p.y_dtype, (size_t)(m0 + row) * p.n + nn, sum);
        }
    }
    if (ks > 1) cluster.sync(); // nobody leaves while a peer may still read its shared memory
}

template <int MT, int D> static int launch_fp8(const Fp8GemvParams &p, int ks, cudaStream_t st)
{
    const int nw = p.row_tiles * p.k_warps;
    const int m_cta = p.m < 8 * MT ? p.m : 8 * MT;
    const size_t smem = (size_t)m_cta * (p.k / ks + 8) * 2 + (size_t)nw * MT * 4 * 32 * 4 + 32;
    auto kern = fp8_gemv_kernel<MT, D>;
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

// True when the tuned kernel applies; otherwise the caller uses the generic row-format kernel.
bool fp8_gemv_fast_supported(int m, int k, int block_in, const void *w)
{
    return m <= 32 && k % 512 == 0 && block_in % 64 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
           (size_t)m * (k / (m > 16 ? 4 : 1) + 8) * 2 <= 160 * 1024;
}

int fp8_gemv_fast(const void *x, const uint8_t *w, const float *scale_inv, int s_in, int block_out, int block_in,
                  const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n, cudaStream_t st)
{
    Fp8GemvParams p;
    p.x = (const __nv_bfloat16 *)x; p.w = w; p.scale_inv = scale_inv; p.bias = bias; p.y = y;
    p.bias_dtype = bias_dtype; p.y_dtype = y_dtype; p.m = m; p.k = k; p.n = n;
    p.s_in = s_in; p.block_out = block_out; p.block_in = block_in;
    // Warps of a CTA = row tiles x k parts, cluster = further k slices (measured on a 14336 x 4096 layer).
    // Few tokens: small row groups, so that every CTA of the grid is resident at once. More tokens:
    // more row tiles per CTA, which share the staged x.
    // mtc = 8-token tiles per CTA; more tokens than 8 * mtc go to neighbouring CTAs of the same rows.
    // Measured: 9..16 tokens run faster as two 8-token CTAs side by side than as one 16-token CTA.
    int nrt = 2, kw = 4, ks = 1, d = 2, mtc = m <= 16 ? 1 : 4;
    if (m > 16) { nrt = 8; kw = 1; ks = 4; }
    else if (m > 8) { nrt = 8; kw = 1; ks = 2; }
    else if (m > 2) { nrt = 4; kw = 2; ks = 2; }
    if (const char *env = tuning_env("OXQ_FP8_GEMV_TUNE")) { // bench-harness knob: "row_tiles,k_warps,cluster,depth[,token tiles per CTA]"
        int a = 0, b = 0, cc = 0, dd = 0, mm = 0;
        const int got = sscanf(env, "%d,%d,%d,%d,%d", &a, &b, &cc, &dd, &mm);
        if (got >= 4 && a >= 1 && b >= 1 && a * b <= 8 && cc >= 1 && cc <= 8 && (cc & (cc - 1)) == 0 &&
            (dd == 1 || dd == 2 || dd == 4) && k % (b * cc * 64 * dd) == 0) {
            nrt = a; kw = b; ks = cc; d = dd;
            if (got >= 5 && (mm == 1 || mm == 2 || mm == 4)) mtc = mm;
        }
    }
    p.row_tiles = nrt; p.k_warps = kw;
    p.token_split = ceil_div(m, 8 * mtc);
    if (mtc == 1) return d == 1 ? launch_fp8<1, 1>(p, ks, st) : d == 2 ? launch_fp8<1, 2>(p, ks, st) : launch_fp8<1, 4>(p, ks, st);
    if (mtc == 2) return d == 1 ? launch_fp8<2, 1>(p, ks, st) : launch_fp8<2, 2>(p, ks, st);
    return launch_fp8<4, 2>(p, ks, st);
}

} // namespace oxq
