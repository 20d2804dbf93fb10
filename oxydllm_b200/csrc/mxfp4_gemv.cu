// MXFP4 (E2M1 codes, one E8M0 scale per 32 weights) decode GEMV (1 <= m <= 32), tuned variant.
//
// Same decomposition as the FP8 kernel: warps of a CTA = row tiles x k parts, a thread-block cluster
// adds further k slices, partial sums meet in (distributed) shared memory and are added in a fixed
// order; tokens beyond 8 per CTA go to neighbouring CTAs that stream the same weights.
// A quantization block is 16 bytes = 32 consecutive k of one row with its own power-of-two scale,
// so the four lanes that feed one row of the tensor-core operand must all work on the SAME block:
// lane c of a quad takes bytes [4c, 4c+4) of the block (k 8c .. 8c+7), which gives two
// mma.sync.m16n8k16 steps per block, and the block's scale is applied in f32 when the block's
// accumulator is folded into the running total. E2M1 pairs widen to f16 pairs in hardware
// (cvt.rn.f16x2.e2m1x2, exact); x is staged as f16 (saturating). The 4-byte loads of one block
// fill half a 32-byte sector; the other half belongs to the next block of the same row, which the
// same lanes read next, so the loads go through L1 (ld.global.nc) instead of streaming past it.
#include <cooperative_groups.h>

#include <cstdio>
#include <cstdlib>

#include "oxq_common.cuh"

namespace oxq {

namespace cg = cooperative_groups;

struct Mx4GemvParams {
    const __nv_bfloat16 *x;
    const uint8_t *blocks; // [n][k/32][16]
    const uint8_t *scales; // [n][k/32]
    const void *bias;
    void *y;
    int bias_dtype, y_dtype;
    int m, k, n;
    int row_tiles, k_warps; // warps of a CTA = row_tiles x k_warps
    int token_split;        // neighbouring CTAs that share their rows and take 8*MT tokens each (>= 1)
    // Batched single-token mode (MoE decode): grid z = (token, slot) pair; the pair's expert id selects
    // the weight, bias and scale slices, its token (pair / x_div) the x row, and y row = pair.
    const int *pair_expert; // null: plain mode
    int x_div, e_lo, e_hi;
};

__device__ __forceinline__ void mx4_mma_f16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Four bytes of E2M1 pairs -> four f16 pairs (low nibble in the low half).
__device__ __forceinline__ void e2m1x8_to_f16x8(uint32_t w, uint32_t (&h)[4])
{
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\tcvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
        : "r"(w));
}

// D = blocks in flight per warp.
template <int MT, int D>
__global__ void __launch_bounds__(256, MT == 1 ? 4 : MT == 2 ? 3 : 2) mxfp4_gemv_kernel(const Mx4GemvParams p)
{
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_launch_dependents();
    if (p.pair_expert) pdl_wait(); // the routing table comes from the kernel before this one
    cg::cluster_group cluster = cg::this_cluster();
    const int nrt = p.row_tiles, ks = (int)gridDim.y, rank = (int)blockIdx.y; // cluster = the y extent of the grid
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    const int rt = warp % nrt, kw = warp / nrt;
    const int zt = blockIdx.x % p.token_split, bx = blockIdx.x / p.token_split;
    const int m0 = zt * 8 * MT, m_loc = min(8 * MT, p.m - m0); // this CTA's tokens [m0, m0 + m_loc)
    const int n0 = (bx * nrt + rt) * 16;
    const int nb = p.k >> 5;                       // blocks per row
    const uint8_t *blocks = p.blocks, *scales = p.scales;
    const __nv_bfloat16 *xin = p.x;
    size_t bias_off = 0, y_off = 0;
    if (p.pair_expert) {
        const int pair = blockIdx.z, e = p.pair_expert[pair];
        if (e < p.e_lo || e >= p.e_hi) return; // the same for every CTA of the cluster: nobody waits for this one
        blocks += (size_t)e * p.n * nb * 16;
        scales += (size_t)e * p.n * nb;
        xin += (size_t)(pair / p.x_div) * p.k;
        bias_off = (size_t)e * p.n;
        y_off = (size_t)pair * p.n;
    }
    const int bl = nb / ks, b_cta = rank * bl;     // this CTA's blocks
    const int wb = bl / p.k_warps, b_off = kw * wb; // this warp's part of them
    const int kl = bl << 5, k_cta = b_cta << 5;
    const int xrow = kl + 8; // halves; 16 bytes of padding: the 16-byte reads of a quarter warp hit distinct banks
    __half *xs = reinterpret_cast<__half *>(smem);
    float *red = reinterpret_cast<float *>(smem + (size_t)m_loc * xrow * 2); // [warp][MT*4][lane]
    float *zeros = red + blockDim.x * MT * 4; // 16 bytes of zeros: what lanes without a token read as x

    const int r0 = min(n0 + g, p.n - 1), r1 = min(n0 + g + 8, p.n - 1); // past-the-end rows re-read the last row
    const uint32_t *q0 = reinterpret_cast<const uint32_t *>(blocks + ((size_t)r0 * nb + b_cta + b_off) * 16) + c;
    const uint32_t *q1 = reinterpret_cast<const uint32_t *>(blocks + ((size_t)r1 * nb + b_cta + b_off) * 16) + c;
    const uint8_t *s0p = scales + (size_t)r0 * nb + b_cta + b_off;
    const uint8_t *s1p = scales + (size_t)r1 * nb + b_cta + b_off;

    uint32_t buf0[D], buf1[D], sb0[D], sb1[D];
#pragma unroll
    for (int d = 0; d < D; d++)
        if (d < wb) {
            buf0[d] = __ldg(q0 + 4 * d);
            buf1[d] = __ldg(q1 + 4 * d);
            sb0[d] = __ldg(s0p + d);
            sb1[d] = __ldg(s1p + d);
        }

    if (tid < 4) zeros[tid] = 0.0f;
    if (!p.pair_expert) pdl_wait(); // x may come from the kernel before this one; the first weights are already on their way
    for (int row = 0; row < m_loc; row++) {
        const uint2 *src = reinterpret_cast<const uint2 *>(xin + (size_t)(m0 + row) * p.k + k_cta);
        uint2 *dst = reinterpret_cast<uint2 *>(xs + (size_t)row * xrow);
        for (int q4 = tid; q4 < (kl >> 2); q4 += blockDim.x) {
            const uint2 raw = __ldg(src + q4);
            dst[q4] = make_uint2(f32x2_to_f16x2_sat(bf16_lo_f32(raw.x), bf16_hi_f32(raw.x)),
                                 f32x2_to_f16x2_sat(bf16_lo_f32(raw.y), bf16_hi_f32(raw.y)));
        }
    }
    __syncthreads();

    // This lane's x for fragment column g of token tile mt: 8 halves per block, or the zeros (stride 0).
    const uint4 *xp[MT];
    int xstep[MT];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        const bool real = 8 * mt + g < m_loc;
        xp[mt] = real ? reinterpret_cast<const uint4 *>(xs + (size_t)(8 * mt + g) * xrow + (b_off << 5) + 8 * c)
                      : reinterpret_cast<const uint4 *>(zeros);
        xstep[mt] = real ? 4 : 0; // 32 halves per block
    }

    float tot[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) tot[mt][0] = tot[mt][1] = tot[mt][2] = tot[mt][3] = 0.0f;

    for (int b = 0; b < wb; b += D) {
#pragma unroll
        for (int d = 0; d < D; d++) {
            if (b + d < wb) {
                const uint32_t w0 = buf0[d], w1 = buf1[d];
                const float s0 = e8m0_to_f32(sb0[d]), s1 = e8m0_to_f32(sb1[d]);
                if (b + D + d < wb) {
                    buf0[d] = __ldg(q0 + 4 * (D + d));
                    buf1[d] = __ldg(q1 + 4 * (D + d));
                    sb0[d] = __ldg(s0p + b + D + d);
                    sb1[d] = __ldg(s1p + b + D + d);
                }
                uint32_t h0[4], h1[4]; // byte q of the lane's piece -> elements (8c + 2q, 8c + 2q + 1) of the block
                e2m1x8_to_f16x8(w0, h0);
                e2m1x8_to_f16x8(w1, h1);
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    const uint4 xv = *xp[mt];
                    xp[mt] += xstep[mt];
                    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    const uint32_t a_lo[4] = {h0[0], h1[0], h0[1], h1[1]}, a_hi[4] = {h0[2], h1[2], h0[3], h1[3]};
                    const uint32_t b_lo[2] = {xv.x, xv.y}, b_hi[2] = {xv.z, xv.w};
                    mx4_mma_f16(acc, a_lo, b_lo);
                    mx4_mma_f16(acc, a_hi, b_hi);
                    tot[mt][0] = fmaf(s0, acc[0], tot[mt][0]);
                    tot[mt][1] = fmaf(s0, acc[1], tot[mt][1]);
                    tot[mt][2] = fmaf(s1, acc[2], tot[mt][2]);
                    tot[mt][3] = fmaf(s1, acc[3], tot[mt][3]);
                }
            }
        }
        q0 += 4 * D;
        q1 += 4 * D;
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
            if (p.bias) sum += load_as_f32(p.bias, p.bias_dtype, bias_off + nn);
            store_as(p.y, p.y_dtype, y_off + (size_t)(m0 + row) * p.n + nn, sum);
        }
    }
    if (ks > 1) cluster.sync(); // nobody leaves while a peer may still read its shared memory
}

template <int MT, int D> static int launch_mx4(const Mx4GemvParams &p, int ks, cudaStream_t st, int batch = 1)
{
    const int nw = p.row_tiles * p.k_warps;
    const int m_cta = p.m < 8 * MT ? p.m : 8 * MT;
    const size_t smem = (size_t)m_cta * (p.k / ks + 8) * 2 + (size_t)nw * MT * 4 * 32 * 4 + 16;
    auto kern = mxfp4_gemv_kernel<MT, D>;
    static size_t configured[64] = {};
    int device = 0;
    OXQ_CUDA(cudaGetDevice(&device));
    if (device >= 64 || configured[device] < smem) {
        OXQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        if (device < 64) configured[device] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ceil_div(p.n, 16 * p.row_tiles) * p.token_split, ks, batch);
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

// Picks warps-per-CTA x cluster so that the k split divides the blocks of a row evenly; false when
// no candidate does (the caller then uses the generic row-format kernel).
static bool mx4_pick(int m, int k, int &nrt, int &kw, int &ks)
{
    const int nb = k / 32;
    // {row tiles, k warps, cluster}: few tokens -> small row groups and a deep k split, so that the grid
    // fills the SMs; more tokens -> more row tiles per CTA, which share the staged x.
    // (measured on the GPT-OSS expert shape 5760 x 2880: one row tile per CTA with 5 or 6 k warps up to 8
    // tokens, eight row tiles per CTA and a cluster of two above)
    static const int few[][3] = {{1, 6, 1}, {1, 5, 1}, {1, 8, 1}, {2, 4, 1}, {2, 3, 1}, {2, 2, 1}, {1, 7, 1}, {2, 1, 1}, {1, 1, 1}};
    static const int many[][3] = {{8, 1, 2}, {4, 2, 2}, {4, 2, 1}, {2, 3, 1}, {8, 1, 1}};
    const int(*cand)[3] = m <= 8 ? few : many;
    const int count = m <= 8 ? 9 : 5;
    for (int t = 0; t < count; t++)
        if (nb % (cand[t][1] * cand[t][2]) == 0) { nrt = cand[t][0]; kw = cand[t][1]; ks = cand[t][2]; return true; }
    return false;
}

bool mxfp4_gemv_fast_supported(int m, int k, const void *blocks, const void *scales)
{
    int a, b, c;
    (void)scales;
    return m <= 32 && k % 32 == 0 && (reinterpret_cast<uintptr_t>(blocks) & 15) == 0 && mx4_pick(m, k, a, b, c) &&
           (size_t)(m < 8 ? m : 8) * (k + 8) * 2 <= 160 * 1024;
}

int mxfp4_gemv_fast(const void *x, const uint8_t *blocks, const uint8_t *scales, const void *bias, int bias_dtype, void *y,
                    int y_dtype, int m, int k, int n, cudaStream_t st)
{
    Mx4GemvParams p;
    p.x = (const __nv_bfloat16 *)x; p.blocks = blocks; p.scales = scales; p.bias = bias; p.y = y;
    p.bias_dtype = bias_dtype; p.y_dtype = y_dtype; p.m = m; p.k = k; p.n = n;
    int nrt = 2, kw = 4, ks = 1;
    mx4_pick(m, k, nrt, kw, ks);
    if (const char *env = tuning_env("OXQ_MXFP4_GEMV_TUNE")) { // bench-harness knob: "row_tiles,k_warps,cluster"
        int a = 0, b = 0, cc = 0;
        if (sscanf(env, "%d,%d,%d", &a, &b, &cc) == 3 && a >= 1 && b >= 1 && a * b <= 8 && cc >= 1 && cc <= 8 &&
            (cc & (cc - 1)) == 0 && (k / 32) % (b * cc) == 0) {
            nrt = a; kw = b; ks = cc;
        }
    }
    p.row_tiles = nrt; p.k_warps = kw;
    p.token_split = ceil_div(m, 8); // 8 tokens per CTA; more on neighbouring CTAs
    p.pair_expert = nullptr; p.x_div = 1; p.e_lo = p.e_hi = 0;
    return launch_mx4<1, 4>(p, ks, st);
}

// One single-token GEMV per (token, slot) pair against the pair's expert, all pairs in one launch:
// y[pair, :] = x[pair / x_div, :] . W[expert(pair)]^T + bias[expert(pair)]; pairs whose expert lies
// outside [e_lo, e_hi) are skipped (their y rows stay untouched). blocks / scales / bias are the
// stacked tensors of all experts ([E, n, k/32, 16], [E, n, k/32], [E, n]).
bool mxfp4_gemv_batched_supported(int k, const void *blocks)
{
    int a, b, c;
    return k % 32 == 0 && (reinterpret_cast<uintptr_t>(blocks) & 15) == 0 && mx4_pick(1, k, a, b, c) &&
           (size_t)(k + 8) * 2 <= 160 * 1024;
}

int mxfp4_gemv_batched(const void *x, int x_div, const uint8_t *blocks, const uint8_t *scales, const void *bias,
                       int bias_dtype, const int *pair_expert, int pairs, int e_lo, int e_hi, void *y, int y_dtype, int k,
                       int n, cudaStream_t st)
{
    Mx4GemvParams p;
    p.x = (const __nv_bfloat16 *)x; p.blocks = blocks; p.scales = scales; p.bias = bias; p.y = y;
    p.bias_dtype = bias_dtype; p.y_dtype = y_dtype; p.m = 1; p.k = k; p.n = n;
    int nrt = 2, kw = 4, ks = 1;
    mx4_pick(1, k, nrt, kw, ks);
    p.row_tiles = nrt; p.k_warps = kw; p.token_split = 1;
    p.pair_expert = pair_expert; p.x_div = x_div; p.e_lo = e_lo; p.e_hi = e_hi;
    return launch_mx4<1, 4>(p, ks, st, pairs);
}

} // namespace oxq
