// GGUF Q4_0 ({f16 d; u8 qs[16]}, 18 bytes per 32 weights: element j < 16 is the low nibble of qs[j],
// element j >= 16 the high nibble of qs[j - 16]; w = (nibble - 8) * d) decode GEMV (1 <= m <= 32), and
// its three siblings: Q4_1 (+ f16 minimum, w = q * d + m), Q5_0 and Q5_1 (+ 32 fifth bits, bit j of qh
// for element j, merged into the f16 operands; the minimum comes back through the sums of x).
//
// Same decomposition as the Q8_0 kernel: warps of a CTA = row tiles x k parts, a thread-block cluster
// adds further k slices, partial sums meet in (distributed) shared memory and are added in a fixed
// order; tokens beyond 8 per CTA go to neighbouring CTAs that stream the same weights. Lane c of the
// quad that feeds one operand row takes bytes qs[4c .. 4c+3] of the block: its low nibbles are the
// weights k = 4c .. 4c+3 (one mma.sync.m16n8k16 step over the block's first half), its high nibbles
// k = 16+4c .. 16+4c+3 (a second step over the second half). Nibbles become f16 pairs with one
// lop3 each -- 0x6400 | q is 1024 + q and 0x6400 | (q << 4) is 1024 + 16 q -- which pairs k with
// k + 2, so x is staged with every group of four in the order [0, 2, 1, 3]. Offsets, the factor 16
// and the -8 come out in f32 with the sums of x over each half block when the block is folded:
//   y += d * ((acc_lo - 1032 * sum_lo) + (acc_hi / 16 - 72 * sum_hi)).
// Blocks are 18 bytes, so a lane's 4 bytes start on a 2-byte boundary in every other block: it
// reads the two aligned words around them and funnel-shifts. Rows must hold an even number of
// blocks (4-byte aligned rows).
#include <cooperative_groups.h>

#include <cstdio>
#include <cstdlib>

#include "oxq_common.cuh"

namespace oxq {

namespace cg = cooperative_groups;

struct Q40GemvParams {
    const __nv_bfloat16 *x;
    const uint8_t *blocks; // [n][k/32][block bytes]
    const void *bias;
    void *y;
    int bias_dtype, y_dtype;
    int m, k, n;
    int row_tiles, k_warps; // warps of a CTA = row_tiles x k_warps
    int token_split;        // neighbouring CTAs that share their rows and take 8 tokens each (>= 1)
};

__device__ __forceinline__ void q40_mma_f16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ uint32_t q40_and_or(uint32_t p, uint32_t mask, uint32_t magic)
{
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(p), "r"(mask), "r"(magic));
    return r;
}

// The four 32-weight formats this kernel serves: V = 0 Q4_0 {d; qs} 18 B, 1 Q4_1 {d; m; qs} 20 B,
// 2 Q5_0 {d; qh; qs} 22 B, 3 Q5_1 {d; m; qh; qs} 24 B. w = (q - off) * d (+ m): off = 8, 0, 16, 0.
template <int V> struct Q40Fmt {
    static constexpr bool HAS_MIN = V == 1 || V == 3, FIVE = V >= 2;
    static constexpr int BLK = 18 + 2 * V, QH = HAS_MIN ? 4 : 2, QS = 2 + (HAS_MIN ? 2 : 0) + (FIVE ? 4 : 0);
    static constexpr float OFF = V == 0 ? 8.0f : V == 2 ? 16.0f : 0.0f;
};

// One lane's share of one block: the two aligned words around its 4 bytes of nibbles, the block's
// scale (and minimum), and for the 5-bit formats the 32 fifth bits.
struct Q40Piece {
    uint32_t w0, w1, qh;
    unsigned short d, m;
};

template <int V> __device__ __forceinline__ void q40_load(Q40Piece &q, const uint8_t *blk, int c)
{
    using Fm = Q40Fmt<V>;
    const uint8_t *p8 = blk + Fm::QS + 4 * c;
    const uint32_t *al = reinterpret_cast<const uint32_t *>(reinterpret_cast<uintptr_t>(p8) & ~(uintptr_t)3);
    q.w0 = __ldg(al);
    // A piece that starts on a word boundary needs no second word (and the last block of the weight has
    // none after it); a shifted piece ends 2 bytes into the next word.
    q.w1 = (reinterpret_cast<uintptr_t>(p8) & 3) ? __ldg(al + 1) : 0u;
    const unsigned short *h = reinterpret_cast<const unsigned short *>(blk);
    q.d = __ldg(h);
    q.m = Fm::HAS_MIN ? __ldg(h + 1) : (unsigned short)0;
    q.qh = Fm::FIVE ? ((uint32_t)__ldg(h + Fm::QH / 2) | ((uint32_t)__ldg(h + Fm::QH / 2 + 1) << 16)) : 0u;
}

// Fifth bits of two elements (bits 0 and 2 of e) placed at bit TO of the low and of the high half:
// (e & 5) * (2^TO + 2^(TO + 14)) puts bit 0 at TO and bit 2 at TO + 16 (the stray copies are masked off).
template <int TO> __device__ __forceinline__ uint32_t q40_fifth(uint32_t e, uint32_t base)
{
    return (((e & 5u) * ((1u << TO) | (1u << (TO + 14)))) & (0x00010001u << TO)) | base;
}

template <int D, int V>
__global__ void __launch_bounds__(256, 3) q40_gemv_kernel(const Q40GemvParams p)
{
    using Fm = Q40Fmt<V>;
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
    float *sx = reinterpret_cast<float *>(smem + (size_t)m_loc * xrow * 2); // [half block][8]: sums of x per 16 k and token
    float *red = sx + (size_t)bl * 16;                                      // [warp][4][lane]
    float *zeros = red + blockDim.x * 4; // 16 bytes of zeros: what lanes without a token read as x

    const int r0 = min(n0 + g, p.n - 1), r1 = min(n0 + g + 8, p.n - 1); // past-the-end rows re-read the last row
    const uint8_t *q0 = p.blocks + ((size_t)r0 * nb + b_cta + b_off) * Fm::BLK;
    const uint8_t *q1 = p.blocks + ((size_t)r1 * nb + b_cta + b_off) * Fm::BLK;

    Q40Piece buf0[D], buf1[D];
#pragma unroll
    for (int d = 0; d < D; d++)
        if (d < wb) {
            q40_load<V>(buf0[d], q0 + Fm::BLK * d, c);
            q40_load<V>(buf1[d], q1 + Fm::BLK * d, c);
        }

    // Stage the slice of x as f16, every group of four in the order [0, 2, 1, 3], with the sums of the
    // staged values over each 16-element half block: four neighbouring threads hold one. Rows without a
    // token keep zero sums.
    if (tid < 4) zeros[tid] = 0.0f;
    for (int idx = tid; idx < bl * 16; idx += blockDim.x) sx[idx] = 0.0f;
    __syncthreads();
    pdl_wait(); // x may come from the kernel before this one; the first weights are already on their way
    for (int row = 0; row < m_loc; row++) {
        const uint2 *src = reinterpret_cast<const uint2 *>(p.x + (size_t)(m0 + row) * p.k + k_cta);
        uint2 *dst = reinterpret_cast<uint2 *>(xs + (size_t)row * xrow);
        // kl / 4 is a multiple of 8, so groups of 4 lanes are valid or not as a whole; the loop bound is
        // rounded up to whole warps because of the shuffles
        for (int q4 = tid; q4 < (((kl >> 2) + 31) & ~31); q4 += blockDim.x) {
            const bool valid = q4 < (kl >> 2);
            const uint2 raw = valid ? __ldg(src + q4) : make_uint2(0u, 0u);
            uint2 o; // elements [0, 2] and [1, 3]
            o.x = f32x2_to_f16x2_sat(bf16_lo_f32(raw.x), bf16_lo_f32(raw.y));
            o.y = f32x2_to_f16x2_sat(bf16_hi_f32(raw.x), bf16_hi_f32(raw.y));
            if (valid) dst[q4] = o;
            const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&o.x));
            const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&o.y)); // sum what the tensor cores will see
            float sum = (a.x + a.y) + (b.x + b.y);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
            if (valid && (lane & 3) == 0) sx[(q4 >> 2) * 8 + row] = sum;
        }
    }
    __syncthreads();

    // This lane's x for fragment column g: four staged halves per half block, or the zeros (stride 0).
    const bool real = g < m_loc;
    const uint2 *xp = real ? reinterpret_cast<const uint2 *>(xs + (size_t)g * xrow + (b_off << 5) + 4 * c)
                           : reinterpret_cast<const uint2 *>(zeros);
    const int xstep = real ? 8 : 0; // 32 halves per block
    const int xhalf = real ? 4 : 0; // 16 halves to the second half block
    const float *sxp = sx + (size_t)b_off * 16 + 2 * c; // sums of tokens 2c, 2c+1 (the accumulator's columns)
    uint32_t mask_lo, mask_hi, magic; // kept opaque so that they stay in registers (one immediate per LOP3)
    asm volatile("mov.b32 %0, 0x000F000F;\n\tmov.b32 %1, 0x00F000F0;\n\tmov.b32 %2, 0x64006400;"
                 : "=r"(mask_lo), "=r"(mask_hi), "=r"(magic));

    float tot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int b = 0; b < wb; b += D) {
#pragma unroll
        for (int d = 0; d < D; d++) {
            if (b + d < wb) {
                const Q40Piece p0 = buf0[d], p1 = buf1[d];
                if (b + D + d < wb) {
                    q40_load<V>(buf0[d], q0 + Fm::BLK * (b + D + d), c);
                    q40_load<V>(buf1[d], q1 + Fm::BLK * (b + D + d), c);
                }
                // with 18- and 22-byte blocks every other block's nibbles start 2 bytes after a word boundary
                const uint32_t sh0 = (uint32_t)(reinterpret_cast<uintptr_t>(q0 + Fm::BLK * (b + d) + Fm::QS) & 3) * 8;
                const uint32_t sh1 = (uint32_t)(reinterpret_cast<uintptr_t>(q1 + Fm::BLK * (b + d) + Fm::QS) & 3) * 8;
                const uint32_t w0 = __funnelshift_r(p0.w0, p0.w1, sh0), w1 = __funnelshift_r(p1.w0, p1.w1, sh1);
                // byte t of the piece: low nibble = element 4c + t, high nibble = element 16 + 4c + t
                uint32_t a_lo[4] = {q40_and_or(w0, mask_lo, magic), q40_and_or(w1, mask_lo, magic),
                                    q40_and_or(w0 >> 8, mask_lo, magic), q40_and_or(w1 >> 8, mask_lo, magic)};
                uint32_t a_hi[4] = {q40_and_or(w0, mask_hi, magic), q40_and_or(w1, mask_hi, magic),
                                    q40_and_or(w0 >> 8, mask_hi, magic), q40_and_or(w1 >> 8, mask_hi, magic)};
                if (Fm::FIVE) {
                    // bit j of qh is the fifth bit of element j: this lane's low elements 4c .. 4c+3 and high
                    // elements 16+4c .. 16+4c+3; worth 16 (bit 4 of 1024 + q) and 16 * 16 (bit 8 of 1024 + 16 q)
                    const uint32_t l0 = p0.qh >> (4 * c), l1 = p1.qh >> (4 * c);
                    const uint32_t h0 = p0.qh >> (16 + 4 * c), h1 = p1.qh >> (16 + 4 * c);
                    a_lo[0] = q40_fifth<4>(l0, a_lo[0]);
                    a_lo[1] = q40_fifth<4>(l1, a_lo[1]);
                    a_lo[2] = q40_fifth<4>(l0 >> 1, a_lo[2]);
                    a_lo[3] = q40_fifth<4>(l1 >> 1, a_lo[3]);
                    a_hi[0] = q40_fifth<8>(h0, a_hi[0]);
                    a_hi[1] = q40_fifth<8>(h1, a_hi[1]);
                    a_hi[2] = q40_fifth<8>(h0 >> 1, a_hi[2]);
                    a_hi[3] = q40_fifth<8>(h1 >> 1, a_hi[3]);
                }
                const uint2 xl = xp[0], xh = xp[xhalf];
                xp += xstep;
                const float2 s_lo = *reinterpret_cast<const float2 *>(sxp + (size_t)(b + d) * 16);
                const float2 s_hi = *reinterpret_cast<const float2 *>(sxp + (size_t)(b + d) * 16 + 8);
                float acc_lo[4] = {0.0f, 0.0f, 0.0f, 0.0f}, acc_hi[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                const uint32_t b_lo[2] = {xl.x, xl.y}, b_hi[2] = {xh.x, xh.y};
                q40_mma_f16(acc_lo, a_lo, b_lo);
                q40_mma_f16(acc_hi, a_hi, b_hi);
                const float d0 = __half2float(__ushort_as_half(p0.d)), d1 = __half2float(__ushort_as_half(p1.d));
                const float m0 = __half2float(__ushort_as_half(p0.m)), m1 = __half2float(__ushort_as_half(p1.m));
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float sl = (e & 1) ? s_lo.y : s_lo.x, sh = (e & 1) ? s_hi.y : s_hi.x;
                    const float v = fmaf(-(1024.0f + Fm::OFF), sl, acc_lo[e]) + fmaf(0.0625f, acc_hi[e], -(64.0f + Fm::OFF) * sh);
                    tot[e] = fmaf((e >> 1) ? d1 : d0, v, tot[e]);
                    if (Fm::HAS_MIN) tot[e] = fmaf((e >> 1) ? m1 : m0, sl + sh, tot[e]);
                }
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

static size_t q40_smem(int m_cta, int kl, int warps)
{
    return (size_t)m_cta * (kl + 8) * 2 + (size_t)(kl / 32) * 16 * 4 + (size_t)warps * 4 * 32 * 4 + 16;
}

template <int V> static int launch_q40(const Q40GemvParams &p, int ks, cudaStream_t st)
{
    const int nw = p.row_tiles * p.k_warps;
    const size_t smem = q40_smem(p.m < 8 ? p.m : 8, p.k / ks, nw);
    auto kern = q40_gemv_kernel<4, V>;
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

// Picks warps-per-CTA x cluster so that the k split divides the blocks of a row evenly.
static bool q40_pick(int m, int k, int &nrt, int &kw, int &ks)
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
bool q40_gemv_supported(int m, int k, const void *blocks)
{
    int a, b, c;
    return m <= 32 && k % 64 == 0 && (reinterpret_cast<uintptr_t>(blocks) & 3) == 0 && q40_pick(m, k, a, b, c) &&
           q40_smem(m < 8 ? m : 8, k, 8) <= 160 * 1024;
}

// variant: 0 Q4_0, 1 Q4_1, 2 Q5_0, 3 Q5_1.
int q40_gemv(int variant, const void *x, const void *blocks, const void *bias, int bias_dtype, void *y, int y_dtype, int m,
             int k, int n, cudaStream_t st)
{
    Q40GemvParams p;
    p.x = (const __nv_bfloat16 *)x; p.blocks = (const uint8_t *)blocks; p.bias = bias; p.y = y;
    p.bias_dtype = bias_dtype; p.y_dtype = y_dtype; p.m = m; p.k = k; p.n = n;
    int nrt = 2, kw = 4, ks = 1;
    q40_pick(m, k, nrt, kw, ks);
    if (const char *env = tuning_env("OXQ_Q40_GEMV_TUNE")) { // bench-harness knob: "row_tiles,k_warps,cluster"
        int a = 0, b = 0, cc = 0;
        if (sscanf(env, "%d,%d,%d", &a, &b, &cc) == 3 && a >= 1 && b >= 1 && a * b <= 8 && cc >= 1 && cc <= 8 &&
            (cc & (cc - 1)) == 0 && (k / 32) % (b * cc) == 0) {
            nrt = a; kw = b; ks = cc;
        }
    }
    p.row_tiles = nrt; p.k_warps = kw;
    p.token_split = ceil_div(m, 8); // 8 tokens per CTA; more on neighbouring CTAs
    switch (variant) {
    case 1: return launch_q40<1>(p, ks, st);
    case 2: return launch_q40<2>(p, ks, st);
    case 3: return launch_q40<3>(p, ks, st);
    default: return launch_q40<0>(p, ks, st);
    }
}

} // namespace oxq
