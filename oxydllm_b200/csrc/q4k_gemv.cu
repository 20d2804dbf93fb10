// GGUF Q4_K and Q5_K decode GEMV (1 <= m <= 32), tuned variant.
//
// Q4_K super-block (144 B / 256 weights): f16 d, f16 dmin, 12 bytes of 6-bit sub-block scales and
// mins, 128 bytes of nibbles; byte t of 32-byte group iq holds element t of sub-block 2*iq (low
// nibble) and of sub-block 2*iq+1 (high nibble); w = (d*sc)*q - dmin*mn.
//
// A thread-block cluster of KS CTAs owns 16 * row_tiles output rows: CTA r of the cluster takes the
// r-th slice of k; inside a CTA the warps are row_tiles x k_warps, the k_warps of a row tile taking
// the slice's super-blocks round-robin. The partial sums of an output are added in a fixed order
// by one thread of the cluster through distributed shared memory (no workspace, no atomics).
// Per super-block a lane streams, straight into registers, the 16-byte header of its two rows
// (lane/4 and lane/4 + 8) and four 8-byte pieces of nibbles: bytes [8c, 8c+8) of each 32-byte
// group (c = lane%4), so the four lanes of a row read 32 contiguous bytes. The k order inside a
// sub-block is free as long as x follows it, which lets every lane feed the tensor cores from its
// own bytes with no exchange: nibbles become f16 pairs with one lop3 each -- 0x6400 | q is
// 1024 + q, and 0x6400 | (q << 4) is 1024 + 16 q, so the high nibbles need no shift -- and go
// into mma.sync m16n8k16 (f16 x f16 -> f32) as the 16-row operand. The CTA stages its slice of x
// as f16 (saturated to +-65504) in the matching element order, together with the per-sub-block
// sums of x; scale, min, the 1024 offset and the factor 16 are folded in f32 once per sub-block:
//   y += d*sc * (acc - 1024*sum_x) / {1,16} - dmin*mn * sum_x.
#include <cooperative_groups.h>

#include <cstdio>
#include <cstdlib>

#include "formats.cuh"

namespace oxq {

struct Q4kGemvParams {
    const __nv_bfloat16 *x;
    const uint8_t *blocks;
    const void *bias;
    void *y;
    int bias_dtype, y_dtype;
    int m, k, n;
    int row_tiles, k_warps; // warps of a CTA = row_tiles x k_warps
    int token_split;        // neighbouring CTAs that share their rows and take 8*MT tokens each (>= 1)
};

namespace cg = cooperative_groups;

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t p, uint32_t mask, uint32_t magic)
{
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(p), "r"(mask), "r"(magic));
    return r;
}

// Byte `idx` (0..3) of v as f32, exact, without the integer-to-float unit.
__device__ __forceinline__ float byte_to_f32(uint32_t v, int idx)
{
    const uint32_t bits = __byte_perm(v, 0x4B000000u, 0x7440 + idx); // [byte idx, 0, 0, 0x4B] = 2^23 + byte
    return __uint_as_float(bits) - 8388608.0f;
}

struct Q4kRow {
    uint4 hdr;     // d | dmin << 16, scales[0..3], scales[4..7], scales[8..11]
    uint2 qs[4];   // bytes [8c, 8c+8) of each 32-byte nibble group
    uint2 qh;      // Q5_K only: bytes [8c, 8c+8) of qh (bit j = fifth bit of sub-block j's element)
};

// FIVE: the Q5_K layout (176 bytes: 32 bytes of fifth bits between the header and the nibbles).
template <bool FIVE> __device__ __forceinline__ void q4k_load_row(Q4kRow &r, const uint8_t *blk, int c)
{
    r.hdr = __ldcs(reinterpret_cast<const uint4 *>(blk));
    constexpr int QS = FIVE ? 48 : 16;
#pragma unroll
    for (int iq = 0; iq < 4; iq++) r.qs[iq] = __ldcs(reinterpret_cast<const uint2 *>(blk + QS + 32 * iq + 8 * c));
    if (FIVE) r.qh = __ldcs(reinterpret_cast<const uint2 *>(blk + 16 + 8 * c));
    else r.qh = make_uint2(0u, 0u);
}

// (word >> or << so that bit `bit` of bytes 0 and 2 lands on bit `to` of the two halves) & (1 << to in both halves), | base.
template <int BIT, int TO> __device__ __forceinline__ uint32_t fifth_bit(uint32_t qhw, uint32_t base)
{
    const uint32_t sh = BIT >= TO ? (qhw >> (BIT - TO >= 0 ? BIT - TO : 0)) : (qhw << (TO - BIT >= 0 ? TO - BIT : 0));
    return (sh & (0x00010001u << TO)) | base;
}

// (d*sc, dmin*mn) of the eight sub-blocks of one row's super-block.
__device__ __forceinline__ void q4k_scales(const uint4 &hdr, float (&dsc)[8], float (&dmn)[8])
{
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFFu)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    const uint32_t sc_lo = hdr.y & 0x3F3F3F3Fu, mn_lo = hdr.z & 0x3F3F3F3Fu;
    const uint32_t sc_hi = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
    const uint32_t mn_hi = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
#pragma unroll
    for (int j = 0; j < 4; j++) {
        dsc[j] = d * byte_to_f32(sc_lo, j);
        dmn[j] = dmin * byte_to_f32(mn_lo, j);
        dsc[4 + j] = d * byte_to_f32(sc_hi, j);
        dmn[4 + j] = dmin * byte_to_f32(mn_hi, j);
    }
}

template <int MT, bool FIVE>
__global__ void __launch_bounds__(256, MT == 1 ? 2 : 1) q4k_gemv_kernel(const Q4kGemvParams p)
{
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_launch_dependents();
    cg::cluster_group cluster = cg::this_cluster();
    const int nrt = p.row_tiles, kwn = p.k_warps, ks = (int)gridDim.y, rank = (int)blockIdx.y; // cluster = grid y extent
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
    const int rt = warp % nrt, kw = warp / nrt;
    // Token tiles of one row group sit in neighbouring CTAs: they stream the same weights at the same
    // time, so all but the first reader hit in L2.
    const int zt = blockIdx.x % p.token_split, bx = blockIdx.x / p.token_split;
    const int m0 = zt * 8 * MT, m_loc = min(8 * MT, p.m - m0); // this CTA's tokens [m0, m0 + m_loc)
    const int n0 = (bx * nrt + rt) * 16;
    const int nsb = p.k >> 8;                 // super-blocks per row
    const int sl_sb = nsb / ks, sb_beg = rank * sl_sb, sb_end = sb_beg + sl_sb; // this CTA's slice
    const int kl = sl_sb << 8, k_cta = sb_beg << 8;
    constexpr int BLK = FIVE ? 176 : 144;
    const size_t row_bytes = (size_t)nsb * BLK;
    const int xrow = kl + 32;                 // halves per staged token row: 64 bytes of padding keep the
                                              // 16-byte fragment reads of a quarter warp on distinct banks
    __half *xs = reinterpret_cast<__half *>(smem);
    float *sx = reinterpret_cast<float *>(smem + (size_t)m_loc * xrow * sizeof(__half)); // [kl/32][8*MT]
    float *red = sx + (size_t)(kl >> 5) * 8 * MT;                                       // [warp][MT*4][lane]
    float *zeros = red + blockDim.x * MT * 4; // 16 bytes of zeros: what lanes without a token read as x

    // Rows past the end re-read the last row; their results are never stored.
    const int r0 = min(n0 + g, p.n - 1), r1 = min(n0 + g + 8, p.n - 1);
    const uint8_t *row0 = p.blocks + (size_t)r0 * row_bytes, *row1 = p.blocks + (size_t)r1 * row_bytes;
    Q4kRow cur0, cur1;
    int sb = sb_beg + kw;
    if (sb < sb_end) {
        q4k_load_row<FIVE>(cur0, row0 + (size_t)sb * BLK, c);
        q4k_load_row<FIVE>(cur1, row1 + (size_t)sb * BLK, c);
    }

    // Stage the slice of x as f16, elements of every group of four stored as [0, 2, 1, 3] (the order in
    // which the nibble masks deliver k), with the per-sub-block sums of the staged values: eight
    // neighbouring threads hold one 32-element sub-block. Only real tokens are staged.
    if (tid < 4) zeros[tid] = 0.0f;
    for (int idx = tid; idx < 8 * MT * (kl >> 5); idx += blockDim.x) sx[idx] = 0.0f; // rows without a token
    __syncthreads();
    pdl_wait(); // x may come from the kernel before this one; the first weights are already on their way
    for (int row = 0; row < m_loc; row++) {
        const uint2 *src = reinterpret_cast<const uint2 *>(p.x + (size_t)(m0 + row) * p.k + k_cta);
        uint2 *dst = reinterpret_cast<uint2 *>(xs + (size_t)row * xrow);
        for (int q4 = tid; q4 < (kl >> 2); q4 += blockDim.x) { // kl / 4 is a multiple of 64: whole warps
            const uint2 raw = __ldg(src + q4);
            uint2 o; // elements [0, 2] and [1, 3]
            o.x = f32x2_to_f16x2_sat(bf16_lo_f32(raw.x), bf16_lo_f32(raw.y));
            o.y = f32x2_to_f16x2_sat(bf16_hi_f32(raw.x), bf16_hi_f32(raw.y));
            dst[q4] = o;
            const __half2 h02 = *reinterpret_cast<const __half2 *>(&o.x), h13 = *reinterpret_cast<const __half2 *>(&o.y);
            const float2 a = __half22float2(h02), b = __half22float2(h13); // sum what the tensor cores will see
            float sum = (a.x + a.y) + (b.x + b.y);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
            if ((lane & 7) == 0) sx[(q4 >> 3) * 8 * MT + row] = sum;
        }
    }
    __syncthreads();

    // This lane's x for fragment column g of token tile mt, or the zeros (stride 0).
    const __half *xp[MT];
    int xstep[MT];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
        const bool real = 8 * mt + g < m_loc;
        xp[mt] = real ? xs + (size_t)(8 * mt + g) * xrow + 8 * c : reinterpret_cast<const __half *>(zeros);
        xstep[mt] = real ? 1 : 0;
    }

    float tot[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) tot[mt][0] = tot[mt][1] = tot[mt][2] = tot[mt][3] = 0.0f;
    uint32_t mask_lo, mask_hi, magic; // kept opaque so that they stay in registers (one immediate per LOP3)
    asm volatile("mov.b32 %0, 0x000F000F;\n\tmov.b32 %1, 0x00F000F0;\n\tmov.b32 %2, 0x64006400;"
                 : "=r"(mask_lo), "=r"(mask_hi), "=r"(magic));

    for (; sb < sb_end; sb += kwn) {
        Q4kRow nxt0 = cur0, nxt1 = cur1;
        if (sb + kwn < sb_end) { // next super-block on its way while this one is consumed
            q4k_load_row<FIVE>(nxt0, row0 + (size_t)(sb + kwn) * BLK, c);
            q4k_load_row<FIVE>(nxt1, row1 + (size_t)(sb + kwn) * BLK, c);
        }
        float dsc0[8], dmn0[8], dsc1[8], dmn1[8];
        q4k_scales(cur0.hdr, dsc0, dmn0);
        q4k_scales(cur1.hdr, dsc1, dmn1);
        const int sub0 = (sb - sb_beg) * 8; // first sub-block of this super-block within the slice
#pragma unroll
        for (int iq = 0; iq < 4; iq++) {
            float acc_lo[MT][4], acc_hi[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int e = 0; e < 4; e++) acc_lo[mt][e] = acc_hi[mt][e] = 0.0f;
            const int sub_lo = sub0 + 2 * iq; // sub-block of the low nibbles
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                // lane c's eight elements of each sub-block, both k steps, in one 16-byte read
                const uint4 xl = *reinterpret_cast<const uint4 *>(xp[mt] + xstep[mt] * (32 * sub_lo));
                const uint4 xh = *reinterpret_cast<const uint4 *>(xp[mt] + xstep[mt] * (32 * sub_lo + 32));
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const uint32_t w0 = j ? cur0.qs[iq].y : cur0.qs[iq].x, w1 = j ? cur1.qs[iq].y : cur1.qs[iq].x;
                    uint32_t a_lo[4] = {lop3_and_or(w0, mask_lo, magic), lop3_and_or(w1, mask_lo, magic),
                                        lop3_and_or(w0 >> 8, mask_lo, magic), lop3_and_or(w1 >> 8, mask_lo, magic)};
                    uint32_t a_hi[4] = {lop3_and_or(w0, mask_hi, magic), lop3_and_or(w1, mask_hi, magic),
                                        lop3_and_or(w0 >> 8, mask_hi, magic), lop3_and_or(w1 >> 8, mask_hi, magic)};
                    if (FIVE) {
                        // fifth bits of the same four elements: bit 2 iq of qh for the low sub-block (worth 16 ->
                        // bit 4 of 1024 + q), bit 2 iq + 1 for the high one (worth 16 * 16 -> bit 8 of 1024 + 16 q);
                        // elements in bytes (0, 2) of the word, then bytes (1, 3)
                        const uint32_t h0 = j ? cur0.qh.y : cur0.qh.x, h1 = j ? cur1.qh.y : cur1.qh.x;
                        a_lo[0] = fifth_bit<2 * 0, 4>(h0 >> (2 * iq), a_lo[0]);
                        a_lo[1] = fifth_bit<2 * 0, 4>(h1 >> (2 * iq), a_lo[1]);
                        a_lo[2] = fifth_bit<8, 4>(h0 >> (2 * iq), a_lo[2]);
                        a_lo[3] = fifth_bit<8, 4>(h1 >> (2 * iq), a_lo[3]);
                        a_hi[0] = fifth_bit<1, 8>(h0 >> (2 * iq), a_hi[0]);
                        a_hi[1] = fifth_bit<1, 8>(h1 >> (2 * iq), a_hi[1]);
                        a_hi[2] = fifth_bit<9, 8>(h0 >> (2 * iq), a_hi[2]);
                        a_hi[3] = fifth_bit<9, 8>(h1 >> (2 * iq), a_hi[3]);
                    }
                    const uint32_t b_lo[2] = {j ? xl.z : xl.x, j ? xl.w : xl.y};
                    const uint32_t b_hi[2] = {j ? xh.z : xh.x, j ? xh.w : xh.y};
                    mma_f16_16816(acc_lo[mt], a_lo, b_lo);
                    mma_f16_16816(acc_hi[mt], a_hi, b_hi);
                }
            }
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                const float2 s_lo = *reinterpret_cast<const float2 *>(sx + (size_t)sub_lo * 8 * MT + 8 * mt + 2 * c);
                const float2 s_hi = *reinterpret_cast<const float2 *>(sx + (size_t)(sub_lo + 1) * 8 * MT + 8 * mt + 2 * c);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float sl = (e & 1) ? s_lo.y : s_lo.x, sh = (e & 1) ? s_hi.y : s_hi.x;
                    const float dl = (e >> 1) ? dsc1[2 * iq] : dsc0[2 * iq], ml = (e >> 1) ? dmn1[2 * iq] : dmn0[2 * iq];
                    const float dh = (e >> 1) ? dsc1[2 * iq + 1] : dsc0[2 * iq + 1], mh = (e >> 1) ? dmn1[2 * iq + 1] : dmn0[2 * iq + 1];
                    float t = tot[mt][e];
                    t = fmaf(dl, fmaf(-1024.0f, sl, acc_lo[mt][e]), t);
                    t = fmaf(-ml, sl, t);
                    t = fmaf(dh * 0.0625f, fmaf(-1024.0f, sh, acc_hi[mt][e]), t);
                    t = fmaf(-mh, sh, t);
                    tot[mt][e] = t;
                }
            }
        }
        cur0 = nxt0;
        cur1 = nxt1;
    }

#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int e = 0; e < 4; e++) red[(warp * MT * 4 + mt * 4 + e) * 32 + lane] = tot[mt][e];
    if (ks > 1) cluster.sync(); else __syncthreads();

    // Every (row tile, accumulator slot, lane) is summed by one thread of the cluster: slices in
    // ascending k, the k warps of a slice in warp order.
    const int slots = nrt * MT * 4 * 32;
    for (int o = rank * blockDim.x + tid; o < slots; o += ks * blockDim.x) {
        const int ln = o & 31, e = (o >> 5) & 3, mt = (o >> 7) % MT, wt = (o >> 7) / MT;
        const int nn = (bx * nrt + wt) * 16 + (ln >> 2) + 8 * (e >> 1), row = 8 * mt + 2 * (ln & 3) + (e & 1);
        if (nn < p.n && row < m_loc) {
            float sum = 0.0f;
            for (int q = 0; q < ks; q++) {
                const float *src = ks > 1 ? cluster.map_shared_rank(red, q) : red;
                for (int w = 0; w < kwn; w++) sum += src[((w * nrt + wt) * MT * 4 + mt * 4 + e) * 32 + ln];
            }
            if (p.bias) sum += load_as_f32(p.bias, p.bias_dtype, nn);
            store_as(p.y, p.y_dtype, (size_t)(m0 + row) * p.n + nn, sum);
        }
    }
    if (ks > 1) cluster.sync(); // nobody leaves while a peer may still read its shared memory
}

static size_t q4k_smem(int mt, int m, int kl, int warps)
{
    return (size_t)m * (kl + 32) * 2 + (size_t)(kl / 32) * 8 * mt * 4 + (size_t)warps * mt * 4 * 32 * 4 + 16;
}

template <int MT, bool FIVE> static int launch_q4k(const Q4kGemvParams &p, int ks, cudaStream_t st)
{
    const int nw = p.row_tiles * p.k_warps;
    const size_t smem = q4k_smem(MT, p.m < 8 * MT ? p.m : 8 * MT, p.k / ks, nw);
    auto kern = q4k_gemv_kernel<MT, FIVE>;
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
bool q4k_gemv_supported(int m, int k)
{
    return m <= 32 && k % 256 == 0 && q4k_smem(m <= 8 ? 1 : 2, m < 16 ? m : 16, k, 8) <= 200 * 1024;
}

// five_bit: the blocks are Q5_K (same kernel with the fifth bits merged into the f16 operands).
int q4k_gemv(const void *x, const void *blocks, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k,
             int n, cudaStream_t st, bool five_bit)
{
    Q4kGemvParams p;
    p.x = (const __nv_bfloat16 *)x; p.blocks = (const uint8_t *)blocks; p.bias = bias; p.y = y;
    p.bias_dtype = bias_dtype; p.y_dtype = y_dtype; p.m = m; p.k = k; p.n = n;
    // Measured on a 4096 x 4096 layer: one row tile per CTA up to 8 tokens, two (sharing the staged x) above.
    int nrt = m > 8 ? 2 : 1, kw = m > 8 ? 4 : 8, ks = 1;
    if (const char *env = tuning_env("OXQ_Q4K_GEMV_TUNE")) { // bench-harness knob: "row_tiles,k_warps,cluster"
        int a = 0, b = 0, cc = 0;
        if (sscanf(env, "%d,%d,%d", &a, &b, &cc) == 3 && a >= 1 && b >= 1 && a * b <= 8 && cc >= 1 && cc <= 8 &&
            (cc & (cc - 1)) == 0 && (k / 256) % cc == 0) {
            nrt = a; kw = b; ks = cc;
        }
    }
    p.row_tiles = nrt; p.k_warps = kw;
    p.token_split = m <= 8 ? 1 : ceil_div(m, 16); // more than 16 tokens: 16 per CTA on neighbouring CTAs
    if (five_bit) return m <= 8 ? launch_q4k<1, true>(p, ks, st) : launch_q4k<2, true>(p, ks, st);
    return m <= 8 ? launch_q4k<1, false>(p, ks, st) : launch_q4k<2, false>(p, ks, st);
}

} // namespace oxq
