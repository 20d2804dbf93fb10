// Decode GEMV (1 <= m <= 32) for the weight formats stored row-major [n, k]
// with their quantization blocks along k: GGUF Q4_0/Q8_0/Q4_K/Q6_K, FP8 E4M3
// with an f32 scale grid, and MXFP4.
//
// A warp owns 16 output rows. Per 16-wide k step each lane decodes four
// consecutive k of two rows (lane/4 and lane/4 + 8) into bf16 pairs, which
// are the 16-row operand of mma.sync m16n8k16; the 8-column operand is up to
// 8 tokens of x; accumulation is f32. The four warps of a CTA split k and are
// summed in warp order through shared memory (fixed order, no atomics).
#include <cstdlib>

#include "formats.cuh"

namespace oxq {

enum RowFormat { RF_Q4_0 = 0, RF_Q8_0, RF_Q4_K, RF_Q6_K, RF_FP8, RF_MXFP4,
                 RF_GGUF_ELEM = 100 }; // RF_GGUF_ELEM + ggml type: any GGUF type through the per-element decoder

struct RowGemvParams {
    const __nv_bfloat16 *x;
    const uint8_t *data;      // blocks / fp8 bytes
    const uint8_t *aux;       // MXFP4 scales
    const float *scale_inv;   // FP8 scale grid or nullptr
    const void *bias;
    void *y;
    int bias_dtype, y_dtype;
    int m, k, n;
    int s_in, block_out, block_in; // FP8 grid geometry
    size_t row_bytes;
};

__device__ __forceinline__ uint32_t ld2x16(const uint8_t *p)
{
    return (uint32_t)reinterpret_cast<const uint16_t *>(p)[0] | ((uint32_t)reinterpret_cast<const uint16_t *>(p)[1] << 16);
}

// Four consecutive weights (k % 4 == 0) of row n, dequantized to f32.
template <int FMT> __device__ __forceinline__ void decode4(const RowGemvParams &p, int n, int k, float (&out)[4])
{
    const uint8_t *row = p.data + (size_t)n * p.row_bytes;
    if (FMT >= RF_GGUF_ELEM) {
        constexpr int TYPE = FMT - RF_GGUF_ELEM;
        int bel = 32, bby = 0;
        gguf_block_layout(TYPE, bel, bby);
        const uint8_t *blk = row + (size_t)(k / bel) * bby;
#pragma unroll
        for (int u = 0; u < 4; u++) out[u] = gguf_decode_elem<TYPE>(blk, (k % bel) + u);
    } else if (FMT == RF_Q4_0) {
        const uint8_t *blk = row + (k >> 5) * 18;
        const int j = k & 31;
        const float d = half_bits_to_f32((uint16_t)ld_u16(blk));
        uint32_t q = ld2x16(blk + 2 + (j & 15));
        if (j >= 16) q >>= 4;
#pragma unroll
        for (int u = 0; u < 4; u++) out[u] = (float)((int)((q >> (8 * u)) & 0xFu) - 8) * d;
    } else if (FMT == RF_Q8_0) {
        const uint8_t *blk = row + (k >> 5) * 34;
        const float d = half_bits_to_f32((uint16_t)ld_u16(blk));
        const uint32_t q = ld2x16(blk + 2 + (k & 31));
#pragma unroll
        for (int u = 0; u < 4; u++) out[u] = (float)(int)(int8_t)((q >> (8 * u)) & 0xFFu) * d;
    } else if (FMT == RF_Q4_K) {
        const uint8_t *blk = row + (k >> 8) * 144;
        const int j = k & 255, sub = j >> 5, el = j & 31;
        const float d = half_bits_to_f32((uint16_t)ld_u16(blk));
        const float dmin = half_bits_to_f32((uint16_t)ld_u16(blk + 2));
        uint32_t sc, mn;
        q4k_scale_min(sub, blk + 4, sc, mn);
        const float sc_v = d * (float)sc, m_v = dmin * (float)mn;
        uint32_t q = *reinterpret_cast<const uint32_t *>(blk + 16 + (sub >> 1) * 32 + el);
        if (sub & 1) q >>= 4;
#pragma unroll
        for (int u = 0; u < 4; u++) out[u] = __fsub_rn(__fmul_rn(sc_v, (float)((q >> (8 * u)) & 0xFu)), m_v);
    } else if (FMT == RF_Q6_K) {
        const uint8_t *blk = row + (k >> 8) * 210;
        const int j = k & 255, half_i = j >> 7, pos = j & 127, quad = pos >> 5, l = pos & 31;
        const uint8_t *ql = blk + 64 * half_i + ((quad & 1) ? l + 32 : l), *qh = blk + 128 + 32 * half_i + l;
        const float d = half_bits_to_f32((uint16_t)ld_u16(blk + 208));
        const float sc_v = d * (float)(int)(int8_t)blk[192 + 8 * half_i + 2 * quad + (l >> 4)];
        const uint32_t qlw = ld2x16(ql), qhw = ld2x16(qh);
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const uint32_t nib = (qlw >> (8 * u + (quad < 2 ? 0 : 4))) & 0xFu;
            const uint32_t hb = (qhw >> (8 * u + 2 * quad)) & 3u;
            out[u] = sc_v * (float)((int)(nib | (hb << 4)) - 32);
        }
    } else if (FMT == RF_FP8) {
        const uint32_t q = *reinterpret_cast<const uint32_t *>(row + k);
        const float s = p.scale_inv ? p.scale_inv[(size_t)(n / p.block_out) * p.s_in + k / p.block_in] : 1.0f;
#pragma unroll
        for (int u = 0; u < 4; u++) out[u] = s * e4m3_to_f32((q >> (8 * u)) & 0xFFu);
    } else { // RF_MXFP4
        const size_t blk = (size_t)n * (p.k >> 5) + (k >> 5);
        const uint32_t q = *reinterpret_cast<const uint16_t *>(p.data + blk * 16 + ((k & 31) >> 1));
        const float s = e8m0_to_f32(p.aux[blk]);
#pragma unroll
        for (int u = 0; u < 4; u++) out[u] = e2m1_to_f32((q >> (4 * u)) & 0xFu) * s;
    }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

__device__ __forceinline__ void mma_bf16_row(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
                 "{%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

bool q4k_gemv_supported(int m, int k);
int q4k_gemv(const void *x, const void *blocks, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k,
             int n, cudaStream_t st, bool five_bit);
bool fp8_gemv_fast_supported(int m, int k, int block_in, const void *w);
int fp8_gemv_fast(const void *x, const uint8_t *w, const float *scale_inv, int s_in, int block_out, int block_in,
                  const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n, cudaStream_t st);

bool q40_gemv_supported(int m, int k, const void *blocks);
int q40_gemv(int variant, const void *x, const void *blocks, const void *bias, int bias_dtype, void *y, int y_dtype, int m,
             int k, int n, cudaStream_t st);
bool q6k_gemv_supported(int m, int k, const void *blocks);
int q6k_gemv(const void *x, const void *blocks, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
             cudaStream_t st);
bool q80_gemv_supported(int m, int k, const void *blocks);
int q80_gemv(const void *x, const void *blocks, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
             cudaStream_t st);
bool mxfp4_gemv_fast_supported(int m, int k, const void *blocks, const void *scales);
int mxfp4_gemv_fast(const void *x, const uint8_t *blocks, const uint8_t *scales, const void *bias, int bias_dtype, void *y,
                    int y_dtype, int m, int k, int n, cudaStream_t st);

constexpr int ROW_NW = 4;

template <int FMT, int MT>
__global__ void __launch_bounds__(ROW_NW * 32) rowfmt_gemv_kernel(const RowGemvParams p)
{
    __shared__ float red[ROW_NW][MT * 4][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const int n0 = blockIdx.x * 16;
    const int r0 = n0 + g, r1 = n0 + g + 8;
    const bool ok0 = r0 < p.n, ok1 = r1 < p.n;
    const int steps = p.k >> 4;
    const int s_beg = (int)((long long)steps * warp / ROW_NW), s_end = (int)((long long)steps * (warp + 1) / ROW_NW);

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.0f;

#pragma unroll 2
    for (int s = s_beg; s < s_end; s++) {
        const int kb = s * 16 + 4 * c;
        float w0[4] = {0, 0, 0, 0}, w1[4] = {0, 0, 0, 0};
        if (ok0) decode4<FMT>(p, r0, kb, w0);
        if (ok1) decode4<FMT>(p, r1, kb, w1);
        // k slots (2c, 2c+1) <- k (4c, 4c+1); slots (2c+8, 2c+9) <- k (4c+2, 4c+3)
        const uint32_t a[4] = {pack_bf16x2(w0[0], w0[1]), pack_bf16x2(w1[0], w1[1]), pack_bf16x2(w0[2], w0[3]),
                               pack_bf16x2(w1[2], w1[3])};
#pragma unroll
        for (int mt = 0; mt < MT; mt++) {
            const int row = 8 * mt + g;
            uint2 xv = make_uint2(0u, 0u);
            if (row < p.m) xv = __ldg(reinterpret_cast<const uint2 *>(p.x + (size_t)row * p.k + kb));
            const uint32_t b[2] = {xv.x, xv.y};
            mma_bf16_row(acc[mt], a, b);
        }
    }

#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int e = 0; e < 4; e++) red[warp][mt * 4 + e][lane] = acc[mt][e];
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                float sum = 0.0f;
#pragma unroll
                for (int w = 0; w < ROW_NW; w++) sum += red[w][mt * 4 + e][lane];
                // acc[e]: out row n0 + g + 8*(e>>1), token 8mt + 2c + (e&1)
                const int nn = n0 + g + 8 * (e >> 1), row = 8 * mt + 2 * c + (e & 1);
                if (nn < p.n && row < p.m) {
                    if (p.bias) sum += load_as_f32(p.bias, p.bias_dtype, nn);
                    store_as(p.y, p.y_dtype, (size_t)row * p.n + nn, sum);
                }
            }
    }
}

template <int FMT> static int launch_rowfmt(const RowGemvParams &p, cudaStream_t st)
{
    const dim3 grid(ceil_div(p.n, 16)), block(ROW_NW * 32);
    if (p.m <= 8) rowfmt_gemv_kernel<FMT, 1><<<grid, block, 0, st>>>(p);
    else if (p.m <= 16) rowfmt_gemv_kernel<FMT, 2><<<grid, block, 0, st>>>(p);
    else rowfmt_gemv_kernel<FMT, 4><<<grid, block, 0, st>>>(p);
    OXQ_LAUNCH_CHECK("rowfmt_gemv_kernel");
    return OXQ_OK;
}

static int check_common(const char *who, const void *x, int x_dtype, const void *w, const void *bias, int bias_dtype,
                        void *y, int y_dtype, int m, int k, int n)
{
    OXQ_REQUIRE(x && w && y, OXQ_ERR_NULL, "%s: null pointer", who);
    OXQ_REQUIRE(x_dtype == OXQ_BF16, OXQ_ERR_UNSUPPORTED, "%s: activations must be bf16", who);
    OXQ_REQUIRE(valid_dtype(y_dtype) && (!bias || valid_dtype(bias_dtype)), OXQ_ERR_UNSUPPORTED,
                "%s: unsupported dtype", who);
    OXQ_REQUIRE(m >= 1 && m <= 32, OXQ_ERR_BAD_SHAPE, "%s: m=%d outside 1..32 (use the GEMM entry)", who, m);
    OXQ_REQUIRE(k > 0 && n > 0, OXQ_ERR_BAD_SHAPE, "%s: non-positive size", who);
    OXQ_REQUIRE(aligned(x, 8) && aligned(y, 4), OXQ_ERR_BAD_ALIGN, "%s: x must be 8-byte aligned", who);
    return OXQ_OK;
}

} // namespace oxq

using namespace oxq;

OXQ_EXPORT int oxq_gguf_gemv(int ggml_type, const void *x, int x_dtype, const void *blocks, const void *bias,
                             int bias_dtype, void *y, int y_dtype, int m, int k, int n, void *stream)
{
    clear_error();
    int rc = check_common("oxq_gguf_gemv", x, x_dtype, blocks, bias, bias_dtype, y, y_dtype, m, k, n);
    if (rc) return rc;
    int bel, bby;
    OXQ_REQUIRE(gguf_block_layout(ggml_type, bel, bby), OXQ_ERR_UNSUPPORTED, "unsupported GGML type %d", ggml_type);
    OXQ_REQUIRE(k % bel == 0, OXQ_ERR_BAD_SHAPE, "GGUF in_features %d is not a multiple of the block size %d", k, bel);
    OXQ_REQUIRE(aligned(blocks, 16), OXQ_ERR_BAD_ALIGN, "GGUF blocks must be 16-byte aligned");
    RowGemvParams p = {};
    p.x = (const __nv_bfloat16 *)x; p.data = (const uint8_t *)blocks; p.bias = bias; p.y = y;
    p.bias_dtype = bias_dtype; p.y_dtype = y_dtype; p.m = m; p.k = k; p.n = n;
    p.row_bytes = (size_t)(k / bel) * bby;
    cudaStream_t st = (cudaStream_t)stream;
    if ((ggml_type == OXQ_GGML_Q4_K || ggml_type == OXQ_GGML_Q5_K) && q4k_gemv_supported(m, k)) {
        const char *env = tuning_env("OXQ_Q4K_FAST"); // bench-harness knob: "0" selects the generic kernel
        if (!(env && env[0] == '0'))
            return q4k_gemv(x, blocks, bias, bias_dtype, y, y_dtype, m, k, n, st, ggml_type == OXQ_GGML_Q5_K);
    }
    const int legacy = ggml_type == OXQ_GGML_Q4_0 ? 0 : ggml_type == OXQ_GGML_Q4_1 ? 1 : ggml_type == OXQ_GGML_Q5_0 ? 2
                       : ggml_type == OXQ_GGML_Q5_1 ? 3 : -1;
    if (legacy >= 0 && q40_gemv_supported(m, k, blocks)) {
        const char *env = tuning_env("OXQ_Q40_FAST"); // bench-harness knob: "0" selects the generic kernel
        if (!(env && env[0] == '0')) return q40_gemv(legacy, x, blocks, bias, bias_dtype, y, y_dtype, m, k, n, st);
    }
    if (ggml_type == OXQ_GGML_Q6_K && q6k_gemv_supported(m, k, blocks)) {
        const char *env = tuning_env("OXQ_Q6K_FAST"); // bench-harness knob: "0" selects the generic kernel
        if (!(env && env[0] == '0')) return q6k_gemv(x, blocks, bias, bias_dtype, y, y_dtype, m, k, n, st);
    }
    if (ggml_type == OXQ_GGML_Q8_0 && q80_gemv_supported(m, k, blocks)) {
        const char *env = tuning_env("OXQ_Q80_FAST"); // bench-harness knob: "0" selects the generic kernel
        if (!(env && env[0] == '0')) return q80_gemv(x, blocks, bias, bias_dtype, y, y_dtype, m, k, n, st);
    }
    switch (ggml_type) {
    case OXQ_GGML_Q4_1: return launch_rowfmt<RF_GGUF_ELEM + OXQ_GGML_Q4_1>(p, st);
    case OXQ_GGML_Q5_0: return launch_rowfmt<RF_GGUF_ELEM + OXQ_GGML_Q5_0>(p, st);
    case OXQ_GGML_Q5_1: return launch_rowfmt<RF_GGUF_ELEM + OXQ_GGML_Q5_1>(p, st);
    case OXQ_GGML_Q5_K: return launch_rowfmt<RF_GGUF_ELEM + OXQ_GGML_Q5_K>(p, st);
    case OXQ_GGML_Q2_K: return launch_rowfmt<RF_GGUF_ELEM + OXQ_GGML_Q2_K>(p, st);
    case OXQ_GGML_Q3_K: return launch_rowfmt<RF_GGUF_ELEM + OXQ_GGML_Q3_K>(p, st);
    case OXQ_GGML_Q4_0: return launch_rowfmt<RF_Q4_0>(p, st);
    case OXQ_GGML_Q8_0: return launch_rowfmt<RF_Q8_0>(p, st);
    case OXQ_GGML_Q4_K: return launch_rowfmt<RF_Q4_K>(p, st);
    default: return launch_rowfmt<RF_Q6_K>(p, st);
    }
}

OXQ_EXPORT int oxq_fp8_gemv(const void *x, int x_dtype, const uint8_t *weight, const float *scale_inv, int s_out,
                            int s_in, const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
                            void *stream)
{
    clear_error();
    int rc = check_common("oxq_fp8_gemv", x, x_dtype, weight, bias, bias_dtype, y, y_dtype, m, k, n);
    if (rc) return rc;
    OXQ_REQUIRE(k % 16 == 0, OXQ_ERR_UNSUPPORTED, "oxq_fp8_gemv: in_features %d must be a multiple of 16", k);
    OXQ_REQUIRE(aligned(weight, 4), OXQ_ERR_BAD_ALIGN, "FP8 weight must be 4-byte aligned");
    RowGemvParams p = {};
    p.x = (const __nv_bfloat16 *)x; p.data = weight; p.scale_inv = scale_inv; p.bias = bias; p.y = y;
    p.bias_dtype = bias_dtype; p.y_dtype = y_dtype; p.m = m; p.k = k; p.n = n;
    p.row_bytes = (size_t)k;
    p.s_in = 1; p.block_out = n; p.block_in = k;
    if (scale_inv) {
        OXQ_REQUIRE(s_out > 0 && s_in > 0 && n % s_out == 0 && k % s_in == 0, OXQ_ERR_BAD_SHAPE,
                    "block-wise FP8 weight_scale_inv [%d, %d] does not tile weight [%d, %d] evenly", s_out, s_in, n, k);
        p.s_in = s_in; p.block_out = n / s_out; p.block_in = k / s_in;
        OXQ_REQUIRE(p.block_in % 4 == 0, OXQ_ERR_UNSUPPORTED, "oxq_fp8_gemv: scale block along k (%d) must be a multiple of 4",
                    p.block_in);
    }
    if (fp8_gemv_fast_supported(m, k, p.block_in, weight)) {
        const char *env = tuning_env("OXQ_FP8_FAST"); // bench-harness knob: "0" selects the generic kernel
        if (!(env && env[0] == '0'))
            return fp8_gemv_fast(x, weight, scale_inv, p.s_in, p.block_out, p.block_in, bias, bias_dtype, y, y_dtype, m, k,
                                 n, (cudaStream_t)stream);
    }
    return launch_rowfmt<RF_FP8>(p, (cudaStream_t)stream);
}

OXQ_EXPORT int oxq_mxfp4_gemv(const void *x, int x_dtype, const uint8_t *blocks, const uint8_t *scales,
                              const void *bias, int bias_dtype, void *y, int y_dtype, int m, int k, int n,
                              void *stream)
{
    clear_error();
    int rc = check_common("oxq_mxfp4_gemv", x, x_dtype, blocks, bias, bias_dtype, y, y_dtype, m, k, n);
    if (rc) return rc;
    OXQ_REQUIRE(scales, OXQ_ERR_NULL, "oxq_mxfp4_gemv: null scales");
    OXQ_REQUIRE(k % 32 == 0, OXQ_ERR_BAD_SHAPE, "MXFP4: cols %d must be a multiple of 32", k);
    OXQ_REQUIRE(aligned(blocks, 2), OXQ_ERR_BAD_ALIGN, "MXFP4 blocks must be 2-byte aligned");
    RowGemvParams p = {};
    p.x = (const __nv_bfloat16 *)x; p.data = blocks; p.aux = scales; p.bias = bias; p.y = y;
    p.bias_dtype = bias_dtype; p.y_dtype = y_dtype; p.m = m; p.k = k; p.n = n;
    p.row_bytes = (size_t)k / 2;
    if (mxfp4_gemv_fast_supported(m, k, blocks, scales)) {
        const char *env = tuning_env("OXQ_MXFP4_FAST"); // bench-harness knob: "0" selects the generic kernel
        if (!(env && env[0] == '0'))
            return mxfp4_gemv_fast(x, blocks, scales, bias, bias_dtype, y, y_dtype, m, k, n, (cudaStream_t)stream);
    }
    return launch_rowfmt<RF_MXFP4>(p, (cudaStream_t)stream);
}
