// Dequantization kernels: packed weights -> dense [n, k] in f32/f16/bf16,
// bit-exact with the reference's CPU dequantizers. They are memory-bound
// elementwise passes (the load-time path of the reference on non-Metal
// devices, and the checking tool for every fused kernel).
#include "formats.cuh"

namespace oxq {

// ---- AWQ -------------------------------------------------------------------
// A CTA converts a tile of TK input rows x 64 out columns (8 packed words per
// row) and transposes it through shared memory so that the dense [n, k] output
// is written in runs along k.
constexpr int AWQ_TK = 32;

template <typename OutT>
__global__ void __launch_bounds__(256)
awq_dequant_kernel(const uint32_t *__restrict__ qweight, const uint32_t *__restrict__ qzeros,
                   const void *__restrict__ scales, int scales_dtype, OutT *__restrict__ w_out, int k, int n,
                   int group_size, int n_full, int n_off)
{
    // Output rows are out columns [n_off, n_off + n) of a layer with n_full columns (n_off % 8 == 0).
    __shared__ float tile[64][AWQ_TK + 1];
    const int packed_out = n >> 3, packed_full = n_full >> 3, jw_off = n_off >> 3;
    const int k0 = blockIdx.y * AWQ_TK;
    const int jw0 = blockIdx.x * 8;
    const int t = threadIdx.x;

    {
        const int r = t >> 3, jw = jw0 + (t & 7);
        const int kk = k0 + r;
        if (kk < k && jw < packed_out) {
            const int g = kk / group_size;
            const uint32_t w = qweight[(size_t)kk * packed_full + jw_off + jw];
            const uint32_t z = qzeros[(size_t)g * packed_full + jw_off + jw];
#pragma unroll
            for (int col = 0; col < 8; col++) {
                const int sh = 4 * awq_slot_of_col(col);
                const int q = (int)((w >> sh) & 0xFu) - (int)((z >> sh) & 0xFu);
                const float s = load_as_f32(scales, scales_dtype, (size_t)g * n_full + n_off + (size_t)jw * 8 + col);
                tile[(t & 7) * 8 + col][r] = __fmul_rn((float)q, s);
            }
        }
    }
    __syncthreads();
    // 64 columns x 32 k: each group of 32 threads writes one column's run.
    for (int c = t >> 5; c < 64; c += 8) {
        const int o = jw0 * 8 + c, kk = k0 + (t & 31);
        if (o < n && kk < k) w_out[(size_t)o * k + kk] = narrow<OutT>(tile[c][t & 31]);
    }
}

// ---- GPTQ ------------------------------------------------------------------
// One thread per output element, consecutive threads along k of one out row;
// a word of qweight serves pf consecutive k so the reads stay cached.
template <typename OutT>
__global__ void __launch_bounds__(256)
gptq_dequant_kernel(const uint32_t *__restrict__ qweight, const uint32_t *__restrict__ qzeros,
                    const void *__restrict__ scales, int scales_dtype, OutT *__restrict__ w_out, int k, int n,
                    int group_size, int bits, int sym, int n_full, int n_off)
{
    const int pf = 32 / bits;
    const uint32_t mask = (1u << bits) - 1u;
    const size_t total = (size_t)n * k;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int o = n_off + (int)(idx / k), i = (int)(idx % k);
        const int g = i / group_size;
        const uint32_t q = (qweight[(size_t)(i / pf) * n_full + o] >> ((i % pf) * bits)) & mask;
        uint32_t zero;
        if (sym) zero = (1u << (bits - 1)) - 1u;
        else zero = (qzeros[(size_t)g * (n_full / pf) + o / pf] >> ((o % pf) * bits)) & mask;
        const float s = load_as_f32(scales, scales_dtype, (size_t)g * n_full + o);
        w_out[idx] = narrow<OutT>(__fmul_rn((float)((int)q - ((int)zero + 1)), s));
    }
}

// ---- W8A16: the AWQ layout at 8 bits ------------------------------------------
// qweight u32 [k, n / 4]: byte c of word j is out column 4 j + c (no interleave); qzeros u32 [k / g, n / 4];
// w[o][i] = (q - zero) * scale (quant_kernels.metal:1-16,40-48). One thread per output element along k.
template <typename OutT>
__global__ void __launch_bounds__(256)
w8a16_dequant_kernel(const uint32_t *__restrict__ qweight, const uint32_t *__restrict__ qzeros,
                     const void *__restrict__ scales, int scales_dtype, OutT *__restrict__ w_out, int k, int n,
                     int group_size, int n_full, int n_off)
{
    const size_t total = (size_t)n * k;
    const int packed_out = n_full / 4;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int o = n_off + (int)(idx / k), i = (int)(idx % k);
        const int g = i / group_size, sh = 8 * (o & 3);
        const int q = (int)((qweight[(size_t)i * packed_out + (o >> 2)] >> sh) & 0xFFu);
        const int zero = (int)((qzeros[(size_t)g * packed_out + (o >> 2)] >> sh) & 0xFFu);
        const float s = load_as_f32(scales, scales_dtype, (size_t)g * n_full + o);
        w_out[idx] = narrow<OutT>(__fmul_rn((float)(q - zero), s));
    }
}

// ---- GGUF ------------------------------------------------------------------
template <int TYPE, typename OutT>
__global__ void __launch_bounds__(256)
gguf_dequant_kernel(const uint8_t *__restrict__ blocks, OutT *__restrict__ w_out, size_t total)
{
    int bel, bby;
    gguf_block_layout(TYPE, bel, bby);
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t b = idx / bel;
        const int j = (int)(idx % bel);
        w_out[idx] = narrow<OutT>(gguf_decode_elem<TYPE>(blocks + b * bby, j));
    }
}

// ---- FP8 -------------------------------------------------------------------
// Four bytes per thread; scale grid [s_out, s_in] tiles the [n, k] weight in
// (n/s_out) x (k/s_in) blocks. scale_inv == nullptr means no scaling.
template <typename OutT>
__global__ void __launch_bounds__(256)
fp8_dequant_kernel(const uint8_t *__restrict__ weight, const float *__restrict__ scale_inv, int s_in, int block_out,
                   int block_in, OutT *__restrict__ w_out, int n, int k, int row_off)
{
    const size_t total4 = (size_t)n * k / 4;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total4;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t e = idx * 4;
        const int r = (int)(e / k), c = (int)(e % k);
        const uint32_t w = reinterpret_cast<const uint32_t *>(weight)[idx];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            float v = e4m3_to_f32((w >> (8 * u)) & 0xFFu);
            if (scale_inv) v = __fmul_rn(scale_inv[(size_t)((row_off + r) / block_out) * s_in + (c + u) / block_in], v);
            w_out[e + u] = narrow<OutT>(v);
        }
    }
}

// ---- MXFP4 -----------------------------------------------------------------
// One thread per packed byte (two consecutive k of one row).
template <typename OutT>
__global__ void __launch_bounds__(256)
mxfp4_dequant_kernel(const uint8_t *__restrict__ blocks, const uint8_t *__restrict__ scales,
                     OutT *__restrict__ w_out, size_t total_bytes)
{
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_bytes;
         idx += (size_t)gridDim.x * blockDim.x) {
        const uint32_t b = blocks[idx];
        const float s = e8m0_to_f32(scales[idx >> 4]);
        w_out[2 * idx] = narrow<OutT>(__fmul_rn(e2m1_to_f32(b & 0xFu), s));
        w_out[2 * idx + 1] = narrow<OutT>(__fmul_rn(e2m1_to_f32(b >> 4), s));
    }
}


// ---- slab producers for the tensor-core GEMM (bf16 out, same bits as the kernels above) --------
// AWQ: a CTA of 256 threads owns 256 out columns x 64 input rows. The 64 x 32 packed words are
// staged with coalesced 128-byte row reads; then each warp walks 32 out columns, and for one
// column the 32 lanes produce the 64 k values (two each) and store them as one contiguous
// 128-byte line of the dense [n, k] weight. Nibble slot, zero point and scale are warp-uniform.
__global__ void __launch_bounds__(256)
awq_slab_bf16_kernel(const uint32_t *__restrict__ qweight, const uint32_t *__restrict__ qzeros,
                     const void *__restrict__ scales, int scales_dtype, __nv_bfloat16 *__restrict__ out, int k,
                     int n_cnt, int group_size, int n_full, int n_off)
{
    __shared__ uint32_t raw[64][33];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int packed_full = n_full >> 3;
    const int jw0 = (n_off >> 3) + blockIdx.x * 32; // first packed word of the tile (absolute)
    const int k0 = blockIdx.y * 64;
    const int jw_end = (n_off + n_cnt) >> 3;
    for (int idx = t; idx < 64 * 32; idx += 256) {
        const int r = idx >> 5, j = idx & 31;
        uint32_t w = 0;
        if (k0 + r < k && jw0 + j < jw_end) w = __ldcs(qweight + (size_t)(k0 + r) * packed_full + jw0 + j);
        raw[r][j] = w;
    }
    __syncthreads();
    const int ka = k0 + 2 * lane, kb = ka + 1; // this lane's two input rows
    const bool pair_ok = kb < k && (k % 2) == 0;
    const bool tile_one_group = (group_size % 64) == 0; // then the 64 rows of the tile share zero point and scale
    const int g_tile = k0 / group_size;
#pragma unroll 4
    for (int i = 0; i < 32; i++) {
        const int cl = warp * 32 + i;           // column inside the tile
        const int col = blockIdx.x * 256 + cl;  // column inside the slab
        if (col >= n_cnt) break;
        const int jl = cl >> 3, sh = 4 * awq_slot_of_col(cl & 7);
        const size_t nn = (size_t)n_off + col;
        int z = 0;
        float sc = 0.0f;
        if (tile_one_group) {
            z = (int)((__ldg(qzeros + (size_t)g_tile * packed_full + jw0 + jl) >> sh) & 0xFu);
            sc = load_as_f32(scales, scales_dtype, (size_t)g_tile * n_full + nn);
        }
        float v[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            if (!tile_one_group) {
                const int g = min(ka + h, k - 1) / group_size;
                z = (int)((__ldg(qzeros + (size_t)g * packed_full + jw0 + jl) >> sh) & 0xFu);
                sc = load_as_f32(scales, scales_dtype, (size_t)g * n_full + nn);
            }
            const int d = (int)((raw[2 * lane + h][jl] >> sh) & 0xFu) - z;
            // exact int -> float for |d| <= 15 without the conversion unit: 1.5 * 2^23 + d, minus 1.5 * 2^23
            const float df = __uint_as_float(0x4B400000u + (uint32_t)d) - 12582912.0f;
            v[h] = __fmul_rn(df, sc);
        }
        __nv_bfloat16 *dst = out + (size_t)col * k;
        if (pair_ok) {
            __nv_bfloat162 hh = __floats2bfloat162_rn(v[0], v[1]);
            *reinterpret_cast<__nv_bfloat162 *>(dst + ka) = hh;
        } else {
            if (ka < k) dst[ka] = __float2bfloat16_rn(v[0]);
            if (kb < k) dst[kb] = __float2bfloat16_rn(v[1]);
        }
    }
}

// ---- fast slab producers (same bits as the kernels above, a fraction of the instructions) -------
__device__ __forceinline__ uint32_t pack_bf16x2_rn(float lo, float hi)
{
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// AWQ: a CTA of 256 threads owns 128 input rows x 32 packed words (256 out columns). The words are
// staged with coalesced 16-byte loads; then thread (word jj = lane, k block kb = warp) turns its 16
// words into, for each of the word's eight out columns, 16 consecutive k of that column's dense row;
// the rows are stored 256 contiguous bytes at a time. q - z is formed exactly in f32 by the 2^23 trick
// ((2^23 + q) - (2^23 + z)), multiplied by the scale in f32 and rounded to bf16 once, as the
// element-wise kernel does. Needs group_size % 16 == 0 and k % 16 == 0.
__global__ void __launch_bounds__(256)
awq_slab16_bf16_kernel(const uint32_t *__restrict__ qweight, const uint32_t *__restrict__ qzeros,
                       const void *__restrict__ scales, int scales_dtype, __nv_bfloat16 *__restrict__ out, int k,
                       int n_cnt, int group_size, int n_full, int n_off, int vec_ok, int row_mul, int row_add)
{
    __shared__ __align__(16) uint32_t raw[128][32];
    __shared__ __align__(16) unsigned char stage[2][32 * 272];
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const int packed_full = n_full >> 3;
    const int jw0 = (n_off >> 3) + blockIdx.x * 32; // first packed word of the tile (absolute)
    const int jw_end = (n_off + n_cnt) >> 3;
    const int k0 = blockIdx.y * 128;
    {
        const int r_in = t >> 3, w4 = (t & 7) * 4;
#pragma unroll
        for (int it = 0; it < 4; it++) {
            const int r = r_in + 32 * it;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (k0 + r < k) {
                const uint32_t *src = qweight + (size_t)(k0 + r) * packed_full + jw0 + w4;
                if (vec_ok && jw0 + w4 + 4 <= jw_end) v = __ldcs(reinterpret_cast<const uint4 *>(src));
                else {
                    if (jw0 + w4 + 0 < jw_end) v.x = __ldcs(src + 0);
                    if (jw0 + w4 + 1 < jw_end) v.y = __ldcs(src + 1);
                    if (jw0 + w4 + 2 < jw_end) v.z = __ldcs(src + 2);
                    if (jw0 + w4 + 3 < jw_end) v.w = __ldcs(src + 3);
                }
            }
            *reinterpret_cast<uint4 *>(&raw[r][w4]) = v;
        }
    }
    __syncthreads();
    const int j = jw0 + lane, kb = k0 + 16 * warp;
    const bool active = j < jw_end && kb < k;
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 16; i++) w[i] = raw[16 * warp + i][lane];
    uint32_t zw = 0u;
    float sc[8]; // scales of out columns 8j .. 8j+7
#pragma unroll
    for (int c = 0; c < 8; c++) sc[c] = 0.0f;
    if (active) {
        const int g = kb / group_size;
        zw = __ldg(qzeros + (size_t)g * packed_full + j);
        const size_t s0 = (size_t)g * n_full + (size_t)j * 8;
#pragma unroll
        for (int c = 0; c < 8; c++) sc[c] = load_as_f32(scales, scales_dtype, s0 + c);
    }
    // The 16 k of one out column go through shared memory so that a warp stores whole rows: for
    // nibble p the tile's 32 rows x 128 k (256 bytes each, padded to 272) are written by their
    // producers, then warp w stores rows 4w .. 4w+3, eight lanes x 32 bytes per row.
    const int row_l = 4 * warp + (lane >> 3), piece = lane & 7; // the row and 32-byte piece this lane stores
    const int j_st = jw0 + row_l;
    const bool st_ok = j_st < jw_end && k0 + 16 * piece < k;
    // Output row of the slab's column n (counted from n_off): row_mul * n + row_add. (1, 0) is the plain
    // dense weight; (2, 0) and (2, 1) on the gate and the up columns of a fused [gate | up] weight make
    // gate j and up j neighbouring rows.
    const int n_st = 8 * (j_st - (n_off >> 3));
    __nv_bfloat16 *st0 = out + k0 + 16 * piece;
#pragma unroll
    for (int p = 0; p < 8; p++) {
        const int c = p < 4 ? 2 * p : 2 * (p - 4) + 1; // nibble p holds out column c of the word
        unsigned char *buf = stage[p & 1];
        if (active) {
            const float zf = __uint_as_float(0x4B000000u | ((zw >> (4 * p)) & 0xFu));
            const float s = sc[c];
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float a = __uint_as_float(0x4B000000u | ((w[2 * i] >> (4 * p)) & 0xFu)) - zf;
                const float b = __uint_as_float(0x4B000000u | ((w[2 * i + 1] >> (4 * p)) & 0xFu)) - zf;
                o[i] = pack_bf16x2_rn(__fmul_rn(a, s), __fmul_rn(b, s));
            }
            uint4 *d = reinterpret_cast<uint4 *>(buf + lane * 272 + warp * 32);
            d[0] = make_uint4(o[0], o[1], o[2], o[3]);
            d[1] = make_uint4(o[4], o[5], o[6], o[7]);
        }
        __syncthreads(); // buffer p & 1 complete; its previous readers (nibble p - 2) passed the sync of p - 1
        if (st_ok) {
            const uint4 *sv = reinterpret_cast<const uint4 *>(buf + row_l * 272 + piece * 32);
            const int n_row = row_mul * (n_st + c) + row_add;
            uint4 *dst = reinterpret_cast<uint4 *>(st0 + (size_t)n_row * k);
            dst[0] = sv[0];
            dst[1] = sv[1];
        }
    }
}

// FP8: a thread converts 16 consecutive bytes of a row: the hardware widens E4M3 pairs to f16 pairs
// (exact), f16 -> f32 is exact, one f32 multiply by the block's scale, one rounding to bf16. Words
// holding a NaN byte take the element-wise route so that the NaN bits stay the same.
// A CTA covers 256 * 16 columns of FP8_SLAB_ROWS rows.
constexpr int FP8_SLAB_ROWS = 4;
__global__ void __launch_bounds__(256)
fp8_slab16_bf16_kernel(const uint8_t *__restrict__ weight, const float *__restrict__ scale_inv, int s_in, int block_out,
                       int block_in, __nv_bfloat16 *__restrict__ out, int n_cnt, int k, int row_off)
{
    const int c16 = blockIdx.x * 256 + threadIdx.x;
    if (c16 * 16 >= k) return;
    const int kb = scale_inv ? (c16 * 16) / block_in : 0;
#pragma unroll
    for (int r = 0; r < FP8_SLAB_ROWS; r++) {
        const int row = blockIdx.y * FP8_SLAB_ROWS + r;
        if (row >= n_cnt) break;
        const uint4 wv = __ldcs(reinterpret_cast<const uint4 *>(weight + (size_t)row * k) + c16);
        const float s = scale_inv ? __ldg(scale_inv + (size_t)((row_off + row) / block_out) * s_in + kb) : 1.0f;
        const uint32_t v[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t o[8];
#pragma unroll
        for (int q = 0; q < 4; q++) {
            if ((((v[q] & 0x7F7F7F7Fu) + 0x01010101u) & 0x80808080u) == 0u) {
                uint32_t h01, h23;
                asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
                    "cvt.rn.f16x2.e4m3x2 %1, hi;\n\t}"
                    : "=r"(h01), "=r"(h23)
                    : "r"(v[q]));
                const float2 f01 = __half22float2(*reinterpret_cast<const __half2 *>(&h01));
                const float2 f23 = __half22float2(*reinterpret_cast<const __half2 *>(&h23));
                if (scale_inv) {
                    o[2 * q] = pack_bf16x2_rn(__fmul_rn(s, f01.x), __fmul_rn(s, f01.y));
                    o[2 * q + 1] = pack_bf16x2_rn(__fmul_rn(s, f23.x), __fmul_rn(s, f23.y));
                } else {
                    o[2 * q] = pack_bf16x2_rn(f01.x, f01.y);
                    o[2 * q + 1] = pack_bf16x2_rn(f23.x, f23.y);
                }
            } else {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    float a = e4m3_to_f32((v[q] >> (16 * h)) & 0xFFu), b = e4m3_to_f32((v[q] >> (16 * h + 8)) & 0xFFu);
                    if (scale_inv) { a = __fmul_rn(s, a); b = __fmul_rn(s, b); }
                    __nv_bfloat162 hh = __floats2bfloat162_rn(a, b);
                    o[2 * q + h] = *reinterpret_cast<uint32_t *>(&hh);
                }
            }
        }
        uint4 *dst = reinterpret_cast<uint4 *>(out + (size_t)row * k) + 2 * c16;
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

// MXFP4: a thread converts one 16-byte block (32 weights, one E8M0 scale). A 256-entry table in
// shared memory maps a byte to its two E2M1 values as a bf16 pair; scaling by 2^(s-127) is an exact
// bf16 multiply while the result stays normal (4 <= s <= 250); other scales, NaN and the
// subnormal 2^-127 among them, take the element-wise route.
__global__ void __launch_bounds__(256)
mxfp4_slab16_bf16_kernel(const uint8_t *__restrict__ blocks, const uint8_t *__restrict__ scales,
                         __nv_bfloat16 *__restrict__ out, size_t total_blocks)
{
    __shared__ uint32_t lut[256];
    {
        const uint32_t b = threadIdx.x;
        __nv_bfloat162 hh = __floats2bfloat162_rn(e2m1_to_f32(b & 0xFu), e2m1_to_f32(b >> 4));
        lut[b] = *reinterpret_cast<uint32_t *>(&hh);
    }
    __syncthreads();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_blocks;
         idx += (size_t)gridDim.x * blockDim.x) {
        const uint4 bv = __ldcs(reinterpret_cast<const uint4 *>(blocks) + idx);
        const uint32_t sb = scales[idx];
        const uint32_t v[4] = {bv.x, bv.y, bv.z, bv.w};
        uint32_t o[16];
        if (sb >= 4u && sb <= 250u) {
            const uint32_t s2 = (sb << 7) | (sb << 23); // 2^(s-127) as a bf16 pair
            const __nv_bfloat162 sc = *reinterpret_cast<const __nv_bfloat162 *>(&s2);
#pragma unroll
            for (int q = 0; q < 4; q++)
#pragma unroll
                for (int h = 0; h < 4; h++) {
                    const uint32_t e = lut[(v[q] >> (8 * h)) & 0xFFu];
                    const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&e), sc);
                    o[4 * q + h] = *reinterpret_cast<const uint32_t *>(&r);
                }
        } else {
            const float s = e8m0_to_f32(sb);
#pragma unroll
            for (int q = 0; q < 4; q++)
#pragma unroll
                for (int h = 0; h < 4; h++) {
                    const uint32_t b = (v[q] >> (8 * h)) & 0xFFu;
                    __nv_bfloat162 hh = __halves2bfloat162(narrow<__nv_bfloat16>(__fmul_rn(e2m1_to_f32(b & 0xFu), s)),
                                                           narrow<__nv_bfloat16>(__fmul_rn(e2m1_to_f32(b >> 4), s)));
                    o[4 * q + h] = *reinterpret_cast<uint32_t *>(&hh);
                }
        }
        uint4 *dst = reinterpret_cast<uint4 *>(out) + 4 * idx;
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
        dst[2] = make_uint4(o[8], o[9], o[10], o[11]);
        dst[3] = make_uint4(o[12], o[13], o[14], o[15]);
    }
}

// Q4_K: a thread converts one 32-byte nibble group of a super-block: sub-block 2*iq from the low
// nibbles and 2*iq+1 from the high ones, 64 weights = 128 contiguous output bytes. The arithmetic
// is the element-wise kernel's, operation for operation: (d*sc)*q - (dmin*mn), three roundings.
// FIVE: the Q5_K layout (176 bytes, 32 bytes of fifth bits after the header: bit j of qh[el] belongs to sub-block j).
template <bool FIVE>
__global__ void __launch_bounds__(256)
q4k_slab_bf16_kernel(const uint8_t *__restrict__ blocks, __nv_bfloat16 *__restrict__ out, size_t total_groups)
{
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_groups;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t sb = idx >> 2;
        const int iq = (int)(idx & 3);
        const uint8_t *blk = blocks + sb * (FIVE ? 176 : 144);
        const uint4 hdr = __ldg(reinterpret_cast<const uint4 *>(blk));
        const uint4 qa = __ldcs(reinterpret_cast<const uint4 *>(blk + (FIVE ? 48 : 16) + 32 * iq));
        const uint4 qb = __ldcs(reinterpret_cast<const uint4 *>(blk + (FIVE ? 64 : 32) + 32 * iq));
        uint4 ha = make_uint4(0u, 0u, 0u, 0u), hb = ha;
        if (FIVE) {
            ha = __ldg(reinterpret_cast<const uint4 *>(blk + 16));
            hb = __ldg(reinterpret_cast<const uint4 *>(blk + 32));
        }
        const uint32_t qhw[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w}; // byte t = fifth bits of element t
        const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFFu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
        const uint32_t sw[3] = {hdr.y, hdr.z, hdr.w}; // the 12 scale bytes
        auto byte_at = [&](int j) -> uint32_t { return (sw[j >> 2] >> (8 * (j & 3))) & 0xFFu; };
        float sc_v[2], m_v[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int j = 2 * iq + h;
            uint32_t sc, mn;
            if (j < 4) {
                sc = byte_at(j) & 63u;
                mn = byte_at(j + 4) & 63u;
            } else {
                sc = (byte_at(j + 4) & 0x0Fu) | ((byte_at(j - 4) >> 6) << 4);
                mn = (byte_at(j + 4) >> 4) | ((byte_at(j) >> 6) << 4);
            }
            sc_v[h] = __fmul_rn(d, (float)sc);
            m_v[h] = __fmul_rn(dmin, (float)mn);
        }
        const uint32_t q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w}; // byte t = element t of both sub-blocks
        uint4 *dst = reinterpret_cast<uint4 *>(out + sb * 256 + 64 * iq);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            uint32_t o[16];
#pragma unroll
            for (int wd = 0; wd < 8; wd++) {
                const uint32_t v = h ? (q[wd] >> 4) : q[wd];
                const uint32_t hv = FIVE ? ((qhw[wd] >> (2 * iq + h)) & 0x01010101u) << 4 : 0u;
                float f[4];
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    const float nib = __uint_as_float(0x4B000000u | (((v >> (8 * b)) & 0x0Fu) | ((hv >> (8 * b)) & 0x10u))) - 8388608.0f;
                    f[b] = __fsub_rn(__fmul_rn(sc_v[h], nib), m_v[h]);
                }
                o[2 * wd] = pack_bf16x2_rn(f[0], f[1]);
                o[2 * wd + 1] = pack_bf16x2_rn(f[2], f[3]);
            }
#pragma unroll
            for (int t = 0; t < 4; t++) dst[4 * h + t] = make_uint4(o[4 * t], o[4 * t + 1], o[4 * t + 2], o[4 * t + 3]);
        }
    }
}

// Q8_0 / Q4_0 / Q6_K producers: one thread per 32 (Q8_0, Q4_0) or 16 (Q6_K) weights, halfword loads
// (the blocks are only 2-byte aligned), the element-wise kernels' arithmetic operation for operation,
// 16-byte stores. Exact small integers come from the 2^23 trick instead of the conversion unit.
__device__ __forceinline__ float small_int_f32(int v) // |v| < 2^22
{
    return __uint_as_float(0x4B400000u + (uint32_t)v) - 12582912.0f; // 1.5 * 2^23 + v, minus 1.5 * 2^23
}

__global__ void __launch_bounds__(256)
q80_slab_bf16_kernel(const uint8_t *__restrict__ blocks, __nv_bfloat16 *__restrict__ out, size_t total_blocks)
{
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_blocks;
         idx += (size_t)gridDim.x * blockDim.x) {
        const unsigned short *h = reinterpret_cast<const unsigned short *>(blocks + idx * 34);
        const float d = __half2float(__ushort_as_half(__ldg(h)));
        uint32_t o[16];
#pragma unroll
        for (int t = 0; t < 16; t++) {
            const uint32_t two = __ldg(h + 1 + t); // elements 2t, 2t+1
            const float a = __fmul_rn(small_int_f32((int)(signed char)(two & 0xFFu)), d);
            const float b = __fmul_rn(small_int_f32((int)(signed char)(two >> 8)), d);
            o[t] = pack_bf16x2_rn(a, b);
        }
        uint4 *dst = reinterpret_cast<uint4 *>(out + idx * 32);
#pragma unroll
        for (int t = 0; t < 4; t++) dst[t] = make_uint4(o[4 * t], o[4 * t + 1], o[4 * t + 2], o[4 * t + 3]);
    }
}

// V = 0 Q4_0 {d; qs} 18 B, 1 Q4_1 {d; m; qs} 20 B, 2 Q5_0 {d; qh; qs} 22 B, 3 Q5_1 {d; m; qh; qs} 24 B.
template <int V>
__global__ void __launch_bounds__(256)
q40_slab_bf16_kernel(const uint8_t *__restrict__ blocks, __nv_bfloat16 *__restrict__ out, size_t total_blocks)
{
    constexpr bool HAS_MIN = V == 1 || V == 3, FIVE = V >= 2;
    constexpr int BLK = 18 + 2 * V, QH = (HAS_MIN ? 4 : 2) / 2, QS = (2 + (HAS_MIN ? 2 : 0) + (FIVE ? 4 : 0)) / 2; // halfword offsets
    constexpr int OFF = V == 0 ? 8 : V == 2 ? 16 : 0;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_blocks;
         idx += (size_t)gridDim.x * blockDim.x) {
        const unsigned short *h = reinterpret_cast<const unsigned short *>(blocks + idx * BLK);
        const float d = __half2float(__ushort_as_half(__ldg(h)));
        const float mn = HAS_MIN ? __half2float(__ushort_as_half(__ldg(h + 1))) : 0.0f;
        const uint32_t qh = FIVE ? ((uint32_t)__ldg(h + QH) | ((uint32_t)__ldg(h + QH + 1) << 16)) : 0u;
        auto value = [&](int q) -> float {
            const float v = __fmul_rn(small_int_f32(q - OFF), d);
            return HAS_MIN ? __fadd_rn(v, mn) : v;
        };
        uint32_t lo[8], hi[8]; // elements 0..15 (low nibbles) and 16..31 (high nibbles)
#pragma unroll
        for (int t = 0; t < 8; t++) {
            const uint32_t two = __ldg(h + QS + t); // bytes 2t, 2t+1
            const int b0 = (int)(two & 0xFFu), b1 = (int)(two >> 8);
            const int f0 = (int)((qh >> (2 * t)) & 1u) << 4, f1 = (int)((qh >> (2 * t + 1)) & 1u) << 4;
            const int g0 = (int)((qh >> (16 + 2 * t)) & 1u) << 4, g1 = (int)((qh >> (17 + 2 * t)) & 1u) << 4;
            lo[t] = pack_bf16x2_rn(value((b0 & 15) | f0), value((b1 & 15) | f1));
            hi[t] = pack_bf16x2_rn(value((b0 >> 4) | g0), value((b1 >> 4) | g1));
        }
        uint4 *dst = reinterpret_cast<uint4 *>(out + idx * 32);
        dst[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        dst[1] = make_uint4(lo[4], lo[5], lo[6], lo[7]);
        dst[2] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        dst[3] = make_uint4(hi[4], hi[5], hi[6], hi[7]);
    }
}

// Q6_K: a thread takes the 16 weights that share one scale: super-block sb, half h, quad q, sixteen s.
__global__ void __launch_bounds__(256)
q6k_slab_bf16_kernel(const uint8_t *__restrict__ blocks, __nv_bfloat16 *__restrict__ out, size_t total_groups)
{
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_groups;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t sb = idx >> 4;
        const int grp = (int)(idx & 15), h = grp >> 3, q = (grp >> 1) & 3, s = grp & 1; // element 128h + 32q + 16s + i
        const uint8_t *blk = blocks + sb * 210;
        const unsigned short *ql = reinterpret_cast<const unsigned short *>(blk + 64 * h + 32 * (q & 1) + 16 * s);
        const unsigned short *qh = reinterpret_cast<const unsigned short *>(blk + 128 + 32 * h + 16 * s);
        const float d = __half2float(__ushort_as_half(__ldg(reinterpret_cast<const unsigned short *>(blk + 208))));
        const int sc = (int)(signed char)blk[192 + 8 * h + 2 * q + s];
        const float ds = __fmul_rn(d, small_int_f32(sc));
        uint32_t o[8];
#pragma unroll
        for (int t = 0; t < 8; t++) {
            const uint32_t l2 = __ldg(ql + t), h2 = __ldg(qh + t); // bytes for elements 2t, 2t+1
            const int n0 = (int)((l2 >> (q < 2 ? 0 : 4)) & 0x0Fu), n1 = (int)((l2 >> (q < 2 ? 8 : 12)) & 0x0Fu);
            const int b0 = (int)((h2 >> (2 * q)) & 3u), b1 = (int)((h2 >> (8 + 2 * q)) & 3u);
            o[t] = pack_bf16x2_rn(__fmul_rn(ds, small_int_f32((n0 | (b0 << 4)) - 32)),
                                  __fmul_rn(ds, small_int_f32((n1 | (b1 << 4)) - 32)));
        }
        uint4 *dst = reinterpret_cast<uint4 *>(out + sb * 256 + 128 * h + 32 * q + 16 * s);
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

// GPTQ 4-bit: a word holds 8 consecutive k of one out column, so a thread turns one word into 16
// contiguous output bytes. A CTA of 256 threads stages 32 word rows (256 k) x 32 out columns with
// coalesced loads along the columns, then reads them transposed: a warp owns 4 columns, its lanes
// walk the word rows, so every column is stored as 512 contiguous bytes. Arithmetic as in the
// element-wise kernel: (q - (zero + 1)) * scale in f32, one rounding. Needs group_size % 8 == 0.
__global__ void __launch_bounds__(256)
gptq4_slab_bf16_kernel(const uint32_t *__restrict__ qweight, const uint32_t *__restrict__ qzeros,
                       const void *__restrict__ scales, int scales_dtype, __nv_bfloat16 *__restrict__ out, int k,
                       int n_cnt, int group_size, int sym, int n_full, int n_off)
{
    __shared__ uint32_t tile[32][33];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int c0 = blockIdx.x * 32, kp0 = blockIdx.y * 32, kwords = k >> 3;
#pragma unroll
    for (int it = 0; it < 4; it++) {
        const int r = warp + 8 * it, kp = kp0 + r, col = c0 + lane;
        tile[r][lane] = (kp < kwords && col < n_cnt) ? __ldcs(qweight + (size_t)kp * n_full + n_off + col) : 0u;
    }
    __syncthreads();
    const int kp = kp0 + lane;
    if (kp >= kwords) return;
    const int g = (kp * 8) / group_size;
#pragma unroll
    for (int it = 0; it < 4; it++) {
        const int cl = warp * 4 + it, col = c0 + cl;
        if (col >= n_cnt) break;
        const int o = n_off + col;
        uint32_t zero = 7u;
        if (!sym) zero = (__ldg(qzeros + (size_t)g * (n_full >> 3) + (o >> 3)) >> ((o & 7) * 4)) & 15u;
        const float sc = load_as_f32(scales, scales_dtype, (size_t)g * n_full + o);
        const float zf = __uint_as_float(0x4B000000u | (zero + 1u)); // 2^23 + zero + 1
        const uint32_t w = tile[lane][cl];
        uint32_t o4[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float a = __uint_as_float(0x4B000000u | ((w >> (8 * j)) & 15u)) - zf;
            const float b = __uint_as_float(0x4B000000u | ((w >> (8 * j + 4)) & 15u)) - zf;
            o4[j] = pack_bf16x2_rn(__fmul_rn(a, sc), __fmul_rn(b, sc));
        }
        *reinterpret_cast<uint4 *>(out + (size_t)col * k + (size_t)kp * 8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
    }
}

static int grid_for(size_t work_items, int block = 256)
{
    size_t blocks = (work_items + block - 1) / block;
    const size_t cap = (size_t)sm_count() * 32; // a few waves of resident CTAs, then grid-stride
    return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

// ---- row-range (slab) dequantization to bf16 for the tensor-core GEMM -----------------------
// Rows [n_off, n_off + n_cnt) of the dense [n, k] weight into a contiguous [n_cnt, k] bf16 buffer.
int awq_dequant_rows_bf16(const uint32_t *qweight, const uint32_t *qzeros, const void *scales, int scales_dtype,
                          __nv_bfloat16 *out, int k, int n_full, int group_size, int n_off, int n_cnt, cudaStream_t st,
                          int row_mul, int row_add)
{
    OXQ_REQUIRE((row_mul == 1 && row_add == 0) ||
                    (group_size % 16 == 0 && k % 16 == 0 && n_off % 8 == 0 && n_cnt % 8 == 0 && aligned(out, 16)),
                OXQ_ERR_UNSUPPORTED, "strided-row dequantization needs group_size and in_features (%d, %d) multiples of 16 "
                "and column ranges in multiples of 8", group_size, k);
    if (group_size % 16 == 0 && k % 16 == 0 && n_off % 8 == 0 && n_cnt % 8 == 0 && aligned(out, 16)) {
        const int vec_ok = aligned(qweight, 16) && (n_full >> 3) % 4 == 0 && (n_off >> 3) % 4 == 0;
        dim3 grid(ceil_div(n_cnt, 256), ceil_div(k, 128));
        awq_slab16_bf16_kernel<<<grid, 256, 0, st>>>(qweight, qzeros, scales, scales_dtype, out, k, n_cnt, group_size,
                                                     n_full, n_off, vec_ok, row_mul, row_add);
        OXQ_LAUNCH_CHECK("awq_slab16_bf16_kernel");
        return OXQ_OK;
    }
    dim3 grid(ceil_div(n_cnt, 256), ceil_div(k, 64));
    awq_slab_bf16_kernel<<<grid, 256, 0, st>>>(qweight, qzeros, scales, scales_dtype, out, k, n_cnt, group_size,
                                               n_full, n_off);
    OXQ_LAUNCH_CHECK("awq_slab_bf16_kernel");
    return OXQ_OK;
}

int gptq_dequant_rows_bf16(const uint32_t *qweight, const uint32_t *qzeros, const void *scales, int scales_dtype,
                           __nv_bfloat16 *out, int k, int n_full, int group_size, int bits, int sym, int n_off,
                           int n_cnt, cudaStream_t st)
{
    if (bits == 4 && group_size % 8 == 0 && k % 8 == 0 && aligned(out, 16)) {
        dim3 grid(ceil_div(n_cnt, 32), ceil_div(k / 8, 32));
        gptq4_slab_bf16_kernel<<<grid, 256, 0, st>>>(qweight, qzeros, scales, scales_dtype, out, k, n_cnt, group_size, sym,
                                                     n_full, n_off);
        OXQ_LAUNCH_CHECK("gptq4_slab_bf16_kernel");
        return OXQ_OK;
    }
    gptq_dequant_kernel<__nv_bfloat16><<<grid_for((size_t)n_cnt * k), 256, 0, st>>>(
        qweight, qzeros, scales, scales_dtype, out, k, n_cnt, group_size, bits, sym, n_full, n_off);
    OXQ_LAUNCH_CHECK("gptq_dequant_kernel");
    return OXQ_OK;
}

int w8a16_dequant_rows_bf16(const uint32_t *qweight, const uint32_t *qzeros, const void *scales, int scales_dtype,
                            __nv_bfloat16 *out, int k, int n_full, int group_size, int n_off, int n_cnt, cudaStream_t st)
{
    w8a16_dequant_kernel<__nv_bfloat16><<<grid_for((size_t)n_cnt * k), 256, 0, st>>>(
        qweight, qzeros, scales, scales_dtype, out, k, n_cnt, group_size, n_full, n_off);
    OXQ_LAUNCH_CHECK("w8a16_dequant_kernel");
    return OXQ_OK;
}

int gguf_dequant_rows_bf16(int ggml_type, const uint8_t *blocks, __nv_bfloat16 *out, int k, int n_off, int n_cnt,
                           cudaStream_t st)
{
    int bel, bby;
    gguf_block_layout(ggml_type, bel, bby);
    const uint8_t *b = blocks + (size_t)n_off * (k / bel) * bby;
    const size_t total = (size_t)n_cnt * k;
    if ((ggml_type == OXQ_GGML_Q4_K || ggml_type == OXQ_GGML_Q5_K) && aligned(b, 16) && aligned(out, 16)) {
        const size_t groups = total / 64;
        if (ggml_type == OXQ_GGML_Q5_K) q4k_slab_bf16_kernel<true><<<grid_for(groups), 256, 0, st>>>(b, out, groups);
        else q4k_slab_bf16_kernel<false><<<grid_for(groups), 256, 0, st>>>(b, out, groups);
        OXQ_LAUNCH_CHECK("q4k_slab_bf16_kernel");
        return OXQ_OK;
    }
    if (aligned(b, 2) && aligned(out, 16) && ggml_type != OXQ_GGML_Q4_K && ggml_type != OXQ_GGML_Q5_K &&
        ggml_type != OXQ_GGML_Q2_K && ggml_type != OXQ_GGML_Q3_K) {
        const int g32 = grid_for(total / 32);
        if (ggml_type == OXQ_GGML_Q8_0) q80_slab_bf16_kernel<<<g32, 256, 0, st>>>(b, out, total / 32);
        else if (ggml_type == OXQ_GGML_Q4_0) q40_slab_bf16_kernel<0><<<g32, 256, 0, st>>>(b, out, total / 32);
        else if (ggml_type == OXQ_GGML_Q4_1) q40_slab_bf16_kernel<1><<<g32, 256, 0, st>>>(b, out, total / 32);
        else if (ggml_type == OXQ_GGML_Q5_0) q40_slab_bf16_kernel<2><<<g32, 256, 0, st>>>(b, out, total / 32);
        else if (ggml_type == OXQ_GGML_Q5_1) q40_slab_bf16_kernel<3><<<g32, 256, 0, st>>>(b, out, total / 32);
        else q6k_slab_bf16_kernel<<<grid_for(total / 16), 256, 0, st>>>(b, out, total / 16);
        OXQ_LAUNCH_CHECK("gguf slab kernel");
        return OXQ_OK;
    }
    const int grid = grid_for(total);
#define OXQ_GGUF_CASE(T) case T: gguf_dequant_kernel<T, __nv_bfloat16><<<grid, 256, 0, st>>>(b, out, total); break;
    switch (ggml_type) {
    OXQ_GGUF_CASE(OXQ_GGML_Q4_0) OXQ_GGUF_CASE(OXQ_GGML_Q8_0) OXQ_GGUF_CASE(OXQ_GGML_Q4_K) OXQ_GGUF_CASE(OXQ_GGML_Q4_1)
    OXQ_GGUF_CASE(OXQ_GGML_Q5_0) OXQ_GGUF_CASE(OXQ_GGML_Q5_1) OXQ_GGUF_CASE(OXQ_GGML_Q5_K)
    OXQ_GGUF_CASE(OXQ_GGML_Q2_K) OXQ_GGUF_CASE(OXQ_GGML_Q3_K)
    default: gguf_dequant_kernel<OXQ_GGML_Q6_K, __nv_bfloat16><<<grid, 256, 0, st>>>(b, out, total); break;
    }
#undef OXQ_GGUF_CASE
    OXQ_LAUNCH_CHECK("gguf_dequant_kernel");
    return OXQ_OK;
}

int fp8_dequant_rows_bf16(const uint8_t *weight, const float *scale_inv, int s_in, int block_out, int block_in,
                          __nv_bfloat16 *out, int k, int n_off, int n_cnt, cudaStream_t st)
{
    if (k % 16 == 0 && block_in % 16 == 0 && aligned(weight, 16) && aligned(out, 16)) {
        dim3 grid(ceil_div(k / 16, 256), ceil_div(n_cnt, FP8_SLAB_ROWS));
        fp8_slab16_bf16_kernel<<<grid, 256, 0, st>>>(weight + (size_t)n_off * k, scale_inv, s_in, block_out, block_in,
                                                     out, n_cnt, k, n_off);
        OXQ_LAUNCH_CHECK("fp8_slab16_bf16_kernel");
        return OXQ_OK;
    }
    fp8_dequant_kernel<__nv_bfloat16><<<grid_for((size_t)n_cnt * k / 4), 256, 0, st>>>(
        weight + (size_t)n_off * k, scale_inv, s_in, block_out, block_in, out, n_cnt, k, n_off);
    OXQ_LAUNCH_CHECK("fp8_dequant_kernel");
    return OXQ_OK;
}

bool gguf_block_layout_host(int ggml_type, int &bel, int &bby) { return gguf_block_layout(ggml_type, bel, bby); }

int mxfp4_dequant_rows_bf16(const uint8_t *blocks, const uint8_t *scales, __nv_bfloat16 *out, int k, int n_off,
                            int n_cnt, cudaStream_t st)
{
    const size_t total_bytes = (size_t)n_cnt * k / 2;
    if (k % 32 == 0 && aligned(blocks + (size_t)n_off * (k / 2), 16) && aligned(out, 16)) {
        const size_t total_blocks = total_bytes / 16;
        mxfp4_slab16_bf16_kernel<<<grid_for(total_blocks), 256, 0, st>>>(
            blocks + (size_t)n_off * (k / 2), scales + (size_t)n_off * (k / 32), out, total_blocks);
        OXQ_LAUNCH_CHECK("mxfp4_slab16_bf16_kernel");
        return OXQ_OK;
    }
    mxfp4_dequant_kernel<__nv_bfloat16><<<grid_for(total_bytes), 256, 0, st>>>(
        blocks + (size_t)n_off * (k / 2), scales + (size_t)n_off * (k / 32), out, total_bytes);
    OXQ_LAUNCH_CHECK("mxfp4_dequant_kernel");
    return OXQ_OK;
}

} // namespace oxq

using namespace oxq;

#define DISPATCH_OUT(dtype, ...)                                              \
    do {                                                                      \
        if ((dtype) == OXQ_F32) { using OutT = float; __VA_ARGS__; }          \
        else if ((dtype) == OXQ_F16) { using OutT = __half; __VA_ARGS__; }    \
        else { using OutT = __nv_bfloat16; __VA_ARGS__; }                     \
    } while (0)

OXQ_EXPORT int oxq_awq_dequant(const uint32_t *qweight, const uint32_t *qzeros, const void *scales, int scales_dtype,
                               void *w_out, int out_dtype, int k, int n, int group_size, void *stream)
{
    clear_error();
    OXQ_REQUIRE(qweight && qzeros && scales && w_out, OXQ_ERR_NULL, "oxq_awq_dequant: null pointer");
    OXQ_REQUIRE(valid_dtype(scales_dtype) && valid_dtype(out_dtype), OXQ_ERR_UNSUPPORTED,
                "oxq_awq_dequant: unsupported dtype");
    OXQ_REQUIRE(k > 0 && n > 0 && group_size > 0, OXQ_ERR_BAD_SHAPE, "oxq_awq_dequant: non-positive size");
    OXQ_REQUIRE(n % 8 == 0, OXQ_ERR_BAD_SHAPE, "AWQ out_features (%d) not divisible by pack factor 8", n);
    OXQ_REQUIRE(k % group_size == 0, OXQ_ERR_BAD_SHAPE,
                "quant in_features (%d) not divisible by group size (%d)", k, group_size);
    if (out_dtype == OXQ_BF16) // same bits, the fast producer of the tensor-core path
        return awq_dequant_rows_bf16(qweight, qzeros, scales, scales_dtype, (__nv_bfloat16 *)w_out, k, n, group_size, 0, n,
                                     (cudaStream_t)stream, 1, 0);
    dim3 grid(ceil_div(n / 8, 8), ceil_div(k, AWQ_TK));
    DISPATCH_OUT(out_dtype, awq_dequant_kernel<OutT><<<grid, 256, 0, (cudaStream_t)stream>>>(
                                qweight, qzeros, scales, scales_dtype, (OutT *)w_out, k, n, group_size, n, 0));
    OXQ_LAUNCH_CHECK("awq_dequant_kernel");
    return OXQ_OK;
}

OXQ_EXPORT int oxq_gptq_dequant(const uint32_t *qweight, const uint32_t *qzeros, const void *scales,
                                int scales_dtype, void *w_out, int out_dtype, int k, int n, int group_size, int bits,
                                int sym, void *stream)
{
    clear_error();
    OXQ_REQUIRE(qweight && scales && w_out, OXQ_ERR_NULL, "oxq_gptq_dequant: null pointer");
    OXQ_REQUIRE(valid_dtype(scales_dtype) && valid_dtype(out_dtype), OXQ_ERR_UNSUPPORTED,
                "oxq_gptq_dequant: unsupported dtype");
    OXQ_REQUIRE(bits == 4 || bits == 8, OXQ_ERR_UNSUPPORTED, "dequantize_gptq: only 4/8-bit supported, got %d", bits);
    OXQ_REQUIRE(k > 0 && n > 0 && group_size > 0, OXQ_ERR_BAD_SHAPE, "oxq_gptq_dequant: non-positive size");
    const int pf = 32 / bits;
    OXQ_REQUIRE(n % pf == 0, OXQ_ERR_BAD_SHAPE, "GPTQ out_features %d not divisible by pack_factor %d", n, pf);
    OXQ_REQUIRE(k % pf == 0 && k % group_size == 0, OXQ_ERR_BAD_SHAPE,
                "GPTQ in_features %d not divisible by pack_factor %d / group size %d", k, pf, group_size);
    const int use_sym = (sym != 0 || qzeros == nullptr) ? 1 : 0;
    if (out_dtype == OXQ_BF16) // same bits; 4-bit takes the fast producer of the tensor-core path
        return gptq_dequant_rows_bf16(qweight, qzeros, scales, scales_dtype, (__nv_bfloat16 *)w_out, k, n, group_size, bits,
                                      use_sym, 0, n, (cudaStream_t)stream);
    DISPATCH_OUT(out_dtype, gptq_dequant_kernel<OutT><<<grid_for((size_t)n * k), 256, 0, (cudaStream_t)stream>>>(
                                qweight, qzeros, scales, scales_dtype, (OutT *)w_out, k, n, group_size, bits, use_sym, n, 0));
    OXQ_LAUNCH_CHECK("gptq_dequant_kernel");
    return OXQ_OK;
}

OXQ_EXPORT int oxq_w8a16_dequant(const uint32_t *qweight, const uint32_t *qzeros, const void *scales, int scales_dtype,
                                 void *w_out, int out_dtype, int k, int n, int group_size, void *stream)
{
    clear_error();
    OXQ_REQUIRE(qweight && qzeros && scales && w_out, OXQ_ERR_NULL, "oxq_w8a16_dequant: null pointer");
    OXQ_REQUIRE(valid_dtype(scales_dtype) && valid_dtype(out_dtype), OXQ_ERR_UNSUPPORTED, "oxq_w8a16_dequant: unsupported dtype");
    OXQ_REQUIRE(k > 0 && n > 0 && group_size > 0, OXQ_ERR_BAD_SHAPE, "oxq_w8a16_dequant: non-positive size");
    OXQ_REQUIRE(n % 4 == 0, OXQ_ERR_BAD_SHAPE, "W8A16 out_features (%d) not divisible by pack factor 4", n);
    OXQ_REQUIRE(k % group_size == 0, OXQ_ERR_BAD_SHAPE, "quant in_features (%d) not divisible by group size (%d)", k, group_size);
    DISPATCH_OUT(out_dtype, w8a16_dequant_kernel<OutT><<<grid_for((size_t)n * k), 256, 0, (cudaStream_t)stream>>>(
                                qweight, qzeros, scales, scales_dtype, (OutT *)w_out, k, n, group_size, n, 0));
    OXQ_LAUNCH_CHECK("w8a16_dequant_kernel");
    return OXQ_OK;
}

OXQ_EXPORT int oxq_gguf_dequant(int ggml_type, const void *blocks, void *w_out, int out_dtype, int n, int k,
                                void *stream)
{
    clear_error();
    OXQ_REQUIRE(blocks && w_out, OXQ_ERR_NULL, "oxq_gguf_dequant: null pointer");
    OXQ_REQUIRE(valid_dtype(out_dtype), OXQ_ERR_UNSUPPORTED, "oxq_gguf_dequant: unsupported out dtype");
    int bel, bby;
    OXQ_REQUIRE(gguf_block_layout(ggml_type, bel, bby), OXQ_ERR_UNSUPPORTED, "unsupported GGML type %d", ggml_type);
    OXQ_REQUIRE(n > 0 && k > 0 && k % bel == 0, OXQ_ERR_BAD_SHAPE,
                "GGUF in_features %d is not a multiple of the block size %d", k, bel);
    OXQ_REQUIRE(aligned(blocks, 2), OXQ_ERR_BAD_ALIGN, "GGUF blocks must be 2-byte aligned");
    const size_t total = (size_t)n * k;
    const uint8_t *b = (const uint8_t *)blocks;
    cudaStream_t st = (cudaStream_t)stream;
    if (out_dtype == OXQ_BF16) // same bits; Q4_K takes the fast producer of the tensor-core path
        return gguf_dequant_rows_bf16(ggml_type, b, (__nv_bfloat16 *)w_out, k, 0, n, st);
    const int grid = grid_for(total);
#define OXQ_GGUF_CASE(T)                                                                                            \
    case T:                                                                                                         \
        DISPATCH_OUT(out_dtype, gguf_dequant_kernel<T, OutT><<<grid, 256, 0, st>>>(b, (OutT *)w_out, total));       \
        break;
    switch (ggml_type) {
    OXQ_GGUF_CASE(OXQ_GGML_Q4_0) OXQ_GGUF_CASE(OXQ_GGML_Q8_0) OXQ_GGUF_CASE(OXQ_GGML_Q4_K) OXQ_GGUF_CASE(OXQ_GGML_Q4_1)
    OXQ_GGUF_CASE(OXQ_GGML_Q5_0) OXQ_GGUF_CASE(OXQ_GGML_Q5_1) OXQ_GGUF_CASE(OXQ_GGML_Q5_K)
    OXQ_GGUF_CASE(OXQ_GGML_Q2_K) OXQ_GGUF_CASE(OXQ_GGML_Q3_K)
    default:
        DISPATCH_OUT(out_dtype, gguf_dequant_kernel<OXQ_GGML_Q6_K, OutT><<<grid, 256, 0, st>>>(b, (OutT *)w_out, total));
        break;
    }
#undef OXQ_GGUF_CASE
    OXQ_LAUNCH_CHECK("gguf_dequant_kernel");
    return OXQ_OK;
}

OXQ_EXPORT int oxq_fp8_dequant(const uint8_t *weight, const float *scale_inv, int s_out, int s_in, void *w_out,
                               int out_dtype, int n, int k, void *stream)
{
    clear_error();
    OXQ_REQUIRE(weight && w_out, OXQ_ERR_NULL, "oxq_fp8_dequant: null pointer");
    OXQ_REQUIRE(valid_dtype(out_dtype), OXQ_ERR_UNSUPPORTED, "oxq_fp8_dequant: unsupported out dtype");
    OXQ_REQUIRE(n > 0 && k > 0 && k % 4 == 0, OXQ_ERR_BAD_SHAPE, "FP8 weight [%d, %d]: in_features must be a multiple of 4",
                n, k);
    OXQ_REQUIRE(aligned(weight, 4), OXQ_ERR_BAD_ALIGN, "FP8 weight must be 4-byte aligned");
    int bo = n, bi = k;
    if (scale_inv) {
        OXQ_REQUIRE(s_out > 0 && s_in > 0 && n % s_out == 0 && k % s_in == 0, OXQ_ERR_BAD_SHAPE,
                    "block-wise FP8 weight_scale_inv [%d, %d] does not tile weight [%d, %d] evenly", s_out, s_in, n, k);
        bo = n / s_out;
        bi = k / s_in;
    }
    if (out_dtype == OXQ_BF16) // same bits, the fast producer of the tensor-core path
        return fp8_dequant_rows_bf16(weight, scale_inv, scale_inv ? s_in : 1, bo, bi, (__nv_bfloat16 *)w_out, k, 0, n,
                                     (cudaStream_t)stream);
    DISPATCH_OUT(out_dtype, fp8_dequant_kernel<OutT><<<grid_for((size_t)n * k / 4), 256, 0, (cudaStream_t)stream>>>(
                                weight, scale_inv, s_in, bo, bi, (OutT *)w_out, n, k, 0));
    OXQ_LAUNCH_CHECK("fp8_dequant_kernel");
    return OXQ_OK;
}

OXQ_EXPORT int oxq_mxfp4_dequant(const uint8_t *blocks, const uint8_t *scales, void *w_out, int out_dtype, int n,
                                 int k, void *stream)
{
    clear_error();
    OXQ_REQUIRE(blocks && scales && w_out, OXQ_ERR_NULL, "oxq_mxfp4_dequant: null pointer");
    OXQ_REQUIRE(valid_dtype(out_dtype), OXQ_ERR_UNSUPPORTED, "oxq_mxfp4_dequant: unsupported out dtype");
    OXQ_REQUIRE(n > 0 && k > 0 && k % 32 == 0, OXQ_ERR_BAD_SHAPE, "MXFP4: cols %d must be a multiple of 32", k);
    if (out_dtype == OXQ_BF16) // same bits, the fast producer of the tensor-core path
        return mxfp4_dequant_rows_bf16(blocks, scales, (__nv_bfloat16 *)w_out, k, 0, n, (cudaStream_t)stream);
    const size_t total_bytes = (size_t)n * k / 2;
    DISPATCH_OUT(out_dtype, mxfp4_dequant_kernel<OutT><<<grid_for(total_bytes), 256, 0, (cudaStream_t)stream>>>(
                                blocks, scales, (OutT *)w_out, total_bytes));
    OXQ_LAUNCH_CHECK("mxfp4_dequant_kernel");
    return OXQ_OK;
}
