/*
 * CPU oracle for the quantized-weight matrix-product path of oxydLLM.
 *
 * TEST INFRASTRUCTURE ONLY. This file is a plain-C restatement of the
 * reference's own CPU algorithms (Rust sources, cited per function by
 * file:line inside the reference project). It is the checker that the CUDA
 * kernels are compared against and the timed "port" CPU baseline; nothing in
 * the shipped library links against it or falls back to it.
 *
 * Parity pin: the reference is Rust on the candle crate and cannot be built
 * where this oracle is developed (no cargo/rustc, candle sources not
 * vendored), so the oracle is pinned by replaying every CPU known-answer test
 * the reference holds for this path (AWQ/GPTQ dequant, FP8 scale grids,
 * E4M3 byte decode, MXFP4 code table and manual dot, GPT-OSS expert scalar
 * reference) and, for the GGUF block formats whose arithmetic lives in the
 * un-vendored candle crate, by the reference's own per-element shader strips
 * cross-checked bit-for-bit against the independent gguf-py dequantizer.
 * The candle Q4_K/Q6_K *quantizer* and candle's CPU int8-activation QMatMul
 * are "parity unpinned": they are absent from the reference tree.
 *
 * Build: gcc -O3 -fopenmp -shared -fPIC oracle.c -o liboracle.so -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------- helpers */

static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* IEEE binary16 -> binary32, exact (what `half::f16::to_f32` does). */
static inline float f16_to_f32(uint16_t h)
{
    uint32_t s = (uint32_t)(h >> 15) << 31;
    uint32_t e = (h >> 10) & 0x1F;
    uint32_t m = h & 0x3FF;
    if (e == 0) {
        if (m == 0) return bits_f32(s);
        /* subnormal: m * 2^-24 */
        float v = (float)m * 5.9604644775390625e-8f;
        return s ? -v : v;
    }
    if (e == 31) return bits_f32(s | 0x7F800000u | (m << 13));
    return bits_f32(s | ((e + 112) << 23) | (m << 13));
}

/* binary32 -> bfloat16, round-to-nearest-even; NaN keeps its sign and sets
 * the quiet bit (the `half` crate's `bf16::from_f32`, used by the reference's
 * dequantizers for DType::BF16 outputs, awq.rs:425-429). */
static inline uint16_t f32_to_bf16(float f)
{
    uint32_t x = f32_bits(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x0040u);
    uint32_t round_bit = 0x00008000u;
    if ((x & round_bit) != 0 && (x & (3 * round_bit - 1)) != 0) return (uint16_t)((x >> 16) + 1);
    return (uint16_t)(x >> 16);
}

/* binary32 -> binary16, round-to-nearest-even (`half::f16::from_f32`). */
static inline uint16_t f32_to_f16(float f)
{
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax > 0x7F800000u) return (uint16_t)(sign | 0x7E00u | ((ax >> 13) & 0x3FFu));
    if (ax == 0x7F800000u) return (uint16_t)(sign | 0x7C00u);
    int32_t exp = (int32_t)(ax >> 23) - 127;
    uint32_t man = ax & 0x7FFFFFu;
    if (exp > 15) return (uint16_t)(sign | 0x7C00u);
    if (exp >= -14) {
        uint32_t half_exp = (uint32_t)(exp + 15) << 10;
        uint32_t half_man = man >> 13;
        uint32_t rem = man & 0x1FFFu;
        uint32_t h = half_exp | half_man;
        if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) h += 1; /* may carry into exp: still right */
        return (uint16_t)(sign | h);
    }
    if (exp < -25) return (uint16_t)sign;
    /* subnormal half */
    man |= 0x800000u;
    uint32_t shift = (uint32_t)(-14 - exp) + 13;
    uint32_t half_man = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_man & 1))) half_man += 1;
    return (uint16_t)(sign | half_man);
}

ORC_API void orc_f32_to_bf16(const float *in, uint16_t *out, int64_t n)
{
    for (int64_t i = 0; i < n; i++) out[i] = f32_to_bf16(in[i]);
}

ORC_API void orc_f32_to_f16(const float *in, uint16_t *out, int64_t n)
{
    for (int64_t i = 0; i < n; i++) out[i] = f32_to_f16(in[i]);
}

ORC_API void orc_f16_to_f32(const uint16_t *in, float *out, int64_t n)
{
    for (int64_t i = 0; i < n; i++) out[i] = f16_to_f32(in[i]);
}

ORC_API void orc_bf16_to_f32(const uint16_t *in, float *out, int64_t n)
{
    for (int64_t i = 0; i < n; i++) out[i] = bits_f32((uint32_t)in[i] << 16);
}

/* ------------------------------------------------------------------- AWQ */

/* Slot k of a packed word holds out column 8*j + ORDER[k] (awq.rs:23-24). */
static const int AWQ_PACK_ORDER[8] = {0, 2, 4, 6, 1, 3, 5, 7};

/*
 * AWQ 4-bit dequantization to a dense [out, in] f32 matrix.
 * Follows dequantize_awq (awq.rs:325-440): zero points are first unpacked to
 * one byte per (group, out) (awq.rs:391-401), then fill_awq_weight
 * (awq.rs:612-633) writes W[o][i] = (nibble - zero) as f32 * scale.
 * `scales` arrives already widened to f32 from its stored dtype with no
 * pre-rounding (awq.rs:362-367). Returns 0, or -1 on a shape the reference
 * rejects (awq.rs:332-358).
 */
ORC_API int orc_awq_dequant_f32(const uint32_t *qweight, const uint32_t *qzeros, const float *scales,
                                int64_t in_features, int64_t out_features, int64_t group_size, float *w_out)
{
    if (out_features % 8 != 0 || group_size <= 0 || in_features % group_size != 0) return -1;
    int64_t groups = in_features / group_size;
    int64_t packed_out = out_features / 8;
    uint8_t *zeros = (uint8_t *)malloc((size_t)(groups * out_features));
    if (!zeros) return -2;
    for (int64_t g = 0; g < groups; g++)
        for (int64_t j = 0; j < packed_out; j++) {
            uint32_t packed = qzeros[g * packed_out + j];
            for (int k = 0; k < 8; k++)
                zeros[g * out_features + j * 8 + AWQ_PACK_ORDER[k]] = (uint8_t)((packed >> (4 * k)) & 0xF);
        }
    int inv_order[8];
    for (int k = 0; k < 8; k++) inv_order[AWQ_PACK_ORDER[k]] = k;

#pragma omp parallel for schedule(static)
    for (int64_t o = 0; o < out_features; o++) {
        int64_t j = o / 8;
        int shift = 4 * inv_order[o % 8];
        float *row = w_out + o * in_features;
        for (int64_t i = 0; i < in_features; i++) {
            int64_t g = i / group_size;
            int32_t nibble = (int32_t)((qweight[i * packed_out + j] >> shift) & 0xF);
            int32_t zero = zeros[g * out_features + o];
            row[i] = (float)(nibble - zero) * scales[g * out_features + o];
        }
    }
    free(zeros);
    return 0;
}

/* ------------------------------------------------------------------ GPTQ */

/*
 * GPTQ 4/8-bit dequantization to [out, in] f32; fill_gptq_weight
 * (awq.rs:561-590). qweight [in/pf, out] packs sequentially LSB-first along
 * in; qzeros [groups, out/pf] packs along out and stores zero-1; with `sym`
 * (or no qzeros, awq.rs:540) the zero is 2^(bits-1) - 1 before the +1.
 */
ORC_API int orc_gptq_dequant_f32(const uint32_t *qweight, const uint32_t *qzeros, const float *scales,
                                 int64_t in_features, int64_t out_features, int64_t group_size, int bits, int sym,
                                 float *w_out)
{
    if (bits != 4 && bits != 8) return -1;
    int64_t pf = 32 / bits;
    if (out_features % pf != 0 || in_features % pf != 0 || group_size <= 0 || in_features % group_size != 0)
        return -1;
    int64_t packed_out = out_features / pf;
    uint32_t mask = (1u << bits) - 1;
    uint32_t sym_zero = (1u << (bits - 1)) - 1;
    int use_sym = sym || qzeros == NULL;
#pragma omp parallel for schedule(static)
    for (int64_t o = 0; o < out_features; o++) {
        int64_t o_word = o / pf;
        uint32_t o_shift = (uint32_t)((o % pf) * bits);
        float *row = w_out + o * in_features;
        for (int64_t i = 0; i < in_features; i++) {
            int64_t g = i / group_size;
            uint32_t i_shift = (uint32_t)((i % pf) * bits);
            uint32_t q = (qweight[(i / pf) * out_features + o] >> i_shift) & mask;
            uint32_t zero = use_sym ? sym_zero : ((qzeros[g * packed_out + o_word] >> o_shift) & mask);
            row[i] = (float)((int32_t)q - ((int32_t)zero + 1)) * scales[g * out_features + o];
        }
    }
    return 0;
}

/* W8A16: the AWQ layout at 8 bits, as the reference's shader source states it (quant_kernels.metal:1-16:
 * qweight u32 [in, out / 4], slot c of word j = out column 4 j + c, identity order at 8 bits;
 * unpack (:40-48); W[o][i] = (q - zero) * scale[group(i)][o]). The reference has no CPU code for it. */
ORC_API int orc_w8a16_dequant_f32(const uint32_t *qweight, const uint32_t *qzeros, const float *scales,
                                  int64_t in_features, int64_t out_features, int64_t group_size, float *w_out)
{
    if (out_features % 4 != 0 || group_size <= 0 || in_features % group_size != 0) return -1;
    int64_t packed_out = out_features / 4;
#pragma omp parallel for schedule(static)
    for (int64_t o = 0; o < out_features; o++) {
        uint32_t sh = (uint32_t)((o % 4) * 8);
        float *row = w_out + o * in_features;
        for (int64_t i = 0; i < in_features; i++) {
            int64_t g = i / group_size;
            int32_t q = (int32_t)((qweight[i * packed_out + o / 4] >> sh) & 0xFFu);
            int32_t z = (int32_t)((qzeros[g * packed_out + o / 4] >> sh) & 0xFFu);
            row[i] = (float)(q - z) * scales[g * out_features + o];
        }
    }
    return 0;
}

/* ------------------------------------------------------------------- FP8 */

/* One E4M3fn byte per the spec decode the reference pins every encoding
 * against (metal_ops.rs:2944-2956): 1-4-3, bias 7, e=0 subnormal,
 * S.1111.111 NaN, no infinities. */
static inline float e4m3_decode(uint8_t v)
{
    uint32_t s = v >> 7, e = (v >> 3) & 0xF, m = v & 0x7;
    float val;
    if (e == 0) val = (float)m * 0.125f * 0.015625f;
    else if (e == 15 && m == 7) val = NAN;
    else val = (1.0f + (float)m * 0.125f) * ldexpf(1.0f, (int)e - 7);
    return s ? -val : val;
}

ORC_API void orc_e4m3_decode(const uint8_t *in, float *out, int64_t n)
{
    for (int64_t i = 0; i < n; i++) out[i] = e4m3_decode(in[i]);
}

/*
 * FP8 weight [out, in] bytes times an f32 scale grid [s_out, s_in] tiled
 * evenly over the weight: W_f32 = f32(e4m3) * scale[r / (out/s_out)][c /
 * (in/s_in)]. Restates Fp8Linear::forward's dequant (linear.rs:96-141) with
 * apply_scale_inv's grid expansion (weights.rs:207-234). Rank-1 per-row and
 * scalar scales are the s_in == 1 / s_out == s_in == 1 cases of the same
 * grid (linear.rs:115-131). Returns -1 when the grid does not tile evenly
 * (weights.rs:220-225).
 */
ORC_API int orc_fp8_block_dequant_f32(const uint8_t *w, const float *scale, int64_t out_features,
                                      int64_t in_features, int64_t s_out, int64_t s_in, float *w_out)
{
    if (s_out <= 0 || s_in <= 0 || out_features % s_out != 0 || in_features % s_in != 0) return -1;
    int64_t bo = out_features / s_out, bi = in_features / s_in;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < out_features; r++)
        for (int64_t c = 0; c < in_features; c++)
            w_out[r * in_features + c] = scale[(r / bo) * s_in + (c / bi)] * e4m3_decode(w[r * in_features + c]);
    return 0;
}

/* ----------------------------------------------------------------- MXFP4 */

static const float MXFP4_LUT[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

static inline float mxfp4_decode(uint8_t nib)
{
    float v = MXFP4_LUT[nib & 7];
    return (nib & 8) ? -v : v;
}

static inline float e8m0_scale(uint8_t s) { return s == 0xFF ? NAN : exp2f((float)s - 127.0f); }

/* dequantize_mxfp4_f32 (mxfp4.rs:35-64): blocks u8 [rows, K/32, 16] low
 * nibble first, scales u8 [rows, K/32] = 2^(s-127), 0xFF -> NaN
 * (mxfp4.rs:13-31). */
ORC_API int orc_mxfp4_dequant_f32(const uint8_t *blocks, const uint8_t *scales, int64_t rows, int64_t cols,
                                  float *w_out)
{
    if (cols % 32 != 0) return -1;
    int64_t nb = cols / 32;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++)
        for (int64_t b = 0; b < nb; b++) {
            float scale = e8m0_scale(scales[r * nb + b]);
            const uint8_t *bytes = blocks + (r * nb + b) * 16;
            float *o = w_out + r * cols + b * 32;
            for (int t = 0; t < 16; t++) {
                o[2 * t] = mxfp4_decode(bytes[t] & 0xF) * scale;
                o[2 * t + 1] = mxfp4_decode(bytes[t] >> 4) * scale;
            }
        }
    return 0;
}

/* ------------------------------------------------------------------ GGUF */

/* GGML type ids as stored in GGUF files. */
enum { ORC_Q4_0 = 2, ORC_Q4_1 = 3, ORC_Q5_0 = 6, ORC_Q5_1 = 7, ORC_Q8_0 = 8, ORC_Q2_K = 10, ORC_Q3_K = 11, ORC_Q4_K = 12, ORC_Q5_K = 13,
       ORC_Q6_K = 14 };

static inline uint16_t ld16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* Sub-block scale/min from the 12 packed bytes (quant_kernels.metal:2438-2450). */
static inline void q4k_scale_min(int j, const uint8_t *q, uint32_t *d, uint32_t *m)
{
    if (j < 4) {
        *d = q[j] & 63u;
        *m = q[j + 4] & 63u;
    } else {
        *d = (q[j + 4] & 0x0Fu) | ((uint32_t)(q[j - 4] >> 6) << 4);
        *m = ((uint32_t)q[j + 4] >> 4) | ((uint32_t)(q[j] >> 6) << 4);
    }
}

/* Keep every product/sum a separately rounded f32 operation, in the order the
 * reference's strips write them; `volatile` stops gcc from contracting a*b-c
 * into one fused multiply-add. */
static inline float mul_rn(float a, float b) { volatile float r = a * b; return r; }
static inline float sub_rn(float a, float b) { volatile float r = a - b; return r; }
static inline float add_rn(float a, float b) { volatile float r = a + b; return r; }

/*
 * Per-element GGUF block dequantization to [rows, cols] f32. The block
 * arithmetic lives in the un-vendored candle crate, so this follows the
 * reference's own per-element strips (plain C arithmetic in its shader
 * source): Q4_0 quant_kernels.metal:2364-2384 (block :792-795), Q8_0
 * :2342-2361 (block :1100-1103), Q4_K :2452-2482 (block :1228-1233), Q6_K
 * :2518-2554 (block :1681-1686). The final bf16 narrowing those strips apply
 * is left to the caller so that f32 and bf16 outputs share one code path.
 */
ORC_API int orc_gguf_dequant_f32(int ggml_type, const uint8_t *data, int64_t rows, int64_t cols, float *w_out)
{
    int64_t bel, bby;
    switch (ggml_type) {
    case ORC_Q4_0: bel = 32; bby = 18; break;
    case ORC_Q8_0: bel = 32; bby = 34; break;
    case ORC_Q4_K: bel = 256; bby = 144; break;
    case ORC_Q6_K: bel = 256; bby = 210; break;
    case ORC_Q4_1: bel = 32; bby = 20; break;
    case ORC_Q5_0: bel = 32; bby = 22; break;
    case ORC_Q5_1: bel = 32; bby = 24; break;
    case ORC_Q5_K: bel = 256; bby = 176; break;
    case ORC_Q2_K: bel = 256; bby = 84; break;
    case ORC_Q3_K: bel = 256; bby = 110; break;
    default: return -3;
    }
    if (cols % bel != 0) return -1;
    int64_t nb = cols / bel;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++) {
        for (int64_t b = 0; b < nb; b++) {
            const uint8_t *blk = data + (r * nb + b) * bby;
            float *o = w_out + r * cols + b * bel;
            if (ggml_type == ORC_Q4_0) {
                float d = f16_to_f32(ld16(blk));
                const uint8_t *qs = blk + 2;
                for (int j = 0; j < 32; j++) {
                    int hi = j / 16, jj = j % 16;
                    int q = (hi == 0 ? (qs[jj] & 0x0F) : (qs[jj] >> 4)) - 8;
                    o[j] = mul_rn((float)q, d);
                }
            } else if (ggml_type == ORC_Q8_0) {
                float d = f16_to_f32(ld16(blk));
                const int8_t *qs = (const int8_t *)(blk + 2);
                for (int j = 0; j < 32; j++) o[j] = mul_rn((float)qs[j], d);
            } else if (ggml_type == ORC_Q4_K) {
                float d = f16_to_f32(ld16(blk)), dmin = f16_to_f32(ld16(blk + 2));
                const uint8_t *sc = blk + 4, *qs = blk + 16;
                for (int j = 0; j < 256; j++) {
                    int sub = j / 32, el = j % 32;
                    uint32_t scb, mb;
                    q4k_scale_min(sub, sc, &scb, &mb);
                    float sc_v = mul_rn(d, (float)scb), m_v = mul_rn(dmin, (float)mb);
                    int iq = sub / 2, lo = sub % 2;
                    uint32_t nib = lo == 0 ? (qs[iq * 32 + el] & 0x0Fu) : (uint32_t)(qs[iq * 32 + el] >> 4);
                    o[j] = sub_rn(mul_rn(sc_v, (float)nib), m_v);
                }
            } else if (ggml_type == ORC_Q4_1) {
                /* {f16 d; f16 m; u8 qs[16]}: q * d + m (quant_kernels.metal:2386-2408) */
                float d = f16_to_f32(ld16(blk)), mn = f16_to_f32(ld16(blk + 2));
                const uint8_t *qs = blk + 4;
                for (int j = 0; j < 32; j++) {
                    int hi = j / 16, jj = j % 16;
                    uint32_t q = hi == 0 ? (qs[jj] & 0x0Fu) : (uint32_t)(qs[jj] >> 4);
                    o[j] = add_rn(mul_rn((float)q, d), mn);
                }
            } else if (ggml_type == ORC_Q5_0 || ggml_type == ORC_Q5_1) {
                /* {f16 d; [f16 m;] u8 qh[4]; u8 qs[16]}: fifth bit of element j is bit j of qh
                 * (quant_kernels.metal:2315-2341, 2410-2437): (q - 16) * d, or q * d + m */
                const int with_min = ggml_type == ORC_Q5_1;
                float d = f16_to_f32(ld16(blk)), mn = with_min ? f16_to_f32(ld16(blk + 2)) : 0.0f;
                const uint8_t *qhb = blk + (with_min ? 4 : 2), *qs = qhb + 4;
                uint32_t qh = (uint32_t)qhb[0] | ((uint32_t)qhb[1] << 8) | ((uint32_t)qhb[2] << 16) | ((uint32_t)qhb[3] << 24);
                for (int j = 0; j < 32; j++) {
                    int hi = j / 16, jj = j % 16;
                    uint32_t xh = ((qh >> (jj + hi * 16)) & 1u) << 4;
                    uint32_t q = (hi == 0 ? (qs[jj] & 0x0Fu) : (uint32_t)(qs[jj] >> 4)) | xh;
                    o[j] = with_min ? add_rn(mul_rn((float)q, d), mn) : mul_rn((float)((int)q - 16), d);
                }
            } else if (ggml_type == ORC_Q5_K) {
                /* {f16 d, dmin; u8 scales[12]; u8 qh[32]; u8 qs[128]} (block_q5_K, quant_kernels.metal:1438-1445):
                 * Q4_K with a fifth bit: sub-block j takes bit j of qh[el]; (d*sc)*q - dmin*mn */
                float d = f16_to_f32(ld16(blk)), dmin = f16_to_f32(ld16(blk + 2));
                const uint8_t *sc = blk + 4, *qh = blk + 16, *qs = blk + 48;
                for (int j = 0; j < 256; j++) {
                    int sub = j / 32, el = j % 32;
                    uint32_t scb, mb;
                    q4k_scale_min(sub, sc, &scb, &mb);
                    float sc_v = mul_rn(d, (float)scb), m_v = mul_rn(dmin, (float)mb);
                    int iq = sub / 2, lo = sub % 2;
                    uint32_t nib = lo == 0 ? (qs[iq * 32 + el] & 0x0Fu) : (uint32_t)(qs[iq * 32 + el] >> 4);
                    uint32_t q = nib | (((uint32_t)(qh[el] >> sub) & 1u) << 4);
                    o[j] = sub_rn(mul_rn(sc_v, (float)q), m_v);
                }
            } else if (ggml_type == ORC_Q2_K) {
                /* {u8 scales[16]; u8 qs[64]; f16 d, dmin} (block_q2_K; the README lists Q2_K among the supported
                 * quants, the arithmetic is ggml's dequantize_row_q2_K as candle's k_quants restates it): sixteen
                 * sub-blocks of 16, scale nibble and min nibble per sub-block, (d*sc)*q - dmin*mn */
                const uint8_t *sc = blk, *qs = blk + 16;
                float d = f16_to_f32(ld16(blk + 80)), dmin = f16_to_f32(ld16(blk + 82));
                for (int j = 0; j < 256; j++) {
                    float dl = mul_rn(d, (float)(sc[j / 16] & 0x0Fu)), ml = mul_rn(dmin, (float)(sc[j / 16] >> 4));
                    uint32_t q = ((uint32_t)qs[(j / 128) * 32 + j % 32] >> (2 * ((j / 32) % 4))) & 3u;
                    o[j] = sub_rn(mul_rn(dl, (float)q), ml);
                }
            } else if (ggml_type == ORC_Q3_K) {
                /* {u8 hmask[32]; u8 qs[64]; u8 scales[12]; f16 d} (block_q3_K, dequantize_row_q3_K): sixteen 6-bit
                 * scales (low nibbles of bytes 0..7, then their high nibbles; two more bits each from bytes 8..11),
                 * (d*(scale-32)) * (two-bit - (hmask bit ? 0 : 4)) */
                const uint8_t *hm = blk, *qs = blk + 32, *scb = blk + 96;
                float d = f16_to_f32(ld16(blk + 108));
                for (int j = 0; j < 256; j++) {
                    int is = j / 16;
                    uint32_t lo4 = is < 8 ? (scb[is] & 0x0Fu) : (uint32_t)(scb[is - 8] >> 4);
                    uint32_t hi2 = ((uint32_t)scb[8 + is % 4] >> (2 * (is / 4))) & 3u;
                    float dl = mul_rn(d, (float)((int)(lo4 | (hi2 << 4)) - 32));
                    int q2 = (int)(((uint32_t)qs[(j / 128) * 32 + j % 32] >> (2 * ((j / 32) % 4))) & 3u);
                    int hb = (hm[j % 32] >> (j / 32)) & 1;
                    o[j] = mul_rn(dl, (float)(q2 - (hb ? 0 : 4)));
                }
            } else { /* Q6_K */
                const uint8_t *ql = blk, *qh = blk + 128;
                const int8_t *sc = (const int8_t *)(blk + 192);
                float d = f16_to_f32(ld16(blk + 208));
                for (int j = 0; j < 256; j++) {
                    int half_i = j / 128, pos = j % 128, quad = pos / 32, l = pos % 32;
                    const uint8_t *qlb = ql + 64 * half_i, *qhb = qh + 32 * half_i;
                    int ql_idx = (quad & 1) ? l + 32 : l;
                    int sh_ql = quad < 2 ? 0 : 4, sh_qh = 2 * quad;
                    uint32_t nib = (qlb[ql_idx] >> sh_ql) & 0x0Fu;
                    uint32_t hb = (qhb[l] >> sh_qh) & 0x03u;
                    int qv = (int)(nib | (hb << 4)) - 32;
                    float sc_v = mul_rn(d, (float)sc[8 * half_i + 2 * quad + l / 16]);
                    o[j] = mul_rn(sc_v, (float)qv);
                }
            }
        }
    }
    return 0;
}

/* ---------------------------------------------------------------- matmul */

/* The inner product is compiled once per ISA level and picked at load time,
 * so one binary runs on whatever host CPU it lands on. */
__attribute__((target_clones("default", "avx2", "avx512f")))
static float dot_f32(const float *a, const float *b, int64_t n)
{
    float acc[16] = {0};
    int64_t i = 0;
    for (; i + 16 <= n; i += 16)
        for (int t = 0; t < 16; t++) acc[t] += a[i + t] * b[i + t];
    float s = 0.0f;
    for (int t = 0; t < 16; t++) s += acc[t];
    for (; i < n; i++) s += a[i] * b[i];
    return s;
}

/*
 * y[m, n] = sum_k x[m, k] * w[n, k] (+ bias[n]) in f32: the reference's dense
 * Linear on the CPU device, x.matmul(W^T) then broadcast_add(bias)
 * (linear.rs:40-68), which is what every non-Metal quantized variant ends in
 * (linear.rs:143-144, 597-600; mxfp4.rs:158-168). Threads split output rows.
 */
ORC_API void orc_linear_f32(const float *x, const float *w, const float *bias, float *y, int64_t m, int64_t k,
                            int64_t n)
{
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < n; j++) {
        const float *wr = w + j * k;
        for (int64_t i = 0; i < m; i++) {
            float s = dot_f32(x + i * k, wr, k);
            y[i * n + j] = bias ? s + bias[j] : s;
        }
    }
}

ORC_API int orc_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Thread count of the parallel loops from now on (a launcher may have exported OMP_NUM_THREADS=1). */
ORC_API void orc_set_num_threads(int n)
{
    if (n > 0) omp_set_num_threads(n);
}

/* ------------------------------------------------------------------- MoE */

/*
 * Router post-processing (moe.rs:472-487): f32 softmax over all experts
 * (max-subtracted, linear.rs:164-176), descending sort, first top_k, gather,
 * optional renormalisation. Ties take the lower expert index.
 */
ORC_API void orc_moe_route(const float *logits, int64_t n_tokens, int num_experts, int top_k, int norm_topk,
                           int32_t *top_idx, float *top_vals)
{
    float *probs = (float *)malloc(sizeof(float) * (size_t)num_experts);
    uint8_t *taken = (uint8_t *)malloc((size_t)num_experts);
    for (int64_t t = 0; t < n_tokens; t++) {
        const float *l = logits + t * num_experts;
        float mx = l[0];
        for (int e = 1; e < num_experts; e++) mx = l[e] > mx ? l[e] : mx;
        float sum = 0.0f;
        for (int e = 0; e < num_experts; e++) { probs[e] = expf(l[e] - mx); sum += probs[e]; }
        for (int e = 0; e < num_experts; e++) probs[e] = probs[e] / sum;
        memset(taken, 0, (size_t)num_experts);
        float denom = 0.0f;
        for (int s = 0; s < top_k; s++) {
            int best = -1;
            for (int e = 0; e < num_experts; e++)
                if (!taken[e] && (best < 0 || probs[e] > probs[best])) best = e;
            taken[best] = 1;
            top_idx[t * top_k + s] = best;
            top_vals[t * top_k + s] = probs[best];
            denom += probs[best];
        }
        if (norm_topk)
            for (int s = 0; s < top_k; s++) top_vals[t * top_k + s] /= denom;
    }
    free(probs);
    free(taken);
}

/*
 * One GPT-OSS expert on m rows (moe.rs:152-173): gu = x W_gu^T + b_gu with
 * gate = gu[..., 0::2], up = gu[..., 1::2]; gate clamped above at `limit`, up
 * clamped to +-limit; glu = gate * sigmoid(1.702 gate); h = (up + 1) * glu;
 * out = h W_dn^T + b_dn. Weights arrive dequantized (mxfp4.rs:158-168).
 */
ORC_API void orc_gptoss_expert_f32(const float *x, const float *w_gu, const float *b_gu, const float *w_dn,
                                   const float *b_dn, float limit, int64_t m, int64_t hidden, int64_t inter,
                                   float *out)
{
    float *gu = (float *)malloc(sizeof(float) * (size_t)(m * 2 * inter));
    float *h = (float *)malloc(sizeof(float) * (size_t)(m * inter));
    orc_linear_f32(x, w_gu, b_gu, gu, m, hidden, 2 * inter);
    for (int64_t i = 0; i < m; i++)
        for (int64_t c = 0; c < inter; c++) {
            float gate = gu[i * 2 * inter + 2 * c], up = gu[i * 2 * inter + 2 * c + 1];
            gate = gate < limit ? gate : limit;
            up = up < -limit ? -limit : (up > limit ? limit : up);
            float z = gate * 1.702f;
            float sig = 1.0f / (expf(-z) + 1.0f);
            h[i * inter + c] = (up + 1.0f) * (gate * sig);
        }
    orc_linear_f32(h, w_dn, b_dn, out, m, inter, hidden);
    free(gu);
    free(h);
}

/*
 * dispatch_sparse (moe.rs:563-607) over GPT-OSS MXFP4 experts: tokens grouped
 * per expert in token order, experts visited in ascending id, each expert's
 * rows gathered, run, multiplied by their gate weight and index-added into a
 * zero [T, hidden] output. Expert weights are dequantized per visit exactly
 * like the reference's CPU forward does (mxfp4.rs:158-168).
 *   gu_blocks [E, 2*inter, hidden/32, 16], gu_scales [E, 2*inter, hidden/32],
 *   gu_bias [E, 2*inter], dn_blocks [E, hidden, inter/32, 16], ... (moe.rs:407-434).
 */
ORC_API int orc_gptoss_moe_f32(const float *x, const int32_t *top_idx, const float *top_vals, int64_t n_tokens,
                               int top_k, int num_experts, int64_t hidden, int64_t inter, const uint8_t *gu_blocks,
                               const uint8_t *gu_scales, const float *gu_bias, const uint8_t *dn_blocks,
                               const uint8_t *dn_scales, const float *dn_bias, float limit, int expert_lo,
                               int expert_hi, float *out)
{
    if (hidden % 32 != 0 || inter % 32 != 0) return -1;
    memset(out, 0, sizeof(float) * (size_t)(n_tokens * hidden));
    float *w_gu = (float *)malloc(sizeof(float) * (size_t)(2 * inter * hidden));
    float *w_dn = (float *)malloc(sizeof(float) * (size_t)(hidden * inter));
    int32_t *tok = (int32_t *)malloc(sizeof(int32_t) * (size_t)(n_tokens * top_k));
    float *wt = (float *)malloc(sizeof(float) * (size_t)(n_tokens * top_k));
    for (int e = expert_lo; e < expert_hi && e < num_experts; e++) {
        int64_t cnt = 0;
        for (int64_t t = 0; t < n_tokens; t++)
            for (int s = 0; s < top_k; s++)
                if (top_idx[t * top_k + s] == e) { tok[cnt] = (int32_t)t; wt[cnt] = top_vals[t * top_k + s]; cnt++; }
        if (cnt == 0) continue;
        orc_mxfp4_dequant_f32(gu_blocks + (int64_t)e * 2 * inter * (hidden / 32) * 16,
                              gu_scales + (int64_t)e * 2 * inter * (hidden / 32), 2 * inter, hidden, w_gu);
        orc_mxfp4_dequant_f32(dn_blocks + (int64_t)e * hidden * (inter / 32) * 16,
                              dn_scales + (int64_t)e * hidden * (inter / 32), hidden, inter, w_dn);
        float *xs = (float *)malloc(sizeof(float) * (size_t)(cnt * hidden));
        float *ys = (float *)malloc(sizeof(float) * (size_t)(cnt * hidden));
        for (int64_t r = 0; r < cnt; r++) memcpy(xs + r * hidden, x + (int64_t)tok[r] * hidden, sizeof(float) * (size_t)hidden);
        orc_gptoss_expert_f32(xs, w_gu, gu_bias + (int64_t)e * 2 * inter, w_dn, dn_bias + (int64_t)e * hidden, limit,
                              cnt, hidden, inter, ys);
        for (int64_t r = 0; r < cnt; r++)
            for (int64_t c = 0; c < hidden; c++) out[(int64_t)tok[r] * hidden + c] += ys[r * hidden + c] * wt[r];
        free(xs);
        free(ys);
    }
    free(w_gu);
    free(w_dn);
    free(tok);
    free(wt);
    return 0;
}
