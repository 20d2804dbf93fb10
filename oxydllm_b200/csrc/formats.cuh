// Per-element decode of every packed weight format, bit-exact with the
// reference's CPU dequantizers. Products and differences use the explicit
// round-to-nearest intrinsics so that nvcc cannot contract them into fused
// multiply-adds, which would change the last bit.
#pragma once

#include "oxq_common.cuh"

namespace oxq {

__host__ __device__ inline bool gguf_block_layout(int ggml_type, int &block_elems, int &block_bytes)
{
    switch (ggml_type) {
    case OXQ_GGML_Q4_0: block_elems = 32; block_bytes = 18; return true;
    case OXQ_GGML_Q8_0: block_elems = 32; block_bytes = 34; return true;
    case OXQ_GGML_Q4_K: block_elems = 256; block_bytes = 144; return true;
    case OXQ_GGML_Q6_K: block_elems = 256; block_bytes = 210; return true;
    case OXQ_GGML_Q4_1: block_elems = 32; block_bytes = 20; return true;
    case OXQ_GGML_Q5_0: block_elems = 32; block_bytes = 22; return true;
    case OXQ_GGML_Q5_1: block_elems = 32; block_bytes = 24; return true;
    case OXQ_GGML_Q5_K: block_elems = 256; block_bytes = 176; return true;
    case OXQ_GGML_Q2_K: block_elems = 256; block_bytes = 84; return true;
    case OXQ_GGML_Q3_K: block_elems = 256; block_bytes = 110; return true;
    default: return false;
    }
}

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t ld_u16(const uint8_t *p)
{
    return *reinterpret_cast<const uint16_t *>(p); // all f16 fields sit at even offsets of even-sized blocks
}

// Q4_K: 6-bit scale and min of sub-block j (0..7) from the 12 packed bytes.
__device__ __forceinline__ void q4k_scale_min(int j, const uint8_t *q, uint32_t &sc, uint32_t &mn)
{
    if (j < 4) {
        sc = q[j] & 63u;
        mn = q[j + 4] & 63u;
    } else {
        sc = (q[j + 4] & 0x0Fu) | ((uint32_t)(q[j - 4] >> 6) << 4);
        mn = ((uint32_t)q[j + 4] >> 4) | ((uint32_t)(q[j] >> 6) << 4);
    }
}

// Element j of one GGML block.
//   Q4_0 {f16 d; u8 qs[16]}: (nibble - 8) * d, j < 16 low nibbles, j >= 16 high.
//   Q8_0 {f16 d; i8 qs[32]}: qs[j] * d.
//   Q4_K {f16 d, dmin; u8 scales[12]; u8 qs[128]}: (d*sc)*nibble - (dmin*mn).
//   Q6_K {u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d}: (d*scale) * (6-bit - 32).
//   Q4_1 {f16 d, m; u8 qs[16]}: nibble * d + m.
//   Q5_0 {f16 d; u8 qh[4]; u8 qs[16]}: ((nibble | bit j of qh << 4) - 16) * d.
//   Q5_1 {f16 d, m; u8 qh[4]; u8 qs[16]}: (nibble | bit j of qh << 4) * d + m.
//   Q5_K {f16 d, dmin; u8 scales[12]; u8 qh[32]; u8 qs[128]}: Q4_K with bit `sub` of qh[el] as fifth bit.
//   Q2_K {u8 scales[16]; u8 qs[64]; f16 d, dmin}: sub-block j / 16 has scale nibble and min nibble in scales[j / 16];
//        (d*sc) * two-bit - (dmin*mn), two-bit = (qs[(j >> 7) * 32 + (j & 31)] >> 2 * ((j >> 5) & 3)) & 3.
//   Q3_K {u8 hmask[32]; u8 qs[64]; u8 scales[12]; f16 d}: 6-bit scale of sub-block j / 16 from the 12 packed bytes;
//        (d * (scale - 32)) * (two-bit - (bit j >> 5 of hmask[j & 31] ? 0 : 4)).
template <int TYPE> __device__ __forceinline__ float gguf_decode_elem(const uint8_t *blk, int j)
{
    if (TYPE == OXQ_GGML_Q4_0) {
        float d = half_bits_to_f32((uint16_t)ld_u16(blk));
        uint32_t b = blk[2 + (j & 15)];
        int q = (int)(j < 16 ? (b & 0x0Fu) : (b >> 4)) - 8;
        return __fmul_rn((float)q, d);
    } else if (TYPE == OXQ_GGML_Q8_0) {
        float d = half_bits_to_f32((uint16_t)ld_u16(blk));
        int q = (int)(int8_t)blk[2 + j];
        return __fmul_rn((float)q, d);
    } else if (TYPE == OXQ_GGML_Q4_1) {
        float d = half_bits_to_f32((uint16_t)ld_u16(blk)), mn = half_bits_to_f32((uint16_t)ld_u16(blk + 2));
        uint32_t b = blk[4 + (j & 15)];
        uint32_t q = j < 16 ? (b & 0x0Fu) : (b >> 4);
        return __fadd_rn(__fmul_rn((float)q, d), mn);
    } else if (TYPE == OXQ_GGML_Q5_0 || TYPE == OXQ_GGML_Q5_1) {
        const bool with_min = TYPE == OXQ_GGML_Q5_1;
        const uint8_t *qhb = blk + (with_min ? 4 : 2);
        float d = half_bits_to_f32((uint16_t)ld_u16(blk));
        uint32_t qh = ld_u16(qhb) | (ld_u16(qhb + 2) << 16);
        uint32_t b = qhb[4 + (j & 15)];
        uint32_t q = (j < 16 ? (b & 0x0Fu) : (b >> 4)) | (((qh >> j) & 1u) << 4);
        if (with_min) return __fadd_rn(__fmul_rn((float)q, d), half_bits_to_f32((uint16_t)ld_u16(blk + 2)));
        return __fmul_rn((float)((int)q - 16), d);
    } else if (TYPE == OXQ_GGML_Q5_K) {
        float d = half_bits_to_f32((uint16_t)ld_u16(blk));
        float dmin = half_bits_to_f32((uint16_t)ld_u16(blk + 2));
        int sub = j >> 5, el = j & 31;
        uint32_t sc, mn;
        q4k_scale_min(sub, blk + 4, sc, mn);
        float sc_v = __fmul_rn(d, (float)sc), m_v = __fmul_rn(dmin, (float)mn);
        uint32_t b = blk[48 + (sub >> 1) * 32 + el];
        uint32_t q = ((sub & 1) ? (b >> 4) : (b & 0x0Fu)) | ((((uint32_t)blk[16 + el] >> sub) & 1u) << 4);
        return __fsub_rn(__fmul_rn(sc_v, (float)q), m_v);
    } else if (TYPE == OXQ_GGML_Q2_K) {
        const float d = half_bits_to_f32((uint16_t)ld_u16(blk + 80)), dmin = half_bits_to_f32((uint16_t)ld_u16(blk + 82));
        const uint32_t sc = blk[j >> 4];
        const float dl = __fmul_rn(d, (float)(sc & 0x0Fu)), ml = __fmul_rn(dmin, (float)(sc >> 4));
        const uint32_t q = ((uint32_t)blk[16 + (j >> 7) * 32 + (j & 31)] >> (2 * ((j >> 5) & 3))) & 3u;
        return __fsub_rn(__fmul_rn(dl, (float)q), ml);
    } else if (TYPE == OXQ_GGML_Q3_K) {
        const uint8_t *scb = blk + 96;
        const int is = j >> 4;
        const uint32_t lo4 = is < 8 ? (scb[is] & 0x0Fu) : ((uint32_t)scb[is - 8] >> 4);
        const uint32_t hi2 = ((uint32_t)scb[8 + (is & 3)] >> (2 * (is >> 2))) & 3u;
        const float dl = __fmul_rn(half_bits_to_f32((uint16_t)ld_u16(blk + 108)), (float)((int)(lo4 | (hi2 << 4)) - 32));
        const int q2 = (int)(((uint32_t)blk[32 + (j >> 7) * 32 + (j & 31)] >> (2 * ((j >> 5) & 3))) & 3u);
        const int hb = (blk[j & 31] >> (j >> 5)) & 1;
        return __fmul_rn(dl, (float)(q2 - (hb ? 0 : 4)));
    } else if (TYPE == OXQ_GGML_Q4_K) {
        float d = half_bits_to_f32((uint16_t)ld_u16(blk));
        float dmin = half_bits_to_f32((uint16_t)ld_u16(blk + 2));
        int sub = j >> 5, el = j & 31;
        uint32_t sc, mn;
        q4k_scale_min(sub, blk + 4, sc, mn);
        float sc_v = __fmul_rn(d, (float)sc), m_v = __fmul_rn(dmin, (float)mn);
        uint32_t b = blk[16 + (sub >> 1) * 32 + el];
        uint32_t nib = (sub & 1) ? (b >> 4) : (b & 0x0Fu);
        return __fsub_rn(__fmul_rn(sc_v, (float)nib), m_v);
    } else {
        int half_i = j >> 7, pos = j & 127, quad = pos >> 5, l = pos & 31;
        const uint8_t *ql = blk + 64 * half_i, *qh = blk + 128 + 32 * half_i;
        uint32_t nib = (ql[(quad & 1) ? l + 32 : l] >> (quad < 2 ? 0 : 4)) & 0x0Fu;
        uint32_t hb = (qh[l] >> (2 * quad)) & 3u;
        int q = (int)(nib | (hb << 4)) - 32;
        float d = half_bits_to_f32((uint16_t)ld_u16(blk + 208));
        int sc = (int)(int8_t)blk[192 + 8 * half_i + 2 * quad + (l >> 4)];
        return __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
    }
}

// AWQ: slot (0..7) inside a packed word that holds out column `col` of the word.
// Columns {0,2,4,6} sit in slots {0,1,2,3}, columns {1,3,5,7} in slots {4,5,6,7}.
__device__ __forceinline__ int awq_slot_of_col(int col) { return (col >> 1) + ((col & 1) << 2); }

#endif // __CUDACC__

} // namespace oxq
