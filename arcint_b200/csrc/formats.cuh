// formats.cuh -- device-side decoders of the five GGUF block formats.
//
// Layouts follow ggml's block structs as the reference kernels read them
// (marfrit/arcint, contrib/llama.cpp/patches; line numbers are lines of the .patch):
//   Q4_0   18 B: fp16 d, 16 B nibbles; byte j low -> weight j, high -> j+16; w = d (n - 8)
//          (0099-opencl-q4_0-q8_0-int8-gemm.patch:323-326)
//   Q8_0   34 B: fp16 d, 32 int8; w = d q                      (0099-...:575-576)
//   IQ4_NL 18 B: Q4_0's block; the nibbles index kvalues_iq4nl; w = d kv[n]   (0000-01-...:2143-2145)
//   Q4_K  144 B: fp16 d, fp16 dmin, 12 B of 6-bit scales/mins, 128 B nibbles; group g of
//          32 bytes: low -> sub-block 2g, high -> 2g+1; w = d sc q - dmin m
//          (0000-01-kquant-integer-dpas.patch:1562-1576, 3735-3739)
//   Q5_K  176 B: Q4_K's header, then 32 B of fifth bits (bit j of byte t: weight t of sub-block j), then Q4_K's
//          128 B of nibbles; w = d sc (n + 16 bit) - dmin m      (0000-01-...:1734-1735, 3735-3739)
//   Q6_K  210 B: ql[128], qh[64], int8 scales[16], fp16 d; w = d sc (q - 32)
//          (0000-01-...:1789-1794, 3798-3802, 3849-3860)
//   IQ4_XS 136 B: fp16 d, u16 scales_h, scales_l[4], 128 B nibbles indexing kvalues_iq4nl;
//          w = d (ls - 32) kv[n]                                (0000-01-...:2143-2145, 2287-2298)
#pragma once

#include "intrin.cuh"
#include "../../include/b200q.h"

namespace b200q {

B200Q_HD float half_bits_to_float(uint16_t h) { return hd_half_bits(h); }

// one IEEE rounding per operation on both sides (no fused multiply-add), so the decode is
// bit-identical to ggml's dequantize_row_* and to gguf-py
B200Q_HD float mul_rn(float a, float b) {
#ifdef __CUDA_ARCH__
    return __fmul_rn(a, b);
#else
    volatile float r = a * b;
    return r;
#endif
}
B200Q_HD float sub_rn(float a, float b) {
#ifdef __CUDA_ARCH__
    return __fsub_rn(a, b);
#else
    volatile float r = a - b;
    return r;
#endif
}

B200Q_HD int kvalue_iq4nl(int n) {
    const int8_t kv[16] = { -127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113 };
    return kv[n & 15];
}

// 6-bit scale and min of Q4_K sub-block j from the 12 scale bytes held as three words
B200Q_HD void q4k_scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int j, int *sc, int *m) {
    const int sh = 8 * (j & 3);
    if (j < 4) {
        *sc = (s0 >> sh) & 63;
        *m  = (s1 >> sh) & 63;
    } else {
        const uint32_t q8 = (s2 >> sh) & 0xFF, lo = (s0 >> sh) & 0xFF, hi = (s1 >> sh) & 0xFF;
        *sc = (q8 & 0xF) | ((lo >> 6) << 4);
        *m  = (q8 >> 4) | ((hi >> 6) << 4);
    }
}

// IQ4_XS sub-block scale in 0..63 from scales_h and the four scales_l bytes as one word
B200Q_HD int iq4xs_ls(uint32_t scales_h, uint32_t scales_l, int p) {
    return ((scales_l >> (4 * p)) & 0xF) | (((scales_h >> (2 * p)) & 3) << 4);
}

// four nibble codes n (one per byte, 0..15) -> four int8 bytes n - 8, no carry between bytes
B200Q_HD uint32_t nib_minus8(uint32_t t) { return (t + 0x78787878u) ^ 0x80808080u; }
// four 6-bit codes (one per byte, 0..63) -> int8 bytes q - 32
B200Q_HD uint32_t six_minus32(uint32_t t) { return (t + 0x60606060u) ^ 0x80808080u; }

// kvalues_iq4nl lookup of four indices (one per byte, 0..15) with byte permutes: the table
// lives in four registers, PRMT picks from eight bytes at a time, bit 3 chooses the half
B200Q_HD uint32_t iq4nl_lookup4(uint32_t idx) {
    const uint32_t t0 = 0xBFAD9881u;   // -127,-104,-83,-65 (little-endian bytes)
    const uint32_t t1 = 0xF6EADDCFu;   // -49,-35,-22,-10
    const uint32_t t2 = 0x26190D01u;   // 1,13,25,38
    const uint32_t t3 = 0x71594535u;   // 53,69,89,113
    // selector: one nibble per output byte, low three bits of each index
    const uint32_t packed = idx | (idx >> 4);                      // bytes 0,2 hold (i1 i0), (i3 i2)
    const uint32_t sel = hd_byte_perm(packed, 0, 0x4420) & 0x7777u; // 16-bit selector
    const uint32_t lo = hd_byte_perm(t0, t1, sel);
    const uint32_t hi = hd_byte_perm(t2, t3, sel);
    const uint32_t msk = ((idx >> 3) & 0x01010101u) * 0xFFu;       // 0xFF where index >= 8
    return (lo & ~msk) | (hi & msk);
}

// The same lookup with the 16-entry byte table in four registers (t0: entries 0..3, ...), split
// so that several tables can share the selector work: `sel` picks among eight entries, `msk`
// is 0xFF in the bytes whose index is 8 or more.
B200Q_HD void lookup4_prepare(uint32_t idx, uint32_t *sel, uint32_t *msk) {
    const uint32_t packed = idx | (idx >> 4);
    *sel = hd_byte_perm(packed, 0, 0x4420) & 0x7777u;
    *msk = hd_byte_perm(idx << 4, 0, 0xBA98);          // sign-replicate: bit 3 of each index
}
B200Q_HD uint32_t lookup4_apply(uint32_t t0, uint32_t t1, uint32_t t2, uint32_t t3, uint32_t sel, uint32_t msk) {
    return (hd_byte_perm(t0, t1, sel) & ~msk) | (hd_byte_perm(t2, t3, sel) & msk);
}

// IQ4_XS for the int8 tensor cores: the product p = (ls - 32) * kvalues[n] of a weight's integer
// sub-scale and codebook value (|p| <= 4064) as two int8 limbs, p = 256 * hi + lo with
// hi = (p + 128) >> 8 in [-16, 16] and lo in [-128, 127]. One MMA per limb against the same
// activation gives sum(p x) = 256 * sum(hi x) + sum(lo x) exactly.
B200Q_HD void iq4xs_limbs(int ls, int n, int *hi, int *lo) {
    const int p = (ls - 32) * kvalue_iq4nl(n);
    const int h = (p + 128) >> 8;                       // arithmetic shift: floor((p + 128) / 256)
    *hi = h;
    *lo = p - 256 * h;
}

// The same limbs for the eight weights of one packed word q (byte b holds weight b of the word's
// group of four in its low nibble and weight 16 + b in its high nibble), in registers only:
//   hi_l / lo_l: limbs of the four low-nibble weights, hi_h / lo_h: of the four high-nibble ones.
// The codebook is looked up biased by 128 (unsigned bytes) with byte permutes whose selectors are
// the nibbles of q as they lie (q & 0x7777 7777 picks among eight entries, bit 3 of each nibble
// chooses the table half), widened to two 16-bit halves per register and multiplied by
// m = ls - 32 with one integer multiply-add per pair of weights:
//   half = (kv + 128) * m + (32896 - 128 m) = p + 128 + 32768, always inside 0..65535,
// so no carry crosses the halves; flipping bit 15 gives the 16-bit two's complement of p + 128,
// whose high byte is hi, and flipping bit 7 of its low byte gives lo.
B200Q_HD void iq4xs_limbs8(uint32_t q, int m, uint32_t *hi_l, uint32_t *lo_l, uint32_t *hi_h, uint32_t *lo_h) {
    const uint32_t t0 = 0x3F2D1801u, t1 = 0x766A5D4Fu, t2 = 0xA6998D81u, t3 = 0xF1D9C5B5u;   // kvalues + 128
    const uint32_t sel_a = q & 0x77777777u, sel_b = sel_a >> 16;      // nibbles (l0 h0 l1 h1), (l2 h2 l3 h3)
    const uint32_t q4 = q << 4;                                       // low nibbles' bit 3 at byte bit 7
    const uint32_t msk_a = hd_byte_perm(q4, q, 0xD9C8), msk_b = hd_byte_perm(q4, q, 0xFBEA);   // sign-replicate
    const uint32_t v_a = (hd_byte_perm(t0, t1, sel_a) & ~msk_a) | (hd_byte_perm(t2, t3, sel_a) & msk_a);
    const uint32_t v_b = (hd_byte_perm(t0, t1, sel_b) & ~msk_b) | (hd_byte_perm(t2, t3, sel_b) & msk_b);
    const uint32_t c = (uint32_t)(32896 - 128 * m) * 0x10001u, um = (uint32_t)m;
    const uint32_t za = (hd_byte_perm(v_a, 0, 0x4240) * um + c) ^ 0x80808080u;     // low-nibble weights 0, 1
    const uint32_t zb = (hd_byte_perm(v_a, 0, 0x4341) * um + c) ^ 0x80808080u;     // high-nibble weights 0, 1
    const uint32_t zc = (hd_byte_perm(v_b, 0, 0x4240) * um + c) ^ 0x80808080u;     // low-nibble weights 2, 3
    const uint32_t zd = (hd_byte_perm(v_b, 0, 0x4341) * um + c) ^ 0x80808080u;     // high-nibble weights 2, 3
    *hi_l = hd_byte_perm(za, zc, 0x7531);
    *lo_l = hd_byte_perm(za, zc, 0x6420);
    *hi_h = hd_byte_perm(zb, zd, 0x7531);
    *lo_h = hd_byte_perm(zb, zd, 0x6420);
}

// Q4_K for the int8 tensor cores: the product p = sc * q of a weight's 6-bit sub-block scale and
// its 4-bit code (0 <= p <= 945) as two int8 limbs, p = 256 * hi + lo with hi = (p + 128) >> 8 in
// 0..4 and lo in [-128, 127], for four codes (one per byte, 0..15) at once: the codes are widened
// to 16-bit halves, one integer multiply-add per pair gives p + 128 (no carry between halves), the
// high bytes are hi and the low bytes with bit 7 flipped are lo. The mins term of the format
// (dmin * m * sum(x)) does not go through the tensor core.
B200Q_HD void q4k_limbs4(uint32_t idx, uint32_t sc, uint32_t *hi4, uint32_t *lo4) {
    const uint32_t za = hd_byte_perm(idx, 0, 0x4140) * sc + 0x00800080u;
    const uint32_t zb = hd_byte_perm(idx, 0, 0x4342) * sc + 0x00800080u;
    *hi4 = hd_byte_perm(za, zb, 0x7531);
    *lo4 = hd_byte_perm(za, zb, 0x6420) ^ 0x80808080u;
}

// Q6_K for the int8 tensor cores: p = sc * (q - 32) with the int8 sub-block scale and the 6-bit code
// (|p| <= 4096) as two int8 limbs, p = 256 * hi + lo, for four codes (one per byte, 0..63) at once:
// half = q * sc + (32896 - 32 sc) = p + 128 + 32768 stays inside 0..65535, the rest as for IQ4_XS.
B200Q_HD void q6k_limbs4(uint32_t q6, int sc, uint32_t *hi4, uint32_t *lo4) {
    const uint32_t c = (uint32_t)(32896 - 32 * sc) * 0x10001u, us = (uint32_t)sc;
    const uint32_t za = (hd_byte_perm(q6, 0, 0x4140) * us + c) ^ 0x80808080u;
    const uint32_t zb = (hd_byte_perm(q6, 0, 0x4342) * us + c) ^ 0x80808080u;
    *hi4 = hd_byte_perm(za, zb, 0x7531);
    *lo4 = hd_byte_perm(za, zb, 0x6420);
}

// the eight 6-bit mins (or scales) of a Q4_K block as two words of four bytes
B200Q_HD void q4k_mins8(uint32_t s0, uint32_t s1, uint32_t s2, uint32_t *m03, uint32_t *m47) {
    *m03 = s1 & 0x3F3F3F3Fu;
    *m47 = ((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u);
    (void)s0;
}
B200Q_HD void q4k_scales8(uint32_t s0, uint32_t s1, uint32_t s2, uint32_t *c03, uint32_t *c47) {
    *c03 = s0 & 0x3F3F3F3Fu;
    *c47 = (s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u);
    (void)s1;
}

// Generic, slow, exact f32 decode of weight i of a row (used by the debug dequantizer
// and as the spec the fast kernels are tested against). One rounding per multiply,
// like ggml's dequantize_row_* and gguf-py.
__host__ __device__ inline float decode_weight(int type, const uint8_t *row, int64_t i) {
    switch (type) {
    case B200Q_TYPE_Q4_0: {
        const uint8_t *b = row + (i / 32) * 18;
        const int j = (int)(i % 32);
        const float d = half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
        const int n = j < 16 ? (b[2 + j] & 0xF) : (b[2 + j - 16] >> 4);
        return mul_rn(d, (float)(n - 8));
    }
    case B200Q_TYPE_IQ4_NL: {
        const uint8_t *b = row + (i / 32) * 18;
        const int j = (int)(i % 32);
        const float d = half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
        const int n = j < 16 ? (b[2 + j] & 0xF) : (b[2 + j - 16] >> 4);
        const uint32_t kv = iq4nl_lookup4((uint32_t)n);
        return mul_rn(d, (float)(int8_t)(kv & 0xFFu));
    }
    case B200Q_TYPE_Q8_0: {
        const uint8_t *b = row + (i / 32) * 34;
        const float d = half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
        return mul_rn((float)(int8_t)b[2 + i % 32], d);
    }
    case B200Q_TYPE_Q4_K: {
        const uint8_t *b = row + (i / 256) * 144;
        const int r = (int)(i % 256), j = r / 32, t = r % 32;
        const float d = half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
        const float dmin = half_bits_to_float((uint16_t)(b[2] | (b[3] << 8)));
        const uint8_t *s = b + 4;
        const uint32_t s0 = s[0] | (s[1] << 8) | (s[2] << 16) | ((uint32_t)s[3] << 24);
        const uint32_t s1 = s[4] | (s[5] << 8) | (s[6] << 16) | ((uint32_t)s[7] << 24);
        const uint32_t s2 = s[8] | (s[9] << 8) | (s[10] << 16) | ((uint32_t)s[11] << 24);
        int sc, m;
        q4k_scale_min(s0, s1, s2, j, &sc, &m);
        const uint8_t qb = b[16 + 32 * (j / 2) + t];
        const int q = (j & 1) ? (qb >> 4) : (qb & 0xF);
        return sub_rn(mul_rn(mul_rn(d, (float)sc), (float)q), mul_rn(dmin, (float)m));
    }
    case B200Q_TYPE_Q5_K: {
        const uint8_t *b = row + (i / 256) * 176;
        const int r = (int)(i % 256), j = r / 32, t = r % 32;
        const float d = half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
        const float dmin = half_bits_to_float((uint16_t)(b[2] | (b[3] << 8)));
        const uint8_t *s = b + 4;
        const uint32_t s0 = s[0] | (s[1] << 8) | (s[2] << 16) | ((uint32_t)s[3] << 24);
        const uint32_t s1 = s[4] | (s[5] << 8) | (s[6] << 16) | ((uint32_t)s[7] << 24);
        const uint32_t s2 = s[8] | (s[9] << 8) | (s[10] << 16) | ((uint32_t)s[11] << 24);
        int sc, m;
        q4k_scale_min(s0, s1, s2, j, &sc, &m);
        const uint8_t qb = b[48 + 32 * (j / 2) + t];
        const int q = ((j & 1) ? (qb >> 4) : (qb & 0xF)) | (((b[16 + t] >> j) & 1) << 4);
        return sub_rn(mul_rn(mul_rn(d, (float)sc), (float)q), mul_rn(dmin, (float)m));
    }
    case B200Q_TYPE_Q6_K: {
        const uint8_t *b = row + (i / 256) * 210;
        const int r = (int)(i % 256), n = r / 128, p = (r % 128) / 32, t = r % 32;
        const uint8_t l = b[64 * n + 32 * (p & 1) + t];
        const uint8_t h = b[128 + 32 * n + t];
        const int q = ((p & 2) ? (l >> 4) : (l & 0xF)) | (((h >> (2 * p)) & 3) << 4);
        const float d = half_bits_to_float((uint16_t)(b[208] | (b[209] << 8)));
        const int sc = (int8_t)b[192 + 8 * n + 2 * p + (t >= 16)];
        return mul_rn(mul_rn(d, (float)sc), (float)(q - 32));
    }
    case B200Q_TYPE_IQ4_XS: {
        const uint8_t *b = row + (i / 256) * 136;
        const int r = (int)(i % 256), p = r / 32, t = r % 32;
        const float d = half_bits_to_float((uint16_t)(b[0] | (b[1] << 8)));
        const uint32_t sh = b[2] | (b[3] << 8);
        const uint32_t sl = b[4] | (b[5] << 8) | (b[6] << 16) | ((uint32_t)b[7] << 24);
        const int ls = iq4xs_ls(sh, sl, p);
        const uint8_t qb = b[8 + 16 * p + (t & 15)];
        const int n = t < 16 ? (qb & 0xF) : (qb >> 4);
        return mul_rn(mul_rn(d, (float)(ls - 32)), (float)kvalue_iq4nl(n));
    }
    }
    return 0.f;
}

}  // namespace b200q
