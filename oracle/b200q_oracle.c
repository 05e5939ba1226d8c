/*
 * b200q_oracle.c -- CPU restatement of the quantized MUL_MAT / MUL_MAT_ID path.
 *
 * TEST INFRASTRUCTURE ONLY (see b200q_oracle.h for the pinning status; the
 * K-quant / IQ4_XS weight quantizers and the per-256 activation quantizer are
 * PARITY UNPINNED stand-ins). The product library never links or loads this.
 *
 * Reference citations are paths inside marfrit/arcint; "P01" etc. are
 *   P01  contrib/llama.cpp/patches/0000-01-kquant-integer-dpas.patch
 *   P02  contrib/llama.cpp/patches/0000-02-lowbit-iq-types.patch
 *   P09  contrib/llama.cpp/patches/0000-09-moe-routing-gemm-tiles.patch
 *   P99  contrib/llama.cpp/patches/0099-opencl-q4_0-q8_0-int8-gemm.patch
 *   P103 contrib/llama.cpp/patches/0103-opencl-id-int8-sg8.patch
 *   P115 contrib/llama.cpp/patches/0115-opencl-few-column-int8-q4_0-q8_0-iq4.patch
 * and line numbers are lines of the .patch file.
 *
 * Build: gcc -O3 -fopenmp -ffp-contract=off -fPIC -shared (see build.py).
 * -ffp-contract=off matters: the decoders must round like the numpy golden
 * vectors (one rounding per multiply, no fused multiply-add).
 */
#include "b200q_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define QK   32
#define QK_K 256

/* ------------------------------------------------------------------ fp16 */

float orc_fp16_to_fp32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {                        /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* round to nearest even, like numpy's astype(float16) and ggml's GGML_FP32_TO_FP16 */
uint16_t orc_fp32_to_fp16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    const uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (ax > 0x7F800000u ? 0x200u : 0));
    if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);       /* overflows to inf after rounding */
    if (ax < 0x33000001u) return sign;                              /* below half the smallest subnormal */
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { shift = 13 + (-14 - e); base = 0; }              /* subnormal half */
    else         { shift = 13; base = (uint32_t)(e + 15) << 10; man &= 0x7FFFFFu; }
    uint32_t q = man >> shift, rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) ++q;
    return (uint16_t)(sign | (base + q));
}

/* ----------------------------------------------------------- block formats */

int orc_block_size(int type) {
    switch (type) {
        case ORC_TYPE_Q4_0: case ORC_TYPE_Q8_0: case ORC_TYPE_IQ4_NL: return QK;
        case ORC_TYPE_Q4_K: case ORC_TYPE_Q5_K: case ORC_TYPE_Q6_K: case ORC_TYPE_IQ4_XS: return QK_K;
        default: return 0;
    }
}

size_t orc_block_bytes(int type) {
    switch (type) {
        case ORC_TYPE_Q4_0:   return 18;
        case ORC_TYPE_IQ4_NL: return 18;
        case ORC_TYPE_Q8_0:   return 34;
        case ORC_TYPE_Q4_K:   return 144;
        case ORC_TYPE_Q5_K:   return 176;
        case ORC_TYPE_Q6_K:   return 210;
        case ORC_TYPE_IQ4_XS: return 136;
        default: return 0;
    }
}

size_t orc_row_bytes(int type, int64_t k) {
    const int bs = orc_block_size(type);
    return bs ? (size_t)(k / bs) * orc_block_bytes(type) : 0;
}

int orc_act_form(int type) {
    return (type == ORC_TYPE_Q4_0 || type == ORC_TYPE_Q8_0 || type == ORC_TYPE_IQ4_NL) ? ORC_ACT_Q8_0 : ORC_ACT_Q8_256;
}

static inline uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static inline void wr16(uint8_t *p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }

/* kvalues_iq4nl (P01:2143-2145) */
static const int8_t KV_IQ4NL[16] = { -127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113 };

/* get_scale_min_k4 (P01:1562-1576, 3684-3701): 6-bit scale and min of sub-block j */
static inline void q4k_scale_min(const uint8_t *s, int j, int *sc, int *m) {
    if (j < 4) {
        *sc = s[j] & 63;
        *m  = s[j + 4] & 63;
    } else {
        *sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4);
        *m  = (s[j + 4] >> 4)  | ((s[j] >> 6) << 4);
    }
}

/* IQ4_XS sub-block scale ls in 0..63 (P01:2287-2298; P115:950-958) */
static inline int iq4xs_ls(const uint8_t *blk, int p) {
    const uint16_t sh = rd16(blk + 2);
    const uint8_t *sl = blk + 4;
    return ((sl[p >> 1] >> (4 * (p & 1))) & 0xF) | (((sh >> (2 * p)) & 3) << 4);
}

/*
 * Integer view of one block: codes as signed integers in block order plus what
 * the float decode needs. One routine per type serves both the f32 dequantizer
 * and the integer vec-dot, so they cannot drift apart.
 */

/* Q4_0 (P99:323-326, P02:6098-6106): byte j low nibble -> weight j, high -> j+16; w = d (n - 8) */
static void q4_0_codes(const uint8_t *blk, int8_t *q /*32*/) {
    for (int j = 0; j < 16; ++j) {
        q[j]      = (int8_t)((blk[2 + j] & 0xF) - 8);
        q[j + 16] = (int8_t)((blk[2 + j] >> 4) - 8);
    }
}

/* IQ4_NL (P01:2143-2145 the codebook; P115:1057-1085 lists the type beside Q4_0): Q4_0's 18-byte block and nibble order,
 * the nibbles index kvalues_iq4nl; w = d kv[n] */
static void iq4_nl_codes(const uint8_t *blk, int8_t *q /*32, codebook values*/) {
    for (int j = 0; j < 16; ++j) {
        q[j]      = KV_IQ4NL[blk[2 + j] & 0xF];
        q[j + 16] = KV_IQ4NL[blk[2 + j] >> 4];
    }
}

/* Q4_K nibble order (P01:3735-3739, 2198-2223): qs group g (32 bytes): low -> sub-block 2g, high -> 2g+1 */
static void q4_K_codes(const uint8_t *blk, uint8_t *q /*256, 0..15*/) {
    const uint8_t *qs = blk + 16;
    for (int g = 0; g < 4; ++g)
        for (int i = 0; i < 32; ++i) {
            q[64 * g + i]      = qs[32 * g + i] & 0xF;
            q[64 * g + 32 + i] = qs[32 * g + i] >> 4;
        }
}

/* Q5_K (P01:1734-1735, 3735-3739): Q4_K's nibble order behind 32 bytes of fifth bits; bit j of byte t belongs to
 * weight t of sub-block j. Block: d, dmin, 12 scale bytes, qh[32], qs[128] (176 bytes). */
static void q5_K_codes(const uint8_t *blk, uint8_t *q /*256, 0..31*/) {
    const uint8_t *qh = blk + 16, *qs = blk + 48;
    for (int g = 0; g < 4; ++g)
        for (int i = 0; i < 32; ++i) {
            q[64 * g + i]      = (uint8_t)((qs[32 * g + i] & 0xF) | (((qh[i] >> (2 * g)) & 1) << 4));
            q[64 * g + 32 + i] = (uint8_t)((qs[32 * g + i] >> 4)  | (((qh[i] >> (2 * g + 1)) & 1) << 4));
        }
}

/* Q6_K (P01:1789-1794, 3798-3802, 3849-3860): q - 32 in -32..31; scale index 8n + 2p + (t >= 16) */
static void q6_K_codes(const uint8_t *blk, int8_t *q /*256*/) {
    const uint8_t *ql = blk, *qh = blk + 128;
    for (int n = 0; n < 2; ++n)
        for (int t = 0; t < 32; ++t) {
            const uint8_t h = qh[32 * n + t];
            q[128 * n + t]      = (int8_t)(((ql[64 * n + t] & 0xF)      | (((h >> 0) & 3) << 4)) - 32);
            q[128 * n + 32 + t] = (int8_t)(((ql[64 * n + 32 + t] & 0xF) | (((h >> 2) & 3) << 4)) - 32);
            q[128 * n + 64 + t] = (int8_t)(((ql[64 * n + t] >> 4)       | (((h >> 4) & 3) << 4)) - 32);
            q[128 * n + 96 + t] = (int8_t)(((ql[64 * n + 32 + t] >> 4)  | (((h >> 6) & 3) << 4)) - 32);
        }
}

/* IQ4_XS (P01:2287-2298, P103:307-314): 16 bytes at qs+16p: low nibbles -> 32p+0..15, high -> 32p+16..31 */
static void iq4_xs_codes(const uint8_t *blk, int8_t *q /*256, codebook values*/) {
    const uint8_t *qs = blk + 8;
    for (int p = 0; p < 8; ++p)
        for (int j = 0; j < 16; ++j) {
            q[32 * p + j]      = KV_IQ4NL[qs[16 * p + j] & 0xF];
            q[32 * p + 16 + j] = KV_IQ4NL[qs[16 * p + j] >> 4];
        }
}

int orc_dequantize_row(int type, const void *src, float *dst, int64_t k) {
    const uint8_t *b = (const uint8_t *)src;
    const int bs = orc_block_size(type);
    if (!bs || k % bs) return -1;
    const int64_t nb = k / bs;
    const size_t bb = orc_block_bytes(type);
    for (int64_t ib = 0; ib < nb; ++ib, b += bb, dst += bs) {
        switch (type) {
        case ORC_TYPE_Q4_0: {
            int8_t q[32];
            q4_0_codes(b, q);
            const float d = orc_fp16_to_fp32(rd16(b));
            for (int i = 0; i < 32; ++i) dst[i] = d * (float)q[i];
        } break;
        case ORC_TYPE_IQ4_NL: {
            int8_t q[32];
            iq4_nl_codes(b, q);
            const float d = orc_fp16_to_fp32(rd16(b));
            for (int i = 0; i < 32; ++i) dst[i] = d * (float)q[i];
        } break;
        case ORC_TYPE_Q8_0: {       /* P99:575-576, P115:922-923: w = d q */
            const float d = orc_fp16_to_fp32(rd16(b));
            for (int i = 0; i < 32; ++i) dst[i] = (float)(int8_t)b[2 + i] * d;
        } break;
        case ORC_TYPE_Q4_K: {       /* w = (d sc) q - (dmin m) */
            uint8_t q[256];
            q4_K_codes(b, q);
            const float d = orc_fp16_to_fp32(rd16(b)), dmin = orc_fp16_to_fp32(rd16(b + 2));
            for (int j = 0; j < 8; ++j) {
                int sc, m;
                q4k_scale_min(b + 4, j, &sc, &m);
                const float dl = d * (float)sc, ml = dmin * (float)m;
                for (int i = 0; i < 32; ++i) dst[32 * j + i] = dl * (float)q[32 * j + i] - ml;
            }
        } break;
        case ORC_TYPE_Q5_K: {       /* w = (d sc) q - (dmin m), q in 0..31 */
            uint8_t q[256];
            q5_K_codes(b, q);
            const float d = orc_fp16_to_fp32(rd16(b)), dmin = orc_fp16_to_fp32(rd16(b + 2));
            for (int j = 0; j < 8; ++j) {
                int sc, m;
                q4k_scale_min(b + 4, j, &sc, &m);
                const float dl = d * (float)sc, ml = dmin * (float)m;
                for (int i = 0; i < 32; ++i) dst[32 * j + i] = dl * (float)q[32 * j + i] - ml;
            }
        } break;
        case ORC_TYPE_Q6_K: {       /* w = (d scale) (q - 32) */
            int8_t q[256];
            q6_K_codes(b, q);
            const float d = orc_fp16_to_fp32(rd16(b + 208));
            for (int g = 0; g < 16; ++g) {
                const float dl = d * (float)(int8_t)b[192 + g];
                for (int i = 0; i < 16; ++i) dst[16 * g + i] = dl * (float)q[16 * g + i];
            }
        } break;
        case ORC_TYPE_IQ4_XS: {     /* w = (d (ls - 32)) kvalues[nibble] */
            int8_t q[256];
            iq4_xs_codes(b, q);
            const float d = orc_fp16_to_fp32(rd16(b));
            for (int p = 0; p < 8; ++p) {
                const float dl = d * (float)(iq4xs_ls(b, p) - 32);
                for (int i = 0; i < 32; ++i) dst[32 * p + i] = dl * (float)q[32 * p + i];
            }
        } break;
        default: return -1;
        }
    }
    return 0;
}

/* ------------------------------------------------------ weight quantizers */

/* roundf: half away from zero */
static inline int nearest_away(float v) { return (int)roundf(v); }

/* Q4_0, ggml rule as published in gguf-py (quants.py Q4_0.quantize_blocks):
 * d = (value of largest magnitude, first on ties) / -8; code = min(15, trunc(x/d + 8.5)) */
static void quantize_q4_0(const float *x, uint8_t *b) {
    float amax = 0.f, max = 0.f;
    for (int i = 0; i < 32; ++i) {
        const float a = fabsf(x[i]);
        if (a > amax) { amax = a; max = x[i]; }
    }
    const float d = max / -8.f;
    const float id = d != 0.f ? 1.f / d : 0.f;
    wr16(b, orc_fp32_to_fp16(d));
    uint8_t q[32];
    for (int i = 0; i < 32; ++i) {
        const float v = truncf(x[i] * id + 8.5f);
        q[i] = (uint8_t)(v < 0.f ? 0 : (v > 15.f ? 15 : (int)v));
    }
    for (int j = 0; j < 16; ++j) b[2 + j] = (uint8_t)(q[j] | (q[j + 16] << 4));
}

/* Q8_0, ggml rule (gguf-py Q8_0.quantize_blocks: "bit-exact same results as ggml-quants.c") */
static void quantize_q8_0(const float *x, uint8_t *b) {
    float amax = 0.f;
    for (int i = 0; i < 32; ++i) { const float a = fabsf(x[i]); if (a > amax) amax = a; }
    const float d = amax / 127.f;
    const float id = d != 0.f ? 1.f / d : 0.f;
    wr16(b, orc_fp32_to_fp16(d));
    for (int i = 0; i < 32; ++i) b[2 + i] = (uint8_t)(int8_t)nearest_away(x[i] * id);
}

/*
 * Stand-in quantizers for Q4_K, Q6_K and IQ4_XS: plain round-to-nearest onto
 * the format's grid. NOT ggml's search-based quantizers (PARITY UNPINNED); the
 * op consumes blocks and is agnostic to how they were made, so these only give
 * the benchmark tensors realistic field distributions.
 */
static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* levels = 15: Q4_K (codes 0..15, 144-byte block); levels = 31: Q5_K (codes 0..31, the fifth bits in qh, 176 bytes) */
static void quantize_q45_K_standin(const float *x, uint8_t *b, int levels) {
    float scale[8], mn[8], smax = 0.f, mmax = 0.f;
    for (int j = 0; j < 8; ++j) {
        float lo = 0.f, hi = 0.f;
        for (int i = 0; i < 32; ++i) { const float v = x[32 * j + i]; if (v < lo) lo = v; if (v > hi) hi = v; }
        scale[j] = (hi - lo) / (float)levels;
        mn[j] = -lo;
        if (scale[j] > smax) smax = scale[j];
        if (mn[j] > mmax) mmax = mn[j];
    }
    const uint16_t dh = orc_fp32_to_fp16(smax / 63.f), dmh = orc_fp32_to_fp16(mmax / 63.f);
    const float d = orc_fp16_to_fp32(dh), dmin = orc_fp16_to_fp32(dmh);
    int sc[8], m[8];
    for (int j = 0; j < 8; ++j) {
        sc[j] = d > 0.f ? clampi(nearest_away(scale[j] / d), 0, 63) : 0;
        m[j]  = dmin > 0.f ? clampi(nearest_away(mn[j] / dmin), 0, 63) : 0;
    }
    wr16(b, dh);
    wr16(b + 2, dmh);
    uint8_t *s = b + 4;
    memset(s, 0, 12);
    for (int j = 0; j < 8; ++j) {           /* inverse of q4k_scale_min */
        if (j < 4) {
            s[j]     |= (uint8_t)sc[j];
            s[j + 4] |= (uint8_t)m[j];
        } else {
            s[j + 4] = (uint8_t)((sc[j] & 0xF) | ((m[j] & 0xF) << 4));
            s[j - 4] |= (uint8_t)((sc[j] >> 4) << 6);
            s[j]     |= (uint8_t)((m[j] >> 4) << 6);
        }
    }
    uint8_t q[256];
    for (int j = 0; j < 8; ++j) {
        const float dl = d * (float)sc[j], ml = dmin * (float)m[j];
        for (int i = 0; i < 32; ++i)
            q[32 * j + i] = (uint8_t)(dl > 0.f ? clampi(nearest_away((x[32 * j + i] + ml) / dl), 0, levels) : 0);
    }
    uint8_t *qs = b + (levels == 31 ? 48 : 16);
    for (int g = 0; g < 4; ++g)
        for (int i = 0; i < 32; ++i) qs[32 * g + i] = (uint8_t)((q[64 * g + i] & 0xF) | ((q[64 * g + 32 + i] & 0xF) << 4));
    if (levels == 31) {
        memset(b + 16, 0, 32);
        for (int j = 0; j < 8; ++j)
            for (int i = 0; i < 32; ++i) b[16 + i] |= (uint8_t)((q[32 * j + i] >> 4) << j);
    }
}
static void quantize_q4_K_standin(const float *x, uint8_t *b) { quantize_q45_K_standin(x, b, 15); }
static void quantize_q5_K_standin(const float *x, uint8_t *b) { quantize_q45_K_standin(x, b, 31); }



static void quantize_q6_K_standin(const float *x, uint8_t *b) {
    float scale[16], smax = 0.f;
    for (int g = 0; g < 16; ++g) {
        float amax = 0.f;
        for (int i = 0; i < 16; ++i) { const float a = fabsf(x[16 * g + i]); if (a > amax) amax = a; }
        scale[g] = amax / 31.f;
        if (scale[g] > smax) smax = scale[g];
    }
    const uint16_t dh = orc_fp32_to_fp16(smax / 127.f);
    const float d = orc_fp16_to_fp32(dh);
    uint8_t q[256];
    for (int g = 0; g < 16; ++g) {
        const int sc = d > 0.f ? clampi(nearest_away(scale[g] / d), 0, 127) : 0;
        b[192 + g] = (uint8_t)(int8_t)sc;
        const float dl = d * (float)sc;
        for (int i = 0; i < 16; ++i)
            q[16 * g + i] = (uint8_t)(dl > 0.f ? clampi(nearest_away(x[16 * g + i] / dl) + 32, 0, 63) : 32);
    }
    wr16(b + 208, dh);
    uint8_t *ql = b, *qh = b + 128;
    for (int n = 0; n < 2; ++n)
        for (int t = 0; t < 32; ++t) {
            const uint8_t q0 = q[128 * n + t], q1 = q[128 * n + 32 + t], q2 = q[128 * n + 64 + t], q3 = q[128 * n + 96 + t];
            ql[64 * n + t]      = (uint8_t)((q0 & 0xF) | ((q2 & 0xF) << 4));
            ql[64 * n + 32 + t] = (uint8_t)((q1 & 0xF) | ((q3 & 0xF) << 4));
            qh[32 * n + t]      = (uint8_t)((q0 >> 4) | ((q1 >> 4) << 2) | ((q2 >> 4) << 4) | ((q3 >> 4) << 6));
        }
}

static void quantize_iq4_xs_standin(const float *x, uint8_t *b) {
    float scale[8], smax = 0.f;
    for (int p = 0; p < 8; ++p) {
        float amax = 0.f;
        for (int i = 0; i < 32; ++i) { const float a = fabsf(x[32 * p + i]); if (a > amax) amax = a; }
        scale[p] = amax / 127.f;
        if (scale[p] > smax) smax = scale[p];
    }
    const uint16_t dh = orc_fp32_to_fp16(smax / 31.f);
    const float d = orc_fp16_to_fp32(dh);
    uint16_t sh = 0;
    uint8_t sl[4] = { 0, 0, 0, 0 };
    for (int p = 0; p < 8; ++p) {
        const int l = d > 0.f ? clampi(nearest_away(scale[p] / d), 0, 31) : 0;
        const int ls = l + 32;
        sl[p >> 1] |= (uint8_t)((ls & 0xF) << (4 * (p & 1)));
        sh |= (uint16_t)((ls >> 4) << (2 * p));
        const float dl = d * (float)l;
        uint8_t q[32];
        for (int i = 0; i < 32; ++i) {
            int best = 8;
            if (dl > 0.f) {
                const float v = x[32 * p + i] / dl;
                float be = INFINITY;
                for (int c = 0; c < 16; ++c) {
                    const float e = fabsf(v - (float)KV_IQ4NL[c]);
                    if (e < be) { be = e; best = c; }
                }
            }
            q[i] = (uint8_t)best;
        }
        for (int j = 0; j < 16; ++j) b[8 + 16 * p + j] = (uint8_t)(q[j] | (q[j + 16] << 4));
    }
    wr16(b, dh);
    wr16(b + 2, sh);
    memcpy(b + 4, sl, 4);
}

/* stand-in: d = amax / 127 with the sign of the largest element's partner value (kv[0] = -127), nearest codebook entry */
static void quantize_iq4_nl_standin(const float *x, uint8_t *b) {
    float amax = 0.f, vmax = 0.f;
    for (int i = 0; i < 32; ++i) { const float a = fabsf(x[i]); if (a > amax) { amax = a; vmax = x[i]; } }
    const uint16_t dh = orc_fp32_to_fp16(vmax / -127.f);        /* the largest element lands on kv[0] = -127 */
    const float d = orc_fp16_to_fp32(dh);
    uint8_t q[32];
    for (int i = 0; i < 32; ++i) {
        int best = 8;
        if (d != 0.f) {
            const float v = x[i] / d;
            float be = INFINITY;
            for (int c = 0; c < 16; ++c) {
                const float e = fabsf(v - (float)KV_IQ4NL[c]);
                if (e < be) { be = e; best = c; }
            }
        }
        q[i] = (uint8_t)best;
    }
    wr16(b, dh);
    for (int j = 0; j < 16; ++j) b[2 + j] = (uint8_t)(q[j] | (q[j + 16] << 4));
}

int orc_quantize_row(int type, const float *src, void *dst, int64_t k) {
    const int bs = orc_block_size(type);
    if (!bs || k % bs) return -1;
    uint8_t *b = (uint8_t *)dst;
    const size_t bb = orc_block_bytes(type);
    for (int64_t ib = 0; ib < k / bs; ++ib, b += bb, src += bs) {
        switch (type) {
        case ORC_TYPE_Q4_0:   quantize_q4_0(src, b); break;
        case ORC_TYPE_Q8_0:   quantize_q8_0(src, b); break;
        case ORC_TYPE_Q4_K:   quantize_q4_K_standin(src, b); break;
        case ORC_TYPE_Q5_K:   quantize_q5_K_standin(src, b); break;
        case ORC_TYPE_Q6_K:   quantize_q6_K_standin(src, b); break;
        case ORC_TYPE_IQ4_XS: quantize_iq4_xs_standin(src, b); break;
        case ORC_TYPE_IQ4_NL: quantize_iq4_nl_standin(src, b); break;
        default: return -1;
        }
    }
    return 0;
}

int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* 0: the OpenMP default (OMP_NUM_THREADS); an explicit count may go up to the processor count, so a
 * launcher that pins OMP_NUM_THREADS=1 does not decide the baseline's core count */
static int pick_threads(int nthreads) {
    const int mx = orc_num_threads();
    if (nthreads <= 0) return mx;
#ifdef _OPENMP
    const int np = omp_get_num_procs();
    return nthreads > np ? np : nthreads;
#else
    return 1;
#endif
}

int orc_quantize_rows(int type, const float *src, void *dst, int64_t nrows, int64_t k, int nthreads) {
    const size_t rb = orc_row_bytes(type, k);
    if (!rb) return -1;
    const int nt = pick_threads(nthreads);
    (void)nt;
    #pragma omp parallel for num_threads(nt) schedule(static)
    for (int64_t r = 0; r < nrows; ++r) orc_quantize_row(type, src + r * k, (uint8_t *)dst + r * rb, k);
    return 0;
}

/* -------------------------------------------------- activation quantizers */

/* ggml block_q8_0 rule per 32 (gguf-py Q8_0.quantize_blocks); the reference's per-32
 * quantizer kq_i8_quant32 (P09:544-553) is the same grid with 127/amax as the inverse */
void orc_quantize_act_q8_0(const float *x, int8_t *q, uint16_t *d, int64_t k) {
    for (int64_t b = 0; b < k / 32; ++b) {
        float amax = 0.f;
        for (int i = 0; i < 32; ++i) { const float a = fabsf(x[32 * b + i]); if (a > amax) amax = a; }
        const float dd = amax / 127.f;
        const float id = dd != 0.f ? 1.f / dd : 0.f;
        d[b] = orc_fp32_to_fp16(dd);
        for (int i = 0; i < 32; ++i) q[32 * b + i] = (int8_t)nearest_away(x[32 * b + i] * id);
    }
}

/* reference kernel_quant_i8 (P01:1862-1889): per 256, scale bm/127, codes rint(v * 127/bm),
 * zero below 1e-30, integer sums of each 32 */
void orc_quantize_act_q8_256(const float *x, int8_t *q, float *d, int16_t *bsums, int64_t k) {
    for (int64_t b = 0; b < k / 256; ++b) {
        float bm = 0.f;
        for (int i = 0; i < 256; ++i) { const float a = fabsf(x[256 * b + i]); if (a > bm) bm = a; }
        const float iq = bm > 1e-30f ? 127.f / bm : 0.f;
        d[b] = bm / 127.f;
        for (int s = 0; s < 8; ++s) {
            int sum = 0;
            for (int i = 0; i < 32; ++i) {
                const int v = (int)rintf(x[256 * b + 32 * s + i] * iq);
                q[256 * b + 32 * s + i] = (int8_t)v;
                sum += v;
            }
            bsums[8 * b + s] = (int16_t)sum;
        }
    }
}

void orc_dequantize_act(int form, const int8_t *q, const void *d, float *dst, int64_t k) {
    if (form == ORC_ACT_Q8_0) {
        const uint16_t *dh = (const uint16_t *)d;
        for (int64_t i = 0; i < k; ++i) dst[i] = orc_fp16_to_fp32(dh[i / 32]) * (float)q[i];
    } else {
        const float *df = (const float *)d;
        for (int64_t i = 0; i < k; ++i) dst[i] = df[i / 256] * (float)q[i];
    }
}

/* ------------------------------------------------------------ the product */

typedef struct {
    int      form;
    int64_t  k;
    int8_t  *q;       /* [n][k]        */
    uint16_t *d16;    /* [n][k/32]     (Q8_0 form)   */
    float   *d32;     /* [n][k/256]    (Q8_256 form) */
    int16_t *bsums;   /* [n][k/32]     (Q8_256 form) */
} act_t;

static int act_alloc(act_t *a, int form, int64_t k, int64_t n) {
    memset(a, 0, sizeof(*a));
    a->form = form;
    a->k = k;
    a->q = (int8_t *)malloc((size_t)(n * k) + 64);
    if (form == ORC_ACT_Q8_0) a->d16 = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)(n * (k / 32)) + 64);
    else {
        a->d32 = (float *)malloc(sizeof(float) * (size_t)(n * (k / 256)) + 64);
        a->bsums = (int16_t *)malloc(sizeof(int16_t) * (size_t)(n * (k / 32)) + 64);
    }
    return a->q && (a->d16 || (a->d32 && a->bsums)) ? 0 : -1;
}

static void act_free(act_t *a) { free(a->q); free(a->d16); free(a->d32); free(a->bsums); }

static void act_quantize_col(act_t *a, int64_t col, const float *x) {
    if (a->form == ORC_ACT_Q8_0) orc_quantize_act_q8_0(x, a->q + col * a->k, a->d16 + col * (a->k / 32), a->k);
    else orc_quantize_act_q8_256(x, a->q + col * a->k, a->d32 + col * (a->k / 256), a->bsums + col * (a->k / 32), a->k);
}

static inline int dot_s8(const int8_t *a, const int8_t *b, int n) {
    int s = 0;
    for (int i = 0; i < n; ++i) s += (int)a[i] * (int)b[i];
    return s;
}

/* one weight row expanded to integer codes + per-block factors, reused for every column */
typedef struct {
    int8_t *q;       /* [k] signed codes (Q4_K: 0..15) */
    float  *f0;      /* per 32-block: d (Q4_0/Q8_0);  per 256: d (K types)       */
    float  *f1;      /* Q4_K: dmin per 256                                      */
    int8_t *isc;     /* integer sub-scales: Q4_K sc[8]/256, Q6_K sc[16]/256, IQ4_XS ls-32 [8]/256 */
    uint8_t *imn;    /* Q4_K mins m[8]/256 */
} rowx_t;

static int rowx_alloc(rowx_t *r, int64_t k) {
    r->q = (int8_t *)malloc((size_t)k + 64);
    r->f0 = (float *)malloc(sizeof(float) * (size_t)(k / 32) + 64);
    r->f1 = (float *)malloc(sizeof(float) * (size_t)(k / 32) + 64);
    r->isc = (int8_t *)malloc((size_t)(k / 16) + 64);
    r->imn = (uint8_t *)malloc((size_t)(k / 16) + 64);
    return r->q && r->f0 && r->f1 && r->isc && r->imn ? 0 : -1;
}

static void rowx_free(rowx_t *r) { free(r->q); free(r->f0); free(r->f1); free(r->isc); free(r->imn); }

static void rowx_expand(rowx_t *r, int type, const uint8_t *row, int64_t k) {
    const size_t bb = orc_block_bytes(type);
    const int bs = orc_block_size(type);
    for (int64_t ib = 0; ib < k / bs; ++ib) {
        const uint8_t *b = row + ib * bb;
        switch (type) {
        case ORC_TYPE_Q4_0:
            q4_0_codes(b, r->q + 32 * ib);
            r->f0[ib] = orc_fp16_to_fp32(rd16(b));
            break;
        case ORC_TYPE_Q8_0:
            memcpy(r->q + 32 * ib, b + 2, 32);
            r->f0[ib] = orc_fp16_to_fp32(rd16(b));
            break;
        case ORC_TYPE_IQ4_NL:
            iq4_nl_codes(b, r->q + 32 * ib);
            r->f0[ib] = orc_fp16_to_fp32(rd16(b));
            break;
        case ORC_TYPE_Q4_K:
        case ORC_TYPE_Q5_K:
            if (type == ORC_TYPE_Q4_K) q4_K_codes(b, (uint8_t *)r->q + 256 * ib);
            else q5_K_codes(b, (uint8_t *)r->q + 256 * ib);
            r->f0[ib] = orc_fp16_to_fp32(rd16(b));
            r->f1[ib] = orc_fp16_to_fp32(rd16(b + 2));
            for (int j = 0; j < 8; ++j) {
                int sc, m;
                q4k_scale_min(b + 4, j, &sc, &m);
                r->isc[8 * ib + j] = (int8_t)sc;
                r->imn[8 * ib + j] = (uint8_t)m;
            }
            break;
        case ORC_TYPE_Q6_K:
            q6_K_codes(b, r->q + 256 * ib);
            r->f0[ib] = orc_fp16_to_fp32(rd16(b + 208));
            memcpy(r->isc + 16 * ib, b + 192, 16);
            break;
        case ORC_TYPE_IQ4_XS:
            iq4_xs_codes(b, r->q + 256 * ib);
            r->f0[ib] = orc_fp16_to_fp32(rd16(b));
            for (int p = 0; p < 8; ++p) r->isc[8 * ib + p] = (int8_t)(iq4xs_ls(b, p) - 32);
            break;
        }
    }
}

/*
 * ggml-form dot of an expanded row with one quantized column. Block dots are
 * exact integers; float enters once per 32 (Q4_0, Q8_0: the reference's
 * af = fma(float(ir), d_w, af) form, P99:430-442) or once per 256 (K types:
 * integer sub-scale accumulation, P01:1986-2011, P103:482-490).
 */
static float rowx_dot(const rowx_t *r, int type, const act_t *a, int64_t col) {
    const int64_t k = a->k;
    const int8_t *xq = a->q + col * k;
    float sum = 0.f;
    switch (type) {
    case ORC_TYPE_Q4_0:
    case ORC_TYPE_Q8_0:
    case ORC_TYPE_IQ4_NL: {
        const uint16_t *xd = a->d16 + col * (k / 32);
        for (int64_t ib = 0; ib < k / 32; ++ib) {
            const int si = dot_s8(r->q + 32 * ib, xq + 32 * ib, 32);
            sum += ((float)si * r->f0[ib]) * orc_fp16_to_fp32(xd[ib]);
        }
    } break;
    case ORC_TYPE_Q4_K:
    case ORC_TYPE_Q5_K: {
        const float *xd = a->d32 + col * (k / 256);
        const int16_t *bs = a->bsums + col * (k / 32);
        for (int64_t ib = 0; ib < k / 256; ++ib) {
            int si = 0, sm = 0;
            for (int j = 0; j < 8; ++j) {
                int s = 0;
                const uint8_t *wq = (const uint8_t *)r->q + 256 * ib + 32 * j;
                for (int i = 0; i < 32; ++i) s += (int)wq[i] * (int)xq[256 * ib + 32 * j + i];
                si += s * (int)r->isc[8 * ib + j];
                sm += (int)bs[8 * ib + j] * (int)r->imn[8 * ib + j];
            }
            sum += xd[ib] * (r->f0[ib] * (float)si - r->f1[ib] * (float)sm);
        }
    } break;
    case ORC_TYPE_Q6_K: {
        const float *xd = a->d32 + col * (k / 256);
        for (int64_t ib = 0; ib < k / 256; ++ib) {
            int si = 0;
            for (int g = 0; g < 16; ++g)
                si += dot_s8(r->q + 256 * ib + 16 * g, xq + 256 * ib + 16 * g, 16) * (int)r->isc[16 * ib + g];
            sum += (xd[ib] * r->f0[ib]) * (float)si;
        }
    } break;
    case ORC_TYPE_IQ4_XS: {
        const float *xd = a->d32 + col * (k / 256);
        for (int64_t ib = 0; ib < k / 256; ++ib) {
            int si = 0;
            for (int p = 0; p < 8; ++p)
                si += dot_s8(r->q + 256 * ib + 32 * p, xq + 256 * ib + 32 * p, 32) * (int)r->isc[8 * ib + p];
            sum += (xd[ib] * r->f0[ib]) * (float)si;
        }
    } break;
    }
    return sum;
}

static int type_ok(int type, int64_t k) {
    const int bs = orc_block_size(type);
    return bs && k > 0 && k % bs == 0;
}

int orc_mul_mat(int type, const void *w, int64_t m, int64_t k,
                const float *x, int64_t n, int64_t ldx,
                float *dst, int64_t ldd, int nthreads) {
    if (!type_ok(type, k)) return -1;
    const int nt = pick_threads(nthreads);
    const size_t rb = orc_row_bytes(type, k);
    act_t a;
    if (act_alloc(&a, orc_act_form(type), k, n)) return -2;
    #pragma omp parallel for num_threads(nt) schedule(static)
    for (int64_t c = 0; c < n; ++c) act_quantize_col(&a, c, x + c * ldx);
    int err = 0;
    #pragma omp parallel num_threads(nt)
    {
        rowx_t r;
        if (rowx_alloc(&r, k)) {
            #pragma omp atomic write
            err = -2;
        } else {
            #pragma omp for schedule(dynamic, 8)
            for (int64_t row = 0; row < m; ++row) {
                rowx_expand(&r, type, (const uint8_t *)w + row * rb, k);
                for (int64_t c = 0; c < n; ++c) dst[row + c * ldd] = rowx_dot(&r, type, &a, c);
            }
        }
        rowx_free(&r);
    }
    act_free(&a);
    return err;
}

int orc_mul_mat_f64(int type, const void *w, int64_t m, int64_t k,
                    const float *x, int64_t n, int64_t ldx,
                    double *dst, int64_t ldd, int quantized_act, int nthreads) {
    if (!type_ok(type, k)) return -1;
    const int nt = pick_threads(nthreads);
    const size_t rb = orc_row_bytes(type, k);
    double *xa = (double *)malloc(sizeof(double) * (size_t)(n * k));   /* d * q exactly, no f32 rounding */
    if (!xa) return -2;
    #pragma omp parallel for num_threads(nt) schedule(static)
    for (int64_t c = 0; c < n; ++c) {
        if (quantized_act) {
            act_t a;
            if (act_alloc(&a, orc_act_form(type), k, 1) == 0) {
                act_quantize_col(&a, 0, x + c * ldx);
                for (int64_t i = 0; i < k; ++i) {
                    const double d = a.form == ORC_ACT_Q8_0 ? (double)orc_fp16_to_fp32(a.d16[i / 32]) : (double)a.d32[i / 256];
                    xa[c * k + i] = d * (double)a.q[i];
                }
            }
            act_free(&a);
        } else {
            for (int64_t i = 0; i < k; ++i) xa[c * k + i] = (double)x[c * ldx + i];
        }
    }
    #pragma omp parallel num_threads(nt)
    {
        float *wr = (float *)malloc(sizeof(float) * (size_t)k);
        #pragma omp for schedule(dynamic, 8)
        for (int64_t row = 0; row < m; ++row) {
            orc_dequantize_row(type, (const uint8_t *)w + row * rb, wr, k);
            for (int64_t c = 0; c < n; ++c) {
                double s = 0.0;
                const double *xc = xa + c * k;
                for (int64_t i = 0; i < k; ++i) s += (double)wr[i] * xc[i];
                dst[row + c * ldd] = s;
            }
        }
        free(wr);
    }
    free(xa);
    return 0;
}

/* MUL_MAT_ID (P01:3917-3934): pair (i,t) -> expert ids[t][i], column (i % ne11) + t*ne11
 * (kq_i8_col, P09:573-577), output dst + (t*n_used + i)*m */
int orc_mul_mat_id(int type, const void *w, int64_t m, int64_t k, int n_expert,
                   const float *x, int ne11, int n_tok,
                   const int32_t *ids, int64_t ids_stride, int n_used,
                   float *dst, int nthreads) {
    if (!type_ok(type, k) || ne11 <= 0) return -1;
    const size_t eb = orc_row_bytes(type, k) * (size_t)m;
    for (int t = 0; t < n_tok; ++t)
        for (int i = 0; i < n_used; ++i) {
            const int e = ids[t * ids_stride + i];
            if (e < 0 || e >= n_expert) return -3;
            const int64_t col = (i % ne11) + (int64_t)t * ne11;
            const int rc = orc_mul_mat(type, (const uint8_t *)w + (size_t)e * eb, m, k, x + col * k, 1, k,
                                       dst + ((int64_t)t * n_used + i) * m, m, nthreads);
            if (rc) return rc;
        }
    return 0;
}

int orc_mul_mat_id_f64(int type, const void *w, int64_t m, int64_t k, int n_expert,
                       const float *x, int ne11, int n_tok,
                       const int32_t *ids, int64_t ids_stride, int n_used,
                       double *dst, int quantized_act, int nthreads) {
    if (!type_ok(type, k) || ne11 <= 0) return -1;
    const size_t eb = orc_row_bytes(type, k) * (size_t)m;
    for (int t = 0; t < n_tok; ++t)
        for (int i = 0; i < n_used; ++i) {
            const int e = ids[t * ids_stride + i];
            if (e < 0 || e >= n_expert) return -3;
            const int64_t col = (i % ne11) + (int64_t)t * ne11;
            const int rc = orc_mul_mat_f64(type, (const uint8_t *)w + (size_t)e * eb, m, k, x + col * k, 1, k,
                                           dst + ((int64_t)t * n_used + i) * m, m, quantized_act, nthreads);
            if (rc) return rc;
        }
    return 0;
}

/* kernel_moe_route_tiles (P01:2417-2444) with the scatter made stable in p: the
 * reference's atomic scatter leaves the order inside an expert unspecified */
int orc_moe_route(const int32_t *ids, int64_t ids_stride, int n_used, int n_tok, int n_expert,
                  int tile, int32_t *pairs, int32_t *tiles) {
    const int n_pairs = n_used * n_tok;
    int *cnt = (int *)calloc((size_t)n_expert, sizeof(int));
    int *base = (int *)calloc((size_t)n_expert, sizeof(int));
    if (!cnt || !base) { free(cnt); free(base); return -2; }
    for (int p = 0; p < n_pairs; ++p) {
        const int e = clampi(ids[(p / n_used) * ids_stride + p % n_used], 0, n_expert - 1);
        ++cnt[e];
    }
    int acc = 0, nt = 0;
    for (int e = 0; e < n_expert; ++e) {
        base[e] = acc;
        for (int s0 = 0; s0 < cnt[e]; s0 += tile) {
            tiles[4 * nt + 0] = e;
            tiles[4 * nt + 1] = acc + s0;
            tiles[4 * nt + 2] = cnt[e] - s0 < tile ? cnt[e] - s0 : tile;
            tiles[4 * nt + 3] = 0;
            ++nt;
        }
        acc += cnt[e];
        cnt[e] = 0;
    }
    for (int p = 0; p < n_pairs; ++p) {
        const int e = clampi(ids[(p / n_used) * ids_stride + p % n_used], 0, n_expert - 1);
        pairs[base[e] + cnt[e]++] = p;
    }
    free(cnt);
    free(base);
    return nt;
}

/* ----------------------------------------------------------- seeded inputs */

static inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

/* value i of stream `seed`: Box-Muller on two hashes of the pair index */
static inline float normal_at(uint64_t seed, int64_t i) {
    const uint64_t pair = (uint64_t)(i >> 1);
    const uint64_t h1 = splitmix64(seed ^ splitmix64(2 * pair));
    const uint64_t h2 = splitmix64(seed ^ splitmix64(2 * pair + 1));
    const double u1 = ((double)(h1 >> 11) + 1.0) * (1.0 / 9007199254740993.0);   /* (0,1) */
    const double u2 = (double)(h2 >> 11) * (1.0 / 9007199254740992.0);
    const double r = sqrt(-2.0 * log(u1)), th = 6.283185307179586476925 * u2;
    return (float)((i & 1) ? r * sin(th) : r * cos(th));
}

void orc_fill_normal(float *dst, int64_t n, uint64_t seed, float sigma, int nthreads) {
    const int nt = pick_threads(nthreads);
    (void)nt;
    #pragma omp parallel for num_threads(nt) schedule(static)
    for (int64_t i = 0; i < n; ++i) dst[i] = sigma * normal_at(seed, i);
}

/* Zipf(s) expert popularity p_e ~ rank_e^-s over a fixed seeded permutation of the
 * experts; each token draws n_used distinct experts from it (Gumbel top-k:
 * logit_e = -s ln(rank_e) - ln(-ln u)), top-n_used by value, ties to the lower id
 * (the reference's top-k rule, P09:901-903) */
void orc_route_ids(int32_t *ids, int n_used, int n_tok, int n_expert, uint64_t seed, float zipf_s) {
    int *rank = (int *)malloc(sizeof(int) * (size_t)n_expert);
    float *logit = (float *)malloc(sizeof(float) * (size_t)n_expert);
    for (int e = 0; e < n_expert; ++e) rank[e] = e;
    for (int e = n_expert - 1; e > 0; --e) {        /* Fisher-Yates */
        const int j = (int)(splitmix64(seed ^ (0xABCD0000ull + (uint64_t)e)) % (uint64_t)(e + 1));
        const int t = rank[e]; rank[e] = rank[j]; rank[j] = t;
    }
    for (int t = 0; t < n_tok; ++t) {
        for (int e = 0; e < n_expert; ++e) {
            const uint64_t h = splitmix64((seed + 1) ^ splitmix64((uint64_t)t * (uint64_t)n_expert + (uint64_t)e));
            const double u = ((double)(h >> 11) + 0.5) * (1.0 / 9007199254740992.0);
            logit[e] = (float)(-(double)zipf_s * log((double)(rank[e] + 1)) - log(-log(u)));
        }
        for (int i = 0; i < n_used; ++i) {
            int best = -1;
            for (int e = 0; e < n_expert; ++e)
                if (logit[e] > -INFINITY && (best < 0 || logit[e] > logit[best])) best = e;
            ids[t * n_used + i] = best;
            logit[best] = -INFINITY;
        }
    }
    free(rank);
    free(logit);
}
