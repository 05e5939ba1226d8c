// gemv_core.cuh -- what ONE LANE of the decode GEMV does. Host+device text: the kernel
// (gemv_kernel.cuh) calls it from the 32 lanes of a warp; the device-free emulation
// (emul.cpp) calls it for lane 0..31 in turn.
//
// A "stage" is 2048 weights of a row (64 per lane); its byte size is a multiple of 16 for
// every type, so stages are fetched with 16-byte copies:
//   Q4_0 64 blocks = 1152 B   Q8_0 64 blocks = 2176 B   Q4_K 8 blocks = 1152 B
//   IQ4_XS 8 blocks = 1088 B  Q6_K 8 blocks = 1680 B    Q5_K 8 blocks = 1408 B
// Work is split in two so the activation side is paid once per stage, not once per row:
//   gemv_load_x   loads the lane's 64 activation codes, scales and block sums of NC columns
//                 for stage s into registers (GemvX);
//   gemv_lane_row multiplies one staged weight row chunk against them.
// A B200 SM receives ~23 weight bytes per clock, i.e. about 100 lane instructions per 32
// four-bit weights, so the lane code is written for instruction count: nibbles stay
// unsigned (the -8 / -32 offsets ride on the activation block sums the quantizer already
// made), high nibbles are multiplied in place (x16, unsigned dp4a) and the 1/16 is folded
// into the float scale, sub-scales are unpacked four at a time.
//
// Integer block dots are exact (dp4a against the int8 activation codes); float enters once
// per 32 (Q4_0/Q8_0: d_w * d_x) or once per 256-block (K types: integer sub-scales first),
// the form of ggml's CPU vec_dot and of the reference GEMV bodies mv_q45_K / mv_q6_K /
// mv_q4_0 / mv_iq (marfrit/arcint contrib/llama.cpp/patches/
// 0000-01-kquant-integer-dpas.patch:3740-3874, 0000-02-lowbit-iq-types.patch:5947-5955,
// 6100-6130) without their residual term.
//
// Red cases (the reference ships a mutant switch with every kernel patch that must turn its suite red:
// -DQ40_RED 0099-opencl-q4_0-q8_0-int8-gemm.patch:304-310, -DID_RED 0103-opencl-id-int8-sg8.patch:338-343,
// -DFEWQ_RED 0115-...patch:742-746): -DB200Q_RED_Q40 takes the Q4_0 codes as n - 4, -DB200Q_RED_SCALE negates
// the Q4_K block scale, -DB200Q_RED_DROP skips every eighth 32-block of Q4_0 / Q8_0. Test builds only.
#pragma once

#include "formats.cuh"

namespace b200q {

template <int TYPE> struct GemvFmt;
template <> struct GemvFmt<B200Q_TYPE_Q4_0>   { enum { BLK_W = 32,  BLK_B = 18,  STAGE_BLOCKS = 64 }; };
template <> struct GemvFmt<B200Q_TYPE_Q8_0>   { enum { BLK_W = 32,  BLK_B = 34,  STAGE_BLOCKS = 64 }; };
template <> struct GemvFmt<B200Q_TYPE_IQ4_NL> { enum { BLK_W = 32,  BLK_B = 18,  STAGE_BLOCKS = 64 }; };
template <> struct GemvFmt<B200Q_TYPE_Q4_K>   { enum { BLK_W = 256, BLK_B = 144, STAGE_BLOCKS = 8 }; };
template <> struct GemvFmt<B200Q_TYPE_Q5_K>   { enum { BLK_W = 256, BLK_B = 176, STAGE_BLOCKS = 8 }; };
template <> struct GemvFmt<B200Q_TYPE_IQ4_XS> { enum { BLK_W = 256, BLK_B = 136, STAGE_BLOCKS = 8 }; };
template <> struct GemvFmt<B200Q_TYPE_Q6_K>   { enum { BLK_W = 256, BLK_B = 210, STAGE_BLOCKS = 8 }; };

template <int TYPE> struct GemvStage {
    enum { BYTES = GemvFmt<TYPE>::STAGE_BLOCKS * GemvFmt<TYPE>::BLK_B,     // multiple of 16
           SLOT  = ((BYTES + 4 + 15) / 16) * 16 };                         // + one word of over-read
};

// Activation pointers already offset to the first column of this launch.
struct GemvAct {
    const int8_t   *q;     // [ ][K]      codes
    const uint16_t *d16;   // [ ][K/32]   per-32 form: fp16 scales
    const float    *d32;   // [ ][K/256]  per-256 form: f32 scales
    const int16_t  *s32;   // [ ][K/32]   sums of each 32 codes (both forms)
    const int16_t  *s16;   // [ ][K/16]   sums of each 16 codes (per-256 form)
    int             K;
    // the f32 activation itself, for the kernels that quantize their slice on the fly: column c at xf + c * xf_stride
    const float    *xf;
    int64_t         xf_stride;
};

// signed x signed and unsigned x signed 4-way byte dot products
B200Q_HD int dp4a_ss(uint32_t a, int b, int c) { return hd_dp4a(a, b, c); }
B200Q_HD int dp4a_us(uint32_t a, int b, int c) {
#ifdef __CUDA_ARCH__
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
#else
    for (int i = 0; i < 4; ++i) c += (int)(uint8_t)(a >> (8 * i)) * (int)(int8_t)((uint32_t)b >> (8 * i));
    return c;
#endif
}

// two signed 16-bit halves of a times the two low unsigned bytes of b, summed into c
B200Q_HD int dp2a_lo_su(uint32_t a, uint32_t b, int c) {
#ifdef __CUDA_ARCH__
    int d;
    asm("dp2a.lo.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
#else
    return c + (int)(int16_t)(a & 0xFFFFu) * (int)(b & 0xFFu) + (int)(int16_t)(a >> 16) * (int)((b >> 8) & 0xFFu);
#endif
}

B200Q_HD int ld_s16(const int16_t *p) {
#ifdef __CUDA_ARCH__
    return (int)__ldg(p);
#else
    return (int)*p;
#endif
}
B200Q_HD uint32_t ld_u32(const void *p) {
#ifdef __CUDA_ARCH__
    return __ldg(reinterpret_cast<const unsigned int *>(p));
#else
    uint32_t v;
    memcpy(&v, p, 4);
    return v;
#endif
}
B200Q_HD float ld_f32(const float *p) {
#ifdef __CUDA_ARCH__
    return __ldg(p);
#else
    return *p;
#endif
}
B200Q_HD uint16_t ld_u16(const uint16_t *p) {
#ifdef __CUDA_ARCH__
    return __ldg(p);
#else
    return *p;
#endif
}
B200Q_HD int sext8(uint32_t v) { return (int)(int8_t)(v & 0xFFu); }
B200Q_HD int sext16(uint32_t v) { return (int)(int16_t)(v & 0xFFFFu); }

// The lane's activation registers for one stage: 64 codes per column plus what the type's
// scale/offset terms need. f0/f1: float factors; i0..i3: integer terms.
template <int NC> struct GemvX {
    I4    x[NC][4];
    float f0[NC], f1[NC];
    int   i0[NC], i1[NC], i2[NC], i3[NC];
    bool  live;           // the lane's block exists in this stage (ragged last stage)
    bool  live2;          // Q4_0/Q8_0: the lane's second block exists
};

// cols[c]: which column of the quantized activation buffer column c of this launch is (the
// identity for a dense product, a routed pair's column for MUL_MAT_ID).
template <int TYPE, int NC>
B200Q_HD void gemv_load_x(int lane, int s, int nblk, const GemvAct &act, const int (&cols)[NC], GemvX<NC> &X) {
    typedef GemvFmt<TYPE> F;
    const int K = act.K;
    if (TYPE == B200Q_TYPE_Q4_0 || TYPE == B200Q_TYPE_Q8_0 || TYPE == B200Q_TYPE_IQ4_NL) {
        // two 32-blocks per lane: lane and lane + 32 of the stage
        const int b0 = s * F::STAGE_BLOCKS + lane, b1 = b0 + 32;
        X.live = b0 < nblk;
        X.live2 = b1 < nblk;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int8_t *xp = act.q + (size_t)cols[c] * K;
            const size_t sc = (size_t)cols[c] * (K / 32);
            if (X.live) {
                X.x[c][0] = hd_ld16(xp + 32 * b0);
                X.x[c][1] = hd_ld16(xp + 32 * b0 + 16);
                X.f0[c] = hd_half_bits(ld_u16(act.d16 + sc + b0));
                if (TYPE == B200Q_TYPE_Q4_0) {
#ifdef B200Q_RED_Q40
                    X.i0[c] = -64 * ld_s16(act.s32 + sc + b0);
#else
                    X.i0[c] = -128 * ld_s16(act.s32 + sc + b0);      // -8 * 16 * sum(x)
#endif
                    X.f0[c] *= 0.0625f;                              // the nibble dot is kept x16
                }
            }
            if (X.live2) {
                X.x[c][2] = hd_ld16(xp + 32 * b1);
                X.x[c][3] = hd_ld16(xp + 32 * b1 + 16);
                X.f1[c] = hd_half_bits(ld_u16(act.d16 + sc + b1));
                if (TYPE == B200Q_TYPE_Q4_0) {
                    X.i1[c] = -128 * ld_s16(act.s32 + sc + b1);
                    X.f1[c] *= 0.0625f;
                }
            }
        }
    } else if (TYPE == B200Q_TYPE_Q4_K || TYPE == B200Q_TYPE_Q5_K) {
        // lane -> block sb of the stage and 32-byte group g: sub-blocks 2g (low nibbles) and
        // 2g+1 (high nibbles), 64 weights
        const int sb = lane >> 2, g = lane & 3, blk = s * F::STAGE_BLOCKS + sb;
        X.live = blk < nblk;
        if (!X.live) return;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int8_t *xp = act.q + (size_t)cols[c] * K + 256 * blk + 64 * g;
#pragma unroll
            for (int j = 0; j < 4; ++j) X.x[c][j] = hd_ld16(xp + 16 * j);
            X.f0[c] = ld_f32(act.d32 + (size_t)cols[c] * (K / 256) + blk);
            // the sums of the lane's two sub-blocks, kept as the pair of 16-bit halves they are stored as
            X.i0[c] = (int)ld_u32(act.s32 + (size_t)cols[c] * (K / 32) + 8 * blk + 2 * g);
        }
    } else if (TYPE == B200Q_TYPE_IQ4_XS) {
        // lane -> block sb and sub-block pair pp: 32 bytes = sub-blocks 2pp and 2pp+1
        const int sb = lane >> 2, pp = lane & 3, blk = s * F::STAGE_BLOCKS + sb;
        X.live = blk < nblk;
        if (!X.live) return;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int8_t *xp = act.q + (size_t)cols[c] * K + 256 * blk + 64 * pp;
#pragma unroll
            for (int j = 0; j < 4; ++j) X.x[c][j] = hd_ld16(xp + 16 * j);
            X.f0[c] = ld_f32(act.d32 + (size_t)cols[c] * (K / 256) + blk);
        }
    } else if (TYPE == B200Q_TYPE_Q6_K) {
        // lane -> block sb, half n, positions t0..t0+15 of the four 32-weight parts of that
        // half: each part's 16 weights are exactly one scale group
        const int sb = lane >> 2, n = (lane >> 1) & 1, hi16 = lane & 1, t0 = 16 * hi16;
        const int blk = s * F::STAGE_BLOCKS + sb;
        X.live = blk < nblk;
        if (!X.live) return;
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int8_t *xp = act.q + (size_t)cols[c] * K + 256 * blk + 128 * n + t0;
#pragma unroll
            for (int p = 0; p < 4; ++p) X.x[c][p] = hd_ld16(xp + 32 * p);
            X.f0[c] = ld_f32(act.d32 + (size_t)cols[c] * (K / 256) + blk);
            // sums of groups 8n + 2p + hi16, p = 0..3: eight int16 from one 16-byte load
            const I4 sv = hd_ld16(act.s16 + (size_t)cols[c] * (K / 16) + 16 * blk + 8 * n);
            X.i0[c] = -32 * sext16((uint32_t)sv.x >> (16 * hi16));     // sum((q-32) x) = sum(q x) - 32 sum(x)
            X.i1[c] = -32 * sext16((uint32_t)sv.y >> (16 * hi16));
            X.i2[c] = -32 * sext16((uint32_t)sv.z >> (16 * hi16));
            X.i3[c] = -32 * sext16((uint32_t)sv.w >> (16 * hi16));
        }
    }
}

// sw: the staged words of one weight row for the stage X was loaded for. acc[c] += partial.
template <int TYPE, int NC>
B200Q_HD void gemv_lane_row(const uint32_t *sw_ptr, int lane, const GemvX<NC> &X, float (&acc)[NC]) {
    typedef GemvFmt<TYPE> F;
    const Stage sw(sw_ptr);
    if (TYPE == B200Q_TYPE_Q4_0) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (!(u ? X.live2 : X.live)) continue;
#ifdef B200Q_RED_DROP
            if (((32 * u + lane) & 7) == 7) continue;
#endif
            const uint32_t off = (uint32_t)F::BLK_B * (uint32_t)(32 * u + lane);
            const float d = hd_half_bits(stage_u16(sw, off));
            uint32_t q[4];
            stage_words<4>(sw, off + 2, q);
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                // weights 4j..4j+3 in the low nibbles, 16+4j.. in the high ones (left x16)
                const I4 xa = X.x[c][2 * u], xb = X.x[c][2 * u + 1];
                int lo0 = dp4a_ss(q[0] & 0x0F0F0F0Fu, xa.x, 0), lo1 = dp4a_ss(q[1] & 0x0F0F0F0Fu, xa.y, 0);
                lo0 = dp4a_ss(q[2] & 0x0F0F0F0Fu, xa.z, lo0);   lo1 = dp4a_ss(q[3] & 0x0F0F0F0Fu, xa.w, lo1);
                int hi0 = dp4a_us(q[0] & 0xF0F0F0F0u, xb.x, u ? X.i1[c] : X.i0[c]);
                int hi1 = dp4a_us(q[1] & 0xF0F0F0F0u, xb.y, 0);
                hi0 = dp4a_us(q[2] & 0xF0F0F0F0u, xb.z, hi0);   hi1 = dp4a_us(q[3] & 0xF0F0F0F0u, xb.w, hi1);
                const int si = 16 * (lo0 + lo1) + (hi0 + hi1);                // 16 * sum((n - 8) x)
                acc[c] += (float)si * (d * (u ? X.f1[c] : X.f0[c]));
            }
        }
    } else if (TYPE == B200Q_TYPE_IQ4_NL) {
        // Q4_0's block with the nibbles as indices into kvalues_iq4nl: the codebook values are signed bytes, so no
        // offset term; the lookup (byte permutes) is shared by all columns
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (!(u ? X.live2 : X.live)) continue;
            const uint32_t off = (uint32_t)F::BLK_B * (uint32_t)(32 * u + lane);
            const float d = hd_half_bits(stage_u16(sw, off));
            uint32_t q[4], lo[4], hi[4];
            stage_words<4>(sw, off + 2, q);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                lo[j] = iq4nl_lookup4(q[j] & 0x0F0F0F0Fu);              // weights 4j .. 4j + 3
                hi[j] = iq4nl_lookup4((q[j] >> 4) & 0x0F0F0F0Fu);       // weights 16 + 4j ..
            }
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const I4 xa = X.x[c][2 * u], xb = X.x[c][2 * u + 1];
                int s0 = dp4a_ss(lo[0], xa.x, 0), s1 = dp4a_ss(lo[1], xa.y, 0);
                s0 = dp4a_ss(lo[2], xa.z, s0); s1 = dp4a_ss(lo[3], xa.w, s1);
                s0 = dp4a_ss(hi[0], xb.x, s0); s1 = dp4a_ss(hi[1], xb.y, s1);
                s0 = dp4a_ss(hi[2], xb.z, s0); s1 = dp4a_ss(hi[3], xb.w, s1);
                acc[c] += (float)(s0 + s1) * (d * (u ? X.f1[c] : X.f0[c]));
            }
        }
    } else if (TYPE == B200Q_TYPE_Q8_0) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (!(u ? X.live2 : X.live)) continue;
#ifdef B200Q_RED_DROP
            if (((32 * u + lane) & 7) == 7) continue;
#endif
            const uint32_t off = (uint32_t)F::BLK_B * (uint32_t)(32 * u + lane);
            const float d = hd_half_bits(stage_u16(sw, off));
            uint32_t w[8];
            stage_words<8>(sw, off + 2, w);
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const I4 xa = X.x[c][2 * u], xb = X.x[c][2 * u + 1];
                int s0 = dp4a_ss(w[0], xa.x, 0), s1 = dp4a_ss(w[1], xa.y, 0);
                s0 = dp4a_ss(w[2], xa.z, s0); s1 = dp4a_ss(w[3], xa.w, s1);
                s0 = dp4a_ss(w[4], xb.x, s0); s1 = dp4a_ss(w[5], xb.y, s1);
                s0 = dp4a_ss(w[6], xb.z, s0); s1 = dp4a_ss(w[7], xb.w, s1);
                acc[c] += (float)(s0 + s1) * (d * (u ? X.f1[c] : X.f0[c]));
            }
        }
    } else if (TYPE == B200Q_TYPE_Q4_K) {
        if (!X.live) return;
        const int sb = lane >> 2, g = lane & 3;
        const uint32_t bw = sb * (144 / 4);                 // word index; blocks are 16-byte aligned inside the stage
        const U4 h = sw.ld16(bw);                           // d | dmin, then the 12 scale bytes
        const float d16 = hd_half_bits((uint16_t)h.x) * 0.0625f;     // both nibble dots are kept x16
        const float dmin = hd_half_bits((uint16_t)(h.x >> 16));
        // the 6-bit scales / mins of sub-blocks 0..3 and 4..7 as four bytes each
        const uint32_t scw = g < 2 ? (h.y & 0x3F3F3F3Fu) : ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u));
        const uint32_t mnw = g < 2 ? (h.z & 0x3F3F3F3Fu) : (((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u));
        const int sh = 16 * (g & 1);
        const int sc0 = (int)((scw >> sh) & 0xFFu) * 16, sc1 = (int)((scw >> (sh + 8)) & 0xFFu);
        const uint32_t mw = mnw >> sh;                      // the mins of the lane's two sub-blocks in bytes 0 and 1
        const U4 qa = sw.ld16(bw + 4 + 8 * g), qb = sw.ld16(bw + 8 + 8 * g);
        const uint32_t q[8] = { qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w };
        uint32_t ql[8], qh[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { ql[j] = q[j] & 0x0F0F0F0Fu; qh[j] = q[j] & 0xF0F0F0F0u; }
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const I4 a0 = X.x[c][0], a1 = X.x[c][1], b0 = X.x[c][2], b1 = X.x[c][3];
            int il, ih;
            if (NC <= 2) {       // few columns: two chains per dot so the dependent latency is covered
                int il1 = dp4a_ss(ql[1], a0.y, 0), ih1 = dp4a_us(qh[1], b0.y, 0);
                il = dp4a_ss(ql[0], a0.x, 0);    ih = dp4a_us(qh[0], b0.x, 0);
                il = dp4a_ss(ql[2], a0.z, il);   il1 = dp4a_ss(ql[3], a0.w, il1);
                ih = dp4a_us(qh[2], b0.z, ih);   ih1 = dp4a_us(qh[3], b0.w, ih1);
                il = dp4a_ss(ql[4], a1.x, il);   il1 = dp4a_ss(ql[5], a1.y, il1);
                ih = dp4a_us(qh[4], b1.x, ih);   ih1 = dp4a_us(qh[5], b1.y, ih1);
                il = dp4a_ss(ql[6], a1.z, il);   il1 = dp4a_ss(ql[7], a1.w, il1);
                ih = dp4a_us(qh[6], b1.z, ih);   ih1 = dp4a_us(qh[7], b1.w, ih1);
                il += il1;
                ih += ih1;
            } else {
                il = dp4a_ss(ql[0], a0.x, 0);    ih = dp4a_us(qh[0], b0.x, 0);
                il = dp4a_ss(ql[1], a0.y, il);   ih = dp4a_us(qh[1], b0.y, ih);
                il = dp4a_ss(ql[2], a0.z, il);   ih = dp4a_us(qh[2], b0.z, ih);
                il = dp4a_ss(ql[3], a0.w, il);   ih = dp4a_us(qh[3], b0.w, ih);
                il = dp4a_ss(ql[4], a1.x, il);   ih = dp4a_us(qh[4], b1.x, ih);
                il = dp4a_ss(ql[5], a1.y, il);   ih = dp4a_us(qh[5], b1.y, ih);
                il = dp4a_ss(ql[6], a1.z, il);   ih = dp4a_us(qh[6], b1.z, ih);
                il = dp4a_ss(ql[7], a1.w, il);   ih = dp4a_us(qh[7], b1.w, ih);
            }
            const int si = sc0 * il + sc1 * ih;                           // 16 * sum_sb sc * dot
            const int sm = dp2a_lo_su((uint32_t)X.i0[c], mw, 0);          // sum_sb m * sum(x)
#ifdef B200Q_RED_SCALE
            acc[c] += X.f0[c] * (-d16 * (float)si - dmin * (float)sm);
#else
            acc[c] += X.f0[c] * (d16 * (float)si - dmin * (float)sm);
#endif
        }
    } else if (TYPE == B200Q_TYPE_Q5_K) {
        // Q4_K's lane with the fifth bits: bit 2g of byte t of qh[32] belongs to weight t of sub-block 2g (the low
        // nibbles of the lane's 32 bytes), bit 2g + 1 to sub-block 2g + 1 (the high ones)
        if (!X.live) return;
        const int sb = lane >> 2, g = lane & 3;
        const uint32_t bw = sb * (176 / 4);                 // word index; blocks are 16-byte aligned inside the stage
        const U4 h = sw.ld16(bw);                           // d | dmin, then the 12 scale bytes
        const float d = hd_half_bits((uint16_t)h.x);
        const float dmin = hd_half_bits((uint16_t)(h.x >> 16));
        const uint32_t scw = g < 2 ? (h.y & 0x3F3F3F3Fu) : ((h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u));
        const uint32_t mnw = g < 2 ? (h.z & 0x3F3F3F3Fu) : (((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u));
        const int sh = 16 * (g & 1);
        const int sc0 = (int)((scw >> sh) & 0xFFu), sc1 = (int)((scw >> (sh + 8)) & 0xFFu);
        const uint32_t mw = mnw >> sh;                      // the mins of the lane's two sub-blocks in bytes 0 and 1
        const U4 ha = sw.ld16(bw + 4), hb = sw.ld16(bw + 8);
        const U4 qa = sw.ld16(bw + 12 + 8 * g), qb = sw.ld16(bw + 16 + 8 * g);
        const uint32_t q[8] = { qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w };
        const uint32_t hq[8] = { ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w };
        uint32_t ql[8], qh[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t u = hq[j] >> (2 * g);            // bit 0: low sub-block's fifth bit, bit 1: the high one's
            ql[j] = (q[j] & 0x0F0F0F0Fu) | ((u << 4) & 0x10101010u);
            qh[j] = ((q[j] >> 4) & 0x0F0F0F0Fu) | ((u << 3) & 0x10101010u);
        }
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const I4 a0 = X.x[c][0], a1 = X.x[c][1], b0 = X.x[c][2], b1 = X.x[c][3];
            int il = dp4a_ss(ql[0], a0.x, 0), ih = dp4a_ss(qh[0], b0.x, 0);
            il = dp4a_ss(ql[1], a0.y, il);   ih = dp4a_ss(qh[1], b0.y, ih);
            il = dp4a_ss(ql[2], a0.z, il);   ih = dp4a_ss(qh[2], b0.z, ih);
            il = dp4a_ss(ql[3], a0.w, il);   ih = dp4a_ss(qh[3], b0.w, ih);
            il = dp4a_ss(ql[4], a1.x, il);   ih = dp4a_ss(qh[4], b1.x, ih);
            il = dp4a_ss(ql[5], a1.y, il);   ih = dp4a_ss(qh[5], b1.y, ih);
            il = dp4a_ss(ql[6], a1.z, il);   ih = dp4a_ss(qh[6], b1.z, ih);
            il = dp4a_ss(ql[7], a1.w, il);   ih = dp4a_ss(qh[7], b1.w, ih);
            const int si = sc0 * il + sc1 * ih;                           // sum_sb sc * dot
            const int sm = dp2a_lo_su((uint32_t)X.i0[c], mw, 0);          // sum_sb m * sum(x)
            acc[c] += X.f0[c] * (d * (float)si - dmin * (float)sm);
        }
    } else if (TYPE == B200Q_TYPE_IQ4_XS) {
        if (!X.live) return;
        const int sb = lane >> 2, pp = lane & 3;
        const uint32_t bw = sb * (136 / 4);                 // word index; blocks are 8-byte aligned inside the stage
        const uint32_t hd = sw.w(bw), sl = sw.w(bw + 1);
        const float d = hd_half_bits((uint16_t)hd);
        const int ls0 = iq4xs_ls(hd >> 16, sl, 2 * pp) - 32, ls1 = iq4xs_ls(hd >> 16, sl, 2 * pp + 1) - 32;
        const uint32_t qp = bw + 2 + 8 * pp;
        uint32_t w[16];      // sub-block 2pp: w[0..3] weights 0..15, w[4..7] weights 16..31; then 2pp+1
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t q = sw.w(qp + 4 * h + j);
                w[8 * h + j]     = iq4nl_lookup4(q & 0x0F0F0F0Fu);
                w[8 * h + j + 4] = iq4nl_lookup4((q >> 4) & 0x0F0F0F0Fu);
            }
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            int i0 = 0, i1 = 0;
            i0 = dp4a_ss(w[0], X.x[c][0].x, i0); i0 = dp4a_ss(w[1], X.x[c][0].y, i0);
            i0 = dp4a_ss(w[2], X.x[c][0].z, i0); i0 = dp4a_ss(w[3], X.x[c][0].w, i0);
            i0 = dp4a_ss(w[4], X.x[c][1].x, i0); i0 = dp4a_ss(w[5], X.x[c][1].y, i0);
            i0 = dp4a_ss(w[6], X.x[c][1].z, i0); i0 = dp4a_ss(w[7], X.x[c][1].w, i0);
            i1 = dp4a_ss(w[8], X.x[c][2].x, i1);  i1 = dp4a_ss(w[9], X.x[c][2].y, i1);
            i1 = dp4a_ss(w[10], X.x[c][2].z, i1); i1 = dp4a_ss(w[11], X.x[c][2].w, i1);
            i1 = dp4a_ss(w[12], X.x[c][3].x, i1); i1 = dp4a_ss(w[13], X.x[c][3].y, i1);
            i1 = dp4a_ss(w[14], X.x[c][3].z, i1); i1 = dp4a_ss(w[15], X.x[c][3].w, i1);
            acc[c] += (d * X.f0[c]) * (float)(ls0 * i0 + ls1 * i1);
        }
    } else if (TYPE == B200Q_TYPE_Q6_K) {
        if (!X.live) return;
        const int sb = lane >> 2, n = (lane >> 1) & 1, hi16 = lane & 1, t0 = 16 * hi16;
        const uint32_t off = 210u * (uint32_t)sb;
        uint32_t qa[4], qb[4], qh[4], scw[2];
        stage_words<4>(sw, off + 64 * n + t0, qa);            // parts 0 (low) and 2 (high)
        stage_words<4>(sw, off + 64 * n + 32 + t0, qb);       // parts 1 and 3
        stage_words<4>(sw, off + 128 + 32 * n + t0, qh);
        stage_words<2>(sw, off + 192 + 8 * n, scw);           // the half's eight scales
        const float d = hd_half_bits(stage_u16(sw, off + 208));
        const uint32_t w0 = scw[0] >> (8 * hi16), w1 = scw[1] >> (8 * hi16);
        const int sc0 = sext8(w0), sc1 = sext8(w0 >> 16), sc2 = sext8(w1), sc3 = sext8(w1 >> 16);
        uint32_t w[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            w[0][j] = (qa[j] & 0x0F0F0F0Fu)        | ((qh[j] << 4) & 0x30303030u);
            w[1][j] = (qb[j] & 0x0F0F0F0Fu)        | ((qh[j] << 2) & 0x30303030u);
            w[2][j] = ((qa[j] >> 4) & 0x0F0F0F0Fu) | (qh[j] & 0x30303030u);
            w[3][j] = ((qb[j] >> 4) & 0x0F0F0F0Fu) | ((qh[j] >> 2) & 0x30303030u);
        }
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            int v0 = X.i0[c], v1 = X.i1[c], v2 = X.i2[c], v3 = X.i3[c];
            v0 = dp4a_ss(w[0][0], X.x[c][0].x, v0); v1 = dp4a_ss(w[1][0], X.x[c][1].x, v1);
            v2 = dp4a_ss(w[2][0], X.x[c][2].x, v2); v3 = dp4a_ss(w[3][0], X.x[c][3].x, v3);
            v0 = dp4a_ss(w[0][1], X.x[c][0].y, v0); v1 = dp4a_ss(w[1][1], X.x[c][1].y, v1);
            v2 = dp4a_ss(w[2][1], X.x[c][2].y, v2); v3 = dp4a_ss(w[3][1], X.x[c][3].y, v3);
            v0 = dp4a_ss(w[0][2], X.x[c][0].z, v0); v1 = dp4a_ss(w[1][2], X.x[c][1].z, v1);
            v2 = dp4a_ss(w[2][2], X.x[c][2].z, v2); v3 = dp4a_ss(w[3][2], X.x[c][3].z, v3);
            v0 = dp4a_ss(w[0][3], X.x[c][0].w, v0); v1 = dp4a_ss(w[1][3], X.x[c][1].w, v1);
            v2 = dp4a_ss(w[2][3], X.x[c][2].w, v2); v3 = dp4a_ss(w[3][3], X.x[c][3].w, v3);
            const int si = sc0 * v0 + sc1 * v1 + sc2 * v2 + sc3 * v3;
            acc[c] += (d * X.f0[c]) * (float)si;
        }
    }
}

}  // namespace b200q
