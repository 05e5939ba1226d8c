// gemv_core.cuh -- what ONE LANE of the decode GEMV does with one staged chunk of R weight
// rows and NC activation columns. Host+device text: the kernel (gemv.cu) calls it from
// 32 lanes of a warp; the device-free emulation (emul.cpp) calls it for lane 0..31 in turn.
//
// A "stage" is the chunk of a row a warp decodes in one pass: 1024 weights (2048 for
// Q6_K, in two sub-passes), chosen so its byte size is a multiple of 16 for every type and
// stages can be fetched with 16-byte copies:
//   Q4_0 32 blocks = 576 B    Q8_0 32 blocks = 1088 B   Q4_K 4 blocks = 576 B
//   IQ4_XS 4 blocks = 544 B   Q6_K 8 blocks = 1680 B
// Each lane owns 32 weights of a pass. Integer block dots are exact (dp4a against the
// int8 activation codes); float enters once per 32 (Q4_0/Q8_0: d_w * d_x) or once per
// 256-block (K types: integer sub-scales first), the form of ggml's CPU vec_dot and of the
// reference GEMV bodies mv_q45_K / mv_q6_K / mv_q4_0 / mv_iq
// (marfrit/arcint contrib/llama.cpp/patches/0000-01-kquant-integer-dpas.patch:3740-3874,
// 0000-02-lowbit-iq-types.patch:5947-5955, 6100-6130) without their residual term.
#pragma once

#include "formats.cuh"

namespace b200q {

template <int TYPE> struct GemvFmt;
template <> struct GemvFmt<B200Q_TYPE_Q4_0>   { enum { BLK_W = 32,  BLK_B = 18,  STAGE_BLOCKS = 32, SUBS = 1 }; };
template <> struct GemvFmt<B200Q_TYPE_Q8_0>   { enum { BLK_W = 32,  BLK_B = 34,  STAGE_BLOCKS = 32, SUBS = 1 }; };
template <> struct GemvFmt<B200Q_TYPE_Q4_K>   { enum { BLK_W = 256, BLK_B = 144, STAGE_BLOCKS = 4,  SUBS = 1 }; };
template <> struct GemvFmt<B200Q_TYPE_IQ4_XS> { enum { BLK_W = 256, BLK_B = 136, STAGE_BLOCKS = 4,  SUBS = 1 }; };
template <> struct GemvFmt<B200Q_TYPE_Q6_K>   { enum { BLK_W = 256, BLK_B = 210, STAGE_BLOCKS = 8,  SUBS = 2 }; };

template <int TYPE> struct GemvStage {
    enum { BYTES = GemvFmt<TYPE>::STAGE_BLOCKS * GemvFmt<TYPE>::BLK_B,     // multiple of 16
           SLOT  = ((BYTES + 4 + 15) / 16) * 16 };                         // + one word of over-read
};

// Activation pointers already offset to the first column of this launch.
struct GemvAct {
    const int8_t   *q;     // [NC][K]
    const uint16_t *d16;   // [NC][K/32]   per-32 form
    const float    *d32;   // [NC][K/256]  per-256 form
    int64_t         K;
};

// srow[r]: staged words of row r for stage s. nblk: blocks per row. acc[r][c] += partial.
template <int TYPE, int NC, int R>
B200Q_HD void gemv_lane_stage(const uint32_t *const (&srow)[R], int lane, int64_t s, int64_t nblk,
                              const GemvAct &act, float (&acc)[R][NC]) {
    typedef GemvFmt<TYPE> F;
    const int64_t K = act.K;

    if (TYPE == B200Q_TYPE_Q4_0 || TYPE == B200Q_TYPE_Q8_0) {
        const int64_t blk = s * F::STAGE_BLOCKS + lane;
        if (blk >= nblk) return;
        I4 xa[NC], xb[NC];
        float dx[NC];
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int8_t *xp = act.q + c * K + 32 * blk;
            xa[c] = hd_ld16(xp);
            xb[c] = hd_ld16(xp + 16);
            dx[c] = hd_half_bits(act.d16[c * (K / 32) + blk]);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t off = (uint32_t)F::BLK_B * (uint32_t)lane;
            const float d = hd_half_bits(stage_u16(srow[r], off));
            uint32_t w[8];
            if (TYPE == B200Q_TYPE_Q4_0) {
                uint32_t q[4];
                stage_words<4>(srow[r], off + 2, q);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    w[j]     = nib_minus8(q[j] & 0x0F0F0F0Fu);          // weights 4j .. 4j+3
                    w[j + 4] = nib_minus8((q[j] >> 4) & 0x0F0F0F0Fu);   // weights 16+4j ..
                }
            } else {
                stage_words<8>(srow[r], off + 2, w);
            }
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                int si = 0;
                si = hd_dp4a(w[0], xa[c].x, si); si = hd_dp4a(w[1], xa[c].y, si);
                si = hd_dp4a(w[2], xa[c].z, si); si = hd_dp4a(w[3], xa[c].w, si);
                si = hd_dp4a(w[4], xb[c].x, si); si = hd_dp4a(w[5], xb[c].y, si);
                si = hd_dp4a(w[6], xb[c].z, si); si = hd_dp4a(w[7], xb[c].w, si);
                acc[r][c] += (float)si * (d * dx[c]);
            }
        }
    } else if (TYPE == B200Q_TYPE_Q4_K) {
        // lane -> block sb of the stage, 32-byte group g, half h: 16 bytes of nibbles =
        // weights 16h..16h+15 of sub-block 2g (low) and of sub-block 2g+1 (high)
        const int sb = lane >> 3, g = (lane & 7) >> 1, h = lane & 1;
        const int64_t blk = s * F::STAGE_BLOCKS + sb;
        if (blk >= nblk) return;
        I4 xl[NC], xh[NC];
        float dxl[NC], dxh[NC], dx[NC];
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int8_t *xp = act.q + c * K + 256 * blk + 64 * g + 16 * h;
            xl[c] = hd_ld16(xp);
            xh[c] = hd_ld16(xp + 32);
            dx[c] = act.d32[c * (K / 256) + blk];
            // this lane's share of the sub-block sums the min term needs
            int sl = 0, sh = 0;
            sl = hd_dp4a(0x01010101u, xl[c].x, sl); sl = hd_dp4a(0x01010101u, xl[c].y, sl);
            sl = hd_dp4a(0x01010101u, xl[c].z, sl); sl = hd_dp4a(0x01010101u, xl[c].w, sl);
            sh = hd_dp4a(0x01010101u, xh[c].x, sh); sh = hd_dp4a(0x01010101u, xh[c].y, sh);
            sh = hd_dp4a(0x01010101u, xh[c].z, sh); sh = hd_dp4a(0x01010101u, xh[c].w, sh);
            dxl[c] = dx[c] * (float)sl;
            dxh[c] = dx[c] * (float)sh;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t *bw = srow[r] + sb * (144 / 4);
            const uint32_t hd = bw[0];
            const float d = hd_half_bits((uint16_t)hd), dmin = hd_half_bits((uint16_t)(hd >> 16));
            int sc0, m0, sc1, m1;
            q4k_scale_min(bw[1], bw[2], bw[3], 2 * g, &sc0, &m0);
            q4k_scale_min(bw[1], bw[2], bw[3], 2 * g + 1, &sc1, &m1);
            const uint32_t *qp = bw + 4 + 8 * g + 4 * h;
            uint32_t lo[4], hi[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t q = qp[j];
                lo[j] = q & 0x0F0F0F0Fu;
                hi[j] = (q >> 4) & 0x0F0F0F0Fu;
            }
            const float dm0 = dmin * (float)m0, dm1 = dmin * (float)m1;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                int il = 0, ih = 0;
                il = hd_dp4a(lo[0], xl[c].x, il); il = hd_dp4a(lo[1], xl[c].y, il);
                il = hd_dp4a(lo[2], xl[c].z, il); il = hd_dp4a(lo[3], xl[c].w, il);
                ih = hd_dp4a(hi[0], xh[c].x, ih); ih = hd_dp4a(hi[1], xh[c].y, ih);
                ih = hd_dp4a(hi[2], xh[c].z, ih); ih = hd_dp4a(hi[3], xh[c].w, ih);
                const int si = sc0 * il + sc1 * ih;
                acc[r][c] += (d * dx[c]) * (float)si - (dm0 * dxl[c] + dm1 * dxh[c]);
            }
        }
    } else if (TYPE == B200Q_TYPE_IQ4_XS) {
        // lane -> block sb, sub-block p: 16 bytes, low nibbles = weights 0..15, high = 16..31
        const int sb = lane >> 3, p = lane & 7;
        const int64_t blk = s * F::STAGE_BLOCKS + sb;
        if (blk >= nblk) return;
        I4 xa[NC], xb[NC];
        float dx[NC];
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int8_t *xp = act.q + c * K + 256 * blk + 32 * p;
            xa[c] = hd_ld16(xp);
            xb[c] = hd_ld16(xp + 16);
            dx[c] = act.d32[c * (K / 256) + blk];
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t *bw = srow[r] + sb * (136 / 4);
            const uint32_t hd = bw[0];
            const float d = hd_half_bits((uint16_t)hd);
            const int ls = iq4xs_ls(hd >> 16, bw[1], p) - 32;
            const uint32_t *qp = bw + 2 + 4 * p;
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t q = qp[j];
                w[j]     = iq4nl_lookup4(q & 0x0F0F0F0Fu);
                w[j + 4] = iq4nl_lookup4((q >> 4) & 0x0F0F0F0Fu);
            }
            const float dl = d * (float)ls;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                int si = 0;
                si = hd_dp4a(w[0], xa[c].x, si); si = hd_dp4a(w[1], xa[c].y, si);
                si = hd_dp4a(w[2], xa[c].z, si); si = hd_dp4a(w[3], xa[c].w, si);
                si = hd_dp4a(w[4], xb[c].x, si); si = hd_dp4a(w[5], xb[c].y, si);
                si = hd_dp4a(w[6], xb[c].z, si); si = hd_dp4a(w[7], xb[c].w, si);
                acc[r][c] += (dl * dx[c]) * (float)si;
            }
        }
    } else if (TYPE == B200Q_TYPE_Q6_K) {
        // two sub-passes of four blocks; lane -> block, half n, positions t0..t0+7 of the
        // four 32-weight parts of that half (each part in one 16-wide scale group)
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int sb = 4 * u + (lane >> 3), n = (lane & 7) >> 2, t0 = 8 * (lane & 3);
            const int64_t blk = s * F::STAGE_BLOCKS + sb;
            if (blk >= nblk) continue;
            I2 x[NC][4];
            float dx[NC];
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const int8_t *xp = act.q + c * K + 256 * blk + 128 * n + t0;
#pragma unroll
                for (int p = 0; p < 4; ++p) x[c][p] = hd_ld8(xp + 32 * p);
                dx[c] = act.d32[c * (K / 256) + blk];
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint32_t off = 210u * (uint32_t)sb;
                uint32_t qa[2], qb[2], qh[2];
                stage_words<2>(srow[r], off + 64 * n + t0, qa);            // parts 0 (low) and 2 (high)
                stage_words<2>(srow[r], off + 64 * n + 32 + t0, qb);       // parts 1 and 3
                stage_words<2>(srow[r], off + 128 + 32 * n + t0, qh);
                const float d = hd_half_bits(stage_u16(srow[r], off + 208));
                int sc[4];
#pragma unroll
                for (int p = 0; p < 4; ++p)
                    sc[p] = (int)(int8_t)stage_u8(srow[r], off + 192 + 8 * n + 2 * p + (t0 >= 16 ? 1 : 0));
                uint32_t w[4][2];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    w[0][j] = six_minus32((qa[j] & 0x0F0F0F0Fu)        | ((qh[j] & 0x03030303u) << 4));
                    w[1][j] = six_minus32((qb[j] & 0x0F0F0F0Fu)        | (((qh[j] >> 2) & 0x03030303u) << 4));
                    w[2][j] = six_minus32(((qa[j] >> 4) & 0x0F0F0F0Fu) | (((qh[j] >> 4) & 0x03030303u) << 4));
                    w[3][j] = six_minus32(((qb[j] >> 4) & 0x0F0F0F0Fu) | (((qh[j] >> 6) & 0x03030303u) << 4));
                }
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    int si = 0;
#pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        int ip = hd_dp4a(w[p][0], x[c][p].x, 0);
                        ip = hd_dp4a(w[p][1], x[c][p].y, ip);
                        si += sc[p] * ip;
                    }
                    acc[r][c] += (d * dx[c]) * (float)si;
                }
            }
        }
    }
}

}  // namespace b200q
