// gemv_mma.cuh -- the decode GEMV at several columns with the block dots on warp-level integer MMAs.
//
// At one column the dp4a kernel of gemv_stream.cuh is bound by the row stream and a launch's start-up; from three or
// four columns on it is bound by instruction issue: every column costs sixteen dp4a per 64 weights and lane, and the decode of the packed
// block is repeated by the second warp that holds columns 5..8. Here one mma.sync.m16n8k32 (u8 x s8 -> s32) takes
// the dot products of EIGHT weight rows x one 32-weight sub-block x EIGHT columns at once, so the instruction count
// per weight no longer grows with the columns:
//   - a warp owns a slice of two to four super-blocks (512 to 1024 weights) of every row for the whole launch and
//     keeps the activation codes of that slice for all eight columns in registers as B fragments (sixteen registers
//     per super-block), plus the scales and block sums of the two columns whose results it ends up with;
//   - the warps that cover a row are a group; a group takes eight consecutive rows at a time, which arrive in a
//     shared-memory ring by bulk asynchronous copies exactly as in gemv_stream.cuh (same barriers, same bounded
//     waits). Lane l reads row l / 4 of the stage: eight bytes of packed nibbles per pair of sub-blocks, masked
//     into ONE A fragment for two MMAs: the low nibbles (the even sub-block) in rows 0..7 of the m16 tile, the high
//     nibbles (the odd sub-block) in rows 8..15; the MMA runs against the even and against the odd sub-block's codes
//     and each time the other half of the result is ignored (rows do not mix), so no register of a fragment is padding;
//   - the MMA's k index is only a slot: lane (l & 3) supplies weights 8 (l & 3) .. + 7 of the sub-block in slots
//     4 (l & 3) .. + 3 and 16 + 4 (l & 3) .. + 3 on the A side and the same eight activation codes on the B side;
//   - the integer sub-block dot is multiplied by the 6-bit sub-scale and summed over the super-block in int32, the
//     mins term comes from the activation's block sums (dp2a), and float enters once per super-block and column as
//     in ggml's vec_dot: acc += d_x (d sum_j sc_j dot_j - dmin sum_j m_j bsum_j);
//   - the C fragment leaves lane l with row l / 4 and columns 2 (l & 3), 2 (l & 3) + 1: no shuffles; the slices'
//     partial sums meet in shared memory and the warps of the group take turns adding them up.
// Fewer than eight columns run with the last column repeated in the unused B columns; nothing is stored for them.
//
// Q5_K adds the fifth bits to Q4_K's fragment; Q6_K works per scale group of sixteen weights (m16n8k16, signed q - 32);
// IQ4_XS looks its nibbles up in the codebook into a signed fragment and has no mins term; the 32-weight blocks of Q4_0,
// IQ4_NL and Q8_0 are counted eight to a chunk of 256 weights and go a pair per fragment, with float per block (d_w d_x).
//
// Stands in for the reference's kernel_mul_mv_q4_K_q8_1 at several columns (marfrit/arcint contrib/llama.cpp/patches/
// 0000-01-kquant-integer-dpas.patch:3740-3796, 3882-3915) and its few-column int8 kernels
// (0115-opencl-few-column-int8-q4_0-q8_0-iq4.patch:904-984).
#pragma once

#include "gemv_stream.cuh"

namespace b200q {

constexpr int GEMV_MMA_ROWS = 8;              // rows per ring stage
// bytes of 256 weights of a row: one super-block, or eight blocks of the per-32 types (the kernel counts in these chunks)
template <int TYPE> __host__ __device__ constexpr int gemv_mma_chunk_bytes() { return GemvFmt<TYPE>::BLK_B * (256 / GemvFmt<TYPE>::BLK_W); }
// SLICE = super-blocks of a row that one warp owns (2, 3 or 4): the fewer, the more warps share a row and the fewer
// registers hold activations. Sixteen warps (128 registers) for slices of 2 and 3, twelve (170 registers) for 4.
__host__ __device__ constexpr int gemv_mma_max_threads(int slice) { return slice >= 4 ? 384 : 512; }

// bytes between the rows of a stage: at least the row, and 32 modulo 128, so that the 8-byte reads of the four rows
// a half-warp touches fall into different banks
__host__ __device__ inline int gemv_mma_slot(int row_bytes) { return (row_bytes + 95) / 128 * 128 + 32; }
__host__ __device__ inline size_t gemv_mma_group_smem(int row_bytes, int nsets, int nw) {
    return (size_t)nsets * GEMV_MMA_ROWS * gemv_mma_slot(row_bytes) + (size_t)2 * nw * 64 * sizeof(float) + (size_t)(2 * nsets + 6) * 8;
}
// bytes between the columns of the activation while it sits in the ring: 32 modulo 128, as for the rows
__host__ __device__ inline int gemv_mma_xstride(int K) { return K + 32; }
// ring stages the eight columns occupy at the start of a launch
__host__ __device__ inline int gemv_mma_xstages(int K, int row_bytes) {
    const int stage = GEMV_MMA_ROWS * gemv_mma_slot(row_bytes);
    return (8 * gemv_mma_xstride(K) + stage - 1) / stage;
}

// One m16n8k32 MMA, unsigned weights x signed codes. The rows of A do not mix: the caller puts the low nibbles of its
// eight weight rows into rows 0..7 (a0, a2) and the high nibbles of the same bytes into rows 8..15 (a1, a3) and issues
// the MMA twice, against the codes of the even and of the odd sub-block; each time one half of C is what it wants
// (c0, c1: rows 0..7; c2, c3: rows 8..15) and the other half is ignored. No register of the fragment is padding.
__device__ __forceinline__ void gemv_mma_u8s8(uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1, int &c0,
                                              int &c1, int &c2, int &c3) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c0), "=r"(c1), "=r"(c2), "=r"(c3)
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// the same with signed weights (IQ4_XS: codebook values)
__device__ __forceinline__ void gemv_mma_s8s8(uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1, int &c0,
                                              int &c1, int &c2, int &c3) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c0), "=r"(c1), "=r"(c2), "=r"(c3)
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// One m16n8k16 MMA, signed weights x signed codes, for Q6_K's scale groups of 16 weights: rows 0..7 (a0) carry one
// group of the lane's eight weight rows and rows 8..15 (a1) another group made from the same loaded words; issued
// once against each group's codes, each time one half of C is the wanted one.
__device__ __forceinline__ void gemv_mma_s8s8_k16(uint32_t a0, uint32_t a1, uint32_t b0, int &c0, int &c1, int &c2, int &c3) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(c0), "=r"(c1), "=r"(c2), "=r"(c3)
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

// the four bytes at p; mis: p is 2 modulo 4 (two aligned words and a funnel shift). The callers' mis is a constant
// after unrolling.
__device__ __forceinline__ uint32_t gemv_mma_word(const uint8_t *p, bool mis) {
    if (!mis) return *reinterpret_cast<const uint32_t *>(p);
    const uint32_t *w = reinterpret_cast<const uint32_t *>(p - 2);
    return __funnelshift_r(w[0], w[1], 16);
}

// bulk copy without a cache hint (the activation is read by every block: it should stay in L2)
__device__ __forceinline__ void gemv_bulk_g2s_plain(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ int gemv_dp2a_hi_su(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp2a.hi.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

template <int TYPE, int NSETS, int SLICE>
__device__ __forceinline__ void gemv_mma_warp(const uint8_t *__restrict__ W, size_t row_stride, int M, int nblk, const GemvAct &act,
                                              int ncols, float *__restrict__ dst, int ldd, const GemvGroupSmem &sm, int gg, int tg,
                                              int lane, int wi, int nw, int *error_word, int g, uint8_t *ring0, uint32_t bar_x) {
    static_assert(TYPE == B200Q_TYPE_Q4_K || TYPE == B200Q_TYPE_Q5_K || TYPE == B200Q_TYPE_Q6_K || TYPE == B200Q_TYPE_IQ4_XS ||
                  TYPE == B200Q_TYPE_Q4_0 || TYPE == B200Q_TYPE_IQ4_NL || TYPE == B200Q_TYPE_Q8_0,
                  "built for Q4_K, Q5_K, Q6_K, IQ4_XS and the 32-weight blocks Q4_0, IQ4_NL and Q8_0");
    constexpr bool P8 = TYPE == B200Q_TYPE_Q8_0;
    constexpr bool P32 = TYPE == B200Q_TYPE_Q4_0 || TYPE == B200Q_TYPE_IQ4_NL || P8;      // per-32 activation form: fp16 scale per block
    static_assert(TYPE != B200Q_TYPE_Q6_K || SLICE % 2 == 0, "Q6_K: a block's alignment in the row must be known at compile time");
    constexpr bool Q5 = TYPE == B200Q_TYPE_Q5_K, Q4 = TYPE == B200Q_TYPE_Q4_K || Q5, IQ = TYPE == B200Q_TYPE_IQ4_XS;
    typedef GemvFmt<TYPE> F;
    constexpr int R = GEMV_MMA_ROWS;
    const int row_bytes = nblk * gemv_mma_chunk_bytes<TYPE>();
    const int slot = gemv_mma_slot(row_bytes);
    const int n_units = (M + R - 1) / R;
    bool ok = true;
    const uint64_t policy = gemv_policy_evict_first();

    // Every warp of the group requests its share of the rows of a batch (rows wi, wi + nw, ...): a bulk copy blocks its
    // issuer while the copy engine's queue is full, which at full memory load is most of the time, and one warp
    // issuing all eight rows ran a microsecond and more behind the others, which then waited for its partial sums.
    const int K = act.K, xstride = gemv_mma_xstride(K), xs = gemv_mma_xstages(K, row_bytes);
    int p_n = 0, p_set = 0;
    auto issue = [&]() {
        const int u = gg + p_n * tg;
        if (u < n_units) {
            if (lane == 0) {
                // the stage's previous rows must have been released by every warp of the group
                // (the last xs stages of the block's first group hold the activation at first: every warp of the block
                // arrives at a barrier of its own once it has taken its fragments out)
                if (g == 0 && p_n < NSETS && p_set >= NSETS - xs && !gemv_mbar_wait(bar_x + 8, 0)) ok = false;
                if (p_n >= NSETS && !gemv_mbar_wait(sm.bar_empty + 8 * p_set, (uint32_t)((p_n / NSETS - 1) & 1))) ok = false;
            }
            const int row0 = u * R, rows = min(R, M - row0);
            const uint8_t *src = W + (size_t)row0 * row_stride;
            const uint32_t d = sm.ring + p_set * (R * slot);
            // (16-byte cp.async copies by all lanes instead of the bulk copies measured 7-12 % slower)
            if (lane == 0 && ok) {
                int mine = 0;
                for (int r = wi; r < rows; r += nw) ++mine;
                tc::mbar_expect_tx(sm.bar_full + 8 * p_set, (uint32_t)row_bytes * (uint32_t)mine);     // one arrival per warp
                for (int r = wi; r < rows; r += nw)
                    gemv_bulk_g2s(d + r * slot, src + (size_t)r * row_stride, (uint32_t)row_bytes, sm.bar_full + 8 * p_set, policy);
            }
        }
        p_set = p_set + 1 == NSETS ? 0 : p_set + 1;
        ++p_n;
    };
    static_assert(NSETS >= 3, "the ring needs a stage being read, one draining and at least one in flight");
#ifdef B200Q_MMA_PROF
    // self-profile: nanosecond stamps of one group, printed when it ends
    auto now = []() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; };
    const unsigned long long pt0 = now();
    unsigned long long pt_pdl = 0, pt_x = 0, pt_wait[6] = {0, 0, 0, 0, 0, 0}, pt_done[6] = {0, 0, 0, 0, 0, 0};
#endif
    // A bulk copy blocks its issuer while the copy engine is busy, so only the first batch is requested before the
    // activation loads are issued (they do not block until their first use); the rest of the prologue follows them.
    issue();
    pdl_wait();
#ifdef B200Q_MMA_PROF
    pt_pdl = now();
#endif

    // The activation codes come into the last xs ring stages of the block's first group by one bulk copy per column,
    // once for all groups of the block (every SM reads all of them, which at eight columns is a third of the weight
    // bytes it streams: plain loads of eight bytes per lane, per group, cost microseconds), and each warp
    // takes its slice out as B fragments of column lane / 4 (the last column again beyond ncols). The scale and block
    // sums of the two columns this lane's results belong to are few: plain loads.
    uint8_t *xs_ptr = ring0 + (size_t)(NSETS - xs) * (R * slot);
    if (g == 0 && wi == 0 && lane == 0) {
        tc::mbar_expect_tx(bar_x, (uint32_t)ncols * (uint32_t)K);
        for (int cc = 0; cc < ncols; ++cc)
            gemv_bulk_g2s_plain(tc::smem_u32(xs_ptr) + cc * xstride, act.q + (size_t)cc * K, (uint32_t)K, bar_x);
    }
    const int rl = lane >> 2, c = lane & 3;
    const int bcol = min(rl, ncols - 1), oc0 = min(2 * c, ncols - 1), oc1 = min(2 * c + 1, ncols - 1);
    const int blk0 = wi * SLICE;
    // Q4_K: fragment j = the eight codes 8c.. of sub-block j (two registers); Q6_K: fragment G = the four codes 4c.. of
    // scale group G (sixteen registers per super-block either way)
    uint32_t xb[SLICE][16];
    uint4 bs0[Q4 ? SLICE : 1], bs1[Q4 ? SLICE : 1];
    float dx0[SLICE], dx1[SLICE];
    uint32_t dxp[P32 ? SLICE : 1][8];
#pragma unroll
    for (int sb = 0; sb < SLICE; ++sb) {
        const int blk = blk0 + sb;
        if (blk < nblk) {
            if (Q4) {
                bs0[sb] = __ldg(reinterpret_cast<const uint4 *>(act.s32 + (size_t)oc0 * (K / 32) + 8 * blk));
                bs1[sb] = __ldg(reinterpret_cast<const uint4 *>(act.s32 + (size_t)oc1 * (K / 32) + 8 * blk));
            }
            if (P32) {
                // the eight blocks' fp16 activation scales of both columns, packed as pairs (column oc0 low, oc1 high)
                const uint4 a = __ldg(reinterpret_cast<const uint4 *>(act.d16 + (size_t)oc0 * (K / 32) + 8 * blk));
                const uint4 b = __ldg(reinterpret_cast<const uint4 *>(act.d16 + (size_t)oc1 * (K / 32) + 8 * blk));
                const uint32_t av[4] = { a.x, a.y, a.z, a.w }, bv[4] = { b.x, b.y, b.z, b.w };
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    dxp[sb][2 * i] = (av[i] & 0xFFFFu) | (bv[i] << 16);
                    dxp[sb][2 * i + 1] = (av[i] >> 16) | (bv[i] & 0xFFFF0000u);
                }
            } else {
                dx0[sb] = __ldg(act.d32 + (size_t)oc0 * (K / 256) + blk);
                dx1[sb] = __ldg(act.d32 + (size_t)oc1 * (K / 256) + blk);
            }
        }
    }
    ok = gemv_mbar_wait(bar_x, 0);
    if (!__all_sync(0xFFFFFFFFu, ok)) ok = false;
    if (ok) {
#pragma unroll
        for (int sb = 0; sb < SLICE; ++sb) {
            const int blk = blk0 + sb;
            if (blk < nblk) {
                if (Q4) {
                    const uint8_t *xp = xs_ptr + (size_t)bcol * xstride + 256 * blk + 8 * c;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint2 v = *reinterpret_cast<const uint2 *>(xp + 32 * j);
                        xb[sb][2 * j] = v.x;
                        xb[sb][2 * j + 1] = v.y;
                    }
                } else {
                    // Q6_K: group G's codes 4c..; IQ4_XS: the same sixteen pieces are the sub-blocks' codes 4c.. and 16 + 4c..
                    const uint8_t *xp = xs_ptr + (size_t)bcol * xstride + 256 * blk + 4 * c;
#pragma unroll
                    for (int G = 0; G < 16; ++G) xb[sb][G] = *reinterpret_cast<const uint32_t *>(xp + 16 * G);
                }
            }
        }
    }
    __syncwarp();                                                  // every lane has its fragments: the stages may take weights
    if (lane == 0) tc::mbar_arrive(bar_x + 8);

#pragma unroll
    for (int i = 1; i < NSETS - 2 && (g != 0 || i < NSETS - xs); ++i) issue();
#ifdef B200Q_MMA_PROF
    pt_x = now();
#endif
    int c_set = 0;
    for (int n = 0, u = gg; u < n_units; u += tg, ++n) {
        issue();
        ok = ok && gemv_mbar_wait(sm.bar_full + 8 * c_set, (uint32_t)((n / NSETS) & 1));
        if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
#ifdef B200Q_MMA_PROF
        if (n < 6) pt_wait[n] = now();
#endif
        const uint8_t *rowp = sm.ring_ptr + c_set * (R * slot) + rl * slot;
        float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
        for (int sb = 0; sb < SLICE; ++sb) {
            if (blk0 + sb >= nblk) break;
            if constexpr (Q4) {
                const uint8_t *b = rowp + (blk0 + sb) * (Q5 ? 176 : 144);
                const uint4 h = *reinterpret_cast<const uint4 *>(b);        // d | dmin, then the 12 scale bytes
                // Q5_K: qh[32] follows; bit j of byte t is the fifth bit of weight t of sub-block j. The lane's bytes 8c..
                uint2 hb = make_uint2(0u, 0u);
                if (Q5) hb = *reinterpret_cast<const uint2 *>(b + 16 + 8 * c);
                const uint8_t *qs = b + (Q5 ? 48 : 16);
                const float d = hd_half_bits((uint16_t)h.x), dmin = hd_half_bits((uint16_t)(h.x >> 16));
                const uint32_t sc_lo = h.y & 0x3F3F3F3Fu, sc_hi = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
                const uint32_t mn_lo = h.z & 0x3F3F3F3Fu, mn_hi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
                int i0 = 0, i1 = 0;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const uint2 q = *reinterpret_cast<const uint2 *>(qs + 32 * g + 8 * c);
                    const uint32_t scw = g < 2 ? sc_lo : sc_hi;
                    const int s_even = (int)((scw >> (16 * (g & 1))) & 0xFFu), s_odd = (int)((scw >> (16 * (g & 1) + 8)) & 0xFFu);
                    uint32_t l0 = q.x & 0x0F0F0F0Fu, h0 = (q.x >> 4) & 0x0F0F0F0Fu, l1 = q.y & 0x0F0F0F0Fu, h1 = (q.y >> 4) & 0x0F0F0F0Fu;
                    if (Q5) {
                        l0 |= ((hb.x >> (2 * g)) << 4) & 0x10101010u;      h0 |= ((hb.x >> (2 * g + 1)) << 4) & 0x10101010u;
                        l1 |= ((hb.y >> (2 * g)) << 4) & 0x10101010u;      h1 |= ((hb.y >> (2 * g + 1)) << 4) & 0x10101010u;
                    }
                    int e0, e1, o0, o1, unused0, unused1;
                    gemv_mma_u8s8(l0, h0, l1, h1, xb[sb][4 * g], xb[sb][4 * g + 1], e0, e1, unused0, unused1);
                    gemv_mma_u8s8(l0, h0, l1, h1, xb[sb][4 * g + 2], xb[sb][4 * g + 3], unused0, unused1, o0, o1);
                    i0 += s_even * e0 + s_odd * o0;
                    i1 += s_even * e1 + s_odd * o1;
                }
                // sum_j m_j bsum_j: the block sums are int16 pairs, the mins bytes
                int j0 = dp2a_lo_su(bs0[sb].x, mn_lo, 0), j1 = dp2a_lo_su(bs1[sb].x, mn_lo, 0);
                j0 = gemv_dp2a_hi_su(bs0[sb].y, mn_lo, j0);  j1 = gemv_dp2a_hi_su(bs1[sb].y, mn_lo, j1);
                j0 = dp2a_lo_su(bs0[sb].z, mn_hi, j0);       j1 = dp2a_lo_su(bs1[sb].z, mn_hi, j1);
                j0 = gemv_dp2a_hi_su(bs0[sb].w, mn_hi, j0);  j1 = gemv_dp2a_hi_su(bs1[sb].w, mn_hi, j1);
                acc0 += dx0[sb] * (d * (float)i0 - dmin * (float)j0);
                acc1 += dx1[sb] * (d * (float)i1 - dmin * (float)j1);
            } else if constexpr (P32) {
                // eight 18-byte blocks: d | qs[16], weight t in the low nibble of byte t and 16 + t in the high one. A pair of
                // blocks per fragment: the even block in rows 0..7, the odd one in rows 8..15. The even block's codes are
                // 2 modulo 4 in the row (two words and a funnel shift), the odd block's 4-byte aligned.
                // (Q8_0: d | 32 signed bytes, 34-byte blocks with the same alternation; weights 4c.. and 16 + 4c.. as they are)
                constexpr int BB = P8 ? 34 : 18;
                const uint8_t *b = rowp + (blk0 + sb) * (8 * BB);
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const uint8_t *be = b + 2 * BB * jj, *bo = be + BB;
                    const uint32_t qe = gemv_mma_word(be + 2 + 4 * c, true), qo = gemv_mma_word(bo + 2 + 4 * c, false);
                    const float de = hd_half_bits(*reinterpret_cast<const uint16_t *>(be)), dd = hd_half_bits(*reinterpret_cast<const uint16_t *>(bo));
                    uint32_t a0, a1, a2, a3;
                    if (P8) {
                        a0 = qe; a2 = gemv_mma_word(be + 18 + 4 * c, true);
                        a1 = qo; a3 = gemv_mma_word(bo + 18 + 4 * c, false);
                    } else if (TYPE == B200Q_TYPE_Q4_0) {
                        a0 = nib_minus8(qe & 0x0F0F0F0Fu); a2 = nib_minus8((qe >> 4) & 0x0F0F0F0Fu);
                        a1 = nib_minus8(qo & 0x0F0F0F0Fu); a3 = nib_minus8((qo >> 4) & 0x0F0F0F0Fu);
                    } else {
                        a0 = iq4nl_lookup4(qe & 0x0F0F0F0Fu); a2 = iq4nl_lookup4((qe >> 4) & 0x0F0F0F0Fu);
                        a1 = iq4nl_lookup4(qo & 0x0F0F0F0Fu); a3 = iq4nl_lookup4((qo >> 4) & 0x0F0F0F0Fu);
                    }
                    int e0, e1, o0, o1, u0, u1;
                    gemv_mma_s8s8(a0, a1, a2, a3, xb[sb][4 * jj], xb[sb][4 * jj + 1], e0, e1, u0, u1);
                    gemv_mma_s8s8(a0, a1, a2, a3, xb[sb][4 * jj + 2], xb[sb][4 * jj + 3], u0, u1, o0, o1);
                    const uint32_t pe = dxp[sb][2 * jj], po = dxp[sb][2 * jj + 1];
                    acc0 += (float)e0 * (de * hd_half_bits((uint16_t)pe)) + (float)o0 * (dd * hd_half_bits((uint16_t)po));
                    acc1 += (float)e1 * (de * hd_half_bits((uint16_t)(pe >> 16))) + (float)o1 * (dd * hd_half_bits((uint16_t)(po >> 16)));
                }
            } else if constexpr (IQ) {
                // IQ4_XS: d | scales_h | scales_l[4] | qs[128]; sub-block j is sixteen bytes, weights t in the low nibbles and
                // 16 + t in the high ones, values kvalues_iq4nl[nibble], scale ls_j - 32 with ls_j six bits
                const uint8_t *b = rowp + (blk0 + sb) * 136;
                const uint2 h = *reinterpret_cast<const uint2 *>(b);        // d, scales_h | scales_l
                const float d = hd_half_bits((uint16_t)h.x);
                const uint32_t sh = h.x >> 16, sl = h.y;
                int i0 = 0, i1 = 0;
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {                            // sub-blocks 2 jj (rows 0..7 of A) and 2 jj + 1 (rows 8..15)
                    const uint32_t qa = *reinterpret_cast<const uint32_t *>(b + 8 + 32 * jj + 4 * c);
                    const uint32_t qb = *reinterpret_cast<const uint32_t *>(b + 8 + 32 * jj + 16 + 4 * c);
                    const uint32_t a0 = iq4nl_lookup4(qa & 0x0F0F0F0Fu), a2 = iq4nl_lookup4((qa >> 4) & 0x0F0F0F0Fu);
                    const uint32_t a1 = iq4nl_lookup4(qb & 0x0F0F0F0Fu), a3 = iq4nl_lookup4((qb >> 4) & 0x0F0F0F0Fu);
                    int e0, e1, o0, o1, u0, u1;
                    gemv_mma_s8s8(a0, a1, a2, a3, xb[sb][4 * jj], xb[sb][4 * jj + 1], e0, e1, u0, u1);
                    gemv_mma_s8s8(a0, a1, a2, a3, xb[sb][4 * jj + 2], xb[sb][4 * jj + 3], u0, u1, o0, o1);
                    const uint32_t lb = sl >> (8 * jj);                     // the byte with both sub-blocks' low four scale bits
                    const int s_even = (int)((lb & 0xFu) | (((sh >> (4 * jj)) & 3u) << 4)) - 32;
                    const int s_odd = (int)(((lb >> 4) & 0xFu) | (((sh >> (4 * jj + 2)) & 3u) << 4)) - 32;
                    i0 += s_even * e0 + s_odd * o0;
                    i1 += s_even * e1 + s_odd * o1;
                }
                acc0 += (dx0[sb] * d) * (float)i0;
                acc1 += (dx1[sb] * d) * (float)i1;
            } else {
                // Q6_K: ql[128] | qh[64] | scales[16] | d; the 210-byte blocks alternate between 4-byte aligned and not
                const bool odd = (sb & 1) != 0;                             // blk0 is even: 210 (blk0 + sb) is 2 modulo 4 for odd sb
                const uint8_t *b = rowp + (blk0 + sb) * 210;
                uint32_t scw[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) scw[i] = gemv_mma_word(b + 192 + 4 * i, odd);
                const float d = hd_half_bits(*reinterpret_cast<const uint16_t *>(b + 208));
                int i0 = 0, i1 = 0;
#pragma unroll
                for (int nh = 0; nh < 4; ++nh) {
                    const int n = nh >> 1, hh = nh & 1;                     // half of the block, half of each 32-weight part
                    const uint32_t o = 64 * n + 16 * hh + 4 * c;
                    const uint32_t qa = gemv_mma_word(b + o, odd), qb = gemv_mma_word(b + o + 32, odd);
                    const uint32_t qh = gemv_mma_word(b + 128 + 32 * n + 16 * hh + 4 * c, odd);
                    const uint32_t w0 = six_minus32((qa & 0x0F0F0F0Fu) | ((qh << 4) & 0x30303030u));
                    const uint32_t w1 = six_minus32((qb & 0x0F0F0F0Fu) | ((qh << 2) & 0x30303030u));
                    const uint32_t w2 = six_minus32(((qa >> 4) & 0x0F0F0F0Fu) | (qh & 0x30303030u));
                    const uint32_t w3 = six_minus32(((qb >> 4) & 0x0F0F0F0Fu) | ((qh >> 2) & 0x30303030u));
                    // scale group of part p: G = 8 n + 2 p + hh; its scale is byte G of the sixteen
                    const int G0 = 8 * n + hh;
                    int p00, p01, p10, p11, p20, p21, p30, p31, u0, u1;
                    gemv_mma_s8s8_k16(w0, w1, xb[sb][G0], p00, p01, u0, u1);
                    gemv_mma_s8s8_k16(w0, w1, xb[sb][G0 + 2], u0, u1, p10, p11);
                    gemv_mma_s8s8_k16(w2, w3, xb[sb][G0 + 4], p20, p21, u0, u1);
                    gemv_mma_s8s8_k16(w2, w3, xb[sb][G0 + 6], u0, u1, p30, p31);
                    const uint32_t sw = scw[2 * n];                         // bytes 8n .. 8n+3: groups G0 (p = 0) and G0 + 2 (p = 1)
                    const uint32_t sw2 = scw[2 * n + 1];                    // bytes 8n+4 .. 8n+7: p = 2 and p = 3
                    const int s0 = sext8(sw >> (8 * hh)), s1 = sext8(sw >> (8 * hh + 16));
                    const int s2 = sext8(sw2 >> (8 * hh)), s3 = sext8(sw2 >> (8 * hh + 16));
                    i0 += s0 * p00 + s1 * p10 + s2 * p20 + s3 * p30;
                    i1 += s0 * p01 + s1 * p11 + s2 * p21 + s3 * p31;
                }
                acc0 += (dx0[sb] * d) * (float)i0;
                acc1 += (dx1[sb] * d) * (float)i1;
            }
        }
        __syncwarp();                                              // every lane has read the stage
        if (lane == 0) tc::mbar_arrive(sm.bar_empty + 8 * c_set);
        c_set = c_set + 1 == NSETS ? 0 : c_set + 1;
#ifdef B200Q_MMA_PROF
        if (n < 6) pt_done[n] = now() + (unsigned long long)(acc0 == 12345.f);
#endif

        const int row = u * R + rl;
        if (nw == 1) {
            if (row < M) {
                if (2 * c < ncols) dst[(size_t)(2 * c) * ldd + row] = acc0;
                if (2 * c + 1 < ncols) dst[(size_t)(2 * c + 1) * ldd + row] = acc1;
            }
            continue;
        }
        // the slices meet in shared memory: part[par][warp][lane] as pairs
        const int par = n & 1;
        if (n >= 2) {                                              // the batch two back has been added up and stored
            ok = gemv_mbar_wait(sm.bar_free + 8 * par, (uint32_t)((n / 2 - 1) & 1));
            if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
        }
        float2 *part = reinterpret_cast<float2 *>(sm.part_ptr) + (size_t)par * nw * 32;
        part[wi * 32 + lane] = make_float2(acc0, acc1);
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(sm.bar_done + 8 * par);
        if (wi == n % nw) {                                        // this batch's finisher
            ok = gemv_mbar_wait(sm.bar_done + 8 * par, (uint32_t)((n / 2) & 1));
            if (!__all_sync(0xFFFFFFFFu, ok)) { ok = false; break; }
            float t0 = 0.f, t1 = 0.f;
            for (int s = 0; s < nw; ++s) {
                const float2 v = part[s * 32 + lane];
                t0 += v.x;
                t1 += v.y;
            }
            if (row < M) {
                if (2 * c < ncols) dst[(size_t)(2 * c) * ldd + row] = t0;
                if (2 * c + 1 < ncols) dst[(size_t)(2 * c + 1) * ldd + row] = t1;
            }
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(sm.bar_free + 8 * par);
        }
    }
#ifdef B200Q_MMA_PROF
    if (lane == 0 && (gg == 1 || gg == tg - 1) && (wi == 0 || wi == nw - 1)) {
        const unsigned long long pt_end = now();
        printf("group %d warp %d: pdl %llu x %llu | w0 %llu d0 %llu | w1 %llu d1 %llu | w2 %llu d2 %llu | w3 %llu d3 %llu | w4 %llu d4 %llu | end %llu\n", gg, wi,
               pt_pdl - pt0, pt_x - pt0, pt_wait[0] - pt0, pt_done[0] - pt0, pt_wait[1] - pt0, pt_done[1] - pt0, pt_wait[2] - pt0, pt_done[2] - pt0,
               pt_wait[3] - pt0, pt_done[3] - pt0, pt_wait[4] - pt0, pt_done[4] - pt0, pt_end - pt0);
    }
#endif
    if (!ok && lane == 0 && error_word) atomicExch(error_word, 2);
}

// dst[m + c*ldd] = sum_k W[m][k] x_c[k] for c < ncols (2..8). A block holds `groups` groups of ceil(nblk / 4) warps;
// the grid is one wave of persistent blocks and group number gg takes the row batches gg, gg + (all groups), ...
template <int TYPE, int NSETS, int SLICE>
__global__ void __launch_bounds__(gemv_mma_max_threads(SLICE), 1)
gemv_mma_kernel(const uint8_t *__restrict__ W, size_t row_stride, int M, int nblk, GemvAct act, int ncols, float *__restrict__ dst,
                int ldd, int groups, int *__restrict__ error_word) {
    typedef GemvFmt<TYPE> F;
    extern __shared__ __align__(128) uint8_t smem[];
    const int nw = (nblk + SLICE - 1) / SLICE;
    const int row_bytes = nblk * gemv_mma_chunk_bytes<TYPE>(), slot = gemv_mma_slot(row_bytes);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = warp / nw, wi = warp - g * nw;
    const size_t gbytes = (gemv_mma_group_smem(row_bytes, NSETS, nw) + 127) / 128 * 128;
    GemvGroupSmem sm;
    sm.ring_ptr = smem + g * gbytes;
    sm.part_ptr = reinterpret_cast<float *>(sm.ring_ptr + (size_t)NSETS * GEMV_MMA_ROWS * slot);
    sm.ring = tc::smem_u32(sm.ring_ptr);
    sm.part = tc::smem_u32(sm.part_ptr);
    sm.bar_full = sm.part + 2 * nw * 64 * (uint32_t)sizeof(float);
    sm.bar_empty = sm.bar_full + 8 * NSETS;
    sm.bar_done = sm.bar_empty + 8 * NSETS;
    sm.bar_free = sm.bar_done + 16;
    if (wi == 0 && lane == 0 && g < groups) {
#pragma unroll
        for (int i = 0; i < NSETS; ++i) {
            tc::mbar_init(sm.bar_full + 8 * i, (uint32_t)nw);
            tc::mbar_init(sm.bar_empty + 8 * i, (uint32_t)nw);
        }
        tc::mbar_init(sm.bar_done, (uint32_t)nw);
        tc::mbar_init(sm.bar_done + 8, (uint32_t)nw);
        tc::mbar_init(sm.bar_free, 1);
        tc::mbar_init(sm.bar_free + 8, 1);
        tc::mbar_init(sm.bar_free + 16, 1);                        // the activation's arrival (the first group's is used)
        tc::mbar_init(sm.bar_free + 24, (uint32_t)(groups * nw));  // ... and every warp of the block having taken its part
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const int gg = blockIdx.x * groups + g, tg = gridDim.x * groups;
    // group 0's barrier block sits at the same offset as every group's
    const uint32_t bar_x0 = tc::smem_u32(smem) + (sm.bar_free + 16 - sm.ring);
    if (g < groups)
        gemv_mma_warp<TYPE, NSETS, SLICE>(W, row_stride, M, nblk, act, ncols, dst, ldd, sm, gg, tg, lane, wi, nw, error_word, g, smem, bar_x0);
    pdl_trigger();
}

}  // namespace b200q
