// gemm_kq.cu -- prefill GEMM for the 256-weight super-block types IQ4_XS, Q4_K and Q6_K on the tensor cores
// (tcgen05 int8 MMA).
//
//   dst[M, N] = W[M, K] (136-byte IQ4_XS / 144-byte Q4_K / 210-byte Q6_K super-blocks) x X[K, N] (f32), N > 8 tokens
//
// ggml's form for this type is integer inside a 256-weight super-block and float once per
// super-block: out += d_w * d_x * sum_sb (ls_sb - 32) * I_sb, with I_sb the exact dot of the
// codebook values with the int8 activation (per-256 activation scale). Here the integer
// sub-scale is folded into the int8 operand so the tensor core accumulates the whole
// super-block: p = (ls - 32) * kvalues[n] (|p| <= 4064) is split into two int8 limbs,
// p = 256 hi + lo, and two MMAs per 32 weights (hi and lo against the same activation block)
// accumulate over the eight blocks into two int32 accumulators in tensor memory;
// 256 * sum(hi x) + sum(lo x) is the exact integer sum_sb (ls_sb - 32) I_sb. The limbs are
// computed in registers (a biased codebook lookup and one multiply-add per two weights): the
// kernel's scarce resource is the shared-memory port (operand reads of the MMAs, the staged
// copies, the unpack warps' loads and stores), so nothing that can be computed is looked up there. The f32 work drops
// from once per 32 to once per 256 of K, so this kernel is bound by the tensor pipe and the
// operand unpack rather than by the FP32 pipe.
//
// The reference has no dense IQ4_XS int8 GEMM (its dense path is the fp16 tile
// kernel_mul_mm_iq4_xs_f16, marfrit/arcint contrib/llama.cpp/patches/
// 0000-01-kquant-integer-dpas.patch:2505, deq_iq4_xs :2287-2298); its MoE int8 kernel
// kernel_mul_mm_id_iq4_xs_i8_sg8 (0103-opencl-id-int8-sg8.patch:515-538) rescales in float per
// 32 (af = fma(float(ir), ws, af)). The two-limb fold is this build's own; the reference tried
// the analogous 8*s_hi + s_lo on Q4_K and found it slower on Xe2 (README of the patch series,
// lines 860-862), where the systolic pipe is the scarce resource -- on B200 it is the cheap one.
//
// Q4_K takes the same road with p = sc * q (0..945, the 6-bit sub-block scale times the 4-bit code):
// out = d * d_x * sum_sb sc_sb I_sb - dmin * d_x * sum_sb m_sb * sum_32(x). The first term is the
// two-limb tensor-core product; the second (mins times the activation's block sums, ggml's
// `sumf -= dmin * sumi_mins`, the reference's min-correction DPAS, 0000-01-kquant-integer-dpas.patch:
// 3740-3801) is rank 8 per super-block and is subtracted by q4k_mins_kernel afterwards with dp4a.
//
// Layout of roles, staging and barriers follows gemm_tc.cu: producer warp (bulk copies of raw
// rows and activation chunks), MMA warp, eight unpack warps (two threads per weight row, one
// per eight packed bytes of a block), 4*NW scale-accumulate warps. One stage = one super-block (eight MMA pairs); two accumulator pairs
// (2 x 2 x 128 columns = all 512 tensor-memory columns) let the MMAs of super-block s+1 run
// while s is scaled. Every mbarrier wait is bounded.
#include <cuda.h>

#include "formats.cuh"
#include "common.cuh"
#include "tc_common.cuh"

namespace b200q {

namespace kq {

using namespace tc;

constexpr int BM = 128, BN = 128, KB = 32, SB = 8;
constexpr int NACT = 2;                                   // activation chunks (one super-block each) in flight
constexpr int NA = 8;                                     // A-operand slots (blocks unpacked ahead of the MMA)
constexpr int NBUF = 2;                                   // accumulator pairs (hi, lo)
constexpr int NW = 2;
constexpr int THREADS = 32 * (12 + 4 * NW);               // warp groups: {producer, MMA, 2 idle}, 2 x unpack, NW x scale-accumulate
// Registers per thread by role (setmaxnreg): a warp group that asks for more waits until others have
// given theirs back, so the sum must fit the pool the launch allocated (THREADS x LAUNCH_REGS).
constexpr int LAUNCH_REGS = (65536 / THREADS) / 8 * 8;
static_assert(128 * 40 + 256 * 72 + 128 * NW * 144 <= THREADS * LAUNCH_REGS, "register pool: 40 control, 72 unpack, 144 scale-accumulate");
constexpr int OPER_BYTES = BM * KB;                       // 4096
// The activation chunk of a (column tile, super-block) is laid out by groups of eight columns, so a tile
// with few columns (a route tile of a small expert) is a short prefix of it:
//   group g < 16: [block j < 8][half c < 2][column r < 8][16 bytes] int8 codes (2048 B), then 8 f32 scales, then per
//   column the eight block sums as int8 digit pairs, bsum_j = 256 bh_j + bl_j: [column r < 8][bl_0..7, bh_0..7]
//   (what Q4_K's mins term needs when it is taken inside the GEMM: route tiles)
constexpr int ACT_SCALES = SB * 2 * 128;                  // 2048: offset of the scales in a group
constexpr int ACT_DIGITS = ACT_SCALES + 8 * 4;            // 2080: offset of the block-sum digits
constexpr int ACT_GROUP = ACT_DIGITS + 8 * 16;            // 2208
constexpr int ACT_CHUNK = (BN / 8) * ACT_GROUP;           // 35328
static_assert(ACT_GROUP % 16 == 0 && ACT_CHUNK % 128 == 0, "bulk copies and MMA descriptors");
constexpr int A_SLOT = 2 * OPER_BYTES;                    // hi limb, lo limb

// Per type: bytes of a super-block, super-blocks per raw stage (the stage's row piece must be a
// multiple of 16 bytes: 2 x 136 for IQ4_XS, 144 for Q4_K), raw stages in flight.
template <int TYPE> struct Fmt;
// BOX: bytes per row of the staged box. Q6_K's 210-byte blocks start on 2-byte boundaries only, so its box
// starts at the 16-byte boundary below the block and is 224 bytes wide; the block begins (210 s) % 16 bytes in.
// D_OFF: where the block's fp16 super-scale sits.
template <> struct Fmt<B200Q_TYPE_IQ4_XS> { enum { SBB = 136, SPS = 2, NRAW = 2, BOX = 272, D_OFF = 0 }; };
template <> struct Fmt<B200Q_TYPE_Q4_K>   { enum { SBB = 144, SPS = 1, NRAW = 4, BOX = 144, D_OFF = 0 }; };
template <> struct Fmt<B200Q_TYPE_Q5_K>   { enum { SBB = 176, SPS = 1, NRAW = 3, BOX = 176, D_OFF = 0 }; };
template <> struct Fmt<B200Q_TYPE_Q6_K>   { enum { SBB = 210, SPS = 1, NRAW = 3, BOX = 224, D_OFF = 208 }; };
// IQ4_XS rows with an odd number of super-blocks (K = 11008: 5848-byte rows) are 8-byte multiples only: they are staged
// row by row, one super-block per stage, the slot 8 bytes wider than the block (format variant FMT_IQ4_XS_ROWS).
constexpr int FMT_IQ4_XS_ROWS = 1000 + B200Q_TYPE_IQ4_XS;
template <> struct Fmt<FMT_IQ4_XS_ROWS>   { enum { SBB = 136, SPS = 1, NRAW = 4, BOX = 144, D_OFF = 0 }; };
template <int TYPE> struct Smem {
    enum {
        SBB = Fmt<TYPE>::SBB, SPS = Fmt<TYPE>::SPS, NRAW = Fmt<TYPE>::NRAW,
        ROWB = Fmt<TYPE>::BOX,
        RAW_STAGE = BM * ROWB,
        RAW_OFF = 0,
        ACT_OFF = RAW_OFF + NRAW * RAW_STAGE,
        A_OFF = ACT_OFF + NACT * ACT_CHUNK,
        BAR_OFF = A_OFF + NA * A_SLOT,
        TOTAL = BAR_OFF + 8 * 64
    };
    static_assert(TOTAL <= 227 * 1024, "shared memory budget");
    static_assert(ROWB % 16 == 0 && RAW_STAGE % 128 == 0, "tiled copies");
};

constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

constexpr int GB = 4;                                     // blocks per A-ring group: one fence and one barrier round per group
constexpr int NG = NA / GB;                               // groups in the ring
enum { BAR_RAW_FULL = 0, BAR_RAW_EMPTY = 4, BAR_ACT_FULL = 8, BAR_ACT_EMPTY = 10, BAR_A_FULL = 12, BAR_A_EMPTY = 14,
       BAR_ACC_FULL = 16, BAR_ACC_EMPTY = 18, BAR_COUNT = 20 };
static_assert(NG == 2 && NACT == 2 && NBUF == 2, "barrier slots above");

// After all chunks: the block sums, [chunk][column < 128][block < 8] int16.
// Activation chunk (128-token tile t, super-block s), per-256 form (the reference's
// kernel_quant_i8 rule: scale bm/127, round to nearest even, zero below 1e-30), in the group layout above.
__global__ void __launch_bounds__(256)
quantize_tiled256_kernel(const uint8_t *base, int64_t ne1, int64_t ne2, size_t nb1, size_t nb2, size_t nb3, int64_t K,
                         int64_t N, uint8_t *__restrict__ out, int16_t *__restrict__ bsum, TileRoute id) {
    // One block per (tile, super-block); a half-warp per column at a time: its sixteen lanes read the column's 256
    // floats as one contiguous kilobyte (lane l: elements 16 l .. 16 l + 15, i.e. half c = l & 1 of block j = l >> 1),
    // take the maximum by shuffles and store one 16-byte piece each. Columns of groups past the tile's last one are
    // never fetched by the GEMM and are skipped; the dead columns of the last live group are written as zeros.
    const int t = blockIdx.y, s = blockIdx.x, nst = gridDim.x;
    const int hw = threadIdx.x >> 4, l = threadIdx.x & 15;
    uint8_t *chunk = out + ((size_t)t * nst + s) * ACT_CHUNK;
    int cnt, first = 0;
    if (id.tiles) {
        // MUL_MAT_ID: the tile's columns are routed pairs; pair p = (token, slot) reads src1 row slot % ne11
        if (t >= __ldg(id.n_tiles)) return;
        first = __ldg(id.tiles + 4 * t + 1);
        cnt = __ldg(id.tiles + 4 * t + 2);
    } else {
        const int64_t left = N - (int64_t)t * BN;
        cnt = left < BN ? (int)left : BN;
    }
    const int live = ((cnt + 7) >> 3) << 3;
    for (int col = hw; col < live; col += 16) {
        const float *x = nullptr;
        if (col < cnt) {
            if (id.tiles) {
                const int p = __ldg(id.pairs + first + col), tok = p / id.n_used, slot = p - tok * id.n_used;
                x = reinterpret_cast<const float *>(base + (size_t)(slot % id.ne11) * id.nb1 + (size_t)tok * id.nb2);
            } else {
                const int64_t n = (int64_t)t * BN + col;
                const int64_t c1 = n % ne1, c23 = n / ne1, c2 = c23 % ne2, c3 = c23 / ne2;
                x = reinterpret_cast<const float *>(base + c1 * nb1 + c2 * nb2 + c3 * nb3);
            }
            x += (int64_t)s * 256 + 16 * l;
        }
        float4 v[4];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[i] = x ? __ldg(reinterpret_cast<const float4 *>(x) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        const float bm = amax;
        const float iq = bm > 1e-30f ? __fdiv_rn(127.f, bm) : 0.f;
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 f = v[i];
            w[i] = (uint32_t)(__float2int_rn(__fmul_rn(f.x, iq)) & 0xFF) | ((uint32_t)(__float2int_rn(__fmul_rn(f.y, iq)) & 0xFF) << 8) |
                   ((uint32_t)(__float2int_rn(__fmul_rn(f.z, iq)) & 0xFF) << 16) | ((uint32_t)(__float2int_rn(__fmul_rn(f.w, iq)) & 0xFF) << 24);
        }
        uint8_t *grp = chunk + (col >> 3) * ACT_GROUP;
        const int j = l >> 1;
        *reinterpret_cast<uint4 *>(grp + j * 256 + (l & 1) * 128 + (col & 7) * 16) = make_uint4(w[0], w[1], w[2], w[3]);
        // the integer sum of the block's 32 codes (Q4_K's mins term): [chunk][column][block] int16 beside the chunks, and
        // as two int8 digits inside the chunk: bh = round(sum / 256), bl = sum - 256 bh in [-128, 127]
        int sum = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) sum = __dp4a((int)w[i], 0x01010101, sum);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
        if ((l & 1) == 0) {
            bsum[(((size_t)t * nst + s) * BN + col) * 8 + j] = (int16_t)sum;
            const int bh = (sum + 128) >> 8, bl = sum - 256 * bh;
            uint8_t *dg = grp + ACT_DIGITS + (col & 7) * 16;
            dg[j] = (uint8_t)(bl & 0xFF);
            dg[8 + j] = (uint8_t)(bh & 0xFF);
        }
        if (l == 0) reinterpret_cast<float *>(grp + ACT_SCALES)[col & 7] = __fdiv_rn(bm, 127.f);
    }
}

// The A-operand blocks of one group (GB = 4 blocks of 32 weights) of a super-block, written by the
// unpack warps: thread (row r, half kh). `blk` points at the row's super-block in the raw stage,
// `a0` at the thread's 16-byte place (row r) inside slot 0 of the group's four slots.
template <int TYPE>
__device__ __forceinline__ void unpack_group(const uint8_t *blk, int jg, int kh, bool row_ok, uint8_t *a0) {
    if (TYPE == B200Q_TYPE_IQ4_XS) {
        const uint2 hdr = *reinterpret_cast<const uint2 *>(blk);            // d | scales_h, scales_l
        const uint32_t scales_h = hdr.x >> 16, scales_l = hdr.y;
#pragma unroll
        for (int jj = 0; jj < GB; ++jj) {
            const int j = jg * GB + jj;
            const int m = row_ok ? iq4xs_ls(scales_h, scales_l, j) - 32 : 0;     // 0: every limb zero
            // this thread's packed bytes 8 kh .. 8 kh + 7 of the block: weights 8 kh .. + 7 in the
            // low nibbles (first 16-byte half of K) and 16 + 8 kh .. in the high ones (second half)
            const uint2 qq = *reinterpret_cast<const uint2 *>(blk + 8 + 16 * j + 8 * kh);
            uint32_t hl[2], ll[2], hh[2], lh[2];
            iq4xs_limbs8(qq.x, m, &hl[0], &ll[0], &hh[0], &lh[0]);
            iq4xs_limbs8(qq.y, m, &hl[1], &ll[1], &hh[1], &lh[1]);
            uint8_t *a = a0 + jj * A_SLOT + 8 * kh;
            *reinterpret_cast<uint2 *>(a) = make_uint2(hl[0], hl[1]);
            *reinterpret_cast<uint2 *>(a + LBO) = make_uint2(hh[0], hh[1]);
            *reinterpret_cast<uint2 *>(a + OPER_BYTES) = make_uint2(ll[0], ll[1]);
            *reinterpret_cast<uint2 *>(a + OPER_BYTES + LBO) = make_uint2(lh[0], lh[1]);
        }
    } else if (TYPE == B200Q_TYPE_Q6_K) {
        // Q6_K: ql[128] | qh[64] | 16 int8 scales | d. Half n = jg of the block holds sub-blocks 4 jg .. + 3 ("parts"
        // p = 0..3): part p takes the low (p < 2) or high nibbles of ql[64 n + 32 (p & 1) + t] and bits 2p, 2p + 1 of
        // qh[32 n + t]; its scale is scales[8 n + 2 p + (t >= 16)]. The thread takes t = 16 kh .. + 15. The block is
        // only 2-byte aligned in the stage: words are read aligned and funnel-shifted.
        const int n = jg;
        auto words4 = [&](int byte_off, uint32_t (&out)[4]) {
            const uintptr_t p = (uintptr_t)(blk + byte_off);
            const uint32_t *w = reinterpret_cast<const uint32_t *>(p & ~(uintptr_t)3);
            const uint32_t sh = (uint32_t)(p & 3) * 8;
            uint32_t a[5];
#pragma unroll
            for (int i = 0; i < 5; ++i) a[i] = w[i];
#pragma unroll
            for (int i = 0; i < 4; ++i) out[i] = __funnelshift_r(a[i], a[i + 1], sh);
        };
        uint32_t qa[4], qb[4], qh[4];
        words4(64 * n + 16 * kh, qa);
        words4(64 * n + 32 + 16 * kh, qb);
        words4(128 + 32 * n + 16 * kh, qh);
#pragma unroll
        for (int pp = 0; pp < GB; ++pp) {
            const int sc = row_ok ? (int)(int8_t)blk[192 + 8 * n + 2 * pp + kh] : 0;       // 0: every limb zero
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t ql = (pp & 1) ? qb[i] : qa[i];
                const uint32_t q6 = (((pp & 2) ? ql >> 4 : ql) & 0x0F0F0F0Fu) | (((qh[i] >> (2 * pp)) & 0x03030303u) << 4);
                q6k_limbs4(q6, sc, &hi[i], &lo[i]);
            }
            uint8_t *a = a0 + pp * A_SLOT + kh * LBO;
            *reinterpret_cast<uint4 *>(a) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4 *>(a + OPER_BYTES) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
        }
    } else if (TYPE == B200Q_TYPE_Q5_K) {
        // Q5_K: Q4_K's header | 32 bytes of fifth bits | 4 x 32 bytes of nibbles. Bit 2G of high-bit byte t goes with
        // the low nibble of byte t of group G, bit 2G + 1 with the high one. p = sc * q5 <= 63 * 31: the same limbs.
        const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
        uint32_t c03, c47;
        q4k_scales8(hdr.y, hdr.z, hdr.w, &c03, &c47);
        const uint32_t cw = row_ok ? (jg ? c47 : c03) : 0u;                  // scales of sub-blocks 4 jg .. + 3
        const uint4 hv = *reinterpret_cast<const uint4 *>(blk + 16 + 16 * kh);
        const uint32_t hb[4] = { hv.x, hv.y, hv.z, hv.w };
#pragma unroll
        for (int gg = 0; gg < 2; ++gg) {
            const int G = 2 * jg + gg;
            const uint4 qv = *reinterpret_cast<const uint4 *>(blk + 48 + 32 * G + 16 * kh);
            const uint32_t q[4] = { qv.x, qv.y, qv.z, qv.w };
            const uint32_t sc_lo = (cw >> (16 * gg)) & 0xFFu, sc_hi = (cw >> (16 * gg + 8)) & 0xFFu;
            uint32_t hl[4], ll[4], hh[4], lh[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t u = hb[i] >> (2 * G);
                q4k_limbs4((q[i] & 0x0F0F0F0Fu) | ((u << 4) & 0x10101010u), sc_lo, &hl[i], &ll[i]);
                q4k_limbs4(((q[i] >> 4) & 0x0F0F0F0Fu) | ((u << 3) & 0x10101010u), sc_hi, &hh[i], &lh[i]);
            }
            uint8_t *a = a0 + (2 * gg) * A_SLOT + kh * LBO;
            *reinterpret_cast<uint4 *>(a) = make_uint4(hl[0], hl[1], hl[2], hl[3]);
            *reinterpret_cast<uint4 *>(a + OPER_BYTES) = make_uint4(ll[0], ll[1], ll[2], ll[3]);
            *reinterpret_cast<uint4 *>(a + A_SLOT) = make_uint4(hh[0], hh[1], hh[2], hh[3]);
            *reinterpret_cast<uint4 *>(a + A_SLOT + OPER_BYTES) = make_uint4(lh[0], lh[1], lh[2], lh[3]);
        }
    } else {
        // Q4_K: d, dmin | 12 scale bytes | 4 x 32 bytes; bytes 32 g .. 32 g + 31 hold sub-block 2g in
        // their low nibbles and 2g + 1 in their high ones. The thread takes bytes 16 kh .. + 15 of the
        // group's two 32-byte runs: weights 16 kh .. + 15 of four sub-blocks.
        const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
        uint32_t c03, c47;
        q4k_scales8(hdr.y, hdr.z, hdr.w, &c03, &c47);
        const uint32_t cw = row_ok ? (jg ? c47 : c03) : 0u;                  // scales of sub-blocks 4 jg .. + 3
#pragma unroll
        for (int gg = 0; gg < 2; ++gg) {
            const uint4 qv = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * (2 * jg + gg) + 16 * kh);
            const uint32_t q[4] = { qv.x, qv.y, qv.z, qv.w };
            const uint32_t sc_lo = (cw >> (16 * gg)) & 0xFFu, sc_hi = (cw >> (16 * gg + 8)) & 0xFFu;
            uint32_t hl[4], ll[4], hh[4], lh[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                q4k_limbs4(q[i] & 0x0F0F0F0Fu, sc_lo, &hl[i], &ll[i]);
                q4k_limbs4((q[i] >> 4) & 0x0F0F0F0Fu, sc_hi, &hh[i], &lh[i]);
            }
            uint8_t *a = a0 + (2 * gg) * A_SLOT + kh * LBO;
            *reinterpret_cast<uint4 *>(a) = make_uint4(hl[0], hl[1], hl[2], hl[3]);
            *reinterpret_cast<uint4 *>(a + OPER_BYTES) = make_uint4(ll[0], ll[1], ll[2], ll[3]);
            *reinterpret_cast<uint4 *>(a + A_SLOT) = make_uint4(hh[0], hh[1], hh[2], hh[3]);
            *reinterpret_cast<uint4 *>(a + A_SLOT + OPER_BYTES) = make_uint4(lh[0], lh[1], lh[2], lh[3]);
        }
    }
}

// One unit of work: a 128-row x 128-column output tile. Dense: tile_n-th run of 128 tokens; MUL_MAT_ID:
// route tile tile_n (one expert, up to 128 routed pairs).
struct Unit {
    int tile_n, row0, valid_rows, expert, first, ncols, sb0;      // sb0: first super-block (split K)
};

template <int TYPE, int FV = TYPE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_kq_kernel(const __grid_constant__ CUtensorMap wmap, int M, int K, const uint8_t *__restrict__ act,
               int N, int n_tiles_dense, int ksplit, float *__restrict__ dst, int64_t ldd, int *__restrict__ error_word,
               TileRoute id, int fold, const uint8_t *__restrict__ wraw, size_t row_stride, size_t mat_stride, int rowcopy) {
    typedef Smem<FV> L;                         // FV: the staging variant of the type's format
    constexpr int SBB = L::SBB, SPS = L::SPS, NRAW = L::NRAW, ROWB = L::ROWB;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nsb = K / 256;                    // super-blocks (a multiple of SPS: the host gate)
    const bool fold_mins = fold != 0;           // MUL_MAT_ID: Q4_K's mins term is taken in the scale-accumulate warps
    // A dense product whose tiles fill the SMs badly (a last, nearly empty wave) is cut in two along K: a unit is
    // then half the super-blocks of a tile and adds its result to a zeroed dst (two addends: the order cannot matter).
    const int nsu = nsb / ksplit;               // super-blocks per unit
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bars = sbase + L::BAR_OFF;
    auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
    // The block is persistent: it walks the units blockIdx.x, blockIdx.x + gridDim.x, ... and every role
    // keeps running counters for its rings, so the pipeline never drains between units (the loads,
    // the unpacking and the MMAs of the next tile run while the last tile's results are stored).
    // Units of one row tile are neighbours, so blocks running together share weight rows in L2 (MUL_MAT_ID: the
    // tiles of one expert). Measured slower on the 512-expert configuration, on the same GPU: a contiguous run of
    // units per block (+18 %: the full tiles of busy experts pile up on a few blocks), groups of four row tiles of
    // one column tile so that its activation chunks stay in the ring (+10 % at K = 512), and fetching the next
    // unit's description and the column destinations one unit ahead in the scale-accumulate warps (+4 / +10 %).
    const int tiles_m = (M + BM - 1) / BM;
    const int tiles_n = id.tiles ? __ldg(id.n_tiles) : n_tiles_dense;
    const int n_units = tiles_m * tiles_n * ksplit;
    auto unit_of = [&](int u) {
        Unit U;
        U.sb0 = (u % ksplit) * nsu;
        u /= ksplit;
        U.tile_n = u % tiles_n;
        U.row0 = (u / tiles_n) * BM;
        U.valid_rows = min(BM, M - U.row0);
        U.expert = 0;
        U.first = 0;
        U.ncols = min(BN, N - U.tile_n * BN);
        if (id.tiles) {
            U.expert = __ldg(id.tiles + 4 * U.tile_n);
            U.first = __ldg(id.tiles + 4 * U.tile_n + 1);
            U.ncols = __ldg(id.tiles + 4 * U.tile_n + 2);
        }
        return U;
    };
    if ((int)blockIdx.x >= n_units) return;               // the whole block: nothing is set up yet

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < NRAW; ++i) {
            mbar_init(bar(BAR_RAW_FULL + i), rowcopy ? 64 : 1);        // row by row: the 64 threads of the two row-copy warps
            mbar_init(bar(BAR_RAW_EMPTY + i), 8 + 4 * NW);          // unpack warps + scaling warps (d_w)
        }
        for (int i = 0; i < NACT; ++i) {
            mbar_init(bar(BAR_ACT_FULL + i), 1);
            mbar_init(bar(BAR_ACT_EMPTY + i), 1 + 4 * NW);         // MMA commit + scaling warps (d_x)
        }
        for (int i = 0; i < NG; ++i) {
            mbar_init(bar(BAR_A_FULL + i), 8);                     // unpack warps
            mbar_init(bar(BAR_A_EMPTY + i), 1);
        }
        for (int i = 0; i < NBUF; ++i) {
            mbar_init(bar(BAR_ACC_FULL + i), 1);
            mbar_init(bar(BAR_ACC_EMPTY + i), 4 * NW);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int *abortp = &abort_flag;
    PROF_DECL

    if (warp == 0) {
        // ---- producer ----
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
        if (lane == 0 && !rowcopy) tma_prefetch_desc(&wmap);
        int rs_run = 0, s_run = 0;                        // raw stages and super-blocks fetched so far
        bool ok = true;
        for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
            const Unit U = unit_of(u);
            const uint8_t *act_tile = act + (size_t)U.tile_n * nsb * ACT_CHUNK;
            for (int su = 0; su < nsu; ++su, ++s_run) {
                const int s = U.sb0 + su;                 // the super-block inside the row
                if (s % SPS == 0 && !rowcopy) {               // (row by row: warps 2 and 3 fetch the raw rows, see below)
                    const int st = rs_run % NRAW;
                    if (!WAITP(1, bar(BAR_RAW_EMPTY + st), ((rs_run / NRAW) & 1) ^ 1)) { ok = false; break; }
                    if (lane == 0) {
                        // the whole [128 rows x ROWB] box in one tiled copy; rows past M arrive as zeros
                        mbar_expect_tx(bar(BAR_RAW_FULL + st), L::RAW_STAGE);
                        tma_load_3d(sbase + L::RAW_OFF + st * L::RAW_STAGE, &wmap, ((s / SPS) * SPS * SBB / 16) * 4, U.row0, U.expert,
                                    bar(BAR_RAW_FULL + st));
                    }
                    ++rs_run;
                }
                const int at = s_run % NACT;
                if (!WAITP(3, bar(BAR_ACT_EMPTY + at), ((s_run / NACT) & 1) ^ 1)) { ok = false; break; }
                if (lane == 0) {
                    // only the column groups the tile has; the MMA still reads 128 columns, the rest of the
                    // buffer holds older codes whose products land in accumulator columns nobody stores
                    const uint32_t bytes = (uint32_t)((U.ncols + 7) >> 3) * ACT_GROUP;
                    mbar_expect_tx(bar(BAR_ACT_FULL + at), bytes);
                    bulk_g2s(sbase + L::ACT_OFF + at * ACT_CHUNK, act_tile + (size_t)s * ACT_CHUNK, bytes, bar(BAR_ACT_FULL + at));
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: per block one MMA per limb, accumulating over the super-block ----
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
        int s_run = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
            for (int su = 0; su < nsu && ok; ++su, ++s_run) {
                const int at = s_run % NACT, buf = s_run % NBUF;
                if (!WAITP(2, bar(BAR_ACT_FULL + at), (s_run / NACT) & 1)) { ok = false; break; }
                if (!WAITP(7, bar(BAR_ACC_EMPTY + buf), ((s_run / NBUF) & 1) ^ 1)) { ok = false; break; }
                for (int jg = 0; jg < SB / GB; ++jg) {
                    const int g = s_run * (SB / GB) + jg, gs = g % NG;          // group index, its place in the ring
                    if (!WAITP(4, bar(BAR_A_FULL + gs), (g / NG) & 1)) { ok = false; break; }
                    tc_fence_after();
                    if (lane == 0) {
                        const uint32_t d = tmem_base + (uint32_t)buf * (2 * BN);
#pragma unroll
                        for (int jj = 0; jj < GB; ++jj) {
                            const int j = jg * GB + jj, slot = gs * GB + jj;
                            const uint64_t db = umma_desc2(sbase + L::ACT_OFF + at * ACT_CHUNK + j * 256, 128, ACT_GROUP);
                            umma_i8_acc(d, umma_desc(sbase + L::A_OFF + slot * A_SLOT), db, IDESC, j > 0);
                            umma_i8_acc(d + BN, umma_desc(sbase + L::A_OFF + slot * A_SLOT + OPER_BYTES), db, IDESC, j > 0);
                        }
                        tc_commit(bar(BAR_A_EMPTY + gs));
                        if (jg == SB / GB - 1) {
                            tc_commit(bar(BAR_ACC_FULL + buf));
                            tc_commit(bar(BAR_ACT_EMPTY + at));
                        }
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 40;" ::: "memory");
        // Idle with a tensor map. Rows that are not 16-byte multiples (Q6_K with K = 11008: 9030-byte rows; IQ4_XS with an odd
        // super-block count) cannot be described by one: these two warps then fetch the raw rows, thread t rows t and
        // t + 64, in 16-byte cp.async pieces from the 16-byte boundary below the row's block. The block begins
        // (address % 16) bytes into the row's slot, which the readers add (row_shift); a slot is 8 or 14 bytes wider than a
        // block, so a piece never reaches past the 16-byte unit that holds the block's last byte. Rows past M are not
        // copied (their threads multiply by a zero scale). 128 bulk copies of 224 bytes per stage were tried first: the
        // copy engine's issue rate, not memory, set the pace (4.8 us per stage).
        if (rowcopy) {
            const int t = (int)threadIdx.x - 64;
            int rs_run = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
                const Unit U = unit_of(u);
                for (int su = 0; su < nsu; ++su) {
                    const int s = U.sb0 + su;
                    if (s % SPS != 0) continue;
                    const int st = rs_run % NRAW;
                    if (!WAITP(1, bar(BAR_RAW_EMPTY + st), ((rs_run / NRAW) & 1) ^ 1)) { ok = false; break; }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int rr = t + 64 * h;
                        if (rr < U.valid_rows) {
                            const uintptr_t src = ((uintptr_t)(wraw + (size_t)U.expert * mat_stride + (size_t)(U.row0 + rr) * row_stride +
                                                               (size_t)(s / SPS) * SPS * SBB)) & ~(uintptr_t)15;
                            const uint32_t dstp = sbase + L::RAW_OFF + st * L::RAW_STAGE + rr * ROWB;
#pragma unroll
                            for (int i = 0; i < ROWB / 16; ++i)
                                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dstp + 16 * i), "l"(src + 16 * i) : "memory");
                        }
                    }
                    // one arrival per thread once its copies have landed (none: at once)
                    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar(BAR_RAW_FULL + st)) : "memory");
                    ++rs_run;
                }
            }
            asm volatile("cp.async.wait_all;" ::: "memory");      // nothing of this thread is in flight when the block ends
        }
    } else if (warp < 12) {
        // ---- unpack: two threads per weight row ----
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;" ::: "memory");
        // A half-warp holds eight rows times the two halves, so that the two threads of a row read
        // neighbouring shared-memory words and rows fall on distinct banks.
        const int r = (warp - 4) * 16 + (lane >> 4) * 8 + (lane & 7), kh = (lane >> 3) & 1;
        int rs_run = 0, g_run = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
            const Unit U = unit_of(u);
            const bool row_ok = r < U.valid_rows;
            // where the row's bytes begin inside a 16-byte unit (0 unless rows are copied one by one, see the producer)
            const int row_shift = rowcopy ? (int)(((uintptr_t)wraw + (size_t)U.expert * mat_stride + (size_t)(U.row0 + r) * row_stride) & 15) : 0;
            for (int rsu = 0; rsu < nsu / SPS && ok; ++rsu, ++rs_run) {
                const int rs = U.sb0 / SPS + rsu;         // the raw stage inside the row
                const int st = rs_run % NRAW;
                if (!WAITP(0, bar(BAR_RAW_FULL + st), (rs_run / NRAW) & 1)) { ok = false; break; }
                const uint8_t *rowp = smem + L::RAW_OFF + st * L::RAW_STAGE + r * ROWB + ((row_shift + rs * SPS * SBB) & 15);
#pragma unroll
                for (int h = 0; h < SPS; ++h) {
#pragma unroll
                    for (int jg = 0; jg < SB / GB; ++jg) {
                        const int g = g_run + h * (SB / GB) + jg, gs = g % NG;
                        if (!WAITP(5, bar(BAR_A_EMPTY + gs), ((g / NG) & 1) ^ 1)) { ok = false; break; }
                        unpack_group<TYPE>(rowp + SBB * h, jg, kh, row_ok,
                                           smem + L::A_OFF + (gs * GB) * A_SLOT + (r >> 3) * 128 + (r & 7) * 16);
                        fence_async_smem();                  // one proxy fence per group of blocks
                        mbar_arrive_warp(bar(BAR_A_FULL + gs), lane);
                    }
                    if (!ok) break;
                }
                g_run += SPS * (SB / GB);
                if (ok) mbar_arrive_warp(bar(BAR_RAW_EMPTY + st), lane);
            }
        }
    } else {
        // ---- scale-accumulate, once per super-block ----
        asm volatile("setmaxnreg.inc.sync.aligned.u32 144;" ::: "memory");
        constexpr int CW = BN / NW;
        const int q4 = warp & 3, u4 = (warp - 12) >> 2;
        const int r = q4 * 32 + lane;
        int rs_run = 0, s_run = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
            const Unit U = unit_of(u);
            const bool row_ok = r < U.valid_rows;
            // The tile's columns are shared out between the two warps of a row quadrant: 64 each for a full tile, and
            // for a short one (the ragged end, a route tile of a small expert) half of what there is, in steps of 16.
            const int row_shift = rowcopy ? (int)(((uintptr_t)wraw + (size_t)U.expert * mat_stride + (size_t)(U.row0 + r) * row_stride) & 15) : 0;
            const int cw_eff = U.ncols > CW ? CW : max(16, (((U.ncols + 1) >> 1) + 15) & ~15);
            const int cbase = u4 * cw_eff;
            f32x2 acc2[CW / 2];
#pragma unroll
            for (int c = 0; c < CW / 2; ++c) acc2[c] = 0ull;
            for (int su = 0; su < nsu; ++su, ++s_run) {
                const int s = U.sb0 + su;
                if (s % SPS == 0 && su > 0) ++rs_run;
                const int st = rs_run % NRAW, at = s_run % NACT, buf = s_run % NBUF;
                // stage barriers cannot advance past this thread: it releases both stages itself
                if (s % SPS == 0 && !WAITP(0, bar(BAR_RAW_FULL + st), (rs_run / NRAW) & 1)) { ok = false; break; }
                if (!WAITP(2, bar(BAR_ACT_FULL + at), (s_run / NACT) & 1)) { ok = false; break; }
                if (!WAITP(6, bar(BAR_ACC_FULL + buf), (s_run / NBUF) & 1)) { ok = false; break; }
                tc_fence_after();
                const float dwb = row_ok ? half_bits_to_float(*reinterpret_cast<const uint16_t *>(
                                               smem + L::RAW_OFF + st * L::RAW_STAGE + r * ROWB + ((row_shift + (s / SPS) * SPS * SBB) & 15) +
                                               SBB * (s % SPS) + Fmt<FV>::D_OFF)) : 0.f;
                const f32x2 dw2 = f2_pack(dwb, dwb);
                // Q4_K route tiles take the mins term here (a short tile leaves these warps idle most of the time, and
                // a separate pass would read and write all of dst again): the row's eight mins and -dmin
                uint32_t m03 = 0, m47 = 0;
                f32x2 ndm2 = 0ull;
                if ((TYPE == B200Q_TYPE_Q4_K || TYPE == B200Q_TYPE_Q5_K) && fold_mins) {
                    const uint4 hdr = *reinterpret_cast<const uint4 *>(smem + L::RAW_OFF + st * L::RAW_STAGE + r * ROWB);
                    q4k_mins8(hdr.y, hdr.z, hdr.w, &m03, &m47);
                    const float ndm = row_ok ? -half_bits_to_float((uint16_t)(hdr.x >> 16)) : 0.f;
                    ndm2 = f2_pack(ndm, ndm);
                }
                const uint32_t dxa = sbase + L::ACT_OFF + at * ACT_CHUNK + (cbase / 8) * ACT_GROUP + ACT_SCALES;   // scales of this thread's first group
                const uint32_t taddr = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)buf * (2 * BN) + (uint32_t)cbase;
                const int ncol = min(cw_eff, U.ncols - cbase);   // this thread's columns inside the tile (warp-uniform)
#pragma unroll
                for (int q = 0; q < CW / 16; ++q) {
                    if (q * 16 >= ncol) {                    // a short tile (the ragged end, a small expert): nothing to scale
                        if (q == CW / 16 - 1) {
                            tc_fence_before();
                            mbar_arrive_warp(bar(BAR_ACC_EMPTY + buf), lane);
                        }
                        continue;
                    }
                    uint32_t vh[16], vl[16];
                    tmem_ld16(taddr + q * 16, vh);
                    tmem_ld16(taddr + BN + q * 16, vl);
                    f32x2 dx[8];                             // sixteen activation scales, in flight under the tensor-memory loads
#pragma unroll
                    for (int c = 0; c < 4; ++c) lds128_f2(dxa + (2 * q + (c >> 1)) * ACT_GROUP + (c & 1) * 16, dx[2 * c], dx[2 * c + 1]);
                    tmem_ld_wait();
                    if (q == CW / 16 - 1) {
                        tc_fence_before();
                        mbar_arrive_warp(bar(BAR_ACC_EMPTY + buf), lane);
                    }
#pragma unroll
                    for (int c = 0; c < 16; c += 4) {
                        const int e = (q * 16 + c) / 2;
                        // 256 hi + lo as an integer, one rounding to float (ggml's float(sumi))
                        const f32x2 s01 = f2_pack(__int2float_rn((int)vl[c] + ((int)vh[c] << 8)), __int2float_rn((int)vl[c + 1] + ((int)vh[c + 1] << 8)));
                        const f32x2 s23 = f2_pack(__int2float_rn((int)vl[c + 2] + ((int)vh[c + 2] << 8)), __int2float_rn((int)vl[c + 3] + ((int)vh[c + 3] << 8)));
                        acc2[e]     = f2_fma(s01, f2_mul(dw2, dx[c / 2]), acc2[e]);
                        acc2[e + 1] = f2_fma(s23, f2_mul(dw2, dx[c / 2 + 1]), acc2[e + 1]);
                    }
                    if ((TYPE == B200Q_TYPE_Q4_K || TYPE == B200Q_TYPE_Q5_K) && fold_mins) {
                        // - dmin d_x sum_j m_j bsum_j per live column: the digits come by broadcast loads from the
                        // chunk, four dp4a per column (as q4k_mins_rows_kernel, without its pass over dst). Eight
                        // columns' loads are issued together and their chains are independent, so the latencies overlap.
                        const uint32_t dga = dxa - ACT_SCALES + ACT_DIGITS + (2 * q) * ACT_GROUP;
#pragma unroll
                        for (int g8 = 0; g8 < 2; ++g8) {
                            if (q * 16 + 8 * g8 < ncol) {        // warp-uniform
                                uint4 dg[8];
#pragma unroll
                                for (int c = 0; c < 8; ++c) dg[c] = *reinterpret_cast<const uint4 *>(smem + (dga - sbase) + g8 * ACT_GROUP + c * 16);
                                float t[8];
#pragma unroll
                                for (int c = 0; c < 8; ++c) {
                                    const int lo = __dp4a((int)m47, (int)dg[c].y, __dp4a((int)m03, (int)dg[c].x, 0));
                                    const int hi = __dp4a((int)m47, (int)dg[c].w, __dp4a((int)m03, (int)dg[c].z, 0));
                                    t[c] = __int2float_rn(lo + (hi << 8));
                                }
#pragma unroll
                                for (int c = 0; c < 8; c += 2) {
                                    const int e = (q * 16 + 8 * g8 + c) / 2;
                                    acc2[e] = f2_fma(f2_pack(t[c], t[c + 1]), f2_mul(ndm2, dx[(8 * g8 + c) / 2]), acc2[e]);
                                }
                            }
                        }
                    }
                }
                mbar_arrive_warp(bar(BAR_ACT_EMPTY + at), lane);
                if (s % SPS == SPS - 1) mbar_arrive_warp(bar(BAR_RAW_EMPTY + st), lane);
            }
            ++rs_run;                                    // past the unit's last raw stage
            if (ok) {
                const int ncol = min(cw_eff, U.ncols - cbase);   // this thread's columns inside the tile
                if (id.tiles) {
                    // where the warp's 64 columns go: every lane looks up two of them (loads in flight
                    // together), the store loop takes them by shuffle -- a load and a division per column
                    // inside that loop would serialize 64 memory latencies
                    long long off[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        off[h] = 0;
                        if (lane + 32 * h < ncol) {
                            const int p = __ldg(id.pairs + U.first + cbase + lane + 32 * h), tok = p / id.n_used, slot = p - tok * id.n_used;
                            off[h] = tok * id.ld2 + slot * id.ld1;
                        }
                    }
#pragma unroll
                    for (int c = 0; c < CW; c += 2) {
                        float a[2];
                        f2_unpack(acc2[c / 2], a[0], a[1]);
#pragma unroll
                        for (int d = 0; d < 2; ++d) {
                            const long long o = __shfl_sync(0xFFFFFFFFu, off[(c + d) >> 5], (c + d) & 31);
                            if (row_ok && c + d < ncol) dst[o + U.row0 + r] = a[d];
                        }
                    }
                } else if (row_ok) {
                    float *o = dst + (int64_t)(U.tile_n * BN + cbase) * ldd + U.row0 + r;
#pragma unroll
                    for (int c = 0; c < CW; c += 2) {
                        float a0, a1;
                        f2_unpack(acc2[c / 2], a0, a1);
                        if (ksplit > 1) {
                            if (c < ncol) atomicAdd(o, a0);
                            if (c + 1 < ncol) atomicAdd(o + ldd, a1);
                        } else {
                            if (c < ncol) *o = a0;
                            if (c + 1 < ncol) o[ldd] = a1;
                        }
                        o += 2 * ldd;
                    }
                }
            }
        }
    }

    PROF_DUMP(warp == 0 ? "prod" : warp == 1 ? "mma " : warp < 4 ? "idle" : warp < 12 ? "unpk" : "epi ")
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        if (threadIdx.x == 0) atomicExch(error_word, 2);
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// Q4_K's second term: dst[c][r] -= sum_sb dmin[r, sb] * d_x[c, sb] * sum_j m_j[r, sb] * bsum_j[c, sb], with
// bsum_j the integer sum of the activation codes of sub-block j (written by the tiled quantizer
// beside the chunks). The inner sum is an exact small-integer product, so it goes through a warp-level
// f16 MMA (m16n8k16, f32 accumulate): a row of A is [m_0..m_7, m_0..m_7], a column of B is
// [bl_0..bl_7, 256 bh_0..256 bh_7] with bsum = 256 bh + bl (bl in [-128, 127], 256 bh a multiple of 256 up
// to 4096: all exact in f16, every partial sum an integer below 2^24, exact in f32). What is left per output
// element and super-block is the scale dmin * d_x and one fused multiply-add.
// A block takes MR = 64 rows (16 per warp) and MC = 64 columns of one column tile.
constexpr int MC = 64, MR = 64;
__device__ __forceinline__ void mma_m16n8k16_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %11, %12, %13};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f), "f"(0.f), "f"(0.f), "f"(0.f));
}
// two small non-negative integers (one per byte of the low 16 bits) as an f16 pair: 1024 + v is the bit
// pattern 0x6400 | v, then subtract 1024
__device__ __forceinline__ uint32_t u8x2_to_h2(uint32_t two_bytes) {
    const uint32_t bits = 0x64006400u | (two_bytes & 0xFFu) | ((two_bytes & 0xFF00u) << 8);
    const __half2 h = __hsub2(*reinterpret_cast<const __half2 *>(&bits), __half2half2(__ushort_as_half((unsigned short)0x6400)));
    return *reinterpret_cast<const uint32_t *>(&h);
}

__global__ void __launch_bounds__(128)
q4k_mins_kernel(const uint8_t *__restrict__ W, size_t row_stride, size_t mat_stride, int M, int nsb,
                const uint8_t *__restrict__ act, const int16_t *__restrict__ bsum, int N, float *__restrict__ dst,
                int64_t ldd, TileRoute id, int blk_bytes) {
    __shared__ __align__(16) uint32_t cb[2][MC][8];       // per column: for q < 4 the f16 pairs (bl_2q, bl_2q+1), 256 (bh_2q, bh_2q+1)
    __shared__ __align__(8) float cdx[2][MC];
    const int tile = blockIdx.x / (BN / MC), cc0 = (blockIdx.x % (BN / MC)) * MC;   // columns cc0 .. cc0 + MC - 1 of the tile
    int expert = 0, first = 0, ncols = min(BN, N - tile * BN);
    if (id.tiles) {
        if (tile >= __ldg(id.n_tiles)) return;
        expert = __ldg(id.tiles + 4 * tile);
        first = __ldg(id.tiles + 4 * tile + 1);
        ncols = __ldg(id.tiles + 4 * tile + 2);
    }
    if (cc0 >= ncols) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
    // the thread's two rows of the warp's sixteen (the MMA's row g and row g + 8)
    const int r0 = blockIdx.y * MR + warp * 16 + g, r1 = r0 + 8;
    const uint8_t *wbase = W + (size_t)expert * mat_stride;
    const uint8_t *w0 = wbase + (size_t)min(r0, M - 1) * row_stride, *w1 = wbase + (size_t)min(r1, M - 1) * row_stride;
    const int n_tiles8 = (min(MC, ncols - cc0) + 7) >> 3;                         // 8-column MMA tiles with live columns
    float acc[MC / 8][4];
#pragma unroll
    for (int t = 0; t < MC / 8; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;
    uint4 h0n = __ldg(reinterpret_cast<const uint4 *>(w0)), h1n = __ldg(reinterpret_cast<const uint4 *>(w1));
    // the staging threads (one per column) keep the next super-block's sums and scale in flight while this one's
    // MMAs run: a load consumed at once would stall them, and everybody else at the barrier behind them
    const int cc = cc0 + (int)threadIdx.x;
    const bool stager = threadIdx.x < MC, col_ok = stager && cc < ncols;
    int4 sv = make_int4(0, 0, 0, 0);
    float dxv = 0.f;
    auto fetch = [&](int sb) {
        const size_t chunk = (size_t)tile * nsb + sb;
        sv = __ldg(reinterpret_cast<const int4 *>(bsum + (chunk * BN + cc) * 8));
        dxv = __ldg(reinterpret_cast<const float *>(act + chunk * ACT_CHUNK + (cc >> 3) * ACT_GROUP + ACT_SCALES) + (cc & 7));
    };
    if (col_ok) fetch(0);
    for (int sb = 0; sb < nsb; ++sb) {
        const int pb = sb & 1;
        if (stager) {
            // stage the column's eight block sums as the B operand's f16 digits, and its scale
            uint32_t w[8] = { 0, 0, 0, 0, 0, 0, 0, 0 };
            if (col_ok) {
                const int v[4] = { sv.x, sv.y, sv.z, sv.w };
#pragma unroll
                for (int qq = 0; qq < 4; ++qq) {
                    const int s0 = (int)(int16_t)((uint32_t)v[qq] & 0xFFFFu), s1 = (int)(int16_t)((uint32_t)v[qq] >> 16);
                    const int h0 = (s0 + 128) >> 8, h1 = (s1 + 128) >> 8;
                    const __half2 lo = __floats2half2_rn((float)(s0 - 256 * h0), (float)(s1 - 256 * h1));
                    const __half2 hi = __floats2half2_rn((float)(256 * h0), (float)(256 * h1));
                    w[2 * qq] = *reinterpret_cast<const uint32_t *>(&lo);
                    w[2 * qq + 1] = *reinterpret_cast<const uint32_t *>(&hi);
                }
            }
            *reinterpret_cast<uint4 *>(&cb[pb][threadIdx.x][0]) = make_uint4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<uint4 *>(&cb[pb][threadIdx.x][4]) = make_uint4(w[4], w[5], w[6], w[7]);
            cdx[pb][threadIdx.x] = col_ok ? dxv : 0.f;
            if (col_ok && sb + 1 < nsb) fetch(sb + 1);
        }
        const uint4 h0 = h0n, h1 = h1n;                      // d, dmin | 12 scale bytes of the two rows' blocks
        if (sb + 1 < nsb) {
            h0n = __ldg(reinterpret_cast<const uint4 *>(w0 + (size_t)(sb + 1) * blk_bytes));      // 144 Q4_K, 176 Q5_K: the same header
            h1n = __ldg(reinterpret_cast<const uint4 *>(w1 + (size_t)(sb + 1) * blk_bytes));
        }
        uint32_t m03, m47, a[4];
        q4k_mins8(h0.y, h0.z, h0.w, &m03, &m47);
        a[0] = u8x2_to_h2(((q < 2 ? m03 : m47) >> (16 * (q & 1))) & 0xFFFFu);          // row g:     m_2q, m_2q+1
        q4k_mins8(h1.y, h1.z, h1.w, &m03, &m47);
        a[1] = u8x2_to_h2(((q < 2 ? m03 : m47) >> (16 * (q & 1))) & 0xFFFFu);          // row g + 8
        a[2] = a[0];                                                                     // k + 8: the same mins against the high digits
        a[3] = a[1];
        const float dm0 = r0 < M ? half_bits_to_float((uint16_t)(h0.x >> 16)) : 0.f;
        const float dm1 = r1 < M ? half_bits_to_float((uint16_t)(h1.x >> 16)) : 0.f;
        __syncthreads();                       // the other buffer is read by nobody: its readers are two barriers back
#pragma unroll
        for (int t = 0; t < MC / 8; ++t) {
            if (t < n_tiles8) {                                  // block-uniform
                const uint2 b = *reinterpret_cast<const uint2 *>(&cb[pb][8 * t + g][2 * q]);
                const float2 dx = *reinterpret_cast<const float2 *>(&cdx[pb][8 * t + 2 * q]);
                float d[4];
                mma_m16n8k16_f16(d, a, b.x, b.y);
                acc[t][0] = fmaf(dm0 * dx.x, d[0], acc[t][0]);
                acc[t][1] = fmaf(dm0 * dx.y, d[1], acc[t][1]);
                acc[t][2] = fmaf(dm1 * dx.x, d[2], acc[t][2]);
                acc[t][3] = fmaf(dm1 * dx.y, d[3], acc[t][3]);
            }
        }
    }
    // Read-modify-write of the outputs. The thread holds rows r0, r1 and columns 8 t + 2 q, + 1 of every MMA
    // tile; all loads of a pass are issued before its stores (a load, a subtraction and a store per element in
    // one loop would serialize the memory latencies).
#pragma unroll
    for (int t0 = 0; t0 < MC / 8; t0 += 4) {
        long long off[4][2];
        float old[4][4];
#pragma unroll
        for (int tt = 0; tt < 4; ++tt)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int c = cc0 + 8 * (t0 + tt) + 2 * q + j;
                off[tt][j] = -1;
                if (c < ncols) {
                    if (id.tiles) {
                        const int p = __ldg(id.pairs + first + c), tok = p / id.n_used, slot = p - tok * id.n_used;
                        off[tt][j] = tok * id.ld2 + slot * id.ld1;
                    } else {
                        off[tt][j] = (int64_t)(tile * BN + c) * ldd;
                    }
                }
            }
#pragma unroll
        for (int tt = 0; tt < 4; ++tt)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                old[tt][j] = off[tt][j] >= 0 && r0 < M ? dst[off[tt][j] + r0] : 0.f;
                old[tt][2 + j] = off[tt][j] >= 0 && r1 < M ? dst[off[tt][j] + r1] : 0.f;
            }
#pragma unroll
        for (int tt = 0; tt < 4; ++tt)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                if (off[tt][j] >= 0 && r0 < M) dst[off[tt][j] + r0] = old[tt][j] - acc[t0 + tt][j];
                if (off[tt][j] >= 0 && r1 < M) dst[off[tt][j] + r1] = old[tt][2 + j] - acc[t0 + tt][2 + j];
            }
    }
}

// The same term with one thread per weight row and four dp4a per element (bsum split into two int8 digits),
// looping over the live columns only: the form for MUL_MAT_ID route tiles, which are mostly short and whose
// K is small, so that a block's fixed costs and the width of its stores weigh more than the arithmetic
// (measured on config 5: 123 / 209 us for gate / down against 178 / 334 us with the MMA form above).
__global__ void __launch_bounds__(128)
q4k_mins_rows_kernel(const uint8_t *__restrict__ W, size_t row_stride, size_t mat_stride, int M, int nsb,
                const uint8_t *__restrict__ act, const int16_t *__restrict__ bsum, int N, float *__restrict__ dst,
                int64_t ldd, TileRoute id, int blk_bytes) {
    __shared__ __align__(16) uint32_t cs[2][MC][4];       // bl 0..3, bl 4..7, bh 0..3, bh 4..7
    __shared__ float cdx[2][MC];
    const int tile = blockIdx.x / (BN / MC), cc0 = (blockIdx.x % (BN / MC)) * MC;   // columns cc0 .. cc0 + MC - 1 of the tile
    int expert = 0, first = 0, ncols = min(BN, N - tile * BN);
    if (id.tiles) {
        if (tile >= __ldg(id.n_tiles)) return;
        expert = __ldg(id.tiles + 4 * tile);
        first = __ldg(id.tiles + 4 * tile + 1);
        ncols = __ldg(id.tiles + 4 * tile + 2);
    }
    if (cc0 >= ncols) return;
    const int r = blockIdx.y * 128 + threadIdx.x;
    const bool row_ok = r < M;
    const uint8_t *wrow = W + (size_t)expert * mat_stride + (size_t)(row_ok ? r : 0) * row_stride;
    float acc[MC];
#pragma unroll
    for (int c = 0; c < MC; ++c) acc[c] = 0.f;
    uint4 hdr_next = __ldg(reinterpret_cast<const uint4 *>(wrow));          // d, dmin | 12 scale bytes of block 0
    for (int sb = 0; sb < nsb; ++sb) {
        const int pb = sb & 1;
        const uint4 hdr = hdr_next;
        if (sb + 1 < nsb) hdr_next = __ldg(reinterpret_cast<const uint4 *>(wrow + (size_t)(sb + 1) * blk_bytes));   // in flight under the math
        if (threadIdx.x < MC) {
            const int cc = cc0 + threadIdx.x;
            uint32_t w[4] = { 0, 0, 0, 0 };
            float dx = 0.f;
            if (cc < ncols) {
                const size_t chunk = (size_t)tile * nsb + sb;
                const int4 sv = *reinterpret_cast<const int4 *>(bsum + (chunk * BN + cc) * 8);
                const int v[4] = { sv.x, sv.y, sv.z, sv.w };
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int s = (int)(int16_t)(((uint32_t)v[i >> 1] >> (16 * (i & 1))) & 0xFFFFu);
                    const int bh = (s + 128) >> 8, bl = s - 256 * bh;
                    w[i >> 2] |= (uint32_t)(bl & 0xFF) << (8 * (i & 3));
                    w[2 + (i >> 2)] |= (uint32_t)(bh & 0xFF) << (8 * (i & 3));
                }
                dx = reinterpret_cast<const float *>(act + chunk * ACT_CHUNK + (cc >> 3) * ACT_GROUP + ACT_SCALES)[cc & 7];
            }
            *reinterpret_cast<uint4 *>(cs[pb][threadIdx.x]) = make_uint4(w[0], w[1], w[2], w[3]);
            cdx[pb][threadIdx.x] = dx;
        }
        uint32_t m03, m47;
        q4k_mins8(hdr.y, hdr.z, hdr.w, &m03, &m47);
        const float dmin = row_ok ? half_bits_to_float((uint16_t)(hdr.x >> 16)) : 0.f;
        __syncthreads();                       // the other buffer is read by nobody: its readers are two barriers back
#pragma unroll
        for (int c8 = 0; c8 < MC; c8 += 8) {
            if (cc0 + c8 < ncols) {                          // block-uniform: route tiles are mostly short
#pragma unroll
                for (int c = c8; c < c8 + 8; ++c) {
                    const uint4 b = *reinterpret_cast<const uint4 *>(cs[pb][c]);
                    const int lo = __dp4a((int)m47, (int)b.y, __dp4a((int)m03, (int)b.x, 0));
                    const int hi = __dp4a((int)m47, (int)b.w, __dp4a((int)m03, (int)b.z, 0));
                    acc[c] = fmaf(dmin * cdx[pb][c], (float)(lo + (hi << 8)), acc[c]);
                }
            }
        }
    }
    // Read-modify-write of the outputs in two passes, all loads first: a load, a subtraction and a store
    // per column in one loop would serialize 64 memory latencies. The destinations of the block's columns
    // are looked up two per lane and handed round by shuffle.
    long long off[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int c = (threadIdx.x & 31) + 32 * h;
        off[h] = 0;
        if (cc0 + c < ncols) {
            if (id.tiles) {
                const int p = __ldg(id.pairs + first + cc0 + c), tok = p / id.n_used, slot = p - tok * id.n_used;
                off[h] = tok * id.ld2 + slot * id.ld1;
            } else {
                off[h] = (int64_t)(tile * BN + cc0 + c) * ldd;
            }
        }
    }
#pragma unroll
    for (int c0 = 0; c0 < MC; c0 += 16) {
        float old[16];
#pragma unroll
        for (int c = c0; c < c0 + 16; ++c) {
            const long long o = __shfl_sync(0xFFFFFFFFu, off[c >> 5], c & 31);
            old[c - c0] = row_ok && cc0 + c < ncols ? dst[o + r] : 0.f;
        }
#pragma unroll
        for (int c = c0; c < c0 + 16; ++c) {
            const long long o = __shfl_sync(0xFFFFFFFFu, off[c >> 5], c & 31);
            if (row_ok && cc0 + c < ncols) dst[o + r] = old[c - c0] - acc[c];
        }
    }
}

}  // namespace kq

static size_t kq_chunks(int64_t K, int64_t N) { return (size_t)(((N + kq::BN - 1) / kq::BN) * (K / 256)); }
static const TileRoute NO_ROUTE = { nullptr, nullptr, nullptr, 1, 1, 0, 0, 0, 0 };

size_t gemm_kq_act_bytes(int64_t K, int64_t N) {
    return kq_chunks(K, N) * (kq::ACT_CHUNK + kq::BN * 8 * sizeof(int16_t));      // chunks, then block sums
}
size_t gemm_kq_id_act_bytes(int64_t K, int64_t max_tiles) { return gemm_kq_act_bytes(K, max_tiles * kq::BN); }

bool gemm_kq_supported(int type, int64_t M, int64_t K, int64_t N, const void *w, size_t row_stride) {
    if (type != B200Q_TYPE_IQ4_XS && type != B200Q_TYPE_Q4_K && type != B200Q_TYPE_Q5_K && type != B200Q_TYPE_Q6_K) return false;
    // raw stages are whole super-blocks in 16-byte pieces: two per stage for IQ4_XS, one for Q4_K. Q6_K rows of 210-byte
    // blocks are 16-byte multiples only every 8 blocks: other lengths (K = 11008) take the row-by-row staging, which
    // needs an even row stride only.
    // IQ4_XS stages two 136-byte super-blocks at a time through a tensor map when K is a multiple of 512, and row by row,
    // one at a time, otherwise (8-byte row stride).
    if (K <= 0 || K % 256 || M <= 0 || N <= 0) return false;
    if ((uintptr_t)w % 16 || row_stride % (type == B200Q_TYPE_Q6_K ? 2 : type == B200Q_TYPE_IQ4_XS ? 8 : 16)) return false;
    if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return false;
    return true;
}

static b200q_status quantize256(b200q_ctx *ctx, const b200q_tensor *src1, uint8_t *out, int64_t n_tiles, const TileRoute &tr) {
    const int64_t K = src1->ne[0];
    dim3 grid((unsigned)(K / 256), (unsigned)n_tiles);
    int16_t *bsum = reinterpret_cast<int16_t *>(out + (size_t)(n_tiles * (K / 256)) * kq::ACT_CHUNK);
    kq::quantize_tiled256_kernel<<<grid, 256, 0, ctx->stream>>>((const uint8_t *)src1->data, src1->ne[1], src1->ne[2], src1->nb[1],
                                                               src1->nb[2], src1->nb[3], K, src1->ne[1] * src1->ne[2] * src1->ne[3],
                                                               out, bsum, tr);
    B200Q_CUDA(ctx, cudaGetLastError());
    count(ctx, ST_GEMM_TC_QUANT);
    return B200Q_OK;
}

b200q_status launch_quantize_tiled256(b200q_ctx *ctx, const b200q_tensor *src1, uint8_t *out) {
    const int64_t N = src1->ne[1] * src1->ne[2] * src1->ne[3];
    return quantize256(ctx, src1, out, (N + kq::BN - 1) / kq::BN, NO_ROUTE);
}

// n_tiles: grid width (dense: the tiles of N; MUL_MAT_ID: the upper bound of the route's tile count,
// blocks past the device-side count leave at once)
template <int TYPE, int FV = TYPE>
static b200q_status launch_kq_t(b200q_ctx *ctx, const void *w, size_t row_stride, size_t mat_stride, int64_t n_mat, int64_t M,
                                int64_t K, const uint8_t *act, int64_t N, int64_t n_tiles, float *dst, int64_t ldd,
                                const TileRoute &tr) {
    typedef kq::Smem<FV> L;
    auto kern = kq::gemm_kq_kernel<TYPE, FV>;
    static bool attr_set_dev[B200Q_MAX_DEVICES] = {};
    bool &attr_set = attr_set_dev[ctx->device % B200Q_MAX_DEVICES];
    if (!attr_set) {
        B200Q_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::TOTAL));
        attr_set = true;
    }
    // rows a tensor map cannot describe (Q6_K whose row length is not a 16-byte multiple) are staged row by row
    const int rowcopy = FV != TYPE || (TYPE == B200Q_TYPE_Q6_K && (row_stride % 16 != 0 || K % 2048 != 0 || mat_stride % 16 != 0));
    CUtensorMap wmap;
    memset(&wmap, 0, sizeof(wmap));
    if (!rowcopy) {
        b200q_status st = make_weight_tmap3(ctx, &wmap, w, row_stride, M, (K / 256) * L::SBB, L::ROWB, n_mat, mat_stride);
        if (st != B200Q_OK) return st;
    } else {
        count(ctx, ST_GEMM_KQ_ROWCOPY);
    }
    // persistent blocks, one per SM, walking the (row tile, column tile) units
    int64_t units = n_tiles * ((M + kq::BM - 1) / kq::BM);
    // split K in two when that shortens the schedule: rounds of whole units against rounds of half units
    int ksplit = 1;
    const int64_t S = ctx->sm_count, nsb = K / 256;
    if (!tr.tiles && nsb % (2 * L::SPS) == 0 && nsb >= 8 && 2 * ((units + S - 1) / S) > (2 * units + S - 1) / S) {
        ksplit = 2;
        B200Q_CUDA(ctx, cudaMemset2DAsync(dst, (size_t)ldd * sizeof(float), 0, (size_t)M * sizeof(float), (size_t)N, ctx->stream));
        units *= 2;
    }
    const unsigned grid = (unsigned)(units < S ? units : S);
    // route tiles of Q4_K: the mins term inside the GEMM (B200Q_MOE_MINS_PASS=1 keeps the separate pass, for comparison)
    const int fold = (TYPE == B200Q_TYPE_Q4_K || TYPE == B200Q_TYPE_Q5_K) && tr.tiles && !ctx->moe_mins_pass;
    kern<<<grid, kq::THREADS, L::TOTAL, ctx->stream>>>(wmap, (int)M, (int)K, act, (int)N, (int)n_tiles, ksplit, dst, ldd,
                                                       ctx->error_word, tr, fold, (const uint8_t *)w, row_stride, mat_stride, rowcopy);
    B200Q_CUDA(ctx, cudaGetLastError());
    count(ctx, ST_GEMM_TC);
    if (TYPE == B200Q_TYPE_Q4_K || TYPE == B200Q_TYPE_Q5_K) {
        // the mins term, subtracted in place
        const int16_t *bsum = reinterpret_cast<const int16_t *>(act + (size_t)(n_tiles * (K / 256)) * kq::ACT_CHUNK);
        if (tr.tiles && ctx->moe_mins_pass) {
            dim3 g2((unsigned)(n_tiles * (kq::BN / kq::MC)), (unsigned)((M + 127) / 128));
            kq::q4k_mins_rows_kernel<<<g2, 128, 0, ctx->stream>>>((const uint8_t *)w, row_stride, mat_stride, (int)M, (int)(K / 256), act,
                                                                 bsum, (int)N, dst, ldd, tr, (int)L::SBB);
        } else if (tr.tiles) {
            return B200Q_OK;                     // route tiles: the term was taken inside the GEMM
        } else {
            dim3 g2((unsigned)(n_tiles * (kq::BN / kq::MC)), (unsigned)((M + kq::MR - 1) / kq::MR));
            kq::q4k_mins_kernel<<<g2, 128, 0, ctx->stream>>>((const uint8_t *)w, row_stride, mat_stride, (int)M, (int)(K / 256), act, bsum,
                                                            (int)N, dst, ldd, tr, (int)L::SBB);
        }
        B200Q_CUDA(ctx, cudaGetLastError());
        count(ctx, ST_GEMM_KQ_MINS);
    }
    return B200Q_OK;
}

// IQ4_XS shapes the two-super-block tensor-map staging cannot take: an odd super-block count, or strides that are not
// 16-byte multiples
static bool iq4_rows(int64_t K, size_t row_stride, size_t mat_stride) { return K % 512 != 0 || row_stride % 16 != 0 || mat_stride % 16 != 0; }

b200q_status launch_gemm_kq(b200q_ctx *ctx, int type, const void *w, size_t row_stride, int64_t M, int64_t K,
                            const uint8_t *act, int64_t N, float *dst, int64_t ldd) {
    const int64_t n_tiles = (N + kq::BN - 1) / kq::BN;
    const size_t ms = row_stride * (size_t)M;
    if (type == B200Q_TYPE_IQ4_XS && iq4_rows(K, row_stride, ms))
        return launch_kq_t<B200Q_TYPE_IQ4_XS, kq::FMT_IQ4_XS_ROWS>(ctx, w, row_stride, ms, 1, M, K, act, N, n_tiles, dst, ldd, NO_ROUTE);
    if (type == B200Q_TYPE_IQ4_XS) return launch_kq_t<B200Q_TYPE_IQ4_XS>(ctx, w, row_stride, ms, 1, M, K, act, N, n_tiles, dst, ldd, NO_ROUTE);
    if (type == B200Q_TYPE_Q4_K) return launch_kq_t<B200Q_TYPE_Q4_K>(ctx, w, row_stride, ms, 1, M, K, act, N, n_tiles, dst, ldd, NO_ROUTE);
    if (type == B200Q_TYPE_Q5_K) return launch_kq_t<B200Q_TYPE_Q5_K>(ctx, w, row_stride, ms, 1, M, K, act, N, n_tiles, dst, ldd, NO_ROUTE);
    if (type == B200Q_TYPE_Q6_K) return launch_kq_t<B200Q_TYPE_Q6_K>(ctx, w, row_stride, ms, 1, M, K, act, N, n_tiles, dst, ldd, NO_ROUTE);
    return fail(ctx, B200Q_UNSUPPORTED, "gemm_kq: type %d", type);
}

// MUL_MAT_ID on the tensor cores: the route's 128-pair tiles are the column tiles; the activation of
// every tile is gathered and quantized into `act` (gemm_kq_id_act_bytes) first.
b200q_status launch_gemm_kq_id(b200q_ctx *ctx, const b200q_tensor *src0, const b200q_tensor *src1, const TileRoute &tr,
                               int64_t max_tiles, uint8_t *act, float *dst, bool act_ready) {
    const int64_t K = src0->ne[0], M = src0->ne[1];
    b200q_status st = act_ready ? B200Q_OK : quantize256(ctx, src1, act, max_tiles, tr);
    if (st != B200Q_OK) return st;
    if (src0->type == B200Q_TYPE_IQ4_XS)
        return iq4_rows(K, src0->nb[1], src0->nb[2])
                   ? launch_kq_t<B200Q_TYPE_IQ4_XS, kq::FMT_IQ4_XS_ROWS>(ctx, src0->data, src0->nb[1], src0->nb[2], src0->ne[2], M, K, act, 0,
                                                                         max_tiles, dst, 0, tr)
                   : launch_kq_t<B200Q_TYPE_IQ4_XS>(ctx, src0->data, src0->nb[1], src0->nb[2], src0->ne[2], M, K, act, 0, max_tiles, dst, 0, tr);
    if (src0->type == B200Q_TYPE_Q4_K)
        return launch_kq_t<B200Q_TYPE_Q4_K>(ctx, src0->data, src0->nb[1], src0->nb[2], src0->ne[2], M, K, act, 0, max_tiles, dst, 0, tr);
    if (src0->type == B200Q_TYPE_Q5_K)
        return launch_kq_t<B200Q_TYPE_Q5_K>(ctx, src0->data, src0->nb[1], src0->nb[2], src0->ne[2], M, K, act, 0, max_tiles, dst, 0, tr);
    if (src0->type == B200Q_TYPE_Q6_K)
        return launch_kq_t<B200Q_TYPE_Q6_K>(ctx, src0->data, src0->nb[1], src0->nb[2], src0->ne[2], M, K, act, 0, max_tiles, dst, 0, tr);
    return fail(ctx, B200Q_UNSUPPORTED, "gemm_kq_id: type %d", src0->type);
}

}  // namespace b200q
