// gemm_tc.cu -- prefill GEMM for the per-32 types (Q4_0, Q8_0, IQ4_NL) on the 5th-generation tensor cores.
//
//   dst[M, N] = W[M, K] (packed GGUF blocks) x X[K, N] (f32), N > 8 tokens
//
// ggml's form is kept exactly: the activation is quantized per 32 to int8 with an fp16
// scale (block_q8_0), every 32-wide block dot I_b[r, c] is an exact int32 from one
// tcgen05.mma kind::i8 (M=128, N=128, K=32) whose accumulator lives in tensor memory,
// and the result is sum_b float(I_b) * d_w[r, b] * d_x[c, b] in f32 -- the arithmetic of
// the reference's int8 GEMM (marfrit/arcint contrib/llama.cpp/patches/
// 0099-opencl-q4_0-q8_0-int8-gemm.patch:377-455, 583-628: one int8 DPAS per 32 weights,
// af = fma(float(ir), d_w, af)), with ggml's per-32 activation scale instead of the
// reference's per-256 one.
//
// One CTA owns a 128-row x 128-token output tile. Warp roles:
//   warp 0      producer: bulk copies (cp.async.bulk + mbarrier complete_tx) of the raw
//               packed weight rows of a k-stage (256 weights per row) and of the
//               activation chunk (int8 codes already in the tensor core's K-major core-matrix
//               order, plus their scales), three stages deep;
//   warp 1      allocates tensor memory, issues the MMAs (one elected thread) and commits
//               them to mbarriers;
//   warps 4..7  one thread per weight row: unpack the row's blocks to int8 (code - 8) into
//               the A-operand ring in core-matrix order and publish the block's fp16 scale;
//   warps 8..   scale-accumulate, NW warps per tensor-memory lane quarter: pull the finished
//               block accumulator out of tensor memory (tcgen05.ld), free it, convert, scale by
//               d_w * d_x and accumulate into f32 registers (thread = row x 128/NW columns).
// Four 128-column accumulators fill the 512 tensor-memory columns, so the MMA of block b+1..
// b+3 runs while block b is being scaled. The scaling is the bound, not the tensor pipe:
// every output element needs a convert, a multiply and a fused multiply-add per 32 of K,
// 16K elements per block against 128 FP32 lanes per SM and clock.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets an error word, all roles
// leave their loops, tensor memory is freed and the launch reports B200Q_TIMEOUT at the
// next synchronize.
#include <cuda.h>

#include "formats.cuh"
#include "common.cuh"
#include "tc_common.cuh"

namespace b200q {

namespace tc {

constexpr int BM = 128;            // weight rows per tile (MMA M, tensor-memory lanes)
constexpr int BN = 128;            // tokens per tile (MMA N, tensor-memory columns per accumulator)
constexpr int KB = 32;             // weights per MMA (one quantization block)
constexpr int SB = 8;              // blocks per k-stage (256 weights)
constexpr int NACC = 4;            // accumulators in tensor memory (4 x 128 = 512 columns)
// One operand block (128 rows or columns x 32 k) is 4096 B as int8 and 8192 B as fp16; both are K-major
// core matrices (8 rows x 16 bytes) with the 16-byte K pieces LBO apart: two pieces per block as int8,
// four as fp16 (an fp16 MMA covers K = 16, so a block is two of them).
template <bool F16> struct Oper {
    enum { BYTES = BM * KB * (F16 ? 2 : 1),
           ACT_CHUNK = SB * BYTES + SB * BN * 4 };          // codes + f32 scales of a stage: 36864 / 69632 B
};
constexpr int NW = 2;              // scale-accumulate warps per tensor-memory lane quarter (4 measured no faster)
constexpr int THREADS = 32 * (8 + 4 * NW);   // warp groups: {producer, MMA, 2 idle}, unpack, NW x scale-accumulate
// Registers per thread by role (setmaxnreg). The launch gives every thread LAUNCH_REGS; a warp group that
// asks for more WAITS until others have given theirs back, so the sum must fit the launch's pool or the
// block never starts working.
constexpr int LAUNCH_REGS = (65536 / THREADS) / 8 * 8;
constexpr int REGS_CTRL = 64, REGS_UNPACK = 112, REGS_SCALE = 168;
static_assert(128 * REGS_CTRL + 128 * REGS_UNPACK + 128 * NW * REGS_SCALE <= THREADS * LAUNCH_REGS, "register pool");
static_assert(REGS_CTRL <= LAUNCH_REGS && REGS_UNPACK <= LAUNCH_REGS && REGS_SCALE >= LAUNCH_REGS, "dec / inc directions below");
#define B200Q_STR2(x) #x
#define B200Q_STR(x) B200Q_STR2(x)


template <int TYPE> struct Raw;     // packed bytes of one row per stage
template <> struct Raw<B200Q_TYPE_Q4_0> { enum { ROW = SB * 18, NSTAGE = 3, A_SLOTS_F16 = 4 }; };     // 144 B per row and stage
template <> struct Raw<B200Q_TYPE_Q8_0> { enum { ROW = SB * 34, NSTAGE = 2, A_SLOTS_F16 = 2 }; };     // 272 B: two stages fit
template <> struct Raw<B200Q_TYPE_IQ4_NL> { enum { ROW = SB * 18, NSTAGE = 3, A_SLOTS_F16 = 4 }; };   // Q4_0's block

template <int TYPE, bool F16> struct Smem {
    enum {
        NSTAGE = F16 ? 2 : Raw<TYPE>::NSTAGE,     // raw-weight / activation stages in flight
        A_SLOTS = F16 ? Raw<TYPE>::A_SLOTS_F16 : SB,      // unpacked A operand blocks in flight
        RAW_STAGE = BM * Raw<TYPE>::ROW,
        RAW_OFF = 0,
        ACT_OFF = RAW_OFF + NSTAGE * RAW_STAGE,
        A_OFF = ACT_OFF + NSTAGE * Oper<F16>::ACT_CHUNK,
        BAR_OFF = A_OFF + A_SLOTS * Oper<F16>::BYTES,
        TOTAL = BAR_OFF + 8 * 64             // room for up to 64 mbarriers (BAR_COUNT of them are used)
    };
};
static_assert(Smem<B200Q_TYPE_Q4_0, true>::TOTAL <= 227 * 1024 && Smem<B200Q_TYPE_Q8_0, true>::TOTAL <= 227 * 1024, "shared memory");

constexpr uint32_t IDESC_I8 = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
// fp16 operands, f32 accumulator: integer-valued halves (|v| <= 255) multiply and add exactly (every
// partial sum of a 32-block stays far below 2^24), so the accumulator holds float(I_b) with the bits the
// int8 MMA's result would convert to -- without the conversion
constexpr uint32_t IDESC_F16 = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

// barrier slots inside the shared block
enum { BAR_RAW_FULL = 0, BAR_RAW_EMPTY = 3, BAR_ACT_FULL = 6, BAR_ACT_EMPTY = 9, BAR_A_FULL = 12, BAR_A_EMPTY = 20,
       BAR_ACC_FULL = 28, BAR_ACC_EMPTY = 32, BAR_COUNT = 36 };
static_assert(BAR_COUNT <= 64, "the shared block reserves 64 mbarrier slots");

// Activation chunk (n-tile t, k-stage s) in global memory, written by quantize_tiled_kernel:
//   codes  [block j < 8][piece c][group g < 16][column r < 8][16 bytes]   column 8g + r; int8: two pieces of 16 k
//          (k = 32j + 16c + byte), fp16: four pieces of 8 k (k = 32j + 8c + half), the codes as exact halves
//   scales [block j < 8][column < 128] f32 (the fp16-rounded block scale)
template <bool F16>
__global__ void __launch_bounds__(256)
quantize_tiled_kernel(const uint8_t *base, int64_t ne1, int64_t ne2, size_t nb1, size_t nb2, size_t nb3, int64_t K,
                      int64_t N, uint8_t *__restrict__ out, TileRoute id) {
    // One block per (tile, k-stage of 256); a half-warp per column at a time: its sixteen lanes read the column's 256
    // floats as one contiguous kilobyte (lane l: k = 16 l .. 16 l + 15, i.e. half l & 1 of block j = l >> 1), the two
    // lanes of a block share their maximum by one shuffle, and every lane stores its 16 codes as one piece (int8) or
    // two (fp16). Columns past the tile's last one are written as zeros.
    const int t = blockIdx.y, s = blockIdx.x, nst = gridDim.x;
    const int hw = threadIdx.x >> 4, l = threadIdx.x & 15;
    constexpr int OPER_BYTES = Oper<F16>::BYTES, ACT_CHUNK = Oper<F16>::ACT_CHUNK;
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
    const int j = l >> 1;
#pragma unroll 1
    for (int col = hw; col < BN; col += 16) {
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
            x += (int64_t)s * (SB * KB) + 16 * l;
        }
        float v[16];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 f = x ? *reinterpret_cast<const float4 *>(x + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(f.x), fabsf(f.y)), fmaxf(fabsf(f.z), fabsf(f.w))));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
        const float d = __fdiv_rn(amax, 127.f);
        const float id = d != 0.f ? __fdiv_rn(1.f, d) : 0.f;
        uint8_t *o = chunk + j * OPER_BYTES + (col >> 3) * 128 + (col & 7) * 16;
        if (F16) {
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const __half2 h = __floats2half2_rn(roundf(__fmul_rn(v[2 * i], id)), roundf(__fmul_rn(v[2 * i + 1], id)));
                w[i] = *reinterpret_cast<const uint32_t *>(&h);
            }
            *reinterpret_cast<uint4 *>(o + (2 * (l & 1)) * LBO) = make_uint4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<uint4 *>(o + (2 * (l & 1) + 1) * LBO) = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t p = 0;
#pragma unroll
                for (int b = 0; b < 4; ++b) p |= (uint32_t)((int)roundf(__fmul_rn(v[4 * i + b], id)) & 0xFF) << (8 * b);
                w[i] = p;
            }
            *reinterpret_cast<uint4 *>(o + (l & 1) * LBO) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        if ((l & 1) == 0) reinterpret_cast<float *>(chunk + SB * OPER_BYTES)[j * BN + col] = __half2float(__float2half_rn(d));
    }
}

// dst[n][m] = sum over the K parts, part 0 first
__global__ void __launch_bounds__(256)
ksplit_sum_kernel(const float *__restrict__ parts, int ksplit, int64_t part_stride, int M, int64_t N, float *__restrict__ dst, int64_t ldd) {
    const int64_t total = N * M;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        float acc = parts[i];
        for (int z = 1; z < ksplit; ++z) acc += parts[(int64_t)z * part_stride + i];
        const int64_t n = i / M, m = i - n * M;
        dst[n * ldd + m] = acc;
    }
}

template <int N> __device__ __forceinline__ uint32_t word_at(const uint32_t (&w)[N], int byte_off) {
    // 32-bit word at a compile-time even byte offset of a register array
    const int i = byte_off >> 2, sh = (byte_off & 3) * 8;
    return sh == 0 ? w[i] : __funnelshift_r(w[i], w[i + 1], sh);
}

// four int8 bytes -> their values as exact fp16 halves: a byte b becomes the half 0x6400 | b = 1024 + b (byte
// permute with the constant 0x64), and one packed subtraction removes 1024 and the code's own offset
__device__ __forceinline__ void bytes_to_halves(uint32_t b4, uint32_t bias2, uint32_t &h01, uint32_t &h23) {
    const uint32_t a = __byte_perm(b4, 0x64646464u, 0x4140), b = __byte_perm(b4, 0x64646464u, 0x4342);
    const __half2 bias = *reinterpret_cast<const __half2 *>(&bias2);
    const __half2 ra = __hsub2(*reinterpret_cast<const __half2 *>(&a), bias), rb = __hsub2(*reinterpret_cast<const __half2 *>(&b), bias);
    h01 = *reinterpret_cast<const uint32_t *>(&ra);
    h23 = *reinterpret_cast<const uint32_t *>(&rb);
}

__device__ __forceinline__ void umma_f16_acc(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}

template <int TYPE, bool F16>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap wmap, int M, int K, const uint8_t *__restrict__ act,
               int N, float *__restrict__ dst, int64_t ldd, int64_t part_stride, int *__restrict__ error_word, TileRoute id) {
    typedef Smem<TYPE, F16> L;
    constexpr int ROWB = Raw<TYPE>::ROW;
    constexpr int NSTAGE = L::NSTAGE;
    constexpr int A_SLOTS = L::A_SLOTS;
    constexpr int OPER_BYTES = Oper<F16>::BYTES, ACT_CHUNK = Oper<F16>::ACT_CHUNK;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_n = blockIdx.x, tile_m = blockIdx.y;
    const int row0 = tile_m * BM;
    // gridDim.z > 1: the product is cut along K (few tiles on many SMs); this block takes nst of the K / 256
    // stages, from s_off, and writes its partial result to part blockIdx.z of a scratch buffer
    const int nst_all = K / (SB * KB);
    const int nst = nst_all / (int)gridDim.z;   // k-stages of this block
    const int s_off = (int)blockIdx.z * nst;
    const int nblk = nst * SB;
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bars = sbase + L::BAR_OFF;
    auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };
    const int valid_rows = min(BM, M - row0);
    // the tile's matrix and columns: dense, tile_n-th run of 128 tokens; MUL_MAT_ID, a route tile (one
    // expert, up to 128 routed pairs)
    int expert = 0, first = 0, ncols = min(BN, N - tile_n * BN);
    if (id.tiles) {
        if (tile_n >= __ldg(id.n_tiles)) return;          // the whole block: nothing is set up yet
        expert = __ldg(id.tiles + 4 * tile_n);
        first = __ldg(id.tiles + 4 * tile_n + 1);
        ncols = __ldg(id.tiles + 4 * tile_n + 2);
    }

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int i = 0; i < NSTAGE; ++i) {
            mbar_init(bar(BAR_RAW_FULL + i), 1);
            mbar_init(bar(BAR_RAW_EMPTY + i), 4 + 4 * NW);      // unpack warps + scaling warps (block scales)
            mbar_init(bar(BAR_ACT_FULL + i), 1);
            mbar_init(bar(BAR_ACT_EMPTY + i), 1 + 4 * NW);     // MMA commit + every scaling warp
        }
        for (int i = 0; i < A_SLOTS; ++i) {
            mbar_init(bar(BAR_A_FULL + i), 4);                  // unpack warps
            mbar_init(bar(BAR_A_EMPTY + i), 1);
        }
        for (int i = 0; i < NACC; ++i) {
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

    // Register budget by role (the launch gives every thread 65536/THREADS registers): each
    // branch below starts by resizing its warp group's share -- the first two groups hand most
    // of theirs back, the scale-accumulate groups take them.
    if (warp == 0) {
        // ---- producer ----
        asm volatile("setmaxnreg.dec.sync.aligned.u32 " B200Q_STR(64) ";" ::: "memory");   // REGS_CTRL
        const uint8_t *act_tile = act + ((size_t)tile_n * nst_all + s_off) * ACT_CHUNK;
        if (lane == 0) tma_prefetch_desc(&wmap);
        for (int s = 0; s < nst; ++s) {
            const int st = s % NSTAGE;
            const uint32_t par = ((s / NSTAGE) & 1) ^ 1;        // first pass over the ring: slots are free
            if (!WAITP(1, bar(BAR_RAW_EMPTY + st), par)) break;
            if (lane == 0) {
                // the stage's [128 rows x ROWB] box in one tiled copy; rows past M arrive as zeros
                mbar_expect_tx(bar(BAR_RAW_FULL + st), L::RAW_STAGE);
                tma_load_3d(sbase + L::RAW_OFF + st * L::RAW_STAGE, &wmap, (s_off + s) * (ROWB / 4), row0, expert, bar(BAR_RAW_FULL + st));
            }
            if (!WAITP(3, bar(BAR_ACT_EMPTY + st), par)) break;
            if (lane == 0) {
                mbar_expect_tx(bar(BAR_ACT_FULL + st), ACT_CHUNK);
                bulk_g2s(sbase + L::ACT_OFF + st * ACT_CHUNK, act_tile + (size_t)s * ACT_CHUNK, ACT_CHUNK,
                         bar(BAR_ACT_FULL + st));
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        asm volatile("setmaxnreg.dec.sync.aligned.u32 " B200Q_STR(64) ";" ::: "memory");   // REGS_CTRL
        for (int b = 0; b < nblk; ++b) {
            const int s = b / SB, j = b % SB, st = s % NSTAGE, acc = b % NACC, slot = b % A_SLOTS;
            if (j == 0 && !WAITP(2, bar(BAR_ACT_FULL + st), (s / NSTAGE) & 1)) break;
            if (!WAITP(4, bar(BAR_A_FULL + slot), (b / A_SLOTS) & 1)) break;
            if (!WAITP(7, bar(BAR_ACC_EMPTY + acc), ((b / NACC) & 1) ^ 1)) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t a_addr = sbase + L::A_OFF + slot * OPER_BYTES, b_addr = sbase + L::ACT_OFF + st * ACT_CHUNK + j * OPER_BYTES;
                if (F16) {
                    // K = 16 per fp16 MMA: the block's first two 16-byte K pieces, then the other two
                    umma_f16_acc(tmem_base + (uint32_t)acc * BN, umma_desc(a_addr), umma_desc(b_addr), IDESC_F16, 0u);
                    umma_f16_acc(tmem_base + (uint32_t)acc * BN, umma_desc(a_addr + 2 * LBO), umma_desc(b_addr + 2 * LBO), IDESC_F16, 1u);
                } else {
                    umma_i8(tmem_base + (uint32_t)acc * BN, umma_desc(a_addr), umma_desc(b_addr), IDESC_I8);
                }
                tc_commit(bar(BAR_ACC_FULL + acc));
                tc_commit(bar(BAR_A_EMPTY + slot));
                if (j == SB - 1) tc_commit(bar(BAR_ACT_EMPTY + st));
            }
            __syncwarp();
        }
    } else if (warp < 4) {
        // idle warps of the first warp group
        asm volatile("setmaxnreg.dec.sync.aligned.u32 " B200Q_STR(64) ";" ::: "memory");   // REGS_CTRL
    } else if (warp < 8) {
        // ---- unpack: one thread per weight row ----
        asm volatile("setmaxnreg.dec.sync.aligned.u32 " B200Q_STR(112) ";" ::: "memory");  // REGS_UNPACK
        const int r = (warp - 4) * 32 + lane;
        const bool row_ok = r < valid_rows;
        bool ok = true;
        for (int s = 0; s < nst && ok; ++s) {
            const int st = s % NSTAGE;
            if (!WAITP(0, bar(BAR_RAW_FULL + st), (s / NSTAGE) & 1)) break;
            uint32_t rw[ROWB / 4 + 1];                     // the row's packed bytes of this stage
            const uint4 *rp = reinterpret_cast<const uint4 *>(smem + L::RAW_OFF + st * L::RAW_STAGE + r * ROWB);
#pragma unroll
            for (int i = 0; i < ROWB / 16; ++i) {
                const uint4 t = row_ok ? rp[i] : make_uint4(0, 0, 0, 0);
                rw[4 * i] = t.x; rw[4 * i + 1] = t.y; rw[4 * i + 2] = t.z; rw[4 * i + 3] = t.w;
            }
            rw[ROWB / 4] = 0;
            mbar_arrive_warp(bar(BAR_RAW_EMPTY + st), lane);
#pragma unroll
            for (int j = 0; j < SB; ++j) {
                const int b = s * SB + j, slot = b % A_SLOTS;
                if (!WAITP(5, bar(BAR_A_EMPTY + slot), ((b / A_SLOTS) & 1) ^ 1)) { ok = false; break; }
                constexpr int BB = TYPE == B200Q_TYPE_Q8_0 ? 34 : 18;
                uint8_t *a = smem + L::A_OFF + slot * OPER_BYTES + (r >> 3) * 128 + (r & 7) * 16;
                if (F16) {
                    // the block's 32 weights as exact fp16 integers, four pieces of eight
                    uint32_t h[16];
                    if (TYPE == B200Q_TYPE_Q4_0) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const uint32_t q = word_at(rw, BB * j + 2 + 4 * i);
                            bytes_to_halves(q & 0x0F0F0F0Fu, 0x64086408u, h[2 * i], h[2 * i + 1]);               // 1024 + n - 1032
                            bytes_to_halves((q >> 4) & 0x0F0F0F0Fu, 0x64086408u, h[8 + 2 * i], h[8 + 2 * i + 1]);
                        }
                    } else if (TYPE == B200Q_TYPE_IQ4_NL) {
                        // the nibbles index kvalues_iq4nl (signed bytes, |v| <= 127: exact halves), then as for Q8_0
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const uint32_t q = word_at(rw, BB * j + 2 + 4 * i);
                            bytes_to_halves(iq4nl_lookup4(q & 0x0F0F0F0Fu) ^ 0x80808080u, 0x64806480u, h[2 * i], h[2 * i + 1]);
                            bytes_to_halves(iq4nl_lookup4((q >> 4) & 0x0F0F0F0Fu) ^ 0x80808080u, 0x64806480u, h[8 + 2 * i], h[8 + 2 * i + 1]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i)                                                               // 1024 + (q + 128) - 1152
                            bytes_to_halves(word_at(rw, BB * j + 2 + 4 * i) ^ 0x80808080u, 0x64806480u, h[2 * i], h[2 * i + 1]);
                    }
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        *reinterpret_cast<uint4 *>(a + c * LBO) = make_uint4(h[4 * c], h[4 * c + 1], h[4 * c + 2], h[4 * c + 3]);
                    fence_async_smem();
                    mbar_arrive_warp(bar(BAR_A_FULL + slot), lane);
                    continue;
                }
                uint32_t lo[4], hi[4];
                if (TYPE == B200Q_TYPE_Q4_0) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t q = word_at(rw, BB * j + 2 + 4 * i);
                        lo[i] = nib_minus8(q & 0x0F0F0F0Fu);           // weights 4i..4i+3
                        hi[i] = nib_minus8((q >> 4) & 0x0F0F0F0Fu);    // weights 16+4i..
                    }
                } else if (TYPE == B200Q_TYPE_IQ4_NL) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t q = word_at(rw, BB * j + 2 + 4 * i);
                        lo[i] = iq4nl_lookup4(q & 0x0F0F0F0Fu);
                        hi[i] = iq4nl_lookup4((q >> 4) & 0x0F0F0F0Fu);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        lo[i] = word_at(rw, BB * j + 2 + 4 * i);
                        hi[i] = word_at(rw, BB * j + 18 + 4 * i);
                    }
                }
                *reinterpret_cast<uint4 *>(a) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                *reinterpret_cast<uint4 *>(a + LBO) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                fence_async_smem();
                mbar_arrive_warp(bar(BAR_A_FULL + slot), lane);
            }
        }
    } else {
        // ---- scale-accumulate: NW warps per tensor-memory lane quarter, BN/NW columns each ----
        asm volatile("setmaxnreg.inc.sync.aligned.u32 " B200Q_STR(168) ";" ::: "memory");  // REGS_SCALE
        constexpr int CW = BN / NW;                        // columns per thread
        const int q4 = warp & 3, u = (warp - 8) >> 2;      // lane quarter (fixed by warp id % 4), column part
        const int r = q4 * 32 + lane;
        const bool row_ok = r < valid_rows;
        f32x2 acc2[CW / 2];                                // column pairs
#pragma unroll
        for (int c = 0; c < CW / 2; ++c) acc2[c] = 0ull;
        bool done = false;                                 // every block was accumulated (no wait gave up)
        for (int b = 0; b < nblk; ++b) {
            const int s = b / SB, j = b % SB, st = s % NSTAGE, acc = b % NACC;
            // A waiter on an mbarrier phase must see it before the phase after it completes:
            // both stage barriers below cannot advance until this thread has released the stage.
            if (j == 0 && !WAITP(2, bar(BAR_ACT_FULL + st), (s / NSTAGE) & 1)) break;
            if (j == 0 && !WAITP(0, bar(BAR_RAW_FULL + st), (s / NSTAGE) & 1)) break;
            if (!WAITP(6, bar(BAR_ACC_FULL + acc), (b / NACC) & 1)) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q4 * 32) << 16) + (uint32_t)acc * BN + (uint32_t)u * CW;
            // the block's fp16 weight scale, straight from the packed row in the raw stage
            constexpr int BB = TYPE == B200Q_TYPE_Q8_0 ? 34 : 18;
            const float dwb = row_ok ? half_bits_to_float(*reinterpret_cast<const uint16_t *>(
                                           smem + L::RAW_OFF + st * L::RAW_STAGE + r * ROWB + BB * j)) : 0.f;
            const f32x2 dw2 = f2_pack(dwb, dwb), negc2 = f2_pack(-12582912.f, -12582912.f);
            const uint32_t dxa = sbase + L::ACT_OFF + st * ACT_CHUNK + SB * OPER_BYTES + (j * BN + u * CW) * 4;
            // the whole accumulator slice in one go: the CW/16 tensor-memory loads are issued back to back and
            // waited for once (one load latency per block, not one per sixteen columns), then the accumulator
            // is free for the MMA three blocks ahead while these registers are scaled
            uint32_t v[CW / 16][16];
#pragma unroll
            for (int q = 0; q < CW / 16; ++q) tmem_ld16(taddr + q * 16, v[q]);
            tmem_ld_wait();
            tc_fence_before();
            mbar_arrive_warp(bar(BAR_ACC_EMPTY + acc), lane);
#pragma unroll
            for (int q = 0; q < CW / 16; ++q) {
                f32x2 dx[8];
#pragma unroll
                for (int c = 0; c < 4; ++c) lds128_f2(dxa + (q * 16 + 4 * c) * 4, dx[2 * c], dx[2 * c + 1]);
#pragma unroll
                for (int c = 0; c < 16; c += 4) {
                    const int e = (q * 16 + c) / 2;
                    // int8 arm: exact int -> float without the conversion pipe (|I| < 2^22): add the magic
                    // exponent as an integer, subtract it as a float; the fp16 arm's accumulator already holds floats
                    const f32x2 x01 = F16 ? f2_pack(__uint_as_float(v[q][c]), __uint_as_float(v[q][c + 1]))
                                          : f2_add(f2_pack(__int_as_float((int)v[q][c] + 0x4B400000),
                                                           __int_as_float((int)v[q][c + 1] + 0x4B400000)), negc2);
                    const f32x2 x23 = F16 ? f2_pack(__uint_as_float(v[q][c + 2]), __uint_as_float(v[q][c + 3]))
                                          : f2_add(f2_pack(__int_as_float((int)v[q][c + 2] + 0x4B400000),
                                                           __int_as_float((int)v[q][c + 3] + 0x4B400000)), negc2);
                    acc2[e]     = f2_fma(x01, f2_mul(dw2, dx[c / 2]), acc2[e]);
                    acc2[e + 1] = f2_fma(x23, f2_mul(dw2, dx[c / 2 + 1]), acc2[e + 1]);
                }
            }
            if (j == SB - 1) {                                         // done with this stage's scales
                mbar_arrive_warp(bar(BAR_ACT_EMPTY + st), lane);
                mbar_arrive_warp(bar(BAR_RAW_EMPTY + st), lane);
            }
            done = b == nblk - 1;
        }
        const int ncol = ncols - u * CW;                         // this thread's columns inside the tile
        if (done && id.tiles) {
            // where the warp's columns go: every lane looks up some of them (loads in flight together), the
            // store loop takes them by shuffle
            long long off[(CW + 31) / 32];
#pragma unroll
            for (int h = 0; h < (CW + 31) / 32; ++h) {
                off[h] = 0;
                if (lane + 32 * h < ncol) {
                    const int p = __ldg(id.pairs + first + u * CW + lane + 32 * h), tok = p / id.n_used, slot = p - tok * id.n_used;
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
                    if (row_ok && c + d < ncol) dst[o + row0 + r] = a[d];
                }
            }
        } else if (done && row_ok) {
            float *o = dst + (int64_t)blockIdx.z * part_stride + (int64_t)(tile_n * BN + u * CW) * ldd + row0 + r;
#pragma unroll
            for (int c = 0; c < CW; c += 2) {
                float a0, a1;
                f2_unpack(acc2[c / 2], a0, a1);
                // (with the product cut along K, dst is this K part's own [N][ldd] scratch: plain stores, added up
                // afterwards in a fixed order)
                if (c < ncol) *o = a0;
                if (c + 1 < ncol) o[ldd] = a1;
                o += 2 * ldd;
            }
        }
    }

    PROF_DUMP(warp == 0 ? "prod" : warp == 1 ? "mma " : warp < 4 ? "idle" : warp < 8 ? "unpk" : "epi ")
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        // a wait ran out: give copies still in flight time to land before the block's shared
        // memory is released, and tell the host
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        if (threadIdx.x == 0) atomicExch(error_word, 1);
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

}  // namespace tc

// sized for the larger (fp16) form, so one scratch serves either arm
size_t gemm_tc_act_bytes(int64_t K, int64_t N) {
    const int64_t ntile = (N + tc::BN - 1) / tc::BN, nst = K / (tc::SB * tc::KB);
    return (size_t)(ntile * nst) * tc::Oper<true>::ACT_CHUNK;
}

bool gemm_tc_supported(int type, int64_t M, int64_t K, int64_t N, const void *w, size_t row_stride) {
    if (type != B200Q_TYPE_Q4_0 && type != B200Q_TYPE_Q8_0 && type != B200Q_TYPE_IQ4_NL) return false;
    if (K % (tc::SB * tc::KB) || K <= 0 || M <= 0 || N <= 0) return false;
    if ((uintptr_t)w % 16 || row_stride % 16) return false;          // bulk copies of row pieces
    if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return false;
    return true;
}

static const TileRoute NO_ROUTE_TC = { nullptr, nullptr, nullptr, 1, 1, 0, 0, 0, 0 };

static b200q_status quantize_tiled(b200q_ctx *ctx, const b200q_tensor *src1, uint8_t *out, int64_t n_tiles, const TileRoute &tr) {
    const int64_t K = src1->ne[0], N = src1->ne[1] * src1->ne[2] * src1->ne[3];
    dim3 grid((unsigned)(K / (tc::SB * tc::KB)), (unsigned)n_tiles);
    if (ctx->tc_f16)
        tc::quantize_tiled_kernel<true><<<grid, 256, 0, ctx->stream>>>((const uint8_t *)src1->data, src1->ne[1], src1->ne[2],
                                                                      src1->nb[1], src1->nb[2], src1->nb[3], K, N, out, tr);
    else
        tc::quantize_tiled_kernel<false><<<grid, 256, 0, ctx->stream>>>((const uint8_t *)src1->data, src1->ne[1], src1->ne[2],
                                                                       src1->nb[1], src1->nb[2], src1->nb[3], K, N, out, tr);
    B200Q_CUDA(ctx, cudaGetLastError());
    count(ctx, ST_GEMM_TC_QUANT);
    return B200Q_OK;
}

b200q_status launch_quantize_tiled(b200q_ctx *ctx, const b200q_tensor *src1, uint8_t *out) {
    const int64_t N = src1->ne[1] * src1->ne[2] * src1->ne[3];
    return quantize_tiled(ctx, src1, out, (N + tc::BN - 1) / tc::BN, NO_ROUTE_TC);
}

// n_tiles: grid width (dense: the tiles of N; MUL_MAT_ID: the upper bound of the route's tile count,
// blocks past the device-side count leave at once)
template <int TYPE, bool F16>
static b200q_status launch_tf(b200q_ctx *ctx, const void *w, size_t row_stride, size_t mat_stride, int64_t n_mat, int64_t M,
                              int64_t K, const uint8_t *act, int64_t N, int64_t n_tiles, float *dst, int64_t ldd,
                              const TileRoute &tr) {
    typedef tc::Smem<TYPE, F16> L;
    auto kern = tc::gemm_tc_kernel<TYPE, F16>;
    static bool attr_set_dev[B200Q_MAX_DEVICES] = {};
    bool &attr_set = attr_set_dev[ctx->device % B200Q_MAX_DEVICES];
    if (!attr_set) {
        B200Q_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L::TOTAL));
        attr_set = true;
    }
    CUtensorMap wmap;
    constexpr int BB = TYPE == B200Q_TYPE_Q8_0 ? 34 : 18;
    b200q_status st = make_weight_tmap3(ctx, &wmap, w, row_stride, M, (K / 32) * BB, tc::Raw<TYPE>::ROW, n_mat, mat_stride);
    if (st != B200Q_OK) return st;
    // Cut K into 2, 4 or 8 parts when the tiles alone leave SMs idle (a 512-row shard of a tensor-parallel product is
    // 16 tiles on 148 SMs and every tile walks all of K): the schedule's length is rounds of blocks x stages per
    // block. Parts write their own scratch and a second kernel adds them in a fixed order, so the result does not
    // depend on which block finishes first.
    const int64_t units = n_tiles * ((M + tc::BM - 1) / tc::BM), S = ctx->sm_count, nst = K / 256;
    unsigned ksplit = 1;
    if (!tr.tiles && !ctx->no_ksplit) {
        // in stages: a block costs about three stages' time beyond its K walk (set-up, drain, stores), the adding pass one
        constexpr int64_t FIXED = 3;
        int64_t best = ((units + S - 1) / S) * (nst + FIXED);
        for (unsigned ks = 2; ks <= 8; ks *= 2) {
            if (nst % ks || nst / ks < 2) break;
            const int64_t len = ((units * ks + S - 1) / S) * (nst / ks + FIXED) + 1;
            if (len < best) { best = len; ksplit = ks; }
        }
    }
    float *out = dst;
    int64_t out_ld = ldd, part_stride = 0;
    if (ksplit > 1) {
        part_stride = N * M;
        if ((st = ws_reserve(ctx, &ctx->moe_ws[9], sizeof(float) * (size_t)part_stride * ksplit)) != B200Q_OK) return st;
        out = (float *)ctx->moe_ws[9].ptr;
        out_ld = M;
    }
    dim3 grid((unsigned)n_tiles, (unsigned)((M + tc::BM - 1) / tc::BM), ksplit);
    kern<<<grid, tc::THREADS, L::TOTAL, ctx->stream>>>(wmap, (int)M, (int)K, act, (int)N, out, out_ld, part_stride, ctx->error_word, tr);
    B200Q_CUDA(ctx, cudaGetLastError());
    if (ksplit > 1) {
        const int64_t total = N * M;
        int64_t blocks = (total + 255) / 256;
        if (blocks > (int64_t)S * 8) blocks = (int64_t)S * 8;
        tc::ksplit_sum_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(out, (int)ksplit, part_stride, (int)M, N, dst, ldd);
        B200Q_CUDA(ctx, cudaGetLastError());
        count(ctx, ST_GEMM_KSPLIT);
    }
    count(ctx, ST_GEMM_TC);
    if (F16) count(ctx, ST_GEMM_TC_F16);
    return B200Q_OK;
}

// The arm: fp16 operands (integer-valued, exact) by default; B200Q_TC_I8=1 keeps the int8 MMA. Both give the
// same block dots bit for bit; the fp16 arm's accumulator needs no int -> float conversion.
template <int TYPE>
static b200q_status launch_t(b200q_ctx *ctx, const void *w, size_t row_stride, size_t mat_stride, int64_t n_mat, int64_t M,
                             int64_t K, const uint8_t *act, int64_t N, int64_t n_tiles, float *dst, int64_t ldd,
                             const TileRoute &tr) {
    return ctx->tc_f16 ? launch_tf<TYPE, true>(ctx, w, row_stride, mat_stride, n_mat, M, K, act, N, n_tiles, dst, ldd, tr)
                       : launch_tf<TYPE, false>(ctx, w, row_stride, mat_stride, n_mat, M, K, act, N, n_tiles, dst, ldd, tr);
}

b200q_status launch_gemm_tc(b200q_ctx *ctx, int type, const void *w, size_t row_stride, int64_t M, int64_t K,
                            const uint8_t *act, int64_t N, float *dst, int64_t ldd) {
    const int64_t n_tiles = (N + tc::BN - 1) / tc::BN;
    const size_t ms = row_stride * (size_t)M;
    if (type == B200Q_TYPE_Q4_0) return launch_t<B200Q_TYPE_Q4_0>(ctx, w, row_stride, ms, 1, M, K, act, N, n_tiles, dst, ldd, NO_ROUTE_TC);
    if (type == B200Q_TYPE_Q8_0) return launch_t<B200Q_TYPE_Q8_0>(ctx, w, row_stride, ms, 1, M, K, act, N, n_tiles, dst, ldd, NO_ROUTE_TC);
    if (type == B200Q_TYPE_IQ4_NL) return launch_t<B200Q_TYPE_IQ4_NL>(ctx, w, row_stride, ms, 1, M, K, act, N, n_tiles, dst, ldd, NO_ROUTE_TC);
    return fail(ctx, B200Q_UNSUPPORTED, "gemm_tc: type %d", type);
}

size_t gemm_tc_id_act_bytes(int64_t K, int64_t max_tiles) { return gemm_tc_act_bytes(K, max_tiles * tc::BN); }

// MUL_MAT_ID on the tensor cores: the route's 128-pair tiles are the column tiles; the activation of
// every tile is gathered and quantized into `act` (gemm_tc_id_act_bytes) first.
b200q_status launch_gemm_tc_id(b200q_ctx *ctx, const b200q_tensor *src0, const b200q_tensor *src1, const TileRoute &tr,
                               int64_t max_tiles, uint8_t *act, float *dst, bool act_ready) {
    const int64_t K = src0->ne[0], M = src0->ne[1];
    b200q_status st = act_ready ? B200Q_OK : quantize_tiled(ctx, src1, act, max_tiles, tr);
    if (st != B200Q_OK) return st;
    if (src0->type == B200Q_TYPE_Q4_0)
        return launch_t<B200Q_TYPE_Q4_0>(ctx, src0->data, src0->nb[1], src0->nb[2], src0->ne[2], M, K, act, 0, max_tiles, dst, 0, tr);
    if (src0->type == B200Q_TYPE_Q8_0)
        return launch_t<B200Q_TYPE_Q8_0>(ctx, src0->data, src0->nb[1], src0->nb[2], src0->ne[2], M, K, act, 0, max_tiles, dst, 0, tr);
    if (src0->type == B200Q_TYPE_IQ4_NL)
        return launch_t<B200Q_TYPE_IQ4_NL>(ctx, src0->data, src0->nb[1], src0->nb[2], src0->ne[2], M, K, act, 0, max_tiles, dst, 0, tr);
    return fail(ctx, B200Q_UNSUPPORTED, "gemm_tc_id: type %d", src0->type);
}

}  // namespace b200q
