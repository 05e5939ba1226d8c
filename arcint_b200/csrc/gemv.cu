// gemv.cu -- decode GEMV for 1..8 activation columns: dst[:, c] = W x_c.
//
// HBM-bound (every packed weight byte is read once for all columns), CUDA cores only:
// each warp streams R rows through a private ring of shared-memory stages filled with
// 16-byte asynchronous copies (coalesced 128-bit reads of the packed GGUF blocks, several
// stages in flight per warp), every lane decodes 32 weights of a stage and runs dp4a
// against the int8 activation codes it holds in registers for all columns, and the warp
// reduces with shuffles. No tensor cores. Rows whose byte length or address is not a
// multiple of 16 take the same kernel with a plain 2-byte copy loop as the loader.
//
// Stands in for the reference's kernel_mul_mv_*_q8_1 family
// (marfrit/arcint contrib/llama.cpp/patches/0000-01-kquant-integer-dpas.patch:3882-3915,
// host side ggml_cl_mul_mv_kq_q8_1 at :817-857).
#include "gemv_core.cuh"
#include "common.cuh"

#include <limits.h>

namespace b200q {

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

template <int TYPE, int NC, int R, int WARPS, int STAGES, bool ALIGNED>
__global__ void __launch_bounds__(WARPS * 32)
gemv_kernel(const uint8_t *__restrict__ W, size_t row_stride, int M, int nblk, GemvAct act,
            float *__restrict__ dst, int ldd) {
    typedef GemvFmt<TYPE> F;
    typedef GemvStage<TYPE> S;
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t *ring = smem + warp * (STAGES * R * S::SLOT);

    const int row_bytes = nblk * F::BLK_B;
    const int nstages = (nblk + F::STAGE_BLOCKS - 1) / F::STAGE_BLOCKS;
    const int n_rg = (M + R - 1) / R;
    const int gw = blockIdx.x * WARPS + warp, tw = gridDim.x * WARPS;

    // producer cursor: (row group, stage) of the next chunk to fetch, and its ring slot
    int p_rg = gw, p_s = 0, p_slot = 0;
    auto issue = [&]() {
        if (p_rg < n_rg) {
            const int off = p_s * S::BYTES;
            const int bytes = min((int)S::BYTES, row_bytes - off);
            uint8_t *slot = ring + p_slot * (R * S::SLOT);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int row = min(p_rg * R + r, M - 1);       // ragged tail: re-read the last row
                const uint8_t *src = W + (size_t)row * row_stride + off;
                uint8_t *d = slot + r * S::SLOT;
                if (ALIGNED) {
                    for (int b = lane * 16; b < bytes; b += 32 * 16) cp_async16(d + b, src + b);
                } else {
                    for (int b = lane * 2; b < bytes; b += 32 * 2)
                        *reinterpret_cast<uint16_t *>(d + b) = *reinterpret_cast<const uint16_t *>(src + b);
                }
            }
            if (++p_s == nstages) { p_s = 0; p_rg += tw; }
        }
        p_slot = p_slot + 1 == STAGES ? 0 : p_slot + 1;
        cp_async_commit();
    };

    float acc[R][NC];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int c = 0; c < NC; ++c) acc[r][c] = 0.f;

#pragma unroll
    for (int i = 0; i < STAGES - 1; ++i) issue();
    int c_slot = 0;
    for (int rg = gw; rg < n_rg; rg += tw) {
        for (int s = 0; s < nstages; ++s) {
            issue();
            cp_async_wait<STAGES - 1>();
            __syncwarp();
            const uint8_t *slot = ring + c_slot * (R * S::SLOT);
            const uint32_t *srow[R];
#pragma unroll
            for (int r = 0; r < R; ++r) srow[r] = reinterpret_cast<const uint32_t *>(slot + r * S::SLOT);
            gemv_lane_stage<TYPE, NC, R>(srow, lane, s, nblk, act, acc);
            c_slot = c_slot + 1 == STAGES ? 0 : c_slot + 1;
            __syncwarp();
        }
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                float v = acc[r][c];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
                if (lane == 0 && rg * R + r < M) dst[(size_t)c * ldd + rg * R + r] = v;
                acc[r][c] = 0.f;
            }
    }
    cp_async_wait<0>();
}

template <int TYPE, int NC, int R, int WARPS, int STAGES>
static b200q_status launch_one(b200q_ctx *ctx, const void *w, size_t row_stride, int64_t M, int64_t K,
                               const GemvAct &act, float *dst, int64_t ldd, bool aligned) {
    typedef GemvStage<TYPE> S;
    const size_t smem = (size_t)WARPS * STAGES * R * S::SLOT;
    if (M > INT32_MAX / 2 || K / GemvFmt<TYPE>::BLK_W > INT32_MAX / 256 || ldd > INT32_MAX)
        return fail(ctx, B200Q_UNSUPPORTED, "gemv: dimensions beyond 32-bit indexing");
    const int64_t n_rg = (M + R - 1) / R;
    int64_t blocks = (n_rg + WARPS - 1) / WARPS;
    const int64_t cap = (int64_t)ctx->sm_count * 16;     // enough CTAs to fill every SM several times over
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    auto kern_a = gemv_kernel<TYPE, NC, R, WARPS, STAGES, true>;
    auto kern_u = gemv_kernel<TYPE, NC, R, WARPS, STAGES, false>;
    auto kern = aligned ? kern_a : kern_u;
    if (smem > 48 * 1024)
        B200Q_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<(unsigned)blocks, WARPS * 32, smem, ctx->stream>>>((const uint8_t *)w, row_stride, (int)M,
                                                              (int)(K / GemvFmt<TYPE>::BLK_W), act, dst, (int)ldd);
    B200Q_CUDA(ctx, cudaGetLastError());
    return B200Q_OK;
}

template <int TYPE, int NC>
static b200q_status launch_nc(b200q_ctx *ctx, const void *w, size_t row_stride, int64_t M, int64_t K,
                              const GemvAct &act, float *dst, int64_t ldd, bool aligned) {
    // rows per warp pass: two while the activation registers allow it
    return launch_one<TYPE, NC, (NC <= 4 ? 2 : 1), 4, 3>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
}

template <int TYPE>
static b200q_status launch_type(b200q_ctx *ctx, const void *w, size_t row_stride, int64_t M, int64_t K,
                                const GemvAct &act, int nc, float *dst, int64_t ldd, bool aligned) {
    switch (nc) {
    case 1: return launch_nc<TYPE, 1>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
    case 2: return launch_nc<TYPE, 2>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
    case 3: return launch_nc<TYPE, 3>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
    case 4: return launch_nc<TYPE, 4>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
    case 5: return launch_nc<TYPE, 5>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
    case 6: return launch_nc<TYPE, 6>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
    case 7: return launch_nc<TYPE, 7>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
    case 8: return launch_nc<TYPE, 8>(ctx, w, row_stride, M, K, act, dst, ldd, aligned);
    }
    return fail(ctx, B200Q_INVALID, "gemv: %d columns", nc);
}

b200q_status launch_gemv(b200q_ctx *ctx, int type, const void *w, size_t row_stride, int64_t M, int64_t K,
                         const ActView &av, int64_t col0, int ncols, float *dst, int64_t ldd) {
    GemvAct act;
    act.q = av.codes + col0 * K;
    act.d16 = av.d16 ? av.d16 + col0 * (K / 32) : nullptr;
    act.d32 = av.d32 ? av.d32 + col0 * (K / 256) : nullptr;
    act.s32 = av.s32 ? av.s32 + col0 * (K / 32) : nullptr;
    act.s16 = av.s16 ? av.s16 + col0 * (K / 16) : nullptr;
    act.K = (int)K;
    TypeInfo ti;
    if (!type_info(type, &ti)) return fail(ctx, B200Q_UNSUPPORTED, "gemv: type %d", type);
    const size_t row_bytes = (size_t)(K / ti.block) * ti.bytes;
    const bool aligned = ((uintptr_t)w % 16 == 0) && (row_stride % 16 == 0) && (row_bytes % 16 == 0);
    count(ctx, (aligned ? ST_GEMV_COL0 : ST_GEMV_UNALIGNED_COL0) + ncols);
    switch (type) {
    case B200Q_TYPE_Q4_0:   return launch_type<B200Q_TYPE_Q4_0>(ctx, w, row_stride, M, K, act, ncols, dst, ldd, aligned);
    case B200Q_TYPE_Q8_0:   return launch_type<B200Q_TYPE_Q8_0>(ctx, w, row_stride, M, K, act, ncols, dst, ldd, aligned);
    case B200Q_TYPE_Q4_K:   return launch_type<B200Q_TYPE_Q4_K>(ctx, w, row_stride, M, K, act, ncols, dst, ldd, aligned);
    case B200Q_TYPE_Q6_K:   return launch_type<B200Q_TYPE_Q6_K>(ctx, w, row_stride, M, K, act, ncols, dst, ldd, aligned);
    case B200Q_TYPE_IQ4_XS: return launch_type<B200Q_TYPE_IQ4_XS>(ctx, w, row_stride, M, K, act, ncols, dst, ldd, aligned);
    }
    return fail(ctx, B200Q_UNSUPPORTED, "gemv: type %d", type);
}

}  // namespace b200q
