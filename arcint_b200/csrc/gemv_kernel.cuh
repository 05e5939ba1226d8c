// gemv_kernel.cuh -- the decode GEMV kernel template (see gemv.cu for the description).
#pragma once

#include "gemv_core.cuh"

namespace b200q {

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// One warp owns a batch of B consecutive rows at a time and walks the row in stages of 2048
// weights. For each stage it holds the activation side (64 codes per lane and column, scales,
// block sums) in registers and runs the B staged row chunks against it, so the activation
// loads, address arithmetic and pipeline bookkeeping are paid once per B rows. The chunks
// arrive through a per-warp ring of NSETS sets of B slots filled with 16-byte asynchronous
// copies: NSETS-1 sets are in flight while the current one is consumed. More
// than four columns are taken as two column groups over the same staged set.
template <int TYPE, int NC, int B, int WARPS, int NSETS, bool ALIGNED>
__global__ void __launch_bounds__(WARPS * 32)
gemv_kernel(const uint8_t *__restrict__ W, size_t row_stride, int M, int nblk, GemvAct act,
            float *__restrict__ dst, int ldd) {
    typedef GemvFmt<TYPE> F;
    typedef GemvStage<TYPE> S;
    constexpr int NCG = NC <= 4 ? NC : (NC + 1) / 2;      // columns of the first group
    constexpr int NC2 = NC - NCG;                         // columns of the second group (0: none)
    constexpr int PIECES = (S::BYTES + 511) / 512;        // 16-byte copies per lane and chunk
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t *ring = smem + warp * (NSETS * B * S::SLOT);

    const int row_bytes = nblk * F::BLK_B;
    const int nstages = (nblk + F::STAGE_BLOCKS - 1) / F::STAGE_BLOCKS;
    const int n_bt = (M + B - 1) / B;
    const int gw = blockIdx.x * WARPS + warp, tw = gridDim.x * WARPS;

    // producer cursor: batch and stage of the next set to fetch, and which half of the ring
    int p_bt = gw, p_s = 0, p_set = 0;
    auto issue = [&]() {
        if (p_bt < n_bt) {
            const int off = p_s * S::BYTES;
            const int bytes = min((int)S::BYTES, row_bytes - off);
            const int row0 = p_bt * B;
            const uint8_t *src = W + (size_t)row0 * row_stride + off;
            uint8_t *d = ring + p_set * (B * S::SLOT);
#pragma unroll
            for (int r = 0; r < B; ++r) {
                if (row0 + r < M) {              // rows past the end keep stale bytes; never stored
                    if (ALIGNED) {
#pragma unroll
                        for (int j = 0; j < PIECES; ++j) {
                            const int b = lane * 16 + j * 512;
                            if (b < bytes) cp_async16(d + b, src + b);
                        }
                    } else {
                        for (int b = lane * 2; b < bytes; b += 64)
                            *reinterpret_cast<uint16_t *>(d + b) = *reinterpret_cast<const uint16_t *>(src + b);
                    }
                }
                src += row_stride;
                d += S::SLOT;
            }
            if (++p_s == nstages) { p_s = 0; p_bt += tw; }
        }
        p_set = p_set + 1 == NSETS ? 0 : p_set + 1;
        cp_async_commit();
    };

    float acc[B][NC];
#pragma unroll
    for (int i = 0; i < NSETS - 1; ++i) issue();
    int c_set = 0;
    for (int bt = gw; bt < n_bt; bt += tw) {
#pragma unroll
        for (int r = 0; r < B; ++r)
#pragma unroll
            for (int c = 0; c < NC; ++c) acc[r][c] = 0.f;
        for (int s = 0; s < nstages; ++s) {
            __syncwarp();                    // every lane is done with the set about to be refilled
            issue();
            cp_async_wait<NSETS - 1>();      // all but the NSETS-1 newest sets have landed
            __syncwarp();
            const uint8_t *set = ring + c_set * (B * S::SLOT);
            c_set = c_set + 1 == NSETS ? 0 : c_set + 1;
            {
                GemvX<NCG> X;
                gemv_load_x<TYPE, NCG>(lane, s, nblk, act, X);
#pragma unroll
                for (int r = 0; r < B; ++r) {
                    float a[NCG];
#pragma unroll
                    for (int c = 0; c < NCG; ++c) a[c] = acc[r][c];
                    gemv_lane_row<TYPE, NCG>(reinterpret_cast<const uint32_t *>(set + r * S::SLOT), lane, X, a);
#pragma unroll
                    for (int c = 0; c < NCG; ++c) acc[r][c] = a[c];
                }
            }
            if (NC2 > 0) {
                constexpr int N2 = NC2 > 0 ? NC2 : 1;
                GemvAct act2 = act;
                act2.q += (size_t)NCG * act.K;
                act2.d16 += (size_t)NCG * (act.K / 32);
                act2.d32 += (size_t)NCG * (act.K / 256);
                act2.s32 += (size_t)NCG * (act.K / 32);
                act2.s16 += (size_t)NCG * (act.K / 16);
                GemvX<N2> X;
                gemv_load_x<TYPE, N2>(lane, s, nblk, act2, X);
#pragma unroll
                for (int r = 0; r < B; ++r) {
                    float a[N2];
#pragma unroll
                    for (int c = 0; c < N2; ++c) a[c] = acc[r][NCG + (c < NC2 ? c : 0)];
                    gemv_lane_row<TYPE, N2>(reinterpret_cast<const uint32_t *>(set + r * S::SLOT), lane, X, a);
#pragma unroll
                    for (int c = 0; c < N2; ++c)
                        if (c < NC2) acc[r][NCG + c] = a[c];
                }
            }
        }
        const int row0 = bt * B;
#pragma unroll
        for (int r = 0; r < B; ++r)
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                float v = acc[r][c];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
                if (lane == 0 && row0 + r < M) dst[(size_t)c * ldd + row0 + r] = v;
            }
    }
    cp_async_wait<0>();
}

}  // namespace b200q
