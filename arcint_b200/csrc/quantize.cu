// quantize.cu -- f32 activations -> int8 codes + scales, and the debug dequantizer.
//
// Two forms, chosen by the weight type the activation meets:
//   per 32  (Q4_0, Q8_0 weights): ggml's block_q8_0 rule -- d = amax/127 stored as fp16,
//           code = roundf(x * (1/d)), half away from zero. The reference's per-32 quantizer
//           kq_i8_quant32 (marfrit/arcint contrib/llama.cpp/patches/
//           0000-09-moe-routing-gemm-tiles.patch:544-553) is the same grid.
//   per 256 (Q4_K, Q6_K, IQ4_XS weights): the reference's kernel_quant_i8
//           (0000-01-kquant-integer-dpas.patch:1862-1889) -- scale bm/127 in f32, code =
//           round-to-nearest-even of x * (127/bm), a block below 1e-30 quantizes to zeros,
//           plus the integer sum of each 32 codes.
// Both also write the integer sum of each 32 codes (and of each 16, per-256 form): the
// kernels keep weight codes unsigned and take the -8 / -32 offsets from these sums.
// Column c of src1 (flattened over dimensions 1..3) lands at codes + c*K.
#include "formats.cuh"
#include "common.cuh"
#include "pdl.cuh"

namespace b200q {

struct ColAddr {
    const uint8_t *base;
    int64_t ne1, ne2;
    size_t  nb1, nb2, nb3;
};

__device__ __forceinline__ const float *col_ptr(const ColAddr &a, int64_t c) {
    const int64_t c1 = c % a.ne1, c23 = c / a.ne1, c2 = c23 % a.ne2, c3 = c23 / a.ne2;
    return reinterpret_cast<const float *>(a.base + c1 * a.nb1 + c2 * a.nb2 + c3 * a.nb3);
}

// 8 lanes per 32-block, 4 values per lane
__global__ void __launch_bounds__(256)
quantize_q8_0_kernel(ColAddr src, int64_t K, int64_t ncols, int8_t *__restrict__ codes, uint16_t *__restrict__ d16,
                     int16_t *__restrict__ sums32) {
    pdl_trigger();
    pdl_wait();                          // src1 may be the output of the kernel before, the scratch its input
    const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t per_col = K / 4;
    const int64_t c = gid / per_col, i4 = gid % per_col;
    const bool live = c < ncols;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) v = *reinterpret_cast<const float4 *>(col_ptr(src, c) + 4 * i4);
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 4));
    const float d = __fdiv_rn(amax, 127.f);
    const float id = d != 0.f ? __fdiv_rn(1.f, d) : 0.f;
    const int q0 = (int)roundf(__fmul_rn(v.x, id)), q1 = (int)roundf(__fmul_rn(v.y, id));
    const int q2 = (int)roundf(__fmul_rn(v.z, id)), q3 = (int)roundf(__fmul_rn(v.w, id));
    int sum = q0 + q1 + q2 + q3;
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
    if (!live) return;
    const uint32_t packed = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) |
                            ((uint32_t)(q3 & 0xFF) << 24);
    reinterpret_cast<uint32_t *>(codes + c * K)[i4] = packed;
    if ((i4 & 7) == 0) {
        d16[c * (K / 32) + i4 / 8] = __half_as_ushort(__float2half_rn(d));
        sums32[c * (K / 32) + i4 / 8] = (int16_t)sum;
    }
}

// one warp per 256-block, 8 values per lane
__global__ void __launch_bounds__(256)
quantize_q8_256_kernel(ColAddr src, int64_t K, int64_t ncols, int8_t *__restrict__ codes, float *__restrict__ d32,
                       int16_t *__restrict__ bsums, int16_t *__restrict__ bsums16) {
    pdl_trigger();
    pdl_wait();                          // src1 may be the output of the kernel before, the scratch its input
    const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int64_t per_col = K / 256;
    const int64_t c = wid / per_col, b = wid % per_col;
    if (c >= ncols) return;                       // whole warps leave together
    const float *x = col_ptr(src, c) + 256 * b + 8 * lane;
    const float4 v0 = *reinterpret_cast<const float4 *>(x), v1 = *reinterpret_cast<const float4 *>(x + 4);
    float bm = fmaxf(fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))),
                     fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) bm = fmaxf(bm, __shfl_xor_sync(0xFFFFFFFFu, bm, o));
    const float iq = bm > 1e-30f ? __fdiv_rn(127.f, bm) : 0.f;
    int q[8];
    q[0] = __float2int_rn(__fmul_rn(v0.x, iq)); q[1] = __float2int_rn(__fmul_rn(v0.y, iq));
    q[2] = __float2int_rn(__fmul_rn(v0.z, iq)); q[3] = __float2int_rn(__fmul_rn(v0.w, iq));
    q[4] = __float2int_rn(__fmul_rn(v1.x, iq)); q[5] = __float2int_rn(__fmul_rn(v1.y, iq));
    q[6] = __float2int_rn(__fmul_rn(v1.z, iq)); q[7] = __float2int_rn(__fmul_rn(v1.w, iq));
    int s = 0;
    uint32_t p0 = 0, p1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        s += q[i] + q[i + 4];
        p0 |= (uint32_t)(q[i] & 0xFF) << (8 * i);
        p1 |= (uint32_t)(q[i + 4] & 0xFF) << (8 * i);
    }
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);      // a group of 16 is two lanes
    if ((lane & 1) == 0) bsums16[c * (K / 16) + 16 * b + lane / 2] = (int16_t)s;
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);      // a 32-block is four lanes
    *reinterpret_cast<uint2 *>(codes + c * K + 256 * b + 8 * lane) = make_uint2(p0, p1);
    if ((lane & 3) == 0) bsums[c * (K / 32) + 8 * b + lane / 4] = (int16_t)s;
    if (lane == 0) d32[c * per_col + b] = __fdiv_rn(bm, 127.f);
}

b200q_status launch_quantize_act(b200q_ctx *ctx, int form, const b200q_tensor *src1, int8_t *codes, void *scales,
                                 int16_t *bsums, int16_t *bsums16) {
    const int64_t K = src1->ne[0];
    const int64_t ncols = src1->ne[1] * src1->ne[2] * src1->ne[3];
    if (ncols == 0) return B200Q_OK;
    ColAddr a;
    a.base = (const uint8_t *)src1->data;
    a.ne1 = src1->ne[1];
    a.ne2 = src1->ne[2];
    a.nb1 = src1->nb[1];
    a.nb2 = src1->nb[2];
    a.nb3 = src1->nb[3];
    if (form == ACT_Q8_0) {
        const int64_t threads = ncols * (K / 4);
        B200Q_CUDA(ctx, launch_pdl(!ctx->no_pdl, quantize_q8_0_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0,
                                   ctx->stream, a, K, ncols, codes, (uint16_t *)scales, bsums));
        count(ctx, ST_QUANT_Q8_0);
    } else {
        const int64_t warps = ncols * (K / 256);
        B200Q_CUDA(ctx, launch_pdl(!ctx->no_pdl, quantize_q8_256_kernel, dim3((unsigned)((warps * 32 + 255) / 256)), dim3(256), 0,
                                   ctx->stream, a, K, ncols, codes, (float *)scales, bsums, bsums16));
        count(ctx, ST_QUANT_Q8_256);
    }
    B200Q_CUDA(ctx, cudaGetLastError());
    return B200Q_OK;
}

__global__ void dequantize_kernel(int type, const uint8_t *w, int64_t M, int64_t K, size_t row_stride, float *out) {
    const int64_t total = M * K;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / K, k = i % K;
        out[i] = decode_weight(type, w + r * row_stride, k);
    }
}

b200q_status launch_dequantize(b200q_ctx *ctx, int type, const void *w, int64_t M, int64_t K, size_t row_stride,
                               float *out) {
    const int64_t total = M * K;
    if (total == 0) return B200Q_OK;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    dequantize_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(type, (const uint8_t *)w, M, K, row_stride, out);
    B200Q_CUDA(ctx, cudaGetLastError());
    return B200Q_OK;
}

}  // namespace b200q
