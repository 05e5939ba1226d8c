// tmap.cu -- tensor maps for the tensor-core kernels' weight staging.
//
// The packed rows of a 128-row tile and one k-stage are a [128 x ROWB bytes] box of the weight
// matrix; described once per launch as a 2-D tensor of 32-bit elements, the producer warp fetches
// it with a single tiled copy instead of one bulk copy per row. The encoder is a driver entry
// point, looked up through the runtime so the library links nothing but the runtime.
#include <cuda.h>

#include "common.cuh"

namespace b200q {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

b200q_status make_weight_tmap(b200q_ctx *ctx, void *tmap_out, const void *w, size_t row_stride, int64_t M, int64_t row_bytes,
                              int box_bytes) {
    static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(ctx, B200Q_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
    if ((uintptr_t)w % 16 || row_stride % 16 || row_bytes % 4 || box_bytes % 16 || box_bytes / 4 > 256)
        return fail(ctx, B200Q_INVALID, "weight tensor map: alignment");
    const cuuint64_t dims[2] = { (cuuint64_t)(row_bytes / 4), (cuuint64_t)M };
    const cuuint64_t strides[1] = { (cuuint64_t)row_stride };
    const cuuint32_t box[2] = { (cuuint32_t)(box_bytes / 4), 128u };
    const cuuint32_t estr[2] = { 1u, 1u };
    const CUresult r = fn((CUtensorMap *)tmap_out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(w), dims, strides, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ctx, B200Q_CUDA_ERROR, "cuTensorMapEncodeTiled: %d", (int)r);
    return B200Q_OK;
}

// The same for a stack of n_mat matrices expert_stride bytes apart: a 3-D tensor, box = 128 rows x
// box_bytes x one matrix.
b200q_status make_weight_tmap3(b200q_ctx *ctx, void *tmap_out, const void *w, size_t row_stride, int64_t M, int64_t row_bytes,
                               int box_bytes, int64_t n_mat, size_t mat_stride) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(ctx, B200Q_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
    if ((uintptr_t)w % 16 || row_stride % 16 || mat_stride % 16 || row_bytes % 4 || box_bytes % 16 || box_bytes / 4 > 256)
        return fail(ctx, B200Q_INVALID, "weight tensor map: alignment");
    const cuuint64_t dims[3] = { (cuuint64_t)(row_bytes / 4), (cuuint64_t)M, (cuuint64_t)n_mat };
    const cuuint64_t strides[2] = { (cuuint64_t)row_stride, (cuuint64_t)mat_stride };
    const cuuint32_t box[3] = { (cuuint32_t)(box_bytes / 4), 128u, 1u };
    const cuuint32_t estr[3] = { 1u, 1u, 1u };
    const CUresult r = fn((CUtensorMap *)tmap_out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void *>(w), dims, strides, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ctx, B200Q_CUDA_ERROR, "cuTensorMapEncodeTiled: %d", (int)r);
    return B200Q_OK;
}

}  // namespace b200q
