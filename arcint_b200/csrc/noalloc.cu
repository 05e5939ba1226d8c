// noalloc.cu -- b200q_mul_mat_noalloc: the decode-width product for callers that cannot
// allocate device memory.
//
// Who that is: a host that handed all of the GPU's memory to its own pool when it started
// (so a later cudaMalloc simply fails), and a serving loop that must never run into the
// device-wide synchronisation cudaMalloc and cudaFree imply. Such a caller cannot create a
// b200q context either, because a context grows its scratch with cudaMalloc. This entry point
// takes no context and allocates nothing: the quantized activation it needs between its two
// kernels lives in a fixed array that is part of the library image. The price is a size limit
// (at most 8 activation columns of at most 32768 values) and 320 KiB of device memory held by
// every GPU that loads the library, until the process exits.
//
// The array is shared by every call and keeps what the last call left in it. Nothing has to
// start at zero: a call overwrites every byte it later reads (codes, scales and block sums of
// its own columns) before the product kernel runs. Two calls that overlap on one GPU (different
// streams, or different host threads) would overwrite each other's activation: callers must
// keep calls on a device ordered.
//
// In host code the array's name is only a stand-in; the address kernels can use comes from
// cudaGetSymbolAddress, asked once per device with that device current. The first call on a
// device does this, so it should happen before any stream capture is opened. The first call for
// a weight type and column count also asks the driver for that kernel's attributes (and, with lazy
// module loading, makes the driver load the kernel's code): a host that is about to hand all device
// memory to its own pool should make one call per weight type and column count it will use first.
//
// The last 256 bytes of the array hold the word a GEMV kernel sets when one of its bounded waits runs
// out (it starts at zero and nothing clears it; b200q_noalloc_device_error reads it).
#include <stdlib.h>

#include <mutex>

#include "common.cuh"

namespace b200q {

constexpr int     NOALLOC_MAX_COLS = 8;
constexpr int64_t NOALLOC_MAX_K = 32768;
// codes 8 x 32768 | scales (fp16 per 32 or f32 per 256: at most 16 KiB) | sums of 32 (16 KiB) | sums of 16 (32 KiB),
// each part on a 256-byte boundary
constexpr size_t NOALLOC_CODES = (size_t)NOALLOC_MAX_COLS * NOALLOC_MAX_K;
constexpr size_t NOALLOC_SCALES = (size_t)NOALLOC_MAX_COLS * (NOALLOC_MAX_K / 32) * 2;
constexpr size_t NOALLOC_SUMS32 = (size_t)NOALLOC_MAX_COLS * (NOALLOC_MAX_K / 32) * 2;
constexpr size_t NOALLOC_SUMS16 = (size_t)NOALLOC_MAX_COLS * (NOALLOC_MAX_K / 16) * 2;
constexpr size_t NOALLOC_ERROR = 256;       // the kernels' error word, on its own 256 bytes
constexpr size_t NOALLOC_BYTES = NOALLOC_CODES + NOALLOC_SCALES + NOALLOC_SUMS32 + NOALLOC_SUMS16 + NOALLOC_ERROR;
static_assert(NOALLOC_BYTES == 320 * 1024 + 256, "the documented size of the fixed array");

static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_BYTES];

constexpr int NOALLOC_MAX_DEVICES = 64;
static unsigned char *g_scratch_ptr[NOALLOC_MAX_DEVICES];    // device address of the array, per device
static int            g_sm_count[NOALLOC_MAX_DEVICES];
static std::mutex     g_setup_mutex;
static thread_local std::string g_noalloc_error;

}  // namespace b200q

using namespace b200q;

extern "C" {

const char *b200q_noalloc_last_error(void) { return g_noalloc_error.c_str(); }

b200q_status b200q_mul_mat_noalloc(int device, void *stream, const b200q_tensor *src0, const b200q_tensor *src1,
                                   b200q_tensor *dst) {
    g_noalloc_error.clear();
    auto bad = [&](b200q_status st, const std::string &msg) { g_noalloc_error = msg; return st; };
    if (!src0 || !src1 || !dst) return bad(B200Q_INVALID, "null tensor");
    if (device < 0 || device >= NOALLOC_MAX_DEVICES) return bad(B200Q_INVALID, "device index out of range");
    // a context on the stack: plain host state for the launch helpers, no device memory behind it
    b200q_ctx ctx;
    ctx.device = device;
    ctx.stream = (cudaStream_t)stream;
    b200q_status st = b200q_supports(nullptr, B200Q_OP_MUL_MAT, src0, src1, nullptr, dst);
    if (st != B200Q_OK) return bad(st, "shape, type or layout outside what b200q_mul_mat takes");
    TypeInfo ti;
    type_info(src0->type, &ti);
    const int64_t K = src0->ne[0], M = src0->ne[1];
    const int64_t N = src1->ne[1] * src1->ne[2] * src1->ne[3];
    if (N > NOALLOC_MAX_COLS)
        return bad(B200Q_UNSUPPORTED, "b200q_mul_mat_noalloc takes at most 8 activation columns, got " + std::to_string(N));
    if (K > NOALLOC_MAX_K)
        return bad(B200Q_UNSUPPORTED, "b200q_mul_mat_noalloc takes rows of at most 32768 weights, got " + std::to_string(K));
    const size_t s1 = dst->nb[1];
    if ((dst->ne[2] != 1 && dst->nb[2] != s1 * (size_t)dst->ne[1]) ||
        (dst->ne[3] != 1 && dst->nb[3] != s1 * (size_t)dst->ne[1] * (size_t)dst->ne[2]))
        return bad(B200Q_UNSUPPORTED, "b200q_mul_mat_noalloc needs evenly spaced dst columns");
    if (M == 0 || N == 0) return B200Q_OK;
    if (cudaSetDevice(device) != cudaSuccess) return bad(B200Q_CUDA_ERROR, "cudaSetDevice failed");
    {
        // once per device, with that device current: the array's address as kernels see it
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (!g_scratch_ptr[device]) {
            unsigned char *p = nullptr;
            cudaError_t e = cudaGetSymbolAddress((void **)&p, g_noalloc_scratch);
            if (e != cudaSuccess || !p)
                return bad(B200Q_CUDA_ERROR, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
            int sms = 0;
            e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
            if (e != cudaSuccess || sms <= 0)
                return bad(B200Q_CUDA_ERROR, std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
            g_sm_count[device] = sms;
            g_scratch_ptr[device] = p;
        }
    }
    ctx.sm_count = g_sm_count[device];
    static const bool no_pdl = [] { const char *v = getenv("B200Q_NO_PDL"); return v && v[0] == '1'; }();
    static const bool no_stream = [] { const char *v = getenv("B200Q_NO_STREAM"); return v && v[0] == '1'; }();
    ctx.no_pdl = no_pdl;
    ctx.no_stream = no_stream;
    unsigned char *base = g_scratch_ptr[device];
    int8_t *codes = (int8_t *)base;
    void *scales = base + NOALLOC_CODES;
    int16_t *sums32 = (int16_t *)(base + NOALLOC_CODES + NOALLOC_SCALES);
    int16_t *sums16 = (int16_t *)(base + NOALLOC_CODES + NOALLOC_SCALES + NOALLOC_SUMS32);
    ctx.error_word = (int *)(base + NOALLOC_BYTES - NOALLOC_ERROR);
    // kernel 1 writes the activation of this call's N columns into the array, kernel 2 reads it
    st = launch_quantize_act(&ctx, ti.act_form, src1, codes, scales, sums32, sums16);
    if (st != B200Q_OK) return bad(st, ctx.last_error);
    ActView act;
    act.codes = codes;
    act.d16 = ti.act_form == ACT_Q8_0 ? (const uint16_t *)scales : nullptr;
    act.d32 = ti.act_form == ACT_Q8_256 ? (const float *)scales : nullptr;
    act.s32 = sums32;
    act.s16 = ti.act_form == ACT_Q8_256 ? sums16 : nullptr;
    act.form = ti.act_form;
    act.K = K;
    act.N = N;
    st = launch_gemv(&ctx, src0->type, src0->data, src0->nb[1], M, K, act, 0, (int)N, (float *)dst->data,
                     (int64_t)(s1 / sizeof(float)));
    if (st != B200Q_OK) return bad(st, ctx.last_error);
    return B200Q_OK;
}

// Nonzero when a kernel of an earlier b200q_mul_mat_noalloc call on `device` gave up a bounded wait
// (its results are then incomplete). Synchronizes the device's default stream copy; not for hot paths.
b200q_status b200q_noalloc_device_error(int device, int *error) {
    if (!error || device < 0 || device >= NOALLOC_MAX_DEVICES) return B200Q_INVALID;
    *error = 0;
    if (!g_scratch_ptr[device]) return B200Q_OK;             // no call has run on this device yet
    if (cudaSetDevice(device) != cudaSuccess) return B200Q_CUDA_ERROR;
    if (cudaMemcpy(error, g_scratch_ptr[device] + NOALLOC_BYTES - NOALLOC_ERROR, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
        return B200Q_CUDA_ERROR;
    return B200Q_OK;
}

}  // extern "C"
