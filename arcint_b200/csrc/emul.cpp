// emul.cpp -- host build of the kernels' per-lane text, for device-free tests.
//
// The GEMV's lane code (gemv_core.cuh), the block decoders and the bit tricks
// (formats.cuh) are written once as host+device text. This file compiles them with g++
// and replays the kernel's loop structure (row groups, stages, 32 lanes) on the CPU, so
// every index computation and byte shuffle can be checked without a GPU -- the method
// of the reference's tests/test-opencl-kq-i8.cpp (marfrit/arcint contrib/llama.cpp/
// patches/0000-09-moe-routing-gemm-tiles.patch:1095-1697), which compiles its kernel
// helpers as C++. Not part of the product library.
#include <stdint.h>
#include <string.h>

#include <vector>

#include "gemv_core.cuh"
#include "peer_ar.cuh"
#include "ep_agree.h"

using namespace b200q;

template <int TYPE, int NC, int B>
static void emul_gemv_t(const uint8_t *W, size_t row_stride, int64_t M, int64_t K, const GemvAct &act, float *dst,
                        int64_t ldd) {
    typedef GemvFmt<TYPE> F;
    typedef GemvStage<TYPE> S;
    constexpr int NCG = NC <= 4 ? NC : (NC + 1) / 2, NC2 = NC - NCG, N2 = NC2 > 0 ? NC2 : 1;
    const int nblk = (int)(K / F::BLK_W), row_bytes = nblk * F::BLK_B;
    const int nstages = (nblk + F::STAGE_BLOCKS - 1) / F::STAGE_BLOCKS;
    const int64_t n_bt = (M + B - 1) / B;
    std::vector<uint32_t> set((size_t)B * S::SLOT / 4);
    for (int64_t bt = 0; bt < n_bt; ++bt) {
        static float acc[32][B][8];
        memset(acc, 0, sizeof(acc));
        for (int s = 0; s < nstages; ++s) {
            const int off = s * S::BYTES;
            const int bytes = (int)(row_bytes - off < S::BYTES ? row_bytes - off : S::BYTES);
            memset(set.data(), 0xA5, set.size() * 4);       // stale ring contents must not matter
            for (int r = 0; r < B; ++r)
                if (bt * B + r < M)
                    memcpy((uint8_t *)set.data() + r * S::SLOT, W + (size_t)(bt * B + r) * row_stride + off, (size_t)bytes);
            for (int lane = 0; lane < 32; ++lane) {
                int cols1[NCG], cols2[N2];
                for (int c = 0; c < NCG; ++c) cols1[c] = c;
                for (int c = 0; c < N2; ++c) cols2[c] = NCG + (c < NC2 ? c : 0);
                GemvX<NCG> X;
                gemv_load_x<TYPE, NCG>(lane, s, nblk, act, cols1, X);
                for (int r = 0; r < B; ++r) {
                    float a[NCG];
                    for (int c = 0; c < NCG; ++c) a[c] = acc[lane][r][c];
                    gemv_lane_row<TYPE, NCG>(set.data() + r * S::SLOT / 4, lane, X, a);
                    for (int c = 0; c < NCG; ++c) acc[lane][r][c] = a[c];
                }
                if (NC2 > 0) {
                    GemvX<N2> X2;
                    gemv_load_x<TYPE, N2>(lane, s, nblk, act, cols2, X2);
                    for (int r = 0; r < B; ++r) {
                        float a[N2];
                        for (int c = 0; c < N2; ++c) a[c] = acc[lane][r][NCG + (c < NC2 ? c : 0)];
                        gemv_lane_row<TYPE, N2>(set.data() + r * S::SLOT / 4, lane, X2, a);
                        for (int c = 0; c < NC2; ++c) acc[lane][r][NCG + c] = a[c];
                    }
                }
            }
        }
        for (int r = 0; r < B; ++r)
            for (int c = 0; c < NC; ++c) {
                float v[32];
                for (int l = 0; l < 32; ++l) v[l] = acc[l][r][c];
                for (int o = 16; o > 0; o >>= 1)            // the shuffle butterfly's order
                    for (int l = 0; l < o; ++l) v[l] += v[l + o];
                if (bt * B + r < M) dst[bt * B + r + c * ldd] = v[0];
            }
    }
}

template <int TYPE, int NC>
static void emul_gemv_r(int R, const uint8_t *W, size_t rs, int64_t M, int64_t K, const GemvAct &a, float *d, int64_t ldd) {
    if (R == 1) emul_gemv_t<TYPE, NC, 1>(W, rs, M, K, a, d, ldd);
    else        emul_gemv_t<TYPE, NC, 4>(W, rs, M, K, a, d, ldd);
}

template <int TYPE>
static int emul_gemv_nc(int nc, int R, const uint8_t *W, size_t rs, int64_t M, int64_t K, const GemvAct &a, float *d,
                        int64_t ldd) {
    switch (nc) {
    case 1: emul_gemv_r<TYPE, 1>(R, W, rs, M, K, a, d, ldd); return 0;
    case 2: emul_gemv_r<TYPE, 2>(R, W, rs, M, K, a, d, ldd); return 0;
    case 3: emul_gemv_r<TYPE, 3>(R, W, rs, M, K, a, d, ldd); return 0;
    case 4: emul_gemv_r<TYPE, 4>(R, W, rs, M, K, a, d, ldd); return 0;
    case 5: emul_gemv_r<TYPE, 5>(R, W, rs, M, K, a, d, ldd); return 0;
    case 7: emul_gemv_r<TYPE, 7>(R, W, rs, M, K, a, d, ldd); return 0;
    case 8: emul_gemv_r<TYPE, 8>(R, W, rs, M, K, a, d, ldd); return 0;
    }
    return -1;
}

extern "C" {

int emul_gemv(int type, const uint8_t *W, size_t row_stride, int64_t M, int64_t K, const int8_t *xq,
              const uint16_t *d16, const float *d32, const int16_t *s32, const int16_t *s16, int ncols, int R,
              float *dst, int64_t ldd) {
    GemvAct a;
    a.q = xq;
    a.d16 = d16;
    a.d32 = d32;
    a.s32 = s32;
    a.s16 = s16;
    a.K = (int)K;
    switch (type) {
    case B200Q_TYPE_Q4_0:   return emul_gemv_nc<B200Q_TYPE_Q4_0>(ncols, R, W, row_stride, M, K, a, dst, ldd);
    case B200Q_TYPE_Q8_0:   return emul_gemv_nc<B200Q_TYPE_Q8_0>(ncols, R, W, row_stride, M, K, a, dst, ldd);
    case B200Q_TYPE_Q4_K:   return emul_gemv_nc<B200Q_TYPE_Q4_K>(ncols, R, W, row_stride, M, K, a, dst, ldd);
    case B200Q_TYPE_Q5_K:   return emul_gemv_nc<B200Q_TYPE_Q5_K>(ncols, R, W, row_stride, M, K, a, dst, ldd);
    case B200Q_TYPE_Q6_K:   return emul_gemv_nc<B200Q_TYPE_Q6_K>(ncols, R, W, row_stride, M, K, a, dst, ldd);
    case B200Q_TYPE_IQ4_XS: return emul_gemv_nc<B200Q_TYPE_IQ4_XS>(ncols, R, W, row_stride, M, K, a, dst, ldd);
    case B200Q_TYPE_IQ4_NL: return emul_gemv_nc<B200Q_TYPE_IQ4_NL>(ncols, R, W, row_stride, M, K, a, dst, ldd);
    }
    return -1;
}

void emul_dequantize_row(int type, const uint8_t *row, int64_t K, float *out) {
    for (int64_t i = 0; i < K; ++i) out[i] = decode_weight(type, row, i);
}

uint32_t emul_iq4nl_lookup4(uint32_t idx) { return iq4nl_lookup4(idx); }

// lookup of four indices in a 16-byte table given as four words
uint32_t emul_lookup4_tab(const uint32_t *t, uint32_t idx) {
    uint32_t sel, msk;
    lookup4_prepare(idx, &sel, &msk);
    return lookup4_apply(t[0], t[1], t[2], t[3], sel, msk);
}

void emul_iq4xs_limbs(int ls, int n, int *hi, int *lo) { iq4xs_limbs(ls, n, hi, lo); }
void emul_q6k_limbs4(uint32_t q6, int sc, uint32_t *out2) { q6k_limbs4(q6, sc, out2, out2 + 1); }
void emul_q4k_limbs4(uint32_t idx, uint32_t sc, uint32_t *out2) { q4k_limbs4(idx, sc, out2, out2 + 1); }
void emul_q4k_scales_mins(uint32_t s0, uint32_t s1, uint32_t s2, uint32_t *out4) {
    q4k_scales8(s0, s1, s2, out4, out4 + 1);
    q4k_mins8(s0, s1, s2, out4 + 2, out4 + 3);
}
void emul_q4k_scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int j, int *sc, int *m) { q4k_scale_min(s0, s1, s2, j, sc, m); }
void emul_iq4xs_limbs8(uint32_t q, int m, uint32_t *out4) { iq4xs_limbs8(q, m, out4, out4 + 1, out4 + 2, out4 + 3); }
// Host replay of the one-shot all-reduce's slot protocol (peer_ar.cuh): nranks receive buffers, two
// all-reduces in a row (both sets of slots), every rank writes its vector into every buffer and then reads
// its own. Rank `silent` (if >= 0) writes nothing in the second all-reduce: the readers' bounded waits must
// then give up (gave_up[r] = 1) instead of spinning, having taken the stale element they found.
// in: [2][nranks][count] floats, out: [2][nranks][count]. Returns 0.
int emul_peer_allreduce(int nranks, int count, const float *in, float *out, int silent, unsigned limit, int *gave_up) {
    if (nranks < 1 || nranks > PEER_AR_MAX_RANKS || count < 0 || count > PEER_AR_MAX_FLOATS) return -1;
    std::vector<std::vector<uint64_t>> buf(nranks, std::vector<uint64_t>(PEER_AR_BUFFER_BYTES / 8, 0));
    auto load = [](const uint64_t *p) { return *p; };
    for (int r = 0; r < nranks; ++r) gave_up[r] = 0;
    for (uint32_t call = 0; call < 2; ++call) {
        const uint32_t seq = call + 1;
        const int set = (int)(seq & 1u);
        for (int r = 0; r < nranks; ++r) {
            if (call == 1 && r == silent) continue;
            for (int e = 0; e < count; ++e)
                for (int p = 0; p < nranks; ++p)
                    buf[p][peer_ar_index(set, r, e)] = peer_ar_pack(in[((size_t)call * nranks + r) * count + e], seq);
        }
        for (int r = 0; r < nranks; ++r)
            for (int e = 0; e < count; ++e) {
                float sum = 0.f;
                bool ok = true;
                for (int q = 0; q < nranks; ++q)
                    sum += peer_ar_value(peer_ar_wait(&buf[r][peer_ar_index(set, q, e)], seq, limit, load, &ok));
                if (!ok) gave_up[r] = 1;
                out[((size_t)call * nranks + r) * count + e] = sum;
            }
    }
    return 0;
}

// The exit rule of the NCCL form of expert parallelism (ep_agree.h): G records of `stride` int32, status at
// `status_at`; what rank `rank` returns (0, its own status, or peer_failed) and the lowest failing rank.
int emul_ep_agree(const int32_t *records, int G, int stride, int status_at, int rank, int peer_failed, int *who) {
    return ep_agree_decide(records, G, stride, status_at, rank, peer_failed, who);
}

uint32_t emul_nib_minus8(uint32_t t) { return nib_minus8(t); }
uint32_t emul_six_minus32(uint32_t t) { return six_minus32(t); }

}
