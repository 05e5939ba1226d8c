// intrin.cuh -- the few machine intrinsics the kernels' per-lane code uses, each with a
// host twin so the same text can be compiled by g++ and run lane by lane on the CPU
// (tests/test_emul.py does that: a device-free check of every index and bit trick).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#define B200Q_HD __host__ __device__ __forceinline__

namespace b200q {

struct alignas(16) I4 { int x, y, z, w; };
struct alignas(8)  I2 { int x, y; };

B200Q_HD uint32_t hd_byte_perm(uint32_t a, uint32_t b, uint32_t s) {
#ifdef __CUDA_ARCH__
    // the PTX instruction itself: bit 3 of a selector nibble replicates the sign of the picked
    // byte, which the lookups below rely on and the __byte_perm intrinsic does not promise
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(s));
    return r;
#else
    const uint64_t v = ((uint64_t)b << 32) | a;
    uint32_t r = 0;
    for (int i = 0; i < 4; ++i) {
        const uint32_t sel = (s >> (4 * i)) & 0xF;
        uint32_t byte = (uint32_t)(v >> (8 * (sel & 7))) & 0xFF;
        if (sel & 8) byte = (byte & 0x80) ? 0xFF : 0x00;   // sign replicate mode
        r |= byte << (8 * i);
    }
    return r;
#endif
}

// (hi:lo) >> shift, low word; shift in 0..31
B200Q_HD uint32_t hd_funnelshift_r(uint32_t lo, uint32_t hi, uint32_t shift) {
#ifdef __CUDA_ARCH__
    return __funnelshift_r(lo, hi, shift);
#else
    return (uint32_t)((((uint64_t)hi << 32) | lo) >> (shift & 31));
#endif
}

// four signed-byte products summed into c
B200Q_HD int hd_dp4a(uint32_t a, int b, int c) {
#ifdef __CUDA_ARCH__
    return __dp4a((int)a, b, c);
#else
    for (int i = 0; i < 4; ++i) c += (int)(int8_t)(a >> (8 * i)) * (int)(int8_t)((uint32_t)b >> (8 * i));
    return c;
#endif
}

B200Q_HD float hd_half_bits(uint16_t h) {
#ifdef __CUDA_ARCH__
    return __half2float(__ushort_as_half(h));
#else
    __half_raw r;
    r.x = h;
    return __half2float(__half(r));
#endif
}

// 16-byte / 8-byte loads through the read-only path on the device
B200Q_HD I4 hd_ld16(const void *p) {
#ifdef __CUDA_ARCH__
    const int4 v = __ldg(reinterpret_cast<const int4 *>(p));
    return I4{ v.x, v.y, v.z, v.w };
#else
    I4 v;
    memcpy(&v, p, 16);
    return v;
#endif
}

B200Q_HD I2 hd_ld8(const void *p) {
#ifdef __CUDA_ARCH__
    const int2 v = __ldg(reinterpret_cast<const int2 *>(p));
    return I2{ v.x, v.y };
#else
    I2 v;
    memcpy(&v, p, 8);
    return v;
#endif
}

// A staged (shared-memory) row chunk held as 32-bit words. Plain loads through the pointer: the
// compiler sees that it points into shared memory and may hoist and pair the loads as it likes
// (explicit ld.shared in volatile asm measured slower: it pins the loads' order).
struct alignas(16) U4 { uint32_t x, y, z, w; };
struct Stage {
    const uint32_t *p;
    B200Q_HD explicit Stage(const uint32_t *q) : p(q) {}
    B200Q_HD uint32_t w(uint32_t i) const { return p[i]; }
    // four words at a 16-byte aligned place (word index i a multiple of 4 from an aligned chunk)
    B200Q_HD U4 ld16(uint32_t i) const {
#ifdef __CUDA_ARCH__
        const uint4 v = *reinterpret_cast<const uint4 *>(p + i);
        return U4{ v.x, v.y, v.z, v.w };
#else
        U4 v;
        memcpy(&v, p + i, 16);
        return v;
#endif
    }
};

// The packed blocks are only 2-byte aligned inside a row (18-, 34- and 210-byte blocks), so a run
// of N words at byte offset `off` (even) is N+1 aligned words and a funnel shift each.
template <int N>
B200Q_HD void stage_words(const Stage &st, uint32_t off, uint32_t (&out)[N]) {
    const uint32_t w = off >> 2, sh = (off & 2u) * 8u;
    uint32_t a[N + 1];
#pragma unroll
    for (int i = 0; i <= N; ++i) a[i] = st.w(w + i);
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = hd_funnelshift_r(a[i], a[i + 1], sh);
}

B200Q_HD uint16_t stage_u16(const Stage &st, uint32_t off) {
    return (uint16_t)(st.w(off >> 2) >> ((off & 2u) * 8u));
}

B200Q_HD uint32_t stage_u8(const Stage &st, uint32_t off) {
    return (st.w(off >> 2) >> ((off & 3u) * 8u)) & 0xFFu;
}

}  // namespace b200q
