// ref_shim.cpp -- C entry points around the reference's own kq_i8_ops.inc
// (contrib/llama.cpp/patches/0000-09-moe-routing-gemm-tiles.patch, the file
// ggml/src/ggml-opencl/kernels/kq_i8_ops.inc it adds). build_ref.py extracts
// that file from the patch into _ref/ and compiles this shim against it, so the
// oracle can be checked against the reference's own text. TEST INFRASTRUCTURE.
#include "kq_i8_ops.inc"

extern "C" {

void ref_kq_i8_quant32(const float *x, signed char *q, float *scale) {
    kq_i8_quant32(x, reinterpret_cast<kq_s8 *>(q), scale);
}

// 16 stored bytes of one IQ4_NL / IQ4_XS 32-block -> 32 signed codebook values in
// ggml's order (low nibbles first), kv = kvalues_iq4nl
void ref_kq_i8_decode_iq4nl(const unsigned char *qs, const signed char *kv, signed char *out) {
    kq_u32 w[8];
    kq_i8_decode_iq4nl(kq_i8_u32(qs), kq_i8_u32(qs + 4), kq_i8_u32(qs + 8), kq_i8_u32(qs + 12),
                       reinterpret_cast<const kq_s8 *>(kv), w);
    for (int i = 0; i < 8; ++i)
        for (int b = 0; b < 4; ++b) out[4 * i + b] = (signed char)((w[i] >> (8 * b)) & 0xFFu);
}

int ref_kq_i8_col(int p, int n_used, int ne11) { return kq_i8_col(p, n_used, ne11); }

long ref_kq_i8_mean_pairs(long n_pairs, int n_expert) { return kq_i8_mean_pairs(n_pairs, n_expert); }

}
