/*
 * b200q_oracle.h -- CPU restatement of the quantized MUL_MAT / MUL_MAT_ID path.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the product library links, loads or
 * calls this file; it exists so the CUDA path has something to be checked
 * against, and so a CPU time can be printed beside the GPU one.
 *
 * Pinning status:
 *   - Q4_0 / Q8_0 weight quantizers and the five dequantizers are pinned
 *     bit-exactly against gguf-py (the ggml authors' numpy implementation,
 *     gguf/quants.py) through committed golden vectors.
 *   - the per-32 activation quantizer and the IQ4 codebook decode are pinned
 *     against the reference's own kq_i8_ops.inc (compiled from the reference
 *     tree where it is present).
 *   - PARITY UNPINNED: the Q4_K / Q6_K / IQ4_XS *weight quantizers* here are
 *     original round-to-nearest stand-ins (ggml's search-based quantizers are
 *     not available), and the per-256 activation quantizer follows the
 *     reference's kernel_quant_i8 rule, not ggml's quantize_row_q8_K.
 */
#ifndef B200Q_ORACLE_H
#define B200Q_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGML type ids (gguf.constants.GGMLQuantizationType). */
enum {
    ORC_TYPE_F32    = 0,
    ORC_TYPE_Q4_0   = 2,
    ORC_TYPE_Q8_0   = 8,
    ORC_TYPE_Q4_K   = 12,
    ORC_TYPE_Q5_K   = 13,
    ORC_TYPE_Q6_K   = 14,
    ORC_TYPE_IQ4_NL = 20,
    ORC_TYPE_IQ4_XS = 23,
    ORC_TYPE_I32    = 26
};

/* Activation forms. */
enum {
    ORC_ACT_Q8_0  = 0,  /* per 32: fp16 scale, int8 codes (ggml block_q8_0)         */
    ORC_ACT_Q8_256 = 1  /* per 256: f32 scale, int8 codes, int16 sums of each 32     */
};

int    orc_block_size(int type);                 /* weights per block, 0 if unknown */
size_t orc_block_bytes(int type);                /* bytes per block                 */
size_t orc_row_bytes(int type, int64_t k);       /* bytes of one row of k weights   */
int    orc_act_form(int type);                   /* activation form a type pairs with */

float    orc_fp16_to_fp32(uint16_t h);
uint16_t orc_fp32_to_fp16(float f);

/* weights */
int orc_dequantize_row(int type, const void *src, float *dst, int64_t k);
int orc_quantize_row(int type, const float *src, void *dst, int64_t k);
int orc_quantize_rows(int type, const float *src, void *dst, int64_t nrows, int64_t k, int nthreads);

/* activations: one column of k values */
void orc_quantize_act_q8_0(const float *x, int8_t *q, uint16_t *d, int64_t k);
void orc_quantize_act_q8_256(const float *x, int8_t *q, float *d, int16_t *bsums, int64_t k);
void orc_dequantize_act(int form, const int8_t *q, const void *d, float *dst, int64_t k);

/* dst[m + t*ldd] = sum_k W[m,k] * x[k + t*ldx], ggml form: quantized activations,
 * exact integer block dots, f32 scale-accumulate. nthreads <= 0: all cores. */
int orc_mul_mat(int type, const void *w, int64_t m, int64_t k,
                const float *x, int64_t n, int64_t ldx,
                float *dst, int64_t ldd, int nthreads);

/* fp64 reference. quantized_act != 0: dequant(W) x dequant(Q(x)); else raw f32 x. */
int orc_mul_mat_f64(int type, const void *w, int64_t m, int64_t k,
                    const float *x, int64_t n, int64_t ldx,
                    double *dst, int64_t ldd, int quantized_act, int nthreads);

/* MUL_MAT_ID: w [k, m, n_expert]; x [k, ne11, n_tok] f32 (ne11 = 1 or n_used);
 * ids [n_used, n_tok] i32 with row stride ids_stride (in int32 elements);
 * dst [m, n_used, n_tok]. Pair (i,t): expert ids[t][i], column (i % ne11) + t*ne11. */
int orc_mul_mat_id(int type, const void *w, int64_t m, int64_t k, int n_expert,
                   const float *x, int ne11, int n_tok,
                   const int32_t *ids, int64_t ids_stride, int n_used,
                   float *dst, int nthreads);
int orc_mul_mat_id_f64(int type, const void *w, int64_t m, int64_t k, int n_expert,
                       const float *x, int ne11, int n_tok,
                       const int32_t *ids, int64_t ids_stride, int n_used,
                       double *dst, int quantized_act, int nthreads);

/* Routing: pairs p = t*n_used + i sorted by expert (stable in p), cut into tiles of
 * at most `tile` pairs of one expert: tiles[4*j] = {expert, first, count, 0}.
 * Returns the tile count. pairs has n_used*n_tok entries; tiles room for
 * ceil(pairs/tile) + min(n_expert, pairs) entries. */
int orc_moe_route(const int32_t *ids, int64_t ids_stride, int n_used, int n_tok, int n_expert,
                  int tile, int32_t *pairs, int32_t *tiles);

/* Seeded inputs: counter-based generator, value i of stream (seed) ~ N(0, sigma^2). */
void orc_fill_normal(float *dst, int64_t n, uint64_t seed, float sigma, int nthreads);
/* Zipf(s)-skewed router logits -> top-n_used ids per token, ties to the lower id. */
void orc_route_ids(int32_t *ids, int n_used, int n_tok, int n_expert, uint64_t seed, float zipf_s);

int orc_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif
