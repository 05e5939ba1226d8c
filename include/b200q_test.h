/*
 * b200q_test.h -- measurement and test helpers of libb200q.so. Not part of the drop-in boundary (include/b200q.h):
 * a backend binding the path needs none of these; the benchmark and the parity tests do.
 */
#ifndef B200Q_TEST_H
#define B200Q_TEST_H

#include "b200q.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Device timing for benchmarks: cudaEvent pairs on the context's stream. */
B200Q_API b200q_status b200q_timer_start(b200q_ctx *ctx);
B200Q_API b200q_status b200q_timer_stop(b200q_ctx *ctx, float *elapsed_ms);  /* synchronizes */
/* writes a buffer larger than L2 so the next launch starts cold */
B200Q_API b200q_status b200q_flush_l2(b200q_ctx *ctx);

/* Debug views of what the kernels see, for bit-exact parity tests: the quantized
 * activation (codes [N][K] int8; scales fp16 [N][K/32] for Q4_0/Q8_0 weights or f32
 * [N][K/256] for the 256-block types; sums int16 [N][K/32] of each 32 codes) and
 * the dequantized weight rows the device decoders produce (f32 [M][K]). */
B200Q_API b200q_status b200q_debug_quantize_act(b200q_ctx *ctx, int weight_type, const b200q_tensor *src1,
                                                void *dev_codes, void *dev_scales, void *dev_sums);
B200Q_API b200q_status b200q_debug_dequantize(b200q_ctx *ctx, const b200q_tensor *src0, float *dev_out);
/* Failure-path check: enqueues a one-thread kernel whose bounded wait (at most `polls` polls of a barrier
 * nobody arrives at) must run out; like every kernel of the library it then sets the context's error word
 * and returns, so the next b200q_synchronize answers B200Q_TIMEOUT and the context stays usable. */
B200Q_API b200q_status b200q_debug_wait_timeout(b200q_ctx *ctx, unsigned polls);

/* Guard words. A context created with B200Q_CANARY=1 in the environment allocates every scratch block (quantized
 * activations, route tables, MoE and split-K scratch) at the size asked for, with 256 guard bytes before and after it.
 * This call synchronizes and checks them on the host: *blocks = blocks looked at, *violated = blocks whose guard was
 * overwritten (the first one is named in b200q_last_error). Without B200Q_CANARY: B200Q_INVALID. */
B200Q_API b200q_status b200q_debug_check_guards(b200q_ctx *ctx, int *blocks, int *violated);

#ifdef __cplusplus
}
#endif
#endif
