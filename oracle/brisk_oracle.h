/* TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * Plain-C restatement of the reference CPU token loop of brisk-llm (generic scalar kernels,
 * Model(file, repack=false) + Session). Used only by tests/, __graft_entry__.smoke() and
 * bench.py's cpu_baseline leg as the checker of the CUDA library; the product never links,
 * loads or calls it.
 *
 * Parity pin: tests/test_oracle_vs_reference.py compares every function here against the
 * unmodified reference (oracle/_ref/libbrisk_ref.so) where a reference checkout is present, and
 * tests/golden/ holds vectors generated from that same reference build for machines without one.
 */
#ifndef BRISK_ORACLE_H
#define BRISK_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#include "../include/brisk_cuda.h" /* the model description structs only */

#ifdef __cplusplus
extern "C" {
#endif

float oracle_half_to_float(uint16_t h);
uint16_t oracle_float_to_half(float f);

void oracle_quantize_q8_0(const float* x, void* out, uint64_t count);
void oracle_quantize_q8_k(const float* x, void* out, uint64_t count);
int oracle_dequantize(int32_t type, const void* blocks, float* out, uint64_t count);
int oracle_matmul(int32_t type, const void* w, uint64_t rows, uint64_t cols, const float* x, uint64_t n, float* out);

typedef struct oracle_session oracle_session;
oracle_session* oracle_session_create(const brisk_cuda_model* model, uint64_t max_context);
void oracle_session_destroy(oracle_session* s);
const char* oracle_last_error(void);
int oracle_session_eval(oracle_session* s, const int32_t* tokens, uint64_t n, int all_logits, float* logits_out);
int oracle_session_rollback(oracle_session* s, uint64_t position);
uint64_t oracle_session_position(const oracle_session* s);
int oracle_session_log_likelihood(oracle_session* s, const int32_t* tokens, uint64_t n, double* out);
int oracle_session_generate_greedy(oracle_session* s, const int32_t* prompt, uint64_t n_prompt, uint64_t steps,
                                   int32_t* out_tokens, float* out_logits);
/* The last token's residual stream after each layer of the most recent eval: [layers][hidden]. */
int oracle_session_layer_trace(const oracle_session* s, float* out);
int oracle_session_debug_buffer(const oracle_session* s, const char* name, float* out, uint64_t count);
uint64_t oracle_lookup_draft(const int32_t* history, uint64_t n, uint64_t count, int32_t* out);
int64_t oracle_session_speculate(oracle_session* s, const int32_t* prompt, uint64_t n_prompt, uint64_t draft_tokens,
                                 uint64_t want, int32_t* out, uint64_t* rounds, uint64_t* accepted);

#ifdef __cplusplus
}
#endif
#endif
