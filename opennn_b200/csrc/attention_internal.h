// Internal interface between the MultiHeadAttention front end and the fused attention-core kernel.
#pragma once
#include <cuda_runtime.h>
#include "../../include/onn_b200.h"

namespace onn
{
// q [B, Sq, E], k and v [B, Sk, E] (head h = columns h * 64 ..), weights [B, H, Sq, Sk], context [B, Sq, E].
// Supported: head size 64, Sk <= 256 and a multiple of 4, 16-byte aligned bases.
bool attention_fwd_fused_supported(const float* q, const float* k, const float* v, const float* weights, const float* context,
                                   long long B, long long Sq, long long Sk, long long E, long long H);
int attention_fwd_fused_launch(const float* q, const float* k, const float* v, const unsigned char* key_is_pad,
                               float* weights, float* context, long long B, long long Sq, long long Sk, long long E, long long H,
                               int causal, float scale, cudaStream_t stream);
// Backward of the same core up to the query gradient: d_scores = P * (dP - rowsum(P * dP)) with dP = dO V^T, and
// d_q = scale * d_scores K (+ its column sums into d_bias_q).  The key and value gradients follow from d_scores
// and the weights with two batched GEMMs.
bool attention_bwd_fused_supported(const float* k, const float* v, const float* weights, const float* context, const float* d_context,
                                   const float* d_scores, const float* d_q, long long B, long long Sq, long long Sk, long long E, long long H);
int attention_bwd_fused_launch(const float* k, const float* v, const float* weights, const float* context, const float* d_context,
                               float* d_scores, float* d_q, float* d_bias_q, long long B, long long Sq, long long Sk, long long E, long long H,
                               float scale, cudaStream_t stream);
// The same core for source lengths above 256 (head size 64): the keys are walked in tiles of 256 (attention_long.cu).
bool attention_long_supported(long long B, long long Sq, long long Sk, long long E, long long H);
int attention_long_fwd_launch(const float* q, const float* k, const float* v, const unsigned char* key_is_pad,
                              float* weights, float* context, long long B, long long Sq, long long Sk, long long E, long long H,
                              int causal, float scale, cudaStream_t stream);
// `causal`: the weights of whole key tiles above the diagonal are zero; those tiles are skipped and d_scores gets zeros there.
int attention_long_bwd_launch(const float* k, const float* v, const float* weights, const float* context, const float* d_context,
                              float* d_scores, float* d_q, float* d_bias_q, long long B, long long Sq, long long Sk, long long E, long long H,
                              int causal, float scale, cudaStream_t stream);
int attention_long_read_status();
const unsigned int* attention_long_status_word();       // device address on the current device
int attention_tc_read_status();
const unsigned int* attention_tc_status_word();      // device address on the current device
}
