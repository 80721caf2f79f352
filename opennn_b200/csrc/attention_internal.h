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
// row_max_out / row_inv_out ([B, H, Sq], optional): per query row, what attention_kv_grad_launch needs to form the weights again.
int attention_fwd_fused_launch(const float* q, const float* k, const float* v, const unsigned char* key_is_pad,
                               float* weights, float* context, float* row_max_out, float* row_inv_out,
                               long long B, long long Sq, long long Sk, long long E, long long H,
                               int causal, float scale, cudaStream_t stream);
// Backward of the same core up to the query gradient: d_scores = P * (dP - rowsum(P * dP)) with dP = dO V^T, and
// d_q = scale * d_scores K (+ its column sums into d_bias_q).  The key and value gradients follow from d_scores
// and the weights with two batched GEMMs.
bool attention_bwd_fused_supported(const float* k, const float* v, const float* weights, const float* context, const float* d_context,
                                   const float* d_scores, const float* d_q, long long B, long long Sq, long long Sk, long long E, long long H);
// delta_out ([B, H, Sq], optional) receives rowsum(dO * O); store_score_gradient = 0 keeps d_scores on the SM (then nothing
// is written to d_scores: the key and value gradients must come from attention_kv_grad_launch, not from GEMMs over it).
int attention_bwd_fused_launch(const float* k, const float* v, const float* weights, const float* context, const float* d_context,
                               float* d_scores, float* d_q, float* d_bias_q, float* delta_out, int store_score_gradient,
                               long long B, long long Sq, long long Sk, long long E, long long H,
                               float scale, cudaStream_t stream);
// dK = scale * dS^T Q and dV = P^T dO by recomputation from Q, K, V, dO and the per-row statistics above (attention_kv_grad.cu);
// their column sums are added to d_bias_k / d_bias_v (optional).  Head size 64, any lengths.
bool attention_kv_grad_supported(const float* q, const float* k, const float* v, const float* d_context, const float* d_k, const float* d_v,
                                 long long B, long long Sq, long long Sk, long long E, long long H);
int attention_kv_grad_launch(const float* q, const float* k, const float* v, const float* d_context, const unsigned char* key_is_pad,
                             const float* row_max, const float* row_inv, const float* delta,
                             float* d_k, float* d_v, float* d_bias_k, float* d_bias_v,
                             long long B, long long Sq, long long Sk, long long E, long long H, int causal, float scale, cudaStream_t stream);
int attention_kv_grad_read_status();
const unsigned int* attention_kv_grad_status_word();
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
