// Internal interface between the GEMM front end (onn_gemm) and its two device paths.
#pragma once
#include <cuda_runtime.h>
#include "../../include/onn_b200.h"

namespace onn
{
// CUDA-core fp32 path: any strides and alignments.
int gemm_simt_launch(const onn_gemm_args& g, cudaStream_t stream);

// tcgen05 (kind::tf32) path.  Needs 16-byte aligned bases, pitches and batch strides.
bool gemm_tc_supported(const onn_gemm_args& g);
int gemm_tc_launch(const onn_gemm_args& g, cudaStream_t stream);
// k_parts > 1: true when the two-CTA kernel can run the product in one launch (else the front end adds up P launches).
bool gemm_tc_takes_parts(const onn_gemm_args& g);
int gemm_tc_read_status();
const unsigned int* gemm_tc_status_word();           // device address on the current device
int gemm_tc_bounded_wait_selftest(int* gave_up_host);

// fp32 CUDA-core kernel for M <= 64 rows against a [K, N] row-major matrix (one decoding step): streams the matrix with
// 8 x N/32 CTAs, cluster reduction over K.  ONN_B200_GEMM_SKINNY=0 turns it off.
bool gemm_skinny_takes(const onn_gemm_args& g);
int gemm_skinny_launch(const onn_gemm_args& g, cudaStream_t stream);
// `count` (at most 4) products that differ in B, bias, C and ldc only, each accepted by gemm_skinny_takes: one launch.
int gemm_skinny_launch_shared_input(const onn_gemm_args* gs, int count, cudaStream_t stream);

// Front end used by the layer code (same as onn_gemm).
int gemm(const onn_gemm_args& g, cudaStream_t stream);
// 0 = automatic, 1 = CUDA-core kernels only, 2 = tensor cores required (onn_gemm_set_mode).
int gemm_mode();
}
