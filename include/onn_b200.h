/* onn_b200.h -- C ABI of libonn_b200.so: sm_100a (B200) kernels for OpenNN's transformer
 * training path (3-D [batch, seq, feature] fp32 tensors; Embedding, MultiHeadAttention,
 * Dense<3>, Normalization3d, Addition<3>, CrossEntropyError3d, Adam).
 *
 * These entry points are what OpenNN's `...Cuda` layer methods would call instead of
 * cuBLAS / cuDNN / opennn/kernel.cu.  Each declaration names the reference code it
 * replaces (paths inside the OpenNN checkout).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless named host_*; tensors are fp32, row-major,
 *     contiguous; token ids and targets are floats holding integers (as in OpenNN);
 *   - weights are [inputs, outputs] (OpenNN's layout); arena sub-buffers are 32-byte aligned;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - every function returns ONN_OK (0) or a negative ONN_ERR_* code, never throws, and
 *     never allocates device memory: scratch is passed in by the caller (`workspace`,
 *     sized by the matching *_workspace_floats query);
 *   - there is no CPU fallback: without a CUDA device every compute call returns ONN_ERR_CUDA.
 *
 * Tensor-core operands.  Contractions run on tcgen05 with kind::tf32 and fp32 accumulation.
 * Operands stay fp32 in HBM; the TMA copy that stages a tile in shared memory rounds each
 * element to the nearest tf32 value (tensor maps of type TFLOAT32), so no conversion pass
 * or shadow copy exists and callers pass ordinary fp32 tensors.
 */
#ifndef ONN_B200_H
#define ONN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ONN_OK                     0
#define ONN_ERR_INVALID_ARGUMENT  -1
#define ONN_ERR_CUDA              -2   /* a CUDA call or launch failed (cudaGetLastError) */
#define ONN_ERR_UNSUPPORTED       -3
#define ONN_ERR_WORKSPACE         -4   /* workspace missing or too small */
#define ONN_ERR_DEVICE_TIMEOUT    -5   /* a bounded device-side wait ran out (see onn_gemm_device_status) */
#define ONN_ERR_NCCL              -6
#define ONN_ERR_LIMIT             -7   /* size beyond a stated fixed maximum */

/* flags */
#define ONN_ACCUMULATE          2u     /* add into the destination instead of overwriting */
#define ONN_DEFER_SOFTMAX       8u     /* Dense "Softmax": leave logits; the loss kernel fuses the softmax */
#define ONN_DELTA_READY        16u     /* Dense backward: dY already holds dY * act'(Y) */
#define ONN_CE_TWO_SWEEPS      32u     /* onn_ce3d_fwd_bwd: keep to the kernel that sweeps each row twice through global memory */

/* activations of Dense<3> used by the transformer (opennn/standard_networks.cpp:745,753,890) */
#define ONN_ACT_LINEAR   0
#define ONN_ACT_RELU     1
#define ONN_ACT_SOFTMAX  2
#define ONN_ACT_SIGMOID  3   /* "Sigmoid" / "Logistic": y = 1 / (1 + exp(-x)) (opennn/layer.h:196-204) */

const char* onn_status_string(int status);
int onn_version(void);

/* ---------------------------------------------------------------------------------------
 * General strided-batched GEMM, the primitive under Dense and MultiHeadAttention.
 * Replaces cublasSgemm / cublasSgemmStridedBatched at opennn/dense_layer.h:1137-1152,
 * 1339-1373 and opennn/multihead_attention_layer.cpp:644-715, 740-756, 804-996.
 *
 *   C[z] = alpha * opA(A[z]) * opB(B[z])  (+ bias)  (relu)  (+ C[z] if ONN_ACCUMULATE)
 *
 * opA(A) is M x K, opB(B) is K x N, C is M x N row-major with leading dimension ldc.
 *   a_major = 0: A stored row-major [M, K] (lda = row pitch);  1: stored [K, M] (transposed).
 *   b_major = 0: B stored row-major [N, K] (i.e. B^T, ldb = row pitch);  1: stored [K, N].
 * Batch z = zo * batch_inner + zi addresses X + zo*stride_outer + zi*stride_inner for each
 * of A, B, C (strides in floats; 0 = shared operand).  bias is per output column (N) or NULL.
 * relu_mask (optional, same layout as C): the result is multiplied by (relu_mask > 0),
 * which fuses the ReLU derivative of the consuming Dense layer into a dX GEMM.
 * relu_bits (optional) is the same mask at one bit per element -- bit n % 32 of the word
 * relu_bits[m * relu_bits_ld + n / 32] -- and costs 1/32 of the memory traffic; relu_bits_out
 * (optional) makes a GEMM write that bit matrix for its own result: bit = (C[m, n] > 0) for the
 * value it stores.  Both need batch 1 and relu_bits_ld >= ceil(N / 32).
 * split_k > 1 splits the reduction over CTAs that accumulate with fp32 reductions; C must
 * then hold the value to accumulate into (zero for a plain product).
 * ------------------------------------------------------------------------------------- */
typedef struct onn_gemm_args
{
    const float* A; const float* B; float* C;
    const float* bias;          /* [N] or NULL */
    const float* relu_mask;     /* [M, N] with ldc / C batch strides, or NULL */
    int64_t M, N, K;
    int64_t lda, ldb, ldc;
    int32_t a_major, b_major;
    int32_t batch_inner, batch_outer;            /* both >= 1 */
    int64_t a_stride_inner, a_stride_outer;
    int64_t b_stride_inner, b_stride_outer;
    int64_t c_stride_inner, c_stride_outer;
    float alpha;
    int32_t relu;               /* apply max(x, 0) after bias */
    int32_t split_k;            /* 0 or 1 = none */
    uint32_t flags;             /* ONN_ACCUMULATE */
    float* colsum_out;          /* optional [N]: column sums of the values written (after bias / ReLU / mask) are */
    int64_t colsum_stride_inner;/* ADDED to colsum_out[zi * colsum_stride_inner + n]; not with split_k.  This is  */
                                /* how a GEMM that produces a layer's delta also produces that layer's bias       */
                                /* gradient (opennn/dense_layer.h:1339-1349 uses a ones-vector GEMM for it).      */
    uint32_t* relu_bits_out;    /* optional [M, relu_bits_ld] words, see above; not with split_k or ONN_ACCUMULATE */
    const uint32_t* relu_bits;  /* optional [M, relu_bits_ld] words, see above; not with split_k */
    int64_t relu_bits_ld;       /* words per row of relu_bits_out / relu_bits */
    int32_t k_parts;            /* 0 or 1 = none; P > 1: C = alpha * sum over p < P of opA(A + p * a_stride_part) * opB(B + p * */
    int64_t a_stride_part;      /* b_stride_part) -- one product whose reduction runs through P operand pairs of equal     */
    int64_t b_stride_part;      /* shape, e.g. dX = dQ Wq^T + dK Wk^T + dV Wv^T in one pass over dX.  Batch 1, no split_k. */
} onn_gemm_args;

int onn_gemm(const onn_gemm_args* args, void* stream);

/* Test hook.  onn_gemm runs on the tcgen05 kernels whenever the operands meet the TMA alignment rules (16-byte aligned
 * bases and pitches); operands that do not are served by a CUDA-core fp32 kernel.  A test can pin the next onn_gemm
 * calls to one of the two to cross-check them against each other: 0 = the rule above (the only setting a product
 * path uses), 1 = the CUDA-core fp32 kernel for everything, 2 = tcgen05 or ONN_ERR_UNSUPPORTED. */
int onn_gemm_set_mode(int mode);
/* Key and value gradients of onn_mha_bwd: 0 (the default) = two batched GEMMs over the stored weights P and the score
 * gradient dS, as the reference computes them (opennn/multihead_attention_layer.cpp:843-887); 1 = where the fused
 * attention kernels serve the layer (head size 64, at most 256 keys), one kernel that forms P and dS again on the SM
 * from Q, K, V, dO and the per-row softmax statistics the forward pass left in its workspace, so that dS is never
 * written and P is not read a third time.  Measured on B200 the second is not faster yet (same results within tf32
 * rounding), which is why it is not the default; the environment variable ONN_B200_ATTENTION_KV_GRAD=1 selects it
 * for a whole process.  A forward/backward pair must run under one setting.  Returns the previous setting. */
int onn_mha_set_kv_grad_by_recomputation(int enabled);
/* 0, or ONN_ERR_DEVICE_TIMEOUT if a kernel of this library (tcgen05 GEMM, fused attention, staged cross-entropy)
 * gave up on a bounded barrier wait since the last call.  The status words are read back and cleared; the call
 * synchronises the whole device first, so it sees every kernel launched before it on any stream. */
int onn_gemm_device_status(void);
/* The same information in stream order and without a host synchronisation: enqueues on `stream` a one-thread kernel
 * that writes the OR of the status words to device_word[0] (0 = no wait has run out).  It sees the kernels that
 * precede it on `stream`; nothing is cleared (onn_gemm_device_status clears).  A caller copies the word to pinned
 * memory with its other read-backs, or hands it to onn_adam_guarded so that a step whose kernels gave up does not
 * reach the parameters.  No counterpart in the reference. */
int onn_device_status_gather(uint32_t* device_word, void* stream);
/* How many SMs the persistent kernels (tcgen05 GEMMs, fused attention, staged cross-entropy: one CTA or CTA pair per
 * SM holding most of its shared memory) occupy from the next launch on: 0 or >= 148 = all of them (the default).
 * A data-parallel caller lowers it while NCCL reduces a gradient bucket, so that NCCL's CTAs find free SMs instead of
 * waiting for a kernel boundary.  Takes effect in stream order (it is read when a kernel is launched). */
int onn_set_sm_limit(int sms);
/* Work items of the persistent kernels (two-CTA GEMM, fused attention): 0 (default) = every CTA owns a fixed share
 * of the launch's tiles; 1 = the CTAs take tiles from a per-launch counter in the order they ask.  The second costs
 * 2-3 % when the kernel has the GPU to itself and saves up to 40 % when another kernel holds some SMs (with fixed shares
 * a CTA that starts late -- its SM was busy with one of NCCL's CTAs -- makes the whole launch wait for its share; measured:
 * FFN GEMM 0.195 ms alone, 0.316 ms with 16 SMs held, 0.212 ms with the counter).  The data-parallel trainer turns it on
 * for as long as it has a communicator.  Takes effect at the next launch; ONN_B200_DYNAMIC_WORK=0 / 1 in the
 * environment overrides the call.  Returns the previous setting. */
int onn_set_dynamic_work(int enabled);
/* Measurement aid for the above (no counterpart in the reference): a kernel of `sms` CTAs that each occupy one SM's
 * shared memory and spin for `cycles` clock cycles (at most 2^26, about 35 ms), then end by themselves -- what a
 * resident CTA of another library is to the persistent kernels.  Launch it on a second stream, then time kernels on
 * the first (tests/test_layers_gpu.py, bench.py --profile-kernel contention). */
int onn_selftest_hold_sms(int sms, int64_t cycles, void* stream);
/* Failure-detection self-test (no counterpart in the reference): runs a one-thread kernel that waits, with a
 * 1 ms limit, on a barrier nothing ever signals.  *gave_up receives 1 when the wait ran out as it must; the
 * kernel returns normally, the context stays usable, and the next onn_gemm_device_status() reports
 * ONN_ERR_DEVICE_TIMEOUT once.  This is the mechanism every wait of the tcgen05 kernels uses (limit ~1 s). */
int onn_selftest_bounded_wait(int* gave_up);
/* Number of kernels this library launched since load (all entry points). */
uint64_t onn_launch_count(void);
/* For a caller that replays launches it captured into a CUDA graph: the library only sees the capture, so the
 * caller adds the captured count on each replay to keep the figure above true. */
void onn_launch_count_add(uint64_t launches);

/* ---------------------------------------------------------------------------------------
 * Embedding.  Forward replaces embedding_forward_kernel (opennn/kernel.cu:714-761, called
 * from opennn/embedding_layer.cpp:331-367); CPU semantics opennn/embedding_layer.cpp:147-186:
 *   out[b,s,:] = W[id,:] * sqrt(E) (if scale) + PE[s,:] (if add_pe and id > 0);
 *   id = (integer) ids[b,s]; id outside [0, V) gives a zero row.
 * The multiply and the add are separate roundings (no FMA), matching the CPU path bit for bit.
 * row_is_zero (optional, [B*S] bytes) receives 1 where every output feature has |x| <= 1e-7:
 * the key-padding flag MultiHeadAttention derives from its source input
 * (opennn/multihead_attention_layer.cpp:574-603).
 * ------------------------------------------------------------------------------------- */
int onn_embedding_fwd(const float* ids, const float* W, const float* PE, float* out,
                      uint8_t* row_is_zero,
                      int64_t B, int64_t S, int64_t E, int64_t V,
                      int scale, int add_pe, uint32_t flags, void* stream);

/* Token ids as 32-bit integers (what a data feed holds; opennn/dataset.cpp:4397-4494 stages them as floats) to the
 * floats-holding-integers the layers and the loss read.  Exact for |id| < 2^24. */
int onn_ids_to_float(const int32_t* ids, float* out, int64_t n, void* stream);

/* Backward replaces embedding_backward_kernel (opennn/kernel.cu:764-800) plus the fan-in
 * sum Layer::add_gradients (opennn/layer.cpp:447-457); CPU semantics
 * opennn/embedding_layer.cpp:193-226:  dW[id,:] += (dY + dY2)[b,s,:] * sqrt(E) for 0 < id < V.
 * dW must be zero on entry (the training loop zeroes the gradient arena each step);
 * dY2 may be NULL. */
int onn_embedding_bwd(const float* ids, const float* dY, const float* dY2, float* dW,
                      int64_t B, int64_t S, int64_t E, int64_t V, int scale, void* stream);

/* ---------------------------------------------------------------------------------------
 * Normalization3d (LayerNorm over the last dimension) with the preceding Addition<3> fused.
 * Forward replaces addition_kernel + layernorm_forward_kernel (opennn/kernel.cu:691-699,
 * 1141-1204; opennn/normalization_layer_3d.cpp:198-215); CPU semantics
 * opennn/normalization_layer_3d.cpp:87-125:
 *   x = A (+ R);  mean = mean(x);  std = sqrt(mean((x-mean)^2) + eps);  y = gamma*(x-mean)/std + beta.
 * R (the residual) may be NULL; `sum` (optional) receives x, the Addition layer's output;
 * mean and inv_std are [rows]; row_is_zero as in onn_embedding_fwd (optional).
 * ------------------------------------------------------------------------------------- */
int onn_layernorm_fwd(const float* A, const float* R, const float* gamma, const float* beta,
                      float* Y, float* sum, float* mean, float* inv_std, uint8_t* row_is_zero,
                      int64_t rows, int64_t E, float eps, uint32_t flags, void* stream);

/* Backward replaces layernorm_backward_kernel (opennn/kernel.cu:1207-1269) and the fan-in
 * sum; CPU semantics opennn/normalization_layer_3d.cpp:128-188.  dY2, dY3 (optional) are
 * further consumer gradients summed on load.  X is the layer input (A + R).  dX is the
 * gradient for the layer input; with the Addition fused both addends receive this same
 * tensor (opennn/addition_layer.h:79-90).  workspace: onn_layernorm_bwd_workspace_floats.
 * dX_colsum (optional, [E]): the column sums of dX are ADDED to it.  When one addend of the fused Addition is
 * the output of a Dense or MultiHeadAttention layer with no other consumer, that layer's output gradient IS dX
 * and these sums are its (projection) bias gradient, which then needs no pass of its own over dX. */
size_t onn_layernorm_bwd_workspace_floats(int64_t rows, int64_t E);
int onn_layernorm_bwd(const float* dY, const float* dY2, const float* dY3, const float* X,
                      const float* mean, const float* inv_std, const float* gamma,
                      float* dX, float* dgamma, float* dbeta, float* dX_colsum,
                      int64_t rows, int64_t E, float* workspace, uint32_t flags, void* stream);

/* No counterpart in the reference.  The same computation as onn_layernorm_bwd for a caller that
 * holds nothing but the layer's inputs and outputs and cannot obtain device memory of its own:
 * code running inside OpenNN's `back_propagate(...) const` overrides sees only the views that the
 * stock propagation structures linked at set-up time (there is no slot for a scratch view unless
 * the structures are changed), and hosts that hand out all device memory once at start-up refuse
 * later cudaMalloc calls.  This entry point therefore takes no workspace and allocates nothing:
 * its partial column sums go to a fixed 2.3 MiB buffer inside the library (held by every GPU that
 * loads the library, until exit).
 *   - E must not exceed ONN_LAYERNORM_BWD_STATIC_MAX_E; larger rows return ONN_ERR_LIMIT.
 *   - The first call on each device looks up the buffer's device address (one
 *     cudaGetSymbolAddress with that device current); make that first call before any stream
 *     capture begins.
 *   - All calls share the one buffer: two calls whose kernels can overlap on the GPU (different
 *     streams, no ordering between them) race on it and corrupt each other's dgamma / dbeta.
 *     Calls on one stream, or ordered by events, are safe.  The buffer keeps the last call's
 *     partial sums; nothing in it needs clearing between calls. */
#define ONN_LAYERNORM_BWD_STATIC_MAX_E 1024
int onn_layernorm_bwd_static(const float* dY, const float* dY2, const float* dY3, const float* X,
                             const float* mean, const float* inv_std, const float* gamma,
                             float* dX, float* dgamma, float* dbeta,
                             int64_t rows, int64_t E, uint32_t flags, void* stream);

/* Addition<3> stand-alone: out = a + b.  Replaces addition_kernel (opennn/kernel.cu:691-699). */
int onn_add(const float* a, const float* b, float* out, int64_t n, uint32_t flags, void* stream);

/* ---------------------------------------------------------------------------------------
 * Dense<3>.  Forward replaces cublasSgemm + cudnnAddTensor + cudnnActivationForward /
 * cudnnSoftmaxForward (opennn/dense_layer.h:1117-1232); CPU semantics dense_layer.h:767-813:
 *   Y = act(X W + b), X [rows, in], W [in, out], b [out].
 * ONN_ACT_SOFTMAX normalises each row unless ONN_DEFER_SOFTMAX is set (then Y holds logits
 * for onn_ce3d_fwd_bwd).
 * relu_bits (optional, ONN_ACT_RELU only, [rows, onn_relu_bits_words_per_row(out)] words): receives
 * (Y > 0) at one bit per element, for the onn_dense_bwd call of the layer that consumes Y.
 * ------------------------------------------------------------------------------------- */
int64_t onn_relu_bits_words_per_row(int64_t features);      /* ceil(features / 32) */
int onn_dense_fwd(const float* X, const float* W, const float* b, float* Y, uint32_t* relu_bits,
                  int64_t rows, int64_t in, int64_t out, int activation,
                  uint32_t flags, void* stream);

/* Backward replaces cudnnActivationBackward + 3 GEMMs (opennn/dense_layer.h:1235-1374);
 * CPU semantics dense_layer.h:816-866:  delta = dY * act'(Y) (ReLU: Y > 0; Sigmoid: Y (1 - Y); Linear and
 * Softmax: delta = dY), dW = X^T delta, db = column sums of delta, dX = delta W^T.
 * dY is overwritten with delta for ReLU and Sigmoid (as the reference does in place) unless
 * ONN_DELTA_READY says it already holds delta.  dX may be NULL (ONN_ACCUMULATE adds into it).
 * dW and db are ACCUMULATED into (the gradient arena is zeroed once per step).
 * dX_relu_mask (optional, [rows, in]): dX is multiplied by (mask > 0), i.e. the ReLU
 * derivative of the layer that produced X, saving that layer a pass over its gradient.
 * dX_relu_bits (optional): the same mask as written by that layer's onn_dense_fwd(relu_bits);
 * give one of the two.  The bit form reads 1/32 of the bytes and is the fast one.
 * dX_colsum (optional, [in]): the column sums of dX (after the mask) are ADDED to it -- that is the
 * bias gradient of the layer that produced X, which may then pass db = NULL in its own call.
 * db may be NULL (bias gradient not wanted here). */
/* Several Linear Dense forward passes over the same input: Y[i] = X W[i] + b[i], i < count <= 4, row pitch ldy[i] >= out
 * (the query, key and value projections of a self-attention layer on one decoding position, whose key and value rows
 * go straight into their cache slots).  One launch when rows <= 64 and the few-rows kernel takes the shape, else one
 * product after the other.  b may be NULL (no biases). */
int onn_dense_fwd_shared_input(const float* X, const float* const* W, const float* const* b, float* const* Y,
                               const int64_t* ldy, int count, int64_t rows, int64_t in, int64_t out, void* stream);
int onn_dense_bwd(const float* X, const float* W, const float* Y, float* dY,
                  float* dW, float* db, float* dX, const float* dX_relu_mask, const uint32_t* dX_relu_bits,
                  float* dX_colsum,
                  int64_t rows, int64_t in, int64_t out, int activation,
                  uint32_t flags, void* stream);

/* ---------------------------------------------------------------------------------------
 * Pooling3d: pooling over the sequence in front of a classification head.  Replaces
 * pooling3d_{max,avg}_{forward,backward}_kernel (opennn/kernel.cu:995-1136, called from
 * opennn/pooling_layer_3d.cpp:235-300); CPU semantics opennn/pooling_layer_3d.cpp:77-232.
 * x [B, S, E] -> y [B, E].  method 0 = MaxPooling: the maximum over the sequence, the first position winning ties;
 * argmax ([B, E], optional for inference) keeps that position for the backward pass.  method 1 = AveragePooling:
 * the mean over the rows that are not padding (a padding row has every feature exactly zero), zeros for a sample
 * of nothing but padding; row_is_valid ([B * S] bytes) and valid_count ([B]) are written by the forward pass and read
 * by the backward pass.  The backward pass writes all of dx (zeros where nothing flows).  Results are bit-identical to
 * the CPU path (same order of additions, same division).
 * ------------------------------------------------------------------------------------- */
#define ONN_POOL_MAX      0
#define ONN_POOL_AVERAGE  1
int onn_pooling3d_fwd(const float* x, float* y, int32_t* argmax, uint8_t* row_is_valid, int32_t* valid_count,
                      int64_t B, int64_t S, int64_t E, int method, void* stream);
int onn_pooling3d_bwd(const float* dy, const int32_t* argmax, const uint8_t* row_is_valid, const int32_t* valid_count,
                      float* dx, int64_t B, int64_t S, int64_t E, int method, void* stream);

/* Row softmax over the last dimension, in place (opennn/layer.cpp:338-371). */
int onn_softmax_rows(float* Y, int64_t rows, int64_t cols, void* stream);

/* ---------------------------------------------------------------------------------------
 * MultiHeadAttention.  Forward replaces the 17 launches of
 * opennn/multihead_attention_layer.cpp:624-776 (4 projections, transposes, strided-batched
 * QK^T, mask kernels, cudnnSoftmaxForward, PV, output projection); CPU semantics
 * multihead_attention_layer.cpp:183-282.
 *   Xq [B,Sq,E]; Xs [B,Sk,E] (pass Xq again for self-attention); W* [E,E] in x out, head h
 *   owns columns h*hd..; Y [B,Sq,E].  Key padding: source rows with all |x| <= 1e-7 get
 *   score -1e9; causal: keys after the query get -inf.
 * source_row_is_zero (optional, [B*Sk] bytes): flags from the producer of Xs; NULL makes
 * the call compute them.
 * The forward workspace doubles as the saved state for onn_mha_bwd (Q, K, V, attention
 * weights, concatenated head outputs) and must be kept until then.
 * ------------------------------------------------------------------------------------- */
typedef struct onn_mha_params
{
    const float* Wq; const float* bq; const float* Wk; const float* bk;
    const float* Wv; const float* bv; const float* Wo; const float* bo;
} onn_mha_params;

typedef struct onn_mha_grads
{
    float* dWq; float* dbq; float* dWk; float* dbk;
    float* dWv; float* dbv; float* dWo; float* dbo;
} onn_mha_grads;

size_t onn_mha_fwd_workspace_floats(int64_t B, int64_t Sq, int64_t Sk, int64_t E, int64_t H);
size_t onn_mha_bwd_workspace_floats(int64_t B, int64_t Sq, int64_t Sk, int64_t E, int64_t H);

int onn_mha_fwd(const float* Xq, const float* Xs, const onn_mha_params* params,
                const uint8_t* source_row_is_zero, float* Y,
                int64_t B, int64_t Sq, int64_t Sk, int64_t E, int64_t H, int causal,
                float* fwd_workspace, uint32_t flags, void* stream);

/* Backward replaces opennn/multihead_attention_layer.cpp:779-1018; CPU semantics :285-454,
 * 493-553.  Parameter gradients are ACCUMULATED into (zeroed arena).  Self-attention
 * (Xs == Xq): dXq receives dXq + dXk + dXv and dXs must be NULL.  Cross-attention: dXs
 * receives dXk + dXv; with ONN_ACCUMULATE it is added into dXs instead (the encoder output
 * feeds every decoder layer, so the fan-in sum of opennn/layer.cpp:447-457 happens here). */
int onn_mha_bwd(const float* Xq, const float* Xs, const onn_mha_params* params,
                const float* fwd_workspace, const float* dY,
                const onn_mha_grads* grads, float* dXq, float* dXs,
                int64_t B, int64_t Sq, int64_t Sk, int64_t E, int64_t H, int causal,
                float* bwd_workspace, uint32_t flags, void* stream);

/* Attention-weight view inside the forward workspace ([B,H,Sq,Sk]), for tests and tools. */
const float* onn_mha_attention_weights(const float* fwd_workspace,
                                       int64_t B, int64_t Sq, int64_t Sk, int64_t E, int64_t H);

/* ---------------------------------------------------------------------------------------
 * CrossEntropyError3d.  One fused pass replaces the softmax of the output layer
 * (opennn/layer.cpp:338-371 / cudnnSoftmaxForward) and
 * cross_entropy_3d_multiple_{forward,counts,backward}_kernel + cudnnReduceTensor + two
 * blocking D2H copies (opennn/kernel.cu:273-347, 466-499; opennn/cross_entropy_error_3d.cpp:
 * 370-454, 498-528).  CPU semantics cross_entropy_error_3d.cpp:78-136, 154-247:
 *   active = 0 < (integer) target < V;  p = softmax(logits);
 *   error = sum over active of -log(p[target] + FLT_EPSILON) / #active;
 *   accuracy = #(argmax p == target) / #active;
 *   gradient wrt logits = (p - onehot) / #active on active tokens, 0 elsewhere.
 * onn_ce3d_count_active writes #active of `targets` to counts[0] (float, device).  With
 * several ranks the counts are summed across ranks before onn_ce3d_fwd_bwd so every rank
 * scales by the global count.
 * onn_ce3d_fwd_bwd: logits [rows, V] is overwritten in place with the gradient
 * (inputs_are_probabilities != 0: the buffer already holds probabilities, as a plain
 * Softmax Dense layer leaves them).  probabilities_out (optional) receives p.
 * stats (device, 4 floats) receives {sum of -log terms, #correct, #active(local), 0};
 * row_scratch is [2*rows] floats.
 * Rows of 4096 to 35712 logits (a multiple of 4, 16-byte aligned, no probabilities_out) are held in registers by a
 * persistent kernel that is fed through shared memory, so each logit crosses HBM once in and once out; other shapes, and calls with
 * ONN_CE_TWO_SWEEPS in flags, take one CTA per row that sweeps the row twice (the second sweep mostly from L2).
 * ------------------------------------------------------------------------------------- */
int onn_ce3d_count_active(const float* targets, int64_t rows, int64_t V, float* counts, void* stream);
int onn_ce3d_fwd_bwd(float* logits, const float* targets, const float* active_count,
                     float* probabilities_out, float* stats, float* row_scratch,
                     int64_t rows, int64_t V, int inputs_are_probabilities,
                     uint32_t flags, void* stream);

/* CrossEntropyError2d with several classes (the loss of the text-classification network).  Replaces
 * calculate_multiple_cross_entropy_cuda + the gradient kernel (opennn/cross_entropy_error.cpp:217-300); CPU semantics
 * opennn/cross_entropy_error.cpp:58-77 and 114-134: error = -sum(t * log(y + FLT_EPSILON)) / rows, gradient
 * (y - t) / rows (the softmax Jacobian is folded in; the Softmax Dense layer passes it on unchanged).
 * probabilities [rows, classes] are overwritten with the gradient; targets [rows, classes] (one-hot or soft);
 * stats (device, 2 floats) receives {error, rows}; row_scratch is [rows] floats. */
int onn_ce2d_fwd_bwd(float* probabilities, const float* targets, float* stats, float* row_scratch,
                     int64_t rows, int64_t classes, void* stream);
/* The same loss with ONE output per sample (a Dense<2> "Sigmoid" head): opennn/cross_entropy_error.cpp:36-55 and 90-110.
 * error = -sum(t log y' + (1 - t) log(1 - y')) / rows with y' = y clipped to [eps, 1 - eps] (NaN or infinity -> 10);
 * outputs [rows] are overwritten with the gradient g = (-t / (y + eps) + (1 - t) / (1 - y + eps)) / rows, which the
 * Sigmoid layer's onn_dense_bwd multiplies by y (1 - y) -- but y is gone once g sits in its place.  A caller whose
 * output buffer doubles as the gradient buffer passes fold_sigmoid != 0: outputs then receive delta = g * (y (1 - y))
 * and that layer's onn_dense_bwd takes ONN_DELTA_READY.  stats (device, 2 floats) receives {error, rows};
 * row_scratch [rows]. */
int onn_ce2d_binary_fwd_bwd(float* outputs, const float* targets, float* stats, float* row_scratch, int64_t rows,
                            int fold_sigmoid, void* stream);

/* Greedy decoding step (the body of the loop at opennn/standard_networks.cpp:1016-1034, which reads the distribution
 * back to the host and scans it there): for each of B samples the arg-max -- first index on ties -- of
 * probabilities[b, position, :] ([B, S, V]) becomes ids[b, position + 1] (floats holding integers, [B, S]) unless
 * finished[b] is set; finished[b] is set when that token is end_id. */
int onn_greedy_next_token(const float* probabilities, float* ids, int* finished, int64_t B, int64_t S, int64_t V,
                          int64_t position, int end_id, void* stream);
/* The same step when only the current position was computed: probabilities is [B, V] and the token goes to
 * ids[b, write_position]. */
int onn_greedy_next_token_rows(const float* probabilities, float* ids, int* finished, int64_t B, int64_t S, int64_t V,
                               int64_t write_position, int end_id, void* stream);

/* The same step from LOGITS [B, V] (a Dense "Softmax" layer run with ONN_DEFER_SOFTMAX): softmax and arg-max in one
 * kernel.  The probabilities are formed exactly as onn_softmax_rows forms them, compared and not stored, so the token is
 * the one onn_softmax_rows + onn_greedy_next_token_rows give; `logits` is left unchanged. */
int onn_greedy_next_token_logits(const float* logits, float* ids, int* finished, int64_t B, int64_t S, int64_t V,
                                 int64_t write_position, int end_id, void* stream);

/* Attention of ONE query row per sample against keys and values kept from earlier decoding steps (no counterpart in
 * the reference, whose decoding loop recomputes every position for every token): q [B, E] (projected), k_cache and
 * v_cache [B, S_cache, E] of which the first `length` rows are valid, key_is_pad bytes or NULL: the flag of key j of
 * sample b is key_is_pad[b * pad_stride_sample + j * pad_stride_key] ([B, S_cache]: strides S_cache and 1; one row of B
 * flags per position, as a producing kernel writes them: strides 1 and B); a set flag overwrites the score with -1e9 as
 * in onn_mha_fwd.  out [B, E] = concatenated head outputs before the output projection.  Scale 1/sqrt(E/H).  fp32. */
int onn_decode_attention(const float* q, const float* k_cache, const float* v_cache, const uint8_t* key_is_pad,
                         int64_t pad_stride_sample, int64_t pad_stride_key, float* out,
                         int64_t B, int64_t S_cache, int64_t length, int64_t E, int64_t H, void* stream);
/* flags[r] = 1 where every feature of row r has |x| <= 1e-7: the key-padding rule of MultiHeadAttention
 * (opennn/multihead_attention_layer.cpp:574-603) for a caller that keeps its own key cache. */
int onn_rows_are_zero(const float* X, uint8_t* flags, int64_t rows, int64_t E, void* stream);

/* ---------------------------------------------------------------------------------------
 * AdaptiveMomentEstimation.  Replaces adam_update_kernel (opennn/kernel.cu:6-68) and adds
 * the global-norm clip only the CPU path has (opennn/adaptive_moment_estimation.cpp:444-473):
 *   norm = ||g||;  g' = g * clip/norm if clip > 0 and norm > clip;
 *   m = b1 m + (1-b1) g';  v = b2 v + (1-b2) g'^2;
 *   p -= lr * (m / bc1) / (sqrt(v / bc2) + eps).
 * onn_grad_sqnorm writes sum(g^2) to sqnorm[0] (device) deterministically; workspace is
 * onn_grad_sqnorm_workspace_floats(n) floats.
 * onn_adam reads the squared norm from device memory (no host sync) and zeroes g for the
 * next step when zero_grad != 0.  grad_scale multiplies g before
 * everything else (1/world for averaged all-reduces; 1 otherwise).
 * ------------------------------------------------------------------------------------- */
size_t onn_grad_sqnorm_workspace_floats(int64_t n);
int onn_grad_sqnorm(const float* g, int64_t n, float* sqnorm, float* workspace, void* stream);
int onn_adam(float* p, float* m, float* v, float* g, int64_t n,
             float lr, float beta1, float beta2, float eps, float bc1, float bc2,
             float clip_norm, const float* sqnorm, float grad_scale, int zero_grad, void* stream);
/* onn_adam that leaves p, m, v and g untouched when skip_if_nonzero[0] != 0 (device word, see
 * onn_device_status_gather; NULL = plain onn_adam). */
int onn_adam_guarded(float* p, float* m, float* v, float* g, int64_t n,
                     float lr, float beta1, float beta2, float eps, float bc1, float bc2,
                     float clip_norm, const float* sqnorm, float grad_scale, int zero_grad,
                     const uint32_t* skip_if_nonzero, void* stream);

/* ---------------------------------------------------------------------------------------
 * Data-parallel gradient exchange (no counterpart in the reference, which is single-GPU):
 * NCCL collectives (sum) on contiguous fp32 buffers on a dedicated communication stream.
 * One process per GPU.  The 128-byte unique id is created on rank 0 with onn_dp_unique_id
 * and handed to the other ranks by the caller (any out-of-band channel).
 * ncclCommInitRank has no time limit: check on the host that every rank is present before
 * calling onn_dp_init (the Python binding does, with a bounded rendezvous).
 * ------------------------------------------------------------------------------------- */
typedef struct onn_dp_comm onn_dp_comm;
int onn_dp_unique_id(void* host_id128);
int onn_dp_init(onn_dp_comm** comm, const void* host_id128, int world, int rank);
/* The same with a cap on the CTAs (SMs) NCCL's kernels may use; 0 = NCCL's own choice. */
int onn_dp_init_config(onn_dp_comm** comm, const void* host_id128, int world, int rank, int max_ctas);
int onn_dp_world(const onn_dp_comm* comm);
int onn_dp_rank(const onn_dp_comm* comm);
/* Enqueue all-reduce(sum) of buf[0..n) in place on the comm stream after `after_stream`'s
 * current work; onn_dp_wait makes `stream` wait for everything enqueued so far. */
int onn_dp_allreduce(onn_dp_comm* comm, float* buf, int64_t n, void* after_stream);
/* Reduce-scatter: send holds world * recv_count floats; recv receives the sum over ranks of this rank's
 * recv_count-float part.  All-gather: every rank contributes send_count floats, recv receives world * send_count
 * (rank r's part at r * send_count; send may lie inside recv at that place).  Ordered like onn_dp_allreduce. */
int onn_dp_reduce_scatter(onn_dp_comm* comm, const float* send, float* recv, int64_t recv_count, void* after_stream);
int onn_dp_all_gather(onn_dp_comm* comm, const float* send, float* recv, int64_t send_count, void* after_stream);
/* Zero buf[0..n) on the comm stream after the collectives enqueued so far (a gradient bucket that has been
 * reduced is cleared for the next step off the compute stream). */
int onn_dp_zero(onn_dp_comm* comm, float* buf, int64_t n);
int onn_dp_wait(onn_dp_comm* comm, void* stream);
/* Finer-grained waits: onn_dp_mark records position `slot` (0 .. ONN_DP_MARKS - 1) on the comm stream after what has
 * been enqueued so far; onn_dp_wait_mark makes `stream` wait for the work before that position only (the comm stream
 * runs in order, so a later mark implies the earlier ones).  The trainer marks each parameter bucket's all-gather and
 * lets the next step's forward pass wait layer by layer, so the gathers run under it.  A slot must have been marked
 * before it is waited for; marking it again moves it. */
#define ONN_DP_MARKS 64
int onn_dp_mark(onn_dp_comm* comm, int slot);
int onn_dp_wait_mark(onn_dp_comm* comm, int slot, void* stream);
/* After a failure between collectives on this rank (an exception half-way through a step) the ranks no longer
 * agree on which collective comes next: mark the communicator, and every later call returns ONN_ERR_NCCL instead
 * of joining a collective the peers are not in.  A failed NCCL call marks it by itself. */
int onn_dp_mark_failed(onn_dp_comm* comm);
int onn_dp_finalize(onn_dp_comm* comm);

#ifdef __cplusplus
}
#endif

#endif /* ONN_B200_H */
