// Layer-level entry points built from the GEMM primitive and the row kernels:
// Dense<3> forward/backward and MultiHeadAttention forward/backward.
#include <math.h>
#include <atomic>
#include <cstdlib>

#include "common.cuh"
#include "gemm_internal.h"
#include "attention_internal.h"
#include "launch_counter.h"

namespace onn
{

int launch_source_row_is_zero(const float* X, uint8_t* flags, long long rows, int E, cudaStream_t s);
int launch_attention_softmax(float* scores, const uint8_t* key_is_pad, long long B, int H, int Sq, int Sk, int causal, cudaStream_t s);
int launch_attention_softmax_bwd(const float* P, float* dP, long long rows, int Sk, cudaStream_t s);
int launch_colsum_accumulate(const float* D, long long rows, long long cols, long long ld, float* out, cudaStream_t s);
int launch_relu_delta(float* dY, const float* Y, long long n, cudaStream_t s);
int launch_sigmoid(float* Y, long long n, cudaStream_t s);
int launch_sigmoid_delta(float* dY, const float* Y, long long n, cudaStream_t s);

#define ONN_TRY(expr) do { const int status_ = (expr); if(status_ != ONN_OK) return status_; } while(0)

static size_t pad64(size_t floats) { return (floats + 63) & ~(size_t)63; }   // 256-byte granules

static onn_gemm_args plain_gemm(const float* A, int a_major, long long lda, const float* B, int b_major, long long ldb,
                                float* C, long long ldc, long long M, long long N, long long K)
{
    onn_gemm_args g = {};
    g.A = A; g.B = B; g.C = C;
    g.M = M; g.N = N; g.K = K;
    g.lda = lda; g.ldb = ldb; g.ldc = ldc;
    g.a_major = a_major; g.b_major = b_major;
    g.batch_inner = 1; g.batch_outer = 1;
    g.alpha = 1.0f;
    return g;
}

// Split the reduction when the output has too few tiles to occupy the SMs (weight
// gradients: small [in, out] outputs with a reduction over every token).
static int choose_split_k(long long M, long long N, long long K)
{
    // work units: 256 x 256 tiles on CTA pairs (74 of them) for large aligned outputs, else 128 x BN tiles on 148 CTAs
    const bool pair = M >= 512 && N >= 256 && M % 32 == 0 && N % 32 == 0;
    const long long bn = N > 128 ? 256 : (N > 64 ? 128 : 64);
    const long long tiles = pair ? ((M + 255) / 256) * ((N + 255) / 256) : ((M + 127) / 128) * ((N + bn - 1) / bn);
    const long long units = pair ? sm_limit() / 2 : sm_limit();
    if(tiles >= 4 * units || K < 1024) return 1;
    // pick the split count whose last wave is fullest; every extra split costs one more pass of
    // reduce-adds over the output, so ties go to the smaller count
    const long long max_splits = K / 512 < 16 ? K / 512 : 16;
    int best = 1;
    double best_score = 0.0;
    for(long long s = 1; s <= max_splits; s++)
    {
        const long long work = tiles * s;
        const long long waves = (work + units - 1) / units;
        const double score = (double)work / (double)(waves * units) - 0.004 * (double)s;
        if(score > best_score + 1e-9) { best_score = score; best = (int)s; }
    }
    return best;
}

// dW += X^T D (X [rows, in], D [rows, out]) and db += column sums of D.
static int weight_gradients(const float* X, const float* D, float* dW, float* db,
                            long long rows, long long in, long long out, cudaStream_t s)
{
    onn_gemm_args g = plain_gemm(X, 1, in, D, 1, out, dW, out, in, out, rows);
    g.split_k = choose_split_k(in, out, rows);
    if(g.split_k <= 1) g.flags = ONN_ACCUMULATE;
    ONN_TRY(gemm(g, s));
    if(db) ONN_TRY(launch_colsum_accumulate(D, rows, out, out, db, s));
    return ONN_OK;
}

}  // namespace onn

using namespace onn;

// ---------------------------------------------------------------------------------------
// Dense<3>
// ---------------------------------------------------------------------------------------

extern "C" int64_t onn_relu_bits_words_per_row(int64_t features) { return (features + 31) / 32; }

extern "C" int onn_dense_fwd(const float* X, const float* W, const float* b, float* Y, uint32_t* relu_bits,
                             int64_t rows, int64_t in, int64_t out, int activation,
                             uint32_t flags, void* stream)
{
    ONN_CHECK_ARG(X && W && Y && rows > 0 && in > 0 && out > 0);
    ONN_CHECK_ARG(activation == ONN_ACT_LINEAR || activation == ONN_ACT_RELU || activation == ONN_ACT_SOFTMAX || activation == ONN_ACT_SIGMOID);
    ONN_CHECK_ARG(!relu_bits || activation == ONN_ACT_RELU);
    cudaStream_t s = (cudaStream_t)stream;
    onn_gemm_args g = plain_gemm(X, 0, in, W, 1, out, Y, out, rows, out, in);
    g.bias = b;
    g.relu = activation == ONN_ACT_RELU;
    g.relu_bits_out = relu_bits;
    g.relu_bits_ld = onn_relu_bits_words_per_row(out);
    ONN_TRY(gemm(g, s));
    if(activation == ONN_ACT_SOFTMAX && !(flags & ONN_DEFER_SOFTMAX)) ONN_TRY(onn_softmax_rows(Y, rows, out, stream));
    if(activation == ONN_ACT_SIGMOID) ONN_TRY(launch_sigmoid(Y, rows * out, s));
    return ONN_OK;
}

extern "C" int onn_dense_fwd_shared_input(const float* X, const float* const* W, const float* const* b, float* const* Y,
                                          const int64_t* ldy, int count, int64_t rows, int64_t in, int64_t out, void* stream)
{
    ONN_CHECK_ARG(X && W && Y && ldy && count >= 1 && count <= 4 && rows > 0 && in > 0 && out > 0);
    cudaStream_t s = (cudaStream_t)stream;
    onn_gemm_args g[4];
    bool one_launch = gemm_mode() == 0;
    for(int i = 0; i < count; i++)
    {
        ONN_CHECK_ARG(W[i] && Y[i] && ldy[i] >= out);
        g[i] = plain_gemm(X, 0, in, W[i], 1, out, Y[i], ldy[i], rows, out, in);
        g[i].bias = b ? b[i] : nullptr;
        one_launch = one_launch && gemm_skinny_takes(g[i]);
    }
    if(one_launch) return gemm_skinny_launch_shared_input(g, count, s);
    for(int i = 0; i < count; i++) ONN_TRY(gemm(g[i], s));
    return ONN_OK;
}

extern "C" int onn_dense_bwd(const float* X, const float* W, const float* Y, float* dY,
                             float* dW, float* db, float* dX, const float* dX_relu_mask, const uint32_t* dX_relu_bits,
                             float* dX_colsum,
                             int64_t rows, int64_t in, int64_t out, int activation,
                             uint32_t flags, void* stream)
{
    ONN_CHECK_ARG(X && W && dY && dW && rows > 0 && in > 0 && out > 0);
    ONN_CHECK_ARG(activation == ONN_ACT_LINEAR || activation == ONN_ACT_RELU || activation == ONN_ACT_SOFTMAX || activation == ONN_ACT_SIGMOID);
    ONN_CHECK_ARG((activation != ONN_ACT_RELU && activation != ONN_ACT_SIGMOID) || Y);
    cudaStream_t s = (cudaStream_t)stream;

    // delta = dY * act'(Y); ReLU rewrites dY in place, as the reference does
    if(activation == ONN_ACT_RELU && !(flags & ONN_DELTA_READY)) ONN_TRY(launch_relu_delta(dY, Y, rows * out, s));
    if(activation == ONN_ACT_SIGMOID && !(flags & ONN_DELTA_READY)) ONN_TRY(launch_sigmoid_delta(dY, Y, rows * out, s));
    const float* delta = dY;

    ONN_TRY(weight_gradients(X, delta, dW, db, rows, in, out, s));

    if(dX)
    {
        onn_gemm_args g = plain_gemm(delta, 0, out, W, 0, out, dX, in, rows, in, out);
        g.relu_mask = dX_relu_bits ? nullptr : dX_relu_mask;
        g.relu_bits = dX_relu_bits;
        g.relu_bits_ld = onn_relu_bits_words_per_row(in);
        g.colsum_out = dX_colsum;
        g.flags = flags & ONN_ACCUMULATE;
        ONN_TRY(gemm(g, s));
    }
    return ONN_OK;
}

// ---------------------------------------------------------------------------------------
// MultiHeadAttention
// ---------------------------------------------------------------------------------------

namespace
{
// how onn_mha_bwd forms dK and dV: 0 = batched GEMMs over P and dS, 1 = the recomputation kernel where it applies
std::atomic<int> g_kv_grad_by_recomputation{ []{ const char* e = std::getenv("ONN_B200_ATTENTION_KV_GRAD"); return (e && e[0] == '1') ? 1 : 0; }() };

struct MhaForwardLayout
{
    size_t q, k, v, p, ctx, pad, row_max, row_inv, total;
    MhaForwardLayout(int64_t B, int64_t Sq, int64_t Sk, int64_t E, int64_t H)
    {
        size_t at = 0;
        auto take = [&](size_t floats) { const size_t here = at; at += pad64(floats); return here; };
        q = take((size_t)B * Sq * E);
        k = take((size_t)B * Sk * E);
        v = take((size_t)B * Sk * E);
        p = take((size_t)B * H * Sq * Sk);
        ctx = take((size_t)B * Sq * E);
        pad = take(((size_t)B * Sk + 3) / 4);
        // per query row, for the key / value gradient kernel: the maximum and 1 / sum the softmax of that row used
        row_max = take((size_t)B * H * Sq);
        row_inv = take((size_t)B * H * Sq);
        total = at;
    }
};

struct MhaBackwardLayout
{
    size_t dctx, dp, dq, dk, dv, delta, total;
    MhaBackwardLayout(int64_t B, int64_t Sq, int64_t Sk, int64_t E, int64_t H)
    {
        size_t at = 0;
        auto take = [&](size_t floats) { const size_t here = at; at += pad64(floats); return here; };
        dctx = take((size_t)B * Sq * E);
        dp = take((size_t)B * H * Sq * Sk);
        dq = take((size_t)B * Sq * E);
        dk = take((size_t)B * Sk * E);
        dv = take((size_t)B * Sk * E);
        delta = take((size_t)B * H * Sq);                 // rowsum(dO * O), from the query-gradient kernel to the key / value one
        total = at;
    }
};

// Per-(batch, head) operand: head h of batch b inside a [B, S, E] tensor (row pitch E).
void head_strides(onn_gemm_args& g, char which, long long S, long long E, long long hd)
{
    if(which == 'a') { g.a_stride_inner = hd; g.a_stride_outer = S * E; }
    if(which == 'b') { g.b_stride_inner = hd; g.b_stride_outer = S * E; }
    if(which == 'c') { g.c_stride_inner = hd; g.c_stride_outer = S * E; }
}

// Per-(batch, head) [Sq, Sk] matrix inside a contiguous [B, H, Sq, Sk] tensor.
void score_strides(onn_gemm_args& g, char which, long long H, long long Sq, long long Sk)
{
    if(which == 'a') { g.a_stride_inner = Sq * Sk; g.a_stride_outer = H * Sq * Sk; }
    if(which == 'c') { g.c_stride_inner = Sq * Sk; g.c_stride_outer = H * Sq * Sk; }
}
}  // namespace

extern "C" int onn_mha_set_kv_grad_by_recomputation(int enabled)
{
    return g_kv_grad_by_recomputation.exchange(enabled != 0 ? 1 : 0, std::memory_order_relaxed);
}

extern "C" size_t onn_mha_fwd_workspace_floats(int64_t B, int64_t Sq, int64_t Sk, int64_t E, int64_t H)
{
    if(B <= 0 || Sq <= 0 || Sk <= 0 || E <= 0 || H <= 0) return 0;
    return MhaForwardLayout(B, Sq, Sk, E, H).total;
}

extern "C" size_t onn_mha_bwd_workspace_floats(int64_t B, int64_t Sq, int64_t Sk, int64_t E, int64_t H)
{
    if(B <= 0 || Sq <= 0 || Sk <= 0 || E <= 0 || H <= 0) return 0;
    return MhaBackwardLayout(B, Sq, Sk, E, H).total;
}

extern "C" const float* onn_mha_attention_weights(const float* fwd_workspace, int64_t B, int64_t Sq, int64_t Sk, int64_t E, int64_t H)
{
    if(!fwd_workspace) return nullptr;
    return fwd_workspace + MhaForwardLayout(B, Sq, Sk, E, H).p;
}

extern "C" int onn_mha_fwd(const float* Xq, const float* Xs, const onn_mha_params* params,
                           const uint8_t* source_row_is_zero, float* Y,
                           int64_t B, int64_t Sq, int64_t Sk, int64_t E, int64_t H, int causal,
                           float* ws, uint32_t flags, void* stream)
{
    ONN_CHECK_ARG(Xq && Xs && params && Y && B > 0 && Sq > 0 && Sk > 0 && E > 0 && H > 0 && E % H == 0);
    ONN_CHECK_ARG(params->Wq && params->Wk && params->Wv && params->Wo);
    if(!ws) return ONN_ERR_WORKSPACE;
    cudaStream_t s = (cudaStream_t)stream;
    const MhaForwardLayout L(B, Sq, Sk, E, H);
    const long long hd = E / H;
    const float scale = 1.0f / sqrtf((float)hd);
    const uint8_t* pad_flags = source_row_is_zero;
    if(!pad_flags)
    {
        uint8_t* mine = reinterpret_cast<uint8_t*>(ws + L.pad);
        ONN_TRY(launch_source_row_is_zero(Xs, mine, B * Sk, (int)E, s));
        pad_flags = mine;
    }

    const float *Wq = params->Wq, *Wk = params->Wk, *Wv = params->Wv, *Wo = params->Wo;

    float *q = ws + L.q, *k = ws + L.k, *v = ws + L.v, *p = ws + L.p, *ctx = ws + L.ctx;

    // projections, kept in [B, S, E] layout: head h is the column slice h*hd .. of each row
    {
        onn_gemm_args g = plain_gemm(Xq, 0, E, Wq, 1, E, q, E, B * Sq, E, E);
        g.bias = params->bq;
        ONN_TRY(gemm(g, s));
        g = plain_gemm(Xs, 0, E, Wk, 1, E, k, E, B * Sk, E, E);
        g.bias = params->bk;
        ONN_TRY(gemm(g, s));
        g = plain_gemm(Xs, 0, E, Wv, 1, E, v, E, B * Sk, E, E);
        g.bias = params->bv;
        ONN_TRY(gemm(g, s));
    }
    // attention core: one fused kernel where the shapes allow (head size 64; source lengths above 256 are walked in
    // key tiles), else scores GEMM -> mask + softmax -> context GEMM
    static const bool fused_enabled = []{ const char* e = std::getenv("ONN_B200_ATTENTION_FUSED"); return !(e && e[0] == '0'); }();
    const bool aligned = host_aligned16(q) && host_aligned16(k) && host_aligned16(v) && host_aligned16(p) && host_aligned16(ctx);
    if(fused_enabled && gemm_mode() != 1 && attention_fwd_fused_supported(q, k, v, p, ctx, B, Sq, Sk, E, H))
    {
        // when back-propagation is to form the weights again from Q, K (onn_mha_set_kv_grad_by_recomputation) it needs
        // these per-row statistics and the key flags; otherwise nothing extra is written or copied
        const bool keep_for_recomputation = g_kv_grad_by_recomputation.load(std::memory_order_relaxed) != 0;
        if(keep_for_recomputation && pad_flags != reinterpret_cast<const uint8_t*>(ws + L.pad) &&
           cudaMemcpyAsync(ws + L.pad, pad_flags, (size_t)(B * Sk), cudaMemcpyDeviceToDevice, s) != cudaSuccess) return ONN_ERR_CUDA;
        ONN_TRY(attention_fwd_fused_launch(q, k, v, pad_flags, p, ctx, keep_for_recomputation ? ws + L.row_max : nullptr,
                                           keep_for_recomputation ? ws + L.row_inv : nullptr, B, Sq, Sk, E, H, causal, scale, s));
    }
    else if(fused_enabled && gemm_mode() != 1 && aligned && attention_long_supported(B, Sq, Sk, E, H))
    {
        ONN_TRY(attention_long_fwd_launch(q, k, v, pad_flags, p, ctx, B, Sq, Sk, E, H, causal, scale, s));
    }
    else
    {
        // scores = scale * Q K^T per (b, h)
        {
            onn_gemm_args g = plain_gemm(q, 0, E, k, 0, E, p, Sk, Sq, Sk, hd);
            g.batch_inner = (int)H; g.batch_outer = (int)B;
            head_strides(g, 'a', Sq, E, hd); head_strides(g, 'b', Sk, E, hd); score_strides(g, 'c', H, Sq, Sk);
            g.alpha = scale;
            ONN_TRY(gemm(g, s));
        }
        ONN_TRY(launch_attention_softmax(p, pad_flags, B, (int)H, (int)Sq, (int)Sk, causal, s));
        // context = P V per (b, h), written straight into the concatenated [B, Sq, E] layout
        {
            onn_gemm_args g = plain_gemm(p, 0, Sk, v, 1, E, ctx, E, Sq, hd, Sk);
            g.batch_inner = (int)H; g.batch_outer = (int)B;
            score_strides(g, 'a', H, Sq, Sk); head_strides(g, 'b', Sk, E, hd); head_strides(g, 'c', Sq, E, hd);
       
            ONN_TRY(gemm(g, s));
        }
    }
    {
        onn_gemm_args g = plain_gemm(ctx, 0, E, Wo, 1, E, Y, E, B * Sq, E, E);
        g.bias = params->bo;
        ONN_TRY(gemm(g, s));
    }
    return ONN_OK;
}

extern "C" int onn_mha_bwd(const float* Xq, const float* Xs, const onn_mha_params* params,
                           const float* fwd_ws, const float* dY,
                           const onn_mha_grads* grads, float* dXq, float* dXs,
                           int64_t B, int64_t Sq, int64_t Sk, int64_t E, int64_t H, int causal,
                           float* ws, uint32_t flags, void* stream)
{
    ONN_CHECK_ARG(Xq && Xs && params && fwd_ws && dY && grads && dXq && B > 0 && Sq > 0 && Sk > 0 && E > 0 && H > 0 && E % H == 0);
    const bool self_attention = Xs == Xq;
    ONN_CHECK_ARG(self_attention ? dXs == nullptr : dXs != nullptr);
    if(!ws) return ONN_ERR_WORKSPACE;
    cudaStream_t s = (cudaStream_t)stream;
    const MhaForwardLayout F(B, Sq, Sk, E, H);
    const MhaBackwardLayout L(B, Sq, Sk, E, H);
    const long long hd = E / H;
    const float scale = 1.0f / sqrtf((float)hd);
    const long long rows_q = B * Sq, rows_s = B * Sk;

    const float *Wq = params->Wq, *Wk = params->Wk, *Wv = params->Wv, *Wo = params->Wo;
    const float *q = fwd_ws + F.q, *k = fwd_ws + F.k, *v = fwd_ws + F.v, *p = fwd_ws + F.p, *ctx = fwd_ws + F.ctx;
    float *dctx = ws + L.dctx, *dp = ws + L.dp, *dq = ws + L.dq, *dk = ws + L.dk, *dv = ws + L.dv;

    // output projection
    ONN_TRY(weight_gradients(ctx, dY, grads->dWo, grads->dbo, rows_q, E, E, s));
    {
        onn_gemm_args g = plain_gemm(dY, 0, E, Wo, 0, E, dctx, E, rows_q, E, E);
        ONN_TRY(gemm(g, s));
    }
    // dP, dS and dQ: one fused kernel where the shapes allow, else GEMM -> softmax backward -> GEMM
    static const bool fused_enabled = []{ const char* e = std::getenv("ONN_B200_ATTENTION_FUSED"); return !(e && e[0] == '0'); }();
    const bool kv_kernel_enabled = g_kv_grad_by_recomputation.load(std::memory_order_relaxed) != 0;
    // Where the forward pass ran on the single-tile fused kernel it left every query row's softmax statistics, and the
    // key and value gradients come from ONE kernel that forms the weights again on the SM (no pass over P or dS, and
    // dS is never written); elsewhere from two batched GEMMs over P and dS.  Back-propagation must therefore run with
    // the kernels its forward pass ran with (the same GEMM mode and environment switches).
    const bool kv_by_recomputation = fused_enabled && kv_kernel_enabled && gemm_mode() != 1 &&
                                     attention_bwd_fused_supported(k, v, p, ctx, dctx, dp, dq, B, Sq, Sk, E, H) &&
                                     attention_kv_grad_supported(q, k, v, dctx, dk, dv, B, Sq, Sk, E, H);
    if(!kv_by_recomputation)
    {
        // dV = P^T dO
        onn_gemm_args g = plain_gemm(p, 1, Sk, dctx, 1, E, dv, E, Sk, hd, Sq);
        g.batch_inner = (int)H; g.batch_outer = (int)B;
        score_strides(g, 'a', H, Sq, Sk); head_strides(g, 'b', Sq, E, hd); head_strides(g, 'c', Sk, E, hd);
        g.colsum_out = grads->dbv; g.colsum_stride_inner = hd;      // dbv = column sums of dV, taken in the epilogue
        ONN_TRY(gemm(g, s));
    }
    const bool aligned = host_aligned16(k) && host_aligned16(v) && host_aligned16(p) && host_aligned16(ctx) && host_aligned16(dctx) &&
                         host_aligned16(dp) && host_aligned16(dq);
    if(kv_by_recomputation)
    {
        float* delta = ws + L.delta;
        ONN_TRY(attention_bwd_fused_launch(k, v, p, ctx, dctx, dp, dq, grads->dbq, delta, 0, B, Sq, Sk, E, H, scale, s));
        ONN_TRY(attention_kv_grad_launch(q, k, v, dctx, reinterpret_cast<const unsigned char*>(fwd_ws + F.pad), fwd_ws + F.row_max, fwd_ws + F.row_inv,
                                         delta, dk, dv, grads->dbk, grads->dbv, B, Sq, Sk, E, H, causal, scale, s));
    }
    else if(fused_enabled && gemm_mode() != 1 && attention_bwd_fused_supported(k, v, p, ctx, dctx, dp, dq, B, Sq, Sk, E, H))
    {
        ONN_TRY(attention_bwd_fused_launch(k, v, p, ctx, dctx, dp, dq, grads->dbq, nullptr, 1, B, Sq, Sk, E, H, scale, s));
    }
    else if(fused_enabled && gemm_mode() != 1 && aligned && attention_long_supported(B, Sq, Sk, E, H))
    {
        // with a causal mask the weights of whole key tiles above the diagonal are zero: the kernel skips them
        ONN_TRY(attention_long_bwd_launch(k, v, p, ctx, dctx, dp, dq, grads->dbq, B, Sq, Sk, E, H, causal, scale, s));
    }
    else
    {
        // dP = dO V^T
        {
            onn_gemm_args g = plain_gemm(dctx, 0, E, v, 0, E, dp, Sk, Sq, Sk, hd);
            g.batch_inner = (int)H; g.batch_outer = (int)B;
            head_strides(g, 'a', Sq, E, hd); head_strides(g, 'b', Sk, E, hd); score_strides(g, 'c', H, Sq, Sk);
            ONN_TRY(gemm(g, s));
        }
        // dS = P * (dP - rowsum(P * dP)), in place
        ONN_TRY(launch_attention_softmax_bwd(p, dp, B * H * Sq, (int)Sk, s));
        // dQ = scale * dS K
        {
            onn_gemm_args g = plain_gemm(dp, 0, Sk, k, 1, E, dq, E, Sq, hd, Sk);
            g.batch_inner = (int)H; g.batch_outer = (int)B;
            score_strides(g, 'a', H, Sq, Sk); head_strides(g, 'b', Sk, E, hd); head_strides(g, 'c', Sq, E, hd);
            g.alpha = scale;
            g.colsum_out = grads->dbq; g.colsum_stride_inner = hd;      // dbq = column sums of dQ, taken in the epilogue
            ONN_TRY(gemm(g, s));
        }
    }
    // dK = scale * dS^T Q
    if(!kv_by_recomputation)
    {
        onn_gemm_args g = plain_gemm(dp, 1, Sk, q, 1, E, dk, E, Sk, hd, Sq);
        g.batch_inner = (int)H; g.batch_outer = (int)B;
        score_strides(g, 'a', H, Sq, Sk); head_strides(g, 'b', Sq, E, hd); head_strides(g, 'c', Sk, E, hd);
        g.alpha = scale;
        g.colsum_out = grads->dbk; g.colsum_stride_inner = hd;
        ONN_TRY(gemm(g, s));
    }
    // input projections (their bias gradients were taken by the epilogues above)
    ONN_TRY(weight_gradients(Xq, dq, grads->dWq, nullptr, rows_q, E, E, s));
    ONN_TRY(weight_gradients(Xs, dk, grads->dWk, nullptr, rows_s, E, E, s));
    ONN_TRY(weight_gradients(Xs, dv, grads->dWv, nullptr, rows_s, E, E, s));

    // Input gradients.  Where the operand pairs lie at equal distances (dQ, dK, dV in the scratch arena; Wq, Wk, Wv in
    // the parameter arena) the sum dQ Wq^T + dK Wk^T + dV Wv^T is ONE product whose reduction runs through the pairs:
    // one pass over the result instead of a store and two read-modify-write passes.
    const long long kv_step = dv - dk, w_kv_step = Wv - Wk;                 // between the key and value operand pairs
    const bool pair_kv = kv_step > 0 && w_kv_step > 0;
    const bool triple = pair_kv && dk - dq == kv_step && Wk - Wq == w_kv_step; // and the same again from query to key
    float* source_grad = self_attention ? dXq : dXs;
    if(self_attention && triple)
    {
        onn_gemm_args g = plain_gemm(dq, 0, E, Wq, 0, E, dXq, E, rows_q, E, E);
        g.k_parts = 3; g.a_stride_part = kv_step; g.b_stride_part = w_kv_step;
        ONN_TRY(gemm(g, s));
    }
    else
    {
        {
            onn_gemm_args g = plain_gemm(dq, 0, E, Wq, 0, E, dXq, E, rows_q, E, E);
            ONN_TRY(gemm(g, s));
        }
        if(pair_kv)
        {
            onn_gemm_args g = plain_gemm(dk, 0, E, Wk, 0, E, source_grad, E, rows_s, E, E);
            g.k_parts = 2; g.a_stride_part = kv_step; g.b_stride_part = w_kv_step;
            if(self_attention || (flags & ONN_ACCUMULATE)) g.flags = ONN_ACCUMULATE;
            ONN_TRY(gemm(g, s));
        }
        else
        {
            onn_gemm_args g = plain_gemm(dk, 0, E, Wk, 0, E, source_grad, E, rows_s, E, E);
            if(self_attention || (flags & ONN_ACCUMULATE)) g.flags = ONN_ACCUMULATE;
            ONN_TRY(gemm(g, s));
            g = plain_gemm(dv, 0, E, Wv, 0, E, source_grad, E, rows_s, E, E);
            g.flags = ONN_ACCUMULATE;
            ONN_TRY(gemm(g, s));
        }
    }
    return ONN_OK;
}
