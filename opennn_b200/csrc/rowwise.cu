// HBM-bound row kernels: Embedding forward/backward, Normalization3d (+ fused Addition)
// forward/backward, Addition.  One warp owns one [E]-row; the row lives in
// registers, reductions are warp shuffles, global access is 128-bit where E % 4 == 0.
#include <mutex>

#include "common.cuh"
#include "launch_counter.h"

namespace onn
{

constexpr int kRowThreads = 256;                  // 8 warps = 8 rows per CTA per sweep
constexpr int kRowWarps = kRowThreads / 32;
constexpr int kMaxVec = 8;                        // float4 per lane kept in registers: E <= 1024

// ---------------------------------------------------------------------------------------
// Embedding
// ---------------------------------------------------------------------------------------

// out = W[id] * sqrt(E) + PE[s]; the product and the sum are rounded separately
// (__fmul_rn / __fadd_rn) so no FMA contraction changes the bits.
__global__ void __launch_bounds__(kRowThreads)
embedding_fwd_kernel(const float* __restrict__ ids, const float* __restrict__ W, const float* __restrict__ PE,
                     float* __restrict__ out, uint8_t* __restrict__ row_is_zero,
                     long long tokens, int S, int E, long long V, float scale_value, int scale, int add_pe)
{
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
    const long long stride = (long long)gridDim.x * kRowWarps;
    const bool vec = (E & 3) == 0;

    for(long long token = warp; token < tokens; token += stride)
    {
        const long long id = token_index(ids[token]);
        const bool in_range = id >= 0 && id < V;
        const bool with_pe = add_pe && id > 0;
        const float* w_row = W + (in_range ? id : 0) * (long long)E;
        const float* pe_row = PE + (long long)(token % S) * E;
        float* out_row = out + token * (long long)E;
        bool all_zero = true;

        if(vec)
        {
            for(int e = lane * 4; e < E; e += 128)
            {
                float4 w = in_range ? ld4(w_row + e) : make_float4(0.f, 0.f, 0.f, 0.f);
                if(scale)
                {
                    w.x = __fmul_rn(w.x, scale_value); w.y = __fmul_rn(w.y, scale_value);
                    w.z = __fmul_rn(w.z, scale_value); w.w = __fmul_rn(w.w, scale_value);
                }
                if(with_pe)
                {
                    const float4 p = ld4(pe_row + e);
                    w.x = __fadd_rn(w.x, p.x); w.y = __fadd_rn(w.y, p.y);
                    w.z = __fadd_rn(w.z, p.z); w.w = __fadd_rn(w.w, p.w);
                }
                all_zero = all_zero && fabsf(w.x) <= 1e-7f && fabsf(w.y) <= 1e-7f && fabsf(w.z) <= 1e-7f && fabsf(w.w) <= 1e-7f;
                st4(out_row + e, w);
            }
        }
        else
        {
            for(int e = lane; e < E; e += 32)
            {
                float w = in_range ? w_row[e] : 0.f;
                if(scale) w = __fmul_rn(w, scale_value);
                if(with_pe) w = __fadd_rn(w, pe_row[e]);
                all_zero = all_zero && fabsf(w) <= 1e-7f;
                out_row[e] = w;
            }
        }

        if(row_is_zero)
        {
            all_zero = __all_sync(0xffffffffu, all_zero);
            if(lane == 0) row_is_zero[token] = all_zero ? 1 : 0;
        }
    }
}

// dW[id] += (dY + dY2) * sqrt(E) for 0 < id < V: fp32 reductions into L2 (vectorised
// where the row is 16-byte aligned).  Row 0 (padding) is never touched, so it stays zero.
__global__ void __launch_bounds__(kRowThreads)
embedding_bwd_kernel(const float* __restrict__ ids, const float* __restrict__ dY, const float* __restrict__ dY2,
                     float* __restrict__ dW, long long tokens, int E, long long V, float scale_value, int scale)
{
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
    const long long stride = (long long)gridDim.x * kRowWarps;
    const bool vec = (E & 3) == 0;

    for(long long token = warp; token < tokens; token += stride)
    {
        const long long id = token_index(ids[token]);
        if(id <= 0 || id >= V) continue;
        const float* g_row = dY + token * (long long)E;
        const float* g2_row = dY2 ? dY2 + token * (long long)E : nullptr;
        float* w_row = dW + id * (long long)E;

        if(vec)
        {
            for(int e = lane * 4; e < E; e += 128)
            {
                float4 g = ld4_stream(g_row + e);
                if(g2_row) { const float4 h = ld4_stream(g2_row + e); g.x += h.x; g.y += h.y; g.z += h.z; g.w += h.w; }
                if(scale) { g.x *= scale_value; g.y *= scale_value; g.z *= scale_value; g.w *= scale_value; }
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                             :: "l"(w_row + e), "f"(g.x), "f"(g.y), "f"(g.z), "f"(g.w) : "memory");
            }
        }
        else
        {
            for(int e = lane; e < E; e += 32)
            {
                float g = g_row[e];
                if(g2_row) g += g2_row[e];
                if(scale) g *= scale_value;
                atomicAdd(w_row + e, g);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Normalization3d
// ---------------------------------------------------------------------------------------

// Register-resident row path (E % 4 == 0, E <= 1024).  Statistics are two passes over the
// registers: mean first, then the mean of centred squares (the reference's formulation).
// gamma and beta are read per row (8 KiB, they stay in L1): keeping them in registers as well would cost 64 registers
// per thread and halve the rows in flight per SM, which is what the memory system is fed by.
// Rows of a row kernel, one warp per row.  Without a counter warp q of the grid takes rows q, q + warps, ...; with one
// (common.cuh: next_work_counter) every warp asks for its next row while it works on the current one, so that CTAs which
// find their SM taken by another kernel do not leave a fixed share of the rows waiting.  The counter wraps to zero when
// the last warp has asked once past the end.
struct RowWalk
{
    unsigned int* counter;
    long long rows, warps, next_fixed;
    uint32_t ahead;

    __device__ __forceinline__ RowWalk(unsigned int* counter_in, long long rows_in, int lane) : counter(counter_in), rows(rows_in)
    {
        warps = (long long)gridDim.x * (blockDim.x >> 5);
        next_fixed = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
        ahead = 0;
        if(counter && lane == 0) ahead = atomicInc(counter, (unsigned int)(rows + warps - 1));
    }
    // the warp's next row, or -1; all lanes call it
    __device__ __forceinline__ long long next(int lane)
    {
        if(!counter)
        {
            const long long row = next_fixed;
            next_fixed += warps;
            return row < rows ? row : -1;
        }
        const uint32_t mine = __shfl_sync(0xffffffffu, ahead, 0);
        if((long long)mine >= rows) return -1;
        if(lane == 0) ahead = atomicInc(counter, (unsigned int)(rows + warps - 1));
        return (long long)mine;
    }
};

template <int VEC>
__global__ void __launch_bounds__(kRowThreads, 4)
layernorm_fwd_kernel(const float* __restrict__ A, const float* __restrict__ R,
                     const float* __restrict__ gamma, const float* __restrict__ beta,
                     float* __restrict__ Y, float* __restrict__ sum_out,
                     float* __restrict__ mean_out, float* __restrict__ inv_std_out, uint8_t* __restrict__ row_is_zero,
                     long long rows, int E, float eps, unsigned int* work_counter)
{
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    RowWalk walk(work_counter, rows, lane);                   // after the wait: the launch before this one may have used the same counter
    const float inv_E = 1.0f / (float)E;

    for(long long row = walk.next(lane); row >= 0; row = walk.next(lane))
    {
        const float* a_row = A + row * (long long)E;
        const float* r_row = R ? R + row * (long long)E : nullptr;
        float4 x[VEC];
        float total = 0.f;
#pragma unroll
        for(int i = 0; i < VEC; i++)
        {
            const int e = (i * 32 + lane) * 4;
            x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if(e < E)
            {
                x[i] = ld4_stream(a_row + e);
                if(r_row) { const float4 r = ld4_stream(r_row + e); x[i].x += r.x; x[i].y += r.y; x[i].z += r.z; x[i].w += r.w; }
                if(sum_out) st4(sum_out + row * (long long)E + e, x[i]);
                total += (x[i].x + x[i].y) + (x[i].z + x[i].w);
            }
        }
        const float mean = warp_sum(total) * inv_E;
        float squares = 0.f;
#pragma unroll
        for(int i = 0; i < VEC; i++)
        {
            const int e = (i * 32 + lane) * 4;
            if(e < E)
            {
                x[i].x -= mean; x[i].y -= mean; x[i].z -= mean; x[i].w -= mean;
                squares += (x[i].x * x[i].x + x[i].y * x[i].y) + (x[i].z * x[i].z + x[i].w * x[i].w);
            }
        }
        const float inv_std = 1.0f / sqrtf(warp_sum(squares) * inv_E + eps);
        bool all_zero = true;
#pragma unroll
        for(int i = 0; i < VEC; i++)
        {
            const int e = (i * 32 + lane) * 4;
            if(e < E)
            {
                const float4 g = ld4(gamma + e), b = ld4(beta + e);
                float4 y;
                y.x = (x[i].x * inv_std * g.x + b.x);
                y.y = (x[i].y * inv_std * g.y + b.y);
                y.z = (x[i].z * inv_std * g.z + b.z);
                y.w = (x[i].w * inv_std * g.w + b.w);
                all_zero = all_zero && fabsf(y.x) <= 1e-7f && fabsf(y.y) <= 1e-7f && fabsf(y.z) <= 1e-7f && fabsf(y.w) <= 1e-7f;
                st4(Y + row * (long long)E + e, y);
            }
        }
        if(lane == 0) { mean_out[row] = mean; inv_std_out[row] = inv_std; }
        if(row_is_zero)
        {
            all_zero = __all_sync(0xffffffffu, all_zero);
            if(lane == 0) row_is_zero[row] = all_zero ? 1 : 0;
        }
    }
}

// Any E: three sweeps over the row; the second and third hit L1/L2.
__global__ void __launch_bounds__(kRowThreads)
layernorm_fwd_generic_kernel(const float* __restrict__ A, const float* __restrict__ R,
                             const float* __restrict__ gamma, const float* __restrict__ beta,
                             float* __restrict__ Y, float* __restrict__ sum_out,
                             float* __restrict__ mean_out, float* __restrict__ inv_std_out, uint8_t* __restrict__ row_is_zero,
                             long long rows, int E, float eps)
{
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
    const long long stride = (long long)gridDim.x * kRowWarps;
    const float inv_E = 1.0f / (float)E;

    for(long long row = warp; row < rows; row += stride)
    {
        const float* a_row = A + row * (long long)E;
        const float* r_row = R ? R + row * (long long)E : nullptr;
        float total = 0.f;
        for(int e = lane; e < E; e += 32) total += a_row[e] + (r_row ? r_row[e] : 0.f);
        const float mean = warp_sum(total) * inv_E;
        float squares = 0.f;
        for(int e = lane; e < E; e += 32)
        {
            const float c = a_row[e] + (r_row ? r_row[e] : 0.f) - mean;
            squares += c * c;
        }
        const float inv_std = 1.0f / sqrtf(warp_sum(squares) * inv_E + eps);
        bool all_zero = true;
        for(int e = lane; e < E; e += 32)
        {
            const float x = a_row[e] + (r_row ? r_row[e] : 0.f);
            if(sum_out) sum_out[row * (long long)E + e] = x;
            const float y = ((x - mean) * inv_std * gamma[e] + beta[e]);
            all_zero = all_zero && fabsf(y) <= 1e-7f;
            Y[row * (long long)E + e] = y;
        }
        if(lane == 0) { mean_out[row] = mean; inv_std_out[row] = inv_std; }
        if(row_is_zero)
        {
            all_zero = __all_sync(0xffffffffu, all_zero);
            if(lane == 0) row_is_zero[row] = all_zero ? 1 : 0;
        }
    }
}

// Backward: dx = (d - mean(d) - x_hat * mean(d * x_hat)) * inv_std with d = dy * gamma.
// Each warp keeps running per-column sums of dy * x_hat and dy in registers across all the
// rows it visits; the CTA folds its 8 warps through shared memory and writes ONE partial
// row pair per CTA to `partials` ([gridDim.x][2][E]); colsum_partials_kernel finishes.
// DX_SUM adds a third running sum, of dx itself: the bias gradient of the layer whose output the
// normalised sum contains (its output gradient IS dx), so partials become [gridDim.x][3][E].
template <int VEC, bool DX_SUM>
__global__ void __launch_bounds__(kRowThreads, 2)
layernorm_bwd_kernel(const float* __restrict__ dY, const float* __restrict__ dY2, const float* __restrict__ dY3,
                     const float* __restrict__ X, const float* __restrict__ mean_in, const float* __restrict__ inv_std_in,
                     const float* __restrict__ gamma, float* __restrict__ dX, float* __restrict__ partials,
                     long long rows, int E, unsigned int* work_counter)
{
    pdl_launch_dependents();
    pdl_wait();
    RowWalk walk(work_counter, rows, threadIdx.x & 31);      // after the wait: the launch before this one may have used the same counter
    // [kRowWarps][2][E]: every warp keeps its running column sums here, and every lane only ever touches
    // its own columns, so plain loads and stores suffice; registers stay free for two CTAs per SM
    extern __shared__ float smem[];
    const int lane = threadIdx.x & 31, warp_in_block = threadIdx.x >> 5;
    const float inv_E = 1.0f / (float)E;
    constexpr int SETS = DX_SUM ? 3 : 2;
    float* acc_gamma = smem + (size_t)warp_in_block * SETS * E;
    float* acc_beta = acc_gamma + E;
    float* acc_dx = acc_beta + E;                            // only touched with DX_SUM

#pragma unroll
    for(int i = 0; i < VEC; i++)
    {
        const int e = (i * 32 + lane) * 4;
        if(e < E)
        {
            st4(acc_gamma + e, make_float4(0.f, 0.f, 0.f, 0.f)); st4(acc_beta + e, make_float4(0.f, 0.f, 0.f, 0.f));
            if(DX_SUM) st4(acc_dx + e, make_float4(0.f, 0.f, 0.f, 0.f));
        }
    }

    for(long long row = walk.next(lane); row >= 0; row = walk.next(lane))
    {
        const long long base = row * (long long)E;
        const float mean = mean_in[row], inv_std = inv_std_in[row];
        float4 d[VEC], xh[VEC];
        float sum_d = 0.f, sum_dx = 0.f;
#pragma unroll
        for(int i = 0; i < VEC; i++)
        {
            const int e = (i * 32 + lane) * 4;
            d[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            xh[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if(e < E)
            {
                float4 dy = ld4_stream(dY + base + e);
                if(dY2) { const float4 t = ld4_stream(dY2 + base + e); dy.x += t.x; dy.y += t.y; dy.z += t.z; dy.w += t.w; }
                if(dY3) { const float4 t = ld4_stream(dY3 + base + e); dy.x += t.x; dy.y += t.y; dy.z += t.z; dy.w += t.w; }
                const float4 x = ld4_stream(X + base + e);
                const float4 g = ld4(gamma + e);
                xh[i].x = (x.x - mean) * inv_std; xh[i].y = (x.y - mean) * inv_std;
                xh[i].z = (x.z - mean) * inv_std; xh[i].w = (x.w - mean) * inv_std;
                float4 ag = ld4(acc_gamma + e), ab = ld4(acc_beta + e);
                ag.x += dy.x * xh[i].x; ag.y += dy.y * xh[i].y; ag.z += dy.z * xh[i].z; ag.w += dy.w * xh[i].w;
                ab.x += dy.x; ab.y += dy.y; ab.z += dy.z; ab.w += dy.w;
                st4(acc_gamma + e, ag); st4(acc_beta + e, ab);
                d[i].x = dy.x * g.x; d[i].y = dy.y * g.y; d[i].z = dy.z * g.z; d[i].w = dy.w * g.w;
                sum_d += (d[i].x + d[i].y) + (d[i].z + d[i].w);
                sum_dx += (d[i].x * xh[i].x + d[i].y * xh[i].y) + (d[i].z * xh[i].z + d[i].w * xh[i].w);
            }
        }
        sum_d = warp_sum(sum_d) * inv_E;
        sum_dx = warp_sum(sum_dx) * inv_E;
#pragma unroll
        for(int i = 0; i < VEC; i++)
        {
            const int e = (i * 32 + lane) * 4;
            if(e < E)
            {
                float4 o;
                o.x = ((d[i].x - sum_d - xh[i].x * sum_dx) * inv_std);
                o.y = ((d[i].y - sum_d - xh[i].y * sum_dx) * inv_std);
                o.z = ((d[i].z - sum_d - xh[i].z * sum_dx) * inv_std);
                o.w = ((d[i].w - sum_d - xh[i].w * sum_dx) * inv_std);
                st4(dX + base + e, o);
                if(DX_SUM)
                {
                    float4 ax = ld4(acc_dx + e);
                    ax.x += o.x; ax.y += o.y; ax.z += o.z; ax.w += o.w;
                    st4(acc_dx + e, ax);
                }
            }
        }
    }

    __syncthreads();
    float* out = partials + (size_t)blockIdx.x * SETS * E;
    for(int c = threadIdx.x; c < SETS * E; c += kRowThreads)
    {
        float total = 0.f;
#pragma unroll
        for(int w = 0; w < kRowWarps; w++) total += smem[(size_t)w * SETS * E + c];
        out[c] = total;
    }
}

// Any E: column sums via shared-memory atomics per CTA, then one partial row pair per CTA.
__global__ void __launch_bounds__(kRowThreads)
layernorm_bwd_generic_kernel(const float* __restrict__ dY, const float* __restrict__ dY2, const float* __restrict__ dY3,
                             const float* __restrict__ X, const float* __restrict__ mean_in, const float* __restrict__ inv_std_in,
                             const float* __restrict__ gamma, float* __restrict__ dX, float* __restrict__ partials,
                             long long rows, int E)
{
    extern __shared__ float smem[];               // [2][E]
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
    const long long stride = (long long)gridDim.x * kRowWarps;
    const float inv_E = 1.0f / (float)E;

    for(int c = threadIdx.x; c < 2 * E; c += kRowThreads) smem[c] = 0.f;
    __syncthreads();

    for(long long row = warp; row < rows; row += stride)
    {
        const long long base = row * (long long)E;
        const float mean = mean_in[row], inv_std = inv_std_in[row];
        float sum_d = 0.f, sum_dx = 0.f;
        for(int e = lane; e < E; e += 32)
        {
            const float dy = dY[base + e] + (dY2 ? dY2[base + e] : 0.f) + (dY3 ? dY3[base + e] : 0.f);
            const float xh = (X[base + e] - mean) * inv_std;
            const float d = dy * gamma[e];
            sum_d += d; sum_dx += d * xh;
            atomicAdd(smem + e, dy * xh);
            atomicAdd(smem + E + e, dy);
        }
        sum_d = warp_sum(sum_d) * inv_E;
        sum_dx = warp_sum(sum_dx) * inv_E;
        for(int e = lane; e < E; e += 32)
        {
            const float dy = dY[base + e] + (dY2 ? dY2[base + e] : 0.f) + (dY3 ? dY3[base + e] : 0.f);
            const float xh = (X[base + e] - mean) * inv_std;
            dX[base + e] = ((dy * gamma[e] - sum_d - xh * sum_dx) * inv_std);
        }
    }
    __syncthreads();
    float* out = partials + (size_t)blockIdx.x * 2 * E;
    for(int c = threadIdx.x; c < 2 * E; c += kRowThreads) out[c] = smem[c];
}

// out[c] (+)= sum over p of partials[p][c].  A CTA of 32 x 8 threads owns 32 columns: the 8 thread rows
// stride the partial rows (eight independent, coalesced 128-byte reads in flight), shared memory folds them.
__global__ void __launch_bounds__(256)
colsum_partials_kernel(const float* __restrict__ partials, int count, int columns,
                       float* __restrict__ out_a, float* __restrict__ out_b, float* __restrict__ out_c, int split, int accumulate)
{
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float fold[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + tx;
    float total = 0.f;
    if(c < columns)
        for(int p = ty; p < count; p += 8) total += partials[(size_t)p * columns + c];
    fold[ty][tx] = total;
    __syncthreads();
    if(ty == 0 && c < columns)
    {
        float sum = 0.f;
#pragma unroll
        for(int w = 0; w < 8; w++) sum += fold[w][tx];
        // columns [0, split) -> out_a, [split, 2 split) -> out_b, the rest is ADDED to out_c (a bias gradient)
        if(c >= 2 * split) out_c[c - 2 * split] += sum;
        else
        {
            float* dst = c < split ? out_a + c : out_b + (c - split);
            *dst = accumulate ? *dst + sum : sum;
        }
    }
}

// ---------------------------------------------------------------------------------------
// Element-wise
// ---------------------------------------------------------------------------------------

__global__ void add_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                           long long n)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long n4 = (aligned16(a) && aligned16(b) && aligned16(out)) ? n / 4 : 0;
    for(long long i = tid; i < n4; i += stride)
    {
        const float4 x = ld4_stream(a + 4 * i), y = ld4_stream(b + 4 * i);
        float4 r = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
        st4(out + 4 * i, r);
    }
    for(long long i = 4 * n4 + tid; i < n; i += stride) out[i] = (a[i] + b[i]);
}

static int vec_count(long long E) { return (int)((E + 127) / 128); }

}  // namespace onn

using namespace onn;

extern "C" int onn_embedding_fwd(const float* ids, const float* W, const float* PE, float* out, uint8_t* row_is_zero,
                                 int64_t B, int64_t S, int64_t E, int64_t V, int scale, int add_pe, uint32_t flags, void* stream)
{
    ONN_CHECK_ARG(ids && W && out && B > 0 && S > 0 && E > 0 && V > 0);
    ONN_CHECK_ARG(!add_pe || PE);
    ONN_CHECK_ARG((E & 3) != 0 || (host_aligned16(W) && host_aligned16(out) && (!add_pe || host_aligned16(PE))));
    const long long tokens = B * S;
    const int grid = grid_for(tokens, kRowWarps, 8);
    embedding_fwd_kernel<<<grid, kRowThreads, 0, (cudaStream_t)stream>>>(
        ids, W, PE, out, row_is_zero, tokens, (int)S, (int)E, V, sqrtf((float)E), scale, add_pe);
    count_launch();
    return launch_status();
}

extern "C" int onn_embedding_bwd(const float* ids, const float* dY, const float* dY2, float* dW,
                                 int64_t B, int64_t S, int64_t E, int64_t V, int scale, void* stream)
{
    ONN_CHECK_ARG(ids && dY && dW && B > 0 && S > 0 && E > 0 && V > 0);
    ONN_CHECK_ARG((E & 3) != 0 || (host_aligned16(dY) && host_aligned16(dW) && (!dY2 || host_aligned16(dY2))));
    const long long tokens = B * S;
    const int grid = grid_for(tokens, kRowWarps, 8);
    embedding_bwd_kernel<<<grid, kRowThreads, 0, (cudaStream_t)stream>>>(
        ids, dY, dY2, dW, tokens, (int)E, V, sqrtf((float)E), scale);
    count_launch();
    return launch_status();
}

extern "C" int onn_layernorm_fwd(const float* A, const float* R, const float* gamma, const float* beta,
                                 float* Y, float* sum, float* mean, float* inv_std, uint8_t* row_is_zero,
                                 int64_t rows, int64_t E, float eps, uint32_t flags, void* stream)
{
    ONN_CHECK_ARG(A && gamma && beta && Y && mean && inv_std && rows > 0 && E > 0);
    const int grid = grid_for(rows, kRowWarps, 8);
    cudaStream_t s = (cudaStream_t)stream;
    const bool fast = (E & 3) == 0 && E <= 128 * kMaxVec && host_aligned16(A) && host_aligned16(Y) &&
                      host_aligned16(gamma) && host_aligned16(beta) && (!R || host_aligned16(R)) && (!sum || host_aligned16(sum));
    unsigned int* work_counter = rows + (long long)grid * kRowWarps < (1LL << 31) ? next_work_counter() : nullptr;
#define ONN_LN_FWD(V) launch_overlapped(layernorm_fwd_kernel<V>, dim3(grid), dim3(kRowThreads), 0, s, A, R, gamma, beta, Y, sum, mean, inv_std, row_is_zero, (long long)rows, (int)E, eps, work_counter)
    if(fast)
    {
        switch(vec_count(E))
        {
            case 1: ONN_LN_FWD(1); break;
            case 2: ONN_LN_FWD(2); break;
            case 3: case 4: ONN_LN_FWD(4); break;
            default: ONN_LN_FWD(8); break;
        }
    }
    else
        layernorm_fwd_generic_kernel<<<grid, kRowThreads, 0, s>>>(A, R, gamma, beta, Y, sum, mean, inv_std, row_is_zero, rows, (int)E, eps);
#undef ONN_LN_FWD
    count_launch();
    return launch_status();
}

// Number of CTAs the backward kernel runs with (= partial row pairs in the workspace).
static int layernorm_bwd_grid(int64_t rows) { return grid_for(rows, kRowWarps, 2); }   // two resident CTAs per SM

// floats of partial sums for `sets` running sums per CTA
static size_t layernorm_bwd_partial_floats(int64_t rows, int64_t E, int sets)
{
    if(rows <= 0 || E <= 0) return 0;
    return (size_t)layernorm_bwd_grid(rows) * (size_t)sets * (size_t)E;
}

extern "C" size_t onn_layernorm_bwd_workspace_floats(int64_t rows, int64_t E) { return layernorm_bwd_partial_floats(rows, E, 3); }

namespace onn
{
int launch_colsum_accumulate(const float* D, long long rows, long long cols, long long ld, float* out, cudaStream_t s);

static bool fast_path_sums_dx(const float* dX_colsum, int64_t E) { return dX_colsum != nullptr && E <= 128 * kMaxVec; }

// Shared by the workspace entry point and any other front end: launches the row kernel
// into `partials` and the column reduction into dgamma / dbeta.
int layernorm_bwd_launch(const float* dY, const float* dY2, const float* dY3, const float* X,
                         const float* mean, const float* inv_std, const float* gamma,
                         float* dX, float* dgamma, float* dbeta, float* dX_colsum, int64_t rows, int64_t E,
                         float* partials, uint32_t flags, cudaStream_t s)
{
    const int grid = layernorm_bwd_grid(rows);
    const bool fast = (E & 3) == 0 && E <= 128 * kMaxVec && host_aligned16(dY) && host_aligned16(X) && host_aligned16(dX) &&
                      host_aligned16(gamma) && (!dY2 || host_aligned16(dY2)) && (!dY3 || host_aligned16(dY3));
    const bool dx_sum = fast_path_sums_dx(dX_colsum, E);
    const int sets = dx_sum ? 3 : 2;
    unsigned int* work_counter = rows + (long long)grid * kRowWarps < (1LL << 31) ? next_work_counter() : nullptr;
#define ONN_LN_BWD(V) do { if(dx_sum) launch_overlapped(layernorm_bwd_kernel<V, true>, dim3(grid), dim3(kRowThreads), smem, s, dY, dY2, dY3, X, mean, inv_std, gamma, dX, partials, (long long)rows, (int)E, work_counter); \
                           else launch_overlapped(layernorm_bwd_kernel<V, false>, dim3(grid), dim3(kRowThreads), smem, s, dY, dY2, dY3, X, mean, inv_std, gamma, dX, partials, (long long)rows, (int)E, work_counter); } while(0)
    if(fast)
    {
        const size_t smem = (size_t)kRowWarps * sets * E * sizeof(float);   // 64 KiB (96 KiB with the dx sums) at E = 1024
        // once per device: attribute calls do not belong inside a stream capture, so the first (eager) call sets both
        static PerDeviceBytes configured_plain, configured_sums;
        if(smem > 48 * 1024 && !(ensure_dynamic_smem(layernorm_bwd_kernel<8, false>, configured_plain, 64 * 1024) &&
                                 ensure_dynamic_smem(layernorm_bwd_kernel<8, true>, configured_sums, 96 * 1024))) return ONN_ERR_CUDA;
        switch(vec_count(E))
        {
            case 1: ONN_LN_BWD(1); break;
            case 2: ONN_LN_BWD(2); break;
            case 3: case 4: ONN_LN_BWD(4); break;
            default: ONN_LN_BWD(8); break;
        }
    }
    else
    {
        const size_t smem = (size_t)2 * E * sizeof(float);
        if(smem > 48 * 1024)
        {
            if(smem > 200 * 1024) return ONN_ERR_UNSUPPORTED;
            static PerDeviceBytes configured;
            if(!ensure_dynamic_smem(layernorm_bwd_generic_kernel, configured, smem)) return ONN_ERR_CUDA;
        }
        layernorm_bwd_generic_kernel<<<grid, kRowThreads, smem, s>>>(dY, dY2, dY3, X, mean, inv_std, gamma, dX, partials, rows, (int)E);
    }
#undef ONN_LN_BWD
    count_launch();
    if(launch_status() != ONN_OK) return ONN_ERR_CUDA;
    const int columns = (int)(((fast && dx_sum) ? 3 : 2) * E);
    launch_overlapped(colsum_partials_kernel, dim3((columns + 31) / 32), dim3(256), 0, s, (const float*)partials, grid, columns, dgamma, dbeta, dX_colsum,
                      (int)E, (int)((flags & ONN_ACCUMULATE) != 0));
    count_launch();
    if(launch_status() != ONN_OK) return ONN_ERR_CUDA;
    // rows the vector kernel cannot take: the column sums of dX come from a pass of their own
    if(dX_colsum && !(fast && dx_sum)) return launch_colsum_accumulate(dX, rows, E, E, dX_colsum, s);
    return ONN_OK;
}
}  // namespace onn

extern "C" int onn_layernorm_bwd(const float* dY, const float* dY2, const float* dY3, const float* X,
                                 const float* mean, const float* inv_std, const float* gamma,
                                 float* dX, float* dgamma, float* dbeta, float* dX_colsum,
                                 int64_t rows, int64_t E, float* workspace, uint32_t flags, void* stream)
{
    ONN_CHECK_ARG(dY && X && mean && inv_std && gamma && dX && dgamma && dbeta && rows > 0 && E > 0);
    if(!workspace) return ONN_ERR_WORKSPACE;
    return layernorm_bwd_launch(dY, dY2, dY3, X, mean, inv_std, gamma, dX, dgamma, dbeta, dX_colsum, rows, E, workspace, flags,
                                (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------
// Normalization3d backward for callers that have no way to provide scratch memory
// ---------------------------------------------------------------------------------------

// Room for the per-CTA partial column sums of the largest supported call:
// (2 CTAs per SM) x {sum dy*x_hat, sum dy} x ONN_LAYERNORM_BWD_STATIC_MAX_E floats = 2.3 MiB.
// It lives in the library image, so every GPU that loads the library holds it until exit.
static __device__ __align__(256) float g_layernorm_bwd_static_partials[2 * kSmCount * 2 * ONN_LAYERNORM_BWD_STATIC_MAX_E];

namespace
{
std::mutex g_static_partials_mutex;
float* g_static_partials_address[kMaxDevices] = {};    // device address of the array above, per device

// In host code the array's name is only a handle: the device address has to be asked for, once per
// device, with that device current.
int static_partials_for_current_device(float** address)
{
    int device = -1;
    if(cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return ONN_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_static_partials_mutex);
    if(!g_static_partials_address[device])
    {
        float* resolved = nullptr;
        if(cudaGetSymbolAddress(reinterpret_cast<void**>(&resolved), g_layernorm_bwd_static_partials) != cudaSuccess || !resolved)
            return ONN_ERR_CUDA;
        g_static_partials_address[device] = resolved;
    }
    *address = g_static_partials_address[device];
    return ONN_OK;
}
}  // namespace

extern "C" int onn_layernorm_bwd_static(const float* dY, const float* dY2, const float* dY3, const float* X,
                                        const float* mean, const float* inv_std, const float* gamma,
                                        float* dX, float* dgamma, float* dbeta,
                                        int64_t rows, int64_t E, uint32_t flags, void* stream)
{
    ONN_CHECK_ARG(dY && X && mean && inv_std && gamma && dX && dgamma && dbeta && rows > 0 && E > 0);
    if(E > ONN_LAYERNORM_BWD_STATIC_MAX_E) return ONN_ERR_LIMIT;      // the fixed buffer holds rows of at most this width
    if(layernorm_bwd_partial_floats(rows, E, 2) > sizeof(g_layernorm_bwd_static_partials) / sizeof(float)) return ONN_ERR_LIMIT;
    float* partials = nullptr;
    const int status = static_partials_for_current_device(&partials);
    if(status != ONN_OK) return status;
    // Nothing in the buffer has to start at zero: the row kernel overwrites one partial row pair per CTA
    // and the column reduction reads exactly those, so whatever an earlier call left behind is never read.
    return layernorm_bwd_launch(dY, dY2, dY3, X, mean, inv_std, gamma, dX, dgamma, dbeta, nullptr, rows, E, partials, flags,
                                (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------
// Pooling3d: [B, S, E] -> [B, E] over the sequence
// ---------------------------------------------------------------------------------------

// One CTA per sample: a row is padding when every feature is exactly zero; flags per row, count per sample.
__global__ void __launch_bounds__(kRowThreads)
pooling_valid_rows_kernel(const float* __restrict__ x, uint8_t* __restrict__ row_is_valid, int32_t* __restrict__ valid_count, int S, int E)
{
    __shared__ int warp_counts[kRowWarps];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long b = blockIdx.x;
    int mine = 0;
    for(int s = warp; s < S; s += kRowWarps)
    {
        const float* row = x + (b * S + s) * (long long)E;
        bool any = false;
        for(int e = lane; e < E; e += 32) any = any || row[e] != 0.f;
        any = __any_sync(0xffffffffu, any);
        if(lane == 0) { row_is_valid[b * S + s] = any ? 1 : 0; mine += any ? 1 : 0; }
    }
    if(lane == 0) warp_counts[warp] = mine;
    __syncthreads();
    if(threadIdx.x == 0)
    {
        int total = 0;
        for(int w = 0; w < kRowWarps; w++) total += warp_counts[w];
        valid_count[b] = total;
    }
}

// One thread per (sample, feature), walking the sequence in order (the reference's order of additions and its
// first-position-wins rule for ties of the maximum); neighbouring threads read neighbouring features.
__global__ void pooling_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int32_t* __restrict__ argmax,
                                   const uint8_t* __restrict__ row_is_valid, const int32_t* __restrict__ valid_count,
                                   long long B, int S, int E, int method)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    for(long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < B * E; i += stride)
    {
        const long long b = i / E;
        const int f = (int)(i % E);
        const float* column = x + b * S * (long long)E + f;
        if(method == 0)
        {
            float best = -INFINITY;
            int where = 0;
            for(int s = 0; s < S; s++)
            {
                const float value = column[(long long)s * E];
                if(value > best) { best = value; where = s; }
            }
            y[i] = best;
            if(argmax) argmax[i] = where;
        }
        else
        {
            float total = 0.f;
            for(int s = 0; s < S; s++)
                if(row_is_valid[b * S + s]) total += column[(long long)s * E];
            const int count = valid_count[b];
            y[i] = count > 0 ? total / (float)count : total;
        }
    }
}

__global__ void pooling_bwd_kernel(const float* __restrict__ dy, const int32_t* __restrict__ argmax, const uint8_t* __restrict__ row_is_valid,
                                   const int32_t* __restrict__ valid_count, float* __restrict__ dx, long long B, int S, int E, int method)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    for(long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < B * E; i += stride)
    {
        const long long b = i / E;
        const int f = (int)(i % E);
        float* column = dx + b * S * (long long)E + f;
        const float delta = dy[i];
        if(method == 0)
        {
            const int where = argmax[i];
            for(int s = 0; s < S; s++) column[(long long)s * E] = s == where ? delta : 0.f;
        }
        else
        {
            const int count = valid_count[b];
            const float share = count > 0 ? delta * (1.0f / (float)count) : 0.f;
            for(int s = 0; s < S; s++) column[(long long)s * E] = (count > 0 && row_is_valid[b * S + s]) ? share : 0.f;
        }
    }
}

extern "C" int onn_pooling3d_fwd(const float* x, float* y, int32_t* argmax, uint8_t* row_is_valid, int32_t* valid_count,
                                 int64_t B, int64_t S, int64_t E, int method, void* stream)
{
    ONN_CHECK_ARG(x && y && B > 0 && S > 0 && E > 0 && S < (1LL << 31) && E < (1LL << 31) && (method == 0 || method == 1));
    ONN_CHECK_ARG(method == 0 || (row_is_valid && valid_count));
    cudaStream_t s = (cudaStream_t)stream;
    if(method == 1)
    {
        pooling_valid_rows_kernel<<<(unsigned)B, kRowThreads, 0, s>>>(x, row_is_valid, valid_count, (int)S, (int)E);
        count_launch();
        if(launch_status() != ONN_OK) return ONN_ERR_CUDA;
    }
    pooling_fwd_kernel<<<grid_for(B * E, 256, 8), 256, 0, s>>>(x, y, argmax, row_is_valid, valid_count, B, (int)S, (int)E, method);
    count_launch();
    return launch_status();
}

extern "C" int onn_pooling3d_bwd(const float* dy, const int32_t* argmax, const uint8_t* row_is_valid, const int32_t* valid_count,
                                 float* dx, int64_t B, int64_t S, int64_t E, int method, void* stream)
{
    ONN_CHECK_ARG(dy && dx && B > 0 && S > 0 && E > 0 && S < (1LL << 31) && E < (1LL << 31) && (method == 0 || method == 1));
    ONN_CHECK_ARG(method == 0 ? argmax != nullptr : (row_is_valid && valid_count));
    pooling_bwd_kernel<<<grid_for(B * E, 256, 8), 256, 0, (cudaStream_t)stream>>>(dy, argmax, row_is_valid, valid_count, dx, B, (int)S, (int)E, method);
    count_launch();
    return launch_status();
}

// Token ids arrive from the data feed as 32-bit integers; the layers read them as floats holding integers
// (the reference's convention), which is exact up to 2^24.
__global__ void ids_to_float_kernel(const int32_t* __restrict__ ids, float* __restrict__ out, long long n)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    for(long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = (float)ids[i];
}

extern "C" int onn_ids_to_float(const int32_t* ids, float* out, int64_t n, void* stream)
{
    ONN_CHECK_ARG(ids && out && n > 0);
    ids_to_float_kernel<<<grid_for(n, 256, 8), 256, 0, (cudaStream_t)stream>>>(ids, out, n);
    count_launch();
    return launch_status();
}

extern "C" int onn_add(const float* a, const float* b, float* out, int64_t n, uint32_t flags, void* stream)
{
    ONN_CHECK_ARG(a && b && out && n > 0);
    const int grid = grid_for((n + 3) / 4, 256, 8);
    add_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a, b, out, n);
    count_launch();
    return launch_status();
}

