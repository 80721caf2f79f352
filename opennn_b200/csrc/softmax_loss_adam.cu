// HBM-bound kernels around the contractions: masked attention softmax (+ backward), plain
// row softmax, the fused CrossEntropyError3d pass, column sums for bias gradients, the
// ReLU-derivative product, the gradient norm and the fused clip + Adam update.
#include <float.h>

#include "common.cuh"
#include "launch_counter.h"
#include "rowwise_internal.h"

namespace onn
{

// ---------------------------------------------------------------------------------------
// Attention softmax: scores [B, H, Sq, Sk] in place.  One warp per (b, h, q) row.
//   key padding: score := -1e9 where the source row is all-zero (overwrite);
//   causal:      score += -inf for key > query.
// ---------------------------------------------------------------------------------------

__global__ void __launch_bounds__(256)
source_row_is_zero_kernel(const float* __restrict__ X, uint8_t* __restrict__ flags, long long rows, int E)
{
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const long long stride = (long long)gridDim.x * 8;
    for(long long row = warp; row < rows; row += stride)
    {
        bool zero = true;
        for(int e = lane; e < E; e += 32) zero = zero && fabsf(X[row * (long long)E + e]) <= 1e-7f;
        zero = __all_sync(0xffffffffu, zero);
        if(lane == 0) flags[row] = zero ? 1 : 0;
    }
}

template <int PER_LANE>   // Sk <= 32 * PER_LANE, row in registers
__global__ void __launch_bounds__(256)
attention_softmax_kernel(float* __restrict__ scores, const uint8_t* __restrict__ key_is_pad,
                         long long rows, int H, int Sq, int Sk, int causal)
{
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const long long stride = (long long)gridDim.x * 8;
    for(long long row = warp; row < rows; row += stride)
    {
        const int q = (int)(row % Sq);
        const long long b = row / ((long long)Sq * H);
        const uint8_t* pad = key_is_pad ? key_is_pad + b * Sk : nullptr;
        float* p = scores + row * (long long)Sk;
        float v[PER_LANE];
        float row_max = -INFINITY;
#pragma unroll
        for(int i = 0; i < PER_LANE; i++)
        {
            const int k = i * 32 + lane;
            v[i] = -INFINITY;
            if(k < Sk)
            {
                float s = p[k];
                if(pad && pad[k]) s = -1e9f;
                if(causal && k > q) s = -INFINITY;
                v[i] = s;
            }
            row_max = fmaxf(row_max, v[i]);
        }
        row_max = warp_max(row_max);
        float total = 0.f;
#pragma unroll
        for(int i = 0; i < PER_LANE; i++)
        {
            v[i] = (i * 32 + lane < Sk) ? __expf(v[i] - row_max) : 0.f;
            total += v[i];
        }
        total = warp_sum(total);
        const float inv = total > 0.f ? 1.0f / total : 0.f;
#pragma unroll
        for(int i = 0; i < PER_LANE; i++)
        {
            const int k = i * 32 + lane;
            if(k < Sk) p[k] = (v[i] * inv);
        }
    }
}

// 128-bit variant for Sk % 4 == 0: each lane owns VEC float4 of the row (Sk <= 128 * VEC).
template <int VEC>
__global__ void __launch_bounds__(256)
attention_softmax_vec_kernel(float* __restrict__ scores, const uint8_t* __restrict__ key_is_pad,
                             long long rows, int H, int Sq, int Sk, int causal)
{
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const long long stride = (long long)gridDim.x * 8;
    for(long long row = warp; row < rows; row += stride)
    {
        const int q = (int)(row % Sq);
        const long long b = row / ((long long)Sq * H);
        const uint8_t* pad = key_is_pad ? key_is_pad + b * Sk : nullptr;
        float* p = scores + row * (long long)Sk;
        float4 v[VEC];
        float row_max = -INFINITY;
#pragma unroll
        for(int i = 0; i < VEC; i++)
        {
            const int k = (i * 32 + lane) * 4;
            v[i] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            if(k < Sk)
            {
                v[i] = ld4_stream(p + k);
                if(pad)
                {
                    const uchar4 f = *reinterpret_cast<const uchar4*>(pad + k);
                    if(f.x) v[i].x = -1e9f; if(f.y) v[i].y = -1e9f; if(f.z) v[i].z = -1e9f; if(f.w) v[i].w = -1e9f;
                }
                if(causal)
                {
                    if(k > q) v[i].x = -INFINITY; if(k + 1 > q) v[i].y = -INFINITY;
                    if(k + 2 > q) v[i].z = -INFINITY; if(k + 3 > q) v[i].w = -INFINITY;
                }
            }
            row_max = fmaxf(row_max, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
        }
        row_max = warp_max(row_max);
        float total = 0.f;
#pragma unroll
        for(int i = 0; i < VEC; i++)
        {
            v[i].x = __expf(v[i].x - row_max); v[i].y = __expf(v[i].y - row_max);
            v[i].z = __expf(v[i].z - row_max); v[i].w = __expf(v[i].w - row_max);
            total += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
        total = warp_sum(total);
        const float inv = total > 0.f ? 1.0f / total : 0.f;
#pragma unroll
        for(int i = 0; i < VEC; i++)
        {
            const int k = (i * 32 + lane) * 4;
            if(k < Sk) st4(p + k, make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv));
        }
    }
}

// Any Sk: three sweeps through global memory (the row stays in L1/L2).
__global__ void __launch_bounds__(256)
attention_softmax_generic_kernel(float* __restrict__ scores, const uint8_t* __restrict__ key_is_pad,
                                 long long rows, int H, int Sq, int Sk, int causal)
{
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const long long stride = (long long)gridDim.x * 8;
    for(long long row = warp; row < rows; row += stride)
    {
        const int q = (int)(row % Sq);
        const long long b = row / ((long long)Sq * H);
        const uint8_t* pad = key_is_pad ? key_is_pad + b * Sk : nullptr;
        float* p = scores + row * (long long)Sk;
        float row_max = -INFINITY;
        for(int k = lane; k < Sk; k += 32)
        {
            float s = p[k];
            if(pad && pad[k]) s = -1e9f;
            if(causal && k > q) s = -INFINITY;
            p[k] = s;
            row_max = fmaxf(row_max, s);
        }
        row_max = warp_max(row_max);
        float total = 0.f;
        for(int k = lane; k < Sk; k += 32) { const float e = __expf(p[k] - row_max); p[k] = e; total += e; }
        total = warp_sum(total);
        const float inv = total > 0.f ? 1.0f / total : 0.f;
        for(int k = lane; k < Sk; k += 32) p[k] = (p[k] * inv);
    }
}

// dS = P * (dP - rowsum(P * dP)), in place over dP.
template <int PER_LANE>
__global__ void __launch_bounds__(256)
attention_softmax_bwd_kernel(const float* __restrict__ P, float* __restrict__ dP, long long rows, int Sk)
{
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const long long stride = (long long)gridDim.x * 8;
    for(long long row = warp; row < rows; row += stride)
    {
        const float* p = P + row * (long long)Sk;
        float* d = dP + row * (long long)Sk;
        float pv[PER_LANE], dv[PER_LANE];
        float dot = 0.f;
#pragma unroll
        for(int i = 0; i < PER_LANE; i++)
        {
            const int k = i * 32 + lane;
            pv[i] = k < Sk ? p[k] : 0.f;
            dv[i] = k < Sk ? d[k] : 0.f;
            dot += pv[i] * dv[i];
        }
        dot = warp_sum(dot);
#pragma unroll
        for(int i = 0; i < PER_LANE; i++)
        {
            const int k = i * 32 + lane;
            if(k < Sk) d[k] = (pv[i] * (dv[i] - dot));
        }
    }
}

__global__ void __launch_bounds__(256)
attention_softmax_bwd_generic_kernel(const float* __restrict__ P, float* __restrict__ dP, long long rows, int Sk)
{
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const long long stride = (long long)gridDim.x * 8;
    for(long long row = warp; row < rows; row += stride)
    {
        const float* p = P + row * (long long)Sk;
        float* d = dP + row * (long long)Sk;
        float dot = 0.f;
        for(int k = lane; k < Sk; k += 32) dot += p[k] * d[k];
        dot = warp_sum(dot);
        for(int k = lane; k < Sk; k += 32) d[k] = (p[k] * (d[k] - dot));
    }
}

// ---------------------------------------------------------------------------------------
// Row softmax / CrossEntropyError3d: one CTA per token row of V logits.
// Sweep 1 (DRAM): online max + sum of exp + argmax.  Sweep 2 (L2): write p or the gradient.
// ---------------------------------------------------------------------------------------

constexpr int kLossThreads = 256;

struct RowStats { float max; float sum; int argmax; };

__device__ __forceinline__ void online_update(float x, int index, float& m, float& s, int& arg)
{
    if(x > m) { s = s * __expf(m - x) + 1.0f; m = x; arg = index; }
    else s += __expf(x - m);
}

__device__ __forceinline__ RowStats row_statistics(const float* __restrict__ row, int V, float* scratch_f, int* scratch_i)
{
    float m = -INFINITY, s = 0.f;
    int arg = 0x7fffffff;
    const bool vec = (V & 3) == 0 && aligned16(row);
    if(vec)
    {
        for(int i = threadIdx.x * 4; i < V; i += kLossThreads * 4)
        {
            const float4 x = ld4(row + i);
            online_update(x.x, i, m, s, arg); online_update(x.y, i + 1, m, s, arg);
            online_update(x.z, i + 2, m, s, arg); online_update(x.w, i + 3, m, s, arg);
        }
    }
    else
        for(int i = threadIdx.x; i < V; i += kLossThreads) online_update(row[i], i, m, s, arg);

    // combine (max, sum, argmax) across the CTA; ties resolve to the smallest index,
    // matching the reference's first-maximum scan.
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for(int offset = 16; offset > 0; offset >>= 1)
    {
        const float om = __shfl_xor_sync(0xffffffffu, m, offset);
        const float os = __shfl_xor_sync(0xffffffffu, s, offset);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, offset);
        const float nm = fmaxf(m, om);
        const float a = (m == -INFINITY) ? 0.f : s * __expf(m - nm);
        const float b = (om == -INFINITY) ? 0.f : os * __expf(om - nm);
        if(om > m || (om == m && oa < arg)) arg = oa;
        m = nm; s = a + b;
    }
    __syncthreads();
    if(lane == 0) { scratch_f[warp] = m; scratch_f[8 + warp] = s; scratch_i[warp] = arg; }
    __syncthreads();
    RowStats r;
    r.max = scratch_f[0]; r.sum = scratch_f[8]; r.argmax = scratch_i[0];
#pragma unroll
    for(int w = 1; w < kLossThreads / 32; w++)
    {
        const float om = scratch_f[w], os = scratch_f[8 + w];
        const int oa = scratch_i[w];
        const float nm = fmaxf(r.max, om);
        const float a = (r.max == -INFINITY) ? 0.f : r.sum * __expf(r.max - nm);
        const float b = (om == -INFINITY) ? 0.f : os * __expf(om - nm);
        if(om > r.max || (om == r.max && oa < r.argmax)) r.argmax = oa;
        r.max = nm; r.sum = a + b;
    }
    return r;
}

__global__ void __launch_bounds__(kLossThreads)
softmax_rows_kernel(float* __restrict__ Y, int V)
{
    __shared__ float scratch_f[16];
    __shared__ int scratch_i[8];
    float* row = Y + (long long)blockIdx.x * V;
    const RowStats st = row_statistics(row, V, scratch_f, scratch_i);
    const float inv = st.sum > 0.f ? 1.0f / st.sum : 0.f;
    const bool vec = (V & 3) == 0 && aligned16(row);
    if(vec)
        for(int i = threadIdx.x * 4; i < V; i += kLossThreads * 4)
        {
            float4 x = ld4(row + i);
            x.x = __expf(x.x - st.max) * inv; x.y = __expf(x.y - st.max) * inv;
            x.z = __expf(x.z - st.max) * inv; x.w = __expf(x.w - st.max) * inv;
            st4(row + i, x);
        }
    else
        for(int i = threadIdx.x; i < V; i += kLossThreads) row[i] = __expf(row[i] - st.max) * inv;
}

__global__ void count_active_kernel(const float* __restrict__ targets, long long rows, long long V, float* __restrict__ count)
{
    __shared__ float scratch[32];
    float mine = 0.f;
    for(long long i = threadIdx.x; i < rows; i += blockDim.x)
    {
        const long long t = token_index(targets[i]);
        mine += (t > 0 && t < V) ? 1.f : 0.f;
    }
    const float total = block_sum(mine, scratch);
    if(threadIdx.x == 0) count[0] = total;
}

// In place: logits -> gradient (p - onehot) / active on active rows, 0 on inactive rows.
// row_scratch[row] = -log(p[target] + eps) (0 if inactive); row_scratch[rows + row] = correct.
__global__ void __launch_bounds__(kLossThreads)
ce3d_fwd_bwd_kernel(float* __restrict__ logits, const float* __restrict__ targets, const float* __restrict__ active_count,
                    float* __restrict__ probabilities_out, float* __restrict__ row_scratch,
                    long long rows, int V, int inputs_are_probabilities)
{
    __shared__ float scratch_f[16];
    __shared__ int scratch_i[8];
    const long long r = blockIdx.x;
    float* row = logits + r * (long long)V;
    float* p_out = probabilities_out ? probabilities_out + r * (long long)V : nullptr;
    const long long target = token_index(targets[r]);
    const bool active = target > 0 && target < V;
    const float count = active_count[0];
    const float scale = count > 0.f ? 1.0f / count : 0.f;
    const bool vec = (V & 3) == 0 && aligned16(row) && (!p_out || aligned16(p_out));

    if(!active && !p_out)
    {
        // nothing of this row is needed: the gradient is zero and it adds nothing to the loss
        if(vec) for(int i = threadIdx.x * 4; i < V; i += kLossThreads * 4) st4(row + i, make_float4(0.f, 0.f, 0.f, 0.f));
        else for(int i = threadIdx.x; i < V; i += kLossThreads) row[i] = 0.f;
        if(threadIdx.x == 0) { row_scratch[r] = 0.f; row_scratch[rows + r] = 0.f; }
        return;
    }

    const RowStats st = row_statistics(row, V, scratch_f, scratch_i);
    // probabilities in: exp(x - max)/sum would distort them; use them as they are
    const float shift = inputs_are_probabilities ? 0.f : st.max;
    const float inv = inputs_are_probabilities ? 1.0f : (st.sum > 0.f ? 1.0f / st.sum : 0.f);

    if(threadIdx.x == 0)
    {
        float term = 0.f, correct = 0.f;
        if(active)
        {
            const float x = row[target];
            const float p = inputs_are_probabilities ? x : __expf(x - shift) * inv;
            term = -logf(p + FLT_EPSILON);
            correct = (st.argmax == (int)target) ? 1.f : 0.f;
        }
        row_scratch[r] = term;
        row_scratch[rows + r] = correct;
    }
    __syncthreads();   // the target logit is read before anyone overwrites it

    const int t = active ? (int)target : -1;
#define ONN_CE_ELEMENT(x, index)                                                         \
    {                                                                                    \
        const float p = inputs_are_probabilities ? (x) : __expf((x) - shift) * inv;      \
        const float g = active ? (p - ((index) == t ? 1.0f : 0.0f)) * scale : 0.0f;      \
        pr = p; (x) = (g);                                             \
    }
    if(vec)
        for(int i = threadIdx.x * 4; i < V; i += kLossThreads * 4)
        {
            float4 x = ld4(row + i), pq;
            float pr;
            ONN_CE_ELEMENT(x.x, i) pq.x = pr;
            ONN_CE_ELEMENT(x.y, i + 1) pq.y = pr;
            ONN_CE_ELEMENT(x.z, i + 2) pq.z = pr;
            ONN_CE_ELEMENT(x.w, i + 3) pq.w = pr;
            st4_stream(row + i, x);
            if(p_out) st4_stream(p_out + i, pq);
        }
    else
        for(int i = threadIdx.x; i < V; i += kLossThreads)
        {
            float x = row[i], pr;
            ONN_CE_ELEMENT(x, i)
            row[i] = x;
            if(p_out) p_out[i] = pr;
        }
#undef ONN_CE_ELEMENT
}

// stats = {sum of loss terms, #correct, #active, 0}: one CTA, fixed order -> deterministic.
__global__ void ce3d_finish_kernel(const float* __restrict__ row_scratch, const float* __restrict__ targets,
                                   long long rows, long long V, float* __restrict__ stats)
{
    __shared__ float scratch[32];
    float loss = 0.f, correct = 0.f, active = 0.f;
    for(long long i = threadIdx.x; i < rows; i += blockDim.x)
    {
        loss += row_scratch[i];
        correct += row_scratch[rows + i];
        const long long t = token_index(targets[i]);
        active += (t > 0 && t < V) ? 1.f : 0.f;
    }
    loss = block_sum(loss, scratch);
    correct = block_sum(correct, scratch);
    active = block_sum(active, scratch);
    if(threadIdx.x == 0) { stats[0] = loss; stats[1] = correct; stats[2] = active; stats[3] = 0.f; }
}

// ---------------------------------------------------------------------------------------
// Bias gradient (column sums) and ReLU derivative
// ---------------------------------------------------------------------------------------

// out[c] += sum over rows of D[r][c].  Each CTA owns a 32-column strip and a slab of rows,
// sums it in registers / shared memory and issues one atomic per column.
__global__ void __launch_bounds__(256)
colsum_accumulate_kernel(const float* __restrict__ D, long long rows, long long cols, long long ld,
                         long long rows_per_block, float* __restrict__ out)
{
    __shared__ float tile[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const long long c = (long long)blockIdx.x * 32 + tx;
    const long long r0 = (long long)blockIdx.y * rows_per_block;
    const long long r1 = min(rows, r0 + rows_per_block);
    float total = 0.f;
    if(c < cols)
        for(long long r = r0 + ty; r < r1; r += 8) total += D[r * ld + c];
    tile[ty][tx] = total;
    __syncthreads();
    if(ty == 0 && c < cols)
    {
        float sum = 0.f;
#pragma unroll
        for(int w = 0; w < 8; w++) sum += tile[w][tx];
        atomicAdd(out + c, sum);
    }
}

// Same sums for 16-byte aligned rows: each CTA owns a 128-column strip (one float4 per lane)
// and a slab of rows; 8 warps stride the slab with four independent loads in flight each.
__global__ void __launch_bounds__(256)
colsum_accumulate_vec_kernel(const float* __restrict__ D, long long rows, long long cols, long long ld,
                             long long rows_per_block, float* __restrict__ out)
{
    __shared__ float4 partial[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long c = (long long)blockIdx.x * 128 + lane * 4;
    const long long r0 = (long long)blockIdx.y * rows_per_block;
    const long long r1 = min(rows, r0 + rows_per_block);
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a, e = a, f = a;
    if(c < cols)
    {
        long long r = r0 + warp;
        for(; r + 24 < r1; r += 32)
        {
            const float4 x0 = ld4_stream(D + r * ld + c), x1 = ld4_stream(D + (r + 8) * ld + c);
            const float4 x2 = ld4_stream(D + (r + 16) * ld + c), x3 = ld4_stream(D + (r + 24) * ld + c);
            a.x += x0.x; a.y += x0.y; a.z += x0.z; a.w += x0.w;
            b.x += x1.x; b.y += x1.y; b.z += x1.z; b.w += x1.w;
            e.x += x2.x; e.y += x2.y; e.z += x2.z; e.w += x2.w;
            f.x += x3.x; f.y += x3.y; f.z += x3.z; f.w += x3.w;
        }
        for(; r < r1; r += 8)
        {
            const float4 x0 = ld4_stream(D + r * ld + c);
            a.x += x0.x; a.y += x0.y; a.z += x0.z; a.w += x0.w;
        }
    }
    partial[warp][lane] = make_float4((a.x + b.x) + (e.x + f.x), (a.y + b.y) + (e.y + f.y), (a.z + b.z) + (e.z + f.z), (a.w + b.w) + (e.w + f.w));
    __syncthreads();
    if(warp == 0 && c < cols)
    {
        float4 total = partial[0][lane];
#pragma unroll
        for(int w = 1; w < 8; w++) { const float4 t = partial[w][lane]; total.x += t.x; total.y += t.y; total.z += t.z; total.w += t.w; }
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                     :: "l"(out + c), "f"(total.x), "f"(total.y), "f"(total.z), "f"(total.w) : "memory");
    }
}

// delta = dY * (Y > 0), in place over dY.
__global__ void relu_delta_kernel(float* __restrict__ dY, const float* __restrict__ Y, long long n)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long n4 = (aligned16(dY) && aligned16(Y)) ? n / 4 : 0;
    for(long long i = tid; i < n4; i += stride)
    {
        float4 d = ld4(dY + 4 * i);
        const float4 y = ld4_stream(Y + 4 * i);
        d.x = y.x > 0.f ? (d.x) : 0.f; d.y = y.y > 0.f ? (d.y) : 0.f;
        d.z = y.z > 0.f ? (d.z) : 0.f; d.w = y.w > 0.f ? (d.w) : 0.f;
        st4(dY + 4 * i, d);
    }
    for(long long i = 4 * n4 + tid; i < n; i += stride) dY[i] = Y[i] > 0.f ? (dY[i]) : 0.f;
}

// ---------------------------------------------------------------------------------------
// Gradient norm and Adam
// ---------------------------------------------------------------------------------------

constexpr int kNormBlocks = kSmCount * 4;

__global__ void __launch_bounds__(256)
sqnorm_partial_kernel(const float* __restrict__ g, long long n, float* __restrict__ partials)
{
    __shared__ float scratch[32];
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long n4 = aligned16(g) ? n / 4 : 0;
    float a = 0.f, b = 0.f;
    for(long long i = tid; i < n4; i += stride)
    {
        const float4 x = ld4(g + 4 * i);
        a += x.x * x.x + x.y * x.y; b += x.z * x.z + x.w * x.w;
    }
    for(long long i = 4 * n4 + tid; i < n; i += stride) a += g[i] * g[i];
    const float total = block_sum(a + b, scratch);
    if(threadIdx.x == 0) partials[blockIdx.x] = total;
}

__global__ void sqnorm_finish_kernel(const float* __restrict__ partials, int count, float* __restrict__ out)
{
    double mine = 0.0;   // few hundred terms: double keeps the final sum order-insensitive in fp32
    for(int i = threadIdx.x; i < count; i += blockDim.x) mine += (double)partials[i];
    // fold doubles through shuffles
    for(int offset = 16; offset > 0; offset >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, offset);
    __shared__ double warp_totals[32];
    if((threadIdx.x & 31) == 0) warp_totals[threadIdx.x >> 5] = mine;
    __syncthreads();
    if(threadIdx.x == 0)
    {
        double total = 0.0;
        for(int w = 0; w < (int)((blockDim.x + 31) >> 5); w++) total += warp_totals[w];
        out[0] = (float)total;
    }
}

__global__ void __launch_bounds__(256)
adam_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v, float* __restrict__ g,
            long long n, float lr, float beta1, float beta2, float eps,
            float bc1, float bc2, float clip_norm, const float* __restrict__ sqnorm, float grad_scale, int zero_grad,
            const unsigned int* __restrict__ skip_if_nonzero)
{
    // a step whose kernels gave up on a bounded wait holds an incomplete gradient: leave p, m, v and g as they are
    if(skip_if_nonzero && skip_if_nonzero[0] != 0u) return;
    float scale = grad_scale;
    if(sqnorm && clip_norm > 0.f)
    {
        const float norm = sqrtf(sqnorm[0]) * fabsf(grad_scale);
        if(norm > clip_norm) scale *= clip_norm / norm;
    }
    const float one_minus_b1 = 1.0f - beta1, one_minus_b2 = 1.0f - beta2;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool vec = aligned16(p) && aligned16(m) && aligned16(v) && aligned16(g);
    const long long n4 = vec ? n / 4 : 0;

#define ONN_ADAM_ELEMENT(pp, mm, vv, gg)                                   \
    {                                                                      \
        const float ge = (gg) * scale;                                     \
        (mm) = beta1 * (mm) + one_minus_b1 * ge;                           \
        (vv) = beta2 * (vv) + one_minus_b2 * ge * ge;                      \
        (pp) -= lr * ((mm) / bc1) / (sqrtf((vv) / bc2) + eps);       \
    }
    for(long long i = tid; i < n4; i += stride)
    {
        float4 pp = ld4(p + 4 * i), mm = ld4(m + 4 * i), vv = ld4(v + 4 * i);
        const float4 gg = ld4(g + 4 * i);
        ONN_ADAM_ELEMENT(pp.x, mm.x, vv.x, gg.x)
        ONN_ADAM_ELEMENT(pp.y, mm.y, vv.y, gg.y)
        ONN_ADAM_ELEMENT(pp.z, mm.z, vv.z, gg.z)
        ONN_ADAM_ELEMENT(pp.w, mm.w, vv.w, gg.w)
        st4(p + 4 * i, pp); st4(m + 4 * i, mm); st4(v + 4 * i, vv);
        if(zero_grad) st4(g + 4 * i, make_float4(0.f, 0.f, 0.f, 0.f));
    }
    for(long long i = 4 * n4 + tid; i < n; i += stride)
    {
        float pp = p[i], mm = m[i], vv = v[i];
        ONN_ADAM_ELEMENT(pp, mm, vv, g[i])
        p[i] = pp; m[i] = mm; v[i] = vv;
        if(zero_grad) g[i] = 0.f;
    }
#undef ONN_ADAM_ELEMENT
}

// ---------------------------------------------------------------------------------------
// Internal launchers used by the layer front ends
// ---------------------------------------------------------------------------------------

int launch_source_row_is_zero(const float* X, uint8_t* flags, long long rows, int E, cudaStream_t s)
{
    source_row_is_zero_kernel<<<grid_for(rows, 8, 8), 256, 0, s>>>(X, flags, rows, E);
    count_launch();
    return launch_status();
}

int launch_attention_softmax(float* scores, const uint8_t* key_is_pad, long long B, int H, int Sq, int Sk,
                             int causal, cudaStream_t s)
{
    const long long rows = B * H * Sq;
    const int grid = grid_for(rows, 8, 8);
    if((Sk & 3) == 0 && Sk <= 1024 && host_aligned16(scores))
    {
#define ONN_SMV(N) attention_softmax_vec_kernel<N><<<grid, 256, 0, s>>>(scores, key_is_pad, rows, H, Sq, Sk, causal)
        if(Sk <= 128) ONN_SMV(1);
        else if(Sk <= 256) ONN_SMV(2);
        else if(Sk <= 512) ONN_SMV(4);
        else ONN_SMV(8);
#undef ONN_SMV
        count_launch();
        return launch_status();
    }
#define ONN_SM(N) attention_softmax_kernel<N><<<grid, 256, 0, s>>>(scores, key_is_pad, rows, H, Sq, Sk, causal)
    if(Sk <= 32) ONN_SM(1);
    else if(Sk <= 64) ONN_SM(2);
    else if(Sk <= 128) ONN_SM(4);
    else if(Sk <= 256) ONN_SM(8);
    else if(Sk <= 512) ONN_SM(16);
    else if(Sk <= 1024) ONN_SM(32);
    else attention_softmax_generic_kernel<<<grid, 256, 0, s>>>(scores, key_is_pad, rows, H, Sq, Sk, causal);
#undef ONN_SM
    count_launch();
    return launch_status();
}

int launch_attention_softmax_bwd(const float* P, float* dP, long long rows, int Sk, cudaStream_t s)
{
    const int grid = grid_for(rows, 8, 8);
#define ONN_SB(N) attention_softmax_bwd_kernel<N><<<grid, 256, 0, s>>>(P, dP, rows, Sk)
    if(Sk <= 32) ONN_SB(1);
    else if(Sk <= 64) ONN_SB(2);
    else if(Sk <= 128) ONN_SB(4);
    else if(Sk <= 256) ONN_SB(8);
    else if(Sk <= 512) ONN_SB(16);
    else attention_softmax_bwd_generic_kernel<<<grid, 256, 0, s>>>(P, dP, rows, Sk);
#undef ONN_SB
    count_launch();
    return launch_status();
}

int launch_colsum_accumulate(const float* D, long long rows, long long cols, long long ld, float* out, cudaStream_t s)
{
    if((cols & 3) == 0 && (ld & 3) == 0 && host_aligned16(D) && host_aligned16(out))
    {
        const long long strips = (cols + 127) / 128;
        long long slabs = (4LL * kSmCount + strips - 1) / strips;       // ~4 CTAs per SM overall
        if(slabs > (rows + 63) / 64) slabs = (rows + 63) / 64;
        if(slabs < 1) slabs = 1;
        if(slabs > 65535) slabs = 65535;
        const long long rows_per_block = (rows + slabs - 1) / slabs;
        dim3 grid((unsigned)strips, (unsigned)((rows + rows_per_block - 1) / rows_per_block));
        colsum_accumulate_vec_kernel<<<grid, 256, 0, s>>>(D, rows, cols, ld, rows_per_block, out);
        count_launch();
        return launch_status();
    }
    const long long strips = (cols + 31) / 32;
    long long slabs = (2LL * kSmCount + strips - 1) / strips;          // ~2 CTAs per SM overall
    if(slabs > (rows + 255) / 256) slabs = (rows + 255) / 256;
    if(slabs < 1) slabs = 1;
    const long long rows_per_block = (rows + slabs - 1) / slabs;
    dim3 grid((unsigned)strips, (unsigned)slabs);
    colsum_accumulate_kernel<<<grid, 256, 0, s>>>(D, rows, cols, ld, rows_per_block, out);
    count_launch();
    return launch_status();
}

// Sigmoid activation (opennn/layer.h:196-204) in place, and its delta dY * y (1 - y) in place on dY.
__global__ void sigmoid_kernel(float* __restrict__ Y, long long n)
{
    for(long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        Y[i] = 1.0f / (1.0f + expf(-Y[i]));
}

__global__ void sigmoid_delta_kernel(float* __restrict__ dY, const float* __restrict__ Y, long long n)
{
    for(long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    {
        const float y = Y[i];
        dY[i] = dY[i] * (y * (1.0f - y));
    }
}

int launch_sigmoid(float* Y, long long n, cudaStream_t s)
{
    sigmoid_kernel<<<grid_for(n, 256, 8), 256, 0, s>>>(Y, n);
    count_launch();
    return launch_status();
}

int launch_sigmoid_delta(float* dY, const float* Y, long long n, cudaStream_t s)
{
    sigmoid_delta_kernel<<<grid_for(n, 256, 8), 256, 0, s>>>(dY, Y, n);
    count_launch();
    return launch_status();
}

int launch_relu_delta(float* dY, const float* Y, long long n, cudaStream_t s)
{
    relu_delta_kernel<<<grid_for((n + 3) / 4, 256, 8), 256, 0, s>>>(dY, Y, n);
    count_launch();
    return launch_status();
}

}  // namespace onn

using namespace onn;

extern "C" int onn_softmax_rows(float* Y, int64_t rows, int64_t cols, void* stream)
{
    ONN_CHECK_ARG(Y && rows > 0 && cols > 0 && rows < (1LL << 31) && cols < (1LL << 31));
    softmax_rows_kernel<<<(unsigned)rows, kLossThreads, 0, (cudaStream_t)stream>>>(Y, (int)cols);
    count_launch();
    return launch_status();
}

// Greedy decoding step: per sample the arg-max (first index on ties) of one distribution, written as a float id into
// the sample's id row unless the sample already produced END; finished[b] is set on END.
__global__ void __launch_bounds__(1024)
greedy_next_token_kernel(const float* __restrict__ probabilities, long long sample_stride, float* __restrict__ ids, long long ids_stride,
                         int write_position, int* __restrict__ finished, int V, int end_id)
{
    __shared__ float best_value[1024];
    __shared__ int best_index[1024];
    const int b = blockIdx.x;
    const float* row = probabilities + (long long)b * sample_stride;
    float value = -INFINITY;
    int index = 0x7fffffff;
    // each thread walks its indices upwards and keeps the first of its maxima
    if((((uintptr_t)row) & 15) == 0)
    {
        const int quads = V >> 2;
        const float4* row4 = reinterpret_cast<const float4*>(row);
#pragma unroll 4
        for(int k4 = threadIdx.x; k4 < quads; k4 += blockDim.x)
        {
            const float4 x = row4[k4];
            if(x.x > value) { value = x.x; index = 4 * k4; }
            if(x.y > value) { value = x.y; index = 4 * k4 + 1; }
            if(x.z > value) { value = x.z; index = 4 * k4 + 2; }
            if(x.w > value) { value = x.w; index = 4 * k4 + 3; }
        }
        for(int k = 4 * quads + threadIdx.x; k < V; k += blockDim.x)
            if(row[k] > value) { value = row[k]; index = k; }
    }
    else
        for(int k = threadIdx.x; k < V; k += blockDim.x)
            if(row[k] > value) { value = row[k]; index = k; }
    best_value[threadIdx.x] = value;
    best_index[threadIdx.x] = index;
    __syncthreads();
    for(int step = blockDim.x / 2; step > 0; step >>= 1)
    {
        if(threadIdx.x < step)
        {
            const float other = best_value[threadIdx.x + step];
            const int other_index = best_index[threadIdx.x + step];
            if(other > best_value[threadIdx.x] || (other == best_value[threadIdx.x] && other_index < best_index[threadIdx.x]))
            {
                best_value[threadIdx.x] = other;
                best_index[threadIdx.x] = other_index;
            }
        }
        __syncthreads();
    }
    if(threadIdx.x == 0 && !finished[b])
    {
        const int token = best_index[0] == 0x7fffffff ? 0 : best_index[0];
        ids[(long long)b * ids_stride + write_position] = (float)token;
        if(token == end_id) finished[b] = 1;
    }
}

// Softmax and greedy step in one kernel for a row of logits: the probabilities are formed exactly as
// softmax_rows_kernel forms them (same statistics, same expression) but only compared, never stored; first index on ties.
__global__ void __launch_bounds__(kLossThreads)
softmax_greedy_kernel(const float* __restrict__ logits, int V, float* __restrict__ ids, long long ids_stride, int write_position,
                      int* __restrict__ finished, int end_id)
{
    __shared__ float scratch_f[16];
    __shared__ int scratch_i[8];
    __shared__ float best_value[kLossThreads];
    __shared__ int best_index[kLossThreads];
    const int b = blockIdx.x;
    const float* row = logits + (long long)b * V;
    const RowStats st = row_statistics(row, V, scratch_f, scratch_i);
    const float inv = st.sum > 0.f ? 1.0f / st.sum : 0.f;
    float value = -INFINITY;
    int index = 0x7fffffff;
    if((V & 3) == 0 && aligned16(row))
        for(int i = threadIdx.x * 4; i < V; i += kLossThreads * 4)
        {
            const float4 x = ld4(row + i);
            const float p0 = __expf(x.x - st.max) * inv, p1 = __expf(x.y - st.max) * inv;
            const float p2 = __expf(x.z - st.max) * inv, p3 = __expf(x.w - st.max) * inv;
            if(p0 > value) { value = p0; index = i; }
            if(p1 > value) { value = p1; index = i + 1; }
            if(p2 > value) { value = p2; index = i + 2; }
            if(p3 > value) { value = p3; index = i + 3; }
        }
    else
        for(int i = threadIdx.x; i < V; i += kLossThreads)
        {
            const float p = __expf(row[i] - st.max) * inv;
            if(p > value) { value = p; index = i; }
        }
    best_value[threadIdx.x] = value;
    best_index[threadIdx.x] = index;
    __syncthreads();
    for(int step = kLossThreads / 2; step > 0; step >>= 1)
    {
        if(threadIdx.x < step)
        {
            const float other = best_value[threadIdx.x + step];
            const int other_index = best_index[threadIdx.x + step];
            if(other > best_value[threadIdx.x] || (other == best_value[threadIdx.x] && other_index < best_index[threadIdx.x]))
            {
                best_value[threadIdx.x] = other;
                best_index[threadIdx.x] = other_index;
            }
        }
        __syncthreads();
    }
    if(threadIdx.x == 0 && !finished[b])
    {
        const int token = best_index[0] == 0x7fffffff ? 0 : best_index[0];
        ids[(long long)b * ids_stride + write_position] = (float)token;
        if(token == end_id) finished[b] = 1;
    }
}

extern "C" int onn_greedy_next_token_logits(const float* logits, float* ids, int* finished, int64_t B, int64_t S, int64_t V,
                                            int64_t write_position, int end_id, void* stream)
{
    ONN_CHECK_ARG(logits && ids && finished && B > 0 && S > 1 && V > 0 && write_position > 0 && write_position < S && V < (1LL << 31));
    softmax_greedy_kernel<<<(unsigned)B, kLossThreads, 0, (cudaStream_t)stream>>>(logits, (int)V, ids, S, (int)write_position, finished, end_id);
    count_launch();
    return launch_status();
}

// 256 threads for a short distribution, 1024 for a vocabulary
static unsigned greedy_threads(int64_t V) { return V >= 4096 ? 1024u : 256u; }

extern "C" int onn_greedy_next_token(const float* probabilities, float* ids, int* finished, int64_t B, int64_t S, int64_t V,
                                     int64_t position, int end_id, void* stream)
{
    ONN_CHECK_ARG(probabilities && ids && finished && B > 0 && S > 1 && V > 0 && position >= 0 && position + 1 < S && V < (1LL << 31));
    greedy_next_token_kernel<<<(unsigned)B, greedy_threads(V), 0, (cudaStream_t)stream>>>(probabilities + position * V, S * V, ids, S, (int)position + 1,
                                                                             finished, (int)V, end_id);
    count_launch();
    return launch_status();
}

extern "C" int onn_greedy_next_token_rows(const float* probabilities, float* ids, int* finished, int64_t B, int64_t S, int64_t V,
                                          int64_t write_position, int end_id, void* stream)
{
    ONN_CHECK_ARG(probabilities && ids && finished && B > 0 && S > 1 && V > 0 && write_position > 0 && write_position < S && V < (1LL << 31));
    greedy_next_token_kernel<<<(unsigned)B, greedy_threads(V), 0, (cudaStream_t)stream>>>(probabilities, V, ids, S, (int)write_position, finished, (int)V, end_id);
    count_launch();
    return launch_status();
}

// One query row per (sample, head) against the keys and values cached so far: scores, softmax and weighted sum in one
// warp.  Lanes own keys for the scores (each a full dot product over the head) and head features for the output.
__global__ void __launch_bounds__(128)
decode_attention_kernel(const float* __restrict__ q, const float* __restrict__ k_cache, const float* __restrict__ v_cache,
                        const uint8_t* __restrict__ key_is_pad, long long pad_stride_sample, long long pad_stride_key,
                        float* __restrict__ out, int B, int H, int S_cache, int length, int E, float scale)
{
    extern __shared__ float shared[];                          // per warp: hd query values, then `length` scores
    const int lane = threadIdx.x & 31, warp_in_block = threadIdx.x >> 5;
    const int hd = E / H;
    const long long item = (long long)blockIdx.x * 4 + warp_in_block;
    if(item >= (long long)B * H) return;
    const int b = (int)(item / H), h = (int)(item % H);
    float* q_shared = shared + (size_t)warp_in_block * (hd + S_cache);
    float* scores = q_shared + hd;
    const float* q_row = q + (long long)b * E + h * hd;
    for(int d = lane; d < hd; d += 32) q_shared[d] = q_row[d];
    __syncwarp();

    float row_max = -INFINITY;
    for(int j = lane; j < length; j += 32)
    {
        const float* k_row = k_cache + ((long long)b * S_cache + j) * E + h * hd;
        float dot = 0.f;
        for(int d = 0; d < hd; d++) dot = fmaf(q_shared[d], k_row[d], dot);
        float s = dot * scale;
        if(key_is_pad && key_is_pad[b * pad_stride_sample + j * pad_stride_key]) s = -1e9f;     // overwrite, as the training path
        scores[j] = s;
        row_max = fmaxf(row_max, s);
    }
    row_max = warp_max(row_max);
    float total = 0.f;
    for(int j = lane; j < length; j += 32)
    {
        const float e = __expf(scores[j] - row_max);
        scores[j] = e;
        total += e;
    }
    total = warp_sum(total);
    const float inv = total > 0.f ? 1.0f / total : 0.f;
    __syncwarp();
    for(int d = lane; d < hd; d += 32)
    {
        float acc = 0.f;
        for(int j = 0; j < length; j++) acc = fmaf(scores[j], v_cache[((long long)b * S_cache + j) * E + h * hd + d], acc);
        out[(long long)b * E + h * hd + d] = acc * inv;
    }
}

// The same for head sizes that are a multiple of 4 (every configuration of the transformer): one CTA of 256 threads per
// (sample, head).  Scores: 8 lanes share a key and read its row as float4 (32 keys per pass, rows read once, coalesced);
// softmax over the scores in shared memory; output: hd/4 threads share a value row, 256/(hd/4) groups of them walk the
// keys side by side, and their partial sums are added in a fixed order.
__global__ void __launch_bounds__(256)
decode_attention_block_kernel(const float* __restrict__ q, const float* __restrict__ k_cache, const float* __restrict__ v_cache,
                              const uint8_t* __restrict__ key_is_pad, long long pad_stride_sample, long long pad_stride_key,
                              float* __restrict__ out, int H, int S_cache, int length, int E, float scale)
{
    extern __shared__ __align__(16) float shared[];            // q[hd] | partial[1024] | reduce[16] | scores[S_cache]
    const int hd = E / H, chunks = hd >> 2;
    float* q_shared = shared;
    float* partial = q_shared + hd;
    float* reduce = partial + 1024;
    float* scores = reduce + 16;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x / H, h = blockIdx.x % H;
    const long long cache_row0 = (long long)b * S_cache;
    for(int d = tid; d < hd; d += 256) q_shared[d] = q[(long long)b * E + h * hd + d];
    __syncthreads();

    // scores
    const int sub = tid & 7, slot = tid >> 3;
    float thread_max = -INFINITY;
    for(int j0 = 0; j0 < length; j0 += 32)
    {
        const int j = j0 + slot;
        float dot = 0.f;
        if(j < length)
        {
            const float4* k_row = reinterpret_cast<const float4*>(k_cache + (cache_row0 + j) * E + h * hd);
            for(int c = sub; c < chunks; c += 8)
            {
                const float4 kv = k_row[c];
                const float4 qv = *reinterpret_cast<const float4*>(q_shared + 4 * c);
                dot = fmaf(qv.x, kv.x, dot); dot = fmaf(qv.y, kv.y, dot); dot = fmaf(qv.z, kv.z, dot); dot = fmaf(qv.w, kv.w, dot);
            }
        }
        dot += __shfl_xor_sync(0xffffffffu, dot, 4);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        if(j < length)
        {
            float s = dot * scale;
            if(key_is_pad && key_is_pad[b * pad_stride_sample + j * pad_stride_key]) s = -1e9f;        // overwrite, as the training path
            if(sub == 0) scores[j] = s;
            thread_max = fmaxf(thread_max, s);
        }
    }
    thread_max = warp_max(thread_max);
    if(lane == 0) reduce[warp] = thread_max;
    __syncthreads();
    float row_max = reduce[0];
#pragma unroll
    for(int w = 1; w < 8; w++) row_max = fmaxf(row_max, reduce[w]);

    float thread_sum = 0.f;
    for(int j = tid; j < length; j += 256)
    {
        const float e = __expf(scores[j] - row_max);
        scores[j] = e;
        thread_sum += e;
    }
    thread_sum = warp_sum(thread_sum);
    if(lane == 0) reduce[8 + warp] = thread_sum;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for(int w = 0; w < 8; w++) total += reduce[8 + w];
    const float inv = total > 0.f ? 1.0f / total : 0.f;

    // weighted sum of the value rows
    const int groups = 256 / chunks;
    if(tid < groups * chunks)
    {
        const int group = tid / chunks, c = tid % chunks;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for(int j = group; j < length; j += groups)
        {
            const float p = scores[j];
            const float4 v = reinterpret_cast<const float4*>(v_cache + (cache_row0 + j) * E + h * hd)[c];
            acc.x = fmaf(p, v.x, acc.x); acc.y = fmaf(p, v.y, acc.y); acc.z = fmaf(p, v.z, acc.z); acc.w = fmaf(p, v.w, acc.w);
        }
        *reinterpret_cast<float4*>(partial + group * hd + 4 * c) = acc;
    }
    __syncthreads();
    for(int d = tid; d < hd; d += 256)
    {
        float sum = 0.f;
        for(int g = 0; g < groups; g++) sum += partial[g * hd + d];
        out[(long long)b * E + h * hd + d] = sum * inv;
    }
}

extern "C" int onn_decode_attention(const float* q, const float* k_cache, const float* v_cache, const uint8_t* key_is_pad,
                                    int64_t pad_stride_sample, int64_t pad_stride_key, float* out,
                                    int64_t B, int64_t S_cache, int64_t length, int64_t E, int64_t H, void* stream)
{
    ONN_CHECK_ARG(q && k_cache && v_cache && out && B > 0 && H > 0 && E > 0 && E % H == 0 && length > 0 && length <= S_cache);
    const int hd = (int)(E / H);
    const bool aligned = ((uintptr_t)q & 15) == 0 && ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0;
    if(hd % 4 == 0 && hd <= 256 && aligned && B * H < (1LL << 31))
    {
        const size_t shared = (size_t)(hd + 1024 + 16 + S_cache) * sizeof(float);
        if(shared > 200 * 1024) return ONN_ERR_UNSUPPORTED;
        static PerDeviceBytes configured;
        if(!ensure_dynamic_smem(decode_attention_block_kernel, configured, shared)) return ONN_ERR_CUDA;
        decode_attention_block_kernel<<<(unsigned)(B * H), 256, shared, (cudaStream_t)stream>>>(q, k_cache, v_cache, key_is_pad, pad_stride_sample,
                                                                                                 pad_stride_key, out, (int)H,
                                                                                                 (int)S_cache, (int)length, (int)E,
                                                                                                 1.0f / sqrtf((float)hd));
        count_launch();
        return launch_status();
    }
    const size_t shared = 4 * (size_t)(hd + S_cache) * sizeof(float);
    if(shared > 200 * 1024) return ONN_ERR_UNSUPPORTED;
    static PerDeviceBytes configured;
    if(!ensure_dynamic_smem(decode_attention_kernel, configured, shared)) return ONN_ERR_CUDA;
    const long long items = B * H;
    decode_attention_kernel<<<(unsigned)((items + 3) / 4), 128, shared, (cudaStream_t)stream>>>(q, k_cache, v_cache, key_is_pad, pad_stride_sample, pad_stride_key,
                                                                                             out, (int)B, (int)H,
                                                                                             (int)S_cache, (int)length, (int)E,
                                                                                             1.0f / sqrtf((float)hd));
    count_launch();
    return launch_status();
}

extern "C" int onn_rows_are_zero(const float* X, uint8_t* flags, int64_t rows, int64_t E, void* stream)
{
    ONN_CHECK_ARG(X && flags && rows > 0 && E > 0 && E < (1LL << 31));
    return launch_source_row_is_zero(X, flags, rows, (int)E, (cudaStream_t)stream);
}

// CrossEntropyError2d for several classes: one warp per sample; the gradient overwrites the probabilities.
__global__ void __launch_bounds__(256)
ce2d_fwd_bwd_kernel(float* __restrict__ probabilities, const float* __restrict__ targets, float* __restrict__ row_terms, long long rows, int classes)
{
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const long long stride = (long long)gridDim.x * 8;
    const float inv_rows = 1.0f / (float)rows;
    for(long long row = warp; row < rows; row += stride)
    {
        float* p = probabilities + row * classes;
        const float* t = targets + row * classes;
        float term = 0.f;
        for(int c = lane; c < classes; c += 32)
        {
            const float y = p[c], target = t[c];
            term += target * logf(y + 1.1920929e-07f);
            p[c] = (y - target) * inv_rows;
        }
        term = warp_sum(term);
        if(lane == 0) row_terms[row] = term;
    }
}

__global__ void ce2d_finish_kernel(const float* __restrict__ row_terms, long long rows, float* __restrict__ stats)
{
    __shared__ float scratch[32];
    float mine = 0.f;
    for(long long i = threadIdx.x; i < rows; i += blockDim.x) mine += row_terms[i];
    const float total = block_sum(mine, scratch);
    if(threadIdx.x == 0) { stats[0] = total / (float)(-rows); stats[1] = (float)rows; }
}

// CrossEntropyError2d with one output: per sample the error term and, in place, the output gradient.
__global__ void ce2d_binary_kernel(float* __restrict__ outputs, const float* __restrict__ targets, float* __restrict__ row_terms, long long rows,
                                   int fold_sigmoid)
{
    const float eps = 1.1920929e-07f, inv_rows = 1.0f / (float)rows;
    for(long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rows; i += (long long)gridDim.x * blockDim.x)
    {
        const float y = outputs[i], t = targets[i];
        const float clipped = fminf(fmaxf(y, eps), 1.0f - eps);
        row_terms[i] = t * logf(clipped) + (1.0f - t) * logf(1.0f - clipped);
        const float gradient = (-t / (y + eps) + (1.0f - t) / (1.0f - y + eps)) * inv_rows;
        outputs[i] = fold_sigmoid ? gradient * (y * (1.0f - y)) : gradient;
    }
}

__global__ void ce2d_binary_finish_kernel(const float* __restrict__ row_terms, long long rows, float* __restrict__ stats)
{
    __shared__ float scratch[32];
    float mine = 0.f;
    for(long long i = threadIdx.x; i < rows; i += blockDim.x) mine += row_terms[i];
    const float total = block_sum(mine, scratch);
    if(threadIdx.x == 0)
    {
        float error = total / (float)(-rows);
        if(isnan(error) || isinf(error)) error = 10.0f;          // opennn/cross_entropy_error.cpp:53-54
        stats[0] = error;
        stats[1] = (float)rows;
    }
}

extern "C" int onn_ce2d_binary_fwd_bwd(float* outputs, const float* targets, float* stats, float* row_scratch, int64_t rows,
                                       int fold_sigmoid, void* stream)
{
    ONN_CHECK_ARG(outputs && targets && stats && row_scratch && rows > 0);
    cudaStream_t s = (cudaStream_t)stream;
    ce2d_binary_kernel<<<grid_for(rows, 256, 8), 256, 0, s>>>(outputs, targets, row_scratch, rows, fold_sigmoid);
    count_launch();
    if(launch_status() != ONN_OK) return ONN_ERR_CUDA;
    ce2d_binary_finish_kernel<<<1, 1024, 0, s>>>(row_scratch, rows, stats);
    count_launch();
    return launch_status();
}

extern "C" int onn_ce2d_fwd_bwd(float* probabilities, const float* targets, float* stats, float* row_scratch,
                                int64_t rows, int64_t classes, void* stream)
{
    ONN_CHECK_ARG(probabilities && targets && stats && row_scratch && rows > 0 && classes > 1 && classes < (1LL << 31));
    cudaStream_t s = (cudaStream_t)stream;
    ce2d_fwd_bwd_kernel<<<grid_for(rows, 8, 8), 256, 0, s>>>(probabilities, targets, row_scratch, rows, (int)classes);
    count_launch();
    if(launch_status() != ONN_OK) return ONN_ERR_CUDA;
    ce2d_finish_kernel<<<1, 1024, 0, s>>>(row_scratch, rows, stats);
    count_launch();
    return launch_status();
}

extern "C" int onn_ce3d_count_active(const float* targets, int64_t rows, int64_t V, float* counts, void* stream)
{
    ONN_CHECK_ARG(targets && counts && rows > 0 && V > 0);
    count_active_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(targets, rows, V, counts);
    count_launch();
    return launch_status();
}

extern "C" int onn_ce3d_fwd_bwd(float* logits, const float* targets, const float* active_count,
                                float* probabilities_out, float* stats, float* row_scratch,
                                int64_t rows, int64_t V, int inputs_are_probabilities, uint32_t flags, void* stream)
{
    ONN_CHECK_ARG(logits && targets && active_count && stats && row_scratch);
    ONN_CHECK_ARG(rows > 0 && V > 1 && rows < (1LL << 31) && V < (1LL << 31));
    cudaStream_t s = (cudaStream_t)stream;
    if(!(flags & ONN_CE_TWO_SWEEPS) && ce3d_staged_takes(logits, probabilities_out, rows, V))
    {
        // long rows: staged in shared memory, each logit crosses HBM once in and once out
        if(ce3d_staged_launch(logits, targets, active_count, row_scratch, rows, (int)V, inputs_are_probabilities, s) != ONN_OK) return ONN_ERR_CUDA;
    }
    else
    {
        ce3d_fwd_bwd_kernel<<<(unsigned)rows, kLossThreads, 0, s>>>(logits, targets, active_count, probabilities_out, row_scratch,
                                                                     rows, (int)V, inputs_are_probabilities);
        count_launch();
        if(launch_status() != ONN_OK) return ONN_ERR_CUDA;
    }
    ce3d_finish_kernel<<<1, 1024, 0, s>>>(row_scratch, targets, rows, V, stats);
    count_launch();
    return launch_status();
}

extern "C" size_t onn_grad_sqnorm_workspace_floats(int64_t n)
{
    return n > 0 ? (size_t)kNormBlocks : 0;
}

extern "C" int onn_grad_sqnorm(const float* g, int64_t n, float* sqnorm, float* workspace, void* stream)
{
    ONN_CHECK_ARG(g && sqnorm && n > 0);
    if(!workspace) return ONN_ERR_WORKSPACE;
    cudaStream_t s = (cudaStream_t)stream;
    const int grid = grid_for((n + 3) / 4, 256, 4);
    sqnorm_partial_kernel<<<grid, 256, 0, s>>>(g, n, workspace);
    count_launch();
    if(launch_status() != ONN_OK) return ONN_ERR_CUDA;
    sqnorm_finish_kernel<<<1, 256, 0, s>>>(workspace, grid, sqnorm);
    count_launch();
    return launch_status();
}

extern "C" int onn_adam_guarded(float* p, float* m, float* v, float* g, int64_t n,
                                float lr, float beta1, float beta2, float eps, float bc1, float bc2,
                                float clip_norm, const float* sqnorm, float grad_scale, int zero_grad,
                                const uint32_t* skip_if_nonzero, void* stream)
{
    ONN_CHECK_ARG(p && m && v && g && n > 0 && bc1 != 0.f && bc2 != 0.f);
    const int grid = grid_for((n + 3) / 4, 256, 8);
    adam_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p, m, v, g, n, lr, beta1, beta2, eps,
                                                        bc1, bc2, clip_norm, sqnorm, grad_scale, zero_grad, skip_if_nonzero);
    count_launch();
    return launch_status();
}

extern "C" int onn_adam(float* p, float* m, float* v, float* g, int64_t n,
                        float lr, float beta1, float beta2, float eps, float bc1, float bc2,
                        float clip_norm, const float* sqnorm, float grad_scale, int zero_grad, void* stream)
{
    return onn_adam_guarded(p, m, v, g, n, lr, beta1, beta2, eps, bc1, bc2, clip_norm, sqnorm, grad_scale, zero_grad, nullptr, stream);
}
