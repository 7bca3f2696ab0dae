// Layer norm with weight and bias, and a residual that is kept as several streams (hyper-connections), in one row kernel.
//
// A model with S residual streams keeps, per token, S rows x_1 .. x_S of d float32 numbers (xs [n, S, d]). A sublayer reads
// one mix of them, u = sum_s read[s] * x_s, through a layer norm, and its output y comes back into all of them at once:
// x_t <- sum_s mix[s, t] * x_s + write[t] * y. One block per row does, as far as it is asked to:
//   1. fold in the output y of the sublayer before (new streams from the old ones; stored unless rows are gathered); y is
//      a stored row, or a weighted sum of rows that the kernel forms on the way (a mixture of experts' results),
//   2. form u (read == nullptr: the plain sum of the streams; with S == 1 that is the row itself),
//   3. store u as float32 and / or its layer norm (u - mean) / sqrt(var + eps) * w + b in the activation dtype,
// so a chain of sublayers costs one launch per sublayer for everything between the products, and the same kernel is the
// plain layer norm of a model with one residual row (S = 1, nothing to fold in). var is the mean of the squared
// deviations from the mean (two passes over the row, which lives in shared memory meanwhile). Everything is float32.
#include "common.cuh"

constexpr int RS_THREADS = 256;
constexpr int RS_MAX_STREAMS = 8;

__device__ __forceinline__ float rs_block_sum(float v, float* partial) {
    v = gb_warp_sum(v);
    __syncthreads();                                  // (partial may still be read from the round before)
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < RS_THREADS / 32; ++w) t += partial[w];
    return t;
}

// One column: v[s] are the streams' values (replaced by the new ones when an output is folded in); returns u.
template <int S>
__device__ __forceinline__ float rs_column(float (&v)[S], float yj, const float* cm, const float* cw, const float* cr, bool fold) {
    if (fold) {
        float nv[S];
#pragma unroll
        for (int t = 0; t < S; ++t) {
            float a = 0.f;
            {
#pragma unroll
                for (int s = 0; s < S; ++s)
                    a = fmaf(cm[s * S + t], v[s], a);
                a = fmaf(cw[t], yj, a);
            }
            nv[t] = a;
        }
#pragma unroll
        for (int s = 0; s < S; ++s) v[s] = nv[s];
    }
    float u = 0.f;
#pragma unroll
    for (int s = 0; s < S; ++s)
        u = fmaf(cr[s], v[s], u);
    return u;
}

// A branch output that is not stored anywhere yet: y[row, :] = sum_k weight[row, k] * pair[row, k, :] + gate[row] * shared[row, :]
// (a mixture of experts' results per (row, choice) and its shared expert); the kernel forms it on the way. pair == nullptr: none.
struct RsWeighted {
    const float* pair;      // [n, top, d]
    const float* weight;    // [n, top]
    const float* shared;    // [n, lds] or nullptr
    const float* gate;      // [n] or nullptr (the shared row is added as it is)
    long long lds;
    int top;
};

__device__ __forceinline__ float4 rs_weighted4(const RsWeighted& w, int row, int d, int j) {
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < w.top; ++k) {
        const float c = w.weight[(size_t)row * w.top + k];
        const float4 v = *reinterpret_cast<const float4*>(w.pair + ((size_t)row * w.top + k) * d + j);
        a.x = fmaf(c, v.x, a.x); a.y = fmaf(c, v.y, a.y); a.z = fmaf(c, v.z, a.z); a.w = fmaf(c, v.w, a.w);
    }
    if (w.shared) {
        const float g = w.gate ? w.gate[row] : 1.f;
        const float4 v = *reinterpret_cast<const float4*>(w.shared + (size_t)row * w.lds + j);
        a.x = fmaf(g, v.x, a.x); a.y = fmaf(g, v.y, a.y); a.z = fmaf(g, v.z, a.z); a.w = fmaf(g, v.w, a.w);
    }
    return a;
}

__device__ __forceinline__ float rs_weighted1(const RsWeighted& w, int row, int d, int j) {
    float a = 0.f;
    for (int k = 0; k < w.top; ++k) a = fmaf(w.weight[(size_t)row * w.top + k], w.pair[((size_t)row * w.top + k) * d + j], a);
    if (w.shared) a = fmaf(w.gate ? w.gate[row] : 1.f, w.shared[(size_t)row * w.lds + j], a);
    return a;
}

template <typename T, int S>
__global__ void __launch_bounds__(RS_THREADS) streams_step_kernel(
    float* __restrict__ xs, int d, const float* __restrict__ y, long long ldy, RsWeighted ws, const float* __restrict__ mix,
    const float* __restrict__ write, const float* __restrict__ read, const float* __restrict__ w, const float* __restrict__ b,
    float eps, T* __restrict__ h, float* __restrict__ u_out, const int* __restrict__ rows, const int* __restrict__ positions,
    int n_out, int n_src) {
    extern __shared__ __align__(16) float rs_u[];     // the row u, d numbers
    __shared__ float partial[RS_THREADS / 32];
    __shared__ float coef[RS_MAX_STREAMS * RS_MAX_STREAMS + 2 * RS_MAX_STREAMS];
    // (weights of the model: nothing of the step writes them, so they may be read before the wait)
    if (threadIdx.x < S * S) coef[threadIdx.x] = mix ? mix[threadIdx.x] : 0.f;
    if (threadIdx.x < S) {
        coef[RS_MAX_STREAMS * RS_MAX_STREAMS + threadIdx.x] = write ? write[threadIdx.x] : 0.f;
        coef[RS_MAX_STREAMS * RS_MAX_STREAMS + RS_MAX_STREAMS + threadIdx.x] = read ? read[threadIdx.x] : 1.f;
    }
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int r = blockIdx.x;
    if (r >= n_out) return;
    const int src = rows ? rows[r] : r;
    if (src < 0 || src >= n_src) return;
    if (!rows && positions && positions[src] < 0) return;      // a padding row of a fixed-shape batch
    __syncthreads();
    const float* cm = coef;
    const float* cw = coef + RS_MAX_STREAMS * RS_MAX_STREAMS;
    const float* cr = cw + RS_MAX_STREAMS;
    float* row = xs + (size_t)src * S * d;
    const bool lazy = ws.pair != nullptr;
    const bool fold = y != nullptr || lazy, keep = fold && rows == nullptr;
    float total = 0.f;
    if ((d & 3) == 0 && (ldy & 3) == 0 && ((uintptr_t)xs & 15) == 0 && (y == nullptr || ((uintptr_t)y & 15) == 0) &&
        (u_out == nullptr || ((uintptr_t)u_out & 15) == 0) &&
        (!lazy || (((uintptr_t)ws.pair & 15) == 0 && (ws.shared == nullptr || (((uintptr_t)ws.shared & 15) == 0 && (ws.lds & 3) == 0))))) {
        // four columns per thread and round: every load of a round (S streams and y) is asked for before the first is used
        for (int j = threadIdx.x * 4; j < d; j += RS_THREADS * 4) {
            float4 q[S];
#pragma unroll
            for (int s = 0; s < S; ++s)
                q[s] = *reinterpret_cast<const float4*>(row + (size_t)s * d + j);
            float4 yq = make_float4(0.f, 0.f, 0.f, 0.f);
            if (lazy) yq = rs_weighted4(ws, src, d, j);
            else if (fold) yq = *reinterpret_cast<const float4*>(y + (size_t)src * ldy + j);
            float v[4][S];
#pragma unroll
            for (int s = 0; s < S; ++s) {
                const float4 t = q[s];
                v[0][s] = t.x; v[1][s] = t.y; v[2][s] = t.z; v[3][s] = t.w;
            }
            const float yv[4] = {yq.x, yq.y, yq.z, yq.w};
            float u[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) u[c] = rs_column<S>(v[c], yv[c], cm, cw, cr, fold);
            if (keep) {
#pragma unroll
                for (int s = 0; s < S; ++s)
                    *reinterpret_cast<float4*>(row + (size_t)s * d + j) = make_float4(v[0][s], v[1][s], v[2][s], v[3][s]);
            }
            *reinterpret_cast<float4*>(rs_u + j) = make_float4(u[0], u[1], u[2], u[3]);
            total += (u[0] + u[1]) + (u[2] + u[3]);
            if (u_out) *reinterpret_cast<float4*>(u_out + (size_t)r * d + j) = make_float4(u[0], u[1], u[2], u[3]);
        }
    } else {
        for (int j = threadIdx.x; j < d; j += RS_THREADS) {
            float v[S];
#pragma unroll
            for (int s = 0; s < S; ++s) v[s] = row[(size_t)s * d + j];
            const float u = rs_column<S>(v, lazy ? rs_weighted1(ws, src, d, j) : (fold ? y[(size_t)src * ldy + j] : 0.f), cm, cw, cr, fold);
            if (keep) {
#pragma unroll
                for (int s = 0; s < S; ++s)
                    row[(size_t)s * d + j] = v[s];
            }
            rs_u[j] = u;
            total += u;
            if (u_out) u_out[(size_t)r * d + j] = u;
        }
    }
    __syncthreads();          // (the norm's second pass reads columns that other threads wrote, in the four-column form)
    if (h == nullptr) return;
    const float mean = rs_block_sum(total, partial) / (float)d;
    float dev = 0.f;
    for (int j = threadIdx.x; j < d; j += RS_THREADS) {
        const float c = rs_u[j] - mean;
        dev = fmaf(c, c, dev);
    }
    const float rstd = 1.0f / sqrtf(rs_block_sum(dev, partial) / (float)d + eps);
    T* dst = h + (size_t)r * d;
    for (int j = threadIdx.x; j < d; j += RS_THREADS)
        dst[j] = gb_from_float<T>((rs_u[j] - mean) * rstd * w[j] + (b ? b[j] : 0.f));
}

// xs[r, s, :] = x[r, :] for every stream s: the streams all start as the embedding's output.
__global__ void __launch_bounds__(256) streams_broadcast_kernel(const float* __restrict__ x, float* __restrict__ xs, long long n,
                                                                int S, int d) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const long long total = n * d;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const long long r = idx / d;
        const int j = (int)(idx % d);
        const float v = x[idx];
        for (int s = 0; s < S; ++s) xs[(r * S + s) * d + j] = v;
    }
}

GB_EXPORT int gb_streams_broadcast(const float* x, float* xs, int n, int S, int d, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && S >= 1 && d > 0, "gb_streams_broadcast: bad sizes");
    if (n == 0) return 0;
    long long total = (long long)n * d;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    gb_launch(GB_PDL_ELEMENTWISE, streams_broadcast_kernel, dim3(blocks), dim3(256), 0, stream, x, xs, (long long)n, S, d);
    return gb_check_launch("gb_streams_broadcast");
}

template <typename T, int S>
static void rs_launch(float* xs, int d, const float* y, long long ldy, RsWeighted ws, const float* mix, const float* write, const float* read,
                      const float* w, const float* b, float eps, T* h, float* u_out, const int* rows, const int* positions, int n_out,
                      int n_src, cudaStream_t stream) {
    const size_t smem = (size_t)d * 4;
    if (smem > 48 * 1024) cudaFuncSetAttribute(streams_step_kernel<T, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gb_launch(GB_PDL_ELEMENTWISE, streams_step_kernel<T, S>, dim3(n_out), dim3(RS_THREADS), smem, stream, xs, d, y, ldy, ws, mix, write, read,
              w, b, eps, h, u_out, rows, positions, n_out, n_src);
}

template <typename T>
static void rs_dispatch(int S, float* xs, int d, const float* y, long long ldy, RsWeighted ws, const float* mix, const float* write, const float* read,
                        const float* w, const float* b, float eps, T* h, float* u_out, const int* rows, const int* positions, int n_out,
                        int n_src, cudaStream_t stream) {
#define RS_CASE(N) case N: rs_launch<T, N>(xs, d, y, ldy, ws, mix, write, read, w, b, eps, h, u_out, rows, positions, n_out, n_src, stream); break;
    switch (S) { RS_CASE(1) RS_CASE(2) RS_CASE(3) RS_CASE(4) RS_CASE(5) RS_CASE(6) RS_CASE(7) RS_CASE(8) }
#undef RS_CASE
}

GB_EXPORT int gb_streams_step(float* xs, int S, int d, const float* y, long long ldy, const float* pair, const float* pair_weight,
                              int top, const float* shared, long long lds, const float* gate, const float* mix, const float* write,
                              const float* read, const float* w, const float* b, float eps, void* h, int h_dtype, float* u_out,
                              const int* rows, const int* positions, int n_out, int n_src, cudaStream_t stream) {
    GB_REQUIRE(S >= 1 && S <= RS_MAX_STREAMS, "gb_streams_step: %d streams, at most %d are supported", S, RS_MAX_STREAMS);
    GB_REQUIRE(n_out >= 0 && n_src >= 0 && d > 0 && (size_t)d * 4 <= 160 * 1024, "gb_streams_step: bad sizes (d=%d)", d);
    GB_REQUIRE((y == nullptr && pair == nullptr) || (mix != nullptr && write != nullptr), "gb_streams_step: folding in an output needs mix and write");
    GB_REQUIRE(pair == nullptr || (y == nullptr && pair_weight != nullptr && top > 0), "gb_streams_step: a weighted sum needs its weights, and excludes a stored output");
    const RsWeighted ws = {pair, pair_weight, shared, gate, lds, top};
    GB_REQUIRE(h == nullptr || w != nullptr, "gb_streams_step: a norm needs its weight");
    GB_REQUIRE(h == nullptr || h_dtype == GB_F32 || h_dtype == GB_BF16, "gb_streams_step: unsupported output dtype %d", h_dtype);
    if (n_out == 0) return 0;
    if (h == nullptr || h_dtype == GB_F32)
        rs_dispatch<float>(S, xs, d, y, ldy, ws, mix, write, read, w, b, eps, (float*)h, u_out, rows, positions, n_out, n_src, stream);
    else
        rs_dispatch<__nv_bfloat16>(S, xs, d, y, ldy, ws, mix, write, read, w, b, eps, (__nv_bfloat16*)h, u_out, rows, positions, n_out, n_src,
                                   stream);
    return gb_check_launch("gb_streams_step");
}
