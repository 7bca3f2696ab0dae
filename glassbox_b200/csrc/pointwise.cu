// Small row-wise and element-wise kernels for layers that norm a branch before it joins the residual stream, for
// activations other than SwiGLU, and for a scaled head:
//   rmsnorm_add   x[r, :] += gain * y[r, :] / sqrt(mean(y[r, :]^2) + eps)   (float32 throughout)
//   relu2         out = max(in, 0)^2
//   scale         t *= s
//   gated_head_norm  out[r, h, :] = w * o[r, h, :] / sqrt(mean_v(o[r, h, :]^2) + eps) * sigmoid(gate[r, h, :])
#include "common.cuh"

// ----------------------------------------------------------------------------------------------
// A branch's output y (float32) is normalised and added into the residual x (float32). One block per row.
// ----------------------------------------------------------------------------------------------
template <int THREADS>
__global__ void __launch_bounds__(THREADS) rmsnorm_add_kernel(const float* __restrict__ y, long long ldy,
                                                              const float* __restrict__ gain, float* __restrict__ x,
                                                              long long ldx, int n, int d, float eps) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int r = blockIdx.x;
    if (r >= n) return;
    const float* src = y + (size_t)r * ldy;
    float* dst = x + (size_t)r * ldx;
    __shared__ float partial[THREADS / 32];
    __shared__ float total;
    constexpr int VMAX = 4;
    const bool quick = d % 4 == 0 && d <= THREADS * 4 * VMAX && ((uintptr_t)src & 15) == 0 && ((uintptr_t)dst & 15) == 0 &&
                       ((uintptr_t)gain & 15) == 0;
    float4 v[VMAX], o[VMAX];
    float ss = 0.f;
    if (quick) {
#pragma unroll
        for (int i = 0; i < VMAX; ++i) {
            const int j = (i * THREADS + threadIdx.x) * 4;
            v[i] = j < d ? *reinterpret_cast<const float4*>(src + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            o[i] = j < d ? *reinterpret_cast<const float4*>(dst + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < VMAX; ++i) {
            ss = fmaf(v[i].x, v[i].x, ss); ss = fmaf(v[i].y, v[i].y, ss);
            ss = fmaf(v[i].z, v[i].z, ss); ss = fmaf(v[i].w, v[i].w, ss);
        }
    } else {
        for (int j = threadIdx.x; j < d; j += THREADS) {
            const float t = src[j];
            ss = fmaf(t, t, ss);
        }
    }
    ss = gb_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < THREADS / 32; ++w) t += partial[w];
        total = 1.0f / sqrtf(t / (float)d + eps);
    }
    __syncthreads();
    const float s = total;
    if (quick) {
#pragma unroll
        for (int i = 0; i < VMAX; ++i) {
            const int j = (i * THREADS + threadIdx.x) * 4;
            if (j < d) {
                const float4 g = *reinterpret_cast<const float4*>(gain + j);
                float4 w;
                w.x = o[i].x + g.x * (v[i].x * s);
                w.y = o[i].y + g.y * (v[i].y * s);
                w.z = o[i].z + g.z * (v[i].z * s);
                w.w = o[i].w + g.w * (v[i].w * s);
                *reinterpret_cast<float4*>(dst + j) = w;
            }
        }
    } else {
        for (int j = threadIdx.x; j < d; j += THREADS) dst[j] += gain[j] * (src[j] * s);
    }
}

GB_EXPORT int gb_rmsnorm_add(const float* y, long long ldy, const float* gain, float* x, long long ldx, int n, int d,
                             float eps, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && d > 0, "gb_rmsnorm_add: bad sizes n=%d d=%d", n, d);
    if (n == 0) return 0;
    gb_launch(GB_PDL_ELEMENTWISE, rmsnorm_add_kernel<128>, dim3(n), dim3(128), 0, stream, y, ldy, gain, x, ldx, n, d, eps);
    return gb_check_launch("gb_rmsnorm_add");
}

// ----------------------------------------------------------------------------------------------
// Squared ReLU.
// ----------------------------------------------------------------------------------------------
template <typename T>
__global__ void relu2_kernel(const T* __restrict__ in, T* __restrict__ out, long long total) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const float v = fmaxf(gb_to_float(in[idx]), 0.f);
        out[idx] = gb_from_float<T>(v * v);
    }
}

GB_EXPORT int gb_relu2(const void* in, void* out, int dtype, long long total, cudaStream_t stream) {
    GB_REQUIRE(total >= 0, "gb_relu2: bad size");
    if (total == 0) return 0;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == GB_F32)
        gb_launch(GB_PDL_ELEMENTWISE, relu2_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)in, (float*)out, total);
    else if (dtype == GB_BF16)
        gb_launch(GB_PDL_ELEMENTWISE, relu2_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)in,
                  (__nv_bfloat16*)out, total);
    else
        GB_REQUIRE(false, "gb_relu2: unsupported dtype %d", dtype);
    return gb_check_launch("gb_relu2");
}

// ----------------------------------------------------------------------------------------------
// t *= s (float32): a head whose logits carry a constant factor.
// ----------------------------------------------------------------------------------------------
__global__ void scale_kernel(float* __restrict__ t, long long total, float s) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; idx < total; idx += (long long)gridDim.x * blockDim.x) t[idx] *= s;
}

GB_EXPORT int gb_scale(float* t, long long total, float s, cudaStream_t stream) {
    GB_REQUIRE(total >= 0, "gb_scale: bad size");
    if (total == 0) return 0;
    int blocks = (int)((total + 255) / 256);
    if (blocks > 148 * 16) blocks = 148 * 16;
    gb_launch(GB_PDL_ELEMENTWISE, scale_kernel, dim3(blocks), dim3(256), 0, stream, t, total, s);
    return gb_check_launch("gb_scale");
}

// ----------------------------------------------------------------------------------------------
// Per-head RMS norm of a mixer's read-out with an output gate: one warp per (row, head).
// o float32 [n, heads * v]; gate float32 (row stride ldg), logits of the gate; w float32 [v] shared by heads.
// ----------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) gated_head_norm_kernel(const float* __restrict__ o, const float* __restrict__ gate,
                                                              long long ldg, const float* __restrict__ w, T* __restrict__ out,
                                                              int n, int heads, int v, float eps) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long task = (long long)blockIdx.x * 4 + warp;
    if (task >= (long long)n * heads) return;
    const int row = (int)(task / heads), head = (int)(task % heads);
    const float* src = o + ((size_t)row * heads + head) * v;
    const float* g = gate + (size_t)row * ldg + (size_t)head * v;
    T* dst = out + ((size_t)row * heads + head) * v;
    float ss = 0.f;
    for (int j = lane; j < v; j += 32) ss = fmaf(src[j], src[j], ss);
    ss = gb_warp_sum(ss);
    const float s = 1.0f / sqrtf(ss / (float)v + eps);
    for (int j = lane; j < v; j += 32) {
        const float sig = 1.0f / (1.0f + expf(-g[j]));
        dst[j] = gb_from_float<T>(src[j] * s * w[j] * sig);
    }
}

GB_EXPORT int gb_gated_head_norm(const float* o, const float* gate, long long ldg, const float* w, void* out, int out_dtype,
                                 int n, int heads, int v, float eps, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && heads > 0 && v > 0, "gb_gated_head_norm: bad sizes");
    if (n == 0) return 0;
    const int blocks = gb_ceil_div((long long)n * heads, 4);
    if (out_dtype == GB_F32)
        gb_launch(GB_PDL_ELEMENTWISE, gated_head_norm_kernel<float>, dim3(blocks), dim3(128), 0, stream, o, gate, ldg, w, (float*)out, n,
                  heads, v, eps);
    else if (out_dtype == GB_BF16)
        gb_launch(GB_PDL_ELEMENTWISE, gated_head_norm_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, stream, o, gate, ldg, w,
                  (__nv_bfloat16*)out, n, heads, v, eps);
    else
        GB_REQUIRE(false, "gb_gated_head_norm: unsupported output dtype %d", out_dtype);
    return gb_check_launch("gb_gated_head_norm");
}
