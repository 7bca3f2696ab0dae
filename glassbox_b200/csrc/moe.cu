// A routed feed-forward (mixture of experts) with sigmoid scores, a choice bias and a limit to the best groups of experts.
//
//   moe_route        per row: logits = W_router h in float32 (h in the activation dtype), scores s = sigmoid(logits);
//                    experts are chosen by s + correction, the weights use s alone. The experts form `groups` equal runs of
//                    neighbours; a run's score is the sum of its two largest choice scores (its only one, if it has one
//                    member); only experts of the `keep` best runs can be chosen, the others count as minus infinity. The
//                    `top` largest are taken (among equals the lowest index), each with the weight s * route_scale, not
//                    renormalised. Also the gate of a shared expert, sigmoid(w_gate . h), one number per row.
//   moe_expert_rows  one block per (row, chosen expert): act = relu(W_up[e] h)^2 in shared memory, then W_down[e] act,
//                    written as float32 per (row, choice). Reads the two matrices of one expert once per block: the
//                    form for few rows (decoding), and the float32 path's form for any number.
//   moe_combine      out[row] (+)= sum_k weight[row, k] * pair[row, k] + gate[row] * shared[row]; a fixed order of sums.
#include "common.cuh"

#include <math.h>

constexpr int MOE_MAX_EXPERTS = 512;
constexpr int MOE_ROUTE_THREADS = 128;

__device__ __forceinline__ float moe_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }

// sum over K of w[k] * x[k]; x float32 in shared memory, w a row of a matrix in global memory; all lanes get the sum
template <typename T>
__device__ __forceinline__ float moe_warp_dot(const T* __restrict__ w, const float* __restrict__ x, int K, int lane);

template <>
__device__ __forceinline__ float moe_warp_dot<float>(const float* __restrict__ w, const float* __restrict__ x, int K, int lane) {
    float d = 0.f;
    if (K % 4 == 0 && ((uintptr_t)w & 15) == 0) {
        for (int i = lane * 4; i < K; i += 128) {
            const float4 v = *reinterpret_cast<const float4*>(w + i);
            d = fmaf(v.x, x[i], d); d = fmaf(v.y, x[i + 1], d); d = fmaf(v.z, x[i + 2], d); d = fmaf(v.w, x[i + 3], d);
        }
    } else {
        for (int i = lane; i < K; i += 32) d = fmaf(w[i], x[i], d);
    }
    return gb_warp_sum(d);
}

template <>
__device__ __forceinline__ float moe_warp_dot<__nv_bfloat16>(const __nv_bfloat16* __restrict__ w, const float* __restrict__ x, int K,
                                                             int lane) {
    float d = 0.f;
    if (K % 8 == 0 && ((uintptr_t)w & 15) == 0) {
        for (int i = lane * 8; i < K; i += 256) {
            const uint4 raw = *reinterpret_cast<const uint4*>(w + i);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const float2 f = __bfloat1622float2(p[t]);
                d = fmaf(f.x, x[i + 2 * t], d);
                d = fmaf(f.y, x[i + 2 * t + 1], d);
            }
        }
    } else {
        for (int i = lane; i < K; i += 32) d = fmaf(__bfloat162float(w[i]), x[i], d);
    }
    return gb_warp_sum(d);
}

// index of the largest of v[0 .. count) (lowest index among equals) over a warp; every lane gets it; -1 if all are -inf
__device__ __forceinline__ int moe_warp_argmax(const float* v, int count, int lane) {
    float best = -INFINITY;
    int at = -1;
    for (int i = lane; i < count; i += 32) {
        const float c = v[i];
        if (c > best) { best = c; at = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (oa >= 0 && (at < 0 || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
    }
    return at;
}

template <typename T>
__global__ void __launch_bounds__(MOE_ROUTE_THREADS) moe_route_kernel(
    const T* __restrict__ h, int d, const float* __restrict__ w_router, const float* __restrict__ correction,
    const float* __restrict__ w_gate, const int* __restrict__ positions, int n, int E, int top, int groups, int keep,
    float route_scale, int* __restrict__ choice_out, float* __restrict__ weight_out, float* __restrict__ gate_out) {
    extern __shared__ __align__(16) float moe_smem[];
    float* hx = moe_smem;                       // the row, float32
    __shared__ float score[MOE_MAX_EXPERTS], choice[MOE_MAX_EXPERTS], run_score[MOE_MAX_EXPERTS];
    __shared__ unsigned char kept[MOE_MAX_EXPERTS];
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int row = blockIdx.x;
    if (row >= n || positions[row] < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* src = h + (size_t)row * d;
    for (int i = threadIdx.x; i < d; i += MOE_ROUTE_THREADS) hx[i] = gb_to_float(src[i]);
    __syncthreads();
    for (int e = warp; e < E + (w_gate ? 1 : 0); e += MOE_ROUTE_THREADS / 32) {
        if (e < E) {
            const float z = moe_warp_dot<float>(w_router + (size_t)e * d, hx, d, lane);
            if (lane == 0) {
                const float s = moe_sigmoid(z);
                score[e] = s;
                choice[e] = s + (correction ? correction[e] : 0.f);
            }
        } else {
            const float z = moe_warp_dot<float>(w_gate, hx, d, lane);
            if (lane == 0) gate_out[row] = moe_sigmoid(z);
        }
    }
    __syncthreads();
    if (warp != 0) return;
    if (groups > 1 && keep < groups) {
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;          // the two largest of the run
            for (int i = 0; i < per; ++i) {
                const float c = choice[g * per + i];
                if (c > a) { b = a; a = c; } else if (c > b) { b = c; }
            }
            run_score[g] = per > 1 ? a + b : a;
            kept[g] = 0;
        }
        __syncwarp();
        for (int k = 0; k < keep; ++k) {
            const int g = moe_warp_argmax(run_score, groups, lane);
            __syncwarp();
            if (lane == 0 && g >= 0) { run_score[g] = -INFINITY; kept[g] = 1; }
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (!kept[e / per]) choice[e] = -INFINITY;
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        const int e = moe_warp_argmax(choice, E, lane);
        __syncwarp();
        if (lane == 0) {
            choice_out[(size_t)row * top + k] = e;                          // -1: fewer experts could be chosen than `top`
            weight_out[(size_t)row * top + k] = e >= 0 ? score[e] * route_scale : 0.f;
            if (e >= 0) choice[e] = -INFINITY;
        }
        __syncwarp();
    }
}

GB_EXPORT int gb_moe_route(const void* h, int h_dtype, int d, const float* w_router, const float* correction, const float* w_gate,
                           const int* positions, int n, int E, int top, int groups, int keep, float route_scale, int* choice_out,
                           float* weight_out, float* gate_out, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && d > 0 && E > 0 && E <= MOE_MAX_EXPERTS && top > 0 && top <= E, "gb_moe_route: bad sizes (experts %d, top %d)", E,
               top);
    GB_REQUIRE(groups >= 1 && E % groups == 0 && keep >= 1 && keep <= groups, "gb_moe_route: %d experts in %d groups, %d kept", E, groups,
               keep);
    GB_REQUIRE((size_t)d * 4 <= 160 * 1024, "gb_moe_route: a row of %d numbers does not fit shared memory", d);
    GB_REQUIRE(w_gate == nullptr || gate_out != nullptr, "gb_moe_route: a gate needs its output");
    if (n == 0) return 0;
    const size_t smem = (size_t)d * 4;
    if (h_dtype == GB_F32) {
        if (smem > 32 * 1024) cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        gb_launch(GB_PDL_ELEMENTWISE, moe_route_kernel<float>, dim3(n), dim3(MOE_ROUTE_THREADS), smem, stream, (const float*)h, d, w_router,
                  correction, w_gate, positions, n, E, top, groups, keep, route_scale, choice_out, weight_out, gate_out);
    } else if (h_dtype == GB_BF16) {
        if (smem > 32 * 1024)
            cudaFuncSetAttribute(moe_route_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        gb_launch(GB_PDL_ELEMENTWISE, moe_route_kernel<__nv_bfloat16>, dim3(n), dim3(MOE_ROUTE_THREADS), smem, stream,
                  (const __nv_bfloat16*)h, d, w_router, correction, w_gate, positions, n, E, top, groups, keep, route_scale, choice_out,
                  weight_out, gate_out);
    } else {
        GB_REQUIRE(false, "gb_moe_route: unsupported dtype %d", h_dtype);
    }
    return gb_check_launch("gb_moe_route");
}

// ----------------------------------------------------------------------------------------------
// One block per (row, choice k): pair[row, k, :] = W_down[e] relu(W_up[e] h[row])^2, e = choice[row, k].
// w_up [E * ff, d], w_down [E * d, ff] (the experts' matrices stacked by rows).
// ----------------------------------------------------------------------------------------------
constexpr int MOE_ROWS_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(MOE_ROWS_THREADS) moe_expert_rows_kernel(
    const T* __restrict__ h, int d, const T* __restrict__ w_up, const T* __restrict__ w_down, int ff, const int* __restrict__ choice,
    const int* __restrict__ positions, int n, int E, int top, float* __restrict__ pair) {
    extern __shared__ __align__(16) float moe_smem[];
    float* hx = moe_smem;            // d
    float* act = moe_smem + ((d + 3) & ~3);     // ff
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int row = blockIdx.x, k = blockIdx.y;
    if (row >= n || positions[row] < 0) return;
    const int e = choice[(size_t)row * top + k];
    float* dst = pair + ((size_t)row * top + k) * d;
    if (e < 0 || e >= E) {
        for (int i = threadIdx.x; i < d; i += MOE_ROWS_THREADS) dst[i] = 0.f;
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* src = h + (size_t)row * d;
    for (int i = threadIdx.x; i < d; i += MOE_ROWS_THREADS) hx[i] = gb_to_float(src[i]);
    __syncthreads();
    const T* up = w_up + (size_t)e * ff * d;
    for (int f = warp; f < ff; f += MOE_ROWS_THREADS / 32) {
        const float a = fmaxf(moe_warp_dot<T>(up + (size_t)f * d, hx, d, lane), 0.f);
        if (lane == 0) act[f] = a * a;
    }
    __syncthreads();
    const T* down = w_down + (size_t)e * d * ff;
    for (int c = warp; c < d; c += MOE_ROWS_THREADS / 32) {
        const float o = moe_warp_dot<T>(down + (size_t)c * ff, act, ff, lane);
        if (lane == 0) dst[c] = o;
    }
}

GB_EXPORT int gb_moe_expert_rows(const void* h, int dtype, int d, const void* w_up, const void* w_down, int ff, const int* choice,
                                 const int* positions, int n, int E, int top, float* pair, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && d > 0 && ff > 0 && E > 0 && top > 0, "gb_moe_expert_rows: bad sizes");
    const size_t smem = ((size_t)((d + 3) & ~3) + ff) * 4;
    GB_REQUIRE(smem <= 200 * 1024, "gb_moe_expert_rows: a row of %d and %d hidden numbers do not fit shared memory", d, ff);
    if (n == 0) return 0;
    dim3 grid(n, top);
    if (dtype == GB_F32) {
        if (smem > 32 * 1024) cudaFuncSetAttribute(moe_expert_rows_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        gb_launch(GB_PDL_GEMM, moe_expert_rows_kernel<float>, grid, dim3(MOE_ROWS_THREADS), smem, stream, (const float*)h, d,
                  (const float*)w_up, (const float*)w_down, ff, choice, positions, n, E, top, pair);
    } else if (dtype == GB_BF16) {
        if (smem > 32 * 1024)
            cudaFuncSetAttribute(moe_expert_rows_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        gb_launch(GB_PDL_GEMM, moe_expert_rows_kernel<__nv_bfloat16>, grid, dim3(MOE_ROWS_THREADS), smem, stream, (const __nv_bfloat16*)h,
                  d, (const __nv_bfloat16*)w_up, (const __nv_bfloat16*)w_down, ff, choice, positions, n, E, top, pair);
    } else {
        GB_REQUIRE(false, "gb_moe_expert_rows: unsupported dtype %d", dtype);
    }
    return gb_check_launch("gb_moe_expert_rows");
}

// ----------------------------------------------------------------------------------------------
// out[row, :] (+)= sum_k weight[row, k] * pair[row, k, :] + gate[row] * shared[row, :]
// ----------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ pair, const float* __restrict__ weight, int top,
                                                          const float* __restrict__ shared, long long lds, const float* __restrict__ gate,
                                                          const int* __restrict__ positions, float* __restrict__ out, long long ldo,
                                                          int n, int d, int accumulate) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int row = blockIdx.x;
    if (row >= n || positions[row] < 0) return;
    const float g = gate ? gate[row] : 1.f;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        float a = 0.f;
        for (int k = 0; k < top; ++k) a = fmaf(weight[(size_t)row * top + k], pair[((size_t)row * top + k) * d + j], a);
        if (shared) a = fmaf(g, shared[(size_t)row * lds + j], a);
        float* o = out + (size_t)row * ldo + j;
        *o = accumulate ? *o + a : a;
    }
}

GB_EXPORT int gb_moe_combine(const float* pair, const float* weight, int top, const float* shared, long long lds, const float* gate,
                             const int* positions, float* out, long long ldo, int n, int d, int accumulate, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && d > 0 && top > 0, "gb_moe_combine: bad sizes");
    if (n == 0) return 0;
    gb_launch(GB_PDL_ELEMENTWISE, moe_combine_kernel, dim3(n), dim3(256), 0, stream, pair, weight, top, shared, lds, gate, positions, out,
              ldo, n, d, accumulate);
    return gb_check_launch("gb_moe_combine");
}
