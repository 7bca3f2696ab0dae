// One small product per head, all heads in one launch: out[row, h, :N] = a[row, h, :K] . w[h]^T with w[h] an [N, K]
// matrix, bfloat16 in and out, float32 sums on the tensor cores (mma.sync m16n8k16).
//
// This is the shape of the up-projections of latent attention once they are moved to the query and to the weighted sum
// of latents: K and N are a head's sizes (tens to a few hundred), so a head's product is far too small for a launch of
// its own. One block = 64 rows x one head x up to 128 output columns; a and w[h] are staged once in shared memory
// (rows padded by 16 bytes so that ldmatrix meets no bank twice), each of the four warps takes 16 rows.
#include "common.cuh"

#include <cuda_pipeline.h>

constexpr int HL_BM = 64, HL_BN = 128, HL_MAX_K = 256;

__device__ __forceinline__ void hl_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void hl_ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__global__ void __launch_bounds__(128) head_linear_kernel(const __nv_bfloat16* __restrict__ a, long long lda, long long a_head,
                                                          const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                                          long long ldc, long long c_head, int n, int N, int K) {
    extern __shared__ __align__(128) unsigned char hl_smem[];
    gb_pdl_launch_dependents();
    const int KS = K + 8;                                    // padded row, elements
    __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(hl_smem);     // [64][KS]
    __nv_bfloat16* Ws = As + HL_BM * KS;                               // [128][KS]
    const int head = blockIdx.y, m0 = blockIdx.x * HL_BM, n0 = blockIdx.z * HL_BN;
    const int cols = min(HL_BN, N - n0);
    const int cpr = K / 8;                                   // 16-byte chunks per row
    const __nv_bfloat16* wh = w + ((size_t)head * N + n0) * K;
    for (int c = threadIdx.x; c < cols * cpr; c += 128) {    // the weights do not depend on the kernel before: ask first
        const int r = c / cpr, ch = c % cpr;
        __pipeline_memcpy_async(Ws + r * KS + ch * 8, wh + (size_t)r * K + ch * 8, 16);
    }
    __pipeline_commit();
    gb_pdl_wait();
    const __nv_bfloat16* ah = a + (size_t)head * a_head;
    for (int c = threadIdx.x; c < HL_BM * cpr; c += 128) {
        const int r = c / cpr, ch = c % cpr;
        __nv_bfloat16* d = As + r * KS + ch * 8;
        if (m0 + r < n) __pipeline_memcpy_async(d, ah + (size_t)(m0 + r) * lda + ch * 8, 16);
        else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
    }
    for (int c = threadIdx.x + cols * cpr; c < HL_BN * cpr; c += 128) {      // rows of the weight tile beyond N: zeros
        const int r = c / cpr, ch = c % cpr;
        *reinterpret_cast<uint4*>(Ws + r * KS + ch * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
    __pipeline_commit();
    __pipeline_wait_prior(0);
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3, m = lane >> 3, r8 = lane & 7;
    const uint32_t a_base = (uint32_t)__cvta_generic_to_shared(As + (size_t)warp * 16 * KS);
    const uint32_t w_base = (uint32_t)__cvta_generic_to_shared(Ws);
    float acc[HL_BN / 8][4];
#pragma unroll
    for (int i = 0; i < HL_BN / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
    const int n_pairs = (cols + 15) / 16;
    for (int ks = 0; ks < K / 16; ++ks) {
        uint32_t af[4];
        // A fragment: matrices (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
        hl_ldmatrix_x4(af, a_base + (uint32_t)((((m & 1) * 8 + r8) * KS + ks * 16 + (m >> 1) * 8) * 2));
#pragma unroll
        for (int np = 0; np < HL_BN / 16; ++np) {
            if (np < n_pairs) {
                uint32_t b[4];
                hl_ldmatrix_x4(b, w_base + (uint32_t)(((np * 16 + (m >> 1) * 8 + r8) * KS + ks * 16 + (m & 1) * 8) * 2));
                hl_mma(acc[2 * np], af, b[0], b[1]);
                hl_mma(acc[2 * np + 1], af, b[2], b[3]);
            }
        }
    }
    const int row_a = m0 + warp * 16 + g, row_b = row_a + 8;
    __nv_bfloat16* oh = out + (size_t)head * c_head + n0;
#pragma unroll
    for (int nt = 0; nt < HL_BN / 8; ++nt) {
        const int col = nt * 8 + 2 * t;
        if (col < cols) {      // (N is even: a pair never straddles the edge)
            if (row_a < n) {
                __nv_bfloat162 v = __floats2bfloat162_rn(acc[nt][0], acc[nt][1]);
                *reinterpret_cast<__nv_bfloat162*>(oh + (size_t)row_a * ldc + col) = v;
            }
            if (row_b < n) {
                __nv_bfloat162 v = __floats2bfloat162_rn(acc[nt][2], acc[nt][3]);
                *reinterpret_cast<__nv_bfloat162*>(oh + (size_t)row_b * ldc + col) = v;
            }
        }
    }
}

GB_EXPORT int gb_head_linear_supported(const void* a, long long lda, long long a_head, const void* w, const void* out,
                                       long long ldc, long long c_head, int N, int K) {
    return K > 0 && K <= HL_MAX_K && K % 16 == 0 && N > 0 && N % 2 == 0 && lda % 8 == 0 && a_head % 8 == 0 &&
           (uintptr_t)a % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)out % 4 == 0 && ldc % 2 == 0 && c_head % 2 == 0;
}

GB_EXPORT int gb_head_linear(const void* a, long long lda, long long a_head, const void* w, void* out, long long ldc,
                             long long c_head, int n, int heads, int N, int K, cudaStream_t stream) {
    GB_REQUIRE(gb_head_linear_supported(a, lda, a_head, w, out, ldc, c_head, N, K),
               "gb_head_linear: K=%d must be a multiple of 16 up to %d, N=%d even, operands aligned", K, HL_MAX_K, N);
    GB_REQUIRE(n >= 0 && heads > 0 && heads <= 65535, "gb_head_linear: bad sizes");
    if (n == 0) return 0;
    const size_t smem = (size_t)(HL_BM + HL_BN) * (K + 8) * sizeof(__nv_bfloat16);
    static size_t allowed = 48 * 1024;
    if (smem > allowed) {
        cudaFuncSetAttribute(head_linear_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        allowed = smem;
    }
    dim3 grid(gb_ceil_div(n, HL_BM), heads, gb_ceil_div(N, HL_BN));
    cudaError_t e = gb_launch(GB_PDL_GEMM, head_linear_kernel, grid, dim3(128), smem, stream, (const __nv_bfloat16*)a, lda, a_head,
                              (const __nv_bfloat16*)w, (__nv_bfloat16*)out, ldc, c_head, n, N, K);
    if (e != cudaSuccess) {
        gb_set_error("gb_head_linear: launch failed: %s", cudaGetErrorString(e));
        return 2;
    }
    return 0;
}
