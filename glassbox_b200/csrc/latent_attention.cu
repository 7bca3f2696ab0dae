// Attention over a compressed (latent) key/value cache.
//
// Per token the cache keeps ONE row of c + r numbers: a latent vector of c numbers (RMS-normed, with a plain gain)
// from which every head's unrotated key and value are linear maps (W_uk, W_uv), and one rotated key part of r numbers
// shared by all heads. Because key and value are linear in the latent, a head's score against a cached token is
//     (W_uk_h^T q_unrotated_h) . latent + q_rotated_h . key_rotated
// and its output is W_uv_h (sum_j p_j latent_j): the up-projections move to the query and to the output, and the
// kernel below is attention of H heads over one shared "key" of c + r numbers whose first c numbers are also the
// "value". Softmax may carry a sink: a learned logit per head that joins the denominator only (no key, no value, not
// scaled, counted once).
//
//   gb_latent_kv_write        rotates each head's rotated query part into the absorbed-query buffer, and (for a layer
//                             that owns its cache) norms the latent, rotates the shared key part and stores both
//   gb_latent_attention_rows  one warp per (row, head), float32 online softmax; any sizes; the float32 path's kernel
//                             and the reference beside the tensor-core one
//
// Rotation: dimension 2i is paired with 2i+1 over the first `rot_dims` numbers of the rotated part; the pair (u, v) at
// position p becomes (u cos a - v sin a, v cos a + u sin a), a = float(p) * inv_freq[i], all in float32.
#include "common.cuh"

#include <float.h>

// proj: [n, ldp]; the queries are columns 0 .. H*(dq+r)-1, head by head [dq unrotated | r rotated]; for a layer that
// writes the cache the c + r columns from `kv_col` on are the raw latent and the raw shared key part.
// qabs: [n, H, c + r]; this kernel fills [.., c:] with the rotated query parts (the first c numbers of each head come
// from the product with W_uk^T).
template <typename T>
__global__ void __launch_bounds__(128) latent_kv_write_kernel(
    const T* __restrict__ proj, long long ldp, int kv_col, T* __restrict__ qabs, T* __restrict__ cache,
    const float* __restrict__ latent_gain, const float* __restrict__ inv_freq, const int* __restrict__ positions,
    const int* __restrict__ slots, int n, int H, int dq, int r, int c, int rot_dims, long long num_slots, float eps,
    int write_kv, int* __restrict__ status) {
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int row = blockIdx.x;
    if (row >= n) return;
    const int pos = positions[row];
    if (pos < 0) return;    // a padding row
    const float fpos = (float)pos;
    const T* prow = proj + (size_t)row * ldp;
    const int half = rot_dims / 2;
    // queries: rotated parts, pair by pair
    T* qrow = qabs + (size_t)row * H * (c + r);
    for (int idx = threadIdx.x; idx < H * (r / 2 + (r & 1)); idx += blockDim.x) {
        const int per = r / 2 + (r & 1);
        const int h = idx / per, i = idx % per;
        const T* src = prow + (size_t)h * (dq + r) + dq;
        T* dst = qrow + (size_t)h * (c + r) + c;
        if (2 * i + 1 >= r) {   // an odd last number passes unchanged
            dst[2 * i] = src[2 * i];
            continue;
        }
        const float u = gb_to_float(src[2 * i]), v = gb_to_float(src[2 * i + 1]);
        if (i < half) {
            float sn, cs;
            sincosf(fpos * inv_freq[i], &sn, &cs);
            dst[2 * i] = gb_from_float<T>(u * cs - v * sn);
            dst[2 * i + 1] = gb_from_float<T>(v * cs + u * sn);
        } else {
            dst[2 * i] = src[2 * i];
            dst[2 * i + 1] = src[2 * i + 1];
        }
    }
    if (!write_kv) return;
    const long long slot = slots[row];
    if (slot < 0 || slot >= num_slots) {
        if (threadIdx.x == 0) atomicOr(status, GB_STATUS_BAD_SLOT);
        return;
    }
    const T* kv = prow + kv_col;
    T* dst = cache + (size_t)slot * (c + r);
    __shared__ float partial[4];
    __shared__ float total;
    float ss = 0.f;
    for (int j = threadIdx.x; j < c; j += blockDim.x) {
        const float t = gb_to_float(kv[j]);
        ss = fmaf(t, t, ss);
    }
    ss = gb_warp_sum(ss);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) total = 1.0f / sqrtf((partial[0] + partial[1] + partial[2] + partial[3]) / (float)c + eps);
    __syncthreads();
    const float s = total;
    for (int j = threadIdx.x; j < c; j += blockDim.x) dst[j] = gb_from_float<T>(latent_gain[j] * (gb_to_float(kv[j]) * s));
    for (int i = threadIdx.x; i < r / 2 + (r & 1); i += blockDim.x) {
        if (2 * i + 1 >= r) {
            dst[c + 2 * i] = kv[c + 2 * i];
            continue;
        }
        const float u = gb_to_float(kv[c + 2 * i]), v = gb_to_float(kv[c + 2 * i + 1]);
        if (i < half) {
            float sn, cs;
            sincosf(fpos * inv_freq[i], &sn, &cs);
            dst[c + 2 * i] = gb_from_float<T>(u * cs - v * sn);
            dst[c + 2 * i + 1] = gb_from_float<T>(v * cs + u * sn);
        } else {
            dst[c + 2 * i] = kv[c + 2 * i];
            dst[c + 2 * i + 1] = kv[c + 2 * i + 1];
        }
    }
}

GB_EXPORT int gb_latent_kv_write(const void* proj, long long ldp, int kv_col, void* qabs, void* cache, int dtype,
                                 const float* latent_gain, const float* inv_freq, const int* positions, const int* slots,
                                 int n, int H, int dq, int r, int c, int rot_dims, long long num_slots, float eps,
                                 int write_kv, int* status, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && H > 0 && dq >= 0 && r >= 0 && c > 0, "gb_latent_kv_write: bad sizes");
    GB_REQUIRE(rot_dims >= 0 && rot_dims <= r && rot_dims % 2 == 0, "gb_latent_kv_write: %d rotated numbers do not fit a part of %d",
               rot_dims, r);
    if (n == 0) return 0;
    if (dtype == GB_F32)
        gb_launch(GB_PDL_ELEMENTWISE, latent_kv_write_kernel<float>, dim3(n), dim3(128), 0, stream, (const float*)proj, ldp, kv_col,
                  (float*)qabs, (float*)cache, latent_gain, inv_freq, positions, slots, n, H, dq, r, c, rot_dims, num_slots, eps,
                  write_kv, status);
    else if (dtype == GB_BF16)
        gb_launch(GB_PDL_ELEMENTWISE, latent_kv_write_kernel<__nv_bfloat16>, dim3(n), dim3(128), 0, stream,
                  (const __nv_bfloat16*)proj, ldp, kv_col, (__nv_bfloat16*)qabs, (__nv_bfloat16*)cache, latent_gain, inv_freq,
                  positions, slots, n, H, dq, r, c, rot_dims, num_slots, eps, write_kv, status);
    else
        GB_REQUIRE(false, "gb_latent_kv_write: unsupported dtype %d", dtype);
    return gb_check_launch("gb_latent_kv_write");
}

// ----------------------------------------------------------------------------------------------
// One warp per (row, head). q: [n, H, c + r] absorbed queries; cache: [pages, page_size, c + r]; out: [n, H, c], the
// probability-weighted sum of latents. Keys are taken 32 at a time from the first visible key, so a row's reduction
// order depends only on its position.
// ----------------------------------------------------------------------------------------------
constexpr int LAT_WARPS = 4;
constexpr int LAT_MAX_QK = 1024;     // c + r
constexpr int LAT_MAX_C = 768;       // c

template <typename T>
__global__ void __launch_bounds__(LAT_WARPS * 32) latent_attention_rows_kernel(
    const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ cache, const int* __restrict__ block_tables,
    int max_pages, const int* __restrict__ row_seq, const int* __restrict__ positions, const float* __restrict__ sink,
    int n, int H, int c, int r, int page_size, long long num_pages, float scale, int window, int* __restrict__ status) {
    extern __shared__ float lat_qs[];     // [LAT_WARPS][c + r]
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long task = (long long)blockIdx.x * LAT_WARPS + warp;
    if (task >= (long long)n * H) return;
    const int row = (int)(task / H), head = (int)(task % H);
    const int w = c + r;
    int pos = positions[row];
    if (pos >= 0 && pos / page_size >= max_pages) {
        if (lane == 0) atomicOr(status, GB_STATUS_BAD_POSITION);
        pos = -1;
    }
    const int* table = block_tables + (size_t)row_seq[row] * max_pages;
    float* qs = lat_qs + (size_t)warp * w;
    const T* qrow = q + ((size_t)row * H + head) * w;
    for (int i = lane; i < w; i += 32) qs[i] = gb_to_float(qrow[i]);
    __syncwarp();

    const int first = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    float m = -FLT_MAX, l = 0.f;
    float acc[LAT_MAX_C / 32];
#pragma unroll
    for (int j = 0; j < LAT_MAX_C / 32; ++j) acc[j] = 0.f;

    for (int base = first; base <= pos; base += 32) {
        const int key = base + lane;
        float s = -FLT_MAX;
        long long krow = -1;
        if (key <= pos) {
            const long long page = table[key / page_size];
            if (page < 0 || page >= num_pages) {
                atomicOr(status, GB_STATUS_BAD_SLOT);
            } else {
                krow = (page * page_size + key % page_size) * w;
                const T* kp = cache + krow;
                float d0 = 0.f, d1 = 0.f;
                int i = 0;
                for (; i + 1 < w; i += 2) {
                    d0 = fmaf(qs[i], gb_to_float(kp[i]), d0);
                    d1 = fmaf(qs[i + 1], gb_to_float(kp[i + 1]), d1);
                }
                if (i < w) d0 = fmaf(qs[i], gb_to_float(kp[i]), d0);
                s = (d0 + d1) * scale;
            }
        }
        const float m_new = fmaxf(m, gb_warp_max(s));
        const float p = (krow >= 0) ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);
        l = l * corr + gb_warp_sum(p);
#pragma unroll
        for (int j = 0; j < LAT_MAX_C / 32; ++j) acc[j] *= corr;
        m = m_new;
        const int count = min(32, pos - base + 1);
        for (int t = 0; t < count; ++t) {
            const float pt = __shfl_sync(0xffffffffu, p, t);
            const long long vr = __shfl_sync(0xffffffffu, krow, t);
            if (vr < 0) continue;
            const T* vp = cache + vr;
#pragma unroll
            for (int j = 0; j < LAT_MAX_C / 32; ++j) {
                const int i = lane + 32 * j;
                if (i < c) acc[j] = fmaf(pt, gb_to_float(vp[i]), acc[j]);
            }
        }
    }
    if (sink != nullptr && pos >= 0) {     // the sink joins the denominator: exp(sink) counted once, unscaled
        const float sk = sink[head];
        const float m_new = fmaxf(m, sk);
        const float corr = expf(m - m_new);
        l = l * corr + expf(sk - m_new);
#pragma unroll
        for (int j = 0; j < LAT_MAX_C / 32; ++j) acc[j] *= corr;
    }
    T* orow = out + ((size_t)row * H + head) * c;
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int j = 0; j < LAT_MAX_C / 32; ++j) {
        const int i = lane + 32 * j;
        if (i < c) orow[i] = gb_from_float<T>(acc[j] * inv);
    }
}

GB_EXPORT int gb_latent_attention_rows(const void* q, void* out, int dtype, const void* cache, const int* block_tables,
                                       int max_pages, const int* row_seq, const int* positions, const float* sink, int n,
                                       int H, int c, int r, int page_size, long long num_pages, float scale, int window,
                                       int* status, cudaStream_t stream) {
    GB_REQUIRE(n >= 0 && H > 0 && c > 0 && r >= 0, "gb_latent_attention_rows: bad sizes");
    GB_REQUIRE(c <= LAT_MAX_C && c + r <= LAT_MAX_QK, "gb_latent_attention_rows: a latent of %d with a rotated part of %d is "
               "outside the kernel's range (%d, %d in all)", c, r, LAT_MAX_C, LAT_MAX_QK);
    GB_REQUIRE(page_size > 0 && max_pages > 0, "gb_latent_attention_rows: bad page geometry");
    if (n == 0) return 0;
    const int blocks = gb_ceil_div((long long)n * H, LAT_WARPS);
    const size_t smem = (size_t)LAT_WARPS * (c + r) * sizeof(float);
    if (dtype == GB_F32)
        gb_launch(GB_PDL_ATTENTION, latent_attention_rows_kernel<float>, dim3(blocks), dim3(LAT_WARPS * 32), smem, stream,
                  (const float*)q, (float*)out, (const float*)cache, block_tables, max_pages, row_seq, positions, sink, n, H, c, r,
                  page_size, num_pages, scale, window, status);
    else if (dtype == GB_BF16)
        gb_launch(GB_PDL_ATTENTION, latent_attention_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(LAT_WARPS * 32), smem, stream,
                  (const __nv_bfloat16*)q, (__nv_bfloat16*)out, (const __nv_bfloat16*)cache, block_tables, max_pages, row_seq,
                  positions, sink, n, H, c, r, page_size, num_pages, scale, window, status);
    else
        GB_REQUIRE(false, "gb_latent_attention_rows: unsupported dtype %d", dtype);
    return gb_check_launch("gb_latent_attention_rows");
}
