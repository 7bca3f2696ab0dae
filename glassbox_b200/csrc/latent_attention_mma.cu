// Attention over a latent cache on the tensor cores (bfloat16 mma.sync m16n8k16, float32 softmax and accumulators).
//
// All heads of a token score against the same cached row (latent | rotated key part) and sum the same latents, so
// the heads are packed into the rows of the matrix tiles: a tile's 16 rows are `tpt` consecutive tokens of one request
// times a group of G heads (G = min(heads, 16), tpt = 16 / G). A cached row is then read once for 16 (token, head)
// pairs instead of once per head, and its first C numbers serve as the value operand of the second product straight
// from the same shared-memory tile.
//
//   prompt portions  one block = 4 warps = 4 consecutive tiles of one request and head group; the block walks the keys
//                    from the first visible one to its last row's position in tiles of 64, staged with cp.async (two
//                    buffers), every warp taking the whole tile for its own 16 rows
//   decoding         one block = one tile (one token of one request, a head group) and one share of the keys; the four
//                    warps take a quarter of each 64-key tile for the same 16 rows and merge at the end; several shares
//                    leave (m, l, O) in float32 and latent_attention_merge_kernel finishes
//
// The sink logit of a head joins the denominator once, at the very end (in the merge when the keys are shared).
#include "common.cuh"

#include <cuda_pipeline.h>

constexpr int LM_BN = 64;                 // keys per staged tile
constexpr float LM_NEG_BIG = -1.0e30f;
constexpr float LM_LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void lm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void lm_ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void lm_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t lm_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct LatentMmaArgs {
    const __nv_bfloat16* q;        // [n, H, C + R]
    __nv_bfloat16* out;            // [n, H, C]
    float* part_o;                 // [n, H, splits, C]   (keys shared between blocks)
    float* part_ml;                // [n, H, splits, 2]
    const __nv_bfloat16* cache;    // [pages, page_size, C + R]
    const int* block_tables;
    int max_pages;
    const int* seq_first_row;
    const int* seq_start_pos;
    const float* sink;             // [H] or null
    int H, G, tpt, page_shift, splits, window;
    long long num_pages;
    float scale_log2;
    int* status;
};

// KEYS_OVER_WARPS false: prompt portions (warps = different rows, same keys); true: decoding (warps = same rows,
// different keys of each tile).
template <int C, int R, bool KEYS_OVER_WARPS>
__global__ void __launch_bounds__(128) latent_attention_mma_kernel(LatentMmaArgs p) {
    constexpr int W = C + R, WS = W + 8;                  // a staged row is padded by 16 bytes: ldmatrix meets no bank twice
    constexpr int KS = W / 16, CT = C / 8, CPR = W / 8;   // k16 steps of the scores, n8 tiles of the output, 16-byte chunks per row
    constexpr int NK = KEYS_OVER_WARPS ? LM_BN / 4 : LM_BN;   // keys of a staged tile that one warp takes
    constexpr int NT = NK / 8;
    extern __shared__ __align__(128) unsigned char lm_smem[];
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(lm_smem);   // [2][LM_BN][WS]
    gb_pdl_launch_dependents();
    gb_pdl_wait();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int hg = blockIdx.y, seq = blockIdx.z;
    const int row0 = p.seq_first_row[seq];
    const int nrows = p.seq_first_row[seq + 1] - row0;
    const int page_size = 1 << p.page_shift;
    int start_pos = p.seq_start_pos[seq];
    // the tokens of this block and of this warp's tile
    int tok_lo, split = 0;
    if (KEYS_OVER_WARPS) {
        tok_lo = 0;
        split = blockIdx.x;
    } else {
        const int groups = gridDim.x;
        tok_lo = (groups - 1 - (int)blockIdx.x) * 4 * p.tpt;       // the blocks with the most keys start first
        if (tok_lo >= nrows) return;
    }
    if (start_pos >= 0 && ((start_pos + nrows - 1) >> p.page_shift) >= p.max_pages) {
        if (threadIdx.x == 0) atomicOr(p.status, GB_STATUS_BAD_POSITION);
        start_pos = -1;
    }
    if (start_pos < 0) {                                     // a padding sequence: its rows read as zeros downstream
        if (blockIdx.x == 0 && hg == 0)
            for (int i = threadIdx.x; i < nrows * p.H * (C / 2); i += 128)
                reinterpret_cast<uint32_t*>(p.out + (size_t)row0 * p.H * C)[i] = 0u;
        return;
    }
    const int block_tokens = KEYS_OVER_WARPS ? 1 : min(4 * p.tpt, nrows - tok_lo);
    const int pos_lo = start_pos + tok_lo, pos_hi = start_pos + tok_lo + block_tokens - 1;
    const int key_lo = (p.window > 0 && pos_lo + 1 > p.window) ? pos_lo + 1 - p.window : 0;
    int kt_begin = key_lo / LM_BN, kt_end = pos_hi / LM_BN + 1;          // tiles [kt_begin, kt_end)
    if (KEYS_OVER_WARPS && p.splits > 1) {
        const int tiles = kt_end - kt_begin, per = (tiles + p.splits - 1) / p.splits;
        kt_begin = kt_begin + split * per;
        kt_end = min(kt_end, kt_begin + per);
    }
    const int* table = p.block_tables + (size_t)seq * p.max_pages;

    // this warp's rows: row g and row g + 8 of its tile
    const int tile_tok = KEYS_OVER_WARPS ? 0 : tok_lo + warp * p.tpt;
    int tok_a = tile_tok + g / p.G, tok_b = tile_tok + (g + 8) / p.G;
    const int head_a = hg * p.G + g % p.G, head_b = hg * p.G + (g + 8) % p.G;
    const bool ok_a = g / p.G < p.tpt && tok_a < nrows && head_a < p.H;
    const bool ok_b = (g + 8) / p.G < p.tpt && tok_b < nrows && head_b < p.H;
    const int pos_a = ok_a ? start_pos + tok_a : -1, pos_b = ok_b ? start_pos + tok_b : -1;
    const int first_a = (p.window > 0 && pos_a + 1 > p.window) ? pos_a + 1 - p.window : 0;
    const int first_b = (p.window > 0 && pos_b + 1 > p.window) ? pos_b + 1 - p.window : 0;
    int warp_pos_hi = max(pos_a, pos_b);                       // the last key any row of this warp sees
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) warp_pos_hi = max(warp_pos_hi, __shfl_xor_sync(0xffffffffu, warp_pos_hi, o));

    // the queries of the two rows, as A fragments
    uint32_t qf[KS][4];
    {
        const __nv_bfloat16* qa = p.q + ((size_t)(row0 + tok_a) * p.H + head_a) * W;
        const __nv_bfloat16* qb = p.q + ((size_t)(row0 + tok_b) * p.H + head_b) * W;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qf[ks][0] = ok_a ? *reinterpret_cast<const uint32_t*>(qa + ks * 16 + 2 * t) : 0u;
            qf[ks][1] = ok_b ? *reinterpret_cast<const uint32_t*>(qb + ks * 16 + 2 * t) : 0u;
            qf[ks][2] = ok_a ? *reinterpret_cast<const uint32_t*>(qa + ks * 16 + 8 + 2 * t) : 0u;
            qf[ks][3] = ok_b ? *reinterpret_cast<const uint32_t*>(qb + ks * 16 + 8 + 2 * t) : 0u;
        }
    }

    // Two threads per key of the tile: one page look-up and one address per thread, then half a row of 16-byte pieces.
    static_assert(CPR % 2 == 0, "a cached row is an even number of 16-byte pieces");
    auto load_tile = [&](int kt, int buf) {
        const int kk = threadIdx.x >> 1, half = threadIdx.x & 1;
        const int key = kt * LM_BN + kk;
        long long page = -1;
        if (key <= pos_hi) {
            page = table[key >> p.page_shift];
            if (page < 0 || page >= p.num_pages) {
                if (key >= key_lo) atomicOr(p.status, GB_STATUS_BAD_SLOT);   // (pages behind a window may be gone)
                page = -1;
            }
        }
        __nv_bfloat16* d = Ks + (size_t)buf * LM_BN * WS + kk * WS + half * (CPR / 2) * 8;
        if (page >= 0) {
            const __nv_bfloat16* src = p.cache + ((size_t)page * page_size + (key & (page_size - 1))) * W + half * (CPR / 2) * 8;
#pragma unroll
            for (int j = 0; j < CPR / 2; ++j) __pipeline_memcpy_async(d + j * 8, src + j * 8, 16);
        } else {
#pragma unroll
            for (int j = 0; j < CPR / 2; ++j) *reinterpret_cast<uint4*>(d + j * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
        __pipeline_commit();
    };

    float o[CT][4];
#pragma unroll
    for (int i = 0; i < CT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_a = LM_NEG_BIG, m_b = LM_NEG_BIG, l_a = 0.f, l_b = 0.f;

    if (kt_begin < kt_end) load_tile(kt_begin, 0);
    for (int kt = kt_begin; kt < kt_end; ++kt) {
        const int buf = (kt - kt_begin) & 1;
        if (kt + 1 < kt_end) {
            load_tile(kt + 1, buf ^ 1);
            __pipeline_wait_prior(1);
        } else {
            __pipeline_wait_prior(0);
        }
        __syncthreads();
        const int key0 = kt * LM_BN + (KEYS_OVER_WARPS ? warp * NK : 0);      // this warp's first key of the tile
        if (key0 <= warp_pos_hi) {
            const uint32_t tile = (uint32_t)__cvta_generic_to_shared(Ks + (size_t)buf * LM_BN * WS + (size_t)(key0 - kt * LM_BN) * WS);
            float s[NT][4];
#pragma unroll
            for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {
                    uint32_t b[4];
                    const int m = lane >> 3, r = lane & 7;
                    lm_ldmatrix_x4(b, tile + (uint32_t)(((np * 16 + (m >> 1) * 8 + r) * WS + ks * 16 + (m & 1) * 8) * 2));
                    lm_mma(s[2 * np], qf[ks], b[0], b[1]);
                    lm_mma(s[2 * np + 1], qf[ks], b[2], b[3]);
                }
            }
            // scale, mask, running maximum
            float mx_a = LM_NEG_BIG, mx_b = LM_NEG_BIG;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int key = key0 + nt * 8 + 2 * t;
                s[nt][0] = (key <= pos_a && key >= first_a) ? s[nt][0] * p.scale_log2 : LM_NEG_BIG;
                s[nt][1] = (key + 1 <= pos_a && key + 1 >= first_a) ? s[nt][1] * p.scale_log2 : LM_NEG_BIG;
                s[nt][2] = (key <= pos_b && key >= first_b) ? s[nt][2] * p.scale_log2 : LM_NEG_BIG;
                s[nt][3] = (key + 1 <= pos_b && key + 1 >= first_b) ? s[nt][3] * p.scale_log2 : LM_NEG_BIG;
                mx_a = fmaxf(mx_a, fmaxf(s[nt][0], s[nt][1]));
                mx_b = fmaxf(mx_b, fmaxf(s[nt][2], s[nt][3]));
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
            const float corr_a = exp2f(m_a - mn_a), corr_b = exp2f(m_b - mn_b);
            m_a = mn_a;
            m_b = mn_b;
            l_a *= corr_a;
            l_b *= corr_b;
#pragma unroll
            for (int i = 0; i < CT; ++i) {
                o[i][0] *= corr_a; o[i][1] *= corr_a;
                o[i][2] *= corr_b; o[i][3] *= corr_b;
            }
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                s[nt][0] = s[nt][0] > 0.5f * LM_NEG_BIG ? exp2f(s[nt][0] - mn_a) : 0.f;
                s[nt][1] = s[nt][1] > 0.5f * LM_NEG_BIG ? exp2f(s[nt][1] - mn_a) : 0.f;
                s[nt][2] = s[nt][2] > 0.5f * LM_NEG_BIG ? exp2f(s[nt][2] - mn_b) : 0.f;
                s[nt][3] = s[nt][3] > 0.5f * LM_NEG_BIG ? exp2f(s[nt][3] - mn_b) : 0.f;
                l_a += s[nt][0] + s[nt][1];
                l_b += s[nt][2] + s[nt][3];
            }
            // O += P V, V = the first C numbers of the same staged rows
#pragma unroll
            for (int kk = 0; kk < NK / 16; ++kk) {
                uint32_t a[4];
                a[0] = lm_pack(s[2 * kk][0], s[2 * kk][1]);
                a[1] = lm_pack(s[2 * kk][2], s[2 * kk][3]);
                a[2] = lm_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                a[3] = lm_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int dp = 0; dp < CT / 2; ++dp) {
                    uint32_t b[4];
                    const int m = lane >> 3, r = lane & 7;
                    lm_ldmatrix_x4_trans(b, tile + (uint32_t)(((kk * 16 + (m & 1) * 8 + r) * WS + dp * 16 + (m >> 1) * 8) * 2));
                    lm_mma(o[2 * dp], a, b[0], b[1]);
                    lm_mma(o[2 * dp + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();      // every warp is done with this buffer before the load after next overwrites it
    }
    // row sums: the four lanes of a row hold the sums of their own columns
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

    if (!KEYS_OVER_WARPS) {
        if (p.sink != nullptr) {
            if (ok_a) {
                const float sk = p.sink[head_a] * LM_LOG2E, mn = fmaxf(m_a, sk), corr = exp2f(m_a - mn);
                l_a = l_a * corr + exp2f(sk - mn);
#pragma unroll
                for (int i = 0; i < CT; ++i) { o[i][0] *= corr; o[i][1] *= corr; }
            }
            if (ok_b) {
                const float sk = p.sink[head_b] * LM_LOG2E, mn = fmaxf(m_b, sk), corr = exp2f(m_b - mn);
                l_b = l_b * corr + exp2f(sk - mn);
#pragma unroll
                for (int i = 0; i < CT; ++i) { o[i][2] *= corr; o[i][3] *= corr; }
            }
        }
        const float inv_a = l_a > 0.f ? 1.0f / l_a : 0.f, inv_b = l_b > 0.f ? 1.0f / l_b : 0.f;
        if (ok_a) {
            __nv_bfloat16* dst = p.out + ((size_t)(row0 + tok_a) * p.H + head_a) * C + 2 * t;
#pragma unroll
            for (int i = 0; i < CT; ++i) *reinterpret_cast<uint32_t*>(dst + i * 8) = lm_pack(o[i][0] * inv_a, o[i][1] * inv_a);
        }
        if (ok_b) {
            __nv_bfloat16* dst = p.out + ((size_t)(row0 + tok_b) * p.H + head_b) * C + 2 * t;
#pragma unroll
            for (int i = 0; i < CT; ++i) *reinterpret_cast<uint32_t*>(dst + i * 8) = lm_pack(o[i][2] * inv_b, o[i][3] * inv_b);
        }
        return;
    }

    // decoding: the four warps hold parts of the same 16 rows; they meet in shared memory (the staging buffers are free)
    float* om = reinterpret_cast<float*>(lm_smem);          // [4][16][C]
    float* ml = om + 4 * 16 * C;                            // [4][16][2]
    __syncthreads();
#pragma unroll
    for (int i = 0; i < CT; ++i) {
        *reinterpret_cast<float2*>(om + ((size_t)warp * 16 + g) * C + i * 8 + 2 * t) = make_float2(o[i][0], o[i][1]);
        *reinterpret_cast<float2*>(om + ((size_t)warp * 16 + g + 8) * C + i * 8 + 2 * t) = make_float2(o[i][2], o[i][3]);
    }
    if (t == 0) {
        ml[(warp * 16 + g) * 2] = m_a; ml[(warp * 16 + g) * 2 + 1] = l_a;
        ml[(warp * 16 + g + 8) * 2] = m_b; ml[(warp * 16 + g + 8) * 2 + 1] = l_b;
    }
    __syncthreads();
    for (int r = warp; r < 16; r += 4) {                    // a warp per row
        const int head = hg * p.G + r % p.G;
        if (r / p.G >= 1 || head >= p.H) continue;          // (decoding: one token per tile)
        float m = LM_NEG_BIG;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, ml[(w * 16 + r) * 2]);
        float wgt[4], l = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            wgt[w] = exp2f(ml[(w * 16 + r) * 2] - m);
            l += ml[(w * 16 + r) * 2 + 1] * wgt[w];
        }
        const size_t row = (size_t)row0 * p.H + head;
        if (p.splits > 1) {
            float* po = p.part_o + (row * p.splits + split) * C;
            for (int d = lane; d < C; d += 32)
                po[d] = om[(0 * 16 + r) * C + d] * wgt[0] + om[(1 * 16 + r) * C + d] * wgt[1] + om[(2 * 16 + r) * C + d] * wgt[2] +
                        om[(3 * 16 + r) * C + d] * wgt[3];
            if (lane == 0) {
                p.part_ml[(row * p.splits + split) * 2] = m;
                p.part_ml[(row * p.splits + split) * 2 + 1] = l;
            }
        } else {
            float corr = 1.f;
            if (p.sink != nullptr) {
                const float sk = p.sink[head] * LM_LOG2E, mn = fmaxf(m, sk);
                corr = exp2f(m - mn);
                l = l * corr + exp2f(sk - mn);
            }
            const float inv = l > 0.f ? corr / l : 0.f;
            __nv_bfloat16* dst = p.out + row * C;
            for (int d = lane; d < C; d += 32)
                dst[d] = __float2bfloat16_rn((om[(0 * 16 + r) * C + d] * wgt[0] + om[(1 * 16 + r) * C + d] * wgt[1] +
                                              om[(2 * 16 + r) * C + d] * wgt[2] + om[(3 * 16 + r) * C + d] * wgt[3]) * inv);
        }
    }
}

// One block per (row, head): merge the shares of the keys and add the sink. Thread s weighs share s, thread d sums
// dimension d over the shares; the loads of a sum do not depend on one another, so they are all in flight together
// (a warp that walked the shares one after the other paid the trip to memory once per share).
constexpr int LM_MAX_SPLITS = 64;

__global__ void __launch_bounds__(128) latent_attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                                     const float* __restrict__ sink, const int* __restrict__ positions,
                                                                     __nv_bfloat16* __restrict__ out, int n, int H, int C, int splits) {
    __shared__ float wgt[LM_MAX_SPLITS];
    __shared__ float red[4];
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int task = blockIdx.x;
    const int row = task / H, head = task % H;
    if (positions[row] < 0) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* ml = part_ml + (size_t)task * splits * 2;
    const float m_s = tid < splits ? ml[2 * tid] : LM_NEG_BIG;
    const float l_s = tid < splits ? ml[2 * tid + 1] : 0.f;
    float m = gb_warp_max(m_s);
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    const float sk = sink != nullptr ? sink[head] * LM_LOG2E : LM_NEG_BIG;
    const float mn = fmaxf(m, sk);
    const float w_s = exp2f(m_s - mn);
    if (tid < splits) wgt[tid] = w_s;
    float l = gb_warp_sum(l_s * w_s);
    __syncthreads();                       // (red is read by everyone before it is written again)
    if (lane == 0) red[warp] = l;
    __syncthreads();
    l = red[0] + red[1] + red[2] + red[3] + (sink != nullptr ? exp2f(sk - mn) : 0.f);
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    for (int d = tid; d < C; d += 128) {
        const float* po = part_o + (size_t)task * splits * C + d;
        float acc = 0.f;
        int s = 0;
        for (; s + 8 <= splits; s += 8) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = po[(size_t)(s + j) * C];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc = fmaf(v[j], wgt[s + j], acc);
        }
        for (; s < splits; ++s) acc = fmaf(po[(size_t)s * C], wgt[s], acc);
        out[(size_t)task * C + d] = __float2bfloat16_rn(acc * inv);
    }
}

GB_EXPORT int gb_latent_attention_mma_supported(int c, int r, int page_size) {
    const bool sizes = (c == 64 || c == 128) && (r == 16 || r == 32 || r == 64);
    return sizes && (page_size == 16 || page_size == 32 || page_size == 64);
}

template <int C, int R>
static int launch_latent_mma(const LatentMmaArgs& p, bool decode, int n_or_groups, int head_groups, int S, cudaStream_t stream) {
    constexpr int W = C + R;
    const size_t stage = (size_t)2 * LM_BN * (W + 8) * sizeof(__nv_bfloat16);
    const size_t merge = (size_t)(4 * 16 * C + 4 * 16 * 2) * sizeof(float);
    const size_t smem = decode && merge > stage ? merge : stage;
    cudaError_t e;
    if (decode) {
        auto kernel = latent_attention_mma_kernel<C, R, true>;
        static bool set = false;
        if (!set) { cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); set = true; }
        e = gb_launch(GB_PDL_ATTENTION, kernel, dim3(p.splits, head_groups, S), dim3(128), smem, stream, p);
    } else {
        auto kernel = latent_attention_mma_kernel<C, R, false>;
        static bool set = false;
        if (!set) { cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); set = true; }
        e = gb_launch(GB_PDL_ATTENTION, kernel, dim3(n_or_groups, head_groups, S), dim3(128), smem, stream, p);
    }
    if (e != cudaSuccess) {
        gb_set_error("gb_latent_attention_mma: launch failed: %s", cudaGetErrorString(e));
        return 2;
    }
    return 0;
}

// decode != 0: every sequence of the step brings one row (row i is sequence i); `splits` shares of the keys per row
// (part_o / part_ml needed when > 1). Otherwise prompt portions: `max_rows_per_seq` bounds the longest portion.
GB_EXPORT int gb_latent_attention_mma(const void* q, void* out, float* part_o, float* part_ml, const void* cache,
                                      const int* block_tables, int max_pages, const int* seq_first_row, const int* seq_start_pos,
                                      const int* positions, const float* sink, int n, int S, int max_rows_per_seq, int H, int c,
                                      int r, int page_size, long long num_pages, float scale, int window, int decode, int splits,
                                      int* status, cudaStream_t stream) {
    GB_REQUIRE(gb_latent_attention_mma_supported(c, r, page_size), "gb_latent_attention_mma: latent %d, rotated part %d, pages of %d "
               "are outside what the kernel is built for", c, r, page_size);
    GB_REQUIRE(n >= 0 && S >= 0 && H > 0 && max_pages > 0 && splits >= 1 && splits <= LM_MAX_SPLITS, "gb_latent_attention_mma: bad sizes");
    GB_REQUIRE(!decode || splits == 1 || (part_o != nullptr && part_ml != nullptr), "gb_latent_attention_mma: shares of the keys need "
               "buffers for their partial results");
    if (n == 0 || S == 0) return 0;
    LatentMmaArgs p = {};
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.part_o = part_o; p.part_ml = part_ml;
    p.cache = (const __nv_bfloat16*)cache; p.block_tables = block_tables; p.max_pages = max_pages;
    p.seq_first_row = seq_first_row; p.seq_start_pos = seq_start_pos; p.sink = sink;
    p.H = H; p.G = H < 16 ? H : 16; p.tpt = decode ? 1 : 16 / p.G;
    p.page_shift = page_size == 16 ? 4 : page_size == 32 ? 5 : 6;
    p.splits = decode ? splits : 1; p.window = window; p.num_pages = num_pages; p.scale_log2 = scale * LM_LOG2E; p.status = status;
    const int head_groups = gb_ceil_div(H, p.G);
    const int groups = decode ? 1 : gb_ceil_div(max_rows_per_seq > 0 ? max_rows_per_seq : 1, 4 * p.tpt);
    int rc;
#define LM_CASE(CC, RR) if (c == CC && r == RR) rc = launch_latent_mma<CC, RR>(p, decode != 0, groups, head_groups, S, stream); else
    LM_CASE(64, 16) LM_CASE(64, 32) LM_CASE(64, 64) LM_CASE(128, 16) LM_CASE(128, 32) LM_CASE(128, 64) rc = 1;
#undef LM_CASE
    if (rc) return rc;
    if (decode && splits > 1) {
        gb_launch(GB_PDL_ATTENTION, latent_attention_merge_kernel, dim3(n * H), dim3(128), 0, stream,
                  (const float*)part_o, (const float*)part_ml, sink, positions, (__nv_bfloat16*)out, n, H, c, splits);
    }
    return gb_check_launch("gb_latent_attention_mma");
}
