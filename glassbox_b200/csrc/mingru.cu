// minGRU: a gated recurrence whose gates read only the current token, so that the state is a first-order linear
// recurrence per channel:
//     z_t = sigmoid(pz_t + bz),  u_t = px_t + bx,  c_t = u_t + 1/2 (u_t >= 0) | sigmoid(u_t) (u_t < 0)
//     S_t = (1 - z_t) S_(t-1) + z_t c_t,           out_t = S_t * silu(pg_t)
// pz | px | pg are the float32 sums of the stacked projection ([n, ld], three blocks of `width` columns), S lives in the
// request's state slot (float32, `width` numbers from `state_off`), and everything between is float32.
//
// mingru_scan_kernel: a block owns MG_CH channels of one request's rows. Its warps (up to MG_PARTS) cut the rows into
// consecutive pieces: each group first composes its piece into (A, B) with S_end = A * S_start + B, the pieces' carries
// are chained in order (a handful of multiply-adds), and a second walk over the piece writes the outputs from the true
// incoming state. The order of the floating-point operations of a row depends on the length of its portion only through
// the piece borders; a portion of one row (decoding) is the plain update.
#include "common.cuh"

constexpr int MG_CH = 32;          // channels per block: a warp's lanes (16 for long portions: twice the pieces per block)
constexpr int MG_PARTS = 64;       // at most this many pieces of the rows (the launch says how many: blockDim.x / channels)
constexpr int MG_MIN_PIECE = 8;    // shorter portions are walked by fewer groups
constexpr int MG_THREADS = 1024;

__device__ __forceinline__ float mg_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }

template <typename T>
__global__ void __launch_bounds__(MG_THREADS) mingru_scan_kernel(
    const float* __restrict__ proj, long long ld, const float* __restrict__ bz, const float* __restrict__ bx,
    float* __restrict__ state, long long state_stride, long long state_off, T* __restrict__ out, long long ldo,
    const int* __restrict__ seq_first_row, const int* __restrict__ seq_start_pos, const int* __restrict__ seq_slots, int S, int width,
    int num_slots, int write_state, int chw, int* __restrict__ status) {
    __shared__ float sa[MG_PARTS][MG_CH], sb[MG_PARTS][MG_CH];
    gb_pdl_launch_dependents();
    gb_pdl_wait();
    const int seq = blockIdx.x;
    if (seq >= S || seq_start_pos[seq] < 0) return;
    const int slot = seq_slots[seq];
    if (slot < 0 || slot >= num_slots) {
        if (threadIdx.x == 0) atomicOr(status, GB_STATUS_BAD_SLOT);
        return;
    }
    const int lane = threadIdx.x % chw, part = threadIdx.x / chw;      // chw channels per block, blockDim.x / chw pieces
    const int ch = blockIdx.y * chw + lane;
    const bool live = ch < width;
    const int r0 = seq_first_row[seq], len = seq_first_row[seq + 1] - r0;
    int parts = (len + MG_MIN_PIECE - 1) / MG_MIN_PIECE;
    const int most = (int)blockDim.x / chw;
    parts = parts < 1 ? 1 : (parts > most ? most : parts);
    const int piece = (len + parts - 1) / parts;
    const int lo = r0 + part * piece, hi = min(lo + piece, r0 + len);
    const float biasz = live ? bz[ch] : 0.f, biasx = live ? bx[ch] : 0.f;
    float* st = state + (size_t)slot * state_stride + state_off;
    if (parts > 1) {
        float A = 1.f, B = 0.f;
        if (live && part < parts) {
#pragma unroll 4
            for (int r = lo; r < hi; ++r) {
                const float* p = proj + (size_t)r * ld;
                const float z = mg_sigmoid(p[ch] + biasz);
                const float u = p[width + ch] + biasx;
                const float c = u >= 0.f ? u + 0.5f : mg_sigmoid(u);
                A *= 1.0f - z;
                B = fmaf(1.0f - z, B, z * c);
            }
        }
        sa[part][lane] = A;
        sb[part][lane] = B;
    }
    __syncthreads();
    float s = 0.f;
    const bool walks = live && part < parts;
    if (walks) {
        s = st[ch];
        for (int k = 0; k < part; ++k) s = fmaf(sa[k][lane], s, sb[k][lane]);      // the state at the start of this piece
#pragma unroll 4
        for (int r = lo; r < hi; ++r) {
            const float* p = proj + (size_t)r * ld;
            const float z = mg_sigmoid(p[ch] + biasz);
            const float u = p[width + ch] + biasx;
            const float c = u >= 0.f ? u + 0.5f : mg_sigmoid(u);
            s = fmaf(1.0f - z, s, z * c);
            const float gte = p[2 * width + ch];
            out[(size_t)r * ldo + ch] = gb_from_float<T>(s * (gte * mg_sigmoid(gte)));
        }
    }
    __syncthreads();          // every group has read the incoming state before the last one replaces it
    if (walks && write_state && part == parts - 1) st[ch] = s;
}

GB_EXPORT int gb_mingru_scan(const float* proj, long long ld, const float* bz, const float* bx, float* state, long long state_stride,
                             long long state_off, void* out, long long ldo, int out_dtype, const int* seq_first_row,
                             const int* seq_start_pos, const int* seq_slots, int S, int width, int num_slots, int write_state,
                             int max_rows, int* status, cudaStream_t stream) {
    GB_REQUIRE(S >= 0 && width > 0 && num_slots > 0, "gb_mingru_scan: bad sizes");
    GB_REQUIRE(state_off >= 0 && state_off + width <= state_stride, "gb_mingru_scan: the state does not fit its slot");
    if (S == 0) return 0;
    // as many pieces as the longest portion of the step has (the caller's bound on a request's rows in this step); long
    // portions take 16 channels per block, so that a block of 1024 threads cuts them into 64 pieces
    int pieces = gb_ceil_div(max_rows > 0 ? max_rows : 1, MG_MIN_PIECE);
    const int chw = pieces > MG_THREADS / MG_CH ? 16 : MG_CH;
    pieces = pieces < 1 ? 1 : (pieces > MG_THREADS / chw ? MG_THREADS / chw : pieces);
    dim3 grid(S, gb_ceil_div(width, chw));
    const dim3 block(((chw * pieces + 31) / 32) * 32);
    if (out_dtype == GB_F32)
        gb_launch(GB_PDL_ELEMENTWISE, mingru_scan_kernel<float>, grid, block, 0, stream, proj, ld, bz, bx, state,
                  state_stride, state_off, (float*)out, ldo, seq_first_row, seq_start_pos, seq_slots, S, width, num_slots, write_state,
                  chw, status);
    else if (out_dtype == GB_BF16)
        gb_launch(GB_PDL_ELEMENTWISE, mingru_scan_kernel<__nv_bfloat16>, grid, block, 0, stream, proj, ld, bz, bx, state,
                  state_stride, state_off, (__nv_bfloat16*)out, ldo, seq_first_row, seq_start_pos, seq_slots, S, width, num_slots,
                  write_state, chw, status);
    else
        GB_REQUIRE(false, "gb_mingru_scan: unsupported output dtype %d", out_dtype);
    return gb_check_launch("gb_mingru_scan");
}
