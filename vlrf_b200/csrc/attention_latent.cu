// Attention over a cache of latents: what a sequence keeps per token is one row [c | r] of C + R numbers, the
// normed latent c from which every head's keys and values are linear maps (k_h = Uk_h c, v_h = Uv_h c), and an
// optional rotated key part r that all heads share.  Per head the score of query position p and key position j is
//     (q_h · Uk_h c_j + qr_h · r_j) · scale  =  ((Uk_hᵀ q_h) · c_j + qr_h · r_j) · scale,
// so with the query carried into the latent space first (q'_h = Uk_hᵀ q_h, a product per head, gemm_heads.cu) every
// head attends the same rows with a "key" of C + R and a "value" of C numbers (the row's first C), and the head's
// output is Uv_h (Σ_j p_j c_j), another product per head.  The keys and values themselves never exist.
//
//   latent_append   one token's row into the paged cache: RMS norm (float32, plain weight) of the first C columns of
//                   the float32 projection, rotation by position of the last R (float32 angles), rounded once to the
//                   cache's dtype
//   latent_q_rows   a float32 query projection laid out per head as [dim | R] becomes the two operands of the
//                   attention: the unrotated parts, compact, in the activation dtype (the per-head product's input),
//                   and the rotated parts, rotated by position, in columns C… of the head's q' row
//   attn_latent     any mix of tokens; a warp per (token, head) walks the rows 0…position of its slot in chunks of
//                   32 with an online softmax in float32.  The 32-bit path's attention and the fallback of the other.
//
// Rotation: of a vector's first `dims` entries, entry i is paired with entry i + dims/2 ("rotate half" pairing), or,
// with `interleaved`, entry 2i with entry 2i + 1; the pair (u, v) at position p becomes (u cos a − v sin a,
// v cos a + u sin a), a = p · inv_freq[i]; entries beyond `dims` pass unchanged.  inv_freq is a float32 table from the
// caller.
//
// The cache of one layer is [block][BT][row_w] with row_w ≥ C + R; block_table as for the key/value cache.
#include "common.cuh"

namespace {
constexpr int LAT_WARPS = 4;
constexpr int LAT_MAX_C = 1024;          // latent width the general kernel holds in registers (32 a lane)

__device__ __forceinline__ void rotate_pair(float u, float v, float pos, float f, float& ou, float& ov) {
    const float a = pos * f;
    float s, c;
    sincosf(a, &s, &c);
    ou = u * c - v * s;
    ov = v * c + u * s;
}

template <typename ET>
__global__ void __launch_bounds__(128)
latent_append_kernel(const float* __restrict__ proj, int ld, int C, int R, const float* __restrict__ norm_w, float eps,
                     const float* __restrict__ inv_freq, int rot_dims, int interleaved, ET* __restrict__ cache, int row_w,
                     const int* __restrict__ block_table, int max_blocks, const int* __restrict__ tok_slot,
                     const int* __restrict__ tok_pos, int BT, int* __restrict__ dev_err) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    __shared__ float part[4];
    const int t = blockIdx.x;
    const int slot = tok_slot[t];
    if (slot < 0) return;                                     // padding row
    const int pos = tok_pos[t];
    const int bi = pos / BT;
    const int blk = (pos >= 0 && bi < max_blocks) ? block_table[(size_t)slot * max_blocks + bi] : -1;
    if (blk < 0) {
        if (threadIdx.x == 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
        return;
    }
    const float* src = proj + (size_t)t * ld;
    ET* dst = cache + ((size_t)blk * BT + (pos % BT)) * row_w;
    float s = 0.f;
    for (int i = threadIdx.x; i < C; i += 128) { const float v = src[i]; s = fmaf(v, v, s); }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    const float inv = 1.f / sqrtf((part[0] + part[1] + part[2] + part[3]) / (float)C + eps);
    for (int i = threadIdx.x; i < C; i += 128) ElemIO<ET>::store(dst + i, src[i] * inv * norm_w[i]);
    const int half = rot_dims / 2;
    for (int i = threadIdx.x; i < half; i += 128) {
        const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
        float ou, ov;
        rotate_pair(src[C + a], src[C + b], (float)pos, inv_freq[i], ou, ov);
        ElemIO<ET>::store(dst + C + a, ou);
        ElemIO<ET>::store(dst + C + b, ov);
    }
    for (int i = rot_dims + threadIdx.x; i < R; i += 128) ElemIO<ET>::store(dst + C + i, src[C + i]);
}

template <typename ET>
__global__ void __launch_bounds__(128)
latent_q_rows_kernel(const float* __restrict__ q, int ld_q, int H, int dim, int R, const float* __restrict__ inv_freq,
                     int rot_dims, int interleaved, const int* __restrict__ tok_pos, ET* __restrict__ qn, int ld_qn,
                     ET* __restrict__ qp, int ld_qp, int C) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const float pos = (float)tok_pos[t];
    const float* src = q + (size_t)t * ld_q;
    const int per = dim + R, half = rot_dims / 2;
    for (int i = threadIdx.x; i < H * dim; i += 128) {
        const int h = i / dim, c = i - h * dim;
        ElemIO<ET>::store(qn + (size_t)t * ld_qn + i, src[h * per + c]);
    }
    for (int i = threadIdx.x; i < H * half; i += 128) {
        const int h = i / half, c = i - h * half;
        const float* s = src + h * per + dim;
        const int a = interleaved ? 2 * c : c, b = interleaved ? 2 * c + 1 : c + half;
        float ou, ov;
        rotate_pair(s[a], s[b], pos, inv_freq[c], ou, ov);
        ET* d = qp + (size_t)t * ld_qp + (size_t)h * (C + R) + C;
        ElemIO<ET>::store(d + a, ou);
        ElemIO<ET>::store(d + b, ov);
    }
    const int rest = R - rot_dims;
    for (int i = threadIdx.x; i < H * rest; i += 128) {
        const int h = i / rest, c = rot_dims + (i - h * rest);
        ElemIO<ET>::store(qp + (size_t)t * ld_qp + (size_t)h * (C + R) + C + c, src[h * per + dim + c]);
    }
}

// the cache rows of the step's own tokens, as two plain matrices: latents [T][C] and rotated key parts [T][R]
template <typename ET>
__global__ void __launch_bounds__(128)
latent_gather_kernel(const ET* __restrict__ cache, int row_w, int C, int R, const int* __restrict__ block_table, int max_blocks,
                     const int* __restrict__ tok_slot, const int* __restrict__ tok_pos, int BT, ET* __restrict__ out_c,
                     ET* __restrict__ out_r, int* __restrict__ dev_err) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int slot = tok_slot[t], pos = tok_pos[t];
    const int blk = (slot >= 0 && pos >= 0 && pos / BT < max_blocks) ? block_table[(size_t)slot * max_blocks + pos / BT] : -1;
    if (slot >= 0 && blk < 0 && threadIdx.x == 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
    const ET* src = cache + ((size_t)max(blk, 0) * BT + (max(pos, 0) % BT)) * row_w;
    for (int i = threadIdx.x; i < C + R; i += 128) {
        const ET x = blk >= 0 ? src[i] : ET(0.f);                  // padding rows and lost blocks: zeros
        if (i < C) out_c[(size_t)t * C + i] = x;
        else out_r[(size_t)t * R + (i - C)] = x;
    }
}

template <typename ET>
__global__ void __launch_bounds__(LAT_WARPS * 32)
attn_latent_kernel(const ET* __restrict__ qp, int ld_q, const ET* __restrict__ cache, int row_w, int C, int R,
                   const int* __restrict__ block_table, int max_blocks, const int* __restrict__ tok_slot,
                   const int* __restrict__ tok_pos, ET* __restrict__ out, int ld_out, int H, int BT, float scale,
                   int window, int* __restrict__ dev_err) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    extern __shared__ float q_sm[];                            // [LAT_WARPS][C + R]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int h = blockIdx.y * LAT_WARPS + warp;
    if (h >= H) return;                                        // whole warps leave; no block-wide barrier below
    const int D = C + R;
    ET* dst = out + (size_t)t * ld_out + (size_t)h * C;
    const int slot = tok_slot[t];
    if (slot < 0) {                                            // a padding row: zeros, so that what follows stays finite
        for (int i = lane; i < C; i += 32) ElemIO<ET>::store(dst + i, 0.f);
        return;
    }
    const int pos = tok_pos[t];
    float* q = q_sm + warp * D;
    const ET* qsrc = qp + (size_t)t * ld_q + (size_t)h * D;
    for (int i = lane; i < D; i += 32) q[i] = ElemIO<ET>::load(qsrc + i) * scale;
    __syncwarp();

    float acc[LAT_MAX_C / 32];
#pragma unroll
    for (int i = 0; i < LAT_MAX_C / 32; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int first = (window > 0) ? max(0, pos - window + 1) : 0;
    const int* table = block_table + (size_t)slot * max_blocks;
    bool lost = false;
    for (int k0 = (first / 32) * 32; k0 <= pos; k0 += 32) {
        const int blk = table[k0 / BT];
        if (blk < 0) { lost = true; break; }
        const ET* base = cache + ((size_t)blk * BT + (k0 % BT)) * row_w;
        const int key = k0 + lane;
        const bool valid = key >= first && key <= pos;
        float s = -INFINITY;
        if (valid) {
            const ET* row = base + (size_t)lane * row_w;
            float dot = 0.f;
            for (int c = 0; c < D; ++c) dot = fmaf(q[c], ElemIO<ET>::load(row + c), dot);
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));             // at least one key of the chunk is visible
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < LAT_MAX_C / 32; ++i) acc[i] *= corr;
        const int n_here = min(32, pos - k0 + 1);
        for (int j = 0; j < n_here; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            if (pj == 0.f) continue;                           // uniform across the warp
            const ET* row = base + (size_t)j * row_w;
#pragma unroll
            for (int i = 0; i < LAT_MAX_C / 32; ++i) {
                const int c = i * 32 + lane;
                if (c < C) acc[i] = fmaf(pj, ElemIO<ET>::load(row + c), acc[i]);
            }
        }
        m = m_new;
    }
    if (lost && lane == 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
    const float inv = (l > 0.f) ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < LAT_MAX_C / 32; ++i) {
        const int c = i * 32 + lane;
        if (c < C) ElemIO<ET>::store(dst + c, acc[i] * inv);
    }
}
}  // namespace

extern "C" int vlrf_latent_append(const float* proj, int ld, int C, int R, const float* norm_w, float eps,
                                  const float* inv_freq, int rot_dims, int interleaved, void* cache, int dtype, int row_w,
                                  const int* block_table, int max_blocks, const int* tok_slot, const int* tok_pos,
                                  int T, int BT, int* dev_err, cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && C > 0 && R >= 0 && ld >= C + R && row_w >= C + R && BT > 0 && max_blocks > 0, "latent_append: bad sizes");
    VLRF_REQUIRE(rot_dims >= 0 && rot_dims <= R && rot_dims % 2 == 0, "latent_append: %d of %d columns cannot be rotated in pairs", rot_dims, R);
    VLRF_REQUIRE(rot_dims == 0 || inv_freq != nullptr, "latent_append: a rotation needs its table of frequencies");
    VLRF_REQUIRE(norm_w != nullptr && dev_err != nullptr, "latent_append: needs the norm's weight and the device error word");
    if (T == 0) return VLRF_OK;
    if (dtype == VLRF_F32)
        launch_chained(latent_append_kernel<float>, dim3(T), dim3(128), (size_t)(0), stream, proj, ld, C, R, norm_w, eps, inv_freq, rot_dims, interleaved, (float*)cache, row_w, block_table, max_blocks, tok_slot, tok_pos, BT, dev_err);
    else if (dtype == VLRF_BF16)
        launch_chained(latent_append_kernel<__nv_bfloat16>, dim3(T), dim3(128), (size_t)(0), stream, proj, ld, C, R, norm_w, eps, inv_freq, rot_dims, interleaved, (__nv_bfloat16*)cache, row_w, block_table, max_blocks, tok_slot, tok_pos, BT, dev_err);
    else return vlrf_fail(VLRF_ERR_INVALID_ARG, "latent_append: unknown dtype %d", dtype);
    return vlrf_check_launch("latent_append");
}

extern "C" int vlrf_latent_q_rows(const float* q, int ld_q, int H, int dim, int R, const float* inv_freq, int rot_dims, int interleaved,
                                  const int* tok_pos, void* qn, int ld_qn, void* qp, int ld_qp, int C, int dtype, int T,
                                  cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && H > 0 && dim > 0 && R >= 0 && C >= 0, "latent_q_rows: bad sizes");
    VLRF_REQUIRE(ld_q >= H * (dim + R) && ld_qn >= H * dim && ld_qp >= H * (C + R), "latent_q_rows: leading sizes are too small");
    VLRF_REQUIRE(rot_dims >= 0 && rot_dims <= R && rot_dims % 2 == 0 && (rot_dims == 0 || inv_freq != nullptr), "latent_q_rows: bad rotation");
    if (T == 0) return VLRF_OK;
    if (dtype == VLRF_F32)
        launch_chained(latent_q_rows_kernel<float>, dim3(T), dim3(128), (size_t)(0), stream, q, ld_q, H, dim, R, inv_freq, rot_dims, interleaved, tok_pos, (float*)qn, ld_qn, (float*)qp, ld_qp, C);
    else if (dtype == VLRF_BF16)
        launch_chained(latent_q_rows_kernel<__nv_bfloat16>, dim3(T), dim3(128), (size_t)(0), stream, q, ld_q, H, dim, R, inv_freq, rot_dims, interleaved, tok_pos, (__nv_bfloat16*)qn, ld_qn, (__nv_bfloat16*)qp, ld_qp, C);
    else return vlrf_fail(VLRF_ERR_INVALID_ARG, "latent_q_rows: unknown dtype %d", dtype);
    return vlrf_check_launch("latent_q_rows");
}

extern "C" int vlrf_latent_gather(const void* cache, int dtype, int row_w, int C, int R, const int* block_table, int max_blocks,
                                  const int* tok_slot, const int* tok_pos, void* out_c, void* out_r, int T, int BT, int* dev_err,
                                  cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && C > 0 && R >= 0 && row_w >= C + R && BT > 0 && max_blocks > 0 && out_c != nullptr && (R == 0 || out_r != nullptr) &&
                 dev_err != nullptr, "latent_gather: bad arguments");
    if (T == 0) return VLRF_OK;
    if (dtype == VLRF_F32)
        launch_chained(latent_gather_kernel<float>, dim3(T), dim3(128), (size_t)0, stream, (const float*)cache, row_w, C, R, block_table, max_blocks,
                       tok_slot, tok_pos, BT, (float*)out_c, (float*)out_r, dev_err);
    else if (dtype == VLRF_BF16)
        launch_chained(latent_gather_kernel<__nv_bfloat16>, dim3(T), dim3(128), (size_t)0, stream, (const __nv_bfloat16*)cache, row_w, C, R,
                       block_table, max_blocks, tok_slot, tok_pos, BT, (__nv_bfloat16*)out_c, (__nv_bfloat16*)out_r, dev_err);
    else return vlrf_fail(VLRF_ERR_INVALID_ARG, "latent_gather: unknown dtype %d", dtype);
    return vlrf_check_launch("latent_gather");
}

extern "C" int vlrf_attn_latent(const void* qp, int dtype, int ld_q, const void* cache, int row_w, int C, int R,
                                const int* block_table, int max_blocks, const int* tok_slot, const int* tok_pos,
                                void* out, int ld_out, int T, int H, int BT, float scale, int window, int* dev_err,
                                cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && H > 0 && C > 0 && R >= 0 && max_blocks > 0, "attn_latent: bad sizes");
    VLRF_REQUIRE(C <= LAT_MAX_C, "attn_latent: a latent of %d numbers is wider than %d", C, LAT_MAX_C);
    VLRF_REQUIRE(row_w >= C + R && ld_q >= H * (C + R) && ld_out >= H * C, "attn_latent: leading sizes are too small");
    VLRF_REQUIRE(BT % 32 == 0, "attn_latent: cache blocks of %d tokens are not a multiple of 32", BT);
    VLRF_REQUIRE(window >= 0 && dev_err != nullptr, "attn_latent: bad window or no device error word");
    if (T == 0) return VLRF_OK;
    dim3 grid(T, (H + LAT_WARPS - 1) / LAT_WARPS);
    const size_t smem = (size_t)LAT_WARPS * (C + R) * sizeof(float);
    if (dtype == VLRF_F32)
        launch_chained(attn_latent_kernel<float>, dim3(grid), dim3(LAT_WARPS * 32), (size_t)(smem), stream, (const float*)qp, ld_q, (const float*)cache, row_w, C, R, block_table, max_blocks, tok_slot, tok_pos, (float*)out, ld_out, H, BT, scale, window, dev_err);
    else if (dtype == VLRF_BF16)
        launch_chained(attn_latent_kernel<__nv_bfloat16>, dim3(grid), dim3(LAT_WARPS * 32), (size_t)(smem), stream, (const __nv_bfloat16*)qp, ld_q, (const __nv_bfloat16*)cache, row_w, C, R, block_table, max_blocks, tok_slot, tok_pos, (__nv_bfloat16*)out, ld_out, H, BT, scale, window, dev_err);
    else return vlrf_fail(VLRF_ERR_INVALID_ARG, "attn_latent: unknown dtype %d", dtype);
    return vlrf_check_launch("attn_latent");
}
