// Products with a weight matrix of their own for every head or every expert, on the CUDA cores (float32 FMAs, any
// sizes, float32 or bfloat16 operands): the form every such product takes in the 32-bit path, and the fallback of the
// bfloat16 path.  Each output element sums over k in an order that does not depend on the number of rows.
//
//   gemm_heads     Y[m][h][:] = X[m][h][:] · W[h]ᵀ for h < H: X rows of stride ldx with head h at column h·x_hs
//                  (K columns), W [H][N][K], Y rows of stride ldy with head h at column h·y_hs (N columns).  What
//                  carries queries into a latent space and latent outputs back to value space (attention_latent.cu).
//   gemm_grouped   rows sorted by group: rows offsets[g] … offsets[g+1]−1 of X [P][K] are multiplied by W[g]
//                  ([G][N][K]) into the same rows of Y [P][N].  `offsets` lives on the device (a router wrote it), so
//                  the grid is sized for the worst case, ceil(P / 64) + G row tiles, and a CTA finds its group and
//                  rows from `offsets` or leaves.
#include "common.cuh"

namespace {
constexpr int HBM = 64, HBN = 64, HBK = 16, HTM = 4, HTN = 4, HTHREADS = 256;

// one 64 × 64 tile of Y = X · Wᵀ; rows m0 … m_end−1 of X/Y (row strides ldx, ldy), columns n0 … of W [N][K]
template <typename IT, typename OT>
__device__ __forceinline__ void tile_product(const IT* __restrict__ X, const IT* __restrict__ W, OT* __restrict__ Y, int m0,
                                             int m_end, int n0, int N, int K, int ldx, int ldy, float (*As)[HBM + 4],
                                             float (*Bs)[HBN + 4], int act = VLRF_ACT_NONE) {
    const int tid = threadIdx.x;
    const int lr = tid >> 2, lk = (tid & 3) * 4;
    const int ty = tid >> 4, tx = tid & 15;
    float acc[HTM][HTN];
#pragma unroll
    for (int i = 0; i < HTM; ++i)
#pragma unroll
        for (int j = 0; j < HTN; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HBK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            const int gm = m0 + lr, gn = n0 + lr;
            As[lk + j][lr] = (gm < m_end && k < K) ? ElemIO<IT>::load(X + (size_t)gm * ldx + k) : 0.f;
            Bs[lk + j][lr] = (gn < N && k < K) ? ElemIO<IT>::load(W + (size_t)gn * K + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < HBK; ++k) {
            float a[HTM], b[HTN];
#pragma unroll
            for (int i = 0; i < HTM; ++i) a[i] = As[k][ty * HTM + i];
#pragma unroll
            for (int j = 0; j < HTN; ++j) b[j] = Bs[k][tx * HTN + j];
#pragma unroll
            for (int i = 0; i < HTM; ++i)
#pragma unroll
                for (int j = 0; j < HTN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < HTM; ++i) {
        const int m = m0 + ty * HTM + i;
        if (m >= m_end) continue;
#pragma unroll
        for (int j = 0; j < HTN; ++j) {
            const int n = n0 + tx * HTN + j;
            if (n < N) ElemIO<OT>::store(Y + (size_t)m * ldy + n, apply_act_rt(acc[i][j], act));
        }
    }
}

template <typename IT, typename OT>
__global__ void __launch_bounds__(HTHREADS)
gemm_heads_kernel(const IT* __restrict__ X, int ldx, int x_hs, const IT* __restrict__ W, OT* __restrict__ Y, int ldy,
                  int y_hs, int M, int N, int K) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    __shared__ float As[HBK][HBM + 4];
    __shared__ float Bs[HBK][HBN + 4];
    const int h = blockIdx.z;
    tile_product<IT, OT>(X + (size_t)h * x_hs, W + (size_t)h * N * K, Y + (size_t)h * y_hs, blockIdx.y * HBM, M,
                         blockIdx.x * HBN, N, K, ldx, ldy, As, Bs);
}

template <typename IT, typename OT>
__global__ void __launch_bounds__(HTHREADS)
gemm_grouped_kernel(const IT* __restrict__ X, const IT* __restrict__ W, OT* __restrict__ Y, const int* __restrict__ offsets,
                    int G, int N, int K, int act) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    __shared__ float As[HBK][HBM + 4];
    __shared__ float Bs[HBK][HBN + 4];
    __shared__ int where[3];                                   // group, first row, end of the group's rows
    if (threadIdx.x == 0) {
        int tile = blockIdx.y, g = 0, m0 = -1;
        for (; g < G; ++g) {
            const int lo = offsets[g], hi = offsets[g + 1];
            const int tiles = (hi - lo + HBM - 1) / HBM;
            if (tile < tiles) { m0 = lo + tile * HBM; where[2] = hi; break; }
            tile -= tiles;
        }
        where[0] = g; where[1] = m0;
    }
    __syncthreads();
    if (where[1] < 0) return;                                  // beyond the last group's tiles
    tile_product<IT, OT>(X, W + (size_t)where[0] * N * K, Y, where[1], where[2], blockIdx.x * HBN, N, K, K, N, As, Bs, act);
}
}  // namespace

extern "C" int vlrf_gemm_heads(const void* X, int ldx, int x_hs, const void* W, void* Y, int ldy, int y_hs, int M,
                               int N, int K, int H, int in_dtype, int out_dtype, cudaStream_t stream) {
    VLRF_REQUIRE(M >= 0 && N > 0 && K > 0 && H > 0, "gemm_heads: bad sizes M=%d N=%d K=%d H=%d", M, N, K, H);
    VLRF_REQUIRE(x_hs >= 0 && y_hs >= 0 && ldx >= (H - 1) * x_hs + K && ldy >= (H - 1) * y_hs + N, "gemm_heads: heads do not fit their rows");
    if (M == 0) return VLRF_OK;
    dim3 grid((N + HBN - 1) / HBN, (M + HBM - 1) / HBM, H);
    VLRF_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "gemm_heads: too many row tiles or heads");
#define LAUNCH(IT, OT) launch_chained(gemm_heads_kernel<IT, OT>, dim3(grid), dim3(HTHREADS), (size_t)(0), stream, (const IT*)X, ldx, x_hs, (const IT*)W, (OT*)Y, ldy, y_hs, M, N, K)
    if (in_dtype == VLRF_F32 && out_dtype == VLRF_F32) LAUNCH(float, float);
    else if (in_dtype == VLRF_BF16 && out_dtype == VLRF_F32) LAUNCH(__nv_bfloat16, float);
    else if (in_dtype == VLRF_BF16 && out_dtype == VLRF_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return vlrf_fail(VLRF_ERR_INVALID_ARG, "gemm_heads: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
#undef LAUNCH
    return vlrf_check_launch("gemm_heads");
}

extern "C" int vlrf_gemm_grouped(const void* X, const void* W, void* Y, const int* offsets, int G, int P, int N, int K,
                                 int in_dtype, int out_dtype, int act, cudaStream_t stream) {
    VLRF_REQUIRE(act >= 0 && act <= VLRF_ACT_LAST_FUSED, "gemm_grouped: activation %d is not taken", act);
    VLRF_REQUIRE(P >= 0 && N > 0 && K > 0 && G > 0 && offsets != nullptr, "gemm_grouped: bad sizes P=%d N=%d K=%d G=%d", P, N, K, G);
    if (P == 0) return VLRF_OK;
    dim3 grid((N + HBN - 1) / HBN, (P + HBM - 1) / HBM + G);
    VLRF_REQUIRE(grid.y <= 65535, "gemm_grouped: too many row tiles");
#define LAUNCH(IT, OT) launch_chained(gemm_grouped_kernel<IT, OT>, dim3(grid), dim3(HTHREADS), (size_t)(0), stream, (const IT*)X, (const IT*)W, (OT*)Y, offsets, G, N, K, act)
    if (in_dtype == VLRF_F32 && out_dtype == VLRF_F32) LAUNCH(float, float);
    else if (in_dtype == VLRF_BF16 && out_dtype == VLRF_F32) LAUNCH(__nv_bfloat16, float);
    else if (in_dtype == VLRF_BF16 && out_dtype == VLRF_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return vlrf_fail(VLRF_ERR_INVALID_ARG, "gemm_grouped: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
#undef LAUNCH
    return vlrf_check_launch("gemm_grouped");
}
