// A residual carried in several streams, and the small row-wise kernels of models that use one.
//
// The residual of a token is S rows of d float32 numbers, [T][S][d].  A sublayer reads one row, a weighted sum of the
// streams, through its norm; its result y is then written back into every stream together with a mix of the old
// streams:
//     read:   u = Σ_s a[s] · x[s]            h = u / sqrt(mean(u²) + eps) · w        (one kernel, sums in float32)
//     write:  x'[j] = Σ_s m[s][j] · x[s] + b[j] · y      for every j at once, from the old streams
// With a = null every coefficient is 1 (the sum of the streams: what the model's last norm reads), and `rows` gathers
// the tokens whose logits are wanted.  S = 1 with a = null is the plain RMS norm of a row.
//
// A write that is followed by the next sublayer's read is one kernel (write_read): one pass over the streams.
//
// embed_streams: x[t][s] = table[token[t]] · scale for every stream s (scale 1 and one stream: a plain lookup).
// embed_bigram: x[t] = table[token[t]] · scale + pairs[row], one stream; row = (token before · mul_prev + token · mul_cur)
//   mod buckets, and row `buckets` (the table's last) for a sequence's first token.  The token before is the row above
//   where the step brings it, else the sequence's kept token: an int32 state [slot][2] holds each sequence's last token
//   twice, a step reading the copy of the parity of the position it begins at and writing the copy of the parity of the
//   position it ends at, so a step of one token leaves what it read and may run twice.  The CTA of a sequence's first
//   token of the step also keeps the sequence's last token of the step, after its own read of the kept one.
// softcap: v ← cap · tanh(v / cap) over float32 rows (logits).  scale_values: v ← v · factor.
#include "common.cuh"

namespace {
constexpr int ST_THREADS = 128;
constexpr int ST_MAX_STREAMS = 16;

template <typename WT>
__global__ void __launch_bounds__(ST_THREADS)
embed_streams_kernel(const WT* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ x, int d, int V,
                     int S, float scale, int* __restrict__ dev_err) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    int id = tokens[t];
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) atomicOr(dev_err, VLRF_DEVERR_TOKEN_RANGE);
        id = min(max(id, 0), V - 1);
    }
    const WT* row = table + (size_t)id * d;
    float* out = x + (size_t)t * S * d;
    for (int i = threadIdx.x; i < d; i += ST_THREADS) {
        const float v = ElemIO<WT>::load(row + i) * scale;
        for (int s = 0; s < S; ++s) out[(size_t)s * d + i] = v;
    }
}

template <typename WT>
__global__ void __launch_bounds__(ST_THREADS)
embed_bigram_kernel(const WT* __restrict__ table, const WT* __restrict__ pairs, const int* __restrict__ tokens,
                    const int* __restrict__ tok_slot, const int* __restrict__ tok_pos, const int* __restrict__ seq_start, int n_seqs,
                    int* __restrict__ kept, float* __restrict__ x, int T, int d, int V, int buckets, int mul_prev, int mul_cur,
                    float scale, __nv_bfloat16* __restrict__ also, int* __restrict__ dev_err) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ int row_sm;
    const int t = blockIdx.x;
    const int slot = tok_slot[t];
    if (slot < 0) return;                     // padding row (the whole CTA leaves)
    int id = tokens[t];
    if (id < 0 || id >= V) {
        if (threadIdx.x == 0) atomicOr(dev_err, VLRF_DEVERR_TOKEN_RANGE);
        id = min(max(id, 0), V - 1);
    }
    if (threadIdx.x == 0) {
        const int pos = tok_pos[t];
        const bool above = t > 0 && tok_slot[t - 1] == slot && tok_pos[t - 1] == pos - 1;   // the step brings the token before
        int prev = -1;
        if (above) prev = tokens[t - 1];
        else {
            if (pos > 0) prev = kept[(size_t)slot * 2 + (pos & 1)];
            // this row begins its sequence's tokens of the step: find where they end and keep the last one
            int lo = 0, hi = n_seqs - 1;
            while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (seq_start[mid] <= t) lo = mid; else hi = mid - 1; }
            const int last = seq_start[lo + 1] - 1;
            if (last >= t && last < T) kept[(size_t)slot * 2 + ((pos + (last - t) + 1) & 1)] = tokens[last];
        }
        int row = buckets;
        if (pos > 0) {
            prev = min(max(prev, 0), V - 1);
            row = (int)(((long long)prev * mul_prev + (long long)id * mul_cur) % buckets);
            if (row < 0) row += buckets;
        }
        row_sm = row;
    }
    __syncthreads();
    const WT* er = table + (size_t)id * d;
    const WT* br = pairs + (size_t)row_sm * d;
    float* out = x + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += ST_THREADS) {
        const float v = fmaf(ElemIO<WT>::load(er + i), scale, ElemIO<WT>::load(br + i));
        out[i] = v;
        if (also != nullptr) also[(size_t)t * d + i] = __float2bfloat16_rn(v);     // what the first sublayer reads of the row
    }
}

__global__ void scale_values_kernel(float* __restrict__ v, long long n, float factor) {
    pdl_wait();
    pdl_launch_dependents();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) v[i] *= factor;
}

template <typename OT>
__global__ void __launch_bounds__(ST_THREADS)
streams_read_norm_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ a,
                         const float* __restrict__ w, OT* __restrict__ out, int d, int S, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float u_sm[];          // [d]
    __shared__ float red[ST_THREADS / 32];
    __shared__ float coef[ST_MAX_STREAMS];
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * S * d;
    if (threadIdx.x < S) coef[threadIdx.x] = a ? a[threadIdx.x] : 1.f;
    __syncthreads();
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += ST_THREADS) {
        float u = 0.f;
        for (int s = 0; s < S; ++s) u = fmaf(coef[s], xr[(size_t)s * d + i], u);
        u_sm[i] = u;
        ss = fmaf(u, u, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < ST_THREADS / 32; ++i) total += red[i];
    const float inv = 1.f / sqrtf(total / (float)d + eps);
    OT* o = out + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += ST_THREADS) ElemIO<OT>::store(o + i, u_sm[i] * inv * w[i]);
}

template <int SMAX>
__global__ void __launch_bounds__(ST_THREADS)
streams_write_kernel(float* __restrict__ x, const float* __restrict__ mix, const float* __restrict__ b,
                     const float* __restrict__ y, int d, int S) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float m_sm[ST_MAX_STREAMS * ST_MAX_STREAMS];
    __shared__ float b_sm[ST_MAX_STREAMS];
    for (int i = threadIdx.x; i < S * S; i += ST_THREADS) m_sm[i] = mix[i];
    if (threadIdx.x < S) b_sm[threadIdx.x] = b[threadIdx.x];
    __syncthreads();
    const int t = blockIdx.x;
    float* xr = x + (size_t)t * S * d;
    const float* yr = y + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += ST_THREADS) {
        float old[SMAX];
#pragma unroll
        for (int s = 0; s < SMAX; ++s) old[s] = s < S ? xr[(size_t)s * d + i] : 0.f;
        const float yv = yr[i];
#pragma unroll
        for (int j = 0; j < SMAX; ++j) {
            if (j < S) {
                float v = b_sm[j] * yv;
#pragma unroll
                for (int s = 0; s < SMAX; ++s)
                    if (s < S) v = fmaf(m_sm[s * S + j], old[s], v);
                xr[(size_t)j * d + i] = v;
            }
        }
    }
}

// The write of one sublayer and the read of the next in one pass over the streams: x' as in the write kernel, then
// h = RMSnorm(Σ_j a[j] · x'[j]) · w.  The row's u stays in shared memory between the two.
template <int SMAX, typename OT>
__global__ void __launch_bounds__(ST_THREADS)
streams_write_read_kernel(float* __restrict__ x, const float* __restrict__ mix, const float* __restrict__ b,
                          const float* __restrict__ y, const float* __restrict__ a, const float* __restrict__ w,
                          OT* __restrict__ out, int d, int S, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float u_sm[];          // [d]
    __shared__ float m_sm[ST_MAX_STREAMS * ST_MAX_STREAMS];
    __shared__ float b_sm[ST_MAX_STREAMS], a_sm[ST_MAX_STREAMS];
    __shared__ float red[ST_THREADS / 32];
    for (int i = threadIdx.x; i < S * S; i += ST_THREADS) m_sm[i] = mix[i];
    if (threadIdx.x < S) { b_sm[threadIdx.x] = b[threadIdx.x]; a_sm[threadIdx.x] = a[threadIdx.x]; }
    __syncthreads();
    const int t = blockIdx.x;
    float* xr = x + (size_t)t * S * d;
    const float* yr = y + (size_t)t * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += ST_THREADS) {
        float old[SMAX];
#pragma unroll
        for (int s = 0; s < SMAX; ++s) old[s] = s < S ? xr[(size_t)s * d + i] : 0.f;
        const float yv = yr[i];
        float u = 0.f;
#pragma unroll
        for (int j = 0; j < SMAX; ++j) {
            if (j < S) {
                float v = b_sm[j] * yv;
#pragma unroll
                for (int s = 0; s < SMAX; ++s)
                    if (s < S) v = fmaf(m_sm[s * S + j], old[s], v);
                xr[(size_t)j * d + i] = v;
                u = fmaf(a_sm[j], v, u);
            }
        }
        u_sm[i] = u;
        ss = fmaf(u, u, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int i = 0; i < ST_THREADS / 32; ++i) total += red[i];
    const float inv = 1.f / sqrtf(total / (float)d + eps);
    OT* o = out + (size_t)t * d;
    for (int i = threadIdx.x; i < d; i += ST_THREADS) ElemIO<OT>::store(o + i, u_sm[i] * inv * w[i]);
}

__global__ void softcap_kernel(float* __restrict__ v, long long n, float cap) {
    pdl_wait();
    pdl_launch_dependents();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) v[i] = cap * tanhf(v[i] / cap);
}
}  // namespace

extern "C" int vlrf_embed_streams(const void* table, int w_dtype, const int* tokens, float* x, int T, int d, int V, int S,
                                  float scale, int* dev_err, cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && d > 0 && V > 0 && S > 0, "embed_streams: bad sizes");
    VLRF_REQUIRE(dev_err != nullptr, "embed_streams: needs the device error word");
    if (T == 0) return VLRF_OK;
    if (w_dtype == VLRF_F32)
        launch_chained(embed_streams_kernel<float>, dim3(T), dim3(ST_THREADS), (size_t)0, stream, (const float*)table, tokens, x, d, V, S,
                       scale, dev_err);
    else if (w_dtype == VLRF_BF16)
        launch_chained(embed_streams_kernel<__nv_bfloat16>, dim3(T), dim3(ST_THREADS), (size_t)0, stream, (const __nv_bfloat16*)table,
                       tokens, x, d, V, S, scale, dev_err);
    else
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "embed_streams: unknown dtype %d", w_dtype);
    return vlrf_check_launch("embed_streams");
}

extern "C" int vlrf_streams_read_norm(const float* x, const int* rows, const float* a, const float* w, void* out, int out_dtype,
                                      int n_rows, int d, int S, float eps, cudaStream_t stream) {
    VLRF_REQUIRE(n_rows >= 0 && d > 0 && S > 0 && S <= ST_MAX_STREAMS, "streams_read_norm: bad sizes rows=%d d=%d streams=%d", n_rows, d, S);
    VLRF_REQUIRE((size_t)d * sizeof(float) <= 160 * 1024, "streams_read_norm: a row of %d numbers does not fit shared memory", d);
    if (n_rows == 0) return VLRF_OK;
    const size_t smem = (size_t)d * sizeof(float);
    if (out_dtype == VLRF_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(streams_read_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_chained(streams_read_norm_kernel<float>, dim3(n_rows), dim3(ST_THREADS), smem, stream, x, rows, a, w, (float*)out, d, S, eps);
    } else if (out_dtype == VLRF_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(streams_read_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_chained(streams_read_norm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(ST_THREADS), smem, stream, x, rows, a, w,
                       (__nv_bfloat16*)out, d, S, eps);
    } else {
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "streams_read_norm: unknown output dtype %d", out_dtype);
    }
    return vlrf_check_launch("streams_read_norm");
}

extern "C" int vlrf_streams_write(float* x, const float* mix, const float* b, const float* y, int T, int d, int S,
                                  cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && d > 0 && S > 0 && S <= ST_MAX_STREAMS, "streams_write: bad sizes rows=%d d=%d streams=%d", T, d, S);
    if (T == 0) return VLRF_OK;
    // (the streams of a column are held in registers: the kernel is instantiated for up to 2, 4, 8 and 16 of them)
    if (S <= 2) launch_chained(streams_write_kernel<2>, dim3(T), dim3(ST_THREADS), (size_t)0, stream, x, mix, b, y, d, S);
    else if (S <= 4) launch_chained(streams_write_kernel<4>, dim3(T), dim3(ST_THREADS), (size_t)0, stream, x, mix, b, y, d, S);
    else if (S <= 8) launch_chained(streams_write_kernel<8>, dim3(T), dim3(ST_THREADS), (size_t)0, stream, x, mix, b, y, d, S);
    else launch_chained(streams_write_kernel<16>, dim3(T), dim3(ST_THREADS), (size_t)0, stream, x, mix, b, y, d, S);
    return vlrf_check_launch("streams_write");
}

extern "C" int vlrf_streams_write_read(float* x, const float* mix, const float* b, const float* y, const float* a, const float* w,
                                       void* out, int out_dtype, int T, int d, int S, float eps, cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && d > 0 && S > 0 && S <= ST_MAX_STREAMS, "streams_write_read: bad sizes rows=%d d=%d streams=%d", T, d, S);
    VLRF_REQUIRE((size_t)d * sizeof(float) <= 160 * 1024, "streams_write_read: a row of %d numbers does not fit shared memory", d);
    VLRF_REQUIRE(out_dtype == VLRF_F32 || out_dtype == VLRF_BF16, "streams_write_read: unknown output dtype %d", out_dtype);
    VLRF_REQUIRE(a != nullptr, "streams_write_read: the read needs its coefficients");
    if (T == 0) return VLRF_OK;
    const size_t smem = (size_t)d * sizeof(float);
#define GO(M, OT) do { if (smem > 48 * 1024) cudaFuncSetAttribute(streams_write_read_kernel<M, OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_chained(streams_write_read_kernel<M, OT>, dim3(T), dim3(ST_THREADS), smem, stream, x, mix, b, y, a, w, (OT*)out, d, S, eps); } while (0)
#define GO_S(OT) do { if (S <= 2) GO(2, OT); else if (S <= 4) GO(4, OT); else if (S <= 8) GO(8, OT); else GO(16, OT); } while (0)
    if (out_dtype == VLRF_F32) GO_S(float); else GO_S(__nv_bfloat16);
#undef GO_S
#undef GO
    return vlrf_check_launch("streams_write_read");
}

extern "C" int vlrf_embed_bigram(const void* table, const void* pairs, int w_dtype, const int* tokens, const int* tok_slot,
                                 const int* tok_pos, const int* seq_start, int n_seqs, int* kept, float* x, int T, int d, int V,
                                 int buckets, int mul_prev, int mul_cur, float scale, void* also, int* dev_err, cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && d > 0 && V > 0 && buckets > 0 && n_seqs >= 0, "embed_bigram: bad sizes");
    VLRF_REQUIRE(dev_err != nullptr && kept != nullptr && seq_start != nullptr, "embed_bigram: needs the error word, the kept tokens and the sequences' rows");
    if (T == 0 || n_seqs == 0) return VLRF_OK;
    if (w_dtype == VLRF_F32)
        launch_chained(embed_bigram_kernel<float>, dim3(T), dim3(ST_THREADS), (size_t)0, stream, (const float*)table, (const float*)pairs,
                       tokens, tok_slot, tok_pos, seq_start, n_seqs, kept, x, T, d, V, buckets, mul_prev, mul_cur, scale, (__nv_bfloat16*)also,
                       dev_err);
    else if (w_dtype == VLRF_BF16)
        launch_chained(embed_bigram_kernel<__nv_bfloat16>, dim3(T), dim3(ST_THREADS), (size_t)0, stream, (const __nv_bfloat16*)table,
                       (const __nv_bfloat16*)pairs, tokens, tok_slot, tok_pos, seq_start, n_seqs, kept, x, T, d, V, buckets, mul_prev,
                       mul_cur, scale, (__nv_bfloat16*)also, dev_err);
    else
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "embed_bigram: unknown dtype %d", w_dtype);
    return vlrf_check_launch("embed_bigram");
}

extern "C" int vlrf_scale_values(float* v, long long n, float factor, cudaStream_t stream) {
    VLRF_REQUIRE(n >= 0, "scale_values: bad size");
    if (n == 0) return VLRF_OK;
    launch_chained(scale_values_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), (size_t)0, stream, v, n, factor);
    return vlrf_check_launch("scale_values");
}

extern "C" int vlrf_softcap(float* v, long long n, float cap, cudaStream_t stream) {
    VLRF_REQUIRE(n >= 0 && cap > 0.f, "softcap: bad sizes or a cap that is not positive");
    if (n == 0) return VLRF_OK;
    launch_chained(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), (size_t)0, stream, v, n, cap);
    return vlrf_check_launch("softcap");
}
