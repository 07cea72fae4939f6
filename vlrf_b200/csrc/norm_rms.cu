// RMS norm in groups, and the small row-wise kernels around it.
//
// group_rmsnorm: a row of d columns is cut into `groups` equal consecutive parts; each part is divided by
// sqrt(mean(part²) + eps) of its own, and the whole row is multiplied by a weight vector.  groups = 1 is the plain
// RMS norm.  The input rows are float32 (a product's float32 result, or the residual stream); sums and the division
// are float32.  The result either replaces the output row (any dtype) or is added to it (float32: the residual
// stream, for blocks that norm a sublayer's output before the sum).  `rows` gathers input rows (the rows whose
// logits are wanted).  The output may be the input: a thread rewrites only elements it has read itself.  `also`: a
// second, bfloat16 copy of the finished rows [n_rows][d], which spares the cast of the residual stream that the next
// sublayer would need.
//
// cast_rows: float32 rows to the activation dtype (what a sublayer reads of the float32 residual stream).
// gate_mul: out = act(a) · b element by element (act: x·sigmoid(x) or max(x, 0) for gated feed-forwards, sigmoid(x) for
// gates on an attention's merged heads), float32 arithmetic.  gate_mul_groups: one column of a for every `per`
// consecutive columns of b (a gate per head on the merged heads).
//
// rmsnorm_shift: the plain RMS norm of a token's residual row followed by a token shift: with n_t the normed row,
// out_t = n_t + (n_(t−1) − n_t) · mu element by element, n_(t−1) being the normed row of the sequence's token before
// (zeros ahead of the first).  The token before is the row above where the step brings it, else the sequence's kept
// row: a float32 state [slot][2][d] holds the normed row of each sequence's last token twice, a step reading the copy
// of the parity of the position it begins at and writing the copy of the parity of the position it ends at, so a step
// of one token leaves what it read and may run twice.  The warp of a sequence's first token of the step also norms the
// sequence's last row of the step and keeps it, each lane after its own read of the kept row.
//
// add_row_vector: x[t] += v for every row (a vector that a model adds to the residual between layers).
#include "common.cuh"

namespace {
__device__ __forceinline__ float gate_f(int act, float g) {
    return act == VLRF_ACT_SILU ? silu_f(g) : act == VLRF_ACT_SIGMOID ? sigmoid_f(g) : act == VLRF_ACT_GELU_TANH ? gelu_tanh_f(g) : fmaxf(g, 0.f);
}

// A gate with bounds: g' = min(g, limit), u' = clamp(u, −limit, limit), out = g' · sigmoid(alpha · g') · (u' + 1).
template <typename AT, typename BT, typename OT>
__global__ void gate_mul_clamped_kernel(const AT* a, int lda, const BT* b, int ldb, OT* out, int ldo, int rows, int cols, float limit,
                                        float alpha) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * cols) return;
    const int r = (int)(i / cols), c = (int)(i - (long long)r * cols);
    const float g = fminf(ElemIO<AT>::load(a + (size_t)r * lda + c), limit);
    const float u = fminf(fmaxf(ElemIO<BT>::load(b + (size_t)r * ldb + c), -limit), limit);
    ElemIO<OT>::store(out + (size_t)r * ldo + c, g * sigmoid_f(alpha * g) * (u + 1.f));
}

// the same, eight bfloat16 a thread (rows and columns on 16-byte boundaries)
__global__ void gate_mul_clamped_bf16x8_kernel(const __nv_bfloat16* a, int lda, const __nv_bfloat16* b, int ldb, __nv_bfloat16* out,
                                               int ldo, int rows, int cols8, float limit, float alpha) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * cols8) return;
    const int r = (int)(i / cols8), c = (int)(i - (long long)r * cols8) * 8;
    const uint4 ga = *reinterpret_cast<const uint4*>(a + (size_t)r * lda + c), va = *reinterpret_cast<const uint4*>(b + (size_t)r * ldb + c);
    const uint32_t gw[4] = {ga.x, ga.y, ga.z, ga.w}, vw[4] = {va.x, va.y, va.z, va.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float g0 = fminf(__uint_as_float(gw[k] << 16), limit), g1 = fminf(__uint_as_float(gw[k] & 0xffff0000u), limit);
        const float v0 = fminf(fmaxf(__uint_as_float(vw[k] << 16), -limit), limit), v1 = fminf(fmaxf(__uint_as_float(vw[k] & 0xffff0000u), -limit), limit);
        const __nv_bfloat162 p = __floats2bfloat162_rn(g0 * sigmoid_f(alpha * g0) * (v0 + 1.f), g1 * sigmoid_f(alpha * g1) * (v1 + 1.f));
        o[k] = *reinterpret_cast<const uint32_t*>(&p);
    }
    *reinterpret_cast<uint4*>(out + (size_t)r * ldo + c) = make_uint4(o[0], o[1], o[2], o[3]);
}
constexpr int NORM_THREADS = 128;
constexpr int NORM_MAX_GROUPS = 1024;

template <typename OT, bool ACC>
__global__ void __launch_bounds__(NORM_THREADS)
group_rmsnorm_kernel(const float* y, int ld_y, const int* __restrict__ rows, const float* __restrict__ w, OT* out,
                     int ld_out, int d, int groups, float eps, __nv_bfloat16* also) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    __shared__ float inv_sm[NORM_MAX_GROUPS];
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    const float* yr = y + (size_t)src * ld_y;
    const int gs = d / groups;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int g = warp; g < groups; g += NORM_THREADS / 32) {
        float s = 0.f;
        for (int i = lane; i < gs; i += 32) { const float v = yr[g * gs + i]; s = fmaf(v, v, s); }
        s = warp_sum(s);
        if (lane == 0) inv_sm[g] = 1.f / sqrtf(s / (float)gs + eps);
    }
    __syncthreads();
    OT* o = out + (size_t)r * ld_out;
    for (int i = threadIdx.x; i < d; i += NORM_THREADS) {
        float v = yr[i] * inv_sm[i / gs] * w[i];
        if (ACC) v += ElemIO<OT>::load(o + i);
        ElemIO<OT>::store(o + i, v);
        if (also != nullptr) also[(size_t)r * d + i] = __float2bfloat16_rn(v);     // what the next sublayer reads of the row
    }
}

template <typename OT>
__global__ void cast_rows_kernel(const float* __restrict__ x, OT* __restrict__ out, long long n) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        const float4 v = *reinterpret_cast<const float4*>(x + i);
        ElemIO<OT>::store(out + i, v.x); ElemIO<OT>::store(out + i + 1, v.y);
        ElemIO<OT>::store(out + i + 2, v.z); ElemIO<OT>::store(out + i + 3, v.w);
    } else {
        for (long long j = i; j < n; ++j) ElemIO<OT>::store(out + j, x[j]);
    }
}

// the same, eight bfloat16 a thread (rows and columns on 16-byte boundaries)
__global__ void gate_mul_bf16x8_kernel(const __nv_bfloat16* a, int lda, const __nv_bfloat16* b, int ldb, __nv_bfloat16* out, int ldo,
                                       int rows, int cols8, int act) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * cols8) return;
    const int r = (int)(i / cols8), c = (int)(i - (long long)r * cols8) * 8;
    const uint4 ga = *reinterpret_cast<const uint4*>(a + (size_t)r * lda + c), va = *reinterpret_cast<const uint4*>(b + (size_t)r * ldb + c);
    const uint32_t gw[4] = {ga.x, ga.y, ga.z, ga.w}, vw[4] = {va.x, va.y, va.z, va.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float g0 = __uint_as_float(gw[k] << 16), g1 = __uint_as_float(gw[k] & 0xffff0000u);
        const float v0 = __uint_as_float(vw[k] << 16), v1 = __uint_as_float(vw[k] & 0xffff0000u);
        const float f0 = gate_f(act, g0), f1 = gate_f(act, g1);
        const __nv_bfloat162 p = __floats2bfloat162_rn(f0 * v0, f1 * v1);
        o[k] = *reinterpret_cast<const uint32_t*>(&p);
    }
    *reinterpret_cast<uint4*>(out + (size_t)r * ldo + c) = make_uint4(o[0], o[1], o[2], o[3]);
}

// float32 gate and value, bfloat16 result, four a thread (rows and columns on 16-byte boundaries)
__global__ void gate_mul_f32x4_kernel(const float* a, int lda, const float* b, int ldb, __nv_bfloat16* out, int ldo, int rows, int cols4,
                                      int act) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * cols4) return;
    const int r = (int)(i / cols4), c = (int)(i - (long long)r * cols4) * 4;
    const float4 g = *reinterpret_cast<const float4*>(a + (size_t)r * lda + c), v = *reinterpret_cast<const float4*>(b + (size_t)r * ldb + c);
    const __nv_bfloat162 lo = __floats2bfloat162_rn(gate_f(act, g.x) * v.x, gate_f(act, g.y) * v.y);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(gate_f(act, g.z) * v.z, gate_f(act, g.w) * v.w);
    *reinterpret_cast<uint2*>(out + (size_t)r * ldo + c) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

// a float32 gate logit per group of `per` columns (per a multiple of 8), bfloat16 values and result, eight a thread
__global__ void gate_mul_groups_bf16x8_kernel(const float* a, int lda, const __nv_bfloat16* b, int ldb, __nv_bfloat16* out, int ldo,
                                              int rows, int cols8, int per8, int act) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * cols8) return;
    const int r = (int)(i / cols8), c8 = (int)(i - (long long)r * cols8);
    const float f = gate_f(act, a[(size_t)r * lda + c8 / per8]);
    const uint4 va = *reinterpret_cast<const uint4*>(b + (size_t)r * ldb + c8 * 8);
    const uint32_t vw[4] = {va.x, va.y, va.z, va.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float v0 = __uint_as_float(vw[k] << 16), v1 = __uint_as_float(vw[k] & 0xffff0000u);
        const __nv_bfloat162 p = __floats2bfloat162_rn(f * v0, f * v1);
        o[k] = *reinterpret_cast<const uint32_t*>(&p);
    }
    *reinterpret_cast<uint4*>(out + (size_t)r * ldo + c8 * 8) = make_uint4(o[0], o[1], o[2], o[3]);
}

template <typename AT, typename BT, typename OT>
__global__ void gate_mul_kernel(const AT* a, int lda, const BT* b, int ldb, OT* out, int ldo, int rows, int cols, int act, int per) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * cols) return;
    const int r = (int)(i / cols), c = (int)(i - (long long)r * cols);
    const float g = ElemIO<AT>::load(a + (size_t)r * lda + c / per);
    const float v = ElemIO<BT>::load(b + (size_t)r * ldb + c);
    const float f = gate_f(act, g);
    ElemIO<OT>::store(out + (size_t)r * ldo + c, f * v);
}

// rmsnorm_shift: a warp per token.  The warp sums the squares of its row, of the row above where that is the token before,
// and (for a sequence's first row of the step) of the sequence's last row of the step, with shuffles only; the second
// pass finds the rows in L1.  VEC: rows and outputs on 16-byte boundaries and d a multiple of 4, four values a lane.
constexpr int SHIFT_WARPS = 4;

template <bool VEC>
__device__ __forceinline__ float warp_inv_rms(const float* __restrict__ row, int d, float eps, int lane) {
    float s = 0.f;
    if (VEC) {
        for (int i = lane * 4; i < d; i += 128) {
            const float4 v = *reinterpret_cast<const float4*>(row + i);
            s = fmaf(v.x, v.x, s); s = fmaf(v.y, v.y, s); s = fmaf(v.z, v.z, s); s = fmaf(v.w, v.w, s);
        }
    } else {
        for (int i = lane; i < d; i += 32) { const float v = row[i]; s = fmaf(v, v, s); }
    }
    s = warp_sum(s);
    return 1.f / sqrtf(s / (float)d + eps);
}

template <typename OT> __device__ __forceinline__ void store4(OT* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

template <typename OT, bool VEC>
__global__ void __launch_bounds__(SHIFT_WARPS * 32)
rmsnorm_shift_kernel(const float* __restrict__ x, int ld_x, const float* __restrict__ w, const float* __restrict__ mu, float eps,
                     float* state, const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                     const int* __restrict__ seq_start, int n_seqs, int T, OT* __restrict__ out, int ld_out, int d) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * SHIFT_WARPS + (threadIdx.x >> 5);
    if (t >= T) return;                                        // (whole warps leave; no block-wide barrier below)
    const int slot = tok_slot[t];
    OT* o = out + (size_t)t * ld_out;
    if (slot < 0) {                                            // padding row
        for (int i = lane; i < d; i += 32) ElemIO<OT>::store(o + i, 0.f);
        return;
    }
    const int pos = tok_pos[t];
    const bool row_above = t > 0 && tok_slot[t - 1] == slot;   // the token before came with this step
    const float* xr = x + (size_t)t * ld_x;
    const float inv = warp_inv_rms<VEC>(xr, d, eps, lane);
    // where the token before lies: a row of x (normed here once more), the kept row, or nowhere (position 0)
    const float* prev = row_above ? xr - ld_x : (pos > 0 ? state + ((size_t)slot * 2 + (pos & 1)) * d : nullptr);
    const float inv_prev = row_above ? warp_inv_rms<VEC>(prev, d, eps, lane) : 1.f;
    // the row that the sequence keeps: that of its last token of this step, normed by the warp of its first
    const float* last = nullptr;
    float inv_last = 0.f;
    float* keep = nullptr;
    if (!row_above) {
        int lo = 0, hi = n_seqs;                               // the sequence that begins at row t
        while (lo < hi) { const int mid = (lo + hi) >> 1; if (seq_start[mid] < t) lo = mid + 1; else hi = mid; }
        const int end = (lo < n_seqs && seq_start[lo] == t) ? seq_start[lo + 1] : t + 1;
        const int n = min(end, T) - t;
        last = xr + (size_t)(n - 1) * ld_x;
        inv_last = n > 1 ? warp_inv_rms<VEC>(last, d, eps, lane) : inv;
        keep = state + ((size_t)slot * 2 + ((pos + n) & 1)) * d;
    }
    if (VEC) {
        for (int i = lane * 4; i < d; i += 128) {
            const float4 g = *reinterpret_cast<const float4*>(w + i), m = *reinterpret_cast<const float4*>(mu + i);
            const float4 v = *reinterpret_cast<const float4*>(xr + i);
            float4 pv = make_float4(0.f, 0.f, 0.f, 0.f);
            if (prev != nullptr) pv = *reinterpret_cast<const float4*>(prev + i);
            const float pg = row_above ? inv_prev : 1.f;       // (the kept row is normed already)
            const float n0 = v.x * inv * g.x, n1 = v.y * inv * g.y, n2 = v.z * inv * g.z, n3 = v.w * inv * g.w;
            const float p0 = row_above ? pv.x * pg * g.x : pv.x, p1 = row_above ? pv.y * pg * g.y : pv.y;
            const float p2 = row_above ? pv.z * pg * g.z : pv.z, p3 = row_above ? pv.w * pg * g.w : pv.w;
            store4<OT>(o + i, n0 + (p0 - n0) * m.x, n1 + (p1 - n1) * m.y, n2 + (p2 - n2) * m.z, n3 + (p3 - n3) * m.w);
            if (keep != nullptr) {                             // (after this lane's read of the kept row)
                const float4 l = *reinterpret_cast<const float4*>(last + i);
                *reinterpret_cast<float4*>(keep + i) = make_float4(l.x * inv_last * g.x, l.y * inv_last * g.y, l.z * inv_last * g.z, l.w * inv_last * g.w);
            }
        }
    } else {
        for (int i = lane; i < d; i += 32) {
            const float g = w[i];
            const float n_t = xr[i] * inv * g;
            float n_prev = 0.f;
            if (prev != nullptr) n_prev = row_above ? prev[i] * inv_prev * g : prev[i];
            ElemIO<OT>::store(o + i, n_t + (n_prev - n_t) * mu[i]);
            if (keep != nullptr) keep[i] = last[i] * inv_last * g;   // (after this lane's read of the kept row)
        }
    }
}

// rmsnorm_shift with a CTA per token, for rows on 16-byte boundaries: a thread holds NV groups of four columns of its
// row and of the row before in registers (both asked for at once), the two sums of squares are reduced together, and
// nothing is read twice.  The CTA of a sequence's first token of the step also norms and keeps the sequence's last row.
constexpr int SHIFT_ROW_MAX_NV = 4, SHIFT_ROW_MAX_THREADS = 512;     // rows of up to 8192 columns; wider ones a warp a token

template <typename OT, int NV>
__global__ void __launch_bounds__(NV == SHIFT_ROW_MAX_NV ? SHIFT_ROW_MAX_THREADS : 128)
rmsnorm_shift_rows_kernel(const float* __restrict__ x, int ld_x, const float* __restrict__ w, const float* __restrict__ mu, float eps,
                          float* state, const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                          const int* __restrict__ seq_start, int n_seqs, int T, OT* __restrict__ out, int ld_out, int d) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    __shared__ float part[3][32];
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int slot = tok_slot[t];
    OT* o = out + (size_t)t * ld_out;
    if (slot < 0) {                                            // padding row (the whole CTA)
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int i = 4 * (threadIdx.x + k * blockDim.x);
            if (i < d) store4<OT>(o + i, 0.f, 0.f, 0.f, 0.f);
        }
        return;
    }
    const int pos = tok_pos[t];
    const bool row_above = t > 0 && tok_slot[t - 1] == slot;   // the token before came with this step
    const float* xr = x + (size_t)t * ld_x;
    // where the token before lies: a row of x (normed here once more), the kept row, or nowhere (position 0)
    const float* prev = row_above ? xr - ld_x : (pos > 0 ? state + ((size_t)slot * 2 + (pos & 1)) * d : nullptr);
    // the row that the sequence keeps: that of its last token of this step, normed by the CTA of its first
    const float* last = nullptr;
    float* keep = nullptr;
    if (!row_above) {
        int lo = 0, hi = n_seqs;                               // the sequence whose rows begin at t
        while (lo < hi) { const int mid = (lo + hi) >> 1; if (seq_start[mid] < t) lo = mid + 1; else hi = mid; }
        const int end = (lo < n_seqs && seq_start[lo] == t) ? seq_start[lo + 1] : t + 1;
        const int n = min(end, T) - t;
        if (n > 1) last = xr + (size_t)(n - 1) * ld_x;         // (one token: the row in registers is the last)
        keep = state + ((size_t)slot * 2 + ((pos + n) & 1)) * d;
    }
    float4 v[NV], pv[NV];
    float s_own = 0.f, s_prev = 0.f, s_last = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = 4 * (threadIdx.x + k * blockDim.x);
        const bool in = i < d;
        v[k] = in ? *reinterpret_cast<const float4*>(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        pv[k] = (in && prev != nullptr) ? *reinterpret_cast<const float4*>(prev + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (in && last != nullptr) {                           // (read again below: one CTA a sequence comes here)
            const float4 l = *reinterpret_cast<const float4*>(last + i);
            s_last = fmaf(l.x, l.x, s_last); s_last = fmaf(l.y, l.y, s_last); s_last = fmaf(l.z, l.z, s_last); s_last = fmaf(l.w, l.w, s_last);
        }
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        s_own = fmaf(v[k].x, v[k].x, s_own); s_own = fmaf(v[k].y, v[k].y, s_own); s_own = fmaf(v[k].z, v[k].z, s_own); s_own = fmaf(v[k].w, v[k].w, s_own);
        s_prev = fmaf(pv[k].x, pv[k].x, s_prev); s_prev = fmaf(pv[k].y, pv[k].y, s_prev); s_prev = fmaf(pv[k].z, pv[k].z, s_prev); s_prev = fmaf(pv[k].w, pv[k].w, s_prev);
    }
    float4 gs[NV], ms[NV];                                     // asked for ahead of the barrier
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = 4 * (threadIdx.x + k * blockDim.x);
        gs[k] = i < d ? *reinterpret_cast<const float4*>(w + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        ms[k] = i < d ? *reinterpret_cast<const float4*>(mu + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    s_own = warp_sum(s_own); s_prev = warp_sum(s_prev); s_last = warp_sum(s_last);
    if (lane == 0) { part[0][warp] = s_own; part[1][warp] = s_prev; part[2][warp] = s_last; }
    __syncthreads();
    float t_own = 0.f, t_prev = 0.f, t_last = 0.f;
    for (int k = 0; k < n_warps; ++k) { t_own += part[0][k]; t_prev += part[1][k]; t_last += part[2][k]; }
    const float inv = 1.f / sqrtf(t_own / (float)d + eps);
    const float inv_prev = row_above ? 1.f / sqrtf(t_prev / (float)d + eps) : 1.f;      // (the kept row is normed already)
    const float inv_last = last != nullptr ? 1.f / sqrtf(t_last / (float)d + eps) : inv;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int i = 4 * (threadIdx.x + k * blockDim.x);
        if (i >= d) continue;
        const float4 g = gs[k], m = ms[k];
        const float n0 = v[k].x * inv * g.x, n1 = v[k].y * inv * g.y, n2 = v[k].z * inv * g.z, n3 = v[k].w * inv * g.w;
        const float p0 = row_above ? pv[k].x * inv_prev * g.x : pv[k].x, p1 = row_above ? pv[k].y * inv_prev * g.y : pv[k].y;
        const float p2 = row_above ? pv[k].z * inv_prev * g.z : pv[k].z, p3 = row_above ? pv[k].w * inv_prev * g.w : pv[k].w;
        store4<OT>(o + i, n0 + (p0 - n0) * m.x, n1 + (p1 - n1) * m.y, n2 + (p2 - n2) * m.z, n3 + (p3 - n3) * m.w);
        if (keep != nullptr) {                                 // (this thread has read these columns of the kept row)
            const float4 l = last != nullptr ? *reinterpret_cast<const float4*>(last + i) : v[k];
            *reinterpret_cast<float4*>(keep + i) = make_float4(l.x * inv_last * g.x, l.y * inv_last * g.y, l.z * inv_last * g.z, l.w * inv_last * g.w);
        }
    }
}

__global__ void add_row_vector_kernel(float* __restrict__ x, int ld, const float* __restrict__ v, int rows, int d) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * d) return;
    const int r = (int)(i / d), c = (int)(i - (long long)r * d);
    x[(size_t)r * ld + c] += v[c];
}
}  // namespace

extern "C" int vlrf_rmsnorm_shift(const float* x, int ld_x, const float* w, const float* mu, float eps, float* state,
                                  const int* tok_slot, const int* tok_pos, const int* seq_start, int n_seqs, int T, void* out,
                                  int out_dtype, int ld_out, int d, cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && d > 0 && ld_x >= d && ld_out >= d && n_seqs >= 0, "rmsnorm_shift: bad sizes");
    VLRF_REQUIRE(x && w && mu && state && tok_slot && tok_pos && seq_start && out, "rmsnorm_shift: a null pointer");
    if (T == 0) return VLRF_OK;
    const bool vec = d % 4 == 0 && ld_x % 4 == 0 && ld_out % 4 == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(mu) |
                       reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    VLRF_REQUIRE(out_dtype == VLRF_F32 || out_dtype == VLRF_BF16, "rmsnorm_shift: unknown output dtype %d", out_dtype);
    const int quads = d / 4;
    if (vec && quads <= SHIFT_ROW_MAX_NV * SHIFT_ROW_MAX_THREADS) {
        // a CTA a token: a quad of columns a thread up to 128 threads, then more quads a thread, then more threads
        int nv = 1, threads = 128;
        while (nv < SHIFT_ROW_MAX_NV && nv * threads < quads) nv *= 2;
        while (nv * threads < quads) threads *= 2;
        threads = min(threads, ((quads + nv - 1) / nv + 31) / 32 * 32);
#define ROWS(OT, NV) launch_chained(rmsnorm_shift_rows_kernel<OT, NV>, dim3(T), dim3(threads), (size_t)0, stream, x, ld_x, w, mu, eps, state, tok_slot, tok_pos, seq_start, n_seqs, T, (OT*)out, ld_out, d)
        if (out_dtype == VLRF_F32) { if (nv == 1) ROWS(float, 1); else if (nv == 2) ROWS(float, 2); else ROWS(float, 4); }
        else { if (nv == 1) ROWS(__nv_bfloat16, 1); else if (nv == 2) ROWS(__nv_bfloat16, 2); else ROWS(__nv_bfloat16, 4); }
#undef ROWS
        return vlrf_check_launch("rmsnorm_shift");
    }
    const dim3 grid((unsigned)((T + SHIFT_WARPS - 1) / SHIFT_WARPS)), block(SHIFT_WARPS * 32);
#define GO(OT, V) launch_chained(rmsnorm_shift_kernel<OT, V>, grid, block, (size_t)0, stream, x, ld_x, w, mu, eps, state, tok_slot, tok_pos, seq_start, n_seqs, T, (OT*)out, ld_out, d)
    if (out_dtype == VLRF_F32) { if (vec) GO(float, true); else GO(float, false); }
    else { if (vec) GO(__nv_bfloat16, true); else GO(__nv_bfloat16, false); }
#undef GO
    return vlrf_check_launch("rmsnorm_shift");
}

extern "C" int vlrf_add_row_vector(float* x, int ld, const float* v, int rows, int d, cudaStream_t stream) {
    VLRF_REQUIRE(rows >= 0 && d > 0 && ld >= d && x && v, "add_row_vector: bad arguments");
    if (rows == 0) return VLRF_OK;
    const long long n = (long long)rows * d;
    launch_chained(add_row_vector_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), (size_t)0, stream, x, ld, v, rows, d);
    return vlrf_check_launch("add_row_vector");
}

extern "C" int vlrf_group_rmsnorm(const float* y, int ld_y, const int* rows, const float* w, void* out, int out_dtype,
                                  int ld_out, int n_rows, int d, int groups, float eps, int accumulate, void* also_bf16,
                                  cudaStream_t stream) {
    VLRF_REQUIRE(n_rows >= 0 && d > 0 && groups > 0 && groups <= NORM_MAX_GROUPS, "group_rmsnorm: bad sizes rows=%d d=%d groups=%d", n_rows, d, groups);
    VLRF_REQUIRE(d % groups == 0, "group_rmsnorm: %d columns cannot be cut into %d equal parts", d, groups);
    VLRF_REQUIRE(ld_y >= d && ld_out >= d, "group_rmsnorm: leading sizes are smaller than the row");
    VLRF_REQUIRE(!accumulate || out_dtype == VLRF_F32, "group_rmsnorm: only float32 rows can be added to");
    if (n_rows == 0) return VLRF_OK;
    if (out_dtype == VLRF_F32) {
        if (accumulate) launch_chained(group_rmsnorm_kernel<float, true>, dim3(n_rows), dim3(NORM_THREADS), (size_t)(0), stream, y, ld_y, rows, w, (float*)out, ld_out, d, groups, eps, (__nv_bfloat16*)also_bf16);
        else launch_chained(group_rmsnorm_kernel<float, false>, dim3(n_rows), dim3(NORM_THREADS), (size_t)(0), stream, y, ld_y, rows, w, (float*)out, ld_out, d, groups, eps, (__nv_bfloat16*)also_bf16);
    } else if (out_dtype == VLRF_BF16) {
        launch_chained(group_rmsnorm_kernel<__nv_bfloat16, false>, dim3(n_rows), dim3(NORM_THREADS), (size_t)(0), stream, y, ld_y, rows, w, (__nv_bfloat16*)out, ld_out, d, groups, eps, (__nv_bfloat16*)also_bf16);
    } else {
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "group_rmsnorm: unknown output dtype %d", out_dtype);
    }
    return vlrf_check_launch("group_rmsnorm");
}

extern "C" int vlrf_cast_rows(const float* x, void* out, int out_dtype, long long n, cudaStream_t stream) {
    VLRF_REQUIRE(n >= 0, "cast_rows: negative size");
    if (n == 0) return VLRF_OK;
    const unsigned blocks = (unsigned)((n + 4 * 256 - 1) / (4 * 256));
    if (out_dtype == VLRF_BF16) launch_chained(cast_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), (size_t)(0), stream, x, (__nv_bfloat16*)out, n);
    else if (out_dtype == VLRF_F32) launch_chained(cast_rows_kernel<float>, dim3(blocks), dim3(256), (size_t)(0), stream, x, (float*)out, n);
    else return vlrf_fail(VLRF_ERR_INVALID_ARG, "cast_rows: unknown output dtype %d", out_dtype);
    return vlrf_check_launch("cast_rows");
}

static int gate_mul_any(const void* a, int lda, int a_dtype, const void* b, int ldb, int b_dtype, void* out, int ldo,
                        int out_dtype, int rows, int cols, int per, int act, cudaStream_t stream);

extern "C" int vlrf_gate_mul_clamped(const void* a, int lda, int a_dtype, const void* b, int ldb, int b_dtype, void* out, int ldo,
                                     int out_dtype, int rows, int cols, float limit, float alpha, cudaStream_t stream) {
    VLRF_REQUIRE(rows >= 0 && cols > 0 && lda >= cols && ldb >= cols && ldo >= cols, "gate_mul_clamped: bad sizes");
    VLRF_REQUIRE(limit > 0.f, "gate_mul_clamped: the bound %f is not positive", (double)limit);
    if (rows == 0) return VLRF_OK;
    const long long n = (long long)rows * cols;
    const dim3 blocks((unsigned)((n + 255) / 256));
    typedef __nv_bfloat16 bf;
    const bool aligned = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
                         cols % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0 && ldo % 8 == 0;
#define GO(AT, BT, OT) launch_chained(gate_mul_clamped_kernel<AT, BT, OT>, blocks, dim3(256), (size_t)0, stream, (const AT*)a, lda, (const BT*)b, ldb, (OT*)out, ldo, rows, cols, limit, alpha)
    if (a_dtype == VLRF_BF16 && b_dtype == VLRF_BF16 && out_dtype == VLRF_BF16 && aligned)
        launch_chained(gate_mul_clamped_bf16x8_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), (size_t)0, stream, (const bf*)a, lda,
                       (const bf*)b, ldb, (bf*)out, ldo, rows, cols / 8, limit, alpha);
    else if (a_dtype == VLRF_BF16 && b_dtype == VLRF_BF16 && out_dtype == VLRF_BF16) GO(bf, bf, bf);
    else if (a_dtype == VLRF_F32 && b_dtype == VLRF_F32 && out_dtype == VLRF_F32) GO(float, float, float);
    else if (a_dtype == VLRF_F32 && b_dtype == VLRF_F32 && out_dtype == VLRF_BF16) GO(float, float, bf);
    else return vlrf_fail(VLRF_ERR_INVALID_ARG, "gate_mul_clamped: dtypes %d, %d -> %d are not taken", a_dtype, b_dtype, out_dtype);
#undef GO
    return vlrf_check_launch("gate_mul_clamped");
}

extern "C" int vlrf_gate_mul(const void* a, int lda, int a_dtype, const void* b, int ldb, int b_dtype, void* out, int ldo,
                             int out_dtype, int rows, int cols, int act, cudaStream_t stream) {
    return gate_mul_any(a, lda, a_dtype, b, ldb, b_dtype, out, ldo, out_dtype, rows, cols, 1, act, stream);
}

extern "C" int vlrf_gate_mul_groups(const void* a, int lda, int a_dtype, const void* b, int ldb, int b_dtype, void* out, int ldo,
                                    int out_dtype, int rows, int cols, int per, int act, cudaStream_t stream) {
    VLRF_REQUIRE(per > 0 && cols % per == 0, "gate_mul_groups: %d columns are no whole groups of %d", cols, per);
    return gate_mul_any(a, lda, a_dtype, b, ldb, b_dtype, out, ldo, out_dtype, rows, cols, per, act, stream);
}

static int gate_mul_any(const void* a, int lda, int a_dtype, const void* b, int ldb, int b_dtype, void* out, int ldo,
                        int out_dtype, int rows, int cols, int per, int act, cudaStream_t stream) {
    VLRF_REQUIRE(rows >= 0 && cols > 0 && per > 0 && lda >= cols / per && ldb >= cols && ldo >= cols, "gate_mul: bad sizes");
    VLRF_REQUIRE(act == VLRF_ACT_SILU || act == VLRF_ACT_SIGMOID || act == VLRF_ACT_RELU || act == VLRF_ACT_GELU_TANH,
                 "gate_mul: the gate is x*sigmoid(x), sigmoid(x), max(x, 0) or the tanh form of GELU, not %d", act);
    if (rows == 0) return VLRF_OK;
    const long long n = (long long)rows * cols;
    const dim3 blocks((unsigned)((n + 255) / 256));
    const bool aligned = per == 1 && ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
                         cols % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0 && ldo % 8 == 0;
    typedef __nv_bfloat16 bf;
#define GO(AT, BT, OT) launch_chained(gate_mul_kernel<AT, BT, OT>, blocks, dim3(256), (size_t)0, stream, (const AT*)a, lda, (const BT*)b, ldb, (OT*)out, ldo, rows, cols, act, per)
    if (per > 1 && per % 8 == 0 && a_dtype == VLRF_F32 && b_dtype == VLRF_BF16 && out_dtype == VLRF_BF16 && ldb % 8 == 0 && ldo % 8 == 0 &&
        ((reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out)) & 15) == 0)
        launch_chained(gate_mul_groups_bf16x8_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), (size_t)0, stream, (const float*)a, lda,
                       (const bf*)b, ldb, (bf*)out, ldo, rows, cols / 8, per / 8, act);
    else if (a_dtype == VLRF_BF16 && b_dtype == VLRF_BF16 && out_dtype == VLRF_BF16 && aligned)
        launch_chained(gate_mul_bf16x8_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), (size_t)0, stream, (const bf*)a, lda, (const bf*)b, ldb,
                       (bf*)out, ldo, rows, cols / 8, act);
    else if (a_dtype == VLRF_BF16 && b_dtype == VLRF_BF16 && out_dtype == VLRF_BF16) GO(bf, bf, bf);
    else if (a_dtype == VLRF_F32 && b_dtype == VLRF_F32 && out_dtype == VLRF_F32) GO(float, float, float);
    else if (a_dtype == VLRF_F32 && b_dtype == VLRF_BF16 && out_dtype == VLRF_BF16) GO(float, bf, bf);
    else if (a_dtype == VLRF_F32 && b_dtype == VLRF_F32 && out_dtype == VLRF_BF16 && aligned && lda % 4 == 0 && ldb % 4 == 0)
        launch_chained(gate_mul_f32x4_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), (size_t)0, stream, (const float*)a, lda,
                       (const float*)b, ldb, (bf*)out, ldo, rows, cols / 4, act);
    else if (a_dtype == VLRF_F32 && b_dtype == VLRF_F32 && out_dtype == VLRF_BF16) GO(float, float, bf);
    else return vlrf_fail(VLRF_ERR_INVALID_ARG, "gate_mul: dtypes %d, %d -> %d are not taken", a_dtype, b_dtype, out_dtype);
#undef GO
    return vlrf_check_launch("gate_mul");
}
