// Routing tokens to experts, entirely on the device (nothing is read back, so a step with routed experts can be
// captured and replayed).
//
//   moe_route    per token: the `top` largest of E float32 router logits (ties: the lower index), their softmax over
//                the chosen ones alone, and the token's rank among the rows of each chosen expert (a counter per
//                expert).  An extra logit in column E, if asked for, becomes sigmoid(·): the gate of a shared expert.
//                Padding rows (slot −1) choose nothing.
//   moe_route_scored   the same places, another rule: s = softmax of all E logits; the choice looks at s + correction,
//                only inside the `keep` groups (of `groups` equal groups of neighbouring experts) whose largest such
//                score is largest; the weights are the chosen s · scale, not renormalized.  The last n_identity
//                router outputs stand for experts that return their input: they get id −2, no rank and no row, and
//                moe_combine adds weight · input for them.  With `scoring` 1 the scores are sigmoid(logit), each
//                output by itself, instead of the softmax over all of them; everything else is the same.
//   moe_plan     offsets[e] = rows of the experts before e (E + 1 entries); the counters are left zero.
//   moe_gather   pair (token, j) gets row offsets[expert] + rank of the expert-sorted buffer: the token's input row
//                is copied there and the row's number kept.
//   moe_combine  y[t] = Σ_j weight[t][j] · expert_out[row[t][j]] (+ gate[t] · shared_out[t]) (+ residual[t]), float32,
//                j in order.
//
// Between gather and combine run the grouped products (gemm_heads.cu: gemm_grouped) and the gate (norm_rms.cu).
// Which row of the sorted buffer a pair gets depends on the order in which CTAs reach the counters; a row's result
// does not depend on where it lies, so the outcome is the same bit for bit.
#include "common.cuh"

namespace {
constexpr int ROUTE_MAX_E = 512;             // 16 logits a lane

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ z, int ld_z, int E, int top, int shared_gate, const int* __restrict__ tok_slot,
                 int* __restrict__ ids, float* __restrict__ wts, int* __restrict__ rank, float* __restrict__ gate,
                 int* __restrict__ counts, int T) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (t >= T) return;
    if (tok_slot != nullptr && tok_slot[t] < 0) {
        for (int j = lane; j < top; j += 32) { ids[(size_t)t * top + j] = -1; wts[(size_t)t * top + j] = 0.f; rank[(size_t)t * top + j] = 0; }
        if (shared_gate && lane == 0) gate[t] = 0.f;
        return;
    }
    const float* zr = z + (size_t)t * ld_z;
    float v[ROUTE_MAX_E / 32];
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_E / 32; ++i) {
        const int e = i * 32 + lane;
        float x = e < E ? zr[e] : -INFINITY;
        v[i] = (x == x) ? x : -INFINITY;                       // a NaN can never be chosen before a number
    }
    unsigned taken = 0;                                        // bit i: this lane's i-th logit is chosen
    float my_val = 0.f;                                        // lane j keeps the j-th chosen logit
    int my_id = -1;
    float first = 0.f;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int idx = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < ROUTE_MAX_E / 32; ++i) {
            const int e = i * 32 + lane;
            if (e < E && !(taken >> i & 1u) && (v[i] > best || (v[i] == best && e < idx))) { best = v[i]; idx = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
        }
        if ((idx & 31) == lane) taken |= 1u << (idx >> 5);
        if (j == 0) first = best;
        if ((j & 31) == lane) { my_val = best; my_id = idx; }
    }
    const float ex = (lane < top) ? expf(my_val - first) : 0.f;
    const float sum = warp_sum(ex);
    if (lane < top) {
        ids[(size_t)t * top + lane] = my_id;
        wts[(size_t)t * top + lane] = ex / sum;
        rank[(size_t)t * top + lane] = atomicAdd(counts + my_id, 1);
    }
    if (shared_gate && lane == 0) gate[t] = sigmoid_f(zr[E]);
}

// NI: logits a lane (the router's outputs are at most 32 · NI)
template <int NI>
__global__ void __launch_bounds__(128)
moe_route_scored_kernel(const float* __restrict__ z, int ld_z, int E, int top, int groups, int keep, int n_identity, float scale,
                        int scoring, const float* __restrict__ correction, const int* __restrict__ tok_slot, int* __restrict__ ids,
                        float* __restrict__ wts, int* __restrict__ rank, int* __restrict__ counts, int T) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    __shared__ float choice_sm[4][NI * 32];                // a warp's choice scores, then its groups' scores
    __shared__ float group_sm[4][NI * 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * 4 + warp;
    if (t >= T) return;                                        // (whole warps leave; only warp barriers below)
    if (tok_slot != nullptr && tok_slot[t] < 0) {
        for (int j = lane; j < top; j += 32) { ids[(size_t)t * top + j] = -1; wts[(size_t)t * top + j] = 0.f; rank[(size_t)t * top + j] = 0; }
        return;
    }
    const float* zr = z + (size_t)t * ld_z;
    float s[NI], v[NI];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const int e = i * 32 + lane;
        const float x = e < E ? zr[e] : -INFINITY;
        s[i] = (x == x) ? x : -INFINITY;                       // a NaN counts as no score at all
        m = fmaxf(m, s[i]);
    }
    m = warp_max(m);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const int e = i * 32 + lane;
        if (scoring == 1) s[i] = e < E ? 1.f / (1.f + expf(-s[i])) : 0.f;       // (a NaN logit became −∞: score 0)
        else s[i] = e < E ? expf(s[i] - m) : 0.f;
        sum += s[i];
    }
    sum = warp_sum(sum);
    const float inv = scoring == 1 ? 1.f : 1.f / sum;
    float* cs = choice_sm[warp];
    float* gs = group_sm[warp];
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const int e = i * 32 + lane;
        s[i] *= inv;
        v[i] = e < E ? s[i] + correction[e] : -INFINITY;
        if (!(v[i] == v[i])) v[i] = -INFINITY;
        if (e < E) cs[e] = v[i];
    }
    __syncwarp();
    const int per = E / groups;
    if (keep < groups) {
        for (int g = lane; g < groups; g += 32) {
            float b = -INFINITY;
            for (int k = 0; k < per; ++k) b = fmaxf(b, cs[g * per + k]);
            gs[g] = b;
        }
        __syncwarp();
        // the `keep` best groups, one after the other (ties: the lower index); a kept group's score becomes NaN as its mark
        for (int r = 0; r < keep; ++r) {
            float best = -INFINITY;
            int idx = 0x7fffffff;
            for (int g = lane; g < groups; g += 32) {
                const float x = gs[g];
                if (x == x && (idx == 0x7fffffff || x > best)) { best = x; idx = g; }      // (ascending g: the first maximum stays)
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
                if (oi != 0x7fffffff && (idx == 0x7fffffff || ob > best || (ob == best && oi < idx))) { best = ob; idx = oi; }
            }
            __syncwarp();
            if (lane == 0 && idx != 0x7fffffff) gs[idx] = __int_as_float(0x7fc00000);
            __syncwarp();
        }
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int e = i * 32 + lane;
            if (e < E) { const float x = gs[e / per]; if (x == x) v[i] = -INFINITY; }       // its group was not kept
        }
    }
    unsigned taken = 0;
    float my_w = 0.f;
    int my_id = -1;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int idx = 0x7fffffff;
        float sb = 0.f;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int e = i * 32 + lane;
            if (e < E && !(taken >> i & 1u) && (idx == 0x7fffffff || v[i] > best)) { best = v[i]; idx = e; sb = s[i]; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            const float os = __shfl_xor_sync(0xffffffffu, sb, o);
            if (oi != 0x7fffffff && (idx == 0x7fffffff || ob > best || (ob == best && oi < idx))) { best = ob; idx = oi; sb = os; }
        }
        if ((idx & 31) == lane) taken |= 1u << (idx >> 5);
        if ((j & 31) == lane) { my_w = sb * scale; my_id = idx; }
    }
    if (lane < top) {
        const bool identity = my_id >= E - n_identity;
        ids[(size_t)t * top + lane] = identity ? -2 : my_id;
        wts[(size_t)t * top + lane] = my_w;
        rank[(size_t)t * top + lane] = identity ? 0 : atomicAdd(counts + my_id, 1);
    }
}

__global__ void moe_plan_kernel(int* __restrict__ counts, int* __restrict__ offsets, int E) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) { offsets[e] = at; at += counts[e]; counts[e] = 0; }
        offsets[E] = at;
    }
}

template <typename ET>
__global__ void __launch_bounds__(128)
moe_gather_kernel(const ET* __restrict__ h, int width, const int* __restrict__ ids, const int* __restrict__ rank,
                  const int* __restrict__ offsets, ET* __restrict__ sorted, int* __restrict__ row_of, int top) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    const int pair = blockIdx.x;
    const int e = ids[pair];
    if (e < 0) { if (threadIdx.x == 0) row_of[pair] = -1; return; }
    const int row = offsets[e] + rank[pair];
    if (threadIdx.x == 0) row_of[pair] = row;
    const ET* src = h + (size_t)(pair / top) * width;
    ET* dst = sorted + (size_t)row * width;
    for (int i = threadIdx.x; i < width; i += 128) dst[i] = src[i];
}

template <typename HT>
__global__ void __launch_bounds__(128)
moe_combine_kernel(const float* __restrict__ expert_out, int width, const int* __restrict__ row_of, const float* __restrict__ wts,
                   int top, const float* __restrict__ shared_out, const float* __restrict__ gate, const float* residual,
                   float* y, const int* __restrict__ ids, const HT* __restrict__ h) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < width; i += 128) {
        float s = 0.f;
        for (int j = 0; j < top; ++j) {
            const int row = row_of[(size_t)t * top + j];
            if (row >= 0) s = fmaf(wts[(size_t)t * top + j], expert_out[(size_t)row * width + i], s);
            else if (ids != nullptr && ids[(size_t)t * top + j] == -2)                      // an expert that returns its input
                s = fmaf(wts[(size_t)t * top + j], ElemIO<HT>::load(h + (size_t)t * width + i), s);
        }
        if (shared_out != nullptr) s += (gate != nullptr ? gate[t] : 1.f) * shared_out[(size_t)t * width + i];
        if (residual != nullptr) s += residual[(size_t)t * width + i];
        y[(size_t)t * width + i] = s;
    }
}
}  // namespace

extern "C" int vlrf_moe_route(const float* z, int ld_z, int E, int top, int shared_gate, const int* tok_slot, int* ids,
                              float* wts, int* rank, float* gate, int* counts, int T, cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && E > 0 && E <= ROUTE_MAX_E, "moe_route: takes 1…%d experts, not %d", ROUTE_MAX_E, E);
    VLRF_REQUIRE(top > 0 && top <= E && top <= 32, "moe_route: a token takes 1…min(32, experts) experts, not %d of %d", top, E);
    VLRF_REQUIRE(ld_z >= E + (shared_gate ? 1 : 0) && (!shared_gate || gate != nullptr), "moe_route: the logits' rows are too short, or no place for the gate");
    if (T == 0) return VLRF_OK;
    launch_chained(moe_route_kernel, dim3((T + 3) / 4), dim3(128), (size_t)(0), stream, z, ld_z, E, top, shared_gate, tok_slot, ids, wts, rank, gate, counts, T);
    return vlrf_check_launch("moe_route");
}

extern "C" int vlrf_moe_route_scored(const float* z, int ld_z, int E, int top, int groups, int keep, int n_identity, float scale,
                                     int scoring, const float* correction, const int* tok_slot, int* ids, float* wts, int* rank, int* counts,
                                     int T, cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && E > 0 && E <= ROUTE_MAX_E && ld_z >= E, "moe_route_scored: takes 1…%d router outputs, not %d", ROUTE_MAX_E, E);
    VLRF_REQUIRE(groups > 0 && E % groups == 0 && keep > 0 && keep <= groups, "moe_route_scored: %d outputs in %d groups of which %d are kept", E, groups, keep);
    VLRF_REQUIRE(top > 0 && top <= 32 && top <= keep * (E / groups), "moe_route_scored: a token takes 1…min(32, %d) experts, not %d", keep * (E / groups), top);
    VLRF_REQUIRE(n_identity >= 0 && n_identity <= E && correction != nullptr, "moe_route_scored: bad arguments");
    VLRF_REQUIRE(scoring == 0 || scoring == 1, "moe_route_scored: scores are a softmax over all outputs (0) or sigmoids (1), not %d", scoring);
    if (T == 0) return VLRF_OK;
    const dim3 grid((T + 3) / 4), block(128);
#define VLRF_ROUTE_SCORED(NI) launch_chained(moe_route_scored_kernel<NI>, grid, block, (size_t)(0), stream, z, ld_z, E, top, groups, keep, n_identity, scale, scoring, correction, tok_slot, ids, wts, rank, counts, T)
    if (E <= 32) VLRF_ROUTE_SCORED(1);
    else if (E <= 64) VLRF_ROUTE_SCORED(2);
    else if (E <= 128) VLRF_ROUTE_SCORED(4);
    else VLRF_ROUTE_SCORED(ROUTE_MAX_E / 32);
#undef VLRF_ROUTE_SCORED
    return vlrf_check_launch("moe_route_scored");
}

extern "C" int vlrf_moe_plan(int* counts, int* offsets, int E, cudaStream_t stream) {
    VLRF_REQUIRE(E > 0 && counts != nullptr && offsets != nullptr, "moe_plan: bad arguments");
    launch_chained(moe_plan_kernel, dim3(1), dim3(32), (size_t)(0), stream, counts, offsets, E);
    return vlrf_check_launch("moe_plan");
}

extern "C" int vlrf_moe_gather(const void* h, int dtype, int width, const int* ids, const int* rank, const int* offsets,
                               void* sorted, int* row_of, int T, int top, cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && width > 0 && top > 0, "moe_gather: bad sizes");
    if (T == 0) return VLRF_OK;
    if (dtype == VLRF_F32)
        launch_chained(moe_gather_kernel<float>, dim3(T * top), dim3(128), (size_t)(0), stream, (const float*)h, width, ids, rank, offsets, (float*)sorted, row_of, top);
    else if (dtype == VLRF_BF16)
        launch_chained(moe_gather_kernel<__nv_bfloat16>, dim3(T * top), dim3(128), (size_t)(0), stream, (const __nv_bfloat16*)h, width, ids, rank, offsets, (__nv_bfloat16*)sorted, row_of, top);
    else return vlrf_fail(VLRF_ERR_INVALID_ARG, "moe_gather: unknown dtype %d", dtype);
    return vlrf_check_launch("moe_gather");
}

extern "C" int vlrf_moe_combine(const float* expert_out, int width, const int* row_of, const float* wts, int top,
                                const float* shared_out, const float* gate, const float* residual, float* y, int T,
                                const int* ids, const void* h, int h_dtype, cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && width > 0 && top > 0, "moe_combine: bad sizes");
    VLRF_REQUIRE((ids == nullptr) == (h == nullptr), "moe_combine: experts that return their input need ids and the input rows");
    if (T == 0) return VLRF_OK;
    if (h != nullptr && h_dtype == VLRF_BF16)
        launch_chained(moe_combine_kernel<__nv_bfloat16>, dim3(T), dim3(128), (size_t)(0), stream, expert_out, width, row_of, wts, top, shared_out, gate, residual, y, ids, (const __nv_bfloat16*)h);
    else if (h == nullptr || h_dtype == VLRF_F32)
        launch_chained(moe_combine_kernel<float>, dim3(T), dim3(128), (size_t)(0), stream, expert_out, width, row_of, wts, top, shared_out, gate, residual, y, ids, (const float*)h);
    else return vlrf_fail(VLRF_ERR_INVALID_ARG, "moe_combine: unknown dtype %d of the input rows", h_dtype);
    return vlrf_check_launch("moe_combine");
}
