// A gated recurrence that runs element by element (the "minGRU" form): per token and channel
//     z = sigmoid(a),   c = u + 1/2 where u ≥ 0, sigmoid(u) below,   S ← (1 − z) · S + z · c,   out = S · g · sigmoid(g),
// with a, u and g three column ranges of one float32 product of the layer's input.  Gates, candidates, the recurrence
// and its state are float32; the result is rounded once to the output's dtype.
//
// The state of a sequence is a float32 row [W], held twice ([slot][2][W]): a step reads the copy of the parity of the
// position it begins at (zeros at position 0) and writes the copy of the parity of the position it ends at, so a step
// of one token leaves what it read untouched and may run twice with the same result.
//
//   mingru_step_kernel   steps of one token a sequence: a thread per (row, channel)
//   mingru_scan_kernel   prompt steps: a CTA per (32 channels, sequence), a lane per channel; the warps cut the
//                        sequence's tokens of the step into consecutive runs.  Since S ← (1 − z) S + z c is linear in
//                        S, a run is the map S ↦ A · S + B with A = Π (1 − z): each warp first forms (A, B) of its run,
//                        the runs' maps are chained through shared memory, and each warp then walks its run again from
//                        the state it begins with, writing the outputs.  The second walk finds its inputs in L2.
#include "common.cuh"

namespace {
constexpr int SCAN_WARPS = 32;
constexpr int SCAN_BATCH = 8;             // tokens whose inputs a lane asks for together

__device__ __forceinline__ float candidate_f(float u) { return u >= 0.f ? u + 0.5f : sigmoid_f(u); }

template <typename OT>
__global__ void __launch_bounds__(256)
mingru_step_kernel(const float* __restrict__ proj, int ld, int z_off, int u_off, int g_off, int W, float* state,
                   const int* __restrict__ seq_slot, const int* __restrict__ seq_start, const int* __restrict__ seq_pos0, int n_seqs,
                   OT* __restrict__ out, int ld_out) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_seqs * W) return;
    const int s = (int)(i / W), ch = (int)(i - (long long)s * W);
    const int slot = seq_slot[s];
    if (slot < 0) return;                                      // padding row
    const int row = seq_start[s], pos = seq_pos0[s];
    const float* p = proj + (size_t)row * ld;
    const float z = sigmoid_f(p[z_off + ch]), c = candidate_f(p[u_off + ch]), g = p[g_off + ch];
    const float before = pos > 0 ? state[((size_t)slot * 2 + (pos & 1)) * W + ch] : 0.f;
    const float S = fmaf(z, c - before, before);               // (1 − z) · S + z · c
    state[((size_t)slot * 2 + ((pos + 1) & 1)) * W + ch] = S;
    ElemIO<OT>::store(out + (size_t)row * ld_out + ch, S * silu_f(g));
}

template <typename OT>
__global__ void __launch_bounds__(SCAN_WARPS * 32)
mingru_scan_kernel(const float* __restrict__ proj, int ld, int z_off, int u_off, int g_off, int W, float* state,
                   const int* __restrict__ seq_slot, const int* __restrict__ seq_start, const int* __restrict__ seq_pos0,
                   OT* __restrict__ out, int ld_out) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    __shared__ float A_sm[SCAN_WARPS][32], B_sm[SCAN_WARPS][32];
    const int s = blockIdx.y;
    const int slot = seq_slot[s];
    if (slot < 0) return;                                      // padding (the whole CTA leaves)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ch = blockIdx.x * 32 + lane;
    const bool live = ch < W;
    const int row0 = seq_start[s], n = seq_start[s + 1] - row0, pos0 = seq_pos0[s];
    const int per = (n + SCAN_WARPS - 1) / SCAN_WARPS;
    const int a = min(n, warp * per), b = min(n, a + per);     // this warp's run of tokens
    const float* p = proj + (size_t)row0 * ld + (live ? ch : 0);
    float A = 1.f, B = 0.f;
    if (live) {
        for (int t0 = a; t0 < b; t0 += SCAN_BATCH) {
            float zl[SCAN_BATCH], ul[SCAN_BATCH];
#pragma unroll
            for (int k = 0; k < SCAN_BATCH; ++k) {             // (beyond the run: a gate that is shut changes nothing)
                const bool in = t0 + k < b;
                zl[k] = in ? p[(size_t)(t0 + k) * ld + z_off] : -INFINITY;
                ul[k] = in ? p[(size_t)(t0 + k) * ld + u_off] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < SCAN_BATCH; ++k) {
                const float z = sigmoid_f(zl[k]), c = candidate_f(ul[k]);
                A *= 1.f - z;
                B = fmaf(z, c - B, B);
            }
        }
    }
    A_sm[warp][lane] = A;
    B_sm[warp][lane] = B;
    __syncthreads();
    float S = 0.f;
    if (live && pos0 > 0) S = state[((size_t)slot * 2 + (pos0 & 1)) * W + ch];
    float S_end = S;
    for (int w = 0; w < SCAN_WARPS; ++w) {
        if (w == warp) S = S_end;                              // the state ahead of this warp's run
        S_end = fmaf(A_sm[w][lane], S_end, B_sm[w][lane]);
    }
    __syncthreads();                                           // every warp has read the kept state
    if (live && warp == 0) state[((size_t)slot * 2 + ((pos0 + n) & 1)) * W + ch] = S_end;
    if (!live) return;
    OT* o = out + (size_t)row0 * ld_out + ch;
    for (int t0 = a; t0 < b; t0 += SCAN_BATCH) {
        float zl[SCAN_BATCH], ul[SCAN_BATCH], gl[SCAN_BATCH];
#pragma unroll
        for (int k = 0; k < SCAN_BATCH; ++k) {
            const bool in = t0 + k < b;
            zl[k] = in ? p[(size_t)(t0 + k) * ld + z_off] : -INFINITY;
            ul[k] = in ? p[(size_t)(t0 + k) * ld + u_off] : 0.f;
            gl[k] = in ? p[(size_t)(t0 + k) * ld + g_off] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < SCAN_BATCH; ++k) {
            const float z = sigmoid_f(zl[k]), c = candidate_f(ul[k]);
            S = fmaf(z, c - S, S);
            if (t0 + k < b) ElemIO<OT>::store(o + (size_t)(t0 + k) * ld_out, S * silu_f(gl[k]));
        }
    }
}
}  // namespace

extern "C" int vlrf_mingru_scan(const float* proj, int ld, int z_off, int u_off, int g_off, int W, float* state, const int* seq_slot,
                                const int* seq_start, const int* seq_pos0, int n_seqs, int max_new, void* out, int out_dtype,
                                int ld_out, cudaStream_t stream) {
    VLRF_REQUIRE(W > 0 && n_seqs >= 0 && max_new >= 0 && ld_out >= W, "mingru_scan: bad sizes");
    VLRF_REQUIRE(z_off >= 0 && u_off >= 0 && g_off >= 0 && ld >= W + max(z_off, max(u_off, g_off)), "mingru_scan: the column ranges leave the product's rows");
    VLRF_REQUIRE(proj && state && seq_slot && seq_start && seq_pos0 && out, "mingru_scan: a null pointer");
    VLRF_REQUIRE(out_dtype == VLRF_F32 || out_dtype == VLRF_BF16, "mingru_scan: unknown output dtype %d", out_dtype);
    if (n_seqs == 0 || max_new == 0) return VLRF_OK;
    if (max_new == 1) {
        const long long n = (long long)n_seqs * W;
        const dim3 grid((unsigned)((n + 255) / 256));
        if (out_dtype == VLRF_F32)
            launch_chained(mingru_step_kernel<float>, grid, dim3(256), (size_t)0, stream, proj, ld, z_off, u_off, g_off, W, state, seq_slot, seq_start, seq_pos0, n_seqs, (float*)out, ld_out);
        else
            launch_chained(mingru_step_kernel<__nv_bfloat16>, grid, dim3(256), (size_t)0, stream, proj, ld, z_off, u_off, g_off, W, state, seq_slot, seq_start, seq_pos0, n_seqs, (__nv_bfloat16*)out, ld_out);
    } else {
        VLRF_REQUIRE(n_seqs <= 65535, "mingru_scan: at most 65535 sequences a step, not %d", n_seqs);
        const dim3 grid((unsigned)((W + 31) / 32), (unsigned)n_seqs);
        if (out_dtype == VLRF_F32)
            launch_chained(mingru_scan_kernel<float>, grid, dim3(SCAN_WARPS * 32), (size_t)0, stream, proj, ld, z_off, u_off, g_off, W, state, seq_slot, seq_start, seq_pos0, (float*)out, ld_out);
        else
            launch_chained(mingru_scan_kernel<__nv_bfloat16>, grid, dim3(SCAN_WARPS * 32), (size_t)0, stream, proj, ld, z_off, u_off, g_off, W, state, seq_slot, seq_start, seq_pos0, (__nv_bfloat16*)out, ld_out);
    }
    return vlrf_check_launch("mingru_scan");
}
