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
//   mingru_scan_kernel   prompt steps: a lane per channel, 32 channels a CTA; the warps of the CTAs of a cluster (1 to 8
//                        CTAs a sequence: as many as fill the GPU while a run keeps four batches of tokens) cut the sequence's
//                        tokens of the step into consecutive runs.  Since S ← (1 − z) S + z c is linear in S, a run is the
//                        map S ↦ A · S + B with A = Π (1 − z): each warp first forms (A, B) of its run; a CTA chains its
//                        runs' maps in shared memory, the CTAs read one another's totals from there after a cluster
//                        barrier; each warp then walks its run again from the state it begins with, writing the outputs.
//                        The second walk finds its inputs in L2.  Loads come in batches of 8 tokens; where runs are
//                        long, a batch's loads are asked for ahead of the arithmetic on the batch before.
#include "common.cuh"

namespace {
constexpr int SCAN_WARPS = 16;
constexpr int SCAN_MAX_CTAS = 8;            // CTAs that share a sequence's tokens (a cluster)
constexpr int SCAN_BATCH = 8;             // tokens whose inputs a lane asks for together

// The gates of a step whose result is rounded to bfloat16 take exp2 and the reciprocal from the special-function unit
// (a sigmoid within about 1e-7 of the exact one, in a handful of instructions); float32 results take the exact forms,
// which cost some forty instructions a sigmoid and bound the prompt kernel by its instruction count.
template <typename OT> struct Gate {
    static __device__ __forceinline__ float sigmoid(float x) { return sigmoid_f(x); }
};
template <> struct Gate<__nv_bfloat16> {
    static __device__ __forceinline__ float sigmoid(float x) {
        float e, r;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));      // e^(−x); ∞ for x = −∞
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
        return r;
    }
};
template <typename OT> __device__ __forceinline__ float candidate_f(float u) { return u >= 0.f ? u + 0.5f : Gate<OT>::sigmoid(u); }
template <typename OT> __device__ __forceinline__ float out_gate_f(float g) { return g * Gate<OT>::sigmoid(g); }

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
    const float z = Gate<OT>::sigmoid(p[z_off + ch]), c = candidate_f<OT>(p[u_off + ch]), g = p[g_off + ch];
    const float before = pos > 0 ? state[((size_t)slot * 2 + (pos & 1)) * W + ch] : 0.f;
    const float S = fmaf(z, c - before, before);               // (1 − z) · S + z · c
    state[((size_t)slot * 2 + ((pos + 1) & 1)) * W + ch] = S;
    ElemIO<OT>::store(out + (size_t)row * ld_out + ch, S * out_gate_f<OT>(g));
}

// PIPE: the loads of a full batch are asked for ahead of the arithmetic on the batch before (two sets of registers:
// two CTAs an SM instead of three), for runs of several batches
template <typename OT, bool PIPE>
__global__ void __launch_bounds__(SCAN_WARPS * 32, PIPE ? 2 : (sizeof(OT) == 2 ? 3 : 1))
mingru_scan_kernel(const float* __restrict__ proj, int ld, int z_off, int u_off, int g_off, int W, float* state,
                   const int* __restrict__ seq_slot, const int* __restrict__ seq_start, const int* __restrict__ seq_pos0,
                   OT* __restrict__ out, int ld_out) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    // maps of this CTA's runs, of the runs ahead of each of its warps taken together, and of all of its runs
    __shared__ float A_sm[SCAN_WARPS][32], B_sm[SCAN_WARPS][32], PA_sm[SCAN_WARPS][32], PB_sm[SCAN_WARPS][32];
    __shared__ __align__(8) float total_sm[32][2];
    const int s = blockIdx.y;
    const int slot = seq_slot[s];
    if (slot < 0) return;                                      // padding (every CTA of the cluster leaves)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_cta = (int)gridDim.z, rank = (int)blockIdx.z;  // the cluster is the grid's z extent
    const int ch = blockIdx.x * 32 + lane;
    const bool live = ch < W;
    const int row0 = seq_start[s], n = seq_start[s + 1] - row0, pos0 = seq_pos0[s];
    const int runs = n_cta * SCAN_WARPS;
    const int per = (n + runs - 1) / runs;
    const int a = min(n, (rank * SCAN_WARPS + warp) * per), b = min(n, a + per);     // this warp's run of tokens
    const float* p = proj + (size_t)row0 * ld + (live ? ch : 0);
    float A = 1.f, B = 0.f;
    if (live) {
        const float* q = p + (size_t)a * ld;                   // the run's next token
        int t0 = a;
        if constexpr (PIPE) {
            if (t0 + SCAN_BATCH <= b) {                            // full batches: the next one's loads ahead of this one's arithmetic
                float zl[SCAN_BATCH], ul[SCAN_BATCH], zn[SCAN_BATCH], un[SCAN_BATCH];
#pragma unroll
                for (int k = 0; k < SCAN_BATCH; ++k) {
                    zl[k] = q[(size_t)k * ld + z_off];
                    ul[k] = q[(size_t)k * ld + u_off];
                }
                for (; t0 + SCAN_BATCH <= b; t0 += SCAN_BATCH) {
                    q += (size_t)SCAN_BATCH * ld;
                    const bool more = t0 + 2 * SCAN_BATCH <= b;
                    if (more) {
#pragma unroll
                        for (int k = 0; k < SCAN_BATCH; ++k) {
                            zn[k] = q[(size_t)k * ld + z_off];
                            un[k] = q[(size_t)k * ld + u_off];
                        }
                    }
#pragma unroll
                    for (int k = 0; k < SCAN_BATCH; ++k) {
                        const float z = Gate<OT>::sigmoid(zl[k]), c = candidate_f<OT>(ul[k]);
                        A *= 1.f - z;
                        B = fmaf(z, c - B, B);
                    }
                    if (more) {
#pragma unroll
                        for (int k = 0; k < SCAN_BATCH; ++k) { zl[k] = zn[k]; ul[k] = un[k]; }
                    }
                }
            }
        } else {
            for (; t0 + SCAN_BATCH <= b; t0 += SCAN_BATCH, q += (size_t)SCAN_BATCH * ld) {
                float zl[SCAN_BATCH], ul[SCAN_BATCH];
#pragma unroll
                for (int k = 0; k < SCAN_BATCH; ++k) {
                    zl[k] = q[(size_t)k * ld + z_off];
                    ul[k] = q[(size_t)k * ld + u_off];
                }
#pragma unroll
                for (int k = 0; k < SCAN_BATCH; ++k) {
                    const float z = Gate<OT>::sigmoid(zl[k]), c = candidate_f<OT>(ul[k]);
                    A *= 1.f - z;
                    B = fmaf(z, c - B, B);
                }
            }
        }
        if (t0 < b) {                                          // the run's last tokens, fewer than a batch
            float zl[SCAN_BATCH], ul[SCAN_BATCH];
#pragma unroll
            for (int k = 0; k < SCAN_BATCH; ++k) {             // (beyond the run: a gate that is shut changes nothing)
                const bool in = t0 + k < b;
                zl[k] = in ? q[(size_t)k * ld + z_off] : -INFINITY;
                ul[k] = in ? q[(size_t)k * ld + u_off] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < SCAN_BATCH; ++k) {
                const float z = Gate<OT>::sigmoid(zl[k]), c = candidate_f<OT>(ul[k]);
                A *= 1.f - z;
                B = fmaf(z, c - B, B);
            }
        }
    }
    A_sm[warp][lane] = A;
    B_sm[warp][lane] = B;
    __syncthreads();
    if (warp == 0) {                                           // the CTA's runs chained, per channel
        float pa = 1.f, pb = 0.f;
#pragma unroll
        for (int w = 0; w < SCAN_WARPS; ++w) {
            PA_sm[w][lane] = pa;
            PB_sm[w][lane] = pb;
            const float aw = A_sm[w][lane];
            pb = fmaf(aw, pb, B_sm[w][lane]);
            pa *= aw;
        }
        total_sm[lane][0] = pa;
        total_sm[lane][1] = pb;
    }
    cluster_sync_all();                                        // every CTA's total is in its shared memory
    float S = 0.f;
    if (live && pos0 > 0) S = state[((size_t)slot * 2 + (pos0 & 1)) * W + ch];
    const uint32_t tot = (uint32_t)__cvta_generic_to_shared(&total_sm[lane][0]);
    for (int c = 0; c < rank; ++c)                             // the CTAs ahead
        S = fmaf(ld_cluster_f32(tot, (uint32_t)c), S, ld_cluster_f32(tot + 4u, (uint32_t)c));
    S = fmaf(PA_sm[warp][lane], S, PB_sm[warp][lane]);         // the state ahead of this warp's run
    cluster_sync_relaxed();                                    // everyone has read the kept state and the totals
    if (live) {
        const float* q = p + (size_t)a * ld;
        OT* o = out + (size_t)(row0 + a) * ld_out + ch;
        int t0 = a;
        if constexpr (PIPE) {
            if (t0 + SCAN_BATCH <= b) {
                float zl[SCAN_BATCH], ul[SCAN_BATCH], gl[SCAN_BATCH], zn[SCAN_BATCH], un[SCAN_BATCH], gn[SCAN_BATCH];
#pragma unroll
                for (int k = 0; k < SCAN_BATCH; ++k) {
                    zl[k] = q[(size_t)k * ld + z_off];
                    ul[k] = q[(size_t)k * ld + u_off];
                    gl[k] = q[(size_t)k * ld + g_off];
                }
                for (; t0 + SCAN_BATCH <= b; t0 += SCAN_BATCH, o += (size_t)SCAN_BATCH * ld_out) {
                    q += (size_t)SCAN_BATCH * ld;
                    const bool more = t0 + 2 * SCAN_BATCH <= b;
                    if (more) {
#pragma unroll
                        for (int k = 0; k < SCAN_BATCH; ++k) {
                            zn[k] = q[(size_t)k * ld + z_off];
                            un[k] = q[(size_t)k * ld + u_off];
                            gn[k] = q[(size_t)k * ld + g_off];
                        }
                    }
#pragma unroll
                    for (int k = 0; k < SCAN_BATCH; ++k) {
                        const float z = Gate<OT>::sigmoid(zl[k]), c = candidate_f<OT>(ul[k]);
                        S = fmaf(z, c - S, S);
                        ElemIO<OT>::store(o + (size_t)k * ld_out, S * out_gate_f<OT>(gl[k]));
                    }
                    if (more) {
#pragma unroll
                        for (int k = 0; k < SCAN_BATCH; ++k) { zl[k] = zn[k]; ul[k] = un[k]; gl[k] = gn[k]; }
                    }
                }
            }
        } else {
            for (; t0 + SCAN_BATCH <= b; t0 += SCAN_BATCH, q += (size_t)SCAN_BATCH * ld, o += (size_t)SCAN_BATCH * ld_out) {
                float zl[SCAN_BATCH], ul[SCAN_BATCH], gl[SCAN_BATCH];
#pragma unroll
                for (int k = 0; k < SCAN_BATCH; ++k) {
                    zl[k] = q[(size_t)k * ld + z_off];
                    ul[k] = q[(size_t)k * ld + u_off];
                    gl[k] = q[(size_t)k * ld + g_off];
                }
#pragma unroll
                for (int k = 0; k < SCAN_BATCH; ++k) {
                    const float z = Gate<OT>::sigmoid(zl[k]), c = candidate_f<OT>(ul[k]);
                    S = fmaf(z, c - S, S);
                    ElemIO<OT>::store(o + (size_t)k * ld_out, S * out_gate_f<OT>(gl[k]));
                }
            }
        }
        if (t0 < b) {
            float zl[SCAN_BATCH], ul[SCAN_BATCH], gl[SCAN_BATCH];
#pragma unroll
            for (int k = 0; k < SCAN_BATCH; ++k) {
                const bool in = t0 + k < b;
                zl[k] = in ? q[(size_t)k * ld + z_off] : -INFINITY;
                ul[k] = in ? q[(size_t)k * ld + u_off] : 0.f;
                gl[k] = in ? q[(size_t)k * ld + g_off] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < SCAN_BATCH; ++k) {
                const float z = Gate<OT>::sigmoid(zl[k]), c = candidate_f<OT>(ul[k]);
                S = fmaf(z, c - S, S);
                if (t0 + k < b) ElemIO<OT>::store(o + (size_t)k * ld_out, S * out_gate_f<OT>(gl[k]));
            }
        }
        // the last run's warp ends at the sequence's last token of the step (an empty run: at the state it was handed)
        if (rank == n_cta - 1 && warp == SCAN_WARPS - 1) state[((size_t)slot * 2 + ((pos0 + n) & 1)) * W + ch] = S;
    }
}
int scan_sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        sms = v > 0 ? v : 148;
    }
    return sms;
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
        // CTAs a sequence: doubled while the grid leaves SMs empty and a warp's run would still keep four batches of tokens
        const int base = ((W + 31) / 32) * n_seqs;
        int n_cta = 1;
        while (n_cta < SCAN_MAX_CTAS && base * n_cta < scan_sm_count() && max_new >= 8 * n_cta * SCAN_WARPS * SCAN_BATCH) n_cta *= 2;
        const bool pipe = max_new >= 4 * n_cta * SCAN_WARPS * SCAN_BATCH;      // the longest sequence's runs have four batches
        const dim3 grid((unsigned)((W + 31) / 32), (unsigned)n_seqs, (unsigned)n_cta), cluster(1, 1, (unsigned)n_cta);
#define VLRF_SCAN(OT, PIPE) launch_chained_cluster(mingru_scan_kernel<OT, PIPE>, grid, dim3(SCAN_WARPS * 32), (size_t)0, cluster, stream, proj, ld, z_off, u_off, g_off, W, state, seq_slot, seq_start, seq_pos0, (OT*)out, ld_out)
        if (out_dtype == VLRF_F32) { if (pipe) VLRF_SCAN(float, true); else VLRF_SCAN(float, false); }
        else { if (pipe) VLRF_SCAN(__nv_bfloat16, true); else VLRF_SCAN(__nv_bfloat16, false); }
#undef VLRF_SCAN
    }
    return vlrf_check_launch("mingru_scan");
}
