// Attention with key and value sizes of their own on the tensor cores (bfloat16), for prompt steps and decode steps.
//
// A CTA of four warps takes one key/value head of one sequence and a tile of 64 rows; a row is one (token, query head)
// pair: the R = H / Hkv query heads that share the key/value head, for 64 / R consecutive new tokens (a decode step has
// one token, so its rows are the R heads).  Key and value tiles of 64 keys, one cache block each, are read once for all
// rows by `cp.async` into two stages (up to four in a decode step, whose CTAs have little else to hide the loads behind); S = Q·Kᵀ and O += P·V run on `mma.sync.m16n8k16` with float32 accumulation, the
// causal and window masks on tiles that touch an edge, the softmax online in float32 (running maximum and sum per row,
// in units of log2 e), P packed to bfloat16 from the accumulator registers.  Head sizes are padded in shared memory
// to the next size the kernel is instantiated for (32, 64, 96, 128) with zeros, so any multiple of 8 up to 128 is taken.
// Rows of a value tile behind the sequence's last token are zero-filled instead of loaded: 0 · V must not meet what
// an earlier owner of the block left there.
//
// A decode step may cut every context into `n_split` parts (CTA x = part; part p takes the key tiles p, p + n_split, …);
// the parts leave unnormalised sums with their maximum and denominator in `partials`, and a second kernel merges them in
// a fixed order.  The result is multiplied by out_scale.
//
// Parameters beside the window: softcap c > 0 squashes every scaled score to c · tanh(score / c); keep_first n > 0 lets
// every query also see the keys at positions below n (the tiles that hold them come first in a CTA's list of tiles,
// ahead of the window's); sink (a float32 per query head) adds exp(sink_h) to the softmax's denominator where the parts
// of a row are complete (in the kernel, or in the merge of a cut context); gate (float32 [rows][ld_gate], a logit per
// query head) multiplies head h's finished result by sigmoid(gate[row][h]), at the same places.
#include "common.cuh"

namespace {
constexpr int WM_WARPS = 4;
constexpr int WM_ROWS = 64;
constexpr int WM_BK = 64;

__device__ __forceinline__ uint32_t wsm(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(wsm(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void w_ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void w_ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void w_mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t w_pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// DEC: a tile of at most 16 rows (a decode step: one token, the R heads of the group).  The four warps then share the
// rows and deal the keys of every tile among themselves, 16 each, and their sums are merged through shared memory.
// NST: stages of key/value tiles (NST − 1 tiles are under way while one is multiplied).
template <int DKP, int DVP, bool DEC, int NST>
__global__ void __launch_bounds__(WM_WARPS * 32)
attn_window_mma_kernel(const __nv_bfloat16* __restrict__ q, int ldq, const __nv_bfloat16* __restrict__ Kc,
                       const __nv_bfloat16* __restrict__ Vc, const int* __restrict__ block_table, int max_blocks,
                       const int* __restrict__ seq_slot, const int* __restrict__ seq_start, const int* __restrict__ seq_pos0,
                       __nv_bfloat16* __restrict__ out, int ld_out, float* __restrict__ partials, int H, int Hkv, int dk, int dv,
                       float scale, int window, float out_scale, int n_split, float softcap, int keep_first,
                       const float* __restrict__ sink, const float* __restrict__ gate, int ld_gate, int* __restrict__ dev_err) {
    constexpr int KS = DKP + 8, VS = DVP + 8;       // row strides in elements: 16 bytes of padding keep ldmatrix off bank conflicts
    constexpr int WKEYS = DEC ? WM_BK / WM_WARPS : WM_BK;      // keys of a tile that one warp takes
    constexpr int NT_S = WKEYS / 8, NT_O = DVP / 8, KS_QK = DKP / 16, KS_PV = WKEYS / 16;
    constexpr int QCH = DKP / 8, VCH = DVP / 8;     // 16-byte pieces of a row
    constexpr int QROWS = DEC ? 16 : WM_ROWS;       // rows of queries that shared memory holds
    extern __shared__ __align__(16) unsigned char wm_raw[];
    __nv_bfloat16* q_tile = reinterpret_cast<__nv_bfloat16*>(wm_raw);            // [QROWS][KS]
    __nv_bfloat16* k_tiles = q_tile + QROWS * KS;                                // [NST][64][KS]
    __nv_bfloat16* v_tiles = k_tiles + NST * WM_BK * KS;                         // [NST][64][VS]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int qt = blockIdx.x / n_split, part = blockIdx.x % n_split, hk = blockIdx.y, seq = blockIdx.z;
    pdl_wait();
    pdl_launch_dependents();
    const int R = H / Hkv, TPT = WM_ROWS / R;       // query heads a key/value head serves; tokens of a tile
    const int row0 = seq_start[seq], n_new = seq_start[seq + 1] - row0;
    const int slot = seq_slot[seq];
    if (slot < 0 || qt * TPT >= n_new) return;      // uniform over the CTA
    const int pos0 = seq_pos0[seq];
    const int n_tok = min(TPT, n_new - qt * TPT);   // tokens of this tile
    const int q_first = pos0 + qt * TPT, q_last = q_first + n_tok - 1;
    const int kt_first = (window > 0) ? max(0, q_first - window + 1) / WM_BK : 0;
    // tiles of kept first keys that the window's tiles do not cover come first in the list: list entry j is tile j for
    // j < n_keep_t, else tile kt_first + j − n_keep_t
    const int n_keep_t = (window > 0 && keep_first > 0) ? min(kt_first, (keep_first + WM_BK - 1) / WM_BK) : 0;
    const int n_kt_all = n_keep_t + q_last / WM_BK - kt_first + 1;
    const int n_kt = (n_kt_all - part + n_split - 1) / n_split;                  // this part's tiles: part, part + n_split, …
    auto tile_of = [&](int i) { const int j = part + i * n_split; return j < n_keep_t ? j : kt_first + j - n_keep_t; };
    const int* table = block_table + (size_t)slot * max_blocks;
    const int n_exist = pos0 + n_new;               // keys of the sequence that the cache holds

    auto load_kv = [&](int i) {                     // all threads: key/value tile number i of this CTA into stage i % NST
        const int kt = tile_of(i);
        const int blk = table[kt];
        __nv_bfloat16* kd = k_tiles + (i % NST) * WM_BK * KS;
        __nv_bfloat16* vd = v_tiles + (i % NST) * WM_BK * VS;
        if (blk < 0 && threadIdx.x == 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
        const int valid = n_exist - kt * WM_BK;     // rows of the tile that hold a key of this sequence
        const __nv_bfloat16* ks = Kc + ((size_t)max(blk, 0) * Hkv + hk) * WM_BK * dk;
        const __nv_bfloat16* vs = Vc + ((size_t)max(blk, 0) * Hkv + hk) * WM_BK * dv;
        for (int idx = threadIdx.x; idx < WM_BK * QCH; idx += WM_WARPS * 32) {
            const int r = idx / QCH, ch = idx - r * QCH;
            if (blk >= 0 && r < valid && ch * 8 < dk) cp_async16(kd + r * KS + ch * 8, ks + (size_t)r * dk + ch * 8);
            else *reinterpret_cast<uint4*>(kd + r * KS + ch * 8) = make_uint4(0, 0, 0, 0);
        }
        for (int idx = threadIdx.x; idx < WM_BK * VCH; idx += WM_WARPS * 32) {
            const int r = idx / VCH, ch = idx - r * VCH;
            if (blk >= 0 && r < valid && ch * 8 < dv) cp_async16(vd + r * VS + ch * 8, vs + (size_t)r * dv + ch * 8);
            else *reinterpret_cast<uint4*>(vd + r * VS + ch * 8) = make_uint4(0, 0, 0, 0);
        }
    };
    // the rows' queries: row r is token r / R of the tile and query head hk·R + r % R
    for (int idx = threadIdx.x; idx < QROWS * QCH; idx += WM_WARPS * 32) {
        const int r = idx / QCH, ch = idx - r * QCH;
        const int ti = r / R;
        if (ti < n_tok && ch * 8 < dk)
            cp_async16(q_tile + r * KS + ch * 8, q + (size_t)(row0 + qt * TPT + ti) * ldq + (size_t)(hk * R + r % R) * dk + ch * 8);
        else
            *reinterpret_cast<uint4*>(q_tile + r * KS + ch * 8) = make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < NST - 1; ++i) {             // (the queries belong to the first group)
        if (i < n_kt) load_kv(i);
        cp_commit();
    }

    const int wrow = DEC ? 0 : warp * 16, wkey = DEC ? warp * WKEYS : 0;          // this warp's first row and first key of a tile
    const bool active = wrow < n_tok * R;           // warps whose 16 rows hold no token only help to load
    uint32_t qf[KS_QK][4];
    float o[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float sl2 = scale * 1.4426950408889634f;  // scores are kept in units of log2(e)
    const float cap2 = softcap * 1.4426950408889634f, cap_in = softcap > 0.f ? 2.f / softcap : 0.f;   // (v · cap_in = 2 x log2e / c)
    const int lr[2] = {wrow + g, wrow + g + 8};                                  // this thread's two rows of the tile
    const int q_row[2] = {q_first + lr[0] / R, q_first + lr[1] / R};             // … and their positions

    for (int i = 0; i < n_kt; ++i) {
        cp_wait<NST - 2>();                         // everything but the newest NST − 2 groups has landed: tile i (and the queries)
        __syncthreads();                            // … for every thread, and every warp is done with tile i − 1
        if (i + NST - 1 < n_kt) load_kv(i + NST - 1);   // into the stage of tile i − 1
        cp_commit();                                // (an empty group keeps the count of groups the same for every pass)
        if (i == 0 && active) {
            const uint32_t qb = wsm(q_tile);
#pragma unroll
            for (int ks = 0; ks < KS_QK; ++ks)
                w_ldsm_x4(qb + ((wrow + (lane & 15)) * KS + ks * 16 + (lane >> 4) * 8) * 2, qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
        }
        if (active) {
            const int k_base = tile_of(i) * WM_BK;
            const uint32_t kb = wsm(k_tiles + (i % NST) * WM_BK * KS), vb = wsm(v_tiles + (i % NST) * WM_BK * VS);
            float s[NT_S][4];
#pragma unroll
            for (int j = 0; j < NT_S; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < KS_QK; ks += 2) {
#pragma unroll
                for (int j = 0; j < NT_S; ++j) {
                    // matrices: (keys 8j…, k-step ks: low, high half), (same keys, k-step ks + 1: low, high half)
                    uint32_t b0, b1, b2, b3;
                    w_ldsm_x4(kb + ((wkey + j * 8 + (lane & 7)) * KS + ks * 16 + (lane >> 3) * 8) * 2, b0, b1, b2, b3);
                    w_mma16816(s[j], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                    w_mma16816(s[j], qf[ks + 1][0], qf[ks + 1][1], qf[ks + 1][2], qf[ks + 1][3], b2, b3);
                }
            }
            const bool need_mask = window > 0 || (k_base + WM_BK - 1 > q_first);
            float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
            for (int j = 0; j < NT_S; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = e >> 1;
                    float v = s[j][e] * sl2;
                    if (softcap > 0.f)      // c · tanh(x / c) = c · (1 − 2 / (2^(2x log2e / c) + 1)), in units of log2 e
                        v = cap2 * (1.f - __fdividef(2.f, exp2f(v * cap_in) + 1.f));
                    if (need_mask) {
                        const int key = k_base + wkey + j * 8 + 2 * t + (e & 1);
                        if (key > q_row[r] || (window > 0 && key <= q_row[r] - window && key >= keep_first)) v = -INFINITY;
                    }
                    s[j][e] = v;
                    m_new[r] = fmaxf(m_new[r], v);
                }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
                m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
            }
            float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
            for (int r = 0; r < 2; ++r) corr[r] = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - m_new[r]);
#pragma unroll
            for (int j = 0; j < NT_S; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = e >> 1;
                    // (the weights are rounded to bfloat16 for the output product; their sum is taken of the rounded values)
                    const float p = (m_new[r] == -INFINITY) ? 0.f : __bfloat162float(__float2bfloat16_rn(exp2f(s[j][e] - m_new[r])));
                    s[j][e] = p;
                    sum[r] += p;
                }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
                sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
                l_run[r] = l_run[r] * corr[r] + sum[r];
                m_run[r] = m_new[r];
            }
#pragma unroll
            for (int j = 0; j < NT_O; ++j) { o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1]; }
#pragma unroll
            for (int kk = 0; kk < KS_PV; ++kk) {
                const uint32_t a0 = w_pack_bf16(s[2 * kk][0], s[2 * kk][1]), a1 = w_pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                const uint32_t a2 = w_pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = w_pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int j = 0; j < NT_O; j += 2) {
                    // transposed loads: (keys 16kk…+7, columns 8j…), (keys +8…, same columns), then the same for columns 8(j+1)…
                    uint32_t b0, b1, b2, b3;
                    w_ldsm_x4_trans(vb + ((wkey + kk * 16 + (lane & 15)) * VS + (j + (lane >> 4)) * 8) * 2, b0, b1, b2, b3);
                    w_mma16816(o[j], a0, a1, a2, a3, b0, b1);
                    w_mma16816(o[j + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
    }
    cp_wait<0>();
    if (DEC) {
        // the warps' sums over their keys meet in shared memory (the tiles are done with): [warp][row][DVP + 2]
        float* mg = reinterpret_cast<float*>(wm_raw);
        constexpr int MS = DVP + 2;
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float* dst = mg + ((size_t)warp * 16 + lr[r]) * MS;
#pragma unroll
            for (int j = 0; j < NT_O; ++j) { dst[j * 8 + 2 * t] = o[j][2 * r]; dst[j * 8 + 2 * t + 1] = o[j][2 * r + 1]; }
            if (t == 0) { dst[DVP] = m_run[r]; dst[DVP + 1] = l_run[r]; }
        }
        __syncthreads();
        const int n_rows = n_tok * R;
        for (int idx = threadIdx.x; idx < n_rows * (dv + 1); idx += WM_WARPS * 32) {
            const int row_l = idx / (dv + 1), c = idx - row_l * (dv + 1);       // column dv: the row's maximum and denominator
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < WM_WARPS; ++w) M = fmaxf(M, mg[((size_t)w * 16 + row_l) * MS + DVP]);
            float acc = 0.f, L = 0.f;
#pragma unroll
            for (int w = 0; w < WM_WARPS; ++w) {
                const float* src = mg + ((size_t)w * 16 + row_l) * MS;
                const float f = (src[DVP] == -INFINITY) ? 0.f : exp2f(src[DVP] - M);
                L = fmaf(src[DVP + 1], f, L);
                if (c < dv) acc = fmaf(src[c], f, acc);
            }
            const int row = row0 + qt * TPT + row_l / R, h = hk * R + row_l % R;
            if (n_split == 1) {
                if (sink != nullptr) {               // exp(sink) joins the denominator
                    const float sk = sink[h] * 1.4426950408889634f, M2 = fmaxf(M, sk);
                    const float f = (M == -INFINITY) ? 0.f : exp2f(M - M2);
                    L = L * f + exp2f(sk - M2);
                    acc *= f;
                }
                const float gf = gate != nullptr ? sigmoid_f(gate[(size_t)row * ld_gate + h]) : 1.f;
                if (c < dv) out[(size_t)row * ld_out + (size_t)h * dv + c] = __float2bfloat16_rn(L > 0.f ? acc * (gf * out_scale / L) : 0.f);
            } else {
                float* dst = partials + (((size_t)row * H + h) * n_split + part) * (dv + 2);
                if (c < dv) dst[c] = acc;
                else { dst[dv] = M; dst[dv + 1] = L; }
            }
        }
        return;
    }
    if (!active) return;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int ti = lr[r] / R;
        if (ti >= n_tok) continue;
        const int row = row0 + qt * TPT + ti, h = hk * R + lr[r] % R;
        if (n_split == 1) {
            float fo = 1.f;
            if (sink != nullptr) {                   // exp(sink) joins the denominator
                const float sk = sink[h] * 1.4426950408889634f, M2 = fmaxf(m_run[r], sk);
                fo = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - M2);
                l_run[r] = l_run[r] * fo + exp2f(sk - M2);
            }
            if (gate != nullptr) fo *= sigmoid_f(gate[(size_t)row * ld_gate + h]);
            const float inv = (l_run[r] > 0.f) ? fo * out_scale / l_run[r] : 0.f;
            __nv_bfloat16* dst = out + (size_t)row * ld_out + (size_t)h * dv + 2 * t;
#pragma unroll
            for (int j = 0; j < NT_O; ++j)
                if (j * 8 + 2 * t < dv) *reinterpret_cast<uint32_t*>(dst + j * 8) = w_pack_bf16(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
        } else {
            float* dst = partials + (((size_t)row * H + h) * n_split + part) * (dv + 2);
#pragma unroll
            for (int j = 0; j < NT_O; ++j)
                if (j * 8 + 2 * t < dv) { dst[j * 8 + 2 * t] = o[j][2 * r]; dst[j * 8 + 2 * t + 1] = o[j][2 * r + 1]; }
            if (t == 0) { dst[dv] = m_run[r]; dst[dv + 1] = l_run[r]; }
        }
    }
}

// The parts of a decode step's contexts: out[row][h] = out_scale · Σ_p o_p 2^(m_p − M) / Σ_p l_p 2^(m_p − M), in the
// order of the parts.  A part that saw no key has l = 0.
__global__ void __launch_bounds__(128)
attn_window_merge_kernel(const float* __restrict__ partials, const int* __restrict__ seq_slot, __nv_bfloat16* __restrict__ out,
                         int ld_out, int H, int dv, int n_split, float out_scale, const float* __restrict__ sink,
                         const float* __restrict__ gate, int ld_gate) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x, h = blockIdx.y;
    if (seq_slot[row] < 0) return;
    const float* p = partials + ((size_t)row * H + h) * n_split * (dv + 2);
    float M = -INFINITY;
    for (int s = 0; s < n_split; ++s)
        if (p[s * (dv + 2) + dv + 1] > 0.f) M = fmaxf(M, p[s * (dv + 2) + dv]);
    const float sk = sink != nullptr ? sink[h] * 1.4426950408889634f : -INFINITY;
    M = fmaxf(M, sk);
    float L = sink != nullptr ? exp2f(sk - M) : 0.f;
    for (int s = 0; s < n_split; ++s) {
        const float l = p[s * (dv + 2) + dv + 1];
        if (l > 0.f) L += l * exp2f(p[s * (dv + 2) + dv] - M);
    }
    const float inv = (L > 0.f ? out_scale / L : 0.f) * (gate != nullptr ? sigmoid_f(gate[(size_t)row * ld_gate + h]) : 1.f);
    for (int c = threadIdx.x; c < dv; c += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_split; ++s)
            if (p[s * (dv + 2) + dv + 1] > 0.f) acc += p[s * (dv + 2) + c] * exp2f(p[s * (dv + 2) + dv] - M);
        out[(size_t)row * ld_out + (size_t)h * dv + c] = __float2bfloat16_rn(acc * inv);
    }
}

template <int DKP, int DVP, bool DEC>
int launch_window_mma(const void* q, int ldq, const void* Kc, const void* Vc, const int* block_table, int max_blocks,
                      const int* seq_slot, const int* seq_start, const int* seq_pos0, void* out, int ld_out, float* partials,
                      int n_seqs, int max_new, int H, int Hkv, int dk, int dv, float scale, int window, float out_scale, int n_split,
                      float softcap, int keep_first, const float* sink, const float* gate, int ld_gate, int* dev_err, cudaStream_t stream) {
    // stages of a decode step: as many as leave room for two or three CTAs an SM
    constexpr int NST = DEC ? (DKP + DVP <= 160 ? 4 : DKP + DVP <= 224 ? 3 : 2) : 2;
    const size_t smem = (size_t)((DEC ? 16 : 64) * (DKP + 8) + NST * 64 * (DKP + 8) + NST * 64 * (DVP + 8)) * 2;
    auto kern = attn_window_mma_kernel<DKP, DVP, DEC, NST>;
    static bool raised = false;
    if (!raised && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_window_mma: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        raised = true;
    }
    const int tpt = WM_ROWS / (H / Hkv);
    dim3 grid(((max_new + tpt - 1) / tpt) * n_split, Hkv, n_seqs);
    cudaError_t e = launch_chained(kern, grid, dim3(WM_WARPS * 32), smem, stream, (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)Kc,
                                   (const __nv_bfloat16*)Vc, block_table, max_blocks, seq_slot, seq_start, seq_pos0,
                                   (__nv_bfloat16*)out, ld_out, partials, H, Hkv, dk, dv, scale, window, out_scale, n_split, softcap,
                                   keep_first, sink, gate, ld_gate, dev_err);
    if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_window_mma: %s", cudaGetErrorString(e));
    return vlrf_check_launch("attn_window_mma");
}
}  // namespace

// Whether the tensor-core kernel takes these sizes (bfloat16 only): head sizes multiples of 8 up to 128, at most 16
// query heads a key/value head, cache blocks of 64 tokens, rows on 16-byte boundaries.
extern "C" int vlrf_attn_window_mma_takes(int H, int Hkv, int dk, int dv, int BT, int ldq, int ld_out) {
    return (H > 0 && Hkv > 0 && H % Hkv == 0 && H / Hkv <= 16 && dk > 0 && dv > 0 && dk % 8 == 0 && dv % 8 == 0 && dk <= 128 &&
            dv <= 128 && BT == WM_BK && ldq % 8 == 0 && ld_out % 2 == 0) ? 1 : 0;
}

extern "C" int vlrf_attn_window_mma_ex(const void* q, int ldq, const void* Kc, const void* Vc, const int* block_table, int max_blocks,
                                       const int* seq_slot, const int* seq_start, const int* seq_pos0, void* out, int ld_out,
                                       float* partials, int n_seqs, int max_new, int H, int Hkv, int dk, int dv, int BT, float scale,
                                       int window, float out_scale, int n_split, float softcap, int keep_first, const float* sink,
                                       const float* gate, int ld_gate, int* dev_err, cudaStream_t stream) {
    VLRF_REQUIRE(vlrf_attn_window_mma_takes(H, Hkv, dk, dv, BT, ldq, ld_out), "attn_window_mma: heads %d/%d, sizes %d and %d, block %d are not taken",
                 H, Hkv, dk, dv, BT);
    VLRF_REQUIRE(n_seqs >= 0 && max_new >= 0 && max_blocks > 0 && window >= 0 && dev_err != nullptr, "attn_window_mma: bad arguments");
    VLRF_REQUIRE(keep_first >= 0 && softcap >= 0.f && (gate == nullptr || ld_gate >= H), "attn_window_mma: negative kept tokens or cap, or gate rows shorter than the heads");
    VLRF_REQUIRE(n_seqs <= 65535 && Hkv <= 65535, "attn_window_mma: too many sequences or heads for one launch");
    VLRF_REQUIRE(n_split >= 1 && (n_split == 1 || (max_new == 1 && partials != nullptr)),
                 "attn_window_mma: contexts are cut into parts in decode steps only, and the parts need scratch");
    VLRF_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 3) == 0, "attn_window_mma: misaligned rows");
    if (n_seqs == 0 || max_new == 0) return VLRF_OK;
    const int kp = dk <= 32 ? 32 : dk <= 64 ? 64 : dk <= 96 ? 96 : 128, vp = dv <= 32 ? 32 : dv <= 64 ? 64 : dv <= 96 ? 96 : 128;
    int st = VLRF_ERR_UNSUPPORTED;
    const bool dec = max_new == 1 && H / Hkv <= 16;            // every tile holds one token's heads: the warps deal the keys
#define GO(A, B) if (kp == A && vp == B) st = dec ? launch_window_mma<A, B, true>(q, ldq, Kc, Vc, block_table, max_blocks, seq_slot, seq_start, seq_pos0, \
        out, ld_out, partials, n_seqs, max_new, H, Hkv, dk, dv, scale, window, out_scale, n_split, softcap, keep_first, sink, gate, ld_gate, dev_err, stream) \
        : launch_window_mma<A, B, false>(q, ldq, Kc, Vc, block_table, max_blocks, seq_slot, seq_start, seq_pos0, \
        out, ld_out, partials, n_seqs, max_new, H, Hkv, dk, dv, scale, window, out_scale, n_split, softcap, keep_first, sink, gate, ld_gate, dev_err, stream);
    GO(32, 32) GO(32, 64) GO(32, 96) GO(32, 128) GO(64, 32) GO(64, 64) GO(64, 96) GO(64, 128)
    GO(96, 32) GO(96, 64) GO(96, 96) GO(96, 128) GO(128, 32) GO(128, 64) GO(128, 96) GO(128, 128)
#undef GO
    if (st != VLRF_OK) return st;
    if (n_split > 1) {
        launch_chained(attn_window_merge_kernel, dim3(n_seqs, H), dim3(128), (size_t)0, stream, (const float*)partials, seq_slot,
                       (__nv_bfloat16*)out, ld_out, H, dv, n_split, out_scale, sink, gate, ld_gate);
        return vlrf_check_launch("attn_window_merge");
    }
    return VLRF_OK;
}

extern "C" int vlrf_attn_window_mma(const void* q, int ldq, const void* Kc, const void* Vc, const int* block_table, int max_blocks,
                                    const int* seq_slot, const int* seq_start, const int* seq_pos0, void* out, int ld_out,
                                    float* partials, int n_seqs, int max_new, int H, int Hkv, int dk, int dv, int BT, float scale,
                                    int window, float out_scale, int n_split, int* dev_err, cudaStream_t stream) {
    return vlrf_attn_window_mma_ex(q, ldq, Kc, Vc, block_table, max_blocks, seq_slot, seq_start, seq_pos0, out, ld_out, partials,
                                   n_seqs, max_new, H, Hkv, dk, dv, BT, scale, window, out_scale, n_split, 0.f, 0, nullptr, nullptr, 0,
                                   dev_err, stream);
}
