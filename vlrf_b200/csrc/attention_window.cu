// Attention whose keys and values have sizes of their own, over a paged cache, with rotated queries and keys.
//
// The cache of one layer is K [block][kv_head][BT][dk] and V [block][kv_head][BT][dv] (dk: the size of queries and
// keys, dv: of values; they need not be equal).  Query head h reads key/value head h / (H / Hkv).  A window w > 0
// hides keys at or before position − w; w = 0 is plain causal attention.
//
// qkv_rope_append: the float32 result of a layer's input product holds, per token, the queries (H·dk columns at
//   q_off), keys (Hkv·dk at k_off) and values (Hkv·dv at v_off), biases included.  Of every query and key head the
//   first `rot` entries are rotated by the token's position: entry i pairs with entry i + rot/2, and the pair (a, b)
//   becomes (a cos t − b sin t, b cos t + a sin t) with t = position · freq[i] (float32; freq holds whatever scaling
//   of the frequencies the model asks for).  Queries go to a matrix of their own in the activation dtype, keys and
//   values into the cache at (slot, position).
// qkv_norm_rope_append: the same with what some designs put between the product and the rotation, each a parameter:
//   an RMS norm of queries and of keys (norm 1: every head by itself, one weight vector of dk entries shared by the
//   heads; norm 2: all heads of the projection as one row, weights of H·dk and Hkv·dk entries; x / sqrt(mean(x²) + eps)
//   · w in float32), the pairing of rotated entries (pairing 1: entry 2i with entry 2i + 1), a factor on every cosine
//   and sine (`magnitude`), and values that are the keys as projected (v_off = k_off: they are read before norm and
//   rotation).  A layer that reads another layer's cache has no key or value columns (write_cache 0).
// attn_window: one warp per (token, head) walks the visible keys of the token's slot in chunks of 32 with an online
//   softmax in float32; any mix of prompt tokens and single tokens.  Every size (dk, dv ≤ 256) is taken; the 32-bit
//   path's attention, and the fallback of the bfloat16 path.  The result is multiplied by out_scale (a mixer that
//   sums several branches puts a branch's weight there) and written at a column offset of wider rows.
//   Further parameters (attn_window_ex): softcap c > 0 squashes every score to c · tanh(score / c) after the scale;
//   keep_first n > 0 lets every query also see the keys at positions below n, whatever the window (they keep their
//   positions); gate (float32 [T][ld_gate], a logit per query head) multiplies head h's result by sigmoid(gate[t][h]);
//   sink (one float32 a query head) adds the term exp(sink_h) to the softmax's denominator and nothing to its numerator.
#include "common.cuh"

namespace {
constexpr int AW_WARPS = 4;
constexpr int AW_MAX = 256;

template <typename ET>
__global__ void __launch_bounds__(128)
qkv_rope_append_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off, const float* __restrict__ freq,
                       int rot, ET* __restrict__ q_out, int ldq, ET* __restrict__ Kc, ET* __restrict__ Vc,
                       const int* __restrict__ block_table, int max_blocks, const int* __restrict__ tok_slot,
                       const int* __restrict__ tok_pos, int H, int Hkv, int dk, int dv, int BT, int write_cache,
                       int norm, const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps, int pairing,
                       float magnitude, int* __restrict__ dev_err) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int slot = tok_slot[t];
    if (slot < 0) return;  // padding row (the whole CTA leaves: no barrier is missed)
    const int pos = tok_pos[t];
    const float* row = proj + (size_t)t * ld;
    const int half = rot / 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // the token's cosines and sines once, for all heads: [half] each; then 1 / rms of every normed head: [H + Hkv]
    extern __shared__ float cs_sm[];
    float* inv_sm = cs_sm + rot;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cn;
        sincosf((float)pos * freq[i], &sn, &cn);
        cs_sm[i] = cn * magnitude;
        cs_sm[half + i] = sn * magnitude;
    }
    const int n_kh = write_cache ? Hkv : 0;
    // Heads normed by themselves, of an even size up to 256: a warp takes a head whole (below), with its entries in registers
    const bool warp_heads = norm == 1 && (dk & 1) == 0 && dk <= 256;
    if (warp_heads) {
    } else if (norm == 1) {
        for (int h = warp; h < H + n_kh; h += 4) {
            const float* head = h < H ? row + q_off + h * dk : row + k_off + (h - H) * dk;
            float ss = 0.f;
            for (int c = lane; c < dk; c += 32) ss = fmaf(head[c], head[c], ss);
            ss = warp_sum(ss);
            if (lane == 0) inv_sm[h] = 1.f / sqrtf(ss / (float)dk + eps);
        }
    } else if (norm == 2) {
        __shared__ float red[2][4];
        float sq = 0.f, sk = 0.f;
        for (int i = threadIdx.x; i < H * dk; i += blockDim.x) sq = fmaf(row[q_off + i], row[q_off + i], sq);
        for (int i = threadIdx.x; i < n_kh * dk; i += blockDim.x) sk = fmaf(row[k_off + i], row[k_off + i], sk);
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        if (lane == 0) { red[0][warp] = sq; red[1][warp] = sk; }
        __syncthreads();
        if (threadIdx.x < H + n_kh) {
            const bool isq = (int)threadIdx.x < H;
            const float tot = red[isq ? 0 : 1][0] + red[isq ? 0 : 1][1] + red[isq ? 0 : 1][2] + red[isq ? 0 : 1][3];
            inv_sm[threadIdx.x] = 1.f / sqrtf(tot / (float)((isq ? H : Hkv) * dk) + eps);
        }
        for (int h = threadIdx.x + 128; h < H + n_kh; h += 128) {          // (more heads than threads)
            const bool isq = h < H;
            const float tot = red[isq ? 0 : 1][0] + red[isq ? 0 : 1][1] + red[isq ? 0 : 1][2] + red[isq ? 0 : 1][3];
            inv_sm[h] = 1.f / sqrtf(tot / (float)((isq ? H : Hkv) * dk) + eps);
        }
    }
    __syncthreads();
    // entry c of a head after the norm: w points at the head's weights (norm 1: the shared vector; norm 2: its own part)
    auto normed = [&](const float* head, const float* w, float inv, int c) -> float {
        return norm ? head[c] * inv * w[c] : head[c];
    };
    auto rotated = [&](const float* head, const float* w, float inv, int c) -> float {
        const float x = normed(head, w, inv, c);
        if (c >= rot) return x;
        if (pairing == 1) {                                   // entry 2i with entry 2i + 1
            const int i = c >> 1;
            const float y = normed(head, w, inv, c ^ 1);
            return (c & 1) ? x * cs_sm[i] + y * cs_sm[half + i] : x * cs_sm[i] - y * cs_sm[half + i];
        }
        if (c < half) return x * cs_sm[c] - normed(head, w, inv, c + half) * cs_sm[half + c];
        return x * cs_sm[c - half] + normed(head, w, inv, c - half) * cs_sm[c];
    };
    if (warp_heads) {
        // A warp per head, queries and keys alike: a lane holds up to four pairs of entries (the two of a rotation, or two
        // neighbours behind the rotated ones), the head's sum of squares is a sum over the warp, and norm, rotation and
        // store follow from the registers: every entry is read once and no warp waits for another.
        const int hd2 = dk / 2;
        int blk = -1;
        if (write_cache) {
            const int bi = pos / BT;
            blk = (pos >= 0 && bi < max_blocks) ? block_table[(size_t)slot * max_blocks + bi] : -1;
            if (blk < 0 && threadIdx.x == 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
        }
        const int n_all = H + (blk >= 0 ? Hkv : 0);
        for (int h = warp; h < n_all; h += 4) {
            const bool isq = h < H;
            const float* head = isq ? row + q_off + h * dk : row + k_off + (h - H) * dk;
            const float* w = isq ? q_norm : k_norm;
            ET* dst = isq ? q_out + (size_t)t * ldq + h * dk : Kc + (((size_t)blk * Hkv + (h - H)) * BT + (pos % BT)) * dk;
            float xa[4], xb[4];
            int ia[4], ib[4];
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int u = lane + 32 * j;
                xa[j] = xb[j] = 0.f;
                ia[j] = ib[j] = 0;
                if (u < hd2) {
                    const bool turns = u < half;
                    ia[j] = turns ? (pairing == 1 ? 2 * u : u) : rot + 2 * (u - half);
                    ib[j] = turns ? (pairing == 1 ? 2 * u + 1 : u + half) : ia[j] + 1;
                    xa[j] = head[ia[j]];
                    xb[j] = head[ib[j]];
                    ss = fmaf(xa[j], xa[j], fmaf(xb[j], xb[j], ss));
                }
            }
            ss = warp_sum(ss);
            const float inv = 1.f / sqrtf(ss / (float)dk + eps);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int u = lane + 32 * j;
                if (u < hd2) {
                    const float na = xa[j] * inv * w[ia[j]], nb = xb[j] * inv * w[ib[j]];
                    const bool turns = u < half;
                    ElemIO<ET>::store(dst + ia[j], turns ? na * cs_sm[u] - nb * cs_sm[half + u] : na);
                    ElemIO<ET>::store(dst + ib[j], turns ? nb * cs_sm[u] + na * cs_sm[half + u] : nb);
                }
            }
        }
        if (blk < 0) return;
        for (int i = threadIdx.x; i < Hkv * dv; i += blockDim.x) {
            const int h = i / dv, c = i - h * dv;
            ElemIO<ET>::store(Vc + (((size_t)blk * Hkv + h) * BT + (pos % BT)) * dv + c, row[v_off + i]);
        }
        return;
    }
    // Heads of an even size: a thread takes a pair of entries at a time, the two of a rotation (entries 2u and 2u + 1, or u
    // and u + rot/2) or two neighbours behind the rotated ones, so every entry is read and normed once.
    const int hd = dk / 2;
    auto pair_of = [&](const float* head, const float* w, float inv, int u, int& ia, int& ib, float& oa, float& ob) {
        const bool turns = u < half;
        ia = turns ? (pairing == 1 ? 2 * u : u) : rot + 2 * (u - half);
        ib = turns ? (pairing == 1 ? 2 * u + 1 : u + half) : ia + 1;
        const float xa = normed(head, w, inv, ia), xb = normed(head, w, inv, ib);
        oa = turns ? xa * cs_sm[u] - xb * cs_sm[half + u] : xa;
        ob = turns ? xb * cs_sm[u] + xa * cs_sm[half + u] : xb;
    };
    const bool by_pairs = (dk & 1) == 0;
    if (by_pairs) {
        for (int i = threadIdx.x; i < H * hd; i += blockDim.x) {
            const int h = i / hd, u = i - h * hd;
            int ia, ib;
            float oa, ob;
            pair_of(row + q_off + h * dk, norm == 2 ? q_norm + h * dk : q_norm, norm ? inv_sm[h] : 1.f, u, ia, ib, oa, ob);
            ET* dst = q_out + (size_t)t * ldq + h * dk;
            ElemIO<ET>::store(dst + ia, oa);
            ElemIO<ET>::store(dst + ib, ob);
        }
    } else {
        for (int i = threadIdx.x; i < H * dk; i += blockDim.x) {
            const int h = i / dk, c = i - h * dk;
            const float* w = norm == 2 ? q_norm + h * dk : q_norm;
            ElemIO<ET>::store(q_out + (size_t)t * ldq + i, rotated(row + q_off + h * dk, w, norm ? inv_sm[h] : 1.f, c));
        }
    }
    if (!write_cache) return;
    const int bi = pos / BT;
    const int blk = (pos >= 0 && bi < max_blocks) ? block_table[(size_t)slot * max_blocks + bi] : -1;
    if (blk < 0) {
        if (threadIdx.x == 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
        return;
    }
    if (by_pairs) {
        for (int i = threadIdx.x; i < Hkv * hd; i += blockDim.x) {
            const int h = i / hd, u = i - h * hd;
            int ia, ib;
            float oa, ob;
            pair_of(row + k_off + h * dk, norm == 2 ? k_norm + h * dk : k_norm, norm ? inv_sm[H + h] : 1.f, u, ia, ib, oa, ob);
            ET* dst = Kc + (((size_t)blk * Hkv + h) * BT + (pos % BT)) * dk;
            ElemIO<ET>::store(dst + ia, oa);
            ElemIO<ET>::store(dst + ib, ob);
        }
    } else {
        for (int i = threadIdx.x; i < Hkv * dk; i += blockDim.x) {
            const int h = i / dk, c = i - h * dk;
            const float* w = norm == 2 ? k_norm + h * dk : k_norm;
            ElemIO<ET>::store(Kc + (((size_t)blk * Hkv + h) * BT + (pos % BT)) * dk + c,
                              rotated(row + k_off + h * dk, w, norm ? inv_sm[H + h] : 1.f, c));
        }
    }
    for (int i = threadIdx.x; i < Hkv * dv; i += blockDim.x) {
        const int h = i / dv, c = i - h * dv;
        ElemIO<ET>::store(Vc + (((size_t)blk * Hkv + h) * BT + (pos % BT)) * dv + c, row[v_off + i]);
    }
}

template <typename ET>
__global__ void __launch_bounds__(AW_WARPS * 32)
attn_window_kernel(const ET* __restrict__ q_in, int ldq, const ET* __restrict__ Kc, const ET* __restrict__ Vc,
                   const int* __restrict__ block_table, int max_blocks, const int* __restrict__ tok_slot,
                   const int* __restrict__ tok_pos, ET* __restrict__ out, int ld_out, int H, int Hkv, int dk, int dv, int BT,
                   float scale, int window, float out_scale, float softcap, int keep_first, const float* __restrict__ sink,
                   const float* __restrict__ gate, int ld_gate, int* __restrict__ dev_err) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float q_sm[];  // [AW_WARPS][dk]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int h = blockIdx.y * AW_WARPS + warp;
    const int slot = tok_slot[t];
    if (h >= H || slot < 0) return;  // whole warp leaves together; no block-wide barrier below
    const int pos = tok_pos[t];
    const int hk = h / (H / Hkv);
    float* q = q_sm + warp * dk;
    const ET* qsrc = q_in + (size_t)t * ldq + (size_t)h * dk;
    for (int i = lane; i < dk; i += 32) q[i] = ElemIO<ET>::load(qsrc + i) * scale;
    __syncwarp();

    float acc[AW_MAX / 32];
#pragma unroll
    for (int i = 0; i < AW_MAX / 32; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int first = (window > 0) ? max(0, pos - window + 1) : 0;
    const int* table = block_table + (size_t)slot * max_blocks;
    bool lost = false;

    // the keys kept whatever the window (positions below keep_first that the window no longer reaches), then the window
    const int n_kept = (window > 0 && keep_first > 0) ? min(keep_first, first) : 0;
    const int kept_end = ((n_kept + 31) / 32) * 32, win_begin = (first / 32) * 32;
    for (int k0 = n_kept > 0 ? 0 : win_begin; k0 <= pos; k0 += 32) {
        if (k0 >= kept_end && k0 < win_begin) { k0 = win_begin - 32; continue; }   // (the chunks between the two ranges)
        const int blk = table[k0 / BT];
        if (blk < 0) { lost = true; break; }
        const size_t kbase = (((size_t)blk * Hkv + hk) * BT + (k0 % BT)) * dk;
        const size_t vbase = (((size_t)blk * Hkv + hk) * BT + (k0 % BT)) * dv;
        const int key = k0 + lane;
        const bool valid = (key >= first || key < n_kept) && key <= pos;
        float s = -INFINITY;
        if (valid) {
            const ET* krow = Kc + kbase + (size_t)lane * dk;
            float dot = 0.f;
            for (int c = 0; c < dk; ++c) dot = fmaf(q[c], ElemIO<ET>::load(krow + c), dot);
            s = softcap > 0.f ? softcap * tanhf(dot / softcap) : dot;
        }
        const float m_new = fmaxf(m, warp_max(s));      // at least one key of the chunk is valid
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < AW_MAX / 32; ++i) acc[i] *= corr;
        const int n_here = min(32, pos - k0 + 1);
        for (int j = 0; j < n_here; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            if (pj == 0.f) continue;  // uniform across the warp
            const ET* vrow = Vc + vbase + (size_t)j * dv;
#pragma unroll
            for (int i = 0; i < AW_MAX / 32; ++i) {
                const int c = i * 32 + lane;
                if (c < dv) acc[i] = fmaf(pj, ElemIO<ET>::load(vrow + c), acc[i]);
            }
        }
        m = m_new;
    }
    if (lost && lane == 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
    if (sink != nullptr) {                               // exp(sink) joins the denominator: no key, no value
        const float sk = sink[h], m_new = fmaxf(m, sk);
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + expf(sk - m_new);
#pragma unroll
        for (int i = 0; i < AW_MAX / 32; ++i) acc[i] *= corr;
    }
    float inv = (l > 0.f) ? out_scale / l : 0.f;
    if (gate != nullptr) inv *= sigmoid_f(gate[(size_t)t * ld_gate + h]);      // a gate per head on the head's result
    ET* dst = out + (size_t)t * ld_out + (size_t)h * dv;
#pragma unroll
    for (int i = 0; i < AW_MAX / 32; ++i) {
        const int c = i * 32 + lane;
        if (c < dv) ElemIO<ET>::store(dst + c, acc[i] * inv);
    }
}
}  // namespace

extern "C" int vlrf_qkv_norm_rope_append(const float* proj, int ld, int q_off, int k_off, int v_off, const float* freq, int rot,
                                         void* q_out, int ldq, void* Kc, void* Vc, int dtype, const int* block_table, int max_blocks,
                                         const int* tok_slot, const int* tok_pos, int T, int H, int Hkv, int dk, int dv, int BT,
                                         int write_cache, int norm, const float* q_norm, const float* k_norm, float eps, int pairing,
                                         float magnitude, int* dev_err, cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && H > 0 && Hkv > 0 && dk > 0 && dv > 0 && BT > 0 && max_blocks > 0, "qkv_rope_append: bad sizes");
    VLRF_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dk, "qkv_rope_append: %d rotated entries of a head of %d", rot, dk);
    VLRF_REQUIRE(rot == 0 || freq != nullptr, "qkv_rope_append: a rotation needs its frequencies");
    VLRF_REQUIRE(q_off >= 0 && q_off + H * dk <= ld && ldq >= H * dk, "qkv_rope_append: columns lie outside the row");
    VLRF_REQUIRE(!write_cache || (k_off >= 0 && v_off >= 0 && k_off + Hkv * dk <= ld && v_off + Hkv * dv <= ld && Kc != nullptr && Vc != nullptr),
                 "qkv_rope_append: key or value columns lie outside the row");
    VLRF_REQUIRE(norm >= 0 && norm <= 2 && (norm == 0 || (q_norm != nullptr && (k_norm != nullptr || !write_cache) && eps > 0.f)),
                 "qkv_rope_append: a norm of queries and keys needs its weights and a positive eps");
    VLRF_REQUIRE(pairing == 0 || pairing == 1, "qkv_rope_append: rotated entries pair by halves (0) or as neighbours (1)");
    VLRF_REQUIRE(dev_err != nullptr, "qkv_rope_append: needs the device error word");
    if (T == 0) return VLRF_OK;
    const size_t smem = (size_t)(rot + H + Hkv) * sizeof(float);
    VLRF_REQUIRE(smem <= 48 * 1024, "qkv_rope_append: %d heads are more than the kernel's shared memory takes", H + Hkv);
    if (dtype == VLRF_F32)
        launch_chained(qkv_rope_append_kernel<float>, dim3(T), dim3(128), smem, stream, proj, ld, q_off, k_off, v_off, freq, rot,
                       (float*)q_out, ldq, (float*)Kc, (float*)Vc, block_table, max_blocks, tok_slot, tok_pos, H, Hkv, dk, dv, BT,
                       write_cache, norm, q_norm, k_norm, eps, pairing, magnitude, dev_err);
    else if (dtype == VLRF_BF16)
        launch_chained(qkv_rope_append_kernel<__nv_bfloat16>, dim3(T), dim3(128), smem, stream, proj, ld, q_off, k_off, v_off, freq,
                       rot, (__nv_bfloat16*)q_out, ldq, (__nv_bfloat16*)Kc, (__nv_bfloat16*)Vc, block_table, max_blocks, tok_slot,
                       tok_pos, H, Hkv, dk, dv, BT, write_cache, norm, q_norm, k_norm, eps, pairing, magnitude, dev_err);
    else
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "qkv_rope_append: unknown dtype %d", dtype);
    return vlrf_check_launch("qkv_rope_append");
}

extern "C" int vlrf_qkv_rope_append(const float* proj, int ld, int q_off, int k_off, int v_off, const float* freq, int rot,
                                    void* q_out, int ldq, void* Kc, void* Vc, int dtype, const int* block_table, int max_blocks,
                                    const int* tok_slot, const int* tok_pos, int T, int H, int Hkv, int dk, int dv, int BT,
                                    int write_cache, int* dev_err, cudaStream_t stream) {
    VLRF_REQUIRE(k_off + Hkv * dk <= ld && v_off + Hkv * dv <= ld, "qkv_rope_append: columns lie outside the row");
    return vlrf_qkv_norm_rope_append(proj, ld, q_off, k_off, v_off, freq, rot, q_out, ldq, Kc, Vc, dtype, block_table, max_blocks,
                                     tok_slot, tok_pos, T, H, Hkv, dk, dv, BT, write_cache, 0, nullptr, nullptr, 0.f, 0, 1.f, dev_err,
                                     stream);
}

extern "C" int vlrf_attn_window_ex(const void* q, int dtype, int ldq, const void* Kc, const void* Vc, const int* block_table,
                                   int max_blocks, const int* tok_slot, const int* tok_pos, void* out, int ld_out, int T, int H,
                                   int Hkv, int dk, int dv, int BT, float scale, int window, float out_scale, float softcap,
                                   int keep_first, const float* sink, const float* gate, int ld_gate, int* dev_err,
                                   cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && H > 0 && Hkv > 0 && max_blocks > 0, "attn_window: bad sizes");
    VLRF_REQUIRE(H % Hkv == 0, "attn_window: %d heads cannot share %d key/value heads", H, Hkv);
    VLRF_REQUIRE(dk > 0 && dk <= AW_MAX && dv > 0 && dv <= AW_MAX, "attn_window: head sizes %d and %d are not in 1…%d", dk, dv, AW_MAX);
    VLRF_REQUIRE(BT % 32 == 0, "attn_window: cache blocks of %d tokens are not a multiple of 32", BT);
    VLRF_REQUIRE(window >= 0 && keep_first >= 0 && softcap >= 0.f, "attn_window: negative window, kept tokens or cap");
    VLRF_REQUIRE(ldq >= H * dk && ld_out >= H * dv && (gate == nullptr || ld_gate >= H), "attn_window: leading sizes are smaller than the rows");
    VLRF_REQUIRE(dev_err != nullptr, "attn_window: needs the device error word");
    if (T == 0) return VLRF_OK;
    dim3 grid(T, (H + AW_WARPS - 1) / AW_WARPS);
    const size_t smem = (size_t)AW_WARPS * dk * sizeof(float);
    if (dtype == VLRF_F32)
        launch_chained(attn_window_kernel<float>, grid, dim3(AW_WARPS * 32), smem, stream, (const float*)q, ldq, (const float*)Kc,
                       (const float*)Vc, block_table, max_blocks, tok_slot, tok_pos, (float*)out, ld_out, H, Hkv, dk, dv, BT, scale,
                       window, out_scale, softcap, keep_first, sink, gate, ld_gate, dev_err);
    else if (dtype == VLRF_BF16)
        launch_chained(attn_window_kernel<__nv_bfloat16>, grid, dim3(AW_WARPS * 32), smem, stream, (const __nv_bfloat16*)q, ldq,
                       (const __nv_bfloat16*)Kc, (const __nv_bfloat16*)Vc, block_table, max_blocks, tok_slot, tok_pos,
                       (__nv_bfloat16*)out, ld_out, H, Hkv, dk, dv, BT, scale, window, out_scale, softcap, keep_first, sink, gate, ld_gate,
                       dev_err);
    else
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "attn_window: unknown dtype %d", dtype);
    return vlrf_check_launch("attn_window");
}

extern "C" int vlrf_attn_window(const void* q, int dtype, int ldq, const void* Kc, const void* Vc, const int* block_table,
                                int max_blocks, const int* tok_slot, const int* tok_pos, void* out, int ld_out, int T, int H,
                                int Hkv, int dk, int dv, int BT, float scale, int window, float out_scale, int* dev_err,
                                cudaStream_t stream) {
    return vlrf_attn_window_ex(q, dtype, ldq, Kc, Vc, block_table, max_blocks, tok_slot, tok_pos, out, ld_out, T, H, Hkv, dk, dv, BT,
                               scale, window, out_scale, 0.f, 0, nullptr, nullptr, 0, dev_err, stream);
}
