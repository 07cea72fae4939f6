// The C interface of libvlrf_b200_kernels.so: every kernel of the library as a plain C function, for callers
// that drive the kernels without Python (the Python package calls exactly these through ctypes).
//
// Conventions, the same for every function (status codes in the manner of the reference's include/api/vlrf.h:32-41):
//   * Pointers are device pointers unless a comment says otherwise; matrices are row-major and contiguous, `ld*` is
//     the distance between rows in elements.  `dtype` arguments are VLRF_F32 or VLRF_BF16.
//   * A function checks its sizes on the host, launches on `stream`, and returns VLRF_OK or a status whose text
//     vlrf_last_error() gives (per thread).  A size that a kernel does not take is refused, never computed wrongly;
//     the *_takes functions say beforehand whether a kernel takes a shape.
//   * Nothing allocates device memory.  Scratch comes from the caller (vlrf_attn_decode_noalloc, declared in
//     attention_decode_noalloc.h, is the one exception: its scratch lies in the library's image).
//   * `dev_err` is one int32 on the device that kernels OR bits into (VLRF_DEVERR_*) instead of faulting: a token id
//     or position out of range is clamped, a token whose cache block is not mapped is skipped, a bounded wait that
//     ran out is recorded.  The caller reads and clears it when it likes.
//   * Kernels are launched with programmatic stream serialization unless vlrf_set_chained_launch(0) was called: a
//     kernel may begin while the one before it on the stream still runs, and waits inside for its completion before
//     it touches what that kernel writes.
//   * The paged cache: K and V of one layer are [n_blocks][Hkv][BT][dh]; block_table is int32 [slots][max_blocks],
//     entry (s, i) the block that holds tokens i·BT … of slot s, or −1; BT is 64 in this library.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VLRF_OK 0
#define VLRF_ERR_INVALID_ARG 1
#define VLRF_ERR_UNSUPPORTED 2
#define VLRF_ERR_CUDA 3

#define VLRF_F32 0
#define VLRF_BF16 1

#define VLRF_ACT_NONE 0
#define VLRF_ACT_GELU_TANH 1
#define VLRF_ACT_GELU_ERF 2
#define VLRF_ACT_RELU2 3          // relu(x)^2
#define VLRF_ACT_LAST_FUSED 3     // the last activation that the products' epilogues take
#define VLRF_ACT_SILU 4           // x * sigmoid(x): vlrf_gate_mul only
#define VLRF_ACT_SIGMOID 5        // vlrf_gate_mul only
#define VLRF_ACT_RELU 6           // max(x, 0): vlrf_gate_mul only

#define VLRF_DEVERR_TOKEN_RANGE 1
#define VLRF_DEVERR_POSITION_RANGE 2
#define VLRF_DEVERR_NO_BLOCK 4
#define VLRF_DEVERR_WAIT_TIMEOUT 8

// ---- status -------------------------------------------------------------------------------------------------
// Text of the calling thread's last failure (host pointer, valid until the thread's next failure).
const char* vlrf_last_error();
// Properties of the current device (host pointers).
int vlrf_device_info(int* sm_count, int* cc_major, int* cc_minor, int* max_smem_optin);
// Whether kernels are launched chained (programmatic stream serialization); on by default.
int vlrf_chained_launch_enabled();
int vlrf_set_chained_launch(int on);
// Time stamps that the decode step's kernels leave in a build with -DVLRF_KERNEL_TRACE: the buffer's sizes (0 slots
// in a build without stamps), and a copy of it to host memory, [slots][ctas][2 + stations] int64 (launch number,
// kind of kernel: 1 few-row product, 2 decode attention, 3 many-row product, 4 prompt attention; then the global timer's nanoseconds at every station),
// after which the buffer is cleared.
long long* vlrf_trace_buffer();                 // the buffer on the device (what the kernels are handed), or null
int vlrf_trace_dims(int* slots, int* ctas, int* stations);
int vlrf_trace_read(long long* host);

// ---- embedding and LayerNorm (embed_norm.cu) ----------------------------------------------------------------
// x[t] = wte[tokens[t]] (+ wpe[positions[t]] if wpe is not null), float32 [T][d]; tables [V][d] and [P][d] of
// w_dtype.  stats (or null): per row and 32-column segment the sum and the squared deviation from the segment's
// mean, [T][ceil(d/32)][2], for a later product that norms these rows (vlrf_gemm_splitk).
int vlrf_embed(const void* wte, const void* wpe, int w_dtype, const int* tokens, const int* positions, float* x, int T,
               int d, int V, int P, float* stats, int* dev_err, cudaStream_t stream);
// out[r] = LayerNorm(x[rows ? rows[r] : r]) · gamma + beta, statistics in float32 over the whole row (two passes);
// x float32 [·][d], out of out_dtype [n_rows][d].
int vlrf_layernorm(const float* x, const int* rows, const float* gamma, const float* beta, void* out, int out_dtype,
                   int n_rows, int d, float eps, cudaStream_t stream);

// ---- products: Y[M][N] = act(X[M][K] · W[N][K]ᵀ + bias) (+ residual) ----------------------------------------------
// bias float32 [N] or null; residual float32 [M][ldy] or null (it may be Y itself); act is VLRF_ACT_*.  The
// optional cache scatter (Kc not null) also writes the K and V columns of a fused q/k/v projection (columns
// k_off … and v_off …, Hkv heads of dh) into one layer's paged cache at each row's (tok_slot, tok_pos).

// Any sizes, any dtype, FMAs only (the true 32-bit product; the sum over k runs in an order that does not depend on M).
int vlrf_gemm_simt(const void* X, const void* W, const float* bias, const float* residual, void* Y, int M, int N, int K,
                   int ldx, int ldy, int in_dtype, int out_dtype, int act, cudaStream_t stream);

// Many rows, bfloat16 X and W, on the tcgen05 tensor cores (TMA ring, accumulators in tensor memory); with few rows
// and very many columns the operands' roles are exchanged.  K a multiple of 8.
int vlrf_gemm_tcgen05_takes(int M, int N, int K, int ldx);
int vlrf_gemm_tcgen05(const void* X, const void* W, const float* bias, const float* residual, void* Y, int M, int N, int K,
                      int ldx, int ldy, int out_dtype, int act, void* Kc, void* Vc, const int* block_table,
                      int max_blocks, const int* tok_slot, const int* tok_pos, int k_off, int v_off, int Hkv, int dh,
                      int BT, int* dev_err, cudaStream_t stream);
// The same kernel with a weight matrix per group.  offsets != null (device, G + 1 entries): rows offsets[g] …
// offsets[g+1]−1 of X [rows][K] times W[g]ᵀ into the same rows of Y [rows][N] (experts over rows sorted by expert;
// x_gs = y_gs = 0).  offsets == null: every group multiplies all rows, reading X at column g·x_gs and writing Y at
// column g·y_gs (heads).  W [G][N][K]; an activation on the result (VLRF_ACT_NONE, _GELU_TANH, _RELU2); no bias,
// residual or scatter.
int vlrf_gemm_tcgen05_groups_takes(int rows, int G, int N, int K, int ldx, int x_gs, int ldy, int y_gs, int by_offsets);
int vlrf_gemm_tcgen05_groups(const void* X, int ldx, int x_gs, const void* W, void* Y, int ldy, int y_gs, const int* offsets,
                             int G, int rows, int N, int K, int out_dtype, int act, int* dev_err, cudaStream_t stream);
// For measurements: force the tile width (64 … 256 in steps of 32), 0 = chosen by size again.
int vlrf_gemm_tcgen05_force_width(int bn);

// Few rows (M ≤ 64), the sum over k cut into parts whose CTAs form a cluster and add through distributed shared
// memory.  x_is_f32_ln: X is the float32 residual stream and LayerNorm (gamma, beta, eps) is applied first, from
// the rows' statistics `stats_in` ([M][ceil(K/32)][2], see vlrf_embed; M ≤ 16).  stats_out (or null): the same
// statistics of the float32 rows of Y.
long long vlrf_row_stats_floats(int rows, int width);
int vlrf_gemm_splitk_takes(int M, int N, int K, int ldx, int x_is_f32_ln);
int vlrf_gemm_splitk(const void* X, int x_is_f32_ln, const void* W, const float* bias, const float* residual, void* Y,
                     int out_dtype, int M, int N, int K, int ldx, int ldy, int act, const float* gamma, const float* beta,
                     float eps, void* Kc, void* Vc, const int* block_table, int max_blocks, const int* tok_slot,
                     const int* tok_pos, int k_off, int v_off, int Hkv, int dh, int BT, const float* stats_in,
                     float* stats_out, int* dev_err, cudaStream_t stream);

// Few rows, weights streamed once through persistent CTAs (`mma.sync`); x_is_f32_ln: the norm of whole rows in
// the prologue (vlrf_gemm_skinny_ln_fits says whether M rows of K columns fit).  sm_count: CTAs to launch.
int vlrf_gemm_skinny_ln_fits(int M, int K);
int vlrf_gemm_skinny(const void* X, int x_is_f32_ln, const void* W, const float* bias, const float* residual, void* Y,
                     int out_dtype, int M, int N, int K, int ldx, int ldy, int act, const float* gamma, const float* beta,
                     float eps, void* Kc, void* Vc, const int* block_table, int max_blocks, const int* tok_slot,
                     const int* tok_pos, int k_off, int v_off, int Hkv, int dh, int BT, int sm_count, int* dev_err,
                     cudaStream_t stream);

// ---- attention over the paged cache ------------------------------------------------------------------------------
// Rows of `qkv` hold a token's fused projection (row stride ld); queries start at column q_off, H heads of dh; Hkv
// key/value heads (H a multiple of Hkv).  A key at position k is visible to the query at position p iff k ≤ p and,
// with window > 0, p − k < window.  Scores are scaled by `scale`; softmax, sums and outputs in float32.  `out` is
// [rows][ld_out] of the dtype of qkv.

// The new tokens' K and V columns into the cache (where no product's epilogue has written them).
int vlrf_kv_append(const void* qkv, int dtype, int ld, int k_off, int v_off, void* Kc, void* Vc, const int* block_table,
                   int max_blocks, const int* tok_slot, const int* tok_pos, int T, int Hkv, int dh, int BT, int* dev_err,
                   cudaStream_t stream);
// Any mix of tokens, any head size that is a multiple of 16, float32 or bfloat16: a warp per (token, head).
int vlrf_attn_generic(const void* qkv, int dtype, int ld, int q_off, const void* Kc, const void* Vc,
                      const int* block_table, int max_blocks, const int* tok_slot, const int* tok_pos, void* out,
                      int ld_out, int T, int H, int Hkv, int dh, int BT, float scale, int window, int* dev_err,
                      cudaStream_t stream);

// A prompt step in bfloat16: sequence i brings the rows seq_start[i] … seq_start[i+1]−1, which continue slot
// seq_slot[i] at position seq_pos0[i]; max_new is the longest run.  n_blocks: blocks of the cache.
// `mma.sync` kernel, head sizes 64 and 128:
int vlrf_attn_prefill_takes(int dh, int BT, int ld, int q_off);
int vlrf_attn_prefill(const void* qkv, int ld, int q_off, const void* Kc, const void* Vc, int n_blocks,
                      const int* block_table, int max_blocks, const int* seq_slot, const int* seq_start,
                      const int* seq_pos0, void* out, int ld_out, int n_tokens, int n_seqs, int max_new, int H, int Hkv,
                      int dh, int BT, float scale, int window, int* dev_err, cudaStream_t stream);
// tcgen05 kernel, head size 64.  With n_parts > 1 the keys of a long tile of queries are dealt to up to n_parts
// CTAs that meet in scratch: partials, float32, (tiles · n_parts · vlrf_attn_prefill_tc_part_floats()) with tiles =
// ceil(max_new / vlrf_attn_prefill_tc_tile()) · n_seqs · H; counters, int32 [tiles], zero before the first call
// (every call leaves them zero).
int vlrf_attn_prefill_tc_takes(int dh, int BT, int ld, int q_off, int ld_out);
int vlrf_attn_prefill_tc_part_floats();
int vlrf_attn_prefill_tc_max_parts();
int vlrf_attn_prefill_tc_min_part_blocks();
int vlrf_attn_prefill_tc_tile();
int vlrf_attn_prefill_tc(const void* qkv, int ld, int q_off, const void* Kc, const void* Vc, int n_blocks,
                         const int* block_table, int max_blocks, const int* seq_slot, const int* seq_start,
                         const int* seq_pos0, void* out, int ld_out, int n_tokens, int n_seqs, int max_new, int H,
                         int Hkv, int dh, int BT, float scale, int window, int n_parts, float* partials, int* counters,
                         int* dev_err, cudaStream_t stream);

// A decode step: one query per row, at position tok_pos[row] of slot tok_slot[row] (−1: padding, skipped); each
// context is cut into n_split parts, one CTA each.  Head sizes 64 and 128 with up to 16 parts merge inside a
// thread-block cluster and need no scratch (vlrf_attn_decode_needs_scratch says); otherwise partials, float32
// (vlrf_attn_decode_scratch_floats), and counters, int32 [rows · H], zero between calls.  n_blocks: blocks of the
// cache, or 0 if unknown (then bfloat16 with head size 64 takes the kernel without tensor maps).
int vlrf_attn_decode_needs_scratch(int dh, int n_split);
long long vlrf_attn_decode_scratch_floats(int rows, int H, int dh, int n_split);
int vlrf_attn_decode(const void* qkv, int dtype, int ld, int q_off, const void* Kc, const void* Vc, int n_blocks,
                     const int* block_table, int max_blocks, const int* tok_slot, const int* tok_pos, void* out,
                     int ld_out, int rows, int H, int Hkv, int dh, int BT, float scale, int window, int n_split,
                     float* partials, int* counters, int* dev_err, cudaStream_t stream);
// The same for callers that cannot allocate scratch: see attention_decode_noalloc.h for its rules and limits.
int vlrf_attn_decode_noalloc(const void* qkv, int dtype, int ld, int q_off, const void* Kc, const void* Vc,
                             const int* block_table, int max_blocks, const int* tok_slot, const int* tok_pos, void* out,
                             int ld_out, int rows, int H, int Hkv, int dh, int BT, float scale, int window, int n_split,
                             int* dev_err, cudaStream_t stream);

// ---- RMS norm in groups and row-wise helpers (norm_rms.cu) ----------------------------------------------------------
// out[r] (+)= y[rows ? rows[r] : r] / sqrt(mean over the column's group of y² + eps) · w: a row's d columns are cut
// into `groups` equal consecutive parts with a root mean square each (groups = 1: the plain RMS norm).  y float32 of
// row stride ld_y; out of out_dtype and row stride ld_out; accumulate (float32 out only) adds to the row instead of
// replacing it.  out may be y.
// also_bf16 (or null): the finished rows once more, as bfloat16 [n_rows][d].
int vlrf_group_rmsnorm(const float* y, int ld_y, const int* rows, const float* w, void* out, int out_dtype, int ld_out,
                       int n_rows, int d, int groups, float eps, int accumulate, void* also_bf16, cudaStream_t stream);
// n float32 numbers to out_dtype.
int vlrf_cast_rows(const float* x, void* out, int out_dtype, long long n, cudaStream_t stream);
// out[r][c] = act(a[r][c]) · b[r][c], act VLRF_ACT_SILU, VLRF_ACT_SIGMOID, VLRF_ACT_RELU or VLRF_ACT_GELU_TANH, each with a row stride of its own (out may be
// a or b).  Dtypes (a, b → out): all bfloat16; all float32; float32, bfloat16 → bfloat16; float32, float32 → bfloat16.
int vlrf_gate_mul(const void* a, int lda, int a_dtype, const void* b, int ldb, int b_dtype, void* out, int ldo, int out_dtype,
                  int rows, int cols, int act, cudaStream_t stream);
// The same with one column of a for every `per` consecutive columns of b: out[r][c] = act(a[r][c / per]) · b[r][c] (a gate
// per head on the merged heads); cols a multiple of per.
int vlrf_gate_mul_groups(const void* a, int lda, int a_dtype, const void* b, int ldb, int b_dtype, void* out, int ldo, int out_dtype,
                         int rows, int cols, int per, int act, cudaStream_t stream);
// A gate with bounds: out[r][c] = g · sigmoid(alpha · g) · (u + 1) with g = min(a[r][c], limit) and u = clamp(b[r][c], −limit,
// limit).  Dtypes (a, b → out): all bfloat16; all float32; float32, float32 → bfloat16.
int vlrf_gate_mul_clamped(const void* a, int lda, int a_dtype, const void* b, int ldb, int b_dtype, void* out, int ldo, int out_dtype,
                          int rows, int cols, float limit, float alpha, cudaStream_t stream);
// Plain RMS norm and token shift of the step's residual rows: with n_t = x[t] / sqrt(mean(x[t]²) + eps) · w,
// out[t] = n_t + (n_before − n_t) · mu, n_before being the normed row of the sequence's token before: the row above
// where tok_slot[t−1] = tok_slot[t], zeros at position 0, else the sequence's kept row.  state: float32 [slots][2][d];
// a step reads copy (position at its start) mod 2 and writes the normed row of the sequence's last token of the step
// into copy (position behind it) mod 2.  seq_start [n_seqs + 1]: the first row of every sequence of the step.  Rows
// with slot −1 get zeros.  x float32 [T][ld_x]; out of out_dtype [T][ld_out]; w, mu float32 [d].
int vlrf_rmsnorm_shift(const float* x, int ld_x, const float* w, const float* mu, float eps, float* state, const int* tok_slot,
                       const int* tok_pos, const int* seq_start, int n_seqs, int T, void* out, int out_dtype, int ld_out, int d,
                       cudaStream_t stream);
// x[r][c] += v[c] for r < rows, c < d; float32.
int vlrf_add_row_vector(float* x, int ld, const float* v, int rows, int d, cudaStream_t stream);

// ---- a residual in several streams (streams.cu) -------------------------------------------------------------------------
// x[t][s] = table[tokens[t]] · scale for every stream s < S: float32 [T][S][d] from a table [V][d] of w_dtype.
int vlrf_embed_streams(const void* table, int w_dtype, const int* tokens, float* x, int T, int d, int V, int S, float scale,
                       int* dev_err, cudaStream_t stream);
// out[r] = u / sqrt(mean(u²) + eps) · w with u = Σ_s a[s] · x[rows ? rows[r] : r][s] (a null: every coefficient 1);
// x float32 [·][S][d], out of out_dtype [n_rows][d].
int vlrf_streams_read_norm(const float* x, const int* rows, const float* a, const float* w, void* out, int out_dtype, int n_rows,
                           int d, int S, float eps, cudaStream_t stream);
// x[t][j] ← Σ_s mix[s][j] · x[t][s] + b[j] · y[t] for every j at once; x float32 [T][S][d], y float32 [T][d].
int vlrf_streams_write(float* x, const float* mix, const float* b, const float* y, int T, int d, int S, cudaStream_t stream);
// The write above followed by the read of the next sublayer (coefficients a, norm weight w) in one pass: x is rewritten,
// out[t] = RMSnorm(Σ_j a[j] · x'[t][j]) · w.
int vlrf_streams_write_read(float* x, const float* mix, const float* b, const float* y, const float* a, const float* w, void* out,
                            int out_dtype, int T, int d, int S, float eps, cudaStream_t stream);
// v ← cap · tanh(v / cap) over n float32 numbers.
int vlrf_softcap(float* v, long long n, float cap, cudaStream_t stream);
// v ← v · factor over n float32 numbers.
int vlrf_scale_values(float* v, long long n, float factor, cudaStream_t stream);
// x[t] = table[tokens[t]] · scale + pairs[row]: float32 [T][d] from tables [V][d] and [buckets + 1][d] of w_dtype; row =
// (token before · mul_prev + token · mul_cur) mod buckets, or `buckets` at position 0.  The token before is the row above
// where tok_slot and tok_pos say so, else kept[slot][position & 1]; kept int32 [slots][2] receives every sequence's last
// token of the step at the parity of the position behind it (seq_start: n_seqs + 1 first rows of the sequences' tokens).
// also: null, or bfloat16 [T][d] that receives the rounding of every written row (padding rows are left alone).
int vlrf_embed_bigram(const void* table, const void* pairs, int w_dtype, const int* tokens, const int* tok_slot, const int* tok_pos,
                      const int* seq_start, int n_seqs, int* kept, float* x, int T, int d, int V, int buckets, int mul_prev,
                      int mul_cur, float scale, void* also, int* dev_err, cudaStream_t stream);

// ---- attention with key and value sizes of their own (attention_window.cu) -------------------------------------------------
// From the float32 rows of a layer's input product (queries at q_off: H·dk columns, keys at k_off: Hkv·dk, values at
// v_off: Hkv·dv): the first `rot` entries of every query and key head rotated by the token's position (entry i with
// entry i + rot/2, angle position · freq[i]); queries into q_out [T][ldq], keys and values (write_cache ≠ 0) into the
// paged cache K [block][Hkv][BT][dk], V [block][Hkv][BT][dv]; all of `dtype`.
int vlrf_qkv_rope_append(const float* proj, int ld, int q_off, int k_off, int v_off, const float* freq, int rot, void* q_out,
                         int ldq, void* Kc, void* Vc, int dtype, const int* block_table, int max_blocks, const int* tok_slot,
                         const int* tok_pos, int T, int H, int Hkv, int dk, int dv, int BT, int write_cache, int* dev_err,
                         cudaStream_t stream);
// The same with an RMS norm of queries and keys ahead of the rotation (norm 1: every head by itself with one weight vector
// of dk entries for all heads; norm 2: all heads of the projection as one row, weights of H·dk and Hkv·dk entries; 0: none),
// the pairing of rotated entries (0: entry i with i + rot/2; 1: entry 2i with 2i + 1) and a factor on every cosine and
// sine.  Values are read as projected, so v_off = k_off keeps the keys from before norm and rotation as values.  With
// write_cache = 0 the key and value columns are not read.
int vlrf_qkv_norm_rope_append(const float* proj, int ld, int q_off, int k_off, int v_off, const float* freq, int rot, void* q_out,
                              int ldq, void* Kc, void* Vc, int dtype, const int* block_table, int max_blocks, const int* tok_slot,
                              const int* tok_pos, int T, int H, int Hkv, int dk, int dv, int BT, int write_cache, int norm,
                              const float* q_norm, const float* k_norm, float eps, int pairing, float magnitude, int* dev_err,
                              cudaStream_t stream);
// out[t][h·dv …] = out_scale · softmax over the visible keys of (q·k · scale) · V: a token sees the keys of its slot at
// positions ≤ its own (window > 0: the last `window` of them, itself included).  Any dk, dv up to 256.
int vlrf_attn_window(const void* q, int dtype, int ldq, const void* Kc, const void* Vc, const int* block_table, int max_blocks,
                     const int* tok_slot, const int* tok_pos, void* out, int ld_out, int T, int H, int Hkv, int dk, int dv, int BT,
                     float scale, int window, float out_scale, int* dev_err, cudaStream_t stream);
// The same with a cap on the scores (softcap > 0: score ← softcap · tanh(score / softcap), after the scale), keys at
// positions below keep_first visible whatever the window, and sink (null, or a float32 per query head): exp(sink[h])
// is one more term of the softmax's denominator, with nothing in the numerator.  gate (null, or float32 [T][ld_gate], a logit
// per query head): head h's result is multiplied by sigmoid(gate[t][h]).
int vlrf_attn_window_ex(const void* q, int dtype, int ldq, const void* Kc, const void* Vc, const int* block_table, int max_blocks,
                        const int* tok_slot, const int* tok_pos, void* out, int ld_out, int T, int H, int Hkv, int dk, int dv, int BT,
                        float scale, int window, float out_scale, float softcap, int keep_first, const float* sink, const float* gate,
                        int ld_gate, int* dev_err, cudaStream_t stream);

// The same attention on the tensor cores (attention_window_mma.cu; bfloat16): a CTA per key/value head, sequence and tile
// of 64 (token, query head) rows, for prompt steps (rows seq_start[i] … of q are sequence i's new tokens, the first at
// position seq_pos0[i]; the cache already holds their keys and values) and decode steps (max_new = 1), whose contexts
// may be cut into n_split parts with float32 scratch `partials` of rows · H · n_split · (dv + 2) numbers.
int vlrf_attn_window_mma_takes(int H, int Hkv, int dk, int dv, int BT, int ldq, int ld_out);
int vlrf_attn_window_mma(const void* q, int ldq, const void* Kc, const void* Vc, const int* block_table, int max_blocks,
                         const int* seq_slot, const int* seq_start, const int* seq_pos0, void* out, int ld_out, float* partials,
                         int n_seqs, int max_new, int H, int Hkv, int dk, int dv, int BT, float scale, int window, float out_scale,
                         int n_split, int* dev_err, cudaStream_t stream);
// … with the cap, the kept first keys, the sinks and the gate per head of vlrf_attn_window_ex.
int vlrf_attn_window_mma_ex(const void* q, int ldq, const void* Kc, const void* Vc, const int* block_table, int max_blocks,
                            const int* seq_slot, const int* seq_start, const int* seq_pos0, void* out, int ld_out, float* partials,
                            int n_seqs, int max_new, int H, int Hkv, int dk, int dv, int BT, float scale, int window, float out_scale,
                            int n_split, float softcap, int keep_first, const float* sink, const float* gate, int ld_gate, int* dev_err,
                            cudaStream_t stream);

// ---- a state-space recurrence with a matrix state per head (ssd.cu) ----------------------------------------------------------
// What a sequence keeps lies in `state`, float32 [slots][2][state_row]: per copy the heads' states [H][N][P] and, at
// conv_off, the last taps − 1 inputs of the convolution [taps − 1][channels].  A step reads the copy of the parity of
// the sequence's position at its start (seq_pos0) and writes the copy of the parity at its end.
// Causal convolution per channel with bias and x·sigmoid(x) over columns x_off … of the float32 rows `proj`; w
// [channels][taps] (the last tap is the current token's); out float32 [T][channels].  Also leaves the kept inputs.
int vlrf_ssd_conv(const float* proj, int ld, int x_off, const float* w, const float* bias, float* state, int state_row,
                  int conv_off, const int* seq_slot, const int* seq_start, const int* seq_pos0, float* out, int n_seqs, int max_new,
                  int channels, int taps, cudaStream_t stream);
// The recurrence over every sequence's new tokens.  xbc float32 [T][channels] = [x: H·P | B: G·N | C: G·N]; the step
// size is softplus(proj[t][dt_off + h] + dt_bias[h]); y float32 [T][H·P].  max_new: the longest run of new tokens of one
// sequence (it sizes the batches in which the inputs are staged; 1 for a decode step).
int vlrf_ssd_scan(const float* xbc, int channels, const float* proj, int ld, int dt_off, const float* dt_bias, const float* a_log,
                  const float* D, float* state, int state_row, const int* seq_slot, const int* seq_start, const int* seq_pos0,
                  float* y, int n_seqs, int max_new, int Hs, int G, int N, int P, cudaStream_t stream);
// out[r] = factor · groupnorm(y[r] · silu(proj[r][z_off …])) · w: RMS norm in `groups` equal parts; out of out_dtype
// with row stride ld_out.
int vlrf_ssd_gate_norm(const float* y, const float* proj, int ld, int z_off, const float* w, void* out, int out_dtype, int ld_out,
                       int n_rows, int d, int groups, float eps, float factor, cudaStream_t stream);

// ---- products per head and per group (gemm_heads.cu) ------------------------------------------------------------------
// Y[m][h·y_hs …] = X[m][h·x_hs …] · W[h]ᵀ for every head h < H; W [H][N][K].
int vlrf_gemm_heads(const void* X, int ldx, int x_hs, const void* W, void* Y, int ldy, int y_hs, int M, int N, int K, int H,
                    int in_dtype, int out_dtype, cudaStream_t stream);
// Rows offsets[g] … offsets[g+1]−1 of X [P][K] times W[g]ᵀ ([G][N][K]) into the same rows of Y [P][N]; offsets
// (G + 1 entries, ascending, offsets[G] ≤ P) on the device; act: an activation on the result.
int vlrf_gemm_grouped(const void* X, const void* W, void* Y, const int* offsets, int G, int P, int N, int K, int in_dtype,
                      int out_dtype, int act, cudaStream_t stream);

// ---- attention over a cache of latents (attention_latent.cu) -----------------------------------------------------------
// The cache of one layer is [n_blocks][BT][row_w] of `dtype`: per token a row [c | r], the normed latent (C numbers)
// and a rotated key part shared by all heads (R numbers, R may be 0).  Rotation: of the first rot_dims entries, entry
// i pairs with entry i + rot_dims/2 (interleaved != 0: entry 2i with entry 2i + 1); angle = position · inv_freq[i]
// (float32 table of rot_dims/2 entries).
// proj: float32 [T][ld], columns 0…C−1 the latent before its RMS norm (weight norm_w, eps), C…C+R−1 the key part
// before its rotation; the token's row is written at (tok_slot, tok_pos).
int vlrf_latent_append(const float* proj, int ld, int C, int R, const float* norm_w, float eps, const float* inv_freq,
                       int rot_dims, int interleaved, void* cache, int dtype, int row_w, const int* block_table, int max_blocks,
                       const int* tok_slot, const int* tok_pos, int T, int BT, int* dev_err, cudaStream_t stream);
// q: float32 [T][ld_q], per head [dim | R].  qn [T][ld_qn]: the heads' first dim columns, compact; qp [T][ld_qp]:
// per head a row of C + R columns whose last R receive the rotated part (the first C are left for vlrf_gemm_heads).
int vlrf_latent_q_rows(const float* q, int ld_q, int H, int dim, int R, const float* inv_freq, int rot_dims, int interleaved, const int* tok_pos,
                       void* qn, int ld_qn, void* qp, int ld_qp, int C, int dtype, int T, cudaStream_t stream);
// qp [T][ld_q]: per head C + R numbers (the query in latent space, then its rotated part).  out [T][ld_out]: per head
// the C numbers Σ_j p_j c_j with p = softmax_j((qp_h · row_j) · scale) over the visible rows j ≤ position (and, with
// window > 0, position − j < window).  Any mix of tokens; rows with slot −1 get zeros.  C ≤ 1024.
int vlrf_attn_latent(const void* qp, int dtype, int ld_q, const void* cache, int row_w, int C, int R, const int* block_table,
                     int max_blocks, const int* tok_slot, const int* tok_pos, void* out, int ld_out, int T, int H, int BT,
                     float scale, int window, int* dev_err, cudaStream_t stream);
// The cache rows of the step's tokens as plain matrices: out_c [T][C] (latents) and out_r [T][R] (rotated key parts; null
// with R = 0); rows of padding tokens are zeros.
int vlrf_latent_gather(const void* cache, int dtype, int row_w, int C, int R, const int* block_table, int max_blocks,
                       const int* tok_slot, const int* tok_pos, void* out_c, void* out_r, int T, int BT, int* dev_err,
                       cudaStream_t stream);
// Prompt attention over keys and values in plain rows (attention_rows.cu; bfloat16, `mma.sync`), for steps whose
// sequences all begin at their first token: sequence i is the rows seq_start[i] … seq_start[i+1]−1, positions from 0.
// Queries and keys in two parts: per head qn, kn [T][H·dim]; with a shared key part qr [T][H·R], kr [T][≥ R] (R may be
// 0).  score = (qn·kn + qr·kr)·scale over keys j ≤ i; v, out [T][H·vdim].  dim + R one of 32, 64, 96, 128, 192, 256.
int vlrf_attn_rows_takes(int dim, int R, int vdim, int ld_qn, int ld_qr, int ld_kn, int ld_kr, int ld_v, int ld_out);
int vlrf_attn_rows(const void* qn, int ld_qn, const void* qr, int ld_qr, const void* kn, int ld_kn, const void* kr, int ld_kr,
                   const void* v, int ld_v, const int* seq_start, void* out, int ld_out, int n_seqs, int max_new, int H, int dim,
                   int R, int vdim, float scale, cudaStream_t stream);
// The same on the tensor cores (`mma.sync`, bfloat16; attention_latent_mma.cu): a token's heads are the rows of the
// MMAs, tiles of 32 cache rows lie in shared memory once for all heads.  Sequence i brings the rows seq_start[i] …
// seq_start[i+1]−1 at positions seq_pos0[i] … of slot seq_slot[i] (−1: padding, zeros); max_new is the longest run.
// Decode steps (max_new = 1) may cut every context into n_split parts, which meet in `partials` (float32,
// vlrf_attn_latent_mma_scratch_floats) and a second kernel.  C a multiple of 32 up to 512, R a multiple of 16.
int vlrf_attn_latent_mma_takes(int C, int R, int row_w, int BT, int ld_q);
long long vlrf_attn_latent_mma_scratch_floats(int n_tokens, int H, int C, int n_split);
int vlrf_attn_latent_mma_group(int C, int R);
int vlrf_attn_latent_mma_ctas_per_sm(int C, int R);     // decode CTAs an SM holds at a time
int vlrf_attn_latent_mma(const void* qp, int ld_q, const void* cache, int row_w, int C, int R, const int* block_table,
                         int max_blocks, const int* seq_slot, const int* seq_start, const int* seq_pos0, void* out, int ld_out,
                         int n_seqs, int max_new, int H, int BT, float scale, int window, int n_split, float* partials,
                         int* dev_err, cudaStream_t stream);

// ---- routed experts (moe.cu) ---------------------------------------------------------------------------------------
// z: float32 router logits [T][ld_z] (column E: the logit of a shared expert's gate, if shared_gate).  ids, wts, rank
// [T][top]: the chosen experts (largest logits, ties to the lower index; −1 for padding rows), the softmax over the
// chosen logits, the pair's rank among its expert's rows; gate [T] = sigmoid(z[t][E]); counts int32 [E], zero before.
int vlrf_moe_route(const float* z, int ld_z, int E, int top, int shared_gate, const int* tok_slot, int* ids, float* wts,
                   int* rank, float* gate, int* counts, int T, cudaStream_t stream);
// Routing by scores: s = softmax(z) over all E router outputs; a token chooses by s + correction (float32 [E]) among
// the outputs of the `keep` best of `groups` equal groups of neighbours (a group's score: its largest s + correction;
// ties to the lower index everywhere) and weighs the chosen by s · scale.  The last n_identity outputs stand for
// experts without matrices that return their input: such a pair gets ids −2 and no row (padding rows: −1); counts
// int32 [E − n_identity], zero before.  top ≤ keep · E / groups.  scoring 1: s = sigmoid(z), each output by itself.
int vlrf_moe_route_scored(const float* z, int ld_z, int E, int top, int groups, int keep, int n_identity, float scale,
                          int scoring, const float* correction, const int* tok_slot, int* ids, float* wts, int* rank, int* counts, int T,
                          cudaStream_t stream);
// offsets[e] = Σ counts[< e], E + 1 entries; counts are left zero.
int vlrf_moe_plan(int* counts, int* offsets, int E, cudaStream_t stream);
// sorted[offsets[ids[p]] + rank[p]] = h[p / top] for every pair p < T·top with an expert; row_of[p] = that row or −1.
int vlrf_moe_gather(const void* h, int dtype, int width, const int* ids, const int* rank, const int* offsets, void* sorted,
                    int* row_of, int T, int top, cudaStream_t stream);
// y[t] = Σ_j wts[t][j] · expert_out[row_of[t][j]] (+ (gate ? gate[t] : 1) · shared_out[t] if shared_out) (+ residual[t]
// if residual, which may be y), float32.  With ids and h (the experts' input rows, of h_dtype [T][width]): a pair
// whose ids entry is −2 adds wts · h[t] (an expert that returns its input).
int vlrf_moe_combine(const float* expert_out, int width, const int* row_of, const float* wts, int top,
                     const float* shared_out, const float* gate, const float* residual, float* y, int T,
                     const int* ids, const void* h, int h_dtype, cudaStream_t stream);

// ---- a gated recurrence element by element (mingru.cu) ---------------------------------------------------------------
// proj: float32 [T][ld] with, per token, W gate logits at column z_off, W candidate inputs at u_off and W output gate
// logits at g_off.  z = sigmoid(·), c = u + 1/2 where u ≥ 0 and sigmoid(u) below, S ← (1 − z) · S + z · c element by
// element along each sequence, out[t] = S_t · g · sigmoid(g) in out_dtype [T][ld_out].  state: float32 [slots][2][W],
// read at copy (seq_pos0 mod 2) unless seq_pos0 = 0 (zeros), written at copy ((seq_pos0 + tokens) mod 2).  Sequence i
// brings the rows seq_start[i] … seq_start[i+1]−1 for slot seq_slot[i] (−1: padding, skipped); max_new the longest run.
int vlrf_mingru_scan(const float* proj, int ld, int z_off, int u_off, int g_off, int W, float* state, const int* seq_slot,
                     const int* seq_start, const int* seq_pos0, int n_seqs, int max_new, void* out, int out_dtype, int ld_out,
                     cudaStream_t stream);

// ---- sampling (sampling.cu) ----------------------------------------------------------------------------------------
// One token per row of float32 logits [n_rows][ld] over V entries, in the order of the reference (include/model/
// transformer.hpp:124-182): temperature[r] ≤ 0 → the first maximum; else softmax(logits / temperature), top_k[r]
// (≤ 0: off), top_p[r] (≥ 1: off), and an inverse-CDF draw from the counter-based stream (rng_key[r], rng_ctr[r]),
// whose counter moves on.  temperature null: every row greedy; top_k or top_p null: off; rows that draw need rng_key
// and rng_ctr.  next_token,
// next_pos, row_slot (or null): the chosen token goes into next_token[r] as well and next_pos[r] grows by one for
// rows with row_slot[r] ≥ 0, so that the next decode step needs nothing from the host.
int vlrf_sample(const float* logits, int ld, int n_rows, int V, const float* temperature, const int* top_k,
                const float* top_p, const unsigned long long* rng_key, unsigned int* rng_ctr, int* out_token,
                int* next_token, int* next_pos, const int* row_slot, cudaStream_t stream);
// Repetition, frequency and presence penalties over the tokens generated so far (gen [n_rows][gen_ld], gen_len)
// and the no-repeat n-gram block (ngram[r] ≤ 0: off), on the raw logits, in place (reference :124-141).
int vlrf_apply_penalties(float* logits, int ld, int n_rows, int V, const int* gen, int gen_ld, const int* gen_len,
                         const float* rep, const float* freq, const float* pres, const int* ngram, cudaStream_t stream);

// ---- a whole decode step as one persistent kernel (decode_program.cu) ----------------------------------------
// The step is a list of operations (embedding; few-row product with an optional norm of its input, bias, activation,
// residual and cache scatter; attention of one query per row and head over the paged cache), filled on the HOST one
// record at a time by the vlrf_decode_op_* functions into an array of vlrf_decode_program_op_bytes() bytes a record,
// copied to the device by the caller, and run by vlrf_decode_program_run: one cooperative launch of one CTA per SM.
// At most vlrf_decode_program_max_rows() rows; bfloat16 weights and caches.  norm: 0 none, 1 LayerNorm (beta may be
// null), 2 RMS norm.  Buffers between operations have a format: 0 float32 rows, 1 bfloat16 rows (`ld` elements a
// row), or flagged rows, 2: groups of 16 bytes holding 3 float32 and a flag, 3: 6 bfloat16 and a flag (`ld` groups a
// row; `seg` > 0 cuts a row's columns into segments that each begin a new group; zero-filled before first use).
// An operation that reads a flagged buffer waits, group by group, for the flag of the operation `dep` (its index in
// the list) that writes it in the same launch; there is no other ordering between operations, so plain buffers must
// be complete before the launch, and a flagged buffer may be rewritten only by an operation that cannot begin before
// every reader of the old contents has finished.  The *_takes functions say whether an operation's sizes are taken.
int vlrf_decode_program_op_bytes();
int vlrf_decode_program_max_rows();
int vlrf_decode_program_gemv_takes(int n_rows, int N, int K, int in_fmt, int out_fmt, int norm);
int vlrf_decode_program_attention_takes(int head_dim, int block_tokens);
int vlrf_decode_op_embed(void* ops_host, int index, const void* wte, const void* wpe, const int* tokens, void* x, int x_fmt,
                         int x_ld, int d, int V, int P);
int vlrf_decode_op_gemv(void* ops_host, int index, int n_rows, const void* in, int in_fmt, int in_ld, int in_seg, int in_dep,
                        int norm, const float* gamma, const float* beta, float eps, const void* W, const float* bias, int N,
                        int K, int act, void* out, int out_fmt, int out_ld, const void* residual, int res_fmt, int res_ld,
                        int res_dep, void* kc, void* vc, const int* block_table, int max_blocks, int k_off, int v_off, int Hkv,
                        int dh, int BT);
// With a flagged q/k/v buffer the newest key and value are read from it (columns k_off, v_off) and the cache up to the
// position before; with a plain one the cache holds every key.  A flagged output has one segment a head.
int vlrf_decode_op_attention(void* ops_host, int index, const void* qkv, int qkv_fmt, int qkv_ld, int qkv_dep, int qkv_cols,
                             int q_off, int k_off, int v_off, const void* kc, const void* vc, const int* block_table,
                             int max_blocks, void* out, int out_fmt, int out_ld, int H, int Hkv, int dh, int BT, float scale,
                             int window, int n_split, float* partials, int* counters);
// sync_words: 4 uint32 on the device, zero before the first launch; [0] counts the launches (flags are made from it, so
// flagged buffers belong to one sync_words).  Launches that share them, or buffers that the operations name, must not
// overlap.  trace: null, or int64 [SMs][n_ops + 1][8] on the device: times (ns), [cta][op][0] the CTA begins the
// operation ([cta][n_ops][0]: it has finished the last), [cta][op][1…4] stages inside it (0: no share of it).
int vlrf_decode_program_run(const void* ops_dev, int n_ops, int n_rows, const int* tok_slot, const int* tok_pos,
                            void* sync_words, int* dev_err, long long* trace, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
