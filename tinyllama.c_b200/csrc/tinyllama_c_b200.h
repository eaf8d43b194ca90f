/* tinyllama_c_b200.h -- the C interface of libtinyllama_c_b200.so (CUDA kernels for sm_100a).
 *
 * CodeClaper/tinyllama.c's programming interface is a pair of headers: core.h:19-52 (engine_open,
 * session_create, ...) and graph.h:51-109 (the op builders and graph_execute).  This header plays that
 * role for the kernel library: every function the shared library exports is declared here, every .cu
 * file includes it (so the compiler holds each definition to its declaration), and the Python package
 * loads the library with ctypes from a table that a test compares with these prototypes.
 *
 * Conventions
 *   * Every pointer is DEVICE memory unless its comment says "host".  Nothing here allocates on behalf of
 *     the caller except the set-up functions (tlc_*_init), which must run before any stream capture.
 *   * A function that launches work returns 0, or a negative code after storing a message that
 *     tlc_last_error() returns (thread-local).  Nothing exits, traps or prints.
 *   * dtype codes: TLC_F32 = 0 (float), TLC_BF16 = 1 (bfloat16).  A "ld" argument is a row stride in
 *     elements.  All launches go to the given stream and return without waiting.
 *   * A batch is packed: row t of the step belongs to sequence row_seq[t] (0..B-1), which owns rows
 *     cu_seqlens[b] .. cu_seqlens[b+1]-1, sits in cache slot slots[b] and began this step at position
 *     start_pos[b]; positions[t] is the row's absolute position.  All of these are int32.
 *   * Keys and values live in pages of TLC_PAGE positions: [n_pages, KV, TLC_PAGE, hd]; block_table
 *     [n_slots, max_pages] gives the page of every TLC_PAGE positions of a slot.
 *   * Softmax, norms, rotation angles, decay factors, states and all accumulators are 32-bit.
 */
#ifndef TINYLLAMA_C_B200_H
#define TINYLLAMA_C_B200_H

#include <cuda_runtime_api.h>

#define TLC_F32 0
#define TLC_BF16 1
#define TLC_PAGE 64
#define TLC_ACT_SILU 0       /* activations of gated products: z * sigmoid(z) */
#define TLC_ACT_GELU_TANH 1  /* 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))) */
#define TLC_ACT_SWISH_CLAMPED 2 /* experts only: g = min(g, limit), u = clamp(u, -limit, limit): g sigmoid(alpha g) (u + 1) */
#define TLC_ACT_RELU_SQUARED 3 /* experts without a gate: max(W_up h, 0)^2 */
#define TLC_ROUTE_SIGMOID 0  /* a chosen expert's weight is the sigmoid of its logit */
#define TLC_ROUTE_SOFTMAX 1  /* the chosen experts' weights are the softmax restricted to their own logits */
#define TLC_ROUTE_SOFTMAX_ALL 2 /* scores are the softmax over ALL router outputs; chosen by score + a bias, weighted by the score */

#ifdef __cplusplus
extern "C" {
#endif

/* ---- library state ------------------------------------------------------------------------------- */
/* Message of the last failed call of this thread. */
const char* tlc_last_error(void);
/* 1: launches carry the programmatic-serialization attribute (a kernel's blocks are scheduled while its
 * predecessor drains); 0: plain stream order.  The embedding kernel never carries it: it is the boundary
 * between steps (see tlc_embed). */
void tlc_set_pdl(int on);
/* Set-up of the tensor-core products, of prompt attention and of the chunked scan (shared-memory
 * attributes, the driver's tensor-map encoder, the error words, scratch).  Once per process, before any
 * stream capture. */
int tlc_linear_init(void);
int tlc_attention_prefill_init(void);
int tlc_ssd_init(void);
/* Error word of kernels whose waits are bounded: 0, or the code of the wait that ran out (1 loader,
 * 2 issuer, 3 epilogue, 4 drain, 5 accumulator of the tcgen05 product; 9 the self-test).  Reading does
 * not synchronise; clear sets it back to 0. */
int tlc_linear_error(void);
void tlc_linear_error_clear(void);
/* How many clock cycles a bounded wait may spin before it gives up (0: the default, about a second). */
int tlc_wait_limit_cycles(long long cycles);
/* Self-test of the error channel: one block waits, bounded, on a barrier that nobody arrives at, records
 * code 9 when the wait runs out, and returns.  It never traps and never spins beyond the limit. */
int tlc_selftest_bounded_wait(cudaStream_t stream);

/* ---- embedding, norms, activations (elementwise.cu) ---------------------------------------------- */
/* out[t] = table[tokens[t]] * scale; out float [T, D].  The first kernel of a step: it is launched with a
 * full dependency on all earlier work of the stream, which is what lets later kernels of the step fetch
 * cache contents of earlier steps ahead of their own dependency wait. */
int tlc_embed(const int* tokens, const void* table, int table_dtype, int T, int D, int V, float scale,
              float* out, cudaStream_t stream);
/* out[r] = x[rows ? rows[r] : r] / sqrt(mean(x^2) + eps) * w;  x float, rows of D values x_ld apart (a range of the
 * columns of a wider matrix will do); out [R, D] of out_dtype. */
int tlc_rmsnorm(const float* x, int x_ld, const int* rows, const float* w, float eps, int R, int D, void* out,
                int out_dtype, cudaStream_t stream);
/* Layer norm without a bias: out1[r] = (x - mean) / sqrt(var + eps) * w1 with var the mean of the squared deviations, x as in
 * tlc_rmsnorm.  w2 and out2 (both or neither): the same normed row times a second weight, for a layer whose two sublayers each
 * norm the same rows. */
int tlc_layernorm(const float* x, int x_ld, const int* rows, const float* w1, const float* w2, float eps, int R, int D,
                  void* out1, void* out2, int out_dtype, cudaStream_t stream);
/* x[t, :D] += v[:D] for every row of x float [T, D]. */
int tlc_add_row(float* x, const float* v, int T, int D, cudaStream_t stream);
/* Two attention maps per query head over the same values: out[t, h] = o / sqrt(mean(o^2) + eps) * out_scale with
 * o = a1 - lambda a2 over vd values.  att [T, ld_in] holds virtual heads of hd values: the first map of head h (group
 * g = h / per_group) at virtual head 2 g per_group + (h - g per_group), the second per_group heads further on; out
 * [T, ld_out], head h at column h * hd_out. */
int tlc_difference_join(const void* att, int dtype, int ld_in, int hd, void* out, int ld_out, int hd_out, int T, int H,
                        int per_group, int vd, float lambda, float eps, float out_scale, cudaStream_t stream);
/* Gate y (+ y2, where y2 is not NULL: an input that comes as two summands) by silu(z) and RMS-normalise per group,
 * in either order; w NULL: gate only.  out [T, Di] with row stride out_ld, multiplied by out_scale. */
#define TLC_GATE_NORM_FIRST 1   /* mode bit: the norm comes before the gate */
#define TLC_GATE_SIGMOID 2      /* mode bit: the gate is sigmoid(z), not silu(z) */
int tlc_gated_rmsnorm(const float* y, const float* y2, const void* z, int z_dtype, int ldz, const float* w, float eps, int T,
                      int Di, int n_groups, int mode, void* out, int out_dtype, int out_ld,
                      float out_scale, cudaStream_t stream);
/* out[T, F] = silu(gate) * up; gu holds gate | up as halves, or (interleave) 8 gates then their 8 ups. */
int tlc_swiglu(const void* gu, int in_dtype, int ld, int F, int T, void* out, int dtype, int interleave,
               cudaStream_t stream);
int tlc_gather_rows(const float* x, const int* rows, int R, int D, float* out, cudaStream_t stream);
/* out[T, F] = act(gate) * up as tlc_swiglu; act 0: SiLU, 1: GELU in its tanh form, 2 (TLC_ACT_SWISH_CLAMPED): with
 * g = min(gate, limit) and u = up held within +-limit, g * sigmoid(alpha g) * (u + 1). */
int tlc_glu(const void* gu, int in_dtype, int ld, int F, int T, void* out, int dtype, int interleave, int act,
            float limit, float alpha, cudaStream_t stream);
/* out[t, :D] = x[t, :D] (act 0), tanh(x[t, :D]) (act 1) or max(x[t, :D], 0)^2 (act 2) in the given type; row strides ldx, ldo. */
int tlc_convert(const float* x, int ldx, int T, int D, void* out, int dtype, int ldo, int act, cudaStream_t stream);
/* x[i] = cap * tanh(x[i] / cap) for n values, in place. */
int tlc_softcap(float* x, long long n, float cap, cudaStream_t stream);
/* The mean of several sublayers' results, each normed by itself: y = scale * sum_p parts[t, p, :] / rms(parts[t, p, :]) *
 * w[p, :] (parts float [T, n_parts, D], w float [n_parts, D], rms with eps inside the root); then res[t] (+)= y, or with
 * an outer weight wo [D]: res[t] (+)= y / rms(y; eps_o) * wo.  copy (or NULL): [T, D] of type copy_dtype that receives
 * the new res as well. */
int tlc_rmsnorm_mean_add(const float* parts, int n_parts, const float* w, float eps, float scale, const float* wo,
                         float eps_o, int T, int D, float* res, int accumulate, void* copy, int copy_dtype,
                         cudaStream_t stream);
/* RMSNorm with token shift: n[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w and out[t] = n[t] + (n[t-1] - n[t]) * mu, with
 * n[t-1] the normed row of the sequence's previous token: the row above in this step, or what the sequence's slot of
 * state [n_slots, D] holds from its last step (zeros at position 0).  The slot then receives the sequence's last normed
 * row of this step.  x float [T, D]; w, mu float [D]. */
int tlc_rmsnorm_shift(const float* x, const float* w, const float* mu, float eps, int T, int D, const int* row_seq,
                      const int* cu_seqlens, const int* slots, const int* start_pos, float* state, void* out,
                      int out_dtype, cudaStream_t stream);
/* res[t] (+)= y[t] / sqrt(mean(y[t]^2) + eps) * w (w NULL: y[t] itself) with y[t] = sum over p < n_parts of
 * parts[t, p, :] + g[t] * extra[t, :]; parts float [T, n_parts, D] (NULL with n_parts 0), extra float [T, D] or NULL,
 * g[t] = gate[t * gate_ld] (its sigmoid with gate_sigmoid; 1 with gate NULL), res float [T, D].  copy (or NULL): [T, D]
 * of type copy_dtype that receives the new res as well. */
int tlc_rmsnorm_add(const float* parts, int n_parts, const float* extra, const float* gate, int gate_ld,
                    int gate_sigmoid, const float* w, float eps, int T, int D, float* res, int accumulate,
                    void* copy, int copy_dtype, cudaStream_t stream);

/* ---- linear layers (gemm_tcgen05.cu, gemm_simt.cu) ----------------------------------------------------
 * out[m, n] (+)= (sum_k a[m, k] w[n, k]) * colscale[n] + colbias[n];  a [M, K], w [N, K], 32-bit sums.
 * tlc_linear chooses: bfloat16 operands go to the tcgen05 kernel (TMA -> shared memory -> tensor memory)
 * from min_rows_for_tensor_cores rows on, to the weight-streaming mma.sync kernel below that; float
 * operands run on the CUDA cores in true 32-bit arithmetic (tlc_linear_simt). */
int tlc_linear(const void* a, int a_dtype, int lda, const void* w, int w_dtype, int ldw, void* out,
               int out_dtype, int ldo, const float* colscale, const float* colbias, int accumulate, int M,
               int N, int K, int min_rows_for_tensor_cores, cudaStream_t stream);
/* out[M, N/2] = act(gate) * up where the rows of w come in groups of 16 (8 gate rows, their 8 up rows); act is
 * TLC_ACT_SILU or TLC_ACT_GELU_TANH.  Returns 1 when no fused kernel takes the operands (run tlc_linear and tlc_glu
 * instead). */
int tlc_linear_swiglu(const void* a, int a_dtype, int lda, const void* w, int w_dtype, int ldw, void* out,
                      int out_dtype, int ldo, const float* colscale, const float* colbias, int M, int N, int K,
                      int min_rows_for_tensor_cores, int act, cudaStream_t stream);
int tlc_linear_simt(const void* a, int a_dtype, int lda, const void* w, int w_dtype, int ldw, void* out,
                    int out_dtype, int ldo, const float* colscale, const float* colbias, int accumulate,
                    int M, int N, int K, cudaStream_t stream);
// The product for 17..64 rows (weights on the 128-row side of tcgen05.mma, K shared among the blocks of a cluster).
void tlc_linear_few_rows(int on);          // 0: never this kernel (for comparisons)
void tlc_linear_few_rows_split(int split); // 0: the number of blocks per tile is chosen; 1, 2, 4, 8: fixed (for tests)
void tlc_linear_few_rows_min_tiles(int tiles);   // outputs of fewer tiles of 128 weight rows stay with the other kernels (0: 16 tiles with more than 32 rows, else 32)
void tlc_linear_few_rows_max_rows(int rows);     // products of more rows go to the tiles of the prompt product (128; for comparisons)
int tlc_linear_few_rows_ok(int a_dtype, int lda, const void* a, int w_dtype, int ldw, const void* w, int M, int N, int K);
void tlc_linear_tma_out(int on);        // 0: the tensor-core product's 32-bit outputs never leave through the copy engine (for comparisons)
void tlc_linear_skinny_pairs(int on);   // 0: the skinny product never splits K over a pair of blocks (for comparisons)
int tlc_linear_skinny_ok(int a_dtype, int lda, const void* a, int w_dtype, int ldw, const void* w, int M, int K);
int tlc_linear_skinny(const void* a, int lda, const void* w, int ldw, void* out, int out_dtype, int ldo,
                      const float* colscale, const float* colbias, int accumulate, int M, int N, int K,
                      cudaStream_t stream);
int tlc_linear_skinny_swiglu(const void* a, int lda, const void* w, int ldw, void* out, int out_dtype, int ldo,
                             const float* colscale, const float* colbias, int M, int N, int K, int act,
                             cudaStream_t stream);
int tlc_linear_tcgen05_ok(int a_dtype, int lda, const void* a, int w_dtype, int ldw, const void* w, int K);
/* Test hooks: force the tile width (0, 64, 128, 256) / how many blocks share a tile's K-steps (0 = choose). */
void tlc_linear_tile_override(int bn);
void tlc_linear_split_override(int n);
/* Test hook: pairs of blocks on 256 x 256 tiles (tcgen05.mma.cta_group::2): 0 = where they pay, 1 = never,
 * 2 = wherever the GPU can run them. */
void tlc_linear_pair_override(int mode);
/* How many pairs of blocks the GPU runs at once; 0 if it runs none (every product then takes single blocks). */
int tlc_linear_pairs(void);

/* ---- attention (attention.cu, attention_decode_fused.cu, attention_prefill.cu) ------------------- */
/* Rotates q and k (split-half pairs over the first rope_dim dims, angle = position * inv_freq[i]); writes
 * q to q_out [T, H*hd] and, when write_kv, k and v into the pages of their sequences. */
int tlc_rope_kv_store(const void* qkv, int in_dtype, int dtype, int ld, int q_off, int k_off, int v_off,
                      void* q_out, void* k_pages, void* v_pages, const float* inv_freq, int rope_dim,
                      const int* positions, const int* row_seq, const int* slots, const int* block_table,
                      int max_pages, int T, int H, int KV, int hd, int write_kv, cudaStream_t stream);
/* Causal grouped-query attention of every row over its sequence's pages (keys 0..position, or the last
 * `window`); any sizes, both element types; a warp per (row, head).  softcap > 0: score <- softcap * tanh(score /
 * softcap) after the scale; sink: one more term of score 0 in the softmax's denominator, which carries no value
 * (sink_values not NULL: of score sink_values[head], not scaled).  keep_first > 0 with a window: the first keep_first keys
 * of the sequence stay visible to every query at their own positions. */
int tlc_attention(const void* q, int dtype, const void* k_pages, const void* v_pages, const int* block_table,
                  int max_pages, const int* positions, const int* row_seq, const int* slots, void* out, int T,
                  int H, int KV, int hd, float scale, int window, int out_ld, float softcap, int sink, int keep_first,
                  const float* sink_values, cudaStream_t stream);
/* Single-token rows: keys split across blocks of 128, partial results in part_o [T, H, splits, hd] and
 * part_ml [T, H, splits, 2], then merged. */
int tlc_attention_decode(const void* q, int dtype, const void* k_pages, const void* v_pages,
                         const int* block_table, int max_pages, const int* positions, const int* row_seq,
                         const int* slots, void* out, float* part_o, float* part_ml, int T, int H, int KV,
                         int hd, float scale, int window, int max_keys, int out_ld, float softcap, int sink,
                         int keep_first, const float* sink_values, cudaStream_t stream);
/* Single-token rows of a bfloat16 cache in one kernel: rotation of q and the new key, store of the new
 * K/V row, scores and outputs on the tensor cores, merge of the splits by the last block to arrive
 * (arrivals: zeroed counters, at least T*KV, back at zero afterwards). */
int tlc_attention_decode_fused_ok(int H, int KV, int hd);
int tlc_attention_decode_fused_passes(int passes);
int tlc_attention_decode_fused(const float* qkv, int ld, int q_off, int k_off, int v_off, void* k_pages,
                               void* v_pages, const float* inv_freq, int rope_dim, int write_kv,
                               const int* block_table, int max_pages, const int* positions, const int* row_seq,
                               const int* slots, void* out, float* part_o, float* part_ml, unsigned* arrivals,
                               int T, int H, int KV, int hd, float scale, int window, int max_keys, int out_ld,
                               float softcap, int sink, int keep_first,
                               const float* sink_values, cudaStream_t stream);
/* Prompt rows (consecutive positions from start_pos) of a bfloat16 cache on the tensor cores. */
int tlc_attention_prefill_ok(int dtype, int hd);
int tlc_attention_prefill_chunks(int n_tiles_bound, int H, int max_tiles, int* chunk_tiles /* host */);
int tlc_attention_prefill(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                          int max_pages, const int* cu_seqlens, const int* slots, const int* start_pos, void* out,
                          int n_seqs, int n_tiles_bound, int H, int KV, int hd, float scale, int window,
                          int max_tiles, const int* row_seq, float* part_o, float* part_ml, int T, int out_ld,
                          cudaStream_t stream);

/* The same on tcgen05.mma (attention_prefill_tc.cu): 128-row tiles, Q and the K and V pages by TMA, scores and
 * output in tensor memory.  n_tiles_bound >= sum_b ceil(n_new_b / 128); n_pages: pages of k_pages / v_pages.
 * Values in pages past a sequence's end must be finite.  softcap, sink, keep_first and sink_values as in tlc_attention. */
int tlc_attention_prefill_tc_ok(int dtype, int hd, int H, int KV);
int tlc_attention_prefill_tc(const void* q, const void* k_pages, const void* v_pages, int n_pages,
                             const int* block_table, int max_pages, const int* cu_seqlens, const int* slots,
                             const int* start_pos, void* out, int n_seqs, int n_tiles_bound, int H, int KV,
                             int hd, float scale, int window, int max_keys, int T, int out_ld, int max_blocks,
                             int n_split, float* part_o, float* part_ml, float softcap, int sink, int keep_first,
                             const float* sink_values, cudaStream_t stream);
int tlc_attention_prefill_tc_splits(int n_tiles_bound, int H, int max_keys);   // suggested n_split (1: none)

/* ---- Mamba2 (mamba.cu, mamba_ssd.cu) ----------------------------------------------------------------- */
/* Causal depthwise convolution + SiLU over the x|B|C columns of proj, continuing each sequence's window
 * conv_state [n_slots, K-1, Cd] (updated in place); dt = softplus(dt + dt_bias), dA = exp(dt * A).
 * xbc_out [T, Cd] has the type xbc_dtype: float for single-token steps and the 32-bit scans, bfloat16
 * for the scan of prompts in matrix form (tlc_ssm_scan_ssd). */
int tlc_mamba_conv(const void* proj, int dtype, int ld, int xbc_off, int dt_off, const float* w,
                   const float* bias, const float* dt_bias, const float* A, float* conv_state,
                   const int* cu_seqlens, const int* row_seq, const int* slots, const int* start_pos,
                   void* xbc_out, int xbc_dtype, float* dt_out, float* dA_out, int T, int B, int Cd, int K,
                   int Hs, int single_rows, int quick, int all_fresh, cudaStream_t stream);
/* S = S * dA + B (x dt), y = S.C + x D, row by row from each slot's state [n_slots, Hs, P, N] (zero at
 * position 0), which is updated in place. */
int tlc_ssm_scan(const float* xbc, const float* dt, const float* dA, const float* Dskip, float* state,
                 const int* cu_seqlens, const int* slots, const int* start_pos, float* y, int B, int Hs, int P,
                 int N, int G, int Cd, cudaStream_t stream);
/* The same with sequences cut into chunks (seg_start [n_seg+1], seg_seq [n_seg], seq_seg_start [B+1]) that
 * run in parallel in three 32-bit passes; chunk_state: n_seg*Hs*(P*N+1) floats of scratch. */
int tlc_ssm_scan_chunked(const float* xbc, const float* dt, const float* dA, const float* Dskip, float* state,
                         float* chunk_state, const int* seg_start, const int* seg_seq, const int* seq_seg_start,
                         const int* slots, const int* start_pos, float* y, int B, int n_seg, int Hs, int P, int N,
                         int G, int Cd, cudaStream_t stream);
/* The chunks (of 128 rows at most) in matrix form on the tensor cores, for bfloat16 runs: xbc is bfloat16
 * [T, Cd]; C B^T of every chunk goes through `scratch` (tlc_ssd_scratch_floats floats); one block per
 * (sequence, head, 32 rows of the head) then walks the sequence's chunks in order with the state in its
 * registers, from the slot's state to the slot's state. */
int tlc_ssd_ok(int Hs, int P, int N, int G, int Cd);
/* Test hook: 0 = the walk uses tcgen05.mma with the state in tensor memory where it is built (states of 128
 * or 256 columns) and mma.sync with the state in registers elsewhere; 1 = always the latter. */
void tlc_ssd_walk_override(int mode);
void tlc_ssd_walk_blocks(int blocks);      // the grid of the tcgen05 walk (0: one block an SM at most; for tests)
long long tlc_ssd_scratch_floats(int n_seg, int T, int Hs, int P, int N, int G);
/* y_part [T, Hs*P] and used_part may be NULL.  Where the walk runs on tcgen05 and they are given, the outputs come as
 * two summands: what needs no state (M x + D x) in y_part, the state's share in y, and *used_part = 1.  With a second
 * stream `aux` (NULL: none) the first summand is computed there, beside the walk; `stream` has waited for it when the
 * call returns.  Otherwise *used_part = 0 and y holds the outputs. */
int tlc_ssm_scan_ssd(const void* xbc, const float* dt, const float* A, const float* Dskip, float* state,
                     float* scratch, const int* seg_start, const int* seg_seq, const int* seq_seg_start,
                     const int* slots, const int* start_pos, float* y, float* y_part, int* used_part, int B, int n_seg,
                     int T, int Hs, int P, int N, int G, int Cd, cudaStream_t stream, cudaStream_t aux);

/* ---- attention over a shared latent (latent_attention.cu) -----------------------------------------------
 * A token's cache row is [c | kr] (R normed latent values, r rotated key values that all heads share); pages
 * [n_pages, TLC_PAGE, R + r].  tlc_latent_prepare reads a row's projections (float: H heads of (dn | r) query values
 * at q_off of qproj, row stride ldq; R + r down-projected values at dkv_off of proj, row stride ld, or dkv_off < 0 for
 * a layer that reads another layer's rows; the two may be one buffer), writes the unrotated query parts to qn [T, H*dn], the rotated ones (interleaved pairs of the
 * first `rot` dimensions, angle = position * inv_freq[i]) into the last r columns of every head of qa [T, H*(R+r)],
 * and the row [rmsnorm(c) * cw | rotated kr] into its page.  qn, qa and pages are of `dtype`. */
int tlc_latent_prepare(const float* qproj, int ldq, int q_off, const float* proj, int ld, int dkv_off, const float* cw, float eps,
                       const float* inv_freq, int rot, const int* positions, const int* row_seq, const int* slots,
                       const int* block_table, int max_pages, void* pages, void* qn, void* qa, int dtype, int T, int H,
                       int dn, int r, int R, cudaStream_t stream);
/* out[t, h, :R] = sum_j p_j c_j over the keys 0..position of the row's sequence, p = softmax of (qa[t, h] . [c_j | kr_j])
 * * scale together with the head's sink (float [H], or NULL for none), which enters the maximum and the denominator
 * only.  window > 0: a row sees only the last `window` keys up to its own position. */
int tlc_latent_attention(const void* qa, const void* pages, int dtype, const float* sink, const int* block_table,
                         int max_pages, const int* positions, const int* row_seq, const int* slots, void* out, int T,
                         int H, int R, int r, float scale, int window, cudaStream_t stream);
/* The same on the tensor cores, for bfloat16 rows with R and R + r multiples of 16 and R <= 256 (tlc_..._ok): a block
 * takes tile_pairs (64 or 128) (row, head) pairs of one sequence and reads every page once, as keys and as values.  Rows of
 * a sequence are consecutive positions from start_pos.  n_tiles: an upper bound of the sum over sequences of
 * ceil(rows / (tile_pairs / HP)),
 * HP = H rounded up to a power of two (at most 64).  n_split > 1 cuts every tile's keys into that many ranges
 * (tlc_..._splits proposes a number for `blocks` tiles and sequences of up to max_keys positions); part_o
 * [T, H, n_split, R] and part_ml [T, H, n_split, 2] floats are then scratch. */
int tlc_latent_attention_tc_ok(int dtype, int H, int R, int r);
int tlc_latent_attention_tc_splits(int blocks, int max_keys);
int tlc_latent_attention_tc_tile(int T, int B, int R, int r);      /* 64 or 128 pairs a tile (tile_pairs below) */
int tlc_latent_attention_tc(const void* qa, const void* pages, const float* sink, const int* block_table, int max_pages,
                            const int* cu_seqlens, const int* slots, const int* start_pos, void* out, float* part_o,
                            float* part_ml, int B, int T, int tile_pairs, int n_tiles, int H, int R, int r, float scale,
                            int n_split, int window, cudaStream_t stream);
/* A product per head: out[t, h, n] = sum_k a[t, h, k] w[h, n, k]; a with row stride lda and head stride a_hs, w
 * [H, N, K] dense, out with row stride ldo and head stride o_hs; 32-bit sums. */
int tlc_linear_heads(const void* a, int a_dtype, int lda, int a_hs, const void* w, int w_dtype, void* out,
                     int out_dtype, int ldo, int o_hs, int T, int H, int N, int K, cudaStream_t stream);

/* ---- minGRU (recurrent.cu) ------------------------------------------------------------------------------
 * Per channel c < W of every row: z = sigmoid(proj[z_off + c]), u = proj[u_off + c], cand = u + 1/2 (u >= 0) or
 * sigmoid(u); S <- (1 - z) S + z cand from the slot's state [n_slots, W] (zero at position 0), which receives the
 * last S; out[t, c] = S * silu(proj[g_off + c]).  With seg_start [n_seg + 1] and seq_seg_start [B + 1] (the step's
 * chunk table) and scratch of 2 * n_seg * W floats the chunks run side by side (same result up to rounding);
 * seg_start NULL: row by row. */
int tlc_mingru_scan(const float* proj, int ld, int z_off, int u_off, int g_off, int W, float* state,
                    const int* cu_seqlens, const int* slots, const int* start_pos, int B, void* out, int out_dtype,
                    int out_ld, const int* seg_start, const int* seq_seg_start, int n_seg, float* scratch,
                    cudaStream_t stream);

/* ---- queries, keys and the output gate of an attention mixer (qk_transform.cu) ---------------------------
 * tlc_qk_rotate_norm, in place on the float projection qkv [T, ld] (H query heads from q_off, KV key heads from k_off,
 * heads `stride` values apart, `dim` <= stride of them in use): the pairs of the first `rot` dimensions turn by
 * position * inv_freq[i] (pairs (2i, 2i+1) with interleaved != 0, else (i, i + rot/2)); then, with norm_eps >= 0, the
 * head is divided by sqrt(mean over dim of x^2 + norm_eps).  q_w, k_w (float [dim], both or neither): before the rotation
 * every query head becomes x / sqrt(mean(x^2) + pre_eps) * q_w, every key head likewise with k_w.  amplitude multiplies the
 * cosines and sines.
 * tlc_gate_mul: x[t, c] *= sigmoid(gate[t, c]) (act 0) or silu(gate[t, c]) (act 1); x [T, n] of `dtype`, row stride ldx;
 * gate float, row stride ldg. */
int tlc_qk_rotate_norm(float* qkv, int ld, int q_off, int k_off, int H, int KV, int stride, int dim, const float* inv_freq,
                       int rot, int interleaved, float norm_eps, const int* positions, int T, const float* q_w,
                       const float* k_w, float pre_eps, float amplitude, cudaStream_t stream);
int tlc_gate_mul(void* x, int dtype, int ldx, const float* gate, int ldg, int n, int T, int act, cudaStream_t stream);
/* In place on the 32-bit projection: the q_n query columns from q_off, all heads together, are divided by their root mean
 * square (eps inside the root) and multiplied by qw [q_n]; the k_n key columns from k_off likewise with kw [k_n]. */
int tlc_qk_whole_norm(float* qkv, int ld, int q_off, int q_n, const float* qw, int k_off, int k_n, const float* kw, float eps,
                      int T, cudaStream_t stream);

/* ---- gated delta rule (delta_rule.cu) -------------------------------------------------------------------
 * Per head: M <- a M; w = b (v - M^T k); M <- M + k w^T; r = M^T q (a the decay, b the write strength `beta`), with M
 * [dk, dv] float per (slot, head) in state
 * [n_slots, H, dk, dv] (zero at position 0).  tlc_delta_prepare normalises, in place in qkv [T, ld] float, the G query
 * heads at q_off (x / sqrt(sum x^2 + l2_eps) * q_scale) and the G key heads at k_off (the same without the scale), and
 * writes beta[t, h] = sigmoid(proj[t, b_off + h]).  tlc_delta_rule walks every sequence's rows: values (H heads of dv) at
 * v_off, beta and decay float [T, H]; y [T, ldy] float receives the read-outs (head h at column h * dv).
 * A decay per key channel: tlc_delta_prepare with chan [T, ldc] (head h's dk values at column h * dk) and A [H] turns chan,
 * in place, into exp(A[h] * softplus(chan)); tlc_delta_rule with ldd > 0 takes decay [T, ldd] laid out like that and
 * multiplies row r of M by its own factor: M <- diag(a) M. */
int tlc_delta_prepare(float* qkv, int ld, int q_off, int k_off, int G, int dk, float l2_eps, float q_scale, const float* proj,
                      int ldp, int b_off, int H, float* beta, int T, float* chan, int ldc, const float* A, cudaStream_t stream);
void tlc_delta_rule_split(int threads);   /* threads that share the rows of a column group: 8 or 16 (0: chosen); for tests */
int tlc_delta_rule(const float* qkv, int ld, int q_off, int k_off, int v_off, const float* beta, const float* decay,
                   float* state, const int* cu_seqlens, const int* slots, const int* start_pos, int B, int T, int H, int G,
                   int dk, int dv, float* y, int ldy, int ldd, cudaStream_t stream);

/* ---- mixture of experts (moe.cu) ------------------------------------------------------------------------
 * tlc_moe_route: logits float [T, ld] (E columns) -> per token its `top` experts by descending logit (lowest index
 * first on ties) in ids [T*top] with weights wts = sigmoid(logit) (mode TLC_ROUTE_SIGMOID) or a softmax restricted to
 * the picked logits (TLC_ROUTE_SOFTMAX); order [T*top] lists the pairs (t * top + k) sorted
 * by expert, offsets [E+1] every expert's first sorted position, tile_off [E+1] its first tile of tile_rows sorted rows
 * (32 for tlc_moe_gate_up / tlc_moe_down; 32 or 64 for tlc_moe_experts_mma, which is told the same number). */
/* TLC_ROUTE_SOFTMAX_ALL: scores s = softmax over all E outputs; chosen by s + choice_bias[e] (choice_bias NULL: by s),
 * weighted by s.  The last n_identity of the E outputs have no expert's weights (they stand for experts that return their
 * input, tlc_moe_identity): their pairs are sorted behind the others and get no tiles, and the expert products are called
 * with E - n_identity experts.  sum_to > 0 (TLC_ROUTE_SOFTMAX_ALL): a token's weights are divided by their sum (+ 1e-20) and
 * multiplied by sum_to. */
int tlc_moe_route(const float* logits, int ld, int T, int E, int top, int mode, const float* choice_bias, int n_identity,
                  int* ids, float* wts, int* order, int* offsets, int* tile_off, int tile_rows, float sum_to, cudaStream_t stream);
/* y[pair, :D] = wts[pair] * x[token(pair), :D] for every pair with ids[pair] >= E. */
int tlc_moe_identity(const void* x, int x_dtype, int ldx, const int* ids, const float* wts, int T, int top, int E, int D,
                     float* y, cudaStream_t stream);
/* act[i, :F] for sorted position i from g | u = wgu[e] x[token], wgu [E, 2F, D], and the pair's weight w: with w_out 0
 * the weight scales the expert's input, act(w g) * (w u); with w_out 1 its output, w * act(g, u).  act: TLC_ACT_SILU,
 * TLC_ACT_GELU_TANH, or TLC_ACT_SWISH_CLAMPED with its limit and alpha; TLC_ACT_RELU_SQUARED: experts without a gate,
 * wgu [E, F, D], act = w * max(wgu[e] x, 0)^2 (one product). */
int tlc_moe_gate_up(const void* x, int x_dtype, int ldx, const void* wgu, int w_dtype, const int* order,
                    const int* offsets, const int* tile_off, const float* wts, int T, int E, int top, int F, int D,
                    void* act, int act_dtype, int act_code, int w_out, float limit, float alpha, cudaStream_t stream);
/* y[pair, :D] = wd[e] act[i, :] for sorted position i of pair (t, k); wd [E, D, F]; y float [T*top, D]. */
int tlc_moe_down(const void* act, int act_dtype, const void* wd, int w_dtype, const int* order, const int* offsets,
                 const int* tile_off, int T, int E, int top, int F, int D, float* y, cudaStream_t stream);

/* ---- grouped products on the tensor cores (grouped_mma.cu) ----------------------------------------------
 * mma.sync with bfloat16 operands for the product per head and for both expert products, where every operand row
 * starts on a 16-byte boundary (tlc_grouped_mma_ok: a with row stride lda and group stride a_hs, w with rows of K).
 * Same results as tlc_linear_heads / tlc_moe_gate_up + tlc_moe_down up to the order of the 32-bit sums. */
int tlc_grouped_mma_ok(int a_dtype, int w_dtype, const void* a, int lda, int a_hs, const void* w, int K);
int tlc_linear_heads_mma(const void* a, int lda, int a_hs, const void* w, void* out, int out_dtype, int ldo, int o_hs,
                         int T, int H, int N, int K, cudaStream_t stream);
int tlc_moe_experts_mma(const void* x, int ldx, const void* wgu, const void* wd, const int* order, const int* offsets,
                        const int* tile_off, const float* wts, int T, int E, int top, int F, int D, void* act, float* y,
                        int tile_rows, int act_code, int w_out, float limit, float alpha, cudaStream_t stream);

/* ---- time mixing with a decaying matrix state (wkv.cu) ------------------------------------------------------
 * tlc_shift_mix: out[t, s, :] = x[t] + (x[t-1] - x[t]) * mu[s] for n_mix learned vectors mu [n_mix, D]; x[t-1] is the row
 * above, or for a sequence's first row of the step what its slot of state [n_slots, D] holds (zeros at position 0); the
 * slot then receives the sequence's last row.  x float [T, D]; out [T, n_mix, D] of out_dtype.
 * tlc_wkv_scan: per (sequence, head) o_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(w_t) S + k_t v_t^T with
 * w_t = exp(-exp(decay_log_t)); r, k, v: columns r_off, k_off, v_off (+ h * d) of rkv float [T, ld]; decay_log float
 * [T, ld_w] (H * d columns); bonus u float [H, d]; state float [n_slots, H, d, d] (zero at position 0, updated in
 * place); out float [T, out_ld] (H * d columns). */
int tlc_shift_mix(const float* x, const float* mu, int n_mix, int T, int D, const int* row_seq, const int* cu_seqlens,
                  const int* slots, const int* start_pos, float* state, void* out, int out_dtype, cudaStream_t stream);
int tlc_wkv_scan(const float* rkv, int ld, int r_off, int k_off, int v_off, const float* decay_log, int ld_w,
                 const float* bonus, float* state, const int* cu_seqlens, const int* slots, const int* start_pos, int B,
                 int H, int d, float* out, int out_ld, cudaStream_t stream);

/* ---- sampling (sampling.cu) ------------------------------------------------------------------------ */
/* out[r] = first index of the maximum of logits[r].  work: NULL (one block a row), or 12 * R bytes, 8-byte
 * aligned and zero (R 64-bit keys, R counters), which every launch leaves zero: a row is then spread over
 * blocks of 2,048 values.  Launches that share `work` must not overlap on the GPU. */
int tlc_argmax(const float* logits, int R, int V, int* out, void* work, cudaStream_t stream);
/* Penalties over history [R, n_history] (-1 = empty), temperature, top-k, min-p, top-p, then one draw per
 * row from uniforms [R]; work: R*V floats of scratch. */
int tlc_sample(const float* logits, float* work, const int* history, const float* uniforms, int R, int V,
               float temperature, int top_k, float top_p, float min_p, float repeat_penalty, int n_history,
               float frequency_penalty, float presence_penalty, int* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

/* The entry point for callers that must not allocate has a header of its own. */
#include "no_alloc.h"

#endif /* TINYLLAMA_C_B200_H */
