// C launch interface of the engine's CUDA kernels. Every function enqueues work on `stream` and
// returns LSE_OK, or a non-zero code with nothing enqueued when an argument cannot be served.
// dtype codes: 0 = float32, 1 = bfloat16.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "status.h"

#define LSE_F32 0
#define LSE_BF16 1
// Sums that several blocks add to in any order: a 64-bit integer holding value * 2^24. Integer
// addition is associative, so the result has the same bits whatever the order was. A kernel that
// takes such an input converts it to float32 and leaves zeros behind, ready for the next sums.
#define LSE_FIXED64 2

extern "C" {

// out[t, :] = float(table[ids[t], :])                      out float32 [T, H]
int lse_embedding(const int* ids, const void* table, int table_dtype, float* out, int T, int H,
                  cudaStream_t stream);

// Residual add and RMS norm.
//   rows == nullptr: for every row t < T: if residual: x[t] += residual[t] (in place, float32);
//                    out[t] = x[t] * rsqrt(mean(x[t]^2) + eps) * weight
//   rows != nullptr: out[r] = norm(x[rows[r]] (+ residual[rows[r]])) for r < T; x is not written.
// residual_dtype LSE_FIXED64 (rows == nullptr only): residual holds fixed-point sums, which are
// cleared as they are read.
int lse_add_rmsnorm(float* x, const void* residual, int residual_dtype, const float* weight,
                    float eps, void* out, int out_dtype, const int* rows, int T, int H,
                    cudaStream_t stream);

// Rotate the q and k heads of the fused projection and write this step's k and v rows into their
// pages. qkv [T, (nq + 2 nk) D] of in_dtype; the rotated queries go to q_out as `dtype`:
//   in_dtype == dtype: q_out must be qkv itself (rotated in place, row stride (nq + 2 nk) D);
//   in_dtype == LSE_F32 or LSE_FIXED64 (cleared as it is read), dtype == LSE_BF16: q_out is a
//   separate [T, nq D] buffer.
//   cos/sin float32 [max_pos, D/2] or nullptr for no rotation;
//   k_pages/v_pages [pages, nk, page_tokens, D] of `dtype`, or nullptr when this layer only reads.
int lse_rope_kv_write(const void* qkv, int in_dtype, void* q_out, int dtype, int T, int nq, int nk,
                      int D, const int* positions, const int* token_seq, const float* cos,
                      const float* sin, void* k_pages, void* v_pages, const int* block_tables,
                      int table_stride, int page_tokens, cudaStream_t stream);

// out[t, i] = act(gu[t, i]) * gu[t, I + i]     gu [T, 2I] of in_dtype, out [T, I] of dtype
// (in_dtype == dtype, or float32 / LSE_FIXED64 in and bfloat16 out; a fixed-point input is cleared
// as it is read). act: LSE_ACT_SILU (a / (1 + exp(-a))) or LSE_ACT_GELU_TANH (the tanh form of gelu).
#define LSE_ACT_SILU 0
#define LSE_ACT_GELU_TANH 1
int lse_silu_mul(const void* gu, int in_dtype, void* out, int dtype, int T, int I, int act,
                 cudaStream_t stream);

// True float32 matrix product: out[T, N] = a[T, K] . w[N, K]^T (+ bias[N]). Each output element is
// accumulated over k in ascending order by one thread, so a row's result does not depend on T.
int lse_gemm_f32(const float* a, const float* w, const float* bias, float* out, int T, int N, int K,
                 cudaStream_t stream);

// bfloat16 product for few rows on tcgen05 tensor cores fed by TMA (gemm_bf16_tc.cu):
//   out[T, N] += a[T, K] . w[N, K]^T (+ bias[N]),  T <= lse_gemm_bf16_skinny_max_rows(), K % 8 == 0.
// out is a buffer of 64-bit fixed-point numbers (see LSE_FIXED64). The work is balanced over all
// SMs whatever N is; the sums do not depend on the order of the additions, so they have the same
// bits on every run. error_flag (device-visible int, may be null) receives a non-zero code if a
// bounded wait inside the kernel ran out.
int lse_gemm_bf16_skinny_max_rows(void);
int lse_gemm_bf16_skinny(const void* a, const void* w, const void* bias, void* out, int T, int N,
                         int K, int* error_flag, cudaStream_t stream);

// out[T, N] = value of the fixed-point sums acc[T, N] (+ what out holds, if add != 0); every
// element of acc that is read is set to zero. out float32 or bfloat16 (add needs float32).
int lse_fixed_to_float(void* acc, void* out, int out_dtype, int add, long long n, cudaStream_t stream);

// Sampling. One token per row of logits [R, V] (float32, row stride V).
//   temperature[r] < 1e-5 selects the largest logit (lowest index on ties). Otherwise the row is
//   divided by its temperature, cut to top_k / top_p / min_p, and a token is drawn by the
//   exponential race: argmax p_i / E_i, E_i ~ Exp(1) from a counter-based generator keyed by
//   (seed[r], draw[r], i).
//   scratch: lse_sample_scratch_ints(scratch_rows) ints, zero before the first launch (every
//   launch leaves its counters zero), or null. With it (and scratch_rows >= R), rows that need no
//   cut (and a temperature) are served by several blocks each. which: bit 0 = some row is greedy
//   or has a cut, bit 1 = some row has a temperature and no cut; 3 if the caller does not know.
//   A kernel whose rows are promised absent is not launched.
size_t lse_sample_scratch_ints(int rows);
int lse_sample(const float* logits, int R, int V, const float* temperature, const int* top_k,
               const float* top_p, const float* min_p, const uint64_t* seed, const int* draw,
               int* out_tokens, int* scratch, int scratch_rows, int which,
               cudaStream_t stream);

// out[r] = log(sum_i exp(logits[r, i]))
int lse_logsumexp(const float* logits, int R, int V, float* out, cudaStream_t stream);

// logits[row, token] += / *= per the penalties; entries are unique (row, token) pairs.
int lse_apply_penalties(float* logits, int V, const int* row, const int* token, const int* count,
                        const float* presence, const float* frequency, const float* repetition,
                        int n, cudaStream_t stream);

// logits[row[i], token[i]] = -inf
// Token state of the penalties on the device: state[slots, V] int32, low 30 bits = times
// generated, bit 30 = occurs in the prompt. lse_token_state_add enters n (slot, token) pairs
// (in_prompt[i] != 0: mark as prompt token; else count one more generation).
// lse_apply_penalties_dense applies presence / frequency / repetition (the rule above) to logits
// row row[j] from the state of slot[j], for j < n.
int lse_token_state_add(int* state, int V, const int* slot, const int* token, const int* in_prompt,
                        int n, cudaStream_t stream);
int lse_apply_penalties_dense(float* logits, int V, const int* row, const int* slot,
                              const float* presence, const float* frequency, const float* repetition,
                              const int* state, int n, cudaStream_t stream);
int lse_ban_tokens(float* logits, int V, const int* row, const int* token, int n,
                   cudaStream_t stream);

// ---- parts with a running state per request, and blocks that norm a branch's output
// (state_mixers.cu). A sequence whose first row of the step is at position 0 (ctx_lens - rows
// == 0) starts from a zero state, whatever its slot holds.

// out = x in out_dtype
int lse_cast(const float* x, void* out, int out_dtype, long long n, cudaStream_t stream);

// out[t] = x[t] + (x[t-1] - x[t]) * mix, with x[t-1] from state[slots[seq]] for a sequence's first
// row; afterwards state[slots[seq]] = the sequence's last row of x.   x float32 [T, W]
int lse_token_shift(const float* x, const float* mix, float* state, void* out, int out_dtype,
                    const int* token_seq, const int* cu_q, const int* ctx_lens, const int* slots,
                    int T, int W, cudaStream_t stream);

// y = a, or with wa: ca * wa * a / rms(a) (+ cb * wb * b / rms(b) if b); x += w * y / rms(y);
// out (may be null) = the new x in out_dtype. rms(v) = sqrt(mean(v^2) + eps), eps_in for a and b.
// branch_dtype: LSE_F32, or LSE_FIXED64 when a (and b) are the sums of few-rows products, which are
// taken (left zero); then H * (b ? 2 : 1) floats must fit 48 KB of shared memory. With then_w,
// out = then_w * x / rms(x) of the new x (eps then_eps) instead of the new x itself.
int lse_rmsnorm_add(float* x, const void* a, const void* b, int branch_dtype, const float* wa,
                    const float* wb, float ca, float cb, float eps_in, const float* w, float eps,
                    void* out, int out_dtype, const float* then_w, float then_eps, int T, int H,
                    cudaStream_t stream);
// out = ca * wa * a / rms(a) (+ cb * wb * b / rms(b) if b)
int lse_mix_normed(const float* a, const float* b, const float* wa, const float* wb, float ca,
                   float cb, float eps, float* out, int T, int H, cudaStream_t stream);

// out[t, g*group + i] = o[t, g*group + i] / rms(o[t, group g]) * weight[g*group + i] (if weight)
//                       * act(gate[t*gate_stride + g*group + i]),  act = silu or (sigmoid != 0) sigmoid
int lse_gated_group_norm(const float* o, const float* gate, long long gate_stride, int T, int N,
                         int group, const float* weight, float eps, int sigmoid, void* out,
                         int out_dtype, cudaStream_t stream);

// qkv float32 [T, (nq + nk + (v_from_k ? 0 : nk)) * D]. q and k heads: divided by their root mean
// square and multiplied by qw / kw [D] (if given), then rotated (cos/sin [positions, D/2], if
// given). q goes to q_out [T, nq*D] of `dtype`; k into k_pages; v (the value heads, or with
// v_from_k the key heads as projected, before norm and rotation) into v_pages. Pages
// [pages, nk, page_tokens, D] of `dtype`, or both null when the layer only reads. D <= 256.
// norm_dim: the mean of the norm is taken over this many dims (the rest of a head is zero padding).
int lse_norm_rope_kv_write(const float* qkv, void* q_out, int dtype, int T, int nq, int nk, int D,
                           int v_from_k, const float* qw, const float* kw, float eps,
                           const int* positions, const int* token_seq, const float* cos,
                           const float* sin, void* k_pages, void* v_pages, const int* block_tables,
                           int table_stride, int page_tokens, int norm_dim, cudaStream_t stream,
                           long long row_stride = 0);  // of qkv, in elements (0: dense rows)

// Linear attention with a decay per head, token by token in float32:
//   S_t = decay[h] * S_{t-1} + k_t v_t^T,  out_t = S_t^T q_t
// proj [T, stride]: per row q (H*dk) | k (H*dk) | v (H*dv) | anything else. silu != 0: silu on q,
// k and v. The first `rot` dims of q and k are rotated (pairs (i, i + rot/2), cos/sin
// [positions, rot/2]); k is then multiplied by key_scale. state [slots, H, dv, dk] float32.
// dk <= 256. A portion of more than lse_linear_attention_chunk() tokens runs as chunks side by
// side (three launches); max_chunks is the largest number of chunks of any sequence of the step
// (or a bound on it), and chunks a scratch of (sum over sequences with more than one chunk of
// their chunks) * H * dv * dk floats, needed when max_chunks > 1.
int lse_linear_attention_chunk(void);
int lse_decay_linear_attention(const float* proj, long long stride, float* out, float* state,
                               const float* decay, const int* cu_q, const int* ctx_lens,
                               const int* slots, int num_seqs, int H, int dk, int dv,
                               const float* cos, const float* sin, int rot, int silu,
                               float key_scale, int max_chunks, float* chunks, cudaStream_t stream,
                               // a decay per key channel and token, alpha = sigmoid(z)^(1/decay_root),
                               // z = gate_z[t, h*dk + i] (decay may then be null); q is multiplied by
                               // query_scale; chunk_decay: scratch of (chunks as above) * H * dk floats.
                               // total_rows: rows of proj and gate_z. With max_chunks > 1 and total_rows > 0
                               // gate_z is overwritten with the decays (it is the caller's temporary).
                               const float* gate_z = nullptr, long long gate_stride = 0, float decay_root = 1.f,
                               float query_scale = 1.f, float* chunk_decay = nullptr, int total_rows = 0);
// ---- several residual streams, rows of q/k/v prepared a token at a time, differential attention
// (streams_mixers.cu). The residual state is float32 [T, S * W]: a token's S streams of W values.

// out[t, s*W + i] = x[t, i] * scale for every stream s.
int lse_streams_spread(const float* x, float* out, int T, int W, int S, float scale, cudaStream_t stream);

// out[r] = u / rms(u) * w with u = sum_s read[s] * x[t, s], t = rows ? rows[r] : r. S <= 16.
int lse_streams_read_norm(const float* x, const float* read, const float* w, float eps, void* out,
                          int out_dtype, const int* rows, int n_rows, int W, int S, cudaStream_t stream);

// x[t, r] <- sum_s mix[s*S + r] * x[t, s] + outw[r] * scale * y[t] for all r at once (scale [W] or
// null). y: LSE_F32, LSE_BF16, or LSE_FIXED64 sums (taken: left zero; W a multiple of 4). With
// then_read: also out[t] = u / rms(u) * then_w, u = sum_r then_read[r] * (new) x[t, r].
int lse_streams_write(float* x, const void* y, int y_dtype, const float* scale, const float* mix,
                      const float* outw, int T, int W, int S, const float* then_read, const float* then_w,
                      float then_eps, void* out, int out_dtype, cudaStream_t stream);

// proj float32 [T, stride]: nq query heads of D, nk key heads of D, then nv value heads of Dv
// (nv == 0: a key head's value is the key as projected; otherwise nk is a multiple of nv and value
// head g goes to the pages of key heads g*nk/nv ..). With qw/kw ([nq*D], [nk*D]): q and k divided
// by the root mean square of all their values of the token and multiplied by the weights. With
// temp_every > 0: q *= 1 + temp_coef * ln((pos + 1) / temp_every + 1) (integer division). With
// cos/sin [positions, rot/2]: the first rot dims of every q and k head turned, dim i paired with
// i + rot/2. q goes to q_out [T, nq*Dp], k and v into pages [pages, nk, page_tokens, Dp] of
// `dtype` (or both null when the layer only reads); dims from D (Dv) up to Dp are zero.
int lse_qkv_norm_rope_write(const float* proj, long long stride, int T, int nq, int nk, int nv, int D, int Dv,
                            int Dp, const float* qw, const float* kw, float eps, float temp_coef,
                            int temp_every, const int* positions, const int* token_seq, const float* cos,
                            const float* sin, int rot, void* q_out, void* k_pages, void* v_pages, int dtype,
                            const int* block_tables, int table_stride, int page_tokens, cudaStream_t stream);

// a [T, 2H*Dp]: for every key group of n heads, the heads' first attention maps, then their second
// ones. out[t, h] (Dv values) = o / rms(o) * out_scale * sigmoid(gate[t*gate_stride + h]),
// o = a1 - lam * a2 over the first Dv dims. a and out have the same dtype, or a is float32 and out
// bfloat16. Dv <= 256.
int lse_differential_combine(const void* a, int a_dtype, const float* gate, long long gate_stride, int T,
                             int H, int n, int Dp, int Dv, float lam, float eps, float out_scale, void* out,
                             int out_dtype, cudaStream_t stream);

// ---- table-sum embeddings, latent attention, routed experts (latent_moe.cu)

// x[t] += table[row], row = (previous token * mul_prev + token * mul_cur) mod buckets, or row
// `buckets` (the table's last) at position 0. The previous token of a sequence's first row of the
// step is state[slots[seq]] (int32, one per slot); afterwards the state holds the sequence's last
// token of the step.   x float32 [T, W], table [buckets + 1, W]
int lse_hashed_pair_add(float* x, const void* table, int table_dtype, int* state, const int* ids,
                        const int* positions, const int* token_seq, const int* cu_q,
                        const int* slots, int T, int num_seqs, int W, long long buckets,
                        long long mul_prev, long long mul_cur, cudaStream_t stream);

// x[t, i] += sin(p * freq[i / 2]) for even i, cos(...) for odd i; p = float(positions[t])
int lse_sinusoid_add(float* x, const int* positions, const float* freq, int T, int W,
                     cudaStream_t stream);

// Row t of proj (columns col0 .. col0 + R - 1, row stride `stride`) divided by its root mean
// square (eps inside the root), times weight[R], written as `dtype` into the token's place of
// pages [pages, 1, page_tokens, Rp]; columns R .. Rp - 1 are written as zeros.
int lse_latent_write(const void* proj, int in_dtype, long long stride, int col0, int R, int Rp,
                     const float* weight, float eps, void* pages, int dtype, const int* positions,
                     const int* token_seq, const int* block_tables, int table_stride,
                     int page_tokens, int T, cudaStream_t stream);

// A product per head: out[t, h*N + n] = sum_k a[t*a_stride + a_col0 + h*K + k] * w[(h*N + n)*K + k]
// with float32 accumulation in ascending k by one thread (a row's result does not depend on T).
// Served: (a, w, out) = (f32, f32, f32), (f32 | bf16, bf16, bf16 | f32).
// kind: 0 = CUDA cores; 1 = mma.sync tensor-core tiles; 2 = a kernel for few rows that streams the
// weights once. 1 and 2 need bfloat16 a and w with K, a_stride and a_col0 multiples of 8 (else the
// call is served as kind 0).
// a_head_cols: columns between the heads of a (0: K); out_head_cols: columns between the heads of
// out (0: N), out_stride its row length (0: H * out_head_cols): a head's result may be the first
// part of a wider slot whose rest another kernel fills.
int lse_head_linear(const void* a, int a_dtype, long long a_stride, long long a_col0, const void* w,
                    int w_dtype, void* out, int out_dtype, int T, int H, int N, int K, int kind,
                    cudaStream_t stream, long long a_head_cols = 0, long long out_head_cols = 0,
                    long long out_stride = 0);

// Routed experts. h [T, W]; router float32 [E (+1), W].
//   lse_moe_route: z = router . h (+ bias); idx [T, top] the experts with the largest z (largest
//     first, the lower index on a tie). mode 0: wts = sigmoid(z) of the chosen; mode 1: wts = the
//     softmax over the chosen z alone. With has_gate, gate[t] = sigmoid(router[E] . h).
//   lse_moe_sort: the n = T * top choices sorted by expert: offsets [E + 1], perm [n] (sorted row ->
//     choice), pos_of [n] (choice -> sorted row), and tiles of at most lse_moe_tile_rows() rows of one
//     expert each (tile_batch, tile_row0: room for n / tile_rows + E entries; num_tiles [1]);
//     tile_rows is lse_moe_tile_rows() for lse_expert_linear.
//   lse_expert_linear: out[r, :] = w[expert of r] . arow(r) for every sorted row r, float32 out
//     [rows, N]; arow(r) = a[a_rows[r] / a_div] * a_scale[a_rows[r]] (a_rows null: a[r], unscaled);
//     w [E, N, K]. Launched for max_tiles tiles; tiles beyond *num_tiles do nothing. kind as above
//     (kinds 1 and 2 multiply the float32 sums by a_scale, which is the same product).
//   lse_moe_combine: out[t] (+)= sum_k wts[t*top + k] * y[pos_of[t*top + k]] (+ gate[t] * shared_out[t]);
//     wts null: 1; gate null: 1.
int lse_moe_tile_rows(void);
int lse_moe_route(const void* h, int h_dtype, const float* router, int T, int W, int E, int has_gate,
                  int top, int* idx, float* wts, float* gate, cudaStream_t stream,
                  const float* bias = nullptr, int mode = 0);
int lse_moe_sort(const int* idx, int n, int E, int tile_rows, int* offsets, int* perm, int* pos_of,
                 int* tile_batch, int* tile_row0, int* num_tiles, cudaStream_t stream);
// out[r] = a[perm[r] / top] for the n sorted rows (bfloat16, K a multiple of 8)
int lse_moe_gather_rows(const void* a, const int* perm, int top, void* out, int n, int K,
                        cudaStream_t stream);
// lse_expert_linear for bfloat16 rows that already lie sorted (a [rows, K], K a multiple of 8), on
// tcgen05 tensor cores (grouped_gemm_tc.cu); the tiles must hold lse_expert_linear_tc_tile_rows()
// rows. out[r] is multiplied by scale[perm[r]] if scale is given.
int lse_expert_linear_tc_tile_rows(void);
int lse_expert_linear_tc(const void* a, const void* w, float* out, int rows, int E, int N, int K,
                         const float* scale, const int* perm, const int* offsets,
                         const int* tile_batch, const int* tile_row0, const int* num_tiles,
                         int max_tiles, int* error_flag, cudaStream_t stream);
int lse_expert_linear(const void* a, int a_dtype, long long a_stride, const int* a_rows, int a_div,
                      const float* a_scale, const void* w, int w_dtype, float* out, int rows, int N,
                      int K, const int* offsets, const int* tile_batch, const int* tile_row0,
                      const int* num_tiles, int max_tiles, int kind, cudaStream_t stream);
int lse_moe_combine(const float* y, const int* pos_of, int top, const float* shared_out,
                    const float* gate, float* out, int accumulate, int T, int W, cudaStream_t stream,
                    const float* wts = nullptr);

// Latent attention with a rotated key part (rotary_latent.cu). cos/sin: float32 [positions, rot/2];
// neighbouring dims (2i, 2i+1) are a pair; of a part's Dr dims the first rot are turned.
//   lse_latent_rope_write: per row of proj (row length `stride`): if Rq > 0, columns q_col0 .. +Rq
//     RMS-normed with q_weight into cq [T, Rq]; if R > 0, columns kv_col0 .. +R RMS-normed with
//     kv_weight and the Dr columns behind them turned by the token's position, written as one row
//     [R | Dr | zeros up to Rp] at the token's place of pages [pages, 1, page_tokens, Rp].
//   lse_latent_query_rope: q [T, H, D + Dr]; out [T, H, Rp]: dims R .. R + Dr of every head take the
//     head's last Dr query dims turned by the position, dims R + Dr .. Rp zeros; dims below R are
//     not touched.
//   lse_sigmoid_gate_mul: o[t, i] *= sigmoid(g[t * g_stride + col0 + i / group]) for i < N.
//   lse_act_rows: out[i] = act(in[i]); act 0: relu(z)^2, 1: relu, 2: gelu_tanh, 3: silu. `in` may be
//     fixed-point sums (LSE_FIXED64, bfloat16 out), which are left zero.
int lse_latent_rope_write(const void* proj, int in_dtype, long long stride, int q_col0, int Rq,
                          const float* q_weight, void* cq, int kv_col0, int R, int Dr, int rot,
                          const float* kv_weight, float eps, const float* cos, const float* sin,
                          void* pages, int Rp, int dtype, const int* positions, const int* token_seq,
                          const int* block_tables, int table_stride, int page_tokens, int T,
                          cudaStream_t stream);
int lse_latent_query_rope(const void* q, int dtype, int T, int H, int D, int Dr, int rot,
                          const float* cos, const float* sin, const int* positions, void* out, int R,
                          int Rp, cudaStream_t stream);
int lse_sigmoid_gate_mul(void* o, int dtype, const void* g, int g_dtype, long long g_stride, int col0,
                         int group, int T, int N, cudaStream_t stream);
int lse_act_rows(const void* in, int in_dtype, void* out, int dtype, long long total, int act,
                 cudaStream_t stream);
}
