// Launchers of every kernel.  All pointers are device pointers; `stream` is the
// CUDA stream to launch on.  dtype: 0 = float32, 1 = bfloat16 (dlmk::DType).
// Launchers validate sizes and throw std::invalid_argument for what a kernel
// cannot take; none of them allocates memory.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace dlmk {

enum Epilogue : int {
    EPI_STORE = 0,    // out[m, n] = acc (+ bias[n]), stored as the output dtype
    EPI_ADD = 1,      // out[m, n] += acc, out is float32 (the residual stream)
    EPI_SWIGLU = 2,   // out[m, n/2] = silu(acc[m, n]) * acc[m, n+1] for even n (interleaved weight rows)
    EPI_GELU = 3,     // out[m, n] = gelu(acc (+ bias[n])) in its exact (erf) form, stored as the output dtype
    EPI_GELU_TANH = 4 // the same with gelu in its tanh form: z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))) / 2
};

// out[T, H] (f32) = table[tokens[t], :] * scale
void embed(const int32_t* tokens, const void* table, float* out, int T, int H, int V, float scale, int dtype,
           cudaStream_t stream);

// out[i, :] = x[rows ? rows[i] : i, :] * rsqrt(mean(x^2) + eps) * w      (x, w f32; out dtype given)
void rmsnorm(const float* x, const float* w, void* out, const int32_t* rows, int n_rows, int H, float eps,
             int out_dtype, cudaStream_t stream);

// C[M, N] = A[M, K] · W[N, K]^T with an epilogue.  Dense: expert_offsets == nullptr.
// Grouped: rows [expert_offsets[e], expert_offsets[e+1]) use W + e * w_expert_stride elements.
// a_rows (optional) gathers the rows of A: row m of the product reads A[a_rows[m], :].
// `fast` != 0 allows tensor-core kernels (bfloat16 inputs only); 0 forces the plain FMA kernel.
// expert_offsets are read before the kernel launched just before this one has ended (the tensor-core kernel lists
// its tiles while it is set up): that kernel must not be the one that writes them (in a layer a gather or the
// experts' first product lies in between).
void gemm(const void* a, int lda, const int32_t* a_rows, const void* w, int ldw, long long w_expert_stride,
          const int32_t* expert_offsets, int num_experts, const float* bias, void* out, int ldo, int M, int N, int K,
          int in_dtype, int out_dtype, int epilogue, int fast, cudaStream_t stream);

// True when the tcgen05 / TMA matrix kernel can be used (it needs the driver's tensor-map encoder; the
// environment variable DLM_B200_NO_TCGEN05=1 switches it off).
bool gemm_tc_enabled();

// out[i, :] = src[rows[i], :] for bfloat16 / float32 rows of `width` elements (width * element size a multiple
// of 16 bytes): the gather that puts an expert's rows side by side before a grouped product.
void gather_rows(const void* src, const int32_t* rows, void* out, int n_rows, int width, int dtype,
                 cudaStream_t stream);

// Rotates q and k heads of qkv[T, (nh + 2 nkv) * hd] (f32) by position * inv_freq within the first rotary_dim
// dims (pair i is dims (i, i + rotary_dim / 2), or (2i, 2i + 1) with interleaved != 0; inv_freq == nullptr: no
// rotation), writes q to q_out[T, nh * hd] and, where slots != nullptr and slots[t] >= 0, k and v to the paged
// caches [pages, nkv, page_size, hd].  positions, slots and inv_freq are read before the kernel launched just
// before this one has ended (they are a step's inputs): that kernel must not be the one that writes them.
void rope_kv_write(const float* qkv, const int32_t* positions, const float* inv_freq, int rotary_dim, int interleaved,
                   const int32_t* slots, void* q_out, void* k_cache, void* v_cache, int T, int nh, int nkv, int hd,
                   int page_size, int total_pages, int dtype, cudaStream_t stream);

// Causal (optionally windowed) attention of every token of the step over its request's paged keys and values.
// A score is dot * scale - slopes[query head] * (query position - key position); slopes (f32 [nh], made at load,
// never written by a kernel) == nullptr: no distance term.  chunk > 0: a query at p sees only keys from
// floor(p / chunk) * chunk on (chunks are counted from a request's position 0).  sinks (f32 [nh]) != nullptr: the
// softmax's denominator also holds exp(sinks[head]), unscaled, without key or value.  softcap c > 0: the scaled dot
// product becomes c * tanh(dot * scale / c) before the distance term and the mask.
// num_single: how many requests have exactly one query token.  With fast != 0 and a scratch buffer of
// attention_scratch_floats(...) floats those go to the split-key decode kernel.
void attention(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_table, int table_width,
               const int32_t* cu_q, const int32_t* kv_len, void* out, int T, int R, int nh, int nkv, int hd,
               int page_size, int total_pages, int window, float scale, const float* slopes, int chunk,
               const float* sinks, float softcap, int max_q_len, int max_kv_len, int num_single, float* scratch, int dtype,
               int fast, cudaStream_t stream);
// Floats of scratch the decode kernel needs for a step of R requests whose longest holds max_kv_len tokens.
size_t attention_scratch_floats(int R, int nh, int nkv, int hd, int max_kv_len);

// Router: logits = h · w^T (32-bit); scores = softmax over E (score_fn 0) or sigmoid of each logit (score_fn 1);
// score_fn 2: softmax as for 0, but select_bias[E] is the router's own bias and is added to the logits first
// (it then enters scores and choice alike; with norm != 0 the weights are the softmax over the chosen logits);
// the k best scores (ties: lower index; with select_bias[E] the choice is made on score + bias and the weight
// stays the score); norm != 0: the chosen weights are divided by their sum (norm 2: by their sum + 1e-20); all are
// multiplied by `scale`.
// has_gate: w has E + 1 rows and gate[t] = sigmoid(h · w[E]).  The input h is: activations of the weights' dtype
// (default); the 32-bit residual, with rmsnorm(h, norm_w, eps) applied first in 32-bit (norm_w != nullptr); or
// 32-bit activations that are already normalised (h_is_f32 != 0).  dtype is the weights' dtype.
// logits: scratch of T * (E + has_gate) floats (the router logits are left there).
void router_topk(const void* h, const void* w, const float* norm_w, float eps, float* logits, int32_t* ids, float* wts,
                 float* gate, int T, int H, int E, int k, int norm, int has_gate, int dtype, int h_is_f32,
                 int score_fn, float scale, const float* select_bias, int x_settled, cudaStream_t stream);

// router_topk followed by moe_permute (below).  One launch up to 16 tokens (blocks of 8 experts per token, the
// block that finishes last chooses for every token and groups) and from 17 to 48 tokens (a block per token
// computes all its logits and chooses; the last block groups); three launches from 49 tokens on.  Returns the
// number of launches.  x_settled != 0: `h` was written before the kernel launched just before this one began its
// work (a step's residual, with a norm kernel in between): the logits of at most 16 tokens, or the first of 512
// and more, are then worked out while that kernel ends (`router_topk` takes the same flag).
int router_topk_permute(const void* h, const void* w, const float* norm_w, float eps, float* logits, int32_t* ids,
                         float* wts, float* gate, int32_t* offsets, int32_t* rows, int32_t* dest, int T, int H, int E,
                         int k, int norm, int has_gate, int dtype, int h_is_f32, int score_fn, float scale,
                         const float* select_bias, int x_settled, cudaStream_t stream);

// Groups the n = T * k (token, choice) pairs by expert: offsets[E + 1], rows[n] = token of each sorted row,
// dest[n] = sorted row of pair (t, j).
void moe_permute(const int32_t* ids, int n, int k, int E, int32_t* offsets, int32_t* rows, int32_t* dest,
                 cudaStream_t stream);

// resid[t, :] += sum_j wts[t, j] * y[dest[t, j], :] (+ shared_scale * gate[t] * shared[t, :]); gate == nullptr: 1.
// ids (i32 [T, k]) != nullptr: a pair whose expert id is num_real or more reads passthrough[t, :] (f32 [T, H]) in
// place of its row of y (an expert that hands its input through; y may then be nullptr when num_real is 0).
void moe_combine(const float* y, const int32_t* dest, const float* wts, const float* shared, const float* gate,
                 float* resid, int T, int H, int k, const int32_t* ids, int num_real, const float* passthrough,
                 float shared_scale, cudaStream_t stream);

// out[i] = index of the first maximum of logits[i, :].  scratch: argmax_scratch_bytes(N, V) bytes (may be
// nullptr when that is 0; a large vocabulary is then searched by one block per row).
void argmax(const float* logits, int32_t* out, int N, int V, void* scratch, cudaStream_t stream);
size_t argmax_scratch_bytes(int N, int V);

// Per row: repetition penalty over seen tokens, then greedy (temperature <= 0) or temperature / top-k / top-p /
// min-p sampling with the uniform number u[i] (candidates ordered by logit descending, ties by index).
// seen_offsets[N + 1] indexes seen_tokens; params[i] = {temperature, top_p, min_p, repetition_penalty}; top_k[i].
// scratch: N * V floats.
void sample(const float* logits, int32_t* out, int N, int V, const float* params, const int32_t* top_k,
            const float* u, const int32_t* seen_offsets, const int32_t* seen_tokens, float* scratch,
            cudaStream_t stream);

// A device-side error flag kernels set instead of touching memory they must not (a page id outside the pool,
// an expert id outside the table).  Returns the flag and clears it.
int take_error_flag();

// Clears what a decode attention launch that ended through a bounded wait's give-up path (error 5) may have
// left in the split-merge counters, so that later steps merge correctly.  Call after take_error_flag() == 5.
void reset_decode_merge_counters(cudaStream_t stream);

// Whether the small kernels are launched so that each may start while the one before it ends
// (programmatic dependent launch; on unless DLM_B200_NO_PDL=1).
bool dep_launch_enabled();
void set_dep_launch(bool on);

// ---- learned positions, residual streams, convolutions over time, state-carrying mixers (seqmix.cu) ----

// x[t, :] += table[idx[t], :]   (x f32; table of `rows` rows in `dtype`; an index outside the table sets error 6)
void add_rows(float* x, const void* table, const int32_t* idx, int T, int H, int rows, int dtype, cudaStream_t stream);

// xs[t, s, :] = x[t, :] for s < S  (both f32)
void streams_expand(const float* x, float* xs, int T, int S, int H, cudaStream_t stream);
// u[t, :] = sum_s a[s] xs[t, s, :] (a == nullptr: every weight 1); norm_w != nullptr: out = u / sqrt(mean(u^2) + eps)
// * norm_w, else out = u.  xs f32 [T, S, H]; out [T, H] in out_dtype.
void streams_reduce(const float* xs, const float* a, const float* norm_w, float eps, void* out, int T, int S, int H,
                    int out_dtype, cudaStream_t stream);
// xs[t, r, :] <- sum_s mix[s, r] xs[t, s, :] + outw[r] * y[t, :]  (in place, all streams from the old ones; S <= 16)
void streams_update(float* xs, const float* mix, const float* outw, const float* y, int T, int S, int H,
                    cudaStream_t stream);

// streams_update followed by streams_reduce with the next sublayer's weights, in one pass (S <= 8): xs is updated in
// place and out[t, :] = rmsnorm(sum_r in_next[r] xs_new[t, r, :]) * norm_w (norm_w == nullptr: the sum itself).
void streams_update_reduce(float* xs, const float* mix, const float* outw, const float* y, const float* in_next,
                           const float* norm_w, float eps, void* out, int T, int S, int H, int out_dtype,
                           cudaStream_t stream);

// Causal convolution over time on each channel, per request, with the request's last taps - 1 inputs carried in
// state[slots, taps - 1, C] (f32, zero at a request's start) and brought up to date by the call:
// out[t, c] = (add_input ? x[t, c] : 0) + bias[c] + sum_j w[c, j] x[t - taps + 1 + j, c]; act 1: silu of that.
// x f32 with row stride ldx; w f32 [C, taps]; bias f32 [C] or nullptr; out in out_dtype with row stride ldo.
void causal_conv(const float* x, int ldx, const float* w, const float* bias, float* state, const int32_t* cu_q,
                 const int32_t* token_req, const int32_t* state_slot, int T, int R, int C, int taps, int add_input,
                 int act, void* out, int ldo, int out_dtype, cudaStream_t stream);

// out[r, c] = f(x[r, c]); op 0 tanh, 1 gelu (erf), 2 silu, 3 gelu (tanh form), 4 copy.  x f32, out in out_dtype.
void activation(const float* x, int ldx, void* out, int ldo, int rows, int cols, int op, int out_dtype,
                cudaStream_t stream);

// ids[t, j] = table[tokens[t], j], wts[t, j] = 1 / top  (table int32 [V, top] of expert ids below E)
void table_lookup(const int32_t* tokens, const int32_t* table, int32_t* ids, float* wts, int T, int V, int top, int E,
                  cudaStream_t stream);

// Norm over groups of `group_size` channels with a gate.  mode 0: v = y * silu(gate), out = v / rms(v) * w;
// mode 1: out = y / rms(y) * w * sigmoid(gate); mode 2: out = y / rms(y) * w * silu(gate).  y, gate f32 (row strides
// ldy, ldg), w f32 [groups * group_size] or nullptr (every weight 1).  row_scale (f32 [T, groups], modes 1 and 2) !=
// nullptr: y[t, group] is multiplied by row_scale[t, group] before anything else.
void gated_rmsnorm(const float* y, int ldy, const float* gate, int ldg, const float* w, void* out, int ldo, int T,
                   int groups, int group_size, float eps, int mode, int out_dtype, const float* row_scale,
                   cudaStream_t stream);

// State-space scan.  xbc f32 rows [x: heads * P | B: groups * N | C: groups * N]; dt_raw f32 [T, heads] (row stride
// lddt); state f32 [slots, heads, N, P]; y f32 [T, heads * P].  Per head (group = head / (heads / groups)):
// dt = softplus(dt_raw + dt_bias); S <- exp(-exp(A_log) dt) S + dt B x^T; y = S^T C + D x.
// fixed_decay f32 [heads] != nullptr: S <- fixed_decay[head] S + B x^T instead (step size 1; dt_raw, dt_bias and
// A_log are not read); D == nullptr: no direct term.  With groups == heads and rows [v | k | q] this is linear
// attention with a constant decay per head: S <- decay S + k v^T, y = S^T q.
void ssm_scan(const float* xbc, int ldx, const float* dt_raw, int lddt, const float* dt_bias, const float* A_log,
              const float* D, float* state, const int32_t* cu_q, const int32_t* state_slot, float* y, int R, int heads,
              int P, int N, int groups, const float* fixed_decay, cudaStream_t stream);

// Delta-rule scan.  proj f32 rows hold r, k, v and the raw removal rate at the given column offsets (heads * d
// each); lw f32 [T, heads * d] the raw decay; state f32 [slots, heads, d, d] (key channel, value channel).
// w = exp(-decay_coef * sigmoid(lw)); a = sigmoid(a_raw + a_bias); u = k / sqrt(sum k^2 + unit_eps);
// S <- diag(w) S - (a u)(u^T S) + k v^T; o = S^T r  (o f32 [T, heads * d]).
void delta_scan(const float* proj, int ld, int off_r, int off_k, int off_v, int off_a, const float* lw, int ldlw,
                const float* a_bias, float* state, const int32_t* cu_q, const int32_t* state_slot, float* o, int R,
                int heads, int d, float unit_eps, float decay_coef, cudaStream_t stream);

// ---- diagonal state-space scan and mixers that run side by side (scanmix.cu) ----

// Selective scan with a step size per channel and token.  x f32 [T, inner] (after its convolution and activation),
// dt_raw f32 [T, inner], bc f32 rows [B: N | C: N], z f32 [T, inner] (row strides given); A_log f32 [inner, N],
// dt_bias and D f32 [inner]; state f32 [slots, inner, N].  Per channel c and state n, with dt = softplus(dt_raw +
// dt_bias): S[c, n] <- exp(-exp(A_log[c, n]) dt) S[c, n] + dt x_c B_n; y_c = sum_n S[c, n] C_n + D_c x_c;
// out[t, c] = y_c * silu(z_c) in out_dtype.
void selective_scan(const float* x, int ldx, const float* dt_raw, int lddt, const float* bc, int ldbc, const float* z,
                    int ldz, const float* dt_bias, const float* A_log, const float* D, float* state,
                    const int32_t* cu_q, const int32_t* state_slot, void* out, int ldo, int R, int inner, int N,
                    int out_dtype, cudaStream_t stream);

// qkv f32 rows [q: nh * d | k: nkv * d | v: nkv * dv] (row stride ld).  q <- q / rms(q over all nh * d entries) * qn_w
// * (1 + temp_coef * ln(floor((position + 1) / temp_every) + 1)); k likewise with kn_w and no temperature (a weight
// pointer of nullptr: that projection is not normed; temp_every 0: no temperature).  q goes to q_out[T, nh * D] and,
// where slots != nullptr and slots[t] >= 0, k and v to the paged caches [pages, nkv, page_size, D], every head D
// wide with zeros beyond its own size (D >= d, dv).
void qk_norm_write(const float* qkv, int ld, const int32_t* positions, const float* qn_w, const float* kn_w, float eps,
                   float temp_coef, int temp_every, const int32_t* slots, void* q_out, void* k_cache, void* v_cache,
                   int T, int nh, int nkv, int d, int dv, int D, int page_size, int total_pages, int dtype,
                   cudaStream_t stream);

// Rotary positions in place on f32 rows: two runs of `heads` heads of `dim` entries at columns off_a and off_b; the
// first rot_dims entries of a head are rotated (entry i with i + rot_dims / 2, angle position * inv_freq[i]), then
// the whole head is multiplied by the run's factor.
void rotate_heads(float* x, int ld, const int32_t* positions, const float* inv_freq, int rot_dims, int T, int heads,
                  int dim, int off_a, float scale_a, int off_b, float scale_b, cudaStream_t stream);

// resid[t, :] += coef * (a[t] / rms(a[t]) * wa + b[t] / rms(b[t]) * wb)   (all f32 [T, H]; b == nullptr: one branch)
void branch_norm_add(float* resid, const float* a, const float* wa, const float* b, const float* wb, float eps,
                     float coef, int T, int H, cudaStream_t stream);

// out_a[t] = x[t] / rms(x[t]) * wa, out_b[t] = x[t] / rms(x[t]) * wb  (x, wa, wb f32; outputs in out_dtype)
void rmsnorm_pair(const float* x, const float* wa, const float* wb, void* out_a, void* out_b, int T, int H, float eps,
                  int out_dtype, cudaStream_t stream);

// out[t, :] = [a[t, :] | b[t, :]] in out_dtype (a, b f32 [T, H])
void concat_rows(const float* a, const float* b, void* out, int T, int H, int out_dtype, cudaStream_t stream);

// ---- attention through a cached latent (latent_attention.cu) ----

// Per token: cq_out = rmsnorm(proj[off_q : +q_rank]) * qn_w (activation dtype); the cache row of slots[t]
// ([rank | dr] wide, pages [pages, 1, page_size, rank + dr]) = [rmsnorm(proj[off_kv : +rank]) * kvn_w |
// rotate(proj[off_kv + rank : +dr])].  Rotation on the first rot_dims entries, pair (i, i + rot_dims / 2), or
// (2i, 2i + 1) with interleaved != 0.  q_rank 0: there is no query latent and cq_out is not written.
void latent_prep(const float* proj, int ld, int off_q, int q_rank, const float* qn_w, int off_kv, int rank,
                 const float* kvn_w, int dr, const float* inv_freq, int rot_dims, int interleaved, const int32_t* positions,
                 const int32_t* slots, float eps, void* cq_out, void* cache, int page_size, int total_pages, int T,
                 int dtype, cudaStream_t stream);

// q f32 [T, H * (dn + dr)] (per head [dn plain | dr to be rotated]) -> qn[H, T, dn] in `dtype` (head by head: the
// left operand of the per-head product with W_uk) and qr[T, H, dr] f32, rotated (pairs as in latent_prep).
void latent_q_split(const float* q, int ldq, const int32_t* positions, const float* inv_freq, int rot_dims,
                    int interleaved, void* qn, float* qr, int T, int H, int dn, int dr, int dtype, cudaStream_t stream);
// Attention over the cached latents.  q_lat f32 [H, T, rank]: the heads' queries through W_uk; q_rot f32 [T, H, dr];
// sink f32 [H] or nullptr (a logit per head that joins the softmax's maximum and denominator only); cache
// [pages, 1, page_size, rank + dr] and lat[H, T, rank] (the normalised weighted sums of latent rows) in `dtype`.
// A query at position p sees keys j with 0 <= p - j < window (window 0: all).  n_splits (from
// latent_attention_splits) > 1 cuts every token's keys over that many blocks; `partial` then holds
// T * H * n_splits * (rank + 2) floats of scratch and a second kernel merges.  fast != 0 allows the tensor-core
// kernel (bfloat16, rank a multiple of 128 up to 512, dr a multiple of 8).
void latent_attention(const float* q_lat, const float* q_rot, const float* sink, const void* cache,
                      const int32_t* block_table, int table_width, const int32_t* token_req, const int32_t* positions,
                      void* lat, float* partial, int n_splits, int T, int H, int dr, int rank, int page_size,
                      int total_pages, int window, float scale, int dtype, int fast, cudaStream_t stream);
// out[t, h * dv + d] = val[h * T + t, d] * sigmoid(gate[t, h]) in `dtype` (val f32 [H, T, dv]; gate f32 raw, or nullptr)
void latent_gate_out(const float* val, const float* gate, int ldg, void* out, int T, int H, int dv, int dtype,
                     cudaStream_t stream);
// Splits that fill the machine for a step of T tokens whose longest visible range is max_keys (1 in 32-bit, where
// the order of every sum is fixed).
int latent_attention_splits(int T, int H, int rank, int dr, int max_keys, int dtype, int fast);

// ---- gated recurrences with a matrix state, per-head norms, sublayers with a norm on both sides (gatedmix.cu) ----

// Recurrence over each request's tokens with a state S [dk, dv] per head (state f32 [slots, heads, dk, dv]):
//   S <- diag(a) S;   u = beta (v - S^T k) (beta given) or u = v (beta == nullptr);   S <- S + k u^T;   o = S^T q.
// q, k f32 rows of qk_heads heads of dk entries (row strides ldq, ldk; head h reads q/k head h / (heads / qk_heads));
// v f32 rows of heads * dv; o f32 rows of heads * dv (stride ldo).  unit != 0: q and k are divided by
// sqrt(sum x^2 + unit_eps) per head first; q is multiplied by q_scale.  beta f32 [T, heads] raw (sigmoid is applied).
// decay_kind 0: one factor per head, a = exp(-exp(A_log[h]) softplus(dec[t, h] + dec_bias[h]));
// decay_kind 1: one per key channel, a_i = sigmoid(dec[t, h * dk + i])^(1 / tau).
void gated_scan(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* dec, int ldd,
                const float* beta, int ldb, const float* A_log, const float* dec_bias, float* state,
                const int32_t* cu_q, const int32_t* state_slot, float* o, int ldo, int R, int heads, int qk_heads,
                int dk, int dv, int unit, float unit_eps, float q_scale, int decay_kind, float tau,
                cudaStream_t stream);

// qkv f32 rows [q: nh * d | k: nkv * d | v: nkv * dv] (row stride ld).  Every q and k head is divided by its root
// mean square over d (eps inside the root) and multiplied by qn_w / kn_w (f32 [d], shared by the heads; nullptr: that
// side is not normed), then its first rot_dims entries are rotated by position * inv_freq[pair] (pair i is entries
// (i, i + rot_dims / 2), or (2i, 2i + 1) with interleaved != 0).  q goes to q_out[T, nh * D] and, where slots !=
// nullptr and slots[t] >= 0, k and v to the paged caches [pages, nkv, page_size, D], every head D wide with zeros
// beyond its own size (D >= d, dv).
void head_norm_rope_write(const float* qkv, int ld, const int32_t* positions, const float* qn_w, const float* kn_w,
                          float eps, const float* inv_freq, int rot_dims, int interleaved, const int32_t* slots,
                          void* q_out, void* k_cache, void* v_cache, int T, int nh, int nkv, int d, int dv, int D,
                          int page_size, int total_pages, int dtype, cudaStream_t stream);

// o[t, h * D + i] *= factor * sigmoid(gate[t * ldg + h]) in place (o in `dtype`, gate f32 raw)
void head_gate(void* o, const float* gate, int ldg, int T, int nh, int D, float factor, int dtype, cudaStream_t stream);

// resid[t] += (y[t] / rms(y[t])) * w_post; then, with w_next != nullptr, out[t] = (resid[t] / rms(resid[t])) * w_next
// in out_dtype: a sublayer's closing norm, the add to the residual and the next sublayer's opening norm in one pass.
void norm_add_norm(float* resid, const float* y, const float* w_post, const float* w_next, float eps, void* out, int T,
                   int H, int out_dtype, cudaStream_t stream);

// x[t, :] += (x0 != nullptr ? x0[t, :] : 0) + vec[:]   (all f32)
void add_vec_rows(float* x, const float* x0, const float* vec, int T, int H, cudaStream_t stream);

// The recurrence of gated_scan with exponential gates kept in range by a running maximum, and a normaliser:
//   i = cap tanh((igate[t, h] + i_bias[h]) / cap);   f = log sigmoid(cap tanh((fgate[t, h] + f_bias[h]) / cap));
//   m' = max(f + m, i);   S <- exp(f + m - m') S + exp(i - m') k v^T;   n <- exp(f + m - m') n + exp(i - m') k;
//   o = S^T q (q times q_scale);   rden[t, h] = 1 / (max(|n . q|, exp(-m')) + den_eps).
// q, k f32 rows of heads * dk, v of heads * dv (row strides given), igate and fgate f32 [T, heads] raw.  state f32
// [slots, heads, dk, dv], nstate [slots, heads, dk], mstate [slots, heads, dv + 1] (equal copies of m, one per column
// of a block; all zero at a request's start).  o f32 rows of heads * dv (not yet divided), rden f32 [T, heads].
void memory_scan(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* igate, int ldi,
                 const float* fgate, int ldf, const float* i_bias, const float* f_bias, float cap, float* state,
                 float* nstate, float* mstate, const int32_t* cu_q, const int32_t* state_slot, float* o, int ldo,
                 float* rden, int R, int heads, int dk, int dv, float q_scale, float den_eps, cudaStream_t stream);

// ---- layers that squash instead of norming (capmix.cu) ----

// out[i, :] = tanh(alpha * x[rows ? rows[i] : i, :]) * w + b   (x, w, b f32; out in out_dtype)
void dyt_norm(const float* x, const int32_t* rows, const float* w, const float* b, float alpha, void* out, int n_rows,
              int H, int out_dtype, cudaStream_t stream);
// The same rows through two such norms in one pass: out_a with (wa, ba, alpha_a), out_b with (wb, bb, alpha_b), and,
// with out_b32 != nullptr, the second result once more in 32-bit.
void dyt_norm_pair(const float* x, const float* wa, const float* ba, float alpha_a, void* out_a, const float* wb,
                   const float* bb, float alpha_b, void* out_b, float* out_b32, int T, int H, int out_dtype,
                   cudaStream_t stream);
// x[i] = cap * tanh(x[i] / cap) for n floats, in place
void tanh_cap(float* x, long long n, float cap, cudaStream_t stream);
// o[t, h * D + i] *= factor * sigmoid(gate[t * ldg + h * dv + i]) for i < dv, in place (o in `dtype`, gate f32 raw);
// resid (f32 [T, W]) != nullptr: also resid[t, :] += bias[:]
void entry_gate(void* o, const float* gate, int ldg, int T, int nh, int dv, int D, float factor, int dtype,
                float* resid, const float* bias, int W, cudaStream_t stream);

}  // namespace dlmk
