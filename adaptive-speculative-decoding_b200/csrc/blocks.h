// Host-side launchers of the sequence-model building blocks that take their sizes and constants as arguments
// (linear_simt.cu, stream_ops.cu, latent_attention.cu, moe.cu, norm_ops.cu, gla.cu, window_attention.cu).  An engine
// (mezilix_engine.cu, rivetar_engine.cu) strings them together;
// none of them knows a model.  `f32` flags select the element type of a buffer: 0 = bf16, 1 = fp32.  Norms, scores,
// softmax weights, router probabilities, the residual stream and the carried state are fp32 in both modes.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace asd {

// ---------------------------------------------------------------------------------------------- linear_simt.cu
// C[z][m][n] = epilogue( sum_k A[z][m][k] * W[z][n][k] ), fp32 FMA accumulation in increasing k (no tensor cores, no
// reduced-precision mode): the exact path of the fp32 engines and the fallback for shapes the tcgen05 GEMM refuses.
// A row of the result depends on nothing but its own A row, so it is identical however the rows are batched.
struct SimtLinear {
    const void* a = nullptr;  // element (z, m, k) at a + z * a_zs + row(m) * lda + k
    const void* w = nullptr;  // element (z, n, k) at w + z * w_zs + n * ldw + k
    void* c = nullptr;        // (z, m, n) at c + z * c_zs + m * ldc + n
    long long lda = 0, ldw = 0, ldc = 0, a_zs = 0, w_zs = 0, c_zs = 0;
    int a_f32 = 0, w_f32 = 0, c_f32 = 1;
    int M = 0, N = 0, K = 0, Z = 1;
    // grouped form (mixture of experts): rows of batch z are [group_off[z], group_off[z + 1]) of A and C (device array,
    // M = upper bound of rows per group, a_zs and c_zs ignored); gather (optional) maps such a row to its row of A
    const int* group_off = nullptr;
    const int* gather = nullptr;
    int epilogue = 0;         // 0 none, 1 relu(x)^2
};
int launch_simt_linear(const SimtLinear& L, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------- linear_tc.cu
// The same operation on tcgen05 (bf16 weights; bf16 or fp32 activations, rounded to bf16; fp32 accumulation in TMEM)
// for shapes it supports: K, ldw and the weight batch stride multiples of 8, 16-byte aligned bases, activation rows
// 16-byte aligned.  err_flag (device int, may be nullptr) is raised if a bounded wait inside the kernel ran out.
bool tc_linear_supports(const SimtLinear& L);
int launch_tc_linear(const SimtLinear& L, int* err_flag, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------- stream_ops.cu
// Carried per-sequence state: rings of `ring` entries indexed by position % ring, so that a caller that re-feeds the
// last few positions (speculative verification after a rejected tail) finds the state of any of them.
struct SeqIndex {
    const int* tokens;      // [M]
    const int* positions;   // [M]
    const int* token_slot;  // [M]
    int M;
};
// x0[m] = embed[token] + pair_table[(prev * mul_prev + token * mul_cur) % buckets] (row `buckets` at position 0), fp32;
// prev = the token one row up if that row is the same sequence's previous position, else tok_ring[slot][(pos-1) % ring].
// Also writes hn = x0 / rms(x0) * g (the first layer's scalar-gain RMS norm, fp32).
int launch_embed_pair(const SeqIndex& ix, const void* embed, const void* pair_table, int wf32, int buckets, int mul_prev,
                      int mul_cur, const int* tok_ring, int ring, float* x0, const void* g, float eps, float* hn, int D,
                      cudaStream_t stream);
// tok_ring[slot][pos % ring] = token for the last `ring` tokens of every run (after launch_embed_pair has read it)
int launch_commit_tokens(const SeqIndex& ix, int* tok_ring, int ring, cudaStream_t stream);
// Token shift: mixed = hn + (hn_prev - hn) * mu, hn_prev = the previous position's UNSHIFTED hn (row above, else
// state ring, zeros at position 0).  Writes h = hn and hs = mixed in the engine's element type.
int launch_token_shift(const SeqIndex& ix, const float* hn, const float* state_ring, int ring, const void* mu, int wf32,
                       void* h, void* hs, int of32, int D, cudaStream_t stream);
int launch_commit_shift_state(const SeqIndex& ix, const float* hn, float* state_ring, int ring, int D, cudaStream_t stream);
// Parallel-layer close with depth-weighted averaging of all earlier results:
//   X[i+1] = x_in + mix + sum_k gate[m][k] * expert_out[slot_of[m][k]]      (no expert term if top == 0)
//   x_next = sum_{j <= i+1} coeff[j] * X[j];  hn = x_next / rms(x_next) * g_next
// X is the stack [layers + 1][stack_stride] of fp32 [M][D] results (X[0] = embedding output); x_in may alias x_next.
struct LayerClose {
    const float* x_in;
    const float* mix;          // [M][D]
    const float* expert_out;   // [M * top][D] rows by slot
    const int* slot_of;        // [M][top]
    const float* gate;         // [M][top]
    int top;
    float* stack;
    size_t stack_stride;
    int layer;                 // i
    const void* coeff;         // [i + 2]
    const void* g_next;        // scalar gain of the norm that follows
    int wf32;
    float eps;
    float* x_next;
    float* hn;
    int M, D;
    // optional: before hn is overwritten, the rows that own a ring entry store their hn (this layer's normed input) as
    // the carried state of the token shift (what launch_commit_shift_state does, without its launch)
    const SeqIndex* ix = nullptr;
    float* state_ring = nullptr;
    int ring = 0;
};
int launch_layer_close(const LayerClose& L, cudaStream_t stream);
// dst[r] = src[rows[r]] converted to the engine's element type (rows == nullptr: identity)
int launch_select_rows(const float* src, const int* rows, void* dst, int of32, int n, int D, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------- latent_attention.cu
// Latent (low-rank) key/value attention with one shared rotated key part, evaluated in latent space: the cache holds
// per position [R latent | dr rotated key] and a query is first carried through the key up-projection, so that
//   score = scale * (q_lat . c + q_rot . k_rot),  out_lat = softmax . c,  and the value up-projection follows.
struct LatentDims {
    int heads, dn, dr, dv, R;   // per head: dn unrotated + dr rotated query dims, dv value dims; R latent size
    int rot_dims;               // leading coordinates of the rotated part that rotate (pairs i, i + rot_dims / 2)
    int window;                 // position p sees p - window < j <= p
    float scale;
    int interleaved = 0;        // 1: the rotating pairs are (2 i, 2 i + 1) instead of (i, i + rot_dims / 2)
};
struct PagedRows {
    void* pool;                // this layer's rows: [num_pages][page_size][row_elems]
    int f32;
    const int* page_table;     // [slots][max_pages]
    int max_pages, page_size;
};
// qd fp32 [M][heads * (dn + dr) + R + dr] = (queries head by head | latent | rotated key).  RMS-norms the latent (vector
// weight), rotates the key part and appends both to the paged cache; rotates every head's query part into
// q_lat[m][head][R .. R + dr) (fp32, row length R + dr).  inv_freq fp32 [rot_dims / 2].
int launch_latent_post(const SeqIndex& ix, const float* qd, const LatentDims& d, const void* c_norm, int wf32, float eps,
                       const float* inv_freq, const PagedRows& cache, float* q_lat, cudaStream_t stream);
// The same with the queries and the (latent | rotated key) part in buffers of their own: q fp32 rows of ldq floats
// (heads * (dn + dr) used), kv fp32 rows of ldkv floats (R + dr used).
int launch_latent_post_split(const SeqIndex& ix, const float* q, long long ldq, const float* kv, long long ldkv,
                             const LatentDims& d, const void* c_norm, int wf32, float eps, const float* inv_freq,
                             const PagedRows& cache, float* q_lat, cudaStream_t stream);
// Workspace of the register-tiled kernel when it cuts a long key range into shares (few query rows, long context):
// o [o_elems] floats, ml [2 * rows] floats; (token, head) pairs x shares must fit `rows`.  tiled = 0 forces the
// one-warp-per-pair kernel, which takes any latent size; 1 the register-tiled fp32 kernel where the sizes allow; 2 (default)
// lets bf16 cache rows run on the tensor cores with the fp32 operands split into two bf16 terms.
struct AttnSplit {
    float* o = nullptr;
    float* ml = nullptr;
    long long rows = 0, o_elems = 0;
    int tiled = 2;
};
// out_lat fp32 [M][heads][R].  cu_q / seq_slot as in asd_engine_forward; a sequence's tokens are consecutive positions;
// max_kv_len bounds position + 1 over the batch.
int launch_latent_attention(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen,
                            int max_kv_len, const float* q_lat, const LatentDims& d, const PagedRows& cache,
                            float* out_lat, const AttnSplit& ws, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------- moe.cu
// Router: probs = softmax(logits) over all E experts (fp32); the `top` largest are kept with their probabilities as
// gates (not renormalised; ties go to the lower index).  Then the (token, choice) pairs are grouped by expert:
// group_off [E + 1], sorted_tok [M * top] (token of each slot), slot_of [M][top].  counters: int [2 E + 1] scratch.
// With `in` the kernel computes the logits itself (fp32, one warp per token): logits = x[M][D] . w[E][D]^T.
struct MoeRouterInput {
    const void* x;          // [M][D]
    int x_f32;
    const void* w;          // [E][D]
    int w_f32;
    int D;
    float* logits_out;      // optional [M][E]
    const float* bias = nullptr;   // optional [E], added to the logits
    int renorm = 0;                // 1: the gates are divided by their sum (softmax over the chosen logits alone)
};
int launch_moe_route(const float* logits, const MoeRouterInput* in, int M, int E, int top, int* expert_of, float* gate,
                     int* counters, int* group_off, int* sorted_tok, int* slot_of, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------- norm_ops.cu
// Row kernels of sandwich-normed layers (a norm before and after every sublayer).  "Offset" RMS norms store their
// weight as the deviation from one: x / sqrt(mean(x^2) + eps) * (1 + w).  Norm weights are fp32 vectors.
// x0[m] = embed[token] * scale, fp32 (x, if given, receives a copy: the stream that the layers go on to change)
int launch_embed_scaled(const SeqIndex& ix, const void* embed, int wf32, float scale, float* x0, float* x, int D,
                        cudaStream_t stream);
// Closes a sublayer and prepares the next one in one pass over a row:
//   x_out = x_in + (post_w ? y / rms(y) * (1 + post_w) : y) + bias          (each term optional)
//   hn    = x_out / rms(x_out) * (1 + next_w)   in the engine's element type (if next_w)
//   hn    = [x_out | cat[m]]                     rows of 2 D elements        (if cat: input of a pass-entry projection)
// plain_w: the weights are taken as they are instead of 1 + w.  groups > 1: the norm before the next sublayer divides
// each of `groups` equal consecutive parts of the row by its own root mean square.  top > 0: the sum also takes the
// routed experts' results, gate[m][k] * expert_out[slot_of[m][k]] for k < top in this order (moe.cu).
struct RowClose {
    const float* x_in = nullptr;    // [M][D]; with `rows`: row r reads x_in[rows[r]]
    const int* rows = nullptr;
    const float* y = nullptr;       // [M][D]
    const float* post_w = nullptr;  // [D]
    const float* bias = nullptr;    // [D]
    float* x_out = nullptr;         // [M][D], may alias x_in
    const float* next_w = nullptr;  // [D]
    const float* cat = nullptr;     // [M][D]
    void* hn = nullptr;
    int hn_f32 = 0;
    float eps = 0.f;
    int M = 0, D = 0;
    int plain_w = 0, groups = 1;
    const float* expert_out = nullptr;  // [M * top][D] rows by slot
    const int* slot_of = nullptr;       // [M][top]
    const float* gate = nullptr;        // [M][top]
    int top = 0;
};
int launch_row_close(const RowClose& c, cudaStream_t stream);
// x[m] = embed[token] with each of `groups` equal consecutive parts divided by its root mean square, times w; fp32
int launch_embed_normed(const SeqIndex& ix, const void* embed, int wf32, const float* w, int groups, float eps, float* x,
                        int D, cudaStream_t stream);
// Feed-forward activations over `rows` rows: out[r][f] = gelu_tanh(z[r][f]) with z rows of F floats, or (gated)
// silu(z[r][f]) * z[r][F + f] with z rows of 2 F floats (gate half, then up half); out in the engine's element type
// mode 2: relu(z[r][f] + bias[f])^2.  bias (optional, fp32 [F]; mode 1: [2 F]) is added to z first in every mode.
int launch_ff_act(const float* z, void* out, int of32, long long rows, int F, int gated, cudaStream_t stream,
                  const float* bias = nullptr);
// out[m][0 .. n) = in[m][0 .. n) / rms * w (plain weight; plus_one: 1 + w), rows ld_in / ld_out apart
int launch_rms_rows(const float* in, long long ld_in, const float* w, int plus_one, float eps, void* out, int of32,
                    long long ld_out, int M, int n, cudaStream_t stream);
// Normalised cubic polynomial over a feed-forward row: a N(z) + b N(z^2) + c N(z^3) + e with powers taken element by
// element, N(u) = u / sqrt(mean(u^2) + eps) and coeff = (a, b, c, e) fp32.
int launch_polynorm(const float* z, const float* coeff, float eps, void* out, int of32, int M, int F, cudaStream_t stream);
// logits <- cap * tanh(logits / cap) in place, n rows of V floats ld apart
int launch_softcap(float* logits, long long ld, int n, int V, float cap, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------- gla.cu
// Gated linear attention: per head a state S [dk][dv] in fp32 with a decay per key channel,
//   S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,   alpha = sigmoid(z)^(1 / tau).
struct GlaDims {
    int heads, dk, dv;
    int low;        // inner size of the decay projection
    float tau;
    float q_scale;  // scale of the queries (applied to the result, which is linear in q)
};
// alpha[m][heads * dk] = exp(log_sigmoid(w_decay . a[m] + b_decay) / tau); a = fp32 rows of `low` floats lda apart
int launch_gla_decay(const float* a, long long lda, const float* w_decay, const float* b_decay, const GlaDims& d,
                     float* alpha, int M, cudaStream_t stream);
// state fp32 [slots][ring][heads][dk][dv]; entry position % ring holds the state after that position.  A sequence whose
// first new position is 0 starts from zero, any other from entry (position - 1) % ring; the last `ring` new positions
// of a sequence store theirs.  q, k (heads * dk used) and v (heads * dv used) are fp32 rows ld floats apart.
// out fp32 [M][heads * dv].
int launch_gla_recurrence(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, const float* q,
                          const float* k, const float* v, long long ld, const float* alpha, const GlaDims& d,
                          float* state, int ring, float* out, cudaStream_t stream);
// y[m][h][:] = o[m][h][:] / rms(o[m][h][:]) * w * silu(gate[m][h][:]) in the engine's element type
int launch_gla_out(const float* o, const float* gate, long long ldg, const float* w, float eps, void* y, int of32, int M,
                   int heads, int dv, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------- window_attention.cu
// Grouped-query softmax attention over a sliding window plus kept first positions, with a sink in the denominator and
// position-rotated values.  Cache row per position: [kv_heads * dk rotated keys | kv_heads * dv rotated values].
struct WindowDims {
    int heads, kv_heads, dk, dv;
    int rot_dims;      // leading key/query coordinates that rotate; the values rotate over all dv
    int interleaved;   // pairs (2 i, 2 i + 1) or (i, i + n / 2)
    int window;        // position i sees j <= i with i - j < window ...
    int keep_first;    // ... or j < keep_first
    float scale;
};
// qkv fp32 rows (ld floats apart) = [heads * dk | kv_heads * dk | kv_heads * dv].  Rotates the queries in place and
// appends the rotated keys and values to the cache.  freq_k fp32 [rot_dims / 2], freq_v fp32 [dv / 2].
int launch_window_post(const SeqIndex& ix, float* qkv, long long ld, const WindowDims& d, const float* freq_k,
                       const float* freq_v, const PagedRows& cache, cudaStream_t stream);
// out[m][heads * dv] in the engine's element type: softmax (denominator + exp(sink[head])) over the visible positions,
// turned back by the query's position.  sink fp32 [heads] (nullptr: none).  tiled = 0: one warp per (token, head);
// else bf16 cache rows run on the tensor cores where the sizes allow.  ws (the AttnSplit workspace of the latent
// kernels; o and ml may be nullptr) holds the partial results when single-token steps cut the keys into shares.
int launch_window_attention(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen,
                            int max_kv_len, const float* q, long long ldq, const WindowDims& d, const float* sink,
                            const float* freq_v, const PagedRows& cache, void* out, int of32, int tiled,
                            const AttnSplit& ws, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------- delta_rule.cu
// Channel functions of a low-rank projection: out[m][c] = post( w2[c] . inner(a[m]) + bias[c] ), fp32 throughout.
enum { LRC_SIGMOID = 0, LRC_EXP_SOFTPLUS = 1, LRC_EXP_SIGMOID = 2 };
struct LowRankChannels {
    const float* w2 = nullptr;     // [n][low]
    const float* bias = nullptr;   // [n] (optional)
    int low = 0, n = 0;
    int inner_tanh = 0;            // the inner vector passes tanh first
    int post = LRC_SIGMOID;        // sigmoid(z) | exp(-exp(head_log_rate[c / per_head]) * softplus(z)) | exp(-rate * sigmoid(z))
    const float* head_log_rate = nullptr;
    int per_head = 0;
    float rate = 1.f;
};
// a = fp32 rows of `low` floats lda apart; out fp32 [M][n]
int launch_lowrank_channels(const float* a, long long lda, const LowRankChannels& p, float* out, int M, cudaStream_t stream);
// Short causal convolution over time per channel, then silu: out[m][c] = silu(sum_j taps[c][j] in[pos - (n - 1 - j)][c]),
// zeros before position 0.  in = fp32 rows ld apart (C used), out fp32 [M][C].  Inputs of earlier forwards come from
// ring fp32 [slots][ring_n][C], entry p % ring_n = the input at position p (ring_n >= n - 1); launch_conv_commit stores
// the last ring_n new positions of every sequence there and must follow the convolution.
int launch_short_conv(const SeqIndex& ix, const float* in, long long ld, const float* taps, int n_taps, int C,
                      const float* ring, int ring_n, float* out, cudaStream_t stream);
int launch_conv_commit(const SeqIndex& ix, const int* cu_q, int nseq, const float* in, long long ld, int C, float* ring,
                       int ring_n, cudaStream_t stream);
// The vectors a position's recurrence step reads, rv fp32 [M][heads][3 or 5][dk] and sc fp32 [M][heads][4] (layout in
// delta_rule.cu).  Gated rule (general = 0): q, k = fp32 rows ld apart holding kv_heads * dk values (head h reads key
// head h / (heads / kv_heads)), made unit vectors (x / sqrt(sum x^2 + tiny)), q times q_scale; beta = raw rows (ld_beta
// apart, one per head) that pass a sigmoid; decay fp32 [M][heads * dk].  Generalised rule (general = 1): q = the
// read-out vectors, k = the keys, rate (raw, ld apart) + rate_bias [heads * dk] pass a sigmoid.
struct DeltaPrep {
    const float* q = nullptr;
    const float* k = nullptr;
    long long ld = 0;
    const float* decay = nullptr;
    const float* beta = nullptr;
    long long ld_beta = 0;
    const float* rate = nullptr;
    const float* rate_bias = nullptr;
    float* rv = nullptr;
    float* sc = nullptr;
    int heads = 0, kv_heads = 0, dk = 0, general = 0;
    float q_scale = 1.f, tiny = 1e-6f;
};
int launch_delta_prep(const DeltaPrep& p, int M, cudaStream_t stream);
// state fp32 [slots][ring][heads][dk][dv]; entry position % ring holds the state after that position.  A sequence whose
// first new position is 0 starts from zero, any other from entry (position - 1) % ring; the last `ring` new positions
// of a sequence store theirs.  v = fp32 rows ldv apart (heads * dv used); out fp32 [M][heads * dv].
int launch_delta_recurrence(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, const float* rv,
                            const float* sc, int general, const float* v, long long ldv, int heads, int dk, int dv,
                            float* state, int ring, float* out, cudaStream_t stream);
// y[m][h][:] = o[m][h][:] / rms(o[m][h][:]) * w * gate[m][h][:] * scale, y = rows ldy apart in the engine's element
// type.  w: [dv] shared by the heads or [heads * dv]; gate: fp32 rows ldg apart, taken as they are or through a sigmoid.
struct HeadNormGate {
    const float* gate = nullptr;
    long long ldg = 0;
    const float* w = nullptr;
    int w_per_head = 0, gate_sigmoid = 0;
    float eps = 0.f, scale = 1.f;
};
int launch_head_norm_gate(const float* o, const HeadNormGate& p, void* y, int of32, long long ldy, int M, int heads, int dv,
                          cudaStream_t stream);

// ---------------------------------------------------------------------------------------------- talking_attention.cu
// Grouped-query softmax attention over a sliding window whose scores are capped (cap * tanh(s / cap)) and then mixed
// across the heads, s'_h = sum_g talk[h][g] s_g, before a softmax with a sink per head in the denominator.
// Cache row per position: [kv_heads * dk normed, rotated keys | kv_heads * dv values].
struct TalkDims {
    int heads, kv_heads, dk, dv;
    int rot_dims;      // leading key/query coordinates that rotate in pairs (2 i, 2 i + 1)
    int window;        // position i sees j <= i with i - j < window
    float scale;
    float softcap;     // 0: scores are not capped
};
// qkv fp32 rows (ld floats apart) = [heads * dk | kv_heads * dk | kv_heads * dv].  Adds the biases (fp32, same layout,
// optional), RMS-norms every query and key head over dk (plain weights q_norm, k_norm [dk]; nullptr: none), rotates
// them, leaves the queries in place and appends keys and values to the cache.  freq fp32 [rot_dims / 2].
int launch_talk_post(const SeqIndex& ix, float* qkv, long long ld, const TalkDims& d, const float* bias, const float* q_norm,
                     const float* k_norm, float eps, const float* freq, const PagedRows& cache, cudaStream_t stream);
// out[m][h][:] (rows ldo apart, engine's element type) = out_scale * sum_j p[h][j] v[j]; talk fp32 [heads][heads]
// (nullptr: no mixing), sink fp32 [heads] (nullptr: none).  ws.o (o_elems floats; may be nullptr) holds the partial
// results when steps of few tokens cut the key tiles into shares for several CTAs; ws.ml (optional: `rows` zeroed
// 32-bit counters, one per token) lets a token's last CTA to arrive merge them instead of a kernel of its own.
int launch_talk_attention(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen, int max_kv_len,
                          const float* q, long long ldq, const TalkDims& d, const float* talk, const float* sink,
                          const PagedRows& cache, void* out, int of32, long long ldo, float out_scale, const AttnSplit& ws,
                          cudaStream_t stream);

// ---------------------------------------------------------------------------------------------- residual_streams.cu
// Several residual streams per token (hyper-connections): xs fp32 [M][S][D].  A sublayer reads u = sum_s read[s] x_s and
// its result y goes back as x_t <- sum_s mix[s][t] x_s + write[t] * y for all t at once.
// xs[m][s] = embed[token] * scale + pos_table[position] for every s (pos_table optional, engine's element type)
int launch_embed_streams(const SeqIndex& ix, const void* embed, const void* pos_table, int wf32, float scale, float* xs,
                         int S, int D, cudaStream_t stream);
// One pass over a row: (1) if y: the streams take the sublayer's result (y_bias, optional [D], is added to y first);
// (2) if read: u = sum_s read[s] x_s over the new streams; u_out (optional, fp32 [M][D]) receives it, and with next_w
// hn = u / rms(u) * next_w in the engine's element type.  With `rows`, row r reads xs[rows[r]] (no write-back then).
struct StreamClose {
    float* xs = nullptr;            // [M][S][D]
    const int* rows = nullptr;
    const float* y = nullptr;       // [M][D]
    const float* y_bias = nullptr;  // [D]
    const float* mix = nullptr;     // [S][S], from-stream major
    const float* write = nullptr;   // [S]
    const float* read = nullptr;    // [S] (nullptr with want_sum: all ones)
    int want_sum = 0;
    float* u_out = nullptr;
    const float* next_w = nullptr;  // [D]
    void* hn = nullptr;
    int hn_f32 = 0;
    float eps = 0.f;
    int M = 0, S = 1, D = 0;
};
int launch_stream_close(const StreamClose& c, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------- mixed_attention.cu
// Grouped-query softmax attention whose softmax WEIGHTS may be mixed across the heads (w'_h = sum_g talk[h][g] w_g),
// with a learned bias per (distance, head) on the scores, a causal mask that may be cut into chunks counted from
// position 0, and a gate per head on the result.  Cache row per position: [kv_heads * dk keys | kv_heads * dv values].
struct MixDims {
    int heads, kv_heads, dk, dv;
    int chunk;          // 0: position i sees every j <= i; else only those with j / chunk == i / chunk
    float scale;
};
// What the projections pass before the attention.  qkv fp32 rows (ld floats apart) = [heads * dk | kv_heads * dk |
// kv_heads * dv].  Adds the biases (same layout, optional); RMS-norms queries and keys either head by head (weights [dk],
// norm_whole = 0) or over the whole projection (weights [heads * dk] and [kv_heads * dk], norm_whole = 1); multiplies the
// queries by 1 + temp_coef * ln(floor((position + 1) / temp_every) + 1) (temp_every 0: not) and by head_factor[head]
// (optional); divides every value head by its root mean square (v_unit); leaves the queries in place and appends keys
// and values to the cache.
struct MixPost {
    const float* bias = nullptr;
    const float* q_norm = nullptr;
    const float* k_norm = nullptr;
    int norm_whole = 0;
    float temp_coef = 0.f;
    int temp_every = 0;
    const float* head_factor = nullptr;
    int v_unit = 0;
    float eps = 0.f;
};
int launch_mix_post(const SeqIndex& ix, float* qkv, long long ld, const MixDims& d, const MixPost& p,
                    const PagedRows& cache, cudaStream_t stream);
// 0 if the kernels take these sizes (dv <= 256, dk <= 512, at most 128 heads when the weights are mixed), else -1 and
// the error text
int mix_attention_check(const MixDims& d, int talk);
// Workspace: stats fp32 [2][shares][M][heads] (maximum and sum of every key share), part fp32 [shares][M][heads * dv].
// scores fp32 [M][heads][keys] of steps of few tokens (optional).  mode 0: steps of few tokens and, in a bf16 engine,
// prompts on the tensor cores take kernels of their own; 1: everything runs the general CUDA-core kernels.
struct MixWork {
    float* stats = nullptr;
    float* part = nullptr;
    float* scores = nullptr;
    long long stats_elems = 0, part_elems = 0, score_elems = 0;
    int mode = 0;
};
// out[m][h][:] (rows ldo apart, engine's element type) = sigmoid(gate[m][h]) * sum_j w'_h[j] v[j].  dist_bias fp32
// [far + 1][heads]: the bias at distance min(i - j, far) (nullptr: none); talk fp32 [heads][heads] (nullptr: no mixing);
// gate fp32 rows ldg apart, one raw value per head (nullptr: none).  Steps of few tokens cut the keys into shares for
// several CTAs.
int launch_mix_attention(const SeqIndex& ix, const int* cu_q, const int* seq_slot, int nseq, int max_qlen, int max_kv_len,
                         const float* q, long long ldq, const MixDims& d, const float* dist_bias, int far,
                         const float* talk, const float* gate, long long ldg, const PagedRows& cache, void* out, int of32,
                         long long ldo, const MixWork& ws, cudaStream_t stream);

int preload_blocks();

}  // namespace asd
