/*
 * asd_b200.h - C ABI of libasd_b200.so, the B200-native (sm_100a) draft-then-verify hot path
 * behind the adaptive-speculative-decoding Python API.
 *
 * The reference (sa2shun/adaptive-speculative-decoding, /root/reference) is 100 % Python and has
 * NO FFI for this path: its engine seam is duck-typed Python that delegates to vLLM
 * (src/serving/real_model_pipeline.py:98-108,135; docs/guides/RESEARCH_PROTOCOL.md:233-304).
 * Each entry point below therefore cites the Python interface it stands behind; the ctypes
 * binding a maintainer of the reference would add is shown in INTEGRATION.md.
 *
 * Conventions: every function returns 0 on success and -1 on error (message from
 * asd_last_error(), thread local).  Unless a name ends in _host, pointers are CUDA device
 * pointers owned by the caller; the library never frees caller memory.  `stream` is a
 * cudaStream_t passed as void* (NULL = legacy default stream).  No torch types appear here.
 */
#ifndef ASD_B200_H
#define ASD_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(ASD_BUILDING_DSO)
#define ASD_API __attribute__((visibility("default")))
#else
#define ASD_API
#endif

#define ASD_B200_ABI_VERSION 1
#define ASD_NUM_FEATURES 6 /* lse, p_max, margin, entropy, ln p(draft tok), ln p(token emitted at this position) */

ASD_API int asd_abi_version(void);
ASD_API const char* asd_last_error(void);
/* number of kernels this library has launched since load / since the last reset (bench "gpu_launches") */
ASD_API long long asd_launch_count(void);
ASD_API void asd_reset_launch_count(void);

/* ---------------------------------------------------------------------------------------------
 * Fused logits -> softmax -> rejection sampling -> residual resample -> stop-rule features.
 * Replaces the per-token softmax/log + .item() loop of
 * src/training/generate_training_data.py:128-134 and the logprob reductions of
 * FeatureExtractor.extract (docs/guides/RESEARCH_PROTOCOL.md:379-398); the accept/resample rule is
 * the canonical speculative sampling of SURVEY.md Appendix C (no reference implementation).
 *
 *   target_logits fp32 [B, k+1, V]   draft_logits fp32 [B, k, V] (may be NULL if k == 0 or T <= 0)
 *   draft_tokens  i32  [B, k]        u_accept fp64 [B, k]        u_resid fp64 [B]
 *   temperature <= 0 selects greedy verification (accept iff draft token == argmax).
 *   accept_mask u8 [B, k]; accepted_len i32 [B]; out_tokens i32 [B, k+1] (-1 padded);
 *   out_logprobs fp32 [B, k+1] (0 padded); features fp32 [B, k+1, ASD_NUM_FEATURES]; features[.., 5] repeats
 *   out_logprobs (the residual / bonus draw is only made for the position that emits the new token).
 *   workspace: asd_reject_sample_workspace_bytes(B, k) bytes, zero-filled once before first use.
 * V must be a multiple of 4 and <= 212992; k <= 64; logits 16-byte aligned.  k == 0 samples one
 * token per row from softmax(target/T) (used for the draft model's own sampling).
 */
ASD_API size_t asd_reject_sample_workspace_bytes(int B, int k);
/* tuning switch of the streaming sampler (bit flags, default 5: 4 = the draw kernel is gated per sequence, 2 = persistent
 * statistics CTAs, 8 = single acq_rel ticket); every setting implements the same arithmetic contract bit for bit */
ASD_API void asd_reject_sample_set_impl(int impl);
ASD_API int asd_reject_sample(const float* target_logits, const float* draft_logits, const int32_t* draft_tokens,
                      const double* u_accept, const double* u_resid, int B, int k, int V, float temperature,
                      uint8_t* accept_mask, int32_t* accepted_len, int32_t* out_tokens, float* out_logprobs,
                      float* features, void* workspace, void* stream);
/* Same call with HOST buffers: copies in, runs the kernel on the current device, copies out. */
ASD_API int asd_reject_sample_host(const float* target_logits, const float* draft_logits, const int32_t* draft_tokens,
                           const double* u_accept, const double* u_resid, int B, int k, int V, float temperature,
                           uint8_t* accept_mask, int32_t* accepted_len, int32_t* out_tokens, float* out_logprobs,
                           float* features);

/* ---------------------------------------------------------------------------------------------
 * Cascade stop rule.  optimal_stopping_rule / bayesian_adjustment of
 * src/algorithms/dp_solver.py:12-71,106-130, bit-exact (binary64, same operation order, `<=` tie).
 *   p, C fp64 [n, L]; k_star i32 [n]; J fp64 [n, L+1].  L <= 64.
 */
ASD_API int asd_stop_rule(const double* p, const double* C, int n, int L, double lam, int risk_adjustment, double alpha,
                  double beta, int32_t* k_star, double* J, void* stream);
/* same with one lambda per row (lam fp64 [n]): OptimalStoppingTable.precompute evaluates its whole
 * lambda x probability grid with ONE call (src/algorithms/dp_solver.py:149-171 loops in Python) */
ASD_API int asd_stop_rule_rows(const double* p, const double* C, const double* lam, int n, int L, int risk_adjustment,
                       double alpha, double beta, int32_t* k_star, double* J, void* stream);
ASD_API int asd_stop_rule_rows_host(const double* p, const double* C, const double* lam, int n, int L, int risk_adjustment,
                            double alpha, double beta, int32_t* k_star, double* J);
/* Scorer -> stop decision in ONE launch, all on the device (north star 3; replaces the chain
 * FeatureExtractor.extract -> QualityPredictor.predict -> bayesian_adjustment -> optimal_stopping_rule of
 * src/serving/pipeline.py:225-256 for n requests that have just finished stage `stage_idx`):
 *   features fp32 [n, T, ASD_NUM_FEATURES]: the rows asd_reject_sample wrote for each request's generated tokens (still
 *     in device memory); n_tokens i32 [n]: how many of the T rows are valid;
 *   scalars fp64 [n, 3]: prompt words / 2048, output words / 512, stage / 4 (RESEARCH_PROTOCOL.md:389-403);
 *   w1 fp32 [128, feature_dim], b1 [128], w2 [128], b2 [1]: the 256 -> 128 -> 1 MLP (RESEARCH_PROTOCOL.md:325-331);
 *   prev_p fp64 [n, L]: acceptance probabilities of the stages before stage_idx; C fp64 [L]: stage costs;
 *   prefix_mode 1: the reference loop's rule (DP over the stages seen so far, stop iff k* == stage_idx, pipeline.py:248-256),
 *   0: DP over all L stages with unseen stages at probability 1 (stop iff k* <= stage_idx).
 * Outputs: prob fp64 [n] (after the optional Bayesian shrinkage with n_obs; 1.0 at the last stage), stop i32 [n],
 * k_star i32 [n].  The host reads three numbers per request; no per-token data leaves the device. */
ASD_API int asd_cascade_decide(const float* features, const int32_t* n_tokens, int n, int T, const double* scalars,
                       const float* w1, const float* b1, const float* w2, const float* b2, int feature_dim,
                       const double* prev_p, const double* C, int L, int stage_idx, int prefix_mode, double lam,
                       int risk_adjustment, double n_obs, double alpha, double beta, double* prob, int32_t* stop,
                       int32_t* k_star, void* stream);
/* scalar host form used by the Python policy seam (pipeline.py:251-256): returns k_star or -1 */
ASD_API int asd_stop_rule_host(const double* p, const double* C, int L, double lam, int risk_adjustment, double alpha,
                       double beta, double* J);
ASD_API double asd_bayesian_adjustment_host(double p_hat, double n_obs, double alpha, double beta);

/* ---------------------------------------------------------------------------------------------
 * Weight-streaming linear layer  Y[m, n] = sum_k X[m, k] * W[n, k]  (bf16 in, fp32 accumulate) on
 * tcgen05/TMEM fed by TMA: the dense contraction of the verify / draft forward that the reference
 * delegates to vLLM (src/serving/real_model_pipeline.py:98-108,135).
 *   x bf16 [M, K]; w bf16 [N, K] (torch nn.Linear layout); K % 8 == 0; 16-byte aligned.
 *   out_mode 0: out fp32 [ksplit_used, M, N] - one slice per K split, the caller (or the fused
 *               add+RMSNorm / RoPE kernels) sums the slices in order;
 *   out_mode 1: out bf16 [M, N] (ksplit forced to 1);
 *   out_mode 2: SwiGLU - w rows interleaved per 128-row tile as 64 gate rows then 64 up rows;
 *               out bf16 [M, N/2] = silu(gate) * up;
 *   out_mode 3: out fp32 [M, N], final: the K splits of a tile form a thread-block cluster and are
 *               reduced through distributed shared memory in rank order (deterministic).
 *   ksplit / stages: 0 = let the library choose (single co-resident wave).
 */
ASD_API int asd_linear_bf16(const void* x, const void* w, void* out, int M, int N, int K, int out_mode, int ksplit,
                    int stages, int* ksplit_used, void* stream);
/* Same contraction on the tensor-bound kernel used above the HBM/tensor ridge (M > 256 tokens: BASELINE configs[4],
 * prefill): CTA pairs (tcgen05 cta_group::2, 256 weight rows x <= 256 tokens per tile), persistent, two TMEM
 * accumulators.  out_mode 0: fp32 [ksplit_used, M, N] slices; out_mode 2: SwiGLU bf16 [M, N/2]. */
ASD_API int asd_linear_bf16_tc(const void* x, const void* w, void* out, int M, int N, int K, int out_mode, int ksplit,
                       int stages, int* ksplit_used, void* stream);
ASD_API int asd_linear_plan(int M, int N, int K, int out_mode, int* ksplit, int* stages, int* token_tile);

/* ---------------------------------------------------------------------------------------------
 * Model forward engine (Qwen2 family: RMSNorm, RoPE, GQA attention with QKV bias, SwiGLU MLP).
 * Stands where the reference calls vllm.LLM(model, tensor_parallel_size, dtype="bfloat16",
 * max_model_len=4096).generate(...)  (src/serving/real_model_pipeline.py:98-108,135;
 * Stage.generate in docs/guides/RESEARCH_PROTOCOL.md:233-304).  One handle per (model, TP rank);
 * calls on one handle must be serialised by the caller (the Python Stage holds a lock).
 *
 * Dimensions in asd_model_config are LOCAL to the tensor-parallel rank: n_heads, n_kv_heads and ffn
 * are the global values divided by tp_size (column-parallel QKV / gate|up, row-parallel O / down);
 * hidden and vocab are global (lm_head is replicated).
 *
 * Weight layouts (bf16, row-major, torch nn.Linear [out, in]):
 *   wqkv [(n_heads + 2 n_kv_heads) * head_dim, hidden] = rows of q heads, then k heads, then v heads;
 *   bqkv [(n_heads + 2 n_kv_heads) * head_dim];  wo [hidden, n_heads * head_dim];
 *   wgateup [2 * ceil(ffn/64)*64, hidden]: per 128-row tile 64 gate rows then 64 up rows (zero padded);
 *   wdown [hidden, ffn];  ln1, ln2, final_norm [hidden];  embed, lm_head [vocab, hidden];
 *   inv_freq fp32 [head_dim / 2].
 * KV pool (bf16, caller allocated, asd_engine_kv_pool_bytes):
 *   [n_layers][2 (K, V)][num_pages][n_kv_heads][page_size][head_dim]; page_table i32
 *   [max_seqs, max_pages_per_seq] maps (sequence slot, position / page_size) -> page.
 */
typedef struct asd_model_config {
    int hidden, n_layers, n_heads, n_kv_heads, head_dim, ffn, vocab;
    float rms_eps;
    int max_tokens; /* largest M of one forward call */
    int page_size;
    int tp_rank, tp_size;
} asd_model_config;
typedef struct asd_engine asd_engine_t;

ASD_API asd_engine_t* asd_engine_create(const asd_model_config* cfg); /* NULL on error */
ASD_API void asd_engine_destroy(asd_engine_t* e);
ASD_API int asd_engine_set_layer(asd_engine_t* e, int layer, const void* wqkv, const void* bqkv, const void* wo,
                         const void* wgateup, const void* wdown, const void* ln1, const void* ln2);
ASD_API int asd_engine_set_globals(asd_engine_t* e, const void* embed, const void* final_norm, const void* lm_head,
                           const float* inv_freq);
ASD_API size_t asd_engine_kv_pool_bytes(const asd_model_config* cfg, int num_pages);
ASD_API int asd_engine_set_kv(asd_engine_t* e, void* kv_pool, int num_pages, const int32_t* page_table, int max_seqs,
                      int max_pages_per_seq);
/* comm: ncclComm_t; nccl_allreduce_fn: address of ncclAllReduce from the NCCL the process loaded.
 * Called (fp32 sum, in place) after the O and down projections when tp_size > 1. */
ASD_API int asd_engine_set_allreduce(asd_engine_t* e, void* comm, void* nccl_allreduce_fn);
/* Tensor-parallel boundary over NVLink peer memory (preferred to the NCCL path above): every rank exports
 * CUDA-IPC handles of its two receive buffers and its flag array (3 x 64 bytes), the host all-gathers them
 * (rank-major, world x 3 x 64 bytes) and each rank imports the table.  From then on the O / down projections
 * either finish the all-reduce inside their own epilogue (owner CTAs push {value, epoch} words into the peers'
 * receive buffers; option "tp_fused", default at 2 ranks / small exchanges) or are followed by ONE kernel that
 * all-reduces through P2P loads (one-shot, or two-shot with a home rank per row: option "tp_two_shot"), adds the
 * residual and emits the norm statistics.  All paths give bit-identical residuals on every rank.
 * asd_engine_tp_error returns 1 if a peer ever failed to show up within the spin bound. */
ASD_API int asd_engine_ipc_export(asd_engine_t* e, void* handles_out);
ASD_API int asd_engine_ipc_import(asd_engine_t* e, const void* all_handles);
ASD_API int asd_engine_tp_error(asd_engine_t* e);
/* In-process tensor parallelism (what Stage(tensor_parallel_size = t, gpu_ids = [...]) builds, mirroring
 * configs/qwen3_models.yaml:10-51 and src/serving/real_model_pipeline.py:98-108): the t rank engines were created in
 * ONE process, rank r on its own device.  Enables peer access between the devices and wires every rank's receive
 * buffers and flags into the others (no IPC, no torchrun).  engines[r] must be rank r of a t-way group. */
ASD_API int asd_engine_peer_connect(asd_engine_t** engines, int n);
/* options: "attn_impl" (2 tcgen05 / TMEM kernel - default; 1 mma.sync kernel, also the fallback for head_dim 64 or more
 * than 128 query rows; 0 one-warp cross-check kernel), "tc_qkvo" (1, default: above 256 tokens QKV and O run on the
 * CTA-pair tensor-bound GEMM like gate|up / down / lm_head; 0: weight-streaming kernel), "gemm_big" (0: never use the
 * CTA-pair GEMM), "attn_prefetch_mb" (L2 prefetch of the following GEMMs' weights from the attention kernel, measured
 * slower, default 0), "pdl" (0/1),
 * "reduce" (1 in-cluster split-K reduction with fused residual add, 0 fp32 slices summed by the glue
 * kernels), "fuse_rope" (1: bias + RoPE + q store + paged K/V append in the QKV GEMM epilogue),
 * "fuse_norm" (1: RMSNorm fused into the GEMMs: the O / down epilogues emit bf16(resid * ln_w) and the
 * per-token sum of squares, the consuming QKV / gate|up / lm_head epilogues apply rstd),
 * "attn_target_ctas", "attn_min_split_keys" (keys per flash-decoding split, default 1024), "glue_pdl",
 * "ksplit", "stages" (0 = automatic), "headroom" (shared memory left for the next kernel's CTAs on <= 32-token
 * tiles), "recv_dedicated", "early_trigger", "next_prefetch_mb" (tuning knobs),
 * "tp_fused" (0 never, 1 where it pays, 2 always), "tp_two_shot" (-1 never, 0 where it pays, 1 always), "p2p",
 * "persist" (1: single-rank forwards of <= 128 tokens run as ONE cooperative launch of the persistent forward
 * kernel, forward_persist.cu; 0, default: one launch per GEMM / attention - measured faster),
 * "persist_ahead" (L2 prefetch distance of the persistent kernel's weight producer, 0 = off), "profile" (0/1) */
ASD_API int asd_engine_set_option(asd_engine_t* e, const char* name, int value);
/* With option "profile" = 1 every launch is bracketed by CUDA events on the launching stream;
 * this call synchronises and returns the summed milliseconds and launch counts by kernel class
 * {0 weight-streaming GEMMs, 1 attention, 2 glue (norm/rope/gather), 3 TP all-reduce, 4 lm_head GEMM}
 * since the previous read (bench.py's roofline numbers come from here). nclass >= 5. */
/* Diagnostics: every following GEMM launch (up to max_launches, <= 1024 CTAs each) records per-CTA globaltimer
 * stamps into buf (device, u64): {entry, setup done, upstream grid done, first tile landed, main loop done,
 * cluster barrier 1, scatter done, cluster barrier 2, exit, smid}.  Returns the u64 stride per launch; buf = NULL
 * switches tracing off. */
ASD_API int asd_debug_gemm_trace(unsigned long long* buf, int max_launches);
/* Same for the attention kernel: {entry, upstream grid done, metadata read, loads issued, first K/V tile landed,
 * key loop done, key groups merged, partials stored, ticket taken, exit of the merging CTA}. */
ASD_API int asd_debug_attn_trace(unsigned long long* buf, int max_launches);
/* Diagnostics of the persistent forward kernel: per-CTA globaltimer stamps into buf (device, u64 [CTAs][643]: slot 0
 * kernel entry, slot p + 1 = this CTA's share of phase p done; phase 0 embedding, 1 + 5 l + {0 QKV, 1 attention, 2 O,
 * 3 gate|up, 4 down} of layer l, then logit-row gather and lm_head); returns the number of CTAs; NULL = off. */
ASD_API int asd_engine_persist_trace(asd_engine_t* e, unsigned long long* buf);
ASD_API int asd_engine_profile_read(asd_engine_t* e, float* ms_by_class, int* launches_by_class, int nclass);
/*
 * One forward pass over M tokens (draft step: q_len 1; verify step: q_len k+1; prefill chunk).
 *   tokens, positions, token_slot i32 [M]: token id, absolute position, sequence slot of each token;
 *     the tokens of one sequence are contiguous and in increasing position;
 *   cu_q i32 [nseq+1]: token range of each active sequence; seq_slot i32 [nseq]: its slot;
 *   max_qlen: largest q_len (q_len * n_heads / n_kv_heads <= 128); max_kv_len: upper bound of
 *     (last position + 1) over the sequences (sizes the flash-decoding split, may over-estimate);
 *   K/V of the M tokens are written in place into the paged pool before attention: a rejected
 *     speculative tail is rolled back by simply not advancing the caller's length (asd_kv_commit is
 *     therefore a no-op in this design);
 *   logit_rows i32 [n_logit_rows] selects rows (NULL = all M rows, n_logit_rows == M; 0 = no logits);
 *   logits_out fp32 [n_logit_rows, vocab] with row stride logits_ld elements (0 = vocab).
 * Asynchronous on `stream`; performs no allocation or synchronisation (CUDA-graph capturable after
 * one warm-up call with the same M when tp_size == 1; a tensor-parallel forward numbers its peer-memory exchanges
 * with a host-side epoch and refuses stream capture).  Runs on the device the engine was created on.
 */
ASD_API int asd_engine_forward(asd_engine_t* e, const int32_t* tokens, const int32_t* positions,
                       const int32_t* token_slot, int M, const int32_t* cu_q, const int32_t* seq_slot, int nseq,
                       int max_qlen, int max_kv_len, const int32_t* logit_rows, int n_logit_rows, float* logits_out,
                       long long logits_ld, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Mezilix family engine: a decoder whose layers are PARALLEL blocks (one scalar-gain RMS norm feeds the mixer and
 * the feed-forward, both are added to the stream), whose mixer is latent key/value attention with a sliding
 * window over a paged cache of [latent | shared rotated key] rows (evaluated in latent space), whose feed-forward
 * is a softmax-routed mixture of squared-ReLU experts, with a hashed token-pair embedding, token shift on the
 * mixer input and a learned average over all earlier layer results after every layer.  The reference has no
 * such model (its stages are vLLM checkpoints, src/serving/real_model_pipeline.py:98-108); the engine sits behind
 * the same forward contract as asd_engine_forward so that the same step loop, sampler and stage drive it.
 *
 * dtype 0: bf16 weights, cache and matrix inputs with fp32 accumulation; dtype 1: everything fp32 (CUDA-core FMA).
 * In both, norms, rotary angles, scores, softmax, router, residual stream and carried state are fp32.
 * Every layer has its own sizes.  experts == 0: the layer has no feed-forward.
 * Carried state besides the cache (caller allocated, zero filled): token ring i32 [max_seqs][ring] and shift ring
 * fp32 [n_layers][max_seqs][ring][width], both indexed by position % ring (ring >= the longest speculative tail
 * that may be re-fed).  Cache pool: per layer [num_pages][page_size][kv_rank + rot_dim], layers back to back.
 */
typedef struct asd_mezilix_layer_config {
    int heads, dim, rot_dim, vdim, kv_rank; /* per head: dim unrotated + rot_dim rotated query/key, vdim value */
    int rot_dims;                           /* rotating coordinates of the rotated part (even, <= rot_dim) */
    int window;                             /* position p attends p - window < j <= p */
    float rot_base, scale;
    int experts, top, ff;
} asd_mezilix_layer_config;
typedef struct asd_mezilix_config {
    int width, vocab, n_layers;
    float eps;
    int buckets, mul_prev, mul_cur; /* token-pair table: row (prev * mul_prev + cur * mul_cur) % buckets, row `buckets` first */
    int max_tokens, page_size, ring, dtype;
} asd_mezilix_config;
typedef struct asd_mezilix_engine asd_mezilix_engine_t;

ASD_API asd_mezilix_engine_t* asd_mezilix_create(const asd_mezilix_config* cfg, const asd_mezilix_layer_config* layers);
ASD_API void asd_mezilix_destroy(asd_mezilix_engine_t* e);
/* all weights in the engine's dtype, row-major [out, in]; embed [vocab, width], pair_table [buckets + 1, width],
 * final_gain [1], head [vocab, width] */
ASD_API int asd_mezilix_set_globals(asd_mezilix_engine_t* e, const void* embed, const void* pair_table,
                                    const void* final_gain, const void* head);
/* gain [1]; shift [width]; depth_coeff [layer + 2]; wqd [heads * (dim + rot_dim) + kv_rank + rot_dim, width] = query
 * rows head by head, then the latent rows, then the rotated key rows; latent_gain [kv_rank]; wuk [heads][kv_rank][dim] (the key
 * up-projection transposed per head);
 * wuv [heads * vdim, kv_rank]; wo [width, heads * vdim]; router [experts, width]; w_up [experts, ff, width];
 * w_down [experts, width, ff] (NULL when experts == 0) */
ASD_API int asd_mezilix_set_layer(asd_mezilix_engine_t* e, int layer, const void* gain, const void* shift,
                                  const void* depth_coeff, const void* wqd, const void* latent_gain, const void* wuk,
                                  const void* wuv, const void* wo, const void* router, const void* w_up,
                                  const void* w_down);
ASD_API size_t asd_mezilix_cache_bytes(const asd_mezilix_engine_t* e, int num_pages);
ASD_API int asd_mezilix_set_cache(asd_mezilix_engine_t* e, void* pool, int num_pages, const int32_t* page_table,
                                  int max_seqs, int max_pages_per_seq, int32_t* token_ring, float* shift_ring);
/* options: "tc_linear" (1, default: bf16 projections whose shape the tcgen05 kernels accept run on them; 0: CUDA-core
 * kernel everywhere), "tc_min_rows" (token count from which dense projections use the tensor-bound CTA-pair GEMM, default
 * 257; 0 = never), "attn_tiled" (2, default: attention of bf16 cache rows on the tensor cores with fp32 operands as two
 * bf16 terms, else as 1; 1: register-tiled fp32 kernel with key-range shares where the latent size allows; 0: one warp
 * per (token, head)), "profile" (1: CUDA events around every launch, read with asd_mezilix_profile_read) */
ASD_API int asd_mezilix_set_option(asd_mezilix_engine_t* e, const char* name, int value);
/* Same contract as asd_engine_forward (M <= max_tokens).  layer_out (optional, fp32 [n_layers][M][width]) receives
 * the stream that leaves every layer. */
ASD_API int asd_mezilix_forward(asd_mezilix_engine_t* e, const int32_t* tokens, const int32_t* positions,
                                const int32_t* token_slot, int M, const int32_t* cu_q, const int32_t* seq_slot, int nseq,
                                int max_qlen, int max_kv_len, const int32_t* logit_rows, int n_logit_rows,
                                float* logits_out, long long logits_ld, float* layer_out, void* stream);
/* ms and launches by kernel class since the last read (nclass >= 7): 0 dense projections, 1 per-head latent products,
 * 2 attention, 3 expert layers, 4 router, 5 embedding / shift / cache append / layer close, 6 output head */
ASD_API int asd_mezilix_profile_read(asd_mezilix_engine_t* e, float* ms_by_class, int* launches_by_class, int nclass);
/* non-zero (and an error message) if a kernel of this engine gave up a bounded wait since creation; synchronises */
ASD_API int asd_mezilix_device_error(asd_mezilix_engine_t* e);
/* Building blocks on their own (tests).  asd_linear_tc: y[z] = x[z] w[z]^T on tcgen05 with bf16 weights [Z][N][K], x
 * bf16 or fp32 [Z][M][K] (rounded to bf16), y bf16 or fp32 [Z][M][N]; K % 8 == 0.  Grouped form (group_off != NULL,
 * int32 [Z + 1] on the device): rows [group_off[z], group_off[z + 1]) of y come from weight z and from the rows
 * gather[.] of x (or the same rows if gather == NULL); M bounds the rows of a group.  relu_sq: y = max(y, 0)^2.
 * err_flag: device int raised if a wait inside the kernel ran out (may be NULL). */
ASD_API int asd_linear_tc(const void* x, int x_f32, const void* w, void* y, int y_f32, int M, int N, int K, int Z,
                          const int32_t* group_off, const int32_t* gather, int relu_sq, int32_t* err_flag, void* stream);
/* y = x W^T on the CUDA cores, any of bf16 (0) / fp32 (1) per operand */
ASD_API int asd_linear_simt(const void* x, int x_f32, const void* w, int w_f32, void* y, int y_f32, int M, int N, int K,
                            void* stream);

/* ---------------------------------------------------------------------------------------------
 * Rivetar family engine: sandwich-normed layers, x += norm_b(f(norm(x))) for the mixer and then for the feed-forward,
 * every such norm an RMS norm with weight (1 + w).  A layer has ONE of three mixers (type):
 *   0 latent attention    queries through a normed latent, keys / values rebuilt from a cached normed latent plus one
 *                         rotated key part shared by the heads (evaluated in latent space, as in the Mezilix engine);
 *   1 gated linear attention   per head a state S [dim][vdim]: S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t, with
 *                         alpha = sigmoid(z)^(1 / tau), z a two-matrix projection plus bias; o is RMS-normed per head,
 *                         multiplied by silu(gate) and projected;
 *   2 windowed attention  grouped-query softmax attention; position i sees j <= i with i - j < window or
 *                         j < keep_first; the denominator also holds exp(sink[head]); values are cached rotated by their
 *                         own position over all vdim coordinates and a head's result is turned back by the query's.
 * The feed-forward is W_down act(W_up h) with act = a N(z) + b N(z^2) + c N(z^3) + e, N = division by the root mean
 * square over ff (ff == 0: none).  Layers loop_start .. loop_stop - 1 run loop_times times with the same weights
 * (loop_times == 0: no repeated span); every execution ("run") has its own cache or state, and a pass starts with
 * x <- W_loop [x; x0] + step[pass], x0 the embedding output.  logits <- cap * tanh(logits / cap) when cap > 0.
 *
 * dtype 0: bf16 matrices, caches and matrix inputs with fp32 accumulation; dtype 1: everything fp32 (CUDA-core FMA).
 * In both, norms, angles, scores, softmax, decays, the recurrent state and the residual stream are fp32.
 * Paged pool: per run with a positional cache [num_pages][page_size][row], row = kv_rank + rot_dim (type 0) or
 * kv_heads * (dim + vdim) (type 2, keys then values), runs back to back.  Recurrent state (type 1, caller allocated,
 * fp32): per run [max_seqs][ring][heads][dim][vdim], entry position % ring holds the state AFTER that position, so a
 * caller may re-feed any of the last `ring` positions; a run that starts at position 0 starts from zero.
 */
typedef struct asd_rivetar_layer_config {
    int type;                               /* 0 latent attention, 1 gated linear attention, 2 windowed attention */
    int heads, kv_heads, dim, vdim;         /* dim: query/key size per head (type 0: the unrotated part) */
    int rot_dim, kv_rank, q_rank;           /* type 0 */
    int decay_rank;                         /* type 1: inner size of the decay projection */
    int rot_dims, rot_interleaved;          /* rotating leading coordinates; pairs (2i, 2i+1) or (i, i + rot_dims/2) */
    int window, keep_first;
    float rot_base, scale, tau;
    int ff;
} asd_rivetar_layer_config;
typedef struct asd_rivetar_config {
    int width, vocab, n_layers;
    float eps, embed_scale, logit_softcap;
    int loop_start, loop_stop, loop_times;
    int max_tokens, page_size, ring, dtype;
} asd_rivetar_config;
typedef struct asd_rivetar_engine asd_rivetar_engine_t;

ASD_API asd_rivetar_engine_t* asd_rivetar_create(const asd_rivetar_config* cfg, const asd_rivetar_layer_config* layers);
ASD_API void asd_rivetar_destroy(asd_rivetar_engine_t* e);
/* Weights by name; matrices row-major [out, in] in the engine's dtype, vectors always fp32.  layer -1: "embed"
 * [vocab, width], "final_norm" [width], "head" [vocab, width], "loop_in" [width, 2 width], "loop_step" [times, width].
 * Every layer: "norm1", "norm1b" (and "norm2", "norm2b", "w_up" [ff, width], "w_down" [width, ff], "act" [4] when
 * ff > 0), "w_o" [width, heads * vdim], "w_in" = the matrices that read the mixer input stacked by rows:
 *   type 0: [q_rank | kv_rank + rot_dim]; also "q_norm" [q_rank], "kv_norm" [kv_rank], "w_uq" [heads * (dim + rot_dim),
 *           q_rank], "w_uk" [heads][kv_rank][dim] (transposed per head), "w_uv" [heads * vdim, kv_rank];
 *   type 1: [q | k | v | gate | decay-in]; also "w_decay" fp32 [heads * dim, decay_rank], "b_decay" [heads * dim],
 *           "out_norm" [vdim];
 *   type 2: [q | k | v]; also "sink" [heads]. */
ASD_API int asd_rivetar_set_tensor(asd_rivetar_engine_t* e, int layer, const char* name, const void* data);
ASD_API size_t asd_rivetar_cache_bytes(const asd_rivetar_engine_t* e, int num_pages);
ASD_API size_t asd_rivetar_state_bytes(const asd_rivetar_engine_t* e, int max_seqs);
ASD_API int asd_rivetar_set_cache(asd_rivetar_engine_t* e, void* pool, int num_pages, const int32_t* page_table,
                                  int max_seqs, int max_pages_per_seq, float* state);
/* options: "tc_linear", "tc_min_rows", "attn_tiled" as for the Mezilix engine; "fused_attn" (1, default: tiled windowed
 * attention kernel; 0: one warp per (token, head)); "profile" */
ASD_API int asd_rivetar_set_option(asd_rivetar_engine_t* e, const char* name, int value);
/* Same arguments as asd_engine_forward (M <= max_tokens).  layer_out (optional, fp32 [runs][M][width]) receives the
 * stream that leaves every layer execution. */
ASD_API int asd_rivetar_forward(asd_rivetar_engine_t* e, const int32_t* tokens, const int32_t* positions,
                                const int32_t* token_slot, int M, const int32_t* cu_q, const int32_t* seq_slot, int nseq,
                                int max_qlen, int max_kv_len, const int32_t* logit_rows, int n_logit_rows,
                                float* logits_out, long long logits_ld, float* layer_out, void* stream);
/* ms and launches by kernel class since the last read (nclass >= 8): 0 dense projections, 1 per-head latent products,
 * 2 latent attention, 3 windowed attention, 4 recurrence, 5 feed-forward activation, 6 norms / rotations / cache
 * append, 7 output head */
ASD_API int asd_rivetar_profile_read(asd_rivetar_engine_t* e, float* ms_by_class, int* launches_by_class, int nclass);
ASD_API int asd_rivetar_device_error(asd_rivetar_engine_t* e);

/* ------------------------------------------------------------------------------------------------------------------
 * Mavipel family engine (mavipel_engine.cu).  x = group_norm(embed[token]) * embed_norm; every layer is pre-normed,
 * x <- x + mixer(norm1(x)), x <- x + ff(norm2(x)); logits = head . final_norm(x).  Every norm splits its row into
 * norm_groups equal consecutive parts, divides each by its root mean square (eps inside the root) and multiplies by a
 * plain weight.  A layer's mixer is
 *   type 0  gated delta rule: q, k (kv_heads x dim) and v (heads x vdim) pass a short causal convolution over time
 *           (`conv` taps per channel) and silu; q and k become unit vectors per head, q times dim^(-1/2); a write
 *           strength beta = sigmoid per head; a decay per head and key channel exp(-exp(a_log[head]) softplus(.)) from
 *           a two-matrix projection of inner size decay_rank; per head S <- diag(g) S, u = beta (v - S^T k),
 *           S <- S + k u^T, o = S^T q; o / rms(o) * out_norm[vdim] * sigmoid(two-matrix projection of inner size
 *           gate_rank), then the output projection.
 *   type 1  two mixers on the same input, left_scale * left + right_scale * right.  Left: grouped-query attention
 *           (a_heads, a_kv_heads, a_dim, a_vdim) with biased projections, RMS norm of every query / key head (weights
 *           [a_dim]), rotation of the leading rot_dims coordinates in pairs (2i, 2i + 1) by position * rot_base^(-2i /
 *           rot_dims), scores * scale, capped by softcap * tanh(. / softcap) (softcap 0: not capped), mixed across the
 *           heads by talk [a_heads][a_heads], a sliding window (i sees j <= i with i - j < window) and a softmax whose
 *           denominator also holds exp(sink[head]).  Right: generalised delta rule over r_heads heads of r_dim: decay
 *           w = exp(-e^(-1/2) sigmoid(W2 tanh(W1 h) + b)) (inner size r_decay_rank), removal rate a = sigmoid(. + bias),
 *           n = unit key; S <- diag(w) S - (a * n)(n^T S) + k v^T (both terms read the old state), o = S^T r;
 *           o / rms(o) per head * out_norm[r_heads * r_dim] * sigmoid(gate projection).
 * ff_kind 0: none; 1: W_down gelu_tanh(W_up h); 2: `experts` gated experts W_down (silu(W_gate h) * W_up h) of which
 * every token takes the `top` with the largest router logits (fp32, biased), weighted by the softmax over those logits
 * alone, plus a shared expert of size shared_ff for every token (0: none).
 * Layers loop_start .. loop_stop - 1 run loop_times times with the same weights (0: no repeated span); every execution
 * ("run") has its own cache and state, and loop_step[pass] is added to x before a pass's first layer.
 *
 * dtype as for the Rivetar engine.  Paged pool: per run of a type 1 layer [num_pages][page_size][a_kv_heads * (a_dim +
 * a_vdim)], keys then values, runs back to back.  State (caller allocated, fp32), per run: the convolution's carried
 * inputs [max_seqs][conv - 1 + ring - 1][channels] (type 0), then the recurrent state [max_seqs][ring][heads][dim][vdim]
 * (type 1: [r_heads][r_dim][r_dim]); entry position % ring holds the state AFTER that position, so a caller may re-feed
 * any of the last `ring` positions; a run that starts at position 0 starts from zero.
 */
typedef struct asd_mavipel_layer_config {
    int type;                                              /* 0 gated delta rule, 1 attention + generalised delta rule */
    int heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank;            /* type 0 */
    int a_heads, a_kv_heads, a_dim, a_vdim, rot_dims, window;               /* type 1, left */
    int r_heads, r_dim, r_decay_rank;                                       /* type 1, right */
    int ff_kind, ff, experts, top, expert_ff, shared_ff;
    float rot_base, scale, softcap, left_scale, right_scale;
} asd_mavipel_layer_config;
typedef struct asd_mavipel_config {
    int width, vocab, n_layers;
    float eps;
    int norm_groups;
    int loop_start, loop_stop, loop_times;
    int max_tokens, page_size, ring, dtype;
} asd_mavipel_config;
typedef struct asd_mavipel_engine asd_mavipel_engine_t;

ASD_API asd_mavipel_engine_t* asd_mavipel_create(const asd_mavipel_config* cfg, const asd_mavipel_layer_config* layers);
ASD_API void asd_mavipel_destroy(asd_mavipel_engine_t* e);
/* Weights by name; matrices row-major [out, in] in the engine's dtype, vectors and everything marked fp32 always fp32.
 * layer -1: "embed" [vocab, width], "embed_norm" [width], "final_norm" [width], "head" [vocab, width], "loop_step"
 * [times, width].  Every layer: "norm1" (and "norm2" when ff_kind > 0), "w_o" = the output projections side by side
 * [width, columns], "w_in" = the matrices that read the mixer input stacked by rows:
 *   type 0: [q | k | v | beta | decay-in | gate-in]; also "conv_w" fp32 [q, k, v channels][conv], "a_log" [heads],
 *           "w_decay" fp32 [heads * dim, decay_rank], "b_decay" [heads * dim], "w_gate" fp32 [heads * vdim, gate_rank],
 *           "out_norm" [vdim];
 *   type 1: [left q | k | v | right r | k | v | gate | rate | decay-in]; also "in_bias" [left q | k | v], "q_norm",
 *           "k_norm" [a_dim], "talk" fp32 [a_heads, a_heads], "sink" [a_heads], "w_decay" fp32 [r_heads * r_dim,
 *           r_decay_rank], "b_decay", "rate_bias", "out_norm" [r_heads * r_dim].
 * ff_kind 1: "w_up" [ff, width], "w_down" [width, ff].  ff_kind 2: "router" fp32 [experts, width], "router_b"
 * [experts], "w_gu" [experts][2 expert_ff, width] (gate rows, then up rows), "w_edown" [experts][width, expert_ff],
 * and with a shared expert "w_sgu" [2 shared_ff, width], "w_sdown" [width, shared_ff]. */
ASD_API int asd_mavipel_set_tensor(asd_mavipel_engine_t* e, int layer, const char* name, const void* data);
ASD_API size_t asd_mavipel_cache_bytes(const asd_mavipel_engine_t* e, int num_pages);
ASD_API size_t asd_mavipel_state_bytes(const asd_mavipel_engine_t* e, int max_seqs);
ASD_API int asd_mavipel_set_cache(asd_mavipel_engine_t* e, void* pool, int num_pages, const int32_t* page_table,
                                  int max_seqs, int max_pages_per_seq, float* state);
/* options: "tc_linear", "tc_min_rows" as for the Mezilix engine; "attn_mma" (1, default: prompts and portions of a bf16
 * engine take the tensor-core window attention where the sizes allow; 0: always the CUDA-core kernel); "profile" */
ASD_API int asd_mavipel_set_option(asd_mavipel_engine_t* e, const char* name, int value);
/* Same arguments as asd_engine_forward (M <= max_tokens).  layer_out (optional, fp32 [runs][M][width]) receives the
 * stream that leaves every layer execution. */
ASD_API int asd_mavipel_forward(asd_mavipel_engine_t* e, const int32_t* tokens, const int32_t* positions,
                                const int32_t* token_slot, int M, const int32_t* cu_q, const int32_t* seq_slot, int nseq,
                                int max_qlen, int max_kv_len, const int32_t* logit_rows, int n_logit_rows,
                                float* logits_out, long long logits_ld, float* layer_out, void* stream);
/* ms and launches by kernel class since the last read (nclass >= 8): 0 dense projections, 1 window attention,
 * 2 recurrences, 3 expert layers, 4 router, 5 feed-forward activations, 6 norms / convolution / channel functions /
 * cache append, 7 output head */
ASD_API int asd_mavipel_profile_read(asd_mavipel_engine_t* e, float* ms_by_class, int* launches_by_class, int nclass);
ASD_API int asd_mavipel_device_error(asd_mavipel_engine_t* e);

/* ------------------------------------------------------------------------------------------------------------------
 * Lukopel family engine (lukopel_engine.cu).  x = embed[token] * embed_scale + pos[position]; a token carries `streams`
 * residual streams, all equal to x at the start.  Sublayer q of a layer (1 mixer, 2 feed-forward) reads
 * u = sum_s hc<q>_read[s] x_s, computes y = sublayer(u / rms(u) * norm<q>) and writes all streams at once from the old
 * ones, x_t <- sum_s hc<q>_mix[s][t] x_s + hc<q>_write[t] y.  A layer without these weights reads the plain sum and
 * adds y (with one stream: the ordinary residual).  logits = head . final_norm(sum of the streams).
 * The mixer is grouped-query softmax attention (heads, kv_heads, dim, vdim; query head h reads key/value head
 * h / (heads / kv_heads)); its steps are parameters:
 *   in_bias (tensor)    biases of q | k | v
 *   norm_whole          0: every query / key head is RMS-normed over dim with weights [dim] shared by the heads;
 *                       1: the whole query (key) projection is normed at once with weights [heads * dim] ([kv_heads * dim])
 *   temp_every, temp_coef   queries times 1 + temp_coef * ln(floor((position + 1) / temp_every) + 1)  (temp_every 0: not)
 *   head_factor (tensor)    queries of head h times head_factor[h]
 *   v_unit              every value head is divided by its root mean square (eps inside the root) before it is cached
 *   dist_bias (tensor)  fp32 [far + 1][heads]: added to the score at distance min(i - j, far), after scores * scale
 *   chunk               0: position i sees every j <= i; else only those with floor(j / chunk) == floor(i / chunk)
 *   talk (tensor)       fp32 [heads][heads]: softmax weights mixed across the heads, w'_h = sum_g talk[h][g] w_g
 *   gated               the input projection has `heads` more rows; head h's result is multiplied by their sigmoid
 *   o_bias (tensor)     bias of the output projection
 * ff_kind 0: none; 1: W_down relu(W_up h + up_bias)^2 + down_bias.
 * Layers loop_start .. loop_stop - 1 run loop_times times with the same weights (0: no repeated span); every execution
 * ("run") has its own cache.  dtype as for the Rivetar engine.  Paged pool: per run [num_pages][page_size][kv_heads *
 * (dim + vdim)], keys then values, runs back to back.  Nothing else is carried between forwards.
 */
typedef struct asd_lukopel_layer_config {
    int heads, kv_heads, dim, vdim;
    int norm_whole, v_unit, gated, chunk, far, temp_every;
    int ff_kind, ff;
    float scale, temp_coef;
} asd_lukopel_layer_config;
typedef struct asd_lukopel_config {
    int width, vocab, n_layers;
    float eps, embed_scale;
    int streams, max_positions;
    int loop_start, loop_stop, loop_times;
    int max_tokens, page_size, ring, dtype;
} asd_lukopel_config;
typedef struct asd_lukopel_engine asd_lukopel_engine_t;

ASD_API asd_lukopel_engine_t* asd_lukopel_create(const asd_lukopel_config* cfg, const asd_lukopel_layer_config* layers);
ASD_API void asd_lukopel_destroy(asd_lukopel_engine_t* e);
/* Weights by name; matrices row-major [out, in] in the engine's dtype, vectors and everything marked fp32 always fp32.
 * layer -1: "embed" [vocab, width], "pos" [max_positions, width] (engine's dtype; optional), "final_norm" [width],
 * "head" [vocab, width].  Every layer: "norm1", "w_in" = [q | k | v | gate rows] stacked by rows, "w_o" [width, heads *
 * vdim], optional "in_bias", "o_bias", "q_norm", "k_norm", "head_factor", "dist_bias", "talk" as above; with ff_kind 1
 * "norm2", "w_up" [ff, width], "up_bias", "w_down" [width, ff], "down_bias"; optional "hc1_read", "hc1_write" [streams],
 * "hc1_mix" [streams][streams] (from-stream major) and the same for "hc2_". */
ASD_API int asd_lukopel_set_tensor(asd_lukopel_engine_t* e, int layer, const char* name, const void* data);
ASD_API size_t asd_lukopel_cache_bytes(const asd_lukopel_engine_t* e, int num_pages);
ASD_API size_t asd_lukopel_state_bytes(const asd_lukopel_engine_t* e, int max_seqs);   /* 0: the cache is all */
ASD_API int asd_lukopel_set_cache(asd_lukopel_engine_t* e, void* pool, int num_pages, const int32_t* page_table,
                                  int max_seqs, int max_pages_per_seq, float* state);
/* options: "tc_linear", "tc_min_rows" as for the Mezilix engine; "attn_general" (1: every attention runs the general
 * CUDA-core kernels; 0, default: steps of few tokens and, in a bf16 engine, prompts on the tensor cores take kernels of
 * their own where the sizes allow); "profile" */
ASD_API int asd_lukopel_set_option(asd_lukopel_engine_t* e, const char* name, int value);
/* Same arguments as asd_engine_forward (M <= max_tokens).  layer_out (optional, fp32 [runs][M][width]) receives the
 * sum of the streams that leaves every layer execution. */
ASD_API int asd_lukopel_forward(asd_lukopel_engine_t* e, const int32_t* tokens, const int32_t* positions,
                                const int32_t* token_slot, int M, const int32_t* cu_q, const int32_t* seq_slot, int nseq,
                                int max_qlen, int max_kv_len, const int32_t* logit_rows, int n_logit_rows,
                                float* logits_out, long long logits_ld, float* layer_out, void* stream);
/* ms and launches by kernel class since the last read (nclass >= 5): 0 dense projections, 1 attention, 2 feed-forward
 * activations, 3 embedding / stream reads and writes / norms / cache append, 4 output head */
ASD_API int asd_lukopel_profile_read(asd_lukopel_engine_t* e, float* ms_by_class, int* launches_by_class, int nclass);
ASD_API int asd_lukopel_device_error(asd_lukopel_engine_t* e);

#ifdef __cplusplus
}
#endif
#endif /* ASD_B200_H */
