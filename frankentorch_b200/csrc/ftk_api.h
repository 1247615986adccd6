// C ABI of the sm_100a kernel library (libftk_sm100.so).
//
// Every launcher takes raw device pointers plus a CUDA stream handle and returns
// 0 on success, a negative value for rejected arguments, or a positive CUDA /
// driver error code.  Launchers never allocate device memory and never
// synchronise; the caller owns all buffers.  Asynchronous protocol failures
// (a bounded wait that ran out) are reported through the per-device status word
// returned by ftk_status_word() / read by ftk_read_status().
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// GEMM epilogues
enum {
  FTK_EPI_NONE = 0,
  FTK_EPI_GELU_TANH = 1,
  FTK_EPI_GELU_ERF = 2,
  FTK_EPI_RELU = 3,
  // the `resid` operand is the saved pre-activation u; result = acc * f'(u)
  FTK_EPI_MUL_DGELU_TANH = 4,
  FTK_EPI_MUL_DGELU_ERF = 5,
  FTK_EPI_MUL_DRELU = 6,
};

typedef struct FtkGemmDesc {
  int M, N, K;
  int L0, L1;            // batch extents (>=1); batch index l = l0 + L0*l1
  int a_mn, b_mn;        // 0: operand stored [rows, K]; 1: stored [K, rows]
  const void* A;         // bf16
  long long lda, a_s0, a_s1;
  const void* B;         // bf16
  long long ldb, b_s0, b_s1;
  void* D;               // bf16 or fp32, [M, N] row-major per batch
  long long ldd, d_s0, d_s1;
  const void* bias;      // bf16 [N] or NULL
  const void* resid;     // bf16, same shape as D, or NULL
  long long ldr, r_s0, r_s1;
  void* aux;             // bf16 pre-activation copy (layout of D) or NULL
  float alpha;
  int epi;
  int out_fp32;
  int accumulate;        // D += result
  int force_bn;          // 0 = heuristic, else 128 or 256
  int max_ctas;          // 0 = all SMs
  // Deterministic split-K (plain fp32/bf16 store epilogues only): partial tiles go to
  // `workspace` (fp32, split_count*M*N*4 bytes needed) and are summed in ascending split order.
  void* workspace;       // NULL disables split-K
  long long workspace_bytes;
  int split_k;           // 0 = heuristic, 1 = off, >1 = forced
  // Stream for the split-K reduction kernel (NULL = the GEMM's stream).  With another stream the
  // launcher orders the reduction behind the GEMM through an event and the caller joins that
  // stream before it reads D or reuses the workspace; the next kernel on the GEMM's stream then
  // overlaps the reduction.
  void* reduce_stream;
  // Ragged rows: the M rows (of every batch) are segments of seg_rows rows, of which only the first
  // seg_counts[batch * ceil(M / seg_rows) + segment] (device, int32) are in use.  128-row tiles
  // without a row in use are skipped entirely: their part of D is left untouched.  NULL = dense.
  // Single-CTA tiles only (no CTA pairs, no split-K).
  const int* seg_counts;
  int seg_rows;
} FtkGemmDesc;

int* ftk_status_word(void);               // device pointer (allocated on first use, per device)
int ftk_read_status(int reset);           // synchronises the device; returns the status word
int ftk_gemm_bf16(const FtkGemmDesc* g, void* stream);
// Which kernel ftk_gemm_bf16 would launch: *bn = 128 / 192 / 256 (one CTA per 128 x bn tile) or
// 512 (CTA-pair kernel, 256 x 256 tiles, cta_group::2); *splits = split-K factor.  No launch.
int ftk_gemm_plan(const FtkGemmDesc* g, int* bn, int* splits);
// `n` (1..8) products with one K and one pair of operand layouts, fp32 outputs (store or accumulate), no other
// epilogue, as one persistent launch of 128 x 192 tiles: the weight gradients of a transformer block fill the
// GPU together where each alone would need split-K and a reduction kernel.
int ftk_gemm_group_bf16(const FtkGemmDesc* descs, int n, void* stream);

// ---- GEMM fused with a collective over NVLink peer memory --------------------------------
// One kernel: `comm_ctas` CTAs move shards / reduce partials while the rest run the GEMM.
//  GATHER_A : A = [world * chunk_rows, K] is row-sharded; shard r is read from src[r]
//             (contiguous [chunk_rows, K], peer or local memory) into g->A (local staging,
//             lda == K) while tiles of shards already staged are multiplied.
//  GATHER_B : the same for B = [world * chunk_rows, K] (weights sharded by output row).
//  SCATTER_D: D = [world * chunk_rows, N] partial sums; rows of rank r go to inbox[r]
//             (bf16 [world][chunk_rows][N] on rank r) and rank r adds the world partials in
//             ascending rank order into g->D ([chunk_rows, N], + bias, + resid, accumulate).
// `epoch` is a device word holding the use count (1, 2, ...) of the flag arrays; the caller
// advances it before each launch, identically on every rank.  Flag arrays start at zero.
enum FtkCommMode {
  FTK_COMM_NONE = 0,
  FTK_COMM_GATHER_A = 1,
  FTK_COMM_GATHER_B = 2,
  FTK_COMM_SCATTER_D = 3,
};
#define FTK_MAX_RANKS 8
typedef struct FtkCommDesc {
  int mode, rank, world;
  int comm_ctas;                       // 0 = default
  int chunk_rows;                      // multiple of 128
  const void* src[FTK_MAX_RANKS];      // gather: shard pointers (entry `rank` is local)
  int* sub_flags;                      // gather: [world * chunk_rows / 128] local words
  int* ready_local;                    // gather: [world] local words, NULL = shards known final
  int* ready_peer[FTK_MAX_RANKS];      // gather: &ready_local[rank] on each peer
  void* inbox[FTK_MAX_RANKS];          // scatter: inbox of every rank
  int* arrive[FTK_MAX_RANKS];          // scatter: [chunk tiles][world] words on every rank
  const int* epoch;
  // gather, push form (push != 0): every rank stores its own shard into the staging buffer of every
  // peer and sets the flags there; the GEMM's staged operand (A or B) must be full_peer[rank] and
  // sub_flags must be flags_peer[rank].  Consecutive calls must alternate two staging buffers.
  // push == 2: the shards are delivered from outside the kernel (ftk_copy_async + ftk_set_flags_sys on
  // another stream, i.e. by the copy engines); the kernel has no copy CTAs and only polls the flags.
  // push == 3: no copy CTAs either; the epilogue warps of every CTA store the shard into the peers' staging
  // buffers while they wait for their accumulators.
  int push;
  void* full_peer[FTK_MAX_RANKS];
  int* flags_peer[FTK_MAX_RANKS];
} FtkCommDesc;
int ftk_gemm_comm_bf16(const FtkGemmDesc* g, const FtkCommDesc* c, void* stream);
int ftk_tick_i32(int* word, void* stream);    // *word += 1 on the stream
int ftk_set_flags_sys(int* flags, int n, const int* epoch, void* stream);   // flags[0..n) = *epoch, release.sys
int ftk_copy_async(void* dst, const void* src, long long bytes, void* stream);   // copy-engine D2D copy

// ---- mixture of experts: top-2 routing and expert-parallel all-to-alls over peer memory ---
// Expert e lives on rank e / (E / world).  A rank sends at most `capacity` rows to each expert;
// receive buffers are [E / world][world][capacity][d] bf16 on every rank (symmetric).
typedef struct FtkMoeDesc {
  int T, d, E, capacity, rank, world;
  const int* idx;      // [T, 2] chosen experts
  const int* slot;     // [T, 2] slot inside (this rank, expert), -1 = dropped
  const int* counts;   // [E] rows this rank sends to each expert
  int* ticket;         // local scratch word, zero between launches
  const int* epoch;    // device word: use count of the flag arrays (advance before each call)
} FtkMoeDesc;
// logits fp32 [T, ld] (first E columns used); d_logits bf16 [T, ld] (columns >= E zeroed)
int ftk_moe_route(const float* logits, float* probs, int* idx, float* gate, int T, int E, int ld,
                  void* stream);
int ftk_moe_route_bwd(const float* probs, const int* idx, const float* d_gate, void* d_logits, int T,
                      int E, int ld, void* stream);
int ftk_moe_gate_grad(const void* g, const void* rows, float* d_gate, int T, int d, void* stream);
int ftk_moe_slots(const int* idx, int* slot, int* counts, int T, int E, int capacity, void* stream);
// rows of x (scaled by scale[t,k] when given) -> recv[expert rank]; waits for all sources and
// zeroes the unused rows of this rank's own buffer.  arrive[r]: [world] words on rank r.
int ftk_moe_dispatch(const FtkMoeDesc* m, const void* x, const float* scale, void* const* recv,
                     int* const* recv_counts, int* const* arrive, void* stream);
// out[t] = gate[t,0] * y[e0][slot0] + gate[t,1] * y[e1][slot1] (+ resid[t]); optionally keeps the
// pulled rows ([T, 2, d]) for the gate gradient.  ready[r]: [world] words on rank r.
int ftk_moe_combine(const FtkMoeDesc* m, void* const* y, int* const* ready, const float* gate, void* out,
                    const void* resid, void* rows, void* stream);

// ---- attention (causal / full), packed QKV layout ---------------------------------------
// q/k/v: bf16 element (b, s, h, e) at base[b*bs + s*ss + h*hs + e]; head_dim in {64, 128}.
// o: same addressing with its own strides.  lse: fp32 [B, H, S], log2 domain.
typedef struct FtkAttnDesc {
  int B, H, S, hd;
  int causal;
  float scale;           // softmax scale (1/sqrt(hd) by default)
  const void *q, *k, *v;
  long long q_bs, q_ss, q_hs;
  long long k_bs, k_ss, k_hs;
  long long v_bs, v_ss, v_hs;
  void* o;
  long long o_bs, o_ss, o_hs;
  float* lse;
  // backward only
  const void* d_o;       // bf16, addressing of o
  float* delta;          // fp32 [B, H, S] scratch: rowsum(dO * O)
  void *dq, *dk, *dv;    // bf16, addressing of q / k / v respectively
} FtkAttnDesc;
int ftk_attn_fwd(const FtkAttnDesc* a, void* stream);
int ftk_attn_bwd(const FtkAttnDesc* a, void* stream);

// ---- row kernels ------------------------------------------------------------------------
// LayerNorm over the last dim (population variance, eps inside the sqrt), bf16 in/out,
// fp32 statistics.  If resid_in != NULL the kernel first forms x = x + resid_in, writes it
// to sum_out (bf16) and normalises that (fused residual-add + LN).
int ftk_layernorm_fwd(const void* x, const void* resid_in, void* sum_out, const void* gamma,
                      const void* beta, void* y, float* mean, float* rstd, int rows, int cols,
                      float eps, void* stream);
// dx (bf16, optionally += dx_accum_in), and per-block partial dgamma/dbeta reduced in a
// second fixed-order pass (dgamma/dbeta fp32 [cols]); partial must hold 2*nblk*cols floats,
// nblk = ftk_layernorm_bwd_blocks(rows).
int ftk_layernorm_bwd_blocks(int rows);
int ftk_layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean,
                      const float* rstd, const void* dx_add, void* dx, float* dgamma, float* dbeta,
                      float* partial, int rows, int cols, int accumulate_param_grads, void* stream);
int ftk_rmsnorm_fwd(const void* x, const void* gamma, void* y, float* rstd, int rows, int cols,
                    float eps, void* stream);
int ftk_rmsnorm_bwd(const void* dy, const void* x, const void* gamma, const float* rstd, void* dx,
                    float* dgamma, float* partial, int rows, int cols, int accumulate_param_grads,
                    void* stream);
// Row softmax over the last dim with the guards of the reference shader (non-finite max ->
// zeros, zero sum -> zeros).  fp32 or bf16 by `is_bf16`.
int ftk_softmax_rows(const void* x, void* y, int rows, int cols, int is_bf16, void* stream);
// Causal row softmax over [L, S, S] score matrices (unfused attention oracle path), bf16.
int ftk_softmax_causal_bf16(const void* x, void* y, int L, int S, float scale, void* stream);
int ftk_softmax_bwd_bf16(const void* y, const void* dy, void* dx, long long rows, int cols,
                         float scale, void* stream);

// Fused softmax-cross-entropy over bf16 logits [rows, ld] (first `vocab` columns valid).
// losses: fp32 [rows]; dlogits (may alias logits) = (softmax - onehot) * grad_scale, bf16,
// padded columns written as zero.  targets: int64.
int ftk_cross_entropy_fwd_bwd(const void* logits, const long long* targets, float* losses,
                              void* dlogits, int rows, int vocab, int ld, float grad_scale,
                              void* stream);
// Fixed-tree mean of `n` fp32 values into out[0] (single block, pairwise tree).
int ftk_reduce_mean_f32(const float* x, float* out, long long n, float scale, void* stream);
// Sum of squares with a fixed two-level tree: out[0] += / = sum(x^2).  `partial` holds
// FTK_SUMSQ_PARTIALS floats (may be NULL for small n).
#define FTK_SUMSQ_PARTIALS 1024
int ftk_sumsq_f32(const float* x, float* out, float* partial, long long n, int accumulate,
                  void* stream);

// ---- elementwise ------------------------------------------------------------------------
int ftk_gelu_fwd(const void* x, void* y, long long n, int tanh_form, void* stream);
int ftk_gelu_bwd(const void* x, const void* dy, void* dx, long long n, int tanh_form, void* stream);
int ftk_add_bf16(const void* a, const void* b, void* out, long long n, void* stream);
int ftk_cast_f32_to_bf16(const float* x, void* y, long long n, void* stream);
int ftk_cast_bf16_to_f32(const void* x, float* y, long long n, int accumulate, void* stream);
// counter-based (Philox-4x32-10) dropout; mask is recomputed in backward from (seed, offset).
int ftk_dropout_bf16(const void* x, void* y, long long n, float p, unsigned long long seed,
                     unsigned long long offset, void* stream);
// column sums of a bf16 [rows, cols] matrix into fp32 [cols] (bias gradients), fixed order.
int ftk_colsum_bf16(const void* x, float* out, float* partial, int rows, int cols, long long ld,
                    int accumulate, void* stream);
int ftk_colsum_blocks(int rows);

// ---- embedding --------------------------------------------------------------------------
// out[r, :] = wte[ids[r], :] + wpe[r % S, :]  (wpe may be NULL).  `vocab` = rows of wte: an id outside
// [0, vocab) is reported through the status word (BAD_INDEX) and row 0 is read in its place.
int ftk_embedding_fwd(const long long* ids, const void* wte, const void* wpe, void* out, int rows,
                      int S, int d, long long vocab, void* stream);
// Deterministic scatter-add: `sorted_ids`/`order` come from a stable sort of the ids, so
// each table row is summed by one CTA in ascending source-row order.
// dwte fp32 [vocab, d] (+=), dwpe fp32 [S, d] (+=); either may be NULL.  Rows of ids outside [0, vocab)
// are skipped and reported through the status word.
int ftk_embedding_bwd(const long long* sorted_ids, const int* order, const void* dout, float* dwte,
                      float* dwpe, int rows, int S, int d, long long vocab, void* stream);

// The same sums without a sort (ids in their original order, d <= 1024): the CTA of a token's first occurrence adds
// the rows of all its occurrences in ascending position order; bit-identical to the sorted form.
int ftk_embedding_bwd_scan(const long long* ids, const void* dout, float* dwte, float* dwpe, int rows, int S,
                           int d, long long vocab, void* stream);

// ---- optimizer --------------------------------------------------------------------------
// Fused AdamW on fp32 master weights with bf16 shadow write-back.  grad fp32.
// Reference math: ft-optim/src/lib.rs:1040-1054.
int ftk_adamw(float* master, void* shadow_bf16, const float* grad, float* m, float* v, long long n,
              float lr, float beta1, float beta2, float eps, float weight_decay, float bc1,
              float bc2, float grad_scale, void* stream);

// ---- presenter / misc -------------------------------------------------------------------
// RGBA8 rows (row_bytes stride) -> normalised float4 or half4 headless buffer.
int ftk_present_rgba8(const unsigned char* src, void* dst, int width, int height,
                      long long row_bytes, int dst_half, void* stream);
// 1-D convolution-over-time gather X[t_in, cin] -> Y[t_out, cin*k] with zero padding.
int ftk_im2col_1d(const float* x, float* y, int t_in, int cin, int k, int stride, int pad,
                  int t_out, void* stream);
// Bounded-wait self test: waits up to budget_cycles (<= 4e9) for *flag >= want; on timeout the
// status word gets FT_ERR_WAIT_PEER and *waited_cycles the cycles spent.  Never blocks longer.
int ftk_wait_probe(const int* flag, int want, long long budget_cycles, long long* waited_cycles,
                   void* stream);

#ifdef __cplusplus
}
#endif

// ---- graph-replayable optimizer step (C linkage) --------------------------------------------
#ifdef __cplusplus
extern "C" {
#endif
// hyper (device, fp32[4]) = {lr, bias_correction1, bias_correction2, grad_scale}; `step`
// (device, int64) is incremented by the tick so a captured graph advances on every replay.
int ftk_adamw_tick(long long* step, float* hyper, double beta1, double beta2, void* stream);
int ftk_clip_scale(const float* sumsq, float max_norm, float* hyper, float* norm_out, void* stream);
int ftk_adamw_dev(float* master, void* shadow_bf16, const float* grad, float* m, float* v, long long n,
                  const float* hyper, float beta1, float beta2, float eps, float weight_decay,
                  void* stream);
int ftk_fill_f32(float* x, long long n, float v, void* stream);
// *out = %globaltimer (ns) when the stream reaches this point (capturable in a CUDA graph).
int ftk_timestamp(unsigned long long* out, void* stream);
#ifdef __cplusplus
}
#endif

// ---- bucketed data-parallel optimizer step over peer memory (dp_fused.cu) --------------------
#ifdef __cplusplus
extern "C" {
#endif
#define FTK_DP_MAX_RANKS 16
#define FTK_DP_MAX_BUCKETS 64
// One bucket of the flat parameter arena (all counts in elements).  `shard` (a multiple of 8) is
// the number of elements of the bucket each rank owns: rank r owns [lo + r*shard, lo + (r+1)*shard)
// clipped to hi.  `off` is where that shard starts in the rank-local shard arrays (fp32 master,
// moments, reduced gradient); the bucket's W inbox slots start at world*off in the inbox.
typedef struct {
  long long lo, hi, shard, off;
} FtkDpBucket;
// This rank's view of the job.  inbox / params / flags / slots: `world` pointers each, entry r
// being rank r's buffer mapped into this process (entry `rank` is the local buffer).
//   flags : u64 [3][FTK_DP_MAX_BUCKETS][FTK_DP_MAX_RANKS], zero-initialised, never cleared
//   slots : fp32 [FTK_DP_MAX_RANKS]
//   inbox : wire type (bf16, or fp32 when wire_fp32) [world * sum of shards]
// Local device memory: buckets (table of n_buckets entries), gshard fp32 [sum of shards],
// partial fp32 [n_buckets * n_ctas] (n_ctas = the widest grid any bucket is launched with),
// counters u32 [2 * FTK_DP_MAX_BUCKETS] (zero-initialised), seq (step sequence number, advanced
// by ftk_dp_begin_step), ok_word (1 = step healthy), pending (1 = reduced gradients wait for their
// update), hyper_pending fp32[4] (the hyper-parameters that update will use).
typedef struct {
  void* const* inbox;
  void* const* params;
  void* const* flags;
  void* const* slots;
  const FtkDpBucket* buckets;
  int rank, world, n_buckets, n_ctas, wire_fp32;
  float* gshard;
  float* partial;
  unsigned int* counters;
  long long* seq;
  int* ok_word;
  int* pending;
  float* hyper_pending;
  void* params_mc;   // multicast address covering every rank's parameter arena (NVLS), or NULL
} FtkDpComm;
int ftk_dp_begin_step(const FtkDpComm* c, void* stream);
int ftk_dp_bucket_reduce(const FtkDpComm* c, int bucket, const float* grads, int n_ctas, void* stream);
// extra_sumsq (device, may be NULL): squared norm of gradients only this rank holds; it is added to
// the rank's share before the exchange, so the clip factor comes from the norm of ALL gradients.
int ftk_dp_norm(const FtkDpComm* c, float max_norm, float* hyper, float* norm_out, const float* extra_sumsq,
                void* stream);
int ftk_dp_update(const FtkDpComm* c, int b0, int b1, float* master, float* m, float* v,
                  float beta1, float beta2, float eps, float weight_decay, int n_ctas, void* stream);
int ftk_dp_clear_pending(const FtkDpComm* c, void* stream);
int ftk_dp_wait_params(const FtkDpComm* c, int b0, void* stream);
#ifdef __cplusplus
}
#endif

// ---- collectives through the NVSwitch multicast object (nvls.cu) -----------------------------
#ifdef __cplusplus
extern "C" {
#endif
#define FTK_NVLS_MAX_RANKS 16
// One symmetric allocation bound to a multicast object.  mc: its multicast address; local: this
// rank's own mapping; flags[r]: rank r's flag block (u64 [4][FTK_NVLS_MAX_RANKS], zero-initialised,
// inside the allocation, addressed through the ordinary peer mapping); counter: a zeroed local
// device word.  `seq` of a call must be larger than that of every earlier call on the same
// allocation and equal on all ranks.
typedef struct {
  void* mc;
  void* local;
  void* flags[FTK_NVLS_MAX_RANKS];
  unsigned int* counter;
  int rank, world;
} FtkNvlsComm;
int ftk_nvls_allgather(const FtkNvlsComm* c, const void* src, long long dst_off, long long chunk_bytes,
                       unsigned long long seq, int n_ctas, void* stream);
int ftk_nvls_allreduce(const FtkNvlsComm* c, long long off, long long n_bytes, int dtype, unsigned long long seq,
                       int n_ctas, void* stream);
#ifdef __cplusplus
}
#endif
