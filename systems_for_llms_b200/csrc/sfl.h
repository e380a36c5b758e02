/* C interface of the sm_100a kernel library (libsfl_b200.so).
 *
 * Every function takes raw device pointers plus the CUDA stream to launch on
 * (as a void*, 0 = legacy default stream) and returns 0 on success.  Nothing
 * here allocates device memory unless the function's comment says so; callers
 * (the Python layer) own all buffers.  Kernels that can wait on something
 * (pipelines, peer flags) bound their waits and report through an optional
 * `int* status` device word: 0 = ok, see StatusCode in ptx.cuh.
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ GEMM -- */
enum {
  SFL_EPI_BF16 = 0,       /* out bf16 [M,N]                                         */
  SFL_EPI_F32 = 1,        /* out fp32 [M,N]; beta=1 accumulates                     */
  SFL_EPI_RESID = 2,      /* out fp32 = aux fp32 + bf16(acc)                        */
  SFL_EPI_ROPE = 3,       /* out bf16, rotary embedding on columns [0, rope_cols)   */
  SFL_EPI_SWIGLU = 4,     /* b = [w1; w3]; out = silu(a1)*a3, out2 = [a1 | a3]      */
  SFL_EPI_SWIGLU_BWD = 5, /* acc = dg; aux = [a1 | a3]; out = [da1 | da3]           */
};

typedef struct SflGemmEpilogue {
  int kind;
  int beta;
  void* out;
  long ldo;
  void* out2;
  long ldo2;
  const void* aux;
  long ldaux;
  const float* rope_cos; /* [rope_T, head_dim/2] fp32 (already rounded to bf16 values) */
  const float* rope_sin;
  int rope_T;
  int rope_cols;
  int head_dim;
  int dual_offset; /* SWIGLU: row of w3 inside b */
  int dual_rows;   /* SWIGLU: total rows of b    */
  int* status;
} SflGemmEpilogue;

/* D[M,N] = A * B^T with bf16 operands and fp32 accumulation.
 * a_mn = 0: a is [M,K] row-major (pitch lda); a_mn = 1: a is [K,M] row-major.
 * b_mn = 0: b is [N,K] row-major (pitch ldb); b_mn = 1: b is [K,N] row-major.
 * Pitches must be multiples of 8 elements and bases 16-byte aligned.
 * bn_hint: 0 = choose tile width automatically, else 128 or 256.
 * max_ctas: 0 = one CTA per SM, else an upper bound on the grid. */
int sfl_gemm_bf16(const void* a, long lda, int a_mn, const void* b, long ldb, int b_mn, int M,
                  int N, int K, const SflGemmEpilogue* epi, int bn_hint, int max_ctas,
                  void* stream);

/* grad[rows, cols] (+)= dy[tokens, rows]^T x[tokens, cols]; bf16 operands, fp32 grad. */
typedef struct SflWgradProblem {
  const void* dy;
  long ld_dy;
  const void* x;
  long ld_x;
  float* grad;
  long ld_grad;
  int rows;
  int cols;
  int tokens;
  int accumulate; /* 0: overwrite grad, 1: add to it */
} SflWgradProblem;

/* Up to four weight-gradient products in one persistent launch, so that their
 * tiles share the SMs.  Returns -2 if a matrix breaks TMA's alignment rules
 * (16-byte base and pitch): compute those with sfl_gemm_bf16 instead. */
int sfl_gemm_wgrad_grouped(const SflWgradProblem* problems, int count, int* status, void* stream);

/* --------------------------------------------------------------- RMSNorm -- */
/* y = bf16(x * rsqrt(mean(x^2) + eps) * w), x fp32 [rows, dim]; rstd fp32 [rows]. */
int sfl_rmsnorm_fwd(const float* x, const float* w, void* y_bf16, float* rstd, int rows, int dim,
                    float eps, void* stream);
/* dx_out = dres_in (may be NULL) + d(norm)/dx, optionally also written as bf16;
 * dw_partial [sfl_rmsnorm_bwd_blocks(rows), dim] receives per-block partial sums
 * of dy * xhat which sfl_rmsnorm_dw_reduce folds into dw (dw += sum). */
int sfl_rmsnorm_bwd_blocks(int rows);
int sfl_rmsnorm_bwd(const void* dy_bf16, const float* x, const float* w, const float* rstd,
                    const float* dres_in, float* dx_out, void* dx_out_bf16, float* dw_partial,
                    int rows, int dim, void* stream);
int sfl_rmsnorm_dw_reduce(const float* dw_partial, int blocks, float* dw, int dim, int accumulate,
                          void* stream);
/* The same for two partial buffers of the same shape in one launch. */
int sfl_rmsnorm_dw_reduce2(const float* partial_a, float* dw_a, int accumulate_a,
                           const float* partial_b, float* dw_b, int accumulate_b, int blocks,
                           int dim, void* stream);

/* --------------------------------------------------------- cross entropy -- */
/* logits bf16 [rows, vocab] (pitch ld).  Writes per-row loss (fp32) and, when
 * dlogits != NULL, (softmax - onehot) * grad_scale as bf16 (may alias logits). */
int sfl_cross_entropy(const void* logits_bf16, long ld, const int64_t* targets, float* row_loss,
                      void* dlogits_bf16, float grad_scale, int rows, int vocab, void* stream);

/* ------------------------------------------------------------- optimizer -- */
/* Sum of squares of a flat fp32 buffer -> partial[blocks]; deterministic. */
int sfl_sqnorm_blocks(long n);
int sfl_sqnorm_partial(const float* x, long n, float* partial, void* stream);
/* out[0] = sqrt(sum(partial[0..n)) * scale); out[1] = clip coefficient
 * min(1, max_norm / (out[0] + 1e-6)); out[2] = 1 if out[0] is finite else 0. */
int sfl_norm_finalize(const float* partial, int n, float sum_scale, float max_norm, float* out,
                      void* stream);
/* AdamW over a flat fp32 range.  The gradient is multiplied by *grad_coef
 * (device pointer, may be NULL) and by grad_scale first.  bf16_shadow (may be
 * NULL) receives the updated parameters rounded to bf16.  Update is skipped
 * when skip_flag != NULL and *skip_flag == 0 (non-finite gradient norm). */
int sfl_adamw(float* p, const float* g, float* m, float* v, void* bf16_shadow, long n, float lr,
              float beta1, float beta2, float eps, float weight_decay, float bias1, float bias2,
              const float* grad_coef, float grad_scale, const float* ok_flag, void* stream);

/* ------------------------------------------------------------- attention -- */
/* A [B,H,N,D] view with D contiguous; strides in elements. */
typedef struct SflAttnTensor {
  void* ptr;
  long stride_b, stride_h, stride_t;
} SflAttnTensor;

/* Block schedule at 128x128 tile granularity plus the token-level predicate.
 * mode 0: CSR over query tiles (row_ptr/col_idx/full[/bitmap]) and, for the
 * backward pass, its transpose over key tiles (t_*).  bitmap (optional) holds
 * one bit per 16x16 sub-block, bit index = (query_sub * 8 + key_sub); absent
 * sub-blocks are masked.  mode 1: interval schedule derived from the windows.
 * window_* = -1 means unbounded.  doc (optional) = int32 label per position. */
typedef struct SflAttnMask {
  int mode;
  int causal;
  int window_left;
  int window_right;
  const int* doc;
  const int* row_ptr;
  const int* col_idx;
  const uint8_t* full;
  const uint64_t* bitmap;
  const int* t_row_ptr;
  const int* t_col_idx;
  const uint8_t* t_full;
  const uint64_t* t_bitmap;
} SflAttnMask;

/* O = softmax(scale * Q K^T + mask) V; lse (may be NULL) fp32 [B,H,N] natural log.
 * 16-bit inputs (bf16, or fp16 when is_fp16), D in {64, 128}. */
int sfl_attn_fwd(const SflAttnTensor* q, const SflAttnTensor* k, const SflAttnTensor* v,
                 const SflAttnTensor* o, float* lse, int B, int H, int N, int D, float scale,
                 const SflAttnMask* mask, int is_fp16, int* status, void* stream);
/* Same with the forward kernel variant chosen by the caller: 0 = default, 1 = one work
 * stream per CTA, 2 = two streams per CTA with P kept in tensor memory, 3 = two streams with
 * P in shared memory (2 and 3 exist for head dimension 64; 128 always runs variant 1). */
int sfl_attn_fwd_pipeline(const SflAttnTensor* q, const SflAttnTensor* k, const SflAttnTensor* v,
                          const SflAttnTensor* o, float* lse, int B, int H, int N, int D,
                          float scale, const SflAttnMask* mask, int is_fp16, int pipeline,
                          int* status, void* stream);
/* Gradients of the above.  delta is fp32 [B,H,N] scratch owned by the caller (the
 * query-owned kernel fills it, the key-owned kernel reads it).  With rope_cos and
 * rope_sin (fp32 [N, D/2], 16-byte aligned; both or neither) dq and dk are written
 * already multiplied by the transposed rotary matrix of their token position, i.e.
 * as gradients of the un-rotated projections. */
int sfl_attn_bwd(const SflAttnTensor* q, const SflAttnTensor* k, const SflAttnTensor* v,
                 const SflAttnTensor* o, const SflAttnTensor* d_o, const float* lse, float* delta,
                 const SflAttnTensor* dq, const SflAttnTensor* dk, const SflAttnTensor* dv, int B,
                 int H, int N, int D, float scale, const SflAttnMask* mask, int is_fp16,
                 int* status, const float* rope_cos, const float* rope_sin, void* stream);
/* In-place inverse rotary embedding on the first `cols` columns of bf16 x[rows, ld]. */
int sfl_rope_bwd(void* x_bf16, long ld, const float* cos, const float* sin, long rows, int cols,
                 int T, int head_dim, void* stream);

/* ---------------------------------------------------------------- decode -- */
/* Single-token attention: q [B,Hq,D], k/v [B,Hkv,N,D] (contiguous, 16-bit),
 * lengths int32 [B] (clamped to [0,N]), out [B,Hq,D].  Hq/Hkv in {1,2,4,8},
 * D in {64,128}, splits in [1,128].  For splits > 1 the caller provides fp32
 * scratch part_m/part_l [B,Hq,splits], part_u [B,Hq,splits,D] and an int32
 * counters [B,Hkv] array that is zero on entry (the kernel leaves it zero). */
int sfl_decode(const void* q, const void* k, const void* v, const int* lengths, float* part_m,
               float* part_l, float* part_u, int* counters, void* out, int B, int Hq, int Hkv,
               int N, int D, int splits, float scale, int tile_variant, int is_fp16, void* stream);

/* The same split-KV decode on the tensor cores (csrc/attention.cu, decode_mma2_kernel): K / V
 * tiles of 128 cached tokens stream in through TMA; the scores are a [tokens] x [head group]
 * tcgen05 product, P^T V accumulates in tensor memory.  Same arguments, scratch layout and partitioning as sfl_decode, plus the
 * status word for its bounded waits; k and v must be 16-byte aligned. */
int sfl_decode_mma(const void* q, const void* k, const void* v, const int* lengths, float* part_m,
                   float* part_l, float* part_u, int* counters, void* out, int B, int Hq, int Hkv,
                   int N, int D, int splits, float scale, int is_fp16, int* status, void* stream);

/* Allocation-free decode.  This entry point has no counterpart in the reference.
 *
 * Same computation as sfl_decode, for callers that cannot allocate device
 * memory where they decode: inside CUDA-graph capture or a serving loop that must
 * not synchronise (cudaMalloc does both harm), in a plug-in that may not touch its
 * host's memory pool, or from plain C without a caching allocator.  The split-KV
 * scratch is a fixed array inside the library image instead of caller memory:
 *   - capacity: batch * query_heads * splits <= sfl_decode_static_capacity_slots()
 *     (8192) and batch * kv_heads <= 1024; about 4.2 MB that every GPU which loads
 *     the library keeps until the process exits.  Larger problems are rejected
 *     with a nonzero code and a message from sfl_decode_static_error().
 *   - the caller still passes q, k, v, lengths and out; nothing is allocated or
 *     freed, neither through the CUDA runtime nor through any library.
 *   - the first call on each device looks up the array's device address
 *     (with that device current); make that first call before starting any
 *     stream capture.
 *   - all calls on a device share the one array.  It keeps the previous call's
 *     contents; this function clears the part that must start at zero.  Two calls
 *     whose kernels overlap on the GPU (different streams, or different threads)
 *     race on the scratch and give wrong results: serialise them. */
int sfl_decode_static(const void* q, const void* k, const void* v, const int* lengths, void* out,
                      int B, int Hq, int Hkv, int N, int D, int splits, float scale,
                      int tile_variant, int is_fp16, void* stream);
long sfl_decode_static_capacity_slots(void);
const char* sfl_decode_static_error(void);

/* --------------------------------------------------------- communication -- */
/* Symmetric (same size on every rank) device buffers shared through CUDA IPC. */
int sfl_ipc_alloc(void** ptr, size_t bytes);               /* cudaMalloc + zero fill  */
int sfl_ipc_free(void* ptr);
int sfl_ipc_get_handle(void* ptr, void* handle64);         /* 64-byte opaque handle   */
int sfl_ipc_open_handle(const void* handle64, void** ptr); /* map a peer's buffer     */
int sfl_ipc_close_handle(void* ptr);
long sfl_comm_flag_bytes(void); /* size every rank's flag buffer must have           */
int sfl_comm_slots(void);       /* independent barrier slots (one per bucket/use)    */
int sfl_comm_max_ctas(void);
/* Polling budget of every peer wait, in iterations of about 200 ns.  The default (48 x 2^20,
 * about ten seconds) is sized for the skew between the ranks of a training job; tests of
 * the timeout path set a millisecond.  Covers the collectives and the fused GEMM +
 * all-reduce kernels (sfl_gemm_tp_set_spin_limit sets only the latter). */
int sfl_comm_set_spin_limit(unsigned iterations);
int sfl_gemm_tp_set_spin_limit(unsigned iterations);

typedef struct SflComm {
  int rank, world;   /* world <= 8                                               */
  void* data[8];     /* peer pointers of the primary symmetric buffer            */
  void* data2[8];    /* peer pointers of a second symmetric buffer (optional)    */
  void* flags[8];    /* peer pointers of the flag buffers (sfl_comm_flag_bytes)  */
} SflComm;

/* All functions below: `slot` selects a barrier slot, `epoch` must increase by
 * one for each use of that slot on every rank, `ctas` sizes the grid (<= max).
 * accumulate_partial = 1 adds this call's squared-norm partials to the slot's
 * running partials instead of replacing them (several buckets sharing a slot).
 * Offsets/counts are in fp32 elements (multiples of 4) unless named *_bytes. */

/* data[*][offset:offset+count] <- scale * sum over ranks; squared-norm partials
 * of the reduced values are left in the flag buffer for sfl_comm_norm_finalize. */
int sfl_allreduce_f32(const SflComm* comm, long offset, long count, float scale, int slot,
                      unsigned epoch, int accumulate_partial, int ctas, int* status, void* stream);
/* Rank r reduces slice r of the range into local_out (slice-relative, compact)
 * or in place when local_out is NULL.  Bit 1 of accumulate_partial (value 2) adds
 * the reduced slice to the existing contents of the destination instead of
 * overwriting it (gradient accumulation over microbatches). */
int sfl_reduce_scatter_f32(const SflComm* comm, long offset, long count, float scale,
                           float* local_out, int slot, unsigned epoch, int accumulate_partial,
                           int ctas, int* status, void* stream);
/* out[0]=global norm over the listed slots (+ *extra_sq), out[1]=clip coef, out[2]=finite. */
int sfl_comm_norm_finalize(const SflComm* comm, const int* slots_dev, int n_slots, int ctas,
                           float max_norm, const float* extra_sq, float* out, void* stream);
/* AdamW on this rank's slice of data[rank][offset:offset+count] using the
 * reduced gradient slice, then write fp32 parameters to data[*] and bf16 to data2[*]. */
int sfl_adamw_allgather(const SflComm* comm, long offset, long count, const float* grad, float* m,
                        float* v, float lr, float beta1, float beta2, float eps, float wd,
                        float bias1, float bias2, const float* coef, const float* ok, int slot,
                        unsigned epoch, int ctas, int* status, void* stream);
/* The same update for a table of ranges in one launch (one barrier pair):
 * ranges (device memory) holds {element offset, element count, offset of this
 * rank's slice inside grad / m / v} per range; counts and offsets are multiples
 * of four elements. */
int sfl_adamw_allgather_ranges(const SflComm* comm, const long* ranges, int num_ranges,
                               const float* grad, float* m, float* v, float lr, float beta1,
                               float beta2, float eps, float wd, float bias1, float bias2,
                               const float* coef, const float* ok, int slot, unsigned epoch,
                               int ctas, int* status, void* stream);
/* Pull chunk r (chunk_bytes at offset_bytes + r*chunk_bytes) from every peer r. */
int sfl_allgather_bytes(const SflComm* comm, long offset_bytes, long chunk_bytes, int slot,
                        unsigned epoch, int ctas, int* status, void* stream);
/* dst[r*chunk_bytes ...] <- peer r's data[src_off_bytes .. +chunk_bytes) for every r;
 * dst is local memory (16-byte aligned). */
int sfl_allgather_into(const SflComm* comm, long src_off_bytes, long chunk_bytes, void* dst,
                       int slot, unsigned epoch, int ctas, int* status, void* stream);
/* data2[*][out_off] (fp32 [rows, cols]) <- resid + bf16(sum_r data[r][in_off] (bf16)). */
int sfl_reduce_rows_resid(const SflComm* comm, long in_off_bytes, long out_off_bytes,
                          const float* resid, long rows, int cols, int slot, unsigned epoch,
                          int ctas, int* status, void* stream);
/* data2[*][out_off] (bf16 [rows, cols]) <- bf16(sum_r data[r][in_off] (bf16)), fp32 sum. */
int sfl_reduce_rows_bf16(const SflComm* comm, long in_off_bytes, long out_off_bytes, long rows,
                         int cols, int slot, unsigned epoch, int ctas, int* status, void* stream);
/* data2[*][out_off] (fp32, count elements) <- sum_r data[r][in_off] (fp32). */
int sfl_allreduce_rows_f32(const SflComm* comm, long in_off_bytes, long out_off_bytes, long count,
                           int slot, unsigned epoch, int ctas, int* status, void* stream);

/* ------------------------------------ GEMM fused with its all-reduce (TP) -- */
/* Pointer tables of one tensor-parallel group; entry r belongs to rank r and is
 * a peer mapping (CUDA IPC) unless r == rank. */
typedef struct SflTpFuse {
  int rank, world;      /* 2 <= world <= 8                                            */
  void* stage[8];       /* staging for partial tiles (opaque layout of 4 KB blocks):  *
                         * sfl_gemm_tp_stage_bytes each                                */
  void* out[8];         /* result buffers                                             */
  void* tile_flags[8];  /* tile arrival words: sfl_gemm_tp_tile_flag_bytes, zeroed    */
  void* flags[8];       /* barrier flag buffers (sfl_comm_flag_bytes)                 */
} SflTpFuse;
long sfl_gemm_tp_stage_bytes(int M, int N, int world);
/* Diagnostics: six uint64 counters in device memory (NULL stops): nanoseconds, summed
 * over later calls, that CTA 0 spent until its first accumulator was ready, waiting
 * for the peers to enter, sending its strip, waiting for the peers' strips, and
 * finishing the rows; the sixth word counts the calls. */
int sfl_gemm_tp_set_trace(void* counters);
long sfl_gemm_tp_tile_flag_bytes(int M, int N);
/* Every rank of the group calls this with its own K-slice of the operands:
 *   partial[M, N] = a[M, K] (K-major, bf16) x b  (b: [N, K] K-major, or [K, N] when b_mn)
 * and, in the same kernel, out[*][out_off] <- resid + bf16(sum over ranks of
 * bf16(partial)) as fp32 [M, N] (out_bf16 = 0; resid is this rank's fp32 [M, N]
 * with pitch ldresid), or the bf16 sum without a residual (out_bf16 = 1).  N must
 * be a multiple of 256.  `slot`/`epoch` follow the communicator's barrier rules;
 * `tile_epoch` must grow by one with every call on every rank. */
int sfl_gemm_tp_reduce(const void* a, long lda, const void* b, long ldb, int b_mn, int M, int N,
                       int K, const SflTpFuse* tp, long out_off_bytes, int out_bf16,
                       const float* resid, long ldresid, int slot, unsigned epoch,
                       unsigned tile_epoch, int* status, void* stream);

/* ------------------------------------------------------------------ misc -- */
int sfl_cast_f32_to_bf16(const float* x, void* y_bf16, long n, void* stream);
int sfl_scale_f32(float* x, long n, const float* coef_dev, float scale, void* stream);
/* bf16 x *= *coef_dev; returns at once on the device when *coef_dev == 1. */
int sfl_scale_bf16_unless_one(void* x_bf16, long n, const float* coef_dev, void* stream);
/* out fp32 [rows, dim] = weight[ids[row]] */
int sfl_embedding_fwd(const float* weight, const int64_t* ids, float* out, int rows, int dim,
                      int vocab, void* stream);
/* dweight fp32 [vocab, dim] (+)= scatter-add of dx fp32 [rows, dim] by ids, added in row
 * order (deterministic).  next_scratch: rows ints, head_scratch: vocab ints.  rows is
 * limited by shared memory (51200); returns -2 beyond that. */
int sfl_embedding_bwd(const float* dx, const int64_t* ids, float* dweight, int rows, int dim,
                      int vocab, int accumulate, int* next_scratch, int* head_scratch,
                      void* stream);
/* Library build tag, for diagnostics. */
const char* sfl_version(void);
/* Writes sizeof(SflGemmEpilogue), sizeof(SflWgradProblem), sizeof(SflAttnTensor),
 * sizeof(SflAttnMask), sizeof(SflComm), sizeof(SflBlockArgs), sizeof(SflTpFuse) and returns how many
 * there are; bindings compare them with their own mirrors. */
int sfl_struct_sizes(int* sizes, int capacity);

/* ------------------------------------------------------ transformer block -- */
/* One pre-norm block (RMSNorm -> fused QKV + RoPE -> causal attention -> output
 * projection + residual -> RMSNorm -> SwiGLU -> down projection + residual) run
 * forward or backward by one call.  Weights are the bf16 copies, [out, in]
 * row-major, with q|k|v and w1|w3 stacked; norms, the residual stream, statistics
 * and parameter gradients are fp32.  `saved` (sfl_block_saved_bytes) carries the
 * activations from forward to backward; `scratch` (sfl_block_scratch_bytes) is
 * only used during backward.  Buffers need 256-byte alignment. */
typedef struct SflBlockArgs {
  int batch, seq_len, d_model, heads, head_dim, d_ff;
  float eps1, eps2, attn_scale;
  const void* wqkv;  /* [3 * heads * head_dim, d_model] */
  const void* wo;    /* [d_model, heads * head_dim]     */
  const void* w13;   /* [2 * d_ff, d_model]             */
  const void* w2;    /* [d_model, d_ff]                 */
  const float* norm1;
  const float* norm2;
  const float* rope_cos; /* [>= seq_len, head_dim / 2] */
  const float* rope_sin;
  const SflAttnMask* mask;
  const float* x; /* [batch * seq_len, d_model] */
  float* x_out;   /* forward only */
  void* saved;
  /* backward only */
  const float* d_out;
  const void* d_out_bf16; /* optional bf16 copy of d_out */
  float* dx;
  void* dx_bf16;
  void* scratch;
  float* g_wqkv;
  float* g_wo;
  float* g_w13;
  float* g_w2;
  float* g_norm1;
  float* g_norm2;
  int acc_wqkv, acc_wo, acc_w13, acc_w2, acc_norm1, acc_norm2; /* 1: add to the gradient */
  int* status;
  /* Tensor parallelism (NULL tp_pool: none).  heads and d_ff above are this rank's
   * share.  The output and down projections (forward) and the input gradients of
   * the qkv and w1|w3 projections (backward) then run as sfl_gemm_tp_reduce: the
   * forward results x_mid and x_out are written into every rank's fp32 pool
   * (tp_pool->out) at the byte offsets below, x_out is ignored, and the backward
   * sums land in every rank's bf16 buffer (tp_small->out).  Entry 0 / 1 of the
   * slot and epoch arrays serve the first / second fused product of the call. */
  const SflTpFuse* tp_pool;
  const SflTpFuse* tp_small;
  long tp_off_mid, tp_off_out;
  int tp_slot[2];
  unsigned tp_epoch[2];
  unsigned tp_tile_epoch[2];
} SflBlockArgs;

long sfl_block_saved_bytes(const SflBlockArgs* args);
long sfl_block_scratch_bytes(const SflBlockArgs* args);
int sfl_block_forward(const SflBlockArgs* args, void* stream);
int sfl_block_backward(const SflBlockArgs* args, void* stream);

#ifdef __cplusplus
}
#endif
