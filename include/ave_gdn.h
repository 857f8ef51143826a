/* C ABI of libave_gdn_b200.so: gated-delta-net (GDN) linear-attention kernels for NVIDIA B200 (sm_100a).
 *
 * The reference project (848267592/avelang) ships kernel libraries as Python functions in the
 * `avelang_kernels` namespace that take torch tensors, validate them, allocate the output unless `out=`
 * is given, launch on the current stream and never synchronise
 * (python/avelang_kernels/amdgpu_gemm.py:458-494).  Under that convention each kernel is reached through
 * a generated per-signature C launcher, `launch(gx,gy,gz,bx,by,bz,stream,func,*args)`
 * (python/avelang/backends/nvidia/driver.py:182-312), which pulls `data_ptr()` out of every tensor,
 * rejects host pointers and enqueues with cuLaunchKernel.  The entry points below take the place of that
 * launcher for the GDN path: plain device pointers, sizes and element strides in, one status code out.
 * The reference has no GDN kernels of its own; `ave_gemm_bf16_nt` is the only entry point with a direct
 * counterpart (gemm_pipeline_transposed_b, amdgpu_gemm.py:458-494).
 *
 * Conventions
 *  - Every pointer is a device pointer on the current CUDA device unless stated; the caller owns all
 *    buffers, including workspace.  No entry point allocates device memory or synchronises the device.
 *  - `stream` is a cudaStream_t passed as void*.  A call enqueues a fixed sequence of kernels on it.
 *  - Strides are in ELEMENTS.  The innermost (head-feature) dimension must be contiguous and every row
 *    16-byte aligned.
 *  - Return value: AVE_GDN_OK or an AveGdnStatus code.  Nothing aborts or throws across the boundary.
 *  - Thread safety: every entry point may be called from several host threads at once.  The prefill enqueues under a
 *    per-device mutex (its schedule forks onto library-owned helper streams through events, and the record/wait pairs
 *    of two callers must not interleave); a small pool of helper-stream sets per device, picked by the caller's stream,
 *    lets prefills on different streams overlap on the GPU.  Calls that overlap on the GPU need their own scratch and
 *    outputs.
 *  - Data-dependent faults (a slot index outside the pool, a bounded device wait that ran out) cannot be
 *    seen by the host without a sync: the kernels skip the offending unit and OR a bit into the optional
 *    device word `status` (see AVE_GDN_DEV_*).
 *  - Tensor roles: q,k [B,T,Hk,dk]; v,z,o [B,T,Hv,dv]; g (log decay, <= 0) and beta [B,T,Hv] fp32;
 *    value head h reads key head h / (Hv/Hk).  State tiles are fp32 [dk][dv], key-major:
 *    o_t = scale * M^T q_t,   M <- exp(g_t) M + k_t (beta_t (v_t - exp(g_t) M^T k_t))^T.
 */
#ifndef AVE_GDN_H_
#define AVE_GDN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AVE_GDN_ABI_VERSION 4

typedef enum AveGdnStatus {
  AVE_GDN_OK = 0,
  AVE_GDN_INVALID_ARGUMENT = 1, /* null pointer, negative size, struct_size mismatch */
  AVE_GDN_UNSUPPORTED = 2,      /* shape outside what the kernels are built for */
  AVE_GDN_MISALIGNED = 3,       /* pointer or stride breaks the 16-byte rule */
  AVE_GDN_CUDA_ERROR = 4,       /* see ave_gdn_last_cuda_error() */
  AVE_GDN_WORKSPACE_TOO_SMALL = 5
} AveGdnStatus;

/* bits OR-ed into the device status word */
#define AVE_GDN_DEV_BAD_SLOT 1u      /* state index >= num_slots: that sequence was skipped */
#define AVE_GDN_DEV_BAD_SEQLEN 2u    /* cu_seqlens not monotone inside [0, T]: the whole batch was skipped (its outputs are
                                        undefined); or a sequence longer than max_seqlen: that sequence was skipped like
                                        one with a negative slot (zero output, state untouched) */
#define AVE_GDN_DEV_WAIT_EXPIRED 4u  /* a bounded wait inside a kernel gave up */

/* flags */
#define AVE_GDN_FLAG_QK_L2NORM 1u    /* normalise q and k per head vector (eps 1e-6) inside the kernel */
#define AVE_GDN_FLAG_GATE_FIRST 2u   /* gated norm computes rmsnorm(o * silu(z)) instead of rmsnorm(o) * silu(z) */

/* One argument block for both recurrences (chunked prefill and token-by-token decode). */
typedef struct AveGdnArgs {
  uint32_t struct_size; /* sizeof(AveGdnArgs), checked */
  uint32_t flags;
  const void* q; /* bf16 */
  const void* k; /* bf16 */
  const void* v; /* bf16 */
  const float* g;
  const float* beta;
  const void* z;             /* bf16, optional: fuses the gated RMSNorm into the output */
  const float* norm_weight;  /* fp32 [dv], optional (unit weight when null) */
  void* o;                   /* bf16 */
  const float* initial_state; /* optional (zero state when null) */
  float* final_state;         /* optional (not written when null); may alias initial_state */
  const int32_t* cu_seqlens;    /* optional int32 [n_seqs+1]; requires B == 1 */
  const int32_t* state_indices; /* optional int32 [n_seqs]: sequence n uses state tile state_indices[n]
                                   of initial_state/final_state (negative: skip the sequence, o = 0) */
  uint32_t* status;           /* optional device status word */
  void* workspace;            /* device scratch, >= ave_gdn_prefill_workspace_bytes(); prefill only */
  uint64_t workspace_bytes;
  int32_t B, T, Hk, Hv, dk, dv;
  int32_t n_seqs;    /* B when cu_seqlens is null */
  int32_t num_slots; /* tiles in the state arrays; n_seqs when state_indices is null */
  int32_t chunk;     /* prefill: 64 */
  int32_t max_seqlen; /* optional, with cu_seqlens: an upper bound of the longest sequence in tokens (0 = unknown).  It
                         sizes the launch schedule of the prefill; a sequence longer than it is skipped (zero output,
                         state untouched) and flagged AVE_GDN_DEV_BAD_SEQLEN. */
  int64_t q_stride_b, q_stride_t, q_stride_h;
  int64_t k_stride_b, k_stride_t, k_stride_h;
  int64_t v_stride_b, v_stride_t, v_stride_h;
  int64_t z_stride_b, z_stride_t, z_stride_h;
  int64_t o_stride_b, o_stride_t, o_stride_h;
  int64_t g_stride_b, g_stride_t; /* g and beta share strides; head stride is 1 */
  float scale;
  float norm_eps;
  /* Optional fused all-gather of the output (prefill with z only): a device array of n_peers base pointers of buffers
   * laid out exactly like `o` (one per GPU of the node, peer-mapped, this GPU's own buffer included).  The gated-norm
   * stage then stores every output row into all of them with plain peer stores instead of into `o`; `o` still defines
   * the layout.  The caller orders the stores against the peers' readers (a barrier after the call). */
  const void* const* o_peers;
  int32_t n_peers;
  int32_t reserved1;
} AveGdnArgs;

/* Chunked prefill (chunk 64, WY/UT form), dense [B,T] or packed varlen via cu_seqlens. */
int ave_gdn_chunk_prefill(const AveGdnArgs* args, void* stream);
size_t ave_gdn_prefill_workspace_bytes(const AveGdnArgs* args);
/* Number of kernels one ave_gdn_chunk_prefill call with these arguments enqueues (a pure function of the shapes and of
 * which optional tensors are present; no device needed).  0 for invalid arguments. */
int ave_gdn_prefill_launch_count(const AveGdnArgs* args);

/* Same computation as ave_gdn_chunk_prefill for callers that may not allocate device memory (a serving runtime
 * that has handed all of HBM to its paged pools, a plug-in callback limited to pre-registered buffers, a path where
 * allocator calls are forbidden): `workspace` / `workspace_bytes` are ignored and the scratch is a fixed 64 MiB
 * array inside the library (AVE_GDN_NOALLOC_SCRATCH_BYTES), held by every GPU that loads the library until the
 * process exits.  Requests needing more scratch than that, i.e. more than about 1000 (chunk, value head) pairs without
 * a gate tensor z and about 670 with one (the un-normalised fp32 output then waits in the array too), return
 * AVE_GDN_WORKSPACE_TOO_SMALL; only dk = dv = 128 is served.  The call runs the plain schedule: one launch per pass on
 * the caller's stream, no helper streams or events.  Calls no cudaMalloc/cudaFree or other allocating routine.
 * The first call on a device looks up the array's device address and should be made outside stream capture.  All
 * calls share the one array: calls that overlap on the GPU (different streams) race; nothing needs clearing between
 * calls.  This entry point has no counterpart in the reference. */
#define AVE_GDN_NOALLOC_SCRATCH_BYTES ((size_t)64 << 20)
int ave_gdn_chunk_prefill_noalloc(const AveGdnArgs* args, void* stream);

/* Token-by-token recurrence with the state tile held on chip; T == 1 with state_indices is the
 * continuous-batching decode step (state streamed once in, once out, updated in place). */
int ave_gdn_decode_step(const AveGdnArgs* args, void* stream);

/* y = w * x * rsqrt(mean(x^2) + eps) * silu(z) over rows of `d` elements. */
typedef struct AveGdnNormArgs {
  uint32_t struct_size;
  uint32_t flags;        /* AVE_GDN_FLAG_GATE_FIRST */
  const void* x;         /* bf16 */
  const void* z;         /* bf16 */
  const float* weight;   /* fp32 [d], optional */
  void* y;               /* bf16 */
  int64_t rows;          /* number of (token, head) rows */
  int32_t d;             /* 64 or 128 */
  int32_t heads;         /* rows are indexed (token, head) = (r / heads, r % heads) */
  int64_t x_stride_t, x_stride_h, z_stride_t, z_stride_h, y_stride_t, y_stride_h;
  float eps;
  float reserved0;
} AveGdnNormArgs;
int ave_gdn_gated_rmsnorm(const AveGdnNormArgs* args, void* stream);

/* C[M,N] = A[M,K] * B[N,K]^T, bf16 in/out, fp32 accumulate: the operand convention of
 * gemm_pipeline_transposed_b (python/avelang_kernels/amdgpu_gemm.py:458-494). */
typedef struct AveGemmArgs {
  uint32_t struct_size;
  uint32_t flags;
  const void* a;
  const void* b;
  void* c;
  int64_t M, N, K;
  int64_t lda, ldb, ldc; /* row strides in elements, multiples of 8 */
  uint32_t* status;      /* optional device status word (AVE_GDN_DEV_WAIT_EXPIRED: tiles were abandoned, C is incomplete) */
} AveGemmArgs;
int ave_gemm_bf16_nt(const AveGemmArgs* args, void* stream);

/* Row-parallel linear layer with the cross-rank sum fused into the GEMM (the output projection of the tensor-parallel
 * block: each rank holds the K slice of its own heads; the reference convention for such a function is the
 * tensor-in/tensor-out GEMM of python/avelang_kernels/amdgpu_gemm.py:458-494, the sum replaces the all-reduce a caller
 * would add behind it).  Two calls with a cross-rank barrier between them and one after:
 *   ave_gemm_bf16_nt_scatter  C_partial = A * B^T; the GEMM's epilogue stores each row, as bf16, straight into slot
 *                             `rank` of the staging buffer of the rank that owns the row (rows_per_owner consecutive
 *                             rows per rank) -- plain peer stores, tile by tile, under the next tile's main loop;
 *   ave_gemm_reduce_push      the owner sums its rows over the n_ranks slots in fp32, in slot order, rounds once to
 *                             bf16 and stores them into every rank's result matrix [M][ldc].
 * stage_peers / out_peers: device arrays of n_ranks addresses (this rank's own included) of buffers every rank can
 * reach (peer-mapped or symmetric memory); each staging buffer holds n_ranks * rows_per_owner * N bf16.  N % 8 == 0. */
typedef struct AveGemmReduceArgs {
  uint32_t struct_size;
  uint32_t flags;
  const void* a;
  const void* b;
  int64_t M, N, K;
  int64_t lda, ldb;
  const void* const* stage_peers;
  void* stage;                   /* this rank's own staging buffer */
  const void* const* out_peers;
  int64_t ldc;                   /* row stride of the result matrices, elements, multiple of 8 */
  int32_t n_ranks, rank;
  int64_t rows_per_owner;        /* >= ceil(M / n_ranks) */
  uint32_t* status;
} AveGemmReduceArgs;
int ave_gemm_bf16_nt_scatter(const AveGemmReduceArgs* args, void* stream);
int ave_gemm_reduce_push(const AveGemmReduceArgs* args, void* stream);

/* Depthwise causal conv over time (kernel width 2..4) followed by SiLU, zero history at each sequence
 * start.  x,y [B,T,C] bf16, w [C,width] bf16, optional bias [C] bf16, optional cu_seqlens (B == 1). */
typedef struct AveConvArgs {
  uint32_t struct_size;
  uint32_t flags;
  const void* x;
  const void* w;
  const void* bias;
  void* y;
  const int32_t* cu_seqlens;
  int32_t B, T, C, width, n_seqs, reserved0;
  int64_t x_stride_b, x_stride_t, y_stride_b, y_stride_t;
} AveConvArgs;
int ave_gdn_conv1d_silu(const AveConvArgs* args, void* stream);

/* Single-token form of the same convolution for decode: per sequence n, the last width-1 inputs live in slot
 * state_indices[n] (or n) of a pool laid out [slots][width-1][C] bf16 (oldest first, channel-contiguous); the call
 * computes y[n] = silu(bias + w . [history, x[n]]) and shifts x[n] into the history in place.  Negative index: skip
 * (no status bit); index >= num_slots: skip and flag. */
typedef struct AveConvUpdateArgs {
  uint32_t struct_size;
  uint32_t flags;
  const void* x;              /* bf16 [n_seqs, C], row stride x_stride */
  const void* w;              /* bf16 [C, width] */
  const void* bias;           /* bf16 [C], optional */
  void* y;                    /* bf16 [n_seqs, C], row stride y_stride */
  void* conv_state;           /* bf16 [num_slots, width-1, C] */
  const int32_t* state_indices; /* optional int32 [n_seqs] */
  int32_t n_seqs, C, width, num_slots;
  int64_t x_stride, y_stride;
  uint32_t* status;           /* optional device status word: AVE_GDN_DEV_BAD_SLOT when an index is >= num_slots (that
                                 sequence is skipped: y[n] and its history are left untouched) */
} AveConvUpdateArgs;
int ave_gdn_conv1d_update(const AveConvUpdateArgs* args, void* stream);

/* One decode step of a whole GDN layer behind its in-projection, fused into one kernel: per sequence n the new token's
 * projection row proj[n] = [q | k | v | z | b | a] (Hk*dk | Hk*dk | Hv*dv | Hv*dv | Hv | Hv columns, bf16) goes through
 * the causal-conv update + SiLU on the q, k, v channels (history of slot state_indices[n] of conv_state shifted in
 * place), the L2 norm of q and k per head (eps 1e-6), g = -exp(A_log) softplus(a + dt_bias), beta = sigmoid(b), the
 * gated-delta-rule update of the fp32 state tiles of that slot of state_pool (in place) and the gated RMSNorm with z.
 * Same rounding points as ave_gdn_conv1d_update + ave_gdn_gate_beta + ave_gdn_decode_step run one after the other.
 * dk = dv = 128.  Negative slot: the sequence is skipped (o = 0, no state access); slot >= num_slots: skipped and
 * flagged AVE_GDN_DEV_BAD_SLOT.  The two pools share the slot index. */
typedef struct AveGdnDecodeLayerArgs {
  uint32_t struct_size;
  uint32_t flags;               /* AVE_GDN_FLAG_GATE_FIRST */
  const void* proj;             /* bf16 [n_seqs, proj_stride] */
  const void* conv_w;           /* bf16 [2*Hk*dk + Hv*dv, width], rows in q | k | v channel order */
  const void* conv_bias;        /* bf16 [2*Hk*dk + Hv*dv], optional */
  void* conv_state;             /* bf16 [num_slots, width-1, 2*Hk*dk + Hv*dv], oldest first */
  const float* A_log;           /* fp32 [Hv] */
  const float* dt_bias;         /* fp32 [Hv] */
  const float* norm_weight;     /* fp32 [dv], optional */
  float* state_pool;            /* fp32 [num_slots, Hv, dk, dv] */
  const int32_t* state_indices; /* optional int32 [n_seqs] */
  void* o;                      /* bf16 [n_seqs, o_stride]: Hv*dv normalised outputs per sequence */
  uint32_t* status;             /* optional device status word */
  int32_t n_seqs, Hk, Hv, dk, dv, width, num_slots, reserved0;
  int64_t proj_stride, o_stride; /* row strides in elements, multiples of 8 */
  float scale, norm_eps;
} AveGdnDecodeLayerArgs;
int ave_gdn_decode_layer_step(const AveGdnDecodeLayerArgs* args, void* stream);

/* Backward pass of the recurrence (dk = dv = 128; q and k as given, i.e. without the in-kernel L2 norm, and without the
 * fused gated norm: those two are differentiated by the caller's framework around this call).  Inputs as for the
 * forward pass plus d_o (bf16, laid out like v) and the optional gradient of the final states; outputs in fp32:
 * dq, dk [B,T,Hv,dk] PER VALUE HEAD (the caller sums the value heads that share a key head), dv [B,T,Hv,dv],
 * dg, dbeta [B,T,Hv], and optionally d_initial_state [n_seqs,Hv,dk,dv]; all contiguous.  Token-by-token reverse sweep
 * in fp32 with the state recomputed from 64-token checkpoints held in `workspace`. */
typedef struct AveGdnBwdArgs {
  uint32_t struct_size;
  uint32_t flags;
  const void* q;  /* bf16 */
  const void* k;  /* bf16 */
  const void* v;  /* bf16 */
  const float* g;
  const float* beta;
  const void* d_o;                /* bf16 [B,T,Hv,dv] */
  const float* initial_state;     /* optional fp32 [n_seqs,Hv,dk,dv] */
  const float* d_final_state;     /* optional fp32 [n_seqs,Hv,dk,dv] */
  const int32_t* cu_seqlens;      /* optional int32 [n_seqs+1]; requires B == 1 */
  float* d_q;                     /* fp32 [B,T,Hv,dk], per value head */
  float* d_k;                     /* fp32 [B,T,Hv,dk], per value head */
  float* d_v;                     /* fp32 [B,T,Hv,dv] */
  float* d_g;                     /* fp32 [B,T,Hv] */
  float* d_beta;                  /* fp32 [B,T,Hv] */
  float* d_initial_state;         /* optional */
  uint32_t* status;
  void* workspace;                /* >= ave_gdn_backward_workspace_bytes() */
  uint64_t workspace_bytes;
  int32_t B, T, Hk, Hv, dk, dv, n_seqs, reserved0;
  int64_t q_stride_b, q_stride_t, q_stride_h;
  int64_t k_stride_b, k_stride_t, k_stride_h;
  int64_t v_stride_b, v_stride_t, v_stride_h;
  int64_t do_stride_b, do_stride_t, do_stride_h;
  int64_t g_stride_b, g_stride_t;
  float scale;
  float reserved1;
} AveGdnBwdArgs;
int ave_gdn_recurrent_backward(const AveGdnBwdArgs* args, void* stream);
size_t ave_gdn_backward_workspace_bytes(const AveGdnBwdArgs* args);

/* g = -exp(A_log[h]) * softplus(a + dt_bias[h]),  beta = sigmoid(b);  a,b bf16 [rows,Hv] (strided),
 * A_log,dt_bias fp32 [Hv];  g,beta fp32 [rows,Hv] contiguous. */
typedef struct AveGateArgs {
  uint32_t struct_size;
  uint32_t flags;
  const void* a;
  const void* b;
  const float* A_log;
  const float* dt_bias;
  float* g;
  float* beta;
  int64_t rows;
  int32_t Hv, reserved0;
  int64_t a_stride_row, b_stride_row;
} AveGateArgs;
int ave_gdn_gate_beta(const AveGateArgs* args, void* stream);

int ave_gdn_abi_version(void);
const char* ave_gdn_status_string(int status);
/* cudaError_t of the most recent failing CUDA call made by this thread through the library (0 if none). */
int ave_gdn_last_cuda_error(void);

#ifdef __cplusplus
}
#endif
#endif /* AVE_GDN_H_ */
