/*
 * flb200 — B200 (sm_100a) attention-variant forward kernels, C ABI.
 *
 * This is the boundary a Flashlight maintainer binds in place of
 * `torch.compile(fn)` around the eager functions of `attention_variants/`:
 * one call computes what the compiled Triton kernel of that function computes
 * (softmax(mod(q k^T * scale) + mask) v in one pass), for
 *
 *   attention_pytorch / attention_pytorch_nogqa   attention_variants/vanilla.py:4-35
 *   attention_pytorch_causal                      attention_variants/causal.py:4-36
 *   attention_pytorch_alibi                       attention_variants/alibi.py:13-33
 *   attention_softcapped                          attention_variants/softcap.py:4-53
 *   attention_pytorch_sliding_window              attention_variants/sliding_window.py:14-44
 *   attention_pytorch_document_mask               attention_variants/document_mask.py:6-41
 *   attention_pytorch_prefix_lm                   attention_variants/prefix_lm.py:5-30
 *   diffattn                                      attention_variants/diff_attn.py:6-30
 *   attention_reference (Evoformer row attention) attention_variants/evoformer.py:8-36
 *
 * The reference has no FFI layer of its own; its kernels are generated at run
 * time (monkeypatch/fusion/reduction_kernel_fusion.py:952-998).  Everything
 * here is plain C: pointers, sizes, strides.  All tensor pointers are DEVICE
 * pointers to bf16 data; the caller owns every buffer (inputs, output,
 * workspace, status word).  The library allocates no device memory and keeps
 * no pointer after a call returns; the one exception is flb200_attn_fwd_noalloc,
 * which works in a static device array of the library and remembers that
 * array's address per device.  Functions never throw or abort: they return 0 or
 * a negative flb200_status.  Calls are thread-safe and may be issued
 * concurrently on different streams and devices; again flb200_attn_fwd_noalloc
 * is the exception (its calls on one device share the array and must not
 * overlap on the GPU, see below).
 */
#ifndef FLB200_ATTN_H_
#define FLB200_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLB200_ABI_VERSION 3u

/* Size of the library-owned scratch behind flb200_attn_fwd_noalloc. */
#define FLB200_NOALLOC_SCRATCH_BYTES (1u << 20)

typedef enum flb200_status {
  FLB200_OK = 0,
  FLB200_E_BAD_ARG = -1,      /* null pointer, non-positive size, bad enum, bad struct_size */
  FLB200_E_UNSUPPORTED = -2,  /* shape / combination no kernel is built for (no fallback exists) */
  FLB200_E_MISALIGNED = -3,   /* pointer not 16-byte aligned or stride not a multiple of 8 elements */
  FLB200_E_WORKSPACE = -4,    /* workspace missing or too small */
  FLB200_E_ARCH = -5,         /* device is not sm_100 */
  FLB200_E_LAUNCH = -6,       /* CUDA reported an error while encoding descriptors or launching */
  FLB200_E_TIMEOUT = -7       /* decoded from a status word: a device-side wait gave up */
} flb200_status;

/* Score modifier applied to s = q.k * scale before masking and softmax. */
typedef enum flb200_score_mod {
  FLB200_SCORE_NONE = 0,
  FLB200_SCORE_ALIBI = 1,   /* s + 2^(-8 (h+1) / alibi_heads) * (j - i)   alibi.py:5-9 */
  FLB200_SCORE_SOFTCAP = 2, /* softcap * tanh(s / softcap)                 softcap.py:46-49 */
  FLB200_SCORE_BIAS = 3     /* s + bias[0] + bias[1]                       evoformer.py:24-27 */
} flb200_score_mod;

/* Pointwise function between the two products of a product chain. */
typedef enum flb200_pointwise {
  FLB200_PW_IDENTITY = 0,
  FLB200_PW_RELU = 1,
  FLB200_PW_TANH = 2,
  FLB200_PW_SIGMOID = 3
} flb200_pointwise;

/* Mask; masked pairs get weight zero.  i = query index, j = key index. */
typedef enum flb200_mask {
  FLB200_MASK_NONE = 0,
  FLB200_MASK_CAUSAL = 1,   /* keep j <= i                                  causal.py:32-33 */
  FLB200_MASK_SLIDING = 2,  /* keep i - window <= j <= i (window + 1 keys)  sliding_window.py:8 */
  FLB200_MASK_PREFIX = 3,   /* keep j <= max(prefix_len[n] - 1, i)          prefix_lm.py:38-41 */
  FLB200_MASK_DOCUMENT = 4  /* keep doc[n][i] == doc[n][j]                  document_mask.py:25-27
                               and additionally j <= i when `causal` != 0 */
} flb200_mask;

/*
 * One attention forward problem.  Strides are in ELEMENTS; the innermost
 * (feature) axis of q, k, v, o and the key axis of a bias are contiguous.
 *
 *   q [N][Hq][L][E]   k [N][Hkv][S][E]   v [N][Hv][S][Ev]   o [N][Ho][L][Ev]
 *
 * Plain variants: Hv = Hkv, Ho = Hq, query head h reads kv head h / (Hq/Hkv).
 * Differential attention (`diff` != 0): Hq = Hkv = 2 * Ho, Hv = Ho; output
 * head h combines (q,k) heads h and h + Ho over v head h (diff_attn.py:14-29).
 * Evoformer layout [*, S, H, D] is expressed through the strides (row stride
 * H*D, head stride D), so no transposed copy is ever made.
 */
typedef struct flb200_attn_params {
  uint32_t struct_size; /* sizeof(flb200_attn_params), checked */
  int32_t diff;         /* 0 plain, 1 differential attention */
  int32_t N, Hq, Hkv, L, S, E, Ev;

  const void* q;
  const void* k;
  const void* v;
  void* o;
  int64_t q_stride[3]; /* batch, head, row */
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];

  float scale; /* > 0; the reference default is 1/sqrt(E) */

  int32_t score_mod;   /* flb200_score_mod */
  int32_t alibi_heads; /* ALIBI: number of heads in the slope formula */
  float softcap;       /* SOFTCAP: cap > 0 */
  /* BIAS: up to two additive bf16 tensors addressed as
   *   bias[b][r][h][i][j],  n = b * bias_inner + r  (bias_inner >= 1)
   * with element strides {b, r, h, i}; a stride of 0 broadcasts.  NULL = absent.
   * -inf entries act as a key mask.  Biases need no alignment beyond their element
   * size; rows that start on 16-byte boundaries are read faster. */
  const void* bias[2];
  int64_t bias_stride[2][4];
  int32_t bias_inner;

  int32_t mask;                /* flb200_mask */
  int32_t causal;              /* DOCUMENT only: compose with j <= i */
  int32_t window;              /* SLIDING */
  const int32_t* prefix_len;   /* PREFIX: device int32[N], or NULL to use prefix_scalar */
  int32_t prefix_scalar;
  const int64_t* document_id;  /* DOCUMENT: device int64 [N][L], row stride doc_stride_n */
  int64_t doc_stride_n;

  float diff_lambda;    /* out = A1 V - lambda * A2 V */
  int32_t diff_rms_norm;/* then x * rsqrt(mean(x^2 over Ev) + eps) per output head */
  float diff_rms_eps;

  /* DOCUMENT needs flb200_attn_workspace_bytes() bytes of device scratch for the
   * block map.  With block_map_ready == 0, flb200_attn_fwd builds the map on the
   * same stream first; a caller that reuses document_id across calls builds it
   * once with flb200_build_block_map and passes block_map_ready = 1.
   * SCORE_BIAS: optional.  When one bias is a pair bias shared by bias_inner >= 4 rows and the other a
   * key vector per row, heads are narrow and flb200_attn_workspace_bytes() bytes (16-byte aligned) are
   * given, a small kernel lays the key vector out there and the tensor cores add it to the scores;
   * with workspace == NULL the same result comes from the softmax threads, more slowly.
   * diff with diff_rms_norm and value heads up to 128: optional too.  Given flb200_attn_workspace_bytes()
   * bytes, a small kernel finds max |v|, the forward kernel rewrites each V tile in shared memory as fp16
   * times the power of two that centres V's range (the normalisation cancels it, eps is scaled alike) and
   * P.V runs in fp16; without scratch P goes as two bf16 terms (same tolerance, 25 % slower). */
  void* workspace;
  size_t workspace_bytes;
  int32_t block_map_ready;

  /* Optional device int32, zeroed by the caller.  Non-zero after the stream
   * synchronises means a bounded device-side wait expired (see
   * flb200_decode_status); outputs are then undefined.  The word is sticky: while it is non-zero
   * every CTA of every later launch that is given the same word ends at once, so that a broken
   * launch drains quickly; the caller clears it after reading it. */
  int32_t* status;

  /* Optional output for a later backward pass (the reference stubs its backward,
   * benchmarks/_utils.py:16-21): device fp32 [N][Hq][L], row axis contiguous, element strides
   * {batch, head}.  Receives the natural-log sum over the unmasked keys of exp(modified score),
   * -inf for a row without a visible key.  NULL = not wanted.  Not available with `diff`. */
  float* lse;
  int64_t lse_stride[2];

  /* Limit of every device-side wait in microseconds; 0 = the default of two seconds.  A wait
   * that runs out ends the launch early through the kernels' common exit (tensor memory freed,
   * status word written); nothing traps or spins without bound. */
  uint32_t wait_limit_us;

  /* Optional second home of the status word: a device-accessible pointer to pinned (mapped) HOST
   * memory, zeroed by the caller.  A CTA that gives up stores the status word here as well, so
   * host code can notice a failed launch by reading host memory, without synchronising.  NULL =
   * not wanted. */
  int32_t* status_host;

  /* ALIBI: index of this call's first query head within the alibi_heads heads of the slope
   * formula (head h of the call uses slope index alibi_head0 + h).  0 unless the heads of one
   * model are split over several calls. */
  int32_t alibi_head0;

  /* Back-to-back matrix product without softmax (monkeypatch/template/fused_bmm.py:332-422 of the
   * reference: `(f(A @ B)) @ C` with a pointwise middle).  With product_chain != 0 the call
   * computes o = f(q k^T * scale) v:  A = q [N][H][M=L][N=E], C = v [N][H][O=S][P=Ev], and B is k,
   * either as rows of features [N][H][S][E] (k_keys_contiguous = 0) or, as the reference's B
   * operand lies in memory, [N][H][E][S] with the keys contiguous (k_keys_contiguous = 1; k_stride
   * is then {batch, head, feature row}).  score_mod and mask must be NONE, diff 0, lse NULL. */
  int32_t product_chain;
  int32_t pointwise;          /* flb200_pointwise */
  int32_t k_keys_contiguous;
} flb200_attn_params;

/* ABI version of the loaded library (FLB200_ABI_VERSION it was built with). */
uint32_t flb200_abi_version(void);

/* Static, human-readable text for a flb200_status. */
const char* flb200_strerror(int status);

/* Host-only check of a problem description: no CUDA call is made. */
int flb200_attn_validate(const flb200_attn_params* p);

/* Device scratch bytes flb200_attn_fwd takes for `p`: required for mask == DOCUMENT, optional for
 * SCORE_BIAS and for RMS-normalised differential attention (see `workspace`), 0 otherwise.  Returns 0 for a NULL or invalid description. */
size_t flb200_attn_workspace_bytes(const flb200_attn_params* p);

/* Build the document-mask block map into p->workspace on `cuda_stream`. */
int flb200_build_block_map(const flb200_attn_params* p, void* cuda_stream);

/* Enqueue the forward pass on `cuda_stream` (a cudaStream_t; NULL = default
 * stream).  Replaces one call of the torch.compile'd variant function. */
int flb200_attn_fwd(const flb200_attn_params* p, void* cuda_stream);

/*
 * Forward pass for callers that cannot allocate device memory.  (No counterpart in the
 * reference, whose runtime is PyTorch's allocator throughout.)
 *
 * A document-mask forward needs scratch for its block map, and flb200_attn_fwd expects the
 * caller to bring it.  Some callers have nothing to bring: plugins that are handed only
 * input and output buffers by their host framework and may not allocate, or tight
 * real-time loops where cudaMalloc's implicit device synchronisation is not acceptable.
 * For them this entry point keeps the block map in a fixed array of
 * FLB200_NOALLOC_SCRATCH_BYTES inside the library (every device that loads the library
 * holds that array until the process exits).  `workspace`, `workspace_bytes` and
 * `block_map_ready` are ignored; everything else is as in flb200_attn_fwd, and the results
 * are identical.  It performs no cudaMalloc/cudaFree and calls no allocating routine.
 *
 *  - A problem whose block map exceeds the array is rejected with FLB200_E_WORKSPACE
 *    (the map needs about N * (ceil(L/128) * (8 + ceil(L/128)) + 8 L) bytes); nothing is launched.
 *  - The first call on a device looks up the array's device address (a one-time set-up
 *    with that device current); that first call should come before any stream capture.
 *  - All calls on a device share the one array and the map is rebuilt on every call.  Two
 *    calls whose kernels can overlap on the GPU (different streams without ordering) race on
 *    it; keep such calls on one stream or order them with events.
 *  - Masks other than DOCUMENT need no scratch and are forwarded with the workspace fields cleared (the
 *    paths that use optional scratch stay off).
 */
int flb200_attn_fwd_noalloc(const flb200_attn_params* p, void* cuda_stream);

/*
 * Self-test of the bounded device-side waits.  Launches the forward kernel of `p` with its
 * loads withheld, so that every role's first wait runs into p->wait_limit_us (0 = 1000 us
 * here) and the CTAs leave through the common exit: tensor memory is freed, p->status (required)
 * receives the timeout code, the output is left untouched, the context stays usable.  Returns
 * FLB200_OK when the launch was enqueued; the caller then synchronises and decodes p->status,
 * which must read FLB200_E_TIMEOUT.  No counterpart in the reference.
 */
int flb200_selftest_wait_timeout(const flb200_attn_params* p, void* cuda_stream);

/*
 * Backward pass of plain and causal attention (with grouped query heads): dq, dk, dv from the
 * forward's inputs, its output `o`, its log-sum-exp `lse` (flb200_attn_params.lse of the forward call)
 * and the output's gradient `dout`.  The reference stubs its backward (benchmarks/_utils.py:16-21), so
 * there is no reference kernel to cite; the arithmetic is the derivative of
 * attention_variants/vanilla.py:4-35 and causal.py:4-36:
 *   P = exp(q k^T * scale - lse), dV = P^T dO, dP = dO V^T, dS = P (dP - rowsum(dO o)) * scale,
 *   dQ = dS K, dK = dS^T Q   (sums over the query heads of a group for dK, dV).
 * All tensors bf16 with the layouts and stride conventions of the forward's parameter block: q, o,
 * dout, dq are [N][Hq][L][E]; k, v, dk, dv are [N][Hkv][S][E]; head dims up to 128, the same for q/k
 * and v.
 * `workspace`: flb200_attn_bwd_workspace_bytes() bytes of device scratch (per query row the fp32 row
 * sum and two 32-byte rows for the dK/dV kernel), 256-byte aligned.  Three launches on `cuda_stream`.
 */
typedef struct flb200_attn_bwd_params {
  uint32_t struct_size;
  int32_t N, Hq, Hkv, L, S, E;
  const void* q;
  const void* k;
  const void* v;
  const void* o;
  const void* dout;
  const float* lse;       /* [N][Hq][L] natural log, element strides {batch, head} */
  void* dq;
  void* dk;
  void* dv;
  int64_t q_stride[3], k_stride[3], v_stride[3], o_stride[3], do_stride[3];
  int64_t dq_stride[3], dk_stride[3], dv_stride[3];
  int64_t lse_stride[2];
  float scale;
  int32_t causal;         /* 0: no mask, 1: keep j <= i */
  void* workspace;
  size_t workspace_bytes;
  int32_t* status;        /* as in flb200_attn_params */
  int32_t* status_host;
  uint32_t wait_limit_us;
} flb200_attn_bwd_params;

size_t flb200_attn_bwd_workspace_bytes(const flb200_attn_bwd_params* p);
int flb200_attn_bwd(const flb200_attn_bwd_params* p, void* cuda_stream);

/* Self-test of the backward kernels' bounded waits, like flb200_selftest_wait_timeout: the kernels of `p`
 * run with their loads withheld, every role's first wait runs into p->wait_limit_us (0 = 1000 us here),
 * the CTAs leave through the common exit, p->status (required) receives the timeout code, dq / dk / dv
 * are left untouched (the workspace is written).  No counterpart in the reference. */
int flb200_selftest_bwd_wait_timeout(const flb200_attn_bwd_params* p, void* cuda_stream);

/* Map the value read back from a status word to a flb200_status
 * (0 -> FLB200_OK, timeout code -> FLB200_E_TIMEOUT).  If `barrier` / `block`
 * are non-NULL they receive which wait expired and the low 16 bits of the index of the thread
 * block that gave up first. */
int flb200_decode_status(int32_t status_word, int32_t* barrier, int32_t* block);

/* Operands of invariant point attention for flb200_attn_fwd (the reference states the operator in
 * tests/test_ipa.py:57-125; it has no kernel or binding of its own).  The logits
 *   q.k / sqrt(c_hidden) + w sum_p |q_p - k_p|^2 + pair_bias
 * equal, up to a term constant along each row, (q'.k') / sqrt(c_hidden) + pair_bias with
 *   q' = [ q | q_p | q_p | 1 | 1 | 0.. ],  k' = [ k | hi(-2a k_p) | lo(-2a k_p) | hi(a |k_p|^2) | lo(a |k_p|^2) | 0.. ],
 * a = w sqrt(c_hidden), hi + lo the two-term bf16 split of an fp32 value, and the values are v' = [ v | v_p | 0.. ].
 * One launch writes the three operands; the caller then runs flb200_attn_fwd on them with
 * score_mod = BIAS, bias[0] = pair_bias and scale = 1 / sqrt(c_hidden).
 * All inputs bf16 and dense: scalars [rows][C], points [rows][P][point_dim]; outputs [rows][E] / [rows_k][Ev]
 * with E >= C + 2 P_qk point_dim + 2 and Ev >= C + P_v point_dim, both multiples of 8, 16-byte aligned. */
typedef struct flb200_ipa_pack_params {
  uint32_t struct_size;
  int32_t rows_q, rows_k;       /* B * H * N query rows; B * H * N_k key / value rows */
  int32_t C, P_qk, P_v, point_dim;
  const void* q_scalar;
  const void* k_scalar;
  const void* v_scalar;
  const void* q_points;
  const void* k_points;
  const void* v_points;
  float a;                      /* w * sqrt(c_hidden), w = -0.5 sqrt(9 / (2 P_qk)) in the reference */
  int32_t E, Ev;                /* row widths of the outputs */
  void* q_aug;
  void* k_aug;
  void* v_aug;
} flb200_ipa_pack_params;
int flb200_ipa_pack(const flb200_ipa_pack_params* p, void* cuda_stream);

/* Number of kernels this library has launched since it was loaded (attention
 * and block-map kernels; for accounting in benchmarks). */
uint64_t flb200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* FLB200_ATTN_H_ */
