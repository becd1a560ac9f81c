/*
 * qfg.h - C ABI of the B200 (sm_100a) implementation of the `qwen.fused_gemm` decode path.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, enqueues work on the
 * CUDA stream it is given and returns a status code; none synchronises, and none of the
 * *_compute / qfg_argmax_rows calls allocates, copies to the host or calls back, so they can
 * be captured in a CUDA graph.  Device pointers are raw `void*`; a stream is the
 * `cudaStream_t` value passed as `void*` (NULL = the legacy default stream).
 *
 * The entry points are the operator interface of the reference library
 * libqwen_fused_gemm_r5.so with the ONNX Runtime types peeled off: a *_create call takes what
 * the reference reads from node attributes at kernel creation, a *_compute call takes what
 * the reference reads from its OrtKernelContext.  Each declaration cites the reference
 * interface it replaces (paths inside the reference project).  The ORT shim
 * (qwen38_flash_ops_b200/csrc/ort_shim/fused_gemm_ort.cc) maps `RegisterCustomOps`,
 * domain `qwen.fused_gemm`, onto these calls one to one.
 *
 * Element types use the ONNX TensorProto codes the reference switches on.
 */
#ifndef QFG_H_
#define QFG_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define QFG_API __attribute__((visibility("default")))
#else
#define QFG_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define QFG_MAX_WEIGHTS 4 /* skinny::kMaxSeg, src/fused_gemm/skinny_gemm.cuh:41 */
#define QFG_MAX_OUTPUTS 8 /* skinny::kMaxOut, src/fused_gemm/skinny_gemm.cuh:39 */

/* Status codes; the values of OK / FAIL / INVALID_ARGUMENT equal OrtErrorCode's, which is what
 * the reference returns through OrtStatus (src/fused_gemm/fused_gemm.cu:589-591, :836-838). */
typedef enum qfg_status {
  QFG_OK = 0,
  QFG_FAIL = 1,             /* a CUDA call failed; qfg_last_error() holds "<Op>: <cuda string>" */
  QFG_INVALID_ARGUMENT = 2, /* bad attributes, shapes or element types; nothing was launched */
  QFG_NOT_IMPLEMENTED = 9
} qfg_status;

/* ONNX tensor element types accepted on this path. */
typedef enum qfg_dtype {
  QFG_FLOAT = 1,
  QFG_UINT8 = 2,        /* block-16 NVFP4, [K, N * 9 / 16] */
  QFG_INT64 = 7,
  QFG_FLOAT16 = 10,
  QFG_BFLOAT16 = 16,
  QFG_FLOAT8E4M3FN = 17 /* [K, N] with an optional per-column scale */
} qfg_dtype;

/* A 2-D weight tensor as the op receives it: `cols` is the stored width (N for BF16 / FP8,
 * N * 9 / 16 for NVFP4), exactly the shape ORT reports for the input. */
typedef struct qfg_tensor2d {
  const void* data; /* device pointer, row-major */
  int32_t dtype;    /* qfg_dtype */
  int64_t rows;     /* K */
  int64_t cols;
} qfg_tensor2d;

typedef struct qfg_skinny_gemm qfg_skinny_gemm;
typedef struct qfg_dequant qfg_dequant;
typedef struct qfg_untile_hc qfg_untile_hc;
typedef struct qfg_shared_expert_down qfg_shared_expert_down;
typedef struct qfg_lmhead qfg_lmhead;

/* Message of the last non-OK status returned on the calling thread ("" if none). */
QFG_API const char* qfg_last_error(void);
/* "qfg-b200 <version> sm_100a". */
QFG_API const char* qfg_version(void);

/* ---------------------------------------------------------------- SkinnyGemm
 * y_j[..., width_j] = x[..., K] @ W_i[K, N_i] column-sliced over the outputs of weight i.
 *
 * Replaces SkinnyGemmKernelState's constructor (src/fused_gemm/fused_gemm.cu:476-501; the
 * op schema is SkinnyGemmOp, :818-840).  Attributes: `seg_outs` (number of outputs slicing
 * each weight), `widths` (output widths in order), optional `w_scale` (host floats, the
 * concatenated per-column scales of the quantised weights, uploaded once here), optional
 * `trigger` (0 off, 1 = release programmatic-dependent-launch dependents at kernel start,
 * 2 = after the K loop; a non-zero value is overridden by the environment variable
 * SKINNY_TRIGGER_FORCE as in the reference, :105-113).  Fails with QFG_INVALID_ARGUMENT
 * unless 1 <= n_seg <= 4 and sum(seg_outs) == n_widths <= 8. */
QFG_API int qfg_skinny_gemm_create(const int64_t* seg_outs, int n_seg, const int64_t* widths, int n_widths,
                           const float* w_scale, size_t n_w_scale, int trigger, qfg_skinny_gemm** out);

/* Replaces SkinnyGemmKernelState::ComputeV2 (src/fused_gemm/fused_gemm.cu:507-592) for every
 * row count: `m` = product of x's leading dims, `k` = its last dim, x is BF16 [m, k];
 * `weights[i]` are the variadic weight inputs; `outs[j]` are caller-allocated BF16 [m, width_j]
 * buffers (ORT allocates them through GetOutput in the reference).  The same checks apply:
 * weight rows == k, widths add up to N, N % 4 == 0, k even, NVFP4 stored width == N * 9 / 16.
 * Stricter than the reference where it misreads memory: weights of one call must share one
 * element type, a BF16/FP8 weight must be 4-byte aligned per row and an NVFP4 weight needs
 * N % 64 == 0.  Rows are processed eight at a time, so any m >= 1 is accepted; row r of an
 * m-row call is computed with the arithmetic of the one-row call on that row.
 *
 * Prefill-shaped calls: with more rows than the "dense_rows" option (unless set: 8 for BF16 and FP8,
 * 16 for NVFP4 weights, where the branch starts to win on a B200; 0 switches it off) and every width a multiple of 8, the call dequantises the weights to BF16 in column
 * tiles (w_scale folded in before the rounding) and runs cublasGemmEx with FP32 accumulation, as
 * the reference does for M > 8 (fused_gemm.cu:365-428, dispatch at :578-583).  Like the
 * reference's, this branch allocates a handle and a buffer on first use, is not graph-capturable,
 * ignores `trigger`, and its accumulation order is the library's; cuBLAS is loaded at run time. */
QFG_API int qfg_skinny_gemm_compute(const qfg_skinny_gemm* op, const void* x, int64_t m, int64_t k,
                            const qfg_tensor2d* weights, int n_weights, void* const* outs, int n_outs,
                            void* stream);

/* Launch options that are not node attributes.  "pdl_wait" = 1 launches the kernel with the
 * programmatic-stream-serialisation attribute and makes it wait for its predecessor
 * (griddepcontrol.wait) only after its first weight tiles are in flight.  "plan" pins the
 * launch geometry ("wn=4,wk=2,ks=1,stages=4,cluster=8,ctas=296"); used by the tuning sweeps.
 * "dense_rows" moves or disables (0) the row count above which the prefill branch is taken. */
QFG_API int qfg_skinny_gemm_set_option(qfg_skinny_gemm* op, const char* key, const char* value);

/* Writes a one-line description of the launch plan chosen for these shapes into buf. */
QFG_API int qfg_skinny_gemm_describe(const qfg_skinny_gemm* op, int64_t k, const qfg_tensor2d* weights, int n_weights,
                             char* buf, size_t buf_len);

/* Diagnostic, needs no device: the launch plan for `nseg` weights of `n[i]` columns, element
 * type `dtype`, K rows, rows aligned to `row_align` (16, 8 or 4) bytes, on a GPU with `sm_count`
 * SMs; `spec` (may be NULL) is a "plan" override as above.  No counterpart in the reference, whose
 * planner is the table at src/fused_gemm/fused_gemm.cu:125-175. */
QFG_API int qfg_plan_describe(int dtype, int64_t k, const int64_t* n, int nseg, int row_align, int sm_count,
                              const char* spec, char* buf, size_t buf_len);

/* Replaces ~SkinnyGemmKernelState (src/fused_gemm/fused_gemm.cu:503-505): frees the uploaded scales. */
QFG_API void qfg_skinny_gemm_destroy(qfg_skinny_gemm* op);

/* ---------------------------------------------------------------- ArgmaxRows
 * idx[r] = argmax_v x[r, v] with numpy semantics (lowest index on ties, the first NaN wins,
 * -0 == +0); `val` (may be NULL) receives the maximum as FP32.
 * Replaces ArgmaxRowsKernelState::ComputeV2 (src/fused_gemm/fused_gemm.cu:735-778) and
 * skinny::LaunchArgmaxRows (src/fused_gemm/argmax_rows.cuh:192-204).  dtype is BFLOAT16,
 * FLOAT16 or FLOAT; rows == 0 is a no-op; vocab must be in [1, INT_MAX). */
QFG_API int qfg_argmax_rows(int dtype, const void* x, int64_t rows, int64_t vocab, int64_t* idx, float* val,
                    void* stream);

/* ---------------------------------------------------------------- DequantWeightBf16
 * Replaces DequantWeightBf16KernelState's constructor (src/fused_gemm/fused_gemm.cu:850-884):
 * attributes `n_cols` (required, multiple of 8), `col_offset` (default 0, multiple of 8),
 * `widths` (default [n_cols]; positive multiples of 8 that add up to n_cols, at most 8),
 * optional `w_scale` indexed by output column. */
QFG_API int qfg_dequant_create(int64_t n_cols, int64_t col_offset, const int64_t* widths, int n_widths,
                       const float* w_scale, size_t n_w_scale, qfg_dequant** out);

/* Replaces DequantWeightBf16KernelState::ComputeV2 (src/fused_gemm/fused_gemm.cu:890-953):
 * outs[i] is BF16 [w.rows, widths[i]].  BF16: column-slice copy; FP8: bf16(float(q) * s[col]);
 * NVFP4: bf16(e2m1 * e4m3_block_scale * s[col]). */
QFG_API int qfg_dequant_compute(const qfg_dequant* op, const qfg_tensor2d* w, void* const* outs, int n_outs,
                        void* stream);
QFG_API void qfg_dequant_destroy(qfg_dequant* op);

/* ---------------------------------------------------------------- SharedExpertDown
 * y[m, :] = routed[m, :] + bf16( bf16( swish_mul(g, u)[m, :] @ W ) * bf16( sigmoid( bf16( dot(gx[m, :], gw) ) ) ) )
 * with swish_mul(g, u) = bf16( bf16( g * bf16(sigmoid(g)) ) * u ), FP32 accumulation in the product and
 * `w_scale[n]` applied to the FP32 sum before the first rounding.  Replaces
 * SharedExpertDownKernelState (src/fused_gemm/fused_gemm.cu:595-727; arithmetic:
 * src/fused_gemm/skinny_gemm.cuh:73-80, 226-240, 302-327, 494-505, src/common/sigmoid_acc.cuh:12-21).
 * Attributes: optional `w_scale` (per column of the quantised weight), `trigger` as for SkinnyGemm.
 * g, u: BF16 [m, k]; weight [k, n] BF16 / FP8 E4M3FN, or UINT8 [k, 9n/16] NVFP4; gx: BF16 [m, gk];
 * gw: BF16 [gk]; routed: BF16 [m, n] (NULL: y is the shared term alone); out: BF16 [m, n].
 * n % 8 == 0 (NVFP4: n % 64 == 0 as for SkinnyGemm), gk even, any m >= 1 (the reference sends m > 4 to a
 * dense prefill kernel; here rows are processed eight at a time) and any k (the reference: k <= 1024).
 * The deferred-merge hook of the reference (QMoESharedExpertBridge, :34-92, :704-718) belongs to an
 * ORT-internal peer and is not reproduced. */
QFG_API int qfg_shared_expert_down_create(const float* w_scale, size_t n_w_scale, int trigger,
                                          qfg_shared_expert_down** out);
QFG_API int qfg_shared_expert_down_compute(const qfg_shared_expert_down* op, const void* g, const void* u, int64_t m,
                                           int64_t k, const qfg_tensor2d* weight, const void* gx, int64_t gk,
                                           const void* gw, const void* routed, int64_t n, void* out, void* stream);
/* The launch options of qfg_skinny_gemm_set_option ("plan", "pdl_wait", ...) for this node. */
QFG_API int qfg_shared_expert_down_set_option(qfg_shared_expert_down* op, const char* key, const char* value);
QFG_API void qfg_shared_expert_down_destroy(qfg_shared_expert_down* op);

/* ---------------------------------------------------------------- UntileHcBf16
 * Replaces UntileHcBf16KernelState (src/fused_gemm/fused_gemm.cu:1013-1072): attribute `kind`
 * (0: output [10240, 320], 1: output [320, 10240]) and optional `w_scale` indexed by output column.
 * The input is the pre-tiled [160, 20480] tensor, BFLOAT16 (pure permutation) or FLOAT8E4M3FN
 * (dequantised: bf16(float(q) * w_scale[col]), 1 if no scale); any other shape or type is refused. */
QFG_API int qfg_untile_hc_create(int kind, const float* w_scale, size_t n_w_scale, qfg_untile_hc** out);
QFG_API int qfg_untile_hc_compute(const qfg_untile_hc* op, const qfg_tensor2d* w, void* out, void* stream);
QFG_API void qfg_untile_hc_destroy(qfg_untile_hc* op);

/* ---------------------------------------------------------------- fused LM head
 * SkinnyGemm over one weight followed by ArgmaxRows over the BF16-rounded logits, in one
 * kernel: the logits are never written unless `logits` is non-NULL.  The reference runs the
 * two ops back to back (SkinnyGemmOp then ArgmaxRowsOp, src/fused_gemm/fused_gemm.cu:781-840);
 * this call returns what that chain returns.
 *
 * `col_offset` is added to every index, so a rank holding columns [c0, c1) of a sharded
 * vocabulary reports global indices.  `key` (may be NULL) receives per row a 64-bit word that
 * orders (value, index) pairs exactly like ArgmaxRows does - larger is better - which is the
 * payload the N-sharded LM head all-gathers; qfg_lmhead_combine folds the gathered words.
 *
 * `workspace` is qfg_lmhead_workspace_bytes() bytes of device memory (about 512 KB: 256 bytes of
 * keys and a counter, then room for the FP32 partial sums of column groups that the CTAs share
 * when the vocabulary does not divide evenly among them).  Its first 256 bytes must be zero
 * before the first call; each call leaves them zero again.  Calls that share a workspace must
 * not overlap on the GPU. */
QFG_API size_t qfg_lmhead_workspace_bytes(void);
QFG_API int qfg_lmhead_create(const float* w_scale, size_t n_w_scale, int trigger, qfg_lmhead** out);
QFG_API int qfg_lmhead_compute(const qfg_lmhead* op, const void* x, int64_t m, int64_t k, const qfg_tensor2d* weight,
                       int64_t n, int64_t col_offset, void* workspace, int64_t* idx, float* val,
                       uint64_t* key, void* logits, void* stream);
/* qfg_lmhead_compute for callers that cannot provide device memory of their own: hosts that
 * forbid allocation once serving has started, or hooks that are handed nothing but their inputs
 * and outputs.  No counterpart in the reference (its ops never need scratch memory).  The keys
 * and the counter live in a 256-byte array built into the library, so: at most
 * qfg_lmhead_static_max_rows() (8) rows per call, larger m is refused with QFG_INVALID_ARGUMENT;
 * all calls on a GPU share the array, so calls that overlap on that GPU race (one stream is
 * safe); the first call on each GPU looks the array up and clears it synchronously and should
 * therefore precede any stream capture.  Nothing is allocated or freed by any call. */
QFG_API size_t qfg_lmhead_static_max_rows(void);
QFG_API int qfg_lmhead_compute_static(const qfg_lmhead* op, const void* x, int64_t m, int64_t k,
                                      const qfg_tensor2d* weight, int64_t n, int64_t col_offset, int64_t* idx,
                                      float* val, uint64_t* key, void* logits, void* stream);
QFG_API int qfg_lmhead_set_option(qfg_lmhead* op, const char* key, const char* value);
QFG_API void qfg_lmhead_destroy(qfg_lmhead* op);

/* The N-sharded LM head without a separate collective: every rank runs qfg_lmhead_compute_sharded on
 * its own columns; the last CTA of each rank stores its per-row keys straight into every rank's
 * exchange buffer (peer memory over NVLink), waits - bounded - until the keys of all ranks have
 * arrived in its own buffer, folds them and writes the same idx / val on every rank.  No counterpart
 * in the reference (single GPU).
 *
 * An exchange buffer is qfg_lmhead_exchange_bytes() bytes of zero-initialised device memory per rank that
 * every other rank can address (qfg_peer_alloc / qfg_peer_open below, or any peer-mapped memory).
 * `peers[r]` is this process's address of rank r's buffer, `peers[rank]` its own.  All ranks must make
 * the same sequence of calls.  If a peer's keys do not arrive within the wait limit the call still
 * returns (the result then lacks that peer) and qfg_lmhead_exchange_status reports 1; qfg_lmhead_host_run
 * returns QFG_FAIL for such a step. */
#define QFG_MAX_RANKS 8
typedef struct qfg_lmhead_exchange {
  int world;
  int rank;
  void* peers[QFG_MAX_RANKS];
} qfg_lmhead_exchange;
QFG_API size_t qfg_lmhead_exchange_bytes(void);
QFG_API int qfg_lmhead_compute_sharded(const qfg_lmhead* op, const void* x, int64_t m, int64_t k,
                                       const qfg_tensor2d* weight, int64_t n, int64_t col_offset, void* workspace,
                                       const qfg_lmhead_exchange* exchange, int64_t* idx, float* val, void* logits,
                                       void* stream);
/* 0 = every wait so far completed, 1 = a wait ran out.  Synchronises the device.  The wait limit is the
 * option "exchange_spin" of qfg_lmhead_set_option (polling iterations of about 50 ns; default 4194304). */
QFG_API int qfg_lmhead_exchange_status(const void* own_buffer, int* status);
/* Device timer (ns) of the owner's last sharded call at three points of the exchange: own keys ready, stores
 * to all peers issued, words of all ranks seen (or given up on).  Differences separate the cost of the stores
 * from the wait for the slowest rank.  Synchronises the device.  No counterpart in the reference. */
QFG_API int qfg_lmhead_exchange_times(const void* own_buffer, uint64_t out[3]);

/* The LM head for a caller whose activations and results live in host memory (the reference's callers
 * hand ORT host tensors for the sampled token; no counterpart in the reference library itself).
 * qfg_lmhead_host_create records, once, a CUDA graph of two kernels on a stream of its own: the copy of
 * `x_host` (pinned, device-addressable, BF16 [m, k]) to `x_dev`, and the fused kernel as its programmatic
 * dependent (it streams its first weight tiles while x crosses the host link), which stores the winners
 * straight into `idx_host` / `val_host` (pinned, device-addressable; val_host may be null).  qfg_lmhead_host_run
 * launches the graph and returns as soon as the results are in idx_host / val_host: it marks those words
 * with values the kernel never stores and reads them until all have changed (bounded; past 20 ms, or on an
 * error, it synchronises the stream instead), so the call does not pay for the stream to drain and the
 * synchronising thread to be woken.  One call per decode step; the private stream may still be finishing
 * when the call returns, which the next call and qfg_lmhead_host_destroy order themselves after.  `exchange` is null on one GPU, or the peer-memory exchange of the sharded head, in which
 * case every rank must create and run in step with the others.  create runs the step once before it
 * records it, so the workspace header must be zero at that point, as for qfg_lmhead_compute. */
typedef struct qfg_lmhead_host qfg_lmhead_host;
QFG_API int qfg_lmhead_host_create(const qfg_lmhead* op, int64_t m, int64_t k, const qfg_tensor2d* weight, int64_t n,
                                   int64_t col_offset, void* workspace, const qfg_lmhead_exchange* exchange,
                                   const void* x_host, void* x_dev, int64_t* idx_host, float* val_host,
                                   qfg_lmhead_host** out);
QFG_API int qfg_lmhead_host_run(qfg_lmhead_host* h);
QFG_API void qfg_lmhead_host_destroy(qfg_lmhead_host* h);
/* Device memory that other processes on the node can map (cudaMalloc + cudaIpcGetMemHandle; `handle`
 * receives 64 bytes), the mapping of another process's handle (peer access enabled lazily), and their
 * releases.  Set-up calls: they allocate and synchronise. */
QFG_API int qfg_peer_alloc(size_t bytes, void** ptr, unsigned char handle[64]);
QFG_API int qfg_peer_open(const unsigned char handle[64], void** ptr);
QFG_API int qfg_peer_close(void* ptr);
QFG_API int qfg_peer_free(void* ptr);

/* Fold `ranks` gathered key rows (keys[rank * m + row]) into idx[row] / val[row]. */
QFG_API int qfg_lmhead_combine(const uint64_t* keys, int ranks, int64_t m, int64_t* idx, float* val, void* stream);

/* Measurement aid, no counterpart in the reference: sweeps `bytes` of device memory at `buf` (16-byte aligned) with
 * 128-bit read-only loads and writes nothing (`sink`, 4 bytes of device memory or null, is never stored to on
 * real data).  Timed over a buffer several times the size of L2 it gives the read-only streaming ceiling of the
 * GPU, the denominator a weight-streaming kernel is compared with besides the copy bandwidth. */
QFG_API int qfg_stream_read_probe(const void* buf, size_t bytes, void* sink, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* QFG_H_ */
