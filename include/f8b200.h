/*
 * f8b200.h -- C ABI of the B200 (sm_100a) float8 training kernels.
 *
 * This is the drop-in boundary for the Float8Linear hot path of
 * pytorch-labs/float8_experimental.  The reference reaches its arithmetic through
 * PyTorch operators; each entry point below names the reference call site(s) it
 * replaces (paths are relative to the reference project root).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the comment says "host";
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *   - calls are asynchronous with respect to the host and never synchronise;
 *   - the library allocates nothing: all buffers belong to the caller;
 *   - every call returns an int status (0 = ok, negative = error, see below), never
 *     throws, aborts or traps;
 *   - fp8 tensors are raw bytes (OCP e4m3fn / e5m2 bit patterns).
 */
#ifndef F8B200_H_
#define F8B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* high-precision element types */
#define F8B200_BF16 0
#define F8B200_FP16 1
#define F8B200_FP32 2

/* fp8 formats */
#define F8B200_E4M3 0 /* torch.float8_e4m3fn, max 448   */
#define F8B200_E5M2 1 /* torch.float8_e5m2,   max 57344 */

/* status codes */
#define F8B200_OK 0
#define F8B200_ERR_BAD_ARG (-1)     /* null pointer, negative size, unknown enum      */
#define F8B200_ERR_ALIGNMENT (-2)   /* pointer or leading dimension not aligned       */
#define F8B200_ERR_ARCH (-3)        /* current device is not compute capability 10.x  */
#define F8B200_ERR_LAUNCH (-4)      /* CUDA reported an error at launch               */
#define F8B200_ERR_DRIVER (-5)      /* tensor-map encode / driver entry point failed  */
#define F8B200_ERR_UNSUPPORTED (-6) /* valid request the kernels do not implement     */
#define F8B200_ERR_TIMEOUT (-7)     /* a bounded device-side wait ran out             */

const char* f8b200_status_string(int status);

/* 0 when the current device can run these kernels (compute capability 10.x). */
int f8b200_device_check(void);

/* Text of the last CUDA error seen by this library on the calling thread. */
const char* f8b200_last_cuda_error(void);

/*
 * amax = max |x| over `numel` contiguous elements, written to amax_out[0] as fp32
 * (exactly representable: it is one of the inputs).  NaN anywhere gives NaN.
 * Replaces torch.max(torch.abs(x)) in float8_experimental/float8_utils.py:102-104
 * (tensor_to_amax).  numel == 0 is F8B200_ERR_BAD_ARG (torch.max raises there).
 */
int f8b200_amax(const void* x, int hp_dtype, int64_t numel, float* amax_out, void* stream);

/*
 * Same reduction for `n` separate tensors in one launch: amax_out[i] = max |x_i|.
 * `ptrs` and `numels` are HOST arrays of length n (device pointers inside `ptrs`).
 * A tensor with numels[i] == 0 yields 0.  Replaces torch._foreach_norm(weights, inf)
 * in float8_experimental/fsdp_utils.py:62 (precompute_float8_dynamic_scale_for_fsdp).
 */
int f8b200_multi_amax(const void* const* ptrs, const int64_t* numels, int n, int hp_dtype,
                      float* amax_out, void* stream);

/*
 * scale_out[i] = amax_to_scale(amax[i]) for i < n:
 *   c = max(amax, RN_T(1e-12)); r = RN_T(1/c); s = RN_T(r * fp8_max);
 *   if orig_dtype == FP16: s = min(s, 65504)
 * with T = amax_dtype (the dtype the reference holds the amax in) and the result
 * stored as fp32.  Replaces float8_experimental/float8_utils.py:35-57 (amax_to_scale),
 * including the reciprocal-then-multiply evaluation of `fp8_max / clamp(amax, EPS)`.
 */
int f8b200_amax_to_scale(const float* amax, int64_t n, int fp8_kind, int amax_dtype,
                         int orig_dtype, float* scale_out, void* stream);

/*
 * Saturating round-to-nearest-even cast of a [rows, cols] matrix (row stride ld_x
 * elements) to fp8:  out = fp8(clamp(RN_P(x * scale), +-fp8_max)).
 *
 *   scale_src    0: `scale_in` points at the fp32 scale to use (delayed scaling,
 *                   precomputed FSDP scale);
 *                1: `scale_in` points at an fp32 amax; the kernel derives the scale
 *                   from it exactly as f8b200_amax_to_scale(amax_dtype = orig_dtype =
 *                   hp_dtype) and, when scale_out != NULL, stores it there (dynamic
 *                   scaling).
 *   product_fp32 0: the product x*scale is rounded to hp_dtype before the clamp
 *                   (PyTorch semantics for a 0-dim scale); 1: it stays fp32 (scale of
 *                   shape [1], or fp32 input).
 *   out          row-major fp8 bytes, row stride ld_out; may be NULL.
 *   out_t        the transposed copy [cols, rows], row stride ld_out_t; may be NULL.
 *   amax_out     optional fp32 word that receives max |x| of this same read
 *                (delayed scaling records the current amax while casting).
 *   reverse      non-zero walks the tiles from the end of the tensor backwards, so
 *                that a cast that follows an amax pass over the same tensor starts on
 *                the part still held in L2.
 *
 * Replaces `tensor * scale` (float8_experimental/float8_tensor.py:158) +
 * to_fp8_saturated (float8_utils.py:123-139), the scale computation of
 * tensor_to_scale (float8_utils.py:115-120) in dynamic mode, the amax fill of
 * hp_tensor_to_float8_delayed (float8_scaling_utils.py:89), and the layout copies of
 * preprocess_addmm (float8_ops.py:150-153) through `out_t`.
 */
int f8b200_cast(const void* x, int hp_dtype, int64_t rows, int64_t cols, int64_t ld_x,
                int scale_src, const float* scale_in, float* scale_out, int product_fp32,
                int fp8_kind, void* out, int64_t ld_out, void* out_t, int64_t ld_out_t,
                float* amax_out, int reverse, void* stream);

/*
 * The whole dynamic cast of a CONTIGUOUS [rows, cols] tensor in one call: f8b200_amax into amax_out,
 * then f8b200_cast(scale_src = 1, reverse = 1) from that amax (scale stored to scale_out when not
 * NULL).  Two kernels and a 4-byte memset on `stream`, one host call: hp_tensor_to_float8_dynamic of
 * float8_experimental/float8_scaling_utils.py:33-62 (about ten operator launches in the reference).
 * One host call per tensor keeps the host ahead of the GPU in models of many small layers.
 */
int f8b200_cast_dynamic(const void* x, int hp_dtype, int64_t rows, int64_t cols, int fp8_kind,
                        float* amax_out, float* scale_out, void* out, void* stream);

/*
 * f8b200_cast whose row-major result goes to n_outs destinations at once (1 <= n_outs <=
 * F8B200_CAST_MAX_EXTRA + 1, all with row pitch ld_out; `outs` is a HOST array of device
 * pointers).  With the destinations being this rank's slot in the gathered buffer of every
 * rank (peer-mapped memory, plain stores over NVLink), the cast IS the all-gather: it
 * replaces the cast followed by the fp8 all-gather of
 * float8_experimental/float8_tensor_parallel.py:49-60 (Float8ColwiseParallel input) and
 * float8_experimental/fsdp_utils.py:168-207.  The caller orders the stores against the
 * readers (one collective on the same stream after the call, another before the next use of
 * the buffers).  No transposed copy, no amax output.
 */
#define F8B200_CAST_MAX_EXTRA 15
int f8b200_cast_scatter(const void* x, int hp_dtype, int64_t rows, int64_t cols, int64_t ld_x,
                        int scale_src, const float* scale_in, float* scale_out, int product_fp32,
                        int fp8_kind, void* const* outs, int n_outs, int64_t ld_out, void* stream);

/*
 * The saturating cast of f8b200_cast(scale_src = 0) for n separate CONTIGUOUS tensors in one
 * launch: outs[i] = fp8(clamp(RN_P(xs[i] * scales[i]))), numels[i] elements each, scales a device
 * array of n fp32 words.  `xs`, `numels`, `outs` are HOST arrays of length n (device pointers
 * inside).  With the scale vector that f8b200_multi_amax + one all-reduce + f8b200_amax_to_scale
 * produce after an optimizer step, this casts every FSDP weight shard of a model with one launch
 * (per 96 tensors) instead of one cast per weight per all-gather
 * (float8_experimental/fsdp_utils.py:168-185, fsdp_pre_all_gather).
 */
int f8b200_multi_cast(const void* const* xs, const int64_t* numels, int n, int hp_dtype,
                      const float* scales, int product_fp32, int fp8_kind, void* const* outs,
                      void* stream);

/*
 * out[c, r] = in[r, c] for an fp8 (byte) matrix [rows, cols].  Replaces the
 * `.contiguous()` / `.t().contiguous().t()` fix-ups in
 * float8_experimental/float8_ops.py:150-153 when no transposed copy was emitted by
 * the cast (for example an fp8 weight that arrived through the FSDP all-gather).
 */
int f8b200_transpose_u8(const void* in, int64_t rows, int64_t cols, int64_t ld_in, void* out,
                        int64_t ld_out, void* stream);

/*
 * Delayed-scaling bookkeeping for R = n_input + n_weight + n_grad_output rows in one
 * launch.  Per row r:  rolled = [amax[r], hist[r,0..H-2]];
 *   scale[r] = amax_to_scale(max(rolled))  in fp32 arithmetic, with fp8_max = 448 for
 *   the first n_e4m3 rows and 57344 for the rest, and the fp16 clamp when
 *   orig_dtype == F8B200_FP16.
 * hist_out == NULL leaves the history untouched (what the reference does: it rolls a
 * stacked copy and never writes it back); otherwise the rolled history is written to
 * hist_out (may alias hist).  Replaces _update_history_stack +
 * amax_history_to_scale_stack + the per-layer copy_ loops in
 * float8_experimental/float8_linear_utils.py:286-319 and float8_utils.py:80-99.
 */
int f8b200_delayed_sync(const float* amax, const float* hist, int64_t ld_hist, int64_t rows,
                        int hist_len, int64_t n_e4m3, int orig_dtype, float* scale_out,
                        float* hist_out, int64_t ld_hist_out, void* stream);

/*
 * out[M,N] = (A[M,K] . B[N,K]^T) * (1/scale_a) * (1/scale_b) (+ bias[N]) in out_dtype.
 *
 *   a, b      fp8 bytes, both with K contiguous ("row-major A, column-major B" in the
 *             reference's words); lda, ldb in elements, multiples of 16, bases 16-byte
 *             aligned (TMA requirement).
 *   scale_a/b fp32 words holding the scales the operands were MULTIPLIED by when they
 *             were cast; the kernel divides them out in its epilogue.
 *   bias      optional [N] vector in out_dtype.
 *   out       row-major, row stride ldo elements, dtype F8B200_BF16/FP16/FP32.
 *   fp32 accumulation in tensor memory; use_fast_accum is accepted and ignored.
 *
 * Replaces addmm_float8_unwrapped -> torch._scaled_mm in
 * float8_experimental/float8_python_api.py:24-64 (and the two scale.reciprocal()
 * launches at :39-40, and the bias add at float8_linear.py:368-369).
 */
int f8b200_gemm_fp8(const void* a, int a_kind, int64_t lda, const void* b, int b_kind, int64_t ldb,
                    const float* scale_a, const float* scale_b, const void* bias, int out_dtype,
                    void* out, int64_t ldo, int64_t m, int64_t n, int64_t k, int use_fast_accum,
                    void* stream);

/*
 * f8b200_gemm_fp8 with a caller-owned workspace, which switches the persistent kernels from a
 * fixed stride of output tiles per CTA to dynamic tile scheduling: CTAs claim tiles from a
 * counter in the workspace, so that a CTA whose SM was held by a kernel of another stream (an
 * all-gather or reduce-scatter running beside the GEMM) does fewer tiles instead of making the
 * launch wait for its full share.  Results are bit-identical to f8b200_gemm_fp8 (each output
 * tile is accumulated the same way whichever CTA computes it).
 *
 *   workspace        device memory, 16-byte aligned, at least F8B200_GEMM_WORKSPACE_BYTES.  The
 *                    contents need no initialisation (the call zeroes what it uses with a
 *                    memset on `stream`) and are undefined afterwards.  Two GEMMs that may run
 *                    at the same time (different streams) must not share a workspace; GEMMs on
 *                    one stream may.  Capturable in a CUDA graph (memset node + kernel node).
 *
 *   a_layout,        F8B200_K_MAJOR: as in f8b200_gemm_fp8.  F8B200_MN_MAJOR: the operand is the
 *   b_layout         TRANSPOSE of that storage, a [K, M] (b [K, N]) byte matrix with M (N)
 *                    contiguous and lda (ldb) its row pitch.  The tensor cores read such a
 *                    tile through an MN-major shared-memory descriptor, so the backward GEMMs
 *                    take grad_output, the input and the weight as they lie in memory and the
 *                    transposed fp8 copies of float8_experimental/float8_ops.py:150-153 are
 *                    never made.  Same alignment rules (base and pitch multiples of 16).
 *
 * Same reference call site as f8b200_gemm_fp8 (float8_experimental/float8_python_api.py:24-64;
 * torch._scaled_mm there draws its workspace from cuBLASLt's own allocation).
 */
#define F8B200_GEMM_WORKSPACE_BYTES 256
#define F8B200_K_MAJOR 0  /* operand stored [rows, K], K contiguous, ld >= K  */
#define F8B200_MN_MAJOR 1 /* operand stored [K, rows], rows contiguous, ld >= rows */
int f8b200_gemm_fp8_ws(const void* a, int a_kind, int a_layout, int64_t lda, const void* b, int b_kind,
                       int b_layout, int64_t ldb, const float* scale_a, const float* scale_b,
                       const void* bias, int out_dtype, void* out, int64_t ldo, int64_t m, int64_t n,
                       int64_t k, int use_fast_accum, void* workspace, int64_t workspace_bytes,
                       void* stream);

/*
 * Reduce-scatter of a row-parallel linear's output, fused into the GEMM: replaces
 * `outputs.redistribute(placements=output_layouts)` of Float8RowwiseParallel
 * (float8_experimental/float8_tensor_parallel.py:116-128; the bf16 reduce-scatter of the partial
 * products) together with the GEMM before it (float8_python_api.py:24-64).
 *
 * f8b200_gemm_fp8_scatter_rows   f8b200_gemm_fp8_ws whose output rows go to n_outs destinations:
 *     row i belongs to block i / rows_per_block; blocks go round-robin to the destinations, so row i
 *     is stored in outs[block % n_outs] at row (block / n_outs) * rows_per_block + i % rows_per_block
 *     (row pitch ldo).  With outs[r] = this rank's slot in rank r's receive buffer (peer-mapped
 *     memory, plain stores over NVLink from the epilogue warps; no TMA touches a destination), the
 *     GEMM's stores ARE the scatter.  `outs` is a HOST array of device pointers, n_outs <= 16, m a
 *     multiple of rows_per_block * n_outs.  bias must be NULL for a partial product that will be
 *     summed (it would be added once per rank).  The caller orders the stores against the reader
 *     (one collective on the same stream after the call).
 * f8b200_sum_slots               out[i] = RN_T(sum over s < n_slots of slots[s * slot_stride + i]) for
 *     i < numel, accumulated in fp32 in slot order (deterministic): the owner's half of the
 *     reduce-scatter.  16-byte aligned pointers and slot pitch.
 */
int f8b200_gemm_fp8_scatter_rows(const void* a, int a_kind, int a_layout, int64_t lda, const void* b, int b_kind,
                                 int b_layout, int64_t ldb, const float* scale_a, const float* scale_b,
                                 const void* bias, int out_dtype, void* const* outs, int n_outs,
                                 int64_t rows_per_block, int64_t ldo, int64_t m, int64_t n, int64_t k,
                                 void* workspace, int64_t workspace_bytes, void* stream);
int f8b200_sum_slots(const void* slots, int n_slots, int64_t slot_stride, int hp_dtype, int64_t numel,
                     void* out, void* stream);

/*
 * Which kernel f8b200_gemm_fp8 / _ws would run for an m x n x k product with the current
 * environment: 0 = one CTA per 128x256 tile, 1 = CTA pair per 256x256 tile, 2 = one CTA per
 * 256x256 tile, 3 = CTA pair per 512x256 tile.  Default: 3 for large products with K >= 8192, 1 where
 * the larger tiles would fill the last wave of CTA pairs badly or K is short (and for at most 256
 * rows).  All four return the same bits; the choice is a matter of speed.  Reporting aid for benchmarks; host only (it reads
 * the SM count of the current device and assumes 148 without one).  (cuBLASLt's heuristic behind torch._scaled_mm, float8_python_api.py:43-63, is the
 * reference-side counterpart.)
 */
int f8b200_gemm_kernel_choice(int64_t m, int64_t n, int64_t k);

/*
 * f8b200_gemm_fp8_ws without the workspace argument: the scheduling words live in a file-scope
 * `static __device__` array of F8B200_STATIC_SCRATCH_BYTES (4096) bytes inside the library, one
 * F8B200_GEMM_WORKSPACE_BYTES slot per stream.  This entry point has NO counterpart in the
 * reference (torch._scaled_mm takes its workspace from cuBLASLt); it exists for callers that
 * cannot pass device memory of their own.  It allocates and frees nothing, on the host or the
 * device, and returns the same bits as f8b200_gemm_fp8 / f8b200_gemm_fp8_ws.
 *
 *   set-up      The first call on each device that passes the argument checks looks the array up
 *               with cudaGetSymbolAddress and keeps the address.  That call must happen outside any
 *               stream capture; make one call per device before capturing a CUDA graph that
 *               contains this entry point.  A lookup that fails is not remembered: the next call
 *               tries again.  Calls that fail their argument checks or have nothing to compute
 *               (m == 0 or n == 0) neither look the array up nor take a slot.
 *   size limit  A stream gets its slot at its first call and keeps it for the life of the
 *               process (slots are not recycled when a stream is destroyed; a new stream that
 *               happens to get the same handle reuses the old slot, which is safe).  The array
 *               holds 16 slots: the call that would need a 17th stream on one device returns
 *               F8B200_ERR_UNSUPPORTED and launches nothing.  Use f8b200_gemm_fp8_ws there.
 *   sharing     The array is shared by every caller of this entry point in the process (all
 *               host threads, all users of the library); the slot table is guarded by a mutex.
 *               Calls on one stream are ordered by the stream and share that stream's slot.
 *               What is NOT safe is one slot used by two launches that can run at the same
 *               time: a captured graph holding this call that is replayed on another stream
 *               while the capture stream issues further calls, or one such graph launched on
 *               two streams at once.  Both launches would claim tiles from one counter and
 *               each would skip the tiles the other claimed.  Give such work
 *               f8b200_gemm_fp8_ws with a workspace of its own.
 */
#define F8B200_STATIC_SCRATCH_BYTES 4096
int f8b200_gemm_fp8_static_scratch(const void* a, int a_kind, int64_t lda, const void* b, int b_kind,
                                   int64_t ldb, const float* scale_a, const float* scale_b,
                                   const void* bias, int out_dtype, void* out, int64_t ldo,
                                   int64_t m, int64_t n, int64_t k, int use_fast_accum, void* stream);

/*
 * RMSNorm fused into the dynamic fp8 cast of its output, in two launches that never write the
 * normalised tensor: 5 bytes of HBM traffic per element instead of 9 (norm 2 + 2, cast 2 + 2 + 1).
 *
 *   y = RN_T( float(RN_T(x * rstd)) * w ),   rstd = 1 / sqrt(mean(x^2 over the row) + eps)
 *
 * with T = hp_dtype (x and weight share it) and the mean accumulated in fp32: RMSNorm.forward
 * of float8_experimental/benchmarks/profile_linear_float8.py:69-74, the producer that the
 * reference leaves to torch.compile to fuse with the cast (same file :129-149).
 *
 * f8b200_rmsnorm_amax  pass A: rstd_out[rows] (fp32) and amax_out[0] = max |y| (fp32; zeroed by
 *                      the call).  Reads x once.
 * f8b200_rmsnorm_cast  pass B: out = fp8(clamp(RN_T(y * scale))) with the scale derived from
 *                      `amax` as in f8b200_cast(scale_src = 1); scale_out (optional) receives
 *                      it.  Reads x once, writes the fp8 bytes (row stride ld_out).
 * Between the two the caller may all-reduce amax (tensor / sequence parallel inputs).
 */
int f8b200_rmsnorm_amax(const void* x, int hp_dtype, int64_t rows, int64_t cols, int64_t ld_x,
                        const void* weight, float eps, float* rstd_out, float* amax_out,
                        void* stream);
int f8b200_rmsnorm_cast(const void* x, int hp_dtype, int64_t rows, int64_t cols, int64_t ld_x,
                        const void* weight, const float* rstd, const float* amax, int fp8_kind,
                        float* scale_out, void* out, int64_t ld_out, void* stream);

/*
 * SwiGLU gate fused into the dynamic fp8 cast of its output, like the RMSNorm pair above:
 *
 *   y = RN_T( float(RN_T(silu(a))) * b ),   silu(a) = a / (1 + exp(-a)) in fp32
 *
 * for a, b [rows, cols] of one dtype T with row pitches ld_a, ld_b (the two halves of a fused
 * w1|w3 output are the usual case): `F.silu(self.w1(x)) * self.w3(x)` of
 * float8_experimental/benchmarks/profile_linear_float8.py:117-118, the producer of the w2
 * input.  9 bytes of traffic per element instead of 17.  exp is the device math library's
 * expf, so results can differ from a CPU evaluation in the last fp32 bit of silu(a).
 *
 * f8b200_swiglu_amax  pass A: amax_out[0] = max |y| (fp32; zeroed by the call).  With y_out !=
 *                     NULL it also writes y (dtype T, row pitch ld_y) and pass B can then be
 *                     f8b200_cast(y, scale_src = 1): same 9 bytes per element, and the gate,
 *                     whose exp and division make it issue-bound, is evaluated once.
 * f8b200_swiglu_cast  pass B from a and b again (y never written): out = fp8(clamp(RN_T(y *
 *                     scale))), scale derived from `amax` as in f8b200_cast(scale_src = 1);
 *                     scale_out (optional) receives it.
 */
int f8b200_swiglu_amax(const void* a, const void* b, int hp_dtype, int64_t rows, int64_t cols,
                       int64_t ld_a, int64_t ld_b, void* y_out, int64_t ld_y, float* amax_out,
                       void* stream);
int f8b200_swiglu_cast(const void* a, const void* b, int hp_dtype, int64_t rows, int64_t cols,
                       int64_t ld_a, int64_t ld_b, const float* amax, int fp8_kind,
                       float* scale_out, void* out, int64_t ld_out, void* stream);
/*
 * Opt-in approximate gate: f8b200_swiglu_amax with sigmoid(a) = rcp.approx(1 + ex2.approx(-a * log2 e))
 * (about 2^-21 relative error in fp32) in place of the correctly rounded division and expf; the
 * roundings to T are the same.  RN_T(silu(a)) is then the exact path's value except where that lies
 * within ~2^-12 ulp of a rounding boundary of T, where it is the neighbouring T value: y, and the
 * amax, are within one ulp of T of the exact path's, so every fp8 byte of the cast that follows is
 * within one fp8 step.  Issue-bound like the exact kernel, with about a third fewer instructions per
 * element.  16-bit dtypes with cols a multiple of 8 and 16-byte aligned rows only
 * (F8B200_ERR_UNSUPPORTED otherwise).  No reference counterpart (the reference evaluates the gate
 * with the framework's exact ops).
 */
int f8b200_swiglu_amax_approx(const void* a, const void* b, int hp_dtype, int64_t rows, int64_t cols,
                              int64_t ld_a, int64_t ld_b, void* y_out, int64_t ld_y, float* amax_out,
                              void* stream);

/*
 * Backward of the two fused producers (the casts are transparent to autograd:
 * float8_experimental/float8_tensor.py:193-195), one pass over the saved inputs each; the
 * formulas are the gradients of float8_experimental/benchmarks/profile_linear_float8.py:69-74
 * and :117-118 as eager autograd evaluates them for 16-bit tensors.
 *
 * f8b200_rmsnorm_bwd  dx = RN_T(rstd * (dn - n * mean(dn * n))) with n = x * rstd, dn = RN_T(g * w);
 *                     dweight[col] = RN_T(sum over rows of g * RN_T(n)).  Reads x and grad_y, writes
 *                     dx (6 bytes per element).  `workspace`: at least
 *                     f8b200_rmsnorm_bwd_workspace_bytes(cols) bytes of device memory for per-CTA
 *                     partial sums (contents need no initialisation).
 * f8b200_swiglu_bwd   da = RN_T(RN_T(g * b) * sig(a) * (1 + a * (1 - sig(a)))), db = RN_T(g * RN_T(silu(a))).
 *                     Reads a, b, grad_y, writes da, db with row pitch ld_out (10 bytes per element).
 *
 * Any of the three dtypes, any column count and row pitch: 16-bit dtypes with cols a multiple of 8
 * (RMSNorm: at most 8192) and 16-byte aligned rows run on the vectorised kernels, everything else on
 * element-wise variants with the same formulas and roundings.
 */
int64_t f8b200_rmsnorm_bwd_workspace_bytes(int64_t cols);
int f8b200_rmsnorm_bwd(const void* x, const void* grad_y, int hp_dtype, int64_t rows, int64_t cols,
                       int64_t ld_x, int64_t ld_g, const void* weight, const float* rstd, void* dx,
                       int64_t ld_dx, void* dweight, void* workspace, int64_t workspace_bytes,
                       void* stream);
int f8b200_swiglu_bwd(const void* a, const void* b, const void* grad_y, int hp_dtype, int64_t rows,
                      int64_t cols, int64_t ld_a, int64_t ld_b, int64_t ld_g, void* da, void* db,
                      int64_t ld_out, void* stream);
/* f8b200_swiglu_bwd with the approximate sigmoid of f8b200_swiglu_amax_approx (same restrictions):
 * da and db within one ulp of T of the exact path's. */
int f8b200_swiglu_bwd_approx(const void* a, const void* b, const void* grad_y, int hp_dtype, int64_t rows,
                             int64_t cols, int64_t ld_a, int64_t ld_b, int64_t ld_g, void* da, void* db,
                             int64_t ld_out, void* stream);

/*
 * Reads and clears the device error word of the current device (synchronises the
 * device).  *flags_out != 0 means a bounded wait inside a kernel gave up since the
 * last read; the result of that launch is undefined.  Test and debugging aid.
 */
int f8b200_read_device_error(uint32_t* flags_out);

/*
 * The same read as a status: F8B200_OK when no bounded wait gave up since the last read,
 * F8B200_ERR_TIMEOUT otherwise (the word is cleared either way; synchronises the device).  A
 * launch returns F8B200_OK as soon as the kernel is queued, so a wait that runs out later can only
 * show up here: C callers poll this at a point where they synchronise anyway (end of a step) and
 * treat F8B200_ERR_TIMEOUT as "the outputs of the GEMMs since the last poll are undefined".  No
 * counterpart in the reference (cuBLASLt reports nothing of the kind).
 */
int f8b200_check_device_error(void);

#ifdef __cplusplus
}
#endif
#endif /* F8B200_H_ */
