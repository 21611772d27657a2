/*
 * mtb200 - C ABI of the B200 (sm_100a) dense-contraction path for minitensor.
 *
 * This is the boundary a minitensor build binds (Rust `extern "C"` block,
 * ctypes, cgo ...).  Every function returns an int32 status (0 = OK); the text
 * of the last failure on the calling thread is at mtb200_last_error().  No
 * exception, abort or C++ type crosses the boundary.  All data pointers are
 * DEVICE pointers owned by the caller (from mtb200_alloc or any other CUDA
 * allocator on the handle's device); matrices are dense row-major.  Work is
 * enqueued on the handle's stream and is asynchronous until mtb200_sync.
 * A handle is used from one host thread at a time; calls on one handle that are issued on
 * different streams (mtb200_set_stream) share its scratch memory and must be ordered by the
 * caller.  Several handles may live on one device.
 *
 * Environment (read when a handle or a communicator is created):
 *   MTB200_NO_PDL=1     launch every kernel the plain way (default: the kernels of a call are chained
 *                       by programmatic dependent launch; results are bit-identical either way)
 *   MTB200_NCCL_LIB     path of the NCCL library to open when none is loaded in the process
 *   MTB200_COMM_CTAS=n  CTA budget asked of NCCL for a communicator (default 16, 0 = leave NCCL alone)
 *
 * File/line references name the minitensor source each entry point stands in
 * for (paths relative to the minitensor repository root).
 */
#ifndef MTB200_H_
#define MTB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MTB200_VERSION 100

/* status codes */
enum {
  MTB200_OK = 0,
  MTB200_ERR_INVALID = 1,      /* bad argument: shape, null pointer, enum out of range   */
  MTB200_ERR_CUDA = 2,         /* a CUDA runtime / driver call failed                    */
  MTB200_ERR_NOMEM = 3,        /* device allocation failed                               */
  MTB200_ERR_UNSUPPORTED = 4,  /* dtype / option not available for this operation        */
  MTB200_ERR_DEVICE_WAIT = 5,  /* a bounded wait inside a kernel ran out (see mtb200_sync) */
  MTB200_ERR_BAD_LABEL = 6     /* class index outside [0, C) seen by cross entropy       */
};

/* element types, numbered like minitensor's DataType (engine/src/tensor/dtype.rs:12-19) */
enum { MTB200_F32 = 0, MTB200_F64 = 1, MTB200_I32 = 2, MTB200_I64 = 3, MTB200_BOOL = 4 };

/* epilogues fused into mtb200_gemm */
enum {
  MTB200_EPI_NONE = 0,
  MTB200_EPI_RELU = 1,      /* activation::relu      engine/src/operations/activation/softmax.rs:161-203 */
  MTB200_EPI_GELU_ERF = 2,  /* activation::gelu exact  engine/src/operations/activation/hyperbolic.rs:697-745 */
  MTB200_EPI_GELU_TANH = 3, /* activation::gelu approximate (same lines)                                  */
  MTB200_EPI_RELU_BWD = 4   /* ReluBackward: multiply by (aux > 0)  engine/src/autograd/mod/shape.rs:724-816 */
};

/* f32 arithmetic modes of mtb200_gemm (argument f32_mode, low byte).  Every mode
 * multiplies on the tensor cores with f32 accumulation; they differ in how an
 * f32 operand is represented. */
enum {
  MTB200_F32_DEFAULT = 0, /* F16X3 when the output is larger than 128 x 128 (pair tiles, or
                           * 128 x 128 tiles of one CTA when the pair tiles are few), else BF16X6;
                           * products with K <= 64 and at most 4e6 multiply-adds run as one
                           * launch of plain f32 multiply-add on the CUDA cores instead       */
  MTB200_F32_BF16X1 = 1,  /* single bf16 product: ~2^-8 relative, for experiments            */
  MTB200_F32_BF16X3 = 3,  /* two bf16 terms, three products: ~2^-16 relative                 */
  MTB200_F32_BF16X6 = 6,  /* three bf16 terms (24 bits), six products                        */
  MTB200_F32_BF16X9 = 9,  /* three bf16 terms, all nine products                             */
  MTB200_F32_F16X3 = 23   /* two fp16 terms (22 bits) after exact power-of-two row/column
                           * scaling, three products: the accuracy class of 3xTF32 at half
                           * its tensor cost; needs M, N > 128                              */
};

/* Second byte of f32_mode (f32_mode = mode | variant << 8), for tests and experiments: 0 = choose;
 * 1..6 = a fixed tile shape of the tensor kernels; 0xFE = the CUDA-core kernel (f32: IEEE multiply-add
 * in one launch; int32: the IMAD kernel); 0xFD = the integer tensor path regardless of size;
 * 0xFF / 0xFB / 0xFC (conv2d entries) = a fixed lowering, see there. */

typedef struct mtb200_ctx* mtb200_handle;

/* ---- library / handle ---------------------------------------------------- */
int32_t mtb200_version(void);
const char* mtb200_last_error(void);

/* Backend::initialize / is_available  (engine/src/backends/mod.rs:21-46,
 * engine/src/backends/cuda/mod.rs:164-197).  Fails (MTB200_ERR_CUDA) when the
 * device is absent or is not compute capability 10.x. */
int32_t mtb200_create(int32_t device_ordinal, mtb200_handle* out);
int32_t mtb200_destroy(mtb200_handle h);
/* Enqueue on an existing cudaStream_t / CUstream from now on (NULL = the CUDA
 * default stream).  A new handle uses a non-blocking stream of its own. */
int32_t mtb200_set_stream(mtb200_handle h, void* cuda_stream);
/* SMs the persistent tensor-core GEMM kernels may occupy from now on (0 = all).  (No counterpart in the
 * reference.)  Those kernels launch one CTA per SM and deal tiles out statically, so a kernel that runs beside
 * them and needs SMs of its own - a collective overlapping the backward pass - otherwise delays some CTAs and
 * with them the whole GEMM; leaving it a few SMs costs less than that. */
int32_t mtb200_set_gemm_sm_limit(mtb200_handle h, int32_t sms);
/* CudaBackend::synchronize (engine/src/backends/cuda/mod.rs:153-161); also
 * reports MTB200_ERR_DEVICE_WAIT if a kernel recorded an expired wait. */
int32_t mtb200_sync(mtb200_handle h);
/* Per-launch timing, the device-side analogue of the reference's manual
 * OperationProfiler (engine/src/debug.rs:273-352).  While enabled, every kernel
 * of the listed classes is bracketed by a CUDA event pair on the handle's
 * stream.  profile_enable(1) clears earlier records; profile_read synchronises
 * and returns launches, summed device time and summed algorithmic work of one
 * class: 0 = split-bf16 tensor-core GEMM kernel (work = 2*M*N*K flops),
 * 1 = operand split kernels (bytes), 2 = f64 GEMM (flops), 3 = integer GEMM
 * (ops), 4 = conv gather kernels (bytes). */
int32_t mtb200_profile_enable(mtb200_handle h, int32_t on);
int32_t mtb200_profile_read(mtb200_handle h, int32_t kernel_class, int64_t* launches,
                            double* total_ms, double* total_work);

/* Bytes of scratch memory the handle currently holds (operand splits, partial sums). */
int32_t mtb200_workspace_bytes(mtb200_handle h, size_t* bytes);

/* ---- memory: Backend::allocate / deallocate / copy_from_host / copy_to_host
 * (engine/src/backends/mod.rs:30-45; CUDA semantics engine/src/backends/cuda/mod.rs:199-317):
 * zero bytes -> NULL pointer and OK; true device memory, not unified memory. */
int32_t mtb200_alloc(mtb200_handle h, size_t bytes, void** dptr);
int32_t mtb200_free(mtb200_handle h, void* dptr, size_t bytes);
int32_t mtb200_h2d(mtb200_handle h, void* dst_device, const void* src_host, size_t bytes);
int32_t mtb200_d2h(mtb200_handle h, void* dst_host, const void* src_device, size_t bytes);
int32_t mtb200_memset_zero(mtb200_handle h, void* dptr, size_t bytes);

/* ---- GEMM: C[b] = epilogue(op(A[b]) * op(B[b]) + bias)
 *
 * Stands in for matmul's dtype dispatch matmul_f32/f64/i32/i64
 * (engine/src/operations/linalg/matmul.rs:376-385, diagonal.rs:400-640), bmm
 * (matmul.rs:738-763), the two products of MatMulBackward
 * (engine/src/autograd/mod/core.rs:752-789: dA = dY*B^T is trans_b = 1,
 * dB = A^T*dY is trans_a = 1, no materialised transpose), DenseLayer::forward
 * (engine/src/nn/dense_layer.rs:139-169: trans_b = 1 on the [out,in] weight,
 * bias fused) and the device op CudaOps::matmul (engine/src/backends/cuda/mod.rs:519-578).
 *
 * op(A) is M x K: A is row-major [M,K] (trans_a = 0) or [K,M] (trans_a = 1).
 * op(B) is K x N: B is row-major [K,N] (trans_b = 0) or [N,K] (trans_b = 1).
 * C is row-major [M,N].  Batch entries are `stride_*` ELEMENTS apart; a stride
 * of 0 for A or B broadcasts one matrix over the batch (matmul.rs:324-345).
 * bias: [N] or NULL.  aux: layout of C, read by MTB200_EPI_RELU_BWD, else NULL.
 * Epilogues other than NONE need a floating dtype.  K == 0 yields
 * epilogue(bias) (zeros without bias, matmul.rs:373-376).  Integer dtypes wrap
 * modulo 2^32 / 2^64. */
int32_t mtb200_gemm(mtb200_handle h, int32_t dtype, int32_t trans_a, int32_t trans_b,
                    int64_t batch, int64_t M, int64_t N, int64_t K,
                    const void* A, int64_t stride_a, const void* B, int64_t stride_b,
                    void* C, int64_t stride_c, const void* bias, int32_t epilogue,
                    const void* aux, int32_t f32_mode);

/* ---- dense layer as one call per direction (f32 / f64)
 * forward:  y[rows][out] = epilogue(x[rows][in] * W[out][in]^T + bias[out])
 *           DenseLayer::forward = transpose + matmul + add (engine/src/nn/dense_layer.rs:139-169)
 * backward: dX[rows][in] = dx_epilogue(dY * W)   (skipped when dX is NULL: input without requires_grad,
 *                                                 engine/src/autograd/mod/core.rs:763)
 *           dW[out][in]  = dY^T * x                (skipped when dW is NULL)
 *           db[out]      = column sums of dY      (skipped when db is NULL)
 *           MatMulBackward (engine/src/autograd/mod/core.rs:743-789), the transpose's backward and the
 *           broadcast reduction of AddBackward (core.rs:195-223).
 * Same results as the corresponding mtb200_gemm / mtb200_colsum calls to within the f32 mode's
 * tolerance.  What the pair adds is shared operand preparation: the forward call leaves the tensor-core
 * form of x and W (two fp16 planes and one power-of-two exponent per row) in `saved`, a caller-owned
 * block of mtb200_dense_saved_bytes() bytes from mtb200_alloc, and the backward call multiplies
 * against those planes as they lie, folding their row scales into dY, whose maxima, column sums and
 * both plane sets come from two passes over dY.  x, W and `saved` must be unchanged between the two
 * calls.  `saved` may be NULL (and is ignored when mtb200_dense_saved_bytes reports 0: f64, or a
 * dimension of 128 or less): both calls then run as plain products.
 * forward `epilogue`/`aux` as in mtb200_gemm (NONE / RELU / GELU_*); backward `dx_epilogue` is NONE or
 * RELU_BWD with `dx_aux` = the previous layer's activation output [rows][in]. */
int32_t mtb200_dense_saved_bytes(int32_t dtype, int64_t rows, int64_t in_features, int64_t out_features,
                                 size_t* bytes);
int32_t mtb200_dense_forward(mtb200_handle h, int32_t dtype, int64_t rows, int64_t in_features,
                             int64_t out_features, const void* x, const void* W, const void* bias,
                             int32_t epilogue, void* y, void* saved);
int32_t mtb200_dense_backward(mtb200_handle h, int32_t dtype, int64_t rows, int64_t in_features,
                              int64_t out_features, const void* x, const void* W, const void* dY,
                              const void* saved, void* dX, int32_t dx_epilogue, const void* dx_aux,
                              void* dW, void* db, void* dy_block, int32_t dy_mode);
/* dy_block / dy_mode (NULL / 0 for the plain use): data-parallel training wants the chain of input gradients
 * first and the parameter gradients afterwards, largest layer first, so that their all-reduces overlap the
 * remaining products.  A call with dy_mode 1 (dW NULL) computes dX and db and also leaves dY's prepared
 * weight-gradient operand in dy_block (mtb200_dense_dy_bytes bytes, caller-owned); a later call with dy_mode 2
 * (dX and db NULL) computes dW from that block without reading dY again.  dY, x and the block must be unchanged
 * in between.  Ignored (plain products) where mtb200_dense_saved_bytes reports 0. */
int32_t mtb200_dense_dy_bytes(int32_t dtype, int64_t rows, int64_t in_features, int64_t out_features,
                              size_t* bytes);

/* ---- bias gradient: out[n] = sum_m X[m][n]  (f32 / f64)
 * reduce_gradient_for_broadcasting -> sum over dim 0
 * (engine/src/autograd/mod/tests.rs:8-68, engine/src/operations/reduction/sum_prod.rs:7-84).
 * Deterministic: the same input always gives the same bits. */
int32_t mtb200_colsum(mtb200_handle h, int32_t dtype, int64_t M, int64_t N, const void* X, void* out);

/* ---- bias gradient for callers that must not allocate.  (No counterpart in the
 * reference: its CPU engine sums into a freshly allocated tensor.)
 * Same result as mtb200_colsum, but the partial sums live in a fixed array
 * inside the library instead of the handle's growable workspace, so the call
 * never reaches cudaMalloc / cudaFree (nor their device-wide synchronisation)
 * and needs no handle: work is enqueued on `cuda_stream` of the CURRENT device.
 * Meant for callers that run where allocation is off limits: inside an
 * application whose own pool owns all device memory (minitensor's memory
 * manager is one), or in a loop that cannot afford the device-wide stall of
 * cudaMalloc / cudaFree.
 * Limits and rules:
 *  - N * sizeof(element) must not exceed MTB200_COLSUM_NOALLOC_SCRATCH_BYTES
 *    (1,048,576 f32 or 524,288 f64 columns); wider inputs are rejected with
 *    MTB200_ERR_INVALID.  Every GPU that loads the library holds that array
 *    until the process exits.
 *  - The first call on each device looks the array's device address up
 *    (cudaGetSymbolAddress); make that first call before starting any stream
 *    capture.
 *  - All calls share the one array.  Each call overwrites what it reads, so
 *    stale contents are harmless, but two calls that may run on the GPU at
 *    the same time (different streams, no ordering between them) race. */
#define MTB200_COLSUM_NOALLOC_SCRATCH_BYTES (4u << 20)
int32_t mtb200_colsum_noalloc(void* cuda_stream, int32_t dtype, int64_t M, int64_t N, const void* X,
                              void* out);

/* ---- activations outside a GEMM (f32 / f64); act uses the MTB200_EPI_* numbers 1..3.
 * forward: relu / gelu (engine/src/operations/activation/trigonometry.rs:308-344,499-544).
 * backward: dx = dy * f'; `ref` is the activation OUTPUT for relu and the
 * activation INPUT for gelu (engine/src/autograd/mod/shape.rs:724-816,
 * engine/src/autograd/mod/linalg.rs:118-264). */
int32_t mtb200_act_fwd(mtb200_handle h, int32_t dtype, int32_t act, int64_t n, const void* x, void* y);
int32_t mtb200_act_bwd(mtb200_handle h, int32_t dtype, int32_t act, int64_t n, const void* ref,
                       const void* dy, void* dx);

/* ---- broadcast bias add with optional activation: y[m][n] = act(x[m][n] + bias[n])
 * the [M,N] + [N] case of arithmetic::add that DenseLayer uses
 * (engine/src/operations/arithmetic/kernels.rs:191-334, engine/src/nn/dense_layer.rs:163-166).
 * act: 0 none or MTB200_EPI_RELU / GELU_ERF / GELU_TANH.  x and y may alias. */
int32_t mtb200_bias_act(mtb200_handle h, int32_t dtype, int64_t M, int64_t N, const void* x,
                        const void* bias, int32_t act, void* y);

/* ---- cross entropy with class-index targets, reduction "mean" | "sum"
 * cross_entropy_loss + CrossEntropyLossBackward
 * (engine/src/operations/loss/regression.rs:178-251,769-862,
 *  engine/src/autograd/mod/activation.rs:364-427).
 * logits f32 [B,C]; labels int32 (label_dtype = MTB200_I32) or int64
 * (MTB200_I64), [B].  loss: 1 float (device).  dlogits: [B,C] or NULL, receives
 * (softmax - onehot) * (mean ? 1/B : 1) * upstream.  A label outside [0,C) is
 * reported by the next mtb200_sync as MTB200_ERR_BAD_LABEL. */
int32_t mtb200_cross_entropy(mtb200_handle h, int64_t B, int64_t C, const float* logits,
                             const void* labels, int32_t label_dtype, int32_t mean,
                             float upstream, float* loss, float* dlogits);

/* ---- Adam / AdamW step over one flat f32 buffer
 * Adam::apply_adam_update without amsgrad (engine/src/optim/adam.rs:245-312).
 * step is the 1-based step count after the increment (adam.rs:261-266).
 * grad_scale multiplies the gradient first (1.0 = reference behaviour). */
int32_t mtb200_adam_step(mtb200_handle h, int64_t n, float* param, const float* grad, float* m,
                         float* v, double lr, double beta1, double beta2, double eps,
                         double weight_decay, int32_t decoupled, int64_t step, float grad_scale);

/* ---- cross entropy, general form (f32 logits [B,C])
 * cross_entropy_loss (engine/src/operations/loss/regression.rs:178-251) with either kind of target it
 * accepts - class indices [B] (target_dtype MTB200_I32 / MTB200_I64; made one-hot at :769-862) or a
 * [B,C] float32 probability matrix (target_dtype MTB200_F32) - and its three reductions.
 * loss: 1 float for SUM / MEAN, B floats for NONE.  dlogits (nullable) receives
 * (softmax - target) * (MEAN ? 1/B : 1) * upstream * (upstream_rows ? upstream_rows[b] : 1)
 * (CrossEntropyLossBackward, engine/src/autograd/mod/activation.rs:364-427; upstream_rows is the
 * per-sample gradient of a NONE loss - the reference multiplies by grad_output through its generic
 * broadcast, which for a [B] gradient only type-checks when B == C). */
#define MTB200_REDUCE_SUM 0
#define MTB200_REDUCE_MEAN 1
#define MTB200_REDUCE_NONE 2
int32_t mtb200_cross_entropy_ex(mtb200_handle h, int64_t B, int64_t C, const float* logits,
                                const void* targets, int32_t target_dtype, int32_t reduction,
                                float upstream, const float* upstream_rows, float* loss, float* dlogits);

/* ---- SGD step over one flat buffer (f32 / f64), in place
 * SGD::apply_simple_update / apply_momentum_update (engine/src/optim/sgd.rs:169-296):
 *   g' = g + weight_decay*p;  momentum > 0: v = momentum*v + (1-dampening)*g',
 *   p -= lr*(nesterov ? g' + momentum*v : v);  otherwise p -= lr*g' (velocity may be NULL).
 * Bit-identical to the CPU arithmetic (same operation order, no fused multiply-add). */
int32_t mtb200_sgd_step(mtb200_handle h, int32_t dtype, int64_t n, void* param, const void* grad,
                        void* velocity, double lr, double momentum, double dampening,
                        double weight_decay, int32_t nesterov);

/* ---- RMSprop step (f32 / f64), in place
 * RMSprop::apply_rmsprop_update (engine/src/optim/rmsprop.rs:187-383):
 *   g' = g + weight_decay*p;  sq = alpha*sq + (1-alpha)*g'*g';
 *   grad_avg != NULL (centered): ga = alpha*ga + (1-alpha)*g', denom = sqrt(sq - ga*ga) + eps,
 *   else denom = sqrt(sq) + eps;  momentum > 0: mb = momentum*mb + lr*g'/denom, p -= mb;
 *   else p -= lr*g'/denom (momentum_buf may be NULL).  Bit-identical to the CPU arithmetic. */
int32_t mtb200_rmsprop_step(mtb200_handle h, int32_t dtype, int64_t n, void* param, const void* grad,
                            void* square_avg, void* momentum_buf, void* grad_avg, double lr,
                            double alpha, double eps, double weight_decay, double momentum);

/* ---- gradient clipping building blocks (f32 / f64)
 * GradientUtils::compute_grad_norm_value / clip_grad_norm / clip_grad_value
 * (engine/src/optim/utils.rs:16-112).
 * sumsq: *out (one DEVICE double) = [*out +] sum of x[i]^2 accumulated in f64, deterministic; the
 *        caller takes the square root of the total over all parameters and, when it exceeds
 *        max_norm, scales every gradient by max_norm / (norm + 1e-6).
 * scale: x[i] *= (element type)coef.   clamp: x[i] = clamp(x[i], lo, hi), NaN stays NaN. */
int32_t mtb200_sumsq(mtb200_handle h, int32_t dtype, int64_t n, const void* x, double* out,
                     int32_t accumulate);
int32_t mtb200_scale(mtb200_handle h, int32_t dtype, int64_t n, void* x, double coef);
int32_t mtb200_clamp(mtb200_handle h, int32_t dtype, int64_t n, void* x, double lo, double hi);

/* ---- the tape's own elementwise and layout operations
 * add_inplace: y[i] += x[i], f32 / f64 / i32 / i64 (integers wrap): gradient accumulation,
 *   arithmetic::add_inplace (engine/src/operations/arithmetic/elementwise.rs:102-160) as called by
 *   accumulate_grad (engine/src/autograd/mod/core.rs:168, engine/src/autograd/graph.rs:266).
 * swap_dims: materialised transpose (engine/src/operations/linalg/diagonal.rs:8-108).  x is read as
 *   [outer][d0][mid][d1][inner] and written as [outer][d1][mid][d0][inner]; elements are moved, not
 *   interpreted (elem_bytes 4 or 8).  transpose(dim0, dim1) of a tensor is outer = product of the
 *   dimensions before dim0, mid = of those between, inner = of those after dim1.  Not in place. */
int32_t mtb200_add_inplace(mtb200_handle h, int32_t dtype, int64_t n, void* y, const void* x);
int32_t mtb200_swap_dims(mtb200_handle h, int32_t elem_bytes, int64_t outer, int64_t d0, int64_t mid,
                         int64_t d1, int64_t inner, const void* x, void* y);

/* ---- batch normalisation (f32 / f64) on x[N][C][S], S = product of the dimensions after the channel
 * batch_norm (engine/src/operations/normalization.rs:64-187; layers engine/src/nn/normalization.rs).
 * forward: statistics per channel over N and S (biased variance) when `training` or when a running
 *   estimate is NULL, else the running estimates; y = (x - mean) / sqrt(var + eps) * weight + bias
 *   (weight / bias nullable); while training, running = running*(1-momentum) + batch*momentum.
 *   save_mean / save_invstd (C elements each, nullable) receive what the backward call needs.
 * backward: the gradient of that composition, which the reference obtains operator by operator:
 *   dbias = sum dy, dweight = sum dy*xhat, dx = weight*invstd*(dy - dbias/n - xhat*dweight/n) when the
 *   forward used batch statistics (batch_stats != 0), weight*invstd*dy otherwise.  Outputs nullable.
 * Sums are accumulated in f64 in a fixed order (deterministic). */
int32_t mtb200_batch_norm_fwd(mtb200_handle h, int32_t dtype, int64_t N, int64_t C, int64_t S,
                              const void* x, const void* weight, const void* bias, void* running_mean,
                              void* running_var, int32_t training, double momentum, double eps, void* y,
                              void* save_mean, void* save_invstd);
int32_t mtb200_batch_norm_bwd(mtb200_handle h, int32_t dtype, int64_t N, int64_t C, int64_t S,
                              const void* x, const void* dy, const void* weight, const void* save_mean,
                              const void* save_invstd, int32_t batch_stats, void* dx, void* dweight,
                              void* dbias);

/* ---- dropout (f32 / f64)
 * generate_dropout_mask + the element-wise product of Dropout / Dropout2d::forward
 * (engine/src/nn/dropout.rs:21-92,164-187,258-289).
 * mask[j] = 1/(1-p) with probability 1-p, else 0 (all ones for p = 0, zeros for p = 1).  The reference
 * draws from its thread-local StdRng, whose stream cannot be reproduced outside it; here, with
 * g = offset + j, entry j keeps when a 24-bit field of mix64(seed + (g/2 + 1) * 0x9E3779B97F4A7C15) -
 * bits 63..40 for even g, bits 39..16 for odd g; mix64 = the splitmix64 finaliser - is below
 * (1-p)*2^24, so a mask is a pure function of (seed, offset, j).
 * dropout_apply: y[i] = x[i] * mask[i / inner] with the entries generated on the fly (one read, one
 *   write, no mask tensor) - inner = 1 for Dropout, H*W for Dropout2d (mask [N][C]); the backward pass is
 *   the same call on the upstream gradient with the same (seed, offset).
 * dropout_mask / mask_mul: the same mask materialised, and the product with a stored mask. */
int32_t mtb200_dropout_apply(mtb200_handle h, int32_t dtype, int64_t n, int64_t inner, const void* x,
                             double p, uint64_t seed, uint64_t offset, void* y);
int32_t mtb200_dropout_mask(mtb200_handle h, int32_t dtype, int64_t n, double p, uint64_t seed,
                            uint64_t offset, void* mask);
int32_t mtb200_mask_mul(mtb200_handle h, int32_t dtype, int64_t n, int64_t inner, const void* x,
                        const void* mask, void* y);

/* ---- the same Adam step with its step count in device memory.  (No counterpart in the reference, whose
 * optimizer keeps the count on the host.)  For training loops replayed from a CUDA graph: a graph freezes
 * kernel arguments, so the bias corrections 1/(1 - beta^t) are computed on the device from
 * *step_counter (one int64 in device memory, 0 before the first step), with the host's own sequence of
 * f64 products, hence the same bits as mtb200_adam_step(step = t).  advance != 0 increments the
 * counter before the update (pass it on the first parameter buffer of a step only). */
int32_t mtb200_adam_step_counted(mtb200_handle h, int64_t n, float* param, const float* grad, float* m,
                                 float* v, double lr, double beta1, double beta2, double eps,
                                 double weight_decay, int32_t decoupled, int64_t* step_counter,
                                 int32_t advance, float grad_scale);

/* ---- conv2d, NCHW input, OIHW weight, f32 (the reference supports nothing
 * else: engine/src/operations/conv.rs:85-93,202-204).
 * forward  = conv2d                     engine/src/operations/conv.rs:24-206
 * bwd_data / bwd_weight / bwd_bias = Conv2dBackward  engine/src/autograd/mod/shape.rs:57-197
 * f32_mode: MTB200_F32_DEFAULT = F16X3 wherever the implicit kernels run - forward, data gradient
 * and weight gradient, stride 1 or strided up to 8 (one power-of-two scale per image and per weight
 * row; per tensor for the weight gradient, whose sums run over images) - and BF16X6 where a layer
 * goes through gathered patches (rows wider than 254 pixels, larger strides); the BF16 modes may be
 * asked for by value.  Inf or NaN in an operand: the call recomputes its result with IEEE multiply-add in
 * the reference's loop order, so non-finite values land where the reference puts them.
 * Variant byte (f32_mode >> 8), for tests: 0xFF the gathered-patch lowering, 0xFB the
 * channels-on-M halo kernel, 0xFC the kernels that load one window per filter tap. */
int32_t mtb200_conv2d_fwd(mtb200_handle h, int64_t n, int64_t c_in, int64_t height, int64_t width,
                          int64_t c_out, int64_t kh, int64_t kw, int64_t stride_h, int64_t stride_w,
                          int64_t pad_h, int64_t pad_w, const float* x, const float* w,
                          const float* bias, float* y, int32_t f32_mode);
int32_t mtb200_conv2d_bwd_data(mtb200_handle h, int64_t n, int64_t c_in, int64_t height,
                               int64_t width, int64_t c_out, int64_t kh, int64_t kw,
                               int64_t stride_h, int64_t stride_w, int64_t pad_h, int64_t pad_w,
                               const float* dy, const float* w, float* dx, int32_t f32_mode);
int32_t mtb200_conv2d_bwd_weight(mtb200_handle h, int64_t n, int64_t c_in, int64_t height,
                                 int64_t width, int64_t c_out, int64_t kh, int64_t kw,
                                 int64_t stride_h, int64_t stride_w, int64_t pad_h, int64_t pad_w,
                                 const float* dy, const float* x, float* dw, int32_t f32_mode);
int32_t mtb200_conv2d_bwd_bias(mtb200_handle h, int64_t n, int64_t c_out, int64_t out_h,
                               int64_t out_w, const float* dy, float* db);

/* ---- gradient exchange of data-parallel training: all-reduce (sum) of f32 buffers over NCCL.
 * The reference has no distributed code.  The step this exchange is inserted into is its
 * single-process training loop (backward engine/src/autograd/graph.rs:222-282, then
 * Adam::step engine/src/optim/adam.rs:483-514): every rank runs that step on its own rows of the
 * batch, the parameter gradients are summed over the ranks between backward and the optimizer, and
 * the optimizer applies 1 / world_size (grad_scale of mtb200_adam_step), so all replicas stay equal.
 * NCCL is looked up at run time (the copy already loaded into the process, else libnccl.so.2 on the
 * loader path, else the file named by the environment variable MTB200_NCCL_LIB); without it these
 * calls return MTB200_ERR_UNSUPPORTED and everything else still works.
 *
 * Two ways to form the communicator:
 *  - one process per GPU: rank 0 calls mtb200_comm_unique_id and hands the MTB200_COMM_ID_BYTES bytes to
 *    every rank (any channel: a file, a socket, MPI); each rank then calls mtb200_comm_init_rank, which
 *    blocks until all world_size ranks have called it;
 *  - one process driving ndev GPUs: mtb200_comm_init(ndev, devs); rank i is devs[i], and the
 *    per-rank calls of one exchange are bracketed by mtb200_comm_group_begin / _end.
 * mtb200_allreduce_sum_f32 enqueues, on the stream set for `rank` (mtb200_comm_set_stream; default: the
 * CUDA default stream), buf[i] = scale * sum over ranks of buf[i] for i < n, in place.  Every rank must
 * issue the same sequence of exchanges with the same n.  scale == 1 skips the multiply.  Asynchronous:
 * ordered after earlier work on that stream; synchronise the stream (or order another stream after it)
 * before reading buf. */
/* A communicator is created with a budget of 16 CTAs for NCCL (through NCCL_MAX_CTAS, unless the host has set
 * that variable itself; MTB200_COMM_CTAS=n changes the budget, 0 leaves NCCL alone): the collectives run beside
 * persistent tensor kernels and must fit in the SMs those leave free. */
typedef struct mtb200_comm_s* mtb200_comm;
#define MTB200_COMM_ID_BYTES 128
int32_t mtb200_comm_unique_id(void* id_out);
int32_t mtb200_comm_init_rank(int32_t world_size, int32_t rank, const void* id, int32_t device_ordinal,
                              mtb200_comm* out);
int32_t mtb200_comm_init(int32_t ndev, const int32_t* devs, mtb200_comm* out);
int32_t mtb200_comm_set_stream(mtb200_comm c, int32_t rank, void* cuda_stream);
int32_t mtb200_comm_group_begin(mtb200_comm c);
int32_t mtb200_comm_group_end(mtb200_comm c);
int32_t mtb200_allreduce_sum_f32(mtb200_comm c, int32_t rank, float* buf, size_t n, float scale);
int32_t mtb200_comm_destroy(mtb200_comm c);

/* ---- self-test of the bounded waits.  (No counterpart in the reference.)
 * Every wait inside the tensor-core kernels (on a shared-memory barrier that a TMA load or an MMA
 * completion signals) gives up after a time limit, records a code in the handle's status word and lets
 * the kernel wind down; mtb200_sync then returns MTB200_ERR_DEVICE_WAIT once and clears the word.  This
 * call exercises exactly that path without any fault: it launches one small block that waits, with a
 * limit of `limit_us` microseconds (1 .. 100000), on a barrier nothing ever signals, and records the
 * expiry the way the GEMM kernels do.  The context stays usable. */
int32_t mtb200_selftest_wait_expiry(mtb200_handle h, int32_t limit_us);

#ifdef __cplusplus
}
#endif
#endif /* MTB200_H_ */
