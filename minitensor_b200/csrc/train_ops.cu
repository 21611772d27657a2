// Training-step operators beside the GEMMs, kept on the device so a step makes no host round trip:
// SGD, RMSprop, gradient clipping (sum of squares, scale, clamp) and cross entropy in its general form
// (class-index or probability targets; reductions sum / mean / none).  All are one pass over their
// operands (HBM-bound).  The optimizers repeat the reference's per-element operation order with
// separately rounded operations (no fused multiply-add), so f32 and f64 results are bit-identical to
// the CPU arithmetic.
#include "mtb200_core.cuh"

#include <algorithm>
#include <cmath>

namespace mtb {

// separately rounded arithmetic for both floating types
__device__ __forceinline__ float r_mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float r_add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float r_sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float r_div(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ float r_sqrt(float a) { return __fsqrt_rn(a); }
__device__ __forceinline__ double r_mul(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ double r_add(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ double r_sub(double a, double b) { return __dsub_rn(a, b); }
__device__ __forceinline__ double r_div(double a, double b) { return __ddiv_rn(a, b); }
__device__ __forceinline__ double r_sqrt(double a) { return __dsqrt_rn(a); }

static inline int ew_grid(long long n, int sm_count) {
  const long long blocks = (n + 255) / 256;
  return int(std::max<long long>(1, std::min<long long>(blocks, (long long)sm_count * 16)));
}

// SGD::apply_simple_update / apply_momentum_update (engine/src/optim/sgd.rs:169-296):
//   g' = g + wd*p ;  v = momentum*v + (1-dampening)*g' ;  p -= lr * (nesterov ? g' + momentum*v : v)
//   without momentum: p -= lr*g'
template <typename T>
static __global__ void sgd_kernel(T* __restrict__ p, const T* __restrict__ g, T* __restrict__ v, long long n, T lr,
                                  T momentum, T damp, T wd, int use_momentum, int nesterov) {
  const T omd = r_sub(T(1), damp);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const T pi = p[i];
    const T gv = r_add(g[i], r_mul(wd, pi));
    if (use_momentum) {
      const T vi = r_add(r_mul(momentum, v[i]), r_mul(omd, gv));
      v[i] = vi;
      const T update = nesterov ? r_add(gv, r_mul(momentum, vi)) : vi;
      p[i] = r_sub(pi, r_mul(lr, update));
    } else {
      p[i] = r_sub(pi, r_mul(lr, gv));
    }
  }
}

// RMSprop::apply_rmsprop_update (engine/src/optim/rmsprop.rs:187-383):
//   g' = g + wd*p ;  sq = alpha*sq + (1-alpha)*g'*g' ;  centered: ga = alpha*ga + (1-alpha)*g', avg = sq - ga*ga
//   denom = sqrt(avg) + eps ;  momentum: mb = momentum*mb + lr*g'/denom, p -= mb ;  else p -= lr*g'/denom
template <typename T>
static __global__ void rmsprop_kernel(T* __restrict__ p, const T* __restrict__ g, T* __restrict__ sq,
                                      T* __restrict__ mb, T* __restrict__ ga, long long n, T lr, T alpha, T eps,
                                      T wd, T momentum) {
  const T oma = r_sub(T(1), alpha);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const T pi = p[i];
    const T gv = r_add(g[i], r_mul(wd, pi));
    const T sqi = r_add(r_mul(alpha, sq[i]), r_mul(r_mul(oma, gv), gv));
    sq[i] = sqi;
    T avg = sqi;
    if (ga) {
      const T gai = r_add(r_mul(alpha, ga[i]), r_mul(oma, gv));
      ga[i] = gai;
      avg = r_sub(sqi, r_mul(gai, gai));
    }
    const T denom = r_add(r_sqrt(avg), eps);
    const T stepv = r_div(r_mul(lr, gv), denom);
    if (mb) {
      const T mbi = r_add(r_mul(momentum, mb[i]), stepv);
      mb[i] = mbi;
      p[i] = r_sub(pi, mbi);
    } else {
      p[i] = r_sub(pi, stepv);
    }
  }
}

// Sum of squares in f64 (GradientUtils::compute_grad_norm_value, engine/src/optim/utils.rs:16-44).
// Stage 1: block b sums its contiguous slice (fixed thread assignment, fixed tree); stage 2: one block
// folds the partials in a fixed tree.  The same input always gives the same bits.
constexpr int SUMSQ_BLOCKS = 1024;
template <typename T>
static __global__ void __launch_bounds__(256) sumsq_stage1_kernel(const T* __restrict__ x, long long n,
                                                                   double* __restrict__ partial) {
  __shared__ double red[256];
  const long long per = (n + gridDim.x - 1) / gridDim.x;
  const long long lo = blockIdx.x * per, hi = min(n, lo + per);
  double s = 0.0;
  for (long long i = lo + threadIdx.x; i < hi; i += 256) {
    const double v = static_cast<double>(x[i]);
    s += v * v;
  }
  red[threadIdx.x] = s;
  __syncthreads();
  for (int o = 128; o; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) partial[blockIdx.x] = red[0];
}
static __global__ void __launch_bounds__(1024) sumsq_stage2_kernel(const double* __restrict__ partial, int count,
                                                                   double* __restrict__ out, int accumulate) {
  __shared__ double red[1024];
  red[threadIdx.x] = threadIdx.x < count ? partial[threadIdx.x] : 0.0;
  __syncthreads();
  for (int o = 512; o; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) *out = accumulate ? *out + red[0] : red[0];
}

template <typename T>
static __global__ void scale_kernel(T* __restrict__ x, long long n, T coef) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    x[i] = r_mul(x[i], coef);
}
// clamp as f32::clamp / f64::clamp: NaN stays NaN (engine/src/optim/utils.rs:83-112)
template <typename T>
static __global__ void clamp_kernel(T* __restrict__ x, long long n, T lo, T hi) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const T v = x[i];
    x[i] = v < lo ? lo : (v > hi ? hi : v);
  }
}

// Cross entropy, general form: one warp per sample row (engine/src/operations/loss/regression.rs:178-251).
// Targets: class indices (LabelT = int / long long, `soft` null) or a [B][C] probability matrix (`soft`).
// log-softmax by max shift, softmax = exp(log-softmax), entries with softmax <= 1e-30 take log-probability
// -inf before the product with the target row (so -inf * 0 = NaN, as in the reference).  row_loss[b] = the
// sample's loss; gradient (softmax - target) * grad_scale * (row_scale ? row_scale[b] : 1).
template <typename LabelT>
static __global__ void __launch_bounds__(256) cross_entropy_general_kernel(
    const float* __restrict__ logits, const LabelT* __restrict__ labels, const float* __restrict__ soft, int B, int C,
    float grad_scale, const float* __restrict__ row_scale, float* __restrict__ row_loss, float* __restrict__ dlogits,
    uint32_t* __restrict__ bad_label) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= B) return;
  const float* x = logits + static_cast<long long>(warp) * C;
  const float* t = soft ? soft + static_cast<long long>(warp) * C : nullptr;
  long long lab = -1;
  if (!soft) {
    lab = static_cast<long long>(labels[warp]);
    if (lab < 0 || lab >= C) {
      if (lane == 0) atomicOr(bad_label, 1u);
      lab = -1;
    }
  }
  float mx = -INFINITY;
  for (int c = lane; c < C; c += 32) mx = fmaxf(mx, x[c]);
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float s = 0.0f;
  for (int c = lane; c < C; c += 32) s += expf(x[c] - mx);
#pragma unroll
  for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const bool all_neg_inf = (mx == -INFINITY);
  const float logsum = logf(s) + mx;
  const float gs = row_scale ? grad_scale * row_scale[warp] : grad_scale;
  float acc = 0.0f;  // sum of -(masked log-probability * target) over this lane's classes
  for (int c = lane; c < C; c += 32) {
    const float lp = all_neg_inf ? -INFINITY : x[c] - logsum;
    const float sm = expf(lp);
    const float tc = soft ? t[c] : (c == lab ? 1.0f : 0.0f);
    const float lpm = (sm <= 1e-30f) ? -INFINITY : lp;
    acc += -(lpm * tc);
    if (dlogits) dlogits[static_cast<long long>(warp) * C + c] = (sm - tc) * gs;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) row_loss[warp] = acc;
}

static __global__ void __launch_bounds__(1024) row_loss_reduce_kernel(const float* __restrict__ row_loss, int B,
                                                                      float inv_count, float* __restrict__ loss) {
  __shared__ float red[1024];
  float s = 0.0f;
  for (int i = threadIdx.x; i < B; i += 1024) s += row_loss[i];
  red[threadIdx.x] = s;
  __syncthreads();
  for (int o = 512; o; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) *loss = red[0] * inv_count;
}

}  // namespace mtb

using namespace mtb;

#define MTB_CHECK_HANDLE(h)                                         \
  if (!(h)) return fail(MTB200_ERR_INVALID, "null handle");         \
  DeviceGuard guard__((h)->device);                                 \
  if (!guard__.ok) return fail(MTB200_ERR_CUDA, "cannot make device %d current", (h)->device)

static int32_t check_float_dtype(int32_t dtype, const char* what) {
  if (dtype != MTB200_F32 && dtype != MTB200_F64)
    return fail(MTB200_ERR_UNSUPPORTED, "%s only supports float32/float64 tensors (dtype %d)", what, dtype);
  return MTB200_OK;
}

extern "C" {

int32_t mtb200_sgd_step(mtb200_handle h, int32_t dtype, int64_t n, void* param, const void* grad, void* velocity,
                        double lr, double momentum, double dampening, double weight_decay, int32_t nesterov) {
  MTB_CHECK_HANDLE(h);
  if (int32_t rc = check_float_dtype(dtype, "SGD")) return rc;
  if (n < 0) return fail(MTB200_ERR_INVALID, "negative length");
  if (n == 0) return MTB200_OK;
  const int use_momentum = momentum > 0.0 ? 1 : 0;  // sgd.rs:323
  if (!param || !grad || (use_momentum && !velocity)) return fail(MTB200_ERR_INVALID, "null pointer");
  const int grid = ew_grid(n, h->sm_count);
  if (dtype == MTB200_F32)
    sgd_kernel<float><<<grid, 256, 0, h->stream>>>(static_cast<float*>(param), static_cast<const float*>(grad),
                                                   static_cast<float*>(velocity), n, float(lr), float(momentum),
                                                   float(dampening), float(weight_decay), use_momentum, nesterov);
  else
    sgd_kernel<double><<<grid, 256, 0, h->stream>>>(static_cast<double*>(param), static_cast<const double*>(grad),
                                                    static_cast<double*>(velocity), n, lr, momentum, dampening,
                                                    weight_decay, use_momentum, nesterov);
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

int32_t mtb200_rmsprop_step(mtb200_handle h, int32_t dtype, int64_t n, void* param, const void* grad,
                            void* square_avg, void* momentum_buf, void* grad_avg, double lr, double alpha,
                            double eps, double weight_decay, double momentum) {
  MTB_CHECK_HANDLE(h);
  if (int32_t rc = check_float_dtype(dtype, "RMSprop")) return rc;
  if (n < 0) return fail(MTB200_ERR_INVALID, "negative length");
  if (n == 0) return MTB200_OK;
  if (!param || !grad || !square_avg) return fail(MTB200_ERR_INVALID, "null pointer");
  if (momentum > 0.0 && !momentum_buf) return fail(MTB200_ERR_INVALID, "momentum > 0 needs a momentum buffer");
  if (!(momentum > 0.0)) momentum_buf = nullptr;  // rmsprop.rs:202
  const int grid = ew_grid(n, h->sm_count);
  if (dtype == MTB200_F32)
    rmsprop_kernel<float><<<grid, 256, 0, h->stream>>>(
        static_cast<float*>(param), static_cast<const float*>(grad), static_cast<float*>(square_avg),
        static_cast<float*>(momentum_buf), static_cast<float*>(grad_avg), n, float(lr), float(alpha), float(eps),
        float(weight_decay), float(momentum));
  else
    rmsprop_kernel<double><<<grid, 256, 0, h->stream>>>(
        static_cast<double*>(param), static_cast<const double*>(grad), static_cast<double*>(square_avg),
        static_cast<double*>(momentum_buf), static_cast<double*>(grad_avg), n, lr, alpha, eps, weight_decay, momentum);
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

int32_t mtb200_sumsq(mtb200_handle h, int32_t dtype, int64_t n, const void* x, double* out, int32_t accumulate) {
  MTB_CHECK_HANDLE(h);
  if (int32_t rc = check_float_dtype(dtype, "gradient norm")) return rc;
  if (n < 0) return fail(MTB200_ERR_INVALID, "negative length");
  if (!out) return fail(MTB200_ERR_INVALID, "null output pointer");
  if (n == 0) {
    if (!accumulate) MTB_CUDA(cudaMemsetAsync(out, 0, sizeof(double), h->stream));
    return MTB200_OK;
  }
  if (!x) return fail(MTB200_ERR_INVALID, "null input pointer");
  const int blocks = int(std::min<int64_t>(SUMSQ_BLOCKS, (n + 255) / 256));
  void* ws = nullptr;
  int32_t rc = workspace_reserve(h, sizeof(double) * SUMSQ_BLOCKS, &ws);
  if (rc) return rc;
  if (dtype == MTB200_F32)
    sumsq_stage1_kernel<float><<<blocks, 256, 0, h->stream>>>(static_cast<const float*>(x), n, static_cast<double*>(ws));
  else
    sumsq_stage1_kernel<double><<<blocks, 256, 0, h->stream>>>(static_cast<const double*>(x), n, static_cast<double*>(ws));
  sumsq_stage2_kernel<<<1, 1024, 0, h->stream>>>(static_cast<const double*>(ws), blocks, out, accumulate);
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

int32_t mtb200_scale(mtb200_handle h, int32_t dtype, int64_t n, void* x, double coef) {
  MTB_CHECK_HANDLE(h);
  if (int32_t rc = check_float_dtype(dtype, "scale")) return rc;
  if (n < 0) return fail(MTB200_ERR_INVALID, "negative length");
  if (n == 0) return MTB200_OK;
  if (!x) return fail(MTB200_ERR_INVALID, "null pointer");
  const int grid = ew_grid(n, h->sm_count);
  if (dtype == MTB200_F32) scale_kernel<float><<<grid, 256, 0, h->stream>>>(static_cast<float*>(x), n, float(coef));
  else scale_kernel<double><<<grid, 256, 0, h->stream>>>(static_cast<double*>(x), n, coef);
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

int32_t mtb200_clamp(mtb200_handle h, int32_t dtype, int64_t n, void* x, double lo, double hi) {
  MTB_CHECK_HANDLE(h);
  if (int32_t rc = check_float_dtype(dtype, "clamp")) return rc;
  if (n < 0) return fail(MTB200_ERR_INVALID, "negative length");
  if (!(lo <= hi)) return fail(MTB200_ERR_INVALID, "clamp needs min <= max (and neither NaN)");  // clamp's own assertion
  if (n == 0) return MTB200_OK;
  if (!x) return fail(MTB200_ERR_INVALID, "null pointer");
  const int grid = ew_grid(n, h->sm_count);
  if (dtype == MTB200_F32) clamp_kernel<float><<<grid, 256, 0, h->stream>>>(static_cast<float*>(x), n, float(lo), float(hi));
  else clamp_kernel<double><<<grid, 256, 0, h->stream>>>(static_cast<double*>(x), n, lo, hi);
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

int32_t mtb200_cross_entropy_ex(mtb200_handle h, int64_t B, int64_t C, const float* logits, const void* targets,
                                int32_t target_dtype, int32_t reduction, float upstream, const float* upstream_rows,
                                float* loss, float* dlogits) {
  MTB_CHECK_HANDLE(h);
  if (B < 0 || C < 0 || B > INT32_MAX || C > INT32_MAX) return fail(MTB200_ERR_INVALID, "bad dimension");
  if (target_dtype != MTB200_I32 && target_dtype != MTB200_I64 && target_dtype != MTB200_F32)
    return fail(MTB200_ERR_UNSUPPORTED, "targets must be int32 / int64 class indices or float32 probabilities");
  if (reduction < MTB200_REDUCE_SUM || reduction > MTB200_REDUCE_NONE)
    return fail(MTB200_ERR_INVALID, "Invalid reduction mode: %d. Must be 'mean', 'sum', or 'none'", reduction);
  if (!loss) return fail(MTB200_ERR_INVALID, "null loss pointer");
  if (B == 0 || C == 0) {
    // an empty sum; the mean over zero samples is 0/0
    if (reduction != MTB200_REDUCE_NONE) {
      const float v = (reduction == MTB200_REDUCE_MEAN && B == 0) ? NAN : 0.0f;
      MTB_CUDA(cudaMemcpyAsync(loss, &v, sizeof(float), cudaMemcpyHostToDevice, h->stream));
      MTB_CUDA(cudaStreamSynchronize(h->stream));  // v lives on this frame
    } else if (B > 0) {
      MTB_CUDA(cudaMemsetAsync(loss, 0, sizeof(float) * size_t(B), h->stream));
    }
    return MTB200_OK;
  }
  if (!logits || !targets) return fail(MTB200_ERR_INVALID, "null pointer");
  float* row_loss = loss;
  if (reduction != MTB200_REDUCE_NONE) {
    void* ws = nullptr;
    int32_t rc = workspace_reserve(h, sizeof(float) * size_t(B), &ws);
    if (rc) return rc;
    row_loss = static_cast<float*>(ws);
  }
  const float grad_scale = (reduction == MTB200_REDUCE_MEAN ? float(1.0 / double(B)) : 1.0f) * upstream;
  const int blocks = int((B * 32 + 255) / 256);
  uint32_t* bad = h->status + 1;
  if (target_dtype == MTB200_I32)
    cross_entropy_general_kernel<int><<<blocks, 256, 0, h->stream>>>(logits, static_cast<const int*>(targets), nullptr,
                                                                     int(B), int(C), grad_scale, upstream_rows,
                                                                     row_loss, dlogits, bad);
  else if (target_dtype == MTB200_I64)
    cross_entropy_general_kernel<long long><<<blocks, 256, 0, h->stream>>>(
        logits, static_cast<const long long*>(targets), nullptr, int(B), int(C), grad_scale, upstream_rows, row_loss,
        dlogits, bad);
  else
    cross_entropy_general_kernel<int><<<blocks, 256, 0, h->stream>>>(logits, nullptr, static_cast<const float*>(targets),
                                                                     int(B), int(C), grad_scale, upstream_rows,
                                                                     row_loss, dlogits, bad);
  if (reduction != MTB200_REDUCE_NONE)
    row_loss_reduce_kernel<<<1, 1024, 0, h->stream>>>(row_loss, int(B),
                                                      reduction == MTB200_REDUCE_MEAN ? float(1.0 / double(B)) : 1.0f,
                                                      loss);
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

}  // extern "C"
