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

// ------------------------------------------------------------------ batch norm
// batch_norm (engine/src/operations/normalization.rs:64-187) on x [N][C][S]: statistics per channel over N and
// S.  Both reductions of the op are "two sums per channel":
//   forward : sum (x - k), sum (x - k)^2 with k = the channel's first element (a shift that keeps the variance
//             formula free of cancellation);  backward: sum dy, sum dy * xhat, xhat = (x - mean) * invstd.
// They share one kernel pair: per-chunk partial sums in f64 (fixed thread assignment and tree), then a fixed-order
// fold over the chunks.  MODE 0 = forward, 1 = backward.
template <typename T, int MODE>
__device__ __forceinline__ void bn_terms(T xv, T dyv, double a, double b, double& t0, double& t1) {
  if (MODE == 0) {
    const double d = static_cast<double>(xv) - a;
    t0 = d;
    t1 = d * d;
  } else {
    const double xh = (static_cast<double>(xv) - a) * b;
    t0 = static_cast<double>(dyv);
    t1 = static_cast<double>(dyv) * xh;
  }
}

// General layout (S > 1): block (c, chunk) walks j = n * S + s of its chunk; consecutive threads read
// consecutive s.  a_c / b_c: MODE 0 unused (k is read from x); MODE 1 mean / invstd per channel.
template <typename T, int MODE>
static __global__ void __launch_bounds__(256)
bn_reduce_general_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ a_c,
                         const T* __restrict__ b_c, long long N, int C, long long S, long long per_chunk,
                         double* __restrict__ partial) {
  __shared__ double r0[256], r1[256];
  const int c = blockIdx.x, chunk = blockIdx.y;
  const long long total = N * S;
  const long long lo = chunk * per_chunk, hi = min(total, lo + per_chunk);
  const double a = MODE == 0 ? static_cast<double>(x[static_cast<long long>(c) * S]) : static_cast<double>(a_c[c]);
  const double b = MODE == 0 ? 0.0 : static_cast<double>(b_c[c]);
  double s0 = 0.0, s1 = 0.0;
  for (long long j = lo + threadIdx.x; j < hi; j += 256) {
    const long long n = j / S, i = j - n * S;
    const long long k = (n * C + c) * S + i;
    double t0, t1;
    bn_terms<T, MODE>(x[k], MODE == 1 ? dy[k] : T(0), a, b, t0, t1);
    s0 += t0;
    s1 += t1;
  }
  r0[threadIdx.x] = s0;
  r1[threadIdx.x] = s1;
  __syncthreads();
  for (int o = 128; o; o >>= 1) {
    if (threadIdx.x < o) {
      r0[threadIdx.x] += r0[threadIdx.x + o];
      r1[threadIdx.x] += r1[threadIdx.x + o];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    partial[(static_cast<long long>(chunk) * C + c) * 2 + 0] = r0[0];
    partial[(static_cast<long long>(chunk) * C + c) * 2 + 1] = r1[0];
  }
}

// [N][C] layout (S = 1): a warp owns 128 consecutive channels (4 per lane, one 512-byte load per row), the 8 warps
// of a block take rows r, r + 8, ... of the band and are folded through shared memory in a fixed order.
template <typename T, int MODE>
static __global__ void __launch_bounds__(256)
bn_reduce_cols_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ a_c,
                      const T* __restrict__ b_c, long long N, int C, long long rows_per_band,
                      double* __restrict__ partial) {
  __shared__ double red[8][128][2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c0 = blockIdx.x * 128 + lane * 4;
  const int band = blockIdx.y;
  const long long lo = band * rows_per_band, hi = min(N, lo + rows_per_band);
  constexpr int V = 16 / sizeof(T);  // elements per 16-byte vector: 4 (f32) or 2 (f64)
  const bool vec = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((C % V) == 0) && (c0 + 3 < C) &&
                   (MODE == 0 || (reinterpret_cast<uintptr_t>(dy) & 15) == 0);
  double a[4], b[4], s0[4], s1[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = min(c0 + j, C - 1);
    a[j] = MODE == 0 ? static_cast<double>(x[c]) : static_cast<double>(a_c[c]);
    b[j] = MODE == 0 ? 0.0 : static_cast<double>(b_c[c]);
    s0[j] = 0.0;
    s1[j] = 0.0;
  }
  for (long long n = lo + warp; n < hi; n += 8) {
    const long long k = n * C + c0;
    T xv[4], dv[4];
    if (vec) {
#pragma unroll
      for (int q = 0; q < 4 / V; ++q) {
        *reinterpret_cast<uint4*>(xv + q * V) = *reinterpret_cast<const uint4*>(x + k + q * V);
        if (MODE == 1) *reinterpret_cast<uint4*>(dv + q * V) = *reinterpret_cast<const uint4*>(dy + k + q * V);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        xv[j] = (c0 + j < C) ? x[k + j] : T(0);
        dv[j] = (MODE == 1 && c0 + j < C) ? dy[k + j] : T(0);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      double t0, t1;
      bn_terms<T, MODE>(xv[j], MODE == 1 ? dv[j] : T(0), a[j], b[j], t0, t1);
      s0[j] += t0;
      s1[j] += t1;
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    red[warp][lane * 4 + j][0] = s0[j];
    red[warp][lane * 4 + j][1] = s1[j];
  }
  __syncthreads();
  if (threadIdx.x < 128) {
    const int c = blockIdx.x * 128 + threadIdx.x;
    if (c < C) {
      double t0 = red[0][threadIdx.x][0], t1 = red[0][threadIdx.x][1];
#pragma unroll
      for (int k = 1; k < 8; ++k) {
        t0 += red[k][threadIdx.x][0];
        t1 += red[k][threadIdx.x][1];
      }
      partial[(static_cast<long long>(band) * C + c) * 2 + 0] = t0;
      partial[(static_cast<long long>(band) * C + c) * 2 + 1] = t1;
    }
  }
}

// Forward finalize: mean, biased variance, invstd, running estimates (rm = rm*(1-m) + mean*m, likewise the variance).
template <typename T>
static __global__ void bn_finalize_fwd_kernel(const double* __restrict__ partial, int chunks, int C, double count,
                                              const T* __restrict__ x, long long S, double eps, T* __restrict__ mean_out,
                                              T* __restrict__ invstd_out, T* __restrict__ rm, T* __restrict__ rv,
                                              T momentum, T one_minus_momentum) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  double s0 = 0.0, s1 = 0.0;
  for (int k = 0; k < chunks; ++k) {
    s0 += partial[(static_cast<long long>(k) * C + c) * 2 + 0];
    s1 += partial[(static_cast<long long>(k) * C + c) * 2 + 1];
  }
  const double shift = static_cast<double>(x[static_cast<long long>(c) * S]);
  const double md = s0 / count;
  const T mean = static_cast<T>(shift + md);
  const T var = static_cast<T>(fmax(s1 / count - md * md, 0.0));
  mean_out[c] = mean;
  invstd_out[c] = T(1) / r_sqrt(r_add(var, static_cast<T>(eps)));
  if (rm && rv) {
    rm[c] = r_add(r_mul(rm[c], one_minus_momentum), r_mul(mean, momentum));
    rv[c] = r_add(r_mul(rv[c], one_minus_momentum), r_mul(var, momentum));
  }
}
// Evaluation with running estimates: mean = rm, invstd = 1 / sqrt(rv + eps).
template <typename T>
static __global__ void bn_from_running_kernel(const T* __restrict__ rm, const T* __restrict__ rv, int C, double eps,
                                              T* __restrict__ mean_out, T* __restrict__ invstd_out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  mean_out[c] = rm[c];
  invstd_out[c] = T(1) / r_sqrt(r_add(rv[c], static_cast<T>(eps)));
}
// Backward finalize: db = sum dy, dw = sum dy*xhat; sums[c] = (db, dw) kept in f64 for the dx pass.
template <typename T>
static __global__ void bn_finalize_bwd_kernel(const double* __restrict__ partial, int chunks, int C,
                                              double* __restrict__ sums, T* __restrict__ dw, T* __restrict__ db) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  double s0 = 0.0, s1 = 0.0;
  for (int k = 0; k < chunks; ++k) {
    s0 += partial[(static_cast<long long>(k) * C + c) * 2 + 0];
    s1 += partial[(static_cast<long long>(k) * C + c) * 2 + 1];
  }
  sums[2 * c] = s0;
  sums[2 * c + 1] = s1;
  if (db) db[c] = static_cast<T>(s0);
  if (dw) dw[c] = static_cast<T>(s1);
}
// Element pass of both directions, indexed without a division per element: a block owns one channel run -
// S > 1: the S contiguous elements of one (n, c) pair (blockIdx.x = n * C + c; blockIdx.y takes a span of
//        rows_per_band elements of the run, a multiple of 256);
// S = 1: 256 consecutive channels of a band of rows (blockIdx.x = channel block, blockIdx.y = row band).
//   MODE 0 (forward):  y  = (x - mean) * invstd * w + b
//   MODE 1 (backward): dx = w*invstd * (dy - k1 - xhat*k2) with k1 = db/n, k2 = dw/n (batch statistics) or
//                      dx = w*invstd * dy (fixed statistics)
template <typename T, int MODE>
static __global__ void __launch_bounds__(256)
bn_element_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ mean,
                  const T* __restrict__ invstd, const T* __restrict__ w, const T* __restrict__ b,
                  const double* __restrict__ sums, double inv_count, int batch_stats, long long N, int C, long long S,
                  long long rows_per_band, T* __restrict__ out) {
  int c;
  long long first, count, stride;
  if (S == 1) {
    c = blockIdx.x * 256 + threadIdx.x;
    if (c >= C) return;
    const long long lo = blockIdx.y * rows_per_band, hi = min(N, lo + rows_per_band);
    first = lo * C + c;
    count = hi - lo;
    stride = C;
  } else {
    c = static_cast<int>(blockIdx.x % C);
    const long long begin = blockIdx.y * rows_per_band + threadIdx.x;
    const long long end = min(S, (blockIdx.y + 1LL) * rows_per_band);
    first = static_cast<long long>(blockIdx.x) * S + begin;
    count = begin < end ? (end - begin + 255) / 256 : 0;
    stride = 256;
  }
  const T mu = mean[c], is = invstd[c];
  const T wc = w ? w[c] : T(1);
  if (MODE == 0) {
    const T bc = b ? b[c] : T(0);
    for (long long k = 0, i = first; k < count; ++k, i += stride) {
      T o = (x[i] - mu) * is;
      if (w) o = o * wc;
      if (b) o = o + bc;
      out[i] = o;
    }
  } else {
    const T g = wc * is;
    const T k1 = batch_stats ? static_cast<T>(sums[2 * c] * inv_count) : T(0);
    const T k2 = batch_stats ? static_cast<T>(sums[2 * c + 1] * inv_count) : T(0);
    for (long long k = 0, i = first; k < count; ++k, i += stride) {
      T v = dy[i];
      if (batch_stats) v = v - k1 - ((x[i] - mu) * is) * k2;
      out[i] = g * v;
    }
  }
}

template <typename T, int MODE>
static int32_t bn_element_launch(mtb200_ctx* h, const T* x, const T* dy, const T* mean, const T* invstd, const T* w,
                                 const T* b, const double* sums, double inv_count, int batch_stats, int64_t N, int64_t C,
                                 int64_t S, T* out) {
  if (S == 1) {
    const int64_t cb = (C + 255) / 256;
    int64_t bands = std::max<int64_t>(1, std::min<int64_t>((N + 15) / 16, (int64_t(h->sm_count) * 16) / cb));
    bands = std::min<int64_t>(bands, 65535);
    const int64_t rpb = (N + bands - 1) / bands;
    bn_element_kernel<T, MODE><<<dim3(unsigned(cb), unsigned((N + rpb - 1) / rpb)), 256, 0, h->stream>>>(
        x, dy, mean, invstd, w, b, sums, inv_count, batch_stats, N, int(C), S, rpb, out);
  } else {
    // (n, c) pairs on grid.x (limit 2^31 - 1, checked by bn_check_dims before anything was launched); the run of S
    // elements is cut into at most 65535 spans of a multiple of 256 elements, about 1024 each when S allows
    const int64_t spans = std::min<int64_t>((S + 1023) / 1024, 65535);
    const int64_t span = ((S + spans - 1) / spans + 255) / 256 * 256;
    bn_element_kernel<T, MODE><<<dim3(unsigned(N * C), unsigned((S + span - 1) / span)), 256, 0, h->stream>>>(
        x, dy, mean, invstd, w, b, sums, inv_count, batch_stats, N, int(C), S, span, out);
  }
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

// ------------------------------------------------------------------ dropout
// Mask of generate_dropout_mask (engine/src/nn/dropout.rs:21-92): 1/(1-p) with probability 1-p, else 0.  With
// g = offset + j, entry j keeps when a 24-bit field of mix64(seed + (g / 2 + 1) * 0x9E3779B97F4A7C15) - bits 63..40
// for even g, 39..16 for odd g; mix64 = the splitmix64 finaliser - is below keep * 2^24: a counter-based stream, so
// any entry can be regenerated from (seed, offset) and no mask tensor needs to exist.
// y[i] = x[i] * mask[i / inner]; inner = 1 for Dropout, H*W for Dropout2d (one entry per (sample, channel)).
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}
__device__ __forceinline__ unsigned long long dropout_hash(unsigned long long seed, unsigned long long pair) {
  return mix64(seed + (pair + 1ULL) * 0x9E3779B97F4A7C15ULL);
}
template <typename T>
__device__ __forceinline__ T dropout_entry(unsigned long long seed, unsigned long long g, double keep, unsigned int thresh,
                                           T scale) {
  if (keep >= 1.0) return T(1);
  if (keep <= 0.0) return T(0);
  const unsigned long long hsh = dropout_hash(seed, g >> 1);
  const unsigned int u = static_cast<unsigned int>((g & 1ULL) ? (hsh >> 16) : (hsh >> 40)) & 0xFFFFFFu;
  return u < thresh ? scale : T(0);
}
template <typename T>
static __global__ void dropout_mask_kernel(long long n, double keep, unsigned long long seed, unsigned long long offset,
                                           T* __restrict__ mask) {
  const T scale = T(1) / static_cast<T>(keep);
  const unsigned int thresh = static_cast<unsigned int>(keep * 16777216.0);
  for (long long j = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; j < n;
       j += static_cast<long long>(gridDim.x) * blockDim.x)
    mask[j] = dropout_entry<T>(seed, offset + static_cast<unsigned long long>(j), keep, thresh, scale);
}
template <typename T>
static __global__ void mask_mul_kernel(const T* __restrict__ x, const T* __restrict__ mask, long long n, long long inner,
                                       T* __restrict__ y) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    y[i] = r_mul(x[i], mask[inner == 1 ? i : i / inner]);
}
// y = x * mask with the mask entries generated on the fly (no mask tensor: one read, one write).  inner = 1: a
// thread owns two neighbouring elements, which share one hash when offset is even.
template <typename T>
static __global__ void dropout_apply_kernel(const T* __restrict__ x, long long n, long long inner, double keep,
                                            unsigned long long seed, unsigned long long offset, T* __restrict__ y) {
  const T scale = T(1) / static_cast<T>(keep);
  const unsigned int thresh = static_cast<unsigned int>(keep * 16777216.0);
  if (inner == 1 && (offset & 1ULL) == 0 && keep > 0.0 && keep < 1.0) {
    const long long pairs = (n + 1) >> 1;
    for (long long q = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; q < pairs;
         q += static_cast<long long>(gridDim.x) * blockDim.x) {
      const unsigned long long hsh = dropout_hash(seed, (offset >> 1) + static_cast<unsigned long long>(q));
      const long long i = q << 1;
      const T m0 = (static_cast<unsigned int>(hsh >> 40) & 0xFFFFFFu) < thresh ? scale : T(0);
      y[i] = r_mul(x[i], m0);
      if (i + 1 < n) {
        const T m1 = (static_cast<unsigned int>(hsh >> 16) & 0xFFFFFFu) < thresh ? scale : T(0);
        y[i + 1] = r_mul(x[i + 1], m1);
      }
    }
    return;
  }
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const unsigned long long g = offset + static_cast<unsigned long long>(inner == 1 ? i : i / inner);
    y[i] = r_mul(x[i], dropout_entry<T>(seed, g, keep, thresh, scale));
  }
}

}  // namespace mtb

using namespace mtb;

#define MTB_CHECK_HANDLE(h)                                         \
  if (!(h)) return fail(MTB200_ERR_INVALID, "null handle");         \
  DeviceGuard guard__((h)->device);                                 \
  if (!guard__.ok) return fail(MTB200_ERR_CUDA, "cannot make device %d current", (h)->device)

// y[i] += x[i]: gradient accumulation (add_inplace, engine/src/operations/arithmetic/elementwise.rs:102-160).
// Integers wrap, as the reference's wrapping_add does.
template <typename T>
static __global__ void add_inplace_kernel(T* __restrict__ y, const T* __restrict__ x, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    y[i] = y[i] + x[i];
}

// Materialised swap of two dimensions (transpose, engine/src/operations/linalg/diagonal.rs:8-108): x viewed as
// [outer][d0][mid][d1][inner] becomes y [outer][d1][mid][d0][inner].
//  * inner == 1 and mid == 1 (the matrix transpose of the last two of the swapped dimensions): 32 x 32 tiles through
//    shared memory, so both the reads and the writes are whole lines;
//  * otherwise runs of `inner` elements move together and a thread per output element is coalesced as it stands.
template <typename T>
static __global__ void __launch_bounds__(256) transpose_tiles_kernel(const T* __restrict__ x, T* __restrict__ y, int d0,
                                                                      int d1) {
  __shared__ T tile[32][33];
  const long long plane = static_cast<long long>(d0) * d1;
  const T* xs = x + blockIdx.z * plane;
  T* ys = y + blockIdx.z * plane;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8)
    if (r0 + r < d0 && c0 + tx < d1) tile[r][tx] = xs[static_cast<long long>(r0 + r) * d1 + c0 + tx];
  __syncthreads();
  for (int c = ty; c < 32; c += 8)
    if (c0 + c < d1 && r0 + tx < d0) ys[static_cast<long long>(c0 + c) * d0 + r0 + tx] = tile[tx][c];
}
template <typename T>
static __global__ void swap_dims_kernel(const T* __restrict__ x, T* __restrict__ y, long long total, long long d0,
                                        long long mid, long long d1, long long inner) {
  for (long long o = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; o < total;
       o += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long r = o;
    const long long i = r % inner; r /= inner;
    const long long a0 = r % d0; r /= d0;       // output layout [outer][d1][mid][d0][inner]
    const long long m = r % mid; r /= mid;
    const long long a1 = r % d1; r /= d1;
    y[o] = x[(((r * d0 + a0) * mid + m) * d1 + a1) * inner + i];
  }
}

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

// Launches the two-sums-per-channel reduction (see bn_terms).
template <typename T, int MODE>
static int32_t bn_reduce(mtb200_ctx* h, const T* x, const T* dy, const T* a_c, const T* b_c, int64_t N, int64_t C,
                         int64_t S, double* partial, int chunks, int64_t per_chunk) {
  if (S == 1)
    bn_reduce_cols_kernel<T, MODE><<<dim3(unsigned((C + 127) / 128), unsigned(chunks)), 256, 0, h->stream>>>(
        x, dy, a_c, b_c, N, int(C), per_chunk, partial);
  else
    bn_reduce_general_kernel<T, MODE><<<dim3(unsigned(C), unsigned(chunks)), 256, 0, h->stream>>>(
        x, dy, a_c, b_c, N, int(C), S, per_chunk, partial);
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}
static void bn_chunking(const mtb200_ctx* h, int64_t N, int64_t C, int64_t S, int* chunks, int64_t* per_chunk) {
  // enough blocks to fill the machine about four times over, at least 2048 reduced elements per block
  const int64_t units = S == 1 ? N : N * S;                       // rows (cols kernel) or (n, s) pairs
  const int64_t blocks_c = S == 1 ? (C + 127) / 128 : C;
  int64_t want = std::max<int64_t>(1, (int64_t(h->sm_count) * 4) / std::max<int64_t>(1, blocks_c));
  want = std::min<int64_t>(want, std::max<int64_t>(1, units / (S == 1 ? 64 : 2048)));
  want = std::min<int64_t>(want, 1024);
  *per_chunk = (units + want - 1) / want;
  *chunks = int((units + *per_chunk - 1) / *per_chunk);
}

template <typename T>
static int32_t batch_norm_fwd_t(mtb200_ctx* h, int64_t N, int64_t C, int64_t S, const T* x, const T* w, const T* b,
                                T* rm, T* rv, int training, double momentum, double eps, T* y, T* save_mean,
                                T* save_invstd) {
  const bool batch_stats = training || !rm || !rv;
  int chunks = 1;
  int64_t per_chunk = 0;
  bn_chunking(h, N, C, S, &chunks, &per_chunk);
  const size_t bytes_partial = sizeof(double) * 2 * size_t(chunks) * size_t(C);
  const size_t bytes_stats = ((sizeof(T) * 2 * size_t(C)) + 15) / 16 * 16;
  void* ws = nullptr;
  int32_t rc = workspace_reserve(h, bytes_partial + bytes_stats, &ws);
  if (rc) return rc;
  double* partial = static_cast<double*>(ws);
  T* mean = save_mean ? save_mean : reinterpret_cast<T*>(static_cast<char*>(ws) + bytes_partial);
  T* invstd = save_invstd ? save_invstd : reinterpret_cast<T*>(static_cast<char*>(ws) + bytes_partial) + C;
  if (batch_stats) {
    rc = bn_reduce<T, 0>(h, x, nullptr, nullptr, nullptr, N, C, S, partial, chunks, per_chunk);
    if (rc) return rc;
    const bool update = training && rm && rv;
    bn_finalize_fwd_kernel<T><<<unsigned((C + 255) / 256), 256, 0, h->stream>>>(
        partial, chunks, int(C), double(N) * double(S), x, S, eps, mean, invstd, update ? rm : nullptr,
        update ? rv : nullptr, static_cast<T>(momentum), static_cast<T>(1.0 - momentum));
  } else {
    bn_from_running_kernel<T><<<unsigned((C + 255) / 256), 256, 0, h->stream>>>(rm, rv, int(C), eps, mean, invstd);
  }
  MTB_CUDA(cudaGetLastError());
  return bn_element_launch<T, 0>(h, x, nullptr, mean, invstd, w, b, nullptr, 0.0, 0, N, C, S, y);
}

template <typename T>
static int32_t batch_norm_bwd_t(mtb200_ctx* h, int64_t N, int64_t C, int64_t S, const T* x, const T* dy, const T* w,
                                const T* mean, const T* invstd, int batch_stats, T* dx, T* dw, T* db) {
  int chunks = 1;
  int64_t per_chunk = 0;
  bn_chunking(h, N, C, S, &chunks, &per_chunk);
  const size_t bytes_partial = sizeof(double) * 2 * size_t(chunks) * size_t(C);
  void* ws = nullptr;
  int32_t rc = workspace_reserve(h, bytes_partial + sizeof(double) * 2 * size_t(C), &ws);
  if (rc) return rc;
  double* partial = static_cast<double*>(ws);
  double* sums = partial + 2 * size_t(chunks) * size_t(C);
  rc = bn_reduce<T, 1>(h, x, dy, mean, invstd, N, C, S, partial, chunks, per_chunk);
  if (rc) return rc;
  bn_finalize_bwd_kernel<T><<<unsigned((C + 255) / 256), 256, 0, h->stream>>>(partial, chunks, int(C), sums, dw, db);
  MTB_CUDA(cudaGetLastError());
  if (dx)
    return bn_element_launch<T, 1>(h, x, dy, mean, invstd, w, nullptr, sums, 1.0 / (double(N) * double(S)), batch_stats, N,
                                   C, S, dx);
  return MTB200_OK;
}

static int32_t bn_check_dims(int64_t N, int64_t C, int64_t S) {
  if (N < 0 || C < 0 || S < 0) return fail(MTB200_ERR_INVALID, "negative dimension");
  if (C > INT32_MAX) return fail(MTB200_ERR_INVALID, "channel count exceeds the 32-bit limit of the device kernels");
  // every geometry the kernels refuse is refused here, before a launch could have touched the running estimates
  if (S > 1 && N > 0 && C > 0 && N > INT32_MAX / C)
    return fail(MTB200_ERR_INVALID, "batch_norm: N * C exceeds 2^31 - 1 for inputs with spatial dimensions");
  return MTB200_OK;
}

extern "C" {

int32_t mtb200_batch_norm_fwd(mtb200_handle h, int32_t dtype, int64_t N, int64_t C, int64_t S, const void* x,
                              const void* weight, const void* bias, void* running_mean, void* running_var,
                              int32_t training, double momentum, double eps, void* y, void* save_mean,
                              void* save_invstd) {
  MTB_CHECK_HANDLE(h);
  if (int32_t rc = check_float_dtype(dtype, "batch_norm")) return rc;
  if (int32_t rc = bn_check_dims(N, C, S)) return rc;
  if (N == 0 || C == 0 || S == 0) return MTB200_OK;
  if (!x || !y) return fail(MTB200_ERR_INVALID, "null pointer");
  if (dtype == MTB200_F32)
    return batch_norm_fwd_t<float>(h, N, C, S, static_cast<const float*>(x), static_cast<const float*>(weight),
                                   static_cast<const float*>(bias), static_cast<float*>(running_mean),
                                   static_cast<float*>(running_var), training, momentum, eps, static_cast<float*>(y),
                                   static_cast<float*>(save_mean), static_cast<float*>(save_invstd));
  return batch_norm_fwd_t<double>(h, N, C, S, static_cast<const double*>(x), static_cast<const double*>(weight),
                                  static_cast<const double*>(bias), static_cast<double*>(running_mean),
                                  static_cast<double*>(running_var), training, momentum, eps, static_cast<double*>(y),
                                  static_cast<double*>(save_mean), static_cast<double*>(save_invstd));
}

int32_t mtb200_batch_norm_bwd(mtb200_handle h, int32_t dtype, int64_t N, int64_t C, int64_t S, const void* x,
                              const void* dy, const void* weight, const void* save_mean, const void* save_invstd,
                              int32_t batch_stats, void* dx, void* dweight, void* dbias) {
  MTB_CHECK_HANDLE(h);
  if (int32_t rc = check_float_dtype(dtype, "batch_norm")) return rc;
  if (int32_t rc = bn_check_dims(N, C, S)) return rc;
  if (N == 0 || C == 0 || S == 0) return MTB200_OK;
  if (!x || !dy || !save_mean || !save_invstd) return fail(MTB200_ERR_INVALID, "null pointer");
  if (dtype == MTB200_F32)
    return batch_norm_bwd_t<float>(h, N, C, S, static_cast<const float*>(x), static_cast<const float*>(dy),
                                   static_cast<const float*>(weight), static_cast<const float*>(save_mean),
                                   static_cast<const float*>(save_invstd), batch_stats, static_cast<float*>(dx),
                                   static_cast<float*>(dweight), static_cast<float*>(dbias));
  return batch_norm_bwd_t<double>(h, N, C, S, static_cast<const double*>(x), static_cast<const double*>(dy),
                                  static_cast<const double*>(weight), static_cast<const double*>(save_mean),
                                  static_cast<const double*>(save_invstd), batch_stats, static_cast<double*>(dx),
                                  static_cast<double*>(dweight), static_cast<double*>(dbias));
}

int32_t mtb200_dropout_mask(mtb200_handle h, int32_t dtype, int64_t n, double p, uint64_t seed, uint64_t offset,
                            void* mask) {
  MTB_CHECK_HANDLE(h);
  if (int32_t rc = check_float_dtype(dtype, "Dropout mask generation")) return rc;
  if (!(p >= 0.0 && p <= 1.0)) return fail(MTB200_ERR_INVALID, "dropout probability must be in [0, 1], got %g", p);
  if (n < 0) return fail(MTB200_ERR_INVALID, "negative length");
  if (n == 0) return MTB200_OK;
  if (!mask) return fail(MTB200_ERR_INVALID, "null pointer");
  const int grid = ew_grid(n, h->sm_count);
  if (dtype == MTB200_F32)
    dropout_mask_kernel<float><<<grid, 256, 0, h->stream>>>(n, 1.0 - p, seed, offset, static_cast<float*>(mask));
  else
    dropout_mask_kernel<double><<<grid, 256, 0, h->stream>>>(n, 1.0 - p, seed, offset, static_cast<double*>(mask));
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

int32_t mtb200_mask_mul(mtb200_handle h, int32_t dtype, int64_t n, int64_t inner, const void* x, const void* mask,
                        void* y) {
  MTB_CHECK_HANDLE(h);
  if (int32_t rc = check_float_dtype(dtype, "dropout")) return rc;
  if (n < 0 || inner < 1) return fail(MTB200_ERR_INVALID, "bad length");
  if (n == 0) return MTB200_OK;
  if (!x || !mask || !y) return fail(MTB200_ERR_INVALID, "null pointer");
  const int grid = ew_grid(n, h->sm_count);
  if (dtype == MTB200_F32)
    mask_mul_kernel<float><<<grid, 256, 0, h->stream>>>(static_cast<const float*>(x), static_cast<const float*>(mask), n,
                                                        inner, static_cast<float*>(y));
  else
    mask_mul_kernel<double><<<grid, 256, 0, h->stream>>>(static_cast<const double*>(x), static_cast<const double*>(mask),
                                                         n, inner, static_cast<double*>(y));
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

int32_t mtb200_dropout_apply(mtb200_handle h, int32_t dtype, int64_t n, int64_t inner, const void* x, double p,
                             uint64_t seed, uint64_t offset, void* y) {
  MTB_CHECK_HANDLE(h);
  if (int32_t rc = check_float_dtype(dtype, "dropout")) return rc;
  if (!(p >= 0.0 && p <= 1.0)) return fail(MTB200_ERR_INVALID, "dropout probability must be in [0, 1], got %g", p);
  if (n < 0 || inner < 1) return fail(MTB200_ERR_INVALID, "bad length");
  if (n == 0) return MTB200_OK;
  if (!x || !y) return fail(MTB200_ERR_INVALID, "null pointer");
  const int grid = ew_grid((n + 1) / 2, h->sm_count);
  if (dtype == MTB200_F32)
    dropout_apply_kernel<float><<<grid, 256, 0, h->stream>>>(static_cast<const float*>(x), n, inner, 1.0 - p, seed, offset,
                                                             static_cast<float*>(y));
  else
    dropout_apply_kernel<double><<<grid, 256, 0, h->stream>>>(static_cast<const double*>(x), n, inner, 1.0 - p, seed,
                                                              offset, static_cast<double*>(y));
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

int32_t mtb200_add_inplace(mtb200_handle h, int32_t dtype, int64_t n, void* y, const void* x) {
  MTB_CHECK_HANDLE(h);
  if (n < 0) return fail(MTB200_ERR_INVALID, "negative length");
  if (n == 0) return MTB200_OK;
  if (!x || !y) return fail(MTB200_ERR_INVALID, "null pointer");
  const int grid = ew_grid(n, h->sm_count);
  switch (dtype) {
    case MTB200_F32: add_inplace_kernel<float><<<grid, 256, 0, h->stream>>>(static_cast<float*>(y), static_cast<const float*>(x), n); break;
    case MTB200_F64: add_inplace_kernel<double><<<grid, 256, 0, h->stream>>>(static_cast<double*>(y), static_cast<const double*>(x), n); break;
    case MTB200_I32: add_inplace_kernel<uint32_t><<<grid, 256, 0, h->stream>>>(static_cast<uint32_t*>(y), static_cast<const uint32_t*>(x), n); break;
    case MTB200_I64: add_inplace_kernel<unsigned long long><<<grid, 256, 0, h->stream>>>(static_cast<unsigned long long*>(y), static_cast<const unsigned long long*>(x), n); break;
    default: return fail(MTB200_ERR_UNSUPPORTED, "add_inplace: unsupported dtype %d", dtype);
  }
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

int32_t mtb200_swap_dims(mtb200_handle h, int32_t elem_bytes, int64_t outer, int64_t d0, int64_t mid, int64_t d1,
                         int64_t inner, const void* x, void* y) {
  MTB_CHECK_HANDLE(h);
  if (elem_bytes != 4 && elem_bytes != 8) return fail(MTB200_ERR_UNSUPPORTED, "swap_dims moves 4- or 8-byte elements");
  if (outer < 0 || d0 < 0 || mid < 0 || d1 < 0 || inner < 0) return fail(MTB200_ERR_INVALID, "negative dimension");
  const long double total_ld = static_cast<long double>(outer) * d0 * mid * d1 * inner;
  if (total_ld > 9.0e18L) return fail(MTB200_ERR_INVALID, "swap_dims: too many elements");
  const long long total = outer * d0 * mid * d1 * inner;
  if (total == 0) return MTB200_OK;
  if (!x || !y) return fail(MTB200_ERR_INVALID, "null pointer");
  if (x == y) return fail(MTB200_ERR_INVALID, "swap_dims does not work in place");
  if (inner == 1 && mid == 1 && d0 <= INT32_MAX && d1 <= INT32_MAX && outer <= 65535 &&
      (d0 + 31) / 32 <= 65535) {
    const dim3 grid(unsigned((d1 + 31) / 32), unsigned((d0 + 31) / 32), unsigned(outer));
    if (elem_bytes == 4)
      transpose_tiles_kernel<uint32_t><<<grid, 256, 0, h->stream>>>(static_cast<const uint32_t*>(x), static_cast<uint32_t*>(y), int(d0), int(d1));
    else
      transpose_tiles_kernel<unsigned long long><<<grid, 256, 0, h->stream>>>(static_cast<const unsigned long long*>(x),
                                                                             static_cast<unsigned long long*>(y), int(d0), int(d1));
  } else {
    const int grid = ew_grid(total, h->sm_count);
    if (elem_bytes == 4)
      swap_dims_kernel<uint32_t><<<grid, 256, 0, h->stream>>>(static_cast<const uint32_t*>(x), static_cast<uint32_t*>(y), total, d0, mid, d1, inner);
    else
      swap_dims_kernel<unsigned long long><<<grid, 256, 0, h->stream>>>(static_cast<const unsigned long long*>(x),
                                                                       static_cast<unsigned long long*>(y), total, d0, mid, d1, inner);
  }
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

}  // extern "C"
