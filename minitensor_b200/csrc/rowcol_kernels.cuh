// HBM-bound kernels either side of the GEMMs in a training step: bias-gradient
// column sum, activation forward/backward, fused cross-entropy, Adam.
#pragma once
#include "ptx_sm100.cuh"
#include <cstdint>
#include <cuda_runtime.h>

namespace mtb {

// ------------------------------------------------------------------ column sum
// out[n] = sum_m X[m][n]: the bias gradient, i.e. what the reference computes
// with reduce_gradient_for_broadcasting -> sum over dim 0
// (engine/src/operations/reduction/sum_prod.rs:7-84).  Two deterministic stages:
// stage 1 sums a contiguous band of rows per block into partial[band][n];
// stage 2 adds the bands in ascending order.  A warp reads 4 rows x 32
// columns per step (8 lanes x float4 = 128 B per row) and folds its 4 row
// lanes with shuffles; the 8 warps of a block are folded through shared memory.
template <typename T>
__global__ void __launch_bounds__(256) colsum_stage1_kernel(const T* __restrict__ X, long long ld,
                                                            int M, int N, int rows_per_band,
                                                            T* __restrict__ partial) {
  constexpr int V = 16 / sizeof(T);  // elements per 16-byte vector
  constexpr int COLS = 8 * V;        // columns per block
  __shared__ T red[8][COLS];
  grid_launch_dependents();          // stage 2 may set itself up meanwhile; it waits before it reads
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rl = lane >> 3, cg = lane & 7;
  const int col = blockIdx.x * COLS + cg * V;
  const int band = blockIdx.y;
  const int m0 = band * rows_per_band;
  const int m1 = min(M, m0 + rows_per_band);
  const bool vec = ((reinterpret_cast<uintptr_t>(X) & 15) == 0) && ((ld % V) == 0) && (col + V <= N);
  T acc[V];
#pragma unroll
  for (int e = 0; e < V; ++e) acc[e] = T(0);
  for (int m = m0 + warp * 4 + rl; m < m1; m += 32) {
    const T* p = X + static_cast<long long>(m) * ld + col;
    if (vec) {
      const uint4 raw = *reinterpret_cast<const uint4*>(p);
      const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int e = 0; e < V; ++e) acc[e] += v[e];
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e)
        if (col + e < N) acc[e] += p[e];
    }
  }
#pragma unroll
  for (int e = 0; e < V; ++e) {
    acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 8);
    acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 16);
  }
  if (rl == 0) {
#pragma unroll
    for (int e = 0; e < V; ++e) red[warp][cg * V + e] = acc[e];
  }
  __syncthreads();
  if (threadIdx.x < COLS) {
    const int c = blockIdx.x * COLS + threadIdx.x;
    if (c < N) {
      T s = T(0);
#pragma unroll
      for (int w = 0; w < 8; ++w) s += red[w][threadIdx.x];
      partial[static_cast<long long>(band) * N + c] = s;
    }
  }
}

template <typename T>
__global__ void colsum_stage2_kernel(const T* __restrict__ partial, int bands, int N,
                                     T* __restrict__ out) {
  grid_dependency_wait();        // the partials come from the kernel before this one (no-op in a plain launch)
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= N) return;
  T s = T(0);
  for (int b = 0; b < bands; ++b) s += partial[static_cast<long long>(b) * N + c];
  out[c] = s;
}

// ------------------------------------------------------------------ activations
// act: 1 relu, 2 gelu (erf), 3 gelu (tanh)   (engine/src/operations/activation/
// softmax.rs:161-203, hyperbolic.rs:697-745)
template <typename T>
__device__ __forceinline__ T act_fwd_value(T x, int act) {
  if (act == 1) return (x != x) ? x : (x > T(0) ? x : T(0));
  if (act == 2) return T(0.5) * x * (T(1) + erf(x * T(0.70710678118654752440)));
  if (act == 3) {
    const T c = sqrt(T(2) / T(3.14159265358979323846));
    const T x3 = x * x * x;
    return T(0.5) * x * (T(1) + tanh(c * (x + T(0.044715) * x3)));
  }
  return x;
}

// dx = dy * f'(.).  For relu `ref` is the activation OUTPUT (y > 0 is the
// reference's saved mask: engine/src/autograd/mod/shape.rs:724-816); for gelu
// it is the activation INPUT (engine/src/autograd/mod/linalg.rs:118-264).
template <typename T>
__device__ __forceinline__ T act_bwd_value(T ref, T dy, int act) {
  if (act == 1) return dy * (ref > T(0) ? T(1) : T(0));
  const T x = ref;
  if (act == 2) {
    const T cdf = T(0.5) * (T(1) + erf(x * T(0.70710678118654752440)));
    const T pdf = exp(T(-0.5) * x * x) * (T(1) / sqrt(T(2) * T(3.14159265358979323846)));
    return dy * (cdf + x * pdf);
  }
  if (act == 3) {
    const T c = sqrt(T(2) / T(3.14159265358979323846));
    const T x2 = x * x;
    const T inner = c * (x + T(0.044715) * x * x2);
    const T th = tanh(inner);
    const T sech2 = T(1) - th * th;
    return dy * (T(0.5) * (T(1) + th) + T(0.5) * x * sech2 * c * (T(1) + T(3) * T(0.044715) * x2));
  }
  return dy;
}

template <typename T>
__global__ void act_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, int act) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    y[i] = act_fwd_value<T>(x[i], act);
}
template <typename T>
__global__ void act_bwd_kernel(const T* __restrict__ ref, const T* __restrict__ dy,
                               T* __restrict__ dx, long long n, int act) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dx[i] = act_bwd_value<T>(ref[i], dy[i], act);
}

// y[m][n] = act(x[m][n] + bias[n]); used for the degenerate K == 0 GEMM and as
// the unfused form of the dense epilogue.
template <typename T>
__global__ void bias_act_kernel(const T* __restrict__ x, const T* __restrict__ bias,
                                T* __restrict__ y, long long rows, int N, long long ld, int act) {
  const long long total = rows * N;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / N;
    const int c = static_cast<int>(i - r * N);
    T v = x ? x[r * ld + c] : T(0);
    if (bias) v += bias[c];
    y[r * ld + c] = act_fwd_value<T>(v, act);
  }
}

// ------------------------------------------------------------------ cross entropy
// One warp per sample row.  Mirrors cross_entropy_loss with class-index
// targets (engine/src/operations/loss/regression.rs:178-251): log-softmax by
// max shift (activation/softmax.rs:848-901), softmax = exp(log-softmax),
// entries with softmax <= 1e-30 have their log-probability replaced by -inf
// before the product with the one-hot row (so a masked non-target entry makes
// the sample loss NaN, a masked target entry makes it +inf), and the gradient
// (softmax - onehot) * scale of CrossEntropyLossBackward
// (engine/src/autograd/mod/activation.rs:364-427).  row_loss[b] receives the
// per-sample loss; a label outside [0, C) sets *bad_label.
template <typename LabelT>
__global__ void __launch_bounds__(256) cross_entropy_rows_kernel(
    const float* __restrict__ logits, const LabelT* __restrict__ labels, int B, int C,
    float grad_scale, float* __restrict__ row_loss, float* __restrict__ dlogits,
    uint32_t* __restrict__ bad_label) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= B) return;
  const float* x = logits + static_cast<long long>(warp) * C;
  long long lab = static_cast<long long>(labels[warp]);
  if (lab < 0 || lab >= C) {
    if (lane == 0) atomicOr(bad_label, 1u);
    lab = -1;
  }
  float mx = -INFINITY;
  for (int c = lane; c < C; c += 32) mx = fmaxf(mx, x[c]);  // NaN entries never win a `>` test either
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float s = 0.0f;
  for (int c = lane; c < C; c += 32) s += expf(x[c] - mx);
#pragma unroll
  for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const bool all_neg_inf = (mx == -INFINITY);
  const float logsum = logf(s) + mx;
  int masked_other = 0;
  float lp_label = 0.0f;
  for (int c = lane; c < C; c += 32) {
    const float lp = all_neg_inf ? -INFINITY : x[c] - logsum;
    const float sm = expf(lp);
    const bool is_lab = (c == lab);
    if (sm <= 1e-30f) {
      if (is_lab) lp_label = -INFINITY; else masked_other = 1;
    } else if (is_lab) {
      lp_label = lp;
    }
    if (dlogits)
      dlogits[static_cast<long long>(warp) * C + c] = (sm - (is_lab ? 1.0f : 0.0f)) * grad_scale;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    masked_other |= __shfl_xor_sync(0xffffffffu, masked_other, o);
    // exactly one lane holds the target's term; the others hold 0
    lp_label += __shfl_xor_sync(0xffffffffu, lp_label, o);
  }
  if (lane == 0) {
    float l = -lp_label;
    if (masked_other || l != l) l = NAN;
    row_loss[warp] = l;
  }
}

// loss = (sum of row_loss in a fixed tree order) * inv_count.  One block.
static __global__ void __launch_bounds__(1024) loss_reduce_kernel(const float* __restrict__ row_loss, int B,
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

// ------------------------------------------------------------------ Adam
// Per-element update of Adam::apply_adam_update without amsgrad
// (engine/src/optim/adam.rs:296-312), same operation order and no fused
// multiply-add so the result is bit-identical to the f32 CPU arithmetic:
//   g' = g + wd*p (coupled) | g (decoupled, after p -= lr*wd*p)
//   m = b1*m + (1-b1)*g' ; v = b2*v + (1-b2)*g'*g'
//   p -= lr * (m*bc1_inv) / (sqrt(v*bc2_inv) + eps)
// grad_scale multiplies g first (1 for the reference semantics; 1/world for
// the mean of per-rank gradients after an all-reduce sum).
__device__ __forceinline__ void adam_update(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                            float* __restrict__ v, long long i, float lr, float b1, float b2, float omb1,
                                            float omb2, float eps, float wd, float bc1_inv, float bc2_inv, int decoupled,
                                            float grad_scale) {
  float pi = p[i];
  float gi = g[i];
  if (grad_scale != 1.0f) gi = __fmul_rn(gi, grad_scale);
  if (decoupled) {
    pi = __fsub_rn(pi, __fmul_rn(__fmul_rn(lr, wd), pi));
  } else {
    gi = __fadd_rn(gi, __fmul_rn(wd, pi));
  }
  const float mi = __fadd_rn(__fmul_rn(b1, m[i]), __fmul_rn(omb1, gi));
  const float vi = __fadd_rn(__fmul_rn(b2, v[i]), __fmul_rn(__fmul_rn(omb2, gi), gi));
  m[i] = mi;
  v[i] = vi;
  const float mhat = __fmul_rn(mi, bc1_inv);
  const float vhat = __fmul_rn(vi, bc2_inv);
  const float denom = __fadd_rn(__fsqrt_rn(vhat), eps);
  p[i] = __fsub_rn(pi, __fdiv_rn(__fmul_rn(lr, mhat), denom));
}

static __global__ void adam_kernel(float* __restrict__ p, const float* __restrict__ g,
                            float* __restrict__ m, float* __restrict__ v, long long n, float lr,
                            float b1, float b2, float eps, float wd, float bc1_inv, float bc2_inv,
                            int decoupled, float grad_scale) {
  const float omb1 = __fsub_rn(1.0f, b1), omb2 = __fsub_rn(1.0f, b2);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    adam_update(p, g, m, v, i, lr, b1, b2, omb1, omb2, eps, wd, bc1_inv, bc2_inv, decoupled, grad_scale);
}

// a^b for b >= 1 by square and multiply in f64, the same sequence of products the host computes
// (what f64::powi lowers to), so the bias corrections match the host's bit for bit.
__device__ __forceinline__ double powi_dev(double a, long long b) {
  double r = 1.0;
  while (true) {
    if (b & 1) r = __dmul_rn(r, a);
    b >>= 1;
    if (b == 0) break;
    a = __dmul_rn(a, a);
  }
  return r;
}

static __global__ void counter_add_kernel(long long* counter, long long delta) { *counter += delta; }

// The same update with the step count read from device memory, so that a loop replayed from a CUDA
// graph (whose kernel arguments are frozen at capture) still advances its bias corrections.
static __global__ void adam_counted_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                           float* __restrict__ v, long long n, float lr, double beta1, double beta2,
                                           float eps, float wd, const long long* __restrict__ step_counter,
                                           int decoupled, float grad_scale) {
  const long long step = max(1LL, *step_counter);
  const float bc1_inv = static_cast<float>(__ddiv_rn(1.0, __dsub_rn(1.0, powi_dev(beta1, step))));
  const float bc2_inv = static_cast<float>(__ddiv_rn(1.0, __dsub_rn(1.0, powi_dev(beta2, step))));
  const float b1 = static_cast<float>(beta1), b2 = static_cast<float>(beta2);
  const float omb1 = __fsub_rn(1.0f, b1), omb2 = __fsub_rn(1.0f, b2);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    adam_update(p, g, m, v, i, lr, b1, b2, omb1, omb2, eps, wd, bc1_inv, bc2_inv, decoupled, grad_scale);
}

}  // namespace mtb
