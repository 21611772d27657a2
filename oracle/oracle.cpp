// CPU oracle for the dense-contraction path of minitensor.
//
// THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It restates, in plain C++,
// the arithmetic minitensor's CPU engine performs for matmul / bmm and their
// backward, DenseLayer, ReLU / GELU, the dim-0 sum behind bias gradients,
// conv2d and its backward, cross entropy and Adam, so that the CUDA kernels
// can be checked against it and so that its speed can be reported as the CPU
// baseline.  Only the tests, the smoke check and the benchmark's CPU-baseline /
// reference legs may call it; the library never does.
//
// Pinning: every function is checked (tests/test_oracle_golden.py) against the
// known answers held by minitensor's own unit tests (tests/golden/known_answers.json
// lists them with file:line).  The reference itself cannot be built here (it is
// Rust; there is no Rust toolchain), and its f32/f64 GEMM inner kernel lives in
// the third-party crate `matrixmultiply` ("0.3", unpinned: the reference ships
// no Cargo.lock), which is not in the reference tree.  For that one routine the
// oracle restates the crate's published scheme: C = A*B accumulated in the
// element type, k ascending inside cache blocks of KC = 256 reduction steps, one
// fused multiply-add per step, block sums added to C in ascending block order.
// For large random f32/f64 matrices nothing in the reference pins values beyond
// NumPy-at-rtol on tiny inputs, so for those sizes parity is "unpinned" and the
// comparison uses the norm-scaled tolerance against this restatement and against
// the f64-accumulated product (gemm_f32_acc64).
//
// All file:line references are paths inside the minitensor repository.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

int orc_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

}  // extern "C"

namespace {

// ---------------------------------------------------------------------------
// gemm_f32 / gemm_f64: engine/src/operations/linalg/matmul.rs:240-258 call
// matrixmultiply::sgemm/dgemm(m,k,n, 1, a, (k,1), b, (n,1), 0, c, (n,1)).
// Restated scheme: see the header.  Rows are independent, so the row loop is
// the threaded one (the crate's `threading` feature also splits C, not K).
template <typename T>
void gemm_rowmajor(int64_t m, int64_t k, int64_t n, const T* a, const T* b, T* c, bool threaded) {
  constexpr int64_t KC = 256;
  // Register block MR x NR: a speed matter only; every output element still sees
  // its products in the order described in the header.
  constexpr int64_t MR = 6, NR = 64 / sizeof(T);
  const int64_t row_blocks = (m + MR - 1) / MR;
#pragma omp parallel for schedule(static) if (threaded)
  for (int64_t ib = 0; ib < row_blocks; ++ib) {
    const int64_t i0 = ib * MR, mr = std::min(MR, m - i0);
    for (int64_t k0 = 0; k0 < k; k0 += KC) {
      const int64_t kc = std::min(KC, k - k0);
      for (int64_t j0 = 0; j0 < n; j0 += NR) {
        const int64_t nr = std::min(NR, n - j0);
        T acc[MR][NR];
        for (int64_t r = 0; r < MR; ++r)
          for (int64_t j = 0; j < NR; ++j) acc[r][j] = T(0);
        if (mr == MR && nr == NR) {
          for (int64_t l = 0; l < kc; ++l) {
            const T* brow = b + (k0 + l) * n + j0;
            for (int64_t r = 0; r < MR; ++r) {
              const T av = a[(i0 + r) * k + k0 + l];
#pragma omp simd
              for (int64_t j = 0; j < NR; ++j) acc[r][j] = std::fma(av, brow[j], acc[r][j]);
            }
          }
        } else {
          for (int64_t l = 0; l < kc; ++l) {
            const T* brow = b + (k0 + l) * n + j0;
            for (int64_t r = 0; r < mr; ++r) {
              const T av = a[(i0 + r) * k + k0 + l];
              for (int64_t j = 0; j < nr; ++j) acc[r][j] = std::fma(av, brow[j], acc[r][j]);
            }
          }
        }
        for (int64_t r = 0; r < mr; ++r) {
          T* crow = c + (i0 + r) * n + j0;
          if (k0 == 0) {
            for (int64_t j = 0; j < nr; ++j) crow[j] = acc[r][j];  // beta = 0
          } else {
            for (int64_t j = 0; j < nr; ++j) crow[j] += acc[r][j];
          }
        }
      }
    }
  }
}

// optimized_matmul_f32/f64: engine/src/operations/linalg/diagonal.rs:550-640.
// batch == 1 -> one gemm; otherwise one gemm per batch entry, entries in parallel.
template <typename T>
void matmul_float(int64_t batch, int64_t m, int64_t k, int64_t n, const T* a, const T* b, T* c) {
  if (m == 0 || k == 0 || n == 0) return;  // diagonal.rs:563-566; output stays zero (matmul.rs:373-376)
  if (batch == 1) {
    gemm_rowmajor<T>(m, k, n, a, b, c, true);
  } else {
#pragma omp parallel for schedule(dynamic)
    for (int64_t bi = 0; bi < batch; ++bi)
      gemm_rowmajor<T>(m, k, n, a + bi * m * k, b + bi * k * n, c + bi * m * n, false);
  }
}

// naive_matmul<T>: engine/src/operations/linalg/diagonal.rs:495-548.
// sum = sum + a*b, l ascending; release-build (wrapping) integer semantics.
template <typename U>
void matmul_int(int64_t batch, int64_t m, int64_t k, int64_t n, const U* a, const U* b, U* c) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bi = 0; bi < batch; ++bi)
    for (int64_t i = 0; i < m; ++i) {
      const U* ab = a + bi * m * k;
      const U* bb = b + bi * k * n;
      U* cb = c + bi * m * n;
      for (int64_t j = 0; j < n; ++j) {
        U sum = 0;
        for (int64_t l = 0; l < k; ++l) sum = sum + ab[i * k + l] * bb[l * n + j];
        cb[i * n + j] = sum;
      }
    }
}

// transpose of the last two dims into a fresh buffer:
// engine/src/operations/linalg/triangular.rs:8-73 (transpose_generic).
template <typename T>
void transpose_last2(int64_t batch, int64_t rows, int64_t cols, const T* src, T* dst) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bi = 0; bi < batch; ++bi)
    for (int64_t j = 0; j < cols; ++j)
      for (int64_t i = 0; i < rows; ++i)
        dst[bi * rows * cols + j * rows + i] = src[bi * rows * cols + i * cols + j];
}

template <typename T>
T relu_value(T v) {  // engine/src/operations/activation/softmax.rs:176-184
  if (std::isnan(v)) return v;
  return v > T(0) ? v : T(0);
}

// gelu_f32/f64: engine/src/operations/activation/hyperbolic.rs:697-745
template <typename T>
T gelu_value(T x, bool approximate) {
  if (approximate) {
    const T coeff = std::sqrt(T(2) / T(3.14159265358979323846264338327950288));
    const T x3 = x * x * x;
    const T inner = coeff * (x + T(0.044715) * x3);
    return T(0.5) * x * (T(1) + std::tanh(inner));
  }
  const T inv_sqrt_2 = T(0.707106781186547524400844362104849039);
  return T(0.5) * x * (T(1) + std::erf(x * inv_sqrt_2));
}

// GeluBackward: engine/src/autograd/mod/linalg.rs:125-264
template <typename T>
T gelu_grad_value(T x, T gout, bool approximate) {
  if (approximate) {
    const T coeff = std::sqrt(T(2) / T(3.14159265358979323846264338327950288));
    const T x2 = x * x;
    const T inner = coeff * (x + T(0.044715) * x * x2);
    const T th = std::tanh(inner);
    const T sech2 = T(1) - th * th;
    const T g = T(0.5) * (T(1) + th) + T(0.5) * x * sech2 * coeff * (T(1) + T(3) * T(0.044715) * x2);
    return gout * g;
  }
  const T inv_sqrt_2 = T(0.707106781186547524400844362104849039);
  const T inv_sqrt_2pi = T(1) / std::sqrt(T(2) * T(3.14159265358979323846264338327950288));
  const T cdf = T(0.5) * (T(1) + std::erf(x * inv_sqrt_2));
  const T pdf = std::exp(T(-0.5) * x * x) * inv_sqrt_2pi;
  return gout * (cdf + x * pdf);
}

// compiler-rt __powidf2, which Rust's f64::powi lowers to (used by adam.rs:249-250).
double powi(double a, int b) {
  const bool recip = b < 0;
  double r = 1.0;
  while (true) {
    if (b & 1) r *= a;
    b /= 2;
    if (b == 0) break;
    a *= a;
  }
  return recip ? 1.0 / r : r;
}

// conv_input_coord: engine/src/autograd/mod/shape.rs:7-41 and the same test in
// engine/src/operations/conv.rs:124-137.
inline bool conv_coord(int64_t oh, int64_t ow, int64_t kh, int64_t kw, int64_t sh, int64_t sw,
                       int64_t ph, int64_t pw, int64_t H, int64_t W, int64_t* ih, int64_t* iw) {
  const int64_t h_in = oh * sh + kh, w_in = ow * sw + kw;
  if (h_in < ph || w_in < pw || h_in >= H + ph || w_in >= W + pw) return false;
  *ih = h_in - ph;
  *iw = w_in - pw;
  return *ih < H && *iw < W;
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------ matmul
void orc_matmul_f32(int64_t batch, int64_t m, int64_t k, int64_t n, const float* a, const float* b, float* c) {
  matmul_float<float>(batch, m, k, n, a, b, c);
}
void orc_matmul_f64(int64_t batch, int64_t m, int64_t k, int64_t n, const double* a, const double* b, double* c) {
  matmul_float<double>(batch, m, k, n, a, b, c);
}
void orc_matmul_i32(int64_t batch, int64_t m, int64_t k, int64_t n, const int32_t* a, const int32_t* b, int32_t* c) {
  matmul_int<uint32_t>(batch, m, k, n, reinterpret_cast<const uint32_t*>(a), reinterpret_cast<const uint32_t*>(b),
                       reinterpret_cast<uint32_t*>(c));
}
void orc_matmul_i64(int64_t batch, int64_t m, int64_t k, int64_t n, const int64_t* a, const int64_t* b, int64_t* c) {
  matmul_int<uint64_t>(batch, m, k, n, reinterpret_cast<const uint64_t*>(a), reinterpret_cast<const uint64_t*>(b),
                       reinterpret_cast<uint64_t*>(c));
}

// f32 inputs, every product and sum carried in f64, result left in f64: the
// value both the reference and the device are compared with at large sizes.
void orc_matmul_f32_acc64(int64_t batch, int64_t m, int64_t k, int64_t n, const float* a, const float* b, double* c) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bi = 0; bi < batch; ++bi)
    for (int64_t i = 0; i < m; ++i) {
      std::vector<double> row(static_cast<size_t>(n), 0.0);
      for (int64_t l = 0; l < k; ++l) {
        const double av = a[bi * m * k + i * k + l];
        const float* brow = b + bi * k * n + l * n;
        for (int64_t j = 0; j < n; ++j) row[j] += av * static_cast<double>(brow[j]);
      }
      std::memcpy(c + bi * m * n + i * n, row.data(), sizeof(double) * n);
    }
}

// Same, f64 inputs carried in long double (checks the f64 device path).
void orc_matmul_f64_acc80(int64_t batch, int64_t m, int64_t k, int64_t n, const double* a, const double* b, double* c) {
#pragma omp parallel for collapse(2) schedule(static)
  for (int64_t bi = 0; bi < batch; ++bi)
    for (int64_t i = 0; i < m; ++i) {
      std::vector<long double> row(static_cast<size_t>(n), 0.0L);
      for (int64_t l = 0; l < k; ++l) {
        const long double av = a[bi * m * k + i * k + l];
        const double* brow = b + bi * k * n + l * n;
        for (int64_t j = 0; j < n; ++j) row[j] += av * static_cast<long double>(brow[j]);
      }
      for (int64_t j = 0; j < n; ++j) c[bi * m * n + i * n + j] = static_cast<double>(row[j]);
    }
}

// Row / column 2-norms that scale the tolerance |delta| <= tol * ||a_row|| * ||b_col||.
void orc_row_norms_f32(int64_t rows, int64_t cols, const float* a, double* out) {
  for (int64_t i = 0; i < rows; ++i) {
    double s = 0;
    for (int64_t j = 0; j < cols; ++j) s += double(a[i * cols + j]) * double(a[i * cols + j]);
    out[i] = std::sqrt(s);
  }
}

void orc_transpose_f32(int64_t batch, int64_t rows, int64_t cols, const float* src, float* dst) {
  transpose_last2<float>(batch, rows, cols, src, dst);
}
void orc_transpose_f64(int64_t batch, int64_t rows, int64_t cols, const double* src, double* dst) {
  transpose_last2<double>(batch, rows, cols, src, dst);
}

// MatMulBackward::backward: engine/src/autograd/mod/core.rs:752-789.
// dA = dY * transpose(B), dB = transpose(A) * dY, transposes materialised.
void orc_matmul_backward_f32(int64_t batch, int64_t m, int64_t k, int64_t n, const float* a, const float* b,
                             const float* dy, float* da /*nullable*/, float* db /*nullable*/) {
  if (da) {
    std::vector<float> bt(static_cast<size_t>(batch * k * n));
    transpose_last2<float>(batch, k, n, b, bt.data());                 // [n,k]
    std::memset(da, 0, sizeof(float) * batch * m * k);
    matmul_float<float>(batch, m, n, k, dy, bt.data(), da);
  }
  if (db) {
    std::vector<float> at(static_cast<size_t>(batch * m * k));
    transpose_last2<float>(batch, m, k, a, at.data());                 // [k,m]
    std::memset(db, 0, sizeof(float) * batch * k * n);
    matmul_float<float>(batch, k, m, n, at.data(), dy, db);
  }
}
void orc_matmul_backward_f64(int64_t batch, int64_t m, int64_t k, int64_t n, const double* a, const double* b,
                             const double* dy, double* da, double* db) {
  if (da) {
    std::vector<double> bt(static_cast<size_t>(batch * k * n));
    transpose_last2<double>(batch, k, n, b, bt.data());
    std::memset(da, 0, sizeof(double) * batch * m * k);
    matmul_float<double>(batch, m, n, k, dy, bt.data(), da);
  }
  if (db) {
    std::vector<double> at(static_cast<size_t>(batch * m * k));
    transpose_last2<double>(batch, m, k, a, at.data());
    std::memset(db, 0, sizeof(double) * batch * k * n);
    matmul_float<double>(batch, k, m, n, at.data(), dy, db);
  }
}

// ------------------------------------------------------------------ DenseLayer
// DenseLayer::forward: engine/src/nn/dense_layer.rs:139-169
//   weight_t = transpose(W [out,in]); y = matmul(x, weight_t); y = y + bias (broadcast
//   [M,N] + [N]: engine/src/operations/arithmetic/kernels.rs:191-334).
void orc_dense_forward_f32(int64_t rows, int64_t in_f, int64_t out_f, const float* x, const float* w,
                           const float* bias /*nullable*/, float* y) {
  std::vector<float> wt(static_cast<size_t>(in_f * out_f));
  transpose_last2<float>(1, out_f, in_f, w, wt.data());
  std::memset(y, 0, sizeof(float) * rows * out_f);
  matmul_float<float>(1, rows, in_f, out_f, x, wt.data(), y);
  if (bias) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < rows; ++i)
      for (int64_t j = 0; j < out_f; ++j) y[i * out_f + j] = y[i * out_f + j] + bias[j];
  }
}

// sum over dim 0 (bias gradient): engine/src/operations/reduction/sum_prod.rs:7-84.
// The reference folds rows with rayon in a split-dependent order; the oracle
// adds rows in ascending order (one of the orders rayon may produce).
void orc_sum_dim0_f32(int64_t rows, int64_t cols, const float* x, float* out) {
  for (int64_t j = 0; j < cols; ++j) out[j] = 0.0f;
  for (int64_t i = 0; i < rows; ++i)
    for (int64_t j = 0; j < cols; ++j) out[j] += x[i * cols + j];
}
void orc_sum_dim0_f64(int64_t rows, int64_t cols, const double* x, double* out) {
  for (int64_t j = 0; j < cols; ++j) out[j] = 0.0;
  for (int64_t i = 0; i < rows; ++i)
    for (int64_t j = 0; j < cols; ++j) out[j] += x[i * cols + j];
}

// ------------------------------------------------------------------ activations
// relu_f32 + mask: engine/src/operations/activation/softmax.rs:161-203
void orc_relu_f32(int64_t n, const float* x, float* y, uint8_t* mask /*nullable*/) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    y[i] = relu_value<float>(x[i]);
    if (mask) mask[i] = (!std::isnan(x[i]) && x[i] > 0.0f) ? 1 : 0;
  }
}
void orc_relu_f64(int64_t n, const double* x, double* y, uint8_t* mask) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    y[i] = relu_value<double>(x[i]);
    if (mask) mask[i] = (!std::isnan(x[i]) && x[i] > 0.0) ? 1 : 0;
  }
}
// ReluBackward: engine/src/autograd/mod/shape.rs:730-816: go * (mask ? 1 : 0)
void orc_relu_backward_f32(int64_t n, const uint8_t* mask, const float* go, float* gi) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) gi[i] = go[i] * (mask[i] ? 1.0f : 0.0f);
}
void orc_relu_backward_f64(int64_t n, const uint8_t* mask, const double* go, double* gi) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) gi[i] = go[i] * (mask[i] ? 1.0 : 0.0);
}
void orc_gelu_f32(int64_t n, const float* x, float* y, int approximate) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) y[i] = gelu_value<float>(x[i], approximate != 0);
}
void orc_gelu_f64(int64_t n, const double* x, double* y, int approximate) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) y[i] = gelu_value<double>(x[i], approximate != 0);
}
void orc_gelu_backward_f32(int64_t n, const float* x, const float* go, float* gi, int approximate) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) gi[i] = gelu_grad_value<float>(x[i], go[i], approximate != 0);
}
void orc_gelu_backward_f64(int64_t n, const double* x, const double* go, double* gi, int approximate) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) gi[i] = gelu_grad_value<double>(x[i], go[i], approximate != 0);
}

// ------------------------------------------------------------------ conv2d
// conv2d: engine/src/operations/conv.rs:24-206 (hot loop :111-157).  Returns 0,
// or 1 for the error cases of :67-79 (stride 0, kernel larger than padded input).
int orc_conv2d_f32(int64_t N, int64_t C, int64_t H, int64_t W, int64_t O, int64_t KH, int64_t KW, int64_t sh,
                   int64_t sw, int64_t ph, int64_t pw, const float* x, const float* w, const float* bias, float* y) {
  if (sh == 0 || sw == 0) return 1;
  if (KH > H + 2 * ph || KW > W + 2 * pw) return 1;
  const int64_t OH = (H + 2 * ph - KH) / sh + 1, OW = (W + 2 * pw - KW) / sw + 1;
#pragma omp parallel for schedule(static)
  for (int64_t chunk = 0; chunk < N * O; ++chunk) {
    const int64_t n = chunk / O, oc = chunk % O;
    float* out = y + chunk * OH * OW;
    for (int64_t oh = 0; oh < OH; ++oh)
      for (int64_t ow = 0; ow < OW; ++ow) {
        float sum = 0.0f;
        for (int64_t ic = 0; ic < C; ++ic)
          for (int64_t kh = 0; kh < KH; ++kh)
            for (int64_t kw = 0; kw < KW; ++kw) {
              int64_t ih, iw;
              if (!conv_coord(oh, ow, kh, kw, sh, sw, ph, pw, H, W, &ih, &iw)) continue;
              // `sum += a * b` in Rust is a separate multiply and add (no contraction)
              const float prod = x[((n * C + ic) * H + ih) * W + iw] * w[((oc * C + ic) * KH + kh) * KW + kw];
              sum = sum + prod;
            }
        if (bias) sum += bias[oc];
        out[oh * OW + ow] = sum;
      }
  }
  return 0;
}

// Conv2dBackward::backward: engine/src/autograd/mod/shape.rs:57-197.
void orc_conv2d_backward_f32(int64_t N, int64_t C, int64_t H, int64_t W, int64_t O, int64_t KH, int64_t KW,
                             int64_t sh, int64_t sw, int64_t ph, int64_t pw, const float* x, const float* w,
                             const float* go, float* gx /*nullable*/, float* gw /*nullable*/,
                             float* gb /*nullable*/) {
  const int64_t OH = (H + 2 * ph - KH) / sh + 1, OW = (W + 2 * pw - KW) / sw + 1;
  if (gx) {  // :86-127, parallel over images
    std::memset(gx, 0, sizeof(float) * N * C * H * W);
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      float* gi = gx + n * C * H * W;
      for (int64_t oc = 0; oc < O; ++oc) {
        const int64_t w_base = oc * C * KH * KW;
        for (int64_t oh = 0; oh < OH; ++oh)
          for (int64_t ow = 0; ow < OW; ++ow) {
            const float g = go[((n * O + oc) * OH + oh) * OW + ow];
            for (int64_t kh = 0; kh < KH; ++kh)
              for (int64_t kw = 0; kw < KW; ++kw) {
                int64_t ih, iw;
                if (!conv_coord(oh, ow, kh, kw, sh, sw, ph, pw, H, W, &ih, &iw)) continue;
                const int64_t spatial = ih * W + iw;
                for (int64_t ic = 0; ic < C; ++ic) {
                  const float prod = g * w[w_base + (ic * KH + kh) * KW + kw];
                  gi[ic * H * W + spatial] = gi[ic * H * W + spatial] + prod;
                }
              }
          }
      }
    }
  }
  if (gw) {  // :130-169, parallel over output channels
    std::memset(gw, 0, sizeof(float) * O * C * KH * KW);
#pragma omp parallel for schedule(static)
    for (int64_t oc = 0; oc < O; ++oc) {
      float* g_w = gw + oc * C * KH * KW;
      for (int64_t n = 0; n < N; ++n)
        for (int64_t oh = 0; oh < OH; ++oh)
          for (int64_t ow = 0; ow < OW; ++ow) {
            const float g = go[((n * O + oc) * OH + oh) * OW + ow];
            for (int64_t kh = 0; kh < KH; ++kh)
              for (int64_t kw = 0; kw < KW; ++kw) {
                int64_t ih, iw;
                if (!conv_coord(oh, ow, kh, kw, sh, sw, ph, pw, H, W, &ih, &iw)) continue;
                const int64_t spatial = ih * W + iw;
                for (int64_t ic = 0; ic < C; ++ic) {
                  const float prod = g * x[(n * C + ic) * H * W + spatial];
                  g_w[(ic * KH + kh) * KW + kw] = g_w[(ic * KH + kh) * KW + kw] + prod;
                }
              }
          }
    }
  }
  if (gb) {  // :172-194
#pragma omp parallel for schedule(static)
    for (int64_t oc = 0; oc < O; ++oc) {
      float sum = 0.0f;
      for (int64_t n = 0; n < N; ++n) {
        const int64_t base = (n * O + oc) * OH * OW;
        for (int64_t q = 0; q < OH * OW; ++q) sum += go[base + q];
      }
      gb[oc] = sum;
    }
  }
}

// ------------------------------------------------------------------ cross entropy
// cross_entropy_loss with class-index targets, reduction mean (1) or sum (0):
// engine/src/operations/loss/regression.rs:178-251 (+ one-hot :769-862,
// log_softmax engine/src/operations/activation/softmax.rs:848-901, negative
// log likelihood engine/src/operations/loss/classification.rs:446-450).
// grad = (softmax - onehot) * (1/B if mean) * upstream:
// engine/src/autograd/mod/activation.rs:364-427.  Returns 1 on a bad label.
int orc_cross_entropy_f32(int64_t B, int64_t C, const float* logits, const int64_t* labels, int mean,
                          float upstream, float* loss, float* grad /*nullable*/) {
  for (int64_t i = 0; i < B; ++i)
    if (labels[i] < 0 || labels[i] >= C) return 1;
  std::vector<float> per_sample(static_cast<size_t>(B));
  const float inv_b = static_cast<float>(1.0 / static_cast<double>(B));
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < B; ++i) {
    const float* x = logits + i * C;
    float mx = -std::numeric_limits<float>::infinity();
    for (int64_t c = 0; c < C; ++c)
      if (x[c] > mx) mx = x[c];
    std::vector<float> lp(static_cast<size_t>(C));
    if (std::isinf(mx) && mx < 0) {
      for (int64_t c = 0; c < C; ++c) lp[c] = -std::numeric_limits<float>::infinity();
    } else {
      float s = 0.0f;
      for (int64_t c = 0; c < C; ++c) s = s + std::exp(x[c] - mx);
      const float logsum = std::log(s) + mx;
      for (int64_t c = 0; c < C; ++c) lp[c] = x[c] - logsum;
    }
    float row = 0.0f;
    for (int64_t c = 0; c < C; ++c) {
      const float sm = std::exp(lp[c]);                       // softmax = exp(log_softmax)
      const float onehot = (c == labels[i]) ? 1.0f : 0.0f;
      const float lpm = (sm <= 1e-30f) ? -std::numeric_limits<float>::infinity() : lp[c];
      const float nll = -(lpm * onehot);                      // -inf * 0 = NaN, as in the reference
      row = row + nll;                                        // sum over dim 1
      if (grad) {
        float g = sm - onehot;
        if (mean) g = g * inv_b;
        grad[i * C + c] = g * upstream;
      }
    }
    per_sample[i] = row;
  }
  float total = 0.0f;  // sum_all_elements: the reference's order is rayon-dependent; ascending here
  for (int64_t i = 0; i < B; ++i) total += per_sample[i];
  *loss = mean ? static_cast<float>(static_cast<double>(total) / static_cast<double>(B)) : total;
  return 0;
}

// cross_entropy_loss in its general form (engine/src/operations/loss/regression.rs:178-251): targets are
// class indices (one-hot: :769-862) or a [B][C] float matrix used as it is; per-sample loss
// = -sum_c t[c] * masked_log_softmax[c] (classification.rs:446-450, sum over dim 1 in class order);
// reduction 0 = sum, 1 = mean, 2 = none (row_loss[B]).  Gradient (engine/src/autograd/mod/activation.rs:364-427):
// (softmax - t) * (1/B if mean) * upstream, with upstream a scalar times an optional per-sample factor
// (the reference multiplies by grad_output with its generic broadcast, which for a [B] gradient of a
// "none" loss only type-checks when B == C; the per-sample factor is the meaning of that product).
int orc_cross_entropy_ex_f32(int64_t B, int64_t C, const float* logits, const int64_t* labels /*nullable*/,
                             const float* soft /*nullable*/, int reduction, float upstream,
                             const float* upstream_rows /*nullable*/, float* loss /*1 or B*/,
                             float* grad /*nullable*/) {
  if (labels)
    for (int64_t i = 0; i < B; ++i)
      if (labels[i] < 0 || labels[i] >= C) return 1;
  std::vector<float> per_sample(static_cast<size_t>(B));
  const float inv_b = static_cast<float>(1.0 / static_cast<double>(B));
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < B; ++i) {
    const float* x = logits + i * C;
    float mx = -std::numeric_limits<float>::infinity();
    for (int64_t c = 0; c < C; ++c)
      if (x[c] > mx) mx = x[c];
    std::vector<float> lp(static_cast<size_t>(C));
    if (std::isinf(mx) && mx < 0) {
      for (int64_t c = 0; c < C; ++c) lp[c] = -std::numeric_limits<float>::infinity();
    } else {
      float s = 0.0f;
      for (int64_t c = 0; c < C; ++c) s = s + std::exp(x[c] - mx);
      const float logsum = std::log(s) + mx;
      for (int64_t c = 0; c < C; ++c) lp[c] = x[c] - logsum;
    }
    float row = 0.0f;
    for (int64_t c = 0; c < C; ++c) {
      const float sm = std::exp(lp[c]);
      const float t = labels ? ((c == labels[i]) ? 1.0f : 0.0f) : soft[i * C + c];
      const float lpm = (sm <= 1e-30f) ? -std::numeric_limits<float>::infinity() : lp[c];
      row = row + (-(lpm * t));
      if (grad) {
        float g = sm - t;
        if (reduction == 1) g = g * inv_b;
        g = g * upstream;
        if (upstream_rows) g = g * upstream_rows[i];
        grad[i * C + c] = g;
      }
    }
    per_sample[i] = row;
  }
  if (reduction == 2) {
    for (int64_t i = 0; i < B; ++i) loss[i] = per_sample[i];
    return 0;
  }
  float total = 0.0f;
  for (int64_t i = 0; i < B; ++i) total += per_sample[i];
  *loss = reduction == 1 ? static_cast<float>(static_cast<double>(total) / static_cast<double>(B)) : total;
  return 0;
}

// ------------------------------------------------------------------ SGD, RMSprop, gradient clipping
// SGD::apply_simple_update / apply_momentum_update (engine/src/optim/sgd.rs:169-296): every constant is
// cast to the element type first, each operation is rounded separately.
}  // extern "C"
template <typename T>
static void sgd_step(int64_t n, T* p, const T* g, T* v /*nullable*/, double lr_, double momentum_, double damp_,
                     double wd_, int nesterov) {
  const T lr = static_cast<T>(lr_), momentum = static_cast<T>(momentum_), damp = static_cast<T>(damp_),
          wd = static_cast<T>(wd_);
  const T one_minus_damp = static_cast<T>(1.0) - damp;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    volatile T t;
    t = wd * p[i];
    const T grad_val = g[i] + t;
    if (momentum_ > 0.0) {
      t = momentum * v[i];
      T u = one_minus_damp * grad_val;
      const T vi = t + u;
      v[i] = vi;
      T update = vi;
      if (nesterov) { t = momentum * vi; update = grad_val + t; }
      t = lr * update;
      p[i] = p[i] - t;
    } else {
      t = lr * grad_val;
      p[i] = p[i] - t;
    }
  }
}
extern "C" {
void orc_sgd_step_f32(int64_t n, float* p, const float* g, float* v, double lr, double momentum, double damp,
                      double wd, int nesterov) { sgd_step<float>(n, p, g, v, lr, momentum, damp, wd, nesterov); }
void orc_sgd_step_f64(int64_t n, double* p, const double* g, double* v, double lr, double momentum, double damp,
                      double wd, int nesterov) { sgd_step<double>(n, p, g, v, lr, momentum, damp, wd, nesterov); }

// RMSprop::apply_rmsprop_update (engine/src/optim/rmsprop.rs:187-383): the four (momentum, centered) variants.
}  // extern "C"
template <typename T>
static void rmsprop_step(int64_t n, T* p, const T* g, T* sq, T* mb /*nullable*/, T* ga /*nullable*/, double lr_,
                         double alpha_, double eps_, double wd_, double momentum_) {
  const T lr = static_cast<T>(lr_), alpha = static_cast<T>(alpha_), eps = static_cast<T>(eps_),
          wd = static_cast<T>(wd_), momentum = static_cast<T>(momentum_);
  const T oma = static_cast<T>(1.0) - alpha;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    volatile T t;
    t = wd * p[i];
    const T gv = g[i] + t;
    t = alpha * sq[i];
    T u = oma * gv;
    u = u * gv;
    const T sqi = t + u;
    sq[i] = sqi;
    T avg = sqi;
    if (ga) {
      t = alpha * ga[i];
      u = oma * gv;
      const T gai = t + u;
      ga[i] = gai;
      t = gai * gai;
      avg = sqi - t;
    }
    const T denom = std::sqrt(avg) + eps;
    t = lr * gv;
    const T stepv = t / denom;
    if (mb) {
      t = momentum * mb[i];
      const T mbi = t + stepv;
      mb[i] = mbi;
      p[i] = p[i] - mbi;
    } else {
      p[i] = p[i] - stepv;
    }
  }
}
extern "C" {
void orc_rmsprop_step_f32(int64_t n, float* p, const float* g, float* sq, float* mb, float* ga, double lr,
                          double alpha, double eps, double wd, double momentum) {
  rmsprop_step<float>(n, p, g, sq, mb, ga, lr, alpha, eps, wd, momentum);
}
void orc_rmsprop_step_f64(int64_t n, double* p, const double* g, double* sq, double* mb, double* ga, double lr,
                          double alpha, double eps, double wd, double momentum) {
  rmsprop_step<double>(n, p, g, sq, mb, ga, lr, alpha, eps, wd, momentum);
}

// GradientUtils (engine/src/optim/utils.rs:16-112): sum of squares in f64 (the reference's order is
// rayon-dependent; ascending here), scale by a coefficient cast to the element type, clamp (NaN stays NaN).
double orc_sumsq_f32(int64_t n, const float* x) {
  double s = 0.0;
  for (int64_t i = 0; i < n; ++i) s += static_cast<double>(x[i]) * static_cast<double>(x[i]);
  return s;
}
double orc_sumsq_f64(int64_t n, const double* x) {
  double s = 0.0;
  for (int64_t i = 0; i < n; ++i) s += x[i] * x[i];
  return s;
}
void orc_scale_f32(int64_t n, float* x, double coef) {
  const float c = static_cast<float>(coef);
  for (int64_t i = 0; i < n; ++i) x[i] = x[i] * c;
}
void orc_scale_f64(int64_t n, double* x, double coef) {
  for (int64_t i = 0; i < n; ++i) x[i] = x[i] * coef;
}
void orc_clamp_f32(int64_t n, float* x, double lo_, double hi_) {
  const float lo = static_cast<float>(lo_), hi = static_cast<float>(hi_);
  for (int64_t i = 0; i < n; ++i) x[i] = x[i] < lo ? lo : (x[i] > hi ? hi : x[i]);
}
void orc_clamp_f64(int64_t n, double* x, double lo, double hi) {
  for (int64_t i = 0; i < n; ++i) x[i] = x[i] < lo ? lo : (x[i] > hi ? hi : x[i]);
}

// ------------------------------------------------------------------ batch norm, dropout
}  // extern "C"
// batch_norm (engine/src/operations/normalization.rs:64-187) on x [N][C][S] (S = product of the trailing
// dimensions): statistics per channel over N and S, biased variance, y = (x - mean) / sqrt(var + eps) * w + b;
// batch statistics are used when training or when a running estimate is missing; while training the running
// estimates become running * (1 - momentum) + batch * momentum.  Sums are accumulated in f64 here (the
// reference's f32 sums depend on its thread count), element arithmetic in T.
template <typename T>
static void batch_norm_fwd(int64_t N, int64_t C, int64_t S, const T* x, const T* w, const T* b, T* rm, T* rv,
                           int training, double momentum, double eps, T* y, T* save_mean, T* save_invstd) {
  const bool batch_stats = training || !rm || !rv;
  const double cnt = static_cast<double>(N) * static_cast<double>(S);
  for (int64_t c = 0; c < C; ++c) {
    T mean, var;
    if (batch_stats) {
      double s = 0.0;
      for (int64_t n = 0; n < N; ++n)
        for (int64_t i = 0; i < S; ++i) s += x[(n * C + c) * S + i];
      mean = static_cast<T>(s / cnt);
      double q = 0.0;
      for (int64_t n = 0; n < N; ++n)
        for (int64_t i = 0; i < S; ++i) {
          const T d = x[(n * C + c) * S + i] - mean;
          q += static_cast<double>(d * d);
        }
      var = static_cast<T>(q / cnt);
    } else {
      mean = rm[c];
      var = rv[c];
    }
    const T stdv = std::sqrt(var + static_cast<T>(eps));
    for (int64_t n = 0; n < N; ++n)
      for (int64_t i = 0; i < S; ++i) {
        T o = (x[(n * C + c) * S + i] - mean) / stdv;
        if (w) o = o * w[c];
        if (b) o = o + b[c];
        y[(n * C + c) * S + i] = o;
      }
    if (save_mean) save_mean[c] = mean;
    if (save_invstd) save_invstd[c] = static_cast<T>(1) / stdv;
    if (training && rm && rv) {
      const T m = static_cast<T>(momentum), om = static_cast<T>(1.0 - momentum);
      rm[c] = rm[c] * om + mean * m;
      rv[c] = rv[c] * om + var * m;
    }
  }
}
// Gradient of the composition above (the reference differentiates it operator by operator): with
// xh = (x - mean) * invstd, db = sum dy, dw = sum dy * xh, and for batch statistics
// dx = w * invstd * (dy - db/n - xh * dw/n); with fixed (running) statistics dx = w * invstd * dy.
template <typename T>
static void batch_norm_bwd(int64_t N, int64_t C, int64_t S, const T* x, const T* dy, const T* w, const T* mean,
                           const T* invstd, int batch_stats, T* dx, T* dw, T* db) {
  const double cnt = static_cast<double>(N) * static_cast<double>(S);
  for (int64_t c = 0; c < C; ++c) {
    double sb = 0.0, sw = 0.0;
    for (int64_t n = 0; n < N; ++n)
      for (int64_t i = 0; i < S; ++i) {
        const int64_t k = (n * C + c) * S + i;
        const double xh = (static_cast<double>(x[k]) - mean[c]) * invstd[c];
        sb += dy[k];
        sw += dy[k] * xh;
      }
    if (db) db[c] = static_cast<T>(sb);
    if (dw) dw[c] = static_cast<T>(sw);
    if (dx) {
      const double g = (w ? static_cast<double>(w[c]) : 1.0) * invstd[c];
      for (int64_t n = 0; n < N; ++n)
        for (int64_t i = 0; i < S; ++i) {
          const int64_t k = (n * C + c) * S + i;
          const double xh = (static_cast<double>(x[k]) - mean[c]) * invstd[c];
          dx[k] = static_cast<T>(batch_stats ? g * (dy[k] - sb / cnt - xh * sw / cnt) : g * dy[k]);
        }
    }
  }
}
extern "C" {
void orc_batch_norm_fwd_f32(int64_t N, int64_t C, int64_t S, const float* x, const float* w, const float* b, float* rm,
                            float* rv, int training, double momentum, double eps, float* y, float* save_mean,
                            float* save_invstd) {
  batch_norm_fwd<float>(N, C, S, x, w, b, rm, rv, training, momentum, eps, y, save_mean, save_invstd);
}
void orc_batch_norm_fwd_f64(int64_t N, int64_t C, int64_t S, const double* x, const double* w, const double* b,
                            double* rm, double* rv, int training, double momentum, double eps, double* y,
                            double* save_mean, double* save_invstd) {
  batch_norm_fwd<double>(N, C, S, x, w, b, rm, rv, training, momentum, eps, y, save_mean, save_invstd);
}
void orc_batch_norm_bwd_f32(int64_t N, int64_t C, int64_t S, const float* x, const float* dy, const float* w,
                            const float* mean, const float* invstd, int batch_stats, float* dx, float* dw, float* db) {
  batch_norm_bwd<float>(N, C, S, x, dy, w, mean, invstd, batch_stats, dx, dw, db);
}
void orc_batch_norm_bwd_f64(int64_t N, int64_t C, int64_t S, const double* x, const double* dy, const double* w,
                            const double* mean, const double* invstd, int batch_stats, double* dx, double* dw,
                            double* db) {
  batch_norm_bwd<double>(N, C, S, x, dy, w, mean, invstd, batch_stats, dx, dw, db);
}

// Dropout mask (engine/src/nn/dropout.rs:21-92): entries are 1/(1-p) with probability 1-p, else 0; p >= 1 gives
// zeros, p <= 0 ones.  The reference draws from its thread-local StdRng, whose stream cannot be reproduced
// outside it; this build's generator is counter-based: with g = offset + j, entry j of a mask keeps when a 24-bit
// field of mix64(seed + (g / 2 + 1) * 0x9E3779B97F4A7C15) is below keep * 2^24 - bits 63..40 for even g, bits
// 39..16 for odd g - mix64 being the splitmix64 finaliser.
static inline uint64_t mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}
void orc_dropout_mask_f32(int64_t n, double p, uint64_t seed, uint64_t offset, float* mask) {
  const double keep = 1.0 - p;
  const float scale = 1.0f / static_cast<float>(keep);
  const uint32_t thresh = static_cast<uint32_t>(keep * 16777216.0);
  for (int64_t j = 0; j < n; ++j) {
    if (keep >= 1.0) { mask[j] = 1.0f; continue; }
    if (keep <= 0.0) { mask[j] = 0.0f; continue; }
    const uint64_t g = offset + static_cast<uint64_t>(j);
    const uint64_t hsh = mix64(seed + ((g >> 1) + 1) * 0x9E3779B97F4A7C15ULL);
    const uint32_t u = static_cast<uint32_t>((g & 1) ? (hsh >> 16) : (hsh >> 40)) & 0xFFFFFFu;
    mask[j] = u < thresh ? scale : 0.0f;
  }
}

// ------------------------------------------------------------------ Adam
// Adam::apply_adam_update, no amsgrad: engine/src/optim/adam.rs:245-312.
void orc_adam_step_f32(int64_t n, float* p, const float* g, float* m, float* v, double lr, double beta1,
                       double beta2, double eps, double weight_decay, int decoupled, int64_t step) {
  const double b1p = powi(beta1, static_cast<int>(step)), b2p = powi(beta2, static_cast<int>(step));
  const float bc1_inv = static_cast<float>(1.0 / (1.0 - b1p));
  const float bc2_inv = static_cast<float>(1.0 / (1.0 - b2p));
  const bool use_decoupled = decoupled && weight_decay != 0.0;
  const float lrf = static_cast<float>(lr), b1 = static_cast<float>(beta1), b2 = static_cast<float>(beta2);
  const float wd = static_cast<float>(weight_decay), epsf = static_cast<float>(eps);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    volatile float t;  // keeps each step a separately rounded f32 operation
    float pi = p[i];
    if (use_decoupled) { t = lrf * wd; t = t * pi; pi = pi - t; }
    float gv = g[i];
    if (!use_decoupled) { t = wd * pi; gv = gv + t; }
    t = b1 * m[i]; float u = (1.0f - b1) * gv; const float mi = t + u;
    t = b2 * v[i]; u = (1.0f - b2) * gv; u = u * gv; const float vi = t + u;
    m[i] = mi;
    v[i] = vi;
    const float m_hat = mi * bc1_inv;
    const float v_hat = vi * bc2_inv;
    t = std::sqrt(v_hat) + epsf;
    u = lrf * m_hat;
    p[i] = pi - u / t;
  }
}

// ------------------------------------------------------------------ MLP step
// One training step of Sequential[DenseLayer, ReLU, ..., DenseLayer] +
// CrossEntropyLoss(mean) + Adam, as the reference executes it
// (engine/src/nn/sequential.rs:74-83, dense_layer.rs:139-169, nn/activation.rs:88-91,
// nn/loss.rs:434-436, autograd/graph.rs:222-282, optim/adam.rs:483-514), including
// the transposes it materialises.  dims = [in, h1, ..., out] (nlayers + 1 entries).
// params / m / v: per layer W [out,in] then b [out], concatenated in layer order.
// grads (nullable) receives the gradients in the same layout.  Returns the loss.
float orc_mlp_train_step_f32(int64_t nlayers, const int64_t* dims, int64_t batch, const float* x,
                             const int64_t* labels, float* params, float* m, float* v, float* grads_out, double lr,
                             double beta1, double beta2, double eps, int64_t step) {
  std::vector<size_t> w_off(nlayers), b_off(nlayers);
  size_t total = 0;
  for (int64_t l = 0; l < nlayers; ++l) {
    w_off[l] = total; total += static_cast<size_t>(dims[l] * dims[l + 1]);
    b_off[l] = total; total += static_cast<size_t>(dims[l + 1]);
  }
  std::vector<float> grads(total, 0.0f);
  std::vector<std::vector<float>> act(nlayers + 1);   // act[l] = input of layer l (post-ReLU of l-1)
  std::vector<std::vector<uint8_t>> mask(nlayers);
  act[0].assign(x, x + batch * dims[0]);
  for (int64_t l = 0; l < nlayers; ++l) {
    const int64_t in_f = dims[l], out_f = dims[l + 1];
    std::vector<float> z(static_cast<size_t>(batch * out_f));
    orc_dense_forward_f32(batch, in_f, out_f, act[l].data(), params + w_off[l], params + b_off[l], z.data());
    if (l + 1 < nlayers) {
      act[l + 1].resize(z.size());
      mask[l].resize(z.size());
      orc_relu_f32(static_cast<int64_t>(z.size()), z.data(), act[l + 1].data(), mask[l].data());
    } else {
      act[l + 1] = std::move(z);
    }
  }
  float loss = 0.0f;
  const int64_t ncls = dims[nlayers];
  std::vector<float> g(static_cast<size_t>(batch * ncls));
  orc_cross_entropy_f32(batch, ncls, act[nlayers].data(), labels, 1, 1.0f, &loss, g.data());
  for (int64_t l = nlayers - 1; l >= 0; --l) {
    const int64_t in_f = dims[l], out_f = dims[l + 1];
    // AddBackward -> bias gradient = sum over dim 0
    orc_sum_dim0_f32(batch, out_f, g.data(), grads.data() + b_off[l]);
    // MatMulBackward on y = x * Wt (Wt = transpose(W), [in,out]):
    //   dX = dY * transpose(Wt) ; dWt = transpose(x) * dY ; TransposeBackward: dW = transpose(dWt)
    std::vector<float> wt(static_cast<size_t>(in_f * out_f));
    transpose_last2<float>(1, out_f, in_f, params + w_off[l], wt.data());
    std::vector<float> dx, dwt(static_cast<size_t>(in_f * out_f));
    const bool need_dx = l > 0;  // the network input does not require grad (core.rs:763)
    if (need_dx) dx.resize(static_cast<size_t>(batch * in_f));
    orc_matmul_backward_f32(1, batch, in_f, out_f, act[l].data(), wt.data(), g.data(), need_dx ? dx.data() : nullptr,
                            dwt.data());
    transpose_last2<float>(1, in_f, out_f, dwt.data(), grads.data() + w_off[l]);
    if (need_dx) {
      g.resize(dx.size());
      orc_relu_backward_f32(static_cast<int64_t>(dx.size()), mask[l - 1].data(), dx.data(), g.data());
    }
  }
  if (grads_out) std::memcpy(grads_out, grads.data(), sizeof(float) * total);
  orc_adam_step_f32(static_cast<int64_t>(total), params, grads.data(), m, v, lr, beta1, beta2, eps, 0.0, 0, step);
  return loss;
}

}  // extern "C"
