// GEMM kernels for the element types the tcgen05 pipe has no kind for.
//
//  * f64: warp-level FP64 tensor-core MMA (mma.sync m8n8k4, f64 accumulate),
//    operands staged in shared memory.  Replaces the dgemm call of the
//    reference (engine/src/operations/linalg/matmul.rs:250-258).
//  * i32 / i64: exact wrapping integer multiply-add on the CUDA cores, same
//    result as the reference triple loop `sum = sum + a*b` in release builds
//    (engine/src/operations/linalg/diagonal.rs:495-548): addition and
//    multiplication modulo 2^32 / 2^64 are associative, so the order of the
//    partial sums cannot change the answer.
//  * f32 on the CUDA cores (same kernel, T = float): plain IEEE multiply-add,
//    run only when an operand of the split-bf16 tensor path held an Inf or
//    NaN, because Inf times the zero low-order split of a finite value would
//    turn the reference's Inf results into NaN.
//
// Operand addressing is by strides so the same kernels serve the NN / NT / TN
// / TT forms: element (i, k) of A is A[i*a_si + k*a_sk], element (k, j) of B
// is B[k*b_sk + j*b_sj].
#pragma once
#include "ptx_sm100.cuh"
#include <cstdint>
#include <type_traits>

namespace mtb {

struct StridedGemmArgs {
  int M, N, K, batch;
  const void* A;
  const void* B;
  void* C;
  long long a_si, a_sk, a_sb;  // element strides of A: row (M), reduction (K), batch
  long long b_sk, b_sj, b_sb;  // element strides of B: reduction (K), column (N), batch
  long long ldc, c_sb;
  const void* bias;            // [N] or nullptr
  const void* aux;             // layout of C, for EPI_RELU_BWD
  int epilogue;
  const uint32_t* gate;        // optional: the kernel runs only when *gate == gate_value
  uint32_t gate_value;
};

__device__ __forceinline__ double apply_epilogue_f64(double x, int epi, double aux) {
  switch (epi) {
    case 1: return (x != x) ? x : (x > 0.0 ? x : 0.0);
    case 2: return 0.5 * x * (1.0 + erf(x * 0.70710678118654752440));
    case 3: {
      const double c = 0.79788456080286535588;
      return 0.5 * x * (1.0 + tanh(c * (x + 0.044715 * x * x * x)));
    }
    case 4: return x * (aux > 0.0 ? 1.0 : 0.0);
    default: return x;
  }
}

// ------------------------------------------------------------------ f64
// Block tile 128 x 128 x 16, 8 warps as 2 (M) x 4 (N), warp tile 64 x 32 =
// 8 x 4 MMA tiles.  Shared tiles are stored [k][i] with a row pitch of 132
// doubles: the fragment reads (k = lane%4, i = lane/4) of one half-warp then
// hit 16 distinct bank pairs.
constexpr int D_BM = 128, D_BN = 128, D_BK = 16, D_PITCH = 132;

__device__ __forceinline__ void dmma_m8n8k4(double (&c)[2], double a, double b) {
  asm volatile(
      "mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
      : "+d"(c[0]), "+d"(c[1])
      : "d"(a), "d"(b));
}

// Load a (rows i0.., k0..) tile of `rows` x 16 into registers, ROWS * 16 / NT per thread.
// The thread->element map follows whichever stride is 1 so reads coalesce.
template <int ROWS, int NT>
__device__ __forceinline__ void dgemm_fetch(const double* __restrict__ base, long long s_i,
                                            long long s_k, int i0, int k0, int imax, int kmax,
                                            double (&r)[ROWS * D_BK / NT]) {
  constexpr int PER = ROWS * D_BK / NT;
  const int tid = threadIdx.x;
  if (s_i == 1) {  // contiguous along i
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int idx = tid + e * NT;
      const int i = idx % ROWS, k = idx / ROWS;
      const bool ok = (i0 + i < imax) && (k0 + k < kmax);
      r[e] = ok ? base[(long long)(i0 + i) * s_i + (long long)(k0 + k) * s_k] : 0.0;
    }
  } else {  // contiguous (or at least closest) along k
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const int idx = tid + e * NT;
      const int k = idx % D_BK, i = idx / D_BK;
      const bool ok = (i0 + i < imax) && (k0 + k < kmax);
      r[e] = ok ? base[(long long)(i0 + i) * s_i + (long long)(k0 + k) * s_k] : 0.0;
    }
  }
}
template <int ROWS, int NT>
__device__ __forceinline__ void dgemm_stash(double* __restrict__ sm, long long s_i,
                                            const double (&r)[ROWS * D_BK / NT]) {
  constexpr int PER = ROWS * D_BK / NT;
  const int tid = threadIdx.x;
#pragma unroll
  for (int e = 0; e < PER; ++e) {
    const int idx = tid + e * NT;
    int i, k;
    if (s_i == 1) { i = idx % ROWS; k = idx / ROWS; } else { k = idx % D_BK; i = idx / D_BK; }
    sm[k * D_PITCH + i] = r[e];
  }
}

// WM x WN warps; each warp owns a (128 / WM) x (128 / WN) piece of the block tile.  2 x 4 (64 x 32 per warp, 256
// threads) is what runs: it reads the least shared memory per MMA.  Measured at 4096^3 on B200: 2 x 4 27.4 TFLOP/s,
// 4 x 4 (512 threads, four warps per scheduler) 26.5, and the same tile on mma.sync.m16n8k16 26.4 - the warp
// layout and the MMA shape are not what holds the kernel at 0.74 of the 37.1 TFLOP/s an MMA-only loop reaches.
// Nor is the register staging: the same tile fed by three or four stages of 8-byte cp.async copies, with the
// fragments of the next k step loaded while the current one multiplies, measured 24.9.
template <int WM, int WN>
static __global__ void __launch_bounds__(32 * WM * WN, 1) gemm_f64_dmma_kernel(const StridedGemmArgs g) {
  constexpr int NT = 32 * WM * WN;
  constexpr int TM = D_BM / WM, TN = D_BN / WN;     // warp tile
  constexpr int FI = TM / 8, FJ = TN / 8;           // 8 x 8 MMA tiles per warp tile
  constexpr int PER = D_BM * D_BK / NT;
  extern __shared__ __align__(16) uint8_t dsm_raw[];
  double* As = reinterpret_cast<double*>(dsm_raw);  // [2][D_BK][D_PITCH]
  double* Bs = As + 2 * D_BK * D_PITCH;             // [2][D_BK][D_PITCH]

  const int tiles_n = (g.N + D_BN - 1) / D_BN;
  const int tm = blockIdx.x / tiles_n, tn = blockIdx.x % tiles_n;
  const int b = blockIdx.y;
  const double* A = static_cast<const double*>(g.A) + b * g.a_sb;
  const double* B = static_cast<const double*>(g.B) + b * g.b_sb;
  double* C = static_cast<double*>(g.C) + b * g.c_sb;
  const double* AUX = g.aux ? static_cast<const double*>(g.aux) + b * g.c_sb : nullptr;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wm = warp / WN, wn = warp % WN;
  const int fr = lane >> 2, fk = lane & 3;

  double acc[FI][FJ][2];
#pragma unroll
  for (int i = 0; i < FI; ++i)
#pragma unroll
    for (int j = 0; j < FJ; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

  const int nkb = (g.K + D_BK - 1) / D_BK;
  double ra[PER], rb[PER];
  dgemm_fetch<D_BM, NT>(A, g.a_si, g.a_sk, tm * D_BM, 0, g.M, g.K, ra);
  dgemm_fetch<D_BN, NT>(B, g.b_sj, g.b_sk, tn * D_BN, 0, g.N, g.K, rb);
  dgemm_stash<D_BM, NT>(As, g.a_si, ra);
  dgemm_stash<D_BN, NT>(Bs, g.b_sj, rb);
  __syncthreads();

  for (int kb = 0; kb < nkb; ++kb) {
    const int cur = kb & 1;
    if (kb + 1 < nkb) {
      dgemm_fetch<D_BM, NT>(A, g.a_si, g.a_sk, tm * D_BM, (kb + 1) * D_BK, g.M, g.K, ra);
      dgemm_fetch<D_BN, NT>(B, g.b_sj, g.b_sk, tn * D_BN, (kb + 1) * D_BK, g.N, g.K, rb);
    }
    const double* as = As + cur * D_BK * D_PITCH;
    const double* bs = Bs + cur * D_BK * D_PITCH;
#pragma unroll
    for (int k4 = 0; k4 < D_BK / 4; ++k4) {
      double af[FI], bf[FJ];
#pragma unroll
      for (int i = 0; i < FI; ++i) af[i] = as[(k4 * 4 + fk) * D_PITCH + wm * TM + i * 8 + fr];
#pragma unroll
      for (int j = 0; j < FJ; ++j) bf[j] = bs[(k4 * 4 + fk) * D_PITCH + wn * TN + j * 8 + fr];
#pragma unroll
      for (int i = 0; i < FI; ++i)
#pragma unroll
        for (int j = 0; j < FJ; ++j) dmma_m8n8k4(acc[i][j], af[i], bf[j]);
    }
    if (kb + 1 < nkb) {
      dgemm_stash<D_BM, NT>(As + (cur ^ 1) * D_BK * D_PITCH, g.a_si, ra);
      dgemm_stash<D_BN, NT>(Bs + (cur ^ 1) * D_BK * D_PITCH, g.b_sj, rb);
    }
    __syncthreads();
  }

  const double* bias = static_cast<const double*>(g.bias);
#pragma unroll
  for (int i = 0; i < FI; ++i) {
    const int row = tm * D_BM + wm * TM + i * 8 + fr;
    if (row >= g.M) continue;
#pragma unroll
    for (int j = 0; j < FJ; ++j) {
      const int col = tn * D_BN + wn * TN + j * 8 + fk * 2;
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        if (col + e < g.N) {
          double x = acc[i][j][e];
          if (bias) x += bias[col + e];
          const double ax = (g.epilogue == 4) ? AUX[(long long)row * g.ldc + col + e] : 0.0;
          C[(long long)row * g.ldc + col + e] = apply_epilogue_f64(x, g.epilogue, ax);
        }
      }
    }
  }
}

// ------------------------------------------------------------------ integers
// Block tile 128 x 128 x 16 (32-bit) or 128 x 64 x 16 (64-bit); 256 threads
// as 16 x 16; each thread owns a TM x TN register tile made of interleaved
// groups of 4 so shared-memory reads are 16-byte vectors.
template <typename T, int TM, int TN>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const StridedGemmArgs g) {
  constexpr int BM = 16 * TM, BN = 16 * TN, BK = 16;
  grid_dependency_wait();        // the gate word is written by the kernels before this one
  if (g.gate && *g.gate != g.gate_value) return;
  constexpr int PA = BM + 4, PB = BN + 4;
  __shared__ T As[BK][PA];
  __shared__ T Bs[BK][PB];

  const int tiles_n = (g.N + BN - 1) / BN;
  const int tm = blockIdx.x / tiles_n, tn = blockIdx.x % tiles_n;
  const int b = blockIdx.y;
  const T* A = static_cast<const T*>(g.A) + b * g.a_sb;
  const T* B = static_cast<const T*>(g.B) + b * g.b_sb;
  T* C = static_cast<T*>(g.C) + b * g.c_sb;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;

  T acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0;

  for (int k0 = 0; k0 < g.K; k0 += BK) {
    // A tile: BM x BK
    for (int idx = threadIdx.x; idx < BM * BK; idx += 256) {
      int i, k;
      if (g.a_si == 1) { i = idx % BM; k = idx / BM; } else { k = idx % BK; i = idx / BK; }
      const bool ok = (tm * BM + i < g.M) && (k0 + k < g.K);
      As[k][i] = ok ? A[(long long)(tm * BM + i) * g.a_si + (long long)(k0 + k) * g.a_sk] : T(0);
    }
    for (int idx = threadIdx.x; idx < BN * BK; idx += 256) {
      int j, k;
      if (g.b_sj == 1) { j = idx % BN; k = idx / BN; } else { k = idx % BK; j = idx / BK; }
      const bool ok = (tn * BN + j < g.N) && (k0 + k < g.K);
      Bs[k][j] = ok ? B[(long long)(k0 + k) * g.b_sk + (long long)(tn * BN + j) * g.b_sj] : T(0);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      T a[TM], bb[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][(i / 4) * 64 + ty * 4 + (i % 4)];
#pragma unroll
      for (int j = 0; j < TN; ++j) bb[j] = Bs[k][(j / 4) * 64 + tx * 4 + (j % 4)];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] += a[i] * bb[j];
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int row = tm * BM + (i / 4) * 64 + ty * 4 + (i % 4);
    if (row >= g.M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int col = tn * BN + (j / 4) * 64 + tx * 4 + (j % 4);
      if (col < g.N) {
        T x = acc[i][j];
        if constexpr (std::is_floating_point<T>::value) {  // fused bias / activation
          if (g.bias) x += static_cast<const T*>(g.bias)[col];
          const T ax = (g.epilogue == 4)
                           ? (static_cast<const T*>(g.aux) + b * g.c_sb)[(long long)row * g.ldc + col]
                           : T(0);
          x = static_cast<T>(apply_epilogue_f64(x, g.epilogue, ax));
        }
        C[(long long)row * g.ldc + col] = x;
      }
    }
  }
}

}  // namespace mtb
