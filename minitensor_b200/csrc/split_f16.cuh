// Operand preparation for the fp16 two-plane mode of the tensor-core GEMM.
//
// An f32 value a is scaled by a power of two chosen per M (or N) index so that
// the largest magnitude of that row lands in [2^14, 2^15), and is then written
// as a0 + a1 with fp16 terms (11 + 11 significand bits; both remainders are
// exact in f32).  The GEMM multiplies a0b1, a1b0, a0b0 - three fp16 tensor
// products per f32 product, half the work of the six-product bf16 mode, with
// the accuracy of a 3xTF32 emulation (which also keeps 22 bits and drops the
// low x low term) - and the epilogue undoes the two scalings exactly (two
// multiplications by powers of two).  Values whose scaled magnitude falls below the fp16 subnormal step
// lose at most 2^-25 of their row's scaled maximum, i.e. 2^-39 of the row's
// largest element.
//
// Plane layout matches split_bf16.cuh with two planes: dst[(b*2 + s)][row][col],
// columns padded with zeros to a multiple of 64.  `expo` receives, per scaled
// index, the integer e with scale = 2^-e.
//   K-major planes (rows = M/N index):   one scale per ROW   -> split16_rows_kernel
//   MN-major planes (rows = K index):    one scale per COLUMN -> colabsmax_kernel + split16_cols_scaled_kernel
#pragma once
#include "ptx_sm100.cuh"
#include <cuda_fp16.h>
#include <cstdint>

#include "split_bf16.cuh"

namespace mtb {

// e such that max * 2^-e lies in [2^14, 2^15); 0 for max == 0 or non-finite.
__device__ __forceinline__ int scale_exponent(float amax) {
  const uint32_t bits = __float_as_uint(amax);
  if (amax == 0.0f || (bits & 0x7f800000u) == 0x7f800000u) return 0;
  int ex;
  frexpf(amax, &ex);  // amax = m * 2^ex, m in [0.5, 1)  ->  amax in [2^(ex-1), 2^ex)
  return ex - 15;
}

__device__ __forceinline__ void split2_f16(float x, int e, __half& h0, __half& h1) {
  if (is_nonfinite(x)) {  // carried as is; the caller has raised the non-finite word
    h0 = __float2half_rn(x);
    h1 = __float2half_rn(0.0f);
    return;
  }
  const float v = scale_pow2(x, -e);  // exact: the result is far above the f32 subnormal range or vanishes in fp16 anyway
  h0 = __float2half_rn(v);
  h1 = __float2half_rn(v - __half2float(h0));
}

// The same split with the scaling done on the exponent field: x * 2^s for a normal x is the bit
// pattern of x with s added to its exponent.  Results below the smallest normal f32 are flushed to
// zero (they are far below the fp16 planes' resolution); zeros, subnormals, Inf and NaN take the
// general route.  s is the negated scale exponent.
__device__ __forceinline__ void split2_f16_shift(float x, int s, __half& h0, __half& h1) {
  const uint32_t b = __float_as_uint(x);
  const int e = int((b >> 23) & 0xffu);
  float v = 0.0f;
  if (e == 255) {
    h0 = __float2half_rn(x);
    h1 = __float2half_rn(0.0f);
    return;
  }
  if (e != 0) {
    const int ne = e + s;
    if (ne >= 255) v = scale_pow2(x, s);
    else if (ne > 0) v = __uint_as_float(b + (static_cast<uint32_t>(s) << 23));
  } else if ((b << 1) != 0u) {
    v = scale_pow2(x, s);  // subnormal input
  }
  h0 = __float2half_rn(v);
  h1 = __float2half_rn(v - __half2float(h0));
}

// One block per row: pass 1 finds the row's largest magnitude, pass 2 (served
// by L1/L2) scales and splits.  src[b][r][k], row stride ld.
static __global__ void __launch_bounds__(256)
split16_rows_kernel(const float* __restrict__ src, long long ld, long long bstride, __half* __restrict__ dst,
                    int* __restrict__ expo, int R, int K, int Kp, uint32_t* __restrict__ nf_word, uint32_t nf_epoch) {
  __shared__ float red[8];
  __shared__ int s_e;
  const int b = blockIdx.z;
  const long long plane = static_cast<long long>(R) * Kp;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int r = blockIdx.x; r < R; r += gridDim.x) {
    const float* p = src + b * bstride + static_cast<long long>(r) * ld;
    const bool vec = ((reinterpret_cast<uintptr_t>(p) & 15) == 0);
    float amax = 0.0f;
    bool nf = false;
    if (vec) {
      for (int k = threadIdx.x * 4; k + 3 < K; k += 1024) {
        const float4 u = *reinterpret_cast<const float4*>(p + k);
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(u.x), fabsf(u.y)), fmaxf(fabsf(u.z), fabsf(u.w))));
        nf |= is_nonfinite(u.x) | is_nonfinite(u.y) | is_nonfinite(u.z) | is_nonfinite(u.w);
      }
      for (int k = (K & ~3) + threadIdx.x; k < K; k += 256) {
        amax = fmaxf(amax, fabsf(p[k]));
        nf |= is_nonfinite(p[k]);
      }
    } else {
      for (int k = threadIdx.x; k < K; k += 256) {
        amax = fmaxf(amax, fabsf(p[k]));
        nf |= is_nonfinite(p[k]);
      }
    }
    if (nf && nf_word) atomicMax(nf_word, nf_epoch);
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) red[warp] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = red[0];
#pragma unroll
      for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
      const int e = scale_exponent(m);
      s_e = e;
      expo[static_cast<long long>(b) * R + r] = e;
    }
    __syncthreads();
    const int e = s_e;
    __half* d0 = dst + (static_cast<long long>(b) * 2) * plane + static_cast<long long>(r) * Kp;
    for (int k0 = threadIdx.x * 8; k0 < Kp; k0 += 2048) {
      __align__(16) __half o0[8], o1[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float x = (k0 + i < K) ? p[k0 + i] : 0.0f;
        split2_f16(x, e, o0[i], o1[i]);
      }
      *reinterpret_cast<uint4*>(d0 + k0) = *reinterpret_cast<const uint4*>(o0);
      *reinterpret_cast<uint4*>(d0 + plane + k0) = *reinterpret_cast<const uint4*>(o1);
    }
    __syncthreads();
  }
}

// The same for rows of at most J * 1024 elements that can be read as float4: the row stays in registers between
// the maximum and the split, so it is read from memory once (the kernel above reads it twice, the second time
// from L1/L2, and its scalar second pass is issue-bound).  K % 4 == 0, 16-byte aligned rows.
template <int J>
static __global__ void __launch_bounds__(256)
split16_rows_reg_kernel(const float* __restrict__ src, long long ld, long long bstride, __half* __restrict__ dst,
                        int* __restrict__ expo, int R, int K, int Kp, uint32_t* __restrict__ nf_word,
                        uint32_t nf_epoch) {
  __shared__ float red[8];
  __shared__ int s_e;
  const int b = blockIdx.z;
  const long long plane = static_cast<long long>(R) * Kp;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int r = blockIdx.x; r < R; r += gridDim.x) {
    const float* p = src + b * bstride + static_cast<long long>(r) * ld;
    float4 v[J];
    float amax = 0.0f;
    bool nf = false;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int k = (j * 256 + threadIdx.x) * 4;
      v[j] = (k < K) ? *reinterpret_cast<const float4*>(p + k) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))));
      nf |= is_nonfinite(v[j].x) | is_nonfinite(v[j].y) | is_nonfinite(v[j].z) | is_nonfinite(v[j].w);
    }
    if (nf && nf_word) atomicMax(nf_word, nf_epoch);
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) red[warp] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = red[0];
#pragma unroll
      for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
      const int e = scale_exponent(m);
      s_e = e;
      expo[static_cast<long long>(b) * R + r] = e;
    }
    __syncthreads();
    const int e = s_e;
    __half* d0 = dst + (static_cast<long long>(b) * 2) * plane + static_cast<long long>(r) * Kp;
#pragma unroll
    for (int j = 0; j < J; ++j) {
      const int k = (j * 256 + threadIdx.x) * 4;
      if (k < Kp) {  // columns K..Kp-1 are written as zeros (v is zero there)
        __align__(8) __half o0[4], o1[4];
        split2_f16(v[j].x, e, o0[0], o1[0]);
        split2_f16(v[j].y, e, o0[1], o1[1]);
        split2_f16(v[j].z, e, o0[2], o1[2]);
        split2_f16(v[j].w, e, o0[3], o1[3]);
        *reinterpret_cast<uint2*>(d0 + k) = *reinterpret_cast<const uint2*>(o0);
        *reinterpret_cast<uint2*>(d0 + plane + k) = *reinterpret_cast<const uint2*>(o1);
      }
    }
    __syncthreads();  // red / s_e are rewritten by the next row
  }
}

// amax_bits[b][c] = max over rows of |src[b][r][c]| as raw bits (non-negative floats order like unsigned ints).
// The vector must be zeroed before the launch.
static __global__ void __launch_bounds__(256)
colabsmax_kernel(const float* __restrict__ src, long long ld, long long bstride, int R, int Cc, int rows_per_band,
                 uint32_t* __restrict__ amax_bits, uint32_t* __restrict__ nf_word, uint32_t nf_epoch) {
  grid_launch_dependents();      // the two small kernels after this one wait inside (programmatic dependent launch)
  const int b = blockIdx.z;
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= Cc) return;
  const int r0 = blockIdx.y * rows_per_band, r1 = min(R, r0 + rows_per_band);
  const float* p = src + b * bstride + c;
  float amax = 0.0f;
  bool nf = false;
  for (int r = r0; r < r1; ++r) {
    const float v = p[static_cast<long long>(r) * ld];
    nf |= is_nonfinite(v);
    amax = fmaxf(amax, fabsf(v));
  }
  if (nf && nf_word) atomicMax(nf_word, nf_epoch);
  atomicMax(amax_bits + static_cast<long long>(b) * Cc + c, __float_as_uint(amax));
}

// expo[i] = scale exponent of the magnitude whose bits are amax_bits[i] (in place is fine).
static __global__ void exponent_from_amax_kernel(const uint32_t* __restrict__ amax_bits, int* __restrict__ expo, int n) {
  grid_dependency_wait();        // the maxima come from the kernel before this one
  grid_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) expo[i] = scale_exponent(__uint_as_float(amax_bits[i]));
}

// MN-major planes: dst[(b*2+s)][r][c], scale per column c.  One thread converts 8 columns of a row.
static __global__ void __launch_bounds__(256)
split16_cols_scaled_kernel(const float* __restrict__ src, long long ld, long long bstride, __half* __restrict__ dst,
                           const int* __restrict__ expo, int R, int Cc, int Cp) {
  grid_dependency_wait();        // the exponents come from the kernel before this one
  const int b = blockIdx.z;
  const int chunks = Cp >> 3;
  const long long total = static_cast<long long>(R) * chunks;
  const long long plane = static_cast<long long>(R) * Cp;
  const float* s = src + b * bstride;
  const int* ex = expo + static_cast<long long>(b) * Cc;
  const bool vec = ((reinterpret_cast<uintptr_t>(s) & 15) == 0) && ((ld & 3) == 0);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / chunks);
    const int c0 = static_cast<int>(i - static_cast<long long>(r) * chunks) << 3;
    const float* p = s + static_cast<long long>(r) * ld + c0;
    float x[8];
    if (vec && c0 + 8 <= Cc) {
      const float4 u = *reinterpret_cast<const float4*>(p);
      const float4 w = *reinterpret_cast<const float4*>(p + 4);
      x[0] = u.x; x[1] = u.y; x[2] = u.z; x[3] = u.w; x[4] = w.x; x[5] = w.y; x[6] = w.z; x[7] = w.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = (c0 + j < Cc) ? p[j] : 0.0f;
    }
    __align__(16) __half o0[8], o1[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) split2_f16(x[j], (c0 + j < Cc) ? ex[c0 + j] : 0, o0[j], o1[j]);
    __half* d = dst + (static_cast<long long>(b) * 2) * plane + static_cast<long long>(r) * Cp + c0;
    *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(o0);
    *reinterpret_cast<uint4*>(d + plane) = *reinterpret_cast<const uint4*>(o1);
  }
}

// amax_bits[b] = largest FINITE magnitude of batch entry b's `count` contiguous values, as raw bits.  Inf and NaN
// are left out so that one of them does not cost the finite values of the same entry their scaling; a block that
// meets one raises *nf_word to nf_value (nullable).  The vector must be zeroed before the launch.  Grid (chunks, batch).
static __global__ void __launch_bounds__(256)
finite_absmax_kernel(const float* __restrict__ src, long long bstride, long long count, uint32_t* __restrict__ amax_bits,
                     uint32_t* __restrict__ nf_word = nullptr, uint32_t nf_value = 0) {
  __shared__ float red[8];
  grid_launch_dependents();      // the split that follows waits inside (programmatic dependent launch)
  const float* p = src + blockIdx.y * bstride;
  float amax = 0.0f;
  bool nf = false;
  const long long step = static_cast<long long>(gridDim.x) * 256;
  const bool vec = ((reinterpret_cast<uintptr_t>(p) & 15) == 0);
  const long long n4 = vec ? (count >> 2) : 0;
#pragma unroll 4
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < n4; i += step) {
    const float4 u = __ldg(reinterpret_cast<const float4*>(p) + i);
    const float a = fabsf(u.x), b = fabsf(u.y), c = fabsf(u.z), d = fabsf(u.w);
    const bool na = is_nonfinite(a), nb = is_nonfinite(b), nc = is_nonfinite(c), nd = is_nonfinite(d);
    nf |= na | nb | nc | nd;
    amax = fmaxf(amax, fmaxf(fmaxf(na ? 0.0f : a, nb ? 0.0f : b), fmaxf(nc ? 0.0f : c, nd ? 0.0f : d)));
  }
  for (long long i = n4 * 4 + blockIdx.x * 256LL + threadIdx.x; i < count; i += step) {
    const float a = fabsf(p[i]);
    const bool na = is_nonfinite(a);
    nf |= na;
    amax = fmaxf(amax, na ? 0.0f : a);
  }
  if (nf && nf_word) atomicMax(nf_word, nf_value);
#pragma unroll
  for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
    atomicMax(amax_bits + blockIdx.y, __float_as_uint(m));
  }
}

// Turning split with ONE scale per batch entry: src[b][k][r] (row stride ld) -> dst[(b*2 + s)][r][k] fp16, K padded
// to Kp with zeros, every value of entry b scaled by 2^-e(b), e(b) = the scale exponent of the magnitude whose bits
// are amax_bits[b * amax_stride] (amax_stride 0: one scale for all entries); the first block of each entry also
// stores e(b) to expo[b] for the GEMM's epilogue.  64 (k) x 64 (r) tiles through shared memory: reads run along r,
// writes along k.
// Optional phase separation of the rows (strided convolutions): with r = y * ph.w + x an image pixel, the row goes
// to ((y % sh) * sw + x % sw) * hq * wq + (y / sh) * wq + x / sw, i.e. the image is stored as sh * sw sub-images of
// hq x wq pixels, one per residue of the coordinates; destination rows no pixel maps to must be zero beforehand.
struct RowPhases {
  int w, sh, sw, hq, wq;   // sh == 1 && sw == 1: rows stay where they are
};
static __global__ void __launch_bounds__(256)
split16_turn_batch_kernel(const float* __restrict__ src, long long ld, long long bstride, __half* __restrict__ dst,
                          const uint32_t* __restrict__ amax_bits, int amax_stride, int* __restrict__ expo, int R, int K,
                          int Kp, RowPhases ph = RowPhases{0, 1, 1, 0, 0}) {
  // [plane][r][9 x 16 bytes]: a row holds 64 k as fp16 (128 bytes) plus 16 bytes of padding, so that the 16-byte
  // stores of lanes with consecutive r and the 16-byte loads of lanes with consecutive k chunks both spread
  // over all banks.  The values are scaled, split and packed BEFORE they cross shared memory.
  __shared__ __align__(16) uint4 tile[2][64][9];
  const int b = blockIdx.z;
  const int r0 = blockIdx.x * 64, k0 = blockIdx.y * 64;
  const float* s = src + b * bstride;
  grid_dependency_wait();        // the maximum comes from the kernel before this one
  grid_launch_dependents();
  const int e = scale_exponent(__uint_as_float(__ldcg(amax_bits + static_cast<long long>(b) * amax_stride)));
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) expo[b] = e;
  const int tx = threadIdx.x & 63, kg = threadIdx.x >> 6;
  const int r = r0 + tx;
  float v[2][8];
#pragma unroll
  for (int g = 0; g < 2; ++g)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int k = k0 + (kg + 4 * g) * 8 + i;
      v[g][i] = (k < K && r < R) ? s[static_cast<long long>(k) * ld + r] : 0.0f;
    }
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    __align__(16) __half o0[8], o1[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) split2_f16(v[g][i], e, o0[i], o1[i]);
    tile[0][tx][kg + 4 * g] = *reinterpret_cast<const uint4*>(o0);
    tile[1][tx][kg + 4 * g] = *reinterpret_cast<const uint4*>(o1);
  }
  __syncthreads();
  const bool phased = ph.sh * ph.sw > 1;
  const long long rows_out = phased ? static_cast<long long>(ph.sh) * ph.sw * ph.hq * ph.wq : R;
  const long long plane = rows_out * Kp;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int idx = threadIdx.x + 256 * j;
    const int pl = idx >> 9, rr = (idx >> 3) & 63, c = idx & 7;
    if (r0 + rr >= R || k0 + c * 8 >= Kp) continue;
    long long row = r0 + rr;
    if (phased) {
      const int y = (r0 + rr) / ph.w, x = (r0 + rr) - y * ph.w;
      row = (static_cast<long long>((y % ph.sh) * ph.sw + x % ph.sw) * ph.hq + y / ph.sh) * ph.wq + x / ph.sw;
    }
    __half* d = dst + (static_cast<long long>(b) * 2 + pl) * plane + row * Kp + k0 + c * 8;
    *reinterpret_cast<uint4*>(d) = tile[pl][rr][c];
  }
}

}  // namespace mtb
