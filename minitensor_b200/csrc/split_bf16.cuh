// Operand preparation for the split-bf16 GEMM: every f32 element x becomes
// three bf16 values x0 + x1 + x2 = x (round-to-nearest at each step; the
// remainders x - x0 and x - x0 - x1 are exact in f32).  Output layout, the
// one the GEMM's tensor maps describe:
//   dst[(b*3 + s)][r][k]  bf16,  r < R rows, k < Kp (K padded with zeros)
// i.e. always K-major, whatever the orientation of the source.  A kernel that
// meets an Inf or NaN raises *nf_word to nf_epoch (the caller's per-GEMM
// counter) so the GEMM can be redone in plain f32 arithmetic afterwards.  The source is
// a row-major f32 matrix per batch entry, either [R][K] (trans = 0) or
// [K][R] (trans = 1); the second form is how the transposes the reference
// materialises (engine/src/operations/linalg/triangular.rs:8-73) are absorbed.
#pragma once
#include <cuda_bf16.h>
#include <cstdint>

namespace mtb {

// x * 2^e for any integer e in [-380, 380], as two multiplications by exactly representable powers
// of two (ldexpf costs ~10x more and sits in the innermost epilogue loop of the fp16 mode).  Exact
// whenever the result is a normal number or zero; a subnormal result may be off by one subnormal step.
__device__ __forceinline__ float scale_pow2(float x, int e) {
  const int e1 = max(-126, min(127, e));
  const int e2 = max(-126, min(127, e - e1));
  return x * __int_as_float((e1 + 127) << 23) * __int_as_float((e2 + 127) << 23);
}


struct Split3 {
  __nv_bfloat16 s0, s1, s2;
};

__device__ __forceinline__ bool is_nonfinite(float x) {
  return (__float_as_uint(x) & 0x7f800000u) == 0x7f800000u;
}

__device__ __forceinline__ Split3 split3(float x) {
  Split3 r;
  const uint32_t bits = __float_as_uint(x);
  if ((bits & 0x7f800000u) == 0x7f800000u) {  // Inf / NaN: carry it in the leading term only
    r.s0 = __float2bfloat16_rn(x);
    r.s1 = __float2bfloat16_rn(0.0f);
    r.s2 = r.s1;
    return r;
  }
  __nv_bfloat16 h0 = __float2bfloat16_rn(x);
  float f0 = __bfloat162float(h0);
  if ((__float_as_uint(f0) & 0x7f800000u) == 0x7f800000u) {  // rounding overflowed: truncate instead
    f0 = __uint_as_float(bits & 0xffff0000u);
    h0 = __float2bfloat16_rn(f0);
  }
  const float r1 = x - f0;
  const __nv_bfloat16 h1 = __float2bfloat16_rn(r1);
  const float r2 = r1 - __bfloat162float(h1);
  r.s0 = h0;
  r.s1 = h1;
  r.s2 = __float2bfloat16_rn(r2);
  return r;
}

// trans = 0: src[b][r][k] (row stride ld).  One thread converts 8 consecutive
// k and writes one 16-byte vector per split.
static __global__ void split_rows_kernel(const float* __restrict__ src, long long ld, long long bstride,
                                  __nv_bfloat16* __restrict__ dst, int R, int K, int Kp,
                                  int nsplit_out, uint32_t* __restrict__ nf_word, uint32_t nf_epoch) {
  const int b = blockIdx.z;
  const int chunks = Kp >> 3;
  const long long total = static_cast<long long>(R) * chunks;
  const float* s = src + b * bstride;
  const bool vec = ((reinterpret_cast<uintptr_t>(s) & 15) == 0) && ((ld & 3) == 0);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / chunks);
    const int k0 = static_cast<int>(i - static_cast<long long>(r) * chunks) << 3;
    float x[8];
    const float* p = s + static_cast<long long>(r) * ld + k0;
    if (vec && k0 + 8 <= K) {
      const float4 u = *reinterpret_cast<const float4*>(p);
      const float4 w = *reinterpret_cast<const float4*>(p + 4);
      x[0] = u.x; x[1] = u.y; x[2] = u.z; x[3] = u.w;
      x[4] = w.x; x[5] = w.y; x[6] = w.z; x[7] = w.w;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] = (k0 + e < K) ? p[e] : 0.0f;
    }
    __align__(16) __nv_bfloat16 o0[8], o1[8], o2[8];
    bool nf = false;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const Split3 t = split3(x[e]);
      nf |= is_nonfinite(x[e]);
      o0[e] = t.s0; o1[e] = t.s1; o2[e] = t.s2;
    }
    if (nf && nf_word) atomicMax(nf_word, nf_epoch);
    const long long plane = static_cast<long long>(R) * Kp;
    __nv_bfloat16* d = dst + (static_cast<long long>(b) * 3) * plane + static_cast<long long>(r) * Kp + k0;
    *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(o0);
    if (nsplit_out > 1) *reinterpret_cast<uint4*>(d + plane) = *reinterpret_cast<const uint4*>(o1);
    if (nsplit_out > 2) *reinterpret_cast<uint4*>(d + 2 * plane) = *reinterpret_cast<const uint4*>(o2);
  }
}

// trans = 1: src[b][k][r] (row stride ld); the tile is turned through shared
// memory so both the f32 reads (along r) and the bf16 writes (along k) are
// coalesced.  Block = 256 threads, tile = 64 (k) x 64 (r).
static __global__ void split_cols_kernel(const float* __restrict__ src, long long ld, long long bstride,
                                  __nv_bfloat16* __restrict__ dst, int R, int K, int Kp,
                                  int nsplit_out, uint32_t* __restrict__ nf_word, uint32_t nf_epoch) {
  __shared__ float tile[64][65];
  const int b = blockIdx.z;
  const int r0 = blockIdx.x * 64;
  const int k0 = blockIdx.y * 64;
  const float* s = src + b * bstride;
  const int tx = threadIdx.x & 63;
  const int ty = threadIdx.x >> 6;  // 0..3
#pragma unroll 4
  for (int kk = ty; kk < 64; kk += 4) {
    const int k = k0 + kk, r = r0 + tx;
    tile[kk][tx] = (k < K && r < R) ? s[static_cast<long long>(k) * ld + r] : 0.0f;
  }
  __syncthreads();
  // each thread: one row r, 8 consecutive k -> 64 rows x 8 chunks = 512 items, 2 per thread
  const long long plane = static_cast<long long>(R) * Kp;
  for (int it = threadIdx.x; it < 512; it += 256) {
    const int rr = it >> 3;
    const int kc = (it & 7) << 3;
    const int r = r0 + rr;
    if (r >= R || k0 + kc >= Kp) continue;
    __align__(16) __nv_bfloat16 o0[8], o1[8], o2[8];
    bool nf = false;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float xv = tile[kc + e][rr];
      const Split3 t = split3(xv);
      nf |= is_nonfinite(xv);
      o0[e] = t.s0; o1[e] = t.s1; o2[e] = t.s2;
    }
    if (nf && nf_word) atomicMax(nf_word, nf_epoch);
    __nv_bfloat16* d = dst + (static_cast<long long>(b) * 3) * plane + static_cast<long long>(r) * Kp + k0 + kc;
    *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(o0);
    if (nsplit_out > 1) *reinterpret_cast<uint4*>(d + plane) = *reinterpret_cast<const uint4*>(o1);
    if (nsplit_out > 2) *reinterpret_cast<uint4*>(d + 2 * plane) = *reinterpret_cast<const uint4*>(o2);
  }
}

}  // namespace mtb
