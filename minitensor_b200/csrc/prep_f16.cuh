// Operand preparation of the fp16 two-plane GEMM mode for BOTH operands of a product in one launch.
//
// What is prepared is described in split_f16.cuh: every f32 operand becomes two fp16 planes after an exact
// power-of-two scaling per M (or N) index, plus the vector of scale exponents.  Issued operand by operand that
// takes one launch for an operand stored [mn][k] (one scale per row) and four (clear, column maxima, exponents,
// split) for one stored [k][mn] (one scale per column), on two streams with fork / join events around them - about
// ten host calls before the tensor kernel starts, which is what bounds products up to 2048^3.
//
// Here one grid of clusters of 8 CTAs does it all.  The first `a.blocks` CTAs serve operand a, the rest operand b.
//  * rows mode ([mn][k], k <= 8192): a CTA takes whole rows; the row stays in registers between its maximum and
//    the split, so it is read from memory once.
//  * columns mode ([k][mn]): a CLUSTER takes a strip of 64 columns and its 8 CTAs take an eighth of the k range each.
//    Pass 1 reads the CTA's slice for the column maxima, the eight partial maxima are exchanged through distributed
//    shared memory, and pass 2 reads the slice again - it is at most a few hundred KB that this CTA has just read,
//    so it comes from L2 - scales, splits and writes the planes.  One read from DRAM, no atomics, no zero-filled
//    scratch vector.
#pragma once
#include <cooperative_groups.h>

#include "ptx_sm100.cuh"
#include "split_f16.cuh"

namespace mtb {

struct PrepOperand {
  const float* src;
  long long ld;         // row stride of the source in elements
  long long bstride;    // batch stride of the source in elements
  __half* planes;       // [(b*2 + s)][rows][pitch]
  int* expo;            // [batch][mn]
  int kmajor;           // 1: source [mn][K], one scale per row; 0: source [K][mn], one scale per column
  int mn, K;
  int pitch;            // plane row pitch: K padded to 64 (kmajor) or mn padded to 64
  int batch;
  int blocks;           // CTAs along grid.x that serve this operand (a multiple of 8)
};

template <int J>
__device__ __forceinline__ void prep16_rows(const PrepOperand& o, int b, int first, int step, uint32_t* nf_word,
                                            uint32_t nf_value, float* red, int* s_e) {
  const int K = o.K, Kp = o.pitch;
  const long long plane = static_cast<long long>(o.mn) * Kp;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int r = first; r < o.mn; r += step) {
    const float* p = o.src + b * o.bstride + static_cast<long long>(r) * o.ld;
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
    if (nf && nf_word) atomicMax(nf_word, nf_value);
#pragma unroll
    for (int o2 = 16; o2; o2 >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o2));
    if (lane == 0) red[warp] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = red[0];
#pragma unroll
      for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
      const int e = scale_exponent(m);
      *s_e = e;
      o.expo[static_cast<long long>(b) * o.mn + r] = e;
    }
    __syncthreads();
    const int e = *s_e;
    __half* d0 = o.planes + (static_cast<long long>(b) * 2) * plane + static_cast<long long>(r) * Kp;
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

// One strip of 64 columns per cluster; this CTA's share of the K rows is [k_lo, k_hi).
__device__ __forceinline__ void prep16_cols(const PrepOperand& o, int b, int cluster_index, int clusters,
                                            uint32_t* nf_word, uint32_t nf_value, uint32_t (*s_part)[64],
                                            uint32_t* s_max, int* s_exp) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = int(cluster.block_rank());
  const int per = (o.K + 7) / 8;
  const int k_lo = min(o.K, rank * per), k_hi = min(o.K, k_lo + per);
  const int hw = threadIdx.x >> 4, l16 = threadIdx.x & 15;          // 16 half-warps, 4 columns per lane
  const int strips = (o.mn + 63) / 64;
  const float* s = o.src + b * o.bstride;
  const long long plane = static_cast<long long>(o.K) * o.pitch;
  const bool vec_src = ((reinterpret_cast<uintptr_t>(s) & 15) == 0) && ((o.ld & 3) == 0);
  for (int strip = cluster_index; strip < strips; strip += clusters) {
    const int c = strip * 64 + l16 * 4;
    const bool full = vec_src && c + 4 <= o.mn;
    auto load4 = [&](int k, float (&x)[4]) {
      const float* p = s + static_cast<long long>(k) * o.ld + c;
      if (full) {
        const float4 u = *reinterpret_cast<const float4*>(p);
        x[0] = u.x; x[1] = u.y; x[2] = u.z; x[3] = u.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) x[j] = (c + j < o.mn) ? p[j] : 0.0f;
      }
    };
    // pass 1: maxima of this CTA's slice
    float am[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    bool nf = false;
#pragma unroll 4
    for (int k = k_lo + hw; k < k_hi; k += 16) {
      float x[4];
      load4(k, x);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        am[j] = fmaxf(am[j], fabsf(x[j]));
        nf |= is_nonfinite(x[j]);
      }
    }
    if (nf && nf_word) atomicMax(nf_word, nf_value);
#pragma unroll
    for (int j = 0; j < 4; ++j) s_part[hw][l16 * 4 + j] = __float_as_uint(am[j]);   // non-negative floats order like uints
    __syncthreads();
    if (threadIdx.x < 64) {
      uint32_t m = 0;
#pragma unroll
      for (int q = 0; q < 16; ++q) m = max(m, s_part[q][threadIdx.x]);
      s_max[threadIdx.x] = m;
    }
    cluster.sync();                                  // every CTA's s_max is written
    if (threadIdx.x < 64) {
      uint32_t m = 0;
#pragma unroll
      for (int q = 0; q < 8; ++q) m = max(m, *cluster.map_shared_rank(s_max + threadIdx.x, q));
      const int e = scale_exponent(__uint_as_float(m));
      s_exp[threadIdx.x] = e;
      const int col = strip * 64 + threadIdx.x;
      if (rank == 0 && col < o.mn) o.expo[static_cast<long long>(b) * o.mn + col] = e;
    }
    cluster.sync();                                  // remote reads done before any s_max is rewritten or its CTA exits
    // pass 2: the slice again (from L2), scaled and split; columns mn..pitch-1 are written as zeros
    int e4[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) e4[j] = s_exp[l16 * 4 + j];
    __half* d = o.planes + (static_cast<long long>(b) * 2) * plane + c;
#pragma unroll 4
    for (int k = k_lo + hw; k < k_hi; k += 16) {
      float x[4];
      load4(k, x);
      __align__(8) __half o0[4], o1[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) split2_f16(x[j], e4[j], o0[j], o1[j]);
      __half* dk = d + static_cast<long long>(k) * o.pitch;
      *reinterpret_cast<uint2*>(dk) = *reinterpret_cast<const uint2*>(o0);
      *reinterpret_cast<uint2*>(dk + plane) = *reinterpret_cast<const uint2*>(o1);
    }
    __syncthreads();                                 // s_part / s_exp are rewritten by the next strip
  }
}

// grid (a.blocks + b.blocks, max batch), clusters of 8 along x.  J: float4 per thread a rows-mode operand needs
// (K <= 1024 * J).
template <int J>
__global__ void __cluster_dims__(8, 1, 1) __launch_bounds__(256)
prep16_pair_kernel(const PrepOperand a, const PrepOperand b, uint32_t* __restrict__ nf_word, uint32_t nf_value) {
  __shared__ float red[8];
  __shared__ int s_e;
  __shared__ uint32_t s_part[16][64];
  __shared__ uint32_t s_max[64];
  __shared__ int s_exp[64];
  grid_launch_dependents();      // the product's kernel may set itself up while this one runs (it waits before it reads)
  const bool second = int(blockIdx.x) >= a.blocks;
  const PrepOperand& o = second ? b : a;
  const int bx = int(blockIdx.x) - (second ? a.blocks : 0);
  const int batch = blockIdx.y;
  if (batch >= o.batch) return;                      // the whole cluster leaves: same operand, same batch entry
  if (o.kmajor) prep16_rows<J>(o, batch, bx, o.blocks, nf_word, nf_value, red, &s_e);
  else prep16_cols(o, batch, bx >> 3, o.blocks >> 3, nf_word, nf_value, s_part, s_max, s_exp);
}

}  // namespace mtb
