// conv2d (NCHW / OIHW, f32) on the split-plane tensor-core kernels: host side, preparation kernels, lowerings.
//
// The reference computes the convolution with direct loops (engine/src/operations/conv.rs:111-157) and its
// backward with three more (engine/src/autograd/mod/shape.rs:57-197).  Here each result is a GEMM:
//   forward    y[n]  [C_out][OH*OW] = W [C_out][C_in*kH*kW] * windows(x[n])^T  (+ bias per channel)
//   bwd data   dx[n] [C_in][H*W]    = W'[C_in][C_out*kH*kW] * windows'(dy[n])^T
//   bwd weight dW [C_out][C_in*kH*kW] = sum over (image, pixel) of dy[.][C_out] * windows(x)[.][C_in*kH*kW]
//   bwd bias   db[oc] = sum_{n,oh,ow} dy
//
// IMPLICIT lowering (default).  The image operand is split once into channels-last planes
// [image*planes+split][h][w][c] (two fp16 planes scaled by a power of two per image - per tensor for the weight
// gradient - or three bf16 planes in the bf16 modes; stride_h x stride_w phase images for strided layers) and the
// kernels' TMA producers read halo blocks of those planes with out-of-range coordinates zero-filled by the hardware:
// the padding and the im2col matrix never exist in memory.  Kernels: conv_pix_umma.cuh (forward and data gradient,
// also strided: the data gradient one output phase at a time), conv_wgrad_halo.cuh (weight gradient, also strided),
// and the earlier conv_halo_umma.cuh / per-tap kernels as fallbacks and test cross-checks.
// EXPLICIT lowering (rows wider than the implicit kernels take, strides above 8, bf16 modes of strided layers, and
// variant byte 0xFF): patches are gathered straight into the split planes of the plain GEMM.
// Inf / NaN in an operand: every lowering ends with a gated direct kernel that recomputes the result in the
// reference's loop order when the call's flag word was raised during preparation.
#include "mtb200_core.cuh"
#include "gemm_launch.cuh"
#include "conv_wgrad_halo.cuh"
#include "conv_wgrad_umma.cuh"
#include "conv_halo_umma.cuh"
#include "conv_pix_umma.cuh"
#include "rowcol_kernels.cuh"

namespace mtb {

struct ConvGeom {
  int n, c_in, h, w, c_out, kh, kw, sh, sw, ph, pw, oh, ow;
};

// Mode byte for the gathered-patch lowerings, whose planes are bf16: the fp16 two-plane mode exists only for the
// implicit (stride-1) kernels, so 23 asks for the default there.
static int bf16_mode_of(int32_t f32_mode) {
  const int m = f32_mode & 0xff;
  return m == 23 ? 0 : m;
}

// Tile-variant byte handed on to the plain GEMM by the gathered-patch lowerings: the conv-only values (0xff = this
// lowering, 0xfc / 0xfb = particular implicit kernels) mean "choose" there.
static int gemm_variant_of(int32_t f32_mode) {
  const int v = (f32_mode >> 8) & 0xff;
  return (v == 0xff || v == 0xfc || v == 0xfb) ? 0 : v;
}

// Gather modes for the patch operand.
//  PATCH_FWD : row = output pixel (oh,ow), k = (ic,kh,kw), value x[n][ic][oh*s+kh-p][ow*s+kw-p]
//  PATCH_BWD : row = input pixel (ih,iw),  k = (oc,kh,kw), value dy[n][oc][(ih+p-kh)/s][(iw+p-kw)/s]
//              when the division is exact and in range
enum { PATCH_FWD = 0, PATCH_BWD = 1 };

template <int MODE>
__device__ __forceinline__ float patch_value(const float* __restrict__ img, const ConvGeom& g, int pix, int k) {
  const int kk = g.kh * g.kw;
  const int ch = k / kk;
  const int r = k - ch * kk;
  const int fh = r / g.kw, fw = r - fh * g.kw;
  if (MODE == PATCH_FWD) {
    const int oy = pix / g.ow, ox = pix - oy * g.ow;
    const int iy = oy * g.sh + fh - g.ph, ix = ox * g.sw + fw - g.pw;
    if (iy < 0 || ix < 0 || iy >= g.h || ix >= g.w) return 0.0f;
    return img[(static_cast<long long>(ch) * g.h + iy) * g.w + ix];
  } else {
    const int iy = pix / g.w, ix = pix - iy * g.w;
    const int ty = iy + g.ph - fh, tx = ix + g.pw - fw;
    if (ty < 0 || tx < 0 || ty % g.sh || tx % g.sw) return 0.0f;
    const int oy = ty / g.sh, ox = tx / g.sw;
    if (oy >= g.oh || ox >= g.ow) return 0.0f;
    return img[(static_cast<long long>(ch) * g.oh + oy) * g.ow + ox];
  }
}

// dst[(n*3+s)][pix][k]: 64 pixels x 64 k per block, turned through shared
// memory (reads run along pixels, writes along k).
template <int MODE>
__global__ void __launch_bounds__(256) patch_split_kernel(const float* __restrict__ src, ConvGeom g,
                                                          int rows, int K, int Kp, long long img_stride,
                                                          __nv_bfloat16* __restrict__ dst,
                                                          uint32_t* __restrict__ nf_word) {
  __shared__ float tile[64][65];
  const int n = blockIdx.z;
  const int r0 = blockIdx.x * 64, k0 = blockIdx.y * 64;
  const float* img = src + n * img_stride;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  for (int kk = ty; kk < 64; kk += 4) {
    const int k = k0 + kk, r = r0 + tx;
    const float v = (k < K && r < rows) ? patch_value<MODE>(img, g, r, k) : 0.0f;
    if (is_nonfinite(v)) atomicMax(nf_word, MTB_FLAG_SET);
    tile[kk][tx] = v;
  }
  __syncthreads();
  const long long plane = static_cast<long long>(rows) * Kp;
  for (int it = threadIdx.x; it < 512; it += 256) {
    const int rr = it >> 3, kc = (it & 7) << 3;
    const int r = r0 + rr;
    if (r >= rows || k0 + kc >= Kp) continue;
    __align__(16) __nv_bfloat16 o0[8], o1[8], o2[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const Split3 t = split3(tile[kc + e][rr]);
      o0[e] = t.s0; o1[e] = t.s1; o2[e] = t.s2;
    }
    __nv_bfloat16* d = dst + (static_cast<long long>(n) * 3) * plane + static_cast<long long>(r) * Kp + k0 + kc;
    *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(o0);
    *reinterpret_cast<uint4*>(d + plane) = *reinterpret_cast<const uint4*>(o1);
    *reinterpret_cast<uint4*>(d + 2 * plane) = *reinterpret_cast<const uint4*>(o2);
  }
}

// Operands of the weight-gradient GEMM, reduction index k = (n, oh, ow):
//  WG_DY    : row = oc,          value dy[n][oc][oh][ow]
//  WG_PATCH : row = (ic,kh,kw),  value x[n][ic][oh*s+kh-p][ow*s+kw-p]
// dst[s][row][k], k < Kp (zeros past n*OH*OW).  One thread converts 8 k.
enum { WG_DY = 0, WG_PATCH = 1 };
template <int MODE>
__global__ void __launch_bounds__(256) wgrad_split_kernel(const float* __restrict__ src, ConvGeom g,
                                                          int rows, long long Ktot, long long Kp,
                                                          __nv_bfloat16* __restrict__ dst,
                                                          uint32_t* __restrict__ nf_word) {
  const long long chunks = Kp >> 3;
  const long long total = rows * chunks;
  const int opix = g.oh * g.ow;
  const long long plane = static_cast<long long>(rows) * Kp;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(i / chunks);
    const long long k0 = (i - row * chunks) << 3;
    int ch = row, fh = 0, fw = 0;
    if (MODE == WG_PATCH) {
      const int kk = g.kh * g.kw;
      ch = row / kk;
      const int r = row - ch * kk;
      fh = r / g.kw;
      fw = r - fh * g.kw;
    }
    __align__(16) __nv_bfloat16 o0[8], o1[8], o2[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const long long k = k0 + e;
      float v = 0.0f;
      if (k < Ktot) {
        const int n = static_cast<int>(k / opix);
        const int pix = static_cast<int>(k - static_cast<long long>(n) * opix);
        if (MODE == WG_DY) {
          v = src[(static_cast<long long>(n) * g.c_out + ch) * opix + pix];
        } else {
          const int oy = pix / g.ow, ox = pix - oy * g.ow;
          const int iy = oy * g.sh + fh - g.ph, ix = ox * g.sw + fw - g.pw;
          if (iy >= 0 && ix >= 0 && iy < g.h && ix < g.w)
            v = src[((static_cast<long long>(n) * g.c_in + ch) * g.h + iy) * g.w + ix];
        }
      }
      if (is_nonfinite(v)) atomicMax(nf_word, MTB_FLAG_SET);
      const Split3 t = split3(v);
      o0[e] = t.s0; o1[e] = t.s1; o2[e] = t.s2;
    }
    __nv_bfloat16* d = dst + static_cast<long long>(row) * Kp + k0;
    *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(o0);
    *reinterpret_cast<uint4*>(d + plane) = *reinterpret_cast<const uint4*>(o1);
    *reinterpret_cast<uint4*>(d + 2 * plane) = *reinterpret_cast<const uint4*>(o2);
  }
}

// w'[ic][oc][kh][kw] = w[oc][ic][kh][kw]
__global__ void permute_weight_kernel(const float* __restrict__ w, float* __restrict__ wp, int c_out,
                                      int c_in, int kk) {
  const long long total = static_cast<long long>(c_out) * c_in * kk;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i % kk);
    const long long r = i / kk;
    const int oc = static_cast<int>(r % c_out), ic = static_cast<int>(r / c_out);
    wp[i] = w[(static_cast<long long>(oc) * c_in + ic) * kk + t];
  }
}

// partial[chunk][oc] = sum over the images of the chunk and all pixels of dy[n][oc][.]; 16-byte loads when the
// pixel planes allow it, four independent accumulators per thread.
__global__ void __launch_bounds__(256) conv_bias_partial_kernel(const float* __restrict__ dy, int n, int c_out,
                                                                int opix, int imgs_per_chunk,
                                                                float* __restrict__ partial) {
  __shared__ float red[8];
  grid_launch_dependents();      // the second stage waits inside
  const int oc = blockIdx.x, chunk = blockIdx.y;
  const int n0 = chunk * imgs_per_chunk, n1 = min(n, n0 + imgs_per_chunk);
  const bool vec = ((opix & 3) == 0) && ((reinterpret_cast<uintptr_t>(dy) & 15) == 0);
  float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
  for (int i = n0; i < n1; ++i) {
    const float* p = dy + (static_cast<long long>(i) * c_out + oc) * opix;
    if (vec) {
      const float4* p4 = reinterpret_cast<const float4*>(p);
      const int q = opix >> 2;
      for (int k = threadIdx.x; k < q; k += 256) {
        const float4 v = __ldg(p4 + k);
        s0 += v.x; s1 += v.y; s2 += v.z; s3 += v.w;
      }
    } else {
      for (int k = threadIdx.x; k < opix; k += 256) s0 += p[k];
    }
  }
  float s = (s0 + s1) + (s2 + s3);
#pragma unroll
  for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) t += red[w];
    partial[static_cast<long long>(chunk) * c_out + oc] = t;
  }
}

// ---- Inf / NaN operands: the same results as the reference's direct loops.
// Any split scheme turns Inf times a finite value into NaN (Inf times the zero low-order plane), where the
// reference's `sum += x * w` (engine/src/operations/conv.rs:121-147, engine/src/autograd/mod/shape.rs:86-169)
// gives +-Inf.  The preparation kernels of a call raise its flag word when they meet a non-finite value and the
// kernels below then recompute the whole result on the CUDA cores with separately rounded multiply and add in the
// reference's summation order; for finite operands they return at once.
__global__ void __launch_bounds__(256) conv_direct_fwd_kernel(ConvGeom g, const float* __restrict__ x,
                                                              const float* __restrict__ w,
                                                              const float* __restrict__ bias, float* __restrict__ y,
                                                              const uint32_t* __restrict__ gate) {
  grid_dependency_wait();        // the flag word is raised by the kernels before this one
  if (*gate != MTB_FLAG_SET) return;
  const long long total = static_cast<long long>(g.n) * g.c_out * g.oh * g.ow;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * 256) {
    const int ox = static_cast<int>(i % g.ow);
    long long q = i / g.ow;
    const int oy = static_cast<int>(q % g.oh);
    q /= g.oh;
    const int oc = static_cast<int>(q % g.c_out), n = static_cast<int>(q / g.c_out);
    float sum = 0.0f;
    for (int ic = 0; ic < g.c_in; ++ic)
      for (int fh = 0; fh < g.kh; ++fh) {
        const int iy = oy * g.sh + fh - g.ph;
        if (iy < 0 || iy >= g.h) continue;
        for (int fw = 0; fw < g.kw; ++fw) {
          const int ix = ox * g.sw + fw - g.pw;
          if (ix < 0 || ix >= g.w) continue;
          const float a = x[((static_cast<long long>(n) * g.c_in + ic) * g.h + iy) * g.w + ix];
          const float b = w[((static_cast<long long>(oc) * g.c_in + ic) * g.kh + fh) * g.kw + fw];
          sum = __fadd_rn(sum, __fmul_rn(a, b));
        }
      }
    if (bias) sum = __fadd_rn(sum, bias[oc]);
    y[i] = sum;
  }
}

// dx[n][ic][iy][ix]: the reference scatters over (oc, oh, ow, kh, kw); gathered per input pixel the same terms arrive
// in ascending (oc, oh, ow).
__global__ void __launch_bounds__(256) conv_direct_dgrad_kernel(ConvGeom g, const float* __restrict__ dy,
                                                                const float* __restrict__ w, float* __restrict__ dx,
                                                                const uint32_t* __restrict__ gate) {
  grid_dependency_wait();        // the flag word is raised by the kernels before this one
  if (*gate != MTB_FLAG_SET) return;
  const long long total = static_cast<long long>(g.n) * g.c_in * g.h * g.w;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * 256) {
    const int ix = static_cast<int>(i % g.w);
    long long q = i / g.w;
    const int iy = static_cast<int>(q % g.h);
    q /= g.h;
    const int ic = static_cast<int>(q % g.c_in), n = static_cast<int>(q / g.c_in);
    float sum = 0.0f;
    for (int oc = 0; oc < g.c_out; ++oc)
      for (int oy = 0; oy < g.oh; ++oy) {
        const int fh = iy + g.ph - oy * g.sh;
        if (fh < 0 || fh >= g.kh) continue;
        for (int ox = 0; ox < g.ow; ++ox) {
          const int fw = ix + g.pw - ox * g.sw;
          if (fw < 0 || fw >= g.kw) continue;
          const float a = dy[((static_cast<long long>(n) * g.c_out + oc) * g.oh + oy) * g.ow + ox];
          const float b = w[((static_cast<long long>(oc) * g.c_in + ic) * g.kh + fh) * g.kw + fw];
          sum = __fadd_rn(sum, __fmul_rn(a, b));
        }
      }
    dx[i] = sum;
  }
}

// dw[oc][ic][fh][fw]: one block per output, the (n, oh, ow) terms dealt round-robin to its threads and the 256
// partial sums folded in a fixed order.
__global__ void __launch_bounds__(256) conv_direct_wgrad_kernel(ConvGeom g, const float* __restrict__ dy,
                                                                const float* __restrict__ x, float* __restrict__ dw,
                                                                const uint32_t* __restrict__ gate) {
  grid_dependency_wait();        // the flag word is raised by the kernels before this one
  if (*gate != MTB_FLAG_SET) return;
  __shared__ float red[256];
  const long long outputs = static_cast<long long>(g.c_out) * g.c_in * g.kh * g.kw;
  const int opix = g.oh * g.ow;
  for (long long o = blockIdx.x; o < outputs; o += gridDim.x) {
    const int fw = static_cast<int>(o % g.kw);
    long long q = o / g.kw;
    const int fh = static_cast<int>(q % g.kh);
    q /= g.kh;
    const int ic = static_cast<int>(q % g.c_in), oc = static_cast<int>(q / g.c_in);
    float sum = 0.0f;
    const long long terms = static_cast<long long>(g.n) * opix;
    for (long long k = threadIdx.x; k < terms; k += 256) {
      const int n = static_cast<int>(k / opix);
      const int pix = static_cast<int>(k - static_cast<long long>(n) * opix);
      const int oy = pix / g.ow, ox = pix - oy * g.ow;
      const int iy = oy * g.sh + fh - g.ph, ix = ox * g.sw + fw - g.pw;
      if (iy < 0 || iy >= g.h || ix < 0 || ix >= g.w) continue;
      const float a = dy[(static_cast<long long>(n) * g.c_out + oc) * opix + pix];
      const float b = x[((static_cast<long long>(n) * g.c_in + ic) * g.h + iy) * g.w + ix];
      sum = __fadd_rn(sum, __fmul_rn(a, b));
    }
    red[threadIdx.x] = sum;
    __syncthreads();
    for (int s = 128; s; s >>= 1) {
      if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
      __syncthreads();
    }
    if (threadIdx.x == 0) dw[o] = red[0];
    __syncthreads();
  }
}

static inline int direct_grid(const mtb200_ctx* h, long long items) {
  return int(std::max<long long>(1, std::min<long long>((items + 255) / 256, 8LL * h->sm_count)));
}

// A sub-filter: the taps (fh0 + a * fh_step, fw0 + b * fw_step), a < nfh, b < nfw, of a kh x kw filter.  The whole
// filter is {0, 1, kh, 0, 1, kw}.  The strided data gradient computes dx one phase at a time, and a phase sees only
// the taps whose offset matches its parity.
struct TapSubset {
  int fh0, fh_step, nfh, fw0, fw_step, nfw;
};

// dst[r][t][cp] (f32, zero for cp >= channels): the A operand of the implicit GEMM; t walks the sub-filter's taps.
//  mode 0 (forward):       r = oc, channel = ic : w[(r*chan + c)*taps_full + tap]
//  mode 1 (data gradient): r = ic, channel = oc : w[(c*rows + r)*taps_full + tap]
__global__ void weight_taps_kernel(const float* __restrict__ w, float* __restrict__ dst, int rows, int chan,
                                   int chan_p, int taps_full, int kw_full, TapSubset sub, int mode) {
  const int taps = sub.nfh * sub.nfw;
  const long long total = static_cast<long long>(rows) * taps * chan_p;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % chan_p);
    const long long q = i / chan_p;
    const int t = static_cast<int>(q % taps), r = static_cast<int>(q / taps);
    const int a = t / sub.nfw, b = t - a * sub.nfw;
    const int tap = (sub.fh0 + a * sub.fh_step) * kw_full + sub.fw0 + b * sub.fw_step;
    float v = 0.0f;
    if (c < chan)
      v = mode == 0 ? w[(static_cast<long long>(r) * chan + c) * taps_full + tap]
                    : w[(static_cast<long long>(c) * rows + r) * taps_full + tap];
    dst[i] = v;
  }
}

// Extras of a call that computes one phase of a strided data gradient (implicit_conv below).
struct ConvPhaseOut {
  TapSubset sub;           // the phase's taps of the full kh_full x kw_full filter
  int kh_full, kw_full;
  bool image_ready;        // the image planes and exponents are in the workspace already (an earlier phase wrote them)
  int out_sy, out_sx;      // pixel strides of the phase inside the full output image
  int out_pitch;           // row pitch of the full output image
  long long out_plane;     // pixels of the full output image
  long long out_offset;    // first pixel of the phase inside it
};

static int32_t image_plane_tmap(CUtensorMap* out, const void* base, int chan_p, int img_w, int img_h, int n,
                                int planes, uint32_t box_c, uint32_t box_w, uint32_t box_h, CUtensorMapSwizzle sw);

// out[n][rows][out_h*out_w] = A[rows][taps*chan_p] * windows(img planes) (+ bias per row), stride 1.
//  img: f32 NCHW [n][chan][img_h][img_w]; wsrc: OIHW weights; mode as in weight_taps_kernel;
//  the window of tap (fh,fw) for output pixel (y,x) starts at (y + h0 + sgn*fh, x + w0 + sgn*fw).
static int32_t implicit_conv(mtb200_ctx* h, const float* img, int n, int chan, int img_h, int img_w,
                             const float* wsrc, int rows, int kh, int kw, int mode, int out_h, int out_w,
                             int w0, int h0, int sgn, const float* bias, float* out, int f32_mode,
                             uint32_t* nf_word, int sh = 1, int sw = 1, int pad_h = 0, int pad_w = 0,
                             const ConvPhaseOut* phase_out = nullptr) {
  // sh, sw > 1 (forward only, fp16 mode only - the caller checks): the image planes are written as sh * sw phase
  // images so that every tap reads a stride-1 window of one of them (conv_pix_umma.cuh).
  constexpr int BK = 32;
  using Cfg = GemmCfg<256, BK, 3>;
  // with phase_out, kh x kw is the sub-filter; the workspace is laid out for the full filter so that every phase
  // call finds the image planes of the first one where it left them
  const int chan_p = padded_k(chan), taps = kh * kw;
  const int Kp = taps * chan_p;
  const int taps_full = phase_out ? phase_out->kh_full * phase_out->kw_full : taps;
  const int Kp_full = taps_full * chan_p;
  const TapSubset sub = phase_out ? phase_out->sub : TapSubset{0, 1, kh, 0, 1, kw};
  const int kw_full = phase_out ? phase_out->kw_full : kw;
  const int phases = sh * sw;
  const int hq = (img_h + sh - 1) / sh, wq = (img_w + sw - 1) / sw;          // phase-image extent
  const int ipix = img_h * img_w, opix = out_h * out_w;
  const int ppix = phases > 1 ? phases * hq * wq : ipix;                      // plane rows per image
  // Default: the fp16 two-plane mode (three products).  The reduction of one output runs over taps and channels
  // of ONE image, so the image operand takes one power-of-two scale per image and the weights one per row; the
  // bf16 modes (three planes, up to nine products, no scaling) stay selectable through the mode byte.
  const int gemm_mode = (f32_mode & 0xff) ? (f32_mode & 0xff) : 23;
  if (gemm_mode != 1 && gemm_mode != 3 && gemm_mode != 6 && gemm_mode != 9 && gemm_mode != 23)
    return fail(MTB200_ERR_INVALID, "unknown f32 mode");
  const bool f16 = gemm_mode == 23;
  const int planes = f16 ? 2 : 3;
  const size_t bytes_img = split_bytes(ppix, chan_p, n);      // sized for three planes; the fp16 mode uses two
  const size_t bytes_w = split_bytes(rows, Kp_full, 1);
  const size_t bytes_tmp = align_up(sizeof(float) * size_t(rows) * Kp_full, 1024);
  const size_t bytes_ea = align_up(sizeof(int) * size_t(rows), 1024), bytes_eb = align_up(sizeof(int) * size_t(n), 1024);
  void* ws = nullptr;
  int32_t rc = workspace_reserve(h, bytes_img + bytes_w + bytes_tmp + bytes_ea + 2 * bytes_eb, &ws);
  if (rc) return rc;
  char* wbase = static_cast<char*>(ws);
  __nv_bfloat16* p_img = static_cast<__nv_bfloat16*>(ws);
  __nv_bfloat16* p_w = reinterpret_cast<__nv_bfloat16*>(wbase + bytes_img);
  float* wtmp = reinterpret_cast<float*>(wbase + bytes_img + bytes_w);
  int* ea = reinterpret_cast<int*>(wbase + bytes_img + bytes_w + bytes_tmp);
  int* eb = reinterpret_cast<int*>(wbase + bytes_img + bytes_w + bytes_tmp + bytes_ea);
  uint32_t* amax = reinterpret_cast<uint32_t*>(wbase + bytes_img + bytes_w + bytes_tmp + bytes_ea + bytes_eb);
  const long long img_elems = static_cast<long long>(chan) * ipix;
  // channels-last planes: per image a [chan][pixels] -> [pixels][chan_p] turning split
  const bool image_ready = phase_out && phase_out->image_ready;
  if (f16 && h->side_stream && !h->profiling) MTB_CUDA(cudaEventRecord(h->ev_fork, h->stream));   // the weights fork here
  if (image_ready) {
    // an earlier phase of the same call prepared the planes
  } else if (f16) {
    ProfScope prof(h, PROF_CONV_GATHER, double(n) * ipix * (8.0 * chan + 4.0 * chan_p));
    MTB_CUDA(cudaMemsetAsync(amax, 0, sizeof(uint32_t) * size_t(n), h->stream));
    const int chunks = int(std::max<long long>(1, std::min<long long>((img_elems + 4095) / 4096,
                                                                      (16LL * h->sm_count + n - 1) / n)));
    finite_absmax_kernel<<<dim3(chunks, n), 256, 0, h->stream>>>(img, img_elems, img_elems, amax, nf_word, MTB_FLAG_SET);
    if (phases > 1 && ppix != ipix)   // phase images have rows / columns no pixel maps to: they must read as zero
      MTB_CUDA(cudaMemsetAsync(p_img, 0, size_t(2) * n * ppix * chan_p * sizeof(__half), h->stream));
    MTB_CUDA(launch_pdl(h, split16_turn_batch_kernel, dim3((ipix + 63) / 64, chan_p / 64, n), dim3(256), 0, img,
                        static_cast<long long>(ipix), img_elems, reinterpret_cast<__half*>(p_img),
                        static_cast<const uint32_t*>(amax), 1, eb, ipix, chan, chan_p, RowPhases{img_w, sh, sw, hq, wq}));
  } else {
    ProfScope prof(h, PROF_CONV_GATHER, double(n) * ipix * (4.0 * chan + 6.0 * chan_p));
    rc = launch_split(h, img, true, ipix, chan, chan_p, n, img_elems, p_img, 3, nf_word, MTB_FLAG_SET);
    if (rc) return rc;
  }
  const long long wtotal = static_cast<long long>(rows) * Kp;
  if (f16) {
    // the weights (a few hundred KB, two launches) are prepared beside the image
    const bool side = h->side_stream && !h->profiling;
    cudaStream_t sw = side ? h->side_stream : h->stream;
    if (side) MTB_CUDA(cudaStreamWaitEvent(sw, h->ev_fork, 0));
    weight_taps_kernel<<<int(std::min<long long>((wtotal + 255) / 256, 4096)), 256, 0, sw>>>(
        wsrc, wtmp, rows, chan, chan_p, taps_full, kw_full, sub, mode);
    MTB_CUDA(cudaGetLastError());
    rc = launch_split16(h, wtmp, true, rows, Kp, 1, 0, reinterpret_cast<__half*>(p_w), ea, nf_word, MTB_FLAG_SET, sw);
    if (rc) return rc;
    if (side) {
      MTB_CUDA(cudaEventRecord(h->ev_join, sw));
      MTB_CUDA(cudaStreamWaitEvent(h->stream, h->ev_join, 0));
    }
  } else {
    weight_taps_kernel<<<int(std::min<long long>((wtotal + 255) / 256, 4096)), 256, 0, h->stream>>>(
        wsrc, wtmp, rows, chan, chan_p, taps_full, kw_full, sub, mode);
    MTB_CUDA(cudaGetLastError());
    rc = launch_split(h, wtmp, false, rows, Kp, Kp, 1, 0, p_w, 3, nf_word, MTB_FLAG_SET);
    if (rc) return rc;
  }

  // Pixels-on-M kernel (conv_pix_umma.cuh): the default.  Pick the channel block (64 or 32 channels per shared-memory
  // row), the output tile (tr x tc), the number of 128-position M blocks and whether the weights stay resident by a
  // small cost model.  Per tile the tensor core runs mb * taps * chan_p / 16 groups of MMAs, each MMA bounded either
  // by its arithmetic (0.273 ns per accumulator column) or by fetching its operands from shared memory (measured:
  // about 150 bytes per ns with 128-byte rows, two thirds of that with 64-byte rows); the TMA engine needs about 4 ns
  // per shared-memory row it writes.  Whichever is longer bounds the tile.
  {
    const size_t smem_limit = 232448;
    const bool three = planes == 3;
    const int nsplit = gemm_mode == 1 ? 1 : ((gemm_mode == 3 || gemm_mode == 23) ? 2 : 3);
    const int products = split_pair_count(gemm_mode);
    struct Plan { double cost; int bk, tr, tc, wp, mb, w_stages, n_tile, tiles_n; bool resident; size_t img_plane; } best =
        {1e300, 0, 0, 0, 0, 0, 0, 0, 0, false, 0};
    // halo origin and reach of the taps, in (phase-)image coordinates relative to the output pixel
    auto fdiv = [](int a, int b) { return (a >= 0) ? a / b : -((-a + b - 1) / b); };
    const int org_x = phases > 1 ? fdiv(-pad_w, sw) : w0 - (sgn < 0 ? kw - 1 : 0);
    const int org_y = phases > 1 ? fdiv(-pad_h, sh) : h0 - (sgn < 0 ? kh - 1 : 0);
    const int dxr = phases > 1 ? fdiv(kw - 1 - pad_w, sw) - org_x : kw - 1;    // halo columns beyond the tile's own
    const int dyr = phases > 1 ? fdiv(kh - 1 - pad_h, sh) - org_y : kh - 1;
    auto mma_ns = [](int n, int bk) {
      return std::max(0.273 * n, (128.0 + n) * 32.0 / (bk == 64 ? 150.0 : 100.0)) * 1.3;
    };
    for (int bk = 64; bk >= 32; bk /= 2)
    for (int n_cap = 256; n_cap >= 64; n_cap /= 2) {    // narrower channel tiles leave room for more weight stages
      const int row_bytes = 2 * bk, cbs = chan_p / bk;
      const int tiles_n = (rows + n_cap - 1) / n_cap;
      if (n_cap < 256 && tiles_n == (rows + 2 * n_cap - 1) / (2 * n_cap)) continue;   // same split as the wider cap
      const int n_tile = (((rows + tiles_n - 1) / tiles_n) + 15) / 16 * 16;
      const size_t w_tile = size_t(n_tile) * row_bytes;
      const bool fold = gemm_mode == 23 && n_tile <= 128;     // hi x [hi; lo] in one MMA (conv_pix_umma.cuh)
      const int acc_n = fold ? 2 * n_tile : n_tile;
      const double group_ns = fold ? mma_ns(2 * n_tile, bk) + mma_ns(n_tile, bk) : products * mma_ns(n_tile, bk);
      for (int mb = 1; mb <= 4 && 2 * mb * acc_n <= 512; mb *= 2)
        for (int sx = 1; sx <= 16; ++sx) {
          const int tc = (out_w + sx - 1) / sx;
          const int wp = tc + dxr;
          if (wp > 256 || wp > 128 * mb) continue;
          const int tr = std::min(out_h, (128 * mb) / wp);
          if (tr < 1 || tr + dyr > 256 || phases * (tr + dyr) * wp * row_bytes > (1 << 20) - 1) continue;
          // a TMA destination must be 128-byte aligned, so every plane of the ring is
          const size_t img_plane = align_up(size_t((phases - 1) * (tr + dyr) * wp + mb * 128 + dyr * wp + dxr) * row_bytes, 128);
          const size_t fixed = conv_pix_fixed_bytes(planes, img_plane);
          if (fixed >= smem_limit) continue;
          const bool resident = tiles_n == 1 && fixed + size_t(taps) * cbs * planes * w_tile <= smem_limit;
          int w_stages = taps * cbs;
          if (!resident) {
            w_stages = int(std::min<size_t>(CONV_PIX_MAX_W_STAGES, (smem_limit - fixed) / (planes * w_tile)));
            if (w_stages < 3) continue;
          }
          const double tiles = double(tiles_n) * ((out_w + tc - 1) / tc) * ((out_h + tr - 1) / tr) * n;
          const double tensor_ns = double(mb) * taps * (chan_p / 16) * group_ns;
          const double tma_ns = (double(phases) * (tr + dyr) * wp * cbs * nsplit +
                                 (resident ? 0.0 : double(taps) * cbs * nsplit * n_tile)) * 4.1;
          const double cost = std::ceil(tiles / h->sm_count) * (std::max(tensor_ns, tma_ns) + 500.0);
          if (cost < best.cost) best = {cost, bk, tr, tc, wp, mb, w_stages, n_tile, tiles_n, resident, img_plane};
        }
    }
    const int vbyte = (f32_mode >> 8) & 0xff;    // test hooks: 0xFB = the channels-on-M halo kernel, 0xFC = the per-tap kernel
    if (best.tr >= 1 && taps <= CONV_PIX_MAX_TAPS && vbyte != 0xFB && vbyte != 0xFC) {
      const int bk = best.bk, n_tile = best.n_tile, tiles_n = best.tiles_n;
      const size_t w_tile = size_t(n_tile) * 2 * bk;
      ConvPixArgs a = {};
      a.n_out = rows; a.out_h = out_h; a.out_w = out_w; a.batch = n;
      a.C = out + (phase_out ? phase_out->out_offset : 0);
      a.bias = bias; a.mode = gemm_mode; a.planes_per_mat = planes;
      a.out_sy = phase_out ? phase_out->out_sy : 1; a.out_sx = phase_out ? phase_out->out_sx : 1;
      a.out_pitch = phase_out ? phase_out->out_pitch : out_w;
      a.out_plane = phase_out ? phase_out->out_plane : static_cast<long long>(opix);
      a.exp_w = f16 ? ea : nullptr; a.exp_img = f16 ? eb : nullptr;
      a.tr = best.tr; a.tc = best.tc; a.wp = best.wp; a.hh = best.tr + dyr; a.mb = best.mb; a.n_tile = n_tile;
      a.kh = kh; a.kw = kw; a.cbs = chan_p / bk; a.chan_p = chan_p;
      a.flip = sgn < 0 ? 1 : 0;
      a.w_org = org_x;
      a.h_org = org_y;
      a.sh = sh; a.sw = sw; a.pad_h = pad_h; a.pad_w = pad_w;
      a.img_plane_bytes = uint32_t(best.img_plane);
      a.w_tile_bytes = uint32_t(w_tile);
      a.w_stages = best.w_stages; a.w_resident = best.resident ? 1 : 0;
      a.fold = (gemm_mode == 23 && n_tile <= 128) ? 1 : 0;
      a.status = h->status;
      const CUtensorMapSwizzle swz = bk == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
      CUtensorMap tw, ti;
      rc = make_split_tmap(&tw, p_w, Kp, rows, planes, bk, uint32_t(n_tile));
      if (rc) return rc;
      if (phases == 1) {
        rc = image_plane_tmap(&ti, p_img, chan_p, img_w, img_h, n, planes, bk, uint32_t(a.wp), uint32_t(a.hh), swz);
      } else {   // {c, x, y, phase, image*planes + split} over the phase images
        EncodeTiledFn enc = get_encode_tiled();
        if (!enc) return fail(MTB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        const cuuint64_t dims[5] = {cuuint64_t(chan_p), cuuint64_t(wq), cuuint64_t(hq), cuuint64_t(phases), cuuint64_t(planes) * n};
        const cuuint64_t strides[4] = {cuuint64_t(chan_p) * 2, cuuint64_t(wq) * chan_p * 2, cuuint64_t(hq) * wq * chan_p * 2,
                                       cuuint64_t(phases) * hq * wq * chan_p * 2};
        const cuuint32_t box[5] = {cuuint32_t(bk), cuuint32_t(a.wp), cuuint32_t(a.hh), cuuint32_t(phases), 1};
        const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
        CUresult r5 = enc(&ti, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, p_img, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        rc = r5 == CUDA_SUCCESS ? MTB200_OK : fail(MTB200_ERR_CUDA, "cuTensorMapEncodeTiled (phase images) failed (%d)", int(r5));
      }
      if (rc) return rc;
      const long long tiles = static_cast<long long>(tiles_n) * ((out_w + a.tc - 1) / a.tc) * ((out_h + a.tr - 1) / a.tr) * n;
      const int grid = int(std::min<long long>(tiles, h->sm_count));
      const size_t smem = conv_pix_fixed_bytes(planes, a.img_plane_bytes) + size_t(a.w_stages) * planes * w_tile;
      ProfScope prof(h, PROF_GEMM_UMMA, 2.0 * rows * double(opix) * taps * chan * n);
      auto launch = [&](auto kernel) -> int32_t {
        if (int32_t rc_attr = grant_dynamic_smem(h, kernel, int(smem))) return rc_attr;
        MTB_CUDA(launch_pdl(h, kernel, dim3(grid), dim3(CONV_PIX_THREADS), smem, tw, ti, a));
        return MTB200_OK;
      };
      if (three) rc = bk == 64 ? launch(conv_pix_umma_kernel<3, 64>) : launch(conv_pix_umma_kernel<3, 32>);
      else rc = bk == 64 ? launch(conv_pix_umma_kernel<2, 64>) : launch(conv_pix_umma_kernel<2, 32>);
      if (rc) return rc;
      MTB_CUDA(cudaGetLastError());
      return MTB200_OK;
    }
  }

  if (phases > 1 || phase_out) return fail(MTB200_ERR_UNSUPPORTED, "strided implicit convolution: no tile plan fits");
  // Halo kernel (conv_halo_umma.cuh): the image block is staged once per (row block, channel block) and every tap
  // multiplies against it.  Geometry: halo row pitch wh (a multiple of 4), th output rows per tile with th * wh <= 256
  // MMA columns, and image stages that fit beside the weights - all of them resident when they fit, a ring otherwise.
  // Very wide rows or very tall filters take the per-tap kernel below.
  {
    const int wh = (out_w + kw - 1 + 3) / 4 * 4;
    const bool three = planes == 3;
    const size_t smem_limit = 232448;
    const int cbs = chan_p / 32;
    auto plane_bytes_for = [&](int th_) {
      const int un = (th_ * wh + 15) / 16 * 16;
      return align_up(size_t((kh - 1) * wh + (kw - 1) + un) * 64, 1024);
    };
    auto fixed_for = [&](int th_) {
      return three ? ConvHaloCfg<3>::fixed_bytes(plane_bytes_for(th_)) : ConvHaloCfg<2>::fixed_bytes(plane_bytes_for(th_));
    };
    const int a_rows = rows <= 64 ? 64 : 128;
    const size_t a_stage = three ? ConvHaloCfg<3>::a_stage_bytes(a_rows) : ConvHaloCfg<2>::a_stage_bytes(a_rows);
    const int th_max = wh <= 256 ? std::min(out_h, 256 / wh) : 0;
    // resident weights: the tallest tile that leaves room for every (tap, channel block) tile; worth it while the
    // MMA keeps a useful width
    int th_res = 0;
    if (rows <= 128 && size_t(taps) * cbs * a_stage < smem_limit) {
      th_res = th_max;
      while (th_res >= 1 && fixed_for(th_res) + size_t(taps) * cbs * a_stage > smem_limit) --th_res;
      if (th_res >= 1 && th_res * wh < 96 && th_res < th_max) th_res = 0;
    }
    // streamed weights: the tallest tile that leaves a ring of at least four tiles
    auto ring_for = [&](int th_) {
      const size_t fixed = fixed_for(th_);
      if (fixed + 2 * a_stage > smem_limit) return 0;
      return int(std::min<size_t>(ConvHaloCfg<2>::MAX_A_STAGES, (smem_limit - fixed) / a_stage));
    };
    int th_ring = th_max;
    while (th_ring > 1 && ring_for(th_ring) < 4) --th_ring;
    const bool resident = th_res >= 1;
    const int th_h = resident ? th_res : th_ring;
    const bool per_tap_forced = ((f32_mode >> 8) & 0xff) == 0xFC;   // test hook: the per-tap kernel
    if (th_h >= 1 && th_h + kh - 1 <= 256 && taps <= ConvHaloCfg<2>::MAX_TAPS && (resident || ring_for(th_h) >= 3) &&
        !per_tap_forced) {
      ConvHaloArgs a = {};
      a.M = rows; a.out_h = out_h; a.out_w = out_w; a.batch = n;
      a.C = out; a.bias = bias; a.mode = gemm_mode; a.planes_per_mat = planes;
      a.exp_a = f16 ? ea : nullptr; a.exp_b = f16 ? eb : nullptr;
      a.th = th_h; a.wh = wh; a.hh = th_h + kh - 1; a.umma_n = (th_h * wh + 15) / 16 * 16;
      a.kh = kh; a.kw = kw; a.cbs = cbs; a.chan_p = chan_p;
      a.flip = sgn < 0 ? 1 : 0;
      a.w_org = w0 - (a.flip ? kw - 1 : 0);
      a.h_org = h0 - (a.flip ? kh - 1 : 0);
      a.b_plane_bytes = uint32_t(plane_bytes_for(th_h));
      a.a_rows = a_rows;
      a.a_resident = resident ? 1 : 0;
      a.a_stages = resident ? taps * cbs : ring_for(th_h);
      a.status = h->status;
      CUtensorMap ta, tb;
      rc = make_split_tmap(&ta, p_w, Kp, rows, planes, 32, uint32_t(a_rows));
      if (rc) return rc;
      rc = image_plane_tmap(&tb, p_img, chan_p, img_w, img_h, n, planes, 32, uint32_t(wh), uint32_t(a.hh),
                            CU_TENSOR_MAP_SWIZZLE_64B);
      if (rc) return rc;
      const long long tiles = static_cast<long long>((rows + 127) / 128) * ((out_h + th_h - 1) / th_h) * n;
      const int grid = int(std::min<long long>(tiles, h->sm_count));
      const size_t smem = three ? ConvHaloCfg<3>::smem_bytes(a.b_plane_bytes, a_rows, a.a_stages)
                                : ConvHaloCfg<2>::smem_bytes(a.b_plane_bytes, a_rows, a.a_stages);
      ProfScope prof(h, PROF_GEMM_UMMA, 2.0 * rows * double(opix) * taps * chan * n);
      if (three) {
        if (int32_t rc_attr = grant_dynamic_smem(h, conv_halo_umma_kernel<3>, int(int(smem)))) return rc_attr;
        conv_halo_umma_kernel<3><<<grid, ConvHaloCfg<3>::NUM_THREADS, smem, h->stream>>>(ta, tb, a);
      } else {
        if (int32_t rc_attr = grant_dynamic_smem(h, conv_halo_umma_kernel<2>, int(int(smem)))) return rc_attr;
        conv_halo_umma_kernel<2><<<grid, ConvHaloCfg<2>::NUM_THREADS, smem, h->stream>>>(ta, tb, a);
      }
      MTB_CUDA(cudaGetLastError());
      return MTB200_OK;
    }
  }

  int th = std::max(1, 256 / out_w);
  th = std::min(th, out_h);
  GemmArgs g = {};
  g.M = rows; g.N = opix; g.batch = n;
  g.num_kb = Kp / BK;
  g.C = out; g.ldc = opix; g.strideC = static_cast<long long>(rows) * opix;
  g.bias = bias; g.aux = nullptr; g.epilogue = EPI_NONE;
  g.mode = gemm_mode;
  g.a_batched = 0; g.b_batched = 1; g.bias_per_row = 1; g.kb_batch_stride = 0;
  g.planes_per_mat = planes;
  g.exp_a = f16 ? ea : nullptr; g.exp_b = f16 ? eb : nullptr; g.exp_b_per_batch = f16 ? 1 : 0;
  g.status = h->status;
  g.cv_th = th; g.cv_n_tile = th * out_w; g.cv_umma_n = (g.cv_n_tile + 15) / 16 * 16;
  g.cv_kb_per_tap = chan_p / BK; g.cv_kw = kw; g.cv_w0 = w0; g.cv_h0 = h0; g.cv_sgn = sgn;

  CUtensorMap ta, tb;
  rc = make_split_tmap(&ta, p_w, Kp, rows, planes, BK, Cfg::BM);
  if (rc) return rc;
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return fail(MTB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[4] = {cuuint64_t(chan_p), cuuint64_t(img_w), cuuint64_t(img_h), cuuint64_t(planes) * n};
  const cuuint64_t strides[3] = {cuuint64_t(chan_p) * 2, cuuint64_t(img_w) * chan_p * 2,
                                 cuuint64_t(ipix) * chan_p * 2};
  const cuuint32_t box[4] = {BK, cuuint32_t(out_w), cuuint32_t(th), 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(&tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, p_img, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MTB200_ERR_CUDA, "cuTensorMapEncodeTiled (image planes) failed (%d)", int(r));
  const long long tiles = static_cast<long long>((rows + Cfg::BM - 1) / Cfg::BM) * ((out_h + th - 1) / th) * n;
  const int grid = int(std::min<long long>(tiles, h->sm_count));
  ProfScope prof(h, PROF_GEMM_UMMA, 2.0 * rows * double(opix) * taps * chan * n);
  if (f16) {   // two planes per operand: four stages of 48 KB instead of three of 72 KB
    using Cfg2 = GemmCfg<256, BK, 4, 2>;
    auto kern = gemm_split_umma_kernel<256, BK, 4, true, 2>;
    if (int32_t rc_attr = grant_dynamic_smem(h, kern, int(Cfg2::SMEM_BYTES))) return rc_attr;
    kern<<<grid, Cfg2::NUM_THREADS, Cfg2::SMEM_BYTES, h->stream>>>(ta, tb, g);
  } else {
    auto kern = gemm_split_umma_kernel<256, BK, 3, true>;
    if (int32_t rc_attr = grant_dynamic_smem(h, kern, int(Cfg::SMEM_BYTES))) return rc_attr;
    kern<<<grid, Cfg::NUM_THREADS, Cfg::SMEM_BYTES, h->stream>>>(ta, tb, g);
  }
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

static int32_t image_plane_tmap(CUtensorMap* out, const void* base, int chan_p, int img_w, int img_h, int n,
                                int planes, uint32_t box_c, uint32_t box_w, uint32_t box_h, CUtensorMapSwizzle sw) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return fail(MTB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[4] = {cuuint64_t(chan_p), cuuint64_t(img_w), cuuint64_t(img_h), cuuint64_t(planes) * n};
  const cuuint64_t strides[3] = {cuuint64_t(chan_p) * 2, cuuint64_t(img_w) * chan_p * 2,
                                 cuuint64_t(img_h) * img_w * chan_p * 2};
  const cuuint32_t box[4] = {box_c, box_w, box_h, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MTB200_ERR_CUDA, "cuTensorMapEncodeTiled (image planes) failed (%d)", int(r));
  return MTB200_OK;
}

// Stride-1 weight gradient as implicit GEMM (conv_wgrad_umma.cuh).
static int32_t implicit_wgrad(mtb200_ctx* h, const ConvGeom& g, const float* dy, const float* x, float* dw,
                              int f32_mode, uint32_t* nf_word) {
  const int cop = padded_k(g.c_out), cip = padded_k(g.c_in), taps = g.kh * g.kw;
  const int opix = g.oh * g.ow, ipix = g.h * g.w;
  WgradArgs a = {};
  a.c_out = g.c_out;
  a.cb_per_tap = cip / 64;
  a.n_chunks = taps * a.cb_per_tap;
  a.kw = g.kw; a.pad_h = g.ph; a.pad_w = g.pw;
  int tw = 1;
  while (tw < std::min(g.ow, 64)) tw *= 2;
  a.tw = tw; a.th = 64 / tw;
  a.wblocks = (g.ow + tw - 1) / tw;
  a.hblocks = (g.oh + a.th - 1) / a.th;
  const long long total_kb = static_cast<long long>(g.n) * a.wblocks * a.hblocks;
  if (total_kb > INT32_MAX) return fail(MTB200_ERR_INVALID, "conv2d weight gradient: too many reduction blocks");
  a.total_kb = int(total_kb);
  a.tiles_m = (g.c_out + 127) / 128;
  a.tiles_n = (a.n_chunks + 1) / 2;
  const int tiles = a.tiles_m * a.tiles_n;
  int splits = int(std::min<long long>(total_kb, std::max(1, h->sm_count / tiles)));
  a.kb_per_split = int((total_kb + splits - 1) / splits);
  a.splits = int((total_kb + a.kb_per_split - 1) / a.kb_per_split);
  a.n_total = a.n_chunks * 64;
  // Default: the fp16 two-plane mode with ONE power-of-two scale per tensor (the reduction runs over images and
  // pixels, so only a scale that is constant over both factors out of the sum).
  a.mode = (f32_mode & 0xff) ? (f32_mode & 0xff) : 23;
  if (a.mode != 1 && a.mode != 3 && a.mode != 6 && a.mode != 9 && a.mode != 23)
    return fail(MTB200_ERR_INVALID, "unknown f32 mode");
  const bool f16 = a.mode == 23;
  a.planes = f16 ? 2 : 3;
  a.status = h->status;
  // Halo kernel (conv_wgrad_halo.cuh) for the fp16 mode: one staged block of x serves every tap.  Rows per step:
  // the tr that wastes least of the reduction (a block is padded to a multiple of 16 indices and carries kw - 1
  // zero columns per row) among those whose two stages fit shared memory.  0xFC in the variant byte keeps the
  // window-per-tap kernel (test hook).
  WgradHaloArgs hw = {};
  bool halo = false;
  const int phases = g.sh * g.sw;
  const int hq = (g.h + g.sh - 1) / g.sh, wq = (g.w + g.sw - 1) / g.sw;     // extent of a phase image of x
  const int ppix = phases > 1 ? phases * hq * wq : ipix;                     // plane rows per image of x
  {
    // reach of the taps in (phase-)image coordinates relative to the output pixel
    auto fdiv = [](int a_, int b_) { return (a_ >= 0) ? a_ / b_ : -((-a_ + b_ - 1) / b_); };
    const int org_x = fdiv(-g.pw, g.sw), org_y = fdiv(-g.ph, g.sh);
    const int dxr = fdiv(g.kw - 1 - g.pw, g.sw) - org_x, dyr = fdiv(g.kh - 1 - g.ph, g.sh) - org_y;
    const int wp = g.ow + dxr;
    const int pairs = (taps + 1) / 2;
    int best_tr = 0;
    double best_waste = 1e30;
    size_t best_x = 0, best_dy = 0;
    if (f16 && wp <= 256 && g.sh <= 8 && g.sw <= 8 && ((f32_mode >> 8) & 0xff) != 0xFC) {
      for (int tr = 1; tr <= std::min(g.oh, 256 - dyr); ++tr) {
        const int kt = (tr * wp + 15) / 16 * 16;
        const int hh = tr + dyr;
        // rows the MMAs may touch: the last tap's shift plus a block of kt indices
        const size_t xb = align_up(size_t((phases - 1) * hh * wp + dyr * wp + dxr + kt) * 128, 1024);
        const size_t db = align_up(size_t(kt) * 128, 1024);
        if (WgradHaloCfg::smem_bytes(xb, db) > 232448) break;
        if (size_t(2) * 128 * wp * (phases * hh + tr) > (size_t(1) << 20) - 1) break;
        // rows of the last, partly filled step of an image count as waste too
        const double waste = double(kt) * ((g.oh + tr - 1) / tr) / (double(g.oh) * g.ow);
        if (waste <= best_waste + 1e-12) { best_waste = waste; best_tr = tr; best_x = xb; best_dy = db; }
      }
    }
    if (best_tr > 0) {
      halo = true;
      hw.c_out = g.c_out; hw.n_total = a.n_total; hw.cb_per_tap = a.cb_per_tap;
      hw.kh = g.kh; hw.kw = g.kw; hw.pad_h = g.ph; hw.pad_w = g.pw; hw.oh = g.oh;
      hw.sh = g.sh; hw.sw = g.sw; hw.org_x = org_x; hw.org_y = org_y; hw.hh = best_tr + dyr;
      hw.tr = best_tr; hw.wp = wp; hw.ksteps = (best_tr * wp + 15) / 16;
      hw.steps_per_image = (g.oh + best_tr - 1) / best_tr;
      const long long steps = static_cast<long long>(g.n) * hw.steps_per_image;
      hw.total_steps = int(steps);
      hw.ocbs = cop / 64; hw.icbs = cip / 64;
      hw.tgs = (pairs + WgradHaloCfg::MAX_UNITS - 1) / WgradHaloCfg::MAX_UNITS;
      hw.taps_per_group = 2 * ((pairs + hw.tgs - 1) / hw.tgs);
      const long long items = static_cast<long long>(hw.ocbs) * hw.icbs * hw.tgs;
      hw.splits = int(std::max<long long>(1, std::min<long long>(steps, h->sm_count / std::max<long long>(1, items))));
      hw.x_plane_bytes = uint32_t(best_x); hw.dy_plane_bytes = uint32_t(best_dy);
      hw.status = h->status;
      if (steps > INT32_MAX || items * hw.splits > INT32_MAX) halo = false;
      else a.splits = hw.splits;
    }
  }
  if (phases > 1 && !halo)
    return fail(MTB200_ERR_UNSUPPORTED, "strided weight gradient: no step of the halo kernel fits shared memory");
  const size_t bytes_dy = split_bytes(opix, cop, g.n), bytes_x = split_bytes(ppix, cip, g.n);   // room for three planes
  const size_t bytes_part = align_up(sizeof(float) * size_t(a.splits) * g.c_out * a.n_total, 1024);
  const size_t bytes_e = align_up(sizeof(int) * size_t(g.n), 1024);
  void* ws = nullptr;
  int32_t rc = workspace_reserve(h, bytes_dy + bytes_x + bytes_part + 2 * bytes_e + 1024, &ws);
  if (rc) return rc;
  char* wbase = static_cast<char*>(ws);
  __nv_bfloat16* p_dy = static_cast<__nv_bfloat16*>(ws);
  __nv_bfloat16* p_x = reinterpret_cast<__nv_bfloat16*>(wbase + bytes_dy);
  a.part = reinterpret_cast<float*>(wbase + bytes_dy + bytes_x);
  int* e_dy = reinterpret_cast<int*>(wbase + bytes_dy + bytes_x + bytes_part);
  int* e_x = reinterpret_cast<int*>(wbase + bytes_dy + bytes_x + bytes_part + bytes_e);
  uint32_t* amax = reinterpret_cast<uint32_t*>(wbase + bytes_dy + bytes_x + bytes_part + 2 * bytes_e);   // [2]
  const long long dy_img = static_cast<long long>(g.c_out) * opix, x_img = static_cast<long long>(g.c_in) * ipix;
  if (f16) {
    ProfScope prof(h, PROF_CONV_GATHER, double(g.n) * (opix * (8.0 * g.c_out + 4.0 * cop) + ipix * (8.0 * g.c_in + 4.0 * cip)));
    MTB_CUDA(cudaMemsetAsync(amax, 0, 2 * sizeof(uint32_t), h->stream));
    auto chunks_of = [&](long long total) {
      return int(std::max<long long>(1, std::min<long long>((total + 4095) / 4096, 16LL * h->sm_count)));
    };
    // the two tensors are prepared side by side: neither pass fills the memory system alone
    const bool side = h->side_stream && !h->profiling;
    cudaStream_t sx = side ? h->side_stream : h->stream;
    if (side) {
      MTB_CUDA(cudaEventRecord(h->ev_fork, h->stream));
      MTB_CUDA(cudaStreamWaitEvent(sx, h->ev_fork, 0));
    }
    finite_absmax_kernel<<<dim3(chunks_of(dy_img * g.n), 1), 256, 0, h->stream>>>(dy, 0, dy_img * g.n, amax, nf_word, MTB_FLAG_SET);
    MTB_CUDA(launch_pdl(h, split16_turn_batch_kernel, dim3((opix + 63) / 64, cop / 64, g.n), dim3(256), 0, dy,
                        static_cast<long long>(opix), dy_img, reinterpret_cast<__half*>(p_dy),
                        static_cast<const uint32_t*>(amax), 0, e_dy, opix, g.c_out, cop, RowPhases{0, 1, 1, 0, 0}));
    finite_absmax_kernel<<<dim3(chunks_of(x_img * g.n), 1), 256, 0, sx>>>(x, 0, x_img * g.n, amax + 1, nf_word, MTB_FLAG_SET);
    if (phases > 1 && ppix != ipix)   // phase images have rows / columns no pixel maps to: they must read as zero
      MTB_CUDA(cudaMemsetAsync(p_x, 0, size_t(2) * g.n * ppix * cip * sizeof(__half), sx));
    split16_turn_batch_kernel<<<dim3((ipix + 63) / 64, cip / 64, g.n), 256, 0, sx>>>(
        x, ipix, x_img, reinterpret_cast<__half*>(p_x), amax + 1, 0, e_x, ipix, g.c_in, cip,
        RowPhases{g.w, g.sh, g.sw, hq, wq});
    MTB_CUDA(cudaGetLastError());
    if (side) {
      MTB_CUDA(cudaEventRecord(h->ev_join, sx));
      MTB_CUDA(cudaStreamWaitEvent(h->stream, h->ev_join, 0));
    }
  } else {
    ProfScope prof(h, PROF_CONV_GATHER, double(g.n) * (opix * (4.0 * g.c_out + 6.0 * cop) + ipix * (4.0 * g.c_in + 6.0 * cip)));
    rc = launch_split(h, dy, true, opix, g.c_out, cop, g.n, dy_img, p_dy, 3, nf_word, MTB_FLAG_SET);
    if (rc) return rc;
    rc = launch_split(h, x, true, ipix, g.c_in, cip, g.n, x_img, p_x, 3, nf_word, MTB_FLAG_SET);
    if (rc) return rc;
  }
  CUtensorMap tdy, tx;
  if (halo) {
    hw.part = a.part;
    rc = image_plane_tmap(&tdy, p_dy, cop, g.ow, g.oh, g.n, 2, 64, uint32_t(hw.wp), uint32_t(hw.tr), CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    if (phases == 1) {
      rc = image_plane_tmap(&tx, p_x, cip, g.w, g.h, g.n, 2, 64, uint32_t(hw.wp), uint32_t(hw.hh), CU_TENSOR_MAP_SWIZZLE_128B);
    } else {   // {c, x, y, phase, image*planes + split} over the phase images
      EncodeTiledFn enc = get_encode_tiled();
      if (!enc) return fail(MTB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
      const cuuint64_t dims[5] = {cuuint64_t(cip), cuuint64_t(wq), cuuint64_t(hq), cuuint64_t(phases), cuuint64_t(2) * g.n};
      const cuuint64_t strides[4] = {cuuint64_t(cip) * 2, cuuint64_t(wq) * cip * 2, cuuint64_t(hq) * wq * cip * 2,
                                     cuuint64_t(phases) * hq * wq * cip * 2};
      const cuuint32_t box[5] = {64, cuuint32_t(hw.wp), cuuint32_t(hw.hh), cuuint32_t(phases), 1};
      const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
      CUresult r5 = enc(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, p_x, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      rc = r5 == CUDA_SUCCESS ? MTB200_OK : fail(MTB200_ERR_CUDA, "cuTensorMapEncodeTiled (phase images) failed (%d)", int(r5));
    }
    if (rc) return rc;
    ProfScope prof(h, PROF_GEMM_UMMA, 2.0 * g.c_out * double(opix) * taps * g.c_in * g.n);
    const size_t smem = WgradHaloCfg::smem_bytes(hw.x_plane_bytes, hw.dy_plane_bytes);
    if (int32_t rc_attr = grant_dynamic_smem(h, conv_wgrad_halo_kernel, int(smem))) return rc_attr;
    MTB_CUDA(launch_pdl(h, conv_wgrad_halo_kernel, dim3(hw.ocbs * hw.icbs * hw.tgs * hw.splits),
                        dim3(WgradHaloCfg::NUM_THREADS), smem, tdy, tx, hw));
  } else {
  rc = image_plane_tmap(&tdy, p_dy, cop, g.ow, g.oh, g.n, a.planes, 64, a.tw, a.th, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = image_plane_tmap(&tx, p_x, cip, g.w, g.h, g.n, a.planes, 64, a.tw, a.th, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  {
    ProfScope prof(h, PROF_GEMM_UMMA, 2.0 * g.c_out * double(opix) * taps * g.c_in * g.n);
    if (f16) {
      using Cfg = WgradCfg<2>;
      if (int32_t rc_attr = grant_dynamic_smem(h, conv_wgrad_umma_kernel<2>, int(Cfg::SMEM_BYTES))) return rc_attr;
      conv_wgrad_umma_kernel<2><<<a.splits * tiles, Cfg::NUM_THREADS, Cfg::SMEM_BYTES, h->stream>>>(tdy, tx, a);
    } else {
      using Cfg = WgradCfg<3>;
      if (int32_t rc_attr = grant_dynamic_smem(h, conv_wgrad_umma_kernel<3>, int(Cfg::SMEM_BYTES))) return rc_attr;
      conv_wgrad_umma_kernel<3><<<a.splits * tiles, Cfg::NUM_THREADS, Cfg::SMEM_BYTES, h->stream>>>(tdy, tx, a);
    }
    MTB_CUDA(cudaGetLastError());
  }
  }
  const long long part_rows = static_cast<long long>(g.c_out) * a.n_total;
  MTB_CUDA(launch_pdl(h, wgrad_reduce_kernel, dim3(unsigned(std::min<long long>((part_rows + 31) / 32, 8192))), dim3(256), 0,
                      static_cast<const float*>(a.part), a.splits, g.c_out, g.c_in, cip, taps, dw,
                      static_cast<const int*>(f16 ? e_dy : nullptr), static_cast<const int*>(f16 ? e_x : nullptr)));
  return MTB200_OK;
}

static int32_t check_geom(int64_t n, int64_t c_in, int64_t h, int64_t w, int64_t c_out, int64_t kh,
                          int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, ConvGeom* g) {
  if (n < 0 || c_in < 0 || h < 0 || w < 0 || c_out < 0 || kh <= 0 || kw <= 0 || ph < 0 || pw < 0)
    return fail(MTB200_ERR_INVALID, "conv2d: negative or empty dimension");
  if (sh <= 0 || sw <= 0) return fail(MTB200_ERR_INVALID, "stride values must be greater than zero");
  if (kh > h + 2 * ph || kw > w + 2 * pw)
    return fail(MTB200_ERR_INVALID, "kernel size cannot be larger than padded input");
  const int64_t oh = (h + 2 * ph - kh) / sh + 1, ow = (w + 2 * pw - kw) / sw + 1;
  const int64_t lim = INT32_MAX;
  if (n > 65535 || c_in * kh * kw > lim || c_out * kh * kw > lim || h * w > lim || oh * ow > lim ||
      c_in * h * w > lim || c_out * oh * ow > lim)
    return fail(MTB200_ERR_INVALID, "conv2d: dimension exceeds the limits of the device kernels");
  *g = ConvGeom{int(n), int(c_in), int(h), int(w), int(c_out), int(kh), int(kw), int(sh), int(sw),
                int(ph), int(pw), int(oh), int(ow)};
  return MTB200_OK;
}

}  // namespace mtb

using namespace mtb;

#define MTB_CHECK_HANDLE(h)                                         \
  if (!(h)) return fail(MTB200_ERR_INVALID, "null handle");         \
  DeviceGuard guard__((h)->device);                                 \
  if (!guard__.ok) return fail(MTB200_ERR_CUDA, "cannot make device %d current", (h)->device)

extern "C" {

int32_t mtb200_conv2d_fwd(mtb200_handle h, int64_t n, int64_t c_in, int64_t height, int64_t width,
                          int64_t c_out, int64_t kh, int64_t kw, int64_t stride_h, int64_t stride_w,
                          int64_t pad_h, int64_t pad_w, const float* x, const float* w, const float* bias,
                          float* y, int32_t f32_mode) {
  MTB_CHECK_HANDLE(h);
  ConvGeom g;
  int32_t rc = check_geom(n, c_in, height, width, c_out, kh, kw, stride_h, stride_w, pad_h, pad_w, &g);
  if (rc) return rc;
  const int opix = g.oh * g.ow;
  if (g.n == 0 || g.c_out == 0 || opix == 0) return MTB200_OK;
  if (!y) return fail(MTB200_ERR_INVALID, "null output pointer");
  const int K = g.c_in * g.kh * g.kw;
  if (K == 0) return fail(MTB200_ERR_UNSUPPORTED, "conv2d with zero input channels is not supported");
  if (!x || !w) return fail(MTB200_ERR_INVALID, "null input pointer");
  const bool force_explicit = ((f32_mode >> 8) & 0xff) == 0xff;  // test hook: gathered-patch lowering
  uint32_t* nf_word = nullptr;
  rc = call_flag_begin(h, &nf_word);
  if (rc) return rc;
  auto redo = [&]() -> int32_t {   // returns at once unless the operands held Inf / NaN
    MTB_CUDA(launch_pdl(h, conv_direct_fwd_kernel, dim3(direct_grid(h, static_cast<long long>(g.n) * g.c_out * opix)),
                        dim3(256), 0, g, x, w, bias, y, static_cast<const uint32_t*>(nf_word)));
    return MTB200_OK;
  };
  if (g.sh == 1 && g.sw == 1 && g.ow <= 256 && !force_explicit) {
    rc = implicit_conv(h, x, g.n, g.c_in, g.h, g.w, w, g.c_out, g.kh, g.kw, 0, g.oh, g.ow, -g.pw, -g.ph, +1,
                       bias, y, f32_mode, nf_word);
    return rc ? rc : redo();
  }
  // Strided forward: the same implicit kernel over phase images (default arithmetic only; strides up to 8 and
  // filters of at most 128 taps; anything else takes the gathered-patch lowering below).
  const int vb = (f32_mode >> 8) & 0xff;
  if ((g.sh > 1 || g.sw > 1) && g.sh <= 8 && g.sw <= 8 && g.kh * g.kw <= 128 && !force_explicit && vb != 0xFB && vb != 0xFC &&
      ((f32_mode & 0xff) == 0 || (f32_mode & 0xff) == 23)) {
    rc = implicit_conv(h, x, g.n, g.c_in, g.h, g.w, w, g.c_out, g.kh, g.kw, 0, g.oh, g.ow, 0, 0, +1, bias, y, f32_mode,
                       nf_word, g.sh, g.sw, g.ph, g.pw);
    if (rc == MTB200_OK) return redo();
    if (rc != MTB200_ERR_UNSUPPORTED) return rc;
  }
  const int Kp = padded_k(K);
  const size_t bytes_w = split_bytes(g.c_out, Kp, 1), bytes_p = split_bytes(opix, Kp, g.n);
  void* ws = nullptr;
  rc = workspace_reserve(h, bytes_w + bytes_p, &ws);
  if (rc) return rc;
  __nv_bfloat16* sw_ = static_cast<__nv_bfloat16*>(ws);
  __nv_bfloat16* sp = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(ws) + bytes_w);
  rc = launch_split(h, w, false, g.c_out, K, Kp, 1, 0, sw_, 3, nf_word, MTB_FLAG_SET);
  if (rc) return rc;
  patch_split_kernel<PATCH_FWD><<<dim3((opix + 63) / 64, Kp / 64, g.n), 256, 0, h->stream>>>(
      x, g, opix, K, Kp, static_cast<long long>(g.c_in) * g.h * g.w, sp, nf_word);
  MTB_CUDA(cudaGetLastError());
  SplitOperand oa{sw_, g.c_out, 0, 1}, ob{sp, opix, g.n > 1, g.n};
  rc = run_split_gemm(h, oa, ob, Kp, g.n, g.c_out, opix, y, opix, static_cast<long long>(g.c_out) * opix,
                      bias, EPI_NONE, nullptr, bf16_mode_of(f32_mode), gemm_variant_of(f32_mode), /*bias_per_row=*/1);
  return rc ? rc : redo();
}

int32_t mtb200_conv2d_bwd_data(mtb200_handle h, int64_t n, int64_t c_in, int64_t height, int64_t width,
                               int64_t c_out, int64_t kh, int64_t kw, int64_t stride_h, int64_t stride_w,
                               int64_t pad_h, int64_t pad_w, const float* dy, const float* w, float* dx,
                               int32_t f32_mode) {
  MTB_CHECK_HANDLE(h);
  ConvGeom g;
  int32_t rc = check_geom(n, c_in, height, width, c_out, kh, kw, stride_h, stride_w, pad_h, pad_w, &g);
  if (rc) return rc;
  const int ipix = g.h * g.w;
  if (g.n == 0 || g.c_in == 0 || ipix == 0) return MTB200_OK;
  if (!dx) return fail(MTB200_ERR_INVALID, "null output pointer");
  const int K = g.c_out * g.kh * g.kw;
  if (K == 0 || g.oh * g.ow == 0) {
    MTB_CUDA(cudaMemsetAsync(dx, 0, sizeof(float) * g.n * g.c_in * ipix, h->stream));
    return MTB200_OK;
  }
  if (!dy || !w) return fail(MTB200_ERR_INVALID, "null input pointer");
  const bool force_explicit = ((f32_mode >> 8) & 0xff) == 0xff;
  uint32_t* nf_word = nullptr;
  rc = call_flag_begin(h, &nf_word);
  if (rc) return rc;
  auto redo = [&]() -> int32_t {
    MTB_CUDA(launch_pdl(h, conv_direct_dgrad_kernel, dim3(direct_grid(h, static_cast<long long>(g.n) * g.c_in * ipix)),
                        dim3(256), 0, g, dy, w, dx, static_cast<const uint32_t*>(nf_word)));
    return MTB200_OK;
  };
  if (g.sh == 1 && g.sw == 1 && g.w <= 256 && !force_explicit) {
    rc = implicit_conv(h, dy, g.n, g.c_out, g.oh, g.ow, w, g.c_in, g.kh, g.kw, 1, g.h, g.w, g.pw, g.ph, -1,
                       nullptr, dx, f32_mode, nf_word);
    return rc ? rc : redo();
  }
  // Strided data gradient, one output phase at a time.  Input pixel iy = sh * y' + py receives, from filter row fh,
  // dy row (iy + ph - fh) / sh - only where that division is exact, i.e. for fh = fh0 + a * sh with
  // fh0 = (py + ph) mod sh - so phase (py, px) of dx is a STRIDE-1 data gradient of dy under the sub-filter
  // {fh0 + a * sh} x {fw0 + b * sw}: dy row y' + (py + ph - fh0) / sh - a.  The dy planes are prepared once; every
  // phase gathers its sub-filter and runs the pixel kernel, which scatters its outputs with the strides.
  if ((g.sh > 1 || g.sw > 1) && (f32_mode & 0xff) == 0 && !force_explicit && g.sh <= 8 && g.sw <= 8 && g.ow <= 4096) {
    bool uncovered = false;     // a phase no tap reaches stays zero
    for (int py = 0; py < g.sh && py < g.h; ++py)
      for (int px = 0; px < g.sw && px < g.w; ++px)
        if ((py + g.ph) % g.sh >= g.kh || (px + g.pw) % g.sw >= g.kw) uncovered = true;
    if (uncovered) MTB_CUDA(cudaMemsetAsync(dx, 0, sizeof(float) * size_t(g.n) * g.c_in * ipix, h->stream));
    bool first = true, fell_back = false;
    for (int py = 0; py < g.sh && py < g.h && !fell_back; ++py)
      for (int px = 0; px < g.sw && px < g.w; ++px) {
        const int fh0 = (py + g.ph) % g.sh, fw0 = (px + g.pw) % g.sw;
        if (fh0 >= g.kh || fw0 >= g.kw) continue;
        const int nfh = (g.kh - 1 - fh0) / g.sh + 1, nfw = (g.kw - 1 - fw0) / g.sw + 1;
        ConvPhaseOut po = {};
        po.sub = TapSubset{fh0, g.sh, nfh, fw0, g.sw, nfw};
        po.kh_full = g.kh; po.kw_full = g.kw;
        po.image_ready = !first;
        po.out_sy = g.sh; po.out_sx = g.sw; po.out_pitch = g.w;
        po.out_plane = ipix;
        po.out_offset = static_cast<long long>(py) * g.w + px;
        rc = implicit_conv(h, dy, g.n, g.c_out, g.oh, g.ow, w, g.c_in, nfh, nfw, 1, (g.h - py + g.sh - 1) / g.sh,
                           (g.w - px + g.sw - 1) / g.sw, (px + g.pw - fw0) / g.sw, (py + g.ph - fh0) / g.sh, -1, nullptr,
                           dx, f32_mode, nf_word, 1, 1, 0, 0, &po);
        if (rc == MTB200_ERR_UNSUPPORTED) { fell_back = true; break; }   // the gathered-patch lowering below writes all of dx
        if (rc) return rc;
        first = false;
      }
    if (!fell_back) return redo();
  }
  const int Kp = padded_k(K);
  const size_t bytes_w = split_bytes(g.c_in, Kp, 1), bytes_p = split_bytes(ipix, Kp, g.n);
  const size_t bytes_perm = align_up(sizeof(float) * size_t(g.c_in) * K, 1024);
  void* ws = nullptr;
  rc = workspace_reserve(h, bytes_w + bytes_p + bytes_perm, &ws);
  if (rc) return rc;
  __nv_bfloat16* sw_ = static_cast<__nv_bfloat16*>(ws);
  __nv_bfloat16* sp = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(ws) + bytes_w);
  float* wperm = reinterpret_cast<float*>(static_cast<char*>(ws) + bytes_w + bytes_p);
  const long long wtotal = static_cast<long long>(g.c_in) * K;
  permute_weight_kernel<<<int(std::min<long long>((wtotal + 255) / 256, 4096)), 256, 0, h->stream>>>(
      w, wperm, g.c_out, g.c_in, g.kh * g.kw);
  MTB_CUDA(cudaGetLastError());
  rc = launch_split(h, wperm, false, g.c_in, K, Kp, 1, 0, sw_, 3, nf_word, MTB_FLAG_SET);
  if (rc) return rc;
  patch_split_kernel<PATCH_BWD><<<dim3((ipix + 63) / 64, Kp / 64, g.n), 256, 0, h->stream>>>(
      dy, g, ipix, K, Kp, static_cast<long long>(g.c_out) * g.oh * g.ow, sp, nf_word);
  MTB_CUDA(cudaGetLastError());
  SplitOperand oa{sw_, g.c_in, 0, 1}, ob{sp, ipix, g.n > 1, g.n};
  rc = run_split_gemm(h, oa, ob, Kp, g.n, g.c_in, ipix, dx, ipix, static_cast<long long>(g.c_in) * ipix,
                      nullptr, EPI_NONE, nullptr, bf16_mode_of(f32_mode), gemm_variant_of(f32_mode));
  return rc ? rc : redo();
}

int32_t mtb200_conv2d_bwd_weight(mtb200_handle h, int64_t n, int64_t c_in, int64_t height, int64_t width,
                                 int64_t c_out, int64_t kh, int64_t kw, int64_t stride_h, int64_t stride_w,
                                 int64_t pad_h, int64_t pad_w, const float* dy, const float* x, float* dw,
                                 int32_t f32_mode) {
  MTB_CHECK_HANDLE(h);
  ConvGeom g;
  int32_t rc = check_geom(n, c_in, height, width, c_out, kh, kw, stride_h, stride_w, pad_h, pad_w, &g);
  if (rc) return rc;
  const int rows_b = g.c_in * g.kh * g.kw;
  if (g.c_out == 0 || rows_b == 0) return MTB200_OK;
  if (!dw) return fail(MTB200_ERR_INVALID, "null output pointer");
  const long long Ktot = static_cast<long long>(g.n) * g.oh * g.ow;
  const size_t out_elems = size_t(g.c_out) * rows_b;
  if (Ktot == 0) {
    MTB_CUDA(cudaMemsetAsync(dw, 0, sizeof(float) * out_elems, h->stream));
    return MTB200_OK;
  }
  if (!dy || !x) return fail(MTB200_ERR_INVALID, "null input pointer");
  uint32_t* nf_word = nullptr;
  rc = call_flag_begin(h, &nf_word);
  if (rc) return rc;
  auto redo = [&]() -> int32_t {
    MTB_CUDA(launch_pdl(h, conv_direct_wgrad_kernel, dim3(unsigned(std::min<size_t>(out_elems, size_t(16) * h->sm_count))),
                        dim3(256), 0, g, dy, x, dw, static_cast<const uint32_t*>(nf_word)));
    return MTB200_OK;
  };
  const bool strided = g.sh > 1 || g.sw > 1;
  if (((f32_mode >> 8) & 0xff) != 0xff && (!strided || (f32_mode & 0xff) == 0)) {
    rc = implicit_wgrad(h, g, dy, x, dw, f32_mode, nf_word);
    if (!(strided && rc == MTB200_ERR_UNSUPPORTED)) return rc ? rc : redo();
    // a strided layer the halo kernel has no step for: the gathered-patch lowering below
  }
  // split K: enough chunks to occupy the machine, each a whole number of 64-wide K blocks
  const long long kblocks = (Ktot + 63) / 64;
  const int tiles = ((g.c_out + 127) / 128) * ((rows_b + 255) / 256);
  int chunks = int(std::min<long long>(kblocks, std::max(1, (2 * h->sm_count + tiles - 1) / tiles)));
  const long long kb_per_chunk = (kblocks + chunks - 1) / chunks;
  chunks = int((kblocks + kb_per_chunk - 1) / kb_per_chunk);
  const long long Kp = kb_per_chunk * chunks * 64;
  if (Kp > INT32_MAX) return fail(MTB200_ERR_INVALID, "conv2d weight gradient: reduction length exceeds 2^31");
  const size_t bytes_a = align_up(size_t(3) * g.c_out * Kp * 2, 1024);
  const size_t bytes_b = align_up(size_t(3) * rows_b * Kp * 2, 1024);
  const size_t bytes_part = align_up(sizeof(float) * out_elems * chunks, 1024);
  void* ws = nullptr;
  rc = workspace_reserve(h, bytes_a + bytes_b + bytes_part, &ws);
  if (rc) return rc;
  __nv_bfloat16* sa = static_cast<__nv_bfloat16*>(ws);
  __nv_bfloat16* sb = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(ws) + bytes_a);
  float* part = reinterpret_cast<float*>(static_cast<char*>(ws) + bytes_a + bytes_b);
  const int gsz = h->sm_count * 16;
  wgrad_split_kernel<WG_DY><<<gsz, 256, 0, h->stream>>>(dy, g, g.c_out, Ktot, Kp, sa, nf_word);
  wgrad_split_kernel<WG_PATCH><<<gsz, 256, 0, h->stream>>>(x, g, rows_b, Ktot, Kp, sb, nf_word);
  MTB_CUDA(cudaGetLastError());
  SplitOperand oa{sa, g.c_out, 0, 1}, ob{sb, rows_b, 0, 1};
  float* gemm_out = chunks == 1 ? dw : part;
  rc = run_split_gemm(h, oa, ob, int(Kp), chunks, g.c_out, rows_b, gemm_out, rows_b, (long long)out_elems,
                      nullptr, EPI_NONE, nullptr, bf16_mode_of(f32_mode), 0, 0,
                      /*kb_batch_stride=*/int(kb_per_chunk), /*num_kb (64-wide)=*/int(kb_per_chunk));
  if (rc) return rc;
  if (chunks > 1) {
    colsum_stage2_kernel<float><<<int((out_elems + 255) / 256), 256, 0, h->stream>>>(part, chunks, int(out_elems), dw);
    MTB_CUDA(cudaGetLastError());
  }
  return redo();
}

int32_t mtb200_conv2d_bwd_bias(mtb200_handle h, int64_t n, int64_t c_out, int64_t out_h, int64_t out_w,
                               const float* dy, float* db) {
  MTB_CHECK_HANDLE(h);
  if (n < 0 || c_out < 0 || out_h < 0 || out_w < 0 || out_h * out_w > INT32_MAX || n > INT32_MAX ||
      c_out > 65535 * 32)
    return fail(MTB200_ERR_INVALID, "conv2d bias gradient: bad dimension");
  if (c_out == 0) return MTB200_OK;
  if (!db) return fail(MTB200_ERR_INVALID, "null output pointer");
  const int opix = int(out_h * out_w);
  if (n == 0 || opix == 0) {
    MTB_CUDA(cudaMemsetAsync(db, 0, sizeof(float) * c_out, h->stream));
    return MTB200_OK;
  }
  if (!dy) return fail(MTB200_ERR_INVALID, "null input pointer");
  int chunks = int(std::min<int64_t>(n, std::max<int64_t>(1, (16 * h->sm_count) / c_out)));
  chunks = std::min(chunks, 65535);
  const int per = int((n + chunks - 1) / chunks);
  chunks = int((n + per - 1) / per);
  void* ws = nullptr;
  int32_t rc = workspace_reserve(h, sizeof(float) * size_t(chunks) * c_out, &ws);
  if (rc) return rc;
  float* part = static_cast<float*>(ws);
  conv_bias_partial_kernel<<<dim3(unsigned(c_out), unsigned(chunks)), 256, 0, h->stream>>>(dy, int(n), int(c_out), opix,
                                                                                         per, part);
  MTB_CUDA(cudaGetLastError());
  MTB_CUDA(launch_pdl(h, colsum_stage2_kernel<float>, dim3(unsigned((c_out + 255) / 256)), dim3(256), 0,
                      static_cast<const float*>(part), chunks, int(c_out), db));
  return MTB200_OK;
}

}  // extern "C"
