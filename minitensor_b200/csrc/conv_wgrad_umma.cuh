// Weight gradient of a stride-1 convolution as an implicit GEMM on the tcgen05
// tensor cores (split-plane arithmetic, see gemm_split_umma.cuh: three bf16 planes, or two fp16 planes of operands
// scaled by one power of two per tensor - the reduction runs over images and pixels, so no finer scale factors out).
//
//   dW[oc][(tap, ic)] = sum over k = (image, oh, ow) of dy[k][oc] * x[k shifted by tap][ic]
//
// Both operands are read straight from channels-last bf16 planes
// {c, w, h, image*planes+split}: a K block is a window of 64 pixels (TH rows x TW
// columns, TW a power of two >= min(OW, 64)); the dy window and the x window
// shifted by the tap's offset land in shared memory as [pixel][64 channels],
// which is exactly an MN-major operand chunk (the reduction index walks down
// the rows).  Pixels outside the image read as zero (hardware fill), which
// supplies both the padding and the unused part of a partly filled window.
// The reference computes the same sums with scalar loops
// (engine/src/autograd/mod/shape.rs:130-169).
//
// M tile = 128 output channels (two 64-channel chunks), N tile = two (tap,
// 64-input-channel) chunks.  The reduction is split across CTAs: CTA z of a
// tile handles K blocks [z*kb_per_split, ...) and writes its partial tile to
// part[z][oc][n_total]; a second kernel adds the partials in order and
// permutes (tap, ic) -> (ic, tap).
#pragma once
#include "gemm_split_umma.cuh"

namespace mtb {

struct WgradArgs {
  int c_out, n_chunks;       // output channels; number of (tap, channel block) chunks = taps * (cin_p / 64)
  int cb_per_tap;            // cin_p / 64
  int kw, pad_h, pad_w;      // filter width; padding
  int th, tw;                // window: th rows x tw columns = 64 pixels
  int wblocks, hblocks;      // windows per image row / column direction
  int total_kb, kb_per_split, splits;
  int tiles_m, tiles_n;      // ceil(c_out / 128), ceil(n_chunks / 2)
  int n_total;               // n_chunks * 64: row length of a partial
  float* part;               // [splits][c_out][n_total]
  int mode;                  // 1, 3, 6, 9: bf16 products; 23: fp16 two-plane mode
  int planes;                // planes stored per image (3 bf16, 2 fp16)
  uint32_t* status;
};

// PLANES = planes per operand held in a stage: 3 (bf16 modes, two stages of 96 KB) or 2 (fp16 mode, three stages
// of 64 KB).
template <int PLANES>
struct WgradCfg {
  static constexpr int BM = 128, BN = 128, BK = 64, STAGES = PLANES == 2 ? 3 : 2;
  static constexpr int CHUNK = 64 * 128;                 // 64 pixels x 64 channels x 2 bytes
  static constexpr int A_TILE = 2 * CHUNK, B_TILE = 2 * CHUNK;
  static constexpr int STAGE_BYTES = PLANES * A_TILE + PLANES * B_TILE;
  static constexpr int TMEM_COLS = 128;
  static constexpr int NUM_THREADS = 192;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

template <int PLANES>
__global__ void __launch_bounds__(192, 1)
conv_wgrad_umma_kernel(const __grid_constant__ CUtensorMap tmapDy, const __grid_constant__ CUtensorMap tmapX,
                       const WgradArgs g) {
  using Cfg = WgradCfg<PLANES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  const uint32_t bars = tiles + Cfg::STAGES * Cfg::STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (Cfg::STAGES + s); };
  const uint32_t acc_full = bars + 8u * (2 * Cfg::STAGES);
  const uint32_t tmem_slot = bars + 8u * (2 * Cfg::STAGES + 1);
  const uint32_t abort_addr = tmem_slot + 4u;
  volatile uint32_t* abort_word = reinterpret_cast<volatile uint32_t*>(smem_raw + (abort_addr - raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // one work item per CTA: (split z, m tile, n tile)
  const int item = blockIdx.x;
  const int per_split = g.tiles_m * g.tiles_n;
  const int z = item / per_split;
  const int tm = (item % per_split) / g.tiles_n, tn = item % g.tiles_n;
  const int kb_begin = z * g.kb_per_split;
  const int kb_end = min(g.total_kb, kb_begin + g.kb_per_split);
  const int nsplit = (g.mode == 1) ? 1 : ((g.mode == 3 || g.mode == 23) ? 2 : 3);
  // chunks of this tile that exist (a tile past the end of M or N has fewer)
  const int a_chunks = min(2, (g.c_out + 63) / 64 - tm * 2);
  const int b_chunks = min(2, g.n_chunks - tn * 2);
  const uint32_t stage_tx = nsplit * (a_chunks + b_chunks) * Cfg::CHUNK;

  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full, 1);
    fence_mbar_init();
    prefetch_tmap(&tmapDy);
    prefetch_tmap(&tmapX);
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  const bool has_work = kb_begin < kb_end;

  if (warp == 0) {
    if (lane == 0 && has_work) {
      int stage = 0;
      uint32_t phase = 0;
      const int per_image = g.hblocks * g.wblocks;
      for (int kb = kb_begin; kb < kb_end; ++kb) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_word)) {
          *abort_word = 1;
          atomicMax(g.status, 0x100u | 5u);
          break;
        }
        const int img = kb / per_image;
        const int r = kb - img * per_image;
        const int h0 = (r / g.wblocks) * g.th, w0 = (r % g.wblocks) * g.tw;
        mbar_expect_tx(full_bar(stage), stage_tx);
        const uint32_t sa = tiles + stage * Cfg::STAGE_BYTES;
        const uint32_t sb = sa + PLANES * Cfg::A_TILE;
        for (int s = 0; s < nsplit; ++s)
          for (int c = 0; c < a_chunks; ++c)
            tma_load_4d(sa + s * Cfg::A_TILE + c * Cfg::CHUNK, &tmapDy, full_bar(stage), (tm * 2 + c) * 64, w0, h0,
                        img * g.planes + s);
        for (int c = 0; c < b_chunks; ++c) {
          const int q = tn * 2 + c;
          const int tap = q / g.cb_per_tap, cb = q - tap * g.cb_per_tap;
          const int fh = tap / g.kw, fw = tap - fh * g.kw;
          for (int s = 0; s < nsplit; ++s)
            tma_load_4d(sb + s * Cfg::B_TILE + c * Cfg::CHUNK, &tmapX, full_bar(stage), cb * 64, w0 + fw - g.pad_w,
                        h0 + fh - g.pad_h, img * g.planes + s);
        }
        if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && has_work) {
      // both operands MN-major; bf16 planes, or fp16 planes in mode 23
      const uint32_t idesc = make_idesc(Cfg::BM, Cfg::BN, g.mode == 23 ? 0u : 1u, 1u, 1u, 1u);
      // issue loop with the product schedule known at compile time (one add per descriptor)
      auto issue_all = [&](auto npairs_tag) {
        constexpr int NPAIRS = decltype(npairs_tag)::value;
        int stage = 0;
        uint32_t phase = 0, accumulate = 0;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_word)) {
            *abort_word = 1;
            atomicMax(g.status, 0x200u | 5u);
            return;
          }
          tc_fence_after();
          const uint32_t sa = tiles + stage * Cfg::STAGE_BYTES;
          const uint32_t sb = sa + PLANES * Cfg::A_TILE;
          const uint64_t da0 = make_mnmajor_desc(sa, Cfg::CHUNK);
          const uint64_t db0 = make_mnmajor_desc(sb, Cfg::CHUNK);
#pragma unroll
          for (int kk = 0; kk < Cfg::BK / 16; ++kk) {
#pragma unroll
            for (int p = 0; p < NPAIRS; ++p) {
              const int code = split_pair_at(NPAIRS, p);
              const uint32_t offa = (code >> 2) * Cfg::A_TILE + kk * 2048;
              const uint32_t offb = (code & 3) * Cfg::B_TILE + kk * 2048;
              umma_f16<1>(tmem_base, da0 + (offa >> 4), db0 + (offb >> 4), idesc, accumulate);
              accumulate = 1;
            }
          }
          umma_commit<1>(empty_bar(stage));
          if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1u; }
        }
        umma_commit<1>(acc_full);
      };
      if constexpr (PLANES == 2) {
        issue_all(std::integral_constant<int, 3>{});   // the fp16 mode's three products
      } else {
        switch (split_pair_count(g.mode)) {
          case 1: issue_all(std::integral_constant<int, 1>{}); break;
          case 3: issue_all(std::integral_constant<int, 3>{}); break;
          case 9: issue_all(std::integral_constant<int, 9>{}); break;
          default: issue_all(std::integral_constant<int, 6>{}); break;
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int row = tm * Cfg::BM + q * 32 + lane;
    float* prow = g.part + (static_cast<long long>(z) * g.c_out + row) * g.n_total;
    const int ncols = b_chunks * 64;  // columns of this tile that exist
    bool ready = has_work;
    if (has_work && !mbar_wait(acc_full, 0, abort_word)) {
      *abort_word = 1;
      if (lane == 0) atomicMax(g.status, 0x300u | 5u);
      ready = false;
    }
    if (ready) tc_fence_after();
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    for (int c0 = 0; c0 < ncols; c0 += 32) {
      uint32_t v[32];
      if (ready) {
        tmem_ld_32x32(t_row + c0, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0u;  // a split with no K blocks contributes zeros
      }
      if (row < g.c_out) {
        float* dst = prow + tn * 128 + c0;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                            __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
      }
    }
    tc_fence_before();
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, Cfg::TMEM_COLS);
  }
}

// dw[oc][ic][tap] = 2^(e1 + e2) * sum_z part[z][oc][tap*cin_p + ic]   (fixed order: deterministic); e1 / e2 = the
// operands' scale exponents in the fp16 mode (first entry of each vector), nullptr otherwise.
__global__ void __launch_bounds__(256)
wgrad_reduce_kernel(const float* __restrict__ part, int splits, int c_out, int c_in, int cin_p,
                    int taps, float* __restrict__ dw, const int* __restrict__ e1,
                    const int* __restrict__ e2) {
  // A block serves 32 consecutive entries of a partial's row (oc, (tap, ic)) - consecutive ic, so every load of a
  // warp is one 128-byte line - with 8 threads per entry: thread zl adds the ranges zl, zl + 8, ... in ascending
  // order and the eight sums are added in ascending zl, a fixed order whatever the launch.
  __shared__ float red[8][33];
  grid_dependency_wait();        // partials and exponents come from the kernels before this one
  grid_launch_dependents();
  const int e = e1 ? __ldcg(e1) + __ldcg(e2) : 0;
  const long long n_total = static_cast<long long>(taps) * cin_p;
  const long long rows = static_cast<long long>(c_out) * n_total;
  const int lane = threadIdx.x & 31, zl = threadIdx.x >> 5;
  for (long long base = static_cast<long long>(blockIdx.x) * 32; base < rows;
       base += static_cast<long long>(gridDim.x) * 32) {
    const long long j = base + lane;
    float s = 0.0f;
    if (j < rows) {
      const float* p = part + j;
      int z = zl;
      for (; z + 24 < splits; z += 32) {      // four loads in flight, added in ascending order
        const float a0 = p[static_cast<long long>(z) * rows], a1 = p[static_cast<long long>(z + 8) * rows];
        const float a2 = p[static_cast<long long>(z + 16) * rows], a3 = p[static_cast<long long>(z + 24) * rows];
        s += a0; s += a1; s += a2; s += a3;
      }
      for (; z < splits; z += 8) s += p[static_cast<long long>(z) * rows];
    }
    red[zl][lane] = s;
    __syncthreads();
    if (zl == 0 && j < rows) {
      float t = red[0][lane];
#pragma unroll
      for (int q = 1; q < 8; ++q) t += red[q][lane];
      const int oc = static_cast<int>(j / n_total);
      const int r = static_cast<int>(j - static_cast<long long>(oc) * n_total);
      const int tap = r / cin_p, ic = r - tap * cin_p;
      if (ic < c_in)
        dw[(static_cast<long long>(oc) * c_in + ic) * taps + tap] = e1 ? scale_pow2(t, e) : t;
    }
    __syncthreads();
  }
}

}  // namespace mtb
