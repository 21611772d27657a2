// f32-accurate GEMM on the tcgen05 tensor cores through bf16 operand splitting.
//
// An f32 value a is written as a0 + a1 + a2 with a_i bf16 (3 x 8 significand
// bits = 24 bits, exact for finite normal inputs).  The product a*b is then
// the sum of bf16 x bf16 products, each exact in the f32 accumulator held in
// tensor memory.  The kernel multiplies pre-split operands (see split_bf16.cuh)
// and keeps the products whose weight is at least 2^-24:
//   mode 6 (default, f32-accurate): a0b2 a2b0 a1b1 a0b1 a1b0 a0b0
//   mode 9: all nine;  mode 3: a0b1 a1b0 a0b0 (~2^-16);  mode 1: a0b0 (plain bf16)
// This replaces the CPU sgemm call of the reference matmul
// (engine/src/operations/linalg/matmul.rs:240-248) on the device.
//
// Kernel structure (one CTA per SM, persistent over output tiles):
//   warp 0     : TMA producer  - loads the A/B split tiles of a K block into a
//                shared-memory ring (tiled 3-D tensor maps, hardware swizzle)
//   warp 1     : MMA issuer    - one elected thread issues tcgen05.mma for every
//                (K step, split pair); owns the TMEM allocation
//   warps 2..5 : epilogue      - tcgen05.ld the finished accumulator, apply
//                bias / activation / mask, store f32 rows to global memory
// Two accumulators live in TMEM so the epilogue of tile i overlaps the main
// loop of tile i+1.
#pragma once
#include "ptx_sm100.cuh"
#include <cuda_bf16.h>

namespace mtb {

enum Epilogue : int {
  EPI_NONE = 0,
  EPI_RELU = 1,       // NaN passes through, x > 0 keeps x, else 0 (softmax.rs:161-203)
  EPI_GELU_ERF = 2,   // 0.5 x (1 + erf(x / sqrt 2))           (hyperbolic.rs:697-745)
  EPI_GELU_TANH = 3,  // 0.5 x (1 + tanh(c (x + 0.044715 x^3)))
  EPI_RELU_BWD = 4,   // multiply by (aux > 0 ? 1 : 0): ReluBackward fused (shape.rs:724-816)
};

struct GemmArgs {
  int M, N;            // logical output extent per batch entry
  int num_kb;          // K blocks (padded K / BK)
  int batch;
  float* C;            // [batch][M][ldc]
  long long ldc;       // row stride of C in elements
  long long strideC;   // batch stride of C in elements
  const float* bias;   // [N] added to every row, or nullptr
  const float* aux;    // same layout as C, read by EPI_RELU_BWD, or nullptr
  int epilogue;
  int mode;            // 1, 3, 6 or 9 bf16 split products; 23 = fp16 two-plane mode (3 products)
  int planes_per_mat;  // planes stored per matrix in the operand arrays (3 bf16, 2 fp16)
  const int* exp_a;    // fp16 mode: per-row scale exponents of A ([batch][M] if A is batched), else nullptr
  const int* exp_b;    // fp16 mode: per-column scale exponents of B ([batch][N] if B is batched)
  int a_batched;       // 0: one A shared by all batch entries
  int b_batched;
  int bias_per_row;    // 0: bias[N] added along columns; 1: bias[M] added along rows
  int kb_batch_stride; // split-K: batch entry b reduces K blocks [b*stride, b*stride + num_kb)
  uint32_t* status;    // device word; a non-zero value reports a wait that ran out
  // Implicit-convolution mode (CONV kernels only): the B operand is read straight
  // from channels-last image planes {c, w, h, image*3+split}; a K block is one
  // (filter tap, channel block) and an N tile is cv_th full image rows.
  int cv_n_tile;       // columns per N tile = cv_th * tile width
  int cv_umma_n;       // MMA N: cv_n_tile rounded up to a multiple of 16
  int cv_th;           // image rows per N tile
  int cv_kb_per_tap;   // channel blocks per filter tap
  int cv_kw;           // filter width (taps per filter row)
  int cv_w0, cv_h0;    // window origin for tap (0,0): -pad (forward) or +pad (data gradient)
  int cv_sgn;          // +1 forward (origin + tap), -1 data gradient (origin - tap)
};

__device__ __forceinline__ float apply_epilogue(float x, int epi, float aux) {
  switch (epi) {
    case EPI_RELU:
      return (x != x) ? x : (x > 0.0f ? x : 0.0f);
    case EPI_GELU_ERF:
      return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
    case EPI_GELU_TANH: {
      const float c = 0.7978845608028654f;  // sqrt(2/pi)
      float x3 = x * x * x;
      return 0.5f * x * (1.0f + tanhf(c * (x + 0.044715f * x3)));
    }
    case EPI_RELU_BWD:
      return x * (aux > 0.0f ? 1.0f : 0.0f);
    default:
      return x;
  }
}

// Split-pair schedule: small-weight products first so they are accumulated
// before the dominant a0*b0 term.  Encoded as (i << 2 | j), i = A split, j = B split.
__device__ __forceinline__ int split_pairs(int mode, uint8_t (&pairs)[9]) {
  if (mode == 1) { pairs[0] = 0; return 1; }
  if (mode == 23) { pairs[0] = (0 << 2) | 1; pairs[1] = (1 << 2) | 0; pairs[2] = 0; return 3; }
  if (mode == 3) { pairs[0] = (0 << 2) | 1; pairs[1] = (1 << 2) | 0; pairs[2] = 0; return 3; }
  if (mode == 9) {
    pairs[0] = (2 << 2) | 2; pairs[1] = (1 << 2) | 2; pairs[2] = (2 << 2) | 1;
    pairs[3] = (0 << 2) | 2; pairs[4] = (2 << 2) | 0; pairs[5] = (1 << 2) | 1;
    pairs[6] = (0 << 2) | 1; pairs[7] = (1 << 2) | 0; pairs[8] = 0; return 9;
  }
  pairs[0] = (0 << 2) | 2; pairs[1] = (2 << 2) | 0; pairs[2] = (1 << 2) | 1;
  pairs[3] = (0 << 2) | 1; pairs[4] = (1 << 2) | 0; pairs[5] = 0; return 6;
}

template <int BN, int BK, int STAGES>
struct GemmCfg {
  static constexpr int BM = 128;
  static constexpr int ROW_BYTES = BK * 2;                 // bf16
  static constexpr int A_TILE = BM * ROW_BYTES;            // one split of A
  static constexpr int B_TILE = BN * ROW_BYTES;
  static constexpr int STAGE_BYTES = 3 * A_TILE + 3 * B_TILE;
  static constexpr int ACC_COLS = BN;                      // f32 columns per accumulator
  static constexpr int TMEM_COLS = 2 * BN;                 // two accumulators (power of two)
  static constexpr int NUM_THREADS = 192;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
  static_assert(ROW_BYTES == 64 || ROW_BYTES == 128, "BK must be 32 or 64");
  static_assert(BN % 32 == 0 && BN >= 32 && BN <= 256, "BN");
  static_assert(TMEM_COLS == 64 || TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512, "TMEM");
};

// Map a linear tile index to (batch, m tile, n tile).  Tiles are walked in
// bands of 8 M tiles with N fastest inside a band... the CTAs that run at the
// same time then share A row panels and B column panels through L2.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& b, int& tm, int& tn) {
  const int per_batch = tiles_m * tiles_n;
  b = t / per_batch;
  int r = t - b * per_batch;
  constexpr int BAND = 8;
  const int band_sz = BAND * tiles_n;
  const int band = r / band_sz;
  const int in_band = r - band * band_sz;
  const int rows_in_band = min(BAND, tiles_m - band * BAND);
  tm = band * BAND + in_band % rows_in_band;
  tn = in_band / rows_in_band;
}

template <int BN, int BK, int STAGES, bool CONV = false>
__global__ void __launch_bounds__(192, 1)
gemm_split_umma_kernel(const __grid_constant__ CUtensorMap tmapA,
                       const __grid_constant__ CUtensorMap tmapB, const GemmArgs g) {
  using Cfg = GemmCfg<BN, BK, STAGES>;
  constexpr int BM = Cfg::BM;
  extern __shared__ uint8_t smem_raw[];

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;           // 1024-byte aligned tile ring
  const uint32_t bars = tiles + STAGES * Cfg::STAGE_BYTES;  // barrier block (8-byte aligned)
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
  const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 4);
  const uint32_t abort_addr = tmem_slot + 4u;
  volatile uint32_t* abort_word =
      reinterpret_cast<volatile uint32_t*>(smem_raw + (abort_addr - raw));
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int n_tile = CONV ? g.cv_n_tile : BN;  // output columns per tile
  const int tiles_m = (g.M + BM - 1) / BM;
  const int tiles_n = (g.N + n_tile - 1) / n_tile;
  const int num_tiles = tiles_m * tiles_n * g.batch;
  const int nsplit = (g.mode == 1) ? 1 : (g.mode == 3 ? 2 : 3);
  const uint32_t stage_tx = nsplit * (Cfg::A_TILE + (CONV ? n_tile * Cfg::ROW_BYTES : Cfg::B_TILE));

  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 4);  // one arrival per epilogue warp
    }
    fence_mbar_init();
    prefetch_tmap(&tmapA);
    prefetch_tmap(&tmapB);
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int b, tm, tn;
        tile_coords(t, tiles_m, tiles_n, b, tm, tn);
        const int za = (g.a_batched ? b : 0) * g.planes_per_mat;
        const int zb = (g.b_batched ? b : 0) * g.planes_per_mat;
        const int kb0 = b * g.kb_batch_stride;
        for (int kb = 0; kb < g.num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_word)) {
            *abort_word = 1;
            atomicMax(g.status, 0x100u | 1u);
            ok = false;
            break;
          }
          mbar_expect_tx(full_bar(stage), stage_tx);
          const uint32_t sa = tiles + stage * Cfg::STAGE_BYTES;
          const uint32_t sb = sa + 3 * Cfg::A_TILE;
          for (int s = 0; s < nsplit; ++s)
            tma_load_3d(sa + s * Cfg::A_TILE, &tmapA, full_bar(stage), (kb0 + kb) * BK, tm * BM, za + s);
          if constexpr (CONV) {
            const int tap = kb / g.cv_kb_per_tap, cb = kb - tap * g.cv_kb_per_tap;
            const int fh = tap / g.cv_kw, fw = tap - fh * g.cv_kw;
            const int w = g.cv_w0 + g.cv_sgn * fw, hh = tn * g.cv_th + g.cv_h0 + g.cv_sgn * fh;
            for (int s = 0; s < nsplit; ++s)
              tma_load_4d(sb + s * Cfg::B_TILE, &tmapB, full_bar(stage), cb * BK, w, hh, zb + s);
          } else {
            for (int s = 0; s < nsplit; ++s)
              tma_load_3d(sb + s * Cfg::B_TILE, &tmapB, full_bar(stage), (kb0 + kb) * BK, tn * BN, zb + s);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint8_t pairs[9];
      const int npairs = split_pairs(g.mode, pairs);
      const uint32_t idesc = make_idesc(BM, CONV ? g.cv_umma_n : BN, /*bf16*/ 1u, /*f32*/ 1u);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, abort_word)) {
          *abort_word = 1;
          atomicMax(g.status, 0x200u | 1u);
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * Cfg::ACC_COLS;
        uint32_t accumulate = 0;
        for (int kb = 0; kb < g.num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_word)) {
            *abort_word = 1;
            atomicMax(g.status, 0x200u | 2u);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = tiles + stage * Cfg::STAGE_BYTES;
          const uint32_t sb = sa + 3 * Cfg::A_TILE;
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            for (int p = 0; p < npairs; ++p) {
              const int i = pairs[p] >> 2, j = pairs[p] & 3;
              const uint64_t da = make_kmajor_desc<Cfg::ROW_BYTES>(sa + i * Cfg::A_TILE + kk * 32);
              const uint64_t db = make_kmajor_desc<Cfg::ROW_BYTES>(sb + j * Cfg::B_TILE + kk * 32);
              umma_f16<1>(d_tmem, da, db, idesc, accumulate);
              accumulate = 1;
            }
          }
          umma_commit<1>(empty_bar(stage));  // stage reusable once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit<1>(acc_full_bar(acc));  // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(g.C) & 15) == 0) && ((g.ldc & 3) == 0) &&
                        ((g.strideC & 3) == 0);
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int b, tm, tn;
      tile_coords(t, tiles_m, tiles_n, b, tm, tn);
      if (!mbar_wait(acc_full_bar(acc), acc_phase, abort_word)) {
        *abort_word = 1;
        if (lane == 0) atomicMax(g.status, 0x300u | 1u);
        break;
      }
      tc_fence_after();
      const int row = tm * BM + q * 32 + lane;
      const bool row_ok = row < g.M;
      float* crow = g.C + b * g.strideC + static_cast<long long>(row) * g.ldc;
      const float* arow =
          g.aux ? g.aux + b * g.strideC + static_cast<long long>(row) * g.ldc : nullptr;
      const float row_bias = (g.bias && g.bias_per_row && row_ok) ? __ldg(g.bias + row) : 0.0f;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * Cfg::ACC_COLS;
#pragma unroll 1
      for (int c0 = 0; c0 < n_tile; c0 += 32) {
        const int col0 = tn * n_tile + c0;
        if (col0 >= g.N) break;  // uniform across the warp
        const int col_end = min(g.N, (tn + 1) * n_tile);  // a conv tile may end inside a 32-column group
        uint32_t v[32];
        tmem_ld_32x32(t_row + c0, v);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const int col = col0 + j;
            if (col >= col_end) break;
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float x = __uint_as_float(v[j + e]);
              if (col + e < col_end) {
                if (g.bias) x += g.bias_per_row ? row_bias : __ldg(g.bias + col + e);
                const float ax = (g.epilogue == EPI_RELU_BWD) ? arow[col + e] : 0.0f;
                x = apply_epilogue(x, g.epilogue, ax);
              }
              o[e] = x;
            }
            if (vec_ok && col + 3 < col_end && ((col & 3) == 0)) {
              *reinterpret_cast<float4*>(crow + col) = make_float4(o[0], o[1], o[2], o[3]);
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (col + e < col_end) crow[col + e] = o[e];
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(acc));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    // A wait ran out: give loads and MMAs still in flight time to land before
    // shared memory and TMEM are handed back.
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace mtb
