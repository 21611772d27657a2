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
#include <climits>
#include <type_traits>
#include "ptx_sm100.cuh"
#include "split_bf16.cuh"
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
  int exp_b_per_batch; // 1: exp_b holds ONE exponent per batch entry ([batch]) that serves all its columns
  int a_batched;       // 0: one A shared by all batch entries
  int b_batched;
  int bias_per_row;    // 0: bias[N] added along columns; 1: bias[M] added along rows
  int kb_batch_stride; // split-K: batch entry b reduces K blocks [b*stride, b*stride + num_kb)
  uint32_t* status;    // device word; a non-zero value reports a wait that ran out
  // Tail splitting (pair-tile kernel): when the tile count leaves a partial last round, each of its tiles may be
  // cut into tail_splits K ranges that are dealt out over the SM pairs like (shorter) tiles; the raw partial
  // accumulators go to `partial` ([tail tile][split][256][256] f32) and a second kernel adds them in a fixed order
  // and applies the epilogue.  tail_splits <= 1: off.
  // Optional gate (the int8 use of the pair-tile kernel): the kernel returns at once unless
  // (*gate == gate_value) == (gate_run_if_equal != 0).  gate == nullptr: always run.
  const uint32_t* gate;
  uint32_t gate_value;
  int gate_run_if_equal;
  int raw_int;         // 1: the accumulators are s32 (int8 product): partial tiles are added as integers
  int tail_splits;
  int tail_rounds;     // full rounds before the tail: tiles [0, tail_rounds * pairs) are whole
  int tail_tiles;      // tiles in the tail round
  float* partial;
  // Implicit-convolution mode (CONV kernels only): the B operand is read straight
  // from channels-last image planes {c, w, h, image*planes+split}; a K block is one
  // (filter tap, channel block) and an N tile is cv_th full image rows.
  int cv_n_tile;       // columns per N tile = cv_th * tile width
  int cv_umma_n;       // MMA N: cv_n_tile rounded up to a multiple of 16
  int cv_th;           // image rows per N tile
  int cv_kb_per_tap;   // channel blocks per filter tap
  int cv_kw;           // filter width (taps per filter row)
  int cv_w0, cv_h0;    // window origin for tap (0,0): -pad (forward) or +pad (data gradient)
  int cv_sgn;          // +1 forward (origin + tap), -1 data gradient (origin - tap)
};

// Compile-time form: the runtime switch below is if-converted by the compiler into "compute every
// branch, then select", which costs an erff and a tanhf per output element whatever the epilogue.
template <int EPI>
__device__ __forceinline__ float apply_epilogue_t(float x, float aux) {
  if constexpr (EPI == EPI_RELU) return (x != x) ? x : (x > 0.0f ? x : 0.0f);
  else if constexpr (EPI == EPI_GELU_ERF) return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
  else if constexpr (EPI == EPI_GELU_TANH) {
    const float c = 0.7978845608028654f;  // sqrt(2/pi)
    const float x3 = x * x * x;
    return 0.5f * x * (1.0f + tanhf(c * (x + 0.044715f * x3)));
  } else if constexpr (EPI == EPI_RELU_BWD) return x * (aux > 0.0f ? 1.0f : 0.0f);
  else return x;
}

// Split-pair schedule: small-weight products first so they are accumulated before the dominant a0*b0 term.
// Encoded as (i << 2 | j), i = A split, j = B split, as a compile-time function of (number of products,
// position), for issue loops that are unrolled completely: the issuing thread then spends one add per
// descriptor instead of a table lookup and a descriptor build per product.  3 products serve both two-plane modes.
__host__ __device__ constexpr int split_pair_at(int npairs, int p) {
  if (npairs == 1) return 0;
  if (npairs == 3) return p == 0 ? ((0 << 2) | 1) : (p == 1 ? ((1 << 2) | 0) : 0);
  if (npairs == 9) {
    switch (p) {
      case 0: return (2 << 2) | 2;
      case 1: return (1 << 2) | 2;
      case 2: return (2 << 2) | 1;
      case 3: return (0 << 2) | 2;
      case 4: return (2 << 2) | 0;
      case 5: return (1 << 2) | 1;
      case 6: return (0 << 2) | 1;
      case 7: return (1 << 2) | 0;
      default: return 0;
    }
  }
  switch (p) {
    case 0: return (0 << 2) | 2;
    case 1: return (2 << 2) | 0;
    case 2: return (1 << 2) | 1;
    case 3: return (0 << 2) | 1;
    case 4: return (1 << 2) | 0;
    default: return 0;
  }
}
__host__ __device__ constexpr int split_pair_count(int mode) {
  return mode == 1 ? 1 : ((mode == 3 || mode == 23) ? 3 : (mode == 9 ? 9 : 6));
}

// Epilogue of one warp for one accumulator: 32 rows (one per lane in tensor memory) x `ncols`
// columns.  tcgen05.ld hands every lane CW consecutive columns of ITS row, which written to
// global memory directly would make each store instruction touch 32 different rows (32 partial
// lines).  The values therefore go through a small shared-memory tile [32][CW + 1] and come back
// with 32 / (CW / 4) rows per instruction, each row segment a contiguous run of float4 stores.
// Scale (fp16 mode), bias, activation and ReLU mask are applied on the way out.
//   stage      : this warp's [32][CW + 1] floats of shared memory
//   t_row      : TMEM address of (first lane of this warp, first column of the accumulator)
//   row0       : global row of lane 0;  col_base / col_end: global column range of the tile
// EPI and SCALED are compile-time so that only the work an output needs is generated.
template <int CW, int EPI, bool SCALED>
__device__ __forceinline__ void epilogue_warp_tile_t(const GemmArgs& g, float* stage, uint32_t t_row, int b, int row0,
                                                  int col_base, int col_end, int lane, bool vec_ok) {
  constexpr int LPR = CW / 4;        // lanes per row when reading back
  constexpr int RPI = 32 / LPR;      // rows per store instruction
  constexpr int PITCH = CW + 1;
  const int my_row = row0 + lane;
  const bool my_row_ok = my_row < g.M;
  const float row_bias_own = (g.bias && g.bias_per_row && my_row_ok) ? __ldg(g.bias + my_row) : 0.0f;
  const int* eb = SCALED ? g.exp_b + (g.exp_b_per_batch ? static_cast<long long>(b)
                                                           : (g.b_batched ? static_cast<long long>(b) * g.N : 0))
                          : nullptr;
  const int eb_all = (SCALED && g.exp_b_per_batch) ? __ldg(eb) : 0;
  const int ea_own =
      (SCALED && my_row_ok) ? __ldg(g.exp_a + (g.a_batched ? static_cast<long long>(b) * g.M : 0) + my_row) : 0;
  float* cbase = g.C + b * g.strideC;
  const float* abase = g.aux ? g.aux + b * g.strideC : nullptr;
  const int cq = (lane % LPR) * 4, rsub = lane / LPR;
  int ea_span = SCALED ? abs(ea_own) : 0;      // largest |row exponent| of this warp's 32 rows
  if constexpr (SCALED) {
#pragma unroll
    for (int o2 = 16; o2; o2 >>= 1) ea_span = max(ea_span, __shfl_xor_sync(0xffffffffu, ea_span, o2));
  }
#pragma unroll 1
  for (int c0 = col_base; c0 < col_end; c0 += CW) {
    // the column group's bias and exponents first: their latency hides behind the TMEM read and the staging
    const int col = c0 + cq;
    float cb[4];
    int ce[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const bool ok = col + e < col_end;
      cb[e] = (g.bias && !g.bias_per_row && ok) ? __ldg(g.bias + col + e) : 0.0f;
      ce[e] = (SCALED && ok) ? (g.exp_b_per_batch ? eb_all : __ldg(eb + col + e)) : 0;
    }
    uint32_t v[CW];
    if constexpr (CW == 32) tmem_ld_32x32(t_row + (c0 - col_base), v);
    else tmem_ld_32x16(t_row + (c0 - col_base), v);
    bool fast = false;
    if constexpr (SCALED) {
      int ce_span = max(max(abs(ce[0]), abs(ce[1])), max(abs(ce[2]), abs(ce[3])));
#pragma unroll
      for (int o2 = 16; o2; o2 >>= 1) ce_span = max(ce_span, __shfl_xor_sync(0xffffffffu, ce_span, o2));
      fast = ea_span + ce_span <= 126;
    }
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < CW; ++j) stage[lane * PITCH + j] = __uint_as_float(v[j]);
    __syncwarp();
#pragma unroll
    for (int it = 0; it < LPR; ++it) {
      const int r = it * RPI + rsub;
      const int ea_r = __shfl_sync(0xffffffffu, ea_own, r);
      const float rb = __shfl_sync(0xffffffffu, row_bias_own, r);
      const int grow = row0 + r;
      if (grow < g.M && col < col_end) {
        float* cptr = cbase + static_cast<long long>(grow) * g.ldc + col;
        const bool full = vec_ok && col + 3 < col_end && ((col & 3) == 0);
        float ax[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if constexpr (EPI == EPI_RELU_BWD) {
          const float* aptr = abase + static_cast<long long>(grow) * g.ldc + col;
          if (full) {
            const float4 a4 = *reinterpret_cast<const float4*>(aptr);
            ax[0] = a4.x; ax[1] = a4.y; ax[2] = a4.z; ax[3] = a4.w;
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (col + e < col_end) ax[e] = aptr[e];
          }
        }
        float o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float x = stage[r * PITCH + cq + e];
          if constexpr (SCALED) {
            // fast: every exponent sum of this warp's rows and columns is a normal float's exponent
            if (fast) x *= __int_as_float((ea_r + ce[e] + 127) << 23);
            else x = scale_pow2(x, ea_r + ce[e]);
          }
          if (g.bias) x += g.bias_per_row ? rb : cb[e];
          o[e] = apply_epilogue_t<EPI>(x, ax[e]);
        }
        if (full) {
          *reinterpret_cast<float4*>(cptr) = make_float4(o[0], o[1], o[2], o[3]);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (col + e < col_end) cptr[e] = o[e];
        }
      }
    }
    __syncwarp();  // the tile is rewritten by the next column group
  }
}

// What an epilogue warp reads besides its accumulator - scale exponents of its rows and of the tile's columns, the
// bias - does not depend on the MMAs: asking for those cache lines before the wait on the accumulator takes their
// latency out of the tail of a tile (an output of one tile per CTA has nothing else to hide it behind).
__device__ __forceinline__ void epilogue_prefetch(const GemmArgs& g, int b, int row0, int col_base, int col_end, int lane) {
  auto touch = [](const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); };
  const int c = col_base + lane * 32;          // one 128-byte line of 4-byte entries per lane
  if (g.exp_b) {
    if (lane == 0 && row0 < g.M) touch(g.exp_a + (g.a_batched ? static_cast<long long>(b) * g.M : 0) + row0);
    if (g.exp_b_per_batch) { if (lane == 0) touch(g.exp_b + b); }
    else if (c < col_end) touch(g.exp_b + (g.b_batched ? static_cast<long long>(b) * g.N : 0) + c);
  }
  if (g.bias) {
    if (g.bias_per_row) { if (lane == 0 && row0 < g.M) touch(g.bias + row0); }
    else if (c < col_end) touch(g.bias + c);
  }
}

template <int CW>
__device__ __forceinline__ void epilogue_warp_tile(const GemmArgs& g, float* stage, uint32_t t_row, int b, int row0,
                                                   int col_base, int col_end, int lane, bool vec_ok) {
#define MTB_EPI_CASE(E)                                                                                         \
  case E:                                                                                                       \
    if (g.exp_b) epilogue_warp_tile_t<CW, E, true>(g, stage, t_row, b, row0, col_base, col_end, lane, vec_ok);  \
    else epilogue_warp_tile_t<CW, E, false>(g, stage, t_row, b, row0, col_base, col_end, lane, vec_ok);         \
    break;
  switch (g.epilogue) {
    MTB_EPI_CASE(EPI_RELU)
    MTB_EPI_CASE(EPI_GELU_ERF)
    MTB_EPI_CASE(EPI_GELU_TANH)
    MTB_EPI_CASE(EPI_RELU_BWD)
    default:
      if (g.exp_b) epilogue_warp_tile_t<CW, EPI_NONE, true>(g, stage, t_row, b, row0, col_base, col_end, lane, vec_ok);
      else epilogue_warp_tile_t<CW, EPI_NONE, false>(g, stage, t_row, b, row0, col_base, col_end, lane, vec_ok);
  }
#undef MTB_EPI_CASE
}

// PLANES = planes per operand a stage has room for: 3 (bf16 modes) or 2 (the fp16 two-plane mode only).
template <int BN, int BK, int STAGES, int PLANES = 3>
struct GemmCfg {
  static constexpr int BM = 128;
  static constexpr int ROW_BYTES = BK * 2;                 // bf16
  static constexpr int A_TILE = BM * ROW_BYTES;            // one split of A
  static constexpr int B_TILE = BN * ROW_BYTES;
  static constexpr int STAGE_BYTES = PLANES * A_TILE + PLANES * B_TILE;
  static constexpr int ACC_COLS = BN;                      // f32 columns per accumulator
  static constexpr int TMEM_COLS = 2 * BN;                 // two accumulators (power of two)
  // epilogue staging: one [32][CW + 1] float tile per epilogue warp; 16-column groups where the ring leaves less
  // room.  Eight epilogue warps (two per TMEM lane quarter, half of the tile's columns each) where their staging
  // fits: an output of one tile per CTA has nothing to overlap the epilogue with, so its latency counts.
  static constexpr int EPI_WARPS = (STAGES * STAGE_BYTES + 1024 + 256 + 8 * 32 * 33 * 4 <= 232448 && BN % 64 == 0) ? 8 : 4;
  static constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int EPI_CW = (STAGES * STAGE_BYTES + 1024 + 256 + 4 * 32 * 33 * 4 <= 232448) ? 32 : 16;
  static constexpr int EPI_BYTES = EPI_WARPS * 32 * (EPI_CW + 1) * 4;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + EPI_BYTES;
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

// A_MN / B_MN: that operand's planes are MN-major ([k][mn] row-major in global memory, loaded as chunks of 64 mn
// elements x BK k rows; needs BK = 64), as the two-CTA kernel takes them (gemm_split_umma2.cuh).
template <int BN, int BK, int STAGES, bool CONV = false, int PLANES = 3, bool A_MN = false, bool B_MN = false>
__global__ void __launch_bounds__(GemmCfg<BN, BK, STAGES, PLANES>::NUM_THREADS, 1)
gemm_split_umma_kernel(const __grid_constant__ CUtensorMap tmapA,
                       const __grid_constant__ CUtensorMap tmapB, const GemmArgs g) {
  using Cfg = GemmCfg<BN, BK, STAGES, PLANES>;
  constexpr int BM = Cfg::BM;
  static_assert(!(A_MN || B_MN) || (BK == 64 && !CONV), "MN-major operands need BK = 64 and the plain GEMM");
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
  const int nsplit = (g.mode == 1) ? 1 : ((g.mode == 3 || g.mode == 23) ? 2 : 3);
  const uint32_t stage_tx = nsplit * (Cfg::A_TILE + (CONV ? n_tile * Cfg::ROW_BYTES : Cfg::B_TILE));

  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), Cfg::EPI_WARPS);  // one arrival per epilogue warp
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
  grid_dependency_wait();        // the operand planes and exponents come from the kernels before this one
  grid_launch_dependents();

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
          const uint32_t sb = sa + PLANES * Cfg::A_TILE;
          for (int s = 0; s < nsplit; ++s) {
            if constexpr (A_MN)
              tma_load_4d(sa + s * Cfg::A_TILE, &tmapA, full_bar(stage), 0, (kb0 + kb) * BK, (tm * BM) >> 6, za + s);
            else
              tma_load_3d(sa + s * Cfg::A_TILE, &tmapA, full_bar(stage), (kb0 + kb) * BK, tm * BM, za + s);
          }
          if constexpr (CONV) {
            const int tap = kb / g.cv_kb_per_tap, cb = kb - tap * g.cv_kb_per_tap;
            const int fh = tap / g.cv_kw, fw = tap - fh * g.cv_kw;
            const int w = g.cv_w0 + g.cv_sgn * fw, hh = tn * g.cv_th + g.cv_h0 + g.cv_sgn * fh;
            for (int s = 0; s < nsplit; ++s)
              tma_load_4d(sb + s * Cfg::B_TILE, &tmapB, full_bar(stage), cb * BK, w, hh, zb + s);
          } else {
            for (int s = 0; s < nsplit; ++s) {
              if constexpr (B_MN)
                tma_load_4d(sb + s * Cfg::B_TILE, &tmapB, full_bar(stage), 0, (kb0 + kb) * BK, (tn * BN) >> 6, zb + s);
              else
                tma_load_3d(sb + s * Cfg::B_TILE, &tmapB, full_bar(stage), (kb0 + kb) * BK, tn * BN, zb + s);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // operand format: bf16 planes, or fp16 planes in the two-plane mode 23
      const uint32_t idesc = make_idesc(BM, CONV ? g.cv_umma_n : BN, g.mode == 23 ? 0u : 1u, /*f32*/ 1u,
                                        A_MN ? 1u : 0u, B_MN ? 1u : 0u);
      // The whole issue loop with the product schedule known at compile time: per product the
      // thread adds a constant to each operand's descriptor and issues the MMA.
      auto issue_all = [&](auto npairs_tag) {
        constexpr int NPAIRS = decltype(npairs_tag)::value;
        // one MMA covers 16 k: 32 bytes along a K-major row, 16 rows of 128 bytes in an MN-major chunk
        constexpr uint32_t A_KSTEP = A_MN ? 2048u : 32u, B_KSTEP = B_MN ? 2048u : 32u;
        int stage = 0, acc = 0;
        uint32_t phase = 0, acc_phase = 0;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
          if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, abort_word)) {
            *abort_word = 1;
            atomicMax(g.status, 0x200u | 1u);
            return;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * Cfg::ACC_COLS;
          uint32_t accumulate = 0;
          for (int kb = 0; kb < g.num_kb; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, abort_word)) {
              *abort_word = 1;
              atomicMax(g.status, 0x200u | 2u);
              return;
            }
            tc_fence_after();
            const uint32_t sa = tiles + stage * Cfg::STAGE_BYTES;
            const uint32_t sb = sa + PLANES * Cfg::A_TILE;
            // descriptors of plane 0, k = 0; the start address sits in the low 14 bits in units of
            // 16 bytes and shared memory ends below 2^18, so adding an offset never carries out
            const uint64_t da0 = A_MN ? make_mnmajor_desc(sa, BK * 128) : make_kmajor_desc<Cfg::ROW_BYTES>(sa);
            const uint64_t db0 = B_MN ? make_mnmajor_desc(sb, BK * 128) : make_kmajor_desc<Cfg::ROW_BYTES>(sb);
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) {
#pragma unroll
              for (int p = 0; p < NPAIRS; ++p) {
                const int code = split_pair_at(NPAIRS, p);
                const uint32_t offa = (code >> 2) * Cfg::A_TILE + kk * A_KSTEP;
                const uint32_t offb = (code & 3) * Cfg::B_TILE + kk * B_KSTEP;
                umma_f16<1>(d_tmem, da0 + (offa >> 4), db0 + (offb >> 4), idesc, accumulate);
                accumulate = 1;
              }
            }
            umma_commit<1>(empty_bar(stage));  // stage reusable once these MMAs have read it
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
          umma_commit<1>(acc_full_bar(acc));  // accumulator complete
          if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
      };
      if constexpr (PLANES == 2) {
        issue_all(std::integral_constant<int, 3>{});   // only the two-plane modes fit this layout
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
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    // with eight epilogue warps the second warp of a quarter takes the upper half of the tile's columns
    const int half_cols = (Cfg::EPI_WARPS == 8) ? ((warp - 2) >> 2) * (BN / 2) : 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(g.C) & 15) == 0) && ((g.ldc & 3) == 0) &&
                        ((g.strideC & 3) == 0);
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int b, tm, tn;
      tile_coords(t, tiles_m, tiles_n, b, tm, tn);
      const int col_first = tn * n_tile + half_cols;
      const int col_last = min(min(g.N, (tn + 1) * n_tile), (Cfg::EPI_WARPS == 8) ? col_first + BN / 2 : INT_MAX);
      epilogue_prefetch(g, b, tm * BM + q * 32, col_first, col_last, lane);
      if (!mbar_wait(acc_full_bar(acc), acc_phase, abort_word)) {
        *abort_word = 1;
        if (lane == 0) atomicMax(g.status, 0x300u | 1u);
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * Cfg::ACC_COLS + half_cols;
      float* stage = reinterpret_cast<float*>(smem_raw + (bars + 256u - raw)) + (warp - 2) * 32 * (Cfg::EPI_CW + 1);
      epilogue_warp_tile<Cfg::EPI_CW>(g, stage, t_row, b, tm * BM + q * 32, col_first, col_last, lane, vec_ok);
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
