// Exact (wrapping) int32 GEMM on the tcgen05 integer tensor cores.
//
// The reference multiplies integers with the scalar loop `sum = sum + a*b`
// (engine/src/operations/linalg/diagonal.rs:495-548), i.e. arithmetic modulo 2^32
// in release builds.  Modulo 2^32 every int32 is the sum of four unsigned byte
// limbs a = a0 + a1*2^8 + a2*2^16 + a3*2^24, and
//     a*b = sum over i+j <= 3 of a_i*b_j * 2^(8(i+j))      (mod 2^32),
// the other limb products being multiples of 2^32.  That is ten u8 x u8 -> s32
// tensor-core products, accumulated by weight class c = i+j in four TMEM
// accumulators S_c; the epilogue forms C = S0 + (S1<<8) + (S2<<16) + (S3<<24)
// in wrapping 32-bit arithmetic.  A K chunk is at most 8192 long so no
// accumulator can overflow (4 products * 255^2 * 8192 < 2^31); longer reductions
// are chained by adding into C.  The result is bit-identical to the scalar loop.
//
// When both operands fit in int8 (the split kernels record that per call) the
// low limb IS the value as a signed byte and one s8 x s8 product suffices: the
// kernel reads the device-side flag and issues one MMA per K step instead of ten.
//
// Tile 128 x 128, K block 64 bytes (64-byte swizzle), 3-stage TMA ring, one CTA
// per SM, persistent.  The four accumulators fill tensor memory (4 x 128
// columns), so the epilogue of a tile is not overlapped with the next main loop.
#pragma once
#include "ptx_sm100.cuh"

namespace mtb {

struct I32LimbArgs {
  int M, N, batch;
  int num_kb;             // K blocks of 64 in this launch
  int kb0;                // first K block (reductions longer than 8192 are launched in chunks)
  int accumulate;         // 1: add into C (a later K chunk)
  uint32_t* C;            // [batch][M][N]
  long long strideC;
  int a_batched, b_batched;
  const uint32_t* wide_word;  // device word: == wide_epoch when some element does not fit in int8
  uint32_t wide_epoch;
  int skip_narrow;        // 1: return at once when the operands fit in int8 (another kernel takes that case)
  uint32_t* status;
};

struct I32LimbCfg {
  static constexpr int BM = 128, BN = 128, BKB = 64, STAGES = 3;
  static constexpr int TILE = 128 * BKB;                  // one limb plane of one operand tile
  static constexpr int STAGE_BYTES = 8 * TILE;            // 4 limbs of A + 4 limbs of B
  static constexpr int TMEM_COLS = 512;
  static constexpr int NUM_THREADS = 192;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

// bytes -> planes: dst[(b*4 + l)][r][k] = limb l of src element (r, k); K padded with zeros to Kp.
// The source is row-major [R][K] (trans = 0, ld = K) or [K][R] (trans = 1, ld = R), 64 x 64 tiles.
static __global__ void __launch_bounds__(256)
limb_split_kernel(const int32_t* __restrict__ src, long long ld, long long bstride, int trans,
                  uint8_t* __restrict__ dst, int R, int K, int Kp, uint32_t* __restrict__ wide_word,
                  uint32_t wide_epoch) {
  __shared__ int32_t tile[64][65];
  const int b = blockIdx.z;
  const int r0 = blockIdx.x * 64, k0 = blockIdx.y * 64;
  const int32_t* s = src + b * bstride;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  bool wide = false;
  for (int j = ty; j < 64; j += 4) {
    int32_t v = 0;
    if (!trans) {                 // tile[r][k], reads run along k
      const int r = r0 + j, k = k0 + tx;
      if (r < R && k < K) v = s[static_cast<long long>(r) * ld + k];
      tile[j][tx] = v;
    } else {                      // source [k][r]: reads run along r, stored transposed
      const int k = k0 + j, r = r0 + tx;
      if (r < R && k < K) v = s[static_cast<long long>(k) * ld + r];
      tile[tx][j] = v;
    }
    wide |= (v < -128 || v > 127);
  }
  if (wide) atomicMax(wide_word, wide_epoch);
  __syncthreads();
  // 64 rows x 4 limbs x 4 chunks of 16 bytes = 1024 stores of 16 bytes, 4 per thread
  const long long plane = static_cast<long long>(R) * Kp;
  for (int it = threadIdx.x; it < 1024; it += 256) {
    const int rr = it >> 4, l = (it >> 2) & 3, ch = it & 3;
    const int r = r0 + rr;
    if (r >= R || k0 + ch * 16 >= Kp) continue;
    __align__(16) uint8_t o[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) o[e] = static_cast<uint8_t>(static_cast<uint32_t>(tile[rr][ch * 16 + e]) >> (8 * l));
    uint8_t* d = dst + (static_cast<long long>(b) * 4 + l) * plane + static_cast<long long>(r) * Kp + k0 + ch * 16;
    *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(o);
  }
}

// The turned case (source [K][R], ld = R) with the bytes packed before they cross shared memory: a block takes
// 128 k x 32 r; a thread loads 16 consecutive k of one r (every load of a warp is 128 contiguous bytes along r),
// packs each group of four k into one word per limb and stores those words at tile[l][r][k / 4] (row pitch 33
// words: lanes of one warp differ in r, so the stores hit 32 banks).  The second phase reads four consecutive
// words (16 bytes of one limb plane row) per thread - lanes (r = lane / 8, chunk = lane % 8) again cover all
// banks - and a warp's store is four rows of 128 contiguous bytes.
static __global__ void __launch_bounds__(256)
limb_split_turn_kernel(const int32_t* __restrict__ src, long long ld, long long bstride, uint8_t* __restrict__ dst,
                       int R, int K, int Kp, uint32_t* __restrict__ wide_word, uint32_t wide_epoch) {
  __shared__ uint32_t tile[4][32][33];
  const int b = blockIdx.z;
  const int r0 = blockIdx.x * 32, k0 = blockIdx.y * 128;
  const int32_t* s = src + b * bstride;
  const int lane = threadIdx.x & 31, kg = threadIdx.x >> 5;     // kg: which 16 of the 128 k
  const int r = r0 + lane;
  int32_t v[16];
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    const int k = k0 + kg * 16 + e;
    v[e] = (r < R && k < K) ? s[static_cast<long long>(k) * ld + r] : 0;
  }
  bool wide = false;
#pragma unroll
  for (int e = 0; e < 16; ++e) wide |= (v[e] < -128 || v[e] > 127);
  if (wide) atomicMax(wide_word, wide_epoch);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint32_t a0 = uint32_t(v[q * 4]), a1 = uint32_t(v[q * 4 + 1]), a2 = uint32_t(v[q * 4 + 2]), a3 = uint32_t(v[q * 4 + 3]);
    // limb l of four elements in one word: byte permutes of the pairs (a0,a1) and (a2,a3), then of the halves
    const uint32_t lo01 = __byte_perm(a0, a1, 0x5140), hi01 = __byte_perm(a0, a1, 0x7362);   // [a0.b0 a1.b0 a0.b1 a1.b1], [a0.b2 a1.b2 a0.b3 a1.b3]
    const uint32_t lo23 = __byte_perm(a2, a3, 0x5140), hi23 = __byte_perm(a2, a3, 0x7362);
    tile[0][lane][kg * 4 + q] = __byte_perm(lo01, lo23, 0x5410);
    tile[1][lane][kg * 4 + q] = __byte_perm(lo01, lo23, 0x7632);
    tile[2][lane][kg * 4 + q] = __byte_perm(hi01, hi23, 0x5410);
    tile[3][lane][kg * 4 + q] = __byte_perm(hi01, hi23, 0x7632);
  }
  __syncthreads();
  const long long plane = static_cast<long long>(R) * Kp;
  const int rr = (threadIdx.x >> 3) & 31, c = threadIdx.x & 7;
  if (r0 + rr < R && k0 + c * 16 < Kp) {
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const uint32_t* t = &tile[l][rr][c * 4];
      uint8_t* d = dst + (static_cast<long long>(b) * 4 + l) * plane + static_cast<long long>(r0 + rr) * Kp + k0 + c * 16;
      *reinterpret_cast<uint4*>(d) = make_uint4(t[0], t[1], t[2], t[3]);
    }
  }
}

// The untransposed case without shared memory: a thread takes 16 consecutive k of one row (four 16-byte loads)
// and writes 16 bytes to each of the four limb planes, so a warp reads 2 KB and writes 4 x 512 B contiguously.
// Needs K % 4 == 0 and 16-byte aligned rows (ld % 4 == 0).
static __global__ void __launch_bounds__(256)
limb_split_rows_kernel(const int32_t* __restrict__ src, long long ld, long long bstride, uint8_t* __restrict__ dst,
                       int R, int K, int Kp, uint32_t* __restrict__ wide_word, uint32_t wide_epoch) {
  const int b = blockIdx.z;
  const int chunks = Kp >> 4;
  const long long total = static_cast<long long>(R) * chunks;
  const long long plane = static_cast<long long>(R) * Kp;
  const int32_t* s = src + b * bstride;
  bool wide = false;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / chunks);
    const int k0 = static_cast<int>(i - static_cast<long long>(r) * chunks) << 4;
    uint32_t v[16];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      int4 t = make_int4(0, 0, 0, 0);
      if (k0 + q * 4 < K) t = *reinterpret_cast<const int4*>(s + static_cast<long long>(r) * ld + k0 + q * 4);
      v[q * 4 + 0] = uint32_t(t.x); v[q * 4 + 1] = uint32_t(t.y); v[q * 4 + 2] = uint32_t(t.z); v[q * 4 + 3] = uint32_t(t.w);
      wide |= (t.x < -128 || t.x > 127) | (t.y < -128 || t.y > 127) | (t.z < -128 || t.z > 127) | (t.w < -128 || t.w > 127);
    }
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      uint32_t w[4];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        w[q] = ((v[q * 4 + 0] >> (8 * l)) & 0xffu) | (((v[q * 4 + 1] >> (8 * l)) & 0xffu) << 8) |
               (((v[q * 4 + 2] >> (8 * l)) & 0xffu) << 16) | (((v[q * 4 + 3] >> (8 * l)) & 0xffu) << 24);
      uint8_t* d = dst + (static_cast<long long>(b) * 4 + l) * plane + static_cast<long long>(r) * Kp + k0;
      *reinterpret_cast<uint4*>(d) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  if (wide) atomicMax(wide_word, wide_epoch);
}

__global__ void __launch_bounds__(192, 1)
gemm_i32_limb_umma_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
                          const I32LimbArgs g) {
  using Cfg = I32LimbCfg;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  const uint32_t bars = tiles + Cfg::STAGES * Cfg::STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (Cfg::STAGES + s); };
  const uint32_t acc_full = bars + 8u * (2 * Cfg::STAGES);
  const uint32_t acc_empty = bars + 8u * (2 * Cfg::STAGES + 1);
  const uint32_t tmem_slot = bars + 8u * (2 * Cfg::STAGES + 2);
  const uint32_t abort_addr = tmem_slot + 4u;
  volatile uint32_t* abort_word = reinterpret_cast<volatile uint32_t*>(smem_raw + (abort_addr - raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (g.M + Cfg::BM - 1) / Cfg::BM, tiles_n = (g.N + Cfg::BN - 1) / Cfg::BN;
  const int num_tiles = tiles_m * tiles_n * g.batch;
  const bool narrow = (*g.wide_word != g.wide_epoch);  // every element of both operands fits in int8
  if (narrow && g.skip_narrow) return;
  const int nlimb = narrow ? 1 : 4;
  const uint32_t stage_tx = 2u * nlimb * Cfg::TILE;

  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 4);
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
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int per = tiles_m * tiles_n;
        const int b = t / per, r = t - b * per;
        const int tm = r / tiles_n, tn = r - tm * tiles_n;
        const int za = (g.a_batched ? b : 0) * 4, zb = (g.b_batched ? b : 0) * 4;
        for (int kb = 0; kb < g.num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_word)) {
            *abort_word = 1;
            atomicMax(g.status, 0x100u | 7u);
            ok = false;
            break;
          }
          mbar_expect_tx(full_bar(stage), stage_tx);
          const uint32_t sa = tiles + stage * Cfg::STAGE_BYTES, sb = sa + 4 * Cfg::TILE;
          for (int l = 0; l < nlimb; ++l) {
            tma_load_3d(sa + l * Cfg::TILE, &tmapA, full_bar(stage), (g.kb0 + kb) * Cfg::BKB, tm * Cfg::BM, za + l);
            tma_load_3d(sb + l * Cfg::TILE, &tmapB, full_bar(stage), (g.kb0 + kb) * Cfg::BKB, tn * Cfg::BN, zb + l);
          }
          if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // kind::i8, s32 accumulate (c format 2); operand format 0 = unsigned, 1 = signed bytes
      const uint32_t idesc = make_idesc(Cfg::BM, Cfg::BN, narrow ? 1u : 0u, 2u);
      // issue loop with the limb count known at compile time: one add per descriptor per product
      auto issue_all = [&](auto nlimb_tag) {
        constexpr int NLIMB = decltype(nlimb_tag)::value;
        int stage = 0;
        uint32_t phase = 0, tile_phase = 0;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
          if (!mbar_wait(acc_empty, tile_phase ^ 1u, abort_word)) {
            *abort_word = 1;
            atomicMax(g.status, 0x200u | 7u);
            return;
          }
          tc_fence_after();
          uint32_t first = 0;  // 0 for the tile's first K block: every accumulator starts from zero there
          for (int kb = 0; kb < g.num_kb; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, abort_word)) {
              *abort_word = 1;
              atomicMax(g.status, 0x200u | 8u);
              return;
            }
            tc_fence_after();
            const uint32_t sa = tiles + stage * Cfg::STAGE_BYTES, sb = sa + 4 * Cfg::TILE;
            const uint64_t da0 = make_kmajor_desc<Cfg::BKB>(sa), db0 = make_kmajor_desc<Cfg::BKB>(sb);
#pragma unroll
            for (int kk = 0; kk < Cfg::BKB / 32; ++kk) {
#pragma unroll
              for (int i = 0; i < NLIMB; ++i)
#pragma unroll
                for (int j = 0; i + j < NLIMB; ++j) {
                  const int c = i + j;
                  // accumulator c is first written by (kk = 0, i = 0, j = c)
                  const uint32_t accumulate = (kk == 0 && i == 0) ? first : 1u;
                  umma_i8<1>(tmem_base + c * Cfg::BN, da0 + ((i * Cfg::TILE + kk * 32) >> 4),
                             db0 + ((j * Cfg::TILE + kk * 32) >> 4), idesc, accumulate);
                }
            }
            first = 1u;
            umma_commit<1>(empty_bar(stage));
            if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1u; }
          }
          umma_commit<1>(acc_full);
          tile_phase ^= 1u;
        }
      };
      if (nlimb == 1) issue_all(std::integral_constant<int, 1>{});
      else issue_all(std::integral_constant<int, 4>{});
    }
  } else {
    const int q = warp & 3;
    uint32_t tile_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const int per = tiles_m * tiles_n;
      const int b = t / per, r = t - b * per;
      const int tm = r / tiles_n, tn = r - tm * tiles_n;
      if (!mbar_wait(acc_full, tile_phase, abort_word)) {
        *abort_word = 1;
        if (lane == 0) atomicMax(g.status, 0x300u | 7u);
        break;
      }
      tc_fence_after();
      const int row = tm * Cfg::BM + q * 32 + lane;
      uint32_t* crow = g.C + b * g.strideC + static_cast<long long>(row) * g.N;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c0 = 0; c0 < Cfg::BN; c0 += 32) {
        const int col0 = tn * Cfg::BN + c0;
        if (col0 >= g.N) break;
        uint32_t v[32], w[32];
        tmem_ld_32x32(t_row + c0, v);
        tmem_ld_wait();
        for (int c = 1; c < nlimb; ++c) {
          tmem_ld_32x32(t_row + c * Cfg::BN + c0, w);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += w[j] << (8 * c);
        }
        if (row < g.M) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < g.N) crow[col0 + j] = g.accumulate ? crow[col0 + j] + v[j] : v[j];
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
      tile_phase ^= 1u;
    }
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

}  // namespace mtb
