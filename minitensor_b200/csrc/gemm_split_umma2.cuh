// Two-CTA form of the split-bf16 tensor-core GEMM (see gemm_split_umma.cuh for
// the arithmetic).  Two CTAs of a cluster on neighbouring SMs work on one
// 256 x 256 output tile with tcgen05.mma.cta_group::2: each CTA stages 128
// rows of A and 128 of the 256 B columns, the pair's tensor cores exchange
// the B halves, and each CTA ends up with its 128 x 256 slice of the
// accumulator in its own tensor memory.  Per SM this halves the B-operand
// shared-memory reads of the one-CTA 128 x 256 tile (8 KB instead of 12 KB per
// MMA) and shrinks the ring writes, which is what limited that kernel.
//
// Roles per CTA: warp 0 lane 0 = TMA producer for this CTA's halves; warp 1 =
// TMEM allocation in both CTAs, MMA issue in the leader (cluster rank 0) only;
// warps 2..5 = epilogue for this CTA's 128 rows.  Barriers:
//   full[s]      leader only, 2 arrivals (one producer per CTA) + the bytes of
//                both CTAs' loads (the peer's loads signal the leader's barrier)
//   empty[s]     one per CTA; the leader's tcgen05.commit arrives on both
//   acc_full[a]  one per CTA; the leader's tcgen05.commit arrives on both
//   acc_empty[a] leader only, 8 arrivals (4 epilogue warps of each CTA)
// No load here uses a cluster broadcast; every CTA fetches its own tiles.
#pragma once
#include <type_traits>
#include "gemm_split_umma.cuh"

namespace mtb {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
  return r;
}
// arrive (count 1) and add `bytes` to the expected transaction count of a barrier anywhere in the cluster
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar_cluster, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(bar_cluster),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster_addr(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}
// Arrival that orders nothing but the barrier itself (the caller has already fenced what matters).
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}

// Work item `it` of SM pair `pair`: a whole tile, or one K range of a tail tile (see GemmArgs::tail_splits).
// part = -1 for a whole tile, else the index of the K range.  Returns false when the pair has no such item.
__device__ __forceinline__ bool pair_work_item(const GemmArgs& g, int it, int pair, int num_pairs, int num_tiles,
                                               int& tile, int& kb0, int& kb1, int& part) {
  part = -1;
  kb0 = 0;
  kb1 = g.num_kb;
  if (g.tail_splits <= 1) {
    tile = pair + it * num_pairs;
    return tile < num_tiles;
  }
  if (it < g.tail_rounds) {
    tile = it * num_pairs + pair;
    return true;
  }
  // the K ranges of the tail tiles are dealt out like tiles, range-major: item j = range j / tail_tiles of tail
  // tile j % tail_tiles; there may be more items than pairs (several short rounds)
  const int j = (it - g.tail_rounds) * num_pairs + pair;
  if (j < g.tail_tiles * g.tail_splits) {
    part = j / g.tail_tiles;
    tile = g.tail_rounds * num_pairs + (j - part * g.tail_tiles);
    kb0 = static_cast<int>(static_cast<long long>(g.num_kb) * part / g.tail_splits);
    kb1 = static_cast<int>(static_cast<long long>(g.num_kb) * (part + 1) / g.tail_splits);
    return true;
  }
  return false;
}

// One warp's 32 rows x 256 columns of a raw accumulator to dst[row][256] (row = lane's row inside the 256-row
// pair tile), through the same shared-memory transposition as the final epilogue so that stores are row segments.
template <int CW>
__device__ __forceinline__ void epilogue_warp_raw(float* stage, uint32_t t_row, float* __restrict__ dst, int row0,
                                                  int lane, int col_begin, int col_end) {
  constexpr int LPR = CW / 4, RPI = 32 / LPR, PITCH = CW + 1;
  const int cq = (lane % LPR) * 4, rsub = lane / LPR;
#pragma unroll 1
  for (int c0 = col_begin; c0 < col_end; c0 += CW) {
    uint32_t v[CW];
    if constexpr (CW == 32) tmem_ld_32x32(t_row + c0, v);
    else tmem_ld_32x16(t_row + c0, v);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < CW; ++j) stage[lane * PITCH + j] = __uint_as_float(v[j]);
    __syncwarp();
#pragma unroll
    for (int it = 0; it < LPR; ++it) {
      const int r = it * RPI + rsub;
      *reinterpret_cast<float4*>(dst + static_cast<long long>(row0 + r) * 256 + c0 + cq) =
          make_float4(stage[r * PITCH + cq], stage[r * PITCH + cq + 1], stage[r * PITCH + cq + 2],
                      stage[r * PITCH + cq + 3]);
    }
    __syncwarp();
  }
}

// Sum of the K-range partials of every tail tile (ascending range order), then scale / bias / activation / store:
// what the in-kernel epilogue does for whole tiles.  blockIdx.x = tail tile, blockIdx.y = group of 4 rows; one
// float4 per thread, so the kernel is a few thousand independent blocks (it is latency-bound otherwise).
template <int EPI>
__device__ __forceinline__ void tail_fixup_body(const GemmArgs& g, int num_pairs, int tiles_m, int tiles_n) {
  const int j = blockIdx.x;
  const int tile = g.tail_rounds * num_pairs + j;
  int b, tm, tn;
  tile_coords(tile, tiles_m, tiles_n, b, tm, tn);
  const int r = blockIdx.y * 4 + (threadIdx.x >> 6), c = (threadIdx.x & 63) * 4;
  const int grow = tm * 256 + r, gcol = tn * 256 + c;
  if (grow >= g.M || gcol >= g.N) return;
  const float* part = g.partial + static_cast<long long>(j) * g.tail_splits * 65536 + r * 256 + c;
  float4 acc = *reinterpret_cast<const float4*>(part);
  for (int p = 1; p < g.tail_splits; ++p) {
    const float4 t = *reinterpret_cast<const float4*>(part + static_cast<long long>(p) * 65536);
    acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
  }
  float* cptr = g.C + b * g.strideC + static_cast<long long>(grow) * g.ldc + gcol;
  if (g.raw_int) {
    // s32 accumulators of an int8 product: the partials were added as floats above, redo the sum on the bit patterns
    uint32_t sum[4];
    const float4 first = *reinterpret_cast<const float4*>(part);
    sum[0] = __float_as_uint(first.x); sum[1] = __float_as_uint(first.y);
    sum[2] = __float_as_uint(first.z); sum[3] = __float_as_uint(first.w);
    for (int p = 1; p < g.tail_splits; ++p) {
      const float4 t = *reinterpret_cast<const float4*>(part + static_cast<long long>(p) * 65536);
      sum[0] += __float_as_uint(t.x); sum[1] += __float_as_uint(t.y);
      sum[2] += __float_as_uint(t.z); sum[3] += __float_as_uint(t.w);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (gcol + e < g.N) cptr[e] = __uint_as_float(sum[e]);
    return;
  }
  float x[4] = {acc.x, acc.y, acc.z, acc.w};
  const float* aptr = (EPI == EPI_RELU_BWD) ? g.aux + b * g.strideC + static_cast<long long>(grow) * g.ldc + gcol : nullptr;
  const int ea = g.exp_b ? g.exp_a[(g.a_batched ? static_cast<long long>(b) * g.M : 0) + grow] : 0;
  const int* eb = g.exp_b ? g.exp_b + (g.b_batched ? static_cast<long long>(b) * g.N : 0) + gcol : nullptr;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    if (gcol + e >= g.N) break;
    float v = x[e];
    if (eb) v = scale_pow2(v, ea + eb[e]);
    if (g.bias) v += g.bias_per_row ? g.bias[grow] : g.bias[gcol + e];
    cptr[e] = apply_epilogue_t<EPI>(v, EPI == EPI_RELU_BWD ? aptr[e] : 0.0f);
  }
}
static __global__ void __launch_bounds__(256)
tail_fixup_kernel(const GemmArgs g, int num_pairs, int tiles_m, int tiles_n) {
  grid_dependency_wait();
  grid_launch_dependents();
  if (g.gate && ((*g.gate == g.gate_value) != (g.gate_run_if_equal != 0))) return;  // the product itself did not run
  switch (g.epilogue) {
    case EPI_RELU: tail_fixup_body<EPI_RELU>(g, num_pairs, tiles_m, tiles_n); break;
    case EPI_GELU_ERF: tail_fixup_body<EPI_GELU_ERF>(g, num_pairs, tiles_m, tiles_n); break;
    case EPI_GELU_TANH: tail_fixup_body<EPI_GELU_TANH>(g, num_pairs, tiles_m, tiles_n); break;
    case EPI_RELU_BWD: tail_fixup_body<EPI_RELU_BWD>(g, num_pairs, tiles_m, tiles_n); break;
    default: tail_fixup_body<EPI_NONE>(g, num_pairs, tiles_m, tiles_n); break;
  }
}

template <int BK, int STAGES, int NP = 3>
struct Gemm2Cfg {
  static constexpr int BM = 128;        // rows per CTA
  static constexpr int BNH = 128;       // B columns staged per CTA
  static constexpr int TILE_M = 256, TILE_N = 256;
  static constexpr int ROW_BYTES = BK * 2;
  static constexpr int A_TILE = BM * ROW_BYTES;
  static constexpr int B_TILE = BNH * ROW_BYTES;
  static constexpr int STAGE_BYTES = NP * (A_TILE + B_TILE);  // NP planes of each operand per stage
  static constexpr int TMEM_COLS = 512;  // two 256-column accumulators
  // Eight epilogue warps per CTA: two per TMEM lane quarter, 128 of the tile's 256 columns each.  While tiles follow
  // one another the epilogue hides behind the next tile's MMAs either way; in the last round of a product, and in
  // products of a single round, its length is exposed and halves.
  static constexpr int EPI_WARPS = 8;
  static constexpr int NUM_THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int EPI_CW = 32;
  static constexpr int EPI_BYTES = EPI_WARPS * 32 * (EPI_CW + 1) * 4;  // epilogue staging, see epilogue_warp_tile
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + EPI_BYTES;
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
  static_assert(ROW_BYTES == 64 || ROW_BYTES == 128, "BK must be 32 or 64");
};

// A_MN / B_MN: that operand's planes are MN-major ([k][mn] row-major in global
// memory, mn padded to a multiple of 64) and its tensor map is the 4-D view
// {64, k, mn / 64, plane}; otherwise K-major planes [mn][k] with the 3-D map.
// MN-major needs BK = 64 (128-byte swizzle rows of 64 elements).
// NP = planes per operand held in a stage: 3 (bf16 modes), 2 (fp16 mode) or 1.
// I8: the planes hold signed bytes (a K block of 64 16-bit units is 128 bytes = 128 k), the product is one
// tcgen05.mma.kind::i8 per 32 k with an s32 accumulator, and the epilogue moves the 32-bit results out unchanged
// (no scaling, bias or activation: the float path of the epilogue only copies bits then).
template <int BK, int STAGES, bool A_MN = false, bool B_MN = false, int NP = 3, bool I8 = false>
__global__ void __launch_bounds__(Gemm2Cfg<BK, STAGES, NP>::NUM_THREADS, 1)
gemm_split_umma2_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
                        const GemmArgs g) {
  using Cfg = Gemm2Cfg<BK, STAGES, NP>;
  static_assert(!(A_MN || B_MN) || BK == 64, "MN-major operands need BK = 64");
  static_assert(!I8 || (!A_MN && !B_MN && BK == 64), "the int8 product takes K-major byte planes");
  if (g.gate) {
    grid_dependency_wait();      // the gate word is written by the kernels before this one
    if ((*g.gate == g.gate_value) != (g.gate_run_if_equal != 0)) return;  // every thread of both CTAs
  }
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  const uint32_t bars = tiles + STAGES * Cfg::STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
  const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 4);
  const uint32_t abort_addr = tmem_slot + 4u;
  volatile uint32_t* abort_word = reinterpret_cast<volatile uint32_t*>(smem_raw + (abort_addr - raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  const int tiles_m = (g.M + Cfg::TILE_M - 1) / Cfg::TILE_M;
  const int tiles_n = (g.N + Cfg::TILE_N - 1) / Cfg::TILE_N;
  const int num_tiles = tiles_m * tiles_n * g.batch;
  const int nsplit = (g.mode == 1) ? 1 : ((g.mode == 3 || g.mode == 23) ? 2 : 3);
  const uint32_t stage_tx = nsplit * (Cfg::A_TILE + Cfg::B_TILE);  // bytes this CTA loads per stage

  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 2);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 2 * Cfg::EPI_WARPS);   // every epilogue warp of both CTAs
    }
    fence_mbar_init();
    prefetch_tmap(&tmapA);
    prefetch_tmap(&tmapB);
  }
  if (warp == 1) {
    tmem_alloc<2>(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish<2>();
  }
  tc_fence_before();
  cluster_sync_all();  // barriers of both CTAs initialised, TMEM allocated
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  grid_dependency_wait();        // the operand planes and exponents come from the kernels before this one
  grid_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int t, kbeg, kend, part;
      for (int it = 0; ok && pair_work_item(g, it, pair, num_pairs, num_tiles, t, kbeg, kend, part); ++it) {
        int b, tm, tn;
        tile_coords(t, tiles_m, tiles_n, b, tm, tn);
        const int za = (g.a_batched ? b : 0) * g.planes_per_mat, zb = (g.b_batched ? b : 0) * g.planes_per_mat;
        const int kb0 = b * g.kb_batch_stride;
        const int row_a = tm * Cfg::TILE_M + int(rank) * Cfg::BM;
        const int row_b = tn * Cfg::TILE_N + int(rank) * Cfg::BNH;
        for (int kb = kbeg; kb < kend; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_word)) {
            *abort_word = 1;
            atomicMax(g.status, 0x100u | 2u);
            ok = false;
            break;
          }
          const uint32_t lead_full = map_to_cta(full_bar(stage), 0);
          mbar_expect_tx_cluster(lead_full, stage_tx);
          const uint32_t sa = tiles + stage * Cfg::STAGE_BYTES;
          const uint32_t sb = sa + NP * Cfg::A_TILE;
          for (int s = 0; s < nsplit; ++s) {
            if constexpr (A_MN)
              tma_load_4d_pair(sa + s * Cfg::A_TILE, &tmapA, lead_full, 0, (kb0 + kb) * BK, row_a >> 6, za + s);
            else
              tma_load_3d_pair(sa + s * Cfg::A_TILE, &tmapA, lead_full, (kb0 + kb) * BK, row_a, za + s);
          }
          for (int s = 0; s < nsplit; ++s) {
            if constexpr (B_MN)
              tma_load_4d_pair(sb + s * Cfg::B_TILE, &tmapB, lead_full, 0, (kb0 + kb) * BK, row_b >> 6, zb + s);
            else
              tma_load_3d_pair(sb + s * Cfg::B_TILE, &tmapB, lead_full, (kb0 + kb) * BK, row_b, zb + s);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = I8 ? make_idesc(Cfg::TILE_M, Cfg::TILE_N, 1u /*signed bytes*/, 2u /*s32*/)
                                : make_idesc(Cfg::TILE_M, Cfg::TILE_N, g.mode == 23 ? 0u /*f16*/ : 1u /*bf16*/, 1u,
                                             A_MN ? 1u : 0u, B_MN ? 1u : 0u);
      // The whole issue loop, with the product schedule known at compile time: per product the
      // thread adds a constant to each operand's descriptor and issues the MMA.
      auto issue_all = [&](auto npairs_tag) {
        constexpr int NPAIRS = decltype(npairs_tag)::value;
        // one MMA covers 16 k: 32 bytes along a K-major row, 16 rows of 128 bytes in an MN-major chunk
        constexpr uint32_t A_KSTEP = A_MN ? 2048u : 32u, B_KSTEP = B_MN ? 2048u : 32u;
        int stage = 0, acc = 0;
        uint32_t phase = 0, acc_phase = 0;
        int t, kbeg, kend, part;
        for (int it = 0; pair_work_item(g, it, pair, num_pairs, num_tiles, t, kbeg, kend, part); ++it) {
          if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u, abort_word)) {
            *abort_word = 1;
            atomicMax(g.status, 0x200u | 3u);
            return;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * Cfg::TILE_N;
          uint32_t accumulate = 0;
          for (int kb = kbeg; kb < kend; ++kb) {
            if (!mbar_wait(full_bar(stage), phase, abort_word)) {
              *abort_word = 1;
              atomicMax(g.status, 0x200u | 4u);
              return;
            }
            tc_fence_after();
            const uint32_t sa = tiles + stage * Cfg::STAGE_BYTES;
            const uint32_t sb = sa + NP * Cfg::A_TILE;
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
                if constexpr (I8) umma_i8<2>(d_tmem, da0 + (offa >> 4), db0 + (offb >> 4), idesc, accumulate);
                else umma_f16<2>(d_tmem, da0 + (offa >> 4), db0 + (offb >> 4), idesc, accumulate);
                accumulate = 1;
              }
            }
            // the stage is free in both CTAs once these MMAs have read it
            umma_commit<2>(empty_bar(stage));
            umma_commit<2>(map_to_cta(empty_bar(stage), 1));
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
          umma_commit<2>(acc_full_bar(acc));
          umma_commit<2>(map_to_cta(acc_full_bar(acc), 1));
          if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
      };
      const int npairs = split_pair_count(g.mode);
      if (npairs == 3) issue_all(std::integral_constant<int, 3>{});
      else if (npairs == 1) issue_all(std::integral_constant<int, 1>{});
      else if constexpr (NP == 3) {
        if (npairs == 9) issue_all(std::integral_constant<int, 9>{});
        else issue_all(std::integral_constant<int, 6>{});
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    const int half_cols = ((warp - 2) >> 2) * (Cfg::TILE_N / 2);   // the quarter's second warp takes the upper columns
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(g.C) & 15) == 0) && ((g.ldc & 3) == 0) && ((g.strideC & 3) == 0);
    int t, kbeg, kend, part;
    for (int it = 0; pair_work_item(g, it, pair, num_pairs, num_tiles, t, kbeg, kend, part); ++it) {
      int b, tm, tn;
      tile_coords(t, tiles_m, tiles_n, b, tm, tn);
      const int row_first = tm * Cfg::TILE_M + int(rank) * Cfg::BM + q * 32;
      const int col_first = tn * Cfg::TILE_N + half_cols;
      const int col_last = min(min(g.N, (tn + 1) * Cfg::TILE_N), col_first + Cfg::TILE_N / 2);
      if (part < 0) epilogue_prefetch(g, b, row_first, col_first, col_last, lane);
      if (!mbar_wait(acc_full_bar(acc), acc_phase, abort_word)) {
        *abort_word = 1;
        if (lane == 0) atomicMax(g.status, 0x300u | 2u);
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * Cfg::TILE_N;
      float* stage = reinterpret_cast<float*>(smem_raw + (bars + 256u - raw)) + (warp - 2) * 32 * (Cfg::EPI_CW + 1);
      if (part >= 0) {
        // one K range of a tail tile: the raw accumulator goes to its slot, the fix-up kernel finishes the tile
        float* slot = g.partial + (static_cast<long long>(t - g.tail_rounds * num_pairs) * g.tail_splits + part) * 65536;
        epilogue_warp_raw<Cfg::EPI_CW>(stage, t_row, slot, int(rank) * Cfg::BM + q * 32, lane, half_cols,
                                       half_cols + Cfg::TILE_N / 2);
      } else {
        epilogue_warp_tile<Cfg::EPI_CW>(g, stage, t_row + half_cols, b, row_first, col_first, col_last, lane, vec_ok);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster_relaxed(map_to_cta(acc_empty_bar(acc), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  cluster_sync_all();  // neither CTA frees tensor memory or exits while the other may still use the pair
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<2>(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace mtb
