// Stride-1 convolution (forward and data gradient) as an implicit GEMM whose image operand is staged ONCE per
// (output row block, channel block) as a halo tile and then multiplied against every filter tap.
//
//   out[n][m][y][x] = sum over taps (fh, fw) and channels c of  A[m][(tap, c)] * img[n][c][y + dy(tap)][x + dx(tap)]
//
// (engine/src/operations/conv.rs:111-157 forward; the data gradient of engine/src/autograd/mod/shape.rs:86-127 is the
// same sum over the upstream gradient with the taps mirrored.)
//
// The image lives in channels-last split planes {c, w, h, image*planes + split} (see conv2d.cu).  For an output tile
// of `th` image rows the producer loads, per channel block of 32, the box {32 channels, wh columns, hh = th + kh - 1
// rows}, wh = out_w + kw - 1 rounded up to a multiple of 4, with the hardware's zero fill standing in for the
// padding.  In shared memory that box is a K-major operand whose rows are the halo pixels in raster order (64-byte
// rows, 64-byte swizzle).  The window of tap (fh, fw) is the SAME rows shifted by off = fh * wh + fw, so its MMA
// descriptor is the tile's descriptor with the start address advanced by off rows: the swizzle is a function of the
// shared-memory address, which makes a start that is not aligned to the swizzle repeat read exactly the rows it
// names.  The MMA's N index then runs over th halo-wide output rows; the columns past out_w in each row (and the
// round-up of N to a multiple of 16) are garbage that depends on nothing but its own B row, and the epilogue drops
// it.  Per tile the image bytes cross L2 -> shared memory once instead of once per tap.
//
// Weights.  One (tap, channel block) of the weights is an A tile of 128 rows x 32 channels per plane - or of 64 rows
// when the layer has at most 64 output rows: the MMA still runs with M = 128 (an M = 64 instruction takes the same
// time) and reads its rows 64..127 from whatever follows the tile in shared memory; those rows only produce
// accumulator rows 64..127, which nothing reads.  When all tiles of the layer fit beside the image ring they are
// loaded once per CTA and stay RESIDENT for every tile the CTA computes (the large conv config: 9 taps x 2 blocks x
// 2 planes x 4 KB = 144 KB); otherwise they stream through a ring that is as deep as shared memory allows.
//
// Epilogue.  tcgen05.ld hands every lane 32 consecutive columns of its own output row; because wh and out_w are
// multiples of 4 (the usual case) every aligned group of four columns is either four consecutive valid pixels or
// garbage, so a lane stores float4s straight from its registers - no transposition through shared memory.  Eight
// epilogue warps (two per TMEM lane quarter, alternating 32-column chunks) keep the epilogue of a tile shorter than
// the next tile's MMAs; two accumulators in TMEM let them overlap.
//
// Roles: warp 0 = weight producer, warp 2 = image producer, warp 1 = TMEM owner and MMA issuer, warps 3..10 =
// epilogue.  Every wait is bounded and reports through the status word (role codes 0x4.. - 0x7..).
#pragma once
#include <type_traits>

#include "gemm_split_umma.cuh"
#include "ptx_sm100.cuh"

namespace mtb {

struct ConvHaloArgs {
  int M;                   // output rows (channels) per image
  int out_h, out_w;        // output image
  int batch;               // images
  float* C;                // [batch][M][out_h * out_w]
  const float* bias;       // [M] or nullptr
  int mode;                // 1, 3, 6, 9 bf16 products or 23 (two fp16 planes, three products)
  int planes_per_mat;      // planes stored per image / weight matrix (3 bf16, 2 fp16)
  const int* exp_a;        // fp16 mode: scale exponent per output row [M], else nullptr
  const int* exp_b;        // fp16 mode: scale exponent per image [batch], else nullptr
  int th, wh, hh;          // output rows per tile, halo width and height
  int umma_n;              // th * wh rounded up to a multiple of 16
  int kh, kw;
  int cbs;                 // channel blocks of 32
  int chan_p;              // padded channel count: the weights' K index is tap * chan_p + c
  int w_org, h_org;        // halo origin relative to (0, first output row of the tile)
  int flip;                // 0: tap (fh, fw) reads halo offset (fh, fw); 1: (kh-1-fh, kw-1-fw)  (data gradient)
  uint32_t b_plane_bytes;  // shared-memory bytes per image plane of a stage (multiple of 1024)
  int a_rows;              // weight rows of an A tile per plane: 128, or 64 when M <= 64
  int a_stages;            // A tiles shared memory holds: the ring depth, or taps * cbs when resident
  int a_resident;          // 1: every (tap, channel block) tile is loaded once and kept (needs M <= 128)
  uint32_t* status;
};

template <int PLANES>
struct ConvHaloCfg {
  static constexpr int BM = 128, BK = 32, ROW_BYTES = 64;
  static constexpr int MAX_A_STAGES = 16, B_STAGES = 2;   // MAX_A_STAGES bounds the streaming ring (barrier room)
  static constexpr int NUM_THREADS = 352;
  static constexpr int TMEM_COLS = 512;              // two accumulators of up to 256 columns
  static constexpr int MAX_TAPS = 128;               // filter taps (kh * kw) the tap table has room for
  static constexpr int BAR_BYTES = 512 + 4 * MAX_TAPS;   // barriers, TMEM slot, abort word; then the tap table
  static constexpr size_t a_stage_bytes(int a_rows) { return size_t(PLANES) * a_rows * ROW_BYTES; }
  // everything but the weight tiles (a 64-row last tile is over-read into what follows it, which is the image ring)
  static constexpr size_t fixed_bytes(size_t b_plane_bytes) {
    return 1024 + size_t(B_STAGES) * PLANES * b_plane_bytes + BAR_BYTES;
  }
  static constexpr size_t smem_bytes(size_t b_plane_bytes, int a_rows, int a_stages) {
    return fixed_bytes(b_plane_bytes) + size_t(a_stages) * a_stage_bytes(a_rows);
  }
};

template <int PLANES>
__global__ void __launch_bounds__(352, 1)
conv_halo_umma_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
                      const ConvHaloArgs g) {
  using Cfg = ConvHaloCfg<PLANES>;
  constexpr int BST = Cfg::B_STAGES;
  const int AST = g.a_resident ? 1 : g.a_stages;     // barrier pairs of the weight tiles
  const uint32_t a_tile = static_cast<uint32_t>(g.a_rows) * Cfg::ROW_BYTES;   // one plane of one (tap, channel block)
  const uint32_t a_stage = PLANES * a_tile;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t a_ring = (raw + 1023u) & ~1023u;
  const uint32_t b_ring = a_ring + g.a_stages * a_stage;   // a 64-row last tile is over-read into the image ring: harmless
  const uint32_t b_stage_bytes = PLANES * g.b_plane_bytes;
  const uint32_t bars = b_ring + BST * b_stage_bytes;
  auto a_full = [&](int s) { return bars + 8u * s; };
  auto a_empty = [&](int s) { return bars + 8u * (AST + s); };
  auto b_full = [&](int s) { return bars + 8u * (2 * AST + s); };
  auto b_empty = [&](int s) { return bars + 8u * (2 * AST + BST + s); };
  auto acc_full = [&](int a) { return bars + 8u * (2 * AST + 2 * BST + a); };
  auto acc_empty = [&](int a) { return bars + 8u * (2 * AST + 2 * BST + 2 + a); };
  const uint32_t tmem_slot = bars + 8u * (2 * AST + 2 * BST + 4);
  const uint32_t abort_addr = tmem_slot + 4u;
  volatile uint32_t* abort_word = reinterpret_cast<volatile uint32_t*>(smem_raw + (abort_addr - raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));
  // tap_off16[tap]: the halo row offset of the tap's window, in 16-byte units of shared-memory address
  uint32_t* tap_off16 = reinterpret_cast<uint32_t*>(smem_raw + (bars + 512u - raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (g.M + Cfg::BM - 1) / Cfg::BM;
  const int row_blocks = (g.out_h + g.th - 1) / g.th;
  const int num_tiles = tiles_m * row_blocks * g.batch;
  const int taps = g.kh * g.kw;
  const int nsplit = (g.mode == 1) ? 1 : ((g.mode == 3 || g.mode == 23) ? 2 : 3);
  auto decode = [&](int t, int& b, int& rb, int& tm) {   // m tiles of one halo next to each other
    tm = t % tiles_m;
    const int q = t / tiles_m;
    rb = q % row_blocks;
    b = q / row_blocks;
  };

  for (int tap = threadIdx.x; tap < g.kh * g.kw; tap += blockDim.x) {
    const int fh = tap / g.kw, fw = tap - fh * g.kw;
    const int off = g.flip ? ((g.kh - 1 - fh) * g.wh + (g.kw - 1 - fw)) : (fh * g.wh + fw);
    tap_off16[tap] = static_cast<uint32_t>(off) * (Cfg::ROW_BYTES >> 4);
  }
  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < AST; ++s) { mbar_init(a_full(s), 1); mbar_init(a_empty(s), 1); }
    for (int s = 0; s < BST; ++s) { mbar_init(b_full(s), 1); mbar_init(b_empty(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(acc_full(a), 1); mbar_init(acc_empty(a), 8); }
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
    // ------------------------------------------------------------ weight producer
    if (lane == 0 && blockIdx.x < num_tiles) {
      if (g.a_resident) {
        // every (channel block, tap) tile once; tile index cb * taps + tap; one barrier counts all the bytes
        int b, rb, tm;
        decode(blockIdx.x, b, rb, tm);
        mbar_expect_tx(a_full(0), static_cast<uint32_t>(g.cbs * taps * nsplit) * a_tile);
        for (int cb = 0; cb < g.cbs; ++cb)
          for (int tap = 0; tap < taps; ++tap) {
            const uint32_t sa = a_ring + (cb * taps + tap) * a_stage;
            for (int s = 0; s < nsplit; ++s)
              tma_load_3d(sa + s * a_tile, &tmapA, a_full(0), tap * g.chan_p + cb * Cfg::BK, tm * Cfg::BM, s);
          }
      } else {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
          int b, rb, tm;
          decode(t, b, rb, tm);
          for (int cb = 0; cb < g.cbs && ok; ++cb)
            for (int tap = 0; tap < taps; ++tap) {
              if (!mbar_wait(a_empty(stage), phase ^ 1u, abort_word)) {
                *abort_word = 1;
                atomicMax(g.status, 0x400u | 1u);
                ok = false;
                break;
              }
              mbar_expect_tx(a_full(stage), nsplit * a_tile);
              const uint32_t sa = a_ring + stage * a_stage;
              for (int s = 0; s < nsplit; ++s)
                tma_load_3d(sa + s * a_tile, &tmapA, a_full(stage), tap * g.chan_p + cb * Cfg::BK, tm * Cfg::BM, s);
              if (++stage == AST) { stage = 0; phase ^= 1u; }
            }
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------ image producer: one halo box per channel block
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t box_bytes = static_cast<uint32_t>(g.wh) * g.hh * Cfg::ROW_BYTES;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int b, rb, tm;
        decode(t, b, rb, tm);
        for (int cb = 0; cb < g.cbs; ++cb) {
          if (!mbar_wait(b_empty(stage), phase ^ 1u, abort_word)) {
            *abort_word = 1;
            atomicMax(g.status, 0x500u | 1u);
            ok = false;
            break;
          }
          mbar_expect_tx(b_full(stage), nsplit * box_bytes);
          const uint32_t sb = b_ring + stage * b_stage_bytes;
          for (int s = 0; s < nsplit; ++s)
            tma_load_4d(sb + s * g.b_plane_bytes, &tmapB, b_full(stage), cb * Cfg::BK, g.w_org, rb * g.th + g.h_org,
                        b * g.planes_per_mat + s);
          if (++stage == BST) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc(Cfg::BM, g.umma_n, g.mode == 23 ? 0u : 1u, /*f32*/ 1u);
      // Issue loop.  One thread feeds the tensor core, so what it executes per MMA decides whether the pipe stays
      // busy: the tap offsets come from the table in shared memory, the descriptors' constant high words are
      // built once, and each MMA costs two 32-bit adds on the low words (start address field, 16-byte units).
      const uint32_t a_tile16 = a_tile >> 4, a_stage16 = a_stage >> 4;
      uint32_t bplane16[3];
#pragma unroll
      for (int j = 0; j < 3; ++j) bplane16[j] = j * (g.b_plane_bytes >> 4);
      const uint64_t dproto = make_kmajor_desc<Cfg::ROW_BYTES>(0);
      const uint32_t d_hi = static_cast<uint32_t>(dproto >> 32), d_lo0 = static_cast<uint32_t>(dproto);
      const uint32_t a_lo_base = d_lo0 + ((a_ring & 0x3FFFFu) >> 4);
      const uint32_t b_lo_base = d_lo0 + ((b_ring & 0x3FFFFu) >> 4);
      const uint32_t b_stage16 = b_stage_bytes >> 4;
      const bool resident = g.a_resident != 0;
      auto issue_all = [&](auto npairs_tag) {
        constexpr int NPAIRS = decltype(npairs_tag)::value;
        int as = 0, bs = 0, acc = 0;
        uint32_t aphase = 0, bphase = 0, acc_phase = 0;
        if (resident && blockIdx.x < num_tiles) {
          if (!mbar_wait(a_full(0), 0, abort_word)) {
            *abort_word = 1;
            atomicMax(g.status, 0x600u | 4u);
            return;
          }
          tc_fence_after();
        }
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
          if (!mbar_wait(acc_empty(acc), acc_phase ^ 1u, abort_word)) {
            *abort_word = 1;
            atomicMax(g.status, 0x600u | 1u);
            return;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * 256;
          uint32_t accumulate = 0;
          uint32_t a_lo_res = a_lo_base;            // resident tiles are walked in storage order (cb, tap)
          for (int cb = 0; cb < g.cbs; ++cb) {
            if (!mbar_wait(b_full(bs), bphase, abort_word)) {
              *abort_word = 1;
              atomicMax(g.status, 0x600u | 2u);
              return;
            }
            tc_fence_after();
            const uint32_t b_lo_stage = b_lo_base + bs * b_stage16;
            uint32_t next_off = tap_off16[0];
            for (int tap = 0; tap < taps; ++tap) {
              const uint32_t b_lo_tap = b_lo_stage + next_off;
              if (tap + 1 < taps) next_off = tap_off16[tap + 1];
              uint32_t a_lo_tap;
              if (resident) {
                a_lo_tap = a_lo_res;
                a_lo_res += a_stage16;
              } else {
                if (!mbar_wait(a_full(as), aphase, abort_word)) {
                  *abort_word = 1;
                  atomicMax(g.status, 0x600u | 3u);
                  return;
                }
                tc_fence_after();
                a_lo_tap = a_lo_base + as * a_stage16;
              }
#pragma unroll
              for (int kk = 0; kk < Cfg::BK / 16; ++kk) {
#pragma unroll
                for (int p = 0; p < NPAIRS; ++p) {
                  const int code = split_pair_at(NPAIRS, p);
                  umma_f16_lohi(d_tmem, a_lo_tap + (code >> 2) * a_tile16 + kk * 2, d_hi,
                                b_lo_tap + bplane16[code & 3] + kk * 2, d_hi, idesc, accumulate);
                  accumulate = 1;
                }
              }
              if (!resident) {
                umma_commit<1>(a_empty(as));
                if (++as == AST) { as = 0; aphase ^= 1u; }
              }
            }
            umma_commit<1>(b_empty(bs));
            if (++bs == BST) { bs = 0; bphase ^= 1u; }
          }
          umma_commit<1>(acc_full(acc));
          if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
      };
      if constexpr (PLANES == 2) {
        if (g.mode == 1) issue_all(std::integral_constant<int, 1>{});
        else issue_all(std::integral_constant<int, 3>{});
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
    // ------------------------------------------------------------ epilogue (warps 3..10)
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    const int half = (warp - 3) >> 2;    // which of the quarter's two warps: it takes every other 32-column chunk
    const long long opix = static_cast<long long>(g.out_h) * g.out_w;
    const bool vec_ok = ((g.out_w & 3) == 0) && ((reinterpret_cast<uintptr_t>(g.C) & 15) == 0);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int b, rb, tm;
      decode(t, b, rb, tm);
      if (!mbar_wait(acc_full(acc), acc_phase, abort_word)) {
        *abort_word = 1;
        if (lane == 0) atomicMax(g.status, 0x700u | 1u);
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * 256;
      const int row = tm * Cfg::BM + q * 32 + lane;
      const int y0 = rb * g.th;
      const int rows_here = min(g.th, g.out_h - y0);
      const int n_valid = rows_here * g.wh;                 // columns beyond belong to rows outside the image
      if (tm * Cfg::BM + q * 32 < g.M) {                    // some lane of this warp owns a real output row
        const bool row_ok = row < g.M;
        const float bias_r = (g.bias && row_ok) ? __ldg(g.bias + row) : 0.0f;
        // the two exact power-of-two factors that undo the operand scalings (scale_pow2's arithmetic, hoisted)
        float f1 = 1.0f, f2 = 1.0f;
        if (g.exp_a && row_ok) {
          const int ex = __ldg(g.exp_a + row) + __ldg(g.exp_b + b);
          const int e1 = max(-126, min(127, ex));
          const int e2 = max(-126, min(127, ex - e1));
          f1 = __int_as_float((e1 + 127) << 23);
          f2 = __int_as_float((e2 + 127) << 23);
        }
        float* crow = g.C + (static_cast<long long>(b) * g.M + (row_ok ? row : 0)) * opix + static_cast<long long>(y0) * g.out_w;
#pragma unroll 1
        for (int c0 = half * 32; c0 < n_valid; c0 += 64) {
          uint32_t v[32];
          tmem_ld_32x32(t_row + c0, v);
          tmem_ld_wait();
          if (row_ok) {
            int hr = c0 / g.wh, cx = c0 - hr * g.wh;        // wh is a multiple of 4, and so are c0 and cx
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              if (hr < rows_here && cx < g.out_w) {
                float o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) o[e] = __uint_as_float(v[4 * k + e]) * f1 * f2 + bias_r;
                float* dst = crow + hr * g.out_w + cx;
                if (vec_ok) {
                  *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
                } else {
#pragma unroll
                  for (int e = 0; e < 4; ++e)
                    if (cx + e < g.out_w) dst[e] = o[e];
                }
              }
              cx += 4;
              if (cx >= g.wh) { cx -= g.wh; ++hr; }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty(acc));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------------------------------------------------------- teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    // a wait ran out: give loads and MMAs still in flight time to land before shared memory and TMEM are handed back
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace mtb
