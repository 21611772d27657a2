// Stride-1 convolution (forward and data gradient) as an implicit GEMM with the OUTPUT PIXELS on the MMA's M side
// and the output channels on its N side:
//
//   out[n][oc][y][x] = sum over taps (fh, fw) and channels c of  img[n][c][y + dy(tap)][x + dx(tap)] * W[oc][(tap, c)]
//
// (engine/src/operations/conv.rs:111-157 forward; the data gradient of engine/src/autograd/mod/shape.rs:86-127 is the
// same sum over the upstream gradient with the taps mirrored.)
//
// Why this orientation: a tcgen05 MMA always spends the time of 128 M rows, so a layer with 64 output channels on
// the M side wastes half of the tensor core (the large conv config has 64).  With pixels on M every row is an
// output pixel whatever the channel count, and N = the channel count (a multiple of 16 up to 256).
//
// Image operand (A).  The image lives in channels-last split planes {c, w, h, image*planes + split} (conv2d.cu).  An
// output tile is tr rows x tc columns; per channel block of BK channels (64, or 32 where 64 does not fit shared
// memory) the producer loads the halo box {BK channels, wp = tc + kw - 1 columns, hh = tr + kh - 1 rows} with the
// hardware's zero fill standing in for the padding.  In shared memory that box is a K-major operand whose rows are
// the halo pixels in raster order (2 * BK bytes per row, swizzle of the same width).  Output pixel (r, c) of the
// tile is "position" n = r * wp + c; its window under tap (fh, fw) is halo row n + fh * wp + fw.  So the A operand
// of a tap is the tile's rows shifted by off = fh * wp + fw: the tile's descriptor with the start address advanced
// by off rows.  The swizzle is a function of the shared-memory address, so a start - or a plane base - that is not
// aligned to the swizzle repeat reads exactly the rows it names, and (measured) at the speed of an aligned one.
// Positions with c >= tc, and positions past the last row, are garbage that depends only on its own A row; they
// land in accumulator lanes the epilogue skips.  A tile has mb blocks of 128 positions, each its own MMA and
// accumulator.  The image bytes cross L2 -> shared memory once per (tile, channel block), not once per tap.
//
// Weights (B).  One (channel block, tap) of the weights is a tile of n_tile rows x BK channels per plane.  When all
// of a layer's tiles fit beside the image ring they are loaded once per CTA and stay RESIDENT (the large conv config:
// 9 tiles x 2 planes x 8 KB = 144 KB); otherwise they stream through a ring.
//
// What bounds the MMAs here.  An MMA of 128 x N x 16 fetches (128 + N) x 32 bytes of operands from shared memory, at
// about 150 bytes per ns measured (two thirds of that with 64-byte rows); below N = 128 that fetch, not the
// arithmetic, sets its duration (N = 64: 27 ns against 17 ns of arithmetic).  With 64 output channels every MMA is
// in that regime, so the fp16 mode FOLDS two of its three products: the hi and lo weight planes of a tile lie back
// to back in shared memory and are multiplied as ONE operand of 2 * n_tile rows - image_hi x [w_hi; w_lo] - into an
// accumulator of 2 * n_tile columns, then image_lo x w_hi goes onto its first n_tile columns.  The image rows are
// fetched twice instead of three times, the issuing thread sends two MMAs instead of three, and the epilogue adds
// the two column halves.
//
// Epilogue.  tcgen05.ld hands lane l of a warp the position 32 q + l of an M block and 32 consecutive output
// channels.  For one channel the 32 lanes hold consecutive positions, i.e. consecutive pixels of an output row, so
// each channel is one coalesced store - the NCHW result needs no transposition.  Eight epilogue warps (two per TMEM
// lane quarter) share the (M block, 32-channel chunk) items of a tile; two accumulator sets in TMEM overlap the
// epilogue of a tile with the next tile's MMAs.
//
// Roles: warp 0 = weight producer, warp 2 = image producer, warp 1 = TMEM owner and MMA issuer, warps 3..10 =
// epilogue.  Every wait is bounded and reports through the status word (role codes 0x8.. - 0xB..).
#pragma once
#include <type_traits>

#include "gemm_split_umma.cuh"
#include "ptx_sm100.cuh"

namespace mtb {

struct ConvPixArgs {
  int n_out;               // output channels
  int out_h, out_w;        // output image
  int batch;               // images
  float* C;                // [batch][n_out][out_h * out_w]
  const float* bias;       // [n_out] or nullptr
  int mode;                // 1, 3, 6, 9 bf16 products or 23 (two fp16 planes, three products)
  int planes_per_mat;      // planes stored per image / weight matrix (3 bf16, 2 fp16)
  const int* exp_w;        // fp16 mode: scale exponent per output channel [n_out], else nullptr
  const int* exp_img;      // fp16 mode: scale exponent per image [batch], else nullptr
  int tr, tc;              // output rows and columns per tile
  int wp, hh;              // halo pitch tc + kw - 1 and halo rows tr + kh - 1
  int mb;                  // blocks of 128 positions per tile: tr * wp <= 128 * mb
  int n_tile;              // output channels per tile = MMA N (multiple of 16, <= 256); two accumulator sets of
                           // mb * n_tile columns (twice that when folded) must fit the 512 TMEM columns
  int kh, kw;
  int cbs;                 // channel blocks of BK
  int chan_p;              // padded channel count: the weights' K index is tap * chan_p + c
  int w_org, h_org;        // halo origin relative to the tile's first output pixel
  int flip;                // 0: tap (fh, fw) reads halo offset (fh, fw); 1: (kh-1-fh, kw-1-fw)  (data gradient)
  // Strided forward convolution: the image planes are stored as sh * sw phase images (split_f16.cuh, RowPhases),
  // output pixel (y, x) under tap (fh, fw) reads phase ((fh - pad_h) mod sh, (fw - pad_w) mod sw) at
  // (y + floor((fh - pad_h) / sh), x + floor((fw - pad_w) / sw)): a stride-1 window again.  The halo box then has
  // a phase dimension and w_org / h_org are in phase-image coordinates.  sh = sw = 1: one phase, as above.
  int sh, sw, pad_h, pad_w;
  // Where output pixel (y, x) of channel oc goes: C[image][oc * out_plane + y * out_sy * out_pitch + x * out_sx].
  // A plain call has out_sy = out_sx = 1, out_pitch = out_w, out_plane = out_h * out_w; the strided data gradient
  // computes one phase of dx per launch and scatters it with the convolution's strides.
  int out_sy, out_sx, out_pitch;
  long long out_plane;
  uint32_t img_plane_bytes;  // shared-memory bytes per image plane of a stage (multiple of 128: TMA destinations)
  uint32_t w_tile_bytes;     // shared-memory bytes per weight plane of one (channel block, tap): n_tile rows
  int w_stages;            // weight tiles shared memory holds: the ring depth, or taps * cbs when resident
  int w_resident;          // 1: every (channel block, tap) tile is loaded once and kept (needs one channel tile)
  uint32_t* status;
  int fold;                // fp16 mode: the two weight planes of a tile are multiplied as ONE operand of 2 * n_tile rows
};

constexpr int CONV_PIX_THREADS = 352;
constexpr int CONV_PIX_MAX_W_STAGES = 16;      // bounds the streaming weight ring (barrier room)
constexpr int CONV_PIX_IMG_STAGES = 2;
constexpr int CONV_PIX_MAX_TAPS = 128;         // filter taps (kh * kw) the tap table has room for
constexpr int CONV_PIX_BAR_BYTES = 384 + 4 * CONV_PIX_MAX_TAPS;   // barriers, TMEM slot, abort word; then the tap table
// shared memory besides the weight tiles: alignment slack, the image ring, barriers and tap table
constexpr size_t conv_pix_fixed_bytes(int planes, size_t img_plane_bytes) {
  return 1024 + size_t(CONV_PIX_IMG_STAGES) * planes * img_plane_bytes + CONV_PIX_BAR_BYTES;
}

template <int PLANES, int BK_>
struct ConvPixCfg {
  static constexpr int BM = 128, BK = BK_, ROW_BYTES = 2 * BK_;
  static constexpr int IMG_STAGES = CONV_PIX_IMG_STAGES;
  static constexpr int TMEM_COLS = 512;
};

template <int PLANES, int BK>
__global__ void __launch_bounds__(CONV_PIX_THREADS, 1)
conv_pix_umma_kernel(const __grid_constant__ CUtensorMap tmapW, const __grid_constant__ CUtensorMap tmapImg,
                     const ConvPixArgs g) {
  using Cfg = ConvPixCfg<PLANES, BK>;
  constexpr int IST = Cfg::IMG_STAGES;
  const int WST = g.w_resident ? 1 : g.w_stages;     // barrier pairs of the weight tiles
  const uint32_t w_stage = PLANES * g.w_tile_bytes;
  const uint32_t img_stage = PLANES * g.img_plane_bytes;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t img_ring = (raw + 1023u) & ~1023u;
  const uint32_t w_ring = img_ring + IST * img_stage;
  const uint32_t bars = w_ring + g.w_stages * w_stage;
  auto w_full = [&](int s) { return bars + 8u * s; };
  auto w_empty = [&](int s) { return bars + 8u * (WST + s); };
  auto i_full = [&](int s) { return bars + 8u * (2 * WST + s); };
  auto i_empty = [&](int s) { return bars + 8u * (2 * WST + IST + s); };
  auto acc_full = [&](int a) { return bars + 8u * (2 * WST + 2 * IST + a); };
  auto acc_empty = [&](int a) { return bars + 8u * (2 * WST + 2 * IST + 2 + a); };
  const uint32_t tmem_slot = bars + 8u * (2 * WST + 2 * IST + 4);
  const uint32_t abort_addr = tmem_slot + 4u;
  volatile uint32_t* abort_word = reinterpret_cast<volatile uint32_t*>(smem_raw + (abort_addr - raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));
  // tap_off16[tap]: the halo row offset of the tap's window, in 16-byte units of shared-memory address
  uint32_t* tap_off16 = reinterpret_cast<uint32_t*>(smem_raw + (bars + 384u - raw));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_x = (g.out_w + g.tc - 1) / g.tc;
  const int tiles_y = (g.out_h + g.tr - 1) / g.tr;
  const int tiles_n = (g.n_out + g.n_tile - 1) / g.n_tile;
  const int num_tiles = tiles_n * tiles_x * tiles_y * g.batch;
  const int taps = g.kh * g.kw;
  const int nsplit = (g.mode == 1) ? 1 : ((g.mode == 3 || g.mode == 23) ? 2 : 3);
  auto decode = [&](int t, int& b, int& ty, int& tx, int& tn) {   // channel tiles of one halo next to each other
    tn = t % tiles_n;
    int q = t / tiles_n;
    tx = q % tiles_x;
    q /= tiles_x;
    ty = q % tiles_y;
    b = q / tiles_y;
  };

  const int phases = g.sh * g.sw;
  for (int tap = threadIdx.x; tap < taps; tap += blockDim.x) {
    const int fh = tap / g.kw, fw = tap - fh * g.kw;
    int off;
    if (phases == 1) {
      off = g.flip ? ((g.kh - 1 - fh) * g.wp + (g.kw - 1 - fw)) : (fh * g.wp + fw);
    } else {
      const int ay = fh - g.pad_h, ax = fw - g.pad_w;
      const int py = ((ay % g.sh) + g.sh) % g.sh, px = ((ax % g.sw) + g.sw) % g.sw;
      const int dy = (ay - py) / g.sh - g.h_org, dx = (ax - px) / g.sw - g.w_org;   // exact divisions
      off = (py * g.sw + px) * (g.hh * g.wp) + dy * g.wp + dx;
    }
    tap_off16[tap] = static_cast<uint32_t>(off) * (Cfg::ROW_BYTES >> 4);
  }
  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < WST; ++s) { mbar_init(w_full(s), 1); mbar_init(w_empty(s), 1); }
    for (int s = 0; s < IST; ++s) { mbar_init(i_full(s), 1); mbar_init(i_empty(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(acc_full(a), 1); mbar_init(acc_empty(a), 8); }
    fence_mbar_init();
    prefetch_tmap(&tmapW);
    prefetch_tmap(&tmapImg);
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  grid_dependency_wait();        // planes and exponents come from the kernels before this one
  grid_launch_dependents();
  const int acc_n = g.fold ? 2 * g.n_tile : g.n_tile;  // TMEM columns of one M block's accumulator
  const int acc_cols = g.mb * acc_n;                 // TMEM columns of one accumulator set

  if (warp == 0) {
    // ------------------------------------------------------------ weight producer
    if (lane == 0 && blockIdx.x < num_tiles) {
      if (g.w_resident) {
        // every (channel block, tap) tile once; tile index cb * taps + tap; one barrier counts all the bytes
        mbar_expect_tx(w_full(0), static_cast<uint32_t>(g.cbs * taps * nsplit) * g.w_tile_bytes);
        for (int cb = 0; cb < g.cbs; ++cb)
          for (int tap = 0; tap < taps; ++tap) {
            const uint32_t sw = w_ring + (cb * taps + tap) * w_stage;
            for (int s = 0; s < nsplit; ++s)
              tma_load_3d(sw + s * g.w_tile_bytes, &tmapW, w_full(0), tap * g.chan_p + cb * Cfg::BK, 0, s);
          }
      } else {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
          int b, ty, tx, tn;
          decode(t, b, ty, tx, tn);
          for (int cb = 0; cb < g.cbs && ok; ++cb)
            for (int tap = 0; tap < taps; ++tap) {
              if (!mbar_wait(w_empty(stage), phase ^ 1u, abort_word)) {
                *abort_word = 1;
                atomicMax(g.status, 0x800u | 1u);
                ok = false;
                break;
              }
              mbar_expect_tx(w_full(stage), nsplit * g.w_tile_bytes);
              const uint32_t sw = w_ring + stage * w_stage;
              for (int s = 0; s < nsplit; ++s)
                tma_load_3d(sw + s * g.w_tile_bytes, &tmapW, w_full(stage), tap * g.chan_p + cb * Cfg::BK,
                            tn * g.n_tile, s);
              if (++stage == WST) { stage = 0; phase ^= 1u; }
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
      const uint32_t box_bytes = static_cast<uint32_t>(g.wp) * g.hh * phases * Cfg::ROW_BYTES;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int b, ty, tx, tn;
        decode(t, b, ty, tx, tn);
        for (int cb = 0; cb < g.cbs; ++cb) {
          if (!mbar_wait(i_empty(stage), phase ^ 1u, abort_word)) {
            *abort_word = 1;
            atomicMax(g.status, 0x900u | 1u);
            ok = false;
            break;
          }
          mbar_expect_tx(i_full(stage), nsplit * box_bytes);
          const uint32_t si = img_ring + stage * img_stage;
          for (int s = 0; s < nsplit; ++s) {
            if (phases == 1)
              tma_load_4d(si + s * g.img_plane_bytes, &tmapImg, i_full(stage), cb * Cfg::BK, tx * g.tc + g.w_org,
                          ty * g.tr + g.h_org, b * g.planes_per_mat + s);
            else   // {c, x, y, phase, plane}: every phase image's halo in one request
              tma_load_5d(si + s * g.img_plane_bytes, &tmapImg, i_full(stage), cb * Cfg::BK, tx * g.tc + g.w_org,
                          ty * g.tr + g.h_org, 0, b * g.planes_per_mat + s);
          }
          if (++stage == IST) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // One thread feeds the tensor core, so what it executes per MMA decides whether the pipe stays busy: the
      // tap offsets come from the table in shared memory, the descriptors' constant high words are built once, and
      // each MMA costs a few 32-bit adds on the low words (start address field, 16-byte units).
      const uint32_t idesc = make_idesc(Cfg::BM, g.n_tile, g.mode == 23 ? 0u : 1u, /*f32*/ 1u);
      const uint32_t idesc_fold = make_idesc(Cfg::BM, 2 * g.n_tile, 0u, /*f32*/ 1u);
      const uint32_t w_tile16 = g.w_tile_bytes >> 4, w_stage16 = w_stage >> 4;
      const uint32_t img_plane16 = g.img_plane_bytes >> 4, img_stage16 = img_stage >> 4;
      const uint64_t dproto = make_kmajor_desc<Cfg::ROW_BYTES>(0);
      const uint32_t d_hi = static_cast<uint32_t>(dproto >> 32), d_lo0 = static_cast<uint32_t>(dproto);
      const uint32_t w_lo_base = d_lo0 + ((w_ring & 0x3FFFFu) >> 4);
      const uint32_t i_lo_base = d_lo0 + ((img_ring & 0x3FFFFu) >> 4);
      const uint32_t mblock16 = (Cfg::BM * Cfg::ROW_BYTES) >> 4;   // 128 positions further down the halo raster
      const bool resident = g.w_resident != 0;
      auto issue_all = [&](auto npairs_tag) {
        constexpr int NPAIRS = decltype(npairs_tag)::value;
        int ws = 0, is = 0, acc = 0;
        uint32_t wphase = 0, iphase = 0, acc_phase = 0;
        if (resident && blockIdx.x < num_tiles) {
          if (!mbar_wait(w_full(0), 0, abort_word)) {
            *abort_word = 1;
            atomicMax(g.status, 0xA00u | 4u);
            return;
          }
          tc_fence_after();
        }
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
          if (!mbar_wait(acc_empty(acc), acc_phase ^ 1u, abort_word)) {
            *abort_word = 1;
            atomicMax(g.status, 0xA00u | 1u);
            return;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * acc_cols;
          uint32_t accumulate = 0;
          uint32_t w_lo_res = w_lo_base;             // resident tiles are walked in storage order (cb, tap)
          for (int cb = 0; cb < g.cbs; ++cb) {
            if (!mbar_wait(i_full(is), iphase, abort_word)) {
              *abort_word = 1;
              atomicMax(g.status, 0xA00u | 2u);
              return;
            }
            tc_fence_after();
            const uint32_t i_lo_stage = i_lo_base + is * img_stage16;
            uint32_t next_off = tap_off16[0];
            for (int tap = 0; tap < taps; ++tap) {
              const uint32_t i_lo_tap = i_lo_stage + next_off;
              if (tap + 1 < taps) next_off = tap_off16[tap + 1];
              uint32_t w_lo_tap;
              if (resident) {
                w_lo_tap = w_lo_res;
                w_lo_res += w_stage16;
              } else {
                if (!mbar_wait(w_full(ws), wphase, abort_word)) {
                  *abort_word = 1;
                  atomicMax(g.status, 0xA00u | 3u);
                  return;
                }
                tc_fence_after();
                w_lo_tap = w_lo_base + ws * w_stage16;
              }
              for (int j = 0; j < g.mb; ++j) {
                const uint32_t a_lo = i_lo_tap + j * mblock16;
                const uint32_t dj = d_tmem + j * acc_n;
                if (NPAIRS == 3 && PLANES == 2 && g.fold) {
                  // hi x [hi; lo] as one MMA of 2 * n_tile columns, then lo x hi onto the first n_tile columns: the
                  // image rows are fetched twice instead of three times and the thread issues two MMAs, not three
#pragma unroll
                  for (int kk = 0; kk < Cfg::BK / 16; ++kk) {
                    umma_f16_lohi(dj, a_lo + kk * 2, d_hi, w_lo_tap + kk * 2, d_hi, idesc_fold, kk == 0 ? accumulate : 1u);
                    umma_f16_lohi(dj, a_lo + img_plane16 + kk * 2, d_hi, w_lo_tap + kk * 2, d_hi, idesc, 1u);
                  }
                  continue;
                }
#pragma unroll
                for (int kk = 0; kk < Cfg::BK / 16; ++kk) {
#pragma unroll
                  for (int p = 0; p < NPAIRS; ++p) {
                    const int code = split_pair_at(NPAIRS, p);
                    // only the very first MMA of a (tile, M block) overwrites its accumulator
                    umma_f16_lohi(dj, a_lo + (code >> 2) * img_plane16 + kk * 2, d_hi,
                                  w_lo_tap + (code & 3) * w_tile16 + kk * 2, d_hi, idesc,
                                  (kk == 0 && p == 0) ? accumulate : 1u);
                  }
                }
              }
              accumulate = 1;
              if (!resident) {
                umma_commit<1>(w_empty(ws));
                if (++ws == WST) { ws = 0; wphase ^= 1u; }
              }
            }
            umma_commit<1>(i_empty(is));
            if (++is == IST) { is = 0; iphase ^= 1u; }
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
    const int half = (warp - 3) >> 2;    // which of the quarter's two warps
    const long long opix = g.out_plane;
    const int chunks = (g.n_tile + 31) / 32;             // 32-channel chunks of an M block
    const int items = g.mb * chunks;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int b, ty, tx, tn;
      decode(t, b, ty, tx, tn);
      if (!mbar_wait(acc_full(acc), acc_phase, abort_word)) {
        *abort_word = 1;
        if (lane == 0) atomicMax(g.status, 0xB00u | 1u);
        break;
      }
      tc_fence_after();
      const int y0 = ty * g.tr, x0 = tx * g.tc;
      const int rows_here = min(g.tr, g.out_h - y0), cols_here = min(g.tc, g.out_w - x0);
      const int eb = g.exp_img ? __ldg(g.exp_img + b) : 0;
      float* cimg = g.C + static_cast<long long>(b) * g.n_out * opix +
                    static_cast<long long>(y0) * g.out_sy * g.out_pitch + static_cast<long long>(x0) * g.out_sx;
      for (int it = half; it < items; it += 2) {
        const int j = it / chunks, c0 = (it - j * chunks) * 32;
        // this lane's output pixel in M block j
        const int n = j * Cfg::BM + q * 32 + lane;
        const int r = n / g.wp, c = n - r * g.wp;
        const bool pix_ok = r < rows_here && c < cols_here;
        const long long pix = static_cast<long long>(r) * g.out_sy * g.out_pitch + static_cast<long long>(c) * g.out_sx;
        // lane e prepares channel c0 + e: bias and the two exact power-of-two factors that undo the operand scalings
        const int oc_own = tn * g.n_tile + c0 + lane;
        const bool oc_ok = oc_own < g.n_out && c0 + lane < g.n_tile;
        const float bias_own = (g.bias && oc_ok) ? __ldg(g.bias + oc_own) : 0.0f;
        float f1_own = 1.0f, f2_own = 1.0f;
        if (g.exp_w && oc_ok) {
          const int ex = __ldg(g.exp_w + oc_own) + eb;
          const int e1 = max(-126, min(127, ex));
          const int e2 = max(-126, min(127, ex - e1));
          f1_own = __int_as_float((e1 + 127) << 23);
          f2_own = __int_as_float((e2 + 127) << 23);
        }
        const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * acc_cols + j * acc_n + c0;
        uint32_t v[32];
        if (c0 + 32 <= g.n_tile) {
          tmem_ld_32x32(t_addr, v);
          if (g.fold) {
            uint32_t v2[32];
            tmem_ld_32x32(t_addr + g.n_tile, v2);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) + __uint_as_float(v2[e]));
          }
        } else {       // n_tile is a multiple of 16: the last chunk may be 16 wide
          uint32_t u[16];
          tmem_ld_32x16(t_addr, u);
          if (g.fold) {
            uint32_t u2[16];
            tmem_ld_32x16(t_addr + g.n_tile, u2);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) u[e] = __float_as_uint(__uint_as_float(u[e]) + __uint_as_float(u2[e]));
          }
#pragma unroll
          for (int e = 0; e < 16; ++e) { v[e] = u[e]; v[16 + e] = 0u; }
        }
        tmem_ld_wait();
        const int oc_lim = min(32, min(g.n_tile - c0, g.n_out - tn * g.n_tile - c0));
        float* cbase = cimg + static_cast<long long>(tn * g.n_tile + c0) * opix + pix;
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const float f1 = __shfl_sync(0xffffffffu, f1_own, e), f2 = __shfl_sync(0xffffffffu, f2_own, e);
          const float bs = __shfl_sync(0xffffffffu, bias_own, e);
          if (pix_ok && e < oc_lim) cbase[static_cast<long long>(e) * opix] = __uint_as_float(v[e]) * f1 * f2 + bs;
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
