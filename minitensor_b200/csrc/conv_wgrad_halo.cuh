// Weight gradient of a stride-1 convolution from ONE staged image block per step (fp16 two-plane mode).
//
//   dW[oc][(tap, ic)] = sum over k = (image, oh, ow) of dy[k][oc] * x[k shifted by tap][ic]
//
// (engine/src/autograd/mod/shape.rs:130-169 computes the same sums with scalar loops.)
//
// conv_wgrad_umma.cuh loads, for every tap, its own shifted window of x: nine loads of nearly the same pixels for a
// 3 x 3 filter, and the TMA engine - about 4 ns per 128-byte row it writes - is what bounds that kernel.  Here a step
// is a block of tr output rows of one image.  The producer loads
//   * the halo block of x: {64 channels, wp = ow + kw - 1 columns, tr + kh - 1 rows} from (-pad_w, y0 - pad_h), and
//   * the block of dy:     {64 channels, wp columns, tr rows} from (0, y0) - its columns ow .. wp-1 lie outside the
//     tensor and read as zero,
// both as [pixel][64 channels] rows of 128 bytes in raster order with the SAME pitch wp.  Output pixel (r, c) is
// reduction index q = r * wp + c in the dy block, and its partner under tap (fh, fw) is row q + fh * wp + fw of the
// halo block.  Both blocks are MN-major operands (the reduction index walks down the rows), so the x operand of a tap
// is the halo block's descriptor with the start address advanced by fh * wp + fw rows (the swizzle is a function of
// the shared-memory address, so a start that is not aligned to the 8-row repeat reads the rows it names).  The q that
// are not output pixels (c >= ow, and the rows that pad a block to a multiple of 16) meet zeros in the dy block.
//
// Orientation.  M = 128 = TWO taps x 64 input channels: the x operand's two 64-channel chunks are the same halo block
// at two different row shifts, which is what the descriptor's leading-dimension offset expresses (offset = the
// difference of the two taps' shifts).  N = 64 output channels (the dy block).  One accumulator of 64 TMEM columns
// per tap pair, all of them live for the CTA's whole range of steps; lanes = (tap of the pair, input channel),
// columns = output channel.  A CTA owns (block of 64 output channels, block of 64 input channels, group of up to 8
// tap pairs, range of steps) and writes its accumulators to part[range][oc][(tap, ic)]; wgrad_reduce_kernel adds
// the ranges in order.
//
// Strides.  For a strided convolution the x planes are stored as sh * sw phase images (split_f16.cuh, RowPhases):
// output pixel (oy, ox) under tap (fh, fw) reads phase ((fh - pad_h) mod sh, (fw - pad_w) mod sw) at
// (oy + floor((fh - pad_h) / sh), ox + floor((fw - pad_w) / sw)) - a stride-1 window again.  The halo block then has
// a phase dimension (one 5-D load), and a tap's row shift is phase * (rows of one phase's block) + the shift inside
// it; nothing else changes.  Stride 1 is the one-phase case of the same formulas.
//
// (Tried and dropped: running x_hi*dy_hi and x_hi*dy_lo as one MMA of N = 128 whose dy operand takes its second
// 64-channel chunk from the lo plane, as the forward kernel folds its weight planes.  With these MN-major operands
// the kernel went from 146 to 216 us at the large conv config.)
//
// Roles: warp 0 producer, warp 1 TMEM owner and MMA issuer, warps 2..5 epilogue.  Every wait is bounded and reports
// through the status word (role codes 0x1.. - 0x3.., site 6).
#pragma once
#include "gemm_split_umma.cuh"
#include "ptx_sm100.cuh"

namespace mtb {

struct WgradHaloArgs {
  int c_out, n_total;        // output channels; row length of a partial = taps * cin_p
  int cb_per_tap;            // cin_p / 64
  int kh, kw, pad_h, pad_w;
  int sh, sw;                // strides (1, 1: one phase)
  int org_x, org_y;          // halo origin relative to the step's first output pixel, in phase-image coordinates
  int hh;                    // rows of one phase's halo block: tr + reach of the taps
  int oh;                    // output rows per image
  int tr, wp;                // output rows per step; pitch = output width + reach of the taps
  int ksteps;                // ceil(tr * wp / 16): MMAs of 16 reduction indices per (step, tap pair, product)
  int steps_per_image;       // ceil(oh / tr)
  int total_steps;           // images * steps_per_image
  int splits;                // ranges the steps are cut into (grid = items * splits)
  int ocbs, icbs, tgs;       // blocks of 64 output / input channels, tap groups
  int taps_per_group;        // even, <= 16
  uint32_t x_plane_bytes;    // shared memory per x plane of a stage (multiple of 1024)
  uint32_t dy_plane_bytes;   // shared memory per dy plane of a stage (multiple of 1024)
  float* part;               // [splits][c_out][n_total]
  uint32_t* status;
};

struct WgradHaloCfg {
  static constexpr int STAGES = 2, NUM_THREADS = 192, TMEM_COLS = 512, MAX_UNITS = 8;
  static constexpr int BAR_BYTES = 256;
  static size_t smem_bytes(size_t x_plane_bytes, size_t dy_plane_bytes) {
    return 1024 + size_t(STAGES) * 2 * (x_plane_bytes + dy_plane_bytes) + BAR_BYTES;
  }
};

__global__ void __launch_bounds__(192, 1)
conv_wgrad_halo_kernel(const __grid_constant__ CUtensorMap tmapDy, const __grid_constant__ CUtensorMap tmapX,
                       const WgradHaloArgs g) {
  using Cfg = WgradHaloCfg;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t ring = (raw + 1023u) & ~1023u;
  const uint32_t stage_bytes = 2 * (g.x_plane_bytes + g.dy_plane_bytes);
  const uint32_t bars = ring + Cfg::STAGES * stage_bytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (Cfg::STAGES + s); };
  const uint32_t acc_full = bars + 8u * (2 * Cfg::STAGES);
  const uint32_t tmem_slot = bars + 8u * (2 * Cfg::STAGES + 1);
  const uint32_t abort_addr = tmem_slot + 4u;
  volatile uint32_t* abort_word = reinterpret_cast<volatile uint32_t*>(smem_raw + (abort_addr - raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - raw));
  // unit_lo[u]: what tap pair u adds to the low word of the x descriptor - the first tap's row shift in the start
  // address field (16-byte units) and the distance to the second tap's rows in the leading-offset field
  uint32_t* unit_lo = reinterpret_cast<uint32_t*>(smem_raw + (bars + 128u - raw));
  uint32_t* unit_swap = unit_lo + Cfg::MAX_UNITS;   // 1: lanes 0..63 of the pair hold its SECOND tap

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x / g.splits, z = blockIdx.x - item * g.splits;
  const int tg = item % g.tgs, icb = (item / g.tgs) % g.icbs, ocb = item / (g.tgs * g.icbs);
  const int taps = g.kh * g.kw;
  const int tap0 = tg * g.taps_per_group, tap_end = min(taps, tap0 + g.taps_per_group);
  const int units = (tap_end - tap0 + 1) / 2;
  const int per = (g.total_steps + g.splits - 1) / g.splits;
  const int step_begin = min(g.total_steps, z * per), step_end = min(g.total_steps, step_begin + per);
  const bool has_work = step_begin < step_end;

  // The rows past a block's box are read by the MMAs (padding of the reduction to 16, the reach of the last taps) and
  // no load ever writes them: they must hold finite values, so the whole ring starts as zeros.
  {
    uint4* p = reinterpret_cast<uint4*>(smem_raw + (ring - raw));
    const uint32_t n16 = (Cfg::STAGES * stage_bytes) >> 4;
    for (uint32_t i = threadIdx.x; i < n16; i += blockDim.x) p[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  const int phases = g.sh * g.sw;
  if (threadIdx.x < units) {
    auto shift_of = [&](int tap) {       // halo row of the tap's window for the step's first output pixel
      const int fh = tap / g.kw, fw = tap - fh * g.kw;
      const int ay = fh - g.pad_h, ax = fw - g.pad_w;
      const int py = ((ay % g.sh) + g.sh) % g.sh, px = ((ax % g.sw) + g.sw) % g.sw;
      const int dy = (ay - py) / g.sh - g.org_y, dx = (ax - px) / g.sw - g.org_x;      // exact divisions
      return (py * g.sw + px) * (g.hh * g.wp) + dy * g.wp + dx;
    };
    const int ta = tap0 + 2 * threadIdx.x, tb = min(ta + 1, tap_end - 1);
    int off_a = shift_of(ta), off_b = shift_of(tb);
    // with phases the second tap's rows may lie before the first's; the leading offset is kept non-negative by
    // letting the pair's lanes swap roles (the epilogue reads the flag)
    const bool swap = off_b < off_a;
    if (swap) { const int t = off_a; off_a = off_b; off_b = t; }
    unit_swap[threadIdx.x] = swap ? 1u : 0u;
    unit_lo[threadIdx.x] = (static_cast<uint32_t>(off_b - off_a) * 8u) << 16 | static_cast<uint32_t>(off_a) * 8u;
  }
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
  fence_proxy_async_smem();      // the zeros are ordered before the TMA writes that follow
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  grid_dependency_wait();        // the planes come from the kernels before this one
  grid_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------ producer: one x halo block and one dy block per step
    if (lane == 0 && has_work) {
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t tx = 2u * static_cast<uint32_t>(g.wp) * 128u * static_cast<uint32_t>(phases * g.hh + g.tr);
      for (int st = step_begin; st < step_end; ++st) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_word)) {
          *abort_word = 1;
          atomicMax(g.status, 0x100u | 6u);
          break;
        }
        const int img = st / g.steps_per_image;
        const int y0 = (st - img * g.steps_per_image) * g.tr;
        mbar_expect_tx(full_bar(stage), tx);
        const uint32_t sx = ring + stage * stage_bytes;
        const uint32_t sd = sx + 2 * g.x_plane_bytes;
        for (int s = 0; s < 2; ++s) {
          if (phases == 1)
            tma_load_4d(sx + s * g.x_plane_bytes, &tmapX, full_bar(stage), icb * 64, g.org_x, y0 + g.org_y, img * 2 + s);
          else   // {c, x, y, phase, plane}: every phase image's halo block in one request
            tma_load_5d(sx + s * g.x_plane_bytes, &tmapX, full_bar(stage), icb * 64, g.org_x, y0 + g.org_y, 0, img * 2 + s);
          tma_load_4d(sd + s * g.dy_plane_bytes, &tmapDy, full_bar(stage), ocb * 64, 0, y0, img * 2 + s);
        }
        if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && has_work) {
      const uint32_t idesc = make_idesc(128, 64, /*f16*/ 0u, /*f32*/ 1u, /*a MN-major*/ 1u, /*b MN-major*/ 1u);
      const uint64_t proto = make_mnmajor_desc(0, 0);
      const uint32_t d_hi = static_cast<uint32_t>(proto >> 32);
      const uint32_t x_plane16 = g.x_plane_bytes >> 4, dy_plane16 = g.dy_plane_bytes >> 4;
      int stage = 0;
      uint32_t phase = 0;
      bool first = true;
      for (int st = step_begin; st < step_end; ++st) {
        if (!mbar_wait(full_bar(stage), phase, abort_word)) {
          *abort_word = 1;
          atomicMax(g.status, 0x200u | 6u);
          break;
        }
        tc_fence_after();
        const uint32_t sx = ring + stage * stage_bytes;
        const uint32_t x_lo = (sx & 0x3FFFFu) >> 4;
        const uint32_t d_lo = ((sx + 2 * g.x_plane_bytes) & 0x3FFFFu) >> 4;
        for (int kk = 0; kk < g.ksteps; ++kk) {
          const uint32_t krow16 = static_cast<uint32_t>(kk) * 128u;     // 16 rows of 128 bytes, in 16-byte units
          const uint32_t b_hi_lo = d_lo + krow16, b_lo_lo = b_hi_lo + dy_plane16;
          const uint32_t overwrite = (first && kk == 0) ? 0u : 1u;
          for (int u = 0; u < units; ++u) {
            const uint32_t a_hi_lo = x_lo + unit_lo[u] + krow16, a_lo_lo = a_hi_lo + x_plane16;
            const uint32_t d = tmem_base + u * 64;
            // small products first: x_hi * dy_lo, x_lo * dy_hi, then x_hi * dy_hi
            umma_f16_lohi(d, a_hi_lo, d_hi, b_lo_lo, d_hi, idesc, overwrite);
            umma_f16_lohi(d, a_lo_lo, d_hi, b_hi_lo, d_hi, idesc, 1u);
            umma_f16_lohi(d, a_hi_lo, d_hi, b_hi_lo, d_hi, idesc, 1u);
          }
        }
        first = false;
        umma_commit<1>(empty_bar(stage));
        if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1u; }
      }
      umma_commit<1>(acc_full);
    }
  } else {
    // ------------------------------------------------------------ epilogue: the accumulators, once
    const int q = warp & 3;
    const int slot = q >> 1, ic = (q & 1) * 32 + lane;       // lane quarter -> (tap of the pair, input channel)
    bool ready = has_work;
    if (has_work && !mbar_wait(acc_full, 0, abort_word)) {
      *abort_word = 1;
      if (lane == 0) atomicMax(g.status, 0x300u | 6u);
      ready = false;
    }
    if (ready) tc_fence_after();
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const int oc_here = min(64, g.c_out - ocb * 64);
    for (int u = 0; u < units; ++u) {
      const int tap = tap0 + 2 * u + (slot ^ int(unit_swap[u]));
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t v[32];
        if (ready) {
          tmem_ld_32x32(t_row + u * 64 + c0, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;    // a range without steps contributes zeros
        }
        if (tap < tap_end) {
          float* dst = g.part + (static_cast<long long>(z) * g.c_out + ocb * 64 + c0) * g.n_total +
                       (static_cast<long long>(tap) * g.cb_per_tap + icb) * 64 + ic;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c0 + j < oc_here) dst[static_cast<long long>(j) * g.n_total] = __uint_as_float(v[j]);   // 32 lanes = 128 contiguous bytes
        }
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

}  // namespace mtb
