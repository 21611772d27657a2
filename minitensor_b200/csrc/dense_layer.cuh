// Dense layer y = act(x W^T + b) and its backward as two entry points that share
// operand preparation between the products (fp16 two-plane mode, pair-tile kernel).
//
// The reference builds the layer from transpose + matmul + add
// (engine/src/nn/dense_layer.rs:139-169) and its backward from MatMulBackward
// (dX = dY W, dW^T = x^T dY; engine/src/autograd/mod/core.rs:743-789), the transpose's
// backward and the bias reduction of AddBackward (core.rs:195-223).  Called one product at a
// time, each of the three products prepares both of its operands (maxima, scaling, two fp16
// planes): 5 passes over dY, 3 over x and 3 over W per backward.  Here
//
//   forward   writes the planes and row exponents of x [M][in] and W [out][in] into a block
//             the caller keeps (`saved`);
//   backward  re-uses those planes as they lie: x~ [b][in] is the MN-major B operand of
//             dW = dY^T x (reduction over b), W~ [o][in] the MN-major B operand of dX = dY W
//             (reduction over o).  Their scales run along the reduction index, so they are folded
//             into dY instead: one pass over dY finds, per row, max_o |dY[b][o]| 2^ew[o], per
//             column, max_b |dY[b][o]| 2^ex[b], and the column sums (the bias gradient); a second
//             pass writes both plane sets of dY.  Neither x nor W is read again.
//
// All scalings are powers of two and exact; the maxima are taken on exponents only (integers),
// so no intermediate can overflow.
#pragma once
#include <climits>

#include "gemm_launch.cuh"
#include "rowcol_kernels.cuh"

namespace mtb {

constexpr int KEY_NONE = INT_MIN / 2;  // exponent key of a zero (or of an empty row/column)

// Layout of the block the forward call leaves for the backward call.
struct DenseSaved {
  size_t off_xp, off_xe, off_wp, off_we, off_flag, total;
  int inp;  // in_features padded to 64
};
inline DenseSaved dense_saved_layout(long long M, long long in, long long out) {
  DenseSaved s;
  s.inp = padded_k(int(in));
  size_t o = 0;
  s.off_xp = o;   o += align_up(size_t(2) * M * s.inp * 2, 1024);
  s.off_xe = o;   o += align_up(sizeof(int) * size_t(M), 1024);
  s.off_wp = o;   o += align_up(size_t(2) * out * s.inp * 2, 1024);
  s.off_we = o;   o += align_up(sizeof(int) * size_t(out), 1024);
  s.off_flag = o; o += 1024;
  s.total = o;
  return s;
}

// flag[0] = 1 when a split kernel of this call met an Inf or NaN operand (the call's flag word holds `epoch`).
static __global__ void save_nonfinite_flag_kernel(const uint32_t* __restrict__ nf_word, uint32_t epoch,
                                                  uint32_t* __restrict__ flag) {
  flag[0] = (*nf_word == epoch) ? 1u : 0u;
}

// One pass over dY [M][N] (row stride ld): rowkey[r] = max_c key(dY[r][c]) + ew[c]  (ROWS only),
// colkey[c] = max_r key(dY[r][c]) + ex[r], partial column sums per band of rows (when part != null).
// A warp owns 256 columns (2 x float4 per lane, each load instruction a contiguous 512 bytes) and walks
// the rows of its band with the next row's loads in flight; a block of 8 warps covers 2048 columns.
// rowkey / colkey must hold KEY_NONE-or-lower before the launch (memset 0x80 bytes does).
template <bool ROWS>
static __global__ void __launch_bounds__(256)
dy_stats_kernel(const float* __restrict__ dy, long long ld, int M, int N, int rows_per_band,
                const int* __restrict__ ex, const int* __restrict__ ew, int* __restrict__ rowkey,
                int* __restrict__ colkey, float* __restrict__ part, const uint32_t* __restrict__ saved_flag,
                uint32_t* __restrict__ nf_word, uint32_t nf_epoch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int Q = 2, E = 4 * Q;                 // float4 loads and elements per lane per row
  const int cw = blockIdx.x * (1024 * Q) + warp * (128 * Q);  // first column of this warp
  const int band = blockIdx.y;
  const int r0 = band * rows_per_band, r1 = min(M, r0 + rows_per_band);
  if (blockIdx.x == 0 && band == 0 && threadIdx.x == 0 && saved_flag && *saved_flag) atomicMax(nf_word, nf_epoch);
  if (cw >= N) return;  // whole warp beyond the last column
  const bool vec_all = ((reinterpret_cast<uintptr_t>(dy) & 15) == 0) && ((ld & 3) == 0) && (cw + 128 * Q <= N);
  auto col_of = [&](int q, int j) { return cw + q * 128 + lane * 4 + j; };
  auto load_row = [&](int r, float (&v)[E]) {
    const float* p = dy + static_cast<long long>(r) * ld;
    if (vec_all) {
#pragma unroll
      for (int q = 0; q < Q; ++q) {
        const float4 t = *reinterpret_cast<const float4*>(p + col_of(q, 0));
        v[q * 4 + 0] = t.x; v[q * 4 + 1] = t.y; v[q * 4 + 2] = t.z; v[q * 4 + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int q = 0; q < Q; ++q)
#pragma unroll
        for (int j = 0; j < 4; ++j) v[q * 4 + j] = (col_of(q, j) < N) ? p[col_of(q, j)] : 0.0f;
    }
  };
  int wk[E], ck[E];
  float cs[E];
#pragma unroll
  for (int q = 0; q < Q; ++q)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      wk[q * 4 + j] = (ROWS && col_of(q, j) < N) ? ew[col_of(q, j)] : 0;
      ck[q * 4 + j] = KEY_NONE;
      cs[q * 4 + j] = 0.0f;
    }
  uint32_t any_bits = 0;  // OR of the exponent fields that were all ones
  float v[E], nv[E];
  if (r0 < r1) load_row(r0, v);
  for (int r = r0; r < r1; ++r) {
    if (r + 1 < r1) load_row(r + 1, nv);
    const int xr = ex[r];
    int rk = KEY_NONE;
#pragma unroll
    for (int i = 0; i < E; ++i) {
      const uint32_t bits = __float_as_uint(v[i]) & 0x7fffffffu;
      // exponent field as the key; subnormals count as 2^-127 (a slightly larger scale than needed)
      const int k = bits ? int(bits >> 23) - 127 : KEY_NONE;
      any_bits |= (bits >= 0x7f800000u) ? 1u : 0u;
      ck[i] = max(ck[i], k + xr);  // KEY_NONE + a few hundred stays far below every real key
      if (ROWS) rk = max(rk, k + wk[i]);
      cs[i] += v[i];
    }
    if (ROWS) {
#pragma unroll
      for (int o = 16; o; o >>= 1) rk = max(rk, __shfl_xor_sync(0xffffffffu, rk, o));
      if (lane == 0 && rk > KEY_NONE / 2) atomicMax(rowkey + r, rk);
    }
#pragma unroll
    for (int i = 0; i < E; ++i) v[i] = nv[i];
  }
  if (any_bits) atomicMax(nf_word, nf_epoch);
#pragma unroll
  for (int q = 0; q < Q; ++q)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = col_of(q, j);
      if (c < N) {
        if (ck[q * 4 + j] > KEY_NONE / 2) atomicMax(colkey + c, ck[q * 4 + j]);
        if (part) part[static_cast<long long>(band) * N + c] = cs[q * 4 + j];
      }
    }
}

// out[c] = sum over bands of part[band][c], in a fixed order: 8 groups of bands per column are summed
// by 8 threads (band g, g + 8, ...) and then folded group 0..7.
static __global__ void __launch_bounds__(256)
colsum_bands_kernel(const float* __restrict__ part, int bands, int N, float* __restrict__ out) {
  __shared__ float red[8][33];
  const int cx = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s = 0.0f;
  if (c < N)
    for (int b = g; b < bands; b += 8) s += part[static_cast<long long>(b) * N + c];
  red[g][cx] = s;
  __syncthreads();
  if (g == 0 && c < N) {
    float t = red[0][cx];
#pragma unroll
    for (int k = 1; k < 8; ++k) t += red[k][cx];
    out[c] = t;
  }
}

// key -> scale exponent: the largest magnitude of the row (column) lands in [2^14, 2^15); 0 when empty.
static __global__ void keys_to_exponents_kernel(int* __restrict__ keys, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) keys[i] = (keys[i] > KEY_NONE / 2) ? keys[i] - 14 : 0;
}

// Second pass over dY: both plane sets, each [2][M][Np] fp16 (Np = N padded to 64, pad written as zero).
//   rows_out (ROWS only): dY[r][c] 2^(ew[c] - er[r])   - the K-major A operand of dX = dY W
//   cols_out (COLS only): dY[r][c] 2^(ex[r] - ec[c])   - the MN-major A operand of dW = dY^T x
// A thread keeps 8 columns (their exponents in registers) and walks the rows of its band.
template <bool ROWS, bool COLS>
static __global__ void __launch_bounds__(256)
dy_split2_kernel(const float* __restrict__ dy, long long ld, int M, int N, int Np, int rows_per_band,
                 const int* __restrict__ ex, const int* __restrict__ ec, const int* __restrict__ ew,
                 const int* __restrict__ er, __half* __restrict__ rows_out, __half* __restrict__ cols_out) {
  const int c0 = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (c0 >= Np) return;
  const int r0 = blockIdx.y * rows_per_band, r1 = min(M, r0 + rows_per_band);
  const long long plane = static_cast<long long>(M) * Np;
  const bool vec = ((reinterpret_cast<uintptr_t>(dy) & 15) == 0) && ((ld & 3) == 0) && (c0 + 8 <= N);
  int ce[8], we[8];
  float fce[8], fwe[8];  // 2^-ec[c], 2^ew[c] as floats (valid when |exponent| <= 63)
  bool small = true;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    ce[j] = (c0 + j < N) ? ec[c0 + j] : 0;
    we[j] = (ROWS && c0 + j < N) ? ew[c0 + j] : 0;
    small &= (abs(ce[j]) <= 63) && (abs(we[j]) <= 63);
    fce[j] = __int_as_float((127 - max(-63, min(63, ce[j]))) << 23);
    fwe[j] = __int_as_float((127 + max(-63, min(63, we[j]))) << 23);
  }
  // Planes of v = x * 2^s with s split into a row and a column part: when both parts are within
  // +-63 the factor 2^s is one exact float product and v one more multiply (zeros, subnormals, Inf and
  // NaN behave as IEEE says); otherwise the general exponent-field route.
  auto emit = [&](const float (&x)[8], bool fast, float frow, const float (&fcol)[8], int srow, const int (&scol)[8],
                  int sign, __half* dst, long long off) {
    __align__(16) __half2 o0[4], o1[4];
    if (fast) {
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        const float v0 = x[j] * (frow * fcol[j]), v1 = x[j + 1] * (frow * fcol[j + 1]);
        const __half2 h = __floats2half2_rn(v0, v1);
        const float2 back = __half22float2(h);
        // Inf - Inf would be NaN: the low plane of a non-finite value is zero
        const float l0 = is_nonfinite(v0) ? 0.0f : v0 - back.x, l1 = is_nonfinite(v1) ? 0.0f : v1 - back.y;
        o0[j >> 1] = h;
        o1[j >> 1] = __floats2half2_rn(l0, l1);
      }
    } else {
      __half a[8], b[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) split2_f16_shift(x[j], sign * (srow - scol[j]), a[j], b[j]);
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        o0[j >> 1] = __halves2half2(a[j], a[j + 1]);
        o1[j >> 1] = __halves2half2(b[j], b[j + 1]);
      }
    }
    *reinterpret_cast<uint4*>(dst + off) = *reinterpret_cast<const uint4*>(o0);
    *reinterpret_cast<uint4*>(dst + plane + off) = *reinterpret_cast<const uint4*>(o1);
  };
  auto load_row = [&](int r, float (&x)[8]) {
    const float* p = dy + static_cast<long long>(r) * ld + c0;
    if (vec) {
      const float4 u = *reinterpret_cast<const float4*>(p);
      const float4 w = *reinterpret_cast<const float4*>(p + 4);
      x[0] = u.x; x[1] = u.y; x[2] = u.z; x[3] = u.w; x[4] = w.x; x[5] = w.y; x[6] = w.z; x[7] = w.w;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = (c0 + j < N) ? p[j] : 0.0f;
    }
  };
  float x[8], nx[8];
  if (r0 < r1) load_row(r0, x);
  for (int r = r0; r < r1; ++r) {
    if (r + 1 < r1) load_row(r + 1, nx);
    const long long off = static_cast<long long>(r) * Np + c0;
    const int xr = ex[r];
    // columns: x * 2^(xr - ce)
    if (COLS)
      emit(x, small && abs(xr) <= 63, __int_as_float((127 + max(-63, min(63, xr))) << 23), fce, xr, ce, 1, cols_out, off);
    if (ROWS) {
      const int rr = er[r];
      // rows: x * 2^(we - rr)
      emit(x, small && abs(rr) <= 63, __int_as_float((127 - max(-63, min(63, rr))) << 23), fwe, rr, we, -1, rows_out, off);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = nx[j];
  }
}

// The pair-tile kernel serves a product when its output is more than one CTA tile in both directions.
inline bool dense_fused_shapes(long long M, long long in, long long out) {
  return M > 128 && in > 128 && out > 128;
}

// Gated IEEE redo of C = op(A) op(B) for operands that held Inf / NaN (returns at once otherwise).
inline int32_t launch_nonfinite_redo(mtb200_ctx* h, bool trans_a, bool trans_b, int M, int N, int K, const float* A,
                                     const float* B, float* C, const float* bias, int epilogue, const float* aux,
                                     const uint32_t* nf_word) {
  StridedGemmArgs s;
  s.M = M; s.N = N; s.K = K; s.batch = 1;
  s.A = A; s.B = B; s.C = C;
  s.a_si = trans_a ? 1 : K;  s.a_sk = trans_a ? M : 1;  s.a_sb = 0;
  s.b_sk = trans_b ? 1 : N;  s.b_sj = trans_b ? K : 1;  s.b_sb = 0;
  s.ldc = N; s.c_sb = 0;
  s.bias = bias; s.aux = aux; s.epilogue = epilogue;
  s.gate = nf_word; s.gate_value = MTB_FLAG_SET;
  const long long tiles = static_cast<long long>((M + 127) / 128) * ((N + 127) / 128);
  gemm_simt_kernel<float, 8, 8><<<dim3(unsigned(tiles), 1), 256, 0, h->stream>>>(s);
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

// y = epilogue(x W^T + bias); planes and exponents of x and W go to `saved`.
inline int32_t dense_forward_f32(mtb200_ctx* h, int M, int in, int out, const float* x, const float* W,
                                 const float* bias, int epilogue, const float* aux, float* y, void* saved) {
  const DenseSaved L = dense_saved_layout(M, in, out);
  char* sv = static_cast<char*>(saved);
  __half* xp = reinterpret_cast<__half*>(sv + L.off_xp);
  int* xe = reinterpret_cast<int*>(sv + L.off_xe);
  __half* wp = reinterpret_cast<__half*>(sv + L.off_wp);
  int* we = reinterpret_cast<int*>(sv + L.off_we);
  uint32_t* flag = reinterpret_cast<uint32_t*>(sv + L.off_flag);
  uint32_t* nf_word = nullptr;
  int32_t rc = call_flag_begin(h, &nf_word);
  if (rc) return rc;
  const uint32_t epoch = MTB_FLAG_SET;
  if ((double(M) + double(out)) * in <= 2.2e6 && prep16_pair_eligible(x, true, in, 1, 0) &&
      prep16_pair_eligible(W, true, in, 1, 0)) {
    rc = launch_prep16_pair(h, prep16_operand(h, x, true, M, in, 1, 0, xp, xe),
                            prep16_operand(h, W, true, out, in, 1, 0, wp, we), nf_word, epoch);
    if (rc) return rc;
  } else {
    rc = launch_split16(h, x, true, M, in, 1, 0, xp, xe, nf_word, epoch);
    if (rc) return rc;
    rc = launch_split16(h, W, true, out, in, 1, 0, wp, we, nf_word, epoch);
    if (rc) return rc;
  }
  save_nonfinite_flag_kernel<<<1, 1, 0, h->stream>>>(nf_word, epoch, flag);
  SplitOperand oa{reinterpret_cast<const __nv_bfloat16*>(xp), M, 0, 1, 0, L.inp, 2, xe};
  SplitOperand ob{reinterpret_cast<const __nv_bfloat16*>(wp), out, 0, 1, 0, L.inp, 2, we};
  rc = run_split_gemm(h, oa, ob, L.inp, 1, M, out, y, out, 0, bias, epilogue, aux, 23, 5, 0, 0, 0, in);
  if (rc) return rc;
  return launch_nonfinite_redo(h, false, true, M, out, in, x, W, y, bias, epilogue, aux, nf_word);
}

// Layout of the optional block that carries dY's weight-gradient operand from one backward call to a later one
// (dy_mode 1 writes it, dy_mode 2 consumes it): column-scaled planes [2][M][outp], their exponents, a non-finite flag.
struct DenseDy {
  size_t off_planes, off_ec, off_flag, total;
};
inline DenseDy dense_dy_layout(long long M, long long out) {
  DenseDy d;
  size_t o = 0;
  d.off_planes = o; o += align_up(size_t(2) * M * padded_k(int(out)) * 2, 1024);
  d.off_ec = o;     o += align_up(sizeof(int) * size_t(out), 1024);
  d.off_flag = o;   o += 1024;
  d.total = o;
  return d;
}

// nf_word = epoch when either flag word is set (the operands of an earlier call held Inf / NaN)
static __global__ void raise_nonfinite_kernel(const uint32_t* __restrict__ flag_a, const uint32_t* __restrict__ flag_b,
                                              uint32_t* __restrict__ nf_word, uint32_t epoch) {
  if ((flag_a && *flag_a) || (flag_b && *flag_b)) atomicMax(nf_word, epoch);
}

// dX = epilogue(dY W) (nullable), dW = dY^T x (nullable), db = column sums of dY (nullable), from the block a forward
// call of the same shapes left in `saved`.  x and W themselves are read only by the Inf / NaN redo.
// dy_mode 1 (dW null): the weight-gradient operand of dY is prepared all the same and left in dy_block;
// dy_mode 2 (dX null): dy_block holds it and dY is not read at all (db must have been taken by the earlier call).
inline int32_t dense_backward_f32(mtb200_ctx* h, int M, int in, int out, const float* x, const float* W,
                                  const float* dY, const void* saved, float* dX, int epilogue, const float* aux,
                                  float* dW, float* db, void* dy_block = nullptr, int dy_mode = 0) {
  const DenseSaved L = dense_saved_layout(M, in, out);
  const char* sv = static_cast<const char*>(saved);
  const __half* xp = reinterpret_cast<const __half*>(sv + L.off_xp);
  const int* xe = reinterpret_cast<const int*>(sv + L.off_xe);
  const __half* wp = reinterpret_cast<const __half*>(sv + L.off_wp);
  const int* we = reinterpret_cast<const int*>(sv + L.off_we);
  const uint32_t* flag = reinterpret_cast<const uint32_t*>(sv + L.off_flag);
  const int outp = padded_k(out);
  const DenseDy D = dense_dy_layout(M, out);
  char* dyb = static_cast<char*>(dy_block);
  const bool keep_cols = dy_mode == 1 && dy_block;   // write the column planes into the block
  const bool have_cols = dy_mode == 2 && dy_block;   // read them from the block
  const bool want_cols = dW != nullptr || keep_cols; // this call prepares column planes

  const int col_blocks = (out + 2047) / 2048;
  int bands = std::max(1, std::min((M + 15) / 16, (h->sm_count * 4) / col_blocks));
  bands = std::min(bands, 512);  // the second colsum stage reads `bands` partials per column
  int rows_per_band = (M + bands - 1) / bands;
  bands = (M + rows_per_band - 1) / rows_per_band;
  const size_t bytes_planes = align_up(size_t(2) * M * outp * 2, 1024);
  const size_t bytes_er = align_up(sizeof(int) * size_t(M), 1024);
  const size_t bytes_ec = align_up(sizeof(int) * size_t(out), 1024);
  const size_t bytes_zero = align_up(sizeof(int) * size_t(in), 1024);
  const size_t bytes_part = db ? align_up(sizeof(float) * size_t(bands) * out, 1024) : 0;
  const int ws_sets = (dX ? 1 : 0) + ((want_cols && !keep_cols && !have_cols) ? 1 : 0);
  void* ws = nullptr;
  int32_t rc = workspace_reserve(h, ws_sets * bytes_planes + bytes_er + bytes_ec + bytes_zero + bytes_part, &ws);
  if (rc) return rc;
  char* base = static_cast<char*>(ws);
  const bool cols_in_ws = want_cols && !keep_cols && !have_cols;
  __half* pc = (keep_cols || have_cols) ? reinterpret_cast<__half*>(dyb + D.off_planes)
                                        : (cols_in_ws ? reinterpret_cast<__half*>(base) : nullptr);   // column-scaled planes (dW)
  __half* pr = dX ? reinterpret_cast<__half*>(base + (cols_in_ws ? bytes_planes : 0)) : nullptr;      // row-scaled planes (dX)
  char* q = base + ws_sets * bytes_planes;
  int* er = reinterpret_cast<int*>(q);
  int* ec_ws = reinterpret_cast<int*>(q + bytes_er);
  int* ec = (keep_cols || have_cols) ? reinterpret_cast<int*>(dyb + D.off_ec) : ec_ws;
  int* zero = reinterpret_cast<int*>(q + bytes_er + bytes_ec);
  float* part = db ? reinterpret_cast<float*>(q + bytes_er + bytes_ec + bytes_zero) : nullptr;
  uint32_t* dy_flag = dy_block ? reinterpret_cast<uint32_t*>(dyb + D.off_flag) : nullptr;

  uint32_t* nf_word = nullptr;
  rc = call_flag_begin(h, &nf_word);
  if (rc) return rc;
  const uint32_t epoch = MTB_FLAG_SET;
  MTB_CUDA(cudaMemsetAsync(zero, 0, bytes_zero, h->stream));
  if (have_cols) {
    // nothing of dY is read: only the Inf / NaN state of the earlier calls is carried over
    raise_nonfinite_kernel<<<1, 1, 0, h->stream>>>(flag, dy_flag, nf_word, epoch);
    MTB_CUDA(cudaGetLastError());
  } else {
    // maxima + column sums: one read of dY; the plane sets: one more read and one write per set
    const int nsets = (dX ? 1 : 0) + (want_cols ? 1 : 0);
    ProfScope prof(h, PROF_SPLIT, double(M) * (8.0 * out + 4.0 * nsets * outp));
    MTB_CUDA(cudaMemsetAsync(er, 0x80, bytes_er, h->stream));  // every key far below KEY_NONE / 2
    MTB_CUDA(cudaMemsetAsync(ec, 0x80, sizeof(int) * size_t(out), h->stream));
    if (dX)
      dy_stats_kernel<true><<<dim3(col_blocks, bands), 256, 0, h->stream>>>(dY, out, M, out, rows_per_band, xe, we, er,
                                                                            ec, part, flag, nf_word, epoch);
    else
      dy_stats_kernel<false><<<dim3(col_blocks, bands), 256, 0, h->stream>>>(dY, out, M, out, rows_per_band, xe,
                                                                             nullptr, nullptr, ec, part, flag,
                                                                             nf_word, epoch);
    if (dX) keys_to_exponents_kernel<<<(M + 255) / 256, 256, 0, h->stream>>>(er, M);
    keys_to_exponents_kernel<<<(out + 255) / 256, 256, 0, h->stream>>>(ec, out);
    if (db) colsum_bands_kernel<<<(out + 31) / 32, 256, 0, h->stream>>>(part, bands, out, db);
    if (keep_cols) save_nonfinite_flag_kernel<<<1, 1, 0, h->stream>>>(nf_word, epoch, dy_flag);
    const int sp_cols = (outp / 8 + 255) / 256;
    const int sp_bands = std::max(1, std::min(M, (h->sm_count * 8 + sp_cols - 1) / sp_cols));
    const int sp_rows = (M + sp_bands - 1) / sp_bands;
    const dim3 sp_grid(sp_cols, (M + sp_rows - 1) / sp_rows);
    if (dX && want_cols)
      dy_split2_kernel<true, true><<<sp_grid, 256, 0, h->stream>>>(dY, out, M, out, outp, sp_rows, xe, ec, we, er, pr, pc);
    else if (dX)
      dy_split2_kernel<true, false><<<sp_grid, 256, 0, h->stream>>>(dY, out, M, out, outp, sp_rows, xe, ec, we, er, pr, nullptr);
    else if (want_cols)
      dy_split2_kernel<false, true><<<sp_grid, 256, 0, h->stream>>>(dY, out, M, out, outp, sp_rows, xe, ec, nullptr, nullptr, nullptr, pc);
    MTB_CUDA(cudaGetLastError());
  }
  // dW [out][in] = dY^T x: A = column-scaled dY planes (MN-major, reduction over the batch rows),
  // B = the forward pass's x planes, also MN-major here; their row scales are already inside A.
  if (dW) {
    SplitOperand oa{reinterpret_cast<const __nv_bfloat16*>(pc), M, 0, 1, 1, outp, 2, ec};
    SplitOperand ob{reinterpret_cast<const __nv_bfloat16*>(xp), M, 0, 1, 1, L.inp, 2, zero};
    rc = run_split_gemm(h, oa, ob, padded_k(M), 1, out, in, dW, in, 0, nullptr, EPI_NONE, nullptr, 23, 5, 0, 0, 0, M);
    if (rc) return rc;
    rc = launch_nonfinite_redo(h, true, false, out, in, M, dY, x, dW, nullptr, EPI_NONE, nullptr, nf_word);
    if (rc) return rc;
  }
  // dX [M][in] = dY W: A = row-scaled dY planes (K-major), B = the forward pass's W planes (MN-major here).
  if (dX) {
    SplitOperand oa{reinterpret_cast<const __nv_bfloat16*>(pr), M, 0, 1, 0, outp, 2, er};
    SplitOperand ob{reinterpret_cast<const __nv_bfloat16*>(wp), out, 0, 1, 1, L.inp, 2, zero};
    rc = run_split_gemm(h, oa, ob, outp, 1, M, in, dX, in, 0, nullptr, epilogue, aux, 23, 5, 0, 0, 0, out);
    if (rc) return rc;
    rc = launch_nonfinite_redo(h, false, false, M, in, out, dY, W, dX, nullptr, epilogue, aux, nf_word);
    if (rc) return rc;
  }
  return MTB200_OK;
}

}  // namespace mtb
