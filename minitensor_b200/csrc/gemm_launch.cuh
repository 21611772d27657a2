// Host-side launch of the split-bf16 GEMM: operand preparation into scratch
// memory, tensor maps, tile-shape choice, kernel launch.
#pragma once
#include "mtb200_core.cuh"
#include "gemm_split_umma.cuh"
#include "gemm_split_umma2.cuh"
#include "split_bf16.cuh"
#include "split_f16.cuh"
#include "prep_f16.cuh"
#include "gemm_f64_int.cuh"
#include <algorithm>
#include <cstdlib>

namespace mtb {

// One prepared operand: bf16 split planes [planes = 3*batch][rows][cols padded to 64].
// K-major (default): rows index M or N, columns index K (the pad is zero).
// MN-major: rows index K, columns index M or N (straight split of a [K][MN] matrix).
struct SplitOperand {
  const __nv_bfloat16* base = nullptr;
  int rows = 0;
  int batched = 0;  // 0: a single matrix shared by every batch entry
  int batch = 1;
  int mn_major = 0;
  int cols_p = 0;   // padded column count of the planes (MN-major operands; K-major use Kp)
  int nplanes = 3;  // planes per matrix: 3 (bf16 split) or 2 (fp16 split)
  const int* expo = nullptr;  // fp16 split: scale exponent per M/N index ([batch][rows or cols])
};

inline int padded_k(int K) { return (K + 63) / 64 * 64; }
// f32 products with a reduction of at most SMALL_GEMM_K and at most SMALL_GEMM_MACS multiply-adds take the
// single-launch CUDA-core path: measured 11-15 us against 20-29 us for split + tensor kernel + gate on such shapes
// (the small MLP's backward products); with longer reductions that kernel's serial K loop loses.
constexpr double SMALL_GEMM_MACS = 4.0e6;
constexpr int SMALL_GEMM_K = 64;
inline size_t split_bytes(int rows, int Kp, int batch) {
  return align_up(size_t(3) * batch * rows * Kp * sizeof(__nv_bfloat16), 1024);
}

// Write the three bf16 planes of a row-major f32 operand.  `trans` = the
// source is [K][rows] rather than [rows][K].
inline int32_t launch_split(mtb200_ctx* h, const float* src, bool trans, int rows, int K, int Kp,
                            int batch, long long bstride, __nv_bfloat16* dst, int nsplit,
                            uint32_t* nf_word = nullptr, uint32_t nf_epoch = 0) {
  ProfScope prof(h, PROF_SPLIT, double(batch) * rows * (4.0 * K + 2.0 * nsplit * Kp));
  if (!trans) {
    const long long total = static_cast<long long>(rows) * (Kp / 8);
    const int blocks = int(std::min<long long>((total + 255) / 256, (long long)h->sm_count * 32));
    split_rows_kernel<<<dim3(blocks, 1, batch), 256, 0, h->stream>>>(src, K, bstride, dst, rows, K, Kp, nsplit,
                                                                     nf_word, nf_epoch);
  } else {
    split_cols_kernel<<<dim3((rows + 63) / 64, Kp / 64, batch), 256, 0, h->stream>>>(
        src, rows, bstride, dst, rows, K, Kp, nsplit, nf_word, nf_epoch);
  }
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

template <int BN, int BK, int STAGES>
inline int32_t launch_variant(mtb200_ctx* h, const SplitOperand& a, const SplitOperand& b, int Kp,
                              GemmArgs g) {
  using Cfg = GemmCfg<BN, BK, STAGES>;
  auto kern = gemm_split_umma_kernel<BN, BK, STAGES>;
  // per-device attribute; setting it on every launch keeps multi-device processes correct
  if (int32_t rc_attr = grant_dynamic_smem(h, kern, int(Cfg::SMEM_BYTES))) return rc_attr;
  CUtensorMap ta, tb;
  int32_t rc = make_split_tmap(&ta, a.base, Kp, a.rows, uint64_t(a.nplanes) * a.batch, BK, Cfg::BM);
  if (rc) return rc;
  rc = make_split_tmap(&tb, b.base, Kp, b.rows, uint64_t(b.nplanes) * b.batch, BK, BN);
  if (rc) return rc;
  // split-K arguments count 64-wide K blocks; rescale to this variant's block
  g.num_kb = g.num_kb ? g.num_kb * (64 / BK) : Kp / BK;
  g.kb_batch_stride *= (64 / BK);
  const long long tiles = static_cast<long long>((g.M + Cfg::BM - 1) / Cfg::BM) * ((g.N + BN - 1) / BN) * g.batch;
  const int grid = int(std::min<long long>(tiles, h->sm_count));
  ProfScope prof(h, PROF_GEMM_UMMA, 2.0 * g.M * g.N * double(g.num_kb) * BK * g.batch);
  kern<<<grid, Cfg::NUM_THREADS, Cfg::SMEM_BYTES, h->stream>>>(ta, tb, g);
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

// 4-D view {64, k, mn/64, plane} of MN-major planes [plane][k rows][cols_p]; box = 64 x bk x chunks x 1.
inline int32_t make_split_tmap_mn(CUtensorMap* out, const void* base, uint64_t k_rows, uint64_t cols_p,
                                  uint64_t planes, uint32_t bk, uint32_t chunks) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return fail(MTB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[4] = {64, k_rows, cols_p / 64, planes};
  const cuuint64_t strides[3] = {cols_p * 2, 128, k_rows * cols_p * 2};
  const cuuint32_t box[4] = {64, bk, chunks, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(MTB200_ERR_CUDA, "cuTensorMapEncodeTiled (MN-major) failed (%d) for k %llu cols %llu planes %llu",
                int(r), (unsigned long long)k_rows, (unsigned long long)cols_p, (unsigned long long)planes);
  return MTB200_OK;
}

// allow_tail: the kernel walks K blocks of 64 and may split the tiles of a short last round (GemmArgs::tail_splits).
// Launch with the programmatic-stream-serialization attribute: the kernel may start while the one before it in the
// stream still runs and must call grid_dependency_wait() before it reads that kernel's results (ptx_sm100.cuh).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_on(mtb200_ctx* h, cudaStream_t stream, void (*kern)(KArgs...), dim3 grid, dim3 block,
                                 size_t smem, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cfg.attrs = attr; cfg.numAttrs = h->pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(mtb200_ctx* h, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
  return launch_pdl_on(h, h->stream, kern, grid, block, smem, std::forward<Args>(args)...);
}

template <typename Kern>
inline int32_t launch_pair_kernel(mtb200_ctx* h, Kern kern, int smem_bytes, int threads, long long tiles,
                                  const CUtensorMap& ta, const CUtensorMap& tb, GemmArgs g, double work,
                                  bool allow_tail = false, int prof_class = PROF_GEMM_UMMA) {
  if (int32_t rc_attr = grant_dynamic_smem(h, kern, int(smem_bytes))) return rc_attr;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = h->stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;      // the occupancy query below takes the cluster shape only
  const int sms = (h->gemm_sm_limit > 0) ? std::min(h->gemm_sm_limit, h->sm_count) : h->sm_count;
  cfg.gridDim = dim3(2 * (sms / 2));
  // clusters of this kernel the device can hold at once: asked once per kernel and SM limit
  const void* occ_key = reinterpret_cast<const char*>(reinterpret_cast<const void*>(kern)) + sms;
  int max_clusters = 0;
  auto occ = h->cluster_occupancy.find(occ_key);
  if (occ != h->cluster_occupancy.end()) {
    max_clusters = occ->second;
  } else {
    if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess || max_clusters <= 0) {
      cudaGetLastError();
      max_clusters = sms / 2;
    }
    h->cluster_occupancy[occ_key] = max_clusters;
  }
  const int max_pairs = std::min(max_clusters, sms / 2);
  int pairs = int(std::min<long long>(tiles, max_pairs));
  // A partial last round costs a whole tile time whatever its size.  Cutting each of its `rem` tiles into s K ranges
  // and dealing the rem * s shorter items out over the pairs costs ceil(rem * s / pairs) / s of a tile time plus the
  // partial-sum traffic and the fix-up kernel (4096^3: 256 tiles on 74 pairs, 34 tail tiles -> 68 half tiles, half a
  // tile time; 8192 x 4096 per rank on 70 pairs: 46 tail tiles -> 138 thirds in two short rounds, two thirds).  An
  // output of fewer tiles than pairs is all tail.
  g.tail_splits = 0;
  if (allow_tail && tiles <= 0x3fffffff) {
    const int rem = tiles > pairs ? int(tiles % pairs) : int(tiles);
    int splits = 0;
    double best = 0.88;     // take a split only when it saves at least an eighth of a tile time
    for (int s2 = 2; rem && s2 <= 6 && g.num_kb >= 4 * s2; ++s2) {
      const double t = double((static_cast<long long>(rem) * s2 + max_pairs - 1) / max_pairs) / s2 + 0.03 * s2;
      if (t < best - 1e-9) { best = t; splits = s2; }
    }
    if (splits >= 2) {
      const size_t slots = size_t(rem) * splits;
      if (slots > h->tail_partial_slots) {
        MTB_CUDA(cudaStreamSynchronize(h->stream));
        if (h->tail_partial) MTB_CUDA(cudaFree(h->tail_partial));
        h->tail_partial = nullptr;
        h->tail_partial_slots = 0;
        const size_t want = std::max(slots, size_t(h->sm_count));
        MTB_CUDA(cudaMalloc(reinterpret_cast<void**>(&h->tail_partial), want * 65536 * sizeof(float)));
        h->tail_partial_slots = want;
      }
      g.tail_splits = splits;
      g.tail_rounds = tiles > pairs ? int(tiles / pairs) : 0;
      g.tail_tiles = rem;
      g.partial = h->tail_partial;
      if (tiles <= pairs) pairs = int(std::min<long long>(static_cast<long long>(rem) * splits, max_pairs));
    }
  }
  cfg.gridDim = dim3(2 * pairs);
  cfg.numAttrs = h->pdl ? 2 : 1;
  ProfScope prof(h, prof_class, work);
  MTB_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, g));
  if (g.tail_splits > 1) {
    const int tiles_m = (g.M + 255) / 256, tiles_n = (g.N + 255) / 256;
    MTB_CUDA(launch_pdl(h, tail_fixup_kernel, dim3(unsigned(g.tail_tiles), 64), dim3(256), 0, g, pairs, tiles_m, tiles_n));
  }
  return MTB200_OK;
}

// Two-CTA kernel: clusters of two CTAs, one 256 x 256 tile per pair at a time.
// K = logical reduction length; Kp = padded column count of K-major planes.
template <int BK, int STAGES, int NP>
inline int32_t launch_variant2(mtb200_ctx* h, const SplitOperand& a, const SplitOperand& b, int Kp, GemmArgs g,
                               int K = 0, bool tail = true) {
  using Cfg = Gemm2Cfg<BK, STAGES, NP>;
  if (K <= 0) K = Kp;
  if (a.nplanes != NP || b.nplanes != NP) return fail(MTB200_ERR_INVALID, "operand planes do not match the GEMM mode");
  CUtensorMap ta, tb;
  int32_t rc;
  if (a.mn_major) rc = make_split_tmap_mn(&ta, a.base, a.rows, a.cols_p, uint64_t(NP) * a.batch, BK, Cfg::BM / 64);
  else            rc = make_split_tmap(&ta, a.base, Kp, a.rows, uint64_t(NP) * a.batch, BK, Cfg::BM);
  if (rc) return rc;
  if (b.mn_major) rc = make_split_tmap_mn(&tb, b.base, b.rows, b.cols_p, uint64_t(NP) * b.batch, BK, Cfg::BNH / 64);
  else            rc = make_split_tmap(&tb, b.base, Kp, b.rows, uint64_t(NP) * b.batch, BK, Cfg::BNH);
  if (rc) return rc;
  g.num_kb = g.num_kb ? g.num_kb * (64 / BK) : (K + BK - 1) / BK;
  g.kb_batch_stride *= (64 / BK);
  g.planes_per_mat = NP;
  const long long tiles = static_cast<long long>((g.M + Cfg::TILE_M - 1) / Cfg::TILE_M) *
                          ((g.N + Cfg::TILE_N - 1) / Cfg::TILE_N) * g.batch;
  const double work = 2.0 * g.M * g.N * double(g.num_kb) * BK * g.batch;
  if constexpr (BK == 64) {
    if (a.mn_major && b.mn_major)
      return launch_pair_kernel(h, gemm_split_umma2_kernel<BK, STAGES, true, true, NP>, Cfg::SMEM_BYTES,
                                Cfg::NUM_THREADS, tiles, ta, tb, g, work, tail);
    if (a.mn_major)
      return launch_pair_kernel(h, gemm_split_umma2_kernel<BK, STAGES, true, false, NP>, Cfg::SMEM_BYTES,
                                Cfg::NUM_THREADS, tiles, ta, tb, g, work, tail);
    if (b.mn_major)
      return launch_pair_kernel(h, gemm_split_umma2_kernel<BK, STAGES, false, true, NP>, Cfg::SMEM_BYTES,
                                Cfg::NUM_THREADS, tiles, ta, tb, g, work, tail);
  } else {
    if (a.mn_major || b.mn_major) return fail(MTB200_ERR_INVALID, "MN-major operands need the K-block-64 kernel");
  }
  return launch_pair_kernel(h, gemm_split_umma2_kernel<BK, STAGES, false, false, NP>, Cfg::SMEM_BYTES,
                            Cfg::NUM_THREADS, tiles, ta, tb, g, work, tail && BK == 64);
}

// One-CTA kernel on the fp16 two-plane operands, 128 x 128 tiles, K block 64: for outputs of so few pair tiles that
// the two-CTA kernel would leave most SMs idle or cut every tile along K and pay the fix-up pass (1024^3 is 16 pair
// tiles but 64 of these).
template <bool A_MN, bool B_MN>
inline int32_t launch_small_f16(mtb200_ctx* h, const SplitOperand& a, const SplitOperand& b, int Kp, GemmArgs g, int K) {
  using Cfg = GemmCfg<128, 64, 3, 2>;
  auto kern = gemm_split_umma_kernel<128, 64, 3, false, 2, A_MN, B_MN>;
  if (int32_t rc_attr = grant_dynamic_smem(h, kern, int(Cfg::SMEM_BYTES))) return rc_attr;
  CUtensorMap ta, tb;
  int32_t rc;
  if (A_MN) rc = make_split_tmap_mn(&ta, a.base, a.rows, a.cols_p, uint64_t(2) * a.batch, 64, 2);
  else      rc = make_split_tmap(&ta, a.base, Kp, a.rows, uint64_t(2) * a.batch, 64, 128);
  if (rc) return rc;
  if (B_MN) rc = make_split_tmap_mn(&tb, b.base, b.rows, b.cols_p, uint64_t(2) * b.batch, 64, 2);
  else      rc = make_split_tmap(&tb, b.base, Kp, b.rows, uint64_t(2) * b.batch, 64, 128);
  if (rc) return rc;
  g.num_kb = (K + 63) / 64;
  g.planes_per_mat = 2;
  const long long tiles = static_cast<long long>((g.M + 127) / 128) * ((g.N + 127) / 128) * g.batch;
  const int grid = int(std::min<long long>(tiles, h->sm_count));
  ProfScope prof(h, PROF_GEMM_UMMA, 2.0 * g.M * g.N * double(g.num_kb) * 64 * g.batch);
  MTB_CUDA(launch_pdl(h, kern, dim3(grid), dim3(Cfg::NUM_THREADS), Cfg::SMEM_BYTES, ta, tb, g));
  return MTB200_OK;
}

// C[b] = epilogue(A_split[b] * B_split[b]^T + bias) on prepared operands.
// variant: 0 = choose by N; 1 = 128x256 tile, K block 32; 2 = 128x128, K block 64;
// 3 = 128x64, K block 64; 4 = 128x128, K block 32; 5 / 6 = two-CTA 256x256 pair tile with K block 64 / 32;
// 7 = 5 without tail splitting; 8 = one-CTA 128x128 on fp16 planes (chosen for outputs of few pair tiles).
inline int32_t run_split_gemm(mtb200_ctx* h, const SplitOperand& a, const SplitOperand& b, int Kp,
                              int batch, int M, int N, float* C, long long ldc, long long strideC,
                              const float* bias, int epilogue, const float* aux, int mode, int variant,
                              int bias_per_row = 0, int kb_batch_stride = 0, int num_kb_override = 0, int K = 0) {
  if (mode == 0) mode = 6;
  if (mode != 1 && mode != 3 && mode != 6 && mode != 9 && mode != 23)
    return fail(MTB200_ERR_INVALID, "unknown f32 mode %d (use 0, 1, 3, 6, 9 or 23)", mode);
  GemmArgs g = {};
  g.M = M; g.N = N; g.batch = batch;
  g.C = C; g.ldc = ldc; g.strideC = strideC;
  g.bias = bias; g.aux = aux; g.epilogue = epilogue; g.mode = mode;
  g.a_batched = a.batched; g.b_batched = b.batched;
  g.status = h->status;
  g.planes_per_mat = a.nplanes;
  g.exp_a = a.expo; g.exp_b = b.expo;
  g.bias_per_row = bias_per_row;
  g.kb_batch_stride = kb_batch_stride;
  g.num_kb = num_kb_override;  // 0: the whole padded K
  // two-CTA pair tiles whenever the output is at least one pair tile tall and wide
  if (variant == 0) variant = (M > 128 && N > 128) ? 5 : ((N > 128) ? 1 : (N > 64 ? 2 : 3));
  // fp16 mode, whole K, few pair tiles: the one-CTA kernel fills more SMs and needs no fix-up pass
  if (variant == 5 && mode == 23 && num_kb_override == 0 && kb_batch_stride == 0 && a.nplanes == 2 && b.nplanes == 2 &&
      static_cast<long long>((M + 255) / 256) * ((N + 255) / 256) * batch <= h->sm_count / 4)
    variant = 8;
  if (variant == 8) {
    const int Kl = K > 0 ? K : Kp;
    if (a.mn_major && b.mn_major) return launch_small_f16<true, true>(h, a, b, Kp, g, Kl);
    if (a.mn_major) return launch_small_f16<true, false>(h, a, b, Kp, g, Kl);
    if (b.mn_major) return launch_small_f16<false, true>(h, a, b, Kp, g, Kl);
    return launch_small_f16<false, false>(h, a, b, Kp, g, Kl);
  }
  if ((a.mn_major || b.mn_major || mode == 23) && variant != 5 && variant != 7)
    return fail(MTB200_ERR_INVALID, "MN-major planes and the fp16 mode need the two-CTA kernel (variant 5)");
  switch (variant) {
    case 1: return launch_variant<256, 32, 3>(h, a, b, Kp, g);
    case 2: return launch_variant<128, 64, 2>(h, a, b, Kp, g);
    case 3: return launch_variant<64, 64, 3>(h, a, b, Kp, g);
    case 4: return launch_variant<128, 32, 4>(h, a, b, Kp, g);
    case 5: return mode == 23 ? launch_variant2<64, 3, 2>(h, a, b, Kp, g, K) : launch_variant2<64, 2, 3>(h, a, b, Kp, g, K);
    case 7: return mode == 23 ? launch_variant2<64, 3, 2>(h, a, b, Kp, g, K, false)   // 5 without tail splitting
                              : launch_variant2<64, 2, 3>(h, a, b, Kp, g, K, false);
    case 6: return launch_variant2<32, 4, 3>(h, a, b, Kp, g);
    default: return fail(MTB200_ERR_INVALID, "unknown GEMM tile variant %d", variant);
  }
}

// Scale + split one f32 operand into two fp16 planes and its exponent vector.
//  k_major: source [mn][k] (scale per row); otherwise source [k][mn] (scale per column).
inline int32_t launch_split16(mtb200_ctx* h, const float* src, bool k_major, int mn, int K, int batch,
                              long long bstride, __half* planes, int* expo, uint32_t* nf_word, uint32_t epoch,
                              cudaStream_t stream = nullptr) {
  if (!stream) stream = h->stream;
  if (k_major) {
    const int Kp = padded_k(K);
    const dim3 grid(unsigned(std::min(mn, 65535)), 1, batch);
    const bool vec = (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0) && ((bstride & 3) == 0);
    // bytes: the row is read once when it is held in registers, twice (second time from L1/L2) otherwise
    ProfScope prof(h, PROF_SPLIT, double(batch) * mn * ((vec && Kp <= 8192 ? 4.0 : 8.0) * K + 4.0 * Kp));
    if (vec && Kp <= 1024)
      split16_rows_reg_kernel<1><<<grid, 256, 0, stream>>>(src, K, bstride, planes, expo, mn, K, Kp, nf_word, epoch);
    else if (vec && Kp <= 2048)
      split16_rows_reg_kernel<2><<<grid, 256, 0, stream>>>(src, K, bstride, planes, expo, mn, K, Kp, nf_word, epoch);
    else if (vec && Kp <= 4096)
      split16_rows_reg_kernel<4><<<grid, 256, 0, stream>>>(src, K, bstride, planes, expo, mn, K, Kp, nf_word, epoch);
    else if (vec && Kp <= 8192)
      split16_rows_reg_kernel<8><<<grid, 256, 0, stream>>>(src, K, bstride, planes, expo, mn, K, Kp, nf_word, epoch);
    else
      split16_rows_kernel<<<grid, 256, 0, stream>>>(src, K, bstride, planes, expo, mn, K, Kp, nf_word, epoch);
  } else {
    const int cp = padded_k(mn);
    ProfScope prof(h, PROF_SPLIT, double(batch) * K * (8.0 * mn + 4.0 * cp));
    MTB_CUDA(cudaMemsetAsync(expo, 0, sizeof(int) * size_t(batch) * mn, stream));
    const int bands = std::max(1, std::min((K + 63) / 64, (h->sm_count * 8) / std::max(1, (mn + 255) / 256)));
    const int rows_per_band = (K + bands - 1) / bands;
    colabsmax_kernel<<<dim3((mn + 255) / 256, (K + rows_per_band - 1) / rows_per_band, batch), 256, 0, stream>>>(
        src, mn, bstride, K, mn, rows_per_band, reinterpret_cast<uint32_t*>(expo), nf_word, epoch);
    MTB_CUDA(launch_pdl_on(h, stream, exponent_from_amax_kernel, dim3((batch * mn + 255) / 256), dim3(256), 0,
                           reinterpret_cast<const uint32_t*>(expo), expo, batch * mn));
    const long long total = static_cast<long long>(K) * (cp / 8);
    const int blocks = int(std::min<long long>((total + 255) / 256, (long long)h->sm_count * 32));
    MTB_CUDA(launch_pdl_on(h, stream, split16_cols_scaled_kernel, dim3(blocks, 1, batch), dim3(256), 0, src,
                           static_cast<long long>(mn), bstride, planes, static_cast<const int*>(expo), K, mn, cp));
  }
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

// Both operands of an fp16-mode product in ONE launch (prep_f16.cuh).  Returns false when an operand does not meet
// the kernel's conditions (a rows-mode operand must be readable as float4 and at most 8192 long); the caller then
// prepares the operands one by one.
inline bool prep16_pair_eligible(const float* src, bool k_major, int K, int batch, long long bstride) {
  if (!k_major) return true;
  return (K % 4 == 0) && padded_k(K) <= 8192 && ((reinterpret_cast<uintptr_t>(src) & 15) == 0) &&
         (batch == 1 || (bstride & 3) == 0);
}
inline PrepOperand prep16_operand(const mtb200_ctx* h, const float* src, bool k_major, int mn, int K, int batch,
                                  long long bstride, __half* planes, int* expo) {
  PrepOperand o;
  o.src = src; o.bstride = bstride; o.planes = planes; o.expo = expo;
  o.kmajor = k_major ? 1 : 0; o.mn = mn; o.K = K; o.batch = batch;
  if (k_major) {
    o.ld = K; o.pitch = padded_k(K);
    o.blocks = std::min((mn + 7) / 8 * 8, 8 * 1024);
  } else {
    o.ld = mn; o.pitch = padded_k(mn);
    const int strips = (mn + 63) / 64;
    o.blocks = 8 * std::min(strips, std::max(1, 2 * h->sm_count));
  }
  return o;
}
inline int32_t launch_prep16_pair(mtb200_ctx* h, const PrepOperand& a, const PrepOperand& b, uint32_t* nf_word,
                                  uint32_t nf_value) {
  int kp_rows = 0;
  if (a.kmajor) kp_rows = std::max(kp_rows, a.pitch);
  if (b.kmajor) kp_rows = std::max(kp_rows, b.pitch);
  auto bytes_of = [](const PrepOperand& o) {
    return double(o.batch) * o.mn * (4.0 * o.K * (o.kmajor ? 1.0 : 2.0)) + double(o.batch) * 4.0 * (o.kmajor ? double(o.mn) * o.pitch : double(o.K) * o.pitch);
  };
  ProfScope prof(h, PROF_SPLIT, bytes_of(a) + bytes_of(b));
  const dim3 grid(unsigned(a.blocks + b.blocks), unsigned(std::max(a.batch, b.batch)));
  if (kp_rows <= 1024) prep16_pair_kernel<1><<<grid, 256, 0, h->stream>>>(a, b, nf_word, nf_value);
  else if (kp_rows <= 2048) prep16_pair_kernel<2><<<grid, 256, 0, h->stream>>>(a, b, nf_word, nf_value);
  else if (kp_rows <= 4096) prep16_pair_kernel<4><<<grid, 256, 0, h->stream>>>(a, b, nf_word, nf_value);
  else prep16_pair_kernel<8><<<grid, 256, 0, h->stream>>>(a, b, nf_word, nf_value);
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

// f32 GEMM in the fp16 two-plane mode (pair-tile kernel only).
inline int32_t gemm_f32_split_f16(mtb200_ctx* h, bool trans_a, bool trans_b, int batch, int M, int N, int K,
                                  const float* A, long long stride_a, const float* B, long long stride_b, float* C,
                                  long long ldc, long long stride_c, const float* bias, int epilogue,
                                  const float* aux, int variant = 5) {
  const int Kp = padded_k(K);
  const int batch_a = (stride_a == 0 || batch == 1) ? 1 : batch;
  const int batch_b = (stride_b == 0 || batch == 1) ? 1 : batch;
  const bool a_kmaj = !trans_a, b_kmaj = trans_b;
  const int a_rows = a_kmaj ? M : K, a_cols_p = a_kmaj ? Kp : padded_k(M);
  const int b_rows = b_kmaj ? N : K, b_cols_p = b_kmaj ? Kp : padded_k(N);
  const size_t bytes_a = align_up(size_t(2) * batch_a * a_rows * a_cols_p * 2, 1024);
  const size_t bytes_b = align_up(size_t(2) * batch_b * b_rows * b_cols_p * 2, 1024);
  const size_t bytes_ea = align_up(sizeof(int) * size_t(batch_a) * M, 1024);
  const size_t bytes_eb = align_up(sizeof(int) * size_t(batch_b) * N, 1024);
  void* ws = nullptr;
  int32_t rc = workspace_reserve(h, bytes_a + bytes_b + bytes_ea + bytes_eb, &ws);
  if (rc) return rc;
  char* base = static_cast<char*>(ws);
  __half* pa = reinterpret_cast<__half*>(base);
  __half* pb = reinterpret_cast<__half*>(base + bytes_a);
  int* ea = reinterpret_cast<int*>(base + bytes_a + bytes_b);
  int* eb = reinterpret_cast<int*>(base + bytes_a + bytes_b + bytes_ea);
  uint32_t* nf_word = nullptr;
  rc = call_flag_begin(h, &nf_word);
  if (rc) return rc;
  const uint32_t epoch = MTB_FLAG_SET;
  // Small products: both operands in one launch.  Otherwise one by one, side by side on two streams when they are
  // small enough not to fill the memory system alone.
  // (measured: for products up to about 1024^3 the single launch wins - 512^3 53 -> 39 us, 1024^3 57 -> 49 us whole
  // call - beyond that the two tuned kernels running side by side do)
  const bool pair = batch == 1 && (double(M) + double(N)) * K <= 2.2e6 &&
                    prep16_pair_eligible(A, a_kmaj, K, batch_a, stride_a) &&
                    prep16_pair_eligible(B, b_kmaj, K, batch_b, stride_b);
  if (pair) {
    rc = launch_prep16_pair(h, prep16_operand(h, A, a_kmaj, M, K, batch_a, stride_a, pa, ea),
                            prep16_operand(h, B, b_kmaj, N, K, batch_b, stride_b, pb, eb), nf_word, epoch);
    if (rc) return rc;
  }
  const bool side_by_side = !pair && h->side_stream && !h->profiling &&
                            double(batch_a) * M * K <= 33554432.0 && double(batch_b) * N * K <= 33554432.0;
  if (side_by_side) {
    MTB_CUDA(cudaEventRecord(h->ev_fork, h->stream));
    MTB_CUDA(cudaStreamWaitEvent(h->side_stream, h->ev_fork, 0));
  }
  if (!pair) {
    rc = launch_split16(h, A, a_kmaj, M, K, batch_a, stride_a, pa, ea, nf_word, epoch);
    if (rc) return rc;
    rc = launch_split16(h, B, b_kmaj, N, K, batch_b, stride_b, pb, eb, nf_word, epoch,
                        side_by_side ? h->side_stream : nullptr);
    if (rc) return rc;
  }
  if (side_by_side) {
    MTB_CUDA(cudaEventRecord(h->ev_join, h->side_stream));
    MTB_CUDA(cudaStreamWaitEvent(h->stream, h->ev_join, 0));
  }
  SplitOperand oa{reinterpret_cast<const __nv_bfloat16*>(pa), a_rows, batch_a > 1, batch_a, a_kmaj ? 0 : 1, a_cols_p, 2, ea};
  SplitOperand ob{reinterpret_cast<const __nv_bfloat16*>(pb), b_rows, batch_b > 1, batch_b, b_kmaj ? 0 : 1, b_cols_p, 2, eb};
  rc = run_split_gemm(h, oa, ob, Kp, batch, M, N, C, ldc, stride_c, bias, epilogue, aux, 23, variant, 0, 0, 0, K);
  if (rc) return rc;
  StridedGemmArgs s;
  s.M = M; s.N = N; s.K = K; s.batch = batch;
  s.A = A; s.B = B; s.C = C;
  s.a_si = trans_a ? 1 : K;  s.a_sk = trans_a ? M : 1;  s.a_sb = stride_a;
  s.b_sk = trans_b ? 1 : N;  s.b_sj = trans_b ? K : 1;  s.b_sb = stride_b;
  s.ldc = ldc; s.c_sb = stride_c;
  s.bias = bias; s.aux = aux; s.epilogue = epilogue;
  s.gate = nf_word; s.gate_value = epoch;
  const long long tiles = static_cast<long long>((M + 127) / 128) * ((N + 127) / 128);
  MTB_CUDA(launch_pdl(h, gemm_simt_kernel<float, 8, 8>, dim3(unsigned(tiles), unsigned(batch)), dim3(256), 0, s));
  return MTB200_OK;
}

// Full f32 GEMM from row-major f32 operands: split both into scratch, multiply.
// With the two-CTA kernel every operand is split as it lies in memory (no
// transposing pass): an operand stored [mn][k] becomes K-major planes, one stored
// [k][mn] becomes MN-major planes, and the kernel's descriptors do the rest.
inline int32_t gemm_f32_split(mtb200_ctx* h, bool trans_a, bool trans_b, int batch, int M, int N, int K,
                              const float* A, long long stride_a, const float* B, long long stride_b,
                              float* C, long long ldc, long long stride_c, const float* bias,
                              int epilogue, const float* aux, int mode, int variant) {
  const int Kp = padded_k(K);
  const int batch_a = (stride_a == 0 || batch == 1) ? 1 : batch;
  const int batch_b = (stride_b == 0 || batch == 1) ? 1 : batch;
  // Products too small to amortise operand preparation (two or three extra launches) run as ONE launch of the
  // CUDA-core kernel in plain f32 multiply-add; variant 0xFE forces that path for any size.
  const double macs = double(M) * double(N) * double(K) * double(batch);
  if (variant == 0xFE || (variant == 0 && mode == 0 && K <= SMALL_GEMM_K && macs <= SMALL_GEMM_MACS)) {
    StridedGemmArgs s;
    s.M = M; s.N = N; s.K = K; s.batch = batch;
    s.A = A; s.B = B; s.C = C;
    s.a_si = trans_a ? 1 : K;  s.a_sk = trans_a ? M : 1;  s.a_sb = stride_a;
    s.b_sk = trans_b ? 1 : N;  s.b_sj = trans_b ? K : 1;  s.b_sb = stride_b;
    s.ldc = ldc; s.c_sb = stride_c;
    s.bias = bias; s.aux = aux; s.epilogue = epilogue;
    s.gate = nullptr; s.gate_value = 0;
    ProfScope prof(h, PROF_GEMM_UMMA, 2.0 * macs);
    const long long tiles = static_cast<long long>((M + 63) / 64) * ((N + 63) / 64);
    gemm_simt_kernel<float, 4, 4><<<dim3(unsigned(tiles), unsigned(batch)), 256, 0, h->stream>>>(s);
    MTB_CUDA(cudaGetLastError());
    return MTB200_OK;
  }
  if (variant == 0 && M > 128 && N > 128) variant = 5;
  // default arithmetic: the fp16 two-plane mode wherever the pair-tile kernel runs, six bf16 products elsewhere
  const bool pair_tile = (variant == 5 || variant == 7);
  const int eff_mode = mode == 0 ? (pair_tile ? 23 : 6) : mode;
  const int nsplit = eff_mode == 1 ? 1 : (eff_mode == 3 ? 2 : 3);
  if (eff_mode == 23) {
    if (!pair_tile) return fail(MTB200_ERR_UNSUPPORTED, "the fp16 mode runs on the pair-tile kernel (M, N > 128)");
    return gemm_f32_split_f16(h, trans_a, trans_b, batch, M, N, K, A, stride_a, B, stride_b, C, ldc, stride_c, bias,
                              epilogue, aux, variant);
  }
  const bool straight = pair_tile;
  // plane geometry: rows x padded cols
  const int a_rows = (straight && trans_a) ? K : M, a_cols_p = (straight && trans_a) ? padded_k(M) : Kp;
  const int b_rows = (straight && !trans_b) ? K : N, b_cols_p = (straight && !trans_b) ? padded_k(N) : Kp;
  const size_t bytes_a = align_up(size_t(3) * batch_a * a_rows * a_cols_p * 2, 1024);
  const size_t bytes_b = align_up(size_t(3) * batch_b * b_rows * b_cols_p * 2, 1024);
  void* ws = nullptr;
  int32_t rc = workspace_reserve(h, bytes_a + bytes_b, &ws);
  if (rc) return rc;
  __nv_bfloat16* sa = static_cast<__nv_bfloat16*>(ws);
  __nv_bfloat16* sb = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(ws) + bytes_a);
  uint32_t* nf_word = nullptr;
  rc = call_flag_begin(h, &nf_word);
  if (rc) return rc;
  const uint32_t epoch = MTB_FLAG_SET;
  SplitOperand oa{sa, a_rows, batch_a > 1, batch_a, 0, a_cols_p}, ob{sb, b_rows, batch_b > 1, batch_b, 0, b_cols_p};
  if (straight) {
    oa.mn_major = trans_a ? 1 : 0;
    ob.mn_major = trans_b ? 0 : 1;
    rc = launch_split(h, A, false, a_rows, trans_a ? M : K, a_cols_p, batch_a, stride_a, sa, nsplit, nf_word, epoch);
    if (rc) return rc;
    rc = launch_split(h, B, false, b_rows, trans_b ? K : N, b_cols_p, batch_b, stride_b, sb, nsplit, nf_word, epoch);
    if (rc) return rc;
  } else {
    // op(A) is [M][K]: stored [M][K] when !trans_a (K-major already), [K][M] when trans_a.
    rc = launch_split(h, A, trans_a, M, K, Kp, batch_a, stride_a, sa, nsplit, nf_word, epoch);
    if (rc) return rc;
    // op(B) is [K][N]: the operand the kernel wants is [N][K]; stored so when trans_b.
    rc = launch_split(h, B, !trans_b, N, K, Kp, batch_b, stride_b, sb, nsplit, nf_word, epoch);
    if (rc) return rc;
  }
  rc = run_split_gemm(h, oa, ob, Kp, batch, M, N, C, ldc, stride_c, bias, epilogue, aux, mode, variant, 0, 0, 0, K);
  if (rc) return rc;
  // Inf / NaN operands: redo the product with IEEE f32 multiply-add.  The kernel
  // returns at once unless a split kernel of THIS call raised the word.
  StridedGemmArgs s;
  s.M = M; s.N = N; s.K = K; s.batch = batch;
  s.A = A; s.B = B; s.C = C;
  s.a_si = trans_a ? 1 : K;  s.a_sk = trans_a ? M : 1;  s.a_sb = stride_a;
  s.b_sk = trans_b ? 1 : N;  s.b_sj = trans_b ? K : 1;  s.b_sb = stride_b;
  s.ldc = ldc; s.c_sb = stride_c;
  s.bias = bias; s.aux = aux; s.epilogue = epilogue;
  s.gate = nf_word; s.gate_value = epoch;
  const long long tiles = static_cast<long long>((M + 127) / 128) * ((N + 127) / 128);
  gemm_simt_kernel<float, 8, 8><<<dim3(unsigned(tiles), unsigned(batch)), 256, 0, h->stream>>>(s);
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

}  // namespace mtb
