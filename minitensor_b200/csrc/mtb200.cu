// C ABI of the B200 dense-contraction path: handle, memory, GEMM dispatch,
// column sum, activations, cross entropy, Adam.  conv2d lives in conv2d.cu.
// Declarations and the reference interfaces they replace: include/mtb200.h.
#include "mtb200_core.cuh"
#include "gemm_split_umma.cuh"
#include "split_bf16.cuh"
#include "gemm_f64_int.cuh"
#include "rowcol_kernels.cuh"
#include "gemm_launch.cuh"
#include "gemm_i32_limb.cuh"
#include "dense_layer.cuh"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <mutex>

namespace mtb {

thread_local std::string g_last_error;

int32_t workspace_reserve(mtb200_ctx* h, size_t bytes, void** out) {
  if (bytes > h->workspace_bytes) {
    MTB_CUDA(cudaStreamSynchronize(h->stream));
    if (h->workspace) {
      MTB_CUDA(cudaFree(h->workspace));
      h->workspace = nullptr;
      h->workspace_bytes = 0;
    }
    const size_t want = align_up(bytes + bytes / 8, size_t(1) << 21);
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(MTB200_ERR_NOMEM, "scratch allocation of %zu bytes failed: %s", want,
                  cudaGetErrorString(e));
    }
    h->workspace = p;
    h->workspace_bytes = want;
  }
  *out = h->workspace;
  return MTB200_OK;
}

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int32_t make_split_tmap(CUtensorMap* out, const void* base, uint64_t Kp, uint64_t rows,
                        uint64_t planes, uint32_t bk, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return fail(MTB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[3] = {Kp, rows, planes};
  const cuuint64_t strides[2] = {Kp * 2, rows * Kp * 2};  // bytes, dims 1 and 2
  const cuuint32_t box[3] = {bk, box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapSwizzle sw = (bk * 2 == 128) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(MTB200_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for dims {%llu,%llu,%llu} box {%u,%u}",
                int(r), (unsigned long long)Kp, (unsigned long long)rows, (unsigned long long)planes, bk,
                box_rows);
  return MTB200_OK;
}

static inline int grid_for(long long n, int threads, int sm_count) {
  long long blocks = (n + threads - 1) / threads;
  return int(std::max<long long>(1, std::min<long long>(blocks, (long long)sm_count * 16)));
}

// compiler-rt's integer power (what Rust's f64::powi lowers to): square and multiply.
static double powi_f64(double a, int b) {
  const bool recip = b < 0;
  double r = 1.0;
  while (true) {
    if (b & 1) r *= a;
    b /= 2;
    if (b == 0) break;
    a *= a;
  }
  return recip ? 1.0 / r : r;
}

}  // namespace mtb

namespace mtb {

// int32 GEMM on the integer tensor cores (gemm_i32_limb.cuh): byte-limb planes of both operands in
// scratch, then one launch per K chunk of at most 8192.
static int32_t gemm_i32_limb(mtb200_ctx* h, bool trans_a, bool trans_b, int batch, int M, int N, int K,
                             const int32_t* A, long long stride_a, const int32_t* B, long long stride_b,
                             int32_t* C, long long stride_c) {
  using Cfg = I32LimbCfg;
  const int Kp = (K + 63) / 64 * 64;
  const int batch_a = (stride_a == 0 || batch == 1) ? 1 : batch;
  const int batch_b = (stride_b == 0 || batch == 1) ? 1 : batch;
  const size_t bytes_a = align_up(size_t(4) * batch_a * M * Kp, 1024), bytes_b = align_up(size_t(4) * batch_b * N * Kp, 1024);
  void* ws = nullptr;
  int32_t rc = workspace_reserve(h, bytes_a + bytes_b, &ws);
  if (rc) return rc;
  uint8_t* pa = static_cast<uint8_t*>(ws);
  uint8_t* pb = pa + bytes_a;
  uint32_t* wide_word = nullptr;
  rc = call_flag_begin(h, &wide_word);
  if (rc) return rc;
  const uint32_t epoch = MTB_FLAG_SET;
  {
    ProfScope prof(h, PROF_SPLIT, 8.0 * (double(batch_a) * M + double(batch_b) * N) * K);
    // op(A) is [M][K]: source [M][K] or, transposed, [K][M];  op(B)^T is [N][K]: source [K][N] needs the turn
    auto split = [&](const int32_t* src, bool turn, int rows, int nb, long long bstride, uint8_t* dst) {
      const bool direct = !turn && (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(src) & 15) == 0) && ((bstride & 3) == 0);
      if (direct) {
        const long long total = static_cast<long long>(rows) * (Kp / 16);
        const int blocks = int(std::min<long long>((total + 255) / 256, (long long)h->sm_count * 32));
        limb_split_rows_kernel<<<dim3(blocks, 1, nb), 256, 0, h->stream>>>(src, K, bstride, dst, rows, K, Kp, wide_word, epoch);
      } else if (turn) {
        limb_split_turn_kernel<<<dim3((rows + 31) / 32, (Kp + 127) / 128, nb), 256, 0, h->stream>>>(
            src, rows, bstride, dst, rows, K, Kp, wide_word, epoch);
      } else {
        limb_split_kernel<<<dim3((rows + 63) / 64, Kp / 64, nb), 256, 0, h->stream>>>(
            src, K, bstride, 0, dst, rows, K, Kp, wide_word, epoch);
      }
    };
    split(A, trans_a, M, batch_a, stride_a, pa);
    split(B, !trans_b, N, batch_b, stride_b, pb);
    MTB_CUDA(cudaGetLastError());
  }
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return fail(MTB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMap ta, tb;
  auto make = [&](CUtensorMap* out, void* base, int rows, int planes) -> int32_t {
    const cuuint64_t dims[3] = {cuuint64_t(Kp), cuuint64_t(rows), cuuint64_t(planes)};
    const cuuint64_t strides[2] = {cuuint64_t(Kp), cuuint64_t(rows) * Kp};
    const cuuint32_t box[3] = {Cfg::BKB, 128, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MTB200_OK : fail(MTB200_ERR_CUDA, "cuTensorMapEncodeTiled (limb planes) failed (%d)", int(r));
  };
  rc = make(&ta, pa, M, 4 * batch_a);
  if (rc) return rc;
  rc = make(&tb, pb, N, 4 * batch_b);
  if (rc) return rc;
  if (int32_t rc_attr = grant_dynamic_smem(h, gemm_i32_limb_umma_kernel, int(Cfg::SMEM_BYTES))) return rc_attr;
  I32LimbArgs g = {};
  g.M = M; g.N = N; g.batch = batch;
  g.C = reinterpret_cast<uint32_t*>(C); g.strideC = stride_c;
  g.a_batched = batch_a > 1; g.b_batched = batch_b > 1;
  g.wide_word = wide_word; g.wide_epoch = epoch; g.status = h->status;
  const long long tiles = static_cast<long long>((M + 127) / 128) * ((N + 127) / 128) * batch;
  const int grid = int(std::min<long long>(tiles, h->sm_count));
  const int total_kb = Kp / 64, chunk_kb = 8192 / 64;
  // Operands that fit in int8 (known only on the device) and a reduction of one chunk: the pair-tile kernel with
  // kind::i8 takes the product - 256 x 256 tiles, six stages, overlapped epilogue - and the limb kernel below
  // returns at once; operands that need all four limbs make the pair-tile kernel return at once instead.
  if (M > 128 && N > 128 && total_kb <= chunk_kb) {
    using PC = Gemm2Cfg<64, 6, 1>;
    CUtensorMap pa_map, pb_map;
    rc = make_split_tmap(&pa_map, pa, uint64_t(Kp) / 2, uint64_t(M), uint64_t(4) * batch_a, 64, PC::BM);
    if (rc) return rc;
    rc = make_split_tmap(&pb_map, pb, uint64_t(Kp) / 2, uint64_t(N), uint64_t(4) * batch_b, 64, PC::BNH);
    if (rc) return rc;
    GemmArgs p = {};
    p.M = M; p.N = N; p.batch = batch;
    p.num_kb = (Kp + 127) / 128;
    p.C = reinterpret_cast<float*>(C); p.ldc = N; p.strideC = stride_c;
    p.epilogue = EPI_NONE; p.mode = 1; p.planes_per_mat = 4;
    p.a_batched = batch_a > 1; p.b_batched = batch_b > 1;
    p.status = h->status;
    p.gate = wide_word; p.gate_value = epoch; p.gate_run_if_equal = 0;
    p.raw_int = 1;
    const long long ptiles = static_cast<long long>((M + 255) / 256) * ((N + 255) / 256) * batch;
    rc = launch_pair_kernel(h, gemm_split_umma2_kernel<64, 6, false, false, 1, true>, PC::SMEM_BYTES, PC::NUM_THREADS,
                            ptiles, pa_map, pb_map, p, 2.0 * M * N * double(Kp) * batch, true, PROF_GEMM_INT);
    if (rc) return rc;
    g.skip_narrow = 1;
  }
  for (int kb0 = 0; kb0 < total_kb; kb0 += chunk_kb) {
    g.kb0 = kb0;
    g.num_kb = std::min(chunk_kb, total_kb - kb0);
    g.accumulate = kb0 > 0;
    ProfScope prof(h, PROF_GEMM_INT, 2.0 * M * N * double(g.num_kb) * 64 * batch);
    gemm_i32_limb_umma_kernel<<<grid, Cfg::NUM_THREADS, Cfg::SMEM_BYTES, h->stream>>>(ta, tb, g);
    MTB_CUDA(cudaGetLastError());
  }
  return MTB200_OK;
}

}  // namespace mtb

using namespace mtb;

#define MTB_CHECK_HANDLE(h)                                         \
  if (!(h)) return fail(MTB200_ERR_INVALID, "null handle");         \
  DeviceGuard guard__((h)->device);                                 \
  if (!guard__.ok) return fail(MTB200_ERR_CUDA, "cannot make device %d current", (h)->device)

extern "C" {

int32_t mtb200_version(void) { return MTB200_VERSION; }
const char* mtb200_last_error(void) { return g_last_error.c_str(); }

int32_t mtb200_create(int32_t device_ordinal, mtb200_handle* out) {
  if (!out) return fail(MTB200_ERR_INVALID, "null output handle");
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) {
    cudaGetLastError();
    return fail(MTB200_ERR_CUDA, "no CUDA device available (%s)",
                e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
  }
  if (device_ordinal < 0 || device_ordinal >= count)
    return fail(MTB200_ERR_INVALID, "device ordinal %d out of range [0,%d)", device_ordinal, count);
  cudaDeviceProp prop;
  MTB_CUDA(cudaGetDeviceProperties(&prop, device_ordinal));
  if (prop.major != 10)
    return fail(MTB200_ERR_CUDA, "device %d is compute capability %d.%d; this library is built for sm_100a only",
                device_ordinal, prop.major, prop.minor);
  DeviceGuard guard(device_ordinal);
  if (!guard.ok) return fail(MTB200_ERR_CUDA, "cannot make device %d current", device_ordinal);
  mtb200_ctx* h = new mtb200_ctx();
  h->device = device_ordinal;
  h->sm_count = prop.multiProcessorCount;
  if (const char* no_pdl = getenv("MTB200_NO_PDL")) h->pdl = !(no_pdl[0] && no_pdl[0] != '0');
  e = cudaStreamCreateWithFlags(&h->own_stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->side_stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->ev_fork, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->ev_join, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&h->status), (4 + MTB_FLAG_SLOTS) * sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemset(h->status, 0, (4 + MTB_FLAG_SLOTS) * sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMallocHost(reinterpret_cast<void**>(&h->status_host), 2 * sizeof(uint32_t));
  if (e != cudaSuccess) {
    if (h->status) cudaFree(h->status);
    if (h->own_stream) cudaStreamDestroy(h->own_stream);
    if (h->side_stream) cudaStreamDestroy(h->side_stream);
    if (h->ev_fork) cudaEventDestroy(h->ev_fork);
    if (h->ev_join) cudaEventDestroy(h->ev_join);
    delete h;
    return fail(MTB200_ERR_CUDA, "handle set-up failed: %s", cudaGetErrorString(e));
  }
  h->stream = h->own_stream;
  *out = h;
  return MTB200_OK;
}

int32_t mtb200_destroy(mtb200_handle h) {
  if (!h) return MTB200_OK;
  DeviceGuard guard(h->device);
  cudaStreamSynchronize(h->stream);
  for (auto& r : h->prof) {
    cudaEventDestroy(r.start);
    cudaEventDestroy(r.stop);
  }
  if (h->workspace) cudaFree(h->workspace);
  if (h->status) cudaFree(h->status);
  if (h->status_host) cudaFreeHost(h->status_host);
  if (h->tail_partial) cudaFree(h->tail_partial);
  if (h->side_stream) {
    cudaStreamSynchronize(h->side_stream);
    cudaStreamDestroy(h->side_stream);
  }
  if (h->ev_fork) cudaEventDestroy(h->ev_fork);
  if (h->ev_join) cudaEventDestroy(h->ev_join);
  if (h->own_stream) cudaStreamDestroy(h->own_stream);
  delete h;
  return MTB200_OK;
}

int32_t mtb200_set_stream(mtb200_handle h, void* cuda_stream) {
  MTB_CHECK_HANDLE(h);
  // No ordering is added between the old and the new stream: a host that moves a handle between streams (the
  // data-parallel trainer runs Adam on a second stream while the backward pass continues on the first) orders them
  // itself with events, and an implicit join here would serialise exactly the overlap it set up (measured at 8
  // GPUs: 8.0 -> 8.7 ms per step).  Calls that share the handle's workspace or flag words must therefore be
  // ordered by the caller when they are issued on different streams.
  h->stream = static_cast<cudaStream_t>(cuda_stream);
  return MTB200_OK;
}

int32_t mtb200_set_gemm_sm_limit(mtb200_handle h, int32_t sms) {
  MTB_CHECK_HANDLE(h);
  if (sms < 0) return fail(MTB200_ERR_INVALID, "negative SM count");
  h->gemm_sm_limit = (sms == 0 || sms >= h->sm_count) ? 0 : std::max(2, sms);
  return MTB200_OK;
}

int32_t mtb200_sync(mtb200_handle h) {
  MTB_CHECK_HANDLE(h);
  MTB_CUDA(cudaMemcpyAsync(h->status_host, h->status, 2 * sizeof(uint32_t), cudaMemcpyDeviceToHost,
                           h->stream));
  MTB_CUDA(cudaStreamSynchronize(h->stream));
  const uint32_t wait_code = h->status_host[0], bad_label = h->status_host[1];
  if (wait_code || bad_label) {
    MTB_CUDA(cudaMemsetAsync(h->status, 0, 2 * sizeof(uint32_t), h->stream));
    MTB_CUDA(cudaStreamSynchronize(h->stream));
    if (wait_code)
      return fail(MTB200_ERR_DEVICE_WAIT,
                  "a bounded wait inside a GEMM kernel ran out (role %u, site %u); results are invalid",
                  wait_code >> 8, wait_code & 0xffu);
    return fail(MTB200_ERR_BAD_LABEL, "cross entropy saw a class index outside [0, C)");
  }
  return MTB200_OK;
}

int32_t mtb200_profile_enable(mtb200_handle h, int32_t on) {
  MTB_CHECK_HANDLE(h);
  for (auto& r : h->prof) {
    cudaEventDestroy(r.start);
    cudaEventDestroy(r.stop);
  }
  h->prof.clear();
  h->profiling = on != 0;
  return MTB200_OK;
}

int32_t mtb200_profile_read(mtb200_handle h, int32_t kernel_class, int64_t* launches, double* total_ms,
                            double* total_work) {
  MTB_CHECK_HANDLE(h);
  if (kernel_class < 0 || kernel_class >= PROF_NUM) return fail(MTB200_ERR_INVALID, "unknown kernel class %d", kernel_class);
  if (!launches || !total_ms || !total_work) return fail(MTB200_ERR_INVALID, "null output pointer");
  MTB_CUDA(cudaStreamSynchronize(h->stream));
  int64_t n = 0;
  double ms = 0.0, work = 0.0;
  for (auto& r : h->prof) {
    if (r.cls != kernel_class) continue;
    float t = 0.0f;
    MTB_CUDA(cudaEventElapsedTime(&t, r.start, r.stop));
    ms += t;
    work += r.work;
    ++n;
  }
  *launches = n; *total_ms = ms; *total_work = work;
  return MTB200_OK;
}

int32_t mtb200_workspace_bytes(mtb200_handle h, size_t* bytes) {
  if (!h || !bytes) return fail(MTB200_ERR_INVALID, "null argument");
  *bytes = h->workspace_bytes;
  return MTB200_OK;
}

int32_t mtb200_alloc(mtb200_handle h, size_t bytes, void** dptr) {
  MTB_CHECK_HANDLE(h);
  if (!dptr) return fail(MTB200_ERR_INVALID, "null output pointer");
  *dptr = nullptr;
  if (bytes == 0) return MTB200_OK;
  cudaError_t e = cudaMalloc(dptr, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    *dptr = nullptr;
    return fail(MTB200_ERR_NOMEM, "device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
  }
  return MTB200_OK;
}

int32_t mtb200_free(mtb200_handle h, void* dptr, size_t bytes) {
  MTB_CHECK_HANDLE(h);
  (void)bytes;
  if (!dptr) return MTB200_OK;
  MTB_CUDA(cudaStreamSynchronize(h->stream));
  MTB_CUDA(cudaFree(dptr));
  return MTB200_OK;
}

int32_t mtb200_h2d(mtb200_handle h, void* dst, const void* src, size_t bytes) {
  MTB_CHECK_HANDLE(h);
  if (bytes == 0) return MTB200_OK;
  if (!dst || !src) return fail(MTB200_ERR_INVALID, "null pointer in host-to-device copy");
  MTB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, h->stream));
  return MTB200_OK;
}

int32_t mtb200_d2h(mtb200_handle h, void* dst, const void* src, size_t bytes) {
  MTB_CHECK_HANDLE(h);
  if (bytes == 0) return MTB200_OK;
  if (!dst || !src) return fail(MTB200_ERR_INVALID, "null pointer in device-to-host copy");
  MTB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, h->stream));
  MTB_CUDA(cudaStreamSynchronize(h->stream));
  return MTB200_OK;
}

int32_t mtb200_memset_zero(mtb200_handle h, void* dptr, size_t bytes) {
  MTB_CHECK_HANDLE(h);
  if (bytes == 0) return MTB200_OK;
  if (!dptr) return fail(MTB200_ERR_INVALID, "null pointer");
  MTB_CUDA(cudaMemsetAsync(dptr, 0, bytes, h->stream));
  return MTB200_OK;
}

// ------------------------------------------------------------------ GEMM
static size_t dtype_size(int32_t dt) {
  switch (dt) {
    case MTB200_F32: case MTB200_I32: return 4;
    case MTB200_F64: case MTB200_I64: return 8;
    default: return 0;
  }
}

int32_t mtb200_gemm(mtb200_handle h, int32_t dtype, int32_t trans_a, int32_t trans_b, int64_t batch,
                    int64_t M, int64_t N, int64_t K, const void* A, int64_t stride_a, const void* B,
                    int64_t stride_b, void* C, int64_t stride_c, const void* bias, int32_t epilogue,
                    const void* aux, int32_t f32_mode) {
  MTB_CHECK_HANDLE(h);
  if (dtype == MTB200_BOOL)
    return fail(MTB200_ERR_UNSUPPORTED, "Matrix multiplication not supported for boolean tensors");
  const size_t es = dtype_size(dtype);
  if (es == 0) return fail(MTB200_ERR_INVALID, "unknown dtype %d", dtype);
  if (batch < 0 || M < 0 || N < 0 || K < 0) return fail(MTB200_ERR_INVALID, "negative dimension");
  if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX || batch > 65535)
    return fail(MTB200_ERR_INVALID, "dimension exceeds the 32-bit limit of the device kernels");
  if (epilogue < 0 || epilogue > MTB200_EPI_RELU_BWD) return fail(MTB200_ERR_INVALID, "unknown epilogue %d", epilogue);
  const bool is_float = (dtype == MTB200_F32 || dtype == MTB200_F64);
  if (!is_float && (epilogue != MTB200_EPI_NONE || bias))
    return fail(MTB200_ERR_UNSUPPORTED, "bias and activation epilogues need a floating dtype");
  if (epilogue == MTB200_EPI_RELU_BWD && !aux) return fail(MTB200_ERR_INVALID, "RELU_BWD epilogue needs aux");
  if (batch == 0 || M == 0 || N == 0) return MTB200_OK;  // nothing to write
  if (!C) return fail(MTB200_ERR_INVALID, "null output pointer");
  if (K > 0 && (!A || !B)) return fail(MTB200_ERR_INVALID, "null operand pointer");
  if (stride_c < M * N && batch > 1) return fail(MTB200_ERR_INVALID, "output batch stride overlaps");

  if (K == 0) {
    // Empty reduction: the reference leaves the zero-initialised output
    // (matmul.rs:373-376); a fused bias / activation still applies.
    for (int64_t b = 0; b < batch; ++b) {
      char* cb = static_cast<char*>(C) + b * stride_c * es;
      if (dtype == MTB200_F32) {
        const float* ax = aux ? static_cast<const float*>(aux) + b * stride_c : nullptr;
        if (epilogue == MTB200_EPI_RELU_BWD) {
          MTB_CUDA(cudaMemsetAsync(cb, 0, size_t(M) * N * es, h->stream));  // 0 * mask, bias added first
          if (bias) {
            bias_act_kernel<float><<<grid_for(M * N, 256, h->sm_count), 256, 0, h->stream>>>(
                nullptr, static_cast<const float*>(bias), reinterpret_cast<float*>(cb), M, int(N), N, 0);
            act_bwd_kernel<float><<<grid_for(M * N, 256, h->sm_count), 256, 0, h->stream>>>(
                ax, reinterpret_cast<float*>(cb), reinterpret_cast<float*>(cb), M * N, 1);
          }
        } else {
          bias_act_kernel<float><<<grid_for(M * N, 256, h->sm_count), 256, 0, h->stream>>>(
              nullptr, static_cast<const float*>(bias), reinterpret_cast<float*>(cb), M, int(N), N, epilogue);
        }
      } else if (dtype == MTB200_F64) {
        const double* ax = aux ? static_cast<const double*>(aux) + b * stride_c : nullptr;
        if (epilogue == MTB200_EPI_RELU_BWD) {
          MTB_CUDA(cudaMemsetAsync(cb, 0, size_t(M) * N * es, h->stream));
          if (bias) {
            bias_act_kernel<double><<<grid_for(M * N, 256, h->sm_count), 256, 0, h->stream>>>(
                nullptr, static_cast<const double*>(bias), reinterpret_cast<double*>(cb), M, int(N), N, 0);
            act_bwd_kernel<double><<<grid_for(M * N, 256, h->sm_count), 256, 0, h->stream>>>(
                ax, reinterpret_cast<double*>(cb), reinterpret_cast<double*>(cb), M * N, 1);
          }
        } else {
          bias_act_kernel<double><<<grid_for(M * N, 256, h->sm_count), 256, 0, h->stream>>>(
              nullptr, static_cast<const double*>(bias), reinterpret_cast<double*>(cb), M, int(N), N, epilogue);
        }
      } else {
        MTB_CUDA(cudaMemsetAsync(cb, 0, size_t(M) * N * es, h->stream));
      }
    }
    MTB_CUDA(cudaGetLastError());
    return MTB200_OK;
  }

  if (dtype == MTB200_F32) {
    const int mode = f32_mode & 0xff, variant = (f32_mode >> 8) & 0xff;
    return gemm_f32_split(h, trans_a != 0, trans_b != 0, int(batch), int(M), int(N), int(K),
                          static_cast<const float*>(A), stride_a, static_cast<const float*>(B), stride_b,
                          static_cast<float*>(C), N, stride_c, static_cast<const float*>(bias), epilogue,
                          static_cast<const float*>(aux), mode, variant);
  }

  // int32: the tensor-core limb path once the product is large enough to amortise the limb split
  // (f32_mode variant byte 0xfe forces the CUDA-core kernel, 0xfd forces the tensor path)
  if (dtype == MTB200_I32) {
    const int variant = (f32_mode >> 8) & 0xff;
    const bool big = double(M) * double(N) * double(K) >= double(1 << 24) && K >= 64;
    if ((big && variant != 0xfe) || variant == 0xfd)
      return gemm_i32_limb(h, trans_a != 0, trans_b != 0, int(batch), int(M), int(N), int(K), static_cast<const int32_t*>(A),
                           stride_a, static_cast<const int32_t*>(B), stride_b, static_cast<int32_t*>(C), stride_c);
  }
  StridedGemmArgs g;
  g.M = int(M); g.N = int(N); g.K = int(K); g.batch = int(batch);
  g.A = A; g.B = B; g.C = C;
  g.a_si = trans_a ? 1 : K;  g.a_sk = trans_a ? M : 1;  g.a_sb = stride_a;
  g.b_sk = trans_b ? 1 : N;  g.b_sj = trans_b ? K : 1;  g.b_sb = stride_b;
  g.ldc = N; g.c_sb = stride_c;
  g.bias = bias; g.aux = aux; g.epilogue = epilogue;
  g.gate = nullptr; g.gate_value = 0;
  ProfScope prof(h, dtype == MTB200_F64 ? PROF_GEMM_F64 : PROF_GEMM_INT, 2.0 * M * N * K * batch);
  if (dtype == MTB200_F64) {
    const int smem = 4 * D_BK * D_PITCH * int(sizeof(double));
    const long long tiles = ((M + D_BM - 1) / D_BM) * ((N + D_BN - 1) / D_BN);
    if (int32_t rc_attr = grant_dynamic_smem(h, gemm_f64_dmma_kernel<2, 4>, int(smem))) return rc_attr;
    gemm_f64_dmma_kernel<2, 4><<<dim3(unsigned(tiles), unsigned(batch)), 256, smem, h->stream>>>(g);
  } else if (dtype == MTB200_I32) {
    const long long tiles = ((M + 127) / 128) * ((N + 127) / 128);
    gemm_simt_kernel<uint32_t, 8, 8><<<dim3(unsigned(tiles), unsigned(batch)), 256, 0, h->stream>>>(g);
  } else {
    const long long tiles = ((M + 127) / 128) * ((N + 63) / 64);
    gemm_simt_kernel<unsigned long long, 8, 4><<<dim3(unsigned(tiles), unsigned(batch)), 256, 0, h->stream>>>(g);
  }
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

// ------------------------------------------------------------------ column sum
int32_t mtb200_colsum(mtb200_handle h, int32_t dtype, int64_t M, int64_t N, const void* X, void* out) {
  MTB_CHECK_HANDLE(h);
  if (dtype != MTB200_F32 && dtype != MTB200_F64)
    return fail(MTB200_ERR_UNSUPPORTED, "column sum supports f32 and f64");
  if (M < 0 || N < 0 || M > INT32_MAX || N > INT32_MAX) return fail(MTB200_ERR_INVALID, "bad dimension");
  if (N == 0) return MTB200_OK;
  if (!out) return fail(MTB200_ERR_INVALID, "null output pointer");
  const size_t es = dtype_size(dtype);
  if (M == 0) {
    MTB_CUDA(cudaMemsetAsync(out, 0, size_t(N) * es, h->stream));
    return MTB200_OK;
  }
  if (!X) return fail(MTB200_ERR_INVALID, "null input pointer");
  const int cols_per_block = 8 * int(16 / es);
  const int col_blocks = int((N + cols_per_block - 1) / cols_per_block);
  // enough bands to fill the machine a few times over, at least 32 rows each
  int bands = int(std::min<int64_t>((M + 31) / 32, std::max<int64_t>(1, (int64_t(h->sm_count) * 8) / col_blocks)));
  bands = std::max(1, std::min(bands, 1024));
  const int rows_per_band = int((M + bands - 1) / bands);
  bands = int((M + rows_per_band - 1) / rows_per_band);
  void* ws = nullptr;
  int32_t rc = workspace_reserve(h, size_t(bands) * N * es, &ws);
  if (rc) return rc;
  if (dtype == MTB200_F32) {
    colsum_stage1_kernel<float><<<dim3(col_blocks, bands), 256, 0, h->stream>>>(
        static_cast<const float*>(X), N, int(M), int(N), rows_per_band, static_cast<float*>(ws));
    MTB_CUDA(launch_pdl(h, colsum_stage2_kernel<float>, dim3(unsigned((N + 255) / 256)), dim3(256), 0,
                        static_cast<const float*>(ws), bands, int(N), static_cast<float*>(out)));
  } else {
    colsum_stage1_kernel<double><<<dim3(col_blocks, bands), 256, 0, h->stream>>>(
        static_cast<const double*>(X), N, int(M), int(N), rows_per_band, static_cast<double*>(ws));
    MTB_CUDA(launch_pdl(h, colsum_stage2_kernel<double>, dim3(unsigned((N + 255) / 256)), dim3(256), 0,
                        static_cast<const double*>(ws), bands, int(N), static_cast<double*>(out)));
  }
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

// ------------------------------------------------------------------ dense layer
static bool dense_uses_saved(int32_t dtype, int64_t rows, int64_t in, int64_t out) {
  return dtype == MTB200_F32 && dense_fused_shapes(rows, in, out) && rows <= INT32_MAX && in <= INT32_MAX &&
         out <= INT32_MAX;
}

int32_t mtb200_dense_saved_bytes(int32_t dtype, int64_t rows, int64_t in_features, int64_t out_features,
                                 size_t* bytes) {
  if (!bytes) return fail(MTB200_ERR_INVALID, "null output pointer");
  if (dtype != MTB200_F32 && dtype != MTB200_F64) return fail(MTB200_ERR_UNSUPPORTED, "dense layer: dtype must be f32 or f64");
  if (rows < 0 || in_features < 0 || out_features < 0) return fail(MTB200_ERR_INVALID, "negative dimension");
  *bytes = dense_uses_saved(dtype, rows, in_features, out_features)
               ? dense_saved_layout(rows, in_features, out_features).total
               : 0;
  return MTB200_OK;
}

int32_t mtb200_dense_forward(mtb200_handle h, int32_t dtype, int64_t rows, int64_t in_features,
                             int64_t out_features, const void* x, const void* W, const void* bias,
                             int32_t epilogue, void* y, void* saved) {
  MTB_CHECK_HANDLE(h);
  if (dtype != MTB200_F32 && dtype != MTB200_F64) return fail(MTB200_ERR_UNSUPPORTED, "dense layer: dtype must be f32 or f64");
  if (epilogue < 0 || epilogue > MTB200_EPI_GELU_TANH)
    return fail(MTB200_ERR_INVALID, "dense forward epilogue must be NONE, RELU or GELU");
  if (!saved || !dense_uses_saved(dtype, rows, in_features, out_features))
    return mtb200_gemm(h, dtype, 0, 1, 1, rows, out_features, in_features, x, 0, W, 0, y, 0, bias, epilogue, nullptr, 0);
  if (!x || !W || !y) return fail(MTB200_ERR_INVALID, "null pointer");
  return dense_forward_f32(h, int(rows), int(in_features), int(out_features), static_cast<const float*>(x),
                           static_cast<const float*>(W), static_cast<const float*>(bias), epilogue, nullptr,
                           static_cast<float*>(y), saved);
}

int32_t mtb200_dense_dy_bytes(int32_t dtype, int64_t rows, int64_t in_features, int64_t out_features, size_t* bytes) {
  if (!bytes) return fail(MTB200_ERR_INVALID, "null output pointer");
  if (dtype != MTB200_F32 && dtype != MTB200_F64) return fail(MTB200_ERR_UNSUPPORTED, "dense layer: dtype must be f32 or f64");
  if (rows < 0 || in_features < 0 || out_features < 0) return fail(MTB200_ERR_INVALID, "negative dimension");
  *bytes = dense_uses_saved(dtype, rows, in_features, out_features) ? dense_dy_layout(rows, out_features).total : 0;
  return MTB200_OK;
}

int32_t mtb200_dense_backward(mtb200_handle h, int32_t dtype, int64_t rows, int64_t in_features,
                              int64_t out_features, const void* x, const void* W, const void* dY,
                              const void* saved, void* dX, int32_t dx_epilogue, const void* dx_aux,
                              void* dW, void* db, void* dy_block, int32_t dy_mode) {
  MTB_CHECK_HANDLE(h);
  if (dtype != MTB200_F32 && dtype != MTB200_F64) return fail(MTB200_ERR_UNSUPPORTED, "dense layer: dtype must be f32 or f64");
  if (dx_epilogue != MTB200_EPI_NONE && dx_epilogue != MTB200_EPI_RELU_BWD)
    return fail(MTB200_ERR_INVALID, "dense backward epilogue must be NONE or RELU_BWD");
  if (dX && dx_epilogue == MTB200_EPI_RELU_BWD && !dx_aux) return fail(MTB200_ERR_INVALID, "RELU_BWD epilogue needs aux");
  if (dy_mode < 0 || dy_mode > 2) return fail(MTB200_ERR_INVALID, "dy_mode must be 0, 1 or 2");
  if (dy_mode == 1 && dW) return fail(MTB200_ERR_INVALID, "dy_mode 1 prepares dY for a LATER weight-gradient call: dW must be NULL");
  if (dy_mode == 2 && (dX || db)) return fail(MTB200_ERR_INVALID, "dy_mode 2 does not read dY: dX and db must be NULL");
  const bool fused = saved && dense_uses_saved(dtype, rows, in_features, out_features);
  if (!fused || !dy_block) dy_mode = 0;  // plain products keep nothing between calls
  if (!fused) {
    int32_t rc = MTB200_OK;
    if (dW) {
      rc = mtb200_gemm(h, dtype, 1, 0, 1, out_features, in_features, rows, dY, 0, x, 0, dW, 0, nullptr,
                       MTB200_EPI_NONE, nullptr, 0);
      if (rc) return rc;
    }
    if (dX) {
      rc = mtb200_gemm(h, dtype, 0, 0, 1, rows, in_features, out_features, dY, 0, W, 0, dX, 0, nullptr, dx_epilogue,
                       dx_aux, 0);
      if (rc) return rc;
    }
    if (db) return mtb200_colsum(h, dtype, rows, out_features, dY, db);
    return MTB200_OK;
  }
  if (!x || !W || !dY) return fail(MTB200_ERR_INVALID, "null pointer");
  return dense_backward_f32(h, int(rows), int(in_features), int(out_features), static_cast<const float*>(x),
                            static_cast<const float*>(W), static_cast<const float*>(dY), saved,
                            static_cast<float*>(dX), dx_epilogue, static_cast<const float*>(dx_aux),
                            static_cast<float*>(dW), static_cast<float*>(db), dy_block, dy_mode);
}

// ------------------------------------------------------------------ activations
int32_t mtb200_act_fwd(mtb200_handle h, int32_t dtype, int32_t act, int64_t n, const void* x, void* y) {
  MTB_CHECK_HANDLE(h);
  if (act < 1 || act > 3) return fail(MTB200_ERR_INVALID, "unknown activation %d", act);
  if (n < 0) return fail(MTB200_ERR_INVALID, "negative length");
  if (n == 0) return MTB200_OK;
  if (!x || !y) return fail(MTB200_ERR_INVALID, "null pointer");
  if (dtype == MTB200_F32)
    act_fwd_kernel<float><<<grid_for(n, 256, h->sm_count), 256, 0, h->stream>>>(
        static_cast<const float*>(x), static_cast<float*>(y), n, act);
  else if (dtype == MTB200_F64)
    act_fwd_kernel<double><<<grid_for(n, 256, h->sm_count), 256, 0, h->stream>>>(
        static_cast<const double*>(x), static_cast<double*>(y), n, act);
  else
    return fail(MTB200_ERR_UNSUPPORTED, "activations support f32 and f64");
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

int32_t mtb200_act_bwd(mtb200_handle h, int32_t dtype, int32_t act, int64_t n, const void* ref,
                       const void* dy, void* dx) {
  MTB_CHECK_HANDLE(h);
  if (act < 1 || act > 3) return fail(MTB200_ERR_INVALID, "unknown activation %d", act);
  if (n < 0) return fail(MTB200_ERR_INVALID, "negative length");
  if (n == 0) return MTB200_OK;
  if (!ref || !dy || !dx) return fail(MTB200_ERR_INVALID, "null pointer");
  if (dtype == MTB200_F32)
    act_bwd_kernel<float><<<grid_for(n, 256, h->sm_count), 256, 0, h->stream>>>(
        static_cast<const float*>(ref), static_cast<const float*>(dy), static_cast<float*>(dx), n, act);
  else if (dtype == MTB200_F64)
    act_bwd_kernel<double><<<grid_for(n, 256, h->sm_count), 256, 0, h->stream>>>(
        static_cast<const double*>(ref), static_cast<const double*>(dy), static_cast<double*>(dx), n, act);
  else
    return fail(MTB200_ERR_UNSUPPORTED, "activations support f32 and f64");
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

int32_t mtb200_bias_act(mtb200_handle h, int32_t dtype, int64_t M, int64_t N, const void* x,
                        const void* bias, int32_t act, void* y) {
  MTB_CHECK_HANDLE(h);
  if (act < 0 || act > 3) return fail(MTB200_ERR_INVALID, "unknown activation %d", act);
  if (M < 0 || N < 0 || N > INT32_MAX) return fail(MTB200_ERR_INVALID, "bad dimension");
  if (M == 0 || N == 0) return MTB200_OK;
  if (!x || !y) return fail(MTB200_ERR_INVALID, "null pointer");
  if (dtype == MTB200_F32)
    bias_act_kernel<float><<<grid_for(M * N, 256, h->sm_count), 256, 0, h->stream>>>(
        static_cast<const float*>(x), static_cast<const float*>(bias), static_cast<float*>(y), M, int(N), N, act);
  else if (dtype == MTB200_F64)
    bias_act_kernel<double><<<grid_for(M * N, 256, h->sm_count), 256, 0, h->stream>>>(
        static_cast<const double*>(x), static_cast<const double*>(bias), static_cast<double*>(y), M, int(N), N, act);
  else
    return fail(MTB200_ERR_UNSUPPORTED, "bias add supports f32 and f64");
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

// ------------------------------------------------------------------ cross entropy
int32_t mtb200_cross_entropy(mtb200_handle h, int64_t B, int64_t C, const float* logits,
                             const void* labels, int32_t label_dtype, int32_t mean, float upstream,
                             float* loss, float* dlogits) {
  MTB_CHECK_HANDLE(h);
  if (B <= 0 || C <= 0 || B > INT32_MAX || C > INT32_MAX)
    return fail(MTB200_ERR_INVALID, "cross entropy needs a non-empty [B,C] logits matrix");
  if (!logits || !labels || !loss) return fail(MTB200_ERR_INVALID, "null pointer");
  if (label_dtype != MTB200_I32 && label_dtype != MTB200_I64)
    return fail(MTB200_ERR_UNSUPPORTED, "Unsupported target dtype for classification loss");
  void* ws = nullptr;
  int32_t rc = workspace_reserve(h, size_t(B) * sizeof(float), &ws);
  if (rc) return rc;
  float* row_loss = static_cast<float*>(ws);
  const float inv = mean ? float(1.0 / double(B)) : 1.0f;
  const float gscale = inv * upstream;
  const int blocks = int((B * 32 + 255) / 256);
  if (label_dtype == MTB200_I32)
    cross_entropy_rows_kernel<int32_t><<<blocks, 256, 0, h->stream>>>(
        logits, static_cast<const int32_t*>(labels), int(B), int(C), gscale, row_loss, dlogits, h->status + 1);
  else
    cross_entropy_rows_kernel<long long><<<blocks, 256, 0, h->stream>>>(
        logits, static_cast<const long long*>(labels), int(B), int(C), gscale, row_loss, dlogits, h->status + 1);
  loss_reduce_kernel<<<1, 1024, 0, h->stream>>>(row_loss, int(B), inv, loss);
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

// ------------------------------------------------------------------ Adam
int32_t mtb200_adam_step(mtb200_handle h, int64_t n, float* param, const float* grad, float* m,
                         float* v, double lr, double beta1, double beta2, double eps,
                         double weight_decay, int32_t decoupled, int64_t step, float grad_scale) {
  MTB_CHECK_HANDLE(h);
  if (n < 0) return fail(MTB200_ERR_INVALID, "negative length");
  if (step < 1 || step > INT32_MAX) return fail(MTB200_ERR_INVALID, "step count must be >= 1");
  if (n == 0) return MTB200_OK;
  if (!param || !grad || !m || !v) return fail(MTB200_ERR_INVALID, "null pointer");
  const double bc1_inv = 1.0 / (1.0 - powi_f64(beta1, int(step)));
  const double bc2_inv = 1.0 / (1.0 - powi_f64(beta2, int(step)));
  const int dec = (decoupled && weight_decay != 0.0) ? 1 : 0;
  adam_kernel<<<grid_for(n, 256, h->sm_count), 256, 0, h->stream>>>(
      param, grad, m, v, n, float(lr), float(beta1), float(beta2), float(eps), float(weight_decay),
      float(bc1_inv), float(bc2_inv), dec, grad_scale);
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

int32_t mtb200_adam_step_counted(mtb200_handle h, int64_t n, float* param, const float* grad, float* m, float* v,
                                 double lr, double beta1, double beta2, double eps, double weight_decay,
                                 int32_t decoupled, int64_t* step_counter, int32_t advance, float grad_scale) {
  MTB_CHECK_HANDLE(h);
  if (n < 0) return fail(MTB200_ERR_INVALID, "negative length");
  if (!step_counter) return fail(MTB200_ERR_INVALID, "null step counter");
  if (advance)
    counter_add_kernel<<<1, 1, 0, h->stream>>>(reinterpret_cast<long long*>(step_counter), 1);
  if (n > 0) {
    if (!param || !grad || !m || !v) return fail(MTB200_ERR_INVALID, "null pointer");
    const int dec = (decoupled && weight_decay != 0.0) ? 1 : 0;
    adam_counted_kernel<<<grid_for(n, 256, h->sm_count), 256, 0, h->stream>>>(
        param, grad, m, v, n, float(lr), beta1, beta2, float(eps), float(weight_decay),
        reinterpret_cast<const long long*>(step_counter), dec, grad_scale);
  }
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

// ------------------------------------------------------------------ bounded-wait self-test
namespace mtb {
// One thread waits on a barrier that nothing signals, with the same loop shape as mbar_wait but a caller-chosen
// limit, and reports the expiry through the status word exactly as the GEMM kernels' roles do (role 15, site 1).
__global__ void wait_expiry_selftest_kernel(uint32_t* __restrict__ status, unsigned long long limit_ns) {
  __shared__ __align__(8) unsigned long long bar;
  const uint32_t b = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(b, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint64_t t0 = globaltimer_ns();
    bool done = mbar_try_wait(b, 0);
    uint32_t spins = 0;
    while (!done) {
      done = mbar_try_wait(b, 0);
      if ((++spins & 0x3f) == 0 && globaltimer_ns() - t0 > limit_ns) break;
    }
    if (!done) atomicMax(status, 0xF00u | 1u);
  }
}
}  // namespace mtb

int32_t mtb200_selftest_wait_expiry(mtb200_handle h, int32_t limit_us) {
  MTB_CHECK_HANDLE(h);
  if (limit_us < 1 || limit_us > 100000) return fail(MTB200_ERR_INVALID, "limit must be 1 .. 100000 microseconds");
  mtb::wait_expiry_selftest_kernel<<<1, 32, 0, h->stream>>>(h->status, 1000ull * static_cast<unsigned long long>(limit_us));
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}

}  // extern "C"
