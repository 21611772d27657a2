// Column sum that performs no allocation of any kind.
//
// mtb200_colsum needs scratch memory for its per-band partial sums and takes it
// from the handle's growable workspace, which may call cudaMalloc (and
// synchronise the device) when a larger input arrives.  Some callers cannot
// tolerate that:
// a host application whose own pool owns every byte of device memory and
// forbids foreign allocations (minitensor's memory manager is such a pool),
// or a latency-critical loop that must never hit the implicit device-wide
// synchronisation of cudaMalloc / cudaFree.  For them this entry point keeps
// its scratch in a fixed array that is part of the library image.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <mutex>

#include "mtb200_core.cuh"
#include "rowcol_kernels.cuh"

namespace {

// Fixed scratch: every GPU that loads the library holds these bytes until the
// process exits.  It bounds the input width: N * sizeof(element) <= this size.
constexpr size_t kScratchBytes = MTB200_COLSUM_NOALLOC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_colsum_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_addr[kMaxDevices] = {};  // device address of g_colsum_scratch, per device ordinal

// In host code `g_colsum_scratch` is only a handle for the runtime, not an
// address a kernel may use; the real device address must be asked for, once per
// device, while that device is current.
int32_t scratch_for_current_device(void** out) {
  int dev = -1;
  MTB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return mtb::fail(MTB200_ERR_INVALID, "device ordinal %d is not supported", dev);
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_colsum_scratch);
    if (e != cudaSuccess || !p) {
      cudaGetLastError();
      return mtb::fail(MTB200_ERR_CUDA, "cudaGetSymbolAddress for the fixed scratch failed: %s", cudaGetErrorString(e));
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return MTB200_OK;
}

}  // namespace

extern "C" int32_t mtb200_colsum_noalloc(void* cuda_stream, int32_t dtype, int64_t M, int64_t N, const void* X,
                                         void* out) {
  using namespace mtb;
  if (dtype != MTB200_F32 && dtype != MTB200_F64) return fail(MTB200_ERR_UNSUPPORTED, "column sum supports f32 and f64");
  if (M < 0 || N < 0 || M > INT32_MAX || N > INT32_MAX) return fail(MTB200_ERR_INVALID, "bad dimension");
  if (N == 0) return MTB200_OK;
  if (!out) return fail(MTB200_ERR_INVALID, "null output pointer");
  const size_t es = dtype == MTB200_F32 ? 4 : 8;
  if (size_t(N) * es > kScratchBytes)
    return fail(MTB200_ERR_INVALID,
                "mtb200_colsum_noalloc: %lld columns of %zu bytes exceed the fixed scratch of %zu bytes "
                "(at most %zu columns); use mtb200_colsum",
                (long long)N, es, kScratchBytes, kScratchBytes / es);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (M == 0) {
    MTB_CUDA(cudaMemsetAsync(out, 0, size_t(N) * es, stream));
    return MTB200_OK;
  }
  if (!X) return fail(MTB200_ERR_INVALID, "null input pointer");
  void* scratch = nullptr;
  int32_t rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  int dev = 0, sms = 0;
  MTB_CUDA(cudaGetDevice(&dev));
  MTB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int cols_per_block = 8 * int(16 / es);
  const int col_blocks = int((N + cols_per_block - 1) / cols_per_block);
  const int64_t fit = int64_t(kScratchBytes / (size_t(N) * es));  // bands the scratch can hold (>= 1)
  int64_t bands = std::min<int64_t>((M + 31) / 32, std::max<int64_t>(1, (int64_t(sms) * 8) / col_blocks));
  bands = std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(bands, fit), 1024));
  const int rows_per_band = int((M + bands - 1) / bands);
  bands = (M + rows_per_band - 1) / rows_per_band;
  // Stage 1 overwrites every partial it later reads, so nothing left in the
  // scratch by an earlier call is ever consumed.
  if (dtype == MTB200_F32) {
    colsum_stage1_kernel<float><<<dim3(col_blocks, unsigned(bands)), 256, 0, stream>>>(
        static_cast<const float*>(X), N, int(M), int(N), rows_per_band, static_cast<float*>(scratch));
    colsum_stage2_kernel<float><<<int((N + 255) / 256), 256, 0, stream>>>(static_cast<const float*>(scratch),
                                                                        int(bands), int(N), static_cast<float*>(out));
  } else {
    colsum_stage1_kernel<double><<<dim3(col_blocks, unsigned(bands)), 256, 0, stream>>>(
        static_cast<const double*>(X), N, int(M), int(N), rows_per_band, static_cast<double*>(scratch));
    colsum_stage2_kernel<double><<<int((N + 255) / 256), 256, 0, stream>>>(
        static_cast<const double*>(scratch), int(bands), int(N), static_cast<double*>(out));
  }
  MTB_CUDA(cudaGetLastError());
  return MTB200_OK;
}
