// Handle, error reporting, scratch memory and tensor-map helpers shared by the
// C-ABI translation units.
#pragma once
#include <utility>
#include <mutex>
#include <map>
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/mtb200.h"

namespace mtb {

extern thread_local std::string g_last_error;

inline int32_t fail(int32_t code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

#define MTB_CUDA(expr)                                                                    \
  do {                                                                                    \
    cudaError_t e__ = (expr);                                                             \
    if (e__ != cudaSuccess)                                                               \
      return ::mtb::fail(e__ == cudaErrorMemoryAllocation ? MTB200_ERR_NOMEM : MTB200_ERR_CUDA, \
                         "%s failed: %s", #expr, cudaGetErrorString(e__));                \
  } while (0)

}  // namespace mtb

// Device status word layout: [0] expired-wait code of the GEMM kernels,
// [1] bad-label flag of cross entropy, [2..3] unused, [4 .. 4 + MTB_FLAG_SLOTS) a ring of per-call
// flag words.  A call that needs a data-dependent decision on the device (an f32 product whose
// operands hold Inf / NaN, an int32 product with an operand element outside the int8 range) takes
// the next slot, clears it on its stream, lets its preparation kernels set it to 1 and gates the
// kernels that depend on it by (word != 0).  Clear, set and test are all stream-ordered work of the
// one call, so a call captured into a CUDA graph decides afresh on every replay.
struct mtb200_ctx {
  int device = 0;
  int sm_count = 0;
  cudaStream_t own_stream = nullptr;
  cudaStream_t stream = nullptr;
  // second stream + fork/join events: the two operands of a mid-size GEMM are prepared side by side
  cudaStream_t side_stream = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  int gemm_sm_limit = 0;            // SMs the persistent tensor kernels may occupy (0 = all), see mtb200_set_gemm_sm_limit
  float* tail_partial = nullptr;    // raw partial accumulators of split tail tiles (256 x 256 slots)
  size_t tail_partial_slots = 0;
  void* workspace = nullptr;
  size_t workspace_bytes = 0;
  uint32_t* status = nullptr;       // device, 4 + MTB_FLAG_SLOTS words
  uint32_t* status_host = nullptr;  // pinned, 2 words
  uint32_t epoch = 0;               // call counter: picks the flag slot of a call
  // optional per-launch timing (mtb200_profile_*): event pairs around kernels
  struct ProfRec { cudaEvent_t start, stop; double work; int cls; };
  bool profiling = false;
  bool pdl = true;             // programmatic dependent launch between a call's kernels (MTB200_NO_PDL=1 turns it off)
  std::vector<ProfRec> prof;
  // per-kernel set-up that costs microseconds of host time and does not change: the largest dynamic shared-memory
  // size already granted to a kernel on this device, and the cluster occupancy of the pair-tile kernels
  std::unordered_map<const void*, int> cluster_occupancy;
};

namespace mtb {

// Make the handle's device current for the duration of a call.
struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
    if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    want = dev;
  }
  ~DeviceGuard() {
    if (prev >= 0 && prev != want) cudaSetDevice(prev);
  }
  int want = -1;
};

// Scratch memory of at least `bytes`, valid for work enqueued on the handle's
// stream until the next call that asks for more.  Growing synchronises the
// stream first so no kernel still reads the old block.
int32_t workspace_reserve(mtb200_ctx* h, size_t bytes, void** out);

// cuTensorMapEncodeTiled looked up through the runtime (no link-time
// dependency on libcuda, so the library also loads on a machine without a driver).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled();

// 3-D bf16 tensor map over split planes: dims {Kp, rows, planes}, box {bk, box_rows, 1}.
int32_t make_split_tmap(CUtensorMap* out, const void* base, uint64_t Kp, uint64_t rows,
                        uint64_t planes, uint32_t bk, uint32_t box_rows);

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// cudaFuncAttributeMaxDynamicSharedMemorySize for `fn` on the handle's device, raised only when a launch needs more
// than any earlier one asked for.  The attribute belongs to the (device, function) pair, not to a handle: a second
// handle on the same device that asked for less would LOWER it and make the first handle's next launch fail, so the
// record of what has been granted is shared by all handles of the process.
template <typename Fn>
inline int32_t grant_dynamic_smem(mtb200_ctx* h, Fn fn, int bytes) {
  static std::mutex mu;
  static std::map<std::pair<int, const void*>, int> granted;
  const std::pair<int, const void*> key(h->device, reinterpret_cast<const void*>(fn));
  std::lock_guard<std::mutex> lock(mu);
  auto it = granted.find(key);
  if (it != granted.end() && it->second >= bytes) return MTB200_OK;
  MTB_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  granted[key] = bytes;
  return MTB200_OK;
}

// Per-call flag word (see the status layout above): takes the next slot of the ring and clears it on
// the handle's stream.  Kernels raise it with atomicMax(word, MTB_FLAG_SET); gated kernels run when
// *word == MTB_FLAG_SET.
constexpr int MTB_FLAG_SLOTS = 64;
constexpr uint32_t MTB_FLAG_SET = 1u;
inline int32_t call_flag_begin(mtb200_ctx* h, uint32_t** word) {
  const uint32_t slot = h->epoch++ % MTB_FLAG_SLOTS;
  uint32_t* w = h->status + 4 + slot;
  // Outside stream capture the words are cleared half a ring at a time, just before the half is handed out again:
  // its previous users are 32 to 64 calls back in the same stream, so their kernels have read them.  (A captured
  // graph replayed in between may leave one of these words set; the call that gets it then repeats its product
  // in the IEEE kernel - slower, still correct.)  Under capture every call clears its own word, because a replay
  // must start from a clear word whatever ran before it.
  constexpr uint32_t HALF = MTB_FLAG_SLOTS / 2;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(h->stream, &cap) != cudaSuccess) { cudaGetLastError(); cap = cudaStreamCaptureStatusActive; }
  if (cap != cudaStreamCaptureStatusNone) {
    MTB_CUDA(cudaMemsetAsync(w, 0, sizeof(uint32_t), h->stream));
  } else if (slot % HALF == 0) {
    MTB_CUDA(cudaMemsetAsync(w, 0, HALF * sizeof(uint32_t), h->stream));
  }
  *word = w;
  return MTB200_OK;
}

// Kernel classes of the launch profiler.
enum ProfClass { PROF_GEMM_UMMA = 0, PROF_SPLIT = 1, PROF_GEMM_F64 = 2, PROF_GEMM_INT = 3, PROF_CONV_GATHER = 4,
                 PROF_NUM = 5 };

// Brackets the launches made in its scope with a CUDA event pair on the handle's
// stream when profiling is on; costs nothing otherwise.
struct ProfScope {
  mtb200_ctx* h;
  bool on;
  cudaEvent_t start = nullptr;
  double work;
  int cls;
  ProfScope(mtb200_ctx* h_, int cls_, double work_) : h(h_), on(h_->profiling), work(work_), cls(cls_) {
    if (!on) return;
    if (cudaEventCreate(&start) != cudaSuccess) { on = false; return; }
    cudaEventRecord(start, h->stream);
  }
  ~ProfScope() {
    if (!on) return;
    cudaEvent_t stop = nullptr;
    if (cudaEventCreate(&stop) != cudaSuccess) { cudaEventDestroy(start); return; }
    cudaEventRecord(stop, h->stream);
    h->prof.push_back({start, stop, work, cls});
  }
};

}  // namespace mtb
