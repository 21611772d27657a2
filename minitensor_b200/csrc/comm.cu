// Gradient exchange of data-parallel training behind the C ABI: NCCL all-reduce (sum) of f32 buffers.
//
// The reference has no distributed code; its training loop (engine/src/optim/adam.rs:483-514 after
// engine/src/autograd/graph.rs:222-282) is the single-process step this exchange is inserted into:
// every rank runs the same step on its rows of the batch, the parameter gradients are summed over the
// ranks, and the optimizer applies 1 / world_size.
//
// NCCL is looked up at run time (dlopen of the copy already in the process, else libnccl.so.2 from the
// loader path, else the file named by MTB200_NCCL_LIB), so the library loads and every other entry
// point works on a machine without NCCL; only the mtb200_comm_* calls then fail with
// MTB200_ERR_UNSUPPORTED.  Only the handful of NCCL entry points below are used; their C signatures
// and enum values are NCCL's public, stable ABI.
#include <dlfcn.h>

#include <algorithm>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "mtb200_core.cuh"

namespace mtb {
namespace {

typedef struct ncclComm* ncclComm_t;
struct NcclUniqueId { char internal[128]; };
static_assert(sizeof(NcclUniqueId) == MTB200_COMM_ID_BYTES, "NCCL unique id is 128 bytes");
constexpr int NCCL_FLOAT32 = 7;  // ncclDataType_t::ncclFloat32
constexpr int NCCL_SUM = 0;      // ncclRedOp_t::ncclSum

struct NcclApi {
  void* lib = nullptr;
  int (*GetVersion)(int*) = nullptr;
  int (*GetUniqueId)(NcclUniqueId*) = nullptr;
  int (*CommInitRank)(ncclComm_t*, int, NcclUniqueId, int) = nullptr;
  int (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  std::string why;  // set when loading failed
};

NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* named = getenv("MTB200_NCCL_LIB");
    if (named && *named) api.lib = dlopen(named, RTLD_NOW | RTLD_GLOBAL);
    if (!api.lib) api.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // the copy the host program loaded
    if (!api.lib) api.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!api.lib) api.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!api.lib) {
      const char* e = dlerror();
      api.why = std::string("NCCL could not be loaded (") + (e ? e : "no loader message") +
                "); set MTB200_NCCL_LIB to the path of libnccl.so.2";
      return;
    }
    auto sym = [&](const char* name) -> void* {
      void* p = dlsym(api.lib, name);
      if (!p && api.why.empty()) api.why = std::string("NCCL symbol missing: ") + name;
      return p;
    };
    api.GetVersion = reinterpret_cast<decltype(api.GetVersion)>(sym("ncclGetVersion"));
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommInitAll = reinterpret_cast<decltype(api.CommInitAll)>(sym("ncclCommInitAll"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
    api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
  });
  return api;
}

int32_t nccl_ready() {
  NcclApi& a = nccl();
  if (!a.why.empty()) return fail(MTB200_ERR_UNSUPPORTED, "%s", a.why.c_str());
  return MTB200_OK;
}

int32_t nccl_fail(const char* what, int rc) {
  NcclApi& a = nccl();
  return fail(MTB200_ERR_CUDA, "%s failed: %s", what, a.GetErrorString ? a.GetErrorString(rc) : "NCCL error");
}

__global__ void __launch_bounds__(256) comm_scale_kernel(float* __restrict__ x, size_t n, float s) {
  const size_t n4 = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) ? n / 4 : 0;
  const size_t step = static_cast<size_t>(gridDim.x) * 256;
  for (size_t i = blockIdx.x * size_t(256) + threadIdx.x; i < n4; i += step) {
    float4 v = reinterpret_cast<float4*>(x)[i];
    v.x *= s; v.y *= s; v.z *= s; v.w *= s;
    reinterpret_cast<float4*>(x)[i] = v;
  }
  for (size_t i = n4 * 4 + blockIdx.x * size_t(256) + threadIdx.x; i < n; i += step) x[i] *= s;
}

}  // namespace
}  // namespace mtb

// One communicator object: the NCCL communicators of the ranks THIS process drives (one, when every
// GPU has its own process; ndev, when one process drives all of them), their devices and streams.
struct mtb200_comm_s {
  int world = 0;
  std::vector<int> ranks;                  // global rank of each local communicator
  std::vector<int> devices;
  std::vector<mtb::ncclComm_t> comms;
  std::vector<cudaStream_t> streams;       // stream of each local rank's collectives (default: the legacy default stream)
};

using namespace mtb;

extern "C" {

int32_t mtb200_comm_unique_id(void* id_out) {
  if (!id_out) return fail(MTB200_ERR_INVALID, "null id buffer");
  int32_t rc = nccl_ready();
  if (rc) return rc;
  NcclUniqueId id;
  const int n = nccl().GetUniqueId(&id);
  if (n) return nccl_fail("ncclGetUniqueId", n);
  memcpy(id_out, &id, sizeof id);
  return MTB200_OK;
}

// The collectives of this library run BESIDE its persistent tensor kernels, which hold one CTA per SM for a whole
// product: a collective with more CTAs than the SMs left free waits for, or displaces, CTAs of a product, and the
// product's static tile deal turns one late CTA into a late product.  Measured on eight B200s (large MLP, steady
// clocks, same box): no limit and 8 SMs free 8.67 ms per step, 16 CTAs / 16 SMs free 8.32, 24 / 24 8.33, 32 / 32 8.41.
// NCCL takes its CTA budget from the environment when a communicator is created, so the default budget is set there
// unless the host has chosen one (NCCL_MAX_CTAS) or opted out (MTB200_COMM_CTAS=0).
static void apply_cta_budget() {
  const char* own = getenv("MTB200_COMM_CTAS");
  if (own && atoi(own) <= 0) return;
  setenv("NCCL_MAX_CTAS", own ? own : "16", /*overwrite=*/0);
}

int32_t mtb200_comm_init_rank(int32_t world_size, int32_t rank, const void* id, int32_t device_ordinal,
                              mtb200_comm* out) {
  if (!out) return fail(MTB200_ERR_INVALID, "null output communicator");
  *out = nullptr;
  if (!id) return fail(MTB200_ERR_INVALID, "null id");
  if (world_size < 1 || rank < 0 || rank >= world_size)
    return fail(MTB200_ERR_INVALID, "rank %d outside a world of %d", rank, world_size);
  int32_t rc = nccl_ready();
  if (rc) return rc;
  DeviceGuard guard(device_ordinal);
  if (!guard.ok) return fail(MTB200_ERR_CUDA, "cannot make device %d current", device_ordinal);
  NcclUniqueId uid;
  memcpy(&uid, id, sizeof uid);
  ncclComm_t c = nullptr;
  apply_cta_budget();
  const int n = nccl().CommInitRank(&c, world_size, uid, rank);
  if (n) return nccl_fail("ncclCommInitRank", n);
  mtb200_comm_s* m = new mtb200_comm_s();
  m->world = world_size;
  m->ranks.push_back(rank);
  m->devices.push_back(device_ordinal);
  m->comms.push_back(c);
  m->streams.push_back(nullptr);
  *out = m;
  return MTB200_OK;
}

int32_t mtb200_comm_init(int32_t ndev, const int32_t* devs, mtb200_comm* out) {
  if (!out) return fail(MTB200_ERR_INVALID, "null output communicator");
  *out = nullptr;
  if (ndev < 1 || !devs) return fail(MTB200_ERR_INVALID, "need at least one device");
  int32_t rc = nccl_ready();
  if (rc) return rc;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    cudaGetLastError();
    return fail(MTB200_ERR_CUDA, "no CUDA device available");
  }
  std::vector<int> list(devs, devs + ndev);
  for (int d : list)
    if (d < 0 || d >= count) return fail(MTB200_ERR_INVALID, "device ordinal %d out of range [0,%d)", d, count);
  std::vector<ncclComm_t> comms(ndev, nullptr);
  apply_cta_budget();
  const int n = nccl().CommInitAll(comms.data(), ndev, list.data());
  if (n) return nccl_fail("ncclCommInitAll", n);
  mtb200_comm_s* m = new mtb200_comm_s();
  m->world = ndev;
  for (int i = 0; i < ndev; ++i) {
    m->ranks.push_back(i);
    m->devices.push_back(list[i]);
    m->comms.push_back(comms[i]);
    m->streams.push_back(nullptr);
  }
  *out = m;
  return MTB200_OK;
}

static int local_slot(mtb200_comm c, int32_t rank) {
  for (size_t i = 0; i < c->ranks.size(); ++i)
    if (c->ranks[i] == rank) return int(i);
  return -1;
}

int32_t mtb200_comm_set_stream(mtb200_comm c, int32_t rank, void* cuda_stream) {
  if (!c) return fail(MTB200_ERR_INVALID, "null communicator");
  const int s = local_slot(c, rank);
  if (s < 0) return fail(MTB200_ERR_INVALID, "rank %d is not driven by this process", rank);
  c->streams[s] = static_cast<cudaStream_t>(cuda_stream);
  return MTB200_OK;
}

int32_t mtb200_comm_group_begin(mtb200_comm c) {
  if (!c) return fail(MTB200_ERR_INVALID, "null communicator");
  const int n = nccl().GroupStart();
  return n ? nccl_fail("ncclGroupStart", n) : MTB200_OK;
}

int32_t mtb200_comm_group_end(mtb200_comm c) {
  if (!c) return fail(MTB200_ERR_INVALID, "null communicator");
  const int n = nccl().GroupEnd();
  return n ? nccl_fail("ncclGroupEnd", n) : MTB200_OK;
}

int32_t mtb200_allreduce_sum_f32(mtb200_comm c, int32_t rank, float* buf, size_t n, float scale) {
  if (!c) return fail(MTB200_ERR_INVALID, "null communicator");
  const int s = local_slot(c, rank);
  if (s < 0) return fail(MTB200_ERR_INVALID, "rank %d is not driven by this process", rank);
  if (n == 0) return MTB200_OK;
  if (!buf) return fail(MTB200_ERR_INVALID, "null buffer");
  DeviceGuard guard(c->devices[s]);
  if (!guard.ok) return fail(MTB200_ERR_CUDA, "cannot make device %d current", c->devices[s]);
  const int rc = nccl().AllReduce(buf, buf, n, NCCL_FLOAT32, NCCL_SUM, c->comms[s], c->streams[s]);
  if (rc) return nccl_fail("ncclAllReduce", rc);
  if (scale != 1.0f) {
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->devices[s]);
    const size_t blocks = std::min<size_t>((n / 4 + 255) / 256 + 1, size_t(std::max(1, sms)) * 8);
    comm_scale_kernel<<<unsigned(blocks), 256, 0, c->streams[s]>>>(buf, n, scale);
    MTB_CUDA(cudaGetLastError());
  }
  return MTB200_OK;
}

int32_t mtb200_comm_destroy(mtb200_comm c) {
  if (!c) return MTB200_OK;
  int32_t rc = MTB200_OK;
  for (size_t i = 0; i < c->comms.size(); ++i) {
    DeviceGuard guard(c->devices[i]);
    cudaStreamSynchronize(c->streams[i]);
    const int n = nccl().CommDestroy(c->comms[i]);
    if (n && rc == MTB200_OK) rc = nccl_fail("ncclCommDestroy", n);
  }
  delete c;
  return rc;
}

}  // extern "C"
