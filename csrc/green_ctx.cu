// Green contexts: a fixed split of the GPU's SMs between two streams.
//
// pg_green_split carves `sms_a` SMs (rounded up by the driver to its granularity) out of the device's SM resource,
// makes one green context of them and one of the remainder, and creates a non-blocking stream in each.  Work launched
// on one of those streams runs only on that partition's SMs; work on the process's ordinary streams may still use
// every SM.  The engine binds its prefill lane to the smaller partition so that prompt chunks can never take the SMs
// decode steps need (`--decode-sm-pct`).  Everything here lives and dies with the process: no device setting changes.
//
// Reference parity: pegainfer-qwen3/src/green_ctx.rs, pegainfer-gemma4/src/green_ctx.rs (decode / prefill SM split).
#include "common.cuh"

#include <cuda.h>

#include <mutex>

namespace {

struct Api {
  CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*DeviceGetDevResource)(CUdevice, CUdevResource*, CUdevResourceType) = nullptr;
  CUresult (*DevSmResourceSplitByCount)(CUdevResource*, unsigned int*, const CUdevResource*, CUdevResource*, unsigned int, unsigned int) = nullptr;
  CUresult (*DevResourceGenerateDesc)(CUdevResourceDesc*, CUdevResource*, unsigned int) = nullptr;
  CUresult (*GreenCtxCreate)(CUgreenCtx*, CUdevResourceDesc, CUdevice, unsigned int) = nullptr;
  CUresult (*GreenCtxStreamCreate)(CUstream*, CUgreenCtx, unsigned int, int) = nullptr;
  CUresult (*GreenCtxDestroy)(CUgreenCtx) = nullptr;
  CUresult (*StreamDestroy)(CUstream) = nullptr;
  bool ok = false;
};

template <typename F>
bool load(const char* name, F& fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
    (void)cudaGetLastError();
    return false;
  }
  fn = reinterpret_cast<F>(p);
  return true;
}

Api& api() {
  static Api a;
  static std::once_flag once;
  std::call_once(once, [] {
    a.ok = load("cuDeviceGet", a.DeviceGet) && load("cuDeviceGetDevResource", a.DeviceGetDevResource) && load("cuDevSmResourceSplitByCount", a.DevSmResourceSplitByCount) &&
           load("cuDevResourceGenerateDesc", a.DevResourceGenerateDesc) && load("cuGreenCtxCreate", a.GreenCtxCreate) && load("cuGreenCtxStreamCreate", a.GreenCtxStreamCreate) &&
           load("cuGreenCtxDestroy", a.GreenCtxDestroy) && load("cuStreamDestroy", a.StreamDestroy);
  });
  return a;
}

struct Split {
  CUgreenCtx ctx[2] = {nullptr, nullptr};
  CUstream stream[2] = {nullptr, nullptr};
  int sms[2] = {0, 0};
};

}  // namespace

extern "C" int pg_green_available() { return api().ok ? 1 : 0; }

// `*handle` receives an opaque pointer; partition 0 has at least `sms_a` SMs, partition 1 the rest.
extern "C" int pg_green_split(int device, int sms_a, void** handle) {
  Api& a = api();
  PG_REQUIRE(a.ok, "green contexts are not available from this driver");
  PG_REQUIRE(sms_a > 0, "green split: the first partition needs at least one SM");
  PG_CUDA(cudaSetDevice(device));
  PG_CUDA(cudaFree(nullptr));  // the primary context exists
  CUdevice dev;
  PG_REQUIRE(a.DeviceGet(&dev, device) == CUDA_SUCCESS, "cuDeviceGet failed");
  CUdevResource all, part, rest;
  PG_REQUIRE(a.DeviceGetDevResource(dev, &all, CU_DEV_RESOURCE_TYPE_SM) == CUDA_SUCCESS, "cuDeviceGetDevResource failed");
  PG_REQUIRE((int)all.sm.smCount > sms_a, "green split: %d SMs asked of %d", sms_a, (int)all.sm.smCount);
  unsigned int groups = 1;
  CUresult r = a.DevSmResourceSplitByCount(&part, &groups, &all, &rest, 0, (unsigned int)sms_a);
  PG_REQUIRE(r == CUDA_SUCCESS && groups == 1, "cuDevSmResourceSplitByCount failed with code %d", (int)r);
  PG_REQUIRE(rest.sm.smCount > 0, "green split: nothing left for the second partition (%d of %d SMs taken)", (int)part.sm.smCount, (int)all.sm.smCount);
  Split* s = new Split();
  CUdevResource res[2] = {part, rest};
  for (int i = 0; i < 2; ++i) {
    CUdevResourceDesc desc;
    r = a.DevResourceGenerateDesc(&desc, &res[i], 1);
    if (r == CUDA_SUCCESS) r = a.GreenCtxCreate(&s->ctx[i], desc, dev, CU_GREEN_CTX_DEFAULT_STREAM);
    if (r == CUDA_SUCCESS) r = a.GreenCtxStreamCreate(&s->stream[i], s->ctx[i], CU_STREAM_NON_BLOCKING, 0);
    if (r != CUDA_SUCCESS) {
      for (int k = 0; k <= i; ++k) {
        if (s->stream[k]) a.StreamDestroy(s->stream[k]);
        if (s->ctx[k]) a.GreenCtxDestroy(s->ctx[k]);
      }
      delete s;
      PG_REQUIRE(false, "green context %d could not be created (code %d)", i, (int)r);
    }
    s->sms[i] = (int)res[i].sm.smCount;
  }
  *handle = s;
  return PG_OK;
}

extern "C" int pg_green_info(void* handle, void** stream_a, void** stream_b, int* sms_a, int* sms_b) {
  Split* s = static_cast<Split*>(handle);
  PG_REQUIRE(s != nullptr, "green info: null handle");
  *stream_a = s->stream[0];
  *stream_b = s->stream[1];
  *sms_a = s->sms[0];
  *sms_b = s->sms[1];
  return PG_OK;
}

extern "C" int pg_green_destroy(void* handle) {
  Split* s = static_cast<Split*>(handle);
  if (s == nullptr) return PG_OK;
  Api& a = api();
  for (int i = 0; i < 2; ++i) {
    if (s->stream[i]) a.StreamDestroy(s->stream[i]);
    if (s->ctx[i]) a.GreenCtxDestroy(s->ctx[i]);
  }
  delete s;
  return PG_OK;
}
