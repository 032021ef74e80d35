/* LD_PRELOAD counter of CUDA runtime calls that matter for steady-state serving: allocations, frees,
 * kernel launches, graph launches, copies and memsets.  A decode loop that is "allocation free" and
 * "one graph launch per step" can be checked from the outside, without a profiler:
 *
 *     gcc -O2 -shared -fPIC -o libcuda_api_counter.so cuda_api_counter.c -ldl
 *     LD_PRELOAD=./libcuda_api_counter.so PEGAINFER_API_COUNTER_OUT=counts.txt python bench.py ...
 *
 * Counts are written at process exit (to the file named by PEGAINFER_API_COUNTER_OUT, else stderr).
 * PEGAINFER_API_COUNTER_RESET names a file; while it exists the counters are held at zero, so a warm-up
 * phase can be excluded (remove the file to start counting).  Only the entry points are interposed; the
 * real functions are found with dlsym(RTLD_NEXT) and called unchanged.
 *
 * Plays the role of the reference's tools/cuda_api_counter.c.
 */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <unistd.h>

typedef int (*fn_generic)();
enum { C_MALLOC, C_MALLOC_ASYNC, C_FREE, C_FREE_ASYNC, C_HOST_ALLOC, C_LAUNCH, C_LAUNCH_EX, C_GRAPH_LAUNCH, C_MEMCPY, C_MEMCPY_ASYNC, C_MEMSET, C_MEMSET_ASYNC, C_STREAM_SYNC, C_DEVICE_SYNC, C_N };
static const char* names[C_N] = {"cudaMalloc", "cudaMallocAsync", "cudaFree", "cudaFreeAsync", "cudaHostAlloc", "cudaLaunchKernel", "cudaLaunchKernelExC", "cudaGraphLaunch", "cudaMemcpy",
                                 "cudaMemcpyAsync", "cudaMemset", "cudaMemsetAsync", "cudaStreamSynchronize", "cudaDeviceSynchronize"};
static unsigned long long counts[C_N];
static void* real[C_N];

static int counting(void) {
  const char* hold = getenv("PEGAINFER_API_COUNTER_RESET");
  return !(hold && access(hold, F_OK) == 0);
}
static void* resolve(int i) {
  if (!real[i]) real[i] = dlsym(RTLD_NEXT, names[i]);
  return real[i];
}
static void bump(int i) {
  if (counting()) __atomic_add_fetch(&counts[i], 1ull, __ATOMIC_RELAXED);
}

__attribute__((destructor)) static void report(void) {
  const char* path = getenv("PEGAINFER_API_COUNTER_OUT");
  FILE* f = path ? fopen(path, "w") : stderr;
  if (!f) f = stderr;
  for (int i = 0; i < C_N; ++i) fprintf(f, "%s %llu\n", names[i], counts[i]);
  if (f != stderr) fclose(f);
}

#define FORWARD(idx, ret_on_missing, ...)                   \
  do {                                                      \
    fn_generic fn = (fn_generic)resolve(idx);               \
    bump(idx);                                              \
    if (!fn) return ret_on_missing;                         \
    return fn(__VA_ARGS__);                                 \
  } while (0)

int cudaMalloc(void** p, size_t n) { FORWARD(C_MALLOC, 999, p, n); }
int cudaMallocAsync(void** p, size_t n, void* s) { FORWARD(C_MALLOC_ASYNC, 999, p, n, s); }
int cudaFree(void* p) { FORWARD(C_FREE, 999, p); }
int cudaFreeAsync(void* p, void* s) { FORWARD(C_FREE_ASYNC, 999, p, s); }
int cudaHostAlloc(void** p, size_t n, unsigned f) { FORWARD(C_HOST_ALLOC, 999, p, n, f); }
struct dim3_ { unsigned x, y, z; };
int cudaLaunchKernel(const void* f, struct dim3_ g, struct dim3_ b, void** a, size_t sm, void* s) { FORWARD(C_LAUNCH, 999, f, g, b, a, sm, s); }
int cudaLaunchKernelExC(const void* cfg, const void* f, void** a) { FORWARD(C_LAUNCH_EX, 999, cfg, f, a); }
int cudaGraphLaunch(void* g, void* s) { FORWARD(C_GRAPH_LAUNCH, 999, g, s); }
int cudaMemcpy(void* d, const void* s, size_t n, int k) { FORWARD(C_MEMCPY, 999, d, s, n, k); }
int cudaMemcpyAsync(void* d, const void* s, size_t n, int k, void* st) { FORWARD(C_MEMCPY_ASYNC, 999, d, s, n, k, st); }
int cudaMemset(void* d, int v, size_t n) { FORWARD(C_MEMSET, 999, d, v, n); }
int cudaMemsetAsync(void* d, int v, size_t n, void* st) { FORWARD(C_MEMSET_ASYNC, 999, d, v, n, st); }
int cudaStreamSynchronize(void* s) { FORWARD(C_STREAM_SYNC, 999, s); }
int cudaDeviceSynchronize(void) { FORWARD(C_DEVICE_SYNC, 999); }
