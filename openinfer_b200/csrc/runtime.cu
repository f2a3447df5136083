// Error reporting of the C ABI and a few device queries.
#include <stdarg.h>

#include "common.cuh"

static thread_local char g_error[512] = "";

void oi_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

// Message of the last failed call on this thread.
OI_API const char* oi_last_error() { return g_error; }

// ABI version: bumped when an entry point's signature changes.
OI_API int oi_abi_version() { return 1; }

// Programmatic dependent launch of the library's kernels (see common.cuh): on unless switched off.
static int g_pdl = 1;
int oi_pdl_enabled() { return g_pdl; }
// A kernel whose writes later kernels read BEFORE their own wait (the step's metadata) asks for the next launch to be
// an ordinary one: that kernel then starts after the writer has completed, and the chain behind it after that.
static int g_fence_next = 0;
void oi_fence_next_launch() { g_fence_next = 1; }
OI_API int oi_launch_fence() {
  g_fence_next = 1;
  return OI_OK;
}
int oi_take_launch_fence() {
  const int v = g_fence_next;
  g_fence_next = 0;
  return v;
}

// Kernels of this library launched so far (through oi_launch; a recorded graph's replays are not seen here).
static unsigned long long g_launches = 0;
void oi_count_launch() { ++g_launches; }
OI_API unsigned long long oi_launches() { return g_launches; }

OI_API int oi_set_pdl(int enabled) {
  g_pdl = enabled ? 1 : 0;
  return OI_OK;
}

OI_API int oi_device_info(int device, int* sm_major, int* sm_minor, int* sm_count, long long* l2_bytes) {
  cudaDeviceProp prop;
  OI_CHECK_CUDA(cudaGetDeviceProperties(&prop, device));
  *sm_major = prop.major;
  *sm_minor = prop.minor;
  *sm_count = prop.multiProcessorCount;
  *l2_bytes = prop.l2CacheSize;
  return OI_OK;
}
