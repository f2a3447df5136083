// Shared helpers of the sm_100a kernels: element types, conversions, reductions,
// the C ABI's error reporting.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <cstring>

// Element-type codes of the C ABI.
enum : int { OI_F32 = 0, OI_BF16 = 1 };

// Error codes returned by every entry point (0 = success). CUDA runtime errors
// are returned as 1000 + cudaError_t.
enum : int {
  OI_OK = 0,
  OI_ERR_BAD_ARGUMENT = 1,   // a size or dtype the kernel refuses
  OI_ERR_UNSUPPORTED = 2,
  OI_ERR_TOO_LARGE = 3,
  OI_ERR_CUDA = 1000,
};

#define OI_API extern "C" __attribute__((visibility("default")))

void oi_set_error(const char* fmt, ...);

#define OI_REQUIRE(cond, ...)            \
  do {                                   \
    if (!(cond)) {                       \
      oi_set_error(__VA_ARGS__);         \
      return OI_ERR_BAD_ARGUMENT;        \
    }                                    \
  } while (0)

#define OI_CHECK_LAUNCH()                                                     \
  do {                                                                        \
    cudaError_t e__ = cudaGetLastError();                                     \
    if (e__ != cudaSuccess) {                                                 \
      oi_set_error("%s:%d: launch failed: %s", __FILE__, __LINE__,            \
                   cudaGetErrorString(e__));                                  \
      return OI_ERR_CUDA + (int)e__;                                          \
    }                                                                         \
  } while (0)

#define OI_CHECK_CUDA(expr)                                                   \
  do {                                                                        \
    cudaError_t e__ = (expr);                                                 \
    if (e__ != cudaSuccess) {                                                 \
      oi_set_error("%s:%d: %s failed: %s", __FILE__, __LINE__, #expr,         \
                   cudaGetErrorString(e__));                                  \
      return OI_ERR_CUDA + (int)e__;                                          \
    }                                                                         \
  } while (0)

typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch. Every kernel of the library is launched through oi_launch and
// opens with pdl_start(): it lets the NEXT kernel on the stream be scheduled at once and then
// waits until the kernel BEFORE it has finished and its writes are visible. Nothing that another
// kernel writes or reads-then-overwrites is touched before that wait, so the memory effects stay
// in stream order; what overlaps is the launch latency, the prologues, and in the weight-streaming
// products the first loads of the (never written) weights, which they request before waiting.
// What a kernel may read before its wait must have been written before the step's kernels began: the
// step's metadata is put in place by a kernel that does NOT trigger early (copy_words_kernel), and the
// kernel launched after that one is launched WITHOUT the attribute (oi_launch_fence, called by whoever uploads it): it starts only
// when the metadata kernel has completed and its writes are visible, and every later kernel of the chain
// starts after that kernel has started. Keys and values of earlier steps lie behind that fence too.
// A kernel launched without the attribute (oi_set_pdl(0), or after a library kernel) sees both
// instructions as no-ops.
// ---------------------------------------------------------------------------------------------
int oi_pdl_enabled();
void oi_fence_next_launch();   // the next kernel launched through oi_launch gets plain stream order (once)
int oi_take_launch_fence();
void oi_count_launch();   // every kernel launched through oi_launch is counted (oi_launches)
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_start() {
  pdl_trigger();
  pdl_wait();
}

// kernel<<<grid, block, smem, stream>>>(args...) with the programmatic-serialization attribute when
// enabled, and optionally a cluster of `cluster_x` CTAs along x. Check with OI_CHECK_LAUNCH().
template <typename... Params, typename... Args>
inline void oi_launch_cluster(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              int cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  const int fenced = oi_take_launch_fence();
  if (oi_pdl_enabled() && !fenced) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (cluster_x > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = (unsigned)cluster_x;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = na ? attr : nullptr;
  cfg.numAttrs = (unsigned)na;
  oi_count_launch();
  (void)cudaLaunchKernelEx(&cfg, kernel, static_cast<Args&&>(args)...);   // the error stays for cudaGetLastError
}
template <typename... Params, typename... Args>
inline void oi_launch(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  oi_launch_cluster(kernel, grid, block, smem, stream, 1, static_cast<Args&&>(args)...);
}

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }

// Gate activations of a gated feed-forward, act(gate) * up. The codes are part of the C interface.
#define OI_ACT_NONE 0
#define OI_ACT_SILU 1        // g * sigmoid(g)
#define OI_ACT_GELU_TANH 2   // 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) = g * sigmoid(2 sqrt(2/pi) (g + 0.044715 g^3))
// kFast: exponential and division by the special-function unit's approximations (2 ulp each, far below the
// rounding of a bfloat16 result), for the epilogues of the bfloat16 products.
template <bool kFast>
__device__ __forceinline__ float gate_act(float g, int act) {
  const float t = act == OI_ACT_GELU_TANH ? 1.5957691216057308f * (g + 0.044715f * g * g * g) : g;
  return kFast ? __fdividef(g, 1.f + __expf(-t)) : g / (1.f + expf(-t));
}

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

// Load element i of an array whose element type is only known at run time.
__device__ __forceinline__ float load_as_f32(const void* p, int dtype, size_t i) {
  return dtype == OI_F32 ? reinterpret_cast<const float*>(p)[i]
                         : __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum with a fixed tree (same order whatever else runs): every thread
// gets the result. `scratch` holds at least 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

static inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }
