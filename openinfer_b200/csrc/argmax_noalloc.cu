// Two-stage argmax whose scratch lives in the library image instead of coming from an allocator.
// See no_alloc.h for who needs this and for the contract. It is a variant of the argmax in
// sampling.cu (same result: largest value, lowest index on ties; NaN never wins) that takes no
// scratch pointers: stage one writes one (value, index) pair per 4096-entry chunk of a row into the
// static array below, stage two reduces a row's pairs.
#include "common.cuh"
#include "no_alloc.h"

namespace {

constexpr int kChunk = 4096;
constexpr int kMaxDevices = 64;

struct Partial {
  float v;
  int i;
};

// The scratch: 16384 pairs = 128 KiB, present on every GPU that loads this library until exit.
// In HOST code this name is only a stand-in for the symbol; its device address is looked up once
// per device below. Device code may name it directly, as the kernels here do.
static __device__ __align__(256) Partial g_argmax_scratch[OI_ARGMAX_NOALLOC_MAX_PARTIALS];

__device__ __forceinline__ Partial better(Partial a, Partial b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ Partial warp_best(Partial p) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Partial other{__shfl_xor_sync(0xffffffffu, p.v, o), __shfl_xor_sync(0xffffffffu, p.i, o)};
    p = better(p, other);
  }
  return p;
}

// `scratch` is the address the host looked up; it equals g_argmax_scratch on this device.
__global__ void argmax_noalloc_partial_kernel(Partial* __restrict__ scratch, const float* __restrict__ logits,
                                              int vocab, long long row_stride, int nchunks) {
  pdl_start();
  __shared__ Partial sh[8];
  const int r = blockIdx.y, chunk = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  const int lo = chunk * kChunk, hi = min(vocab, lo + kChunk);
  Partial best{-INFINITY, 0x7fffffff};
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = row[i];
    if (v == v) best = better(best, Partial{v, i});
  }
  best = warp_best(best);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    Partial b = sh[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) b = better(b, sh[w]);
    scratch[(size_t)r * nchunks + chunk] = b;   // every pair that stage two reads is written here first
  }
}

__global__ void argmax_noalloc_final_kernel(int* __restrict__ out, const Partial* __restrict__ scratch, int nchunks) {
  pdl_start();
  const int r = blockIdx.x;
  Partial best{-INFINITY, 0x7fffffff};
  for (int c = threadIdx.x; c < nchunks; c += 32) best = better(best, scratch[(size_t)r * nchunks + c]);
  best = warp_best(best);
  if (threadIdx.x == 0) out[r] = best.i == 0x7fffffff ? 0 : best.i;
}

// device address of the scratch array, per device ordinal (0 = not looked up yet)
Partial* g_scratch_addr[kMaxDevices] = {};

}  // namespace

OI_API int oi_argmax_noalloc(int* out, const float* logits, int rows, int vocab, long long row_stride, void* stream) {
  OI_REQUIRE(out && logits, "argmax_noalloc: null pointer");
  OI_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "argmax_noalloc: bad sizes rows=%d vocab=%d", rows, vocab);
  if (rows == 0) return OI_OK;
  const long long nchunks = ((long long)vocab + kChunk - 1) / kChunk;
  if ((long long)rows * nchunks > OI_ARGMAX_NOALLOC_MAX_PARTIALS || rows > 65535) {
    oi_set_error("argmax_noalloc: %d rows x %lld chunks of %d entries need %lld partial results; the built-in "
                 "scratch holds %d (no memory is allocated by this entry point)",
                 rows, nchunks, kChunk, (long long)rows * nchunks, OI_ARGMAX_NOALLOC_MAX_PARTIALS);
    return OI_ERR_TOO_LARGE;
  }
  int device = -1;
  OI_CHECK_CUDA(cudaGetDevice(&device));
  OI_REQUIRE(device >= 0 && device < kMaxDevices, "argmax_noalloc: device ordinal %d not supported", device);
  if (g_scratch_addr[device] == nullptr) {
    // set-up, once per device, with that device current: the symbol's address ON THIS DEVICE
    Partial* addr = nullptr;
    OI_CHECK_CUDA(cudaGetSymbolAddress((void**)&addr, g_argmax_scratch));
    OI_REQUIRE(addr != nullptr, "argmax_noalloc: the scratch symbol has no device address");
    g_scratch_addr[device] = addr;
  }
  Partial* scratch = g_scratch_addr[device];
  cudaStream_t s = (cudaStream_t)stream;
  oi_launch(argmax_noalloc_partial_kernel, dim3((unsigned)nchunks, rows), 256, 0, s, scratch, logits, vocab, row_stride, (int)nchunks);
  OI_CHECK_LAUNCH();
  oi_launch(argmax_noalloc_final_kernel, rows, 32, 0, s, out, scratch, (int)nchunks);
  OI_CHECK_LAUNCH();
  return OI_OK;
}
