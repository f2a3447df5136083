// Token selection from float32 logits: argmax (ties -> lowest index) and temperature /
// top-k / top-p / min-p sampling by inverse CDF with a uniform number supplied per row.
//
// Parameter meanings follow the reference (pegainfer-frontend/src/sampler.rs:2-38): softmax of
// logits / temperature in float32; top_k <= 0 or >= vocab disables; top_p >= 1 disables;
// min_p masks p < min_p * p_max; filter order top-k -> top-p (on the renormalised rest) -> min-p
// (pegainfer-kernels/csrc/shared/flashinfer_sampling.cu:99-128). Argmax ties go to the lowest
// index (csrc/shared/argmax.cu:15-18). The reference draws by rejection sampling with a philox
// stream; here the caller supplies one uniform number per row (made from the request's own seed
// and step, so a row's draw does not depend on its place in the batch) and the kernel walks the
// cumulative distribution in vocabulary order. Thresholds are found by bisection on the bit
// pattern of the (non-negative) probabilities, so no sort and no scratch beyond one float per
// vocabulary entry and row.
#include "common.cuh"

namespace {

struct ArgPair {
  float v;
  int i;
};
__device__ __forceinline__ ArgPair better(ArgPair a, ArgPair b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__global__ void argmax_kernel(int* __restrict__ out, const float* __restrict__ logits, int vocab,
                              long long row_stride) {
  pdl_start();
  __shared__ float sv[32];
  __shared__ int si[32];
  const float* row = logits + (size_t)blockIdx.x * row_stride;
  ArgPair best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    ArgPair c{v, i};
    // NaN never wins; an all -inf row returns index 0 below
    if (v == v) best = better(best, c);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best.v; si[warp] = best.i; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    ArgPair b{lane < nw ? sv[lane] : -INFINITY, lane < nw ? si[lane] : 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgPair other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
      b = better(b, other);
    }
    if (lane == 0) out[blockIdx.x] = b.i == 0x7fffffff ? 0 : b.i;
  }
}

// Two-stage argmax for a few rows of a large vocabulary: many blocks per row, then one block per row.
constexpr int kArgmaxChunk = 4096;

__global__ void argmax_partial_kernel(float* __restrict__ pv, int* __restrict__ pi, const float* __restrict__ logits,
                                      int vocab, long long row_stride, int nchunks) {
  pdl_start();
  __shared__ float sv[8];
  __shared__ int si[8];
  const int r = blockIdx.y, chunk = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  const int lo = chunk * kArgmaxChunk, hi = min(vocab, lo + kArgmaxChunk);
  ArgPair best{-INFINITY, 0x7fffffff};
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = row[i];
    if (v == v) best = better(best, ArgPair{v, i});
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best.v; si[warp] = best.i; }
  __syncthreads();
  if (threadIdx.x == 0) {
    ArgPair b{sv[0], si[0]};
    for (int wdx = 1; wdx < (int)(blockDim.x >> 5); ++wdx) b = better(b, ArgPair{sv[wdx], si[wdx]});
    pv[(size_t)r * nchunks + chunk] = b.v;
    pi[(size_t)r * nchunks + chunk] = b.i;
  }
}

__global__ void argmax_final_kernel(int* __restrict__ out, const float* __restrict__ pv, const int* __restrict__ pi,
                                    int nchunks) {
  pdl_start();
  const int r = blockIdx.x;
  ArgPair best{-INFINITY, 0x7fffffff};
  for (int c = threadIdx.x; c < nchunks; c += 32) best = better(best, ArgPair{pv[(size_t)r * nchunks + c], pi[(size_t)r * nchunks + c]});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  if (threadIdx.x == 0) out[r] = best.i == 0x7fffffff ? 0 : best.i;
}

// count and mass of { p >= thr } over one row (p >= 0, compared as bit patterns)
__device__ __forceinline__ void count_mass(const float* __restrict__ p, int vocab, unsigned thr_bits,
                                           unsigned floor_bits, float* red, int& count, float& mass) {
  float c = 0.f, m = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = p[i];
    const unsigned b = __float_as_uint(v);
    if (b >= thr_bits && b >= floor_bits) { c += 1.f; m += v; }
  }
  c = block_sum(c, red);
  m = block_sum(m, red);
  count = (int)(c + 0.5f);
  mass = m;
}

// One block per row. probs: scratch [rows, vocab] float32.
__global__ void sample_kernel(int* __restrict__ out, const float* __restrict__ logits, long long row_stride,
                              float* __restrict__ probs, int vocab, const float* __restrict__ temperature,
                              const int* __restrict__ top_k, const float* __restrict__ top_p,
                              const float* __restrict__ min_p, const float* __restrict__ uniform) {
  pdl_start();
  __shared__ float red[32];
  __shared__ float chunk_sum[1024];
  __shared__ int picked;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  float* p = probs + (size_t)r * vocab;
  const float inv_t = 1.f / temperature[r];

  float mx = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, row[i]);
  mx = block_max(mx, red);
  float z = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float e = expf((row[i] - mx) * inv_t);
    p[i] = e;
    z += e;
  }
  z = block_sum(z, red);  // also orders the writes of p before the reads below (barriers inside)
  // p holds unnormalised e in [0, 1]; p_max = 1. Thresholds are scale-free.

  unsigned floor_bits = 0;  // running lower bound of kept values (bit pattern)
  float kept_mass = z;
  int k = top_k[r];
  if (k > 0 && k < vocab) {
    // largest t with count(p >= t) >= k: the k-th largest value
    unsigned cur = 0;
    for (int b = 30; b >= 0; --b) {
      const unsigned cand = cur | (1u << b);
      int cnt; float mass;
      count_mass(p, vocab, cand, 0u, red, cnt, mass);
      if (cnt >= k) cur = cand;
    }
    floor_bits = cur;
    int cnt;
    count_mass(p, vocab, floor_bits, 0u, red, cnt, kept_mass);
  }
  const float tp = top_p[r];
  if (tp < 1.f) {
    // largest t with mass(p >= t, kept) >= top_p * kept_mass
    const float need = tp * kept_mass;
    unsigned cur = 0;
    for (int b = 30; b >= 0; --b) {
      const unsigned cand = cur | (1u << b);
      int cnt; float mass;
      count_mass(p, vocab, cand, floor_bits, red, cnt, mass);  // counts p >= max(cand, floor)
      if (cnt > 0 && mass >= need) cur = cand;
    }
    if (cur > floor_bits) floor_bits = cur;
  }
  const float mp = min_p[r];
  if (mp > 0.f) {
    const unsigned b = __float_as_uint(mp);  // p_max = 1 in the unnormalised scale
    if (b > floor_bits) floor_bits = b;
  }

  // inverse CDF in vocabulary order: thread t owns a contiguous chunk
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int lo = threadIdx.x * chunk, hi = min(vocab, lo + chunk);
  float local = 0.f;
  for (int i = lo; i < hi; ++i) {
    const float v = p[i];
    if (__float_as_uint(v) >= floor_bits) local += v;
  }
  chunk_sum[threadIdx.x] = local;
  if (threadIdx.x == 0) picked = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int t = 0; t < blockDim.x; ++t) total += chunk_sum[t];
    const float target = uniform[r] * total;
    float run = 0.f;
    int owner = -1, last_nonempty = -1;
    for (int t = 0; t < blockDim.x; ++t) {
      if (chunk_sum[t] > 0.f) last_nonempty = t;
      if (owner < 0 && chunk_sum[t] > 0.f && run + chunk_sum[t] > target) { owner = t; break; }
      run += chunk_sum[t];
    }
    if (owner < 0) { owner = last_nonempty; run -= chunk_sum[owner]; }  // rounding at the very end
    // walk the owner's chunk
    const int clo = owner * chunk, chi = min(vocab, clo + chunk);
    int pick = -1, last_kept = -1;
    for (int i = clo; i < chi; ++i) {
      const float v = p[i];
      if (__float_as_uint(v) >= floor_bits && v > 0.f) {
        last_kept = i;
        run += v;
        if (run > target) { pick = i; break; }
      }
    }
    picked = pick >= 0 ? pick : last_kept;
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = picked;
}

}  // namespace

// Number of float/int pairs of scratch per row that oi_argmax wants for this vocabulary.
OI_API int oi_argmax_chunks(int vocab) { return (vocab + kArgmaxChunk - 1) / kArgmaxChunk; }

// partial_vals / partial_idx: scratch of rows * oi_argmax_chunks(vocab) entries each; may be null,
// then one block scans each row.
OI_API int oi_argmax(int* out, const float* logits, int rows, int vocab, long long row_stride, float* partial_vals,
                     int* partial_idx, void* stream) {
  OI_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "argmax: bad sizes rows=%d vocab=%d", rows, vocab);
  if (rows == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int nchunks = (vocab + kArgmaxChunk - 1) / kArgmaxChunk;
  if (partial_vals && partial_idx && nchunks >= 4 && rows * nchunks <= 65535 * 16) {
    oi_launch(argmax_partial_kernel, dim3(nchunks, rows), 256, 0, s, partial_vals, partial_idx, logits, vocab, row_stride, nchunks);
    OI_CHECK_LAUNCH();
    oi_launch(argmax_final_kernel, rows, 32, 0, s, out, partial_vals, partial_idx, nchunks);
  } else {
    oi_launch(argmax_kernel, rows, 1024, 0, s, out, logits, vocab, row_stride);
  }
  OI_CHECK_LAUNCH();
  return OI_OK;
}

// Per-row parameter arrays live on the device. `probs` is caller-provided scratch of
// rows * vocab floats. temperature must be > 0 (greedy rows go to oi_argmax).
OI_API int oi_sample(int* out, const float* logits, long long row_stride, float* probs, int rows, int vocab,
                     const float* temperature, const int* top_k, const float* top_p, const float* min_p,
                     const float* uniform, void* stream) {
  OI_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
  OI_REQUIRE(probs != nullptr, "sample: scratch missing");
  if (rows == 0) return OI_OK;
  oi_launch(sample_kernel, rows, 1024, 0, (cudaStream_t)stream, out, logits, row_stride, probs, vocab, temperature,
                                                         top_k, top_p, min_p, uniform);
  OI_CHECK_LAUNCH();
  return OI_OK;
}
