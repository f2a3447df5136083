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
// cumulative distribution in vocabulary order. Thresholds are found by radix selection on the bit
// pattern of the (non-negative) probabilities, over the few thousand largest of them where that
// suffices (see sample_kernel), so no sort and no scratch beyond one float per vocabulary entry and row.
#include <cooperative_groups.h>

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

constexpr int kRadixBins = 2048;
constexpr float kFixedScale = 549755813888.f;    // 2^39: masses of list values are added up in this fixed point

// Count and mass of { p >= thr, p >= floor } over the candidate list in shared memory (p >= 0, compared as
// bit patterns). The list's ORDER differs from run to run (it is filled through an atomic counter): the mass
// is added up in 2^-39 fixed point, where addition is associative, so the result does not depend on the order.
__device__ __forceinline__ void count_mass_list(const float* p, int n, unsigned thr_bits, unsigned floor_bits,
                                                unsigned long long* red64, int& count, float& mass) {
  unsigned long long acc = 0;     // mass in units of 2^-39 (at most 4096 values <= 1.0: at most 2^51)
  int c = 0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = p[i];
    const unsigned b = __float_as_uint(v);
    if (b >= thr_bits && b >= floor_bits) {
      acc += (unsigned long long)(v * kFixedScale);
      ++c;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    acc += __shfl_xor_sync(0xffffffffu, acc, o);
    c += __shfl_xor_sync(0xffffffffu, c, o);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red64[warp] = acc + ((unsigned long long)c << 52);     // count above the mass bits
  __syncthreads();
  acc = 0;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) acc += red64[w];
  count = (int)(acc >> 52);
  mass = (float)(acc & ((1ull << 52) - 1)) * (1.f / kFixedScale);
}

// Thresholds by radix selection over n non-negative values (the candidate list, or the whole row when the
// list does not reach far enough): three rounds (11 + 11 + 9 bits of the pattern, from the top), each a
// histogram of the still undecided values over the round's digit (count and fixed-point mass per bin, shared-
// memory atomics) and a scan of the bins from the top for the largest digit at which the condition still
// holds. Sums are integers (2^-39 fixed point), so neither the order of the values nor that of the atomics
// changes the result. by_mass: largest t with mass{ v >= max(t, floor) } >= need (and at least one such
// v); else largest t with count{ v >= t } >= k. kept_count / kept_mass: of { v >= max(t, floor) }.
__device__ __forceinline__ bool radix_holds(int cnt, unsigned long long mass, bool by_mass, int k, float need) {
  if (!by_mass) return cnt >= k;
  return cnt > 0 && (float)mass * (1.f / kFixedScale) >= need;
}
struct RadixScratch {
  unsigned long long mass[kRadixBins];
  int count[kRadixBins];
  unsigned long long warp_mass[32];
  int warp_count[32];
  unsigned long long above_mass;
  int above_count;
  int digit;
};
__device__ __forceinline__ unsigned radix_threshold(const float* v_in, int n, unsigned floor_bits, bool by_mass, int k,
                                                    float need, RadixScratch& sc, int& kept_count, float& kept_mass) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  unsigned prefix = 0;
  unsigned long long above_m = 0;                // mass and count of the values above the prefix's range
  int above_c = 0;
  int decided = 31;                              // bits [decided, 31) of the threshold are fixed
#pragma unroll 1
  for (int round = 0; round < 3; ++round) {
    const int width = round == 2 ? 9 : 11, shift = decided - width, nb = 1 << width;
    for (int i = tid; i < nb; i += blockDim.x) { sc.mass[i] = 0; sc.count[i] = 0; }
    if (tid == 0) sc.digit = -1;
    __syncthreads();
    for (int i = tid; i < n; i += blockDim.x) {
      const float v = v_in[i];
      const unsigned b = __float_as_uint(v);
      if (b >= floor_bits && (b >> decided) == (prefix >> decided)) {
        const int d = (int)((b >> shift) & (unsigned)(nb - 1));
        atomicAdd(&sc.mass[d], (unsigned long long)(v * kFixedScale));
        atomicAdd(&sc.count[d], 1);
      }
    }
    __syncthreads();
    // suffix sums over the digits, two bins per thread (thread t: digits 2t, 2t + 1)
    const bool has = 2 * tid < nb;
    const unsigned long long m0 = has ? sc.mass[2 * tid] : 0, m1 = has ? sc.mass[2 * tid + 1] : 0;
    const int c0 = has ? sc.count[2 * tid] : 0, c1 = has ? sc.count[2 * tid + 1] : 0;
    unsigned long long sm = m0 + m1;             // become the sums over this and all later threads' bins
    int scn = c0 + c1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long dm = __shfl_down_sync(0xffffffffu, sm, o);
      const int dc = __shfl_down_sync(0xffffffffu, scn, o);
      if (lane + o < 32) { sm += dm; scn += dc; }
    }
    if (lane == 0) { sc.warp_mass[warp] = sm; sc.warp_count[warp] = scn; }
    __syncthreads();
    unsigned long long later_m = above_m;
    int later_c = above_c;
    for (int w = warp + 1; w < nwarps; ++w) { later_m += sc.warp_mass[w]; later_c += sc.warp_count[w]; }
    const unsigned long long from1_m = later_m + sm - m0;   // everything at or above digit 2t + 1
    const int from1_c = later_c + scn - c0;
    const unsigned long long from0_m = from1_m + m0;        // ... digit 2t
    const int from0_c = from1_c + c0;
    if (has) {
      int best = -1;
      if (radix_holds(from1_c, from1_m, by_mass, k, need)) best = 2 * tid + 1;
      else if (radix_holds(from0_c, from0_m, by_mass, k, need)) best = 2 * tid;
      if (best >= 0) atomicMax(&sc.digit, best);
    }
    __syncthreads();
    const int digit = sc.digit < 0 ? 0 : sc.digit;          // nothing holds (the callers rule it out): digit 0
    if (has && (digit >> 1) == tid) {                       // what lies above the chosen digit
      sc.above_mass = (digit & 1) ? from1_m - m1 : from0_m - m0;
      sc.above_count = (digit & 1) ? from1_c - c1 : from0_c - c0;
    }
    __syncthreads();
    above_m = sc.above_mass;
    above_c = sc.above_count;
    prefix |= (unsigned)digit << shift;
    decided = shift;
  }
  // { v >= max(prefix, floor) }: what lies above the last digit plus that digit's bin (still in the scratch)
  const int last = (int)(prefix & ((1u << 9) - 1));
  kept_count = above_c + sc.count[last];
  kept_mass = (float)(above_m + sc.mass[last]) * (1.f / kFixedScale);
  __syncthreads();                                          // before the scratch is used again
  return prefix;
}

constexpr int kSampleThreads = 1024;
constexpr int kListCap = 4096;       // candidates kept in shared memory for the threshold searches
constexpr int kExpBins = 128;        // exponents of values in [0, 1]
constexpr int kCountedOneIn = 8;     // the exponent histogram counts one value in eight
constexpr int kNoAnswer = -1;        // written for a row that the cluster kernel leaves to sample_kernel

// One block per row. probs: scratch [rows, vocab] float32.
//
// After the softmax numerators e = exp((x - max) / T) are written (p_max = 1), a histogram over the
// binary exponents of one value in eight estimates how many values lie at or above every power of two.
// The largest values, down to the power of two at which about half of kListCap qualify, are copied
// into shared memory (a list that overflows all the same is not used); when the k-th largest value /
// the top-p mass lies inside that list (the usual case: a peaked distribution) the threshold searches
// run over the list instead of the whole vocabulary. Otherwise (a flat distribution) they run over
// the vocabulary: same thresholds, three more passes each.
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits, long long row_stride,
              float* __restrict__ probs, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ min_p, const float* __restrict__ uniform, int only_unanswered) {
  pdl_start();
  if (only_unanswered && out[blockIdx.x] != kNoAnswer) return;    // the cluster kernel has drawn this row's token
  __shared__ float red[32];
  __shared__ float chunk_sum[kSampleThreads];
  __shared__ float list[kListCap];
  __shared__ unsigned long long red64[32];
  __shared__ int hist_cnt[kExpBins];
  __shared__ RadixScratch radix;
  __shared__ int picked, list_n, cut_exp;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  float* p = probs + (size_t)r * vocab;
  const float inv_t = 1.f / temperature[r];
  const int tid = threadIdx.x;
  const int k_req = top_k[r];
  const bool want_list = (k_req > 0 && k_req < vocab) || top_p[r] < 1.f;   // a threshold search will follow
  const bool vec = (vocab % 4 == 0) && (((uintptr_t)row) % 16 == 0) && (((uintptr_t)p) % 16 == 0);

  static_assert(kRadixBins * 2 == (kSampleThreads / 32) * kExpBins, "one histogram per warp in the radix bins' words");
  for (int i = tid; i < kRadixBins * 2; i += kSampleThreads) reinterpret_cast<int*>(radix.mass)[i] = 0;
  if (tid == 0) { list_n = 0; picked = -1; }
  __syncthreads();
  // ---- maximum
  float mx = -INFINITY;
  if (vec) {
    const float4* row4 = reinterpret_cast<const float4*>(row);
#pragma unroll 4
    for (int i = tid; i < vocab / 4; i += kSampleThreads) {
      const float4 v = row4[i];
      mx = fmaxf(fmaxf(mx, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
    }
  } else {
    for (int i = tid; i < vocab; i += kSampleThreads) mx = fmaxf(mx, row[i]);
  }
  mx = block_max(mx, red);
  // ---- numerators, their sum, and the histogram over exponents (how many values per power of two)
  float z = 0.f;
  // every warp counts into a histogram of its own (in the words that the radix selection uses later), so
  // the atomics of different warps never meet; the warps' histograms are added up below
  int* const warp_hist = reinterpret_cast<int*>(radix.mass) + (tid >> 5) * kExpBins;
  // Only every eighth value is counted: the histogram just has to place the list's cut so that the list
  // neither overflows nor comes out needlessly short, and the thresholds found do not depend on the cut.
  auto note = [&](float e, bool counted) {
    z += e;
    if (counted) atomicAdd(&warp_hist[__float_as_uint(e) >> 23], 1);       // e in [0, 1]: exponent 0 .. 127
  };
  if (vec) {
    const float4* row4 = reinterpret_cast<const float4*>(row);
    float4* p4 = reinterpret_cast<float4*>(p);
    bool even = true;
#pragma unroll 2
    for (int i = tid; i < vocab / 4; i += kSampleThreads, even = !even) {
      const float4 v = row4[i];
      float4 e;
      e.x = expf((v.x - mx) * inv_t); e.y = expf((v.y - mx) * inv_t);
      e.z = expf((v.z - mx) * inv_t); e.w = expf((v.w - mx) * inv_t);
      p4[i] = e;
      note(e.x, want_list && even); note(e.y, false); note(e.z, false); note(e.w, false);
    }
  } else {
    int it = 0;
    for (int i = tid; i < vocab; i += kSampleThreads, ++it) {
      const float e = expf((row[i] - mx) * inv_t);
      p[i] = e;
      note(e, want_list && (it & 7) == 0);
    }
  }
  z = block_sum(z, red);  // also orders the writes of p and of the histograms before the reads below
  if (want_list && tid < kExpBins) {
    int c = 0;
    for (int w = 0; w < kSampleThreads / 32; ++w) c += reinterpret_cast<int*>(radix.mass)[w * kExpBins + tid];
    hist_cnt[tid] = c;
  }
  __syncthreads();
  // p holds unnormalised e in [0, 1]; p_max = 1. Thresholds are scale-free.

  // ---- the candidate list: every value at or above 2^(cut_exp - 127)
  if (tid == 0) {
    int total = 0, e = kExpBins;
    if (want_list)
      while (e > 0 && total + kCountedOneIn * hist_cnt[e - 1] <= kListCap / 2) { --e; total += kCountedOneIn * hist_cnt[e]; }
    cut_exp = e;    // bins [e, 128) are in the list; e == 128: not even the top bin fits (no list)
  }
  __syncthreads();
  const unsigned cut_bits = (unsigned)cut_exp << 23;
  const bool have_list = cut_exp < kExpBins;
  if (have_list) {
    // one atomic per warp and round: the lanes that take a value share out the places among themselves
    const unsigned lane = tid & 31, below = (1u << lane) - 1u;
    auto take = [&](float v, bool valid) {
      const bool mine = valid && __float_as_uint(v) >= cut_bits;
      const unsigned takers = __ballot_sync(0xffffffffu, mine);
      if (takers == 0) return;
      int base = 0;
      if (lane == (unsigned)(__ffs(takers) - 1)) base = atomicAdd(&list_n, __popc(takers));
      base = __shfl_sync(0xffffffffu, base, __ffs(takers) - 1);
      const int at = base + __popc(takers & below);
      if (mine && at < kListCap) list[at] = v;      // the estimate was off by more than a factor of two: see below
    };
    if (vec) {
      const float4* p4 = reinterpret_cast<const float4*>(p);
      const int n4 = vocab / 4, rounds = (n4 + kSampleThreads - 1) / kSampleThreads;
      for (int it = 0; it < rounds; ++it) {
        const int i = it * kSampleThreads + tid;
        const bool valid = i < n4;
        const float4 v = valid ? p4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        take(v.x, valid); take(v.y, valid); take(v.z, valid); take(v.w, valid);
      }
    } else {
      const int rounds = (vocab + kSampleThreads - 1) / kSampleThreads;
      for (int it = 0; it < rounds; ++it) {
        const int i = it * kSampleThreads + tid;
        take(i < vocab ? p[i] : 0.f, i < vocab);
      }
    }
  }
  __syncthreads();
  const int ln = (have_list && list_n <= kListCap) ? list_n : 0;   // an overflowed list is not used at all

  unsigned floor_bits = 0;  // running lower bound of kept values (bit pattern)
  float kept_mass = z;
  const int k = k_req;
  if (k > 0 && k < vocab) {
    // the k-th largest value: among the list's values when it holds at least k (it holds the largest ones)
    int cnt;
    if (k <= ln) floor_bits = radix_threshold(list, ln, 0u, false, k, 0.f, radix, cnt, kept_mass);
    else floor_bits = radix_threshold(p, vocab, 0u, false, k, 0.f, radix, cnt, kept_mass);
  }
  const float tp = top_p[r];
  if (tp < 1.f) {
    // largest t with mass(p >= t, kept) >= top_p * kept_mass. When the kept values that the list holds
    // already reach that mass, t is at or above the list's cut and every value >= t is in the list.
    const float need = tp * kept_mass;
    int cnt; float in_list, m;
    count_mass_list(list, ln, floor_bits, 0u, red64, cnt, in_list);
    unsigned cur;
    if (ln > 0 && cnt > 0 && in_list >= need) cur = radix_threshold(list, ln, floor_bits, true, 0, need, radix, cnt, m);
    else cur = radix_threshold(p, vocab, floor_bits, true, 0, need, radix, cnt, m);
    if (cur > floor_bits) floor_bits = cur;
  }
  const float mp = min_p[r];
  if (mp > 0.f) {
    const unsigned b = __float_as_uint(mp);  // p_max = 1 in the unnormalised scale
    if (b > floor_bits) floor_bits = b;
  }

  // inverse CDF in vocabulary order: thread t owns a contiguous chunk
  const int chunk = ((vocab + kSampleThreads - 1) / kSampleThreads + 3) & ~3;   // a multiple of 4: 16-byte loads
  const int lo = min(vocab, tid * chunk), hi = min(vocab, lo + chunk);
  float local = 0.f;
  {
    int i = lo;
    if (vec) {
      for (; i + 4 <= hi; i += 4) {
        const float4 v = *reinterpret_cast<const float4*>(p + i);
        if (__float_as_uint(v.x) >= floor_bits) local += v.x;
        if (__float_as_uint(v.y) >= floor_bits) local += v.y;
        if (__float_as_uint(v.z) >= floor_bits) local += v.z;
        if (__float_as_uint(v.w) >= floor_bits) local += v.w;
      }
    }
    for (; i < hi; ++i) {
      const float v = p[i];
      if (__float_as_uint(v) >= floor_bits) local += v;
    }
  }
  chunk_sum[tid] = local;
  __syncthreads();
  if (tid < 32) {
    // warp 0 walks the cumulative distribution: lane l owns chunk sums [32 l, 32 l + 32), then the owning
    // chunk's values are shared out among the lanes in the same way. The first kept value at which the
    // running sum exceeds u * total is drawn; rounding at the very end falls back to the last kept value.
    const int lane = tid;
    float mine = 0.f;
#pragma unroll 8
    for (int t = 0; t < 32; ++t) mine += chunk_sum[lane * 32 + t];
    float incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    const float total = __shfl_sync(0xffffffffu, incl, 31);
    const float target = uniform[r] * total;
    float run = incl - mine;
    int found = -1, last_nonempty = -1;
    for (int t = 0; t < 32; ++t) {
      const float c = chunk_sum[lane * 32 + t];
      if (c > 0.f) {
        last_nonempty = lane * 32 + t;
        if (found < 0 && run + c > target) found = lane * 32 + t;
      }
      if (found < 0) run += c;
    }
    const unsigned who = __ballot_sync(0xffffffffu, found >= 0);
    int owner, src_lane;
    if (who) {
      src_lane = __ffs(who) - 1;
      owner = __shfl_sync(0xffffffffu, found, src_lane);
    } else {   // rounding at the very end: the last chunk that holds anything, entered with the sum before it
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) last_nonempty = max(last_nonempty, __shfl_xor_sync(0xffffffffu, last_nonempty, o));
      owner = last_nonempty < 0 ? 0 : last_nonempty;   // (nothing kept cannot happen: the largest value always is)
      src_lane = owner >> 5;
      if (lane == src_lane) {
        run = incl - mine;
        for (int t = lane * 32; t < owner; ++t) run += chunk_sum[t];
      }
    }
    float before = __shfl_sync(0xffffffffu, run, src_lane);    // cumulative sum in front of the owning chunk
    // the owning chunk: lane l takes its values [per l, per l + per)
    const int clo = min(vocab, owner * chunk), chi = min(vocab, clo + chunk);
    const int per = (chunk + 31) / 32;
    float vals[8];
    float lsum = 0.f;
    const int l0 = clo + lane * per;
    for (int e = 0; e < 8; ++e) {
      const int i = l0 + e;
      float v = (e < per && i < chi) ? p[i] : 0.f;
      if (!(__float_as_uint(v) >= floor_bits && v > 0.f)) v = 0.f;
      vals[e] = v;
      lsum += v;
    }
    float lincl = lsum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, lincl, o);
      if (lane >= o) lincl += up;
    }
    float lrun = before + lincl - lsum;
    int pick = -1, last_kept = -1;
    for (int e = 0; e < 8; ++e) {
      if (vals[e] > 0.f) {
        last_kept = l0 + e;
        lrun += vals[e];
        if (pick < 0 && lrun > target) pick = l0 + e;
      }
    }
    const unsigned got = __ballot_sync(0xffffffffu, pick >= 0);
    int result;
    if (got) {
      result = __shfl_sync(0xffffffffu, pick, __ffs(got) - 1);
    } else {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) last_kept = max(last_kept, __shfl_xor_sync(0xffffffffu, last_kept, o));
      result = last_kept < 0 ? 0 : last_kept;
    }
    if (lane == 0) picked = result;
  }
  __syncthreads();
  if (tid == 0) out[r] = picked;
}

// ------------------------------------------------------------------------------------------------
// The same selection by a thread-block cluster of kRowCtas CTAs per row, for rows that can be read 16
// bytes at a time. One block per row is bound by what one SM can pull from L2 (three passes over 600 KB
// for a 152k vocabulary, and a scratch row written and read back); here every CTA owns an eighth of the
// row and every thread 32 consecutive values of it, which stay in registers from the one load to the
// draw. The CTAs exchange through distributed shared memory, behind the cluster's barrier: their maxima;
// their sums and exponent histograms; their candidates, appended to the list of the CTA of rank 0, which
// alone searches the thresholds and sends them back; their kept masses, after which the CTA that holds
// the target of the inverse CDF walks to it. Sums over CTAs are formed in rank order by everyone, so
// all CTAs agree and a seeded draw is reproducible. A row whose thresholds the list does not hold (a
// flat distribution, or a list that overflowed) is left to sample_kernel: the cluster writes -1 for it.
constexpr int kRowCtas = 8;
constexpr int kOwn4 = 8;             // float4 per thread: 32 values

struct RowExchange {                 // what the CTAs of a row write into one another's shared memory
  float max_of[kRowCtas];
  float sum_of[kRowCtas];
  float mass_of[kRowCtas];
  int hist_of[kRowCtas][kExpBins];
  unsigned floor_bits;               // from rank 0, with ...
  int answered;                      // ... 1, or 0 when the list did not hold the thresholds
  int list_n;                        // rank 0's counts
  float list[kListCap];              // rank 0's is filled
};

__global__ void __launch_bounds__(kSampleThreads)
sample_cluster_kernel(int* __restrict__ out, const float* __restrict__ logits, long long row_stride, int vocab,
                      const float* __restrict__ temperature, const int* __restrict__ top_k,
                      const float* __restrict__ top_p, const float* __restrict__ min_p,
                      const float* __restrict__ uniform) {
  pdl_start();
  // "this CTA runs": waited for before the first write into another CTA's shared memory
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float red[32];
  __shared__ unsigned long long red64[32];
  __shared__ RowExchange ex;
  __shared__ RadixScratch radix;
  __shared__ int cut_exp, first_tid, last_tid;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rank = (int)cluster.block_rank();
  const int r = blockIdx.x / kRowCtas;
  const float4* row4 = reinterpret_cast<const float4*>(logits + (size_t)r * row_stride);
  const int n4 = vocab / 4, per4 = (n4 + kRowCtas - 1) / kRowCtas;
  const int lo4 = rank * per4, hi4 = min(n4, lo4 + per4);
  const int mine4 = lo4 + tid * kOwn4;           // this thread's values: float4 [mine4, mine4 + kOwn4) below hi4
  const float inv_t = 1.f / temperature[r];
  const int k_req = top_k[r];
  const float tp = top_p[r];
  const bool want_list = (k_req > 0 && k_req < vocab) || tp < 1.f;

  for (int i = tid; i < kRadixBins * 2; i += kSampleThreads) reinterpret_cast<int*>(radix.mass)[i] = 0;
  if (tid == 0) { ex.list_n = 0; ex.answered = 1; ex.floor_bits = 0; }

  // ---- the one load, and the maximum
  float4 x[kOwn4];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kOwn4; ++j) {
    const bool valid = mine4 + j < hi4;
    x[j] = valid ? row4[mine4 + j] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    mx = fmaxf(fmaxf(mx, fmaxf(x[j].x, x[j].y)), fmaxf(x[j].z, x[j].w));
  }
  mx = block_max(mx, red);
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");        // 0: every CTA of the row runs
  if (tid < kRowCtas) *cluster.map_shared_rank(&ex.max_of[rank], tid) = mx;
  cluster.sync();                                // 1: the maxima
  float gmax = ex.max_of[0];
#pragma unroll
  for (int c = 1; c < kRowCtas; ++c) gmax = fmaxf(gmax, ex.max_of[c]);

  // ---- numerators (kept in the registers), their sum, the histogram over exponents of one value in eight
  int* const warp_hist = reinterpret_cast<int*>(radix.mass) + warp * kExpBins;
  float z = 0.f;
#pragma unroll
  for (int j = 0; j < kOwn4; ++j) {
    float4 e;
    e.x = expf((x[j].x - gmax) * inv_t); e.y = expf((x[j].y - gmax) * inv_t);     // exp(-inf) = 0 beyond the slice
    e.z = expf((x[j].z - gmax) * inv_t); e.w = expf((x[j].w - gmax) * inv_t);
    x[j] = e;
    z += (e.x + e.y) + (e.z + e.w);
    if (want_list && (j & 1) == 0 && mine4 + j < hi4) atomicAdd(&warp_hist[__float_as_uint(e.x) >> 23], 1);
  }
  z = block_sum(z, red);                         // also orders the histograms before the reads below
  if (tid < kRowCtas) *cluster.map_shared_rank(&ex.sum_of[rank], tid) = z;
  if (want_list && tid < kExpBins) {
    int c = 0;
    for (int w = 0; w < kSampleThreads / 32; ++w) c += reinterpret_cast<int*>(radix.mass)[w * kExpBins + tid];
    for (int to = 0; to < kRowCtas; ++to) *cluster.map_shared_rank(&ex.hist_of[rank][tid], to) = c;
  }
  cluster.sync();                                // 2: sums and histograms
  float ztot = 0.f;
#pragma unroll
  for (int c = 0; c < kRowCtas; ++c) ztot += ex.sum_of[c];

  unsigned floor_bits = 0;                       // running lower bound of kept values (bit pattern)
  if (want_list) {
    // ---- the candidate list, in the CTA of rank 0: every value at or above 2^(cut_exp - 127)
    if (tid == 0) {
      int total = 0, e = kExpBins;
      while (e > 0) {
        int c = 0;
        for (int q = 0; q < kRowCtas; ++q) c += ex.hist_of[q][e - 1];
        if (total + kCountedOneIn * c > kListCap / 2) break;
        --e;
        total += kCountedOneIn * c;
      }
      cut_exp = e;                               // the same in every CTA: all add the same counts
    }
    __syncthreads();
    const unsigned cut_bits = (unsigned)cut_exp << 23;
    if (cut_exp < kExpBins) {
      int* const n_at_0 = cluster.map_shared_rank(&ex.list_n, 0);
      float* const list_at_0 = cluster.map_shared_rank(&ex.list[0], 0);
      const unsigned below = (1u << lane) - 1u;
      auto take = [&](float v) {
        const bool mine = __float_as_uint(v) >= cut_bits;     // values beyond the slice are 0: never taken (cut_bits > 0 ...
        const unsigned takers = __ballot_sync(0xffffffffu, mine && v > 0.f);   // ... unless the cut is at the bottom)
        if (takers == 0) return;
        int base = 0;
        if (lane == __ffs(takers) - 1) base = atomicAdd(n_at_0, __popc(takers));
        base = __shfl_sync(0xffffffffu, base, __ffs(takers) - 1);
        const int at = base + __popc(takers & below);
        if (mine && v > 0.f && at < kListCap) list_at_0[at] = v;
      };
#pragma unroll
      for (int j = 0; j < kOwn4; ++j) { take(x[j].x); take(x[j].y); take(x[j].z); take(x[j].w); }
    }
    cluster.sync();                              // 3: the list is complete
    if (rank == 0) {
      const int ln = (cut_exp < kExpBins && ex.list_n <= kListCap) ? ex.list_n : 0;
      bool ok = true;
      float kept_mass = ztot;
      if (k_req > 0 && k_req < vocab) {
        int cnt;
        if (k_req <= ln) floor_bits = radix_threshold(ex.list, ln, 0u, false, k_req, 0.f, radix, cnt, kept_mass);
        else ok = false;
      }
      if (ok && tp < 1.f) {
        const float need = tp * kept_mass;
        int cnt; float in_list, m;
        count_mass_list(ex.list, ln, floor_bits, 0u, red64, cnt, in_list);
        if (ln > 0 && cnt > 0 && in_list >= need) {
          const unsigned cur = radix_threshold(ex.list, ln, floor_bits, true, 0, need, radix, cnt, m);
          if (cur > floor_bits) floor_bits = cur;
        } else {
          ok = false;
        }
      }
      if (tid < kRowCtas) {
        *cluster.map_shared_rank(&ex.floor_bits, tid) = floor_bits;
        *cluster.map_shared_rank(&ex.answered, tid) = ok ? 1 : 0;
      }
    }
    cluster.sync();                              // 4: the thresholds
    floor_bits = ex.floor_bits;
    if (!ex.answered) {                          // nobody touches anybody's shared memory after this barrier
      if (rank == 0 && tid == 0) out[r] = kNoAnswer;
      return;
    }
  }
  const float mp = min_p[r];
  if (mp > 0.f && __float_as_uint(mp) > floor_bits) floor_bits = __float_as_uint(mp);   // p_max = 1 in this scale

  // ---- inverse CDF in vocabulary order: thread t of CTA c owns values [32 (1024 c' + t), +32) of the row
  float own = 0.f;
#pragma unroll
  for (int j = 0; j < kOwn4; ++j) {
    if (__float_as_uint(x[j].x) >= floor_bits) own += x[j].x;
    if (__float_as_uint(x[j].y) >= floor_bits) own += x[j].y;
    if (__float_as_uint(x[j].z) >= floor_bits) own += x[j].z;
    if (__float_as_uint(x[j].w) >= floor_bits) own += x[j].w;
  }
  // what the threads before this one hold (warp scan, then the warps before this one)
  float incl = own;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  __syncthreads();                               // red is free again
  if (lane == 31) red[warp] = incl;
  if (tid == 0) { first_tid = kSampleThreads; last_tid = -1; }
  __syncthreads();
  float before = 0.f, cta_mass = 0.f;
  for (int w = 0; w < kSampleThreads / 32; ++w) {
    if (w < warp) before += red[w];
    cta_mass += red[w];
  }
  before += incl - own;
  if (tid < kRowCtas) *cluster.map_shared_rank(&ex.mass_of[rank], tid) = cta_mass;
  cluster.sync();                                // 5: the kept masses; no remote access after this
  float total = 0.f, offset = 0.f;
#pragma unroll
  for (int c = 0; c < kRowCtas; ++c) {
    if (c < rank) offset += ex.mass_of[c];
    total += ex.mass_of[c];
  }
  const float target = uniform[r] * total;
  // the CTA that holds the target: the first whose range ends beyond it; rounding at the very end falls to
  // the last CTA that keeps anything
  int owner = -1, last_with_mass = -1;
  {
    float run = 0.f;
    for (int c = 0; c < kRowCtas; ++c) {
      const float m = ex.mass_of[c];
      if (m > 0.f) {
        last_with_mass = c;
        if (owner < 0 && run + m > target) owner = c;
      }
      run += m;
    }
    if (owner < 0) owner = last_with_mass < 0 ? 0 : last_with_mass;
  }
  if (rank != owner) return;
  if (own > 0.f) {
    atomicMax(&last_tid, tid);
    if (offset + before + own > target) atomicMin(&first_tid, tid);
  }
  __syncthreads();
  const int chosen = first_tid < kSampleThreads ? first_tid : last_tid;    // (nothing kept cannot happen: the largest value always is)
  if (tid != (chosen < 0 ? 0 : chosen)) return;
  float run = offset + before;
  int pick = -1, last_kept = -1;
#pragma unroll
  for (int j = 0; j < kOwn4; ++j) {
    const float v[4] = {x[j].x, x[j].y, x[j].z, x[j].w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (__float_as_uint(v[e]) >= floor_bits && v[e] > 0.f) {
        last_kept = 4 * (mine4 + j) + e;
        run += v[e];
        if (pick < 0 && run > target) pick = last_kept;
      }
    }
  }
  out[r] = pick >= 0 ? pick : (last_kept >= 0 ? last_kept : 0);
}

// Log-probabilities for requests that ask for them: for each listed row of the logits, the log-softmax
// value of the picked token and the `k` largest entries (id and log-probability, in descending order of
// the raw logits, ties to the lowest id, so that rounding of the subtraction cannot change the order).
// The log-sum-exp is accumulated in double precision (a 150k-wide sum loses digits in float32). As the
// reference's host routine (pegainfer-sample/src/lib.rs:305-358), on the device.
constexpr int kLogprobThreads = 512;

__global__ void __launch_bounds__(kLogprobThreads)
token_logprob_kernel(const float* __restrict__ logits, long long row_stride, int vocab, const int* __restrict__ rows,
                     const int* __restrict__ picked, const int* __restrict__ ks, int k_max, float* __restrict__ out_lp,
                     float* __restrict__ top_vals, int* __restrict__ top_ids) {
  pdl_start();
  __shared__ float red[32];
  __shared__ double redd[32];
  __shared__ float sv[32];
  __shared__ int si[32];
  const int r = blockIdx.x;
  const float* row = logits + (size_t)rows[r] * row_stride;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float mx = -INFINITY;
  for (int i = tid; i < vocab; i += kLogprobThreads) mx = fmaxf(mx, row[i]);
  mx = block_max(mx, red);
  double sum = 0.0;
  for (int i = tid; i < vocab; i += kLogprobThreads) sum += (double)expf(row[i] - mx);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) redd[warp] = sum;
  __syncthreads();
  sum = 0.0;
  for (int w = 0; w < kLogprobThreads / 32; ++w) sum += redd[w];
  const float lse = mx + (float)log(sum);
  if (tid == 0) {
    int pk = picked[r];
    pk = pk < 0 ? 0 : (pk >= vocab ? vocab - 1 : pk);
    out_lp[r] = row[pk] - lse;
  }
  int k = ks[r];
  k = k < k_max ? k : k_max;
  k = k < vocab ? k : vocab;
  ArgPair last{INFINITY, -1};     // everything comes after this in the order (value descending, id ascending)
  for (int j = 0; j < k; ++j) {
    ArgPair best{-INFINITY, 0x7fffffff};
    for (int i = tid; i < vocab; i += kLogprobThreads) {
      const float v = row[i];
      if (v == v && (v < last.v || (v == last.v && i > last.i))) best = better(best, ArgPair{v, i});
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgPair other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
      best = better(best, other);
    }
    __syncthreads();
    if (lane == 0) { sv[warp] = best.v; si[warp] = best.i; }
    __syncthreads();
    ArgPair b{sv[0], si[0]};
    for (int w = 1; w < kLogprobThreads / 32; ++w) b = better(b, ArgPair{sv[w], si[w]});
    if (tid == 0) {
      const bool found = b.i != 0x7fffffff;
      top_ids[(size_t)r * k_max + j] = found ? b.i : -1;
      top_vals[(size_t)r * k_max + j] = found ? b.v - lse : -INFINITY;
    }
    last = b;
  }
  if (tid == 0)
    for (int j = k; j < k_max; ++j) { top_ids[(size_t)r * k_max + j] = -1; top_vals[(size_t)r * k_max + j] = -INFINITY; }
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

static int g_sample_no_clusters = 0;
// 1: every row goes to the kernel of one block per row (for tests and comparisons)
OI_API int oi_sample_use_clusters(int on) { g_sample_no_clusters = on ? 0 : 1; return OI_OK; }

// Per-row parameter arrays live on the device. `probs` is caller-provided scratch of
// rows * vocab floats. temperature must be > 0 (greedy rows go to oi_argmax).
OI_API int oi_sample(int* out, const float* logits, long long row_stride, float* probs, int rows, int vocab,
                     const float* temperature, const int* top_k, const float* top_p, const float* min_p,
                     const float* uniform, void* stream) {
  OI_REQUIRE(rows >= 0 && vocab > 0 && row_stride >= vocab, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
  OI_REQUIRE(probs != nullptr, "sample: scratch missing");
  OI_REQUIRE(vocab <= 8 * 32 * kSampleThreads, "sample: vocabulary %d beyond %d", vocab, 8 * 32 * kSampleThreads);
  if (rows == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  // rows that can be read 16 bytes at a time go to the clusters first; what they leave unanswered, and every
  // other shape, to the kernel of one block per row
  const bool clusters = vocab % 4 == 0 && row_stride % 4 == 0 && ((uintptr_t)logits) % 16 == 0 &&
                        vocab <= kRowCtas * kSampleThreads * kOwn4 * 4 && !g_sample_no_clusters;
  if (clusters) {
    oi_launch_cluster(sample_cluster_kernel, rows * kRowCtas, kSampleThreads, 0, s, kRowCtas, out, logits, row_stride, vocab,
                      temperature, top_k, top_p, min_p, uniform);
    OI_CHECK_LAUNCH();
  }
  oi_launch(sample_kernel, rows, kSampleThreads, 0, s, out, logits, row_stride, probs, vocab, temperature, top_k, top_p, min_p,
            uniform, clusters ? 1 : 0);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

// For n listed rows of float32 logits: out_lp[i] = log-softmax of token picked[i] (ids on the device: they
// may come straight from the sampler), and the ks[i] <= k_max largest entries of the row into
// top_ids / top_vals [n, k_max] (unused places: -1 / -inf).
OI_API int oi_token_logprobs(const float* logits, long long row_stride, int vocab, const int* rows, const int* picked,
                             const int* ks, int n, int k_max, float* out_lp, float* top_vals, int* top_ids, void* stream) {
  OI_REQUIRE(n >= 0 && vocab > 0 && row_stride >= vocab && k_max >= 0, "token_logprobs: bad sizes");
  OI_REQUIRE(k_max == 0 || (top_vals && top_ids), "token_logprobs: outputs missing");
  if (n == 0) return OI_OK;
  oi_launch(token_logprob_kernel, n, kLogprobThreads, 0, (cudaStream_t)stream, logits, row_stride, vocab, rows, picked, ks,
            k_max, out_lp, top_vals, top_ids);
  OI_CHECK_LAUNCH();
  return OI_OK;
}
