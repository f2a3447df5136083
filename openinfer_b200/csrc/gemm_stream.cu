// out[M, N] = x[M, K] * W[N, K]^T for few rows of x (decode: M <= 128) as a weight STREAM through the
// 5th-generation tensor cores. The product is formed transposed: 128 weight rows are the M side of
// tcgen05.mma (operand A), the tokens its N side (operand B, padded to 16 / 32 / 64 / 128 by TMA's
// zero fill), so a weight byte goes HBM -> TMA -> shared memory -> tensor core without passing
// through a register, and the accumulator [128 weight rows x tokens] lies in tensor memory.
//
// Grid (c, ceil(N / 128)): a cluster of c CTAs along x shares one tile of 128 weight rows, CTA r of
// the cluster streaming k blocks [r * kb_per_rank, ...) of it. Roles in a CTA:
//   warp 0     one thread issues the TMA loads into a ring of stages (a [128 x 64] box of W with an
//              evict-first L2 policy, a [tokens x 64] box of x); the first ring-full of WEIGHT boxes
//              is requested before waiting for the kernel that produces x (programmatic dependent
//              launch), so the stream starts under the predecessor's tail;
//   warp 1     one thread issues four tcgen05.mma (K = 16 each) per stage, commits the stage back to
//              the producer, and commits the accumulator once at the end;
//   warps 2-5  read the accumulator (tcgen05.ld, one weight row per thread) and either store it
//              (c = 1) or leave it as a float32 partial in shared memory.
// With c > 1 every CTA deposits its partial sums of a row in the shared memory of the CTA that owns the
// row (CTA r owns rows [r * 128 / c, ...) of the tile), through distributed shared memory; after ONE
// cluster barrier each CTA adds up what it was given, in rank order, so the result does not depend on
// timing, and nobody reads remote memory after the barrier (no second barrier before leaving).
// Two CTAs fit on an SM (<= 112 KB of stages each). Every mbarrier wait is bounded (two seconds): a
// wait that runs out sets an error word and a flag that ends all roles of the CTA, which still
// joins its cluster's barriers, frees its tensor memory and returns. No load uses cluster multicast.
//
// Two optional additions where the K slices are added up take the two norm kernels out of a decode layer
// (OiStreamEpilogue, oi_api.h). A product that ENDS a residual branch (O, down) adds the residual stream,
// out = round(h + sum), and leaves behind what the next norm needs: the row's new values times the norm's
// weight (xs) and, per block of columns it owns, the sum of their squares. The product that FOLLOWS (gate/up,
// QKV) takes xs as its input and multiplies row m of its sums by rsqrt(mean square + eps), added up from those
// partial sums in a fixed order. One rounding of the normalised activations, as with the norm kernel; the
// residual sum is formed from the float32 sums (the norm kernel adds a branch output that was rounded first).
//
// The reference calls a library product for every projection, also in decode
// (pegainfer-kernels/csrc/shared/linear.cu:312-362: bf16 in, float32 accumulate, row-major weight).
#include <cooperative_groups.h>

#include <type_traits>

#include "oi_api.h"
#include "tcgen05.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int BM = 128;                // weight rows per tile
constexpr int BK = 64;                 // 64 bf16 = 128 bytes = one swizzle row
constexpr int kThreads = 192;

__device__ int g_stream_error = 0;     // set to a non-zero code when a bounded wait ran out

template <int BN>
struct Layout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // where the other CTAs of a cluster deposit their partial sums: a region of its own, because they may
  // do so while this CTA still streams (up to 32 tokens; more tokens run without clusters)
  static constexpr int kRecvBytes = BN <= 32 ? BN * BM * 4 : 0;
  // Two CTAs of 112 KB per SM. Measured with less (three CTAs of 64 KB and three stages, so that the next product's CTAs
  // find room beside this one's): Qwen3-8B sizes, batch 8, 3.73 ms a step against 3.50 ms; 80 KB: 3.56 ms.
  static constexpr int kStages = (112 * 1024 - kRecvBytes) / kStageBytes;   // 5, 4, 4, 3 for BN 16, 32, 64, 128
  static constexpr int kRecvOffset = kStages * kStageBytes;
  static constexpr int kBarOffset = kRecvOffset + kRecvBytes;           // full[kStages], empty[kStages], acc_full
  static constexpr int kNumBars = 2 * kStages + 1;
  static constexpr int kEpiOffset = kBarOffset + kNumBars * 8 + 16;     // rstd[32], squares [32][4]
  static constexpr int kTotal = kEpiOffset + (32 + 32 * 4) * 4;
  static constexpr int kTmemCols = BN < 32 ? 32 : BN;
  static_assert(BN * BM * 4 <= kStages * kStageBytes, "without a cluster the partial sums reuse the stages");
};

// the residual stream's value: read past L1, another SM wrote it a few kernels ago
__device__ __forceinline__ float load_residual(const OiStreamEpilogue& ep, int m, int col) {
  const unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(ep.residual) + (size_t)m * ep.ld_residual + col);
  return __bfloat162float(__ushort_as_bfloat16(raw));
}
__device__ __forceinline__ float load_norm_weight(const OiStreamEpilogue& ep, int col) {
  return ep.w_offset + (ep.norm_w_bf16 ? __bfloat162float(reinterpret_cast<const bf16*>(ep.norm_w)[col])
                                       : reinterpret_cast<const float*>(ep.norm_w)[col]);
}

// kSiluMul: W's rows come in blocks of 64 gate rows followed by the 64 up rows of the same indices, so a
// tile holds gate rows in lanes 0-63 of the accumulator and their up rows in lanes 64-127; the result
// is out[M, N / 2] = act(gate) * up (act: OI_ACT_SILU or OI_ACT_GELU_TANH), formed where the K slices are added up.
struct NoEpilogue {};

// kEpi: 0 none; 1 the product follows a norm (rows scaled by the reciprocal root mean square); 2 it ends a residual branch
template <int BN, typename TOut, bool kSiluMul, int kEpi>
__global__ void __launch_bounds__(kThreads)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   TOut* __restrict__ out, long long ldc, int M, int N, int num_kb, int kb_per_rank, int act,
                   const typename std::conditional<kEpi == 0, NoEpilogue, OiStreamEpilogue>::type ep_arg) {
  pdl_trigger();
  OiStreamEpilogue ep = {};
  if constexpr (kEpi != 0) ep = ep_arg;
  constexpr bool kFollowsNorm = kEpi == 1, kEndsBranch = kEpi == 2;   // the next kernel may be scheduled now: it reads nothing of ours before we are done
  using L = Layout<BN>;
  constexpr int kStages = L::kStages;
  // the swizzled tiles need a 1024-byte aligned base; no slack is added for it (two CTAs must fit on an SM)
  extern __shared__ __align__(1024) unsigned char smem[];
  const unsigned smem_base = tc::smem_u32(smem);
  const bool misaligned = (smem_base & 1023u) != 0;   // never seen; refuse rather than compute garbage
  const unsigned bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  const unsigned acc_full = bar_base + 8u * (2 * kStages);
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(smem + L::kBarOffset + L::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // partial sums [K slice][token][rows of this CTA's share]: in the region of its own when a cluster adds
  // up, else over the drained stages
  float* recv = reinterpret_cast<float*>(gridDim.x > 1 ? smem + L::kRecvOffset : smem);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = blockIdx.x, csize = gridDim.x;
  const int n0 = blockIdx.y * BM;
  const int kb0 = rank * kb_per_rank;
  int nkb = num_kb - kb0;
  nkb = nkb < kb_per_rank ? nkb : kb_per_rank;
  nkb = nkb > 0 ? nkb : 0;
  if (misaligned) {
    nkb = 0;
    if (threadIdx.x == 0) atomicCAS(&g_stream_error, 0, 9);
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(full_bar(s), 1);
      tc::mbar_init(empty_bar(s), 1);
    }
    tc::mbar_init(acc_full, 1);
    *abort_flag = 0;
    tc::mbar_fence_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(tc::smem_u32(tmem_slot), L::kTmemCols);
    tc::tmem_relinquish();
  }
  tc::fence_before();
  __syncthreads();
  tc::fence_after();
  const unsigned tmem_base = *tmem_slot;
  if (csize > 1) tc::cluster_arrive();   // phase 0: "this CTA runs"; waited for before anyone writes into it

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const unsigned long long once = tc::policy_evict_first();
      const int pre = nkb < kStages ? nkb : kStages;
      for (int s = 0; s < pre; ++s) {
        tc::mbar_expect_tx(full_bar(s), L::kStageBytes);
        tc::tma_load_2d_hint(smem_base + s * L::kStageBytes, &map_w, (kb0 + s) * BK, n0, full_bar(s), once);
      }
      // x is written by the kernel before this one: nothing of it is read before that kernel is done
      pdl_wait();
      for (int s = 0; s < pre; ++s)
        tc::tma_load_2d(smem_base + s * L::kStageBytes + L::kABytes, &map_x, (kb0 + s) * BK, 0, full_bar(s));
      for (int kb = pre; kb < nkb; ++kb) {
        const int s = kb % kStages;
        if (!tc::mbar_wait(empty_bar(s), (unsigned)((kb / kStages) - 1) & 1, abort_flag, &g_stream_error, 1)) break;
        tc::mbar_expect_tx(full_bar(s), L::kStageBytes);
        const unsigned dst = smem_base + s * L::kStageBytes;
        tc::tma_load_2d_hint(dst, &map_w, (kb0 + kb) * BK, n0, full_bar(s), once);
        tc::tma_load_2d(dst + L::kABytes, &map_x, (kb0 + kb) * BK, 0, full_bar(s));
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr unsigned idesc = tc::idesc_bf16_f32(BM, BN);
      bool ok = true;
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % kStages;
        ok = tc::mbar_wait(full_bar(s), (unsigned)(kb / kStages) & 1, abort_flag, &g_stream_error, 2);
        if (!ok) break;
        tc::fence_after();
        const unsigned a_addr = smem_base + s * L::kStageBytes;
        const unsigned long long da = tc::desc_k_major_sw128(a_addr), db = tc::desc_k_major_sw128(a_addr + L::kABytes);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          // 16 elements = 32 bytes further along K inside the swizzle row: +2 in the address field
          tc::umma_bf16(tmem_base, da + 2ull * k, db + 2ull * k, idesc, (kb | k) != 0 ? 1u : 0u);
        }
        tc::umma_commit(empty_bar(s));       // the stage may be refilled once these MMAs have read it
      }
      if (ok && nkb > 0) tc::umma_commit(acc_full);
    }
  } else {
    // ------------------------------------------------------------------ accumulator read-out (warps 2..5)
    const int quarter = warp & 3;            // a warp may only touch lanes [32 * (warp % 4), +32)
    const int row = quarter * 32 + lane;     // weight row of this thread within the tile
    const int n = n0 + row;
    bool ok = true;
    if constexpr (kFollowsNorm) {
      // The reciprocal root mean square of every row, from the partial sums of squares that the product before this
      // one left ([row][unit], 16 bytes per load). A warp takes rows warp, warp + 4, ...; all of a lane's loads are
      // in flight at once, its values are added in index order and the lanes' sums by a fixed shuffle tree. This
      // runs beside the first products of the K loop; the rows are scaled after the loop.
      pdl_wait();
      float* rstd_out = reinterpret_cast<float*>(smem + L::kEpiOffset);
      const int units = ep.ssq_units, quads = (units + 3) >> 2;
      for (int m0 = warp - 2; m0 < M; m0 += 16) {          // four rows of this warp at a time
        float total[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int m = m0 + 4 * r;
          if (m < M) {
            const float4* src = reinterpret_cast<const float4*>(ep.ssq_in + (size_t)m * ep.ssq_stride);
            for (int j = lane; j < quads; j += 32) {
              const float4 v = __ldcg(src + j);
              const int u = 4 * j;
              total[r] += v.x + (u + 1 < units ? v.y : 0.f) + (u + 2 < units ? v.z : 0.f) + (u + 3 < units ? v.w : 0.f);
            }
          }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          float t = total[r];
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
          const int m = m0 + 4 * r;
          if (lane == 0 && m < M) rstd_out[m] = rsqrtf(t * ep.inv_width + ep.eps);
        }
      }
    }
    if (nkb > 0) {
      ok = tc::mbar_wait(acc_full, 0, abort_flag, &g_stream_error, 3);
      tc::fence_after();
    }
    const unsigned tmem_row = tmem_base + ((unsigned)(quarter * 32) << 16);
#pragma unroll 1
    for (int c0 = 0; c0 < BN && c0 < M; c0 += 16) {
      unsigned v[16];
      if (nkb > 0 && ok) {
        tc::tmem_ld16(tmem_row + (unsigned)c0, v);
        tc::tmem_ld_wait();
      } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = 0u;
      }
      if (csize == 1 && !kSiluMul && kEpi == 0) {
        if (n < N) {
#pragma unroll
          for (int e = 0; e < 16; ++e)
            if (c0 + e < M) out[(size_t)(c0 + e) * ldc + n] = from_f32<TOut>(__uint_as_float(v[e]));
        }
      } else {
        // Deposit this row's partial sums with the CTA that adds the row up. Rows are shared out evenly:
        // CTA j takes rows [j * 128 / c, ...) (with the activation: gate rows [j * 64 / c, ...) and, behind
        // them in its buffer, the up rows of the same indices).
        const int share = BM / csize;                       // values per (slice, token) in a CTA's buffer
        int owner, local;
        if (kSiluMul) {
          const int idx = row & (BM / 2 - 1), per = BM / 2 / csize;
          owner = idx / per;
          local = (row >= BM / 2 ? per : 0) + idx % per;
        } else {
          owner = row / share;
          local = row % share;
        }
        if (c0 == 0 && csize > 1) tc::cluster_wait();       // phase 0: every CTA of the cluster runs
        float* dst = (csize > 1 ? cg::this_cluster().map_shared_rank(recv, owner) : recv) + (size_t)(rank * BN + c0) * share + local;
#pragma unroll
        for (int e = 0; e < 16; ++e) dst[e * share] = __uint_as_float(v[e]);
      }
    }
  }

  // ------------------------------------------------------------------ sum over the K slices, teardown
  tc::fence_before();
  if (csize > 1 || kSiluMul || kEpi != 0) {
    // What the residual form adds to an element is requested here, before the barrier behind which the sums stand
    // ready: the L2 latency of the residual stream passes under the barrier's.
    float h_pre[2] = {0.f, 0.f}, w_pre[2] = {0.f, 0.f};
    if constexpr (kEndsBranch) {
      pdl_wait();   // every thread reads what kernels before this one wrote
      constexpr int kOut = kSiluMul ? BM / 2 : BM;
      const int mine = kOut / csize, first = (kSiluMul ? n0 / 2 : n0) + rank * mine, width = kSiluMul ? N / 2 : N;
#pragma unroll
      for (int it = 0; it < 2; ++it) {
        const int i = it * kThreads + threadIdx.x;
        if (i < M * mine) {
          const int m = i / mine, col = first + (i - m * mine);
          if (col < width) {
            h_pre[it] = load_residual(ep, m, col);
            if (ep.xs) w_pre[it] = load_norm_weight(ep, col);
          }
        }
      }
    }
    if (csize > 1) {
      if (warp < 2) tc::cluster_wait();   // the read-out warps waited before their first deposit
      tc::cluster_arrive();               // phase 1: this CTA's deposits are made ...
      tc::cluster_wait();                 // ... and so are everybody's; nothing remote is touched after this
    } else {
      __syncthreads();
    }
    constexpr int kOutRows = kSiluMul ? BM / 2 : BM;   // output columns per tile
    const int share = BM / csize;
    const int rows_mine = kOutRows / csize;
    const int n_out = kSiluMul ? N / 2 : N, o0 = (kSiluMul ? n0 / 2 : n0) + rank * rows_mine;
    float* rstd_s = reinterpret_cast<float*>(smem + L::kEpiOffset);
    float* sq_s = rstd_s + 32;                          // [token][chunk of 32 (or 16) columns]
    const int chunk = rows_mine < 32 ? rows_mine : 32;  // columns whose squares one shuffle reduction adds up
    const int total_elems = M * rows_mine;
    for (int i0 = 0, it = 0; i0 < total_elems; i0 += kThreads, ++it) {
      const int i = i0 + threadIdx.x;
      const bool live = i < total_elems;
      const int m = live ? i / rows_mine : 0, l = live ? i - m * rows_mine : 0;
      const bool valid = live && o0 + l < n_out;
      const int col = o0 + l;
      // the residual and the norm weight of this element: requested before the sums are read (the first two
      // elements of a thread even before the cluster's barrier, see above)
      float hv = 0.f, wv = 0.f;
      if constexpr (kEndsBranch) {
        if (it < 2) {
          hv = h_pre[it];
          wv = w_pre[it];
        } else if (valid) {
          hv = load_residual(ep, m, col);
          if (ep.xs) wv = load_norm_weight(ep, col);
        }
      }
      float sum = 0.f, up = 0.f;
      if (live) {
        for (int q = 0; q < csize; ++q) {                // slice order: the result does not depend on timing
          sum += recv[(size_t)(q * BN + m) * share + l];
          if (kSiluMul) up += recv[(size_t)(q * BN + m) * share + rows_mine + l];
        }
        if constexpr (kFollowsNorm) {
          sum *= rstd_s[m];
          up *= rstd_s[m];
        }
        if (kSiluMul) sum = gate_act<true>(sum, act) * up;
      }
      float sq = 0.f;
      if constexpr (kEndsBranch) {
        if (valid) {
          const float hr = __bfloat162float(__float2bfloat16_rn(hv + sum));
          out[(size_t)m * ldc + col] = from_f32<TOut>(hr);
          if (ep.xs) {
            ep.xs[(size_t)m * ep.ld_xs + col] = __float2bfloat16_rn(hr * wv);
            sq = hr * hr;
          }
        }
        if (ep.xs) {
          // squares of `chunk` neighbouring columns of one token, added up in a fixed pattern
          for (int off = chunk >> 1; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
          if (live && (l & (chunk - 1)) == 0) sq_s[m * 4 + l / chunk] = sq;
        }
      } else {
        if (valid) out[(size_t)m * ldc + col] = from_f32<TOut>(sum);
      }
    }
    if (kEndsBranch && ep.xs) {
      __syncthreads();
      if (threadIdx.x < 32) {
        float total = 0.f;
        if (threadIdx.x < M)
          for (int c = 0; c < rows_mine / chunk; ++c) total += sq_s[threadIdx.x * 4 + c];
        if (threadIdx.x < M) ep.ssq_out[(size_t)threadIdx.x * ep.ssq_stride + blockIdx.y * csize + rank] = total;
      }
    }
  } else {
    __syncthreads();
  }
  if (*abort_flag && threadIdx.x == 0) {
    // copies that were issued may still be landing in this CTA's shared memory: give them time
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) {
    tc::fence_after();
    tc::tmem_dealloc(tmem_base, L::kTmemCols);
  }
}

template <int BN, typename TOut, bool kSiluMul, int kEpi>
int launch_variant(void* out, long long ldc, const void* x, long long ldx, const void* W, long long ldw, int M, int N, int K,
                   int csize, int act, const OiStreamEpilogue& ep, cudaStream_t s) {
  using L = Layout<BN>;
  CUtensorMap mw, mx;
  int rc = tc::make_map_2d_bf16(&mw, W, N, K, ldw, BM);
  OI_REQUIRE(rc == 0, "gemm_stream: tensor map for the weight failed (%d)", rc);
  rc = tc::make_map_2d_bf16(&mx, x, M, K, ldx, BN);
  OI_REQUIRE(rc == 0, "gemm_stream: tensor map for x failed (%d)", rc);
  auto kernel = gemm_stream_kernel<BN, TOut, kSiluMul, kEpi>;
  static bool configured = false;
  if (!configured) {
    OI_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
    configured = true;
  }
  const int num_kb = (K + BK - 1) / BK;
  const int kb_per_rank = (num_kb + csize - 1) / csize;
  if constexpr (kEpi == 0)
    oi_launch_cluster(kernel, dim3(csize, (N + BM - 1) / BM, 1), kThreads, L::kTotal, s, csize, mw, mx, (TOut*)out, ldc, M, N,
                      num_kb, kb_per_rank, act, NoEpilogue{});
  else
    oi_launch_cluster(kernel, dim3(csize, (N + BM - 1) / BM, 1), kThreads, L::kTotal, s, csize, mw, mx, (TOut*)out, ldc, M, N,
                      num_kb, kb_per_rank, act, ep);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

// the variants with additions exist for bfloat16 output and up to 32 rows (BN 16 and 32) only
template <int BN, typename TOut, bool kSiluMul>
int launch(void* out, long long ldc, const void* x, long long ldx, const void* W, long long ldw, int M, int N, int K,
           int csize, int act, const OiStreamEpilogue& ep, cudaStream_t s) {
  if constexpr (BN <= 32 && std::is_same<TOut, bf16>::value) {
    if (ep.ssq_in) return launch_variant<BN, TOut, kSiluMul, 1>(out, ldc, x, ldx, W, ldw, M, N, K, csize, act, ep, s);
    if constexpr (!kSiluMul) {
      if (ep.residual) return launch_variant<BN, TOut, false, 2>(out, ldc, x, ldx, W, ldw, M, N, K, csize, act, ep, s);
    }
  }
  return launch_variant<BN, TOut, kSiluMul, 0>(out, ldc, x, ldx, W, ldw, M, N, K, csize, act, ep, s);
}

}  // namespace

// x: [M, K] bfloat16 (row stride ldx), W: [N, K] bfloat16 (row stride ldw), out: [M, N] bfloat16 or
// float32 (row stride ldc), 1 <= M <= 128. K and the row strides of x and W must be multiples of 8
// elements and their bases 16-byte aligned (TMA). cluster_size in {1, 2, 4, 8}: the number of K
// slices; it must not exceed the number of 64-wide k blocks. act != 0 (OI_ACT_SILU or OI_ACT_GELU_TANH; N a
// multiple of 128): W's rows come in blocks of 64 gate rows followed by their 64 up rows and out is
// [M, N / 2] = act(gate) * up.
OI_API int oi_gemm_stream(void* out, int out_dtype, long long ldc, const void* x, long long ldx, const void* W,
                          long long ldw, int M, int N, int K, int cluster_size, int act, void* stream) {
  return oi_gemm_stream_fused(out, out_dtype, ldc, x, ldx, W, ldw, M, N, K, cluster_size, act, nullptr, stream);
}

// The same with the additions of OiStreamEpilogue (null: none). They need up to 32 rows of x, bfloat16 output, and for
// the residual form no activation; the partial squares are float32 [32 rows][ssq_stride], one entry per (tile of 128
// weight rows, K slice), 16-byte aligned.
OI_API int oi_gemm_stream_fused(void* out, int out_dtype, long long ldc, const void* x, long long ldx, const void* W,
                                long long ldw, int M, int N, int K, int cluster_size, int act, const OiStreamEpilogue* epilogue,
                                void* stream) {
  const int silu_mul = act;
  OiStreamEpilogue ep;
  memset(&ep, 0, sizeof(ep));
  if (epilogue) ep = *epilogue;
  OI_REQUIRE(act >= OI_ACT_NONE && act <= OI_ACT_GELU_TANH, "gemm_stream: unknown activation code %d", act);
  OI_REQUIRE(M >= 1 && M <= 128, "gemm_stream: M=%d outside 1..128", M);
  OI_REQUIRE(N >= 1 && K >= 8, "gemm_stream: bad sizes N=%d K=%d", N, K);
  OI_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0, "gemm_stream: K and row strides must be multiples of 8");
  OI_REQUIRE((uintptr_t)x % 16 == 0 && (uintptr_t)W % 16 == 0, "gemm_stream: operands must be 16-byte aligned");
  OI_REQUIRE(cluster_size == 1 || cluster_size == 2 || cluster_size == 4 || cluster_size == 8,
             "gemm_stream: cluster size %d", cluster_size);
  OI_REQUIRE(cluster_size == 1 || M <= 32, "gemm_stream: clusters take up to 32 rows of x (M=%d)", M);
  OI_REQUIRE(!silu_mul || N % BM == 0, "gemm_stream: the fused activation needs N %% 128 == 0 (N=%d)", N);
  if (ep.ssq_in || ep.residual) {
    OI_REQUIRE(M <= 32 && out_dtype == OI_BF16, "gemm_stream: the norm additions take up to 32 rows and bfloat16 output (M=%d)", M);
    OI_REQUIRE(!(ep.ssq_in && ep.residual), "gemm_stream: a product either follows a norm or ends a residual branch");
    OI_REQUIRE(!ep.ssq_in || (ep.ssq_units > 0 && ep.inv_width > 0.f), "gemm_stream: partial squares without their count or width");
    OI_REQUIRE((!ep.ssq_in && !ep.ssq_out) ||
                   (ep.ssq_stride % 4 == 0 && ep.ssq_stride >= (ep.ssq_in ? ep.ssq_units : ((N + BM - 1) / BM) * cluster_size) &&
                    (uintptr_t)(ep.ssq_in ? (const void*)ep.ssq_in : (const void*)ep.ssq_out) % 16 == 0),
               "gemm_stream: the partial squares are [row][unit] with a row stride that is a multiple of 4 and holds every unit");
    OI_REQUIRE(!ep.residual || (!silu_mul && ep.ld_residual >= N), "gemm_stream: the residual form takes no activation");
    OI_REQUIRE(!ep.xs || (ep.residual && ep.norm_w && ep.ssq_out && ep.ld_xs >= N),
               "gemm_stream: the scaled copy needs the residual form, a norm weight and a place for the partial squares");
  }
  const int num_kb = (K + BK - 1) / BK;
  OI_REQUIRE((cluster_size - 1) * ((num_kb + cluster_size - 1) / cluster_size) < num_kb,
             "gemm_stream: %d slices leave one without a k block (K=%d)", cluster_size, K);
  cudaStream_t s = (cudaStream_t)stream;
#define OI_STREAM(BN_)                                                                                            \
  do {                                                                                                            \
    if (out_dtype == OI_BF16 && silu_mul) return launch<BN_, bf16, true>(out, ldc, x, ldx, W, ldw, M, N, K, cluster_size, act, ep, s);  \
    if (out_dtype == OI_BF16) return launch<BN_, bf16, false>(out, ldc, x, ldx, W, ldw, M, N, K, cluster_size, 0, ep, s); \
    if (out_dtype == OI_F32 && silu_mul) return launch<BN_, float, true>(out, ldc, x, ldx, W, ldw, M, N, K, cluster_size, act, ep, s);  \
    if (out_dtype == OI_F32) return launch<BN_, float, false>(out, ldc, x, ldx, W, ldw, M, N, K, cluster_size, 0, ep, s); \
  } while (0)
  if (M <= 16) OI_STREAM(16);
  else if (M <= 32) OI_STREAM(32);
  else if (M <= 64) OI_STREAM(64);
  else OI_STREAM(128);
#undef OI_STREAM
  OI_REQUIRE(false, "gemm_stream: unknown output dtype code %d", out_dtype);
}

// 0 when no bounded wait has run out since the last call; otherwise which role gave up (1 producer,
// 2 MMA issuer, 3 read-out, 9 misaligned shared memory). Synchronises the device; clears the word.
OI_API int oi_gemm_stream_status(int* status) {
  int v = 0;
  OI_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_stream_error, sizeof(int)));
  if (v != 0) {
    int zero = 0;
    OI_CHECK_CUDA(cudaMemcpyToSymbol(g_stream_error, &zero, sizeof(int)));
  }
  *status = v;
  return OI_OK;
}
