// C[M, N] = A[M, K] * W[N, K]^T for bfloat16 operands on the 5th-generation tensor cores:
// tcgen05.mma with the accumulator in tensor memory, operands staged in shared memory by TMA.
//
// A persistent CTA per SM computes 128 x BN tiles of C (BN = 256 or 128) one after the other, the
// accumulator double buffered in tensor memory so that a tile's epilogue overlaps the next tile's
// products. Warp roles:
//   warp 0     one elected thread issues the TMA loads of the A tile [128 x 64] and the W tile
//              [BN x 64] of every k block into a ring of stages (128-byte swizzle, the layout the
//              tensor core reads directly), signalling an mbarrier per stage with the byte count;
//   warp 1     allocates tensor memory; one elected thread issues four tcgen05.mma (K = 16 each)
//              per stage and commits them to the stage's "empty" barrier, and after the last k
//              block to the "accumulator ready" barrier;
//   warps 2-9  wait for the accumulator, read it back with tcgen05.ld (a warp reads the quarter of the 128 lanes
//              that its number modulo four names, 32 columns at a time; the two warps of a quarter take half
//              of the tile's columns each), round once and store rows of C. Eight warps, two per scheduler: one
//              warp's chain of tensor-memory load, conversion (with the activation: two special-function
//              operations per value) and store is latency-bound on its own, 26 k cycles for a 128 x 256 tile
//              with four warps, which is more than the products of a tile take when K is 1,024 or 2,048.
// Every wait on an mbarrier is bounded: a wait that runs out sets an error word in global memory
// and a flag in shared memory that ends all roles; the CTA then lets its copies land (bounded),
// frees its tensor memory and returns. No load uses cluster multicast: every CTA fetches its own
// tiles (W tiles are shared between neighbouring CTAs through L2).
//
// This is the hand-written counterpart of the library call the reference makes for every projection
// (pegainfer-kernels/csrc/shared/linear.cu:312-362: bf16 in, float32 accumulate, row-major weight).
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                 // 64 bf16 = 128 bytes = one swizzle row
constexpr int kEpilogueWarps = 8;      // measured: 4 -> 8 warps 4.5 -> 4.1 ms for a 2,048-token prompt at Qwen3-0.6B sizes; 16: no further gain
constexpr int kParts = kEpilogueWarps / 4;          // warps that share a lane quarter split the tile's columns
constexpr int kThreads = 64 + 32 * kEpilogueWarps;  // warps 0, 1: copies and products; the others: the epilogue
constexpr int kPairStages = 6;        // 32 KB each in the kernel of CTA pairs

__device__ int g_gemm_error = 0;       // set to a non-zero code when a bounded wait ran out

using namespace tc;

__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag, int code) {
  return tc::mbar_wait(bar, parity, abort_flag, &g_gemm_error, code);
}
__device__ __forceinline__ void tc_fence_before() { tc::fence_before(); }
__device__ __forceinline__ void tc_fence_after() { tc::fence_after(); }
__device__ __forceinline__ unsigned long long make_desc(unsigned smem_addr) { return tc::desc_k_major_sw128(smem_addr); }

template <int BN, int kStages>
struct Smem {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = kStages * kStageBytes;   // full[kStages], empty[kStages], acc_full[2], acc_empty[2], tmem slot, abort
  static constexpr int kNumBars = 2 * kStages + 4;
  static constexpr int kTotal = kBarOffset + kNumBars * 8 + 16 + 1024;   // + slack to align the base to 1024
};

// One epilogue thread's row of a tile: reads BN float32 columns of its lane of tensor memory, 32 at
// a time, rounds once and stores them (or silu(gate) * up of the column blocks, see the kernels).
template <typename TOut>
__device__ __forceinline__ void store_32(TOut* dst, const float (&a)[32], int valid) {
  if (valid >= 32 && (((uintptr_t)dst) & 15) == 0) {
    if constexpr (sizeof(TOut) == 2) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 o;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) o2[e] = __floats2bfloat162_rn(a[q * 8 + 2 * e], a[q * 8 + 2 * e + 1]);
        reinterpret_cast<uint4*>(dst)[q] = o;
      }
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q)
        reinterpret_cast<float4*>(dst)[q] = make_float4(a[q * 4], a[q * 4 + 1], a[q * 4 + 2], a[q * 4 + 3]);
    }
  } else {
    for (int e = 0; e < 32; ++e)
      if (e < valid) dst[e] = from_f32<TOut>(a[e]);
  }
}

// `part` (0 or 1): which half of the tile's columns this warp takes.
template <int BN, typename TOut, bool kSiluMul>
__device__ __forceinline__ void store_accumulator(unsigned tmem_acc, TOut* __restrict__ C, long long ldc, int row, int n0,
                                                  int M, int N, int act, int part) {
  auto load = [&](int col, float (&a)[32]) {
    unsigned v[32];
    tmem_ld32(tmem_acc + (unsigned)col, v);
    tmem_ld_wait();
#pragma unroll
    for (int e = 0; e < 32; ++e) a[e] = __uint_as_float(v[e]);
  };
  if constexpr (kSiluMul) {
    // the tile's columns: [64 gate | their 64 up] twice; output columns n0 / 2 + 64 * half + c
    const int n_out = N / 2, o0 = n0 / 2;
#pragma unroll 1
    for (int cc = part * (BN / 2 / kParts); cc < (part + 1) * (BN / 2 / kParts); cc += 32) {
      const int half = cc / 64, c = cc % 64;
      float g[32], u[32];
      load(half * 128 + c, g);
      load(half * 128 + 64 + c, u);
      if (row < M) {
#pragma unroll
        for (int e = 0; e < 32; ++e) g[e] = gate_act<true>(g[e], act) * u[e];
        store_32(C + (size_t)row * ldc + o0 + cc, g, n_out - (o0 + cc));
      }
    }
  } else {
#pragma unroll 1
    for (int c = part * (BN / kParts); c < (part + 1) * (BN / kParts); c += 32) {
      float a[32];
      load(c, a);
      if (row < M) store_32(C + (size_t)row * ldc + n0 + c, a, N - (n0 + c));
    }
  }
}

// Persistent: CTA b works on tiles b, b + gridDim.x, ... (row tiles fastest, so CTAs that run at the
// same time share W tiles through L2). The accumulator is double buffered in tensor memory
// (2 x BN columns): while the epilogue warps drain tile i, the MMA warp already fills tile i + 1.
// kSiluMul: W's rows come in blocks of 64 gate rows followed by the 64 up rows of the same indices
// (two such pairs per tile of 256); the epilogue writes silu(gate) * up, [M, N/2] with row stride
// ldc, instead of the product.
template <int BN, int kStages, typename TOut, bool kSiluMul>
__global__ void __launch_bounds__(kThreads)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    TOut* __restrict__ C, long long ldc, int M, int N, int K, int act) {
  pdl_start();
  using L = Smem<BN, kStages>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const unsigned smem_base = smem_u32(smem);
  const unsigned bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(smem + L::kBarOffset + L::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), kEpilogueWarps);      // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 2 * BN);   // two accumulators of BN float32 columns x 128 lanes
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      long long it = 0;   // k blocks issued so far, over all tiles
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = (int)(it % kStages);
          if (it >= kStages && !mbar_wait(empty_bar(s), (unsigned)((it / kStages) - 1) & 1, abort_flag, 1)) { ok = false; break; }
          mbar_expect_tx(full_bar(s), L::kStageBytes);
          const unsigned a_dst = smem_base + s * L::kStageBytes;
          tma_load_2d(a_dst, &map_a, kb * BK, m0, full_bar(s));
          tma_load_2d(a_dst + L::kABytes, &map_b, kb * BK, n0, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptor: D = float32, A = B = bfloat16, both K-major, N = BN, M = 128
      constexpr unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
      long long it = 0;
      int local = 0;      // tiles done by this CTA
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int a = local & 1;
        if (local >= 2) {   // the epilogue must have drained this accumulator (tile local - 2)
          ok = mbar_wait(acc_empty_bar(a), (unsigned)((local >> 1) - 1) & 1, abort_flag, 4);
          if (!ok) break;
          tc_fence_after();
        }
        const unsigned tmem_acc = tmem_base + (unsigned)(a * BN);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = (int)(it % kStages);
          ok = mbar_wait(full_bar(s), (unsigned)(it / kStages) & 1, abort_flag, 2);
          if (!ok) break;
          tc_fence_after();
          const unsigned a_addr = smem_base + s * L::kStageBytes;
          const unsigned long long da = make_desc(a_addr), db = make_desc(a_addr + L::kABytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // 16 elements = 32 bytes further along K inside the swizzle row: +2 in the address field
            umma_bf16(tmem_acc, da + 2ull * k, db + 2ull * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(s));         // the stage may be refilled once these MMAs have read it
        }
        if (ok) umma_commit(acc_full_bar(a));   // this tile's accumulator is complete
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int quarter = warp & 3;            // a warp may only touch lanes [32 * (warp % 4), +32)
    const int part = (warp - 2) >> 2;        // the two warps of a quarter take half of the columns each
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int a = local & 1;
      if (!mbar_wait(acc_full_bar(a), (unsigned)(local >> 1) & 1, abort_flag, 3)) break;
      tc_fence_after();
      const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
      const int row = m0 + quarter * 32 + lane;
      const unsigned tmem_acc = tmem_base + (unsigned)(a * BN) + ((unsigned)(quarter * 32) << 16);
      store_accumulator<BN, TOut, kSiluMul>(tmem_acc, C, ldc, row, n0, M, N, act, part);
      // this warp has read its part of the accumulator: hand it back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(acc_empty_bar(a)) : "memory");
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // copies that were issued may still be landing in this CTA's shared memory: give them time
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ------------------------------------------------------------------------------------------------
// Two CTAs as one tensor-core unit (a cluster of two, tcgen05 cta_group::2): a pair computes
// 256 x 256 tiles of C. The CTA of rank r holds rows [128 r, +128) of the tile's A rows and of its
// W rows in its own shared memory (so each stage is 32 KB per CTA instead of 48 KB for the same
// products per SM, and each SM's shared memory is read and written a third less per product), and
// the float32 accumulator of its 128 rows of C x all 256 columns in its own tensor memory, double
// buffered (512 columns). Roles as above, with these differences:
//   warp 0     of both CTAs loads its own halves; all bytes of a stage are counted on the even
//              CTA's "full" barrier, which that CTA arms with the sum;
//   warp 1     of the even CTA alone issues the products (M = 256, N = 256, K = 16) and commits
//              them to the "empty" barrier of the stage in both CTAs, and each tile's last ones to
//              "accumulator ready" in both; warp 1 of both CTAs allocates and frees tensor memory;
//   warps 2-9  of both CTAs drain their own tensor memory and arrive on the even CTA's
//              "accumulator drained" barrier (16 arrivals).
// Loads carry no cluster multicast: each CTA fetches what it holds. Every wait is bounded as above;
// the two CTAs meet at the cluster's barrier before the tensor memory is freed.
template <int kStages, typename TOut, bool kSiluMul>
__global__ void __launch_bounds__(kThreads)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         TOut* __restrict__ C, long long ldc, int M, int N, int K, int act) {
  pdl_start();
  constexpr int BN = 256, kPairM = 256;
  using L = Smem<128, kStages>;             // per CTA: 128 rows of A and 128 rows of W per stage
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const unsigned smem_base = smem_u32(smem);
  const unsigned bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(smem + L::kBarOffset + L::kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int m_tiles = (M + kPairM - 1) / kPairM, n_tiles = (N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 2 * kEpilogueWarps);      // one arrival per epilogue warp of both CTAs
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), 2 * BN);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_arrive();                        // barriers and tensor memory of both CTAs are ready
  cluster_wait();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      long long it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int m0 = (tile % m_tiles) * kPairM + (int)rank * 128, n0 = (tile / m_tiles) * BN + (int)rank * 128;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = (int)(it % kStages);
          if (it >= kStages && !mbar_wait(empty_bar(s), (unsigned)((it / kStages) - 1) & 1, abort_flag, 1)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(full_bar(s), 2 * L::kStageBytes);
          const unsigned counted_on = map_to_rank(full_bar(s), 0);
          const unsigned a_dst = smem_base + s * L::kStageBytes;
          tma_load_2d_pair(a_dst, &map_a, kb * BK, m0, counted_on);
          tma_load_2d_pair(a_dst + L::kABytes, &map_b, kb * BK, n0, counted_on);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA)
    if (lane == 0 && rank == 0) {
      constexpr unsigned idesc = idesc_bf16_f32(kPairM, BN);
      long long it = 0;
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
        const int a = local & 1;
        if (local >= 2) {
          ok = tc::mbar_wait_cluster(acc_empty_bar(a), (unsigned)((local >> 1) - 1) & 1, abort_flag, &g_gemm_error, 4);
          if (!ok) break;
          tc_fence_after();
        }
        const unsigned tmem_acc = tmem_base + (unsigned)(a * BN);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = (int)(it % kStages);
          ok = mbar_wait(full_bar(s), (unsigned)(it / kStages) & 1, abort_flag, 2);
          if (!ok) break;
          tc_fence_after();
          const unsigned a_addr = smem_base + s * L::kStageBytes;
          const unsigned long long da = make_desc(a_addr), db = make_desc(a_addr + L::kABytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            umma_bf16_pair(tmem_acc, da + 2ull * k, db + 2ull * k, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(empty_bar(s), 3);
        }
        if (ok) umma_commit_pair(acc_full_bar(a), 3);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;
    int local = 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs, ++local) {
      const int a = local & 1;
      if (!mbar_wait(acc_full_bar(a), (unsigned)(local >> 1) & 1, abort_flag, 3)) break;
      tc_fence_after();
      const int m0 = (tile % m_tiles) * kPairM + (int)rank * 128, n0 = (tile / m_tiles) * BN;
      const int row = m0 + quarter * 32 + lane;
      const unsigned tmem_acc = tmem_base + (unsigned)(a * BN) + ((unsigned)(quarter * 32) << 16);
      store_accumulator<BN, TOut, kSiluMul>(tmem_acc, C, ldc, row, n0, M, N, act, part);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_rank(acc_empty_bar(a), 0));
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  cluster_arrive();                        // neither CTA reads or is read by the other from here on
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 2 * BN);
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
template <int BN, int kStages, typename TOut, bool kSiluMul = false>
int launch(void* C, long long ldc, const void* A, long long lda, const void* W, long long ldw, int M, int N, int K,
           cudaStream_t s, int act = 0) {
  CUtensorMap ma, mb;
  int rc = tc::make_map_2d_bf16(&ma, A, M, K, lda, BM);
  OI_REQUIRE(rc == 0, "gemm_tcgen05: tensor map for A failed (%d; -1: cuTensorMapEncodeTiled is not available)", rc);
  rc = tc::make_map_2d_bf16(&mb, W, N, K, ldw, BN);
  OI_REQUIRE(rc == 0, "gemm_tcgen05: tensor map for W failed (%d)", rc);
  auto kernel = gemm_tcgen05_kernel<BN, kStages, TOut, kSiluMul>;
  constexpr int smem = Smem<BN, kStages>::kTotal;
  static bool configured = false;
  if (!configured) {
    OI_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    OI_CHECK_CUDA(cudaGetDevice(&dev));
    OI_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  oi_launch(kernel, tiles < sm_count ? tiles : sm_count, kThreads, smem, s, ma, mb, (TOut*)C, ldc, M, N, K, act);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

template <int kStages, typename TOut, bool kSiluMul = false>
int launch_pair(void* C, long long ldc, const void* A, long long lda, const void* W, long long ldw, int M, int N, int K,
                cudaStream_t s, int act = 0) {
  CUtensorMap ma, mb;
  int rc = tc::make_map_2d_bf16(&ma, A, M, K, lda, 128);
  OI_REQUIRE(rc == 0, "gemm_tcgen05: tensor map for A failed (%d; -1: cuTensorMapEncodeTiled is not available)", rc);
  rc = tc::make_map_2d_bf16(&mb, W, N, K, ldw, 128);
  OI_REQUIRE(rc == 0, "gemm_tcgen05: tensor map for W failed (%d)", rc);
  auto kernel = gemm_tcgen05_pair_kernel<kStages, TOut, kSiluMul>;
  constexpr int smem = Smem<128, kStages>::kTotal;
  static bool configured = false;
  if (!configured) {
    OI_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  static int sm_count = 0;
  if (!sm_count) {
    int dev = 0;
    OI_CHECK_CUDA(cudaGetDevice(&dev));
    OI_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  const int tiles = ((M + 255) / 256) * ((N + 255) / 256);
  const int pairs = tiles < sm_count / 2 ? tiles : sm_count / 2;
  oi_launch_cluster(kernel, 2 * pairs, kThreads, smem, s, 2, ma, mb, (TOut*)C, ldc, M, N, K, act);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

}  // namespace

// A: [M, K] bfloat16, row stride lda; W: [N, K] bfloat16, row stride ldw; C: [M, N] bfloat16 or
// float32, row stride ldc. K and the row strides must be multiples of 8 elements and the bases
// 16-byte aligned (TMA). tile_n: 256 or 128.
// act != 0 (OI_ACT_SILU or OI_ACT_GELU_TANH; tile_n 256, bfloat16 out, N a multiple of 256): W's rows come in
// blocks of 64 gate rows followed by their 64 up rows, and C is [M, N / 2] = act(gate) * up.
OI_API int oi_gemm_tcgen05(void* C, int c_dtype, long long ldc, const void* A, long long lda, const void* W,
                           long long ldw, int M, int N, int K, int tile_n, int act, void* stream) {
  const int silu_mul = act;
  OI_REQUIRE(act >= OI_ACT_NONE && act <= OI_ACT_GELU_TANH, "gemm_tcgen05: unknown activation code %d", act);
  OI_REQUIRE(M >= 1 && N >= 1 && K >= 8, "gemm_tcgen05: bad sizes M=%d N=%d K=%d", M, N, K);
  OI_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0, "gemm_tcgen05: K and row strides must be multiples of 8");
  OI_REQUIRE((uintptr_t)A % 16 == 0 && (uintptr_t)W % 16 == 0, "gemm_tcgen05: operands must be 16-byte aligned");
  OI_REQUIRE(tile_n == 256 || tile_n == 128, "gemm_tcgen05: tile_n %d", tile_n);
  cudaStream_t s = (cudaStream_t)stream;
  if (silu_mul) {
    OI_REQUIRE(tile_n == 256 && c_dtype == OI_BF16 && N % 256 == 0,
               "gemm_tcgen05: the fused activation needs tile_n 256, bfloat16 output and N %% 256 == 0 (N=%d)", N);
    return launch<256, 4, bf16, true>(C, ldc, A, lda, W, ldw, M, N, K, s, act);
  }
  if (c_dtype == OI_BF16) {
    if (tile_n == 256) return launch<256, 4, bf16>(C, ldc, A, lda, W, ldw, M, N, K, s);
    return launch<128, 6, bf16>(C, ldc, A, lda, W, ldw, M, N, K, s);
  }
  if (c_dtype == OI_F32) {
    if (tile_n == 256) return launch<256, 4, float>(C, ldc, A, lda, W, ldw, M, N, K, s);
    return launch<128, 6, float>(C, ldc, A, lda, W, ldw, M, N, K, s);
  }
  OI_REQUIRE(false, "gemm_tcgen05: unknown output dtype code %d", c_dtype);
}

// The same product with 256 x 256 tiles computed by pairs of CTAs (tcgen05 cta_group::2).
OI_API int oi_gemm_tcgen05_pair(void* C, int c_dtype, long long ldc, const void* A, long long lda, const void* W,
                                long long ldw, int M, int N, int K, int act, void* stream) {
  const int silu_mul = act;
  OI_REQUIRE(act >= OI_ACT_NONE && act <= OI_ACT_GELU_TANH, "gemm_tcgen05_pair: unknown activation code %d", act);
  OI_REQUIRE(M >= 1 && N >= 1 && K >= 8, "gemm_tcgen05_pair: bad sizes M=%d N=%d K=%d", M, N, K);
  OI_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0, "gemm_tcgen05_pair: K and row strides must be multiples of 8");
  OI_REQUIRE((uintptr_t)A % 16 == 0 && (uintptr_t)W % 16 == 0, "gemm_tcgen05_pair: operands must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  if (silu_mul) {
    OI_REQUIRE(c_dtype == OI_BF16 && N % 256 == 0,
               "gemm_tcgen05_pair: the fused activation needs bfloat16 output and N %% 256 == 0 (N=%d)", N);
    return launch_pair<kPairStages, bf16, true>(C, ldc, A, lda, W, ldw, M, N, K, s, act);
  }
  if (c_dtype == OI_BF16) return launch_pair<kPairStages, bf16>(C, ldc, A, lda, W, ldw, M, N, K, s);
  if (c_dtype == OI_F32) return launch_pair<kPairStages, float>(C, ldc, A, lda, W, ldw, M, N, K, s);
  OI_REQUIRE(false, "gemm_tcgen05_pair: unknown output dtype code %d", c_dtype);
}

// 0 when no bounded wait has run out since the last call; otherwise which role gave up
// (1 producer, 2 MMA issuer waiting for operands, 3 epilogue, 4 MMA issuer waiting for a drained
// accumulator). Synchronises the device; clears the word.
OI_API int oi_gemm_tcgen05_status(int* status) {
  int v = 0;
  OI_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_gemm_error, sizeof(int)));
  if (v != 0) {
    int zero = 0;
    OI_CHECK_CUDA(cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int)));
  }
  *status = v;
  return OI_OK;
}
