// Skinny product for decode: out[M, N] = x[M, K] * W[N, K]^T with M <= 16 rows of activations,
// bfloat16 operands, float32 accumulation. The step is bound by streaming W from HBM once, so the
// kernel is built around memory parallelism, not tensor throughput:
//
//  * a CTA (8 warps) owns 128 rows of W and one slice of K; the CTAs of a thread-block CLUSTER own
//    the slices of the same rows and add their partial sums through distributed shared memory in
//    rank order (deterministic, no atomics, no scratch in global memory);
//  * each warp streams its 16 rows with 16-byte loads, 8 loads per lane in flight, and feeds
//    mma.sync m16n8k16 with W as the A operand and the activations (staged once per CTA in shared
//    memory) as B. The k index inside a 32-wide block is permuted identically for both operands
//    (a dot product does not care), so a lane's 16 contiguous bytes ARE its fragment registers;
//  * optionally the activation is formed while it is staged: x = silu(g) * u from a fused
//    [M, 2K] gate|up buffer, rounded to bfloat16 exactly as the stand-alone kernel does, which
//    removes a kernel and a round trip through memory from the feed-forward.
//
// The reference calls the vendor library for these products and tunes its algorithm choice per
// shape (pegainfer-kernels/csrc/shared/linear.cu:426-614); same contract: row-major weight,
// no bias, float32 accumulate.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int kRowsPerCta = 128;
constexpr int kWarps = 8;
// Token rows in shared memory are padded so that the row stride is 4 (mod 8) 16-byte chunks: the
// eight lanes that a 128-bit shared load serves at once (two tokens x four chunks) then hit
// eight different bank groups.
__host__ __device__ constexpr int row_stride_elems(int k_slice) {
  return k_slice + (((k_slice / 8) % 8 == 0) ? 32 : 64);
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const bf16* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ float silu(float g) { return g / (1.f + expf(-g)); }

// NT: token tiles of 8 (M <= 8 * NT). kCluster: CTAs along K add up through distributed shared memory.
template <int NT, typename TOut, bool kSiluMul, bool kCluster>
__global__ void __launch_bounds__(kWarps * 32)
gemm_skinny_kernel(TOut* __restrict__ out, long long ldc, const bf16* __restrict__ x, long long ldx,
                   const bf16* __restrict__ W, long long ldw, int M, int N, int K, int k_slice) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int stride = row_stride_elems(k_slice);                 // elements per token row
  bf16* x_s = reinterpret_cast<bf16*>(smem_raw);                // [8 * NT][stride]
  float* part = reinterpret_cast<float*>(smem_raw + (size_t)8 * NT * stride * sizeof(bf16));  // [8 * NT][128]

  const int rank = blockIdx.x;                                  // slice of K == rank in the cluster
  const int k0 = rank * k_slice;
  const int n0 = blockIdx.y * kRowsPerCta;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // ---- stage the activation slice (rows >= M are zero)
  {
    const int vec_per_row = k_slice / 8;
    for (int i = tid; i < 8 * NT * vec_per_row; i += kWarps * 32) {
      const int m = i / vec_per_row, v = i - m * vec_per_row;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (m < M) {
        if (kSiluMul) {
          const uint4 gv = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + k0 + v * 8);
          const uint4 uv = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + K + k0 + v * 8);
          const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
          const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
          __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&val);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 g = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
            o2[e] = __floats2bfloat162_rn(silu(g.x) * u.x, silu(g.y) * u.y);
          }
        } else {
          val = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + k0 + v * 8);
        }
      }
      *reinterpret_cast<uint4*>(x_s + (size_t)m * stride + v * 8) = val;
    }
  }
  __syncthreads();

  // ---- stream W: lane (g, c) owns 8 consecutive k of rows g and g + 8 in every 32-wide block
  const int g = lane >> 2, c = lane & 3;
  const int row_a = min(n0 + warp * 16 + g, N - 1), row_b = min(n0 + warp * 16 + g + 8, N - 1);
  const bf16* pa = W + (size_t)row_a * ldw + k0 + c * 8;
  const bf16* pb = W + (size_t)row_b * ldw + k0 + c * 8;
  const bf16* xs = x_s + (size_t)g * stride + c * 8;
  float acc[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;

  const int nkb = k_slice / 32;
  constexpr int U = 8;
  int kb = 0;
  for (; kb + U <= nkb; kb += U) {
    uint4 wa[U], wb[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      wa[u] = ldg_stream(pa + (kb + u) * 32);
      wb[u] = ldg_stream(pb + (kb + u) * 32);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const uint4 xv = *reinterpret_cast<const uint4*>(xs + (size_t)t * 8 * stride + (kb + u) * 32);
        mma_bf16(acc[t], wa[u].x, wb[u].x, wa[u].y, wb[u].y, xv.x, xv.y);
        mma_bf16(acc[t], wa[u].z, wb[u].z, wa[u].w, wb[u].w, xv.z, xv.w);
      }
    }
  }
  for (; kb < nkb; ++kb) {
    const uint4 wa = ldg_stream(pa + kb * 32), wb = ldg_stream(pb + kb * 32);
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const uint4 xv = *reinterpret_cast<const uint4*>(xs + (size_t)t * 8 * stride + kb * 32);
      mma_bf16(acc[t], wa.x, wb.x, wa.y, wb.y, xv.x, xv.y);
      mma_bf16(acc[t], wa.z, wb.z, wa.w, wb.w, xv.z, xv.w);
    }
  }

  // ---- partial sums of this K slice: part[token][row in tile]
#pragma unroll
  for (int t = 0; t < NT; ++t) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int token = t * 8 + c * 2 + (e & 1);
      const int row = warp * 16 + g + (e >> 1) * 8;
      part[token * kRowsPerCta + row] = acc[t][e];
    }
  }

  if (kCluster) {
    cg::cluster_group cluster = cg::this_cluster();
    const int csize = (int)cluster.num_blocks();
    cluster.sync();
    // rank r adds up rows [r * 128 / csize, (r + 1) * 128 / csize) over all slices, in rank order
    const int rows_mine = kRowsPerCta / csize;
    const int row_lo = rank * rows_mine;
    for (int i = tid; i < M * rows_mine; i += kWarps * 32) {
      const int m = i / rows_mine, row = row_lo + (i - m * rows_mine);
      float sum = 0.f;
      for (int q = 0; q < csize; ++q) {
        const float* remote = cluster.map_shared_rank(part, q);
        sum += remote[m * kRowsPerCta + row];
      }
      const int n = n0 + row;
      if (n < N) out[(size_t)m * ldc + n] = from_f32<TOut>(sum);
    }
    cluster.sync();   // nobody leaves while its shared memory may still be read
  } else {
    __syncthreads();
    for (int i = tid; i < M * kRowsPerCta; i += kWarps * 32) {
      const int m = i / kRowsPerCta, row = i - m * kRowsPerCta;
      const int n = n0 + row;
      if (n < N) out[(size_t)m * ldc + n] = from_f32<TOut>(part[m * kRowsPerCta + row]);
    }
  }
}

template <int NT, typename TOut, bool kSiluMul>
int launch(void* out, long long ldc, const void* x, long long ldx, const void* W, long long ldw, int M, int N,
           int K, int csize, cudaStream_t s) {
  const int k_slice = K / csize;
  const size_t smem = (size_t)8 * NT * row_stride_elems(k_slice) * sizeof(bf16) + (size_t)8 * NT * kRowsPerCta * sizeof(float);
  static size_t configured[2] = {0, 0};   // largest dynamic shared memory set so far, per kernel variant
  const int row_tiles = (N + kRowsPerCta - 1) / kRowsPerCta;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(csize, row_tiles, 1);
  cfg.blockDim = dim3(kWarps * 32, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  if (csize > 1) {
    auto kernel = gemm_skinny_kernel<NT, TOut, kSiluMul, true>;
    if (smem > configured[1]) {
      OI_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured[1] = smem;
    }
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    OI_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kernel, (TOut*)out, ldc, (const bf16*)x, ldx, (const bf16*)W, ldw, M, N, K, k_slice));
  } else {
    auto kernel = gemm_skinny_kernel<NT, TOut, kSiluMul, false>;
    if (smem > configured[0]) {
      OI_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured[0] = smem;
    }
    cfg.attrs = nullptr;
    cfg.numAttrs = 0;
    OI_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kernel, (TOut*)out, ldc, (const bf16*)x, ldx, (const bf16*)W, ldw, M, N, K, k_slice));
  }
  return OI_OK;
}

}  // namespace

// silu_mul != 0: x is a fused [M, 2K] gate|up buffer and the activation silu(gate) * up is formed
// on the fly. cluster_size in {1, 2, 4, 8}: the number of K slices (CTAs per cluster).
OI_API int oi_gemm_skinny(void* out, int out_dtype, long long ldc, const void* x, long long ldx, const void* W,
                          long long ldw, int M, int N, int K, int silu_mul, int cluster_size, void* stream) {
  OI_REQUIRE(M >= 1 && M <= 16, "gemm_skinny: M=%d outside 1..16", M);
  OI_REQUIRE(N >= 1 && K >= 32, "gemm_skinny: bad sizes N=%d K=%d", N, K);
  OI_REQUIRE(cluster_size == 1 || cluster_size == 2 || cluster_size == 4 || cluster_size == 8,
             "gemm_skinny: cluster size %d", cluster_size);
  OI_REQUIRE(K % (32 * cluster_size) == 0, "gemm_skinny: K=%d is not a multiple of 32 * %d", K, cluster_size);
  OI_REQUIRE(ldx % 8 == 0 && ldw % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)W % 16 == 0,
             "gemm_skinny: operands must be 16-byte aligned with row strides that are multiples of 8");
  const int NT = M <= 8 ? 1 : 2;
  const size_t smem = (size_t)8 * NT * row_stride_elems(K / cluster_size) * sizeof(bf16) + (size_t)8 * NT * kRowsPerCta * sizeof(float);
  OI_REQUIRE(smem <= 200 * 1024, "gemm_skinny: K slice %d needs %zu bytes of shared memory", K / cluster_size, smem);
  cudaStream_t s = (cudaStream_t)stream;
#define OI_SKINNY(NT_, T_, S_) return launch<NT_, T_, S_>(out, ldc, x, ldx, W, ldw, M, N, K, cluster_size, s)
  if (out_dtype == OI_BF16) {
    if (NT == 1) { if (silu_mul) OI_SKINNY(1, bf16, true); else OI_SKINNY(1, bf16, false); }
    else         { if (silu_mul) OI_SKINNY(2, bf16, true); else OI_SKINNY(2, bf16, false); }
  } else if (out_dtype == OI_F32) {
    if (NT == 1) { if (silu_mul) OI_SKINNY(1, float, true); else OI_SKINNY(1, float, false); }
    else         { if (silu_mul) OI_SKINNY(2, float, true); else OI_SKINNY(2, float, false); }
  }
#undef OI_SKINNY
  OI_REQUIRE(false, "gemm_skinny: unknown output dtype code %d", out_dtype);
}
