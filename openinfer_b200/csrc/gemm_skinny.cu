// Skinny product for decode: out[M, N] = x[M, K] * W[N, K]^T with M <= 16 rows of activations,
// bfloat16 operands, float32 accumulation. The step is bound by streaming W from HBM once, so the
// kernel is built around memory parallelism, not tensor throughput:
//
//  * a CTA (4 warps) owns 64 rows of W and one slice of K; the CTAs of a thread-block CLUSTER own
//    the slices of the same rows and add their partial sums through distributed shared memory in
//    rank order (deterministic, no atomics, no scratch in global memory);
//  * each warp streams its 16 rows through a private ring in shared memory filled by 16-byte
//    cp.async copies, five stages (10 KB) in flight per warp and no barrier (a lane reads back what
//    it copied itself), and feeds mma.sync m16n8k16 with W as the A operand and the activations
//    (staged once per CTA in shared memory) as B. The k index inside a 32-wide block is permuted
//    identically for both operands (a dot product does not care), so a lane's 16 contiguous
//    bytes ARE its fragment registers;
//  * the ring is primed before the kernel waits for its predecessor on the stream (programmatic
//    dependent launch), so weights stream in under the tail of the kernel that produces x;
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

constexpr int kWarps = 4;
constexpr int kRowsPerCta = kWarps * 16;
constexpr int kU = 2;          // 32-wide k blocks per ring stage
constexpr int kStages = 6;     // ring depth per warp: five stages (10 KB) in flight per warp

// Token rows in shared memory are padded so that the row stride is 4 (mod 8) 16-byte chunks: the
// eight lanes that a 128-bit shared load serves at once (two tokens x four chunks) then hit
// eight different bank groups.
__host__ __device__ constexpr int row_stride_elems(int k_slice) {
  return k_slice + (((k_slice / 8) % 8 == 0) ? 32 : 64);
}
__host__ __device__ constexpr size_t ring_bytes() { return (size_t)kWarps * kStages * kU * 2 * 32 * 16; }

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(unsigned dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // src-size 0: zero fill
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ uint4 lds128(unsigned addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// NT: token tiles of 8 (M <= 8 * NT). kCluster: CTAs along K add up through distributed shared memory.
// The weight ring is primed BEFORE waiting for the kernel that produces x (programmatic dependent
// launch), so the first 40 KB of W per CTA stream in under its tail.
template <int NT, typename TOut, bool kSiluMul, bool kCluster>
__global__ void __launch_bounds__(kWarps * 32)
gemm_skinny_kernel(TOut* __restrict__ out, long long ldc, const bf16* __restrict__ x, long long ldx,
                   const bf16* __restrict__ W, long long ldw, int M, int N, int K, int k_slice, int act_block, int act) {
  pdl_trigger();
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int stride = row_stride_elems(k_slice);                 // elements per token row
  unsigned char* ring_raw = smem_raw;                           // [warp][stage][u][row a | row b][lane] 16 B
  bf16* x_s = reinterpret_cast<bf16*>(smem_raw + ring_bytes()); // [8 * NT][stride]
  float* part = reinterpret_cast<float*>(smem_raw + ring_bytes() + (size_t)8 * NT * stride * sizeof(bf16));  // [8 * NT][64]

  const int rank = blockIdx.x;                                  // slice of K == rank in the cluster
  const int k0 = rank * k_slice;
  const int n0 = blockIdx.y * kRowsPerCta;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // ---- the weight stream: lane (g, c) owns 8 consecutive k of rows g and g + 8 in every 32-wide block
  const int g = lane >> 2, c = lane & 3;
  const int row_a = min(n0 + warp * 16 + g, N - 1), row_b = min(n0 + warp * 16 + g + 8, N - 1);
  const bf16* pa = W + (size_t)row_a * ldw + k0 + c * 8;
  const bf16* pb = W + (size_t)row_b * ldw + k0 + c * 8;
  const unsigned my_ring = (unsigned)__cvta_generic_to_shared(ring_raw) + (unsigned)(warp * kStages * kU * 2 * 32 + lane) * 16u;
  const int nkb = k_slice / 32;
  const int n_it = (nkb + kU - 1) / kU;
  // the stream is issued through running pointers: no multiplication or division per stage
  int ld_it = 0, ld_slot = 0;
  const bf16* ld_a = pa;
  const bf16* ld_b = pb;
  const bool even = (nkb % kU) == 0;   // every stage holds kU whole blocks
  auto issue = [&]() {   // the next stage of the stream into its ring slot; one commit per call
    if (ld_it < n_it) {
      const unsigned dst = my_ring + (unsigned)(ld_slot * kU * 2 * 32) * 16u;
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const bool valid = even || ld_it * kU + u < nkb;   // past the end: zero fill
        cp_async16(dst + (unsigned)(u * 2 * 32) * 16u, valid ? ld_a + u * 32 : W, valid);
        cp_async16(dst + (unsigned)((u * 2 + 1) * 32) * 16u, valid ? ld_b + u * 32 : W, valid);
      }
      ld_a += kU * 32;
      ld_b += kU * 32;
      ++ld_it;
      ld_slot = ld_slot + 1 == kStages ? 0 : ld_slot + 1;
    }
    cp_async_commit();
  };
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) issue();

  // ---- stage the activation slice (rows >= M are zero); x is the previous kernel's output
  pdl_wait();
  {
    const int vec_per_row = k_slice / 8;
    for (int i = tid; i < 8 * NT * vec_per_row; i += kWarps * 32) {
      const int m = i / vec_per_row, v = i - m * vec_per_row;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (m < M) {
        if (kSiluMul) {
          const int k = k0 + v * 8;   // gate block b, then up block b: see oi_silu_mul
          const size_t gi = (size_t)m * ldx + (size_t)(k / act_block) * 2 * act_block + (k % act_block);
          const uint4 gv = *reinterpret_cast<const uint4*>(x + gi);
          const uint4 uv = *reinterpret_cast<const uint4*>(x + gi + act_block);
          const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
          const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
          __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&val);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 gg = __bfloat1622float2(g2[e]), u = __bfloat1622float2(u2[e]);
            o2[e] = __floats2bfloat162_rn(gate_act<false>(gg.x, act) * u.x, gate_act<false>(gg.y, act) * u.y);
          }
        } else {
          val = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + k0 + v * 8);
        }
      }
      *reinterpret_cast<uint4*>(x_s + (size_t)m * stride + v * 8) = val;
    }
  }
  __syncthreads();

  const unsigned xs = (unsigned)__cvta_generic_to_shared(x_s) + (unsigned)(g * stride + c * 8) * 2u;
  float acc[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;

  int slot = 0;
  unsigned xk = xs;                     // this lane's activation chunk of the current k block
  for (int it = 0; it < n_it; ++it) {
    issue();                            // refills the slot consumed in the previous iteration
    cp_async_wait<kStages - 1>();       // stage `it` (this lane's own copies) has landed
    const unsigned src = my_ring + (unsigned)(slot * kU * 2 * 32) * 16u;
    slot = slot + 1 == kStages ? 0 : slot + 1;
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const uint4 wa = lds128(src + (unsigned)(u * 2 * 32) * 16u);
      const uint4 wb = lds128(src + (unsigned)((u * 2 + 1) * 32) * 16u);
      const int kb = it * kU + u;
      if (kb >= nkb) break;   // the zero-filled tail of the last stage: nothing to add (and x_s ends here)
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const uint4 xv = lds128(xk + (unsigned)(t * 8 * stride) * 2u);
        mma_bf16(acc[t], wa.x, wb.x, wa.y, wb.y, xv.x, xv.y);
        mma_bf16(acc[t], wa.z, wb.z, wa.w, wb.w, xv.z, xv.w);
      }
      xk += 64u;                        // 32 elements further along k
    }
  }
  cp_async_wait<0>();

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
    // rank r adds up rows [r * 64 / csize, (r + 1) * 64 / csize) over all slices, in rank order
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

size_t smem_bytes(int NT, int k_slice) {
  return ring_bytes() + (size_t)8 * NT * row_stride_elems(k_slice) * sizeof(bf16) + (size_t)8 * NT * kRowsPerCta * sizeof(float);
}

template <int NT, typename TOut, bool kSiluMul>
int launch(void* out, long long ldc, const void* x, long long ldx, const void* W, long long ldw, int M, int N,
           int K, int csize, int act_block, int act, cudaStream_t s) {
  const int k_slice = K / csize;
  const size_t smem = smem_bytes(NT, k_slice);
  static size_t configured[2] = {0, 0};   // largest dynamic shared memory set so far, per kernel variant
  const int row_tiles = (N + kRowsPerCta - 1) / kRowsPerCta;
  const dim3 grid(csize, row_tiles, 1);
  if (csize > 1) {
    auto kernel = gemm_skinny_kernel<NT, TOut, kSiluMul, true>;
    if (smem > configured[1]) {
      OI_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured[1] = smem;
    }
    oi_launch_cluster(kernel, grid, kWarps * 32, smem, s, csize, (TOut*)out, ldc, (const bf16*)x, ldx, (const bf16*)W, ldw, M, N, K,
                      k_slice, act_block, act);
  } else {
    auto kernel = gemm_skinny_kernel<NT, TOut, kSiluMul, false>;
    if (smem > configured[0]) {
      OI_CHECK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      configured[0] = smem;
    }
    oi_launch(kernel, grid, kWarps * 32, smem, s, (TOut*)out, ldc, (const bf16*)x, ldx, (const bf16*)W, ldw, M, N, K, k_slice, act_block, act);
  }
  OI_CHECK_LAUNCH();
  return OI_OK;
}

}  // namespace

// silu_mul != 0: x is a fused [M, 2K] gate|up buffer laid out in blocks of `silu_mul` gate values
// followed by their up values (silu_mul == K: all gates, then all ups) and the activation
// act(gate) * up (act: OI_ACT_SILU or OI_ACT_GELU_TANH) is formed on the fly. cluster_size in {1, 2, 4, 8}: the number of K slices (CTAs per cluster).
OI_API int oi_gemm_skinny(void* out, int out_dtype, long long ldc, const void* x, long long ldx, const void* W,
                          long long ldw, int M, int N, int K, int silu_mul, int act, int cluster_size, void* stream) {
  OI_REQUIRE(silu_mul == 0 || act == OI_ACT_SILU || act == OI_ACT_GELU_TANH, "gemm_skinny: unknown activation code %d", act);
  OI_REQUIRE(M >= 1 && M <= 16, "gemm_skinny: M=%d outside 1..16", M);
  OI_REQUIRE(N >= 1 && K >= 32, "gemm_skinny: bad sizes N=%d K=%d", N, K);
  OI_REQUIRE(cluster_size == 1 || cluster_size == 2 || cluster_size == 4 || cluster_size == 8,
             "gemm_skinny: cluster size %d", cluster_size);
  OI_REQUIRE(K % (32 * cluster_size) == 0, "gemm_skinny: K=%d is not a multiple of 32 * %d", K, cluster_size);
  OI_REQUIRE(silu_mul == 0 || (silu_mul % 8 == 0 && K % silu_mul == 0), "gemm_skinny: activation block %d does not fit K=%d", silu_mul, K);
  OI_REQUIRE(ldx % 8 == 0 && ldw % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)W % 16 == 0,
             "gemm_skinny: operands must be 16-byte aligned with row strides that are multiples of 8");
  const int NT = M <= 8 ? 1 : 2;
  const size_t smem = smem_bytes(NT, K / cluster_size);
  OI_REQUIRE(smem <= 200 * 1024, "gemm_skinny: K slice %d needs %zu bytes of shared memory", K / cluster_size, smem);
  cudaStream_t s = (cudaStream_t)stream;
#define OI_SKINNY(NT_, T_, S_) return launch<NT_, T_, S_>(out, ldc, x, ldx, W, ldw, M, N, K, cluster_size, silu_mul, act, s)
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
