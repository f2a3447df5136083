// Paged causal attention, general form: any head_dim that is a multiple of 8 (up to 256), any
// number of heads and groups, an optional window, float32 or bfloat16 storage; prompt portions
// and single decoded tokens alike. One warp per (token, query head).
//
// s[i,j] = (q_i . k_j) * scale for j <= pos_i (and j > pos_i - window), online softmax in float32,
// o_i = sum_j p[i,j] v_j; query head h reads kv head h / (nq / nkv)
// (pegainfer-kernels/csrc/shared/paged_attention.cu:439-567; pegainfer-kernels/src/ops/attention.rs:507).
// The keys of a request are visited in position order, 32 at a time, whatever else is in the
// batch, so a row's result does not depend on how the batch was cut.
//
// This is the kernel of the true 32-bit path and of every shape the tuned kernels refuse.
#include "common.cuh"

#define ATTN_MAX_HD 256

template <typename T>
struct Vec16;  // 16 bytes of T
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* out) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  }
};
template <>
struct Vec16<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const bf16* p, float* out) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      out[2 * k] = f.x; out[2 * k + 1] = f.y;
    }
  }
};

template <typename T, int kWarps>
__global__ void attention_generic_kernel(
    const T* __restrict__ q, int q_row_stride, T* __restrict__ out, int out_row_stride,
    const T* __restrict__ k_cache, const T* __restrict__ v_cache, long long page_stride, int page_size,
    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ token_req,
    const int* __restrict__ positions, int nq, int nkv, int hd, float scale, int window, int tokens) {
  pdl_start();
  __shared__ float q_sh[kWarps][ATTN_MAX_HD];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int token = blockIdx.x;
  const int head = blockIdx.y * kWarps + warp;
  if (head >= nq) return;  // whole warp leaves; no block-wide barrier below
  const int req = token_req[token];
  if (req < 0) return;     // padding row
  const int pos = positions[token];
  const int kvh = head / (nq / nkv);
  const int* bt = block_table + (size_t)req * bt_stride;

  const T* qp = q + (size_t)token * q_row_stride + (size_t)head * hd;
  for (int d = lane; d < hd; d += 32) q_sh[warp][d] = to_f32(qp[d]);
  __syncwarp();

  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const size_t row_elems = (size_t)nkv * hd;
  constexpr int VN = Vec16<T>::N;
  constexpr int kAccs = ATTN_MAX_HD / 32;
  float acc[kAccs];
#pragma unroll
  for (int r = 0; r < kAccs; ++r) acc[r] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int base = first; base <= pos; base += 32) {
    const int j = base + lane;
    float s = -INFINITY;
    if (j <= pos) {
      const int page = bt[j / page_size];
      const T* kp = k_cache + (size_t)page * page_stride + (size_t)(j % page_size) * row_elems + (size_t)kvh * hd;
      float dot = 0.f;
      for (int d = 0; d < hd; d += VN) {
        float kv[VN];
        Vec16<T>::load(kp + d, kv);
#pragma unroll
        for (int e = 0; e < VN; ++e) dot += q_sh[warp][d + e] * kv[e];
      }
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = (j <= pos) ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);  // m = -inf on the first tile gives 0
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int r = 0; r < kAccs; ++r) acc[r] *= corr;
    const int n_valid = min(32, pos - base + 1);
    for (int jj = 0; jj < n_valid; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int jv = base + jj;
      const int page = bt[jv / page_size];
      const T* vp = v_cache + (size_t)page * page_stride + (size_t)(jv % page_size) * row_elems + (size_t)kvh * hd;
#pragma unroll
      for (int r = 0; r < kAccs; ++r) {
        const int d = lane + 32 * r;
        if (d < hd) acc[r] += pj * to_f32(vp[d]);
      }
    }
    m = m_new;
  }
  T* op = out + (size_t)token * out_row_stride + (size_t)head * hd;
  const float inv_l = 1.f / l;
#pragma unroll
  for (int r = 0; r < kAccs; ++r) {
    const int d = lane + 32 * r;
    if (d < hd) op[d] = from_f32<T>(acc[r] * inv_l);
  }
}

OI_API int oi_attention_generic(const void* q, int q_row_stride, void* out, int out_row_stride, int dtype,
                                const void* k_cache, const void* v_cache, long long page_stride,
                                int page_size, const int* block_table, int bt_stride,
                                const int* token_req, const int* positions, int tokens, int nq, int nkv,
                                int hd, float scale, int window, void* stream) {
  OI_REQUIRE(tokens >= 0 && nq > 0 && nkv > 0 && nq % nkv == 0, "attention: bad head counts nq=%d nkv=%d", nq, nkv);
  OI_REQUIRE(hd > 0 && hd % 8 == 0 && hd <= ATTN_MAX_HD,
             "attention: head_dim %d unsupported (multiples of 8 up to %d)", hd, ATTN_MAX_HD);
  OI_REQUIRE(q_row_stride % 8 == 0 && page_stride % 8 == 0, "attention: strides must be multiples of 8 elements");
  OI_REQUIRE(page_size > 0, "attention: page_size %d", page_size);
  if (tokens == 0) return OI_OK;
  constexpr int kWarps = 4;
  dim3 grid(tokens, (nq + kWarps - 1) / kWarps);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == OI_F32) {
    oi_launch(attention_generic_kernel<float, kWarps>, grid, kWarps * 32, 0, s, 
        (const float*)q, q_row_stride, (float*)out, out_row_stride, (const float*)k_cache,
        (const float*)v_cache, page_stride, page_size, block_table, bt_stride, token_req, positions, nq,
        nkv, hd, scale, window, tokens);
  } else if (dtype == OI_BF16) {
    oi_launch(attention_generic_kernel<bf16, kWarps>, grid, kWarps * 32, 0, s, 
        (const bf16*)q, q_row_stride, (bf16*)out, out_row_stride, (const bf16*)k_cache,
        (const bf16*)v_cache, page_stride, page_size, block_table, bt_stride, token_req, positions, nq,
        nkv, hd, scale, window, tokens);
  } else {
    OI_REQUIRE(false, "attention: unknown dtype code %d", dtype);
  }
  OI_CHECK_LAUNCH();
  return OI_OK;
}
