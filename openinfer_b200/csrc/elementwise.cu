// Embedding gather, RMSNorm (with fused residual add or row gather), SiLU*mul.
//
// What each computes follows the reference's ops (embedding:
// pegainfer-kernels/csrc/shared/elementwise.cu:368-384; RMSNorm and fused add+RMSNorm:
// csrc/shared/flashinfer_norm.cu:39-132, 204-210; SiLU*mul: elementwise.cu:259-273), with all
// arithmetic in float32 and ONE rounding to the storage type at the output.
#include "common.cuh"

// ---------------------------------------------------------------------------
// embedding: out[t, :] = table[ids[t], :]
// ---------------------------------------------------------------------------
template <typename TO, typename TW>
__global__ void embedding_kernel(TO* __restrict__ out, const TW* __restrict__ table,
                                 const int* __restrict__ ids, int hidden, int vocab) {
  pdl_start();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // the host validates ids; never read outside
  const TW* src = table + (size_t)id * hidden;
  TO* dst = out + (size_t)t * hidden;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) dst[d] = from_f32<TO>(to_f32(src[d]));
}

// same element type on both sides and rows that are whole 16-byte vectors: a plain copy
__global__ void embedding_vec_kernel(uint4* __restrict__ out, const uint4* __restrict__ table,
                                     const int* __restrict__ ids, int vecs_per_row, int vocab) {
  pdl_start();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const uint4* src = table + (size_t)id * vecs_per_row;
  uint4* dst = out + (size_t)t * vecs_per_row;
  for (int d = threadIdx.x; d < vecs_per_row; d += blockDim.x) dst[d] = src[d];
}

OI_API int oi_embedding(void* out, int out_dtype, const void* table, int table_dtype,
                        const int* ids, int tokens, int hidden, int vocab, void* stream) {
  OI_REQUIRE(tokens >= 0 && hidden > 0 && vocab > 0, "embedding: bad sizes tokens=%d hidden=%d vocab=%d",
             tokens, hidden, vocab);
  if (tokens == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t esize = out_dtype == OI_F32 ? 4 : 2;
  if (out_dtype == table_dtype && (hidden * esize) % 16 == 0 &&
      ((uintptr_t)out % 16 == 0) && ((uintptr_t)table % 16 == 0)) {
    const int vecs = (int)(hidden * esize / 16);
    oi_launch(embedding_vec_kernel, tokens, vecs < 256 ? ((vecs + 31) / 32) * 32 : 256, 0, s, 
        (uint4*)out, (const uint4*)table, ids, vecs, vocab);
  } else if (out_dtype == OI_F32 && table_dtype == OI_F32) {
    oi_launch(embedding_kernel<float, float>, tokens, 256, 0, s, (float*)out, (const float*)table, ids, hidden, vocab);
  } else if (out_dtype == OI_BF16 && table_dtype == OI_BF16) {
    oi_launch(embedding_kernel<bf16, bf16>, tokens, 256, 0, s, (bf16*)out, (const bf16*)table, ids, hidden, vocab);
  } else if (out_dtype == OI_F32 && table_dtype == OI_BF16) {
    oi_launch(embedding_kernel<float, bf16>, tokens, 256, 0, s, (float*)out, (const bf16*)table, ids, hidden, vocab);
  } else if (out_dtype == OI_BF16 && table_dtype == OI_F32) {
    oi_launch(embedding_kernel<bf16, float>, tokens, 256, 0, s, (bf16*)out, (const float*)table, ids, hidden, vocab);
  } else {
    OI_REQUIRE(false, "embedding: unknown dtype codes %d/%d", out_dtype, table_dtype);
  }
  OI_CHECK_LAUNCH();
  return OI_OK;
}

// ids[i] = from[src[i]] where src[i] >= 0: token ids that the previous step drew and the host has not
// seen yet (indices outside `from` leave the id alone; the host checks them before the launch).
__global__ void gather_tokens_kernel(int* __restrict__ ids, const int* __restrict__ src, const int* __restrict__ from,
                                     int n, int n_from) {
  pdl_wait();   // no early trigger: see copy_words_kernel
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int j = src[i];
  if (j >= 0 && j < n_from) ids[i] = from[j];
}

OI_API int oi_gather_tokens(int* ids, const int* src, const int* from, int n, int n_from, void* stream) {
  OI_REQUIRE(n >= 0 && n_from >= 0, "gather_tokens: bad sizes");
  if (n == 0) return OI_OK;
  oi_launch(gather_tokens_kernel, (n + 127) / 128, 128, 0, (cudaStream_t)stream, ids, src, from, n, n_from);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

// dst[i] = src[i] for a few thousand 32-bit words, by a kernel: `src` or `dst` may be PINNED HOST memory
// (which the device reads and writes directly), so that a step's metadata reaches the device, and its
// drawn tokens the host, in the stream's kernel order without a copy-engine operation in between. With
// ids_off >= 0 the words [ids_off, ids_off + n_ids) are token ids, and those whose source index
// (the words at src_off) is >= 0 are taken from `from` instead (see oi_gather_tokens).
__global__ void copy_words_kernel(int* __restrict__ dst, const int* __restrict__ src, int n, int ids_off, int src_off,
                                  int n_ids, const int* __restrict__ from, int n_from) {
  // No early trigger here: what this kernel writes (a step's lengths, block tables, positions) is read by
  // later kernels BEFORE their own wait, so nothing after it may start until it has finished. It is the
  // fence between two steps: whoever copies such data asks for the kernel launched next to be launched without
  // the programmatic attribute (oi_launch_fence), so that it starts only when this one has completed and its
  // writes are visible.
  pdl_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    int v = src[i];
    if (ids_off >= 0 && i >= ids_off && i < ids_off + n_ids) {
      const int j = src[src_off + (i - ids_off)];
      if (j >= 0 && j < n_from) v = from[j];
    }
    dst[i] = v;
  }
}

OI_API int oi_copy_words(int* dst, const int* src, int n, int ids_off, int src_off, int n_ids, const int* from, int n_from,
                         void* stream) {
  OI_REQUIRE(n >= 0 && (ids_off < 0 || (src_off >= 0 && n_ids >= 0 && ids_off + n_ids <= n && src_off + n_ids <= n)),
             "copy_words: bad sizes");
  OI_REQUIRE(ids_off < 0 || n_from == 0 || from != nullptr, "copy_words: token source missing");
  if (n == 0) return OI_OK;
  const int blocks = (n + 255) / 256 > 64 ? 64 : (n + 255) / 256;
  oi_launch(copy_words_kernel, blocks, 256, 0, (cudaStream_t)stream, dst, src, n, ids_off, src_off, n_ids, from, n_from);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

// ---------------------------------------------------------------------------
// ---------------------------------------------------------------------------
// RMSNorm. One block per output row.
//   delta != null : x[row] <- round(x[row] + delta[row]) first (the residual sum, stored), and the
//                   norm is taken of the ROUNDED sum (flashinfer_norm.cu:76-83, 107-124).
//   row_idx != null : output row r reads x[row_idx[r]] (+ delta[row_idx[r]], not stored): the rows
//                   whose logits are wanted.
//   out[r] = round( x * rsqrt(mean(x^2) + eps) * (w_offset + w) )
template <typename T, bool kCache>
__global__ void rmsnorm_kernel(T* __restrict__ out, T* __restrict__ x, const T* __restrict__ delta,
                               const void* __restrict__ w, int w_dtype, const int* __restrict__ row_idx,
                               int hidden, float eps, float w_offset) {
  pdl_start();
  extern __shared__ float row_cache[];
  __shared__ float red[32];
  const int r = blockIdx.x;
  const size_t src = row_idx ? (size_t)row_idx[r] : (size_t)r;
  T* xr = x + src * hidden;
  const T* dr = delta ? delta + src * hidden : nullptr;
  float ss = 0.f;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    float v = to_f32(xr[d]);
    if (dr) {
      v = to_f32(from_f32<T>(v + to_f32(dr[d])));
      if (!row_idx) xr[d] = from_f32<T>(v);  // gathered rows may repeat: the sum is not stored
    }
    if (kCache) row_cache[d] = v;
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  T* orow = out + (size_t)r * hidden;
  for (int d = threadIdx.x; d < hidden; d += blockDim.x) {
    float v;
    if (kCache) v = row_cache[d];
    else if (dr && row_idx) v = to_f32(from_f32<T>(to_f32(xr[d]) + to_f32(dr[d])));
    else v = to_f32(xr[d]);
    orow[d] = from_f32<T>(v * inv * (w_offset + load_as_f32(w, w_dtype, d)));
  }
}

// bfloat16 rows whose length is a multiple of 8 and a bfloat16 weight: every thread moves whole
// 16-byte vectors, all loads (row, residual, weight) are issued before anything waits on them.
template <int VPT>
__global__ void rmsnorm_bf16_vec_kernel(bf16* __restrict__ out, bf16* __restrict__ x, const bf16* __restrict__ delta,
                                        const bf16* __restrict__ w, const int* __restrict__ row_idx, int hidden,
                                        float eps, float w_offset) {
  pdl_trigger();
  __shared__ float red[32];
  const int r = blockIdx.x;
  const int nvec = hidden / 8;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4 xv[VPT], dv[VPT], wv[VPT];
  // the norm weight does not depend on the kernels ahead on the stream: fetched before waiting for them
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * blockDim.x;
    if (v < nvec) wv[k] = wr[v];
  }
  pdl_wait();
  const size_t src = row_idx ? (size_t)row_idx[r] : (size_t)r;
  uint4* xr = reinterpret_cast<uint4*>(x + src * hidden);
  const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + src * hidden) : nullptr;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * blockDim.x;
    if (v < nvec) {
      xv[k] = xr[v];
      if (dr) dv[k] = dr[v];
    }
  }
  float vals[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * blockDim.x;
    if (v < nvec) {
      const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv[k]);
      const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dv[k]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = __bfloat1622float2(x2[e]);
        if (dr) {
          const float2 d = __bfloat1622float2(d2[e]);
          const __nv_bfloat162 rounded = __floats2bfloat162_rn(f.x + d.x, f.y + d.y);
          reinterpret_cast<__nv_bfloat162*>(&xv[k])[e] = rounded;
          f = __bfloat1622float2(rounded);
        }
        vals[k][2 * e] = f.x;
        vals[k][2 * e + 1] = f.y;
        ss += f.x * f.x + f.y * f.y;
      }
      if (dr && !row_idx) xr[v] = xv[k];   // the residual sum is stored (gathered rows may repeat: not stored)
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  uint4* orow = reinterpret_cast<uint4*>(out + (size_t)r * hidden);
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * blockDim.x;
    if (v < nvec) {
      const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv[k]);
      uint4 ov;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 wf = __bfloat1622float2(w2[e]);
        o2[e] = __floats2bfloat162_rn(vals[k][2 * e] * inv * (w_offset + wf.x), vals[k][2 * e + 1] * inv * (w_offset + wf.y));
      }
      orow[v] = ov;
    }
  }
}

static int launch_rmsnorm_bf16_vec(void* out, void* x, const void* delta, const void* w, const int* row_idx, int rows,
                                   int hidden, float eps, float w_offset, cudaStream_t s) {
  const int nvec = hidden / 8;
  int threads = ((nvec + 31) / 32) * 32;
  int vpt = 1;
  while (threads > 1024) {
    vpt *= 2;
    threads = (((nvec + vpt - 1) / vpt + 31) / 32) * 32;
  }
#define OI_NORM_VEC(V)                                                                                       \
  oi_launch(rmsnorm_bf16_vec_kernel<V>, rows, threads, 0, s, (bf16*)out, (bf16*)x, (const bf16*)delta, (const bf16*)w, \
                                                      row_idx, hidden, eps, w_offset)
  if (vpt == 1) OI_NORM_VEC(1);
  else if (vpt == 2) OI_NORM_VEC(2);
  else OI_NORM_VEC(4);
#undef OI_NORM_VEC
  OI_CHECK_LAUNCH();
  return OI_OK;
}

template <typename T>
static int launch_rmsnorm(void* out, void* x, const void* delta, const void* w, int w_dtype,
                          const int* row_idx, int rows, int hidden, float eps, float w_offset,
                          cudaStream_t s) {
  int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem <= 48 * 1024) {
    oi_launch(rmsnorm_kernel<T, true>, rows, threads, smem, s, (T*)out, (T*)x, (const T*)delta, w, w_dtype,
                                                        row_idx, hidden, eps, w_offset);
  } else {
    oi_launch(rmsnorm_kernel<T, false>, rows, threads, 0, s, (T*)out, (T*)x, (const T*)delta, w, w_dtype,
                                                      row_idx, hidden, eps, w_offset);
  }
  OI_CHECK_LAUNCH();
  return OI_OK;
}

OI_API int oi_rmsnorm(void* out, void* x, const void* delta, int dtype, const void* w, int w_dtype,
                      const int* row_idx, int rows, int hidden, float eps, float w_offset,
                      void* stream) {
  OI_REQUIRE(rows >= 0 && hidden > 0, "rmsnorm: bad sizes rows=%d hidden=%d", rows, hidden);
  OI_REQUIRE(!(delta && out == x), "rmsnorm: with a residual add, out must not alias x");
  if (rows == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == OI_F32) return launch_rmsnorm<float>(out, x, delta, w, w_dtype, row_idx, rows, hidden, eps, w_offset, s);
  if (dtype == OI_BF16) {
    const bool aligned = ((uintptr_t)out % 16 == 0) && ((uintptr_t)x % 16 == 0) && ((uintptr_t)w % 16 == 0) &&
                         (!delta || (uintptr_t)delta % 16 == 0);
    if (w_dtype == OI_BF16 && hidden % 8 == 0 && hidden <= 32768 && aligned)
      return launch_rmsnorm_bf16_vec(out, x, delta, w, row_idx, rows, hidden, eps, w_offset, s);
    return launch_rmsnorm<bf16>(out, x, delta, w, w_dtype, row_idx, rows, hidden, eps, w_offset, s);
  }
  OI_REQUIRE(false, "rmsnorm: unknown dtype code %d", dtype);
}

// ---------------------------------------------------------------------------
// residual add without a norm: x <- round(x + delta)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void add_inplace_kernel(T* __restrict__ x, const T* __restrict__ delta, size_t n) {
  pdl_start();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] = from_f32<T>(to_f32(x[i]) + to_f32(delta[i]));
}

OI_API int oi_add_inplace(void* x, const void* delta, int dtype, long long n, void* stream) {
  OI_REQUIRE(n >= 0, "add: bad size %lld", n);
  if (n == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
  if (dtype == OI_F32) oi_launch(add_inplace_kernel<float>, blocks, 256, 0, s, (float*)x, (const float*)delta, (size_t)n);
  else if (dtype == OI_BF16) oi_launch(add_inplace_kernel<bf16>, blocks, 256, 0, s, (bf16*)x, (const bf16*)delta, (size_t)n);
  else OI_REQUIRE(false, "add: unknown dtype code %d", dtype);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

// ---------------------------------------------------------------------------
// x = x * scale, then (cap > 0) x = cap * tanh(x / cap): an embedding scale, or the soft cap of logits.
// float32 math, one rounding.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void scale_cap_kernel(T* __restrict__ x, size_t n, float scale, float cap) {
  pdl_start();
  const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float v = to_f32(x[i]) * scale;
    if (cap > 0.f) v = cap * tanhf(v * inv_cap);
    x[i] = from_f32<T>(v);
  }
}

OI_API int oi_scale_cap(void* x, int dtype, long long n, float scale, float cap, void* stream) {
  OI_REQUIRE(n >= 0 && cap >= 0.f, "scale_cap: bad size %lld or cap %f", n, (double)cap);
  if (n == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
  if (dtype == OI_F32) oi_launch(scale_cap_kernel<float>, blocks, 256, 0, s, (float*)x, (size_t)n, scale, cap);
  else if (dtype == OI_BF16) oi_launch(scale_cap_kernel<bf16>, blocks, 256, 0, s, (bf16*)x, (size_t)n, scale, cap);
  else OI_REQUIRE(false, "scale_cap: unknown dtype code %d", dtype);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

// ---------------------------------------------------------------------------
// act * mul on a fused [rows, 2*inter] gate|up buffer: out[r, i] = act(g_i) * u_i, act = SiLU or tanh-GELU.
// Layout of a row: blocks of `block` gate values followed by the `block` up values of the same
// indices; block == inter is the plain [all gates | all ups] layout. (A product kernel whose tile
// holds a gate block and its up block side by side can form the activation in its epilogue.)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter, int block, size_t n, int act) {
  pdl_start();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / inter, c = i - r * inter;
    const size_t gi = r * 2 * inter + (c / block) * 2 * block + (c % block);
    const float g = to_f32(gate_up[gi]);
    const float u = to_f32(gate_up[gi + block]);
    out[i] = from_f32<T>(gate_act<false>(g, act) * u);
  }
}

// 8 bf16 per thread when inter and block are multiples of 8
__global__ void silu_mul_bf16x8_kernel(uint4* __restrict__ out, const uint4* __restrict__ gate_up,
                                       int inter8, int block8, size_t n8, int act) {
  pdl_start();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / inter8, c = i - r * inter8;
    const size_t gi = r * 2 * inter8 + (c / block8) * 2 * block8 + (c % block8);
    uint4 gv = gate_up[gi];
    uint4 uv = gate_up[gi + block8];
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = __bfloat1622float2(g2[k]);
      const float2 u = __bfloat1622float2(u2[k]);
      o2[k] = __floats2bfloat162_rn(gate_act<false>(g.x, act) * u.x, gate_act<false>(g.y, act) * u.y);
    }
    out[i] = ov;
  }
}

OI_API int oi_silu_mul(void* out, const void* gate_up, int dtype, int rows, int inter, int block, int act, void* stream) {
  OI_REQUIRE(act == OI_ACT_SILU || act == OI_ACT_GELU_TANH, "silu_mul: unknown activation code %d", act);
  OI_REQUIRE(rows >= 0 && inter > 0, "silu_mul: bad sizes rows=%d inter=%d", rows, inter);
  OI_REQUIRE(block > 0 && inter % block == 0, "silu_mul: block %d does not divide inter %d", block, inter);
  if (rows == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t n = (size_t)rows * inter;
  if (dtype == OI_BF16 && inter % 8 == 0 && block % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)gate_up % 16 == 0) {
    const size_t n8 = n / 8;
    const int blocks = (int)((n8 + 255) / 256 > 148 * 16 ? 148 * 16 : (n8 + 255) / 256);
    oi_launch(silu_mul_bf16x8_kernel, blocks, 256, 0, s, (uint4*)out, (const uint4*)gate_up, inter / 8, block / 8, n8, act);
  } else {
    const int blocks = (int)((n + 255) / 256 > 148 * 16 ? 148 * 16 : (n + 255) / 256);
    if (dtype == OI_F32) oi_launch(silu_mul_kernel<float>, blocks, 256, 0, s, (float*)out, (const float*)gate_up, inter, block, n, act);
    else if (dtype == OI_BF16) oi_launch(silu_mul_kernel<bf16>, blocks, 256, 0, s, (bf16*)out, (const bf16*)gate_up, inter, block, n, act);
    else OI_REQUIRE(false, "silu_mul: unknown dtype code %d", dtype);
  }
  OI_CHECK_LAUNCH();
  return OI_OK;
}
