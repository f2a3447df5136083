// Fused per-head q/k norm + position rotation + write of K and V into the paged cache. The rotation turns the
// pair (d, d + half) by angle d ("rotate half", the reference's) or, with `interleaved`, the neighbours (2 d, 2 d + 1);
// the tuned bfloat16 kernels below cover the first, the general kernel both.
//
// One warp per (token, head) over the fused projection output [tokens, (nq + 2*nkv) * hd]:
//   q heads: norm, rotate, written back in place (attention reads q from this buffer);
//   k heads: norm, rotate, written to the K page of (request, position);
//   v heads: copied to the V page.
// Formulas: per-head RMSNorm before the rotation with the layer's eps, v untouched
// (pegainfer-kernels/csrc/shared/prefill_attention.cu:84-99); rotate-half over the pair
// (d, d + half) (prefill_attention.cu:101-122); cache address page*page_stride + (pos % P)*nkv*hd
// + head*hd (pegainfer-kv-cache/src/layout.rs:5-33). The reference replaces three kernels' worth
// of traffic (norm+rope, then a separate scatter: csrc/shared/paged_attention.cu:309-348) — here
// K and V go from the projection output straight to their page. Arithmetic is float32 with one
// rounding at the store; cos/sin come from float32 tables [max_pos, rot_half].
#include "common.cuh"

template <typename T>
__global__ void qk_norm_rope_kv_kernel(
    T* __restrict__ qkv, int row_stride, int nq, int nkv, int hd,
    const void* __restrict__ q_norm_w, const void* __restrict__ k_norm_w, int norm_dtype, float eps,
    float w_offset, const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
    int rot_half, int max_pos, const int* __restrict__ positions, const int* __restrict__ slots,
    T* __restrict__ k_cache, T* __restrict__ v_cache, long long page_stride, int page_size,
    int heads_total, int tokens, int interleaved) {
  pdl_start();
  const int lane = threadIdx.x & 31;
  const long long gw = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gw >= (long long)tokens * heads_total) return;
  const int token = (int)(gw / heads_total);
  const int head = (int)(gw - (long long)token * heads_total);
  T* src = qkv + (size_t)token * row_stride + (size_t)head * hd;

  const int kind = head < nq ? 0 : (head < nq + nkv ? 1 : 2);
  T* dst = src;  // q: in place
  if (kind != 0) {
    const int slot = slots[token];
    if (slot < 0) return;  // a padding row: nothing to store
    const int kvh = kind == 1 ? head - nq : head - nq - nkv;
    T* base = kind == 1 ? k_cache : v_cache;
    dst = base + (size_t)(slot / page_size) * page_stride +
          (size_t)(slot % page_size) * nkv * hd + (size_t)kvh * hd;
  }
  if (kind == 2) {
    for (int d = lane; d < hd; d += 32) dst[d] = src[d];
    return;
  }
  const void* w = kind == 0 ? q_norm_w : k_norm_w;
  float inv = 1.f;
  if (w) {
    float ss = 0.f;
    for (int d = lane; d < hd; d += 32) {
      const float v = to_f32(src[d]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    inv = rsqrtf(ss / (float)hd + eps);
  }
  int pos = positions[token];
  pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);  // admission bounds positions
  for (int i = lane; i < rot_half; i += 32) {
    // the pair that angle i turns: (i, i + half) ("rotate half"), or the neighbours (2 i, 2 i + 1) when interleaved
    const int ia = interleaved ? 2 * i : i, ib = interleaved ? 2 * i + 1 : i + rot_half;
    float a = to_f32(src[ia]), b = to_f32(src[ib]);
    if (w) {
      a = a * inv * (w_offset + load_as_f32(w, norm_dtype, ia));
      b = b * inv * (w_offset + load_as_f32(w, norm_dtype, ib));
    }
    const float c = cos_tab[(size_t)pos * rot_half + i];
    const float s = sin_tab[(size_t)pos * rot_half + i];
    dst[ia] = from_f32<T>(a * c - b * s);
    dst[ib] = from_f32<T>(a * s + b * c);
  }
  for (int d = 2 * rot_half + lane; d < hd; d += 32) {  // dims beyond the rotary part
    float a = to_f32(src[d]);
    if (w) a = a * inv * (w_offset + load_as_f32(w, norm_dtype, d));
    dst[d] = from_f32<T>(a);
  }
}

// bfloat16 fast path: a lane handles PAIRS of neighbouring elements with 4-byte accesses (the
// element (2p, 2p+1) of the first rotary half together with its partner pair in the second half),
// so a head of 128 is two loads and two stores per lane. A warp walks over `heads_per_warp` heads of
// ONE token: the position, the cache slot, the cos/sin values and the norm weights of its lanes are
// fetched once and reused for every head.
template <typename TW, int kMax>   // TW: storage type of the norm weights; kMax: pair sets per lane (1: rotary_dim <= 128)
__global__ void qk_norm_rope_kv_bf16x2_kernel(
    bf16* __restrict__ qkv, int row_stride, int nq, int nkv, int hd,
    const TW* __restrict__ q_norm_w, const TW* __restrict__ k_norm_w, float eps,
    float w_offset, const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
    int rot_half, int max_pos, const int* __restrict__ positions, const int* __restrict__ slots,
    bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, long long page_stride, int page_size,
    int heads_total, int heads_per_warp) {
  pdl_start();
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x;
  const int head0 = (blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5)) * heads_per_warp;
  if (head0 >= heads_total) return;
  const int head1 = min(heads_total, head0 + heads_per_warp);
  const int npairs = hd / 2;
  const int rot_pairs = rot_half / 2;          // pairs in one rotary half
  int pos = positions[token];
  pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
  const int slot = slots ? slots[token] : -1;
  const size_t cache_off = slot >= 0 ? (size_t)(slot / page_size) * page_stride + (size_t)(slot % page_size) * nkv * hd : 0;
  const float2* cos2 = reinterpret_cast<const float2*>(cos_tab + (size_t)pos * rot_half);
  const float2* sin2 = reinterpret_cast<const float2*>(sin_tab + (size_t)pos * rot_half);
  // per-lane constants: a lane holds kMax (pair, partner pair) sets
  float2 c[kMax], sn[kMax], wqa[kMax], wqb[kMax], wka[kMax], wkb[kMax];
#pragma unroll
  for (int k = 0; k < kMax; ++k) {
    const int p = lane + 32 * k;
    if (p < rot_pairs) {
      c[k] = cos2[p];
      sn[k] = sin2[p];
      if (q_norm_w) {
        wqa[k] = make_float2(w_offset + to_f32(q_norm_w[2 * p]), w_offset + to_f32(q_norm_w[2 * p + 1]));
        wqb[k] = make_float2(w_offset + to_f32(q_norm_w[2 * p + rot_half]), w_offset + to_f32(q_norm_w[2 * p + rot_half + 1]));
      }
      if (k_norm_w) {
        wka[k] = make_float2(w_offset + to_f32(k_norm_w[2 * p]), w_offset + to_f32(k_norm_w[2 * p + 1]));
        wkb[k] = make_float2(w_offset + to_f32(k_norm_w[2 * p + rot_half]), w_offset + to_f32(k_norm_w[2 * p + rot_half + 1]));
      }
    }
  }
  bf16* row = qkv + (size_t)token * row_stride;
  for (int head = head0; head < head1; ++head) {
    const int kind = head < nq ? 0 : (head < nq + nkv ? 1 : 2);
    const __nv_bfloat162* src2 = reinterpret_cast<const __nv_bfloat162*>(row + head * hd);
    __nv_bfloat162* dst2 = const_cast<__nv_bfloat162*>(src2);   // q: in place
    if (kind != 0) {
      if (slot < 0) continue;    // a padding row: nothing to store
      const int kvh = kind == 1 ? head - nq : head - nq - nkv;
      dst2 = reinterpret_cast<__nv_bfloat162*>((kind == 1 ? k_cache : v_cache) + cache_off + (size_t)kvh * hd);
    }
    if (kind == 2) {
      for (int p = lane; p < npairs; p += 32) dst2[p] = src2[p];
      continue;
    }
    const TW* w = kind == 0 ? q_norm_w : k_norm_w;
    float2 a[kMax], b[kMax];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kMax; ++k) {
      const int p = lane + 32 * k;
      if (p < rot_pairs) {
        a[k] = __bfloat1622float2(src2[p]);
        b[k] = __bfloat1622float2(src2[p + rot_pairs]);
        ss += a[k].x * a[k].x + a[k].y * a[k].y + b[k].x * b[k].x + b[k].y * b[k].y;
      }
    }
    for (int p = 2 * rot_pairs + lane; p < npairs; p += 32) {   // dims beyond the rotary part
      const float2 t = __bfloat1622float2(src2[p]);
      ss += t.x * t.x + t.y * t.y;
    }
    float inv = 1.f;
    if (w) {
      ss = warp_sum(ss);
      inv = rsqrtf(ss / (float)hd + eps);
    }
#pragma unroll
    for (int k = 0; k < kMax; ++k) {
      const int p = lane + 32 * k;
      if (p < rot_pairs) {
        float2 x = a[k], y = b[k];
        if (w) {
          const float2 wa = kind == 0 ? wqa[k] : wka[k], wb = kind == 0 ? wqb[k] : wkb[k];
          x.x *= inv * wa.x; x.y *= inv * wa.y;
          y.x *= inv * wb.x; y.y *= inv * wb.y;
        }
        dst2[p] = __floats2bfloat162_rn(x.x * c[k].x - y.x * sn[k].x, x.y * c[k].y - y.y * sn[k].y);
        dst2[p + rot_pairs] = __floats2bfloat162_rn(x.x * sn[k].x + y.x * c[k].x, x.y * sn[k].y + y.y * c[k].y);
      }
    }
    for (int p = 2 * rot_pairs + lane; p < npairs; p += 32) {
      float2 t = __bfloat1622float2(src2[p]);
      if (w) {
        t.x *= inv * (w_offset + to_f32(w[2 * p]));
        t.y *= inv * (w_offset + to_f32(w[2 * p + 1]));
      }
      dst2[p] = __floats2bfloat162_rn(t.x, t.y);
    }
  }
}

// bfloat16, full rotation (rotary_dim == head_dim), head_dim 32 / 64 / 128, everything 16-byte aligned:
// a lane moves EIGHT neighbouring elements of the first half of a head and their partners in the second
// half with 16-byte accesses, so HD / 16 lanes cover a head and a warp handles 512 / HD heads of one token
// at once; a block of four warps takes 2048 / HD consecutive heads. Many independent 16-byte loads per
// lane (row, cos, sin, weights) are in flight before anything is used: prompt-sized launches run at the
// speed of memory instead of the latency of 4-byte accesses.
template <int HD, typename TW>
__global__ void __launch_bounds__(128)
qk_norm_rope_kv_vec_kernel(bf16* __restrict__ qkv, int row_stride, int nq, int nkv, const TW* __restrict__ q_norm_w,
                           const TW* __restrict__ k_norm_w, float eps, float w_offset, const float* __restrict__ cos_tab,
                           const float* __restrict__ sin_tab, int max_pos, const int* __restrict__ positions,
                           const int* __restrict__ slots, bf16* __restrict__ k_cache, bf16* __restrict__ v_cache,
                           long long page_stride, int page_size, int heads_total) {
  pdl_start();
  constexpr int kHalf = HD / 2;
  constexpr int kLanes = HD / 16;            // lanes per head
  constexpr int kHeadsPerWarp = 32 / kLanes;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int token = blockIdx.x;
  const int head = (blockIdx.y * 4 + warp) * kHeadsPerWarp + lane / kLanes;
  const int sub = lane % kLanes;             // elements [8 sub, 8 sub + 8) of each half
  const bool live = head < heads_total;
  const int kind = head < nq ? 0 : (head < nq + nkv ? 1 : 2);
  int pos = positions[token];
  pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
  const int slot = slots ? slots[token] : -1;
  bf16* src = qkv + (size_t)token * row_stride + (size_t)head * HD;
  bf16* dst = src;   // q: in place
  bool store = live;
  if (live && kind != 0) {
    store = slot >= 0;   // a padding row stores nothing
    const int kvh = kind == 1 ? head - nq : head - nq - nkv;
    if (store)
      dst = (kind == 1 ? k_cache : v_cache) + (size_t)(slot / page_size) * page_stride + (size_t)(slot % page_size) * nkv * HD +
            (size_t)kvh * HD;
  }
  uint4 ra = make_uint4(0, 0, 0, 0), rb = ra;
  if (live) {
    ra = *reinterpret_cast<const uint4*>(src + sub * 8);
    rb = *reinterpret_cast<const uint4*>(src + kHalf + sub * 8);
  }
  if (live && kind == 2) {
    if (store) {
      *reinterpret_cast<uint4*>(dst + sub * 8) = ra;
      *reinterpret_cast<uint4*>(dst + kHalf + sub * 8) = rb;
    }
  }
  // all lanes stay for the shuffles below
  const TW* w = kind == 0 ? q_norm_w : k_norm_w;
  const bool rotate = live && kind != 2;
  float c[8], sn[8], wa[8], wb[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { c[e] = 1.f; sn[e] = 0.f; wa[e] = 1.f; wb[e] = 1.f; }
  if (rotate) {
    const float4* c4 = reinterpret_cast<const float4*>(cos_tab + (size_t)pos * kHalf + sub * 8);
    const float4* s4 = reinterpret_cast<const float4*>(sin_tab + (size_t)pos * kHalf + sub * 8);
    const float4 c0 = c4[0], c1 = c4[1], s0 = s4[0], s1 = s4[1];
    c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
    sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    if (w) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        wa[e] = w_offset + to_f32(w[sub * 8 + e]);
        wb[e] = w_offset + to_f32(w[kHalf + sub * 8 + e]);
      }
    }
  }
  float a[8], b[8];
  {
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&ra);
    const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&rb);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x = __bfloat1622float2(a2[e]), y = __bfloat1622float2(b2[e]);
      a[2 * e] = x.x; a[2 * e + 1] = x.y; b[2 * e] = y.x; b[2 * e + 1] = y.y;
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) ss += a[e] * a[e] + b[e] * b[e];
#pragma unroll
  for (int o = kLanes / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (!rotate || !store) return;
  if (w) {
    const float inv = rsqrtf(ss / (float)HD + eps);
#pragma unroll
    for (int e = 0; e < 8; ++e) { a[e] *= inv * wa[e]; b[e] *= inv * wb[e]; }
  }
  uint4 oa, ob;
  __nv_bfloat162* oa2 = reinterpret_cast<__nv_bfloat162*>(&oa);
  __nv_bfloat162* ob2 = reinterpret_cast<__nv_bfloat162*>(&ob);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    oa2[e] = __floats2bfloat162_rn(a[2 * e] * c[2 * e] - b[2 * e] * sn[2 * e], a[2 * e + 1] * c[2 * e + 1] - b[2 * e + 1] * sn[2 * e + 1]);
    ob2[e] = __floats2bfloat162_rn(a[2 * e] * sn[2 * e] + b[2 * e] * c[2 * e], a[2 * e + 1] * sn[2 * e + 1] + b[2 * e + 1] * c[2 * e + 1]);
  }
  *reinterpret_cast<uint4*>(dst + sub * 8) = oa;
  *reinterpret_cast<uint4*>(dst + kHalf + sub * 8) = ob;
}

// write_kv = 0: only the nq query heads are processed (a mixer that reads another layer's cache).
OI_API int oi_qk_norm_rope_kv(void* qkv, int dtype, int row_stride, int tokens, int nq, int nkv, int hd,
                              const void* q_norm_w, const void* k_norm_w, int norm_dtype, float eps,
                              float w_offset, const float* cos_tab, const float* sin_tab, int rot_half,
                              int max_pos, const int* positions, const int* slots, void* k_cache,
                              void* v_cache, long long page_stride, int page_size, int write_kv,
                              int interleaved, void* stream) {
  OI_REQUIRE(tokens >= 0 && nq > 0 && nkv >= 0 && hd > 0, "qk_norm_rope_kv: bad sizes");
  OI_REQUIRE(rot_half >= 0 && 2 * rot_half <= hd, "qk_norm_rope_kv: rotary_dim %d exceeds head_dim %d",
             2 * rot_half, hd);
  OI_REQUIRE(rot_half == 0 || (cos_tab && sin_tab && max_pos > 0), "qk_norm_rope_kv: rotation without tables");
  OI_REQUIRE(!write_kv || (k_cache && v_cache && slots && page_size > 0), "qk_norm_rope_kv: cache write without a cache");
  if (tokens == 0) return OI_OK;
  const int heads_total = write_kv ? nq + 2 * nkv : nq;
  const long long warps = (long long)tokens * heads_total;
  const int blocks = (int)((warps + 3) / 4);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == OI_F32) {
    oi_launch(qk_norm_rope_kv_kernel<float>, blocks, 128, 0, s, 
        (float*)qkv, row_stride, nq, nkv, hd, q_norm_w, k_norm_w, norm_dtype, eps, w_offset, cos_tab,
        sin_tab, rot_half, max_pos, positions, slots, (float*)k_cache, (float*)v_cache, page_stride,
        page_size, heads_total, tokens, interleaved);
  } else if (dtype == OI_BF16 && !interleaved && 2 * rot_half == hd && (hd == 32 || hd == 64 || hd == 128) && row_stride % 8 == 0 &&
             (uintptr_t)qkv % 16 == 0 && page_stride % 8 == 0 && (uintptr_t)cos_tab % 16 == 0 && (uintptr_t)sin_tab % 16 == 0 &&
             (!write_kv || ((uintptr_t)k_cache % 16 == 0 && (uintptr_t)v_cache % 16 == 0)) &&
             ((!q_norm_w && !k_norm_w) || norm_dtype == OI_BF16 || norm_dtype == OI_F32)) {
    // the 16-byte path: full rotation, aligned operands
    const int heads_per_block = 4 * (512 / hd);
    const dim3 grid(tokens, (heads_total + heads_per_block - 1) / heads_per_block);
#define OI_ROPE_VEC(HD_, TW_)                                                                                        \
  oi_launch(qk_norm_rope_kv_vec_kernel<HD_, TW_>, grid, 128, 0, s, (bf16*)qkv, row_stride, nq, nkv, (const TW_*)q_norm_w, \
            (const TW_*)k_norm_w, eps, w_offset, cos_tab, sin_tab, max_pos, positions, slots, (bf16*)k_cache,         \
            (bf16*)v_cache, page_stride, page_size, heads_total)
    if (norm_dtype == OI_BF16) {
      if (hd == 128) OI_ROPE_VEC(128, bf16); else if (hd == 64) OI_ROPE_VEC(64, bf16); else OI_ROPE_VEC(32, bf16);
    } else {
      if (hd == 128) OI_ROPE_VEC(128, float); else if (hd == 64) OI_ROPE_VEC(64, float); else OI_ROPE_VEC(32, float);
    }
#undef OI_ROPE_VEC
  } else if (dtype == OI_BF16 && !interleaved && rot_half > 0 && rot_half % 2 == 0 && hd % 2 == 0 && hd <= 256 && row_stride % 2 == 0 && tokens <= 2147483647 &&
             (uintptr_t)qkv % 4 == 0 && page_stride % 2 == 0 && (!write_kv || ((uintptr_t)k_cache % 4 == 0 && (uintptr_t)v_cache % 4 == 0)) &&
             (uintptr_t)cos_tab % 8 == 0 && (uintptr_t)sin_tab % 8 == 0) {
    // few tokens (decode): one head per warp for parallelism; many tokens: a warp walks over 2 heads
    const int heads_per_warp = tokens >= 256 ? 2 : 1;
    const dim3 grid(tokens, (heads_total + 4 * heads_per_warp - 1) / (4 * heads_per_warp));
#define OI_ROPE_ARGS(TW_)                                                                                          \
  (bf16*)qkv, row_stride, nq, nkv, hd, (const TW_*)q_norm_w, (const TW_*)k_norm_w, eps, w_offset, cos_tab, sin_tab, \
      rot_half, max_pos, positions, slots, (bf16*)k_cache, (bf16*)v_cache, page_stride, page_size, heads_total,     \
      heads_per_warp
    if (rot_half <= 64) {
      if (norm_dtype == OI_BF16) oi_launch(qk_norm_rope_kv_bf16x2_kernel<bf16, 1>, grid, 128, 0, s, OI_ROPE_ARGS(bf16));
      else oi_launch(qk_norm_rope_kv_bf16x2_kernel<float, 1>, grid, 128, 0, s, OI_ROPE_ARGS(float));
    } else {
      if (norm_dtype == OI_BF16) oi_launch(qk_norm_rope_kv_bf16x2_kernel<bf16, 2>, grid, 128, 0, s, OI_ROPE_ARGS(bf16));
      else oi_launch(qk_norm_rope_kv_bf16x2_kernel<float, 2>, grid, 128, 0, s, OI_ROPE_ARGS(float));
    }
#undef OI_ROPE_ARGS
  } else if (dtype == OI_BF16) {
    oi_launch(qk_norm_rope_kv_kernel<bf16>, blocks, 128, 0, s, 
        (bf16*)qkv, row_stride, nq, nkv, hd, q_norm_w, k_norm_w, norm_dtype, eps, w_offset, cos_tab,
        sin_tab, rot_half, max_pos, positions, slots, (bf16*)k_cache, (bf16*)v_cache, page_stride,
        page_size, heads_total, tokens, interleaved);
  } else {
    OI_REQUIRE(false, "qk_norm_rope_kv: unknown dtype code %d", dtype);
  }
  OI_CHECK_LAUNCH();
  return OI_OK;
}
