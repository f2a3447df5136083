// Paged causal GQA attention on tensor cores for bfloat16, head_dim 32, 64 or 128: prompt portions
// over a cached prefix and split-KV decode in ONE kernel.
//
// A CTA (4 warps) owns 64 query ROWS of one (request, kv head): row r is (token r / group,
// query head r % group), so the `group` query heads that share a kv head sit next to each other
// and every K/V tile is fetched once for all of them. A decoded token is simply a request with one
// query token (group rows). Work items are planned on the host once per step and shared by all
// layers, as the reference plans its attention tiles (pegainfer-kernels/src/ops/attention.rs:396-477);
// an item may cover only a slice of the keys (split-KV, the reference's decode path:
// pegainfer-kernels/csrc/shared/paged_attention.cu:189-263), in which case it writes a normalised
// partial output and its log-sum-exp to scratch and `attention_merge_kernel` combines the slices.
//
// Math: s = (q . k) / sqrt(hd) for keys j <= pos (and j > pos - window), online softmax in float32
// (exp2 with the scale folded in), o = sum p v (paged_attention.cu:439-567). K/V tiles of 64 keys
// are gathered page by page with cp.async into swizzled shared memory, double buffered;
// S = Q K^T and O = P V run as mma.sync m16n8k16 with float32 accumulators.
#include <cooperative_groups.h>

#include "oi_api.h"

namespace cg = cooperative_groups;

namespace {

constexpr int kKeys = 64;      // keys per tile
constexpr int kThreads = 128;

struct AttnParams {
  const bf16* q; int q_row_stride;
  bf16* out; int out_row_stride;
  const bf16* k_cache; const bf16* v_cache; long long page_stride; int page_size;
  const int* block_table; int bt_stride;
  const int* cu_seqlens;   // [requests + 1] first row of each request in this step
  const int* kv_lens;      // [requests] keys visible after this step
  const int4* items;       // (request, first token of the tile, split, nsplits)
  int nq, nkv, group;
  float scale_log2;        // softmax scale * log2(e)
  int window;              // 0 = none
  float* part_o; float* part_lse; int max_splits;  // scratch for split items
  int merge_in_kernel;     // decode kernel: the CTAs of a row form a cluster and merge their slices themselves:
                           // 1 by reading each other's shared memory, 2 by depositing partials with the merging CTA
  // decode kernel, fuse_rope != 0: `q` is the raw fused projection [rows, (nq + 2 nkv) * hd]; the per-head
  // q/k norm, the rotation and the write of the step's key and value into their page happen in the kernel
  int fuse_rope, write_kv;
  const void* q_norm_w; const void* k_norm_w; int norm_dtype; float eps, w_offset;
  const float* cos_tab; const float* sin_tab; int rot_half, max_pos;
  const int* positions; const int* slots;
};

__device__ __forceinline__ unsigned smem_u32(const void* p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(unsigned dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x on the special-function unit (x <= 0 here; -inf gives 0)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// Shared-memory tile [kKeys][HD] bf16, 16-byte chunks XOR-swizzled by the row so that the eight
// rows an ldmatrix reads fall into different banks.
template <int HD>
__device__ __forceinline__ int tile_offset(int row, int chunk) {
  constexpr int kChunks = HD / 8;
  return row * HD + ((chunk ^ (row & 7)) & (kChunks - 1)) * 8 + ((chunk & ~(kChunks - 1)) * 8);
}

// The page that holds this thread's key row of the tile starting at key0 (-1 beyond key_end).
// Looked up one tile ahead of its use, so that the copies are not held up by the table read.
__device__ __forceinline__ int tile_page(const AttnParams& p, const int* bt, int key0, int key_end) {
  const int key = key0 + (threadIdx.x >> 1);
  return key < key_end ? bt[key / p.page_size] : -1;
}

template <int HD>
__device__ __forceinline__ void load_tile(bf16* smem, const bf16* cache, const AttnParams& p, int page,
                                          int kvh, int key0) {
  // 64 rows x (HD/8) chunks; two threads per row, each HD/16 chunks
  constexpr int kChunks = HD / 8;
  const int row = threadIdx.x >> 1;
  const int c0 = (threadIdx.x & 1) * (kChunks / 2);
  const int key = key0 + row;
  const bool valid = page >= 0;
  const bf16* src = cache;
  if (valid) src = cache + (size_t)page * p.page_stride + (size_t)(key % p.page_size) * p.nkv * HD + (size_t)kvh * HD;
#pragma unroll
  for (int c = 0; c < kChunks / 2; ++c) {
    const int chunk = c0 + c;
    cp_async16(smem_u32(smem + tile_offset<HD>(row, chunk)), src + chunk * 8, valid);
  }
}

// MT: 16-row slabs per warp. MT = 2 (128 rows per CTA) lets every K/V fragment read from shared
// memory feed two MMAs, which halves the shared-memory traffic per flop: the version for prompt
// portions. MT = 1 (64 rows per CTA) wastes less on short portions.
template <int HD, int MT>
__global__ void __launch_bounds__(kThreads)
attention_mma_kernel(const AttnParams p) {
  pdl_start();
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int kTileRows = 64 * MT;
  // [Q: kTileRows x HD][stage][K | V][kKeys][HD]
  bf16* const q_sm = reinterpret_cast<bf16*>(smem_raw);
  bf16* const tiles = q_sm + kTileRows * HD;
  auto k_tile = [&](int stage) { return tiles + (size_t)stage * 2 * kKeys * HD; };
  auto v_tile = [&](int stage) { return tiles + (size_t)stage * 2 * kKeys * HD + kKeys * HD; };

  // items come longest first; the kv heads of an item are neighbours in the grid, so the launch
  // order is longest first over the whole grid
  const int4 item = p.items[blockIdx.x / p.nkv];
  const int req = item.x, tok0 = item.y, split = item.z, nsplits = item.w;
  const int kvh = blockIdx.x % p.nkv;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int group = p.group;
  const int q_start = p.cu_seqlens[req];
  const int q_len = p.cu_seqlens[req + 1] - q_start;
  const int kv_len = p.kv_lens[req];
  const int* bt = p.block_table + (size_t)req * p.bt_stride;
  const int toks_per_tile = kTileRows / group;
  const int tile_toks = min(toks_per_tile, q_len - tok0);
  const int pos0 = kv_len - q_len + tok0;                 // position of the tile's first token
  // keys any row of the tile may see
  int lo = 0;
  if (p.window > 0) lo = max(0, pos0 - p.window + 1);
  const int hi = pos0 + tile_toks;                        // exclusive: last token's own key included
  lo &= ~(kKeys - 1);
  // this item's slice of [lo, hi), in whole tiles
  const int span_tiles = (hi - lo + kKeys - 1) / kKeys;
  const int tiles_per_split = (span_tiles + nsplits - 1) / nsplits;
  const int t_begin = split * tiles_per_split;
  const int t_end = min(span_tiles, t_begin + tiles_per_split);

  // ---- Q tile into shared memory (rows = (token, head) pairs; rows past the tile are zero)
  {
    constexpr int kChunks = HD / 8;
    for (int i = threadIdx.x; i < kTileRows * kChunks; i += kThreads) {
      const int r = i / kChunks, chunk = i % kChunks;
      const int t = r / group;
      const bool valid = t < tile_toks;
      const bf16* src = p.q;
      if (valid) src = p.q + (size_t)(q_start + tok0 + t) * p.q_row_stride + (size_t)(kvh * group + r % group) * HD + chunk * 8;
      cp_async16(smem_u32(q_sm + tile_offset<HD>(r, chunk)), src, valid);
    }
    cp_async_commit();
  }

  // ---- the rows this thread owns: slab mt, halves i: row = warp*16*MT + mt*16 + lane/4 + 8*i
  const int warp_row0 = warp * 16 * MT;
  int pos[MT][2];
  bool row_ok[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = warp_row0 + mt * 16 + (lane >> 2) + 8 * i;
      const int t = r / group;
      row_ok[mt][i] = t < tile_toks;
      pos[mt][i] = pos0 + t;
    }
  // the last position any row of this warp holds: tiles beyond it are skipped by this warp
  const int warp_last_pos = pos0 + min(tile_toks - 1, (warp_row0 + 16 * MT - 1) / group);
  const int warp_first_pos = pos0 + warp_row0 / group;
  const bool warp_active = warp_row0 < tile_toks * group;

  constexpr int kSteps = HD / 16;
  constexpr int kOTiles = HD / 8;
  float o[MT][kOTiles][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int j = 0; j < kOTiles; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[mt][j][e] = 0.f;
  float m[MT][2], l[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) { m[mt][0] = m[mt][1] = -INFINITY; l[mt][0] = l[mt][1] = 0.f; }

  // ldmatrix lane constants (element offsets; chunk indices enter through one XOR)
  const int lm_mat = lane >> 3, lm_rin = lane & 7;
  const int q_row = (lm_mat & 1) * 8 + lm_rin;              // A operand: matrices 0,2 rows 0-7; 1,3 rows 8-15
  const int q_swz_hi = lm_mat >> 1;                         // chunk = 2 ks + (mat >> 1)
  const int k_row = (lm_mat >> 1) * 8 + lm_rin;             // K: matrices 0,1 keys 0-7; 2,3 keys 8-15
  const int k_swz = (lm_mat & 1) ^ (k_row & 7);             // chunk = 2 ks + (mat & 1)
  const int v_row = (lm_mat & 1) * 8 + lm_rin;              // V: matrices 0,2 keys 0-7; 1,3 keys 8-15
  const int v_swz = (lm_mat >> 1) ^ (v_row & 7);            // chunk = j + (mat >> 1)
  constexpr int kMask = HD / 8 - 1;

  int page_next = -1;      // page of this thread's row in the tile after the one being loaded
  if (t_begin < t_end) {
    const int page0 = tile_page(p, bt, lo + t_begin * kKeys, hi);
    page_next = t_begin + 1 < t_end ? tile_page(p, bt, lo + (t_begin + 1) * kKeys, hi) : -1;
    load_tile<HD>(k_tile(0), p.k_cache, p, page0, kvh, lo + t_begin * kKeys);
    cp_async_commit();
    load_tile<HD>(v_tile(0), p.v_cache, p, page0, kvh, lo + t_begin * kKeys);
    cp_async_commit();
  }
  for (int t = t_begin; t < t_end; ++t) {
    const int buf = (t - t_begin) & 1;
    const int key0 = lo + t * kKeys;
    const bool more = t + 1 < t_end;
    if (more) {
      const int page = page_next;
      page_next = t + 2 < t_end ? tile_page(p, bt, key0 + 2 * kKeys, hi) : -1;   // used next iteration
      load_tile<HD>(k_tile(buf ^ 1), p.k_cache, p, page, kvh, key0 + kKeys);
      cp_async_commit();
      load_tile<HD>(v_tile(buf ^ 1), p.v_cache, p, page, kvh, key0 + kKeys);
      cp_async_commit();
      cp_async_wait<3>();   // Q and K of this tile have landed
    } else {
      cp_async_wait<1>();
    }
    __syncthreads();

    // a warp all of whose rows lie before this tile's first key has nothing to do here
    const bool compute = warp_active && key0 <= warp_last_pos;
    unsigned pf[MT][kKeys / 16][4];
    if (compute) {
      // ---- S = Q K^T : 16*MT rows x 64 keys per warp
      float s[MT][kKeys / 8][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int j = 0; j < kKeys / 8; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) s[mt][j][e] = 0.f;
      {
        const unsigned kbase = smem_u32(k_tile(buf));
        const unsigned qbase = smem_u32(q_sm);
#pragma unroll
        for (int ks = 0; ks < kSteps; ++ks) {
          unsigned qf[MT][4];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const int r = warp_row0 + mt * 16 + q_row;
            ldmatrix_x4(qf[mt][0], qf[mt][1], qf[mt][2], qf[mt][3],
                        qbase + (r * HD + ((((ks * 2) ^ q_swz_hi ^ (r & 7)) & kMask) * 8)) * 2);
          }
#pragma unroll
          for (int j = 0; j < kKeys / 8; j += 2) {
            unsigned b0, b1, b2, b3;   // (keys j*8.., d lo), (same keys, d hi), (keys (j+1)*8.., d lo), (.., d hi)
            ldmatrix_x4(b0, b1, b2, b3, kbase + ((j * 8 + k_row) * HD + ((((ks * 2) ^ k_swz) & kMask) * 8)) * 2);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              mma_bf16(s[mt][j], qf[mt], b0, b1);
              mma_bf16(s[mt][j + 1], qf[mt], b2, b3);
            }
          }
        }
      }
      // ---- mask (only where a row may not see the whole tile) + online softmax
      const bool full = key0 + kKeys - 1 <= warp_first_pos && (p.window <= 0 || key0 > warp_last_pos - p.window) &&
                        warp_row0 + 16 * MT <= tile_toks * group;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        // the running maximum m is kept of the RAW scores; the scale enters in one fused
        // multiply-add per element: p = 2^(s * scale - m * scale)
        float m_new[2] = {m[mt][0], m[mt][1]};
        if (full) {
#pragma unroll
          for (int j = 0; j < kKeys / 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) m_new[e >> 1] = fmaxf(m_new[e >> 1], s[mt][j][e]);
        } else {
#pragma unroll
          for (int j = 0; j < kKeys / 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = e >> 1;
              const int key = key0 + j * 8 + (lane & 3) * 2 + (e & 1);
              const bool ok = row_ok[mt][i] && key <= pos[mt][i] && (p.window <= 0 || key > pos[mt][i] - p.window);
              s[mt][j][e] = ok ? s[mt][j][e] : -INFINITY;
              m_new[i] = fmaxf(m_new[i], s[mt][j][e]);
            }
        }
        float corr[2], base[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
          m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
          corr[i] = (m[mt][i] == -INFINITY) ? 0.f : fast_exp2((m[mt][i] - m_new[i]) * p.scale_log2);
          l[mt][i] *= corr[i];
          base[i] = m_new[i] == -INFINITY ? 0.f : m_new[i] * p.scale_log2;
          m[mt][i] = m_new[i];
        }
#pragma unroll
        for (int j = 0; j < kKeys / 8; ++j) {
          const float p0 = fast_exp2(fmaf(s[mt][j][0], p.scale_log2, -base[0])), p1 = fast_exp2(fmaf(s[mt][j][1], p.scale_log2, -base[0]));
          const float p2 = fast_exp2(fmaf(s[mt][j][2], p.scale_log2, -base[1])), p3 = fast_exp2(fmaf(s[mt][j][3], p.scale_log2, -base[1]));
          l[mt][0] += p0 + p1;
          l[mt][1] += p2 + p3;
          // accumulator tiles (2i, 2i+1) are the A fragment of key step i
          pf[mt][j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
          pf[mt][j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        if (!__all_sync(0xffffffffu, corr[0] == 1.f && corr[1] == 1.f)) {
#pragma unroll
          for (int j = 0; j < kOTiles; ++j) {
            o[mt][j][0] *= corr[0]; o[mt][j][1] *= corr[0];
            o[mt][j][2] *= corr[1]; o[mt][j][3] *= corr[1];
          }
        }
      }
    }

    if (more) cp_async_wait<2>(); else cp_async_wait<0>();   // V of this tile has landed
    __syncthreads();
    // ---- O += P V : k = 64 keys (4 steps), n = HD
    if (compute) {
      const unsigned vbase = smem_u32(v_tile(buf));
#pragma unroll
      for (int kk = 0; kk < kKeys / 16; ++kk) {
#pragma unroll
        for (int j = 0; j < kOTiles; j += 2) {
          unsigned b0, b1, b2, b3;   // (keys kk*16.., d j*8..), (keys +8, same d), (keys kk*16.., d (j+1)*8..), (keys +8, ..)
          ldmatrix_x4_trans(b0, b1, b2, b3, vbase + ((kk * 16 + v_row) * HD + (((j ^ v_swz) & kMask) * 8)) * 2);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            mma_bf16(o[mt][j], pf[mt][kk], b0, b1);
            mma_bf16(o[mt][j + 1], pf[mt][kk], b2, b3);
          }
        }
      }
    }
    __syncthreads();  // everyone is done with this buffer before the next prefetch overwrites it
  }
  cp_async_wait<0>();

  // ---- epilogue
  const int col = (lane & 3) * 2;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float li = l[mt][i];
      li += __shfl_xor_sync(0xffffffffu, li, 1);
      li += __shfl_xor_sync(0xffffffffu, li, 2);
      if (!row_ok[mt][i]) continue;
      const int r = warp_row0 + mt * 16 + (lane >> 2) + 8 * i;
      const int head = kvh * group + r % group;
      const size_t grow = (size_t)(q_start + tok0 + r / group);
      const float inv = li > 0.f ? 1.f / li : 0.f;
      if (nsplits == 1) {
        bf16* op = p.out + grow * p.out_row_stride + (size_t)head * HD + col;
#pragma unroll
        for (int j = 0; j < kOTiles; ++j)
          *reinterpret_cast<unsigned*>(op + j * 8) = pack_bf16(o[mt][j][2 * i] * inv, o[mt][j][2 * i + 1] * inv);
      } else {
        const size_t slot = (grow * p.nq + head) * p.max_splits + split;
        float* op = p.part_o + slot * HD + col;
#pragma unroll
        for (int j = 0; j < kOTiles; ++j)
          *reinterpret_cast<float2*>(op + j * 8) = make_float2(o[mt][j][2 * i] * inv, o[mt][j][2 * i + 1] * inv);
        if ((lane & 3) == 0) p.part_lse[slot] = li > 0.f ? m[mt][i] * p.scale_log2 + log2f(li) : -INFINITY;  // base-2 log-sum-exp
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Decode rows (one query token per request): every WARP owns one slice of a request's keys for
// one kv head, with a private ring of 16-key K/V tiles in shared memory filled by cp.async. No
// block-wide barrier: a warp waits only for its own copies, so several tiles per warp are in
// flight all the time, which is what a bandwidth-bound gather over pages needs. Each warp ends with
// a normalised partial output and its log-sum-exp. The CTAs of a row (up to 8: 32 slices) run as a
// thread-block cluster and merge the slices themselves through distributed shared memory (partials
// deposited with the merging CTA behind one cluster barrier, or read from each other's shared memory
// when the receive buffer would not fit); with more slices the partials go to scratch in global
// memory and attention_merge_kernel combines them. The tiles of earlier steps' keys are requested
// before the kernel waits for its predecessor on the stream (programmatic dependent launch), and on
// request the kernel also does the per-head q/k norm, the rotation and the write of the step's key
// and value (fuse_rope), which otherwise take a kernel of their own in front of it; the new key and value
// reach the scores through shared memory (put into the row's last tile by the warp that owns it), so no
// warp waits for a store to come back from global memory.
// ---------------------------------------------------------------------------
constexpr int kDecWarps = 4;
constexpr int kDecKeys = 16;     // keys per tile
constexpr int kDecStages = 3;

// Per-lane constants of the 16-key tile copy: which (row, chunk) pairs a lane moves, where they go
// in the swizzled tile and where they come from relative to the tile's first key.
template <int HD>
struct TileLane {
  static constexpr int kChunks = HD / 8;                 // 16-byte chunks per key row
  static constexpr int kPerLane = kDecKeys * kChunks / 32;
  int smem_off[kPerLane];    // element offset inside the tile
  int glob_off[kPerLane];    // element offset from the first key's row of this kv head
  int row[kPerLane];
  __device__ __forceinline__ void init(int lane, int nkv) {
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int id = lane + 32 * i;
      row[i] = id / kChunks;
      const int chunk = id % kChunks;
      smem_off[i] = tile_offset<HD>(row[i], chunk);
      glob_off[i] = row[i] * nkv * HD + chunk * 8;
    }
  }
};

// Copy keys [key0, key0 + 16) of one kv head into a K tile and a V tile; rows at or beyond key_end
// are zero-filled. V lies at a fixed distance from K in the cache (`v_delta` elements).
// `aligned`: the page size is a multiple of 16, so the tile lies in one page: one table lookup, and
// (page index, offset in page) are advanced by the caller without a division.
template <int HD>
__device__ __forceinline__ void load_kv_tile16(bf16* k_smem, bf16* v_smem, const AttnParams& p, const int* bt,
                                               long long v_delta, int kvh, int key0, int key_end,
                                               const TileLane<HD>& tl, bool aligned, int pg, int off) {
  constexpr int kPerLane = TileLane<HD>::kPerLane;
  const unsigned kb = smem_u32(k_smem), vb = smem_u32(v_smem);
  if (aligned) {
    const int page = bt[pg];
    const bf16* base = p.k_cache + (size_t)page * p.page_stride + (size_t)off * p.nkv * HD + (size_t)kvh * HD;
    if (key0 + kDecKeys <= key_end) {
#pragma unroll
      for (int i = 0; i < kPerLane; ++i) cp_async16(kb + tl.smem_off[i] * 2, base + tl.glob_off[i], true);
#pragma unroll
      for (int i = 0; i < kPerLane; ++i) cp_async16(vb + tl.smem_off[i] * 2, base + v_delta + tl.glob_off[i], true);
    } else {
#pragma unroll
      for (int i = 0; i < kPerLane; ++i) {
        const bool valid = key0 + tl.row[i] < key_end;
        cp_async16(kb + tl.smem_off[i] * 2, valid ? base + tl.glob_off[i] : p.k_cache, valid);
        cp_async16(vb + tl.smem_off[i] * 2, valid ? base + v_delta + tl.glob_off[i] : p.k_cache, valid);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int key = key0 + tl.row[i];
      const bool valid = key < key_end;
      const bf16* src = p.k_cache;
      if (valid) {
        const int page = bt[key / p.page_size];
        src = p.k_cache + (size_t)page * p.page_stride + (size_t)(key % p.page_size) * p.nkv * HD + (size_t)kvh * HD +
              (tl.glob_off[i] - tl.row[i] * p.nkv * HD);
      }
      cp_async16(kb + tl.smem_off[i] * 2, src, valid);
      cp_async16(vb + tl.smem_off[i] * 2, valid ? src + v_delta : src, valid);
    }
  }
}

// One head of the fused projection, by one warp: per-head RMSNorm (weights optional), rotate-half of the
// pairs (d, d + rot_half) with the position's cos/sin row, dims beyond 2 * rot_half only normalised;
// float32 arithmetic, one rounding at the store. The formulas of qk_norm_rope_kv_bf16x2_kernel (rope_kv.cu).
// A lane owns the element pair (2 lane, 2 lane + 1) of the first rotary half and its partner pair in the
// second (head_dim <= 128: at most 32 such pairs); its cos/sin values and norm weights (wa, wb, with the
// offset added) are fetched by the caller ahead of time.
struct HeadIn { float2 x, y; };
__device__ __forceinline__ HeadIn head_load(const bf16* __restrict__ src, int rot_half, int lane) {
  const __nv_bfloat162* src2 = reinterpret_cast<const __nv_bfloat162*>(src);
  const int rot_pairs = rot_half / 2;
  HeadIn in;
  in.x = in.y = make_float2(0.f, 0.f);
  if (lane < rot_pairs) {
    in.x = __bfloat1622float2(src2[lane]);
    in.y = __bfloat1622float2(src2[lane + rot_pairs]);
  }
  return in;
}
__device__ __forceinline__ void head_finish(HeadIn in, const bf16* __restrict__ src, bf16* __restrict__ dst, int hd,
                                            const void* w, int norm_dtype, float eps, float w_offset, float2 wa,
                                            float2 wb, float2 c, float2 sn, int rot_half, int lane) {
  const __nv_bfloat162* src2 = reinterpret_cast<const __nv_bfloat162*>(src);
  __nv_bfloat162* dst2 = reinterpret_cast<__nv_bfloat162*>(dst);
  const int npairs = hd / 2, rot_pairs = rot_half / 2;
  const bool mine = lane < rot_pairs;
  float2 x = in.x, y = in.y;
  float inv = 1.f;
  if (w) {
    float ss = x.x * x.x + x.y * x.y + y.x * y.x + y.y * y.y;
    for (int pr = 2 * rot_pairs + lane; pr < npairs; pr += 32) {
      const float2 t = __bfloat1622float2(src2[pr]);
      ss += t.x * t.x + t.y * t.y;
    }
    ss = warp_sum(ss);
    inv = rsqrtf(ss / (float)hd + eps);
    x.x *= inv * wa.x; x.y *= inv * wa.y;
    y.x *= inv * wb.x; y.y *= inv * wb.y;
  }
  if (mine) {
    dst2[lane] = __floats2bfloat162_rn(x.x * c.x - y.x * sn.x, x.y * c.y - y.y * sn.y);
    dst2[lane + rot_pairs] = __floats2bfloat162_rn(x.x * sn.x + y.x * c.x, x.y * sn.y + y.y * c.y);
  }
  for (int pr = 2 * rot_pairs + lane; pr < npairs; pr += 32) {
    float2 t = __bfloat1622float2(src2[pr]);
    if (w) {
      t.x *= inv * (w_offset + load_as_f32(w, norm_dtype, 2 * pr));
      t.y *= inv * (w_offset + load_as_f32(w, norm_dtype, 2 * pr + 1));
    }
    dst2[pr] = __floats2bfloat162_rn(t.x, t.y);
  }
}
__device__ __forceinline__ void warp_norm_rope_head(const bf16* __restrict__ src, bf16* __restrict__ dst, int hd,
                                                    const void* w, int norm_dtype, float eps, float w_offset, float2 wa,
                                                    float2 wb, float2 c, float2 sn, int rot_half, int lane) {
  head_finish(head_load(src, rot_half, lane), src, dst, hd, w, norm_dtype, eps, w_offset, wa, wb, c, sn, rot_half, lane);
}

template <int HD>
__global__ void __launch_bounds__(kDecWarps * 32)
attention_decode_kernel(const AttnParams p) {
  pdl_trigger();
  const bool deposit = p.merge_in_kernel == 2 && gridDim.x > 0 && p.max_splits > kDecWarps;   // a cluster that pushes
  if (deposit) asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");   // phase 0: "this CTA runs"
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // [warp][stage][K | V][16][HD]
  bf16* const ring = reinterpret_cast<bf16*>(smem_raw) + (size_t)warp * kDecStages * 2 * kDecKeys * HD;
  auto k_tile = [&](int stage) { return ring + (size_t)stage * 2 * kDecKeys * HD; };
  auto v_tile = [&](int stage) { return ring + (size_t)stage * 2 * kDecKeys * HD + kDecKeys * HD; };

  const int4 item = p.items[blockIdx.x];          // (request, -, first slice of this CTA, nsplits)
  const int req = item.x, split = item.z + warp, nsplits = item.w;
  const int kvh = blockIdx.y;
  const int group = p.group;
  const int row_q = p.cu_seqlens[req];            // the request's single row in this step
  const int kv_len = p.kv_lens[req];
  const int* bt = p.block_table + (size_t)req * p.bt_stride;
  const int pos = kv_len - 1;
  int lo = 0;
  if (p.window > 0) lo = max(0, pos - p.window + 1) & ~(kDecKeys - 1);
  const int span_tiles = (kv_len - lo + kDecKeys - 1) / kDecKeys;
  const int tiles_per_split = (span_tiles + nsplits - 1) / nsplits;
  const int t_begin = min(span_tiles, split * tiles_per_split);
  const int t_end = min(span_tiles, t_begin + tiles_per_split);
  const bool split_ok = split < nsplits;
  const bool aligned = (p.page_size % kDecKeys) == 0;
  TileLane<HD> tl;
  tl.init(lane, p.nkv);
  // ldmatrix addresses: lane -> (matrix, row in matrix); element offset = row * HD + ((chunk ^ (row & 7)) & mask) * 8
  const int lm_mat = lane >> 3, lm_rin = lane & 7;
  const int k_row = (lm_mat >> 1) * 8 + lm_rin;             // K: matrices 0,1 keys 0-7; 2,3 keys 8-15
  const int k_row_off = k_row * HD, k_swz = (lm_mat & 1) ^ (k_row & 7);   // chunk = 2 ks + (mat & 1)
  const int v_row = (lm_mat & 1) * 8 + lm_rin;              // V: matrices 0,2 keys 0-7; 1,3 keys 8-15
  const int v_row_off = v_row * HD, v_swz = (lm_mat >> 1) ^ (v_row & 7);  // chunk = j + (mat >> 1)

  constexpr int kOTiles = HD / 8;
  float o[kOTiles][4];
#pragma unroll
  for (int j = 0; j < kOTiles; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  // the next tile to copy: its first key, its page (index into the block table) and offset there
  const long long v_delta = p.v_cache - p.k_cache;
  int ld_t = t_begin, ld_stage = 0;
  int ld_key = lo + t_begin * kDecKeys;
  int ld_pg = ld_key / p.page_size, ld_off = ld_key % p.page_size;
  auto issue_next = [&]() {   // one commit per call, empty when past the end
    if (ld_t < t_end) {
      load_kv_tile16<HD>(k_tile(ld_stage), v_tile(ld_stage), p, bt, v_delta, kvh, ld_key, kv_len, tl, aligned, ld_pg, ld_off);
      ++ld_t;
      ld_key += kDecKeys;
      ld_off += kDecKeys;
      if (ld_off >= p.page_size) { ld_off -= p.page_size; ++ld_pg; }   // aligned case: exact
      ld_stage = ld_stage + 1 == kDecStages ? 0 : ld_stage + 1;
    }
    cp_async_commit();
  };
  // Prologue: the ring is filled (kDecStages tiles in flight). Keys of earlier steps do not change any more, so
  // their tiles are requested BEFORE waiting for the kernels ahead on the stream. The row's last tile holds the
  // key and value of this step: when another kernel has stored them it is requested, like q, only after the wait;
  // when this kernel stores them itself (fuse_rope with write_kv) the tile is requested early as well, and the
  // warp that owns it puts the new row into the tile in shared memory once the copy has landed. (The lengths, the
  // block table and the items were copied to the device before the step's first kernel.)
  const bool inserts_row = p.fuse_rope && p.write_kv;
  int primed = 0;
  if (split_ok) {
    for (; primed < kDecStages && (inserts_row || ld_t != span_tiles - 1); ++primed) issue_next();
  }
  // fuse_rope: this lane's cos/sin values and norm weights do not depend on the step's kernels either
  float2 rc = make_float2(1.f, 1.f), rs = make_float2(0.f, 0.f);
  float2 wqa = rc, wqb = rc, wka = rc, wkb = rc;
  const bool owns_last_tile = split_ok && t_begin < t_end && t_end == span_tiles;
  if (p.fuse_rope && lane < p.rot_half / 2) {
    int rpos = p.positions[row_q];
    rpos = rpos < 0 ? 0 : (rpos >= p.max_pos ? p.max_pos - 1 : rpos);
    rc = reinterpret_cast<const float2*>(p.cos_tab + (size_t)rpos * p.rot_half)[lane];
    rs = reinterpret_cast<const float2*>(p.sin_tab + (size_t)rpos * p.rot_half)[lane];
    if (p.q_norm_w) {
      wqa = make_float2(p.w_offset + load_as_f32(p.q_norm_w, p.norm_dtype, 2 * lane), p.w_offset + load_as_f32(p.q_norm_w, p.norm_dtype, 2 * lane + 1));
      wqb = make_float2(p.w_offset + load_as_f32(p.q_norm_w, p.norm_dtype, 2 * lane + p.rot_half),
                        p.w_offset + load_as_f32(p.q_norm_w, p.norm_dtype, 2 * lane + p.rot_half + 1));
    }
    if (p.k_norm_w && p.write_kv && owns_last_tile) {
      wka = make_float2(p.w_offset + load_as_f32(p.k_norm_w, p.norm_dtype, 2 * lane), p.w_offset + load_as_f32(p.k_norm_w, p.norm_dtype, 2 * lane + 1));
      wkb = make_float2(p.w_offset + load_as_f32(p.k_norm_w, p.norm_dtype, 2 * lane + p.rot_half),
                        p.w_offset + load_as_f32(p.k_norm_w, p.norm_dtype, 2 * lane + p.rot_half + 1));
    }
  }
  pdl_wait();
  // ---- with fuse_rope: this kv head's query heads are normalised and rotated into shared memory (every CTA of
  // the row does its own copy), and the warp that owns the row's last tile normalises and rotates the step's
  // key and stores it, and the value, into their page before it requests that tile
  const bf16* q_src = p.q + (size_t)row_q * p.q_row_stride + (size_t)(kvh * group) * HD;   // [group][HD]
  bool insert = false;   // this warp puts the step's key and value into the row's last tile
  bf16* const q_s = reinterpret_cast<bf16*>(smem_raw + (size_t)kDecWarps * kDecStages * 2 * kDecKeys * HD * sizeof(bf16));
  bf16* const new_k = q_s + 16 * HD;   // the step's key (normalised, rotated) and value of this kv head
  bf16* const new_v = new_k + HD;
  if (p.fuse_rope) {
    // the owner of the last tile asks for the raw key and value together with the query heads
    const bf16* row = p.q + (size_t)row_q * p.q_row_stride;
    const bf16* k_raw = row + (size_t)(p.nq + kvh) * HD;
    int slot = -1;
    HeadIn kin;
    uint4 vin = make_uint4(0u, 0u, 0u, 0u);
    if (inserts_row && owns_last_tile) {
      slot = p.slots[row_q];   // a padding row (slot < 0) stores nothing
      insert = slot >= 0;
    }
    if (insert) {
      kin = head_load(k_raw, p.rot_half, lane);
      if (lane < HD / 8) vin = reinterpret_cast<const uint4*>(row + (size_t)(p.nq + p.nkv + kvh) * HD)[lane];
    }
    for (int r = warp; r < group; r += kDecWarps)
      warp_norm_rope_head(q_src + (size_t)r * HD, q_s + r * HD, HD, p.q_norm_w, p.norm_dtype, p.eps, p.w_offset, wqa, wqb,
                          rc, rs, p.rot_half, lane);
    if (insert) {
      head_finish(kin, k_raw, new_k, HD, p.k_norm_w, p.norm_dtype, p.eps, p.w_offset, wka, wkb, rc, rs, p.rot_half, lane);
      __syncwarp();
      const size_t off = (size_t)(slot / p.page_size) * p.page_stride + (size_t)(slot % p.page_size) * p.nkv * HD + (size_t)kvh * HD;
      if (lane < HD / 8) {
        reinterpret_cast<uint4*>(new_v)[lane] = vin;
        reinterpret_cast<uint4*>(const_cast<bf16*>(p.v_cache) + off)[lane] = vin;
        reinterpret_cast<uint4*>(const_cast<bf16*>(p.k_cache) + off)[lane] = reinterpret_cast<const uint4*>(new_k)[lane];
      }
    }
    __syncthreads();
    q_src = q_s;
  }
  // ---- Q fragments: rows are the `group` query heads of this kv head (rows >= group are zero)
  constexpr int kSteps = HD / 16;
  const int r_lo = lane >> 2;                     // rows r_lo and r_lo + 8
  unsigned qf[kSteps][4];
  {
    const int col = (lane & 3) * 2;
#pragma unroll
    for (int ks = 0; ks < kSteps; ++ks) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = r_lo + 8 * i;
        unsigned a = 0, b = 0;
        if (r < group && split_ok) {
          const bf16* qp = q_src + (size_t)r * HD + ks * 16 + col;
          a = *reinterpret_cast<const unsigned*>(qp);
          b = *reinterpret_cast<const unsigned*>(qp + 8);
        }
        qf[ks][i] = a;
        qf[ks][i + 2] = b;
      }
    }
  }
  if (split_ok) {
    for (; primed < kDecStages; ++primed) issue_next();
    int stage = 0;
    for (int t = t_begin; t < t_end; ++t) {
      cp_async_wait<kDecStages - 1>();   // tile t (this thread's part) has landed ...
      __syncwarp();                      // ... and so have the other lanes' parts
      const int key0 = lo + t * kDecKeys;
      if (insert && t == span_tiles - 1) {
        // what the copy brought for the step's own row is whatever the page held: the new key and value replace it
        const int r = pos - key0;
        if (lane < HD / 8)
          *reinterpret_cast<uint4*>(k_tile(stage) + tile_offset<HD>(r, lane)) = reinterpret_cast<const uint4*>(new_k)[lane];
        else if (lane >= 16 && lane - 16 < HD / 8)
          *reinterpret_cast<uint4*>(v_tile(stage) + tile_offset<HD>(r, lane - 16)) = reinterpret_cast<const uint4*>(new_v)[lane - 16];
        __syncwarp();
      }

      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      {
        const unsigned kbase = smem_u32(k_tile(stage));
#pragma unroll
        for (int ks = 0; ks < kSteps; ++ks) {
          unsigned b0, b1, b2, b3;   // (keys 0-7, d lo), (keys 0-7, d hi), (keys 8-15, d lo), (keys 8-15, d hi)
          // the chunk index only enters through an XOR with the (fixed) row: one XOR per step
          ldmatrix_x4(b0, b1, b2, b3, kbase + (k_row_off + ((((ks * 2) ^ k_swz) & (HD / 8 - 1)) * 8)) * 2);
          mma_bf16(s[0], qf[ks], b0, b1);
          mma_bf16(s[1], qf[ks], b2, b3);
        }
      }
      float m_new[2] = {m[0], m[1]};
      // a tile whose every key every row sees needs no mask (rows beyond the group hold zeros
      // and are never stored)
      const bool full = key0 + kDecKeys <= kv_len && (p.window <= 0 || key0 > pos - p.window);
      if (full) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s[j][e] *= p.scale_log2;
            m_new[e >> 1] = fmaxf(m_new[e >> 1], s[j][e]);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = e >> 1;
            const int key = key0 + j * 8 + (lane & 3) * 2 + (e & 1);
            const bool ok = key <= pos && (p.window <= 0 || key > pos - p.window);
            s[j][e] = ok ? s[j][e] * p.scale_log2 : -INFINITY;
            m_new[i] = fmaxf(m_new[i], s[j][e]);
          }
        }
      }
      float corr[2], base[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 1));
        m_new[i] = fmaxf(m_new[i], __shfl_xor_sync(0xffffffffu, m_new[i], 2));
        corr[i] = (m[i] == -INFINITY) ? 0.f : exp2f(m[i] - m_new[i]);
        l[i] *= corr[i];
        base[i] = m_new[i] == -INFINITY ? 0.f : m_new[i];
        m[i] = m_new[i];
      }
      unsigned pf[4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float p0 = exp2f(s[j][0] - base[0]), p1 = exp2f(s[j][1] - base[0]);
        const float p2 = exp2f(s[j][2] - base[1]), p3 = exp2f(s[j][3] - base[1]);
        l[0] += p0 + p1;
        l[1] += p2 + p3;
        pf[j * 2 + 0] = pack_bf16(p0, p1);
        pf[j * 2 + 1] = pack_bf16(p2, p3);
      }
      {
        const unsigned vbase = smem_u32(v_tile(stage));
        // the running maximum rarely moves once a slice is under way: skip the rescaling then
        if (!__all_sync(0xffffffffu, corr[0] == 1.f && corr[1] == 1.f)) {
#pragma unroll
          for (int j = 0; j < kOTiles; ++j) {
            o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1];
          }
        }
#pragma unroll
        for (int j = 0; j < kOTiles; j += 2) {
          unsigned b0, b1, b2, b3;   // (keys 0-7, d tile j), (keys 8-15, j), (keys 0-7, j+1), (keys 8-15, j+1)
          ldmatrix_x4_trans(b0, b1, b2, b3, vbase + (v_row_off + (((j ^ v_swz) & (HD / 8 - 1)) * 8)) * 2);
          mma_bf16(o[j], pf, b0, b1);
          mma_bf16(o[j + 1], pf, b2, b3);
        }
      }
      __syncwarp();   // all lanes are done reading this stage before it is refilled
      issue_next();   // keeps the ring full: goes into the stage just read
      stage = stage + 1 == kDecStages ? 0 : stage + 1;
    }
    cp_async_wait<0>();
  }

  // ---- partial result of this slice
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
  }
  const int col = (lane & 3) * 2;
  if (deposit) {
    // The CTAs of this (request, kv head) are one cluster. Output idx = head * HD + dim of the row belongs to
    // CTA (idx / 128) % csize. Every warp deposits its normalised partial with the owners of its outputs
    // (their receive buffer [pass][slice][128], behind the rings: a CTA may still be streaming when others
    // deposit) and its log-sum-exps with everyone; after ONE cluster barrier each CTA merges what it was
    // given, in slice order (the formula of attention_merge_kernel), and nobody touches remote memory again.
    cg::cluster_group cluster = cg::this_cluster();
    const int csize = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
    float* const recv_o = reinterpret_cast<float*>(smem_raw + (size_t)(kDecWarps * kDecStages * 2 * kDecKeys + 18) * HD * sizeof(bf16));
    const int passes = (group * HD + 128 * csize - 1) / (128 * csize);
    float* const recv_lse = recv_o + (size_t)passes * nsplits * 128;    // [slice][16]
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");   // phase 0: every CTA of the cluster runs
    if (split < nsplits) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = r_lo + 8 * i;
        if (r >= group) continue;
        const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
#pragma unroll
        for (int j = 0; j < kOTiles; ++j) {
          const int idx = r * HD + j * 8 + col;
          const int blk = idx >> 7;                      // which block of 128 outputs
          float* dst = cluster.map_shared_rank(recv_o, blk % csize) + ((size_t)(blk / csize) * nsplits + split) * 128 + (idx & 127);
          *reinterpret_cast<float2*>(dst) = make_float2(o[j][2 * i] * inv, o[j][2 * i + 1] * inv);
        }
        if ((lane & 3) == 0) {
          const float lse = l[i] > 0.f ? m[i] + log2f(l[i]) : -INFINITY;
          for (int q = 0; q < csize; ++q) cluster.map_shared_rank(recv_lse, q)[split * 16 + r] = lse;
        }
      }
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    for (int pass = 0; pass < passes; ++pass) {
      const int idx = (pass * csize + rank) * 128 + threadIdx.x;
      if (idx >= group * HD) break;
      const int r = idx / HD, d = idx - r * HD;
      float mx = -INFINITY;
      for (int sl = 0; sl < nsplits; ++sl) mx = fmaxf(mx, recv_lse[sl * 16 + r]);
      float acc = 0.f, wsum = 0.f;
      for (int sl = 0; sl < nsplits; ++sl) {
        const float lse = recv_lse[sl * 16 + r];
        const float w = lse == -INFINITY ? 0.f : exp2f(lse - mx);
        wsum += w;
        acc += w * recv_o[((size_t)pass * nsplits + sl) * 128 + threadIdx.x];
      }
      p.out[(size_t)row_q * p.out_row_stride + (size_t)(kvh * group + r) * HD + d] =
          __float2bfloat16_rn(wsum > 0.f ? acc / wsum : 0.f);
    }
    return;
  }
  if (p.merge_in_kernel) {
    // The CTAs of this (request, kv head) are one cluster. Every warp leaves its normalised partial
    // [group][HD] and log-sum-exps [group] in its own drained ring; then CTA r of the cluster merges
    // the outputs r * 128 + t, ... over all slices in slice order, reading the other CTAs' shared
    // memory directly (the formula of attention_merge_kernel, without the trip through global memory).
    float* my_o = reinterpret_cast<float*>(ring);
    float* my_lse = my_o + 16 * HD;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = r_lo + 8 * i;
      if (r >= group) continue;
      const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
#pragma unroll
      for (int j = 0; j < kOTiles; ++j)
        *reinterpret_cast<float2*>(my_o + r * HD + j * 8 + col) = make_float2(o[j][2 * i] * inv, o[j][2 * i + 1] * inv);
      if ((lane & 3) == 0) my_lse[r] = (split_ok && l[i] > 0.f) ? m[i] + log2f(l[i]) : -INFINITY;
    }
    cg::cluster_group cluster = cg::this_cluster();
    const int csize = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
    if (csize > 1) cluster.sync(); else __syncthreads();
    constexpr size_t kRingFloats = (size_t)kDecStages * 2 * kDecKeys * HD / 2;   // one warp's ring, in floats
    float* const cta_base = reinterpret_cast<float*>(smem_raw);
    for (int idx = rank * (kDecWarps * 32) + threadIdx.x; idx < group * HD; idx += csize * kDecWarps * 32) {
      const int r = idx / HD, d = idx - r * HD;
      float mx = -INFINITY;
      for (int sl = 0; sl < nsplits; ++sl) {
        const float* base = csize > 1 ? cluster.map_shared_rank(cta_base, sl / kDecWarps) : cta_base;
        mx = fmaxf(mx, base[(sl % kDecWarps) * kRingFloats + 16 * HD + r]);
      }
      float acc = 0.f, wsum = 0.f;
      for (int sl = 0; sl < nsplits; ++sl) {
        const float* base = (csize > 1 ? cluster.map_shared_rank(cta_base, sl / kDecWarps) : cta_base) + (sl % kDecWarps) * kRingFloats;
        const float lse = base[16 * HD + r];
        const float w = lse == -INFINITY ? 0.f : exp2f(lse - mx);
        wsum += w;
        acc += w * base[r * HD + d];
      }
      p.out[(size_t)row_q * p.out_row_stride + (size_t)(kvh * group + r) * HD + d] =
          __float2bfloat16_rn(wsum > 0.f ? acc / wsum : 0.f);
    }
    if (csize > 1) cluster.sync();   // nobody leaves while its shared memory may still be read
    return;
  }
  if (!split_ok) return;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = r_lo + 8 * i;
    if (r >= group) continue;
    const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
    const size_t slot = ((size_t)row_q * p.nq + kvh * group + r) * p.max_splits + split;
    float* op = p.part_o + slot * HD + col;
#pragma unroll
    for (int j = 0; j < kOTiles; ++j)
      *reinterpret_cast<float2*>(op + j * 8) = make_float2(o[j][2 * i] * inv, o[j][2 * i + 1] * inv);
    if ((lane & 3) == 0) p.part_lse[slot] = l[i] > 0.f ? m[i] + log2f(l[i]) : -INFINITY;
  }
}

// out[token, head] = sum_s w_s o_s / sum_s w_s with w_s = 2^(lse_s - max lse). One warp per
// (token, head): the lanes fetch the slices' log-sum-exps side by side (up to kMaxMergeSlices), and the
// partial outputs are read eight slices at a time so that the loads overlap.
constexpr int kMaxMergeSlices = 128;
template <int HD>
__global__ void attention_merge_kernel(bf16* __restrict__ out, int out_row_stride, const float* __restrict__ part_o,
                                       const float* __restrict__ part_lse, const int* __restrict__ row_splits,
                                       int nq, int max_splits, int tokens) {
  pdl_start();
  const int lane = threadIdx.x & 31;
  const long long gw = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gw >= (long long)tokens * nq) return;
  const int token = (int)(gw / nq), head = (int)(gw % nq);
  const int ns = row_splits[token];
  if (ns <= 1) return;  // written directly by the attention kernel
  const size_t base = ((size_t)token * nq + head) * max_splits;
  constexpr int kPer = HD / 32;
  constexpr int kLaneSlices = kMaxMergeSlices / 32;
  float acc[kPer];
#pragma unroll
  for (int e = 0; e < kPer; ++e) acc[e] = 0.f;
  // ns <= kMaxMergeSlices (checked by the entry points): lane i holds slices i, i + 32, i + 64, i + 96
  float lse[kLaneSlices], w[kLaneSlices];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < kLaneSlices; ++j) {
    lse[j] = 32 * j + lane < ns ? part_lse[base + 32 * j + lane] : -INFINITY;
    mx = fmaxf(mx, lse[j]);
  }
  mx = warp_max(mx);
  float wsum = 0.f;
#pragma unroll
  for (int j = 0; j < kLaneSlices; ++j) {
    w[j] = lse[j] == -INFINITY ? 0.f : exp2f(lse[j] - mx);
    wsum += w[j];
  }
  wsum = warp_sum(wsum);
  for (int s = 0; s < ns; s += 8) {
    float v[8][kPer];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (s + u < ns) {
        const float* op = part_o + (base + s + u) * HD + lane * kPer;
#pragma unroll
        for (int e = 0; e < kPer; ++e) v[u][e] = op[e];
      }
    }
    // the eight slices of a round lie in one block of 32: the same register of every lane holds their weights
    float wj = w[0];
#pragma unroll
    for (int j = 1; j < kLaneSlices; ++j) wj = (s >> 5) == j ? w[j] : wj;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int idx = s + u;
      const float ws = __shfl_sync(0xffffffffu, wj, idx & 31);
      if (idx < ns) {
#pragma unroll
        for (int e = 0; e < kPer; ++e) acc[e] += ws * v[u][e];
      }
    }
  }
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  bf16* dst = out + (size_t)token * out_row_stride + (size_t)head * HD + lane * kPer;
#pragma unroll
  for (int e = 0; e < kPer; ++e) dst[e] = __float2bfloat16_rn(acc[e] * inv);
}

template <int HD, int MT>
int launch_tiles(const AttnParams& p, int num_items, cudaStream_t s) {
  constexpr int smem = (64 * MT + 4 * kKeys) * HD * (int)sizeof(bf16);
  static bool configured = false;
  if (!configured) {
    OI_CHECK_CUDA(cudaFuncSetAttribute(attention_mma_kernel<HD, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  oi_launch(attention_mma_kernel<HD, MT>, (unsigned)((long long)num_items * p.nkv), kThreads, smem, s, p);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

template <int HD>
int launch(const AttnParams& p, int num_items, const int* row_splits, int tokens, int any_split, int rows_per_cta,
           cudaStream_t s) {
  const int rc = rows_per_cta == 128 ? launch_tiles<HD, 2>(p, num_items, s) : launch_tiles<HD, 1>(p, num_items, s);
  if (rc) return rc;
  if (any_split) {
    const long long warps = (long long)tokens * p.nq;
    oi_launch(attention_merge_kernel<HD>, (unsigned)((warps + 3) / 4), 128, 0, s, 
        p.out, p.out_row_stride, p.part_o, p.part_lse, row_splits, p.nq, p.max_splits, tokens);
    OI_CHECK_LAUNCH();
  }
  return OI_OK;
}

template <int HD>
int launch_merge(void* out, int out_row_stride, const float* part_o, const float* part_lse, const int* row_splits, int nq,
                 int max_splits, int tokens, cudaStream_t s) {
  const long long warps = (long long)tokens * nq;
  oi_launch(attention_merge_kernel<HD>, (unsigned)((warps + 3) / 4), 128, 0, s, (bf16*)out, out_row_stride, part_o, part_lse,
            row_splits, nq, max_splits, tokens);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

template <int HD>
int launch_decode(const AttnParams& p, int num_items, const int* row_splits, int tokens, cudaStream_t s) {
  // the warps' rings, room for the rotated query heads of one kv head and the step's key and value
  // (fuse_rope), and the receive buffer of the merge by deposit
  constexpr int kRecvMax = 12 * 1024;
  constexpr int smem = (kDecWarps * kDecStages * 2 * kDecKeys + 18) * HD * (int)sizeof(bf16) + kRecvMax;
  static bool configured = false;
  if (!configured) {
    OI_CHECK_CUDA(cudaFuncSetAttribute(attention_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  dim3 grid(num_items, p.nkv);
  if (p.merge_in_kernel) {
    // deposit when the receive buffer fits: [passes][slices][128] floats and [slices][16] log-sum-exps
    const int csize = p.max_splits / kDecWarps;
    const int passes = (p.group * HD + 128 * csize - 1) / (128 * csize);
    AttnParams q = p;
    q.merge_in_kernel = (csize > 1 && (passes * p.max_splits * 128 + p.max_splits * 16) * 4 <= kRecvMax) ? 2 : 1;
    oi_launch_cluster(attention_decode_kernel<HD>, grid, kDecWarps * 32, smem, s, csize, q);
    OI_CHECK_LAUNCH();
    return OI_OK;
  }
  oi_launch(attention_decode_kernel<HD>, grid, kDecWarps * 32, smem, s, p);
  OI_CHECK_LAUNCH();
  const long long warps = (long long)tokens * p.nq;
  oi_launch(attention_merge_kernel<HD>, (unsigned)((warps + 3) / 4), 128, 0, s,
      p.out, p.out_row_stride, p.part_o, p.part_lse, row_splits, p.nq, p.max_splits, tokens);
  OI_CHECK_LAUNCH();
  return OI_OK;
}

}  // namespace

namespace {
struct RopeArgs {
  const void* q_norm_w; const void* k_norm_w; int norm_dtype; float eps, w_offset;
  const float* cos_tab; const float* sin_tab; int rot_half, max_pos;
  const int* positions; const int* slots; int write_kv;
};

int decode_entry(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_cache,
                 const void* v_cache, long long page_stride, int page_size, const int* block_table,
                 int bt_stride, const int* cu_seqlens, const int* kv_lens, const int* items,
                 int num_items, const int* row_splits, int tokens, int nq, int nkv, int hd,
                 float scale, int window, float* part_o, float* part_lse, int max_splits,
                 int merge_in_kernel, const RopeArgs* rope, void* stream) {
  OI_REQUIRE(hd == 32 || hd == 64 || hd == 128, "attention_decode: head_dim %d not covered (32, 64 or 128)", hd);
  OI_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0 && nq / nkv <= 16, "attention_decode: group %d/%d not covered (<= 16)", nq, nkv);
  OI_REQUIRE(q_row_stride % 2 == 0 && page_stride % 8 == 0, "attention_decode: misaligned strides");
  OI_REQUIRE(((uintptr_t)q % 4 == 0) && ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0),
             "attention_decode: misaligned pointers");
  if (merge_in_kernel) {
    OI_REQUIRE(max_splits >= 4 && max_splits <= 32 && max_splits % 4 == 0 && num_items % (max_splits / 4) == 0,
               "attention_decode: %d slices cannot be merged in the kernel (a multiple of 4 up to 32)", max_splits);
    OI_REQUIRE((uintptr_t)out % 2 == 0, "attention_decode: misaligned output");
  } else {
    OI_REQUIRE(part_o && part_lse && row_splits && max_splits >= 2 && max_splits <= kMaxMergeSlices,
               "attention_decode: scratch missing, or slices outside 2..%d", kMaxMergeSlices);
  }
  if (num_items == 0 || tokens == 0) return OI_OK;
  AttnParams p;
  p.q = (const bf16*)q; p.q_row_stride = q_row_stride;
  p.out = (bf16*)out; p.out_row_stride = out_row_stride;
  p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
  p.page_stride = page_stride; p.page_size = page_size;
  p.block_table = block_table; p.bt_stride = bt_stride;
  p.cu_seqlens = cu_seqlens; p.kv_lens = kv_lens; p.items = (const int4*)items;
  p.nq = nq; p.nkv = nkv; p.group = nq / nkv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window;
  p.part_o = part_o; p.part_lse = part_lse; p.max_splits = max_splits;
  p.merge_in_kernel = merge_in_kernel ? 1 : 0;
  p.fuse_rope = 0;
  if (rope) {
    OI_REQUIRE(rope->rot_half > 0 && rope->rot_half % 2 == 0 && 2 * rope->rot_half <= hd && rope->cos_tab && rope->sin_tab &&
                   rope->max_pos > 0 && rope->positions,
               "attention_decode: rotation tables, positions and an even rotary half <= head_dim / 2 are needed (half %d)", rope->rot_half);
    OI_REQUIRE(!rope->write_kv || rope->slots, "attention_decode: cache write without slots");
    OI_REQUIRE(q_row_stride % 8 == 0 && (uintptr_t)q % 16 == 0, "attention_decode: the fused projection's rows must be 16-byte aligned");
    OI_REQUIRE((rope->q_norm_w == nullptr) == (rope->k_norm_w == nullptr) || !rope->write_kv,
               "attention_decode: q and k norm weights come together");
    p.fuse_rope = 1; p.write_kv = rope->write_kv ? 1 : 0;
    p.q_norm_w = rope->q_norm_w; p.k_norm_w = rope->k_norm_w; p.norm_dtype = rope->norm_dtype;
    p.eps = rope->eps; p.w_offset = rope->w_offset;
    p.cos_tab = rope->cos_tab; p.sin_tab = rope->sin_tab; p.rot_half = rope->rot_half; p.max_pos = rope->max_pos;
    p.positions = rope->positions; p.slots = rope->slots;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (hd == 32) return launch_decode<32>(p, num_items, row_splits, tokens, s);
  if (hd == 64) return launch_decode<64>(p, num_items, row_splits, tokens, s);
  return launch_decode<128>(p, num_items, row_splits, tokens, s);
}
}  // namespace

// Decode rows only (requests that bring one token): items are (request, 0, first slice, nsplits),
// one CTA per four consecutive slices, every item with nsplits == max_splits. With
// merge_in_kernel != 0 (max_splits a multiple of 4, at most 32; the items of a request adjacent
// and in slice order) the max_splits / 4 CTAs of a row run as a thread-block cluster and merge their
// slices through distributed shared memory; part_o, part_lse and row_splits are not used. Otherwise
// every listed request's row is merged by a second kernel from scratch in global memory, so
// row_splits[row] must be nsplits (>= 2) for those rows and <= 1 for all others.
OI_API int oi_attention_decode(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_cache,
                               const void* v_cache, long long page_stride, int page_size, const int* block_table,
                               int bt_stride, const int* cu_seqlens, const int* kv_lens, const int* items,
                               int num_items, const int* row_splits, int tokens, int nq, int nkv, int hd,
                               float scale, int window, float* part_o, float* part_lse, int max_splits,
                               int merge_in_kernel, void* stream) {
  return decode_entry(q, q_row_stride, out, out_row_stride, k_cache, v_cache, page_stride, page_size, block_table, bt_stride,
                      cu_seqlens, kv_lens, items, num_items, row_splits, tokens, nq, nkv, hd, scale, window, part_o, part_lse,
                      max_splits, merge_in_kernel, nullptr, stream);
}

// The same with the per-head q/k norm, the rotation and the write of the step's key and value fused in:
// `qkv` is the raw fused projection [rows, >= (nq + 2 nkv) * hd] (only the nq query heads when write_kv
// is 0: a call that reads another call's cache), norm weights [hd] of norm_dtype or null, cos/sin float32
// [max_pos, rot_half], positions and slots int32 [rows] (a slot < 0 stores nothing). q is not written back.
OI_API int oi_attention_decode_rope(const void* qkv, int q_row_stride, void* out, int out_row_stride, void* k_cache,
                                    void* v_cache, long long page_stride, int page_size, const int* block_table,
                                    int bt_stride, const int* cu_seqlens, const int* kv_lens, const int* items,
                                    int num_items, const int* row_splits, int tokens, int nq, int nkv, int hd,
                                    float scale, int window, float* part_o, float* part_lse, int max_splits,
                                    int merge_in_kernel, const void* q_norm_w, const void* k_norm_w, int norm_dtype,
                                    float eps, float w_offset, const float* cos_tab, const float* sin_tab, int rot_half,
                                    int max_pos, const int* positions, const int* slots, int write_kv, void* stream) {
  RopeArgs r{q_norm_w, k_norm_w, norm_dtype, eps, w_offset, cos_tab, sin_tab, rot_half, max_pos, positions, slots, write_kv};
  return decode_entry(qkv, q_row_stride, out, out_row_stride, k_cache, v_cache, page_stride, page_size, block_table, bt_stride,
                      cu_seqlens, kv_lens, items, num_items, row_splits, tokens, nq, nkv, hd, scale, window, part_o, part_lse,
                      max_splits, merge_in_kernel, &r, stream);
}

// items: int32 [num_items, 4] = (request, first token of the tile, split, nsplits), planned by the
// host for tiles of rows_per_cta (64 or 128) query rows = rows_per_cta / group tokens. row_splits: int32 [tokens], the number of slices each row's keys were cut into.
// part_o: float32 [tokens * nq * max_splits * hd], part_lse: float32 [tokens * nq * max_splits]
// (only touched by rows with more than one slice).
OI_API int oi_attention_mma(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_cache,
                            const void* v_cache, long long page_stride, int page_size, const int* block_table,
                            int bt_stride, const int* cu_seqlens, const int* kv_lens, const int* items,
                            int num_items, const int* row_splits, int tokens, int any_split, int nq, int nkv,
                            int hd, float scale, int window, float* part_o, float* part_lse, int max_splits,
                            int rows_per_cta, void* stream) {
  OI_REQUIRE(rows_per_cta == 64 || rows_per_cta == 128, "attention_mma: rows_per_cta %d (64 or 128)", rows_per_cta);
  OI_REQUIRE(hd == 32 || hd == 64 || hd == 128, "attention_mma: head_dim %d not covered (32, 64 or 128)", hd);
  OI_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0 && nq / nkv <= rows_per_cta, "attention_mma: bad head counts nq=%d nkv=%d", nq, nkv);
  OI_REQUIRE(q_row_stride % 2 == 0 && out_row_stride % 2 == 0 && page_stride % 8 == 0, "attention_mma: misaligned strides");
  OI_REQUIRE(((uintptr_t)q % 4 == 0) && ((uintptr_t)out % 4 == 0) && ((uintptr_t)k_cache % 16 == 0) && ((uintptr_t)v_cache % 16 == 0),
             "attention_mma: misaligned pointers");
  OI_REQUIRE(!any_split || (part_o && part_lse && row_splits && max_splits > 0 && max_splits <= 64),
             "attention_mma: split items without scratch, or more than 64 slices");
  if (num_items == 0 || tokens == 0) return OI_OK;
  AttnParams p;
  p.q = (const bf16*)q; p.q_row_stride = q_row_stride;
  p.out = (bf16*)out; p.out_row_stride = out_row_stride;
  p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
  p.page_stride = page_stride; p.page_size = page_size;
  p.block_table = block_table; p.bt_stride = bt_stride;
  p.cu_seqlens = cu_seqlens; p.kv_lens = kv_lens; p.items = (const int4*)items;
  p.nq = nq; p.nkv = nkv; p.group = nq / nkv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window;
  p.part_o = part_o; p.part_lse = part_lse; p.max_splits = max_splits;
  p.merge_in_kernel = 0;
  p.fuse_rope = 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (hd == 32) return launch<32>(p, num_items, row_splits, tokens, any_split, rows_per_cta, s);
  if (hd == 64) return launch<64>(p, num_items, row_splits, tokens, any_split, rows_per_cta, s);
  return launch<128>(p, num_items, row_splits, tokens, any_split, rows_per_cta, s);
}

// Merge the slices that another attention kernel left in scratch (the layout of oi_attention_mma's part_o and
// part_lse): rows whose row_splits entry is above one get out = sum_s w_s o_s / sum_s w_s.
OI_API int oi_attention_merge_slices(void* out, int out_row_stride, const float* part_o, const float* part_lse,
                                     const int* row_splits, int nq, int max_splits, int tokens, int hd, void* stream) {
  OI_REQUIRE(out && part_o && part_lse && row_splits && tokens >= 0 && nq > 0 && max_splits >= 1 && max_splits <= kMaxMergeSlices,
             "attention_merge: bad arguments");
  if (tokens == 0) return OI_OK;
  cudaStream_t s = (cudaStream_t)stream;
  if (hd == 128) return launch_merge<128>(out, out_row_stride, part_o, part_lse, row_splits, nq, max_splits, tokens, s);
  if (hd == 64) return launch_merge<64>(out, out_row_stride, part_o, part_lse, row_splits, nq, max_splits, tokens, s);
  if (hd == 32) return launch_merge<32>(out, out_row_stride, part_o, part_lse, row_splits, nq, max_splits, tokens, s);
  OI_REQUIRE(false, "attention_merge: head_dim %d not covered (32, 64, 128)", hd);
}
