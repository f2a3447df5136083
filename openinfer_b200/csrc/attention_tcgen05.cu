// Causal paged GQA attention for prompt portions on the 5th-generation tensor cores (bfloat16,
// head_dim 128): S = Q K^T and O_tile = P V run as tcgen05.mma with their results in tensor memory;
// Q, K and V tiles are fetched by TMA, K and V straight out of the cache pages.
//
// A CTA owns 128 query rows of one (request, kv head): row r is (token r / group, head r % group),
// as in the mma.sync kernels. Roles:
//   warp 0      producer: the Q tile once (two 128 x 64 boxes out of the projection buffer, rows
//               ordered token-major by a 3-D box), then per 64-key tile the K and V boxes of the pages
//               the block table names (4-D maps over the layer's cache; one box for the whole tile when
//               the tile's pages have consecutive ids). Each box is issued by a lane
//               of its own (a box of one 16-key page costs about 90 cycles of issue, one after the
//               other from a single thread), page ids are read 32 at a time one round ahead, and K
//               and V have barriers of their own: a K stage is free as soon as S has been computed
//               from it, so the next K tiles never wait for a P V product;
//   warp 1      MMA issuer: per tile S = Q K^T (M 128, N 64, K 128: 8 instructions, both operands
//               K-major in shared memory), and, once the softmax warps have put P into shared memory,
//               O += P V (M 128, N 128, K 64: 4 instructions, V read MN-major as it lies in its page),
//               accumulated in tensor memory over all tiles;
//   warps 2-5   one thread per query row: reads its row of S from tensor memory, masks, keeps the
//               running maximum and sum in float32 (no shuffles: the row is the thread's own) and writes
//               P as bfloat16 into the swizzled shared tile (the exponentials are computed into
//               registers first, beside the previous tile's P V product, and stored once that product
//               has released the tile). P is taken relative to a REFERENCE maximum
//               that is only moved when the true maximum has outgrown it by a factor 2^8; only then is
//               the accumulator in tensor memory rescaled (load, multiply, store). At the end the
//               thread reads its output row, divides by the sum and stores it.
// S is double buffered so that the next tile's S is computed while this tile's softmax runs; two
// CTAs fit on an SM (112 KB of shared memory, 256 columns of tensor memory each) and fill each
// other's gaps. Every mbarrier wait is bounded (two seconds): a wait that runs out sets an error word
// and a flag that ends all roles, after which the CTA frees its tensor memory and returns.
// No load uses cluster multicast.
//
// Math as the other attention kernels: s = (q . k) / sqrt(hd) for keys j <= pos (and j > pos - window),
// softmax in float32 with exp2 and the scale folded in, o = sum p v
// (pegainfer-kernels/csrc/shared/paged_attention.cu:439-567).
#include "oi_api.h"
#include "tcgen05.cuh"

namespace {

constexpr int HD = 128;
constexpr int kRows = 128;          // query rows per CTA
constexpr int kKeys = 64;           // keys per tile
constexpr int kStages = 2;
constexpr int kThreads = 192;

__device__ int g_attn_error = 0;

struct Params {
  const int4* items;        // (request, first token of the tile, slice of its keys, slices)
  const int* cu_seqlens;
  const int* kv_lens;
  const int* block_table;
  int bt_stride;
  int page_size, box_keys;  // keys per TMA box = min(page_size, 64)
  int num_pages;
  int run_boxes;            // maps over runs of 64 / page_size neighbouring pages exist (pages of fewer than 64 keys)
  int nq, nkv, group;
  float scale_log2;
  int window;
  bf16* out;
  int out_row_stride;
  float* part_o;            // partial results of tiles whose keys are cut into slices (see oi_attention_mma)
  float* part_lse;
  int max_splits;
};

using namespace tc;

__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag, int code) {
  return tc::mbar_wait(bar, parity, abort_flag, &g_attn_error, code);
}
__device__ __forceinline__ void tc_fence_before() { tc::fence_before(); }
__device__ __forceinline__ void tc_fence_after() { tc::fence_after(); }
__device__ __forceinline__ unsigned long long desc_k_major(unsigned smem_addr) { return tc::desc_k_major_sw128(smem_addr); }
__device__ __forceinline__ unsigned long long desc_mn_major(unsigned smem_addr, unsigned lbo_bytes) {
  return tc::desc_mn_major_sw128(smem_addr, lbo_bytes);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// the largest of three values in one instruction (sm_100)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// shared memory map (bytes from a 1024-aligned base)
constexpr int kQBytes = kRows * HD * 2;            // 32 KB: two halves [128 rows][64 dims]
constexpr int kKBytes = kKeys * HD * 2;            // 16 KB: two halves [64 keys][64 dims]
constexpr int kVBytes = kKeys * HD * 2;            // 16 KB
constexpr int kPBytes = kRows * kKeys * 2;         // 16 KB: [128 rows][64 keys]
constexpr int kOffK = kQBytes;
constexpr int kOffV = kOffK + kStages * kKBytes;
constexpr int kOffP = kOffV + kStages * kVBytes;
constexpr int kOffBar = kOffP + kPBytes;
// barriers: q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full, o_full
constexpr int kNumBars = 1 + 4 * kStages + 2 + 2;
constexpr float kRescaleThreshold = 8.f;           // in log2 units: P stays below 2^8
constexpr int kSmemTotal = kOffBar + kNumBars * 8 + 16;   // 112 KB + barriers: two CTAs per SM
constexpr unsigned kTmemCols = 256;                // S0 [0,64) S1 [64,128) O_tile [128,256)

__global__ void __launch_bounds__(kThreads)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_k_run,
                         const __grid_constant__ CUtensorMap map_v_run, const Params p) {
  pdl_start();
  // the swizzled tiles need a 1024-byte aligned base; no slack is added for it (two CTAs must fit on an SM)
  extern __shared__ __align__(1024) unsigned char smem[];
  const unsigned sbase = smem_u32(smem);
  if (sbase & 1023u) {                 // never seen; refuse rather than compute garbage
    if (threadIdx.x == 0) atomicCAS(&g_attn_error, 0, 9);
    return;
  }
  const unsigned bar0 = sbase + kOffBar;
  const unsigned q_full = bar0;
  auto k_full = [&](int s) { return bar0 + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar0 + 8u * (1 + kStages + s); };
  auto v_full = [&](int s) { return bar0 + 8u * (1 + 2 * kStages + s); };
  auto v_empty = [&](int s) { return bar0 + 8u * (1 + 3 * kStages + s); };
  auto s_full = [&](int b) { return bar0 + 8u * (1 + 4 * kStages + b); };
  const unsigned p_full = bar0 + 8u * (3 + 4 * kStages);
  const unsigned o_full = bar0 + 8u * (4 + 4 * kStages);
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(smem + kOffBar + kNumBars * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int4 item = p.items[blockIdx.x / p.nkv];
  const int req = item.x, tok0 = item.y;
  const int kvh = blockIdx.x % p.nkv;
  const int group = p.group;
  const int q_start = p.cu_seqlens[req];
  const int q_len = p.cu_seqlens[req + 1] - q_start;
  const int kv_len = p.kv_lens[req];
  const int toks_per_tile = kRows / group;
  const int tile_toks = min(toks_per_tile, q_len - tok0);
  const int pos0 = kv_len - q_len + tok0;
  int lo = 0;
  if (p.window > 0) lo = max(0, pos0 - p.window + 1);
  lo &= ~(kKeys - 1);
  const int hi = pos0 + tile_toks;
  // An item may cover a slice of the tile's keys (when whole tiles would leave SMs idle): key tiles
  // [t_begin, t_end) of the span, cut as in the mma.sync kernel; its result goes to scratch, normalised and with
  // its log-sum-exp, and a second kernel merges the slices.
  const int split = item.z, nsplits = item.w > 1 ? item.w : 1;
  const int span_tiles = (hi - lo + kKeys - 1) / kKeys;
  const int tiles_per_split = (span_tiles + nsplits - 1) / nsplits;
  const int t_begin = min(span_tiles, split * tiles_per_split);
  const int num_tiles = min(span_tiles, t_begin + tiles_per_split) - t_begin;
  lo += t_begin * kKeys;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(k_full(s), 1); mbar_init(k_empty(s), 1);
      mbar_init(v_full(s), 1); mbar_init(v_empty(s), 1);
    }
    mbar_init(s_full(0), 1);
    mbar_init(s_full(1), 1);
    mbar_init(p_full, 4);      // one arrival per softmax warp
    mbar_init(o_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (the whole warp runs the loop)
    if (lane == 0) {
      // Q: rows (token, head) of this kv head's group; box (64 dims, group heads, 128 / group tokens)
      mbar_expect_tx(q_full, kQBytes);
      tma_load_3d(sbase, &map_q, 0, kvh * group, q_start + tok0, q_full);
      tma_load_3d(sbase + kQBytes / 2, &map_q, 64, kvh * group, q_start + tok0, q_full);
    }
    const int* bt = p.block_table + (size_t)req * p.bt_stride;
    const int boxes = kKeys / p.box_keys;
    // Page ids come 32 boxes at a time, one per lane and one round ahead of their use, so that no copy
    // waits for a read of the block table.
    auto pages_of_round = [&](int round) {
      const int key = lo + (round * 32 + lane) * p.box_keys;
      int col = key / p.page_size;
      col = col < p.bt_stride ? col : p.bt_stride - 1;           // keys past the request are masked anyway
      const int page = bt[col];
      return page < 0 ? 0 : (page >= p.num_pages ? p.num_pages - 1 : page);
    };
    int pages_now = pages_of_round(0), pages_next = pages_of_round(1);
    bool ok = true;
    for (int t = 0; t < num_tiles; ++t) {
      const int s = t % kStages;
      const int key0 = lo + t * kKeys;
      int my_page[4];                                           // boxes <= 4 (pages of 16 keys and more)
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int g = t * boxes + b;
        if (b < boxes) {
          if ((g & 31) == 0 && g > 0) { pages_now = pages_next; pages_next = pages_of_round((g >> 5) + 1); }
          my_page[b] = __shfl_sync(0xffffffffu, pages_now, g & 31);
        }
      }
      // Pages whose ids follow one another (as a fresh pool hands them out) lie side by side in the cache: the
      // tile's keys are then ONE box over `boxes` pages, and one copy per half of the head dims does what otherwise
      // takes a copy per page. With pages of 16 keys the copy unit is otherwise the bound: 16 boxes per tile and CTA.
      bool run = p.run_boxes != 0;
#pragma unroll
      for (int b = 1; b < 4; ++b)
        if (b < boxes) run = run && my_page[b] == my_page[0] + b;
      // every lane below 2 * boxes issues one copy of K and one of V: (box, half of the head dims)
      const int my_box = run ? 0 : lane >> 1, my_half = lane & 1;
      const int copies = run ? 2 : 2 * boxes;
      int page = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) page = my_box == b ? my_page[b] : page;
      const int in_page = (key0 + my_box * p.box_keys) & (p.page_size - 1);
      const unsigned off = (unsigned)(my_box * p.box_keys) * 128u + (unsigned)my_half * (kKBytes / 2);   // rows of 128 bytes
      const unsigned k_dst = sbase + kOffK + s * kKBytes + off, v_dst = sbase + kOffV + s * kVBytes + off;
      if (t >= kStages) ok = mbar_wait(k_empty(s), (unsigned)((t / kStages) - 1) & 1, abort_flag, 1);
      if (!ok) break;
      if (lane == 0) mbar_expect_tx(k_full(s), kKBytes);
      __syncwarp();
      if (lane < copies) tma_load_4d(k_dst, run ? &map_k_run : &map_k, my_half * 64, kvh, in_page, page, k_full(s));
      if (t >= kStages) ok = mbar_wait(v_empty(s), (unsigned)((t / kStages) - 1) & 1, abort_flag, 5);
      if (!ok) break;
      if (lane == 0) mbar_expect_tx(v_full(s), kVBytes);
      __syncwarp();
      if (lane < copies) tma_load_4d(v_dst, run ? &map_v_run : &map_v, my_half * 64, kvh, in_page, page, v_full(s));
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // S: D f32, A = Q (bf16, K-major), B = K (bf16, K-major), M 128, N 64
      constexpr unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(kKeys >> 3) << 17) | ((unsigned)(kRows >> 4) << 24);
      // O_tile: A = P (K-major), B = V (MN-major: bit 16), M 128, N 128
      constexpr unsigned idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(HD >> 3) << 17) | ((unsigned)(kRows >> 4) << 24);
      bool ok = mbar_wait(q_full, 0, abort_flag, 2);
      auto issue_s = [&](int t) {   // S(t) = Q K(t)^T into S buffer t & 1
        const int s = t % kStages;
        if (!mbar_wait(k_full(s), (unsigned)(t / kStages) & 1, abort_flag, 3)) return false;
        tc_fence_after();
        const unsigned k_addr = sbase + kOffK + s * kKBytes;
        const unsigned tmem_s = tmem + (unsigned)((t & 1) * kKeys);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          // 16 dims = 32 bytes along the swizzle row; dims 64.. are in the second half tile
          const unsigned a = sbase + (k >= 4 ? kQBytes / 2 : 0) + (k & 3) * 32;
          const unsigned b = k_addr + (k >= 4 ? kKBytes / 2 : 0) + (k & 3) * 32;
          umma_bf16(tmem_s, desc_k_major(a), desc_k_major(b), idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(s_full(t & 1));
        umma_commit(k_empty(s));        // K(t) has been read: its stage may be refilled
        return true;
      };
      if (ok && num_tiles > 0) ok = issue_s(0);
      for (int t = 0; t < num_tiles && ok; ++t) {
        if (t + 1 < num_tiles) {        // the next S is computed while this tile's softmax runs
          ok = issue_s(t + 1);
          if (!ok) break;
        }
        const int s = t % kStages;
        ok = mbar_wait(v_full(s), (unsigned)(t / kStages) & 1, abort_flag, 10) &&
             mbar_wait(p_full, (unsigned)t & 1, abort_flag, 4);   // P(t) is in shared memory, O is rescaled
        if (!ok) break;
        tc_fence_after();
        const unsigned v_addr = sbase + kOffV + s * kVBytes;
        const unsigned p_addr = sbase + kOffP;
#pragma unroll
        for (int k = 0; k < kKeys / 16; ++k) {
          // A: P rows of 128 bytes (64 keys), 16 keys = 32 bytes along the row
          // B: V, 16 keys = two 8-key groups = 2048 bytes further; the second 64 dims kVBytes / 2 away
          umma_bf16(tmem + 128u, desc_k_major(p_addr + k * 32), desc_mn_major(v_addr + k * 2048, kVBytes / 2), idesc_o,
                    (t | k) != 0 ? 1u : 0u);
        }
        umma_commit(o_full);
        umma_commit(v_empty(s));        // V(t) has been read
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax: one row per thread
    const int quarter = warp & 3;                       // TMEM lanes [32 * quarter, +32)
    const int r = quarter * 32 + lane;                  // query row of this thread
    const int t_row = r / group;
    const bool row_ok = t_row < tile_toks;
    const int pos = pos0 + t_row;
    const unsigned lane_base = tmem + ((unsigned)(quarter * 32) << 16);
    float m_ref = -INFINITY;                            // the maximum P is taken relative to (raw score units)
    float l = 0.f;
    unsigned char* p_row = smem + kOffP + r * 128;      // this row of the P tile (128 bytes, swizzled chunks)
    bool ok = true;
    for (int t = 0; t < num_tiles && ok; ++t) {
      const int key0 = lo + t * kKeys;
      ok = mbar_wait(s_full(t & 1), (unsigned)(t >> 1) & 1, abort_flag, 6);
      if (!ok) break;
      tc_fence_after();
      float sv[kKeys];
      {
        unsigned v0[32], v1[32];
        tmem_ld32(lane_base + (unsigned)((t & 1) * kKeys), v0);
        tmem_ld32(lane_base + (unsigned)((t & 1) * kKeys + 32), v1);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) { sv[e] = __uint_as_float(v0[e]); sv[32 + e] = __uint_as_float(v1[e]); }
      }
      const bool full = row_ok && key0 + kKeys - 1 <= pos && (p.window <= 0 || key0 > pos - p.window);
      if (!full) {
#pragma unroll
        for (int e = 0; e < kKeys; ++e) {
          const int key = key0 + e;
          const bool vis = row_ok && key <= pos && (p.window <= 0 || key > pos - p.window);
          sv[e] = vis ? sv[e] : -INFINITY;
        }
      }
      // The softmax warps are bound by the instructions they issue (a cubic exponential on the multiply-add pipe beside
      // the special-function unit's made long prompts 6 % slower), so the row's arithmetic uses the instructions that
      // do two things at once: three-input maxima, and multiply-adds and additions on PAIRS of float32.
      // row maximum with eight independent chains (a single chain of 64 would be pure latency)
      float mx[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) mx[e] = sv[e];
#pragma unroll
      for (int e = 8; e < kKeys - 8; e += 16)
#pragma unroll
        for (int c = 0; c < 8; ++c) mx[c] = max3(mx[c], sv[e + c], sv[e + 8 + c]);
#pragma unroll
      for (int c = 0; c < 8; ++c) mx[c] = fmaxf(mx[c], sv[kKeys - 8 + c]);
      const float m_tile = fmaxf(max3(mx[0], mx[1], mx[2]), max3(max3(mx[3], mx[4], mx[5]), mx[6], mx[7]));
      // move the reference only when the maximum has outgrown it by 2^8 (or there is none yet)
      const bool move = m_tile > m_ref && (m_ref == -INFINITY || (m_tile - m_ref) * p.scale_log2 > kRescaleThreshold);
      // P(t) = 2^(s * scale - m_ref * scale), rounded to bfloat16, kept in registers: the second product
      // of the previous tile still reads the P tile, and this arithmetic runs beside it
      const bool rescale = move && t > 0 && m_ref != -INFINITY;
      const float f = rescale ? fast_exp2((m_ref - m_tile) * p.scale_log2) : 1.f;
      if (move) m_ref = m_tile;
      const float base = m_ref == -INFINITY ? 0.f : m_ref * p.scale_log2;
      float2 lsum[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
      const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), nbase2 = make_float2(-base, -base);
      uint4 chunks[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&chunks[c]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x = __ffma2_rn(make_float2(sv[c * 8 + 2 * e], sv[c * 8 + 2 * e + 1]), scale2, nbase2);
          const float2 pp = make_float2(fast_exp2(x.x), fast_exp2(x.y));
          lsum[e] = __fadd2_rn(lsum[e], pp);
          h[e] = __floats2bfloat162_rn(pp.x, pp.y);
        }
      }
      const float2 lsum_all = __fadd2_rn(__fadd2_rn(lsum[0], lsum[1]), __fadd2_rn(lsum[2], lsum[3]));
      l = l * f + (lsum_all.x + lsum_all.y);
      // the second product of the previous tile reads the P tile and updates O until o_full(t - 1)
      if (t > 0) {
        ok = mbar_wait(o_full, (unsigned)(t - 1) & 1, abort_flag, 7);
        if (!ok) break;
        tc_fence_after();
      }
      if (__any_sync(0xffffffffu, rescale)) {
        // rescale this warp's rows of the accumulator in tensor memory (factor 1 for rows that stay)
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
          unsigned v[32];
          tmem_ld32(lane_base + 128u + (unsigned)c, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * f);
          asm volatile(
              "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
              "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
              "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
              ::"r"(lane_base + 128u + (unsigned)c), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
                "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
                "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]),
                "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]) : "memory");
        }
        asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(p_row + ((c ^ (r & 7)) << 4)) = chunks[c];
      // make the generic-proxy writes of P visible to the tensor core (async proxy), then hand over
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (nsplits > 1) {
      // a slice: the normalised partial result in float32 and the base-2 log-sum-exp of its keys
      bool have = ok && num_tiles > 0;
      if (have) {
        have = mbar_wait(o_full, (unsigned)(num_tiles - 1) & 1, abort_flag, 8);
        tc_fence_after();
      }
      const float inv = (have && l > 0.f) ? 1.f / l : 0.f;
      const size_t slot = ((size_t)(q_start + tok0 + t_row) * p.nq + (size_t)(kvh * group + r % group)) * p.max_splits + split;
      float* dst = p.part_o + slot * HD;
#pragma unroll 1
      for (int c = 0; c < HD; c += 32) {
        unsigned v[32];
        if (have) {                    // uniform in the warp: the waits above are the same for all its lanes
          tmem_ld32(lane_base + 128u + (unsigned)c, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4)
            reinterpret_cast<float4*>(dst + c)[q4] = make_float4(__uint_as_float(v[q4 * 4]) * inv, __uint_as_float(v[q4 * 4 + 1]) * inv,
                                                               __uint_as_float(v[q4 * 4 + 2]) * inv, __uint_as_float(v[q4 * 4 + 3]) * inv);
        }
      }
      if (row_ok) p.part_lse[slot] = (have && l > 0.f) ? m_ref * p.scale_log2 + log2f(l) : -INFINITY;
    } else if (ok && num_tiles > 0) {
      ok = mbar_wait(o_full, (unsigned)(num_tiles - 1) & 1, abort_flag, 8);
      if (ok) {
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        bf16* dst = p.out + (size_t)(q_start + tok0 + t_row) * p.out_row_stride + (size_t)(kvh * group + r % group) * HD;
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
          unsigned v[32];
          tmem_ld32(lane_base + 128u + (unsigned)c, v);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 o;
              __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int e = 0; e < 4; ++e)
                h[e] = __floats2bfloat162_rn(__uint_as_float(v[q4 * 8 + 2 * e]) * inv, __uint_as_float(v[q4 * 8 + 2 * e + 1]) * inv);
              reinterpret_cast<uint4*>(dst + c)[q4] = o;
            }
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);   // let copies in flight land
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace

// Prompt tiles of 128 query rows; items as for oi_attention_mma with rows_per_cta 128, key slices included
// (any_split != 0: some item covers a slice; part_o float32 [tokens * nq * max_splits * 128] and part_lse
// [tokens * nq * max_splits] take the slices' results and a second kernel merges them by row_splits). Requirements (else the caller uses the mma.sync kernel): head_dim 128, 128 % group == 0,
// page_size a power of two >= 16 (64 % page_size == 0 or page_size % 64 == 0), 16-byte aligned
// buffers with row strides that are multiples of 8 elements. q: [tokens, q_row_stride] (heads of
// 128 from column 0); cache: [num_pages, page_size, nkv, 128] with page_stride elements per page.
OI_API int oi_attention_tcgen05(const void* q, long long q_row_stride, int tokens, void* out, int out_row_stride,
                                const void* k_cache, const void* v_cache, long long page_stride, int page_size,
                                int num_pages, const int* block_table, int bt_stride, const int* cu_seqlens,
                                const int* kv_lens, const int* items, int num_items, int nq, int nkv, int hd,
                                float scale, int window, const int* row_splits, int any_split, float* part_o,
                                float* part_lse, int max_splits, void* stream) {
  OI_REQUIRE(hd == HD, "attention_tcgen05: head_dim %d not covered (128)", hd);
  OI_REQUIRE(!any_split || (part_o && part_lse && row_splits && max_splits >= 2 && max_splits <= 64 && (uintptr_t)part_o % 16 == 0),
             "attention_tcgen05: key slices need 16-byte aligned scratch, the rows' slice counts and 2..64 slices");
  OI_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0 && kRows % (nq / nkv) == 0, "attention_tcgen05: group %d/%d not covered", nq, nkv);
  OI_REQUIRE(page_size >= 16 && (page_size & (page_size - 1)) == 0, "attention_tcgen05: page size %d not covered", page_size);
  OI_REQUIRE(q_row_stride % 8 == 0 && page_stride % 8 == 0 && out_row_stride % 8 == 0 && (uintptr_t)q % 16 == 0 &&
                 (uintptr_t)k_cache % 16 == 0 && (uintptr_t)v_cache % 16 == 0 && (uintptr_t)out % 16 == 0,
             "attention_tcgen05: misaligned operands");
  if (num_items == 0 || tokens == 0) return OI_OK;
  tc::EncodeTiledFn enc = tc::encode_fn();
  OI_REQUIRE(enc != nullptr, "attention_tcgen05: cuTensorMapEncodeTiled is not available from this driver");
  const int group = nq / nkv;
  const int box_keys = page_size < kKeys ? page_size : kKeys;
  CUtensorMap mq, mk, mv, mk_run, mv_run;
  const int boxes = kKeys / box_keys;
  const int run_boxes = (boxes > 1 && num_pages >= boxes) ? 1 : 0;
  {
    cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)nq, (cuuint64_t)tokens};
    cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)q_row_stride * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)group, (cuuint32_t)(kRows / group)};
    cuuint32_t es[3] = {1, 1, 1};
    CUresult r = enc(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    OI_REQUIRE(r == CUDA_SUCCESS, "attention_tcgen05: tensor map for q failed (%d)", (int)r);
  }
  for (int which = 0; which < 4; ++which) {   // K, V; then K, V with a box over a run of pages
    const bool v = (which & 1) != 0, wide = which >= 2;
    CUtensorMap* m = wide ? (v ? &mv_run : &mk_run) : (v ? &mv : &mk);
    if (wide && !run_boxes) {
      *m = v ? mv : mk;   // never used
      continue;
    }
    cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)nkv, (cuuint64_t)page_size, (cuuint64_t)num_pages};
    cuuint64_t strides[3] = {(cuuint64_t)HD * 2, (cuuint64_t)nkv * HD * 2, (cuuint64_t)page_stride * 2};
    cuuint32_t box[4] = {64, 1, (cuuint32_t)box_keys, (cuuint32_t)(wide ? boxes : 1)};
    cuuint32_t es[4] = {1, 1, 1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(v ? v_cache : k_cache),
                     dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    OI_REQUIRE(r == CUDA_SUCCESS, "attention_tcgen05: tensor map for the cache failed (%d)", (int)r);
  }
  Params p;
  p.items = (const int4*)items; p.cu_seqlens = cu_seqlens; p.kv_lens = kv_lens;
  p.block_table = block_table; p.bt_stride = bt_stride;
  p.page_size = page_size; p.box_keys = box_keys; p.num_pages = num_pages; p.run_boxes = run_boxes;
  p.nq = nq; p.nkv = nkv; p.group = group;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window;
  p.out = (bf16*)out; p.out_row_stride = out_row_stride;
  p.part_o = part_o; p.part_lse = part_lse; p.max_splits = any_split ? max_splits : 1;
  static bool configured = false;
  if (!configured) {
    OI_CHECK_CUDA(cudaFuncSetAttribute(attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal));
    configured = true;
  }
  oi_launch(attention_tcgen05_kernel, (unsigned)((long long)num_items * nkv), kThreads, kSmemTotal, (cudaStream_t)stream, mq, mk, mv, mk_run, mv_run, p);
  OI_CHECK_LAUNCH();
  if (any_split) return oi_attention_merge_slices(out, out_row_stride, part_o, part_lse, row_splits, nq, max_splits, tokens, hd, stream);
  return OI_OK;
}

OI_API int oi_attention_tcgen05_status(int* status) {
  int v = 0;
  OI_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_attn_error, sizeof(int)));
  if (v != 0) {
    int zero = 0;
    OI_CHECK_CUDA(cudaMemcpyToSymbol(g_attn_error, &zero, sizeof(int)));
  }
  *status = v;
  return OI_OK;
}
