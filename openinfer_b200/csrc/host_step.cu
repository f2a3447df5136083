// The host side of a step in native code: which kernel takes which product, the gated feed-forward,
// one layer's attention, and the whole stack of layers of a step (see oi_api.h).
//
// The reference's step is native host code that launches one kernel after the other
// (pegainfer-qwen3/src/executor.rs:365-620, unified_forward.rs:383-611); so is this. Everything here only
// chooses and launches: the kernels are the ones in the other files of this folder, called through
// their checked entry points.
#include "oi_api.h"

namespace {

int g_opt[OI_OPT_COUNT] = {0, 0, 0, 0, 129, 0};
constexpr int kDecodeMaxRows = 32;    // rows up to which the streaming product takes a product
constexpr int kSkinnyMaxRows = 16;
constexpr int kFusedMinRows = 128;    // rows from which gate/up forms the activation in the tcgen05 product's epilogue
constexpr int kPair = 0;              // tile_n value that stands for 256 x 256 tiles of a pair of CTAs

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      n = 148;
  }
  return n;
}

// operands that TMA can fetch: rows contiguous in k, 16-byte aligned bases and row strides
bool tma_ok(const void* x, long long ldx, const void* w, long long ldw, int K) {
  return K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0;
}

// How many K slices (CTAs per cluster) the streaming kernel uses: one when the tiles of 128 weight rows alone
// fill the GPU, else the fewest slices that give every SM a CTA, each slice at least two k blocks long.
// Measured on B200 at M = 8 (us, inside a CUDA graph): N 6144 K 4096: 14.2 with 4 slices (16.1 with 2, 17.0
// with 8); N 4096 K 4096: 11.1 with 8 (11.8 with 4); N 4096 K 12288: 20.9 with 8 (22.1 with 4); N 24576 and
// N 151936: one slice (34.4 and 188).
int stream_slices(int N, int K) {
  const int tiles = (N + 127) / 128, num_kb = (K + 63) / 64;
  int c = 1;
  while (c < 8 && tiles * c < sm_count() && num_kb / (2 * c) >= 2) c *= 2;
  if (g_opt[OI_OPT_FORCE_SLICES] > 0) c = g_opt[OI_OPT_FORCE_SLICES];
  while (c > 1 && (c - 1) * ((num_kb + c - 1) / c) >= num_kb) c /= 2;   // no slice may be left without a k block
  return c;
}

// K slices of the mma.sync decode product, 0 if it does not take the shape (a slice's activations must fit in
// shared memory beside the 48 KB of weight rings). Four slices measured best for the short products.
int skinny_slices(int K) {
  auto fits = [&](int c) { return K % (32 * c) == 0 && 49152 + 32 * (K / c + 64) + 4096 <= 200 * 1024; };
  int chosen = 0;
  for (int c : {4, 2, 8, 1})
    if (fits(c)) {
      chosen = c;
      break;
    }
  const int forced = g_opt[OI_OPT_FORCE_SLICES];
  if (chosen && (forced == 1 || forced == 2 || forced == 4 || forced == 8) && fits(forced)) chosen = forced;
  return chosen;
}

int linear_bf16(void* out, int out_dtype, long long ldc, const void* x, long long ldx, const void* W, long long ldw, int M,
                int N, int K, void* stream) {
  const bool tma = tma_ok(x, ldx, W, ldw, K);
  if (g_opt[OI_OPT_BATCH_INVARIANT]) {
    // one kernel for every step shape: a row's sums are formed in the same order whatever else is in the step
    OI_REQUIRE(tma, "linear: batch-invariant products need 16-byte aligned bfloat16 operands with K %% 8 == 0");
    return oi_gemm_tcgen05(out, out_dtype, ldc, x, ldx, W, ldw, M, N, K, 256, OI_ACT_NONE, stream);
  }
  const int decode_gemm = g_opt[OI_OPT_DECODE_GEMM];
  if (M <= kDecodeMaxRows) {
    if (decode_gemm == 0 && tma)
      return oi_gemm_stream(out, out_dtype, ldc, x, ldx, W, ldw, M, N, K, stream_slices(N, K), OI_ACT_NONE, stream);
    if (decode_gemm <= 1 && M <= kSkinnyMaxRows && tma && K >= 32) {
      const int c = skinny_slices(K);
      if (c) return oi_gemm_skinny(out, out_dtype, ldc, x, ldx, W, ldw, M, N, K, 0, 0, c, stream);
    }
  }
  if (M >= g_opt[OI_OPT_PAIR_MIN_ROWS] && g_opt[OI_OPT_PREFILL_GEMM] == 1 && tma)
    return oi_gemm_tcgen05_pair(out, out_dtype, ldc, x, ldx, W, ldw, M, N, K, OI_ACT_NONE, stream);
  if (oi_library_gemm_ready()) {
    if (oi_library_gemm(out, out_dtype, ldc, x, ldx, W, ldw, M, N, K, stream) == OI_OK) return OI_OK;
  }
  // without the vendor library (or for a shape it has no algorithm for): the hand-written kernels
  if (tma) {
    if (M >= g_opt[OI_OPT_PAIR_MIN_ROWS]) return oi_gemm_tcgen05_pair(out, out_dtype, ldc, x, ldx, W, ldw, M, N, K, OI_ACT_NONE, stream);
    return oi_gemm_tcgen05(out, out_dtype, ldc, x, ldx, W, ldw, M, N, K, 256, OI_ACT_NONE, stream);
  }
  return oi_gemm_generic(out, out_dtype, x, OI_BF16, W, OI_BF16, M, N, K, ldx, ldw, ldc, stream);
}

#define OI_TRY(expr)                  \
  do {                                \
    const int rc__ = (expr);          \
    if (rc__ != OI_OK) return rc__;   \
  } while (0)

}  // namespace

OI_API int oi_configure(int option, int value) {
  OI_REQUIRE(option >= 0 && option < OI_OPT_COUNT, "configure: unknown option %d", option);
  g_opt[option] = value;
  return OI_OK;
}

OI_API int oi_option(int option) { return option >= 0 && option < OI_OPT_COUNT ? g_opt[option] : -1; }

OI_API int oi_stream_slices(int N, int K) { return stream_slices(N, K); }

OI_API int oi_linear(void* out, int out_dtype, long long ldc, const void* x, int x_dtype, long long ldx, const void* W,
                     int w_dtype, long long ldw, int M, int N, int K, void* stream) {
  OI_REQUIRE(M >= 0 && N > 0 && K > 0, "linear: bad sizes M=%d N=%d K=%d", M, N, K);
  if (M == 0) return OI_OK;
  if (x_dtype == OI_BF16 && w_dtype == OI_BF16) return linear_bf16(out, out_dtype, ldc, x, ldx, W, ldw, M, N, K, stream);
  // anything with a float32 operand: float32 accumulation on the ordinary pipes, k ascending
  return oi_gemm_generic(out, out_dtype, x, x_dtype, W, w_dtype, M, N, K, ldx, ldw, ldc, stream);
}

namespace {
// 2: the tcgen05 product forms the activation in its epilogue; 1: the streaming product does; 0: nobody does
int gated_mlp_fusion(int dtype, int w_dtype, int M, int hidden, int inter, int act_block, const void* x, const void* w) {
  if (dtype != OI_BF16 || w_dtype != OI_BF16 || act_block != 64) return 0;
  const bool tma = tma_ok(x, hidden, w, hidden, hidden);
  if ((M >= kFusedMinRows || g_opt[OI_OPT_BATCH_INVARIANT]) && inter % 128 == 0) return tma ? 2 : 0;
  if (!g_opt[OI_OPT_BATCH_INVARIANT] && g_opt[OI_OPT_DECODE_GEMM] == 0 && M > 0 && M <= kDecodeMaxRows && tma &&
      (2 * inter) % 128 == 0)
    return 1;
  return 0;
}
}  // namespace

OI_API int oi_gated_mlp_needs_gate_up(int dtype, int w_dtype, int M, int hidden, int inter, int act_block) {
  // for 16-byte aligned operands, which is what this package's buffers and weights are
  return gated_mlp_fusion(dtype, w_dtype, M, hidden, inter, act_block, nullptr, nullptr) == 0 ? 1 : 0;
}

OI_API int oi_gated_mlp(void* out, const void* x, int dtype, int M, int hidden, int inter, const void* w_gate_up,
                        int w_dtype, const void* w_down, int w_down_dtype, int act, int act_block, void* act_buf,
                        void* gate_up_buf, void* stream) {
  OI_REQUIRE(M >= 0 && hidden > 0 && inter > 0, "gated_mlp: bad sizes M=%d hidden=%d inter=%d", M, hidden, inter);
  OI_REQUIRE(act == OI_ACT_SILU || act == OI_ACT_GELU_TANH, "gated_mlp: unknown activation code %d", act);
  OI_REQUIRE(act_block > 0 && inter % act_block == 0, "gated_mlp: block %d does not divide inter %d", act_block, inter);
  if (M == 0) return OI_OK;
  const int fusion = gated_mlp_fusion(dtype, w_dtype, M, hidden, inter, act_block, x, w_gate_up);
  if (fusion == 2) {
    // Short sums (K <= 2048) of fewer than 2,048 rows stay with single CTAs: a tile's products are then no longer than
    // its epilogue, which the pairs' larger tile does not hide, and there are too few of the larger tiles to go round.
    const bool pairs = M >= g_opt[OI_OPT_PAIR_MIN_ROWS] && (hidden > 2048 || M >= 2048);
    const int tile = g_opt[OI_OPT_BATCH_INVARIANT] ? 256 : (pairs ? kPair : 256);
    if (tile == kPair)
      OI_TRY(oi_gemm_tcgen05_pair(act_buf, OI_BF16, inter, x, hidden, w_gate_up, hidden, M, 2 * inter, hidden, act, stream));
    else
      OI_TRY(oi_gemm_tcgen05(act_buf, OI_BF16, inter, x, hidden, w_gate_up, hidden, M, 2 * inter, hidden, tile, act, stream));
  } else if (fusion == 1) {
    OI_TRY(oi_gemm_stream(act_buf, OI_BF16, inter, x, hidden, w_gate_up, hidden, M, 2 * inter, hidden,
                          stream_slices(2 * inter, hidden), act, stream));
  } else {
    OI_REQUIRE(gate_up_buf != nullptr, "gated_mlp: this shape needs the gate|up scratch buffer");
    OI_TRY(oi_linear(gate_up_buf, dtype, 2 * inter, x, dtype, hidden, w_gate_up, w_dtype, hidden, M, 2 * inter, hidden, stream));
    OI_TRY(oi_silu_mul(act_buf, gate_up_buf, dtype, M, inter, act_block, act, stream));
  }
  return oi_linear(out, dtype, hidden, act_buf, dtype, inter, w_down, w_down_dtype, inter, M, hidden, inter, stream);
}

OI_API int oi_attention_layer(const OiAttnStep* s, const OiAttnLayer* l, void* stream) {
  OI_REQUIRE(s && l, "attention_layer: null description");
  const int tokens = s->tokens;
  if (tokens == 0) return OI_OK;
  const bool fused = l->rope_mode == 1 && s->tensor_core && s->fuse_rope && !l->interleaved;
  OI_REQUIRE(l->qkv && l->out && l->k_cache && l->v_cache && s->block_table && s->kv_lens && s->cu_seqlens,
             "attention_layer: a tensor of the step or of the layer is missing");
  OI_REQUIRE(l->rope_mode == 0 || ((!l->write_kv || s->slot_mapping) && (!l->cos_tab || s->positions)),
             "attention_layer: the rotation and the cache write need the step's positions and slots");
  OI_REQUIRE(s->tensor_core || (s->token_req && s->positions), "attention_layer: the general kernel needs token_req and positions");
  if (l->rope_mode == 1 && !fused)
    OI_TRY(oi_qk_norm_rope_kv(l->qkv, l->dtype, l->q_row_stride, tokens, l->nq, l->nkv, l->hd, l->q_norm_w, l->k_norm_w,
                              l->norm_dtype, l->eps, l->w_offset, l->cos_tab, l->sin_tab, l->cos_tab ? l->rot_half : 0,
                              l->cos_tab ? l->max_pos : 0, s->positions, s->slot_mapping, l->k_cache, l->v_cache,
                              s->page_stride, s->page_size, l->write_kv, l->interleaved, stream));
  if (!s->tensor_core)
    return oi_attention_generic(l->qkv, l->q_row_stride, l->out, l->out_row_stride, l->dtype, l->k_cache, l->v_cache,
                                s->page_stride, s->page_size, s->block_table, s->bt_stride, s->token_req, s->positions,
                                tokens, l->nq, l->nkv, l->hd, l->scale, l->window, stream);
  if (fused) {
    OI_REQUIRE(s->num_tile_items == 0 && s->num_decode_items > 0, "attention_layer: the fused rotation needs a step of single tokens");
    return oi_attention_decode_rope(l->qkv, l->q_row_stride, l->out, l->out_row_stride, l->k_cache, l->v_cache, s->page_stride,
                                    s->page_size, s->block_table, s->bt_stride, s->cu_seqlens, s->kv_lens, s->decode_items,
                                    s->num_decode_items, s->row_splits, tokens, l->nq, l->nkv, l->hd, l->scale, l->window,
                                    s->part_o, s->part_lse, s->max_splits, s->merge_in_kernel, l->q_norm_w, l->k_norm_w,
                                    l->norm_dtype, l->eps, l->w_offset, l->cos_tab, l->sin_tab, l->rot_half, l->max_pos,
                                    s->positions, s->slot_mapping, l->write_kv, stream);
  }
  if (s->num_tile_items && s->use_tcgen05)
    OI_TRY(oi_attention_tcgen05(l->qkv, l->q_row_stride, tokens, l->out, l->out_row_stride, l->k_cache, l->v_cache,
                                s->page_stride, s->page_size, s->num_pages, s->block_table, s->bt_stride, s->cu_seqlens,
                                s->kv_lens, s->tile_items, s->num_tile_items, l->nq, l->nkv, l->hd, l->scale, l->window,
                                s->row_splits, s->tile_split, s->part_o, s->part_lse, s->max_splits, stream));
  else if (s->num_tile_items)
    OI_TRY(oi_attention_mma(l->qkv, l->q_row_stride, l->out, l->out_row_stride, l->k_cache, l->v_cache, s->page_stride,
                            s->page_size, s->block_table, s->bt_stride, s->cu_seqlens, s->kv_lens, s->tile_items,
                            s->num_tile_items, s->row_splits, tokens, s->tile_split, l->nq, l->nkv, l->hd, l->scale, l->window,
                            s->part_o, s->part_lse, s->max_splits, s->rows_per_cta, stream));
  if (s->num_decode_items)
    OI_TRY(oi_attention_decode(l->qkv, l->q_row_stride, l->out, l->out_row_stride, l->k_cache, l->v_cache, s->page_stride,
                               s->page_size, s->block_table, s->bt_stride, s->cu_seqlens, s->kv_lens, s->decode_items,
                               s->num_decode_items, s->row_splits, tokens, l->nq, l->nkv, l->hd, l->scale, l->window,
                               s->part_o, s->part_lse, s->max_splits, s->merge_in_kernel, stream));
  return OI_OK;
}

namespace {
// A decode-sized step without norm kernels inside the layer stack: the products that end a residual branch (O, down)
// add the residual and leave the next norm's inputs behind, the products that follow (gate/up, QKV) scale their
// rows (gemm_stream.cu). Taken, when switched on (OI_OPT_FUSE_NORM, off by default), for up to 32 rows of a bfloat16
// model whose weights are all bfloat16 and TMA-readable.
// Measured on B200, it is no gain: 5 instead of 7 kernels per layer, but Qwen3-8B sizes at batch 8 run 3.56 ms a step
// against 3.50 ms with the norm kernels (batch 1: 3.22 against 3.19; Qwen3-0.6B sizes, batch 8: 1.19 against 1.11).
// The norm kernel's 2-3 us are not idle time: under it the product behind it, already resident, fills its ring of
// weight tiles, which it can only do once the product before has left the SMs; without the norm kernel that filling
// stands in the open, and the products that end a branch are 1-3 us longer for the residual's round trip through L2.
bool fused_norm_step(const OiModelDesc* m, const OiStepDesc* st) {
  if (!g_opt[OI_OPT_FUSE_NORM] || g_opt[OI_OPT_BATCH_INVARIANT] || g_opt[OI_OPT_DECODE_GEMM] != 0) return false;
  if (st->tokens > kDecodeMaxRows || m->dtype != OI_BF16 || !st->xs || !st->ssq || m->hidden % 8) return false;
  if (st->ssq_stride % 4 || st->ssq_stride < 8 * ((m->hidden + 127) / 128)) return false;
  for (int i = 0; i < m->num_layers; ++i) {
    const OiLayerDesc& L = m->layers[i];
    const int q_dim = L.attn.nq * L.attn.hd;
    if (L.w_qkv_dtype != OI_BF16 || L.w_o_dtype != OI_BF16 || L.w_gate_up_dtype != OI_BF16 || L.w_down_dtype != OI_BF16) return false;
    if (L.act_block != 64 || (2 * L.inter) % 128 || L.inter % 8 || q_dim % 8) return false;
    if ((uintptr_t)L.w_qkv % 16 || (uintptr_t)L.w_o % 16 || (uintptr_t)L.w_gate_up % 16 || (uintptr_t)L.w_down % 16) return false;
  }
  return true;
}

int forward_fused_norm(const OiModelDesc* m, const OiStepDesc* st, void* stream) {
  const int T = st->tokens, H = m->hidden;
  __nv_bfloat16* h = (__nv_bfloat16*)st->h;
  __nv_bfloat16* xs = (__nv_bfloat16*)st->xs;
  const float inv_width = 1.f / (float)H;
  int units = 0;   // partial sums of squares that the last residual product left per row
  for (int i = 0; i < m->num_layers; ++i) {
    const OiLayerDesc& L = m->layers[i];
    OI_REQUIRE(L.attn_step >= 0 && L.attn_step < st->num_attn_steps, "forward: layer %d names attention step %d of %d", i,
               L.attn_step, st->num_attn_steps);
    const int q_dim = L.attn.nq * L.attn.hd;
    // ---- input norm + QKV
    if (i == 0) {
      OI_TRY(oi_rmsnorm(st->x, st->h, nullptr, OI_BF16, L.input_norm_w, L.input_norm_dtype, nullptr, T, H, L.input_eps,
                        L.input_offset, stream));
      OI_TRY(oi_gemm_stream(st->qkv, OI_BF16, L.qkv_rows, st->x, H, L.w_qkv, H, T, L.qkv_rows, H, stream_slices(L.qkv_rows, H),
                            OI_ACT_NONE, stream));
    } else {
      OiStreamEpilogue ep = {};
      ep.ssq_in = st->ssq, ep.ssq_units = units, ep.ssq_stride = st->ssq_stride, ep.inv_width = inv_width, ep.eps = L.input_eps;
      OI_TRY(oi_gemm_stream_fused(st->qkv, OI_BF16, L.qkv_rows, xs, H, L.w_qkv, H, T, L.qkv_rows, H,
                                  stream_slices(L.qkv_rows, H), OI_ACT_NONE, &ep, stream));
    }
    // ---- attention
    OiAttnLayer a = L.attn;
    a.qkv = st->qkv, a.q_row_stride = L.qkv_rows, a.out = st->attn, a.out_row_stride = q_dim, a.dtype = OI_BF16;
    OI_TRY(oi_attention_layer(&st->attn_steps[L.attn_step], &a, stream));
    // ---- O + residual, and what the post norm needs
    {
      const int c = stream_slices(H, q_dim);
      OiStreamEpilogue ep = {};
      ep.residual = h, ep.ld_residual = H, ep.norm_w = L.post_norm_w, ep.norm_w_bf16 = L.post_norm_dtype == OI_BF16;
      ep.w_offset = L.post_offset, ep.xs = xs, ep.ld_xs = H, ep.ssq_out = st->ssq, ep.ssq_stride = st->ssq_stride;
      OI_TRY(oi_gemm_stream_fused(h, OI_BF16, H, st->attn, q_dim, L.w_o, q_dim, T, H, q_dim, c, OI_ACT_NONE, &ep, stream));
      units = ((H + 127) / 128) * c;
    }
    // ---- post norm + gate/up with the activation
    {
      OiStreamEpilogue ep = {};
      ep.ssq_in = st->ssq, ep.ssq_units = units, ep.ssq_stride = st->ssq_stride, ep.inv_width = inv_width, ep.eps = L.post_eps;
      OI_TRY(oi_gemm_stream_fused(st->act, OI_BF16, L.inter, xs, H, L.w_gate_up, H, T, 2 * L.inter, H,
                                  stream_slices(2 * L.inter, H), L.act, &ep, stream));
    }
    // ---- down + residual, and what the next layer's input norm needs (the last layer: only the residual)
    {
      const int c = stream_slices(H, L.inter);
      OiStreamEpilogue ep = {};
      ep.residual = h, ep.ld_residual = H;
      if (i + 1 < m->num_layers) {
        const OiLayerDesc& next = m->layers[i + 1];
        ep.norm_w = next.input_norm_w, ep.norm_w_bf16 = next.input_norm_dtype == OI_BF16, ep.w_offset = next.input_offset;
        ep.xs = xs, ep.ld_xs = H, ep.ssq_out = st->ssq, ep.ssq_stride = st->ssq_stride;
      }
      OI_TRY(oi_gemm_stream_fused(h, OI_BF16, H, st->act, L.inter, L.w_down, L.inter, T, H, L.inter, c, OI_ACT_NONE, &ep, stream));
      units = ((H + 127) / 128) * c;
    }
  }
  return OI_OK;
}
}  // namespace

OI_API int oi_forward(const OiModelDesc* m, const OiStepDesc* st, void* stream) {
  OI_REQUIRE(m && st && m->layers && (st->num_attn_steps == 0 || st->attn_steps), "forward: null description");
  const int T = st->tokens, H = m->hidden, dt = m->dtype;
  OI_REQUIRE(T >= 0 && H > 0, "forward: bad sizes tokens=%d hidden=%d", T, H);
  if (T == 0) return OI_OK;
  OI_TRY(oi_embedding(st->h, dt, m->embedding, m->embedding_dtype, st->token_ids, T, H, m->vocab, stream));
  if (m->embedding_scale != 1.f) OI_TRY(oi_scale_cap(st->h, dt, (long long)T * H, m->embedding_scale, 0.f, stream));
  const void* pending = nullptr;   // the last branch output, added by the norm that reads the row next
  const bool fused = fused_norm_step(m, st);
  if (fused) OI_TRY(forward_fused_norm(m, st, stream));
  for (int i = 0; i < (fused ? 0 : m->num_layers); ++i) {
    const OiLayerDesc& L = m->layers[i];
    OI_REQUIRE(L.attn_step >= 0 && L.attn_step < st->num_attn_steps, "forward: layer %d names attention step %d of %d", i,
               L.attn_step, st->num_attn_steps);
    OI_TRY(oi_rmsnorm(st->x, st->h, pending, dt, L.input_norm_w, L.input_norm_dtype, nullptr, T, H, L.input_eps,
                      L.input_offset, stream));
    OI_TRY(oi_linear(st->qkv, dt, L.qkv_rows, st->x, dt, H, L.w_qkv, L.w_qkv_dtype, H, T, L.qkv_rows, H, stream));
    OiAttnLayer a = L.attn;
    const int q_dim = a.nq * a.hd;
    a.qkv = st->qkv;
    a.q_row_stride = L.qkv_rows;
    a.out = st->attn;
    a.out_row_stride = q_dim;
    a.dtype = dt;
    OI_TRY(oi_attention_layer(&st->attn_steps[L.attn_step], &a, stream));
    OI_TRY(oi_linear(st->branch_a, dt, H, st->attn, dt, q_dim, L.w_o, L.w_o_dtype, q_dim, T, H, q_dim, stream));
    OI_TRY(oi_rmsnorm(st->x, st->h, st->branch_a, dt, L.post_norm_w, L.post_norm_dtype, nullptr, T, H, L.post_eps,
                      L.post_offset, stream));
    OI_TRY(oi_gated_mlp(st->branch_m, st->x, dt, T, H, L.inter, L.w_gate_up, L.w_gate_up_dtype, L.w_down, L.w_down_dtype, L.act, L.act_block,
                        st->act, st->gate_up, stream));
    pending = st->branch_m;
  }
  if (st->num_want > 0) {
    OI_REQUIRE(st->want_rows && st->wanted && st->logits, "forward: wanted rows without buffers");
    OI_TRY(oi_rmsnorm(st->wanted, st->h, pending, dt, m->final_norm_w, m->final_norm_dtype, st->want_rows, st->num_want, H,
                      m->final_eps, m->final_offset, stream));
    OI_TRY(oi_linear(st->logits, OI_F32, m->vocab, st->wanted, dt, H, m->head, m->head_dtype, H, st->num_want, m->vocab, H, stream));
    if (m->logit_soft_cap > 0.f)
      OI_TRY(oi_scale_cap(st->logits, OI_F32, (long long)st->num_want * m->vocab, 1.f, m->logit_soft_cap, stream));
  }
  return OI_OK;
}
