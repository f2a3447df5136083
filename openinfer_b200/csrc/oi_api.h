// The C interface of the library: every entry point, and the structures of its host-side step code.
//
// All entry points return 0 on success or an error code (common.cuh); oi_last_error() gives the
// message. Pointers are device pointers unless said otherwise; `stream` is a cudaStream_t. Element
// type codes: OI_F32 = 0, OI_BF16 = 1. Activation codes: OI_ACT_NONE / OI_ACT_SILU / OI_ACT_GELU_TANH.
#pragma once

#include "common.cuh"

// What the streaming product can do where it adds up its K slices, to take the norm kernels out of a decode layer
// (gemm_stream.cu). All pointers are device pointers; a null `ssq_in` / `residual` switches the part off.
typedef struct OiStreamEpilogue {
  // the product FOLLOWS a norm whose weight is already in its input: row m of the sums is multiplied by
  // rsqrt(sum_u ssq_in[m * ssq_stride + u] * inv_width + eps), u < ssq_units
  const float* ssq_in;
  int ssq_units;
  int ssq_stride;              // floats between rows of the partial squares (both directions), a multiple of 4
  float inv_width, eps;
  // the product ENDS a residual branch: out[m, n] = round(residual[m, n] + sum) (out may be the residual itself), and
  // for the norm that reads the row next (xs null: none): xs[m, n] = round(out[m, n] * (w_offset + norm_w[n])) and
  // ssq_out[m * ssq_stride + tile * slices + slice] = the sum of out[m, n]^2 over the columns that slice of that tile owns
  const __nv_bfloat16* residual;
  long long ld_residual;
  const void* norm_w;
  int norm_w_bf16;
  float w_offset;
  __nv_bfloat16* xs;
  long long ld_xs;
  float* ssq_out;
} OiStreamEpilogue;

// argmax_noalloc.cu
OI_API int oi_argmax_noalloc(int* out, const float* logits, int rows, int vocab, long long row_stride, void* stream);

// attention_generic.cu
OI_API int oi_attention_generic(const void* q, int q_row_stride, void* out, int out_row_stride, int dtype, const void*
       k_cache, const void* v_cache, long long page_stride, int page_size, const int* block_table, int bt_stride,
       const int* token_req, const int* positions, int tokens, int nq, int nkv, int hd, float scale, int window, void*
       stream);

// attention_mma.cu
OI_API int oi_attention_decode(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_cache,
       const void* v_cache, long long page_stride, int page_size, const int* block_table, int bt_stride, const int*
       cu_seqlens, const int* kv_lens, const int* items, int num_items, const int* row_splits, int tokens, int nq, int
       nkv, int hd, float scale, int window, float* part_o, float* part_lse, int max_splits, int merge_in_kernel,
       void* stream);
OI_API int oi_attention_decode_rope(const void* qkv, int q_row_stride, void* out, int out_row_stride, void* k_cache,
       void* v_cache, long long page_stride, int page_size, const int* block_table, int bt_stride, const int*
       cu_seqlens, const int* kv_lens, const int* items, int num_items, const int* row_splits, int tokens, int nq, int
       nkv, int hd, float scale, int window, float* part_o, float* part_lse, int max_splits, int merge_in_kernel,
       const void* q_norm_w, const void* k_norm_w, int norm_dtype, float eps, float w_offset, const float* cos_tab,
       const float* sin_tab, int rot_half, int max_pos, const int* positions, const int* slots, int write_kv, void*
       stream);
OI_API int oi_attention_mma(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_cache, const
       void* v_cache, long long page_stride, int page_size, const int* block_table, int bt_stride, const int*
       cu_seqlens, const int* kv_lens, const int* items, int num_items, const int* row_splits, int tokens, int
       any_split, int nq, int nkv, int hd, float scale, int window, float* part_o, float* part_lse, int max_splits,
       int rows_per_cta, void* stream);

// attention_tcgen05.cu
OI_API int oi_attention_tcgen05(const void* q, long long q_row_stride, int tokens, void* out, int out_row_stride,
       const void* k_cache, const void* v_cache, long long page_stride, int page_size, int num_pages, const int*
       block_table, int bt_stride, const int* cu_seqlens, const int* kv_lens, const int* items, int num_items, int nq,
       int nkv, int hd, float scale, int window, const int* row_splits, int any_split, float* part_o, float* part_lse,
       int max_splits, void* stream);
OI_API int oi_attention_merge_slices(void* out, int out_row_stride, const float* part_o, const float* part_lse,
       const int* row_splits, int nq, int max_splits, int tokens, int hd, void* stream);
OI_API int oi_attention_tcgen05_status(int* status);

// elementwise.cu
OI_API int oi_embedding(void* out, int out_dtype, const void* table, int table_dtype, const int* ids, int tokens, int
       hidden, int vocab, void* stream);
OI_API int oi_gather_tokens(int* ids, const int* src, const int* from, int n, int n_from, void* stream);
OI_API int oi_copy_words(int* dst, const int* src, int n, int ids_off, int src_off, int n_ids, const int* from, int
       n_from, void* stream);
OI_API int oi_rmsnorm(void* out, void* x, const void* delta, int dtype, const void* w, int w_dtype, const int*
       row_idx, int rows, int hidden, float eps, float w_offset, void* stream);
OI_API int oi_add_inplace(void* x, const void* delta, int dtype, long long n, void* stream);
OI_API int oi_scale_cap(void* x, int dtype, long long n, float scale, float cap, void* stream);
OI_API int oi_silu_mul(void* out, const void* gate_up, int dtype, int rows, int inter, int block, int act, void*
       stream);

// gemm_generic.cu
OI_API int oi_gemm_generic(void* C, int c_dtype, const void* A, int a_dtype, const void* W, int w_dtype, int M, int N,
       int K, long long lda, long long ldw, long long ldc, void* stream);

// gemm_skinny.cu
OI_API int oi_gemm_skinny(void* out, int out_dtype, long long ldc, const void* x, long long ldx, const void* W, long
       long ldw, int M, int N, int K, int silu_mul, int act, int cluster_size, void* stream);

// gemm_stream.cu
OI_API int oi_gemm_stream(void* out, int out_dtype, long long ldc, const void* x, long long ldx, const void* W, long
       long ldw, int M, int N, int K, int cluster_size, int act, void* stream);
OI_API int oi_gemm_stream_fused(void* out, int out_dtype, long long ldc, const void* x, long long ldx, const void* W,
       long long ldw, int M, int N, int K, int cluster_size, int act, const OiStreamEpilogue* epilogue, void* stream);
OI_API int oi_gemm_stream_status(int* status);

// gemm_tcgen05.cu
OI_API int oi_gemm_tcgen05(void* C, int c_dtype, long long ldc, const void* A, long long lda, const void* W, long long
       ldw, int M, int N, int K, int tile_n, int act, void* stream);
OI_API int oi_gemm_tcgen05_pair(void* C, int c_dtype, long long ldc, const void* A, long long lda, const void* W, long
       long ldw, int M, int N, int K, int act, void* stream);
OI_API int oi_gemm_tcgen05_status(int* status);

// rope_kv.cu
OI_API int oi_qk_norm_rope_kv(void* qkv, int dtype, int row_stride, int tokens, int nq, int nkv, int hd, const void*
       q_norm_w, const void* k_norm_w, int norm_dtype, float eps, float w_offset, const float* cos_tab, const float*
       sin_tab, int rot_half, int max_pos, const int* positions, const int* slots, void* k_cache, void* v_cache, long
       long page_stride, int page_size, int write_kv, int interleaved, void* stream);

// runtime.cu
OI_API const char* oi_last_error();
OI_API int oi_abi_version();
OI_API unsigned long long oi_launches();
OI_API int oi_launch_fence();   // the next kernel launched by this library gets plain stream order (once)
OI_API int oi_set_pdl(int enabled);
OI_API int oi_device_info(int device, int* sm_major, int* sm_minor, int* sm_count, long long* l2_bytes);

// sampling.cu
OI_API int oi_argmax_chunks(int vocab);
OI_API int oi_argmax(int* out, const float* logits, int rows, int vocab, long long row_stride, float* partial_vals,
       int* partial_idx, void* stream);
OI_API int oi_sample_use_clusters(int on);
OI_API int oi_sample(int* out, const float* logits, long long row_stride, float* probs, int rows, int vocab, const
       float* temperature, const int* top_k, const float* top_p, const float* min_p, const float* uniform, void*
       stream);
OI_API int oi_token_logprobs(const float* logits, long long row_stride, int vocab, const int* rows, const int* picked,
       const int* ks, int n, int k_max, float* out_lp, float* top_vals, int* top_ids, void* stream);

// library_gemm.cu
OI_API int oi_library_gemm_ready();
OI_API int oi_library_gemm_init(const char* path, void* workspace, long long workspace_bytes);
OI_API int oi_library_gemm(void* out, int out_dtype, long long ldc, const void* x, long long ldx, const void* W,
       long long ldw, int M, int N, int K, void* stream);

// ------------------------------------------------------------------------------------------------
// host_step.cu: the host side of a step in native code. Which kernel takes which product, the gated
// feed-forward, one layer's attention, and the whole stack of layers of a model assembled from this
// package's own parts. The Python parts call the first three one by one (so a model that mixes them
// with parts of its own runs the same code); a model made of package parts only runs the fourth, one
// call for all layers of a step.
// ------------------------------------------------------------------------------------------------

// Options of the dispatch (oi_configure): values are ints.
enum : int {
  OI_OPT_BATCH_INVARIANT = 0,   // 1: every choice depends on the request alone (one product kernel for all shapes)
  OI_OPT_DECODE_GEMM = 1,       // products of up to 32 rows: 0 streaming tcgen05 kernel, 1 mma.sync kernel, 2 library
  OI_OPT_PREFILL_GEMM = 2,      // plain products of more rows: 0 library, 1 the pair kernel of gemm_tcgen05.cu
  OI_OPT_FORCE_SLICES = 3,      // > 0: K slices of the decode products, whatever the shape (measurements)
  OI_OPT_PAIR_MIN_ROWS = 4,     // rows from which the fused gate/up product uses pairs of CTAs
  OI_OPT_FUSE_NORM = 5,         // 1: steps of up to 32 rows run without norm kernels inside the layer stack (oi_forward);
                                // off by default: measured slower, see host_step.cu
  OI_OPT_COUNT = 6,
};
OI_API int oi_configure(int option, int value);
OI_API int oi_option(int option);

// y[M, N] = x[M, K] W[N, K]^T by the kernel that the operand types, the shape and the options select.
OI_API int oi_linear(void* out, int out_dtype, long long ldc, const void* x, int x_dtype, long long ldx, const void* W,
       int w_dtype, long long ldw, int M, int N, int K, void* stream);
// How many K slices the streaming product uses for a shape (what oi_linear passes to oi_gemm_stream).
OI_API int oi_stream_slices(int N, int K);

// down( act(gate x) * (up x) ): out[M, hidden]. w_gate_up [2 inter, hidden] with rows in blocks of `act_block`
// gate rows followed by the up rows of the same indices; w_down [hidden, inter]. Scratch: `act_buf` [M, inter]
// and `gate_up_buf` [M, 2 inter] in x's type (the second is only written when no kernel forms the activation
// inside the product; it may be null if the caller knows that, see oi_gated_mlp_needs_gate_up).
OI_API int oi_gated_mlp(void* out, const void* x, int dtype, int M, int hidden, int inter, const void* w_gate_up,
       int w_gate_up_dtype, const void* w_down, int w_down_dtype, int act, int act_block, void* act_buf,
       void* gate_up_buf, void* stream);
OI_API int oi_gated_mlp_needs_gate_up(int dtype, int w_dtype, int M, int hidden, int inter, int act_block);

// What one step's attention calls share, per cache group and attention geometry: the step's metadata on the
// device and the work items planned on the host.
typedef struct OiAttnStep {
  const int* slot_mapping;   // [tokens] page * page_size + offset where the row's key and value go, -1: nowhere
  const int* block_table;    // [requests, bt_stride]
  const int* kv_lens;        // [requests]
  const int* cu_seqlens;     // [requests + 1]
  const int* token_req;      // [tokens]
  const int* positions;      // [tokens]
  int bt_stride, tokens, page_size, num_pages;
  long long page_stride;     // elements between pages of a layer's K (and V) tensor
  int tensor_core;           // 0: the general kernel; 1: the tile / decode kernels below
  int use_tcgen05;           // prompt tiles go to the tcgen05 kernel (else mma.sync)
  int fuse_rope;             // the decode kernel normalises, rotates and stores (single-token steps)
  const int* tile_items;     // [num_tile_items, 4]
  const int* decode_items;   // [num_decode_items, 4]
  const int* row_splits;     // [tokens]
  int num_tile_items, num_decode_items, rows_per_cta, tile_split, max_splits, merge_in_kernel;
  float* part_o;             // partial results of key slices that are merged by a second kernel (or null)
  float* part_lse;
} OiAttnStep;

// One layer's (more exactly: one run-order entry's) attention.
typedef struct OiAttnLayer {
  void* qkv;                 // [tokens, q | k | v] raw projections (q only when write_kv is 0 and rope_mode is 0)
  void* out;                 // [tokens, nq * hd]
  void* k_cache;             // this layer's pages [pages, page_size, nkv, hd]
  void* v_cache;
  const void* q_norm_w;      // [hd] or null
  const void* k_norm_w;
  const float* cos_tab;      // [max_pos, rot_half] or null
  const float* sin_tab;
  int q_row_stride, out_row_stride, dtype;
  int nq, nkv, hd, window;   // window 0: every key
  float scale, eps, w_offset;
  int norm_dtype, rot_half, max_pos;
  int interleaved;           // the rotation turns neighbours (2 d, 2 d + 1) instead of (d, d + half)
  int write_kv;              // the call owns its cache: keys and values of the step's rows are stored
  int rope_mode;             // 0: q is ready and the cache is written; 1: norm + rotation + cache write first (in its own
                             // kernel, or inside the decode kernel when the step says fuse_rope)
} OiAttnLayer;

OI_API int oi_attention_layer(const OiAttnStep* step, const OiAttnLayer* layer, void* stream);

// One entry of a model's run order, assembled from this package's parts: pre-norm block of attention and a
// gated feed-forward, each residual add carried out by the norm that follows.
typedef struct OiLayerDesc {
  const void* input_norm_w;
  const void* post_norm_w;
  const void* w_qkv;         // [qkv_rows, hidden]
  const void* w_o;           // [hidden, nq * hd]
  const void* w_gate_up;     // [2 inter, hidden]
  const void* w_down;        // [hidden, inter]
  OiAttnLayer attn;          // qkv / out are filled in per step
  int input_norm_dtype, post_norm_dtype, w_qkv_dtype, w_o_dtype, w_gate_up_dtype, w_down_dtype;
  float input_eps, input_offset, post_eps, post_offset;
  int qkv_rows;              // (nq + 2 nkv) * hd, or nq * hd when the entry reads another entry's cache
  int attn_step;             // which OiAttnStep of the step this entry uses
  int inter, act, act_block;
} OiLayerDesc;

typedef struct OiModelDesc {
  const OiLayerDesc* layers;  // host pointer, num_layers entries in run order
  const void* embedding;      // [vocab, hidden]
  const void* final_norm_w;
  const void* head;           // [vocab, hidden]
  int num_layers, hidden, vocab, dtype;
  int embedding_dtype, final_norm_dtype, head_dtype;
  float embedding_scale, final_eps, final_offset, logit_soft_cap;
  int max_qkv_rows, max_q_dim, max_inter;   // widths of the step's scratch rows
} OiModelDesc;

typedef struct OiStepDesc {
  const int* token_ids;       // [tokens]
  const OiAttnStep* attn_steps;   // host pointer
  const int* want_rows;       // [num_want] rows whose logits are wanted (or null)
  void* h;                    // [tokens, hidden]  the residual stream
  void* x;                    // [tokens, hidden]  normed rows
  void* qkv;                  // [tokens, max_qkv_rows]
  void* attn;                 // [tokens, max_q_dim]
  void* branch_a;             // [tokens, hidden]  output of the mixer
  void* branch_m;             // [tokens, hidden]  output of the feed-forward
  void* act;                  // [tokens, max_inter]
  void* gate_up;              // [tokens, 2 max_inter] or null (see oi_gated_mlp_needs_gate_up)
  void* wanted;               // [num_want, hidden] normed wanted rows
  float* logits;              // [num_want, vocab]
  void* xs;                   // [tokens, hidden] rows times the next norm's weight (steps of up to 32 rows; or null)
  float* ssq;                 // [32, ssq_stride] partial sums of squares (with xs); ssq_stride >= 8 * ceil(hidden / 128)
  int ssq_stride;
  int tokens, num_attn_steps, num_want;
} OiStepDesc;

// Embedding, every layer, final norm of the wanted rows, head: all kernels of one step, launched from native code.
OI_API int oi_forward(const OiModelDesc* model, const OiStepDesc* step, void* stream);
