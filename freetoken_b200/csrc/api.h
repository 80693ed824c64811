// C interface of the native library: every entry point validates its arguments on the host,
// launches on the given stream, allocates nothing and returns 0 or a non-zero status whose
// text ftk_last_error() gives.  Pointers are device pointers unless said otherwise.
#pragma once
#include <stdint.h>

#define FTK_F32 0
#define FTK_BF16 1
#define FTK_ACT_SILU 0
#define FTK_ACT_SWIGLUOAI 1
#define FTK_SCORE_SIGMOID 0
#define FTK_SCORE_SOFTMAX 1

#ifdef __cplusplus
extern "C" {
#endif

// One destination of ftk_norm_rope_store: heads [first_head, first_head + n_heads) of every
// token, optionally normed and rotated, written densely or scattered into a paged slab.
typedef struct {
  int first_head;
  int n_heads;
  const float* norm_weight;  // [head_dim] or null
  int rotate;
  void* dense_out;           // [T, n_heads, head_dim] or null
  void* slab;                // [num_pages, n_heads, page_size, head_dim] or null
  const int32_t* slot_map;   // [T] slot = page * page_size + offset; negative skips the token
  int page_size;
  int num_pages;
} FtkSection;

const char* ftk_last_error(void);

int ftk_embedding_gather(const void* table, int dtype, const int32_t* ids, int n_tokens, int hidden,
                         int vocab, float* out, void* stream);
int ftk_add_rmsnorm(const void* x, int x_dtype, float* residual, const float* weight, void* out,
                    int out_dtype, float* out_f32, const int32_t* rows, int n_rows, int hidden,
                    float eps, int gemma, void* stream);
// The same with the row that is added taken as a sum over routes: sum_j y[route_pos[row * top_k + j]]
// (+ shared[row]), rounded to y's type (what ftk_moe_combine would have written).
int ftk_add_rmsnorm_routes(const void* y, int y_dtype, const int32_t* route_pos, int top_k, int n_routes,
                           const void* shared, float* residual, const float* weight, void* out, int out_dtype,
                           float* out_f32, const int32_t* rows, int n_rows, int hidden, float eps, int gemma,
                           void* stream);
int ftk_act_and_mul(const void* gate_up, int dtype, int n_rows, int inter, int act, float alpha,
                    float limit, void* out, void* stream);
int ftk_cast(const void* src, int src_dtype, void* dst, int dst_dtype, long long n, void* stream);
int ftk_table_update(int32_t* table, long long table_len, const int32_t* updates, int n_updates,
                     void* stream);
int ftk_copy_tokens(int32_t* dst, int dst_len, const int32_t* pairs, const int32_t* src, int src_len, int n,
                    int vocab, void* stream);
int ftk_norm_rope_store(const void* x, int dtype, int n_tokens, int row_elems, int head_dim,
                        int rotary_dim, const int32_t* positions, const float* rope_table, int max_pos,
                        float eps, int gemma, int n_sections, const FtkSection* sections, void* stream);
int ftk_paged_attention(const void* q, const void* k_slab, const void* v_slab, int dtype,
                        const int32_t* block_table, int bt_stride, const int32_t* seg_info, int n_segs,
                        const int32_t* items, int n_items, float* part_o, float* part_ml, int n_slots,
                        void* out, int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                        int num_pages, int tile_rows, float scale, int window, void* stream);
// Long steps in bfloat16 on tcgen05: tiles of 128 query rows (plan the items with tile_rows = 128), head
// size 128, pages of a multiple of 16 tokens; n_tokens = rows of q.  ftk_attention_tc_fits says whether
// the sizes are taken.
int ftk_attention_tc_fits(int head_dim, int page_size, int group);
int ftk_paged_attention_tc(const void* q, const void* k_slab, const void* v_slab, const int32_t* block_table,
                           int bt_stride, const int32_t* seg_info, int n_segs, const int32_t* items, int n_items,
                           float* part_o, float* part_ml, int n_slots, void* out, int n_tokens, int n_q_heads,
                           int n_kv_heads, int head_dim, int page_size, int num_pages, float scale, int window,
                           void* stream);
// Decode steps in bfloat16 on the same kernel with tiles of at most 16 query rows (plan the items with
// tile_rows = 16 and key pieces that are multiples of 128; at most 16 query heads per KV head): one
// warp takes the softmax of the tile's rows.  part_o [slots, Hkv, 16, 128], part_ml [slots, Hkv, 16, 2].
int ftk_attention_tc_few_fits(int head_dim, int page_size, int group);
int ftk_paged_attention_tc_few(const void* q, const void* k_slab, const void* v_slab, const int32_t* block_table,
                               int bt_stride, const int32_t* seg_info, int n_segs, const int32_t* items, int n_items,
                               float* part_o, float* part_ml, int n_slots, void* out, int n_tokens, int n_q_heads,
                               int n_kv_heads, int head_dim, int page_size, int num_pages, float scale, int window,
                               void* stream);
int ftk_paged_attention_sparse(const void* q, const void* k_slab, const void* v_slab, int dtype,
                               const int32_t* block_table, int bt_stride, const int32_t* seg_info, int n_segs,
                               const int32_t* items, int n_items, float* part_o, float* part_ml, int n_slots,
                               void* out, int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                               int num_pages, int tile_rows, float scale, const int32_t* sel, int sel_stride,
                               int block_size, void* stream);
int ftk_sparse_select(const void* iq, const void* ik_slab, int dtype, const int32_t* block_table, int bt_stride,
                      const int32_t* seg_info, int n_segs, int n_tokens, int n_heads, int dim, int page_size,
                      int num_pages, int block_size, int topk, int local_blocks, int init_blocks, int max_blocks,
                      int live_blocks, int32_t* sel, float* scores, void* stream);
// Whether bfloat16 block scores of these sizes can be taken on the tensor cores (`scores [T, n_heads, max_blocks]`
// float32 scratch must then be given to ftk_sparse_select).
int ftk_sparse_score_fits(int n_heads, int dim, int block_size);
int ftk_router_topk(const float* logits, int n_parts, const float* bias, int n_tokens, int n_experts, int top_k,
                    int scoring, float scale, int32_t* ids, float* weights, void* stream);
// Router logits (float32 x [T, hidden] times gate_w [E, hidden]), choice and sort of the routes in one
// launch, for steps of at most 32 tokens (beyond that the
// separate kernels are faster); ftk_moe_route_fits says whether the sizes are taken.
int ftk_moe_route_fits(int n_tokens, int hidden, int n_experts, int top_k);
int ftk_moe_route(const float* x, const float* gate_w, const float* bias, int n_tokens, int hidden, int n_experts,
                  int top_k, int scoring, float scale, float* logits, int32_t* ids, float* weights,
                  int32_t* counts, int32_t* offsets, int32_t* routes, int32_t* pos, int do_sort, void* stream);
// Products of very few tokens (bfloat16): the weights are streamed once by warps of every SM (gemv.cu).
int ftk_small_linear_fits(int n_tokens, int n_out, int k);
int ftk_small_linear(const void* x, const void* w, void* out, int n_tokens, int n_out, int k, void* stream);
int ftk_moe_small_fits(int n_tokens, int hidden, int inter, int top_k);
int ftk_moe_small_gate_up(const void* h, const int32_t* ids, const void* w1, void* a, int n_tokens, int top_k,
                          int n_experts, int hidden, int inter, int act, float alpha, float limit, void* stream);
int ftk_moe_small_down(const void* a, const int32_t* ids, const float* weights, const void* w2, void* y, int n_tokens,
                       int top_k, int n_experts, int hidden, int inter, void* stream);
int ftk_moe_permute(const int32_t* topk_ids, int n_tokens, int top_k, int n_experts,
                    int32_t* expert_counts, int32_t* expert_offsets, int32_t* sorted_routes,
                    int32_t* route_pos, void* stream);
int ftk_moe_gather(const void* h, int dtype, const int32_t* sorted_routes, int n_routes, int top_k,
                   int hidden, void* out, void* stream);
int ftk_moe_gemm1_act(const void* x_sorted, const void* w1, int dtype, const int32_t* expert_offsets,
                      int n_experts, int n_routes, int hidden, int inter, int act, float alpha,
                      float limit, void* out, void* stream);
// The same from the tokens' rows x [n_tokens, hidden] in their own order (bfloat16, tensor cores): row r of
// expert order is the row of token sorted_routes[r] / top_k, gathered by the kernel (steps whose token tiles have
// at most 32 rows: ask ftk_moe_gemm1_gather_fits).
int ftk_moe_gemm1_gather_fits(int hidden, int inter, int n_experts, int n_routes);
int ftk_moe_gemm1_act_gather(const void* x, const void* w1, const int32_t* expert_offsets, const int32_t* sorted_routes,
                             int top_k, int n_tokens, int n_experts, int n_routes, int hidden, int inter, int act,
                             float alpha, float limit, void* out, void* stream);
int ftk_moe_gemm2(const void* a, const void* w2, int dtype, const int32_t* expert_offsets,
                  const int32_t* sorted_routes, const float* topk_weights, int n_experts, int n_routes,
                  int hidden, int inter, void* out, void* stream);
int ftk_moe_combine(const void* y, int dtype, const int32_t* route_pos, int n_tokens, int top_k,
                    int hidden, const void* shared, void* out, void* stream);
// Status words of the kernels' bounded waits: out[0] = first code since the last call (0 = none),
// out[1] = block that recorded it.  Synchronises with the device and clears the words.
// Kernel forms launched so far, as "name<TAB>count" lines (see ftk::note_variant); returns the bytes needed.
int ftk_variant_counts(char* buf, int cap, int reset);
int ftk_read_status(int* out);
// Writes `code` into a status word from the host (unit 0: grouped GEMM, 1: attention), so that a caller's
// handling of a given-up wait can be tested without any wait running out on the device.
int ftk_debug_set_status(int unit, int code);
// 0 sends bfloat16 grouped expert products to the CUDA-core kernels; default 1 (tcgen05).
int ftk_set_moe_tensor_cores(int enabled);
int ftk_set_moe_pairs(int enabled);
int ftk_sample(const float* logits, int n_rows, int vocab, const float* temperature,
               const int32_t* top_k, const float* top_p, const float* u, int32_t* out, void* stream);

#ifdef __cplusplus
}
#endif
