// Entry point of the generic paged attention; the kernels are in attention_kernels.cuh.
#include "attention_kernels.cuh"

SRB_DEFINE_LAST_ERROR()

// Scratch (only when split_size > 0): part_acc holds rows * n_q * max_splits * head_dim
// floats and part_ml rows * n_q * max_splits * 2 floats.
extern "C" int srb_paged_attention(const void* q, const void* k_pool, const void* v_pool, void* out,
                                   float* part_acc, float* part_ml, const int* positions,
                                   const int* row_request, const int* block_table, int table_stride, int rows,
                                   int n_q, int n_kv, int head_dim, int page_size, int num_pages, int window,
                                   int split_size, int max_splits, float scale, int* error_word, int dtype,
                                   void* stream) {
  return paged_attention_dispatch(q, k_pool, v_pool, out, part_acc, part_ml, positions, row_request, block_table,
                                  table_stride, rows, n_q, n_kv, head_dim, page_size, num_pages, window, split_size,
                                  max_splits, scale, error_word, dtype, stream);
}
