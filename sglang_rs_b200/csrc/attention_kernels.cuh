// Attention over the paged cache, generic form: any head_dim up to 512, any number of
// query heads per kv head up to 32, any page size, optional
// window, 32-bit arithmetic throughout.  T is the storage type of q, the pages and the
// output.  It is the whole attention of the 32-bit path and the fallback of the bfloat16
// path for sizes its tensor-core kernels refuse.
//
// Formula (crates/sglang-kernel/src/cpu.rs:475-517): kv head = q head / (n_q / n_kv);
// s_t = (q . k_t) * scale over the keys the row may see; softmax with the maximum
// subtracted; o = sum_t p_t v_t.  The mask is by length only: a row at position pos sees
// keys max(0, pos - window + 1) .. pos (crates/sglang-srt/src/cuda_attention.rs:285-297 for
// the causal length).  The running maximum and denominator follow the online form of
// cuda_attention.rs:137-151.
//
// Work split: one block per (row, kv head, split); warp g of the block owns query head
// kv_head * G + g.  Keys are visited in blocks of 32 aligned to absolute multiples of 32,
// and a split covers `split_size` keys aligned to absolute multiples of split_size, so a
// row's arithmetic depends on its own position only, never on how the step was cut or
// what else is in the batch.  With split_size == 0 the block walks all keys and writes
// the output; otherwise it writes an unnormalised partial (acc, m, l) to scratch memory
// and srb_attention_combine merges the partials in split order.
#pragma once
#include "common.cuh"
#include <math.h>

#define KEY_BLOCK 32

struct AttnParams {
  const int* positions;      // [rows] position of the row in its sequence
  const int* row_request;    // [rows] index of the row's request in the block table
  const int* block_table;    // [requests, table_stride] page ids, -1 where none
  int table_stride;
  int n_q, n_kv, head_dim, page_size, num_pages;
  int window;                // 0 = all keys
  int split_size;            // 0 = no split
  int max_splits;
  float scale;
  int* error_word;
};

__device__ __forceinline__ void row_key_range(const AttnParams& p, int pos, int split, int& lo, int& hi) {
  const int begin = (p.window > 0 && pos + 1 > p.window) ? pos + 1 - p.window : 0;
  const int end = pos + 1;
  if (p.split_size == 0) {
    lo = begin;
    hi = end;
    return;
  }
  const int first = begin / p.split_size;
  lo = max(begin, (first + split) * p.split_size);
  hi = min(end, (first + split + 1) * p.split_size);
}

__device__ __forceinline__ int row_split_count(const AttnParams& p, int pos) {
  if (p.split_size == 0) return 1;
  const int begin = (p.window > 0 && pos + 1 > p.window) ? pos + 1 - p.window : 0;
  return pos / p.split_size - begin / p.split_size + 1;
}

template <typename T, int DIM_PER_LANE>
__global__ void paged_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_pool,
                                       const T* __restrict__ v_pool, T* __restrict__ out,
                                       float* __restrict__ part_acc, float* __restrict__ part_ml,
                                       AttnParams p) {
  extern __shared__ float smem[];
  const int d = p.head_dim;
  const int groups = p.n_q / p.n_kv;
  float* k_tile = smem;                                  // [32][d + 1]
  float* v_tile = k_tile + KEY_BLOCK * (d + 1);          // [32][d]
  float* q_tile = v_tile + KEY_BLOCK * d;                // [groups][d]
  __shared__ long long key_offset[KEY_BLOCK];            // element offset of each key's row, -1 = masked

  const int row = blockIdx.z, kv_head = blockIdx.y, split = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = p.positions[row];
  int lo, hi;
  row_key_range(p, pos, split, lo, hi);
  if (lo >= hi) return;
  const int request = p.row_request[row];
  const int q_head = kv_head * groups + warp;

  for (int i = threadIdx.x; i < groups * d; i += blockDim.x)
    q_tile[i] = srb_to_float(q[((size_t)row * p.n_q + (size_t)kv_head * groups) * d + i]);

  float m = -INFINITY, l = 0.f;
  float acc[DIM_PER_LANE];
#pragma unroll
  for (int j = 0; j < DIM_PER_LANE; ++j) acc[j] = 0.f;

  for (int base = lo & ~(KEY_BLOCK - 1); base < hi; base += KEY_BLOCK) {
    __syncthreads();                                     // previous tile fully consumed
    if (threadIdx.x < KEY_BLOCK) {
      const int key = base + threadIdx.x;
      long long offset = -1;
      if (key >= lo && key < hi) {
        const int page = p.block_table[(size_t)request * p.table_stride + key / p.page_size];
        if (page < 0 || page >= p.num_pages) {
          atomicOr(p.error_word, SRB_FLAG_BAD_PAGE);
        } else {
          offset = (((long long)page * p.n_kv + kv_head) * p.page_size + key % p.page_size) * d;
        }
      }
      key_offset[threadIdx.x] = offset;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < KEY_BLOCK * d; i += blockDim.x) {
      const int key = i / d, e = i - key * d;
      const long long offset = key_offset[key];
      k_tile[key * (d + 1) + e] = offset < 0 ? 0.f : srb_to_float(k_pool[offset + e]);
      v_tile[key * d + e] = offset < 0 ? 0.f : srb_to_float(v_pool[offset + e]);
    }
    __syncthreads();

    // one key per lane: the dot product runs over the head in index order
    float s = 0.f;
    const float* qv = q_tile + warp * d;
    const float* kv = k_tile + lane * (d + 1);
    for (int e = 0; e < d; ++e) s += qv[e] * kv[e];
    s = key_offset[lane] < 0 ? -INFINITY : s * p.scale;

    const float m_new = fmaxf(m, srb_warp_max(s));       // finite: the tile holds a visible key
    const float correction = expf(m - m_new);            // exp(-inf) = 0 on the first tile
    const float prob = expf(s - m_new);                  // 0 for masked keys
    l = l * correction + srb_warp_sum(prob);
    m = m_new;
#pragma unroll
    for (int j = 0; j < DIM_PER_LANE; ++j) acc[j] *= correction;
    for (int key = 0; key < KEY_BLOCK; ++key) {
      const float pk = __shfl_sync(0xffffffffu, prob, key);
#pragma unroll
      for (int j = 0; j < DIM_PER_LANE; ++j) {
        const int e = lane + 32 * j;
        if (e < d) acc[j] += pk * v_tile[key * d + e];
      }
    }
  }

  if (p.split_size == 0) {
    const float inv = 1.0f / l;
#pragma unroll
    for (int j = 0; j < DIM_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (e < d) out[((size_t)row * p.n_q + q_head) * d + e] = srb_from_float<T>(acc[j] * inv);
    }
  } else {
    const size_t slot = ((size_t)row * p.n_q + q_head) * p.max_splits + split;
#pragma unroll
    for (int j = 0; j < DIM_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (e < d) part_acc[slot * d + e] = acc[j];
    }
    if (lane == 0) {
      part_ml[slot * 2] = m;
      part_ml[slot * 2 + 1] = l;
    }
  }
}

// Merges a row's partials in split order: M = max m_s, out = sum acc_s e^(m_s - M) / sum l_s e^(m_s - M).
template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                         T* __restrict__ out, AttnParams p) {
  const int row = blockIdx.x, q_head = blockIdx.y;
  const int pos = p.positions[row];
  if (pos < 0) return;                                   // a padding row: no block wrote partials for it
  const int wanted = row_split_count(p, pos);
  if (wanted > p.max_splits) {
    // the launch has too few blocks along the splits for this row: its newest keys were left out
    if (q_head == 0 && threadIdx.x == 0 && p.error_word) atomicOr(p.error_word, SRB_FLAG_TOO_FEW_SPLITS);
  }
  const int count = min(wanted, p.max_splits);
  const size_t first = ((size_t)row * p.n_q + q_head) * p.max_splits;
  float m = -INFINITY;
  for (int s = 0; s < count; ++s) m = fmaxf(m, part_ml[(first + s) * 2]);
  float l = 0.f;
  for (int s = 0; s < count; ++s) l += part_ml[(first + s) * 2 + 1] * expf(part_ml[(first + s) * 2] - m);
  const float inv = 1.0f / l;
  for (int e = threadIdx.x; e < p.head_dim; e += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < count; ++s)
      acc += part_acc[(first + s) * p.head_dim + e] * expf(part_ml[(first + s) * 2] - m);
    out[((size_t)row * p.n_q + q_head) * p.head_dim + e] = srb_from_float<T>(acc * inv);
  }
}

template <typename T, int DIM_PER_LANE>
static int launch_attention(const void* q, const void* k_pool, const void* v_pool, void* out, float* part_acc,
                            float* part_ml, const AttnParams& p, int rows, cudaStream_t s) {
  const int groups = p.n_q / p.n_kv;
  const size_t smem = ((size_t)KEY_BLOCK * (p.head_dim + 1) + (size_t)KEY_BLOCK * p.head_dim +
                       (size_t)groups * p.head_dim) * sizeof(float);
  if (smem > 227 * 1024) SRB_FAIL("paged_attention: %zu bytes of shared memory exceed 232448", smem);
  if (smem > 48 * 1024)
    SRB_CUDA_CALL(cudaFuncSetAttribute(paged_attention_kernel<T, DIM_PER_LANE>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(p.split_size == 0 ? 1 : p.max_splits, p.n_kv, rows);
  paged_attention_kernel<T, DIM_PER_LANE><<<grid, groups * 32, smem, s>>>(
      (const T*)q, (const T*)k_pool, (const T*)v_pool, (T*)out, part_acc, part_ml, p);
  SRB_LAUNCH_CHECK("paged_attention");
  if (p.split_size != 0) {
    dim3 cgrid(rows, p.n_q);
    attention_combine_kernel<T><<<cgrid, 64, 0, s>>>(part_acc, part_ml, (T*)out, p);
    SRB_LAUNCH_CHECK("attention_combine");
  }
  return SRB_OK;
}

// Checks the sizes and launches; shared by every entry point.  Scratch (only when split_size > 0):
// part_acc holds rows * n_q * max_splits * head_dim floats and part_ml rows * n_q * max_splits * 2.
static int paged_attention_dispatch(const void* q, const void* k_pool, const void* v_pool, void* out,
                                   float* part_acc, float* part_ml, const int* positions,
                                   const int* row_request, const int* block_table, int table_stride, int rows,
                                   int n_q, int n_kv, int head_dim, int page_size, int num_pages, int window,
                                   int split_size, int max_splits, float scale, int* error_word, int dtype,
                                   void* stream) {
  if (rows <= 0) return SRB_OK;
  if (n_q <= 0 || n_kv <= 0 || n_q % n_kv != 0)
    SRB_FAIL("paged_attention: %d query heads are not a multiple of %d kv heads", n_q, n_kv);
  if (n_q / n_kv > 32) SRB_FAIL("paged_attention: %d query heads per kv head exceed 32", n_q / n_kv);
  if (head_dim <= 0 || head_dim > 512) SRB_FAIL("paged_attention: head_dim %d must be positive, at most 512", head_dim);
  if (page_size <= 0 || num_pages <= 0 || table_stride <= 0)
    SRB_FAIL("paged_attention: page size, page count and table stride must be positive");
  if (window < 0 || split_size < 0) SRB_FAIL("paged_attention: window and split size must be non-negative");
  if (split_size != 0 && (max_splits <= 0 || !part_acc || !part_ml))
    SRB_FAIL("paged_attention: a split run needs scratch memory and max_splits > 0");
  if (rows > 65535) {
    // grid.z is limited to 65535 blocks
    SRB_FAIL("paged_attention: %d rows exceed 65535 in one launch", rows);
  }
  AttnParams p;
  p.positions = positions; p.row_request = row_request; p.block_table = block_table;
  p.table_stride = table_stride; p.n_q = n_q; p.n_kv = n_kv; p.head_dim = head_dim;
  p.page_size = page_size; p.num_pages = num_pages; p.window = window; p.split_size = split_size;
  p.max_splits = split_size == 0 ? 1 : max_splits; p.scale = scale; p.error_word = error_word;
  cudaStream_t s = (cudaStream_t)stream;
  const int per_lane = (head_dim + 31) / 32;
#define SRB_ATTN_CASE(T, N) \
  return launch_attention<T, N>(q, k_pool, v_pool, out, part_acc, part_ml, p, rows, s)
#define SRB_ATTN_DISPATCH(T)                        \
  if (per_lane <= 1) { SRB_ATTN_CASE(T, 1); }       \
  else if (per_lane <= 2) { SRB_ATTN_CASE(T, 2); }  \
  else if (per_lane <= 4) { SRB_ATTN_CASE(T, 4); }  \
  else if (per_lane <= 8) { SRB_ATTN_CASE(T, 8); }  \
  else { SRB_ATTN_CASE(T, 16); }
  if (dtype == SRB_DTYPE_F32) { SRB_ATTN_DISPATCH(float) }
  if (dtype == SRB_DTYPE_BF16) { SRB_ATTN_DISPATCH(__nv_bfloat16) }
  SRB_FAIL("paged_attention: unknown dtype %d", dtype);
}
