// Attention of decoded tokens over the paged cache in bfloat16, tensor-core form.
//
// Same formula, key ranges, split of the keys and scratch layout as the generic kernel
// (attention_kernels.cuh), so the same combine kernel merges its partials.  One block per
// (row, kv head, split of `split_size` = 128 keys); each of its four warps owns 32 keys at
// fixed absolute positions, brings them from the pages into shared memory with 16-byte
// asynchronous copies (all in flight at once, XOR-swizzled against bank conflicts), and
// computes S = Q K^T and O = P V with mma.sync m16n8k16: the 16 rows of the tile are the
// query heads that share the kv head (up to 16, zero-padded), so every key and value is
// read from memory once for all of them.  Scores, maximum, exponentials and sums are
// 32-bit; P is rounded to bfloat16 for the second product.  The four warps' results are
// merged in warp order in shared memory and written as one partial (acc, m, l).
//
// Sizes: head_dim 64 or 128, up to 16 query heads per kv head, split_size 128 (64 KB of
// shared memory per block at head_dim 128, so three blocks share an SM and one block's
// copies overlap another's arithmetic).  Other
// sizes are refused here and the caller uses the generic kernel.
#include "attention_kernels.cuh"
#include "mma_helpers.cuh"

SRB_DEFINE_LAST_ERROR()
SRB_DEFINE_PDL_SWITCH()

#define DEC_WARPS 4
#define DEC_KEYS 32                       // keys per warp
#define DEC_SPLIT (DEC_WARPS * DEC_KEYS)  // keys per block

template <int D>
__global__ void __launch_bounds__(DEC_WARPS * 32)
decode_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                        const __nv_bfloat16* __restrict__ v_pool, float* __restrict__ part_acc,
                        float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out, int* __restrict__ counters,
                        AttnParams p) {
  constexpr int CHUNKS = D / 8;            // 16-byte chunks per key row
  constexpr int KSTEPS = D / 16;           // k16 steps of Q K^T
  constexpr int NT_S = DEC_KEYS / 8;       // n8 tiles of S
  constexpr int NT_O = D / 8;              // n8 tiles of O
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.z, kv_head = blockIdx.y, split = blockIdx.x;
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int pos = p.positions[row];
  int lo, hi;
  row_key_range(p, pos, split, lo, hi);
  if (lo >= hi) return;
  const int groups = p.n_q / p.n_kv;
  const int request = p.row_request[row];
  const int begin = (p.window > 0 && pos + 1 > p.window) ? pos + 1 - p.window : 0;
  const int warp_base = (begin / p.split_size + split) * p.split_size + warp * DEC_KEYS;
  const int k_lo = max(lo, warp_base), k_hi = min(hi, warp_base + DEC_KEYS);
  const bool has_keys = k_lo < k_hi;

  __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(smem_raw) + (size_t)warp * 2 * DEC_KEYS * D;
  __nv_bfloat16* vs = ks + DEC_KEYS * D;

  if (has_keys) {
    // lane i looks up the page of key i once; the copies below fetch the row offset by shuffle
    long long my_offset = -1;
    {
      const int abs_key = warp_base + lane;
      if (abs_key >= k_lo && abs_key < k_hi) {
        const int page = p.block_table[(size_t)request * p.table_stride + abs_key / p.page_size];
        if (page < 0 || page >= p.num_pages)
          atomicOr(p.error_word, SRB_FLAG_BAD_PAGE);
        else
          my_offset = (((long long)page * p.n_kv + kv_head) * p.page_size + abs_key % p.page_size) * D;
      }
    }
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
      const __nv_bfloat16* pool = pass == 0 ? k_pool : v_pool;
      __nv_bfloat16* dst_base = pass == 0 ? ks : vs;
#pragma unroll
      for (int j = 0; j < DEC_KEYS * CHUNKS / 32; ++j) {
        const int i = lane + 32 * j;
        const int key = i / CHUNKS, c = i % CHUNKS;
        const long long offset = __shfl_sync(0xffffffffu, my_offset, key);
        const bool valid = offset >= 0;
        cp_async_16(dst_base + key * D + ((c ^ (key & 7)) * 8), pool + (valid ? offset + c * 8 : 0), valid ? 16 : 0);
      }
      cp_async_commit();
    }
  }

  // Q fragments: rows of the tile are the query heads of this kv head; rows >= groups are zero
  unsigned qa[KSTEPS][4];
  {
    const int r0 = lane >> 2, r1 = r0 + 8, col = (lane & 3) * 2;
    const __nv_bfloat16* qrow = q + ((size_t)row * p.n_q + (size_t)kv_head * groups) * D;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      const int d0 = kk * 16 + col;
      qa[kk][0] = r0 < groups ? *reinterpret_cast<const unsigned*>(qrow + (size_t)r0 * D + d0) : 0u;
      qa[kk][1] = r1 < groups ? *reinterpret_cast<const unsigned*>(qrow + (size_t)r1 * D + d0) : 0u;
      qa[kk][2] = r0 < groups ? *reinterpret_cast<const unsigned*>(qrow + (size_t)r0 * D + d0 + 8) : 0u;
      qa[kk][3] = r1 < groups ? *reinterpret_cast<const unsigned*>(qrow + (size_t)r1 * D + d0 + 8) : 0u;
    }
  }

  float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
  float o[NT_O][4];
#pragma unroll
  for (int t = 0; t < NT_O; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;

  if (has_keys) {
    cp_async_wait<1>();
    __syncwarp();
    float s[NT_S][4];
#pragma unroll
    for (int t = 0; t < NT_S; ++t) s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.f;
    // S = Q K^T: B operand = K rows (keys) by d; ldmatrix.x4 brings two n8 tiles of one k16 step
    const int mat = lane >> 3, mrow = lane & 7;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
      for (int t = 0; t < NT_S; t += 2) {
        const int key = (t + (mat >> 1)) * 8 + mrow;
        const int chunk = kk * 2 + (mat & 1);
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, ks + key * D + ((chunk ^ (key & 7)) * 8));
        mma_bf16(s[t], qa[kk], b0, b1);
        mma_bf16(s[t + 1], qa[kk], b2, b3);
      }
    }
    // scale, mask by the row's key range, softmax over this warp's keys
    const int col = (lane & 3) * 2;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int t = 0; t < NT_S; ++t) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int abs_key = warp_base + t * 8 + col + (e & 1);
        const float v = (abs_key >= k_lo && abs_key < k_hi) ? s[t][e] * p.scale : -INFINITY;
        s[t][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int t = 0; t < NT_S; ++t) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = expf(s[t][e] - mx[e >> 1]);     // masked keys give exp(-inf) = 0
        s[t][e] = pv;
        sum[e >> 1] += pv;
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
      sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
      m_row[h] = mx[h];
      l_row[h] = sum[h];
    }
    cp_async_wait<0>();
    __syncwarp();
    // O = P V: A operand = P from the S accumulators, B operand = V rows (keys) by d, transposed on load
#pragma unroll
    for (int kk = 0; kk < DEC_KEYS / 16; ++kk) {
      unsigned pa[4];
      pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int t = 0; t < NT_O; t += 2) {
        const int key = kk * 16 + (mat & 1) * 8 + mrow;
        const int chunk = t + (mat >> 1);
        unsigned b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, vs + key * D + ((chunk ^ (key & 7)) * 8));
        mma_bf16(o[t], pa, b0, b1);
        mma_bf16(o[t + 1], pa, b2, b3);
      }
    }
  }

  // merge the four warps in warp order: staged as [warp][head][D + 2] floats over the key tiles
  __syncthreads();
  float* stage = reinterpret_cast<float*>(smem_raw);
  {
    const int r0 = lane >> 2, col = (lane & 3) * 2;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int head = r0 + 8 * h;
      if (head < groups) {
        float* dst = stage + ((size_t)warp * groups + head) * (D + 2);
#pragma unroll
        for (int t = 0; t < NT_O; ++t) {
          dst[t * 8 + col] = o[t][2 * h];
          dst[t * 8 + col + 1] = o[t][2 * h + 1];
        }
        if ((lane & 3) == 0) {
          dst[D] = m_row[h];
          dst[D + 1] = l_row[h];
        }
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < groups * D; i += blockDim.x) {
    const int head = i / D, e = i % D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, stage[((size_t)w * groups + head) * (D + 2) + D]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float* src = stage + ((size_t)w * groups + head) * (D + 2);
      const float weight = src[D + 1] > 0.f ? expf(src[D] - m) : 0.f;     // a warp without keys adds nothing
      acc += src[e] * weight;
      l += src[D + 1] * weight;
    }
    const size_t slot = ((size_t)row * p.n_q + (size_t)kv_head * groups + head) * p.max_splits + split;
    part_acc[slot * D + e] = acc;
    if (e == 0) {
      part_ml[slot * 2] = m;
      part_ml[slot * 2 + 1] = l;
    }
  }
  if (!counters) return;                 // a separate kernel merges the splits

  // The block that arrives last at this (row, kv head) merges all splits, in split order, so
  // the result does not depend on which block that is.  The counter returns to zero.
  __shared__ int is_last;
  const int count = min(row_split_count(p, pos), p.max_splits);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* counter = counters + (size_t)row * p.n_kv + kv_head;
    const int ticket = atomicAdd(counter, 1);
    is_last = ticket == count - 1;
    if (is_last) *counter = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  float* weights = stage;                // [groups][count + 1]: e^(m_s - M) per split, then 1 / sum
  for (int head = warp; head < groups; head += DEC_WARPS) {
    const size_t first = ((size_t)row * p.n_q + (size_t)kv_head * groups + head) * p.max_splits;
    float m = -INFINITY;
    for (int sp = lane; sp < count; sp += 32) m = fmaxf(m, __ldcg(part_ml + (first + sp) * 2));
    m = srb_warp_max(m);
    float l = 0.f;
    for (int base = 0; base < count; base += 32) {      // sums in split order: lane order inside, chunks outside
      const int sp = base + lane;
      float w = 0.f, lw = 0.f;
      if (sp < count) {
        w = expf(__ldcg(part_ml + (first + sp) * 2) - m);
        lw = __ldcg(part_ml + (first + sp) * 2 + 1) * w;
        weights[head * (count + 1) + sp] = w;
      }
      for (int k = 0; k < 32; ++k) l += __shfl_sync(0xffffffffu, lw, k);
    }
    if (lane == 0) weights[head * (count + 1) + count] = 1.0f / l;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < groups * D; i += blockDim.x) {
    const int head = i / D, e = i % D;
    const size_t first = ((size_t)row * p.n_q + (size_t)kv_head * groups + head) * p.max_splits;
    const float* w = weights + head * (count + 1);
    float acc = 0.f;
    for (int sp = 0; sp < count; ++sp) acc += __ldcg(part_acc + (first + sp) * D + e) * w[sp];
    out[((size_t)row * p.n_q + (size_t)kv_head * groups + head) * D + e] = __float2bfloat16_rn(acc * w[count]);
  }
}

template <int D>
static int launch_decode(const void* q, const void* k_pool, const void* v_pool, void* out, float* part_acc,
                         float* part_ml, int* counters, const AttnParams& p, int rows, cudaStream_t s) {
  const size_t smem = (size_t)DEC_WARPS * 2 * DEC_KEYS * D * sizeof(__nv_bfloat16);
  SRB_CUDA_CALL(cudaFuncSetAttribute(decode_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)smem));
  dim3 grid(p.max_splits, p.n_kv, rows);
  SRB_CUDA_CALL(srb_launch(decode_attention_kernel<D>, grid, dim3(DEC_WARPS * 32), smem, s, (const __nv_bfloat16*)q,
                           (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, part_acc, part_ml,
                           (__nv_bfloat16*)out, counters, p));
  if (counters) return SRB_OK;
  dim3 cgrid(rows, p.n_q);
  attention_combine_kernel<__nv_bfloat16><<<cgrid, 64, 0, s>>>(part_acc, part_ml, (__nv_bfloat16*)out, p);
  SRB_LAUNCH_CHECK("attention_combine");
  return SRB_OK;
}

// 1 if this kernel takes the sizes, 0 if the generic one has to be used.
extern "C" int srb_decode_attention_supports(int n_q, int n_kv, int head_dim, int split_size, int dtype) {
  return dtype == SRB_DTYPE_BF16 && (head_dim == 64 || head_dim == 128) && n_kv > 0 && n_q % n_kv == 0 &&
         n_q / n_kv <= 16 && split_size == DEC_SPLIT;
}

// Arguments as srb_paged_attention; bfloat16 only; split_size must be 128.  `counters` (optional)
// holds rows * n_kv ints that are zero before the call and zero again after it: with it the
// last block of each (row, kv head) merges the splits and no second kernel runs.
extern "C" int srb_decode_attention(const void* q, const void* k_pool, const void* v_pool, void* out,
                                    float* part_acc, float* part_ml, int* counters, const int* positions,
                                    const int* row_request, const int* block_table, int table_stride, int rows,
                                    int n_q, int n_kv, int head_dim, int page_size, int num_pages, int window,
                                    int split_size, int max_splits, float scale, int* error_word, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (!srb_decode_attention_supports(n_q, n_kv, head_dim, split_size, SRB_DTYPE_BF16))
    SRB_FAIL("decode_attention: head_dim %d (64 or 128), %d query heads per kv head (at most 16) or split size %d "
             "(128) is not taken by this kernel", head_dim, n_kv > 0 ? n_q / n_kv : 0, split_size);
  if (page_size <= 0 || num_pages <= 0 || table_stride <= 0 || max_splits <= 0 || window < 0)
    SRB_FAIL("decode_attention: page size, page count, table stride and split count must be positive");
  if (!part_acc || !part_ml) SRB_FAIL("decode_attention: scratch memory is needed");
  if (rows > 65535) SRB_FAIL("decode_attention: %d rows exceed 65535 in one launch", rows);
  AttnParams p;
  p.positions = positions; p.row_request = row_request; p.block_table = block_table;
  p.table_stride = table_stride; p.n_q = n_q; p.n_kv = n_kv; p.head_dim = head_dim;
  p.page_size = page_size; p.num_pages = num_pages; p.window = window; p.split_size = split_size;
  p.max_splits = max_splits; p.scale = scale; p.error_word = error_word;
  cudaStream_t s = (cudaStream_t)stream;
  if (head_dim == 64) return launch_decode<64>(q, k_pool, v_pool, out, part_acc, part_ml, counters, p, rows, s);
  return launch_decode<128>(q, k_pool, v_pool, out, part_acc, part_ml, counters, p, rows, s);
}
