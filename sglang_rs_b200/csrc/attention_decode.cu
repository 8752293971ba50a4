// Attention of decoded tokens over the paged cache in bfloat16, tensor-core form.
//
// Same formula and key ranges as the generic kernel (attention_kernels.cuh).  The keys a row
// may see are cut into units of 64 at absolute positions; a block owns a contiguous run of
// units of one (row, kv head) and walks it with a two-stage pipeline of 16-byte asynchronous
// copies, so copies of the next unit are in flight while the current one is multiplied.  The
// number of blocks per (row, kv head) is a launch parameter (`num_splits`): the caller picks
// it so that about three blocks per SM exist, whatever the batch (one row: many short runs;
// many rows: one long run each).
//
// Inside a block each of the four warps owns 16 keys of every unit, in buffers of its own
// (no block-wide barrier inside the loop), and keeps its own running maximum, sum and output
// for the up to 16 query heads that share the kv head: S = Q K^T and O += P V run on mma.sync
// m16n8k16 with the heads as the 16 rows, so every key and value is read once for all of
// them.  Scores are kept in units of log2 (s * scale * log2 e) so that exponentials are
// single ex2 instructions; maximum, sums and O are 32-bit; P is rounded to bfloat16 for the
// second product.  At the end the four warps are merged in warp order, the block writes one
// partial (acc, m, l) and the block that arrives last at its (row, kv head) merges the
// partials in split order and writes the output (a counter per (row, kv head), zero before
// and after the launch).
//
// Sizes: head_dim 64 or 128, up to 16 query heads per kv head.  Other sizes are refused
// here and the caller uses the generic kernel.
#include "attention_kernels.cuh"
#include "mma_helpers.cuh"

SRB_DEFINE_LAST_ERROR()
SRB_DEFINE_PDL_SWITCH()

#define DEC_WARPS 4
#define DEC_KEYS 16                       // keys per warp and unit
#define DEC_UNIT (DEC_WARPS * DEC_KEYS)   // keys per unit
#define DEC_STAGES 2

struct DecodeParams {
  AttnParams a;              // split_size is unused; max_splits = blocks per (row, kv head)
  float scale_log2;
};

__device__ __forceinline__ void decode_units(const AttnParams& p, int pos, int& first_unit, int& units, int& lo,
                                             int& hi) {
  lo = (p.window > 0 && pos + 1 > p.window) ? pos + 1 - p.window : 0;
  hi = pos + 1;
  first_unit = lo / DEC_UNIT;
  units = (hi - 1) / DEC_UNIT - first_unit + 1;
}

// CLUSTER: the blocks of a (row, kv head) form a thread-block cluster (at most 8 of them) and merge
// their partial results through each other's shared memory; otherwise through global memory, where
// the block that arrives last merges.
template <int D, bool CLUSTER>
__global__ void __launch_bounds__(DEC_WARPS * 32, 3)
decode_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                        const __nv_bfloat16* __restrict__ v_pool, float* __restrict__ part_acc,
                        float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out, int* __restrict__ counters,
                        DecodeParams dp) {
  constexpr int CHUNKS = D / 8;            // 16-byte chunks per key row
  constexpr int KSTEPS = D / 16;           // k16 steps of Q K^T
  constexpr int NT_O = D / 8;              // n8 tiles of O
  constexpr int STAGE_ELEMS = 2 * DEC_KEYS * D;        // K and V of one warp and unit
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const AttnParams& p = dp.a;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.z, kv_head = blockIdx.y, split = blockIdx.x;
  // The step's index arrays were copied in before its first kernel, so they may be read at once.
  // q and the key and value at the row's own position come from the kernel ahead: they are read
  // after the dependency wait.  Keys before that position are from earlier steps (a row of this
  // launch is the only row of its request in the step), so a block whose first unit ends before
  // the row's position asks for it before the wait and overlaps the kernel ahead.
  srb_mark(SRB_MARK_DECODE_ATTENTION, 0);
  srb_launch_dependents();
  const int pos = p.positions[row];
  int first_unit, units, lo, hi;
  decode_units(p, pos, first_unit, units, lo, hi);
  const int per_split = (units + p.max_splits - 1) / p.max_splits;
  const int count = (units + per_split - 1) / per_split;           // splits that have work
  if (!CLUSTER && split >= count) {
    srb_grid_dependency_wait();
    return;
  }
  const int unit_begin = first_unit + split * per_split;
  const int unit_end = min(first_unit + units, unit_begin + per_split);     // a block without work: begin >= end
  const int groups = p.n_q / p.n_kv;
  const int request = p.row_request[row];
  const int page_shift = (p.page_size & (p.page_size - 1)) == 0 ? __ffs(p.page_size) - 1 : -1;

  __nv_bfloat16* warp_smem = reinterpret_cast<__nv_bfloat16*>(smem_raw) + (size_t)warp * DEC_STAGES * STAGE_ELEMS;

  // copies of one unit: lanes 0..15 look up the page of one key each, the row offsets travel by shuffle
  auto issue = [&](int unit, int stage) {
    __nv_bfloat16* ks = warp_smem + (size_t)stage * STAGE_ELEMS;
    __nv_bfloat16* vs = ks + DEC_KEYS * D;
    long long my_offset = -1;
    const int abs_key = unit * DEC_UNIT + warp * DEC_KEYS + (lane & (DEC_KEYS - 1));
    if (abs_key >= lo && abs_key < hi) {
      const int logical = page_shift >= 0 ? abs_key >> page_shift : abs_key / p.page_size;
      const int within = page_shift >= 0 ? abs_key & (p.page_size - 1) : abs_key % p.page_size;
      const int page = p.block_table[(size_t)request * p.table_stride + logical];
      if (page < 0 || page >= p.num_pages) {
        if (lane < DEC_KEYS) atomicOr(p.error_word, SRB_FLAG_BAD_PAGE);
      } else {
        my_offset = (((long long)page * p.n_kv + kv_head) * p.page_size + within) * D;
      }
    }
#pragma unroll
    for (int j = 0; j < DEC_KEYS * CHUNKS / 32; ++j) {
      const int i = lane + 32 * j;
      const int key = i / CHUNKS, c = i % CHUNKS;
      const long long offset = __shfl_sync(0xffffffffu, my_offset, key);
      const bool valid = offset >= 0;
      const int where = key * D + ((c ^ (key & 7)) * 8);
      cp_async_16(ks + where, k_pool + (valid ? offset + c * 8 : 0), valid ? 16 : 0);
      cp_async_16(vs + where, v_pool + (valid ? offset + c * 8 : 0), valid ? 16 : 0);
    }
    cp_async_commit();
  };
  const bool has_work = unit_begin < unit_end;
  const bool first_unit_is_old = (unit_begin + 1) * DEC_UNIT <= pos;
  if (has_work && first_unit_is_old) issue(unit_begin, 0);
  srb_grid_dependency_wait();
  srb_mark(SRB_MARK_DECODE_ATTENTION, 1);
  if (has_work && !first_unit_is_old) issue(unit_begin, 0);

  // Q fragments: rows of the tile are the query heads of this kv head; rows >= groups are zero
  unsigned qa[KSTEPS][4];
  {
    const int r0 = lane >> 2, r1 = r0 + 8, col0 = (lane & 3) * 2;
    const __nv_bfloat16* qrow = q + ((size_t)row * p.n_q + (size_t)kv_head * groups) * D;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      const int d0 = kk * 16 + col0;
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
  const int mat = lane >> 3, mrow = lane & 7, col = (lane & 3) * 2;

#pragma unroll 1
  for (int unit = unit_begin; unit < unit_end; ++unit) {
    const int stage = (unit - unit_begin) & 1;
    if (unit + 1 < unit_end) {
      issue(unit + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncwarp();
    const __nv_bfloat16* ks = warp_smem + (size_t)stage * STAGE_ELEMS;
    const __nv_bfloat16* vs = ks + DEC_KEYS * D;
    const int key_base = unit * DEC_UNIT + warp * DEC_KEYS;
    if (key_base < hi && key_base + DEC_KEYS > lo) {         // this warp's 16 keys are not all outside
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        const int key = (mat >> 1) * 8 + mrow;
        const int chunk = kk * 2 + (mat & 1);
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, ks + key * D + ((chunk ^ (key & 7)) * 8));
        mma_bf16(s[0], qa[kk], b0, b1);
        mma_bf16(s[1], qa[kk], b2, b3);
      }
      const bool all_visible = key_base >= lo && key_base + DEC_KEYS <= hi;
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int t = 0; t < 2; ++t) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int abs_key = key_base + t * 8 + col + (e & 1);
          const float v = (all_visible || (abs_key >= lo && abs_key < hi)) ? s[t][e] * dp.scale_log2 : -INFINITY;
          s[t][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
      float corr[2], safe[2], sum[2] = {0.f, 0.f};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m_row[h], mx[h]);
        safe[h] = m_new == -INFINITY ? 0.f : m_new;
        corr[h] = exp2f(m_row[h] - safe[h]);                 // 2^(-inf) = 0 the first time
        m_row[h] = m_new;
      }
#pragma unroll
      for (int t = 0; t < 2; ++t) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = exp2f(s[t][e] - safe[e >> 1]);    // masked keys give 0
          s[t][e] = pv;
          sum[e >> 1] += pv;
        }
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 1);
        sum[h] += __shfl_xor_sync(0xffffffffu, sum[h], 2);
        l_row[h] = l_row[h] * corr[h] + sum[h];
      }
      unsigned pa[4];
      pa[0] = pack_bf16(s[0][0], s[0][1]);
      pa[1] = pack_bf16(s[0][2], s[0][3]);
      pa[2] = pack_bf16(s[1][0], s[1][1]);
      pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
      for (int t = 0; t < NT_O; t += 2) {
        o[t][0] *= corr[0]; o[t][1] *= corr[0]; o[t][2] *= corr[1]; o[t][3] *= corr[1];
        o[t + 1][0] *= corr[0]; o[t + 1][1] *= corr[0]; o[t + 1][2] *= corr[1]; o[t + 1][3] *= corr[1];
        const int key = (mat & 1) * 8 + mrow;
        const int chunk = t + (mat >> 1);
        unsigned b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, vs + key * D + ((chunk ^ (key & 7)) * 8));
        mma_bf16(o[t], pa, b0, b1);
        mma_bf16(o[t + 1], pa, b2, b3);
      }
    }
    __syncwarp();                          // this stage is overwritten by the copies of the round after next
  }

  // merge the four warps in warp order: staged as [warp][head][D + 2] floats over the key buffers
  __syncthreads();
  float* stage_f = reinterpret_cast<float*>(smem_raw);
  {
    const int r0 = lane >> 2;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int head = r0 + 8 * h;
      if (head < groups) {
        float* dst = stage_f + ((size_t)warp * groups + head) * (D + 2);
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
  float* mine = stage_f + (size_t)DEC_WARPS * groups * (D + 2);          // CLUSTER: this block's [head][D + 2]
  for (int i = threadIdx.x; i < groups * D; i += blockDim.x) {
    const int head = i / D, e = i % D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, stage_f[((size_t)w * groups + head) * (D + 2) + D]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float* src = stage_f + ((size_t)w * groups + head) * (D + 2);
      const float weight = src[D + 1] > 0.f ? exp2f(src[D] - m) : 0.f;    // a warp without keys adds nothing
      acc += src[e] * weight;
      l += src[D + 1] * weight;
    }
    if (CLUSTER) {
      mine[head * (D + 2) + e] = acc;
      if (e == 0) {
        mine[head * (D + 2) + D] = m;      // in units of log2
        mine[head * (D + 2) + D + 1] = l;
      }
      continue;
    }
    const size_t slot = ((size_t)row * p.n_q + (size_t)kv_head * groups + head) * p.max_splits + split;
    part_acc[slot * D + e] = acc;
    if (e == 0) {
      part_ml[slot * 2] = m;             // in units of log2
      part_ml[slot * 2 + 1] = l;
    }
  }
  if (CLUSTER) {
    // Every block of the cluster takes a slice of the (head, element) pairs and merges the blocks'
    // results for it, in block order, reading the others' shared memory.
    srb_cluster_sync();
    const int blocks = p.max_splits;                       // = cluster size
    const int total = groups * D;
    const int per_block = (total + blocks - 1) / blocks;
    const int begin = min(total, (int)srb_cluster_rank() * per_block), end = min(total, begin + per_block);
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
      const int head = i / D, e = i % D;
      const float* base = mine + head * (D + 2);
      float ms[8], ls[8], as[8];
      float m = -INFINITY;
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        if (b < blocks) {
          ms[b] = srb_load_peer_shared(base + D, b);
          ls[b] = srb_load_peer_shared(base + D + 1, b);
          as[b] = srb_load_peer_shared(base + e, b);
          m = fmaxf(m, ms[b]);
        }
      }
      float acc = 0.f, l = 0.f;
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        if (b < blocks) {
          const float weight = ls[b] > 0.f ? exp2f(ms[b] - m) : 0.f;      // a block without keys adds nothing
          acc += as[b] * weight;
          l += ls[b] * weight;
        }
      }
      out[((size_t)row * p.n_q + (size_t)kv_head * groups + head) * D + e] =
          __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    }
    srb_cluster_sync();                                    // nobody leaves while its memory may still be read
    srb_mark(SRB_MARK_DECODE_ATTENTION, 2);
    return;
  }

  // The block that arrives last at this (row, kv head) merges all splits, in split order, so
  // the result does not depend on which block that is.  The counter returns to zero.
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* counter = counters + (size_t)row * p.n_kv + kv_head;
    const int ticket = atomicAdd(counter, 1);
    is_last = ticket == count - 1;
    if (is_last) *counter = 0;
  }
  __syncthreads();
  if (!is_last) {
    srb_mark(SRB_MARK_DECODE_ATTENTION, 2);
    return;
  }
  __threadfence();
  float* weights = stage_f;              // [groups][count + 1]: 2^(m_s - M) per split, then 1 / sum
  for (int head = warp; head < groups; head += DEC_WARPS) {
    const size_t first = ((size_t)row * p.n_q + (size_t)kv_head * groups + head) * p.max_splits;
    // lane s holds split s (and s + 32, ...): maxima and sums go through the fixed butterfly of the warp,
    // so their order does not depend on which block merges
    float m = -INFINITY;
    for (int sp = lane; sp < count; sp += 32) m = fmaxf(m, __ldcg(part_ml + (first + sp) * 2));
    m = srb_warp_max(m);
    float lw = 0.f;
    for (int sp = lane; sp < count; sp += 32) {
      const float w = exp2f(__ldcg(part_ml + (first + sp) * 2) - m);
      lw += __ldcg(part_ml + (first + sp) * 2 + 1) * w;
      weights[head * (count + 1) + sp] = w;
    }
    const float l = srb_warp_sum(lw);
    if (lane == 0) weights[head * (count + 1) + count] = 1.0f / l;
  }
  __syncthreads();
  // four (head, element) pairs per thread and eight splits at a time: 32 loads in flight, added in split order
  const int total = groups * D;
  for (int i0 = threadIdx.x; i0 < total; i0 += 4 * blockDim.x) {
    const float* src[4];
    const float* w[4];
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int i = min(i0 + q * (int)blockDim.x, total - 1);
      const int head = i / D, e = i % D;
      src[q] = part_acc + ((size_t)row * p.n_q + (size_t)kv_head * groups + head) * p.max_splits * D + e;
      w[q] = weights + head * (count + 1);
    }
    for (int base = 0; base < count; base += 8) {
      float v[4][8];
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int j = 0; j < 8; ++j) v[q][j] = base + j < count ? __ldcg(src[q] + (size_t)(base + j) * D) : 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (base + j < count) acc[q] += v[q][j] * w[q][base + j];
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int i = i0 + q * (int)blockDim.x;
      if (i < total) {
        const int head = i / D, e = i % D;
        out[((size_t)row * p.n_q + (size_t)kv_head * groups + head) * D + e] = __float2bfloat16_rn(acc[q] * w[q][count]);
      }
    }
  }
  srb_mark(SRB_MARK_DECODE_ATTENTION, 2);
}

template <int D>
static int launch_decode(const void* q, const void* k_pool, const void* v_pool, void* out, float* part_acc,
                         float* part_ml, int* counters, const DecodeParams& dp, int rows, cudaStream_t s) {
  const int groups = dp.a.n_q / dp.a.n_kv;
  const size_t keys = (size_t)DEC_WARPS * DEC_STAGES * 2 * DEC_KEYS * D * sizeof(__nv_bfloat16);
  // up to 8 blocks per (row, kv head) merge inside a cluster, when all blocks run at once (then the
  // merge is the tail of the kernel; with several waves of blocks the placement of whole clusters costs
  // more than it saves); the merge needs room for one more [head][D + 2]
  const bool cluster = dp.a.max_splits > 1 && dp.a.max_splits <= 8 &&
                       (long long)rows * dp.a.n_kv * dp.a.max_splits <= 3 * srb_sm_count();
  const size_t merge = (size_t)(DEC_WARPS + 1) * groups * (D + 2) * sizeof(float);
  const size_t smem = cluster && merge > keys ? merge : keys;
  auto kernel = cluster ? decode_attention_kernel<D, true> : decode_attention_kernel<D, false>;
  if (smem > 48 * 1024)
    SRB_CUDA_CALL(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(dp.a.max_splits, dp.a.n_kv, rows);
  SRB_CUDA_CALL(srb_launch_clustered(kernel, grid, dim3(DEC_WARPS * 32), smem, s, dim3(cluster ? dp.a.max_splits : 1, 1, 1),
                                     (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool,
                                     part_acc, part_ml, (__nv_bfloat16*)out, counters, dp));
  return SRB_OK;
}

// 1 if this kernel takes the sizes, 0 if the generic one has to be used.
extern "C" int srb_decode_attention_supports(int n_q, int n_kv, int head_dim, int dtype) {
  return dtype == SRB_DTYPE_BF16 && (head_dim == 64 || head_dim == 128) && n_kv > 0 && n_q % n_kv == 0 &&
         n_q / n_kv <= 16;
}

// q, out: [rows, n_q, head_dim] bfloat16; pools [pages, n_kv, page_size, head_dim]; one row per decoded
// token.  `num_splits` blocks share the keys of a (row, kv head); scratch: part_acc holds
// rows * n_q * num_splits * head_dim floats, part_ml rows * n_q * num_splits * 2; `counters` holds
// rows * n_kv ints that are zero before the call and zero again after it.
extern "C" int srb_decode_attention(const void* q, const void* k_pool, const void* v_pool, void* out,
                                    float* part_acc, float* part_ml, int* counters, const int* positions,
                                    const int* row_request, const int* block_table, int table_stride, int rows,
                                    int n_q, int n_kv, int head_dim, int page_size, int num_pages, int window,
                                    int num_splits, float scale, int* error_word, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (!srb_decode_attention_supports(n_q, n_kv, head_dim, SRB_DTYPE_BF16))
    SRB_FAIL("decode_attention: head_dim %d (64 or 128) or %d query heads per kv head (at most 16) is not taken "
             "by this kernel", head_dim, n_kv > 0 ? n_q / n_kv : 0);
  if (page_size <= 0 || num_pages <= 0 || table_stride <= 0 || num_splits <= 0 || window < 0)
    SRB_FAIL("decode_attention: page size, page count, table stride and split count must be positive");
  if (!part_acc || !part_ml || !counters) SRB_FAIL("decode_attention: scratch memory and counters are needed");
  if (rows > 65535 || n_kv > 65535) SRB_FAIL("decode_attention: %d rows or %d kv heads exceed one launch", rows, n_kv);
  DecodeParams dp;
  AttnParams& p = dp.a;
  p.positions = positions; p.row_request = row_request; p.block_table = block_table;
  p.table_stride = table_stride; p.n_q = n_q; p.n_kv = n_kv; p.head_dim = head_dim;
  p.page_size = page_size; p.num_pages = num_pages; p.window = window; p.split_size = 0;
  p.max_splits = num_splits; p.scale = scale; p.error_word = error_word;
  dp.scale_log2 = scale * 1.4426950408889634f;
  cudaStream_t s = (cudaStream_t)stream;
  if (head_dim == 64) return launch_decode<64>(q, k_pool, v_pool, out, part_acc, part_ml, counters, dp, rows, s);
  return launch_decode<128>(q, k_pool, v_pool, out, part_acc, part_ml, counters, dp, rows, s);
}
