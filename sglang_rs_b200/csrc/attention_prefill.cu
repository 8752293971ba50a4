// Attention of prompt portions over the paged cache in bfloat16, tensor-core form.
//
// Same formula and key ranges as the generic kernel (attention_kernels.cuh).  One block per
// (tile of up to 64 consecutive rows of one request, query head).  Its four warps own 16
// rows each.  The keys the tile may see are walked in blocks of 64 aligned to absolute
// positions, brought from the pages into shared memory by 16-byte asynchronous copies, two
// blocks in flight; S = Q K^T and O += P V run on mma.sync m16n8k16 with the running
// maximum and sum of the online softmax in 32-bit (crates/sglang-kernel/src/cuda_attention.rs:
// 137-151 is the reference's per-key form of the same recurrence); exponentials are taken as
// 2^(s log2 e - m), one ex2 instruction each.  A row's arithmetic
// depends only on its own position: blocks are absolute, and a block that lies wholly
// outside a warp's rows is skipped without changing anything.
//
// `tiles` holds four ints per tile: first row of the step, number of rows, index of the
// request in the block table, position of the first row.
//
// Sizes: head_dim 64 or 128; any number of heads and groups, any page size, optional window.
#include "attention_kernels.cuh"
#include "mma_helpers.cuh"

SRB_DEFINE_LAST_ERROR()

#define PF_ROWS 64
#define PF_KEYS 64
#define PF_WARPS 4

template <int D>
__global__ void __launch_bounds__(PF_WARPS * 32, 3)
prefill_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                         const __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ out,
                         const int* __restrict__ tiles, AttnParams p) {
  constexpr int CHUNKS = D / 8;
  constexpr int KSTEPS = D / 16;
  constexpr int NT_S = PF_KEYS / 8;
  constexpr int NT_O = D / 8;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __nv_bfloat16* kv = reinterpret_cast<__nv_bfloat16*>(smem_raw);        // [2 stages][K, V][64][D]
  // Q passes through the second stage before the first copy into it is issued; it then lives in
  // registers, so a block needs 64 KB at head_dim 128 and three blocks share an SM.
  __nv_bfloat16* qs = kv + 2 * PF_KEYS * D;                              // [64][D]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heads are the fast grid dimension: tiles arrive sorted by falling work, so the long ones start first
  const int tile = blockIdx.y, head = blockIdx.x;
  const int groups = p.n_q / p.n_kv;
  const int kv_head = head / groups;
  const int row_begin = tiles[4 * tile], n_rows = tiles[4 * tile + 1];
  const int request = tiles[4 * tile + 2], pos_begin = tiles[4 * tile + 3];
  const int kv_lo = (p.window > 0 && pos_begin + 1 > p.window) ? pos_begin + 1 - p.window : 0;
  const int kv_hi = pos_begin + n_rows;                                  // keys 0 .. last row's position
  const int first_block = kv_lo / PF_KEYS, last_block = (kv_hi - 1) / PF_KEYS;

  for (int i = threadIdx.x; i < PF_ROWS * CHUNKS; i += blockDim.x) {
    const int r = i / CHUNKS, c = i % CHUNKS;
    const bool valid = r < n_rows;
    const __nv_bfloat16* src = q + ((size_t)(row_begin + (valid ? r : 0)) * p.n_q + head) * D + c * 8;
    cp_async_16(qs + r * D + ((c ^ (r & 7)) * 8), src, valid ? 16 : 0);
  }
  cp_async_commit();

  const int page_shift = (p.page_size & (p.page_size - 1)) == 0 ? __ffs(p.page_size) - 1 : -1;
  auto load_block = [&](int block, int stage) {
    __nv_bfloat16* ks = kv + (size_t)stage * 2 * PF_KEYS * D;
    __nv_bfloat16* vs = ks + PF_KEYS * D;
    for (int i = threadIdx.x; i < PF_KEYS * CHUNKS; i += blockDim.x) {
      const int key = i / CHUNKS, c = i % CHUNKS;
      const int abs_key = block * PF_KEYS + key;
      bool valid = abs_key >= kv_lo && abs_key < kv_hi;
      long long offset = 0;
      if (valid) {
        const int logical = page_shift >= 0 ? abs_key >> page_shift : abs_key / p.page_size;
        const int within = page_shift >= 0 ? abs_key & (p.page_size - 1) : abs_key % p.page_size;
        const int page = p.block_table[(size_t)request * p.table_stride + logical];
        if (page < 0 || page >= p.num_pages) {
          atomicOr(p.error_word, SRB_FLAG_BAD_PAGE);
          valid = false;
        } else {
          offset = (((long long)page * p.n_kv + kv_head) * p.page_size + within) * D + c * 8;
        }
      }
      const int where = key * D + ((c ^ (key & 7)) * 8);
      cp_async_16(ks + where, k_pool + offset, valid ? 16 : 0);
      cp_async_16(vs + where, v_pool + offset, valid ? 16 : 0);
    }
    cp_async_commit();
  };
  load_block(first_block, 0);

  const int g = lane >> 2, col = (lane & 3) * 2;
  const int mat = lane >> 3, mrow = lane & 7;
  // rows of this thread inside the tile and their positions
  const int r_in[2] = {warp * 16 + g, warp * 16 + g + 8};
  const int pos_r[2] = {pos_begin + r_in[0], pos_begin + r_in[1]};
  const int lowest_r[2] = {(p.window > 0 && pos_r[0] + 1 > p.window) ? pos_r[0] + 1 - p.window : 0,
                           (p.window > 0 && pos_r[1] + 1 > p.window) ? pos_r[1] + 1 - p.window : 0};
  const float scale_log2 = p.scale * 1.4426950408889634f;
  const int warp_first_pos = pos_begin + warp * 16;
  const int warp_last_pos = pos_begin + min(warp * 16 + 15, n_rows - 1);
  const bool warp_has_rows = warp * 16 < n_rows;

  unsigned qa[KSTEPS][4];
  cp_async_wait<0>();
  __syncthreads();
#pragma unroll
  for (int kk = 0; kk < KSTEPS; ++kk) {
    const int r = warp * 16 + (mat & 1) * 8 + mrow;
    const int chunk = kk * 2 + (mat >> 1);
    ldmatrix_x4(qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], qs + r * D + ((chunk ^ (r & 7)) * 8));
  }
  __syncthreads();                                      // the second stage may be overwritten from here on
  float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
  float o[NT_O][4];
#pragma unroll
  for (int t = 0; t < NT_O; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;

  for (int block = first_block; block <= last_block; ++block) {
    const int stage = (block - first_block) & 1;
    if (block < last_block) {
      load_block(block + 1, stage ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int block_lo = block * PF_KEYS, block_hi = block_lo + PF_KEYS;
    // the block matters to this warp if some key in it is visible to one of the warp's rows
    const int warp_window_lo = (p.window > 0 && warp_first_pos + 1 > p.window) ? warp_first_pos + 1 - p.window : 0;
    if (warp_has_rows && block_lo <= warp_last_pos && block_hi > warp_window_lo) {
      const __nv_bfloat16* ks = kv + (size_t)stage * 2 * PF_KEYS * D;
      const __nv_bfloat16* vs = ks + PF_KEYS * D;
      float s[NT_S][4];
#pragma unroll
      for (int t = 0; t < NT_S; ++t) s[t][0] = s[t][1] = s[t][2] = s[t][3] = 0.f;
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
      // Scores are kept in units of log2: s * scale * log2(e), so that the exponentials are
      // single ex2 instructions; the maximum and the sum are 32-bit as before.  A block whose
      // keys are visible to every row of the warp (the common case below the diagonal) skips
      // the comparisons.
      float mx[2] = {-INFINITY, -INFINITY};
      const bool all_visible = warp * 16 + 15 < n_rows && block_hi - 1 <= warp_first_pos &&
                               (p.window == 0 || block_lo >= pos_begin + warp * 16 + 15 + 1 - p.window);
      if (all_visible) {
#pragma unroll
        for (int t = 0; t < NT_S; ++t) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            s[t][e] *= scale_log2;
            mx[e >> 1] = fmaxf(mx[e >> 1], s[t][e]);
          }
        }
      } else {
#pragma unroll
        for (int t = 0; t < NT_S; ++t) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int h = e >> 1;
            const int key = block_lo + t * 8 + col + (e & 1);
            const bool visible = r_in[h] < n_rows && key <= pos_r[h] && key >= lowest_r[h];
            const float v = visible ? s[t][e] * scale_log2 : -INFINITY;
            s[t][e] = v;
            mx[h] = fmaxf(mx[h], v);
          }
        }
      }
      float corr[2], safe[2], sum[2] = {0.f, 0.f};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m_row[h], mx[h]);
        safe[h] = m_new == -INFINITY ? 0.f : m_new;       // a row that has seen no key yet
        corr[h] = exp2f(m_row[h] - safe[h]);              // 2^(-inf) = 0 the first time
        m_row[h] = m_new;
      }
#pragma unroll
      for (int t = 0; t < NT_S; ++t) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = exp2f(s[t][e] - safe[e >> 1]);
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
#pragma unroll
      for (int t = 0; t < NT_O; ++t) {
        o[t][0] *= corr[0]; o[t][1] *= corr[0];
        o[t][2] *= corr[1]; o[t][3] *= corr[1];
      }
#pragma unroll
      for (int kk = 0; kk < PF_KEYS / 16; ++kk) {
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
    __syncthreads();          // this stage is overwritten by the copy issued in the next round
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (r_in[h] >= n_rows) continue;
    const float inv = 1.0f / l_row[h];
    __nv_bfloat16* dst = out + ((size_t)(row_begin + r_in[h]) * p.n_q + head) * D;
#pragma unroll
    for (int t = 0; t < NT_O; ++t)
      *reinterpret_cast<unsigned*>(dst + t * 8 + col) = pack_bf16(o[t][2 * h] * inv, o[t][2 * h + 1] * inv);
  }
}

template <int D>
static int launch_prefill(const void* q, const void* k_pool, const void* v_pool, void* out, const int* tiles,
                          int num_tiles, const AttnParams& p, cudaStream_t s) {
  const size_t smem = (size_t)(4 * PF_KEYS) * D * sizeof(__nv_bfloat16);
  SRB_CUDA_CALL(cudaFuncSetAttribute(prefill_attention_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)smem));
  dim3 grid(p.n_q, num_tiles);
  if (num_tiles > 65535) SRB_FAIL("prefill_attention: %d tiles exceed one launch", num_tiles);
  prefill_attention_kernel<D><<<grid, PF_WARPS * 32, smem, s>>>(
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out,
      tiles, p);
  SRB_LAUNCH_CHECK("prefill_attention");
  return SRB_OK;
}

extern "C" int srb_prefill_attention_supports(int n_q, int n_kv, int head_dim, int dtype) {
  return dtype == SRB_DTYPE_BF16 && (head_dim == 64 || head_dim == 128) && n_kv > 0 && n_q % n_kv == 0;
}

extern "C" int srb_prefill_tile_rows() { return PF_ROWS; }

// q, out: [rows, n_q, head_dim] of the whole step; tiles: [num_tiles, 4] ints (see the top).
extern "C" int srb_prefill_attention(const void* q, const void* k_pool, const void* v_pool, void* out,
                                     const int* tiles, int num_tiles, const int* block_table, int table_stride,
                                     int n_q, int n_kv, int head_dim, int page_size, int num_pages, int window,
                                     float scale, int* error_word, void* stream) {
  if (num_tiles <= 0) return SRB_OK;
  if (!srb_prefill_attention_supports(n_q, n_kv, head_dim, SRB_DTYPE_BF16))
    SRB_FAIL("prefill_attention: head_dim %d is not 64 or 128, or %d query heads are no multiple of %d kv heads",
             head_dim, n_q, n_kv);
  if (page_size <= 0 || num_pages <= 0 || table_stride <= 0 || window < 0)
    SRB_FAIL("prefill_attention: page size, page count and table stride must be positive");
  AttnParams p;
  p.positions = nullptr; p.row_request = nullptr; p.block_table = block_table;
  p.table_stride = table_stride; p.n_q = n_q; p.n_kv = n_kv; p.head_dim = head_dim;
  p.page_size = page_size; p.num_pages = num_pages; p.window = window; p.split_size = 0;
  p.max_splits = 1; p.scale = scale; p.error_word = error_word;
  cudaStream_t s = (cudaStream_t)stream;
  if (head_dim == 64) return launch_prefill<64>(q, k_pool, v_pool, out, tiles, num_tiles, p, s);
  return launch_prefill<128>(q, k_pool, v_pool, out, tiles, num_tiles, p, s);
}
