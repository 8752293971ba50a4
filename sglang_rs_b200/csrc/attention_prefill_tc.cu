// Attention of prompt portions over the paged cache in bfloat16 on the 5th-generation tensor
// cores: S = Q K^T and O += P V are tcgen05.mma with S, P and O in tensor memory; Q, K and V
// come into shared memory by TMA (128-byte swizzle), K and V page by page through the block
// table.
//
// Same formula and key ranges as the generic kernel (attention_kernels.cuh).  One block per
// (tile of up to 128 consecutive rows of one request, HEADS query heads of one kv head).  Two
// heads share a block when the heads of a kv head pair up: they read the same K and V tiles,
// which halves the traffic from L2.  Warps:
//   warp 0           copies Q and the K tiles;  the last warp copies the V tiles;
//   warps 1..HEADS   issue the products of one head each (warp 1 owns the tensor memory);
//   4 warps per head softmax: thread t owns row t of the tile (one TMEM lane), so a row's maximum
//                    and sum need no exchange between threads.  Scores are kept in units of log2;
//                    the running maximum only moves (and O is only rescaled) when it grows by more
//                    than 2^8, which bounds P by 2^8 and keeps the result exact up to 32-bit
//                    rounding.
// Copy and product warps run converged and let one elected lane issue, so that addresses and
// descriptors stay in uniform registers.  S has two buffers per head: S of block i+1 is computed
// while the softmax of block i runs; P overwrites the scores it was computed from.
// Key blocks are aligned to absolute multiples of 64, so a row's arithmetic depends on its
// own position only.  `tiles` holds four ints per tile: first row of the step, number of rows,
// index of the request in the block table, position of the first row.
//
// Sizes: head_dim 64 or 128; page size a multiple of 8 that divides 64.  With one head a block
// needs 96 KB of shared memory and 256 columns of tensor memory and two blocks share an SM; with
// two heads a block takes 193 KB, all 512 columns and the SM.
// Every mbarrier wait is bounded; a wait that runs out flags SRB_FLAG_WAIT_TIMEOUT, every role
// leaves its loop, tensor memory is freed and the block returns.  No TMA load uses multicast.
#include "attention_kernels.cuh"
#include "tcgen05_helpers.cuh"

SRB_DEFINE_LAST_ERROR()
SRB_DEFINE_TIMELINE()

#define TC_ROWS 128
#define TC_KEYS 64
#define TC_RESCALE_STEP 8.0f      // in units of log2

struct TcArgs {
  const int* tiles;
  const int* block_table;
  __nv_bfloat16* out;
  int table_stride, n_q, n_kv, page_size, pool_rows, window;
  float scale_log2;
  int* error_word;
};

// M = 128, N = n, A and B bfloat16, D float; b_mn_major: B is [K rows][N contiguous] (V), else K-major
__host__ __device__ constexpr unsigned tc_idesc(int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((unsigned)(n >> 3) << 17) |
         ((unsigned)(TC_ROWS >> 4) << 24);
}

// descriptor of a tile read as [K rows of 128 bytes][N]: 8-row groups 1024 bytes apart (stride), blocks
// of 64 N-elements `lbo` bytes apart (leading)
__device__ __forceinline__ unsigned long long smem_descriptor_mn(unsigned address, unsigned lbo) {
  unsigned long long d = 0;
  d |= (unsigned long long)((address & 0x3ffffu) >> 4);
  d |= (unsigned long long)((lbo >> 4) & 0x3fffu) << 16;
  d |= (unsigned long long)(1024u >> 4) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}


// ---- arithmetic of the softmax threads: sm_100 has a three-input maximum and two-wide 32-bit
// multiply-add and add; ex2.approx is the hardware's base-2 exponential (2 ulp, 2^-inf = 0)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float ex2(float a) {
  float d;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(d) : "f"(a));
  return d;
}
__device__ __forceinline__ unsigned long long pack2(float a, float b) {
  unsigned long long d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(a), "f"(b));
  return d;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// HEADS query heads of one kv head share a block (1 or 2): they read the same K and V tiles from
// shared memory, which halves the traffic from L2.  STAGES tiles of K and of V are in flight.

template <int D, int HEADS, int STAGES>
__global__ void __launch_bounds__(64 + 160 * HEADS, HEADS == 1 ? 2 : 1)
prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_out,
                            TcArgs args) {
  constexpr int HALVES = D / 64;                           // 64-element (128-byte) column blocks of a head
  constexpr int Q_HALF_BYTES = TC_ROWS * 128;              // [128 rows][64] bfloat16
  constexpr int HALF_BYTES = TC_KEYS * 128;                // [64 keys][64] bfloat16
  constexpr int Q_BYTES = HALVES * Q_HALF_BYTES;
  constexpr int KV_BYTES = HALVES * HALF_BYTES;
  // tensor-memory columns, 256 per head: two S buffers of 64 columns, then O.  P (bfloat16 pairs,
  // 32 columns) overwrites the first half of the S buffer it was computed from.
  constexpr unsigned S_COL = 0, O_COL = 128, HEAD_COLUMNS = 256;
  constexpr unsigned TMEM_COLUMNS = HEAD_COLUMNS * HEADS;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
  unsigned char* q_smem = smem;                            // HEADS tiles of Q
  unsigned char* k_smem = smem + HEADS * Q_BYTES;          // STAGES tiles of K, then STAGES tiles of V
  unsigned char* v_smem = k_smem + STAGES * KV_BYTES;
  __shared__ __align__(8) unsigned long long q_full, k_full[STAGES], v_full[STAGES], k_empty[STAGES], v_empty[STAGES],
      s_ready[HEADS][2], p_ready[HEADS][2], pv_done[HEADS][2], o_ready[HEADS];
  __shared__ unsigned tmem_holder;
  __shared__ int abort_flag;

  srb_mark(SRB_MARK_PREFILL_ATTENTION, 0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heads are the fast grid dimension: tiles arrive sorted by falling work, so the long ones start first
  const int tile = blockIdx.y, head0 = blockIdx.x * HEADS;
  const int groups = args.n_q / args.n_kv;
  const int kv_head = head0 / groups;
  const int row_begin = args.tiles[4 * tile], n_rows = args.tiles[4 * tile + 1];
  const int request = args.tiles[4 * tile + 2], pos_begin = args.tiles[4 * tile + 3];
  const int kv_lo = (args.window > 0 && pos_begin + 1 > args.window) ? pos_begin + 1 - args.window : 0;
  const int kv_hi = pos_begin + n_rows;
  const int first_block = kv_lo / TC_KEYS, last_block = (kv_hi - 1) / TC_KEYS;
  const int num_blocks = last_block - first_block + 1;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&q_full), 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&k_full[s]), 1);
      mbar_init(smem_u32(&v_full[s]), 1);
      mbar_init(smem_u32(&k_empty[s]), HEADS);             // one arrival per head's product warp
      mbar_init(smem_u32(&v_empty[s]), HEADS);
    }
    for (int t = 0; t < HEADS; ++t) {
      for (int b = 0; b < 2; ++b) {
        mbar_init(smem_u32(&s_ready[t][b]), 1);
        mbar_init(smem_u32(&p_ready[t][b]), 128);
        mbar_init(smem_u32(&pv_done[t][b]), 1);
      }
      mbar_init(smem_u32(&o_ready[t]), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_holder), TMEM_COLUMNS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = tmem_holder;
  srb_mark(SRB_MARK_PREFILL_ATTENTION, 1);                 // (no wait for the kernels ahead here: set-up is complete)

  constexpr int V_WARP = 1 + 5 * HEADS;                    // the last warp
  if (warp == 0 || warp == V_WARP) {
    // Copies, by two whole warps: warp 0 brings Q and the K tiles, the last warp the V tiles (the
    // issue of a copy costs some tens of cycles, and a 64-key tile of 16-token pages is 8 copies).
    // Lane l looks up page l of a 64-key block, one block ahead of its use, so the look-ups of a
    // block run side by side; one elected lane issues the copies.
    const bool is_k = warp == 0;
    const int pages_per_block = TC_KEYS / args.page_size;
    if (is_k && elect_one()) {
      // Q: [128 rows][D] of each head, as HALVES tiles of [128][64]
      mbar_expect_tx(smem_u32(&q_full), HEADS * Q_BYTES);
      for (int t = 0; t < HEADS; ++t)
        for (int h = 0; h < HALVES; ++h)
          tma_load_3d(smem_u32(q_smem + t * Q_BYTES + h * Q_HALF_BYTES), &map_q, smem_u32(&q_full), h * 64, head0 + t,
                      row_begin);
    }
    auto pool_row_of = [&](int block) {
      int row = args.pool_rows;                             // outside the pool: TMA fills zeros
      if (lane < pages_per_block && block < num_blocks) {
        const int key = (first_block + block) * TC_KEYS + lane * args.page_size;
        if (key < kv_hi && key + args.page_size > kv_lo) {
          const int page = args.block_table[(size_t)request * args.table_stride + key / args.page_size];
          if (page < 0 || (long long)(page + 1) * args.n_kv * args.page_size > args.pool_rows)
            atomicOr(args.error_word, SRB_FLAG_BAD_PAGE);
          else
            row = (page * args.n_kv + kv_head) * args.page_size;
        }
      }
      return row;
    };
    const unsigned ring = smem_u32(is_k ? k_smem : v_smem);
    const CUtensorMap* map = is_k ? &map_k : &map_v;
    unsigned long long* full = is_k ? k_full : v_full;
    unsigned long long* empty = is_k ? k_empty : v_empty;
    const unsigned page_bytes = (unsigned)args.page_size * 128u;
    int issued = 0;
    int rows_now = pool_row_of(0);
    for (int i = 0; i < num_blocks; ++i) {
      const int rows_next = pool_row_of(i + 1);             // in flight during this block's copies
      const int s = i % STAGES;
      if (!mbar_wait_warp(smem_u32(&empty[s]), ((unsigned)(i / STAGES) & 1u) ^ 1u, &abort_flag)) break;
      issued = i + 1;
      const unsigned bar = smem_u32(&full[s]);
      if (elect_one()) mbar_expect_tx(bar, KV_BYTES);
      const unsigned stage = ring + s * KV_BYTES;
      for (int pg = 0; pg < pages_per_block; ++pg) {
        const int row = __shfl_sync(0xffffffffu, rows_now, pg);
        if (elect_one())
          for (int h = 0; h < HALVES; ++h) tma_load_2d(stage + h * HALF_BYTES + pg * page_bytes, map, bar, h * 64, row);
      }
      rows_now = rows_next;
    }
    // copies still in flight write into this block's shared memory: wait for them before leaving
    __syncwarp();
    if (lane == 0 && abort_flag) {
      if (is_k) mbar_wait_timed(smem_u32(&q_full), 0);
      for (int i = max(0, issued - STAGES); i < issued; ++i)
        mbar_wait_timed(smem_u32(&full[i % STAGES]), (unsigned)(i / STAGES) & 1u);
    }
  } else if (warp <= HEADS) {
    // Products of one head, by the whole warp with one elected lane issuing (a warp per head: the
    // issue of a product costs some tens of cycles, and 64-key products are short).  S of block
    // i+1 is issued before the wait for P of block i, so the tensor pipe computes it while the
    // softmax warps work on block i; the pipe runs a warp's products in issue order, so S of block
    // i+1 lands in its buffer only after P V of block i-1 has read P from there.
    const int t = warp - 1;
    constexpr unsigned idesc_s = tc_idesc(TC_KEYS, false);
    constexpr unsigned idesc_o = tc_idesc(D, true);
    const unsigned long long q_desc = smem_descriptor(smem_u32(q_smem) + t * Q_BYTES);
    const unsigned long long k_desc = smem_descriptor(smem_u32(k_smem));
    const unsigned long long v_desc = smem_descriptor_mn(smem_u32(v_smem), HALF_BYTES);
    const unsigned head_tmem = tmem_base + t * HEAD_COLUMNS;
    bool ok = mbar_wait_warp(smem_u32(&q_full), 0, &abort_flag);
    auto issue_s = [&](int j) {
      const int s = j % STAGES;
      ok = mbar_wait_warp(smem_u32(&k_full[s]), (unsigned)(j / STAGES) & 1u, &abort_flag);
      if (!ok) return;
      tc_fence_after();
      const unsigned long long k_stage = k_desc + (unsigned long long)((s * KV_BYTES) >> 4);
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const unsigned q_off = (unsigned)((k / 4) * Q_HALF_BYTES + (k % 4) * 32) >> 4;
          const unsigned k_off = (unsigned)((k / 4) * HALF_BYTES + (k % 4) * 32) >> 4;
          umma_bf16(head_tmem + S_COL + (j & 1) * TC_KEYS, q_desc + q_off, k_stage + k_off, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&s_ready[t][j & 1]));
        umma_commit(smem_u32(&k_empty[s]));
      }
      __syncwarp();
    };
    if (ok) issue_s(0);
    for (int i = 0; i < num_blocks && ok; ++i) {
      if (i + 1 < num_blocks) {
        issue_s(i + 1);
        if (!ok) break;
      }
      const int s = i % STAGES;
      ok = mbar_wait_warp(smem_u32(&v_full[s]), (unsigned)(i / STAGES) & 1u, &abort_flag) &&
           mbar_wait_warp(smem_u32(&p_ready[t][i & 1]), (unsigned)(i >> 1) & 1u, &abort_flag);
      if (!ok) break;
      tc_fence_after();
      const unsigned long long v_stage = v_desc + (unsigned long long)((s * KV_BYTES) >> 4);
      // O += P V over the 64 keys in steps of 16 once the head's softmax warps have written P
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < TC_KEYS / 16; ++k)
          umma_bf16_tmem_a(head_tmem + O_COL, head_tmem + S_COL + (i & 1) * TC_KEYS + k * 8,
                           v_stage + (unsigned long long)((k * 16 * 128) >> 4), idesc_o, (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(smem_u32(&pv_done[t][i & 1]));
        umma_commit(smem_u32(&v_empty[s]));
        if (i == num_blocks - 1) umma_commit(smem_u32(&o_ready[t]));
      }
      __syncwarp();
    }
  } else {
    // softmax: four warps per head, thread = row
    const int t = (warp - 1 - HEADS) >> 2;
    const int head = head0 + t;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int pos_r = pos_begin + r;
    const int lowest_r = (args.window > 0 && pos_r + 1 > args.window) ? pos_r + 1 - args.window : 0;
    const bool row_live = r < n_rows;
    const unsigned lane_address = tmem_base + t * HEAD_COLUMNS + ((unsigned)(quarter * 32) << 16);
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int i = 0; i < num_blocks && ok; ++i) {
      const unsigned s_col = S_COL + (i & 1) * TC_KEYS;
      ok = mbar_wait(smem_u32(&s_ready[t][i & 1]), (unsigned)(i >> 1) & 1u, &abort_flag);
      if (!ok) break;
      tc_fence_after();
      const int key0 = (first_block + i) * TC_KEYS;
      const bool all_visible = n_rows == TC_ROWS && key0 + TC_KEYS - 1 <= pos_begin &&
                               (args.window == 0 || key0 >= pos_begin + TC_ROWS - args.window);
      // the row's 64 raw scores, once; masked keys become -inf
      float sv[TC_KEYS];
      tmem_load_64(lane_address + s_col, sv);
      if (!all_visible) {
#pragma unroll
        for (int j = 0; j < TC_KEYS; ++j) {
          const int key = key0 + j;
          if (!(row_live && key <= pos_r && key >= lowest_r)) sv[j] = -INFINITY;
        }
      }
      // three-input maxima, four chains
      float mx[4] = {sv[0], sv[1], sv[2], sv[3]};
#pragma unroll
      for (int j = 4; j < TC_KEYS - 4; j += 8) {
        mx[0] = max3(mx[0], sv[j], sv[j + 1]); mx[1] = max3(mx[1], sv[j + 2], sv[j + 3]);
        mx[2] = max3(mx[2], sv[j + 4], sv[j + 5]); mx[3] = max3(mx[3], sv[j + 6], sv[j + 7]);
      }
      mx[0] = max3(mx[0], sv[TC_KEYS - 4], sv[TC_KEYS - 3]);
      mx[1] = max3(mx[1], sv[TC_KEYS - 2], sv[TC_KEYS - 1]);
      const float m_block = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * args.scale_log2;   // in units of log2
      // the running maximum moves only when it must: P stays below 2^8
      float corr = 1.f;
      bool rescale = false;
      if (m_block > m_run + TC_RESCALE_STEP || m_run == -INFINITY) {
        const float m_new = fmaxf(m_run, m_block);
        if (m_new > -INFINITY) {
          corr = ex2(m_run - m_new);                       // 0 the first time
          rescale = m_run > -INFINITY;
          m_run = m_new;
        }
      }
      const float m_use = m_run == -INFINITY ? 0.f : m_run;
      if (__any_sync(0xffffffffu, rescale)) {
        // O is still being added to by P V of the block before: wait for that product
        ok = mbar_wait(smem_u32(&pv_done[t][(i - 1) & 1]), (unsigned)((i - 1) >> 1) & 1u, &abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          float ov[32];
          tmem_load_32(lane_address + O_COL + c, ov);
#pragma unroll
          for (int j = 0; j < 32; ++j) ov[j] *= corr;
          tmem_store_32(lane_address + O_COL + c, ov);
        }
      }
      l_run *= corr;
      // P = 2^(s * scale * log2 e - m), rounded to bfloat16 pairs, over the scores it came from; the row's sum
      // (two-wide 32-bit multiply-adds and adds; the exponential is one ex2 per score)
      const unsigned long long scale2 = pack2(args.scale_log2, args.scale_log2), neg_m2 = pack2(-m_use, -m_use);
      unsigned long long sums2[2] = {0ull, 0ull};
#pragma unroll
      for (int c = 0; c < TC_KEYS; c += 32) {
        unsigned packed[16];
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          float a0, a1, a2, a3;
          unpack2(fma2(pack2(sv[c + j], sv[c + j + 1]), scale2, neg_m2), a0, a1);
          unpack2(fma2(pack2(sv[c + j + 2], sv[c + j + 3]), scale2, neg_m2), a2, a3);
          const float p0 = ex2(a0), p1 = ex2(a1), p2 = ex2(a2), p3 = ex2(a3);          // 2^(-inf) = 0 for masked keys
          sums2[0] = add2(sums2[0], pack2(p0, p1));
          sums2[1] = add2(sums2[1], pack2(p2, p3));
          __nv_bfloat162 lo = __floats2bfloat162_rn(p0, p1), hi = __floats2bfloat162_rn(p2, p3);
          packed[j / 2] = *reinterpret_cast<unsigned*>(&lo);
          packed[j / 2 + 1] = *reinterpret_cast<unsigned*>(&hi);
        }
        tmem_store_16(lane_address + s_col + c / 2, packed);
      }
      float sum_a, sum_b, sum_c, sum_d;
      unpack2(sums2[0], sum_a, sum_b);
      unpack2(sums2[1], sum_c, sum_d);
      const float sum = (sum_a + sum_b) + (sum_c + sum_d);
      tmem_store_wait();
      l_run += sum;
      tc_fence_before();
      mbar_arrive(smem_u32(&p_ready[t][i & 1]));
    }
    if (ok) ok = mbar_wait(smem_u32(&o_ready[t]), 0, &abort_flag);
    // A whole tile leaves through shared memory and one bulk store per 64 columns: a thread's row lies 8 KB from its
    // neighbour's in the output, so stores from registers touch 32 lines per instruction.  The head's Q tile is free
    // (every S product has completed) and has the layout the store wants: [128 rows][128 bytes] per 64 columns,
    // 16-byte pieces exchanged by the 128-byte swizzle.
    const bool whole_tile = n_rows == TC_ROWS;
    unsigned char* stage = q_smem + t * Q_BYTES;
    if (ok) {
      tc_fence_after();
      const float inv = row_live && l_run > 0.f ? 1.0f / l_run : 0.f;
      __nv_bfloat16* dst = args.out + ((size_t)(row_begin + r) * args.n_q + head) * D;
#pragma unroll 2
      for (int c = 0; c < D; c += 32) {
        float ov[32];
        tmem_load_32(lane_address + O_COL + c, ov);
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 packed;
          __nv_bfloat162* pair = reinterpret_cast<__nv_bfloat162*>(&packed);
          pair[0] = __floats2bfloat162_rn(ov[j] * inv, ov[j + 1] * inv);
          pair[1] = __floats2bfloat162_rn(ov[j + 2] * inv, ov[j + 3] * inv);
          pair[2] = __floats2bfloat162_rn(ov[j + 4] * inv, ov[j + 5] * inv);
          pair[3] = __floats2bfloat162_rn(ov[j + 6] * inv, ov[j + 7] * inv);
          if (whole_tile) {
            const int column = c + j, piece = (column & 63) >> 3;
            *reinterpret_cast<uint4*>(stage + (column >> 6) * Q_HALF_BYTES + r * 128 + ((piece ^ (r & 7)) << 4)) = packed;
          } else if (row_live) {
            *reinterpret_cast<uint4*>(dst + c + j) = packed;
          }
        }
      }
    }
    if (whole_tile) {
      // (every warp of the head comes here, also one whose wait gave up: the barrier below counts all four)
      fence_proxy_async_shared();
      if (t == 0)
        asm volatile("bar.sync 1, 128;" ::: "memory");
      else
        asm volatile("bar.sync 2, 128;" ::: "memory");
      if (quarter == 0 && lane == 0 && !abort_flag) {
#pragma unroll
        for (int h = 0; h < HALVES; ++h)
          tma_store_3d(&map_out, smem_u32(stage + h * Q_HALF_BYTES), h * 64, head, row_begin);
        tma_store_commit_and_wait_read();
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag) atomicOr(args.error_word, SRB_FLAG_WAIT_TIMEOUT);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLUMNS);
  }
#ifdef SRB_TIMELINE
  // (thread 0 is in the K copy warp, which reaches the barrier above long before the softmax warps: its clock is read
  // only after a second barrier, which the warp that freed the tensor memory reaches last)
  __syncthreads();
  srb_mark(SRB_MARK_PREFILL_ATTENTION, 2);
#endif
}

// ------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool looked = false;
  if (!looked) {
    looked = true;
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &entry, 12000, cudaEnableDefault, &result) ==
            cudaSuccess && result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(entry);
  }
  return fn;
}

extern "C" int srb_prefill_tc_supports(int n_q, int n_kv, int head_dim, int page_size, int dtype) {
  return dtype == SRB_DTYPE_BF16 && (head_dim == 64 || head_dim == 128) && n_kv > 0 && n_q % n_kv == 0 &&
         page_size >= 8 && page_size % 8 == 0 && TC_KEYS % page_size == 0;
}

extern "C" int srb_prefill_tc_tile_rows() { return TC_ROWS; }

template <int D, int HEADS, int STAGES>
static int launch_tc(const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v, const CUtensorMap& map_out,
                     const TcArgs& args, int num_tiles, cudaStream_t s) {
  const size_t smem = (size_t)(D / 64) * 128 * (HEADS * TC_ROWS + 2 * STAGES * TC_KEYS) + 1024;
  auto kernel = prefill_attention_tc_kernel<D, HEADS, STAGES>;
  SRB_CUDA_CALL(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(args.n_q / HEADS, num_tiles);
  if (num_tiles > 65535) SRB_FAIL("prefill_attention_tc: %d tiles exceed one launch", num_tiles);
  kernel<<<grid, 64 + 160 * HEADS, smem, s>>>(map_q, map_k, map_v, map_out, args);
  SRB_LAUNCH_CHECK("prefill_attention_tc");
  return SRB_OK;
}

// q, out: [rows, n_q, head_dim] bfloat16 of the whole step; pools [pages, n_kv, page_size, head_dim];
// tiles: [num_tiles, 4] ints with at most 128 rows each.
extern "C" int srb_prefill_attention_tc(const void* q, const void* k_pool, const void* v_pool, void* out,
                                        const int* tiles, int num_tiles, int rows, const int* block_table,
                                        int table_stride, int n_q, int n_kv, int head_dim, int page_size,
                                        int num_pages, int window, float scale, int* error_word, void* stream) {
  if (num_tiles <= 0) return SRB_OK;
  if (!srb_prefill_tc_supports(n_q, n_kv, head_dim, page_size, SRB_DTYPE_BF16))
    SRB_FAIL("prefill_attention_tc: head_dim %d (64 or 128), page size %d (a multiple of 8 dividing 64) or the "
             "head counts are not taken by this kernel", head_dim, page_size);
  if (num_pages <= 0 || table_stride <= 0 || window < 0 || rows <= 0)
    SRB_FAIL("prefill_attention_tc: page count, table stride and rows must be positive");
  if ((((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15) != 0)
    SRB_FAIL("prefill_attention_tc: operands must be 16-byte aligned");
  EncodeTiledFn encode = encode_tiled();
  if (!encode) SRB_FAIL("prefill_attention_tc: the driver does not offer cuTensorMapEncodeTiled");
  CUtensorMap map_q, map_k, map_v, map_out;
  for (int pass = 0; pass < 2; ++pass) {                     // q, and the output of the same shape
    const cuuint64_t dims[3] = {(cuuint64_t)head_dim, (cuuint64_t)n_q, (cuuint64_t)rows};
    const cuuint64_t strides[2] = {(cuuint64_t)head_dim * 2, (cuuint64_t)n_q * head_dim * 2};
    const cuuint32_t box[3] = {64, 1, TC_ROWS};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult status = encode(pass == 0 ? &map_q : &map_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                                   pass == 0 ? const_cast<void*>(q) : out, dims, strides,
                                   box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (status != CUDA_SUCCESS) SRB_FAIL("prefill_attention_tc: tensor map of %s failed with %d", pass == 0 ? "q" : "the output", (int)status);
  }
  const long long pool_rows = (long long)num_pages * n_kv * page_size;
  if (pool_rows > 0x7fffffffll) SRB_FAIL("prefill_attention_tc: the pool has too many rows for one tensor map");
  for (int pass = 0; pass < 2; ++pass) {
    const cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)pool_rows};
    const cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult status = encode(pass == 0 ? &map_k : &map_v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                                   const_cast<void*>(pass == 0 ? k_pool : v_pool), dims, strides, box, elem,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (status != CUDA_SUCCESS) SRB_FAIL("prefill_attention_tc: tensor map of a pool failed with %d", (int)status);
  }
  TcArgs args;
  args.tiles = tiles; args.block_table = block_table; args.out = (__nv_bfloat16*)out; args.table_stride = table_stride;
  args.n_q = n_q; args.n_kv = n_kv; args.page_size = page_size; args.pool_rows = (int)pool_rows; args.window = window;
  args.scale_log2 = scale * 1.4426950408889634f; args.error_word = error_word;
  cudaStream_t s = (cudaStream_t)stream;
  // two query heads per block when the heads of a kv head pair up
  const bool pairs = (n_q / n_kv) % 2 == 0;
  if (head_dim == 64)
    return pairs ? launch_tc<64, 2, 4>(map_q, map_k, map_v, map_out, args, num_tiles, s)
                 : launch_tc<64, 1, 2>(map_q, map_k, map_v, map_out, args, num_tiles, s);
  return pairs ? launch_tc<128, 2, 4>(map_q, map_k, map_v, map_out, args, num_tiles, s)
               : launch_tc<128, 1, 2>(map_q, map_k, map_v, map_out, args, num_tiles, s);
}
