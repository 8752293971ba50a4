// Y = X W^T in bfloat16 with 32-bit accumulation on the 5th-generation tensor cores:
// tcgen05.mma with the accumulator in tensor memory, operands brought into shared memory
// by TMA (cp.async.bulk.tensor, 128-byte swizzle), mbarrier pipelines between a copy warp,
// an issue warp and four epilogue warps.
//
// The weight is the M side of the instruction ("swap-AB"): a block owns 128 rows of W
// [features, K] and up to 256 tokens of X [tokens, K]; both are K-major, so no transpose is
// needed anywhere, and a step with few tokens (decode) still fills the 128-wide M side of
// the unit while it streams W exactly once.  The accumulator tile is [128 features (TMEM
// lanes) x tokens (TMEM columns)]; the epilogue reads it with tcgen05.ld and stores
// out[token][feature], 32 consecutive features per warp store.
//
// Modes of the epilogue: bfloat16 store; float store (logits); SiLU(gate) * up, where the
// block's 128 weight rows are 64 gate rows over the 64 up rows of the same features, the two
// halves of the accumulator meet through shared memory and only the product is written; and
// float partials per K split, [split][token][feature], which
// the consumer adds in split order (few tokens cannot fill 148 SMs with 128-row blocks alone,
// so K is cut; the cut depends on the shape only); and the sum of the K splits added to a float
// tensor in place (the residual stream): the up to 8 blocks of a tile form a thread-block cluster,
// leave their partial tiles in shared memory and each adds a slice of the tile, over all blocks in
// block order, to the tensor.
//
// Weight layout and meaning as the reference's projection: row-major [out, in],
// y[o] = sum_i x[i] W[o, i] (crates/sglang-kernel/src/cpu.rs:73-108), bfloat16 inputs with
// 32-bit accumulation as its cuBLAS call (crates/sglang-kernel/src/cublas.rs:383-410).
//
// Every wait on an mbarrier is bounded (about a second of spinning); a wait that runs out
// sets SRB_FLAG_WAIT_TIMEOUT in the error word, every role leaves its loop, outstanding
// copies are waited for with the same bound, tensor memory is freed and the block returns.
// No TMA load uses cluster multicast.
#include "common.cuh"
#include "tcgen05_helpers.cuh"
#include "activations.cuh"
#include <mutex>

SRB_DEFINE_LAST_ERROR()
SRB_DEFINE_PDL_SWITCH()

#define GEMM_BLOCK_F 128      // weight rows (features) per block = M of the instruction
#define GEMM_BLOCK_K 64       // bfloat16 elements per 128-byte swizzle row
#define GEMM_UMMA_K 16
#define GEMM_THREADS 192      // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue

#define EPI_BF16 0
#define EPI_F32 1
#define EPI_SILU 2
#define EPI_PARTIAL 3
#define EPI_ADD 4          // out (float) += sum over the K splits, reduced inside a cluster

// Instruction descriptor: D float, A and B bfloat16, both K-major, M = 128, N = tokens.
__host__ __device__ constexpr unsigned instruction_descriptor(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(GEMM_BLOCK_F >> 4) << 24);
}

struct GemmArgs {
  void* out;                 // bf16 / float [tokens, ldo] or float partials [splits, tokens, ldo]
  int tokens, features, k;   // problem
  int ldo;                   // row pitch of out, in elements
  int up_row_offset;         // EPI_SILU: rows of the up matrix start here in W
  int activation;            // EPI_SILU: which SRB_ACT_* is applied to the gate half
  int k_blocks_per_split;
  int* error_word;
};

template <int BLOCK_T, int EPI, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, BLOCK_T <= 64 ? 2 : 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                 GemmArgs args) {
  // SiLU mode: the 128 rows of the A tile are 64 gate rows over the 64 up rows of the same features
  constexpr int A_BYTES = GEMM_BLOCK_F * GEMM_BLOCK_K * 2;
  constexpr int B_BYTES = BLOCK_T * GEMM_BLOCK_K * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int ACC_COLUMNS = BLOCK_T;
  constexpr int FEATURES_PER_BLOCK = EPI == EPI_SILU ? GEMM_BLOCK_F / 2 : GEMM_BLOCK_F;
  constexpr unsigned TMEM_COLUMNS = ACC_COLUMNS <= 32 ? 32 : ACC_COLUMNS <= 64 ? 64 : ACC_COLUMNS <= 128 ? 128
                                                                               : ACC_COLUMNS <= 256 ? 256 : 512;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_bar;
  __shared__ unsigned tmem_holder;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // token tiles are the fastest grid dimension: blocks that share a weight tile run together
  const int token0 = blockIdx.x * BLOCK_T;
  const int feature0 = blockIdx.y * FEATURES_PER_BLOCK;
  const int total_k_blocks = (args.k + GEMM_BLOCK_K - 1) / GEMM_BLOCK_K;
  const int kb_begin = blockIdx.z * args.k_blocks_per_split;
  const int kb_end = min(total_k_blocks, kb_begin + args.k_blocks_per_split);
  const int num_kb = max(kb_end - kb_begin, 0);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(&acc_bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&tmem_holder), TMEM_COLUMNS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = tmem_holder;

  srb_mark(SRB_MARK_PRODUCT, 0);
  srb_launch_dependents();
  if (warp == 0) {
    // Copies, by the whole warp with one elected lane issuing: addresses and coordinates stay in
    // uniform registers, which the copy instruction takes its operands from.
    int issued = 0;
    // The weights are written by no kernel of the step, so the first stages of W are
    // requested before the wait for the kernels ahead; X follows once they have completed.
    const int early = min(num_kb, STAGES);
    const unsigned smem_base = smem_u32(smem);
    bool ok = true;
    for (int i = 0; i < early && ok; ++i) {
      ok = mbar_wait_warp(smem_u32(&empty_bar[i]), 1u, &abort_flag);      // first use of a stage: free
      if (!ok) break;
      const unsigned bar = smem_u32(&full_bar[i]);
      const unsigned stage = smem_base + i * STAGE_BYTES;
      const int kx = (kb_begin + i) * GEMM_BLOCK_K;
      if (elect_one()) {
        mbar_expect_tx(bar, STAGE_BYTES);
        tma_load_2d(stage, &map_w, bar, kx, feature0);
        if (EPI == EPI_SILU) tma_load_2d(stage + A_BYTES / 2, &map_w, bar, kx, args.up_row_offset + feature0);
      }
      issued = i + 1;
    }
    srb_grid_dependency_wait();
    srb_mark(SRB_MARK_PRODUCT, 1);
    for (int i = 0; i < issued; ++i) {
      if (elect_one())
        tma_load_2d(smem_base + i * STAGE_BYTES + A_BYTES, &map_x, smem_u32(&full_bar[i]), (kb_begin + i) * GEMM_BLOCK_K,
                    token0);
    }
    for (int i = issued; i < num_kb && ok; ++i) {
      const int s = i % STAGES;
      const unsigned phase = (unsigned)(i / STAGES) & 1u;
      if (!mbar_wait_warp(smem_u32(&empty_bar[s]), phase ^ 1u, &abort_flag)) break;
      const unsigned bar = smem_u32(&full_bar[s]);
      const unsigned stage = smem_base + s * STAGE_BYTES;
      const int kx = (kb_begin + i) * GEMM_BLOCK_K;
      if (elect_one()) {
        mbar_expect_tx(bar, STAGE_BYTES);
        tma_load_2d(stage, &map_w, bar, kx, feature0);
        if (EPI == EPI_SILU) tma_load_2d(stage + A_BYTES / 2, &map_w, bar, kx, args.up_row_offset + feature0);
        tma_load_2d(stage + A_BYTES, &map_x, bar, kx, token0);
      }
      issued = i + 1;
    }
    // copies still in flight write into this block's shared memory: wait for them before leaving
    __syncwarp();
    if (lane == 0 && abort_flag) {
      for (int i = max(0, issued - STAGES); i < issued; ++i)
        mbar_wait_timed(smem_u32(&full_bar[i % STAGES]), (unsigned)(i / STAGES) & 1u);
    }
  } else if (warp == 1) {
    // Products, by the whole warp with one elected lane issuing.
    constexpr unsigned idesc = instruction_descriptor(BLOCK_T);
    const unsigned long long a_desc0 = smem_descriptor(smem_u32(smem));
    const unsigned long long b_desc0 = smem_descriptor(smem_u32(smem) + A_BYTES);
    bool ok = true;
    for (int i = 0; i < num_kb && ok; ++i) {
      const int s = i % STAGES;
      const unsigned phase = (unsigned)(i / STAGES) & 1u;
      ok = mbar_wait_warp(smem_u32(&full_bar[s]), phase, &abort_flag);
      if (!ok) break;
      tc_fence_after();
      const unsigned long long stage_step = (unsigned long long)((s * STAGE_BYTES) >> 4);
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < GEMM_BLOCK_K / GEMM_UMMA_K; ++k) {
          const unsigned accumulate = (i > 0 || k > 0) ? 1u : 0u;
          const unsigned long long step = stage_step + (unsigned long long)((k * GEMM_UMMA_K * 2) >> 4);
          umma_bf16(tmem_base, a_desc0 + step, b_desc0 + step, idesc, accumulate);
        }
        umma_commit(smem_u32(&empty_bar[s]));        // frees the stage when these products have read it
      }
      __syncwarp();
    }
    if (ok && elect_one()) umma_commit(smem_u32(&acc_bar));       // the accumulator is complete
    __syncwarp();
  } else {
    // epilogue: warp w may read TMEM lanes 32 * (w % 4) .. + 32
    srb_grid_dependency_wait();             // the output buffer may still be read by a kernel ahead
    const int quarter = warp & 3;
    // SiLU mode: lanes 0..63 hold gate, lanes 64..127 up of the same 64 features
    const int feature = EPI == EPI_SILU ? feature0 + (quarter & 1) * 32 + lane : feature0 + quarter * 32 + lane;
    bool ok = true;
    if (num_kb > 0) {
      ok = mbar_wait(smem_u32(&acc_bar), 0, &abort_flag);
      tc_fence_after();
    }
    // The pipeline's stages are idle once the accumulator is complete: in SiLU mode the up half
    // passes through them to the warps that hold the gate half ([64 features][16 tokens] floats).
    float* exchange = reinterpret_cast<float*>(smem);
    const unsigned lane_address = tmem_base + ((unsigned)(quarter * 32) << 16);
#pragma unroll 1
    for (int c = 0; c < BLOCK_T; c += 16) {
      if (token0 + c >= args.tokens) break;            // the same for all epilogue warps
      float acc[16];
      if (ok && num_kb > 0) {
        tmem_load_16(lane_address + c, acc);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = 0.f;
      }
      if (EPI == EPI_SILU) {
        if (quarter >= 2) {
#pragma unroll
          for (int j = 0; j < 16; ++j) exchange[((quarter & 1) * 32 + lane) * 16 + j] = acc[j];
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");       // the four epilogue warps only
        if (quarter < 2 && ok && feature < args.features) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int token = token0 + c + j;
            if (token >= args.tokens) break;
            const float g = acc[j], u = exchange[((quarter & 1) * 32 + lane) * 16 + j];
            reinterpret_cast<__nv_bfloat16*>(args.out)[(size_t)token * args.ldo + feature] =
                __float2bfloat16_rn(srb_gated<true>(args.activation, g, u));
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");       // the buffer is reused by the next 16 tokens
      } else if (EPI == EPI_ADD) {
        // this block's partial tile as [token][128 features] floats over the idle pipeline stages
#pragma unroll
        for (int j = 0; j < 16; ++j) exchange[(c + j) * GEMM_BLOCK_F + quarter * 32 + lane] = acc[j];
      } else if (ok && feature < args.features) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int token = token0 + c + j;
          if (token >= args.tokens) break;
          if (EPI == EPI_BF16) {
            reinterpret_cast<__nv_bfloat16*>(args.out)[(size_t)token * args.ldo + feature] = __float2bfloat16_rn(acc[j]);
          } else if (EPI == EPI_F32) {
            reinterpret_cast<float*>(args.out)[(size_t)token * args.ldo + feature] = acc[j];
          } else {
            reinterpret_cast<float*>(args.out)[((size_t)blockIdx.z * args.tokens + token) * args.ldo + feature] = acc[j];
          }
        }
      }
    }
    tc_fence_before();
  }
  if (EPI == EPI_ADD) {
    // The blocks of the cluster hold the K splits of one tile.  Block r adds slice r of the tile:
    // the sum over all blocks, in block order, goes onto the float tensor (each element once).
    const float* tile = reinterpret_cast<const float*>(smem);
    srb_cluster_sync();
    if (warp >= 2) {
      const int blocks = gridDim.z;                          // = cluster size
      const int live_tokens = min(BLOCK_T, args.tokens - token0);
      const int total = max(live_tokens, 0) * GEMM_BLOCK_F;
      const int per_block = (total + blocks - 1) / blocks;
      const int begin = min(total, (int)srb_cluster_rank() * per_block), end = min(total, begin + per_block);
      for (int i = begin + (int)threadIdx.x - 64; i < end; i += GEMM_THREADS - 64) {
        const int token = i / GEMM_BLOCK_F, f = i % GEMM_BLOCK_F;
        if (feature0 + f >= args.features) continue;
        float sum = 0.f;
        for (int b = 0; b < blocks; ++b) sum += srb_load_peer_shared(tile + i, b);
        float* dst = reinterpret_cast<float*>(args.out) + (size_t)(token0 + token) * args.ldo + feature0 + f;
        *dst += sum;
      }
    }
    srb_cluster_sync();                                      // nobody leaves while its tile may still be read
  }
  __syncthreads();
  srb_mark(SRB_MARK_PRODUCT, 2);
  if (threadIdx.x == 0 && abort_flag) atomicOr(args.error_word, SRB_FLAG_WAIT_TIMEOUT);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLUMNS);
  }
}

// ------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &entry, 12000, cudaEnableDefault, &result) ==
            cudaSuccess && result == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(entry);
  });
  return fn;
}

// A [rows, k] bfloat16 row-major matrix cut into boxes of [box_rows, 64] with 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, long long rows, long long k, long long pitch, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) SRB_FAIL("gemm_bf16: the driver does not offer cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)pitch * 2};
  const cuuint32_t box[2] = {GEMM_BLOCK_K, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult status = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                             elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (status != CUDA_SUCCESS) SRB_FAIL("gemm_bf16: cuTensorMapEncodeTiled failed with %d", (int)status);
  return SRB_OK;
}

template <int BLOCK_T, int EPI>
static int launch_gemm(const CUtensorMap& map_w, const CUtensorMap& map_x, const GemmArgs& args, int splits,
                       cudaStream_t s) {
  constexpr int STAGE_BYTES = GEMM_BLOCK_F * GEMM_BLOCK_K * 2 + BLOCK_T * GEMM_BLOCK_K * 2;
  // Few tokens (decode): about 100 KB of stages, so that two blocks share an SM and one block's
  // set-up and epilogue hide behind the other's stream of weights.  Many tokens: one block per SM.
  constexpr int BUDGET = BLOCK_T <= 64 ? 108 * 1024 : 200 * 1024;
  constexpr int STAGES = BUDGET / STAGE_BYTES >= 8 ? 8 : BUDGET / STAGE_BYTES;
  static_assert(STAGES >= 3, "a pipeline needs at least three stages");
  constexpr int FEATURES_PER_BLOCK = EPI == EPI_SILU ? GEMM_BLOCK_F / 2 : GEMM_BLOCK_F;
  const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;
  auto kernel = gemm_bf16_kernel<BLOCK_T, EPI, STAGES>;
  SRB_CUDA_CALL(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((args.tokens + BLOCK_T - 1) / BLOCK_T, (args.features + FEATURES_PER_BLOCK - 1) / FEATURES_PER_BLOCK, splits);
  if (grid.y > 65535) SRB_FAIL("gemm_bf16: %d features exceed one launch", args.features);
  SRB_CUDA_CALL(srb_launch_clustered(kernel, grid, dim3(GEMM_THREADS), smem, s,
                                     dim3(1, 1, EPI == EPI_ADD ? splits : 1), map_w, map_x, args));
  return SRB_OK;
}

template <int EPI>
static int dispatch_tokens(int block_t, const CUtensorMap& map_w, const CUtensorMap& map_x, const GemmArgs& args,
                           int splits, cudaStream_t s) {
  switch (block_t) {
    case 16: return launch_gemm<16, EPI>(map_w, map_x, args, splits, s);
    case 32: return launch_gemm<32, EPI>(map_w, map_x, args, splits, s);
    case 64: return launch_gemm<64, EPI>(map_w, map_x, args, splits, s);
    case 128: return launch_gemm<128, EPI>(map_w, map_x, args, splits, s);
    default: return launch_gemm<256, EPI>(map_w, map_x, args, splits, s);
  }
}

// Tokens per block for a step of `tokens` rows: the smallest tile that holds them, 256 at most.
extern "C" int srb_gemm_bf16_block_tokens(int tokens, int mode) {
  const int cap = 256;
  int block = 16;
  while (block < tokens && block < cap) block *= 2;
  return block;
}

// x [tokens, k] (row pitch ldx), w [rows_of_w, k] (row pitch ldw), both bfloat16, k a multiple of 8.
// mode 0: out bf16 [tokens, ldo] = x w^T over `features` rows of w.
// mode 1: the same as float.
// mode 2: w stacks gate rows [0, features) and up rows [up_row_offset, up_row_offset + features);
//         out bf16 [tokens, ldo] = act(x gate^T) * (x up^T), act being SRB_ACT_* `activation` (activations.cuh).
// mode 3: `splits` partial sums over K as float [splits, tokens, ldo]; the caller adds them in order.
// mode 4: out float [tokens, ldo] += x w^T, K cut into `splits` (at most 8) blocks that form a cluster and add
//         their sums in block order.
extern "C" int srb_gemm_bf16(const void* x, const void* w, void* out, int tokens, int features, int k, int ldx,
                             int ldw, int ldo, int rows_of_w, int up_row_offset, int mode, int splits,
                             int activation, int* error_word, void* stream) {
  if (tokens <= 0 || features <= 0) return SRB_OK;
  if (k <= 0 || k % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0)
    SRB_FAIL("gemm_bf16: inner size %d and the row pitches %d, %d must be positive multiples of 8 (16-byte rows "
             "for TMA)", k, ldx, ldw);
  if (((uintptr_t)x | (uintptr_t)w) & 15) SRB_FAIL("gemm_bf16: operands must be 16-byte aligned");
  if (mode < 0 || mode > 4) SRB_FAIL("gemm_bf16: unknown mode %d", mode);
  if (mode == EPI_SILU && (activation < 0 || activation >= SRB_ACT_COUNT))
    SRB_FAIL("gemm_bf16: unknown activation %d", activation);
  if (ldo < features) SRB_FAIL("gemm_bf16: output pitch %d is smaller than %d features", ldo, features);
  if (mode == EPI_SILU && up_row_offset + features > rows_of_w)
    SRB_FAIL("gemm_bf16: the up rows %d..%d lie outside the %d rows of w", up_row_offset, up_row_offset + features,
             rows_of_w);
  if (mode != EPI_SILU && features > rows_of_w) SRB_FAIL("gemm_bf16: %d features exceed %d rows of w", features, rows_of_w);
  const int total_k_blocks = (k + GEMM_BLOCK_K - 1) / GEMM_BLOCK_K;
  if (mode != EPI_PARTIAL && mode != EPI_ADD) splits = 1;
  if (mode == EPI_ADD && splits > 8) SRB_FAIL("gemm_bf16: %d splits exceed a cluster of 8 blocks", splits);
  if (splits < 1 || splits > total_k_blocks) SRB_FAIL("gemm_bf16: %d splits do not fit %d blocks of K", splits, total_k_blocks);
  const int block_t = srb_gemm_bf16_block_tokens(tokens, mode);

  CUtensorMap map_w, map_x;
  // rows beyond `features` (or beyond the matrix) are never stored; the map covers all rows of w
  if (make_map(&map_w, w, rows_of_w, k, ldw, mode == EPI_SILU ? GEMM_BLOCK_F / 2 : GEMM_BLOCK_F) != SRB_OK)
    return SRB_ERR_INVALID;
  if (make_map(&map_x, x, tokens, k, ldx, block_t) != SRB_OK) return SRB_ERR_INVALID;

  GemmArgs args;
  args.out = out; args.tokens = tokens; args.features = features; args.k = k; args.ldo = ldo;
  args.up_row_offset = up_row_offset; args.activation = activation; args.error_word = error_word;
  args.k_blocks_per_split = (total_k_blocks + splits - 1) / splits;
  const int used_splits = (total_k_blocks + args.k_blocks_per_split - 1) / args.k_blocks_per_split;
  if (used_splits != splits) SRB_FAIL("gemm_bf16: %d splits leave one without work for %d blocks of K", splits, total_k_blocks);
  cudaStream_t s = (cudaStream_t)stream;
  switch (mode) {
    case EPI_BF16: return dispatch_tokens<EPI_BF16>(block_t, map_w, map_x, args, splits, s);
    case EPI_F32: return dispatch_tokens<EPI_F32>(block_t, map_w, map_x, args, splits, s);
    case EPI_SILU: return dispatch_tokens<EPI_SILU>(block_t, map_w, map_x, args, 1, s);
    case EPI_ADD: return dispatch_tokens<EPI_ADD>(block_t, map_w, map_x, args, splits, s);
    default: return dispatch_tokens<EPI_PARTIAL>(block_t, map_w, map_x, args, splits, s);
  }
}
