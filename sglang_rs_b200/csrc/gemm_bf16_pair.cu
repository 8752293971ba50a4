// Y = X W^T in bfloat16 for many tokens (prompt portions): tiles of 256 features x 256 tokens computed
// by pairs of CTAs on neighbouring SMs with tcgen05.mma.cta_group::2, in a persistent loop.
//
// The pair is a thread-block cluster of two.  CTA r of the pair brings 128 rows of W (its half of the
// M side) and 128 tokens of X (its half of the N side) into its own shared memory by TMA; one thread of
// the even CTA issues the products for both, and each CTA's tensor memory receives the 128 x 256
// accumulator of its own W rows.  Per product step a CTA reads 8 KB of operands from shared memory and
// the pair asks L2 for 1 byte per 131 FLOP (a single CTA with a 128 x 256 tile: 12 KB and 1 byte per
// 85 FLOP).  The kernel is persistent: 74 pairs walk the tiles, the accumulator has two buffers in
// tensor memory, and the epilogue of a tile (tensor memory -> registers -> shared memory -> 16-byte
// stores, 128 tokens at a time) runs while the products of the next tile are issued.  Six stages of
// 32 KB keep 160 KB of operands in flight per CTA.
//
// Warps of each CTA: 0 copies (TMA), 1 issues products (even CTA only) and owns the tensor memory,
// 2-5 epilogue.  Barriers: full[s] lives in the even CTA and counts the bytes of both CTAs' copies;
// empty[s] and acc_full[b] live in both and are signalled by tcgen05.commit with a multicast to the
// pair; acc_empty[b] lives in the even CTA and is signalled by the epilogue warps of both.
// Every wait is bounded; a wait that runs out flags SRB_FLAG_WAIT_TIMEOUT and every role leaves its
// loop.  No TMA load uses multicast.
//
// Modes: bfloat16 store; SiLU(gate) * up where a CTA's 128 weight rows are 64 gate rows over the 64 up
// rows of the same features (as in gemm_bf16.cu).
#include "common.cuh"
#include "tcgen05_helpers.cuh"
#include "activations.cuh"
#include <algorithm>
#include <mutex>

SRB_DEFINE_LAST_ERROR()

#define PAIR_F 128            // weight rows per CTA (256 per pair)
#define PAIR_T 256            // tokens per tile (128 copied by each CTA)
#define PAIR_K 64
#define PAIR_STAGES 6
#define PAIR_OUT_T 128         // tokens of a tile that are staged for the stores at a time
#define PAIR_THREADS 192
#define PAIR_EPI_BF16 0
#define PAIR_EPI_SILU 2

struct PairArgs {
  __nv_bfloat16* out;
  int tokens, features, k, ldo, up_row_offset;
  int activation;            // which SRB_ACT_* the gated mode applies to the gate half
  int tiles_t, tiles_f, num_tiles;
  int* error_word;
};

// ---- the cta_group::2 forms of the instructions
__device__ __forceinline__ void tmem_alloc_pair(unsigned holder, unsigned columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(holder), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(unsigned address, unsigned columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(unsigned tmem_d, unsigned long long a_desc, unsigned long long b_desc,
                                               unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs of the pair once the products issued so far are done
__device__ __forceinline__ void umma_commit_pair(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((unsigned short)3) : "memory");
}
// a tile copy whose bytes are counted by the barrier of the even CTA of the pair (bit 24 of a shared
// address names the odd CTA)
__device__ __forceinline__ void tma_load_2d_pair(unsigned dst, const CUtensorMap* map, unsigned bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar & 0xFEFFFFFFu), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(unsigned bar, unsigned rank) {
  asm volatile("{\n.reg .b32 remote;\nmapa.shared::cluster.u32 remote, %0, %1;\n"
               "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [remote];\n}\n" ::"r"(bar), "r"(rank) : "memory");
}

__host__ __device__ constexpr unsigned pair_idesc() {
  // D float, A and B bfloat16, both K-major, M = 256 (the pair), N = 256
  return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(PAIR_T >> 3) << 17) | ((unsigned)(256 >> 4) << 24);
}

template <int EPI>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      PairArgs args) {
  constexpr int A_BYTES = PAIR_F * PAIR_K * 2;               // 16 KB: this CTA's rows of W
  constexpr int B_BYTES = (PAIR_T / 2) * PAIR_K * 2;         // 16 KB: this CTA's tokens of X
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int FEATURES_PER_CTA = EPI == PAIR_EPI_SILU ? PAIR_F / 2 : PAIR_F;
  extern __shared__ unsigned char smem_unaligned[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_unaligned + 1023) & ~(uintptr_t)1023);
  unsigned char* out_smem = smem + PAIR_STAGES * STAGE_BYTES;
  __shared__ __align__(8) unsigned long long full_bar[PAIR_STAGES], empty_bar[PAIR_STAGES], acc_full[2], acc_empty[2];
  __shared__ unsigned tmem_holder;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = srb_cluster_rank();                  // 0: the CTA that issues the products
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int total_kb = (args.k + PAIR_K - 1) / PAIR_K;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < PAIR_STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&acc_full[b]), 1);
      mbar_init(smem_u32(&acc_empty[b]), 8);                 // one lane of each epilogue warp of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(smem_u32(&tmem_holder), 512);
  tc_fence_before();
  srb_cluster_sync();                                        // both CTAs' barriers exist before anyone signals them
  tc_fence_after();
  const unsigned tmem_base = tmem_holder;

  if (warp == 0) {
    // copies: both CTAs, each its own halves, into its own stages; the bytes count on the even CTA's barrier
    int issued = 0;
    long long round = 0;
    bool ok = true;
    for (int tile = pair; tile < args.num_tiles && ok; tile += num_pairs) {
      const int ft = tile / args.tiles_t, tt = tile % args.tiles_t;
      const int feature0 = ft * 2 * FEATURES_PER_CTA + (int)rank * FEATURES_PER_CTA;
      const int token0 = tt * PAIR_T + (int)rank * (PAIR_T / 2);
      for (int kb = 0; kb < total_kb && ok; ++kb, ++round) {
        const int s = (int)(round % PAIR_STAGES);
        const unsigned phase = (unsigned)(round / PAIR_STAGES) & 1u;
        ok = mbar_wait_warp(smem_u32(&empty_bar[s]), phase ^ 1u, &abort_flag);
        if (!ok) break;
        const unsigned bar = smem_u32(&full_bar[s]);
        const unsigned stage = smem_u32(smem) + s * STAGE_BYTES;
        const int kx = kb * PAIR_K;
        if (elect_one()) {
          if (rank == 0) mbar_expect_tx(bar, 2 * STAGE_BYTES);
          if (EPI == PAIR_EPI_SILU) {
            tma_load_2d_pair(stage, &map_w, bar, kx, feature0);
            tma_load_2d_pair(stage + A_BYTES / 2, &map_w, bar, kx, args.up_row_offset + feature0);
          } else {
            tma_load_2d_pair(stage, &map_w, bar, kx, feature0);
          }
          tma_load_2d_pair(stage + A_BYTES, &map_x, bar, kx, token0);
        }
        ++issued;
      }
    }
    // copies that were still in flight when a wait ran out write into this CTA's memory: give them time to land
    if (abort_flag && issued > 0) {
      const long long start = clock64();
      while (clock64() - start < 4000000ll) {}
    }
  } else if (warp == 1) {
    if (rank == 0) {
      // products of the pair, issued by one elected lane of the even CTA
      constexpr unsigned idesc = pair_idesc();
      const unsigned long long a_desc0 = smem_descriptor(smem_u32(smem));
      const unsigned long long b_desc0 = smem_descriptor(smem_u32(smem) + A_BYTES);
      long long round = 0;
      int local_tile = 0;
      bool ok = true;
      for (int tile = pair; tile < args.num_tiles && ok; tile += num_pairs, ++local_tile) {
        const int b = local_tile & 1;
        // the epilogue warps of both CTAs have read this accumulator buffer (two tiles ago)
        ok = mbar_wait_warp(smem_u32(&acc_empty[b]), (((unsigned)(local_tile >> 1)) & 1u) ^ 1u, &abort_flag);
        if (!ok) break;
        tc_fence_after();
        const unsigned acc = tmem_base + b * PAIR_T;
        for (int kb = 0; kb < total_kb && ok; ++kb, ++round) {
          const int s = (int)(round % PAIR_STAGES);
          const unsigned phase = (unsigned)(round / PAIR_STAGES) & 1u;
          ok = mbar_wait_warp(smem_u32(&full_bar[s]), phase, &abort_flag);
          if (!ok) break;
          tc_fence_after();
          const unsigned long long stage_step = (unsigned long long)((s * STAGE_BYTES) >> 4);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < PAIR_K / 16; ++k) {
              const unsigned long long step = stage_step + (unsigned long long)((k * 16 * 2) >> 4);
              umma_bf16_pair(acc, a_desc0 + step, b_desc0 + step, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit_pair(smem_u32(&empty_bar[s]));       // frees the stage in both CTAs
            if (kb == total_kb - 1) umma_commit_pair(smem_u32(&acc_full[b]));
          }
          __syncwarp();
        }
      }
    }
  } else {
    // epilogue: warp w reads TMEM lanes 32 * (w % 4) .. + 32 of its own CTA
    const int quarter = warp & 3;
    const int row_in_cta = quarter * 32 + lane;              // the W row (TMEM lane) this thread holds
    const unsigned lane_address = tmem_base + ((unsigned)(quarter * 32) << 16);
    __nv_bfloat16* staged = reinterpret_cast<__nv_bfloat16*>(out_smem);   // [token][FEATURES_PER_CTA]
    int local_tile = 0;
    bool ok = true;
    for (int tile = pair; tile < args.num_tiles && ok; tile += num_pairs, ++local_tile) {
      const int b = local_tile & 1;
      const int ft = tile / args.tiles_t, tt = tile % args.tiles_t;
      const int feature0 = ft * 2 * FEATURES_PER_CTA + (int)rank * FEATURES_PER_CTA;
      const int token_base = tt * PAIR_T;
      ok = mbar_wait(smem_u32(&acc_full[b]), ((unsigned)(local_tile >> 1)) & 1u, &abort_flag);
      if (!ok) break;
      tc_fence_after();
      // 128 tokens at a time: accumulator -> registers -> staging tile [token][feature] -> 16-byte stores
#pragma unroll 1
      for (int half = 0; half < PAIR_T / PAIR_OUT_T; ++half) {
        if (EPI == PAIR_EPI_SILU) {
          // lanes 0..63 hold gate, lanes 64..127 up of the same 64 features: up passes through shared
          // memory, 32 tokens at a time, in two buffers that take turns (one barrier per round)
          float* exchange = reinterpret_cast<float*>(out_smem + PAIR_OUT_T * FEATURES_PER_CTA * 2);   // [2][64][32] floats
#pragma unroll 1
          for (int c = 0; c < PAIR_OUT_T; c += 32) {
            float acc[32];
            tmem_load_32(lane_address + b * PAIR_T + half * PAIR_OUT_T + c, acc);
            float* buffer = exchange + ((c >> 5) & 1) * 64 * 32;
            if (quarter >= 2) {
#pragma unroll
              for (int j = 0; j < 32; ++j) buffer[j * 64 + (quarter & 1) * 32 + lane] = acc[j];
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (quarter < 2) {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float g = acc[j], u = buffer[j * 64 + (quarter & 1) * 32 + lane];
                staged[(c + j) * FEATURES_PER_CTA + row_in_cta] = __float2bfloat16_rn(srb_gated<false>(args.activation, g, u));
              }
            }
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < PAIR_OUT_T; c += 16) {
            float acc[16];
            tmem_load_16(lane_address + b * PAIR_T + half * PAIR_OUT_T + c, acc);
#pragma unroll
            for (int j = 0; j < 16; ++j) staged[(c + j) * FEATURES_PER_CTA + row_in_cta] = __float2bfloat16_rn(acc[j]);
          }
        }
        if (half == PAIR_T / PAIR_OUT_T - 1) {
          // the accumulator buffer is free for the tile after next
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_remote(smem_u32(&acc_empty[b]), 0);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");        // the staged rows are complete
        // 16-byte stores: a token's FEATURES_PER_CTA features are consecutive in the output
        constexpr int CHUNKS = FEATURES_PER_CTA / 8;
        for (int i = threadIdx.x - 64; i < PAIR_OUT_T * CHUNKS; i += 128) {
          const int token = i / CHUNKS, chunk = i % CHUNKS;
          const int feature = feature0 + chunk * 8;
          const int out_token = token_base + half * PAIR_OUT_T + token;
          if (out_token >= args.tokens || feature >= args.features) continue;
          const uint4 value = *reinterpret_cast<const uint4*>(staged + token * FEATURES_PER_CTA + chunk * 8);
          __nv_bfloat16* dst = args.out + (size_t)out_token * args.ldo + feature;
          if (feature + 8 <= args.features) {
            *reinterpret_cast<uint4*>(dst) = value;
          } else {
            const __nv_bfloat16* v = reinterpret_cast<const __nv_bfloat16*>(&value);
            for (int e = 0; feature + e < args.features; ++e) dst[e] = v[e];
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");        // the staging tile may be written again
      }
    }
    tc_fence_before();
  }
  srb_cluster_sync();                                        // nobody leaves while the other CTA may still signal or read
  if (threadIdx.x == 0 && abort_flag) atomicOr(args.error_word, SRB_FLAG_WAIT_TIMEOUT);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
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

static int make_map(CUtensorMap* map, const void* base, long long rows, long long k, long long pitch, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) SRB_FAIL("gemm_bf16_pair: the driver does not offer cuTensorMapEncodeTiled");
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)pitch * 2};
  const cuuint32_t box[2] = {PAIR_K, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult status = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                             elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (status != CUDA_SUCCESS) SRB_FAIL("gemm_bf16_pair: cuTensorMapEncodeTiled failed with %d", (int)status);
  return SRB_OK;
}

// x [tokens, k] (row pitch ldx), w [rows_of_w, k] (row pitch ldw), out [tokens, ldo], all bfloat16; k and the
// pitches multiples of 8.  mode 0: out = x w^T over `features` rows of w.  mode 2: w stacks gate rows
// [0, features) and up rows [up_row_offset, up_row_offset + features); out = act(x gate^T) * (x up^T), act being SRB_ACT_* `activation` (activations.cuh).
extern "C" int srb_gemm_bf16_pair(const void* x, const void* w, void* out, int tokens, int features, int k, int ldx,
                                  int ldw, int ldo, int rows_of_w, int up_row_offset, int mode, int activation,
                                  int* error_word, void* stream) {
  if (tokens <= 0 || features <= 0) return SRB_OK;
  if (k <= 0 || k % 8 != 0 || ldx % 8 != 0 || ldw % 8 != 0 || ldo % 8 != 0)
    SRB_FAIL("gemm_bf16_pair: inner size %d and the row pitches %d, %d, %d must be positive multiples of 8", k, ldx, ldw,
             ldo);
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) SRB_FAIL("gemm_bf16_pair: operands must be 16-byte aligned");
  if (mode != PAIR_EPI_BF16 && mode != PAIR_EPI_SILU) SRB_FAIL("gemm_bf16_pair: unknown mode %d", mode);
  if (mode == PAIR_EPI_SILU && (activation < 0 || activation >= SRB_ACT_COUNT))
    SRB_FAIL("gemm_bf16_pair: unknown activation %d", activation);
  if (mode == PAIR_EPI_SILU && up_row_offset + features > rows_of_w)
    SRB_FAIL("gemm_bf16_pair: the up rows lie outside the %d rows of w", rows_of_w);
  if (mode == PAIR_EPI_BF16 && features > rows_of_w) SRB_FAIL("gemm_bf16_pair: %d features exceed %d rows of w", features, rows_of_w);
  CUtensorMap map_w, map_x;
  if (make_map(&map_w, w, rows_of_w, k, ldw, mode == PAIR_EPI_SILU ? PAIR_F / 2 : PAIR_F) != SRB_OK) return SRB_ERR_INVALID;
  if (make_map(&map_x, x, tokens, k, ldx, PAIR_T / 2) != SRB_OK) return SRB_ERR_INVALID;
  const int features_per_pair = mode == PAIR_EPI_SILU ? PAIR_F : 2 * PAIR_F;
  PairArgs args;
  args.out = (__nv_bfloat16*)out; args.tokens = tokens; args.features = features; args.k = k; args.ldo = ldo;
  args.up_row_offset = up_row_offset; args.activation = activation; args.error_word = error_word;
  args.tiles_t = (tokens + PAIR_T - 1) / PAIR_T;
  args.tiles_f = (features + features_per_pair - 1) / features_per_pair;
  args.num_tiles = args.tiles_t * args.tiles_f;
  int device = 0, sms = 0;
  SRB_CUDA_CALL(cudaGetDevice(&device));
  SRB_CUDA_CALL(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  const int pairs = std::max(1, std::min(sms / 2, args.num_tiles));
  // the stages, the staging tile of the stores (and in SiLU mode, inside it, the exchange of the up half), alignment
  const size_t smem = (size_t)PAIR_STAGES * (PAIR_F * PAIR_K * 2 + (PAIR_T / 2) * PAIR_K * 2) + PAIR_OUT_T * PAIR_F * 2 + 1024;
  cudaStream_t s = (cudaStream_t)stream;
  if (mode == PAIR_EPI_SILU) {
    SRB_CUDA_CALL(cudaFuncSetAttribute(gemm_bf16_pair_kernel<PAIR_EPI_SILU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    SRB_CUDA_CALL(srb_launch_clustered(gemm_bf16_pair_kernel<PAIR_EPI_SILU>, dim3(2 * pairs), dim3(PAIR_THREADS), smem, s,
                                       dim3(2, 1, 1), map_w, map_x, args));
  } else {
    SRB_CUDA_CALL(cudaFuncSetAttribute(gemm_bf16_pair_kernel<PAIR_EPI_BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    SRB_CUDA_CALL(srb_launch_clustered(gemm_bf16_pair_kernel<PAIR_EPI_BF16>, dim3(2 * pairs), dim3(PAIR_THREADS), smem, s,
                                       dim3(2, 1, 1), map_w, map_x, args));
  }
  return SRB_OK;
}
