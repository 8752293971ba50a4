// Fused per-head RMSNorm of q and k, rotary position encoding, and the write of k and v
// into the layer's pages.  One warp handles one head vector of one row.
//
// Order of operations as in the reference's attention half
// (crates/sglang-srt/src/cpu_reference.rs:485-525): project, norm each q and k head with
// the shared [head_dim] weight, rotate q and k, then store k and v at the row's slot.
// Rotation (crates/sglang-kernel/src/rotary.rs:216-236): half-split pairs (i, i + rot/2) or
// interleaved pairs (2i, 2i + 1); angle = float(pos) * inv_freq[i] in 32-bit; the table
// inv_freq[i] = theta^(-2i/rot) is computed in 64-bit on the host (rotary.rs:76-80).  Instead of
// the table the caller may give the angle of every (row, pair) itself (`angles` [rows, rot/2]):
// that covers every encoding of the rotary family without a change here.
//
// Page pool layout: [page, kv_head, slot_in_page, head_dim].
#include "common.cuh"

SRB_DEFINE_LAST_ERROR()
SRB_DEFINE_PDL_SWITCH()

#define ROPE_WARPS 4
#define ROPE_MAX_ROUNDS 3             // many rows: a block handles 12 head vectors of one row with one table of angles

// The projection may arrive as `num_parts` float partial sums (a product cut along K),
// `part_stride` elements apart, instead of one tensor of type T; they are added in part order.
template <typename T>
__global__ void qk_norm_rope_kv_kernel(const T* __restrict__ qkv, const float* __restrict__ qkv_parts, int num_parts,
                                       size_t part_stride, int qkv_stride, T* __restrict__ q_out,
                                       T* __restrict__ k_pool, T* __restrict__ v_pool,
                                       const int* __restrict__ positions, const int* __restrict__ slots,
                                       const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                                       float eps, const float* __restrict__ inv_freq,
                                       const float* __restrict__ angles, int rotary_dim,
                                       int interleaved, int n_q, int n_kv, int head_dim, int page_size,
                                       int num_pages, int heads_to_do, int vector_ok, int rounds, int* error_word) {
  extern __shared__ __align__(16) float staged_all[];  // ROPE_WARPS * head_dim floats
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x;
  float* staged = staged_all + warp * head_dim;
  // cos and sin of the row's angles, once per block: every q and k head of the row turns by the same angles
  float* cos_table = staged_all + ROPE_WARPS * head_dim;
  float* sin_table = cos_table + (rotary_dim >> 1);
  const bool rotate = inv_freq || angles;
  if (angles) {            // the angles of every row and pair are given: any encoding of the rotary family
    for (int i = threadIdx.x; i < (rotary_dim >> 1); i += blockDim.x)
      sincosf(angles[(size_t)row * (rotary_dim >> 1) + i], &sin_table[i], &cos_table[i]);
  } else if (inv_freq) {
    const float pos = (float)positions[row];
    for (int i = threadIdx.x; i < (rotary_dim >> 1); i += blockDim.x) sincosf(pos * inv_freq[i], &sin_table[i], &cos_table[i]);
  }
  __syncthreads();
#pragma unroll 1
  for (int round = 0; round < rounds; ++round) {
  const int head = (blockIdx.y * rounds + round) * ROPE_WARPS + warp;     // q heads, then k heads, then v heads
  if (head >= heads_to_do) break;
  const size_t src_offset = (size_t)row * qkv_stride + (size_t)head * head_dim;

  const bool is_q = head < n_q;
  const bool is_k = !is_q && head < n_q + n_kv;
  const float* norm_weight = is_q ? q_norm : (is_k ? k_norm : nullptr);

  float partial = 0.f;
  if (num_parts > 0 && vector_ok) {
    // four consecutive values per lane and part: all loads of a lane are in flight together
    for (int e = lane * 4; e < head_dim; e += 128) {
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int part = 0; part < num_parts; ++part) {
        const float4 d = *reinterpret_cast<const float4*>(qkv_parts + part * part_stride + src_offset + e);
        x.x += d.x; x.y += d.y; x.z += d.z; x.w += d.w;
      }
      *reinterpret_cast<float4*>(staged + e) = x;
      partial += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
  } else if (vector_ok) {
    for (int e = lane * 4; e < head_dim; e += 128) {
      float4 x;
      if (sizeof(T) == 2) {
        const uint2 raw = *reinterpret_cast<const uint2*>(qkv + src_offset + e);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        x = make_float4(a.x, a.y, b.x, b.y);
      } else {
        x = *reinterpret_cast<const float4*>(qkv + src_offset + e);
      }
      *reinterpret_cast<float4*>(staged + e) = x;
      partial += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
  } else {
    for (int e = lane; e < head_dim; e += 32) {
      float x = 0.f;
      if (num_parts == 0) {
        x = srb_to_float(qkv[src_offset + e]);
      } else {
        for (int part = 0; part < num_parts; ++part) x += qkv_parts[part * part_stride + src_offset + e];
      }
      staged[e] = x;
      partial += x * x;
    }
  }
  if (norm_weight) {
    const float total = srb_warp_sum(partial);
    const float inv = 1.0f / sqrtf(total / (float)head_dim + eps);
    for (int e = lane; e < head_dim; e += 32) staged[e] = staged[e] * inv * norm_weight[e];
  }
  __syncwarp();
  if ((is_q || is_k) && rotate) {
    const int half = rotary_dim >> 1;
    for (int i = lane; i < half; i += 32) {
      const int ia = interleaved ? 2 * i : i;
      const int ib = interleaved ? 2 * i + 1 : i + half;
      const float sn = sin_table[i], cs = cos_table[i];
      const float a = staged[ia], b = staged[ib];
      staged[ia] = a * cs - b * sn;      // each element belongs to exactly one pair
      staged[ib] = b * cs + a * sn;
    }
  }
  __syncwarp();

  T* dst;
  if (is_q) {
    dst = q_out + ((size_t)row * n_q + head) * head_dim;
  } else {
    const int slot = slots[row];
    if (slot < 0 || slot >= num_pages * page_size) {
      if (lane == 0) atomicOr(error_word, SRB_FLAG_BAD_SLOT);
      __syncwarp();
      continue;
    }
    const int kv_head = is_k ? head - n_q : head - n_q - n_kv;
    const size_t offset =
        (((size_t)(slot / page_size) * n_kv + kv_head) * page_size + (slot % page_size)) * head_dim;
    dst = (is_k ? k_pool : v_pool) + offset;
  }
  if (vector_ok) {
    for (int e = lane * 4; e < head_dim; e += 128) {
      const float4 x = *reinterpret_cast<const float4*>(staged + e);
      if (sizeof(T) == 2) {
        uint2 raw;
        *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(x.x, x.y);
        *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(x.z, x.w);
        *reinterpret_cast<uint2*>(dst + e) = raw;
      } else {
        *reinterpret_cast<float4*>(dst + e) = x;
      }
    }
  } else {
    for (int e = lane; e < head_dim; e += 32) dst[e] = srb_from_float<T>(staged[e]);
  }
  __syncwarp();                            // the staging row is reused by the warp's next head
  }
}

// `slots` may be null: then only the q heads are processed (a layer that reads another
// layer's cache writes nothing).
extern "C" int srb_qk_norm_rope_kv(const void* qkv, const float* qkv_parts, int num_parts, long long part_stride,
                                   int qkv_stride, void* q_out, void* k_pool, void* v_pool,
                                   const int* positions, const int* slots, const float* q_norm,
                                   const float* k_norm, float eps, const float* inv_freq, const float* angles,
                                   int rotary_dim,
                                   int interleaved, int rows, int n_q, int n_kv, int head_dim, int page_size,
                                   int num_pages, int* error_word, int dtype, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (n_q <= 0 || n_kv <= 0 || head_dim <= 0 || page_size <= 0)
    SRB_FAIL("qk_norm_rope_kv: head counts, head_dim and page size must be positive");
  if ((inv_freq || angles) && (rotary_dim <= 0 || rotary_dim > head_dim || (rotary_dim & 1)))
    SRB_FAIL("qk_norm_rope_kv: rotary width %d must be even, positive and at most head_dim %d", rotary_dim,
             head_dim);
  if (head_dim > 2048) SRB_FAIL("qk_norm_rope_kv: head_dim %d exceeds 2048", head_dim);
  if (num_parts < 0 || (num_parts > 0 && !qkv_parts) || (num_parts == 0 && !qkv))
    SRB_FAIL("qk_norm_rope_kv: the projection is missing");
  const int heads = slots ? n_q + 2 * n_kv : n_q;
  // four values per lane and access need 16-byte rows
  const int vector_ok = head_dim % 4 == 0 && qkv_stride % 4 == 0 && part_stride % 4 == 0 &&
                        (((uintptr_t)qkv_parts | (uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pool |
                          (uintptr_t)v_pool) & 15) == 0;
  // few rows (decode): one head per warp, so that the row is finished soonest; many rows: fewer tables of angles
  const int rounds = rows >= 64 ? ROPE_MAX_ROUNDS : 1;
  const int heads_per_block = ROPE_WARPS * rounds;
  dim3 grid(rows, (heads + heads_per_block - 1) / heads_per_block);
  const size_t smem = ((size_t)ROPE_WARPS * head_dim + ((inv_freq || angles) ? rotary_dim : 0)) * sizeof(float);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32)
    SRB_CUDA_CALL(srb_launch(qk_norm_rope_kv_kernel<float>, grid, dim3(ROPE_WARPS * 32), smem, s, (const float*)qkv,
                             qkv_parts, num_parts, (size_t)part_stride, qkv_stride, (float*)q_out, (float*)k_pool,
                             (float*)v_pool, positions, slots, q_norm, k_norm, eps, inv_freq, angles, rotary_dim,
                             interleaved, n_q, n_kv, head_dim, page_size, num_pages, heads, vector_ok, rounds, error_word));
  else if (dtype == SRB_DTYPE_BF16)
    SRB_CUDA_CALL(srb_launch(qk_norm_rope_kv_kernel<__nv_bfloat16>, grid, dim3(ROPE_WARPS * 32), smem, s,
                             (const __nv_bfloat16*)qkv, qkv_parts, num_parts, (size_t)part_stride, qkv_stride,
                             (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, positions, slots,
                             q_norm, k_norm, eps, inv_freq, angles, rotary_dim, interleaved, n_q, n_kv, head_dim,
                             page_size, num_pages, heads, vector_ok, rounds, error_word));
  else
    SRB_FAIL("qk_norm_rope_kv: unknown dtype %d", dtype);
  SRB_LAUNCH_CHECK("qk_norm_rope_kv");
  return SRB_OK;
}
