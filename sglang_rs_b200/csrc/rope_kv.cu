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
#include "mma_helpers.cuh"
#include <algorithm>

SRB_DEFINE_LAST_ERROR()
SRB_DEFINE_PDL_SWITCH()

#define ROPE_WARPS 4
#define ROPE_MAX_ROUNDS 3             // many rows: a block handles 12 head vectors of one row with one table of angles


// The arithmetic that both kernels below share, written with explicit roundings so that a value
// does not depend on which kernel computed it.
__device__ __forceinline__ float sum_squares4(float4 x) {
  return __fmaf_rn(x.w, x.w, __fmaf_rn(x.z, x.z, __fmaf_rn(x.y, x.y, __fmul_rn(x.x, x.x))));
}
__device__ __forceinline__ float rotate_first(float a, float b, float cs, float sn) {    // a cos - b sin
  return __fmaf_rn(a, cs, -__fmul_rn(b, sn));
}
__device__ __forceinline__ float rotate_second(float a, float b, float cs, float sn) {   // b cos + a sin
  return __fmaf_rn(b, cs, __fmul_rn(a, sn));
}
__device__ __forceinline__ float normed(float x, float inv, float w) { return __fmul_rn(__fmul_rn(x, inv), w); }

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
  // The table of angles needs only the step's index arrays and constants: it is computed before
  // the wait for the kernel ahead (whose product this kernel reads) and overlaps that kernel's end.
  srb_mark(SRB_MARK_ROPE, 0);
  srb_launch_dependents();
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
  srb_grid_dependency_wait();
  srb_mark(SRB_MARK_ROPE, 1);
  __syncthreads();
#pragma unroll 1
  for (int round = 0; round < rounds; ++round) {
  const int head = (blockIdx.y * rounds + round) * ROPE_WARPS + warp;     // q heads, then k heads, then v heads
  if (head >= heads_to_do) break;
  const size_t src_offset = (size_t)row * qkv_stride + (size_t)head * head_dim;

  const bool is_q = head < n_q;
  const bool is_k = !is_q && head < n_q + n_kv;
  const float* norm_weight = is_q ? q_norm : (is_k ? k_norm : nullptr);
  // the norm's weight (heads of up to 128 values) and the row's slot are asked for together with the head's
  // values, not after the sum of squares and after the rotation: one trip to L2 instead of three
  const bool weight_early = norm_weight && head_dim <= 128;
  float early[4] = {0.f, 0.f, 0.f, 0.f};
  if (weight_early) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (lane + 32 * j < head_dim) early[j] = norm_weight[lane + 32 * j];
  }
  const int slot = is_q ? 0 : slots[row];

  float partial = 0.f;
  if (num_parts > 0 && vector_ok) {
    // four consecutive values per lane and part: all loads of a lane are in flight together
    for (int e = lane * 4; e < head_dim; e += 128) {
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int first = 0; first < num_parts; first += 8) {
        float4 d[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (first + j < num_parts) d[j] = *reinterpret_cast<const float4*>(qkv_parts + (first + j) * part_stride + src_offset + e);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (first + j < num_parts) {
            x.x += d[j].x; x.y += d[j].y; x.z += d[j].z; x.w += d[j].w;
          }
        }
      }
      *reinterpret_cast<float4*>(staged + e) = x;
      partial += sum_squares4(x);
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
      partial += sum_squares4(x);
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
    const float inv = __frsqrt_rn(total / (float)head_dim + eps);
    if (weight_early) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (lane + 32 * j < head_dim) staged[lane + 32 * j] = normed(staged[lane + 32 * j], inv, early[j]);
    } else {
      for (int e = lane; e < head_dim; e += 32) staged[e] = normed(staged[e], inv, norm_weight[e]);
    }
  }
  __syncwarp();
  if ((is_q || is_k) && rotate) {
    const int half = rotary_dim >> 1;
    for (int i = lane; i < half; i += 32) {
      const int ia = interleaved ? 2 * i : i;
      const int ib = interleaved ? 2 * i + 1 : i + half;
      const float sn = sin_table[i], cs = cos_table[i];
      const float a = staged[ia], b = staged[ib];
      staged[ia] = rotate_first(a, b, cs, sn);      // each element belongs to exactly one pair
      staged[ib] = rotate_second(a, b, cs, sn);
    }
  }
  __syncwarp();

  T* dst;
  if (is_q) {
    dst = q_out + ((size_t)row * n_q + head) * head_dim;
  } else {
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
  srb_mark(SRB_MARK_ROPE, 2);
}


// Many rows (256 and more), head_dim 128, rotation of the whole head in half-split pairs, the
// projection in one tensor.  Blocks of four warps stay on their SM and walk the rows blockIdx.x, blockIdx.x +
// gridDim.x, ...  A row's bytes come into a ring of ROW_STAGES buffers in shared memory by asynchronous 16-byte
// copies (one group of copies per row), two rows ahead of the arithmetic, so that the copies of later rows
// travel under the arithmetic of the current one and no register waits for them.  Eight lanes take a head:
// lane l of the eight holds the elements 8l..8l+7 and 64+8l..64+8l+7, that is both members of its eight
// rotation pairs, so the rotation needs no exchange between lanes and the sum of squares three.  A warp takes
// four heads per pass, the block sixteen.  The angles come from the step's table (copied with the row), or are
// computed when the row's copies are issued.  v heads are copied as they are.  Same arithmetic as the kernel
// above, bit for bit: the sum of squares is added up in the order of that kernel's warp reduction (four
// elements per lane there: this lane's four quadruples stand for its lanes 2l, 2l + 1, 2l + 16 and 2l + 17).
#define ROW_THREADS 128
#define ROW_STAGES 3
#define ROW_BLOCKS_PER_SM 5
struct Head16 { float a[8], b[8]; };             // the first and the second member of eight rotation pairs
template <typename T> struct Raw16;
template <> struct Raw16<__nv_bfloat16> { uint4 a, b; };
template <> struct Raw16<float> { float4 a0, a1, b0, b1; };
__device__ __forceinline__ Raw16<__nv_bfloat16> load_raw16(const __nv_bfloat16* p) {
  Raw16<__nv_bfloat16> r;
  r.a = *reinterpret_cast<const uint4*>(p);
  r.b = *reinterpret_cast<const uint4*>(p + 64);
  return r;
}
__device__ __forceinline__ Raw16<float> load_raw16(const float* p) {
  Raw16<float> r;
  r.a0 = *reinterpret_cast<const float4*>(p);
  r.a1 = *reinterpret_cast<const float4*>(p + 4);
  r.b0 = *reinterpret_cast<const float4*>(p + 64);
  r.b1 = *reinterpret_cast<const float4*>(p + 68);
  return r;
}
__device__ __forceinline__ void widen8(const uint4& raw, float* out) {
  const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(pairs[j]);
    out[2 * j] = f.x;
    out[2 * j + 1] = f.y;
  }
}
__device__ __forceinline__ Head16 widen16(const Raw16<__nv_bfloat16>& r) {
  Head16 h;
  widen8(r.a, h.a);
  widen8(r.b, h.b);
  return h;
}
__device__ __forceinline__ Head16 widen16(const Raw16<float>& r) {
  Head16 h;
  h.a[0] = r.a0.x; h.a[1] = r.a0.y; h.a[2] = r.a0.z; h.a[3] = r.a0.w;
  h.a[4] = r.a1.x; h.a[5] = r.a1.y; h.a[6] = r.a1.z; h.a[7] = r.a1.w;
  h.b[0] = r.b0.x; h.b[1] = r.b0.y; h.b[2] = r.b0.z; h.b[3] = r.b0.w;
  h.b[4] = r.b1.x; h.b[5] = r.b1.y; h.b[6] = r.b1.z; h.b[7] = r.b1.w;
  return h;
}
__device__ __forceinline__ uint4 pack8(const float* v) {
  uint4 raw;
  __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) pairs[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
  return raw;
}
__device__ __forceinline__ void store16(__nv_bfloat16* p, const Head16& h) {
  *reinterpret_cast<uint4*>(p) = pack8(h.a);
  *reinterpret_cast<uint4*>(p + 64) = pack8(h.b);
}
__device__ __forceinline__ void store16(float* p, const Head16& h) {
  *reinterpret_cast<float4*>(p) = make_float4(h.a[0], h.a[1], h.a[2], h.a[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(h.a[4], h.a[5], h.a[6], h.a[7]);
  *reinterpret_cast<float4*>(p + 64) = make_float4(h.b[0], h.b[1], h.b[2], h.b[3]);
  *reinterpret_cast<float4*>(p + 68) = make_float4(h.b[4], h.b[5], h.b[6], h.b[7]);
}
__device__ __forceinline__ void store_raw16(__nv_bfloat16* p, const Raw16<__nv_bfloat16>& r) {
  *reinterpret_cast<uint4*>(p) = r.a;
  *reinterpret_cast<uint4*>(p + 64) = r.b;
}
__device__ __forceinline__ void store_raw16(float* p, const Raw16<float>& r) {
  *reinterpret_cast<float4*>(p) = r.a0;
  *reinterpret_cast<float4*>(p + 4) = r.a1;
  *reinterpret_cast<float4*>(p + 64) = r.b0;
  *reinterpret_cast<float4*>(p + 68) = r.b1;
}

// Two 32-bit floats in one 64-bit register, for the instructions that work on both at once (each half is
// rounded as the single instruction would round it).
typedef unsigned long long Float2x;
__device__ __forceinline__ Float2x pair_of(float lo, float hi) {
  Float2x p;
  asm("mov.b64 %0, {%1, %2};" : "=l"(p) : "f"(lo), "f"(hi));
  return p;
}
__device__ __forceinline__ float low_of(Float2x p) {
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p));
  return lo;
}
__device__ __forceinline__ float high_of(Float2x p) {
  float lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p));
  return hi;
}
__device__ __forceinline__ Float2x mul_pairs(Float2x a, Float2x b) {
  Float2x d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ Float2x fma_pairs(Float2x a, Float2x b, Float2x c) {
  Float2x d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

// norm (if the head has one) and rotation of the sixteen values this lane holds of one head; eight lanes hold
// the head.  wa, wb: the norm's weights at this lane's elements; cs, sn: cosines and sines of its eight pairs.
// The two members of a rotation pair travel in one 64-bit register.
__device__ __forceinline__ Head16 norm_and_rotate16(const Head16& x, bool has_norm, const float* wa, const float* wb, float eps,
                                                    bool rotate, const float* cs, const float* sn) {
  Float2x p[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) p[j] = pair_of(x.a[j], x.b[j]);
  // The other kernel sums four elements per lane (x^2, then y, z, w by fused multiply-adds) over 32 lanes by a
  // butterfly (16, 8, 4, 2, 1).  This lane's four quadruples are that kernel's lanes 2l, 2l + 1 (first members) and
  // 2l + 16, 2l + 17 (second members): its exchange over 16 is a sum inside this lane, those over 8, 4 and 2 are
  // exchanges over 4, 2 and 1 among the eight lanes, and the last one is again a sum inside the lane.  (The
  // exchanges run whether or not the head has a norm: the heads of a warp may differ in that.)
  const Float2x lo = fma_pairs(p[3], p[3], fma_pairs(p[2], p[2], fma_pairs(p[1], p[1], mul_pairs(p[0], p[0]))));
  const Float2x hi = fma_pairs(p[7], p[7], fma_pairs(p[6], p[6], fma_pairs(p[5], p[5], mul_pairs(p[4], p[4]))));
  float even = __fadd_rn(low_of(lo), high_of(lo)), odd = __fadd_rn(low_of(hi), high_of(hi));
#pragma unroll
  for (int offset = 4; offset > 0; offset >>= 1) {
    even += __shfl_xor_sync(0xffffffffu, even, offset);
    odd += __shfl_xor_sync(0xffffffffu, odd, offset);
  }
  if (has_norm) {
    const float inv = __frsqrt_rn((even + odd) * (1.0f / 128.0f) + eps);
    const Float2x inv2 = pair_of(inv, inv);
#pragma unroll
    for (int j = 0; j < 8; ++j) p[j] = mul_pairs(mul_pairs(p[j], inv2), pair_of(wa[j], wb[j]));      // (x inv) w, as normed()
  }
  Head16 y;
  if (rotate) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      // (a cos - b sin, b cos + a sin): the products with the sine are rounded first, as rotate_first/_second do
      const float a = low_of(p[j]), b = high_of(p[j]);
      const Float2x r = fma_pairs(p[j], pair_of(cs[j], cs[j]), pair_of(-__fmul_rn(b, sn[j]), __fmul_rn(a, sn[j])));
      y.a[j] = low_of(r);
      y.b[j] = high_of(r);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      y.a[j] = low_of(p[j]);
      y.b[j] = high_of(p[j]);
    }
  }
  return y;
}

template <typename T>
__global__ void __launch_bounds__(ROW_THREADS, ROW_BLOCKS_PER_SM)
qk_norm_rope_kv_row_kernel(const T* __restrict__ qkv, int qkv_stride, T* __restrict__ q_out, T* __restrict__ k_pool,
                           T* __restrict__ v_pool, const int* __restrict__ positions, const int* __restrict__ slots,
                           const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                           const float* __restrict__ inv_freq, const float* __restrict__ angles,
                           const float* __restrict__ cos_sin, int rows, int n_q, int n_kv, int page_size, int num_pages,
                           int* error_word) {
  // cos_sin: the rows' cosines and sines [rows, 128] (64 cosines, then 64 sines) computed once for the step by
  // rope_table_kernel, or null: then this block computes its rows' own, with the same arithmetic
  constexpr int D = 128, HALF = 64, HEADS_PER_PASS = ROW_THREADS / 8, STAGES = ROW_STAGES;
  extern __shared__ __align__(16) unsigned char staged_bytes[];       // [STAGES][heads of a row][128] of T
  __shared__ __align__(16) float row_cos_sin[STAGES][D];              // per row: 64 cosines, then 64 sines
  __shared__ __align__(16) float norm_weights[2][D];                  // of q heads, of k heads (ones where there is no norm)
  __shared__ int row_slot[STAGES];                                    // -1: the row's k and v are not stored
  srb_launch_dependents();
  norm_weights[0][threadIdx.x] = q_norm ? q_norm[threadIdx.x] : 1.f;
  norm_weights[1][threadIdx.x] = k_norm ? k_norm[threadIdx.x] : 1.f;
  const int group = threadIdx.x >> 3, l = threadIdx.x & 7;     // this thread's head of a pass, its place in the head
  const bool rotate = inv_freq || angles;
  const int heads_stored = slots ? n_q + 2 * n_kv : n_q;       // heads of a row that are brought in
  const size_t stage_bytes = (size_t)heads_stored * D * sizeof(T);
  const int row_chunks = (int)(stage_bytes / 16);              // 16-byte pieces of a row
  const int pair0 = l * 8;                                     // the eight pairs this lane holds
  srb_grid_dependency_wait();

  // asks for row number `turn` of this block (if there is one) into the ring; one group of copies either way
  auto request = [&](int turn) {
    const int row = blockIdx.x + turn * gridDim.x, stage = turn % STAGES;
    if (row < rows) {
      const unsigned char* src = reinterpret_cast<const unsigned char*>(qkv + (size_t)row * qkv_stride);
      unsigned char* dst = staged_bytes + stage * stage_bytes;
      for (int c = threadIdx.x; c < row_chunks; c += ROW_THREADS) cp_async_16(dst + c * 16, src + (size_t)c * 16, 16);
      if (rotate) {
        if (cos_sin) {
          if (threadIdx.x < D / 4)
            cp_async_16(&row_cos_sin[stage][threadIdx.x * 4], cos_sin + (size_t)row * D + threadIdx.x * 4, 16);
        } else if (threadIdx.x < HALF) {
          const float angle = angles ? angles[(size_t)row * HALF + threadIdx.x] : (float)positions[row] * inv_freq[threadIdx.x];
          sincosf(angle, &row_cos_sin[stage][HALF + threadIdx.x], &row_cos_sin[stage][threadIdx.x]);
        }
      }
      if (threadIdx.x == ROW_THREADS - 1) {
        int slot = -1;
        if (slots) {
          slot = slots[row];
          if (slot < 0 || slot >= num_pages * page_size) {
            atomicOr(error_word, SRB_FLAG_BAD_SLOT);
            slot = -1;
          }
        }
        row_slot[stage] = slot;
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int turn = 0; turn < STAGES - 1; ++turn) request(turn);
  for (int turn = 0;; ++turn) {
    const int row = blockIdx.x + turn * gridDim.x, stage = turn % STAGES;
    if (row >= rows) break;
    cp_async_wait<STAGES - 2>();      // all groups but the newest STAGES - 2: this row's has landed
    __syncthreads();                  // ... for every thread; and every thread has left the row before this one,
    request(turn + STAGES - 1);       // whose buffer the row STAGES - 1 ahead takes
    float cs[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f}, sn[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (rotate) {
      const float4* mine = reinterpret_cast<const float4*>(&row_cos_sin[stage][pair0]);
      const float4 c0 = mine[0], c1 = mine[1], s0 = mine[HALF / 4], s1 = mine[HALF / 4 + 1];
      cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
      sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    }
    const int slot = row_slot[stage];
    const int heads = slot >= 0 ? heads_stored : n_q;
    // where the row's k and v go: element offset of kv head 0, and the step from one kv head to the next
    const size_t kv_base = slot >= 0 ? ((size_t)(slot / page_size) * n_kv * page_size + (slot % page_size)) * D + l * 8 : 0;
    const size_t kv_step = (size_t)page_size * D;
    const T* src = reinterpret_cast<const T*>(staged_bytes + stage * stage_bytes) + l * 8;
    for (int first = 0; first < heads; first += HEADS_PER_PASS) {
      const int head = first + group;
      // The four heads of a warp run the exchanges together (they use the full mask, and stay inside a group of
      // eight lanes); a group whose head lies beyond the last one, or is a v head, computes on the last head's
      // values and stores nothing.
      const bool live = head < heads;
      const bool is_q = head < n_q, is_k = !is_q && head < n_q + n_kv;
      const Raw16<T> raw = load_raw16(src + (size_t)min(head, heads - 1) * D);
      if (live && !is_q && !is_k) {                            // a v head: no arithmetic
        store_raw16(v_pool + kv_base + (size_t)(head - n_q - n_kv) * kv_step, raw);
      }
      const bool work = live && (is_q || is_k);
      if (!__any_sync(0xffffffffu, work)) continue;
      const float* weights = norm_weights[is_q ? 0 : 1];
      const float4 wa0 = *reinterpret_cast<const float4*>(weights + pair0), wa1 = *reinterpret_cast<const float4*>(weights + pair0 + 4);
      const float4 wb0 = *reinterpret_cast<const float4*>(weights + HALF + pair0);
      const float4 wb1 = *reinterpret_cast<const float4*>(weights + HALF + pair0 + 4);
      const float wa[8] = {wa0.x, wa0.y, wa0.z, wa0.w, wa1.x, wa1.y, wa1.z, wa1.w};
      const float wb[8] = {wb0.x, wb0.y, wb0.z, wb0.w, wb1.x, wb1.y, wb1.z, wb1.w};
      const Head16 x = norm_and_rotate16(widen16(raw), (is_q ? q_norm : k_norm) != nullptr, wa, wb, eps, rotate, cs, sn);
      if (work) {
        if (is_q)
          store16(q_out + ((size_t)row * n_q + head) * D + l * 8, x);
        else
          store16(k_pool + kv_base + (size_t)(head - n_q) * kv_step, x);
      }
    }
  }
  cp_async_wait<0>();                 // (groups without copies may still be counted)
}

// The cosines and sines of every row's angles, once for a step: out[r, 0..half) = cos, out[r, half..2 half) = sin
// of float(positions[r]) * inv_freq[i] (or of angles[r, i]), the arithmetic of the kernels above.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  const float* __restrict__ angles, int rows, int half, float* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * half) return;
  const int row = i / half, pair = i - row * half;
  float sn, cs;
  sincosf(angles ? angles[i] : (float)positions[row] * inv_freq[pair], &sn, &cs);
  out[(size_t)row * 2 * half + pair] = cs;
  out[(size_t)row * 2 * half + half + pair] = sn;
}

extern "C" int srb_rope_table(const int* positions, const float* inv_freq, const float* angles, int rows, int rotary_dim,
                              float* out, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (rotary_dim <= 0 || (rotary_dim & 1) || (!inv_freq && !angles) || !out)
    SRB_FAIL("rope_table: an even rotary width, frequencies or angles, and an output are needed");
  const int total = rows * (rotary_dim >> 1);
  rope_table_kernel<<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>(positions, inv_freq, angles, rows, rotary_dim >> 1, out);
  SRB_LAUNCH_CHECK("rope_table");
  return SRB_OK;
}

// How many rows a step must have for the kernel that can take the table of srb_rope_table (fewer rows compute
// their angles inside the kernel, under the tail of the kernel ahead).
extern "C" int srb_rope_table_min_rows() { return 256; }

extern "C" int srb_qk_norm_rope_kv_table(const void* qkv, const float* qkv_parts, int num_parts, long long part_stride,
                                         int qkv_stride, void* q_out, void* k_pool, void* v_pool, const int* positions,
                                         const int* slots, const float* q_norm, const float* k_norm, float eps,
                                         const float* inv_freq, const float* angles, const float* cos_sin, int rotary_dim,
                                         int interleaved, int rows, int n_q, int n_kv, int head_dim, int page_size,
                                         int num_pages, int* error_word, int dtype, void* stream);

// `slots` may be null: then only the q heads are processed (a layer that reads another
// layer's cache writes nothing).
extern "C" int srb_qk_norm_rope_kv(const void* qkv, const float* qkv_parts, int num_parts, long long part_stride,
                                   int qkv_stride, void* q_out, void* k_pool, void* v_pool,
                                   const int* positions, const int* slots, const float* q_norm,
                                   const float* k_norm, float eps, const float* inv_freq, const float* angles,
                                   int rotary_dim,
                                   int interleaved, int rows, int n_q, int n_kv, int head_dim, int page_size,
                                   int num_pages, int* error_word, int dtype, void* stream) {
  return srb_qk_norm_rope_kv_table(qkv, qkv_parts, num_parts, part_stride, qkv_stride, q_out, k_pool, v_pool, positions,
                                   slots, q_norm, k_norm, eps, inv_freq, angles, nullptr, rotary_dim, interleaved, rows, n_q,
                                   n_kv, head_dim, page_size, num_pages, error_word, dtype, stream);
}

// The same with `cos_sin`: the table of srb_rope_table for these rows (float [rows, rotary_dim], 16-byte aligned),
// or null.  Only the kernel for many rows reads it; the values are those the kernels compute themselves.
extern "C" int srb_qk_norm_rope_kv_table(const void* qkv, const float* qkv_parts, int num_parts, long long part_stride,
                                         int qkv_stride, void* q_out, void* k_pool, void* v_pool, const int* positions,
                                         const int* slots, const float* q_norm, const float* k_norm, float eps,
                                         const float* inv_freq, const float* angles, const float* cos_sin, int rotary_dim,
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
  cudaStream_t s = (cudaStream_t)stream;
  const bool whole_head_pairs = !(inv_freq || angles) || (rotary_dim == head_dim && !interleaved);
  // (with fewer rows than about two per SM the kernel below, which spreads a row over blocks, is quicker)
  const int row_bytes_ok = dtype == SRB_DTYPE_F32 || qkv_stride % 8 == 0;      // 16-byte accesses of eight values
  const size_t staged = (size_t)ROW_STAGES * heads * 128 * (dtype == SRB_DTYPE_F32 ? 4 : 2);     // the ring of rows
  if (rows >= srb_rope_table_min_rows() && head_dim == 128 && vector_ok && whole_head_pairs && num_parts == 0 && row_bytes_ok &&
      staged <= 200 * 1024) {
    const float* table = (cos_sin && (((uintptr_t)cos_sin) & 15) == 0) ? cos_sin : nullptr;
    // as many blocks as stay on the chip together (fewer where the ring is large), every block with the same number of
    // rows, give or take one
    const int per_sm = (int)std::max<size_t>(1, std::min<size_t>(ROW_BLOCKS_PER_SM, (220 * 1024) / (staged + 3 * 1024)));
    const int resident = srb_sm_count() * per_sm;
    const int rows_per_block = (rows + resident - 1) / resident;
    const int blocks = (rows + rows_per_block - 1) / rows_per_block;
    if (dtype == SRB_DTYPE_F32) {
      SRB_CUDA_CALL(cudaFuncSetAttribute(qk_norm_rope_kv_row_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)staged));
      SRB_CUDA_CALL(srb_launch(qk_norm_rope_kv_row_kernel<float>, dim3(blocks), dim3(ROW_THREADS), staged, s,
                               (const float*)qkv, qkv_stride, (float*)q_out, (float*)k_pool, (float*)v_pool, positions,
                               slots, q_norm, k_norm, eps, inv_freq, angles, table, rows, n_q, n_kv, page_size, num_pages,
                               error_word));
    } else if (dtype == SRB_DTYPE_BF16) {
      SRB_CUDA_CALL(cudaFuncSetAttribute(qk_norm_rope_kv_row_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)staged));
      SRB_CUDA_CALL(srb_launch(qk_norm_rope_kv_row_kernel<__nv_bfloat16>, dim3(blocks), dim3(ROW_THREADS), staged, s,
                               (const __nv_bfloat16*)qkv, qkv_stride, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool,
                               (__nv_bfloat16*)v_pool, positions, slots, q_norm, k_norm, eps, inv_freq, angles, table, rows, n_q,
                               n_kv, page_size, num_pages, error_word));
    } else {
      SRB_FAIL("qk_norm_rope_kv: unknown dtype %d", dtype);
    }
    SRB_LAUNCH_CHECK("qk_norm_rope_kv_row");
    return SRB_OK;
  }
  // few rows (decode): one head per warp, so that the row is finished soonest; many rows: fewer tables of angles
  const int rounds = rows >= 64 ? ROPE_MAX_ROUNDS : 1;
  const int heads_per_block = ROPE_WARPS * rounds;
  dim3 grid(rows, (heads + heads_per_block - 1) / heads_per_block);
  const size_t smem = ((size_t)ROPE_WARPS * head_dim + ((inv_freq || angles) ? rotary_dim : 0)) * sizeof(float);
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
