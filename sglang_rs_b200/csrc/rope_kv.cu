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
    for (int e = lane; e < head_dim; e += 32) staged[e] = normed(staged[e], inv, norm_weight[e]);
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


// Many rows (256 and more), head_dim 128, rotation of the whole head in half-split pairs, the
// projection in one tensor: one block per row.  Half a warp takes a head: lane l of the half holds the
// eight elements 8l..8l+7 (one 16-byte access in bfloat16, two in 32-bit), its rotation partner sits eight
// lanes away.  A block's sixteen half-warps take sixteen heads per pass, and a thread asks for the data of
// all its passes (up to ROW_PASSES) before it touches any of them, so that each SM has some hundred KB in
// flight; the table of angles is computed while those loads travel.  v heads are copied as they are.
// Same arithmetic as the kernel above, bit for bit: the sum of squares is added up in the order of that
// kernel's warp reduction (four elements per lane there: this lane's two halves stand for two of its lanes).
#define ROW_WARPS 8
#define ROW_PASSES 4
struct Head8 { float v[8]; };
template <typename T> struct Raw8;
template <> struct Raw8<__nv_bfloat16> { uint4 a; };
template <> struct Raw8<float> { float4 a, b; };
__device__ __forceinline__ Raw8<__nv_bfloat16> load_raw8(const __nv_bfloat16* p) {
  Raw8<__nv_bfloat16> r;
  r.a = *reinterpret_cast<const uint4*>(p);
  return r;
}
__device__ __forceinline__ Raw8<float> load_raw8(const float* p) {
  Raw8<float> r;
  r.a = *reinterpret_cast<const float4*>(p);
  r.b = *reinterpret_cast<const float4*>(p + 4);
  return r;
}
__device__ __forceinline__ Head8 widen8(const Raw8<__nv_bfloat16>& r) {
  Head8 h;
  const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&r.a);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(pairs[j]);
    h.v[2 * j] = f.x;
    h.v[2 * j + 1] = f.y;
  }
  return h;
}
__device__ __forceinline__ Head8 widen8(const Raw8<float>& r) {
  Head8 h;
  h.v[0] = r.a.x; h.v[1] = r.a.y; h.v[2] = r.a.z; h.v[3] = r.a.w;
  h.v[4] = r.b.x; h.v[5] = r.b.y; h.v[6] = r.b.z; h.v[7] = r.b.w;
  return h;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const Head8& h) {
  uint4 raw;
  __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) pairs[j] = __floats2bfloat162_rn(h.v[2 * j], h.v[2 * j + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}
__device__ __forceinline__ void store8(float* p, const Head8& h) {
  *reinterpret_cast<float4*>(p) = make_float4(h.v[0], h.v[1], h.v[2], h.v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(h.v[4], h.v[5], h.v[6], h.v[7]);
}
__device__ __forceinline__ void store_raw8(__nv_bfloat16* p, const Raw8<__nv_bfloat16>& r) { *reinterpret_cast<uint4*>(p) = r.a; }
__device__ __forceinline__ void store_raw8(float* p, const Raw8<float>& r) {
  *reinterpret_cast<float4*>(p) = r.a;
  *reinterpret_cast<float4*>(p + 4) = r.b;
}

// norm (if a weight is given) and rotation of the eight values this lane holds of one head; the sixteen lanes
// of a half-warp hold the head; `sn` holds the sines with the sign of this lane's side of the rotation pairs
__device__ __forceinline__ Head8 norm_and_rotate8(Head8 x, bool has_norm, const float* w, float eps, bool rotate,
                                                  const float* cs, const float* sn) {
  // The other kernel sums four elements per lane over 32 lanes by a butterfly (16, 8, 4, 2, 1); here a lane's
  // two quadruples are that kernel's lanes 2l and 2l + 1, so its first four exchanges become 8, 4, 2, 1 within
  // the half-warp for each quadruple, and its last one is the sum of the two quadruples.  (The exchanges run
  // whether or not this half's head has a norm: the two halves of a warp may differ in that.)
  float lo = sum_squares4(make_float4(x.v[0], x.v[1], x.v[2], x.v[3]));
  float hi = sum_squares4(make_float4(x.v[4], x.v[5], x.v[6], x.v[7]));
#pragma unroll
  for (int offset = 8; offset > 0; offset >>= 1) {
    lo += __shfl_xor_sync(0xffffffffu, lo, offset);
    hi += __shfl_xor_sync(0xffffffffu, hi, offset);
  }
  if (has_norm) {
    const float inv = __frsqrt_rn((lo + hi) * (1.0f / 128.0f) + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) x.v[j] = normed(x.v[j], inv, w[j]);
  }
  if (rotate) {
    // rotate_first(a, b) = a cos - b sin for the first of a pair, rotate_second(a, b) = b cos + a sin for the second:
    // with the partner's value in `other` both are own * cos + other * (-+ sin), and `sn` comes with that sign
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, x.v[j], 8);
      x.v[j] = __fmaf_rn(x.v[j], cs[j], __fmul_rn(other, sn[j]));
    }
  }
  return x;
}

template <typename T>
__global__ void __launch_bounds__(ROW_WARPS * 32, 3)
qk_norm_rope_kv_row_kernel(const T* __restrict__ qkv, int qkv_stride, T* __restrict__ q_out, T* __restrict__ k_pool,
                           T* __restrict__ v_pool, const int* __restrict__ positions, const int* __restrict__ slots,
                           const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                           const float* __restrict__ inv_freq, const float* __restrict__ angles,
                           const float* __restrict__ cos_sin, int n_q, int n_kv, int page_size, int num_pages,
                           int* error_word) {
  // cos_sin: the rows' cosines and sines [rows, 128] (64 cosines, then 64 sines) computed once for the step by
  // rope_table_kernel, or null: then this block computes its row's own, with the same arithmetic
  constexpr int D = 128, HALF = 64, HEADS_PER_PASS = ROW_WARPS * 2;
  __shared__ __align__(16) float cos_table[HALF], sin_table[HALF];
  __shared__ __align__(16) float norm_weights[2][D];          // of q heads, of k heads (ones where there is no norm)
  srb_launch_dependents();
  norm_weights[threadIdx.x >> 7][threadIdx.x & 127] =
      (threadIdx.x < D ? q_norm : k_norm) ? (threadIdx.x < D ? q_norm : k_norm)[threadIdx.x & 127] : 1.f;
  const int lane = threadIdx.x & 31;
  const int half_warp = threadIdx.x >> 4, l = lane & 15;      // this thread's head of a pass, its place in the head
  const int row = blockIdx.x;
  const bool rotate = inv_freq || angles;
  int slot = 0;
  bool slot_ok = true;
  if (slots) {
    slot = slots[row];
    slot_ok = slot >= 0 && slot < num_pages * page_size;
    if (!slot_ok && threadIdx.x == 0) atomicOr(error_word, SRB_FLAG_BAD_SLOT);
  }
  const int heads = (slots && slot_ok) ? n_q + 2 * n_kv : n_q;
  const bool first_half = l < 8;
  const int pair0 = (l & 7) * 8;                               // the eight pairs this lane takes part in
  srb_grid_dependency_wait();
  const T* src = qkv + (size_t)row * qkv_stride + l * 8;
  // where the row's k and v go: element offset of kv head 0, and the step from one kv head to the next
  const size_t kv_base = ((size_t)(slot / page_size) * n_kv * page_size + (slot % page_size)) * D + l * 8;
  const size_t kv_step = (size_t)page_size * D;
  bool table_ready = !rotate;
  float cs[8], sn[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    cs[j] = 1.f;
    sn[j] = 0.f;
  }
  if (rotate && cos_sin) {                                     // these loads travel together with the first heads'
    const float* mine = cos_sin + (size_t)row * D + pair0;
    const float4 c0 = *reinterpret_cast<const float4*>(mine), c1 = *reinterpret_cast<const float4*>(mine + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(mine + HALF), s1 = *reinterpret_cast<const float4*>(mine + HALF + 4);
    cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
    sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    if (first_half) {
#pragma unroll
      for (int j = 0; j < 8; ++j) sn[j] = -sn[j];
    }
    table_ready = true;
  }
  bool synced = false;
  for (int first = 0; first < heads; first += HEADS_PER_PASS * ROW_PASSES) {
    Raw8<T> raw[ROW_PASSES];
#pragma unroll
    for (int p = 0; p < ROW_PASSES; ++p) {
      const int head = first + p * HEADS_PER_PASS + half_warp;
      if (head < heads) raw[p] = load_raw8(src + (size_t)head * D);
    }
    if (!synced) {
      // while the loads above are on their way: the angles of the row, unless the step brought their table
      if (!table_ready && threadIdx.x < HALF) {
        if (angles) {
          sincosf(angles[(size_t)row * HALF + threadIdx.x], &sin_table[threadIdx.x], &cos_table[threadIdx.x]);
        } else if (inv_freq) {
          sincosf((float)positions[row] * inv_freq[threadIdx.x], &sin_table[threadIdx.x], &cos_table[threadIdx.x]);
        }
      }
      __syncthreads();                                         // the norm weights and the angles are in shared memory
      if (!table_ready) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          cs[j] = cos_table[pair0 + j];
          sn[j] = first_half ? -sin_table[pair0 + j] : sin_table[pair0 + j];
        }
        table_ready = true;
      }
      synced = true;
    }
#pragma unroll
    for (int p = 0; p < ROW_PASSES; ++p) {
      const int head = first + p * HEADS_PER_PASS + half_warp;
      // both halves of a warp run the exchanges together; a half whose head lies beyond the last one idles
      const bool live = head < heads;
      const bool is_q = head < n_q, is_k = !is_q && head < n_q + n_kv;
      if (!__any_sync(0xffffffffu, live)) continue;
      if (live && !is_q && !is_k) {                            // a v head: no arithmetic
        store_raw8(v_pool + kv_base + (size_t)(head - n_q - n_kv) * kv_step, raw[p]);
      }
      const bool work = live && (is_q || is_k);
      if (!__any_sync(0xffffffffu, work)) continue;
      Head8 x;
      if (work) {
        x = widen8(raw[p]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) x.v[j] = 0.f;
      }
      // the exchanges inside use the full mask, so every lane of the warp calls it; a half without work carries zeros
      const bool q_side = is_q || !live;
      const float4 w0 = *reinterpret_cast<const float4*>(&norm_weights[q_side ? 0 : 1][l * 8]);
      const float4 w1 = *reinterpret_cast<const float4*>(&norm_weights[q_side ? 0 : 1][l * 8 + 4]);
      const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      x = norm_and_rotate8(x, (q_side ? q_norm : k_norm) != nullptr, w, eps, rotate, cs, sn);
      if (work) {
        if (is_q)
          store8(q_out + ((size_t)row * n_q + head) * D + l * 8, x);
        else
          store8(k_pool + kv_base + (size_t)(head - n_q) * kv_step, x);
      }
    }
  }
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
  if (rows >= srb_rope_table_min_rows() && head_dim == 128 && vector_ok && whole_head_pairs && num_parts == 0 && row_bytes_ok) {
    const float* table = (cos_sin && (((uintptr_t)cos_sin) & 15) == 0) ? cos_sin : nullptr;
    if (dtype == SRB_DTYPE_F32)
      SRB_CUDA_CALL(srb_launch(qk_norm_rope_kv_row_kernel<float>, dim3(rows), dim3(ROW_WARPS * 32), 0, s,
                               (const float*)qkv, qkv_stride, (float*)q_out, (float*)k_pool, (float*)v_pool, positions,
                               slots, q_norm, k_norm, eps, inv_freq, angles, table, n_q, n_kv, page_size, num_pages,
                               error_word));
    else if (dtype == SRB_DTYPE_BF16)
      SRB_CUDA_CALL(srb_launch(qk_norm_rope_kv_row_kernel<__nv_bfloat16>, dim3(rows), dim3(ROW_WARPS * 32), 0, s,
                               (const __nv_bfloat16*)qkv, qkv_stride, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool,
                               (__nv_bfloat16*)v_pool, positions, slots, q_norm, k_norm, eps, inv_freq, angles, table, n_q,
                               n_kv, page_size, num_pages, error_word));
    else
      SRB_FAIL("qk_norm_rope_kv: unknown dtype %d", dtype);
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
