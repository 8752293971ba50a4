// Row-wise kernels of the decoder: embedding gather, fused residual-add + RMSNorm,
// SiLU(gate)*up, bias add.  All arithmetic is 32-bit; T is the storage type of
// activations and weights (float or bfloat16).  The residual stream is 32-bit in both.
//
// Reference formulas: RMSNorm y = x / sqrt(mean(x^2) + eps) * w
// (crates/sglang-kernel/src/cpu.rs:26-34), SiLU*mul g / (1 + exp(-g)) * u (cpu.rs:119-123),
// embedding row copy with out-of-range ids flagged (cuda_bf16_kernels.rs:14-37).
#include "common.cuh"
#include "activations.cuh"

SRB_DEFINE_LAST_ERROR()
SRB_DEFINE_PDL_SWITCH()

// residual[row, :] = float(table[ids[row], :]); a bad id writes zeros and flags.
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ residual, int width, int vocab, int* error_word) {
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int row = blockIdx.x;
  const int id = ids[row];
  const bool bad = id < 0 || id >= vocab;
  if (bad && threadIdx.x == 0) atomicOr(error_word, SRB_FLAG_BAD_TOKEN);
  const T* src = table + (size_t)(bad ? 0 : id) * width;
  float* dst = residual + (size_t)row * width;
  if (sizeof(T) == 2 && width % 8 == 0 && (((uintptr_t)table | (uintptr_t)residual) & 15) == 0) {
    for (int i = threadIdx.x * 8; i < width; i += blockDim.x * 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src + i);
      const __nv_bfloat162* pair = reinterpret_cast<const __nv_bfloat162*>(&raw);
      float4 lo, hi;
      const float2 a = __bfloat1622float2(pair[0]), b = __bfloat1622float2(pair[1]);
      const float2 c = __bfloat1622float2(pair[2]), d = __bfloat1622float2(pair[3]);
      lo = bad ? make_float4(0.f, 0.f, 0.f, 0.f) : make_float4(a.x, a.y, b.x, b.y);
      hi = bad ? make_float4(0.f, 0.f, 0.f, 0.f) : make_float4(c.x, c.y, d.x, d.y);
      *reinterpret_cast<float4*>(dst + i) = lo;
      *reinterpret_cast<float4*>(dst + i + 4) = hi;
    }
    return;
  }
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = bad ? 0.f : srb_to_float(src[i]);
}

// x = residual[src] (+ delta[src]); optionally residual[src] = x; out[row] = T(x * rsqrt * w).
// `row_index` (optional) picks the source rows, so the final norm touches only the rows
// whose logits are wanted.  The row is staged in shared memory between the two passes.
// The pending sum may also arrive as `num_parts` float partial sums (a matrix product cut
// along K), `part_stride` elements apart; they are added in part order.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const float* __restrict__ delta_parts, int num_parts, size_t part_stride,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ row_index, int width, float eps,
                                   int write_residual) {
  extern __shared__ float staged[];          // width floats, then 33 floats of scratch
  float* scratch = staged + width;
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int row = blockIdx.x;
  const size_t src = (size_t)(row_index ? row_index[row] : row) * width;
  float partial = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float x = residual[src + i];
    if (delta) x += srb_to_float(delta[src + i]);
    for (int part = 0; part < num_parts; ++part) x += delta_parts[part * part_stride + src + i];
    if (write_residual) residual[src + i] = x;
    staged[i] = x;
    partial += x * x;
  }
  const float total = srb_block_sum(partial, scratch);
  const float inv = 1.0f / sqrtf(total / (float)width + eps);
  T* dst = out + (size_t)row * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x)
    dst[i] = srb_from_float<T>(staged[i] * inv * weight[i]);
}


// four consecutive values in one access (the address is a multiple of 4 elements)
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = raw;
}

// The same for widths that are a multiple of 4 and fit 4 * ITER values per thread: the row
// stays in registers, every load of a thread is issued before the first use (the row is
// small and the kernel is bound by latency, not by bandwidth), and the additions keep the
// order residual, delta, part 0, part 1, ...
template <typename T, int ITER>
__global__ void __launch_bounds__(1024)
add_rmsnorm_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                       const float* __restrict__ delta_parts, int num_parts, size_t part_stride,
                       const float* __restrict__ weight, T* __restrict__ out, const int* __restrict__ row_index,
                       int width, float eps, int write_residual) {
  // the partial sums of a thread's four columns are asked for eight at a time, so that a row of a decode step
  // costs one or two trips to L2, not one per few parts (measured at Qwen3-8B sizes: 3 % at batch 1, 7 % at 16)
  constexpr int PART_BATCH = ITER == 1 ? 8 : 4;
  __shared__ float scratch[33];
  srb_mark(SRB_MARK_NORM, 0);
  srb_launch_dependents();
  srb_grid_dependency_wait();
  srb_mark(SRB_MARK_NORM, 1);
  // the norm's weight travels with the row's loads, not after the sum of squares
  float4 w[ITER];
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int i = (it * blockDim.x + threadIdx.x) * 4;
    w[it] = i < width ? *reinterpret_cast<const float4*>(weight + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const int row = blockIdx.x;
  const size_t src = (size_t)(row_index ? row_index[row] : row) * width;
  float4 x[ITER];
  float partial = 0.f;
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int i = (it * blockDim.x + threadIdx.x) * 4;
    x[it] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < width) {
      x[it] = *reinterpret_cast<const float4*>(residual + src + i);
      float4 whole = make_float4(0.f, 0.f, 0.f, 0.f);
      if (delta) whole = load4(delta + src + i);
      for (int first = 0; first < num_parts || first == 0; first += PART_BATCH) {
        float4 d[PART_BATCH];
#pragma unroll
        for (int j = 0; j < PART_BATCH; ++j)
          if (first + j < num_parts) d[j] = *reinterpret_cast<const float4*>(delta_parts + (first + j) * part_stride + src + i);
        if (first == 0 && delta) {
          x[it].x += whole.x; x[it].y += whole.y; x[it].z += whole.z; x[it].w += whole.w;
        }
#pragma unroll
        for (int j = 0; j < PART_BATCH; ++j) {
          if (first + j < num_parts) {
            x[it].x += d[j].x; x[it].y += d[j].y; x[it].z += d[j].z; x[it].w += d[j].w;
          }
        }
      }
      if (write_residual) *reinterpret_cast<float4*>(residual + src + i) = x[it];
      partial += x[it].x * x[it].x + x[it].y * x[it].y + x[it].z * x[it].z + x[it].w * x[it].w;
    }
  }
  const float total = srb_block_sum(partial, scratch);
  const float inv = 1.0f / sqrtf(total / (float)width + eps);
  T* dst = out + (size_t)row * width;
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int i = (it * blockDim.x + threadIdx.x) * 4;
    if (i < width)
      store4(dst + i, make_float4(x[it].x * inv * w[it].x, x[it].y * inv * w[it].y, x[it].z * inv * w[it].z, x[it].w * inv * w[it].w));
  }
  srb_mark(SRB_MARK_NORM, 2);
}

// out[row, j] = act(gate_up[row, j]) * gate_up[row, inner + j], act being SRB_ACT_* `activation`
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int rows, int inner, int activation) {
  const size_t total = (size_t)rows * inner;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t row = idx / inner, col = idx % inner;
    const float g = srb_to_float(gate_up[row * 2 * inner + col]);
    const float u = srb_to_float(gate_up[row * 2 * inner + inner + col]);
    out[idx] = srb_from_float<T>(srb_gated<true>(activation, g, u));
  }
}

// The same with eight bfloat16 values (16 bytes) per thread and access; `inner` a multiple of 8.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out,
                                       int rows, int inner, int activation) {
  const int per_row = inner / 8;
  const size_t total = (size_t)rows * per_row;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t row = idx / per_row, col = (idx % per_row) * 8;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gate_up + row * 2 * inner + col);
    const uint4 u4 = *reinterpret_cast<const uint4*>(gate_up + row * 2 * inner + inner + col);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
      // the result is rounded to bfloat16 (8 bits): the hardware's exponential and division are exact enough
      o2[j] = __floats2bfloat162_rn(srb_gated<false>(activation, g.x, u.x), srb_gated<false>(activation, g.y, u.y));
    }
    *reinterpret_cast<uint4*>(out + row * inner + col) = o4;
  }
}

template <typename T>
__global__ void add_bias_kernel(T* __restrict__ values, const float* __restrict__ bias, int rows, int width) {
  const size_t total = (size_t)rows * width;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x)
    values[idx] = srb_from_float<T>(srb_to_float(values[idx]) + bias[idx % width]);
}

static int elementwise_grid(size_t total, int block) {
  size_t blocks = (total + block - 1) / block;
  const size_t cap = (size_t)srb_sm_count() * 16;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

extern "C" int srb_embedding(const int* ids, const void* table, float* residual, int rows, int width,
                             int vocab, int* error_word, int dtype, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (width <= 0 || vocab <= 0) SRB_FAIL("embedding: width %d and vocabulary %d must be positive", width, vocab);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32)
    SRB_CUDA_CALL(srb_launch(embedding_kernel<float>, dim3(rows), dim3(256), 0, s, ids, (const float*)table, residual,
                             width, vocab, error_word));
  else if (dtype == SRB_DTYPE_BF16)
    SRB_CUDA_CALL(srb_launch(embedding_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, s, ids,
                             (const __nv_bfloat16*)table, residual, width, vocab, error_word));
  else
    SRB_FAIL("embedding: unknown dtype %d", dtype);
  SRB_LAUNCH_CHECK("embedding");
  return SRB_OK;
}

template <typename T>
static int launch_add_rmsnorm(float* residual, const void* delta, const float* delta_parts, int num_parts,
                              size_t part_stride, const float* weight, void* out, const int* row_index, int rows,
                              int width, float eps, int write_residual, cudaStream_t s) {
  // widths that are a multiple of 4 (so float4 accesses stay aligned) and fit the registers
  const bool aligned = width % 4 == 0 && (((uintptr_t)residual | (uintptr_t)delta_parts | (uintptr_t)weight) & 15) == 0 &&
                       (((uintptr_t)delta | (uintptr_t)out) & (4 * sizeof(T) - 1)) == 0 && part_stride % 4 == 0;
  if (aligned && width <= 4 * 1024 * 2) {
    int threads = ((width / 4 + 31) / 32) * 32;
    if (threads > 1024) threads = 1024;
    if (width <= 4 * threads)
      SRB_CUDA_CALL(srb_launch(add_rmsnorm_vec_kernel<T, 1>, dim3(rows), dim3(threads), 0, s, residual, (const T*)delta,
                               delta_parts, num_parts, part_stride, weight, (T*)out, row_index, width, eps,
                               write_residual));
    else
      SRB_CUDA_CALL(srb_launch(add_rmsnorm_vec_kernel<T, 2>, dim3(rows), dim3(threads), 0, s, residual, (const T*)delta,
                               delta_parts, num_parts, part_stride, weight, (T*)out, row_index, width, eps,
                               write_residual));
    SRB_LAUNCH_CHECK("add_rmsnorm");
    return SRB_OK;
  }
  const size_t smem = (size_t)(width + 33) * sizeof(float);
  if (smem > 227 * 1024) SRB_FAIL("add_rmsnorm: width %d needs %zu bytes of shared memory (limit 232448)", width, smem);
  if (smem > 48 * 1024)
    SRB_CUDA_CALL(cudaFuncSetAttribute(add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int block = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
  SRB_CUDA_CALL(srb_launch(add_rmsnorm_kernel<T>, dim3(rows), dim3(block), smem, s, residual, (const T*)delta,
                           delta_parts, num_parts, part_stride, weight, (T*)out, row_index, width, eps,
                           write_residual));
  SRB_LAUNCH_CHECK("add_rmsnorm");
  return SRB_OK;
}

// delta: [rows_of_residual, width] of the output's type, or null; delta_parts: `num_parts` float
// tensors of that shape, `part_stride` elements apart, or null.
extern "C" int srb_add_rmsnorm(float* residual, const void* delta, const float* delta_parts, int num_parts,
                               long long part_stride, const float* weight, void* out, const int* row_index,
                               int rows, int width, float eps, int write_residual, int dtype, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (width <= 0) SRB_FAIL("add_rmsnorm: width %d must be positive", width);
  if (!(eps >= 0.f)) SRB_FAIL("add_rmsnorm: eps must be finite and non-negative");
  if (num_parts < 0 || (num_parts > 0 && !delta_parts)) SRB_FAIL("add_rmsnorm: partial sums are missing");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32)
    return launch_add_rmsnorm<float>(residual, delta, delta_parts, num_parts, (size_t)part_stride, weight, out,
                                     row_index, rows, width, eps, write_residual, s);
  if (dtype == SRB_DTYPE_BF16)
    return launch_add_rmsnorm<__nv_bfloat16>(residual, delta, delta_parts, num_parts, (size_t)part_stride, weight,
                                             out, row_index, rows, width, eps, write_residual, s);
  SRB_FAIL("add_rmsnorm: unknown dtype %d", dtype);
}

extern "C" int srb_gated_mul(const void* gate_up, void* out, int rows, int inner, int activation, int dtype,
                             void* stream) {
  if (rows <= 0) return SRB_OK;
  if (inner <= 0) SRB_FAIL("gated_mul: inner width %d must be positive", inner);
  if (activation < 0 || activation >= SRB_ACT_COUNT) SRB_FAIL("gated_mul: unknown activation %d", activation);
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = elementwise_grid((size_t)rows * inner, 256);
  if (dtype == SRB_DTYPE_F32)
    silu_mul_kernel<float><<<grid, 256, 0, s>>>((const float*)gate_up, (float*)out, rows, inner, activation);
  else if (dtype == SRB_DTYPE_BF16 && inner % 8 == 0 && (((uintptr_t)gate_up | (uintptr_t)out) & 15) == 0) {
    size_t blocks = ((size_t)rows * (inner / 8) + 255) / 256;
    if (blocks > srb_sm_count() * 64) blocks = srb_sm_count() * 64;
    silu_mul_bf16x8_kernel<<<(int)blocks, 256, 0, s>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, rows, inner, activation);
  } else if (dtype == SRB_DTYPE_BF16)
    silu_mul_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, rows,
                                                        inner, activation);
  else
    SRB_FAIL("gated_mul: unknown dtype %d", dtype);
  SRB_LAUNCH_CHECK("gated_mul");
  return SRB_OK;
}

extern "C" int srb_add_bias(void* values, const float* bias, int rows, int width, int dtype, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (width <= 0) SRB_FAIL("add_bias: width %d must be positive", width);
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = elementwise_grid((size_t)rows * width, 256);
  if (dtype == SRB_DTYPE_F32)
    add_bias_kernel<float><<<grid, 256, 0, s>>>((float*)values, bias, rows, width);
  else if (dtype == SRB_DTYPE_BF16)
    add_bias_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((__nv_bfloat16*)values, bias, rows, width);
  else
    SRB_FAIL("add_bias: unknown dtype %d", dtype);
  SRB_LAUNCH_CHECK("add_bias");
  return SRB_OK;
}

// tokens[i] = source[index[i]] where index[i] >= 0: rows whose token was chosen on the device by
// the step before and has not been to the host yet.  An index outside the source flags a bad token.
__global__ void take_tokens_kernel(int* __restrict__ tokens, const int* __restrict__ source,
                                   const int* __restrict__ index, int rows, int source_rows, int* error_word) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows) return;
  const int from = index[i];
  if (from < 0) return;
  if (from >= source_rows) {
    atomicOr(error_word, SRB_FLAG_BAD_TOKEN);
    return;
  }
  tokens[i] = source[from];
}

extern "C" int srb_take_tokens(int* tokens, const int* source, const int* index, int rows, int source_rows,
                               int* error_word, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (source_rows <= 0) SRB_FAIL("take_tokens: the source has no rows");
  take_tokens_kernel<<<(rows + 127) / 128, 128, 0, (cudaStream_t)stream>>>(tokens, source, index, rows, source_rows,
                                                                          error_word);
  SRB_LAUNCH_CHECK("take_tokens");
  return SRB_OK;
}
