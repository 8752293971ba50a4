// Token choice on the device: argmax and temperature sampling over 32-bit logits.
//
// Greedy: the index of the largest logit; among equal logits the lowest index (the
// reference's host argmax returns the last one, crates/sglang-srt/src/model_executor.rs:592-599;
// with 32-bit logits ties do not occur in practice).
// Temperature (model_executor.rs:471-480, :532-555): p_i = exp(l_i / T - max_j l_j / T); the
// uniform u in [0, 1) picks the first index, in vocabulary order, whose running sum of
// p exceeds u * sum(p).  A row with temperature <= 0 falls back to argmax.
#include "common.cuh"
#include <math.h>

SRB_DEFINE_LAST_ERROR()

#define SAMPLE_THREADS 1024

__device__ __forceinline__ void argmax_reduce(float& value, int& index, float* sh_value, int* sh_index) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, value, offset);
    const int other_index = __shfl_xor_sync(0xffffffffu, index, offset);
    if (other > value || (other == value && other_index < index)) {
      value = other;
      index = other_index;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) {
    sh_value[warp] = value;
    sh_index[warp] = index;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float best = sh_value[0];
    int best_index = sh_index[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (sh_value[w] > best || (sh_value[w] == best && sh_index[w] < best_index)) {
        best = sh_value[w];
        best_index = sh_index[w];
      }
    sh_value[0] = best;
    sh_index[0] = best_index;
  }
  __syncthreads();
  value = sh_value[0];
  index = sh_index[0];
  __syncthreads();
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, int stride, const float* __restrict__ temperature,
              const float* __restrict__ uniform, int* __restrict__ out) {
  __shared__ float sh_value[32];
  __shared__ int sh_index[32];
  __shared__ float chunk_sum[SAMPLE_THREADS];
  __shared__ float scratch[33];
  const int row = blockIdx.x;
  const float* l = logits + (size_t)row * stride;
  const float temp = temperature ? temperature[row] : 0.f;

  float best = -INFINITY;
  int best_index = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = l[i];
    if (v > best || (v == best && i < best_index)) {
      best = v;
      best_index = i;
    }
  }
  argmax_reduce(best, best_index, sh_value, sh_index);
  if (!(temp > 0.f)) {
    if (threadIdx.x == 0) out[row] = best_index == 0x7fffffff ? 0 : best_index;
    return;
  }

  // contiguous chunk per thread, so that the running sum follows vocabulary order
  const float max_scaled = best / temp;
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int begin = min(vocab, (int)threadIdx.x * chunk), end = min(vocab, begin + chunk);
  float mine = 0.f;
  for (int i = begin; i < end; ++i) mine += expf(l[i] / temp - max_scaled);
  chunk_sum[threadIdx.x] = mine;
  const float total = srb_block_sum(mine, scratch);
  const float target = uniform[row] * total;
  __shared__ int owner;
  __shared__ float owner_prefix;
  if (threadIdx.x == 0) {
    float running = 0.f;
    int who = -1;
    float prefix = 0.f;
    for (int t = 0; t < (int)blockDim.x; ++t) {
      if (target < running + chunk_sum[t]) {
        who = t;
        prefix = running;
        break;
      }
      running += chunk_sum[t];
    }
    owner = who;
    owner_prefix = prefix;
  }
  __syncthreads();
  if (owner < 0) {
    // rounding left the target at or past the total: take the last token with p > 0
    if (threadIdx.x == 0) {
      int last = vocab - 1;
      while (last > 0 && !(expf(l[last] / temp - max_scaled) > 0.f)) --last;
      out[row] = last;
    }
    return;
  }
  if ((int)threadIdx.x == owner) {
    float running = owner_prefix;
    int pick = end - 1;
    for (int i = begin; i < end; ++i) {
      running += expf(l[i] / temp - max_scaled);
      if (target < running) {
        pick = i;
        break;
      }
    }
    out[row] = pick;
  }
}

// logits [rows, stride] with `vocab` valid columns; temperature and uniform are [rows] or
// null (null temperature = greedy for every row); out [rows] int32.
extern "C" int srb_sample(const float* logits, int rows, int vocab, int stride, const float* temperature,
                          const float* uniform, int* out, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (vocab <= 0 || stride < vocab) SRB_FAIL("sample: vocabulary %d and stride %d do not fit", vocab, stride);
  if (temperature && !uniform) SRB_FAIL("sample: temperature sampling needs uniform numbers");
  sample_kernel<<<rows, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(logits, vocab, stride, temperature, uniform, out);
  SRB_LAUNCH_CHECK("sample");
  return SRB_OK;
}
