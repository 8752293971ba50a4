// Token choice on the device: argmax and temperature sampling over 32-bit logits.
//
// Greedy: the index of the largest logit; among equal logits the lowest index (the
// reference's host argmax returns the last one, crates/sglang-srt/src/model_executor.rs:592-599;
// with 32-bit logits ties do not occur in practice).
// Temperature (model_executor.rs:471-480, :532-555): p_i = exp((l_i - max_j l_j) / T); the
// uniform u in [0, 1) picks the first index, in vocabulary order, whose running sum of
// p exceeds u * sum(p).  A row with temperature <= 0 falls back to argmax.
// Two kernels: 64 blocks per row reduce their chunk of the vocabulary, one block per row
// finishes (a vocabulary of 150 thousand entries is too long for one block per row).
#include "common.cuh"
#include <math.h>

SRB_DEFINE_LAST_ERROR()

#define SAMPLE_CHUNKS 64        // blocks that share one row's vocabulary in the first pass
#define SAMPLE_THREADS 256

// Pass 1, grid (SAMPLE_CHUNKS, rows): maximum, its lowest index, and sum of exp((l - max) / T)
// over the block's contiguous chunk of the vocabulary.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_chunk_kernel(const float* __restrict__ logits, int vocab, int stride, const float* __restrict__ temperature,
                    float* __restrict__ chunk_max, int* __restrict__ chunk_arg, float* __restrict__ chunk_sum) {
  __shared__ float sh_value[SAMPLE_THREADS / 32];
  __shared__ int sh_index[SAMPLE_THREADS / 32];
  __shared__ float scratch[33];
  const int row = blockIdx.y, chunk = blockIdx.x;
  const float* l = logits + (size_t)row * stride;
  const int per_chunk = (vocab + SAMPLE_CHUNKS - 1) / SAMPLE_CHUNKS;
  const int begin = min(vocab, chunk * per_chunk), end = min(vocab, begin + per_chunk);
  float best = -INFINITY;
  int best_index = 0x7fffffff;
  for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const float v = l[i];
    if (v > best || (v == best && i < best_index)) {
      best = v;
      best_index = i;
    }
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, best, offset);
    const int other_index = __shfl_xor_sync(0xffffffffu, best_index, offset);
    if (other > best || (other == best && other_index < best_index)) {
      best = other;
      best_index = other_index;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sh_value[warp] = best;
    sh_index[warp] = best_index;
  }
  __syncthreads();
  best = sh_value[0];
  best_index = sh_index[0];
  for (int w = 1; w < SAMPLE_THREADS / 32; ++w)
    if (sh_value[w] > best || (sh_value[w] == best && sh_index[w] < best_index)) {
      best = sh_value[w];
      best_index = sh_index[w];
    }
  const float temp = temperature ? temperature[row] : 0.f;
  float total = 0.f;
  if (temp > 0.f && best > -INFINITY) {
    float mine = 0.f;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) mine += expf((l[i] - best) / temp);
    total = srb_block_sum(mine, scratch);
  }
  if (threadIdx.x == 0) {
    const size_t at = (size_t)row * SAMPLE_CHUNKS + chunk;
    chunk_max[at] = best;
    chunk_arg[at] = best_index;
    chunk_sum[at] = total;
  }
}

// Pass 2, one block per row: the row's maximum; for a sampled row the chunk in which the
// running sum (in vocabulary order) passes u * total, then the token inside that chunk.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_pick_kernel(const float* __restrict__ logits, int vocab, int stride, const float* __restrict__ temperature,
                   const float* __restrict__ uniform, const float* __restrict__ chunk_max,
                   const int* __restrict__ chunk_arg, const float* __restrict__ chunk_sum, int* __restrict__ out) {
  __shared__ float part_sum[SAMPLE_THREADS];
  __shared__ float sh_max, sh_target, sh_prefix;
  __shared__ int sh_chunk;
  const int row = blockIdx.x;
  const float* l = logits + (size_t)row * stride;
  const float temp = temperature ? temperature[row] : 0.f;
  const size_t base = (size_t)row * SAMPLE_CHUNKS;
  if (threadIdx.x == 0) {
    float best = chunk_max[base];
    int best_index = chunk_arg[base];
    for (int c = 1; c < SAMPLE_CHUNKS; ++c)
      if (chunk_max[base + c] > best) {           // chunks are in index order: ties keep the lower index
        best = chunk_max[base + c];
        best_index = chunk_arg[base + c];
      }
    sh_max = best;
    sh_chunk = -1;
    if (!(temp > 0.f)) {
      out[row] = best_index == 0x7fffffff ? 0 : best_index;
    } else {
      float total = 0.f;
      for (int c = 0; c < SAMPLE_CHUNKS; ++c) total += chunk_sum[base + c] * expf((chunk_max[base + c] - best) / temp);
      const float target = uniform[row] * total;
      float running = 0.f;
      int owner = -1;
      for (int c = 0; c < SAMPLE_CHUNKS; ++c) {
        const float mass = chunk_sum[base + c] * expf((chunk_max[base + c] - best) / temp);
        if (target < running + mass) {
          owner = c;
          break;
        }
        running += mass;
      }
      if (owner < 0) {                             // rounding left the target at the total: last chunk with mass
        owner = SAMPLE_CHUNKS - 1;
        while (owner > 0 && !(chunk_sum[base + owner] > 0.f)) --owner;
        running = target;                          // forces the last token with p > 0 below
      }
      sh_chunk = owner;
      sh_target = target;
      sh_prefix = running;
    }
  }
  __syncthreads();
  if (sh_chunk < 0) return;
  const int per_chunk = (vocab + SAMPLE_CHUNKS - 1) / SAMPLE_CHUNKS;
  const int begin = min(vocab, sh_chunk * per_chunk), end = min(vocab, begin + per_chunk);
  const int per_thread = (end - begin + blockDim.x - 1) / blockDim.x;
  const int mine_begin = min(end, begin + (int)threadIdx.x * per_thread), mine_end = min(end, mine_begin + per_thread);
  const float scaled_max = sh_max;
  float mine = 0.f;
  for (int i = mine_begin; i < mine_end; ++i) mine += expf((l[i] - scaled_max) / temp);
  part_sum[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    float running = sh_prefix;
    int owner = -1;
    for (int t = 0; t < (int)blockDim.x; ++t) {
      if (sh_target < running + part_sum[t]) {
        owner = t;
        break;
      }
      running += part_sum[t];
    }
    if (owner < 0) {                               // take the last token of the chunk that has p > 0
      int last = end - 1;
      while (last > begin && !(expf((l[last] - scaled_max) / temp) > 0.f)) --last;
      out[row] = last;
      sh_chunk = -1;
    } else {
      sh_chunk = owner;
      sh_prefix = running;
    }
  }
  __syncthreads();
  if (sh_chunk < 0 || (int)threadIdx.x != sh_chunk) return;
  float running = sh_prefix;
  int pick = mine_end - 1;
  for (int i = mine_begin; i < mine_end; ++i) {
    running += expf((l[i] - scaled_max) / temp);
    if (sh_target < running) {
      pick = i;
      break;
    }
  }
  out[row] = pick;
}

extern "C" int srb_sample_scratch_floats(int rows) { return rows * SAMPLE_CHUNKS * 3; }

// logits [rows, stride] with `vocab` valid columns; temperature and uniform are [rows] or
// null (null temperature = greedy for every row); out [rows] int32; scratch holds
// srb_sample_scratch_floats(rows) 4-byte words.
extern "C" int srb_sample(const float* logits, int rows, int vocab, int stride, const float* temperature,
                          const float* uniform, int* out, float* scratch, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (vocab <= 0 || stride < vocab) SRB_FAIL("sample: vocabulary %d and stride %d do not fit", vocab, stride);
  if (temperature && !uniform) SRB_FAIL("sample: temperature sampling needs uniform numbers");
  if (!scratch) SRB_FAIL("sample: scratch memory is needed");
  if (rows > 65535) SRB_FAIL("sample: %d rows exceed one launch", rows);
  float* chunk_max = scratch;
  int* chunk_arg = reinterpret_cast<int*>(scratch + (size_t)rows * SAMPLE_CHUNKS);
  float* chunk_sum = scratch + (size_t)rows * SAMPLE_CHUNKS * 2;
  cudaStream_t s = (cudaStream_t)stream;
  sample_chunk_kernel<<<dim3(SAMPLE_CHUNKS, rows), SAMPLE_THREADS, 0, s>>>(logits, vocab, stride, temperature,
                                                                          chunk_max, chunk_arg, chunk_sum);
  SRB_LAUNCH_CHECK("sample_chunk");
  sample_pick_kernel<<<rows, SAMPLE_THREADS, 0, s>>>(logits, vocab, stride, temperature, uniform, chunk_max,
                                                     chunk_arg, chunk_sum, out);
  SRB_LAUNCH_CHECK("sample_pick");
  return SRB_OK;
}
