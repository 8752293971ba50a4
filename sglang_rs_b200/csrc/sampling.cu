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

// ---------------------------------------------------------------------------------------------
// Sampling with top-k, top-p and min-p (the reference's rule, model_executor.rs:471-555): the
// probabilities p_i = exp(l_i / T - max_j l_j / T) are sorted descending (equal ones in index
// order); the first k are kept; an item is kept while the mass before it, as a fraction of the
// mass of those k, is below top_p, and while p_i >= p_0 * min_p; u * (kept mass) picks the first
// kept item whose running mass exceeds it.
//
// Nothing is sorted here.  Every cut keeps a prefix of the sorted order, and a prefix is named by
// a probability tau and a number n: all items above tau and the first n, in index order, of
// those equal to tau.  The item at which a running count or a running mass crosses a threshold
// is found by a radix search over the bits of p (11 + 11 + 10 bits): the histogram of the first
// 11 bits (counts and masses per bin) is built once per row, together with the p themselves,
// which go to scratch memory; each search then refines inside one bin with two light passes
// over the stored p.  The position among equal items follows by division.  Masses are integers
// (p * 2^40, rounded), so sums do not depend on the order in which threads add them and a row's
// token does not depend on timing.  Up to eight blocks per row (a thread-block cluster) share the
// passes that build the first histogram; one of them does the searches.
#define FS_THREADS 1024
#define FS_BINS 2048
#define FS_BATCH 8          // loads of a thread in flight at once
#define FS_QUADS 4          // the same for 16-byte loads of the stored probabilities
typedef unsigned long long u64;

__device__ __forceinline__ u64 fs_mass(float p) { return __float2ull_rn(p * 1099511627776.0f); }   // p * 2^40

struct FsShared {
  u64 first_mass[FS_BINS];        // histogram of the first 11 bits of p: mass and count per bin
  u64 mass[FS_BINS + 1];          // histogram of the level being refined; the last entry is a mailbox
  u64 totals[99];
  unsigned first_count[FS_BINS];
  unsigned count[FS_BINS];
  unsigned found[4];
  float warp_max[FS_THREADS / 32];
  float slice_max;
  int index;
};

// loads from the shared memory of another block of the cluster
__device__ __forceinline__ unsigned fs_peer_u32(const unsigned* mine, unsigned rank) {
  unsigned local = (unsigned)__cvta_generic_to_shared(mine), remote, v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
  return v;
}
__device__ __forceinline__ u64 fs_peer_u64(const u64* mine, unsigned rank) {
  unsigned local = (unsigned)__cvta_generic_to_shared(mine), remote;
  u64 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(remote) : "memory");
  return v;
}

// sum over the block; every thread gets it
__device__ __forceinline__ u64 fs_block_sum(u64 v, u64* scratch /* 33 */) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    u64 t = lane < FS_THREADS / 32 ? scratch[lane] : 0ull;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) t += __shfl_xor_sync(0xffffffffu, t, offset);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// One item per lane (or none) into a histogram.  Called by whole warps.  Lanes that fall into the same
// bin as the first lane still waiting add once, through that lane (up to three such groups: a flat row
// puts a whole warp into one or two bins, and thirty-two additions to one address would queue up);
// the lanes left after that add for themselves (a peaked row spreads a warp over many bins).
__device__ __forceinline__ void fs_add(unsigned* count, u64* mass, bool mine, unsigned bin, u64 w) {
  unsigned waiting = __ballot_sync(0xffffffffu, mine);
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int round = 0; round < 3; ++round) {
    if (waiting == 0) return;
    const int leader = __ffs(waiting) - 1;
    const unsigned lead_bin = __shfl_sync(0xffffffffu, bin, leader);
    const bool in_group = ((waiting >> lane) & 1u) && bin == lead_bin;
    const unsigned group = __ballot_sync(0xffffffffu, in_group);
    if (__popc(group) >= 4) {
      const unsigned lo = __reduce_add_sync(0xffffffffu, in_group ? (unsigned)(w & 0xFFFFFu) : 0u);
      const unsigned mid = __reduce_add_sync(0xffffffffu, in_group ? (unsigned)((w >> 20) & 0xFFFFFu) : 0u);
      const unsigned hi = __reduce_add_sync(0xffffffffu, in_group ? (unsigned)(w >> 40) : 0u);
      if (lane == leader) {
        atomicAdd(&count[lead_bin], (unsigned)__popc(group));
        atomicAdd(&mass[lead_bin], (u64)lo + ((u64)mid << 20) + ((u64)hi << 40));
      }
    } else if (in_group) {
      atomicAdd(&count[bin], 1u);
      atomicAdd(&mass[bin], w);
    }
    waiting &= ~group;
  }
  if ((waiting >> lane) & 1u) {
    atomicAdd(&count[bin], 1u);
    atomicAdd(&mass[bin], w);
  }
}

#define FS_BY_COUNT 0
#define FS_BY_MASS 1
#define FS_BY_KEY 2

// Walks a histogram from its top bin down.  BY_COUNT / BY_MASS: the bin in which the running count or
// mass (starting at `base`, what lies above the histogram's range) first exceeds `want`.  BY_KEY: the
// bin `want`.  Leaves the bin in found[0], the count of the bins above it in found[1] and their mass
// in the mailbox; every thread reads them after the call.
template <int MODE>
__device__ void fs_scan(const unsigned* count, const u64* mass, int nbins, u64 want, u64 base, FsShared& sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {                        // what holds if no bin is found (a row of NaN)
    sh.found[0] = 0;
    sh.found[1] = 0;
    sh.mass[FS_BINS] = 0;
  }
  // thread t owns bins nbins - 1 - 2t and nbins - 2 - 2t; an inclusive scan over the threads, in the order
  // of falling bins, tells each what lies above its bins
  const int b0 = nbins - 1 - 2 * (int)threadIdx.x, b1 = b0 - 1;
  const u64 c0 = b0 >= 0 ? (u64)count[b0] : 0ull, c1 = b1 >= 0 ? (u64)count[b1] : 0ull;
  const u64 m0 = b0 >= 0 ? mass[b0] : 0ull, m1 = b1 >= 0 ? mass[b1] : 0ull;
  u64 run_c = c0 + c1, run_m = m0 + m1;
#pragma unroll
  for (int offset = 1; offset < 32; offset <<= 1) {
    const u64 tc = __shfl_up_sync(0xffffffffu, run_c, offset), tm = __shfl_up_sync(0xffffffffu, run_m, offset);
    if (lane >= offset) {
      run_c += tc;
      run_m += tm;
    }
  }
  __syncthreads();
  if (lane == 31) {
    sh.totals[33 + warp] = run_c;
    sh.totals[66 + warp] = run_m;
  }
  __syncthreads();
  u64 start_c = run_c - (c0 + c1), start_m = run_m - (m0 + m1);       // above this thread's bins, inside the range
  for (int w = 0; w < warp; ++w) {
    start_c += sh.totals[33 + w];
    start_m += sh.totals[66 + w];
  }
  bool first = false, second = false;
  if (MODE == FS_BY_KEY) {
    first = b0 >= 0 && (u64)b0 == want;
    second = b1 >= 0 && (u64)b1 == want;
  } else {
    const u64 v0 = MODE == FS_BY_COUNT ? c0 : m0, v1 = MODE == FS_BY_COUNT ? c1 : m1;
    const u64 start_v = base + (MODE == FS_BY_COUNT ? start_c : start_m);
    first = b0 >= 0 && start_v <= want && want < start_v + v0;
    second = b1 >= 0 && start_v + v0 <= want && want < start_v + v0 + v1;
  }
  if (first) {
    sh.found[0] = (unsigned)b0;
    sh.found[1] = (unsigned)start_c;
    sh.mass[FS_BINS] = start_m;
  } else if (second) {
    sh.found[0] = (unsigned)b1;
    sh.found[1] = (unsigned)(start_c + c0);
    sh.mass[FS_BINS] = start_m + m0;
  }
  __syncthreads();
}

struct FsCrossing {
  unsigned key;      // bits of the probability at which the threshold is crossed
  u64 above;         // items with a larger probability
  u64 mass_above;    // their mass
  u64 equal;         // items with exactly this probability
};

// BY_COUNT / BY_MASS: the item, in descending order of p, at which the running count or the running
// mass first exceeds `want` (before <= want < before + own); the caller guarantees that it exists.
// BY_KEY: the probability with the bits `want`.  `p` is the row of stored probabilities.
template <int MODE>
__device__ FsCrossing fs_search(const float* __restrict__ p, int vocab, u64 want, FsShared& sh) {
  FsCrossing c;
  c.above = 0;
  c.mass_above = 0;
  unsigned prefix = 0;
  int fixed_bits = 0;
#pragma unroll 1
  for (int level = 0; level < 3; ++level) {
    const int bits = level < 2 ? 11 : 10;
    const int shift = 32 - fixed_bits - bits;
    const u64 target = MODE == FS_BY_KEY ? (u64)(((unsigned)want >> shift) & ((1u << bits) - 1)) : want;
    const u64 base = MODE == FS_BY_COUNT ? c.above : c.mass_above;
    if (level == 0) {
      fs_scan<MODE>(sh.first_count, sh.first_mass, 1 << bits, target, base, sh);
    } else {
      for (int b = threadIdx.x; b < FS_BINS; b += FS_THREADS) {
        sh.count[b] = 0;
        sh.mass[b] = 0;
      }
      __syncthreads();
      // the stored row is padded to a multiple of four with values that match no prefix
      const float4* p4 = reinterpret_cast<const float4*>(p);
      const int quads = (vocab + 3) >> 2;
      for (int start = 0; start < quads; start += FS_THREADS * FS_QUADS) {
        float4 value[FS_QUADS];
#pragma unroll
        for (int j = 0; j < FS_QUADS; ++j) {
          const int i = start + j * FS_THREADS + (int)threadIdx.x;
          value[j] = i < quads ? p4[i] : make_float4(-1.f, -1.f, -1.f, -1.f);     // the sign bit never matches a prefix
        }
#pragma unroll
        for (int j = 0; j < FS_QUADS; ++j) {
          const float four[4] = {value[j].x, value[j].y, value[j].z, value[j].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const unsigned key = __float_as_uint(four[e]);
            const bool mine = (key >> (32 - fixed_bits)) == prefix;
            fs_add(sh.count, sh.mass, mine, (key >> shift) & ((1u << bits) - 1), fs_mass(four[e]));
          }
        }
      }
      __syncthreads();
      fs_scan<MODE>(sh.count, sh.mass, 1 << bits, target, base, sh);
    }
    const unsigned bin = sh.found[0];
    c.above += sh.found[1];
    c.mass_above += sh.mass[FS_BINS];
    prefix = (prefix << bits) | bin;
    fixed_bits += bits;
    if (level == 2) c.equal = sh.count[bin];
    __syncthreads();
  }
  c.key = prefix;
  return c;
}

// rows_index (or null: row b is block b) picks the rows of `logits` that are sampled here; the
// per-row options are indexed by the row.  top_k <= 0 or >= vocab, top_p >= 1 and min_p <= 0
// switch the cut off.  `stored` holds one row of `vocab` floats per block.
__global__ void __launch_bounds__(FS_THREADS)
sample_filtered_kernel(const float* __restrict__ logits, int vocab, long long stride, const int* __restrict__ rows_index,
                       const float* __restrict__ temperature, const int* __restrict__ top_k,
                       const float* __restrict__ top_p, const float* __restrict__ min_p,
                       const float* __restrict__ uniform, float* __restrict__ stored, int* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char fs_raw[];
  FsShared& sh = *reinterpret_cast<FsShared*>(fs_raw);
  // grid (blocks per row, rows): the blocks of a row form a thread-block cluster.  Each takes a slice of
  // the vocabulary through the two heavy passes (the maximum; the probabilities and the histogram of
  // their first bits), block 0 adds the histograms up through the cluster's shared memory and goes on alone.
  const int r = rows_index ? rows_index[blockIdx.y] : blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int blocks = gridDim.x, rank = blockIdx.x;
  const float* l = logits + (size_t)r * stride;
  const int pitch = (vocab + 3) & ~3;                 // rows of `stored` start on 16-byte boundaries
  float* p = stored + (size_t)blockIdx.y * pitch;
  const float t = temperature[r];
  const int slice = (pitch + blocks - 1) / blocks;
  const int slice_begin = min(pitch, rank * slice), slice_end = min(pitch, slice_begin + slice);
  // the largest scaled logit
  float best = -INFINITY;
#pragma unroll 8
  for (int i = slice_begin + threadIdx.x; i < min(slice_end, vocab); i += FS_THREADS) best = fmaxf(best, __fdiv_rn(l[i], t));
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, offset));
  if (lane == 0) sh.warp_max[warp] = best;
  for (int b = threadIdx.x; b < FS_BINS; b += FS_THREADS) {
    sh.first_count[b] = 0;
    sh.first_mass[b] = 0;
  }
  __syncthreads();
  best = sh.warp_max[0];
  for (int w = 1; w < FS_THREADS / 32; ++w) best = fmaxf(best, sh.warp_max[w]);
  if (blocks > 1) {
    __syncthreads();
    if (threadIdx.x == 0) sh.slice_max = best;
    srb_cluster_sync();
    for (int b = 0; b < blocks; ++b) best = fmaxf(best, srb_load_peer_shared(&sh.slice_max, b));
  }
  // the probabilities, stored for the passes to come, and the histogram of their first 11 bits
  for (int start = slice_begin; start < slice_end; start += FS_THREADS * FS_BATCH) {
    float raw[FS_BATCH];
#pragma unroll
    for (int j = 0; j < FS_BATCH; ++j) {
      const int i = start + j * FS_THREADS + (int)threadIdx.x;
      raw[j] = i < slice_end && i < vocab ? l[i] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < FS_BATCH; ++j) {
      const int i = start + j * FS_THREADS + (int)threadIdx.x;
      const bool live = i < slice_end && i < vocab;
      const float value = expf(__fdiv_rn(raw[j], t) - best);
      if (i < slice_end) p[i] = live ? value : -1.f;
      fs_add(sh.first_count, sh.first_mass, live, __float_as_uint(value) >> 21, fs_mass(value));
    }
  }
  if (blocks > 1) {
    srb_cluster_sync();                              // every block's histogram and slice of `stored` are complete
    if (rank == 0) {
      for (int b = threadIdx.x; b < FS_BINS; b += FS_THREADS) {
        unsigned c = sh.first_count[b];
        u64 m = sh.first_mass[b];
        for (int other = 1; other < blocks; ++other) {
          c += fs_peer_u32(&sh.first_count[b], other);
          m += fs_peer_u64(&sh.first_mass[b], other);
        }
        sh.first_count[b] = c;
        sh.first_mass[b] = m;
      }
    }
    srb_cluster_sync();                              // nobody leaves while its histogram may still be read
    if (rank != 0) return;
  }
  __syncthreads();                                   // the block reads what was written to `stored`

  // a prefix of the sorted order: everything above `key`, and the first `n` of those equal to it
  FsCrossing cut;
  cut.key = 0;
  u64 n = ~0ull;
  bool any_cut = false;
  auto tighten = [&](const FsCrossing& c, u64 ties) {
    if (!any_cut || c.key > cut.key || (c.key == cut.key && ties < n)) {
      cut = c;
      n = ties;
      any_cut = true;
    }
  };
  // top-k, and the mass that top-p is a fraction of
  const int k = top_k[r];
  u64 total;
  if (k > 0 && k < vocab) {
    const FsCrossing c = fs_search<FS_BY_COUNT>(p, vocab, (u64)(k - 1), sh);
    const u64 ties = (u64)k - c.above;               // of the items equal to the k-th, those that make k full
    tighten(c, ties);
    total = c.mass_above + ties * fs_mass(__uint_as_float(c.key));
  } else {
    u64 mine = 0;
    for (int b = threadIdx.x; b < FS_BINS; b += FS_THREADS) mine += sh.first_mass[b];
    total = fs_block_sum(mine, sh.totals);
  }
  // top-p.  Kept: mass before the item < top_p * total.  The last kept item is the one that holds the
  // mass position limit - 1; of the items equal to it, those that start below the limit are kept.
  const float tp = top_p[r];
  if (tp < 1.0f && total > 0) {
    u64 limit = (u64)ceil((double)tp * (double)total);
    if (limit < 1) limit = 1;
    if (limit > total) limit = total;
    const FsCrossing c = fs_search<FS_BY_MASS>(p, vocab, limit - 1, sh);
    const u64 w = fs_mass(__uint_as_float(c.key));
    if (w > 0) tighten(c, (limit - c.mass_above + w - 1) / w);
  }
  // min-p: p_i >= p_0 * min_p, and p_0 = 1
  const float mp = min_p[r];
  if (mp > 0.f) tighten(fs_search<FS_BY_KEY>(p, vocab, (u64)__float_as_uint(1.0f * mp), sh), ~0ull);

  // mass of what is kept, and the pick: the first kept item whose running mass exceeds u * kept
  u64 kept = total;
  if (any_cut) {
    if (n > cut.equal) n = cut.equal;
    kept = cut.mass_above + n * fs_mass(__uint_as_float(cut.key));
  }
  int answer = 0;
  if (kept > 0) {
    u64 target = (u64)((double)uniform[r] * (double)kept);
    if (target >= kept) target = kept - 1;
    const FsCrossing c = fs_search<FS_BY_MASS>(p, vocab, target, sh);
    const u64 w = fs_mass(__uint_as_float(c.key));
    u64 which = w > 0 ? (target - c.mass_above) / w : 0;       // among the items equal to it, in index order
    if (c.equal > 0 && which >= c.equal) which = c.equal - 1;
    // Its index: thread t owns the items t * per .. (t + 1) * per - 1, a scan over the threads' counts of
    // matches finds the thread that holds the wanted one, and it walks its items again.
    if (threadIdx.x == 0) sh.index = 0;
    const int per = ((pitch / 4 + FS_THREADS - 1) / FS_THREADS) * 4;      // a multiple of four: 16-byte loads
    const int begin = min(pitch, (int)threadIdx.x * per), end = min(pitch, begin + per);
    unsigned mine = 0;
#pragma unroll 4
    for (int i = begin; i < end; i += 4) {
      const float4 v = *reinterpret_cast<const float4*>(p + i);
      mine += (__float_as_uint(v.x) == c.key) + (__float_as_uint(v.y) == c.key) + (__float_as_uint(v.z) == c.key) +
              (__float_as_uint(v.w) == c.key);
    }
    unsigned run = mine;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
      const unsigned other = __shfl_up_sync(0xffffffffu, run, offset);
      if (lane >= offset) run += other;
    }
    __syncthreads();
    if (lane == 31) sh.count[warp] = run;
    __syncthreads();
    unsigned before = run - mine;
    for (int w2 = 0; w2 < warp; ++w2) before += sh.count[w2];
    if (mine > 0 && before <= (unsigned)which && (unsigned)which < before + mine) {
      unsigned rank = before;
      for (int i = begin; i < end; ++i) {
        if (__float_as_uint(p[i]) == c.key) {
          if (rank == (unsigned)which) sh.index = i;
          ++rank;
        }
      }
    }
    __syncthreads();
    answer = sh.index;
  }
  if (threadIdx.x == 0) out[r] = answer;
}

// One token for each of the `count` rows named in rows_index (null: rows 0 .. count - 1), into out[row].
// Per-row options are indexed by the row: temperature (> 0), top_k (<= 0: off), top_p (>= 1: off),
// min_p (<= 0: off), uniform in [0, 1).  `scratch` holds count rows of vocab floats, each rounded up to a
// multiple of four.
extern "C" int srb_sample_filtered(const float* logits, int vocab, long long stride, const int* rows_index, int count,
                                   const float* temperature, const int* top_k, const float* top_p, const float* min_p,
                                   const float* uniform, float* scratch, int* out, void* stream) {
  if (count <= 0) return SRB_OK;
  if (vocab <= 0 || stride < vocab) SRB_FAIL("sample_filtered: vocabulary %d and stride %lld do not fit", vocab, stride);
  if (!temperature || !top_k || !top_p || !min_p || !uniform || !out || !scratch)
    SRB_FAIL("sample_filtered: an option array, the scratch memory or the output is missing");
  static bool configured = false;
  if (!configured) {
    SRB_CUDA_CALL(cudaFuncSetAttribute(sample_filtered_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)sizeof(FsShared)));
    configured = true;
  }
  // blocks per row: as many (a power of two, 8 at most) as keep all of them resident at once
  int blocks = 1;
  while (blocks < 8 && count * blocks * 2 <= srb_sm_count()) blocks *= 2;
  if (count > 65535) SRB_FAIL("sample_filtered: %d rows exceed one launch", count);
  SRB_CUDA_CALL(srb_launch_clustered(sample_filtered_kernel, dim3(blocks, count), dim3(FS_THREADS), sizeof(FsShared),
                                     (cudaStream_t)stream, dim3(blocks, 1, 1), logits, vocab, stride, rows_index,
                                     temperature, top_k, top_p, min_p, uniform, scratch, out));
  SRB_LAUNCH_CHECK("sample_filtered");
  return SRB_OK;
}

// ---------------------------------------------------------------------------------------------
// Penalties (model_executor.rs:558-590): a token seen c > 0 times in the request's prompt and output
// has its logit divided by the repetition penalty if positive, multiplied if negative, and then
// lowered by presence + frequency * c.  How often each token was seen is kept on the device, one row
// of `vocab` counts per request with penalties: the prompt is counted once, every sampled token as
// it is chosen, so no token has to come back to the host before the next step is sampled.
__global__ void count_tokens_kernel(int* __restrict__ counts_row, const int* __restrict__ tokens, int n, int vocab) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const int token = tokens[i];
    if (token >= 0 && token < vocab) atomicAdd(&counts_row[token], 1);
  }
}

// grid (blocks over the vocabulary, rows); index[r] < 0: the row has no penalties
__global__ void apply_penalties_kernel(float* __restrict__ logits, long long stride, int vocab,
                                       const int* __restrict__ counts, const int* __restrict__ index,
                                       const float* __restrict__ presence, const float* __restrict__ frequency,
                                       const float* __restrict__ repetition) {
  const int r = blockIdx.y;
  const int table_row = index[r];
  if (table_row < 0) return;
  const int* seen = counts + (size_t)table_row * vocab;
  float* l = logits + (size_t)r * stride;
  const float rep = repetition[r], pres = presence[r], freq = frequency[r];
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < vocab; i += gridDim.x * blockDim.x) {
    const int c = seen[i];
    if (c > 0) {
      float v = l[i];
      if (rep != 1.0f) v = v < 0.f ? v * rep : v / rep;
      l[i] = v - pres - freq * (float)c;
    }
  }
}

__global__ void count_picked_kernel(int* __restrict__ counts, int vocab, const int* __restrict__ index,
                                    const int* __restrict__ picked, int rows) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int table_row = index[r], token = picked[r];
  if (table_row >= 0 && token >= 0 && token < vocab) atomicAdd(&counts[(size_t)table_row * vocab + token], 1);
}

// counts_row: one row of `vocab` ints; tokens: n token ids on the device
extern "C" int srb_count_tokens(int* counts_row, const int* tokens, int n, int vocab, void* stream) {
  if (n <= 0) return SRB_OK;
  const int blocks = (n + 255) / 256;
  count_tokens_kernel<<<blocks > 64 ? 64 : blocks, 256, 0, (cudaStream_t)stream>>>(counts_row, tokens, n, vocab);
  SRB_LAUNCH_CHECK("count_tokens");
  return SRB_OK;
}

// logits [rows, stride] float, changed in place; counts [table rows, vocab]; index, presence, frequency,
// repetition: one entry per row of logits
extern "C" int srb_apply_penalties(float* logits, int rows, int vocab, long long stride, const int* counts,
                                   const int* index, const float* presence, const float* frequency,
                                   const float* repetition, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (vocab <= 0 || stride < vocab) SRB_FAIL("apply_penalties: vocabulary %d and stride %lld do not fit", vocab, stride);
  if (rows > 65535) SRB_FAIL("apply_penalties: %d rows exceed one launch", rows);
  apply_penalties_kernel<<<dim3(16, rows), 256, 0, (cudaStream_t)stream>>>(logits, stride, vocab, counts, index, presence,
                                                                           frequency, repetition);
  SRB_LAUNCH_CHECK("apply_penalties");
  return SRB_OK;
}

extern "C" int srb_count_picked(int* counts, int vocab, const int* index, const int* picked, int rows, void* stream) {
  if (rows <= 0) return SRB_OK;
  count_picked_kernel<<<(rows + 255) / 256, 256, 0, (cudaStream_t)stream>>>(counts, vocab, index, picked, rows);
  SRB_LAUNCH_CHECK("count_picked");
  return SRB_OK;
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
