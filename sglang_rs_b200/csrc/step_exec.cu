// The launch sequence of a whole model step behind one call.
//
// The parts of a model (norm, attention, gated feed-forward, their arrangement in a block) hand over
// records of their constants and weight pointers once, when the model is loaded (step_exec.h).  A step then
// is one call: sx_run walks the model's program and launches every kernel of every layer call from the
// step's index arrays, with the same choices of kernel, of key splits and of K splits that the Python face
// makes when it launches a part at a time.  The reference does a layer in one native call too
// (crates/sglang-srt/src/cuda_dense_decoder.rs:295-489); here the whole step is one, so the host's cost of a
// step is that of its launches and no longer that of an interpreter between them.
//
// The kernels live in libraries of their own (one per .cu file); this library receives their entry points as
// a table of function pointers (sx_set_kernels), so nothing is compiled twice.  Matrix products with more
// rows than this package's few-token kernel takes go to cuBLAS (cublasGemmEx, 32-bit accumulation), which
// is the call the reference makes for every projection (crates/sglang-kernel/src/cublas.rs:383-410); the
// library is looked up in the process (torch has loaded it) and never linked.
//
// The heuristics that are functions of the shape (K splits of a few-token product, blocks per row of the
// decode attention) are defined here and nowhere else; the Python face calls them through this library.
#include "step_exec.h"

#include "common.cuh"

#include <cublas_v2.h>
#include <dlfcn.h>

#include <algorithm>
#include <mutex>

SRB_DEFINE_LAST_ERROR()

// ---------------------------------------------------------------------------------------------- heuristics
extern "C" int sx_gemm_splits(int tokens, int features, int k, int sms, int own_gemm_max_tokens) {
  // Blocks of 128 weight rows alone cannot occupy the SMs when there are few of them, so K is cut until about
  // two blocks per SM exist (two fit), each with at least 8 blocks of K.
  if (tokens > own_gemm_max_tokens) return 1;
  const int tiles = (features + 127) / 128;
  const int k_blocks = (k + 63) / 64;
  const int splits = std::max(1, std::min(2 * sms / std::max(tiles, 1), k_blocks / 8));
  if (splits <= 1) return 1;
  const int per_split = (k_blocks + splits - 1) / splits;
  return (k_blocks + per_split - 1) / per_split;
}

#define SX_DECODE_BLOCKS_PER_SM 3
#define SX_DECODE_MAX_SPLITS 64
#define SX_DECODE_MIN_UNITS 2            // a block walks at least this many 64-key units
#define SX_DECODE_BLOCK_OVERHEAD_UNITS 3 // what a block costs beside its keys (set-up, q, the merge), in units
#define SX_DECODE_GLOBAL_MERGE_UNITS 3   // more than a cluster's worth of blocks merge through global memory
#define SX_DECODE_CLUSTER_SPLITS 8

extern "C" int sx_decode_splits(int rows, int n_kv, int max_keys, int sms) {
  // Blocks per (row, kv head).  Without max_keys (< 0): as many as make about three blocks per SM.  With it,
  // the count that makes the step shortest under a simple model: the blocks run in waves of three per SM, and
  // a wave lasts as long as one block's share of the keys plus a fixed cost.
  const long long base = std::max(1LL, (long long)rows * n_kv);
  const long long target = (long long)SX_DECODE_BLOCKS_PER_SM * sms;
  if (max_keys < 0) return (int)std::max(1LL, std::min<long long>(SX_DECODE_MAX_SPLITS, target / base));
  const int units = std::max(1, (max_keys + 63) / 64);
  const int cap = std::max(1, std::min(SX_DECODE_MAX_SPLITS, units / SX_DECODE_MIN_UNITS));
  int best = 1;
  long long best_cost = -1;
  for (int splits = 1; splits <= cap; ++splits) {
    const long long waves = (base * splits + target - 1) / target;
    const long long cost = waves * ((units + splits - 1) / splits + SX_DECODE_BLOCK_OVERHEAD_UNITS) +
                           (splits > SX_DECODE_CLUSTER_SPLITS ? SX_DECODE_GLOBAL_MERGE_UNITS : 0);
    if (best_cost < 0 || cost < best_cost) {
      best = splits;
      best_cost = cost;
    }
  }
  return best;
}

extern "C" int sx_decode_splits_bound(int max_keys) {
  return std::max(1, std::min(SX_DECODE_MAX_SPLITS, ((max_keys + 63) / 64) / SX_DECODE_MIN_UNITS));
}

extern "C" int sx_decode_max_splits() { return SX_DECODE_MAX_SPLITS; }

// ---------------------------------------------------------------------------------------------- kernels
static SxKernels kernels;
static bool kernels_set = false;

extern "C" void sx_set_kernels(const SxKernels* table) {
  kernels = *table;
  kernels_set = true;
}

// A kernel library failed: its message becomes this library's.
#define SX_KERNEL(slot, call)                                                                        \
  do {                                                                                               \
    if (!kernels.slot) SRB_FAIL("step_exec: the kernel library of `" #slot "` was not handed over");  \
    const int sx_status = kernels.slot call;                                                         \
    ++launches;                                                                                      \
    if (sx_status != 0) {                                                                            \
      const char* text = kernels.slot##_error ? kernels.slot##_error() : "";                         \
      snprintf(srb_error_buffer, sizeof(srb_error_buffer), "%s", text && *text ? text : #slot " failed"); \
      return sx_status;                                                                              \
    }                                                                                                \
  } while (0)

// ---------------------------------------------------------------------------------------------- cuBLAS
struct Blas {
  void* library = nullptr;
  cublasStatus_t (*create)(cublasHandle_t*) = nullptr;
  cublasStatus_t (*set_stream)(cublasHandle_t, cudaStream_t) = nullptr;
  cublasStatus_t (*set_workspace)(cublasHandle_t, void*, size_t) = nullptr;
  cublasStatus_t (*set_math_mode)(cublasHandle_t, cublasMath_t) = nullptr;
  cublasStatus_t (*gemm_ex)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void*, const void*,
                            cudaDataType, int, const void*, cudaDataType, int, const void*, void*, cudaDataType, int,
                            cublasComputeType_t, cublasGemmAlgo_t) = nullptr;
  cublasHandle_t handle[64] = {};
  void* workspace[64] = {};
  size_t workspace_bytes[64] = {};
};
static Blas blas;
static std::mutex blas_mutex;

// `path`: the cuBLAS library that the process has loaded already (or a name for the loader to find).
extern "C" int sx_load_cublas(const char* path) {
  std::lock_guard<std::mutex> guard(blas_mutex);
  if (blas.library) return SRB_OK;
  void* library = dlopen(path && *path ? path : "libcublas.so.12", RTLD_NOW | RTLD_GLOBAL);
  if (!library) SRB_FAIL("step_exec: cuBLAS could not be opened (%s): %s", path ? path : "libcublas.so.12", dlerror());
  blas.create = (decltype(blas.create))dlsym(library, "cublasCreate_v2");
  blas.set_stream = (decltype(blas.set_stream))dlsym(library, "cublasSetStream_v2");
  blas.set_workspace = (decltype(blas.set_workspace))dlsym(library, "cublasSetWorkspace_v2");
  blas.set_math_mode = (decltype(blas.set_math_mode))dlsym(library, "cublasSetMathMode");
  blas.gemm_ex = (decltype(blas.gemm_ex))dlsym(library, "cublasGemmEx");
  if (!blas.create || !blas.set_stream || !blas.set_workspace || !blas.set_math_mode || !blas.gemm_ex)
    SRB_FAIL("step_exec: the cuBLAS library lacks an entry point this engine calls");
  blas.library = library;
  return SRB_OK;
}

// The library's scratch memory on the current device: given by the caller (who keeps it alive), so that
// cuBLAS allocates nothing of its own, which it may not do while a stream is captured into a graph.
extern "C" int sx_set_cublas_workspace(void* memory, long long bytes) {
  int device = 0;
  SRB_CUDA_CALL(cudaGetDevice(&device));
  if (device < 0 || device >= 64) SRB_FAIL("step_exec: device index %d is outside 0..63", device);
  std::lock_guard<std::mutex> guard(blas_mutex);
  blas.workspace[device] = memory;
  blas.workspace_bytes[device] = (size_t)bytes;
  if (blas.handle[device] && blas.set_workspace(blas.handle[device], memory, (size_t)bytes) != CUBLAS_STATUS_SUCCESS)
    SRB_FAIL("step_exec: cuBLAS refused the workspace");
  return SRB_OK;
}

static int blas_handle(cublasHandle_t* out, int* device_out) {
  int device = 0;
  SRB_CUDA_CALL(cudaGetDevice(&device));
  if (device < 0 || device >= 64) SRB_FAIL("step_exec: device index %d is outside 0..63", device);
  if (!blas.library) SRB_FAIL("step_exec: cuBLAS was not loaded (sx_load_cublas)");
  if (!blas.handle[device]) {
    std::lock_guard<std::mutex> guard(blas_mutex);
    if (!blas.handle[device]) {
      cublasHandle_t handle = nullptr;
      if (blas.create(&handle) != CUBLAS_STATUS_SUCCESS) SRB_FAIL("step_exec: cublasCreate failed");
      // every product accumulates in 32 bits to the end: no partial sums of a split along K in bfloat16
      blas.set_math_mode(handle, (cublasMath_t)(CUBLAS_DEFAULT_MATH | CUBLAS_MATH_DISALLOW_REDUCED_PRECISION_REDUCTION));
      if (blas.workspace[device]) blas.set_workspace(handle, blas.workspace[device], blas.workspace_bytes[device]);
      blas.handle[device] = handle;
    }
  }
  *out = blas.handle[device];
  *device_out = device;
  return SRB_OK;
}

// y[m, n] = x[m, k] w[n, k]^T, bfloat16 operands, 32-bit accumulation; y bfloat16 or float.
static int blas_product(const void* x, const void* w, void* y, int m, int n, int k, int ldx, int ldw, int ldy, bool y_float,
                        cudaStream_t stream) {
  cublasHandle_t handle;
  int device = 0;
  const int status = blas_handle(&handle, &device);
  if (status != SRB_OK) return status;
  if (blas.set_stream(handle, stream) != CUBLAS_STATUS_SUCCESS) SRB_FAIL("step_exec: cublasSetStream failed");
  // setting the stream puts the library back on its own workspace pool: this package's is given again
  if (blas.workspace[device] &&
      blas.set_workspace(handle, blas.workspace[device], blas.workspace_bytes[device]) != CUBLAS_STATUS_SUCCESS)
    SRB_FAIL("step_exec: cuBLAS refused the workspace");
  const float one = 1.0f, zero = 0.0f;
  // row-major y = x w^T is column-major y^T = w x^T: A = w (k x n stored, transposed), B = x (k x m stored)
  const cublasStatus_t result =
      blas.gemm_ex(handle, CUBLAS_OP_T, CUBLAS_OP_N, n, m, k, &one, w, CUDA_R_16BF, ldw, x, CUDA_R_16BF, ldx, &zero, y,
                   y_float ? CUDA_R_32F : CUDA_R_16BF, ldy, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
  if (result != CUBLAS_STATUS_SUCCESS) SRB_FAIL("step_exec: cublasGemmEx failed with status %d for %d x %d x %d", (int)result, m, n, k);
  return SRB_OK;
}

// A product from outside a step (the Python face's products of many rows may use it instead of torch's call).
extern "C" int sx_cublas_product(const void* x, const void* w, void* y, int m, int n, int k, int ldx, int ldw, int ldy,
                                 int y_float, void* stream) {
  return blas_product(x, w, y, m, n, k, ldx, ldw, ldy, y_float != 0, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------- workspace
static inline long long aligned(long long bytes) { return (bytes + 255) / 256 * 256; }

struct Layout {
  long long residual, normed, qkv, q, attended, delta, activation, gate_up, final_normed, rope_table, total;
};

// From this many rows on the rows' cosines and sines are computed once per step (and per table of frequencies)
// and handed to the rope kernel for many rows; fewer rows compute them inside the kernel, under the tail of
// the kernel ahead.
#define SX_ROPE_TABLE_MIN_ROWS 256

static long long product_bytes(const SxStep& step, const SxLinear& linear, int rows, int element, bool partial_ok) {
  long long bytes = (long long)rows * linear.out_features * element;
  if (element == 2 && partial_ok && rows <= step.own_gemm_max_tokens && linear.in_features % 8 == 0) {
    const int splits = sx_gemm_splits(rows, linear.out_features, linear.in_features, step.sms, step.own_gemm_max_tokens);
    if (splits > 1) bytes = std::max(bytes, (long long)splits * rows * linear.out_features * 4);
  }
  return bytes;
}

static Layout layout_of(const SxModel& model, const SxStep& step) {
  const int rows = step.rows, element = model.dtype == SRB_DTYPE_F32 ? 4 : 2;
  long long qkv = 0, q = 0, delta = 0, activation = 0, gate_up = 0, rope_table = 0;
  for (int b = 0; b < model.num_blocks; ++b) {
    const SxBlock& block = model.blocks[b];
    if (rows >= SX_ROPE_TABLE_MIN_ROWS && block.mixer.inv_freq && block.mixer.head_dim == 128)
      rope_table = std::max(rope_table, (long long)rows * block.mixer.rotary_dim * 4);
    qkv = std::max(qkv, product_bytes(step, block.mixer.qkv, rows, element, true));
    q = std::max(q, (long long)rows * block.mixer.n_q * block.mixer.head_dim * element);
    delta = std::max(delta, product_bytes(step, block.mixer.o, rows, element, true));
    delta = std::max(delta, product_bytes(step, block.feed_forward.down, rows, element, true));
    activation = std::max(activation, (long long)rows * block.feed_forward.inner * element);
    gate_up = std::max(gate_up, (long long)rows * block.feed_forward.gate_up.out_features * element);
  }
  Layout l;
  long long at = 0;
  auto take = [&](long long bytes) { const long long here = at; at += aligned(bytes); return here; };
  l.residual = take((long long)rows * model.hidden * 4);
  l.normed = take((long long)rows * model.hidden * element);
  l.qkv = take(qkv);
  l.q = take(q);
  l.attended = take(q);
  l.delta = take(delta);
  l.activation = take(activation);
  l.gate_up = take(gate_up);
  l.final_normed = take((long long)std::max(step.num_wanted, 1) * model.hidden * element);
  l.rope_table = take(rope_table);
  l.total = at;
  return l;
}

extern "C" long long sx_workspace_bytes(const SxModel* model, const SxStep* step) { return layout_of(*model, *step).total; }

// ---------------------------------------------------------------------------------------------- the parts
struct Produced {          // what a product left: one tensor of the compute type, or float partial sums
  void* whole = nullptr;
  float* parts = nullptr;
  int num_parts = 0;
  long long part_stride = 0;
};

struct Run {
  const SxModel& model;
  const SxStep& step;
  cudaStream_t stream;
  int launches = 0;
  const float* table_of = nullptr;       // the frequencies whose table of cosines and sines the workspace holds
  int table_width = 0;
  int element() const { return model.dtype == SRB_DTYPE_F32 ? 4 : 2; }

  bool skipped(int bit) const { return (step.skip & bit) != 0; }

  // y = x w^T (+ bias) into `out` (room for partial sums included when partial_ok)
  int linear(const void* x, int rows, const SxLinear& l, void* out, bool out_float, bool partial_ok, Produced* produced,
             int skip_bit) {
    const int m = rows, n = l.out_features, k = l.in_features;
    *produced = Produced();
    produced->whole = out;
    if (skipped(skip_bit)) return SRB_OK;                      // a measurement leaves this product out
    if (model.dtype == SRB_DTYPE_F32) {
      SX_KERNEL(gemm_f32, ((const float*)x, (const float*)l.weight, l.bias, (float*)out, m, n, k, k, k, n, stream));
      return SRB_OK;
    }
    if (m <= step.own_gemm_max_tokens && k % 8 == 0) {
      const int splits = partial_ok ? sx_gemm_splits(m, n, k, step.sms, step.own_gemm_max_tokens) : 1;
      if (splits > 1) {
        SX_KERNEL(gemm_bf16, (x, l.weight, out, m, n, k, k, k, n, n, 0, SX_GEMM_PARTIAL, splits, 0, step.error_word, stream));
        if (l.bias) SX_KERNEL(add_bias, (out, l.bias, m, n, SRB_DTYPE_F32, stream));      // onto the first partial sum
        produced->whole = nullptr;
        produced->parts = (float*)out;
        produced->num_parts = splits;
        produced->part_stride = (long long)m * n;
        return SRB_OK;
      }
      SX_KERNEL(gemm_bf16, (x, l.weight, out, m, n, k, k, k, n, n, 0, out_float ? SX_GEMM_F32 : SX_GEMM_BF16, 1, 0,
                            step.error_word, stream));
    } else {
      const int status = blas_product(x, l.weight, out, m, n, k, k, k, n, out_float, stream);
      if (status != SRB_OK) return status;
      ++launches;
    }
    if (l.bias) SX_KERNEL(add_bias, (out, l.bias, m, n, out_float ? SRB_DTYPE_F32 : model.dtype, stream));
    return SRB_OK;
  }

  int add_norm(float* residual, const Produced* delta, const SxNorm& norm, void* out, const int* row_index, int rows,
               bool write_residual) {
    if (skipped(SX_SKIP_NORM)) return SRB_OK;
    SX_KERNEL(add_rmsnorm, (residual, delta ? delta->whole : nullptr, delta ? delta->parts : nullptr,
                            delta ? delta->num_parts : 0, delta ? delta->part_stride : 0, norm.weight, out, row_index, rows,
                            norm.width, norm.eps, write_residual ? 1 : 0, model.dtype, stream));
    return SRB_OK;
  }

  int attention(const SxAttention& a, const SxCall& call, const void* x, char* base, const Layout& l, Produced* produced) {
    const int rows = step.rows;
    if (call.group < 0 || call.group >= step.num_groups) SRB_FAIL("step_exec: a layer call names cache group %d", call.group);
    const SxGroup& group = step.groups[call.group];
    Produced qkv;
    int status = linear(x, rows, a.qkv, base + l.qkv, false, true, &qkv, SX_SKIP_QKV);
    if (status != SRB_OK) return status;
    void* q = base + l.q;
    void* out = base + l.attended;
    const long long width = (long long)a.qkv.out_features;
    const float* table = nullptr;
    // (only the kernel for many rows of 128-wide heads rotated whole, in half-split pairs, reads the table)
    if (rows >= SX_ROPE_TABLE_MIN_ROWS && a.inv_freq && kernels.rope_table && a.head_dim == 128 && a.rotary_dim == 128 &&
        !a.interleaved) {
      // every layer of a model usually turns by the same frequencies: the table is made for the first of them
      table = (const float*)(base + l.rope_table);
      if (table_of != a.inv_freq || table_width != a.rotary_dim) {
        SX_KERNEL(rope_table, (step.positions, a.inv_freq, nullptr, rows, a.rotary_dim, (float*)(base + l.rope_table), stream));
        table_of = a.inv_freq;
        table_width = a.rotary_dim;
      }
    }
    if (!skipped(SX_SKIP_ROPE))
    SX_KERNEL(qk_norm_rope_kv,
              (qkv.whole, qkv.parts, qkv.num_parts, qkv.part_stride, (int)width, q, call.writable ? call.k_pool : nullptr,
               call.writable ? call.v_pool : nullptr, step.positions, call.writable ? group.slots : nullptr, a.q_norm, a.k_norm,
               a.qk_eps, a.inv_freq, nullptr, table, a.inv_freq ? a.rotary_dim : 0, a.interleaved, rows, a.n_q, a.n_kv, a.head_dim,
               call.writable ? call.page_size : 1, call.writable ? call.num_pages : 1, step.error_word, model.dtype, stream));
    const bool bf16 = model.dtype == SRB_DTYPE_BF16;
    const bool heads_ok = a.n_kv > 0 && a.n_q % a.n_kv == 0 && (a.head_dim == 64 || a.head_dim == 128);
    const bool tc_takes = bf16 && heads_ok && call.page_size >= 8 && call.page_size % 8 == 0 && 64 % call.page_size == 0;
    const bool tiled_takes = bf16 && heads_ok;
    const bool decode_takes = bf16 && heads_ok && a.n_q / a.n_kv <= 16;
    const long long row_bytes = (long long)a.n_q * a.head_dim * element();
    for (int i = 0; i < group.num_launches; ++i) {
      const SxLaunch& launch = group.launches[i];
      const int count = launch.end - launch.begin;
      if (count <= 0 || skipped(SX_SKIP_ATTENTION)) continue;
      if (launch.wide_tiles && tc_takes) {
        SX_KERNEL(prefill_attention_tc, (q, call.k_pool, call.v_pool, out, launch.wide_tiles, launch.num_wide_tiles, rows,
                                         group.block_table, group.table_stride, a.n_q, a.n_kv, a.head_dim, call.page_size,
                                         call.num_pages, a.window, a.scale, step.error_word, stream));
        continue;
      }
      if (launch.tiles && tiled_takes) {
        SX_KERNEL(prefill_attention, (q, call.k_pool, call.v_pool, out, launch.tiles, launch.num_tiles, group.block_table,
                                      group.table_stride, a.n_q, a.n_kv, a.head_dim, call.page_size, call.num_pages, a.window,
                                      a.scale, step.error_word, stream));
        continue;
      }
      const char* q_rows = (const char*)q + launch.begin * row_bytes;
      char* out_rows = (char*)out + launch.begin * row_bytes;
      const long long per_split = (long long)count * a.n_q * a.head_dim;
      if (!launch.tiles && launch.split_size && group.counters && group.num_counters >= count * a.n_kv && decode_takes) {
        // never more blocks than the scratch memory holds partial results for
        long long splits = sx_decode_splits(count, a.n_kv, launch.max_keys, step.sms);
        splits = std::min(splits, group.scratch_acc_floats / per_split);
        splits = std::min(splits, group.scratch_ml_floats / ((long long)count * a.n_q * 2));
        splits = std::max(splits, 1LL);
        if (group.scratch_acc_floats < per_split * splits) SRB_FAIL("step_exec: the split scratch is too small for the decode attention");
        SX_KERNEL(decode_attention, (q_rows, call.k_pool, call.v_pool, out_rows, group.scratch_acc, group.scratch_ml,
                                     group.counters, step.positions + launch.begin, step.row_request + launch.begin,
                                     group.block_table, group.table_stride, count, a.n_q, a.n_kv, a.head_dim, call.page_size,
                                     call.num_pages, a.window, (int)splits, a.scale, step.error_word, stream));
        continue;
      }
      if (launch.split_size && (group.scratch_acc_floats < per_split * launch.max_splits ||
                                group.scratch_ml_floats < (long long)count * a.n_q * 2 * launch.max_splits))
        SRB_FAIL("step_exec: the split scratch is too small for this split run");
      SX_KERNEL(paged_attention, (q_rows, call.k_pool, call.v_pool, out_rows, group.scratch_acc, group.scratch_ml,
                                  step.positions + launch.begin, step.row_request + launch.begin, group.block_table,
                                  group.table_stride, count, a.n_q, a.n_kv, a.head_dim, call.page_size, call.num_pages, a.window,
                                  launch.split_size, launch.max_splits, a.scale, step.error_word, model.dtype, stream));
      if (launch.split_size) ++launches;                       // the merge of the splits is a launch of its own
    }
    return linear(out, rows, a.o, base + l.delta, false, true, produced, SX_SKIP_O);
  }

  int gated_mlp(const SxGatedMlp& f, const void* x, char* base, const Layout& l, Produced* produced) {
    const int rows = step.rows, k = f.gate_up.in_features;
    void* act = base + l.activation;
    const bool bf16 = model.dtype == SRB_DTYPE_BF16;
    if (skipped(SX_SKIP_GATE_UP)) {
    } else if (bf16 && rows <= step.own_gemm_max_tokens && k % 8 == 0) {
      SX_KERNEL(gemm_bf16, (x, f.gate_up.weight, act, rows, f.inner, k, k, k, f.inner, f.gate_up.out_features, f.inner,
                            SX_GEMM_GATED, 1, f.activation, step.error_word, stream));
    } else if (bf16 && f.gate_up.out_features == 2 * f.inner && rows >= step.pair_gemm_min_tokens && f.inner % 8 == 0 && k % 8 == 0) {
      SX_KERNEL(gemm_bf16_pair, (x, f.gate_up.weight, act, rows, f.inner, k, k, k, f.inner, f.gate_up.out_features, f.inner,
                                 SX_GEMM_GATED, f.activation, step.error_word, stream));
    } else {
      Produced both;
      const int status = linear(x, rows, f.gate_up, base + l.gate_up, false, false, &both, 0);
      if (status != SRB_OK) return status;
      SX_KERNEL(gated_mul, (both.whole, act, rows, f.inner, f.activation, model.dtype, stream));
    }
    return linear(act, rows, f.down, base + l.delta, false, true, produced, SX_SKIP_DOWN);
  }
};

// Runs the rows of `step` through `model`; logits of the wanted rows go to step->logits (float [wanted, vocab]).
// Returns the number of kernels launched, or a negative status with the text in srb_last_error().
extern "C" int sx_run(const SxModel* model_pointer, const SxStep* step_pointer) {
  if (!kernels_set) SRB_FAIL("step_exec: the kernels were not handed over (sx_set_kernels)");
  const SxModel& model = *model_pointer;
  const SxStep& step = *step_pointer;
  if (step.rows <= 0) return 0;
  const Layout l = layout_of(model, step);
  if (!step.workspace || step.workspace_bytes < l.total)
    SRB_FAIL("step_exec: the workspace holds %lld bytes, the step needs %lld", step.workspace_bytes, l.total);
  if (((uintptr_t)step.workspace) & 255) SRB_FAIL("step_exec: the workspace must be 256-byte aligned");
  char* base = (char*)step.workspace;
  Run run{model, step, (cudaStream_t)step.stream};
  int& launches = run.launches;
  cudaStream_t stream = run.stream;
  float* residual = (float*)(base + l.residual);
  SX_KERNEL(embedding, (step.token_ids, model.embedding, residual, step.rows, model.hidden, model.vocab, step.error_word,
                        model.dtype, stream));
  Produced delta;
  bool have_delta = false;
  for (int c = 0; c < model.num_calls; ++c) {
    const SxCall& call = model.calls[c];
    if (call.block < 0 || call.block >= model.num_blocks) SRB_FAIL("step_exec: call %d names block %d", c, call.block);
    const SxBlock& block = model.blocks[call.block];
    void* normed = base + l.normed;
    int status = run.add_norm(residual, have_delta ? &delta : nullptr, block.input_norm, normed, nullptr, step.rows, true);
    if (status != SRB_OK) return status;
    status = run.attention(block.mixer, call, normed, base, l, &delta);
    if (status != SRB_OK) return status;
    status = run.add_norm(residual, &delta, block.post_norm, normed, nullptr, step.rows, true);
    if (status != SRB_OK) return status;
    status = run.gated_mlp(block.feed_forward, normed, base, l, &delta);
    if (status != SRB_OK) return status;
    have_delta = true;
  }
  if (step.num_wanted > 0) {
    if (!step.logits || !step.logit_rows) SRB_FAIL("step_exec: logits are wanted but there is nowhere to put them");
    void* final_normed = base + l.final_normed;
    int status = run.add_norm(residual, have_delta ? &delta : nullptr, model.final_norm, final_normed, step.logit_rows,
                              step.num_wanted, false);
    if (status != SRB_OK) return status;
    Produced logits;
    status = run.linear(final_normed, step.num_wanted, model.head, step.logits, true, false, &logits, SX_SKIP_HEAD);
    if (status != SRB_OK) return status;
  }
  return run.launches;
}
