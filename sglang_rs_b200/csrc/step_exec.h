// Records that the parts of a model hand to the step executor (step_exec.cu), and the record of a step.
//
// All of them are plain C structures of pointers and numbers; the Python face fills them through ctypes
// (engine/native.py mirrors every field in the same order) and keeps the tensors they point at alive.
// A part owns the contents of its record: which weights, which constants.  The executor owns the order of
// the launches and the scratch memory between them.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// modes of the few-token and the CTA-pair product (the numbers of gemm_bf16.cu)
#define SX_GEMM_BF16 0
#define SX_GEMM_F32 1
#define SX_GEMM_GATED 2
#define SX_GEMM_PARTIAL 3

typedef struct SxLinear {
  const void* weight;          // [out_features, in_features], the compute type, row-major
  const float* bias;           // [out_features] or null
  int out_features, in_features;
} SxLinear;

typedef struct SxNorm {
  const float* weight;         // [width]
  float eps;
  int width;
} SxNorm;

typedef struct SxAttention {
  SxLinear qkv, o;             // q rows, then k rows, then v rows in one matrix; the output projection
  const float* q_norm;         // [head_dim] or null
  const float* k_norm;
  const float* inv_freq;       // [rotary_dim / 2] or null (no rotation)
  float qk_eps, scale;
  int rotary_dim, interleaved, n_q, n_kv, head_dim, window;    // window 0: all keys
} SxAttention;

typedef struct SxGatedMlp {
  SxLinear gate_up, down;      // gate rows stacked over up rows; the down projection
  int inner, activation;       // activation: SRB_ACT_* of activations.cuh
} SxGatedMlp;

// a pre-norm block: h += mixer(norm(h)); h += feed_forward(norm(h))
typedef struct SxBlock {
  SxNorm input_norm;
  SxAttention mixer;
  SxNorm post_norm;
  SxGatedMlp feed_forward;
} SxBlock;

// one entry of the model's program: which block runs, and on which cache
typedef struct SxCall {
  int block, group, writable;  // group: index of the cache group whose block table the call reads
  int page_size, num_pages;
  void* k_pool;                // [pages, n_kv, page_size, head_dim]
  void* v_pool;
} SxCall;

typedef struct SxModel {
  int dtype;                   // SRB_DTYPE_*
  int vocab, hidden;
  const void* embedding;       // [vocab, hidden]
  SxNorm final_norm;
  SxLinear head;
  int num_blocks, num_calls;
  const SxBlock* blocks;
  const SxCall* calls;
} SxModel;

// rows [begin, end) of the step as one attention launch (engine/runner.py AttentionLaunch)
typedef struct SxLaunch {
  int begin, end, split_size, max_splits, max_keys, num_tiles, num_wide_tiles, reserved;
  const int* tiles;            // [num_tiles, 4] or null
  const int* wide_tiles;       // [num_wide_tiles, 4] or null
} SxLaunch;

typedef struct SxGroup {
  const int* block_table;      // [requests, table_stride]
  const int* slots;            // [rows]
  float* scratch_acc;
  float* scratch_ml;
  int* counters;
  long long scratch_acc_floats, scratch_ml_floats;
  int table_stride, num_counters, num_launches, reserved;
  const SxLaunch* launches;
} SxGroup;

#define SX_MAX_GROUPS 4

// Kernels of a step that a measurement may leave out (SxStep.skip): the step then computes nothing of use, but
// its time shows what the kernels left in cost.  Used by `bench.py --mode ablate` only.
#define SX_SKIP_NORM 1
#define SX_SKIP_ROPE 2
#define SX_SKIP_ATTENTION 4
#define SX_SKIP_QKV 8
#define SX_SKIP_O 16
#define SX_SKIP_GATE_UP 32
#define SX_SKIP_DOWN 64
#define SX_SKIP_HEAD 128

typedef struct SxStep {
  int rows, num_wanted, sms, own_gemm_max_tokens, pair_gemm_min_tokens, num_groups;
  int skip, reserved;          // skip: SX_SKIP_* bits, 0 in every step that is meant to compute
  const int* token_ids;        // [rows]
  const int* positions;        // [rows]
  const int* row_request;      // [rows]
  const int* logit_rows;       // [num_wanted] or null
  int* error_word;
  void* workspace;             // sx_workspace_bytes(model, step) bytes, 256-byte aligned
  long long workspace_bytes;
  float* logits;               // [num_wanted, vocab] or null
  void* stream;
  SxGroup groups[SX_MAX_GROUPS];
} SxStep;

// The kernels' entry points, each with the srb_last_error of its library.
typedef const char* (*SxLastError)(void);
typedef struct SxKernels {
  int (*embedding)(const int*, const void*, float*, int, int, int, int*, int, void*);
  SxLastError embedding_error;
  int (*add_rmsnorm)(float*, const void*, const float*, int, long long, const float*, void*, const int*, int, int, float, int,
                     int, void*);
  SxLastError add_rmsnorm_error;
  int (*gated_mul)(const void*, void*, int, int, int, int, void*);
  SxLastError gated_mul_error;
  int (*add_bias)(void*, const float*, int, int, int, void*);
  SxLastError add_bias_error;
  int (*gemm_f32)(const float*, const float*, const float*, float*, int, int, int, int, int, int, void*);
  SxLastError gemm_f32_error;
  int (*gemm_bf16)(const void*, const void*, void*, int, int, int, int, int, int, int, int, int, int, int, int*, void*);
  SxLastError gemm_bf16_error;
  int (*gemm_bf16_pair)(const void*, const void*, void*, int, int, int, int, int, int, int, int, int, int, int*, void*);
  SxLastError gemm_bf16_pair_error;
  int (*qk_norm_rope_kv)(const void*, const float*, int, long long, int, void*, void*, void*, const int*, const int*,
                         const float*, const float*, float, const float*, const float*, const float*, int, int, int, int, int,
                         int, int, int, int*, int, void*);                    // srb_qk_norm_rope_kv_table
  SxLastError qk_norm_rope_kv_error;
  int (*rope_table)(const int*, const float*, const float*, int, int, float*, void*);
  SxLastError rope_table_error;
  int (*paged_attention)(const void*, const void*, const void*, void*, float*, float*, const int*, const int*, const int*, int,
                         int, int, int, int, int, int, int, int, int, float, int*, int, void*);
  SxLastError paged_attention_error;
  int (*decode_attention)(const void*, const void*, const void*, void*, float*, float*, int*, const int*, const int*,
                          const int*, int, int, int, int, int, int, int, int, int, float, int*, void*);
  SxLastError decode_attention_error;
  int (*prefill_attention)(const void*, const void*, const void*, void*, const int*, int, const int*, int, int, int, int, int,
                           int, int, float, int*, void*);
  SxLastError prefill_attention_error;
  int (*prefill_attention_tc)(const void*, const void*, const void*, void*, const int*, int, int, const int*, int, int, int, int,
                              int, int, int, float, int*, void*);
  SxLastError prefill_attention_tc_error;
} SxKernels;

void sx_set_kernels(const SxKernels* table);
int sx_load_cublas(const char* path);
int sx_set_cublas_workspace(void* memory, long long bytes);
int sx_cublas_product(const void* x, const void* w, void* y, int m, int n, int k, int ldx, int ldw, int ldy, int y_float,
                      void* stream);
long long sx_workspace_bytes(const SxModel* model, const SxStep* step);
int sx_run(const SxModel* model, const SxStep* step);

int sx_gemm_splits(int tokens, int features, int k, int sms, int own_gemm_max_tokens);
int sx_decode_splits(int rows, int n_kv, int max_keys, int sms);
int sx_decode_splits_bound(int max_keys);
int sx_decode_max_splits(void);
const char* srb_last_error(void);

#ifdef __cplusplus
}
#endif
