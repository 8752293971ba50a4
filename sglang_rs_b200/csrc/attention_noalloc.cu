// The allocation-free entry point of the split-key paged attention (see attention_noalloc.h
// for who needs it and for its limits).  The kernels are the ones srb_paged_attention
// launches; only the home of the scratch differs: a file-scope device array.
#include "attention_noalloc.h"

#include "attention_kernels.cuh"

SRB_DEFINE_LAST_ERROR()

#define SRB_NOALLOC_MAX_DEVICES 64

// In host code this name is only a handle for the runtime, not an address a kernel can
// use; the device address is asked for once per device below.
static __device__ __align__(256) float srb_noalloc_scratch[SRB_NOALLOC_SCRATCH_FLOATS];

static float* scratch_address[SRB_NOALLOC_MAX_DEVICES];   // per device, filled at its first call

extern "C" int srb_noalloc_scratch_floats(void) { return SRB_NOALLOC_SCRATCH_FLOATS; }

extern "C" int srb_paged_attention_noalloc(const void* q, const void* k_pool, const void* v_pool, void* out,
                                           const int* positions, const int* row_request,
                                           const int* block_table, int table_stride, int rows, int n_q, int n_kv,
                                           int head_dim, int page_size, int num_pages, int window, int split_size,
                                           int max_splits, float scale, int* error_word, int dtype,
                                           void* stream) {
  if (rows <= 0) return SRB_OK;
  if (split_size <= 0 || max_splits <= 0)
    SRB_FAIL("paged_attention_noalloc: split_size and max_splits must be positive (this entry point is the "
             "split run; an unsplit run needs no scratch, use srb_paged_attention)");
  if (n_q <= 0 || head_dim <= 0) SRB_FAIL("paged_attention_noalloc: head count and head_dim must be positive");
  const long long slots = (long long)rows * n_q * max_splits;
  const long long need = slots * head_dim + slots * 2;
  if (need > SRB_NOALLOC_SCRATCH_FLOATS)
    SRB_FAIL("paged_attention_noalloc: rows %d x heads %d x splits %d x (head_dim %d + 2) = %lld floats of "
             "scratch exceed the built-in %d; use srb_paged_attention with scratch of your own",
             rows, n_q, max_splits, head_dim, need, SRB_NOALLOC_SCRATCH_FLOATS);
  int device = -1;
  SRB_CUDA_CALL(cudaGetDevice(&device));
  if (device < 0 || device >= SRB_NOALLOC_MAX_DEVICES)
    SRB_FAIL("paged_attention_noalloc: device index %d is outside 0..%d", device, SRB_NOALLOC_MAX_DEVICES - 1);
  if (!scratch_address[device]) {
    float* address = nullptr;
    SRB_CUDA_CALL(cudaGetSymbolAddress((void**)&address, srb_noalloc_scratch));
    if (!address) SRB_FAIL("paged_attention_noalloc: the scratch array has no address on device %d", device);
    scratch_address[device] = address;
  }
  float* part_acc = scratch_address[device];
  float* part_ml = part_acc + slots * head_dim;          // 256-byte alignment is not needed for 4-byte stores
  return paged_attention_dispatch(q, k_pool, v_pool, out, part_acc, part_ml, positions, row_request, block_table,
                                  table_stride, rows, n_q, n_kv, head_dim, page_size, num_pages, window, split_size,
                                  max_splits, scale, error_word, dtype, stream);
}
