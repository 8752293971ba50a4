// Shared helpers of the sm_100a kernels: the C ABI's status codes, element
// conversion between the storage type and 32-bit, and fixed-order reductions.
//
// Every launcher is `extern "C" int srb_<name>(..., void* stream)` and returns 0 or a
// negative status; `srb_last_error()` of the same library gives the message.  Kernels
// never trap: an index that is out of range sets bits in a device-side error word and
// the access is skipped, as the reference's kernels do
// (crates/sglang-kernel/src/cuda_bf16_kernels.rs:30-35).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define SRB_OK 0
#define SRB_ERR_INVALID (-1)   // a size or option this kernel does not take
#define SRB_ERR_CUDA (-2)      // the CUDA runtime refused the launch

#define SRB_DTYPE_F32 0
#define SRB_DTYPE_BF16 1

// bits of the device-side error word
#define SRB_FLAG_BAD_TOKEN 1
#define SRB_FLAG_BAD_SLOT 2
#define SRB_FLAG_BAD_PAGE 4
#define SRB_FLAG_WAIT_TIMEOUT 8
#define SRB_FLAG_TOO_FEW_SPLITS 16   // a row of a split attention run has more key splits than the launch was given

static thread_local char srb_error_buffer[512] = "";

#define SRB_DEFINE_LAST_ERROR() \
  extern "C" const char* srb_last_error() { return srb_error_buffer; }

#define SRB_FAIL(...)                                                   \
  do {                                                                  \
    snprintf(srb_error_buffer, sizeof(srb_error_buffer), __VA_ARGS__);  \
    return SRB_ERR_INVALID;                                             \
  } while (0)

#define SRB_LAUNCH_CHECK(name)                                                              \
  do {                                                                                      \
    cudaError_t srb_status = cudaGetLastError();                                            \
    if (srb_status != cudaSuccess) {                                                        \
      snprintf(srb_error_buffer, sizeof(srb_error_buffer), "%s: %s", name,                  \
               cudaGetErrorString(srb_status));                                             \
      return SRB_ERR_CUDA;                                                                  \
    }                                                                                       \
  } while (0)

#define SRB_CUDA_CALL(call)                                                                 \
  do {                                                                                      \
    cudaError_t srb_status = (call);                                                        \
    if (srb_status != cudaSuccess) {                                                        \
      snprintf(srb_error_buffer, sizeof(srb_error_buffer), "%s: %s", #call,                 \
               cudaGetErrorString(srb_status));                                             \
      return SRB_ERR_CUDA;                                                                  \
    }                                                                                       \
  } while (0)

__device__ __forceinline__ float srb_to_float(float v) { return v; }
__device__ __forceinline__ float srb_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T srb_from_float(float v);
template <> __device__ __forceinline__ float srb_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 srb_from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// All lanes receive the same sum; the order of additions is fixed by the butterfly.
__device__ __forceinline__ float srb_warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}
__device__ __forceinline__ float srb_warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// Sum over a block of up to 1024 threads; every thread receives the result.  Warp
// partials are added in warp order, so the result does not depend on timing.
__device__ __forceinline__ float srb_block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = srb_warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int w = 0; w < warps; ++w) total += scratch[w];
    scratch[32] = total;
  }
  __syncthreads();
  return scratch[32];
}

// The number of SMs of the current device, asked once per device: launch heuristics size their grids by it.
static inline int srb_sm_count() {
  static int cached[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 1;
  if (cached[device] == 0) {
    int count = 0;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0) return 1;
    cached[device] = count;
  }
  return cached[device];
}

// ---- programmatic dependent launch ------------------------------------------------------
// A kernel launched through srb_launch with the switch on may become resident while the
// kernel before it in the stream is still running: its set-up (barriers, tensor memory,
// loads of weights that no earlier kernel writes) overlaps that kernel's tail.  Such a
// kernel calls srb_grid_dependency_wait() before it reads or writes anything an earlier
// kernel may touch; the call returns once every earlier kernel has completed and its writes
// are visible.  srb_launch_dependents() tells the device that the next kernel may be brought
// in.  Without the launch attribute both calls do nothing.
static int srb_pdl_enabled = 0;

// ---- a timeline of blocks, for builds with -DSRB_TIMELINE only --------------------------------------
// Every block of the kernels that make a decode step writes (time, kind, phase, SM, block) records into a
// buffer that the caller hands to each library: phase 0 when the block starts, 1 when its wait for the kernels
// ahead returns, 2 when it leaves.  From them one reads how far a kernel runs under the one before it.  Without
// the flag the marks compile to nothing.
#ifdef SRB_TIMELINE
static __device__ unsigned long long* srb_timeline_buffer = nullptr;    // [0]: records written; then two words each
static __device__ unsigned long long srb_timeline_capacity = 0;
#define SRB_DEFINE_TIMELINE()                                                                             \
  extern "C" int srb_set_timeline(void* buffer, long long records) {                                      \
    unsigned long long capacity = (unsigned long long)records;                                            \
    if (cudaMemcpyToSymbol(srb_timeline_buffer, &buffer, sizeof(buffer)) != cudaSuccess) return -1;       \
    return cudaMemcpyToSymbol(srb_timeline_capacity, &capacity, sizeof(capacity)) == cudaSuccess ? 0 : -1; \
  }
// The timer is read under a predicate computed from a volatile load of shared memory: the assembler is free to move a
// plain read of the timer up across a barrier or a wait that comes before it (a block's last barrier, measured: every
// warp's "time after the barrier" was the time it had arrived), but not a load of shared memory, nor what depends on it.
__device__ __forceinline__ unsigned long long srb_now() {
  __shared__ unsigned srb_timer_anchor;                    // never written: any value will do
  const unsigned anchor = *reinterpret_cast<volatile unsigned*>(&srb_timer_anchor);
  unsigned long long now;
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.u32 p, %1, 0x9e3779b9;\nmov.u64 %0, 0;\n@p mov.u64 %0, %%globaltimer;\n}\n"
      : "=l"(now) : "r"(anchor) : "memory");
  return now;
}
// a record of a time taken earlier with srb_now() (a kernel that wants several marks close together takes the
// times on the way and writes the records at its end, so that writing them delays nothing it measures)
__device__ __forceinline__ void srb_mark_at(unsigned kind, unsigned phase, unsigned long long now) {
  if (threadIdx.x == 0 && srb_timeline_buffer) {
    unsigned sm;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
    const unsigned long long at = atomicAdd(srb_timeline_buffer, 1ULL);
    if (at < srb_timeline_capacity) {
      const unsigned block = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
      srb_timeline_buffer[1 + 2 * at] = now;
      srb_timeline_buffer[2 + 2 * at] = ((unsigned long long)kind << 56) | ((unsigned long long)phase << 48) |
                                        ((unsigned long long)(sm & 0xffff) << 32) | block;
    }
  }
}
__device__ __forceinline__ void srb_mark(unsigned kind, unsigned phase) { srb_mark_at(kind, phase, srb_now()); }
#else
#define SRB_DEFINE_TIMELINE()
__device__ __forceinline__ unsigned long long srb_now() { return 0; }
__device__ __forceinline__ void srb_mark_at(unsigned, unsigned, unsigned long long) {}
__device__ __forceinline__ void srb_mark(unsigned, unsigned) {}
#endif
#define SRB_MARK_NORM 1
#define SRB_MARK_PRODUCT 2
#define SRB_MARK_ROPE 3
#define SRB_MARK_DECODE_ATTENTION 4
#define SRB_MARK_PREFILL_ATTENTION 5

#define SRB_DEFINE_PDL_SWITCH() \
  extern "C" void srb_set_pdl(int on) { srb_pdl_enabled = on; } \
  SRB_DEFINE_TIMELINE()

__device__ __forceinline__ void srb_grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void srb_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// A cluster dimension > 1 launches thread-block clusters of that shape (the grid is a multiple of it).
template <typename... KernelArgs, typename... Args>
static cudaError_t srb_launch_clustered(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                                        cudaStream_t stream, dim3 cluster, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  unsigned count = 0;
  if (srb_pdl_enabled) {
    attribute[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  if (cluster.x * cluster.y * cluster.z > 1) {
    attribute[count].id = cudaLaunchAttributeClusterDimension;
    attribute[count].val.clusterDim.x = cluster.x;
    attribute[count].val.clusterDim.y = cluster.y;
    attribute[count].val.clusterDim.z = cluster.z;
    ++count;
  }
  config.attrs = attribute;
  config.numAttrs = count;
  return cudaLaunchKernelEx(&config, kernel, KernelArgs(args)...);
}

template <typename... KernelArgs, typename... Args>
static cudaError_t srb_launch(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
  return srb_launch_clustered(kernel, grid, block, smem, stream, dim3(1, 1, 1), args...);
}

// ---- thread-block clusters: rank, barrier, and loads from another block's shared memory ------------
__device__ __forceinline__ unsigned srb_cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// every thread of every block of the cluster arrives; writes to shared memory before it are visible after it
__device__ __forceinline__ void srb_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float srb_load_peer_shared(const float* mine, unsigned rank) {
  unsigned local = (unsigned)__cvta_generic_to_shared(mine), remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}
