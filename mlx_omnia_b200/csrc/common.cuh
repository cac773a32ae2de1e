// Shared device helpers for the sm_100a kernels of this package.
//
// Every exported function is `extern "C"`, takes raw device pointers, sizes and
// the CUDA stream to launch on, allocates nothing, and returns the cudaError_t of
// its launch as an int (0 = launched). Element types are chosen by a code:
// 0 = float32, 1 = bfloat16. Reductions, softmax, norms and rotation angles are
// always computed in float32 whatever the element type.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define OMNIA_F32 0
#define OMNIA_BF16 1

// Bits of the device error word (see omnia_error_fetch in elementwise.cu).
#define OMNIA_ERR_TOKEN_ID 1   // a token id outside the embedding table
#define OMNIA_ERR_SLOT 2       // a cache slot outside the page pool
#define OMNIA_ERR_PAGE 4       // a block-table entry outside the page pool was needed
#define OMNIA_ERR_WORK 16      // a work list asks a kernel for what it does not do

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over the block; every thread gets the result. `scratch` holds 33 floats.
// The order of the additions depends only on blockDim, never on the data.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    const int warps = (blockDim.x + 31) >> 5;
    float t = lane < warps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Whether the phase of the mbarrier at shared address `bar` with this parity is complete, without
// waiting. A bounded wait asks this first: a try_wait that finds the phase complete still costs
// the thread some 250 cycles (measured on B200), a test_wait a few dozen.
__device__ __forceinline__ bool omnia_mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Programmatic dependent launch. A kernel launched through launch_pdl may begin while the kernel
// before it in the stream is still running; it must call pdl_wait() before it touches anything an
// earlier kernel wrote (reading weights before that is fine and hides their latency), and calls
// pdl_launch_dependents() to let the kernel after it start its own preamble early. In a kernel
// launched the ordinary way both calls do nothing.
// Rule of this package: a kernel calls pdl_launch_dependents() only after its own pdl_wait(), so
// at most two kernels ever overlap. (Were it called first, a third kernel's block could start on
// an SM where the first kernel still runs, and later find in L1, through a cached load, lines
// that the first kernel's blocks fetched from memory which has since been freed, handed out
// again and rewritten. That was seen as a rare wrong token.)
#ifndef OMNIA_TIMELINE
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#define OMNIA_TRACE_BLOCK(phase) do { } while (0)
#define OMNIA_TRACE_IF(condition, phase) do { } while (0)
#else
// Tracing build (-DOMNIA_TIMELINE): thread 0 of block (0, 0, 0) of every kernel stamps the GPU's
// nanosecond clock when it reaches its wait and when the wait is over, i.e. when the kernel
// before it has finished, tagged with the source line of the call. Each library keeps its own
// marks; omnia_timeline_take hands them to the host and starts afresh. The distance between two
// kernels' second marks is the time the earlier one takes in the stream as it really runs,
// overlaps included, which no profiler that serialises launches shows.
#define OMNIA_TIMELINE_MARKS 65536
static __device__ unsigned long long omnia_marks[3 * OMNIA_TIMELINE_MARKS];
static __device__ unsigned omnia_mark_count;
// A mark: time, tag, and where it was made (block number within the grid, and the SM above bit 32).
__device__ __forceinline__ void timeline_stamp(unsigned tag) {
  unsigned long long now;
  unsigned sm;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
  asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
  const unsigned at = atomicAdd(&omnia_mark_count, 1u);
  const unsigned long long block = blockIdx.x + (unsigned long long)gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z);
  if (at < OMNIA_TIMELINE_MARKS)
    omnia_marks[3 * at] = now, omnia_marks[3 * at + 1] = tag, omnia_marks[3 * at + 2] = block | ((unsigned long long)sm << 32);
}
__device__ __forceinline__ void timeline_mark(unsigned tag) {
  if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) timeline_stamp(tag);
}
// For looking inside one kernel (-DOMNIA_TIMELINE=2): thread 0 of every block stamps (phases 2 to 7).
#if OMNIA_TIMELINE >= 2
#define OMNIA_TRACE_BLOCK(phase) do { if (threadIdx.x == 0) timeline_stamp(8 * __LINE__ + (phase)); } while (0)
#define OMNIA_TRACE_IF(condition, phase) do { if (condition) timeline_stamp(8 * __LINE__ + (phase)); } while (0)
#else
#define OMNIA_TRACE_BLOCK(phase) do { } while (0)
#define OMNIA_TRACE_IF(condition, phase) do { } while (0)
#endif
__device__ __forceinline__ void pdl_wait_at(unsigned line) {
  timeline_mark(8 * line);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  timeline_mark(8 * line + 1);
}
#define pdl_wait() pdl_wait_at(__LINE__)
// -> the number of marks copied: out[3 i] nanoseconds, out[3 i + 1] = 8 * line + phase (0 at the
// wait, 1 after it, 2.. a block trace), out[3 i + 2] = block | sm << 32.
extern "C" int omnia_timeline_take(unsigned long long* out, int capacity) {
  unsigned count = 0;
  if (cudaMemcpyFromSymbol(&count, omnia_mark_count, sizeof count) != cudaSuccess) return -1;
  if (count > OMNIA_TIMELINE_MARKS) count = OMNIA_TIMELINE_MARKS;
  if ((int)count > capacity) count = capacity;
  if (count && cudaMemcpyFromSymbol(out, omnia_marks, 3 * sizeof(unsigned long long) * count) != cudaSuccess) return -1;
  const unsigned zero = 0;
  if (cudaMemcpyToSymbol(omnia_mark_count, &zero, sizeof zero) != cudaSuccess) return -1;
  return (int)count;
}
#endif
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

#define OMNIA_LAUNCH_RESULT() ((int)cudaGetLastError())

// How many SMs the current device has (asked once per device, then remembered). Grid sizes and
// tilings are made from this, never from a number written into the source.
inline int omnia_sm_count() {
  static int counts[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) device = 0;
  if (counts[device] == 0) {
    int count = 0;
    cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
    counts[device] = count > 0 ? count : 1;
  }
  return counts[device];
}

#define OMNIA_DISPATCH_DTYPE(code, ...)                    \
  do {                                                     \
    if ((code) == OMNIA_F32) {                             \
      using T = float;                                     \
      __VA_ARGS__;                                         \
    } else if ((code) == OMNIA_BF16) {                     \
      using T = __nv_bfloat16;                             \
      __VA_ARGS__;                                         \
    } else {                                               \
      return (int)cudaErrorInvalidValue;                   \
    }                                                      \
  } while (0)
