// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (gabfssilva/mlx-omnia); it exists
// for users of this library who call the compiled kernels directly from C or C++.
//
// Who needs it: a host program that has already handed every free byte of the GPU to a
// pool of its own (an inference server that embeds this library, for instance) has nothing
// left for cudaMalloc to give, and a caller on a latency-critical path cannot accept the
// device-wide synchronisation that cudaMalloc and cudaFree imply. `omnia_attention_decode_tc`
// asks such callers to bring three scratch buffers (partial accumulators, partial softmax statistics
// and a ticket per head group). This variant brings its own: a fixed array that lives in the
// library's device image. The caller still passes every input and the output.
//
// The scratch:
//   * is a file-scope `static __device__` array of OMNIA_STATIC_SCRATCH_BYTES (4 MiB plus a
//     16 KiB ticket area). Every GPU on which this library is loaded holds that much memory
//     from the load of the library until the process exits, whether or not the entry point
//     is ever called. One array exists per compiled (HEAD_DIM, GROUP) variant of the library.
//   * limits the problem size: requests * nq * max_chunks * (HEAD_DIM + 2) floats must fit in
//     4 MiB, and requests * nkv tickets in 16 KiB. A larger call is refused with
//     OMNIA_STATIC_TOO_LARGE and launches nothing; `omnia_attention_static_error()` then
//     returns a sentence with the sizes.
//   * is shared by every call on that GPU and keeps the previous call's contents. The ticket
//     area, which must start at zero, is cleared on the stream before each launch. Two calls
//     that overlap on the same GPU (different streams, or different host threads) use the
//     same scratch at the same time and race: serialise them.
//
// The first call on each device looks the array's device address up
// (cudaGetSymbolAddress, with that device current) and raises the kernel's shared-memory
// limit; later calls on that device only launch. That set-up is done under a lock, so host
// threads may make a device's first call at the same time (their launches still share the
// scratch, as said above). Make that first call before any stream capture begins. No call
// allocates: there is no cudaMalloc, cudaFree or allocating library
// routine on this path.
#pragma once

#include <cuda_runtime.h>

#define OMNIA_STATIC_SCRATCH_FLOATS (1 << 20)   // 4 MiB of partial results
#define OMNIA_STATIC_TICKETS (1 << 12)          // 16 KiB of tickets
#define OMNIA_STATIC_SCRATCH_BYTES (OMNIA_STATIC_SCRATCH_FLOATS * 4 + OMNIA_STATIC_TICKETS * 4)
#define OMNIA_STATIC_TOO_LARGE (-2)             // the call needs more scratch than the array holds
#define OMNIA_STATIC_NO_DEVICE (-3)             // the current device could not be queried

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and meaning as omnia_attention_decode_tc, without part_o, part_ml and tickets.
// Returns 0 when the kernel was launched, a cudaError_t value when CUDA refused something or an
// argument is out of range (requests < 0; nkv, max_chunks, max_pages, num_pages or page_size
// < 1; chunk_keys not a positive multiple of 32; nq != nkv * GROUP), or one of the negative
// codes above. Nothing is launched unless 0 is returned.
int omnia_attention_decode_tc_static(const void* q, const void* pages, const int* block_table,
                                     const int* cu_seqlens, const int* seq_lens, const int* seq_ids,
                                     int requests, int chunk_keys, int max_chunks, const void* gate,
                                     int gate_stride, void* out, int max_pages, int num_pages, int nq,
                                     int nkv, int page_size, int window, float scale, int* err,
                                     cudaStream_t stream);

// The reason for the last non-zero return of the function above on this host thread.
const char* omnia_attention_static_error(void);

#ifdef __cplusplus
}
#endif
