// Allocation-free weighted combine.
//
// This entry point has no counterpart in the reference.  It exists for callers that are
// not allowed to allocate device memory at the point where they need the combine:
// a process whose GPU memory is entirely handed to a pool at start-up (any later cudaMalloc
// fails with out-of-memory), or a latency-critical loop where the device-wide
// synchronisation implied by cudaMalloc/cudaFree would stall every stream.
//
// It computes, for caller-provided device buffers,
//     out[i] = post_scale * (self_w * self_in[i] + sum_j src_w[j] * src_in[j][i])
// exactly like Channel::PullCombine does for buffers that sit in a channel arena, but the
// control words the kernel needs (block-arrival counter, per-source completion counters,
// call sequence number) live in a file-scope `static __device__` array instead of a
// cudaMalloc'ed control block.
//
// Limits and rules
//  * at most kNoAllocMaxSources sources; more is rejected with an error message;
//  * numel * element size must be a multiple of 16 and all pointers 16-byte aligned
//    (the kernel moves 16-byte vectors), anything else is rejected;
//  * element types: kF32, kF64, kF16, kBF16 (see ElemType in comm_kernels.h);
//  * the scratch array (kNoAllocScratchBytes = 16640 bytes) is part of the loaded library: every
//    GPU that loads it holds that much memory until the process exits;
//  * the first call on a device resolves the device address of the array
//    (cudaGetSymbolAddress with that device current); make that first call before any
//    stream capture begins;
//  * all calls on one device share the array, which keeps the previous call's contents; each
//    call clears what it needs with a stream-ordered memset.  Two calls that overlap on the
//    GPU (different streams, no ordering between them) race on the array: order them.
//  * the call works on the CURRENT device: the stream must be a stream of the current device (checked), self_in and
//    out must be memory that device can address (plain host memory is rejected), and the scratch array used is the
//    current device's copy.  Source pointers may be peer-mapped memory of other GPUs.  Set the device
//    (cudaSetDevice) before calling, as for any kernel launch.
//  * no cudaMalloc, cudaFree or other allocating routine (PyTorch's included) is called.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define BFB200_NOALLOC_MAX_SOURCES 64
#define BFB200_NOALLOC_SCRATCH_BYTES (256 + 64 * 256)

// Returns 0 on success. On failure returns a non-zero code and, when err != NULL, writes a
// zero-terminated message of at most err_len bytes.
//   self_in, out : device pointers;  src_in: HOST array of n_src device pointers;
//   src_w        : HOST array of n_src weights;  stream: cudaStream_t (NULL = default stream).
__attribute__((visibility("default")))
int bfb200_combine_noalloc(const void* self_in, const void* const* src_in, const double* src_w, int n_src,
                           double self_w, double post_scale, void* out, unsigned long long numel,
                           int elem_type, void* stream, char* err, int err_len);

#ifdef __cplusplus
}
#endif

#ifdef __cplusplus
#include <cuda_runtime.h>
namespace bfb {
// Test helper: copies the control words of the current device's scratch array to the host (a blocking copy; it
// allocates nothing).  After a finished call with n_src sources: block_counter == 0, calls_done == 1 and
// done[j] == 1 for every j < n_src.
cudaError_t NoAllocScratchRead(int n_src, unsigned int* block_counter, unsigned long long* calls_done,
                               unsigned long long* done);
}  // namespace bfb
#endif
