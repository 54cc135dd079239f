// Scatter-gather copy for callers that must not allocate.
//
// This entry point has no counterpart in the original SplitRPC sources; it exists
// for embedders of this library whose threads may not call cudaMalloc: a serving
// thread that runs next to live traffic (cudaMalloc takes a device-wide lock and
// can stall every stream for milliseconds), a process that pre-sized all of its
// GPU memory at start-up and treats any later allocation as a leak, or a host
// that hands this library a stream from another runtime whose allocator it must
// not disturb.  The regular path (sg_copy / the GPU engine) uploads the copy list
// into device memory it allocates; this one keeps the list in a fixed device
// array that is part of the library image.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest copy list one call accepts.  The device array behind it
// (SRPC_NOALLOC_MAX_ITEMS * 24 bytes = 24 KiB) is held by every GPU that loads the
// library until the process exits.
#define SRPC_NOALLOC_MAX_ITEMS 1024

// Copies len[i] bytes from src[i] to dst[i] for i in [0, n) with one kernel launch
// on `stream` (a cudaStream_t; null = the default stream) of the current device.
// The arrays are host arrays; the addresses in them are device-visible addresses
// (device memory, mapped pinned host memory or peer memory).  The call returns
// once the list has been handed to the runtime and the kernel has been queued;
// it does not wait for the copy itself.  The list is uploaded from this thread's
// stack, i.e. from pageable memory, which the runtime stages before returning
// and may do synchronously with the host; the caller's arrays can be reused as
// soon as the call returns.
//
// Nothing is allocated: no cudaMalloc/cudaFree, no allocating library routine.
// The first call on each device looks up the device address of the built-in list
// array (cudaGetSymbolAddress with that device current) and keeps it.
//
// Never call this while `stream` is being captured into a CUDA graph, neither the
// first time nor later: the upload would be recorded as a copy from a stack frame
// that is gone when the graph runs.  The call checks for an active capture and
// refuses (-5) without touching the stream.
//
// All calls on a device share the one list array, and it keeps the previous
// call's list until the next call overwrites it.  Two calls whose GPU work may
// overlap (different streams, or the same stream from two threads) race on it:
// serialise them, e.g. keep all calls on one stream.
//
// Returns 0 on success.  Errors (nothing was launched):
//   -1  n > SRPC_NOALLOC_MAX_ITEMS (split the list and call again)
//   -2  a null array with n > 0, or a zero-length / over-4-GiB item
//   -3  no usable CUDA device, or the set-up lookup failed
//   -4  the list upload or the launch failed (see cudaGetLastError on the caller's runtime)
//   -5  `stream` is being captured into a graph
int srpc_sg_copy_noalloc(const uint64_t* src, const uint64_t* dst, const uint64_t* len, uint32_t n, void* stream);

#ifdef __cplusplus
}
#endif
