// Split-key decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for embedders of this
// library. mlxone_attention_decode needs scratch memory for the partial results of the key
// splits, and its caller provides it. Some callers cannot: a host that pre-allocated all of
// the device for its own arenas and forbids the allocator afterwards, code that runs inside a
// region where cudaMalloc is illegal or would synchronise the device, a plug-in that is
// handed fixed input and output buffers and nothing else. For them the scratch lives in a
// fixed array in the library's own device image (MLXONE_STATIC_SCRATCH_FLOATS floats, 8 MiB;
// every GPU that loads the library holds one copy until the process exits).
//
// * Same arguments and same result as mlxone_attention_decode, without `partial`. The caller
//   still passes the inputs and the output.
// * It calls no cudaMalloc, cudaFree or allocating library routine. A shape whose partial
//   results need more than MLXONE_STATIC_SCRATCH_FLOATS floats is refused with an error text
//   (mlxone_last_error) and nothing is launched; fewer splits or requests per call fit.
// * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//   that device current) and keeps it. Make this first call before any stream capture begins;
//   a first call that finds its stream capturing is refused with an error text. Devices 0 to 63
//   are served. Calls from several host threads are safe: the address is kept with an atomic
//   store, and threads that look it up at the same time store the same value.
// * All calls on a device share the one array. It keeps what the last call left there; this
//   kernel writes every partial result before it reads it, so nothing has to be cleared. Two
//   calls that overlap on the GPU (different streams, no ordering between them) would write
//   the same scratch and race: order them.
// * The kernel is launched as a programmatic dependent of the kernel before it in the stream
//   (unless dependent launches are switched off). Before it waits for that kernel it reads
//   `positions`, `block_table` and the keys and values of positions before the newest one:
//   a kernel that writes any of these and lets its dependents start early
//   (griddepcontrol.launch_dependents) must not be the one before this call. Kernels that do
//   not use that instruction, and copies, are safe.
#pragma once

#include <cuda_runtime.h>

#define MLXONE_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)

extern "C" __attribute__((visibility("default"))) int mlxone_attention_decode_static(
    const void* q, const void* kv, const int* block_table, int table_width, int page_size,
    int pages, const int* positions, void* out, int requests, int heads, int kv_heads,
    int head_dim, int splits, float scale, int window, cudaStream_t stream);

// Floats of the fixed scratch array (for callers that size their batches by it).
extern "C" __attribute__((visibility("default"))) long long mlxone_attention_decode_static_capacity();
