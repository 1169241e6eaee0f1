// C entry points of the decode attention kernels (attention_decode.cu), one library per head size.
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Head size this library was compiled for.
int tlie_decode_attention_head_dim(void);

// Floats of scratch memory tlie_decode_attention needs for this launch shape.
long long tlie_decode_attention_scratch_floats(int requests, int q_heads, int splits);

// Split-KV paged decode attention; the caller provides `scratch` (zero-filled once, then reusable).
int tlie_decode_attention(const void* q, int q_row_stride, void* pages, const int* positions, const int* block_table,
                          int table_stride, void* out, float* scratch, int requests, int q_heads, int kv_heads,
                          int page_size, int window, float scale, int splits, int fuse_rope, const float* inv_freq,
                          int write_cache, cudaStream_t stream);

// The same computation for callers that cannot allocate device memory.
//
// Who that is: code that runs where cudaMalloc is off limits, because the process was handed a fixed memory
// budget by its host (an embedding application, a plugin inside somebody else's runtime), because it sits in a
// latency-critical loop where an allocation may synchronise the device, or because its allocator is owned by a
// framework it must not call into.  Such a caller still owns its inputs and outputs and passes them in; what it
// cannot provide is the kernel's scratch: the per-part partial results and the arrival counters of the split-KV merge.
//
// Here that scratch lives in a file-scope `static __device__` array inside the library.  Every GPU that loads the
// library holds it until the process exits: 16384 counters plus room for 8192 (request, head, part) triples,
// (16384 + 8192 * (HEAD_DIM + 2)) * 4 bytes, about 2.2 MB at head size 64 and 4.3 MB at 128.  A launch shape with
// requests * q_heads * splits > 8192 or requests * kv_heads > 16384 is refused with cudaErrorInvalidValue and
// nothing is launched.  The function calls no cudaMalloc, cudaFree or other allocating routine.
//
// The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
// current); make that first call outside any stream capture.  Each call clears the counters on `stream` before the
// kernel (cudaMemsetAsync), so a call that was cut short cannot poison the next.  All calls on a device share the one
// array and it keeps the last call's contents: two calls that overlap on the GPU (different streams without
// ordering between them) race on it.  Serialise them, or use tlie_decode_attention with separate scratch buffers.
//
// This entry point has no counterpart in the reference, whose decode attention needs no scratch memory.
int tlie_decode_attention_static(const void* q, int q_row_stride, void* pages, const int* positions,
                                 const int* block_table, int table_stride, void* out, int requests, int q_heads,
                                 int kv_heads, int page_size, int window, float scale, int splits, int fuse_rope,
                                 const float* inv_freq, int write_cache, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
