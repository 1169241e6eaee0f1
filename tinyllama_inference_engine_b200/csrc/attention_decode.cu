// Split-KV paged grouped-query attention for decode steps (one query token per request), bfloat16.
//
// Replaces the reference's one-block-per-head decode kernel, which keeps every score in shared
// memory and sums P.V serially (src/cuda/kernels.cu:147-196).  Same mathematics
// (src/operators.cpp:102-146): out = softmax(q.K^T * scale) . V over keys lo..pos, 32-bit softmax.
//
// Decode attention is bound by reading the cache, so the design is about bytes in flight:
//   * one CTA per (request, kv head, split of the key range); the query heads that share the
//     kv head (the group, up to 16) are the rows of one tensor-core tile, so every key and value
//     is read from HBM once per group, not once per head;
//   * the key range of a request is cut into SPLITS parts so that small batches still fill the
//     148 SMs; a second small kernel merges the parts (none is needed when SPLITS == 1);
//   * each of the four warps of a CTA walks its own 32-key tiles with a private multi-stage
//     cp.async pipeline (no block-wide barrier in the loop); rows in shared memory are padded
//     by 16 bytes so that ldmatrix reads are free of bank conflicts for any head size;
//   * q.K^T and P.V run on the tensor cores (mma.sync m16n8k16, bf16 in, 32-bit accumulate):
//     with at most 16 rows per tile the 128-row tcgen05 shapes would be idle weight, and the
//     CUDA cores alone cannot keep up with 8 flop per cache byte at HBM speed.
//   * the rotation of q and of the new key (src/operators.cpp:47-78) and the write of the new key and
//     value into the request's page happen here too when the caller asks for it: q is rotated in the
//     registers of its tensor-core fragments, and the CTA whose key range holds the new position
//     stores k and v before it starts reading, so a decode step needs no separate rotation / cache
//     write kernel (src/cuda/kernels.cu:86-145 in the reference);
//   * the parts are merged by whichever CTA of a (request, kv head) finishes last (a counter in
//     scratch memory, reset by that CTA), not by a second kernel; nobody waits for anybody.
// The grid depends only on (requests, kv heads, SPLITS); lengths are read on the device, so one
// captured graph serves every later step.
//
// Compile-time: HEAD_DIM (multiple of 16, <= 256).
#include <mutex>

#include "attention_decode.h"
#include "attention_decode_core.cuh"

namespace tlie {

__global__ void __launch_bounds__(kWarps * 32) decode_attention_kernel(const DecodeAttnParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int last_arrival;
  DecodeAttnItem it;
  it.split = blockIdx.x;
  it.kvh = blockIdx.y;
  it.seq = blockIdx.z;
  grid_launch_dependents();
  // With fuse_rope nothing this kernel reads before its q comes from the kernel just before it: positions and block
  // tables were set before the step began, and every cached key but the new one is from earlier steps.  So the cache
  // tiles are fetched first and the wait for the previous kernel (which produces q, k, v of the new token) comes after.
  if (!p.fuse_rope) grid_dependency_wait();
  decode_attn_prologue(p, it, smem_raw);
  if (p.fuse_rope) grid_dependency_wait();
  decode_attn_main(p, it, smem_raw, &last_arrival);
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_decode_attention_head_dim() { return kD; }

constexpr int kMaxTickets = 16384;   // requests * kv_heads a launch may have

// Scratch: kMaxTickets counters (zero when first used; every launch leaves them zero), then for splits > 1 the parts.
TLIE_EXPORT long long tlie_decode_attention_scratch_floats(int requests, int q_heads, int splits) {
  return kMaxTickets + (splits <= 1 ? 0 : (long long)requests * q_heads * splits * (kD + 2));
}

// fuse_rope 0: q in `q` is rotated and the cache holds the new keys.  fuse_rope 1: rows of `q` are [q | k | v] of the new
// token, unrotated; inv_freq (kD / 2 frequencies, or null for no rotation) rotates q and k here, and write_cache stores k, v.
TLIE_EXPORT int tlie_decode_attention(const void* q, int q_row_stride, void* pages, const int* positions,
                                      const int* block_table, int table_stride, void* out, float* scratch, int requests,
                                      int q_heads, int kv_heads, int page_size, int window, float scale, int splits,
                                      int fuse_rope, const float* inv_freq, int write_cache, cudaStream_t stream) {
  if (requests <= 0) return 0;
  if (kv_heads <= 0 || q_heads % kv_heads != 0 || q_heads / kv_heads > 16 || splits < 1 || splits > 32 || scratch == nullptr ||
      (long long)requests * kv_heads > kMaxTickets || (fuse_rope && inv_freq != nullptr && kD % 32 != 0) || !(scale > 0.0f))   // the maximum is taken before the scale
    return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  DecodeAttnParams p;
  p.q = (const __nv_bfloat16*)q;
  p.q_row_stride = q_row_stride;
  p.pages = (__nv_bfloat16*)pages;
  p.positions = positions;
  p.block_table = block_table;
  p.table_stride = table_stride;
  p.out = (__nv_bfloat16*)out;
  p.tickets = reinterpret_cast<int*>(scratch);
  p.partial_o = scratch + kMaxTickets;
  p.partial_ml = p.partial_o + (size_t)requests * q_heads * splits * kD;
  p.q_heads = q_heads;
  p.kv_heads = kv_heads;
  p.page_size = page_size;
  p.page_shift = -1;
  for (int shift = 0; shift < 31; ++shift)
    if ((1 << shift) == page_size) p.page_shift = shift;
  p.window = window;
  p.scale = scale;
  p.splits = splits;
  p.fuse_rope = fuse_rope;
  p.inv_freq = inv_freq;
  p.write_cache = write_cache;
  dim3 grid(splits, kv_heads, requests);
  return (int)launch_pdl(decode_attention_kernel, grid, dim3(kWarps * 32), kSmemBytes, stream, p);
}

// --- the entry point that allocates nothing (declared and documented in attention_decode.h) --------------------
constexpr int kStaticMaxSlots = 8192;   // (request, head, part) triples the built-in scratch has room for
constexpr size_t kStaticScratchFloats = (size_t)kMaxTickets + (size_t)kStaticMaxSlots * (kD + 2);
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address: the address a kernel can
// use is looked up once per device, with that device current.
static float* static_scratch_address(cudaError_t* error) {
  static float* address[64] = {};
  static std::mutex guard;   // first calls on several devices may come from several host threads
  std::lock_guard<std::mutex> lock(guard);
  int device = 0;
  *error = cudaGetDevice(&device);
  if (*error != cudaSuccess) return nullptr;
  if (device < 0 || device >= 64) {
    *error = cudaErrorInvalidDevice;
    return nullptr;
  }
  if (address[device] == nullptr) {
    void* found = nullptr;
    *error = cudaGetSymbolAddress(&found, g_static_scratch);
    if (*error != cudaSuccess) return nullptr;
    address[device] = static_cast<float*>(found);
  }
  return address[device];
}

TLIE_EXPORT int tlie_decode_attention_static(const void* q, int q_row_stride, void* pages, const int* positions,
                                             const int* block_table, int table_stride, void* out, int requests,
                                             int q_heads, int kv_heads, int page_size, int window, float scale, int splits,
                                             int fuse_rope, const float* inv_freq, int write_cache, cudaStream_t stream) {
  if (requests <= 0) return 0;
  // every shape rule of tlie_decode_attention is applied here first, so that nothing at all is enqueued for a refused shape
  if (kv_heads <= 0 || q_heads <= 0 || q_heads % kv_heads != 0 || q_heads / kv_heads > 16 || splits < 1 || splits > 32 ||
      (fuse_rope && inv_freq != nullptr && kD % 32 != 0) || !(scale > 0.0f))
    return (int)cudaErrorInvalidValue;
  if ((long long)requests * q_heads * splits > kStaticMaxSlots || (long long)requests * kv_heads > kMaxTickets)
    return (int)cudaErrorInvalidValue;   // beyond the built-in scratch: nothing is launched
  cudaError_t error = cudaSuccess;
  float* scratch = static_scratch_address(&error);
  if (scratch == nullptr) return (int)error;
  // the arrival counters must start at zero; the rest of the array is written before it is read
  error = cudaMemsetAsync(scratch, 0, (size_t)requests * kv_heads * sizeof(int), stream);
  if (error != cudaSuccess) return (int)error;
  return tlie_decode_attention(q, q_row_stride, pages, positions, block_table, table_stride, out, scratch, requests, q_heads,
                               kv_heads, page_size, window, scale, splits, fuse_rope, inv_freq, write_cache, stream);
}
