// Paged grouped-query attention for any mixture of prompt portions and decode tokens:
// the general kernel of the 32-bit path, and the reference shape for the faster ones.
//
// For query token t of request s at absolute position p, head h (kv head g = h / group):
//   score_j = (q . k_j) * scale  for j in [lo, p],  lo = window > 0 ? max(0, p - window + 1) : 0
//   out = softmax(score) . v                         (src/operators.cpp:102-146)
// Causality comes from attending only to positions <= p, exactly as the reference attends
// to the first position+1 cache entries (src/model.cpp:159-169).  Keys and values are read
// through the request's block table from pages laid out
// [page][2 (k, v)][kv head][slot][head_dim].
//
// One warp owns one (token, head) pair and walks the keys in ascending order, 32 at a
// time, with a running maximum and sum in 32-bit.  The order of operations for a row
// depends only on the row's own position, never on the batch, so the 32-bit path gives
// bit-identical rows however the tokens were cut into steps.
#include "common.cuh"

namespace tlie {

constexpr int kMaxHeadDim = 256;
constexpr int kWarpsPerBlock = 4;

template <typename T>
__global__ void paged_attention_generic_kernel(const T* __restrict__ q, int q_row_stride, const T* __restrict__ pages,
                                               const int* __restrict__ positions, const int* __restrict__ token_seq,
                                               const int* __restrict__ block_table, int table_stride,
                                               T* __restrict__ out, int tokens, int q_heads, int kv_heads,
                                               int head_dim, int page_size, int window, float scale) {
  __shared__ float q_smem[kWarpsPerBlock][kMaxHeadDim];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long pair = (long long)blockIdx.x * kWarpsPerBlock + warp;
  if (pair >= (long long)tokens * q_heads) return;
  const int t = (int)(pair / q_heads);
  const int h = (int)(pair - (long long)t * q_heads);
  const int g = h / (q_heads / kv_heads);
  const int pos = positions[t];
  const int* table = block_table + (size_t)token_seq[t] * table_stride;

  const T* q_row = q + (size_t)t * q_row_stride + (size_t)h * head_dim;
  for (int d = lane; d < head_dim; d += 32) q_smem[warp][d] = to_float(q_row[d]);
  __syncwarp();

  const size_t plane = (size_t)kv_heads * page_size * head_dim;
  const size_t head_offset = (size_t)g * page_size * head_dim;
  const int dims_per_lane = (head_dim + 31) / 32;

  float acc[kMaxHeadDim / 32];
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = 0.0f;
  float running_max = -INFINITY;
  float running_sum = 0.0f;

  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  for (int base = lo; base <= pos; base += 32) {
    const int key = base + lane;
    const bool valid = key <= pos;
    float score = -INFINITY;
    if (valid) {
      const int page = table[key / page_size];
      const T* k_row = pages + (size_t)page * 2 * plane + head_offset + (size_t)(key % page_size) * head_dim;
      float dot = 0.0f;
      for (int d = 0; d < head_dim; ++d) dot += q_smem[warp][d] * to_float(k_row[d]);
      score = dot * scale;
    }
    const float chunk_max = warp_max(score);
    const float new_max = fmaxf(running_max, chunk_max);
    const float rescale = expf(running_max - new_max);  // exp(-inf) = 0 on the first chunk
    const float p = valid ? expf(score - new_max) : 0.0f;
    running_sum = running_sum * rescale + warp_sum(p);
    running_max = new_max;
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] *= rescale;
    const int count = min(32, pos - base + 1);
    for (int j = 0; j < count; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int kj = base + j;
      const int page = table[kj / page_size];
      const T* v_row = pages + (size_t)page * 2 * plane + plane + head_offset + (size_t)(kj % page_size) * head_dim;
#pragma unroll
      for (int i = 0; i < kMaxHeadDim / 32; ++i) {
        const int d = lane + 32 * i;
        if (i < dims_per_lane && d < head_dim) acc[i] += pj * to_float(v_row[d]);
      }
    }
  }
  T* o_row = out + (size_t)t * q_heads * head_dim + (size_t)h * head_dim;
  const float inv = 1.0f / running_sum;
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) {
    const int d = lane + 32 * i;
    if (i < dims_per_lane && d < head_dim) o_row[d] = from_float<T>(acc[i] * inv);
  }
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_paged_attention_generic(int dtype, const void* q, int q_row_stride, const void* pages,
                                             const int* positions, const int* token_seq, const int* block_table,
                                             int table_stride, void* out, int tokens, int q_heads, int kv_heads,
                                             int head_dim, int page_size, int window, float scale,
                                             cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (head_dim > kMaxHeadDim || head_dim <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0)
    return (int)cudaErrorInvalidValue;
  const long long pairs = (long long)tokens * q_heads;
  const int blocks = (int)((pairs + kWarpsPerBlock - 1) / kWarpsPerBlock);
  if (dtype == TLIE_F32)
    paged_attention_generic_kernel<float><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(
        (const float*)q, q_row_stride, (const float*)pages, positions, token_seq, block_table, table_stride,
        (float*)out, tokens, q_heads, kv_heads, head_dim, page_size, window, scale);
  else
    paged_attention_generic_kernel<__nv_bfloat16><<<blocks, kWarpsPerBlock * 32, 0, stream>>>(
        (const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)pages, positions, token_seq, block_table,
        table_stride, (__nv_bfloat16*)out, tokens, q_heads, kv_heads, head_dim, page_size, window, scale);
  return (int)cudaGetLastError();
}
