// Rotary position encoding of q and k, fused with the write of k and v into cache pages.
//
// Rotation as in the reference (src/operators.cpp:47-78, src/cuda/kernels.cu:86-115):
// "half-split" pairs (d, d + R/2) of the first R = rotary_dim elements of a head,
// angle = float(position) * inv_freq[d], all in 32-bit.  inv_freq[d] = theta^(-2d/R) is
// a table the host computes once, so host reference and kernel use the same frequencies.
// The reference rotates one token per launch and copies k, v with a second kernel
// (kernels.cu:137-145); here one launch handles every token of the step and stores
// through the request's block table.
//
// qkv row layout: [q heads | k heads | v heads], each head head_dim wide.
// Page layout (one layer): [page][2 (k, v)][kv head][slot in page][head_dim].
#include "common.cuh"

namespace tlie {

// One block per token.  The block first computes the token's rotary_dim / 2 cosines and sines once into shared
// memory (every head uses the same ones), then walks the heads two elements at a time.
constexpr int kMaxRotaryHalf = 128;

template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                  const int* __restrict__ token_seq, const int* __restrict__ block_table,
                                  int table_stride, const float* __restrict__ inv_freq, int rotary_dim,
                                  T* __restrict__ pages, int q_heads, int kv_heads, int head_dim, int page_size,
                                  int write_cache) {
  __shared__ float cos_s[kMaxRotaryHalf], sin_s[kMaxRotaryHalf];
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int row_width = (q_heads + 2 * kv_heads) * head_dim;
  T* row = qkv + (size_t)t * row_width;
  const int half = rotary_dim / 2;
  for (int d = threadIdx.x; d < half; d += blockDim.x) {
    const float angle = (float)pos * inv_freq[d];
    cos_s[d] = cosf(angle);
    sin_s[d] = sinf(angle);
  }
  __syncthreads();

  T* k_dst = nullptr;
  T* v_dst = nullptr;
  if (write_cache) {
    const int seq = token_seq[t];
    const int page = block_table[(size_t)seq * table_stride + pos / page_size];
    const int slot = pos % page_size;
    const size_t plane = (size_t)kv_heads * page_size * head_dim;
    k_dst = pages + (size_t)page * 2 * plane + (size_t)slot * head_dim;
    v_dst = k_dst + plane;
  }
  const size_t head_stride_in_page = (size_t)page_size * head_dim;

  // q heads and k heads: rotate the first rotary_dim elements, pass the rest through.
  const int rot_heads = q_heads + (write_cache ? kv_heads : 0);
  const int per_head = head_dim - half;  // one work item per pair, one per unrotated element
  int head = threadIdx.x / per_head;
  int d = threadIdx.x - head * per_head;
  const int head_step = blockDim.x / per_head, d_step = blockDim.x - head_step * per_head;
  for (; head < rot_heads;) {
    T* x = row + (size_t)head * head_dim;
    const bool is_k = head >= q_heads;
    T* dst = is_k ? (k_dst + (size_t)(head - q_heads) * head_stride_in_page) : x;
    if (d < half) {
      float first = to_float(x[d]);
      float second = to_float(x[d + half]);
      if (inv_freq != nullptr) {
        const float c = cos_s[d], s = sin_s[d];
        const float a = first * c - second * s;
        const float b = second * c + first * s;
        first = a;
        second = b;
      }
      dst[d] = from_float<T>(first);
      dst[d + half] = from_float<T>(second);
    } else {
      const int e = d + half;  // elements rotary_dim .. head_dim-1
      if (is_k) dst[e] = x[e];
    }
    // next work item, blockDim.x further on, without a division
    head += head_step;
    d += d_step;
    if (d >= per_head) {
      d -= per_head;
      head += 1;
    }
  }
  if (write_cache) {
    const T* v = row + (size_t)(q_heads + kv_heads) * head_dim;
    int vh = threadIdx.x / head_dim, vd = threadIdx.x - vh * head_dim;
    const int vh_step = blockDim.x / head_dim, vd_step = blockDim.x - vh_step * head_dim;
    for (; vh < kv_heads;) {
      v_dst[(size_t)vh * head_stride_in_page + vd] = v[vh * head_dim + vd];
      vh += vh_step;
      vd += vd_step;
      if (vd >= head_dim) {
        vd -= head_dim;
        vh += 1;
      }
    }
  }
}

// The same for bfloat16 rows whose pieces are multiples of 8 elements: 16-byte loads and stores, eight pairs per work item.
// (The kernel above moves two bytes at a time: a step of 2,048 tokens took it five times as long as its bytes need.)
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __bfloat162float(h[i].x);
    f[2 * i + 1] = __bfloat162float(h[i].y);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

// A block takes kRopeTokens tokens: their cosines and sines are computed by that many times rotary_dim / 2 threads at once (one
// token per block left all but 32 threads of a block of head size 64 idle while those walked through cosf and sinf, and a
// 2,048-token step took 12 us where its bytes need 4), and every thread then has a few 16-byte pairs of its own in flight.
constexpr int kRopeTokens = 4;

__global__ void rope_store_vec_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ token_seq,
                                      const int* __restrict__ block_table, int table_stride, const float* __restrict__ inv_freq, int rotary_dim,
                                      __nv_bfloat16* __restrict__ pages, int tokens, int q_heads, int kv_heads, int head_dim, int page_size, int write_cache) {
  __shared__ float cos_s[kRopeTokens][kMaxRotaryHalf], sin_s[kRopeTokens][kMaxRotaryHalf];
  __shared__ long long k_offset[kRopeTokens];   // where a token's k head 0 goes in the pool, in elements
  grid_launch_dependents();   // launched as a programmatic dependent: the kernel before it has completed when the wait returns
  grid_dependency_wait();
  const int t0 = blockIdx.x * kRopeTokens;
  const int here = min(kRopeTokens, tokens - t0);
  const int row_width = (q_heads + 2 * kv_heads) * head_dim;
  const int half = rotary_dim / 2;
  // pairs of 8 + 8 elements of the rotated part of the q heads and (when the cache is written) the k heads
  const int pieces = half / 8;
  const int items = (q_heads + (write_cache ? kv_heads : 0)) * pieces;
  const int all_items = here * items;
  // A thread's first pair is fetched before anything that waits for the position (the angles, the page of the cache): the
  // row does not depend on it, and a block lives for one memory round trip instead of two in a row.
  uint4 first_lo = make_uint4(0, 0, 0, 0), first_hi = first_lo;
  if ((int)threadIdx.x < all_items) {
    const int token = threadIdx.x / items, item = threadIdx.x - token * items;
    const int head = item / pieces, d = (item - head * pieces) * 8;
    const __nv_bfloat16* x = qkv + (size_t)(t0 + token) * row_width + (size_t)head * head_dim + d;
    first_lo = *reinterpret_cast<const uint4*>(x);
    first_hi = *reinterpret_cast<const uint4*>(x + half);
  }
  if (inv_freq != nullptr) {
    for (int index = threadIdx.x; index < here * half; index += blockDim.x) {
      const int token = index / half, d = index - token * half;
      const float angle = (float)positions[t0 + token] * inv_freq[d];
      cos_s[token][d] = cosf(angle);
      sin_s[token][d] = sinf(angle);
    }
  }
  const size_t head_stride_in_page = (size_t)page_size * head_dim;
  const size_t plane = (size_t)kv_heads * page_size * head_dim;
  if (write_cache && (int)threadIdx.x < here) {
    const int t = t0 + threadIdx.x, pos = positions[t];
    const int page = block_table[(size_t)token_seq[t] * table_stride + pos / page_size];
    k_offset[threadIdx.x] = (long long)((size_t)page * 2 * plane + (size_t)(pos % page_size) * head_dim);
  }
  __syncthreads();
  for (int index = threadIdx.x; index < all_items; index += blockDim.x) {
    const int token = index / items, item = index - token * items;
    const int head = item / pieces, d = (item - head * pieces) * 8;
    __nv_bfloat16* x = qkv + (size_t)(t0 + token) * row_width + (size_t)head * head_dim;
    __nv_bfloat16* dst = head >= q_heads ? pages + k_offset[token] + (size_t)(head - q_heads) * head_stride_in_page : x;
    uint4 lo = first_lo, hi = first_hi;
    if (index != (int)threadIdx.x) {
      lo = *reinterpret_cast<const uint4*>(x + d);
      hi = *reinterpret_cast<const uint4*>(x + d + half);
    }
    if (inv_freq != nullptr) {
      float a[8], b[8], ra[8], rb[8];
      unpack8(lo, a);
      unpack8(hi, b);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float c = cos_s[token][d + i], sn = sin_s[token][d + i];
        ra[i] = a[i] * c - b[i] * sn;
        rb[i] = b[i] * c + a[i] * sn;
      }
      lo = pack8(ra);
      hi = pack8(rb);
    }
    if (inv_freq != nullptr || head >= q_heads) {
      *reinterpret_cast<uint4*>(dst + d) = lo;
      *reinterpret_cast<uint4*>(dst + d + half) = hi;
    }
  }
  if (!write_cache) return;
  // what lies past the rotated part of the k heads, and the v heads, go to the cache as they are
  const int tail = (head_dim - rotary_dim) / 8, whole = head_dim / 8;
  for (int index = threadIdx.x; index < here * kv_heads * tail; index += blockDim.x) {
    const int token = index / (kv_heads * tail), item = index - token * (kv_heads * tail);
    const int head = item / tail, d = rotary_dim + (item - head * tail) * 8;
    *reinterpret_cast<uint4*>(pages + k_offset[token] + (size_t)head * head_stride_in_page + d) =
        *reinterpret_cast<const uint4*>(qkv + (size_t)(t0 + token) * row_width + (size_t)(q_heads + head) * head_dim + d);
  }
  for (int index = threadIdx.x; index < here * kv_heads * whole; index += blockDim.x) {
    const int token = index / (kv_heads * whole), item = index - token * (kv_heads * whole);
    const int head = item / whole, d = (item - head * whole) * 8;
    *reinterpret_cast<uint4*>(pages + k_offset[token] + plane + (size_t)head * head_stride_in_page + d) =
        *reinterpret_cast<const uint4*>(qkv + (size_t)(t0 + token) * row_width + (size_t)(q_heads + kv_heads + head) * head_dim + d);
  }
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_rope_store(int dtype, void* qkv, const int* positions, const int* token_seq,
                                const int* block_table, int table_stride, const float* inv_freq, int rotary_dim,
                                void* pages, int tokens, int q_heads, int kv_heads, int head_dim, int page_size,
                                int write_cache, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1) || rotary_dim / 2 > kMaxRotaryHalf) return (int)cudaErrorInvalidValue;
  const int block = 256;
  const int half = rotary_dim / 2;
  if (dtype != TLIE_F32 && half % 8 == 0 && head_dim % 8 == 0 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)pages & 15) == 0) {
    return (int)launch_pdl(rope_store_vec_kernel, dim3((tokens + kRopeTokens - 1) / kRopeTokens), dim3(block), 0, stream, (__nv_bfloat16*)qkv, positions, token_seq,
                           block_table, table_stride, inv_freq, rotary_dim, (__nv_bfloat16*)pages, tokens, q_heads, kv_heads, head_dim, page_size, write_cache);
  }
  if (dtype == TLIE_F32)
    rope_store_kernel<float><<<tokens, block, 0, stream>>>((float*)qkv, positions, token_seq, block_table,
                                                           table_stride, inv_freq, rotary_dim, (float*)pages, q_heads,
                                                           kv_heads, head_dim, page_size, write_cache);
  else
    rope_store_kernel<__nv_bfloat16><<<tokens, block, 0, stream>>>(
        (__nv_bfloat16*)qkv, positions, token_seq, block_table, table_stride, inv_freq, rotary_dim,
        (__nv_bfloat16*)pages, q_heads, kv_heads, head_dim, page_size, write_cache);
  return (int)cudaGetLastError();
}
