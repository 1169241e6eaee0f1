// Row-wise kernels: embedding gather, residual add + RMSNorm, SiLU(gate) * up.
//
// Formulas follow the reference's operators (src/operators.cpp:22-45 RmsNorm,
// :148-164 SiluMultiply) and its CUDA twins (src/cuda/kernels.cu:67-84, 198-215); the
// fusion of the residual add into the norm and the 32-bit residual stream are this
// engine's own.
#include "common.cuh"

namespace tlie {

// residual[t, :] = float(table[ids[t], :]).  An id outside [0, vocab) (a sampler fed non-finite logits can produce one on
// the device, where no host check sees it) reads row 0 instead and sets bit 1 of *error_flag, if one is given.
template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ residual, int hidden, int vocab, int* __restrict__ error_flag) {
  const int row = blockIdx.x;
  int id = ids[row];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0 && error_flag != nullptr) atomicOr(error_flag, 2);
    id = 0;
  }
  const T* src = table + (size_t)id * hidden;
  float* dst = residual + (size_t)row * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_float(src[i]);
}

// Optional add, then RMSNorm.  For output row r the source row is rows ? rows[r] : r.
//   if delta:  residual[src, :] += float(delta[src, :])        (32-bit sum, stored back)
//   scale = 1 / sqrt(mean(residual[src]^2) + eps);  out[r, :] = (x * scale) * weight
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const int* __restrict__ rows, const float* __restrict__ weight,
                                   float eps, T* __restrict__ out, int hidden) {
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* x = residual + (size_t)src * hidden;
  float sum = 0.0f;
  if (delta) {
    const T* d = delta + (size_t)src * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float v = x[i] + to_float(d[i]);
      x[i] = v;
      sum += v * v;
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float v = x[i];
      sum += v * v;
    }
  }
  sum = block_sum(sum, scratch);
  const float scale = 1.0f / sqrtf(sum / (float)hidden + eps);
  T* y = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) y[i] = from_float<T>((x[i] * scale) * weight[i]);
}

// The same for widths that are multiples of 4 up to 8192: every value is read once (16-byte loads, all in flight
// together), kept in registers across the reduction, and written once.
template <typename T>
struct Vec4;
template <>
struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <>
struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__bfloat162float(a.x), __bfloat162float(a.y), __bfloat162float(b.x), __bfloat162float(b.y));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<unsigned*>(&a);
    raw.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};

constexpr int kNormThreads = 256;
constexpr int kNormChunks = 8;   // float4 chunks per thread: widths up to 256 * 8 * 4 = 8192

template <typename T>
__global__ void __launch_bounds__(kNormThreads) add_rmsnorm_vec_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                                                     const int* __restrict__ rows, const float* __restrict__ weight,
                                                                     float eps, T* __restrict__ out, int hidden) {
  __shared__ float scratch[32];
  grid_launch_dependents();   // launched as a programmatic dependent: the kernel before it has completed when the wait returns
  grid_dependency_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* x = residual + (size_t)src * hidden;
  const int chunks = hidden / 4;
  float4 v[kNormChunks];
#pragma unroll
  for (int i = 0; i < kNormChunks; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
    v[i] = c < chunks ? *reinterpret_cast<const float4*>(x + c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (delta) {
    const T* d = delta + (size_t)src * hidden;
#pragma unroll
    for (int i = 0; i < kNormChunks; ++i) {
      const int c = threadIdx.x + i * kNormThreads;
      if (c < chunks) {
        const float4 dv = Vec4<T>::load(d + c * 4);
        v[i].x += dv.x;
        v[i].y += dv.y;
        v[i].z += dv.z;
        v[i].w += dv.w;
        *reinterpret_cast<float4*>(x + c * 4) = v[i];
      }
    }
  }
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < kNormChunks; ++i) sum += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  sum = block_sum(sum, scratch);
  const float scale = 1.0f / sqrtf(sum / (float)hidden + eps);
  T* y = out + (size_t)r * hidden;
#pragma unroll
  for (int i = 0; i < kNormChunks; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
    if (c < chunks) {
      const float4 w = *reinterpret_cast<const float4*>(weight + c * 4);
      Vec4<T>::store(y + c * 4, make_float4((v[i].x * scale) * w.x, (v[i].y * scale) * w.y, (v[i].z * scale) * w.z, (v[i].w * scale) * w.w));
    }
  }
}

// The same for steps of many rows (prompt portions), bfloat16 out: a warp owns a row, so there is no block-wide barrier and a
// CTA of eight warps lives for one memory round trip; a lane keeps its share of the row (every 32nd float4) in registers.
// Widths that are multiples of 4 up to 4096.  (One CTA per row, two block barriers each, took 9.9 us for 2,048 rows of
// 2,048: 2.5 TB/s.)  The sum's order differs from the kernel above, which is why the 32-bit path does not use this one: there
// a row's bits must not depend on how many rows its step has.
constexpr int kRowWarps = 8;
constexpr int kRowChunks = 32;   // float4 per lane at most
template <int CHUNKS>
__global__ void __launch_bounds__(kRowWarps * 32) add_rmsnorm_rows_kernel(float* __restrict__ residual, const __nv_bfloat16* __restrict__ delta,
                                                                        const int* __restrict__ rows, const float* __restrict__ weight, float eps,
                                                                        __nv_bfloat16* __restrict__ out, int out_rows, int hidden) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  if (r >= out_rows) return;
  const int src = rows ? rows[r] : r;
  float* x = residual + (size_t)src * hidden;
  const int chunks = hidden / 4;
  float4 v[CHUNKS];
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = lane + i * 32;
    v[i] = c < chunks ? *reinterpret_cast<const float4*>(x + c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (delta) {
    const __nv_bfloat16* d = delta + (size_t)src * hidden;
#pragma unroll
    for (int i = 0; i < CHUNKS; ++i) {
      const int c = lane + i * 32;
      if (c < chunks) {
        const float4 dv = Vec4<__nv_bfloat16>::load(d + c * 4);
        v[i].x += dv.x;
        v[i].y += dv.y;
        v[i].z += dv.z;
        v[i].w += dv.w;
        *reinterpret_cast<float4*>(x + c * 4) = v[i];
      }
    }
  }
  float sum = 0.0f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) sum += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
  sum = warp_sum(sum);
  const float scale = 1.0f / sqrtf(sum / (float)hidden + eps);
  __nv_bfloat16* y = out + (size_t)r * hidden;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    const int c = lane + i * 32;
    if (c < chunks) {
      const float4 w = *reinterpret_cast<const float4*>(weight + c * 4);
      Vec4<__nv_bfloat16>::store(y + c * 4, make_float4((v[i].x * scale) * w.x, (v[i].y * scale) * w.y, (v[i].z * scale) * w.z, (v[i].w * scale) * w.w));
    }
  }
}

// out[t, i..i+3] = silu(gate) * up for four neighbours at a time (inter % 4 == 0)
template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total4) {
  const int per_row = inter / 4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / per_row;
    const int col = (int)(i - row * per_row) * 4;
    const float4 g = Vec4<T>::load(gate_up + row * 2 * inter + col);
    const float4 u = Vec4<T>::load(gate_up + row * 2 * inter + inter + col);
    Vec4<T>::store(out + row * inter + col, make_float4((g.x / (1.0f + expf(-g.x))) * u.x, (g.y / (1.0f + expf(-g.y))) * u.y,
                                                        (g.z / (1.0f + expf(-g.z))) * u.z, (g.w / (1.0f + expf(-g.w))) * u.w));
  }
}

// residual[t, :] += float(delta[t, :]) without a norm (the last add when no norm follows).
template <typename T>
__global__ void add_kernel(float* __restrict__ residual, const T* __restrict__ delta, size_t count) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
    residual[i] += to_float(delta[i]);
}

// out[t, i] = silu(gate_up[t, i]) * gate_up[t, inter + i]
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, size_t total) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / inter;
    const int col = (int)(i - row * inter);
    const float g = to_float(gate_up[row * 2 * inter + col]);
    const float u = to_float(gate_up[row * 2 * inter + inter + col]);
    out[i] = from_float<T>((g / (1.0f + expf(-g))) * u);
  }
}

}  // namespace tlie

using namespace tlie;

static inline int grid_for(size_t total, int block) {
  size_t blocks = (total + block - 1) / block;
  const size_t most = (size_t)device_sm_count() * 16;
  if (blocks > most) blocks = most;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

TLIE_EXPORT int tlie_embedding(int dtype, const void* table, const int* ids, float* residual, int rows, int hidden, int vocab,
                               int* error_flag, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return (int)cudaErrorInvalidValue;
  if (dtype == TLIE_F32)
    embedding_kernel<float><<<rows, 256, 0, stream>>>((const float*)table, ids, residual, hidden, vocab, error_flag);
  else
    embedding_kernel<__nv_bfloat16><<<rows, 256, 0, stream>>>((const __nv_bfloat16*)table, ids, residual, hidden, vocab, error_flag);
  return (int)cudaGetLastError();
}

TLIE_EXPORT int tlie_add_rmsnorm(int dtype, float* residual, const void* delta, const int* rows, const float* weight,
                                 float eps, void* out, int out_rows, int hidden, cudaStream_t stream) {
  if (out_rows <= 0) return 0;
  if (dtype == TLIE_BF16 && hidden % 4 == 0 && hidden <= 32 * kRowChunks * 4 && out_rows >= 256) {
    // many rows (a prompt portion): a warp per row
    const dim3 grid((out_rows + kRowWarps - 1) / kRowWarps), block(kRowWarps * 32);
    if (hidden <= 32 * 16 * 4)
      return (int)launch_pdl(add_rmsnorm_rows_kernel<16>, grid, block, 0, stream, residual, (const __nv_bfloat16*)delta, rows, weight, eps, (__nv_bfloat16*)out, out_rows, hidden);
    return (int)launch_pdl(add_rmsnorm_rows_kernel<kRowChunks>, grid, block, 0, stream, residual, (const __nv_bfloat16*)delta, rows, weight, eps, (__nv_bfloat16*)out, out_rows,
                           hidden);
  }
  if (hidden % 4 == 0 && hidden <= kNormThreads * kNormChunks * 4) {
    // The order of a row's sum differs from the scalar kernel's but is still a function of the row alone.
    if (dtype == TLIE_F32)
      return (int)launch_pdl(add_rmsnorm_vec_kernel<float>, dim3(out_rows), dim3(kNormThreads), 0, stream, residual, (const float*)delta, rows, weight, eps,
                             (float*)out, hidden);
    return (int)launch_pdl(add_rmsnorm_vec_kernel<__nv_bfloat16>, dim3(out_rows), dim3(kNormThreads), 0, stream, residual, (const __nv_bfloat16*)delta, rows,
                           weight, eps, (__nv_bfloat16*)out, hidden);
  }
  const int block = hidden >= 1024 ? 256 : 128;
  if (dtype == TLIE_F32)
    add_rmsnorm_kernel<float><<<out_rows, block, 0, stream>>>(residual, (const float*)delta, rows, weight, eps,
                                                              (float*)out, hidden);
  else
    add_rmsnorm_kernel<__nv_bfloat16><<<out_rows, block, 0, stream>>>(residual, (const __nv_bfloat16*)delta, rows,
                                                                      weight, eps, (__nv_bfloat16*)out, hidden);
  return (int)cudaGetLastError();
}

TLIE_EXPORT int tlie_add(int dtype, float* residual, const void* delta, long long count, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (dtype == TLIE_F32)
    add_kernel<float><<<grid_for(count, 256), 256, 0, stream>>>(residual, (const float*)delta, (size_t)count);
  else
    add_kernel<__nv_bfloat16><<<grid_for(count, 256), 256, 0, stream>>>(residual, (const __nv_bfloat16*)delta,
                                                                        (size_t)count);
  return (int)cudaGetLastError();
}

TLIE_EXPORT int tlie_silu_mul(int dtype, const void* gate_up, void* out, int rows, int inter, cudaStream_t stream) {
  const size_t total = (size_t)rows * inter;
  if (total == 0) return 0;
  if (inter % 4 == 0) {
    const size_t total4 = total / 4;
    const size_t most = (size_t)device_sm_count() * 32;
    const int blocks = (int)((total4 + 255) / 256 < most ? (total4 + 255) / 256 : most);
    if (dtype == TLIE_F32)
      silu_mul_vec_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gate_up, (float*)out, inter, total4);
    else
      silu_mul_vec_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total4);
    return (int)cudaGetLastError();
  }
  if (dtype == TLIE_F32)
    silu_mul_kernel<float><<<grid_for(total, 256), 256, 0, stream>>>((const float*)gate_up, (float*)out, inter, total);
  else
    silu_mul_kernel<__nv_bfloat16><<<grid_for(total, 256), 256, 0, stream>>>((const __nv_bfloat16*)gate_up,
                                                                             (__nv_bfloat16*)out, inter, total);
  return (int)cudaGetLastError();
}

