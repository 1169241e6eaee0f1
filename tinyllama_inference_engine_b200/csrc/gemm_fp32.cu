// True 32-bit matrix product for the float32 path: out[M, N] = x[M, K] . w[N, K]^T.
//
// The reference's 32-bit model computes each output as one dot product over K in index
// order (src/model.cpp:53-78).  This kernel keeps that property on the GPU: every output
// element is accumulated by one thread with fused multiply-adds in ascending k, so its
// value depends on neither M nor N nor the tile it falls in, and no reduced-precision
// tensor-core mode can be involved.  It is not a performance path.
#include "common.cuh"

namespace tlie {

constexpr int kTile = 64;
constexpr int kTileK = 16;

__global__ void __launch_bounds__(256) gemm_nt_f32_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                          float* __restrict__ out, int M, int N, int K) {
  __shared__ float xs[kTileK][kTile + 1];
  __shared__ float ws[kTileK][kTile + 1];
  const int tx = threadIdx.x % 16;
  const int ty = threadIdx.x / 16;
  const int row0 = blockIdx.y * kTile;
  const int col0 = blockIdx.x * kTile;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += kTileK) {
    for (int idx = threadIdx.x; idx < kTile * kTileK; idx += 256) {
      const int r = idx / kTileK;
      const int k = idx % kTileK;
      const int gk = k0 + k;
      const int gr = row0 + r;
      const int gc = col0 + r;
      xs[k][r] = (gr < M && gk < K) ? x[(size_t)gr * K + gk] : 0.0f;
      ws[k][r] = (gc < N && gk < K) ? w[(size_t)gc * K + gk] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kTileK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gr = row0 + ty * 4 + i;
    if (gr >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gc = col0 + tx * 4 + j;
      if (gc < N) out[(size_t)gr * N + gc] = acc[i][j];
    }
  }
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_gemm_nt_f32(const float* x, const float* w, float* out, int M, int N, int K,
                                 cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return (int)cudaErrorInvalidValue;
  dim3 grid((N + kTile - 1) / kTile, (M + kTile - 1) / kTile);
  gemm_nt_f32_kernel<<<grid, 256, 0, stream>>>(x, w, out, M, N, K);
  return (int)cudaGetLastError();
}
