// Weight-streaming matrix product for decode steps: out[M, N] = x[M, K] . w[N, K]^T with M <= 64, bfloat16.
//
// With a handful of rows the product is bound by reading w once from HBM (the reference calls cuBLAS
// here, src/cuda/kernels.cu:342-368; at M = 8 the library's kernels on this GPU take 8-12 us for a
// 10-20 MB matrix, several times the time the bytes need).  Design:
//   * swap the roles: a tile of 16 weight rows is the 16-row A operand of mma.sync m16n8k16 and 8
//     rows of x are the 8-column B operand, so M = 8 wastes nothing;
//   * the contraction index may be permuted freely as long as A and B agree, so each thread reads
//     its part of a weight row as ONE 16-byte load (8 consecutive k) that feeds two MMAs, instead
//     of the fragment layout's scattered 4-byte pieces: a quad reads 64 contiguous bytes of a row;
//   * the 8 warps of a CTA split K among themselves (interleaved 32-wide blocks, every load of a
//     warp's share in flight before the first MMA) and sum their tiles through shared memory;
//     weight loads bypass L1 (read once), x stays in L1/L2;
//   * MODE 1 computes x = silu(gate) * up on the fly from [gate | up] rows (src/operators.cpp:148-164),
//     rounding to bfloat16 exactly as the separate kernel would, which removes that kernel and its
//     traffic from the decode step.
// Accumulation is 32-bit; output bfloat16 or 32-bit (the logits head).
#include "common.cuh"
#include "mma_utils.cuh"

namespace tlie {

constexpr int kSkinnyWarps = 8;
constexpr int kUnroll = 4;

__device__ __forceinline__ uint4 load_stream_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ unsigned silu_mul_pair(unsigned gate, unsigned up) {
  const __nv_bfloat162 g2 = *reinterpret_cast<const __nv_bfloat162*>(&gate);
  const __nv_bfloat162 u2 = *reinterpret_cast<const __nv_bfloat162*>(&up);
  const float g0 = __bfloat162float(g2.x), g1 = __bfloat162float(g2.y);
  const float u0 = __bfloat162float(u2.x), u1 = __bfloat162float(u2.y);
  return pack_bf16((g0 / (1.0f + expf(-g0))) * u0, (g1 / (1.0f + expf(-g1))) * u1);
}

// MT: number of 8-row tiles of x (M <= 8 * MT).  MODE 0: x is [M, K] with row stride ldx.
// MODE 1: x row m is [gate (K) | up (K)] with row stride ldx; the operand is silu(gate) * up.
template <int MT, int MODE, typename OutT>
__global__ void __launch_bounds__(kSkinnyWarps * 32)
    gemm_skinny_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ w,
                       OutT* __restrict__ out, int M, int N, int K) {
  __shared__ float red[kSkinnyWarps][16][8 * MT + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16;
  const int row_a = min(n0 + g, N - 1);       // rows past N repeat the last row; their results are not stored
  const int row_b = min(n0 + g + 8, N - 1);
  const __nv_bfloat16* wa = w + (size_t)row_a * K + t * 8;
  const __nv_bfloat16* wb = w + (size_t)row_b * K + t * 8;

  float c[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) c[mt][0] = c[mt][1] = c[mt][2] = c[mt][3] = 0.0f;

  const int blocks = (K + 31) / 32;
  for (int kb0 = warp; kb0 < blocks; kb0 += kSkinnyWarps * kUnroll) {
    uint4 a[kUnroll], b[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int k = (kb0 + u * kSkinnyWarps) * 32 + t * 8;
      if (k < K) {
        a[u] = load_stream_16(wa + (size_t)(kb0 + u * kSkinnyWarps) * 32);
        b[u] = load_stream_16(wb + (size_t)(kb0 + u * kSkinnyWarps) * 32);
      } else {
        a[u] = make_uint4(0, 0, 0, 0);
        b[u] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int k = (kb0 + u * kSkinnyWarps) * 32 + t * 8;
      const unsigned a_lo[4] = {a[u].x, b[u].x, a[u].y, b[u].y};
      const unsigned a_hi[4] = {a[u].z, b[u].z, a[u].w, b[u].w};
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int m = mt * 8 + g;
        uint4 xv = make_uint4(0, 0, 0, 0);
        if (m < M && k < K) {
          if (MODE == 0) {
            xv = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + k);
          } else {
            const uint4 gate = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + k);
            const uint4 up = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + K + k);
            xv = make_uint4(silu_mul_pair(gate.x, up.x), silu_mul_pair(gate.y, up.y), silu_mul_pair(gate.z, up.z),
                            silu_mul_pair(gate.w, up.w));
          }
        }
        mma_bf16(c[mt], a_lo, xv.x, xv.y);
        mma_bf16(c[mt], a_hi, xv.z, xv.w);
      }
    }
  }
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    red[warp][g][mt * 8 + 2 * t] = c[mt][0];
    red[warp][g][mt * 8 + 2 * t + 1] = c[mt][1];
    red[warp][g + 8][mt * 8 + 2 * t] = c[mt][2];
    red[warp][g + 8][mt * 8 + 2 * t + 1] = c[mt][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 16 * 8 * MT; idx += kSkinnyWarps * 32) {
    const int m = idx / 16;          // consecutive threads write consecutive n of one row of out
    const int r = idx - m * 16;
    if (m >= M || n0 + r >= N) continue;
    float sum = 0.0f;
#pragma unroll
    for (int wi = 0; wi < kSkinnyWarps; ++wi) sum += red[wi][r][m];
    out[(size_t)m * N + n0 + r] = from_float<OutT>(sum);
  }
}

template <int MODE, typename OutT>
static int launch_skinny(const void* x, int ldx, const void* w, void* out, int M, int N, int K, cudaStream_t stream) {
  const int grid = (N + 15) / 16;
  const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
  const __nv_bfloat16* wp = (const __nv_bfloat16*)w;
  OutT* op = (OutT*)out;
  if (M <= 8)
    gemm_skinny_kernel<1, MODE, OutT><<<grid, kSkinnyWarps * 32, 0, stream>>>(xp, ldx, wp, op, M, N, K);
  else if (M <= 16)
    gemm_skinny_kernel<2, MODE, OutT><<<grid, kSkinnyWarps * 32, 0, stream>>>(xp, ldx, wp, op, M, N, K);
  else if (M <= 32)
    gemm_skinny_kernel<4, MODE, OutT><<<grid, kSkinnyWarps * 32, 0, stream>>>(xp, ldx, wp, op, M, N, K);
  else if (M <= 64)
    gemm_skinny_kernel<8, MODE, OutT><<<grid, kSkinnyWarps * 32, 0, stream>>>(xp, ldx, wp, op, M, N, K);
  else
    return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}

}  // namespace tlie

using namespace tlie;

// mode 0: x [M, K] (row stride ldx);  mode 1: x rows are [gate | up], operand silu(gate) * up.
// out_f32: 1 writes 32-bit outputs, 0 bfloat16.  Needs K % 8 == 0, ldx % 8 == 0 and 16-byte aligned bases.
TLIE_EXPORT int tlie_gemm_skinny(const void* x, int ldx, const void* w, void* out, int M, int N, int K, int mode,
                                 int out_f32, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || M > 64) return (int)cudaErrorInvalidValue;
  if (mode == 0) {
    return out_f32 ? launch_skinny<0, float>(x, ldx, w, out, M, N, K, stream)
                   : launch_skinny<0, __nv_bfloat16>(x, ldx, w, out, M, N, K, stream);
  }
  if (mode == 1) {
    return out_f32 ? launch_skinny<1, float>(x, ldx, w, out, M, N, K, stream)
                   : launch_skinny<1, __nv_bfloat16>(x, ldx, w, out, M, N, K, stream);
  }
  return (int)cudaErrorInvalidValue;
}
