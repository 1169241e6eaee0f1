// Fused weight-streaming products for decode steps of up to 16 rows, bfloat16 weights.
//
//     out[M, N] (+)= f(x)[M, K] . w[N, K]^T
//
// A decode step of this model is ~2 GB of weights read once and a few kilobytes of activations; it
// is bound by HBM and by the fixed cost of every kernel boundary.  The reference runs 15 launches
// per layer and token (src/cuda/model.cu:406-475: norm, 7 library products, rotation, cache write,
// attention, activation, 2 adds).  Here one kernel family does product + neighbours:
//   input   X_PLAIN  x is bfloat16 [M, K];
//           X_NORM   x = rmsnorm(residual[rows]) * norm_weight, computed from the 32-bit residual
//                    stream by every CTA for itself (M * K * 4 bytes out of L2), statistics in
//                    32-bit exactly as the separate kernel (src/operators.cpp:22-45);
//   output  STORE    bfloat16 or 32-bit [M, N];
//           ACCUM    residual[m, n] += result in 32-bit (each element owned by one thread, so the
//                    sum is deterministic): the reference's add kernel (src/cuda/kernels.cu:208-215);
//           GATED    the CTA computes rows n of the gate half and of the up half of w and stores
//                    silu(gate) * up (src/operators.cpp:148-164) as bfloat16 [M, N/2].
// Mechanics: 16 weight rows are the A operand of mma.sync m16n8k16 and 8 rows of x the B operand
// (M = 8 wastes nothing); the contraction index is permuted so that a thread fetches 8 consecutive
// k of a weight row with one 16-byte load feeding two MMAs; the 8 warps of a CTA split K, keep
// their whole share of the weights in flight in registers, and sum through shared memory.  Weight
// loads are issued BEFORE the programmatic-dependency wait: while the previous kernel of the step
// still runs, this one already streams its weights.
#include "common.cuh"
#include "mma_utils.cuh"

namespace tlie {

constexpr int kGemvWarps = 8;
enum { X_PLAIN = 0, X_NORM = 1 };
enum { EPI_STORE_BF16 = 0, EPI_STORE_F32 = 1, EPI_ACCUM = 2, EPI_GATED = 3 };

struct GemvArgs {
  const void* x;            // X_PLAIN: bf16 [M, ldx];  X_NORM: float residual [*, K]
  int ldx;
  const int* rows;          // X_NORM: optional gather of residual rows (nullptr: row m)
  const float* norm_weight; // X_NORM
  float eps;                // X_NORM
  const __nv_bfloat16* w;   // [N, K]
  void* out;                // STORE: [M, N]; ACCUM: float residual [M, N]; GATED: bf16 [M, N / 2]
  int M, N, K;
  int x_stride;             // shared-memory row stride of x, in elements
};

__device__ __forceinline__ uint4 load_stream_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// TILES: 1 (16 weight rows) or 2 (GATED: 16 gate rows + the 16 up rows N/2 below).
template <int MT, int XMODE, int EPI>
__global__ void __launch_bounds__(kGemvWarps * 32) gemv_fused_kernel(const GemvArgs a) {
  constexpr int TILES = (EPI == EPI_GATED) ? 2 : 1;
  constexpr int UNROLL = (EPI == EPI_GATED) ? 4 : 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                       // [MT * 8][x_stride]
  float* red = reinterpret_cast<float*>(smem_raw + (size_t)MT * 8 * a.x_stride * 2);   // [warps][TILES][16][MT * 8 + 1]
  __shared__ float row_scale[MT * 8];
  constexpr int kRedRow = MT * 8 + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int K = a.K;
  const int n_rows = (EPI == EPI_GATED) ? a.N / 2 : a.N;      // rows of one half
  const int n0 = blockIdx.x * 16;
  const __nv_bfloat16* wrow[TILES][2];
#pragma unroll
  for (int tile = 0; tile < TILES; ++tile) {
    const int base = tile * n_rows;
    wrow[tile][0] = a.w + (size_t)(base + min(n0 + g, n_rows - 1)) * K + t * 8;
    wrow[tile][1] = a.w + (size_t)(base + min(n0 + g + 8, n_rows - 1)) * K + t * 8;
  }
  const int blocks = (K + 31) / 32;

  // --- weights of the first round, before anything that depends on the previous kernel ---------
  uint4 wreg[UNROLL][TILES][2];
  auto issue = [&](int kb0) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int kb = kb0 + u * kGemvWarps;
      const bool valid = kb * 32 + t * 8 < K;
#pragma unroll
      for (int tile = 0; tile < TILES; ++tile) {
        wreg[u][tile][0] = valid ? load_stream_16(wrow[tile][0] + (size_t)kb * 32) : make_uint4(0, 0, 0, 0);
        wreg[u][tile][1] = valid ? load_stream_16(wrow[tile][1] + (size_t)kb * 32) : make_uint4(0, 0, 0, 0);
      }
    }
  };
  issue(warp);
  grid_launch_dependents();
  grid_dependency_wait();

  // --- stage x in shared memory as bfloat16 -----------------------------------------------------
  if (XMODE == X_PLAIN) {
    const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(a.x);
    const int chunks = K / 8;
    for (int idx = threadIdx.x; idx < MT * 8 * chunks; idx += kGemvWarps * 32) {
      const int m = idx / chunks;
      const int c = idx - m * chunks;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (m < a.M) v = *reinterpret_cast<const uint4*>(x + (size_t)m * a.ldx + c * 8);
      *reinterpret_cast<uint4*>(xs + (size_t)m * a.x_stride + c * 8) = v;
    }
  } else {
    const float* residual = reinterpret_cast<const float*>(a.x);
    // one warp per row: sum of squares in 32-bit, then scale
    for (int m = warp; m < MT * 8; m += kGemvWarps) {
      float sum = 0.0f;
      if (m < a.M) {
        const float* r = residual + (size_t)(a.rows ? a.rows[m] : m) * K;
        for (int c = lane; c < K / 4; c += 32) {
          const float4 v = *reinterpret_cast<const float4*>(r + c * 4);
          sum += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
      }
      sum = warp_sum(sum);
      if (lane == 0) row_scale[m] = 1.0f / sqrtf(sum / (float)K + a.eps);
    }
    __syncthreads();
    const int chunks = K / 4;
    for (int idx = threadIdx.x; idx < MT * 8 * chunks; idx += kGemvWarps * 32) {
      const int m = idx / chunks;
      const int c = idx - m * chunks;
      uint2 packed = make_uint2(0, 0);
      if (m < a.M) {
        const float* r = residual + (size_t)(a.rows ? a.rows[m] : m) * K;
        const float4 v = *reinterpret_cast<const float4*>(r + c * 4);
        const float4 nw = *reinterpret_cast<const float4*>(a.norm_weight + c * 4);
        const float s = row_scale[m];
        packed.x = pack_bf16((v.x * s) * nw.x, (v.y * s) * nw.y);
        packed.y = pack_bf16((v.z * s) * nw.z, (v.w * s) * nw.w);
      }
      *reinterpret_cast<uint2*>(xs + (size_t)m * a.x_stride + c * 4) = packed;
    }
  }
  __syncthreads();

  // --- main loop: this warp's 32-wide k blocks warp, warp + 8, ... -------------------------------
  float acc[TILES][MT][4];
#pragma unroll
  for (int tile = 0; tile < TILES; ++tile)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) acc[tile][mt][0] = acc[tile][mt][1] = acc[tile][mt][2] = acc[tile][mt][3] = 0.0f;

  for (int kb0 = warp; kb0 < blocks; kb0 += kGemvWarps * UNROLL) {
    if (kb0 != warp) issue(kb0);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int kb = kb0 + u * kGemvWarps;
      if (kb >= blocks) continue;          // the same for every lane: mma.sync needs the whole warp
      const int k = kb * 32 + t * 8;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        // lanes past K (a last block of fewer than 32) contribute zeros: their weights are zero too
        const uint4 xv = k < K ? *reinterpret_cast<const uint4*>(xs + (size_t)(mt * 8 + g) * a.x_stride + k) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int tile = 0; tile < TILES; ++tile) {
          const unsigned lo[4] = {wreg[u][tile][0].x, wreg[u][tile][1].x, wreg[u][tile][0].y, wreg[u][tile][1].y};
          const unsigned hi[4] = {wreg[u][tile][0].z, wreg[u][tile][1].z, wreg[u][tile][0].w, wreg[u][tile][1].w};
          mma_bf16(acc[tile][mt], lo, xv.x, xv.y);
          mma_bf16(acc[tile][mt], hi, xv.z, xv.w);
        }
      }
    }
  }

  // --- sum the warps' tiles, then the epilogue -----------------------------------------------------
#pragma unroll
  for (int tile = 0; tile < TILES; ++tile) {
    float* base = red + ((size_t)warp * TILES + tile) * 16 * kRedRow;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      base[g * kRedRow + mt * 8 + 2 * t] = acc[tile][mt][0];
      base[g * kRedRow + mt * 8 + 2 * t + 1] = acc[tile][mt][1];
      base[(g + 8) * kRedRow + mt * 8 + 2 * t] = acc[tile][mt][2];
      base[(g + 8) * kRedRow + mt * 8 + 2 * t + 1] = acc[tile][mt][3];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < 16 * MT * 8; idx += kGemvWarps * 32) {
    const int m = idx / 16;
    const int r = idx - m * 16;
    if (m >= a.M || n0 + r >= n_rows) continue;
    float sum[TILES];
#pragma unroll
    for (int tile = 0; tile < TILES; ++tile) {
      sum[tile] = 0.0f;
#pragma unroll
      for (int wi = 0; wi < kGemvWarps; ++wi) sum[tile] += red[((size_t)wi * TILES + tile) * 16 * kRedRow + r * kRedRow + m];
    }
    const size_t o = (size_t)m * n_rows + n0 + r;
    if (EPI == EPI_STORE_BF16) {
      reinterpret_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn(sum[0]);
    } else if (EPI == EPI_STORE_F32) {
      reinterpret_cast<float*>(a.out)[o] = sum[0];
    } else if (EPI == EPI_ACCUM) {
      reinterpret_cast<float*>(a.out)[o] += sum[0];
    } else {
      // gate and up are rounded to bfloat16 first, as when the product is stored and read back
      const float gate = __bfloat162float(__float2bfloat16_rn(sum[0]));
      const float up = __bfloat162float(__float2bfloat16_rn(sum[TILES - 1]));
      reinterpret_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn((gate / (1.0f + expf(-gate))) * up);
    }
  }
}

template <int MT, int XMODE, int EPI>
static int launch_one(const GemvArgs& a, cudaStream_t stream) {
  constexpr int TILES = (EPI == EPI_GATED) ? 2 : 1;
  const size_t smem = (size_t)MT * 8 * a.x_stride * 2 + (size_t)kGemvWarps * TILES * 16 * (MT * 8 + 1) * sizeof(float);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemv_fused_kernel<MT, XMODE, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  const int n_rows = (EPI == EPI_GATED) ? a.N / 2 : a.N;
  return (int)launch_pdl(gemv_fused_kernel<MT, XMODE, EPI>, dim3((n_rows + 15) / 16), dim3(kGemvWarps * 32), smem, stream, a);
}

template <int XMODE, int EPI>
static int launch_rows(const GemvArgs& a, cudaStream_t stream) {
  if (a.M <= 8) return launch_one<1, XMODE, EPI>(a, stream);
  if (a.M <= 16) return launch_one<2, XMODE, EPI>(a, stream);
  return (int)cudaErrorInvalidValue;
}

template <int XMODE>
static int launch_epilogue(const GemvArgs& a, int epilogue, cudaStream_t stream) {
  switch (epilogue) {
    case EPI_STORE_BF16: return launch_rows<XMODE, EPI_STORE_BF16>(a, stream);
    case EPI_STORE_F32: return launch_rows<XMODE, EPI_STORE_F32>(a, stream);
    case EPI_ACCUM: return launch_rows<XMODE, EPI_ACCUM>(a, stream);
    case EPI_GATED: return launch_rows<XMODE, EPI_GATED>(a, stream);
  }
  return (int)cudaErrorInvalidValue;
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_gemv_max_rows() { return 16; }

// x_mode 0: x bf16 [M, K] with row stride ldx.  x_mode 1: x is the 32-bit residual [*, K]; rows (optional) gathers,
// norm_weight [K] and eps give the RMSNorm.  epilogue 0: bf16 out [M, N]; 1: 32-bit out; 2: out (32-bit [M, N]) += result;
// 3: w holds [gate rows | up rows] (N even), out = silu(gate) * up as bf16 [M, N / 2].
// Needs K % 8 == 0 (K % 4 == 0 suffices for x_mode 1 is NOT enough: weights are read 8 at a time), M <= 16.
TLIE_EXPORT int tlie_gemv_fused(int x_mode, const void* x, int ldx, const int* rows, const float* norm_weight, float eps,
                                const void* w, void* out, int M, int N, int K, int epilogue, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || M > 16 || (x_mode == X_PLAIN && ldx % 8 != 0) || (epilogue == EPI_GATED && (N & 1)))
    return (int)cudaErrorInvalidValue;
  GemvArgs a;
  a.x = x;
  a.ldx = ldx;
  a.rows = rows;
  a.norm_weight = norm_weight;
  a.eps = eps;
  a.w = (const __nv_bfloat16*)w;
  a.out = out;
  a.M = M;
  a.N = N;
  a.K = K;
  a.x_stride = K + ((32 - K % 64) + 64) % 64;   // rows shifted by 64 bytes against each other: 16-byte reads without bank conflicts
  if (a.x_stride == K) a.x_stride += 64;
  if (x_mode == X_PLAIN) return launch_epilogue<X_PLAIN>(a, epilogue, stream);
  if (x_mode == X_NORM) return launch_epilogue<X_NORM>(a, epilogue, stream);
  return (int)cudaErrorInvalidValue;
}
