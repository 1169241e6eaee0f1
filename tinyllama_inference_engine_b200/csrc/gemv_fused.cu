// Fused weight-streaming products for decode steps of up to 16 rows, bfloat16 weights.
//
//     out[M, N] (+)= f(x)[M, K] . w[N, K]^T
//
// A decode step of this model is ~2 GB of weights read once and a few kilobytes of activations; it
// is bound by HBM and by the fixed cost of every kernel boundary.  The reference runs 15 launches
// per layer and token (src/cuda/model.cu:406-475: norm, 7 library products, rotation, cache write,
// attention, activation, 2 adds).  Here one kernel family does product + neighbours:
//   input   X_PLAIN  x is bfloat16 [M, K];
//           X_NORM   x = rmsnorm(residual[rows]) * norm_weight, from the 32-bit residual stream, by
//                    every CTA for itself (M * K * 4 bytes out of L2): one pass stores
//                    bfloat16(residual * norm_weight) and sums the squares in 32-bit; the row's
//                    scale 1 / sqrt(mean + eps) (src/operators.cpp:22-45) multiplies the 32-bit
//                    result, which is the same product because the scale is one number per row;
//           X_DIRECT x is bfloat16 [M, K] and is not staged in shared memory at all (a CTA that
//                    computes a single tile uses every element of x once);
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
enum { X_PLAIN = 0, X_NORM = 1, X_DIRECT = 2 };
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
  constexpr int UNROLL = (EPI == EPI_GATED || (XMODE == X_DIRECT && MT > 1)) ? 4 : 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                       // [MT * 8][x_stride]
  float* red = reinterpret_cast<float*>(smem_raw + (XMODE == X_DIRECT ? 0 : (size_t)MT * 8 * a.x_stride * 2));   // [warps][TILES][16][MT * 8 + 1]
  constexpr int kRedRow = MT * 8 + 1;
  __shared__ float row_scale[MT * 8];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int K = a.K;
  const int n_rows = (EPI == EPI_GATED) ? a.N / 2 : a.N;      // rows of one half
  const int tiles = (n_rows + 15) / 16;
  const int blocks = (K + 31) / 32;

  uint4 wreg[UNROLL][TILES][2];
  // this warp's weights of k blocks kb0, kb0 + 8, ... of the 16-row tile at n0
  auto issue = [&](int n0, int kb0) {
#pragma unroll
    for (int tile = 0; tile < TILES; ++tile) {
      const int base = tile * n_rows;
      const __nv_bfloat16* r0 = a.w + (size_t)(base + min(n0 + g, n_rows - 1)) * K + t * 8;
      const __nv_bfloat16* r1 = a.w + (size_t)(base + min(n0 + g + 8, n_rows - 1)) * K + t * 8;
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int kb = kb0 + u * kGemvWarps;
        const bool valid = kb * 32 + t * 8 < K;
        wreg[u][tile][0] = valid ? load_stream_16(r0 + (size_t)kb * 32) : make_uint4(0, 0, 0, 0);
        wreg[u][tile][1] = valid ? load_stream_16(r1 + (size_t)kb * 32) : make_uint4(0, 0, 0, 0);
      }
    }
  };

  // --- weights of the first round, before anything that depends on the previous kernel ---------
  issue(blockIdx.x * 16, warp);
  grid_launch_dependents();
  grid_dependency_wait();

  // --- stage x in shared memory as bfloat16, once per CTA ----------------------------------------
  // Shared memory is kept small on purpose: the weight loads in flight are tracked in L1, which shrinks as
  // shared memory grows, and with it the bandwidth a CTA can pull.
  if (XMODE == X_PLAIN) {
    const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(a.x);
    const int chunks = K / 8;
    for (int idx = threadIdx.x; idx < MT * 8 * chunks; idx += kGemvWarps * 32) {
      const int m = idx / chunks;
      const int c = idx - m * chunks;
      cp_async_16(xs + (size_t)m * a.x_stride + c * 8, x + (size_t)(m < a.M ? m : 0) * a.ldx + c * 8, m < a.M);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
  } else if (XMODE == X_NORM) {
    const float* residual = reinterpret_cast<const float*>(a.x);
    const int chunks = K / 4;
    constexpr int kBatch = 8;   // float4 per lane in flight
    for (int m = warp; m < MT * 8; m += kGemvWarps) {
      __nv_bfloat16* dst = xs + (size_t)m * a.x_stride;
      float sum = 0.0f;
      if (m < a.M) {
        const float* r = residual + (size_t)(a.rows ? a.rows[m] : m) * K;
        for (int c0 = lane; c0 < chunks; c0 += 32 * kBatch) {
          float4 v[kBatch];
#pragma unroll
          for (int i = 0; i < kBatch; ++i) {
            const int c = c0 + 32 * i;
            v[i] = c < chunks ? *reinterpret_cast<const float4*>(r + c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
#pragma unroll
          for (int i = 0; i < kBatch; ++i) {
            const int c = c0 + 32 * i;
            sum += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
            if (c < chunks) {
              const float4 nw = __ldg(reinterpret_cast<const float4*>(a.norm_weight + c * 4));   // every warp reads these: L1 hits
              *reinterpret_cast<uint2*>(dst + c * 4) = make_uint2(pack_bf16(v[i].x * nw.x, v[i].y * nw.y), pack_bf16(v[i].z * nw.z, v[i].w * nw.w));
            }
          }
        }
      } else {
        for (int c = lane; c < chunks; c += 32) *reinterpret_cast<uint2*>(dst + c * 4) = make_uint2(0, 0);
      }
      sum = warp_sum(sum);
      if (lane == 0) row_scale[m] = 1.0f / sqrtf(sum / (float)K + a.eps);
    }
    __syncthreads();
  }

  // --- tiles of 16 weight rows: blockIdx.x, + gridDim.x, ... -----------------------------------------
  for (int tile_index = blockIdx.x; tile_index < tiles; tile_index += gridDim.x) {
    const int n0 = tile_index * 16;
    float acc[TILES][MT][4];
#pragma unroll
    for (int tile = 0; tile < TILES; ++tile)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) acc[tile][mt][0] = acc[tile][mt][1] = acc[tile][mt][2] = acc[tile][mt][3] = 0.0f;

    for (int kb0 = warp; kb0 < blocks; kb0 += kGemvWarps * UNROLL) {
      if (kb0 != warp || tile_index != (int)blockIdx.x) issue(n0, kb0);
      uint4 xdirect[XMODE == X_DIRECT ? UNROLL : 1][MT];
      if (XMODE == X_DIRECT) {
        const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(a.x);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const int k = (kb0 + u * kGemvWarps) * 32 + t * 8;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const int m = mt * 8 + g;
            xdirect[u][mt] = (k < K && m < a.M) ? *reinterpret_cast<const uint4*>(x + (size_t)m * a.ldx + k) : make_uint4(0, 0, 0, 0);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int kb = kb0 + u * kGemvWarps;
        if (kb >= blocks) continue;          // the same for every lane: mma.sync needs the whole warp
        const int k = kb * 32 + t * 8;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          // lanes past K (a last block of fewer than 32) contribute zeros: their weights are zero too
          uint4 xv = make_uint4(0, 0, 0, 0);
          if (XMODE == X_DIRECT) {
            xv = xdirect[u][mt];
          } else if (k < K) {
            xv = *reinterpret_cast<const uint4*>(xs + (size_t)(mt * 8 + g) * a.x_stride + k);
          }
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

    // sum the warps' tiles, then the epilogue
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
        if (XMODE == X_NORM) sum[tile] *= row_scale[m];
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
    __syncthreads();   // red is written again by the next tile
  }
}

template <int MT, int XMODE, int EPI>
static int launch_one(const GemvArgs& a, int grid, cudaStream_t stream) {
  constexpr int TILES = (EPI == EPI_GATED) ? 2 : 1;
  const size_t smem = (XMODE == X_DIRECT ? 0 : (size_t)MT * 8 * a.x_stride * 2) + (size_t)kGemvWarps * TILES * 16 * (MT * 8 + 1) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemv_fused_kernel<MT, XMODE, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  return (int)launch_pdl(gemv_fused_kernel<MT, XMODE, EPI>, dim3(grid), dim3(kGemvWarps * 32), smem, stream, a);
}

template <int XMODE, int EPI>
static int launch_rows(const GemvArgs& a, cudaStream_t stream) {
  const int n_rows = (EPI == EPI_GATED) ? a.N / 2 : a.N;
  const int tiles = (n_rows + 15) / 16;
  // x is staged once per CTA, so a CTA takes several tiles when there are more than two CTAs per SM; equal shares
  const int per_cta = (tiles + 2 * 148 - 1) / (2 * 148);
  const int grid = (tiles + per_cta - 1) / per_cta;
  if (XMODE == X_PLAIN && per_cta == 1) {   // every element of x is used once per CTA: no point in staging it
    if (a.M <= 8) return launch_one<1, X_DIRECT, EPI>(a, grid, stream);
    if (a.M <= 16) return launch_one<2, X_DIRECT, EPI>(a, grid, stream);
    return (int)cudaErrorInvalidValue;
  }
  if (a.M <= 8) return launch_one<1, XMODE, EPI>(a, grid, stream);
  if (a.M <= 16) return launch_one<2, XMODE, EPI>(a, grid, stream);
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
