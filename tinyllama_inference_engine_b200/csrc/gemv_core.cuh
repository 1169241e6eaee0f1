// The weight-streaming product for up to 16 rows as building blocks: one struct per (rows, input, output) variant with
// the three steps a kernel strings together -- issue the weight loads of a round, stage x, run the tiles.  The stand-alone
// kernels (gemv_fused.cu) call them around a programmatic-dependency wait.  Activations another CTA may have written are read through L2 (ld.global.cg /
// cp.async.cg), never through a stale L1 line; weights are read-only and bypass L1.
#pragma once

#include "common.cuh"
#include "mma_utils.cuh"

namespace tlie {

constexpr int kGemvWarps = 8;       // warps of a CTA; the kernels that stream long rows without staging x take 16 (template parameter WARPS)
enum { X_PLAIN = 0, X_NORM = 1, X_DIRECT = 2, X_PREPARED = 3 };
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
  // ACCUM may prepare the norm that follows it: for the completed residual r it also stores bfloat16(r * prepare_weight)
  // and, per row and 16-column tile, the sum of r^2 (what X_NORM would work out again in every CTA of the next product)
  const float* prepare_weight;   // [N], or nullptr
  __nv_bfloat16* prepare_x;      // [M, N]
  float* prepare_squares;        // [M, tiles of 16 columns]
  // X_PREPARED: x is such a bfloat16 [M, K]; squares [M, square_tiles] are summed into the row's scale with eps
  const float* squares;
  int square_tiles;
};

__device__ __forceinline__ uint4 load_stream_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}


// x into shared memory as bfloat16 (nothing for X_DIRECT); ends with a block-wide barrier.  X_NORM stores
// bf16(residual * norm_weight) and leaves 1 / rms of each row in row_scale: the epilogue applies it.
// kBatch: 16-byte loads of the residual a lane has in flight (more: fewer dependent round trips, more registers).
template <int MT, int XMODE, int kBatch = 8, int WARPS = kGemvWarps>
__device__ __forceinline__ void gemv_stage_x(const GemvArgs& a, __nv_bfloat16* xs, float* row_scale) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = a.K;
  // --- stage x in shared memory as bfloat16, once per CTA ----------------------------------------
  // Shared memory is kept small on purpose: the weight loads in flight are tracked in L1, which shrinks as
  // shared memory grows, and with it the bandwidth a CTA can pull.
  if (XMODE == X_PLAIN || XMODE == X_PREPARED) {
    const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(a.x);
    const int chunks = K / 8;
    for (int idx = threadIdx.x; idx < MT * 8 * chunks; idx += WARPS * 32) {
      const int m = idx / chunks;
      const int c = idx - m * chunks;
      cp_async_16(xs + (size_t)m * a.x_stride + c * 8, x + (size_t)(m < a.M ? m : 0) * a.ldx + c * 8, m < a.M);
    }
    cp_async_commit();
    if (XMODE == X_PREPARED) {   // the rows' scales from the sums of squares the previous product left, while the copies fly
      for (int m = warp; m < MT * 8; m += WARPS) {
        float sum = 0.0f;
        if (m < a.M)
          for (int t = lane; t < a.square_tiles; t += 32) sum += __ldcg(a.squares + (size_t)m * a.square_tiles + t);
        sum = warp_sum(sum);
        if (lane == 0) row_scale[m] = 1.0f / sqrtf(sum / (float)K + a.eps);
      }
    }
    cp_async_wait<0>();
    __syncthreads();
  } else if (XMODE == X_NORM) {
    const float* residual = reinterpret_cast<const float*>(a.x);
    const int chunks = K / 4;
    for (int m = warp; m < MT * 8; m += WARPS) {
      __nv_bfloat16* dst = xs + (size_t)m * a.x_stride;
      float sum = 0.0f;
      if (m < a.M) {
        const float* r = residual + (size_t)(a.rows ? a.rows[m] : m) * K;
        for (int c0 = lane; c0 < chunks; c0 += 32 * kBatch) {
          float4 v[kBatch];
#pragma unroll
          for (int i = 0; i < kBatch; ++i) {
            const int c = c0 + 32 * i;
            v[i] = c < chunks ? __ldcg(reinterpret_cast<const float4*>(r + c * 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
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
}

// The end of a tile: the warps' partial tiles are summed through `red` ([warp][16][MT * 8 + 1] floats) and stored by the
// variant's epilogue.  acc[mt] is a warp's m16n8 accumulator (weight rows x activation rows).  A gated tile holds 8 gate
// rows in the upper half of the accumulator's rows and the 8 up rows of the same outputs in the lower half.
template <int MT, int XMODE, int EPI, int WARPS = kGemvWarps>
// prior, prior_weight (ACCUM): the residual element this thread will add to and the next norm's weight for its column, asked for
// before the k loop (gemv_epilogue_prefetch) so that the end of the tile does not wait for two trips to L2.
__device__ __forceinline__ void gemv_reduce_store(const GemvArgs& a, const float (&acc)[MT][4], float* red, const float* row_scale, int n0, float prior = 0.0f,
                                                  float prior_weight = 0.0f) {
  constexpr int kRedRow = MT * 8 + 1;
  constexpr int kTileRows = (EPI == EPI_GATED) ? 8 : 16;      // outputs of a tile
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n_rows = (EPI == EPI_GATED) ? a.N / 2 : a.N;
  float* base = red + (size_t)warp * 16 * kRedRow;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    base[g * kRedRow + mt * 8 + 2 * t] = acc[mt][0];
    base[g * kRedRow + mt * 8 + 2 * t + 1] = acc[mt][1];
    base[(g + 8) * kRedRow + mt * 8 + 2 * t] = acc[mt][2];
    base[(g + 8) * kRedRow + mt * 8 + 2 * t + 1] = acc[mt][3];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < kTileRows * MT * 8; idx += WARPS * 32) {   // whole warps: 16 * MT * 8 is 128 or 256
    const int m = idx / kTileRows;
    const int r = idx - m * kTileRows;
    const bool live = m < a.M && n0 + r < n_rows;
    float sum = 0.0f, second = 0.0f;
#pragma unroll
    for (int wi = 0; wi < WARPS; ++wi) {
      sum += red[(size_t)wi * 16 * kRedRow + r * kRedRow + m];
      if (EPI == EPI_GATED) second += red[(size_t)wi * 16 * kRedRow + (r + 8) * kRedRow + m];
    }
    if (XMODE == X_NORM || XMODE == X_PREPARED) {
      sum *= row_scale[m];
      second *= row_scale[m];
    }
    const size_t o = (size_t)m * n_rows + n0 + r;
    if (EPI == EPI_STORE_BF16) {
      if (live) reinterpret_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn(sum);
    } else if (EPI == EPI_STORE_F32) {
      if (live) reinterpret_cast<float*>(a.out)[o] = sum;
    } else if (EPI == EPI_ACCUM) {
      float value = 0.0f;
      if (live) {
        value = prior + sum;
        reinterpret_cast<float*>(a.out)[o] = value;
      }
      if (a.prepare_weight != nullptr) {   // the same for the whole block
        if (live) a.prepare_x[o] = __float2bfloat16_rn(value * prior_weight);
        float squares = value * value;     // zero where nothing lives; the 16 columns of a row are 16 neighbouring lanes
#pragma unroll
        for (int offset = 8; offset > 0; offset >>= 1) squares += __shfl_xor_sync(0xffffffffu, squares, offset);
        if (r == 0 && m < a.M) a.prepare_squares[(size_t)m * ((n_rows + 15) / 16) + n0 / 16] = squares;
      }
    } else if (live) {
      // gate and up are rounded to bfloat16 first, as when the product is stored and read back
      const float gate = __bfloat162float(__float2bfloat16_rn(sum));
      const float up = __bfloat162float(__float2bfloat16_rn(second));
      reinterpret_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn((gate / (1.0f + expf(-gate))) * up);
    }
  }
  __syncthreads();   // red is written again by the next tile
}

// A tile is 16 weight rows (the A operand of the MMA), or for GATED 8 gate rows and the 8 up rows N / 2 below them: the
// outputs of a gated tile are 8, so that the tiles of the widest product can be dealt evenly to the CTAs.  (Tiles of 8 rows
// with the other half of the MMA empty were tried for the down projection, 128 tiles of 16 x 5632: 11.1 us against 7.9 us.)
template <int MT, int XMODE, int EPI, int WARPS = kGemvWarps>
struct GemvPhase {
  static constexpr int kTileRows = (EPI == EPI_GATED) ? 8 : 16;
  static constexpr int UNROLL = 8;   // k blocks of 32 a thread holds in flight per round (four were tried for the 16-row direct kernels: slower)
  static constexpr int kRedRow = MT * 8 + 1;
  uint4 wreg[UNROLL][2];

  // Shared memory this variant needs: x as bfloat16 (unless read directly) and the warps' partial tiles.
  static __host__ __device__ size_t smem_bytes(int x_stride) {
    return (XMODE == X_DIRECT ? 0 : (size_t)MT * 8 * x_stride * 2) + (size_t)WARPS * 16 * kRedRow * sizeof(float);
  }
  static __device__ __forceinline__ float* red_of(unsigned char* smem, int x_stride) {
    return reinterpret_cast<float*>(smem + (XMODE == X_DIRECT ? 0 : (size_t)MT * 8 * x_stride * 2));
  }

  // this warp's weights of k blocks kb0, kb0 + 8, ... of the tile whose first output is n0
  __device__ __forceinline__ void issue(const GemvArgs& a, int n0, int kb0) {
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int K = a.K;
    const int n_rows = (EPI == EPI_GATED) ? a.N / 2 : a.N;
    // MMA rows g and g + 8: two weight rows 8 apart, or the gate row and the up row of output n0 + g
    const __nv_bfloat16* r0 = a.w + (size_t)min(n0 + g, n_rows - 1) * K + t * 8;
    const __nv_bfloat16* r1 = a.w + (size_t)(EPI == EPI_GATED ? n_rows + min(n0 + g, n_rows - 1) : min(n0 + g + 8, n_rows - 1)) * K + t * 8;
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int kb = kb0 + u * WARPS;
      const bool valid = kb * 32 + t * 8 < K;
      wreg[u][0] = valid ? load_stream_16(r0 + (size_t)kb * 32) : make_uint4(0, 0, 0, 0);
      wreg[u][1] = valid ? load_stream_16(r1 + (size_t)kb * 32) : make_uint4(0, 0, 0, 0);
    }
  }

  __device__ __forceinline__ void stage_x(const GemvArgs& a, __nv_bfloat16* xs, float* row_scale) { gemv_stage_x<MT, XMODE, 8, WARPS>(a, xs, row_scale); }

  // tiles first_tile, first_tile + tile_step, ...; the first round of the first tile is in wreg already if first_round_issued
  __device__ __forceinline__ void run(const GemvArgs& a, __nv_bfloat16* xs, float* red, const float* row_scale, int first_tile, int tile_step,
                                      bool first_round_issued) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int K = a.K;
    const int n_rows = (EPI == EPI_GATED) ? a.N / 2 : a.N;      // rows of one half
    const int tiles = (n_rows + kTileRows - 1) / kTileRows;
    const int blocks = (K + 31) / 32;
    bool issued = first_round_issued;
    for (int tile_index = first_tile; tile_index < tiles; tile_index += tile_step) {
      const int n0 = tile_index * kTileRows;
      float acc[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.0f;
      // what the end of the tile will add to (the epilogue gives a thread at most one output: the block is at least as wide as the tile)
      float prior = 0.0f, prior_weight = 0.0f;
      if (EPI == EPI_ACCUM && threadIdx.x < kTileRows * MT * 8) {
        static_assert(kTileRows * MT * 8 <= WARPS * 32, "one output per thread at most");
        const int m = threadIdx.x / kTileRows, r = threadIdx.x - m * kTileRows;
        if (m < a.M && n0 + r < n_rows) {
          prior = __ldcg(reinterpret_cast<const float*>(a.out) + (size_t)m * n_rows + n0 + r);
          if (a.prepare_weight != nullptr) prior_weight = __ldg(a.prepare_weight + n0 + r);
        }
      }

      for (int kb0 = warp; kb0 < blocks; kb0 += WARPS * UNROLL) {
        if (kb0 != warp || !issued) issue(a, n0, kb0);
        uint4 xdirect[XMODE == X_DIRECT ? UNROLL : 1][MT];
        if (XMODE == X_DIRECT) {
          const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(a.x);
#pragma unroll
          for (int u = 0; u < UNROLL; ++u) {
            const int k = (kb0 + u * WARPS) * 32 + t * 8;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const int m = mt * 8 + g;
              xdirect[u][mt] = (k < K && m < a.M) ? __ldcg(reinterpret_cast<const uint4*>(x + (size_t)m * a.ldx + k)) : make_uint4(0, 0, 0, 0);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const int kb = kb0 + u * WARPS;
          if (kb >= blocks) continue;          // the same for every lane: mma.sync needs the whole warp
          const int k = kb * 32 + t * 8;
          const unsigned lo[4] = {wreg[u][0].x, wreg[u][1].x, wreg[u][0].y, wreg[u][1].y};
          const unsigned hi[4] = {wreg[u][0].z, wreg[u][1].z, wreg[u][0].w, wreg[u][1].w};
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            // lanes past K (a last block of fewer than 32) contribute zeros: their weights are zero too
            uint4 xv = make_uint4(0, 0, 0, 0);
            if (XMODE == X_DIRECT) {
              xv = xdirect[u][mt];
            } else if (k < K) {
              xv = *reinterpret_cast<const uint4*>(xs + (size_t)(mt * 8 + g) * a.x_stride + k);
            }
            mma_bf16(acc[mt], lo, xv.x, xv.y);
            mma_bf16(acc[mt], hi, xv.z, xv.w);
          }
        }
      }
      // the weights of the next tile's first round go out before this tile is summed and stored.  (Refilling every slot of
      // wreg right after the MMAs that read it was tried: a warp then waits for its newest loads whenever it waits for an
      // old one, and the widest products took half as long again.)
      issued = tile_index + tile_step < tiles;
      if (issued) issue(a, (tile_index + tile_step) * kTileRows, warp);
      gemv_reduce_store<MT, XMODE, EPI, WARPS>(a, acc, red, row_scale, n0, prior, prior_weight);
    }
  }
};

// The shared-memory row stride of x for K columns: rows shifted by 64 bytes against each other, so that 16-byte reads of
// eight rows hit different banks.
__host__ __device__ inline int gemv_x_stride(int K) {
  int stride = K + ((32 - K % 64) + 64) % 64;
  if (stride == K) stride += 64;
  return stride;
}

}  // namespace tlie
