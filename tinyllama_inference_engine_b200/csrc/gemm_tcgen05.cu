// Tensor-core matrix product for prompt portions: out[M, N] = x[M, K] . w[N, K]^T, bfloat16 in, 32-bit accumulate.
//
// The reference calls cuBLAS for every product (src/cuda/kernels.cu:342-368).  This is the engine's own kernel
// for the 5th-generation tensor cores of sm_100a:
//   * operands travel global -> shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), 64 k per stage,
//     through a ring of STAGES buffers guarded by full / empty mbarriers;
//   * one elected thread issues tcgen05.mma (128 x BN x 16 per instruction, four per stage); the accumulator
//     (128 lanes x BN 32-bit columns) lives in tensor memory, not in registers;
//   * tcgen05.commit hands a stage back to the TMA producer when its MMAs have read it, and signals the
//     epilogue when the last MMA is done;
//   * four epilogue warps read the accumulator with tcgen05.ld (each warp its 32 lanes), convert and store.
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer, warp 2 = tensor-memory allocation (and epilogue),
// warps 2..5 = epilogue.  CTAs are persistent: one per SM walks the 128 x BN output tiles blockIdx.x, + gridDim.x, ...
// (m fastest, so the CTAs running together share a few column blocks of w in L2).  Two accumulators in tensor memory
// alternate between tiles, so the epilogue of one tile runs under the MMAs of the next.  TMA zero-fills out-of-range
// rows and k, the epilogue stores only what is inside [M, N].
// Every mbarrier wait is bounded: on a timeout the CTA raises `error_flag`, stops issuing work, lets copies in
// flight land, frees its tensor memory and returns.
#include <cuda.h>

#include "common.cuh"

namespace tlie {

constexpr int kBM = 128;
constexpr int kBK = 64;                 // 64 bf16 = 128 bytes = one swizzle span
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;
constexpr long long kWaitLimit = 1ll << 20;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// Waits for the barrier's phase with a limit; false (and the CTA-wide abort flag set) when it gives up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (long long i = 0; i < kWaitLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(smem_u32(smem_dst)),
               "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
               : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_addr >> 4) & 0x3FFF);        // start address, 16-byte units
  desc |= (uint64_t)1 << 16;                            // leading byte offset (unused for swizzled K-major)
  desc |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset between 8-row groups
  desc |= (uint64_t)1 << 46;                            // descriptor version of sm_100
  desc |= (uint64_t)2 << 61;                            // layout: 128-byte swizzle
  return desc;
}

// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, tile M x N.
__host__ __device__ constexpr uint32_t umma_instr_desc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_load_16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

// BN: any multiple of 16 up to 256 (the N of one tcgen05.mma with M = 128).  Widths between 128 and 256 exist for products
// whose tiles would otherwise fill one wave of CTAs and a sliver of a second one.
template <int BN>
struct GemmShape {
  static constexpr int kStageBytes = (kBM + BN) * kBK * 2;
  static constexpr int kStages = (220 * 1024 / kStageBytes) < 6 ? (220 * 1024 / kStageBytes) : 6;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
  static constexpr int kAccStride = BN <= 128 ? 128 : 256;   // tensor memory is allocated in powers of two
  static_assert(BN % 16 == 0 && BN >= 16 && BN <= 256, "the N of a tcgen05.mma with M = 128");
  static_assert(2 * kAccStride <= 512, "two accumulators must fit the 512 columns of tensor memory");
};

// EPI 0: bfloat16 out; EPI 1: 32-bit out; EPI 2 (BN = 256): w holds [gate rows | up rows] (`N` = rows of one half);
// the tile's B operand is 128 gate rows and the 128 up rows at the same offset, and the epilogue stores
// silu(gate) * up (src/operators.cpp:148-164) as bfloat16 [M, N]: the activation kernel and the round trip of the
// [M, 2N] intermediate through memory disappear.
template <int BN, int EPI>
__global__ void __launch_bounds__(kGemmThreads)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, void* __restrict__ out, int M,
                        int N, int K, int* __restrict__ error_flag) {
  using Shape = GemmShape<BN>;
  constexpr int kStages = Shape::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzled tiles need 1024-byte alignment
  uint64_t* full = reinterpret_cast<uint64_t*>(tiles + kStages * Shape::kStageBytes);
  uint64_t* empty = full + kStages;
  uint64_t* accum_full = empty + kStages;     // [2]: the MMAs of a tile are done
  uint64_t* accum_empty = accum_full + 2;      // [2]: the epilogue has read the accumulator
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(accum_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kTileN = EPI == 2 ? BN / 2 : BN;   // output columns of a tile
  constexpr int kTmemCols = 2 * Shape::kAccStride;   // two accumulators
  const int m_blocks = (M + kBM - 1) / kBM;
  const int num_tiles = m_blocks * ((N + kTileN - 1) / kTileN);
  const int k_blocks = (K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&accum_full[a], 1);
      mbar_init(&accum_empty[a], 4);   // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 2) {   // the whole warp allocates BN columns of tensor memory and lets other CTAs allocate too
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_holder)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {   // TMA producer: one ring of stages across all of this CTA's tiles
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % m_blocks) * kBM, n0 = (tile / m_blocks) * kTileN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t phase = (it / kStages) & 1;
          ok = mbar_wait(&empty[s], phase ^ 1, abort_flag);
          if (!ok) break;
          uint8_t* a_tile = tiles + s * Shape::kStageBytes;
          uint8_t* b_tile = a_tile + kBM * kBK * 2;
          mbar_expect_tx(&full[s], Shape::kStageBytes);
          tma_load_2d(a_tile, &map_a, kb * kBK, m0, &full[s]);
          if (EPI == 2) {
            tma_load_2d(b_tile, &map_b, kb * kBK, n0, &full[s]);                                  // gate rows
            tma_load_2d(b_tile + (BN / 2) * kBK * 2, &map_b, kb * kBK, N + n0, &full[s]);        // up rows
          } else {
            tma_load_2d(b_tile, &map_b, kb * kBK, n0, &full[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {   // MMA issuer
      constexpr uint32_t idesc = umma_instr_desc(kBM, BN);
      int it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        ok = mbar_wait(&accum_empty[acc], ((local >> 1) & 1) ^ 1, abort_flag);   // the epilogue has drained this accumulator
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t tmem_acc = tmem_base + acc * Shape::kAccStride;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t phase = (it / kStages) & 1;
          ok = mbar_wait(&full[s], phase, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint32_t a_addr = smem_u32(tiles + s * Shape::kStageBytes);
          const uint32_t b_addr = a_addr + kBM * kBK * 2;
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            // 16 k = 32 bytes further inside the 128-byte swizzle span
            umma_bf16(tmem_acc, umma_smem_desc(a_addr + k * kUmmaK * 2), umma_smem_desc(b_addr + k * kUmmaK * 2), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);   // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(&accum_full[acc]);
      }
    }
  }
  if (warp >= 2) {   // epilogue: warp w reads tensor-memory lanes 32 * (w % 4) ... + 31
    const int sub = warp & 3;
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      const int m0 = (tile % m_blocks) * kBM, n0 = (tile / m_blocks) * kTileN;
      if (!mbar_wait(&accum_full[acc], (local >> 1) & 1, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t tmem_acc = tmem_base + acc * Shape::kAccStride + ((uint32_t)(sub * 32) << 16);
      const int row = m0 + sub * 32 + lane;
      if (EPI == 2) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t gate[16], up[16];
          tmem_load_16(tmem_acc + c * 16, gate);
          tmem_load_16(tmem_acc + BN / 2 + c * 16, up);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
          const int col = n0 + c * 16;
          if (row < M && col < N) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * N + col;
            float act[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              // gate and up are rounded to bfloat16 first, as when the product is stored and read back
              const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(gate[i])));
              const float u = __bfloat162float(__float2bfloat16_rn(__uint_as_float(up[i])));
              act[i] = (g / (1.0f + expf(-g))) * u;
            }
            if (col + 16 <= N && (N % 8) == 0) {
              uint32_t packed[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                __nv_bfloat162 p = __floats2bfloat162_rn(act[2 * i], act[2 * i + 1]);
                packed[i] = *reinterpret_cast<uint32_t*>(&p);
              }
              *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
              *reinterpret_cast<uint4*>(dst + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            } else {
              for (int i = 0; i < 16 && col + i < N; ++i) dst[i] = __float2bfloat16_rn(act[i]);
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 16; ++c) {
          uint32_t r[16];
          tmem_load_16(tmem_acc + c * 16, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
          const int col = n0 + c * 16;
          if (row < M && col < N) {
            if (EPI == 0) {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)row * N + col;
              if (col + 16 <= N && (N % 8) == 0) {
                uint32_t packed[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                  packed[i] = *reinterpret_cast<uint32_t*>(&p);
                }
                *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                *reinterpret_cast<uint4*>(dst + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
              } else {
                for (int i = 0; i < 16 && col + i < N; ++i) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
              }
            } else {
              float* dst = reinterpret_cast<float*>(out) + (size_t)row * N + col;
              for (int i = 0; i < 16 && col + i < N; ++i) dst[i] = __uint_as_float(r[i]);
            }
          }
        }
      }
      // this warp is done with the accumulator: hand it back to the MMA issuer
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&accum_empty[acc])) : "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  }
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(error_flag, 1);
    // copies that were issued may still be landing in this CTA's shared memory: give them time before it is released
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols));
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* found = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &found, cudaEnableDefault, &status) == cudaSuccess && status == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(found);
  }
  return fn;
}

// A [rows, K] bfloat16 row-major matrix as a 2-D tensor map with boxes of box_rows x 64 and 128-byte swizzle.
static bool make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int EPI>
static int launch_gemm(const void* x, const void* w, void* out, int M, int N, int K, int* error_flag, cudaStream_t stream) {
  CUtensorMap map_a, map_b;
  // EPI 2: w has 2 N rows, fetched as two boxes of BN / 2 rows; N is the width of the output
  if (!make_map(&map_a, x, M, K, kBM) || !make_map(&map_b, w, EPI == 2 ? 2 * N : N, K, EPI == 2 ? BN / 2 : BN)) return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmShape<BN>::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  constexpr int kTileN = EPI == 2 ? BN / 2 : BN;
  const int num_tiles = ((N + kTileN - 1) / kTileN) * ((M + kBM - 1) / kBM);
  static int sm_count = 0;
  if (sm_count == 0) {
    int device = 0;
    cudaGetDevice(&device);
    if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sm_count <= 0) sm_count = 148;
  }
  dim3 grid(num_tiles < sm_count ? num_tiles : sm_count);
  gemm_tcgen05_kernel<BN, EPI><<<grid, kGemmThreads, GemmShape<BN>::kSmemBytes, stream>>>(map_a, map_b, out, M, N, K, error_flag);
  return (int)cudaGetLastError();
}

}  // namespace tlie

using namespace tlie;

// out[M, N] = x[M, K] . w[N, K]^T.  x and w bfloat16 row-major with 16-byte aligned bases and K % 8 == 0 (TMA strides);
// out bfloat16 (out_f32 = 0), 32-bit (1), or out_f32 = 2: w is [gate rows | up rows] of N rows each and out [M, N] = silu(gate) * up.
// tile_n is 128, 160, 192 or 256.  `error_flag` (device int, zero) becomes 1 if a wait gave up.
TLIE_EXPORT int tlie_gemm_tcgen05(const void* x, const void* w, void* out, int M, int N, int K, int out_f32, int tile_n, int* error_flag,
                                  cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || error_flag == nullptr || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return (int)cudaErrorInvalidValue;
  if (out_f32 == 2) return launch_gemm<256, 2>(x, w, out, M, N, K, error_flag, stream);   // gated: N = rows of one half of w
  if (tile_n == 256) {
    return out_f32 ? launch_gemm<256, 1>(x, w, out, M, N, K, error_flag, stream) : launch_gemm<256, 0>(x, w, out, M, N, K, error_flag, stream);
  }
  if (tile_n == 192) {
    return out_f32 ? launch_gemm<192, 1>(x, w, out, M, N, K, error_flag, stream) : launch_gemm<192, 0>(x, w, out, M, N, K, error_flag, stream);
  }
  if (tile_n == 160) {
    return out_f32 ? launch_gemm<160, 1>(x, w, out, M, N, K, error_flag, stream) : launch_gemm<160, 0>(x, w, out, M, N, K, error_flag, stream);
  }
  if (tile_n == 128) {
    return out_f32 ? launch_gemm<128, 1>(x, w, out, M, N, K, error_flag, stream) : launch_gemm<128, 0>(x, w, out, M, N, K, error_flag, stream);
  }
  return (int)cudaErrorInvalidValue;
}
