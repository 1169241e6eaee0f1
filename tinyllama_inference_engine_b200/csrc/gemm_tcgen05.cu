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
//   * four epilogue warps read the accumulator with tcgen05.ld (each warp its 32 lanes), convert, pack 32 columns of their
//     32 rows into shared memory and let one thread write the 32 x 32 box with a bulk tensor store (or add it into a
//     32-bit matrix with a bulk tensor reduction); where the output's shape rules that out, rows go straight from registers;
//   * the kernel is launched as a programmatic dependent: barriers and tensor memory are set up while the kernel before
//     it drains, global memory is touched only after the dependency wait.
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer, warp 2 = tensor-memory allocation (and epilogue),
// warps 2..5 = epilogue.  CTAs are persistent: one per SM walks the 128 x BN output tiles blockIdx.x, + gridDim.x, ...
// (m fastest, so the CTAs running together share a few column blocks of w in L2).  Two accumulators in tensor memory
// alternate between tiles, so the epilogue of one tile runs under the MMAs of the next.  TMA zero-fills out-of-range
// rows and k, the epilogue stores only what is inside [M, N].
// Every mbarrier wait is bounded: on a timeout the CTA raises `error_flag`, stops issuing work, lets copies in
// flight land, frees its tensor memory and returns.
#include "tcgen05_utils.cuh"

namespace tlie {

// BN: any multiple of 16 up to 256 (the N of one tcgen05.mma with M = 128), or a multiple of 32 up to 512 that two such
// instructions per 16 k fill, half each.  Widths between 128 and 256 exist for products whose tiles would otherwise fill one
// wave of CTAs and a sliver of a second one; widths beyond 256 for products that fit ONE wave so (2,048 x 2,560 is 160
// tiles of 256 columns, two waves on 148 SMs, and 144 tiles of 288): such a tile has all of tensor memory for its one
// accumulator, so nothing of its epilogue runs under a next tile's MMAs, and the host asks for it only when every CTA has one tile.
template <int BN, int EPI = 0>
struct GemmShape {
  static constexpr int kHalves = BN > 256 ? 2 : 1;   // MMAs per 16 k
  static constexpr int kMmaN = BN / kHalves;
  static constexpr int kStageBytes = (kBM + BN) * kBK * 2;
  // staging boxes of the epilogue's bulk stores (EPI 3: 32-bit boxes for bulk reductions): one per warp at least, two where
  // they fit beside the ring
  static constexpr int kBoxBytes = EPI == 3 ? kAddBoxBytes : kStoreBoxBytes;
  static constexpr int kRoom = 227 * 1024 - 1024 /* alignment slack */ - 256 /* barriers */;
  static constexpr int kFit = (kRoom - kStoreWarps * kBoxBytes) / kStageBytes;
  static constexpr int kStages = kFit < 6 ? kFit : 6;
  static constexpr int kStoreBuffers = (kStages * kStageBytes + kStoreWarps * 2 * kBoxBytes <= kRoom) ? 2 : 1;
  static constexpr int kStoreBytes = kStoreWarps * kStoreBuffers * kBoxBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + 1024 + 256;
  static constexpr int kAccStride = BN <= 128 ? 128 : BN <= 256 ? 256 : 512;   // tensor memory is allocated in powers of two
  static constexpr int kAccumulators = kAccStride <= 256 ? 2 : 1;
  static_assert(kMmaN % 16 == 0 && kMmaN >= 16 && kMmaN <= 256, "the N of a tcgen05.mma with M = 128");
  static_assert(kAccumulators * kAccStride <= 512, "the accumulators must fit the 512 columns of tensor memory");
  static_assert(EPI != 2 || kHalves == 1, "the gated tile is one instruction wide");
  static_assert(BN % kStoreCols == 0, "the epilogue hands the tile over in boxes of kStoreCols columns");
  static_assert(kStages >= 2 && kSmemBytes <= 227 * 1024, "shared memory of one CTA");
};

// EPI 0: bfloat16 out; EPI 1: 32-bit out; EPI 2 (BN = 256): w holds [gate rows | up rows] (`N` = rows of one half);
// the tile's B operand is 128 gate rows and the 128 up rows at the same offset, and the epilogue stores
// silu(gate) * up (src/operators.cpp:148-164) as bfloat16 [M, N]: the activation kernel and the round trip of the
// [M, 2N] intermediate through memory disappear.  EPI 3: out is the 32-bit residual stream and the tile is added to it by bulk
// tensor reductions (the add kernel and the round trip of the product through memory disappear).
template <int BN, int EPI>
__global__ void __launch_bounds__(kGemmThreads)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const __grid_constant__ CUtensorMap map_out, int staged, void* __restrict__ out, int M, int N, int K,
                        int* __restrict__ error_flag) {
  using Shape = GemmShape<BN, EPI>;
  constexpr int kStages = Shape::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzled tiles need 1024-byte alignment
  uint8_t* staging = tiles + kStages * Shape::kStageBytes;   // [4 warps][kStoreBuffers] boxes of the epilogue's bulk stores
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + Shape::kStoreBytes);
  uint64_t* empty = full + kStages;
  uint64_t* accum_full = empty + kStages;     // [2]: the MMAs of a tile are done
  uint64_t* accum_empty = accum_full + 2;      // [2]: the epilogue has read the accumulator
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(accum_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kTileN = EPI == 2 ? BN / 2 : BN;   // output columns of a tile
  constexpr int kAccumulators = Shape::kAccumulators;
  constexpr int kTmemCols = kAccumulators * Shape::kAccStride;
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
  // Programmatic dependent launch: the CTA is set up (barriers, tensor memory) while the kernel before it in the stream still
  // runs; nothing of global memory is touched before the wait, which returns when that kernel has completed.
  grid_launch_dependents();
  grid_dependency_wait();

  if (warp == 0) {
    if (lane == 0) {   // TMA producer: one ring of stages across all of this CTA's tiles
      RingPosition<kStages> ring;
      const uint32_t tiles_addr = smem_u32(tiles), full_addr = smem_u32(full), empty_addr = smem_u32(empty);
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % m_blocks) * kBM, n0 = (tile / m_blocks) * kTileN;
        for (int kb = 0; kb < k_blocks; ++kb, ring.advance()) {
          ok = mbar_wait(empty_addr + 8 * ring.stage, ring.phase ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t a_tile = tiles_addr + ring.stage * Shape::kStageBytes, b_tile = a_tile + kBM * kBK * 2;
          const uint32_t bar = full_addr + 8 * ring.stage;
          mbar_expect_tx(bar, Shape::kStageBytes);
          tma_load_2d(a_tile, &map_a, kb * kBK, m0, bar);
          if (EPI == 2) {
            tma_load_2d(b_tile, &map_b, kb * kBK, n0, bar);                                  // gate rows
            tma_load_2d(b_tile + (BN / 2) * kBK * 2, &map_b, kb * kBK, N + n0, bar);        // up rows
          } else {
#pragma unroll
            for (int h = 0; h < Shape::kHalves; ++h)   // rows past N are filled with zeros
              tma_load_2d(b_tile + h * Shape::kMmaN * kBK * 2, &map_b, kb * kBK, n0 + h * Shape::kMmaN, bar);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {   // MMA issuer
      constexpr uint32_t idesc = umma_instr_desc(kBM, Shape::kMmaN);
      RingPosition<kStages> ring;
      const uint32_t tiles_low = umma_desc_low(smem_u32(tiles)), full_addr = smem_u32(full), empty_addr = smem_u32(empty);
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local % kAccumulators;
        ok = mbar_wait(&accum_empty[acc], ((local / kAccumulators) & 1) ^ 1, abort_flag);   // the epilogue has drained this accumulator
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t tmem_acc = tmem_base + acc * Shape::kAccStride;
        for (int kb = 0; kb < k_blocks; ++kb, ring.advance()) {
          ok = mbar_wait(full_addr + 8 * ring.stage, ring.phase, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          // descriptors by their lower words, in 16-byte units: a stage further, then B behind A
          const uint32_t a_low = tiles_low + ring.stage * (Shape::kStageBytes >> 4), b_low = a_low + ((kBM * kBK * 2) >> 4);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            // 16 k = 32 bytes further inside the 128-byte swizzle span; the second half of a wide tile: kMmaN rows of B further, kMmaN columns on
#pragma unroll
            for (int h = 0; h < Shape::kHalves; ++h)
              umma_bf16(tmem_acc + h * Shape::kMmaN, a_low + k * ((kUmmaK * 2) >> 4), b_low + h * ((Shape::kMmaN * kBK * 2) >> 4) + k * ((kUmmaK * 2) >> 4), idesc,
                        (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty_addr + 8 * ring.stage);   // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(&accum_full[acc]);
      }
    }
  }
  if (warp >= 2) {   // epilogue: warp w reads tensor-memory lanes 32 * (w % 4) ... + 31
    const int sub = warp & 3;
    int local = 0, boxes = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local) {
      const int acc = local % kAccumulators;
      const int m0 = (tile % m_blocks) * kBM, n0 = (tile / m_blocks) * kTileN;
      if (!mbar_wait(&accum_full[acc], (local / kAccumulators) & 1, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t tmem_acc = tmem_base + acc * Shape::kAccStride + ((uint32_t)(sub * 32) << 16);
      const int row = m0 + sub * 32 + lane;
      if (EPI == 3) {
        add_tile_staged<BN, Shape::kStoreBuffers>(tmem_acc, m0 + sub * 32, n0, M, N, &map_out, staging + sub * Shape::kStoreBuffers * kAddBoxBytes, lane, boxes);
      } else if (EPI != 1 && staged) {
        store_tile_staged<BN, EPI, Shape::kStoreBuffers>(tmem_acc, m0 + sub * 32, n0, M, N, &map_out,
                                                         staging + sub * Shape::kStoreBuffers * kStoreBoxBytes, lane, boxes);
      } else {
        store_tile_direct<BN, EPI>(tmem_acc, row, n0, out, M, N);
      }
      // this warp is done with the accumulator: hand it back to the MMA issuer
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&accum_empty[acc])) : "memory");
    }
    if (lane == 0) bulk_wait_all();   // this warp's staging boxes have been read and written out
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  }
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicOr(error_flag, 1);
    // copies that were issued may still be landing in this CTA's shared memory: give them time before it is released
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols));
  }
}

template <int BN, int EPI>
static int launch_gemm(const void* x, const void* w, void* out, int M, int N, int K, int* error_flag, cudaStream_t stream) {
  CUtensorMap map_a, map_b, map_out;
  // EPI 2: w has 2 N rows, fetched as two boxes of BN / 2 rows; N is the width of the output
  if (!make_map(&map_a, x, M, K, kBM) || !make_map(&map_b, w, EPI == 2 ? 2 * N : N, K, EPI == 2 ? BN / 2 : GemmShape<BN, EPI>::kMmaN)) return (int)cudaErrorInvalidValue;
  if (EPI == 3 && !make_add_map(&map_out, out, M, N)) return (int)cudaErrorInvalidValue;
  const int staged = EPI == 3 || (EPI != 1 && make_store_map(&map_out, out, M, N)) ? 1 : 0;   // else rows are stored straight from registers
  if (!staged) map_out = map_a;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmShape<BN, EPI>::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  constexpr int kTileN = EPI == 2 ? BN / 2 : BN;
  const int num_tiles = ((N + kTileN - 1) / kTileN) * ((M + kBM - 1) / kBM);
  const int sm_count = device_sm_count();
  dim3 grid(num_tiles < sm_count ? num_tiles : sm_count);
  return (int)launch_pdl(gemm_tcgen05_kernel<BN, EPI>, grid, dim3(kGemmThreads), GemmShape<BN, EPI>::kSmemBytes, stream, map_a, map_b, map_out, staged, out, M, N, K,
                         error_flag);
}

}  // namespace tlie

using namespace tlie;

// out[M, N] = x[M, K] . w[N, K]^T.  x and w bfloat16 row-major with 16-byte aligned bases and K % 8 == 0 (TMA strides);
// out bfloat16 (out_f32 = 0), 32-bit (1), out_f32 = 2: w is [gate rows | up rows] of N rows each and out [M, N] = silu(gate) * up,
// or out_f32 = 3: out is 32-bit (16-byte aligned, N % 4 == 0) and the product is added to it.
// tile_n is 128, 160, 192, 256, 288 or 320.  `error_flag` (device int, zero) becomes 1 if a wait gave up.
TLIE_EXPORT int tlie_gemm_tcgen05(const void* x, const void* w, void* out, int M, int N, int K, int out_f32, int tile_n, int* error_flag,
                                  cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || error_flag == nullptr || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return (int)cudaErrorInvalidValue;
  if (out_f32 == 2) return launch_gemm<256, 2>(x, w, out, M, N, K, error_flag, stream);   // gated: N = rows of one half of w
  if (out_f32 == 3) return launch_gemm<256, 3>(x, w, out, M, N, K, error_flag, stream);   // out (32-bit) += the product
  if (tile_n == 320) {
    return out_f32 ? launch_gemm<320, 1>(x, w, out, M, N, K, error_flag, stream) : launch_gemm<320, 0>(x, w, out, M, N, K, error_flag, stream);
  }
  if (tile_n == 288) {
    return out_f32 ? launch_gemm<288, 1>(x, w, out, M, N, K, error_flag, stream) : launch_gemm<288, 0>(x, w, out, M, N, K, error_flag, stream);
  }

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
