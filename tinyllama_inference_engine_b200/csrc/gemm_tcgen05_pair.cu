// The tcgen05 product on pairs of SMs: out[M, N] = x[M, K] . w[N, K]^T, bfloat16 in, 32-bit accumulate.
//
// gemm_tcgen05.cu gives every CTA a 128 x BN tile and loads (128 + BN) x 64 elements per stage; at full tensor speed that
// asks more of the path from L2 to the SMs than it delivers, and the tensor pipe idles a third to a half of the time.
// Here two CTAs of a cluster share a 256 x BN tile (tcgen05.mma.cta_group::2): each loads its own 128 rows of x and only
// HALF of the BN rows of w, the MMA reads both halves out of both CTAs' shared memory, and each CTA's tensor memory
// receives its own 128 rows of the result.  A third less comes in per flop, and six stages fit where four did.
//   * rank 0 of the pair (the leader) issues every MMA; both CTAs run a TMA producer and four epilogue warps;
//   * both producers' copies complete on the LEADER's `full` barrier (the copy names it by its address in the pair's
//     shared window); the leader expects the bytes of both;
//   * tcgen05.commit arrives on the `empty` (stage read) and `accum_full` (tile done) barriers of both CTAs at once;
//   * the epilogue warps of both CTAs arrive on the leader's `accum_empty` barrier (eight arrivals).
// No copy is multicast: every CTA fetches what it needs itself.  Tiles: 256 rows x BN columns, pair p takes tiles
// p, p + pairs, ... (m fastest).  Every wait is bounded as in gemm_tcgen05.cu; the pair leaves together (cluster barrier).
#include "tcgen05_utils.cuh"

namespace tlie {

constexpr uint32_t kLeaderWindow = 0xFEFFFFFFu;   // a shared-memory address with the pair-rank bit cleared: the same offset in rank 0

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
  return rank;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// a tile load of this CTA into its own shared memory whose bytes are counted on the leader's barrier
// (shared-memory and barrier addresses are 32-bit addresses of this CTA's window)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(smem_dst),
               "l"(map), "r"(bar & kLeaderWindow), "r"(x), "r"(y)
               : "memory");
}
// descriptors given by their lower words (umma_desc_low)
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint32_t a_low, uint32_t b_low, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 da, db;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "mov.b64 da, {%1, %5};\n"
      "mov.b64 db, {%2, %5};\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(a_low), "r"(b_low), "r"(idesc), "r"(accumulate), "r"(kUmmaDescHigh)
      : "memory");
}
// arrives on the barrier at this offset in both CTAs of the pair when the MMAs issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n" ::"r"(bar), "h"(both)
               : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) { umma_commit_pair(smem_u32(bar)); }
__device__ __forceinline__ void arrive_at_leader(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(smem_u32(bar) & kLeaderWindow) : "memory");
}

// BN up to 256 is the N of one MMA; beyond that (up to 512, a multiple of 32) two MMAs per 16 k fill the tile, half each, and the one
// accumulator takes all of tensor memory: for products whose 256-wide tiles would be a wave and a half or two of the pairs and that
// fit ONE wave so (2,048 x 4,096: 128 tiles of 256 columns on 74 pairs, or 72 tiles of 480).  The host asks for such a width only
// when no pair gets a second tile, since nothing of a tile's epilogue could run under the next tile's MMAs.
template <int BN, int EPI = 0>
struct PairShape {
  static constexpr int kHalves = BN > 256 ? 2 : 1;   // MMAs per 16 k
  static constexpr int kMmaN = BN / kHalves;
  static constexpr int kStageBytes = (kBM + BN / 2) * kBK * 2;   // per CTA: its rows of x and its half of the rows of w
  // staging boxes of the epilogue's bulk stores (EPI 3: 32-bit boxes for bulk reductions): two per warp where they fit beside the
  // ring, else one
  static constexpr int kBoxBytes = EPI == 3 ? kAddBoxBytes : kStoreBoxBytes;
  // room for the ring: what is left beside alignment slack, barriers and the boxes (two per warp for the reductions, else one at least)
  static constexpr int kRing = 227 * 1024 - 1280 - kStoreWarps * (EPI == 3 ? 2 : 1) * kBoxBytes;
  static constexpr int kStages = (kRing / kStageBytes) < 8 ? (kRing / kStageBytes) : 8;
  static constexpr int kStoreBuffers = (kStages * kStageBytes + kStoreWarps * 2 * kBoxBytes + 1280 <= 227 * 1024) ? 2 : 1;
  static constexpr int kStoreBytes = kStoreWarps * kStoreBuffers * kBoxBytes;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + 1024 /* alignment slack */ + 256 /* barriers */;
  static_assert(kSmemBytes <= 227 * 1024, "shared memory of one CTA");
  static constexpr int kAccStride = BN <= 128 ? 128 : BN <= 256 ? 256 : 512;       // tensor memory is allocated in powers of two
  static constexpr int kAccumulators = kAccStride <= 256 ? 2 : 1;
  static_assert(kMmaN % 16 == 0 && kMmaN >= 32 && kMmaN <= 256, "N of an MMA is a multiple of 16, and each CTA holds half of its rows of w, in groups of 8");
  static_assert(BN % kStoreCols == 0, "the epilogue hands the tile over in boxes of kStoreCols columns");
  static_assert(EPI != 2 || kHalves == 1, "the gated tile is one instruction wide");
  static_assert(kStages >= 2, "a ring needs two stages");
};

// EPI as in gemm_tcgen05.cu: 0 bfloat16 out, 1 32-bit out, 2 (BN = 256) w = [gate rows | up rows] and out = silu(gate) * up,
// 3 the tile is added into the 32-bit `out` by bulk tensor reductions.
template <int BN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_out, int staged, void* __restrict__ out, int M, int N, int K,
                     int* __restrict__ error_flag) {
  using Shape = PairShape<BN, EPI>;
  constexpr int kStages = Shape::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzled tiles need 1024-byte alignment
  uint8_t* staging = tiles + kStages * Shape::kStageBytes;   // [4 warps][kStoreBuffers] boxes of the epilogue's bulk stores
  uint64_t* full = reinterpret_cast<uint64_t*>(staging + Shape::kStoreBytes);   // used in the leader only
  uint64_t* empty = full + kStages;
  uint64_t* accum_full = empty + kStages;      // [2]: the MMAs of a tile are done
  uint64_t* accum_empty = accum_full + 2;      // [2], used in the leader only: both CTAs' epilogues have read the accumulator
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(accum_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = (int)cluster_rank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  constexpr int kTileN = EPI == 2 ? BN / 2 : BN;   // output columns of a tile
  constexpr int kAccumulators = Shape::kAccumulators;
  constexpr int kTmemCols = kAccumulators * Shape::kAccStride;
  const int m_blocks = (M + 2 * kBM - 1) / (2 * kBM);
  const int num_tiles = m_blocks * ((N + kTileN - 1) / kTileN);
  const int k_blocks = (K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&accum_full[a], 1);
      mbar_init(&accum_empty[a], 8);   // one arrival per epilogue warp of either CTA
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 2) {   // the same warp of both CTAs allocates, for the pair
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_holder)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anything arrives on them
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;
  // Programmatic dependent launch: the CTA is set up (barriers, tensor memory) while the kernel before it in the stream still
  // runs; nothing of global memory is touched before the wait, which returns when that kernel has completed.
  grid_launch_dependents();
  grid_dependency_wait();

  if (warp == 0) {
    if (lane == 0) {   // TMA producer of this CTA: one ring of stages across all of the pair's tiles
      RingPosition<kStages> ring;
      const uint32_t tiles_addr = smem_u32(tiles), full_addr = smem_u32(full), empty_addr = smem_u32(empty);
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += pairs) {
        const int m0 = (tile % m_blocks) * 2 * kBM + rank * kBM, n0 = (tile / m_blocks) * kTileN;
        // this CTA's half of the rows of w of every MMA of the tile: rank 0 the first kMmaN / 2 (the gate rows if gated), rank 1 the rest (the up rows)
        const int w_row = EPI == 2 ? rank * N + n0 : n0 + rank * (Shape::kMmaN / 2);
        for (int kb = 0; kb < k_blocks; ++kb, ring.advance()) {
          ok = mbar_wait(empty_addr + 8 * ring.stage, ring.phase ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t a_tile = tiles_addr + ring.stage * Shape::kStageBytes, b_tile = a_tile + kBM * kBK * 2;
          const uint32_t bar = full_addr + 8 * ring.stage;
          if (rank == 0) mbar_expect_tx(bar, 2 * Shape::kStageBytes);   // this CTA's bytes and the peer's
          tma_load_2d_pair(a_tile, &map_a, kb * kBK, m0, bar);
#pragma unroll
          for (int h = 0; h < Shape::kHalves; ++h)   // rows past N are filled with zeros
            tma_load_2d_pair(b_tile + h * (Shape::kMmaN / 2) * kBK * 2, &map_b, kb * kBK, w_row + h * Shape::kMmaN, bar);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {   // MMA issuer of the pair
      constexpr uint32_t idesc = umma_instr_desc(2 * kBM, Shape::kMmaN);
      RingPosition<kStages> ring;
      const uint32_t tiles_low = umma_desc_low(smem_u32(tiles)), full_addr = smem_u32(full), empty_addr = smem_u32(empty);
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++local) {
        const int acc = local % kAccumulators;
        ok = mbar_wait(&accum_empty[acc], ((local / kAccumulators) & 1) ^ 1, abort_flag);   // both epilogues have drained this accumulator
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
            // the second half of a wide tile: this CTA's kMmaN / 2 rows of w further, kMmaN columns on
#pragma unroll
            for (int h = 0; h < Shape::kHalves; ++h)
              umma_bf16_pair(tmem_acc + h * Shape::kMmaN, a_low + k * ((kUmmaK * 2) >> 4), b_low + h * (((Shape::kMmaN / 2) * kBK * 2) >> 4) + k * ((kUmmaK * 2) >> 4), idesc,
                             (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(empty_addr + 8 * ring.stage);   // the stage is free in both CTAs once these MMAs have read it
        }
        if (ok) umma_commit_pair(&accum_full[acc]);
      }
    }
  }
  if (warp >= 2) {   // epilogue: warp w reads tensor-memory lanes 32 * (w % 4) ... + 31 of this CTA's 128 rows
    const int sub = warp & 3;
    int local = 0, boxes = 0;
    for (int tile = pair; tile < num_tiles; tile += pairs, ++local) {
      const int acc = local % kAccumulators;
      const int m0 = (tile % m_blocks) * 2 * kBM + rank * kBM, n0 = (tile / m_blocks) * kTileN;
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
      // this warp is done with the accumulator: tell the pair's MMA issuer
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      __syncwarp();
      if (lane == 0) arrive_at_leader(&accum_empty[acc]);
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
  cluster_sync_all();   // neither CTA leaves while the other may still read its shared memory or arrive on its barriers
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kTmemCols));
  }
}

template <int BN, int EPI>
static int launch_pair(const void* x, const void* w, void* out, int M, int N, int K, int* error_flag, cudaStream_t stream) {
  CUtensorMap map_a, map_b, map_out;
  // each CTA fetches boxes of 128 rows of x and BN / 2 rows of w (gated: w has 2 N rows, one CTA takes gate rows, the other up rows)
  if (!make_map(&map_a, x, M, K, kBM) || !make_map(&map_b, w, EPI == 2 ? 2 * N : N, K, PairShape<BN, EPI>::kMmaN / 2)) return (int)cudaErrorInvalidValue;
  if (EPI == 3 && !make_add_map(&map_out, out, M, N)) return (int)cudaErrorInvalidValue;
  const int staged = EPI == 3 || (EPI != 1 && make_store_map(&map_out, out, M, N)) ? 1 : 0;   // else rows are stored straight from registers
  if (!staged) map_out = map_a;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairShape<BN, EPI>::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  constexpr int kTileN = EPI == 2 ? BN / 2 : BN;
  const int num_tiles = ((N + kTileN - 1) / kTileN) * ((M + 2 * kBM - 1) / (2 * kBM));
  const int sm_count = device_sm_count();
  const int pairs = num_tiles < sm_count / 2 ? num_tiles : sm_count / 2;
  return (int)launch_pdl(gemm_pair_kernel<BN, EPI>, dim3(2 * pairs), dim3(kGemmThreads), PairShape<BN, EPI>::kSmemBytes, stream, map_a, map_b, map_out, staged, out,
                         M, N, K, error_flag);
}

}  // namespace tlie

using namespace tlie;

// As tlie_gemm_tcgen05 (gemm_tcgen05.cu), on pairs of SMs; tile_n is 128, 160, 192, 256, or 288, 384 or 480 (two MMAs wide, one accumulator);
// adding into a 32-bit out (out_f32 = 3): 256, 384 or 480.
TLIE_EXPORT int tlie_gemm_tcgen05_pair(const void* x, const void* w, void* out, int M, int N, int K, int out_f32, int tile_n, int* error_flag,
                                       cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || error_flag == nullptr || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return (int)cudaErrorInvalidValue;
  if (out_f32 == 2) return launch_pair<256, 2>(x, w, out, M, N, K, error_flag, stream);   // gated: N = rows of one half of w
  if (out_f32 == 3) {   // out (32-bit, 16-byte aligned, N % 4 == 0) += the product
    if (tile_n == 480) return launch_pair<480, 3>(x, w, out, M, N, K, error_flag, stream);
    if (tile_n == 384) return launch_pair<384, 3>(x, w, out, M, N, K, error_flag, stream);
    return launch_pair<256, 3>(x, w, out, M, N, K, error_flag, stream);
  }
  if (tile_n == 480) return out_f32 ? launch_pair<480, 1>(x, w, out, M, N, K, error_flag, stream) : launch_pair<480, 0>(x, w, out, M, N, K, error_flag, stream);
  if (tile_n == 384) return out_f32 ? launch_pair<384, 1>(x, w, out, M, N, K, error_flag, stream) : launch_pair<384, 0>(x, w, out, M, N, K, error_flag, stream);
  if (tile_n == 288) return out_f32 ? launch_pair<288, 1>(x, w, out, M, N, K, error_flag, stream) : launch_pair<288, 0>(x, w, out, M, N, K, error_flag, stream);
  if (tile_n == 256) return out_f32 ? launch_pair<256, 1>(x, w, out, M, N, K, error_flag, stream) : launch_pair<256, 0>(x, w, out, M, N, K, error_flag, stream);
  if (tile_n == 192) return out_f32 ? launch_pair<192, 1>(x, w, out, M, N, K, error_flag, stream) : launch_pair<192, 0>(x, w, out, M, N, K, error_flag, stream);
  if (tile_n == 160) return out_f32 ? launch_pair<160, 1>(x, w, out, M, N, K, error_flag, stream) : launch_pair<160, 0>(x, w, out, M, N, K, error_flag, stream);
  if (tile_n == 128) return out_f32 ? launch_pair<128, 1>(x, w, out, M, N, K, error_flag, stream) : launch_pair<128, 0>(x, w, out, M, N, K, error_flag, stream);
  return (int)cudaErrorInvalidValue;
}
