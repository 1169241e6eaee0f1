// What the tcgen05 products share: mbarrier waits with a limit, TMA tile loads, shared-memory and instruction descriptors,
// the MMA / commit / tensor-memory load instructions, and the host side's tensor maps.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace tlie {

constexpr int kBM = 128;
constexpr int kBK = 64;                 // 64 bf16 = 128 bytes = one swizzle span
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;
constexpr uint32_t kWaitLimit = 1u << 20;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
// Barriers are named by pointer or by their 32-bit shared-memory address; the one-thread roles (TMA producer, MMA issuer) use
// the address form and a running ring position, so that a lone thread spends its time on few dependent instructions.
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) { mbar_expect_tx(smem_u32(bar), bytes); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) { return mbar_try_wait(smem_u32(bar), parity); }
// Waits for the barrier's phase with a limit; false (and the CTA-wide abort flag set) when it gives up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) { return mbar_wait(smem_u32(bar), parity, abort_flag); }

// Position in a ring of STAGES buffers: the stage and the phase bit of its barriers, advanced without a division.
template <int STAGES>
struct RingPosition {
  uint32_t stage = 0, phase = 0;
  __device__ __forceinline__ void advance() {
    if (++stage == STAGES) {
      stage = 0;
      phase ^= 1;
    }
  }
};

__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(smem_dst), "l"(map),
               "r"(bar), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  tma_load_2d(smem_u32(smem_dst), map, x, y, smem_u32(bar));
}

// Shared-memory matrix descriptor of a K-major tile with the 128-byte swizzle and 8-row groups 1024 bytes apart: start
// address in 16-byte units (bits 0-13), leading byte offset (bits 16-29, unused for swizzled K-major: 1), stride byte offset
// between 8-row groups (bits 32-45), descriptor version of sm_100 (bit 46), layout 128-byte swizzle (bits 61-63 = 2).
// It is kept in halves: the upper word is a constant and the lower one holds the address, so that the one issuing thread
// adds 2 per 32 bytes (16 k inside the swizzle span) or a stage's size in 16-byte units instead of building descriptors.
constexpr uint32_t kUmmaDescHigh = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t umma_desc_low(uint32_t smem_addr) { return ((smem_addr >> 4) & 0x3FFF) | (1u << 16); }

// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, tile M x N.
__host__ __device__ constexpr uint32_t umma_instr_desc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// descriptors given by their lower words (umma_desc_low)
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint32_t a_low, uint32_t b_low, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 da, db;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "mov.b64 da, {%1, %5};\n"
      "mov.b64 db, {%2, %5};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(a_low), "r"(b_low), "r"(idesc), "r"(accumulate), "r"(kUmmaDescHigh)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) { umma_commit(smem_u32(bar)); }
__device__ __forceinline__ void tmem_load_16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

// 32 consecutive 32-bit columns of this thread's lane of tensor memory (no wait).
__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, "
      "%22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
        "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

// --- the epilogue of the products: one warp's 32 rows of an accumulator tile to global memory ---------------------
// A thread owns one row of the accumulator (its lane of tensor memory).  Written straight from registers, a warp's store
// instruction touches 32 different rows, 16 bytes each: 32 memory transactions for 512 bytes.  The staged way packs 32
// columns (64 bytes of bfloat16) per row into shared memory in the 64-byte swizzle and one bulk tensor store writes the
// 32 x 32 box; rows and columns past the matrix are clipped by the tensor map.
constexpr int kStoreCols = 32;
constexpr int kStoreBoxBytes = 32 * kStoreCols * 2;   // 32 rows x 64 bytes
constexpr int kStoreWarps = 4;

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];\n" ::"l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
template <int PENDING>
__device__ __forceinline__ void bulk_wait_read() {   // all but the PENDING newest bulk stores of this thread have read their shared memory
  asm volatile("cp.async.bulk.wait_group.read %0;\n" ::"n"(PENDING) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;\n" ::: "memory"); }

__device__ __forceinline__ float silu_gated(uint32_t gate_bits, uint32_t up_bits) {
  // gate and up are rounded to bfloat16 first, as when the product is stored and read back (src/operators.cpp:148-164)
  const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(gate_bits)));
  const float u = __bfloat162float(__float2bfloat16_rn(__uint_as_float(up_bits)));
  return (g / (1.0f + expf(-g))) * u;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&p);
}

// Staged: EPI 0 (bfloat16 out) or 2 (gated).  tmem_acc: the accumulator with this warp's lane offset; row0: the warp's first
// row; n0: the tile's first output column; staging: this warp's BUFFERS boxes (1024-byte aligned); boxes: running count.
template <int BN, int EPI, int BUFFERS>
__device__ __forceinline__ void store_tile_staged(uint32_t tmem_acc, int row0, int n0, int M, int N, const CUtensorMap* map_out, uint8_t* staging,
                                                  int lane, int& boxes) {
  constexpr int kOutCols = EPI == 2 ? BN / 2 : BN;
  const int swizzle = (lane >> 1) & 3;   // 64-byte swizzle: 16-byte chunk j of row r lies at chunk j ^ ((r / 2) % 4)
  if (row0 >= M) return;   // nothing of this warp's rows is inside the matrix
  // Only boxes that reach into the matrix are staged: a box is handed over with every pass, which is what the wait before
  // the next pass over the same buffer counts on.
#pragma unroll 1
  for (int c = 0; c < kOutCols / kStoreCols && n0 + c * kStoreCols < N; ++c) {
    uint32_t packed[kStoreCols / 2];
    if (EPI == 2) {
      uint32_t gate[32], up[32];
      tmem_load_32(tmem_acc + c * kStoreCols, gate);
      tmem_load_32(tmem_acc + BN / 2 + c * kStoreCols, up);
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
      for (int i = 0; i < kStoreCols / 2; ++i) packed[i] = pack_bf16(silu_gated(gate[2 * i], up[2 * i]), silu_gated(gate[2 * i + 1], up[2 * i + 1]));
    } else {
      uint32_t r[32];
      tmem_load_32(tmem_acc + c * kStoreCols, r);
      asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
      for (int i = 0; i < kStoreCols / 2; ++i) packed[i] = pack_bf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
    }
    uint8_t* box = staging + (boxes % BUFFERS) * kStoreBoxBytes;
    ++boxes;
    if (lane == 0) bulk_wait_read<BUFFERS - 1>();   // the store that last read this box is done with it
    __syncwarp();
    uint8_t* my_row = box + lane * (kStoreCols * 2);
#pragma unroll
    for (int j = 0; j < kStoreCols / 8; ++j)
      *reinterpret_cast<uint4*>(my_row + ((j ^ swizzle) << 4)) = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic-proxy writes -> visible to the bulk store
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(map_out, box, n0 + c * kStoreCols, row0);
      asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
    }
  }
}

// out (32-bit) += the tile: 32 columns of the warp's 32 rows as 32-bit values into shared memory (128-byte rows, 128-byte swizzle)
// and one bulk tensor reduction (add) per box.  Every element of out belongs to one tile, so it is added to exactly once: the
// sum does not depend on any order.  This is the reference's add kernel (src/cuda/kernels.cu:208-215) inside the product.
constexpr int kAddBoxBytes = 32 * kStoreCols * 4;
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];\n" ::"l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
template <int BN, int BUFFERS>
__device__ __forceinline__ void add_tile_staged(uint32_t tmem_acc, int row0, int n0, int M, int N, const CUtensorMap* map_out, uint8_t* staging, int lane,
                                                int& boxes) {
  const int swizzle = lane & 7;   // 128-byte swizzle: 16-byte chunk j of row r lies at chunk j ^ (r % 8)
  if (row0 >= M) return;
#pragma unroll 1
  for (int c = 0; c < BN / kStoreCols && n0 + c * kStoreCols < N; ++c) {   // as above: every pass hands a box over
    uint32_t r[32];
    tmem_load_32(tmem_acc + c * kStoreCols, r);
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
    uint8_t* box = staging + (boxes % BUFFERS) * kAddBoxBytes;
    ++boxes;
    if (lane == 0) bulk_wait_read<BUFFERS - 1>();   // the reduction that last read this box is done with it
    __syncwarp();
    uint8_t* my_row = box + lane * (kStoreCols * 4);
#pragma unroll
    for (int j = 0; j < kStoreCols / 4; ++j) *reinterpret_cast<uint4*>(my_row + ((j ^ swizzle) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    __syncwarp();
    if (lane == 0) {
      tma_reduce_add_2d(map_out, box, n0 + c * kStoreCols, row0);
      asm volatile("cp.async.bulk.commit_group;\n" ::: "memory");
    }
  }
}

// Straight from registers: any N, bfloat16 or 32-bit out.
template <int BN, int EPI>
__device__ __forceinline__ void store_tile_direct(uint32_t tmem_acc, int row, int n0, void* out, int M, int N) {
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
        for (int i = 0; i < 16 && col + i < N; ++i) dst[i] = __float2bfloat16_rn(silu_gated(gate[i], up[i]));
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
          for (int i = 0; i < 16 && col + i < N; ++i) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
        } else {
          float* dst = reinterpret_cast<float*>(out) + (size_t)row * N + col;
          if (col + 16 <= N && (N % 4) == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<uint4*>(dst + 4 * i) = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
          } else {
            for (int i = 0; i < 16 && col + i < N; ++i) dst[i] = __uint_as_float(r[i]);
          }
        }
      }
    }
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

// out [M, N] bfloat16 row-major as a 2-D tensor map with boxes of 32 rows x 32 columns and 64-byte swizzle (for stores).
// Needs a 16-byte aligned base and N % 8 == 0 (the row stride in bytes must be a multiple of 16).
static bool make_store_map(CUtensorMap* map, const void* base, int M, int N) {
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr || ((uintptr_t)base & 15) || N % 8 != 0) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)N * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kStoreCols, 32};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// out [M, N] 32-bit row-major with boxes of 32 rows x 32 columns (128 bytes) and 128-byte swizzle, for reductions into it.
// Needs a 16-byte aligned base and N % 4 == 0.
static bool make_add_map(CUtensorMap* map, const void* base, int M, int N) {
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr || ((uintptr_t)base & 15) || N % 4 != 0) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)N * 4};
  const cuuint32_t box[2] = {(cuuint32_t)kStoreCols, 32};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tlie
