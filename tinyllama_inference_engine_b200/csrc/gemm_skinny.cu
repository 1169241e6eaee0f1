// Weight-streaming tensor-core product for steps of 17 to 128 rows: out[M, N] (+)= f(x[M, K] . w[N, K]^T), bfloat16 in.
//
// Decode steps of 32 or 64 requests (and small mixed steps) have too many rows for the register-fed kernels of
// gemv_fused.cu and too few for the persistent 128-row tiles of gemm_tcgen05.cu.  The reference sends every product to
// cuBLAS (src/cuda/kernels.cu:342-368).  Such a product is bound by reading w once, so this kernel is built around the
// weight stream:
//   * the step's rows (padded by the hardware to the 128 rows of a tcgen05.mma) are the A operand and BN = 256 (128 for more
//     than 64 rows) rows of w the B operand; the accumulator is 128 lanes x BN columns of tensor memory.  (With the
//     operands swapped, 128 weight rows as A and the rows as a narrow B, four times the MMAs are issued for the same weight
//     bytes; each cost the issuing thread's k loop about as long as a wide one, and that thread, not HBM, set the pace:
//     measured 0.3 us per 16 KB.)
//   * the weights are read from a packed copy made once per matrix (tlie_gemm_skinny_pack): block (128-row group, k block)
//     is the 16 KB image of a 128 x 64 operand tile exactly as tcgen05.mma wants it in shared memory (K-major, 128-byte
//     swizzle), so a stage is one or two contiguous bulk copies;
//   * a matrix has few such tiles (10 for 2560 rows), so K is cut into S parts and the S CTAs of a tile form a thread-block
//     cluster.  Each streams its k range through a ring of stages (the weights of the first stages are requested before
//     the programmatic-dependency wait), then the partial accumulators meet in distributed shared memory: CTA r of the
//     cluster receives, from every CTA, the columns it is to finish (16-byte stores straight from the registers the
//     accumulator was read into, a warp's store being 512 contiguous bytes at the receiver), adds the S parts in rank order
//     (a fixed order: the result does not depend on timing) and runs the epilogue for them.  No global scratch memory, no
//     atomics, no second kernel.  (Laying the part out in the CTA's own shared memory and sending it with one bulk copy per
//     receiver, completing on the receiver's mbarrier, measured 1 us slower per product: the exchange is bound by what the
//     SM-to-SM network moves, 64 KB per CTA in about 2 us, not by how it is issued.)
//   * epilogues: store (bfloat16 or 32-bit), gated (a 128-row group of the packed copy is 64 gate rows + the 64 up rows of the
//     same outputs; the epilogue stores silu(gate) * up, src/operators.cpp:148-164), accumulate (residual[m, n] += result in
//     32-bit, the reference's add kernel, src/cuda/kernels.cu:208-215), optionally leaving bfloat16(residual * norm weight)
//     and partial sums of squares of the rows for the product after it ("prepared norm");
//   * a product fed with such a prepared norm multiplies every result by its row's 1 / sqrt(mean + eps)
//     (src/operators.cpp:22-45) in the epilogue.
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..9 = epilogue (warp 2 allocates tensor memory).
// Every mbarrier wait is bounded; a CTA that gives up raises `error_flag` and still takes part in the cluster barrier.
#include "tcgen05_utils.cuh"

namespace tlie {

constexpr int kSkinnyThreads = 320;
constexpr int kSkinnyMaxSplit = 8;   // portable cluster size

enum SkinnyEpilogue { SKINNY_BF16 = 0, SKINNY_F32 = 1, SKINNY_GATED = 2, SKINNY_ACCUM = 3 };

struct SkinnyArgs {
  void* out;                       // bf16 / f32 [M, n_out] or the 32-bit residual
  int M, N, K;                     // N: rows of w (both halves for gated)
  int n_out;                       // output columns: N, or N / 2 for gated
  int split, kb_per;               // cluster size and k blocks per CTA
  int stages;
  int slice;                       // columns of every 64-column piece of the tile that one CTA finishes (a multiple of 4)
  const float* squares_in;         // prepared input: [M, tiles_in] (row stride squares_in_stride) partial sums of squares, or null
  int tiles_in, squares_in_stride;
  float eps;
  const float* prepare_weight;     // accumulate only: norm weight [N] of the norm that reads the residual next, or null
  __nv_bfloat16* prepare_x;        // [M, N] bfloat16(residual * prepare_weight)
  float* prepare_squares;          // [M, prepare_stride]: partial sums of squares, one per (tile, CTA, warp's run of columns)
  int prepare_stride;
  int* error_flag;
  long long* timeline;             // diagnostics: clock64 stamps of CTA 0's phases, or null
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(smem_addr), "r"(rank));
  return remote;
}
// global -> shared bulk copy (no tensor map): both addresses 16-byte aligned, a multiple of 16 bytes
__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(smem_dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all() {
  cluster_arrive();
  cluster_wait();
}

// MROWS: rows of x a stage brings (32, 64 or 128).  BN: weight rows of a tile.
template <int MROWS>
struct SkinnyShape {
  static constexpr int kBN = MROWS > 64 ? 128 : 256;
  static constexpr int kPieces = kBN / 64;                        // the tile's columns in runs of 64: a CTA finishes `slice` columns of each
  static constexpr int kBytesX = MROWS * kBK * 2, kBytesW = kBN * kBK * 2;
  static constexpr int kStageBytes = kBytesX + kBytesW;
  static constexpr int kControlBytes = 1024;                      // barriers, tensor-memory address, row scales
  static constexpr int kTailBytes = 0;                            // the MMA reads 128 rows (16 KB) of A from a stage's start: a stage is never smaller than that
  static_assert(kStageBytes >= kBM * kBK * 2, "the A operand's 128 rows must lie inside the stage");
  static constexpr int slice_of(int split) { return (((64 + split - 1) / split) + 3) & ~3; }
  // The parts a CTA receives: [sender][group of 4 columns][MROWS + 1] float4.  A warp of a sender holds 32 consecutive rows, so
  // its store of one group is 512 contiguous bytes at the receiver (16-byte pieces scattered over a row-major buffer took
  // 5 us per 64 KB); the odd row count keeps the receiver's reads, which walk a row's groups, off each other's banks.
  static constexpr int kGroupStride = MROWS + 1;                  // float4 per group
  static constexpr int groups_of(int split) { return kPieces * (slice_of(split) >> 2); }
  static constexpr int part_bytes(int split) { return split * groups_of(split) * kGroupStride * 16; }
  static constexpr int fixed_bytes(int split) { return part_bytes(split) + 1024 /* alignment */ + kControlBytes + kTailBytes; }
  static constexpr int max_stages(int split, int budget) {
    return (budget - fixed_bytes(split)) / kStageBytes < 8 ? (budget - fixed_bytes(split)) / kStageBytes : 8;
  }
};

template <int MROWS, int EPI>
__global__ void __launch_bounds__(kSkinnyThreads)
    gemm_skinny_kernel(const __nv_bfloat16* __restrict__ packed_w, const __grid_constant__ CUtensorMap map_x, const SkinnyArgs a) {
  using Shape = SkinnyShape<MROWS>;
  constexpr int kBN = Shape::kBN, kPieces = Shape::kPieces;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int split = a.split, stages = a.stages, slice = a.slice;
  const int runs = slice >> 2;                                     // groups of 4 columns per 64-column piece that one CTA finishes
  const int groups = kPieces * runs;                               // per sender
  float4* parts = reinterpret_cast<float4*>(tiles + stages * Shape::kStageBytes + Shape::kTailBytes);   // [split][groups][MROWS + 1]
  uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(parts) + split * groups * Shape::kGroupStride * 16);
  uint64_t* empty = full + 8;
  uint64_t* accum_full = empty + 8;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(accum_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
  float* row_scale = reinterpret_cast<float*>(tmem_holder + 4);    // [MROWS <= 128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int tile = blockIdx.x / split;
  const int k_blocks = (a.K + kBK - 1) / kBK;
  const int kb_begin = min(k_blocks, (int)rank * a.kb_per), kb_end = min(k_blocks, kb_begin + a.kb_per);
  const int my_blocks = kb_end - kb_begin;
  auto stamp = [&](int slot) {
    if (a.timeline != nullptr && blockIdx.x == 0) a.timeline[slot] = clock64();
  };
  if (threadIdx.x == 0) stamp(0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_holder)), "r"(kBN));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;
  grid_launch_dependents();
  if (threadIdx.x == 0) stamp(1);

  // The two one-thread roles run a handful of dependent instructions per k block: running addresses and ring positions, no
  // divisions, nothing recomputed (a lone thread issues an instruction every few cycles; forty of them were 0.4 us per block).
  if (warp == 0) {
    if (lane == 0) {   // TMA producer
      const uint32_t tiles_addr = smem_u32(tiles), full_addr = smem_u32(full), empty_addr = smem_u32(empty);
      // the tile's first 128-row group at this CTA's first k block; the second group (BN = 256) lies k_blocks blocks further
      const __nv_bfloat16* next_w = packed_w + ((size_t)tile * (kBN / 128) * k_blocks + kb_begin) * (kBM * kBK);
      const size_t second = (size_t)k_blocks * (kBM * kBK);
      auto load_w = [&](uint32_t dst, uint32_t bar) {
        bulk_load(dst, next_w, kBM * kBK * 2, bar);
        if (kBN == 256) bulk_load(dst + kBM * kBK * 2, next_w + second, kBM * kBK * 2, bar);
      };
      // the weights of the first stages do not depend on the kernel before this one: they are requested before the wait
      const int ahead = my_blocks < stages ? my_blocks : stages;
      for (int i = 0; i < ahead; ++i, next_w += kBM * kBK) {
        mbar_expect_tx(full_addr + 8 * i, Shape::kStageBytes);
        load_w(tiles_addr + i * Shape::kStageBytes + Shape::kBytesX, full_addr + 8 * i);
      }
      grid_dependency_wait();
      stamp(2);
      int x_k = kb_begin * kBK;
      for (int i = 0; i < ahead; ++i, x_k += kBK) tma_load_2d(tiles_addr + i * Shape::kStageBytes, &map_x, x_k, 0, full_addr + 8 * i);
      uint32_t stage = 0, parity = 0;   // block `ahead` reuses stage 0 once the MMAs of its first use have read it (phase 0 of `empty`)
      for (int i = ahead; i < my_blocks; ++i, next_w += kBM * kBK, x_k += kBK) {
        if (!mbar_wait(empty_addr + 8 * stage, parity, abort_flag)) break;
        const uint32_t dst = tiles_addr + stage * Shape::kStageBytes, bar = full_addr + 8 * stage;
        mbar_expect_tx(bar, Shape::kStageBytes);
        load_w(dst + Shape::kBytesX, bar);
        tma_load_2d(dst, &map_x, x_k, 0, bar);
        if (++stage == (uint32_t)stages) {
          stage = 0;
          parity ^= 1;
        }
      }
    } else {
      grid_dependency_wait();
    }
  } else if (warp == 1) {
    grid_dependency_wait();
    if (lane == 0 && my_blocks > 0) {   // MMA issuer
      // A: 128 rows from the stage's start.  Only MROWS of them were loaded; the rows behind (the stage's own weights) give
      // accumulator lanes nobody reads: a row of the result depends on its own row of A alone.
      constexpr uint32_t idesc = umma_instr_desc(kBM, kBN);
      const uint32_t full_addr = smem_u32(full), empty_addr = smem_u32(empty);
      const uint32_t first_low = umma_desc_low(smem_u32(tiles));
      uint32_t stage = 0, parity = 0, a_low = first_low;
      bool ok = true;
      for (int i = 0; i < my_blocks; ++i) {
        ok = mbar_wait(full_addr + 8 * stage, parity, abort_flag);
        if (!ok) break;
        if (i == 0) stamp(3);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t b_low = a_low + (Shape::kBytesX >> 4);
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; ++k)
          umma_bf16(tmem_base, a_low + k * ((kUmmaK * 2) >> 4), b_low + k * ((kUmmaK * 2) >> 4), idesc, (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(empty_addr + 8 * stage);
        a_low += Shape::kStageBytes >> 4;
        if (++stage == (uint32_t)stages) {
          stage = 0;
          parity ^= 1;
          a_low = first_low;
        }
      }
      if (ok) umma_commit(accum_full);
      stamp(4);
    }
  } else {
    grid_dependency_wait();
    // --- epilogue, part one: this CTA's partial accumulator goes to the CTAs that finish its columns -----------------
    // warp e of the eight: rows (tensor-memory lanes) 32 (e % 4) ..., columns (kBN / 2) (e / 4) ... of the tile
    const int e = warp - 2, quad = warp & 3, half = e >> 2;   // a warp may touch the tensor-memory lanes of its own quarter, 32 (warp % 4) ...
    const int m = quad * 32 + lane;
    // scales of the step's rows, for a prepared-norm input (every CTA finishes some columns of every row)
    for (int row = threadIdx.x - 64; row < a.M; row += 256) {
      float scale = 1.0f;
      if (a.squares_in != nullptr) {
        float total = 0.0f;
        for (int t = 0; t < a.tiles_in; ++t) total += a.squares_in[(size_t)row * a.squares_in_stride + t];
        scale = 1.0f / sqrtf(total / (float)a.K + a.eps);
      }
      row_scale[row] = scale;
    }
    bool have = my_blocks > 0;
    if (have) have = mbar_wait(accum_full, 0, abort_flag);
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    if (threadIdx.x == 64) stamp(5);
    if (quad * 32 < a.M) {   // else: none of this warp's rows belongs to the step
      const uint32_t tmem_lane = tmem_base + ((uint32_t)(quad * 32) << 16) + half * (kBN / 2);
      // this thread's row in a finishing CTA's buffer: [this sender][group][row m]
      const uint32_t local = smem_u32(parts) + (uint32_t)((rank * groups * Shape::kGroupStride + m) * 16);
      constexpr uint32_t kGroupBytes = Shape::kGroupStride * 16;
#pragma unroll 1
      for (int c0 = 0; c0 < kBN / 2; c0 += 32) {
        uint32_t r[32];
        if (have) {
          tmem_load_32(tmem_lane + c0, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;   // no k block fell to this CTA: its part is zero
        }
        // column c of the tile lies in piece c / 64 at c % 64; CTA (c % 64) / slice finishes it
        const int piece = (half * (kBN / 2) + c0) >> 6;
        const uint32_t in_piece = (uint32_t)((half * (kBN / 2) + c0) & 63);
        uint32_t dest = in_piece / (uint32_t)slice, run = (in_piece - dest * slice) >> 2;
        uint32_t remote = map_to_rank(local, dest) + (uint32_t)(piece * runs) * kGroupBytes;
        if (m < a.M) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(remote + run * kGroupBytes), "r"(r[i]), "r"(r[i + 1]), "r"(r[i + 2]), "r"(r[i + 3]) : "memory");
            if (++run == (uint32_t)runs) {
              run = 0;
              ++dest;
              if (dest < (uint32_t)split) remote = map_to_rank(local, dest) + (uint32_t)(piece * runs) * kGroupBytes;
            }
          }
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  }
  // every thread of every CTA of the cluster: the parts are written (release) and may be read (acquire)
  __syncwarp();
  if (threadIdx.x == 64) stamp(6);
  cluster_sync_all();
  if (threadIdx.x == 64) stamp(7);

  if (warp >= 2 && !*abort_flag) {
    // --- epilogue, part two: add the S parts of this CTA's columns in rank order and finish them ---------------------
    // Work items are (row, run of 4 columns): a row's items lie side by side, so a warp writes runs of consecutive outputs.
    constexpr int kOutPieces = EPI == SKINNY_GATED ? kPieces / 2 : kPieces;   // gated: gate pieces 0, 2 pair with up pieces 1, 3
    const int per_row = kOutPieces * runs;
    const int items = a.M * per_row;
    const int t = threadIdx.x - 64;
    const int first_column = (int)rank * slice;      // inside every 64-column piece
#pragma unroll 1
    for (int base = 0; base < items; base += 256) {
      const int item = base + t;
      const bool active = item < items;
      const int row = active ? item / per_row : 0;
      const int within = active ? item - row * per_row : 0;
      const int out_piece = within / runs, j = (within - out_piece * runs) << 2;
      const int piece = EPI == SKINNY_GATED ? out_piece * 2 : out_piece;
      const float4* cell = parts + (piece * runs + (j >> 2)) * Shape::kGroupStride + row;   // sender 0's part; the up piece lies `runs` groups on
      const int sender_stride = groups * Shape::kGroupStride;
      float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f), up = sum;
      if (active) {
        sum = cell[0];
        if (EPI == SKINNY_GATED) up = cell[runs * Shape::kGroupStride];
        for (int s = 1; s < split; ++s) {
          const float4 part = cell[s * sender_stride];
          sum.x += part.x, sum.y += part.y, sum.z += part.z, sum.w += part.w;
          if (EPI == SKINNY_GATED) {
            const float4 more = cell[s * sender_stride + runs * Shape::kGroupStride];
            up.x += more.x, up.y += more.y, up.z += more.z, up.w += more.w;
          }
        }
      }
      const float value[4] = {sum.x, sum.y, sum.z, sum.w};
      const int in_piece = first_column + j;                           // 0 .. 63 for columns that exist
      const float scale = row_scale[row];
      float squares = 0.0f;
      if (EPI == SKINNY_GATED) {
        const float ups[4] = {up.x, up.y, up.z, up.w};
        const int n = tile * (kBN / 2) + out_piece * 64 + in_piece;   // output column of value[0]
        if (active && in_piece < 64) {   // columns come in fours: a group lies inside the piece or outside as a whole
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.out) + (size_t)row * a.n_out + n;
          float y[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) y[i] = silu_gated(__float_as_uint(value[i] * scale), __float_as_uint(ups[i] * scale));
          if (n + 3 < a.n_out && (a.n_out & 3) == 0) {
            *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(y[0], y[1]), pack_bf16(y[2], y[3]));
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              if (n + i < a.n_out) dst[i] = __float2bfloat16_rn(y[i]);
          }
        }
      } else {
        const int n = tile * kBN + piece * 64 + in_piece;
        const bool whole = active && in_piece < 64 && n + 3 < a.N && (a.N & 3) == 0;   // four columns of one row, 16-byte aligned in 32-bit
        if (whole && EPI == SKINNY_BF16) {
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.out) + (size_t)row * a.N + n) =
              make_uint2(pack_bf16(value[0] * scale, value[1] * scale), pack_bf16(value[2] * scale, value[3] * scale));
        } else if (whole && EPI == SKINNY_F32) {
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(a.out) + (size_t)row * a.N + n) = make_float4(value[0] * scale, value[1] * scale, value[2] * scale, value[3] * scale);
        } else if (whole && EPI == SKINNY_ACCUM) {
          float4* at = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.out) + (size_t)row * a.N + n);
          float4 updated = *at;
          updated.x += value[0], updated.y += value[1], updated.z += value[2], updated.w += value[3];
          *at = updated;
          if (a.prepare_weight != nullptr) {
            const float4 w4 = *reinterpret_cast<const float4*>(a.prepare_weight + n);
            *reinterpret_cast<uint2*>(a.prepare_x + (size_t)row * a.N + n) = make_uint2(pack_bf16(updated.x * w4.x, updated.y * w4.y), pack_bf16(updated.z * w4.z, updated.w * w4.w));
            squares = (updated.x * updated.x + updated.y * updated.y) + (updated.z * updated.z + updated.w * updated.w);
          }
        } else if (active && in_piece < 64) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (n + i >= a.N) continue;
            const size_t at = (size_t)row * a.N + n + i;
            if (EPI == SKINNY_BF16) {
              reinterpret_cast<__nv_bfloat16*>(a.out)[at] = __float2bfloat16_rn(value[i] * scale);
            } else if (EPI == SKINNY_F32) {
              reinterpret_cast<float*>(a.out)[at] = value[i] * scale;
            } else {
              const float updated = reinterpret_cast<float*>(a.out)[at] + value[i];
              reinterpret_cast<float*>(a.out)[at] = updated;
              if (a.prepare_weight != nullptr) {
                a.prepare_x[at] = __float2bfloat16_rn(updated * a.prepare_weight[n + i]);
                squares += updated * updated;
              }
            }
          }
        }
      }
      if (EPI == SKINNY_ACCUM && a.prepare_weight != nullptr) {
        // Partial sums of squares: the lanes of a warp that hold items of one row are side by side (per_row is a power of two
        // here, the plan sees to it); each such run of lanes adds up in a fixed order and its first lane stores the sum.
        const int lanes_in_row = per_row < 32 ? per_row : 32;
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1) {
          const float other = __shfl_down_sync(0xffffffffu, squares, offset);
          if (offset < lanes_in_row) squares += other;
        }
        if (active && (lane & (lanes_in_row - 1)) == 0) {
          const int runs_per_row = per_row <= 32 ? 1 : per_row >> 5;
          const int run = per_row <= 32 ? 0 : within >> 5;
          a.prepare_squares[(size_t)row * a.prepare_stride + ((size_t)tile * split + rank) * runs_per_row + run] = squares;
        }
      }
    }
  }
  if (threadIdx.x == 64) stamp(8);
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicOr(a.error_flag, 1);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // copies in flight may still land in this CTA's shared memory
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 2) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kBN));
  if (threadIdx.x == 64) stamp(9);
}

// The packed copy of w: [128-row group][k block][128 rows][64 k] bfloat16, every 128 x 64 block in the 128-byte swizzle (the
// 16-byte chunk j of row r lies at chunk j ^ (r % 8)).  Plain: group g holds rows 128 g ...; gated (w = [gate | up], n_out rows
// each): group g holds gate rows 64 g ... 64 g + 63, then the up rows of the same outputs.  Rows and k outside the matrix are
// zero; the number of groups is even, so that a tile of two groups never reads past the copy.
__global__ void skinny_pack_kernel(const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ packed, int N, int K, int gated, int n_out,
                                   int k_blocks, long long chunks) {
  for (long long index = (long long)blockIdx.x * blockDim.x + threadIdx.x; index < chunks; index += (long long)gridDim.x * blockDim.x) {
    const int physical = (int)(index & 7), r = (int)((index >> 3) & 127);
    const long long block = index >> 10;
    const int kb = (int)(block % k_blocks), group = (int)(block / k_blocks);
    const int j = physical ^ (r & 7);
    long long row;
    if (gated) row = r < 64 ? (long long)group * 64 + r : (long long)n_out + (long long)group * 64 + (r - 64);
    else row = (long long)group * 128 + r;
    const bool inside = gated ? ((long long)group * 64 + (r & 63) < n_out) : (row < N);
    const int k = kb * kBK + j * 8;
    uint4 value = make_uint4(0u, 0u, 0u, 0u);
    if (inside && k < K) value = *reinterpret_cast<const uint4*>(w + (size_t)row * K + k);   // K % 8 == 0: a chunk is inside or outside as a whole
    *reinterpret_cast<uint4*>(packed + index * 8) = value;
  }
}

static long long packed_groups(int N, int gated) {
  const long long groups = gated ? (N / 2 + 63) / 64 : (N + 127) / 128;
  return (groups + 1) & ~1LL;
}

struct SkinnyPlan {
  int split, kb_per, stages, slice, two_per_sm, tiles, square_runs;
};
static int g_force_split = 0;                  // tlie_gemm_skinny_force_split: 0 = plan freely
static int g_last_plan[5] = {0, 0, 0, 0, 0};   // split, k blocks per CTA, stages, CTAs, clusters the device can hold at once (for diagnostics)
static long long* g_timeline = nullptr;

// How K is cut: `split` parts (a cluster per tile) so that the CTAs fill the SMs, with what the device can hold of clusters of
// that size in mind: measured on a B200 (cudaOccupancyMaxActiveClusters, one CTA per SM): 148 single CTAs, 74 pairs, 45 of 3,
// 33 of 4, 15 of 7 or 8.  The measure is the k blocks the busiest SM has to stream, plus a fixed part per wave.
template <int MROWS>
static SkinnyPlan make_plan(int n_out, int K, bool gated, bool power_of_two) {
  using Shape = SkinnyShape<MROWS>;
  const int tile_out = gated ? Shape::kBN / 2 : Shape::kBN;
  const int tiles = (n_out + tile_out - 1) / tile_out;
  const int k_blocks = (K + kBK - 1) / kBK;
  const int sm_count = device_sm_count();
  static const int clusters_at_once[9] = {0, 148, 74, 45, 33, 24, 20, 15, 15};
  SkinnyPlan best = {1, k_blocks, 0, 64, 0, tiles, 1};
  double best_cost = 1e30;
  for (int split = 1; split <= kSkinnyMaxSplit; ++split) {
    if (split > k_blocks) break;
    if (power_of_two && (split & (split - 1))) continue;
    if (g_force_split > 0 && split != (g_force_split > k_blocks ? k_blocks : g_force_split)) continue;
    const int kb_per = (k_blocks + split - 1) / split;
    if ((k_blocks + kb_per - 1) / kb_per != split) continue;   // the same k blocks per CTA with fewer CTAs
    for (int two = 0; two < 2; ++two) {
      const int stages = Shape::max_stages(split, two ? 113 * 1024 : 227 * 1024);
      if (stages < 2) continue;
      const int capacity = clusters_at_once[split] * sm_count / 148 * (two ? 2 : 1);
      const int waves = (tiles + capacity - 1) / capacity;
      // a wave: the CTA's k blocks (two CTAs on an SM share its bandwidth), the prologue and the exchange of the parts
      const double cost = waves * (kb_per * (two && tiles * split > sm_count ? 2.0 : 1.0) + 6.0 + 0.5 * split);
      if (cost < best_cost - 1e-9) {
        best_cost = cost;
        best.split = split;
        best.kb_per = kb_per;
        best.stages = stages > kb_per ? (kb_per < 2 ? 2 : kb_per) : stages;
        best.two_per_sm = two;
      }
    }
  }
  best.slice = Shape::slice_of(best.split);
  const int per_row = (gated ? Shape::kPieces / 2 : Shape::kPieces) * (best.slice >> 2);
  best.square_runs = tiles * best.split * (per_row <= 32 ? 1 : per_row >> 5);
  return best;
}

template <int MROWS, int EPI>
static int launch_skinny(const void* x, const void* w, SkinnyArgs a, cudaStream_t stream) {
  using Shape = SkinnyShape<MROWS>;
  CUtensorMap map_x;   // x [M, K] row-major with boxes of MROWS rows x 64 k and 128-byte swizzle (rows past M read as zero)
  if (!make_map(&map_x, x, a.M, a.K, MROWS)) return (int)cudaErrorInvalidValue;
  const SkinnyPlan plan = make_plan<MROWS>(a.n_out, a.K, EPI == SKINNY_GATED, EPI == SKINNY_ACCUM && a.prepare_weight != nullptr);
  if (plan.stages < 2) return (int)cudaErrorInvalidValue;
  if (EPI == SKINNY_ACCUM && a.prepare_weight != nullptr && a.prepare_stride < plan.square_runs) return (int)cudaErrorInvalidValue;
  a.split = plan.split;
  a.kb_per = plan.kb_per;
  a.stages = plan.stages;
  a.slice = plan.slice;
  a.timeline = g_timeline;
  const size_t smem = (size_t)plan.stages * Shape::kStageBytes + Shape::fixed_bytes(plan.split);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<MROWS, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(plan.tiles * plan.split);
  config.blockDim = dim3(kSkinnyThreads);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = plan.split;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  static const bool pdl = [] {
    const char* v = std::getenv("TLIE_PDL");
    return !(v && v[0] == '0');
  }();
  config.numAttrs = pdl ? 2 : 1;
  g_last_plan[0] = plan.split;
  g_last_plan[1] = plan.kb_per;
  g_last_plan[2] = plan.stages;
  g_last_plan[3] = plan.tiles * plan.split;
  if (g_last_plan[4] < 0) {   // asked for by tlie_gemm_skinny_last_plan: how many clusters of this shape the device holds at once
    config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, gemm_skinny_kernel<MROWS, EPI>, &config) != cudaSuccess) clusters = 0;
    g_last_plan[4] = clusters;
    config.numAttrs = pdl ? 2 : 1;
  }
  return (int)cudaLaunchKernelEx(&config, gemm_skinny_kernel<MROWS, EPI>, (const __nv_bfloat16*)w, map_x, a);
}

template <int MROWS>
static int launch_skinny_epilogue(const void* x, const void* w, const SkinnyArgs& a, int epilogue, cudaStream_t stream) {
  switch (epilogue) {
    case SKINNY_BF16: return launch_skinny<MROWS, SKINNY_BF16>(x, w, a, stream);
    case SKINNY_F32: return launch_skinny<MROWS, SKINNY_F32>(x, w, a, stream);
    case SKINNY_GATED: return launch_skinny<MROWS, SKINNY_GATED>(x, w, a, stream);
    case SKINNY_ACCUM: return launch_skinny<MROWS, SKINNY_ACCUM>(x, w, a, stream);
  }
  return (int)cudaErrorInvalidValue;
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_gemm_skinny_max_rows() { return 128; }
// Diagnostics: cut K into this many parts whatever the plan says (0: plan freely); what the last launch used:
// {parts, k blocks per CTA, stages, CTAs, clusters of that shape the device can hold at once (asked for by `measure_next`)};
// and a device buffer of 16 int64 that CTA 0 of every launch fills with clock64 stamps of its phases (null: off).
TLIE_EXPORT void tlie_gemm_skinny_force_split(int split) { g_force_split = split; }
TLIE_EXPORT void tlie_gemm_skinny_last_plan(int* out5, int measure_next) {
  for (int i = 0; i < 5; ++i) out5[i] = g_last_plan[i];
  if (measure_next) g_last_plan[4] = -1;
}
TLIE_EXPORT void tlie_gemm_skinny_timeline(long long* buffer) { g_timeline = buffer; }

// Elements of the packed copy of a [N, K] matrix (gated: [gate | up] of N / 2 rows each).
TLIE_EXPORT long long tlie_gemm_skinny_packed_elements(int N, int K, int gated) {
  return packed_groups(N, gated) * ((K + kBK - 1) / kBK) * (kBM * kBK);
}

// packed (tlie_gemm_skinny_packed_elements bfloat16, 16-byte aligned) = the tile images of w [N, K] (16-byte aligned, K % 8 == 0).
TLIE_EXPORT int tlie_gemm_skinny_pack(const void* w, void* packed, int N, int K, int gated, cudaStream_t stream) {
  if (N <= 0 || K <= 0 || K % 8 != 0 || (gated && (N & 1)) || ((uintptr_t)w & 15) || ((uintptr_t)packed & 15)) return (int)cudaErrorInvalidValue;
  const long long chunks = tlie_gemm_skinny_packed_elements(N, K, gated) / 8;
  const long long blocks = (chunks + 255) / 256;
  skinny_pack_kernel<<<(unsigned)(blocks < 65535 * 8 ? blocks : 65535 * 8), 256, 0, stream>>>((const __nv_bfloat16*)w, (__nv_bfloat16*)packed, N, K, gated, N / 2,
                                                                                              (K + kBK - 1) / kBK, chunks);
  return (int)cudaGetLastError();
}

// Partial sums of squares per row that a call with `prepare_weight` writes for this shape (the row stride of prepare_squares must
// be at least this; the product that consumes them is told the same number as tiles_in).
TLIE_EXPORT int tlie_gemm_skinny_square_runs(int M, int N, int K) {
  if (M <= 32) return make_plan<32>(N, K, false, true).square_runs;
  if (M <= 64) return make_plan<64>(N, K, false, true).square_runs;
  return make_plan<128>(N, K, false, true).square_runs;
}

// out (+)= x . w^T for 1 <= M <= 128 rows.  x bfloat16 [M, K] contiguous (16-byte aligned, K % 8 == 0); w: the PACKED copy of the
// bfloat16 [N, K] matrix (tlie_gemm_skinny_pack, gated for epilogue 2).
// epilogue 0: out bfloat16 [M, N]; 1: out 32-bit [M, N]; 2: w = [gate rows | up rows] (N even), out bfloat16 [M, N / 2] =
// silu(gate) * up; 3: out is 32-bit [M, N] and the product is added to it.
// squares_in (or null): x is bfloat16(residual * norm weight) and squares_in [M, tiles_in] (row stride squares_in_stride) holds
// partial sums of squares of the residual's rows; every result is multiplied by 1 / sqrt(sum / K + eps) of its row (not with epilogue 3).
// prepare_weight (epilogue 3 only, or null): also store bfloat16(out * prepare_weight) in prepare_x [M, N] and
// tlie_gemm_skinny_square_runs(M, N, K) partial sums of squares per row in prepare_squares (row stride prepare_stride).
TLIE_EXPORT int tlie_gemm_skinny(const void* x, const void* w, void* out, int M, int N, int K, int epilogue, const float* squares_in,
                                 int tiles_in, int squares_in_stride, float eps, const float* prepare_weight, void* prepare_x,
                                 float* prepare_squares, int prepare_stride, int* error_flag, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 128 || K <= 0 || K % 8 != 0 || error_flag == nullptr || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || epilogue < 0 || epilogue > 3 ||
      (epilogue == SKINNY_GATED && (N & 1)) || (squares_in != nullptr && (tiles_in <= 0 || squares_in_stride < tiles_in || epilogue == SKINNY_ACCUM)) ||
      (prepare_weight != nullptr && (epilogue != SKINNY_ACCUM || prepare_x == nullptr || prepare_squares == nullptr)))
    return (int)cudaErrorInvalidValue;
  SkinnyArgs a;
  a.out = out;
  a.M = M;
  a.N = N;
  a.K = K;
  a.n_out = epilogue == SKINNY_GATED ? N / 2 : N;
  a.squares_in = squares_in;
  a.tiles_in = tiles_in;
  a.squares_in_stride = squares_in_stride;
  a.eps = eps;
  a.prepare_weight = prepare_weight;
  a.prepare_x = (__nv_bfloat16*)prepare_x;
  a.prepare_squares = prepare_squares;
  a.prepare_stride = prepare_stride;
  a.error_flag = error_flag;
  if (M <= 32) return launch_skinny_epilogue<32>(x, w, a, epilogue, stream);
  if (M <= 64) return launch_skinny_epilogue<64>(x, w, a, epilogue, stream);
  return launch_skinny_epilogue<128>(x, w, a, epilogue, stream);
}
