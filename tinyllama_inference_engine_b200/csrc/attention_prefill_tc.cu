// Paged grouped-query flash attention for prompt portions on the 5th-generation tensor cores (head size 64, bfloat16).
//
// Same mathematics as attention_prefill.cu (src/operators.cpp:102-146 per row, 32-bit softmax, causal by position,
// optional window), built the way this GPU wants it:
//   * a CTA owns 128 consecutive query rows of one request and one query head; thread i of the four softmax warps
//     owns row i, which is lane i of tensor memory, so row maxima and sums need no shuffles at all;
//   * Q (from the step's [q | k | v] rows) and each page of K and V (64 keys x 64 dims = one 8 KB box, exactly one
//     page of the cache) arrive by TMA with the 128-byte swizzle; the block table gives the page of every tile;
//   * S = Q . K^T is one tcgen05.mma group (128 x 64 x 64) into tensor memory, double-buffered so that the scores of
//     the next tile are computed while the softmax of this one runs;
//   * the softmax warps read S with tcgen05.ld, mask, exponentiate (scale folded into the exponent), write P as
//     bfloat16 into shared memory in the swizzled K-major layout, and a second tcgen05.mma group computes P . V with
//     V as an MN-major operand (V stays [key][dim], as the cache stores it);
//   * the running output lives in registers: O = O * 2^(old max - new max) + (P . V), read back from tensor memory.
// Roles: warp 0 TMA producer, warp 1 MMA issuer and tensor-memory owner, warps 2..5 softmax (128 threads).
// Every mbarrier wait is bounded; on a timeout the CTA raises `error_flag`, stops, lets copies land, frees its tensor
// memory and returns.  Needs page_size % 64 == 0; other shapes use the mma.sync kernel.
#include <cuda.h>

#include "common.cuh"

namespace tlie {

constexpr int kD = 64;            // head size
constexpr int kRowsTC = 128;      // query rows per CTA
constexpr int kKeysTC = 64;       // keys per tile (one box)
constexpr int kKvStages = 3;
constexpr int kThreadsTC = 192;
constexpr long long kWaitLimitTC = 1ll << 20;
constexpr float kLog2eTC = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void bar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool bar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (long long i = 0; i < kWaitLimitTC; ++i) {
    if (bar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_box_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(smem_addr(smem_dst)),
               "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y)
               : "memory");
}
// 128-byte-swizzled tile of 128-byte rows, 8-row groups 1024 bytes apart (both the K-major and the MN-major use).
__device__ __forceinline__ uint64_t tile_desc(uint32_t addr) {
  uint64_t desc = 0;
  desc |= (uint64_t)((addr >> 4) & 0x3FFF);
  desc |= (uint64_t)1 << 16;
  desc |= (uint64_t)(1024 >> 4) << 32;
  desc |= (uint64_t)1 << 46;
  desc |= (uint64_t)2 << 61;
  return desc;
}
// bf16 x bf16 -> f32, A K-major, B K-major (b_mn = 0) or MN-major (b_mn = 1), tile m x n.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_addr(bar)) : "memory");
}
// 64 consecutive 32-bit columns of this thread's lane: four loads in flight, one wait.
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&v)[64]) {
  uint32_t r[64];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[c * 16 + 0]), "=r"(r[c * 16 + 1]), "=r"(r[c * 16 + 2]), "=r"(r[c * 16 + 3]), "=r"(r[c * 16 + 4]), "=r"(r[c * 16 + 5]),
          "=r"(r[c * 16 + 6]), "=r"(r[c * 16 + 7]), "=r"(r[c * 16 + 8]), "=r"(r[c * 16 + 9]), "=r"(r[c * 16 + 10]), "=r"(r[c * 16 + 11]),
          "=r"(r[c * 16 + 12]), "=r"(r[c * 16 + 13]), "=r"(r[c * 16 + 14]), "=r"(r[c * 16 + 15])
        : "r"(taddr + c * 16));
  }
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}

struct SmemTC {
  // all tiles are 1024-byte aligned (the struct is placed on a 1024-byte boundary)
  __nv_bfloat16 q[kRowsTC * kD];                     // 16 KB
  __nv_bfloat16 k[kKvStages][kKeysTC * kD];          // 8 KB each
  __nv_bfloat16 v[kKvStages][kKeysTC * kD];          // 8 KB each
  __nv_bfloat16 p[2][kRowsTC * kKeysTC];             // 16 KB each
  uint64_t q_full, q_empty, kv_full[kKvStages], kv_empty[kKvStages], s_full[2], s_empty[2], p_full[2], pv_full, pv_empty;
  uint32_t tmem_base;
  int abort_flag;
};

// tiles: [n_items][4] = (request, first row, request, first row): one or two 128-row tiles per CTA (second request -1: none)
__global__ void __launch_bounds__(kThreadsTC)
    prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                                const int* __restrict__ tiles, const int* __restrict__ seq_starts, const int* __restrict__ first_positions,
                                const int* __restrict__ block_table, int table_stride, __nv_bfloat16* __restrict__ out, int q_heads,
                                int kv_heads, int page_size, int window, float scale, int* __restrict__ error_flag) {
  extern __shared__ uint8_t smem_raw[];
  SmemTC& sm = *reinterpret_cast<SmemTC*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  volatile int* abort_flag = &sm.abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // A work item is a pair of row tiles (the second may be absent): the host pairs a tile that sees many keys with one
  // that sees few, so that all CTAs carry about the same work and the grid ends together.
  const int* item = tiles + (size_t)blockIdx.x * 4;
  const int head = blockIdx.y;
  const int kvh = head / (q_heads / kv_heads);
  constexpr int kTmemCols = 256;   // S0 [0,64), S1 [64,128), PV [128,192)

  struct RowTile {
    int row0, rows_here, pos0, n_keys, first_kt, num_kt;
    const int* table;
  };
  auto row_tile = [&](int u) {
    RowTile t;
    const int seq = item[2 * u];
    t.row0 = item[2 * u + 1];
    if (seq < 0) {
      t.num_kt = 0;
      t.rows_here = t.pos0 = t.n_keys = t.first_kt = 0;
      t.table = block_table;
      return t;
    }
    t.rows_here = min(kRowsTC, seq_starts[seq + 1] - t.row0);
    t.pos0 = first_positions[seq] + (t.row0 - seq_starts[seq]);
    t.n_keys = t.pos0 + t.rows_here;                 // keys the last row of the tile sees
    const int lo_tile = (window > 0 && t.pos0 - window + 1 > 0) ? t.pos0 - window + 1 : 0;
    t.first_kt = lo_tile / kKeysTC;
    t.num_kt = (t.n_keys + kKeysTC - 1) / kKeysTC - t.first_kt;
    t.table = block_table + (size_t)seq * table_stride;
    return t;
  };

  if (threadIdx.x == 0) {
    bar_init(&sm.q_full, 1);
    bar_init(&sm.q_empty, 1);
    for (int s = 0; s < kKvStages; ++s) {
      bar_init(&sm.kv_full[s], 1);
      bar_init(&sm.kv_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      bar_init(&sm.s_full[b], 1);
      bar_init(&sm.s_empty[b], 4);   // one arrival per softmax warp
      bar_init(&sm.p_full[b], 4);
    }
    bar_init(&sm.pv_full, 1);
    bar_init(&sm.pv_empty, 4);
    sm.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(&sm.tmem_base)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem = sm.tmem_base;

  // g counts key tiles over both row tiles: every ring (kv stages, the two S / P buffers, the P.V buffer) is indexed by it.
  if (warp == 0) {
    if (lane == 0) {   // TMA producer: per row tile Q once, then one K box and one V box per key tile
      int g = 0;
      bool ok = true;
      for (int u = 0; u < 2 && ok; ++u) {
        const RowTile t = row_tile(u);
        if (t.num_kt == 0) continue;
        if (u > 0) ok = bar_wait(&sm.q_empty, 0, abort_flag);   // the first row tile's score products have read Q
        if (!ok) break;
        bar_expect_tx(&sm.q_full, kRowsTC * kD * 2);
        tma_box_2d(sm.q, &map_q, head * kD, t.row0, &sm.q_full);
        for (int j = 0; j < t.num_kt; ++j, ++g) {
          const int s = g % kKvStages;
          ok = bar_wait(&sm.kv_empty[s], ((g / kKvStages) & 1) ^ 1, abort_flag);
          if (!ok) break;
          const int key0 = (t.first_kt + j) * kKeysTC;
          const int page = t.table[key0 / page_size];
          const int in_page = key0 % page_size;
          const int k_row = ((page * 2 + 0) * kv_heads + kvh) * page_size + in_page;   // row of the [rows, 64] view of the pool
          const int v_row = ((page * 2 + 1) * kv_heads + kvh) * page_size + in_page;
          bar_expect_tx(&sm.kv_full[s], 2 * kKeysTC * kD * 2);
          tma_box_2d(sm.k[s], &map_kv, 0, k_row, &sm.kv_full[s]);
          tma_box_2d(sm.v[s], &map_kv, 0, v_row, &sm.kv_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {   // MMA issuer
      constexpr uint32_t idesc_s = instr_desc(kRowsTC, kKeysTC, 0);    // S = Q . K^T   (B = K tile, K-major)
      constexpr uint32_t idesc_pv = instr_desc(kRowsTC, kD, 1);        // PV = P . V    (B = V tile, MN-major)
      const uint32_t q_addr = smem_addr(sm.q);
      auto issue_s = [&](int g) {   // scores of key tile g into S buffer g & 1
        const int s = g % kKvStages, b = g & 1;
        if (!bar_wait(&sm.kv_full[s], (g / kKvStages) & 1, abort_flag)) return false;
        if (!bar_wait(&sm.s_empty[b], ((g >> 1) & 1) ^ 1, abort_flag)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t k_addr = smem_addr(sm.k[s]);
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) mma_ss(tmem + b * kKeysTC, tile_desc(q_addr + kk * 32), tile_desc(k_addr + kk * 32), idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(&sm.s_full[b]);
        return true;
      };
      int g = 0, q_phase = 0;
      bool ok = true;
      for (int u = 0; u < 2 && ok; ++u) {
        const RowTile t = row_tile(u);
        if (t.num_kt == 0) continue;
        ok = bar_wait(&sm.q_full, q_phase, abort_flag);
        q_phase ^= 1;
        if (ok) ok = issue_s(g);
        for (int j = 0; j < t.num_kt && ok; ++j, ++g) {
          if (j + 1 < t.num_kt) {
            ok = issue_s(g + 1);   // the next tile's scores run under this tile's softmax
          } else {
            mma_commit(&sm.q_empty);   // all score products of this row tile are issued: Q may be replaced when they are done
          }
          if (!ok) break;
          const int s = g % kKvStages, b = g & 1;
          ok = bar_wait(&sm.p_full[b], (g >> 1) & 1, abort_flag) && bar_wait(&sm.pv_empty, (g & 1) ^ 1, abort_flag);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint32_t p_addr = smem_addr(sm.p[b]), v_addr = smem_addr(sm.v[s]);
#pragma unroll
          for (int kk = 0; kk < kKeysTC / 16; ++kk)   // 16 keys further: 32 bytes inside P's rows, 16 rows (2048 bytes) down in V
            mma_ss(tmem + 2 * kKeysTC, tile_desc(p_addr + kk * 32), tile_desc(v_addr + kk * 16 * kD * 2), idesc_pv, kk > 0 ? 1u : 0u);
          mma_commit(&sm.pv_full);
          mma_commit(&sm.kv_empty[s]);   // both products of this stage are done when this fires
        }
      }
    }
  } else {   // softmax: thread = one query row = one lane of tensor memory
    const int sub = warp & 3;
    const int row = sub * 32 + lane;
    const uint32_t lane_base = (uint32_t)(sub * 32) << 16;
    const float sl2 = scale * kLog2eTC;
    int g = 0;
    bool ok = true;
    for (int u = 0; u < 2 && ok; ++u) {
      const RowTile t = row_tile(u);
      if (t.num_kt == 0) continue;
      const int my_pos = t.pos0 + min(row, t.rows_here - 1);   // rows past the end behave like the last row; never stored
      const int my_lo = (window > 0 && my_pos - window + 1 > 0) ? my_pos - window + 1 : 0;
      float o[kD];
#pragma unroll
      for (int i = 0; i < kD; ++i) o[i] = 0.0f;
      float row_max = -INFINITY, row_sum = 0.0f;
      float pending_alpha = 1.0f;   // the factor that belongs to the product P . V still in flight
      // O = O * alpha + (P . V of key tile gg): read one tile late, so that the product runs under the next tile's softmax
      auto absorb_pv = [&](int gg) {
        if (!bar_wait(&sm.pv_full, gg & 1, abort_flag)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        float pv[kD];
        tmem_ld64(tmem + lane_base + 2 * kKeysTC, pv);
#pragma unroll
        for (int i = 0; i < kD; ++i) o[i] = fmaf(o[i], pending_alpha, pv[i]);
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) bar_arrive(&sm.pv_empty);
        return true;
      };
      for (int j = 0; j < t.num_kt && ok; ++j, ++g) {
        const int b = g & 1, s = g % kKvStages;
        const int key0 = (t.first_kt + j) * kKeysTC;
        ok = bar_wait(&sm.s_full[b], (g >> 1) & 1, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        float sc[kKeysTC];
        tmem_ld64(tmem + lane_base + b * kKeysTC, sc);
        // S_b has been read: the issuer may overwrite it with key tile g + 2
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) bar_arrive(&sm.s_empty[b]);
        const bool need_mask = key0 + kKeysTC - 1 > t.pos0 || (window > 0 && key0 < t.pos0 + t.rows_here - window);
        float tile_max = -INFINITY;
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < kKeysTC; ++i) {
            const int key = key0 + i;
            sc[i] = (key >= my_lo && key <= my_pos) ? sc[i] : -INFINITY;
            tile_max = fmaxf(tile_max, sc[i]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < kKeysTC; ++i) tile_max = fmaxf(tile_max, sc[i]);
        }
        const float new_max = fmaxf(row_max, tile_max);
        const float finite_max = (new_max == -INFINITY) ? 0.0f : new_max;
        const float base = finite_max * sl2;
        const float alpha = exp2f((row_max - finite_max) * sl2);
        row_max = new_max;
        uint32_t packed[kKeysTC / 2];
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < kKeysTC / 2; ++i) {
          const float p0 = exp2_approx(fmaf(sc[2 * i], sl2, -base));
          const float p1 = exp2_approx(fmaf(sc[2 * i + 1], sl2, -base));
          sum += p0 + p1;
          __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
          packed[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        row_sum = row_sum * alpha + sum;
        // the previous tile's product has had this tile's softmax to finish: take it in before its buffer is reused
        if (j > 0) {
          ok = absorb_pv(g - 1);
          if (!ok) break;
        }
        pending_alpha = alpha;
        // P as bfloat16 into the swizzled K-major tile: row r at (r / 8) * 1024 + (r % 8) * 128, 16-byte chunk c at c ^ (r % 8)
        uint8_t* p_row = reinterpret_cast<uint8_t*>(sm.p[b]) + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
        for (int c = 0; c < kKeysTC / 8; ++c)
          *reinterpret_cast<uint4*>(p_row + ((c ^ (row & 7)) << 4)) = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
        // The last tile of a request may hold keys past its end whose values were never written: zero those V rows,
        // so that 0 * (whatever is there) stays 0.  A V row is 128 contiguous bytes whatever the swizzle.
        if (key0 + kKeysTC > t.n_keys) {
          const int first_bad = t.n_keys - key0;
          for (int r = first_bad + (row >> 3); r < kKeysTC; r += kRowsTC / 8) {
            uint8_t* v_row = reinterpret_cast<uint8_t*>(sm.v[s]) + (r >> 3) * 1024 + (r & 7) * 128;
            *reinterpret_cast<uint4*>(v_row + (row & 7) * 16) = make_uint4(0, 0, 0, 0);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic-proxy writes -> visible to the tensor core
        __syncwarp();
        if (lane == 0) bar_arrive(&sm.p_full[b]);
      }
      if (ok) ok = absorb_pv(g - 1);
      if (ok && row < t.rows_here) {
        const float inv = 1.0f / row_sum;
        __nv_bfloat16* dst = out + ((size_t)(t.row0 + row) * q_heads + head) * kD;
#pragma unroll
        for (int c = 0; c < kD / 8; ++c) {
          uint32_t packed[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(o[c * 8 + 2 * i] * inv, o[c * 8 + 2 * i + 1] * inv);
            packed[i] = *reinterpret_cast<uint32_t*>(&h);
          }
          *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  }
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(error_flag, 1);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // copies that were issued may still be landing
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols));
  }
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                             const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeFn encoder() {
  static EncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* found = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &found, cudaEnableDefault, &status) == cudaSuccess && status == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(found);
  }
  return fn;
}
// [rows, width] bfloat16 with a row stride in elements, boxes of box_rows x 64, 128-byte swizzle.
static bool make_map_2d(CUtensorMap* map, const void* base, long long rows, long long width, long long row_stride, int box_rows) {
  EncodeFn fn = encoder();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_prefill_attention_tc_tile_rows() { return kRowsTC; }

// q: the step's rows [tokens, q_row_stride] starting with the rotated q heads (head size 64); pages: one layer's pool
// [num_pages, 2, kv_heads, page_size, 64]; tiles: int32 [n_tiles, 4] work items of one or two 128-row tiles (request, first
// row, request or -1, first row); error_flag: device int, zero.
TLIE_EXPORT int tlie_prefill_attention_tc(const void* q, int q_row_stride, int tokens, const void* pages, int num_pages, const int* tiles,
                                          int n_tiles, const int* seq_starts, const int* first_positions, const int* block_table,
                                          int table_stride, void* out, int q_heads, int kv_heads, int page_size, int window, float scale,
                                          int* error_flag, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (kv_heads <= 0 || q_heads % kv_heads != 0 || q_heads > 65535 || page_size % kKeysTC != 0 || q_row_stride % 8 != 0 || error_flag == nullptr)
    return (int)cudaErrorInvalidValue;
  CUtensorMap map_q, map_kv;
  if (!make_map_2d(&map_q, q, tokens, (long long)q_heads * kD, q_row_stride, kRowsTC)) return (int)cudaErrorInvalidValue;
  if (!make_map_2d(&map_kv, pages, (long long)num_pages * 2 * kv_heads * page_size, kD, kD, kKeysTC)) return (int)cudaErrorInvalidValue;
  const int smem = (int)sizeof(SmemTC) + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(n_tiles, q_heads);
  prefill_attention_tc_kernel<<<grid, kThreadsTC, smem, stream>>>(map_q, map_kv, tiles, seq_starts, first_positions, block_table, table_stride,
                                                                  (__nv_bfloat16*)out, q_heads, kv_heads, page_size, window, scale, error_flag);
  return (int)cudaGetLastError();
}
