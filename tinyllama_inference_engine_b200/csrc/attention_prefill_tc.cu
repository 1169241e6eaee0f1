// Paged grouped-query flash attention for prompt portions on the 5th-generation tensor cores (head size 64 or 128, bfloat16).
//
// Same mathematics as attention_prefill.cu (src/operators.cpp:102-146 per row, 32-bit softmax, causal by position,
// optional window), built the way this GPU wants it:
//   * a CTA owns 128 consecutive query rows of one request and one query head; thread i of the four softmax warps
//     owns row i, which is lane i of tensor memory, so row maxima and sums need no shuffles at all.  (Two threads per row,
//     32 scores each and both reading all 64 for the maximum, was built and measured: sixteen softmax warps on an SM, but
//     32 M warp instructions where this form has 18 M, since what a warp does per tile besides the scores is the same for 32
//     scores as for 64, and the kernel took half as long again);
//   * Q (from the step's [q | k | v] rows) and each page of K and V (64 keys x 64 dims = one 8 KB box; a head of 128 is two
//     such boxes side by side, the two halves of a row 128 bytes each) arrive by TMA with the 128-byte swizzle; the block
//     table gives the page of every tile.  K and V have rings of their own: a K buffer is free as soon as its scores are
//     computed, a whole tile before the V buffer of the same keys is, so the K loads run one tile further ahead than the V
//     loads and the score products never wait for memory (with one ring for both and two stages, at head size 128, every
//     score product waited 1,450 of a tile's 3,470 cycles for its keys);
//   * S = Q . K^T is one tcgen05.mma group (128 x 64 x head size) into tensor memory, double-buffered so that the scores of
//     the next tile are computed while the softmax of this one runs;
//   * the softmax warps read S with tcgen05.ld, mask, exponentiate (scale folded into the exponent) and write P as
//     bfloat16 back into tensor memory, over the first half of the very columns its scores came from (a thread has its row
//     in registers by then, and nobody else reads that lane); a second tcgen05.mma group computes P . V with P as the
//     A operand from tensor memory and V as an MN-major operand from shared memory (V stays [key][dim], as the cache stores
//     it).  P through shared memory (swizzled 16-byte stores, a proxy fence, then the arrival) cost a thread 700 of a tile's
//     2,400 cycles and 16 KB per buffer;
//   * the running output lives in tensor memory: every P . V accumulates onto it, against a reference maximum per row;
//     when a tile's maximum is more than 2^8 above the reference, the row's thread multiplies its lane of the output
//     and its sum by 2^(old reference - new one) (a warp-wide load, multiply and store; rows that need nothing use 1)
//     before P of that tile is handed over, and the output is read once, after the last tile, and divided by the sum;
//   * the kernel is launched as a programmatic dependent: barriers and tensor memory are set up while the kernel before
//     it drains, global memory is touched only after the dependency wait.
// Roles: warp 0 TMA producer, warp 1 issuer of the score products and tensor-memory owner, warp 2 issuer of the P . V products,
// warp 3 idle, warps 4..7 softmax (128 threads).  The launch gives every thread 128 registers (two CTAs of 256 threads fill the
// register file); the first four warps hand most of theirs back at once (setmaxnreg) and the softmax warps, whose threads hold a
// row's 64 scores, take them: 200 each, with nothing spilled.  The two issuers are lone threads that share their schedulers with
// busy softmax warps, so every instruction of theirs takes its time; one thread issuing both kinds of product had 2,100 of a tile's 2,500 cycles of
// work at head size 64 (2,670 of 2,830 at 128) and the softmax threads waited for their scores 930 (1,190) cycles of every tile.
// Apart, the score issuer runs ahead as far as the two S buffers let it and a P . V product starts as soon as its P is there.
// Every mbarrier wait is bounded; on a timeout the CTA raises `error_flag`, stops, lets copies land, frees its tensor
// memory and returns.  Needs page_size % 64 == 0; other shapes use the mma.sync kernel.
// Two CTAs share an SM, so that one's products run under the other's softmax.  Head size 64: three K and three V stages, 65 KB of
// shared memory and 256 columns of tensor memory (two score buffers, whose first halves take P, and one running output per row
// tile).  Head size 128 is made to fit the same way: two stages and ONE running output of 128 columns that the second row tile
// takes over when the first has been read out: 96 KB and 256 columns.  (One CTA per SM with everything doubled ran the
// 8,192-token prefill of the 8B shapes at 1.41 ms a layer.)
// A work item is one row tile or two.  Steps send single row tiles, heaviest first (ops.fast.single_attention_tiles): a CTA is a
// chain of dependent waits, so twice the CTAs with half the work each were faster at every length measured (one request of 512 to
// 4,096 tokens: by 3 to 24 %) than pairs of a heavy and a light tile (paired_attention_tiles), which the kernel also takes.
#include "tcgen05_utils.cuh"

namespace tlie {

constexpr int kRowsTC = 128;      // query rows per CTA
constexpr int kKeysTC = 64;       // keys per tile (one box)
constexpr int kBoxDims = 64;      // dims of one box: 128 bytes, the swizzle span
constexpr int kThreadsTC = 256;
constexpr int kFirstSoftmaxWarpTC = 4;
constexpr int kControlRegsTC = 56, kSoftmaxRegsTC = 200;   // (128 - 56) * 128 threads handed over = 72 more for each of the 128 softmax threads
constexpr float kLog2eTC = 1.4426950408889634f;
// The running output stays in tensor memory and is rescaled only when a row's maximum has grown by more than this many
// powers of two since its reference was set: until then the probabilities are taken against the old reference and are at
// most 2^kLazyRescale, which bfloat16 and the 32-bit sum hold without loss.
constexpr float kLazyRescale = 8.0f;

// bf16 x bf16 -> f32, A K-major, B MN-major (V stays [key][dim], as the cache stores it), tile m x n.
__host__ __device__ constexpr uint32_t instr_desc_b_mn(int m, int n) { return umma_instr_desc(m, n) | (1u << 16); }

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

// The reverse: 64 columns of this thread's lane written from registers (and waited for).
__device__ __forceinline__ void tmem_st64(uint32_t taddr, const float (&v)[64]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n" ::"r"(taddr + c * 16),
        "r"(__float_as_uint(v[c * 16 + 0])), "r"(__float_as_uint(v[c * 16 + 1])), "r"(__float_as_uint(v[c * 16 + 2])), "r"(__float_as_uint(v[c * 16 + 3])),
        "r"(__float_as_uint(v[c * 16 + 4])), "r"(__float_as_uint(v[c * 16 + 5])), "r"(__float_as_uint(v[c * 16 + 6])), "r"(__float_as_uint(v[c * 16 + 7])),
        "r"(__float_as_uint(v[c * 16 + 8])), "r"(__float_as_uint(v[c * 16 + 9])), "r"(__float_as_uint(v[c * 16 + 10])), "r"(__float_as_uint(v[c * 16 + 11])),
        "r"(__float_as_uint(v[c * 16 + 12])), "r"(__float_as_uint(v[c * 16 + 13])), "r"(__float_as_uint(v[c * 16 + 14])), "r"(__float_as_uint(v[c * 16 + 15]))
        : "memory");
  }
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}

// 32 columns of this thread's lane written from registers (and waited for).
__device__ __forceinline__ void tmem_store_32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
      "%23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
      "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
      "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}

// The product with its A operand in tensor memory (lane = row, 16 k = 8 columns of two bfloat16) and B by its descriptor's lower word.
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_low, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 db;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "mov.b64 db, {%2, %5};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "r"(b_low), "r"(idesc), "r"(accumulate), "r"(kUmmaDescHigh)
      : "memory");
}

// A softmax thread's time is its instruction count (a warp issues an instruction every two to three cycles at best), so the loop
// over a row's scores uses what this GPU has for it: the maximum of three numbers in one instruction, and multiply-add and add
// on two floats at once (the same roundings as one at a time).
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
struct Float2Bits {
  unsigned long long bits;
};
__device__ __forceinline__ Float2Bits pair_of(float lo, float hi) {
  Float2Bits r;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(r.bits) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpair(Float2Bits v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v.bits)); }
__device__ __forceinline__ Float2Bits fma2(Float2Bits a, Float2Bits b, Float2Bits c) {
  Float2Bits r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(r.bits) : "l"(a.bits), "l"(b.bits), "l"(c.bits));
  return r;
}
__device__ __forceinline__ Float2Bits add2(Float2Bits a, Float2Bits b) {
  Float2Bits r;
  asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(r.bits) : "l"(a.bits), "l"(b.bits));
  return r;
}

// Where a CTA's time goes, when compiled with TLIE_ATTN_TIMELINE: one thread of each role of CTA (0, 0) reports the cycles of its
// whole loop (slot 6 of its group: softmax 0-7, issuer 8-15, producer 16-23), its tiles (slot 7) and, with TLIE_ATTN_TIMELINE_SLOT = k,
// the cycles spent between stamp k - 1 and stamp k (slot k).  One slot per build: more would cost registers the kernel does not have.
#ifdef TLIE_ATTN_TIMELINE
#ifndef TLIE_ATTN_TIMELINE_SLOT
#define TLIE_ATTN_TIMELINE_SLOT -1
#endif
__device__ long long tlie_attn_stamps[24];
#define TL_BEGIN(on) const bool tl_on = (on); const long long tl_first = clock64(); unsigned tl_last = (unsigned)tl_first, tl_acc = 0, tl_count = 0;
#define TL(i) if (TLIE_ATTN_TIMELINE_SLOT >= 0) { const unsigned tl_now = (unsigned)clock64(); if ((i) == TLIE_ATTN_TIMELINE_SLOT) tl_acc += tl_now - tl_last; tl_last = tl_now; }
#define TL_COUNT() { tl_count += 1; }
#define TL_END(base) if (tl_on) { tlie_attn_stamps[(base) + 6] = clock64() - tl_first; tlie_attn_stamps[(base) + 7] = tl_count; \
    if (TLIE_ATTN_TIMELINE_SLOT >= 0 && TLIE_ATTN_TIMELINE_SLOT < 6) tlie_attn_stamps[(base) + TLIE_ATTN_TIMELINE_SLOT] = tl_acc; }
#else
#define TL_BEGIN(on)
#define TL(i)
#define TL_COUNT()
#define TL_END(base)
#endif

// A tile of D dims is D / 64 sub-tiles of 64 dims side by side in memory, each [rows][64] in the 128-byte swizzle.
template <int D>
struct SmemTC {
  static constexpr int kStages = D <= 64 ? 3 : 2;
  // all tiles are 1024-byte aligned (the struct is placed on a 1024-byte boundary)
  __nv_bfloat16 q[kRowsTC * D];                      // 16 KB per 64 dims
  __nv_bfloat16 k[kStages][kKeysTC * D];             // 8 KB per 64 dims each
  __nv_bfloat16 v[kStages][kKeysTC * D];
  // k_full / v_full: a tile has landed.  s_done: the scores of the tile in this K stage are computed (the softmax threads wait for it,
  // and the producer before it loads K again).  v_done: the P . V of the tile in this V stage is done (the producer waits for it, and the
  // softmax threads before they touch O, and the score issuer before it writes the S buffer that holds this tile's P).  p_full: the
  // softmax threads have written P.
  uint64_t q_full, q_empty, k_full[kStages], s_done[kStages], v_full[kStages], v_done[kStages], p_full[2], o_full[2], o_read;
  uint32_t tmem_base;
  int abort_flag;
};

// tiles: [n_items][4] = (request, first row, request, first row): one or two 128-row tiles per CTA (second request -1: none)
template <int kD>
__global__ void __launch_bounds__(kThreadsTC, 2)
    prefill_attention_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                                const int* __restrict__ tiles, const int* __restrict__ seq_starts, const int* __restrict__ first_positions,
                                const int* __restrict__ block_table, int table_stride, __nv_bfloat16* __restrict__ out, int q_heads,
                                int kv_heads, int page_size, int window, float scale, int* __restrict__ error_flag) {
  extern __shared__ uint8_t smem_raw[];
  using Smem = SmemTC<kD>;
  constexpr int kKvStages = Smem::kStages;
  constexpr int kSubTiles = kD / kBoxDims;
  Smem& sm = *reinterpret_cast<Smem*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  volatile int* abort_flag = &sm.abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // A work item is one row tile or a pair of them (the second absent: -1).
  // The heads of a work item are neighbours in the order CTAs are handed out (x runs fastest), and the items come heaviest first:
  // with more CTAs than the SMs hold at once, every slot that comes free takes the heaviest work left, and the CTAs that run
  // together read the same keys and values (the heads of a group) out of L2.
  const int* item = tiles + (size_t)blockIdx.y * 4;
  const int head = blockIdx.x;
  const int kvh = head / (q_heads / kv_heads);
  // S0 [0,64), S1 [64,128), O of the first row tile [128, 128 + D), of the second [128 + D, 128 + 2 D)
  // (head size 128: both row tiles use [128, 256), one after the other)
  constexpr int kTmemCols = 256;
  constexpr int kOutCol0 = 2 * kKeysTC;
  constexpr bool kCompact = kD > 64;
  constexpr int kOutStride = kCompact ? 0 : kD;
  if (kCompact && (smem_u32(smem_raw) & 1023u) != 0) {   // no room was asked for to align by hand: the tiles must lie on 1 KB boundaries as they are
    if (threadIdx.x == 0) atomicOr(error_flag, 1);
    return;
  }

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
    mbar_init(&sm.q_full, 1);
    mbar_init(&sm.q_empty, 1);
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(&sm.k_full[s], 1);
      mbar_init(&sm.s_done[s], 1);
      mbar_init(&sm.v_full[s], 1);
      mbar_init(&sm.v_done[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.p_full[b], 4);   // one arrival per softmax warp
    }
    mbar_init(&sm.o_full[0], 1);   // used once each: all products of a row tile are done
    mbar_init(&sm.o_full[1], 1);
    mbar_init(&sm.o_read, 4);      // the first row tile's output has been read out of tensor memory (one arrival per softmax warp)
    sm.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sm.tmem_base)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem = sm.tmem_base;
  // Programmatic dependent launch: the CTA is set up (barriers, tensor memory) while the kernel before it in the stream still
  // runs; nothing of global memory is touched before the wait, which returns when that kernel has completed.
  grid_launch_dependents();
  grid_dependency_wait();

  // g counts key tiles over both row tiles (n0 of the first, G in all): every ring (K stages, V stages, the two S / P buffers,
  // the P.V barrier) is indexed by it.
  if (warp < kFirstSoftmaxWarpTC) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(kControlRegsTC));
  if (warp == 0) {
    if (lane == 0) {   // TMA producer: per row tile Q once, then per key tile one K box and one V box (two each at head size 128)
      const RowTile t0 = row_tile(0), t1 = row_tile(1);
      const int n0 = t0.num_kt, G = n0 + t1.num_kt;
      const int tiles_per_page = page_size / kKeysTC;
      RingPosition<kKvStages> k_ring, v_ring;
      TL_BEGIN(blockIdx.x == 0 && blockIdx.y == 0)
      const uint32_t k_addr = smem_u32(sm.k), v_addr = smem_u32(sm.v);
      const uint32_t k_full = smem_u32(sm.k_full), k_empty = smem_u32(sm.s_done), v_full = smem_u32(sm.v_full), v_empty = smem_u32(sm.v_done);
      // One tile of K (plane 0 of the page) or of V (plane 1).  The page's number is asked for before the wait for a free buffer,
      // so that its trip to memory runs under the wait.
      auto load = [&](int g, int plane, RingPosition<kKvStages>& ring, uint32_t tiles_addr, uint32_t full, uint32_t empty) {
        const RowTile& t = g >= n0 ? t1 : t0;
        const int kt = t.first_kt + (g >= n0 ? g - n0 : g);
        int page_index = kt, in_page = 0;
        if (tiles_per_page != 1) {
          page_index = kt / tiles_per_page;
          in_page = (kt - page_index * tiles_per_page) * kKeysTC;
        }
        const int page = t.table[page_index];
        TL(0)
        if (!mbar_wait(empty + 8 * ring.stage, ring.phase ^ 1, abort_flag)) return false;
        TL(1)
        const int row = ((page * 2 + plane) * kv_heads + kvh) * page_size + in_page;   // row of the [rows, head size] view of the pool
        const uint32_t bar = full + 8 * ring.stage;
        mbar_expect_tx(bar, kKeysTC * kD * 2);
#pragma unroll
        for (int c = 0; c < kSubTiles; ++c)
          tma_load_2d(tiles_addr + ring.stage * (kKeysTC * kD * 2) + c * (kKeysTC * kBoxDims * 2), &map_kv, c * kBoxDims, row, bar);
        ring.advance();
        return true;
      };
      auto load_q = [&](const RowTile& t) {
        mbar_expect_tx(&sm.q_full, kRowsTC * kD * 2);
#pragma unroll
        for (int c = 0; c < kSubTiles; ++c) tma_load_2d(sm.q + c * kRowsTC * kBoxDims, &map_q, head * kD + c * kBoxDims, t.row0, &sm.q_full);
      };
      bool ok = G > 0;
      if (ok) {
        load_q(n0 > 0 ? t0 : t1);
        ok = load(0, 0, k_ring, k_addr, k_full, k_empty);
      }
      for (int g = 0; g < G && ok; ++g) {   // K of the next tile, then V of this one
        if (g + 1 < G) {
          if (g + 1 == n0) {                 // the second row tile begins: its Q replaces the first one's when all score products of that are done
            ok = mbar_wait(&sm.q_empty, 0, abort_flag);
            if (ok) load_q(t1);
          }
          if (ok) ok = load(g + 1, 0, k_ring, k_addr, k_full, k_empty);
        }
        if (ok) ok = load(g, 1, v_ring, v_addr, v_full, v_empty);
        TL_COUNT()
      }
      TL_END(16)
    }
  } else if (warp == 1) {
    if (lane == 0) {   // issuer of the score products: S(g) = Q . K(g)^T into S buffer g & 1, as far ahead as the buffers allow
      constexpr uint32_t idesc_s = umma_instr_desc(kRowsTC, kKeysTC);      // B = K tile, K-major
      constexpr uint32_t kTileLow = (kKeysTC * kD * 2) >> 4;               // one K tile further, in descriptor units
      const int n0 = row_tile(0).num_kt, G = n0 + row_tile(1).num_kt;
      const uint32_t q_low = umma_desc_low(smem_u32(sm.q)), k_low = umma_desc_low(smem_u32(sm.k));
      const uint32_t k_full = smem_u32(sm.k_full), s_done = smem_u32(sm.s_done), v_done = smem_u32(sm.v_done);
      RingPosition<kKvStages> ring, before, two_before;   // where tile g, g - 1, g - 2 lie in the rings
      int q_phase = 0;
      bool ok = true;
      TL_BEGIN(blockIdx.x == 0 && blockIdx.y == 0)
      for (int g = 0; g < G && ok; ++g, two_before = before, before = ring, ring.advance()) {
        const uint32_t b = g & 1;
        TL(0)
        if (g == 0 || g == n0) {    // a row tile begins: its Q
          ok = mbar_wait(&sm.q_full, q_phase, abort_flag);
          q_phase ^= 1;
        }
        if (ok) ok = mbar_wait(k_full + 8 * ring.stage, ring.phase, abort_flag);
        TL(1)
        // This S buffer still holds P of tile g - 2: the product that reads it must be done.  (Its barrier cannot be further on than that:
        // the product that completes it next needs the scores issued here.)
        if (ok && g > 1) ok = mbar_wait(v_done + 8 * two_before.stage, two_before.phase, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        TL(2)
        const uint32_t k_tile = k_low + ring.stage * kTileLow;
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {   // 16 dims further: 32 bytes inside a sub-tile's rows, then the next sub-tile
          constexpr uint32_t kQSub = (kRowsTC * kBoxDims * 2) >> 4, kKSub = (kKeysTC * kBoxDims * 2) >> 4;
          umma_bf16(tmem + b * kKeysTC, q_low + (kk >> 2) * kQSub + (kk & 3) * 2, k_tile + (kk >> 2) * kKSub + (kk & 3) * 2, idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(s_done + 8 * ring.stage);
        if (g + 1 == n0 && G > n0) umma_commit(&sm.q_empty);   // all score products of the first row tile are issued: Q may be replaced when they are done
        TL(3)
        TL_COUNT()
      }
      TL_END(8)
    }
  } else if (warp == 2) {
    if (lane == 0) {   // issuer of the P . V products: O += P(g) . V(g) as soon as P(g) is written
      constexpr uint32_t idesc_pv = instr_desc_b_mn(kRowsTC, kD);          // B = V tile, MN-major
      constexpr uint32_t kTileLow = (kKeysTC * kD * 2) >> 4;
      // V is the MN-major operand: its dims run along N.  Beyond 64 dims the next sub-tile of 64 lies kKeysTC * 128 bytes on,
      // which the descriptor's leading-dimension offset says (bits 16-29, in 16-byte units); one sub-tile needs none.
      constexpr uint32_t kVLeading = kSubTiles > 1 ? ((uint32_t)(kKeysTC * kBoxDims * 2) >> 4) : 1u;
      const int n0 = row_tile(0).num_kt, G = n0 + row_tile(1).num_kt;
      const uint32_t v_low = ((smem_u32(sm.v) >> 4) & 0x3FFF) | (kVLeading << 16);
      const uint32_t v_full = smem_u32(sm.v_full), v_done = smem_u32(sm.v_done), p_full = smem_u32(sm.p_full);
      RingPosition<kKvStages> ring;
      bool ok = true;
      TL_BEGIN(false)
      for (int g = 0; g < G && ok; ++g, ring.advance()) {
        const uint32_t b = g & 1;
        const bool second = g >= n0;          // which row tile this key tile belongs to
        const bool first_of_row_tile = g == 0 || g == n0;
        ok = mbar_wait(v_full + 8 * ring.stage, ring.phase, abort_flag);
        if (ok && kCompact && second && first_of_row_tile && n0 > 0)
          ok = mbar_wait(&sm.o_read, 0, abort_flag);   // the one output buffer: the softmax warps must have read the first row tile's result out of it
        if (ok) ok = mbar_wait(p_full + 8 * b, (g >> 1) & 1, abort_flag);   // P is written (and O rescaled, if it had to be)
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t tmem_o = tmem + kOutCol0 + (second ? kOutStride : 0);   // this row tile's running output
        const uint32_t p_tile = tmem + b * kKeysTC, v_tile = v_low + ring.stage * kTileLow;   // P: 32 columns of two bfloat16 each, where S of this tile was
#pragma unroll
        for (int kk = 0; kk < kKeysTC / 16; ++kk)   // 16 keys further: 8 columns of P, 16 rows (2048 bytes) down in a V sub-tile
          umma_bf16_a_tmem(tmem_o, p_tile + kk * 8, v_tile + kk * ((16 * kBoxDims * 2) >> 4), idesc_pv, (!first_of_row_tile || kk > 0) ? 1u : 0u);
        umma_commit(v_done + 8 * ring.stage);
        if (g + 1 == n0) umma_commit(&sm.o_full[0]);   // a row tile's output is complete when this fires
        if (g + 1 == G && G > n0) umma_commit(&sm.o_full[1]);
      }
      TL_END(8)
    }
  } else if (warp >= kFirstSoftmaxWarpTC) {   // softmax: thread = one query row = one lane of tensor memory
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(kSoftmaxRegsTC));
    const int sub = warp & 3;
    const int row = sub * 32 + lane;
    const uint32_t lane_base = (uint32_t)(sub * 32) << 16;
    const float sl2 = scale * kLog2eTC;
    int g = 0;
    bool ok = true;
    // Where tile g, g - 1 and g - 2 lie in the K / V rings (stage and phase bit of their barriers).
    RingPosition<kKvStages> at, before, two_before;
    TL_BEGIN(blockIdx.x == 0 && blockIdx.y == 0 && warp == kFirstSoftmaxWarpTC && lane == 0)
    for (int u = 0; u < 2 && ok; ++u) {
      const RowTile t = row_tile(u);
      if (t.num_kt == 0) continue;
      const int my_pos = t.pos0 + min(row, t.rows_here - 1);   // rows past the end behave like the last row; never stored
      const int my_lo = (window > 0 && my_pos - window + 1 > 0) ? my_pos - window + 1 : 0;
      const uint32_t tmem_o = tmem + lane_base + kOutCol0 + u * kOutStride;
      // The row's reference maximum (times scale * log2 e) that the exponents are taken against, and the sum against it.
      float reference = -INFINITY, row_sum = 0.0f;
      for (int j = 0; j < t.num_kt && ok; ++j, ++g, two_before = before, before = at, at.advance()) {
        const int b = g & 1;
        const int key0 = (t.first_kt + j) * kKeysTC;
        TL(0)
        ok = mbar_wait(&sm.s_done[at.stage], at.phase, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        TL(1)
        TL_COUNT()
        float sc[kKeysTC];
        tmem_ld64(tmem + lane_base + b * kKeysTC, sc);
        TL(2)
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
          float m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;   // four chains of eight three-way maxima instead of one of 64 dependent ones
#pragma unroll
          for (int i = 0; i < kKeysTC; i += 8) {
            tile_max = max3(tile_max, sc[i], sc[i + 1]);
            m1 = max3(m1, sc[i + 2], sc[i + 3]);
            m2 = max3(m2, sc[i + 4], sc[i + 5]);
            m3 = max3(m3, sc[i + 6], sc[i + 7]);
          }
          tile_max = fmaxf(fmaxf(tile_max, m1), fmaxf(m2, m3));
        }
        const float scaled_max = tile_max * sl2;
        if (j == 0) {
          reference = scaled_max;   // nothing accumulated yet: the first product overwrites O
        } else {
          // O (in tensor memory) and the sum are taken against `reference`.  They are brought to a new one only when this
          // tile's maximum is far above it; the loads and stores are warp-wide, rows that need nothing multiply by one.
          const bool grown = scaled_max > reference + kLazyRescale;
          if (__any_sync(0xffffffffu, grown)) {
            // The product that last added to O must be done (the one of this tile waits for this P, so its barrier cannot be further on).
            ok = mbar_wait(&sm.v_done[before.stage], before.phase, abort_flag);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const float alpha = grown ? exp2f(reference - scaled_max) : 1.0f;
#pragma unroll
            for (int c = 0; c < kSubTiles; ++c) {   // 64 columns of the output at a time
              float o[64];
              tmem_ld64(tmem_o + c * 64, o);
#pragma unroll
              for (int i = 0; i < 64; ++i) o[i] *= alpha;
              tmem_st64(tmem_o + c * 64, o);
            }
            row_sum *= alpha;
            if (grown) reference = scaled_max;
          }
        }
        const float base = (reference == -INFINITY) ? 0.0f : reference;   // a row that has seen no key yet: every p is 0
        TL(3)
        uint32_t packed[kKeysTC / 2];
        const Float2Bits scale2 = pair_of(sl2, sl2), minus_base2 = pair_of(-base, -base);
        Float2Bits sums = pair_of(0.0f, 0.0f);   // the even keys' sum and the odd keys'
        // (Taking a share of the exponentials on the FMA pipe, by a polynomial, was measured: a quarter of them gains 2 %, half
        // of them loses 17 %.)
#pragma unroll
        for (int i = 0; i < kKeysTC / 2; ++i) {
          float x0, x1;
          unpair(fma2(pair_of(sc[2 * i], sc[2 * i + 1]), scale2, minus_base2), x0, x1);
          const float p0 = exp2_approx(x0), p1 = exp2_approx(x1);
          sums = add2(sums, pair_of(p0, p1));
          packed[i] = pack_bf16(p0, p1);
        }
        float sum0, sum1;
        unpair(sums, sum0, sum1);
        row_sum += sum0 + sum1;
        TL(4)
        // P over the first 32 columns of this tile's scores: key 2 i in the lower half of column i, key 2 i + 1 in the upper.  The
        // buffer is free for it: its scores were issued after the product that read P of two tiles back had completed.
        tmem_store_32(tmem + lane_base + b * kKeysTC, packed);
        // The last tile of a request may hold keys past its end whose values were never written: zero those V rows,
        // so that 0 * (whatever is there) stays 0.  A V row is 128 contiguous bytes whatever the swizzle.
        if (key0 + kKeysTC > t.n_keys) {
          const int first_bad = t.n_keys - key0;
          // V of this tile must have landed first (its scores being there says nothing about it: K and V arrive on their own)
          ok = mbar_wait(&sm.v_full[at.stage], at.phase, abort_flag);
          if (!ok) break;
          uint8_t* v_tile = reinterpret_cast<uint8_t*>(sm.v[at.stage]);
          for (int r = first_bad + (row >> 3); r < kKeysTC; r += kRowsTC / 8)
#pragma unroll
            for (int c = 0; c < kSubTiles; ++c)
              *reinterpret_cast<uint4*>(v_tile + c * (kKeysTC * kBoxDims * 2) + (r >> 3) * 1024 + (r & 7) * 128 + (row & 7) * 16) = make_uint4(0, 0, 0, 0);
          asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic-proxy writes -> visible to the tensor core
        }
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");   // P, and a rescaled O, before the product that reads them
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.p_full[b]);
        TL(5)
      }
      // The row tile's output is read when all its products are done: a barrier of its own that completes once (a ring barrier's parity
      // tells only its last phase from the one before, and a warp may be a tile ahead of the slowest one).
      if (ok) ok = mbar_wait(&sm.o_full[u], 0, abort_flag);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const float inv = 1.0f / row_sum;
#pragma unroll
        for (int half = 0; half < kSubTiles; ++half) {   // 64 columns of the output at a time (the load is warp-wide: every row takes part)
          float o[64];
          tmem_ld64(tmem_o + half * 64, o);
          if (row < t.rows_here) {
            __nv_bfloat16* dst = out + ((size_t)(t.row0 + row) * q_heads + head) * kD + half * 64;
#pragma unroll
            for (int c = 0; c < 8; ++c)
              *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(pack_bf16(o[c * 8] * inv, o[c * 8 + 1] * inv), pack_bf16(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv),
                                                                 pack_bf16(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv), pack_bf16(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv));
          }
        }
        if (kCompact && u == 0) {   // the output buffer may be written again
          asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&sm.o_read);
        }
      }
    }
    TL_END(0)
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  }
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicOr(error_flag, 1);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // copies that were issued may still be landing
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols));
  }
}

// [rows, width] bfloat16 with a row stride in elements, boxes of box_rows x 64, 128-byte swizzle.
static bool make_map_2d(CUtensorMap* map, const void* base, long long rows, long long width, long long row_stride, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (fn == nullptr) return false;
  if (rows > 0x7fffffffLL) return false;   // a copy's row is a 32-bit coordinate (a pool this large only exists for tiny heads)
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

#ifdef TLIE_ATTN_TIMELINE
TLIE_EXPORT int tlie_prefill_attention_tc_timeline(long long* host) { return (int)cudaMemcpyFromSymbol(host, tlie_attn_stamps, sizeof(long long) * 24); }
#endif

template <int kD>
static int launch_attention_tc(const void* q, int q_row_stride, int tokens, const void* pages, int num_pages, const int* tiles, int n_tiles,
                               const int* seq_starts, const int* first_positions, const int* block_table, int table_stride, void* out, int q_heads,
                               int kv_heads, int page_size, int window, float scale, int* error_flag, cudaStream_t stream) {
  CUtensorMap map_q, map_kv;
  if (!make_map_2d(&map_q, q, tokens, (long long)q_heads * kD, q_row_stride, kRowsTC)) return (int)cudaErrorInvalidValue;
  if (!make_map_2d(&map_kv, pages, (long long)num_pages * 2 * kv_heads * page_size, kD, kD, kKeysTC)) return (int)cudaErrorInvalidValue;
  // head size 128: exactly the structure, no room to align it by hand (the kernel checks that it need not): 1 KB more and two CTAs no longer share an SM
#ifdef TLIE_ATTN_ONE_PER_SM   // for measurements: so much shared memory that a CTA has its SM to itself
  const int smem = 200 * 1024;
#else
  const int smem = (int)sizeof(SmemTC<kD>) + (kD <= 64 ? 1024 : 0);
#endif
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_attention_tc_kernel<kD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(q_heads, n_tiles);
  return (int)launch_pdl(prefill_attention_tc_kernel<kD>, grid, dim3(kThreadsTC), (size_t)smem, stream, map_q, map_kv, tiles, seq_starts, first_positions,
                         block_table, table_stride, (__nv_bfloat16*)out, q_heads, kv_heads, page_size, window, scale, error_flag);
}

// q: the step's rows [tokens, q_row_stride] starting with the rotated q heads (head size 64 or 128); pages: one layer's pool
// [num_pages, 2, kv_heads, page_size, head size]; tiles: int32 [n_tiles, 4] work items of one or two 128-row tiles (request, first
// row, request or -1, first row); error_flag: device int, zero.
TLIE_EXPORT int tlie_prefill_attention_tc(const void* q, int q_row_stride, int tokens, const void* pages, int num_pages, const int* tiles,
                                          int n_tiles, const int* seq_starts, const int* first_positions, const int* block_table,
                                          int table_stride, void* out, int q_heads, int kv_heads, int head_dim, int page_size, int window, float scale,
                                          int* error_flag, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (kv_heads <= 0 || q_heads % kv_heads != 0 || n_tiles > 65535 || page_size % kKeysTC != 0 || q_row_stride % 8 != 0 || error_flag == nullptr ||
      (head_dim != 64 && head_dim != 128))
    return (int)cudaErrorInvalidValue;
  if (head_dim == 64)
    return launch_attention_tc<64>(q, q_row_stride, tokens, pages, num_pages, tiles, n_tiles, seq_starts, first_positions, block_table, table_stride, out,
                                   q_heads, kv_heads, page_size, window, scale, error_flag, stream);
  return launch_attention_tc<128>(q, q_row_stride, tokens, pages, num_pages, tiles, n_tiles, seq_starts, first_positions, block_table, table_stride, out,
                                  q_heads, kv_heads, page_size, window, scale, error_flag, stream);
}
