// The split-KV decode attention of attention_decode.cu as two steps a kernel strings together: `prologue` works out this
// CTA's key range and starts fetching its cache tiles (nothing it touches depends on the current step's q, k, v), `main`
// reads q, rotates, attends, and merges the parts.  The kernel puts its programmatic-dependency wait between the two.
// What another CTA may have written this step (q, k, v of the new token, the parts) is read through L2.
#pragma once

#include "common.cuh"
#include "mma_utils.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif

namespace tlie {

constexpr int kD = HEAD_DIM;
constexpr int kTileKeys = 32;
#ifndef DECODE_WARPS
#define DECODE_WARPS ((HEAD_DIM <= 64) ? 8 : 4)
#endif
#ifndef DECODE_STAGES
#define DECODE_STAGES 2
#endif
constexpr int kWarps = DECODE_WARPS;
constexpr int kStages = DECODE_STAGES;
constexpr int kRow = kD + 8;                       // padded row, in elements (16 bytes of padding)
constexpr int kTileElems = kTileKeys * kRow;       // one K or V tile
constexpr int kChunks = kD / 8;                    // 16-byte chunks per row
constexpr float kLog2e = 1.4426950408889634f;

// Loads one 32-key tile of K and V of kv head `kvh` into a warp's stage buffer.  Rows whose key is
// outside [lo, n_keys) are zero-filled (their pages may not exist, and 0 * garbage must stay 0).
// A page holds a multiple of 16 keys, so each 16-key half of the tile lies in one page: two table
// lookups per tile, no division per row.
__device__ __forceinline__ void load_tile(__nv_bfloat16* k_smem, __nv_bfloat16* v_smem, const __nv_bfloat16* pages,
                                          const int* table, int key0, int lo, int n_keys, int kvh, int kv_heads,
                                          int page_size, int page_shift, int lane) {
  const size_t plane = (size_t)kv_heads * page_size * kD;
  // A warp runs a few hundred instructions per tile, and at large batches they, not memory, set the kernel's pace: a tile that
  // lies wholly inside [lo, n_keys) (all but a request's first and last) takes the short way, with no row asked whether it counts.
  if (key0 >= lo && key0 + kTileKeys <= n_keys) {
    const __nv_bfloat16* half_base[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int k = key0 + 16 * h;
      const int page_index = page_shift >= 0 ? k >> page_shift : k / page_size;   // pages of a power of two: no division
      half_base[h] = pages + (size_t)table[page_index] * 2 * plane + ((size_t)kvh * page_size + (k - page_index * page_size)) * kD;
    }
    if constexpr (32 % kChunks == 0) {
      // A lane's chunks lie a fixed distance apart, in the page and in the buffer: two source addresses per half of the tile and
      // one destination each for K and V, everything else is an immediate offset (one instruction per 16 bytes, where the general
      // loop below works out two 64-bit addresses for every chunk).
      constexpr int kRowsPerPass = 32 / kChunks;   // rows that one pass of the warp covers: 4 at head size 64, 2 at 128
      const int r = lane / kChunks, c = lane % kChunks;
      const unsigned k_dst = (unsigned)__cvta_generic_to_shared(k_smem + r * kRow + c * 8);
      const unsigned v_dst = (unsigned)__cvta_generic_to_shared(v_smem + r * kRow + c * 8);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const __nv_bfloat16* k_src = half_base[h] + r * kD + c * 8;
        const __nv_bfloat16* v_src = k_src + plane;
#pragma unroll
        for (int i = 0; i < 16 / kRowsPerPass; ++i) {
          constexpr int kRowBytes = kRow * (int)sizeof(__nv_bfloat16);
          cp_async_16_to(k_dst + (h * 16 + i * kRowsPerPass) * kRowBytes, k_src + i * kRowsPerPass * kD);
          cp_async_16_to(v_dst + (h * 16 + i * kRowsPerPass) * kRowBytes, v_src + i * kRowsPerPass * kD);
        }
      }
      return;
    }
#pragma unroll
    for (int idx = lane; idx < kTileKeys * kChunks; idx += 32) {
      const int row = idx / kChunks;
      const int chunk = idx - row * kChunks;
      const __nv_bfloat16* src = (row < 16 ? half_base[0] : half_base[1]) + (row & 15) * kD + chunk * 8;
      cp_async_16(k_smem + row * kRow + chunk * 8, src, true);
      cp_async_16(v_smem + row * kRow + chunk * 8, src + plane, true);
    }
    return;
  }
  const __nv_bfloat16* half_base[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int k = key0 + 16 * h;
    const bool any = k < n_keys && k + 16 > lo;
    const int page = any ? table[k / page_size] : 0;
    half_base[h] = pages + (size_t)page * 2 * plane + ((size_t)kvh * page_size + (k % page_size)) * kD;
  }
#pragma unroll
  for (int idx = lane; idx < kTileKeys * kChunks; idx += 32) {
    const int row = idx / kChunks;
    const int chunk = idx - row * kChunks;
    const int key = key0 + row;
    const bool valid = key >= lo && key < n_keys;
    const __nv_bfloat16* src = (row < 16 ? half_base[0] : half_base[1]) + (row & 15) * kD + chunk * 8;
    cp_async_16(k_smem + row * kRow + chunk * 8, valid ? src : pages, valid);
    cp_async_16(v_smem + row * kRow + chunk * 8, valid ? src + plane : pages, valid);
  }
}

__device__ __forceinline__ float ldcg_bf16(const __nv_bfloat16* p) {
  const unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(p));
  return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&raw));
}

// partial_o: [request, q head, split, D] 32-bit, unnormalised; partial_ml: [request, q head, split, 2] = (max in log2 units, sum).
// fuse_rope: 0 = q is rotated and the cache is written already; 1 = rotate q (and the new key) here with inv_freq
// (full-head rotation, kD % 32 == 0) or not at all if inv_freq is null, and, if write_cache, store the new key and value.
struct DecodeAttnParams {
  const __nv_bfloat16* q;
  int q_row_stride;
  __nv_bfloat16* pages;
  const int* positions;
  const int* block_table;
  int table_stride;
  __nv_bfloat16* out;
  float* partial_o;
  float* partial_ml;
  int* tickets;
  int q_heads, kv_heads, page_size, window;
  int page_shift;   // log2(page_size) if that is a whole number, else -1
  float scale;
  int splits, fuse_rope;
  const float* inv_freq;
  int write_cache;
};

// What a CTA knows about its (request, kv head, part) between the two steps.
struct DecodeAttnItem {
  int seq, kvh, split;
  int pos, n_keys, lo, tile_begin, tile_end, next_load;
  const int* table;
  bool patch_new;
  // cos (first half) and sin (second half) of this position's rotation angles, in shared memory: worked out in the first
  // step, one angle per thread, since positions are known before q is
  float* rotation;
};

constexpr size_t kPipelineBytes = (size_t)kWarps * kStages * 2 * kTileElems * sizeof(__nv_bfloat16);
constexpr size_t kMergeBytes = (size_t)kWarps * 16 * kD * sizeof(float) + (size_t)kWarps * 16 * 2 * sizeof(float);
constexpr size_t kSmemBytes = kPipelineBytes > kMergeBytes ? kPipelineBytes : kMergeBytes;

__device__ __forceinline__ void decode_attn_prologue(const DecodeAttnParams& p, DecodeAttnItem& it, unsigned char* smem_raw) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  it.pos = p.positions[it.seq];
  it.n_keys = it.pos + 1;
  it.lo = (p.window > 0 && it.n_keys > p.window) ? it.n_keys - p.window : 0;
  it.table = p.block_table + (size_t)it.seq * p.table_stride;

  // this CTA's tiles: [it.tile_begin, it.tile_end)
  const int first_tile = it.lo / kTileKeys;
  const int all_tiles = (it.n_keys + kTileKeys - 1) / kTileKeys - first_tile;
  const int per_split = (all_tiles + p.splits - 1) / p.splits;
  it.tile_begin = first_tile + it.split * per_split;
  it.tile_end = min(first_tile + all_tiles, it.tile_begin + per_split);

  __nv_bfloat16* stage_base = reinterpret_cast<__nv_bfloat16*>(smem_raw) + (size_t)warp * kStages * 2 * kTileElems;

  // The new token's key (rotated) and value are not in the cache yet.  The warp that owns the tile holding the
  // new position computes them, stores them in the page for later steps, and patches them into its own copy of
  // the tile in shared memory, so nothing has to travel through global memory first.  (A run that only reads a
  // cache another run wrote finds the key in the page already.)
  it.patch_new = p.fuse_rope && p.write_cache && it.pos / kTileKeys >= it.tile_begin && it.pos / kTileKeys < it.tile_end &&
                         ((it.pos / kTileKeys - it.tile_begin) % kWarps) == warp;

  __shared__ float rotation_table[kD];
  it.rotation = rotation_table;
  if (p.fuse_rope && p.inv_freq != nullptr) {
    for (int d = threadIdx.x; d < kD / 2; d += kWarps * 32) {
      const float angle = (float)it.pos * p.inv_freq[d];
      rotation_table[d] = cosf(angle);
      rotation_table[kD / 2 + d] = sinf(angle);
    }
  }

  // prologue: this warp's tiles are it.tile_begin + warp, + kWarps, ...
  it.next_load = it.tile_begin + warp;
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (it.next_load < it.tile_end) {
      __nv_bfloat16* ks = stage_base + (size_t)s * 2 * kTileElems;
      load_tile(ks, ks + kTileElems, p.pages, it.table, it.next_load * kTileKeys, it.lo, it.n_keys, it.kvh, p.kv_heads, p.page_size, p.page_shift, lane);
    }
    cp_async_commit();
    it.next_load += kWarps;
  }
}

__device__ __forceinline__ void decode_attn_main(const DecodeAttnParams& p, DecodeAttnItem& it, unsigned char* smem_raw, int* last_arrival) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int group = p.q_heads / p.kv_heads;
  __nv_bfloat16* stage_base = reinterpret_cast<__nv_bfloat16*>(smem_raw) + (size_t)warp * kStages * 2 * kTileElems;
  // The warp whose tile holds the new token's position patches that tile with the new key and value (and stores them in the
  // cache).  It asks for them here, together with q, so that both come back in one trip to L2 instead of one after the other.
  constexpr int kNewPerLane = (kD / 2 + 31) / 32, kNewValuesPerLane = (kD + 31) / 32;
  float k_new_first[kNewPerLane], k_new_second[kNewPerLane], v_new_value[kNewValuesPerLane];
  const int new_tile = it.pos / kTileKeys;
  const bool patches = it.patch_new && new_tile >= it.tile_begin + warp && new_tile < it.tile_end && (new_tile - it.tile_begin - warp) % kWarps == 0;
  if (patches) {
    const __nv_bfloat16* k_new = p.q + (size_t)it.seq * p.q_row_stride + (size_t)(p.q_heads + it.kvh) * kD;
    const __nv_bfloat16* v_new = k_new + (size_t)p.kv_heads * kD;
#pragma unroll
    for (int i = 0; i < kNewPerLane; ++i) {
      const int d = lane + 32 * i;
      k_new_first[i] = d < kD / 2 ? ldcg_bf16(k_new + d) : 0.0f;
      k_new_second[i] = d < kD / 2 ? ldcg_bf16(k_new + d + kD / 2) : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < kNewValuesPerLane; ++i) {
      const int d = lane + 32 * i;
      v_new_value[i] = d < kD ? ldcg_bf16(v_new + d) : 0.0f;
    }
  }
  // Q fragments: rows = query heads of the group (row r valid if r < group), k = head dims
  unsigned qa[kD / 16][4];
  {
    const __nv_bfloat16* q_base = p.q + (size_t)it.seq * p.q_row_stride + (size_t)it.kvh * group * kD;
#pragma unroll
    for (int ks = 0; ks < kD / 16; ++ks) {
      const int c0 = ks * 16 + 2 * t;
      const unsigned zero = 0u;
      qa[ks][0] = g < group ? __ldcg(reinterpret_cast<const unsigned*>(q_base + (size_t)g * kD + c0)) : zero;
      qa[ks][1] = g + 8 < group ? __ldcg(reinterpret_cast<const unsigned*>(q_base + (size_t)(g + 8) * kD + c0)) : zero;
      qa[ks][2] = g < group ? __ldcg(reinterpret_cast<const unsigned*>(q_base + (size_t)g * kD + c0 + 8)) : zero;
      qa[ks][3] = g + 8 < group ? __ldcg(reinterpret_cast<const unsigned*>(q_base + (size_t)(g + 8) * kD + c0 + 8)) : zero;
    }
  }

  if (p.fuse_rope && p.inv_freq != nullptr) {
    __syncthreads();   // the rotation table of the first step is complete
    // pair (d, d + kD/2): k-steps ks and ks + kD/32 hold them in the same register slot of the same thread
    if constexpr (kD % 32 == 0) {
#pragma unroll
      for (int ks = 0; ks < kD / 32; ++ks) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int d = ks * 16 + 2 * t + half * 8;
          const float c0 = it.rotation[d], s0 = it.rotation[kD / 2 + d], c1 = it.rotation[d + 1], s1 = it.rotation[kD / 2 + d + 1];
#pragma unroll
          for (int row = 0; row < 2; ++row) {
            const int r = half * 2 + row;
            const __nv_bfloat162 low = *reinterpret_cast<const __nv_bfloat162*>(&qa[ks][r]);
            const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&qa[ks + kD / 32][r]);
            const float f0 = __bfloat162float(low.x), f1 = __bfloat162float(low.y);
            const float g0 = __bfloat162float(hi.x), g1 = __bfloat162float(hi.y);
            qa[ks][r] = pack_bf16(f0 * c0 - g0 * s0, f1 * c1 - g1 * s1);
            qa[ks + kD / 32][r] = pack_bf16(g0 * c0 + f0 * s0, g1 * c1 + f1 * s1);
          }
        }
      }
    }
  }

  float o[kD / 8][4];
#pragma unroll
  for (int i = 0; i < kD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float row_max[2] = {-INFINITY, -INFINITY};
  float row_sum[2] = {0.0f, 0.0f};
  const float sl2 = p.scale * kLog2e;
  const bool upper_rows = group > 8;

  int stage = 0;
  for (int tile = it.tile_begin + warp; tile < it.tile_end; tile += kWarps) {
    // prefetch the tile kStages-1 ahead into the stage consumed last iteration
    {
      const int s = (stage + kStages - 1) % kStages;
      if (it.next_load < it.tile_end) {
        __nv_bfloat16* ks = stage_base + (size_t)s * 2 * kTileElems;
        load_tile(ks, ks + kTileElems, p.pages, it.table, it.next_load * kTileKeys, it.lo, it.n_keys, it.kvh, p.kv_heads, p.page_size, p.page_shift, lane);
      }
      cp_async_commit();
      it.next_load += kWarps;
    }
    cp_async_wait<kStages - 1>();
    __syncwarp();
    __nv_bfloat16* k_smem = stage_base + (size_t)stage * 2 * kTileElems;
    __nv_bfloat16* v_smem = k_smem + kTileElems;
    if (patches && tile == new_tile) {
      const size_t plane = (size_t)p.kv_heads * p.page_size * kD;
      __nv_bfloat16* k_dst = p.pages + (size_t)it.table[it.pos / p.page_size] * 2 * plane + ((size_t)it.kvh * p.page_size + (it.pos % p.page_size)) * kD;
      const int row = it.pos % kTileKeys;
#pragma unroll
      for (int i = 0; i < kNewPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d >= kD / 2) break;
        float first = k_new_first[i], second = k_new_second[i];
        if (p.inv_freq != nullptr) {
          const float c = it.rotation[d], sn = it.rotation[kD / 2 + d];
          const float a = first * c - second * sn, b = second * c + first * sn;
          first = a;
          second = b;
        }
        const __nv_bfloat16 kf = __float2bfloat16_rn(first), ks2 = __float2bfloat16_rn(second);
        k_smem[row * kRow + d] = kf;
        k_smem[row * kRow + d + kD / 2] = ks2;
        k_dst[d] = kf;
        k_dst[d + kD / 2] = ks2;
      }
#pragma unroll
      for (int i = 0; i < kNewValuesPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d >= kD) break;
        const __nv_bfloat16 v = __float2bfloat16_rn(v_new_value[i]);
        v_smem[row * kRow + d] = v;
        k_dst[plane + d] = v;
      }
      __syncwarp();
    }

    // S = Q . K^T  (16 rows x 32 keys)
    float s_frag[kTileKeys / 8][4];
#pragma unroll
    for (int j = 0; j < kTileKeys / 8; ++j) s_frag[j][0] = s_frag[j][1] = s_frag[j][2] = s_frag[j][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < kD / 16; ++ks) {
#pragma unroll
      for (int jp = 0; jp < kTileKeys / 16; ++jp) {
        unsigned b[4];
        const int row = (jp * 2 + (lane >> 4)) * 8 + (lane & 7);
        const int col = ks * 16 + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(b, k_smem + row * kRow + col);
        mma_bf16(s_frag[jp * 2], qa[ks], b[0], b[1]);
        mma_bf16(s_frag[jp * 2 + 1], qa[ks], b[2], b[3]);
      }
    }
    // mask and online softmax (log2 domain); only a request's first and last tile hold keys that do not count.  The scores stay
    // as the product left them: the scale goes into the exponent's multiply-add (it is positive, so the maximum can be taken first).
    // Rows 8..15 of the tile exist only for groups of more than eight query heads: otherwise nothing is worked out for them.
    const int key0 = tile * kTileKeys;
    float tile_max[2] = {-INFINITY, -INFINITY};
    if (!(key0 >= it.lo && key0 + kTileKeys <= it.n_keys)) {
#pragma unroll
      for (int j = 0; j < kTileKeys / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key0 + j * 8 + 2 * t + (e & 1);
          if (!(key >= it.lo && key < it.n_keys)) s_frag[j][e] = -INFINITY;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kTileKeys / 8; ++j) tile_max[0] = fmaxf(tile_max[0], fmaxf(s_frag[j][0], s_frag[j][1]));
    if (upper_rows) {
#pragma unroll
      for (int j = 0; j < kTileKeys / 8; ++j) tile_max[1] = fmaxf(tile_max[1], fmaxf(s_frag[j][2], s_frag[j][3]));
    }
    float rescale[2] = {1.0f, 1.0f};
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (r == 1 && !upper_rows) break;
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
      const float new_max = fmaxf(row_max[r], tile_max[r] * sl2);
      // a tile holds at least one valid key (tiles start at or after it.lo's tile and before it.n_keys), so new_max is finite
      rescale[r] = exp2f(row_max[r] - new_max);
      row_max[r] = new_max;
      row_sum[r] *= rescale[r];
    }
    unsigned pa[kTileKeys / 16][4];
#pragma unroll
    for (int j = 0; j < kTileKeys / 8; ++j) {
      const float p0 = exp2_approx(fmaf(s_frag[j][0], sl2, -row_max[0]));
      const float p1 = exp2_approx(fmaf(s_frag[j][1], sl2, -row_max[0]));
      row_sum[0] += p0 + p1;
      pa[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
      pa[j >> 1][(j & 1) * 2 + 1] = 0u;
    }
    if (upper_rows) {
#pragma unroll
      for (int j = 0; j < kTileKeys / 8; ++j) {
        const float p2 = exp2_approx(fmaf(s_frag[j][2], sl2, -row_max[1]));
        const float p3 = exp2_approx(fmaf(s_frag[j][3], sl2, -row_max[1]));
        row_sum[1] += p2 + p3;
        pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
    }
    if (__any_sync(0xffffffffu, rescale[0] != 1.0f || rescale[1] != 1.0f)) {   // after a request's first tiles the maxima seldom move
#pragma unroll
      for (int i = 0; i < kD / 8; ++i) {
        o[i][0] *= rescale[0];
        o[i][1] *= rescale[0];
        o[i][2] *= rescale[1];
        o[i][3] *= rescale[1];
      }
    }
    // O += P . V
#pragma unroll
    for (int kk = 0; kk < kTileKeys / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < kD / 16; ++np) {
        unsigned b[4];
        const int row = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
        const int col = np * 16 + (lane >> 4) * 8;
        ldmatrix_x4_trans(b, v_smem + row * kRow + col);
        mma_bf16(o[np * 2], pa[kk], b[0], b[1]);
        mma_bf16(o[np * 2 + 1], pa[kk], b[2], b[3]);
      }
    }
    __syncwarp();
    stage = (stage + 1) % kStages;
  }
  cp_async_wait<0>();
  // row sums live in the four threads of a quad
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
  }
  __syncthreads();  // every warp is done with its stage buffers: reuse them to merge the warps

  float* merge_o = reinterpret_cast<float*>(smem_raw);                   // [warp][16][kD]
  float* merge_ml = merge_o + kWarps * 16 * kD;                          // [warp][16][2]
#pragma unroll
  for (int i = 0; i < kD / 8; ++i) {
    float* base = merge_o + ((size_t)warp * 16) * kD + i * 8 + 2 * t;
    base[(size_t)g * kD] = o[i][0];
    base[(size_t)g * kD + 1] = o[i][1];
    base[(size_t)(g + 8) * kD] = o[i][2];
    base[(size_t)(g + 8) * kD + 1] = o[i][3];
  }
  if (t == 0) {
    merge_ml[(warp * 16 + g) * 2] = row_max[0];
    merge_ml[(warp * 16 + g) * 2 + 1] = row_sum[0];
    merge_ml[(warp * 16 + g + 8) * 2] = row_max[1];
    merge_ml[(warp * 16 + g + 8) * 2 + 1] = row_sum[1];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < group * kD; idx += kWarps * 32) {
    const int r = idx / kD;
    const int d = idx - r * kD;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) m = fmaxf(m, merge_ml[(w * 16 + r) * 2]);
    float acc = 0.0f, sum = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float wm = merge_ml[(w * 16 + r) * 2];
      const float f = (wm == -INFINITY) ? 0.0f : exp2f(wm - m);
      acc += f * merge_o[((size_t)w * 16 + r) * kD + d];
      sum += f * merge_ml[(w * 16 + r) * 2 + 1];
    }
    const int head = it.kvh * group + r;
    if (p.splits == 1) {
      p.out[((size_t)it.seq * p.q_heads + head) * kD + d] = __float2bfloat16_rn(acc / sum);
    } else {
      const size_t slot = ((size_t)it.seq * p.q_heads + head) * p.splits + it.split;
      p.partial_o[slot * kD + d] = acc;
      if (d == 0) {
        p.partial_ml[slot * 2] = m;       // -inf when this it.split had no keys
        p.partial_ml[slot * 2 + 1] = sum;
      }
    }
  }
  if (p.splits == 1) return;
  // The CTA of this (request, kv head) that arrives last merges all parts.  No CTA waits for another.
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(&p.tickets[it.seq * p.kv_heads + it.kvh], 1);
    *last_arrival = (ticket == p.splits - 1);
  }
  __syncthreads();
  if (!*last_arrival) return;
  __threadfence();
  // One warp per query head, lane sp holds part sp's maximum and sum (p.splits <= 32).  The parts' outputs do not depend
  // on those, so their loads go out first, eight parts at a time, and everything is one trip to L2 and back.
  for (int r = warp; r < group; r += kWarps) {
    const size_t pair = (size_t)it.seq * p.q_heads + it.kvh * group + r;
    const float* ml = p.partial_ml + pair * p.splits * 2;
    constexpr int kPerLane = (kD + 31) / 32;
    float acc[kPerLane];
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) acc[i] = 0.0f;
    float part_max = -INFINITY, part_sum = 0.0f, m = 0.0f, f = 0.0f, sum = 0.0f;
    for (int sp0 = 0; sp0 < p.splits; sp0 += 8) {
      float part[8][kPerLane];
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
          const int d = lane + 32 * i;
          part[j][i] = (sp0 + j < p.splits && d < kD) ? __ldcg(p.partial_o + (pair * p.splits + sp0 + j) * kD + d) : 0.0f;
        }
      if (sp0 == 0) {
        if (lane < p.splits) {
          part_max = __ldcg(ml + lane * 2);
          part_sum = __ldcg(ml + lane * 2 + 1);
        }
        m = warp_max(part_max);
        f = (part_max == -INFINITY) ? 0.0f : exp2f(part_max - m);
        sum = warp_sum(f * part_sum);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float fs = __shfl_sync(0xffffffffu, f, (sp0 + j) & 31);
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) acc[i] += fs * part[j][i];   // parts past p.splits were loaded as zeros
      }
    }
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < kD) p.out[pair * kD + d] = __float2bfloat16_rn(acc[i] / sum);
    }
  }
  if (threadIdx.x == 0) p.tickets[it.seq * p.kv_heads + it.kvh] = 0;   // ready for the next launch
}

}  // namespace tlie
