// Split-KV paged grouped-query attention for decode steps (one query token per request), bfloat16.
//
// Replaces the reference's one-block-per-head decode kernel, which keeps every score in shared
// memory and sums P.V serially (src/cuda/kernels.cu:147-196).  Same mathematics
// (src/operators.cpp:102-146): out = softmax(q.K^T * scale) . V over keys lo..pos, 32-bit softmax.
//
// Decode attention is bound by reading the cache, so the design is about bytes in flight:
//   * one CTA per (request, kv head, split of the key range); the query heads that share the
//     kv head (the group, up to 16) are the rows of one tensor-core tile, so every key and value
//     is read from HBM once per group, not once per head;
//   * the key range of a request is cut into SPLITS parts so that small batches still fill the
//     148 SMs; a second small kernel merges the parts (none is needed when SPLITS == 1);
//   * each of the four warps of a CTA walks its own 32-key tiles with a private multi-stage
//     cp.async pipeline (no block-wide barrier in the loop); rows in shared memory are padded
//     by 16 bytes so that ldmatrix reads are free of bank conflicts for any head size;
//   * q.K^T and P.V run on the tensor cores (mma.sync m16n8k16, bf16 in, 32-bit accumulate):
//     with at most 16 rows per tile the 128-row tcgen05 shapes would be idle weight, and the
//     CUDA cores alone cannot keep up with 8 flop per cache byte at HBM speed.
//   * the rotation of q and of the new key (src/operators.cpp:47-78) and the write of the new key and
//     value into the request's page happen here too when the caller asks for it: q is rotated in the
//     registers of its tensor-core fragments, and the CTA whose key range holds the new position
//     stores k and v before it starts reading, so a decode step needs no separate rotation / cache
//     write kernel (src/cuda/kernels.cu:86-145 in the reference);
//   * the parts are merged by whichever CTA of a (request, kv head) finishes last (a counter in
//     scratch memory, reset by that CTA), not by a second kernel; nobody waits for anybody.
// The grid depends only on (requests, kv heads, SPLITS); lengths are read on the device, so one
// captured graph serves every later step.
//
// Compile-time: HEAD_DIM (multiple of 16, <= 256).
#include "attention_decode.h"
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
                                          int page_size, int lane) {
  const size_t plane = (size_t)kv_heads * page_size * kD;
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

// partial_o: [request, q head, split, D] 32-bit, unnormalised; partial_ml: [request, q head, split, 2] = (max in log2 units, sum).
// fuse_rope: 0 = q is rotated and the cache is written already; 1 = rotate q (and the new key) here with inv_freq
// (full-head rotation, kD % 32 == 0) or not at all if inv_freq is null, and, if write_cache, store the new key and value.
__global__ void __launch_bounds__(kWarps * 32)
    decode_attention_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride, __nv_bfloat16* __restrict__ pages,
                            const int* __restrict__ positions, const int* __restrict__ block_table, int table_stride,
                            __nv_bfloat16* __restrict__ out, float* __restrict__ partial_o, float* __restrict__ partial_ml,
                            int* __restrict__ tickets, int q_heads, int kv_heads, int page_size, int window, float scale,
                            int splits, int fuse_rope, const float* __restrict__ inv_freq, int write_cache) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int last_arrival;
  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int group = q_heads / kv_heads;
  grid_launch_dependents();
  // With fuse_rope nothing this kernel reads before its q comes from the kernel just before it: positions and block
  // tables were set before the step began, and every cached key but the new one is from earlier steps.  So the cache
  // tiles are fetched first and the wait for the previous kernel (which produces q, k, v of the new token) comes after.
  if (!fuse_rope) grid_dependency_wait();
  const int pos = positions[seq];
  const int n_keys = pos + 1;
  const int lo = (window > 0 && n_keys > window) ? n_keys - window : 0;
  const int* table = block_table + (size_t)seq * table_stride;

  // this CTA's tiles: [tile_begin, tile_end)
  const int first_tile = lo / kTileKeys;
  const int all_tiles = (n_keys + kTileKeys - 1) / kTileKeys - first_tile;
  const int per_split = (all_tiles + splits - 1) / splits;
  const int tile_begin = first_tile + split * per_split;
  const int tile_end = min(first_tile + all_tiles, tile_begin + per_split);

  __nv_bfloat16* stage_base = reinterpret_cast<__nv_bfloat16*>(smem_raw) + (size_t)warp * kStages * 2 * kTileElems;

  // The new token's key (rotated) and value are not in the cache yet.  The warp that owns the tile holding the
  // new position computes them, stores them in the page for later steps, and patches them into its own copy of
  // the tile in shared memory, so nothing has to travel through global memory first.  (A run that only reads a
  // cache another run wrote finds the key in the page already.)
  const bool patch_new = fuse_rope && write_cache && pos / kTileKeys >= tile_begin && pos / kTileKeys < tile_end &&
                         ((pos / kTileKeys - tile_begin) % kWarps) == warp;

  // prologue: this warp's tiles are tile_begin + warp, + kWarps, ...
  int next_load = tile_begin + warp;
#pragma unroll
  for (int s = 0; s < kStages - 1; ++s) {
    if (next_load < tile_end) {
      __nv_bfloat16* ks = stage_base + (size_t)s * 2 * kTileElems;
      load_tile(ks, ks + kTileElems, pages, table, next_load * kTileKeys, lo, n_keys, kvh, kv_heads, page_size, lane);
    }
    cp_async_commit();
    next_load += kWarps;
  }
  if (fuse_rope) grid_dependency_wait();

  // Q fragments: rows = query heads of the group (row r valid if r < group), k = head dims
  unsigned qa[kD / 16][4];
  {
    const __nv_bfloat16* q_base = q + (size_t)seq * q_row_stride + (size_t)kvh * group * kD;
#pragma unroll
    for (int ks = 0; ks < kD / 16; ++ks) {
      const int c0 = ks * 16 + 2 * t;
      const unsigned zero = 0u;
      qa[ks][0] = g < group ? *reinterpret_cast<const unsigned*>(q_base + (size_t)g * kD + c0) : zero;
      qa[ks][1] = g + 8 < group ? *reinterpret_cast<const unsigned*>(q_base + (size_t)(g + 8) * kD + c0) : zero;
      qa[ks][2] = g < group ? *reinterpret_cast<const unsigned*>(q_base + (size_t)g * kD + c0 + 8) : zero;
      qa[ks][3] = g + 8 < group ? *reinterpret_cast<const unsigned*>(q_base + (size_t)(g + 8) * kD + c0 + 8) : zero;
    }
  }

  if (fuse_rope && inv_freq != nullptr) {
    // pair (d, d + kD/2): k-steps ks and ks + kD/32 hold them in the same register slot of the same thread
    if constexpr (kD % 32 == 0) {
#pragma unroll
      for (int ks = 0; ks < kD / 32; ++ks) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int d = ks * 16 + 2 * t + half * 8;
          const float a0 = (float)pos * inv_freq[d], a1 = (float)pos * inv_freq[d + 1];
          const float c0 = cosf(a0), s0 = sinf(a0), c1 = cosf(a1), s1 = sinf(a1);
#pragma unroll
          for (int row = 0; row < 2; ++row) {
            const int r = half * 2 + row;
            const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&qa[ks][r]);
            const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&qa[ks + kD / 32][r]);
            const float f0 = __bfloat162float(lo.x), f1 = __bfloat162float(lo.y);
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
  const float sl2 = scale * kLog2e;

  int stage = 0;
  for (int tile = tile_begin + warp; tile < tile_end; tile += kWarps) {
    // prefetch the tile kStages-1 ahead into the stage consumed last iteration
    {
      const int s = (stage + kStages - 1) % kStages;
      if (next_load < tile_end) {
        __nv_bfloat16* ks = stage_base + (size_t)s * 2 * kTileElems;
        load_tile(ks, ks + kTileElems, pages, table, next_load * kTileKeys, lo, n_keys, kvh, kv_heads, page_size, lane);
      }
      cp_async_commit();
      next_load += kWarps;
    }
    cp_async_wait<kStages - 1>();
    __syncwarp();
    __nv_bfloat16* k_smem = stage_base + (size_t)stage * 2 * kTileElems;
    __nv_bfloat16* v_smem = k_smem + kTileElems;
    if (patch_new && tile == pos / kTileKeys) {
      const __nv_bfloat16* k_new = q + (size_t)seq * q_row_stride + (size_t)(q_heads + kvh) * kD;
      const __nv_bfloat16* v_new = k_new + (size_t)kv_heads * kD;
      const size_t plane = (size_t)kv_heads * page_size * kD;
      __nv_bfloat16* k_dst = pages + (size_t)table[pos / page_size] * 2 * plane + ((size_t)kvh * page_size + (pos % page_size)) * kD;
      const int row = pos % kTileKeys;
      for (int d = lane; d < kD / 2; d += 32) {
        float first = __bfloat162float(k_new[d]), second = __bfloat162float(k_new[d + kD / 2]);
        if (inv_freq != nullptr) {
          const float angle = (float)pos * inv_freq[d];
          const float c = cosf(angle), sn = sinf(angle);
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
      for (int d = lane; d < kD; d += 32) {
        const __nv_bfloat16 v = v_new[d];
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
    // mask and online softmax (log2 domain)
    const int key0 = tile * kTileKeys;
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < kTileKeys / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + j * 8 + 2 * t + (e & 1);
        const float v = (key >= lo && key < n_keys) ? s_frag[j][e] * sl2 : -INFINITY;
        s_frag[j][e] = v;
        tile_max[e >> 1] = fmaxf(tile_max[e >> 1], v);
      }
    }
    float rescale[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
      const float new_max = fmaxf(row_max[r], tile_max[r]);
      // a tile holds at least one valid key (tiles start at or after lo's tile and before n_keys), so new_max is finite
      rescale[r] = exp2f(row_max[r] - new_max);
      row_max[r] = new_max;
      row_sum[r] *= rescale[r];
    }
    unsigned pa[kTileKeys / 16][4];
#pragma unroll
    for (int j = 0; j < kTileKeys / 8; ++j) {
      const float p0 = exp2f(s_frag[j][0] - row_max[0]);
      const float p1 = exp2f(s_frag[j][1] - row_max[0]);
      const float p2 = exp2f(s_frag[j][2] - row_max[1]);
      const float p3 = exp2f(s_frag[j][3] - row_max[1]);
      row_sum[0] += p0 + p1;
      row_sum[1] += p2 + p3;
      pa[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
      pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int i = 0; i < kD / 8; ++i) {
      o[i][0] *= rescale[0];
      o[i][1] *= rescale[0];
      o[i][2] *= rescale[1];
      o[i][3] *= rescale[1];
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
    const int head = kvh * group + r;
    if (splits == 1) {
      out[((size_t)seq * q_heads + head) * kD + d] = __float2bfloat16_rn(acc / sum);
    } else {
      const size_t slot = ((size_t)seq * q_heads + head) * splits + split;
      partial_o[slot * kD + d] = acc;
      if (d == 0) {
        partial_ml[slot * 2] = m;       // -inf when this split had no keys
        partial_ml[slot * 2 + 1] = sum;
      }
    }
  }
  if (splits == 1) return;
  // The CTA of this (request, kv head) that arrives last merges all parts.  No CTA waits for another.
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(&tickets[seq * kv_heads + kvh], 1);
    last_arrival = (ticket == splits - 1);
  }
  __syncthreads();
  if (!last_arrival) return;
  __threadfence();
  // one warp per query head; lane sp holds part sp's maximum and sum (splits <= 32), so every load is issued at once
  for (int r = warp; r < group; r += kWarps) {
    const size_t pair = (size_t)seq * q_heads + kvh * group + r;
    const float* ml = partial_ml + pair * splits * 2;
    float part_max = -INFINITY, part_sum = 0.0f;
    if (lane < splits) {
      part_max = __ldcg(ml + lane * 2);
      part_sum = __ldcg(ml + lane * 2 + 1);
    }
    const float m = warp_max(part_max);
    const float f = (part_max == -INFINITY) ? 0.0f : exp2f(part_max - m);
    const float sum = warp_sum(f * part_sum);
    for (int d0 = 0; d0 < kD; d0 += 32) {
      const int d = d0 + lane;
      float acc = 0.0f;
#pragma unroll 8
      for (int sp = 0; sp < splits; ++sp) {
        const float fs = __shfl_sync(0xffffffffu, f, sp);
        if (d < kD) acc += fs * __ldcg(partial_o + (pair * splits + sp) * kD + d);
      }
      if (d < kD) out[pair * kD + d] = __float2bfloat16_rn(acc / sum);
    }
  }
  if (threadIdx.x == 0) tickets[seq * kv_heads + kvh] = 0;   // ready for the next launch
}

constexpr size_t kPipelineBytes = (size_t)kWarps * kStages * 2 * kTileElems * sizeof(__nv_bfloat16);
constexpr size_t kMergeBytes = (size_t)kWarps * 16 * kD * sizeof(float) + (size_t)kWarps * 16 * 2 * sizeof(float);
constexpr size_t kSmemBytes = kPipelineBytes > kMergeBytes ? kPipelineBytes : kMergeBytes;

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_decode_attention_head_dim() { return kD; }

constexpr int kMaxTickets = 16384;   // requests * kv_heads a launch may have

// Scratch: kMaxTickets counters (zero when first used; every launch leaves them zero), then for splits > 1 the parts.
TLIE_EXPORT long long tlie_decode_attention_scratch_floats(int requests, int q_heads, int splits) {
  return kMaxTickets + (splits <= 1 ? 0 : (long long)requests * q_heads * splits * (kD + 2));
}

// fuse_rope 0: q in `q` is rotated and the cache holds the new keys.  fuse_rope 1: rows of `q` are [q | k | v] of the new
// token, unrotated; inv_freq (kD / 2 frequencies, or null for no rotation) rotates q and k here, and write_cache stores k, v.
TLIE_EXPORT int tlie_decode_attention(const void* q, int q_row_stride, void* pages, const int* positions,
                                      const int* block_table, int table_stride, void* out, float* scratch, int requests,
                                      int q_heads, int kv_heads, int page_size, int window, float scale, int splits,
                                      int fuse_rope, const float* inv_freq, int write_cache, cudaStream_t stream) {
  if (requests <= 0) return 0;
  if (kv_heads <= 0 || q_heads % kv_heads != 0 || q_heads / kv_heads > 16 || splits < 1 || splits > 32 || scratch == nullptr ||
      (long long)requests * kv_heads > kMaxTickets || (fuse_rope && inv_freq != nullptr && kD % 32 != 0))
    return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int* tickets = reinterpret_cast<int*>(scratch);
  float* partial_o = scratch + kMaxTickets;
  float* partial_ml = partial_o + (size_t)requests * q_heads * splits * kD;
  dim3 grid(splits, kv_heads, requests);
  return (int)launch_pdl(decode_attention_kernel, grid, dim3(kWarps * 32), kSmemBytes, stream, (const __nv_bfloat16*)q, q_row_stride,
                         (__nv_bfloat16*)pages, positions, block_table, table_stride, (__nv_bfloat16*)out, partial_o, partial_ml,
                         tickets, q_heads, kv_heads, page_size, window, scale, splits, fuse_rope, inv_freq, write_cache);
}

// --- the entry point that allocates nothing (declared and documented in attention_decode.h) --------------------
constexpr int kStaticMaxSlots = 8192;   // (request, head, part) triples the built-in scratch has room for
constexpr size_t kStaticScratchFloats = (size_t)kMaxTickets + (size_t)kStaticMaxSlots * (kD + 2);
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address: the address a kernel can
// use is looked up once per device, with that device current.
static float* static_scratch_address(cudaError_t* error) {
  static float* address[64] = {};
  int device = 0;
  *error = cudaGetDevice(&device);
  if (*error != cudaSuccess) return nullptr;
  if (device < 0 || device >= 64) {
    *error = cudaErrorInvalidDevice;
    return nullptr;
  }
  if (address[device] == nullptr) {
    void* found = nullptr;
    *error = cudaGetSymbolAddress(&found, g_static_scratch);
    if (*error != cudaSuccess) return nullptr;
    address[device] = static_cast<float*>(found);
  }
  return address[device];
}

TLIE_EXPORT int tlie_decode_attention_static(const void* q, int q_row_stride, void* pages, const int* positions,
                                             const int* block_table, int table_stride, void* out, int requests,
                                             int q_heads, int kv_heads, int page_size, int window, float scale, int splits,
                                             int fuse_rope, const float* inv_freq, int write_cache, cudaStream_t stream) {
  if (requests <= 0) return 0;
  if (splits < 1 || q_heads <= 0 || (long long)requests * q_heads * splits > kStaticMaxSlots ||
      (long long)requests * kv_heads > kMaxTickets)
    return (int)cudaErrorInvalidValue;   // beyond the built-in scratch: nothing is launched
  cudaError_t error = cudaSuccess;
  float* scratch = static_scratch_address(&error);
  if (scratch == nullptr) return (int)error;
  // the arrival counters must start at zero; the rest of the array is written before it is read
  error = cudaMemsetAsync(scratch, 0, (size_t)requests * kv_heads * sizeof(int), stream);
  if (error != cudaSuccess) return (int)error;
  return tlie_decode_attention(q, q_row_stride, pages, positions, block_table, table_stride, out, scratch, requests, q_heads,
                               kv_heads, page_size, window, scale, splits, fuse_rope, inv_freq, write_cache, stream);
}
