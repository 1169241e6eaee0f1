// Paged grouped-query flash attention for prompt portions (and any mixed batch), bfloat16.
//
// The reference has no kernel that takes more than one query token (prompts go through its decode
// kernel one token at a time, docs/adr/0002-m2-fp16-cuda-contracts.md:65-66).  Mathematics as in
// src/operators.cpp:102-146 for every row: a query at absolute position p of its request attends to
// the cached keys lo..p of that request (lo = max(0, p - window + 1) with a window), with a 32-bit
// running maximum and sum, so the scores are never materialised.
//
// Work is a host-built list of tiles (request, first row): up to PREFILL_ROWS (64) consecutive query rows of one request,
// one CTA per (tile, query head), one warp per 16 rows.  Keys and values stream through shared
// memory in 64-key tiles with a two-stage cp.async pipeline, read through the request's block table
// (rows padded by 16 bytes: ldmatrix without bank conflicts at any head size); q.K^T and P.V run on
// the tensor cores (mma.sync m16n8k16, bf16 in, 32-bit accumulate).  The eight query heads of a
// TinyLlama group re-read their kv head's tiles from L2, not from HBM.
//
// Compile-time: HEAD_DIM (multiple of 16, <= 128 here).
#include "common.cuh"
#include "mma_utils.cuh"

#ifndef HEAD_DIM
#define HEAD_DIM 64
#endif

namespace tlie {

constexpr int kD = HEAD_DIM;
#ifndef PREFILL_ROWS
#define PREFILL_ROWS 64
#endif
constexpr int kRows = PREFILL_ROWS;   // query rows per CTA (16 per warp)
constexpr int kKeys = 64;             // keys per tile
constexpr int kWarps = kRows / 16;
constexpr int kRow = kD + 8;    // padded shared-memory row (elements)
constexpr int kChunks = kD / 8;
constexpr float kLog2e = 1.4426950408889634f;

// A page holds a multiple of 16 keys, so each 16-key quarter of a tile lies in one page: the table is read
// once per quarter, not once per row.
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* k_smem, __nv_bfloat16* v_smem, const __nv_bfloat16* pages,
                                             const int* table, int key0, int lo, int n_keys, int kvh, int kv_heads,
                                             int page_size) {
  const size_t plane = (size_t)kv_heads * page_size * kD;
  const __nv_bfloat16* quarter_base[kKeys / 16];
#pragma unroll
  for (int h = 0; h < kKeys / 16; ++h) {
    const int k = key0 + 16 * h;
    const bool any = k < n_keys && k + 16 > lo;
    const int page = any ? table[k / page_size] : 0;
    quarter_base[h] = pages + (size_t)page * 2 * plane + ((size_t)kvh * page_size + (k % page_size)) * kD;
  }
#pragma unroll
  for (int idx = threadIdx.x; idx < kKeys * kChunks; idx += kWarps * 32) {
    const int row = idx / kChunks;
    const int chunk = idx - row * kChunks;
    const int key = key0 + row;
    const bool valid = key >= lo && key < n_keys;
    const int quarter = row >> 4;
    const __nv_bfloat16* src = (quarter == 0 ? quarter_base[0] : quarter == 1 ? quarter_base[1] : quarter == 2 ? quarter_base[2] : quarter_base[3]) + (row & 15) * kD + chunk * 8;
    cp_async_16(k_smem + row * kRow + chunk * 8, valid ? src : pages, valid);
    cp_async_16(v_smem + row * kRow + chunk * 8, valid ? src + plane : pages, valid);
  }
}

// tiles: [n_tiles][2] = (request index in the step, first row of the tile in the step's row numbering)
__global__ void __launch_bounds__(kWarps * 32, kD <= 64 ? (kRows == 64 ? 3 : 2) : 1)
    prefill_attention_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride, const __nv_bfloat16* __restrict__ pages,
                             const int* __restrict__ tiles, const int* __restrict__ seq_starts,
                             const int* __restrict__ first_positions, const int* __restrict__ block_table, int table_stride,
                             __nv_bfloat16* __restrict__ out, int q_heads, int kv_heads, int page_size, int window, float scale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* q_smem = smem;                                   // [64][kRow]
  __nv_bfloat16* kv_smem = smem + kRows * kRow;                   // [2 stages][K, V][64][kRow]
  // later tiles of a request see more keys and take longer: start them first so that the tail of the grid is short
  const int tile_index = gridDim.x - 1 - blockIdx.x;
  const int seq = tiles[tile_index * 2];
  const int row0 = tiles[tile_index * 2 + 1];
  const int head = blockIdx.y;
  const int kvh = head / (q_heads / kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int seq_start = seq_starts[seq];
  const int rows_here = min(kRows, seq_starts[seq + 1] - row0);    // valid rows of this tile
  const int pos0 = first_positions[seq] + (row0 - seq_start);      // position of the tile's first row
  const int last_pos = pos0 + rows_here - 1;
  const int n_keys = last_pos + 1;
  const int lo_tile = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;  // lowest key any row reads
  const int* table = block_table + (size_t)seq * table_stride;

  // Q tile -> shared memory (rows past the end repeat nothing: zero-filled)
  for (int idx = threadIdx.x; idx < kRows * kChunks; idx += kWarps * 32) {
    const int row = idx / kChunks;
    const int chunk = idx - row * kChunks;
    const bool valid = row < rows_here;
    const __nv_bfloat16* src = q + (size_t)(row0 + (valid ? row : 0)) * q_row_stride + (size_t)head * kD + chunk * 8;
    cp_async_16(q_smem + row * kRow + chunk * 8, src, valid);
  }
  cp_async_commit();

  const int first_tile = lo_tile / kKeys;
  const int end_tile = (n_keys + kKeys - 1) / kKeys;
  auto stage_k = [&](int s) { return kv_smem + (size_t)s * 2 * kKeys * kRow; };
  load_kv_tile(stage_k(0), stage_k(0) + kKeys * kRow, pages, table, first_tile * kKeys, lo_tile, n_keys, kvh, kv_heads, page_size);
  cp_async_commit();

  cp_async_wait<1>();   // Q has landed
  __syncthreads();
  unsigned qa[kD / 16][4];
#pragma unroll
  for (int ks = 0; ks < kD / 16; ++ks) {
    const int row = warp * 16 + (lane & 15);
    const int col = ks * 16 + (lane >> 4) * 8;
    ldmatrix_x4(qa[ks], q_smem + row * kRow + col);
  }

  // the two rows this thread owns
  const int my_row[2] = {warp * 16 + g, warp * 16 + g + 8};
  int my_pos[2], my_lo[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    my_pos[r] = pos0 + min(my_row[r], rows_here - 1);   // rows past the end behave like the last row; never stored
    my_lo[r] = (window > 0 && my_pos[r] - window + 1 > 0) ? my_pos[r] - window + 1 : 0;
  }

  float o[kD / 8][4];
#pragma unroll
  for (int i = 0; i < kD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  float row_max[2] = {-INFINITY, -INFINITY};
  float row_sum[2] = {0.0f, 0.0f};
  const float sl2 = scale * kLog2e;

  for (int tile = first_tile; tile < end_tile; ++tile) {
    const int stage = (tile - first_tile) & 1;
    if (tile + 1 < end_tile) {
      __nv_bfloat16* ks = stage_k(stage ^ 1);
      load_kv_tile(ks, ks + kKeys * kRow, pages, table, (tile + 1) * kKeys, lo_tile, n_keys, kvh, kv_heads, page_size);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const __nv_bfloat16* k_smem = stage_k(stage);
    const __nv_bfloat16* v_smem = k_smem + kKeys * kRow;
    const int key0 = tile * kKeys;
    // a warp whose 16 rows all lie before this tile's first key has nothing to do here (causal)
    const int warp_last_pos = pos0 + min(warp * 16 + 15, rows_here - 1);
    if (key0 <= warp_last_pos) {
      float s_frag[kKeys / 8][4];
#pragma unroll
      for (int j = 0; j < kKeys / 8; ++j) s_frag[j][0] = s_frag[j][1] = s_frag[j][2] = s_frag[j][3] = 0.0f;
#pragma unroll
      for (int ks = 0; ks < kD / 16; ++ks) {
#pragma unroll
        for (int jp = 0; jp < kKeys / 16; ++jp) {
          unsigned b[4];
          const int row = (jp * 2 + (lane >> 4)) * 8 + (lane & 7);
          const int col = ks * 16 + ((lane >> 3) & 1) * 8;
          ldmatrix_x4(b, k_smem + row * kRow + col);
          mma_bf16(s_frag[jp * 2], qa[ks], b[0], b[1]);
          mma_bf16(s_frag[jp * 2 + 1], qa[ks], b[2], b[3]);
        }
      }
      // Scores stay unscaled; the scale is folded into the exponent: p = 2^(s * sl2 - max * sl2).
      // Only tiles that touch the diagonal (or the window's edge) of this warp's rows need the mask.
      const int warp_first_pos = pos0 + min(warp * 16, rows_here - 1);
      const bool need_mask = key0 + kKeys - 1 > warp_first_pos || (window > 0 && key0 < warp_last_pos - window + 1);
      float tile_max[2] = {-INFINITY, -INFINITY};
      if (need_mask) {
#pragma unroll
        for (int j = 0; j < kKeys / 8; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = key0 + j * 8 + 2 * t + (e & 1);
            const int r = e >> 1;
            const float v = (key >= my_lo[r] && key <= my_pos[r]) ? s_frag[j][e] : -INFINITY;
            s_frag[j][e] = v;
            tile_max[r] = fmaxf(tile_max[r], v);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < kKeys / 8; ++j) {
          tile_max[0] = fmaxf(tile_max[0], fmaxf(s_frag[j][0], s_frag[j][1]));
          tile_max[1] = fmaxf(tile_max[1], fmaxf(s_frag[j][2], s_frag[j][3]));
        }
      }
      float rescale[2], base[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
        const float new_max = fmaxf(row_max[r], tile_max[r]);
        const float finite_max = (new_max == -INFINITY) ? 0.0f : new_max;   // a row may see no key in an early tile (window)
        base[r] = finite_max * sl2;
        rescale[r] = exp2f((row_max[r] - finite_max) * sl2);
        row_max[r] = new_max;
        row_sum[r] *= rescale[r];
      }
      unsigned pa[kKeys / 16][4];
#pragma unroll
      for (int j = 0; j < kKeys / 8; ++j) {
        const float p0 = exp2_approx(fmaf(s_frag[j][0], sl2, -base[0]));
        const float p1 = exp2_approx(fmaf(s_frag[j][1], sl2, -base[0]));
        const float p2 = exp2_approx(fmaf(s_frag[j][2], sl2, -base[1]));
        const float p3 = exp2_approx(fmaf(s_frag[j][3], sl2, -base[1]));
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
#pragma unroll
      for (int kk = 0; kk < kKeys / 16; ++kk) {
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
    }
    __syncthreads();   // everyone is done with this stage before the next iteration overwrites it
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (my_row[r] >= rows_here) continue;
    const float inv = 1.0f / row_sum[r];
    __nv_bfloat16* dst = out + ((size_t)(row0 + my_row[r]) * q_heads + head) * kD + 2 * t;
#pragma unroll
    for (int i = 0; i < kD / 8; ++i) {
      *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(o[i][r * 2] * inv, o[i][r * 2 + 1] * inv);
    }
  }
}

constexpr size_t kSmemBytes = ((size_t)kRows * kRow + 2 * 2 * (size_t)kKeys * kRow) * sizeof(__nv_bfloat16);

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_prefill_attention_head_dim() { return kD; }
TLIE_EXPORT int tlie_prefill_attention_tile_rows() { return kRows; }

TLIE_EXPORT int tlie_prefill_attention(const void* q, int q_row_stride, const void* pages, const int* tiles, int n_tiles,
                                       const int* seq_starts, const int* first_positions, const int* block_table,
                                       int table_stride, void* out, int q_heads, int kv_heads, int page_size, int window,
                                       float scale, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (kv_heads <= 0 || q_heads % kv_heads != 0 || q_heads > 65535) return (int)cudaErrorInvalidValue;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(prefill_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid(n_tiles, q_heads);
  prefill_attention_kernel<<<grid, kWarps * 32, kSmemBytes, stream>>>(
      (const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)pages, tiles, seq_starts, first_positions, block_table,
      table_stride, (__nv_bfloat16*)out, q_heads, kv_heads, page_size, window, scale);
  return (int)cudaGetLastError();
}
