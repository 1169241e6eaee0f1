// Fused weight-streaming products for decode steps of up to 16 rows, bfloat16 weights.
//
//     out[M, N] (+)= f(x)[M, K] . w[N, K]^T
//
// A decode step of this model is ~2 GB of weights read once and a few kilobytes of activations; it
// is bound by HBM and by the fixed cost of every kernel boundary.  The reference runs 15 launches
// per layer and token (src/cuda/model.cu:406-475: norm, 7 library products, rotation, cache write,
// attention, activation, 2 adds).  Here one kernel family does product + neighbours:
//   input   X_PLAIN  x is bfloat16 [M, K];
//           X_NORM   x = rmsnorm(residual[rows]) * norm_weight, from the 32-bit residual stream, by
//                    every CTA for itself (M * K * 4 bytes out of L2): one pass stores
//                    bfloat16(residual * norm_weight) and sums the squares in 32-bit; the row's
//                    scale 1 / sqrt(mean + eps) (src/operators.cpp:22-45) multiplies the 32-bit
//                    result, which is the same product because the scale is one number per row;
//           X_DIRECT x is bfloat16 [M, K] and is not staged in shared memory at all (a CTA that
//                    computes a single tile uses every element of x once);
//           X_PREPARED x is bfloat16(residual * norm_weight) as the product that completed the residual left it
//                    (ACCUM with prepare_*), with the rows' sums of squares per 16-column tile: the CTAs copy half
//                    the bytes X_NORM reads and none of them squares anything;
//   output  STORE    bfloat16 or 32-bit [M, N];
//           ACCUM    residual[m, n] += result in 32-bit (each element owned by one thread, so the
//                    sum is deterministic): the reference's add kernel (src/cuda/kernels.cu:208-215);
//           GATED    a tile is 8 rows of the gate half of w and the 8 rows of the up half for the same outputs (the
//                    two halves of the MMA's 16 rows); the CTA stores silu(gate) * up (src/operators.cpp:148-164)
//                    as bfloat16 [M, N/2].  Tiles of 8 outputs deal the widest product evenly to the CTAs.
// Mechanics: 16 weight rows are the A operand of mma.sync m16n8k16 and 8 rows of x the B operand
// (M = 8 wastes nothing); the contraction index is permuted so that a thread fetches 8 consecutive
// k of a weight row with one 16-byte load feeding two MMAs; the 8 warps of a CTA split K, keep
// their whole share of the weights in flight in registers, and sum through shared memory.  Weight
// loads are issued BEFORE the programmatic-dependency wait: while the previous kernel of the step
// still runs, this one already streams its weights.
#include "gemv_core.cuh"

namespace tlie {

template <int MT, int XMODE, int EPI, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) gemv_fused_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float row_scale[MT * 8];
  GemvPhase<MT, XMODE, EPI, WARPS> phase;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);   // [MT * 8][x_stride]
  float* red = phase.red_of(smem_raw, a.x_stride);                  // [warps][16][MT * 8 + 1]
  // weights of the first round, before anything that depends on the previous kernel
  phase.issue(a, blockIdx.x * phase.kTileRows, threadIdx.x >> 5);
  grid_launch_dependents();
  grid_dependency_wait();
  phase.stage_x(a, xs, row_scale);
  phase.run(a, xs, red, row_scale, blockIdx.x, gridDim.x, true);
}

template <int MT, int XMODE, int EPI, int WARPS = kGemvWarps>
static int launch_one(const GemvArgs& a, int grid, cudaStream_t stream) {
  const size_t smem = GemvPhase<MT, XMODE, EPI, WARPS>::smem_bytes(a.x_stride);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemv_fused_kernel<MT, XMODE, EPI, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  return (int)launch_pdl(gemv_fused_kernel<MT, XMODE, EPI, WARPS>, dim3(grid), dim3(WARPS * 32), smem, stream, a);
}

static int gemv_wide_ctas = 1;      // tlie_gemv_set_wide_ctas
constexpr int kGemvCtasPerSm = 2;   // how many CTAs of a product an SM is dealt at most (measured: 1 and 3 are slower for the wide products)

template <int XMODE, int EPI>
static int launch_rows(const GemvArgs& a, cudaStream_t stream) {
  const int n_rows = (EPI == EPI_GATED) ? a.N / 2 : a.N;
  const int tile_rows = (EPI == EPI_GATED) ? 8 : 16;
  const int tiles = (n_rows + tile_rows - 1) / tile_rows;
  // x is staged once per CTA, so a CTA takes several tiles when there are more than `slots` of them; equal shares
  const int slots = kGemvCtasPerSm * device_sm_count();
  const int per_cta = (tiles + slots - 1) / slots;
  // All slots are filled and a CTA walks tiles blockIdx.x, + gridDim.x, ...: an SM's CTAs then hold tile counts that differ
  // by one at most.  (Equal shares per CTA in fewer CTAs left some SMs with two CTAs and some with one: twice the work.)
  const int grid = tiles < slots ? tiles : slots;
  if (XMODE == X_PLAIN && per_cta == 1) {   // every element of x is used once per CTA: no point in staging it
    // long rows and no more tiles than SMs: sixteen warps split K, so that a CTA has twice the bytes in flight and half the rounds
    if (a.M <= 8 && gemv_wide_ctas && tiles <= device_sm_count() && a.K > kGemvWarps * 8 * 32) return launch_one<1, X_DIRECT, EPI, 16>(a, grid, stream);
    if (a.M <= 8) return launch_one<1, X_DIRECT, EPI>(a, grid, stream);
    if (a.M <= 16) return launch_one<2, X_DIRECT, EPI>(a, grid, stream);
    return (int)cudaErrorInvalidValue;
  }
  if (a.M <= 8) return launch_one<1, XMODE, EPI>(a, grid, stream);
  if (a.M <= 16) return launch_one<2, XMODE, EPI>(a, grid, stream);
  return (int)cudaErrorInvalidValue;
}

template <int XMODE>
static int launch_epilogue(const GemvArgs& a, int epilogue, cudaStream_t stream) {
  switch (epilogue) {
    case EPI_STORE_BF16: return launch_rows<XMODE, EPI_STORE_BF16>(a, stream);
    case EPI_STORE_F32: return launch_rows<XMODE, EPI_STORE_F32>(a, stream);
    case EPI_ACCUM: return launch_rows<XMODE, EPI_ACCUM>(a, stream);
    case EPI_GATED: return launch_rows<XMODE, EPI_GATED>(a, stream);
  }
  return (int)cudaErrorInvalidValue;
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_gemv_max_rows() { return 16; }
// 0: products of long rows never take sixteen warps per CTA (for comparison)
TLIE_EXPORT void tlie_gemv_set_wide_ctas(int on) { gemv_wide_ctas = on; }

// x_mode 0: x bf16 [M, K] with row stride ldx.  x_mode 1: x is the 32-bit residual [*, K]; rows (optional) gathers,
// norm_weight [K] and eps give the RMSNorm.  x_mode 3: x is bf16(residual * norm weight) [M, K] and `squares`
// [M, square_tiles] the rows' sums of squares, as an earlier call with epilogue 2 and prepare_* left them.
// prepare_weight (epilogue 2 only, else null): also store bf16(out * prepare_weight) in prepare_x [M, N] and the rows' sums of
// squares per 16 columns in prepare_squares [M, ceil(N / 16)].  epilogue 0: bf16 out [M, N]; 1: 32-bit out; 2: out (32-bit [M, N]) += result;
// 3: w holds [gate rows | up rows] (N even), out = silu(gate) * up as bf16 [M, N / 2].
// Needs K % 8 == 0 (K % 4 == 0 suffices for x_mode 1 is NOT enough: weights are read 8 at a time), M <= 16.
TLIE_EXPORT int tlie_gemv_fused(int x_mode, const void* x, int ldx, const int* rows, const float* norm_weight, float eps,
                                const void* w, void* out, int M, int N, int K, int epilogue, const float* squares, int square_tiles,
                                const float* prepare_weight, void* prepare_x, float* prepare_squares, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || M > 16 || ((x_mode == X_PLAIN || x_mode == X_PREPARED) && ldx % 8 != 0) || (epilogue == EPI_GATED && (N & 1)) ||
      (x_mode == X_PREPARED && (squares == nullptr || square_tiles <= 0)) ||
      (prepare_weight != nullptr && (epilogue != EPI_ACCUM || prepare_x == nullptr || prepare_squares == nullptr)))
    return (int)cudaErrorInvalidValue;
  GemvArgs a;
  a.x = x;
  a.ldx = ldx;
  a.rows = rows;
  a.norm_weight = norm_weight;
  a.eps = eps;
  a.w = (const __nv_bfloat16*)w;
  a.out = out;
  a.M = M;
  a.N = N;
  a.K = K;
  a.x_stride = gemv_x_stride(K);
  a.squares = squares;
  a.square_tiles = square_tiles;
  a.prepare_weight = prepare_weight;
  a.prepare_x = (__nv_bfloat16*)prepare_x;
  a.prepare_squares = prepare_squares;
  if (x_mode == X_PLAIN) return launch_epilogue<X_PLAIN>(a, epilogue, stream);
  if (x_mode == X_NORM) return launch_epilogue<X_NORM>(a, epilogue, stream);
  if (x_mode == X_PREPARED) return launch_epilogue<X_PREPARED>(a, epilogue, stream);
  return (int)cudaErrorInvalidValue;
}
