// Measurements of this GPU that the kernels' designs rest on, each a loop of one primitive timed with clock64 by the thread that runs it:
// how long the tensor core is busy with a tcgen05.mma of a given shape, what the hand-off primitives cost a lone thread, and how fast
// one warp (or two on a scheduler) gets through the pieces of a softmax tile.  Run by `kernel-bench --probes`; nothing of the engine
// calls them.  Every wait is bounded (tcgen05_utils.cuh: mbar_wait) and reports through the device error word.
#include "tcgen05_utils.cuh"

namespace tlie {

constexpr int kProbeOperandBytes = 16384 + 32768;   // an A tile of 128 x 64 and a B tile of 256 x 64 bfloat16, zeros

// out[2 * block] = cycles from the first issue to the arrival of the commit after `chain` MMAs of 128 x n x 16 (bfloat16, both
// operands K-major in shared memory with the 128-byte swizzle), out[2 * block + 1] = 1 if the wait returned.  `straight`: four
// MMAs per turn of the loop and nothing computed between them; else one per turn with its index arithmetic, as a k loop has it.
__global__ void __launch_bounds__(128) probe_mma_kernel(int n, int chain, int straight, long long* out, int* error_flag) {
  extern __shared__ __align__(1024) uint8_t probe_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(probe_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base;
  __shared__ int abort_word;
  for (int i = threadIdx.x; i < kProbeOperandBytes / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) {
    abort_word = 0;
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;\n" ::"r"(smem_u32(&tmem_base)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem = tmem_base;
  if (threadIdx.x == 0) {
    const uint32_t a_low = umma_desc_low(smem_u32(smem)), b_low = umma_desc_low(smem_u32(smem + 16384));
    const uint32_t idesc = umma_instr_desc(128, n);
    const long long t0 = clock64();
    if (straight) {
#pragma unroll 1
      for (int i = 0; i < chain; i += 4) {
        umma_bf16(tmem, a_low, b_low, idesc, 1);
        umma_bf16(tmem, a_low + 2, b_low + 2, idesc, 1);
        umma_bf16(tmem, a_low + 4, b_low + 4, idesc, 1);
        umma_bf16(tmem, a_low + 6, b_low + 6, idesc, 1);
      }
    } else {
      for (int i = 0; i < chain; ++i) {
        const uint32_t k = static_cast<uint32_t>(i & 3) * 2;
        umma_bf16(tmem, a_low + k, b_low + k, idesc, 1);
      }
    }
    umma_commit(&bar);
    const bool ok = mbar_wait(&bar, 0, &abort_word);
    out[blockIdx.x * 2] = clock64() - t0;
    out[blockIdx.x * 2 + 1] = ok ? 1 : 0;
    if (!ok) atomicOr(error_flag, 1);
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (threadIdx.x < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;\n" ::"r"(tmem) : "memory");
}

// Cycles per operation for a lone thread with nothing to wait for: out[0] arrive + wait on the barrier just completed, [1] wait on a
// barrier long complete, [2] tcgen05.commit with no product outstanding, [3] commit and the wait for its arrival, [4] fence.proxy.async.
__global__ void __launch_bounds__(32) probe_handoff_kernel(long long* out, int* error_flag) {
  __shared__ uint64_t bar[4];
  __shared__ int abort_word;
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int i = 0; i < 4; ++i) mbar_init(&bar[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    constexpr int kTurns = 64;
    bool ok = true;
    uint32_t phase = 0;
    long long t0 = clock64();
    for (int i = 0; i < kTurns; ++i) {
      mbar_arrive(&bar[0]);
      ok = mbar_wait(&bar[0], phase, &abort_word) && ok;
      phase ^= 1;
    }
    out[0] = (clock64() - t0) / kTurns;
    mbar_arrive(&bar[1]);
    t0 = clock64();
    for (int i = 0; i < kTurns; ++i) ok = mbar_wait(&bar[1], 0, &abort_word) && ok;
    out[1] = (clock64() - t0) / kTurns;
    t0 = clock64();
    for (int i = 0; i < kTurns; ++i) umma_commit(&bar[2]);
    out[2] = (clock64() - t0) / kTurns;
    phase = 0;
    t0 = clock64();
    for (int i = 0; i < kTurns; ++i) {
      umma_commit(&bar[3]);
      ok = mbar_wait(&bar[3], phase, &abort_word) && ok;
      phase ^= 1;
    }
    out[3] = (clock64() - t0) / kTurns;
    t0 = clock64();
    for (int i = 0; i < kTurns; ++i) asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    out[4] = (clock64() - t0) / kTurns;
    if (!ok) atomicOr(error_flag, 1);
  }
}

// One softmax tile's arithmetic on 64 values per thread, repeated: mode 0 = 64 exp2, 1 = 64 multiply-adds and 64 adds (two sums).
// Every turn works on the results of the turn before, so nothing can be taken out of the loop.  cycles[0]: per turn, thread 0 of block 0.
template <int MODE>
__global__ void probe_arithmetic_kernel(const float* __restrict__ in, float* __restrict__ out, long long* cycles, int turns) {
  float v[64];
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = in[(threadIdx.x * 64 + i) & 4095];
  float s0 = 0.0f, s1 = 0.0f;
  __syncthreads();
  const long long t0 = clock64();
  for (int r = 0; r < turns; ++r) {
    if (MODE == 0) {
#pragma unroll
      for (int i = 0; i < 64; ++i) v[i] = exp2_approx(v[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        v[2 * i] = fmaf(v[2 * i], 1.0009765625f, -0.25f);
        v[2 * i + 1] = fmaf(v[2 * i + 1], 1.0009765625f, -0.25f);
        s0 += v[2 * i];
        s1 += v[2 * i + 1];
      }
    }
  }
  const long long t1 = clock64();
  float sink = s0 + s1;
#pragma unroll
  for (int i = 0; i < 64; ++i) sink += v[i];
  out[blockIdx.x * blockDim.x + threadIdx.x] = sink;
  if (blockIdx.x == 0 && threadIdx.x == 0) cycles[0] = (t1 - t0) / turns;
}

}  // namespace tlie

using namespace tlie;

// out: int64 [2 * blocks] on the device.  n: 32 .. 256, a multiple of 16; chain: a multiple of 4.
TLIE_EXPORT int tlie_probe_mma(int blocks, int n, int chain, int straight, long long* out, int* error_flag, cudaStream_t stream) {
  if (blocks <= 0 || n < 32 || n > 256 || n % 16 != 0 || chain <= 0 || chain % 4 != 0 || out == nullptr || error_flag == nullptr) return (int)cudaErrorInvalidValue;
  const int smem = kProbeOperandBytes + 1024;
  cudaError_t e = cudaFuncSetAttribute(probe_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return (int)e;
  probe_mma_kernel<<<blocks, 128, smem, stream>>>(n, chain, straight, out, error_flag);
  return (int)cudaGetLastError();
}

// out: int64 [5] on the device.
TLIE_EXPORT int tlie_probe_handoff(long long* out, int* error_flag, cudaStream_t stream) {
  if (out == nullptr || error_flag == nullptr) return (int)cudaErrorInvalidValue;
  probe_handoff_kernel<<<1, 32, 0, stream>>>(out, error_flag);
  return (int)cudaGetLastError();
}

// in: float [4096]; out: float [blocks * threads]; cycles: int64 [1]; all on the device.
TLIE_EXPORT int tlie_probe_arithmetic(int mode, int blocks, int threads, const float* in, float* out, long long* cycles, int turns, cudaStream_t stream) {
  if (blocks <= 0 || threads <= 0 || threads > 1024 || turns <= 0) return (int)cudaErrorInvalidValue;
  if (mode == 0)
    probe_arithmetic_kernel<0><<<blocks, threads, 0, stream>>>(in, out, cycles, turns);
  else if (mode == 1)
    probe_arithmetic_kernel<1><<<blocks, threads, 0, stream>>>(in, out, cycles, turns);
  else
    return (int)cudaErrorInvalidValue;
  return (int)cudaGetLastError();
}
