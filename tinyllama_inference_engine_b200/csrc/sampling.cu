// Token selection on the device: greedy argmax and temperature / top-p sampling.
//
// Greedy: the largest logit, the lowest id on ties (src/operators.cpp:166-175,
// tests/unit_tests.cpp:198-202).
// Temperature / top-p (app/server.cpp:237-277): p_i = exp((l_i - max) / T); keep the
// smallest set of most probable tokens whose share of the total reaches top_p (the token
// that crosses the line included); draw a point uniformly in the kept mass and return the
// token it falls on.  The reference sorts and walks the sorted list with a per-request
// mt19937; here the kept set is found by bisecting on the probability threshold (no sort),
// the walk is in token-id order, and the uniform number comes from a counter-based hash
// of (seed, draw index), so a request's draws do not depend on what else is in the batch.
// All arithmetic is 32-bit; one block owns one row.
#include "common.cuh"

namespace tlie {

constexpr int kSampleThreads = 1024;

// A thread's share of a row's maximum and the lowest index that holds it.  Rows that allow it are read 16 bytes at a
// time, four loads in flight per thread: one block reads a whole row, so its time is the latency of its loads in turn.
__device__ __forceinline__ void row_max_and_arg(const float* __restrict__ row, int vocab, float& best, int& arg) {
  auto take = [&](float v, int i) {
    if (v > best || (v == best && i < arg)) {
      best = v;
      arg = i;
    }
  };
  if ((vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int quads = vocab >> 2;
    constexpr int kInFlight = 4;
    for (int q0 = threadIdx.x; q0 < quads; q0 += kInFlight * blockDim.x) {
      float4 v[kInFlight];
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const int q = q0 + u * blockDim.x;
        v[u] = q < quads ? row4[q] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
#pragma unroll
      for (int u = 0; u < kInFlight; ++u) {
        const int i = (q0 + u * blockDim.x) * 4;
        take(v[u].x, i);
        take(v[u].y, i + 1);
        take(v[u].z, i + 2);
        take(v[u].w, i + 3);
      }
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) take(row[i], i);
  }
}

__global__ void __launch_bounds__(kSampleThreads) argmax_kernel(const float* __restrict__ logits, int vocab,
                                                                int* __restrict__ out) {
  __shared__ float best_value[32];
  __shared__ int best_index[32];
  const float* row = logits + (size_t)blockIdx.x * vocab;
  float value = -INFINITY;
  int index = 0x7fffffff;
  row_max_and_arg(row, vocab, value, index);
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, value, offset);
    const int oi = __shfl_xor_sync(0xffffffffu, index, offset);
    if (ov > value || (ov == value && oi < index)) {
      value = ov;
      index = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    best_value[warp] = value;
    best_index[warp] = index;
  }
  __syncthreads();
  if (warp == 0) {
    const int warps = (blockDim.x + 31) >> 5;
    value = lane < warps ? best_value[lane] : -INFINITY;
    index = lane < warps ? best_index[lane] : 0x7fffffff;
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, value, offset);
      const int oi = __shfl_xor_sync(0xffffffffu, index, offset);
      if (ov > value || (ov == value && oi < index)) {
        value = ov;
        index = oi;
      }
    }
    if (lane == 0) out[blockIdx.x] = index == 0x7fffffff ? 0 : index;
  }
}

// splitmix64 finaliser over (seed, counter): the uniform number of draw `counter` of a request.
__host__ __device__ inline float uniform_from(unsigned long long seed, unsigned long long counter) {
  unsigned long long z = seed * 0x9E3779B97F4A7C15ull + (counter + 1ull) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return (float)(z >> 40) * (1.0f / 16777216.0f);  // 24 bits -> [0, 1)
}

// One block per row.  temperature <= 0 means greedy for that row.
__global__ void __launch_bounds__(kSampleThreads)
    sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
                  const float* __restrict__ top_p, const long long* __restrict__ seeds,
                  const long long* __restrict__ counters, int* __restrict__ out) {
  __shared__ float scratch[32];
  __shared__ float prefix[kSampleThreads];
  __shared__ int chosen;
  const float* row = logits + (size_t)blockIdx.x * vocab;
  const float temp = temperature[blockIdx.x];

  float local_max = -INFINITY;
  int local_arg = 0x7fffffff;
  row_max_and_arg(row, vocab, local_max, local_arg);
  const float row_max = block_max(local_max, scratch);
  if (!(temp > 0.0f)) {
    // greedy: lowest id among the maxima
    __shared__ int arg_smem;
    if (threadIdx.x == 0) arg_smem = 0x7fffffff;
    __syncthreads();
    if (local_max == row_max) atomicMin(&arg_smem, local_arg);
    __syncthreads();
    // a row without any comparable value (all NaN) leaves no maximum: token 0, as argmax_kernel answers
    if (threadIdx.x == 0) out[blockIdx.x] = (arg_smem < 0 || arg_smem >= vocab) ? 0 : arg_smem;
    return;
  }
  const float inv_temp = 1.0f / temp;
  // contiguous slice of the row per thread, so that the walk is in token-id order
  const int per_thread = (vocab + blockDim.x - 1) / blockDim.x;
  const int begin = min(vocab, (int)threadIdx.x * per_thread);
  const int end = min(vocab, begin + per_thread);

  float sum = 0.0f;
  for (int i = begin; i < end; ++i) sum += expf((row[i] - row_max) * inv_temp);
  const float total = block_sum(sum, scratch);

  // Largest threshold tau with mass{p >= tau} >= top_p * total, by bisection on the bit
  // pattern of positive floats (monotone in value).  The kept set is {p >= tau}.
  float tau = 0.0f;
  const float want = top_p[blockIdx.x] * total;
  if (top_p[blockIdx.x] < 1.0f) {
    unsigned lo = 0u;                    // mass{p >= 0} = total >= want
    unsigned hi = __float_as_uint(1.0f) + 1u;  // p <= 1, so mass{p >= hi} = 0 < want
    while (hi - lo > 1u) {
      const unsigned mid = lo + (hi - lo) / 2u;
      const float threshold = __uint_as_float(mid);
      float mass = 0.0f;
      for (int i = begin; i < end; ++i) {
        const float p = expf((row[i] - row_max) * inv_temp);
        if (p >= threshold) mass += p;
      }
      mass = block_sum(mass, scratch);
      if (mass >= want) lo = mid; else hi = mid;
    }
    tau = __uint_as_float(lo);
  }
  float kept = 0.0f;
  for (int i = begin; i < end; ++i) {
    const float p = expf((row[i] - row_max) * inv_temp);
    if (p >= tau) kept += p;
  }
  prefix[threadIdx.x] = kept;
  __syncthreads();
  if (threadIdx.x == 0) {
    float running = 0.0f;
    for (int i = 0; i < blockDim.x; ++i) {  // exclusive scan in thread order
      const float v = prefix[i];
      prefix[i] = running;
      running += v;
    }
    scratch[0] = running;
    chosen = -1;
  }
  __syncthreads();
  const float kept_total = scratch[0];
  const float target = uniform_from((unsigned long long)seeds[blockIdx.x], (unsigned long long)counters[blockIdx.x]) * kept_total;
  // the slice whose [start, start + kept) holds the target walks its tokens
  const float start = prefix[threadIdx.x];
  if (kept > 0.0f && target >= start && target < start + kept) {
    float cursor = start;
    int pick = -1;
    for (int i = begin; i < end; ++i) {
      const float p = expf((row[i] - row_max) * inv_temp);
      if (p >= tau) {
        cursor += p;
        pick = i;
        if (target < cursor) break;
      }
    }
    atomicMax(&chosen, pick);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int pick = chosen;
    if (pick < 0) {  // rounding put the target past the last kept token: take the last kept one
      for (int i = vocab - 1; i >= 0 && pick < 0; --i)
        if (expf((row[i] - row_max) * inv_temp) >= tau) pick = i;
    }
    // non-finite logits can leave nothing kept at all; the answer must still be a token of the vocabulary
    out[blockIdx.x] = (pick < 0 || pick >= vocab) ? 0 : pick;
  }
}

}  // namespace tlie

using namespace tlie;

TLIE_EXPORT int tlie_argmax(const float* logits, int rows, int vocab, int* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  argmax_kernel<<<rows, kSampleThreads, 0, stream>>>(logits, vocab, out);
  return (int)cudaGetLastError();
}

TLIE_EXPORT int tlie_sample(const float* logits, int rows, int vocab, const float* temperature, const float* top_p,
                            const long long* seeds, const long long* counters, int* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  sample_kernel<<<rows, kSampleThreads, 0, stream>>>(logits, vocab, temperature, top_p, seeds, counters, out);
  return (int)cudaGetLastError();
}

TLIE_EXPORT float tlie_uniform_from(long long seed, long long counter) {
  return uniform_from((unsigned long long)seed, (unsigned long long)counter);
}

// After a decode step: the sampled tokens become the next step's inputs and every request
// moves one position on.  Lets a run of decode steps stay on the device.
// `mailbox` (optional): pinned host memory of count + 2 words, written by this kernel over the bus: the sampled tokens, the device
// error word, and last (after a system-wide fence) the number of the step, which the host polls instead of asking the stream.
// One block: the block barrier orders every token's store before the number's.
__global__ void decode_advance_kernel(int* __restrict__ token_ids, const int* __restrict__ sampled,
                                      int* __restrict__ positions, int* __restrict__ seq_lens,
                                      int* __restrict__ first_positions, long long* __restrict__ counters, int count,
                                      volatile int* mailbox, const int* __restrict__ error_word, int* __restrict__ steps_done) {
  for (int i = threadIdx.x; i < count; i += blockDim.x) {
    const int token = sampled[i];
    token_ids[i] = token;
    positions[i] += 1;
    seq_lens[i] += 1;
    first_positions[i] += 1;
    counters[i] += 1;
    if (mailbox != nullptr) mailbox[i] = token;
  }
  if (mailbox == nullptr) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    mailbox[count] = error_word != nullptr ? *error_word : 0;
    const int number = *steps_done + 1;
    *steps_done = number;
    __threadfence_system();
    mailbox[count + 1] = number;
  }
}

// mailbox: null, or pinned host memory of count + 2 int32 (then steps_done: a device int32 that counts the steps; error_word may be null).
TLIE_EXPORT int tlie_decode_advance(int* token_ids, const int* sampled, int* positions, int* seq_lens,
                                    int* first_positions, long long* counters, int count, int* mailbox, const int* error_word,
                                    int* steps_done, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (mailbox != nullptr && steps_done == nullptr) return (int)cudaErrorInvalidValue;
  decode_advance_kernel<<<1, count <= 128 ? 128 : 256, 0, stream>>>(token_ids, sampled, positions, seq_lens, first_positions, counters, count, mailbox,
                                                                    error_word, steps_done);
  return (int)cudaGetLastError();
}
