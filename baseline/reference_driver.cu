// Times the reference's own batched decode step (tlie::cuda::TinyLlamaCuda::ForwardBatch, src/cuda/model.cu:531-725)
// for bench.py's reference arm.  Everything model-related here is the reference's unmodified code, reached through its
// public API: ModelConfig::Load, CudaWeightStore::Load, TinyLlamaCuda::Create / ForwardBatch / Reset, GreedySample.
// The loop mirrors app/batch_benchmark.cu:67-114: feed the prompt one position per step to every request of the batch,
// then decode greedily on the host, one ForwardBatch per generated token.
//
//   reference_driver CONFIG_JSON WEIGHTS FILE_SHA256 SOURCE_SHA256 PROMPT_TOKENS WARMUP STEPS BATCH [BATCH ...]
//
// One JSON line per batch size on standard output:
//   {"batch": B, "device_ms_per_step": compute time by the reference's own CUDA events (CudaStepTimings::compute_ms),
//    "wall_ms_per_step": host clock around ForwardBatch + greedy sampling, "transfer_ms_per_step": ..., "steps": K}
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <numeric>
#include <string>
#include <vector>

#include "tlie/cuda/model.hpp"
#include "tlie/cuda/weight_store.hpp"
#include "tlie/model_config.hpp"
#include "tlie/operators.hpp"

namespace {

int Fail(const tlie::Error& error) {
  std::fprintf(stderr, "reference error: %s\n", error.message.c_str());
  return 1;
}

// uniform token ids from a seeded 64-bit generator (splitmix64), the same for every run
struct Ids {
  unsigned long long state;
  int next(int vocab) {
    unsigned long long z = (state += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return static_cast<int>((z ^ (z >> 31)) % static_cast<unsigned long long>(vocab));
  }
};

}  // namespace

int main(int argc, char** argv) {
  if (argc < 9) {
    std::fprintf(stderr, "usage: reference_driver CONFIG_JSON WEIGHTS FILE_SHA256 SOURCE_SHA256 PROMPT_TOKENS WARMUP STEPS BATCH...\n");
    return 2;
  }
  const std::size_t prompt_tokens = std::strtoul(argv[5], nullptr, 10);
  const std::size_t warmup = std::strtoul(argv[6], nullptr, 10);
  const std::size_t steps = std::strtoul(argv[7], nullptr, 10);
  std::vector<std::size_t> batches;
  for (int i = 8; i < argc; ++i) batches.push_back(std::strtoul(argv[i], nullptr, 10));
  const std::size_t largest = *std::max_element(batches.begin(), batches.end());

  auto config = tlie::ModelConfig::Load(argv[1]);
  if (!config.ok()) return Fail(config.error());
  tlie::WeightLoadOptions options;
  options.expected_file_sha256 = argv[3];
  options.expected_source_sha256 = argv[4];
  auto weights = tlie::cuda::CudaWeightStore::Load(argv[2], options);
  if (!weights.ok()) return Fail(weights.error());
  const int vocab = static_cast<int>(config.value().vocab_size);
  const std::size_t context = prompt_tokens + warmup + steps + 1;
  auto created = tlie::cuda::TinyLlamaCuda::Create(std::move(config).value(), std::move(weights).value(), context, false, largest, largest);
  if (!created.ok()) return Fail(created.error());
  tlie::cuda::TinyLlamaCuda model = std::move(created).value();

  for (const std::size_t batch : batches) {
    auto reset = model.Reset();
    if (!reset.ok()) return Fail(reset.error());
    std::vector<std::size_t> slots(batch), positions(batch);
    std::iota(slots.begin(), slots.end(), 0);
    std::vector<int> input(batch);
    std::vector<std::vector<float>> logits;
    Ids ids{1234567ull + batch};
    for (std::size_t position = 0; position < prompt_tokens; ++position) {
      for (std::size_t row = 0; row < batch; ++row) {
        input[row] = ids.next(vocab);
        positions[row] = position;
      }
      auto output = model.ForwardBatch(input, positions, slots);
      if (!output.ok()) return Fail(output.error());
      logits = std::move(output).value();
    }
    double device_ms = 0.0, transfer_ms = 0.0, wall_ms = 0.0;
    for (std::size_t step = 0; step < warmup + steps; ++step) {
      const bool timed = step >= warmup;
      const auto start = std::chrono::steady_clock::now();
      for (std::size_t row = 0; row < batch; ++row) {
        auto sampled = tlie::GreedySample(logits[row]);
        if (!sampled.ok()) return Fail(sampled.error());
        input[row] = sampled.value();
        positions[row] = prompt_tokens + step;
      }
      tlie::cuda::CudaStepTimings timings;
      auto output = model.ForwardBatch(input, positions, slots, &timings);
      if (!output.ok()) return Fail(output.error());
      logits = std::move(output).value();
      if (timed) {
        wall_ms += std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - start).count();
        device_ms += timings.compute_ms;
        transfer_ms += timings.transfer_ms;
      }
    }
    std::printf("{\"batch\": %zu, \"device_ms_per_step\": %.6f, \"transfer_ms_per_step\": %.6f, \"wall_ms_per_step\": %.6f, \"steps\": %zu}\n", batch,
                device_ms / steps, transfer_ms / steps, wall_ms / steps, steps);
    std::fflush(stdout);
  }
  return 0;
}
