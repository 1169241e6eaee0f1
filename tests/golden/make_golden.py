#!/usr/bin/env python3
"""Makes tests/golden/reference_logits.json from the reference's own compiled CPU model.

What it does (CPU only, no network):
  1. writes two tiny random Llama checkpoints (tests/tiny_configs.py A and B) with the
     engine's random-weights mode into a temporary folder;
  2. converts them to the reference's TLIEWGT container with the reference's own writer
     (scripts/tlie_format.py:write_tensor_file); a tied head is written out as a copy
     of the embedding because the reference always reads lm_head.weight (src/model.cpp:210);
  3. compiles the reference's unmodified src/{error,kv_cache,operators,sha256,weight_store,model}.cpp
     with a small driver and a stand-in for src/model_config.cpp whose
     ValidateFixedTinyLlama() accepts any size (the original pins TinyLlama 1.1B,
     src/model_config.cpp:54-76) and whose ExpectedTensors() is the same list;
  4. runs TinyLlamaCpu::Forward token by token and stores the logits of every position.

Usage:  python tests/golden/make_golden.py --reference /path/to/reference
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

DRIVER = r"""
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>
#include "tlie/model.hpp"
namespace tlie {
Result<void> ModelConfig::ValidateFixedTinyLlama() const { return Result<void>::Success(); }
std::vector<TensorSpec> ModelConfig::ExpectedTensors() const {
  std::vector<TensorSpec> s;
  s.push_back({"model.embed_tokens.weight", {vocab_size, hidden_size}});
  for (std::size_t l = 0; l < num_hidden_layers; ++l) {
    const std::string p = "model.layers." + std::to_string(l) + ".";
    s.push_back({p + "input_layernorm.weight", {hidden_size}});
    s.push_back({p + "self_attn.q_proj.weight", {hidden_size, hidden_size}});
    s.push_back({p + "self_attn.k_proj.weight", {kv_dim(), hidden_size}});
    s.push_back({p + "self_attn.v_proj.weight", {kv_dim(), hidden_size}});
    s.push_back({p + "self_attn.o_proj.weight", {hidden_size, hidden_size}});
    s.push_back({p + "post_attention_layernorm.weight", {hidden_size}});
    s.push_back({p + "mlp.gate_proj.weight", {intermediate_size, hidden_size}});
    s.push_back({p + "mlp.up_proj.weight", {intermediate_size, hidden_size}});
    s.push_back({p + "mlp.down_proj.weight", {hidden_size, intermediate_size}});
  }
  s.push_back({"model.norm.weight", {hidden_size}});
  s.push_back({"lm_head.weight", {vocab_size, hidden_size}});
  return s;
}
}  // namespace tlie
// argv: weights H I L NH NKV MAXPOS V EPS THETA token...
int main(int argc, char** argv) {
  tlie::ModelConfig c;
  c.hidden_size = std::strtoul(argv[2], nullptr, 10);
  c.intermediate_size = std::strtoul(argv[3], nullptr, 10);
  c.num_hidden_layers = std::strtoul(argv[4], nullptr, 10);
  c.num_attention_heads = std::strtoul(argv[5], nullptr, 10);
  c.num_key_value_heads = std::strtoul(argv[6], nullptr, 10);
  c.max_position_embeddings = std::strtoul(argv[7], nullptr, 10);
  c.vocab_size = std::strtoul(argv[8], nullptr, 10);
  c.rms_norm_eps = std::strtof(argv[9], nullptr);
  c.rope_theta = std::strtof(argv[10], nullptr);
  c.hidden_act = "silu";
  c.source_dtype = "bfloat16";
  auto weights = tlie::WeightStore::Load(argv[1]);
  if (!weights.ok()) { std::fprintf(stderr, "%s\n", weights.error().message.c_str()); return 1; }
  auto model = tlie::TinyLlamaCpu::Create(c, std::move(weights).value(), argc - 11);
  if (!model.ok()) { std::fprintf(stderr, "%s\n", model.error().message.c_str()); return 1; }
  for (int i = 11; i < argc; ++i) {
    auto logits = model.value().Forward(std::atoi(argv[i]), i - 11);
    if (!logits.ok()) { std::fprintf(stderr, "%s\n", logits.error().message.c_str()); return 1; }
    for (float v : logits.value()) std::printf("%.9g ", v);
    std::printf("\n");
  }
  return 0;
}
"""


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", type=Path, required=True)
    parser.add_argument("--out", type=Path, default=HERE / "reference_logits.json")
    args = parser.parse_args()
    sys.path.insert(0, str(args.reference / "scripts"))
    from tlie_format import write_tensor_file  # the reference's own container writer

    import plain_llama
    from tiny_configs import ALL
    from tinyllama_inference_engine_b200.weights import write_random_model

    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        (tmp / "driver.cpp").write_text(DRIVER)
        sources = [args.reference / "src" / f"{n}.cpp" for n in ("error", "kv_cache", "operators", "sha256", "weight_store", "model")]
        binary = tmp / "driver"
        subprocess.run(["g++", "-std=c++20", "-O2", f"-I{args.reference / 'include'}", str(tmp / "driver.cpp"), *map(str, sources), "-o", str(binary)], check=True)
        result = {}
        for key in ("a", "b"):
            config, seed = ALL[key]
            folder = write_random_model(tmp / key, config, seed)
            _, weights = plain_llama.load_model(folder)
            if "lm_head.weight" not in weights:
                weights["lm_head.weight"] = weights["model.embed_tokens.weight"]
            order = [n for n in weights if n != "lm_head.weight"] + ["lm_head.weight"]
            write_tensor_file(tmp / f"{key}.tliewgt", "00" * 32, ((n, weights[n].numpy()) for n in order), len(order))
            rng = np.random.default_rng(seed + 100)
            tokens = [int(t) for t in rng.integers(0, config["vocab_size"], size=9)]
            argv = [str(binary), str(tmp / f"{key}.tliewgt")] + [str(config[k]) for k in (
                "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                "max_position_embeddings", "vocab_size")] + [repr(config["rms_norm_eps"]), repr(config["rope_theta"])] + [str(t) for t in tokens]
            done = subprocess.run(argv, check=True, capture_output=True, text=True)
            logits = [[float(x) for x in line.split()] for line in done.stdout.strip().splitlines()]
            result[key] = {"config": config, "seed": seed, "tokens": tokens, "logits": logits}
            print(key, "positions", len(logits), "vocab", len(logits[0]))
    args.out.write_text(json.dumps(result) + "\n")


if __name__ == "__main__":
    main()
