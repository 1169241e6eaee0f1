"""Command line in the manner of the reference's binaries.

    tinyllama_b200 generate  MODEL_DIR PROMPT MAX_TOKENS [GOLDEN_JSON]
    tinyllama_b200 logits    MODEL_DIR PROMPT
    tinyllama_b200 benchmark MODEL_DIR CONTEXT OUTPUT_TOKENS WARMUP SAMPLES
    tinyllama_b200 reference MODEL_DIR PROMPT MAX_TOKENS [EXPECTED_FIRST_TOKEN]
    tinyllama_b200 random-model OUT_DIR CONFIG_JSON SEED
    tinyllama_b200 kernel-bench MODEL_DIR ROWS CONTEXT SAMPLES

The first three are the subcommands of ``tinyllama_cuda`` (app/cuda_reference.cu:476-521)
with the same positional arguments and JSON on standard output; ``reference`` prints
``token_ids:`` / ``text:`` like ``tinyllama_reference`` (app/reference_cli.cpp:40-125).
Errors are one JSON object ``{"error": {"code", "message"}}`` on standard error and
exit status 1 (app/reference_cli.cpp:20-25).  PROMPT is text when MODEL_DIR holds a
``tokenizer.model`` (SentencePiece, BOS prepended as src/tokenizer.cpp:103-105 does),
otherwise a list of token ids separated by commas or spaces; with ``--prompt-len N``
(and ``--prompt-seed S``) the PROMPT argument is left out and N seeded random token ids
stand in for it.  Options, before or after the positionals: ``--dtype bfloat16|float32``,
``--temperature``, ``--top-p``, ``--seed``, ``--batch``, ``--max-batch-tokens``,
``--page-size``, ``--num-pages`` (cache pages; by default what the request needs),
``--device`` (a CUDA device; there is no CPU path and ``cpu`` is refused with an error), ``--random-config FILE --weights-seed N``
(the command runs on a model of that config.json with seeded random weights, written to MODEL_DIR, or to a temporary folder
if MODEL_DIR is ``-``), ``--weights-sha256`` (the digest the
folder's weights must have, as the reference pins its checkpoints: src/weight_store.cpp:150-190).  ``kernel-bench`` times every kernel family at the model's own shapes with CUDA events
(median and 95th percentile), like the reference's benchmarks/kernel_benchmarks.cu:127-325; with ``--probes`` it also measures what the
kernels' designs rest on (tensor-core time per MMA shape, the cost of a barrier hand-off, a warp's arithmetic rate), with
``--attention-phases TOKENS`` where a key tile's cycles go in the tensor-memory prompt attention, with ``--products ROWS[,ROWS...]`` the
layer's four products at those row counts on the engine's own tcgen05 kernels (one SM, SM pairs) and on the library's.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

from .errors import EngineError

USAGE = __doc__.split("\n\n")[1]


def _positive(text: str, name: str, minimum: int = 1) -> int:
    try:
        value = int(text)
    except ValueError:
        value = None
    if value is None or value < minimum:
        raise EngineError(f"{name} must be an integer >= {minimum}", code="invalid_argument")
    return value


class _Tokens:
    """Text <-> ids with the folder's SentencePiece model if there is one, else ids as text."""

    def __init__(self, model_dir: Path, bos_id):
        self.processor = None
        self.bos_id = bos_id
        path = model_dir / "tokenizer.model"
        if path.exists():
            try:
                import sentencepiece

                self.processor = sentencepiece.SentencePieceProcessor(model_file=str(path))
            except Exception as exc:  # noqa: BLE001
                raise EngineError(f"unable to load tokenizer: {exc}", code="tokenizer") from exc

    def encode(self, prompt: str) -> list[int]:
        if self.processor is not None:
            ids = list(self.processor.encode(prompt))
            return ([self.bos_id] if self.bos_id is not None else []) + ids
        try:
            ids = [int(piece) for piece in prompt.replace(",", " ").split()]
        except ValueError:
            raise EngineError("PROMPT must be token ids (no tokenizer.model in MODEL_DIR)", code="tokenizer") from None
        if not ids:
            raise EngineError("PROMPT holds no token", code="invalid_argument")
        return ids

    def decode(self, ids: list[int]) -> str:
        if self.processor is not None:
            return self.processor.decode(ids)
        return " ".join(str(i) for i in ids)


def _engine(args, max_cache_tokens: int, max_requests: int = 1):
    from . import EngineConfig
    from .engine.api import Engine

    page = args.page_size
    cache_tokens = args.num_pages * page if args.num_pages else max(page, -(-max_cache_tokens // page) * page)
    config = EngineConfig(dtype=args.dtype, page_size=page, max_cache_tokens=cache_tokens, max_requests=max(1, max_requests),
                          max_batch_tokens=args.max_batch_tokens, device=args.device, weights_sha256=args.weights_sha256 or None)
    return Engine(args.model_dir, config)


def _prompt(args, tokens: "_Tokens", vocab: int) -> list[int]:
    """The PROMPT argument, or --prompt-len seeded random token ids."""
    if args.prompt_len:
        import numpy as np

        return [int(t) for t in np.random.default_rng(args.prompt_seed).integers(0, vocab, size=args.prompt_len)]
    return tokens.encode(args.rest[0])


def _generate(args) -> int:
    from .config import load_model_config
    from .engine.request import SamplingParams

    max_tokens = _positive(args.rest[1], "MAX_TOKENS")
    _, model_config = load_model_config(args.model_dir)
    tokens = _Tokens(Path(args.model_dir), getattr(model_config, "bos_token_id", None))
    prompt = _prompt(args, tokens, model_config.vocab_size)
    engine = _engine(args, len(prompt) + max_tokens)
    from .engine.timing import StepTimings

    prefill, decode = StepTimings(), StepTimings()   # device time of compute and of copies, as the reference reports them (app/cuda_reference.cu:149-226)
    started = time.perf_counter()
    request_id = engine.add_request(prompt, SamplingParams(max_tokens=max_tokens, temperature=args.temperature, top_p=args.top_p, seed=args.seed))
    while not engine.requests[request_id].generated and engine.has_unfinished():
        engine.step(prefill)
    prefill_ms = (time.perf_counter() - started) * 1e3
    while engine.has_unfinished():
        engine.step(decode)
    total_ms = (time.perf_counter() - started) * 1e3
    generated = engine.requests[request_id].generated
    if args.command == "reference":
        if len(args.rest) > 2 and generated[0] != _positive(args.rest[2], "EXPECTED_FIRST_TOKEN", 0):
            print("first generated token did not match expectation", file=sys.stderr)
            return 1
        print("token_ids:" + "".join(f" {t}" for t in generated))
        print("text: " + tokens.decode(generated))
        return 0
    result = {"prompt_tokens": len(prompt), "generated_tokens": generated, "text": tokens.decode(generated),
              "prefill_ms": prefill_ms, "decode_ms": total_ms - prefill_ms, "dtype": args.dtype,
              "prefill_compute_ms": prefill.compute_ms, "prefill_transfer_ms": prefill.transfer_ms,
              "decode_compute_ms": decode.compute_ms, "decode_transfer_ms": decode.transfer_ms, "decode_steps": decode.steps}
    if len(args.rest) > 2:
        golden = json.loads(Path(args.rest[2]).read_text())
        expected = golden.get("generated_tokens", golden.get("greedy_token_ids"))
        result["golden_match"] = expected is not None and list(expected)[: len(generated)] == generated
        if not result["golden_match"]:
            print(json.dumps(result))
            raise EngineError("generated tokens differ from the golden file", code="numerical")
    print(json.dumps(result))
    return 0


def _logits(args) -> int:
    from .config import load_model_config
    from .engine.batch import StepEntry

    _, model_config = load_model_config(args.model_dir)
    prompt = _prompt(args, _Tokens(Path(args.model_dir), getattr(model_config, "bos_token_id", None)), model_config.vocab_size)
    engine = _engine(args, len(prompt))
    logits = engine.runner.step([StepEntry("logits", prompt, [len(prompt) - 1])])
    print(json.dumps({"prompt_tokens": len(prompt), "logits": logits[0].cpu().tolist()}))
    return 0


def _benchmark(args) -> int:
    """CONTEXT prompt tokens (seeded random ids), OUTPUT_TOKENS greedy tokens, per-sample TTFT / TPOT / tokens per second."""
    import numpy as np
    import torch

    from .engine.request import SamplingParams

    context, output_tokens = _positive(args.rest[0], "CONTEXT"), _positive(args.rest[1], "OUTPUT_TOKENS")
    warmup, samples = _positive(args.rest[2], "WARMUP", 0), _positive(args.rest[3], "SAMPLES")
    engine = _engine(args, args.batch * (context + output_tokens + 64), args.batch)
    vocab = engine.runner.spec.vocab_size
    rng = np.random.default_rng(0)
    prompts = [[int(t) for t in rng.integers(0, vocab, size=context)] for _ in range(args.batch)]
    records = []
    for index in range(warmup + samples):
        ids = [engine.add_request(p, SamplingParams(max_tokens=output_tokens)) for p in prompts]
        torch.cuda.synchronize()
        started = time.perf_counter()
        first = None
        while engine.has_unfinished():
            engine.step()
            if first is None and all(engine.requests[i].generated for i in ids):
                torch.cuda.synchronize()
                first = time.perf_counter()
        torch.cuda.synchronize()
        ended = time.perf_counter()
        generated = [engine.requests.pop(i).generated for i in ids]
        if index >= warmup:
            decode_tokens = args.batch * (output_tokens - 1)
            records.append({
                "ttft_ms": (first - started) * 1e3,
                "tpot_ms": (ended - first) * 1e3 / max(1, output_tokens - 1),
                "decode_tokens_per_second": decode_tokens / (ended - first) if decode_tokens else 0.0,
                "total_tokens_per_second": args.batch * output_tokens / (ended - started),
                "tokens": generated[0][:8],
            })
    deterministic = all(r["tokens"] == records[0]["tokens"] for r in records)
    median = lambda key: float(np.median([r[key] for r in records]))  # noqa: E731
    print(json.dumps({
        "context": context, "output_tokens": output_tokens, "batch": args.batch, "warmup": warmup, "samples": samples, "dtype": args.dtype,
        "median_ttft_ms": median("ttft_ms"), "median_tpot_ms": median("tpot_ms"),
        "median_decode_tokens_per_second": median("decode_tokens_per_second"), "median_total_tokens_per_second": median("total_tokens_per_second"),
        "deterministic": deterministic, "device": torch.cuda.get_device_name(0), "samples_detail": records,
    }))
    return 0


def _kernel_bench(args) -> int:
    """Median / p95 of each kernel family at this model's shapes: ROWS tokens in the step, CONTEXT cached tokens each."""
    import numpy as np
    import torch

    from . import ops
    from .config import load_model_config
    from .ops import fast

    rows, context, samples = _positive(args.rest[0], "ROWS"), _positive(args.rest[1], "CONTEXT"), _positive(args.rest[2], "SAMPLES")
    _, c = load_model_config(args.model_dir)
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    dev = torch.device("cuda:0")
    H, I, V, D, QH, KVH, P = c.hidden_size, c.intermediate_size, c.vocab_size, c.head_dim, c.num_attention_heads, c.num_key_value_heads, 64
    rand = lambda *shape: (torch.randn(*shape, device=dev) * 0.05).to(dtype)  # noqa: E731
    residual, delta, normed = torch.randn(rows, H, device=dev), rand(rows, H), torch.empty(rows, H, device=dev, dtype=dtype)
    norm_w = torch.ones(H, device=dev)
    w_qkv, w_o, w_gu, w_dn, w_head = rand((QH + 2 * KVH) * D, H), rand(H, QH * D), rand(2 * I, H), rand(H, I), rand(V, H)
    qkv, mixed = rand(rows, (QH + 2 * KVH) * D), torch.empty(rows, QH * D, device=dev, dtype=dtype)
    gate_up, act, out_h = rand(rows, 2 * I), torch.empty(rows, I, device=dev, dtype=dtype), torch.empty(rows, H, device=dev, dtype=dtype)
    logits = torch.empty(min(rows, 64), V, device=dev)
    # a decode-shaped batch: ROWS requests with CONTEXT cached tokens each
    pages_per = -(-(context + 1) // P)
    pool = rand(rows * pages_per, 2, KVH, P, D)
    table = torch.arange(rows * pages_per, dtype=torch.int32, device=dev).view(rows, pages_per).contiguous()
    positions = torch.full((rows,), context, dtype=torch.int32, device=dev)
    token_seq = torch.arange(rows, dtype=torch.int32, device=dev)
    inv_freq = torch.from_numpy(np.power(np.float32(c.rope_theta), (np.float32(-2.0) * np.arange(D // 2, dtype=np.float32)) / np.float32(D))).to(dev)
    ids = torch.randint(0, V, (rows,), device=dev, dtype=torch.int32)
    table_e = rand(V, H)
    sampled = torch.empty(min(rows, 64), dtype=torch.int32, device=dev)
    cases = {
        "embedding": lambda: ops.embedding(table_e, ids, residual),
        "add_rmsnorm": lambda: ops.add_rmsnorm(residual, delta, norm_w, c.rms_norm_eps, normed),
        "linear_qkv": lambda: ops.linear(normed, w_qkv, qkv),
        "rope_store": lambda: ops.rope_store(qkv, positions, token_seq, table, inv_freq, D, pool, QH, KVH, D, P, True),
        "attention_generic": lambda: ops.core().tlie_paged_attention_generic and ops.paged_attention(qkv, pool, positions, token_seq, table, mixed, QH, KVH, D, P, 0, None, None),
        "linear_o": lambda: ops.linear(mixed, w_o, out_h),
        "linear_gate_up": lambda: ops.linear(normed, w_gu, gate_up),
        "silu_mul": lambda: ops.silu_mul(gate_up, act),
        "linear_down": lambda: ops.linear(act, w_dn, out_h),
        "linear_head": lambda: ops.linear(normed[: logits.shape[0]], w_head, logits),
        "argmax": lambda: ops.argmax(logits, sampled),
    }
    if dtype == torch.bfloat16 and D <= 128:
        splits = fast.decode_splits(rows, KVH, context + 1)
        cases["attention_decode_split_kv"] = lambda: fast.decode_attention(qkv, pool, positions, table, mixed, QH, KVH, D, P, 0, D ** -0.5, splits)
    report = {}
    for name, call in cases.items():
        for _ in range(3):
            call()
        times = []
        for _ in range(samples):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            call()
            end.record()
            end.synchronize()
            times.append(start.elapsed_time(end) * 1e3)
        times.sort()
        report[name] = {"median_us": times[len(times) // 2], "p95_us": times[min(len(times) - 1, int(len(times) * 0.95))]}
    record = {"rows": rows, "context": context, "samples": samples, "dtype": args.dtype, "device": torch.cuda.get_device_name(0), "kernels": report}
    if args.probes:
        from .ops.probes import hardware_probes

        record["probes"] = hardware_probes(dev)
    if args.attention_phases:
        from .ops.probes import attention_phase_cycles

        record["attention_phases"] = attention_phase_cycles(args.attention_phases, QH, KVH, D, dev)
    if args.products:
        from .ops.probes import product_comparison

        record["products"] = {str(r): product_comparison(r, H, I, (QH + 2 * KVH) * D, dev) for r in args.products}
    print(json.dumps(record))
    return 0


def _random_model(args) -> int:
    from .config import architecture_for
    from .weights import write_random_model

    data = json.loads(Path(args.rest[0]).read_text())
    config = architecture_for(data).config_class.from_dict(data)
    folder = write_random_model(args.model_dir, config, _positive(args.rest[1], "SEED", 0))
    print(json.dumps({"model_dir": str(folder)}))
    return 0


_COMMANDS = {"generate": (_generate, (2, 3)), "reference": (_generate, (2, 3)), "logits": (_logits, (1, 1)),
             "benchmark": (_benchmark, (4, 4)), "random-model": (_random_model, (2, 2)), "kernel-bench": (_kernel_bench, (3, 3))}


def _random_folder(args):
    """--random-config FILE: write the model folder (config.json and seeded random weights) the command then runs on.
    Returns the temporary directory to remove afterwards, if MODEL_DIR was ``-``."""
    import tempfile

    from .config import architecture_for
    from .weights import write_random_model

    scratch = None
    try:
        data = json.loads(Path(args.random_config).read_text())
        config = architecture_for(data).config_class.from_dict(data)
        if args.model_dir == "-":
            scratch = tempfile.TemporaryDirectory(prefix="tlie_random_model_")
            args.model_dir = str(Path(scratch.name) / "model")
        write_random_model(args.model_dir, config, args.weights_seed)
    except (OSError, json.JSONDecodeError) as exc:
        print(json.dumps(EngineError(f"unable to read {args.random_config}: {exc}", code="io").to_json()), file=sys.stderr)
        raise SystemExit(1) from exc
    except EngineError as exc:
        print(json.dumps(exc.to_json()), file=sys.stderr)
        raise SystemExit(1) from exc
    return scratch


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="tinyllama_b200", usage=USAGE, add_help=True)
    parser.add_argument("command", choices=sorted(_COMMANDS))
    parser.add_argument("model_dir")
    parser.add_argument("rest", nargs="*")
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--top-p", type=float, default=1.0)
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--batch", type=int, default=1)
    parser.add_argument("--max-batch-tokens", type=int, default=2048)
    parser.add_argument("--page-size", type=int, default=64, help="tokens per cache page (a multiple of 16)")
    parser.add_argument("--num-pages", type=int, default=0, help="cache pages (default: what the request needs)")
    parser.add_argument("--prompt-len", type=int, default=0, help="use this many seeded random token ids as the prompt; the PROMPT argument is then left out")
    parser.add_argument("--prompt-seed", type=int, default=0)
    parser.add_argument("--device", default="cuda:0", help="the CUDA device to run on (there is no CPU path)")
    parser.add_argument("--random-config", default="", metavar="FILE",
                        help="run a model of this config.json with seeded random weights; MODEL_DIR is then the folder it is written to, or - for a temporary one")
    parser.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights of --random-config")
    parser.add_argument("--weights-sha256", default="", help="the SHA-256 the model folder's weights must have; another digest is refused with checksum_mismatch")
    parser.add_argument("--probes", action="store_true", help="kernel-bench: also what an MMA of each shape, a barrier hand-off and a warp's arithmetic cost on this GPU")
    parser.add_argument("--products", type=lambda text: [int(v) for v in text.split(",")], default=[], metavar="ROWS[,ROWS...]",
                        help="kernel-bench: also the layer's four products at these row counts (128 or more), the engine's own tcgen05 kernels against the library's")
    parser.add_argument("--attention-phases", type=int, default=0, metavar="TOKENS",
                        help="kernel-bench: also where a key tile's cycles go in the tensor-memory prompt attention, for one request of TOKENS tokens (seven builds of the kernel)")
    try:
        args = parser.parse_intermixed_args(argv)
    except SystemExit as exc:
        return int(exc.code or 0) and 1
    handler, (low, high) = _COMMANDS[args.command]
    scratch = None
    if args.random_config and args.command != "random-model":
        scratch = _random_folder(args)
    if args.prompt_len and args.command in ("generate", "reference", "logits"):
        args.rest.insert(0, "")   # the place of the PROMPT that --prompt-len stands in for
    try:
        if not low <= len(args.rest) <= high:
            raise EngineError("invalid tinyllama_b200 command or arguments\n" + USAGE, code="invalid_argument")
        return handler(args)
    except EngineError as exc:
        print(json.dumps(exc.to_json()), file=sys.stderr)
        return 1
    finally:
        if scratch is not None:
            scratch.cleanup()


if __name__ == "__main__":
    sys.exit(main())
