"""Generality of the parts: a toy mixer with per-request state of its own, a toy feed-forward that routes every token to
one of two experts, and a toy position encoding that is no rotation, all defined here, are registered, built into a model
beside attention layers, and stepped, without touching the framework's files.

The toys are no model of anyone's.  Mixer: s_t = decay * s_{t-1} + W_in x_t, y_t = W_out s_t, one state vector per
request.  Feed-forward: y_t = W_e x_t with e = argmax(R x_t), the router in 32-bit.  Position: q and k are multiplied by
1 + 0.1 sin(0.3 position + dim).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass

import numpy as np
import pytest
import torch

import plain_ops
from tinyllama_inference_engine_b200 import EngineConfig
from tinyllama_inference_engine_b200.config import Architecture, register_architecture, unregister_architecture
from tinyllama_inference_engine_b200.engine.batch import StepEntry
from tinyllama_inference_engine_b200.engine.runner import ModelRunner
from tinyllama_inference_engine_b200.parts import (Block, CacheNeed, FeedForward, LayerSpec, Mixer, ModelSpec, OrderEntry, PartSpec, PositionEncoding, TensorSpec,
                                                   build_part, norm_then_part, part_class, register_part, unregister_part)
from tinyllama_inference_engine_b200.weights import write_random_model


class DecayMixer(Mixer):
    @classmethod
    def tensor_specs(cls, spec, prefix):
        h, s = spec["hidden_size"], spec["state_size"]
        return [TensorSpec(f"{prefix}.in.weight", (s, h), std=0.1), TensorSpec(f"{prefix}.out.weight", (h, s), std=0.1)]

    @classmethod
    def cache_need(cls, spec):
        return CacheNeed("state", state_shape=(spec["state_size"],))

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.w_in = weights.get(f"{prefix}.in.weight", torch.float32)
        self.w_out = weights.get(f"{prefix}.out.weight", torch.float32)
        self.decay = float(spec["decay"])

    def forward(self, x, ctx, cache):
        out = torch.empty_like(x)
        drive = x.float() @ self.w_in.T
        start = 0
        for slot, count in zip(ctx.host_state_slots, ctx.host_q_lens):  # every request's portion, in order
            state = cache.state[slot]
            for row in range(start, start + count):
                state = self.decay * state + drive[row]
                out[row] = (self.w_out @ state).to(x.dtype)
            cache.state[slot] = state
            start += count
        return out


class RoutedFeedForward(FeedForward):
    @classmethod
    def tensor_specs(cls, spec, prefix):
        h = spec["hidden_size"]
        return [TensorSpec(f"{prefix}.router.weight", (2, h), std=1.0)] + [TensorSpec(f"{prefix}.expert{e}.weight", (h, h), std=0.1) for e in range(2)]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.router = weights.get(f"{prefix}.router.weight", torch.float32)
        self.experts = torch.stack([weights.get(f"{prefix}.expert{e}.weight", torch.float32) for e in range(2)])

    def forward(self, x, ctx):
        choice = (x.float() @ self.router.T).argmax(1)                      # router logits in 32-bit
        return torch.einsum("thk,tk->th", self.experts[choice], x.float()).to(x.dtype)


class WavePosition(PositionEncoding):
    def apply(self, qkv, ctx, q_heads, kv_heads, head_dim):                # rotary_table() stays None: no rotation kernel applies
        dims = torch.arange(head_dim, device=qkv.device, dtype=torch.float32)
        factor = 1 + 0.1 * torch.sin(0.3 * ctx.positions.float()[:, None] + dims[None, :])
        heads = qkv.view(qkv.shape[0], q_heads + 2 * kv_heads, head_dim)
        heads[:, : q_heads + kv_heads] = (heads[:, : q_heads + kv_heads].float() * factor[:, None, :]).to(qkv.dtype)


@dataclass(frozen=True)
class ToyConfig:
    hidden_size: int = 48
    state_size: int = 24
    vocab_size: int = 97
    intermediate_size: int = 80
    decay: float = 0.9
    max_position_embeddings: int = 160
    architectures: tuple = ("ToyDecayForCausalLM",)

    @classmethod
    def from_dict(cls, data):
        return cls(**{k: (tuple(v) if k == "architectures" else v) for k, v in data.items() if k in cls.__dataclass_fields__})

    def to_dict(self):
        return {**asdict(self), "architectures": list(self.architectures)}


def build_toy_spec(c: ToyConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": c.hidden_size, "eps": 1e-5})
    ff = PartSpec("gated_mlp", {"hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size, "activation": "silu"})
    attention = PartSpec("attention", {"hidden_size": c.hidden_size, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16, "window": 0, "scale": None,
                                       "position": PartSpec("rotary", {"rotary_dim": 16, "theta": 100.0})})
    windowed = PartSpec("attention", {**attention.params, "window": 20})
    decay = PartSpec("toy_decay", {"hidden_size": c.hidden_size, "state_size": c.state_size, "decay": c.decay})
    waved = PartSpec("attention", {**attention.params, "num_heads": 2, "num_kv_heads": 2, "position": PartSpec("toy_wave", {})})
    routed = PartSpec("toy_routed", {"hidden_size": c.hidden_size})

    def block(mixer, feed_forward=ff):
        return PartSpec("pre_norm_residual", {"mixer_norm": norm, "mixer_norm_name": "n1", "mixer": mixer, "mixer_name": "mix",
                                              "feed_forward_norm": norm, "feed_forward_norm_name": "n2", "feed_forward": feed_forward, "feed_forward_name": "ff"})

    layers = (LayerSpec("toy.l0", block(attention)), LayerSpec("toy.l1", block(decay)), LayerSpec("toy.l2", block(windowed)),
              LayerSpec("toy.l3", block(waved, routed)))
    # layer 1 runs twice (two cache streams of its own); the last run of layer 0 reads the keys its first run cached;
    # layer 3 has the toy position encoding and the routed feed-forward
    order = (OrderEntry(0, cache=0), OrderEntry(1, cache=1), OrderEntry(2, cache=2), OrderEntry(1, cache=3), OrderEntry(3, cache=4),
             OrderEntry(0, cache=0, writes_cache=False))
    return ModelSpec("ToyDecayForCausalLM", c.hidden_size, c.vocab_size, c.max_position_embeddings,
                     PartSpec("token_embedding", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size, "name": "toy.embed"}),
                     layers, order, PartSpec("rmsnorm", {"size": c.hidden_size, "eps": 1e-5, "name": "toy.norm"}),
                     PartSpec("linear_head", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size, "name": "toy.head", "tied_to": "toy.embed"}))


@pytest.fixture()
def toy_folder(tmp_path):
    register_part("mixer", "toy_decay", DecayMixer, replace=True)
    register_part("feed_forward", "toy_routed", RoutedFeedForward, replace=True)
    register_part("position", "toy_wave", WavePosition, replace=True)
    register_architecture(Architecture("ToyDecayForCausalLM", ToyConfig, build_toy_spec), replace=True)
    yield write_random_model(tmp_path / "toy", ToyConfig(), seed=8, storage_dtype="bfloat16")
    unregister_architecture("ToyDecayForCausalLM")
    unregister_part("mixer", "toy_decay")
    unregister_part("feed_forward", "toy_routed")
    unregister_part("position", "toy_wave")


def _check_toy(folder, device, dtype, fraction):
    config = EngineConfig(dtype=dtype, page_size=16, max_cache_tokens=320, max_requests=4, max_batch_tokens=64, device=device)
    rng = np.random.default_rng(2)
    requests = {name: [int(t) for t in rng.integers(0, 97, size=n)] for name, n in (("p", 61), ("q", 45), ("r", 30))}
    whole = ModelRunner(folder, config)
    groups = whole.cache.page_groups
    assert [(g.need.window, g.need.kv_heads, g.streams) for g in groups] == [(0, 1, [0]), (20, 1, [2]), (0, 2, [4])]
    assert [g.streams for g in whole.cache.state_groups] == [[1, 3]]
    full = {}
    for name, tokens in requests.items():
        full[name] = whole.step([StepEntry(name, tokens, list(range(len(tokens))))]).cpu()
        whole.finish(name)
    atol = fraction * max(float(v.abs().max()) for v in full.values())  # a fraction of the largest |logit|
    cut = ModelRunner(folder, config)
    at = {name: 0 for name in requests}
    sizes = iter([5, 2, 1, 9, 3, 1, 1, 16, 2, 7] * 20)
    worst = 0.0
    while any(at[n] < len(t) for n, t in requests.items()):
        entries, rows = [], []
        for name, tokens in requests.items():
            if at[name] < len(tokens):
                n = min(next(sizes), len(tokens) - at[name])
                entries.append(StepEntry(name, tokens[at[name] : at[name] + n], [n - 1]))
                rows.append(full[name][at[name] + n - 1])
                at[name] += n
        got = cut.step(entries).cpu()
        worst = max(worst, float((got - torch.stack(rows)).abs().max()))
        cut.cache.check()
    assert worst <= atol, worst
    # the windowed group gave pages back while the requests were still live
    assert cut.cache.page_groups[1].pool.free_count > cut.cache.page_groups[0].pool.free_count
    for name in requests:
        cut.finish(name)
    # a slot used again starts from a zero state: run r again after the others dirtied every slot
    again = cut.step([StepEntry("again", requests["r"], [len(requests["r"]) - 1])]).cpu()
    assert float((again[0] - full["r"][-1]).abs().max()) <= atol


def test_toy_mixer_with_state_steps_on_cpu(toy_folder, monkeypatch):
    plain_ops.install(monkeypatch)
    _check_toy(toy_folder, "cpu", "float32", 2e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,fraction", [("float32", 2e-5), ("bfloat16", 2.5e-2)])
def test_toy_mixer_with_state_steps_on_gpu(toy_folder, dtype, fraction):
    _check_toy(toy_folder, "cuda:0", dtype, fraction)


class DeviceDecayMixer(DecayMixer):
    """The same recurrence from the step's device tensors alone: every row's state is a decayed sum over the earlier rows of
    its own entry plus the decayed state its request carried in, so nothing of the step is read on the host and a step
    through it may be captured and replayed with other tokens, positions and slots."""

    capturable = True

    def forward(self, x, ctx, cache):
        drive = x.float() @ self.w_in.T
        entry = ctx.token_seq.long()
        position = ctx.positions.float()
        gap = position[:, None] - position[None, :]
        weight = torch.where((entry[:, None] == entry[None, :]) & (gap >= 0), self.decay ** gap.clamp(min=0), torch.zeros_like(gap))
        slots = ctx.state_slots.long()
        carried = cache.state[slots[entry]] * (self.decay ** (position - ctx.first_positions.float()[entry] + 1))[:, None]
        states = weight @ drive + carried
        cache.state[slots] = states[ctx.seq_starts[1:].long() - 1]          # each entry's last row is what its request keeps
        return (states @ self.w_out.T).to(x.dtype)


@pytest.mark.gpu
def test_a_part_with_state_that_vouches_for_itself_runs_in_the_graphs(toy_folder):
    """Whether steps are captured is each part's own word (``capturable``), not a property of having state: the toy model with
    the host-loop mixer runs kernel by kernel, with the device-only mixer its decode steps and repeated prompt shapes are
    captured, and both generate what the uncaptured engine generates."""
    from tinyllama_inference_engine_b200 import Engine, SamplingParams

    rng = np.random.default_rng(5)
    prompts = [[int(t) for t in rng.integers(0, 97, size=n)] for n in (33, 33, 33, 20)]

    class DeviceRouted(RoutedFeedForward):      # the other two toys read nothing on the host as they are: they only have to say so
        capturable = True

    class DeviceWave(WavePosition):
        capturable = True

    def run(mixer, graphs):
        register_part("mixer", "toy_decay", mixer, replace=True)
        register_part("feed_forward", "toy_routed", DeviceRouted, replace=True)
        register_part("position", "toy_wave", DeviceWave, replace=True)
        engine = Engine(toy_folder, EngineConfig(dtype="float32", page_size=16, max_cache_tokens=640, max_requests=4, max_batch_tokens=40, use_cuda_graphs=graphs))
        out = []
        for wave in range(3):                      # the same step shapes come up again: prompt steps are captured the second time
            out.append([r.generated_tokens for r in engine.generate(prompts, SamplingParams(max_tokens=12))])
        captured = sum(1 for s in engine._sessions.values() if s.graph is not None), sum(1 for g in engine.runner._step_graphs.values() if g.graph is not None)
        return out, engine.runner.model.capturable, captured

    plain, vouched, captured = run(DecayMixer, True)
    assert not vouched and captured == (0, 0)
    eager, vouched, captured = run(DeviceDecayMixer, False)
    assert vouched and captured == (0, 0) and eager == plain
    graphed, vouched, captured = run(DeviceDecayMixer, True)
    assert vouched and captured[0] >= 1 and captured[1] >= 1
    assert graphed == plain


# --- a block kind of its own ----------------------------------------------------------------------------------------------
class TwoFeedForwardBlock(Block):
    """x + mixer(n1 x), then x + ff(n2 x), then x + ff2(n3 x): an arrangement the framework does not have, made of its parts.
    ``norm_then_part`` gives it what the framework's own block gets from the small-step kernels (norm inside the first product,
    residual add and the next norm's input inside the last) without the block knowing any of it."""

    capturable = True
    accepts_next_norm = True
    _SLOTS = (("n1", "norm"), ("mix", "mixer"), ("n2", "norm"), ("ff", "feed_forward"), ("n3", "norm"), ("ff2", "feed_forward"))

    @classmethod
    def tensor_specs(cls, spec, prefix):
        specs = []
        for slot, category in cls._SLOTS:
            specs += part_class(category, spec[slot]).tensor_specs(spec[slot], f"{prefix}.{slot}")
        return specs

    @classmethod
    def cache_need(cls, spec):
        return part_class("mixer", spec["mix"]).cache_need(spec["mix"])

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        for slot, category in self._SLOTS:
            setattr(self, slot, build_part(category, spec[slot], f"{prefix}.{slot}", weights, runtime))

    @property
    def first_norm(self):
        return self.n1

    def forward(self, residual, pending, ctx, cache, next_norm=None):
        from tinyllama_inference_engine_b200 import ops

        fused = residual.shape[0] <= ops.fused_rows_limit(self.runtime.dtype, residual.device)
        pending = norm_then_part(self.n1, self.mix, residual, pending, fused, self.n2, ctx, cache)
        pending = norm_then_part(self.n2, self.ff, residual, pending, fused, self.n3, ctx)
        pending = norm_then_part(self.n3, self.ff2, residual, pending, fused, next_norm, ctx)
        return residual, pending


@dataclass(frozen=True)
class TwoFFConfig:
    hidden_size: int = 128
    vocab_size: int = 211
    first_intermediate: int = 96
    second_intermediate: int = 160
    num_layers: int = 2
    max_position_embeddings: int = 128
    architectures: tuple = ("ToyTwoFFForCausalLM",)

    @classmethod
    def from_dict(cls, data):
        return cls(**{k: (tuple(v) if k == "architectures" else v) for k, v in data.items() if k in cls.__dataclass_fields__})

    def to_dict(self):
        return {**asdict(self), "architectures": list(self.architectures)}


def build_two_ff_spec(c: TwoFFConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": c.hidden_size, "eps": 1e-5})
    attention = PartSpec("attention", {"hidden_size": c.hidden_size, "num_heads": 4, "num_kv_heads": 2, "head_dim": 32, "window": 0, "scale": None,
                                       "position": PartSpec("rotary", {"rotary_dim": 32, "theta": 500.0})})
    mlp = lambda inter: PartSpec("gated_mlp", {"hidden_size": c.hidden_size, "intermediate_size": inter, "activation": "silu"})  # noqa: E731
    block = PartSpec("toy_two_ff", {"n1": norm, "mix": attention, "n2": norm, "ff": mlp(c.first_intermediate), "n3": norm, "ff2": mlp(c.second_intermediate)})
    layers = tuple(LayerSpec(f"t.l{i}", block) for i in range(c.num_layers))
    return ModelSpec("ToyTwoFFForCausalLM", c.hidden_size, c.vocab_size, c.max_position_embeddings,
                     PartSpec("token_embedding", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size, "name": "t.embed"}),
                     layers, tuple(OrderEntry(i, cache=i) for i in range(c.num_layers)), PartSpec("rmsnorm", {"size": c.hidden_size, "eps": 1e-5, "name": "t.norm"}),
                     PartSpec("linear_head", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size, "name": "t.head", "tied_to": None}))


def _plain_two_ff(folder, tokens):
    """The same arrangement from the plain functions (whole sequence, no cache)."""
    import plain_llama

    w = plain_llama.read_safetensors(folder / "model.safetensors")
    c = TwoFFConfig()
    n = len(tokens)
    positions = torch.arange(n)
    x = w["t.embed.weight"].float()[torch.tensor(tokens)]
    for i in range(c.num_layers):
        p = f"t.l{i}"
        h = plain_llama.rms_norm(x, w[f"{p}.n1.weight"].float(), 1e-5)
        q = plain_llama.rope(plain_llama.linear(w[f"{p}.mix.q_proj.weight"].float(), h).view(n, 4, 32), positions, 500.0)
        k = plain_llama.rope(plain_llama.linear(w[f"{p}.mix.k_proj.weight"].float(), h).view(n, 2, 32), positions, 500.0)
        v = plain_llama.linear(w[f"{p}.mix.v_proj.weight"].float(), h).view(n, 2, 32)
        x = x + plain_llama.linear(w[f"{p}.mix.o_proj.weight"].float(), plain_llama.attention(q, k, v).reshape(n, 128))
        for norm, ff in (("n2", "ff"), ("n3", "ff2")):
            h = plain_llama.rms_norm(x, w[f"{p}.{norm}.weight"].float(), 1e-5)
            gated = plain_llama.silu_multiply(plain_llama.linear(w[f"{p}.{ff}.gate_proj.weight"].float(), h), plain_llama.linear(w[f"{p}.{ff}.up_proj.weight"].float(), h))
            x = x + plain_llama.linear(w[f"{p}.{ff}.down_proj.weight"].float(), gated)
    return plain_llama.linear(w["t.head.weight"].float(), plain_llama.rms_norm(x, w["t.norm.weight"].float(), 1e-5))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,fraction", [("float32", 2e-5), ("bfloat16", 2.5e-2)])
def test_a_block_kind_of_its_own_is_registered_and_gets_the_small_step_kernels(tmp_path, dtype, fraction):
    register_part("block", "toy_two_ff", TwoFeedForwardBlock, replace=True)
    register_architecture(Architecture("ToyTwoFFForCausalLM", TwoFFConfig, build_two_ff_spec), replace=True)
    try:
        folder = write_random_model(tmp_path / "two_ff", TwoFFConfig(), seed=11, storage_dtype="bfloat16")
        rng = np.random.default_rng(3)
        tokens = [int(t) for t in rng.integers(0, 211, size=70)]
        want = _plain_two_ff(folder, tokens)
        atol = fraction * float(want.abs().max())
        runner = ModelRunner(folder, EngineConfig(dtype=dtype, page_size=16, max_cache_tokens=256, max_requests=2, max_batch_tokens=64))
        assert runner.model.capturable
        got = [runner.step([StepEntry("r", tokens[:40], list(range(40)))]).cpu()]             # a prompt portion: the many-row kernels
        got.append(runner.step([StepEntry("r", tokens[40:55], list(range(15)))]).cpu())       # 15 rows: the fused small-step kernels
        for i in range(55, 70):                                                              # decoded one by one: prepared norms from product to product
            got.append(runner.step([StepEntry("r", [tokens[i]], [0])]).cpu())
        worst = float((torch.cat(got) - want).abs().max())
        assert worst <= atol, (worst, atol)
    finally:
        unregister_architecture("ToyTwoFFForCausalLM")
        unregister_part("block", "toy_two_ff")
