"""Generation through the Python entry point and the continuous-batching engine
on the GPU, against the plain model; and a toy mixer with state of its own
that is registered, built and stepped without touching the package."""

from __future__ import annotations

import pytest
import torch

import kernel_refs as R
import plain_qwen2 as P
from conftest import TINY
from helpers import bf16_round, check_logits, plain_logits, random_tokens

pytestmark = pytest.mark.gpu


def plain_generate(cfg, w, prompt, n_new, params=None, schedule=None):
    """Tokens of the plain model with the engine's sampling rule, and per token the margin between the chosen token's
    score and the runner-up (greedy only)."""
    toks, out, margin = list(prompt), [], []
    for i in range(n_new):
        lg = P.plain_forward(cfg, w, toks, schedule)[-1]
        if params is None:
            top2 = torch.topk(lg, 2).values
            margin.append(float(top2[0] - top2[1]))
            t = P.plain_argmax(lg)
        else:
            t, _ = R.sample_row(lg, params["temperature"], params["top_k"], params["top_p"], params["seed"], i)
        out.append(t)
        toks.append(t)
    return out, margin


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_entry_point(dtype, model_dirs):
    from litinfer_b200 import Qwen2

    cfg, w = P.read_model_folder(model_dirs["A"])
    if dtype == "bfloat16":
        w = bf16_round(w)
    model = Qwen2(str(model_dirs["A"]), dtype=dtype)
    exact = 0
    for n in (5, 11, 17):
        prompt = random_tokens(n, cfg["vocab_size"], 300 + n)
        ref, margins = plain_generate(cfg, w, prompt, 8)
        got = model.generate(prompt, max_new_tokens=8)
        assert len(got) == 8
        exact += got == ref
        if dtype == "float32":
            assert min(margins) > 1e-4
            assert got == ref
        else:
            # bfloat16 may legitimately pick the runner-up, but only where the plain model's own margin is tiny
            assert P.same_up_to_a_near_tie(got, ref, margins), f"prompt {n}: {got} vs {ref}, margins {margins}"
    assert exact >= 2, "bfloat16 flipped a near-tie in more than one prompt of three"
    assert model.generate(prompt, max_new_tokens=0) == []
    assert len(model.generate(prompt)) == 1                      # None means one token (qwen2.py:324)
    with pytest.raises(ValueError):
        model.generate(prompt, max_new_tokens=cfg["max_position_embeddings"])
    toks, metrics = model.generate_profile(prompt, max_new_tokens=4)
    assert metrics["generated_tokens"] == 4 and metrics["decode_tokens"] == 3 and metrics["prefill_seconds"] > 0
    assert list(model.generate_stream(prompt, max_new_tokens=4)) == toks


@pytest.mark.parametrize("name", ["B", "B0"])
def test_engine_sampling_is_reproducible_and_batch_independent(name, model_dirs):
    """Config B's workload: prompts of 1/9/33/40 tokens in 16-token portions mixed with
    decoding, temperature 0.8 from a fixed seed, 12 tokens each; on the configuration exactly as given and on its
    variant with a window and sizes that are no round numbers."""
    from litinfer_b200 import Qwen2

    cfg, w = P.read_model_folder(model_dirs[name])
    model = Qwen2(str(model_dirs[name]), dtype="float32", num_pages=24, max_num_seqs=4, max_tokens_per_step=32, prefill_chunk=16)
    prompts = [random_tokens(n, cfg["vocab_size"], 500 + n) for n in (1, 9, 33, 40)]
    par = dict(temperature=0.8, top_k=0, top_p=1.0)
    model.engine_start()
    ids = [model.engine_add_request(p, 12, seed=70 + i, **par) for i, p in enumerate(prompts)]
    steps = 0
    while model.engine_has_unfinished():
        model.engine_step()
        steps += 1
    together = [model.engine_get_output(i) for i in ids]
    assert all(model.engine_is_finished(i) for i in ids) and all(len(t) == 12 for t in together)
    model.engine_stop()
    for i, p in enumerate(prompts):
        alone = model.generate(p, max_new_tokens=12, seed=70 + i, **par)
        assert alone == together[i], f"request {i}: tokens depend on the batch"
        ref, _ = plain_generate(cfg, w, p, 12, dict(seed=70 + i, **par))
        assert alone == ref, f"request {i}: differs from the plain model with the same draws"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_run_ahead_on_the_device(dtype, model_dirs):
    """Decode steps launched ahead (captured graphs, token ids passed from the sampler's output on the device): the same
    tokens as step by step, greedy and sampled, with requests that end at different lengths and on an end-of-sequence
    token; and through the entry point."""
    from litinfer_b200 import Qwen2

    cfg, _ = P.read_model_folder(model_dirs["B"])
    prompts = [random_tokens(n, cfg["vocab_size"], 500 + n) for n in (5, 40, 17, 3, 64)]
    new = [30, 12, 45, 7, 20]

    def run(run_ahead, eos, sampled):
        front = Qwen2(str(model_dirs["B"]), dtype=dtype, max_num_seqs=8, run_ahead=run_ahead)
        front.engine_start()
        front._eng().scheduler.eos = set(eos)
        ids = [front.engine_add_request(p, n, **(dict(top_k=30, top_p=0.9, temperature=0.7, seed=11 + i) if sampled else {}))
               for i, (p, n) in enumerate(zip(prompts, new))]
        steps = 0
        while front.engine_has_unfinished():
            front.engine_step()
            steps += 1
            assert steps < 1000
        outs = [front.engine_get_output(i) for i in ids]
        eng = front._eng()
        eng.manager.check()
        assert eng.manager.num_free_slots() == 8
        replays = eng.runner.graph_replays
        front.engine_stop()
        return outs, replays

    plain, _ = run(False, (), False)
    assert [len(o) for o in plain] == new
    eos = plain[2][20]
    for sampled in (False, True):
        for e in ((), (eos,)):
            a, _ = run(False, e, sampled)
            b, replays = run(True, e, sampled)
            assert a == b, f"run_ahead changes the outputs (eos {e}, sampled {sampled})"
            assert replays > 20, "decode steps were meant to run through captured graphs"
    # through the entry point, a request alone (in bfloat16 a request alone and in a batch may differ by rounding: other kernels)
    ahead, plainly = Qwen2(str(model_dirs["B"]), dtype=dtype, run_ahead=True), Qwen2(str(model_dirs["B"]), dtype=dtype)
    for i in (2, 0, 4):                                                       # the engine of generate is used again
        assert ahead.generate(prompts[i], max_new_tokens=new[i]) == plainly.generate(prompts[i], max_new_tokens=new[i])
    assert list(ahead.generate_stream(prompts[1], max_new_tokens=5))[:3] == plainly.generate(prompts[1], max_new_tokens=5)[:3]


def test_engine_preempts_and_recomputes_when_pages_run_out(model_dirs):
    from litinfer_b200 import DecoderModel, Engine, EngineConfig

    cfg, w = P.read_model_folder(model_dirs["A"])
    model = DecoderModel.from_dir(model_dirs["A"], "float32", "cuda:0")
    eng = Engine(model, EngineConfig(num_pages=7, max_num_seqs=4, max_tokens_per_step=64, prefill_chunk=32))
    prompts = [random_tokens(n, cfg["vocab_size"], 600 + n) for n in (30, 28, 27)]
    ids = [eng.add_request(p, 24) for p in prompts]
    eng.run_to_completion()
    assert eng.scheduler.num_preemptions > 0, "the pool was meant to be too small for all three"
    eng.manager.check()
    assert eng.manager.num_free_pages(0) == 7
    for rid, p in zip(ids, prompts):
        ref, margins = plain_generate(cfg, w, p, 24)
        assert min(margins) > 1e-4
        assert eng.get_output(rid) == ref


# --------------------------------------------------------------------------
# a toy mixer with state of its own
# --------------------------------------------------------------------------

def test_toy_mixer_with_state_registers_builds_and_steps(model_dirs):
    run_toy_mixer(model_dirs, "cuda:0")


def run_toy_mixer(model_dirs, device):
    """An exponential moving average over the sequence, y_t = s_t, s_t = a * s_{t-1} + (1 - a) * W h_t,
    with s kept in the request's state slot.  Defined here, registered from outside, chosen
    per layer by a spec; the package's files are not touched."""
    from litinfer_b200 import DecoderModel, StepItem
    from litinfer_b200.cache import CacheManager
    from litinfer_b200.config import ScheduleEntry, load_config
    from litinfer_b200.engine import ModelRunner
    from litinfer_b200.parts import MIXERS, FixedState, FusedLinear, Mixer
    from litinfer_b200.config import PartSpec
    from dataclasses import replace

    MIXERS.register("toy_ema", _ema_mixer_class())
    try:
        base = load_config(model_dirs["A"]).to_model_spec()
        blocks = list(base.blocks)
        toy = PartSpec("toy_ema", {"hidden_size": base.hidden_size, "decay": 0.75})
        blocks[1] = blocks[1].with_part("mixer", toy, "ema.")
        spec = replace(base, blocks=tuple(blocks))
        model = DecoderModel.from_random(spec, 5, "float32", device)
        manager = CacheManager(model.cache_requirements(), [e.cache_from for e in spec.schedule], 16, 16, 3, model.dtype, model.device)
        assert [e.kind for e in manager.entries] == ["paged", "state"]
        runner = ModelRunner(model, manager)
        toks = random_tokens(40, spec.vocab_size, 9)

        def run(cuts, rid):
            rc = manager.admit(rid)
            outs, pos = [], 0
            for n in cuts:
                manager.extend(rc, pos + n)
                outs.append(runner.step([StepItem(rc, toks[pos:pos + n], list(range(n)))]).clone())
                pos += n
            manager.release(rc)
            return torch.cat(outs)

        whole = run([40], 1)
        cut = run([7, 2, 16, 1, 1, 13], 2)               # the same slot again: it must have been cleared
        assert torch.isfinite(whole).all()
        assert (whole - cut).abs().max() < 1e-4
        # the state matters: another decay gives other logits
        assert (whole[5:] - whole[:-5]).abs().max() > 1e-3
    finally:
        MIXERS.unregister("toy_ema")


def _ema_mixer_class():
    """The toy mixer with state of its own (see run_toy_mixer), as a class to register."""
    from litinfer_b200.parts import FixedState, FusedLinear, Mixer

    class EmaMixer(Mixer):
        def __init__(self, spec, prefix, dtype, device):
            super().__init__(spec, prefix, dtype, device)
            self.hidden = int(spec["hidden_size"])
            self.decay = float(spec["decay"])
            self.proj = FusedLinear(prefix, ["in_proj"], self.hidden, [self.hidden], False, dtype)

        def params(self):
            return self.proj.params()

        def bind(self, tensors):
            self.proj.bind(tensors)

        def cache_requirement(self):
            return FixedState((self.hidden,), torch.float32)

        def forward(self, h, ctx, cache):
            u = self.proj(h).float()
            y = torch.empty_like(u)
            for s in range(ctx.num_seqs):
                lo, hi = ctx.host_q_start[s], ctx.host_q_start[s + 1]
                st = cache.state[ctx.host_state_slots[s]]
                for t in range(lo, hi):
                    st.mul_(self.decay).add_((1 - self.decay) * u[t])
                    y[t] = st
            return y.to(self.dtype)

    return EmaMixer


def test_toy_mixer_with_state_through_the_engine_and_the_entry_point(model_dirs):
    run_toy_mixer_through_engine(model_dirs, "cuda:0")


def run_toy_mixer_through_engine(model_dirs, device):
    """The mixer with state of its own under the scheduler: default engine options (graphs asked for: the runner must
    not capture anything for such a model), several requests decoding together, a pool so small that a request is
    preempted and recomputed (its slot is cleared when it is admitted again), and the entry point's generate.  Every
    request's tokens equal those of the same request run alone."""
    from dataclasses import replace

    from litinfer_b200 import CausalLM, DecoderModel, Engine, EngineConfig
    from litinfer_b200.config import PartSpec, load_config
    from litinfer_b200.parts import MIXERS

    MIXERS.register("toy_ema", _ema_mixer_class())
    try:
        base = load_config(model_dirs["A"]).to_model_spec()
        blocks = list(base.blocks)
        blocks[1] = blocks[1].with_part("mixer", PartSpec("toy_ema", {"hidden_size": base.hidden_size, "decay": 0.75}), "ema.")
        spec = replace(base, blocks=tuple(blocks))
        model = DecoderModel.from_random(spec, 5, "float32", device)
        prompts = [random_tokens(n, spec.vocab_size, 900 + n) for n in (30, 28, 27)]

        alone = []
        for p in prompts:
            eng = Engine(model, EngineConfig(num_pages=16, max_num_seqs=1))          # use_graphs is on by default
            assert not eng.runner.use_graphs, "nothing of a model with state of its own may be captured"
            rid = eng.add_request(p, 24)
            eng.run_to_completion()
            alone.append(eng.get_output(rid))
        assert len({tuple(a) for a in alone}) == 3

        for run_ahead in (False, True):
            eng = Engine(model, EngineConfig(num_pages=7, max_num_seqs=4, max_tokens_per_step=64, prefill_chunk=16, run_ahead=run_ahead))
            ids = [eng.add_request(p, 24) for p in prompts]
            eng.run_to_completion()
            assert eng.scheduler.num_preemptions > 0, "the pool was meant to be too small for all three"
            eng.manager.check()
            assert eng.manager.num_free_pages(0) == 7 and eng.manager.num_free_slots() == 4
            assert eng.runner.graph_replays == 0
            for rid, a in zip(ids, alone):
                assert eng.get_output(rid) == a, f"request {rid} (run_ahead {run_ahead}): tokens differ from the request run alone"

        front = CausalLM(None, device=device, model=model, num_pages=16)
        for p, a in zip(prompts, alone):
            assert front.generate(p, max_new_tokens=24) == a
    finally:
        MIXERS.unregister("toy_ema")


def _ema_mixer_on_device_class():
    """The same toy mixer, which takes steps of single tokens from the device's copy of the step: its decode steps may
    be captured (parts.base.Mixer.decodes_from_device)."""
    host = _ema_mixer_class()

    class EmaMixerOnDevice(host):
        decodes_from_device = True

        def forward(self, h, ctx, cache):
            if ctx.max_q_len != 1:
                return super().forward(h, ctx, cache)
            u = self.proj(h).float()                       # token s is sequence s
            slots = ctx.state_slots.long()
            st = cache.state.index_select(0, slots) * self.decay + (1 - self.decay) * u
            cache.state.index_copy_(0, slots, st)          # padded sequences of a captured step all name the spare slot
            return st.to(self.dtype)

    return EmaMixerOnDevice


def test_toy_mixer_with_state_in_captured_decode_steps(model_dirs):
    run_toy_mixer_in_captured_steps(model_dirs, "cuda:0")


def run_toy_mixer_in_captured_steps(model_dirs, device):
    """A mixer with state of its own that says it decodes from the device's copy of the step: its model's decode steps are
    captured and replayed (portions of prompts still run plainly and unsplit), the runs that warm a capture up advance
    nobody's state, and every request gives the tokens of the mixer that walks the step on the host: alone, and three
    together in a pool so small that one is preempted and recomputed."""
    from dataclasses import replace

    from litinfer_b200 import DecoderModel, Engine, EngineConfig
    from litinfer_b200.config import PartSpec, load_config
    from litinfer_b200.parts import MIXERS

    MIXERS.register("toy_ema", _ema_mixer_class())
    MIXERS.register("toy_ema_on_device", _ema_mixer_on_device_class())
    try:
        base = load_config(model_dirs["A"]).to_model_spec()
        models = {}
        for kind in ("toy_ema", "toy_ema_on_device"):
            blocks = list(base.blocks)
            blocks[1] = blocks[1].with_part("mixer", PartSpec(kind, {"hidden_size": base.hidden_size, "decay": 0.75}), "ema.")
            models[kind] = DecoderModel.from_random(replace(base, blocks=tuple(blocks)), 5, "float32", device)
        prompts = [random_tokens(n, base.vocab_size, 900 + n) for n in (30, 28, 27)]
        on_gpu = torch.device(device).type == "cuda"

        def alone(model, p):
            eng = Engine(model, EngineConfig(num_pages=16, max_num_seqs=1))          # use_graphs is on by default
            rid = eng.add_request(p, 24)
            eng.run_to_completion()
            return eng, eng.get_output(rid)

        want = []
        for p in prompts:
            eng, out = alone(models["toy_ema"], p)
            assert not eng.runner.use_graphs and eng.runner.graph_replays == 0 and not eng.runner._state_in_graphs
            want.append(out)
            eng, out = alone(models["toy_ema_on_device"], p)
            assert eng.runner.use_graphs == on_gpu and not eng.runner._may_split and eng.runner._state_in_graphs
            assert (eng.runner.graph_replays >= 20) == on_gpu and not eng.runner._step_graphs
            assert out == want[-1], "decoding from the device's copy of the step gives other tokens than the walk on the host"
        assert len({tuple(a) for a in want}) == 3

        for run_ahead in (False, True):
            eng = Engine(models["toy_ema_on_device"],
                         EngineConfig(num_pages=7, max_num_seqs=4, max_tokens_per_step=64, prefill_chunk=16, run_ahead=run_ahead))
            ids = [eng.add_request(p, 24) for p in prompts]
            eng.run_to_completion()
            assert eng.scheduler.num_preemptions > 0, "the pool was meant to be too small for all three"
            eng.manager.check()
            assert eng.manager.num_free_pages(0) == 7 and eng.manager.num_free_slots() == 4
            assert (eng.runner.graph_replays > 0) == on_gpu
            for rid, a in zip(ids, want):
                assert eng.get_output(rid) == a, f"request {rid} (run_ahead {run_ahead}): tokens differ from the request run alone"
    finally:
        MIXERS.unregister("toy_ema")
        MIXERS.unregister("toy_ema_on_device")


# --------------------------------------------------------------------------
# a whole architecture from outside the package: its own config.json keys and tensor names
# --------------------------------------------------------------------------

def _toy_architecture_class():
    """A configuration class that shares nothing with Qwen2's: other config.json keys, other tensor-name stems.  What it
    describes is the same arithmetic, so that the plain model can say what the logits must be."""
    import math
    from dataclasses import dataclass

    from litinfer_b200.config import BlockSpec, ModelSpec, PartSpec
    from litinfer_b200.config.spec import default_schedule

    @dataclass(frozen=True)
    class ToyConfig:
        width: int
        depth: int
        heads: int
        groups: int
        head_size: int
        inner: int
        vocab: int
        limit: int
        eps: float
        theta: float
        own_head: bool
        torch_dtype: str = "float32"

        @classmethod
        def from_dict(cls, d):
            return cls(int(d["toy_width"]), int(d["toy_depth"]), int(d["toy_heads"]), int(d["toy_groups"]), int(d["toy_head_size"]),
                       int(d["toy_inner"]), int(d["toy_vocab"]), int(d["toy_limit"]), float(d["toy_eps"]), float(d["toy_theta"]),
                       bool(d["toy_own_head"]), str(d.get("torch_dtype", "float32")))

        def to_model_spec(self):
            norm = PartSpec("rmsnorm", {"size": self.width, "eps": self.eps})
            rope = PartSpec("rope", {"theta": self.theta, "rotary_dim": self.head_size, "pairing": "half"})
            ffn = PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": self.inner})
            mixer = PartSpec("attention", {"hidden_size": self.width, "num_heads": self.heads, "num_kv_heads": self.groups,
                                           "head_dim": self.head_size, "qkv_bias": True, "out_bias": False,
                                           "scale": 1.0 / math.sqrt(self.head_size), "window": None, "position": rope})
            stems = {"mixer": "mix.", "feed_forward": "ffn.", "mixer_norm": "ln1.", "feed_forward_norm": "ln2."}
            blocks = tuple(BlockSpec.of("prenorm", f"net.h.{i}.", stems, mixer=mixer, feed_forward=ffn, mixer_norm=norm, feed_forward_norm=norm)
                           for i in range(self.depth))
            return ModelSpec(architecture="ToyForCausalLM", vocab_size=self.vocab, hidden_size=self.width, blocks=blocks,
                             schedule=default_schedule(self.depth), final_norm=norm, tie_word_embeddings=not self.own_head,
                             max_position_embeddings=self.limit, embedding_name="net.tok.weight", final_norm_prefix="net.ln_out.",
                             lm_head_name="net.head.weight")

    return ToyConfig


_TOY_STEMS = ((".self_attn.", ".mix."), (".mlp.", ".ffn."), (".input_layernorm.", ".ln1."), (".post_attention_layernorm.", ".ln2."),
              ("model.layers.", "net.h."), ("model.embed_tokens.", "net.tok."), ("model.norm.", "net.ln_out."), ("lm_head.", "net.head."))


def test_toy_architecture_from_a_folder(model_dirs, tmp_path):
    run_toy_architecture("A", "float32", model_dirs, tmp_path, "cuda:0")


def run_toy_architecture(name, dtype, model_dirs, tmp_path, device):
    """An architecture registered from outside the package, with config.json keys and tensor names of its own, goes the
    whole way without a change to the package: configuration by name, weights by name (with the loader's one error for
    what does not match), the generic model, the step function in portions and single tokens, random weights into a
    folder, the front end.  Its folder holds a tiny Qwen2 model's tensors under the toy names, so the plain model of that
    Qwen2 folder says what the logits are."""
    import json

    from litinfer_b200 import CausalLM, DecoderModel
    from litinfer_b200.config import ConfigError, load_config, register_architecture, registry, supported_architectures
    from litinfer_b200.engine.replay import Replayer
    from litinfer_b200.weights import WeightError, iter_tensors, write_file, write_model_folder

    cfg = TINY[name]
    toy_cfg = dict(architectures=["ToyForCausalLM"], torch_dtype="float32", toy_width=cfg["hidden_size"], toy_depth=cfg["num_hidden_layers"],
                   toy_heads=cfg["num_attention_heads"], toy_groups=cfg["num_key_value_heads"], toy_head_size=cfg["head_dim"],
                   toy_inner=cfg["intermediate_size"], toy_vocab=cfg["vocab_size"], toy_limit=cfg["max_position_embeddings"],
                   toy_eps=cfg["rms_norm_eps"], toy_theta=cfg["rope_theta"], toy_own_head=not cfg["tie_word_embeddings"])
    folder = tmp_path / "toy"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(toy_cfg))
    tensors = {}
    for tensor_name, t in iter_tensors(model_dirs[name] / "model.safetensors"):
        for old, new in _TOY_STEMS:
            tensor_name = tensor_name.replace(old, new)
        tensors[tensor_name] = t
    write_file(folder / "model.safetensors", tensors)

    with pytest.raises(ConfigError, match="ToyForCausalLM"):
        load_config(folder)
    register_architecture("ToyForCausalLM", _toy_architecture_class())
    try:
        assert "ToyForCausalLM" in supported_architectures()
        spec = load_config(folder).to_model_spec()
        assert spec.architecture == "ToyForCausalLM" and len(spec.blocks) == cfg["num_hidden_layers"]
        model = DecoderModel.from_dir(folder, dtype, torch.device(device))
        toks = random_tokens(40, cfg["vocab_size"], 77)
        ref = plain_logits(model_dirs[name], toks, dtype)
        rp = Replayer(model, 64, max_live=2, use_graphs=True)
        got = [rp.step(dict(step=0, entries=[dict(id="a", tokens=toks[:23], want=[0, 22])])).clone().cpu()]
        got.append(rp.step(dict(step=1, entries=[dict(id="a", tokens=toks[23:30], want=[6])])).clone().cpu())
        for i in range(30, 40):
            got.append(rp.step(dict(step=i, entries=[dict(id="a", tokens=[toks[i]], want=[0])])).clone().cpu())
        check_logits(torch.cat(got), ref[[0, 22, 29] + list(range(30, 40))], dtype, f"toy architecture over the tensors of {name}, {dtype}")

        # a tensor under a name the toy architecture does not declare, and one it declares missing: one error for both
        broken = tmp_path / "broken"
        broken.mkdir()
        (broken / "config.json").write_text(json.dumps(toy_cfg))
        wrong = dict(tensors)
        wrong["model.norm.weight"] = wrong.pop("net.ln_out.weight")
        write_file(broken / "model.safetensors", wrong)
        with pytest.raises(WeightError) as err:
            DecoderModel.from_dir(broken, dtype, torch.device(device))
        assert "net.ln_out.weight" in str(err.value) and "model.norm.weight" in str(err.value)

        # random weights into a folder (the same for the same seed, others for another) and the front end's generate
        outs, drawn = [], []
        for seed, sub in ((11, "r1"), (11, "r2"), (12, "r3")):
            d = write_model_folder(tmp_path / sub, dict(toy_cfg), seed=seed, store_dtype="float32")
            drawn.append(dict(iter_tensors(d / "model.safetensors")))
            front = CausalLM(None, device=device, model=DecoderModel.from_dir(d, dtype, torch.device(device)), num_pages=8)
            outs.append(front.generate(toks[:12], max_new_tokens=8))
        assert sorted(drawn[0]) == sorted(tensors) and all(drawn[0][k].shape == tensors[k].shape for k in tensors)
        assert all(torch.equal(drawn[0][k], drawn[1][k]) for k in tensors) and not torch.equal(drawn[0]["net.tok.weight"], drawn[2]["net.tok.weight"])
        assert len(outs[0]) == 8 and outs[0] == outs[1]
    finally:
        registry._ARCHITECTURES.pop("ToyForCausalLM", None)


# --------------------------------------------------------------------------
# toy position encodings that are no rotation, and a block of another shape
# --------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_positions_and_block_arrangements(dtype, model_dirs):
    run_toy_positions_and_blocks(model_dirs, "cuda:0", dtype)


def run_toy_positions_and_blocks(model_dirs, device, dtype):
    """Registered from here, with no change to the package: learned absolute positions (a table added to the residual
    stream after the embedding: the model's own position part), attention without any position encoding, a block with
    four norms (one before and one after each of mixer and feed-forward), a block without a feed-forward, a factor on
    the embedding and a cap on the logits.  Each model whole, in portions and token by token: bitwise equal in float32."""
    from dataclasses import replace

    from litinfer_b200 import DecoderModel, StepItem
    from litinfer_b200 import kernels as K
    from litinfer_b200.cache import CacheManager
    from litinfer_b200.config import PartSpec, load_config
    from litinfer_b200.engine import ModelRunner
    from litinfer_b200.parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Block, Position
    from litinfer_b200.weights.loader import ParamSpec

    class LearnedPositions(Position):
        def __init__(self, spec, prefix, dtype, device):
            super().__init__(spec, prefix, dtype, device)
            self.size, self.positions = int(spec["size"]), int(spec["positions"])
            self.table = None

        def params(self):
            return [ParamSpec(self.prefix + "positions.weight", (self.positions, self.size), role="keep", std=0.5)]

        def bind(self, tensors):
            self.table = tensors.pop(self.prefix + "positions.weight").float()

        def add_to_stream(self, x32, ctx):
            x32.add_(self.table[ctx.positions.long()])

    class SandwichBlock(Block):
        """x += post_norm(Mixer(pre_norm(x))); x += post_norm(FeedForward(pre_norm(x)))."""

        def __init__(self, spec, prefix, dtype, device):
            super().__init__(spec, prefix, dtype, device)
            self.mixer_norm = self.build(NORMS, "mixer_norm")
            self.mixer = self.build(MIXERS, "mixer")
            self.mixer_post_norm = self.build(NORMS, "mixer_post_norm")
            self.feed_forward_norm = self.build(NORMS, "feed_forward_norm")
            self.feed_forward = self.build(FEED_FORWARDS, "feed_forward")
            self.feed_forward_post_norm = self.build(NORMS, "feed_forward_post_norm")

        def parts(self):
            return [self.mixer_norm, self.mixer, self.mixer_post_norm, self.feed_forward_norm, self.feed_forward, self.feed_forward_post_norm]

        def forward(self, x32, ctx, cache, carry, next_entry=None):
            if carry is not None and carry.delta is not None:
                K.residual_add(x32, carry.delta)
            y = self.mixer.forward(self.mixer_norm.forward(x32), ctx, cache)
            K.residual_add(x32, self.mixer_post_norm.forward(y.float()))
            y = self.feed_forward.forward(self.feed_forward_norm.forward(x32), ctx)
            K.residual_add(x32, self.feed_forward_post_norm.forward(y.float()))
            return x32, None

    POSITIONS.register("toy_learned", LearnedPositions)
    BLOCKS.register("toy_sandwich", SandwichBlock)
    try:
        base = load_config(model_dirs["A"]).to_model_spec()
        H = base.hidden_size
        norm = base.blocks[0].part("mixer_norm")
        toks = random_tokens(50, base.vocab_size, 9)
        cuts_list = ([50], [7, 2, 16, 1, 1, 13, 1, 1, 1, 7], [1] * 50)

        def logits_of(spec, cuts):
            model = DecoderModel.from_random(spec, 5, dtype, device)
            manager = CacheManager(model.cache_requirements(), [e.cache_from for e in spec.schedule], 16, 16, 2, model.dtype, model.device)
            runner = ModelRunner(model, manager)
            rc = manager.admit(1)
            outs, pos = [], 0
            for n in cuts:
                manager.extend(rc, pos + n)
                outs.append(runner.step([StepItem(rc, toks[pos:pos + n], list(range(n)))]).clone())
                pos += n
            manager.release(rc)
            return torch.cat(outs)

        def all_cuts_agree(spec, what):
            whole = logits_of(spec, cuts_list[0])
            assert torch.isfinite(whole).all(), what
            for cuts in cuts_list[1:]:
                cut = logits_of(spec, cuts)
                if dtype == "float32" and str(device).startswith("cuda"):
                    assert torch.equal(whole, cut), f"{what}: float32 logits differ between cuts by {(whole - cut).abs().max()}"
                elif dtype == "float32":                   # the plain references under the CPU twin of this test sum in other orders
                    assert (whole - cut).abs().max() <= 1e-5, what
                else:
                    assert (whole - cut).abs().max() <= 0.03 * float(whole.abs().max()), what
            return whole

        reference = all_cuts_agree(base, "the unchanged model")

        # attention without positions: the same keys in another order give the same logits at the last token
        bare = tuple(b.with_part("mixer", b.part("mixer").replace(position=None)) for b in base.blocks)
        no_pos = replace(base, blocks=bare)
        got = all_cuts_agree(no_pos, "no positions")
        assert (got - reference).abs().max() > 1e-3, "dropping the rotation must matter"

        # learned absolute positions on top of it, as the model's own position part
        learned = replace(no_pos, position=PartSpec("toy_learned", {"size": H, "positions": base.max_position_embeddings}))
        got_learned = all_cuts_agree(learned, "learned positions")
        assert (got_learned - got).abs().max() > 1e-2, "the table of positions must matter"
        names = [p.name for p in DecoderModel(learned, "float32", "meta").params()]
        assert "model.positions.weight" in names

        # a block with four norms in the second layer, under tensor names of its own
        sandwich = base.blocks[1].with_kind("toy_sandwich").with_part("mixer_post_norm", norm).with_part("feed_forward_post_norm", norm, "post_ffn_norm.")
        spec4 = replace(base, blocks=(base.blocks[0], sandwich))
        got4 = all_cuts_agree(spec4, "a block with four norms")
        assert (got4 - reference).abs().max() > 1e-3
        names = [p.name for p in DecoderModel(spec4, "float32", "meta").params()]
        assert "model.layers.1.mixer_post_norm.weight" in names and "model.layers.1.post_ffn_norm.weight" in names

        # a layer without a feed-forward, first and last
        for where in (0, 1):
            blocks = list(base.blocks)
            blocks[where] = blocks[where].with_part("feed_forward", None).with_part("feed_forward_norm", None)
            got = all_cuts_agree(replace(base, blocks=tuple(blocks)), f"layer {where} without a feed-forward")
            assert (got - reference).abs().max() > 1e-3

        # a factor on the embedding and a cap on the logits
        scaled = all_cuts_agree(replace(base, embedding_scale=3.0, logit_cap=2.0), "embedding scale and logit cap")
        assert float(scaled.abs().max()) <= 2.0 and (scaled - reference).abs().max() > 1e-3
        capped = all_cuts_agree(replace(base, logit_cap=0.5), "logit cap")
        want = 0.5 * torch.tanh(reference / 0.5)
        assert (capped - want).abs().max() <= (1e-5 if dtype == "float32" else 0.02)
    finally:
        POSITIONS.unregister("toy_learned")
        BLOCKS.unregister("toy_sandwich")


# --------------------------------------------------------------------------
# a toy feed-forward with routing and a toy position encoding
# --------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_feed_forward_and_toy_positions(dtype, model_dirs):
    run_toy_feed_forward_and_positions(model_dirs, "cuda:0", dtype)


def run_toy_feed_forward_and_positions(model_dirs, device, dtype):
    """Two more kinds of parts registered from outside the package and chosen per layer by a spec.

    A feed-forward with routing: the router's logits (float32) pick one of four small gated experts per token.
    A position encoding: rotary with the positions stretched by a factor (it owns its table of denominators, which is
    all the attention kernels ask of it).  Checked: the parts alone against plain formulas; a model built from them
    whole, in portions and token by token; and that each of them changes the logits."""
    from dataclasses import replace

    from litinfer_b200 import DecoderModel, StepItem
    from litinfer_b200.cache import CacheManager
    from litinfer_b200.config import PartSpec, load_config
    from litinfer_b200.engine import ModelRunner
    from litinfer_b200.parts import FEED_FORWARDS, POSITIONS, FeedForward, FusedLinear, Position, Rotary
    from litinfer_b200.weights.loader import ParamSpec

    class RoutedFF(FeedForward):
        def __init__(self, spec, prefix, dtype, device):
            super().__init__(spec, prefix, dtype, device)
            self.hidden, self.inner, self.experts = int(spec["hidden_size"]), int(spec["expert_size"]), int(spec["experts"])
            self.up = [FusedLinear(prefix, [f"experts.{e}.up"], self.hidden, [self.inner], False, dtype) for e in range(self.experts)]
            self.gate = [FusedLinear(prefix, [f"experts.{e}.gate"], self.hidden, [self.inner], False, dtype) for e in range(self.experts)]
            self.down = [FusedLinear(prefix, [f"experts.{e}.down"], self.inner, [self.hidden], False, dtype) for e in range(self.experts)]
            self.router = None

        def params(self):
            out = [ParamSpec(self.prefix + "router.weight", (self.experts, self.hidden), role="keep", std=0.5)]
            for group in (self.up, self.gate, self.down):
                for lin in group:
                    out += lin.params()
            return out

        def bind(self, tensors):
            self.router = tensors.pop(self.prefix + "router.weight").float()
            for group in (self.up, self.gate, self.down):
                for lin in group:
                    lin.bind(tensors)

        def forward(self, h, ctx):
            logits = h.float() @ self.router.t()                      # routing in float32
            choice = logits.argmax(-1)
            weight = torch.softmax(logits, -1).gather(1, choice[:, None])
            y = torch.zeros(h.shape[0], self.hidden, dtype=torch.float32, device=h.device)
            for e in range(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    x = h[rows].contiguous()
                    g, u = self.gate[e](x).float(), self.up[e](x).float()
                    y[rows] = self.down[e]((u * (g / (1 + torch.exp(-g)))).to(self.dtype)).float()
            return (y * weight).to(self.dtype)

    class StretchedRope(Position):
        def __init__(self, spec, prefix, dtype, device, head_dim=None):
            super().__init__(spec, prefix, dtype, device)
            self.rotary_dim = int(head_dim)
            j = torch.arange(self.rotary_dim // 2, dtype=torch.float32)
            self.denominators = (float(spec["stretch"]) * torch.pow(torch.tensor(float(spec["theta"])), 2.0 * j / self.rotary_dim)).to(self.device)

        def rotary(self, ctx):
            return Rotary(self.denominators, self.rotary_dim)

    FEED_FORWARDS.register("toy_routed", RoutedFF)
    POSITIONS.register("toy_stretched_rope", StretchedRope)
    try:
        base = load_config(model_dirs["A"]).to_model_spec()
        H = base.hidden_size
        tdt = torch.float32 if dtype == "float32" else torch.bfloat16
        # the routed part alone against the plain formula
        ff = RoutedFF(PartSpec("toy_routed", {"hidden_size": H, "expert_size": 48, "experts": 4}), "ff.", tdt, device)
        g = torch.Generator().manual_seed(3)
        tensors = {p.name: (torch.randn(p.shape, generator=g) * (p.std or 0.1)).to(device) for p in ff.params()}
        plain = {k: v.float().cpu() if "router" in k else v.to(tdt).float().cpu() for k, v in tensors.items()}
        ff.bind({k: (v if "router" in k else v.to(tdt)) for k, v in tensors.items()})
        h = (torch.randn(23, H, generator=g)).to(tdt)
        got = ff.forward(h.to(device), None).float().cpu()
        logits = h.float() @ plain["ff.router.weight"].t()
        choice, prob = logits.argmax(-1), torch.softmax(logits, -1).max(-1).values
        assert len(set(choice.tolist())) >= 3, "the test wants several experts in use"
        ref = torch.zeros(23, H)
        for t in range(23):
            e = int(choice[t])
            gate, up = h[t].float() @ plain[f"ff.experts.{e}.gate.weight"].t(), h[t].float() @ plain[f"ff.experts.{e}.up.weight"].t()
            act = up * (gate / (1 + torch.exp(-gate)))
            ref[t] = prob[t] * (act.to(tdt).float() @ plain[f"ff.experts.{e}.down.weight"].t())
        tol = 1e-5 if dtype == "float32" else 0.02
        assert (got - ref).abs().max() <= tol * max(1.0, float(ref.abs().max())), f"routed feed-forward: {(got - ref).abs().max()}"

        # a model with both toy parts in its second layer
        blocks = list(base.blocks)
        routed = PartSpec("toy_routed", {"hidden_size": H, "expert_size": 48, "experts": 4})

        def with_stretch(stretch):
            mixer = blocks[1].part("mixer")
            pos = PartSpec("toy_stretched_rope", {"theta": mixer["position"]["theta"], "stretch": stretch})
            return blocks[1].with_part("mixer", mixer.replace(position=pos)).with_part("feed_forward", routed)

        def logits_of(stretch, cuts):
            spec = replace(base, blocks=(blocks[0], with_stretch(stretch)) + tuple(blocks[2:]))
            model = DecoderModel.from_random(spec, 5, dtype, device)
            manager = CacheManager(model.cache_requirements(), [e.cache_from for e in spec.schedule], 16, 16, 2, model.dtype, model.device)
            runner = ModelRunner(model, manager)
            toks = random_tokens(50, spec.vocab_size, 9)
            rc = manager.admit(1)
            outs, pos = [], 0
            for n in cuts:
                manager.extend(rc, pos + n)
                outs.append(runner.step([StepItem(rc, toks[pos:pos + n], list(range(n)))]).clone())
                pos += n
            manager.release(rc)
            return torch.cat(outs)

        whole = logits_of(2.0, [50])
        cut = logits_of(2.0, [7, 2, 16, 1, 1, 13, 1, 1, 1, 7])
        assert torch.isfinite(whole).all()
        scale = float(whole.abs().max())
        assert (whole - cut).abs().max() <= (1e-4 if dtype == "float32" else 0.03 * scale)
        other = logits_of(1.0, [50])
        # with random weights attention is nearly uniform and positions move the logits little, but measurably
        assert (whole[10:] - other[10:]).abs().max() > 1e-3, "the stretch of the positions must matter"
    finally:
        FEED_FORWARDS.unregister("toy_routed")
        POSITIONS.unregister("toy_stretched_rope")



@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_that_come_back_run_from_captured_shapes(dtype, model_dirs):
    """The same longer prompt again and again through the entry point, and a batch of requests in portions under a
    small token budget: from the second time on a step's shape is replayed from its captured graph, and the tokens stay
    what the plain model generates."""
    from litinfer_b200 import Qwen2

    cfg, w = P.read_model_folder(model_dirs["C"])
    if dtype == "bfloat16":
        w = bf16_round(w)
    front = Qwen2(str(model_dirs["C"]), dtype=dtype, max_num_seqs=4, max_tokens_per_step=96, prefill_chunk=80)
    prompt = random_tokens(150, cfg["vocab_size"], 321)
    ref, margins = plain_generate(cfg, w, prompt, 6)
    for _ in range(3):
        got = front.generate(prompt, max_new_tokens=6)
        assert got == ref or (dtype == "bfloat16" and P.same_up_to_a_near_tie(got, ref, margins)), f"{got} vs {ref} (margins {margins})"
    assert len(front._single.runner._step_graphs) >= 1, "the portions of 80 and 70 tokens came back and were meant to be captured"
    prompts = [random_tokens(n, cfg["vocab_size"], 700 + n) for n in (150, 97, 130, 66)]
    front.engine_start()
    ids = [front.engine_add_request(p, 5) for p in prompts]
    while front.engine_has_unfinished():
        front.engine_step()
    outs = [front.engine_get_output(i) for i in ids]
    assert front._eng().runner.graph_replays > 0
    front.engine_stop()
    exact = 0
    for p, o in zip(prompts, outs):
        r, m = plain_generate(cfg, w, p, 5)
        exact += o == r
        assert o == r or (dtype == "bfloat16" and P.same_up_to_a_near_tie(o, r, m)), f"prompt of {len(p)}: {o} vs {r} (margins {m})"
    assert exact >= len(prompts) - 1


def test_profile_and_trace_switches_of_the_command_line(model_dirs):
    """LLAISYS_PROFILE=1 and LLAISYS_TRACE=1 (LitInfer's switches) on the command line as a user runs it: a table of device
    time per phase and kernel at exit, a line per call, and the same tokens as without them."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    cmd = [sys.executable, "-m", "litinfer_b200", "--model", str(model_dirs["A"]), "--prompt", "5 17 3 200 41", "--max_steps", "6", "--test"]
    plain = subprocess.run(cmd, capture_output=True, text=True, cwd=root, timeout=600)
    assert plain.returncode == 0, plain.stderr[-2000:]
    env = dict(os.environ, LLAISYS_PROFILE="1", LLAISYS_TRACE="1")
    prof = subprocess.run(cmd, capture_output=True, text=True, cwd=root, timeout=600, env=env)
    assert prof.returncode == 0, prof.stderr[-2000:]
    assert prof.stdout == plain.stdout
    err = prof.stderr
    assert "LLAISYS PROFILE" in err and "total op time" in err
    assert "prefill/linear" in err and "decode/paged_attention" in err and "decode/linear_rope_kv" in err
    assert "[LLAISYS] Calling generate ntokens=5" in err and "[LLAISYS] step sequences=1" in err
    assert "LLAISYS PROFILE" not in plain.stderr
