"""Each part of a layer alone against its plain statement, at sizes no tiny model has, and a toy
mixer with state of its own that is defined here, registered from outside the package, built
from a configuration and stepped without a change to the package's files."""
import json
import math
import os
import tempfile
from types import SimpleNamespace

import pytest
import torch

import plain_qwen2 as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def _rand(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


def _rel(got, ref):
    from infero_b200.kernels import Partials
    if isinstance(got, Partials):                       # a product left as split-K partial sums
        got = got.materialize(torch.float32)
    return float((got.double().cpu() - ref).abs().max() / ref.abs().max())


# ---- norm, feed-forward --------------------------------------------------------------------------
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dt):
    from infero_b200.config.spec import NormSpec
    from infero_b200.parts import RmsNorm
    d, T, eps = 200, 6, 3e-4
    norm = RmsNorm(NormSpec("rmsnorm", d, eps), "n.weight")
    assert [t.name for t in norm.declare()] == ["n.weight"] and norm.declare()[0].shape == (d,)
    w = _rand((d,), dt, 1) + 1
    norm.bind({"n.weight": w})
    x = _rand((T, d), torch.float32, 2)
    delta = _rand((T, d), dt, 3)
    ref_x = x.double().cpu() + delta.double().cpu()
    ref = P.rms_norm(ref_x, w.double().cpu(), eps)
    h = norm.forward(SimpleNamespace(act_dtype=dt), x, delta)
    assert h.dtype == dt and _rel(h, ref) <= TOL[dt]
    assert _rel(x, ref_x) <= 1e-6                        # the residual stream moved on


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_swiglu_part(dt):
    from infero_b200.config.spec import FeedForwardSpec
    from infero_b200.parts import SwiGluMlp
    d, ff, T = 72, 200, 5
    mlp = SwiGluMlp(FeedForwardSpec("swiglu", d, ff), "L")
    names = {t.name: t.shape for t in mlp.declare()}
    assert names == {"L.mlp.gate_proj.weight": (ff, d), "L.mlp.up_proj.weight": (ff, d),
                     "L.mlp.down_proj.weight": (d, ff)}
    w = {n: _rand(s, dt, i, 0.2) for i, (n, s) in enumerate(names.items())}
    mlp.bind(w)
    h = _rand((T, d), dt, 9)
    out = mlp.forward(SimpleNamespace(act_dtype=dt), h)
    ref = P.swiglu_mlp(h.double().cpu(), *(w[n].double().cpu() for n in names))
    assert _rel(out, ref) <= TOL[dt]


def test_rope_part_table():
    """The part owns the table of inverse frequencies: 64-bit on the host, rounded once."""
    from infero_b200.config.spec import PositionSpec
    from infero_b200.parts import RopeNeox
    theta, rotary = 12345.0, 24
    inv = RopeNeox(PositionSpec("rope_neox", theta, rotary)).inv_freq(DEV)
    ref = torch.tensor([theta ** (-2.0 * i / rotary) for i in range(rotary // 2)], dtype=torch.float64)
    assert inv.dtype == torch.float32 and inv.device.type == "cuda" and inv.shape == (rotary // 2,)
    assert torch.equal(inv.cpu(), ref.float())
    with pytest.raises(ValueError):
        RopeNeox(PositionSpec("rope_neox", theta, 7))


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_block_alone(dt):
    """One pre-norm block, called directly on a residual stream with a pending delta, against the
    plain layer: the block adds the pending delta, leaves x after the mixer's add, and returns the
    feed-forward's delta for the next norm to add."""
    from infero_b200.engine import StepEntry
    spec = _spec(layers=1, H=4, Hkv=4, D=16, d=88, ff=136, theta=777.0, eps=1e-4)
    model, runner, w = _build(spec, dt)
    block = model.blocks[0]
    T = 37
    cfg = {"num_attention_heads": 4, "num_key_value_heads": 4, "head_dim": 16, "hidden_size": 88,
           "rms_norm_eps": 1e-4, "rope_theta": 777.0}
    x0 = _rand((T, 88), torch.float32, 21)
    pending = _rand((T, 88), dt, 22, 0.3)
    start = x0.double().cpu() + pending.double().cpu()
    ref = P.decoder_layer(start, w, cfg, 0, torch.arange(T))
    # a step's context for one whole request of T tokens (the token ids play no part here)
    runner.open("r")
    captured = {}
    real_forward = block.forward

    def spy(ctx, x, delta, slot):
        x.copy_(x0)
        captured["delta"] = real_forward(ctx, x, pending, slot)
        captured["x"] = x.clone()
        return captured["delta"]

    block.forward = spy
    runner.step([StepEntry("r", [1] * T, [T - 1])])
    block.forward = real_forward
    from infero_b200.kernels import Partials
    delta = captured["delta"]
    delta = delta.materialize(torch.float32) if isinstance(delta, Partials) else delta.float()
    got = captured["x"].double().cpu() + delta.double().cpu()
    assert _rel(got, ref) <= TOL[dt]


# ---- a model assembled from a hand-written spec: mixer, block, schedule ----------------------------
def _spec(window=None, layers=1, schedule=None, H=6, Hkv=2, D=48, d=80, ff=144, V=300, theta=5000.0, eps=2e-5,
          tie=False):
    from infero_b200.config.spec import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                                          ScheduleEntry)
    pos = PositionSpec("rope_neox", theta, D)
    norm = NormSpec("rmsnorm", d, eps)
    blocks = tuple(BlockSpec("prenorm", f"model.layers.{i}",
                             MixerSpec("gqa_attention", d, H, Hkv, D, qkv_bias=True, scale=1 / math.sqrt(D),
                                       window=window, position=pos),
                             FeedForwardSpec("swiglu", d, ff), norm, norm) for i in range(layers))
    sched = schedule or tuple(ScheduleEntry(i, i) for i in range(layers))
    return ModelSpec("Hand", V, d, blocks, sched, norm, tie)


def _build(spec, dt, seed=3, pages=32, std=0.08):
    from infero_b200.config import EngineConfig
    from infero_b200.engine import ModelRunner
    from infero_b200.models.decoder import DecoderModel
    from infero_b200.weights import random_tensors
    model = DecoderModel(spec)
    tensors = random_tensors(model.declare(), seed, dt, std=std, norm_std=0.1, device="cpu")
    model.bind({k: v.to(DEV) for k, v in tensors.items()})
    cfg = EngineConfig(dtype="float32" if dt == torch.float32 else "bfloat16", page_size=16, num_pages=pages,
                       max_seqs=4, ctx=pages * 16, max_batch_tokens=512, max_logit_rows=512, cuda_graphs=False)
    return model, ModelRunner(model, cfg), {k: v.double() for k, v in tensors.items()}


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 24])
def test_attention_mixer_alone(dt, window):
    """GqaAttention.forward on a two-request batch whose second request already has keys in the
    cache, against the plain q/k/v + rotary + attention + output product."""
    from infero_b200.engine import StepEntry
    spec = _spec(window=window)
    model, runner, w = _build(spec, dt)
    mixer = model.blocks[0].mixer
    d = spec.hidden
    m = spec.blocks[0].mixer
    lens = {"a": (0, 37), "b": (21, 9)}                    # (already cached, new)
    h_all = {r: _rand((o + n, d), dt, 40 + i) for i, (r, (o, n)) in enumerate(lens.items())}
    # request b's first 21 tokens go through the mixer first, in a step of their own
    for rid in lens:
        runner.open(rid)
    rcs = [runner.manager.get("b")]
    e = [StepEntry("b", [1] * 21, [])]
    runner.manager.reserve(rcs[0], 21)
    ctx, _ = runner._build_context(e, rcs)
    mixer.forward(ctx, h_all["b"][:21].contiguous(), spec.schedule[0])
    runner.manager.commit(rcs[0], 21)
    ents = [StepEntry("a", [1] * 37, []), StepEntry("b", [1] * 9, [])]
    rcs = [runner.manager.get("a"), runner.manager.get("b")]
    for rc, en in zip(rcs, ents):
        runner.manager.reserve(rc, len(en.tokens))
    ctx, _ = runner._build_context(ents, rcs)
    h = torch.cat([h_all["a"], h_all["b"][21:]]).contiguous()
    out = mixer.forward(ctx, h, spec.schedule[0])
    from infero_b200.kernels import Partials
    full = out.materialize(torch.float32) if isinstance(out, Partials) else out
    p = "model.layers.0.self_attn."
    worst = 0.0
    row = 0
    for rid, (old, new) in lens.items():
        hh = h_all[rid].double().cpu()
        T = old + new
        q = hh @ w[p + "q_proj.weight"].T + w[p + "q_proj.bias"]
        k = hh @ w[p + "k_proj.weight"].T + w[p + "k_proj.bias"]
        v = hh @ w[p + "v_proj.weight"].T + w[p + "v_proj.bias"]
        pos = torch.arange(T)
        q = P.rope_neox(q.view(T, m.num_heads, m.head_dim), pos, m.position.theta, m.position.rotary_dim)
        k = P.rope_neox(k.view(T, m.num_kv_heads, m.head_dim), pos, m.position.theta, m.position.rotary_dim)
        a = P.attention(q, k, v.view(T, m.num_kv_heads, m.head_dim), m.scale, window)
        ref = a.reshape(T, -1) @ w[p + "o_proj.weight"].T
        worst = max(worst, _rel(full[row:row + new], ref[old:]))
        row += new
    assert worst <= TOL[dt], f"{worst:.3e}"


@pytest.mark.parametrize("dt,sizes", [(torch.float32, dict(H=6, Hkv=2, D=48, d=80, ff=144)),
                                      (torch.bfloat16, dict(H=6, Hkv=2, D=48, d=80, ff=144)),
                                      # head size 64: the bf16 steps go through the native launcher, and the steps
                                      # of single tokens through the fused decode attention (which appends nothing
                                      # in the read-only execution) and the folded norms
                                      (torch.bfloat16, dict(H=4, Hkv=2, D=64, d=128, ff=320))],
                         ids=["float32", "bfloat16", "bfloat16-serving-kernels"])
def test_schedule_names_a_layer_twice_and_shares_a_cache(dt, sizes):
    """Three executions of two blocks: block 0, block 1, block 0 again; the third execution reads
    the cache the first one filled and writes nothing."""
    from infero_b200.config.spec import ScheduleEntry
    from infero_b200.engine import StepEntry
    from infero_b200.parts import native_block as NB
    sched = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 0, write_cache=False))
    spec = _spec(layers=2, schedule=sched, **sizes)
    model, runner, w = _build(spec, dt)
    assert model.spec.num_cache_slots() == 2
    native_before = NB.CALLS[0]
    toks = [int(t) for t in torch.randint(0, 300, (45,), generator=torch.Generator().manual_seed(5))]
    # plain: run the layers in that order; a read-only execution attends over the keys of the
    # first execution's input
    cfg = {"num_attention_heads": sizes["H"], "num_key_value_heads": sizes["Hkv"], "head_dim": sizes["D"],
           "hidden_size": sizes["d"], "rms_norm_eps": 2e-5, "rope_theta": 5000.0}
    x = w["model.embed_tokens.weight"][torch.tensor(toks)]
    pos = torch.arange(len(toks))
    x1 = P.decoder_layer(x, w, cfg, 0, pos)
    x2 = P.decoder_layer(x1, w, cfg, 1, pos)
    x3 = _layer_reading_cache(x2, x, w, cfg, 0, pos)
    ref = P.rms_norm(x3, w["model.norm.weight"], 2e-5) @ w["lm_head.weight"].T
    runner.open("r")
    got = [runner.step([StepEntry("r", toks[:30], list(range(30)))]),
           runner.step([StepEntry("r", toks[30:41], list(range(11)))])]
    got += [runner.step([StepEntry("r", [t], [0])]) for t in toks[41:]]
    got = torch.cat(got)
    assert _rel(got, ref) <= TOL[dt] * 1.5
    if sizes["D"] == 64:
        assert NB.CALLS[0] - native_before == 3 * 6, "every execution of every step should have gone the native way"


def _layer_reading_cache(x, x_keys, w, cfg, i, pos):
    """Block i on x, with keys and values computed from x_keys (the input the writing execution saw)."""
    p = f"model.layers.{i}."
    H, Hkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    T = x.shape[0]
    h = P.rms_norm(x, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
    hk = P.rms_norm(x_keys, w[p + "input_layernorm.weight"], cfg["rms_norm_eps"])
    q = h @ w[p + "self_attn.q_proj.weight"].T + w[p + "self_attn.q_proj.bias"]
    k = hk @ w[p + "self_attn.k_proj.weight"].T + w[p + "self_attn.k_proj.bias"]
    v = hk @ w[p + "self_attn.v_proj.weight"].T + w[p + "self_attn.v_proj.bias"]
    q = P.rope_neox(q.view(T, H, D), pos, cfg["rope_theta"], D)
    k = P.rope_neox(k.view(T, Hkv, D), pos, cfg["rope_theta"], D)
    a = P.attention(q, k, v.view(T, Hkv, D), 1 / math.sqrt(D), None)
    x = x + a.reshape(T, H * D) @ w[p + "self_attn.o_proj.weight"].T
    h = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    return x + P.swiglu_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                            w[p + "mlp.down_proj.weight"])



@pytest.mark.parametrize("shape", [dict(H=4, Hkv=2, D=64, d=128, ff=320), dict(H=2, Hkv=1, D=128, d=256, ff=616),
                                   # a residual width of 512 lets the few-token products cut K into splits: gate and
                                   # up then come as partial sums and the SwiGLU kernel adds them up
                                   dict(H=8, Hkv=2, D=64, d=512, ff=200)],
                         ids=["head64", "head128", "split_k"])
@pytest.mark.parametrize("window", [None, 24])
def test_native_block_launcher_changes_nothing(window, shape):
    """The block launched by one native call per layer gives, bit for bit, what its parts give when
    they launch their kernels one by one: prompts in portions (more than 256 rows: finished products;
    fewer: partial sums), mixed batches, single tokens; with and without a window; at both head sizes
    of the TMA-fed attention kernels.  That holds with the norm kernels kept as kernels; with them folded
    into the products around them (steps of single tokens) bf16 rounding falls elsewhere and the logits
    agree closely instead."""
    from infero_b200.engine import StepEntry
    from infero_b200.kernels import tc_gemm
    from infero_b200.parts import native_block as NB
    spec = _spec(layers=3, window=window, V=400, **shape)
    if shape["d"] == 512:
        assert tc_gemm.plan(8, 2 * shape["ff"], 512, DEV)[0] >= 2, "this shape was meant to cut K into splits"
    toks = {r: [int(t) for t in torch.randint(0, 400, (n,), generator=torch.Generator().manual_seed(s))]
            for r, n, s in (("a", 300, 1), ("b", 41, 2), ("c", 7, 3))}

    from infero_b200.models import native_decoder as ND

    def run(native, fold_norms=False, whole_step=False):
        NB.set_enabled(native)
        NB.set_fusion(True, fold_norms)
        ND.set_enabled(whole_step)
        steps_before = ND.CALLS[0]
        try:
            model, runner, _ = _build(spec, torch.bfloat16, pages=40)
            before = NB.CALLS[0]
            for r in toks:
                runner.open(r)
            out = [runner.step([StepEntry("a", toks["a"][:280], [279])]),                       # many rows
                   runner.step([StepEntry("b", toks["b"][:40], [5, 39]), StepEntry("a", toks["a"][280:290], [9])]),
                   runner.step([StepEntry("a", toks["a"][290:291], [0]), StepEntry("b", toks["b"][40:], [0]),
                                StepEntry("c", toks["c"], [6])]),                                # decodes beside a prompt
                   runner.step([StepEntry("a", toks["a"][291:292], [0])]),
                   runner.step([StepEntry("a", toks["a"][292:293], [0]), StepEntry("b", [7], [0])])]   # single tokens only
            assert ND.CALLS[0] - steps_before == (5 if whole_step else 0)
            return [o.float().cpu() for o in out], NB.CALLS[0] - before
        finally:
            NB.set_enabled(True)
            NB.set_fusion(True, True)
            ND.set_enabled(True)

    plain, n_plain = run(False)
    native, n_native = run(True)
    assert n_plain == 0 and n_native == 5 * 3, "every layer of every step should have gone the native way"
    for a, b in zip(plain, native):
        assert torch.equal(a, b)
    # the whole step in one native call: launch for launch what the loop over blocks does
    whole, n_whole = run(True, whole_step=True)
    assert n_whole == 5 * 3
    for a, b in zip(plain, whole):
        assert torch.equal(a, b)
    folded_whole, _ = run(True, fold_norms=True, whole_step=True)
    folded, _ = run(True, fold_norms=True)
    for a, b in zip(folded, folded_whole):
        assert torch.equal(a, b)
    for a, b in zip(plain[:3], folded[:3]):            # steps with a prompt portion: nothing is folded
        assert torch.equal(a, b)
    # two bf16 paths whose roundings fall in different places (bf16(x * rstd * w) against bf16(x * w) * rstd):
    # each is held to the bf16 bound against the plain implementation by the replay tests; against each
    # other they are held to the same bound here
    from engine_fixtures import TOL
    for a, b in zip(plain[3:], folded[3:]):
        gap = float((a - b).abs().max() / a.abs().max())
        assert gap <= TOL["bfloat16"], f"folded norms: {gap:.3e}"


# ---- a toy mixer with state of its own, from outside the package ------------------------------------
def _register_toy():
    """A mixer that keeps a running, decaying sum of its projected inputs per request:
    s_t = decay * s_{t-1} + h_t W^T, delta_t = s_t.  Its state is one vector per request, kept in
    the cache manager's state slots; it has no paged cache.  Plain torch on the device: it is a
    test part, not a product kernel."""
    from infero_b200 import register_architecture, register_part
    from infero_b200.config.spec import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                                          ScheduleEntry)
    from infero_b200.parts.base import Mixer, StateSpec, TensorDecl

    class DecaySum(Mixer):
        def __init__(self, spec, prefix):
            self.spec, self.prefix = spec, prefix
            self.decay = float(spec.get("decay"))
            self.w = None

        def declare(self):
            return [TensorDecl(f"{self.prefix}.toy.proj.weight", (self.spec.hidden, self.spec.hidden))]

        def bind(self, tensors):
            self.w = tensors[f"{self.prefix}.toy.proj.weight"]

        def state_spec(self):
            return StateSpec((self.spec.hidden,), torch.float32)

        def forward(self, ctx, h, slot):
            state = ctx.state(slot.cache)                    # [max requests, hidden]
            u = h.float() @ self.w.float().T
            out = torch.empty_like(u)
            for e in range(ctx.n_entries):
                s = state[int(ctx.h_slot[e])]
                r0 = int(ctx.h_q_start[e])
                for r in range(r0, r0 + int(ctx.h_q_len[e])):
                    s.mul_(self.decay).add_(u[r])
                    out[r] = s
            return out.to(h.dtype)

    def read_config(raw):
        return dict(raw)

    def to_spec(c):
        d = c["width"]
        norm = NormSpec("rmsnorm", d, c["eps"])
        blocks = []
        for i, kind in enumerate(c["mixers"]):
            if kind == "decay_sum":
                mixer = MixerSpec("decay_sum", d, extra=(("decay", c["decay"]),))
            else:
                D = c["head"]
                mixer = MixerSpec("gqa_attention", d, c["heads"], c["kv_heads"], D, qkv_bias=True,
                                  scale=1 / math.sqrt(D), position=PositionSpec("rope_neox", c["theta"], D))
            blocks.append(BlockSpec("prenorm", f"model.layers.{i}", mixer, FeedForwardSpec("swiglu", d, c["inner"]),
                                    norm, norm))
        return ModelSpec("ToyDecayForCausalLM", c["vocab"], d, tuple(blocks),
                         tuple(ScheduleEntry(i, i) for i in range(len(blocks))), norm, True)

    register_part("mixer", "decay_sum", DecaySum)
    register_architecture("ToyDecayForCausalLM", read_config, to_spec)


TOY = {"architectures": ["ToyDecayForCausalLM"], "width": 56, "inner": 120, "vocab": 211, "eps": 1e-5,
       "decay": 0.8, "mixers": ["decay_sum", "attention", "decay_sum"], "heads": 2, "kv_heads": 1, "head": 32,
       "theta": 10000.0}


def _toy_plain(w, toks):
    c = TOY
    x = w["model.embed_tokens.weight"][torch.tensor(toks)]
    pos = torch.arange(len(toks))
    cfg = {"num_attention_heads": c["heads"], "num_key_value_heads": c["kv_heads"], "head_dim": c["head"],
           "hidden_size": c["width"], "rms_norm_eps": c["eps"], "rope_theta": c["theta"]}
    for i, kind in enumerate(c["mixers"]):
        p = f"model.layers.{i}."
        if kind == "attention":
            x = P.decoder_layer(x, w, cfg, i, pos)
            continue
        h = P.rms_norm(x, w[p + "input_layernorm.weight"], c["eps"])
        u = h @ w[p + "toy.proj.weight"].T
        s = torch.zeros(c["width"], dtype=x.dtype)
        rows = []
        for t in range(len(toks)):
            s = c["decay"] * s + u[t]
            rows.append(s)
        x = x + torch.stack(rows)
        h = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"])
        x = x + P.swiglu_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                             w[p + "mlp.down_proj.weight"])
    return P.rms_norm(x, w["model.norm.weight"], c["eps"]) @ w["model.embed_tokens.weight"].T


def test_a_toy_mixer_with_its_own_state_plugs_in():
    """Registered here, built from a config.json by its architecture name, loaded from a model
    folder written in random-weights mode, and stepped in portions beside other requests, with
    state slots given back and used again."""
    from infero_b200.config import EngineConfig
    from infero_b200.engine import ModelRunner, StepEntry
    from infero_b200.loading import load_model, write_random_model_dir
    _register_toy()
    with tempfile.TemporaryDirectory(prefix="infero_b200_toy_") as tmp:
        write_random_model_dir(tmp, TOY, seed=5, dtype="float32", std=0.1, norm_std=0.1)
        assert json.load(open(os.path.join(tmp, "config.json")))["architectures"] == ["ToyDecayForCausalLM"]
        model, _ = load_model(tmp, "float32", DEV)
        _, w = P.read_model(tmp, torch.float64)
    assert set(model.state_specs) == {0, 2} and set(model.kv_specs) == {1}
    runner = ModelRunner(model, EngineConfig(dtype="float32", page_size=16, num_pages=12, max_seqs=2, ctx=192,
                                             max_batch_tokens=256, max_logit_rows=256, cuda_graphs=False))
    g = torch.Generator().manual_seed(1)
    reqs = {r: [int(t) for t in torch.randint(0, TOY["vocab"], (n,), generator=g)]
            for r, n in (("a", 50), ("b", 23), ("c", 31))}
    plain = {r: _toy_plain(w, t) for r, t in reqs.items()}
    got = {r: [] for r in reqs}

    def run(parts):
        out = runner.step([StepEntry(r, reqs[r][a:b], list(range(b - a))) for r, a, b in parts])
        row = 0
        for r, a, b in parts:
            got[r].append(out[row:row + b - a])
            row += b - a

    runner.open("a"); runner.open("b")
    run([("a", 0, 20), ("b", 0, 2)])
    run([("b", 2, 3), ("a", 20, 37)])
    run([("a", 37, 38), ("b", 3, 23)])
    slot_b = runner.manager.get("b").slot
    runner.close("b")
    runner.open("c")                                      # takes b's state slot: it must start from zero
    assert runner.manager.get("c").slot == slot_b
    run([("c", 0, 30), ("a", 38, 50)])
    run([("c", 30, 31)])
    for r in reqs:
        err = _rel(torch.cat(got[r]), plain[r])
        assert err <= 2e-5, f"request {r}: {err:.3e}"
