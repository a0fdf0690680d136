"""The layer sizes the engine is measured at (two layers of each): bfloat16 against the 32-bit path.

The tiny configurations never reach the kernels that only take head sizes 64 and 128 (TMA-fed
decode attention, tensor-memory prompt attention) or widths above 4096; these do, through
prompt portions, mixed steps and captured decode steps.  The 32-bit path itself is checked
against the plain implementation elsewhere; here it is the reference for sizes the plain
implementation would take minutes for.
"""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = {
    "0.5B": dict(hidden_size=896, num_attention_heads=14, num_key_value_heads=2, head_dim=64,
                 intermediate_size=4864, vocab_size=151936, rms_norm_eps=1e-6, tie_word_embeddings=True),
    "7B": dict(hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
               intermediate_size=18944, vocab_size=152064, rms_norm_eps=1e-6, tie_word_embeddings=False),
    "14B": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
                intermediate_size=13824, vocab_size=152064, rms_norm_eps=1e-5, tie_word_embeddings=False),
}


@pytest.mark.parametrize("name", list(SHAPES))
def test_serving_sizes_bfloat16_against_32_bit(name):
    from infero_b200.config import EngineConfig
    from infero_b200.engine import ModelRunner, StepEntry
    from infero_b200.kernels import tc_gemm
    from infero_b200.loading import random_model
    c = SHAPES[name]
    cfg = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_act="silu", num_hidden_layers=2,
               rope_theta=1e6, max_position_embeddings=8192, **c)
    out = {}
    for dtype in ("float32", "bfloat16"):
        model, _ = random_model(cfg, seed=3, dtype=dtype, device="cuda:0", generate_on_device=True)
        r = ModelRunner(model, EngineConfig(dtype=dtype, page_size=16, num_pages=256, max_seqs=4, ctx=2048,
                                            max_batch_tokens=2048, max_logit_rows=64,
                                            cuda_graphs=(dtype == "bfloat16")))
        # poison what the allocator hands out next: scratch must not be read before it is written
        junk = torch.full((8 << 20,), float("nan"), dtype=torch.float32, device="cuda:0")
        del junk
        rng = random.Random(5)
        toks = {i: [rng.randrange(c["vocab_size"]) for _ in range(n)] for i, n in enumerate((1200, 300, 33))}
        rows = []
        for i in toks:
            r.open(i)
        # (a captured step returns its graph's own output tensor, which the next replay overwrites:
        # every result is copied out at once)
        # (eleven blocks of 128 query rows: at the larger shapes the prompt attention then gives a CTA
        # two heads; the second step's four blocks run with one head per CTA)
        rows.append(r.step([StepEntry(0, toks[0][:1100], [0, 1099]), StepEntry(1, toks[1][:290], [289])]).float().cpu())
        rows.append(r.step([StepEntry(2, toks[2][:32], [31]), StepEntry(0, toks[0][1100:1190], [89])]).float().cpu())
        for k in range(10):                 # first eager, then captured and replayed
            rows.append(r.step([StepEntry(0, [toks[0][1190 + k]], [0]),
                                StepEntry(1, [toks[1][290 + k]], [0])]).float().cpu())
        out[dtype] = torch.cat(rows)
        if dtype == "bfloat16":
            assert r.graph_replays >= 8
        del r, model
        torch.cuda.empty_cache()
    a, b = out["float32"], out["bfloat16"]
    assert torch.isfinite(a).all() and torch.isfinite(b).all()
    err = float((a - b).abs().max() / a.abs().max())
    assert err <= 3e-2, f"{name}: bfloat16 differs from the 32-bit path by {err:.3e} of the largest logit"
    assert tc_gemm.error_flag() == 0


# ---- the measured model's layer widths against the plain implementation ------------------------------
WIDTHS_7B = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_act="silu", num_hidden_layers=2,
                 hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
                 intermediate_size=18944, vocab_size=2999, rms_norm_eps=1e-6, rope_theta=1e6,
                 tie_word_embeddings=False, max_position_embeddings=4096)
_WIDE = {}


def _wide_model():
    """Two layers of the measured 7B widths (group 7, hidden 3584, feed-forward 18944) with the
    vocabulary cut to 2,999 rows so that the head stays cheap: a folder of bf16 tensors, and the plain
    implementation's float64 copy of it on the GPU (torch is the oracle's arithmetic, not the engine's)."""
    if not _WIDE:
        import os
        import tempfile
        import plain_qwen2
        from infero_b200.loading import write_random_model_dir
        d = os.path.join(tempfile.mkdtemp(prefix="infero_b200_wide_"), "m")
        write_random_model_dir(d, WIDTHS_7B, seed=11, dtype="bfloat16", std=0.02, norm_std=0.1)
        cfg, w = plain_qwen2.read_model(d, torch.float64)
        _WIDE.update(dir=d, cfg=cfg, w={k: v.to("cuda:0") for k, v in w.items()})
    return _WIDE


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_measured_widths_equal_the_plain_implementation(dtype):
    """The four cuts (whole, last 32 one by one, changing portions, mixed with page reuse) at the widths
    the benchmark runs, in true 32-bit against the plain implementation (2e-5 of the largest logit) and
    in bfloat16 through the serving kernels."""
    import plain_qwen2
    import replay_util as R
    from engine_fixtures import TOL, make_runner
    from infero_b200.kernels import tc_gemm
    from infero_b200.parts import native_block
    m = _wide_model()
    rng = random.Random(2)
    reqs = {f"r{i}": [rng.randrange(WIDTHS_7B["vocab_size"]) for _ in range(n)]
            for i, n in enumerate([300, 40, 129, 70, 205])}
    plain = {rid: plain_qwen2.forward(m["cfg"], m["w"], toks).cpu().numpy() for rid, toks in reqs.items()}
    cuts = {"whole": R.steps_whole(reqs), "last 32 one by one": R.steps_tail_decode(reqs, 32),
            "changing portions": R.steps_chunked(reqs, seed=1), "mixed": R.steps_mixed(reqs, seed=2, max_live=3)}
    calls = native_block.CALLS[0]
    for what, steps in cuts.items():
        runner = make_runner(m["dir"], dtype, R.max_live_tokens(steps, reqs))
        got = R.replay_inprocess(runner, steps)
        err, where = R.compare(got, plain)
        assert err <= TOL[dtype], f"{what}, {dtype}: relative error {err:.3e} at {where}"
        if what == "mixed":
            assert runner.manager.pages_reused > 0
        del runner
    if dtype == "bfloat16":
        assert native_block.CALLS[0] > calls and tc_gemm.error_flag() == 0
