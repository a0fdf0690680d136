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
