"""safetensors reading/writing, name binding and its one error (no GPU)."""
import json
import os
import struct

import pytest
import torch

from infero_b200.config import Qwen2Config
from infero_b200.loading import write_random_model_dir
from infero_b200.models import DecoderModel
from infero_b200.weights import (SafetensorsDir, SafetensorsError, WeightsError, load_tensors,
                                 write_safetensors)
from tiny_configs import TINY_A, TINY_B


def _model(cfg):
    return DecoderModel(Qwen2Config.from_dict(cfg).to_model_spec())


def test_random_model_folder_round_trips_and_matches_the_other_reader(tmp_path):
    d = str(tmp_path / "m")
    write_random_model_dir(d, TINY_B, seed=7, dtype="bfloat16", norm_std=0.1)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    assert json.load(open(os.path.join(d, "config.json")))["architectures"] == ["Qwen2ForCausalLM"]
    model = _model(TINY_B)
    t = load_tensors(d, model.declare(), "bfloat16", "cpu")
    assert set(t) == {x.name for x in model.declare()}
    assert t["model.layers.2.self_attn.q_proj.weight"].dtype == torch.bfloat16
    assert "lm_head.weight" in t and t["lm_head.weight"].shape == (1000, 96)
    from safetensors import safe_open
    with safe_open(os.path.join(d, "model.safetensors"), framework="pt") as sf:
        for k in sf.keys():
            assert torch.equal(sf.get_tensor(k), t[k]), k
    # same seed, same values; another seed, other values; independent of tensor order
    d2 = str(tmp_path / "m2")
    write_random_model_dir(d2, TINY_B, seed=7, dtype="bfloat16", norm_std=0.1)
    t2 = load_tensors(d2, model.declare(), "bfloat16", "cpu")
    assert all(torch.equal(t[k], t2[k]) for k in t)
    w = t["model.layers.0.mlp.down_proj.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    n = t["model.norm.weight"].float()
    assert abs(n.mean().item() - 1.0) < 0.05 and 0.05 < n.std().item() < 0.15


def test_tied_model_has_no_head_tensor(tmp_path):
    d = str(tmp_path / "a")
    write_random_model_dir(d, TINY_A, seed=1, dtype="float32")
    names = SafetensorsDir(d).names()
    assert "lm_head.weight" not in names and "model.embed_tokens.weight" in names


def test_precision_policy(tmp_path):
    p = str(tmp_path / "model.safetensors")
    decls = [("a", torch.bfloat16, (2, 3)), ("b", torch.float32, (4,)), ("c", torch.float16, (2,)),
             ("d", torch.int64, (3,))]
    vals = {"a": torch.ones(2, 3, dtype=torch.bfloat16), "b": torch.arange(4, dtype=torch.float32),
            "c": torch.tensor([0.5, 1.5], dtype=torch.float16), "d": torch.tensor([1, 2, 3])}
    write_safetensors(p, decls, lambda n: vals[n])
    from infero_b200.parts.base import TensorDecl
    ds = [TensorDecl(n, s, role="norm" if n == "b" else "matrix") for n, _, s in decls]
    bf = load_tensors(str(tmp_path), ds, "bfloat16", "cpu")
    assert bf["a"].dtype == torch.bfloat16      # stored bf16 stays bf16
    assert bf["b"].dtype == torch.float32       # a norm weight stored in 32-bit stays so
    as_matrix = load_tensors(str(tmp_path), [TensorDecl(n, s) for n, _, s in decls], "bfloat16", "cpu")
    assert as_matrix["b"].dtype == torch.bfloat16   # an operand of a matrix product is rounded once
    as_own = load_tensors(str(tmp_path), [TensorDecl(n, s, role="decay") for n, _, s in decls], "bfloat16", "cpu")
    assert as_own["b"].dtype == torch.float32       # a role a part invents keeps what was stored
    assert bf["c"].dtype == torch.bfloat16      # f16 becomes bf16
    assert bf["d"].dtype == torch.int32         # integer tables as int32
    f32 = load_tensors(str(tmp_path), ds, "float32", "cpu")
    assert all(f32[k].dtype == torch.float32 for k in "abc") and f32["d"].dtype == torch.int32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = str(tmp_path / "m")
    write_random_model_dir(d, TINY_A, seed=3, dtype="float32")
    from safetensors.torch import load_file, save_file
    p = os.path.join(d, "model.safetensors")
    w = load_file(p)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    w["model.layers.0.self_attn.k_proj.bias"] = torch.zeros(31)
    w["model.embed_tokens.weight"] = torch.zeros(512, 63)
    save_file(w, p)
    with pytest.raises(WeightsError) as e:
        load_tensors(d, _model(TINY_A).declare(), "float32", "cpu")
    err = e.value
    assert sorted(err.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert sorted(n for n, _, _ in err.wrong_shape) == ["model.embed_tokens.weight", "model.layers.0.self_attn.k_proj.bias"]
    msg = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (2)", "expected [32] found [31]"):
        assert word in msg, msg


def test_untied_model_without_head_is_a_missing_tensor(tmp_path):
    d = str(tmp_path / "m")
    write_random_model_dir(d, TINY_A, seed=3, dtype="float32")
    with pytest.raises(WeightsError) as e:
        load_tensors(d, _model(dict(TINY_A, tie_word_embeddings=False)).declare(), "float32", "cpu")
    assert e.value.missing == ["lm_head.weight"]


def test_broken_containers_are_refused(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01")
    with pytest.raises(WeightsError):
        load_tensors(str(tmp_path), [], "float32", "cpu")
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 12)
    with pytest.raises(WeightsError) as e:
        load_tensors(str(tmp_path), [], "float32", "cpu")
    assert "needs 16" in str(e.value)
    hdr = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(WeightsError) as e:
        load_tensors(str(tmp_path), [], "float32", "cpu")
    assert "outside the payload" in str(e.value)
    empty = tmp_path / "none"
    empty.mkdir()
    with pytest.raises(WeightsError):
        load_tensors(str(empty), [], "float32", "cpu")


def test_duplicate_name_across_shards(tmp_path):
    for fn in ("a.safetensors", "b.safetensors"):
        write_safetensors(str(tmp_path / fn), [("x", torch.float32, (1,))], lambda n: torch.zeros(1))
    with pytest.raises(SafetensorsError) as e:
        SafetensorsDir(str(tmp_path))
    assert "both" in str(e.value)


def _raw_file(path, header: bytes, payload: bytes = b"", hlen=None):
    import struct
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header) if hlen is None else hlen))
        f.write(header)
        f.write(payload)


@pytest.mark.parametrize("case,needle", [
    ("short", "too short"),
    ("header_past_end", "does not fit"),
    ("not_json", "not valid JSON"),
    ("unknown_dtype", "unsupported dtype"),
    ("offsets_outside", "outside the payload"),
    ("size_mismatch", "needs"),
    ("missing_key", "lacks"),
])
def test_damaged_containers_are_refused(tmp_path, case, needle):
    """The native reader's checks, one damaged file each (crates/safetensors/src/lib.rs:390-436)."""
    from infero_b200.weights.safetensors_io import SafetensorsFile
    p = str(tmp_path / "m.safetensors")
    good = b'{"x":{"dtype":"F32","shape":[2,3],"data_offsets":[0,24]}}'
    if case == "short":
        open(p, "wb").write(b"\x01\x02")
    elif case == "header_past_end":
        _raw_file(p, good, b"\0" * 24, hlen=10_000)
    elif case == "not_json":
        _raw_file(p, b'{"x":{"dtype":"F32","shape":[2,3],"data_offsets":[0,24]', b"\0" * 24)
    elif case == "unknown_dtype":
        _raw_file(p, good.replace(b"F32", b"F8X"), b"\0" * 24)
    elif case == "offsets_outside":
        _raw_file(p, good, b"\0" * 20)
    elif case == "size_mismatch":
        _raw_file(p, good.replace(b"[2,3]", b"[2,4]"), b"\0" * 24)
    elif case == "missing_key":
        _raw_file(p, b'{"x":{"dtype":"F32","shape":[2,3]}}', b"\0" * 24)
    with pytest.raises(SafetensorsError) as e:
        SafetensorsFile(p)
    assert needle in str(e.value), str(e.value)


def test_native_reader_reads_what_the_writer_wrote(tmp_path):
    """Names with escapes and non-ASCII letters, metadata, an empty tensor, every dtype; values
    come back bit for bit as views of the mapping."""
    from infero_b200.weights.safetensors_io import SafetensorsFile
    g = torch.Generator().manual_seed(0)
    tensors = {
        "plain.weight": torch.randn(3, 5, generator=g),
        'quote"and\\slash': torch.randn(4, generator=g).to(torch.bfloat16),
        "größe.层": torch.randint(-5, 5, (2, 2), generator=g, dtype=torch.int32),
        "half": torch.randn(7, generator=g).to(torch.float16),
        "long": torch.arange(6, dtype=torch.int64).view(2, 3),
        "bytes": torch.arange(9, dtype=torch.uint8),
        "empty": torch.zeros((0, 4)),
        "scalar": torch.tensor(3.5),
    }
    p = str(tmp_path / "m.safetensors")
    write_safetensors(p, [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()], lambda n: tensors[n],
                      metadata={"format": "pt", "note": "x\ny"})
    f = SafetensorsFile(p)
    assert set(f.entries) == set(tensors)
    for n, t in tensors.items():
        got = f.tensor(n)
        assert got.dtype == t.dtype and tuple(got.shape) == tuple(t.shape)
        assert torch.equal(got, t)
    f.close()
