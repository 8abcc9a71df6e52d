"""Safetensors IO, the one weight error, dtype placement, random weights (no GPU)."""
import os

import pytest
import torch

import helpers as H
from dinfer_b200.weights.loader import (DictSource, SafetensorsSource, WeightError, load_tensors, placed_dtype,
                                        verify)
from dinfer_b200.weights.random_init import model_declarations, write_random_model
from dinfer_b200.weights.safetensors_io import SafetensorsError, SafetensorsFiles, write_safetensors


def test_round_trip_against_the_safetensors_package(tmp_path):
    from safetensors.torch import load_file, save_file
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32),
         "d": torch.randn(2, 2).to(torch.float16)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t.items(), {"note": "hi"})
    back = load_file(p)                       # their reader, our writer
    assert set(back) == set(t) and all(torch.equal(back[k], t[k]) for k in t)
    p2 = str(tmp_path / "y.safetensors")
    save_file(t, p2)                          # their writer, our reader
    f = SafetensorsFiles(p2)
    assert set(f.names()) == set(t)
    assert all(torch.equal(f.tensor(k), t[k]) and f.tensor(k).dtype == t[k].dtype for k in t)
    f.close()


def test_broken_files(tmp_path):
    p = tmp_path / "m.safetensors"
    p.write_bytes(b"\x05\x00")
    with pytest.raises(SafetensorsError, match="shorter"):
        SafetensorsFiles(str(p))
    p.write_bytes((1 << 40).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds"):
        SafetensorsFiles(str(p))
    hdr = b'{"w":{"dtype":"F32","shape":[4],"data_offsets":[0,8]}}'
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="does not fit"):
        SafetensorsFiles(str(p))
    with pytest.raises(SafetensorsError, match="no \\*.safetensors"):
        SafetensorsFiles(str(_empty(tmp_path)))


def _empty(tmp_path):
    d = tmp_path / "empty"
    d.mkdir()
    return d


def test_one_error_lists_everything(tmp_path):
    d = str(tmp_path / "m")
    write_random_model(d, H.TINY_B, 1, 0.03, 0.2, torch.bfloat16)
    from safetensors.torch import load_file
    W = load_file(os.path.join(d, "model.safetensors"))
    del W["model.layers.1.mlp.up_proj.weight"]
    del W["lm_head.weight"]                                   # untied: must be reported
    W["model.layers.0.self_attn.q_norm.weight"] = torch.ones(16)
    W["model.layers.2.self_attn.o_proj.weight"] = torch.zeros(96, 100)
    W["model.extra.bias"] = torch.zeros(3)
    W["model.norm.weight"] = torch.ones(96, dtype=torch.int32)
    decls = model_declarations(H.TINY_B) + []
    from dinfer_b200.parts.spec import TensorDecl
    decls.append(TensorDecl("lm_head.weight", (517, 96), optional=False))
    with pytest.raises(WeightError) as e:
        verify(DictSource(W, "test"), decls)
    err = e.value
    assert set(err.missing) == {"model.layers.1.mlp.up_proj.weight", "lm_head.weight"}
    assert err.unexpected == ["model.extra.bias"]
    assert {n for n, _, _ in err.wrong_shape} == {"model.layers.0.self_attn.q_norm.weight",
                                                   "model.layers.2.self_attn.o_proj.weight"}
    assert [n for n, _, _ in err.wrong_dtype] == ["model.norm.weight"]
    msg = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (2)", "[96, 100], expected [96, 192]",
                 "model.extra.bias", "up_proj"):
        assert word in msg


def test_tied_head_is_optional_and_taken_when_present(tmp_path):
    d = str(tmp_path / "m")
    write_random_model(d, H.TINY_A, 0, 0.05, 0.1, torch.float32)
    src = SafetensorsSource(d)
    assert "lm_head.weight" not in src.names()
    from dinfer_b200.models.decoder import DecoderModel
    from dinfer_b200.config.registry import resolve_architecture
    from dinfer_b200.parts.base import BuildEnv
    arch = resolve_architecture(H.TINY_A)
    spec = arch.build_spec(arch.parse_config(H.TINY_A))
    model = DecoderModel(spec, BuildEnv(torch.device("cpu"), torch.float32, spec.hidden_size, spec.max_positions))
    t = load_tensors(src, model.declarations(), torch.float32, "cpu")
    model.bind(t)
    assert model.lm_head.weight.data_ptr() == model.embedding.data_ptr()
    t["lm_head.weight"] = torch.zeros(256, 64)
    model.bind(t)
    assert model.lm_head.weight.data_ptr() != model.embedding.data_ptr()
    src.close()


def test_placed_dtypes():
    bf, f32 = torch.bfloat16, torch.float32
    assert placed_dtype(bf, "float", bf) == bf
    assert placed_dtype(torch.float16, "float", bf) == bf
    assert placed_dtype(f32, "float", bf) == f32          # stored in 32-bit stays so
    assert placed_dtype(torch.float64, "float", bf) == f32
    assert placed_dtype(bf, "float", f32) == f32          # the 32-bit engine widens everything
    assert placed_dtype(torch.int64, "int", bf) == torch.int32
    src = DictSource({"w": torch.randn(4, 4), "v": torch.randn(4).to(bf)})
    from dinfer_b200.parts.spec import TensorDecl
    out = load_tensors(src, [TensorDecl("w", (4, 4)), TensorDecl("v", (4,))], bf, "cpu")
    assert out["w"].dtype == f32 and out["v"].dtype == bf


def test_random_weights_follow_seed_and_rules(tmp_path):
    from safetensors.torch import load_file
    a = load_file(os.path.join(write_random_model(str(tmp_path / "a"), H.TINY_B, 1, 0.03, 0.2, torch.float32), "model.safetensors"))
    b = load_file(os.path.join(write_random_model(str(tmp_path / "b"), H.TINY_B, 1, 0.03, 0.2, torch.float32), "model.safetensors"))
    c = load_file(os.path.join(write_random_model(str(tmp_path / "c"), H.TINY_B, 2, 0.03, 0.2, torch.float32), "model.safetensors"))
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    w = a["model.layers.0.mlp.gate_proj.weight"]
    assert abs(float(w.std()) - 0.03) < 0.003 and abs(float(w.mean())) < 0.003
    n = a["model.layers.1.input_layernorm.weight"]
    assert float(n.min()) >= 0.8 and float(n.max()) <= 1.2 and float(n.std()) > 0.05
    assert os.path.isfile(tmp_path / "a" / "config.json")
    assert set(a) == {d.name for d in model_declarations(H.TINY_B)}


def test_unused_tensors_are_an_error_unless_allowed(tmp_path):
    """A file with a tensor the model does not use: refused by default (listed in the one error); with
    ``allow_unexpected`` the model loads and the name is reported.  Anything else that does not fit stays an error."""
    import torch
    from dinfer_b200.weights.loader import SafetensorsSource, WeightError, load_tensors
    from dinfer_b200.weights.random_init import model_declarations, random_tensor
    from dinfer_b200.weights.safetensors_io import write_safetensors
    import helpers as H
    decls = model_declarations(H.TINY_A)
    d = tmp_path / "m"
    d.mkdir()
    tensors = [(x.name, random_tensor(x, 0, 0.02, 0.0, torch.float32)) for x in decls]
    tensors.append(("model.layers.0.self_attn.rotary_emb.inv_freq", torch.ones(8)))
    write_safetensors(str(d / "model.safetensors"), tensors)
    src = SafetensorsSource(str(d))
    try:
        with pytest.raises(WeightError) as e:
            load_tensors(src, decls, torch.float32, "cpu")
        assert e.value.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"] and not e.value.missing
        unused = []
        got = load_tensors(src, decls, torch.float32, "cpu", allow_unexpected=True, unused=unused)
        assert unused == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
        assert set(got) == {x.name for x in decls}
        with pytest.raises(WeightError) as e:                       # a missing tensor is never tolerated
            load_tensors(src, decls + [type(decls[0])("model.extra.weight", (3,))], torch.float32, "cpu",
                         allow_unexpected=True)
        assert e.value.missing == ["model.extra.weight"]
    finally:
        src.close()
