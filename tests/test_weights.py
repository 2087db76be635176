"""safetensors reading and writing, the loader's single error, the random-weights mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

from conftest import TINY
from rust_inference_b200 import config_from_dict, write_random_model
from rust_inference_b200.config.registry import get_architecture
from rust_inference_b200.engine.model import declared_tensors
from rust_inference_b200.weights.loader import WeightError, random_tensors, read_model_tensors
from rust_inference_b200.weights.safetensors_io import (ModelFiles, SafetensorsFile, WeightFileError,
                                                        write_safetensors)


def _spec(name):
    cfg = config_from_dict(TINY[name])
    return cfg, get_architecture(cfg.architecture).build_spec(cfg)


def test_round_trip_keeps_stored_precision(tmp_path):
    t = {
        "a": torch.randn(3, 5),
        "b": torch.randn(7, 2).bfloat16(),
        "c": torch.randn(4).half(),
        "d": torch.arange(6, dtype=torch.int64).view(2, 3),
        "e": torch.arange(4, dtype=torch.int32),
    }
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, t, metadata={"k": "v"})
    f = SafetensorsFile(path)
    assert set(f.names()) == set(t) and f.metadata == {"k": "v"}
    assert f.tensor("a").dtype == torch.float32 and torch.equal(f.tensor("a"), t["a"])
    assert f.tensor("b").dtype == torch.bfloat16 and torch.equal(f.tensor("b"), t["b"])       # stays bf16
    assert f.tensor("c").dtype == torch.float32 and torch.equal(f.tensor("c"), t["c"].float())  # exact widening
    assert f.tensor("d").dtype == torch.int32 and torch.equal(f.tensor("d"), t["d"].int())      # tables are int32
    assert f.tensor("e").dtype == torch.int32
    f.close()
    # the file is readable by the reference reader of the format too
    from safetensors.torch import load_file
    other = load_file(path)
    assert torch.equal(other["b"], t["b"]) and torch.equal(other["a"], t["a"])


def test_bad_files(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(WeightFileError, match="too short"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 10_000) + b"{}")
    with pytest.raises(WeightFileError, match="header length"):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 5) + b"{oops")
    with pytest.raises(WeightFileError, match="JSON"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)             # truncated data
    with pytest.raises(WeightFileError, match="outside"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)            # size does not match shape
    with pytest.raises(WeightFileError, match="needs"):
        SafetensorsFile(str(p))
    with pytest.raises(WeightFileError, match="no model.safetensors"):
        ModelFiles(str(tmp_path / "nowhere"))


def test_headers_the_way_other_writers_make_them(tmp_path):
    """Escapes and non-ASCII names, keys in any order, keys this library does not know, a dtype it does
    not read, metadata that is null or holds other things than strings, a scalar: the header reader takes
    what the format allows and only refuses what it must."""
    p = tmp_path / "odd.safetensors"
    name_json = r'bl\u00f6ck.\"q\"\\0\/\ud83d\ude00'         # as it stands in the header: JSON escapes, a surrogate pair
    hdr = (r'{ "__metadata__": {"k": "v\n", "n": 3, "z": null},' + "\n" + ' "' + name_json + r'": {"data_offsets": [0, 8], '
           r'"extra": [1, {"a": true}], "shape": [2], "dtype": "F32"}, "s": {"dtype": "I64", "shape": [], "data_offsets": [8, 16]}, '
           r'"q": {"dtype": "F8_E4M3", "shape": [3], "data_offsets": [16, 19]} }').encode()
    data = struct.pack("<2f", 1.5, -2.0) + struct.pack("<q", 7) + b"abc"
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + data)
    f = SafetensorsFile(str(p))
    want = json.loads(hdr)                                     # the interpreter's own JSON reader agrees on the names
    want.pop("__metadata__")
    assert set(f.names()) == set(want) and f.metadata == {"k": "v\n"}
    odd = [n for n in f.names() if n.startswith("bl")][0]
    assert odd == 'bl\u00f6ck."q"\\0/\U0001f600'
    assert f.tensor(odd).tolist() == [1.5, -2.0] and f.shape(odd) == (2,)
    assert f.tensor("s").dtype == torch.int32 and f.tensor("s").item() == 7 and f.shape("s") == ()
    assert not f.supported("q") and f.dtype_name("q") == "F8_E4M3"
    with pytest.raises(WeightFileError, match="unsupported dtype"):
        f.tensor("q")
    f.close()
    for bad in (b'[1, 2]', b'{"w": 5}', b'{"w": {"dtype": "F32", "shape": [1.5], "data_offsets": [0, 4]}}',
                b'{"w": {"dtype": "F32", "shape": [1]}}', b'{"w": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}} x',
                b'{"w": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4, 8]}}'):
        p.write_bytes(struct.pack("<Q", len(bad)) + bad + b"\0" * 8)
        with pytest.raises(WeightFileError, match="JSON object|malformed|not valid JSON"):
            SafetensorsFile(str(p))


def test_declared_tensors_follow_the_config():
    cfg, spec = _spec("B")
    d = declared_tensors(spec)
    assert d["model.embed_tokens.weight"].shape == (391, 192)
    assert d["model.layers.2.self_attn.q_proj.weight"].shape == (768, 192)
    assert d["model.layers.2.self_attn.k_proj.weight"].shape == (256, 192)
    assert d["model.layers.0.self_attn.o_proj.weight"].shape == (192, 768)
    assert d["model.layers.0.self_attn.v_proj.bias"].shape == (256,)
    assert d["model.layers.1.mlp.gate_proj.weight"].shape == (328, 192)
    assert d["model.layers.1.mlp.down_proj.weight"].shape == (192, 328)
    assert d["model.layers.1.input_layernorm.weight"].role == "vector"
    assert d["lm_head.weight"].shape == (391, 192) and d["model.norm.weight"].shape == (192,)
    cfg_a, spec_a = _spec("A")
    da = declared_tensors(spec_a)
    assert "lm_head.weight" not in da and "model.layers.0.self_attn.q_proj.bias" not in da


def test_random_mode_writes_a_folder_and_is_deterministic(tmp_path):
    cfg, spec = _spec("A")
    d1 = write_random_model(str(tmp_path / "m1"), cfg, seed=3)
    d2 = write_random_model(str(tmp_path / "m2"), cfg, seed=3)
    d3 = write_random_model(str(tmp_path / "m3"), cfg, seed=4)
    assert sorted(os.listdir(d1)) == ["config.json", "model.safetensors"]
    assert config_from_dict(json.load(open(os.path.join(d1, "config.json")))) == cfg
    t1 = dict(read_model_tensors(d1, declared_tensors(spec)))
    t2 = dict(read_model_tensors(d2, declared_tensors(spec)))
    t3 = dict(read_model_tensors(d3, declared_tensors(spec)))
    assert all(torch.equal(t1[k], t2[k]) for k in t1)
    assert not torch.equal(t1["model.embed_tokens.weight"], t3["model.embed_tokens.weight"])
    assert t1["model.embed_tokens.weight"].dtype == torch.bfloat16            # matrices in bf16
    assert t1["model.norm.weight"].dtype == torch.float32                     # stored in 32-bit, stays so
    assert torch.all(t1["model.norm.weight"] == 1.0)
    w = t1["model.layers.0.mlp.up_proj.weight"].float()
    assert abs(w.std().item() - 0.02) < 0.003 and abs(w.mean().item()) < 0.002
    # tensors are keyed by name, not by creation order
    sub = {k: v for k, v in declared_tensors(spec).items() if "layers.1" in k}
    again = dict(random_tensors(sub, 3))
    assert all(torch.equal(again[k], t1[k]) for k in sub)


def _rewrite(folder, change):
    files = ModelFiles(folder)
    tensors = {n: files.tensor(n) for n in files.names()}
    files.close()
    change(tensors)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)


def test_one_error_lists_everything(tmp_path):
    cfg, spec = _spec("B")
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=0)

    def change(t):
        del t["model.layers.1.mlp.up_proj.weight"]                    # missing
        del t["model.layers.0.self_attn.k_proj.bias"]                 # missing
        t["model.layers.0.rotary.inv_freq"] = torch.zeros(4)          # unexpected
        t["model.layers.2.self_attn.o_proj.weight"] = torch.zeros(5, 5).bfloat16()   # wrong shape
        t["model.norm.weight"] = torch.zeros(192, dtype=torch.int32)  # integer where floats belong
    _rewrite(folder, change)
    with pytest.raises(WeightError) as e:
        list(read_model_tensors(folder, declared_tensors(spec)))
    err = e.value
    assert err.missing == ["model.layers.0.self_attn.k_proj.bias", "model.layers.1.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.0.rotary.inv_freq"]
    assert err.wrong_shape == [("model.layers.2.self_attn.o_proj.weight", (192, 768), (5, 5))]
    assert err.bad_dtype == [("model.norm.weight", "I32")]
    msg = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape", "expected [192, 768], found [5, 5]", "unsupported dtype"):
        assert word in msg


def test_bias_and_tied_head_must_match_the_config(tmp_path):
    cfg, spec = _spec("A")                                   # no biases, tied head
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=0)

    def change(t):
        t["lm_head.weight"] = torch.zeros(264, 128).bfloat16()
        t["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(256)
    _rewrite(folder, change)
    with pytest.raises(WeightError) as e:
        list(read_model_tensors(folder, declared_tensors(spec)))
    assert e.value.unexpected == ["lm_head.weight", "model.layers.0.self_attn.q_proj.bias"]
    # with the architecture's own list of tensors a folder may carry unused, the stored head of a tied
    # model is left unread with a warning; the bias the config rules out stays an error
    assert spec.ignored_tensors == ("lm_head.weight", "*.rotary_emb.inv_freq")
    with pytest.raises(WeightError) as e:
        list(read_model_tensors(folder, declared_tensors(spec), spec.ignored_tensors))
    assert e.value.unexpected == ["model.layers.0.self_attn.q_proj.bias"]


def test_a_folder_may_carry_tensors_the_model_does_not_read(tmp_path):
    """A stored head beside tied embeddings and the rotary frequency tables of old exports: the
    reference takes what it needs by name and leaves the rest (model.rs:157-203)."""
    cfg, spec = _spec("A")
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=0)

    def change(t):
        t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
        t["model.layers.1.self_attn.rotary_emb.inv_freq"] = torch.ones(32)
    _rewrite(folder, change)
    expected = declared_tensors(spec)
    with pytest.warns(UserWarning, match="lm_head.weight.*rotary_emb.inv_freq"):
        got = dict(read_model_tensors(folder, expected, spec.ignored_tensors))
    assert set(got) == set(expected)
    # an untied model must have its head: nothing is ignorable there
    cfg_b, spec_b = _spec("B")
    assert "lm_head.weight" not in spec_b.ignored_tensors


def test_a_file_written_by_the_safetensors_package_loads(tmp_path):
    """The other direction of the round trip: tensors made with torch, stored by the `safetensors`
    package, fetched by name through the library's own reader."""
    from safetensors.torch import save_file
    cfg, spec = _spec("B")
    expected = declared_tensors(spec)
    g = torch.Generator().manual_seed(11)
    tensors = {}
    for i, (name, ts) in enumerate(expected.items()):
        t = torch.randn(ts.shape, generator=g)
        tensors[name] = t.bfloat16() if ts.role == "matrix" and i % 2 else t       # both stored precisions
    folder = tmp_path / "pkg"
    folder.mkdir()
    save_file(tensors, str(folder / "model.safetensors"), metadata={"format": "pt"})
    (folder / "config.json").write_text(json.dumps(cfg.to_dict()))
    got = dict(read_model_tensors(str(folder), expected))
    assert list(got) == list(expected)
    for name, t in tensors.items():
        assert got[name].dtype == t.dtype and torch.equal(got[name], t), name


def test_norm_weights_of_test_models_are_all_different():
    cfg, spec = _spec("B")
    expected = declared_tensors(spec)
    plain = dict(random_tensors(expected, 3, matrix_dtype=torch.float32))
    assert all(torch.equal(t, torch.ones_like(t)) for n, t in plain.items() if n.endswith("norm.weight"))
    varied = dict(random_tensors(expected, 3, matrix_dtype=torch.float32, norm_std=0.2))
    norms = [t for n, t in varied.items() if n.endswith("norm.weight") or n.endswith("layernorm.weight")]
    assert len(norms) == 2 * cfg.num_hidden_layers + 1
    for i, a in enumerate(norms):
        assert (a - 1).abs().mean() > 0.05
        for b in norms[i + 1:]:
            assert not torch.equal(a, b)
    # matrices do not depend on norm_std
    assert torch.equal(plain["model.layers.0.mlp.up_proj.weight"], varied["model.layers.0.mlp.up_proj.weight"])


def test_unsupported_dtype_is_reported(tmp_path):
    cfg, spec = _spec("A")
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=0)
    path = os.path.join(folder, "model.safetensors")
    raw = open(path, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    e = header["model.norm.weight"]
    e["dtype"] = "F8_E4M3"
    e["shape"] = [128 * 4]
    blob = json.dumps(header, separators=(",", ":")).encode()
    open(path, "wb").write(struct.pack("<Q", len(blob)) + blob + raw[8 + hlen:])
    with pytest.raises(WeightError) as ex:
        list(read_model_tensors(folder, declared_tensors(spec)))
    assert ("model.norm.weight", "F8_E4M3") in ex.value.bad_dtype


def test_sharded_folder(tmp_path):
    cfg, spec = _spec("A")
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=1)
    files = ModelFiles(folder)
    tensors = {n: files.tensor(n) for n in files.names()}
    files.close()
    os.remove(os.path.join(folder, "model.safetensors"))
    names = sorted(tensors)
    half = len(names) // 2
    parts = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    weight_map = {}
    for fname, ns in parts.items():
        write_safetensors(os.path.join(folder, fname), {n: tensors[n] for n in ns})
        weight_map.update({n: fname for n in ns})
    json.dump({"weight_map": weight_map}, open(os.path.join(folder, "model.safetensors.index.json"), "w"))
    got = dict(read_model_tensors(folder, declared_tensors(spec)))
    assert all(torch.equal(got[n], tensors[n]) for n in names)


def test_state_dict_takes_the_packing_apart():
    """The model keeps q, k and v in one matrix; `state_dict()` gives every tensor back under the weight
    file's name with the values it was loaded with (8 tensors per layer without biases, 11 with)."""
    from rust_inference_b200.engine.model import DecoderModel
    for name in ("A", "B"):
        cfg, spec = _spec(name)
        model = DecoderModel(spec, dtype=torch.float32, device="cpu")
        src = dict(random_tensors(model.declared_tensors(), 5, matrix_dtype=torch.float32, norm_std=0.2))
        model.load(src.items())
        sd = model.state_dict()
        assert list(sd) == list(src)
        assert all(torch.equal(sd[k], src[k]) for k in src)
        assert ("lm_head.weight" in sd) == (not cfg.tie_word_embeddings)


def test_malformed_files_are_refused_never_read_wrongly(tmp_path):
    """The reader's header parser and its checks meet damaged files: bytes flipped, cut out or added
    in the header, absurd numbers, deep nesting, a header cut short, offsets and shapes that do not fit
    the data, a wrong header length, a body cut short.  Every file is either refused with
    WeightFileError or read completely; a tensor that is read lies inside the file."""
    import random
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, {"a.weight": torch.randn(4, 6), "b": torch.randn(3).bfloat16(),
                             "c": torch.arange(5, dtype=torch.int32)}, metadata={"k": "v"})
    raw = open(path, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    hdr = raw[8:8 + hlen]
    rng = random.Random(0)
    out = str(tmp_path / "m.safetensors")
    loaded = refused = 0
    for _ in range(700):
        h = bytearray(hdr)
        kind = rng.randrange(8)
        if kind == 0:
            for _ in range(rng.randint(1, 4)):
                h[rng.randrange(len(h))] = rng.randrange(256)
        elif kind == 1:
            i = rng.randrange(len(h))
            del h[i:i + rng.randint(1, 10)]
        elif kind == 2:
            i = rng.randrange(len(h))
            h[i:i] = bytes(rng.choice(b'{}[]",:0123456789-eE.\\u ') for _ in range(rng.randint(1, 12)))
        elif kind == 3:
            h = bytearray(hdr.replace(b"24", str(rng.choice([0, -1, 2 ** 31, 2 ** 63, 2 ** 64, 10 ** 30])).encode(), 1))
        elif kind == 4:
            h = bytearray(b"[" * rng.randint(1, 5000))
        elif kind == 5:
            h = bytearray(b'{"a":' * rng.randint(1, 3000))
        elif kind == 6:
            h = bytearray(hdr[:rng.randrange(len(hdr))])
        else:
            j = json.loads(hdr)
            k = rng.choice([k for k in j if k != "__metadata__"])
            j[k]["data_offsets"] = [rng.randrange(-5, 200), rng.randrange(-5, 200)]
            j[k]["shape"] = [rng.randrange(-2, 10) for _ in range(rng.randint(0, 4))]
            h = bytearray(json.dumps(j).encode())
        claimed = len(h) if rng.random() < 0.8 else rng.choice([0, 1, len(h) - 1, len(h) + 1, 2 ** 40, 2 ** 63])
        body = raw[8 + hlen:] if rng.random() < 0.8 else raw[8 + hlen:][:rng.randrange(60)]
        with open(out, "wb") as f:
            f.write(struct.pack("<Q", claimed & (2 ** 64 - 1)) + bytes(h) + body)
        try:
            f = SafetensorsFile(out)
        except WeightFileError:
            refused += 1
            continue
        try:
            for n in f.names():
                t = f.tensor(n)                                        # a dtype the library does not read is refused here
                assert t.numel() * t.element_size() <= 2 * len(body) + 8      # what was read lies inside the file (F16 widens)
            loaded += 1
        except WeightFileError:
            refused += 1
        f.close()
    assert refused > 400 and loaded > 20
