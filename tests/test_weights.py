"""The safetensors reader/writer, the loader's single error, and the random-weights mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

from conftest import TINY_A, TINY_B
from nanoinfer_b200 import load_model
from nanoinfer_b200.config import GPT2Config
from nanoinfer_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, write_random_model,
                                    write_safetensors)


def _folder(tmp_path, raw, dtype=torch.float32, seed=3):
    d = str(tmp_path / "m")
    write_random_model(GPT2Config.from_dict(raw), d, seed, dtype)
    return d


def _rewrite(d, fn):
    path = os.path.join(d, "model.safetensors")
    st = SafetensorsFile(path)
    tensors = {n: st.tensor(n) for n in st.names()}
    st.close()
    tensors = fn(tensors)
    write_safetensors(path, tensors)


def test_roundtrip_dtypes(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32),
         "d": torch.randn(2, 2).to(torch.float16)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, metadata={"k": "v"})
    st = SafetensorsFile(p)
    assert sorted(st.names()) == ["a", "b", "c", "d"]
    for k, v in t.items():
        got = st.tensor(k)
        assert got.dtype == v.dtype and torch.equal(got, v)
    # the same bytes are read by the reference library
    from safetensors.torch import load_file
    other = load_file(p)
    assert all(torch.equal(other[k], v) for k, v in t.items())


@pytest.mark.parametrize("blob, word", [
    (b"abc", "too small"),
    (struct.pack("<Q", 1000) + b"{}", "truncated"),
    (struct.pack("<Q", 2) + b"[]", "not an object"),
    (struct.pack("<Q", 9) + b'{"a":{} }', "missing dtype"),
])
def test_format_errors(tmp_path, blob, word):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(blob)
    with pytest.raises(SafetensorsError) as e:
        SafetensorsFile(str(p))
    assert word in str(e.value)


def test_out_of_bounds_and_length(tmp_path):
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p = tmp_path / "short.safetensors"
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="out of bounds"):
        SafetensorsFile(str(p))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 16)
    with pytest.raises(SafetensorsError, match="byte length"):
        SafetensorsFile(str(p))


def test_random_folder_loads_and_keeps_the_layout(tmp_path):
    d = _folder(tmp_path, TINY_B)
    st = SafetensorsFile(os.path.join(d, "model.safetensors"))
    # Conv1D tensors are stored [in, out]; the untied head [vocab, width]
    assert st.info("h.0.attn.c_attn.weight").shape == (120, 360)
    assert st.info("h.2.mlp.c_proj.weight").shape == (200, 120)
    assert st.info("lm_head.weight").shape == (1000, 120)
    stored = st.tensor("h.1.mlp.c_fc.weight")
    gamma = st.tensor("ln_f.weight")
    st.close()
    m = load_model(d, "float32", "cpu")
    w = m.layers[1].feed_forward.params["fc_weight"]
    assert w.shape == (200, 120) and torch.equal(w, stored.t())       # transposed once, at load
    assert abs(float(gamma.mean()) - 1.0) < 0.02                         # norm scales are 1 + N(0, 0.02)
    assert m.head.params["weight"] is not m.embedding.params["table"]


def test_same_seed_same_bytes_other_seed_other_bytes(tmp_path):
    a = _folder(tmp_path / "a", TINY_A, seed=5)
    b = _folder(tmp_path / "b", TINY_A, seed=5)
    c = _folder(tmp_path / "c", TINY_A, seed=6)
    ra = open(os.path.join(a, "model.safetensors"), "rb").read()
    assert ra == open(os.path.join(b, "model.safetensors"), "rb").read()
    assert ra != open(os.path.join(c, "model.safetensors"), "rb").read()


def test_dtype_policy(tmp_path):
    d = _folder(tmp_path, TINY_A, dtype=torch.bfloat16)
    m16 = load_model(d, "bfloat16", "cpu")
    m32 = load_model(d, "float32", "cpu")
    att16, att32 = m16.layers[0].mixer.params, m32.layers[0].mixer.params
    assert att16["qkv_weight"].dtype == torch.bfloat16 and att32["qkv_weight"].dtype == torch.float32
    assert att16["qkv_bias"].dtype == torch.float32              # vectors are always 32-bit
    assert m16.final_norm.params["weight"].dtype == torch.float32
    assert torch.equal(att16["qkv_weight"].float(), att32["qkv_weight"])   # bf16 -> fp32 is exact
    assert m16.head.params["weight"] is m16.embedding.params["table"]      # tied: one tensor on the device


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = _folder(tmp_path, TINY_A)

    def damage(t):
        del t["h.1.ln_2.bias"]
        del t["wpe.weight"]
        t["h.0.mlp.c_fc.weight"] = t["h.0.mlp.c_fc.weight"].t().contiguous()   # [out, in] instead of [in, out]
        t["ln_f.weight"] = torch.zeros(65)
        t["h.0.attn.rotary.inv_freq"] = torch.zeros(8)
        t["extra.weight"] = torch.zeros(2, 2)
        t["h.0.attn.bias"] = torch.ones(1, 1, 128, 128)      # the causal-mask buffer some checkpoints carry
        return t

    _rewrite(d, damage)
    with pytest.raises(WeightError) as e:
        load_model(d, "float32", "cpu")
    err = e.value
    assert err.missing == ["h.1.ln_2.bias", "wpe.weight"]
    assert err.unexpected == ["extra.weight", "h.0.attn.rotary.inv_freq"]
    assert len(err.wrong) == 2 and "h.0.mlp.c_fc.weight" in err.wrong[0] + err.wrong[1]
    msg = str(err)
    for name in ("h.1.ln_2.bias", "wpe.weight", "extra.weight", "expected shape [64, 256], got [256, 64]", "ln_f.weight"):
        assert name in msg
    assert "h.0.attn.bias" not in msg


def test_transformer_prefix_and_integer_for_float(tmp_path):
    d = _folder(tmp_path, TINY_A)
    _rewrite(d, lambda t: {"transformer." + k: v for k, v in t.items()})
    load_model(d, "float32", "cpu")

    def as_int(t):
        t["transformer.ln_f.bias"] = torch.zeros(64, dtype=torch.int32)
        return t

    _rewrite(d, as_int)
    with pytest.raises(WeightError, match="floating-point"):
        load_model(d, "float32", "cpu")


def test_missing_files(tmp_path):
    with pytest.raises(Exception, match="config.json"):
        load_model(str(tmp_path), "float32", "cpu")
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    with pytest.raises(FileNotFoundError, match="model.safetensors"):
        load_model(str(tmp_path), "float32", "cpu")


@pytest.mark.gpu
@pytest.mark.parametrize("stored", [torch.float32, torch.bfloat16, torch.float16])
def test_streamed_load_on_the_device_gives_the_host_path_s_tensors(tmp_path, stored, monkeypatch):
    """On a CUDA device the file's bytes go through pinned staging buffers and a kernel converts and
    transposes them in place.  Every bound tensor must be bit-for-bit what the host path makes (file
    in 32-bit, bfloat16 or 16-bit floats; engine in either dtype), also when the staging buffers are
    so small that every matrix goes over in many pieces."""
    from nanoinfer_b200.weights import loader, random_tensors, write_safetensors
    from nanoinfer_b200.models.model import Model
    from nanoinfer_b200.registry import get_architecture
    cfg = GPT2Config.from_dict(TINY_B)
    model = Model(get_architecture(cfg.architecture).build_spec(cfg), cfg)
    tensors = {k: v.to(stored) for k, v in random_tensors(model, 5, 0.05, torch.float32).items()}
    d = str(tmp_path)
    with open(os.path.join(d, "config.json"), "w") as fh:
        json.dump(cfg.to_dict(), fh)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    for engine_dtype in (torch.float32, torch.bfloat16):
        host = load_model(d, engine_dtype, "cpu")
        for staging in (loader.STAGING_BYTES, 4096):
            monkeypatch.setattr(loader, "STAGING_BYTES", staging)
            dev = load_model(d, engine_dtype, "cuda")
            for a, b in zip(host.bindings(), dev.bindings()):
                ta, tb = a.part.params[a.spec.key], b.part.params[b.spec.key]
                assert tb.is_cuda and ta.dtype == tb.dtype and ta.shape == tb.shape, b.where
                assert torch.equal(ta, tb.cpu()), f"{b.where}.{b.spec.key}"
