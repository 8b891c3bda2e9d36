"""Weights: the file format, the one error that lists every fault, random-weights mode (no GPU)."""
import json
import os

import pytest
import torch

import util
from lmsf_b200 import models  # noqa: F401
from lmsf_b200.config import LlamaConfig
from lmsf_b200.models.llama import llama_spec
from lmsf_b200.parts.decoder import DecoderModel
from lmsf_b200.weights import (SafetensorsError, WeightError, check_tensors, open_model_tensors, write_random_model,
                               write_safetensors)
from lmsf_b200.weights.loader import target_dtype


def _model(cfg):
    return DecoderModel(llama_spec(LlamaConfig.from_dict(cfg)))


def _rewrite(folder, out, edit):
    ents = open_model_tensors(folder)
    tensors = {n: e.load().clone() for n, e in ents.items()}
    edit(tensors)
    os.makedirs(out, exist_ok=True)
    write_safetensors(os.path.join(out, "model.safetensors"), [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()],
                      lambda n: tensors[n])
    return out


def test_random_model_folder_is_complete_and_deterministic(tmp_path):
    a = write_random_model(str(tmp_path / "a"), dict(util.TINY_A), seed=5, dtype="bfloat16")
    b = write_random_model(str(tmp_path / "b"), dict(util.TINY_A), seed=5, dtype="bfloat16")
    c = write_random_model(str(tmp_path / "c"), dict(util.TINY_A), seed=6, dtype="bfloat16")
    ea, eb, ec = open_model_tensors(a), open_model_tensors(b), open_model_tensors(c)
    assert json.load(open(os.path.join(a, "config.json")))["intermediate_size"] == 172
    assert set(ea) == set(eb) and len(ea) == 2 * 9 + 3
    check_tensors(_model(util.TINY_A), ea)
    for n in ea:
        assert ea[n].dtype == torch.bfloat16
        assert torch.equal(ea[n].load(), eb[n].load())
    assert not torch.equal(ea["lm_head.weight"].load(), ec["lm_head.weight"].load())
    assert torch.all(ea["model.norm.weight"].load() == 1)
    w = ea["model.layers.1.mlp.down_proj.weight"].load().float()
    assert tuple(w.shape) == (64, 172) and abs(w.std().item() - 0.02) < 0.002
    # tied embeddings: no lm_head in the file
    t = write_random_model(str(tmp_path / "t"), dict(util.TINY_B), seed=1, dtype="float32")
    assert "lm_head.weight" not in open_model_tensors(t)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    src = util.model_folder("A", "float32")

    def edit(t):
        del t["model.layers.0.self_attn.k_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.1.mlp.up_proj.weight"] = torch.zeros(171, 64)
        t["lm_head.weight"] = torch.zeros(64, 256)
        t["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(16)
        t["extra.bias"] = torch.zeros(3)
    bad = _rewrite(src, str(tmp_path / "bad"), edit)
    with pytest.raises(WeightError) as e:
        check_tensors(_model(util.TINY_A), open_model_tensors(bad), bad)
    err = e.value
    assert set(err.missing) == {"model.layers.0.self_attn.k_proj.weight", "model.norm.weight"}
    assert set(err.unexpected) == {"model.layers.0.self_attn.q_norm.weight", "extra.bias"}
    assert {n for n, _, _ in err.wrong_shape} == {"model.layers.1.mlp.up_proj.weight", "lm_head.weight"}
    msg = str(err)
    for needle in ("k_proj", "model.norm.weight", "q_norm", "extra.bias", "(172, 64)", "(171, 64)", "(256, 64)"):
        assert needle in msg


def test_ignored_and_tied_names(tmp_path):
    src = util.model_folder("B", "float32")

    def edit(t):
        t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
        t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    ok = _rewrite(src, str(tmp_path / "ok"), edit)
    check_tensors(_model(util.TINY_B), open_model_tensors(ok))


def test_dtype_rule():
    bf, f32 = torch.bfloat16, torch.float32
    assert target_dtype(bf, bf, False) == bf and target_dtype(f32, bf, False) == bf      # matrices: run dtype
    assert target_dtype(f32, bf, True) == f32 and target_dtype(bf, bf, True) == bf        # a 32-bit vector stays
    assert target_dtype(bf, f32, False) == f32 and target_dtype(torch.float16, bf, False) == bf
    assert target_dtype(torch.int64, bf, False) == torch.int32                             # integer tables


def test_broken_files(tmp_path):
    d = tmp_path / "m"
    d.mkdir()
    with pytest.raises(SafetensorsError):
        open_model_tensors(str(d))
    (d / "model.safetensors").write_bytes(b"\x05\x00\x00")
    with pytest.raises(SafetensorsError):
        open_model_tensors(str(d))
    (d / "model.safetensors").write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(SafetensorsError):
        open_model_tensors(str(d))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    (d / "model.safetensors").write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError):
        open_model_tensors(str(d))


def test_sharded_folder(tmp_path):
    src = util.model_folder("A", "float32")
    ents = open_model_tensors(src)
    names = sorted(ents)
    half = len(names) // 2
    wm = {}
    for shard, part in (("model-00001-of-00002.safetensors", names[:half]), ("model-00002-of-00002.safetensors", names[half:])):
        write_safetensors(str(tmp_path / shard), [(n, ents[n].dtype, ents[n].shape) for n in part], lambda n: ents[n].load())
        wm.update({n: shard for n in part})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    got = open_model_tensors(str(tmp_path))
    assert set(got) == set(ents)
    assert torch.equal(got[names[-1]].load(), ents[names[-1]].load())
