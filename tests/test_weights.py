"""Safetensors container, weight binding errors, random-weights folders (no GPU)."""
import json
import struct

import pytest
import torch

from conftest import TINY, TINY_A, TINY_B
from lucciola_b200.config import resolve_architecture
from lucciola_b200.parts import Runtime
from lucciola_b200.weights import (CheckpointFolder, SafetensorsError, SafetensorsFile, WeightError, bind_weights,
                                   check_weights, write_random_model, write_safetensors)
from lucciola_b200.weights.loader import engine_dtype_of


def _model(cfg, dtype=torch.float32):
    arch = resolve_architecture(cfg)
    return arch.build(arch.config_from_dict(cfg), Runtime("cpu", dtype))


def test_container_round_trip(tmp_path):
    ts = {"a": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int32), "c": torch.randn(2, 2), "e": torch.zeros(0, 4)}
    write_safetensors(tmp_path / "m.safetensors", ts, {"k": "v"})
    with SafetensorsFile(tmp_path / "m.safetensors") as f:
        assert f.metadata == {"k": "v"} and set(f.names()) == set(ts)
        for k, v in ts.items():
            assert torch.equal(f.get(k), v) and f.get(k).dtype == v.dtype


def _raw(tmp_path, header: dict, data: bytes = b"", name="x.safetensors"):
    blob = json.dumps(header).encode()
    p = tmp_path / name
    p.write_bytes(struct.pack("<Q", len(blob)) + blob + data)
    return p


def test_container_corruption(tmp_path):
    p = tmp_path / "short.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 10 ** 9) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 4) + b"{{{{")
    with pytest.raises(SafetensorsError, match="not valid JSON"):
        SafetensorsFile(p)
    with pytest.raises(SafetensorsError, match="outside the file"):
        SafetensorsFile(_raw(tmp_path, {"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8))
    with pytest.raises(SafetensorsError, match="needs 16 bytes, has 8"):
        SafetensorsFile(_raw(tmp_path, {"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}, b"\0" * 8))
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(_raw(tmp_path, {"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}, b"\0" * 4))
    with pytest.raises(SafetensorsError, match="malformed"):
        SafetensorsFile(_raw(tmp_path, {"w": {"dtype": "F32"}}, b""))


def test_random_folder_fits_its_model(tmp_path):
    for name, (cfg, seed, std, nstd, _) in TINY.items():
        folder = write_random_model(cfg, tmp_path / name, seed, std=std, norm_std=nstd)
        assert (folder / "config.json").is_file() and (folder / "model.safetensors").is_file()
        src = CheckpointFolder(folder)
        model = _model(cfg)
        check_weights(model.all_param_specs(), src, model.ignored_names())
        names = set(src.names())
        assert ("lm_head.weight" in names) == (not cfg["tie_word_embeddings"])
        w = src.get("model.layers.0.self_attn.q_proj.weight")
        assert w.dtype == torch.bfloat16 and abs(w.float().std().item() - std) < 0.2 * std
        n = src.get("model.layers.0.input_layernorm.weight").float()
        assert abs(n.mean().item() - 1.0) < 4 * nstd / n.numel() ** 0.5 + 0.02
        src.close()


def test_same_seed_same_weights_other_seed_other_weights(tmp_path):
    a = write_random_model(TINY_A, tmp_path / "a", 0)
    b = write_random_model(TINY_A, tmp_path / "b", 0)
    c = write_random_model(TINY_A, tmp_path / "c", 1)
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert (a / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = write_random_model(TINY_B, tmp_path / "m", 1)
    src = CheckpointFolder(folder)
    tensors = {n: src.get(n) for n in src.names()}
    src.close()
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(256)
    tensors["model.layers.2.self_attn.k_norm.weight"] = torch.ones(16).bfloat16()
    tensors["model.embed_tokens.weight"] = tensors["model.embed_tokens.weight"][:, :64].contiguous()
    write_safetensors(folder / "model.safetensors", tensors)
    src = CheckpointFolder(folder)
    with pytest.raises(WeightError) as ei:
        bind_weights(_model(TINY_B), src, torch.float32, "cpu")
    msg = str(ei.value)
    assert "missing tensors (2): model.layers.1.mlp.up_proj.weight, model.norm.weight" in msg
    assert "unexpected tensors (1): model.layers.0.self_attn.q_proj.bias" in msg
    assert "model.layers.2.self_attn.k_norm.weight: expected [32], found [16]" in msg
    assert "model.embed_tokens.weight: expected [503, 96], found [503, 64]" in msg


def test_untied_model_without_head_and_tied_model_with_head(tmp_path):
    folder = write_random_model(TINY_B, tmp_path / "b", 1)
    src = CheckpointFolder(folder)
    tensors = {n: src.get(n) for n in src.names() if n != "lm_head.weight"}
    src.close()
    write_safetensors(folder / "model.safetensors", tensors)
    with pytest.raises(WeightError, match="missing tensors \\(1\\): lm_head.weight"):
        bind_weights(_model(TINY_B), CheckpointFolder(folder), torch.float32, "cpu")
    # A tied model tolerates a head tensor in the file and uses the embedding table.
    folder = write_random_model(TINY_A, tmp_path / "a", 0)
    src = CheckpointFolder(folder)
    tensors = {n: src.get(n) for n in src.names()}
    src.close()
    tensors["lm_head.weight"] = torch.zeros(256, 64).bfloat16()
    write_safetensors(folder / "model.safetensors", tensors)
    m = _model(TINY_A)
    bind_weights(m, CheckpointFolder(folder), torch.float32, "cpu")
    assert m.head.proj.weight is m.embedding.weight


def test_several_files_and_duplicates(tmp_path):
    folder = write_random_model(TINY_A, tmp_path / "a", 0)
    src = CheckpointFolder(folder)
    tensors = {n: src.get(n) for n in src.names()}
    src.close()
    (folder / "model.safetensors").unlink()
    names = sorted(tensors)
    write_safetensors(folder / "model-00001-of-00002.safetensors", {n: tensors[n] for n in names[:5]})
    write_safetensors(folder / "model-00002-of-00002.safetensors", {n: tensors[n] for n in names[5:]})
    bind_weights(_model(TINY_A), CheckpointFolder(folder), torch.float32, "cpu")
    write_safetensors(folder / "model-00003.safetensors", {names[0]: tensors[names[0]]})
    with pytest.raises(WeightError, match="is in both"):
        CheckpointFolder(folder)
    with pytest.raises(WeightError, match="no \\*.safetensors"):
        CheckpointFolder(tmp_path)


def test_types_kept(tmp_path):
    bf, f32, i64 = torch.zeros(2).bfloat16(), torch.zeros(2), torch.zeros(2, dtype=torch.int64)
    assert engine_dtype_of(bf, torch.bfloat16) == torch.bfloat16
    assert engine_dtype_of(f32, torch.bfloat16) == torch.float32          # stored in 32-bit: stays so
    assert engine_dtype_of(torch.zeros(2).half(), torch.bfloat16) == torch.bfloat16
    assert engine_dtype_of(i64, torch.bfloat16) == torch.int32
    assert engine_dtype_of(bf, torch.float32) == torch.float32
    folder = write_random_model(TINY_A, tmp_path / "a", 0)
    m = _model(TINY_A, torch.bfloat16)
    bind_weights(m, CheckpointFolder(folder), torch.bfloat16, "cpu")
    assert m.blocks[0].mixer.qkv.weight.dtype == torch.bfloat16
    assert m.blocks[0].mixer.qkv.weight.shape == (64 + 2 * 32, 64)
    assert m.blocks[0].mixer_norm.weight.dtype == torch.float32        # norm weights are read as float32 (exact)


def test_random_model_program_writes_a_loadable_folder(tmp_path):
    """bin/lucciola_random_model: config.json + seed -> a folder the loader accepts; same seed, same bytes."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    from conftest import TINY
    cfg = TINY["B"][0]
    (tmp_path / "c.json").write_text(json.dumps(cfg))
    prog = Path(__file__).resolve().parents[1] / "bin" / "lucciola_random_model"
    for out in ("m1", "m2"):
        r = subprocess.run([sys.executable, str(prog), "--config", str(tmp_path / "c.json"), "--seed", "4", "--out", str(tmp_path / out),
                            "--std", "0.05", "--norm-std", "0.1"], capture_output=True, text=True, timeout=120)
        assert r.returncode == 0, r.stderr
    a, b = (tmp_path / "m1" / "model.safetensors").read_bytes(), (tmp_path / "m2" / "model.safetensors").read_bytes()
    assert a == b and json.loads((tmp_path / "m1" / "config.json").read_text()) == cfg
    from lucciola_b200.weights.loader import CheckpointFolder
    folder = CheckpointFolder(tmp_path / "m1")
    assert "model.embed_tokens.weight" in folder.names()


def test_ranges_of_a_tensors_bytes_can_be_read_from_the_file(tmp_path):
    """What the loader's pinned buffers are filled with: any range of a tensor's bytes, and nothing outside it."""
    from lucciola_b200.weights.safetensors_io import SafetensorsError, SafetensorsFile, write_safetensors
    t = torch.randn(301, 37)
    write_safetensors(tmp_path / "a.safetensors", {"first": torch.arange(7, dtype=torch.int32), "x": t, "last": torch.ones(3)})
    raw = t.view(torch.uint8).reshape(-1)
    with SafetensorsFile(tmp_path / "a.safetensors") as f:
        for start, n in ((0, raw.numel()), (5, 1), (1000, 4096), (raw.numel() - 3, 3), (17, 0)):
            buf = torch.full((n + 8,), 255, dtype=torch.uint8)
            f.read_into("x", buf, start, n)
            assert torch.equal(buf[:n], raw[start:start + n]) and bool((buf[n:] == 255).all())
        with pytest.raises(SafetensorsError):
            f.read_into("x", torch.empty(64, dtype=torch.uint8), raw.numel() - 10, 11)
        with pytest.raises(SafetensorsError):
            f.read_into("x", torch.empty(4, dtype=torch.uint8), 0, 5)
