"""Host-side parts of the Zaverax family that need no GPU: configuration reading and run order, the architecture registry,
the flat-tensor loader's strictness, the trace replay's dtype refusal, and the oracle's own consistency."""
import json
import os
import struct
import subprocess
import sys

import pytest
import torch

from evo_b200.models import ARCHITECTURES, load_model_dir, read_architecture
from evo_b200.zaverax import Zaverax, ZaveraxConfig
from oracle import zaverax_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _write_checkpoint(folder, cfg, tensors):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        raw = t.contiguous().reshape(-1).view(torch.uint8).numpy().tobytes()          # reshape: 0-dim tensors too
        header[name] = {"dtype": {torch.bfloat16: "BF16", torch.float32: "F32"}[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header).encode()
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + b"".join(blobs))


def test_run_order_follows_the_loop():
    cfg = ZaveraxConfig.from_dict(O.make_config(layers=("hgrn2", "attention", "hgrn2", "attention"), loop=(1, 3, 3)))
    assert [(r.layer, r.inject) for r in cfg.runs] == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert [(r.layer, r.inject) for r in cfg.runs] == O.run_order(4, 1, 3, 3)
    once = ZaveraxConfig.from_dict(O.make_config(layers=("hgrn2", "attention"), loop=(0, 2, 1)))
    assert [(r.layer, r.inject) for r in once.runs] == [(0, False), (1, False)]
    none = O.make_config(layers=("attention",))
    del none["loop"]
    assert [(r.layer, r.inject) for r in ZaveraxConfig.from_dict(none).runs] == [(0, False)]
    with pytest.raises(ValueError):
        ZaveraxConfig.from_dict(O.make_config(layers=("hgrn2",), loop=(0, 2, 2)))


def test_config_reads_every_size_and_constant():
    d = O.make_config(width=104, vocab=77, heads=6, kv_heads=2, dim=10, vdim=14, r_heads=5, r_dim=6, r_vdim=22, ff=50, window=13, keep_first=2,
                      diff=0.25, taps=4, residual_mult=0.7, softcap=9.0, eps=3e-6, no_ff_layers=(0,))
    c = ZaveraxConfig.from_dict(d)
    a, r = c.layers[1].mixer, c.layers[0].mixer
    assert (c.width, c.vocab_size, c.taps, c.residual_mult, c.logit_softcap, c.eps) == (104, 77, 4, 0.7, 9.0, 3e-6)
    assert (a.kind, a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.keep_first, a.diff) == ("attention", 6, 2, 10, 14, 13, 2, 0.25)
    assert (r.kind, r.heads, r.dim, r.vdim) == ("hgrn2", 5, 6, 22)
    assert c.layers[0].ff is None and c.layers[1].ff == 50
    shapes = c.tensor_shapes()
    assert shapes["l1.mix.q"] == (6 * 2 * 10, 104) and shapes["l1.mix.k"] == (2 * 2 * 10, 104) and shapes["l0.mix.f.b"] == (30,)
    assert "l0.norm2" not in shapes and "l0.mlp.up" not in shapes and shapes["l1.canon1"] == (104, 4)
    assert sorted(shapes) == sorted(O.random_weights(d))
    with pytest.raises(NotImplementedError):
        bad = O.make_config()
        bad["layers"][0]["type"] = "mamba"
        ZaveraxConfig.from_dict(bad)


def test_registry_picks_the_class_and_the_loader_is_strict(tmp_path):
    cfg = O.make_config()
    W = O.random_weights(cfg, seed=1)
    _write_checkpoint(tmp_path / "ok", cfg, W)
    arch, read = read_architecture(str(tmp_path / "ok"))
    assert arch == "Zaverax" and read["width"] == cfg["width"] and torch.float32 in ARCHITECTURES[arch][1]
    model = load_model_dir(str(tmp_path / "ok"))
    assert isinstance(model, Zaverax) and model.ingest_stats["tensors"] == len(W)
    assert all(torch.equal(model.weights[k], W[k]) for k in W)
    missing = dict(W)
    missing.pop("l0.mix.lower")
    _write_checkpoint(tmp_path / "missing", cfg, missing)
    with pytest.raises(RuntimeError, match="Missing"):
        load_model_dir(str(tmp_path / "missing"))
    _write_checkpoint(tmp_path / "shape", cfg, dict(W, head=W["head"][:-1]))
    with pytest.raises(RuntimeError, match="size mismatch"):
        load_model_dir(str(tmp_path / "shape"))
    _write_checkpoint(tmp_path / "other", dict(cfg, architecture="Nonesuch"), W)
    with pytest.raises(ValueError, match="Nonesuch"):
        load_model_dir(str(tmp_path / "other"))
    with pytest.raises(NotImplementedError):
        load_model_dir(str(tmp_path / "ok"), dtype=torch.float16)


def test_model_refuses_to_run_without_cuda(tmp_path):
    from evo_b200 import _lib
    cfg = O.make_config()
    m = Zaverax(ZaveraxConfig.from_dict(cfg))
    m.load_state_dict(O.random_weights(cfg))
    with pytest.raises(RuntimeError):
        m.load_state_dict({"embed": torch.zeros(2, 2)})
    with pytest.raises(_lib.EvoError, match="no CPU"):
        m(torch.zeros(1, 4, dtype=torch.long))


def test_trace_replay_refuses_a_dtype_the_model_class_lacks(tmp_path):
    folder = tmp_path / "sh"
    os.makedirs(folder)
    with open(folder / "config.json", "w") as f:
        json.dump({"architecture": "StripedHyena"}, f)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(tmp_path / "o")],
                       input="", capture_output=True, text=True, timeout=300)
    assert r.returncode == 3, r.stderr


def test_oracle_recurrence_carries_its_state_and_masks_by_distance():
    g = torch.Generator().manual_seed(0)
    H, dk, dv, T = 2, 5, 7, 12
    q, f, v = (torch.randn(T, H * n, generator=g, dtype=torch.float64) for n in (dk, dk, dv))
    fb, lo, nw = torch.randn(H * dk, generator=g).double(), torch.rand(H * dk, generator=g).double(), torch.ones(dv).double()
    whole, _ = O.hgrn2(q, f, v, fb, lo, nw, H, dk, dv, 1e-5)
    a, s = O.hgrn2(q[:5], f[:5], v[:5], fb, lo, nw, H, dk, dv, 1e-5)
    b, _ = O.hgrn2(q[5:], f[5:], v[5:], fb, lo, nw, H, dk, dv, 1e-5, state=s)
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-12)
    assert O.visible(10, 4, 7, 0) and not O.visible(10, 3, 7, 0) and O.visible(10, 3, 7, 4) and not O.visible(3, 4, 7, 9) and O.visible(50, 0, 0, 0)
    h = torch.randn(6, 3, generator=g, dtype=torch.float64)
    c = torch.randn(3, 2, generator=g, dtype=torch.float64)
    out = O.conv_skip(h, c)
    assert torch.allclose(out[0], h[0] * (1 + c[:, 1])) and torch.allclose(out[3], h[3] * (1 + c[:, 1]) + c[:, 0] * h[2])
