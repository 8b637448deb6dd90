"""Host-side parts of the Movalorn family that need no GPU: configuration reading and run order, the architecture registry,
the flat-tensor loader's strictness (scalar tensors included), and the oracle's own consistency."""
import math

import pytest
import torch

from evo_b200.models import ARCHITECTURES, load_model_dir, read_architecture
from evo_b200.movalorn import Movalorn, MovalornConfig
from evo_b200.stream_model import StreamDecoder
from oracle import movalorn_oracle as O
from tests.test_zaverax_host import _write_checkpoint


def test_run_order_follows_the_loop():
    cfg = MovalornConfig.from_dict(O.make_config(layers=("mingru", "latent_attention", "mingru", "latent_attention"), loop=(1, 3, 3)))
    got = [(r.layer, r.loop_pass, r.first) for r in cfg.runs]
    assert got == [(0, None, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False), (1, 2, True), (2, 2, False), (3, None, False)]
    assert got == O.run_order(4, 1, 3, 3)
    once = MovalornConfig.from_dict(O.make_config(layers=("mingru", "latent_attention"), loop=(0, 2, 1)))
    assert [(r.layer, r.loop_pass, r.first) for r in once.runs] == [(0, 0, True), (1, 0, False)] and once.looped
    none = MovalornConfig.from_dict(O.make_config(layers=("latent_attention",)))
    assert [(r.layer, r.loop_pass, r.first) for r in none.runs] == [(0, None, False)] and not none.looped
    assert "loop.in" not in none.tensor_shapes() and once.tensor_shapes()["loop.step"] == (1, once.width)
    with pytest.raises(ValueError):
        MovalornConfig.from_dict(O.make_config(layers=("mingru",), loop=(0, 2, 2)))


def test_config_reads_every_size_and_constant():
    d = O.make_config(width=104, vocab=77, layers=("latent_attention", "mingru", "mingru"), heads=6, dim=10, rot_dim=6, vdim=14, kv_rank=22, window=13,
                      rot_base=777.0, att_scale=0.31, gru_width=50, ff=58, moe_layers=(1,), experts=7, top=3, expert_ff=18, shared_ff=26, router_scale=2.5,
                      no_ff_layers=(2,), buckets=91, mul_prev=11, mul_cur=13, embed_scale=4.5, logit_scale=0.25, eps=3e-6)
    c = MovalornConfig.from_dict(d)
    a, r, f = c.layers[0].mixer, c.layers[1].mixer, c.layers[1].mlp
    assert (c.width, c.vocab_size, c.eps, c.embed_scale, c.buckets, c.mul_prev, c.mul_cur, c.logit_scale) == (104, 77, 3e-6, 4.5, 91, 11, 13, 0.25)
    assert (a.kind, a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank, a.window, a.rot_base, a.rot_dims, a.scale) == ("latent_attention", 6, 10, 6, 14, 22, 13, 777.0, 6, 0.31)
    assert (r.kind, r.width) == ("mingru", 50)
    assert (f.kind, f.ff, f.experts, f.top, f.router_scale, f.shared_ff) == ("moe", 18, 7, 3, 2.5, 26)
    assert c.layers[0].mlp.kind == "dense" and c.layers[0].mlp.ff == 58 and c.layers[2].mlp is None
    shapes = c.tensor_shapes()
    assert shapes["l0.mix.q"] == (6 * 16, 104) and shapes["l0.mix.dkv"] == (28, 104) and shapes["l0.mix.uv"] == (84, 22) and shapes["l0.mix.g"] == (6, 104)
    assert shapes["bigram"] == (92, 104) and shapes["l1.mlp.e6.down"] == (104, 18) and shapes["l1.mlp.shared.up"] == (26, 104) and shapes["l0.norm1b"] == ()
    assert "l2.norm2" not in shapes and "l2.rg2" not in shapes and "l1.mlp.e7.gate" not in shapes
    assert shapes == O.tensor_shapes(d)
    no_shared = O.make_config(layers=("mingru",), moe_layers=(0,), shared_ff=0)
    assert "l0.mlp.shared.gate" not in MovalornConfig.from_dict(no_shared).tensor_shapes()
    for breakage in ("type", "kind"):
        bad = O.make_config()
        if breakage == "type":
            bad["layers"][0]["type"] = "mamba"
        else:
            bad["layers"][0]["mlp"]["kind"] = "sparse"
        with pytest.raises(NotImplementedError):
            MovalornConfig.from_dict(bad)


def test_registry_picks_the_class_and_the_loader_is_strict(tmp_path):
    cfg = O.make_config(moe_layers=(1,), loop=(0, 2, 2))
    W = O.random_weights(cfg, seed=1)
    _write_checkpoint(tmp_path / "ok", cfg, W)
    arch, read = read_architecture(str(tmp_path / "ok"))
    assert arch == "Movalorn" and read["width"] == cfg["width"] and torch.float32 in ARCHITECTURES[arch][1]
    model = load_model_dir(str(tmp_path / "ok"))
    assert isinstance(model, Movalorn) and isinstance(model, StreamDecoder) and model.ingest_stats["tensors"] == len(W)
    assert all(torch.equal(model.weights[k], W[k]) for k in W)
    assert model.weights["l0.norm1"].shape == () and model.weights["final.norm"].dtype == torch.bfloat16
    missing = dict(W)
    missing.pop("l1.mlp.correction")
    _write_checkpoint(tmp_path / "missing", cfg, missing)
    with pytest.raises(RuntimeError, match="Missing"):
        load_model_dir(str(tmp_path / "missing"))
    _write_checkpoint(tmp_path / "shape", cfg, dict(W, bigram=W["bigram"][:-1]))
    with pytest.raises(RuntimeError, match="size mismatch"):
        load_model_dir(str(tmp_path / "shape"))
    with pytest.raises(NotImplementedError):
        load_model_dir(str(tmp_path / "ok"), dtype=torch.float16)
    # a loop over no layers: its tensors may be in the file, nothing reads them
    flat = O.make_config(loop=(1, 1, 2))
    Wf = O.random_weights(flat, seed=2)
    assert "loop.in" not in Wf
    _write_checkpoint(tmp_path / "flat", flat, dict(Wf, **{"loop.in": W["loop.in"], "loop.step": W["loop.step"]}))
    m2 = load_model_dir(str(tmp_path / "flat"))
    assert not m2.config.looped and "loop.in" not in m2.weights and len(m2.config.runs) == len(flat["layers"])


def test_model_refuses_to_run_without_cuda():
    from evo_b200 import _lib
    cfg = O.make_config()
    m = Movalorn(MovalornConfig.from_dict(cfg))
    m.load_state_dict(O.random_weights(cfg))
    with pytest.raises(RuntimeError):
        m.load_state_dict({"embed": torch.zeros(2, 2)})
    with pytest.raises(_lib.EvoError, match="no CPU"):
        m(torch.zeros(1, 4, dtype=torch.long))
    rnd = Movalorn(MovalornConfig.from_dict(cfg)).init_random(seed=3)
    assert set(rnd.weights) == set(O.tensor_shapes(cfg)) and all(torch.isfinite(v.float()).all() for v in rnd.weights.values())


def test_oracle_continues_a_sequence_and_masks_by_distance():
    cfg = O.make_config(layers=("mingru", "latent_attention"), moe_layers=(1,), loop=(0, 2, 2), window=5)
    W = O.random_weights(cfg, seed=2)
    tokens = torch.randint(0, cfg["vocab"], (17,), generator=torch.Generator().manual_seed(0)).tolist()
    whole = O.forward(cfg, W, tokens)
    st = O.new_state(cfg)
    parts = torch.cat([O.forward(cfg, W, tokens[:6], st), O.forward(cfg, W, tokens[6:7], st), O.forward(cfg, W, tokens[7:], st)])
    assert torch.allclose(parts, whole, atol=1e-10)
    # rotation: a pair turns by pos * base^(-2i/dims); entries past `dims` pass unchanged; position 0 is the identity
    v = torch.arange(1.0, 7.0, dtype=torch.float64)
    assert torch.equal(O.rotate_pairs(v, 0, 50.0, 4), v)
    r = O.rotate_pairs(v, 3, 50.0, 4)
    a1 = 3 * 50.0 ** -0.5
    assert torch.allclose(r[:2], torch.tensor([math.cos(3.0) - 2 * math.sin(3.0), 2 * math.cos(3.0) + math.sin(3.0)], dtype=torch.float64))
    assert torch.allclose(r[2:4], torch.tensor([3 * math.cos(a1) - 4 * math.sin(a1), 4 * math.cos(a1) + 3 * math.sin(a1)], dtype=torch.float64))
    assert torch.equal(r[4:], v[4:])
    # candidate of the recurrence is continuous at 0 and the state is a convex mix
    h = torch.zeros(1, cfg["width"], dtype=torch.float64)
    w = {k: v.double() for k, v in W.items()}
    s = torch.zeros(cfg["layers"][0]["mixer"]["width"], dtype=torch.float64)
    O.mingru(h, dict(w, **{"l0.mix.z.b": torch.zeros_like(w["l0.mix.z.b"]), "l0.mix.x.b": torch.zeros_like(w["l0.mix.x.b"])}), "l0.mix.", s)
    assert torch.allclose(s, torch.full_like(s, 0.25))           # z = 1/2, candidate = 1/2
    # embedding: first token uses the last row of the pair table
    e = O.embed_tokens([4, 9], None, w, cfg["embedding"])
    bg = cfg["embedding"]["bigram"]
    assert torch.equal(e[0], w["embed"][4] * cfg["embedding"]["scale"] + w["bigram"][bg["buckets"]])
    assert torch.equal(e[1], w["embed"][9] * cfg["embedding"]["scale"] + w["bigram"][(4 * bg["mul_prev"] + 9 * bg["mul_cur"]) % bg["buckets"]])
