"""Configuration of a Movalorn model: read from the checkpoint folder's config.json (keys as the checkpoints carry them).

Every size and constant comes from here or from a tensor's shape; nothing below is specialised to one checkpoint.  `runs` is the
flattened execution order: the layers [loop.start, loop.stop) are executed loop.times times in a row with the same weights but
separate caches, so caches and recurrent states are keyed by the RUN index, not by the layer index."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class MixerConfig:
    kind: str                      # "latent_attention" | "mingru"
    width: int = 0                 # mingru: channels of the recurrence
    heads: int = 0                 # latent attention from here on
    dim: int = 0                   # per-head unrotated query/key size
    rot_dim: int = 0               # per-head rotated query size = size of the shared rotated key part
    vdim: int = 0
    kv_rank: int = 0               # latent size
    window: int = 0                # visible distance (0: plain causal)
    rot_base: float = 10000.0
    rot_dims: int = 0              # leading entries of the rotated part that are actually turned
    scale: float = 1.0


@dataclass
class MlpConfig:
    kind: str                      # "dense" | "moe"
    ff: int = 0                    # dense: hidden size; moe: hidden size of one expert
    experts: int = 0
    top: int = 0
    router_scale: float = 1.0
    shared_ff: int = 0             # hidden size of the always-on expert (0: none)


@dataclass
class LayerConfig:
    mixer: MixerConfig
    mlp: Optional[MlpConfig]


@dataclass
class Run:
    layer: int
    loop_pass: Optional[int]       # number of the pass through the looped span this run belongs to
    first: bool                    # first run of its pass: the stream is re-projected together with the embedding output before it


@dataclass
class MovalornConfig:
    vocab_size: int
    width: int
    layers: List[LayerConfig]
    eps: float
    embed_scale: float
    buckets: int
    mul_prev: int
    mul_cur: int
    logit_scale: float = 1.0
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    max_seqlen: int = 8192
    max_batch_size: int = 1
    runs: List[Run] = field(default_factory=list)

    def __post_init__(self):
        n = len(self.layers)
        lo, hi, times = self.loop_start, self.loop_stop, max(1, self.loop_times)
        if not (0 <= lo <= hi <= n):
            raise ValueError(f"loop [{lo}, {hi}) does not fit {n} layers")
        runs = [Run(i, None, False) for i in range(lo)]
        for t in range(times if hi > lo else 0):
            runs += [Run(i, t, i == lo) for i in range(lo, hi)]
        runs += [Run(i, None, False) for i in range(hi, n)]
        self.runs = runs

    @property
    def looped(self) -> bool:
        return self.loop_stop > self.loop_start

    @property
    def unused_tensor_names(self):
        """Tensors a checkpoint may carry although this configuration never reads them (a loop over no layers)."""
        return () if self.looped else ("loop.in", "loop.step")

    # dict-style access used by the framework's generic code paths (model.config.get("max_seqlen"))
    def get(self, key, default=None):
        return getattr(self, key, default)

    @classmethod
    def from_dict(cls, d: dict) -> "MovalornConfig":
        layers = []
        for entry in d["layers"]:
            m, kind = entry["mixer"], entry["type"]
            if kind == "latent_attention":
                rot, mask = m.get("rot") or {}, m.get("mask") or {}
                rd = int(m["rot_dim"])
                mixer = MixerConfig(kind, heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=rd, vdim=int(m["vdim"]), kv_rank=int(m["kv_rank"]),
                                    window=int(mask.get("size", 0)), rot_base=float(rot.get("base", 10000.0)), rot_dims=int(rot.get("dims", rd)),
                                    scale=float(m["scale"]))
                if mixer.rot_dims > rd or mixer.rot_dims % 2 or rd % 2:
                    raise ValueError(f"rotated sizes must be even and rot.dims ({mixer.rot_dims}) <= rot_dim ({rd})")
            elif kind == "mingru":
                mixer = MixerConfig(kind, width=int(m["width"]))
            else:
                raise NotImplementedError(f"mixer type {kind!r}")
            mlp = entry.get("mlp")
            if mlp is None:
                ff = None
            elif mlp.get("kind", "dense") == "dense":
                ff = MlpConfig("dense", ff=int(mlp["ff"]))
            elif mlp["kind"] == "moe":
                r, sh = mlp["router"], mlp.get("shared")
                ff = MlpConfig("moe", ff=int(mlp["expert"]["ff"]), experts=int(r["experts"]), top=int(r["top"]), router_scale=float(r.get("scale", 1.0)),
                               shared_ff=int(sh["ff"]) if sh else 0)
                if not 0 < ff.top <= ff.experts:
                    raise ValueError(f"router picks {ff.top} of {ff.experts} experts")
            else:
                raise NotImplementedError(f"feed-forward kind {mlp.get('kind')!r}")
            layers.append(LayerConfig(mixer, ff))
        loop = d.get("loop") or {}
        emb = d.get("embedding") or {}
        bg = emb.get("bigram")
        if not bg:
            raise ValueError("config.json: embedding.bigram is missing")
        return cls(vocab_size=int(d["vocab"]), width=int(d["width"]), layers=layers, eps=float(d["norm"]["eps"]),
                   embed_scale=float(emb.get("scale", 1.0)), buckets=int(bg["buckets"]), mul_prev=int(bg["mul_prev"]), mul_cur=int(bg["mul_cur"]),
                   logit_scale=float(d.get("logit_scale", 1.0)),
                   loop_start=int(loop.get("start", 0)), loop_stop=int(loop.get("stop", 0)), loop_times=int(loop.get("times", 1)),
                   max_seqlen=int(d.get("max_seqlen", 8192)))

    @classmethod
    def from_dir(cls, model_dir: str) -> "MovalornConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def tensor_shapes(self) -> dict:
        """checkpoint tensor name -> shape, in checkpoint naming."""
        d = self.width
        out = {"embed": (self.vocab_size, d), "bigram": (self.buckets + 1, d)}
        if self.looped:
            out["loop.in"] = (d, 2 * d)
            out["loop.step"] = (max(1, self.loop_times), d)
        for i, layer in enumerate(self.layers):
            m, p = layer.mixer, f"l{i}."
            out.update({p + "norm1": (), p + "norm1b": (), p + "rg1": (d, d), p + "rg1.b": (d,)})
            if m.kind == "mingru":
                out.update({p + "mix.z": (m.width, d), p + "mix.z.b": (m.width,), p + "mix.x": (m.width, d), p + "mix.x.b": (m.width,),
                            p + "mix.g": (m.width, d), p + "mix.o": (d, m.width)})
            else:
                out.update({p + "mix.q": (m.heads * (m.dim + m.rot_dim), d), p + "mix.dkv": (m.kv_rank + m.rot_dim, d), p + "mix.dkv.norm": (m.kv_rank,),
                            p + "mix.uk": (m.heads * m.dim, m.kv_rank), p + "mix.uv": (m.heads * m.vdim, m.kv_rank), p + "mix.g": (m.heads, d),
                            p + "mix.o": (d, m.heads * m.vdim)})
            f = layer.mlp
            if f is None:
                continue
            out.update({p + "norm2": (), p + "norm2b": (), p + "rg2": (d, d), p + "rg2.b": (d,)})
            if f.kind == "dense":
                out.update({p + "mlp.gate": (f.ff, d), p + "mlp.up": (f.ff, d), p + "mlp.down": (d, f.ff)})
            else:
                for e in range(f.experts):
                    out.update({f"{p}mlp.e{e}.gate": (f.ff, d), f"{p}mlp.e{e}.up": (f.ff, d), f"{p}mlp.e{e}.down": (d, f.ff)})
                out.update({p + "mlp.router": (f.experts, d), p + "mlp.correction": (f.experts,)})
                if f.shared_ff:
                    out.update({p + "mlp.shared.gate": (f.shared_ff, d), p + "mlp.shared.up": (f.shared_ff, d), p + "mlp.shared.down": (d, f.shared_ff)})
        out["final.norm"] = ()
        out["head"] = (self.vocab_size, d)
        return out
