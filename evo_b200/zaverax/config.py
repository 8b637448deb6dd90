"""Configuration of a Zaverax model: read from the checkpoint folder's config.json (keys as the checkpoints carry them).

Every size comes from here or from a tensor's shape; nothing below is specialised to one checkpoint.  `runs` is the
flattened execution order: the layers [loop.start, loop.stop) are executed loop.times times in a row with the same
weights but separate caches, so caches and recurrent states are keyed by the RUN index, not by the layer index."""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class MixerConfig:
    kind: str                      # "attention" | "hgrn2"
    heads: int
    dim: int                       # per-head query/key size
    vdim: int                      # per-head value size
    kv_heads: int = 0              # attention
    scale: float = 1.0
    diff: float = 0.0              # differential-attention constant
    window: int = 0                # visible distance (0: plain causal)
    keep_first: int = 0            # first tokens that stay visible


@dataclass
class LayerConfig:
    mixer: MixerConfig
    ff: Optional[int]              # feed-forward width, None: no feed-forward
    ff_kind: str = "dense"


@dataclass
class Run:
    layer: int
    inject: bool                   # add the embedding output to the stream right before this run


@dataclass
class ZaveraxConfig:
    vocab_size: int
    width: int
    layers: List[LayerConfig]
    eps: float
    residual_mult: float
    taps: int                      # input-convolution taps (0: none)
    logit_softcap: float
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
        runs = [Run(i, False) for i in range(lo)]
        for t in range(times if hi > lo else 0):
            runs += [Run(i, t > 0 and i == lo) for i in range(lo, hi)]
        runs += [Run(i, False) for i in range(hi, n)]
        self.runs = runs

    # dict-style access used by the framework's generic code paths (model.config.get("max_seqlen"))
    def get(self, key, default=None):
        return getattr(self, key, default)

    @classmethod
    def from_dict(cls, d: dict) -> "ZaveraxConfig":
        layers = []
        for entry in d["layers"]:
            m = entry["mixer"]
            kind = entry["type"]
            if kind == "attention":
                mask = m.get("mask") or {}
                mixer = MixerConfig(kind, int(m["heads"]), int(m["dim"]), int(m["vdim"]), kv_heads=int(m.get("kv_heads", m["heads"])),
                                    scale=float(m["scale"]), diff=float(m.get("diff", 0.0)), window=int(mask.get("size", 0)),
                                    keep_first=int(mask.get("keep_first", 0)))
            elif kind == "hgrn2":
                mixer = MixerConfig(kind, int(m["heads"]), int(m["dim"]), int(m["vdim"]))
            else:
                raise NotImplementedError(f"mixer type {kind!r}")
            mlp = entry.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") != "dense":
                raise NotImplementedError(f"feed-forward kind {mlp.get('kind')!r}")
            layers.append(LayerConfig(mixer, None if mlp is None else int(mlp["ff"])))
        loop = d.get("loop") or {}
        return cls(vocab_size=int(d["vocab"]), width=int(d["width"]), layers=layers, eps=float(d["norm"]["eps"]),
                   residual_mult=float(d.get("residual_mult", 1.0)), taps=int((d.get("canon") or {}).get("taps", 0)),
                   logit_softcap=float(d.get("logit_softcap", 0.0) or 0.0),
                   loop_start=int(loop.get("start", 0)), loop_stop=int(loop.get("stop", 0)), loop_times=int(loop.get("times", 1)),
                   max_seqlen=int(d.get("max_seqlen", 8192)))

    @classmethod
    def from_dir(cls, model_dir: str) -> "ZaveraxConfig":
        with open(os.path.join(model_dir, "config.json")) as f:
            return cls.from_dict(json.load(f))

    def tensor_shapes(self) -> dict:
        """checkpoint tensor name -> shape, in checkpoint naming."""
        d, out = self.width, {"embed": (self.vocab_size, self.width)}
        for i, layer in enumerate(self.layers):
            m, p = layer.mixer, f"l{i}."
            out[p + "norm1"] = (d,)
            if layer.ff is not None:
                out[p + "norm2"] = (d,)
            if m.kind == "hgrn2":
                out.update({p + "mix.q": (m.heads * m.dim, d), p + "mix.f": (m.heads * m.dim, d), p + "mix.f.b": (m.heads * m.dim,),
                            p + "mix.lower": (m.heads * m.dim,), p + "mix.v": (m.heads * m.vdim, d), p + "mix.norm": (m.vdim,),
                            p + "mix.o": (d, m.heads * m.vdim)})
            else:
                out.update({p + "mix.q": (m.heads * 2 * m.dim, d), p + "mix.k": (m.kv_heads * 2 * m.dim, d), p + "mix.v": (m.kv_heads * m.vdim, d),
                            p + "mix.lq1": (m.dim,), p + "mix.lk1": (m.dim,), p + "mix.lq2": (m.dim,), p + "mix.lk2": (m.dim,),
                            p + "mix.g": (m.heads * m.vdim, d), p + "mix.o": (d, m.heads * m.vdim)})
            if layer.ff is not None:
                out.update({p + "mlp.up": (layer.ff, d), p + "mlp.down": (d, layer.ff), p + "mlp.act": (4,)})
            if self.taps > 0:
                out[p + "canon1"] = (d, self.taps)
        out["final.norm"] = (d,)
        out["head"] = (self.vocab_size, d)
        return out
