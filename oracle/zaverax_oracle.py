"""Plain, slow statement of the Zaverax design in PyTorch, one function per mechanism, whole sequences only, any dtype
(float64 by default).  It shares no code with evo_b200: the product is compared against it.

Notation: T tokens, D width, H heads, G key/value heads, dk / dv per-head key / value sizes.
  rms(u)            = u / sqrt(mean(u^2) + eps)                                  (over the last axis)
  offset_norm(x, w) = rms(x) * (1 + w)
  conv_skip(h, c)   = h + sum_j c[:, j] * shift(h, taps - 1 - j)                 (zeros before the first token)
  polynorm(z; a)    = a0 rms(z) + a1 rms(z^2) + a2 rms(z^3) + a3
  hgrn2             : g = lo + (1 - lo) sigmoid(f + b);  S_t = g_t[:, None] * S_{t-1} + (1 - g_t)[:, None] * v_t[None, :];  o_t = S_t^T silu(q_t)
  diff attention    : two softmax maps over the same values, o = a1 - lam * a2, lam = exp(<lq1, lk1>) - exp(<lq2, lk2>) + diff,
                      then rms over dv times (1 - diff), times sigmoid(gate); key j visible from i iff j <= i and
                      (i - j < window or j < keep_first)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(u: torch.Tensor, eps: float) -> torch.Tensor:
    return u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def conv_skip(h: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """h (T, D), c (D, taps): h_t + sum_j c[:, j] * h_{t - (taps-1) + j}."""
    T, taps = h.shape[0], c.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += c[:, j] * h[s]
    return out


def polynorm(z, a, eps):
    return a[0] * rms(z, eps) + a[1] * rms(z ** 2, eps) + a[2] * rms(z ** 3, eps) + a[3]


def visible(i: int, j: int, window: int, keep_first: int) -> bool:
    return j <= i and (window <= 0 or i - j < window or j < keep_first)


def diff_attention(q, k, v, gate, lam, H, G, dk, dv, scale, window, keep_first, diff, eps, rows=None):
    """q (T, H*2*dk), k (T, G*2*dk), v (T, G*dv), gate (T, H*dv) raw -> (T, H*dv); rows: only these queries (others stay 0)."""
    T = q.shape[0]
    q = q.view(T, H, 2, dk)
    k = k.view(T, G, 2, dk)
    v = v.view(T, G, dv)
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in (range(T) if rows is None else rows):
            js = [j for j in range(T) if visible(i, j, window, keep_first)]
            maps = []
            for m in range(2):
                s = (k[js, g, m] * q[i, h, m]).sum(-1) * scale
                p = torch.softmax(s, 0)
                maps.append((p[:, None] * v[js, g]).sum(0))
            o = maps[0] - lam * maps[1]
            out[i, h] = rms(o, eps) * (1.0 - diff)
    return out.reshape(T, H * dv) * torch.sigmoid(gate)


def hgrn2(q, f, v, f_bias, lower, norm_w, H, dk, dv, eps, state: Optional[torch.Tensor] = None):
    """raw projections q, f (T, H*dk), v (T, H*dv) -> (T, H*dv), final state (H, dk, dv)."""
    T = q.shape[0]
    qa = torch.nn.functional.silu(q).view(T, H, dk)
    g = (lower + (1.0 - lower) * torch.sigmoid(f + f_bias)).view(T, H, dk)
    v = v.view(T, H, dv)
    S = torch.zeros(H, dk, dv, dtype=q.dtype) if state is None else state.clone()
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        for h in range(H):
            S[h] = g[t, h][:, None] * S[h] + (1.0 - g[t, h])[:, None] * v[t, h][None, :]
            out[t, h] = rms(S[h].T @ qa[t, h], eps) * norm_w
    return out.reshape(T, H * dv), S


def run_order(n_layers: int, start: int, stop: int, times: int):
    """[(layer, add_embedding_first)] in execution order."""
    order = [(i, False) for i in range(start)]
    for t in range(max(1, times) if stop > start else 0):
        order += [(i, t > 0 and i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n_layers)]


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64, stream_out: Optional[list] = None) -> torch.Tensor:
    """cfg: the checkpoint's config.json as a dict; W: checkpoint tensors; -> logits (T, vocab)."""
    W = {k: t.to(dtype) for k, t in W.items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    taps = (cfg.get("canon") or {}).get("taps", 0)
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    x = W["embed"][torch.tensor(tokens)]
    x0 = x.clone()
    for i, add_first in run_order(len(cfg["layers"]), loop["start"], loop["stop"], loop["times"]):
        if add_first:
            x = x + x0
        layer, p = cfg["layers"][i], f"l{i}."
        m = layer["mixer"]
        h = offset_norm(x, W[p + "norm1"], eps)
        if taps > 0:
            h = conv_skip(h, W[p + "canon1"])
        lin = lambda name: h @ W[p + "mix." + name].T
        if layer["type"] == "attention":
            lam = math.exp(float((W[p + "mix.lq1"] * W[p + "mix.lk1"]).sum())) - math.exp(float((W[p + "mix.lq2"] * W[p + "mix.lk2"]).sum())) + m["diff"]
            mask = m.get("mask") or {}
            y = diff_attention(lin("q"), lin("k"), lin("v"), lin("g"), lam, m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"],
                               m["scale"], mask.get("size", 0), mask.get("keep_first", 0), m["diff"], eps)
        else:
            y, _ = hgrn2(lin("q"), lin("f"), lin("v"), W[p + "mix.f.b"], W[p + "mix.lower"], W[p + "mix.norm"], m["heads"], m["dim"], m["vdim"], eps)
        x = x + mult * (y @ W[p + "mix.o"].T)
        if layer.get("mlp") is not None:
            z = offset_norm(x, W[p + "norm2"], eps) @ W[p + "mlp.up"].T
            x = x + mult * (polynorm(z, W[p + "mlp.act"], eps) @ W[p + "mlp.down"].T)
        if stream_out is not None:
            stream_out.append(x.clone())
    logits = offset_norm(x, W["final.norm"], eps) @ W["head"].T
    cap = cfg.get("logit_softcap", 0.0)
    return cap * torch.tanh(logits / cap) if cap else logits


def make_config(width=96, vocab=300, layers=("hgrn2", "attention"), heads=3, kv_heads=1, dim=20, vdim=24, r_heads=2, r_dim=12, r_vdim=40,
                ff=136, window=9, keep_first=3, diff=0.3, taps=3, loop=(0, 0, 1), residual_mult=0.5, softcap=12.0, eps=1e-5, no_ff_layers=()):
    """A small config.json-shaped dict; every size differs from every other one by default."""
    entries = []
    for n, kind in enumerate(layers):
        mlp = None if n in no_ff_layers else {"kind": "dense", "ff": ff}
        if kind == "attention":
            mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 1.0 / math.sqrt(dim), "diff": diff,
                     "mask": {"size": window, "keep_first": keep_first}}
        else:
            mixer = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim}
        entries.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Zaverax", "vocab": vocab, "width": width, "layers": entries, "norm": {"eps": eps}, "canon": {"taps": taps},
            "loop": {"start": loop[0], "stop": loop[1], "times": loop[2]}, "residual_mult": residual_mult, "logit_softcap": softcap}


def random_weights(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Checkpoint-named random tensors (values exactly representable in bf16) for a config dict."""
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]
    taps = (cfg.get("canon") or {}).get("taps", 0)
    rn = lambda *shape, s=1.0: torch.randn(*shape, generator=g) * s
    W = {"embed": rn(V, D), "final.norm": rn(D, s=0.1), "head": rn(V, D, s=1.0 / math.sqrt(D))}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        W[p + "norm1"] = rn(D, s=0.1)
        if taps > 0:
            W[p + "canon1"] = rn(D, taps, s=0.3)
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        lin = lambda n, k: rn(n, k, s=1.0 / math.sqrt(k))
        if layer["type"] == "attention":
            G = m.get("kv_heads", H)
            W.update({p + "mix.q": lin(H * 2 * dk, D) * 2.0, p + "mix.k": lin(G * 2 * dk, D) * 2.0, p + "mix.v": lin(G * dv, D), p + "mix.g": lin(H * dv, D),
                      p + "mix.o": lin(D, H * dv)})
            for n in ("lq1", "lk1", "lq2", "lk2"):
                W[p + "mix." + n] = rn(dk, s=0.15)
        else:
            W.update({p + "mix.q": lin(H * dk, D), p + "mix.f": lin(H * dk, D) * 2.0, p + "mix.f.b": rn(H * dk), p + "mix.lower": torch.rand(H * dk, generator=g) * 0.9,
                      p + "mix.v": lin(H * dv, D), p + "mix.norm": 1.0 + rn(dv, s=0.1), p + "mix.o": lin(D, H * dv)})
        if layer.get("mlp") is not None:
            F = layer["mlp"]["ff"]
            W.update({p + "norm2": rn(D, s=0.1), p + "mlp.up": lin(F, D), p + "mlp.down": lin(D, F), p + "mlp.act": torch.tensor([0.7, 0.25, 0.1, 0.05]) + rn(4, s=0.05)})
    return {k: t.to(torch.bfloat16) for k, t in W.items()}
