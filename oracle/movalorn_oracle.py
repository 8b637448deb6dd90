"""Plain, slow statement of the Movalorn design in PyTorch, one function per mechanism, any dtype (float64 by default).
It shares no code with evo_b200: the product is compared against it.

Notation: T tokens, D width, H heads.  rms(u) = u / sqrt(mean(u^2) + eps) over the last axis.
  scalar_norm(x, g)  = rms(x) * g                                   g one number
  embedding          : E[tok] * s + Bg[(prev * a + tok * b) mod n]   (row n of Bg for a sequence's first token)
  branch             : x + scalar_norm(f(h) * sigmoid(R h + r), g_b),  h = scalar_norm(x, g_a)
  rotation           : pairs (2i, 2i+1) of a vector turned by the angle pos * base^(-2i/dims)
  latent attention   : c = rms(A h)[:rank] * w,  kr = rot(A h [rank:]);  head: key = [U_k c ; kr], value = U_v c,
                       query = [q_a ; rot(q_b)], softmax over keys j with 0 <= i - j < window, output times sigmoid of one number per head
  minGRU             : z = sigmoid(Z h + bz), u = X h + bx, cand = u + 1/2 (u >= 0) | sigmoid(u) (u < 0),
                       S_t = (1 - z) S_{t-1} + z cand, out = O (S_t * silu(G h))
  dense feed-forward : W_d (gelu_tanh(W_g h) * W_u h)
  expert mixture     : s = softmax(Rt h); the `top` experts with the largest s + corr; weights s * scale (not renormalised);
                       experts W_d (silu(W_g h) * W_u h); a shared expert is added with weight 1
  loop               : layers [start, stop) run `times` times; before every pass x <- W_in [x ; x0] + step[t]
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(u: torch.Tensor, eps: float) -> torch.Tensor:
    return u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    return rms(x, eps) * g


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def embed_tokens(tokens: List[int], prev: Optional[int], w: Dict[str, torch.Tensor], emb: dict) -> torch.Tensor:
    """Rows of the token table times the scale plus the hashed pair table; prev is the token before tokens[0] (None: none)."""
    bg = emb["bigram"]
    n, a, b = int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"])
    rows = []
    for t, tok in enumerate(tokens):
        p = prev if t == 0 else tokens[t - 1]
        idx = n if p is None else (p * a + tok * b) % n
        rows.append(w["embed"][tok] * emb["scale"] + w["bigram"][idx])
    return torch.stack(rows)


def rotate_pairs(v: torch.Tensor, pos: int, base: float, dims: int) -> torch.Tensor:
    """v (..., n): the first `dims` entries are turned pair by pair (2i with 2i+1), the rest pass unchanged."""
    out = v.clone()
    for i in range(dims // 2):
        ang = pos * base ** (-2.0 * i / dims)
        c, s = math.cos(ang), math.sin(ang)
        a, b = v[..., 2 * i], v[..., 2 * i + 1]
        out[..., 2 * i] = a * c - b * s
        out[..., 2 * i + 1] = b * c + a * s
    return out


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, cache: list, rows=None) -> torch.Tensor:
    """h (T, D) continues the sequence held in `cache` (a list of (latent, rotated key part) per earlier token)."""
    H, dim, rd, vd, rank = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    base, dims, window, scale = float(m["rot"]["base"]), int(m["rot"]["dims"]), int(m["mask"]["size"]), float(m["scale"])
    T = h.shape[0]
    out = torch.zeros(T, H * vd, dtype=h.dtype)
    for t in range(T):
        pos = len(cache)
        a = w[p + "dkv"] @ h[t]
        c = rms(a[:rank], eps) * w[p + "dkv.norm"]
        kr = rotate_pairs(a[rank:], pos, base, dims)
        cache.append((c, kr))
        if rows is not None and t not in rows:
            continue
        q = (w[p + "q"] @ h[t]).view(H, dim + rd)
        gate = torch.sigmoid(w[p + "g"] @ h[t])
        lo = max(0, pos - window + 1)
        for hd in range(H):
            qa, qb = q[hd, :dim], rotate_pairs(q[hd, dim:], pos, base, dims)
            uk = w[p + "uk"][hd * dim:(hd + 1) * dim]
            uv = w[p + "uv"][hd * vd:(hd + 1) * vd]
            s = torch.stack([(qa @ (uk @ cache[j][0]) + qb @ cache[j][1]) * scale for j in range(lo, pos + 1)])
            a_ = torch.softmax(s, 0)
            o = sum(a_[j - lo] * (uv @ cache[j][0]) for j in range(lo, pos + 1))
            out[t, hd * vd:(hd + 1) * vd] = o * gate[hd]
    return out @ w[p + "o"].T


def mingru(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, state: torch.Tensor) -> torch.Tensor:
    """h (T, D); state (width,) is updated in place."""
    T = h.shape[0]
    outs = []
    for t in range(T):
        z = torch.sigmoid(w[p + "z"] @ h[t] + w[p + "z.b"])
        u = w[p + "x"] @ h[t] + w[p + "x.b"]
        cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
        state.copy_((1.0 - z) * state + z * cand)
        outs.append(w[p + "o"] @ (state * silu(w[p + "g"] @ h[t])))
    return torch.stack(outs)


def glu(h, w, p, act):
    return (act(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def expert_mixture(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mlp: dict) -> torch.Tensor:
    r = mlp["router"]
    E, top, rscale = int(r["experts"]), int(r["top"]), float(r["scale"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        s = torch.softmax(w[p + "router"] @ h[t], 0)
        chosen = torch.topk(s + w[p + "correction"], top).indices.tolist()
        for e in chosen:
            out[t] += s[e] * rscale * glu(h[t], w, f"{p}e{e}.", silu)
        if mlp.get("shared") is not None:
            out[t] += glu(h[t], w, p + "shared.", silu)
    return out


def feed_forward(h, w, p, mlp):
    if mlp["kind"] == "dense":
        return glu(h, w, p, gelu_tanh)
    if mlp["kind"] == "moe":
        return expert_mixture(h, w, p, mlp)
    raise NotImplementedError(mlp["kind"])


def run_order(n_layers: int, start: int, stop: int, times: int):
    """[(layer, pass number or None, first of its pass)] in execution order."""
    runs = [(i, None, False) for i in range(start)]
    for t in range(times if stop > start else 0):
        runs += [(i, t, i == start) for i in range(start, stop)]
    runs += [(i, None, False) for i in range(stop, n_layers)]
    return runs


def new_state(cfg: dict) -> dict:
    return {"prev": None, "runs": {}}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], state: Optional[dict] = None, dtype=torch.float64,
            tap: Optional[list] = None) -> torch.Tensor:
    """Logits (T, vocab) of `tokens` continuing `state` (new_state(cfg); None: a fresh sequence).  tap receives the stream after every run."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    st = new_state(cfg) if state is None else state
    eps = float(cfg["norm"]["eps"])
    x = embed_tokens(tokens, st["prev"], w, cfg["embedding"])
    st["prev"] = tokens[-1]
    x0 = x.clone()
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    for r, (i, t, first) in enumerate(run_order(len(cfg["layers"]), int(loop["start"]), int(loop["stop"]), int(loop["times"]))):
        layer = cfg["layers"][i]
        p = f"l{i}."
        if first:
            x = torch.cat([x, x0], -1) @ w["loop.in"].T + w["loop.step"][t]
        h = scalar_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            y = latent_attention(h, w, p + "mix.", layer["mixer"], eps, st["runs"].setdefault(r, []))
        elif layer["type"] == "mingru":
            y = mingru(h, w, p + "mix.", st["runs"].setdefault(r, torch.zeros(int(layer["mixer"]["width"]), dtype=dtype)))
        else:
            raise NotImplementedError(layer["type"])
        y = y * torch.sigmoid(h @ w[p + "rg1"].T + w[p + "rg1.b"])
        x = x + scalar_norm(y, w[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            h = scalar_norm(x, w[p + "norm2"], eps)
            y = feed_forward(h, w, p + "mlp.", layer["mlp"])
            y = y * torch.sigmoid(h @ w[p + "rg2"].T + w[p + "rg2.b"])
            x = x + scalar_norm(y, w[p + "norm2b"], eps)
        if tap is not None:
            tap.append(x.clone())
    return (scalar_norm(x, w["final.norm"], eps) @ w["head"].T) * float(cfg.get("logit_scale", 1.0))


# ---- small configurations and random weights for the tests -------------------------------------------------------------
def make_config(width=48, vocab=61, layers=("mingru", "latent_attention"), heads=3, dim=8, rot_dim=4, vdim=10, kv_rank=12, window=7, rot_base=100.0,
                att_scale=None, gru_width=40, ff=36, moe_layers=(), experts=5, top=2, expert_ff=20, shared_ff=24, router_scale=1.5, no_ff_layers=(),
                loop=None, buckets=53, mul_prev=5, mul_cur=3, embed_scale=3.0, logit_scale=0.5, eps=1e-5) -> dict:
    out = []
    for i, kind in enumerate(layers):
        if kind == "latent_attention":
            mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "mask": {"size": window},
                     "rot": {"base": rot_base, "dims": rot_dim}, "scale": att_scale if att_scale is not None else 1.0 / math.sqrt(dim + rot_dim)}
        else:
            mixer = {"width": gru_width}
        if i in no_ff_layers:
            mlp = None
        elif i in moe_layers:
            mlp = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top, "scale": router_scale},
                   "shared": {"ff": shared_ff} if shared_ff else None}
        else:
            mlp = {"kind": "dense", "ff": ff}
        out.append({"type": kind, "mixer": mixer, "mlp": mlp})
    cfg = {"architecture": "Movalorn", "vocab": vocab, "width": width, "layers": out, "norm": {"eps": eps}, "logit_scale": logit_scale,
           "embedding": {"scale": embed_scale, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}}
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    D, V = int(cfg["width"]), int(cfg["vocab"])
    s = {"embed": (V, D), "bigram": (int(cfg["embedding"]["bigram"]["buckets"]) + 1, D)}
    loop = cfg.get("loop")
    if loop is not None and loop["stop"] > loop["start"]:
        s["loop.in"] = (D, 2 * D)
        s["loop.step"] = (int(loop["times"]), D)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for n in ("norm1", "norm1b"):
            s[p + n] = ()
        s[p + "rg1"], s[p + "rg1.b"] = (D, D), (D,)
        if layer["type"] == "mingru":
            W = int(m["width"])
            s.update({p + "mix.z": (W, D), p + "mix.z.b": (W,), p + "mix.x": (W, D), p + "mix.x.b": (W,), p + "mix.g": (W, D), p + "mix.o": (D, W)})
        else:
            H, dim, rd, vd, rank = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
            s.update({p + "mix.q": (H * (dim + rd), D), p + "mix.dkv": (rank + rd, D), p + "mix.dkv.norm": (rank,), p + "mix.uk": (H * dim, rank),
                      p + "mix.uv": (H * vd, rank), p + "mix.g": (H, D), p + "mix.o": (D, H * vd)})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        for n in ("norm2", "norm2b"):
            s[p + n] = ()
        s[p + "rg2"], s[p + "rg2.b"] = (D, D), (D,)
        if mlp["kind"] == "dense":
            F = int(mlp["ff"])
            s.update({p + "mlp.gate": (F, D), p + "mlp.up": (F, D), p + "mlp.down": (D, F)})
        else:
            F, E = int(mlp["expert"]["ff"]), int(mlp["router"]["experts"])
            for e in range(E):
                s.update({f"{p}mlp.e{e}.gate": (F, D), f"{p}mlp.e{e}.up": (F, D), f"{p}mlp.e{e}.down": (D, F)})
            s[p + "mlp.router"], s[p + "mlp.correction"] = (E, D), (E,)
            if mlp.get("shared") is not None:
                Fs = int(mlp["shared"]["ff"])
                s.update({p + "mlp.shared.gate": (Fs, D), p + "mlp.shared.up": (Fs, D), p + "mlp.shared.down": (D, Fs)})
    s["final.norm"] = ()
    s["head"] = (V, D)
    return s


def random_weights(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """bf16 tensors of a usable scale, named and shaped as a checkpoint's."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2", "norm1b", "norm2b"):
            v = 0.5 + torch.rand(shape, generator=g)
        elif name == "final.norm":
            v = 0.8 + 0.4 * torch.rand(shape, generator=g)
        elif name.endswith("dkv.norm"):
            v = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "b" or name.endswith("correction"):
            v = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            v = torch.randn(shape, generator=g) / float(cfg["embedding"]["scale"])
        elif name in ("bigram", "loop.step"):
            v = 0.3 * torch.randn(shape, generator=g)
        elif name.endswith("router"):
            v = 2.0 * torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        else:
            v = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = v.to(torch.bfloat16)
    return out
