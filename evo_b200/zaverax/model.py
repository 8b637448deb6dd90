"""Zaverax: a decoder-only model with an fp32 residual stream, a short causal convolution in front of every mixer, two
kinds of mixer (windowed differential attention with kept first tokens; the HGRN2 gated linear recurrence), a PolyNorm
feed-forward, a weight-shared loop over a span of layers and soft-capped logits -- executed by libevo_b200.so.

It follows the object protocol of the framework's other model (StripedHyena), so the same generation loop, scheduler
and command line drive it:
    model(ids) -> (logits, None)                          stateless, whole sequences
    model(ids, inference_params_dict=d) -> (logits, d)    continues from the caches in d at d["mha"].seqlen_offset
    model.initialize_inference_params()                   the framework's two state holders
    model.decode_loop(...)                                one CUDA graph per generated token
State (keyed by RUN index, a looped layer has one entry per pass):
    d["mha"].key_value_memory_dict[r]   (B, max_seqlen, G*(2*dim) + G*vdim): keys of both score maps, then values
    d["hyena"].fir_state_dict[r]        (B, taps-1, width) fp32: the last normed inputs of the input convolution
    d["hyena"].state_dict[r]            (B, heads, dim, vdim) fp32: the recurrence's matrix state
Per layer:  x += m * mixer(conv(norm1(x)));  x += m * ff(norm2(x))   with x fp32.  The residual update of one branch is
fused into the norm that opens the next (evo_resid_norm), so x is read and written once per branch.
Linear layers: bf16 activations -> the framework's tcgen05 GEMMs (weights zero-padded once to their tiles);
fp32 activations (dtype=torch.float32) -> evo_gemm_simt, true fp32 multiply-add.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Dict, Optional

import torch
import torch.nn as nn

from .. import _lib
from .._lib import EPI_NONE, CausalConvParams, Hgrn2Params, ResidNormParams, WindowAttnParams, check, ptr
from ..stream_model import StreamDecoder, _Packed, _round_up
from ..stripedhyena.cache import InferenceParams, RecurrentInferenceParams
from .config import ZaveraxConfig


class Zaverax(StreamDecoder):
    architecture = "Zaverax"
    gemm_env = "EVO_B200_ZAVERAX_GEMM"

    def __init__(self, config: ZaveraxConfig, dtype: torch.dtype = torch.bfloat16):
        super().__init__(config, dtype)
        self.fir_taps = config.taps

    # ---- parameters ----------------------------------------------------------------------------
    def init_random(self, seed: int = 0, device=None) -> "Zaverax":
        """Random weights of a usable scale (benchmarks, tests)."""
        g = torch.Generator().manual_seed(seed)
        for name, t in self.weights.items():
            shape = t.shape
            leaf = name.split(".")[-1]
            if name.endswith(("norm1", "norm2", "final.norm")):
                v = torch.randn(shape, generator=g) * 0.1
            elif name.endswith("mix.norm"):
                v = 1.0 + torch.randn(shape, generator=g) * 0.1
            elif name.endswith("lower"):
                v = torch.rand(shape, generator=g) * 0.9
            elif name.endswith("f.b"):
                v = torch.randn(shape, generator=g)
            elif leaf in ("lq1", "lk1", "lq2", "lk2"):
                v = torch.randn(shape, generator=g) * 0.1
            elif name.endswith("act"):
                v = torch.tensor([0.6, 0.3, 0.1, 0.05]) + torch.randn(4, generator=g) * 0.05
            elif "canon" in name:
                v = torch.randn(shape, generator=g) * 0.2
            elif name == "embed":
                v = torch.randn(shape, generator=g)
            else:
                v = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
            self.weights[name] = v.to(torch.bfloat16)
        self._invalidate()
        return self.to(device) if device is not None else self

    # ---- packing -------------------------------------------------------------------------------
    def _ensure_packed(self):
        if self._packed is not None:
            return self._packed
        dev = self.device
        if dev.type != "cuda":
            raise _lib.EvoError("evo_b200 runs on CUDA (sm_100a) only: move the model with .to('cuda:N'); there is no CPU path")
        w = self.weights
        packed = {"head": _Packed(w["head"]), "layers": []}
        for i, layer in enumerate(self.config.layers):
            m, p = layer.mixer, f"l{i}."
            e = {}
            if m.kind == "hgrn2":
                e["in"] = _Packed(torch.cat([w[p + "mix.q"], w[p + "mix.f"], w[p + "mix.v"]], 0))
            else:
                e["in"] = _Packed(torch.cat([w[p + "mix.q"], w[p + "mix.k"], w[p + "mix.v"], w[p + "mix.g"]], 0))
                f32 = lambda n: w[p + "mix." + n].float().cpu()
                e["lambda"] = float(torch.exp((f32("lq1") * f32("lk1")).sum()) - torch.exp((f32("lq2") * f32("lk2")).sum())) + m.diff
            e["out"] = _Packed(w[p + "mix.o"])
            if layer.ff is not None:
                e["up"], e["down"] = _Packed(w[p + "mlp.up"]), _Packed(w[p + "mlp.down"])
            packed["layers"].append(e)
        self._packed = packed
        return packed

    # ---- kernels ---------------------------------------------------------------------------------
    def _resid_norm(self, x, y, ldy, weight, offset, out, ldo, out_f32, B, L, halo=0, halo_src=None, x_add=None, gather=None, y_scale=None):
        cfg = self.config
        p = ResidNormParams(x=x.data_ptr(), y=y.data_ptr() if y is not None else None, ldy=ldy, y_dtype=self._dt,
                            y_scale=cfg.residual_mult if y_scale is None else y_scale,
                            x_add=x_add.data_ptr() if x_add is not None else None, weight=weight.data_ptr() if weight is not None else None,
                            weight_offset=offset, eps=cfg.eps, out=out.data_ptr(), ldo=ldo, out_dtype=1 if out_f32 else self._dt,
                            B=B, seq_len=L, halo=halo, D=cfg.width, halo_src=halo_src.data_ptr() if halo_src is not None else None,
                            gather=gather.data_ptr() if gather is not None else None)
        esz = 4 if self._dt else 2
        nbytes = B * L * cfg.width * (4.0 + (4.0 + esz if y is not None else 0.0) + (4.0 if x_add is not None else 0.0) + (4.0 if out_f32 else esz))
        self._record("resid_norm", nbytes, lambda: check(_lib.lib().evo_resid_norm(C.byref(p), self._stream()), "evo_resid_norm"))

    def _mixer_input(self, r, i, x, y, ldy, B, L, rec: Optional[RecurrentInferenceParams], x_add):
        """x <- x + m*y (+ embedding output); h = norm1(x); returns h + conv(h) as (B*L, Kp) activations."""
        cfg, dev = self.config, x.device
        D, Kp = cfg.width, _round_up(cfg.width, 64)
        w = self.weights
        h = torch.empty(B * L, Kp, dtype=self.act_dtype, device=dev)
        if cfg.taps <= 0:
            self._resid_norm(x, y, ldy, w[f"l{i}.norm1"], 1.0, h, Kp, False, B, L, x_add=x_add)
            return h
        halo = cfg.taps - 1
        carry = rec.fir_state_dict.get(r) if rec is not None else None
        hn = torch.empty(B, halo + L, D, dtype=torch.float32, device=dev)
        self._resid_norm(x, y, ldy, w[f"l{i}.norm1"], 1.0, hn, D, True, B, L, halo=halo, halo_src=carry, x_add=x_add)
        if rec is not None and carry is None:
            carry = rec.fir_state_dict[r] = torch.empty(B, halo, D, dtype=torch.float32, device=dev)
        cp = CausalConvParams(inp=hn.data_ptr(), weight=w[f"l{i}.canon1"].data_ptr(), out=h.data_ptr(), ldo=Kp, out_dtype=self._dt,
                              carry_out=carry.data_ptr() if carry is not None else None, B=B, seq_len=L, D=D, taps=cfg.taps)
        self._record("causal_conv", B * L * D * (4.0 + h.element_size()), lambda: check(_lib.lib().evo_causal_conv(C.byref(cp), self._stream()), "evo_causal_conv"))
        return h

    def _hgrn2(self, r, i, m, h, B, L, rec: Optional[RecurrentInferenceParams]):
        pk = self._packed["layers"][i]
        M, dev = B * L, h.device
        z = self._linear(h, pk["in"], M)
        esz = z.element_size()
        inner = m.heads * m.vdim
        ldo = _round_up(inner, 64)
        out = torch.empty(M, ldo, dtype=self.act_dtype, device=dev)
        state, zero = None, 1
        if rec is not None:
            state = rec.state_dict.get(r)
            zero = 0
            if state is None:
                state = rec.state_dict[r] = torch.empty(B, m.heads, m.dim, m.vdim, dtype=torch.float32, device=dev)
                zero = 1
        w = self.weights
        hp = Hgrn2Params(q=z.data_ptr(), f=z.data_ptr() + m.heads * m.dim * esz, v=z.data_ptr() + 2 * m.heads * m.dim * esz, ld=pk["in"].Np,
                         f_bias=w[f"l{i}.mix.f.b"].data_ptr(), lower=w[f"l{i}.mix.lower"].data_ptr(), norm_w=w[f"l{i}.mix.norm"].data_ptr(),
                         eps=self.config.eps, state=state.data_ptr() if state is not None else None, zero_start=zero,
                         out=out.data_ptr(), ldo=ldo, dtype=self._dt, B=B, L=L, H=m.heads, dk=m.dim, dv=m.vdim)
        nws = _lib.lib().evo_hgrn2_workspace(C.byref(hp))
        ws = torch.empty(nws, dtype=torch.uint8, device=dev) if nws else None
        self._record("hgrn2", 3.0 * M * m.heads * m.dim * m.vdim, lambda: check(_lib.lib().evo_hgrn2_fwd(C.byref(hp), ptr(ws), nws, self._stream()), "evo_hgrn2_fwd"))
        return self._linear(out, pk["out"], M), pk["out"].Np

    def _attention(self, r, i, m, h, B, L, ip: Optional[InferenceParams], off: int, pos_dev):
        pk = self._packed["layers"][i]
        M, dev = B * L, h.device
        lib = _lib.lib()
        z = self._linear(h, pk["in"], M)
        esz = z.element_size()
        ld = pk["in"].Np
        qw, kw, vw = m.heads * 2 * m.dim, m.kv_heads * 2 * m.dim, m.kv_heads * m.vdim
        inner = m.heads * m.vdim
        ldo = _round_up(inner, 64)
        out = torch.empty(M, ldo, dtype=self.act_dtype, device=dev)
        ap = WindowAttnParams(q=z.data_ptr(), q_tok_stride=ld, gate=z.data_ptr() + (qw + kw + vw) * esz, gate_tok_stride=ld,
                              out=out.data_ptr(), ldo=ldo, dtype=self._dt, B=B, Lq=L, H=m.heads, G=m.kv_heads, dk=m.dim, dv=m.vdim, n_maps=2,
                              q_pos0=off, pos_dev=pos_dev.data_ptr() if pos_dev is not None else None, window=m.window, keep_first=m.keep_first,
                              scale=m.scale, lambda_=pk["lambda"], head_norm=1, norm_eps=self.config.eps, out_scale=1.0 - m.diff)
        if ip is None:
            ap.k, ap.v = z.data_ptr() + qw * esz, z.data_ptr() + (qw + kw) * esz
            ap.k_tok_stride = ap.v_tok_stride = ld
            ap.k_batch_stride = ap.v_batch_stride = L * ld
        else:
            cache = self._kv_rows(ip, r, kw + vw, B, off, L, pos_dev)
            cw = kw + vw
            check(lib.evo_copy_rows(C.c_void_p(z.data_ptr() + qw * esz), ld, ptr(cache), cw, cache.shape[1] * cw, B, L, cw, off,
                                    ptr(pos_dev), self._dt, self._stream()), "evo_copy_rows")
            ap.k, ap.v = cache.data_ptr(), cache.data_ptr() + kw * esz
            ap.k_tok_stride = ap.v_tok_stride = cw
            ap.k_batch_stride = ap.v_batch_stride = cache.shape[1] * cw
        span = min(off + L, m.window + m.keep_first) if m.window > 0 else off + (L + 1) / 2.0
        self._record("window_attn", 4.0 * M * m.heads * span * (m.dim + m.vdim), lambda: check(lib.evo_window_attn_fwd(C.byref(ap), self._stream()), "evo_window_attn_fwd"))
        return self._linear(out, pk["out"], M), pk["out"].Np

    def _feed_forward(self, i, layer, x, y, ldy, B, L):
        cfg, dev = self.config, x.device
        M, Kp = B * L, _round_up(cfg.width, 64)
        pk = self._packed["layers"][i]
        h = torch.empty(M, Kp, dtype=self.act_dtype, device=dev)
        self._resid_norm(x, y, ldy, self.weights[f"l{i}.norm2"], 1.0, h, Kp, False, B, L)
        z = self._linear(h, pk["up"], M)
        a = torch.empty(M, pk["down"].Kp, dtype=self.act_dtype, device=dev)
        self._record("polynorm", 2.0 * z.element_size() * M * layer.ff, lambda: check(_lib.lib().evo_polynorm(
            ptr(z), pk["up"].Np, ptr(self.weights[f"l{i}.mlp.act"]), ptr(a), pk["down"].Kp, M, layer.ff, cfg.eps, self._dt, self._stream()), "evo_polynorm"))
        return self._linear(a, pk["down"], M), pk["down"].Np

    def _body(self, ids, B, L, ipd, off: int, pos_dev=None, rows=None):
        """embed -> every run -> final norm -> head -> soft cap.  Returns fp32 logits (B*L, V), or (len(rows), V) for the
        flat row indices in `rows` (int64 tensor on the device)."""
        cfg, dev = self.config, ids.device
        lib = _lib.lib()
        M, D, V = B * L, cfg.width, cfg.vocab_size
        ip = ipd["mha"] if ipd is not None else None
        rec = ipd["hyena"] if ipd is not None else None
        x = torch.empty(M, D, dtype=torch.float32, device=dev)
        check(lib.evo_embed_f32(ptr(ids), int(ids.dtype == torch.int64), ptr(self.weights["embed"]), ptr(x), M, D, V, self._stream()), "evo_embed_f32")
        x0 = x.clone() if any(run.inject for run in cfg.runs) else None
        y, ldy = None, 0
        for r, run in enumerate(cfg.runs):
            layer = cfg.layers[run.layer]
            m = layer.mixer
            h = self._mixer_input(r, run.layer, x, y, ldy, B, L, rec, x0 if run.inject else None)
            if m.kind == "hgrn2":
                y, ldy = self._hgrn2(r, run.layer, m, h, B, L, rec)
            else:
                y, ldy = self._attention(r, run.layer, m, h, B, L, ip, off, pos_dev)
            if layer.ff is not None:
                y, ldy = self._feed_forward(run.layer, layer, x, y, ldy, B, L)
            if self._tap is not None:
                self._tap.append(x + cfg.residual_mult * y[:, :D].float())
        n_out = M if rows is None else int(rows.numel())
        if n_out == 0:
            return torch.empty(0, V, dtype=torch.float32, device=dev)
        Kp = _round_up(D, 64)
        hf = torch.empty(n_out, Kp, dtype=self.act_dtype, device=dev)
        if rows is None:
            self._resid_norm(x, y, ldy, self.weights["final.norm"], 1.0, hf, Kp, False, B, L)
        else:
            self._resid_norm(x, y, ldy, self.weights["final.norm"], 1.0, hf, Kp, False, 1, n_out, gather=rows)
        raw = self._linear(hf, self._packed["head"], n_out)
        logits = torch.empty(n_out, V, dtype=torch.float32, device=dev)
        check(lib.evo_softcap_logits(ptr(raw), self._packed["head"].Np, ptr(logits), n_out, V, cfg.logit_softcap, self._dt, self._stream()), "evo_softcap_logits")
        return logits
