"""Zaverax on the GPU against the plain oracle (oracle/zaverax_oracle.py): every mechanism's kernel alone, then the model --
whole prompts, token-by-token decoding, portions, batches, reused cache memory, window / kept-token edges, long decoding,
other sizes -- and greedy generation through the framework's Generator.  Small configurations, random weights; where random
weights would hide a fault one score is made to stand out."""
import ctypes as C
import math

import pytest
import torch

from evo_b200 import _lib
from evo_b200._lib import CausalConvParams, Hgrn2Params, ResidNormParams, WindowAttnParams, check, ptr
from oracle import zaverax_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F32, B16 = torch.float32, torch.bfloat16


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _bf(t):
    return t.to(B16)


def _close(got, want, tol, what=""):
    err = (got.double().cpu() - want.double()).abs().max().item()
    ref = max(want.abs().max().item(), 1e-6)
    assert err <= tol * ref, f"{what}: max err {err:.3e} vs scale {ref:.3e} (tol {tol})"


# ------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("D,ldo,halo,L,B", [(96, 128, 2, 7, 2), (130, 192, 0, 5, 1), (1032, 1088, 3, 2, 1)])
def test_resid_norm_matches_the_oracle(D, ldo, halo, L, B):
    g = torch.Generator().manual_seed(D)
    x = torch.randn(B * L, D, generator=g)
    y = _bf(torch.randn(B * L, D + 6, generator=g))
    add = torch.randn(B * L, D, generator=g)
    w = _bf(torch.randn(D, generator=g) * 0.2)
    carry = torch.randn(B, max(halo, 1), D, generator=g)
    xd, out = x.to(DEV), torch.full((B, halo + L, ldo), 7.0, device=DEV)
    p = ResidNormParams(x=xd.data_ptr(), y=y.to(DEV).data_ptr(), ldy=D + 6, y_dtype=0, y_scale=0.3, x_add=add.to(DEV).data_ptr(), weight=w.to(DEV).data_ptr(),
                        weight_offset=1.0, eps=1e-5, out=out.data_ptr(), ldo=ldo, out_dtype=1, B=B, seq_len=L, halo=halo, D=D,
                        halo_src=carry.to(DEV).data_ptr() if halo else None, gather=None)
    keep = [t for t in (y, add, w, carry)]
    yd, addd, wd, cd = y.to(DEV), add.to(DEV), w.to(DEV), carry.to(DEV)
    p.y, p.x_add, p.weight = yd.data_ptr(), addd.data_ptr(), wd.data_ptr()
    p.halo_src = cd.data_ptr() if halo else None
    check(_lib.lib().evo_resid_norm(C.byref(p), _stream()))
    xn = x.double() + 0.3 * y[:, :D].double() + add.double()
    want = O.offset_norm(xn, w.double(), 1e-5).view(B, L, D)
    _close(xd, xn, 1e-6, "stream update")
    _close(out[:, halo:, :D], want, 1e-5, "norm")
    assert (out[:, :, D:] == 0).all()
    if halo:
        _close(out[:, :halo, :D], carry[:, :halo].double(), 0, "carried rows")
    del keep


@pytest.mark.parametrize("taps,L", [(3, 9), (2, 1), (4, 2), (1, 5)])
def test_causal_conv_with_carry_equals_the_whole_sequence(taps, L):
    D, B, ldo = 70, 2, 128
    g = torch.Generator().manual_seed(taps)
    full = torch.randn(B, 20 + L, D, generator=g)
    w = _bf(torch.randn(D, taps, generator=g))
    want = torch.stack([O.conv_skip(full[b].double(), w.double()) for b in range(B)])[:, 20:]
    halo = taps - 1
    inp = full[:, 20 - halo:].contiguous().to(DEV)                 # the carried rows are the taps-1 inputs before the portion
    out = torch.full((B * L, ldo), 5.0, device=DEV)
    carry = torch.zeros(B, max(halo, 1), D, device=DEV)
    wd = w.to(DEV)
    p = CausalConvParams(inp=inp.data_ptr(), weight=wd.data_ptr(), out=out.data_ptr(), ldo=ldo, out_dtype=1, carry_out=carry.data_ptr(), B=B, seq_len=L, D=D, taps=taps)
    check(_lib.lib().evo_causal_conv(C.byref(p), _stream()))
    _close(out.view(B, L, ldo)[:, :, :D], want, 1e-6, "conv")
    assert (out[:, D:] == 0).all()
    if halo:
        _close(carry[:, :halo], full[:, 20 + L - halo:].double(), 0, "next carry")


@pytest.mark.parametrize("F", [136, 1000])
def test_polynorm_and_softcap(F):
    g = torch.Generator().manual_seed(F)
    z = torch.randn(5, F + 8, generator=g) * 1.7
    a = _bf(torch.tensor([0.7, -0.3, 0.15, 0.05]))
    zd, ad, out = z.to(DEV), a.to(DEV), torch.full((5, F + 24), 3.0, device=DEV)
    check(_lib.lib().evo_polynorm(ptr(zd), F + 8, ptr(ad), ptr(out), F + 24, 5, F, 1e-5, 1, _stream()))
    _close(out[:, :F], O.polynorm(z[:, :F].double(), a.double(), 1e-5), 2e-6, "polynorm")
    assert (out[:, F:] == 0).all()
    capped = torch.empty(5, F, device=DEV)
    check(_lib.lib().evo_softcap_logits(ptr(zd), F + 8, ptr(capped), 5, F, 2.5, 1, _stream()))
    _close(capped, 2.5 * torch.tanh(z[:, :F].double() / 2.5), 2e-6, "softcap")


@pytest.mark.parametrize("M,N,K", [(1, 300, 96), (3, 70, 130), (8, 256, 64), (9, 33, 17), (150, 200, 333)])
@pytest.mark.parametrize("dtype", [F32, B16])
def test_gemm_simt(M, N, K, dtype):
    g = torch.Generator().manual_seed(M * N)
    a, w = torch.randn(M, K + 3, generator=g).to(dtype), _bf(torch.randn(N, K + 5, generator=g))
    ad, wd, c = a.to(DEV), w.to(DEV), torch.zeros(M, N + 2, dtype=dtype, device=DEV)
    check(_lib.lib().evo_gemm_simt(ptr(ad), K + 3, ptr(wd), K + 5, ptr(c), N + 2, M, N, K, int(dtype == F32), _stream()))
    _close(c[:, :N], a[:, :K].double() @ w[:, :K].double().T, 1e-5 if dtype == F32 else 6e-3, "gemm")


@pytest.mark.parametrize("H,dk,dv", [(2, 12, 40), (1, 56, 64), (3, 130, 96), (1, 256, 320), (2, 7, 5)])
def test_hgrn2_scan_step_and_carried_state(H, dk, dv):
    """whole sequence == portions (2, 1 and 17 tokens among them) through the carried state == the oracle; heads too large for
    one CTA take the split path."""
    T, B = 40, 2
    g = torch.Generator().manual_seed(dk * dv)
    ld = 2 * H * dk + H * dv + 5
    z = torch.randn(B, T, ld, generator=g)
    fb, lo, nw = _bf(torch.randn(H * dk, generator=g)), _bf(torch.rand(H * dk, generator=g) * 0.95), _bf(1 + 0.2 * torch.randn(dv, generator=g))
    want = torch.stack([O.hgrn2(z[b, :, :H * dk].double(), z[b, :, H * dk:2 * H * dk].double(), z[b, :, 2 * H * dk:2 * H * dk + H * dv].double(),
                                fb.double(), lo.double(), nw.double(), H, dk, dv, 1e-5)[0] for b in range(B)])
    fbd, lod, nwd = fb.to(DEV), lo.to(DEV), nw.to(DEV)
    ldo = H * dv + 3
    lib = _lib.lib()

    def run(zs, state, zero):
        L = zs.shape[1]
        zd = zs.contiguous().to(DEV)
        out = torch.full((B * L, ldo), 9.0, device=DEV)
        p = Hgrn2Params(q=zd.data_ptr(), f=zd.data_ptr() + 4 * H * dk, v=zd.data_ptr() + 8 * H * dk, ld=ld, f_bias=fbd.data_ptr(), lower=lod.data_ptr(),
                        norm_w=nwd.data_ptr(), eps=1e-5, state=state.data_ptr() if state is not None else None, zero_start=zero, out=out.data_ptr(), ldo=ldo,
                        dtype=1, B=B, L=L, H=H, dk=dk, dv=dv)
        n = lib.evo_hgrn2_workspace(C.byref(p))
        ws = torch.empty(max(n, 1), dtype=torch.uint8, device=DEV)
        check(lib.evo_hgrn2_fwd(C.byref(p), ptr(ws), n, _stream()))
        assert (out[:, H * dv:] == 0).all()
        return out.view(B, L, ldo)[:, :, :H * dv]

    _close(run(z, None, 1), want, 2e-5, "whole")
    state = torch.full((B, H, dk, dv), float("nan"), device=DEV)
    parts, t = [], 0
    for n in (2, 1, 17, 1, 3, 16):
        parts.append(run(z[:, t:t + n], state, 1 if t == 0 else 0))
        t += n
    _close(torch.cat(parts, 1), want, 2e-5, "portions")


def _attn_case(H, G, dk, dv, T, window, keep, maps=2, seed=0, spike=None):
    g = torch.Generator().manual_seed(seed)
    q, k, v = torch.randn(T, H * maps * dk, generator=g), torch.randn(T, G * maps * dk, generator=g), torch.randn(T, G * dv, generator=g)
    gate = torch.randn(T, H * dv, generator=g)
    if spike is not None:                      # (query, key): that key's score dominates both maps of head 0 if it is visible at all
        i, j = spike
        u = torch.randn(dk, generator=g)
        u = u / u.norm()
        for m in range(maps):
            q[i, m * dk:(m + 1) * dk] = 30.0 * u
            k[j, m * dk:(m + 1) * dk] = 30.0 * u * (1.0 if m == 0 else 0.5)
    return q, k, v, gate


def _attn_gpu(q, k, v, gate, H, G, dk, dv, window, keep, lam, diff, portions, dtype=F32, cache_len=None, maps=2):
    """Runs the kernel over the sequence in the given portions through a cache (as the model does); returns (T, H*dv)."""
    T = q.shape[0]
    kw, vw = G * maps * dk, G * dv
    cache = torch.full((1, cache_len or T + 5, kw + vw), float("nan"), dtype=dtype, device=DEV)
    outs, t = [], 0
    lib = _lib.lib()
    esz = 4 if dtype == F32 else 2
    for n in portions:
        z = torch.cat([q[t:t + n], k[t:t + n], v[t:t + n], gate[t:t + n]], 1).to(dtype).to(DEV).contiguous()
        ld = z.shape[1]
        check(lib.evo_copy_rows(C.c_void_p(z.data_ptr() + q.shape[1] * esz), ld, ptr(cache), kw + vw, cache.shape[1] * (kw + vw), 1, n, kw + vw, t, None, int(dtype == F32), _stream()))
        out = torch.full((n, H * dv + 4), 2.0, dtype=dtype, device=DEV)
        p = WindowAttnParams(q=z.data_ptr(), q_tok_stride=ld, k=cache.data_ptr(), v=cache.data_ptr() + kw * esz, k_tok_stride=kw + vw, v_tok_stride=kw + vw,
                             k_batch_stride=0, v_batch_stride=0, gate=z.data_ptr() + (q.shape[1] + kw + vw) * esz, gate_tok_stride=ld, out=out.data_ptr(), ldo=H * dv + 4,
                             dtype=int(dtype == F32), B=1, Lq=n, H=H, G=G, dk=dk, dv=dv, n_maps=maps, q_pos0=t, pos_dev=None, window=window, keep_first=keep,
                             scale=1.0 / math.sqrt(dk), lambda_=lam, head_norm=1, norm_eps=1e-5, out_scale=1.0 - diff)
        check(lib.evo_window_attn_fwd(C.byref(p), _stream()))
        assert (out[:, H * dv:] == 0).all()
        outs.append(out[:, :H * dv].float())
        t += n
    assert t == T
    return torch.cat(outs, 0)


@pytest.mark.parametrize("H,G,dk,dv,window,keep", [(3, 1, 20, 24, 9, 3), (4, 2, 40, 88, 40, 5), (2, 2, 8, 130, 33, 0), (1, 1, 64, 300, 5, 12), (2, 1, 16, 32, 64, 32), (2, 2, 12, 16, 0, 0)])
def test_window_attention_prompt_steps_and_portions(H, G, dk, dv, window, keep):
    T = 90
    q, k, v, gate = _attn_case(H, G, dk, dv, T, window, keep, seed=dk)
    lam, diff = 0.37, 0.2
    want = O.diff_attention(q.double(), k.double(), v.double(), gate.double(), lam, H, G, dk, dv, 1.0 / math.sqrt(dk), window, keep, diff, 1e-5)
    for portions in ([T], [50] + [1] * 40, [2, 3, 30, 1, 4, 41, 2, 7]):
        _close(_attn_gpu(q, k, v, gate, H, G, dk, dv, window, keep, lam, diff, portions), want, 3e-5, f"portions {portions[:4]}")
    # bf16 activations (the tensor-core kernel where the shape allows it): same inputs rounded to bf16 first, so only the
    # kernel's own arithmetic and the bf16 rounding of its output remain
    qb, kb, vb, gb = (_bf(t).float() for t in (q, k, v, gate))
    want_b = O.diff_attention(qb.double(), kb.double(), vb.double(), gb.double(), lam, H, G, dk, dv, 1.0 / math.sqrt(dk), window, keep, diff, 1e-5)
    for portions in ([T], [33, 1, 1, 55], [17, 16, 40, 17]):
        _close(_attn_gpu(qb, kb, vb, gb, H, G, dk, dv, window, keep, lam, diff, portions, dtype=B16), want_b, 6e-3, f"bf16 {portions}")


@pytest.mark.parametrize("mode", ["prompt", "steps", "prompt_bf16", "steps_bf16"])
def test_window_and_kept_token_edges_with_a_dominant_key(mode):
    """One key is given a score far above all others: the output must switch exactly where the mask says -- distance
    window-1 vs window, kept index keep-1 vs keep -- in a prompt and in single-token steps, across tile borders."""
    H, G, dk, dv, window, keep = 1, 1, 16, 32, 37, 6
    lam, diff = 0.0, 0.0
    T = 130
    for i in (36, 37, 64, 65, 100, 129):
        for j in {i - window + 1, i - window, keep - 1, keep, 0, i}:
            if j < 0 or j > i:
                continue
            q, k, v, gate = _attn_case(H, G, dk, dv, T, window, keep, seed=i * 1000 + j, spike=(i, j))
            gate[:] = 30.0                                  # gate -> 1
            want = O.diff_attention(q.double(), k.double(), v.double(), gate.double(), lam, H, G, dk, dv, 1.0 / math.sqrt(dk), window, keep, diff, 1e-5, rows=[i])
            portions = [i] + [1] * (T - i) if mode.startswith("steps") else [T]
            if mode.endswith("bf16"):
                q, k, v, gate = (_bf(t).float() for t in (q, k, v, gate))
                want = O.diff_attention(q.double(), k.double(), v.double(), gate.double(), lam, H, G, dk, dv, 1.0 / math.sqrt(dk), window, keep, diff, 1e-5, rows=[i])
            got = _attn_gpu(q, k, v, gate, H, G, dk, dv, window, keep, lam, diff, portions, dtype=B16 if mode.endswith("bf16") else F32)
            _close(got[i], want[i], 3e-5 if not mode.endswith("bf16") else 6e-3, f"query {i} key {j}")
            seen = O.visible(i, j, window, keep)
            picks = torch.allclose(want[i].float(), (O.rms(v[j].double(), 1e-5)).float(), atol=1e-3) and torch.allclose(got[i].cpu(), O.rms(v[j].double(), 1e-5).float(), atol=2e-2)
            assert picks == seen, (i, j, seen)


@pytest.mark.parametrize("dtype", [F32, B16])
def test_long_window_single_steps(dtype):
    """A window of several hundred keys: the single-token kernel spreads its key tiles over more warps.  One far key, exactly at
    the window's edge for the last query and one past it for the query after, dominates where it is visible."""
    H, G, dk, dv, window, keep = 2, 1, 16, 32, 800, 3
    T, lam, diff = 860, 0.4, 0.25
    i = 840
    q, k, v, gate = _attn_case(H, G, dk, dv, T, window, keep, seed=11, spike=(i, i - window + 1))
    q[i + 1, :2 * dk] = q[i, :2 * dk]                       # the next query asks for the same key, now one step outside
    if dtype == B16:
        q, k, v, gate = (_bf(t).float() for t in (q, k, v, gate))
    rows = list(range(820, T))
    want = O.diff_attention(q.double(), k.double(), v.double(), gate.double(), lam, H, G, dk, dv, 1.0 / math.sqrt(dk), window, keep, diff, 1e-5, rows=rows)
    got = _attn_gpu(q, k, v, gate, H, G, dk, dv, window, keep, lam, diff, [820] + [1] * (T - 820), dtype=dtype)
    _close(got[820:], want[820:], 3e-5 if dtype == F32 else 6e-3, "steps behind a long window")
    assert (want[i, :dv] - want[i + 1, :dv]).abs().max() > 0.1          # the edge shows in the expected values


# ------------------------------------------------------------------ the model
def _model(cfg, W, dtype=F32):
    from evo_b200.zaverax import Zaverax, ZaveraxConfig
    m = Zaverax(ZaveraxConfig.from_dict(cfg), dtype=dtype)
    m.load_state_dict(W)
    return m.to(DEV)


def _portions(model, tokens, sizes, max_seqlen=None, state=None):
    state = state or model.initialize_inference_params(max_seqlen=max_seqlen or len(tokens) + 8, max_batch_size=1)
    outs, t = [], 0
    for n in sizes:
        state["mha"].seqlen_offset = state["hyena"].seqlen_offset = t
        lg, _ = model(torch.tensor([tokens[t:t + n]], device=DEV), inference_params_dict=state)
        outs.append(lg[0])
        t += n
    assert t == len(tokens)
    return torch.cat(outs, 0)


CONFIGS = {
    "mixed": dict(layers=("hgrn2", "attention", "hgrn2"), loop=(1, 3, 2)),
    "loop_from_0": dict(layers=("attention", "hgrn2"), loop=(0, 1, 3), kv_heads=3, window=4, keep_first=0, taps=2, width=72, vocab=257),
    "no_loop_no_ff": dict(layers=("hgrn2", "attention", "attention"), loop=(0, 0, 1), no_ff_layers=(0, 2), heads=2, kv_heads=2, dim=16, vdim=16,
                          r_heads=1, r_dim=16, r_vdim=16, taps=4, residual_mult=1.0, keep_first=20, window=6, diff=0.5, softcap=30.0),
    "wide_heads": dict(layers=("hgrn2", "attention"), r_heads=1, r_dim=136, r_vdim=72, heads=2, kv_heads=1, dim=72, vdim=136, width=200, ff=264, taps=1),
}


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_model_whole_steps_and_portions_match_the_oracle_in_fp32(name):
    cfg = O.make_config(**CONFIGS[name])
    W = O.random_weights(cfg, seed=len(name))
    g = torch.Generator().manual_seed(1)
    T = 75
    tokens = torch.randint(0, cfg["vocab"], (T,), generator=g).tolist()
    streams = []
    want = O.forward(cfg, W, tokens, stream_out=streams)
    model = _model(cfg, W)
    model._tap = []
    got, _ = model(torch.tensor([tokens], device=DEV))
    for r, (a, b) in enumerate(zip(model._tap, streams)):
        _close(a, b, 2e-5, f"{name}: residual stream after run {r}")
    model._tap = None
    _close(got[0], want, 2e-5, f"{name}: whole")
    _close(_portions(model, tokens, [1] * T), want, 2e-5, f"{name}: token by token from the first token")
    _close(_portions(model, tokens, [40] + [1] * 35), want, 2e-5, f"{name}: prompt then steps")
    _close(_portions(model, tokens, [2, 2, 3, 30, 1, 2, 17, 9, 2, 5, 2]), want, 2e-5, f"{name}: portions")


def test_layers_with_their_own_sizes_and_a_cache_that_has_to_grow():
    """Every layer brings its own head counts, head sizes, window and feed-forward width (one has none); the KV cache starts
    smaller than the request and grows while the request runs."""
    cfg = O.make_config(layers=("attention", "hgrn2", "attention", "hgrn2"), loop=(1, 3, 2), width=104, vocab=211, taps=2)
    cfg["layers"][2]["mixer"] = {"heads": 4, "kv_heads": 4, "dim": 8, "vdim": 40, "scale": 0.2, "diff": 0.6, "mask": {"size": 3, "keep_first": 9}}
    cfg["layers"][3]["mixer"] = {"heads": 5, "dim": 24, "vdim": 8}
    cfg["layers"][1]["mlp"] = None
    cfg["layers"][2]["mlp"]["ff"] = 72
    W = O.random_weights(cfg, seed=21)
    tokens = torch.randint(0, cfg["vocab"], (70,), generator=torch.Generator().manual_seed(8)).tolist()
    want = O.forward(cfg, W, tokens)
    model = _model(cfg, W)
    got, _ = model(torch.tensor([tokens], device=DEV))
    _close(got[0], want, 2e-5, "whole")
    state = model.initialize_inference_params(max_seqlen=16, max_batch_size=1)
    _close(_portions(model, tokens, [9, 2, 20, 1, 1, 30, 7], state=state), want, 2e-5, "portions through a growing cache")
    assert all(c.shape[1] >= 70 for c in state["mha"].key_value_memory_dict.values())


def test_model_bf16_stays_within_rounding_of_the_oracle_and_of_itself():
    cfg = O.make_config(**CONFIGS["mixed"])
    W = O.random_weights(cfg, seed=3)
    tokens = torch.randint(0, cfg["vocab"], (90,), generator=torch.Generator().manual_seed(2)).tolist()
    want = O.forward(cfg, W, tokens)
    model = _model(cfg, W, B16)
    whole, _ = model(torch.tensor([tokens], device=DEV))
    cut = _portions(model, tokens, [50, 2, 1, 1, 30, 6])
    rel = lambda a, b: ((a.double().cpu() - b.double().cpu()).pow(2).mean().sqrt() / b.double().pow(2).mean().sqrt()).item()
    assert rel(whole[0], want) < 2e-2
    assert rel(cut, want) < 2e-2
    assert rel(cut, whole[0].cpu()) < 2e-2
    model.gemm_path = "simt"                              # the tensor-core linear layers against the CUDA-core ones
    simt, _ = model(torch.tensor([tokens], device=DEV))
    assert rel(simt[0], whole[0].cpu()) < 1e-2


def test_batch_rows_equal_each_sequence_alone_and_wanted_rows_select():
    cfg = O.make_config(**CONFIGS["mixed"])
    W = O.random_weights(cfg, seed=5)
    model = _model(cfg, W)
    ids = torch.randint(0, cfg["vocab"], (3, 33), generator=torch.Generator().manual_seed(4)).to(DEV)
    both, _ = model(ids)
    for b in range(3):
        alone, _ = model(ids[b:b + 1])
        _close(both[b], alone[0].double().cpu(), 1e-6, f"row {b}")
    state = model.initialize_inference_params(max_seqlen=64, max_batch_size=3)
    a, _ = model(ids[:, :20], inference_params_dict=state)
    state["mha"].seqlen_offset = 20
    b_, _ = model(ids[:, 20:], inference_params_dict=state)
    _close(torch.cat([a, b_], 1), both.double().cpu(), 1e-5, "batched portions")
    rows = [0, 7, 32, 40, 98]
    picked, _ = model(ids, logits_rows=rows)
    _close(picked, both.reshape(-1, both.shape[-1])[rows].double().cpu(), 1e-6, "wanted rows")


def test_reused_cache_memory_and_long_decoding_past_the_window():
    """A cache that still holds another request's keys (and NaNs beyond) serves a new request; decoding runs far past the window
    and the kept tokens; a request interleaved with another one keeps its own state."""
    cfg = O.make_config(**dict(CONFIGS["mixed"], window=11, keep_first=4))
    W = O.random_weights(cfg, seed=7)
    model = _model(cfg, W)
    g = torch.Generator().manual_seed(6)
    a = torch.randint(0, cfg["vocab"], (120,), generator=g).tolist()
    b = torch.randint(0, cfg["vocab"], (60,), generator=g).tolist()
    want_a, want_b = O.forward(cfg, W, a), O.forward(cfg, W, b)
    state = model.initialize_inference_params(max_seqlen=128, max_batch_size=1)
    _close(_portions(model, a, [20] + [1] * 100, state=state), want_a, 2e-5, "long decoding")
    for cache in state["mha"].key_value_memory_dict.values():
        cache[:, 100:] = float("nan")
    reused = model.initialize_inference_params(max_seqlen=128, max_batch_size=1)
    reused["mha"].key_value_memory_dict = state["mha"].key_value_memory_dict           # same memory, stale contents
    _close(_portions(model, b, [7, 2, 51], state=reused), want_b, 2e-5, "reused cache memory")
    sa = model.initialize_inference_params(max_seqlen=128, max_batch_size=1)
    sb = model.initialize_inference_params(max_seqlen=128, max_batch_size=1)
    outs_a, outs_b = [], []
    for lo, hi in ((0, 30), (30, 31), (31, 60)):
        for tokens, st, outs in ((a, sa, outs_a), (b, sb, outs_b)):
            st["mha"].seqlen_offset = lo
            lg, _ = model(torch.tensor([tokens[lo:hi]], device=DEV), inference_params_dict=st)
            outs.append(lg[0])
    _close(torch.cat(outs_a), want_a[:60], 2e-5, "interleaved a")
    _close(torch.cat(outs_b), want_b[:60], 2e-5, "interleaved b")


@pytest.mark.parametrize("device_loop", [True, False])
def test_greedy_generation_through_the_generator(device_loop):
    from evo_b200 import CharLevelTokenizer, Generator
    cfg = O.make_config(**dict(CONFIGS["mixed"], vocab=512))
    W = O.random_weights(cfg, seed=11)
    model = _model(cfg, W)
    gen = Generator(model, CharLevelTokenizer(512), top_k=1, top_p=1.0, temperature=1.0)
    gen.device_loop = device_loop
    prompt = torch.randint(0, 512, (1, 21), generator=torch.Generator().manual_seed(8)).to(DEV)
    n_new = 24
    picked, logits, _ = gen.generate(DEV, input_ids=prompt, num_tokens=n_new, cached_generation=True, force_prompt_threshold=64, print_generation=False, stop_at_eos=False)
    assert picked.shape == (1, n_new) and logits.shape == (1, n_new, 512)
    full = prompt[0].tolist() + picked[0].tolist()
    want = O.forward(cfg, W, full)
    for s in range(n_new):                                    # each picked token is (within rounding) the oracle's argmax given the same prefix
        row = want[len(full) - n_new - 1 + s]
        assert row[picked[0, s]] >= row.max() - 2e-2, s
        _close(logits[0, s], row, 2e-5 if not device_loop else 1e-2, f"kept logits {s}")     # the device loop keeps the sampler's bf16 view of the logits


def test_command_line_generates_from_a_checkpoint_folder(tmp_path, capsys):
    """scripts/generate.py --model-dir: config.json picks the model class, the streaming loader fills it, generate() runs greedy."""
    from tests.test_zaverax_host import _write_checkpoint
    from scripts import generate as cli
    cfg = O.make_config(**dict(CONFIGS["mixed"], vocab=512))
    W = O.random_weights(cfg, seed=13)
    _write_checkpoint(str(tmp_path / "ckpt"), cfg, W)
    texts, scores = cli.main(["--model-dir", str(tmp_path / "ckpt"), "--prompt", "ACGTTGCA", "--n-samples", "2", "--n-tokens", "9", "--top-k", "1", "--device", DEV, "--verbose", "0"])
    assert len(texts) == 2 and texts[0] == texts[1] and len(scores) == 2
    ids = [ord(c) for c in "ACGTTGCA"]
    want = O.forward(cfg, W, ids)
    model = _model(cfg, W, B16)
    first, _ = model(torch.tensor([ids], device=DEV))
    assert first[0, -1].argmax().item() == want[-1].argmax().item() or want[-1].max() - want[-1][first[0, -1].argmax().item()] < 0.1
