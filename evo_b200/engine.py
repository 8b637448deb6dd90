"""Launch helpers shared by the model classes: the current stream, optional per-kernel event records, and the two tensor-core
linear-layer launchers (evo_gemm for many rows, evo_gemm_smallm for the few rows of a decode step).  A model class mixes this in and
provides `gemm_variant`, `gemm_variant_gate`, `_prof`, `_smallm_ws` and `_decode` (see StripedHyena.__init__)."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import EPI_GELU_GATE, EPI_HYENA_STEP, GemmParams, GemmSmallMParams, check


class KernelOps:
    @staticmethod
    def _stream():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def _record(self, kind, work, launch):
        """Run `launch()`; when profiling is on, bracket it with CUDA events on the launch stream."""
        if self._prof is None:
            return launch()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        launch()
        e1.record()
        self._prof.append((kind, work, e0, e1))

    def _gemm(self, a, w, out, M, N, K, epi, bias=None, resid=None, ldc=None, variant=None, rope=None, peers=None):
        """rope = (cos_ptr, sin_ptr, tokens_per_sequence, rotated_columns) for EPI_BIAS_ROPE;
        peers = (ctypes array of peer pointers, n, period, inner, row0): peer-scattered output (see evo_gemm_params), out may be None."""
        if variant is None:
            variant = self.gemm_variant_gate if epi == EPI_GELU_GATE else self.gemm_variant
        p = GemmParams(A=a.data_ptr(), lda=K, W=w.data_ptr(), C=out.data_ptr() if out is not None else None, ldc=ldc or N,
                       bias=bias.data_ptr() if bias is not None else None,
                       residual=resid.data_ptr() if resid is not None else None, ldr=ldc or N,
                       M=M, N=N, K=K, epilogue=epi, variant=variant)
        if rope is not None:
            p.rope_cos, p.rope_sin, p.rope_L, p.rope_cols = rope
        if peers is not None:
            arr, n, period, inner, row0 = peers
            p.c_peers, p.n_c_peers, p.peer_period, p.peer_inner, p.peer_row0 = C.cast(arr, C.c_void_p), n, period, inner, row0
        self._record(f"gemm/{N}x{K}/e{epi}/v{variant}", 2.0 * M * N * K, lambda: check(_lib.lib().evo_gemm(C.byref(p), self._stream()), "evo_gemm"))

    def _gemm_smallm(self, a, w, out, M, N, K, epi, bias=None, resid=None, step=None):
        """Decode-step linear layer (M <= 64): stream-K weight-streaming kernel, gate epilogue fused.
        step = (fir_state, state_real, filter module) for EPI_HYENA_STEP: the in-projection with the operator's decode step
        in its epilogue (out is then y (M, N/3))."""
        lib = _lib.lib()
        need = lib.evo_gemm_smallm_workspace(M, N, K, epi)
        ws = self._smallm_ws
        if ws is None or ws.numel() < need or ws.device != a.device:
            self._decode = None      # a captured decode graph holds the old workspace address
            ws = self._smallm_ws = torch.zeros(max(need, lib.evo_gemm_smallm_workspace(M, 256, 64, EPI_GELU_GATE), lib.evo_gemm_smallm_workspace(M, 384, 64, EPI_HYENA_STEP)),
                                               dtype=torch.uint8, device=a.device)
        n_out = N // 2 if epi == EPI_GELU_GATE else (N // 3 if epi == EPI_HYENA_STEP else N)
        p = GemmSmallMParams(A=a.data_ptr(), lda=K, W=w.data_ptr(), C=out.data_ptr(), ldc=n_out,
                             bias=bias.data_ptr() if bias is not None else None,
                             residual=resid.data_ptr() if resid is not None else None, ldr=n_out,
                             M=M, N=N, K=K, epilogue=epi, workspace=ws.data_ptr(), workspace_bytes=ws.numel())
        if step is not None:
            fs, st, f = step
            p.fir_state, p.state = fs.data_ptr(), st.data_ptr()
            p.fir_w, p.fir_b, p.Dskip = f.short_filter_weight.data_ptr(), f.short_filter_bias.data_ptr(), f.D.data_ptr()
            p.poles, p.residues = f.poles.data_ptr(), f.residues.data_ptr()
        self._record(f"gemm/{N}x{K}/e{epi}/streamk", 2.0 * M * N * K, lambda: check(lib.evo_gemm_smallm(C.byref(p), self._stream()), "evo_gemm_smallm"))
