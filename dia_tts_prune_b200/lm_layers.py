"""Mechanisms of the decoder-only language-model path, as parameter holders that describe themselves to the kernels.

Beside ``layers.py`` (Dia's RMSNorm / rotary attention / gated MLP modules) this file adds
  * :class:`DynamicTanh` - a norm without statistics, ``tanh(alpha x) w + b``;
  * :class:`TapMix` - a causal per-channel short convolution over time added to its input, with a per-sequence tail;
  * :class:`SinkAttention` - grouped-query softmax attention whose values are the projected keys, with whole-projection
    q / k RMS norms, per-head temperature, tanh score cap, linear distance bias, a sliding window that keeps the first
    tokens, and a value-less sink logit in the denominator;
  * :class:`RoutedExperts` - sigmoid-scored top-k mixture of gated units whose score multiplies the expert's INPUT,
    plus an optional shared unit.
All constants are constructor arguments; a design picks and combines them per layer (:class:`MixLayer`).  The
arithmetic lives in ``csrc/lm_kernels.cu``; these classes only keep device tensors alive and fill ``lm_b200_layer``.
"""

from __future__ import annotations

import torch


def _f32(t: torch.Tensor, device) -> torch.Tensor:
    return t.detach().to(device=device, dtype=torch.float32).contiguous()


def _bf16(t: torch.Tensor, device) -> torch.Tensor:
    return t.detach().to(device=device, dtype=torch.bfloat16).contiguous()


class DynamicTanh:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor, alpha: float, device):
        self.w, self.b, self.alpha = _f32(weight, device), _f32(bias, device), float(alpha)

    def fill(self, rec) -> None:
        rec.w, rec.b, rec.alpha = self.w.data_ptr(), self.b.data_ptr(), self.alpha


class TapMix:
    def __init__(self, taps: torch.Tensor, device):
        """``taps [width, n]``: out_t = h_t + sum_j taps[:, j] * h_(t - n + 1 + j)."""
        self.w = _f32(taps, device)
        self.n = int(taps.shape[1])


class SinkAttention:
    def __init__(self, w_q, w_k, q_norm, k_norm, w_o, *, heads: int, kv_heads: int, dim: int, scale: float,
                 temp=None, slopes=None, sink=None, softcap: float | None = None, window: int | None = None,
                 keep_first: int = 0, device=None):
        self.heads, self.kv_heads, self.dim = int(heads), int(kv_heads), int(dim)
        self.scale, self.softcap = float(scale), float(softcap) if softcap else 0.0
        self.window, self.keep_first = int(window) if window else 0, int(keep_first or 0)
        if tuple(w_q.shape)[0] != heads * dim or tuple(w_k.shape)[0] != kv_heads * dim:
            raise ValueError("projection shapes do not match heads x dim")
        self.w_qk = _bf16(torch.cat([w_q, w_k], dim=0), device)          # one GEMM for both projections
        self.q_norm, self.k_norm = _f32(q_norm, device), _f32(k_norm, device)
        self.temp = None if temp is None else _f32(temp, device)
        self.slopes = None if slopes is None else _f32(slopes, device)
        self.sink = None if sink is None else _f32(sink, device)
        self.w_o = _bf16(w_o, device)


class RoutedExperts:
    def __init__(self, router, gates: list, ups: list, downs: list, *, top: int, shared=None, device=None):
        """``gates[e] / ups[e]: [ff, width]``, ``downs[e]: [width, ff]``; ``shared``: (gate, up, down) or None."""
        self.experts, self.top, self.ff = len(gates), int(top), int(gates[0].shape[0])
        self.w_router = _bf16(router, device)
        self.w_gate_up = _bf16(torch.stack([torch.cat([g, u], dim=0) for g, u in zip(gates, ups)]), device)
        self.w_down = _bf16(torch.stack(list(downs)), device)
        self.shared_ff = 0
        self.ws_gate_up = self.ws_down = None
        if shared is not None:
            g, u, d = shared
            self.shared_ff = int(g.shape[0])
            self.ws_gate_up, self.ws_down = _bf16(torch.cat([g, u], dim=0), device), _bf16(d, device)


class MixLayer:
    """x += norm_out(mixer(tap(norm_in(x))));  x += norm_out'(ff(tap'(norm_in'(x))))  (the second line only with ``ff``)."""

    def __init__(self, mixer: SinkAttention, norm_mix_in: DynamicTanh, norm_mix_out: DynamicTanh, tap_mix: TapMix | None,
                 ff: RoutedExperts | None = None, norm_ff_in: DynamicTanh | None = None,
                 norm_ff_out: DynamicTanh | None = None, tap_ff: TapMix | None = None):
        self.mixer, self.ff = mixer, ff
        self.norm_mix_in, self.norm_mix_out, self.norm_ff_in, self.norm_ff_out = norm_mix_in, norm_mix_out, norm_ff_in, norm_ff_out
        self.tap_mix, self.tap_ff = tap_mix, tap_ff

    def fill(self, rec, k_pages, v_pages, tail_mix, tail_ff) -> None:
        from ._lm_lib import FF_NONE, FF_ROUTED_EXPERTS, MIXER_SINK_ATTENTION
        a = self.mixer
        rec.mixer = MIXER_SINK_ATTENTION
        rec.heads, rec.kv_heads, rec.dim = a.heads, a.kv_heads, a.dim
        rec.window, rec.keep_first, rec.scale, rec.softcap = a.window, a.keep_first, a.scale, a.softcap
        self.norm_mix_in.fill(rec.norm_mix_in)
        self.norm_mix_out.fill(rec.norm_mix_out)
        rec.tap_mix = self.tap_mix.w.data_ptr() if self.tap_mix is not None else None
        rec.w_qk, rec.q_norm, rec.k_norm, rec.w_o = a.w_qk.data_ptr(), a.q_norm.data_ptr(), a.k_norm.data_ptr(), a.w_o.data_ptr()
        rec.temp = a.temp.data_ptr() if a.temp is not None else None
        rec.slopes = a.slopes.data_ptr() if a.slopes is not None else None
        rec.sink = a.sink.data_ptr() if a.sink is not None else None
        rec.k_pages, rec.v_pages = k_pages.data_ptr(), v_pages.data_ptr()
        rec.tail_mix, rec.tail_ff = tail_mix.data_ptr(), tail_ff.data_ptr()
        rec.ff = FF_NONE
        f = self.ff
        if f is not None:
            rec.ff = FF_ROUTED_EXPERTS
            rec.experts, rec.top, rec.expert_ff, rec.shared_ff = f.experts, f.top, f.ff, f.shared_ff
            self.norm_ff_in.fill(rec.norm_ff_in)
            self.norm_ff_out.fill(rec.norm_ff_out)
            rec.tap_ff = self.tap_ff.w.data_ptr() if self.tap_ff is not None else None
            rec.w_router, rec.w_gate_up, rec.w_down = f.w_router.data_ptr(), f.w_gate_up.data_ptr(), f.w_down.data_ptr()
            if f.shared_ff:
                rec.ws_gate_up, rec.ws_down = f.ws_gate_up.data_ptr(), f.ws_down.data_ptr()
