"""Mechanisms of the decoder-only language-model path, as parameter holders that describe themselves to the kernels.

Beside ``layers.py`` (Dia's RMSNorm / rotary attention / gated MLP modules) this file adds
  * :class:`DynamicTanh` - a norm without statistics, ``tanh(alpha x) w + b``;
  * :class:`TapMix` - a causal per-channel short convolution over time added to its input, with a per-sequence tail;
  * :class:`SinkAttention` - grouped-query softmax attention whose values are the projected keys, with whole-projection
    q / k RMS norms, per-head temperature, tanh score cap, linear distance bias, a sliding window that keeps the first
    tokens, and a value-less sink logit in the denominator;
  * :class:`RoutedExperts` - sigmoid-scored top-k mixture of gated units whose score multiplies the expert's INPUT,
    plus an optional shared unit.
  * :class:`LayerNorm` - mean / variance norm with weight and bias;
  * :class:`TalkingAttention` - grouped-query softmax attention with biased projections, per-head q / k RMS norms, rotary
    positions on the leading channels of every head (interleaved pairs, optional wavelength-band rescaling), scores
    mixed across heads before the softmax, a value-less sink logit and a per-head sigmoid output gate;
  * :class:`Hgrn2` - gated linear recurrence whose forget gate (with a learned lower bound) also sets the write strength;
  * :class:`ChannelDelta` - gated delta rule with a decay per head and key channel, short causal convolutions on q, k, v,
    unit-vector q and k, and a low-rank sigmoid output gate;
  * :class:`DenseXielu` - up projection, xIELU activation, down projection.
All constants are constructor arguments; a design picks and combines them per layer (:class:`MixLayer` runs its
sublayers one after the other, :class:`ParallelLayer` feeds one norm to mixer and feed-forward and adds both).  The
arithmetic lives in ``csrc/lm_kernels.cu`` and ``csrc/lm_mixers.cu``; these classes only keep device tensors alive and
fill ``lm_b200_layer``.
"""

from __future__ import annotations

import math

import torch

from .lm_state import StateSpec


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

    def state_spec(self) -> StateSpec:
        return StateSpec(kv=(self.mixer.kv_heads, self.mixer.dim, self.mixer.dim), tap_tails=2)

    def fill(self, rec, st) -> None:
        from ._lm_lib import FF_NONE, FF_ROUTED_EXPERTS, MIXER_SINK_ATTENTION
        k_pages, v_pages, (tail_mix, tail_ff) = st.k_pages, st.v_pages, st.tails
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


# ---- the parallel form ------------------------------------------------------------------------------------------------
class LayerNorm:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor, device):
        self.w, self.b = _f32(weight, device), _f32(bias, device)

    def fill(self, rec) -> None:
        from ._lm_lib import NORM_LAYER
        rec.w, rec.b, rec.alpha, rec.kind = self.w.data_ptr(), self.b.data_ptr(), 0.0, NORM_LAYER


def rotary_angles(base: float, dims: int, scaling=None) -> torch.Tensor:
    """Angle per position of each of the ``dims / 2`` rotary pairs: ``base^(-2i/dims)``.  ``scaling`` (factor, low, high,
    original) stretches long waves: a pair whose wavelength exceeds ``original / low`` turns ``factor`` times slower, one
    below ``original / high`` is kept, and in between the two rates are blended linearly in ``original / wavelength``."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, orig = (float(getattr(scaling, k)) for k in ("factor", "low", "high", "original"))
            turns = orig * f / (2.0 * math.pi)                    # original / wavelength
            if turns < low:
                f = f / factor
            elif turns <= high:
                t = (turns - low) / (high - low)
                f = (1.0 - t) * f / factor + t * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


class TalkingAttention:
    kind = "talk_attention"

    def __init__(self, w_q, w_k, w_v, w_o, q_norm, k_norm, *, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                 b_q=None, b_k=None, b_v=None, w_gate=None, talk=None, sink=None, rot_angles=None, device=None):
        self.heads, self.kv_heads, self.dim, self.vdim, self.scale = int(heads), int(kv_heads), int(dim), int(vdim), float(scale)
        if tuple(w_q.shape)[0] != heads * dim or tuple(w_k.shape)[0] != kv_heads * dim or tuple(w_v.shape)[0] != kv_heads * vdim:
            raise ValueError("projection shapes do not match heads x dim")
        zeros = lambda n: torch.zeros(n, dtype=torch.float32)    # noqa: E731
        gate_bias = zeros(heads)
        if w_gate is None:                                        # no gate: zero rows with a bias whose sigmoid is 1.0f
            w_gate, gate_bias = torch.zeros((heads, w_q.shape[1]), dtype=w_q.dtype), torch.full((heads,), 40.0)
        self.in_rows = [w_q, w_k, w_v, w_gate]
        self.in_bias = [b if b is not None else zeros(w.shape[0]) for b, w in ((b_q, w_q), (b_k, w_k), (b_v, w_v))] + [gate_bias]
        self.has_bias = any(b is not None for b in (b_q, b_k, b_v)) or bool(gate_bias.any())
        self.w_o = w_o
        self.q_norm, self.k_norm = _f32(q_norm, device), _f32(k_norm, device)
        self.talk = None if talk is None else _f32(talk, device)
        self.sink = None if sink is None else _f32(sink, device)
        self.rot = None if rot_angles is None or rot_angles.numel() == 0 else _f32(rot_angles, device)

    def out_columns(self) -> int:
        return self.heads * self.vdim

    def state_spec(self) -> StateSpec:
        return StateSpec(kv=(self.kv_heads, self.dim, self.vdim))

    def fill(self, rec, st) -> None:
        from ._lm_lib import MIXER_TALK_ATTENTION
        rec.mixer = MIXER_TALK_ATTENTION
        rec.heads, rec.kv_heads, rec.dim, rec.vdim, rec.scale = self.heads, self.kv_heads, self.dim, self.vdim, self.scale
        rec.q_norm, rec.k_norm = self.q_norm.data_ptr(), self.k_norm.data_ptr()
        rec.talk = self.talk.data_ptr() if self.talk is not None else None
        rec.sink = self.sink.data_ptr() if self.sink is not None else None
        rec.rot_dims = 2 * self.rot.numel() if self.rot is not None else 0
        rec.rot_freq = self.rot.data_ptr() if self.rot is not None else None
        rec.k_pages, rec.v_pages = st.k_pages.data_ptr(), st.v_pages.data_ptr()


class Hgrn2:
    kind = "hgrn2"

    def __init__(self, w_q, w_f, w_v, w_o, head_norm, *, heads: int, dim: int, vdim: int, b_f=None, lower=None, device=None):
        self.heads, self.dim, self.vdim = int(heads), int(dim), int(vdim)
        if tuple(w_q.shape)[0] != heads * dim or tuple(w_f.shape)[0] != heads * dim or tuple(w_v.shape)[0] != heads * vdim:
            raise ValueError("projection shapes do not match heads x dim")
        self.in_rows = [w_q, w_f, w_v]
        zeros = lambda n: torch.zeros(n, dtype=torch.float32)    # noqa: E731
        self.in_bias = [zeros(heads * dim), b_f if b_f is not None else zeros(heads * dim), zeros(heads * vdim)]
        self.has_bias = b_f is not None
        self.w_o = w_o
        self.head_norm = _f32(head_norm, device)
        self.lower = None if lower is None else _f32(lower, device)

    def out_columns(self) -> int:
        return self.heads * self.vdim

    def state_spec(self) -> StateSpec:
        return StateSpec(recurrent=(self.heads, self.vdim, self.dim))

    def fill(self, rec, st) -> None:
        from ._lm_lib import MIXER_HGRN2
        rec.mixer = MIXER_HGRN2
        rec.heads, rec.kv_heads, rec.dim, rec.vdim = self.heads, self.heads, self.dim, self.vdim
        rec.head_norm = self.head_norm.data_ptr()
        rec.lower = self.lower.data_ptr() if self.lower is not None else None
        rec.rec_state = st.rec_state.data_ptr()


class ChannelDelta:
    kind = "channel_delta"

    def __init__(self, w_q, w_k, w_v, w_beta, w_a1, w_a2, w_g1, w_g2, w_o, conv_q, conv_k, conv_v, a_log, dt_bias, head_norm, *,
                 heads: int, kv_heads: int, dim: int, vdim: int, unit_eps: float = 1e-6, device=None):
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        if tuple(w_q.shape)[0] != kv_heads * dim or tuple(w_k.shape)[0] != kv_heads * dim or tuple(w_v.shape)[0] != heads * vdim:
            raise ValueError("projection shapes do not match heads x dim")
        self.taps = int(conv_q.shape[1])
        self.rank_a, self.rank_g = int(w_a1.shape[0]), int(w_g1.shape[0])
        if tuple(w_a2.shape) != (heads * dim, self.rank_a) or tuple(w_g2.shape) != (heads * vdim, self.rank_g):
            raise ValueError("the second steps of the decay / gate projections do not match heads x dim / heads x vdim")
        self.in_rows = [w_q, w_k, w_v, w_beta, w_a1, w_g1]
        self.in_bias, self.has_bias = None, False
        self.w_o = w_o
        self.conv_w = _f32(torch.cat([conv_q, conv_k, conv_v], dim=0), device)
        self.a_log, self.dt_bias = _f32(a_log, device), _f32(dt_bias, device)
        self.w_a2, self.w_g2 = _bf16(w_a2, device), _bf16(w_g2, device)
        self.head_norm = _f32(head_norm, device)
        self.unit_eps = float(unit_eps)

    def out_columns(self) -> int:
        return self.heads * self.vdim

    def state_spec(self) -> StateSpec:
        return StateSpec(recurrent=(self.heads, self.vdim, self.dim),
                         conv=(self.taps, 2 * self.kv_heads * self.dim + self.heads * self.vdim))

    def fill(self, rec, st) -> None:
        from ._lm_lib import MIXER_CHANNEL_DELTA
        rec.mixer = MIXER_CHANNEL_DELTA
        rec.heads, rec.kv_heads, rec.dim, rec.vdim = self.heads, self.kv_heads, self.dim, self.vdim
        rec.conv_taps, rec.rank_a, rec.rank_g, rec.unit_eps = self.taps, self.rank_a, self.rank_g, self.unit_eps
        rec.conv_w, rec.a_log, rec.dt_bias = self.conv_w.data_ptr(), self.a_log.data_ptr(), self.dt_bias.data_ptr()
        rec.w_a2, rec.w_g2, rec.head_norm = self.w_a2.data_ptr(), self.w_g2.data_ptr(), self.head_norm.data_ptr()
        rec.rec_state, rec.conv_tail = st.rec_state.data_ptr(), st.conv_tail.data_ptr()


def _softplus(z: float) -> float:
    return z if z > 30.0 else math.log1p(math.exp(z))


class DenseXielu:
    def __init__(self, w_up, w_down, act):
        """``act``: the two raw numbers (p, q) of the activation; z > 0: softplus(p) z^2 + z / 2, z <= 0:
        (1/2 + softplus(q)) (e^z - 1 - z) + z / 2."""
        self.w_up, self.w_down, self.ff = w_up, w_down, int(w_up.shape[0])
        p, q = (float(v) for v in act.detach().to(torch.float64).reshape(-1)[:2])
        self.act_p, self.act_q = _softplus(p), 0.5 + _softplus(q)


class ParallelLayer:
    """h = norm(x);  x += mixer(h) + ff(h).  Every projection that reads h is one stacked matrix, and the mixer's output
    projection stands beside the feed-forward's down projection in one matrix, so a layer is two products around its
    mixer kernels."""

    def __init__(self, norm: LayerNorm, mixer, ff: DenseXielu | None, device):
        self.norm, self.mixer, self.ff = norm, mixer, ff
        rows = [_bf16(r, device) for r in list(mixer.in_rows) + ([ff.w_up] if ff is not None else [])]
        n = sum(int(r.shape[0]) for r in rows)
        self.n_in = (n + 3) & ~3
        width = int(rows[0].shape[1])
        if self.n_in > n:
            rows.append(torch.zeros((self.n_in - n, width), dtype=torch.bfloat16, device=device))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.in_bias = None
        if mixer.has_bias:
            b = torch.cat([_f32(x, device).reshape(-1) for x in mixer.in_bias])
            self.in_bias = torch.cat([b, torch.zeros(self.n_in - b.numel(), dtype=torch.float32, device=device)]).contiguous()
        outs = [_bf16(o, device) for o in [mixer.w_o] + ([ff.w_down] if ff is not None else [])]
        self.w_out = torch.cat(outs, dim=1).contiguous()
        self.k_out = int(self.w_out.shape[1])

    def state_spec(self) -> StateSpec:
        return self.mixer.state_spec()

    def fill(self, rec, st) -> None:
        from ._lm_lib import ACT_XIELU, FF_DENSE, FF_NONE, FORM_PARALLEL
        rec.form = FORM_PARALLEL
        self.norm.fill(rec.norm_mix_in)
        self.mixer.fill(rec, st)
        rec.n_in, rec.k_out = self.n_in, self.k_out
        rec.w_in, rec.w_out = self.w_in.data_ptr(), self.w_out.data_ptr()
        rec.in_bias = self.in_bias.data_ptr() if self.in_bias is not None else None
        rec.ff = FF_NONE
        if self.ff is not None:
            rec.ff, rec.dense_ff, rec.act = FF_DENSE, self.ff.ff, ACT_XIELU
            rec.act_p, rec.act_q = self.ff.act_p, self.ff.act_q


class LayerRun:
    """One execution of a layer: the layer's weights with a state of its own, and optionally the input mix
    ``x <- W [x; embedding output]`` in front of it (the first layer of a pass over a repeated block)."""

    def __init__(self, layer, pre: torch.Tensor | None = None, device=None):
        self.layer = layer
        self.pre = None if pre is None else _bf16(pre, device)
        self.mixer, self.ff = layer.mixer, layer.ff

    def state_spec(self) -> StateSpec:
        return self.layer.state_spec()

    def fill(self, rec, st) -> None:
        self.layer.fill(rec, st)
        rec.w_pre = self.pre.data_ptr() if self.pre is not None else None
