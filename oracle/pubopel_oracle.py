"""Plain, slow restatement of the Pubopel decoder-only language model (test infrastructure only).

Torch on the CPU, one function per mechanism, whole sequences at once and no cache: every position is
recomputed from the start of its sequence.  Nothing here is imported by the product path and nothing of
the product path is imported here.  ``dtype`` is the arithmetic type (float64 gives a reference whose
own rounding is negligible).

Notation: ``x[t]`` is the residual stream at position t (positions count from 0), ``W`` matrices are
``[out, in]`` and applied as ``W @ x``; a weight dictionary maps the checkpoint's tensor names
(``l<i>.mix.q``, ``l<i>.mlp.e<j>.gate`` ...) to tensors.
"""

from __future__ import annotations

import math

import torch


def dynamic_tanh(x, w, b, alpha):
    """y = tanh(alpha * x) * w + b  (elementwise; no mean, no variance)."""
    return torch.tanh(alpha * x) * w + b


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def causal_tap_mix(h, w):
    """h[t] + sum_j w[:, j] * h[t - (taps - 1) + j], rows before the start count as zero.  h: [T, D], w: [D, taps]."""
    T, D = h.shape
    taps = w.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] = out[t] + w[:, j] * h[s]
    return out


def visible(i, j, size, keep_first):
    """Query position i sees key position j."""
    return j <= i and (i - j < size or j < keep_first)


def sink_attention(h, p, m, eps):
    """The attention mixer on its input rows h [T, D].  p: the layer's 'mix.*' tensors by short name, m: its sizes."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    size = m["mask"]["size"] if m.get("mask") else None
    keep = (m["mask"].get("keep_first") or 0) if m.get("mask") else 0
    cap = m.get("softcap")
    q = h @ p["q"].T                                    # [T, H*d]
    k = h @ p["k"].T                                    # [T, G*d]
    v = k.clone()                                       # the values are the projected keys, before their norm
    q = rms_unit(q, eps) * p["q.norm"]
    k = rms_unit(k, eps) * p["k.norm"]
    q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, d)
    out = torch.zeros(T, H, d, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        slope = 2.0 ** (-8.0 * (hh + 1) / H)
        for i in range(T):
            js = [j for j in range(i + 1) if size is None or visible(i, j, size, keep)]
            s = torch.stack([q[i, hh] @ k[j, g] for j in js]) * m["scale"] * p["temp"][hh]
            if cap:
                s = cap * torch.tanh(s / cap)
            s = s - slope * torch.tensor([float(i - j) for j in js], dtype=h.dtype)
            mx = torch.maximum(s.max(), p["sink"][hh])
            e = torch.exp(s - mx)
            den = e.sum() + torch.exp(p["sink"][hh] - mx)       # the sink: one more term, no key, no value
            w = e / den
            out[i, hh] = (w[:, None] * torch.stack([v[j, g] for j in js])).sum(dim=0)
    return out.reshape(T, H * d) @ p["o"].T


def gated_unit(h, gate, up, down):
    """down @ (silu(gate @ h) * (up @ h)) for rows h [T, D]."""
    a = h @ gate.T
    return ((a * torch.sigmoid(a)) * (h @ up.T)) @ down.T


def routed_experts(h, p, mlp):
    """Sigmoid-scored mixture: every row goes through its ``top`` best experts, each fed score * row, plus the shared unit."""
    T = h.shape[0]
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = torch.sigmoid(h.to(torch.float32) @ p["router"].to(torch.float32).T).to(h.dtype)      # [T, E]
    out = torch.zeros_like(h)
    for t in range(T):
        best = torch.topk(s[t], top).indices.tolist()
        for e in best:
            out[t] = out[t] + gated_unit((s[t, e] * h[t])[None, :], p[f"e{e}.gate"], p[f"e{e}.up"], p[f"e{e}.down"])[0]
    if mlp.get("shared"):
        out = out + gated_unit(h, p["shared.gate"], p["shared.up"], p["shared.down"])
    return out


def _sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def _norm(weights, name, x):
    return dynamic_tanh(x, weights[name], weights[name + ".b"], weights[name + ".alpha"])


def forward(config, weights, tokens, dtype=torch.float32, keep_layers=False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer if asked)."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    streams = []
    for i, layer in enumerate(config["layers"]):
        L = f"l{i}."
        if layer["type"] != "attention":
            raise ValueError(layer["type"])
        h = causal_tap_mix(_norm(W, L + "norm1", x), W[L + "canon1"])
        x = x + _norm(W, L + "norm1b", sink_attention(h, _sub(W, L + "mix."), layer["mixer"], eps))
        if layer.get("mlp"):
            h = causal_tap_mix(_norm(W, L + "norm2", x), W[L + "canon2"])
            x = x + _norm(W, L + "norm2b", routed_experts(h, _sub(W, L + "mlp."), layer["mlp"]))
        streams.append(x.clone())
    logits = _norm(W, "final.norm", x) @ W["head"].T
    return (logits, torch.stack(streams)) if keep_layers else logits


def random_weights(config, seed, spread=1.0):
    """Random bfloat16-representable weights with the checkpoint's names and shapes, for small test models."""
    g = torch.Generator().manual_seed(seed)
    D, V = config["width"], config["vocab"]
    taps = config["canon"]["taps"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * (s * spread / math.sqrt(i))).to(torch.bfloat16).to(torch.float32)

    def vec(n, mean=0.0, s=1.0):
        return (mean + s * torch.randn(n, generator=g)).to(torch.bfloat16).to(torch.float32)

    w = {"embed": vec(V * D, 0.0, 1.0).reshape(V, D), "head": mat(V, D)}

    def norm(name, alpha):
        w[name] = vec(D, 1.0, 0.1)
        w[name + ".b"] = vec(D, 0.0, 0.05)
        w[name + ".alpha"] = torch.tensor(alpha).to(torch.bfloat16).to(torch.float32)

    norm("final.norm", 0.75)
    for i, layer in enumerate(config["layers"]):
        L = f"l{i}."
        for n, a in (("norm1", 0.6), ("norm2", 0.7), ("norm1b", 1.5), ("norm2b", 1.25)):
            norm(L + n, a)
        w[L + "canon1"] = vec(D * taps, 0.0, 0.3).reshape(D, taps)
        w[L + "canon2"] = vec(D * taps, 0.0, 0.3).reshape(D, taps)
        m = layer["mixer"]
        H, G, d = m["heads"], m["kv_heads"], m["dim"]
        w[L + "mix.q"], w[L + "mix.k"] = mat(H * d, D, 2.0), mat(G * d, D, 2.0)
        w[L + "mix.q.norm"], w[L + "mix.k.norm"] = vec(H * d, 1.0, 0.2), vec(G * d, 1.0, 0.2)
        w[L + "mix.temp"], w[L + "mix.sink"] = vec(H, 1.0, 0.3), vec(H, 0.5, 1.0)
        w[L + "mix.o"] = mat(D, H * m["vdim"])
        mlp = layer.get("mlp")
        if mlp:
            F = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                w[L + f"mlp.e{e}.gate"], w[L + f"mlp.e{e}.up"], w[L + f"mlp.e{e}.down"] = mat(F, D, 2.0), mat(F, D, 2.0), mat(D, F, 2.0)
            w[L + "mlp.router"] = mat(mlp["router"]["experts"], D, 3.0)
            if mlp.get("shared"):
                S = mlp["shared"]["ff"]
                w[L + "mlp.shared.gate"], w[L + "mlp.shared.up"], w[L + "mlp.shared.down"] = mat(S, D, 2.0), mat(S, D, 2.0), mat(D, S, 2.0)
    return w
