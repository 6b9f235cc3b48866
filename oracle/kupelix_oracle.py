"""Plain, slow restatement of the Kupelix decoder-only language model (test infrastructure only).

Torch on the CPU, one function per mechanism, whole sequences at once, no cache and no carried state: every
position is recomputed from the start of its sequence, recurrences are explicit loops over time.  Nothing here is
imported by the product path and nothing of the product path is imported here.  The arithmetic type is the type of
the tensors handed in (float64 gives a reference whose own rounding is negligible).

Notation: ``x[t]`` is the residual stream at position t (positions count from 0); matrices are ``[out, in]`` and
applied as ``W @ x``; ``p`` maps the short tensor names of one mixer (``q``, ``k.conv``, ``f.b`` ...) to tensors and
``m`` is the mixer's size dictionary from the configuration.
"""

from __future__ import annotations

import math

import torch


# ---- elementwise pieces ---------------------------------------------------------------------------------------------
def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b over the last axis, var = mean of squared deviations."""
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    return d / torch.sqrt((d * d).mean(dim=-1, keepdim=True) + eps) * w + b


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z / 2."""
    ap, an = softplus(p), 0.5 + softplus(q)
    pos = ap * z * z + 0.5 * z
    neg = an * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def causal_conv(u, w):
    """out[t, c] = sum_j w[c, j] * u[t - (taps - 1) + j, c]; rows before the start are zero.  u [T, C], w [C, taps]."""
    T, _ = u.shape
    taps = w.shape[1]
    out = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] = out[t] + w[:, j] * u[s]
    return out


# ---- rotary positions -------------------------------------------------------------------------------------------------
def rotary_frequencies(rot, dtype=torch.float64):
    """f_i = base^(-2 i / dims), i < dims / 2, rescaled by wavelength bands when ``rot['scaling']`` is given:
    short waves keep f, long waves use f / factor, the band between is blended linearly in original / wavelength."""
    dims = int(rot["dims"])
    f = [float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = []
        for fi in f:
            wave = 2.0 * math.pi / fi
            if wave < orig / high:
                out.append(fi)
            elif wave > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wave - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = out
    return torch.tensor(f, dtype=dtype)


def rotate_interleaved(x, pos, freqs):
    """x [T, heads, dim]: the pair (x[2i], x[2i+1]) of the first 2 * len(freqs) channels turns by pos * f_i."""
    n = freqs.shape[0]
    ang = pos.to(freqs.dtype)[:, None] * freqs[None, :]               # [T, n]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out[..., 0:2 * n:2] = a * c - b * s
    out[..., 1:2 * n:2] = b * c + a * s
    return out


# ---- mixers -----------------------------------------------------------------------------------------------------------
def talking_attention(h, p, m, eps):
    """Grouped-query softmax attention with biased projections, per-head q / k RMS norm, partial interleaved rotary
    positions, scores mixed across heads before the softmax, a value-less sink in the denominator and a per-head
    sigmoid output gate.  h [T, D]."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T + p["q.b"]).reshape(T, H, d)
    k = (h @ p["k"].T + p["k.b"]).reshape(T, G, d)
    v = (h @ p["v"].T + p["v.b"]).reshape(T, G, dv)
    q = rms_unit(q, eps) * p["q.norm"]
    k = rms_unit(k, eps) * p["k.norm"]
    if m.get("rot"):
        fr = rotary_frequencies(m["rot"], h.dtype)
        pos = torch.arange(T)
        q, k = rotate_interleaved(q, pos, fr), rotate_interleaved(k, pos, fr)
    rep = H // G
    raw = torch.stack([q[:, g_] @ k[:, g_ // rep].T for g_ in range(H)]) * m["scale"]       # [H, T, T]
    mixed = torch.einsum("hg,gij->hij", p["talk"], raw)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for i in range(T):
        for hh in range(H):
            s = mixed[hh, i, :i + 1]
            top = torch.maximum(s.max(), p["sink"][hh])
            w = torch.exp(s - top)
            den = w.sum() + torch.exp(p["sink"][hh] - top)
            out[i, hh] = (w[:, None] * v[:i + 1, hh // rep]).sum(0) / den
    gate = torch.sigmoid(h @ p["g"].T)                                                     # [T, H]
    out = out * gate[:, :, None]
    return out.reshape(T, H * dv) @ p["o"].T


def hgrn2(h, p, m, eps):
    """Gated linear recurrence whose forget gate also sets the write strength.  Per head, S [dim, vdim] from zero:
    S <- diag(f_t) S + (1 - f_t) v_t^T;  o_t = S^T q_t;  then RMS norm of o_t over vdim and the output projection."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ p["q"].T).reshape(T, H, d)
    v = (h @ p["v"].T).reshape(T, H, dv)
    low = p["lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ p["f"].T + p["f.b"])).reshape(T, H, d)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_unit(o, eps) * p["norm"]
    return o.reshape(T, H * dv) @ p["o"].T


def channel_delta(h, p, m, eps):
    """Gated delta rule with a decay per head and key channel.  q, k, v pass a short causal convolution and silu; q, k
    become unit vectors per head (q also times dim^-1/2).  Per head, S [dim, vdim] from zero:
    S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ p["q"].T, p["q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(h @ p["k"].T, p["k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(h @ p["v"].T, p["v.conv"])).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ p["b"].T)                                                     # [T, H]
    step = softplus((h @ p["a1"].T) @ p["a2"].T + p["dt_bias"]).reshape(T, H, d)
    g = torch.exp(-torch.exp(p["A_log"])[None, :, None] * step)                            # [T, H, d]
    rep = H // G
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        kt = k[t].repeat_interleave(rep, dim=0)                                             # [H, d]
        qt = q[t].repeat_interleave(rep, dim=0)
        S = g[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, kt))
        S = S + kt[:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, qt)
    gate = torch.sigmoid((h @ p["g1"].T) @ p["g2"].T).reshape(T, H, dv)
    o = rms_unit(o, eps) * p["norm"] * gate
    return o.reshape(T, H * dv) @ p["o"].T


MIXERS = {"attention": talking_attention, "hgrn2": hgrn2, "channel_delta": channel_delta}


def dense_ff(h, p):
    """W_down xielu(W_up h) with the two activation numbers of ``act``."""
    return xielu(h @ p["up"].T, p["act"][0], p["act"][1]) @ p["down"].T


# ---- the model --------------------------------------------------------------------------------------------------------
def layer_runs(cfg):
    """(layer index, starts a pass) in execution order: layers start .. stop-1 repeat ``times`` times in a row."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(a)]
    for _ in range(times):
        runs += [(i, i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


def sub(w, prefix, dtype):
    return {k[len(prefix):]: v.to(dtype) for k, v in w.items() if k.startswith(prefix)}


def forward(cfg, w, tokens, dtype=torch.float64):
    """Logits [T, vocab] and the residual stream after every layer run [runs, T, width] of one whole sequence."""
    eps = float(cfg["norm"]["eps"])
    x0 = w["embed"].to(dtype)[torch.as_tensor(tokens, dtype=torch.long)]
    x, streams = x0.clone(), []
    for i, starts_pass in layer_runs(cfg):
        lc = cfg["layers"][i]
        if starts_pass:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].to(dtype).T
        h = layer_norm(x, w[f"l{i}.norm1"].to(dtype), w[f"l{i}.norm1.b"].to(dtype), eps)
        y = MIXERS[lc["type"]](h, sub(w, f"l{i}.mix.", dtype), lc["mixer"], eps)
        if lc.get("mlp"):
            y = y + dense_ff(h, sub(w, f"l{i}.mlp.", dtype))
        x = x + y
        streams.append(x)
    hN = layer_norm(x, w["final.norm"].to(dtype), w["final.norm.b"].to(dtype), eps)
    return hN @ w["head"].to(dtype).T * float(cfg["logit_scale"]), torch.stack(streams)


def greedy(cfg, w, prompt, n_new, dtype=torch.float64):
    """Greedy continuation by recomputing the whole sequence for every new token; also the logits that chose each token."""
    toks, rows = list(prompt), []
    for _ in range(n_new):
        logits, _ = forward(cfg, w, toks, dtype)
        rows.append(logits[-1])
        toks.append(int(torch.argmax(logits[-1])))
    return toks[len(prompt):], torch.stack(rows)


def random_weights(cfg, seed, spread=1.0):
    """Random bfloat16-representable weights with the checkpoint's names and shapes, for small test models."""
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * (s * spread / math.sqrt(i))).to(torch.bfloat16).to(torch.float32)

    def vec(n, mean=0.0, s=1.0):
        return (mean + s * torch.randn(n, generator=g)).to(torch.bfloat16).to(torch.float32)

    w = {"embed": vec(V * D).reshape(V, D), "head": mat(V, D), "final.norm": vec(D, 1.0, 0.1), "final.norm.b": vec(D, 0.0, 0.05)}
    if cfg.get("loop"):
        w["loop.in"] = mat(D, 2 * D, 1.4)
    for i, lc in enumerate(cfg["layers"]):
        L, m = f"l{i}.", lc["mixer"]
        w[L + "norm1"], w[L + "norm1.b"] = vec(D, 1.0, 0.1), vec(D, 0.0, 0.05)
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        G = m.get("kv_heads") or H
        if lc["type"] == "attention":
            w[L + "mix.q"], w[L + "mix.k"], w[L + "mix.v"] = mat(H * d, D, 2.0), mat(G * d, D, 2.0), mat(G * dv, D)
            w[L + "mix.q.b"], w[L + "mix.k.b"], w[L + "mix.v.b"] = vec(H * d, 0.0, 0.2), vec(G * d, 0.0, 0.2), vec(G * dv, 0.0, 0.2)
            w[L + "mix.q.norm"], w[L + "mix.k.norm"] = vec(d, 1.0, 0.2), vec(d, 1.0, 0.2)
            w[L + "mix.talk"] = (torch.eye(H) + 0.4 * torch.randn(H, H, generator=g) / math.sqrt(H)).to(torch.bfloat16).to(torch.float32)
            w[L + "mix.sink"], w[L + "mix.g"] = vec(H, 0.5, 1.0), mat(H, D, 2.0)
            w[L + "mix.o"] = mat(D, H * dv)
        elif lc["type"] == "hgrn2":
            w[L + "mix.q"], w[L + "mix.f"], w[L + "mix.v"] = mat(H * d, D, 2.0), mat(H * d, D, 2.0), mat(H * dv, D)
            w[L + "mix.f.b"] = vec(H * d, 1.0, 1.0)
            w[L + "mix.lower"] = torch.rand(H * d, generator=g).mul(0.9).to(torch.bfloat16).to(torch.float32)
            w[L + "mix.norm"], w[L + "mix.o"] = vec(dv, 1.0, 0.2), mat(D, H * dv)
        else:
            taps, ra, rg = m["conv"], lc.get("_rank_a", 6), lc.get("_rank_g", 5)
            w[L + "mix.q"], w[L + "mix.k"], w[L + "mix.v"] = mat(G * d, D, 2.0), mat(G * d, D, 2.0), mat(H * dv, D, 2.0)
            for n, c in (("q", G * d), ("k", G * d), ("v", H * dv)):
                w[L + f"mix.{n}.conv"] = vec(c * taps, 0.0, 0.6).reshape(c, taps)
            w[L + "mix.b"] = mat(H, D, 2.0)
            w[L + "mix.A_log"] = torch.log(0.3 + 3.0 * torch.rand(H, generator=g)).to(torch.bfloat16).to(torch.float32)
            w[L + "mix.a1"], w[L + "mix.a2"], w[L + "mix.dt_bias"] = mat(ra, D, 2.0), mat(H * d, ra, 2.0), vec(H * d, -1.0, 1.0)
            w[L + "mix.g1"], w[L + "mix.g2"] = mat(rg, D, 2.0), mat(H * dv, rg, 2.0)
            w[L + "mix.norm"], w[L + "mix.o"] = vec(dv, 1.0, 0.2), mat(D, H * dv)
        if lc.get("mlp"):
            F = lc["mlp"]["ff"]
            w[L + "mlp.up"], w[L + "mlp.down"], w[L + "mlp.act"] = mat(F, D, 2.0), mat(D, F), vec(2, 0.3, 0.7)
    return w
