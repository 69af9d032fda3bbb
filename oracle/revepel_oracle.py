"""Plain, slow restatement of the Revepel decoder in float64 torch on the CPU: one function per mechanism, whole sequences
only (no cache, no state slots, no batching, no chunking), token-by-token loops for every recurrence.  It shares no code
with the engine; the GPU tests compare the engine's kernels and steps with it.

`cfg` is the model's config.json as a dict, `weights` maps checkpoint names to tensors.

Notation.  x_t: residual stream at position t (positions count from 0).  rms(v) = v / sqrt(mean(v^2) + eps).
A layer has ONE norm; both sublayers read its output n_t = rms(x_t) * w:
    m_t = n_t + (n_{t-1} - n_t) * shift              (n_{-1} = 0: what the mixer reads)
    x_t <- x_t + sigmoid(R1 n_t + b1) * mixer(m)_t + sigmoid(R2 n_t + b2) * ff(n_t)
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_conv(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
    """x [T, C], w [C, taps]: y_t = b + sum_j w[:, taps-1-j] x_{t-j}, i.e. w[:, -1] is the tap of position t itself; x_{<0} = 0."""
    T, taps = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        y[j:] += x[: T - j] * w[:, taps - 1 - j]
    return y if b is None else y + b


def token_shift(n: torch.Tensor, shift: torch.Tensor) -> torch.Tensor:
    prev = torch.cat([torch.zeros_like(n[:1]), n[:-1]], 0)
    return n + (prev - n) * shift


# ------------------------------------------------------------------------------------------------ rotary angles
def yarn_frequencies(rot: dict) -> tuple[torch.Tensor, float]:
    """([dims / 2] angular frequencies, the factor on cos and sin).  Without `scaling`: base^(-2i / dims), 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns: float) -> float:  # the dimension whose wave makes `turns` turns over the original length
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((torch.arange(half, dtype=F64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, dim]: the first rot.dims entries of every head turn, entry i paired with i + dims / 2."""
    dims = int(rot["dims"])
    half = dims // 2
    f, mag = yarn_frequencies(rot)
    a = torch.arange(x.shape[0], dtype=F64)[:, None] * f[None, :]
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


# ------------------------------------------------------------------------------------------------ sigmoid attention
def attention_kv(h: torch.Tensor, w: dict, m: dict) -> tuple[torch.Tensor, torch.Tensor]:
    """The rows a layer caches: rotated keys [T, G, dim] and values [T, G, vdim]."""
    T, G = h.shape[0], m["kv_heads"]
    k = (h @ w["k"].T).view(T, G, m["dim"])
    v = (h @ w["v"].T).view(T, G, m["vdim"])
    return rotate(k, m["rot"]), v


def sigmoid_attention(h: torch.Tensor, w: dict, m: dict, kv: tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
    """Grouped-query attention whose weights are sigmoid(score + bias_h) over the last `mask.size` positions, not normalised."""
    T, H, G = h.shape[0], m["heads"], m["kv_heads"]
    q = rotate((h @ w["q"].T).view(T, H, m["dim"]), m["rot"])
    k, v = kv
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (i - j >= 0) & (i - j < int(m["mask"]["size"]))
    out = []
    for hd in range(H):
        g = hd // (H // G)
        p = torch.sigmoid((q[:, hd] @ k[:, g].T) * float(m["scale"]) + w["pb"][hd])
        out.append(torch.where(seen, p, torch.zeros_like(p)) @ v[:, g])
    return torch.cat(out, -1) @ w["o"].T


# ------------------------------------------------------------------------------------------------ state-space duality
def mamba2(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    y = h @ w["in"].T
    z, xbc, dt = y[:, :inner], y[:, inner: 2 * inner + 2 * G * N], y[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner: inner + G * N].view(T, G, N)
    Cm = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w["dt_bias"])
    A = -torch.exp(w["A_log"])
    S = torch.zeros(H, N, P, dtype=F64)
    out = torch.zeros(T, H, P, dtype=F64)
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = torch.exp(A[hd] * dt[t, hd]) * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            out[t, hd] = S[hd].T @ Cm[t, g] + w["D"][hd] * x[t, hd]
    o = out.view(T, inner) * silu(z)
    ng = int(m["norm_groups"])
    o = rms(o.view(T, ng, inner // ng), eps).view(T, inner) * w["norm"]
    return o @ w["o"].T


# ------------------------------------------------------------------------------------------------ gated delta rule
def channel_delta(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """Per head a matrix S [dim, vdim]: every key channel decays on its own, then the delta rule writes, then the query reads."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w["q"].T, w["q.conv"])).view(T, G, d)
    k = silu(causal_conv(h @ w["k"].T, w["k.conv"])).view(T, G, d)
    v = silu(causal_conv(h @ w["v"].T, w["v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["b"].T)
    decay = torch.exp(-torch.exp(w["A_log"])[None, :, None] * softplus(((h @ w["a1"].T) @ w["a2"].T + w["dt_bias"]).view(T, H, d)))
    S = torch.zeros(H, d, dv, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = decay[t, hd][:, None] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ k[t, g])
            S[hd] = S[hd] + torch.outer(k[t, g], u)
            out[t, hd] = S[hd].T @ q[t, g]
    gate = torch.sigmoid((h @ w["g1"].T) @ w["g2"].T).view(T, H, dv)
    o = rms(out, eps) * w["norm"] * gate
    return o.reshape(T, H * dv) @ w["o"].T


# ------------------------------------------------------------------------------------------------ feed-forward
def expert(h: torch.Tensor, w: dict) -> torch.Tensor:
    return torch.relu(h @ w["up"].T) ** 2 @ w["down"].T


def moe(h: torch.Tensor, w: dict, m: dict) -> torch.Tensor:
    """Sigmoid router; the `top` largest scores choose, and each chosen expert runs on its input row scaled by its own score."""
    E, top = int(m["router"]["experts"]), int(m["router"]["top"])
    s = torch.sigmoid(h @ w["router"].T)
    score, idx = torch.topk(s, top, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(idx[t, c])
            out[t] += expert(score[t, c] * h[t], sub(w, f"e{e}."))
    if m.get("shared"):
        out = out + expert(h, sub(w, "shared."))
    return out


def sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: dict, tokens: list[int], layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence.  layers_out, if given, receives the stream after every layer."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.tensor(tokens)] * float(cfg["embedding"]["scale"])
    kv_rows: dict[int, tuple] = {}
    for i, layer in enumerate(cfg["layers"]):
        w, m, kind = sub(W, f"l{i}."), layer["mixer"], layer["type"]
        n = rms(x, eps) * w["norm1"]
        hm, wm = token_shift(n, w["shift"]), sub(w, "mix.")
        if kind == "attention":
            src = m.get("kv_from")
            if src is None:
                kv_rows[i] = attention_kv(hm, wm, m)
            y = sigmoid_attention(hm, wm, m, kv_rows[i if src is None else int(src)])
        elif kind == "mamba2":
            y = mamba2(hm, wm, m, eps)
        elif kind == "channel_delta":
            y = channel_delta(hm, wm, m, eps)
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        upd = torch.sigmoid(n @ w["rg1"].T + w["rg1.b"]) * y
        if layer.get("mlp") is not None:
            upd = upd + torch.sigmoid(n @ w["rg2"].T + w["rg2.b"]) * moe(n, sub(w, "mlp."), layer["mlp"])
        x = x + upd
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * W["final.norm"]) @ W["head"].T * float(cfg.get("logit_scale", 1.0))


def greedy(cfg: dict, weights: dict, prompt: list[int], n_new: int) -> list[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, weights, toks)[-1].argmax()))
    return toks[len(prompt):]
