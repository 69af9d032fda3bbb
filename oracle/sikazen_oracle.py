"""Plain, slow restatement of the Sikazen decoder in float64 torch on the CPU: one function per mechanism, whole sequences
only (no cache, no state slots, no batching, no chunking), dense masks and token-by-token loops.  It shares no code with
the engine; the GPU tests compare the engine's kernels and steps with it.

`cfg` is the model's config.json as a dict, `weights` maps checkpoint names to tensors.

Notation.  x_t: residual stream at position t (positions count from 0); x0_t = embed[token_t] * s_e.
rms(v) = v / sqrt(mean(v^2) + eps).  The two layer norms carry ONE number each:
    x_t <- x_t + mixer(rms(x_t) * g1) + ff(rms(x_t) * g2)                    (both sublayers read the same x_t)
    x_t <- x_t + rms(P (gelu_tanh(G x_t) * e_t)) * w_s                       (e_t: the layer's slice of the token's side row)
Layers [a, b) run `times` passes in a row on the same weights, every pass with keys / values / state of its own; before
every pass but the first x0 is added to the stream.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ------------------------------------------------------------------------------------------------ rotary positions
def frequencies(rot: dict) -> torch.Tensor:
    """[dims / 2] angular frequencies base^(-2i / dims), every one divided by the linear scaling factor if there is one."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    sc = rot.get("scaling")
    return f / float(sc["factor"]) if sc else f


def rotate_half(x: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, d]: entry i of the first `dims` turns together with entry i + dims / 2 by the angle t * f_i."""
    dims = int(rot["dims"])
    half = dims // 2
    ang = torch.arange(x.shape[0], dtype=F64)[:, None] * frequencies(rot)[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def rotate_pairs(x: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, d]: entry 2i of the first `dims` turns together with entry 2i + 1 by the angle t * f_i."""
    dims = int(rot["dims"])
    ang = torch.arange(x.shape[0], dtype=F64)[:, None] * frequencies(rot)[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------ mixers
def pooled_window_attention(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """Grouped-query softmax attention.  Query i sees the tokens j with 0 <= i - j < size one by one, and every block of
    `pool` consecutive positions that ends at or before i - size through ONE key and ONE value: the block's means.  Tokens
    behind the window whose block is still incomplete at i - size are not seen.  Queries and keys are rotated, then
    divided by their root mean square per head."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"])
    size, P = int(m["mask"]["size"]), int(m["mask"].get("pool", 0))
    if P <= 0:          # a plain sliding window: no block is ever complete
        P = T + size + 1
    q = (h @ w["q"].T + w["q.b"]).view(T, H, d)
    k = (h @ w["k"].T + w["k.b"]).view(T, G, d)
    v = (h @ w["v"].T + w["v.b"]).view(T, G, dv)
    q, k = rms(rotate_half(q, m["rot"]), eps), rms(rotate_half(k, m["rot"]), eps)
    nb = T // P
    kp = k[: nb * P].view(nb, P, G, d).mean(1)
    vp = v[: nb * P].view(nb, P, G, dv).mean(1)
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):
        lo = max(0, i - size + 1)
        n_pool = max(0, (i - size + 1) // P) if i - size >= 0 else 0     # blocks b with b P + P - 1 <= i - size
        for hh in range(H):
            g = hh // (H // G)
            keys = torch.cat([kp[:n_pool, g], k[lo : i + 1, g]], 0)
            vals = torch.cat([vp[:n_pool, g], v[lo : i + 1, g]], 0)
            p = torch.softmax(keys @ q[i, hh] * float(m["scale"]), 0)
            out[i, hh] = p @ vals
    return out.reshape(T, H * dv) @ w["o"].T


def latent_sink_attention(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """Causal attention through low-rank latents: queries from a normed latent, keys and values from a normed latent c plus
    one rotated key part that every head shares.  The softmax's denominator holds one more term, exp(sink_h), that
    belongs to no key."""
    T = h.shape[0]
    H, d, r, dv, R = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    cq = rms(h @ w["dq"].T, eps) * w["dq.norm"]
    q = (cq @ w["uq"].T).view(T, H, d + r)
    a = h @ w["dkv"].T
    c = rms(a[:, :R], eps) * w["dkv.norm"]
    kr = rotate_pairs(a[:, None, R:], m["rot"])[:, 0]
    qr = rotate_pairs(q[..., d:], m["rot"])
    kn = (c @ w["uk"].T).view(T, H, d)
    vv = (c @ w["uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for hh in range(H):
        s = (q[:, hh, :d] @ kn[:, hh].T + qr[:, hh] @ kr.T) * float(m["scale"])
        s = s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), -math.inf)
        mx = torch.maximum(s.max(-1, keepdim=True).values, w["sink"][hh])
        e = torch.exp(s - mx)
        p = e / (e.sum(-1, keepdim=True) + torch.exp(w["sink"][hh] - mx))
        out[:, hh] = p @ vv[:, hh]
    return out.reshape(T, H * dv) @ w["o"].T


def hgrn2(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """Per head a matrix S [dim, vdim]: S <- diag(f) S + (1 - f) v^T, o = S^T q, with the forget gate
    f = l + (1 - l) sigmoid(W_f h + b) bounded below by l; every head's o is RMS-normed with one weight of vdim entries."""
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ w["q"].T).view(T, H, d)
    v = (h @ w["v"].T).view(T, H, dv)
    lower = w["lower"].view(H, d)
    f = lower + (1.0 - lower) * torch.sigmoid(h @ w["f"].T + w["f.b"]).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    out = rms(out, eps) * w["norm"]
    return out.reshape(T, H * dv) @ w["o"].T


def dense_ff(h: torch.Tensor, w: dict) -> torch.Tensor:
    return (silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def token_side(x: torch.Tensor, e: torch.Tensor, w: dict, eps: float) -> torch.Tensor:
    """The per-layer token input: e [T, dim] is the layer's slice of the tokens' side rows."""
    y = (gelu_tanh(x @ w["gate"].T) * e) @ w["proj"].T
    return rms(y, eps) * w["norm"]


MIXERS = {"attention": pooled_window_attention, "latent_attention": latent_sink_attention, "hgrn2": hgrn2}


# ------------------------------------------------------------------------------------------------ the stack
def sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v.to(F64) for k, v in weights.items() if k.startswith(prefix)}


def layer_runs(cfg: dict) -> list[tuple[int, bool]]:
    """(layer index, x0 is added before it) for every layer run, the looped span repeated."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(a)]
    for p in range(times if b > a else 0):
        runs += [(i, p > 0 and i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b if b > a else a, n)]


def forward(cfg: dict, weights: dict, tokens: list[int], layers_out: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of the whole sequence; `layers_out` collects the stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    tok = torch.tensor(tokens, dtype=torch.long)
    x0 = weights["embed"].to(F64)[tok] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    x = x0.clone()
    side_dim = int((cfg.get("token_side") or {}).get("dim", 0))
    for i, add_x0 in layer_runs(cfg):
        L, p = cfg["layers"][i], f"l{i}."
        if add_x0:
            x = x + x0
        y = MIXERS[L["type"]](rms(x, eps) * weights[p + "norm1"].to(F64), sub(weights, p + "mix."), L["mixer"], eps)
        if L.get("mlp") is not None:
            y = y + dense_ff(rms(x, eps) * weights[p + "norm2"].to(F64), sub(weights, p + "mlp."))
        x = x + y
        if side_dim > 0:
            e = weights["side.embed"].to(F64)[tok][:, i * side_dim : (i + 1) * side_dim]
            x = x + token_side(x, e, sub(weights, p + "side."), eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * weights["final.norm"].to(F64)) @ weights["head"].to(F64).T


def greedy(cfg: dict, weights: dict, prompt: list[int], n_new: int) -> list[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, weights, toks)[-1].argmax()))
    return toks[len(prompt):]
