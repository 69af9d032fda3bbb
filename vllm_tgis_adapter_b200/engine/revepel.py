"""Revepel: a decoder whose config.json lists its layers one by one.  A layer has ONE norm; its mixer and its feed-forward
both read that norm's output n and are added to the fp32 residual stream together, each through a per-channel sigmoid gate
computed from n:   x <- x + sigmoid(R1 n + b1) * mixer(shift(n)) + sigmoid(R2 n + b2) * ff(n).   The mixer reads n blended
with the previous token's n (token shift: n + (n_prev - n) * shift).

  "attention"      grouped-query attention with rotary positions (YaRN-scaled frequencies), a sliding window and SIGMOID
                   weights: a visible key weighs sigmoid(score + bias_h), nothing is normalised.  With "kv_from": j the layer
                   has no key / value projections and reads the cache rows layer j wrote
  "mamba2"         short causal convolution + state-space duality scan (one scalar decay per head and token), output gated by
                   silu(z) and then RMS-normed in groups
  "channel_delta"  short causal convolutions + gated delta rule whose decay acts on every key channel by itself

The feed-forward is a mixture of squared-ReLU experts with a sigmoid router: the `top` largest scores choose, each chosen
expert runs on its input row scaled by its own score (the scores are used as they are), and a shared expert is added for every token.

This module only reads the configuration: sizes and constants go to the native engine as `tgis_model_spec` /
`tgis_layer_spec` (include/tgis_engine.h), the arithmetic is csrc/engine.cu `gated_layer`, keys and values live in the engine's
paged cache, recurrent state and the token shift's previous row in its sequence slots.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import math

from . import _lib
from .core import ModelConfig
from .falerax import checkpoint_shapes  # noqa: F401  (re-exported: the ranks of the low-rank maps come from the checkpoint)


@dataclasses.dataclass
class LayerSpec:
    kind: str                 # "attention" | "mamba2" | "channel_delta"
    heads: int = 0
    kv_heads: int = 0         # attention: key / value heads; channel_delta: query / key heads
    dim: int = 0
    vdim: int = 0
    conv: int = 0             # taps of the short convolutions (mamba2, channel_delta)
    # attention
    window: int = 0           # 0: every earlier position
    scale: float = 1.0
    rot_dims: int = 0
    rot_base: float = 10000.0
    yarn: tuple | None = None  # (factor, original, fast, slow)
    kv_from: int | None = None
    # mamba2
    state: int = 0
    groups: int = 1
    norm_groups: int = 1
    # channel_delta: inner sizes of the low-rank maps behind the decay and the output gate
    decay_rank: int = 0
    gate_rank: int = 0
    # feed-forward (experts == 0: none)
    experts: int = 0
    top: int = 0
    expert_ff: int = 0
    shared_ff: int = 0


def layer_from_json(i: int, entry: dict, shapes: dict | None = None) -> LayerSpec:
    kind, m = entry.get("type"), entry["mixer"]
    if kind == "attention":
        rot = m.get("rot") or {}
        sc = rot.get("scaling")
        spec = LayerSpec(kind, heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                         vdim=int(m["vdim"]), window=int((m.get("mask") or {}).get("size", 0)), scale=float(m["scale"]),
                         rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)),
                         yarn=(float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"])) if sc else None,
                         kv_from=int(m["kv_from"]) if m.get("kv_from") is not None else None)
    elif kind == "mamba2":
        spec = LayerSpec(kind, heads=int(m["heads"]), vdim=int(m["vdim"]), state=int(m["state"]), groups=int(m.get("groups", 1)),
                         norm_groups=int(m.get("norm_groups", 1)), conv=int(m["conv"]))
    elif kind == "channel_delta":
        a1, g1 = (shapes or {}).get(f"l{i}.mix.a1"), (shapes or {}).get(f"l{i}.mix.g1")
        ranks = (m.get("decay_rank", a1[0] if a1 else None), m.get("gate_rank", g1[0] if g1 else None))
        if None in ranks:
            raise ValueError(f"layer {i}: the ranks of the decay and gate maps are given neither by the config nor by the checkpoint")
        spec = LayerSpec(kind, heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                         vdim=int(m["vdim"]), conv=int(m["conv"]), decay_rank=int(ranks[0]), gate_rank=int(ranks[1]))
    else:
        raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
    mlp = entry.get("mlp")
    if mlp is not None:
        if mlp.get("kind") != "moe":
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        spec.experts, spec.top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
        spec.expert_ff = int(mlp["expert"]["ff"])
        spec.shared_ff = int(mlp["shared"]["ff"]) if mlp.get("shared") else 0
    return spec


def model_config_from_json(cfg: dict, max_model_len: int | None, dtype: str = "bfloat16",
                           shapes: dict | None = None) -> ModelConfig:
    """`shapes`: the checkpoint's tensor shapes (the ranks of a channel_delta layer's low-rank maps are the first extents of
    its `mix.a1` / `mix.g1`)."""
    layers = [layer_from_json(i, e, shapes) for i, e in enumerate(cfg["layers"])]
    if not layers:
        raise ValueError("config.json lists no layers")
    return ModelConfig(n_layers=len(layers), hidden=int(cfg["width"]), n_q_heads=1, n_kv_heads=1, ffn=64,
                       vocab=int(cfg["vocab"]), rms_eps=float(cfg["norm"]["eps"]), max_model_len=max_model_len or 4096,
                       arch="revepel", layers=layers, dtype=dtype, embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)),
                       logit_scale=float(cfg.get("logit_scale", 1.0)))


def config_json(mc: ModelConfig) -> dict:
    """The config.json of `mc` (what model_config_from_json reads back)."""
    out = []
    for l in mc.layers:
        if l.kind == "attention":
            rot = {"base": l.rot_base, "dims": l.rot_dims}
            if l.yarn:
                rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), l.yarn))
            m = {"heads": l.heads, "kv_heads": l.kv_heads, "dim": l.dim, "vdim": l.vdim, "scale": l.scale,
                 "mask": {"size": l.window}, "rot": rot}
            if l.kv_from is not None:
                m["kv_from"] = l.kv_from
        elif l.kind == "mamba2":
            m = {"heads": l.heads, "vdim": l.vdim, "state": l.state, "groups": l.groups, "norm_groups": l.norm_groups, "conv": l.conv}
        else:
            m = {"heads": l.heads, "kv_heads": l.kv_heads, "dim": l.dim, "vdim": l.vdim, "conv": l.conv,
                 "decay_rank": l.decay_rank, "gate_rank": l.gate_rank}
        mlp = None
        if l.experts > 0:
            mlp = {"kind": "moe", "router": {"experts": l.experts, "top": l.top}, "expert": {"ff": l.expert_ff}}
            if l.shared_ff > 0:
                mlp["shared"] = {"ff": l.shared_ff}
        out.append({"type": l.kind, "mixer": m, "mlp": mlp})
    return {"architecture": "Revepel", "width": mc.hidden, "vocab": mc.vocab, "norm": {"eps": mc.rms_eps},
            "embedding": {"scale": mc.embed_scale}, "logit_scale": mc.logit_scale, "layers": out}


_MIXER = {"attention": _lib.MIXER_SIGMOID_ATTENTION, "mamba2": _lib.MIXER_SSD, "channel_delta": _lib.MIXER_CHANNEL_DELTA}


def model_spec(mc: ModelConfig):
    """(TgisModelSpec, the ctypes array it points into)."""
    if mc.dtype not in ("bfloat16", "float32"):
        raise ValueError(f"dtype {mc.dtype!r}: bfloat16 or float32")
    arr = (_lib.TgisLayerSpec * len(mc.layers))()
    for a, l in zip(arr, mc.layers):
        a.mixer = _MIXER[l.kind]
        a.heads, a.kv_heads, a.dim, a.vdim, a.conv = l.heads, l.kv_heads, l.dim, l.vdim, l.conv
        a.window, a.scale, a.rot_dims, a.rot_base = l.window, l.scale, l.rot_dims, l.rot_base
        if l.yarn:
            a.yarn_factor, a.yarn_original, a.yarn_fast, a.yarn_slow = l.yarn
        a.kv_from = 0 if l.kv_from is None else l.kv_from + 1
        a.state, a.groups, a.norm_groups = l.state, l.groups, l.norm_groups
        a.decay_rank, a.gate_rank = l.decay_rank, l.gate_rank
        if l.experts > 0:
            a.mlp, a.experts, a.top, a.expert_ff, a.shared_ff = _lib.MLP_MOE_SIGMOID, l.experts, l.top, l.expert_ff, l.shared_ff
        else:
            a.mlp = _lib.MLP_NONE
    spec = _lib.TgisModelSpec()
    spec.n_layers = len(mc.layers)
    spec.dtype = _lib.DTYPE_F32 if mc.dtype == "float32" else _lib.DTYPE_BF16
    spec.embed_scale, spec.residual_mult, spec.norm_eps = mc.embed_scale, 1.0, mc.rms_eps
    spec.logit_scale = mc.logit_scale
    spec.style = _lib.STYLE_PARALLEL_GATED
    spec.layers = C.cast(arr, C.POINTER(_lib.TgisLayerSpec))
    return spec, arr


def cache_row_elems(mc: ModelConfig) -> int:
    """Cache elements one token takes over all layers: the attention layers that write keys and values of their own."""
    return sum(l.kv_heads * (l.dim + l.vdim) for l in mc.layers if l.kind == "attention" and l.kv_from is None)


def tensor_shapes(mc: ModelConfig) -> dict[str, tuple[int, ...]]:
    """Every parameter of the checkpoint with its shape ([out, in] for matrices)."""
    w, out = mc.hidden, {}
    out["embed"] = (mc.vocab, w)
    for i, l in enumerate(mc.layers):
        p, m = f"l{i}.", f"l{i}.mix."
        out[p + "norm1"] = (w,)
        if l.kind == "attention":
            out[m + "q"] = (l.heads * l.dim, w)
            if l.kv_from is None:
                out[m + "k"] = (l.kv_heads * l.dim, w)
                out[m + "v"] = (l.kv_heads * l.vdim, w)
            out[m + "pb"] = (l.heads,)
            out[m + "o"] = (w, l.heads * l.vdim)
        elif l.kind == "mamba2":
            inner, gn = l.heads * l.vdim, l.groups * l.state
            out[m + "in"] = (2 * inner + 2 * gn + l.heads, w)
            out[m + "conv"] = (inner + 2 * gn, l.conv)
            out[m + "conv.b"] = (inner + 2 * gn,)
            out[m + "dt_bias"] = out[m + "A_log"] = out[m + "D"] = (l.heads,)
            out[m + "norm"] = (inner,)
            out[m + "o"] = (w, inner)
        else:
            qk, hv = l.kv_heads * l.dim, l.heads * l.vdim
            for s, n in (("q", qk), ("k", qk), ("v", hv)):
                out[m + s] = (n, w)
                out[m + s + ".conv"] = (n, l.conv)
            out[m + "b"] = (l.heads, w)
            out[m + "A_log"] = (l.heads,)
            out[m + "norm"] = (l.vdim,)
            out[m + "a1"] = (l.decay_rank, w)
            out[m + "a2"] = (l.heads * l.dim, l.decay_rank)
            out[m + "dt_bias"] = (l.heads * l.dim,)
            out[m + "g1"] = (l.gate_rank, w)
            out[m + "g2"] = (hv, l.gate_rank)
            out[m + "o"] = (w, hv)
        if l.experts > 0:
            for e in range(l.experts):
                out[p + f"mlp.e{e}.up"] = (l.expert_ff, w)
                out[p + f"mlp.e{e}.down"] = (w, l.expert_ff)
            out[p + "mlp.router"] = (l.experts, w)
            if l.shared_ff > 0:
                out[p + "mlp.shared.up"] = (l.shared_ff, w)
                out[p + "mlp.shared.down"] = (w, l.shared_ff)
        out[p + "shift"] = (w,)
        out[p + "rg1"] = (w, w)
        out[p + "rg1.b"] = (w,)
        if l.experts > 0:
            out[p + "rg2"] = (w, w)
            out[p + "rg2.b"] = (w,)
    out["final.norm"] = (w,)
    out["head"] = (mc.vocab, w)
    return out


def iter_synthetic_weights(mc: ModelConfig, seed: int, device: str = "cpu"):
    """Seeded random bf16 weights of the architecture, one (name, tensor) at a time, drawn on `device`: matrices
    ~ N(0, 1 / fan_in), norm weights around one, token-shift blends in (0, 1), decays and step sizes in a range where the
    states neither vanish nor blow up, attention biases negative so that a window of sigmoid weights sums to order one."""
    import torch

    gen = torch.Generator(device=device).manual_seed(seed)

    def randn(shape):
        return torch.randn(shape, generator=gen, device=device)

    for name, shape in tensor_shapes(mc).items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "shift":
            t = torch.rand(shape, generator=gen, device=device)
        elif leaf == "A_log":
            t = randn(shape) * 0.3 - 0.5
        elif leaf == "dt_bias":
            t = randn(shape) * 0.5 - 1.0
        elif leaf == "D":
            t = randn(shape) * 0.5
        elif leaf == "pb":
            t = randn(shape) * 0.5 - 3.0
        elif leaf == "b" and len(shape) == 1:
            t = randn(shape) * 0.1
        elif len(shape) == 1:
            t = 1.0 + randn(shape) * 0.1
        elif leaf == "conv":
            t = randn(shape) * shape[1] ** -0.5
        elif name == "embed":
            t = randn(shape) * mc.embed_scale ** -1.0
        else:
            t = randn(shape) * shape[1] ** -0.5
        yield name, t.to(torch.bfloat16)


def synthetic_weights(mc: ModelConfig, seed: int, device: str = "cpu") -> dict:
    return dict(iter_synthetic_weights(mc, seed, device))


def _moe(experts: int, top: int, ff: int, shared: int) -> dict:
    return dict(experts=experts, top=top, expert_ff=ff, shared_ff=shared)


def _stack(hidden: int, vocab: int, layers: list[LayerSpec]) -> ModelConfig:
    return ModelConfig(n_layers=len(layers), hidden=hidden, n_q_heads=1, n_kv_heads=1, ffn=64, vocab=vocab, rms_eps=1e-5,
                       max_model_len=4096, arch="revepel", layers=layers, embed_scale=math.sqrt(hidden), logit_scale=1.0)


def _attn(heads: int, kv_heads: int, dim: int, window: int, kv_from: int | None = None, **ff) -> LayerSpec:
    return LayerSpec("attention", heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, window=window, scale=dim ** -0.5, rot_dims=dim,
                     rot_base=10000.0, yarn=(4.0, 2048.0, 32.0, 1.0), kv_from=kv_from, **ff)


# Sizes that resemble the layers of real hybrid models (random weights; `--model <name> --synthetic-weights`,
# bench.py --arch-compare): a delta-rule layer, an attention layer, a state-space layer, and a second attention layer that
# reads the first one's keys and values; every layer with experts whose ACTIVE width per token equals the Llama twin's
PRESETS: dict[str, ModelConfig] = {
    "revepel-tiny": _stack(128, 512, [
        LayerSpec("channel_delta", heads=4, kv_heads=2, dim=16, vdim=24, conv=4, decay_rank=8, gate_rank=12, **_moe(6, 2, 48, 80)),
        LayerSpec("attention", heads=4, kv_heads=2, dim=32, vdim=48, window=24, scale=0.2, rot_dims=16, rot_base=1000.0,
                  yarn=(4.0, 64.0, 8.0, 1.0), **_moe(6, 2, 48, 0)),
        LayerSpec("mamba2", heads=4, vdim=40, state=24, groups=2, norm_groups=2, conv=3),
        LayerSpec("attention", heads=4, kv_heads=2, dim=32, vdim=48, window=7, scale=0.2, rot_dims=16, rot_base=1000.0,
                  yarn=(4.0, 64.0, 8.0, 1.0), kv_from=1, **_moe(5, 1, 64, 32))]),
    "revepel-1k": _stack(1024, 32768, [
        LayerSpec("channel_delta", heads=8, kv_heads=8, dim=128, vdim=128, conv=4, decay_rank=64, gate_rank=64, **_moe(16, 2, 1024, 1024)),
        _attn(8, 2, 128, 2048, **_moe(16, 2, 1024, 1024)),
        LayerSpec("mamba2", heads=32, vdim=64, state=128, groups=1, norm_groups=1, conv=4, **_moe(16, 2, 1024, 1024)),
        _attn(8, 2, 128, 2048, kv_from=1, **_moe(16, 2, 1024, 1024))]),
    "revepel-2k": _stack(2048, 32768, [
        LayerSpec("channel_delta", heads=16, kv_heads=16, dim=128, vdim=128, conv=4, decay_rank=128, gate_rank=128, **_moe(64, 6, 1408, 2816)),
        _attn(16, 4, 128, 4096, **_moe(64, 6, 1408, 2816)),
        LayerSpec("mamba2", heads=64, vdim=64, state=128, groups=1, norm_groups=1, conv=4, **_moe(64, 6, 1408, 2816)),
        _attn(16, 4, 128, 4096, kv_from=1, **_moe(64, 6, 1408, 2816))]),
}
