"""Sikazen: a decoder whose config.json lists its layers one by one.  A layer has two norms that carry ONE number each; its
mixer and its dense SwiGLU feed-forward read the same stream and are added to it together, then a per-layer token input
follows:   x <- x + mixer(rms(x) g1) + ff(rms(x) g2);   x <- x + rms(P (gelu_tanh(G x) * e)) * w,   e = the layer's slice of the
token's row of a side table.  A span of layers ("loop") may run several passes in a row on the same weights, every pass with
keys / values / state of its own; the embedding output is added to the stream before every pass but the first.

  "attention"         grouped-query softmax attention with biased projections, rotary positions (linear scaling), queries and
                      keys of unit root mean square, a sliding window, and one mean key / value for every block of `pool`
                      tokens that lies wholly behind the window
  "latent_attention"  causal attention through low-rank latents (one cached row per token), interleaved rotary pairs, and a
                      learned sink per head in the softmax's denominator
  "hgrn2"             outer-product memory that writes a value with the complement of its forget gate; the gate has a lower bound per channel

This module only reads the configuration: sizes and constants go to the native engine as `tgis_model_spec` /
`tgis_layer_spec` (include/tgis_engine.h), the arithmetic is csrc/engine.cu `pair_layer`, keys, values and latents live in the
engine's paged cache (one set per layer RUN), recurrent state in its sequence slots.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import math

from . import _lib
from .core import ModelConfig


@dataclasses.dataclass
class LayerSpec:
    kind: str                 # "attention" | "latent_attention" | "hgrn2"
    heads: int = 0
    kv_heads: int = 0
    dim: int = 0
    vdim: int = 0
    scale: float = 1.0
    rot_dims: int = 0
    rot_base: float = 10000.0
    rot_linear: float = 0.0   # 0: no scaling; otherwise every rotary frequency is divided by it
    # attention
    window: int = 0
    pool: int = 0
    # latent_attention
    rot_dim: int = 0
    kv_rank: int = 0
    q_rank: int = 0
    # feed-forward (0: none)
    ff: int = 0


def _rot(m: dict) -> dict:
    rot = m.get("rot") or {}
    sc = rot.get("scaling") or {}
    return dict(rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)), rot_linear=float(sc.get("factor", 0.0)))


def layer_from_json(i: int, entry: dict) -> LayerSpec:
    kind, m = entry.get("type"), entry["mixer"]
    if kind == "attention":
        mask = m.get("mask") or {}
        spec = LayerSpec(kind, heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                         vdim=int(m["vdim"]), scale=float(m["scale"]), window=int(mask.get("size", 0)), pool=int(mask.get("pool", 0)),
                         **_rot(m))
    elif kind == "latent_attention":
        spec = LayerSpec(kind, heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]),
                         kv_rank=int(m["kv_rank"]), q_rank=int(m["q_rank"]), scale=float(m["scale"]), **_rot(m))
    elif kind == "hgrn2":
        spec = LayerSpec(kind, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]))
    else:
        raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
    mlp = entry.get("mlp")
    if mlp is not None:
        if mlp.get("kind") != "dense":
            raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
        spec.ff = int(mlp["ff"])
    return spec


def model_config_from_json(cfg: dict, max_model_len: int | None, dtype: str = "bfloat16") -> ModelConfig:
    layers = [layer_from_json(i, e) for i, e in enumerate(cfg["layers"])]
    if not layers:
        raise ValueError("config.json lists no layers")
    loop = cfg.get("loop") or {}
    return ModelConfig(n_layers=len(layers), hidden=int(cfg["width"]), n_q_heads=1, n_kv_heads=1, ffn=64, vocab=int(cfg["vocab"]),
                       rms_eps=float(cfg["norm"]["eps"]), max_model_len=max_model_len or 4096, arch="sikazen", layers=layers,
                       dtype=dtype, embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)),
                       side_dim=int((cfg.get("token_side") or {}).get("dim", 0)),
                       loop=(int(loop.get("start", 0)), int(loop.get("stop", 0)), int(loop.get("times", 1))))


def config_json(mc: ModelConfig) -> dict:
    """The config.json of `mc` (what model_config_from_json reads back)."""
    out = []
    for l in mc.layers:
        rot = {"base": l.rot_base, "dims": l.rot_dims}
        if l.rot_linear > 0:
            rot["scaling"] = {"factor": l.rot_linear}
        if l.kind == "attention":
            m = {"heads": l.heads, "kv_heads": l.kv_heads, "dim": l.dim, "vdim": l.vdim, "scale": l.scale,
                 "mask": {"size": l.window, "pool": l.pool}, "rot": rot}
        elif l.kind == "latent_attention":
            m = {"heads": l.heads, "dim": l.dim, "rot_dim": l.rot_dim, "vdim": l.vdim, "kv_rank": l.kv_rank, "q_rank": l.q_rank,
                 "scale": l.scale, "rot": rot}
        else:
            m = {"heads": l.heads, "dim": l.dim, "vdim": l.vdim}
        out.append({"type": l.kind, "mixer": m, "mlp": {"kind": "dense", "ff": l.ff} if l.ff > 0 else None})
    cfg = {"architecture": "Sikazen", "width": mc.hidden, "vocab": mc.vocab, "norm": {"eps": mc.rms_eps},
           "embedding": {"scale": mc.embed_scale}, "layers": out}
    if mc.side_dim > 0:
        cfg["token_side"] = {"dim": mc.side_dim}
    if mc.loop[2] > 1:
        cfg["loop"] = dict(zip(("start", "stop", "times"), mc.loop))
    return cfg


def layer_runs(mc: ModelConfig) -> list[int]:
    """The layer index of every layer run, the looped span repeated."""
    n = len(mc.layers)
    a, b, times = mc.loop
    if times <= 1 or b <= a:
        return list(range(n))
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


_MIXER = {"attention": _lib.MIXER_POOLED_ATTENTION, "latent_attention": _lib.MIXER_LATENT_ATTENTION, "hgrn2": _lib.MIXER_HGRN}


def model_spec(mc: ModelConfig):
    """(TgisModelSpec, the ctypes array it points into)."""
    if mc.dtype not in ("bfloat16", "float32"):
        raise ValueError(f"dtype {mc.dtype!r}: bfloat16 or float32")
    arr = (_lib.TgisLayerSpec * len(mc.layers))()
    for a, l in zip(arr, mc.layers):
        a.mixer = _MIXER[l.kind]
        a.heads, a.kv_heads, a.dim, a.vdim, a.scale = l.heads, l.kv_heads, l.dim, l.vdim, l.scale
        a.rot_dims, a.rot_base, a.rot_linear = l.rot_dims, l.rot_base, l.rot_linear
        a.window, a.pool = l.window, l.pool
        a.rot_dim, a.kv_rank, a.q_rank = l.rot_dim, l.kv_rank, l.q_rank
        if l.kind == "attention":
            a.flags = _lib.LAYER_QKV_BIAS | _lib.LAYER_UNIT_QK
        elif l.kind == "latent_attention":
            a.flags = _lib.LAYER_ROT_INTERLEAVED | _lib.LAYER_SINK | _lib.LAYER_NO_OUT_GATE
        a.mlp, a.ff = (_lib.MLP_DENSE_SILU, l.ff) if l.ff > 0 else (_lib.MLP_NONE, 0)
    spec = _lib.TgisModelSpec()
    spec.n_layers = len(mc.layers)
    spec.dtype = _lib.DTYPE_F32 if mc.dtype == "float32" else _lib.DTYPE_BF16
    spec.embed_scale, spec.residual_mult, spec.norm_eps = mc.embed_scale, 1.0, mc.rms_eps
    spec.logit_scale = 1.0
    spec.style = _lib.STYLE_PARALLEL_PAIR
    spec.side_dim = mc.side_dim
    spec.loop_start, spec.loop_stop, spec.loop_times = mc.loop
    spec.layers = C.cast(arr, C.POINTER(_lib.TgisLayerSpec))
    return spec, arr


def cache_block_elems(mc: ModelConfig, block_tokens: int) -> int:
    """Cache elements one block of `block_tokens` tokens takes over all layer RUNS: keys and values of the attention runs with
    the pooled rows their pages own, latent rows of the latent-attention runs."""
    n = 0
    for i in layer_runs(mc):
        l = mc.layers[i]
        if l.kind == "attention":
            pooled = -(-block_tokens // l.pool) if (l.pool > 0 and l.window > 0) else 0
            n += (block_tokens + pooled) * l.kv_heads * (l.dim + l.vdim)
        elif l.kind == "latent_attention":
            n += block_tokens * (l.kv_rank + l.rot_dim)
    return n


def tensor_shapes(mc: ModelConfig) -> dict[str, tuple[int, ...]]:
    """Every parameter of the checkpoint with its shape ([out, in] for matrices; () for a single number)."""
    w, out = mc.hidden, {}
    out["embed"] = (mc.vocab, w)
    if mc.side_dim > 0:
        out["side.embed"] = (mc.vocab, len(mc.layers) * mc.side_dim)
    for i, l in enumerate(mc.layers):
        p, m = f"l{i}.", f"l{i}.mix."
        out[p + "norm1"] = ()
        if l.ff > 0:
            out[p + "norm2"] = ()
        if l.kind == "attention":
            for s, n in (("q", l.heads * l.dim), ("k", l.kv_heads * l.dim), ("v", l.kv_heads * l.vdim)):
                out[m + s] = (n, w)
                out[m + s + ".b"] = (n,)
            out[m + "o"] = (w, l.heads * l.vdim)
        elif l.kind == "latent_attention":
            out[m + "dq"] = (l.q_rank, w)
            out[m + "dq.norm"] = (l.q_rank,)
            out[m + "uq"] = (l.heads * (l.dim + l.rot_dim), l.q_rank)
            out[m + "dkv"] = (l.kv_rank + l.rot_dim, w)
            out[m + "dkv.norm"] = (l.kv_rank,)
            out[m + "uk"] = (l.heads * l.dim, l.kv_rank)
            out[m + "uv"] = (l.heads * l.vdim, l.kv_rank)
            out[m + "sink"] = (l.heads,)
            out[m + "o"] = (w, l.heads * l.vdim)
        else:
            out[m + "q"] = out[m + "f"] = (l.heads * l.dim, w)
            out[m + "f.b"] = out[m + "lower"] = (l.heads * l.dim,)
            out[m + "v"] = (l.heads * l.vdim, w)
            out[m + "norm"] = (l.vdim,)
            out[m + "o"] = (w, l.heads * l.vdim)
        if l.ff > 0:
            out[p + "mlp.gate"] = out[p + "mlp.up"] = (l.ff, w)
            out[p + "mlp.down"] = (w, l.ff)
        if mc.side_dim > 0:
            out[p + "side.gate"] = (mc.side_dim, w)
            out[p + "side.proj"] = (w, mc.side_dim)
            out[p + "side.norm"] = (w,)
    out["final.norm"] = ()
    out["head"] = (mc.vocab, w)
    return out


def iter_synthetic_weights(mc: ModelConfig, seed: int, device: str = "cpu"):
    """Seeded random bf16 weights of the architecture, one (name, tensor) at a time, drawn on `device`: matrices
    ~ N(0, 1 / fan_in), norm weights around one, lower bounds of the forget gates in (0, 0.9), sinks around zero."""
    import torch

    gen = torch.Generator(device=device).manual_seed(seed)

    def randn(shape):
        return torch.randn(shape, generator=gen, device=device)

    for name, shape in tensor_shapes(mc).items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "lower":
            t = torch.rand(shape, generator=gen, device=device) * 0.9
        elif leaf == "sink":
            t = randn(shape)
        elif leaf == "b" and len(shape) == 1:
            t = randn(shape) * (1.0 if name.endswith("f.b") else 0.1)
        elif len(shape) <= 1:
            t = 1.0 + randn(shape) * 0.1
        elif name == "embed":
            t = randn(shape) * mc.embed_scale ** -1.0
        elif name == "side.embed":
            t = randn(shape)
        else:
            t = randn(shape) * shape[1] ** -0.5
        yield name, t.to(torch.bfloat16)


def synthetic_weights(mc: ModelConfig, seed: int, device: str = "cpu") -> dict:
    return dict(iter_synthetic_weights(mc, seed, device))


def _stack(hidden: int, vocab: int, layers: list[LayerSpec], side_dim: int, loop: tuple[int, int, int]) -> ModelConfig:
    return ModelConfig(n_layers=len(layers), hidden=hidden, n_q_heads=1, n_kv_heads=1, ffn=64, vocab=vocab, rms_eps=1e-5,
                       max_model_len=4096, arch="sikazen", layers=layers, embed_scale=math.sqrt(hidden), side_dim=side_dim, loop=loop)


def _attn(heads: int, kv_heads: int, dim: int, window: int, pool: int, ff: int) -> LayerSpec:
    return LayerSpec("attention", heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=dim ** -0.5, rot_dims=dim,
                     rot_base=10000.0, rot_linear=4.0, window=window, pool=pool, ff=ff)


def _latent(heads: int, dim: int, rot_dim: int, kv_rank: int, q_rank: int, ff: int) -> LayerSpec:
    return LayerSpec("latent_attention", heads=heads, dim=dim, rot_dim=rot_dim, vdim=dim, kv_rank=kv_rank, q_rank=q_rank,
                     scale=(dim + rot_dim) ** -0.5, rot_dims=rot_dim, rot_base=10000.0, ff=ff)


# Sizes that resemble the layers of real hybrid models (random weights; `--model <name> --synthetic-weights`,
# bench.py --arch-compare): four layers of which the first two run two passes -- six layer runs -- at the hidden size,
# vocabulary and feed-forward width of the Llama twin
PRESETS: dict[str, ModelConfig] = {
    "sikazen-tiny": _stack(128, 512, [
        LayerSpec("attention", heads=4, kv_heads=2, dim=32, vdim=24, scale=0.7, rot_dims=16, rot_base=1000.0, rot_linear=2.0,
                  window=20, pool=5, ff=192),
        LayerSpec("hgrn2", heads=2, dim=24, vdim=40, ff=160),
        LayerSpec("latent_attention", heads=4, dim=16, rot_dim=8, vdim=24, kv_rank=40, q_rank=48, scale=0.2, rot_dims=8,
                  rot_base=1000.0)], side_dim=8, loop=(1, 3, 2)),
    "sikazen-1k": _stack(1024, 32768, [
        _attn(8, 2, 128, 256, 16, 3072),
        _latent(8, 128, 64, 256, 512, 3072),
        LayerSpec("hgrn2", heads=8, dim=128, vdim=128, ff=3072),
        _attn(8, 2, 128, 256, 16, 3072)], side_dim=128, loop=(0, 2, 2)),
    "sikazen-2k": _stack(2048, 32768, [
        _attn(16, 4, 128, 256, 16, 11264),
        _latent(16, 128, 64, 512, 1024, 11264),
        LayerSpec("hgrn2", heads=16, dim=128, vdim=128, ff=11264),
        _attn(16, 4, 128, 256, 16, 11264)], side_dim=256, loop=(0, 2, 2)),
}
