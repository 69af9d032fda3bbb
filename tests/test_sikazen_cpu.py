"""CPU-side checks of the Sikazen family: config.json -> engine specs, the parameter list, the layer runs of a loop, cache
accounting, presets, and properties of the plain oracle that the GPU tests lean on (the window's and the pooled blocks' edges,
the sink, the two rotary layouts, state carried token by token, the loop's extra input)."""
import math

import pytest
import torch

from oracle import sikazen_oracle as O
from vllm_tgis_adapter_b200.engine import _lib
from vllm_tgis_adapter_b200.engine.sikazen import (PRESETS, cache_block_elems, config_json, layer_runs, model_config_from_json,
                                                   model_spec, synthetic_weights, tensor_shapes)

F64 = torch.float64
CFG = {
    "architecture": "Sikazen", "width": 24, "vocab": 50, "norm": {"eps": 1e-3}, "embedding": {"scale": 3.0},
    "token_side": {"dim": 4}, "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        {"type": "hgrn2", "mixer": {"heads": 2, "dim": 5, "vdim": 3}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 3, "scale": 0.3, "mask": {"size": 8, "pool": 3},
                                        "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 2.0}}}, "mlp": {"kind": "dense", "ff": 7}},
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 4, "rot_dim": 2, "vdim": 5, "kv_rank": 6, "q_rank": 7, "scale": 0.4,
                                               "rot": {"base": 50.0, "dims": 2}}, "mlp": {"kind": "dense", "ff": 9}},
        {"type": "attention", "mixer": {"heads": 2, "dim": 4, "vdim": 4, "scale": 0.5, "mask": {"size": 5, "pool": 40},
                                        "rot": {"base": 10.0, "dims": 2}}, "mlp": None},
    ],
}


def test_config_json_to_specs():
    mc = model_config_from_json(CFG, 256, "float32")
    assert (mc.arch, mc.hidden, mc.vocab, mc.n_layers, mc.max_model_len, mc.rms_eps, mc.dtype) == ("sikazen", 24, 50, 4, 256, 1e-3, "float32")
    assert (mc.embed_scale, mc.side_dim, mc.loop) == (3.0, 4, (1, 3, 3))
    a, b, c, d = mc.layers
    assert (a.kind, a.heads, a.dim, a.vdim, a.ff) == ("hgrn2", 2, 5, 3, 0)
    assert (b.heads, b.kv_heads, b.dim, b.vdim, b.scale, b.window, b.pool, b.rot_dims, b.rot_base, b.rot_linear, b.ff) == \
        (4, 2, 6, 3, 0.3, 8, 3, 4, 100.0, 2.0, 7)
    assert (c.heads, c.dim, c.rot_dim, c.vdim, c.kv_rank, c.q_rank, c.scale, c.rot_dims, c.rot_linear, c.ff) == (3, 4, 2, 5, 6, 7, 0.4, 2, 0.0, 9)
    assert (d.kv_heads, d.window, d.pool, d.rot_linear) == (2, 5, 40, 0.0)       # kv_heads defaults to heads, no scaling
    spec, keep = model_spec(mc)
    assert spec.n_layers == 4 and spec.dtype == _lib.DTYPE_F32 and spec.style == _lib.STYLE_PARALLEL_PAIR
    assert (spec.embed_scale, spec.side_dim, spec.loop_start, spec.loop_stop, spec.loop_times) == (3.0, 4, 1, 3, 3)
    assert [k.mixer for k in keep] == [_lib.MIXER_HGRN, _lib.MIXER_POOLED_ATTENTION, _lib.MIXER_LATENT_ATTENTION, _lib.MIXER_POOLED_ATTENTION]
    assert [k.mlp for k in keep] == [_lib.MLP_NONE, _lib.MLP_DENSE_SILU, _lib.MLP_DENSE_SILU, _lib.MLP_NONE]
    assert keep[1].flags == _lib.LAYER_QKV_BIAS | _lib.LAYER_UNIT_QK
    assert keep[2].flags == _lib.LAYER_ROT_INTERLEAVED | _lib.LAYER_SINK | _lib.LAYER_NO_OUT_GATE
    assert (keep[1].pool, keep[1].window, keep[1].rot_linear, keep[2].window) == (3, 8, 2.0, 0)
    back = model_config_from_json(config_json(mc), 256, "float32")
    assert back.layers == mc.layers and back.loop == mc.loop and back.side_dim == mc.side_dim      # round trip
    with pytest.raises(ValueError):
        model_config_from_json({**CFG, "layers": [{**CFG["layers"][0], "type": "something_else"}]}, None)
    with pytest.raises(ValueError):
        model_config_from_json({**CFG, "layers": [{**CFG["layers"][1], "mlp": {"kind": "moe"}}]}, None)
    plain = model_config_from_json({k: v for k, v in CFG.items() if k not in ("loop", "token_side", "embedding")}, None)
    assert (plain.loop[2], plain.side_dim, plain.embed_scale) == (1, 0, 1.0)


def test_layer_runs_and_cache_accounting():
    mc = model_config_from_json(CFG, 256)
    assert layer_runs(mc) == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [i for i, _ in O.layer_runs(CFG)] == layer_runs(mc)
    assert [add for _, add in O.layer_runs(CFG)] == [False, False, False, True, False, True, False, False]
    # per 32-token page: three runs of layer 1 (2 kv heads x (6 + 3), 32 rows + ceil(32 / 3) pooled rows), three of layer 2
    # (6 + 2 per row), one of layer 3 (2 x (4 + 4), 32 rows + 1 pooled row)
    assert cache_block_elems(mc, 32) == 3 * (32 + 11) * 2 * 9 + 3 * 32 * 8 + (32 + 1) * 2 * 8
    no_loop = model_config_from_json({**CFG, "loop": {"start": 0, "stop": 4, "times": 1}}, 256)
    assert layer_runs(no_loop) == [0, 1, 2, 3]
    whole = model_config_from_json({**CFG, "loop": {"start": 0, "stop": 4, "times": 2}}, 256)
    assert layer_runs(whole) == [0, 1, 2, 3, 0, 1, 2, 3]


def test_parameter_list_and_presets():
    mc = model_config_from_json(CFG, 256)
    shapes = tensor_shapes(mc)
    assert shapes["embed"] == (50, 24) and shapes["side.embed"] == (50, 16) and shapes["final.norm"] == () and shapes["l1.norm2"] == ()
    assert "l0.norm2" not in shapes and "l3.mlp.gate" not in shapes
    assert shapes["l1.mix.k.b"] == (12,) and shapes["l2.mix.dkv"] == (8, 24) and shapes["l2.mix.uq"] == (18, 7) and shapes["l2.mix.sink"] == (3,)
    assert shapes["l0.mix.lower"] == (10,) and shapes["l0.mix.norm"] == (3,) and shapes["l3.side.proj"] == (24, 4)
    w = synthetic_weights(mc, 3)
    assert set(w) == set(shapes) and all(tuple(w[k].shape) == shapes[k] and w[k].dtype == torch.bfloat16 for k in shapes)
    assert float(w["l0.mix.lower"].min()) >= 0.0 and float(w["l0.mix.lower"].max()) < 1.0
    for name, p in PRESETS.items():
        assert p.arch == "sikazen" and model_config_from_json(config_json(p), None).layers == p.layers, name
        for l in p.layers:
            assert l.rot_dims % 2 == 0 and (l.kind != "attention" or l.heads % l.kv_heads == 0)


def _eye(n):
    return torch.eye(n, dtype=F64)


def _attn_w(H, G, d, dv):
    width = H * d + G * d + G * dv
    rows = lambda a, n: _eye(width)[a:a + n]  # noqa: E731
    return width, {"q": rows(0, H * d), "k": rows(H * d, G * d), "v": rows(H * d + G * d, G * dv), "q.b": torch.zeros(H * d, dtype=F64),
                   "k.b": torch.zeros(G * d, dtype=F64), "v.b": torch.zeros(G * dv, dtype=F64), "o": _eye(H * dv)}


def test_oracle_window_and_pooled_block_edges():
    """A marked value is seen one by one while its token is inside the window, not at all while its block is incomplete
    behind the window, and through the block's mean from the token on at which the block's last position leaves the window."""
    m = dict(heads=1, kv_heads=1, dim=2, vdim=1, scale=1.0, mask=dict(size=4, pool=3), rot=dict(base=10.0, dims=0))
    width, w = _attn_w(1, 1, 2, 1)
    T, j = 16, 4                                   # block 1 = positions 3, 4, 5
    h = torch.zeros(T, width, dtype=F64)
    h[:, 0] = h[:, 2] = 1.0                        # equal queries and keys: uniform weights over whatever is visible
    h[j, 4] = 1.0                                  # the marked value
    out = O.pooled_window_attention(h, w, m, 1e-6)[:, 0]
    for i in range(T):
        if i < j:
            want = 0.0
        elif i - j < 4:
            want = 1.0 / min(i + 1, 4 + max(0, (i - 3) // 3))      # a token among the window's tokens and the visible blocks
        elif 5 > i - 4:
            want = 0.0                                              # behind the window, block 1 not complete at i - 4
        else:
            want = (1.0 / 3.0) / (4 + (i - 3) // 3)                 # a third of block 1's mean
        assert abs(float(out[i]) - want) < 1e-12, (i, float(out[i]), want)
    no_pool = O.pooled_window_attention(h, w, dict(m, mask=dict(size=4, pool=0)), 1e-6)[:, 0]
    assert float(no_pool[j + 3]) == 0.25 and float(no_pool[j + 4:].abs().max()) == 0.0


def test_oracle_sink_and_rotary_layouts():
    m = dict(heads=2, dim=2, rot_dim=4, vdim=3, kv_rank=5, q_rank=6, scale=0.3, rot=dict(base=7.0, dims=4))
    g = torch.Generator().manual_seed(1)
    w = {k: torch.randn(s, generator=g, dtype=F64) for k, s in dict(dq=(6, 10), uq=(12, 6), dkv=(9, 10), uk=(4, 5), uv=(6, 5), o=(10, 6)).items()}
    w.update({"dq.norm": torch.ones(6, dtype=F64), "dkv.norm": torch.ones(5, dtype=F64)})
    h = torch.randn(9, 10, generator=g, dtype=F64)
    far = O.latent_sink_attention(h, {**w, "sink": torch.full((2,), -1e9, dtype=F64)}, m, 1e-6)    # a sink that weighs nothing
    half = O.latent_sink_attention(h, {**w, "sink": torch.full((2,), 50.0, dtype=F64)}, m, 1e-6)   # ... that takes all the weight
    assert float(half.abs().max()) < 1e-12 * max(1.0, float(far.abs().max())) * 1e3 and float(far.abs().max()) > 1e-3
    # the first token: softmax over itself and the sink
    one = O.latent_sink_attention(h[:1], {**w, "sink": torch.zeros(2, dtype=F64)}, m, 1e-6)
    none = O.latent_sink_attention(h[:1], {**w, "sink": torch.full((2,), -1e9, dtype=F64)}, m, 1e-6)
    a = h[:1] @ w["dkv"].T
    c = O.rms(a[:, :5], 1e-6)
    q = (O.rms(h[:1] @ w["dq"].T, 1e-6) @ w["uq"].T).view(1, 2, 6)
    for hh in range(2):
        s = float((q[0, hh, :2] @ (c @ w["uk"].T).view(1, 2, 2)[0, hh] + q[0, hh, 2:] @ a[0, 5:]) * 0.3)    # position 0: no turn
        share = math.exp(s) / (math.exp(s) + 1.0)
        assert torch.allclose(one.new_tensor(share) * (none @ torch.linalg.pinv(w["o"].T))[0, hh * 3:hh * 3 + 3],
                              (one @ torch.linalg.pinv(w["o"].T))[0, hh * 3:hh * 3 + 3], atol=1e-9)
    # the two layouts turn the same pairs: interleaving the halves of a vector and rotating pairwise = rotating halves
    x = torch.randn(5, 1, 6, generator=g, dtype=F64)
    rot = dict(base=9.0, dims=4, scaling=dict(factor=3.0))
    a_ = O.rotate_half(x, rot)
    perm = [0, 2, 1, 3, 4, 5]
    b_ = O.rotate_pairs(x[..., perm], rot)
    assert torch.allclose(a_[..., perm], b_, atol=1e-12)
    assert torch.allclose(O.frequencies(rot), torch.tensor([1.0, 9.0 ** -0.5], dtype=F64) / 3.0)


def test_oracle_state_and_loop():
    m = dict(heads=2, dim=3, vdim=2)
    g = torch.Generator().manual_seed(2)
    w = {"q": torch.randn(6, 8, generator=g, dtype=F64), "f": torch.randn(6, 8, generator=g, dtype=F64),
         "v": torch.randn(4, 8, generator=g, dtype=F64), "f.b": torch.randn(6, generator=g, dtype=F64),
         "lower": torch.rand(6, generator=g, dtype=F64), "norm": torch.ones(2, dtype=F64), "o": _eye(4)}
    h = torch.randn(12, 8, generator=g, dtype=F64)
    full = O.hgrn2(h, w, m, 1e-6)
    assert torch.allclose(full[:7], O.hgrn2(h[:7], w, m, 1e-6), atol=1e-12)          # causal
    # a gate bounded below by one never forgets and never writes: the state stays zero
    still = O.hgrn2(h, {**w, "lower": torch.ones(6, dtype=F64)}, m, 1e-6)
    assert float(still.abs().max()) == 0.0
    mc = model_config_from_json(CFG, 64)
    weights = synthetic_weights(mc, 5)
    toks = [3, 9, 1, 40, 22, 7, 7, 30, 2, 11, 5, 48]
    runs = []
    logits = O.forward(CFG, weights, toks, runs)
    assert logits.shape == (12, 50) and len(runs) == 8
    assert torch.allclose(O.forward(CFG, weights, toks[:5]), logits[:5], atol=1e-9)   # causal through every mechanism
    once = O.forward({**CFG, "loop": {"start": 1, "stop": 3, "times": 1}}, weights, toks)
    assert float((once - logits).abs().max()) > 1e-3
    assert O.greedy(CFG, weights, toks[:4], 3) == O.greedy(CFG, weights, toks[:4], 5)[:3]
