"""CPU-side checks of the Revepel family: config.json (+ checkpoint header) -> engine specs, the parameter list, presets, and
properties of the plain oracle that the GPU tests lean on (the window's edges, shared keys and values, the rotary scaling's
limits, the token shift, state carried token by token, weighted expert inputs)."""
import json
import math
import struct

import pytest
import torch

from oracle import revepel_oracle as O
from vllm_tgis_adapter_b200.engine import _lib
from vllm_tgis_adapter_b200.engine.revepel import (PRESETS, config_json, model_config_from_json, model_spec, synthetic_weights,
                                                   tensor_shapes)

F64 = torch.float64
ROT = {"base": 100.0, "dims": 4, "scaling": {"factor": 4.0, "original": 32, "fast": 4.0, "slow": 1.0}}
CFG = {
    "architecture": "Revepel", "width": 24, "vocab": 50, "norm": {"eps": 1e-3}, "embedding": {"scale": 3.0}, "logit_scale": 0.5,
    "layers": [
        {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 5, "vdim": 3, "conv": 3}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 3, "scale": 0.3, "mask": {"size": 5}, "rot": ROT},
         "mlp": {"kind": "moe", "router": {"experts": 5, "top": 2}, "expert": {"ff": 7}, "shared": {"ff": 9}}},
        {"type": "mamba2", "mixer": {"heads": 4, "vdim": 3, "state": 5, "groups": 2, "norm_groups": 2, "conv": 4},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 1}, "expert": {"ff": 4}}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 3, "scale": 0.3, "mask": {"size": 11}, "rot": ROT,
                                        "kv_from": 1}, "mlp": None},
    ],
}
SHAPES = {"l0.mix.a1": (7, 24), "l0.mix.g1": (2, 24)}


def test_config_json_to_specs():
    mc = model_config_from_json(CFG, 256, "float32", SHAPES)
    assert (mc.arch, mc.hidden, mc.vocab, mc.n_layers, mc.max_model_len, mc.rms_eps, mc.dtype) == ("revepel", 24, 50, 4, 256, 1e-3, "float32")
    assert (mc.embed_scale, mc.logit_scale) == (3.0, 0.5)
    a, b, c, d = mc.layers
    assert (a.kind, a.heads, a.kv_heads, a.dim, a.vdim, a.conv, a.decay_rank, a.gate_rank, a.experts) == ("channel_delta", 4, 2, 5, 3, 3, 7, 2, 0)
    assert (b.heads, b.kv_heads, b.dim, b.vdim, b.scale, b.window, b.rot_dims, b.rot_base, b.yarn, b.kv_from) == \
        (4, 2, 6, 3, 0.3, 5, 4, 100.0, (4.0, 32.0, 4.0, 1.0), None)
    assert (b.experts, b.top, b.expert_ff, b.shared_ff) == (5, 2, 7, 9)
    assert (c.heads, c.vdim, c.state, c.groups, c.norm_groups, c.conv, c.experts, c.top, c.shared_ff) == (4, 3, 5, 2, 2, 4, 3, 1, 0)
    assert (d.kv_from, d.window) == (1, 11)
    spec, keep = model_spec(mc)
    assert spec.n_layers == 4 and spec.dtype == _lib.DTYPE_F32 and spec.style == _lib.STYLE_PARALLEL_GATED
    assert (spec.embed_scale, spec.logit_scale) == (3.0, 0.5)
    assert [k.mixer for k in keep] == [_lib.MIXER_CHANNEL_DELTA, _lib.MIXER_SIGMOID_ATTENTION, _lib.MIXER_SSD, _lib.MIXER_SIGMOID_ATTENTION]
    assert [k.mlp for k in keep] == [_lib.MLP_NONE, _lib.MLP_MOE_SIGMOID, _lib.MLP_MOE_SIGMOID, _lib.MLP_NONE]
    assert [k.kv_from for k in keep] == [0, 0, 0, 2]                       # the ABI counts the source layer from one
    assert (keep[1].yarn_factor, keep[1].yarn_original, keep[1].yarn_fast, keep[1].yarn_slow) == (4.0, 32.0, 4.0, 1.0)
    assert model_config_from_json(config_json(mc), 256, "float32").layers == mc.layers      # round trip
    with pytest.raises(ValueError):
        model_config_from_json({**CFG, "layers": [{**CFG["layers"][0], "type": "something_else"}]}, None, shapes=SHAPES)
    with pytest.raises(ValueError):
        model_config_from_json(CFG, None)                                                    # the ranks are nowhere
    with pytest.raises(ValueError):
        model_config_from_json({**CFG, "layers": [{**CFG["layers"][1], "mlp": {"kind": "dense", "ff": 3}}]}, None)
    # optional parts: no scaling, no window, kv_heads defaults to heads
    l = model_config_from_json({**CFG, "layers": [{"type": "attention", "mlp": None, "mixer": {
        "heads": 2, "dim": 4, "vdim": 4, "scale": 0.5, "rot": {"base": 10.0, "dims": 2}}}]}, None).layers[0]
    assert (l.kv_heads, l.yarn, l.window) == (2, None, 0)


def test_loader_reads_family_and_ranks_from_the_checkpoint(tmp_path):
    from vllm_tgis_adapter_b200.engine.loader import model_config_from_hf

    (tmp_path / "config.json").write_text(json.dumps(CFG))
    header = json.dumps({"l0.mix.a1": {"dtype": "BF16", "shape": [5, 24], "data_offsets": [0, 240]},
                         "l0.mix.g1": {"dtype": "BF16", "shape": [3, 24], "data_offsets": [240, 384]}}).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(header)) + header + bytes(384))
    mc = model_config_from_hf(tmp_path, 128, "bfloat16")
    assert mc.arch == "revepel" and (mc.layers[0].decay_rank, mc.layers[0].gate_rank) == (5, 3) and mc.max_model_len == 128


def test_parameter_list_and_presets():
    mc = model_config_from_json(CFG, 64, shapes=SHAPES)
    shapes = tensor_shapes(mc)
    assert shapes["l0.mix.a2"] == (20, 7) and shapes["l0.mix.dt_bias"] == (20,) and shapes["l0.mix.norm"] == (3,)
    assert shapes["l2.mix.in"] == (2 * 12 + 2 * 10 + 4, 24) and shapes["l2.mix.conv"] == (12 + 20, 4)
    assert "l3.mix.k" not in shapes and "l3.mix.v" not in shapes and shapes["l3.mix.q"] == (24, 24)
    assert "l0.rg2" not in shapes and shapes["l1.rg2"] == (24, 24) and shapes["l1.mlp.e4.down"] == (24, 7)
    w = synthetic_weights(mc, 3)
    assert set(w) == set(shapes) and all(tuple(w[k].shape) == v and w[k].dtype == torch.bfloat16 for k, v in shapes.items())
    for name, p in PRESETS.items():
        assert p.arch == "revepel" and len(tensor_shapes(p)) > 0, name
        for i, l in enumerate(p.layers):
            if l.kv_from is not None:
                o = p.layers[l.kv_from]
                assert l.kv_from < i and o.kind == "attention" and o.kv_from is None and (o.kv_heads, o.dim, o.vdim) == (l.kv_heads, l.dim, l.vdim)


def _attn_weights(m, width, gen):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    r = lambda *s: torch.randn(*s, generator=gen, dtype=F64)  # noqa: E731
    return {"q": r(H * d, width), "k": r(G * d, width), "v": r(G * dv, width), "pb": r(H), "o": r(width, H * dv)}


def test_oracle_window_edges_and_shared_keys():
    gen = torch.Generator().manual_seed(0)
    m = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 3, "scale": 0.3, "mask": {"size": 5}, "rot": ROT}
    w = _attn_weights(m, 10, gen)
    h = torch.randn(20, 10, generator=gen, dtype=F64)
    base = O.sigmoid_attention(h, w, m, O.attention_kv(h, w, m))
    h2 = h.clone()
    h2[7] += 1.0                                       # token 7 is a key for queries 7 .. 11 only
    moved = (O.sigmoid_attention(h2, w, m, O.attention_kv(h2, w, m)) - base).abs().amax(-1) > 1e-9
    assert moved.nonzero().flatten().tolist() == [7, 8, 9, 10, 11]
    # another layer's keys and values, this layer's own queries and window
    wide = {**m, "mask": {"size": 9}}
    kv = O.attention_kv(h2, w, m)
    out = O.sigmoid_attention(h, w, wide, kv)
    assert not torch.allclose(out, O.sigmoid_attention(h, w, wide, O.attention_kv(h, w, m)))
    # weights are not normalised: two identical visible keys count twice
    one = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1, "scale": 1.0, "mask": {"size": 8}, "rot": {"base": 10.0, "dims": 0}}
    w1 = {"q": torch.zeros(2, 3, dtype=F64), "k": torch.zeros(2, 3, dtype=F64), "v": torch.tensor([[0.0, 0.0, 1.0]], dtype=F64),
          "pb": torch.tensor([0.0], dtype=F64), "o": torch.ones(1, 1, dtype=F64)}
    hh = torch.zeros(3, 3, dtype=F64)
    hh[:, 2] = 1.0
    assert torch.allclose(O.sigmoid_attention(hh, w1, one, O.attention_kv(hh, w1, one)).flatten(), torch.tensor([0.5, 1.0, 1.5], dtype=F64))


def test_oracle_rotary_scaling_limits():
    plain, _ = O.yarn_frequencies({"base": 100.0, "dims": 8})
    assert torch.allclose(plain, torch.tensor([100.0 ** (-2 * i / 8) for i in range(4)], dtype=F64))
    f, mag = O.yarn_frequencies({"base": 100.0, "dims": 8, "scaling": {"factor": 1.0, "original": 64, "fast": 8.0, "slow": 1.0}})
    assert torch.allclose(f, plain) and mag == 1.0                       # factor one changes nothing
    f, mag = O.yarn_frequencies({"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}})
    assert mag == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert f[0] == plain[0] and f[-1] == pytest.approx(float(plain[-1]) / 4.0) and all(plain[i] / 4 <= f[i] <= plain[i] for i in range(4))
    # a rotation keeps the length of every pair (up to the magnitude) and leaves the unrotated tail alone
    x = torch.randn(5, 2, 10, generator=torch.Generator().manual_seed(1), dtype=F64)
    rot = {"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    y = O.rotate(x, rot)
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.allclose(y[0, ..., :8], x[0, ..., :8] * mag)
    assert torch.allclose(y[..., :4] ** 2 + y[..., 4:8] ** 2, (x[..., :4] ** 2 + x[..., 4:8] ** 2) * mag ** 2)


def test_oracle_state_is_carried_token_by_token_and_experts_weigh_their_input():
    mc = model_config_from_json(CFG, 64, shapes=SHAPES)
    w = synthetic_weights(mc, 5)
    toks = torch.randint(0, 50, (40,), generator=torch.Generator().manual_seed(2)).tolist()
    full = O.forward(CFG, w, toks)
    assert torch.allclose(O.forward(CFG, w, toks[:17]), full[:17], atol=1e-9)     # causal: a prefix does not see what follows
    assert torch.isfinite(full).all() and full.shape == (40, 50)
    # token shift: the first token blends with zeros
    n = torch.randn(3, 4, dtype=F64)
    s = torch.tensor([0.0, 1.0, 0.25, 0.5], dtype=F64)
    t = O.token_shift(n, s)
    assert torch.allclose(t[0], n[0] * (1 - s)) and torch.allclose(t[2], n[2] + (n[1] - n[2]) * s)
    # an expert runs on its input row scaled by its score: with squared ReLU the output scales with the score's square
    mlp = {"router": {"experts": 1, "top": 1}, "expert": {"ff": 3}}
    ew = {"router": torch.tensor([[2.0, 0.0]], dtype=F64), "e0.up": torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]], dtype=F64),
          "e0.down": torch.ones(2, 3, dtype=F64)}
    h = torch.tensor([[0.5, 1.0]], dtype=F64)
    sc = 1.0 / (1.0 + math.exp(-1.0))
    assert torch.allclose(O.moe(h, ew, mlp), torch.full((1, 2), sc * sc * (0.25 + 1.0 + 2.25), dtype=F64))
