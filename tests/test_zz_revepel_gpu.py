"""-m gpu parity of the Revepel architecture against oracle/revepel_oracle.py.

Kernel level (include/tgis_kernels.h hooks): sigmoid attention over a paged cache in portions, with inputs built so that ONE
key decides a query's output -- just inside and just outside the window, on both sides of a cache block's border, the first
token, far away -- in fp32 and on the bf16 tensor-core path; the delta-rule scan in portions through two state slots.
Engine level (trace replay = the engine's own step function, sequence slots and block manager): every mixer alone, whole
prompts in fp32 and bf16, portions down to two tokens, token-by-token decoding, mixed batches against each request alone
with blocks and state slots that are used again, long decoding across window and block borders, other sizes and layer
orders (values equal to 1, parts absent, shared keys and values), and greedy generation through add_request + the step
loop with and without CUDA-graph replay."""
import ctypes as C
import json
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

F32, BF16 = 0, 1
KV_BLOCK = 32
F64 = torch.float64


def _lib():
    from vllm_tgis_adapter_b200.engine import _lib as L

    return L.load_library()


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _ok(rc):
    assert rc == 0, (_lib().tgis_k_last_error() or b"").decode()


_KEEP = []   # device tensors whose pointers went into a C call stay alive until the test ends


@pytest.fixture(autouse=True)
def _release_device_tensors():
    yield
    _KEEP.clear()


def _dev(t, dt=torch.float32):
    d = t.to(dt).cuda().contiguous()
    _KEEP.append(d)
    return d


def _ints(v):
    return (C.c_int32 * len(v))(*v)


def _i32(v):
    d = torch.tensor(v, dtype=torch.int32).cuda()
    _KEEP.append(d)
    return d


def _portions(total, sizes):
    out, at, i = [], 0, 0
    while at < total:
        n = min(sizes[i % len(sizes)], total - at)
        out.append((at, n))
        at += n
        i += 1
    return out


def _eye_rows(width, start, n):
    w = torch.zeros(n, width, dtype=F64)
    w[torch.arange(n), start + torch.arange(n)] = 1.0
    return w


# ====================================================================================================== attention kernels
def _run_sigattn(h, m, pb, dt, sizes, pool_blocks=24, seed=0):
    """h [T, width] whose columns are [q | k | v]: the sequence goes through the kernels in portions of the given sizes over a
    paged cache whose blocks are scattered through the pool.  Returns the heads' outputs [T, heads * vdim]."""
    from oracle import revepel_oracle as O
    from vllm_tgis_adapter_b200.engine._lib import TgisKSigAttnGeom

    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rd = int(m["rot"]["dims"])
    tdt = torch.bfloat16 if dt == BF16 else torch.float32
    geom = TgisKSigAttnGeom(H, G, d, dv, int(m["mask"]["size"]), rd, float(m["scale"]))
    f, mag = O.yarn_frequencies(m["rot"])
    ang = torch.arange(T, dtype=F64)[:, None] * f[None, :]
    table = _dev(torch.cat([torch.cos(ang) * mag, torch.sin(ang) * mag], -1)) if rd > 0 else None
    n_blocks = (T + KV_BLOCK - 1) // KV_BLOCK
    blocks = torch.randperm(pool_blocks, generator=torch.Generator().manual_seed(seed))[:n_blocks].tolist()
    kc = torch.randn(pool_blocks * KV_BLOCK, G * d, device="cuda").to(tdt)     # stale rows of earlier owners: finite, never visible
    vc = torch.randn(pool_blocks * KV_BLOCK, G * dv, device="cuda").to(tdt)
    y = _dev(h)
    out = torch.full((T, H * dv), float("nan"), dtype=tdt, device="cuda")
    pb_d = _dev(pb)
    for at, n in _portions(T, sizes):
        pos = list(range(at, at + n))
        slots = [blocks[p // KV_BLOCK] * KV_BLOCK + p % KV_BLOCK for p in pos]
        q = torch.zeros(n, H * d, dtype=tdt, device="cuda")
        yp = y[at:at + n].contiguous()
        _ok(_lib().tgis_k_sigattn_prep(_p(yp), y.shape[1], 0, H * d, H * d + G * d, C.byref(geom), _p(table), _p(_i32(pos)),
                                       _p(_i32(slots)), _p(q), _p(kc), _p(vc), dt, n))
        o = torch.full((n, H * dv), float("nan"), dtype=tdt, device="cuda")
        _ok(_lib().tgis_k_sigattn(_p(q), _p(kc), _p(vc), dt, _ints([0, n, at + n, 0]), 1, _ints(blocks), 1, len(blocks), _p(pb_d),
                                  _p(o), C.byref(geom)))
        out[at:at + n] = o
    return out


def _sig_weights(m, pb):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    width = H * d + G * d + G * dv
    return width, {"q": _eye_rows(width, 0, H * d), "k": _eye_rows(width, H * d, G * d), "v": _eye_rows(width, H * d + G * d, G * dv),
                   "pb": pb.double(), "o": torch.eye(H * dv, dtype=F64)}


_ATTN = [
    dict(heads=4, kv_heads=2, dim=6, vdim=10, scale=0.4, mask=dict(size=9), rot=dict(base=50.0, dims=4)),
    dict(heads=3, kv_heads=1, dim=40, vdim=33, scale=0.2, mask=dict(size=70),
         rot=dict(base=1000.0, dims=40, scaling=dict(factor=4.0, original=64, fast=8.0, slow=1.0))),
    dict(heads=2, kv_heads=2, dim=5, vdim=140, scale=0.5, mask=dict(size=1), rot=dict(base=10.0, dims=0)),
    dict(heads=1, kv_heads=1, dim=64, vdim=64, scale=0.125, mask=dict(size=33), rot=dict(base=10000.0, dims=32)),
    # sizes the tensor-core kernel takes in bf16
    dict(heads=2, kv_heads=2, dim=96, vdim=200, scale=0.1, mask=dict(size=300), rot=dict(base=500.0, dims=96)),
    dict(heads=4, kv_heads=2, dim=32, vdim=48, scale=0.2, mask=dict(size=32),
         rot=dict(base=20000.0, dims=16, scaling=dict(factor=8.0, original=128, fast=16.0, slow=2.0))),
]


@pytest.mark.parametrize("m", _ATTN)
def test_sigmoid_attention_in_portions_matches_oracle(m):
    from oracle import revepel_oracle as O

    T = 150
    pb = torch.randn(m["heads"], generator=torch.Generator().manual_seed(2)) - 2.0
    width, w = _sig_weights(m, pb)
    h = torch.randn(T, width, generator=torch.Generator().manual_seed(1), dtype=F64).float().double()
    ref = O.sigmoid_attention(h, w, m, O.attention_kv(h, w, m))
    for sizes in ([T], [1], [2], [5, 31, 1, 33, 16, 2]):
        got = _run_sigattn(h, m, pb, F32, sizes)
        err = float((got.double().cpu() - ref).abs().max() / ref.abs().max())
        assert err < 2e-5, (sizes, err)
    hb = h.to(torch.bfloat16).double()
    refb = O.sigmoid_attention(hb, w, m, O.attention_kv(hb, w, m))
    for sizes in ([T], [7, 1, 40, 2]):
        got = _run_sigattn(hb, m, pb, BF16, sizes)
        err = float((got.double().cpu() - refb).abs().max() / refb.abs().max())
        assert err < 3e-2, (sizes, err)


@pytest.mark.parametrize("dt,m", [(F32, _ATTN[0]), (F32, _ATTN[3]), (BF16, _ATTN[3]), (BF16, _ATTN[4]), (BF16, _ATTN[5])])
def test_one_key_decides_at_window_and_block_edges(dt, m):
    """Every key but one weighs next to nothing (bias -12); the one whose (unrotated) key equals the query direction weighs
    nearly one, and its value is a code of its position.  The query's output then names the key it saw -- or nothing, if
    that key lies outside the window."""
    from oracle import revepel_oracle as O

    m = {**m, "rot": {**m["rot"], "dims": 0}}       # no rotation: the chosen pair's score does not move with the distance
    H, G, d, dv, win = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["mask"]["size"]
    T = 400
    pb = torch.full((H,), -12.0)
    width, w = _sig_weights(m, pb)
    gen = torch.Generator().manual_seed(5)
    big = math.sqrt(24.0 / m["scale"])              # chosen pair: score 24, weight sigmoid(24 - 12) = 1 - 6e-6
    for target_of in (lambda i: i - (win - 1), lambda i: i - win, lambda i: (i // KV_BLOCK) * KV_BLOCK - 1,
                      lambda i: (i // KV_BLOCK) * KV_BLOCK, lambda i: 0, lambda i: i):
        h = torch.randn(T, width, generator=gen, dtype=F64) * 0.05
        queries = [37, 63, 64, 65, 127, 128, 200, 333, 399]
        targets = {}
        for n, i in enumerate(queries):
            j = target_of(i)
            if j < 0 or j in targets.values() or j in queries:
                continue
            targets[i] = j
            u = torch.zeros(d, dtype=F64)
            u[n % d] = big
            h[i, :H * d] = u.repeat(H)                          # every head of query i looks along u
            h[j, H * d:H * d + G * d] = u.repeat(G)             # ... and key j lies along it
            h[j, H * d + G * d:] = 1.0 + j / 50.0               # the value says which key it was
        if dt == BF16:
            h = h.to(torch.bfloat16).double()
        ref = O.sigmoid_attention(h, w, m, O.attention_kv(h, w, m))
        got = _run_sigattn(h, m, pb, dt, [64, 1, 1, 62, 3, 33], seed=3).double().cpu()
        tol = 2e-2 if dt == BF16 else 1e-4
        for i, j in targets.items():
            seen = 0 <= i - j < win
            assert abs(float(ref[i, 0]) - ((1.0 + j / 50.0) if seen else 0.0)) < 0.05, (i, j)      # the oracle agrees with the story
            assert float((got[i] - ref[i]).abs().max()) < tol * max(1.0, float(ref[i].abs().max())), (i, j, seen)


def test_delta_rule_scan_in_portions_and_two_slots_matches_oracle():
    """delta_scan_kernel against the oracle's channel_delta with selector projections, one-tap convolutions of weight one, unit
    norm weight and a gate fixed at one half: what is compared is the RMS-normed read-out."""
    from oracle import revepel_oracle as O

    for (H, G, d, dv, T) in ((4, 2, 6, 5, 70), (2, 2, 64, 40, 50), (3, 1, 130, 33, 40), (1, 1, 1, 1, 20)):
        eps, ra = 1e-5, 3
        gen = torch.Generator().manual_seed(H * 100 + d)
        qk, hv = G * d, H * dv
        width = 2 * qk + hv + H + ra
        m = dict(heads=H, kv_heads=G, dim=d, vdim=dv, conv=1)
        w = {"q": _eye_rows(width, 0, qk), "k": _eye_rows(width, qk, qk), "v": _eye_rows(width, 2 * qk, hv),
             "b": _eye_rows(width, 2 * qk + hv, H), "a1": _eye_rows(width, 2 * qk + hv + H, ra),
             "a2": torch.randn(H * d, ra, generator=gen, dtype=F64), "dt_bias": torch.randn(H * d, generator=gen, dtype=F64) - 1.0,
             "A_log": torch.randn(H, generator=gen, dtype=F64) * 0.3, "norm": torch.ones(dv, dtype=F64),
             "g1": torch.zeros(2, width, dtype=F64), "g2": torch.zeros(hv, 2, dtype=F64), "o": torch.eye(hv, dtype=F64)}
        for s in "qkv":
            w[s + ".conv"] = torch.ones(w[s].shape[0], 1, dtype=F64)
        hs = [torch.randn(T, width, generator=gen, dtype=F64).float().double() for _ in range(2)]
        refs = [O.channel_delta(h, w, m, eps) for h in hs]
        S = torch.full((3, H, d, dv), float("nan"), device="cuda")      # slots 2 and 0; a fresh sequence never reads its slot
        outs = [torch.zeros(T, hv, device="cuda") for _ in range(2)]
        for at, n in _portions(T, [5, 1, 2, 17, 1]):
            for r, slot in ((0, 2), (1, 0)):                            # the two sequences advance in separate launches
                h = hs[r][at:at + n]
                act = O.silu(h[:, :2 * qk + hv])
                dec = (h[:, 2 * qk + hv + H:] @ w["a2"].T)
                o = torch.zeros(n, hv, device="cuda")
                _ok(_lib().tgis_k_delta_scan(_p(_dev(act[:, :qk])), _p(_dev(act[:, qk:2 * qk])), _p(_dev(act[:, 2 * qk:])), qk, qk, hv,
                                             _p(_dev(dec)), H * d, _p(_dev(w["dt_bias"])), _p(_dev(w["A_log"])),
                                             _p(_dev(h[:, 2 * qk + hv:2 * qk + hv + H])), H, _p(S), _p(o), hv, H, G, d, dv,
                                             _ints([0, n, at + n, 0]), 1, _p(_i32([slot] * n))))
                outs[r][at:at + n] = o
        for r in range(2):
            got = O.rms(outs[r].double().cpu().view(T, H, dv), eps).reshape(T, hv) * 0.5
            err = float((got - refs[r]).abs().max() / refs[r].abs().max())
            assert err < 5e-5, (H, G, d, dv, r, err)


def test_state_space_scan_in_portions_and_two_slots_matches_oracle():
    """outer_scan_kernel's state-space mode against the oracle's mamba2 with selector projections, a one-tap convolution of
    weight one and unit norm weight: what is compared is the gated, RMS-normed read-out."""
    from oracle import revepel_oracle as O

    for (H, G, N, P, T) in ((6, 3, 5, 4, 70), (4, 1, 64, 40, 50), (2, 2, 200, 33, 40), (1, 1, 1, 1, 20)):
        eps, inner, gn = 1e-5, H * P, G * N
        gen = torch.Generator().manual_seed(H * 100 + N)
        width = 2 * inner + 2 * gn + H
        m = dict(heads=H, vdim=P, state=N, groups=G, norm_groups=1, conv=1)
        w = {"in": torch.eye(width, dtype=F64), "conv": torch.ones(inner + 2 * gn, 1, dtype=F64), "conv.b": torch.zeros(inner + 2 * gn, dtype=F64),
             "dt_bias": torch.randn(H, generator=gen, dtype=F64) - 1.0, "A_log": torch.randn(H, generator=gen, dtype=F64) * 0.3,
             "D": torch.randn(H, generator=gen, dtype=F64), "norm": torch.ones(inner, dtype=F64), "o": torch.eye(inner, dtype=F64)}
        hs = [torch.randn(T, width, generator=gen, dtype=F64).float().double() for _ in range(2)]
        refs = [O.mamba2(h, w, m, eps) for h in hs]
        S = torch.full((3, H, N, P), float("nan"), device="cuda")
        outs = [torch.zeros(T, inner, device="cuda") for _ in range(2)]
        for at, n in _portions(T, [5, 1, 2, 17, 1]):
            for r, slot in ((0, 1), (1, 2)):
                h = hs[r][at:at + n]
                act = O.silu(h[:, inner:2 * inner + 2 * gn])      # x | B | C after the one-tap convolution
                o = torch.zeros(n, inner, device="cuda")
                _ok(_lib().tgis_k_ssd_scan(_p(_dev(act[:, inner + gn:])), _p(_dev(act[:, inner:inner + gn])), _p(_dev(act[:, :inner])), gn, gn,
                                           inner, _p(_dev(h[:, 2 * inner + 2 * gn:])), H, _p(_dev(w["dt_bias"])), _p(_dev(w["A_log"])),
                                           _p(_dev(w["D"])), _p(S), _p(o), inner, H, G, N, P, _ints([0, n, at + n, 0]), 1, _p(_i32([slot] * n))))
                outs[r][at:at + n] = o
        for r in range(2):
            got = O.rms(outs[r].double().cpu() * O.silu(hs[r][:, :inner]), eps)
            err = float((got - refs[r]).abs().max() / refs[r].abs().max())
            assert err < 5e-5, (H, G, N, P, r, err)


# ====================================================================================================== engine
def _moe(experts, top, ff, shared=0):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _att(heads, kv_heads, dim, vdim, window, rot_dims, scaling=True, kv_from=None, base=300.0, scale=0.3):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = {"factor": 4.0, "original": 48, "fast": 6.0, "slow": 1.5}
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}, "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _cfg(layers=None, width=40, vocab=97, logit_scale=1.7, embed_scale=5.5):
    layers = layers or [
        {"type": "mamba2", "mixer": {"heads": 6, "vdim": 4, "state": 5, "groups": 3, "norm_groups": 2, "conv": 4}, "mlp": _moe(5, 2, 12, 20)},
        {"type": "attention", "mixer": _att(4, 2, 6, 10, 9, 4), "mlp": None},
        {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "conv": 2}, "mlp": _moe(7, 3, 9)},
        {"type": "attention", "mixer": _att(4, 2, 6, 10, 37, 4, kv_from=1), "mlp": _moe(3, 1, 16, 8)},
    ]
    return {"architecture": "Revepel", "width": width, "vocab": vocab, "norm": {"eps": 1e-4}, "embedding": {"scale": embed_scale},
            "logit_scale": logit_scale, "layers": layers}


def _model(cfg, dtype="float32", max_model_len=512, ranks=(3, 4)):
    from vllm_tgis_adapter_b200.engine.revepel import model_config_from_json

    shapes = {}
    for i, l in enumerate(cfg["layers"]):
        if l["type"] == "channel_delta":
            shapes[f"l{i}.mix.a1"], shapes[f"l{i}.mix.g1"] = (ranks[0], cfg["width"]), (ranks[1], cfg["width"])
    return model_config_from_json(cfg, max_model_len, dtype, shapes)


def _engine(mc, weights, *, blocks=16, seqs=4, graphs=False, tokens=512):
    from vllm_tgis_adapter_b200.engine.core import NativeEngine, cache_block_bytes

    eng = NativeEngine(mc, max_num_seqs=seqs, max_batched_tokens=tokens, kv_cache_bytes=cache_block_bytes(mc) * blocks,
                       use_cuda_graphs=graphs)
    eng.load_weights(weights)
    return eng


def _tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _rel(got, ref):
    """Error of logit rows the way a user sees it: mean removed, root mean square, relative to the rows' own spread."""
    d = torch.as_tensor(got).double() - ref
    d = d - d.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / ref.std(-1)).max())


def _bf16_close(got, ref):
    """bf16 operands on widths this small: rounding alone moves single rows by several percent of their spread, so the bound
    is on the typical row and on the tail (the sharp comparison is the float32 one).  A router score that is a close call
    in float64 may pick another expert once the normed row is rounded: one row in fifty may leave the tail's bound."""
    rows = sorted(_rel(got[t:t + 1], ref[t:t + 1]) for t in range(len(ref)))
    return rows[len(rows) // 2] < 3e-2 and rows[int(0.95 * len(rows))] < 0.1 and rows[-1 - len(rows) // 50] < 0.3


def _whole(eng, toks, rid="w"):
    return eng.trace_step([(rid, toks, list(range(len(toks))))], [rid])


def _in_parts(eng, toks, sizes, rid="p"):
    return np.concatenate([eng.trace_step([(rid, toks[a:a + n], list(range(n)))], [rid] if a + n == len(toks) else [])
                           for a, n in _portions(len(toks), sizes)])


TOL = 3e-5


def test_whole_prompt_matches_oracle_fp32_and_bf16():
    from oracle import revepel_oracle as O
    from vllm_tgis_adapter_b200.engine.revepel import synthetic_weights

    cfg = _cfg()
    toks = _tokens(150, 97, 1)
    for dtype in ("float32", "bfloat16"):
        mc = _model(cfg, dtype)
        weights = synthetic_weights(mc, 11)
        ref = O.forward(cfg, weights, toks)
        eng = _engine(mc, weights)
        got = _whole(eng, toks)
        if dtype == "float32":
            for n in (1, 2):    # the first tokens of a sequence on their own
                assert _rel(_whole(eng, toks[:n]), O.forward(cfg, weights, toks[:n])) < TOL
        eng.close()
        assert _rel(got, ref) < TOL if dtype == "float32" else _bf16_close(got, ref), dtype


def _alone():
    return {
        "attention": {"type": "attention", "mixer": _att(4, 2, 6, 10, 9, 4), "mlp": None},
        "attention_whole_head_rotates_no_scaling": {"type": "attention", "mixer": _att(3, 3, 8, 5, 40, 8, scaling=False), "mlp": None},
        "mamba2": {"type": "mamba2", "mixer": {"heads": 6, "vdim": 4, "state": 5, "groups": 2, "norm_groups": 3, "conv": 3}, "mlp": None},
        "mamba2_one_wide_norm_group": {"type": "mamba2", "mixer": {"heads": 16, "vdim": 66, "state": 8, "groups": 4, "norm_groups": 1, "conv": 2},
                                       "mlp": None},
        "channel_delta": {"type": "channel_delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "conv": 3}, "mlp": None},
        "channel_delta_keys_of_33": {"type": "channel_delta", "mixer": {"heads": 2, "kv_heads": 1, "dim": 33, "vdim": 35, "conv": 2}, "mlp": None},
        "experts": {"type": "attention", "mixer": _att(1, 1, 2, 2, 1, 0), "mlp": _moe(6, 2, 10, 14)},
    }


@pytest.mark.parametrize("name", list(_alone()))
def test_each_mechanism_alone_whole_and_in_portions(name):
    from oracle import revepel_oracle as O
    from vllm_tgis_adapter_b200.engine.revepel import synthetic_weights

    cfg = _cfg([_alone()[name]], width=24, vocab=61)
    toks = _tokens(90, 61, 4)
    mc = _model(cfg)
    weights = synthetic_weights(mc, 17)
    layers = []
    ref = O.forward(cfg, weights, toks, layers)
    eng = _engine(mc, weights)
    whole = _whole(eng, toks)
    parts = _in_parts(eng, toks, [3, 1, 40, 2])
    single = _in_parts(eng, toks[:45], [1])
    eng.close()
    assert _rel(whole, ref) < TOL and _rel(parts, ref) < TOL and _rel(single, ref[:45]) < TOL, name


def _variants():
    lay = lambda kind, mixer, mlp=None: {"type": kind, "mixer": mixer, "mlp": mlp}  # noqa: E731
    return {
        "ones": _cfg([lay("attention", _att(1, 1, 2, 1, 1, 2, scaling=False), _moe(1, 1, 1, 1)),
                      lay("mamba2", {"heads": 1, "vdim": 1, "state": 1, "groups": 1, "norm_groups": 1, "conv": 1}),
                      lay("channel_delta", {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1, "conv": 1})], width=6, vocab=11,
                     logit_scale=1.0, embed_scale=1.0),
        "only_recurrent_no_ff": _cfg([lay("channel_delta", {"heads": 3, "kv_heads": 3, "dim": 5, "vdim": 7, "conv": 5}),
                                      lay("mamba2", {"heads": 5, "vdim": 10, "state": 9, "groups": 5, "norm_groups": 1, "conv": 2}),
                                      lay("channel_delta", {"heads": 2, "kv_heads": 1, "dim": 70, "vdim": 3, "conv": 4})], width=30),
        "attention_first_window_longer_than_the_prompt": _cfg(
            [lay("attention", _att(2, 2, 32, 32, 1000, 32), _moe(4, 4, 16)),
             lay("attention", _att(2, 2, 32, 32, 3, 32, kv_from=0), _moe(9, 2, 8, 64)),
             lay("mamba2", {"heads": 2, "vdim": 32, "state": 16, "groups": 1, "norm_groups": 4, "conv": 4}, _moe(2, 1, 64)),
             lay("attention", _att(4, 1, 16, 24, 50, 8, base=20000.0), None),
             lay("attention", _att(4, 1, 16, 24, 20, 8, base=20000.0, kv_from=3), None)], width=64, vocab=130),
        "wide_states": _cfg([lay("mamba2", {"heads": 2, "vdim": 40, "state": 200, "groups": 1, "norm_groups": 1, "conv": 3}, _moe(3, 2, 24, 8)),
                             lay("channel_delta", {"heads": 2, "kv_heads": 2, "dim": 136, "vdim": 40, "conv": 3})], width=48),
        "tensor_core_sizes": _cfg([lay("channel_delta", {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "conv": 4}, _moe(8, 2, 128, 256)),
                                   lay("attention", _att(4, 2, 64, 96, 64, 32, scale=0.125), _moe(8, 2, 128, 256)),
                                   lay("mamba2", {"heads": 8, "vdim": 64, "state": 64, "groups": 2, "norm_groups": 2, "conv": 4}),
                                   lay("attention", _att(4, 2, 64, 96, 100, 32, scale=0.125, kv_from=1), _moe(4, 1, 256))],
                                  width=320, vocab=300),
    }


@pytest.mark.parametrize("name", list(_variants()))
def test_other_sizes_orders_and_absent_parts(name):
    from oracle import revepel_oracle as O
    from vllm_tgis_adapter_b200.engine.revepel import synthetic_weights

    cfg = _variants()[name]
    toks = _tokens(70, cfg["vocab"], 7)
    for dtype in ("float32", "bfloat16"):
        mc = _model(cfg, dtype, ranks=(1, 1) if name == "ones" else (5, 2))
        weights = synthetic_weights(mc, 23)
        ref = O.forward(cfg, weights, toks)
        eng = _engine(mc, weights)
        whole = _whole(eng, toks)
        parts = _in_parts(eng, toks, [3, 1, 40, 2])
        eng.close()
        if dtype == "float32":
            assert _rel(whole, ref) < TOL and _rel(parts, ref) < TOL, (name, dtype)
        elif name != "ones":    # (single-entry heads in bf16: a norm of one rounded number is a sign, nothing to bound)
            assert _bf16_close(whole, ref) and _bf16_close(parts, ref), (name, dtype)


def test_prefill_portions_and_token_by_token_agree_with_whole_prompt():
    from oracle import revepel_oracle as O
    from vllm_tgis_adapter_b200.engine.revepel import synthetic_weights

    cfg = _cfg()
    mc = _model(cfg)
    weights = synthetic_weights(mc, 31)
    toks = _tokens(131, 97, 3)
    ref = O.forward(cfg, weights, toks)
    eng = _engine(mc, weights)
    for sizes in ([2], [1], [31, 33, 2, 64, 1], [64, 1, 1, 1, 1, 1, 1], [9, 37, 8]):
        assert _rel(_in_parts(eng, toks, sizes, "s"), ref) < TOL, sizes
    eng.close()


def test_long_decoding_crosses_window_and_block_borders_bf16_stays_close():
    from oracle import revepel_oracle as O
    from vllm_tgis_adapter_b200.engine.revepel import synthetic_weights

    cfg = _cfg()
    toks = _tokens(300, 97, 9)
    for dtype in ("float32", "bfloat16"):
        mc = _model(cfg, dtype)
        weights = synthetic_weights(mc, 37)
        ref = O.forward(cfg, weights, toks)
        eng = _engine(mc, weights)
        got = [eng.trace_step([("d", toks[:30], list(range(30)))], [])]
        for t in range(30, 300):
            got.append(eng.trace_step([("d", [toks[t]], [0])], ["d"] if t == 299 else []))
        eng.close()
        got = np.concatenate(got)
        assert _rel(got, ref) < TOL if dtype == "float32" else _bf16_close(got, ref), dtype


def test_mixed_batches_of_unequal_requests_match_each_alone_and_reuse_blocks_and_slots():
    from oracle import revepel_oracle as O
    from vllm_tgis_adapter_b200.engine.revepel import synthetic_weights

    cfg = _cfg()
    mc = _model(cfg)
    weights = synthetic_weights(mc, 41)
    reqs = {f"q{i}": _tokens(n, 97, 50 + i) for i, n in enumerate([97, 40, 3, 130, 64, 33, 71, 1, 90])}
    ref = {k: O.forward(cfg, weights, v) for k, v in reqs.items()}
    # 3 slots and a pool of 10 blocks: the requests only fit because finished ones give their state slot and blocks back
    eng = _engine(mc, weights, blocks=10, seqs=3)
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    nb = lambda k: (len(reqs[k]) + KV_BLOCK - 1) // KV_BLOCK  # noqa: E731
    waiting, live, step = list(reqs), [], 0
    while waiting or live:
        while waiting and len(live) < 3 and sum(nb(k) for k in live) + nb(waiting[0]) <= 10:
            live.append(waiting.pop(0))
        entries, ends = [], []
        for j, k in enumerate(live):
            if (step + j) % 5 == 4:
                continue                                        # a request may sit a step out
            n = min(len(reqs[k]) - at[k], [1, 7, 2, 29, 1, 33][(step + 2 * j) % 6])   # single tokens beside portions
            entries.append((k, reqs[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
            if at[k] == len(reqs[k]):
                ends.append(k)
        if entries:
            out = eng.trace_step(entries, ends)
            o = 0
            for k, t, _ in entries:
                got[k].append(out[o:o + len(t)])
                o += len(t)
        live = [k for k in live if k not in ends]
        step += 1
    st = eng.status()
    eng.close()
    assert st.free_blocks == st.total_blocks == 10
    for k in reqs:
        assert _rel(np.concatenate(got[k]), ref[k]) < TOL, k


def test_greedy_generation_through_the_scheduler_matches_oracle():
    from oracle import revepel_oracle as O
    from vllm_tgis_adapter_b200.engine.core import make_sampling_params
    from vllm_tgis_adapter_b200.engine.revepel import synthetic_weights

    cfg = _cfg()
    mc = _model(cfg)
    weights = synthetic_weights(mc, 61)
    prompts = [_tokens(45, 97, 70), _tokens(3, 97, 71), _tokens(80, 97, 72)]
    n_new = 40
    for graphs in (False, True):
        eng = _engine(mc, weights, graphs=graphs, tokens=64)     # 64-token steps: the prompts are prefilled in portions
        sp = make_sampling_params(greedy=True, max_tokens=n_new, min_tokens=n_new, eos_token_id=-1, num_logprobs=1)
        outs = eng.generate_sync(prompts, sp)
        st = eng.status()
        eng.close()
        assert st.errored == 0 and (st.graph_launches > 0) == graphs
        for p, recs in zip(prompts, outs):
            toks = [r.new_token for r in recs if r.new_token is not None]
            assert toks == O.greedy(cfg, weights, p, n_new), graphs
            lp = torch.log_softmax(O.forward(cfg, weights, p + toks[:-1])[len(p) - 1:], -1)
            for i, r in enumerate([r for r in recs if r.new_token is not None]):
                assert abs(r.logprob - float(lp[i, r.new_token])) < 1e-3


def test_generate_over_grpc_matches_oracle():
    """grpc client -> TextGenerationService -> AsyncTGISEngine -> the engine's step loop on a Revepel preset (float32): greedy
    tokens and their logprobs of a batched Generate call against the oracle."""
    from test_server_gpu import LiveServer

    from oracle import revepel_oracle as O
    from vllm_tgis_adapter_b200.engine.revepel import config_json
    from vllm_tgis_adapter_b200.engine.tokenizer import synthetic_prompt
    from vllm_tgis_adapter_b200.grpc.pb import generation_pb2 as pb

    srv = LiveServer("revepel-tiny", seed=29)
    try:
        cfg = config_json(srv.cfg.model_config)
        rs = np.random.RandomState(5)
        prompts = [rs.randint(3, srv.cfg.vocab, size=n).tolist() for n in (12, 70, 7)]     # 70: prefilled in two portions
        params = pb.Parameters()
        params.stopping.max_new_tokens = 10
        params.stopping.min_new_tokens = 10
        params.response.generated_tokens = True
        params.response.token_logprobs = True
        call = srv.channel.unary_unary("/fmaas.GenerationService/Generate",
                                       request_serializer=pb.BatchedGenerationRequest.SerializeToString,
                                       response_deserializer=pb.BatchedGenerationResponse.FromString)
        resp = call(pb.BatchedGenerationRequest(model_id="m", requests=[pb.GenerationRequest(text=synthetic_prompt(p)) for p in prompts],
                                                params=params), timeout=120)
    finally:
        srv.close()
    assert len(resp.responses) == 3
    for p, r in zip(prompts, resp.responses):
        assert r.input_token_count == len(p) and r.generated_token_count == 10
        got = [int(t.text[1:]) for t in r.tokens]
        assert got == O.greedy(cfg, srv.weights, p, 10)
        lp = torch.log_softmax(O.forward(cfg, srv.weights, p + got[:-1])[len(p) - 1:], -1)
        for i, t in enumerate(r.tokens):
            assert abs(t.logprob - float(lp[i, got[i]])) < 1e-3


def test_trace_runner_command_line_on_a_model_directory(tmp_path):
    """bin/trace_run on a directory with config.json + model.safetensors: the family and the ranks of the low-rank maps come
    from the files, a mixed schedule with a reused slot goes through standard input, the logits land in the output folder."""
    import subprocess
    import sys
    from pathlib import Path

    from safetensors.torch import save_file

    from oracle import revepel_oracle as O
    from vllm_tgis_adapter_b200.engine.revepel import synthetic_weights

    cfg = _cfg()
    weights = synthetic_weights(_model(cfg, ranks=(2, 6)), 71)
    model = tmp_path / "model"
    model.mkdir()
    (model / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(model / "model.safetensors"))
    a, b, c = _tokens(70, 97, 1), _tokens(9, 97, 2), _tokens(40, 97, 3)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:33], "want": [0, 32]}, {"id": "b", "tokens": b[:2], "want": [1]}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[2:], "want": [6]}, {"id": "a", "tokens": a[33:69], "want": []}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": a[69:], "want": [0]}, {"id": "c", "tokens": c, "want": [39]}], "end": ["a", "c"]},
    ]
    want = {0: [("a", 0), ("a", 32), ("b", 1)], 1: [("b", 8)], 2: [("a", 69), ("c", 39)]}
    ref = {"a": O.forward(cfg, weights, a), "b": O.forward(cfg, weights, b), "c": O.forward(cfg, weights, c)}
    root = Path(__file__).resolve().parent.parent
    for dtype, tol in (("float32", TOL), ("bfloat16", 0.1)):
        out = tmp_path / f"out_{dtype}"
        p = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(model), "--dtype", dtype, "--out", str(out),
                            "--max-tokens", "192"], input="".join(json.dumps(s) + "\n" for s in steps), text=True, capture_output=True)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        for n, rows in want.items():
            got = np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(len(rows), -1)
            for g, (rid, pos) in zip(got, rows):
                assert _rel(g[None], ref[rid][pos:pos + 1]) < tol, (dtype, n, rid, pos)
