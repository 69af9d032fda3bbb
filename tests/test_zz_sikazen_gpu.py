"""-m gpu parity of the Sikazen architecture against oracle/sikazen_oracle.py.

Kernel level (include/tgis_kernels.h hooks): pooled-window attention over a paged cache in portions, on random inputs and on
inputs built so that ONE key decides a query's output -- just inside and just outside the window, in a pooled block that is
just complete or one token short, on both sides of a cache page's border, the first token, far away --, in fp32 and in bf16;
the HGRN2 scan in portions through two state slots.
Engine level (trace replay = the engine's own step function, sequence slots and block manager): every mechanism alone, whole
prompts in fp32 and bf16, portions down to two tokens, token-by-token decoding, mixed batches against each request alone
with pages and state slots that are used again, long decoding across window, pool and page borders, other sizes, loops and
layer orders (values equal to 1, parts absent), and greedy generation through add_request + the step loop with and without
CUDA-graph replay, over gRPC, and through the trace runner's command line."""
import ctypes as C
import json

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

F32, BF16 = 0, 1
KV_BLOCK = 32
F64 = torch.float64
EPS = 1e-5


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
def _run_poolattn(h, bias, m, dt, sizes, pool_pages=40, seed=0):
    """h [T, width] whose columns are [q | k | v]: the sequence goes through the kernels in portions of the given sizes over a
    paged cache whose pages are scattered through the pool.  Returns the heads' outputs [T, heads * vdim]."""
    from oracle import sikazen_oracle as O
    from vllm_tgis_adapter_b200.engine._lib import TgisKPoolAttnGeom

    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rd, W, P = int(m["rot"]["dims"]), int(m["mask"]["size"]), int(m["mask"]["pool"])
    tdt = torch.bfloat16 if dt == BF16 else torch.float32
    geom = TgisKPoolAttnGeom(H, G, d, dv, W, P, rd, float(m["scale"]), 1)
    ang = torch.arange(T, dtype=F64)[:, None] * O.frequencies(m["rot"])[None, :]
    table = _dev(torch.cat([torch.cos(ang), torch.sin(ang)], -1)) if rd > 0 else None
    n_pages = (T + KV_BLOCK - 1) // KV_BLOCK
    pages = torch.randperm(pool_pages, generator=torch.Generator().manual_seed(seed))[:n_pages].tolist()
    rpp = (KV_BLOCK + P - 1) // P
    kc = torch.randn(pool_pages * KV_BLOCK, G * d, device="cuda").to(tdt)     # stale rows of earlier owners: finite, never visible
    vc = torch.randn(pool_pages * KV_BLOCK, G * dv, device="cuda").to(tdt)
    pk = torch.randn(pool_pages * rpp, G * d, device="cuda").to(tdt)
    pv = torch.randn(pool_pages * rpp, G * dv, device="cuda").to(tdt)
    y = _dev(h)
    b = _dev(bias) if bias is not None else None
    out = torch.full((T, H * dv), float("nan"), dtype=tdt, device="cuda")
    for at, n in _portions(T, sizes):
        pos = list(range(at, at + n))
        slots = [pages[p // KV_BLOCK] * KV_BLOCK + p % KV_BLOCK for p in pos]
        q = torch.zeros(n, H * d, dtype=tdt, device="cuda")
        yp = y[at:at + n].contiguous()
        _ok(_lib().tgis_k_poolattn_prep(_p(yp), y.shape[1], 0, H * d, H * d + G * d, _p(b), C.byref(geom), _p(table), EPS,
                                        _p(_i32(pos)), _p(_i32(slots)), _p(q), _p(kc), _p(vc), dt, n))
        o = torch.full((n, H * dv), float("nan"), dtype=tdt, device="cuda")
        _ok(_lib().tgis_k_poolattn(_p(q), _p(kc), _p(vc), _p(pk), _p(pv), dt, _ints([0, n, at + n, 0]), 1, _ints(pages), 1, len(pages),
                                   _p(o), C.byref(geom)))
        out[at:at + n] = o
    return out


def _pool_weights(m, bias):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    width = H * d + G * d + G * dv
    z = torch.zeros(width, dtype=F64) if bias is None else bias.double()
    return width, {"q": _eye_rows(width, 0, H * d), "k": _eye_rows(width, H * d, G * d), "v": _eye_rows(width, H * d + G * d, G * dv),
                   "q.b": z[:H * d], "k.b": z[H * d:H * d + G * d], "v.b": z[H * d + G * d:], "o": torch.eye(H * dv, dtype=F64)}


def _pa(heads, kv_heads, dim, vdim, size, pool, rot_dims, base=300.0, factor=None, scale=0.3):
    rot = {"base": base, "dims": rot_dims}
    if factor:
        rot["scaling"] = {"factor": factor}
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, mask=dict(size=size, pool=pool), rot=rot)


_ATTN = [
    _pa(4, 2, 6, 10, 9, 4, 4, base=50.0, factor=2.0),
    _pa(3, 1, 40, 33, 70, 7, 40, base=1000.0, factor=8.0, scale=0.2),
    _pa(2, 2, 5, 140, 1, 1, 0),                                   # a window of one token, blocks of one token
    _pa(1, 1, 64, 64, 33, 40, 32, base=10000.0, scale=0.125),     # blocks longer than a cache page
    _pa(2, 1, 8, 8, 32, 32, 8, factor=3.0),                       # window and blocks as long as a page
    # sizes the tensor-core kernel takes in bf16
    _pa(2, 2, 96, 200, 100, 12, 96, base=500.0, scale=0.1),
    _pa(4, 2, 32, 48, 24, 5, 16, base=20000.0, factor=4.0, scale=0.2),
]


@pytest.mark.parametrize("m", _ATTN)
def test_pooled_window_attention_in_portions_matches_oracle(m):
    from oracle import sikazen_oracle as O

    g = torch.Generator().manual_seed(5)
    width, _ = _pool_weights(m, None)
    bias = torch.randn(width, generator=g) * 0.3
    _, w = _pool_weights(m, bias)
    T = 300
    h = torch.randn(T, width, generator=g)
    ref = O.pooled_window_attention(h.double(), w, m, EPS)
    for sizes in ([T], [3, 1, 40, 2, 64, 1, 1, 17], [1]):
        got = _run_poolattn(h, bias, m, F32, sizes).double().cpu()
        assert float((got - ref).abs().max()) < 2e-5 * max(1.0, float(ref.abs().max())), sizes
    if m["dim"] % 16 == 0:
        ref16 = O.pooled_window_attention(h.double(), w, m, EPS)
        got = _run_poolattn(h, bias, m, BF16, [3, 1, 40, 2, 64, 1, 1, 17]).double().cpu()
        assert float((got - ref16).abs().max()) < 0.06 * max(1.0, float(ref16.abs().max()))


@pytest.mark.parametrize("dt,m", [(F32, _ATTN[0]), (F32, _ATTN[3]), (F32, _ATTN[4]), (BF16, _ATTN[3]), (BF16, _ATTN[6])])
def test_one_key_decides_at_window_pool_and_page_edges(dt, m):
    """Every key but one points along one axis, the marked key along another, and so does the query under test (no rotation of
    those axes: the test model rotates nothing there); the marked value stands out.  The query either sees the marked key as a
    token, through its block's mean, or not at all: a window, a block or a page that is one token off changes the output by
    the marked value's size."""
    from oracle import sikazen_oracle as O

    m = dict(m, rot=dict(m["rot"], dims=0), scale=60.0 / m["dim"])     # a lone marked key outweighs the rest by e^60, its block's mean by e^(60 / pool)
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    W, P = m["mask"]["size"], m["mask"]["pool"]
    width, w = _pool_weights(m, None)
    T = 4 * KV_BLOCK + 3 * W + 2 * P + 5
    cases = set()
    for j in (0, 1, KV_BLOCK - 1, KV_BLOCK, P - 1, P, 2 * P - 1, 2 * KV_BLOCK + 1):
        for delta in (0, 1, W - 1, W, W + 1, W + P - 2, W + P - 1, W + P, W + 2 * P - 1, W + 2 * P, 3 * KV_BLOCK, T - 1 - j):
            if 0 <= delta and j + delta < T:
                cases.add((j, j + delta))
    worst = 0.0
    for j, i in sorted(cases):
        h = torch.zeros(T, width, dtype=F64)
        h[:, 1:H * d:d] = 1.0                       # every query along axis 1 ...
        h[:, H * d + 1:H * d + G * d:d] = 1.0       # ... and every key
        h[:, H * d + G * d:] = torch.linspace(-0.1, 0.1, G * dv, dtype=F64)
        h[j, H * d:H * d + G * d] = 0.0
        h[j, H * d:H * d + G * d:d] = 1.0           # the marked key along axis 0
        h[j, H * d + G * d:] = 7.0                  # its value
        h[i, :H * d] = 0.0
        h[i, 0:H * d:d] = 1.0                       # the query under test along axis 0
        ref = O.pooled_window_attention(h, w, m, EPS)[i]
        got = _run_poolattn(h.float(), None, m, dt, [j + 1, 2, 33, 1], seed=j)[i].double().cpu()
        err = float((got - ref).abs().max())
        worst = max(worst, err)
        assert err < (2e-4 if dt == F32 else 0.08), (j, i, float(ref[0]), float(got[0]))
    assert worst < 1.0


def test_hgrn_scan_in_portions_and_two_slots_matches_oracle():
    from oracle import sikazen_oracle as O

    g = torch.Generator().manual_seed(3)
    for H, d, dv in ((3, 6, 5), (2, 70, 40), (1, 1, 1), (2, 130, 33)):
        T = 150
        m = dict(heads=H, dim=d, vdim=dv)
        width = 2 * H * d + H * dv
        w = {"q": _eye_rows(width, 0, H * d), "f": _eye_rows(width, H * d, H * d), "v": _eye_rows(width, 2 * H * d, H * dv),
             "f.b": torch.randn(H * d, generator=g).double(), "lower": torch.rand(H * d, generator=g).double() * 0.95,
             "norm": torch.ones(dv, dtype=F64), "o": torch.eye(H * dv, dtype=F64)}
        seqs = [torch.randn(T, width, generator=g) * 2.0, torch.randn(T - 13, width, generator=g) * 2.0]
        refs = []
        for h in seqs:   # the scan's raw output: the oracle's head norm taken back out
            hd = h.double()
            q = O.silu(hd[:, :H * d]).view(-1, H, d)
            v = hd[:, 2 * H * d:].view(-1, H, dv)
            lower = w["lower"].view(H, d)
            f = lower + (1 - lower) * torch.sigmoid(hd[:, H * d:2 * H * d] + w["f.b"]).view(-1, H, d)
            S = torch.zeros(H, d, dv, dtype=F64)
            o = []
            for t in range(h.shape[0]):
                S = f[t][:, :, None] * S + (1 - f[t])[:, :, None] * v[t][:, None, :]
                o.append(torch.einsum("hdv,hd->hv", S, q[t]).reshape(-1))
            refs.append(torch.stack(o))
        S_dev = torch.randn(4, H, d, dv, device="cuda")       # slots 1 and 3 are used; what an earlier owner left is never read
        outs = [torch.zeros(s.shape[0], H * dv, device="cuda") for s in seqs]
        ys = [_dev(s) for s in seqs]
        at = [0, 0]
        sizes = [[5, 1, 40, 2, 17], [33, 1, 1, 64]]
        step = 0
        while at[0] < seqs[0].shape[0] or at[1] < seqs[1].shape[0]:
            rows, meta, tok_slot, dst = [], [], [], []
            for s in (0, 1):
                n = min(sizes[s][step % len(sizes[s])], seqs[s].shape[0] - at[s])
                if n <= 0:
                    continue
                meta += [sum(r.shape[0] for r in rows), n, at[s] + n, 0]
                rows.append(ys[s][at[s]:at[s] + n])
                tok_slot += [1 + 2 * s] * n
                dst.append((s, at[s], n))
                at[s] += n
            y = torch.cat(rows).contiguous()
            _KEEP.append(y)
            out = torch.zeros(y.shape[0], H * dv, device="cuda")
            _ok(_lib().tgis_k_outer_scan(3, _p(y), None, _p(y[:, 2 * H * d:]), width, width, width, 1.0, _p(y[:, H * d:]), width,
                                         _p(_dev(w["f.b"])), _p(_dev(w["lower"])), None, None, 0, None, None, 0.0, _p(S_dev), None, None,
                                         _p(out), H * dv, H, d, dv, None, None, 0, _ints(meta), len(meta) // 4, _p(_i32(tok_slot))))
            o = 0
            for s, a, n in dst:
                outs[s][a:a + n] = out[o:o + n]
                o += n
            step += 1
        for s in (0, 1):
            assert float((outs[s].double().cpu() - refs[s]).abs().max()) < 2e-5 * max(1.0, float(refs[s].abs().max())), (H, d, dv, s)


# ====================================================================================================== engine level
def _att(heads, kv_heads, dim, vdim, size, pool, rot_dims, **kw):
    return _pa(heads, kv_heads, dim, vdim, size, pool, rot_dims, **kw)


def _lat(heads, dim, rot_dim, vdim, kv_rank, q_rank, base=300.0, scale=0.25):
    return dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale,
                rot=dict(base=base, dims=rot_dim))


def _lay(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _cfg(layers=None, width=40, vocab=97, embed_scale=2.5, side=6, loop=(1, 3, 2)):
    if layers is None:
        layers = [_lay("hgrn2", dict(heads=3, dim=6, vdim=5), 30),
                  _lay("attention", _att(4, 2, 6, 10, 9, 4, 4, base=50.0, factor=2.0), 24),
                  _lay("latent_attention", _lat(3, 6, 4, 5, 10, 12), 20),
                  _lay("attention", _att(3, 3, 8, 5, 40, 7, 8), None)]
    cfg = {"architecture": "Sikazen", "width": width, "vocab": vocab, "norm": {"eps": EPS}, "embedding": {"scale": embed_scale},
           "layers": layers}
    if side:
        cfg["token_side"] = {"dim": side}
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


def _model(cfg, dtype="float32", max_model_len=512):
    from vllm_tgis_adapter_b200.engine.sikazen import model_config_from_json

    return model_config_from_json(cfg, max_model_len, dtype)


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
    is on the typical row and on the tail (the sharp comparison is the float32 one)."""
    rows = sorted(_rel(got[t:t + 1], ref[t:t + 1]) for t in range(len(ref)))
    return rows[len(rows) // 2] < 3e-2 and rows[int(0.95 * len(rows))] < 0.1 and rows[-1] < 0.3


def _whole(eng, toks, rid="w"):
    return eng.trace_step([(rid, toks, list(range(len(toks))))], [rid])


def _in_parts(eng, toks, sizes, rid="p"):
    return np.concatenate([eng.trace_step([(rid, toks[a:a + n], list(range(n)))], [rid] if a + n == len(toks) else [])
                           for a, n in _portions(len(toks), sizes)])


TOL = 3e-5


def test_whole_prompt_matches_oracle_fp32_and_bf16():
    from oracle import sikazen_oracle as O
    from vllm_tgis_adapter_b200.engine.sikazen import synthetic_weights

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
        "attention": dict(layers=[_lay("attention", _att(4, 2, 6, 10, 9, 4, 4, base=50.0, factor=2.0))], side=0, loop=None),
        "attention_whole_head_rotates_no_scaling": dict(layers=[_lay("attention", _att(3, 3, 8, 5, 40, 3, 8))], side=0, loop=None),
        "attention_window_only": dict(layers=[_lay("attention", _att(2, 1, 8, 8, 11, 0, 4))], side=0, loop=None),
        "latent_attention": dict(layers=[_lay("latent_attention", _lat(3, 6, 4, 5, 10, 12))], side=0, loop=None),
        "latent_attention_17_heads": dict(layers=[_lay("latent_attention", _lat(17, 4, 2, 3, 9, 7))], side=0, loop=None),
        "hgrn2": dict(layers=[_lay("hgrn2", dict(heads=3, dim=6, vdim=5))], side=0, loop=None),
        "hgrn2_keys_of_70": dict(layers=[_lay("hgrn2", dict(heads=2, dim=70, vdim=35))], side=0, loop=None),
        "feed_forward": dict(layers=[_lay("hgrn2", dict(heads=1, dim=1, vdim=1), 50)], side=0, loop=None),
        "token_input": dict(layers=[_lay("hgrn2", dict(heads=1, dim=1, vdim=1))], side=5, loop=None),
        "loop_of_one_layer_three_passes": dict(layers=[_lay("attention", _att(2, 1, 8, 8, 11, 3, 4), 16)], side=0, loop=(0, 1, 3)),
    }


@pytest.mark.parametrize("name", list(_alone()))
def test_each_mechanism_alone_whole_and_in_portions(name):
    from oracle import sikazen_oracle as O
    from vllm_tgis_adapter_b200.engine.sikazen import synthetic_weights

    cfg = _cfg(width=24, vocab=61, **_alone()[name])
    toks = _tokens(90, 61, 4)
    mc = _model(cfg)
    weights = synthetic_weights(mc, 17)
    ref = O.forward(cfg, weights, toks)
    eng = _engine(mc, weights)
    whole = _whole(eng, toks)
    parts = _in_parts(eng, toks, [3, 1, 40, 2])
    single = _in_parts(eng, toks[:45], [1])
    eng.close()
    assert _rel(whole, ref) < TOL and _rel(parts, ref) < TOL and _rel(single, ref[:45]) < TOL, name


def _variants():
    return {
        "ones": _cfg([_lay("attention", _att(1, 1, 2, 1, 1, 1, 2), 1), _lay("hgrn2", dict(heads=1, dim=1, vdim=1), 1),
                      _lay("latent_attention", _lat(1, 1, 2, 1, 1, 1), None)], width=6, vocab=11, embed_scale=1.0, side=1, loop=(0, 3, 1)),
        "no_loop_no_token_input_no_ff": _cfg([_lay("latent_attention", _lat(2, 8, 4, 8, 16, 8)), _lay("hgrn2", dict(heads=5, dim=9, vdim=10)),
                                              _lay("attention", _att(4, 4, 10, 6, 16, 16, 6))], width=30, side=0, loop=None),
        "whole_stack_loops_four_times": _cfg([_lay("hgrn2", dict(heads=2, dim=12, vdim=12), 40),
                                              _lay("latent_attention", _lat(4, 8, 8, 8, 24, 20), 40)], width=32, side=4, loop=(0, 2, 4)),
        "loop_in_the_middle_window_longer_than_the_prompt": _cfg(
            [_lay("attention", _att(2, 2, 32, 32, 1000, 12, 32), 64), _lay("hgrn2", dict(heads=2, dim=16, vdim=24), 48),
             _lay("attention", _att(4, 1, 16, 24, 50, 50, 8, base=20000.0, factor=4.0), None),
             _lay("latent_attention", _lat(4, 16, 8, 24, 32, 40), 64), _lay("hgrn2", dict(heads=1, dim=64, vdim=64), 32)],
            width=64, vocab=130, side=16, loop=(1, 4, 2)),
        "tensor_core_sizes": _cfg([_lay("attention", _att(4, 2, 64, 64, 64, 16, 64, scale=0.125), 512),
                                   _lay("latent_attention", _lat(4, 64, 32, 64, 128, 192, scale=0.1), 512),
                                   _lay("hgrn2", dict(heads=4, dim=64, vdim=64), 512),
                                   _lay("attention", _att(4, 4, 32, 96, 100, 12, 16, scale=0.2, factor=2.0), 256)],
                                  width=256, vocab=300, side=64, loop=(0, 2, 2)),
    }


@pytest.mark.parametrize("name", list(_variants()))
def test_other_sizes_orders_loops_and_absent_parts(name):
    from oracle import sikazen_oracle as O
    from vllm_tgis_adapter_b200.engine.sikazen import synthetic_weights

    cfg = _variants()[name]
    V = cfg["vocab"]
    toks = _tokens(140, V, 6)
    for dtype in ("float32", "bfloat16") if name == "tensor_core_sizes" else ("float32",):
        mc = _model(cfg, dtype)
        weights = synthetic_weights(mc, 23)
        ref = O.forward(cfg, weights, toks)
        eng = _engine(mc, weights)
        whole = _whole(eng, toks)
        parts = _in_parts(eng, toks, [2, 45, 1, 1, 33])
        eng.close()
        if dtype == "float32":
            assert _rel(whole, ref) < TOL and _rel(parts, ref) < TOL, name
        else:
            assert _bf16_close(whole, ref) and _bf16_close(parts, ref), name


def test_prefill_portions_and_token_by_token_agree_with_whole_prompt():
    from oracle import sikazen_oracle as O
    from vllm_tgis_adapter_b200.engine.sikazen import synthetic_weights

    cfg = _cfg()
    mc = _model(cfg)
    weights = synthetic_weights(mc, 31)
    toks = _tokens(131, 97, 3)
    ref = O.forward(cfg, weights, toks)
    eng = _engine(mc, weights)
    for sizes in ([2], [1], [31, 33, 2, 64, 1], [64, 1, 1, 1, 1, 1, 1], [9, 37, 8]):
        assert _rel(_in_parts(eng, toks, sizes, "s"), ref) < TOL, sizes
    eng.close()


def test_long_decoding_crosses_window_pool_and_page_borders_bf16_stays_close():
    from oracle import sikazen_oracle as O
    from vllm_tgis_adapter_b200.engine.sikazen import synthetic_weights

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


def test_sink_takes_weight_in_prompts_decoding_and_split_decoding():
    """Sinks large enough to hold a good part of the softmax's weight even among hundreds of keys: leaving the sink out of a
    prompt's rows, of a decoded token's row, or of the merge of a long sequence's key splits (bf16, more than 256 keys) changes
    the output by tens of percent."""
    from oracle import sikazen_oracle as O
    from vllm_tgis_adapter_b200.engine.sikazen import synthetic_weights

    cfg = _cfg(width=64, vocab=61, layers=[_lay("latent_attention", _lat(4, 16, 8, 16, 32, 24))], side=0, loop=None)
    toks = _tokens(400, 61, 8)
    for dtype in ("float32", "bfloat16"):
        mc = _model(cfg, dtype)
        weights = synthetic_weights(mc, 19)
        weights["l0.mix.sink"] = torch.tensor([6.0, 4.0, -2.0, 7.5]).to(torch.bfloat16)
        ref = O.forward(cfg, weights, toks)
        no_sink = O.forward(cfg, {**weights, "l0.mix.sink": torch.full((4,), -1e4).to(torch.bfloat16)}, toks)
        assert _rel(no_sink.numpy(), ref) > 0.1        # the sinks matter at every length
        eng = _engine(mc, weights)
        got = [eng.trace_step([("d", toks[:330], list(range(330)))], [])]
        for t in range(330, 400):
            got.append(eng.trace_step([("d", [toks[t]], [0])], ["d"] if t == 399 else []))
        eng.close()
        got = np.concatenate(got)
        assert _rel(got, ref) < TOL if dtype == "float32" else _bf16_close(got, ref), dtype


def test_mixed_batches_of_unequal_requests_match_each_alone_and_reuse_pages_and_slots():
    from oracle import sikazen_oracle as O
    from vllm_tgis_adapter_b200.engine.sikazen import synthetic_weights

    cfg = _cfg()
    mc = _model(cfg)
    weights = synthetic_weights(mc, 41)
    reqs = {f"q{i}": _tokens(n, 97, 50 + i) for i, n in enumerate([97, 40, 3, 130, 64, 33, 71, 1, 90])}
    ref = {k: O.forward(cfg, weights, v) for k, v in reqs.items()}
    # 3 slots and a pool of 10 pages: the requests only fit because finished ones give their state slot and pages back
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
    from oracle import sikazen_oracle as O
    from vllm_tgis_adapter_b200.engine.core import make_sampling_params
    from vllm_tgis_adapter_b200.engine.sikazen import synthetic_weights

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
    """grpc client -> TextGenerationService -> AsyncTGISEngine -> the engine's step loop on a Sikazen preset (float32): greedy
    tokens and their logprobs of a batched Generate call against the oracle."""
    from test_server_gpu import LiveServer

    from oracle import sikazen_oracle as O
    from vllm_tgis_adapter_b200.engine.sikazen import config_json
    from vllm_tgis_adapter_b200.engine.tokenizer import synthetic_prompt
    from vllm_tgis_adapter_b200.grpc.pb import generation_pb2 as pb

    srv = LiveServer("sikazen-tiny", seed=29)
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
    """bin/trace_run on a directory with config.json + model.safetensors: the family, the loop and every size come from the
    files, a mixed schedule with a reused slot goes through standard input, the logits land in the output folder."""
    import subprocess
    import sys
    from pathlib import Path

    from safetensors.torch import save_file

    from oracle import sikazen_oracle as O
    from vllm_tgis_adapter_b200.engine.sikazen import synthetic_weights

    cfg = _cfg()
    weights = synthetic_weights(_model(cfg), 71)
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
