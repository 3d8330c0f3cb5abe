"""Gekupel on the GPU against the plain implementation in plain_gekupel.py: each kernel and each mechanism alone, then
whole models through the step engine under different cuts of the same requests (whole prompts, token-by-token
decoding, portions down to two tokens, mixed batches on reused pages), edges of windows and blocks made visible by
construction, and greedy generation through the engine's own entry point and scheduler."""
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import gekupel_configs as gc
import plain_gekupel as pg
import tiny_configs as tc
import trace_tools as tt
from test_gpu_nipadra import MiniCtx, _run_mixer

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]
F = torch.float64


def _build(dtype, max_position=4096):
    from geneinfer_b200.parts import BuildContext
    return BuildContext(DEV, dtype, max_position)


def _bf(t):
    return t.to(torch.bfloat16).float()


def _close(got, want, dtype, what, f32=2e-5, b16=2e-2):
    err = float((got.double() - want.double()).abs().max() / max(1.0, float(want.abs().max())))
    assert err < (f32 if dtype is torch.float32 else b16), f"{what}: {err}"


class PagesCtx(MiniCtx):
    """MiniCtx whose layer keeps keys of ``hd`` and values of ``vd`` values (vd 0: no value pages)."""

    def __init__(self, dtype, n_requests, Hkv, hd, vd, page_size=8, max_len=256):
        super().__init__(dtype, n_requests, Hkv=Hkv, hd=hd, page_size=page_size, max_len=max_len)
        n = self._pages[0].shape[0]
        v = None if vd == 0 else torch.full((n, Hkv, page_size, vd), float("nan"), dtype=dtype, device=DEV)
        self._pages = (self._pages[0], v)
        self.max_step_tokens = 512

    def scratch(self, name, shape, dtype, capacity=None):
        if dtype in (torch.int32, torch.int64):
            return torch.full(shape, -7, dtype=dtype, device=DEV)
        return super().scratch(name, shape, dtype, capacity)


# ------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_add_normed(dtype):
    from geneinfer_b200.ops import kernels
    g = torch.Generator().manual_seed(1)
    for D in (200, 7, 1024):
        x, y, w = torch.randn(9, D, generator=g) * 3, torch.randn(9, D, generator=g), 1 + 0.1 * torch.randn(D, generator=g)
        xd, yd = x.to(DEV), y.to(DEV)
        xn = torch.empty(9, D, dtype=dtype, device=DEV)
        kernels.add_normed(yd, w.to(DEV), xd, 1e-3, xn_out=xn, clear_y=True)
        want = x.double() + pg.rms_norm(y.double(), w.double(), 1e-3)
        assert float((xd.cpu() - want).abs().max()) < 2e-6 * float(want.abs().max())
        assert torch.equal(xn.cpu().float(), xd.cpu().to(dtype).float()) and not yd.any()
        kernels.add_normed(y.to(DEV), w.to(DEV), xd, 1e-3)            # neither cast nor cleared


def _paged(rows, dtype, page_size, seed):
    """Lays rows [n, Hkv, d] of one request into scattered pages; returns (pages [P, Hkv, page, d], table [1, stride])."""
    n, Hkv, d = rows.shape
    per = (n + page_size - 1) // page_size
    order = torch.randperm(per + 3, generator=torch.Generator().manual_seed(seed))[:per]
    pages = torch.full((per + 3, Hkv, page_size, d), float("nan"), dtype=dtype)
    for p in range(n):
        pages[order[p // page_size], :, p % page_size] = rows[p].to(dtype)
    return pages.to(DEV), order.int().view(1, per).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, Hkv, hd, vd, window, chunk, biased, sunk, alias", [
    (4, 2, 16, 24, None, 13, True, True, False),        # blocks, bias, sink, values wider than keys
    (6, 6, 10, 8, 9, None, False, False, False),        # a warp per head, window only
    (8, 1, 40, 12, 50, 33, True, False, False),         # four heads to a warp; window and blocks together
    (9, 1, 36, 28, 21, None, False, True, True),        # values inside the key rows, heads beyond a full group of four
    (20, 1, 136, 136, None, None, False, True, True),   # two blocks of heads, no mask but causality
    (3, 3, 300, 260, 7, None, False, False, False),     # long heads
    (16, 1, 80, 64, 29, None, False, True, True),       # bfloat16: the tensor-core form (a latent of 64 + 16)
    (24, 1, 144, 128, None, 40, True, True, True),      # two blocks of heads, the second half full
    (16, 2, 32, 64, 50, None, True, False, False),      # eight heads to a key/value head, values in pages of their own
    (16, 1, 528, 512, 64, None, False, False, True),    # the widest value
])
def test_attention_rows(dtype, H, Hkv, hd, vd, window, chunk, biased, sunk, alias):
    from geneinfer_b200.ops import kernels
    g = torch.Generator().manual_seed(3)
    n, page = 77, 8
    q = torch.randn(n, H, hd, generator=g)
    k = _bf(torch.randn(n, Hkv, hd, generator=g))
    v = k[..., :vd] if alias else _bf(torch.randn(n, Hkv, vd, generator=g))
    slopes = torch.rand(H, generator=g) * 0.3 if biased else None
    sinks = torch.randn(H, generator=g) * 2 if sunk else None
    k_pages, table = _paged(k, dtype, page, 1)
    v_pages = None if alias else _paged(v, dtype, page, 1)[0]
    pos = torch.arange(n)
    mask = torch.ones(n, n, dtype=torch.bool).tril()
    if window:
        mask &= pg.window_mask(pos, window)
    if chunk:
        mask &= pg.chunk_mask(pos, chunk)
    per = H // Hkv
    scores = torch.einsum("ihd,jhd->hij", q.double(), k.double().repeat_interleave(per, 1)) * 0.21
    if biased:
        scores = scores - slopes.double().view(H, 1, 1) * (pos[:, None] - pos[None, :]).double()[None]
    p = pg.softmax_rows(scores, mask, None if sinks is None else sinks.double())
    want = torch.einsum("hij,jhd->ihd", p, v.double().repeat_interleave(per, 1)).reshape(n, H * vd)
    rows = torch.tensor([76, 5, 0, 40, 41, 13, 26, 39, 12, 63, 64], dtype=torch.int32)       # any rows, in any order
    for q_dtype, out_dtype in ((torch.float32, torch.float32), (dtype, dtype)):
        out = torch.full((len(rows), H * vd), float("nan"), dtype=out_dtype, device=DEV)
        kernels.attention_rows(q[rows.long()].reshape(len(rows), H * hd).to(DEV).to(q_dtype), k_pages, v_pages, out,
                               torch.zeros(len(rows), dtype=torch.int32, device=DEV), rows.to(DEV), table, H, Hkv, hd, vd, page,
                               0.21, window=window, chunk=chunk, slopes=None if slopes is None else slopes.to(DEV),
                               sinks=None if sinks is None else sinks.to(DEV))
        on_tensor_cores = dtype is torch.bfloat16 and H // Hkv >= 8 and hd % 16 == 0 and vd % 64 == 0
        exact = q_dtype is torch.float32 and out_dtype is torch.float32 and not on_tensor_cores
        _close(out.cpu().float(), want[rows.long()], torch.float32 if exact else torch.bfloat16, "attention rows", f32=1e-5)
        if on_tensor_cores:          # and the CUDA-core form at the same sizes
            old = kernels.attention_rows_tensor_cores(False)
            other = torch.full_like(out, float("nan"))
            kernels.attention_rows(q[rows.long()].reshape(len(rows), H * hd).to(DEV).to(q_dtype), k_pages, v_pages, other,
                                   torch.zeros(len(rows), dtype=torch.int32, device=DEV), rows.to(DEV), table, H, Hkv, hd, vd, page,
                                   0.21, window=window, chunk=chunk, slopes=None if slopes is None else slopes.to(DEV),
                                   sinks=None if sinks is None else sinks.to(DEV))
            kernels.attention_rows_tensor_cores(old)
            _close(other.cpu().float(), want[rows.long()], torch.float32 if q_dtype is torch.float32 and out_dtype is torch.float32
                   else torch.bfloat16, "attention rows, CUDA cores", f32=1e-5)


@pytest.mark.parametrize("H, Hkv, hd, vd, window, chunk, biased, sunk, alias", [
    (4, 2, 16, 64, None, 13, True, True, False),        # a warp owns sixteen rows: 32 tokens of two heads to a tile; blocks, bias, sinks
    (16, 1, 80, 64, 29, None, False, True, True),       # four tokens of sixteen heads over a latent of 64 + 16
    (8, 8, 32, 64, 20, None, False, False, False),      # 64 tokens to a tile
    (6, 2, 48, 128, 17, 25, True, True, False),         # groups of three: 21 tokens to a tile and a row left over
    (40, 1, 144, 128, 64, None, False, True, True),     # two tokens of sixteen heads a block: three blocks of heads, the last one half full
    (16, 1, 544, 512, 100, None, False, True, True),    # the same with the widest value
    (16, 2, 160, 192, 33, None, True, True, False),     # shared rows, two tokens of eight heads to a tile
])
def test_attention_rows_in_tiles_and_ranges_of_keys(H, Hkv, hd, vd, window, chunk, biased, sunk, alias):
    """The tensor-core form over tiles of consecutive tokens (every row with its own first and last key), over listed
    rows, and with the keys cut into ranges that a second kernel merges: all agree with the plain softmax."""
    from geneinfer_b200.ops import kernels
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(5)
    n, page = 150, 16
    q = torch.randn(n, H, hd, generator=g)
    k = _bf(torch.randn(n, Hkv, hd, generator=g))
    v = k[..., :vd] if alias else _bf(torch.randn(n, Hkv, vd, generator=g))
    slopes = torch.rand(H, generator=g) * 0.3 if biased else None
    sinks = torch.randn(H, generator=g) * 2 if sunk else None
    k_pages, table = _paged(k, dtype, page, 2)
    v_pages = None if alias else _paged(v, dtype, page, 2)[0]
    pos = torch.arange(n)
    mask = torch.ones(n, n, dtype=torch.bool).tril()
    if window:
        mask &= pg.window_mask(pos, window)
    if chunk:
        mask &= pg.chunk_mask(pos, chunk)
    per = H // Hkv
    scores = torch.einsum("ihd,jhd->hij", q.double(), k.double().repeat_interleave(per, 1)) * 0.21
    if biased:
        scores = scores - slopes.double().view(H, 1, 1) * (pos[:, None] - pos[None, :]).double()[None]
    p = pg.softmax_rows(scores, mask, None if sinks is None else sinks.double())
    want = torch.einsum("hij,jhd->ihd", p, v.double().repeat_interleave(per, 1)).reshape(n, H * vd)
    per_tile = kernels.attention_rows_tile_tokens(H, Hkv, hd, vd, alias)
    assert per_tile == (64 // per if hd <= 128 and vd <= 128 and per <= 16 else 2 if per >= 16 else max(1, 16 // per))
    # the step: rows 0..n-1 of one request in order; tiles start at an odd row so that they straddle blocks and pages
    tiles = [(0, 3, 0)] + [(t, min(per_tile, n - t), 0) for t in range(3, n, per_tile)] if per_tile >= 3 else \
        [(t, min(per_tile, n - t), 0) for t in range(0, n, per_tile)]
    tiles_d = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    some = torch.tensor([149, 0, 77, 31, 32, 12, 13], dtype=torch.int32, device=DEV)
    args = (q.reshape(n, H * hd).to(DEV), k_pages, v_pages)
    rest = (torch.zeros(n, dtype=torch.int32, device=DEV), pos.int().to(DEV), table, H, Hkv, hd, vd, page, 0.21)
    kw = dict(window=window, chunk=chunk, slopes=None if slopes is None else slopes.to(DEV), sinks=None if sinks is None else sinks.to(DEV))
    for splits in (1, 3, 16):
        ws = None
        if splits > 1:
            ws = torch.full((kernels.attention_rows_workspace_rows(len(tiles), H, Hkv, splits), vd + 2), float("nan"), device=DEV)
        out = torch.full((n, H * vd), float("nan"), device=DEV)
        kernels.attention_rows(*args, out, *rest, tiles=tiles_d, splits=splits, workspace=ws, **kw)
        _close(out.cpu(), want, dtype, f"tiles of {per_tile} tokens, {splits} ranges")
        out2 = torch.full((n, H * vd), float("nan"), device=DEV)
        ws2 = None if splits == 1 else torch.full((kernels.attention_rows_workspace_rows(len(some), H, Hkv, splits), vd + 2), float("nan"), device=DEV)
        kernels.attention_rows(*args, out2, *rest, rows=some, splits=splits, workspace=ws2, **kw)
        _close(out2.cpu()[some.cpu().long()], want[some.cpu().long()], dtype, f"listed rows, {splits} ranges")
        untouched = torch.ones(n, dtype=torch.bool)
        untouched[some.cpu().long()] = False
        assert torch.isnan(out2.cpu()[untouched]).all()


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_product_with_a_rotated_tail(dtype):
    from geneinfer_b200.ops import kernels
    g = torch.Generator().manual_seed(4)
    for T, H, N, K, tail, off in ((37, 3, 70, 24, 8, 5), (1, 5, 8, 100, 0, 5), (16, 2, 64, 32, 2, 5), (3, 4, 40, 64, 0, 8), (20, 2, 33, 48, 0, 16),
                                  (200, 3, 70, 24, 8, 8), (129, 2, 64, 100, 0, 4), (300, 1, 130, 36, 4, 0)):
        a = torch.randn(T, off + H * (K + tail) + (4 if off % 4 == 0 else 3), generator=g)
        w = _bf(torch.randn(H, N, K, generator=g))
        freq = torch.rand(max(tail // 2, 1), generator=g)[:tail // 2]
        pos = torch.randint(0, 900, (T,), generator=g)
        out = torch.full((T, 2 + H * (N + tail)), float("nan"), dtype=torch.float32, device=DEV)
        kernels.head_product(a.to(DEV), off, K + tail, w.to(DEV).to(dtype), out, 2, N + tail, tail=tail,
                             freq=freq.to(DEV) if tail else None, amplitude=1.3, positions=pos.int().to(DEV) if tail else None)
        x = a[:, off:off + H * (K + tail)].view(T, H, K + tail).double()
        want = torch.einsum("thk,hnk->thn", x[..., :K], w.double())
        got = out.cpu()[:, 2:].view(T, H, N + tail)
        _close(got[..., :N], want, torch.float32, "head product")
        if tail:
            _close(got[..., N:], pg.rotate_pairs(x[..., K:], pos, freq.double(), 1.3), torch.float32, "rotated tail")
        assert torch.isnan(out.cpu()[:, :2]).all()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T, E, top, D, I", [(1, 4, 1, 64, 24), (5, 3, 3, 40, 72), (150, 9, 2, 96, 40), (64, 40, 6, 72, 16)])
def test_routing_and_expert_products(dtype, T, E, top, D, I):
    from geneinfer_b200.ops import kernels
    g = torch.Generator().manual_seed(6)
    x = _bf(torch.randn(T, D, generator=g))
    router, corr = torch.randn(E, D, generator=g) * 0.3, torch.randn(E, generator=g) * 0.5
    wgu, wd = _bf(torch.randn(E, 2 * I, D, generator=g) * 0.2), _bf(torch.randn(E, D, I, generator=g) * 0.2)
    tiles, tm = kernels.route_tiles(T, top, E), kernels.grouped_tile_rows()
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    srt = torch.empty(tiles * tm, dtype=torch.int32, device=DEV)
    grp = torch.empty(tiles, dtype=torch.int32, device=DEV)
    cnt = torch.empty(1, dtype=torch.int32, device=DEV)
    kernels.route(x.to(DEV).to(dtype), router.to(DEV), corr.to(DEV), top, ids, wts, srt, grp, cnt)
    chosen, weight = pg.route(x.double(), router.double(), corr.double(), top)
    assert torch.equal(ids.cpu().long(), chosen), "chosen experts (in the order of their choice scores)"
    assert float((wts.cpu() - weight).abs().max()) < 1e-6
    n = int(cnt.item())
    pairs = srt.cpu()[:n * tm]
    assert sorted(pairs[pairs >= 0].tolist()) == list(range(T * top))
    for i in range(n):                         # a tile's rows all chose the tile's expert
        mine = pairs[i * tm:(i + 1) * tm]
        assert all(int(ids.view(-1)[p]) == int(grp[i]) for p in mine[mine >= 0].tolist())
    hidden = torch.full((T * top, I), float("nan"), device=DEV)
    kernels.expert_product(x.to(DEV).to(dtype), top, wgu.to(DEV).to(dtype), hidden, srt, grp, cnt, gated="silu")
    part = torch.full((T * top, D), float("nan"), device=DEV)
    kernels.expert_product(hidden, 1, wd.to(DEV).to(dtype), part, srt, grp, cnt)
    y = torch.ones(T, D, device=DEV)
    kernels.route_combine(part, wts, y)
    w = {"router": router.double(), "correction": corr.double()}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = wgu[e, :I].double(), wgu[e, I:].double(), wd[e].double()
    want = 1.0 + pg.moe_ff(x.double(), {"router": {"top": top}}, w)
    _close(y.cpu(), want, torch.float32, "routed experts", f32=1e-5)


# ------------------------------------------------------------------------------------------ mixers alone
ATT = {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 24, "mask": {"size": 11}, "scale": 0.45}
LAT = {"heads": 3, "dim": 24, "rot_dim": 8, "vdim": 40, "q_rank": 32, "kv_rank": 48, "mask": {"size": 13}, "scale": 0.3,
       "rot": {"base": 300.0, "dims": 8, "scaling": {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}}}
CUTS = {"whole": [[40]], "decode": [[1]] * 40, "portions": [[2], [3], [11], [2], [1], [9], [2], [10]],
        "tail": [[23]] + [[1]] * 17}


def _att_weights(D, m, g, std=0.25):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    r = lambda *s: _bf(torch.randn(*s, generator=g) * std)      # noqa: E731
    return {"q": r(H * d, D), "k": r(G * d, D), "v": r(G * dv, D), "o": r(D, H * dv), "sink": torch.randn(H, generator=g)}


def _att_part(D, m, w, dtype):
    from geneinfer_b200.config import PartSpec
    from geneinfer_b200.config.gekupel import distance_slopes
    from geneinfer_b200.parts import MIXERS
    params = {"hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
              "scale": m["scale"], "window": None, "chunk": m["mask"]["size"], "position": PartSpec("none", {}), "qk_norm_eps": 1e-5,
              "qk_norm_weights": False, "distance_slopes": distance_slopes(m["heads"]), "sink": "learned"}
    return MIXERS["attention"](params, {"w_qkv": torch.cat([w["q"], w["k"], w["v"]]), "w_o": w["o"], "sink": w["sink"]}, _build(dtype))


def _lat_weights(D, m, g, second, std=0.25):
    H, d, r, dv, qr, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
    rn = lambda *s: _bf(torch.randn(*s, generator=g) * std)      # noqa: E731
    w = {"dq": rn(qr, D), "dq.norm": 1 + 0.2 * torch.randn(qr, generator=g), "uq": rn(H * (d + r), qr), "dkv": rn(kr + r, D),
         "dkv.norm": 1 + 0.2 * torch.randn(kr, generator=g), "uk": rn(H * d, kr), "uv": rn(H * dv, kr), "o": rn(D, H * dv)}
    if second:
        w["sink"] = torch.randn(H, generator=g)
    return w


def _lat_part(D, m, w, dtype, second):
    from geneinfer_b200.config import PartSpec
    from geneinfer_b200.parts import MIXERS
    rope = PartSpec("rope_on_device", {"head_dim": m["rot_dim"], "rotary_dim": m["rot_dim"], "theta": m["rot"]["base"],
                                       "pairing": "interleaved", "ramp_scaling": m["rot"]["scaling"] if second else None})
    params = {"hidden_size": D, "num_heads": m["heads"], "head_dim": m["dim"], "rotary_dim": m["rot_dim"], "value_dim": m["vdim"],
              "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": m["scale"], "window": m["mask"]["size"], "norm_eps": 1e-5,
              "position": rope, "sink": "learned" if second else None}
    weights = {"w_down": torch.cat([w["dq"], w["dkv"]]), "q_latent_norm": w["dq.norm"], "kv_latent_norm": w["dkv.norm"],
               "w_uq": w["uq"], "w_uk": w["uk"], "w_uv": w["uv"], "w_o": w["o"]}
    if second:
        weights["sink"] = w["sink"]
    return MIXERS["latent_attention"](params, weights, _build(dtype))


def _dbl(w):
    return {k: v.double() for k, v in w.items()}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cut", sorted(CUTS))
def test_attention_mixer_under_every_cut(dtype, cut):
    D = 48
    g = torch.Generator().manual_seed(7)
    w = _att_weights(D, ATT, g)
    part = _att_part(D, ATT, w, dtype)
    need = part.cache_need()
    assert (need.chunk, need.window, need.value_width, need.head_dim) == (11, None, 24, 16)
    x = _bf(torch.randn(40, D, generator=g))
    want = pg.attention_mixer(x.double(), ATT, _dbl(w), 1e-5, torch.arange(40), pg.ident if dtype is torch.float32 else pg.bf16)
    got = _run_mixer(part, PagesCtx(dtype, 1, 2, 16, 24), [x], CUTS[cut], dtype, D)[0]
    _close(got, want, dtype, f"attention mixer, {cut}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("second", [False, True])
@pytest.mark.parametrize("cut", sorted(CUTS))
def test_latent_mixer_under_every_cut(dtype, second, cut):
    D = 56
    g = torch.Generator().manual_seed(8)
    w = _lat_weights(D, LAT, g, second)
    part = _lat_part(D, LAT, w, dtype, second)
    need = part.cache_need()
    assert (need.num_kv_heads, need.head_dim, need.value_width, need.window) == (1, 56, 0, 13)
    x = _bf(torch.randn(40, D, generator=g))
    want = pg.latent_attention_mixer(x.double(), LAT, _dbl(w), 1e-5, torch.arange(40), second,
                                     pg.ident if dtype is torch.float32 else pg.bf16)
    got = _run_mixer(part, PagesCtx(dtype, 1, 1, 56, 0), [x], CUTS[cut], dtype, D)[0]
    _close(got, want, dtype, f"latent mixer {second}, {cut}", b16=3e-2)


def test_the_ramp_scaling_moves_the_slow_pairs_only():
    from geneinfer_b200.parts import POSITION_ENCODINGS
    for dims, base, sc in ((8, 300.0, LAT["rot"]["scaling"]), (32, 50000.0, {"factor": 3.0, "original": 40, "fast": 4.0, "slow": 0.5}),
                           (4, 10.0, {"factor": 2.0, "original": 8, "fast": 1.0, "slow": 1.0})):
        part = POSITION_ENCODINGS["rope_on_device"]({"head_dim": dims, "rotary_dim": dims, "theta": base, "pairing": "interleaved",
                                                     "ramp_scaling": sc}, {}, _build(torch.float32))
        freq, amp = pg.rotation_frequencies(dims, base, sc)
        assert torch.allclose(part.freq.cpu().double(), freq, rtol=1e-6, atol=0) and abs(part.amplitude - amp) < 1e-12
        plain = base ** (-2.0 * torch.arange(dims // 2, dtype=F) / dims)
        assert freq[0] == plain[0] and abs(float(freq[-1] / plain[-1]) - 1.0 / sc["factor"]) < 1e-12


@pytest.mark.parametrize("dtype", DTYPES)
def test_two_requests_in_one_batch_equal_each_alone(dtype):
    """Unequal requests side by side, one sitting steps out, on scattered pages: each equals its run alone."""
    D = 56
    g = torch.Generator().manual_seed(9)
    wl, wa = _lat_weights(D, LAT, g, True), _att_weights(D, ATT, g)
    xs = [_bf(torch.randn(n, D, generator=g)) for n in (37, 9, 22)]
    cuts = [[5, 0, 1], [1, 2, 1], [20, 0, 1], [1, 7, 0], [10, 0, 19]]
    for part, ctx_of, plain in (
            (_lat_part(D, LAT, wl, dtype, True), lambda n: PagesCtx(dtype, n, 1, 56, 0),
             lambda x: pg.latent_attention_mixer(x.double(), LAT, _dbl(wl), 1e-5, torch.arange(len(x)), True)),
            (_att_part(D, ATT, wa, dtype), lambda n: PagesCtx(dtype, n, 2, 16, 24),
             lambda x: pg.attention_mixer(x.double(), ATT, _dbl(wa), 1e-5, torch.arange(len(x))))):
        got = _run_mixer(part, ctx_of(3), xs, cuts, dtype, D)
        for r, x in enumerate(xs):
            alone = _run_mixer(part, ctx_of(1), [x], [[len(x)]], dtype, D)[0]
            _close(got[r], alone, dtype, f"request {r} in a batch", f32=2e-6, b16=1.5e-2)
            _close(got[r], plain(x), dtype, f"request {r} against the plain mixer", b16=4e-2)


# one score made to stand out: the query at ``qi`` asks for the key ``distance`` back
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("distance", [0, 1, 12, 13, 14, 30])
def test_latent_window_edge(distance, decoded):
    """Window 13: the key 12 back is the last one seen, the key 13 back the first one not seen."""
    D, T, qi, dtype = 56, 60, 45, torch.float32
    g = torch.Generator().manual_seed(10)
    w = _lat_weights(D, LAT, g, True, std=0.1)
    # input feature 0 makes a strong key, feature 1 a query that asks for it, through latents of their own
    for name in ("dq", "dkv"):
        w[name][:, :2] = 0
    w["dkv"][0, 0] = 3.0
    w["dq"][0, 1] = 3.0
    w["uq"][:] = 0
    w["uk"][:] = 0
    for h in range(LAT["heads"]):
        w["uq"][h * 32, 0] = 4.0          # the head's first unrotated query dimension reads the query latent's first value
        w["uk"][h * 24, 0] = 4.0
    part = _lat_part(D, LAT, w, dtype, True)
    x = 0.3 * torch.randn(T, D, generator=g)
    x[:, :2] = 0
    x[qi - distance, 0] = 6.0
    x[qi, 1] = 6.0
    x = _bf(x)
    cuts = [[T]] if not decoded else [[qi - 3]] + [[1]] * (T - qi + 3)
    got = _run_mixer(part, PagesCtx(dtype, 1, 1, 56, 0), [x], cuts, dtype, D)[0]
    want = pg.latent_attention_mixer(x.double(), LAT, _dbl(w), 1e-5, torch.arange(T), True)
    _close(got, want, dtype, f"key {distance} back")
    x2 = x.clone()
    x2[qi - distance, 0] = 0
    moved = float((pg.latent_attention_mixer(x2.double(), LAT, _dbl(w), 1e-5, torch.arange(T), True)[qi] - want[qi]).abs().max())
    assert (moved > 0.02) == (distance < 13), f"the key {distance} back moves the output by {moved}"


@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("qi, ki", [(43, 33), (43, 32), (44, 43), (44, 44), (54, 44), (55, 54), (10, 0), (11, 10)])
def test_attention_block_edge_and_sink(qi, ki, decoded):
    """Blocks of 11 positions: 33..43 see each other, 44 starts the next block. With the strong key out of sight the
    sink takes most of the weight."""
    D, T, dtype = 48, 60, torch.float32
    g = torch.Generator().manual_seed(11)
    w = _att_weights(D, ATT, g, std=0.1)
    w["q"][:, :2] = 0
    w["k"][:, :2] = 0
    w["q"][::16, 1] = 5.0            # every query head's first dimension
    w["k"][::16, 0] = 5.0
    w["sink"][:] = torch.tensor([1.0, -2.0, 0.5, 3.0, 0.0, -0.5])
    part = _att_part(D, ATT, w, dtype)
    x = 0.3 * torch.randn(T, D, generator=g)
    x[:, :2] = 0
    x[ki, 0] = 6.0
    x[qi, 1] = 6.0
    x = _bf(x)
    cuts = [[T]] if not decoded else [[max(qi - 3, 1)]] + [[1]] * (T - max(qi - 3, 1))
    got = _run_mixer(part, PagesCtx(dtype, 1, 2, 16, 24), [x], cuts, dtype, D)[0]
    want = pg.attention_mixer(x.double(), ATT, _dbl(w), 1e-5, torch.arange(T))
    _close(got, want, dtype, f"query {qi}, key {ki}")
    x2 = x.clone()
    x2[ki, 0] = 0
    moved = float((pg.attention_mixer(x2.double(), ATT, _dbl(w), 1e-5, torch.arange(T))[qi] - want[qi]).abs().max())
    assert (moved > 0.02) == (qi // 11 == ki // 11), f"key {ki} moves query {qi} by {moved}"
    if qi // 11 != ki // 11:
        no_sink = dict(_dbl(w), sink=torch.full((6,), -30.0, dtype=F))
        assert float((pg.attention_mixer(x.double(), ATT, no_sink, 1e-5, torch.arange(T))[qi] - want[qi]).abs().max()) > 0.02


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("distance", [299, 300])
def test_latent_far_key_among_hundreds(distance, decoded, dtype):
    """A window of 300 over 330 tokens: one key 299 back decides the output, the same key 300 back is not seen; in
    bfloat16 the tensor-core kernel walks ten key tiles for it, as a prompt portion and token by token."""
    far = dict(LAT, mask={"size": 300})
    D, T, qi = 56, 330, 325
    g = torch.Generator().manual_seed(14)
    w = _lat_weights(D, far, g, True, std=0.1)
    for name in ("dq", "dkv"):
        w[name][:, :2] = 0
    w["dkv"][0, 0] = 3.0
    w["dq"][0, 1] = 3.0
    w["uq"][:] = 0
    w["uk"][:] = 0
    for h in range(far["heads"]):
        w["uq"][h * 32, 0] = 4.0
        w["uk"][h * 24, 0] = 4.0
    part = _lat_part(D, far, w, dtype, True)
    x = 0.3 * torch.randn(T, D, generator=g)
    x[:, :2] = 0
    x[qi - distance, 0] = 6.0
    x[qi, 1] = 6.0
    x = _bf(x)
    cuts = [[T]] if not decoded else [[qi - 2]] + [[1]] * (T - qi + 2)
    got = _run_mixer(part, PagesCtx(dtype, 1, 1, 56, 0, max_len=512), [x], cuts, dtype, D)[0]
    want = pg.latent_attention_mixer(x.double(), far, _dbl(w), 1e-5, torch.arange(T), True)
    _close(got, want, dtype, f"key {distance} back", b16=3e-2)
    x2 = x.clone()
    x2[qi - distance, 0] = 0
    moved = float((pg.latent_attention_mixer(x2.double(), far, _dbl(w), 1e-5, torch.arange(T), True)[qi] - want[qi]).abs().max())
    assert (moved > 0.1) == (distance < 300), f"the key {distance} back moves the output by {moved}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("decoded", [False, True])
def test_attention_far_key_inside_a_long_block(decoded, dtype):
    """Blocks of 500 positions: the key 400 back lies in the query's block and is seen by the heads whose bias is small."""
    far = dict(ATT, mask={"size": 500})
    D, T, qi, ki = 48, 440, 430, 30
    g = torch.Generator().manual_seed(15)
    w = _att_weights(D, far, g, std=0.1)
    w["q"][:, :2] = 0
    w["k"][:, :2] = 0
    w["q"][::16, 1] = 5.0
    w["k"][::16, 0] = 5.0
    part = _att_part(D, far, w, dtype)
    x = 0.3 * torch.randn(T, D, generator=g)
    x[:, :2] = 0
    x[ki, 0] = 6.0
    x[qi, 1] = 6.0
    x = _bf(x)
    cuts = [[T]] if not decoded else [[qi - 2]] + [[1]] * (T - qi + 2)
    got = _run_mixer(part, PagesCtx(dtype, 1, 2, 16, 24, max_len=512), [x], cuts, dtype, D)[0]
    want = pg.attention_mixer(x.double(), far, _dbl(w), 1e-5, torch.arange(T))
    _close(got, want, dtype, "far key in the block", b16=3e-2)
    x2 = x.clone()
    x2[ki, 0] = 0
    moved = float((pg.attention_mixer(x2.double(), far, _dbl(w), 1e-5, torch.arange(T))[qi] - want[qi]).abs().max())
    assert moved > 0.05, f"the far key moves the output by {moved} only"


@pytest.mark.parametrize("dtype", DTYPES)
def test_routed_experts_part_and_output_norm_block(dtype):
    from geneinfer_b200.config import LayerSpec, PartSpec
    from geneinfer_b200.parts import BLOCKS, LayerRun
    D, E, top, I = 48, 5, 2, 40
    g = torch.Generator().manual_seed(12)
    wa = _att_weights(D, ATT, g)
    ff = {"router": torch.randn(E, D, generator=g) * 0.4, "correction": torch.randn(E, generator=g) * 0.3}
    for e in range(E):
        ff[f"e{e}.gate"], ff[f"e{e}.up"], ff[f"e{e}.down"] = (_bf(torch.randn(*s, generator=g) * 0.2) for s in ((I, D), (I, D), (D, I)))
    n1, n2 = 1 + 0.2 * torch.randn(D, generator=g), 1 + 0.2 * torch.randn(D, generator=g)
    from geneinfer_b200.config.gekupel import distance_slopes
    mixer = PartSpec("attention", {"hidden_size": D, "num_heads": 6, "num_kv_heads": 2, "head_dim": 16, "value_dim": 24, "scale": 0.45,
                                   "window": None, "chunk": 11, "position": PartSpec("none", {}), "qk_norm_eps": 1e-5,
                                   "qk_norm_weights": False, "distance_slopes": distance_slopes(6), "sink": "learned"})
    norm = PartSpec("rmsnorm", {"size": D, "eps": 1e-5})
    spec = LayerSpec(mixer=mixer, feed_forward=PartSpec("routed_experts", {"hidden_size": D, "intermediate_size": I, "experts": E, "top": top}),
                     mixer_norm=norm, feed_forward_norm=norm, block="output_norm")
    weights = {"mixer.w_qkv": torch.cat([wa["q"], wa["k"], wa["v"]]), "mixer.w_o": wa["o"], "mixer.sink": wa["sink"],
               "mixer_norm.weight": n1, "feed_forward_norm.weight": n2, "feed_forward.router": ff["router"],
               "feed_forward.correction": ff["correction"],
               "feed_forward.w_gate_up": torch.stack([torch.cat([ff[f"e{e}.gate"], ff[f"e{e}.up"]]) for e in range(E)]),
               "feed_forward.w_down": torch.stack([ff[f"e{e}.down"] for e in range(E)])}
    block = BLOCKS["output_norm"](spec, weights, _build(dtype))
    x0 = 2.0 * torch.randn(30, D, generator=g)
    rnd = pg.ident if dtype is torch.float32 else pg.bf16
    x = x0.double()
    x = x + pg.rms_norm(pg.attention_mixer(x, ATT, _dbl(wa), 1e-5, torch.arange(30), rnd), n1.double(), 1e-5)
    want = x + pg.rms_norm(pg.moe_ff(x, {"router": {"top": top}}, _dbl(ff), rnd), n2.double(), 1e-5)
    ctx = PagesCtx(dtype, 1, 2, 16, 24)
    ctx.tap = lambda *a: None
    outs = []
    at = 0
    for n in (13, 1, 2, 14):               # the stream itself goes in and out; two layers' worth of carry is not assumed
        ctx.begin([n])
        ctx.carry.clear()
        xs = x0[at:at + n].to(DEV).clone()
        block.forward(ctx, LayerRun(0, 0, True), xs)
        outs.append(xs.cpu())
        at += n
    _close(torch.cat(outs), want, dtype, "output-norm block with routed experts", b16=4e-2)


@pytest.mark.parametrize("T, E, top, D, I", [(300, 6, 2, 64, 40), (130, 3, 2, 128, 136), (700, 20, 5, 72, 8)])
def test_routed_experts_on_the_tensor_cores(T, E, top, D, I):
    """Many pairs in bfloat16: rows gathered into tiles of 128 per expert, both products on the tensor cores. The
    same part with few rows (the CUDA cores) must agree with it row by row."""
    from geneinfer_b200.parts import FEED_FORWARDS
    g = torch.Generator().manual_seed(13)
    ff = {"router": torch.randn(E, D, generator=g) * 0.4, "correction": torch.randn(E, generator=g) * 0.3}
    for e in range(E):
        ff[f"e{e}.gate"], ff[f"e{e}.up"], ff[f"e{e}.down"] = (_bf(torch.randn(*s, generator=g) * 0.2) for s in ((I, D), (I, D), (D, I)))
    weights = {"router": ff["router"], "correction": ff["correction"],
               "w_gate_up": torch.stack([torch.cat([ff[f"e{e}.gate"], ff[f"e{e}.up"]]) for e in range(E)]),
               "w_down": torch.stack([ff[f"e{e}.down"] for e in range(E)])}
    part = FEED_FORWARDS["routed_experts"]({"hidden_size": D, "intermediate_size": I, "experts": E, "top": top}, weights,
                                           _build(torch.bfloat16))
    assert T * top >= part.TC_FROM_PAIRS
    x = _bf(torch.randn(T, D, generator=g))
    ctx = PagesCtx(torch.bfloat16, 1, 1, 8, 8)
    ctx.max_step_tokens = 1024
    y = torch.zeros(T, D, device=DEV)
    part.forward(ctx, x.to(DEV).to(torch.bfloat16), y)
    want = pg.moe_ff(x.double(), {"router": {"top": top}}, _dbl(ff), pg.bf16)
    _close(y.cpu(), want, torch.bfloat16, "routed experts on the tensor cores", b16=1.5e-2)
    few = torch.zeros(40, D, device=DEV)
    part.forward(ctx, x[:40].to(DEV).to(torch.bfloat16), few)
    _close(few.cpu(), y.cpu()[:40], torch.bfloat16, "few rows against many", b16=1e-2)


# ------------------------------------------------------------------------------------------ whole models
_TMP = {}
LENGTHS = {"a": [1, 2, 3, 75, 20, 120, 47, 30], "b": [150, 4, 64, 1, 99], "c": [90, 2, 33, 1, 140, 17]}
CONFIGS = {"a": gc.GEK_A, "b": gc.GEK_B, "c": gc.GEK_C}


def _model_dir(case, tmp_path_factory):
    if case not in _TMP:
        _TMP[case] = gc.make_model_dir(CONFIGS[case], {"a": 23, "b": 31, "c": 37}[case], str(tmp_path_factory.mktemp("gekupel_" + case)))
    return _TMP[case]


def _requests(case):
    return {f"r{i}": tc.random_tokens(n, CONFIGS[case]["vocab"], 400 + i) for i, n in enumerate(LENGTHS[case])}


_PLAIN = {}


def _plain(case, folder, rounded=False):
    key = (case, rounded)
    if key not in _PLAIN:
        cfg, w = pg.load(folder)
        _PLAIN[key] = {rid: pg.forward(cfg, w, toks, pg.bf16 if rounded else pg.ident)[0].numpy() for rid, toks in _requests(case).items()}
    return _PLAIN[key]


def _tolerance(case, folder, dtype):
    """32-bit: rounding of the logits' size. bfloat16: the engine rounds at other places than the plain model's
    ``bf16`` (it applies the heads' key matrices to the queries), so it is compared with the exact plain model and
    allowed three times the distance between the plain model's two precisions; a wrong key or expert in these sharp
    models moves the logits by far more."""
    if dtype == "float32":
        return 3e-5
    exact, rounded = _plain(case, folder), _plain(case, folder, True)
    return 3.0 * max(tt.rel_err(rounded[r], exact[r]) for r in exact)


def _engine(folder, dtype, n_pages, max_requests=4, page_size=16, max_step_tokens=512):
    from geneinfer_b200.engine.loading import load_model
    from geneinfer_b200.engine.step import StepEngine
    model = load_model(folder, dtype=dtype, max_position=512)
    return StepEngine(model, page_size=page_size, n_pages=n_pages, max_requests=max_requests, max_step_tokens=max_step_tokens,
                      debug_checks=True)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["a", "b", "c"])
def test_whole_prompts_decoding_portions_and_mixed_batches_agree_with_the_plain_model(case, dtype, tmp_path_factory):
    folder = _model_dir(case, tmp_path_factory)
    reqs, plain, tol = _requests(case), _plain(case, folder), _tolerance(case, folder, dtype)
    traces = {"whole": tt.trace_whole(reqs), "decode": tt.trace_tail_decode(reqs, tail=40), "portions": tt.trace_portions(reqs),
              "mixed": tt.trace_mixed(reqs, seed=3, tail=12), "mixed2": tt.trace_mixed(reqs, seed=8, max_live=3, tail=30)}
    results = {}
    for name, steps in traces.items():
        # the pool holds what the trace's live requests need, no more: pages are used again
        n_pages = tt.max_tokens_of(steps, reqs, 16) // 16 + (8 if name.startswith("mixed") else 0)
        engine = _engine(folder, dtype, n_pages)
        got = tt.run_in_process(engine, steps)
        engine.check_status()
        tt.compare(got, plain, tol, f"Gekupel {case} {dtype} {name}")
        engine.cache.check_invariants()
        assert engine.cache.slots.free_count == 4 and all(g.pool.free_count == g.pool.n_pages for g in engine.cache.groups)
        results[name] = got
    if dtype == "float32":       # the same position under different cuts: equal but for rounding
        for name in ("decode", "portions", "mixed"):
            for key, row in results[name].items():
                ref = results["whole"][key]
                assert float(np.abs(row - ref).max()) < 2e-5 * max(1.0, float(np.abs(ref).max())), (name, key)


def test_layers_share_weights_but_not_caches(tmp_path_factory):
    folder = _model_dir("a", tmp_path_factory)
    engine = _engine(folder, "float32", n_pages=8)
    model = engine.model
    assert model.layers[3] is model.layers[1] and (model.runs[3].layer, model.runs[3].cache_layer) == (1, 3)
    k1, k3 = engine.layer_pages[1][0], engine.layer_pages[3][0]
    assert k1.data_ptr() != k3.data_ptr() and engine.layer_pages[0][1] is None and engine.layer_pages[1][1].shape[-1] == 40
    # blocks and windows give pages back while a request runs: 100 tokens in a pool of 8 pages of 16
    cfg, w = pg.load(folder)
    toks = tc.random_tokens(100, 190, 5)
    got = tt.run_in_process(engine, tt.trace_portions({"r": toks}, sizes=(7, 30, 2, 16)))
    tt.compare(got, {"r": pg.forward(cfg, w, toks)[0].numpy()}, 3e-5, "pages given back behind blocks and windows")
    assert [g.need.chunk for g in engine.cache.groups if g.need.chunk] == [19]


def test_long_decoding_under_graphs(tmp_path_factory):
    """160 tokens decoded one by one after a 12-token prompt: windows and blocks pass over decoded tokens only, pages go
    back behind them, CUDA graphs replay the steps."""
    folder = _model_dir("a", tmp_path_factory)
    toks = tc.random_tokens(172, 190, 77)
    cfg, w = pg.load(folder)
    want = {"r": pg.forward(cfg, w, toks)[0].numpy()}
    for dtype in ("float32", "bfloat16"):
        engine = _engine(folder, dtype, n_pages=6)
        got = tt.run_in_process(engine, tt.trace_tail_decode({"r": toks}, tail=160))
        tt.compare(got, want, _tolerance("a", folder, dtype), f"long decoding {dtype}")
        assert engine.graph_replays > 100
        assert all(g.pool.free_count == g.pool.n_pages for g in engine.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine_and_its_scheduler(dtype, tmp_path_factory):
    from geneinfer_b200 import Engine
    folder = _model_dir("b", tmp_path_factory)
    cfg, w = pg.load(folder)
    prompts = [tc.random_tokens(n, 260, 900 + n) for n in (5, 40, 1, 18, 9)]
    engine = Engine(folder, dtype=dtype, max_seq_len=256, max_running=3, kv_pages=40, step_tokens=32, prefill_chunk=16)
    got = engine.generate(prompts, max_new_tokens=10, temperature=0.0)
    for prompt, gen in zip(prompts, got):
        assert len(gen) == 10
        tokens = list(prompt)
        for k, t in enumerate(gen):
            logits = pg.forward(cfg, w, tokens)[0][-1].numpy()
            best = int(np.argmax(logits))
            if t != best:                 # only a near-tie may differ
                assert float(logits[best] - logits[t]) < (1e-4 if dtype == "float32" else 8e-2), (k, t, best)
            tokens.append(t)
    assert engine.stats.max_running_seen == 3 and engine.steps.cache.slots.free_count == 3


@pytest.mark.parametrize("page_size", [8, 12, 64])
def test_other_page_sizes(page_size, tmp_path_factory):
    folder = _model_dir("b", tmp_path_factory)
    reqs = {k: v for k, v in list(_requests("b").items())[:3]}
    from geneinfer_b200.engine.loading import load_model
    from geneinfer_b200.engine.step import StepEngine
    for dtype in ("float32", "bfloat16"):
        steps = tt.trace_mixed(reqs, seed=2, tail=20)
        model = load_model(folder, dtype=dtype, max_position=504)
        engine = StepEngine(model, page_size=page_size, n_pages=tt.max_tokens_of(steps, reqs, 64) // page_size + 8, max_requests=4,
                            max_step_tokens=512, debug_checks=True)
        got = tt.run_in_process(engine, steps)
        engine.check_status()
        tt.compare(got, _plain("b", folder), _tolerance("b", folder, dtype), f"page size {page_size} {dtype}")


def test_trace_replay_tool_and_command_line(tmp_path, tmp_path_factory):
    folder = _model_dir("a", tmp_path_factory)
    reqs = {k: v for k, v in list(_requests("a").items())[3:6]}
    steps = tt.trace_mixed(reqs, seed=5, max_live=2, tail=6)
    got = tt.run_trace_tool(folder, "float32", steps, tt.max_tokens_of(steps, reqs), str(tmp_path / "out"), 190)
    tt.compare(got, _plain("a", folder), 3e-5, "trace replay")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "gi_generate"), "--model", folder, "--prompt-ids", "5 9 2 100",
                        "--steps", "12", "--temperature", "0", "--no-echo", "--dtype", "fp32", "--max-seq-len", "64"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr
    out = [int(t) for t in p.stdout.split()]
    cfg, w = pg.load(folder)
    tokens = [5, 9, 2, 100]
    for t in out[:4]:
        logits = pg.forward(cfg, w, tokens)[0][-1].numpy()
        assert t == int(np.argmax(logits)) or float(logits.max() - logits[t]) < 1e-4
        tokens.append(t)
    assert len(out) == 9
