"""Nipadra on the GPU against the plain implementation in plain_nipadra.py: each mechanism alone, then whole
models through the step engine under different cuts of the same requests (whole prompts, token-by-token
decoding, portions down to two tokens, mixed batches on reused pages and state slots), window edges made
visible by construction, and greedy generation through the engine's own entry point and scheduler."""
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import nipadra_configs as nc
import plain_nipadra as pn
import tiny_configs as tc
import trace_tools as tt

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]


def _build(dtype, max_position=4096):
    from geneinfer_b200.parts import BuildContext
    return BuildContext(DEV, dtype, max_position)


def _bf(t):
    return t.to(torch.bfloat16).float()


class MiniCtx:
    """The least a mixer needs of a step, kept across steps: pages and block tables of one layer, state slots,
    and the row arrays of the current step. ``begin(lengths)`` starts a step in which request r brings
    ``lengths[r]`` more tokens (0: it sits this step out)."""

    def __init__(self, dtype, n_requests, Hkv=1, hd=16, page_size=8, max_len=256, state_floats=0, slots=None):
        self.page_size, self.dtype = page_size, dtype
        self.fed = [0] * n_requests
        per = (max_len + page_size - 1) // page_size
        order = torch.randperm(n_requests * per, generator=torch.Generator().manual_seed(5)).int()
        self._all_tables = order.view(n_requests, per)            # pages scattered over the pool
        self._pages = tuple(torch.full((n_requests * per, Hkv, page_size, hd), float("nan"), dtype=dtype, device=DEV)
                            for _ in range(2))
        self._slots = list(slots) if slots is not None else list(range(n_requests))[::-1]
        self._state = torch.zeros(n_requests + 1, max(state_floats, 1), dtype=torch.float32, device=DEV)
        self.carry = {}

    def begin(self, lengths):
        live = [r for r, n in enumerate(lengths) if n > 0]
        self.n_requests = len(live)
        self.max_requests = len(lengths)
        self.positions = torch.cat([torch.arange(self.fed[r], self.fed[r] + lengths[r]) for r in live]).int().to(DEV)
        self.row_req = torch.cat([torch.full((lengths[r],), i) for i, r in enumerate(live)]).int().to(DEV)
        starts = np.cumsum([0] + [lengths[r] for r in live])
        self.seg_start = torch.tensor(starts[:-1], dtype=torch.int32, device=DEV)
        self.seg_len = torch.tensor([lengths[r] for r in live], dtype=torch.int32, device=DEV)
        self.state_slots = torch.tensor([self._slots[r] for r in live], dtype=torch.int32, device=DEV)
        self._tables = self._all_tables[live].contiguous().to(DEV)
        self.n_tokens = int(starts[-1])
        self.rows = {r: slice(int(starts[i]), int(starts[i + 1])) for i, r in enumerate(live)}
        for r in live:
            self.fed[r] += lengths[r]
        return self

    def pages(self, layer):
        return self._pages

    def block_tables(self, layer):
        return self._tables

    def state(self, layer):
        return self._state

    def scratch(self, name, shape, dtype, capacity=None):
        return torch.full(shape, float("nan"), dtype=dtype, device=DEV)

    def attention_work(self, per_tile):
        """(rows of requests that bring one token, tiles (first row, tokens, request) of the others, longest context
        among the single tokens), as the tensor-core attention kernels take them."""
        starts, lens = self.seg_start.tolist(), self.seg_len.tolist()
        pos = self.positions.tolist()
        single = [s for s, n in zip(starts, lens) if n == 1]
        tiles = [(s + t, min(per_tile, n - t), r) for r, (s, n) in enumerate(zip(starts, lens)) if n > 1
                 for t in range(0, n, per_tile)]
        longest = max([pos[s] + 1 for s in single], default=0)
        return (torch.tensor(single, dtype=torch.int32, device=DEV),
                torch.tensor(tiles, dtype=torch.int32, device=DEV).reshape(len(tiles), 3), longest)


def _run_mixer(part, ctx, inputs, cuts, dtype, D):
    """Feeds each request's rows of ``inputs`` [n][T_r, D] through ``part`` under the schedule ``cuts`` (a list
    of per-request lengths per step); returns each request's output rows in order."""
    from geneinfer_b200.parts import LayerRun
    outs = [[] for _ in inputs]
    at = [0] * len(inputs)
    for lengths in cuts:
        ctx.begin(lengths)
        xn = torch.zeros(ctx.n_tokens, D)
        for r, sl in ctx.rows.items():
            xn[sl] = inputs[r][at[r]:at[r] + lengths[r]]
        acc = torch.zeros(ctx.n_tokens, D, device=DEV)
        part.forward(ctx, LayerRun(0, 0, True), xn.to(DEV).to(dtype), acc)
        res = acc.cpu()
        for r, sl in ctx.rows.items():
            outs[r].append(res[sl])
            at[r] += lengths[r]
    return [torch.cat(o) for o in outs]


def _close(got, want, dtype, what):
    err = float((got - want).abs().max() / max(1.0, float(want.abs().max())))
    assert err < (2e-5 if dtype is torch.float32 else 2e-2), f"{what}: {err}"


# ------------------------------------------------------------------------------------------ elementwise kernels
@pytest.mark.parametrize("dtype", DTYPES)
def test_scale_cast_and_residual_norm(dtype):
    from geneinfer_b200.ops import kernels
    g = torch.Generator().manual_seed(1)
    for D in (200, 7, 1024):
        x = torch.randn(11, D, generator=g) * 3
        w = 0.1 * torch.randn(D, generator=g)
        acc = torch.empty(11, D, device=DEV)
        xn = torch.empty(11, D, dtype=dtype, device=DEV)
        kernels.scale_cast(x.to(DEV), acc, xn, 1.7)
        assert torch.equal(acc.cpu(), 1.7 * x) and torch.equal(xn.cpu().float(), x.to(dtype).float())
        y = torch.randn(11, D, generator=g)
        acc += y.to(DEV)
        x_out = torch.empty(11, D, device=DEV)
        kernels.residual_norm(acc, (1.0 + w).to(DEV), x_out, 1e-3, 1.7, acc_out=acc, xn_out=xn)
        want = pn.norm_one_plus(1.7 * x + y, w, 1e-3)
        assert float((x_out.cpu() - want).abs().max()) < 2e-6 * max(1.0, float(want.abs().max()))
        assert torch.equal(acc.cpu(), 1.7 * x_out.cpu()) and torch.equal(xn.cpu().float(), x_out.cpu().to(dtype).float())


@pytest.mark.parametrize("act", ["relu", "silu", "gelu_tanh"])
def test_gated_activation(act):
    from geneinfer_b200.ops import kernels
    gu = torch.randn(9, 2 * 37, generator=torch.Generator().manual_seed(2)) * 3
    out = torch.empty(9, 37, device=DEV)
    kernels.gated_act(gu.to(DEV), out, act)
    want = pn.ACTS[act](gu[:, :37]) * gu[:, 37:]
    assert float((out.cpu() - want).abs().max()) < 1e-5


@pytest.mark.parametrize("rows", [13, 200])          # 200 rows in bfloat16: the activation runs in the product's epilogue
@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_feed_forward_part(dtype, rows):
    from geneinfer_b200.parts import FEED_FORWARDS
    D, I = 40, 112
    g = torch.Generator().manual_seed(4)
    w = {"p.gate": _bf(torch.randn(I, D, generator=g) * 0.3), "p.up": _bf(torch.randn(I, D, generator=g) * 0.3),
         "p.down": _bf(torch.randn(D, I, generator=g) * 0.3)}
    for act in ("relu", "gelu_tanh"):
        part = FEED_FORWARDS["gated_mlp"]({"hidden_size": D, "intermediate_size": I, "activation": act},
                                          {"w_gate_up": torch.cat([w["p.gate"], w["p.up"]]), "w_down": w["p.down"]}, _build(dtype))
        xn = torch.randn(rows, D, generator=g).to(dtype)
        x = torch.randn(rows, D, generator=g)
        x_dev = x.clone().to(DEV)
        part.forward(MiniCtx(dtype, 1), xn.to(DEV), x_dev)
        rnd = pn.ident if dtype is torch.float32 else pn.bf16
        want = x + pn.dense_ff(xn.float(), w, "p.", {"act": act}, rnd=rnd)
        _close(x_dev.cpu(), want, dtype, f"gated feed-forward {act}")


# ------------------------------------------------------------------------------------------ the mixers alone
LIN = {"heads": 3, "dim": 16, "vdim": 40, "decay": [1.0, 0.8, 0.3]}


def _lin_weights(D, m, g):
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    return {"p.q": _bf(torch.randn(H * dk, D, generator=g) * 0.4), "p.k": _bf(torch.randn(H * dk, D, generator=g) * 0.4),
            "p.v": _bf(torch.randn(H * dv, D, generator=g) * 0.4), "p.g": _bf(torch.randn(H * dv, D, generator=g) * 0.4),
            "p.o": _bf(torch.randn(D, H * dv, generator=g) * 0.3), "p.norm": 1 + 0.2 * torch.randn(H * dv, generator=g)}


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_attention_mixer_with_its_state_carried_across_steps(dtype):
    from geneinfer_b200.parts import MIXERS
    D, m = 56, LIN
    g = torch.Generator().manual_seed(7)
    w = _lin_weights(D, m, g)
    part = MIXERS["linear_attention"]({"hidden_size": D, "num_heads": m["heads"], "key_dim": m["dim"], "value_dim": m["vdim"],
                                       "decay": m["decay"], "norm_eps": 1e-5, "out_scale": 0.75},
                                      {"w_in": torch.cat([w["p.q"], w["p.k"], w["p.v"], w["p.g"]]), "w_o": w["p.o"], "norm": w["p.norm"]},
                                      _build(dtype))
    assert part.cache_need() is None and part.state_need().shape == (3 * 16 * 40,)
    inputs = [_bf(torch.randn(n, D, generator=g)) for n in (45, 1, 23)]
    rnd = pn.ident if dtype is torch.float32 else pn.bf16
    want = [0.75 * pn.lightning_mixer(x, w, "p.", m, 1e-5, rnd=rnd) for x in inputs]
    # whole; then cut into steps of unequal portions and single tokens, with a request left out of a step
    for cuts in ([[45, 1, 23]], [[17, 0, 2], [1, 1, 0], [20, 0, 19], [1, 0, 1], [6, 0, 1]]):
        ctx = MiniCtx(dtype, 3, state_floats=3 * 16 * 40)
        got = _run_mixer(part, ctx, inputs, cuts, dtype, D)
        for r in range(3):
            _close(got[r], want[r], dtype, f"linear attention, request {r}, {len(cuts)} steps")


SSM = {"heads": 4, "vdim": 24, "state": 16, "groups": 2, "conv": 4, "norm_groups": 2}


def _ssm_weights(D, m, g):
    inner, C = m["heads"] * m["vdim"], m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
    return {"p.in": _bf(torch.randn(2 * inner + 2 * m["groups"] * m["state"] + m["heads"], D, generator=g) * 0.4),
            "p.conv": torch.randn(C, m["conv"], generator=g) * 0.5, "p.conv.b": torch.randn(C, generator=g) * 0.2,
            "p.dt_bias": torch.rand(m["heads"], generator=g) * 2 - 1.5, "p.A_log": torch.rand(m["heads"], generator=g) * 2 - 1,
            "p.D": 1 + 0.3 * torch.randn(m["heads"], generator=g), "p.norm": 1 + 0.2 * torch.randn(inner, generator=g),
            "p.o": _bf(torch.randn(D, inner, generator=g) * 0.3)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", [SSM, dict(SSM, conv=1, groups=4, norm_groups=1, state=40), dict(SSM, heads=2, groups=1, vdim=70, conv=2)])
def test_state_space_mixer_with_state_and_convolution_inputs_carried_across_steps(dtype, m):
    from geneinfer_b200.parts import MIXERS
    D = 48
    g = torch.Generator().manual_seed(8)
    w = _ssm_weights(D, m, g)
    part = MIXERS["state_space"]({"hidden_size": D, "num_heads": m["heads"], "head_dim": m["vdim"], "state_size": m["state"],
                                  "groups": m["groups"], "conv_taps": m["conv"], "norm_groups": m["norm_groups"], "norm_eps": 1e-5},
                                 {"w_in": w["p.in"], "w_o": w["p.o"], "conv": w["p.conv"], "conv_bias": w["p.conv.b"],
                                  "dt_bias": w["p.dt_bias"], "a_log": w["p.A_log"], "skip": w["p.D"], "norm": w["p.norm"]}, _build(dtype))
    floats = part.state_need().shape[0]
    assert floats == m["heads"] * m["state"] * m["vdim"] + (m["conv"] - 1) * (m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"])
    inputs = [_bf(torch.randn(n, D, generator=g)) for n in (40, 2, 19)]
    rnd = pn.ident if dtype is torch.float32 else pn.bf16
    want = [rnd(pn.right_mixer(x, w, "p.", m, 1e-5, rnd=rnd)) @ w["p.o"].T for x in inputs]
    # portions shorter than the convolution's reach (1 and 2 tokens with 4 taps) follow one another
    for cuts in ([[40, 2, 19]], [[1, 1, 2], [1, 1, 0], [2, 0, 1], [1, 0, 16], [30, 0, 0], [5, 0, 0]]):
        ctx = MiniCtx(dtype, 3, state_floats=floats)
        got = _run_mixer(part, ctx, inputs, cuts, dtype, D)
        for r in range(3):
            _close(got[r], want[r], dtype, f"state space, request {r}, {len(cuts)} steps")


@pytest.mark.parametrize("kind", ["linear_attention", "state_space"])
def test_long_portions_are_cut_into_parts_that_run_side_by_side(kind):
    """Steps of more than 128 tokens cut every segment into parts of 128 (zero-state scans, linked start states,
    the start states' share added): the same results as token by token, parts ending inside and at the end of
    segments, beside single tokens, from states that earlier steps left."""
    from geneinfer_b200.parts import MIXERS
    D, dtype = 40, torch.float32
    g = torch.Generator().manual_seed(21)
    if kind == "linear_attention":
        m = {"heads": 2, "dim": 32, "vdim": 48, "decay": [1.0, 0.93]}
        w = _lin_weights(D, m, g)
        part = MIXERS[kind]({"hidden_size": D, "num_heads": 2, "key_dim": 32, "value_dim": 48, "decay": m["decay"], "norm_eps": 1e-5},
                            {"w_in": torch.cat([w["p.q"], w["p.k"], w["p.v"], w["p.g"]]), "w_o": w["p.o"], "norm": w["p.norm"]},
                            _build(dtype))
        plain = lambda x: pn.lightning_mixer(x, w, "p.", m, 1e-5)
    else:
        m = dict(SSM, heads=2, groups=1, state=24)
        w = _ssm_weights(D, m, g)
        part = MIXERS[kind]({"hidden_size": D, "num_heads": 2, "head_dim": 24, "state_size": 24, "groups": 1, "conv_taps": 4,
                             "norm_groups": 2, "norm_eps": 1e-5},
                            {"w_in": w["p.in"], "w_o": w["p.o"], "conv": w["p.conv"], "conv_bias": w["p.conv.b"],
                             "dt_bias": w["p.dt_bias"], "a_log": w["p.A_log"], "skip": w["p.D"], "norm": w["p.norm"]}, _build(dtype))
        plain = lambda x: pn.right_mixer(x, w, "p.", m, 1e-5) @ w["p.o"].T
    inputs = [_bf(0.5 * torch.randn(n, D, generator=g)) for n in (300, 2, 259)]
    want = [plain(x) for x in inputs]
    for cuts in ([[300, 2, 259]], [[129, 1, 3], [43, 1, 128], [128, 0, 128]]):
        ctx = MiniCtx(dtype, 3, state_floats=part.state_need().shape[0], max_len=320)
        got = _run_mixer(part, ctx, inputs, cuts, dtype, D)
        for r in range(3):
            _close(got[r], want[r], dtype, f"{kind} in parts, request {r}, {len(cuts)} steps")


ATT = {"heads": 6, "kv_heads": 2, "dim": 32, "vdim": 32, "mask": {"size": 11}, "rot": {"base": 300.0, "dims": 16}, "scale": 0.4}


def _att_weights(D, m, g):
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    return {"p.q": _bf(torch.randn(H * d, D, generator=g) * 0.4), "p.k": _bf(torch.randn(G * d, D, generator=g) * 0.4),
            "p.g": _bf(torch.randn(H, D, generator=g) * 0.4), "p.q.norm": 1 + 0.3 * torch.randn(d, generator=g),
            "p.k.norm": 1 + 0.3 * torch.randn(d, generator=g), "p.o": _bf(torch.randn(D, H * d, generator=g) * 0.3)}


def _att_part(D, m, w, dtype):
    from geneinfer_b200.config import PartSpec
    from geneinfer_b200.parts import MIXERS
    rope = PartSpec("rope_on_device", {"head_dim": m["dim"], "rotary_dim": m["rot"]["dims"], "theta": m["rot"]["base"],
                                       "pairing": "interleaved"})
    return MIXERS["attention"]({"hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                                "scale": m["scale"], "window": m["mask"]["size"], "position": rope, "values": "keys",
                                "qk_norm_eps": 1e-5, "sink": True, "head_gate": True},
                               {"w_qkv": torch.cat([w["p.q"], w["p.k"], w["p.g"]]), "w_o": w["p.o"], "q_norm": w["p.q.norm"],
                                "k_norm": w["p.k.norm"]}, _build(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_window_attention_with_sink_gate_and_keys_as_values(dtype):
    D, m = 40, ATT
    g = torch.Generator().manual_seed(9)
    w = _att_weights(D, m, g)
    part = _att_part(D, m, w, dtype)
    need = part.cache_need()
    assert (need.num_kv_heads, need.head_dim, need.window) == (2, 32, 11) and part.state_need() is None
    inputs = [_bf(torch.randn(n, D, generator=g)) for n in (37, 1, 26)]
    rnd = pn.ident if dtype is torch.float32 else pn.bf16
    want = [rnd(pn.left_mixer(x, w, "p.", m, 1e-5, rnd=rnd)) @ w["p.o"].T for x in inputs]
    for cuts in ([[37, 1, 26]], [[9, 1, 2], [1, 0, 1], [14, 0, 1], [2, 0, 22], [11, 0, 0]]):
        ctx = MiniCtx(dtype, 3, Hkv=2, hd=32)
        got = _run_mixer(part, ctx, inputs, cuts, dtype, D)
        for r in range(3):
            _close(got[r], want[r], dtype, f"window attention, request {r}, {len(cuts)} steps")


@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("distance", [10, 11, 8, 16])
def test_a_key_that_stands_out_at_the_windows_edge(decoded, distance):
    """One key is made to dominate the softmax of one query (the two inputs are large along directions that the
    unrotated dimensions of q and k share). With the key ``distance`` tokens back and a window of 11 the
    output of that query is the key's value row when distance <= 10 and is not when distance = 11; the
    distances 8 and 16 put the key at a page border (pages of 8)."""
    D, m, dtype = 40, ATT, torch.float32
    g = torch.Generator().manual_seed(10 + distance)
    w = _att_weights(D, m, g)
    for name in ("p.q", "p.k"):
        w[name][:, :2] = 0
    # input direction 0 drives unrotated dimension 20 of every key head, direction 1 the same dimension of every query head
    for h in range(m["kv_heads"]):
        w["p.k"][h * 32 + 20, 0] = 4.0
    for h in range(m["heads"]):
        w["p.q"][h * 32 + 20, 1] = 4.0
    w["p.q.norm"][20] = w["p.k.norm"][20] = 3.0
    part = _att_part(D, m, w, dtype)
    T, qi = 40, 33
    x = 0.3 * torch.randn(T, D, generator=g)
    x[:, :2] = 0
    x[qi - distance, 0] = 5.0
    x[qi, 1] = 5.0
    x = _bf(x)
    cuts = [[T]] if not decoded else [[qi - 3]] + [[1]] * (T - qi + 3)
    got = _run_mixer(part, MiniCtx(dtype, 1, Hkv=2, hd=32), [x], cuts, dtype, D)[0]
    want = pn.left_mixer(x, w, "p.", m, 1e-5) @ w["p.o"].T
    _close(got, want, dtype, f"key {distance} back")
    # the construction works: leaving the key out changes that query's output by much more than the tolerance
    x2 = x.clone()
    x2[qi - distance, 0] = 0
    moved = float(((pn.left_mixer(x2, w, "p.", m, 1e-5) @ w["p.o"].T)[qi] - want[qi]).abs().max())
    assert (moved > 0.05) == (distance < 11), f"the key {distance} back moves the output by {moved}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_parallel_mixer_adds_its_scaled_branches(dtype):
    from geneinfer_b200.config import PartSpec
    from geneinfer_b200.parts import MIXERS
    D = 48
    g = torch.Generator().manual_seed(12)
    wa, ws = _att_weights(D, ATT, g), _ssm_weights(D, SSM, g)
    rope = PartSpec("rope_on_device", {"head_dim": 32, "rotary_dim": 16, "theta": 300.0, "pairing": "interleaved"})
    left = PartSpec("attention", {"hidden_size": D, "num_heads": 6, "num_kv_heads": 2, "head_dim": 32, "scale": 0.4, "window": 11,
                                  "position": rope, "values": "keys", "qk_norm_eps": 1e-5, "sink": True, "head_gate": True})
    right = PartSpec("state_space", {"hidden_size": D, "num_heads": 4, "head_dim": 24, "state_size": 16, "groups": 2,
                                     "conv_taps": 4, "norm_groups": 2, "norm_eps": 1e-5})
    weights = {"left.w_qkv": torch.cat([wa["p.q"], wa["p.k"], wa["p.g"]]), "left.w_o": wa["p.o"], "left.q_norm": wa["p.q.norm"],
               "left.k_norm": wa["p.k.norm"], "right.w_in": ws["p.in"], "right.w_o": ws["p.o"], "right.conv": ws["p.conv"],
               "right.conv_bias": ws["p.conv.b"], "right.dt_bias": ws["p.dt_bias"], "right.a_log": ws["p.A_log"],
               "right.skip": ws["p.D"], "right.norm": ws["p.norm"]}
    part = MIXERS["parallel"]({"branches": [("left", left, 0.6), ("right", right, -1.5)]}, weights, _build(dtype))
    assert part.cache_need().window == 11 and part.state_need() is not None
    w = {"p.left." + k[2:]: v for k, v in wa.items()}
    w.update({"p.right." + k[2:]: v for k, v in ws.items()})
    x = _bf(torch.randn(30, D, generator=g))
    rnd = pn.ident if dtype is torch.float32 else pn.bf16
    want = pn.parallel_mixer(x, w, "p.", {"left": ATT, "right": SSM, "left_scale": 0.6, "right_scale": -1.5}, 1e-5, rnd=rnd)
    ctx = MiniCtx(dtype, 1, Hkv=2, hd=32, state_floats=part.state_need().shape[0])
    got = _run_mixer(part, ctx, [x], [[13], [1], [16]], dtype, D)[0]
    _close(got, want, dtype, "parallel mixer")


# ------------------------------------------------------------------------------------------ whole models
_TMP = {}
LENGTHS = {"p": [1, 2, 3, 60, 17, 100, 41, 25], "q": [200, 3, 90, 1, 170]}
CONFIGS = {"p": nc.NIP_P, "q": nc.NIP_Q}


def _model_dir(case, tmp_path_factory):
    if case not in _TMP:
        _TMP[case] = nc.make_model_dir(CONFIGS[case], 17 if case == "p" else 19, str(tmp_path_factory.mktemp("nipadra_" + case)))
    return _TMP[case]


def _requests(case):
    return {f"r{i}": tc.random_tokens(n, CONFIGS[case]["vocab"], 500 + i) for i, n in enumerate(LENGTHS[case])}


_PLAIN = {}


def _plain(case, folder, dtype):
    key = (case, dtype)
    if key not in _PLAIN:
        w, cfg = pn.load(folder)
        rnd = pn.ident if dtype == "float32" else pn.bf16
        _PLAIN[key] = {rid: pn.forward(w, cfg, toks, rnd=rnd).numpy() for rid, toks in _requests(case).items()}
    return _PLAIN[key]


def _tolerance(case, folder, dtype):
    if dtype == "float32":
        return 3e-5
    exact, rounded = _plain(case, folder, "float32"), _plain(case, folder, "bfloat16")
    noise = max(float((np.abs(rounded[r] - exact[r]).max(axis=-1) / np.maximum(1.0, np.abs(exact[r]).max(axis=-1))).max())
                for r in exact)
    # two bfloat16 computations that round at different places (the engine keeps the recurrences' inputs and the
    # attention weights in 32-bit where the plain model rounds them) differ by about the model's own bfloat16
    # noise; a wrong key, state or position in these sharp models moves the logits by ten times as much
    return 2.0 * noise


def _engine(folder, dtype, n_pages, max_requests=4, page_size=16, max_step_tokens=512):
    from geneinfer_b200.engine.loading import load_model
    from geneinfer_b200.engine.step import StepEngine
    model = load_model(folder, dtype=dtype, max_position=512)
    return StepEngine(model, page_size=page_size, n_pages=n_pages, max_requests=max_requests,
                      max_step_tokens=max_step_tokens, debug_checks=True)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["p", "q"])
def test_whole_prompts_decoding_portions_and_mixed_batches_agree_with_the_plain_model(case, dtype, tmp_path_factory):
    folder = _model_dir(case, tmp_path_factory)
    reqs = _requests(case)
    plain = _plain(case, folder, dtype)
    tol = _tolerance(case, folder, dtype)
    traces = {"whole": tt.trace_whole(reqs), "decode": tt.trace_tail_decode(reqs, tail=40), "portions": tt.trace_portions(reqs),
              "mixed": tt.trace_mixed(reqs, seed=3, tail=12), "mixed2": tt.trace_mixed(reqs, seed=8, max_live=3, tail=30)}
    results = {}
    for name, steps in traces.items():
        # the pool holds what the trace's live requests need, no more: pages and state slots are used again
        n_pages = tt.max_tokens_of(steps, reqs, 16) // 16 + (8 if name.startswith("mixed") else 0)
        engine = _engine(folder, dtype, n_pages)
        got = tt.run_in_process(engine, steps)
        engine.check_status()
        tt.compare(got, plain, tol, f"Nipadra {case} {dtype} {name}")
        engine.cache.check_invariants()
        assert engine.cache.slots.free_count == 4 and all(g.pool.free_count == g.pool.n_pages for g in engine.cache.groups)
        results[name] = got
    # the same position under different cuts: equal but for rounding (32-bit: a few ulp of the logits' size)
    if dtype == "float32":
        for name in ("decode", "portions", "mixed"):
            for key, row in results[name].items():
                ref = results["whole"][key]
                assert float(np.abs(row - ref).max()) < 2e-5 * max(1.0, float(np.abs(ref).max())), (name, key)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["NIP_L", "NIP_A"])
def test_models_of_one_kind_of_mixer(name, dtype, tmp_path):
    """Linear attention only (no pages at all: the cache manager has no group) and the parallel pair only (one window
    group per layer, a head size the tensor-core attention kernels are not built for)."""
    config = getattr(nc, name)
    folder = nc.make_model_dir(config, 29, str(tmp_path / name))
    reqs = {f"r{i}": tc.random_tokens(n, config["vocab"], 700 + i) for i, n in enumerate([70, 1, 33, 140, 12])}
    w, cfg = pn.load(folder)
    exact = {rid: pn.forward(w, cfg, toks).numpy() for rid, toks in reqs.items()}
    plain, tol = exact, 3e-5
    if dtype == "bfloat16":
        plain = {rid: pn.forward(w, cfg, toks, rnd=pn.bf16).numpy() for rid, toks in reqs.items()}
        tol = 2.0 * max(tt.rel_err(plain[r], exact[r]) for r in reqs)
    for steps in (tt.trace_whole(reqs), tt.trace_portions(reqs), tt.trace_mixed(reqs, seed=11, tail=10)):
        engine = _engine(folder, dtype, n_pages=tt.max_tokens_of(steps, reqs, 16) // 16 + 4)
        assert len(engine.cache.groups) == (0 if name == "NIP_L" else 2)
        got = tt.run_in_process(engine, steps)
        engine.check_status()
        tt.compare(got, plain, tol, f"{name} {dtype}")
        engine.cache.check_invariants()
        assert engine.cache.slots.free_count == 4


def test_long_decoding_past_the_window_and_over_page_borders(tmp_path_factory):
    """150 tokens decoded one by one after a 20-token prompt: the windows of 20 and 7 tokens pass over decoded
    tokens only, pages are given back behind the window, CUDA graphs replay the steps."""
    folder = _model_dir("p", tmp_path_factory)
    toks = tc.random_tokens(170, 211, 77)
    w, cfg = pn.load(folder)
    for dtype in ("float32", "bfloat16"):
        want = {"r": pn.forward(w, cfg, toks, rnd=pn.ident if dtype == "float32" else pn.bf16).numpy()}
        engine = _engine(folder, dtype, n_pages=12)
        got = tt.run_in_process(engine, tt.trace_tail_decode({"r": toks}, tail=150))
        tol = 3e-5 if dtype == "float32" else _tolerance("p", folder, dtype)
        tt.compare(got, want, tol, f"long decoding {dtype}")
        assert engine.graph_replays > 100
        pool = engine.cache.groups[0].pool
        assert pool.free_count == pool.n_pages


def test_state_slots_start_from_zero_when_they_are_used_again(tmp_path_factory):
    folder = _model_dir("p", tmp_path_factory)
    from geneinfer_b200.engine.step import StepEntry
    engine = _engine(folder, "float32", n_pages=16, max_requests=1)
    a, b = tc.random_tokens(30, 211, 1), tc.random_tokens(22, 211, 2)
    engine.open("a")
    engine.step([StepEntry("a", a, [29])])
    engine.close("a")
    engine.open("b")                      # the same slot and the same pages
    got = engine.step([StepEntry("b", b, [21])]).cpu().numpy()[0]
    w, cfg = pn.load(folder)
    want = pn.forward(w, cfg, b).numpy()[-1]
    assert tt.rel_err(got, want) < 3e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine_and_its_scheduler(dtype, tmp_path_factory):
    from geneinfer_b200 import Engine
    folder = _model_dir("q", tmp_path_factory)
    w, cfg = pn.load(folder)
    prompts = [tc.random_tokens(n, 300, 900 + n) for n in (5, 40, 1, 18, 9)]
    engine = Engine(folder, dtype=dtype, max_seq_len=256, max_running=3, kv_pages=40, step_tokens=32, prefill_chunk=16)
    got = engine.generate(prompts, max_new_tokens=12, temperature=0.0)
    rnd = pn.ident if dtype == "float32" else pn.bf16
    for prompt, g in zip(prompts, got):
        assert len(g) == 12
        tokens = list(prompt)
        for k, t in enumerate(g):
            logits = pn.forward(w, cfg, tokens, rnd=rnd, positions=[len(tokens) - 1])[0].numpy()
            best = int(np.argmax(logits))
            if t != best:                 # only a near-tie may differ
                assert float(logits[best] - logits[t]) < (1e-4 if dtype == "float32" else 6e-2), (k, t, best)
            tokens.append(t)
    assert engine.stats.max_running_seen == 3 and engine.steps.cache.slots.free_count == 3


def test_a_preempted_request_is_recomputed_from_a_zeroed_state(tmp_path_factory):
    """A pool too small for all requests: the scheduler preempts the youngest, whose state slot and pages go back;
    it is recomputed later from its first token and must generate what it generates with room for all."""
    from geneinfer_b200 import Engine
    folder = _model_dir("q", tmp_path_factory)            # a window of 150: no page goes back while these requests run
    prompts = [tc.random_tokens(n, 300, 300 + n) for n in (70, 64, 90)]
    roomy = Engine(folder, dtype="float32", max_seq_len=256, max_running=3, kv_pages=64, step_tokens=48)
    want = roomy.generate(prompts, max_new_tokens=40, temperature=0.0)
    tight = Engine(folder, dtype="float32", max_seq_len=256, max_running=3, kv_pages=14, step_tokens=48)
    got = tight.generate(prompts, max_new_tokens=40, temperature=0.0)
    assert tight.stats.preemptions > 0, "the pool was meant to be too small: no request was preempted"
    for a, b in zip(got, want):
        assert sum(x != y for x, y in zip(a, b)) <= 1, (a, b)       # 32-bit: a near-tie at most
    assert tight.steps.cache.slots.free_count == 3


@pytest.mark.parametrize("page_size", [8, 12, 64])
def test_other_page_sizes(page_size, tmp_path_factory):
    """Pages of 8 and 64 positions (TMA-fed attention kernels) and of 12 (the general kernel also in bfloat16)."""
    folder = _model_dir("q", tmp_path_factory)
    reqs = {k: v for k, v in list(_requests("q").items())[:3]}
    for dtype in ("float32", "bfloat16"):
        plain, tol = _plain("q", folder, dtype), _tolerance("q", folder, dtype)
        steps = tt.trace_mixed(reqs, seed=2, tail=20)
        from geneinfer_b200.engine.loading import load_model
        from geneinfer_b200.engine.step import StepEngine
        model = load_model(folder, dtype=dtype, max_position=504)
        engine = StepEngine(model, page_size=page_size, n_pages=tt.max_tokens_of(steps, reqs, 64) // page_size + 8, max_requests=4,
                            max_step_tokens=512, debug_checks=True)
        got = tt.run_in_process(engine, steps)
        engine.check_status()
        tt.compare(got, plain, tol, f"page size {page_size} {dtype}")


def test_trace_replay_tool_and_command_line(tmp_path, tmp_path_factory):
    folder = _model_dir("p", tmp_path_factory)
    reqs = {k: v for k, v in list(_requests("p").items())[3:6]}
    steps = tt.trace_mixed(reqs, seed=5, max_live=2, tail=6)
    got = tt.run_trace_tool(folder, "float32", steps, tt.max_tokens_of(steps, reqs), str(tmp_path / "out"), 211)
    tt.compare(got, _plain("p", folder, "float32"), 3e-5, "trace replay")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "gi_generate"), "--model", folder, "--prompt-ids", "5 9 2 100",
                        "--steps", "12", "--temperature", "0", "--no-echo", "--dtype", "fp32", "--max-seq-len", "64"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr
    out = [int(t) for t in p.stdout.split()]
    w, cfg = pn.load(folder)
    tokens = [5, 9, 2, 100]
    for t in out[:4]:
        logits = pn.forward(w, cfg, tokens, positions=[len(tokens) - 1])[0].numpy()
        assert t == int(np.argmax(logits)) or float(logits.max() - logits[t]) < 1e-4
        tokens.append(t)
    assert len(out) == 9
    prof = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "gi_generate"), "--model", folder, "--prompt-ids", "5 9 2 100 7 7",
                           "--steps", "9", "--temperature", "0", "--quiet", "--profile", "--max-seq-len", "64"],
                          capture_output=True, text=True, timeout=600)
    assert prof.returncode == 0, prof.stderr
    for op in ("recurrence (state update + output)", "norm after the residual sum", "causal convolution", "attention", "gated norm"):
        assert op in prof.stderr, f"--profile does not report '{op}':\n{prof.stderr}"
