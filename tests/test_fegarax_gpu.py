"""Fegarax on the GPU against the plain implementation (``plain_fegarax``, float64 on the CPU): every mechanism alone, then
whole models under every way of cutting the work: each request alone and whole; most of it in one step and the rest one
token at a time (eagerly and from captured graphs); portions of changing size down to two tokens; mixed batches of unequal
requests with so few pages that they are used again; greedy generation through the engine's entry point and scheduler; and
the trace replay as a user runs it.

Tolerances.  float32: |diff| <= 2e-4 (1 + |ref|), the plain result being float64.  bfloat16: the root mean square of the
difference over a row at most 0.06 of the reference's own root mean square, and at most 0.03 on average.  Whole models in
bfloat16 choose experts from rounded numbers, and a choice that is a close call in float64 may fall the other way: there up
to 4 % of the rows may lie beyond 0.06 (the mechanisms alone, and everything in float32, are held to every row).
"""
import json
import math
import os
import random
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_fegarax as plain
from fegarax_models import CONFIGS, PAGE, make_model_dir
from helpers import mixed_schedule, portions, random_prompt, run_mixed, run_portions, run_whole

pytestmark = pytest.mark.gpu
DEV = torch.device(os.environ.get("MARIN_B200_TEST_DEVICE", "cuda:0"))
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]
LENGTHS = {"A": {"a": 37, "b": 9, "c": 150, "d": 1, "e": 66, "f": 41, "g": 27},
           "B": {"a": 100, "b": 1, "c": 190, "d": 17, "e": 64},
           "C": {"a": 140, "b": 2, "c": 65, "d": 300, "e": 31, "f": 129, "g": 400},
           "D": {"a": 33, "b": 3, "c": 80, "d": 1, "e": 19}}


def close(got, want, dtype, what="", loose_rows=0.0):
    got, want = got.detach().double().cpu(), want.double()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    if str(dtype).endswith("float32"):
        bad = (got - want).abs() > 2e-4 * (1 + want.abs())
        if bad.any():
            first = int(torch.nonzero(bad.reshape(bad.shape[0], -1).any(dim=1))[0])
            raise AssertionError(f"{what}: first wrong row {first} of {got.shape[0]}, max err {(got - want).abs().max():.3e}")
    else:
        scale = want.pow(2).mean().sqrt()
        rows = (got - want).reshape(got.shape[0], -1).pow(2).mean(dim=1).sqrt() / scale
        over = rows > 0.06
        allowed = int(loose_rows * rows.numel())
        if int(over.sum()) > allowed or rows[~over].mean() > 0.03:
            raise AssertionError(f"{what}: {int(over.sum())} of {rows.numel()} rows beyond 0.06 (first {int(torch.nonzero(over)[0]) if over.any() else -1}, "
                                 f"max {rows.max():.3e}), mean of the others {rows[~over].mean():.3e}")


def torch_dtype(name):
    return torch.float32 if name == "float32" else torch.bfloat16


def runtime(dtype):
    from marin_b200.parts import Runtime
    return Runtime(DEV, torch_dtype(dtype))


def bf(t):
    return t.to(torch.bfloat16)


# ---- the mechanisms alone -------------------------------------------------------------------------------------------

def test_embedding_scale_leaves_a_tied_head_unscaled():
    from marin_b200.parts import lookup

    rt = runtime("float32")
    emb = lookup("embedding", "token_table")(vocab=19, hidden=24, name="e", tensor="e", scale=7.5)
    table = torch.randn(19, 24)
    emb.load({"e": table.clone()}, rt)
    ids = torch.tensor([3, 18, 0, 3], dtype=torch.int32)
    out = torch.empty(4, 24, device=DEV)
    emb.forward(ids.to(DEV), out)
    assert torch.equal(out.cpu(), table[ids.long()] * 7.5)
    assert torch.equal(emb.table.cpu(), table)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("S, h", [(1, 40), (2, 72), (3, 256), (4, 1000), (8, 64)])
def test_stream_steps_alone(dtype, S, h):
    """A write and the next read in one kernel, each alone, the spread of the first stream and the sum of all."""
    from marin_b200.kernels import ops

    g = torch.Generator().manual_seed(S * 100 + h)
    T = 11
    td = torch_dtype(dtype)
    x0 = torch.randn(T, h, generator=g)
    streams = torch.empty(S, T, h, device=DEV)
    streams[0] = x0.to(DEV)
    ops.hc_spread(streams)
    assert all(torch.equal(streams[s].cpu(), x0) for s in range(S))
    streams = (streams + torch.randn(S, T, h, generator=g).to(DEV)).contiguous()
    before = [streams[s].double().cpu() for s in range(S)]
    w_in, w_out, w_mix = torch.randn(S, generator=g), torch.randn(S, generator=g), torch.randn(S, S, generator=g)
    nw = 0.2 * torch.randn(h, generator=g)
    y = torch.randn(T, h, generator=g)
    y_dev = y.to(DEV).contiguous()
    rows = torch.empty(T, h, device=DEV, dtype=td)
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == "float32" else dict(rtol=1e-2, atol=1e-2)
    # read alone
    ops.hc_step(streams, y_dev.clone(), read=(w_in.to(DEV), nw.to(DEV), 1e-5, True, rows))
    u = sum(w_in[s].double() * before[s] for s in range(S))
    torch.testing.assert_close(rows.double().cpu(), plain.rms_norm(u, nw, 1e-5, True), **tol)
    # write and the next read together: y is consumed and left zeroed
    w_in2 = torch.randn(S, generator=g)
    ops.hc_step(streams, y_dev, write=(w_mix.to(DEV), w_out.to(DEV)), read=(w_in2.to(DEV), nw.to(DEV), 1e-5, False, rows))
    after = plain.hyper_step(before, w_in.double(), w_out.double(), w_mix.double(), lambda _: y.double())
    for s in range(S):
        torch.testing.assert_close(streams[s].double().cpu(), after[s], rtol=1e-5, atol=1e-5)
    assert float(y_dev.abs().max()) == 0.0
    u2 = sum(w_in2[s].double() * after[s] for s in range(S))
    torch.testing.assert_close(rows.double().cpu(), plain.rms_norm(u2, nw, 1e-5, False), **tol)
    total = torch.empty(3, h, device=DEV)
    ops.hc_sum(streams, torch.tensor([4, 0, 10], dtype=torch.int32, device=DEV), total)
    torch.testing.assert_close(total.double().cpu(), sum(after)[[4, 0, 10]], rtol=1e-5, atol=1e-5)
    # a row alone gives the same bits as the row among others
    one = streams[:, 5:6].contiguous()
    alone = torch.empty(1, h, device=DEV, dtype=td)
    ops.hc_step(one, None, read=(w_in2.to(DEV), nw.to(DEV), 1e-5, False, alone))
    ops.hc_step(streams, None, read=(w_in2.to(DEV), nw.to(DEV), 1e-5, False, rows))
    assert torch.equal(alone[0], rows[5])


def harness(needs, rt, page=8, pages=80, ctx_len=1024):
    from marin_b200.cache import CacheManager
    from marin_b200.engine import Runner

    cache = CacheManager(list(needs), [None] * len(needs), page, pages, 4)
    cache.allocate(rt.device, rt.dtype)
    return Runner(SimpleNamespace(spec=SimpleNamespace(vocab_size=1 << 30)), cache, rt, ctx_len)


def feed(mixers, runner, x, cuts, req="r"):
    """Runs ``x`` [T, hidden] through the mixers (one after the other on the same input, each with a cache of its own) in
    portions ``cuts``; returns what each added to a zero residual."""
    from marin_b200.engine import StepEntry

    runner.begin(req)
    got, at = [[] for _ in mixers], 0
    for n in cuts:
        runner.cache.reserve(req, at + n)
        ctx = runner.build_context([StepEntry(req, [0] * n, [])])
        for i, mixer in enumerate(mixers):
            residual = torch.zeros(n, x.shape[1], device=DEV)
            mixer.forward(x[at:at + n].to(DEV).contiguous(), ctx, runner.views.view(i, ctx), residual)
            got[i].append(residual.cpu())
        runner.cache.commit(req, at + n)
        at += n
    runner.end(req)
    assert at == x.shape[0]
    return [torch.cat(g) for g in got]


def attention_weights(hidden, m, seed, same_qk=False):
    g = torch.Generator().manual_seed(seed)
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]

    def mat(r, c, gain=1.0):
        return torch.randn(r, c, generator=g) * gain / math.sqrt(c)

    w = {"m.q": mat(H * d, hidden), "m.k": mat(G * d, hidden), "m.v": mat(G * dv, hidden), "m.g": mat(H * dv, hidden, 2.0),
         "m.o": mat(hidden, H * dv), "m.q.b": 0.5 * torch.randn(H * d, generator=g), "m.k.b": 0.5 * torch.randn(G * d, generator=g),
         "m.v.b": 0.3 * torch.randn(G * dv, generator=g), "m.q.norm": 1.5 + 0.3 * torch.randn(H * d, generator=g),
         "m.k.norm": 1.5 + 0.3 * torch.randn(G * d, generator=g), "m.vmix": torch.tensor(0.4)}
    if same_qk:
        assert H == G
        w["m.k"], w["m.k.b"], w["m.k.norm"] = w["m.q"].clone(), w["m.q.b"].clone(), w["m.q.norm"].clone()
    return {k: bf(v) for k, v in w.items()}


def build_mixer(hidden, m, name="m", first=False, sink=True):
    from marin_b200.config.fegarax import FegaraxLayer
    from marin_b200.models.fegarax import MIXER_NAMES, _position
    from marin_b200.parts import lookup

    parsed = FegaraxLayer.parse({"type": "attention", "mixer": m, "mlp": None}, 0).mixer
    return lookup("mixer", "sink_attention")(
        hidden=hidden, heads=m["heads"], kv_heads=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"], scale=m["scale"], bias=True,
        qk_norm="whole", norm_eps=1e-5, position=_position(parsed), chunk=(m.get("mask") or {}).get("size"), sink=sink,
        value_mix="v" if m.get("v_mix") else None, first_of_mix=first, gate=True, names=MIXER_NAMES, name=name)


def plain_mixer(x, w, m, first=True, shared=None, sink=True):
    T = x.shape[0]
    return plain.attention_mixer(x.double(), torch.arange(T), w, "m.", m, 1e-5, shared if shared is not None else {}, first, sink)


CUTS = [[61], [29, 1, 1, 30], [2, 2, 1, 56], [1] * 61, [16, 17, 15, 13]]
YARN = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", [
    {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3, "mask": {"size": 13}, "rot": {"base": 100.0, "dims": 8, "scaling": YARN}},
    {"heads": 3, "kv_heads": 3, "dim": 32, "vdim": 16, "scale": 0.2, "mask": {"size": 1}, "rot": {"base": 100.0, "dims": 32}},
    {"heads": 8, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.125, "mask": {"size": 16}, "rot": {"base": 500.0, "dims": 32, "scaling": YARN}},
    {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 64, "scale": 0.09, "mask": {"size": 50}},
    {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.09, "mask": {"size": 50}, "rot": {"base": 500.0, "dims": 64, "scaling": YARN}},
    {"heads": 2, "kv_heads": 1, "dim": 80, "vdim": 48, "scale": 0.11, "rot": {"base": 100.0, "dims": 80, "scaling": YARN}},
    {"heads": 8, "kv_heads": 1, "dim": 16, "vdim": 128, "scale": 0.25, "mask": {"size": 64}, "rot": {"base": 100.0, "dims": 2}},
    {"heads": 6, "kv_heads": 2, "dim": 8, "vdim": 520, "scale": 0.35, "mask": {"size": 7}},
], ids=lambda m: f"{m['heads']}x{m['kv_heads']}x{m['dim']}x{m['vdim']}")
def test_attention_alone(dtype, m):
    if m["vdim"] > 512:
        rt = runtime(dtype)
        mixer = build_mixer(48, m)
        from marin_b200.kernels.ops import KernelError
        mixer.load(dict(attention_weights(48, m, 1)), rt)
        with pytest.raises(KernelError):
            feed([mixer], harness([mixer.cache_need()], rt), torch.randn(4, 48).to(rt.dtype), [4])
        return
    rt = runtime(dtype)
    hidden = 48
    mixer = build_mixer(hidden, m)
    w = attention_weights(hidden, m, 1)
    mixer.load(dict(w), rt)
    x = torch.randn(61, hidden, generator=torch.Generator().manual_seed(2)).to(rt.dtype)
    want = plain_mixer(x, w, m)
    # heads of 64 or 128 with values as wide and pages of 16: prompt portions go to the kernel plain causal attention uses
    page = 16 if m["dim"] == m["vdim"] and m["dim"] in (64, 128) else 8
    for cuts in CUTS:
        close(feed([mixer], harness([mixer.cache_need()], rt, page=page), x, cuts)[0], want, dtype, f"cuts {cuts[:4]}")
    if page == 16:        # and a longer sequence: several key blocks, chunk edges inside and on block borders
        x = torch.randn(333, hidden, generator=torch.Generator().manual_seed(3)).to(rt.dtype)
        want = plain_mixer(x, w, m)
        for cuts in ([333], [130, 1, 1, 201], [64, 64, 64, 141]):
            close(feed([mixer], harness([mixer.cache_need()], rt, page=page), x, cuts)[0], want, dtype, f"long, cuts {cuts[:4]}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_values_mixed_with_the_first_layers(dtype):
    """Two layers on the same tokens: the second caches (1 - lam) v + lam v_first, in prompts and token by token."""
    rt = runtime(dtype)
    hidden = 40
    m = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 32, "scale": 0.3, "mask": {"size": 20}, "rot": {"base": 100.0, "dims": 16}, "v_mix": True}
    first, second = build_mixer(hidden, m, first=True), build_mixer(hidden, m)
    w1, w2 = attention_weights(hidden, m, 5), attention_weights(hidden, m, 6)
    first.load(dict(w1), rt)
    second.load(dict(w2), rt)
    x = torch.randn(47, hidden, generator=torch.Generator().manual_seed(3)).to(rt.dtype)
    shared = {}
    want1 = plain_mixer(x, w1, m, True, shared)
    want2 = plain_mixer(x, w2, m, False, shared)
    unmixed = plain_mixer(x, w2, dict(m, v_mix=False), False, {})
    assert (want2 - unmixed).abs().max() > 0.05
    for cuts in ([47], [20, 1, 1, 25], [1] * 47, [2] * 23 + [1]):
        got = feed([first, second], harness([first.cache_need(), second.cache_need()], rt), x, cuts)
        close(got[0], want1, dtype, f"first layer, cuts {cuts[:3]}")
        close(got[1], want2, dtype, f"second layer, cuts {cuts[:3]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sink", [True, False])
def test_the_sink_takes_its_share(dtype, sink):
    """Keys that score far below zero leave nearly everything to the sink (the output vanishes); without the sink the same
    keys share the whole weight."""
    rt = runtime(dtype)
    hidden = 32
    m = {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.5}
    mixer = build_mixer(hidden, m, sink=sink)
    w = attention_weights(hidden, m, 7, same_qk=True)
    w["m.k"], w["m.k.b"] = -w["m.q"], -w["m.q.b"]              # k = -q before the norm: every score is strongly negative
    mixer.load(dict(w), rt)
    x = torch.randn(1, hidden, generator=torch.Generator().manual_seed(4)).repeat(9, 1).to(rt.dtype)
    want = plain_mixer(x, w, m, sink=sink)
    other = plain_mixer(x, w, m, sink=not sink)
    assert (want - other).abs().max() > 0.1
    if sink:
        assert want.abs().max() < 1e-3 * other.abs().max()
    for cuts in ([9], [1] * 9, [4, 1, 4]):
        got = feed([mixer], harness([mixer.cache_need()], rt), x, cuts)[0]
        if sink:
            assert got.abs().max() < 2e-3 * other.abs().max()
        else:
            close(got, want, dtype, f"cuts {cuts}")


def standout_case(T, at_query, at_key, chunk, hidden=32, seed=8):
    """A sequence in which the query at ``at_query`` and the key at ``at_key`` come from one strong input row (the key's a
    shorter copy: the norm over the projection gives it the same direction, its value differs) while all other rows are
    weak: with k = q (same matrix, bias and norm) that score stands far above the rest, level with the query's own key."""
    m = {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3}     # (no rotation: it would turn the far key away)
    if chunk:
        m["mask"] = {"size": chunk}
    w = attention_weights(hidden, m, seed, same_qk=True)
    g = torch.Generator().manual_seed(seed + 1)
    x = 0.3 * torch.randn(T, hidden, generator=g)
    strong = 4.0 * torch.randn(hidden, generator=g)
    x[at_query] = strong
    x[at_key] = 0.4 * strong
    return m, w, x


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_far_key_stands_out_among_hundreds(dtype):
    rt = runtime(dtype)
    T = 700
    m, w, x = standout_case(T, T - 1, 5, None)
    x = x.to(rt.dtype)
    mixer = build_mixer(32, m)
    mixer.load(dict(w), rt)
    want = plain_mixer(x, w, m)
    x_without = x.clone()
    x_without[5] = 0.3 * torch.randn(32, generator=torch.Generator().manual_seed(1)).to(rt.dtype)
    assert (plain_mixer(x_without, w, m)[-1] - want[-1]).abs().max() > 0.1 * want[-1].abs().max()     # the far key matters
    for cuts in ([T], [T - 1, 1], [300, 399, 1], [64] * 10 + [59, 1]):
        got = feed([mixer], harness([mixer.cache_need()], rt, page=16, pages=60), x, cuts)[0]
        close(got[-3:], want[-3:], dtype, f"cuts {cuts[:3]}")
        close(got, want, dtype, f"all rows, cuts {cuts[:3]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("chunk", [64, 50, 200])
def test_chunk_edges_in_prompts_and_in_decoding(dtype, chunk):
    """The strong key sits on the first position of the query's chunk (seen) or on the last position of the chunk before
    (not seen); the query is the chunk's first, second or last position or lies in the middle.  Pages of 16 put page
    borders inside and on the chunk's edge."""
    rt = runtime(dtype)
    T = 2 * chunk + 40
    start = 2 * chunk
    for at_query, at_key, seen in ((start + 7, start, True), (start + 7, start - 1, False), (start, start - 1, False),
                                   (start + 1, start, True), (start - 1, start - chunk, True), (start - 1, start - chunk - 1, False)):
        m, w, x = standout_case(T, at_query, at_key, chunk, seed=20 + at_query % 7)
        x = x.to(rt.dtype)
        mixer = build_mixer(32, m)
        mixer.load(dict(w), rt)
        want = plain_mixer(x, w, m)
        x_without = x.clone()
        x_without[at_key] = 0.0
        moved = (plain_mixer(x_without, w, m)[at_query] - want[at_query]).abs().max() > 0.1 * want[at_query].abs().max()
        assert bool(moved) == seen
        for cuts in ([T], [at_query, 1, T - at_query - 1], [at_key, 1] + [1] * (at_query - at_key) + [T - at_query - 1],
                     [start - 3, 2, 2, 2] + [1] * 20 + [T - start - 23]):
            cuts = [c for c in cuts if c > 0]
            got = feed([mixer], harness([mixer.cache_need()], rt, page=16, pages=60), x, cuts)[0]
            close(got[at_query:at_query + 1], want[at_query:at_query + 1], dtype, f"query {at_query} key {at_key} cuts {cuts[:4]}")
            close(got, want, dtype, f"all rows, query {at_query} key {at_key} cuts {cuts[:4]}")


def expert_weights(hidden, ff, E, seed):
    g = torch.Generator().manual_seed(seed)
    w = {"f.router": torch.randn(E, hidden, generator=g) * 3.0 / math.sqrt(hidden)}
    for e in range(E):
        w[f"f.e{e}.gate"] = torch.randn(ff, hidden, generator=g) * 2.0 / math.sqrt(hidden)
        w[f"f.e{e}.up"] = torch.randn(ff, hidden, generator=g) * 2.0 / math.sqrt(hidden)
        w[f"f.e{e}.down"] = torch.randn(hidden, ff, generator=g) * 1.5 / math.sqrt(ff)
    return {k: bf(v) for k, v in w.items()}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden, ff, E, top, T", [(48, 40, 5, 2, 37), (64, 16, 7, 3, 150), (256, 128, 8, 2, 300), (96, 48, 4, 1, 64),
                                                   (32, 24, 3, 3, 9), (128, 64, 16, 1, 1), (256, 64, 6, 2, 700)])
@pytest.mark.parametrize("options", [{}, {"score": "softmax", "renormalize": True, "weight_on": "output"}], ids=["design", "other"])
def test_routed_experts_alone(dtype, hidden, ff, E, top, T, options):
    """Rows whose choice of experts is a close call in float64 (a router margin under 0.1) are left out: the rest must match
    row by row, alone and in any batch."""
    from marin_b200.models.fegarax import EXPERT_NAMES
    from marin_b200.parts import lookup

    rt = runtime(dtype)
    part = lookup("feedforward", "routed_experts")(hidden=hidden, intermediate=ff, experts=E, top=top, name="f", names=EXPERT_NAMES, **options)
    w = expert_weights(hidden, ff, E, hidden + E)
    part.load(dict(w), rt)
    mlp = {"router": {"experts": E, "top": top}}
    x = torch.randn(4 * T, hidden, generator=torch.Generator().manual_seed(9)).to(rt.dtype)
    x = x[plain.router_margins(x.double(), w, "f.", mlp) > 0.1][:T].contiguous()
    assert x.shape[0] >= min(T, 1)
    want = plain.routed_experts(x.double(), w, "f.", mlp, **options)
    ctx = SimpleNamespace(workspace=__import__("marin_b200.engine.context", fromlist=["Workspace"]).Workspace(DEV))
    y = torch.zeros(x.shape[0], hidden, device=DEV)
    part.forward(x.to(DEV), ctx, y)
    close(y, want, dtype, "all rows at once")
    for lo, hi in ((0, 1), (x.shape[0] // 2, min(x.shape[0], x.shape[0] // 2 + 3))):
        part_y = torch.ones(hi - lo, hidden, device=DEV)            # it adds into what is there
        part.forward(x[lo:hi].contiguous().to(DEV), ctx, part_y)
        close(part_y - 1.0, want[lo:hi], dtype, f"rows {lo}:{hi} alone")
        if dtype == "float32":
            again = torch.zeros(hi - lo, hidden, device=DEV)
            part.forward(x[lo:hi].contiguous().to(DEV), ctx, again)
            assert torch.equal(again, y[lo:hi])


# ---- whole models -----------------------------------------------------------------------------------------------------

class Case:
    def __init__(self, tmp, name, dtype):
        from marin_b200.engine import load_model

        self.name, self.dtype = name, dtype
        self.raw = CONFIGS[name]
        self.dir = make_model_dir(str(tmp / f"{name}-{dtype}"), name, seed=11)
        self.w = plain.read_weights(self.dir)
        rng = random.Random(5)
        self.tokens = {rid: random_prompt(rng, self.raw["vocab"], n) for rid, n in LENGTHS[name].items()}
        self.want = {rid: plain.forward(self.raw, self.w, t)[0] for rid, t in self.tokens.items()}
        self.rt = runtime(dtype)
        self.config, self.model = load_model(self.dir, self.rt)
        self.page = PAGE[name]
        self.loose = 0.0 if dtype == "float32" else 0.04

    def runner(self, num_pages, max_requests=4, graphs=False):
        from marin_b200.cache import CacheManager
        from marin_b200.engine import Runner

        cache = CacheManager(self.model.cache_needs(), [e.cache_of for e in self.model.spec.schedule], self.page, num_pages, max_requests)
        cache.allocate(self.rt.device, self.rt.dtype)
        runner = Runner(self.model, cache, self.rt, 512)
        if graphs:
            runner.enable_graphs((1, 2, 4))
        return runner

    def close(self, got, rid, what):
        close(got, self.want[rid], self.dtype, what, self.loose)


@pytest.fixture(scope="module", params=[(n, d) for n in CONFIGS for d in DTYPES], ids=lambda p: f"{p[0]}-{p[1]}")
def case(request, tmp_path_factory):
    return Case(tmp_path_factory.mktemp("fegarax"), *request.param)


def test_the_residual_stream_after_every_layer(case):
    from marin_b200.engine import StepEntry

    rid = "a"
    _, want = plain.forward(case.raw, case.w, case.tokens[rid])
    got = {}
    runner = case.runner(64)
    runner.begin(rid)
    runner.step([StepEntry(rid, case.tokens[rid], [0])], observe=lambda i, h: got.__setitem__(i, h.clone()))
    assert len(got) == want.shape[0] + 1
    for i in range(want.shape[0]):
        close(got[i + 1], want[i], case.dtype, f"after layer {i}", case.loose)


def test_whole_prompts_and_the_first_tokens(case):
    runner = case.runner(64)
    for rid, tokens in case.tokens.items():
        case.close(run_whole(runner, rid, tokens), rid, f"{rid} whole")
    runner.cache.check()


@pytest.mark.parametrize("graphs", [False, True])
def test_prefill_then_token_by_token(case, graphs):
    """Most of a prompt in one step and the rest one token at a time, eagerly and from captured graphs: a tail long enough
    to pass over several chunk edges; and a request decoded from its very first token."""
    runner = case.runner(64, graphs=graphs)
    for rid, tail in (("c", 70), ("a", 30), ("e", 5)):
        tokens = case.tokens[rid]
        n = max(len(tokens) - tail, 0)
        sizes = ([n] if n > 0 else []) + [1] * (len(tokens) - n)
        case.close(run_portions(runner, rid + "t", tokens, sizes), rid, f"{rid}, last {tail} one by one")
    rid = "e"
    case.close(run_portions(runner, rid + "1", case.tokens[rid], [1] * len(case.tokens[rid])), rid, f"{rid} token by token")
    runner.cache.check()


def test_portions_of_changing_size_down_to_two_tokens(case):
    runner = case.runner(64)
    for rid in ("c", "a"):
        tokens = case.tokens[rid]
        for sizes in ([7, 2, 13, 3, 2, 5], [2], [case.page, case.page + 1, case.page - 1] if case.page > 1 else [3], [64, 1, 2]):
            sizes = [s for s in sizes if s > 0]
            case.close(run_portions(runner, rid + "p", tokens, portions(len(tokens), sizes)), rid, f"{rid} in {sizes}")


@pytest.mark.parametrize("graphs", [False, True])
def test_mixed_batches_reuse_pages(case, graphs):
    """Up to four live requests, portions of some beside single tokens of others, in a pool that holds the four largest
    only: pages of finished requests are handed to the next ones."""
    rng = random.Random(9)
    lengths = {rid: len(t) for rid, t in case.tokens.items()}
    sched = mixed_schedule(rng, lengths, max_live=4, decode_tail=6)
    pool = sum(sorted((-(-n // case.page) for n in lengths.values()), reverse=True)[:4])
    runner = case.runner(pool, max_requests=4, graphs=graphs)
    got = run_mixed(runner, case.tokens, sched)
    for rid in case.tokens:
        case.close(got[rid], rid, f"{rid} mixed")
    runner.cache.check()
    assert all(g.pool.num_held == 0 for g in runner.cache.groups)
    again = run_mixed(runner, case.tokens, sched)
    for rid in case.tokens:
        case.close(again[rid], rid, f"{rid} mixed, second time")


def test_a_batch_gives_each_request_what_it_gets_alone(case):
    """float32: the logits of a request are the same bits whatever else the step holds and however its prompt was cut."""
    if case.dtype != "float32":
        pytest.skip("bit equality is the 32-bit path's claim")
    from marin_b200.engine import StepEntry

    runner = case.runner(64)
    alone = {rid: run_whole(runner, rid, case.tokens[rid]) for rid in ("a", "b", "e")}
    for rid in alone:
        runner.begin(rid)
    logits = runner.step([StepEntry(rid, case.tokens[rid], list(range(len(case.tokens[rid])))) for rid in ("a", "b", "e")])
    k = 0
    for rid in ("a", "b", "e"):
        n = len(case.tokens[rid])
        assert torch.equal(logits[k:k + n], alone[rid]), rid
        k += n
        runner.end(rid)
    cut = run_portions(runner, "ap", case.tokens["a"], portions(len(case.tokens["a"]), [5, 2, 9, 1]))
    assert torch.equal(cut, alone["a"])


def test_greedy_generation_through_the_engine(case):
    """The entry point, the scheduler and device sampling: the tokens are those the plain implementation's logits rank
    first (a token whose plain logit lies within 1e-3 (32-bit) or 0.15 (16-bit) of the largest counts as first).  In
    16-bit a request stops being compared at a step whose choice of experts was a close call."""
    from marin_b200.engine import Engine
    from marin_b200.sampling.sampler import SamplingParams

    engine = Engine(case.dir, dtype=case.dtype, ctx=256, page_size=case.page, num_pages=64, max_batch=4, token_budget=32)
    prompts = [case.tokens["a"][:21], case.tokens["e"][:3], case.tokens["c"][:40]]
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10))
    slack = 1e-3 if case.dtype == "float32" else 0.15
    for prompt, out in zip(prompts, outs):
        assert len(out.tokens) == 10
        seq = list(prompt)
        for token in out.tokens:
            margins = []
            logits = plain.forward(case.raw, case.w, seq, margins)[0][-1]
            if case.dtype != "float32" and margins and min(float(mm.min()) for mm in margins) < 0.1:
                break
            assert logits[token] >= logits.max() - slack, (len(seq), token, int(logits.argmax()))
            seq.append(token)


def test_trace_replay_as_a_user_runs_it(tmp_path):
    """bin/trace_run in a process of its own: steps on standard input, logits read back from files."""
    name, dtype = "A", "float32"
    raw = CONFIGS[name]
    d = make_model_dir(str(tmp_path / "model"), name, seed=12)
    w = plain.read_weights(d)
    rng = random.Random(3)
    lengths = {"a": 70, "b": 130, "c": 41, "d": 64, "e": 100, "f": 2}
    tokens = {rid: random_prompt(rng, raw["vocab"], n) for rid, n in lengths.items()}
    want = {rid: plain.forward(raw, w, t)[0] for rid, t in tokens.items()}
    sched = mixed_schedule(rng, lengths, max_live=4, decode_tail=5)
    pool = sum(sorted((-(-n // 64) * 64 for n in lengths.values()), reverse=True)[:4])
    out = str(tmp_path / "out")
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", out,
                             "--max-tokens", str(pool)], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    fed = {rid: 0 for rid in tokens}
    for i, (entries, ends) in enumerate(sched):
        line, rows = [], []
        for rid, n in entries:
            wanted = [n - 1] if n > 2 else list(range(n))
            line.append({"id": rid, "tokens": tokens[rid][fed[rid]:fed[rid] + n], "want": wanted})
            rows.append(want[rid][[fed[rid] + k for k in wanted]])
            fed[rid] += n
        proc.stdin.write(json.dumps({"step": i, "entries": line, "end": ends}) + "\n")
        proc.stdin.flush()
        assert proc.stdout.readline().strip() == f"done {i}"
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(-1, raw["vocab"]).copy())
        close(got, torch.cat(rows), dtype, f"step {i}")
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0


def test_the_command_line_takes_a_fegarax_folder(tmp_path):
    """Random-weights mode from a config.json of this design, greedy generation, and the bench command with its stage table."""
    run = [sys.executable, os.path.join(ROOT, "bin", "marin-run")]
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(CONFIGS["C"]))
    model = str(tmp_path / "model")
    out = subprocess.run(run + ["random", "--config", str(cfg), "--seed", "3", "--out", model], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert sorted(os.listdir(model)) == ["config.json", "model.safetensors"]
    a = subprocess.run(run + [model, "--prompt-ids", "5,6,7,8,9", "--temp", "0", "--max-tokens", "6"], capture_output=True, text=True)
    b = subprocess.run(run + [model, "--prompt-ids", "5 6 7 8 9", "--temp", "0", "--max-tokens", "6"], capture_output=True, text=True)
    assert a.returncode == 0 and b.returncode == 0, a.stderr + b.stderr
    assert a.stdout == b.stdout and len(a.stdout.split()) == 6
    e = subprocess.run(run + ["bench", model, "--prompt-tokens", "16", "--tokens", "8", "--runs", "2", "--warmup", "1", "--profile"],
                       capture_output=True, text=True)
    assert e.returncode == 0, e.stderr
    for stage in ("embedding", "streams, norm", "q|k|v|g", "heads", "attention", "router", "experts", "head", "sampling"):
        assert stage in e.stdout, stage
