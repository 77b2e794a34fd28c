"""Lakulix on the GPU against the plain implementation (``plain_lakulix``, float64 on the CPU): every mechanism alone,
then whole models under every way of cutting the work: each request alone and whole; most of it in one step and the
rest one token at a time (eagerly and from captured graphs); portions of changing size down to two tokens; mixed
batches of unequal requests with so few pages and slots that both are used again; greedy generation through the
engine's entry point and scheduler; and the trace replay as a user runs it.

Tolerances.  float32: |diff| <= 2e-4 (1 + |ref|) on logits, the plain result being float64.  bfloat16: the root mean
square of the difference over a position's logits at most 0.06 of the logits' own root mean square, at every position,
and at most 0.03 on average.
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

import plain_lakulix as plain
from helpers import mixed_schedule, portions, random_prompt, run_mixed, run_portions, run_whole
from lakulix_models import CONFIGS, PAGE, make_model_dir

pytestmark = pytest.mark.gpu
DEV = torch.device(os.environ.get("MARIN_B200_TEST_DEVICE", "cuda:0"))
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]
LENGTHS = {"A": {"a": 37, "b": 9, "c": 150, "d": 1, "e": 64, "f": 41, "g": 33},
           "B": {"a": 100, "b": 1, "c": 190, "d": 17, "e": 64, "f": 129, "g": 48},
           "C": {"a": 140, "b": 2, "c": 65, "d": 300, "e": 31}}


def close(got, want, dtype, what=""):
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
        if rows.max() > 0.06 or rows.mean() > 0.03:
            raise AssertionError(f"{what}: relative error max {rows.max():.3e} (row {int(rows.argmax())}) mean {rows.mean():.3e}")


def torch_dtype(name):
    return torch.float32 if name == "float32" else torch.bfloat16


def runtime(dtype):
    from marin_b200.parts import Runtime
    return Runtime(DEV, torch_dtype(dtype))


def rounded(t, dtype):
    """What the engine of this dtype holds of a tensor handed to it."""
    return t.to(torch_dtype(dtype)).double()


# ---- the mechanisms alone -------------------------------------------------------------------------------------------

def test_embedding_with_a_learned_position_table():
    from marin_b200.parts import lookup

    rt = runtime("float32")
    emb = lookup("embedding", "token_table")(vocab=19, hidden=24, name="e", tensor="e", positions=40, position_tensor="p")
    assert [(s.name, s.shape) for s in emb.tensor_specs()] == [("e", (19, 24)), ("p", (40, 24))]
    table, pos = torch.randn(19, 24), torch.randn(40, 24)
    emb.load({"e": table.clone(), "p": pos.clone()}, rt)
    ids = torch.tensor([3, 18, 0, 3, 7], dtype=torch.int32)
    where = torch.tensor([0, 1, 39, 5, 0], dtype=torch.int32)      # positions restart with every sequence of a batch
    out = torch.empty(5, 24, device=DEV)
    emb.forward(ids.to(DEV), out, where.to(DEV))
    assert torch.equal(out.cpu(), table[ids.long()] + pos[where.long()])
    for i, p in ((0, 0), (2, 39)):
        assert torch.equal(out[i].cpu(), plain.embed([int(ids[i])], table, pos, first_position=p)[0])


@pytest.mark.parametrize("dtype", DTYPES)
def test_dynamic_tanh_norm(dtype):
    from marin_b200.parts import lookup

    rt = runtime(dtype)
    norm = lookup("norm", "dynamic_tanh")(dim=72, name="n", names=("", "b", "alpha"))
    assert [(s.name, s.shape) for s in norm.tensor_specs()] == [("n", (72,)), ("n.b", (72,)), ("n.alpha", ())]
    w, b, alpha = 1 + 0.2 * torch.randn(72), 0.3 * torch.randn(72), torch.tensor(0.7)
    norm.load({"n": w.clone(), "n.b": b.clone(), "n.alpha": alpha.clone()}, rt)
    x = 3 * torch.randn(9, 72)
    out = torch.empty(9, 72, device=DEV, dtype=rt.dtype)
    norm.forward(x.to(DEV), out)
    want = plain.dynamic_tanh(x.double(), alpha.double(), w.double(), b.double())
    tol = dict(rtol=1e-5, atol=1e-6) if dtype == "float32" else dict(rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(out.double().cpu(), want, **tol)
    # no statistic of the row enters: a row alone gives the same bits as the row among others
    alone = torch.empty(1, 72, device=DEV, dtype=rt.dtype)
    norm.forward(x[4:5].to(DEV), alone)
    assert torch.equal(alone[0], out[4])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [48, 1000])
def test_polynorm_and_the_gated_norm(dtype, n):
    from marin_b200.kernels import ops

    td = torch_dtype(dtype)
    z = 1.5 * torch.randn(7, n)
    coef = torch.tensor([0.8, -0.5, 0.3, 0.1])
    out = torch.empty(7, n, device=DEV, dtype=td)
    ops.polynorm(z.to(DEV), coef.to(DEV), 1e-5, out)
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == "float32" else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out.double().cpu(), plain.polynorm(z.double(), coef.double(), 1e-5), **tol)
    # the gated norm over whole rows, the gate a column slice of a wider matrix
    o, w = torch.randn(7, n), 1 + 0.1 * torch.randn(n)
    wide = torch.randn(7, 2 * n + 8).to(td)
    for gate, fn in (("sigmoid", plain.sigmoid), ("silu", plain.silu)):
        ops.gated_rmsnorm(o.to(DEV), w.to(DEV), wide.to(DEV)[:, n + 8:], gate, 1e-5, out)
        want = plain.unit_rms(o.double(), 1e-5) * w.double() * fn(wide[:, n + 8:].double())
        torch.testing.assert_close(out.double().cpu(), want, **tol)
    logits = 30 * torch.randn(5, 33)
    dev = logits.to(DEV)
    ops.tanh_cap(dev, 12.0)
    torch.testing.assert_close(dev.cpu().double(), 12.0 * torch.tanh(logits.double() / 12.0), rtol=1e-5, atol=1e-5)


def harness(mixer, rt, page=8, pages=40, ctx_len=512):
    from marin_b200.cache import CacheManager
    from marin_b200.engine import Runner

    cache = CacheManager([mixer.cache_need()], [None], page, pages, 4)
    cache.allocate(rt.device, rt.dtype)
    return Runner(SimpleNamespace(spec=SimpleNamespace(vocab_size=1 << 30)), cache, rt, ctx_len)


def feed(mixer, runner, x, cuts, req="r"):
    """Runs ``x`` [T, hidden] through the mixer alone in portions ``cuts``; returns what it added to a zero residual."""
    from marin_b200.engine import StepEntry

    runner.begin(req)
    got, at = [], 0
    for n in cuts:
        runner.cache.reserve(req, at + n)
        ctx = runner.build_context([StepEntry(req, [0] * n, [])])
        residual = torch.zeros(n, x.shape[1], device=DEV)
        mixer.forward(x[at:at + n].to(DEV).contiguous(), ctx, runner.views.view(0, ctx), residual)
        runner.cache.commit(req, at + n)
        got.append(residual.cpu())
        at += n
    runner.end(req)
    assert at == x.shape[0]
    return torch.cat(got)


def mixer_weights(mixer, dtype, seed, std=None):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for s in mixer.tensor_specs():
        if s.role == "norm":
            t = 1 + 0.1 * torch.randn(s.shape, generator=g)
        elif s.role == "bias":
            t = torch.rand(s.shape, generator=g) if ".mu." in s.name else torch.randn(s.shape, generator=g)
        else:
            t = torch.randn(s.shape, generator=g) / math.sqrt(s.shape[-1])
        out[s.name] = t.to(torch.bfloat16)
    return out


CUTS = [[29], [13, 1, 1, 14], [2, 2, 1, 24], [1] * 29]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, dim, vdim", [(3, 8, 16), (2, 40, 72), (1, 64, 128), (2, 16, 16), (1, 128, 64), (2, 32, 32), (1, 96, 32)])
def test_linear_attention_alone(dtype, heads, dim, vdim):
    from marin_b200.parts import lookup

    rt = runtime(dtype)
    hidden = 48
    decay = [0.5, 0.95, 0.999][:heads]
    mixer = lookup("mixer", "linear_attention")(hidden=hidden, heads=heads, dim=dim, vdim=vdim, decay=decay, name="m", norm_eps=1e-5)
    w = mixer_weights(mixer, dtype, 1)
    mixer.load(dict(w), rt)
    x = torch.randn(29, hidden).to(rt.dtype)
    want = plain.lightning(x.double(), {k: v.double() for k, v in w.items()}, "m", heads, dim, vdim, decay, 1e-5)
    for cuts in CUTS:
        close(feed(mixer, harness(mixer, rt), x, cuts), want, dtype, f"cuts {cuts[:4]}")


@pytest.mark.parametrize("heads, dim, vdim", [(2, 32, 64), (1, 128, 128), (2, 16, 32), (1, 64, 96)])
def test_linear_attention_in_chunks_of_64(heads, dim, vdim):
    """Prompt portions long enough for several chunks of the tensor-core kernel, cut at, just before and just after chunk
    edges, with single tokens (the scan kernel) in between: both kernels carry the same state.  A slow decay keeps the
    first tokens visible to the last."""
    from marin_b200.kernels import ops
    from marin_b200.parts import lookup

    dtype = "bfloat16"
    rt = runtime(dtype)
    hidden, T = 48, 200
    decay = [0.999, 0.9][:heads]
    assert ops.linear_attention_chunked_supported(rt.dtype, dim, vdim)
    mixer = lookup("mixer", "linear_attention")(hidden=hidden, heads=heads, dim=dim, vdim=vdim, decay=decay, name="m", norm_eps=1e-5)
    w = mixer_weights(mixer, dtype, 9)
    mixer.load(dict(w), rt)
    x = torch.randn(T, hidden, generator=torch.Generator().manual_seed(10)).to(rt.dtype)
    want = plain.lightning(x.double(), {k: v.double() for k, v in w.items()}, "m", heads, dim, vdim, decay, 1e-5)
    for cuts in ([200], [64, 64, 72], [63, 1, 65, 1, 70], [2, 128, 1, 1, 68], [129, 71]):
        close(feed(mixer, harness(mixer, rt), x, cuts), want, dtype, f"cuts {cuts}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, dim, rank", [(2, 16, 8), (3, 24, 12), (1, 64, 16), (1, 128, 16), (2, 32, 8), (1, 80, 8)])
def test_wkv_alone(dtype, heads, dim, rank):
    from marin_b200.parts import lookup

    rt = runtime(dtype)
    hidden = 56
    mixer = lookup("mixer", "wkv")(hidden=hidden, heads=heads, dim=dim, decay_rank=rank, name="m", norm_eps=1e-5)
    w = mixer_weights(mixer, dtype, 2)
    w["m.w0"] = (torch.rand(heads * dim) * 4.5 - 4.0).to(torch.bfloat16)
    mixer.load(dict(w), rt)
    x = torch.randn(29, hidden).to(rt.dtype)
    want = plain.wkv(x.double(), {k: v.double() for k, v in w.items()}, "m", heads, dim, 1e-5)
    for cuts in CUTS:
        close(feed(mixer, harness(mixer, rt), x, cuts), want, dtype, f"cuts {cuts[:4]}")


@pytest.mark.parametrize("heads, dim", [(2, 64), (1, 128), (2, 32), (3, 16)])
def test_wkv_long_portions_in_blocks_side_by_side(heads, dim):
    """Portions long enough to be cut into blocks that are walked side by side (bfloat16), cut at and around block edges,
    with single tokens and short portions (one walk) in between: all of them carry the same state and the same last row."""
    from marin_b200.kernels import ops
    from marin_b200.parts import lookup

    dtype = "bfloat16"
    rt = runtime(dtype)
    hidden, T = 40, 700
    mixer = lookup("mixer", "wkv")(hidden=hidden, heads=heads, dim=dim, decay_rank=8, name="m", norm_eps=1e-5)
    w = mixer_weights(mixer, dtype, 12)
    w["m.w0"] = (torch.rand(heads * dim, generator=torch.Generator().manual_seed(13)) * 5.0 - 4.5).to(torch.bfloat16)
    mixer.load(dict(w), rt)
    x = torch.randn(T, hidden, generator=torch.Generator().manual_seed(14)).to(rt.dtype)
    want = plain.wkv(x.double(), {k: v.double() for k, v in w.items()}, "m", heads, dim, 1e-5)
    assert ops.WKV_BLOCKS_FROM <= 256 and ops.WKV_BLOCK_TOKENS == 128
    for cuts in ([700], [256, 444], [257, 1, 1, 441], [300, 100, 300], [383, 317]):
        close(feed(mixer, harness(mixer, rt, ctx_len=1024), x, cuts), want, dtype, f"cuts {cuts}")


def attention_mixer(hidden, H, K, d, dv, rows, farthest, coef=0.3, every=5, scale=0.25):
    from marin_b200.parts import lookup

    return lookup("mixer", "sigmoid_attention")(
        hidden=hidden, heads=H, kv_heads=K, head_dim=d, v_head_dim=dv, name="m", scale=scale, norm_eps=1e-5, temp_coef=coef,
        temp_every=every, bias_rows=rows, bias_max=farthest,
        names={"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "rel": "rel", "pb": "pb"})


def plain_attention(x, w, H, K, d, dv, rows, farthest, coef=0.3, every=5, scale=0.25, slow=False):
    fn = plain.sigmoid_attention if slow else plain.sigmoid_attention_fast
    return fn(x.double(), {k: v.double() for k, v in w.items()}, "m", H, K, d, dv, scale, farthest, coef, every, 1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H, K, d, dv, rows, farthest", [(4, 2, 16, 24, 10, 14), (2, 2, 32, 16, 7, 9.5), (8, 2, 64, 64, 12, 20),
                                                         (6, 2, 32, 48, 12, 40), (8, 1, 16, 128, 2, 5)])
def test_sigmoid_attention_alone(dtype, H, K, d, dv, rows, farthest):
    rt = runtime(dtype)
    hidden = 40
    mixer = attention_mixer(hidden, H, K, d, dv, rows, farthest)
    w = mixer_weights(mixer, dtype, 3)
    mixer.load(dict(w), rt)
    x = torch.randn(29, hidden).to(rt.dtype)
    want = plain_attention(x, w, H, K, d, dv, rows, farthest)
    torch.testing.assert_close(want, plain_attention(x, w, H, K, d, dv, rows, farthest, slow=True), rtol=1e-9, atol=1e-9)
    for cuts in CUTS:
        close(feed(mixer, harness(mixer, rt), x, cuts), want, dtype, f"cuts {cuts[:4]}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_far_key_stands_out_among_hundreds(dtype):
    """Every weight is made tiny by the heads' offset except where one query meets one key far back, whose score is large:
    the output there is that key's value.  The pair is placed across pages, in a prompt portion and for a decoded token."""
    rt = runtime(dtype)
    hidden, H, K, d, dv, T = 48, 2, 1, 32, 16, 300
    mixer = attention_mixer(hidden, H, K, d, dv, rows=8, farthest=50, coef=0.0, every=1, scale=0.25)
    w = mixer_weights(mixer, dtype, 4)
    eye = torch.zeros(d, hidden)
    eye[:, :d] = torch.eye(d)
    w["m.q"], w["m.k"] = torch.cat([eye, eye]).to(torch.bfloat16), eye.to(torch.bfloat16)      # q = k = the first d inputs
    w["m.q.norm"] = w["m.k.norm"] = torch.full((d,), 2.0).to(torch.bfloat16)                  # normed heads of elements +-2
    w["m.rel"] = torch.zeros(8, H).to(torch.bfloat16)
    w["m.pb"] = torch.full((H,), -26.0).to(torch.bfloat16)
    mixer.load(dict(w), rt)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, hidden, generator=g)
    # keys are random sign vectors: q.k scale = d = 32 for a key equal to the query (score +6), 20 or less otherwise (-6 or less)
    x[:, :d] = torch.randn(T, d, generator=g).sign()
    asks = {260: 17, 299: 40}                                  # query row -> the far key it equals: one in a prompt portion, one decoded
    for row, key in asks.items():
        x[row, :d] = x[key, :d]
    x = x.to(rt.dtype)
    want = plain_attention(x, w, H, K, d, dv, 8, 50, coef=0.0, every=1, scale=0.25)
    v = plain.linear(x.double(), w["m.v"].double())

    def through_o(row):                                        # both heads share the one kv head
        return plain.linear(torch.cat([v[row], v[row]])[None], w["m.o"].double())[0]

    for row, key in asks.items():                              # the far key and the query's own dominate the plain result too
        assert (want[row] - through_o(key) - through_o(row)).abs().max() < 0.05 * through_o(key).abs().max()
    got = feed(mixer, harness(mixer, rt, page=16, pages=24), x, [256, 43, 1])
    close(got, want, dtype, "far key")
    for row, key in asks.items():
        assert (got[row].double() - through_o(key) - through_o(row)).abs().max() < 0.1 * through_o(key).abs().max()


@pytest.mark.parametrize("dtype", DTYPES)
def test_distance_table_edges_in_prompts_and_in_decoding(dtype):
    """The table lets exactly one row through (+12 against -12 elsewhere), so a query sees only the keys whose distance falls
    into that row: a bucket edge that is one off, or a table that does not saturate, changes which values are summed."""
    rt = runtime(dtype)
    hidden, H, K, d, dv, T, rows, farthest = 24, 2, 2, 8, 8, 90, 10, 30
    for open_row in (3, 5, 7, 9):
        mixer = attention_mixer(hidden, H, K, d, dv, rows, farthest, coef=0.0, every=1, scale=0.01)
        w = mixer_weights(mixer, dtype, 6)
        rel = torch.full((rows, H), -12.0)
        rel[open_row] = 12.0
        w["m.rel"], w["m.pb"] = rel.to(torch.bfloat16), torch.zeros(H).to(torch.bfloat16)
        mixer.load(dict(w), rt)
        x = torch.randn(T, hidden, generator=torch.Generator().manual_seed(7)).to(rt.dtype)
        want = plain_attention(x, w, H, K, d, dv, rows, farthest, coef=0.0, every=1, scale=0.01)
        # what the open row lets through, written out: the sum of the values at the distances of that row
        v = plain.linear(x.double(), w["m.v"].double()).view(T, K, dv)
        dist = [n for n in range(T) if plain.distance_bucket(n, rows, farthest) == open_row]
        i = T - 1
        seen = sum(v[i - n] for n in dist if i - n >= 0).reshape(-1)
        assert (plain.linear(seen[None], w["m.o"].double())[0] - want[i]).abs().max() < 2e-3 * len(dist)
        for cuts in ([T], [61, 1, 1, 2, 25], [40] + [1] * 50):
            close(feed(mixer, harness(mixer, rt, page=8), x, cuts), want, dtype, f"row {open_row}, cuts {cuts[:3]}")


def test_query_temperature_follows_the_position():
    """The factor on the queries changes every ``every`` positions, also for tokens that arrive one at a time."""
    rt = runtime("float32")
    hidden, H, K, d, dv, T = 24, 2, 1, 8, 8, 40
    mixer = attention_mixer(hidden, H, K, d, dv, 6, 12, coef=0.9, every=4, scale=0.5)
    w = mixer_weights(mixer, "float32", 8)
    mixer.load(dict(w), rt)
    x = torch.randn(T, hidden)
    want = plain_attention(x, w, H, K, d, dv, 6, 12, coef=0.9, every=4, scale=0.5)
    flat = plain_attention(x, w, H, K, d, dv, 6, 12, coef=0.0, every=4, scale=0.5)
    assert (want[:2] - flat[:2]).abs().max() < 1e-12 and (want[3:] - flat[3:]).abs().max() > 1e-3     # floor((p + 1) / 4) = 0 up to p = 2
    for cuts in ([T], [3, 1, 1, 35], [1] * T):
        close(feed(mixer, harness(mixer, rt), x, cuts), want, "float32", f"cuts {cuts[:3]}")


# ---- whole models -----------------------------------------------------------------------------------------------------

class Case:
    def __init__(self, tmp, name, dtype):
        from marin_b200.engine import load_model

        self.name, self.dtype = name, dtype
        self.raw = CONFIGS[name][0]
        self.dir = make_model_dir(str(tmp / f"{name}-{dtype}"), name, seed=11)
        self.w = plain.read_weights(self.dir)
        rng = random.Random(5)
        self.tokens = {rid: random_prompt(rng, self.raw["vocab"], n) for rid, n in LENGTHS[name].items()}
        self.want = {rid: plain.forward(self.raw, self.w, t) for rid, t in self.tokens.items()}
        self.rt = runtime(dtype)
        self.config, self.model = load_model(self.dir, self.rt)
        self.page = PAGE[name]

    def runner(self, num_pages, max_requests=4, graphs=False):
        from marin_b200.cache import CacheManager
        from marin_b200.engine import Runner

        cache = CacheManager(self.model.cache_needs(), [e.cache_of for e in self.model.spec.schedule], self.page, num_pages, max_requests)
        cache.allocate(self.rt.device, self.rt.dtype)
        runner = Runner(self.model, cache, self.rt, self.raw["max_positions"])
        if graphs:
            runner.enable_graphs((1, 2, 4))
        return runner


@pytest.fixture(scope="module", params=[(n, d) for n in CONFIGS for d in DTYPES], ids=lambda p: f"{p[0]}-{p[1]}")
def case(request, tmp_path_factory):
    return Case(tmp_path_factory.mktemp("lakulix"), *request.param)


def test_the_residual_stream_after_every_layer_run(case):
    from marin_b200.engine import StepEntry

    rid = "a"
    want = []
    plain.forward(case.raw, case.w, case.tokens[rid], observe=lambda run, x: want.append(x.clone()))
    got = {}
    runner = case.runner(64)
    runner.begin(rid)
    runner.step([StepEntry(rid, case.tokens[rid], [0])], observe=lambda i, h: got.__setitem__(i, h.clone()))
    assert len(want) == len(plain.layer_runs(case.raw)) == len(got) - 1
    for run, x in enumerate(want):
        close(got[run + 1], x, case.dtype, f"after layer run {run}")


def test_whole_prompts_and_the_first_tokens(case):
    runner = case.runner(64)
    for rid, tokens in case.tokens.items():
        close(run_whole(runner, rid, tokens), case.want[rid], case.dtype, f"{rid} whole")
    runner.cache.check()


@pytest.mark.parametrize("graphs", [False, True])
def test_prefill_then_token_by_token(case, graphs):
    """Most of a prompt in one step and the rest one token at a time, eagerly and from captured graphs; a long tail, so
    that the recurrent states are carried through many single steps; and a request decoded from its very first token."""
    from marin_b200.engine import StepEntry

    runner = case.runner(64, graphs=graphs)
    for rid, tail in (("c", 40), ("a", 36), ("e", 5)):
        tokens = case.tokens[rid]
        n = len(tokens) - tail
        sizes = ([n] if n > 0 else []) + [1] * min(tail, len(tokens))
        close(run_portions(runner, rid + "t", tokens, sizes), case.want[rid], case.dtype, f"{rid}, last {tail} one by one")
    rid = "g" if "g" in case.tokens else "e"
    close(run_portions(runner, rid + "1", case.tokens[rid], [1] * len(case.tokens[rid])), case.want[rid], case.dtype, f"{rid} token by token")
    runner.cache.check()


def test_portions_of_changing_size_down_to_two_tokens(case):
    runner = case.runner(64)
    for rid in ("c", "a"):
        tokens = case.tokens[rid]
        for sizes in ([7, 2, 13, 3, 2, 5], [2], [case.page, case.page + 1, case.page - 1], [64, 1, 2]):
            close(run_portions(runner, rid + "p", tokens, portions(len(tokens), sizes)), case.want[rid], case.dtype, f"{rid} in {sizes}")


@pytest.mark.parametrize("graphs", [False, True])
def test_mixed_batches_reuse_pages_and_slots(case, graphs):
    """Up to four live requests, portions of some beside single tokens of others, in a pool that holds the four largest
    only: pages and state slots of finished requests are handed to the next ones, and a slot's old state must not leak."""
    rng = random.Random(9)
    lengths = {rid: len(t) for rid, t in case.tokens.items()}
    sched = mixed_schedule(rng, lengths, max_live=4, decode_tail=6)
    pool = sum(sorted((-(-n // case.page) for n in lengths.values()), reverse=True)[:4])
    runner = case.runner(pool, max_requests=4, graphs=graphs)
    got = run_mixed(runner, case.tokens, sched)
    for rid in case.tokens:
        close(got[rid], case.want[rid], case.dtype, f"{rid} mixed")
    runner.cache.check()
    assert runner.cache.slots.num_held == 0 and all(g.pool.num_held == 0 for g in runner.cache.groups)
    # the same requests once more through the same runner: every slot and page has been used before
    again = run_mixed(runner, case.tokens, sched)
    for rid in case.tokens:
        close(again[rid], case.want[rid], case.dtype, f"{rid} mixed, second time")


def test_a_long_portion_beside_single_tokens(case):
    """One step that holds a portion long enough for the kernels made for long portions (chunks of 64, blocks walked side by
    side) and, beside it, requests that bring a single token each: every request gets what it gets alone."""
    from marin_b200.engine import StepEntry

    long_id = max(case.tokens, key=lambda r: len(case.tokens[r]))
    if len(case.tokens[long_id]) < 256:
        pytest.skip("no request of this configuration is long enough")
    singles = [rid for rid in ("a", "c") if rid != long_id]
    runner = case.runner(96)
    for rid in singles:                                     # all but the last token, alone
        runner.begin(rid)
        runner.step([StepEntry(rid, case.tokens[rid][:-1], [])])
    runner.begin(long_id)
    n = len(case.tokens[long_id])
    entries = [StepEntry(singles[0], case.tokens[singles[0]][-1:], [0]), StepEntry(long_id, case.tokens[long_id], list(range(n))),
               StepEntry(singles[1], case.tokens[singles[1]][-1:], [0])]
    logits = runner.step(entries)
    close(logits[0:1], case.want[singles[0]][-1:], case.dtype, "a single token beside a long portion")
    close(logits[1:1 + n], case.want[long_id], case.dtype, "a long portion beside single tokens")
    close(logits[1 + n:], case.want[singles[1]][-1:], case.dtype, "another single token beside a long portion")
    for rid in singles + [long_id]:
        runner.end(rid)
    runner.cache.check()


def test_a_batch_gives_each_request_what_it_gets_alone(case):
    """float32: the logits of a request are the same bits whatever else the step holds and however its prompt was cut."""
    if case.dtype != "float32":
        pytest.skip("bit equality is the 32-bit path's claim")
    from marin_b200.engine import StepEntry

    runner = case.runner(64)
    alone = {rid: run_whole(runner, rid, case.tokens[rid]) for rid in ("a", "b", "e")}
    for rid in alone:
        runner.begin(rid)
    batch = [StepEntry(rid, case.tokens[rid], list(range(len(case.tokens[rid])))) for rid in ("a", "b", "e")]
    logits = runner.step(batch)
    at = {}
    k = 0
    for rid in ("a", "b", "e"):
        at[rid] = k
        k += len(case.tokens[rid])
    for rid in alone:
        assert torch.equal(logits[at[rid]:at[rid] + len(case.tokens[rid])], alone[rid]), rid
        runner.end(rid)
    cut = run_portions(runner, "ap", case.tokens["a"], portions(len(case.tokens["a"]), [5, 2, 9, 1]))
    assert torch.equal(cut, alone["a"])


def test_greedy_generation_through_the_engine(case):
    """The entry point, the scheduler and device sampling: the tokens are those the plain implementation's logits rank
    first (a token whose plain logit lies within 1e-3 (32-bit) or 0.1 (16-bit) of the largest counts as first)."""
    from marin_b200.engine import Engine
    from marin_b200.sampling.sampler import SamplingParams

    engine = Engine(case.dir, dtype=case.dtype, ctx=case.raw["max_positions"], page_size=case.page, num_pages=48, max_batch=4,
                    token_budget=32)
    prompts = [case.tokens["a"][:21], case.tokens["e"][:3], case.tokens["f" if "f" in case.tokens else "c"][:40]]
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10))
    slack = 1e-3 if case.dtype == "float32" else 0.1
    for prompt, out in zip(prompts, outs):
        assert len(out.tokens) == 10
        seq = list(prompt)
        for token in out.tokens:
            logits = plain.forward(case.raw, case.w, seq)[-1]
            assert logits[token] >= logits.max() - slack, (len(seq), token, int(logits.argmax()))
            seq.append(token)


def test_trace_replay_as_a_user_runs_it(tmp_path):
    """bin/trace_run in a process of its own: steps on standard input, logits read back from files."""
    name, dtype = "A", "float32"
    raw = CONFIGS[name][0]
    d = make_model_dir(str(tmp_path / "model"), name, seed=12)
    w = plain.read_weights(d)
    rng = random.Random(3)
    lengths = {"a": 70, "b": 130, "c": 41, "d": 64, "e": 100, "f": 2}
    tokens = {rid: random_prompt(rng, raw["vocab"], n) for rid, n in lengths.items()}
    want = {rid: plain.forward(raw, w, t) for rid, t in tokens.items()}
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
