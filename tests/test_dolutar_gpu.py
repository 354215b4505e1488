"""Dolutar on the GPU against the plain implementation (`dolutar_plain`): each mechanism's kernels
alone, then the engine whole, decoded token by token, in portions down to two tokens, in mixed
batches with pages and state slots used again, with keys far away, at page borders and at the edges
of the window and of the kept first positions, and through the generation entry point, the command
line and the replay program."""

from __future__ import annotations

import math
import subprocess
import sys

import pytest
import torch

import dolutar_configs as dc
import dolutar_plain as plain
from mlx_omnia_b200 import GenerationOptions, load
from mlx_omnia_b200.engine.engine import Engine, EngineArgs
from mlx_omnia_b200.engine.step import StepEntry
from mlx_omnia_b200.engine.trace import poison_free_pages
from mlx_omnia_b200.kernels import ops
from mlx_omnia_b200.parts.base import KVSpec, KVView
from trace_tools import ROOT, Trace, stacked

pytestmark = pytest.mark.gpu
CUDA = torch.device("cuda:0")
F64 = torch.float64
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rel(a, b) -> float:
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


class Batch:
    """A step's metadata for kernels that are called alone: requests that bring `lens` tokens each
    and held `starts` positions before, in state slots `slots`."""

    def __init__(self, lens, starts=None, slots=None, tokens=None):
        starts = starts or [0] * len(lens)
        self.num_seqs, self.q_lens = len(lens), list(lens)
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        self.num_tokens = cu[-1]
        self.cu_seqlens = torch.tensor(cu, dtype=torch.int32, device=CUDA)
        self.state_slots = torch.tensor(slots or list(range(len(lens))), dtype=torch.int32, device=CUDA)
        self.positions = torch.tensor([s + i for s, n in zip(starts, lens) for i in range(n)], dtype=torch.int32, device=CUDA)
        self.seq_lens = torch.tensor([s + n for s, n in zip(starts, lens)], dtype=torch.int32, device=CUDA)
        self.seq_lens_host = [s + n for s, n in zip(starts, lens)]
        self.max_q_len, self.max_seq_len, self.workspace = max(lens), max(self.seq_lens_host), None
        self.decode_only = all(n == 1 for n in lens)
        self.token_ids = None if tokens is None else torch.tensor(tokens, dtype=torch.int32, device=CUDA)


# ---- each mechanism alone -------------------------------------------------------------------


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pair_embedding_over_portions_and_slots(dtype):
    """Two requests in portions of 1 to 5 tokens: the token before a portion comes from the state
    slot, a request's first token takes the table's extra row, and a slot that another request used
    before starts afresh because its first position is 0."""
    raw, W = dc.config("P"), dc.tensors("P")
    e = raw["embedding"]
    table, pairs = (W[k].to(DTYPES[dtype]).to(CUDA) for k in ("embed", "bigram"))
    a, b = dc.prompt(11, raw["vocab"], 1), dc.prompt(6, raw["vocab"], 2)
    prev = torch.full((4,), 77, dtype=torch.int32, device=CUDA)  # what earlier owners of the slots left
    got = {"a": [], "b": []}
    for (a0, a1), (b0, b1) in [((0, 5), (0, 1)), ((5, 6), (1, 3)), ((6, 11), (3, 6))]:
        step = Batch([a1 - a0, b1 - b0], [a0, b0], [2, 0], a[a0:a1] + b[b0:b1])
        x = ops.embed_pair(step, table, pairs, prev, e["scale"], e["bigram"]["mul_prev"], e["bigram"]["mul_cur"])
        got["a"].append(x[: a1 - a0])
        got["b"].append(x[a1 - a0:])
    assert prev.tolist()[2] == a[-1] and prev.tolist()[0] == b[-1] and prev.tolist()[1] == 77
    for name, ids in (("a", a), ("b", b)):
        assert rel(torch.cat(got[name]), plain.embedding(ids, W, raw, F64)) < 1e-6
    ops.raise_on_error(CUDA)


def _cache(G, dk, dv, page, count, dtype, window, keep):
    spec = KVSpec(((G, dk), (G, dv)), window, keep_first=keep)
    shape = (count, 2, G, page, dk) if dk == dv else (count, (dk + dv) * G * page)
    pages = torch.full(shape, float("nan"), dtype=dtype, device=CUDA)
    return spec, pages


def _view(spec, pages, tables, page, slots=None, writes=True):
    width = max(len(t) for t in tables)
    table = torch.full((len(tables), width), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        table[i, : len(t)] = torch.tensor(t, dtype=torch.int32)
    slot_mapping = torch.tensor(slots if slots is not None else [0], dtype=torch.int64, device=CUDA)
    return KVView(pages, table.to(CUDA), slot_mapping, page, spec.window, writes=writes, spec=spec)


@pytest.mark.parametrize("dtype,H,G,dk,dv,rot", [("float32", 4, 2, 16, 24, 8), ("bfloat16", 5, 1, 40, 40, 40),
                                                  ("bfloat16", 3, 3, 24, 8, 0), ("float32", 2, 1, 64, 64, 32)])
def test_bias_norm_rotation_and_cache_write(dtype, H, G, dk, dv, rot):
    """The step between the input projection and the attention: biases, weighted head norms, a
    rotation of part of the head, keys and values of unequal width into shuffled pages."""
    g = torch.Generator().manual_seed(H * 10 + dk)
    T, page, dt = 13, 4, DTYPES[dtype]
    cols = H * dk + G * dk + G * dv
    proj = torch.randn(T, cols + 3, generator=g).to(dt)
    bias = torch.randn(cols + 3, generator=g).to(dt)
    wq, wk = torch.randn(dk, generator=g), torch.randn(dk, generator=g)
    positions = torch.arange(40, 40 + T)
    inv = torch.tensor([300.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32) if rot else None
    spec, pages = _cache(G, dk, dv, page, 8, dt, None, 0)
    order = [5, 2, 7, 0]
    slots = [order[j // page] * page + j % page for j in range(T)]
    kv = _view(spec, pages, [order], page, slots)
    step = Batch([T], [40])
    q = ops.qkv_prepare(proj.to(CUDA), 0, H * dk, H * dk + G * dk, H, dk, bias.to(CUDA), wq.to(CUDA), wk.to(CUDA), 1e-5,
                        None if inv is None else inv.to(CUDA), step.positions, kv, store=True)
    full = proj.to(F64) + bias.to(F64)
    want_q = plain.rms(full[:, : H * dk].view(T, H, dk), 1e-5, wq.to(F64))
    want_k = plain.rms(full[:, H * dk: H * dk + G * dk].view(T, G, dk), 1e-5, wk.to(F64))
    if rot:
        want_q, want_k = (plain.rotate(x, positions, rot, 300.0) for x in (want_q, want_k))
    want_v = full[:, H * dk + G * dk: cols].view(T, G, dv)
    tol = 1e-5 if dtype == "float32" else 1.5e-2
    assert rel(q, want_q) < tol
    got_k = torch.stack([kv.row(0)[slots[j] // page, :, slots[j] % page] for j in range(T)])
    got_v = torch.stack([kv.row(1)[slots[j] // page, :, slots[j] % page] for j in range(T)])
    assert rel(got_k, want_k) < tol and rel(got_v, want_v) < tol
    ops.raise_on_error(CUDA)


def _attention_reference(q, K, V, positions, window, keep, scale, sink):
    """q [n, H, dk] at `positions` over K [T, G, dk], V [T, G, dv], in float64."""
    n, H, _ = q.shape
    G = K.shape[1]
    out = torch.zeros(n, H, V.shape[2], dtype=F64)
    j = torch.arange(K.shape[0])
    for r in range(n):
        i = int(positions[r])
        see = (j <= i) & ((i - j < window) | (j < keep)) if window else j <= i
        for h in range(H):
            s = (K[:, h // (H // G)].to(F64) @ q[r, h].to(F64)) * scale
            s = s.masked_fill(~see, -math.inf)
            top = max(float(s.max()), float(sink[h]) if sink is not None else -math.inf)
            e = torch.exp(s - top)
            denominator = e.sum() + (math.exp(float(sink[h]) - top) if sink is not None else 0.0)
            out[r, h] = (e / denominator) @ V[:, h // (H // G)].to(F64)
    return out.reshape(n, -1)


def _filled(spec, pages, K, V, page, order):
    """The cache of one request whose logical pages are the physical pages `order`."""
    for j in range(K.shape[0]):
        p, off = order[j // page], j % page
        view = KVView(pages, None, None, page, spec.window, spec=spec)
        view.row(0)[p, :, off] = K[j].to(pages.dtype)
        view.row(1)[p, :, off] = V[j].to(pages.dtype)


ATTENTION_CASES = [("float32", 4, 2, 16, 24, 4), ("bfloat16", 6, 1, 16, 16, 16), ("bfloat16", 4, 2, 64, 64, 16),
                   ("bfloat16", 2, 2, 24, 8, 8), ("float32", 2, 1, 32, 32, 16), ("bfloat16", 8, 2, 128, 128, 16),
                   ("bfloat16", 4, 2, 64, 64, 8)]
# (heads of 64 and 128 over pages of 16: the prompts' portions run on the tcgen05 kernel; over pages of 8 on mma.sync)


@pytest.mark.parametrize("dtype,H,G,dk,dv,page", ATTENTION_CASES)
@pytest.mark.parametrize("window,keep", [(None, 0), (9, 0), (9, 3), (44, 17), (64, 33), (5, 14), (150, 70)])
def test_attention_with_window_kept_positions_and_sink(dtype, H, G, dk, dv, page, window, keep):
    """A prompt read whole, a portion over a context, single tokens (alone and beside a portion), from
    shuffled pages; pages behind the window are not in the block table, free pages hold NaN."""
    g = torch.Generator().manual_seed(dk + (window or 0))
    T, dt, scale = 300, DTYPES[dtype], 0.3
    K, V = (torch.randn(T, G, d, generator=g).to(dt).float() for d in (dk, dv))
    other_T = 37
    K2, V2 = (torch.randn(other_T, G, d, generator=g).to(dt).float() for d in (dk, dv))
    sink = torch.randn(H, generator=g)
    count = -(-T // page) + -(-other_T // page) + 3
    spec, pages = _cache(G, dk, dv, page, count, dt, window, keep)
    perm = torch.randperm(count, generator=g).tolist()
    order, order2 = perm[: -(-T // page)], perm[-(-T // page): -(-T // page) + -(-other_T // page)]
    _filled(spec, pages, K, V, page, order)
    _filled(spec, pages, K2, V2, page, order2)
    tol = 2e-5 if dtype == "float32" else 2e-2

    def dead(table, first_query):
        """The table as the cache manager leaves it ahead of a step whose first query stands at `first_query`."""
        if not window:
            return table
        kept_pages = -(-keep // page)
        gone = max(first_query - window + 1, 0) // page
        return [p if i < kept_pages or i >= gone else -1 for i, p in enumerate(table)]

    for lens, starts in [([T], [0]), ([120], [180]), ([1], [T - 1]), ([1], [130]), ([2, 1, 30, 1], [200, 36, 7, 63]),
                         ([1, 1, 1], [299, 20, 0])]:
        step = Batch(lens, starts)
        which = [0 if i != 1 or len(lens) != 4 else 1 for i in range(len(lens))]  # the second of four is the other request
        if len(lens) == 4:
            tables = [dead(order, 200), dead(order2, 36), dead(order, 7), dead(order, 63)]
        elif len(lens) == 3:
            tables = [dead(order, 299), dead(order, 20), dead(order, 0)]
        else:
            tables = [dead(order, starts[0])]
        kv = _view(spec, pages, tables, page)
        q = torch.randn(step.num_tokens, H, dk, generator=g).to(dt)
        got = ops.paged_attention(q.to(CUDA), kv, step, scale, sink=sink.to(CUDA), window=window, keep_first=keep)
        at = 0
        for i, (n, s) in enumerate(zip(lens, starts)):
            Ks, Vs = (K2, V2) if which[i] else (K, V)
            want = _attention_reference(q[at: at + n].float(), Ks, Vs, range(s, s + n), window, keep, scale, sink)
            assert rel(got[at: at + n], want) < tol, (lens, starts, i)
            at += n
    ops.raise_on_error(CUDA)


@pytest.mark.parametrize("dtype,H,G,dk,dv,page", ATTENTION_CASES)
def test_a_far_kept_key_a_window_edge_and_the_sink(dtype, H, G, dk, dv, page):
    """One key's score is made to stand out among 640: the last kept position is found from far away,
    the position after it is not; the oldest key of the window is seen, the one before it is not; and
    the sink takes its share. Each time the query is a single token and the last of a portion."""
    g = torch.Generator().manual_seed(7 * dk)
    T, dt, scale, window, keep = 640, DTYPES[dtype], 0.5, 48, 21
    sink = torch.full((H,), 13.0)  # against the boosted key's score of 15: the sink takes an eighth
    tol = 2e-5 if dtype == "float32" else 2e-2
    for boosted, seen in [(keep - 1, True), (keep, False), (T - window, True), (T - window - 1, False)]:
        K, V = (torch.randn(T, G, d, generator=g).to(dt).float() for d in (dk, dv))
        q = torch.randn(1, G, dk, generator=g).repeat_interleave(H // G, dim=1)  # a group's heads look the same way
        q = (q / q.norm(dim=-1, keepdim=True) * 6.0).to(dt)
        K[boosted] = (q[0, :: H // G].float() / 6.0 * 5.0).to(dt).float()  # a score of about 15 against a few
        spec, pages = _cache(G, dk, dv, page, T // page + 2, dt, window, keep)
        order = torch.randperm(T // page + 2, generator=g).tolist()[: T // page]
        _filled(spec, pages, K, V, page, order)
        want = _attention_reference(q.float(), K, V, [T - 1], window, keep, scale, sink)
        share = rel(want.view(H, dv), V[boosted].repeat_interleave(H // G, dim=0).double())
        assert (share < 0.4) == seen  # with the key seen, the output is close to its value
        without = _attention_reference(q.float(), K, V, [T - 1], window, keep, scale, None)
        assert rel(without, want) > 1e-3
        for lens, starts in [([1], [T - 1]), ([17], [T - 17])]:
            step = Batch(lens, starts)
            rows = torch.cat([torch.randn(lens[0] - 1, H, dk, generator=g).to(dt), q])
            kv = _view(spec, pages, [order], page)
            got = ops.paged_attention(rows.to(CUDA), kv, step, scale, sink=sink.to(CUDA), window=window, keep_first=keep)
            assert rel(got[-1:], want) < tol, (boosted, lens)
    ops.raise_on_error(CUDA)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_clamped_gated_unit(dtype):
    g = torch.Generator().manual_seed(3)
    gu = (torch.randn(7, 2 * 40, generator=g) * 3).to(DTYPES[dtype])
    got = ops.clamped_glu(gu.to(CUDA), 1.702, 1.25)
    a, b = gu[:, :40].double().clamp(max=1.25), gu[:, 40:].double().clamp(-1.25, 1.25)
    assert rel(got, a * torch.sigmoid(1.702 * a) * (b + 1)) < (1e-6 if dtype == "float32" else 8e-3)


@pytest.mark.parametrize("dtype,tensor_cores", [("float32", False), ("bfloat16", True), ("bfloat16", False)])
@pytest.mark.parametrize("rows,hidden,inner,experts,identity,top", [(50, 96, 24, 5, 2, 2), (1, 64, 40, 3, 0, 1),
                                                                  (200, 128, 72, 9, 3, 4), (3, 64, 8, 2, 5, 3),
                                                                  (700, 192, 136, 3, 1, 2), (1100, 64, 24, 6, 1, 2)])
def test_routed_experts(dtype, tensor_cores, rows, hidden, inner, experts, identity, top):
    """Router, sorted order, grouped products and the weighted sum, on the ordinary cores and on the
    tensor cores, against the plain function; the buffers that must be zero between calls are."""
    g = torch.Generator().manual_seed(rows + experts)
    dt = DTYPES[dtype]
    W = {"m.router": torch.randn(experts + identity, hidden, generator=g) * 0.4,
         "m.correction": torch.randn(experts + identity, generator=g) * 0.1}
    for e in range(experts):
        W[f"m.e{e}.gate"] = (torch.randn(inner, hidden, generator=g) * hidden ** -0.5).to(dt).float()
        W[f"m.e{e}.up"] = (torch.randn(inner, hidden, generator=g) * hidden ** -0.5).to(dt).float()
        W[f"m.e{e}.down"] = (torch.randn(hidden, inner, generator=g) * inner ** -0.5).to(dt).float()
    h = torch.randn(rows, hidden, generator=g).to(dt)
    gate_up = torch.stack([torch.cat([W[f"m.e{e}.gate"], W[f"m.e{e}.up"]]) for e in range(experts)]).to(dt).to(CUDA)
    down = torch.stack([W[f"m.e{e}.down"] for e in range(experts)]).to(dt).to(CUDA)
    router = {"experts": experts, "identity": identity, "top": top}
    want = plain.moe_ff(h.double(), W, "m.", router)
    for _ in range(2):  # the second call finds the counters as the first one left them
        got = ops.moe_experts(h.to(CUDA), W["m.router"].to(CUDA), W["m.correction"].to(CUDA), gate_up, down, top,
                              tensor_cores=tensor_cores)
        assert rel(got, want) < (2e-5 if dtype == "float32" else 2.5e-2)
    if tensor_cores:  # the same on the tcgen05 kernel's grouped form, whatever the number of rows
        got = ops.moe_experts(h.to(CUDA), W["m.router"].to(CUDA), W["m.correction"].to(CUDA), gate_up, down, top,
                              tcgen05=True)
        assert rel(got, want) < 2.5e-2
        ops.raise_on_error(CUDA)
    counts = torch.zeros(experts, dtype=torch.int32, device=CUDA)
    choice, weight = ops.moe_route(h.to(CUDA), W["m.router"].to(CUDA), W["m.correction"].to(CUDA), experts, top, counts)
    chosen, weights = plain.route(h.double(), W, "m.", top)
    assert torch.equal(choice.cpu().sort(-1).values.long(), chosen.sort(-1).values)
    assert rel(weight.cpu().sum(-1), weights.sum(-1)) < 1e-5
    assert counts.cpu().tolist() == [int((chosen == e).sum()) for e in range(experts)]


# ---- the engine ------------------------------------------------------------------------------


def engine_for(name, dtype="float32", page=4, tokens=1024, requests=4, graphs=True, seed=0, raw=None):
    raw = raw or dc.config(name)
    weights = dc.tensors(raw, seed)
    engine = Engine.from_tensors(raw, weights, EngineArgs(dtype=dtype, page_size=page, cache_tokens=tokens,
                                                          max_requests=requests, cuda_graphs=graphs))
    return raw, weights, engine


TOLERANCE = {"float32": 3e-4, "bfloat16": 6e-2}


def assert_rows(got, want, dtype, what="", tolerance=None):
    """Rows of logits against rows of the plain implementation. In float32 every row is within the
    tolerance. In bfloat16 a routed layer's choice between two experts of nearly equal score can
    fall the other way than in float64, which moves that token's row by far more than rounding does
    (and rows after it a little): so all rows but 3 in 100 (or one), and the median row within a
    quarter of the tolerance."""
    tolerance = tolerance or TOLERANCE[dtype]
    got, want = got.detach().cpu().double(), want.detach().cpu().double()
    assert got.shape == want.shape
    err = (got - want).abs().amax(-1) / want.abs().max().clamp_min(1e-30)
    assert not torch.isnan(err).any(), what
    if dtype == "float32":
        assert float(err.max()) < tolerance, (what, int(err.argmax()), float(err.max()))
    else:
        over = int((err > tolerance).sum())
        assert over <= max(1, (3 * err.numel()) // 100), (what, over, (err > tolerance).nonzero().flatten().tolist()[:20])
        assert float(err.median()) < tolerance / 4, (what, float(err.median()))


@pytest.mark.parametrize("name", ["P", "Q", "R", "O"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts(name, dtype):
    raw, weights, engine = engine_for(name, dtype)
    for n in (1, 2, 3, 41, 230):
        ids = dc.prompt(n, raw["vocab"], n)
        request = engine.cache.open("r")
        got = engine.runner.run([StepEntry(request, ids, list(range(n)))])
        engine.cache.close("r")
        assert_rows(got, plain.forward(ids, weights, raw), dtype, n)
    ops.raise_on_error(CUDA)


@pytest.mark.parametrize("name,page", [("P", 4), ("Q", 16), ("R", 8), ("O", 16)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_decoding_and_mixed_batches(tmp_path, name, page, dtype):
    """Six requests over four state slots: prompts read whole, in portions of 2 to 9 tokens and
    token by token, decoded tokens beside portions of other requests, requests that end and whose
    pages and slots the next ones take (free pages are filled with NaN before every step)."""
    raw, weights, engine = engine_for(name, dtype, page=page, tokens=448)
    V = raw["vocab"]
    ids = {r: dc.prompt(n, V, i) for i, (r, n) in enumerate({"a": 170, "b": 33, "c": 2, "d": 58, "e": 60, "f": 17}.items())}
    trace = Trace()
    at = {r: 0 for r in ids}

    def take(r, n):
        out = ids[r][at[r]: at[r] + n]
        at[r] += len(out)
        return out

    trace.step({"a": take("a", 9), "b": take("b", 33)})
    trace.step({"a": take("a", 2), "c": take("c", 1), "d": take("d", 5)}, end=["b"])
    trace.step({"a": take("a", 7), "c": take("c", 1), "d": take("d", 3), "e": take("e", 40)}, end=["c"])
    for _ in range(6):
        trace.step({"a": take("a", 1), "d": take("d", 2), "e": take("e", 1)})
    trace.step({"f": take("f", 17), "a": take("a", 1)}, end=["f"])
    for _ in range(3):
        trace.step({"e": take("e", 1), "a": take("a", 4), "d": take("d", 1)})
    trace.step({"a": take("a", 97)})
    for _ in range(12):
        trace.step({"a": take("a", 1), "d": take("d", 1)})
    trace.step({"a": take("a", 170), "d": take("d", 58), "e": take("e", 60)}, end=["a", "d", "e"])
    got = trace.run_engine(engine, tmp_path / "out", before_step=lambda e, record: poison_free_pages(e))
    assert not engine.cache.requests
    engine.cache.check()
    for r in ids:
        positions, logits = stacked(got[r])
        assert positions == list(range(len(ids[r])))
        assert_rows(logits, plain.forward(ids[r], weights, raw), dtype, r)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_heads_of_64_over_pages_of_16(tmp_path, dtype):
    """Sizes at which bfloat16 prompts take the tcgen05 attention kernel: whole prompts from 1 to 400
    tokens (kept positions beyond, at and inside the window's first tile), portions over a context,
    single tokens beside portions, a reader whose kept positions outnumber its owner's."""
    raw, weights, engine = engine_for("S", dtype, page=16, tokens=1536)
    for n in (1, 9, 70, 71, 140, 400):
        ids = dc.prompt(n, raw["vocab"], n)
        request = engine.cache.open("r")
        got = engine.runner.run([StepEntry(request, ids, list(range(n)))])
        engine.cache.close("r")
        assert_rows(got, plain.forward(ids, weights, raw), dtype, n)
    ids = {"a": dc.prompt(330, raw["vocab"], 1), "b": dc.prompt(90, raw["vocab"], 2), "c": dc.prompt(40, raw["vocab"], 3)}
    trace = Trace()
    trace.step({"a": ids["a"][:130]})
    trace.step({"a": ids["a"][130:263], "b": ids["b"][:64]})
    trace.step({"a": ids["a"][263:264], "b": ids["b"][64:90], "c": ids["c"][:2]}, end=["b"])
    trace.step({"a": ids["a"][264:330], "c": ids["c"][2:40]}, end=["a", "c"])
    got = trace.run_engine(engine, tmp_path / "out", before_step=lambda e, record: poison_free_pages(e))
    for r in ids:
        positions, logits = stacked(got[r])
        assert positions == list(range(len(ids[r])))
        assert_rows(logits, plain.forward(ids[r], weights, raw), dtype, r)
    ops.raise_on_error(CUDA)


@pytest.mark.parametrize("name", ["P", "Q"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_equals_decoding_token_by_token(name, dtype):
    """The same prompt whole, and one token a step (captured decode steps, and launched one by one)."""
    for graphs in (True, False):
        raw, weights, engine = engine_for(name, dtype, graphs=graphs)
        ids = dc.prompt(75, raw["vocab"], 77)
        request = engine.cache.open("w")
        whole = engine.runner.run([StepEntry(request, ids, list(range(len(ids))))])
        engine.cache.close("w")
        request = engine.cache.open("t")
        single = torch.cat([engine.runner.run([StepEntry(request, [t], [0])]) for t in ids])
        engine.cache.close("t")
        assert_rows(single, whole, dtype, "token by token against whole", 2e-5 if dtype == "float32" else 4e-2)
        assert_rows(single, plain.forward(ids, weights, raw), dtype)
    ops.raise_on_error(CUDA)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_across_tiles_chunks_and_pages(dtype):
    """700 tokens with windows of 150 and 64 and 70 and 33 kept positions: portions that start and end
    inside tiles of 64 keys, decode chunks of 128 and pages of 16, then 40 tokens decoded beside a
    short request whose pages are the ones the long request gave back."""
    raw, weights, engine = engine_for("R", dtype, page=16, tokens=1024)
    ids = dc.prompt(700, raw["vocab"], 5)
    ids[-1] = ids[11]
    other = dc.prompt(50, raw["vocab"], 6)
    a = engine.cache.open("a")
    rows = {}
    at = 0
    for n in (193, 2, 130, 61, 255, 19):
        out = engine.runner.run([StepEntry(a, ids[at: at + n], [n - 1])])
        rows[at + n - 1] = out[0]
        at += n
    b = engine.cache.open("b")
    engine.runner.run([StepEntry(b, other[:10], [])])
    for t in range(at, 700):
        out = engine.runner.run([StepEntry(a, ids[t: t + 1], [0]), StepEntry(b, other[10 + t - at: 11 + t - at], [0])])
        rows[t] = out[0]
        rows[("b", 10 + t - at)] = out[1]
    expect, expect_b = plain.forward(ids, weights, raw), plain.forward(other, weights, raw)
    keys = list(rows)
    assert_rows(torch.stack([rows[key] for key in keys]),
                torch.stack([expect_b[key[1]] if isinstance(key, tuple) else expect[key] for key in keys]), dtype, keys)
    ops.raise_on_error(CUDA)


def test_the_edges_show_in_the_logits():
    """One position more or less in a window or among the kept positions, or a missing sink, moves the
    plain implementation's logits by far more than the engine is from it: the comparisons above see
    such a fault. In a prompt and in decoding."""
    raw, weights, engine = engine_for("P", "float32")
    ids = dc.prompt(48, raw["vocab"], 8)
    request = engine.cache.open("r")
    got = [engine.runner.run([StepEntry(request, ids[:30], list(range(30)))])]
    got += [engine.runner.run([StepEntry(request, [t], [0])]) for t in ids[30:]]
    expect = plain.forward(ids, weights, raw)
    assert rel(torch.cat(got), expect) < TOLERANCE["float32"]
    for layer, key, change in [(0, "size", 1), (0, "size", -1), (0, "keep_first", 1), (1, "keep_first", -1), (3, "size", 1)]:
        other = dc.config("P")
        other["layers"][layer]["mixer"]["mask"][key] += change
        moved = plain.forward(ids, weights, other)
        assert rel(moved[:30], expect[:30]) > 1e-3 and rel(moved[30:], expect[30:]) > 1e-3, (layer, key, change)
    no_sink = dict(weights)
    no_sink["l2.mix.sink"] = torch.full_like(weights["l2.mix.sink"], -1e30)
    assert rel(plain.forward(ids, no_sink, raw), expect) > 1e-3


def test_greedy_generation_long_decoding_and_the_scheduler(tmp_path):
    """Through `load(...).generate`: the scheduler admits, batches and chunks; greedy ids are the plain
    implementation's best, 200 tokens past a two-token prompt included (the window passes over
    decoded tokens many times)."""
    raw = dc.config("P")
    weights = dc.tensors(raw, 3)
    folder = tmp_path / "m"
    dc.write_folder(folder, raw, weights)
    model = load(folder, dtype="float32", page_size=8, cache_tokens=1024, max_requests=4, max_tokens_per_step=16)
    prompts = [dc.prompt(n, raw["vocab"], 20 + n) for n in (2, 5, 23, 40, 9, 31)]
    counts = [200, 12, 12, 12, 12, 12]
    got = [model.generate([prompts[0]], GenerationOptions(max_tokens=200, stop=()))[0]]
    got += model.generate(prompts[1:], GenerationOptions(max_tokens=12, stop=()))
    for prompt, ids, count in zip(prompts, got, counts):
        assert len(ids) == count
        logits = plain.forward(prompt + ids, weights, raw)[len(prompt) - 1: -1]
        best = logits.max(dim=-1).values
        chosen = logits[torch.arange(count), torch.tensor(ids)]
        assert float((best - chosen).max()) <= 1e-3 * float(logits.abs().max())
    assert not model.engine.cache.requests
    done = subprocess.run([sys.executable, str(ROOT / "bin" / "omnia"), "run", "-m", str(folder), "--max-tokens", "5",
                           "--temperature", "0", "--dtype", "float32", *map(str, prompts[1])],
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-3000:]
    assert [int(t) for t in done.stdout.split()[:5]] == got[1][:5]


def test_replay_program_on_a_model_folder(tmp_path):
    """`bin/trace_run` as a user runs it, in bfloat16, on a folder written by the random-weights mode."""
    from safetensors.torch import load_file

    from mlx_omnia_b200.weights.random_init import write_random_model

    raw = dc.config("Q")
    folder = write_random_model(tmp_path / "m", raw, seed=4)
    weights = {k: v.float() for k, v in load_file(str(folder / "model.safetensors")).items()}
    ids = dc.prompt(90, raw["vocab"], 1)
    trace = Trace()
    trace.step({"p": ids[:50]}, want="last")
    trace.step({"p": ids[50:52], "q": ids[:7]})
    for t in range(52, 90):
        trace.step({"p": ids[t: t + 1]}, end=["p"] if t == 89 else ["q"] if t == 52 else [])
    got = trace.run(folder, "bfloat16", tmp_path / "out", vocab=raw["vocab"])
    expect = plain.forward(ids, weights, raw)
    positions, logits = stacked(got["p"])
    assert positions == [49] + list(range(50, 90))
    assert_rows(logits, expect[positions], "bfloat16")
