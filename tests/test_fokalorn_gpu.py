"""Fokalorn on the GPU against the plain implementation (`fokalorn_plain`): each mechanism's kernels
alone, then the engine whole, decoded token by token, in portions down to two tokens, in mixed
batches with pages and state slots used again, with keys far away and at page borders, and through
the generation entry point and the command line."""

from __future__ import annotations

import json
import math
import subprocess
import sys

import pytest
import torch
from safetensors.torch import save_file

import fokalorn_configs as fc
import fokalorn_plain as plain
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


def rel(a, b) -> float:
    a, b = a.detach().cpu().double(), b.detach().cpu().double()
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


class Batch:
    """A step's metadata for kernels that are called alone: requests with `lens` tokens each that
    held `starts` positions before, in state slots `slots`."""

    def __init__(self, lens, starts=None, slots=None):
        starts = starts or [0] * len(lens)
        self.num_seqs, self.q_lens = len(lens), list(lens)
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        self.cu = cu
        self.cu_seqlens = torch.tensor(cu, dtype=torch.int32, device=CUDA)
        self.state_slots = torch.tensor(slots or list(range(len(lens))), dtype=torch.int32, device=CUDA)
        self.positions = torch.tensor([s + i for s, n in zip(starts, lens) for i in range(n)], dtype=torch.int32, device=CUDA)
        self.seq_lens = torch.tensor([s + n for s, n in zip(starts, lens)], dtype=torch.int32, device=CUDA)
        self.max_q_len, self.max_seq_len, self.workspace = max(lens), max(s + n for s, n in zip(starts, lens)), None


# ---- each mechanism alone -------------------------------------------------------------------


@pytest.mark.parametrize("streams,groups,width", [(3, 4, 96), (1, 1, 64), (2, 5, 80), (4, 16, 1024), (2, 1, 2048)])
def test_streams_norm_and_shift(streams, groups, width):
    """Two requests of unequal length, each in two portions (the second request's second portion a
    single token): the normed, shifted input and the streams after the branch is written back."""
    g = torch.Generator().manual_seed(streams * 100 + groups)
    lens = (7, 4)
    xs = [torch.randn(n, streams, width, generator=g) for n in lens]
    coef, mix, outc = torch.randn(streams, generator=g), torch.randn(streams, streams, generator=g), torch.randn(streams, generator=g)
    w, mu = torch.randn(width, generator=g), torch.rand(width, generator=g)
    ys = [torch.randn(n, width, generator=g) for n in lens]
    expect_h, expect_x = [], []
    for x, y in zip(xs, ys):
        u = (x.to(F64) * coef.to(F64)[None, :, None]).sum(1)
        expect_h.append(plain.token_shift(plain.grouped_rms_norm(u, w.to(F64), 1e-5, groups), mu.to(F64)))
        expect_x.append(torch.einsum("st,nsd->ntd", mix.to(F64), x.to(F64)) + outc.to(F64)[None, :, None] * y.to(F64)[:, None])
    prev = torch.full((5, width), 9.0, device=CUDA)
    prev[[3, 1]] = 0
    got_h, got_x = [[], []], [[], []]
    for cut in ((0, 5, 0, 3), (5, 7, 3, 4)):
        a0, a1, b0, b1 = cut
        step = Batch([a1 - a0, b1 - b0], [a0, b0], [3, 1])
        x = torch.cat([xs[0][a0:a1], xs[1][b0:b1]]).reshape(-1, streams * width).to(CUDA).contiguous()
        y = torch.cat([ys[0][a0:a1], ys[1][b0:b1]]).to(CUDA)
        last = torch.empty(2, width, device=CUDA)
        h = ops.streams_enter(x, coef.to(CUDA), streams, w.to(CUDA), 1e-5, groups, torch.float32, step, mu.to(CUDA), prev, last)
        ops.streams_leave(x, y, mix.to(CUDA), outc.to(CUDA), streams, step, last, prev)
        x = x.view(-1, streams, width)
        for r, (lo, hi) in enumerate(((0, a1 - a0), (a1 - a0, a1 - a0 + b1 - b0))):
            got_h[r].append(h[lo:hi]), got_x[r].append(x[lo:hi])
    for r in range(2):
        assert rel(torch.cat(got_h[r]), expect_h[r]) < 1e-5
        assert rel(torch.cat(got_x[r]), expect_x[r]) < 1e-5
    assert float((prev[[0, 2, 4]] - 9.0).abs().max()) == 0.0  # other requests' slots are left alone
    # leaving one branch and entering the next in one kernel
    x = torch.cat(xs).reshape(-1, streams * width).to(CUDA).contiguous()
    h2 = ops.streams_leave(x, torch.cat(ys).to(CUDA), mix.to(CUDA), outc.to(CUDA), streams,
                           enter=(coef.to(CUDA), w.to(CUDA), 1e-5, groups))
    new = torch.cat(expect_x)
    expect_h2 = plain.grouped_rms_norm((new * coef.to(F64)[None, :, None]).sum(1), w.to(F64), 1e-5, groups)
    assert rel(h2, expect_h2) < 1e-5 and rel(x.view(-1, streams, width), new) < 1e-5


def test_plain_residual_is_one_stream_without_mixing():
    x, y = torch.randn(5, 64, device=CUDA), torch.randn(5, 64, device=CUDA)
    expect = x + y
    ops.streams_leave(x, y, None, None, 1)
    assert rel(x, expect) < 1e-6
    w = torch.randn(64, device=CUDA)
    h = ops.streams_enter(x, None, 1, w, 1e-6, 1, torch.float32)
    assert rel(h, plain.grouped_rms_norm(x.cpu().double(), w.cpu().double(), 1e-6)) < 1e-5


@pytest.mark.parametrize("kind", ["relu2", "gelu_tanh", "silu"])
def test_activation(kind):
    z = torch.randn(33, 70, device=CUDA) * 3
    assert rel(ops.activation(z, kind), plain.ACTIVATIONS[kind](z.cpu().double())) < 1e-5
    zb = z.to(torch.bfloat16)
    assert rel(ops.activation(zb, kind), plain.ACTIVATIONS[kind](zb.cpu().double())) < 1e-2


@pytest.mark.parametrize("H,G,dk,dv,K,parts", [(4, 2, 24, 40, 4, 1), (1, 1, 8, 8, 1, None), (3, 3, 12, 20, 5, 5),
                                                (2, 1, 64, 128, 2, None), (2, 2, 128, 64, 3, 4), (1, 1, 32, 200, 2, 2),
                                                (2, 2, 128, 128, 4, 1), (4, 2, 24, 40, 4, 2)])
def test_short_convolution_and_delta_rule(H, G, dk, dv, K, parts):
    """The recurrent mixer's two kernels over three requests cut into portions of 1 to 9 tokens, one
    request joining late into a slot that another has left, against the whole-sequence recurrence."""
    g = torch.Generator().manual_seed(H * 7 + dk)
    C = 2 * G * dk + H * dv
    lens = {"a": 60, "b": 9, "c": 14}
    raw = {r: torch.randn(n, C, generator=g) for r, n in lens.items()}
    beta_l = {r: torch.randn(n, H, generator=g) for r, n in lens.items()}
    a_l = {r: torch.randn(n, H * dk, generator=g) for r, n in lens.items()}
    gate_l = {r: torch.randn(n, H * dv, generator=g) for r, n in lens.items()}
    taps = torch.randn(C, K, generator=g) * 0.5
    A_log, dt_bias, nw = torch.randn(H, generator=g) * 0.5 - 1, torch.randn(H * dk, generator=g), torch.randn(dv, generator=g)

    def whole(r):
        y = plain.short_conv_silu(raw[r].to(F64), taps.to(F64))
        q = plain.unit(y[:, : G * dk].reshape(-1, G, dk)) * dk ** -0.5
        k = plain.unit(y[:, G * dk: 2 * G * dk].reshape(-1, G, dk))
        v = y[:, 2 * G * dk:].reshape(-1, H, dv)
        step = torch.nn.functional.softplus(a_l[r].to(F64) + dt_bias.to(F64)).reshape(-1, H, dk)
        decay = torch.exp(-torch.exp(A_log.to(F64)).reshape(1, H, 1) * step)
        outs = []
        for h in range(H):
            o, _ = plain.delta_rule(q[:, h // (H // G)], k[:, h // (H // G)], v[:, h], torch.sigmoid(beta_l[r].to(F64))[:, h], decay[:, h])
            o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + 1e-5) * nw.to(F64)
            outs.append(o * torch.sigmoid(gate_l[r].to(F64)).reshape(-1, H, dv)[:, h])
        return torch.cat(outs, -1)

    S = torch.full((4, H, dk, dv), 3.0, device=CUDA)
    conv_state = torch.full((4, K - 1, C), 3.0, device=CUDA)
    lens = {"a": 60, "b": 9, "c": 14}
    plan = [{"a": 9, "b": 2}, {"a": 1, "b": 7}, {"a": 3}, {"a": 2, "c": 5}, {"c": 1, "a": 8}, {"c": 8, "a": 37}]
    slots, at, got = {"a": 2, "b": 0, "c": 0}, {r: 0 for r in lens}, {r: [] for r in lens}
    for portions in plan:
        for r in portions:
            if at[r] == 0:  # a fresh request's slot starts as zeros
                S[slots[r]] = 0
                conv_state[slots[r]] = 0
        step = Batch(list(portions.values()), [at[r] for r in portions], [slots[r] for r in portions])
        cut = lambda store: torch.cat([store[r][at[r]: at[r] + n] for r, n in portions.items()])
        proj = torch.cat([cut(raw), cut(beta_l)], dim=1).to(CUDA).contiguous()
        conv = ops.short_conv(proj, 0, C, taps.to(CUDA), conv_state, step, 2 * G * dk, dk, 1e-6, G * dk, dk ** -0.5,
                              cut(a_l).to(CUDA), A_log.to(CUDA), dt_bias.to(CUDA), C, H)
        out = ops.delta_rule(conv, C, G, H, dk, dv, proj, 0, cut(gate_l).to(CUDA), nw.to(CUDA), 1e-5, S, conv_state, K,
                             step, parts=parts)
        lo = 0
        for r, n in portions.items():
            got[r].append(out[lo: lo + n])
            lo, at[r] = lo + n, at[r] + n
    for r in lens:
        assert rel(torch.cat(got[r]), whole(r)) < 2e-5, r
    assert float((S[[1, 3]] - 3.0).abs().max()) == 0.0


def latent_case(H, dn, dr, dims, rank, page, lens, window=None, sink=True, seed=0, dtype=torch.float32, boost=None,
                tensor_cores=None, first=None):
    """Latent attention's two kernels over requests of `lens` tokens, each read in two portions into
    scattered pages, against the plain implementation's expanded form (identity expansions, so that
    its keys and values are the latent rows themselves)."""
    g = torch.Generator().manual_seed(seed)
    qd, width = dn + dr, rank + dr
    base = 50.0
    inv = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32, device=CUDA)
    norm_w, sinks = torch.randn(rank, generator=g), torch.randn(H, generator=g) + 1.0
    pages_per = [-(-n // page) for n in lens]
    order = torch.randperm(sum(pages_per) + 3, generator=g).tolist()
    cache = torch.full((sum(pages_per) + 3, 1, 1, page, width), float("nan"), dtype=dtype, device=CUDA)
    table = torch.full((len(lens), max(pages_per)), -1, dtype=torch.int32)
    for s, count in enumerate(pages_per):
        table[s, :count] = torch.tensor([order.pop() for _ in range(count)])
    table = table.to(CUDA)
    qs = [torch.randn(n, H, qd, generator=g) for n in lens]
    downs = [torch.randn(n, width, generator=g) for n in lens]
    q_lats = [torch.randn(n, H, rank, generator=g) for n in lens]  # stands for uk^T q_plain
    gates = [torch.randn(n, H, generator=g) for n in lens]
    if boost is not None:  # one far key that one query must find among all others
        s, query, key = boost
        downs[s][key, :rank] = q_lats[s][query, 0] * 1.0
        q_lats[s][query, 0] *= 6.0
    expect = []
    for s, n in enumerate(lens):
        pos = torch.arange(n)
        c = plain.grouped_rms_norm(downs[s][:, :rank].to(F64), norm_w.to(F64), 1e-5)
        if dtype == torch.bfloat16:
            c = c.to(dtype).to(F64)
        kr = plain.rotate_interleaved(downs[s][:, rank:].to(F64), pos, dims, base)
        qr = plain.rotate_interleaved(qs[s][:, :, dn:].to(F64), pos, dims, base)
        scores = (torch.einsum("thr,sr->hts", q_lats[s].to(F64), c) + torch.einsum("thd,sd->hts", qr, kr)) * 0.3
        scores = scores.masked_fill(torch.ones(n, n, dtype=torch.bool).triu(1), -math.inf)
        if window:
            scores = scores.masked_fill(torch.ones(n, n, dtype=torch.bool).tril(-window), -math.inf)
        if sink:
            scores = torch.cat([scores, sinks.to(F64).reshape(H, 1, 1).expand(H, n, 1)], dim=-1)
        weights = torch.softmax(scores, dim=-1)[..., :n]
        expect.append(torch.einsum("hts,sr->thr", weights, c) * torch.sigmoid(gates[s].to(F64))[:, :, None])
    got = [[] for _ in lens]
    for part in (0, 1):
        at = [min(max(first or n // 2, 1), n) for n in lens]
        cuts = [(0, c) if part == 0 else (c, n) for c, n in zip(at, lens)]
        live = [s for s, (lo, hi) in enumerate(cuts) if hi > lo]
        step = Batch([cuts[s][1] - cuts[s][0] for s in live], [cuts[s][0] for s in live])
        take = lambda store: torch.cat([store[s][cuts[s][0]: cuts[s][1]] for s in live])
        tokens = int(step.positions.shape[0])
        proj = torch.cat([take(qs).reshape(tokens, H * qd), take(downs), take(gates)], dim=1)
        proj = torch.nn.functional.pad(proj, (0, -proj.shape[1] % 8)).to(dtype).to(CUDA).contiguous()
        slot = torch.cat([table[s].long()[torch.arange(*cuts[s]) // page].cpu() * page + torch.arange(*cuts[s]) % page
                          for s in live]).to(CUDA)
        kv = KVView(cache, table[live].contiguous(), slot, page, window, True, KVSpec(((1, width),), window))
        ops.latent_prepare(proj, 0, H, qd, H * qd, rank, dr, norm_w.to(CUDA), 1e-5, inv, step.positions, kv)
        q3 = proj[:, : H * qd].view(tokens, H, qd)
        q_lat = take(q_lats).to(dtype).to(CUDA).transpose(0, 1).contiguous()
        out = torch.empty(H, tokens, rank, dtype=dtype, device=CUDA)
        if tensor_cores:
            assert ops.latent_tc_supported(q_lat, q3[:, :, dn:], out, 0.3)
        ops.latent_attention(q_lat, q3[:, :, dn:], kv, step, 0.3, sinks.to(CUDA) if sink else None, proj[:, H * qd + width:], out,
                             tensor_cores=tensor_cores)
        lo = 0
        for s in live:
            n = cuts[s][1] - cuts[s][0]
            got[s].append(out[:, lo: lo + n].transpose(0, 1))
            lo += n
    ops.raise_on_error(CUDA)
    return [torch.cat(parts) for parts in got], expect


@pytest.mark.parametrize("H,dn,dr,dims,rank,page,window,sink", [
    (3, 24, 8, 4, 40, 4, None, True), (1, 8, 4, 4, 16, 16, None, False), (5, 16, 16, 16, 48, 8, 7, True),
    (2, 32, 64, 64, 512, 16, None, True), (4, 12, 6, 6, 24, 4, 16, True)])
def test_latent_attention_kernels(H, dn, dr, dims, rank, page, window, sink):
    """Lengths on, just under and just over page borders; windows that end inside a portion."""
    got, expect = latent_case(H, dn, dr, dims, rank, page, [1, page, page + 1, 3 * page - 1, 37], window, sink, seed=H)
    for a, b in zip(got, expect):
        assert rel(a, b) < 2e-5


def test_latent_attention_finds_a_far_key_and_counts_the_sink():
    """Position 600 asks for position 3 of 640, a score that stands out from hundreds; and leaving
    the sink out of the same case moves the result, so the comparison above would notice."""
    got, expect = latent_case(2, 16, 8, 8, 32, 16, [640], seed=9, boost=(0, 600, 3))
    assert rel(got[0], expect[0]) < 2e-5
    without, _ = latent_case(2, 16, 8, 8, 32, 16, [640], sink=False, seed=9, boost=(0, 600, 3))
    assert rel(without[0], expect[0]) > 1e-2
    got16, expect16 = latent_case(2, 16, 8, 8, 32, 16, [640], seed=9, boost=(0, 600, 3), dtype=torch.bfloat16)
    assert rel(got16[0], expect16[0]) < 3e-2


@pytest.mark.parametrize("H,dn,dr,dims,rank,page,window,sink", [
    (3, 24, 32, 8, 64, 16, None, True), (16, 64, 64, 64, 128, 16, None, True), (20, 32, 64, 32, 192, 4, 21, False),
    (1, 16, 32, 32, 64, 8, None, True), (5, 8, 64, 64, 512, 16, 40, True)])
def test_latent_attention_on_the_tensor_cores(H, dn, dr, dims, rank, page, window, sink):
    """The bfloat16 kernel against the plain implementation and against the generic kernel, with
    lengths around page and tile borders; blocks of 16, 32 and 64 rows come from the head counts."""
    lens = [1, 31, 32, 33, 65, 100]
    got, expect = latent_case(H, dn, dr, dims, rank, page, lens, window, sink, seed=H, dtype=torch.bfloat16, tensor_cores=True)
    plain_kernel, _ = latent_case(H, dn, dr, dims, rank, page, lens, window, sink, seed=H, dtype=torch.bfloat16, tensor_cores=False)
    for a, b, c in zip(got, expect, plain_kernel):
        assert rel(a, b) < 3e-2
        assert rel(a, c) < 2e-2


def test_latent_attention_on_the_tensor_cores_with_the_keys_cut():
    """Few rows over many keys: the key range is cut into chunks that are merged afterwards (a long
    prompt's last portion, then its last token alone), a far key among them; the sink counts once."""
    for first in (1100, 1199):
        got, expect = latent_case(4, 32, 32, 32, 64, 16, [1200, 37], seed=3, dtype=torch.bfloat16, tensor_cores=True,
                                  boost=(0, 1199, 70), first=first)
        assert ops.latent_split_plan([1200 - first], 4, 1200, 64, ops.sm_count(CUDA))[0] > 1
        for a, b in zip(got, expect):
            assert rel(a, b) < 3e-2
        without, _ = latent_case(4, 32, 32, 32, 64, 16, [1200, 37], seed=3, dtype=torch.bfloat16, tensor_cores=True,
                                 boost=(0, 1199, 70), first=first, sink=False)
        assert rel(without[0], expect[0]) > 3e-2


# ---- the engine ------------------------------------------------------------------------------


def engine_for(name, dtype="float32", page=4, tokens=1024, requests=4, graphs=True, seed=0, raw=None):
    raw = raw or fc.config(name)
    weights = fc.tensors(raw, seed)
    engine = Engine.from_tensors(raw, weights, EngineArgs(dtype=dtype, page_size=page, cache_tokens=tokens,
                                                          max_requests=requests, cuda_graphs=graphs))
    return raw, weights, engine


TOLERANCE = {"float32": 3e-4, "bfloat16": 6e-2}


def test_engine_with_tensor_core_latent_attention(tmp_path):
    """Sizes at which bfloat16 latent attention runs on the tensor cores: whole, in portions, decoded
    from captured steps, two requests side by side, against the plain implementation."""
    raw = fc.config("Y")
    raw["width"] = 128
    raw["layers"][1]["mixer"].update(heads=6, dim=32, rot_dim=32, kv_rank=64, vdim=24, rot={"base": 1000.0, "dims": 32})
    raw["layers"].append(fc.config("X")["layers"][1])
    raw, weights, engine = engine_for("Y", "bfloat16", page=16, tokens=1024, raw=raw)
    ids = {"a": fc.prompt(150, raw["vocab"], 1), "b": fc.prompt(61, raw["vocab"], 2), "c": fc.prompt(20, raw["vocab"], 3)}
    trace = Trace()
    trace.step({"a": ids["a"][:97]})
    trace.step({"a": ids["a"][97:130], "b": ids["b"][:60]})
    for t in range(130, 150):
        portions = {"a": ids["a"][t: t + 1]}
        if t == 130:
            portions["b"] = ids["b"][60:]
        if 132 <= t < 142:  # the same shape ten times over: such mixed steps come to run from a captured graph
            portions["c"] = ids["c"][2 * (t - 132): 2 * (t - 131)]
        trace.step(portions, end=["b"] if t == 130 else ["c"] if t == 141 else [])
    got = trace.run_engine(engine, tmp_path / "out", before_step=lambda e, record: poison_free_pages(e))
    for r in ids:
        positions, logits = stacked(got[r])
        assert rel(logits, plain.forward(raw, weights, ids[r])) < TOLERANCE["bfloat16"], r


@pytest.mark.parametrize("name", ["X", "Y", "Z"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_and_layer_outputs(name, dtype):
    raw, weights, engine = engine_for(name, dtype)
    for n in (1, 2, 3, 41):
        ids = fc.prompt(n, raw["vocab"], n)
        request = engine.cache.open("r")
        got = engine.runner.run([StepEntry(request, ids, list(range(n)))])
        engine.cache.close("r")
        assert rel(got, plain.forward(raw, weights, ids)) < TOLERANCE[dtype], n
    ops.raise_on_error(CUDA)


@pytest.mark.parametrize("name,page", [("X", 4), ("Y", 16), ("Z", 8)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_decoding_and_mixed_batches(tmp_path, name, page, dtype):
    """Five requests over four state slots: prompts read whole, in portions of 2 to 9 tokens and
    token by token, decoded tokens beside portions of other requests, requests that end and whose
    pages and slots the next ones take (free pages are filled with NaN before every step)."""
    raw, weights, engine = engine_for(name, dtype, page=page, tokens=384)
    V = raw["vocab"]
    ids = {r: fc.prompt(n, V, i) for i, (r, n) in enumerate({"a": 70, "b": 33, "c": 2, "d": 58, "e": 60, "f": 17}.items())}
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
    trace.step({"a": take("a", 70), "d": take("d", 58), "e": take("e", 60)}, end=["a", "d", "e"])
    got = trace.run_engine(engine, tmp_path / "out", before_step=lambda e, record: poison_free_pages(e))
    assert not engine.cache.requests
    engine.cache.check()
    for r in ids:
        positions, logits = stacked(got[r])
        assert positions == list(range(len(ids[r])))
        assert rel(logits, plain.forward(raw, weights, ids[r])) < TOLERANCE[dtype], r


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_equals_decoding_token_by_token(dtype):
    """The same prompt whole, and one token a step (captured decode steps, and launched one by one)."""
    for graphs in (True, False):
        raw, weights, engine = engine_for("X", dtype, graphs=graphs)
        ids = fc.prompt(45, raw["vocab"], 77)
        request = engine.cache.open("w")
        whole = engine.runner.run([StepEntry(request, ids, list(range(len(ids))))])
        engine.cache.close("w")
        request = engine.cache.open("t")
        single = torch.cat([engine.runner.run([StepEntry(request, [t], [0])]) for t in ids])
        engine.cache.close("t")
        assert rel(single, whole) < (2e-5 if dtype == "float32" else 4e-2)
        assert rel(single, plain.forward(raw, weights, ids)) < TOLERANCE[dtype]
    ops.raise_on_error(CUDA)


def test_a_far_token_through_the_whole_model():
    """A long prompt whose last token repeats one from far back: decoding from a cache of hundreds of
    rows over many pages stays on the plain implementation, in a batch with a short request."""
    raw, weights, engine = engine_for("Z", "float32", page=16, tokens=1024)
    ids = fc.prompt(700, raw["vocab"], 5)
    ids[-1] = ids[11]
    other = fc.prompt(30, raw["vocab"], 6)
    a, b = engine.cache.open("a"), engine.cache.open("b")
    engine.runner.run([StepEntry(a, ids[:650], [])])
    rows = [engine.runner.run([StepEntry(b, other[:29], []), StepEntry(a, ids[650:699], [48])])]
    rows.append(engine.runner.run([StepEntry(a, ids[699:], [0]), StepEntry(b, other[29:], [0])]))
    expect = plain.forward(raw, weights, ids)
    assert rel(rows[0][0], expect[698]) < TOLERANCE["float32"]
    assert rel(rows[1][0], expect[699]) < TOLERANCE["float32"]
    assert rel(rows[1][1], plain.forward(raw, weights, other)[29]) < TOLERANCE["float32"]


def test_a_window_on_the_latent_cache():
    """The mixer's optional window: keys just inside and just outside it, in a prompt and in decoding."""
    raw = fc.config("Y")
    raw["layers"][1]["mixer"]["window"] = 9
    raw, weights, engine = engine_for("Y", "float32", page=4, raw=raw)
    ids = fc.prompt(40, raw["vocab"], 8)
    request = engine.cache.open("r")
    got = [engine.runner.run([StepEntry(request, ids[:20], list(range(20)))])]
    got += [engine.runner.run([StepEntry(request, [t], [0])]) for t in ids[20:]]
    expect = plain.forward(raw, weights, ids)
    assert rel(torch.cat(got), expect) < TOLERANCE["float32"]
    raw["layers"][1]["mixer"]["window"] = 10
    assert rel(plain.forward(raw, weights, ids), expect) > 1e-3  # one more key would show


def test_greedy_generation_long_decoding_and_the_scheduler(tmp_path):
    """Through `load(...).generate`: the scheduler admits, batches and chunks; greedy ids equal the
    plain implementation's, 200 tokens past a two-token prompt included."""
    raw = fc.config("X")
    weights = fc.tensors(raw, 3)
    folder = tmp_path / "m"
    folder.mkdir()
    save_file({k: (t if t.dim() < 2 else t.to(torch.bfloat16)).contiguous() for k, t in weights.items()},
              str(folder / "model.safetensors"))
    (folder / "config.json").write_text(json.dumps(raw))
    model = load(folder, dtype="float32", page_size=8, cache_tokens=1024, max_requests=4, max_tokens_per_step=16)
    prompts = [fc.prompt(n, raw["vocab"], 20 + n) for n in (2, 5, 23, 40, 9, 31)]
    counts = [200, 12, 12, 12, 12, 12]
    got = [model.generate([p], GenerationOptions(max_tokens=c, stop=()))[0] for p, c in zip(prompts[:1], counts[:1])]
    got += model.generate(prompts[1:], GenerationOptions(max_tokens=12, stop=()))
    for prompt, ids, count in zip(prompts, got, counts):
        assert len(ids) == count
        logits = plain.forward(raw, weights, prompt + ids)[len(prompt) - 1: -1]
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
    from mlx_omnia_b200.weights.random_init import write_random_model

    raw = fc.config("Z")
    folder = write_random_model(tmp_path / "m", raw, seed=4)
    from safetensors.torch import load_file
    weights = {k: v.float() for k, v in load_file(str(folder / "model.safetensors")).items()}
    ids = fc.prompt(90, raw["vocab"], 1)
    trace = Trace()
    trace.step({"p": ids[:50]}, want="last")
    trace.step({"p": ids[50:52], "q": ids[:7]})
    for t in range(52, 90):
        trace.step({"p": ids[t: t + 1]}, end=["p"] if t == 89 else ["q"] if t == 52 else [])
    got = trace.run(folder, "bfloat16", tmp_path / "out", vocab=raw["vocab"])
    expect = plain.forward(raw, weights, ids)
    positions, logits = stacked(got["p"])
    assert positions == [49] + list(range(50, 90))
    assert rel(logits, expect[positions]) < TOLERANCE["bfloat16"]
