"""Dokodra through the engine against the plain implementation of ``plain_dokodra``.

Small configurations with random weights of their own (sizes that differ from layer to layer, head counts
that are no multiple of a warp's rows, several groups in the state-space mixer and its norm, value sizes
unlike key sizes, layers with and without a feed-forward, a layer that reads another layer's latent).
Every mechanism alone as a one-layer model; whole prompts against token-by-token decoding and portions
down to two tokens; unequal requests in one batch; pages and state slots that are freed and used again;
keys that are far away or sit at page and split borders, with inputs made so that one key dominates;
the sink; long decoding; greedy generation through ``Engine.generate`` and the scheduler.
"""

from __future__ import annotations

import copy
import json
import math
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_dokodra as plain

ROOT = Path(__file__).resolve().parent.parent

ATT = {"heads": 5, "dim": 16, "rot_dim": 12, "vdim": 24, "kv_rank": 48, "scale": 0.21, "rot": {"base": 900.0, "dims": 12}}
ATT2 = {"heads": 3, "dim": 24, "rot_dim": 8, "vdim": 40, "kv_rank": 72, "q_rank": 40, "scale": 0.17,
        "rot": {"base": 20000.0, "dims": 8}}
SSM = {"heads": 6, "vdim": 16, "state": 24, "groups": 2, "conv": 3, "norm_groups": 3}
SSM_B = {"heads": 4, "vdim": 48, "state": 80, "groups": 4, "conv": 2, "norm_groups": 1}
FF = {"kind": "dense", "ff": 136, "limit": 0.7}


def config(layers, width=88, vocab=211, scale=1.7, eps=1e-6, cap=12.0):
    return {"architecture": "Dokodra", "width": width, "vocab": vocab, "embedding": {"scale": scale}, "norm": {"eps": eps},
            "logit_softcap": cap, "layers": copy.deepcopy(layers)}


def layer(kind, mixer, mlp=None, **more):
    return {"type": kind, "mixer": {**mixer, **more}, "mlp": mlp}


FULL = config([
    layer("mamba2", SSM, FF),
    layer("latent_attention_2", ATT2),
    layer("latent_attention", ATT, FF),
    layer("mamba2", SSM_B),
    layer("latent_attention", ATT, {"kind": "dense", "ff": 64, "limit": 2.5}, kv_from=2),
    layer("latent_attention_2", ATT2, FF),
])

ALONE = {
    "latent": config([layer("latent_attention", ATT)]),
    "latent_sink_qrank": config([layer("latent_attention_2", ATT2)]),
    "shared_latent": config([layer("latent_attention", ATT), layer("latent_attention", ATT, kv_from=0)]),
    "ssm": config([layer("mamba2", SSM)]),
    "ssm_wide_state": config([layer("mamba2", SSM_B)], width=72),
    "ssm_no_conv_history": config([layer("mamba2", {**SSM, "conv": 1})]),
    "ffn": config([layer("mamba2", {**SSM, "heads": 2, "groups": 1, "norm_groups": 1}, FF)], width=40, cap=0.0),
}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """Model folders written once: config.json and bfloat16 weights from the plain implementation's generator."""
    from edgerag_b200.weights.safetensors_io import write_safetensors

    base = tmp_path_factory.mktemp("dokodra")
    made = {}

    def get(name: str, raw: dict, seed: int = 0):
        if name not in made:
            folder = base / name
            folder.mkdir()
            tensors = plain.random_tensors(raw, seed)
            (folder / "config.json").write_text(json.dumps(raw))
            write_safetensors(folder / "model.safetensors", tensors)
            made[name] = (folder, raw, tensors)
        return made[name]

    return get


def make_engine(folder, dtype, **over):
    from edgerag_b200.engine.engine import Engine, EngineOptions

    opts = dict(dtype=dtype, block_size=16, num_blocks=64, max_batch_size=4, max_step_tokens=512, max_model_len=1 << 20,
                cuda_graphs=False, poison_freed_pages=True)
    opts.update(over)
    return Engine.from_pretrained(folder, EngineOptions(**opts))


def feed(runner, rid, tokens, cuts, start=0):
    """Feed ``tokens[start:]`` of an admitted request in portions; logits at every place, [fed, vocab] on the CPU."""
    from edgerag_b200.engine.step import StepEntry

    rows, pos = [], start
    for c in cuts:
        c = min(c, len(tokens) - pos)
        if c <= 0:
            break
        out = runner.step([StepEntry(rid, tokens=tokens[pos: pos + c], want=list(range(c)))])
        rows.append(out.float().cpu().clone())
        pos += c
    assert pos == len(tokens), "the cuts do not cover the tokens"
    return torch.cat(rows)


def row_errors(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row: rms of the difference (mean taken off) over the rms of the expected row (mean taken off)."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-9)


#: float32: only the order of sums differs from the plain implementation; bfloat16: activations are rounded to 8 bits
#: between the products.  A wrong key, a lost state or a sink left out moves a row by 10 % and more.
BANDS = {"float32": (2e-4, 5e-5), "bfloat16": (6e-2, 2e-2)}


def assert_close(got, want, dtype, what=""):
    e = row_errors(got, want)
    worst, mean = BANDS[dtype]
    assert e.max() <= worst and e.mean() <= mean, f"{what} {dtype}: worst {e.max():.2e} (row {int(e.argmax())}), mean {e.mean():.2e}"


def tokens_for(raw, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, raw["vocab"], (n,), generator=g).tolist()


# --- configuration and plan (CPU) ---------------------------------------------------------------

def test_plan_names_every_tensor_of_the_design():
    from edgerag_b200.config.registry import architecture_of
    from edgerag_b200.models.decoder import DecoderModel

    arch = architecture_of(FULL)
    model = DecoderModel(arch.make_plan(arch.read_config(FULL, "test")), torch.float32, torch.device("cpu"))
    assert {s.name: tuple(s.shape) for s in model.weight_specs()} == plain.tensor_shapes(FULL)
    layout = model.cache_layout
    # two latent geometries -> two page groups; the layer that borrows a latent has no cache layer of its own
    assert sorted((g.head_dim, g.n_layers, g.value_dim) for g in layout.groups) == [(60, 1, 0), (80, 2, 0)]
    assert len([s for s in layout.states if s.name.startswith("ssm@")]) == 2
    assert [c.writes_cache for c in model.schedule] == [True, True, True, True, False, True]


def test_configuration_errors_name_the_key():
    from edgerag_b200.config.model_config import ConfigError
    from edgerag_b200.models.dokodra import DokodraConfig

    bad = config([layer("latent_attention", ATT, kv_from=0)])
    with pytest.raises(ConfigError, match="kv_from"):
        DokodraConfig.from_dict(bad, "t")
    bad = config([layer("sliding", ATT)])
    with pytest.raises(ConfigError, match="unknown layer type"):
        DokodraConfig.from_dict(bad, "t")
    bad = config([layer("mamba2", {k: v for k, v in SSM.items() if k != "state"})])
    with pytest.raises(ConfigError, match="state"):
        DokodraConfig.from_dict(bad, "t")
    bad = config([layer("latent_attention", ATT), layer("latent_attention", {**ATT, "kv_rank": 32}, kv_from=0)])
    with pytest.raises(ConfigError, match="another latent size"):
        DokodraConfig.from_dict(bad, "t")


def test_plain_recurrence_equals_its_quadratic_form():
    """The oracle checked against itself: the token-by-token recurrence of one head equals the masked
    'attention' form  y_t = sum_{s<=t} (C_t . B_s) exp(sum_{s<r<=t} log a_r) dt_s x_s."""
    g = torch.Generator().manual_seed(3)
    T, N, P = 9, 5, 4
    x, B, C = (torch.randn(T, d, generator=g, dtype=torch.float64) for d in (P, N, N))
    dt, a = torch.rand(T, generator=g, dtype=torch.float64), 0.8
    S, rec = torch.zeros(N, P, dtype=torch.float64), []
    for t in range(T):
        S = math.exp(-a * dt[t]) * S + dt[t] * torch.outer(B[t], x[t])
        rec.append(S.T @ C[t])
    quad = []
    for t in range(T):
        quad.append(sum((C[t] @ B[s]) * math.exp(-a * float(dt[s + 1: t + 1].sum())) * dt[s] * x[s] for s in range(t + 1)))
    assert torch.allclose(torch.stack(rec), torch.stack(quad), atol=1e-12)


def test_plain_sink_is_a_key_without_a_value():
    """The oracle's sink equals an extra key of that logit whose value is zero."""
    g = torch.Generator().manual_seed(4)
    s, v, sink = torch.randn(7, generator=g).double(), torch.randn(7, 3, generator=g).double(), torch.tensor(0.4).double()
    with_sink = (torch.exp(s - s.max()) / (torch.exp(s - s.max()).sum() + torch.exp(sink - s.max()))) @ v
    extra = torch.softmax(torch.cat([s, sink[None]]), 0) @ torch.cat([v, torch.zeros(1, 3).double()])
    assert torch.allclose(with_sink, extra, atol=1e-12)


# --- every mechanism alone ------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_one_mechanism_alone(name, dtype, folders):
    folder, raw, tensors = folders(name, ALONE[name], seed=11)
    toks = tokens_for(raw, 45, 5)
    want = plain.forward(raw, tensors, toks)
    eng = make_engine(folder, dtype)
    eng.runner.admit("a")
    whole = feed(eng.runner, "a", toks, [45])
    eng.runner.release("a")
    assert_close(whole, want, dtype, f"{name} whole")
    eng.runner.admit("b")
    cut = feed(eng.runner, "b", toks, [17, 2, 1, 1, 16, 3, 1, 1, 1, 2])
    assert_close(cut, want, dtype, f"{name} in portions")


# --- the whole model: prompts, decoding, portions, batches ------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_decoding_and_portions_agree_with_plain(dtype, folders):
    folder, raw, tensors = folders("full", FULL, seed=1)
    toks = tokens_for(raw, 150, 6)
    want = plain.forward(raw, tensors, toks)
    eng = make_engine(folder, dtype)
    r = eng.runner
    for rid, cuts in (("whole", [150]), ("decode", [40] + [1] * 110), ("chunks", [2, 31, 2, 16, 15, 1, 2, 33, 3, 2, 2, 17] + [1] * 30),
                      ("pairs", [2] * 75)):
        r.admit(rid)
        got = feed(r, rid, toks, cuts)
        r.release(rid)
        assert_close(got, want, dtype, rid)
        eng.cache.check_invariants()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_equal_each_alone(dtype, folders):
    """Portions of some requests beside single tokens of others; a request pauses for a step; requests end and
    their pages and state slots go to new ones (four slots, six requests, freed pages poisoned)."""
    from edgerag_b200.engine.step import StepEntry

    folder, raw, tensors = folders("full", FULL, seed=1)
    lens = {"a": 70, "b": 33, "c": 1, "d": 90, "e": 18, "f": 47}
    toks = {k: tokens_for(raw, n, 20 + i) for i, (k, n) in enumerate(lens.items())}
    want = {k: plain.forward(raw, tensors, t) for k, t in toks.items()}
    eng = make_engine(folder, dtype, num_blocks=14)       # 224 tokens of pages: never room for all at once
    r = eng.runner
    plan = [  # (request, tokens) per step
        [("a", 30), ("b", 2)], [("a", 1), ("b", 16), ("c", 1)], [("a", 17), ("b", 1)], [("b", 14), ("d", 40), ("a", 1)],
        [("a", 21), ("d", 1)], [("d", 33), ("e", 2)], [("d", 16), ("e", 1), ("f", 3)], [("e", 15), ("f", 1)], [("f", 43)],
    ]
    fed = {k: 0 for k in lens}
    got = {k: [] for k in lens}
    for step in plan:
        entries = []
        for rid, n in step:
            if fed[rid] == 0:
                r.admit(rid)
            entries.append(StepEntry(rid, tokens=toks[rid][fed[rid]: fed[rid] + n], want=list(range(n))))
        out = r.step(entries).float().cpu()
        row = 0
        for rid, n in step:
            got[rid].append(out[row: row + n].clone())
            row += n
            fed[rid] += n
            if fed[rid] == lens[rid]:
                r.release(rid)
        eng.cache.check_invariants()
    assert fed == lens
    for rid in lens:
        assert_close(torch.cat(got[rid]), want[rid], dtype, f"request {rid}")


@pytest.mark.gpu
def test_a_slot_used_again_starts_from_nothing(folders):
    """One state slot: the second request gets the first one's slot and must not see its state or its
    convolution history (float32, so that a leak of any size shows)."""
    folder, raw, tensors = folders("ssm", ALONE["ssm"], seed=11)
    eng = make_engine(folder, "float32", max_batch_size=1, num_blocks=8)
    for seed in (1, 2, 3):
        toks = tokens_for(raw, 37, seed)
        eng.runner.admit("only")
        got = feed(eng.runner, "only", toks, [5, 1, 31])
        eng.runner.release("only")
        assert_close(got, plain.forward(raw, tensors, toks), "float32", f"request {seed} in the one slot")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, folders):
    folder, raw, tensors = folders("full", FULL, seed=1)
    toks = tokens_for(raw, 330, 9)
    want = plain.forward(raw, tensors, toks)
    eng = make_engine(folder, dtype)
    eng.runner.admit("long")
    got = feed(eng.runner, "long", toks, [3] + [1] * 327)
    assert_close(got, want, dtype, "330 tokens, 327 of them one by one")


# --- kernels with inputs made so that a fault shows ---------------------------------------------------

def _latent_reference(q_lat, rows, positions_of, scale, rank, sink=None, gate=None):
    """Plain attention over cache rows: q_lat [n, H, dk] float64, rows[seq] [len, dk]; -> [n, H, rank]."""
    out = torch.zeros(q_lat.shape[0], q_lat.shape[1], rank, dtype=torch.float64)
    for t, (seq, pos) in enumerate(positions_of):
        keys = rows[seq][: pos + 1]
        for h in range(q_lat.shape[1]):
            s = keys @ q_lat[t, h] * scale
            top = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - top)
            den = e.sum() + (torch.exp(sink[h] - top) if sink is not None else 0.0)
            out[t, h] = (e / den) @ keys[:, :rank]
            if gate is not None:
                out[t, h] *= torch.sigmoid(gate[t, h])
    return out


def _paged(rows, page_size, dtype, shuffle_seed=0):
    """Scatter each sequence's rows over shuffled pages; (pages [P, 1, page_size, dk], block tables)."""
    dk = rows[0].shape[1]
    need = [-(-r.shape[0] // page_size) for r in rows]
    order = torch.randperm(sum(need) + 3, generator=torch.Generator().manual_seed(shuffle_seed)).tolist()
    pages = torch.full((sum(need) + 3, 1, page_size, dk), float("nan"), dtype=torch.float64)
    tables = torch.zeros(len(rows), max(need), dtype=torch.int32)
    for s, r in enumerate(rows):
        for i in range(need[s]):
            page = order.pop()
            tables[s, i] = page
            chunk = r[i * page_size: (i + 1) * page_size]
            pages[page, 0, : chunk.shape[0]] = chunk
    return pages.to(dtype).cuda(), tables.cuda()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_splits,split_keys", [(1, 0), (5, 192), (13, 64)])
def test_latent_attention_finds_one_far_key(dtype, n_splits, split_keys):
    """Among 800 keys one is made to match the query (scaled so that its score stands out by far): the result
    must be that key's latent, wherever it sits: the first tokens, either side of a page border, either
    side of a split border, the last visible key, and never the key just behind the query's position."""
    from edgerag_b200.ops import kernels

    H, rank, rot, L = 3, 40, 8, 800
    dk = rank + rot
    g = torch.Generator().manual_seed(7)
    rows = [torch.randn(L, dk, generator=g, dtype=torch.float64).to(dtype).double()]
    targets = [0, 1, 15, 16, 17, 63, 64, 191, 192, 193, 400, 767, 768, 798]
    pos = 798
    q = torch.zeros(len(targets) + 1, H, dk, dtype=torch.float64)
    for t, j in enumerate(targets):
        for h in range(H):
            q[t, h] = rows[0][j] * (40.0 + h)
    q[-1] = rows[0][799] * 40.0           # aims at the key one past the position: must not be found
    n = q.shape[0]
    pages, tables = _paged(rows, 16, dtype)
    positions = torch.full((n,), pos, dtype=torch.int32).cuda()
    seq_of = torch.zeros(n, dtype=torch.int32).cuda()
    out = torch.zeros(n, H, rank, dtype=dtype).cuda()
    part = torch.zeros(max(1, kernels.latent_scratch_floats(n, H, rank, n_splits)), dtype=torch.float32).cuda()
    kernels.latent_attention(q.float().cuda(), pages, tables, seq_of, positions, out, 1.0, 0, n,
                             split_keys=split_keys, n_splits=n_splits, part=part if n_splits > 1 else None)
    got = out.double().cpu()
    want = _latent_reference(q, rows, [(0, pos)] * n, 1.0, rank)
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert torch.allclose(got, want, atol=tol, rtol=tol)
    for t, j in enumerate(targets):
        assert torch.allclose(got[t, 0], rows[0][j, :rank], atol=tol, rtol=tol), f"key {j} was not the one found"
    assert not torch.allclose(got[-1, 0], rows[0][799, :rank], atol=0.2), "a key behind the query's position was seen"


@pytest.mark.gpu
@pytest.mark.parametrize("heads,rank,rot", [(5, 40, 8), (16, 128, 16), (3, 72, 24), (20, 64, 0)])
def test_latent_attention_on_tensor_cores(heads, rank, rot):
    """The tensor-core form against the plain one: single tokens of three sequences (in splits of 64 and 128 keys
    and unsplit) and portions of two others whose 16- and 32-row blocks straddle tokens, with sink and gate;
    one query aims at a far key, one at the key at a split's edge, one at a key just behind its position."""
    from edgerag_b200.ops import kernels

    dk = rank + rot
    g = torch.Generator().manual_seed(9)
    lens = [1, 64, 701, 137, 3]                       # cached tokens per sequence, this step's included
    new = [1, 1, 1, 37, 3]                            # tokens of this step: three single ones, two portions
    rows = [torch.randn(n, dk, generator=g, dtype=torch.float64).to(torch.bfloat16).double() for n in lens]
    where = [(s, lens[s] - new[s] + i) for s in range(5) for i in range(new[s])]
    n = len(where)
    q = torch.randn(n, heads, dk, generator=g, dtype=torch.float64) * dk ** -0.5
    q[2, 0] = rows[2][5] * 30.0                        # a far key among 700
    q[2, 1] = rows[2][639] * 30.0                      # the last key of a split of 128
    q[2, 2] = rows[2][640] * 30.0                      # the first key of the next
    q[5, 0] = rows[3][lens[3] - new[3] + 3] * 0.3      # third token of the portion aims one key ahead of itself (softly: what it does see stays well-conditioned)
    q = q.float().double()
    sink = torch.randn(heads, generator=g, dtype=torch.float64)
    gate = torch.randn(n, heads, generator=g).to(torch.bfloat16).double()
    pages, tables = _paged(rows, 16, torch.bfloat16, shuffle_seed=3)
    starts = torch.tensor([0, 1, 2, 3, 40, 43], dtype=torch.int32).cuda()
    positions = torch.tensor([p for _, p in where], dtype=torch.int32).cuda()
    want = _latent_reference(q, rows, where, 0.9, rank, sink=sink, gate=gate)
    mt = 1 if heads <= 16 else 2
    for n_splits, split in ((1, 0), (6, 128), (11, 64)):
        out = torch.zeros(n, heads, rank, dtype=torch.bfloat16).cuda()
        part = torch.zeros(max(1, kernels.latent_scratch_floats(3, heads, rank, n_splits))).cuda()
        kernels.latent_attention_mma(q.float().cuda(), pages, tables, starts, positions, out, 0.9, 0, 3, 0, 3,
                                     kernels.latent_mma_tiles([1, 1, 1], heads, mt), mt, gate=gate.to(torch.bfloat16).cuda(),
                                     sink=sink.float().cuda(), split_keys=split, n_splits=n_splits, part=part if n_splits > 1 else None)
        kernels.latent_attention_mma(q.float().cuda(), pages, tables, starts, positions, out, 0.9, 3, 2, 3, 40,
                                     kernels.latent_mma_tiles([37, 3], heads, 2), 2, gate=gate.to(torch.bfloat16).cuda(),
                                     sink=sink.float().cuda())
        got = out.double().cpu()
        assert torch.allclose(got, want, atol=2e-2, rtol=3e-2), f"{n_splits} splits: {(got - want).abs().max():.3f}"
    assert torch.allclose(want[2, 0], rows[2][5, :rank] * torch.sigmoid(gate[2, 0]), atol=1e-3)
    assert not torch.allclose(want[5, 0], rows[3][lens[3] - new[3] + 3, :rank] * torch.sigmoid(gate[5, 0]), atol=0.2)


@pytest.mark.gpu
@pytest.mark.parametrize("n_splits,split_keys", [(1, 0), (3, 64)])
def test_latent_attention_sink_and_gate(n_splits, split_keys):
    """A sink far above every score takes almost the whole denominator, one far below changes nothing; the gate
    multiplies per head.  Two sequences of unequal length, tokens of both in one call."""
    from edgerag_b200.ops import kernels

    H, rank, rot = 4, 24, 4
    g = torch.Generator().manual_seed(8)
    rows = [torch.randn(n, rank + rot, generator=g, dtype=torch.float64) for n in (130, 19)]
    where = [(0, 129), (1, 18), (0, 64), (1, 0), (0, 5)]
    n = len(where)
    q = torch.randn(n, H, rank + rot, generator=g, dtype=torch.float64)
    sink = torch.tensor([30.0, -30.0, 0.3, 2.0], dtype=torch.float64)
    gate = torch.randn(n, H, generator=g, dtype=torch.float64)
    pages, tables = _paged(rows, 8, torch.float32, shuffle_seed=2)
    out = torch.zeros(n, H, rank).cuda()
    part = torch.zeros(max(1, kernels.latent_scratch_floats(n, H, rank, n_splits))).cuda()
    kernels.latent_attention(q.float().cuda(), pages, tables, torch.tensor([s for s, _ in where], dtype=torch.int32).cuda(),
                             torch.tensor([p for _, p in where], dtype=torch.int32).cuda(), out, 0.3, 0, n,
                             gate=gate.float().cuda(), sink=sink.float().cuda(), split_keys=split_keys, n_splits=n_splits,
                             part=part if n_splits > 1 else None)
    want = _latent_reference(q, rows, where, 0.3, rank, sink=sink, gate=gate)
    assert torch.allclose(out.double().cpu(), want, atol=2e-5, rtol=2e-4)
    no_sink = _latent_reference(q, rows, where, 0.3, rank, gate=gate)
    assert want[:, 0].abs().max() < 1e-6 * no_sink[:, 0].abs().max() + 1e-9      # head 0: swallowed by its sink
    assert torch.allclose(want[:, 1], no_sink[:, 1], atol=1e-9)                 # head 1: the sink is nothing


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,P,N,G", [(4, 24, 20, 2), (4, 32, 32, 2), (2, 16, 48, 1), (2, 64, 128, 2)])
def test_scan_carries_state_over_any_cut(dtype, H, P, N, G):
    """The recurrence kernel over 70 tokens at once equals the same tokens in portions of 1, 2, 15, 16, 17 and 19
    (the kernel stages 16 tokens at a time) through a state slot, for two requests with swapped slots."""
    from edgerag_b200.ops import kernels

    inner, ch = H * P, H * P + 2 * G * N
    hd, gr = H - 1, G - 1                            # the head (of the last group) that is checked against the plain loop
    g = torch.Generator().manual_seed(5)
    T = 70
    xbc = (torch.randn(2 * T, ch, generator=g) * 0.5).to(dtype).cuda()
    proj = torch.randn(2 * T, 8, generator=g).to(dtype).cuda()              # the raw step sizes sit in columns 2 .. 2 + H
    dt_bias, a_log, d_skip = (torch.randn(H, generator=g).cuda() for _ in range(3))

    def run(cuts):
        state = torch.zeros(3, H, N, P).cuda()
        y = torch.zeros(2 * T, inner).cuda()
        at = 0
        for c in cuts:
            rows = torch.cat([torch.arange(at, at + c), torch.arange(T + at, T + at + c)]).cuda()
            yy = torch.zeros(2 * c, inner).cuda()
            kernels.ssm_scan(xbc[rows].contiguous(), proj[rows].contiguous(), 2, dt_bias, a_log, d_skip, state, 2,
                             torch.tensor([0, c, 2 * c], dtype=torch.int32).cuda(), torch.tensor([2, 0], dtype=torch.int32).cuda(),
                             yy, G)
            y[rows] = yy
            at += c
        return y, state

    y_whole, s_whole = run([T])
    y_cut, s_cut = run([1, 2, 15, 16, 17, 19])
    assert torch.allclose(y_whole, y_cut, atol=1e-5, rtol=1e-5) and torch.allclose(s_whole, s_cut, atol=1e-5, rtol=1e-5)
    assert s_whole[1].abs().max() == 0                                        # the slot nobody holds stays untouched
    # against the plain recurrence: request 0 (slot 2), the last head, which belongs to the last group
    x64 = xbc[:T].double().cpu()
    dt = torch.nn.functional.softplus(proj[:T, 2 + hd].double().cpu() + dt_bias[hd].double().cpu())
    S = torch.zeros(N, P, dtype=torch.float64)
    for t in range(T):
        x_t = x64[t, hd * P: (hd + 1) * P]
        S = torch.exp(-torch.exp(a_log[hd].double().cpu()) * dt[t]) * S + dt[t] * torch.outer(
            x64[t, inner + gr * N: inner + (gr + 1) * N], x_t)
        y_t = S.T @ x64[t, inner + G * N + gr * N: inner + G * N + (gr + 1) * N] + d_skip[hd].double().cpu() * x_t
        assert torch.allclose(y_whole[t, hd * P: (hd + 1) * P].double().cpu(), y_t, atol=1e-4, rtol=1e-4)
    assert torch.allclose(s_whole[2, hd].double().cpu(), S, atol=1e-4, rtol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bounded_gate_softcap_and_offset_norm_kernels(dtype):
    from edgerag_b200.ops import kernels

    g = torch.Generator().manual_seed(6)
    gu = (torch.randn(7, 2 * 50, generator=g) * 2).to(dtype).cuda()
    act = torch.zeros(7, 50, dtype=dtype).cuda()
    kernels.glu_bounded(gu, act, limit=0.9, alpha=1.702, shift=1.0)
    gg, uu = gu[:, :50].double().clamp(max=0.9), gu[:, 50:].double().clamp(-0.9, 0.9)
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    assert torch.allclose(act.double(), gg * torch.sigmoid(1.702 * gg) * (uu + 1.0), atol=tol, rtol=tol)
    assert (gu[:, :50] > 0.9).any() and (gu[:, 50:] < -0.9).any()             # the bounds were in play

    logits = (torch.randn(5, 37, generator=g) * 40).cuda()
    capped = logits.clone()
    kernels.softcap(capped, 25.0, dtype)
    assert torch.allclose(capped.double(), 25.0 * torch.tanh(logits.double() / 25.0), atol=1e-4)

    hidden = torch.randn(6, 52, generator=g).cuda()
    w = (torch.randn(52, generator=g) * 0.2).cuda()
    out = torch.zeros(6, 52, dtype=dtype).cuda()
    kernels.add_rmsnorm(hidden, w + 1.0, out, 1e-3, exact=True)
    want = plain.offset_norm(hidden.double().cpu(), w.double().cpu(), 1e-3)
    assert torch.allclose(out.double().cpu(), want, atol=1e-5 if dtype == torch.float32 else 2e-2, rtol=tol)

    y = torch.randn(4, 48, generator=g).cuda()
    z = torch.randn(4, 48, generator=g).to(dtype).cuda()
    nw = torch.rand(48, generator=g).cuda()
    normed = torch.zeros(4, 48, dtype=dtype).cuda()
    kernels.gated_group_norm(y, nw, normed, 1e-4, parts=3, gate=z)
    v = (y.double() * plain.silu(z.double())).cpu().reshape(4, 3, 16)
    want = plain.unit_rms(v, 1e-4).reshape(4, 48) * nw.double().cpu()
    assert torch.allclose(normed.double().cpu(), want, atol=1e-5 if dtype == torch.float32 else 2e-2, rtol=tol)


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [1, 5, 16])
def test_bounded_gate_in_the_product_equals_the_two_kernels(rows):
    """The few-rows product with the bounded gate in its epilogue gives the bits of the product followed by the gate kernel."""
    from edgerag_b200.ops import kernels

    g = torch.Generator().manual_seed(12)
    x = torch.randn(rows, 96, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(2 * 72, 96, generator=g) * 0.3).to(torch.bfloat16).cuda()
    assert kernels.linear_glu_supported(x, w)
    fused = torch.zeros(rows, 72, dtype=torch.bfloat16).cuda()
    kernels.linear_glu(x, w, fused, bounded=(0.8, 1.702, 1.0))
    gate_up = torch.zeros(rows, 144, dtype=torch.bfloat16).cuda()
    kernels.linear(x, w, gate_up)
    two = torch.zeros(rows, 72, dtype=torch.bfloat16).cuda()
    kernels.glu_bounded(gate_up, two, 0.8, 1.702, 1.0)
    assert torch.equal(fused, two)
    assert (gate_up[:, :72].float() > 0.8).any()


# --- generation through the engine's own entry point -----------------------------------------------

def plain_greedy(raw, tensors, prompt, n_new):
    """(tokens, top-2 margin at every step) of greedy decoding with the plain implementation."""
    toks, margins = list(prompt), []
    for _ in range(n_new):
        last = plain.forward(raw, tensors, toks)[-1]
        top = torch.topk(last, 2).values
        margins.append(float(top[0] - top[1]))
        toks.append(int(last.argmax()))
    return toks[len(prompt):], margins


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,graphs", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
def test_greedy_generation_through_the_scheduler(dtype, graphs, folders):
    """Five prompts through ``Engine.generate`` with two state slots and portions of 8 tokens: the scheduler
    cuts prompts, batches them with decoding requests and hands slots and pages on.  Tokens equal the plain
    implementation's up to the first step whose top-2 margin is too small to tell."""
    from edgerag_b200.sampling.params import SamplingParams

    folder, raw, tensors = folders("full", FULL, seed=1)
    prompts = [tokens_for(raw, n, 40 + n) for n in (21, 3, 34, 9, 1)]
    eng = make_engine(folder, dtype, max_batch_size=2, num_blocks=6, chunk_size=8, max_step_tokens=None, cuda_graphs=graphs)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=12))
    eng.cache.check_invariants()
    assert eng.cache.free_pages() == [6] * len(eng.cache.layout.groups) and not eng.cache.requests
    compared = 0
    for prompt, got in zip(prompts, outs):
        want, margins = plain_greedy(raw, tensors, prompt, 12)
        assert len(got) == 12
        clear = next((i for i, m in enumerate(margins) if m < (1e-3 if dtype == "float32" else 0.08)), 12)
        assert list(got[:clear]) == want[:clear], f"prompt of {len(prompt)} tokens"
        compared += clear
    # (bfloat16 moves a logit by about 0.02 here, and few steps of a random model have a clearer margin than 0.08)
    assert compared >= (20 if dtype == "float32" else 5), "the margins left too little to compare"


@pytest.mark.gpu
def test_trace_replay_program(folders, tmp_path):
    """bin/trace_run on a Dokodra folder: two requests in mixed steps, logits against the plain implementation."""
    folder, raw, tensors = folders("full", FULL, seed=1)
    a, b = tokens_for(raw, 40, 1), tokens_for(raw, 9, 2)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]}, {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[8:], "want": [0]}, {"id": "a", "tokens": a[31:], "want": [8]}], "end": ["a", "b"]},
    ]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb = plain.forward(raw, tensors, a), plain.forward(raw, tensors, b)
    V = raw["vocab"]
    got = [torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)) for i in range(3)]
    assert_close(got[0], wa[[0, 29]], "float32", "step 0")
    assert_close(got[1], torch.stack([wa[30], wb[7]]), "float32", "step 1")
    assert_close(got[2], torch.stack([wb[8], wa[39]]), "float32", "step 2")


@pytest.mark.gpu
def test_command_line_with_random_weights(tmp_path):
    """``python -m edgerag_b200`` on a Dokodra configuration: seeded random weights written as a model folder, the
    folder loaded again, a few greedy tokens for two prompts; the same tokens when the folder is given as --model."""
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(FULL))
    base = [sys.executable, "-m", "edgerag_b200", "--dtype", "fp32", "--num-blocks", "16", "--max-batch-size", "2", "--chunk-size", "16",
            "--max-new-tokens", "5", "--prompt-ids", "3,1,4,1,5,9,2,6", "--prompt-ids", "7", "--json"]
    first = subprocess.run(base + ["--random-weights", "3", "--config", str(cfg), "--save-model", str(tmp_path / "m"), "--weights-std", "0.1"],
                           capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert first.returncode == 0, first.stderr[-2000:]
    again = subprocess.run(base + ["--model", str(tmp_path / "m")], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert again.returncode == 0, again.stderr[-2000:]
    a, b = (json.loads(p.stdout.strip().splitlines()[-1])["outputs"] for p in (first, again))
    assert [len(o["token_ids"]) for o in a] == [5, 5] and a == b
