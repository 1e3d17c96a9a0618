"""Vokusun through the engine against the plain implementation of ``plain_vokusun``.

Small configurations with random weights of their own: head counts, head sizes, windows, kept first tokens,
rotated widths, scaling factors, latent sizes and looped runs that differ from layer to layer and from test
to test (also the degenerate ones: one key/value head, as many as query heads, full rotation, no scaling, no
mask, a loop over one layer, a loop that starts at the first or ends at the last layer, layers without a
feed-forward).  Every mechanism alone; whole prompts against token-by-token decoding and portions down to two
tokens; unequal requests in one batch with pages and slots that are freed, poisoned and used again; keys made
dominant just inside and just outside the window, at the last kept and the first not kept position, at page
borders and far away; long decoding; greedy generation through ``Engine.generate`` and the scheduler; the
trace replay program.
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

import plain_vokusun as plain

ROOT = Path(__file__).resolve().parent.parent

ATT = plain.attention_layer(heads=6, kv_heads=2, dim=32, rot_dims=12, size=21, keep_first=5, factor=4.0, base=700.0, ff=88, scale=0.3)
ATT_B = plain.attention_layer(heads=3, kv_heads=3, dim=48, rot_dims=48, size=40, keep_first=0, factor=1.0, base=50000.0, ff=None)
ATT_C = plain.attention_layer(heads=4, kv_heads=1, dim=16, rot_dims=8, size=17, keep_first=18, factor=1.5, base=10000.0, ff=40)
LAT = plain.latent_layer(heads=5, dim=16, rot_dim=12, vdim=24, kv_rank=40, base=900.0, ff=72, scale=0.21)
LAT_B = plain.latent_layer(heads=2, dim=24, rot_dim=8, vdim=16, kv_rank=56, base=30000.0, ff=None)

FULL = plain.make_config([ATT_C, LAT, ATT, ATT_B, LAT_B, ATT], width=80, vocab=203, eps=1e-5, loop={"start": 1, "stop": 4, "times": 3})


def no_mask(layer):
    out = copy.deepcopy(layer)
    del out["mixer"]["mask"]
    del out["mixer"]["rot"]["scaling"]
    return out


ALONE = {
    "window": plain.make_config([ATT]),
    "window_all_kv_heads_full_rotation": plain.make_config([ATT_B], width=72),
    "window_shorter_than_the_kept": plain.make_config([ATT_C], width=48),
    "no_mask_no_scaling": plain.make_config([no_mask(ATT)]),
    "latent": plain.make_config([LAT]),
    "latent_without_ffn": plain.make_config([LAT_B], width=56),
    "loop_of_one_layer": plain.make_config([ATT_C], width=48, loop={"start": 0, "stop": 1, "times": 3}),
    "loop_once_at_the_end": plain.make_config([LAT_B, ATT_C], width=56, loop={"start": 1, "stop": 2, "times": 1}),
}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from edgerag_b200.weights.safetensors_io import write_safetensors

    base = tmp_path_factory.mktemp("vokusun")
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
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean(-1).sqrt().clamp_min(1e-9)


#: float32: only the order of sums differs from the plain implementation; bfloat16: activations are rounded to 8 bits
#: between the products.  A wrong key, a window off by one or a lost kept token moves a row by 10 % and more.
BANDS = {"float32": (2e-4, 5e-5), "bfloat16": (6e-2, 2e-2)}


def assert_close(got, want, dtype, what=""):
    assert torch.isfinite(got).all(), f"{what} {dtype}: non-finite logits"
    e = row_errors(got, want)
    worst, mean = BANDS[dtype]
    assert e.max() <= worst and e.mean() <= mean, f"{what} {dtype}: worst {e.max():.2e} (row {int(e.argmax())}), mean {e.mean():.2e}"


def tokens_for(raw, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, raw["vocab"], (n,), generator=g).tolist()


# --- configuration, plan, cache bookkeeping (CPU) ---------------------------------------------------

def test_plan_names_every_tensor_and_gives_each_pass_a_cache():
    from edgerag_b200.config.registry import architecture_of
    from edgerag_b200.models.decoder import DecoderModel
    from edgerag_b200.parts.base import LayerCall, StreamCall

    arch = architecture_of(FULL)
    cfg = arch.read_config(FULL, "test")
    model = DecoderModel(arch.make_plan(cfg), torch.float32, torch.device("cpu"))
    assert {s.name: tuple(s.shape) for s in model.weight_specs()} == plain.tensor_shapes(FULL)
    runs = [c.layer for c in model.schedule if isinstance(c, LayerCall)]
    assert runs == [i for i, _ in plain.run_order(FULL)] == [0, 1, 2, 3, 1, 2, 3, 1, 2, 3, 4, 5]
    assert [c.cache_layer for c in model.schedule if isinstance(c, LayerCall)] == list(range(12))
    enters = [(i, c.index) for i, c in enumerate(model.schedule) if isinstance(c, StreamCall)]
    assert enters == [(1, 0), (5, 1), (9, 2)]
    groups = {(g.n_kv_heads, g.head_dim, g.window, g.keep_first, g.value_dim): g.n_layers for g in model.cache_layout.groups}
    assert groups == {(1, 16, 17, 18, 16): 1, (1, 52, 0, 0, 0): 3, (2, 32, 21, 5, 32): 4, (3, 48, 40, 0, 48): 3, (1, 64, 0, 0, 0): 1}
    assert model.graph_safe


def test_configuration_errors_name_the_key():
    from edgerag_b200.config.model_config import ConfigError
    from edgerag_b200.models.vokusun import VokusunConfig

    def broken(change):
        raw = copy.deepcopy(ALONE["window"])
        change(raw)
        return raw

    cases = [
        (lambda r: r["layers"][0].update(type="sliding"), "unknown layer type"),
        (lambda r: r["layers"][0]["mixer"].pop("kv_heads"), "kv_heads"),
        (lambda r: r["layers"][0]["mixer"].update(kv_heads=4), "kv_heads must divide"),
        (lambda r: r["layers"][0]["mixer"].update(vdim=8), "vdim"),
        (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=34), "rot.dims"),
        (lambda r: r["layers"][0]["mixer"]["mask"].pop("size"), "size"),
        (lambda r: r.update(loop={"start": 0, "stop": 2, "times": 2}), "loop"),
        (lambda r: r.update(loop={"start": 0, "stop": 1}), "times"),
        (lambda r: r["layers"][0]["mlp"].update(kind="routed"), "mlp.kind"),
        (lambda r: r.pop("norm"), "norm"),
    ]
    for change, word in cases:
        with pytest.raises(ConfigError, match=word):
            VokusunConfig.from_dict(broken(change), "t")


def test_plain_mask_against_its_definition():
    """The oracle checked against itself, entry by entry, and at the window's and the kept tokens' edges."""
    T, size, keep = 40, 7, 3
    m = plain.visible(T, size, keep)
    for i in range(T):
        for j in range(T):
            assert bool(m[i, j]) == (j <= i and (i - j < size or j < keep))
    assert m[30, 24] and not m[30, 23] and m[30, 2] and not m[30, 3]
    assert plain.visible(9, None).equal(torch.tril(torch.ones(9, 9, dtype=torch.bool)))


def test_plain_turn_is_a_rotation_of_pairs_with_scaled_positions():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 2, 10, generator=g, dtype=torch.float64)
    pos = torch.tensor([0, 3, 8, 21, 400])
    y = plain.turn_pairs(x, pos, 100.0, 6, factor=2.0)
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.equal(y[0], x[0])
    assert torch.allclose(y[..., :6].pow(2).sum(-1), x[..., :6].pow(2).sum(-1))
    a = 21 * 100.0 ** (-2.0 / 6) / 2.0                          # pair 1 of the token at position 21
    assert torch.allclose(y[3, 1, 2], x[3, 1, 2] * math.cos(a) - x[3, 1, 3] * math.sin(a))
    assert torch.allclose(y[3, 1, 3], x[3, 1, 3] * math.cos(a) + x[3, 1, 2] * math.sin(a))
    # a turned query times a turned key depends on the distance only
    q, k = torch.randn(1, 6, generator=g, dtype=torch.float64), torch.randn(1, 6, generator=g, dtype=torch.float64)
    dot = lambda i, j: float(plain.turn_pairs(q, torch.tensor([i]), 100.0, 6, 2.0)[0] @ plain.turn_pairs(k, torch.tensor([j]), 100.0, 6, 2.0)[0])  # noqa: E731
    assert abs(dot(9, 4) - dot(105, 100)) < 1e-9


def test_pages_of_kept_tokens_outlive_the_window():
    from edgerag_b200.cache.manager import NO_PAGE, CacheLayout, CacheManager, KVGroupSpec

    layout = CacheLayout(groups=[KVGroupSpec(1, 1, 8, window=10, keep_first=5), KVGroupSpec(1, 1, 8, window=10),
                                 KVGroupSpec(1, 1, 8)], placement=[(0, 0), (1, 0), (2, 0)])
    cm = CacheManager(layout, page_size=4, num_pages=40, max_requests=2)
    cm.admit("r")
    for n in (3, 1, 9, 1, 1, 30, 2):
        cm.grow("r", n)
        cm.advance("r", n)
        cm.check_invariants()
    total = 47
    kept, plain_window, everything = (t.pages for t in cm.requests["r"].tables)
    dead = [i for i in range(len(kept)) if (i + 1) * 4 - 1 <= total - 10]
    assert [i for i, p in enumerate(plain_window) if p == NO_PAGE] == dead
    assert [i for i, p in enumerate(kept) if p == NO_PAGE] == [i for i in dead if i >= 2]     # pages 0, 1 hold tokens 0..4
    assert NO_PAGE not in everything
    assert cm.held_pages("r") == [len(kept) - len(dead) + 2, len(kept) - len(dead), len(kept)]
    cm.release("r")
    cm.check_invariants()
    assert cm.free_pages() == [40, 40, 40]


# --- every mechanism alone ------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALONE))
def test_one_mechanism_alone(name, dtype, folders):
    folder, raw, tensors = folders(name, ALONE[name], seed=11)
    toks = tokens_for(raw, 75, 5)
    want = plain.forward(raw, tensors, toks)
    eng = make_engine(folder, dtype)
    eng.runner.admit("a")
    whole = feed(eng.runner, "a", toks, [75])
    eng.runner.release("a")
    assert_close(whole, want, dtype, f"{name} whole")
    eng.runner.admit("b")
    cut = feed(eng.runner, "b", toks, [17, 2, 1, 1, 16, 3, 1, 1, 1, 2, 20, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1])
    assert_close(cut, want, dtype, f"{name} in portions")
    eng.cache.check_invariants()


@pytest.mark.gpu
def test_layers_agree_with_plain_one_by_one(folders):
    """The residual stream after every layer run (float32), with the pending update closed and added."""
    from edgerag_b200.engine.step import StepEntry
    from edgerag_b200.parts.base import StreamCall, settle_update

    folder, raw, tensors = folders("full", FULL, seed=1)
    toks = tokens_for(raw, 50, 2)
    _, want = plain.forward(raw, tensors, toks, return_layers=True)
    eng = make_engine(folder, "float32")
    r, model = eng.runner, eng.model
    r.admit("x")
    ctx, ordered = r.prepare([StepEntry("x", tokens=toks, want=[])])
    hidden = ctx.buf("model.hidden", (len(toks), model.hidden_size), torch.float32)
    model.embedding.forward(ctx, hidden)
    for op in model.stream_ops:
        op.begin(ctx, hidden)
    delta, run = None, 0
    for call in model.schedule:
        if isinstance(call, StreamCall):
            delta = model.stream_ops[call.op].forward(hidden, delta, ctx, call)
            continue
        delta = model.blocks[call.layer].forward(hidden, delta, ctx, call)
        settle_update(hidden, delta, model.dtype)
        delta = None
        err = (hidden.cpu().double() - want[run]).abs().max() / want[run].abs().max()
        assert err < 5e-5, f"layer run {run} (layer {call.layer}): {err:.2e}"
        run += 1
    r.finish(ordered)


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


ATT_64 = plain.attention_layer(heads=4, kv_heads=2, dim=64, rot_dims=24, size=70, keep_first=9, factor=3.0, base=2000.0, ff=64, scale=0.2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_heads_of_64_with_a_prompt_of_many_windows(dtype, folders):
    """Heads of 64 in bfloat16 take the tensor-core kernel for portions: a prompt several windows and key tiles long,
    whole, in portions that end inside tiles, and with decoded tokens behind it."""
    raw = plain.make_config([ATT_64, LAT, ATT_64], width=64, vocab=96, loop={"start": 0, "stop": 2, "times": 2})
    folder, raw, tensors = folders("heads_of_64", raw, seed=3)
    toks = tokens_for(raw, 700, 9)
    want = plain.forward(raw, tensors, toks)
    eng = make_engine(folder, dtype, num_blocks=256, max_step_tokens=1024)
    r = eng.runner
    for rid, cuts in (("whole", [700]), ("portions", [300, 2, 129, 257, 5] + [1] * 7)):
        r.admit(rid)
        got = feed(r, rid, toks, cuts)
        r.release(rid)
        assert_close(got, want, dtype, rid)
        eng.cache.check_invariants()


@pytest.mark.gpu
@pytest.mark.parametrize("page", [4, 64])
def test_other_page_sizes(page, folders):
    folder, raw, tensors = folders("full", FULL, seed=1)
    toks = tokens_for(raw, 90, 8)
    want = plain.forward(raw, tensors, toks)
    eng = make_engine(folder, "float32", block_size=page, num_blocks=256 // page)
    eng.runner.admit("p")
    assert_close(feed(eng.runner, "p", toks, [33, 2, 1, 1, 19] + [1] * 34), want, "float32", f"pages of {page}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_equal_each_alone(dtype, folders):
    """Portions of some requests beside single tokens of others; a request pauses for a step; requests end and
    their pages and slots go to new ones (four slots, six requests, freed pages poisoned: also the pages that a
    window has passed, which go back while their request is still running)."""
    from edgerag_b200.engine.step import StepEntry

    folder, raw, tensors = folders("full", FULL, seed=1)
    lens = {"a": 70, "b": 33, "c": 1, "d": 90, "e": 18, "f": 47}
    toks = {k: tokens_for(raw, n, 20 + i) for i, (k, n) in enumerate(lens.items())}
    want = {k: plain.forward(raw, tensors, t) for k, t in toks.items()}
    eng = make_engine(folder, dtype, num_blocks=14)       # 224 tokens of pages: never room for all at once
    r = eng.runner
    plan = [
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
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype, folders):
    folder, raw, tensors = folders("full", FULL, seed=1)
    toks = tokens_for(raw, 330, 9)
    want = plain.forward(raw, tensors, toks)
    eng = make_engine(folder, dtype)
    eng.runner.admit("long")
    got = feed(eng.runner, "long", toks, [3] + [1] * 327)
    assert_close(got, want, dtype, "330 tokens, 327 of them one by one")
    held = eng.cache.held_pages("long")
    windows = [g.window for g in eng.cache.layout.groups]
    assert all(h < 21 for h, w in zip(held, windows) if w > 0) and all(h == 21 for h, w in zip(held, windows) if w == 0)


# --- kernels with inputs made so that a fault shows ---------------------------------------------------

def _window_reference(q, keys, values, positions_of, scale, window, keep, rep):
    """Plain attention: q [n, H, d] float64; keys/values[seq] [len, G, d]; -> [n, H, d]."""
    out = torch.zeros_like(q)
    for t, (seq, pos) in enumerate(positions_of):
        see = [j for j in range(pos + 1) if window <= 0 or pos - j < window or j < keep]
        for h in range(q.shape[1]):
            s = keys[seq][see, h // rep] @ q[t, h] * scale
            out[t, h] = torch.softmax(s, 0) @ values[seq][see, h // rep]
    return out


def _paged(rows, page_size, dtype, shuffle_seed=0):
    """Scatter each sequence's rows [len, G, d] over shuffled pages; (pages [P, G, page_size, d], block tables)."""
    G, d = rows[0].shape[1:]
    need = [-(-r.shape[0] // page_size) for r in rows]
    order = torch.randperm(sum(need) + 3, generator=torch.Generator().manual_seed(shuffle_seed)).tolist()
    pages = torch.full((sum(need) + 3, G, page_size, d), float("nan"), dtype=torch.float64)
    tables = torch.zeros(len(rows), max(need), dtype=torch.int32)
    for s, r in enumerate(rows):
        for i in range(need[s]):
            page = order.pop()
            tables[s, i] = page
            chunk = r[i * page_size: (i + 1) * page_size]
            pages[page, :, : chunk.shape[0]] = chunk.transpose(0, 1)
    return pages.to(dtype).cuda(), tables.cuda()


WINDOW_CASES = [  # (heads, kv heads, head size, page, window, kept)
    (4, 2, 32, 16, 24, 5), (6, 1, 48, 8, 17, 0), (2, 2, 64, 16, 64, 16), (8, 2, 128, 32, 40, 33), (3, 3, 16, 16, 9, 20),
    (4, 2, 24, 16, 30, 2), (6, 2, 64, 8, 100, 12), (8, 1, 32, 16, 33, 40), (8, 2, 64, 16, 40, 21), (4, 2, 64, 32, 200, 70),
]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", WINDOW_CASES)
def test_window_attention_with_one_key_made_dominant(case, dtype):
    """Every query gets one key whose score stands far out, placed in turn just inside the window, just outside
    it, at the last kept position, at the first one not kept, at a page's last and first slot and far away: a
    kernel that reads or skips the wrong key returns another value row.  Prompt rows and single tokens, the
    single tokens also in splits."""
    from edgerag_b200.ops import kernels as k

    H, G, d, page, window, keep = case
    tdt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    g = torch.Generator().manual_seed(H * 100 + d)
    lens = [150, 77, 2 * window + 3]
    keys = [torch.randn(n, G, d, generator=g, dtype=torch.float64) * 0.3 for n in lens]
    values = [torch.randn(n, G, d, generator=g, dtype=torch.float64) for n in lens]
    queries, where = [], []
    for s, n in enumerate(lens):
        for pos in sorted({n - 1, n - 2, window, window - 1, keep, max(keep - 1, 0), page - 1, page, 2 * page, 0, n // 2}):
            if not 0 <= pos < n:
                continue
            for target in (pos - window + 1, pos - window, keep - 1, keep, (pos // page) * page - 1, (pos // page) * page, 1, pos):
                if 0 <= target <= pos:
                    q = torch.randn(H, d, generator=g, dtype=torch.float64) * 0.3
                    for h in range(H):                      # the target's key, scaled up, is what the query looks for
                        q[h] += 6.0 * keys[s][target, h // (H // G)] / keys[s][target, h // (H // G)].norm() ** 2 / 0.5
                    queries.append(q)
                    where.append((s, pos))
    q = torch.stack(queries)
    want = _window_reference(q, keys, values, where, 0.5, window, keep, H // G)
    kp, tables = _paged(keys, page, tdt, 1)
    vp, _ = _paged(values, page, tdt, 1)
    # what the kernels see after rounding to the element type
    if dtype == "bfloat16":
        rk = [x.to(tdt).double() for x in keys]
        rv = [x.to(tdt).double() for x in values]
        want = _window_reference(q.to(tdt).double(), rk, rv, where, 0.5, window, keep, H // G)
    n = q.shape[0]
    qd = q.reshape(n, H * d).to(tdt).cuda()
    seq_of = torch.tensor([s for s, _ in where], dtype=torch.int32).cuda()
    pos = torch.tensor([p for _, p in where], dtype=torch.int32).cuda()
    tol = 2e-5 if dtype == "float32" else 2e-2
    out = torch.empty_like(qd)
    k.attention_rows(qd, kp, vp, tables, seq_of, pos, out, H, 0.5, window=window, keep_first=keep)
    err = (out.double().cpu().reshape(n, H, d) - want).abs().amax((1, 2))
    assert err.max() < tol, f"rows: query {int(err.argmax())} {where[int(err.argmax())]}: {err.max():.2e}"
    # the same queries as single tokens: one "sequence" per query (its table row repeated)
    for split in (16, 64):
        if split % page and page % split:
            continue
        tables1 = tables[seq_of.long()].contiguous()
        tok = torch.arange(n, dtype=torch.int32).cuda()
        splits = max(1, window // split + 2)
        acc, ml = k.decode_scratch_floats(n, H, d, splits)
        out1 = torch.empty_like(qd)
        k.attention_decode(qd, kp, vp, tables1, tok, pos, out1, H, 0.5, torch.empty(acc, device="cuda"), torch.empty(ml, device="cuda"),
                           splits, window=window, split_keys=split, keep_first=keep)
        err = (out1.double().cpu().reshape(n, H, d) - want).abs().amax((1, 2))
        assert err.max() < tol, f"single tokens, splits of {split}: query {int(err.argmax())} {where[int(err.argmax())]}: {err.max():.2e}"
        if k.decode_gqa_supported(tdt, d, window, H, G, page, split, splits):
            # grouped query heads of 64 on tensor cores
            out4 = torch.full_like(qd, float("nan"))
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            k.attention_decode_gqa(qd, kp, vp, tables1, tok, pos, out4, H, 0.5, torch.empty(acc, device="cuda"),
                                   torch.empty(ml, device="cuda"), splits, status, split_keys=split, window=window, keep_first=keep)
            assert int(status.item()) == 0
            err = (out4.double().cpu().reshape(n, H, d) - want).abs().amax((1, 2))
            assert err.max() < tol, f"grouped heads, splits of {split}: query {int(err.argmax())} {where[int(err.argmax())]}: {err.max():.2e}"
        if k.decode_bulk_supported(tdt, d, window, H, G, splits):
            # the kernel that streams pages with bulk copies: one kv head per block, and as many as it likes to group
            for group in (1, 0):
                out3 = torch.full_like(qd, float("nan"))
                status = torch.zeros(1, dtype=torch.int32, device="cuda")
                k.attention_decode_bulk(qd, kp, vp, tables1, tok, pos, out3, H, 0.5, torch.empty(acc, device="cuda"),
                                        torch.empty(ml, device="cuda"), splits, status, split_keys=split, head_group=group,
                                        window=window, keep_first=keep)
                assert int(status.item()) == 0
                err = (out3.double().cpu().reshape(n, H, d) - want).abs().amax((1, 2))
                assert err.max() < tol, (f"bulk copies, splits of {split}, group {group}: query {int(err.argmax())} "
                                         f"{where[int(err.argmax())]}: {err.max():.2e}")
    if k.prefill_tc_supported(tdt, d, window, page):
        # the tensor-core kernel for portions: every query as a portion of one row at its position
        out2 = torch.full_like(qd, float("nan"))
        tables1 = tables[seq_of.long()].contiguous()
        starts = torch.arange(n + 1, dtype=torch.int32).cuda()
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        k.attention_prefill_tc(qd, kp, vp, tables1, starts, pos, out2, n, H, 0.5, status, window=window, keep_first=keep)
        assert int(status.item()) == 0
        err = (out2.double().cpu().reshape(n, H, d) - want).abs().amax((1, 2))
        assert err.max() < tol, f"tensor cores: query {int(err.argmax())} {where[int(err.argmax())]}: {err.max():.2e}"


PORTION_CASES = [  # (page, window, kept, [(past, new tokens)], key ranges)
    (16, 100, 0, [(0, 700)], 1), (16, 128, 5, [(0, 300), (517, 260)], 1), (8, 129, 128, [(40, 530)], 1),
    (64, 300, 130, [(1000, 2), (3, 900)], 1), (16, 257, 20, [(0, 1030)], 3), (32, 40, 300, [(2100, 200), (0, 31)], 2),
    (128, 1, 0, [(5, 300)], 1), (16, 640, 0, [(777, 513)], 4),
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", PORTION_CASES)
def test_window_attention_of_portions_on_tensor_cores(case):
    """Portions of prompts behind pasts of several lengths: every row looks for one key, in turn the first of its
    window, the one before it, the last kept one, the first not kept, its own and a far one.  Pages that no row of
    the step sees hold NaN, as pages do that were given back and used again."""
    from edgerag_b200.ops import kernels as k

    page, window, keep, portions, ranges = case
    H, G, d, scale = 4, 2, 64, 0.25
    if not k.prefill_tc_supported(torch.bfloat16, d, window, page):
        pytest.skip("sizes the tensor-core kernel does not take")
    g = torch.Generator().manual_seed(window * 7 + keep)
    keys = [(torch.randn(past + new, G, d, generator=g, dtype=torch.float64) * 0.3).bfloat16().double() for past, new in portions]
    values = [torch.randn(past + new, G, d, generator=g, dtype=torch.float64).bfloat16().double() for past, new in portions]
    queries, where = [], []
    for s, (past, new) in enumerate(portions):
        for r in range(new):
            pos = past + r
            targets = [t for t in (pos - window + 1, pos - window, keep - 1, keep, pos, pos // 2) if 0 <= t <= pos]
            target = targets[r % len(targets)]
            q = torch.randn(H, d, generator=g, dtype=torch.float64) * 0.3
            for h in range(H):
                kt = keys[s][target, h // (H // G)]
                q[h] += 6.0 * kt / kt.norm() ** 2 / scale
            queries.append(q)
            where.append((s, pos))
    q = torch.stack(queries).bfloat16().double()
    want = _window_reference(q, keys, values, where, scale, window, keep, H // G)
    # keys that no row of the step sees are NaN
    for s, (past, new) in enumerate(portions):
        first_seen = max(past - window + 1, 0)
        dead_pages = range(-(-keep // page), first_seen // page)
        for pg in dead_pages:
            keys[s][pg * page: (pg + 1) * page] = float("nan")
            values[s][pg * page: (pg + 1) * page] = float("nan")
    kp, tables = _paged(keys, page, torch.bfloat16, 2)
    vp, _ = _paged(values, page, torch.bfloat16, 2)
    n = q.shape[0]
    qd = q.reshape(n, H * d).bfloat16().cuda()
    pos = torch.tensor([p for _, p in where], dtype=torch.int32).cuda()
    starts = torch.tensor([0] + list(np.cumsum([new for _, new in portions])), dtype=torch.int32).cuda()
    blocks = k.prefill_tc_blocks([new for _, new in portions])
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.full_like(qd, float("nan"))
    part_o = part_ml = None
    if ranges > 1:
        need_o, need_ml = k.prefill_tc_scratch_floats(n, H, ranges)
        part_o, part_ml = torch.empty(need_o, device="cuda"), torch.empty(need_ml, device="cuda")
    k.attention_prefill_tc(qd, kp, vp, tables, starts, pos, out, blocks, H, scale, status, key_splits=ranges, part_o=part_o,
                           part_ml=part_ml, window=window, keep_first=keep)
    assert int(status.item()) == 0
    err = (out.double().cpu().reshape(n, H, d) - want).abs().amax((1, 2))
    assert err.max() < 2e-2, f"query {int(err.argmax())} {where[int(err.argmax())]}: {err.max():.2e}"
    # and the general kernel on the same rows
    seq_of = torch.tensor([s for s, _ in where], dtype=torch.int32).cuda()
    out_rows = torch.empty_like(qd)
    k.attention_rows(qd, kp, vp, tables, seq_of, pos, out_rows, H, scale, window=window, keep_first=keep)
    err = (out_rows.double().cpu().reshape(n, H, d) - want).abs().amax((1, 2))
    assert err.max() < 2e-2, f"rows: query {int(err.argmax())} {where[int(err.argmax())]}: {err.max():.2e}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_queries_and_keys_made_ready(dtype):
    """Bias, head norm, turn of pairs on part of the head, values that are the keys before norm and turn, cache write."""
    from edgerag_b200.ops import kernels as k

    tdt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    g = torch.Generator().manual_seed(5)
    # (heads of 64, 128 and 256 with pairs take the kernel in which a lane owns neighbouring entries; many tokens
    # make a warp of it walk several heads)
    for (H, G, d, rot, page, pairs, shared, n) in ((4, 2, 32, 12, 16, True, True, 37), (3, 3, 48, 48, 8, True, True, 37),
                                                   (2, 1, 16, 8, 4, False, False, 37), (5, 5, 24, 0, 16, True, True, 37),
                                                   (4, 2, 64, 24, 16, True, True, 37), (3, 1, 128, 128, 8, True, True, 21),
                                                   (2, 2, 256, 64, 16, True, False, 9), (2, 1, 64, 0, 16, True, True, 5),
                                                   (9, 3, 64, 64, 16, True, True, 1100), (6, 2, 128, 32, 16, True, False, 900),
                                                   (4, 4, 64, 32, 16, False, False, 37)):
        width = (H + G * (1 if shared else 2)) * d
        x = (torch.randn(n, width, generator=g) * 1.5).to(tdt)
        qb, kb = torch.randn(H * d, generator=g), torch.randn(G * d, generator=g)
        qn, kn = 1 + 0.3 * torch.randn(d, generator=g), 1 + 0.3 * torch.randn(d, generator=g)
        pos = torch.randint(0, 3000, (n,), generator=g, dtype=torch.int32)
        n_pages = max(15, -(-n // page) + 2)
        slots = torch.randperm(n_pages * page, generator=g)[:n].to(torch.int32)
        slots[3] = -1
        inv = (100.0 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1)) / 3.0).float()
        kp = torch.zeros(n_pages, G, page, d, dtype=tdt).cuda()
        vp = torch.zeros_like(kp)
        xd = x.clone().cuda()
        k.qk_prepare(xd, pos.cuda(), H, G, d, q_bias=qb.cuda(), k_bias=kb.cuda(), q_norm=qn.cuda(), k_norm=kn.cuda(), eps=1e-5,
                     inv_freq=inv.cuda() if rot else None, rot_dim=rot, pairs=pairs, values_are_keys=shared, slots=slots.cuda(),
                     k_pages=kp, v_pages=vp, page_size=page)
        xs = x.double()
        q = xs[:, : H * d] + qb.double()
        kk = xs[:, H * d: (H + G) * d] + kb.double()
        vv = kk if shared else xs[:, (H + G) * d:]
        def ready(t, heads, w):
            t = plain.unit_rms(t.reshape(n, heads, d), 1e-5) * w.double()
            if not rot:
                return t
            if pairs:
                return plain.turn_pairs(t, pos, 100.0, rot, 3.0)
            ang = pos.double()[:, None] * inv.double()[None, :]
            cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            out = t.clone()
            a, b = t[..., : rot // 2], t[..., rot // 2: rot]
            out[..., : rot // 2], out[..., rot // 2: rot] = a * cs - b * sn, b * cs + a * sn
            return out
        # float32: an angle of up to 1,000 radians is a float32 product, exact to 2**-24 of its size (6e-5), times entries of up to 5
        tol = 3e-4 if dtype == "float32" else 3e-2
        assert (xd[:, : H * d].double().cpu() - ready(q, H, qn).reshape(n, H * d)).abs().max() < tol
        kr = ready(kk, G, kn)
        kc, vc = kp.double().cpu(), vp.double().cpu()
        for t in range(n):
            s = int(slots[t])
            if s < 0:
                continue
            assert (kc[s // page, :, s % page] - kr[t]).abs().max() < tol
            assert (vc[s // page, :, s % page] - vv[t].reshape(G, d)).abs().max() < tol
        written = {int(s) for s in slots if s >= 0}
        untouched = [(p, o) for p in range(n_pages) for o in range(page) if p * page + o not in written]
        assert all(float(kp[p, :, o].abs().max()) == 0 and float(vp[p, :, o].abs().max()) == 0 for p, o in untouched[:50])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_residual_add_between_two_layer_norms(dtype):
    from edgerag_b200.ops import kernels as k

    tdt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    g = torch.Generator().manual_seed(9)
    # (rows of up to 8,192 entries, a multiple of four, stay in registers; the others are parked in shared memory)
    for width in (6, 48, 50, 80, 256, 1000, 2048, 4096, 8192, 8200):
        n = 21
        hidden = torch.randn(n, width, generator=g) * 3 + 0.7
        delta = (torch.randn(n, width, generator=g) * 2 - 0.3).to(tdt)
        w1, b1, w2, b2 = (torch.randn(width, generator=g) * s + o for s, o in ((0.2, 1), (0.2, 0), (0.3, 1), (0.1, 0)))
        closed = plain.layer_norm(delta.double(), w1.double(), b1.double(), 1e-5)
        total = hidden.double() + closed
        want = plain.layer_norm(total, w2.double(), b2.double(), 1e-5)
        h = hidden.clone().cuda()
        out = torch.empty(n, width, dtype=tdt).cuda()
        k.add_layernorm(h, w2.cuda(), b2.cuda(), out, 1e-5, delta=delta.cuda(), post=(w1.cuda(), b1.cuda(), 1e-5))
        tol = 2e-5 if dtype == "float32" else 4e-2
        assert (h.double().cpu() - total).abs().max() < 2e-5 and (out.double().cpu() - want).abs().max() < tol
        # selected rows, nothing written back; no update at all; the update alone; partial sums
        rows = torch.tensor([5, 0, 20], dtype=torch.int32).cuda()
        h2 = hidden.clone().cuda()
        out3 = torch.empty(3, width, dtype=tdt).cuda()
        k.add_layernorm(h2, w2.cuda(), b2.cuda(), out3, 1e-5, delta=delta.cuda(), post=(w1.cuda(), b1.cuda(), 1e-5), rows=rows, write_back=False)
        assert torch.equal(h2.cpu(), hidden) and (out3.double().cpu() - want[[5, 0, 20]]).abs().max() < tol
        k.add_layernorm(h2, w2.cuda(), b2.cuda(), out, 1e-5)
        assert (out.double().cpu() - plain.layer_norm(hidden.double(), w2.double(), b2.double(), 1e-5)).abs().max() < tol
        k.add_layernorm(h2, None, None, None, 1e-5, delta=delta.cuda(), post=(w1.cuda(), b1.cuda(), 1e-5))
        assert (h2.double().cpu() - total).abs().max() < 2e-5
        parts = torch.randn(3, n, width, generator=g)
        summed = (parts[0] + parts[1] + parts[2]).to(tdt).double()
        h3 = hidden.clone().cuda()
        wide = torch.zeros(n, 2 * width, dtype=tdt).cuda()
        k.add_layernorm(h3, None, None, wide[:, :width], 1e-5, delta=parts.cuda(), post=(w1.cuda(), b1.cuda(), 1e-5), write_back=False)
        want_cast = hidden.double() + plain.layer_norm(summed, w1.double(), b1.double(), 1e-5)
        assert (wide[:, :width].double().cpu() - want_cast).abs().max() < (2e-5 if dtype == "float32" else 8e-2)
        assert float(wide[:, width:].abs().max()) == 0 and torch.equal(h3.cpu(), hidden)


@pytest.mark.gpu
def test_gelu_gate_and_its_fused_form():
    from edgerag_b200.ops import kernels as k

    g = torch.Generator().manual_seed(2)
    for tdt, tol in ((torch.float32, 1e-6), (torch.bfloat16, 2e-2)):
        gu = (torch.randn(19, 2 * 136, generator=g) * 2).to(tdt)
        out = torch.empty(19, 136, dtype=tdt).cuda()
        k.glu_bounded(gu.cuda(), out, act="gelu_tanh")
        want = plain.gelu_tanh(gu[:, :136].double()) * gu[:, 136:].double()
        assert (out.double().cpu() - want).abs().max() < tol * max(1.0, float(want.abs().max()))
    x = (torch.randn(7, 256, generator=g)).to(torch.bfloat16).cuda()
    w = (torch.randn(2 * 136, 256, generator=g) / 16).to(torch.bfloat16).cuda()
    fused = torch.empty(7, 136, dtype=torch.bfloat16).cuda()
    k.linear_glu(x, w, fused, bounded=(0.0, 1.0, 0.0, "gelu_tanh"))
    gate_up = torch.empty(7, 272, dtype=torch.bfloat16).cuda()
    k.linear(x, w, gate_up)
    two = torch.empty_like(fused)
    k.glu_bounded(gate_up, two, act="gelu_tanh")
    assert torch.equal(fused, two)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_model_whose_scores_single_out_far_and_edge_keys(dtype, folders):
    """A one-layer model whose query and key weights are scaled up, so that its softmax is sharp and a token that
    sits just inside or outside a window's edge, among the kept ones or right after them decides the row."""
    raw = plain.make_config([plain.attention_layer(heads=4, kv_heads=2, dim=32, rot_dims=8, size=19, keep_first=4, factor=2.0, ff=None,
                                                   scale=1.5)], width=64, vocab=97)
    folder, raw, tensors = folders("sharp", raw, seed=4)
    toks = tokens_for(raw, 120, 3)
    want = plain.forward(raw, tensors, toks)
    blind = plain.forward({**raw, "layers": [{**raw["layers"][0], "mixer": {**raw["layers"][0]["mixer"], "mask": {"size": 20, "keep_first": 4}}}]},
                          tensors, toks)
    assert row_errors(blind[30:], want[30:]).max() > 0.05, "the test's weights do not tell a window of 19 from one of 20"
    eng = make_engine(folder, dtype)
    for rid, cuts in (("whole", [120]), ("tail", [18] + [1] * 102), ("mixed", [3, 2, 14, 1, 1, 30, 2, 2, 1, 40] + [1] * 24)):
        eng.runner.admit(rid)
        assert_close(feed(eng.runner, rid, toks, cuts), want, dtype, rid)
        eng.runner.release(rid)


# --- generation through the engine's own entry point -----------------------------------------------

def plain_greedy(raw, tensors, prompt, n_new):
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
    """Five prompts through ``Engine.generate`` with two slots and portions of 8 tokens: the scheduler cuts
    prompts, batches them with decoding requests and hands slots and pages on."""
    from edgerag_b200.sampling.params import SamplingParams

    folder, raw, tensors = folders("full", FULL, seed=1)
    prompts = [tokens_for(raw, n, 40 + n) for n in (21, 3, 34, 9, 1)]
    eng = make_engine(folder, dtype, max_batch_size=2, num_blocks=8, chunk_size=8, max_step_tokens=None, cuda_graphs=graphs)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=30))
    eng.cache.check_invariants()
    assert eng.cache.free_pages() == [8] * len(eng.cache.layout.groups) and not eng.cache.requests
    compared = 0
    for prompt, got in zip(prompts, outs):
        want, margins = plain_greedy(raw, tensors, prompt, 30)
        assert len(got) == 30
        clear = next((i for i, m in enumerate(margins) if m < (1e-3 if dtype == "float32" else 0.08)), 30)
        assert list(got[:clear]) == want[:clear], f"prompt of {len(prompt)} tokens"
        compared += clear
    assert compared >= (40 if dtype == "float32" else 5), "the margins left too little to compare"


@pytest.mark.gpu
def test_trace_replay_program(folders, tmp_path):
    folder, raw, tensors = folders("full", FULL, seed=1)
    a, b = tokens_for(raw, 60, 1), tokens_for(raw, 9, 2)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]}, {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": a[31:58], "want": []}], "end": []},
        {"step": 3, "entries": [{"id": "b", "tokens": b[8:], "want": [0]}, {"id": "a", "tokens": a[58:], "want": [0, 1]}], "end": ["a", "b"]},
    ]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    assert not (out / "2.f32").exists()
    wa, wb = plain.forward(raw, tensors, a), plain.forward(raw, tensors, b)
    V = raw["vocab"]
    got = {i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)) for i in (0, 1, 3)}
    assert_close(got[0], wa[[0, 29]], "float32", "step 0")
    assert_close(got[1], torch.stack([wa[30], wb[7]]), "float32", "step 1")
    assert_close(got[3], torch.stack([wb[8], wa[58], wa[59]]), "float32", "step 3")


@pytest.mark.gpu
def test_command_line_with_random_weights(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(FULL))
    base = [sys.executable, "-m", "edgerag_b200", "--dtype", "fp32", "--num-blocks", "16", "--max-batch-size", "2", "--chunk-size", "16",
            "--max-new-tokens", "5", "--prompt-ids", "3,1,4,1,5,9,2,6", "--prompt-ids", "7", "--json"]
    first = subprocess.run(base + ["--random-weights", "3", "--config", str(cfg), "--save-model", str(tmp_path / "m"), "--weights-std", "0.1"],
                           capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert first.returncode == 0, first.stderr[-2000:]
    again = subprocess.run(base + ["--model", str(tmp_path / "m")], capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert again.returncode == 0, again.stderr[-2000:]
    a, b = (json.loads(p.stdout.strip().splitlines()[-1])["outputs"] for p in (first, again))
    assert [len(o["token_ids"]) for o in a] == [5, 5] and a == b
