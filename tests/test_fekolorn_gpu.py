"""The Fekolorn design on the GPU against the plain implementation (tests/plain_fekolorn.py, float64, no cache): each
mechanism's kernels alone (the streams' write, read and norm in one pass and their sum at the end, the pair-table
embedding with its previous token kept per slot, PolyNorm, the softmax mixer with a distance bias, a sink, normed or
mixed values and a window, the gated delta rule behind its convolutions, the two side by side), keys at the window's
edge, far back and among the first tokens made to stand out, then whole models replayed whole, with a tail decoded token
by token, in portions down to one and two tokens and in mixed batches with so few pages and slots that they are used
again; float32 and bfloat16; long decoding beyond the pool; greedy generation through the engine's entry point and
scheduler, with and without CUDA graphs; the trace program and the command line."""
import json
import math
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_fekolorn as P
import replay_util as RU
from fekolorn_configs import FEKOLORN, write_fekolorn_model

pytestmark = pytest.mark.gpu

TOL_F32 = 2e-4          # float32 engine against float64: rounding only
TOL_BF16_REL = 0.05     # of the largest logit; a wrong key, window, state or stream moves logits by their own size
DEV = "cuda:0"
LENGTHS = {"A": [2, 19, 40, 77, 131, 260], "B": [1, 9, 33, 70, 128, 161], "C": [5, 31, 66, 150, 300],
           "D": [1, 2, 18, 65, 140, 230], "E": [3, 16, 47, 90, 200], "F": [1, 6, 29, 64, 133, 210]}
MODES = ["whole", "tail", "portions", "mixed"]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    folder = tmp_path_factory.mktemp("fekolorn")
    out = {}
    for name in FEKOLORN:
        path = write_fekolorn_model(name, str(folder))
        cfg, w = P.load_model_dir(path)
        rng = np.random.default_rng(17 + ord(name))
        reqs = {f"r{i}": rng.integers(0, cfg["vocab"], n).tolist() for i, n in enumerate(LENGTHS[name])}
        ref = {r: P.forward(toks, cfg, w).numpy() for r, toks in reqs.items()}
        out[name] = (path, cfg, w, reqs, ref)
    return out


class _Ctx(SimpleNamespace):
    """The index arrays of a step, as the step function gives them to the parts, with a mixer's plan and workspace."""

    def plan(self, key):
        return self.plans[key]

    def scratch(self, name, n_floats):
        return torch.zeros((max(n_floats, 1),), dtype=torch.float32, device=DEV)


def _ctx(n_new, cached, slots=None, planners=(), page_size=16, token_ids=None):
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    q_start = np.concatenate([[0], np.cumsum(n_new)[:-1]]).astype(int).tolist()
    token_req = [r for r, n in enumerate(n_new) for _ in range(n)]
    positions = [c + i for c, n in zip(cached, n_new) for i in range(n)]
    slots = list(slots if slots is not None else range(len(n_new)))
    ctx = _Ctx(n_tokens=sum(n_new), n_requests=len(n_new), q_start=i32(q_start), n_new=i32(n_new),
               cached_len=i32(cached), slot_ids=i32(slots), token_req=i32(token_req), positions=i32(positions), plans={},
               shared={}, token_ids=None if token_ids is None else i32(token_ids))
    from llm_rs_b200.parts.base import StepInfo
    a32 = lambda v: np.asarray(v, np.int32)
    for key, planner in planners:
        plan = planner.plan(StepInfo(sum(n_new), len(n_new), a32(q_start), a32(n_new), a32(cached), a32(slots),
                                     [], [], page_size, False))
        ctx.plans[key] = SimpleNamespace(
            arrays={k: torch.from_numpy(np.ascontiguousarray(v)).to(DEV) for k, v in plan.arrays.items()},
            values=dict(plan.values))
    return ctx


def _planners(part):
    return part.planners() if hasattr(part, "planners") else ([(part.plan_key(), part)] if part.plan_key() else [])


def _assert_logits(got, ref, dtype, what):
    """float32: every position within TOL_F32 (this pins the logic). bfloat16: three positions in a hundred may exceed
    the tolerance. A wrong key, window, state or stream in a bfloat16 kernel moves every later position."""
    scale = max(float(np.abs(r).max()) for r in ref.values())
    diffs = {k: float(np.abs(row.astype(np.float64) - ref[k[0].replace("again", "")][k[1]]).max())
             for k, row in got.items()}
    assert all(np.isfinite(d) for d in diffs.values()), what
    worst = max(diffs, key=diffs.get)
    if dtype == "float32":
        assert diffs[worst] <= TOL_F32 * max(1.0, scale), f"{what}: max |diff| {diffs[worst]:.3e} at {worst}"
        return
    tol = TOL_BF16_REL * scale
    over = [k for k, d in diffs.items() if d > tol]
    assert len(over) <= max(1, 3 * len(diffs) // 100), \
        f"{what}: max |diff| {diffs[worst]:.3e} at {worst}, {len(over)} of {len(diffs)} over {tol:.3e}: {sorted(over)[:12]}"


def _weights(part, g, dtype, sigma=1.0):
    """Random tensors for a part's ``weight_specs``: matrices ~ sigma / sqrt(columns), vectors ~ sigma, rounded to
    bfloat16 so that both precisions and the plain implementation see the same numbers."""
    w = {}
    for s in part.weight_specs():
        t = sigma * torch.randn(s.shape, generator=g)
        if s.role == "conv":
            t = 0.6 * torch.randn(s.shape, generator=g)
        elif len(s.shape) == 2:
            t = t / math.sqrt(s.shape[-1])
        if s.role == "norm":
            t = 1.0 + 0.3 * torch.randn(s.shape, generator=g)
        w[s.name] = t.bfloat16().float()
    dev = {k: v.to(DEV, dtype if v.dim() == 2 and not k.endswith(("conv", "rel", "mix")) else torch.float32)
           for k, v in w.items()}
    return w, dev


def _close(got, want, dtype, what, f32=3e-5, bf16=0.03):
    """float32: every element against the largest of the wanted ones. bfloat16: every row but one in fifty."""
    scale = want.abs().max().item()
    d = (got.double() - want).abs().reshape(want.shape[0], -1).amax(dim=1) if want.dim() > 1 else (got.double() - want).abs()
    if dtype == torch.float32:
        assert d.max().item() <= f32 * max(1.0, scale), (what, d.max().item(), scale)
        return
    over = int((d > bf16 * scale).sum())
    assert over <= max(1, d.numel() // 50), (what, over, d.max().item(), scale)


def _rounded(x, dtype):
    return x.bfloat16().float() if dtype == torch.bfloat16 else x


def _double(w):
    return {k: v.double() for k, v in w.items()}


# ---- mechanisms alone -----------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("streams,width,rows", [(1, 70, 33), (2, 256, 5), (3, 1, 3), (4, 100, 1), (5, 2050, 9),
                                                (9, 48, 7), (16, 33, 4)])
def test_streams_write_read_norm_and_sum(streams, width, rows, dtype):
    """Two sublayers in a row through ``hyper_step`` (a read alone, a write with the next read, a write alone) and the
    sum of the streams with the last write folded in, on some rows only."""
    from llm_rs_b200 import ops
    g = torch.Generator().manual_seed(streams * 1000 + width)
    x0 = torch.randn(rows, width, generator=g)
    w = {f"hc{q}.{n}": torch.randn(*s, generator=g) for q in (1, 2) for n, s in
         (("in", (streams,)), ("out", (streams,)), ("mix", (streams, streams)))}
    gains = [torch.tensor(1.3), torch.tensor(0.7)]
    ys = [_rounded(torch.randn(rows, width, generator=g), dtype) for _ in range(2)]
    seen = []

    def branch(q):
        def fn(h):
            seen.append(h)
            return ys[q].double()
        return fn
    st = x0.double()[None].repeat(streams, 1, 1)
    st = P.sublayer(st, branch(0), gains[0].double(), 1e-5, _double(w), "hc1.")
    st = P.sublayer(st, branch(1), gains[1].double(), 1e-5, _double(w), "hc2.")
    d = {k: v.to(DEV) for k, v in w.items()}
    gd = [t.reshape(1).to(DEV) for t in gains]
    x = x0[:, None, :].repeat(1, streams, 1).reshape(rows, streams * width).contiguous().to(DEV)
    u1 = ops.hyper_step(x, read=(d["hc1.in"], gd[0]), eps=1e-5, act_dtype=dtype)
    u2 = ops.hyper_step(x, write=(ys[0].to(DEV, dtype), d["hc1.mix"], d["hc1.out"]), read=(d["hc2.in"], gd[1]), eps=1e-5,
                        act_dtype=dtype)
    _close(u1.float().cpu(), seen[0], dtype, "first read", bf16=0.01)
    _close(u2.float().cpu(), seen[1], dtype, "second read", bf16=0.01)
    pick = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    pending = (ys[1].to(DEV, torch.float32), d["hc2.mix"], d["hc2.out"])        # a branch output may be float32 too
    total = ops.hyper_leave(x, streams, write=pending, rows=pick)
    _close(total.cpu(), st.sum(0)[[rows - 1, 0]], torch.float32, "sum of the streams")
    ops.hyper_step(x, write=pending)
    _close(x.view(rows, streams, width).permute(1, 0, 2).cpu(), st, torch.float32, "streams after the last write")
    _close(ops.hyper_leave(x, streams).cpu(), st.sum(0), torch.float32, "plain sum")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("buckets,mul_prev,mul_cur,copies", [(101, 13, 5, 2), (1, 7, 7, 1), (4099, 100003, 99991, 3), (0, 0, 0, 2)])
def test_pair_embedding_keeps_the_previous_token_per_slot(dtype, buckets, mul_prev, mul_cur, copies):
    """Two requests cut differently, a third that takes over a slot: the row before a step's first token comes from the
    slot, a sequence's first token takes the table's last row whatever the slot held."""
    from llm_rs_b200 import ops
    g = torch.Generator().manual_seed(buckets + copies)
    V, D = 300, 24
    table = torch.randn(V, D, generator=g).bfloat16().float()
    pairs = torch.randn(buckets + 1, D, generator=g).bfloat16().float() if buckets else None
    cfg = {"embedding": {"scale": 0.75}}
    if buckets:
        cfg["embedding"]["bigram"] = {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}
    w = {"embed": table.double(), "bigram": None if pairs is None else pairs.double()}
    seqs = [torch.randint(0, V, (n,), generator=g).tolist() for n in (23, 9, 14)]
    want = [P.embed(s, cfg, w) for s in seqs]
    state = torch.full((2, 1), 123.0, device=DEV)              # what an earlier request left in the slots
    td, pd = table.to(DEV, dtype), None if pairs is None else pairs.to(DEV, dtype)
    got = [[], [], []]
    at = [0, 0, 0]
    # (request, tokens) per step; request 2 takes slot 1 after request 1 is done
    steps = [[(0, 5), (1, 1)], [(0, 1), (1, 6)], [(1, 2)], [(0, 2), (2, 3)], [(0, 15), (2, 1)], [(2, 10)]]
    slot_of = {0: 0, 1: 1, 2: 1}
    for step in steps:
        ids = [t for r, n in step for t in seqs[r][at[r]: at[r] + n]]
        ctx = _ctx([n for _, n in step], [at[r] for r, _ in step], slots=[slot_of[r] for r, _ in step], token_ids=ids)
        y = ops.bigram_embedding(td, pd, ctx, state if buckets else None, copies, 0.75, buckets, mul_prev, mul_cur)
        y = y.view(len(ids), copies, D).cpu()
        assert all(torch.equal(y[:, 0], y[:, c]) for c in range(copies))
        o = 0
        for r, n in step:
            got[r].append(y[o:o + n, 0])
            o += n
            at[r] += n
    for r in range(3):
        _close(torch.cat(got[r]), want[r], torch.float32, f"request {r}", f32=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width", [(5, 64), (1, 1), (33, 100), (3, 3000)])
def test_poly_norm_against_plain(rows, width, dtype):
    from llm_rs_b200 import ops
    g = torch.Generator().manual_seed(width)
    z = _rounded(2.0 * torch.randn(rows, width, generator=g), dtype)
    c = torch.tensor([0.8, -1.1, 0.4, 0.3])
    got = ops.poly_norm(z.to(DEV, dtype), c.to(DEV), 1e-5)
    _close(got.float().cpu(), P.poly_norm(z.double(), c.double(), 1e-5), dtype, "poly_norm", bf16=0.01)


def _pages(kv_heads, dk, dv, page, n_pages, dtype):
    pages = torch.zeros(n_pages, kv_heads, page * (dk + dv), dtype=dtype, device=DEV)
    return [pages[:, :, : page * dk].unflatten(2, (page, dk)), pages[:, :, page * dk:].unflatten(2, (page, dv))]


def _softmax_setup(dtype, heads, kv, dk, dv, window, rot, bias, alone, page, n_pages, seed, v_mix="none", scale=None,
                   D=56, base=3000.0, sink=True):
    """The softmax mixer as the design's two layer types use it: ``alone`` norms the whole q and k rows, else the
    values are normed per head."""
    from llm_rs_b200.parts import Runtime
    from llm_rs_b200.parts.scored_attention import ScoredAttention
    g = torch.Generator().manual_seed(seed)
    scale = 1.0 / math.sqrt(dk) if scale is None else scale
    part = ScoredAttention(D, heads, kv, dk, dv, scale=scale, sink=sink, mask="window" if window else "causal",
                           mask_size=window, qk_norm="whole" if alone else "none", norm_eps=1e-5, rot_dims=rot,
                           rot_base=base, v_norm="none" if alone else "head_unit", v_mix=v_mix,
                           bias_rows=bias[0] if bias else 0, bias_max=bias[1] if bias else 0.0, prefix="m.")
    w, wd = _weights(part, g, dtype, 1.5)
    if v_mix != "none":
        w["m.vmix"] = torch.tensor(0.35)
        wd["m.vmix"] = w["m.vmix"].to(DEV)
    part.bind(wd, Runtime(torch.device(DEV), dtype, 4096))
    m = {"heads": heads, "kv_heads": kv, "dim": dk, "vdim": dv, "scale": scale}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
    if window:
        m["mask"] = {"size": window}
    if bias:
        m["bias_max"] = bias[1]
    if v_mix != "none":
        m["v_mix"] = True
    return part, w, _pages(kv, dk, dv, page, n_pages, dtype), m, g, D


def _run_in_cuts(part, planes, state, seqs, cuts, page, dtype, g, n_pages, shared=None):
    """Two requests over scattered pages and their own slots: a prompt portion each, then portions and single tokens
    in the same steps, steps that one request sits out. ``shared``: per request, rows that another layer left."""
    lens = [s.shape[0] for s in seqs]
    assert all(sum(c[r] for c in cuts) == n for r, n in enumerate(lens))
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = -(-max(lens) // page)
    table = torch.tensor([perm[:width], perm[width:2 * width]], dtype=torch.int32, device=DEV)
    cache = SimpleNamespace(planes=planes, block_table=table, page_size=page, owns=True, state=state)
    at, got = [0, 0], [[], []]
    for cut in cuts:
        live = [r for r in range(2) if cut[r]]
        ctx = _ctx([cut[r] for r in live], [at[r] for r in live], slots=[3 - r for r in live], planners=_planners(part),
                   page_size=page)
        if shared is not None:
            ctx.shared[shared[0]] = torch.cat([shared[1][r][at[r]: at[r] + cut[r]] for r in live]).to(DEV, dtype)
        cache.block_table = table[live].contiguous()
        x = torch.cat([seqs[r][at[r]: at[r] + cut[r]] for r in live]).to(DEV, dtype)
        y = part.forward(x, ctx, cache).float().cpu()
        o = 0
        for r in live:
            got[r].append(y[o:o + cut[r]])
            o += cut[r]
            at[r] += cut[r]
    return [torch.cat(rows) for rows in got]


CUTS = [(97, 30), (2, 1), (1, 1), (30, 2), (1, 1), (19, 6), (0, 1), (1, 0)]       # 151 and 42 tokens


@pytest.mark.parametrize("generic", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dk,dv,window,rot,bias,alone,page", [
    (4, 2, 16, 32, 20, 0, (8, 64), True, 16), (5, 1, 24, 8, 7, 0, (6, 5), True, 8), (2, 2, 8, 40, 1, 0, (2, 3), True, 4),
    (6, 6, 64, 64, 96, 0, (14, 100), True, 16), (8, 4, 64, 32, 130, 0, (20, 130), True, 32), (3, 3, 128, 128, 0, 0, (32, 2000), True, 64),
    (4, 4, 16, 16, 0, 8, None, False, 16), (6, 3, 96, 32, 0, 64, None, False, 16), (2, 1, 20, 12, 0, 4, None, False, 16),
    (6, 1, 48, 32, 75, 48, (9, 40), False, 16), (7, 1, 40, 40, 0, 0, (3, 50), True, 16), (12, 3, 80, 48, 16, 80, None, False, 16),
    (4, 2, 128, 32, 0, 64, None, False, 16), (3, 1, 64, 16, 33, 0, (12, 33), True, 16)])
def test_softmax_mixer_against_plain(dtype, heads, kv, dk, dv, window, rot, bias, alone, page, generic):
    """The mixer part alone as both layer types configure it: norms over the whole q and k rows or values of unit root
    mean square, a bias per distance bucket whose reach lies inside and beyond the window, windows shorter and longer
    than a page, of one key and none, rotation of none, some and all channels, a sink; on the tensor cores and on the
    kernel for any type."""
    from llm_rs_b200 import ops
    if generic and dtype == torch.float32:
        pytest.skip("float32 has one kernel")
    part, w, planes, m, g, D = _softmax_setup(dtype, heads, kv, dk, dv, window, rot, bias, alone, page, 128, dk + heads)
    seqs = [_rounded(torch.randn(n, D, generator=g), dtype) for n in (151, 42)]
    want = [P.softmax_mixer(s.double(), m, _double(w), "m.", 1e-5, torch.arange(len(s)), alone, not alone)[0] for s in seqs]
    ops.scored_generic_only(generic)
    try:
        got = _run_in_cuts(part, planes, {}, seqs, CUTS, page, dtype, g, 128)
    finally:
        ops.scored_generic_only(False)
    for r in range(2):
        _close(got[r], want[r], dtype, r)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("alone", [True, False])
def test_values_mixed_with_another_layers(dtype, alone):
    """The kept value is (1 - m) v + m v_first, after the values' own norm where there is one; what a source layer
    publishes is its own projection of the step's tokens."""
    part, w, planes, m, g, D = _softmax_setup(dtype, 4, 2, 16, 24, 12, 0 if alone else 8, (8, 30) if alone else None, alone,
                                              16, 64, 5, v_mix="mixed")
    seqs = [_rounded(torch.randn(n, D, generator=g), dtype) for n in (151, 42)]
    firsts = [_rounded(torch.randn(n, 2 * 24, generator=g), dtype) for n in (151, 42)]
    want = [P.softmax_mixer(s.double(), m, _double(w), "m.", 1e-5, torch.arange(len(s)), alone, not alone,
                            v_first=f.double().view(-1, 2, 24))[0] for s, f in zip(seqs, firsts)]
    got = _run_in_cuts(part, planes, {}, seqs, CUTS, 16, dtype, g, 64, shared=("v_first", firsts))
    for r in range(2):
        _close(got[r], want[r], dtype, r)
    src, w2, planes2, _, g2, _ = _softmax_setup(dtype, 4, 2, 16, 24, 12, 0, None, True, 16, 64, 6, v_mix="source")
    ctx = _ctx([9], [0], planners=_planners(src))
    cache = SimpleNamespace(planes=planes2, block_table=torch.arange(4, dtype=torch.int32, device=DEV)[None], page_size=16,
                            owns=True, state={})
    x = seqs[0][:9]
    src.forward(x.to(DEV, dtype), ctx, cache)
    _close(ctx.shared["v_first"].float().cpu(), x.double() @ w2["m.v"].double().T, dtype, "published values", bf16=0.01)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("window,page,key_at", [(13, 8, 48), (16, 16, 31), (33, 32, 64), (1, 16, 40), (70, 16, 17), (40, 16, 0)])
def test_window_edges(dtype, decode, window, page, key_at):
    """One token's row is replaced by a row 25 times larger (its value grows 25-fold; the norm over the whole row keeps
    its key's size). The output must move when that key is the last one inside the window and must stay bit for bit
    when it is one step outside; for a query inside a prompt's portion and for one decoded alone; keys at a page's
    first and last row and the sequence's first token; the bias table's reach ends inside the window."""
    part, w, planes, m, g, D = _softmax_setup(dtype, 2, 1, 16, 12, window, 0, (6, max(4, window // 2)), True, page, 32, 5)
    n = 160
    base = torch.randn(n, D, generator=g)
    other = 25.0 * torch.randn(D, generator=g)
    outs = {}
    for name, query_at in (("inside", key_at + window - 1), ("outside", key_at + window)):
        for planted in (False, True):
            x = base.clone()
            if planted:
                x[key_at] = other
            x = _rounded(x, dtype)
            want = P.softmax_mixer(x.double(), m, _double(w), "m.", 1e-5, torch.arange(n), True, False)[0][query_at]
            for p in planes:
                p.zero_()
            table = torch.arange(31, -1, -1, dtype=torch.int32, device=DEV)[None, : -(-n // page)].contiguous()
            cache = SimpleNamespace(planes=planes, block_table=table, page_size=page, owns=True, state={})
            pl = _planners(part)
            if decode and query_at > 0:
                part.forward(x[:query_at].to(DEV, dtype), _ctx([query_at], [0], planners=pl, page_size=page), cache)
                y = part.forward(x[query_at:query_at + 1].to(DEV, dtype), _ctx([1], [query_at], planners=pl, page_size=page),
                                 cache)[0]
            else:
                y = part.forward(x[: query_at + 3].to(DEV, dtype), _ctx([query_at + 3], [0], planners=pl, page_size=page),
                                 cache)[query_at]
            scale = want.abs().max().item()
            d = (y.float().cpu().double() - want).abs().max().item()
            assert d <= (3e-5 * max(1, scale) if dtype == torch.float32 else 0.03 * scale), (name, planted, d, scale)
            outs[(name, planted)] = y.float().cpu()
    moved = (outs[("inside", True)] - outs[("inside", False)]).abs().max().item()
    still = (outs[("outside", True)] - outs[("outside", False)]).abs().max().item()
    assert moved > 0.02 * outs[("inside", False)].abs().max().item(), moved
    assert still == 0.0, still


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("alone", [False, True])
def test_a_far_key_among_hundreds_and_a_sink_that_shows(dtype, alone):
    """No window: with a score scale several times the usual one the softmax of every query rests on the few keys whose
    score stands out, and among 900 keys those lie anywhere: hundreds of positions back, at page borders, among the
    first tokens; sinks of the size of the largest scores take a visible share. A kernel that loses a far key or leaves
    the sink out gives another output. Whole, and with the last 60 positions decoded one by one."""
    n, page = 900, 16
    part, w, planes, m, g, D = _softmax_setup(dtype, 2, 1, 16, 12, 0, 0 if alone else 8, (16, 600) if alone else None, alone,
                                              page, 64, 9, scale=1.2 if alone else 0.45)
    w["m.sink"] = torch.tensor([2.0, 4.0])
    part.sink = w["m.sink"].to(DEV)
    x = _rounded(torch.randn(n, D, generator=torch.Generator().manual_seed(77)), dtype)
    plain = lambda ww: P.softmax_mixer(x.double(), m, _double(ww), "m.", 1e-5, torch.arange(n), alone, not alone)[0]
    want = plain(w)
    no_sink = {k: v for k, v in w.items() if k != "m.sink"}
    assert (plain(no_sink) - want).abs().max() > 0.1 * want.abs().max(), "the sink would not show"
    table = torch.randperm(64, generator=g).to(torch.int32)[None, : -(-n // page)].contiguous().to(DEV)
    cache = SimpleNamespace(planes=planes, block_table=table, page_size=page, owns=True, state={})
    ctx = lambda k, at: _ctx([k], [at], planners=_planners(part), page_size=page)
    whole = part.forward(x.to(DEV, dtype), ctx(n, 0), cache).float().cpu()
    _close(whole, want, dtype, "whole", bf16=0.06)
    for p in planes:
        p.zero_()
    head = n - 60
    rows = [part.forward(x[:head].to(DEV, dtype), ctx(head, 0), cache).float().cpu()]
    rows += [part.forward(x[i:i + 1].to(DEV, dtype), ctx(1, i), cache).float().cpu() for i in range(head, n)]
    _close(torch.cat(rows), want, dtype, "tail decoded", bf16=0.06)


def _delta_setup(dtype, heads, kv, dk, dv, conv, seed, D=56):
    from llm_rs_b200.parts import Runtime
    from llm_rs_b200.parts.delta_rule import GatedDelta
    g = torch.Generator().manual_seed(seed)
    part = GatedDelta(D, heads, kv, dk, dv, conv, norm_eps=1e-5, prefix="m.")
    w, wd = _weights(part, g, dtype, 1.5)
    for name in ("m.A_log", "m.dt_bias"):       # decays that forget within tens of tokens, not at once
        w[name] = (w[name] * 0.5 - 1.5).bfloat16().float()
        wd[name] = w[name].to(DEV)
    part.bind(wd, Runtime(torch.device(DEV), dtype, 4096))
    state = {n: torch.randn(5, *shape, device=DEV) for n, shape in part.state_need().tensors.items()}    # junk to clear
    m = {"heads": heads, "kv_heads": kv, "dim": dk, "vdim": dv, "conv": conv}
    return part, w, state, m, g, D


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dk,dv,conv", [(4, 2, 16, 8, 4), (2, 2, 8, 24, 2), (3, 1, 12, 20, 1), (4, 4, 32, 16, 5),
                                                 (4, 2, 64, 64, 4), (2, 1, 128, 32, 3), (1, 1, 200, 40, 4), (6, 3, 20, 17, 3)])
def test_gated_delta_mixer_against_plain(dtype, heads, kv, dk, dv, conv, ):
    """The recurrent mixer alone over two requests in their own slots: portions, single tokens, portions shorter than
    the convolution, steps that a request sits out; key heads shared by several value heads; keys of 8 to 200 channels,
    value widths that are no multiple of the kernel's slices; convolutions of one to five taps."""
    part, w, state, m, g, D = _delta_setup(dtype, heads, kv, dk, dv, conv, dk + heads)
    for t in state.values():
        t[2:4].zero_()          # what the cache manager does when a request takes a slot
    seqs = [_rounded(torch.randn(n, D, generator=g), dtype) for n in (151, 42)]
    want = [P.gated_delta(s.double(), m, _double(w), "m.", 1e-5) for s in seqs]
    got = _run_in_cuts(part, None, state, seqs, CUTS, 16, dtype, g, 32)
    for r in range(2):
        _close(got[r], want[r], dtype, r, f32=1e-4, bf16=0.04)


@pytest.mark.parametrize("chunked", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dk,dv,conv,lens,cuts", [
    (4, 2, 16, 8, 4, (300, 77), [(64, 77), (100, 0), (136, 0)]),            # whole chunks, a ragged one, a short neighbour
    (2, 1, 128, 32, 3, (257, 65), [(129, 1), (1, 64), (127, 0)]),           # one token beside a long portion
    (3, 1, 12, 20, 2, (200, 200), [(33, 167), (167, 33)]),                  # value width no multiple of a slice
    (1, 1, 200, 40, 4, (95, 96), [(95, 96)]),                               # keys of 200 channels
    (4, 4, 32, 16, 5, (640, 3), [(639, 1), (1, 2)])])                       # twenty chunks in a row
def test_long_portions_in_chunks_against_plain(dtype, heads, kv, dk, dv, conv, lens, cuts, chunked):
    """Long portions token by token, and in chunks of 32 tokens (the form that ``LLMRS_GD_CHUNKED=1`` switches on for
    portions of 64 tokens and more): the same numbers, from and into the same state, whatever the cut."""
    from llm_rs_b200 import ops
    part, w, state, m, g, D = _delta_setup(dtype, heads, kv, dk, dv, conv, dk + heads)
    for t in state.values():
        t[2:4].zero_()
    seqs = [_rounded(torch.randn(n, D, generator=g), dtype) for n in lens]
    want = [P.gated_delta(s.double(), m, _double(w), "m.", 1e-5) for s in seqs]
    ops.gated_delta_chunked(chunked)
    try:
        got = _run_in_cuts(part, None, state, seqs, cuts, 16, dtype, g, 128)
    finally:
        ops.gated_delta_chunked(ops.GD_CHUNKED)
    for r in range(2):
        _close(got[r], want[r], dtype, r, f32=1e-4, bf16=0.04)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_recurrence_carries_its_state_over_a_long_decoding(dtype):
    """400 tokens one by one after a portion of two: the state and the convolution's rows travel through 400 steps; a
    second request is decoded beside it from another slot."""
    part, w, state, m, g, D = _delta_setup(dtype, 2, 1, 16, 12, 4, 3)
    for t in state.values():
        t.zero_()
    seqs = [_rounded(torch.randn(n, D, generator=g), dtype) for n in (402, 401)]
    want = [P.gated_delta(s.double(), m, _double(w), "m.", 1e-5) for s in seqs]
    cuts = [(2, 1)] + [(1, 1)] * 400
    got = _run_in_cuts(part, None, state, seqs, cuts, 16, dtype, g, 64)
    for r in range(2):
        _close(got[r], want[r], dtype, r, f32=2e-4, bf16=0.05)


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_parallel_mixer_against_plain(dtype, fused, monkeypatch):
    """The two side by side, with the two output projections as one product and as two products and a sum."""
    from llm_rs_b200.parts import PartSpec, Runtime, parallel
    monkeypatch.setattr(parallel, "FUSE_PARALLEL", fused)
    D, g = 56, torch.Generator().manual_seed(11)
    left = {"hidden_size": D, "n_heads": 4, "n_kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.3, "sink": True,
            "qk_norm": "none", "v_norm": "head_unit", "norm_eps": 1e-5, "rot_dims": 8, "rot_base": 500.0}
    right = {"hidden_size": D, "n_heads": 3, "n_kv_heads": 1, "dim": 12, "vdim": 20, "conv": 3, "norm_eps": 1e-5}
    part = parallel.ParallelMixer(PartSpec("scored_attention", left), PartSpec("gated_delta", right), 0.6, 1.7, prefix="m.")
    w, wd = _weights(part, g, dtype, 1.5)
    part.bind(wd, Runtime(torch.device(DEV), dtype, 4096))
    assert (part.fused is not None) == fused
    m = {"left": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.3, "rot": {"base": 500.0, "dims": 8}},
         "right": {"heads": 3, "kv_heads": 1, "dim": 12, "vdim": 20, "conv": 3}, "left_scale": 0.6, "right_scale": 1.7}
    state = {n: torch.zeros(5, *shape, device=DEV) for n, shape in part.state_need().tensors.items()}
    seqs = [_rounded(torch.randn(n, D, generator=g), dtype) for n in (151, 42)]
    want = [P.parallel_mixer(s.double(), m, _double(w), "m.", 1e-5, torch.arange(len(s)))[0] for s in seqs]
    got = _run_in_cuts(part, _pages(2, 16, 8, 16, 64, dtype), state, seqs, CUTS, 16, dtype, g, 64)
    for r in range(2):
        _close(got[r], want[r], dtype, r, f32=1e-4, bf16=0.04)


# ---- whole models -----------------------------------------------------------------------------------
def _steps(mode, reqs):
    if mode == "tail":
        return RU.tail_one_by_one(reqs, tail=70)      # longer than every window but the widest
    if mode == "portions":
        return RU.portions(reqs, sizes=(1, 1, 2, 7, 2, 13, 5, 2, 31, 3, 17, 2, 64))
    return {"whole": RU.whole, "mixed": RU.mixed}[mode](reqs)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("name", list(FEKOLORN))
def test_replay_matches_plain(models, name, mode, dtype):
    from llm_rs_b200.engine import ModelRunner
    path, cfg, w, reqs, ref = models[name]
    steps = _steps(mode, reqs)
    runner = ModelRunner.from_model_dir(path, dtype=getattr(torch, dtype), max_tokens=RU.live_token_peak(steps),
                                        page_size=FEKOLORN[name][3], max_requests=4)
    free_before = [runner.manager.free_pages(g) for g in range(len(runner.manager.groups))]
    got = RU.run_steps(runner, steps)
    assert [runner.manager.free_pages(g) for g in range(len(runner.manager.groups))] == free_before, "pages were lost"
    runner.check_kernels()
    assert len(got) == sum(len(t) for t in reqs.values())
    _assert_logits(got, ref, dtype, f"{name} {mode} {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [21, 22])
@pytest.mark.parametrize("name", list(FEKOLORN))
def test_mixed_replay_with_other_cuts_and_pages_and_slots_used_again(models, name, seed, dtype):
    """Mixed batches with other seeds and portion sizes, two or three live requests, the requests twice over, so that
    every page and every state slot serves several requests."""
    from llm_rs_b200.engine import ModelRunner
    path, cfg, w, reqs, ref = models[name]
    rng = np.random.default_rng(seed)
    sizes = tuple(int(x) for x in rng.choice([2, 3, 7, 16, 31, 33, 64, 65, 129], size=5, replace=False))
    twice = {**reqs, **{r + "again": t for r, t in reqs.items()}}
    steps = RU.mixed(twice, seed=seed, max_live=2 + seed % 2, decode_tail=5 + seed % 7, sizes=sizes)
    runner = ModelRunner.from_model_dir(path, dtype=getattr(torch, dtype), max_tokens=RU.live_token_peak(steps),
                                        page_size=FEKOLORN[name][3], max_requests=3)
    got = RU.run_steps(runner, steps)
    assert len(got) == 2 * sum(len(t) for t in reqs.values())
    _assert_logits(got, ref, dtype, f"{name} seed {seed} {dtype}")


def test_residual_stream_after_every_layer(models):
    """The sum of the streams after each layer (float32 engine), read with the block's own ``leave``."""
    from llm_rs_b200.engine import ModelRunner, StepEntry
    path, cfg, w, reqs, ref = models["A"]
    toks = reqs["r3"]
    want = []
    P.forward(toks, cfg, w, residuals=want)
    runner = ModelRunner.from_model_dir(path, dtype=torch.float32, max_tokens=128, page_size=16, max_requests=2)
    seen = []
    for block in runner.model.blocks:
        inner = block.forward

        def wrapped(h, pending, ctx, cache, inner=inner, block=block):
            h, pending = inner(h, pending, ctx, cache)
            seen.append(block.leave(h, pending, None).cpu())
            return h, pending
        block.forward = wrapped
    runner.step([StepEntry("x", toks, [len(toks) - 1])])
    assert len(seen) == len(want)
    for i, (got, ref_i) in enumerate(zip(seen, want)):
        _close(got, ref_i, torch.float32, f"layer {i}", f32=1e-5)


def test_long_decoding_beyond_the_pool(models):
    """A request of 600 tokens through model F (windows only beside the recurrence) with pages for 192 tokens: the
    windows give pages back as they pass, the recurrence keeps its state. 60 tokens as portions, the other 540 decoded
    one by one."""
    from llm_rs_b200.engine import ModelRunner
    path, cfg, w, reqs, ref = models["F"]
    toks = np.random.default_rng(5).integers(0, cfg["vocab"], 600).tolist()
    want = P.forward(toks, cfg, w).numpy()
    runner = ModelRunner.from_model_dir(path, dtype=torch.float32, max_tokens=192, page_size=32, max_requests=2)
    steps = [{"entries": [{"id": "long", "tokens": toks[a:a + 30], "want": list(range(30))}], "end": []} for a in (0, 30)]
    steps += [{"entries": [{"id": "long", "tokens": [t], "want": [0]}], "end": []} for t in toks[60:]]
    got = RU.run_steps(runner, steps)
    worst, where, n = RU.max_diff(got, {"long": want})
    assert n == 600 and worst <= TOL_F32 * max(1.0, float(np.abs(want).max())), (worst, where)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(FEKOLORN))
def test_greedy_generation_through_the_engine(models, name, dtype, graphs):
    """Prompts of unequal length through ``Engine.generate``: scheduler, prompt portions, decoding (captured in CUDA
    graphs or not: the previous token, the recurrence's state and the convolutions' rows live on the device), the device
    sampler's argmax. float32 gives the plain implementation's tokens; bfloat16 may choose another token only where
    the plain logits of the two are closer than its rounding."""
    from llm_rs_b200.engine import Engine, EngineConfig
    from llm_rs_b200.sampling import SamplingParams
    path, cfg, w, reqs, ref = models[name]
    prompts = [reqs[r][:n] for r, n in zip(list(reqs)[1:4], (9, 33, 20))]
    engine = Engine(EngineConfig(model_path=path, block_pool_size=64, page_size=FEKOLORN[name][3], dtype=dtype,
                                 max_requests=4, cuda_graphs=graphs, prefill_chunk=16, max_tokens_per_step=24))
    got = engine.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12, ignore_eos=True))
    for prompt, new in zip(prompts, got):
        assert len(new) == 12
        toks = list(prompt)
        for t in new:
            row = P.forward(toks, cfg, w)[-1]
            gap = float(row.max() - row[t])
            assert gap <= (1e-4 if dtype == "float32" else 0.06) * float(row.abs().max()), (name, gap)
            toks.append(t)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_program_on_a_fekolorn_folder(models, tmp_path, dtype):
    """bin/trace_run picks the design by config.json and replays a mixed trace."""
    path, cfg, w, reqs, ref = models["B"]
    steps = RU.want_only(RU.mixed(reqs, seed=9), {r: set(range(0, len(t), 3)) | {len(t) - 1} for r, t in reqs.items()})
    out_dir = tmp_path / "out"
    lines = [json.dumps({"step": i, **st}) for i, st in enumerate(steps)]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", dtype, "--out", str(out_dir),
         "--max-tokens", str(RU.live_token_peak(steps)), "--max-requests", "4", "--page-size", "8"],
        input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split("\n")[:len(steps)] == [f"done {i}" for i in range(len(steps))]
    at, got, V = {}, {}, cfg["vocab"]
    for i, st in enumerate(steps):
        n_want = sum(len(e["want"]) for e in st["entries"])
        if not n_want:
            assert not (out_dir / f"{i}.f32").exists()
        else:
            data = np.fromfile(out_dir / f"{i}.f32", dtype="<f4").reshape(-1, V)
            assert data.shape[0] == n_want
        k = 0
        for e in st["entries"]:
            base = at.get(e["id"], 0)
            for wnt in e["want"]:
                got[(e["id"], base + wnt)] = data[k]
                k += 1
            at[e["id"]] = base + len(e["tokens"])
    _assert_logits(got, ref, dtype, f"trace program {dtype}")


def test_command_line_writes_and_runs_a_fekolorn_folder(tmp_path):
    """``random_model`` from a config.json of the design, then ``run_model`` with sampling switched off: the registry,
    the loader, the engine and the sampler through the command line; the tokens are the plain implementation's."""
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(FEKOLORN["A"][0]))
    out = tmp_path / "model"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    run = lambda *a: subprocess.run([sys.executable, "-m", "llm_rs_b200.cli", *a], cwd=root, capture_output=True,
                                    text=True, timeout=600)
    made = run("random_model", "--config", str(cfg_path), "--out", str(out), "--seed", "5", "--sigma", "0.15",
               "--norm-jitter", "0.2")
    assert made.returncode == 0, made.stderr[-2000:]
    prompt = [5, 17, 3, 9, 200, 41, 7, 7, 150]
    done = run("run_model", "--model-path", str(out), "--prompt-ids", ",".join(map(str, prompt)), "--dtype", "float32",
               "--max-new-tokens", "10", "--ignore-eos", "--page-size", "16", "--block-pool-size", "32")
    assert done.returncode == 0, done.stderr[-2000:]
    lines = dict(l.split(":", 1) for l in done.stdout.splitlines() if ":" in l)
    got = [int(t) for t in lines["Generated token ids"].split(",")]
    cfg, w = P.load_model_dir(str(out))
    seq = list(prompt)
    for tok in got:
        row = P.forward(seq, cfg, w)[-1]
        assert float(row.max() - row[tok]) <= 1e-4 * float(row.abs().max())
        seq.append(tok)
    assert len(got) == 10
