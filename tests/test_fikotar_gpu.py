"""The side-by-side design on the GPU against its plain implementation.

Each mechanism alone (kernels, parts and one-layer models, with weights made so that the
key in question stands out), then whole models in every replay regime, both precisions,
with page pools and state slots so small that everything freed is used again, and
generation through the engine's own entry point and scheduler.
"""
import copy

import pytest
import torch

import helpers as H
import fikotar_plain as P

pytestmark = pytest.mark.gpu

# largest |difference| / largest |logit|, and rms of the difference / rms of the logits.  The
# float32 bounds are the sharp ones; in bfloat16 every product reads activations rounded to
# eight bits, and rounding alone moves single logits of the two tiniest models by a tenth
# (the wider one stays under 0.1).
TOL = {torch.float32: 6e-5, torch.bfloat16: 0.25}
TOL_RMS = {torch.float32: 1e-5, torch.bfloat16: 6e-2}


def _runner(model_dir, dtype, page_size, num_pages, max_requests=4):
    from binfer_b200.engine import make_env, make_runner, model_from_dir
    env = make_env(dtype)
    model = model_from_dir(model_dir, env)
    return make_runner(model, env, page_size=page_size, num_pages=num_pages,
                       max_requests=max_requests)


def _compare(got, ref, dtype, what, tol_scale=1.0):
    """In bfloat16 a router may decide a close call the other way once its input is rounded,
    which moves that token's logits by more than rounding does: up to two in a hundred
    positions may lie over the bound there (they stay out of the rms too); in float32 none."""
    assert got, "the trace produced no logits"
    worst, worst_at, over = 0.0, None, []
    for (rid, pos), row in got.items():
        e = H.rel_err(row, ref[rid][pos])
        if not e <= TOL[dtype] * tol_scale:
            over.append((rid, pos))
        if not e <= worst:
            worst, worst_at = e, (rid, pos)
    allowed = 0 if dtype == torch.float32 else len(got) // 50
    assert len(over) <= allowed, (f"{what}: {len(over)} of {len(got)} positions over the bound, "
                                  f"worst relative error {worst:.3g} at {worst_at}")
    keep = [k for k in got if k not in set(over)]
    g = torch.stack([got[k] for k in keep])
    r = torch.stack([ref[rid][pos] for (rid, pos) in keep])
    assert H.rel_rms(g, r) <= TOL_RMS[dtype] * tol_scale, f"{what}: rms error {H.rel_rms(g, r):.3g}"
    for rid, lg in ref.items():
        assert all((rid, p) in got for p in range(lg.shape[0])), f"{what}: {rid} incomplete"


def _all_regimes(reqs, tail=10):
    return {"whole": H.trace_whole(reqs), "tail": H.trace_decode_tail(reqs, tail),
            "portions": H.trace_portions(reqs), "mixed": H.trace_mixed(reqs)}


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("width", [40, 256, 1000])
def test_layer_norm_with_its_pending_adds(cuda_device, dtype, width):
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(width)
    x = torch.randn(7, width, generator=g) * 3 + 5.0          # a mean far from zero
    d1 = torch.randn(7, width, generator=g).to(dtype)
    d2 = (torch.randn(7, width, generator=g) * 2).to(dtype)
    w, b = torch.randn(width, generator=g), torch.randn(width, generator=g)
    rows = torch.tensor([5, 0, 3], dtype=torch.int32)
    tol = 2e-6 if dtype == torch.float32 else 5e-3
    for deltas in ((None, None), (d1, None), (d1, d2)):
        total = x.double() + sum(d.double() for d in deltas if d is not None)
        want = P.layer_norm(total, w.double(), b.double(), 1e-5)
        resid = x.to(cuda_device)
        out = torch.empty(7, width, dtype=dtype, device=cuda_device)
        dev = [None if d is None else d.to(cuda_device) for d in deltas]
        ops.add_layernorm(resid, dev[0], dev[1], w.to(cuda_device), b.to(cuda_device), out, 1e-5)
        assert H.rel_err(out.cpu(), want) <= tol
        assert H.rel_err(resid.cpu(), total) <= 1e-6          # the sum is written back
        resid = x.to(cuda_device)
        some = torch.empty(3, width, dtype=dtype, device=cuda_device)
        ops.add_layernorm(resid, dev[0], dev[1], w.to(cuda_device), b.to(cuda_device), some, 1e-5,
                          rows=rows.to(cuda_device), write_back=False)
        assert H.rel_err(some.cpu(), want[rows.long()]) <= tol
        assert torch.equal(resid.cpu(), x)                    # and here it is not


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("experts,top,ff,shared", [(4, 2, 24, 40), (5, 1, 40, 0), (3, 3, 56, 16),
                                                   (40, 4, 8, 8), (1, 1, 30, 0)])
def test_mixture_of_experts_alone(cuda_device, dtype, experts, top, ff, shared):
    """The feed-forward part by itself: router, choice, weights, experts, shared expert."""
    from binfer_b200.config import MoESpec
    from binfer_b200.parts.base import BuildEnv
    from binfer_b200.parts.moe import MoEFeedForward
    from binfer_b200.weights import random_tensors
    width, T = 48, 37
    part = MoEFeedForward(MoESpec(num_experts=experts, top=top, expert_size=ff, shared_size=shared,
                                  shared_gate=bool(shared)), width, "m.",
                          BuildEnv(dtype, cuda_device))
    w = random_tensors(part.param_specs(), 3, 0.15, 0.1, dtype)
    w["m.router"] = w["m.router"].float() * 4.0               # logits well apart
    part.load(lambda s: w[s.name].to(cuda_device, torch.float32 if s.role == "vector" else dtype))
    h = torch.randn(T, width, generator=torch.Generator().manual_seed(5)).to(dtype)
    mlp = {"router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    want = P.mixture_of_experts(h.double(), {n: t.double() for n, t in w.items()}, "m.", mlp)
    got = part.forward(h.to(cuda_device), None).cpu()
    assert H.rel_err(got, want) <= (2e-5 if dtype == torch.float32 else 3e-2)
    # one token alone gives what it gives in the batch (in bfloat16, where experts are many
    # enough, a lone token reads its chosen experts only: another kernel, the same result)
    from binfer_b200.profiling import Profiler
    prof = Profiler()
    alone = part.forward(h[11:12].to(cuda_device), None).cpu()
    prof.stop()
    ops_seen = set(prof.collect())
    from binfer_b200.csrc import ops
    ops.set_profiler(None)
    assert H.rel_err(alone, got[11:12]) <= (1e-6 if dtype == torch.float32 else 2e-2)
    assert H.rel_err(alone, want[11:12]) <= (2e-5 if dtype == torch.float32 else 3e-2)
    assert ("moe_sparse" in ops_seen) == (dtype == torch.bfloat16 and 2 * top <= experts)


def _one_layer(left, right, mlp=None, ls=1.0, rs=1.0, vocab=260, width=48, eps=1e-5):
    return {"architecture": "Fikotar", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "logit_scale": 1.0, "layers": [H._fik_layer(left, right, mlp, ls, rs)]}


@pytest.mark.parametrize("heads,dk,dv,decay,rot", [
    (2, 16, 32, (0.9, 0.999), 16), (1, 40, 24, (1.0,), 20), (3, 8, 8, (0.5, 0.98, 0.75), 0),
    (2, 72, 96, (0.97, 0.99), 72), (2, 12, 20, (0.95, 0.9), 4), (1, 264, 40, (0.99,), 64),
    (1, 6, 300, (0.98,), 6)])
def test_retention_alone(cuda_device, tmp_path, heads, dk, dv, decay, rot):
    """One layer whose attention branch counts for nothing: a prompt at once, portions, and
    token by token from the first token on, over 200 tokens."""
    right = H._fik_right(heads, dk, dv, decay, rot or 2)
    if not rot:
        right.pop("rot")
    raw = _one_layer(H._fik_left(2, 1, 8, 8, 5, 0, 4), right, None, ls=0.0, rs=1.5)
    d = H.make_fikotar_dir(tmp_path, "A", raw=raw, tag=f"r{heads}{dk}{dv}")
    raw, w = H.read_model_dir(d)
    reqs = {"a": H.random_tokens(200, raw["vocab"], 3), "b": H.random_tokens(37, raw["vocab"], 4)}
    ref = {r: P.forward(raw, w, t) for r, t in reqs.items()}
    for name, steps in _all_regimes(reqs, tail=150).items():
        got = H.run_trace(_runner(d, torch.float32, 8, H.peak_pages(steps, 8)), steps)
        _compare(got, ref, torch.float32, f"retention {heads}x{dk}x{dv}/{name}")


def _stand_out(raw, toks, marked, amp=3.0, boost=30.0):
    """A tweak for a one-layer model whose retention branch counts for nothing.  One
    direction ``e`` of the width is taken out of every embedding and put back, large, into
    those of the tokens at the positions ``marked``; the first query head of every group
    answers ``e`` with a strong fixed vector in the sizes that are not rotated, and the
    group's key head projects exactly like it, so that a marked query's score with a marked
    key towers over all others.  The convolutions of q and k pass the newest token alone,
    so that a mark stays on its token; the value projection is blind to ``e``."""
    mx = raw["layers"][0]["mixer"]["left"]
    H_, G_, dk, rot = mx["heads"], mx["kv_heads"], mx["dim"], mx["rot"]["dims"]

    def tweak(w):
        p = "l0.mix.left."
        gen = torch.Generator().manual_seed(9)
        e = torch.randn(w["embed"].shape[1], generator=gen)
        e = (e / e.norm()).to(w["embed"].dtype)
        a = torch.randn(dk, generator=gen).to(w["embed"].dtype)
        a[:rot] = 0.0
        w["embed"] -= torch.outer(w["embed"] @ e, e)
        for pos in marked:
            w["embed"][toks[pos]] += e * amp
        w["l0.norm1"][:] = 1.0
        w["l0.norm1.b"][:] = 0.0
        for g in range(G_):
            h0 = g * (H_ // G_)
            w[p + "q"][h0 * dk:(h0 + 1) * dk] += boost * torch.outer(a, e)
            w[p + "k"][g * dk:(g + 1) * dk] = w[p + "q"][h0 * dk:(h0 + 1) * dk]
        for n in ("q.conv", "k.conv"):
            if p + n in w:
                w[p + n][:] = 0.0
                w[p + n][:, -1] = 1.0
        w[p + "v"] -= torch.outer(w[p + "v"] @ e, e)
        w[p + "sink"][:] = torch.tensor([1.0, -2.0, 0.5, 3.0][:H_])
    return tweak


def _distinct_tokens(n, vocab, seed):
    return torch.randperm(vocab, generator=torch.Generator().manual_seed(seed))[:n].tolist()


# window 20, 5 kept tokens, pages of 8: the marked key and the query that asks for it
EDGES = {"window_in": (41, 60), "window_out": (40, 60), "kept_in": (4, 150), "kept_out": (5, 150),
         "far_kept": (0, 230), "page_border": (8, 27), "second_token": (0, 1)}


@pytest.mark.parametrize("case", sorted(EDGES))
def test_attention_alone_at_its_edges(cuda_device, tmp_path, case):
    """One layer whose retention branch counts for nothing.  A marked key sits just inside
    or just outside the window of a marked query, among the kept first tokens or just
    behind them, hundreds of tokens back, or at a page's border; the plain implementation
    first shows that a window or a kept count one token off moves that query's logits far
    beyond the bound, then the engine is held to it in every regime (the marked query is
    once part of a prompt and once decoded alone)."""
    key, query = EDGES[case]
    left = H._fik_left(4, 2, 16, 24, 20, 5, 8, conv=3, scale=0.6)
    raw = _one_layer(left, H._fik_right(1, 8, 8, (0.9,), 8), None, ls=1.3, rs=0.0, vocab=400)
    toks = _distinct_tokens(240, raw["vocab"], 21)
    d = H.make_fikotar_dir(tmp_path, "A", raw=raw, tweak=_stand_out(raw, toks, (key, query)),
                           tag=case)
    raw, w = H.read_model_dir(d)
    ref = {"a": P.forward(raw, w, toks)}
    if case not in ("far_kept", "page_border", "second_token"):
        off = copy.deepcopy(raw)
        m = off["layers"][0]["mixer"]["left"]["mask"]
        if case.startswith("window"):
            m["size"] += 1 if case == "window_out" else -1
        else:
            m["keep_first"] += 1 if case == "kept_out" else -1
        moved = H.rel_err(P.forward(off, w, toks)[query], ref["a"][query])
        assert moved > 100 * TOL[torch.float32], f"{case}: one token off moves the logits by {moved:.3g} only"
    reqs = {"a": toks}
    for name, steps in _all_regimes(reqs, tail=100).items():
        got = H.run_trace(_runner(d, torch.float32, 8, H.peak_pages(steps, 8)), steps)
        _compare(got, ref, torch.float32, f"attention {case}/{name}")


def test_sink_and_first_tokens(cuda_device, tmp_path):
    """At the first tokens the sink is most of the denominator: with large sink logits a wrong
    or missing sink would move every early logit."""
    left = H._fik_left(3, 3, 12, 20, 6, 2, 12, conv=2, scale=0.4)
    raw = _one_layer(left, H._fik_right(1, 8, 8, (0.9,), 8), None, ls=1.0, rs=0.0)

    def tweak(w):
        w["l0.mix.left.sink"][:] = torch.tensor([4.0, -3.0, 1.5])

    d = H.make_fikotar_dir(tmp_path, "A", raw=raw, tweak=tweak, tag="sink")
    raw, w = H.read_model_dir(d)
    toks = H.random_tokens(30, raw["vocab"], 8)
    ref = {"a": P.forward(raw, w, toks)}
    w0 = dict(w)
    w0["l0.mix.left.sink"] = torch.full((3,), -60.0)
    assert H.rel_err(P.forward(raw, w0, toks)[:3], ref["a"][:3]) > 1e-2
    for name, steps in _all_regimes({"a": toks}, tail=29).items():
        got = H.run_trace(_runner(d, torch.float32, 4, 10), steps)
        _compare(got, ref, torch.float32, f"sink/{name}")


@pytest.mark.parametrize("W,keep,T,marked", [
    (20, 5, 240, (4, 150)), (20, 5, 240, (5, 150)), (64, 70, 500, (69, 420)),
    (130, 3, 700, (500, 629)), (130, 3, 700, (499, 629)), (64, 0, 300, (100, 163)),
    (1000, 2, 300, (0, 299)), (None, 0, 300, (10, 299))])
def test_tensor_core_attention_beside_the_plain_kernel(cuda_device, tmp_path, W, keep, T, marked):
    """bfloat16: the tiled kernel and the one-warp-per-row kernel on the same one-layer model
    with a marked key at a window's or the kept tokens' edge, whole, cut and token by token
    (a single token's key tiles are shared out over CTAs and merged): both within rounding of
    the plain implementation, and of each other.  (The last case has no window at all.)"""
    from binfer_b200.csrc import ops
    from binfer_b200.parts import attention_conv_window as mod
    from binfer_b200.profiling import Profiler
    left = H._fik_left(4, 2, 32, 48, W, keep, 16, conv=3, scale=0.5)
    raw = _one_layer(left, H._fik_right(1, 8, 8, (0.9,), 8), None, ls=1.3, rs=0.0, vocab=800,
                     width=64)
    toks = _distinct_tokens(T, raw["vocab"], 22)
    d = H.make_fikotar_dir(tmp_path, "A", torch.bfloat16, raw=raw,
                           tweak=_stand_out(raw, toks, marked, boost=12.0), tag=f"tc{W}{keep}")
    raw, w = H.read_model_dir(d)
    ref = {"a": P.forward(raw, w, toks)}
    regimes = {"whole": H.trace_whole({"a": toks}), "tail": H.trace_decode_tail({"a": toks}, 150),
               "portions": H.trace_portions({"a": toks}, sizes=(70, 5, 130, 2, 64, 33))}
    keep_rows = lambda rid, pos: pos % 7 == 0 or pos in marked or pos > T - 3   # noqa: E731
    outs = []
    for on in (True, False):
        mod.TENSOR_CORES = on
        seen = set()
        try:
            got = {}
            for name, steps in regimes.items():
                steps = H.thin_wants(steps, keep_rows)
                prof = Profiler()
                got[name] = H.run_trace(_runner(d, torch.bfloat16, 16, H.peak_pages(steps, 16)),
                                        steps)
                prof.stop()
                seen |= set(prof.collect())
                worst = max(H.rel_err(row, ref[rid][pos]) for (rid, pos), row in got[name].items())
                assert worst <= 0.05, f"{name} (tensor cores {on}): {worst:.3g}"
        finally:
            ops.set_profiler(None)
            mod.TENSOR_CORES = True
        assert ("pwm_attention" in seen) == on and ("paged_attention_generic" in seen) != on
        outs.append(got)
    for name in outs[0]:
        worst = max(H.rel_err(outs[0][name][k], outs[1][name][k]) for k in outs[0][name])
        assert worst <= 0.05, f"{name}: the two kernels differ by {worst:.3g}"


# ----------------------------------------------------------------------- whole models
LENGTHS = {"A": [5, 17, 33, 70, 121], "B": [1, 9, 40, 70, 101], "C": [3, 30, 64, 47, 2],
           "D": [2, 45, 150, 210, 90]}


def _requests(which, extra=()):
    vocab = H.FIK[which]["raw"]["vocab"]
    lens = list(LENGTHS[which]) + list(extra)
    return {f"r{i}": H.random_tokens(n, vocab, 100 * i + n) for i, n in enumerate(lens)}


@pytest.fixture(scope="module")
def plain_logits(tmp_path_factory):
    cache = {}

    def get(which, dtype, reqs):
        d = H.make_fikotar_dir(tmp_path_factory.getbasetemp(), which, dtype)
        raw, w = H.read_model_dir(d)
        out = cache.setdefault((which, dtype), {})
        for rid, toks in reqs.items():
            k = (rid, tuple(toks))
            if k not in out:
                out[k] = P.forward(raw, w, toks)
        return d, {rid: out[(rid, tuple(toks))] for rid, toks in reqs.items()}

    return get


@pytest.mark.parametrize("which,dtype", [("A", torch.float32), ("B", torch.float32),
                                         ("C", torch.float32), ("A", torch.bfloat16),
                                         ("B", torch.bfloat16), ("C", torch.bfloat16),
                                         ("D", torch.bfloat16)],
                         ids=["A-f32", "B-f32", "C-f32", "A-bf16", "B-bf16", "C-bf16", "D-bf16"])
@pytest.mark.parametrize("regime", ["whole", "tail", "portions", "mixed"])
def test_replay(cuda_device, plain_logits, which, dtype, regime):
    """Seven requests through four state slots and page pools of exactly the peak need."""
    reqs = _requests(which, (55, 61) if regime == "mixed" else ())
    model_dir, ref = plain_logits(which, dtype, reqs)
    steps = _all_regimes(reqs)[regime]
    ps = H.FIK[which]["page_size"]
    runner = _runner(model_dir, dtype, ps, H.peak_pages(steps, ps))
    got = H.run_trace(runner, steps)
    assert not runner.cache.requests and all(g.pool.num_held == 0 for g in runner.cache.groups)
    assert runner.cache.slots.num_free == 4
    _compare(got, ref, dtype, f"{which}/{regime}")


@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_regimes_agree_bitwise_in_float32(cuda_device, plain_logits, which):
    """Every sum's order depends on positions alone: cutting and batching change no bit."""
    reqs = _requests(which)
    model_dir, _ = plain_logits(which, torch.float32, reqs)
    ps = H.FIK[which]["page_size"]
    outs = []
    for steps in _all_regimes(reqs).values():
        outs.append(H.run_trace(_runner(model_dir, torch.float32, ps, H.peak_pages(steps, ps)),
                                steps))
    for other in outs[1:]:
        for key, row in outs[0].items():
            assert torch.equal(row, other[key]), f"{which}: logits at {key} depend on the cut"


def test_long_decoding(cuda_device, plain_logits):
    """A short prompt, then 300 tokens one by one: the window passes over decoded tokens, the
    pages behind it are given back while those of the kept first tokens stay."""
    which, dtype = "B", torch.float32
    reqs = {"long": H.random_tokens(304, H.FIK[which]["raw"]["vocab"], 7)}
    model_dir, ref = plain_logits(which, dtype, reqs)
    steps = H.trace_decode_tail(reqs, tail=300)
    runner = _runner(model_dir, dtype, 4, 12)        # far fewer pages than 304 tokens fill
    _compare(H.run_trace(runner, steps), ref, dtype, "long decoding")


def test_decoding_from_captured_steps(cuda_device, plain_logits):
    """Steps of single tokens replayed from CUDA graphs (padded rows use the scratch page and
    the scratch state slot) give what eager steps give."""
    which, dtype = "A", torch.float32
    reqs = _requests(which, (55, 61))
    model_dir, ref = plain_logits(which, dtype, reqs)
    steps = H.trace_mixed(reqs, tail=20)
    ps = H.FIK[which]["page_size"]
    runner = _runner(model_dir, dtype, ps, H.peak_pages(steps, ps))
    runner.enable_decode_graphs(max_batch=4, max_seq_len=256)
    got = H.run_trace(runner, steps)
    assert getattr(runner, "graph_replays", 0) > 0
    _compare(got, ref, dtype, "captured decode steps")


# ------------------------------------------------------------------------- generation
@pytest.mark.parametrize("graphs,step_tokens", [(True, 2048), (False, 7)],
                         ids=["graphs", "portions"])
def test_greedy_generation_through_the_engine(cuda_device, tmp_path, graphs, step_tokens):
    """Prompts of 5/17/33/2 tokens through ``Engine.generate``: the scheduler's admission,
    portions of at most seven tokens beside decoding (second case), captured decode steps
    (first case); every token is the plain implementation's choice."""
    from binfer_b200 import Engine
    d = H.make_fikotar_dir(tmp_path, "A")
    raw, w = H.read_model_dir(d)
    prompts = [H.random_tokens(n, raw["vocab"], n) for n in (5, 17, 33, 2)]
    eng = Engine(d, "float32", num_pages=40, page_size=16, max_seq_len=128, max_batch_size=3,
                 max_tokens_per_step=step_tokens, cuda_graphs=graphs)
    got = eng.generate(prompts, max_tokens=12, ignore_eos=True)
    for p, out in zip(prompts, got):
        assert len(out) == 12
        logits = P.forward(raw, w, list(p) + list(out))
        for n, tok in enumerate(out):
            row = logits[len(p) - 1 + n]
            assert float(row[tok]) >= float(row.max()) - 1e-4 * float(row.abs().max()), (
                f"token {n} after a prompt of {len(p)}: {tok}, plain {int(row.argmax())}")
    st = eng.stats()
    assert st["pages_free"] == st["pages_total"]
    if graphs:
        assert getattr(eng.runner, "graph_replays", 0) > 0


def test_trace_replay_tool_with_four_state_slots(cuda_device, tmp_path):
    """``bin/trace_run`` as a user runs it on a side-by-side model: six requests through its
    four state slots and a page pool sized by ``--max-tokens``."""
    import test_trace_run_gpu as TR
    d = H.make_fikotar_dir(tmp_path, "B")
    raw, w = H.read_model_dir(d)
    reqs = {f"r{i}": H.random_tokens(n, raw["vocab"], 31 * i + n)
            for i, n in enumerate([70, 33, 90, 12, 64, 41])}
    steps = H.trace_mixed(reqs)
    live, peak = {}, 0
    for st in steps:
        for e in st["entries"]:
            live[e["id"]] = live.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // 64) * 64 for n in live.values()))
        for rid in st["end"]:
            live.pop(rid)
    out_dir = str(tmp_path / "out")
    TR._replay(d, "float32", steps, out_dir, peak)
    got = TR._collect(steps, out_dir, raw["vocab"])
    ref = {rid: P.forward(raw, w, toks) for rid, toks in reqs.items()}
    worst = max(H.rel_err(row, ref[rid][p]) for (rid, p), row in got.items())
    assert got and worst <= TOL[torch.float32], f"worst relative error {worst:.3g}"
