"""The hybrid design on the GPU against its plain implementation.

Each mechanism alone (one-layer models, weights made so that the key in question stands
out), then whole models in every replay regime, both precisions, with page pools and state
slots so small that everything freed is used again, and generation through the engine's
own entry point and scheduler.
"""
import copy

import pytest
import torch

import helpers as H
import gukidra_plain as G

pytestmark = pytest.mark.gpu

# largest |difference| / largest |logit|, and rms of the difference / rms of the logits.  The
# float32 bounds are the sharp ones.  In bfloat16 every product reads a stream of magnitude
# ten rounded to eight bits and every sublayer's output is normed to unit size before it is
# added, so rounding alone moves single logits of these tiny models by a tenth.
TOL = {torch.float32: 6e-5, torch.bfloat16: 0.25}
TOL_RMS = {torch.float32: 1e-5, torch.bfloat16: 6e-2}


def _runner(model_dir, dtype, page_size, num_pages, max_requests=4):
    from binfer_b200.engine import make_env, make_runner, model_from_dir
    env = make_env(dtype)
    model = model_from_dir(model_dir, env)
    return make_runner(model, env, page_size=page_size, num_pages=num_pages,
                       max_requests=max_requests)


def _compare(got, ref, dtype, what, tol_scale=1.0):
    assert got, "the trace produced no logits"
    worst, worst_at = 0.0, None
    for (rid, pos), row in got.items():
        e = H.rel_err(row, ref[rid][pos])
        if not e <= worst:
            worst, worst_at = e, (rid, pos)
    assert worst <= TOL[dtype] * tol_scale, f"{what}: worst relative error {worst:.3g} at {worst_at}"
    g = torch.stack([row for row in got.values()])
    r = torch.stack([ref[rid][pos] for (rid, pos) in got])
    assert H.rel_rms(g, r) <= TOL_RMS[dtype] * tol_scale, f"{what}: rms error {H.rel_rms(g, r):.3g}"
    for rid, lg in ref.items():
        assert all((rid, p) in got for p in range(lg.shape[0])), f"{what}: {rid} incomplete"


def _all_regimes(reqs, tail=10):
    return {"whole": H.trace_whole(reqs), "tail": H.trace_decode_tail(reqs, tail),
            "portions": H.trace_portions(reqs), "mixed": H.trace_mixed(reqs)}


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("width", [40, 256, 1000])
def test_norm_on_a_sublayer_output(cuda_device, dtype, width):
    from binfer_b200.csrc import ops
    g = torch.Generator().manual_seed(width)
    x = torch.randn(7, width, generator=g)
    y = (torch.randn(7, width, generator=g) * 3).to(dtype)
    w = torch.randn(width, generator=g) * 0.2
    want = x.double() + G.unit_offset_rms_norm(y.double(), w.double(), 1e-5)
    resid = x.to(cuda_device)
    reading = None if dtype == torch.float32 else torch.empty(7, width, dtype=dtype,
                                                              device=cuda_device)
    ops.rmsnorm_add(resid, y.to(cuda_device), (w + 1.0).to(cuda_device), reading, 1e-5)
    assert H.rel_err(resid.cpu(), want) <= (2e-6 if dtype == torch.float32 else 2e-6)
    if reading is not None:
        assert torch.equal(reading.cpu(), resid.cpu().to(dtype))


def _one_layer(layer, vocab=260, width=48, scale=4.0, eps=1e-6):
    return {"architecture": "Gukidra", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": scale}, "layers": [layer]}


@pytest.mark.parametrize("heads,dk,dv,cap,ff", [(2, 16, 32, 8.0, None), (1, 40, 24, 2.0, 64),
                                                (3, 8, 8, 30.0, None), (2, 72, 96, 6.0, None),
                                                (2, 12, 20, 9.0, None), (1, 256, 40, 12.0, None)])
def test_matrix_memory_alone(cuda_device, tmp_path, heads, dk, dv, cap, ff):
    """One memory layer: a prompt at once, portions, and token by token from the first
    token on, over 200 tokens.  The gate weights are scaled up so that pre-activations
    reach the cap, forget gates close and the running maximum moves."""
    raw = _one_layer(H._guk_layer("mlstm", H._guk_mlstm(heads, dk, dv, cap), ff))

    def tweak(w):
        w["l0.mix.i"] *= 6.0
        w["l0.mix.f"] *= 6.0
        w["l0.mix.f.b"] -= 1.0

    d = H.make_gukidra_dir(tmp_path, "A", raw=raw, tweak=tweak, tag=f"m{heads}{dk}{dv}")
    raw, w = H.read_model_dir(d)
    reqs = {"a": H.random_tokens(200, raw["vocab"], 3), "b": H.random_tokens(37, raw["vocab"], 4)}
    ref = {r: G.forward(raw, w, t) for r, t in reqs.items()}
    for name, steps in _all_regimes(reqs, tail=150).items():
        got = H.run_trace(_runner(d, torch.float32, 8, H.peak_pages(steps, 8)), steps)
        _compare(got, ref, torch.float32, f"memory {heads}x{dk}x{dv}/{name}")


def _stand_out(raw, toks, marked, layer=0, amp=2.0, boost=20.0):
    """A tweak for a one-layer attention model.  One direction ``e`` of the width is taken out
    of every embedding and put back, large, into those of the tokens at the positions
    ``marked``; the first query head of every group answers ``e`` with a strong fixed
    vector and the group's key head projects exactly like it, so that a marked query's score
    with a marked key towers over all others; the value projection is blind to ``e``, so
    that marked tokens' values differ like any others'."""
    mx = raw["layers"][layer]["mixer"]
    H_, G_, dk = mx["heads"], mx["kv_heads"], mx["dim"]

    def tweak(w):
        p = f"l{layer}.mix."
        gen = torch.Generator().manual_seed(9)
        e = torch.randn(w["embed"].shape[1], generator=gen)
        e = (e / e.norm()).to(w["embed"].dtype)
        a = torch.randn(dk, generator=gen).to(w["embed"].dtype)
        w["embed"] -= torch.outer(w["embed"] @ e, e)
        for pos in marked:
            w["embed"][toks[pos]] += e * amp / raw["embedding"]["scale"]
        for g in range(G_):
            h0 = g * (H_ // G_)
            w[p + "q"][h0 * dk:(h0 + 1) * dk] += boost * torch.outer(a, e)
            w[p + "k"][g * dk:(g + 1) * dk] = w[p + "q"][h0 * dk:(h0 + 1) * dk]
        w[p + "k.norm"][:] = w[p + "q.norm"]
        w[p + "v"] -= torch.outer(w[p + "v"] @ e, e)
    return tweak


def _distinct_tokens(n, vocab, seed):
    return torch.randperm(vocab, generator=torch.Generator().manual_seed(seed))[:n].tolist()


@pytest.mark.parametrize("case", ["window", "block", "far_block", "small_window"])
def test_attention_alone_at_its_edges(cuda_device, tmp_path, case):
    """One attention layer.  A marked key sits just inside the window of one marked query and
    just outside that of the next; or a marked block is first seen by one query and not yet
    by the one before; or the marked block lies hundreds of tokens back.  First the plain
    implementation shows that the case is sharp (a window or a block one token off moves
    the logits far beyond the bound), then every regime must agree with it."""
    if case == "small_window":
        W, P, T = 3, 8, 60          # tokens leave the window long before their block is seen
        mx = H._guk_attn(4, 2, 16, 24, W, P, 4, scale=0.9)
        marked, probes = list(range(8, 16)) + [18, 19, 20], [18, 19, 20]
    elif case == "window":
        W, P, T = 12, 4, 70
        mx = H._guk_attn(4, 2, 32, 16, W, P, 8, scale=0.5)
        marked, probes = [30, 41, 42], [41, 42]          # 30 is the last key 41 sees; 42 does not
    elif case == "block":
        W, P, T = 10, 6, 70
        mx = H._guk_attn(2, 1, 32, 48, W, P, 8, scale=0.5)
        marked, probes = list(range(12, 18)) + [26, 27], [26, 27]   # block 2 ends at 17 = 27 - W
    else:
        W, P, T = 16, 8, 420
        mx = H._guk_attn(6, 3, 16, 16, W, P, 4, scale=0.9)
        marked, probes = list(range(8, 16)) + [300, 419], [300, 419]
    raw = _one_layer(H._guk_layer("attention", mx, 64), vocab=500)
    toks = _distinct_tokens(T, 500, 21)
    d = H.make_gukidra_dir(tmp_path, "A", raw=raw, tweak=_stand_out(raw, toks, marked), tag=case)
    raw, w = H.read_model_dir(d)
    ref = {"a": G.forward(raw, w, toks)}
    for key, delta in (("size", 1), ("size", -1), ("pool", 1)):
        off = copy.deepcopy(raw)
        off["layers"][0]["mixer"]["mask"][key] += delta
        wrong = G.forward(off, w, toks)
        moved = max(H.rel_err(wrong[p], ref["a"][p]) for p in probes)
        assert moved > 100 * TOL[torch.float32], f"{case}: mask.{key}{delta:+d} moves {moved:.2g}"
    for name, steps in _all_regimes({"a": toks}, tail=T - 5).items():
        got = H.run_trace(_runner(d, torch.float32, 4, H.peak_pages(steps, 4)), steps)
        _compare(got, ref, torch.float32, f"attention/{case}/{name}")


def test_attention_sink_and_first_tokens(cuda_device, tmp_path):
    """The first tokens of a sequence, where the sink holds most of the weight: without it the
    first token's output would be its own value whatever the score."""
    raw = _one_layer(H._guk_layer("attention", H._guk_attn(2, 2, 8, 8, 4, 2, 8, scale=0.2)))
    d = H.make_gukidra_dir(tmp_path, "A", raw=raw, tag="sink")
    raw, w = H.read_model_dir(d)
    toks = H.random_tokens(9, raw["vocab"], 1)
    ref = {"a": G.forward(raw, w, toks)}
    steps = H.trace_decode_tail({"a": toks}, tail=8)
    _compare(H.run_trace(_runner(d, torch.float32, 16, 2), steps), ref, torch.float32, "sink")


@pytest.mark.parametrize("W,P,T,marked", [
    (40, 8, 300, list(range(16, 24)) + [100, 139, 140, 250, 299]),
    # long enough for single tokens to share their key tiles out over several CTAs
    (200, 4, 520, list(range(16, 20)) + [250, 449, 450, 519])], ids=["short", "long"])
def test_tensor_core_attention_beside_the_plain_kernel(cuda_device, tmp_path, W, P, T, marked):
    """bfloat16: the tiled tensor-core kernel (rows of a group's heads side by side, prompt
    portions and single tokens, whose keys are shared out over warps and, in long contexts,
    over CTAs with a merge) and the one-warp-per-row kernel give the same logits to
    rounding, on a case whose marked keys make a wrong mask show."""
    import importlib
    from binfer_b200.csrc import ops
    mod = importlib.import_module("binfer_b200.parts.attention_pooled")
    mx = H._guk_attn(6, 2, 32, 48, W, P, 16, scale=0.4)
    raw = _one_layer(H._guk_layer("attention", mx, 64), vocab=600, width=64)
    toks = _distinct_tokens(T, 600, 33)
    d = H.make_gukidra_dir(tmp_path, "A", torch.bfloat16, raw=raw,
                           tweak=_stand_out(raw, toks, marked), tag=f"tc{T}")
    raw, w = H.read_model_dir(d)
    ref = {"a": G.forward(raw, w, toks)}
    outs = []
    for on in (True, False):
        seen = set()

        class Names:
            def begin(self, name):
                seen.add(name)

            def end(self, name):
                pass

        mod.TENSOR_CORES = on
        ops.set_profiler(Names())
        try:
            got = {}
            for name, steps in _all_regimes({"a": toks}, tail=70).items():
                got[name] = H.run_trace(_runner(d, torch.bfloat16, 16, H.peak_pages(steps, 16)),
                                        steps)
                _compare(got[name], ref, torch.bfloat16, f"tensor cores {on}/{name}")
        finally:
            ops.set_profiler(None)
            mod.TENSOR_CORES = True
        assert ("pwm_attention" in seen) == on and ("apw_attention" in seen) != on
        outs.append(got)
    for name in outs[0]:
        worst = max(H.rel_err(outs[0][name][k], outs[1][name][k]) for k in outs[0][name])
        assert worst <= 0.05, f"{name}: the two kernels differ by {worst:.3g}"


# ----------------------------------------------------------------------- whole models
LENGTHS = {"A": [5, 17, 33, 70, 121], "B": [1, 9, 40, 70, 101], "C": [3, 30, 64, 47, 2],
           "D": [2, 45, 150, 333, 90], "E": [4, 19, 37, 66, 83]}


def _requests(which, extra=()):
    vocab = H.GUK[which]["raw"]["vocab"]
    lens = list(LENGTHS[which]) + list(extra)
    return {f"r{i}": H.random_tokens(n, vocab, 100 * i + n) for i, n in enumerate(lens)}


@pytest.fixture(scope="module")
def plain_logits(tmp_path_factory):
    cache = {}

    def get(which, dtype, reqs):
        d = H.make_gukidra_dir(tmp_path_factory.getbasetemp(), which, dtype)
        raw, w = H.read_model_dir(d)
        out = cache.setdefault((which, dtype), {})
        for rid, toks in reqs.items():
            k = (rid, tuple(toks))
            if k not in out:
                out[k] = G.forward(raw, w, toks)
        return d, {rid: out[(rid, tuple(toks))] for rid, toks in reqs.items()}

    return get


@pytest.mark.parametrize("which,dtype", [("A", torch.float32), ("B", torch.float32),
                                         ("C", torch.float32), ("E", torch.float32),
                                         ("A", torch.bfloat16), ("B", torch.bfloat16),
                                         ("D", torch.bfloat16), ("E", torch.bfloat16)],
                         ids=["A-f32", "B-f32", "C-f32", "E-f32", "A-bf16", "B-bf16", "D-bf16",
                              "E-bf16"])
@pytest.mark.parametrize("regime", ["whole", "tail", "portions", "mixed"])
def test_replay(cuda_device, plain_logits, which, dtype, regime):
    """Seven requests through four state slots and page pools of exactly the peak need."""
    reqs = _requests(which, (55, 61) if regime == "mixed" else ())
    model_dir, ref = plain_logits(which, dtype, reqs)
    steps = _all_regimes(reqs)[regime]
    ps = H.GUK[which]["page_size"]
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
    ps = H.GUK[which]["page_size"]
    outs = []
    for steps in _all_regimes(reqs).values():
        outs.append(H.run_trace(_runner(model_dir, torch.float32, ps, H.peak_pages(steps, ps)),
                                steps))
    for other in outs[1:]:
        for key, row in outs[0].items():
            assert torch.equal(row, other[key]), f"{which}: logits at {key} depend on the cut"


def test_long_decoding(cuda_device, plain_logits):
    """A short prompt, then 300 tokens one by one: windows pass over decoded tokens, blocks
    are completed and first seen while decoding, and the token pages behind are given back."""
    which, dtype = "B", torch.float32
    reqs = {"long": H.random_tokens(304, H.GUK[which]["raw"]["vocab"], 7)}
    model_dir, ref = plain_logits(which, dtype, reqs)
    steps = H.trace_decode_tail(reqs, tail=300)
    runner = _runner(model_dir, dtype, 4, 30)       # far fewer token pages than 304 tokens fill
    _compare(H.run_trace(runner, steps), ref, dtype, "long decoding")


def test_decoding_from_captured_steps(cuda_device, plain_logits):
    """Steps of single tokens replayed from CUDA graphs (padded rows use the scratch page and
    the scratch state slot) give what eager steps give."""
    which, dtype = "A", torch.float32
    reqs = _requests(which, (55, 61))
    model_dir, ref = plain_logits(which, dtype, reqs)
    steps = H.trace_mixed(reqs, tail=20)
    ps = H.GUK[which]["page_size"]
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
    d = H.make_gukidra_dir(tmp_path, "A")
    raw, w = H.read_model_dir(d)
    prompts = [H.random_tokens(n, raw["vocab"], n) for n in (5, 17, 33, 2)]
    eng = Engine(d, "float32", num_pages=40, page_size=16, max_seq_len=128, max_batch_size=3,
                 max_tokens_per_step=step_tokens, cuda_graphs=graphs)
    got = eng.generate(prompts, max_tokens=12, ignore_eos=True)
    for p, out in zip(prompts, got):
        assert len(out) == 12
        logits = G.forward(raw, w, list(p) + list(out))
        for n, tok in enumerate(out):
            row = logits[len(p) - 1 + n]
            assert float(row[tok]) >= float(row.max()) - 1e-4 * float(row.abs().max()), (
                f"token {n} after a prompt of {len(p)}: {tok}, plain {int(row.argmax())}")
    st = eng.stats()
    assert st["pages_free"] == st["pages_total"]
    if graphs:
        assert getattr(eng.runner, "graph_replays", 0) > 0


def test_trace_replay_tool_with_four_state_slots(cuda_device, tmp_path):
    """``bin/trace_run`` as a user runs it on a hybrid model: six requests through its four
    state slots and a page pool sized by ``--max-tokens``."""
    import test_trace_run_gpu as TR
    d = H.make_gukidra_dir(tmp_path, "B")
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
    ref = {rid: G.forward(raw, w, toks) for rid, toks in reqs.items()}
    worst = max(H.rel_err(row, ref[rid][p]) for (rid, p), row in got.items())
    assert got and worst <= TOL[torch.float32], f"worst relative error {worst:.3g}"
