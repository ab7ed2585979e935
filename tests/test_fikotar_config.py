"""The side-by-side design's configuration, tensor names, cache and state needs, and the
plain implementation's own mechanisms (no GPU)."""
import copy
import math

import pytest
import torch

import helpers as H
import fikotar_plain as P
from binfer_b200.cache.manager import CacheManager, KVNeed
from binfer_b200.config import (ConfigError, ConvWindowAttentionSpec, FikotarConfig, MoESpec,
                                ParallelMixersSpec, RetentionSpec, RopeSpec, WavelengthScaling,
                                parse_config)
from binfer_b200.parts.base import BuildEnv
from binfer_b200.parts.model import DecoderModel, param_specs_for
from binfer_b200.parts.rope import RotaryEncoding


def test_the_registry_picks_the_family_by_its_one_name():
    cfg = parse_config(H.FIK_A)
    assert isinstance(cfg, FikotarConfig)
    assert cfg.to_dict() == H.FIK_A and cfg.to_dict() is not H.FIK_A


def test_layers_become_specs_with_their_own_sizes():
    spec = FikotarConfig.from_dict(H.FIK_B).to_spec()
    assert spec.hidden_size == 48 and spec.vocab_size == 211 and not spec.tie_word_embeddings
    assert spec.logit_scale == 1.0 and spec.final_norm.kind == "layernorm"
    assert spec.final_norm.bias_suffix == ".b" and spec.final_norm.eps == 1e-6
    assert all(l.block == "parallel" for l in spec.layers)
    m0, m1 = [l.mixer for l in spec.layers]
    assert isinstance(m0, ParallelMixersSpec) and [b.prefix for b in m0.branches] == ["left.", "right."]
    assert [b.scale for b in m0.branches] == [1.0, 1.0] and [b.scale for b in m1.branches] == [0.5, 0.5]
    a, r = m0.branches[0].spec, m0.branches[1].spec
    assert isinstance(a, ConvWindowAttentionSpec) and isinstance(r, RetentionSpec)
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.value_dim) == (3, 3, 24, 40)
    assert (a.conv_taps, a.window, a.keep_first, a.scale, a.sinks) == (4, 3, 6, 0.3, True)
    assert a.position.theta == 500.0 and a.position.rotary_dim == 24
    assert a.position.wavelength_scaling is None and a.norm_eps == 1e-6
    assert (r.num_heads, r.qk_dim, r.v_dim, r.decays) == (3, 8, 8, (1.0, 0.5, 0.98))
    b = m1.branches[0].spec
    assert b.conv_taps == 0 and b.position.wavelength_scaling == WavelengthScaling(2.0, 0.5, 3.0, 40.0)
    f = spec.layers[1].ffn
    assert isinstance(f, MoESpec) and (f.num_experts, f.top, f.expert_size, f.shared_size,
                                       f.shared_gate) == (6, 2, 32, 72, True)
    assert FikotarConfig.from_dict(H.FIK_A).to_spec().layers[1].ffn is None
    assert FikotarConfig.from_dict(H.FIK_A).to_spec().layers[2].ffn.shared_size == 0


def test_tensor_names_and_shapes():
    shapes = {s.name: s.shape for s in param_specs_for(FikotarConfig.from_dict(H.FIK_A).to_spec())}
    assert shapes["embed"] == (300, 64) and shapes["head"] == (300, 64)
    assert shapes["final.norm"] == (64,) and shapes["final.norm.b"] == (64,)
    assert shapes["l0.norm1"] == (64,) and shapes["l0.norm1.b"] == (64,)
    assert shapes["l0.mix.left.q"] == (128, 64) and shapes["l0.mix.left.k"] == (64, 64)
    assert shapes["l0.mix.left.v"] == (32, 64) and shapes["l0.mix.left.o"] == (64, 64)
    assert shapes["l0.mix.left.q.conv"] == (128, 3) and shapes["l0.mix.left.v.conv"] == (32, 3)
    assert shapes["l0.mix.left.sink"] == (4,)
    assert shapes["l0.mix.right.q"] == (32, 64) and shapes["l0.mix.right.v"] == (64, 64)
    assert shapes["l0.mix.right.g"] == (64, 64) and shapes["l0.mix.right.o"] == (64, 64)
    assert shapes["l0.mlp.router"] == (4, 64) and shapes["l0.mlp.e3.down"] == (64, 48)
    assert shapes["l0.mlp.shared.gate"] == (64, 64) and shapes["l0.mlp.shared.sg"] == (1, 64)
    assert not any(n.startswith("l1.mlp") for n in shapes)               # no feed-forward
    assert shapes["l2.mix.left.k.conv"] == (16, 2) and shapes["l2.mlp.e4.up"] == (40, 64)
    assert "l2.mlp.shared.gate" not in shapes and "l2.mlp.shared.sg" not in shapes
    shapes_b = {s.name for s in param_specs_for(FikotarConfig.from_dict(H.FIK_B).to_spec())}
    assert "l1.mix.left.q.conv" not in shapes_b                          # no convolution


@pytest.mark.parametrize("change,message", [
    (lambda r: r.pop("width"), "width"),
    (lambda r: r["norm"].pop("eps"), "norm.eps"),
    (lambda r: r["layers"][0].__setitem__("type", "serial"), "not supported"),
    (lambda r: r["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3), "multiple of kv_heads"),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 34), "dims"),
    (lambda r: r["layers"][0]["mixer"]["right"].__setitem__("decay", [0.9]), "decay"),
    (lambda r: r["layers"][0]["mixer"].pop("right"), "right"),
    (lambda r: r["layers"][0]["mlp"].__setitem__("kind", "dense"), "not supported"),
    (lambda r: r["layers"][0]["mlp"]["router"].__setitem__("top", 5), "exceeds"),
])
def test_what_is_wrong_is_refused(change, message):
    raw = copy.deepcopy(H.FIK_A)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        FikotarConfig.from_dict(raw)


def _model(raw):
    return DecoderModel(FikotarConfig.from_dict(raw).to_spec(),
                        BuildEnv(torch.float32, torch.device("cpu")))


def test_cache_and_state_needs_of_the_branches():
    model = _model(H.FIK_B)
    needs, states = model.kv_needs(), model.state_needs()
    assert needs[0] == KVNeed(3, 24, 3, 40, keep_first=6)
    assert needs[1] == KVNeed(1, 24, 20, 40, keep_first=1)
    # four taps: three rows of 3*24 + 3*24 + 3*40 channels; three heads of 8 x 8
    assert states[0].shape == (3 * 264 + 3 * 64,)
    assert states[1].shape == (0 + 2 * 12 * 20,)                         # no convolution


def test_pages_of_the_kept_first_tokens_are_never_given_back():
    need = KVNeed(1, 8, 6, None, keep_first=5)
    cm = CacheManager([need], [], page_size=2, num_pages=40, max_requests=2)
    g = cm.groups[0]
    assert g.kept_pages == 3
    rc = cm.add_request("r")
    held = []
    for n in range(1, 60):
        cm.reserve("r", n)
        cm.commit("r", n)
        table = rc.tables[0]
        assert all(p > 0 for p in table[:min(3, len(table))])            # positions 0..4 stay
        first_in_window = max(0, n - 6 + 1)
        assert all(table[i] > 0 for i in range(first_in_window // 2, len(table)))
        held.append(sum(1 for p in table if p > 0))
    assert max(held) <= 3 + 6 // 2 + 2                                   # kept + window, not 59
    cm.check_consistent()
    cm.free_request("r")
    assert g.pool.num_held == 0
    assert KVNeed(1, 8, None, keep_first=5).group_key == (1, 8, None)    # no window: all stay anyway
    assert KVNeed(1, 8, 6, keep_first=5).group_key != KVNeed(1, 8, 6).group_key
    assert cm.can_ever_hold(1000) and not CacheManager(
        [need], [], page_size=2, num_pages=5, max_requests=1).can_ever_hold(1000)


def test_frequencies_stretched_by_wavelength():
    rot = {"base": 100.0, "dims": 16, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0,
                                                   "original": 64}}
    f = P.rotary_frequencies(rot)
    plain = torch.tensor([100.0 ** (-2 * i / 16) for i in range(8)], dtype=torch.float64)
    wave = 2 * math.pi / plain
    assert (wave < 16).any() and (wave > 64).any() and ((wave >= 16) & (wave <= 64)).any()
    assert torch.equal(f[wave < 16], plain[wave < 16])
    assert torch.allclose(f[wave > 64], plain[wave > 64] / 8.0)
    mid = (wave >= 16) & (wave <= 64)
    assert ((f[mid] < plain[mid]) & (f[mid] > plain[mid] / 8.0)).all()
    enc = RotaryEncoding(RopeSpec(theta=100.0, rotary_dim=16,
                                  wavelength_scaling=WavelengthScaling(8.0, 1.0, 4.0, 64.0)),
                         24, BuildEnv(torch.float32, torch.device("cpu")))
    assert torch.allclose(enc.inv_freq.double(), f, rtol=1e-6)


def test_the_plain_mechanisms_on_cases_small_enough_to_do_by_hand():
    u = torch.tensor([[1.0], [2.0], [3.0]], dtype=torch.float64)
    w = torch.tensor([[10.0, 1.0]], dtype=torch.float64)
    assert P.causal_conv(u, w).flatten().tolist() == [1.0, 12.0, 23.0]
    mask = {"size": 3, "keep_first": 2}
    assert [j for j in range(8) if P.visible(7, j, mask)] == [0, 1, 5, 6, 7]
    assert [j for j in range(8) if P.visible(3, j, mask)] == [0, 1, 2, 3]
    assert [j for j in range(4) if P.visible(2, j, None)] == [0, 1, 2]
    x = torch.tensor([[1.0, 3.0]], dtype=torch.float64)
    y = P.layer_norm(x, torch.tensor([2.0, 2.0]), torch.tensor([0.5, 0.5]), 0.0)
    assert torch.allclose(y, torch.tensor([[-1.5, 2.5]], dtype=torch.float64))
    h = torch.eye(3, dtype=torch.float64)
    wts = {"m.router": torch.tensor([[1.0, 0.0, 3.0], [2.0, 0.0, 1.0]], dtype=torch.float64)}
    ids, a = P.chosen_experts(h, wts, "m.", {"router": {"experts": 2, "top": 1}})
    assert ids.flatten().tolist() == [1, 0, 0] and a.flatten().tolist() == [1.0, 1.0, 1.0]
