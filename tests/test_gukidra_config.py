"""The hybrid design's configuration, tensor names and cache needs (no GPU)."""
import copy

import pytest
import torch

import helpers as H
from binfer_b200.cache.manager import CacheManager, KVNeed
from binfer_b200.config import (ConfigError, GukidraConfig, MLSTMSpec,
                                PooledWindowAttentionSpec, parse_config)
from binfer_b200.parts.base import BuildEnv
from binfer_b200.parts.model import DecoderModel, param_specs_for


def test_the_registry_picks_the_family_by_its_one_name():
    cfg = parse_config(H.GUK_A)
    assert isinstance(cfg, GukidraConfig)
    assert cfg.to_dict() == H.GUK_A and cfg.to_dict() is not H.GUK_A


def test_layers_become_specs_with_their_own_sizes():
    spec = GukidraConfig.from_dict(H.GUK_B).to_spec()
    assert spec.hidden_size == 48 and spec.vocab_size == 211 and spec.tie_word_embeddings
    assert spec.embedding_scale == 1.0 and spec.final_norm.offset == 1.0
    a, m, r, m2 = [l.mixer for l in spec.layers]
    assert isinstance(a, PooledWindowAttentionSpec) and isinstance(m, MLSTMSpec)
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.value_dim) == (3, 3, 24, 40)
    assert (a.window, a.pool, a.scale, a.sink, a.own_cache) == (7, 8, 0.3, 0.0, True)
    assert a.position.theta == 500.0 and a.position.rotary_dim == 24
    assert a.value_rotation.rotary_dim == 40
    assert (r.window, r.pool, r.scale, r.own_cache) == (20, 5, 0.25, False)
    assert (m.num_heads, m.qk_dim, m.v_dim, m.gate_cap) == (1, 40, 24, 5.0)
    assert [e.cache_from for e in spec.schedule] == [None, None, 0, None]
    assert [l.ffn is None for l in spec.layers] == [False, True, False, False]
    assert spec.layers[2].ffn.intermediate_size == 72 and m2.norm_eps == 1e-5


def test_tensor_names_and_shapes():
    shapes = {s.name: s.shape for s in param_specs_for(GukidraConfig.from_dict(H.GUK_A).to_spec())}
    assert shapes["embed"] == (300, 64) and shapes["final.norm"] == (64,)
    assert shapes["l0.mix.q"] == (32, 64) and shapes["l0.mix.v"] == (64, 64)
    assert shapes["l0.mix.i"] == (2, 64) and shapes["l0.mix.f.b"] == (2,)
    assert shapes["l0.mix.norm"] == (64,) and shapes["l0.mix.o"] == (64, 64)
    assert "l0.norm2" not in shapes and "l0.mlp.gate" not in shapes       # no feed-forward
    assert shapes["l2.norm2"] == (64,) and shapes["l2.mlp.down"] == (64, 80)
    assert shapes["l1.mix.q"] == (128, 64) and shapes["l1.mix.k"] == (64, 64)
    assert shapes["l1.mix.v"] == (32, 64) and shapes["l1.mix.g"] == (4, 64)
    assert shapes["l1.mix.o"] == (64, 64) and shapes["l1.mix.k.norm"] == (32,)
    # the reader has queries, gates and an output projection only
    assert "l3.mix.k" not in shapes and "l3.mix.v" not in shapes and "l3.mix.k.norm" not in shapes
    assert shapes["l3.mix.q.norm"] == (32,) and "l3.norm2" not in shapes
    assert "head" not in shapes


@pytest.mark.parametrize("change,message", [
    (lambda r: r.pop("width"), "width"),
    (lambda r: r["norm"].pop("eps"), "norm.eps"),
    (lambda r: r["layers"][0].__setitem__("type", "conv"), "not supported"),
    (lambda r: r["layers"][1]["mixer"].__setitem__("kv_heads", 3), "multiple of kv_heads"),
    (lambda r: r["layers"][3]["mixer"].__setitem__("kv_from", 0), "kv_from"),
    (lambda r: r["layers"][3]["mixer"].__setitem__("kv_from", 3), "kv_from"),
    (lambda r: r["layers"][3]["mixer"].__setitem__("vdim", 8), "differ"),
    (lambda r: r["layers"][1]["mixer"]["rot"].__setitem__("dims", 34), "rot.dims"),
    (lambda r: r["layers"][1]["mlp"].__setitem__("kind", "experts"), "not supported"),
])
def test_what_is_wrong_is_refused(change, message):
    raw = copy.deepcopy(H.GUK_A)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        GukidraConfig.from_dict(raw)


def _model(raw):
    return DecoderModel(GukidraConfig.from_dict(raw).to_spec(),
                        BuildEnv(torch.float32, torch.device("cpu")))


def test_cache_needs_of_readers_are_merged_into_the_source():
    needs = _model(H.GUK_B).kv_needs()
    # layer 0 keeps window 7 / blocks of 8, its reader looks back 20 tokens over blocks of 5
    assert needs[0] == KVNeed(3, 24, 20, 40, (5, 8)) and needs[2] is None
    assert needs[1] is None and needs[3] is None
    states = _model(H.GUK_B).state_needs()
    assert states[0] is None and states[1].shape == (1, 40 * 24 + 40 + 4)
    assert states[3].shape == (3, 8 * 8 + 8 + 4)


def test_summary_groups_hold_one_entry_per_block():
    model = _model(H.GUK_B)
    cm = CacheManager(model.kv_needs(), model.state_needs(), page_size=4, num_pages=40,
                      max_requests=3)
    assert len(cm.groups) == 3                       # tokens, blocks of 5, blocks of 8
    assert sorted(cm.summary_location) == [(0, 5), (0, 8)]
    by_stride = {g.stride: g for g in cm.groups}
    rc = cm.add_request("a")
    cm.reserve("a", 23)
    cm.commit("a", 23)
    assert len(rc.tables[by_stride[1].index]) == 6   # 23 tokens in pages of 4
    assert len(rc.tables[by_stride[5].index]) == 1   # 4 blocks of 5
    assert len(rc.tables[by_stride[8].index]) == 1   # 2 blocks of 8
    cm.reserve("a", 60)
    cm.commit("a", 60)
    assert len(rc.tables[by_stride[5].index]) == 3 and len(rc.tables[by_stride[8].index]) == 2
    cm.check_consistent()
    cm.free_request("a")
    assert all(g.pool.num_held == 0 for g in cm.groups)


def test_token_pages_stay_until_window_and_blocks_are_done():
    """A page is given back only when every token on it has left the widest window and
    belongs to a block whose mean is taken, for every block size."""
    need = KVNeed(1, 8, 6, None, (4, 16))
    cm = CacheManager([need], [], page_size=2, num_pages=64, max_requests=2)
    tokens = cm.groups[0]
    for length in range(0, 70):
        first = tokens.first_needed_page(length) * 2
        assert first <= max(0, length - 6 + 1)           # nothing inside the window is gone
        assert first <= (length // 16) * 16              # nor of the unfinished large block
        assert first <= (length // 4) * 4
        bound = min(max(0, length - 5), (length // 16) * 16)
        assert first >= bound - 1                        # and no more than a page is kept beyond
    rc = cm.add_request("r")
    held = []
    for n in range(1, 50):
        cm.reserve("r", n)
        cm.commit("r", n)
        held.append(sum(1 for p in rc.tables[0] if p > 0))
    assert max(held) <= 16 // 2 + 6 // 2 + 2             # a block and a window, not the sequence
    cm.check_consistent()


def test_a_request_without_pooled_blocks_keeps_the_old_group_key():
    assert KVNeed(2, 64, None).group_key == (2, 64, None)
    assert KVNeed(2, 64, 8, 32).group_key != KVNeed(2, 64, 8).group_key
    assert KVNeed(2, 64, None).merged(KVNeed(2, 64, 9, None, (3,))) == KVNeed(2, 64, None)
    with pytest.raises(ValueError):
        KVNeed(2, 64, 8).merged(KVNeed(1, 64, 8))
