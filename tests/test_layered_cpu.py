"""CPU tests of the layered family's host side: config parsing and registry, the page pool (slots and pages
that are freed and handed out again, growth, truncation), gate/up interleaving, and the NumPy oracle's own
mechanisms on hand-made cases (so that the oracle the GPU tests lean on is itself pinned)."""
import numpy as np
import pytest

from pygpukit_b200.llm.config import LAYERED_ARCHITECTURES, AttentionMixerSpec, layered_config_from_json
from pygpukit_b200.llm.layers.linear import interleave_gate_up
from pygpukit_b200.llm.paged_cache import PagePool
from tests import dolurax_ref as R


def test_config_reads_every_size_from_the_file():
    d = R.make_config(vocab=77, width=40, layers=3, heads=6, kv_heads=3, dim=10, vdim=14, chunk=5, scale=0.3, softcap=11.0,
                      experts=12, top=3, groups=(4, 2), ff=18, shared_ff=26, eps=3e-6, logit_scale=0.7, logit_softcap=9.0)
    d["layers"][1]["mlp"] = None
    d["layers"][2]["mixer"]["v_mix"] = False
    d["layers"][2]["mixer"]["mask"] = None
    d["layers"][2]["mlp"]["shared"] = None
    c = layered_config_from_json(d)
    assert (c.architecture, c.vocab_size, c.hidden_size, c.num_layers) == ("Dolurax", 77, 40, 3)
    assert (c.norm_eps, c.logit_scale, c.logit_softcap) == (3e-6, 0.7, 9.0)
    m = c.layers[0].mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.chunk, m.scale, m.softcap, m.v_mix) == (6, 3, 10, 14, 5, 0.3, 11.0, True)
    f = c.layers[0].mlp
    assert (f.experts, f.top, f.ff, f.group_count, f.group_keep, f.shared_ff) == (12, 3, 18, 4, 2, 26)
    assert c.layers[1].mlp is None
    assert c.layers[2].mixer.chunk == 0 and not c.layers[2].mixer.v_mix and c.layers[2].mlp.shared_ff == 0


def test_registry_and_rejections():
    assert "dolurax" in LAYERED_ARCHITECTURES
    assert layered_config_from_json({"model_type": "llama"}) is None
    d = R.make_config()
    d["layers"][0]["type"] = "recurrent"
    with pytest.raises(ValueError, match="unknown type"):
        layered_config_from_json(d)
    d = R.make_config(heads=4, kv_heads=3)
    with pytest.raises(ValueError, match="key/value heads"):
        layered_config_from_json(d)
    d = R.make_config(experts=10, groups=(4, 1))
    with pytest.raises(ValueError, match="groups"):
        layered_config_from_json(d)


def test_head_slopes():
    s = AttentionMixerSpec(heads=4, kv_heads=1, dim=8, vdim=8, scale=1.0).slopes()
    assert np.allclose(s, [0.25, 0.0625, 0.015625, 0.00390625])
    assert np.allclose(AttentionMixerSpec(heads=3, kv_heads=3, dim=8, vdim=8, scale=1.0).slopes(), R.head_slopes(3))


def test_interleave_gate_up():
    g, u = np.arange(6.0).reshape(3, 2), -np.arange(6.0).reshape(3, 2)
    w = interleave_gate_up(g, u)
    assert np.array_equal(w[0::2], g) and np.array_equal(w[1::2], u)


# ---------------------------------------------------------------- page pool
def test_pool_allocates_lowest_pages_and_positions():
    p = PagePool(page_size=4, pages=8, slots=2, max_pages_per_seq=4)
    assert p.extend("a", 5) == (0, 0)
    assert p.page_list("a") == [0, 1] and p.length("a") == 5
    assert p.extend("b", 1) == (1, 0) and p.page_list("b") == [2]
    assert p.extend("a", 3) == (0, 5) and p.page_list("a") == [0, 1]          # fills page 1 exactly
    assert p.extend("a", 1) == (0, 8) and p.page_list("a") == [0, 1, 3]
    assert list(p.table[0, :3]) == [0, 1, 3] and p.table[1, 0] == 2


def test_pool_hands_freed_slots_and_pages_out_again():
    p = PagePool(page_size=2, pages=6, slots=2, max_pages_per_seq=4)
    p.extend("a", 4)
    p.extend("b", 3)
    p.release("a")
    assert "a" not in p and p.free_pages == 4
    assert p.extend("c", 5) == (0, 0)                 # a's slot
    assert p.page_list("c") == [0, 1, 4]              # a's pages first, then a fresh one
    p.release("b")
    p.release("c")
    assert p.free_pages == 6 and p.live_sequences == 0


def test_pool_grows_pages_slots_and_table():
    p = PagePool(page_size=2, pages=2, slots=1, max_pages_per_seq=1)
    p.extend("a", 2)
    p.extend("b", 7)                                  # needs a second slot, 4 pages and a wider table
    assert p.slots >= 2 and p.pages >= 5 and p.max_pages >= 4
    assert p.page_list("a") == [0] and len(set(p.page_list("b"))) == 4 and 0 not in p.page_list("b")
    assert list(p.table[p.slot("b"), :4]) == p.page_list("b")
    assert p.table[p.slot("a"), 0] == 0


def test_pool_truncate_frees_whole_pages_only():
    p = PagePool(page_size=4, pages=8, slots=1, max_pages_per_seq=8)
    p.extend("a", 11)
    p.truncate("a", 5)
    assert p.length("a") == 5 and p.page_list("a") == [0, 1] and p.free_pages == 6
    assert p.extend("a", 4) == (0, 5) and p.page_list("a") == [0, 1, 2]
    with pytest.raises(ValueError):
        p.truncate("a", 99)


# ---------------------------------------------------------------- the oracle's mechanisms on hand-made cases
def test_oracle_visibility():
    v = R.visible(7, 3)
    assert v[2, 0] and v[2, 2] and not v[2, 3]          # causal
    assert not v[3, 2] and v[3, 3]                      # position 3 opens a chunk: it sees only itself
    assert v[5, 3] and not v[5, 2] and not v[6, 5]
    assert R.visible(4, 0).sum() == 10                  # no chunks: plain causal


def test_oracle_route_group_limit_and_renormalisation():
    z = np.log(np.array([[0.30, 0.05, 0.02, 0.03, 0.25, 0.20, 0.10, 0.05]]))
    idx, w = R.route(z, top=2, group_count=2, group_keep=1)           # groups {0..3}, {4..7}: the first has the best member
    assert list(idx[0]) == [0, 1] and np.allclose(w[0], [0.30 / 0.35, 0.05 / 0.35])
    idx, w = R.route(z, top=2, group_count=1, group_keep=1)
    assert list(idx[0]) == [0, 4] and np.allclose(w.sum(), 1.0)
    idx, _ = R.route(z, top=3, group_count=4, group_keep=2)           # groups of two: best {0,1} and {4,5}
    assert list(idx[0]) == [0, 4, 5]


def test_oracle_attention_prefers_the_standout_key_only_inside_the_chunk():
    T, D = 9, 4
    q = np.zeros((T, 1, D)); k = np.zeros((T, 1, D)); v = np.zeros((T, 1, 2))
    q[8, 0, 0], k[6, 0, 0], k[5, 0, 0] = 10.0, 10.0, 20.0
    v[6, 0, 0], v[5, 0, 1] = 1.0, 1.0
    o = R.attention_core(q, k, v, scale=1.0, softcap=0.0, chunk=3)    # query 8 sees 6..8
    assert o[8, 0, 0] > 0.99 and o[8, 0, 1] == 0.0
    o = R.attention_core(q, k, v, scale=1.0, softcap=0.0, chunk=0)
    assert o[8, 0, 1] > 0.99
