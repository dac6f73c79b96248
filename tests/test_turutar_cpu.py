"""CPU tests of the Turutar design's host side: config parsing (every size and constant from the file, the order of
layer runs under a loop, rejections), the work buffers and cache shapes the specs ask for, and the NumPy oracle's own
mechanisms on hand-made cases, so that the oracle the GPU tests lean on is itself pinned."""
import numpy as np
import pytest

from pygpukit_b200.llm.config import LAYERED_ARCHITECTURES, layered_config_from_json
from tests import turutar_ref as R


def test_config_reads_every_size_and_constant_from_the_file():
    d = R.make_config([R.latent_layer(heads=5, dim=6, rot_dim=10, vdim=14, kv_rank=22, q_rank=18, scale=0.37, dims=4, base=777.0, ff=26, limit=0.9),
                       R.windowed_layer(heads=6, kv_heads=3, dim=10, window=13, scale=0.21, ff=0)],
                      vocab=77, width=40, side=3, loop=(1, 2, 4), eps=3e-6)
    c = layered_config_from_json(d)
    assert (c.architecture, c.vocab_size, c.hidden_size, c.num_layers, c.norm_eps) == ("Turutar", 77, 40, 2, 3e-6)
    assert (c.block, c.norm, c.embed_norm, c.layer_scale, c.side_dim) == ("parallel", "rmsnorm_1p", True, True, 3)
    assert (c.loop_start, c.loop_stop, c.loop_times) == (1, 2, 4)
    m = c.layers[0].mixer
    assert (m.kind, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.q_rank, m.scale, m.rot_dims, m.rot_base) == \
        ("latent_attention", 5, 6, 10, 14, 22, 18, 0.37, 4, 777.0)
    assert (m.sink, m.gate_per_head, m.cache_shape(), m.proj_cols) == ("learned", True, (1, 32, 0), 18 + 22 + 10 + 5)
    assert m.inv_freq() == [1.0, 777.0 ** -0.5]
    f = c.layers[0].mlp
    assert (f.kind, f.ff, f.activation, f.limit, f.alpha) == ("dense", 26, "clamped_swish", 0.9, 1.702)
    w = c.layers[1].mixer
    assert (w.kind, w.heads, w.kv_heads, w.dim, w.vdim, w.window, w.scale) == ("attention", 6, 3, 10, 10, 13, 0.21)
    assert (w.sink, w.norm_scope, w.qk_bias, w.values, w.gate_per_head, w.chunk) == ("zero", "all", True, "keys", True, 0)
    assert (w.cache_shape(), w.proj_cols, w.slopes()) == ((3, 10, 10), 60 + 30 + 6, [])
    assert c.layers[1].mlp is None


def test_layer_runs_under_a_loop():
    def runs(n, loop):
        return layered_config_from_json(R.make_config([R.windowed_layer() for _ in range(n)], loop=loop)).layer_runs()
    assert runs(3, None) == [(0, False), (1, False), (2, False)]
    assert runs(4, (1, 3, 3)) == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert runs(2, (0, 2, 2)) == [(0, False), (1, False), (0, True), (1, False)]
    assert runs(2, (0, 2, 1)) == [(0, False), (1, False)] and runs(2, (1, 1, 5)) == [(0, False), (1, False)]
    assert runs(4, (1, 3, 3)) == R.layer_runs(R.make_config([R.windowed_layer() for _ in range(4)], loop=(1, 3, 3)))


def test_registry_and_rejections():
    assert "turutar" in LAYERED_ARCHITECTURES
    d = R.make_config([R.windowed_layer()])
    d["layers"][0]["type"] = "recurrent"
    with pytest.raises(ValueError, match="unknown type"):
        layered_config_from_json(d)
    with pytest.raises(ValueError, match="key/value heads"):
        layered_config_from_json(R.make_config([R.windowed_layer(heads=4, kv_heads=3)]))
    d = R.make_config([R.windowed_layer()])
    d["layers"][0]["mixer"]["vdim"] = 5
    with pytest.raises(ValueError, match="values are the keys"):
        layered_config_from_json(d)
    d = R.make_config([R.windowed_layer()])
    d["layers"][0]["mlp"]["kind"] = "moe"
    with pytest.raises(ValueError, match="feed-forward kind"):
        layered_config_from_json(d)
    with pytest.raises(ValueError, match="rotated dimensions"):
        layered_config_from_json(R.make_config([R.latent_layer(rot_dim=6, dims=8)]))
    with pytest.raises(ValueError, match="loop"):
        layered_config_from_json(R.make_config([R.windowed_layer()], loop=(0, 3, 2)))
    d = R.make_config([R.windowed_layer()])
    d["layers"][0]["mixer"]["mask"] = None                               # no window: plain causal
    assert layered_config_from_json(d).layers[0].mixer.window == 0


def test_oracle_window_and_sink():
    vis = R.window_mask(6, 3)
    assert vis[5].tolist() == [False, False, False, True, True, True] and vis[1].tolist() == [True, True, False, False, False, False]
    assert R.window_mask(4, 0)[3].all() and R.window_mask(4, 1).sum() == 4
    s = np.log(np.array([[1.0, 3.0]]))
    p = R.softmax_with_sink(s, np.array([[True, True]]), 0.0)            # denominator 1 + 1 + 3
    assert np.allclose(p, [[0.2, 0.6]])
    assert np.allclose(R.softmax_with_sink(s, np.array([[True, True]]), np.log(4.0)), [[0.125, 0.375]])
    assert np.allclose(R.softmax_with_sink(s, np.array([[True, False]]), None), [[1.0, 0.0]])


def test_oracle_rotation_is_relative_and_leaves_the_tail():
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal((1, 8)), rng.standard_normal((1, 8))
    def dot(i, j):
        return float(R.rotate_pairs(a, [i], 6, 50.0)[0] @ R.rotate_pairs(b, [j], 6, 50.0)[0])
    assert abs(dot(3, 1) - dot(903, 901)) < 1e-9 and abs(dot(3, 1) - dot(3, 2)) > 1e-3
    assert np.array_equal(R.rotate_pairs(a, [17], 6, 50.0)[0, 6:], a[0, 6:])
    one = R.rotate_pairs(np.array([[1.0, 0.0]]), [1], 2, 10.0)[0]        # pair 0 turns by one radian per position
    assert np.allclose(one, [np.cos(1.0), np.sin(1.0)])


def test_oracle_clamped_feed_forward_and_norms():
    P = {"gate": np.array([[2.0], [-1.0]]), "up": np.array([[3.0], [-3.0]]), "down": np.eye(2)}
    y = R.clamped_ffn(np.array([[1.0]]), P, "", 1.5)
    g0, g1 = 1.5, -1.0                                                   # the gate is cut from above only, up on both sides
    assert np.allclose(y, [[g0 * R.sigmoid(1.702 * g0) * 2.5, g1 * R.sigmoid(1.702 * g1) * -0.5]])
    x = np.array([[3.0, 4.0]])
    assert np.allclose(R.rms_norm(x, np.array([0.0, 1.0]), 0.0, 1.0), [[3 / np.sqrt(12.5), 8 / np.sqrt(12.5)]])
    assert np.allclose(R.rms_norm(x, np.array([0.0, 1.0]), 0.0), [[0.0, 4 / np.sqrt(12.5)]])
    assert abs(R.gelu_tanh(1.0) - 0.841192) < 1e-6


def test_oracle_windowed_mixer_values_are_the_keys_before_their_norm():
    """One token: softmax over itself and the sink, so the output is p * (k as projected), gated per head."""
    rng = np.random.default_rng(3)
    W, H, D = 6, 2, 4
    P = {k: rng.standard_normal(s) for k, s in (("q", (H * D, W)), ("k", (H * D, W)), ("q.b", H * D), ("k.b", H * D),
                                                 ("q.norm", H * D), ("k.norm", H * D), ("g", (H, W)))}
    P["o"] = np.eye(H * D)
    h = rng.standard_normal((1, W))
    out = R.windowed_mixer(h, P, "", {"heads": H, "kv_heads": H, "dim": D, "scale": 0.5, "mask": {"size": 4}}, 1e-6)
    q, k = h @ P["q"].T + P["q.b"], h @ P["k"].T + P["k.b"]
    qn, kn = R.rms_norm(q, P["q.norm"], 1e-6), R.rms_norm(k, P["k.norm"], 1e-6)
    for hh in range(H):
        s = float(qn[0, hh * D:(hh + 1) * D] @ kn[0, hh * D:(hh + 1) * D]) * 0.5
        p = np.exp(s) / (1 + np.exp(s))
        assert np.allclose(out[0, hh * D:(hh + 1) * D], p * k[0, hh * D:(hh + 1) * D] * R.sigmoid(h @ P["g"].T)[0, hh])
