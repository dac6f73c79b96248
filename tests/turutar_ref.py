"""NumPy float64 oracle of the Turutar design: whole sequences at once, no cache, one function per mechanism, no code
shared with the package.  Notation: T tokens, W width, H query heads, G key/value heads, D key size, Dv value size,
n_c latent size, D_r rotated size.

    block        h = rms1p(x);  x += s1 * mixer(h) + s2 * ff(h);  x += rms_plain(P_side (gelu(G_side x) * e_tok)) * w_side
    rms1p(x)     x / sqrt(mean(x^2) + eps) * (1 + w)          rms_plain: the same with w
    windowed     q = Wq h + bq, k = Wk h + bk, v = k;  q, k <- rms_plain over the whole projection;
                 key j visible from i when 0 <= i - j < window;  p_j = exp(s_j) / (1 + sum exp(s_j))
    latent       cq = rms_plain(Wdq h), q = Wuq cq = per head [nope D | rot D_r];  Wdkv h = [c' | r'];  c = rms_plain(c');
                 k_h = [Wuk_h c | rot(r')], v_h = Wuv_h c;  causal;  p_j = exp(s_j) / (exp(sink_h) + sum exp(s_j))
    gate         every head's output times sigmoid(Wg h)_h
    ff           g = min(Wgate h, lim), u = clip(Wup h, -lim, lim), Wdown (g sigmoid(1.702 g) (u + 1))
"""
import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def rms_norm(x, w, eps, offset=0.0):
    """x / sqrt(mean(x^2) + eps) * (offset + w) over the last axis"""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * (offset + w)


def rotate_pairs(x, positions, dims, base):
    """x [T, ..., n]: elements (2i, 2i + 1), i < dims / 2, turn by positions * base^(-2i / dims); the rest stay."""
    out = np.array(x, np.float64)
    half = dims // 2
    ang = np.asarray(positions, np.float64)[:, None] * base ** (-2.0 * np.arange(half) / dims)
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    a, b = out[..., 0:dims:2].copy(), out[..., 1:dims:2].copy()
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def softmax_with_sink(s, visible, sink):
    """rows of s over the visible keys; the denominator also holds exp(sink) (sink None: plain softmax)"""
    s = np.where(visible, s, -np.inf)
    m = s.max(-1, keepdims=True)
    if sink is not None:
        m = np.maximum(m, sink)
    e = np.exp(s - m)
    den = e.sum(-1, keepdims=True) + (np.exp(sink - m) if sink is not None else 0.0)
    return e / den


def window_mask(T, window):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & ((i - j < window) if window > 0 else True)


def windowed_core(q, k, v, scale, window, sink=0.0):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv]"""
    T, H, _ = q.shape
    G = k.shape[1]
    vis = window_mask(T, window)
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        out[:, h] = softmax_with_sink((q[:, h] @ k[:, g].T) * scale, vis, sink) @ v[:, g]
    return out


def windowed_mixer(h, P, pre, mx, eps):
    T = h.shape[0]
    H, G, D = mx["heads"], mx.get("kv_heads") or mx["heads"], mx["dim"]
    q = h @ P[pre + "q"].T + P[pre + "q.b"]
    k = h @ P[pre + "k"].T + P[pre + "k.b"]
    v = k.reshape(T, G, D)
    q = rms_norm(q, P[pre + "q.norm"], eps).reshape(T, H, D)
    k = rms_norm(k, P[pre + "k.norm"], eps).reshape(T, G, D)
    o = windowed_core(q, k, v, mx["scale"], (mx.get("mask") or {}).get("size", 0))
    o = o * sigmoid(h @ P[pre + "g"].T)[:, :, None]
    return o.reshape(T, -1) @ P[pre + "o"].T


def latent_mixer(h, P, pre, mx, eps):
    T = h.shape[0]
    H, D, Dr, Dv, nc = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    dims, base = mx["rot"]["dims"], mx["rot"]["base"]
    pos = np.arange(T)
    q = (rms_norm(h @ P[pre + "dq"].T, P[pre + "dq.norm"], eps) @ P[pre + "uq"].T).reshape(T, H, D + Dr)
    q_rot = rotate_pairs(q[..., D:], pos, dims, base)
    ckv = h @ P[pre + "dkv"].T
    c = rms_norm(ckv[:, :nc], P[pre + "dkv.norm"], eps)
    r = rotate_pairs(ckv[:, nc:], pos, dims, base)
    kn = (c @ P[pre + "uk"].T).reshape(T, H, D)
    v = (c @ P[pre + "uv"].T).reshape(T, H, Dv)
    vis = window_mask(T, 0)
    o = np.zeros((T, H, Dv))
    for hh in range(H):
        s = (q[:, hh, :D] @ kn[:, hh].T + q_rot[:, hh] @ r.T) * mx["scale"]
        o[:, hh] = softmax_with_sink(s, vis, P[pre + "sink"][hh]) @ v[:, hh]
    o = o * sigmoid(h @ P[pre + "g"].T)[:, :, None]
    return o.reshape(T, -1) @ P[pre + "o"].T


def clamped_ffn(h, P, pre, limit, alpha=1.702):
    g = np.minimum(h @ P[pre + "gate"].T, limit)
    u = np.clip(h @ P[pre + "up"].T, -limit, limit)
    return (g * sigmoid(alpha * g) * (u + 1.0)) @ P[pre + "down"].T


def token_side(x, e, P, pre, eps):
    y = (gelu_tanh(x @ P[pre + "gate"].T) * e) @ P[pre + "proj"].T
    return rms_norm(y, P[pre + "norm"], eps)


def layer_runs(cfg):
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp or lp["times"] <= 1:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t > 0 and i == lp["start"]) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, False) for i in range(lp["stop"], n)]


def forward(cfg, P, tokens, return_layers=False):
    """logits [T, vocab] (and the residual stream after every layer run)"""
    P = {k: np.asarray(v, np.float64) for k, v in P.items()}
    eps, toks = cfg["norm"]["eps"], np.asarray(tokens)
    sd = (cfg.get("token_side") or {}).get("dim", 0)
    x = rms_norm(P["embed"][toks], P["embed.norm"], eps, 1.0)
    x0, layers = x.copy(), []
    for i, add in layer_runs(cfg):
        if add:
            x = x + x0
        L, pre = cfg["layers"][i], f"l{i}."
        h = rms_norm(x, P[pre + "norm1"], eps, 1.0)
        mix = (windowed_mixer if L["type"] == "attention" else latent_mixer)(h, P, pre + "mix.", L["mixer"], eps)
        upd = mix * P[pre + "ls1"]
        if L.get("mlp"):
            upd = upd + clamped_ffn(h, P, pre + "mlp.", L["mlp"]["limit"]) * P[pre + "ls2"]
        x = x + upd
        if sd:
            x = x + token_side(x, P["side.embed"][toks][:, i * sd:(i + 1) * sd], P, pre + "side.", eps)
        layers.append(x.copy())
    logits = rms_norm(x, P["final.norm"], eps, 1.0) @ P["head"].T
    return (logits, layers) if return_layers else logits


def windowed_layer(heads=4, kv_heads=2, dim=16, window=7, scale=0.3, ff=24, limit=1.5):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale,
                                           "mask": {"size": window}},
            "mlp": {"kind": "dense", "ff": ff, "limit": limit} if ff else None}


def latent_layer(heads=3, dim=8, rot_dim=12, vdim=10, kv_rank=20, q_rank=28, scale=0.2, dims=None, base=300.0, ff=24, limit=1.5):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": scale, "rot": {"dims": rot_dim if dims is None else dims, "base": base}},
            "mlp": {"kind": "dense", "ff": ff, "limit": limit} if ff else None}


def make_config(layers, vocab=90, width=48, side=6, loop=None, eps=1e-5):
    cfg = {"architecture": "Turutar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if side:
        cfg["token_side"] = {"dim": side}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def random_params(cfg, seed=0):
    """float32 weights that are exact in bfloat16 would hide rounding differences; these are not.  Scales chosen so that
    scores, gates and clamps all operate in their interesting range."""
    rng = np.random.default_rng(seed)
    W, V = cfg["width"], cfg["vocab"]
    sd = (cfg.get("token_side") or {}).get("dim", 0)
    n = len(cfg["layers"])

    def mat(o, i, gain=1.0):
        return (rng.standard_normal((o, i)) * gain / np.sqrt(i)).astype(np.float32)

    def around(c, size, spread=0.2):
        return (c + spread * rng.standard_normal(size)).astype(np.float32)

    P = {"embed": rng.standard_normal((V, W)).astype(np.float32), "embed.norm": around(0.0, W), "final.norm": around(0.0, W),
         "head": mat(V, W)}
    if sd:
        P["side.embed"] = rng.standard_normal((V, n * sd)).astype(np.float32)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        P[p + "norm1"], P[p + "ls1"], P[p + "ls2"] = around(0.0, W), around(0.8, W), around(0.8, W)
        H = m["heads"]
        if L["type"] == "attention":
            G, D = m.get("kv_heads") or H, m["dim"]
            P[p + "mix.q"], P[p + "mix.k"] = mat(H * D, W, 2.0), mat(G * D, W, 2.0)
            P[p + "mix.q.b"], P[p + "mix.k.b"] = around(0.0, H * D, 0.3), around(0.0, G * D, 0.3)
            P[p + "mix.q.norm"], P[p + "mix.k.norm"] = around(1.2, H * D, 0.3), around(1.2, G * D, 0.3)
            P[p + "mix.g"], P[p + "mix.o"] = mat(H, W), mat(W, H * D)
        else:
            D, Dr, Dv, nc, nq = m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            P[p + "mix.dq"], P[p + "mix.dq.norm"], P[p + "mix.uq"] = mat(nq, W), around(1.0, nq), mat(H * (D + Dr), nq, 2.0)
            P[p + "mix.dkv"], P[p + "mix.dkv.norm"] = mat(nc + Dr, W, 2.0), around(1.0, nc)
            P[p + "mix.uk"], P[p + "mix.uv"] = mat(H * D, nc, 2.0), mat(H * Dv, nc)
            P[p + "mix.sink"] = around(1.0, H, 1.0)
            P[p + "mix.g"], P[p + "mix.o"] = mat(H, W), mat(W, H * Dv)
        if L.get("mlp"):
            f = L["mlp"]["ff"]
            P[p + "mlp.gate"], P[p + "mlp.up"], P[p + "mlp.down"] = mat(f, W, 2.0), mat(f, W, 2.0), mat(W, f)
        if sd:
            P[p + "side.gate"], P[p + "side.proj"], P[p + "side.norm"] = mat(sd, W), mat(W, sd), around(0.5, W, 0.15)
    return P
