"""Plain NumPy restatement of the Dolurax design, one function per mechanism, in float64.

It is the slow oracle of tests/test_dolurax_*.py: it takes the parsed config.json dictionary and a
{tensor name: ndarray} dictionary and shares no code with the package.  Everything is computed for one
whole sequence at once (no cache, no batching), so any disagreement that shows up only with a cache, a
batch or a cut prompt is the product's.

Notation: T tokens, W model width, H query heads, G key/value heads, D query/key size, Dv value size,
E experts, C chunk size.
"""
from __future__ import annotations

import numpy as np


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b over the last axis, var = mean squared deviation."""
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis (plain weight)."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def head_slopes(H):
    """slope of head h = 2^(-8 (h + 1) / H)"""
    return np.array([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)])


def visible(T, chunk):
    """[T, T] boolean: key j is visible from query i when j <= i and both lie in the same chunk of
    `chunk` positions counted from position 0 (chunk None or 0: plain causal)."""
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    m = j <= i
    if chunk:
        m &= (i // chunk) == (j // chunk)
    return m


def attention_core(q, k, v, scale, softcap, chunk):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv].
    score = scale q.k, squashed to softcap tanh(score / softcap), minus slope_h (i - j); softmax over
    the visible keys."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    slopes = head_slopes(H)
    vis = visible(T, chunk)
    dist = (np.arange(T)[:, None] - np.arange(T)[None, :]).astype(np.float64)
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // rep
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        if softcap:
            s = softcap * np.tanh(s / softcap)
        s = s - slopes[h] * dist
        s = np.where(vis, s, -np.inf)
        s = s - s.max(-1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(-1, keepdims=True)
        out[:, h, :] = p @ v[:, g, :]
    return out


def value_mix(v, v_first, lam):
    """(1 - lam) v + lam v_first"""
    return (1.0 - lam) * v + lam * v_first


def attention_mixer(h, P, pre, mx, eps, v_first):
    """The whole mixer on its input h [T, W].  `v_first` is None in the first value-mixing layer (and in
    layers that do not mix).  Returns (output [T, W], the values this layer caches [T, G, Dv])."""
    T = h.shape[0]
    H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (h @ P[pre + "q"].T).reshape(T, H, D)
    k = (h @ P[pre + "k"].T).reshape(T, G, D)
    v = (h @ P[pre + "v"].T).reshape(T, G, Dv)
    q = rms_norm(q, P[pre + "q.norm"], eps)
    k = rms_norm(k, P[pre + "k.norm"], eps)
    if v_first is not None:
        v = value_mix(v, v_first, float(P[pre + "vmix"]))
    o = attention_core(q, k, v, mx["scale"], mx.get("softcap"), (mx.get("mask") or {}).get("size"))
    o = o.reshape(T, H * Dv) * sigmoid(h @ P[pre + "g"].T)
    return o @ P[pre + "o"].T, v


def route(z, top, group_count, group_keep):
    """Router logits z [T, E] -> (chosen experts [T, top] by falling score, weights [T, top]).
    Scores are softmax(z); a group's score is its largest member; only members of the `group_keep`
    best of `group_count` equal groups of neighbours may be chosen; weights are the chosen scores
    over their sum (+1e-20)."""
    T, E = z.shape
    s = np.exp(z - z.max(-1, keepdims=True))
    s /= s.sum(-1, keepdims=True)
    allowed = np.ones((T, E), bool)
    if group_count and group_count > 1 and group_keep < group_count:
        per = E // group_count
        gs = s.reshape(T, group_count, per).max(-1)
        best = np.argsort(-gs, axis=-1, kind="stable")[:, :group_keep]
        ok = np.zeros((T, group_count), bool)
        np.put_along_axis(ok, best, True, axis=-1)
        allowed = np.repeat(ok, per, axis=-1)
    masked = np.where(allowed, s, -1.0)
    idx = np.argsort(-masked, axis=-1, kind="stable")[:, :top]
    w = np.take_along_axis(s, idx, axis=-1)
    return idx, w / (w.sum(-1, keepdims=True) + 1e-20)


def gated_ffn(h, P, pre):
    """W_down (silu(W_gate h) * (W_up h))"""
    return (silu(h @ P[pre + "gate"].T) * (h @ P[pre + "up"].T)) @ P[pre + "down"].T


def moe(h, P, pre, ml):
    r = ml["router"]
    groups = r.get("groups") or {}
    idx, w = route(h @ P[pre + "router"].T, r["top"], groups.get("count", 1), groups.get("keep", 1))
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, c in zip(idx[t], w[t]):
            out[t] += c * gated_ffn(h[t:t + 1], P, f"{pre}e{e}.")[0]
    if ml.get("shared"):
        out += gated_ffn(h, P, pre + "shared.")
    return out


def forward(cfg, P, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer)."""
    P = {k: np.asarray(v, np.float64) for k, v in P.items()}
    eps = cfg["norm"]["eps"]
    x = P["embed"][np.asarray(tokens)]
    v_first, seen_mix, layers = None, False, []
    for i, L in enumerate(cfg["layers"]):
        pre = f"l{i}."
        mx = L["mixer"]
        assert L["type"] == "attention"
        mixes = bool(mx.get("v_mix"))
        y, v = attention_mixer(x, P, pre + "mix.", mx, eps, v_first if (mixes and seen_mix) else None)
        if mixes and not seen_mix:
            v_first, seen_mix = v, True
        x = x + layer_norm(y, P[pre + "norm1"], P[pre + "norm1.b"], eps)
        if L.get("mlp"):
            x = x + layer_norm(moe(x, P, pre + "mlp.", L["mlp"]), P[pre + "norm2"], P[pre + "norm2.b"], eps)
        layers.append(x.copy())
    xn = layer_norm(x, P["final.norm"], P["final.norm.b"], eps)
    z = xn @ P["head"].T * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    if cap:
        z = cap * np.tanh(z / cap)
    return (z, np.stack(layers)) if return_layers else z


def random_params(cfg, seed=0, std=None):
    """Random tensors under the checkpoint's names for a config dictionary (float32 values that are exact
    in bfloat16, so that the same numbers reach the product and the oracle)."""
    rng = np.random.default_rng(seed)

    def bf(a):
        u = np.asarray(a, np.float32).view(np.uint32)
        u = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
        return u.view(np.float32)

    def lin(o, i, gain=1.0):
        return bf(rng.standard_normal((o, i)) * (gain / np.sqrt(i) if std is None else std))

    W, V = cfg["width"], cfg["vocab"]
    P = {"embed": bf(rng.standard_normal((V, W))), "head": lin(V, W),
         "final.norm": bf(1 + 0.1 * rng.standard_normal(W)), "final.norm.b": bf(0.1 * rng.standard_normal(W))}
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        for n in ("norm1", "norm2"):
            P[p + n] = bf(1 + 0.1 * rng.standard_normal(W))
            P[p + n + ".b"] = bf(0.1 * rng.standard_normal(W))
        H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
        P[p + "mix.q"], P[p + "mix.k"], P[p + "mix.v"] = lin(H * D, W, 2.0), lin(G * D, W, 2.0), lin(G * Dv, W)
        P[p + "mix.q.norm"] = bf(1 + 0.2 * rng.standard_normal(D))
        P[p + "mix.k.norm"] = bf(1 + 0.2 * rng.standard_normal(D))
        P[p + "mix.vmix"] = bf(np.array(rng.uniform(0.2, 0.6)))
        P[p + "mix.g"], P[p + "mix.o"] = lin(H * Dv, W), lin(W, H * Dv)
        ml = L.get("mlp")
        if ml:
            F = ml["expert"]["ff"]
            for e in range(ml["router"]["experts"]):
                q = f"{p}mlp.e{e}."
                P[q + "gate"], P[q + "up"], P[q + "down"] = lin(F, W), lin(F, W), lin(W, F)
            P[p + "mlp.router"] = lin(ml["router"]["experts"], W, 3.0)
            if ml.get("shared"):
                Fs = ml["shared"]["ff"]
                q = p + "mlp.shared."
                P[q + "gate"], P[q + "up"], P[q + "down"] = lin(Fs, W), lin(Fs, W), lin(W, Fs)
    return P


def make_config(vocab=96, width=64, layers=2, heads=4, kv_heads=2, dim=16, vdim=8, chunk=8, scale=0.25, softcap=20.0,
                v_mix=True, experts=8, top=2, groups=(2, 1), ff=16, shared_ff=24, eps=1e-5, logit_scale=1.5,
                logit_softcap=25.0, mlp=True):
    """A config.json dictionary with the same mixer / feed-forward in every layer (tests edit the entries
    of `layers` for mixed stacks)."""
    def layer():
        mx = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"size": chunk}, "scale": scale,
              "softcap": softcap, "v_mix": v_mix, "vdim": vdim}
        ml = None
        if mlp:
            ml = {"expert": {"ff": ff}, "kind": "moe",
                  "router": {"experts": experts, "groups": {"count": groups[0], "keep": groups[1]}, "top": top},
                  "shared": {"ff": shared_ff} if shared_ff else None}
        return {"type": "attention", "mixer": mx, "mlp": ml}
    return {"architecture": "Dolurax", "layers": [layer() for _ in range(layers)], "logit_scale": logit_scale,
            "logit_softcap": logit_softcap, "norm": {"eps": eps}, "vocab": vocab, "width": width}
