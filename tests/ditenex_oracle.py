"""Plain float64 numpy statement of the Ditenex design, one function per mechanism, token rows in order.

Shares no code with the library.  Weights are a dict name -> array (matrices [out, in]); the configuration is the
dict of a config.json.  `forward(cfg, w, tokens)` runs a whole sequence at once and returns the logits of every
position and the residual stream after every layer; `Stepper` carries the same computation token by token with
explicit per-layer state (previous mixer input, cached keys and values), which is what the engine's cache has to
reproduce.
"""
import math

import numpy as np


def rms_norm(x, w, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def softplus(z):
    return np.log1p(np.exp(-np.abs(z))) + np.maximum(z, 0.0)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def xielu(z, p, q):
    """Positive side: softplus(p) z^2 + z/2.  Negative side: (1/2 + softplus(q)) (expm1(z) - z) + z/2."""
    ap, an = softplus(p), 0.5 + softplus(q)
    zn = np.minimum(z, 0.0)
    return np.where(z > 0, ap * z * z + 0.5 * z, an * (np.expm1(zn) - zn) + 0.5 * z)


def token_shift(h, prev, mu):
    """h [T, W] in order; prev [W] is the row before h[0] (zeros at the start of a sequence)."""
    before = np.concatenate([prev[None, :], h[:-1]], axis=0)
    return h + (before - h) * mu


def distance_slopes(heads):
    return np.array([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)])


def talking_window_attention(q, k, v, pos_q, pos_k, scale, window, talk):
    """q [Tq, H, d], k [Tk, G, d], v [Tk, G, dv]; pos_* absolute positions.  Scores get the linear distance
    penalty, are mixed over heads by `talk` [H, H], masked to the window (None: all earlier keys), then softmax."""
    Tq, H, d = q.shape
    G = k.shape[1]
    rep = H // G
    s = np.einsum("ihd,jhd->hij", q, np.repeat(k, rep, axis=1)) * scale
    dist = pos_q[:, None] - pos_k[None, :]
    s = s - distance_slopes(H)[:, None, None] * dist[None]
    s = np.einsum("hg,gij->hij", talk, s)
    ok = dist >= 0
    if window is not None:
        ok &= dist < window
    s = np.where(ok[None], s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=-1, keepdims=True)
    return np.einsum("hij,jhe->ihe", p, np.repeat(v, rep, axis=1))


def swiglu_expert(h, gate, up, down):
    a = h @ gate.T
    return (a * sigmoid(a) * (h @ up.T)) @ down.T


def route(h, router, correction, top, n_groups, keep, scale):
    """Returns (chosen [T, top], weights [T, top]).  The choice uses sigmoid scores plus `correction`, limited to
    the `keep` groups whose two best choice scores add up highest; the weights use the plain scores times scale."""
    s = sigmoid(h @ router.T)
    c = s + correction
    T, E = c.shape
    per = E // n_groups
    chosen = np.zeros((T, top), dtype=np.int64)
    weights = np.zeros((T, top))
    for t in range(T):
        g = c[t].reshape(n_groups, per)
        gs = np.sort(g, axis=1)[:, ::-1][:, :2].sum(axis=1)
        kept = sorted(range(n_groups), key=lambda i: (-gs[i], i))[:keep]
        allowed = np.full(E, -np.inf)
        for i in kept:
            allowed[i * per:(i + 1) * per] = c[t, i * per:(i + 1) * per]
        order = sorted(range(E), key=lambda e: (-allowed[e], e))[:top]
        chosen[t] = order
        weights[t] = s[t, order] * scale
    return chosen, weights


def _attn_cfg(mx):
    mask = mx.get("mask")
    return dict(H=mx["heads"], G=mx.get("kv_heads", mx["heads"]), d=mx["dim"], dv=mx.get("vdim", mx["dim"]), scale=mx["scale"],
                window=mask["size"] if mask else None, v_mix=bool(mx.get("v_mix", False)))


def first_vmix_layer(cfg):
    for i, L in enumerate(cfg["layers"]):
        if L["mixer"].get("v_mix"):
            return i
    return -1


def feed_forward(mlp, w, p, h):
    if mlp["kind"] == "dense":
        act = w[p + "act"]
        return xielu(h @ w[p + "up"].T, act[0], act[1]) @ w[p + "down"].T
    r = mlp["router"]
    grp = r.get("groups") or {"count": 1, "keep": 1}
    chosen, weights = route(h, w[p + "router"], w[p + "correction"], r["top"], grp["count"], grp["keep"], r.get("scale", 1.0))
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t], weights[t]):
            q = "%se%d." % (p, e)
            out[t] += wt * swiglu_expert(h[t:t + 1], w[q + "gate"], w[q + "up"], w[q + "down"])[0]
    if mlp.get("shared"):
        out += swiglu_expert(h, w[p + "shared.gate"], w[p + "shared.up"], w[p + "shared.down"])
    return out


class Stepper:
    """Runs portions of one sequence in order, keeping per layer: the last mixer input and all keys / values."""

    def __init__(self, cfg, w):
        self.cfg, self.w = cfg, w
        n = len(cfg["layers"])
        W = cfg["width"]
        self.prev = [np.zeros(W) for _ in range(n)]
        self.k = [None] * n
        self.v = [None] * n
        self.len = 0
        self.first = first_vmix_layer(cfg)

    def run(self, tokens):
        cfg, w = self.cfg, self.w
        eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
        T = len(tokens)
        pos = np.arange(self.len, self.len + T)
        x = w["embed"][np.asarray(tokens)] + w["pos"][pos]
        after = []
        v_first = None
        for i, L in enumerate(cfg["layers"]):
            p = "l%d." % i
            a = _attn_cfg(L["mixer"])
            h = rms_norm(x, w[p + "norm1"], eps)
            hs = token_shift(h, self.prev[i], w[p + "shift"])
            self.prev[i] = h[-1].copy()
            q = (hs @ w[p + "mix.q"].T + w[p + "mix.q.b"]).reshape(T, a["H"], a["d"])
            k = (hs @ w[p + "mix.k"].T + w[p + "mix.k.b"]).reshape(T, a["G"], a["d"])
            v = (hs @ w[p + "mix.v"].T + w[p + "mix.v.b"]).reshape(T, a["G"], a["dv"])
            if a["v_mix"]:
                if i == self.first:
                    v_first = v
                else:
                    lam = float(np.asarray(w[p + "mix.vmix"]).reshape(-1)[0])
                    v = (1.0 - lam) * v + lam * v_first.reshape(v.shape)
            self.k[i] = k if self.k[i] is None else np.concatenate([self.k[i], k])
            self.v[i] = v if self.v[i] is None else np.concatenate([self.v[i], v])
            o = talking_window_attention(q, self.k[i], self.v[i], pos, np.arange(self.len + T), a["scale"], a["window"], w[p + "mix.talk"])
            o = o.reshape(T, -1) * sigmoid(hs @ w[p + "mix.g"].T)
            x = x + m * rms_norm(o @ w[p + "mix.o"].T, w[p + "norm1b"], eps)
            if L.get("mlp"):
                h2 = rms_norm(x, w[p + "norm2"], eps)
                x = x + m * rms_norm(feed_forward(L["mlp"], w, p + "mlp.", h2), w[p + "norm2b"], eps)
            after.append(x.copy())
        self.len += T
        logits = rms_norm(x, w["final.norm"], eps) @ w["embed"].T
        return logits, np.stack(after)


def forward(cfg, w, tokens):
    return Stepper(cfg, w).run(tokens)
