"""A plain, slow float64 restatement of the Dedunex design, one function per mechanism, token by token.

It shares no code with the library: attention keeps per-head keys and values in Python lists (the latent attention
expands every cached latent to per-head keys and values, it does not fold projections into the query), the recurrence
is a loop over tokens, the loop over layers is unrolled into a list of (layer, pass) pairs.

Notation: W is applied as W @ x; `w` maps tensor names to float64 arrays; a mixer's tensors are '<layer>.mix.<name>'.
"""
import math

import numpy as np


# ------------------------------------------------------------------------------------------------ small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis (weight None: no weight)"""
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if weight is None else y * weight


def group_rms_norm(x, weight, groups, eps):
    """the vector in `groups` equal consecutive parts, each divided by its own root mean square, the whole times weight"""
    parts = np.split(np.asarray(x, np.float64), groups)
    return np.concatenate([p / math.sqrt(float(np.mean(p * p)) + eps) for p in parts]) * weight


# ------------------------------------------------------------------------------------------------ rotary positions
def rotary_frequencies(rot):
    """(frequencies [dims/2], magnitude): base^(-2i/dims), blended between f/factor and f with a ramp when scaled"""
    dims, base = rot["dims"], rot["base"]
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0

    def turns_to_dim(t):
        return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(turns_to_dim(sc["fast"])), 0)
    hi = min(math.ceil(turns_to_dim(sc["slow"])), dims - 1)
    out = np.empty_like(f)
    for i in range(dims // 2):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out[i] = f[i] / sc["factor"] * ramp + f[i] * (1.0 - ramp)
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate_half(vec, pos, rot, pairing="half"):
    """rotary positions on the first rot.dims elements of vec: element i pairs with i + dims/2 ('half'; 'neighbours'
    pairs 2i with 2i+1 and exists so that a test can show that the pairing matters)"""
    if not rot or not rot.get("dims"):
        return vec.copy()
    dims = rot["dims"]
    f, mag = rotary_frequencies(rot)
    out = vec.copy()
    for i in range(dims // 2):
        a, b = (i, i + dims // 2) if pairing == "half" else (2 * i, 2 * i + 1)
        c, s = math.cos(pos * f[i]) * mag, math.sin(pos * f[i]) * mag
        out[a] = vec[a] * c - vec[b] * s
        out[b] = vec[b] * c + vec[a] * s
    return out


# ------------------------------------------------------------------------------------------------ attention
def softmax_attend(q, keys, values, scale, cap=0.0):
    """one query against a list of keys: softmax over (q.k * scale, soft-capped) weighs the values"""
    s = np.array([float(q @ k) * scale for k in keys])
    if cap:
        s = cap * np.tanh(s / cap)
    p = np.exp(s - s.max())
    p /= p.sum()
    return sum(pi * v for pi, v in zip(p, values))


def differential_lambda(w, p, diff):
    return math.exp(float(w[p + "lq1"] @ w[p + "lk1"])) - math.exp(float(w[p + "lq2"] @ w[p + "lk2"])) + diff


def differential_attention_step(w, p, mx, h, pos, cache, eps, pairing="half"):
    """one token of the differential attention; cache: list of (keys [G, 2, dim], values [G, vdim]) of all earlier tokens"""
    H, G, d, vd = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx.get("vdim", mx["dim"])
    rot = mx.get("rot")
    q = (w[p + "q"] @ h + w[p + "q.b"]).reshape(H, 2, d)
    k = (w[p + "k"] @ h + w[p + "k.b"]).reshape(G, 2, d)
    v = (w[p + "v"] @ h + w[p + "v.b"]).reshape(G, vd)
    for a in range(H):
        for m in range(2):
            q[a, m] = rotate_half(rms_norm(q[a, m], w[p + "q.norm"], eps), pos, rot, pairing)
    for g in range(G):
        for m in range(2):
            k[g, m] = rotate_half(rms_norm(k[g, m], w[p + "k.norm"], eps), pos, rot, pairing)
    cache.append((k, v))
    size = (mx.get("mask") or {}).get("size", 0)
    seen = cache if not size else cache[max(0, len(cache) - size):]  # the token itself and the size - 1 before it
    lam, diff = differential_lambda(w, p, mx.get("diff", 0.0)), mx.get("diff", 0.0)
    out = np.zeros((H, vd))
    for a in range(H):
        g = a // (H // G)
        maps = [softmax_attend(q[a, m], [kk[g, m] for kk, _ in seen], [vv[g] for _, vv in seen], mx["scale"], mx.get("softcap", 0.0)) for m in range(2)]
        o = maps[0] - lam * maps[1]
        out[a] = rms_norm(o, None, eps) * (1.0 - diff)
    return w[p + "o"] @ out.reshape(-1)


def latent_attention_step(w, p, mx, h, pos, cache, eps, pairing="half"):
    """one token of the latent attention; cache: list of (normed latent [kv_rank], rotated shared key [rot_dim])"""
    H, d, vd, r, kr = mx["heads"], mx["dim"], mx.get("vdim", mx["dim"]), mx.get("rot_dim", 0), mx["kv_rank"]
    rot = mx.get("rot")
    cq = rms_norm(w[p + "dq"] @ h, w[p + "dq.norm"], eps)
    q = (w[p + "uq"] @ cq).reshape(H, d + r)
    dkv = w[p + "dkv"] @ h
    c = rms_norm(dkv[:kr], w[p + "dkv.norm"], eps)
    cache.append((c, rotate_half(dkv[kr:], pos, rot, pairing)))
    gate = sigmoid(w[p + "g"] @ h)
    out = np.zeros((H, vd))
    for a in range(H):
        uk, uv = w[p + "uk"][a * d:(a + 1) * d], w[p + "uv"][a * vd:(a + 1) * vd]
        qa = np.concatenate([q[a, :d], rotate_half(q[a, d:], pos, rot, pairing)])
        keys = [np.concatenate([uk @ cc, kk]) for cc, kk in cache]  # every earlier token and this one
        vals = [uv @ cc for cc, _ in cache]
        out[a] = softmax_attend(qa, keys, vals, mx["scale"]) * gate[a]
    return w[p + "o"] @ out.reshape(-1)


# ------------------------------------------------------------------------------------------------ minGRU, feed-forward
def mingru_step(w, p, h, state):
    """state (float64 [width]) is updated in place"""
    z = sigmoid(w[p + "z"] @ h + w[p + "z.b"])
    u = w[p + "x"] @ h + w[p + "x.b"]
    cand = np.where(u >= 0.0, u + 0.5, sigmoid(u))
    state[:] = (1.0 - z) * state + z * cand
    return w[p + "o"] @ (state * silu(w[p + "g"] @ h))


def gated_feed_forward(w, p, h):
    return w[p + "down"] @ (gelu_tanh(w[p + "gate"] @ h) * (w[p + "up"] @ h))


# ------------------------------------------------------------------------------------------------ the model
def layer_runs(cfg):
    """[(layer, pass or None)]: layers start .. stop-1 run `times` times in a row; pass t is set on the first layer of pass t"""
    n = len(cfg["layers"])
    lp = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    runs = [(i, None) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t if i == lp["start"] else None) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, None) for i in range(lp["stop"], n)]


class Stepper:
    """feeds tokens one by one; every layer run keeps what its mixer carries (keys and values, latents, or a state)"""

    def __init__(self, cfg, w, pairing="half"):
        self.cfg, self.w, self.pairing, self.pos = cfg, w, pairing, 0
        self.runs = layer_runs(cfg)
        self.carried = []
        for i, _ in self.runs:
            ly = cfg["layers"][i]
            self.carried.append(np.zeros(ly["mixer"]["width"]) if ly["type"] == "mingru" else [])

    def step(self, token):
        cfg, w = self.cfg, self.w
        eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups", 1)
        x = group_rms_norm(w["embed"][token], w["embed.norm"], groups, eps)
        after = []
        for k, (i, t) in enumerate(self.runs):
            ly, p = cfg["layers"][i], f"l{i}."
            if t is not None:
                x = x + w["loop.step"][t]
            h = group_rms_norm(x, w[p + "norm1"], groups, eps)
            if ly["type"] == "attention":
                y = differential_attention_step(w, p + "mix.", ly["mixer"], h, self.pos, self.carried[k], eps, self.pairing)
            elif ly["type"] == "latent_attention":
                y = latent_attention_step(w, p + "mix.", ly["mixer"], h, self.pos, self.carried[k], eps, self.pairing)
            else:
                y = mingru_step(w, p + "mix.", h, self.carried[k])
            if ly.get("mlp"):
                y = y + gated_feed_forward(w, p + "mlp.", h)
            x = x + y
            after.append(x.copy())
        self.pos += 1
        return w["head"] @ group_rms_norm(x, w["final.norm"], groups, eps), np.stack(after)

    def run(self, tokens):
        """-> logits [n, vocab], stream after every layer run [runs, n, width]"""
        out = [self.step(t) for t in tokens]
        return np.stack([o[0] for o in out]), np.stack([o[1] for o in out], axis=1)


def forward(cfg, w, tokens, pairing="half"):
    return Stepper(cfg, w, pairing).run(tokens)
