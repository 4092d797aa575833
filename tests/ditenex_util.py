"""Helpers of the Ditenex tests: small configurations and bf16-exact random weights written as a model folder
(config.json + model.safetensors)."""
import numpy as np

from nogatar_util import bf16_round, rel_err, values, write_model  # noqa: F401  (format helpers, not model code)


def attn(heads=4, kv_heads=2, dim=6, vdim=5, window=7, scale=0.4, v_mix=True, mlp=None):
    mx = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "v_mix": v_mix, "vdim": vdim}
    if window:
        mx["mask"] = {"size": window}
    return {"type": "attention", "mixer": mx, "mlp": mlp}


def dense(ff=14):
    return {"ff": ff, "kind": "dense"}


def moe(experts=6, top=2, ff=9, groups=3, keep=2, scale=1.25, shared_ff=10):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "scale": scale, "top": top}}
    if groups:
        m["router"]["groups"] = {"count": groups, "keep": keep}
    if shared_ff:
        m["shared"] = {"ff": shared_ff}
    return m


def make_config(layers, width=20, vocab=37, eps=1e-5, res_mult=0.4, max_positions=512):
    return {"architecture": "Ditenex", "layers": layers, "max_positions": max_positions, "norm": {"eps": eps}, "residual_mult": res_mult,
            "vocab": vocab, "width": width}


def tensor_shapes(cfg):
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "pos": (cfg["max_positions"], W)}
    for i, ly in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", ly["mixer"]
        H, G, d, vd = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
        out.update({p + "norm1": (W,), p + "norm1b": (W,), p + "shift": (W,), p + "mix.q": (H * d, W), p + "mix.q.b": (H * d,),
                    p + "mix.k": (G * d, W), p + "mix.k.b": (G * d,), p + "mix.v": (G * vd, W), p + "mix.v.b": (G * vd,), p + "mix.vmix": (),
                    p + "mix.talk": (H, H), p + "mix.g": (H * vd, W), p + "mix.o": (W, H * vd)})
        mlp = ly.get("mlp")
        if not mlp:
            continue
        out.update({p + "norm2": (W,), p + "norm2b": (W,)})
        if mlp["kind"] == "dense":
            out.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"]), p + "mlp.act": (2,)})
        else:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            for e in range(E):
                out.update({p + f"mlp.e{e}.gate": (ff, W), p + f"mlp.e{e}.up": (ff, W), p + f"mlp.e{e}.down": (W, ff)})
            out.update({p + "mlp.router": (E, W), p + "mlp.correction": (E,)})
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (sf, W), p + "mlp.shared.up": (sf, W), p + "mlp.shared.down": (W, sf)})
    out["final.norm"] = (W,)
    return out


def random_weights(cfg, seed=0, gain=1.0):
    """name -> (bf16 bits, float64 values)"""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if last == "talk":
            a = np.eye(shape[0]) + 0.4 * rng.standard_normal(shape)
        elif name == "pos":
            a = 0.5 * rng.standard_normal(shape)
        elif last == "router":
            a = 3.0 * rng.standard_normal(shape) / np.sqrt(shape[1])
        elif len(shape) == 2:
            a = rng.standard_normal(shape) * gain / np.sqrt(shape[1])
        elif "norm" in name:
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif last in ("shift", "vmix"):
            a = rng.uniform(0.1, 0.9, shape)
        elif last == "correction":
            a = 0.3 * rng.standard_normal(shape)
        else:
            a = 0.5 * rng.standard_normal(shape)
        out[name] = bf16_round(np.asarray(a, np.float32))
    return out


def set_values(weights, name, vals):
    weights[name] = bf16_round(np.asarray(vals, np.float32))
