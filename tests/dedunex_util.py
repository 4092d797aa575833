"""Helpers of the Dedunex tests: small configurations and bf16-exact random weights written as a model folder
(config.json + model.safetensors)."""
import numpy as np

from nogatar_util import bf16_round, rel_err, values, write_model  # noqa: F401  (format helpers, not model code)


def rot(dims, base=10000.0, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        r["scaling"] = scaling
    return r


YARN = {"factor": 8.0, "fast": 16.0, "original": 64, "slow": 2.0}


def attn(heads=4, kv_heads=2, dim=6, vdim=5, window=7, scale=0.8, softcap=12.0, diff=0.3, rot_dims=4, base=100.0, scaling=None, mlp=None):
    mx = {"diff": diff, "dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if softcap:
        mx["softcap"] = softcap
    if window:
        mx["mask"] = {"size": window}
    if rot_dims:
        mx["rot"] = rot(rot_dims, base, scaling)
    return {"type": "attention", "mixer": mx, "mlp": mlp}


def latent(heads=3, dim=6, vdim=5, rot_dim=4, kv_rank=10, q_rank=9, scale=0.5, base=100.0, scaling=None, mlp=None):
    mx = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "q_rank": q_rank, "rot_dim": rot_dim, "scale": scale, "vdim": vdim}
    if rot_dim:
        mx["rot"] = rot(rot_dim, base, scaling)
    return {"type": "latent_attention", "mixer": mx, "mlp": mlp}


def gru(width=14, mlp=None):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def dense(ff=14):
    return {"ff": ff, "kind": "dense"}


def make_config(layers, width=20, vocab=37, eps=1e-5, groups=2, loop=None):
    cfg = {"architecture": "Dedunex", "layers": layers, "norm": {"eps": eps, "groups": groups}, "vocab": vocab, "width": width}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def tensor_shapes(cfg):
    W = cfg["width"]
    out = {"embed": (cfg["vocab"], W), "embed.norm": (W,)}
    if cfg.get("loop"):
        out["loop.step"] = (cfg["loop"]["times"], W)
    for i, ly in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", ly["mixer"]
        out[p + "norm1"] = (W,)
        if ly["type"] == "attention":
            H, G, d, vd = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
            out.update({p + "mix.q": (H * 2 * d, W), p + "mix.q.b": (H * 2 * d,), p + "mix.k": (G * 2 * d, W), p + "mix.k.b": (G * 2 * d,),
                        p + "mix.v": (G * vd, W), p + "mix.v.b": (G * vd,), p + "mix.q.norm": (d,), p + "mix.k.norm": (d,),
                        p + "mix.lq1": (d,), p + "mix.lk1": (d,), p + "mix.lq2": (d,), p + "mix.lk2": (d,), p + "mix.o": (W, H * vd)})
        elif ly["type"] == "latent_attention":
            H, d, vd, r, kr, qr = mx["heads"], mx["dim"], mx["vdim"], mx["rot_dim"], mx["kv_rank"], mx["q_rank"]
            out.update({p + "mix.dq": (qr, W), p + "mix.dq.norm": (qr,), p + "mix.uq": (H * (d + r), qr), p + "mix.dkv": (kr + r, W),
                        p + "mix.dkv.norm": (kr,), p + "mix.uk": (H * d, kr), p + "mix.uv": (H * vd, kr), p + "mix.g": (H, W), p + "mix.o": (W, H * vd)})
        else:
            C = mx["width"]
            out.update({p + "mix.z": (C, W), p + "mix.z.b": (C,), p + "mix.x": (C, W), p + "mix.x.b": (C,), p + "mix.g": (C, W), p + "mix.o": (W, C)})
        if ly.get("mlp"):
            ff = ly["mlp"]["ff"]
            out.update({p + "mlp.gate": (ff, W), p + "mlp.up": (ff, W), p + "mlp.down": (W, ff)})
    out["final.norm"] = (W,)
    out["head"] = (cfg["vocab"], W)
    return out


def random_weights(cfg, seed=0, gain=1.0):
    """name -> (bf16 bits, float64 values)"""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if name == "embed":
            a = rng.standard_normal(shape)
        elif name == "loop.step":
            a = 0.7 * rng.standard_normal(shape)
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            a = 0.6 * rng.standard_normal(shape) / np.sqrt(shape[0]) ** 0.5
        elif len(shape) == 2:
            a = rng.standard_normal(shape) * gain / np.sqrt(shape[1])
        elif "norm" in name:
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        else:
            a = 0.5 * rng.standard_normal(shape)
        out[name] = bf16_round(np.asarray(a, np.float32))
    return out


def set_values(weights, name, vals):
    weights[name] = bf16_round(np.asarray(vals, np.float32))
