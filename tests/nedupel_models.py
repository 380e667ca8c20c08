"""Small Nedupel configurations and weights for the tests (numpy generator; values that bfloat16 holds exactly)."""
import json
import os
import zlib

import numpy as np
import torch


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, scaling=None, kv_from=None, rot=True):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if rot:
        m["rot"] = {"dims": rot_dim, "base": base}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def retention(heads, dim, vdim, decay, rot=None, scaling=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "retention", "mixer": m}


def dense(layer, ff):
    return dict(layer, mlp={"kind": "dense", "ff": ff})


def moe(layer, ff, limit, experts, top):
    return dict(layer, mlp={"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}})


def bare(layer):
    return dict(layer, mlp=None)


def config(width, vocab, layers, eps=1e-5, emb=3.0, mult=0.8, logit=0.5, **extra):
    return {"architecture": "Nedupel", "vocab": vocab, "width": width, "embedding": {"scale": emb}, "residual_mult": mult,
            "logit_scale": logit, "norm": {"eps": eps}, "layers": layers, **extra}


# both mixers, both feed-forwards and none, two layers that read an earlier layer's cache (one of them not the layer
# before), interpolated and plain rotations, different heads and sizes in every layer
HYBRID = config(64, 300, [
    moe(retention(4, 16, 24, [0.9, 0.95, 0.99, 0.999], rot=(16, 10000.0)), 40, 1.5, 6, 2),
    dense(latent(4, 16, 8, 24, 40, 0.3, base=5000.0, scaling=(4.0, 64, 16.0, 1.0)), 96),
    bare(latent(3, 8, 16, 8, 24, 0.25, base=300.0)),
    moe(latent(2, 24, 8, 16, 40, 0.2, base=5000.0, scaling=(4.0, 64, 16.0, 1.0), kv_from=1), 32, 3.0, 5, 3),
    dense(retention(2, 32, 8, [0.97, 0.5], rot=(8, 50.0)), 72),
    moe(latent(5, 8, 16, 16, 24, 0.4, base=300.0, kv_from=2), 24, 0.7, 4, 1),
])
# sizes that are no multiple of 8, one head, one expert, top 1, all constants 1, no rotation in one layer of each kind,
# a decay of 1 (nothing forgotten) and of 0 (nothing kept)
ODD = config(40, 131, [
    moe(latent(1, 6, 10, 5, 13, 1.0, base=77.0), 12, 1.0, 1, 1),
    dense(retention(3, 10, 6, [1.0, 0.0, 0.75], rot=(6, 20.0)), 52),
    bare(latent(3, 10, 6, 7, 9, 0.5, rot=False)),
    moe(retention(1, 12, 20, [0.9]), 20, 2.5, 7, 7),
], eps=1e-3, emb=1.0, mult=1.0, logit=1.0)
ONLY_LATENT = config(48, 200, [bare(latent(4, 16, 8, 8, 24, 0.25, base=300.0, scaling=(8.0, 32, 8.0, 2.0)))])
ONLY_RETENTION = config(48, 200, [bare(retention(4, 24, 16, [0.9, 0.99, 0.8, 0.999], rot=(12, 1000.0)))])
ONLY_MOE = config(48, 200, [moe(retention(1, 8, 8, [0.5]), 56, 1.2, 9, 2)])
ONLY_DENSE = config(48, 200, [dense(retention(1, 8, 8, [0.5]), 128)])
# attention whose softmax is sharp (large query and latent weights): one key stands out among hundreds
SHARP = config(64, 150, [
    bare(latent(4, 16, 16, 16, 32, 1.0, base=1000.0)),
    dense(latent(2, 32, 16, 16, 32, 0.8, base=1000.0, kv_from=0), 64),
])
# cache rows of 64 and 128 values with at most 16 heads: the sizes the tensor-core attention kernels take in bfloat16
WIDE = config(128, 200, [
    dense(latent(4, 32, 16, 32, 48, 0.125, base=10000.0), 128),
    moe(latent(16, 16, 32, 8, 96, 0.2, base=500.0, scaling=(2.0, 128, 32.0, 1.0)), 64, 2.0, 8, 2),
    bare(latent(2, 64, 16, 64, 48, 0.1, base=10000.0, kv_from=0)),
    bare(retention(2, 128, 64, [0.99, 0.9], rot=(128, 10000.0))),
    bare(latent(20, 8, 16, 8, 48, 0.3, base=700.0)),              # more than 16 heads: decode steps take them in groups
])
# the large ends: a cache row of 256 values, keys of 256 and 300 in retention, many experts, a wide expert
LARGE = config(96, 180, [
    bare(latent(8, 40, 64, 24, 192, 0.06, base=10000.0)),
    moe(retention(2, 256, 40, [0.99, 0.95], rot=(64, 10000.0)), 200, 2.0, 70, 4),
    bare(retention(1, 300, 12, [0.9])),
])

# a width, a vocabulary and inner sizes that are no multiple of 8 or of 4 anywhere
RAGGED = config(52, 97, [
    moe(retention(2, 14, 9, [0.9, 0.8], rot=(10, 33.0)), 18, 1.1, 3, 2),
    dense(latent(3, 7, 6, 5, 11, 0.4, base=90.0), 30),
    bare(latent(2, 5, 6, 9, 11, 0.6, base=90.0, kv_from=1)),
], eps=1e-4, emb=2.0, mult=0.9, logit=1.5)

CONFIGS = {"ragged": RAGGED, "hybrid": HYBRID, "odd": ODD, "latent": ONLY_LATENT, "retention": ONLY_RETENTION, "moe": ONLY_MOE,
           "dense": ONLY_DENSE, "sharp": SHARP, "wide": WIDE, "large": LARGE}


def tensor_shapes(cfg):
    D, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s[p + "norm1"] = (D,)
        mlp = L.get("mlp")
        if mlp:
            s[p + "norm2"] = (D,)
            if mlp["kind"] == "dense":
                s[p + "mlp.up"], s[p + "mlp.down"] = (mlp["ff"], D), (D, mlp["ff"])
            else:
                F = mlp["expert"]["ff"]
                for e in range(mlp["router"]["experts"]):
                    s[f"{p}mlp.e{e}.gate"] = s[f"{p}mlp.e{e}.up"] = (F, D)
                    s[f"{p}mlp.e{e}.down"] = (D, F)
                s[p + "mlp.table"] = (V, mlp["router"]["top"])
        p += "mix."
        H = m["heads"]
        if L["type"] == "latent_attention":
            s.update({p + "q": (H * (m["dim"] + m["rot_dim"]), D), p + "uk": (H * m["dim"], m["kv_rank"]),
                      p + "uv": (H * m["vdim"], m["kv_rank"]), p + "o": (D, H * m["vdim"])})
            if m.get("kv_from") is None:
                s.update({p + "dkv": (m["kv_rank"] + m["rot_dim"], D), p + "dkv.norm": (m["kv_rank"],)})
        else:
            s.update({p + "q": (H * m["dim"], D), p + "k": (H * m["dim"], D), p + "v": (H * m["vdim"], D),
                      p + "g": (H * m["vdim"], D), p + "o": (D, H * m["vdim"])})
    return s


def make_weights(cfg, seed, sharp=False):
    rng = np.random.default_rng(seed)
    W = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if last == "table":
            E = next(L for i, L in enumerate(cfg["layers"]) if name.startswith(f"l{i}."))["mlp"]["router"]["experts"]
            W[name] = torch.tensor(np.stack([rng.permutation(E)[:shape[1]] for _ in range(shape[0])]), dtype=torch.int32)
            continue
        if name == "embed":
            w = rng.normal(0, 1.0, shape)
        elif name.endswith("dkv.norm"):
            w = (3.0 if sharp else 1.0) * (1.0 + 0.1 * rng.normal(size=shape))
        elif last in ("norm", "norm1", "norm2"):
            w = 0.1 * rng.normal(size=shape)                    # stored around zero
        elif len(shape) == 2:
            w = rng.normal(0, (3.0 if sharp and last == "q" else 1.0) / np.sqrt(shape[1]), shape)
        else:
            w = 0.1 * rng.normal(size=shape)
        W[name] = torch.tensor(np.asarray(w), dtype=torch.float32).to(torch.bfloat16)
    return W


def write_models(root, names=None):
    """name -> (folder, config, weights as float64 numpy; tables as int64)."""
    from mynah_slm_b200.weights.safetensors_io import write_safetensors
    out = {}
    for name, cfg in CONFIGS.items():
        if names is not None and name not in names:
            continue
        folder = os.path.join(str(root), name)
        os.makedirs(folder)
        W = make_weights(cfg, zlib.crc32(name.encode()) % 1000, sharp=name == "sharp")      # a seed that stays with the name
        with open(os.path.join(folder, "config.json"), "w") as f:
            json.dump(cfg, f)
        write_safetensors(os.path.join(folder, "model.safetensors"), W)
        out[name] = (folder, cfg, {n: (t.to(torch.float64) if t.dtype.is_floating_point else t.to(torch.int64)).numpy()
                                   for n, t in W.items()})
    return out
