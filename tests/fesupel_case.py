"""Small Fesupel configurations and weights for the tests (not the product's generator: shapes are derived here from
the config, so the product's own shape table is checked against this one)."""
import math

import torch


def left(heads, kv_heads, dim, vdim, size=None, rot_dims=None, base=10000.0, scaling=None, cap=20.0, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if size:
        m["mask"] = {"size": size}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    if cap:
        m["softcap"] = cap
    return m


def right(heads, kv_heads, dim, vdim, taps=4):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, identity=0, groups=None, shared_ff=None, limit=1.5, shared_limit=1.0):
    r = {"experts": experts, "top": top}
    if identity:
        r["identity"] = identity
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    f = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}
    if shared_ff:
        f["shared"] = {"ff": shared_ff, "limit": shared_limit}
    return f


def config(layers, width=64, vocab=97, eps=1e-5, side=8, embed_scale=None, lowrank=6):
    """layers: list of (left entry, right entry, mlp entry or None)."""
    cfg = {"architecture": "Fesupel", "width": width, "vocab": vocab, "norm": {"eps": eps},
           "embedding": {"scale": embed_scale if embed_scale is not None else math.sqrt(width)},
           "layers": [{"type": "parallel", "mixer": {"left": a, "right": b}, "mlp": f} for a, b, f in layers]}
    if side:
        cfg["token_side"] = {"dim": side}
    cfg["_lowrank"] = lowrank            # the tests' own key: the rank of the decay and gate pairs of the weights made here
    return cfg


def shapes(cfg):
    W, V, r = cfg["width"], cfg["vocab"], cfg["_lowrank"]
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    side = cfg.get("token_side")
    if side:
        out["side.embed"] = (V, len(cfg["layers"]) * side["dim"])
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        a, b, f = L["mixer"]["left"], L["mixer"]["right"], L["mlp"]
        out[p + "norm1"] = out[p + "norm1b"] = (W,)
        H, G, d, v = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        q = p + "mix.left."
        out.update({q + "q": (H * d, W), q + "q.b": (H * d,), q + "k": (G * d, W), q + "k.b": (G * d,),
                    q + "v": (G * v, W), q + "v.b": (G * v,), q + "talk": (H, H), q + "pb": (H,), q + "o": (W, H * v),
                    q + "out": (W,)})
        H, G, d, v, t = b["heads"], b["kv_heads"], b["dim"], b["vdim"], b["conv"]
        q = p + "mix.right."
        out.update({q + "q": (G * d, W), q + "q.conv": (G * d, t), q + "k": (G * d, W), q + "k.conv": (G * d, t),
                    q + "v": (H * v, W), q + "v.conv": (H * v, t), q + "b": (H, W), q + "A_log": (H,),
                    q + "norm": (v,), q + "a1": (r, W), q + "a2": (H * d, r), q + "dt_bias": (H * d,),
                    q + "g1": (r, W), q + "g2": (H * v, r), q + "o": (W, H * v), q + "out": (W,)})
        if f is not None:
            out[p + "norm2"] = out[p + "norm2b"] = (W,)
            q = p + "mlp."
            if f["kind"] == "dense":
                out.update({q + "up": (f["ff"], W), q + "down": (W, f["ff"])})
            else:
                E, n_out = f["router"]["experts"], f["router"]["experts"] + f["router"].get("identity", 0)
                out.update({q + "router": (n_out, W), q + "correction": (n_out,)})
                for e in range(E):
                    out.update({q + f"e{e}.gate": (f["expert"]["ff"], W), q + f"e{e}.up": (f["expert"]["ff"], W),
                                q + f"e{e}.down": (W, f["expert"]["ff"])})
                if "shared" in f:
                    sf = f["shared"]["ff"]
                    out.update({q + "shared.gate": (sf, W), q + "shared.up": (sf, W), q + "shared.down": (W, sf),
                                q + "shared.sg": (1, W)})
        if side:
            out.update({p + "side.gate": (side["dim"], W), p + "side.proj": (W, side["dim"]), p + "side.norm": (W,)})
    return out


def weights(cfg, seed=0):
    """bf16 tensors: projections N(0, 1/in) (the left half's queries and keys larger, so that its weights spread
    over (0, 1) and a key more or less shows), gains around one, a router whose choices are not near ties, decays that
    forget over tens of tokens."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shp in shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2", "norm1b", "norm2b", "out", "norm") or name == "final.norm":
            t = 1.0 + 0.3 * torch.randn(shp, generator=g)
        elif leaf == "talk":
            t = torch.eye(shp[0]) + 0.4 * torch.randn(shp, generator=g)
        elif leaf == "pb":
            t = -1.0 + torch.randn(shp, generator=g)
        elif leaf == "A_log":
            t = torch.log(0.3 + 3.0 * torch.rand(shp, generator=g))
        elif leaf == "dt_bias":
            t = -3.0 + 3.0 * torch.rand(shp, generator=g)
        elif leaf == "conv":
            t = torch.randn(shp, generator=g) * 0.6
        elif leaf == "correction":
            t = 0.3 * torch.randn(shp, generator=g)
        elif leaf == "router":
            t = 3.0 * torch.randn(shp, generator=g) / math.sqrt(shp[-1])
        elif leaf == "b" and len(shp) == 1:
            t = 0.3 * torch.randn(shp, generator=g)
        elif name in ("embed", "side.embed"):
            t = torch.randn(shp, generator=g)
        elif ".mix.left.q" in name or ".mix.left.k" in name:
            t = 2.0 * torch.randn(shp, generator=g) / math.sqrt(shp[-1])
        else:
            t = torch.randn(shp, generator=g) / math.sqrt(shp[-1])
        out[name] = t.to(torch.bfloat16)
    return out


def public(cfg):
    """The config as a model folder carries it (without the tests' own key)."""
    return {k: v for k, v in cfg.items() if not k.startswith("_")}


def logits_error(got, want):
    """Root mean square over the vocabulary of the difference of the mean-free logits, over that of the wanted ones;
    the largest over the rows."""
    got, want = got.double().cpu(), want.double().cpu()
    got = got - got.mean(dim=-1, keepdim=True)
    want = want - want.mean(dim=-1, keepdim=True)
    return float(((got - want).pow(2).mean(dim=-1).sqrt() / want.pow(2).mean(dim=-1).sqrt()).max())


SCALING = (8.0, 1.0, 4.0, 64)        # wavelengths of the small tables fall in all three bands

CONFIGS = {
    # grouped heads on both sides, sizes that differ from each other, every feed-forward kind, a layer without one
    "mix": config([
        (left(4, 2, 16, 24, size=10, rot_dims=8, scaling=SCALING), right(4, 2, 16, 8, taps=4), dense(96)),
        (left(4, 4, 12, 12, size=7, rot_dims=12), right(2, 2, 24, 32, taps=3),
         moe(6, 3, 32, identity=2, groups=(4, 2), shared_ff=48)),
        (left(6, 2, 8, 20, size=33, rot_dims=4, cap=0.0), right(3, 1, 8, 40, taps=2), None),
        (left(2, 1, 32, 16, size=10, rot_dims=16), right(4, 4, 32, 16, taps=4), moe(4, 2, 24)),
    ]),
    # no block limit, no turn, one group of experts with pass-through ones, no per-token term, one tap
    "plain": config([
        (left(2, 2, 16, 16, cap=5.0), right(2, 2, 16, 16, taps=1), moe(3, 2, 16, identity=1, shared_ff=16)),
        (left(3, 1, 20, 12, size=64, rot_dims=20, scaling=SCALING), right(2, 1, 12, 20, taps=5), dense(40)),
    ], width=48, side=0, embed_scale=1.0),
    # head sizes that fit the tensor-core tiles: blocks of positions that are no multiple of a tile, one layer without
    # a block limit, more heads than warps
    "tiles": config([
        (left(8, 2, 32, 32, size=24, rot_dims=16, scaling=SCALING), right(2, 1, 16, 16, taps=4), dense(64)),
        (left(4, 4, 16, 48, rot_dims=16), right(2, 2, 16, 16, taps=2), moe(4, 2, 16, identity=1)),
        (left(20, 5, 16, 16, size=50, rot_dims=8, cap=0.0), right(2, 2, 8, 8, taps=3), None),
    ], width=64, side=4),
    # sizes that are no multiple of four, blocks of one position and of two, many small heads
    "odd": config([
        (left(5, 5, 6, 10, size=1, rot_dims=2), right(5, 5, 10, 6, taps=3), moe(8, 4, 10, identity=4, groups=(3, 1))),
        (left(8, 2, 10, 6, size=2, rot_dims=6), right(6, 3, 6, 10, taps=4), dense(30)),
    ], width=40, vocab=61, side=3),
}
