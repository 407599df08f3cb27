"""Small Zomurax configurations and weights for the tests (not the product's generator: shapes are derived
here from the config, so the product's own shape table is checked against this one)."""
import math

import torch


def attn(heads, kv_heads, dim, vdim, temp=None, v_mix=False, scale=None):
    """temp: (coef, every) or None."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if temp is not None:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m}


def latent(heads, dim, rot_dim, vdim, rank, window=None, base=10000.0, scale=None, rot_dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
         "rot": {"base": base, "dims": rot_dims if rot_dims is not None else rot_dim},
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def moe(experts, top, ff, shared_ff=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared_ff:
        f["shared"] = {"ff": shared_ff}
    return f


def config(layers, width=64, vocab=97, eps=1e-5, alpha=1.5, softcap=20.0):
    """layers: list of (mixer entry, mlp entry or None)."""
    cfg = {"architecture": "Zomurax", "width": width, "vocab": vocab, "norm": {"eps": eps}, "postln_alpha": alpha,
           "layers": [dict(m, mlp=f) for m, f in layers]}
    if softcap:
        cfg["logit_softcap"] = softcap
    return cfg


def shapes(cfg):
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "final.norm": (), "head": (V, W)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = ()
        if L["type"] == "attention":
            H, G, d, v = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.v": (G * v, W), p + "mix.o": (W, H * v),
                        p + "mix.r1": (H,), p + "mix.r2": (H,), p + "mix.sink": (H,)})
            if m.get("v_mix"):
                out[p + "mix.vmix"] = ()
        else:
            H, d, rd, v, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out.update({p + "mix.q": (H * (d + rd), W), p + "mix.dkv": (r + rd, W), p + "mix.dkv.norm": (r,),
                        p + "mix.uk": (H * d, r), p + "mix.uv": (H * v, r), p + "mix.o": (W, H * v)})
        f = L["mlp"]
        if f is not None:
            out[p + "norm2"] = ()
            out[p + "mlp.table"] = (V, f["router"]["top"])
            for e in range(f["router"]["experts"]):
                out.update({p + f"mlp.e{e}.gate": (f["expert"]["ff"], W), p + f"mlp.e{e}.up": (f["expert"]["ff"], W),
                            p + f"mlp.e{e}.down": (W, f["expert"]["ff"])})
            if "shared" in f:
                sf = f["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (sf, W), p + "mlp.shared.up": (sf, W), p + "mlp.shared.down": (W, sf)})
    return out


def weights(cfg, seed=0):
    """bf16 tensors (tables int32): projections N(0, 1/in) (queries and keys of the latent attention larger so that
    it is peaked and the window's edge matters), gains around one, sinks and bias numbers of a size that shows."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shp in shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf == "table":
            E = cfg["layers"][int(name.split(".")[0][1:])]["mlp"]["router"]["experts"]
            out[name] = torch.stack([torch.randperm(E, generator=g)[: shp[1]] for _ in range(shp[0])]).to(torch.int32)
            continue
        if leaf in ("norm1", "norm2") or name == "final.norm":
            t = 1.0 + 0.3 * torch.randn(shp, generator=g)
        elif leaf == "norm":
            t = 1.0 + 0.3 * torch.randn(shp, generator=g)
        elif leaf == "vmix":
            t = 0.2 + 0.6 * torch.rand(shp, generator=g)
        elif leaf == "r1":
            t = 0.1 + 0.6 * torch.rand(shp, generator=g)
        elif leaf == "r2":
            t = 0.05 + 0.5 * torch.rand(shp, generator=g)
        elif leaf == "sink":
            t = 1.0 + torch.randn(shp, generator=g)
        elif name == "embed":
            t = torch.randn(shp, generator=g)
        elif leaf in ("q", "dkv", "uk") and ".mix." in name:
            t = 2.0 * torch.randn(shp, generator=g) / math.sqrt(shp[-1])
        else:
            t = torch.randn(shp, generator=g) / math.sqrt(shp[-1])
        out[name] = t.to(torch.bfloat16)
    return out


def logits_error(got: torch.Tensor, want: torch.Tensor) -> float:
    """Largest per-row error: rms over the vocabulary of the difference (mean removed) over the rms of the
    expected logits."""
    d = got.double().cpu() - want.double().cpu()
    d = d - d.mean(-1, keepdim=True)
    scale = want.double().pow(2).mean().sqrt()
    return float(d.pow(2).mean(-1).sqrt().max() / scale)


# the configurations the model-level tests run: both mixers in several orders; key/value heads shared by 1, 2, 3 and 4
# query heads; widths that are no powers of two; 1, 2 and 3 experts per token with and without a shared expert; a
# layer without feed-forward; value sharing over two and three layers with an attention layer outside the set between
# them; windows 5 to 40; temperatures that step every 7 to 16 tokens; residual weights 1, 1.5 and 3; with and
# without the logit cap; head sizes that fit the tensor-core kernels (multiples of 16) and head sizes that do not
CONFIGS = {
    "mix": config([(latent(4, 16, 8, 24, 20, window=9), moe(5, 2, 24, 40)),
                   (attn(4, 2, 16, 32, temp=(0.4, 7), v_mix=True), moe(5, 2, 24, 40)),
                   (latent(4, 16, 8, 24, 20, window=5), None),
                   (attn(6, 6, 8, 8), moe(3, 3, 16)),
                   (attn(4, 2, 16, 32, temp=(0.4, 7), v_mix=True), moe(5, 2, 24, 40)),
                   (attn(4, 2, 16, 32, v_mix=True, scale=0.31), moe(4, 1, 32, 8))],
                  width=64, vocab=97),
    "attn_first": config([(attn(6, 2, 12, 20, temp=(0.25, 16), v_mix=True), moe(7, 3, 20)),
                          (latent(3, 10, 6, 12, 14, window=24, base=500.0), moe(2, 2, 36, 12)),
                          (attn(6, 2, 12, 20, v_mix=True), None)],
                         width=48, vocab=61, eps=1e-6, alpha=1.0, softcap=0.0),
    # every product a multiple of 128 wide and deep: decode-sized bf16 steps hand split-K partials to fused consumers
    "wide": config([(attn(4, 1, 32, 32, temp=(0.3, 9), v_mix=True), moe(4, 2, 128, 128)),
                    (latent(4, 32, 16, 32, 48, window=40), moe(4, 2, 128, 128)),
                    (attn(4, 1, 32, 32, v_mix=True), moe(4, 1, 128))],
                   width=128, vocab=160, alpha=3.0, softcap=8.0),
    "plain": config([(latent(2, 32, 16, 16, 32, rot_dims=8), moe(3, 1, 48)), (attn(3, 1, 16, 48, temp=(1.0, 10)), moe(3, 1, 48, 16))],
                    width=80, vocab=130, alpha=2.0),
}
