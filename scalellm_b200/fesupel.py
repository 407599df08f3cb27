"""Fesupel: a decoder-only model whose layers are listed in its config.json.

    x          = "embedding.scale" * embed[tok]                                              (fp32 residual)
    per layer  : x <- x + norm(mixer(norm(x, norm1)), norm1b) ; x <- x + norm(ff(norm(x, norm2)), norm2b) (unless
                 "mlp" is null) ; x <- x + norm(P_i (gelu_tanh(G_i x) * side[tok, i-th slice]), n_i)  (config
                 "token_side");  norm(z, w) = z / sqrt(mean(z^2) + eps) * w
    mixer      : "parallel": two mixers on the same rows, (norm(left, "left.out") + norm(right, "right.out")) / 2
                 (layers.ParallelMixer + layers.BranchNormResidual)
                 left  — layers.SigmoidBlockAttention: biased q / k / v, partial rotary turn over channel pairs
                         (t, t + dims / 2) with wavelength-band frequency scaling, score cap, sigmoid weights with a
                         bias per head inside blocks of "mask.size" positions, head mix "talk", grouped key/value heads
                 right — layers.GatedDeltaMixer: short causal filters + silu on q, k, v, unit-length q and k, decay per
                         head and key channel through a low-rank pair, write strength beta, per-head RMS norm of the
                         read-out with an output gate through a low-rank pair
    feed-forward: "dense" (layers.ReluSquaredMLP) or "moe" (layers.GroupLimitedMoE: softmax router with a choice
                 correction, group limit, pass-through experts ("router.identity"), clamped-GLU experts, a gated shared
                 expert)
    output     : norm(x, "final.norm"), then the vocabulary projection.

Every size and constant is read from config.json or a tensor's shape.  Tensor names: "embed", "side.embed", "head",
"final.norm", and per layer i "l<i>.norm1|norm1b|norm2|norm2b", "l<i>.side.gate|proj|norm",
"l<i>.mix.left.q|k|v(.b)|talk|pb|o|out", "l<i>.mix.right.q|k|v(.conv)|b|A_log|dt_bias|a1|a2|g1|g2|norm|o|out",
"l<i>.mlp.up|down" (dense) or "l<i>.mlp.e<j>.gate|up|down", "l<i>.mlp.router|correction",
"l<i>.mlp.shared.gate|up|down|sg".

State per sequence: the turned keys and the values of the left halves in paged KVCache rows; the delta-rule matrices
and the last filter inputs of the right halves in state slots.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from . import _lib, kernels
from .layers import (BranchNormResidual, ClampedGLU, GatedDeltaMixer, GroupLimitedMoE, InputParameters, KVCache,
                     Linear, ParallelMixer, PostNormResidual, ReluSquaredMLP, SigmoidBlockAttention, TokenSideInput)
from .registry import register_model

# constants the design fixes
GLU_SLOPE = 1.702            # an expert's gate is g * sigmoid(1.702 g)
UNIT_EPS = 1e-6              # under the root of the recurrent half's unit queries and keys
ROUTE_WEIGHT_EPS = 1e-20     # added to the sum of the chosen experts' probabilities


def rotary_table(rot: Optional[dict]):
    """(inv_freq [dims / 2] fp32 or None, dims) of a mixer's "rot" entry: f_t = base^(-2 t / dims); with "scaling"
    {factor, low, high, original} a frequency whose wavelength l = 2 pi / f is longer than original / low is divided
    by factor, one shorter than original / high is kept, and in between it is (1 - s) f / factor + s f with
    s = (original / l - low) / (high - low).  Evaluated in float64 and rounded once."""
    if not rot or not int(rot.get("dims", 0)):
        return None, 0
    dims, base = int(rot["dims"]), float(rot["base"])
    t = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * t / dims)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = (float(sc[k]) for k in ("factor", "low", "high", "original"))
        wl = 2.0 * math.pi / f
        s = (orig / wl - low) / (high - low)
        mid = (1.0 - s) * f / factor + s * f
        f = torch.where(wl < orig / high, f, torch.where(wl > orig / low, f / factor, mid))
    return f.to(torch.float32), dims


def _left_sizes(m: dict):
    H, dim = int(m["heads"]), int(m["dim"])
    return H, int(m.get("kv_heads") or H), dim, int(m.get("vdim") or dim)


def tensor_shapes(config: dict, lowrank: int = 0) -> Dict[str, tuple]:
    """Names and shapes of a checkpoint of this config.  The ranks of the decay and gate pairs of the recurrent half
    are a property of the checkpoint (the shapes of a1 / g1), not of the config: `lowrank` is what a generator uses
    (default: a quarter of the key size, at least 4)."""
    W, V = int(config["width"]), int(config["vocab"])
    layers = config["layers"]
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    side = config.get("token_side")
    if side:
        out["side.embed"] = (V, len(layers) * int(side["dim"]))
    for i, L in enumerate(layers):
        p = f"l{i}."
        if L["type"] != "parallel":
            raise ValueError(f"unknown mixer type {L['type']!r}")
        out[p + "norm1"] = (W,)
        out[p + "norm1b"] = (W,)
        H, G, dim, vd = _left_sizes(L["mixer"]["left"])
        a = p + "mix.left."
        out.update({a + "q": (H * dim, W), a + "q.b": (H * dim,), a + "k": (G * dim, W), a + "k.b": (G * dim,),
                    a + "v": (G * vd, W), a + "v.b": (G * vd,), a + "talk": (H, H), a + "pb": (H,),
                    a + "o": (W, H * vd), a + "out": (W,)})
        H, G, dim, vd = _left_sizes(L["mixer"]["right"])
        taps = int(L["mixer"]["right"]["conv"])
        r = lowrank or max(4, dim // 4)
        a = p + "mix.right."
        out.update({a + "q": (G * dim, W), a + "q.conv": (G * dim, taps), a + "k": (G * dim, W),
                    a + "k.conv": (G * dim, taps), a + "v": (H * vd, W), a + "v.conv": (H * vd, taps),
                    a + "b": (H, W), a + "A_log": (H,), a + "norm": (vd,), a + "a1": (r, W), a + "a2": (H * dim, r),
                    a + "dt_bias": (H * dim,), a + "g1": (r, W), a + "g2": (H * vd, r), a + "o": (W, H * vd),
                    a + "out": (W,)})
        mlp = L.get("mlp")
        if mlp is not None:
            out[p + "norm2"] = (W,)
            out[p + "norm2b"] = (W,)
            f = p + "mlp."
            if mlp["kind"] == "dense":
                ff = int(mlp["ff"])
                out.update({f + "up": (ff, W), f + "down": (W, ff)})
            elif mlp["kind"] == "moe":
                ff, E = int(mlp["expert"]["ff"]), int(mlp["router"]["experts"])
                n_out = E + int(mlp["router"].get("identity") or 0)
                out.update({f + "router": (n_out, W), f + "correction": (n_out,)})
                for e in range(E):
                    out.update({f + f"e{e}.gate": (ff, W), f + f"e{e}.up": (ff, W), f + f"e{e}.down": (W, ff)})
                if mlp.get("shared"):
                    sf = int(mlp["shared"]["ff"])
                    out.update({f + "shared.gate": (sf, W), f + "shared.up": (sf, W), f + "shared.down": (W, sf),
                                f + "shared.sg": (1, W)})
            else:
                raise ValueError(f"unknown feed-forward kind {mlp['kind']!r}")
        if side:
            sd = int(side["dim"])
            out.update({p + "side.gate": (sd, W), p + "side.proj": (W, sd), p + "side.norm": (W,)})
    return out


def random_tensors(config: dict, seed: int = 0, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Random weights of the architecture (bench and tests): projections N(0, 1/in), gains around one, small biases,
    decay parameters in the range where the state forgets over tens to hundreds of tokens."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2", "norm1b", "norm2b", "out", "norm") or name == "final.norm":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "talk":
            t = torch.eye(shape[0]) + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "A_log":
            t = torch.log(0.5 + 4.0 * torch.rand(shape, generator=g))
        elif leaf == "dt_bias":
            t = -4.0 + 3.0 * torch.rand(shape, generator=g)
        elif leaf == "conv":
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        elif leaf == "correction":
            t = 0.05 * torch.randn(shape, generator=g)
        elif leaf in ("pb",):
            t = -2.0 + torch.randn(shape, generator=g)
        elif name in ("embed", "side.embed"):
            t = torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = 0.2 * torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = t.to(dtype)
    return out


class _Layer:
    norm1: torch.Tensor                       # input norm of the mixer (fp32 weight)
    mixer: ParallelMixer
    post1: BranchNormResidual
    norm2: Optional[torch.Tensor] = None
    ff = None
    post2: Optional[BranchNormResidual] = None
    side: Optional[TokenSideInput] = None
    cache: Optional[KVCache] = None


@register_model("Fesupel")
class FesupelDecoder:
    needs_state_slots = True
    CSRC = ("postnorm.cu", "hyper.cu", "sigmoid_attn.cu", "delta_rule.cu", "moe.cu")

    def __init__(self, config: dict, dtype: torch.dtype, device, max_seqs: int = 4):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Fesupel runs in bfloat16 or float32")
        _lib.ensure(self.CSRC)
        self.config, self.dtype, self.device, self.max_seqs = config, dtype, torch.device(device), max_seqs
        self.width, self.n_vocab = int(config["width"]), int(config["vocab"])
        self.eps = float(config["norm"]["eps"])
        self.embed_scale = float((config.get("embedding") or {}).get("scale", 1.0))
        self.layers: List[_Layer] = []
        self.embed = self.final_norm = self.head = None

    @classmethod
    def from_config(cls, config: dict, dtype, device, max_seqs: int = 4) -> "FesupelDecoder":
        return cls(config, dtype, device, max_seqs)

    # ------------------------------------------------------------------ weights
    def init_random(self, seed: int = 0) -> None:
        self.load_weights(random_tensors(self.config, seed))

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        dev, dt, eps = self.device, self.dtype, self.eps
        optional = (".q.b", ".k.b", ".v.b", ".talk", ".pb", ".correction")
        missing = [n for n in tensor_shapes(self.config) if n not in tensors and not n.endswith(optional)]
        if missing:
            raise KeyError(f"checkpoint lacks {missing[:5]}{' ...' if len(missing) > 5 else ''}")
        w = lambda name: tensors[name].to(dev).to(dt)
        f32 = lambda name: tensors[name].to(dev).to(torch.float32).contiguous()
        self.embed = w("embed").contiguous()
        self.final_norm = f32("final.norm")
        self.head = Linear(w("head"))
        side_cfg = self.config.get("token_side")
        side_table = w("side.embed").contiguous() if side_cfg else None
        self.layers = []
        for i, L in enumerate(self.config["layers"]):
            p = f"l{i}."
            if L["type"] != "parallel":
                raise ValueError(f"unknown mixer type {L['type']!r}")
            lay = _Layer()
            sub = lambda pre: {k[len(pre):]: w(k) for k in tensors if k.startswith(pre)}
            ml, mr = L["mixer"]["left"], L["mixer"]["right"]
            H, G, dim, vd = _left_sizes(ml)
            inv_freq, rot_dims = rotary_table(ml.get("rot"))
            left = SigmoidBlockAttention(sub(p + "mix.left."), H, G, dim, vd, float(ml["scale"]),
                                         float(ml.get("softcap") or 0.0), int((ml.get("mask") or {}).get("size") or 0),
                                         inv_freq, rot_dims, dt, dev)
            H, G, dim, vd = _left_sizes(mr)
            rw = sub(p + "mix.right.")
            if rw["q.conv"].shape[1] != int(mr["conv"]):
                raise ValueError(f"layer {i}: the filters have {rw['q.conv'].shape[1]} taps, the config says {mr['conv']}")
            right = GatedDeltaMixer(rw, H, G, dim, vd, UNIT_EPS, eps, self.max_seqs, dt, dev)
            lay.mixer = ParallelMixer(left, right)
            lay.norm1 = f32(p + "norm1")
            lay.post1 = BranchNormResidual(f32(p + "norm1b"), eps, f32(p + "mix.left.out"), f32(p + "mix.right.out"))
            mlp = L.get("mlp")
            if mlp is not None:
                f = p + "mlp."
                if mlp["kind"] == "dense":
                    lay.ff = ReluSquaredMLP(w(f + "up"), w(f + "down"))
                elif mlp["kind"] == "moe":
                    r = mlp["router"]
                    E = int(r["experts"])
                    grp = r.get("groups") or {}
                    stack = lambda leaf: torch.stack([w(f"{f}e{e}.{leaf}") for e in range(E)], dim=0)
                    shared = shared_gate = None
                    if mlp.get("shared") and f + "shared.gate" in tensors:
                        shared = ClampedGLU(w(f + "shared.gate"), w(f + "shared.up"), w(f + "shared.down"),
                                            float(mlp["shared"]["limit"]), GLU_SLOPE)
                        shared_gate = tensors[f + "shared.sg"].to(dev)
                    router = tensors[f + "router"].to(dev)
                    if router.shape[0] != E + int(r.get("identity") or 0):
                        raise ValueError(f"layer {i}: the router has {router.shape[0]} outputs, the config says "
                                         f"{E} experts and {r.get('identity') or 0} pass-through ones")
                    lay.ff = GroupLimitedMoE(router, tensors[f + "correction"].to(dev) if f + "correction" in tensors else None,
                                             stack("gate"), stack("up"), stack("down"), int(r["top"]),
                                             int(grp.get("count") or 1), int(grp.get("keep") or grp.get("count") or 1),
                                             float(mlp["expert"]["limit"]), GLU_SLOPE, ROUTE_WEIGHT_EPS, shared,
                                             shared_gate)
                else:
                    raise ValueError(f"unknown feed-forward kind {mlp['kind']!r}")
                lay.norm2 = f32(p + "norm2")
                lay.post2 = BranchNormResidual(f32(p + "norm2b"), eps)
            if side_cfg:
                sd = int(side_cfg["dim"])
                lay.side = TokenSideInput(side_table, i * sd, w(p + "side.gate"), w(p + "side.proj"),
                                          PostNormResidual(f32(p + "side.norm"), 1, 1.0, eps))
            self.layers.append(lay)

    # ------------------------------------------------------------------ cache
    def alloc_cache(self, n_blocks: int, block_size: int) -> None:
        for lay, L in zip(self.layers, self.config["layers"]):
            _, G, dim, vd = _left_sizes(L["mixer"]["left"])
            lay.cache = KVCache(n_blocks, block_size, G, dim, self.dtype, self.device, value_dim=vd)

    # ------------------------------------------------------------------ forward
    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, params: InputParameters,
                last_token_idxes: Optional[torch.Tensor] = None, layer_out: Optional[list] = None) -> torch.Tensor:
        """One step over the packed rows of all sequences; logits [rows or len(last_token_idxes), vocab].
        layer_out, if given, receives the residual after every layer (fp32)."""
        dt, eps, n_layers = self.dtype, self.eps, len(self.layers)
        x, _ = kernels.bigram_embed(self.embed, None, tokens, None, 0, 0, 0, self.embed_scale, want_h=False)
        h = None                      # norm1(x) of the coming layer where the step before could make it
        for i, lay in enumerate(self.layers):
            if h is None:
                h = kernels.group_rms_norm(x, lay.norm1, 1, eps, dt)
            a, b = lay.mixer(h, positions, lay.cache, params)
            nxt = self.layers[i + 1].norm1 if i + 1 < n_layers else None
            # what follows the mixer decides what its residual step hands on: the feed-forward's input norm, the
            # plain rows (the per-token term reads x itself), or the next layer's input norm
            after_mixer = lay.norm2 if lay.ff is not None else (None if lay.side is not None else nxt)
            want = lay.ff is not None or lay.side is not None or nxt is not None
            x, h = lay.post1(x, a, b, next_weight=after_mixer, want_h=want)
            if lay.ff is not None:
                y = lay.ff(h)
                after_ff = None if lay.side is not None else nxt
                x, h = lay.post2(x, y, None, next_weight=after_ff, want_h=lay.side is not None or nxt is not None)
            if lay.side is not None:
                x, _ = lay.side(x, x if dt == torch.float32 else h, tokens)
                h = None
            if layer_out is not None:
                layer_out.append(x.clone())
        if last_token_idxes is not None:
            x = x.index_select(0, last_token_idxes.to(torch.int64))
        return self.head(kernels.group_rms_norm(x, self.final_norm, 1, eps, dt))

    __call__ = forward
