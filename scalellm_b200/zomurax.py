"""Zomurax: a decoder-only model whose layers are listed in its config.json.

    x          = embed[tok]                                                 (fp32 residual)
    per layer  : x <- norm1(a x + mixer(x)) ; x <- norm2(a x + ff(x)) (unless "mlp" is null), a = "postln_alpha";
                 the sublayers read x itself and the norm FOLLOWS the sum (layers.SumNormResidual); a norm is
                 x / rms(x) times ONE learned number
    mixers     : "attention" (layers.SinkAttention: unit-length queries and keys, query temperature "q_temp",
                 logarithmic distance bias, sink, grouped key/value heads; the layers whose config says "v_mix"
                 blend their values with those of the first such layer),
                 "latent_attention" (layers.LatentAttention with a sliding window "mask.size" and the rotary turn
                 over channel pairs (t, t + dims / 2))
    feed-forward: "moe" (layers.TableMoE: the token id's row of an integer table names its experts, each weighted
                 1 / top, plus a shared expert "shared" for every token)
    output     : the model's norm with "final.norm", the vocabulary projection, then cap * tanh(logits / cap)
                 ("logit_softcap").

Every size and constant is read from config.json or a tensor's shape.  Tensor names: "embed", "head", "final.norm",
and per layer i "l<i>.norm1|norm2", "l<i>.mix.*" (attention: q, k, v, o, r1, r2, sink, vmix; latent attention: q, dkv,
dkv.norm, uk, uv, o), "l<i>.mlp.e<j>.gate|up|down", "l<i>.mlp.table", "l<i>.mlp.shared.gate|up|down".

State per sequence: unit keys and (blended) values of the attention layers in paged KVCache rows, latents and rotary
keys of the latent-attention layers in paged LatentKVCache rows.  Nothing is recurrent: the model takes no state slots.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from . import _lib, kernels
from .layers import (GatedMLP, InputParameters, KVCache, LatentAttention, LatentKVCache, Linear, SinkAttention,
                     SumNormResidual, TableMoE)
from .registry import register_model

# constants the design fixes
EXPERT_ACT = "silu"


def rotary_table(rot: dict) -> torch.Tensor:
    """inv_freq [dims / 2] fp32 of a mixer's "rot" entry: base^(-2 t / dims), evaluated in float64."""
    dims, base = int(rot["dims"]), float(rot["base"])
    t = torch.arange(dims // 2, dtype=torch.float64)
    return torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * t / dims).to(torch.float32)


def tensor_shapes(config: dict) -> Dict[str, tuple]:
    """Names and shapes of a checkpoint of this config."""
    W, V = int(config["width"]), int(config["vocab"])
    out = {"embed": (V, W), "final.norm": (), "head": (V, W)}
    for i, L in enumerate(config["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = ()
        if L["type"] == "attention":
            H, dim = int(m["heads"]), int(m["dim"])
            G, vd = int(m.get("kv_heads", H)), int(m.get("vdim", dim))
            out.update({p + "mix.q": (H * dim, W), p + "mix.k": (G * dim, W), p + "mix.v": (G * vd, W),
                        p + "mix.o": (W, H * vd), p + "mix.r1": (H,), p + "mix.r2": (H,), p + "mix.sink": (H,)})
            if m.get("v_mix"):
                out[p + "mix.vmix"] = ()
        elif L["type"] == "latent_attention":
            H, dim, rd, vd, rank = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
            out.update({p + "mix.q": (H * (dim + rd), W), p + "mix.dkv": (rank + rd, W), p + "mix.dkv.norm": (rank,),
                        p + "mix.uk": (H * dim, rank), p + "mix.uv": (H * vd, rank), p + "mix.o": (W, H * vd)})
        else:
            raise ValueError(f"unknown mixer type {L['type']!r}")
        mlp = L.get("mlp")
        if mlp is None:
            continue
        if mlp["kind"] != "moe":
            raise ValueError(f"unknown feed-forward kind {mlp['kind']!r}")
        ff, E, top = int(mlp["expert"]["ff"]), int(mlp["router"]["experts"]), int(mlp["router"]["top"])
        out[p + "norm2"] = ()
        out[p + "mlp.table"] = (V, top)
        for e in range(E):
            out.update({p + f"mlp.e{e}.gate": (ff, W), p + f"mlp.e{e}.up": (ff, W), p + f"mlp.e{e}.down": (W, ff)})
        if mlp.get("shared"):
            sf = int(mlp["shared"]["ff"])
            out.update({p + "mlp.shared.gate": (sf, W), p + "mlp.shared.up": (sf, W), p + "mlp.shared.down": (W, sf)})
    return out


def random_tensors(config: dict, seed: int = 0, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Random weights of the architecture (bench and tests): projections N(0, 1/in), small vectors, tables of
    distinct experts per row."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if leaf == "table":
            E = int(config["layers"][int(name.split(".")[0][1:])]["mlp"]["router"]["experts"])
            out[name] = torch.stack([torch.randperm(E, generator=g)[: shape[1]] for _ in range(shape[0])]).to(torch.int32)
            continue
        if leaf in ("norm1", "norm2") or name == "final.norm":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "norm":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "vmix":
            t = torch.rand(shape, generator=g)
        elif leaf in ("r1", "r2"):
            t = 0.05 + 0.5 * torch.rand(shape, generator=g)
        elif leaf == "sink":
            t = torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        out[name] = t.to(dtype)
    return out


class _Layer:
    kind: str = ""
    mixer = None
    norm1: SumNormResidual
    ff: Optional[TableMoE] = None
    norm2: Optional[SumNormResidual] = None
    cache = None                      # KVCache (attention) or LatentKVCache (latent attention)
    shares_values: bool = False       # an attention layer of the value-sharing set


@register_model("Zomurax")
class ZomuraxDecoder:
    needs_state_slots = False
    CSRC = ("postnorm.cu", "hyper.cu", "latent_attn.cu", "sink_attn.cu", "moe.cu")

    def __init__(self, config: dict, dtype: torch.dtype, device, max_seqs: int = 4):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Zomurax runs in bfloat16 or float32")
        _lib.ensure(self.CSRC)
        self.config, self.dtype, self.device, self.max_seqs = config, dtype, torch.device(device), max_seqs
        self.width, self.n_vocab = int(config["width"]), int(config["vocab"])
        self.eps = float(config["norm"]["eps"])
        self.alpha = float(config.get("postln_alpha", 1.0))
        cap = config.get("logit_softcap")
        self.softcap = float(cap) if cap else 0.0
        self.layers: List[_Layer] = []
        self.embed = self.final_norm = self.head = None

    @classmethod
    def from_config(cls, config: dict, dtype, device, max_seqs: int = 4) -> "ZomuraxDecoder":
        return cls(config, dtype, device, max_seqs)

    # ------------------------------------------------------------------ weights
    def init_random(self, seed: int = 0) -> None:
        self.load_weights(random_tensors(self.config, seed))

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        dev, dt, eps, W = self.device, self.dtype, self.eps, self.width
        optional = (".r1", ".r2", ".sink", ".vmix")      # (the first value-sharing layer has no use for its ".vmix")
        missing = [n for n in tensor_shapes(self.config) if n not in tensors and not n.endswith(optional)]
        if missing:
            raise KeyError(f"checkpoint lacks {missing[:5]}{' ...' if len(missing) > 5 else ''}")
        w = lambda name: tensors[name].to(dev).to(dt)
        f32 = lambda name: tensors[name].to(dev).to(torch.float32).contiguous()
        self.embed = w("embed").contiguous()
        self.final_norm = f32("final.norm").reshape(1).expand(W).contiguous()    # one number, per channel for the kernel
        self.head = Linear(w("head"))
        self.layers = []
        sharing_seen = False
        for i, L in enumerate(self.config["layers"]):
            p, m = f"l{i}.", L["mixer"]
            lay = _Layer()
            lay.kind = L["type"]
            mw = {k[len(p) + 4:]: (w(k) if tensors[k].is_floating_point() else tensors[k].to(dev))
                  for k in tensors if k.startswith(p + "mix.")}
            if L["type"] == "attention":
                qt = m.get("q_temp") or {}
                lay.shares_values = bool(m.get("v_mix"))
                lam = None
                if lay.shares_values and sharing_seen:      # the first sharing layer gives, the later ones blend
                    lam = float(tensors[p + "mix.vmix"].float())
                sharing_seen = sharing_seen or lay.shares_values
                lay.mixer = SinkAttention(mw, int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]),
                                          int(m.get("vdim", m["dim"])),
                                          float(m["scale"]), float(qt.get("coef", 0.0)), int(qt.get("every", 0)), lam,
                                          eps, dt, dev)
            elif L["type"] == "latent_attention":
                rot = m.get("rot") or {"dims": 0, "base": 1.0}
                mask = m.get("mask") or {}
                lay.mixer = LatentAttention(mw, int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]),
                                            int(m["kv_rank"]), float(m["scale"]), rotary_table(rot), 1.0,
                                            int(rot["dims"]), eps, dt, dev, window=int(mask.get("size") or 0),
                                            half_pairs=True, fusable_out=True)
            else:
                raise ValueError(f"unknown mixer type {L['type']!r}")
            lay.norm1 = SumNormResidual(f32(p + "norm1"), self.alpha, eps)
            mlp = L.get("mlp")
            if mlp is not None:
                if mlp["kind"] != "moe":
                    raise ValueError(f"unknown feed-forward kind {mlp['kind']!r}")
                f = p + "mlp."
                E = int(mlp["router"]["experts"])
                stack = lambda leaf: torch.stack([w(f"{f}e{e}.{leaf}") for e in range(E)], dim=0)
                shared = None
                if f + "shared.gate" in tensors:
                    shared = GatedMLP(w(f + "shared.gate"), w(f + "shared.up"), w(f + "shared.down"), EXPERT_ACT)
                table = tensors[f + "table"].to(dev)
                if table.shape[1] != int(mlp["router"]["top"]):
                    raise ValueError(f"layer {i}: the expert table has {table.shape[1]} columns, top is {mlp['router']['top']}")
                lay.ff = TableMoE(table, stack("gate"), stack("up"), stack("down"), EXPERT_ACT, shared)
                lay.norm2 = SumNormResidual(f32(p + "norm2"), self.alpha, eps)
            self.layers.append(lay)

    # ------------------------------------------------------------------ cache
    def alloc_cache(self, n_blocks: int, block_size: int) -> None:
        for lay, L in zip(self.layers, self.config["layers"]):
            m = L["mixer"]
            if L["type"] == "attention":
                lay.cache = KVCache(n_blocks, block_size, int(m.get("kv_heads", m["heads"])), int(m["dim"]), self.dtype,
                                    self.device, value_dim=int(m.get("vdim", m["dim"])))
            else:
                lay.cache = LatentKVCache(n_blocks, block_size, int(m["kv_rank"]), int(m["rot_dim"]), self.dtype,
                                          self.device)

    # ------------------------------------------------------------------ forward
    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, params: InputParameters,
                last_token_idxes: Optional[torch.Tensor] = None, layer_out: Optional[list] = None) -> torch.Tensor:
        """One step over the packed rows of all sequences; logits [rows or len(last_token_idxes), vocab].
        layer_out, if given, receives the residual after every layer (fp32)."""
        x, h = kernels.bigram_embed(self.embed, None, tokens, None, 0, 0, 0, 1.0)
        h = x if h is None else h
        first_values = None           # the first value-sharing layer's values of this step's rows
        for lay in self.layers:
            if lay.kind == "attention":
                y, v_own = lay.mixer(h, positions, lay.cache, params, first_values if lay.shares_values else None)
                if lay.shares_values and first_values is None:
                    first_values = v_own
            else:
                y = lay.mixer(h, positions, lay.cache, params)
            x, h = lay.norm1(x, y, self.dtype)
            if lay.ff is not None:
                x, h = lay.norm2(x, lay.ff(h, tokens), self.dtype)
            if layer_out is not None:
                layer_out.append(x.clone())
        if last_token_idxes is not None:
            x = x.index_select(0, last_token_idxes.to(torch.int64))
        logits = self.head(kernels.group_rms_norm(x, self.final_norm, 1, self.eps, self.dtype))
        if self.softcap > 0.0:
            logits = kernels.softcap_(logits.contiguous(), self.softcap)
        return logits

    __call__ = forward
