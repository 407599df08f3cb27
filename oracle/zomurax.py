"""oracle.zomurax — the Zomurax decoder restated in plain torch on the CPU.  TEST INFRASTRUCTURE.

One function per mechanism, written from the design's equations and sharing nothing with the
product path (`scalellm_b200/`).  Everything runs in one floating-point type (float64 by default)
over an explicit per-sequence state, so the same functions serve whole prompts, portions and
single decoded tokens.

Notation (W = width, a = "postln_alpha"):

    unit(x)     = x / sqrt(mean(x^2) + eps)
    layer       : x <- unit(a x + mixer(x)) * g1 ; x <- unit(a x + ff(x)) * g2      g1, g2 one number each
    attention   : q, k unit-normalised per head; q *= 1 + c ln(floor((p + 1) / n) + 1) at position p;
                  s_ij = scale q_i . k_j - r1 ln(1 + r2 (i - j)),  j <= i;
                  weights = exp(s_ij) / (exp(sink) + sum_j exp(s_ij));
                  layers that share values: v <- (1 - lam) v + lam v(first such layer, same token)
    latent      : c = unit(D h [:rank]) * w_c ; kr = turn(D h [rank:]) ; k_h = [Uk_h c | kr] ; v_h = Uv_h c ;
                  q_h = [.. | turn(..)] ; softmax over the keys j with 0 <= i - j < window
    turn        : channel t pairs with t + dims / 2; angle p * base^(-2 t / dims)
    ff          : sum over the token id's experts (a table row) of expert(h) / top, plus a shared expert
    output      : cap * tanh(head(unit(x) * g) / cap)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .kigalix import read_safetensors  # noqa: F401  (same file format)


def unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def scalar_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    return unit(x, eps) * g.reshape(())


def turn_half(x: torch.Tensor, pos: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, ..., n]: the first rot.dims channels turn, channel t with channel t + dims / 2."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * t / dims) for t in range(half)], dtype=torch.float64)
    ang = pos.to(torch.float64)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).to(x.dtype).reshape(shape), torch.sin(ang).to(x.dtype).reshape(shape)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def query_temperature(pos: torch.Tensor, q_temp: Optional[dict]) -> torch.Tensor:
    if not q_temp:
        return torch.ones(pos.shape[0], dtype=torch.float64)
    steps = torch.div(pos + 1, int(q_temp["every"]), rounding_mode="floor").to(torch.float64)
    return 1.0 + float(q_temp["coef"]) * torch.log(steps + 1.0)


def sink_attend(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, pos: torch.Tensor, scale: float,
                r1: Optional[torch.Tensor], r2: Optional[torch.Tensor], sink: Optional[torch.Tensor]) -> torch.Tensor:
    """q [T, H, dim] at positions pos over the keys K [n, G, dim] and values V [n, G, vd] of positions 0 .. n - 1."""
    T, H, G = q.shape[0], q.shape[1], K.shape[1]
    out = torch.zeros(T, H, V.shape[2], dtype=q.dtype)
    for t in range(T):
        i = int(pos[t])
        dist = torch.arange(i, -1, -1, dtype=q.dtype)          # i - j for j = 0 .. i
        for hh in range(H):
            g = hh // (H // G)
            s = (K[: i + 1, g] @ q[t, hh]) * scale
            if r1 is not None:
                s = s - r1[hh] * torch.log(1.0 + r2[hh] * dist)
            mx = s.max()
            e = torch.exp(s - mx)
            den = e.sum()
            if sink is not None:
                den = den + torch.exp(sink[hh] - mx)
            out[t, hh] = (e / den) @ V[: i + 1, g]
    return out


def sink_attention(h: torch.Tensor, pos: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, st: dict,
                   shared_v: dict, first_of_shared: bool) -> torch.Tensor:
    """st: this layer's cached keys and values of the sequence; shared_v: where the first value-sharing layer leaves
    its values of the step's tokens for the later ones."""
    H, G, dim, vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = unit((h @ w["q"].T).reshape(T, H, dim), eps)
    k = unit((h @ w["k"].T).reshape(T, G, dim), eps)
    v = (h @ w["v"].T).reshape(T, G, vd)
    q = q * query_temperature(pos, m.get("q_temp")).to(h.dtype)[:, None, None]
    if m.get("v_mix"):
        if first_of_shared:
            shared_v["v"] = v
        else:
            lam = w["vmix"].reshape(())
            v = (1.0 - lam) * v + lam * shared_v["v"]
    K = torch.cat([st["k"], k]) if "k" in st else k
    V = torch.cat([st["v"], v]) if "v" in st else v
    st["k"], st["v"] = K, V
    out = sink_attend(q, K, V, pos, float(m["scale"]), w.get("r1"), w.get("r2"), w.get("sink"))
    return out.reshape(T, H * vd) @ w["o"].T


def window_visible(i: int, j: int, window: int) -> bool:
    return j <= i and (window <= 0 or i - j < window)


def latent_attend(q: torch.Tensor, C: torch.Tensor, KR: torch.Tensor, uk: torch.Tensor, uv: torch.Tensor,
                  pos: torch.Tensor, scale: float, window: int) -> torch.Tensor:
    """q [T, H, dim + rd] (turned) over latents C [n, rank] and turned shared key parts KR [n, rd];
    uk [H, dim, rank], uv [H, vd, rank]."""
    T, H = q.shape[0], q.shape[1]
    out = torch.zeros(T, H, uv.shape[1], dtype=q.dtype)
    for t in range(T):
        i = int(pos[t])
        js = [j for j in range(i + 1) if window_visible(i, j, window)]
        cj, krj = C[js], KR[js]
        for hh in range(H):
            kk = torch.cat([cj @ uk[hh].T, krj], dim=-1)           # [keys, dim + rd]
            p = torch.softmax((kk @ q[t, hh]) * scale, dim=0)
            out[t, hh] = p @ (cj @ uv[hh].T)
    return out


def latent_window_attention(h: torch.Tensor, pos: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float,
                            st: dict) -> torch.Tensor:
    H, dim, rd, vd, rank = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
    T = h.shape[0]
    q = (h @ w["q"].T).reshape(T, H, dim + rd)
    q = torch.cat([q[..., :dim], turn_half(q[..., dim:], pos, m["rot"])], dim=-1)
    d = h @ w["dkv"].T
    c = unit(d[:, :rank], eps) * w["dkv.norm"]
    kr = turn_half(d[:, rank:], pos, m["rot"])
    C = torch.cat([st["c"], c]) if "c" in st else c
    KR = torch.cat([st["kr"], kr]) if "kr" in st else kr
    st["c"], st["kr"] = C, KR
    window = int((m.get("mask") or {}).get("size", 0))
    out = latent_attend(q, C, KR, w["uk"].reshape(H, dim, rank), w["uv"].reshape(H, vd, rank), pos, float(m["scale"]),
                        window)
    return out.reshape(T, H * vd) @ w["o"].T


def expert(h: torch.Tensor, w: Dict[str, torch.Tensor], pre: str) -> torch.Tensor:
    return (silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def table_moe(h: torch.Tensor, tokens: List[int], w: Dict[str, torch.Tensor], mlp: dict) -> torch.Tensor:
    top = int(mlp["router"]["top"])
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=h.dtype)
    for t, tok in enumerate(tokens):
        for e in w["table"][tok].tolist():
            out[t] += expert(h[t: t + 1], w, f"e{int(e)}.")[0] / top
    if "shared.gate" in w:
        out = out + expert(h, w, "shared.")
    return out


class Zomurax:
    def __init__(self, config: dict, tensors: Dict[str, torch.Tensor], dtype=torch.float64):
        self.cfg, self.dtype = config, dtype
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
        self.eps = float(config["norm"]["eps"])
        self.alpha = float(config.get("postln_alpha", 1.0))
        shared = [i for i, L in enumerate(config["layers"]) if L["type"] == "attention" and L["mixer"].get("v_mix")]
        self.first_shared = shared[0] if shared else -1

    def sub(self, prefix: str) -> Dict[str, torch.Tensor]:
        n = len(prefix)
        return {k[n:]: v for k, v in self.w.items() if k.startswith(prefix)}

    def new_state(self) -> dict:
        return {"layers": [dict() for _ in self.cfg["layers"]], "n": 0}

    def forward(self, tokens: List[int], state: dict, layer_out: Optional[list] = None) -> torch.Tensor:
        """Runs the next tokens of one sequence; returns logits [T, vocab]."""
        w, eps, a = self.w, self.eps, self.alpha
        T = len(tokens)
        pos = torch.arange(state["n"], state["n"] + T)
        state["n"] += T
        x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
        shared_v: dict = {}
        for i, L in enumerate(self.cfg["layers"]):
            st, p = state["layers"][i], f"l{i}."
            mw = self.sub(p + "mix.")
            if L["type"] == "attention":
                y = sink_attention(x, pos, mw, L["mixer"], eps, st, shared_v, i == self.first_shared)
            elif L["type"] == "latent_attention":
                y = latent_window_attention(x, pos, mw, L["mixer"], eps, st)
            else:
                raise ValueError(L["type"])
            x = scalar_norm(a * x + y, w[p + "norm1"], eps)
            if L.get("mlp") is not None:
                x = scalar_norm(a * x + table_moe(x, tokens, self.sub(p + "mlp."), L["mlp"]), w[p + "norm2"], eps)
            if layer_out is not None:
                layer_out.append(x)
        logits = scalar_norm(x, w["final.norm"], eps) @ w["head"].T
        cap = self.cfg.get("logit_softcap")
        return float(cap) * torch.tanh(logits / float(cap)) if cap else logits
