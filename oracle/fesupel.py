"""oracle.fesupel — the Fesupel decoder restated in plain torch on the CPU.  TEST INFRASTRUCTURE.

One function per mechanism, written from the design's equations and sharing nothing with the
product path (`scalellm_b200/`).  Everything runs in one floating-point type (float64 by default)
over an explicit per-sequence state, so the same functions serve whole prompts, portions and
single decoded tokens.

Notation (W = width, unit(x) = x / sqrt(mean(x^2) + eps), norm(x, w) = unit(x) * w):

    x_0         = s_e * embed[tok]
    layer       : x <- x + norm(mixer(norm(x, n1)), n1b) ; x <- x + norm(ff(norm(x, n2)), n2b)   (no ff: skipped) ;
                  x <- x + norm(P (gelu_tanh(G x) * side[tok, layer's slice]), n_s)               (if "token_side")
    mixer       : 1/2 (norm(left(h), w_l) + norm(right(h), w_r))
    left        : q, k, v = affine maps of h; the first rot.dims channels of every q and k head turn (channel t with
                  t + dims/2, angle p f_t, f_t = base^(-2t/dims) rescaled per wavelength band);
                  s_ij = cap tanh(scale q_i . k_j / cap) for the keys j <= i of i's block of `mask.size` positions;
                  a_h(i, j) = sigmoid(s_ij + b_h) (not normalised); a'_h = sum_g T[h, g] a_g ;
                  o_h(i) = sum_j a'_h(i, j) v_{kv(h)}(j) ; result = Wo concat(o)
    right       : q, k, v = silu(conv(W h)) with a causal per-channel filter of `conv` taps; q, k made unit length
                  per head (x / sqrt(sum x^2 + 1e-6)), q scaled by dim^(-1/2); beta = sigmoid(Wb h);
                  d = exp(-exp(A_h) softplus(W2 W1 h + dt)) per head and key channel;
                  S <- diag(d) S ; u = beta (v - S^T k) ; S <- S + k u^T ; o = S^T q  (S [dim, vdim] per head);
                  o <- o / sqrt(mean(o^2) + eps) * w_n * sigmoid(G2 G1 h) ; result = Wo concat(o)
    ff "dense"  : Wd relu(Wu h)^2
    ff "moe"    : p = softmax(R h) over real and pass-through experts; c = p + correction; only the `keep` groups (of
                  `count` equal runs of neighbours) with the largest max c may be chosen; the `top` largest c are
                  chosen; weights p_e / (sum of chosen p + 1e-20); a pass-through expert returns h;
                  expert(h) = Wd (g sigmoid(1.702 g) (u + 1)), g = min(Wg h, L), u = clamp(Wu h, -L, L);
                  plus sigmoid(w_sg . h) * shared expert(h)
    output      : head(norm(x, final))
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .kigalix import read_safetensors  # noqa: F401  (same file format)

UNIT_EPS = 1e-6          # under the root of the unit queries and keys of the recurrent half
GLU_SLOPE = 1.702
WEIGHT_EPS = 1e-20       # added to the sum of the chosen experts' probabilities


def unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit(x, eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------------------------------------ left half
def turn_frequencies(rot: dict) -> List[float]:
    """f_t for t < dims / 2, after the per-band rescaling of "scaling" (if any)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    out = []
    sc = rot.get("scaling")
    for t in range(dims // 2):
        f = base ** (-2.0 * t / dims)
        if sc:
            factor, low, high, orig = (float(sc[k]) for k in ("factor", "low", "high", "original"))
            wl = 2.0 * math.pi / f
            if wl > orig / low:
                f = f / factor
            elif wl >= orig / high:
                s = (orig / wl - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def turn_half(x: torch.Tensor, pos: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x [T, heads, n]: the first rot.dims channels of every head turn, channel t with channel t + dims / 2."""
    if not rot:
        return x
    dims = int(rot["dims"])
    half = dims // 2
    f = torch.tensor(turn_frequencies(rot), dtype=torch.float64)
    ang = pos.to(torch.float64)[:, None] * f[None, :]
    c, s = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def block_visible(i: int, j: int, size: int) -> bool:
    """Key j for query i: causal, and (size > 0) in the same block of `size` positions counted from 0."""
    return j <= i and (size <= 0 or i // size == j // size)


def sigmoid_attend(q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, pos: torch.Tensor, scale: float, cap: float,
                   head_bias: torch.Tensor, talk: Optional[torch.Tensor], size: int) -> torch.Tensor:
    """q [T, H, dim] at positions pos over keys K [n, G, dim] and values V [n, G, vd] of positions 0 .. n - 1."""
    T, H, G = q.shape[0], q.shape[1], K.shape[1]
    out = torch.zeros(T, H, V.shape[2], dtype=q.dtype)
    for t in range(T):
        i = int(pos[t])
        js = [j for j in range(i + 1) if block_visible(i, j, size)]
        a = torch.zeros(H, len(js), dtype=q.dtype)
        for hh in range(H):
            g = hh // (H // G)
            s = (K[js, g] @ q[t, hh]) * scale
            if cap > 0.0:
                s = cap * torch.tanh(s / cap)
            a[hh] = torch.sigmoid(s + head_bias[hh])
        if talk is not None:
            a = talk @ a
        for hh in range(H):
            out[t, hh] = a[hh] @ V[js, hh // (H // G)]
    return out


def left_half(h: torch.Tensor, pos: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, st: dict) -> torch.Tensor:
    H, dim = int(m["heads"]), int(m["dim"])
    G, vd = int(m.get("kv_heads", H)), int(m.get("vdim", dim))
    T = h.shape[0]
    q = (h @ w["q"].T + w["q.b"]).reshape(T, H, dim)
    k = (h @ w["k"].T + w["k.b"]).reshape(T, G, dim)
    v = (h @ w["v"].T + w["v.b"]).reshape(T, G, vd)
    q, k = turn_half(q, pos, m.get("rot")), turn_half(k, pos, m.get("rot"))
    K = torch.cat([st["k"], k]) if "k" in st else k
    V = torch.cat([st["v"], v]) if "v" in st else v
    st["k"], st["v"] = K, V
    size = int((m.get("mask") or {}).get("size") or 0)
    o = sigmoid_attend(q, K, V, pos, float(m["scale"]), float(m.get("softcap") or 0.0), w["pb"], w.get("talk"), size)
    return o.reshape(T, H * vd) @ w["o"].T


# ------------------------------------------------------------------------------------------------ right half
def short_filter(x: torch.Tensor, taps_w: torch.Tensor, st: dict, key: str) -> torch.Tensor:
    """x [T, C], taps_w [C, taps] (last column: the current token).  st[key]: the last taps - 1 inputs."""
    taps = taps_w.shape[1]
    past = st.get(key)
    if past is None:
        past = torch.zeros(taps - 1, x.shape[1], dtype=x.dtype)
    full = torch.cat([past, x])
    y = torch.zeros_like(x)
    for t in range(x.shape[0]):
        y[t] = (full[t: t + taps] * taps_w.T).sum(dim=0)
    st[key] = full[full.shape[0] - (taps - 1):]
    return y


def delta_scan(q, k, v, beta, decay, S):
    """q, k [T, dim], v [T, vd], beta [T], decay [T, dim], S [dim, vd] (updated in place).  Returns o [T, vd]."""
    out = torch.zeros_like(v)
    for t in range(q.shape[0]):
        S.mul_(decay[t][:, None])
        u = beta[t] * (v[t] - S.T @ k[t])
        S.add_(torch.outer(k[t], u))
        out[t] = S.T @ q[t]
    return out


def right_half(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, st: dict) -> torch.Tensor:
    H, dim = int(m["heads"]), int(m["dim"])
    G, vd = int(m.get("kv_heads", H)), int(m.get("vdim", dim))
    T = h.shape[0]
    q = silu(short_filter(h @ w["q"].T, w["q.conv"], st, "cq")).reshape(T, G, dim)
    k = silu(short_filter(h @ w["k"].T, w["k.conv"], st, "ck")).reshape(T, G, dim)
    v = silu(short_filter(h @ w["v"].T, w["v.conv"], st, "cv")).reshape(T, H, vd)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + UNIT_EPS) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + UNIT_EPS)
    beta = torch.sigmoid(h @ w["b"].T)                                            # [T, H]
    dt = torch.nn.functional.softplus((h @ w["a1"].T) @ w["a2"].T + w["dt_bias"]).reshape(T, H, dim)
    decay = torch.exp(-torch.exp(w["A_log"])[None, :, None] * dt)
    gate = torch.sigmoid((h @ w["g1"].T) @ w["g2"].T).reshape(T, H, vd)
    if "S" not in st:
        st["S"] = torch.zeros(H, dim, vd, dtype=h.dtype)
    o = torch.zeros(T, H, vd, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        o[:, hh] = delta_scan(q[:, g], k[:, g], v[:, hh], beta[:, hh], decay[:, hh], st["S"][hh])
    o = unit(o, eps) * w["norm"] * gate
    return o.reshape(T, H * vd) @ w["o"].T


def parallel_mixer(h, pos, w: Dict[str, torch.Tensor], m: dict, eps: float, st: dict) -> torch.Tensor:
    lw = {k[5:]: t for k, t in w.items() if k.startswith("left.")}
    rw = {k[6:]: t for k, t in w.items() if k.startswith("right.")}
    a = left_half(h, pos, lw, m["left"], st.setdefault("left", {}))
    b = right_half(h, rw, m["right"], eps, st.setdefault("right", {}))
    return 0.5 * (norm(a, lw["out"], eps) + norm(b, rw["out"], eps))


# ------------------------------------------------------------------------------------------------ feed-forward
def relu2_ff(h, up, down):
    return torch.relu(h @ up.T) ** 2 @ down.T


def clamped_expert(h, gate, up, down, limit: float):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, -limit, limit)
    return (g * torch.sigmoid(GLU_SLOPE * g) * (u + 1.0)) @ down.T


def route(h, router, correction, r: dict):
    """-> (ids [T, top], weights [T, top]) over real + pass-through experts."""
    p = torch.softmax(h @ router.T, dim=-1)
    c = p + correction if correction is not None else p.clone()
    n = c.shape[1]
    grp = r.get("groups")
    if grp and int(grp["count"]) > 1:
        count, keep = int(grp["count"]), int(grp["keep"])
        best = c.reshape(-1, count, n // count).max(dim=-1).values
        kept = best.topk(keep, dim=-1).indices
        allow = torch.zeros(c.shape[0], count, dtype=torch.bool)
        allow.scatter_(1, kept, True)
        c = torch.where(allow.repeat_interleave(n // count, dim=1), c, torch.full_like(c, -math.inf))
    ids = c.topk(int(r["top"]), dim=-1).indices
    chosen = p.gather(1, ids)
    return ids, chosen / (chosen.sum(dim=-1, keepdim=True) + WEIGHT_EPS)


def moe_ff(h, w: Dict[str, torch.Tensor], mlp: dict):
    r = mlp["router"]
    n_real = int(r["experts"])
    ids, wts = route(h, w["router"], w.get("correction"), r)
    limit = float(mlp["expert"]["limit"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), wts[t]):
            if e >= n_real:
                out[t] += a * h[t]
            else:
                out[t] += a * clamped_expert(h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], limit)
    if "shared.gate" in w:
        sh = clamped_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], float(mlp["shared"]["limit"]))
        out = out + torch.sigmoid(h @ w["shared.sg"].T) * sh
    return out


def side_input(x, tok, table, gate, proj, nw, col0: int, dim: int, eps: float):
    e = table[tok.long(), col0: col0 + dim]
    y = (gelu_tanh(x @ gate.T) * e) @ proj.T
    return x + norm(y, nw, eps)


# ------------------------------------------------------------------------------------------------ model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: torch.Tensor, state: dict,
            layer_out: Optional[list] = None, dtype=torch.float64) -> torch.Tensor:
    """Runs `tokens` (1-D) of ONE sequence on top of `state` ({} at the start); logits [T, vocab]."""
    W = {k: (t.to(dtype) if t.is_floating_point() else t) for k, t in w.items()}
    eps = float(cfg["norm"]["eps"])
    n0 = state.get("n", 0)
    T = tokens.numel()
    pos = torch.arange(n0, n0 + T)
    state["n"] = n0 + T
    x = W["embed"][tokens.long()] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    side = cfg.get("token_side")
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        st = state.setdefault(i, {})
        if L["type"] != "parallel":
            raise ValueError(L["type"])
        mw = {k[len(p) + 4:]: t for k, t in W.items() if k.startswith(p + "mix.")}
        y = parallel_mixer(norm(x, W[p + "norm1"], eps), pos, mw, L["mixer"], eps, st)
        x = x + norm(y, W[p + "norm1b"], eps)
        mlp = L.get("mlp")
        if mlp is not None:
            h = norm(x, W[p + "norm2"], eps)
            fw = {k[len(p) + 4:]: t for k, t in W.items() if k.startswith(p + "mlp.")}
            y = relu2_ff(h, fw["up"], fw["down"]) if mlp["kind"] == "dense" else moe_ff(h, fw, mlp)
            x = x + norm(y, W[p + "norm2b"], eps)
        if side:
            d = int(side["dim"])
            x = side_input(x, tokens, W["side.embed"], W[p + "side.gate"], W[p + "side.proj"], W[p + "side.norm"],
                           i * d, d, eps)
        if layer_out is not None:
            layer_out.append(x.clone())
    return norm(x, W["final.norm"], eps) @ W["head"].T


class Fesupel:
    """The functions above bound to one config and one set of weights."""

    def __init__(self, cfg: dict, weights: Dict[str, torch.Tensor], dtype=torch.float64):
        self.cfg, self.dtype = cfg, dtype
        self.w = {k: (t.to(dtype) if t.is_floating_point() else t) for k, t in weights.items()}

    def new_state(self) -> dict:
        return {}

    def forward(self, tokens, state: dict, layer_out: Optional[list] = None) -> torch.Tensor:
        return forward(self.cfg, self.w, torch.as_tensor(tokens), state, layer_out, self.dtype)
