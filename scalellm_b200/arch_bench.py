"""Prefill and decode throughput of the Kigalix, Pokadra, Zomurax and Fesupel designs beside the Llama decoder (Zomurax
and Fesupel also beside Kigalix, the design nearest to them) at equal size (`bench.py --arch
kigalix|pokadra|zomurax|fesupel`), all through the serving engine, random weights, bf16.

Per size: tokens/s of a prompt step (B sequences of L tokens in one batch) and of decode steps (B sequences
with L cached tokens, one token each), timed with CUDA events after warm-up; and, per kind of kernel, the
device time per step (events around every call of the kernel wrappers) with its algorithmic bytes and FLOPs
against the measured copy bandwidth and bf16 GEMM throughput.  Weights and caches are larger than L2 at the
larger size; the smaller one says so in its line.
"""
from __future__ import annotations

import json
import os
import time
from typing import Callable, Dict, List

import torch

SIZES = {
    # width, layers, attention heads x (dim + rot), latent rank, value size, delta heads x dim, dense ff, experts
    "w2048": dict(width=2048, layers=4, heads=16, dim=128, rot=64, vdim=128, rank=512, dheads=32, ddim=64,
                  ff=5632, experts=8, top=2, eff=1408, vocab=32000),
    "w4096": dict(width=4096, layers=4, heads=32, dim=128, rot=64, vdim=128, rank=512, dheads=64, ddim=64,
                  ff=11008, experts=8, top=2, eff=2752, vocab=32000),
}


def kigalix_config(s: dict) -> dict:
    rot = {"base": 10000.0, "dims": s["rot"]}
    yarn = dict(rot, scaling={"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0})
    scale = (s["dim"] + s["rot"]) ** -0.5
    la = lambda kind, r: {"type": kind, "mixer": {"heads": s["heads"], "dim": s["dim"], "rot_dim": s["rot"],
                                                   "vdim": s["vdim"], "kv_rank": s["rank"], "rot": r, "scale": scale}}
    dl = {"type": "general_delta", "mixer": {"heads": s["dheads"], "dim": s["ddim"]}}
    moe = {"kind": "moe", "expert": {"ff": s["eff"]}, "router": {"experts": s["experts"], "top": s["top"]}}
    pattern = [dict(la("latent_attention_2", yarn), mlp={"kind": "dense", "ff": s["ff"]}), dict(dl, mlp=moe),
               dict(la("latent_attention", rot), mlp=moe), dict(la("latent_attention", rot), mlp=moe)]
    return {"architecture": "Kigalix", "width": s["width"], "vocab": s["vocab"], "streams": 2,
            "norm": {"eps": 1e-5}, "layers": [pattern[i % 4] for i in range(s["layers"])]}


def llama_config(s: dict) -> dict:
    return {"architectures": ["LlamaForCausalLM"], "hidden_size": s["width"], "num_hidden_layers": s["layers"],
            "num_attention_heads": s["width"] // 128, "num_key_value_heads": max(1, s["width"] // 512),
            "intermediate_size": s["ff"], "vocab_size": s["vocab"], "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
            "max_position_embeddings": 8192, "rope_scaling": None}


class KernelTimer:
    """Wraps functions of a module so that every call is bracketed by CUDA events on the current stream."""

    def __init__(self):
        self.events: Dict[str, List] = {}
        self._undo: List = []

    def wrap(self, owner, names: List[str], label: Callable[[str], str] = lambda n: n) -> None:
        for n in names:
            fn = getattr(owner, n)

            def timed(*a, __fn=fn, __l=label(n), **k):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                out = __fn(*a, **k)
                e1.record()
                self.events.setdefault(__l, []).append((e0, e1))
                return out
            self._undo.append((owner, n, fn))
            setattr(owner, n, timed)

    def restore(self) -> None:
        for owner, n, fn in self._undo:
            setattr(owner, n, fn)
        self._undo = []

    def totals_ms(self) -> Dict[str, float]:
        torch.cuda.synchronize()
        out = {k: sum(a.elapsed_time(b) for a, b in v) for k, v in self.events.items()}
        self.events = {}
        return out


def _time_steps(fn: Callable[[], None], warmup: int, steps: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def _run_model(config: dict, batch: int, seqlen: int, warmup: int, steps: int, kernel_names, seed: int = 0):
    from . import kernels, registry
    from .engine import Engine, StepEntry
    dev = torch.device("cuda", torch.cuda.current_device())
    model = registry.create_model(config, torch.bfloat16, dev, max_seqs=batch)
    model.init_random(seed)
    bs = 16
    eng = Engine(model, max_tokens=batch * (seqlen + 64 + bs), block_size=bs, max_seqs=batch,
                 max_step_tokens=batch * seqlen, use_graphs=True)
    g = torch.Generator().manual_seed(seed)
    V = config.get("vocab", config.get("vocab_size"))
    prompts = [[int(x) for x in torch.randint(0, V, (seqlen,), generator=g)] for _ in range(batch)]
    res = {}

    def prefill():
        eng.step([StepEntry(f"s{i}", p, [len(p) - 1]) for i, p in enumerate(prompts)])

    def reset():
        for rid in list(eng.seqs):
            eng.finish(rid)

    # prompt steps: every timed step admits the batch afresh (blocks and slots are reused)
    def prefill_once():
        reset()
        prefill()
    ms = _time_steps(prefill_once, min(warmup, 2), max(2, min(steps, 5)))
    res["prefill"] = {"ms_per_step": ms, "tokens_per_s": batch * seqlen / ms * 1e3}
    reset()
    prefill()

    def decode():
        eng.step([StepEntry(f"s{i}", [7], [0]) for i in range(batch)])
    ms = _time_steps(decode, warmup, min(steps, 48))
    res["decode"] = {"ms_per_step": ms, "tokens_per_s": batch / ms * 1e3}
    # per-kernel device time of one prompt step and one decode step
    timer = KernelTimer()
    timer.wrap(kernels, kernel_names)
    timer.wrap(kernels, ["dense_gemm", "dense_gemm_splitk"], lambda n: "linear (dense GEMMs)")
    timer.wrap(torch.nn.functional, ["linear"], lambda n: "linear (dense GEMMs)")
    timer.wrap(torch, ["bmm"], lambda n: "bmm (per-head key / value maps)")
    try:
        eng.use_graphs = False          # per-kernel times come from eager steps; the first of each kind is
        decode()                        # discarded: it pays for allocations the caching allocator then keeps
        timer.totals_ms()
        decode()
        res["decode"]["kernels_ms"] = timer.totals_ms()
        prefill_once()
        timer.totals_ms()
        prefill_once()
        res["prefill"]["kernels_ms"] = timer.totals_ms()
    finally:
        timer.restore()
    reset()
    del eng, model
    torch.cuda.empty_cache()
    return res


KIGALIX_KERNELS = ["embed_streams", "hc_norm", "token_shift", "gated_hc_update", "gated_act", "heads_to_rows",
                   "latent_prepare", "latent_attn", "delta_rule", "moe_route", "moe_plan", "grouped_gemm", "moe_combine"]
LLAMA_KERNELS = ["rms_norm", "rms_norm_residual", "rope_and_set_kv_cache", "paged_kv_varlen_mha", "silu_mul",
                 "silu_with_mul", "apply_rotary_pos_emb", "set_kv_cache", "rms_norm_residual_splitk", "silu_mul_splitk",
                 "rope_and_set_kv_cache_splitk"]


def rooflines(s: dict, batch: int, seqlen: int, k: dict, l: dict, peaks: dict) -> dict:
    """Achieved fraction of the nearer roof (copy bandwidth or bf16 GEMM rate) for the attention kernels of
    both models and the expert GEMMs, from the per-kernel times of one step."""
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    n_lat = sum(1 for i in range(s["layers"]) if i % 4 != 1)
    n_moe = sum(1 for i in range(s["layers"]) if i % 4 != 0)
    Dk, out = s["rank"] + s["rot"], {}

    def frac(ms, nbytes, flops):
        t = ms * 1e-3
        if t <= 0:
            return None
        return {"ms": ms, "of_copy_peak": nbytes / t / hbm, "of_gemm_peak": flops / t / tf,
                "roof_ms": max(nbytes / hbm, flops / tf) * 1e3, "of_roof": max(nbytes / hbm, flops / tf) / t}
    for phase, keys in (("decode", batch * (seqlen + 1)), ("prefill", batch * seqlen * (seqlen + 1) // 2)):
        rows = batch if phase == "decode" else batch * seqlen
        cached = batch * (seqlen + (1 if phase == "decode" else 0))
        ms = k[phase]["kernels_ms"].get("latent_attn", 0.0)
        out[f"kigalix latent_attn {phase}"] = frac(ms, n_lat * (cached * Dk * 2 + rows * s["heads"] * (Dk + s["rank"]) * 4),
                                                  n_lat * keys * s["heads"] * 2 * (Dk + s["rank"]))
        H, Hkv = s["width"] // 128, max(1, s["width"] // 512)
        ms = l[phase]["kernels_ms"].get("paged_kv_varlen_mha", 0.0)
        out[f"llama paged attention {phase}"] = frac(ms, s["layers"] * (cached * 2 * Hkv * 128 * 2 + rows * H * 128 * 4),
                                                     s["layers"] * keys * H * 4 * 128)
        pairs = rows * s["top"]
        ms = k[phase]["kernels_ms"].get("grouped_gemm", 0.0)
        out[f"kigalix expert GEMMs {phase}"] = frac(ms, n_moe * (s["experts"] * 3 * s["eff"] * s["width"] * 2
                                                              + pairs * (s["width"] * 2 + 3 * s["eff"]) * 2),
                                                   n_moe * pairs * 6 * s["eff"] * s["width"])
        ms = l[phase]["kernels_ms"].get("linear (dense GEMMs)", 0.0)
        wbytes = s["layers"] * (s["width"] * (s["width"] + 2 * max(1, s["width"] // 512) * 128) + s["width"] * s["width"]
                                + 3 * s["ff"] * s["width"]) * 2
        nlog = batch
        out[f"llama dense GEMMs {phase}"] = frac(ms, wbytes + s["vocab"] * s["width"] * 2,
                                                 (wbytes // 2) * 2 * rows + nlog * 2 * s["vocab"] * s["width"])
        ms = k[phase]["kernels_ms"].get("delta_rule", 0.0)
        n_d = s["layers"] - n_lat
        dn = s["dheads"] * s["ddim"]
        out[f"kigalix delta_rule {phase}"] = frac(ms, n_d * (rows * 7 * dn * 2 + batch * 2 * dn * s["ddim"] * 4),
                                                  n_d * rows * s["dheads"] * 6 * s["ddim"] ** 2)
    return out


def attention_kernels(s: dict, peaks: dict, cases=((64, 4096, 1), (4, 2048, 2048))) -> dict:
    """The two designs' attention kernels alone, on caches larger than L2: (batch, cached length, new tokens per
    sequence) = decoding over long contexts and one prompt portion.  CUDA events around 10 launches after 3."""
    from . import kernels
    from .decode_step import BlockPool, StepBuffers, build_step_batch
    dev = torch.device("cuda", torch.cuda.current_device())
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    H, dim, rd, rank = s["heads"], s["dim"], s["rot"], s["rank"]
    Hl, Hkv, D, bs = s["width"] // 128, max(1, s["width"] // 512), 128, 16
    out = {}
    for batch, ctx, q_len in cases:
        n_blocks = batch * (-(-ctx // bs)) + 8
        pool = BlockPool(n_blocks, bs, seed=1)
        seqs = []
        for _ in range(batch):
            sq = pool.open_sequence()
            pool.reserve(sq, ctx)
            seqs.append(sq)
        hb = build_step_batch(pool, seqs, [[0] * q_len] * batch, [ctx - q_len] * batch, list(range(batch)))
        tokens, positions, prm = StepBuffers(dev, batch * q_len, batch, n_blocks).upload(hb)
        rows = batch * q_len
        keys = batch * (q_len * (ctx - q_len) + q_len * (q_len + 1) // 2)      # visible (query, key) pairs
        g = torch.Generator(device=dev).manual_seed(0)
        rnd = lambda *shape: torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        cache = rnd(n_blocks * bs, rank + rd)
        qa, q = rnd(H, rows, rank), rnd(rows, H * (dim + rd))
        f_lat = lambda: kernels.latent_attn(qa, q, cache, prm.q_cu_seq_lens, prm.kv_cu_seq_lens, prm.block_tables,
                                            prm.cu_block_lens, prm.token_seq, H, dim, rd, rank, bs, 0.07, ctx)
        kc, vc = rnd(n_blocks * bs, Hkv, D), rnd(n_blocks * bs, Hkv, D)
        ql, ol = rnd(rows, Hl, D), torch.empty((rows, Hl, D), dtype=torch.bfloat16, device=dev)
        f_llama = lambda: kernels.paged_kv_varlen_mha(ol, ql, kc, vc, prm.q_cu_seq_lens, prm.kv_cu_seq_lens,
                                                      prm.block_tables, prm.cu_block_lens, None, bs, q_len, ctx,
                                                      D ** -0.5, 0.0, -1)
        for name, fn, nbytes, flops in (
                ("kigalix latent_attn", f_lat, batch * ctx * (rank + rd) * 2 + rows * H * (2 * rank + rd) * 2,
                 keys * H * 2 * (2 * rank + rd)),
                ("llama paged attention", f_llama, batch * ctx * 2 * Hkv * D * 2 + rows * Hl * D * 4, keys * Hl * 4 * D)):
            ms = _time_steps(fn, 3, 10)
            roof = max(nbytes / hbm, flops / tf) * 1e3
            out[f"{name}, {batch} x {ctx} cached, {q_len} new"] = {
                "ms": ms, "GB": nbytes / 1e9, "TFLOP": flops / 1e12, "of_copy_peak": nbytes / (ms * 1e-3) / hbm,
                "of_gemm_peak": flops / (ms * 1e-3) / tf, "roof_ms": roof, "of_roof": roof / ms}
        del cache, kc, vc
        torch.cuda.empty_cache()
    return out


def run(args) -> None:
    torch.cuda.set_device(0)
    torch.backends.cuda.matmul.allow_tf32 = False
    peaks_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    peaks = json.load(open(peaks_path)) if os.path.exists(peaks_path) else {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    out = {"metric": "kigalix_vs_llama_tokens_per_s", "unit": "tokens/s", "dtype": "bf16",
           "data": "synthetic (random-init weights, random token ids)", "n_gpus": 1,
           "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"],
                     "source": "measured" if os.path.exists(peaks_path) else "fallback"}, "sizes": {}}
    names = [args.arch_size] if args.arch_size != "all" else list(SIZES)
    for name in names:
        s = SIZES[name]
        batch, seqlen = args.arch_batch, args.arch_seqlen
        t0 = time.time()
        k = _run_model(kigalix_config(s), batch, seqlen, args.warmup, args.steps, KIGALIX_KERNELS)
        l = _run_model(llama_config(s), batch, seqlen, args.warmup, args.steps, LLAMA_KERNELS)
        out["sizes"][name] = {"shape": s, "batch": batch, "seq_len": seqlen, "kigalix": k, "llama": l,
                              "kernel_rooflines": rooflines(s, batch, seqlen, k, l, peaks),
                              "attention_kernels": attention_kernels(s, peaks),
                              "seconds": round(time.time() - t0, 1)}
    print(json.dumps(out))


# ---------------------------------------------------------------------------
# Pokadra beside Llama
# ---------------------------------------------------------------------------
POKADRA_SIZES = {
    # width, layers (mingru, attention, mingru, attention over layer 1's keys), heads x 2 maps x dim, value size,
    # key/value heads, window + kept tokens, recurrence width, dense ff, per-token side width
    "w2048": dict(width=2048, layers=4, heads=16, kv_heads=4, dim=64, vdim=128, window=512, keep=4, gru=2560,
                  ff=5632, side=64, buckets=100003, vocab=32000),
    "w4096": dict(width=4096, layers=4, heads=32, kv_heads=8, dim=64, vdim=128, window=512, keep=4, gru=5120,
                  ff=11008, side=64, buckets=100003, vocab=32000),
}
POKADRA_KERNELS = ["bigram_embed", "postnorm_residual", "postnorm_residual_splitk", "group_rms_norm", "glu_clamped",
                   "glu_clamped_splitk", "token_gated_gelu", "token_side_postnorm", "mingru_scan", "diff_attn_prepare",
                   "diff_attn"]


def pokadra_config(s: dict) -> dict:
    at = lambda src: {"type": "attention", "mixer": dict(
        {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"], "diff": 0.5,
         "scale": s["dim"] ** -0.5, "mask": {"size": s["window"], "keep_first": s["keep"]},
         "rot": {"base": 10000.0, "dims": s["dim"] // 2,
                 "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}},
        **({"kv_from": src} if src is not None else {}))}
    gru = {"type": "mingru", "mixer": {"width": s["gru"]}}
    mlp = {"kind": "dense", "ff": s["ff"], "limit": 7.0}
    pattern = [gru, at(None), gru, at(1)]
    layers = []
    for i in range(s["layers"]):
        L = dict(pattern[i % 4], mlp=mlp)
        if i % 4 == 3:      # the sharing layer reads the cache of the attention layer two places before it
            L = dict(at(i - 2), mlp=mlp)
        layers.append(L)
    return {"architecture": "Pokadra", "width": s["width"], "vocab": s["vocab"], "norm": {"eps": 1e-5, "groups": 4},
            "residual_mult": 0.5, "token_side": {"dim": s["side"]},
            "embedding": {"scale": 2.0, "bigram": {"buckets": s["buckets"], "mul_prev": 1000003, "mul_cur": 31}},
            "layers": layers}


def _visible_pairs(ctx: int, q_len: int, window: int, keep: int) -> int:
    """(query, key) pairs of one sequence with ctx tokens in all whose last q_len are the step's rows."""
    n = 0
    for i in range(ctx - q_len, ctx):
        lo = max(0, i - window + 1) if window else 0
        n += min(keep, lo) + (i - lo + 1)
    return n


def _frac(ms, nbytes, flops, hbm, tf):
    t = ms * 1e-3
    if t <= 0:
        return None
    roof = max(nbytes / hbm, flops / tf)
    return {"ms": ms, "GB": nbytes / 1e9, "TFLOP": flops / 1e12, "of_copy_peak": nbytes / t / hbm,
            "of_gemm_peak": flops / t / tf, "roof_ms": roof * 1e3, "of_roof": roof / t}


def pokadra_rooflines(s: dict, batch: int, seqlen: int, k: dict, l: dict, peaks: dict) -> dict:
    """Achieved fraction of the nearer roof per kind of kernel, from the per-kernel times of one step of each
    model (all layers of that kind together)."""
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    n_at = sum(1 for i in range(s["layers"]) if i % 2 == 1)
    n_gru = s["layers"] - n_at
    H, G, dim, vd, W = s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["width"]
    out = {}
    for phase in ("decode", "prefill"):
        q_len = 1 if phase == "decode" else seqlen
        ctx = seqlen + 1 if phase == "decode" else seqlen
        rows = batch * q_len
        pairs = batch * _visible_pairs(ctx, q_len, s["window"], s["keep"])
        touched = batch * (min(ctx, s["window"] + s["keep"]) if phase == "decode" else ctx)
        km, lm = k[phase]["kernels_ms"], l[phase]["kernels_ms"]
        out[f"pokadra diff_attn {phase}"] = _frac(
            km.get("diff_attn", 0.0), n_at * (touched * G * (2 * dim + vd) * 2 + rows * H * (2 * dim * 4 + vd * 2)),
            n_at * pairs * H * 4 * (dim + vd), hbm, tf)
        Hl, Hkv = W // 128, max(1, W // 512)
        lpairs = batch * _visible_pairs(ctx, q_len, 0, 0)
        out[f"llama paged attention {phase}"] = _frac(
            lm.get("paged_kv_varlen_mha", 0.0), s["layers"] * (batch * ctx * 2 * Hkv * 128 * 2 + rows * Hl * 128 * 4),
            s["layers"] * lpairs * Hl * 4 * 128, hbm, tf)
        out[f"pokadra mingru_scan {phase}"] = _frac(km.get("mingru_scan", 0.0), n_gru * rows * s["gru"] * 4 * 2, 0, hbm, tf)
        n_post = s["layers"] * 3
        out[f"pokadra postnorm_residual {phase}"] = _frac(
            km.get("postnorm_residual", 0.0),
            rows * W * (n_post * (4 + 4 + 2 + 2) + sum(4 * (i + 2) for i in range(s["layers"]))), 0, hbm, tf)
        out[f"llama rms_norm_residual {phase}"] = _frac(
            lm.get("rms_norm_residual", 0.0) + lm.get("rms_norm", 0.0) + lm.get("rms_norm_residual_splitk", 0.0), rows * W * (2 * s["layers"] + 1) * 4 * 2, 0, hbm, tf)
        pw = (n_gru * 4 * s["gru"] * W + n_at * ((2 * H * dim + H * vd + H) * W) + (G * (2 * dim + vd)) * W * (n_at + 1) // 2
              + s["layers"] * (3 * s["ff"] * W + 2 * s["side"] * W))
        nlog = batch
        out[f"pokadra dense GEMMs {phase}"] = _frac(km.get("linear (dense GEMMs)", 0.0), (pw + s["vocab"] * W) * 2,
                                                   2 * pw * rows + nlog * 2 * s["vocab"] * W, hbm, tf)
        lw = s["layers"] * (W * (W + 2 * Hkv * 128) + W * W + 3 * s["ff"] * W)
        out[f"llama dense GEMMs {phase}"] = _frac(lm.get("linear (dense GEMMs)", 0.0), (lw + s["vocab"] * W) * 2,
                                                 2 * lw * rows + nlog * 2 * s["vocab"] * W, hbm, tf)
    return out


def pokadra_attention_kernels(s: dict, peaks: dict, cases=((64, 4096, 1), (4, 2048, 2048))) -> dict:
    """The differential attention kernel and the Llama paged attention alone, on caches larger than L2: (batch,
    cached length, new tokens per sequence) = decoding over long contexts and one prompt portion.  CUDA events
    around 10 launches after 3."""
    from . import kernels
    from .decode_step import BlockPool, StepBuffers, build_step_batch
    dev = torch.device("cuda", torch.cuda.current_device())
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    H, G, dim, vd, win, keep = s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["window"], s["keep"]
    Hl, Hkv, D, bs = s["width"] // 128, max(1, s["width"] // 512), 128, 16
    out = {}
    for batch, ctx, q_len in cases:
        n_blocks = batch * (-(-ctx // bs)) + 8
        pool = BlockPool(n_blocks, bs, seed=1)
        seqs = []
        for _ in range(batch):
            sq = pool.open_sequence()
            pool.reserve(sq, ctx)
            seqs.append(sq)
        hb = build_step_batch(pool, seqs, [[0] * q_len] * batch, [ctx - q_len] * batch, list(range(batch)))
        tokens, positions, prm = StepBuffers(dev, batch * q_len, batch, n_blocks).upload(hb)
        rows = batch * q_len
        g = torch.Generator(device=dev).manual_seed(0)
        rnd = lambda *shape: torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        kc, vc = rnd(n_blocks * bs, G, 2 * dim), rnd(n_blocks * bs, G, vd)
        q = torch.randn((rows, H, 2, dim), generator=g, device=dev, dtype=torch.float32)
        gate = rnd(rows, H)
        f_diff = lambda: kernels.diff_attn(q, kc, vc, gate, prm.q_cu_seq_lens, prm.kv_cu_seq_lens, prm.block_tables,
                                           prm.cu_block_lens, prm.token_seq, bs, dim ** -0.5, win, keep, 0.4, 0.5, 1e-5,
                                           batch, q_len, ctx)
        kl, vl = rnd(n_blocks * bs, Hkv, D), rnd(n_blocks * bs, Hkv, D)
        ql, ol = rnd(rows, Hl, D), torch.empty((rows, Hl, D), dtype=torch.bfloat16, device=dev)
        f_llama = lambda: kernels.paged_kv_varlen_mha(ol, ql, kl, vl, prm.q_cu_seq_lens, prm.kv_cu_seq_lens,
                                                      prm.block_tables, prm.cu_block_lens, None, bs, q_len, ctx,
                                                      D ** -0.5, 0.0, -1)
        pairs = batch * _visible_pairs(ctx, q_len, win, keep)
        touched = batch * (min(ctx, win + keep) if q_len == 1 else ctx)
        lpairs = batch * _visible_pairs(ctx, q_len, 0, 0)
        for name, fn, nbytes, flops in (
                ("pokadra diff_attn", f_diff, touched * G * (2 * dim + vd) * 2 + rows * H * (2 * dim * 4 + vd * 2),
                 pairs * H * 4 * (dim + vd)),
                ("llama paged attention", f_llama, batch * ctx * 2 * Hkv * D * 2 + rows * Hl * D * 4, lpairs * Hl * 4 * D)):
            ms = _time_steps(fn, 3, 10)
            out[f"{name}, {batch} x {ctx} cached, {q_len} new"] = _frac(ms, nbytes, flops, hbm, tf)
        del kc, vc, kl, vl
        torch.cuda.empty_cache()
    return out


def run_pokadra(args) -> None:
    torch.cuda.set_device(0)
    torch.backends.cuda.matmul.allow_tf32 = False
    peaks_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    peaks = json.load(open(peaks_path)) if os.path.exists(peaks_path) else {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    out = {"metric": "pokadra_vs_llama_tokens_per_s", "unit": "tokens/s", "dtype": "bf16",
           "data": "synthetic (random-init weights, random token ids)", "n_gpus": 1,
           "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"],
                     "source": "measured" if os.path.exists(peaks_path) else "fallback"}, "sizes": {}}
    names = [args.arch_size] if args.arch_size != "all" else list(POKADRA_SIZES)
    for name in names:
        s = POKADRA_SIZES[name]
        batch, seqlen = args.arch_batch, args.arch_seqlen
        t0 = time.time()
        k = _run_model(pokadra_config(s), batch, seqlen, args.warmup, args.steps, POKADRA_KERNELS)
        l = _run_model(llama_config(s), batch, seqlen, args.warmup, args.steps, LLAMA_KERNELS)
        out["sizes"][name] = {"shape": s, "batch": batch, "seq_len": seqlen, "pokadra": k, "llama": l,
                              "kernel_rooflines": pokadra_rooflines(s, batch, seqlen, k, l, peaks),
                              "attention_kernels": pokadra_attention_kernels(s, peaks),
                              "seconds": round(time.time() - t0, 1)}
    print(json.dumps(out))


# ---------------------------------------------------------------------------
# Zomurax beside Kigalix (latent attention, experts) and Llama (grouped-head attention, dense products)
# ---------------------------------------------------------------------------
ZOMURAX_EXTRA = {"w2048": dict(kv_heads=4, window=512, shared=1408, temp_every=1024),
                 "w4096": dict(kv_heads=8, window=512, shared=2752, temp_every=1024)}
ZOMURAX_KERNELS = ["bigram_embed", "sumnorm_residual", "group_rms_norm", "softcap_", "gated_act", "heads_to_rows",
                   "latent_prepare", "latent_attn", "sink_attn_prepare", "sink_attn", "moe_table_route", "moe_plan",
                   "grouped_gemm", "moe_combine"]


def zomurax_config(s: dict) -> dict:
    """Layers in the order latent, latent, attention, attention (the attention layers share values)."""
    lat = {"type": "latent_attention", "mixer": {
        "heads": s["heads"], "dim": s["dim"], "rot_dim": s["rot"], "vdim": s["vdim"], "kv_rank": s["rank"],
        "rot": {"base": 10000.0, "dims": s["rot"]}, "mask": {"size": s["window"]}, "scale": (s["dim"] + s["rot"]) ** -0.5}}
    att = {"type": "attention", "mixer": {
        "heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"], "scale": s["dim"] ** -0.5,
        "q_temp": {"coef": 0.1, "every": s["temp_every"]}, "v_mix": True}}
    moe = {"kind": "moe", "expert": {"ff": s["eff"]}, "router": {"experts": s["experts"], "top": s["top"]},
           "shared": {"ff": s["shared"]}}
    pattern = [lat, lat, att, att]
    return {"architecture": "Zomurax", "width": s["width"], "vocab": s["vocab"], "norm": {"eps": 1e-5},
            "postln_alpha": 2.0, "logit_softcap": 30.0,
            "layers": [dict(pattern[i % 4], mlp=moe) for i in range(s["layers"])]}


def zomurax_rooflines(s: dict, batch: int, seqlen: int, z: dict, k: dict, l: dict, peaks: dict) -> dict:
    """Achieved fraction of the nearer roof per kind of kernel, from the per-kernel times of one step of each model
    (all layers of that kind together), each beside the like kernel of the nearest existing model."""
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    n_lat = sum(1 for i in range(s["layers"]) if i % 4 < 2)
    n_att = s["layers"] - n_lat
    k_lat = sum(1 for i in range(s["layers"]) if i % 4 != 1)
    k_moe = sum(1 for i in range(s["layers"]) if i % 4 != 0)
    H, G, dim, vd, W, Dk = s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["width"], s["rank"] + s["rot"]
    out = {}
    for phase in ("decode", "prefill"):
        q_len = 1 if phase == "decode" else seqlen
        ctx = seqlen + 1 if phase == "decode" else seqlen
        rows = batch * q_len
        zm, km, lm = z[phase]["kernels_ms"], k[phase]["kernels_ms"], l[phase]["kernels_ms"]
        pairs = batch * _visible_pairs(ctx, q_len, 0, 0)
        wpairs = batch * _visible_pairs(ctx, q_len, s["window"], 0)
        touched = batch * (min(ctx, s["window"]) if phase == "decode" else ctx)
        out[f"zomurax sink_attn {phase}"] = _frac(
            zm.get("sink_attn", 0.0), n_att * (batch * ctx * G * (dim + vd) * 2 + rows * H * (dim * 4 + vd * 2)),
            n_att * pairs * H * 2 * (dim + vd), hbm, tf)
        Hl, Hkv = W // 128, max(1, W // 512)
        out[f"llama paged attention {phase}"] = _frac(
            lm.get("paged_kv_varlen_mha", 0.0), s["layers"] * (batch * ctx * 2 * Hkv * 128 * 2 + rows * Hl * 128 * 4),
            s["layers"] * pairs * Hl * 4 * 128, hbm, tf)
        out[f"zomurax latent_attn (window {s['window']}) {phase}"] = _frac(
            zm.get("latent_attn", 0.0), n_lat * (touched * Dk * 2 + rows * H * (Dk + s["rank"]) * 4),
            n_lat * wpairs * H * 2 * (Dk + s["rank"]), hbm, tf)
        out[f"kigalix latent_attn {phase}"] = _frac(
            km.get("latent_attn", 0.0), k_lat * (batch * ctx * Dk * 2 + rows * H * (Dk + s["rank"]) * 4),
            k_lat * pairs * H * 2 * (Dk + s["rank"]), hbm, tf)
        npairs = rows * s["top"]
        ebytes = s["experts"] * 3 * s["eff"] * W * 2 + npairs * (W * 2 + 3 * s["eff"]) * 2
        out[f"zomurax expert GEMMs {phase}"] = _frac(zm.get("grouped_gemm", 0.0), s["layers"] * ebytes,
                                                    s["layers"] * npairs * 6 * s["eff"] * W, hbm, tf)
        out[f"kigalix expert GEMMs {phase}"] = _frac(km.get("grouped_gemm", 0.0), k_moe * ebytes,
                                                    k_moe * npairs * 6 * s["eff"] * W, hbm, tf)
        # norm after the sum: reads x (4) and y (2), writes x (4) and its 16-bit copy (2) per channel, twice a layer
        out[f"zomurax sumnorm_residual {phase}"] = _frac(zm.get("sumnorm_residual", 0.0), rows * W * 2 * s["layers"] * 12,
                                                        0, hbm, tf)
        out[f"llama rms_norm_residual {phase}"] = _frac(
            lm.get("rms_norm_residual", 0.0) + lm.get("rms_norm", 0.0) + lm.get("rms_norm_residual_splitk", 0.0),
            rows * W * (2 * s["layers"] + 1) * 4 * 2, 0, hbm, tf)
        out[f"zomurax sink_attn_prepare {phase}"] = _frac(
            zm.get("sink_attn_prepare", 0.0), n_att * rows * ((H + G) * dim * 2 + G * vd * 4 + H * dim * 4 + G * (dim + vd) * 2),
            0, hbm, tf)
        out[f"zomurax latent_prepare {phase}"] = _frac(
            zm.get("latent_prepare", 0.0), n_lat * rows * (H * s["rot"] * 4 + 2 * Dk * 2), 0, hbm, tf)
        out[f"kigalix latent_prepare {phase}"] = _frac(
            km.get("latent_prepare", 0.0), k_lat * rows * (H * s["rot"] * 4 + 2 * Dk * 2), 0, hbm, tf)
    return out


def zomurax_attention_kernels(s: dict, peaks: dict, cases=((64, 4096, 1), (4, 2048, 2048))) -> dict:
    """The two attention kernels of the design alone beside their like kernels (Llama's paged attention with the same
    heads; latent attention without a window), on caches larger than L2: (batch, cached length, new tokens per
    sequence) = decoding over long contexts and one prompt portion.  CUDA events around 10 launches after 3."""
    from . import kernels
    from .decode_step import BlockPool, StepBuffers, build_step_batch
    dev = torch.device("cuda", torch.cuda.current_device())
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    H, G, dim, vd, rd, rank, win = s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["rot"], s["rank"], s["window"]
    bs, out = 16, {}
    for batch, ctx, q_len in cases:
        n_blocks = batch * (-(-ctx // bs)) + 8
        pool = BlockPool(n_blocks, bs, seed=1)
        seqs = []
        for _ in range(batch):
            sq = pool.open_sequence()
            pool.reserve(sq, ctx)
            seqs.append(sq)
        hb = build_step_batch(pool, seqs, [[0] * q_len] * batch, [ctx - q_len] * batch, None)
        tokens, positions, prm = StepBuffers(dev, batch * q_len, batch, n_blocks).upload(hb)
        rows = batch * q_len
        g = torch.Generator(device=dev).manual_seed(0)
        rnd = lambda *shape: torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        kc, vc = rnd(n_blocks * bs, G, dim), rnd(n_blocks * bs, G, vd)
        q = torch.randn((rows, H, dim), generator=g, device=dev, dtype=torch.float32)
        r1 = 0.1 + 0.3 * torch.rand(H, generator=g, device=dev)
        r2 = 0.05 + 0.3 * torch.rand(H, generator=g, device=dev)
        sk = torch.randn(H, generator=g, device=dev)
        f_sink = lambda: kernels.sink_attn(q, kc, vc, r1, r2, sk, prm.q_cu_seq_lens, prm.kv_cu_seq_lens, prm.block_tables,
                                           prm.cu_block_lens, prm.token_seq, bs, dim ** -0.5, batch, q_len, ctx)
        f_plain = lambda: kernels.sink_attn(q, kc, vc, None, None, None, prm.q_cu_seq_lens, prm.kv_cu_seq_lens,
                                            prm.block_tables, prm.cu_block_lens, prm.token_seq, bs, dim ** -0.5, batch,
                                            q_len, ctx)
        kl, vl = rnd(n_blocks * bs, G, dim), rnd(n_blocks * bs, G, dim)
        ql, ol = rnd(rows, H, dim), torch.empty((rows, H, dim), dtype=torch.bfloat16, device=dev)
        f_llama = lambda: kernels.paged_kv_varlen_mha(ol, ql, kl, vl, prm.q_cu_seq_lens, prm.kv_cu_seq_lens,
                                                      prm.block_tables, prm.cu_block_lens, None, bs, q_len, ctx,
                                                      dim ** -0.5, 0.0, -1)
        cache = rnd(n_blocks * bs, rank + rd)
        qa, qq = rnd(H, rows, rank), rnd(rows, H * (dim + rd))
        f_lat = lambda w: (lambda: kernels.latent_attn(qa, qq, cache, prm.q_cu_seq_lens, prm.kv_cu_seq_lens,
                                                       prm.block_tables, prm.cu_block_lens, prm.token_seq, H, dim, rd,
                                                       rank, bs, 0.07, ctx, w))
        pairs = batch * _visible_pairs(ctx, q_len, 0, 0)
        wpairs = batch * _visible_pairs(ctx, q_len, win, 0)
        touched = batch * (min(ctx, win) if q_len == 1 else ctx)
        a_bytes = batch * ctx * G * (dim + vd) * 2 + rows * H * (dim * 4 + vd * 2)
        for name, fn, nbytes, flops in (
                ("zomurax sink_attn", f_sink, a_bytes, pairs * H * 2 * (dim + vd)),
                ("zomurax sink_attn without bias and sink", f_plain, a_bytes, pairs * H * 2 * (dim + vd)),
                ("llama paged attention, same heads", f_llama, batch * ctx * 2 * G * dim * 2 + rows * H * dim * 4,
                 pairs * H * 4 * dim),
                (f"zomurax latent_attn, window {win}", f_lat(win), touched * (rank + rd) * 2 + rows * H * (2 * rank + rd) * 2,
                 wpairs * H * 2 * (2 * rank + rd)),
                ("kigalix latent_attn (no window)", f_lat(0), batch * ctx * (rank + rd) * 2 + rows * H * (2 * rank + rd) * 2,
                 pairs * H * 2 * (2 * rank + rd))):
            ms = _time_steps(fn, 3, 10)
            out[f"{name}, {batch} x {ctx} cached, {q_len} new"] = _frac(ms, nbytes, flops, hbm, tf)
        del kc, vc, kl, vl, cache
        torch.cuda.empty_cache()
    return out


def run_zomurax(args) -> None:
    torch.cuda.set_device(0)
    torch.backends.cuda.matmul.allow_tf32 = False
    peaks_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    peaks = json.load(open(peaks_path)) if os.path.exists(peaks_path) else {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    out = {"metric": "zomurax_vs_kigalix_vs_llama_tokens_per_s", "unit": "tokens/s", "dtype": "bf16",
           "data": "synthetic (random-init weights, random token ids)", "n_gpus": 1,
           "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"],
                     "source": "measured" if os.path.exists(peaks_path) else "fallback"}, "sizes": {}}
    names = [args.arch_size] if args.arch_size != "all" else list(SIZES)
    for name in names:
        s = dict(SIZES[name], **ZOMURAX_EXTRA[name])
        batch, seqlen = args.arch_batch, args.arch_seqlen
        t0 = time.time()
        z = _run_model(zomurax_config(s), batch, seqlen, args.warmup, args.steps, ZOMURAX_KERNELS)
        k = _run_model(kigalix_config(s), batch, seqlen, args.warmup, args.steps, KIGALIX_KERNELS)
        l = _run_model(llama_config(s), batch, seqlen, args.warmup, args.steps, LLAMA_KERNELS)
        out["sizes"][name] = {"shape": s, "batch": batch, "seq_len": seqlen, "zomurax": z, "kigalix": k, "llama": l,
                              "kernel_rooflines": zomurax_rooflines(s, batch, seqlen, z, k, l, peaks),
                              "attention_kernels": zomurax_attention_kernels(s, peaks),
                              "seconds": round(time.time() - t0, 1)}
    print(json.dumps(out))


# ---------------------------------------------------------------------------
# Fesupel beside Kigalix (a delta-rule layer, attention layers, routed experts) and Llama
# ---------------------------------------------------------------------------
FESUPEL_EXTRA = {"w2048": dict(kv_heads=4, block=512, rheads=16, rkv=8, rdim=128, rvdim=128, taps=4, shared=1408,
                               identity=2, side=64),
                 "w4096": dict(kv_heads=8, block=512, rheads=32, rkv=16, rdim=128, rvdim=128, taps=4, shared=2752,
                               identity=2, side=64)}
FESUPEL_KERNELS = ["bigram_embed", "group_rms_norm", "branch_norm_residual", "sigmoid_attn_prepare", "sigmoid_attn",
                   "gated_delta_prepare", "gated_delta_scan", "relu_squared", "glu_clamped", "glu_clamped_splitk",
                   "moe_route_softmax", "moe_plan", "grouped_gemm", "moe_combine_weighted", "token_side_postnorm",
                   "token_gated_gelu", "postnorm_residual"]


def fesupel_config(s: dict) -> dict:
    """Every layer runs both mixers; the first feed-forward is dense, the others are routed."""
    left = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["vdim"],
            "mask": {"size": s["block"]}, "scale": s["dim"] ** -0.5, "softcap": 30.0,
            "rot": {"base": 10000.0, "dims": s["rot"],
                    "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 4096}}}
    right = {"heads": s["rheads"], "kv_heads": s["rkv"], "dim": s["rdim"], "vdim": s["rvdim"], "conv": s["taps"]}
    moe = {"kind": "moe", "expert": {"ff": s["eff"], "limit": 7.0},
           "router": {"experts": s["experts"], "top": s["top"], "identity": s["identity"],
                      "groups": {"count": 2, "keep": 1}},
           "shared": {"ff": s["shared"], "limit": 7.0}}
    dense = {"kind": "dense", "ff": s["ff"]}
    return {"architecture": "Fesupel", "width": s["width"], "vocab": s["vocab"], "norm": {"eps": 1e-5},
            "embedding": {"scale": s["width"] ** 0.5}, "token_side": {"dim": s["side"]},
            "layers": [{"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": dense if i == 0 else moe}
                       for i in range(s["layers"])]}


def _block_pairs(ctx: int, q_len: int, block: int) -> int:
    """(query, key) pairs of one sequence with ctx tokens whose last q_len are the step's rows, keys limited to the
    row's block of `block` positions."""
    return sum(i % block + 1 if block else i + 1 for i in range(ctx - q_len, ctx))


def fesupel_rooflines(s: dict, batch: int, seqlen: int, f: dict, k: dict, l: dict, peaks: dict) -> dict:
    """Achieved fraction of the nearer roof per kind of kernel, from the per-kernel times of one step of each model
    (all layers of that kind together), each beside the like kernel of the nearest existing model."""
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    L, W = s["layers"], s["width"]
    H, G, dim, vd, blk = s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["block"]
    RH, RG, rd, rv = s["rheads"], s["rkv"], s["rdim"], s["rvdim"]
    k_lat = sum(1 for i in range(L) if i % 4 != 1)
    k_moe = sum(1 for i in range(L) if i % 4 != 0)
    Dk = s["rank"] + s["rot"]
    out = {}
    for phase in ("decode", "prefill"):
        q_len = 1 if phase == "decode" else seqlen
        ctx = seqlen + 1 if phase == "decode" else seqlen
        rows = batch * q_len
        fm, km, lm = f[phase]["kernels_ms"], k[phase]["kernels_ms"], l[phase]["kernels_ms"]
        bpairs = batch * _block_pairs(ctx, q_len, blk)
        pairs = batch * _visible_pairs(ctx, q_len, 0, 0)
        touched = batch * (min(ctx, (ctx - 1) % blk + 1) if phase == "decode" else ctx)
        out[f"fesupel sigmoid_attn (blocks of {blk}) {phase}"] = _frac(
            fm.get("sigmoid_attn", 0.0), L * (touched * G * (dim + vd) * 2 + rows * H * (dim * 4 + vd * 2)),
            L * bpairs * H * 2 * (dim + vd), hbm, tf)
        out[f"kigalix latent_attn {phase}"] = _frac(
            km.get("latent_attn", 0.0), k_lat * (batch * ctx * Dk * 2 + rows * s["heads"] * (Dk + s["rank"]) * 4),
            k_lat * pairs * s["heads"] * 2 * (Dk + s["rank"]), hbm, tf)
        Hl, Hkv = W // 128, max(1, W // 512)
        out[f"llama paged attention {phase}"] = _frac(
            lm.get("paged_kv_varlen_mha", 0.0), L * (batch * ctx * 2 * Hkv * 128 * 2 + rows * Hl * 128 * 4),
            L * pairs * Hl * 4 * 128, hbm, tf)
        # the scan reads q, k, decay (fp32), v (fp32), the gate (16 bits) and writes 16 bits per value channel; the
        # matrices go in and out once per sequence
        out[f"fesupel gated_delta_scan {phase}"] = _frac(
            fm.get("gated_delta_scan", 0.0),
            L * (rows * (2 * RG * rd * 4 + RH * rd * 4 + RH * rv * 8) + batch * 2 * RH * rd * rv * 4),
            L * rows * RH * 6 * rd * rv, hbm, tf)
        n_d, dn = L - k_lat, s["dheads"] * s["ddim"]
        out[f"kigalix delta_rule {phase}"] = _frac(
            km.get("delta_rule", 0.0), n_d * (rows * 7 * dn * 2 + batch * 2 * dn * s["ddim"] * 4),
            n_d * rows * s["dheads"] * 6 * s["ddim"] ** 2, hbm, tf)
        nch = 2 * RG * rd + RH * rv
        out[f"fesupel gated_delta_prepare {phase}"] = _frac(
            fm.get("gated_delta_prepare", 0.0), L * rows * (nch * 2 + RH * rd * 2 + nch * 4 + RH * rd * 4), 0, hbm, tf)
        out[f"fesupel sigmoid_attn_prepare {phase}"] = _frac(
            fm.get("sigmoid_attn_prepare", 0.0), L * rows * ((H + G) * dim * 2 + G * vd * 2 + H * dim * 4 + G * (dim + vd) * 2),
            0, hbm, tf)
        out[f"kigalix latent_prepare {phase}"] = _frac(
            km.get("latent_prepare", 0.0), k_lat * rows * (s["heads"] * s["rot"] * 4 + 2 * Dk * 2), 0, hbm, tf)
        npairs = rows * s["top"]
        ebytes = s["experts"] * 3 * s["eff"] * W * 2 + npairs * (W * 2 + 3 * s["eff"]) * 2
        out[f"fesupel expert GEMMs {phase}"] = _frac(fm.get("grouped_gemm", 0.0), (L - 1) * ebytes,
                                                    (L - 1) * npairs * 6 * s["eff"] * W, hbm, tf)
        out[f"kigalix expert GEMMs {phase}"] = _frac(km.get("grouped_gemm", 0.0), k_moe * ebytes,
                                                    k_moe * npairs * 6 * s["eff"] * W, hbm, tf)
        # branch norms: the mixer's launch reads x (4) and two results (2 + 2), writes x (4) and 16 bits; the
        # feed-forward's reads x and one result
        out[f"fesupel branch_norm_residual {phase}"] = _frac(fm.get("branch_norm_residual", 0.0),
                                                            rows * W * L * (14 + 12), 0, hbm, tf)
        out[f"llama rms_norm_residual {phase}"] = _frac(
            lm.get("rms_norm_residual", 0.0) + lm.get("rms_norm", 0.0) + lm.get("rms_norm_residual_splitk", 0.0),
            rows * W * (2 * L + 1) * 4 * 2, 0, hbm, tf)
    return out


def fesupel_kernels_alone(s: dict, peaks: dict, cases=((64, 4096, 1), (4, 2048, 2048))) -> dict:
    """The design's attention and recurrence kernels alone beside their like kernels (Llama's paged attention with the
    same heads; Kigalix's delta rule with the same state size), on caches larger than L2: (batch, cached length, new
    tokens per sequence) = decoding over long contexts and one prompt portion.  CUDA events around 10 launches after
    3."""
    from . import kernels
    from .decode_step import BlockPool, StepBuffers, build_step_batch
    dev = torch.device("cuda", torch.cuda.current_device())
    hbm, tf = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12
    H, G, dim, vd, blk = s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["block"]
    RH, RG, rd, rv = s["rheads"], s["rkv"], s["rdim"], s["rvdim"]
    bs, out = 16, {}
    for batch, ctx, q_len in cases:
        n_blocks = batch * (-(-ctx // bs)) + 8
        pool = BlockPool(n_blocks, bs, seed=1)
        seqs = []
        for _ in range(batch):
            sq = pool.open_sequence()
            pool.reserve(sq, ctx)
            seqs.append(sq)
        hb = build_step_batch(pool, seqs, [[0] * q_len] * batch, [ctx - q_len] * batch, list(range(batch)))
        tokens, positions, prm = StepBuffers(dev, batch * q_len, batch, n_blocks).upload(hb)
        rows = batch * q_len
        g = torch.Generator(device=dev).manual_seed(0)
        rnd = lambda *shape: torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        r32 = lambda *shape: torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
        kc, vc = rnd(n_blocks * bs, G, dim), rnd(n_blocks * bs, G, vd)
        q = r32(rows, H, dim)
        hbias, mix = r32(H) - 3.0, torch.eye(H, device=dev) + 0.1 * r32(H, H)
        f_sig = lambda size: (lambda: kernels.sigmoid_attn(q, kc, vc, hbias, mix, prm.q_cu_seq_lens, prm.kv_cu_seq_lens,
                                                           prm.block_tables, prm.cu_block_lens, prm.token_seq, bs,
                                                           dim ** -0.5, 30.0, size, q_len, batch, ctx))
        kl, vl = rnd(n_blocks * bs, G, dim), rnd(n_blocks * bs, G, dim)
        ql, ol = rnd(rows, H, dim), torch.empty((rows, H, dim), dtype=torch.bfloat16, device=dev)
        f_llama = lambda: kernels.paged_kv_varlen_mha(ol, ql, kl, vl, prm.q_cu_seq_lens, prm.kv_cu_seq_lens,
                                                      prm.block_tables, prm.cu_block_lens, None, bs, q_len, ctx,
                                                      dim ** -0.5, 0.0, -1)
        pairs = batch * _visible_pairs(ctx, q_len, 0, 0)
        bpairs = batch * _block_pairs(ctx, q_len, blk)
        touched = batch * ((ctx - 1) % blk + 1 if q_len == 1 else ctx)
        qb = rows * H * (dim * 4 + vd * 2)
        # the recurrence: S [rd x rv] per head in and out once per sequence, the rows' inputs once
        dq, dk = torch.nn.functional.normalize(r32(rows, RG, rd), dim=-1), torch.nn.functional.normalize(r32(rows, RG, rd), dim=-1)
        dv, dd, db = r32(rows, RH, rv), torch.sigmoid(r32(rows, RH, rd) + 3.0), torch.sigmoid(r32(rows, RH))
        dg, dn = rnd(rows, RH * rv), torch.ones(rv, device=dev)
        st = torch.zeros((batch, RH, rd, rv), dtype=torch.float32, device=dev)
        f_gd = lambda: kernels.gated_delta_scan(dq, dk, dv, dd, db, dg, dn, st, prm.q_cu_seq_lens, positions,
                                                prm.state_slots, 1e-5, q_len)
        n = RH * rd
        proj = rnd(rows, 5 * n)
        wl = rnd(rows, n)
        w0, a0, nw = r32(n), r32(n), torch.ones(n, device=dev)
        st2 = torch.zeros((batch, RH, rd, rd), dtype=torch.float32, device=dev)
        f_kd = lambda: kernels.delta_rule(*(proj[:, i * n:(i + 1) * n] for i in range(3)), wl, proj[:, 3 * n:4 * n],
                                          proj[:, 4 * n:], w0, a0, nw, st2, prm.q_cu_seq_lens, positions,
                                          prm.state_slots, RH, rd, 0.6, 1e-6, 1e-5)
        for name, fn, nbytes, flops in (
                (f"fesupel sigmoid_attn, blocks of {blk}", f_sig(blk), touched * G * (dim + vd) * 2 + qb,
                 bpairs * H * 2 * (dim + vd)),
                ("fesupel sigmoid_attn, no block limit", f_sig(0), batch * ctx * G * (dim + vd) * 2 + qb,
                 pairs * H * 2 * (dim + vd)),
                ("llama paged attention, same heads", f_llama, batch * ctx * 2 * G * dim * 2 + rows * H * dim * 4,
                 pairs * H * 4 * dim),
                ("fesupel gated_delta_scan", f_gd,
                 rows * (2 * RG * rd * 4 + RH * rd * 4 + RH * rv * 8) + batch * 2 * RH * rd * rv * 4, rows * RH * 6 * rd * rv),
                ("kigalix delta_rule, same heads and state", f_kd, rows * 7 * n * 2 + batch * 2 * n * rd * 4,
                 rows * RH * 6 * rd * rd)):
            if q_len > 1 and "no block limit" in name:
                continue            # the walk over every earlier key on CUDA cores is not a prompt kernel
            ms = _time_steps(fn, 3, 10)
            out[f"{name}, {batch} x {ctx} cached, {q_len} new"] = _frac(ms, nbytes, flops, hbm, tf)
        del kc, vc, kl, vl
        torch.cuda.empty_cache()
    return out


def run_fesupel(args) -> None:
    torch.cuda.set_device(0)
    torch.backends.cuda.matmul.allow_tf32 = False
    peaks_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    peaks = json.load(open(peaks_path)) if os.path.exists(peaks_path) else {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    out = {"metric": "fesupel_vs_kigalix_vs_llama_tokens_per_s", "unit": "tokens/s", "dtype": "bf16",
           "data": "synthetic (random-init weights, random token ids)", "n_gpus": 1,
           "peaks": {"hbm_gbs": peaks["hbm_gbs"], "bf16_tflops": peaks["bf16_tflops"],
                     "source": "measured" if os.path.exists(peaks_path) else "fallback"}, "sizes": {}}
    names = [args.arch_size] if args.arch_size != "all" else list(SIZES)
    for name in names:
        s = dict(SIZES[name], **FESUPEL_EXTRA[name])
        batch, seqlen = args.arch_batch, args.arch_seqlen
        t0 = time.time()
        f = _run_model(fesupel_config(s), batch, seqlen, args.warmup, args.steps, FESUPEL_KERNELS)
        k = _run_model(kigalix_config(s), batch, seqlen, args.warmup, args.steps, KIGALIX_KERNELS)
        l = _run_model(llama_config(s), batch, seqlen, args.warmup, args.steps, LLAMA_KERNELS)
        out["sizes"][name] = {"shape": s, "batch": batch, "seq_len": seqlen, "fesupel": f, "kigalix": k, "llama": l,
                              "kernel_rooflines": fesupel_rooflines(s, batch, seqlen, f, k, l, peaks),
                              "kernels_alone": fesupel_kernels_alone(s, peaks),
                              "seconds": round(time.time() - t0, 1)}
    print(json.dumps(out))
