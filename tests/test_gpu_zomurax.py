"""GPU: the Zomurax decoder through the serving engine against the plain CPU restatement (oracle/zomurax.py,
float64): every mechanism alone, whole prompts, token-by-token decoding, portions, mixed batches, reuse of blocks,
keys far away, at block borders and on both sides of the window's edge, the first tokens, the sink, the distance
bias and the temperature's steps, generation through the scheduler."""
import math

import numpy as np
import pytest
import torch

from oracle import zomurax as oz
from tests import zomurax_case as zc

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None
TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}
DTYPES = [torch.float32, torch.bfloat16]


def build(cfg, dtype, seed=0, max_seqs=4):
    from scalellm_b200 import registry
    w = zc.weights(cfg, seed)
    model = registry.create_model(cfg, dtype, DEV, max_seqs=max_seqs)
    model.load_weights({k: v.to(DEV) for k, v in w.items()})
    return model, oz.Zomurax(cfg, w)


def engine_for(model, max_tokens=512, block_size=4, max_seqs=4, use_graphs=False):
    from scalellm_b200.engine import Engine
    return Engine(model, max_tokens, block_size=block_size, max_seqs=max_seqs, use_graphs=use_graphs)


def oracle_logits(oracle, tokens):
    return oracle.forward(tokens, oracle.new_state())


def run_schedule(eng, tokens, cuts, rid="r"):
    """Feed `tokens` in portions of the given sizes (the rest one by one); logits of every position."""
    from scalellm_b200.engine import StepEntry
    out, at = [], 0
    sizes = list(cuts)
    while at < len(tokens):
        n = sizes.pop(0) if sizes else 1
        n = min(n, len(tokens) - at)
        out.append(eng.step([StepEntry(rid, tokens[at:at + n], list(range(n)))]).float().cpu())
        at += n
    eng.finish(rid)
    return torch.cat(out, 0)


def toks(n, vocab, seed):
    return [int(x) for x in np.random.default_rng(seed).integers(0, vocab, size=n)]


def _params(n_tokens_per_seq, cached, block_size=4, n_blocks=256, pool_seed=3):
    from scalellm_b200.decode_step import BlockPool, StepBuffers, build_step_batch
    pool = BlockPool(n_blocks, block_size, seed=pool_seed)
    seqs = []
    for n, c in zip(n_tokens_per_seq, cached):
        s = pool.open_sequence()
        pool.reserve(s, n + c)
        seqs.append(s)
    hb = build_step_batch(pool, seqs, [[0] * n for n in n_tokens_per_seq], list(cached), None)
    bufs = StepBuffers(DEV, sum(n_tokens_per_seq) + 8, len(seqs) + 1, n_blocks + 8)
    return bufs.upload(hb), hb


def _slots(hb, seq_index, n, block_size):
    lo = int(hb.cu_block_lens[seq_index])
    return [int(hb.block_tables[lo + j // block_size]) + j % block_size for j in range(n)]


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("W", [1, 48, 200, 1024])
@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_after_the_sum(W, dtype):
    """One gain for the row and one per channel; residual weights 1 and not 1; in place and into another buffer."""
    from scalellm_b200 import kernels
    g = torch.Generator().manual_seed(W)
    for rows, alpha, per_channel in ((5, 1.0, False), (3, 2.5, False), (4, 0.5, True)):
        x = torch.randn(rows, W, generator=g) * 3.0
        y = torch.randn(rows, W, generator=g).to(dtype)
        w = (0.5 + torch.rand(W if per_channel else 1, generator=g))
        s = alpha * x.double() + y.double()
        want = oz.unit(s, 1e-5) * w.double()
        xd = x.to(DEV)
        out, h = kernels.sumnorm_residual(xd, y.to(DEV), w.to(DEV), alpha, 1e-5)
        assert out.data_ptr() == xd.data_ptr()
        assert float((out.cpu().double() - want).abs().max()) < 1e-5 * max(1.0, float(want.abs().max()))
        if dtype == torch.float32:
            assert h is None
        else:
            assert torch.equal(h.cpu(), out.cpu().to(dtype))
        other = torch.empty_like(xd)
        xd2 = x.to(DEV)
        out2, _ = kernels.sumnorm_residual(xd2, y.to(DEV), w.to(DEV), alpha, 1e-5, x_out=other)
        assert out2.data_ptr() == other.data_ptr() and torch.equal(xd2.cpu(), x) and torch.equal(out2.cpu(), out.cpu())


@pytest.mark.parametrize("rows", [1, 7, 128])
def test_norm_after_the_sum_takes_split_k_partials(rows):
    from scalellm_b200 import kernels
    if not kernels.splitk_consumers_available():
        pytest.skip("the loaded library has no split-K dense product")
    g = torch.Generator().manual_seed(rows)
    W, K = 256, 384
    a = torch.randn(rows, K, generator=g).to(torch.bfloat16).to(DEV)
    wt = (torch.randn(W, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    x = torch.randn(rows, W, generator=g).to(DEV)
    gain = torch.tensor([1.3], device=DEV)
    parts = kernels.dense_gemm_splitk(a, wt, poison=True)
    y = (a.float() @ wt.float().T).to(torch.bfloat16)
    want, want_h = kernels.sumnorm_residual(x.clone(), y, gain, 2.0, 1e-5)
    got, got_h = kernels.sumnorm_residual(x.clone(), parts, gain, 2.0, 1e-5, torch.bfloat16)
    assert float((got - want).abs().max()) < 2e-2 and float((got_h.float() - want_h.float()).abs().max()) < 4e-2
    ref = oz.unit(2.0 * x.cpu().double() + (a.cpu().double() @ wt.cpu().double().T), 1e-5) * 1.3
    assert float((got.cpu().double() - ref).abs().max()) < 3e-2


@pytest.mark.parametrize("rows", [1, 7, 128, 200])
def test_shared_expert_with_and_without_split_k_partials(rows):
    """Widths that let decode-sized bf16 steps hand the gate-up product's partials to the activation launch (up to
    128 rows) and a step too large for it: both against the restatement."""
    from scalellm_b200.layers import GatedMLP
    g = torch.Generator().manual_seed(rows)
    W, ff = 256, 128
    w = {k: (torch.randn((W, ff) if k == "down" else (ff, W), generator=g) / math.sqrt(W)).to(torch.bfloat16)
         for k in ("gate", "up", "down")}
    mlp = GatedMLP(w["gate"].to(DEV), w["up"].to(DEV), w["down"].to(DEV), "silu")
    h = torch.randn(rows, W, generator=g).to(torch.bfloat16)
    got = mlp(h.to(DEV)).float().cpu().double()
    want = oz.expert(h.double(), {"s." + k: v.double() for k, v in w.items()}, "s.")
    assert float((got - want).abs().max()) < 0.03 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
def test_logit_cap(dtype):
    from scalellm_b200 import kernels
    x = torch.linspace(-90.0, 90.0, 1001).reshape(7, 143).to(dtype)
    got = kernels.softcap_(x.to(DEV).clone(), 30.0).cpu()
    want = 30.0 * torch.tanh(x.double() / 30.0)
    assert float((got.double() - want).abs().max()) < (1e-5 if dtype == torch.float32 else 0.13)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,top,shared", [(5, 1, 0), (5, 2, 24), (3, 3, 8), (11, 4, 0)])
def test_experts_by_token_table(dtype, E, top, shared):
    """Few rows (the weight-streaming kernel) and many (the grouped product), every expert used and some unused."""
    from scalellm_b200.layers import GatedMLP, TableMoE
    g = torch.Generator().manual_seed(E * 10 + top)
    W, ff, V = 64, 40, 50
    w = {f"e{e}.{k}": (torch.randn((W, ff) if k == "down" else (ff, W), generator=g) / math.sqrt(W)).to(torch.bfloat16)
         for e in range(E) for k in ("gate", "up", "down")}
    if shared:
        w.update({f"shared.{k}": (torch.randn((W, shared) if k == "down" else (shared, W), generator=g) / math.sqrt(W))
                  .to(torch.bfloat16) for k in ("gate", "up", "down")})
    w["table"] = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(V)]).to(torch.int32)
    d = lambda t: t.to(DEV).to(dtype)
    stack = lambda leaf: torch.stack([d(w[f"e{e}.{leaf}"]) for e in range(E)])
    sh = GatedMLP(d(w["shared.gate"]), d(w["shared.up"]), d(w["shared.down"]), "silu") if shared else None
    moe = TableMoE(w["table"].to(DEV), stack("gate"), stack("up"), stack("down"), "silu", sh)
    mlp = {"router": {"experts": E, "top": top}}
    for rows, vocab_used in ((3, V), (300, V), (40, 2)):
        tokens = toks(rows, vocab_used, rows)
        h = torch.randn(rows, W, generator=g).to(torch.bfloat16)
        got = moe(d(h), torch.tensor(tokens, dtype=torch.int32, device=DEV))
        want = oz.table_moe(h.double(), tokens, {k: (v.double() if v.is_floating_point() else v) for k, v in w.items()}, mlp)
        tol = 1e-4 if dtype == torch.float32 else 0.04
        assert float((got.cpu().double() - want).abs().max()) < tol * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,dim,vdim", [(4, 2, 16, 24), (3, 3, 20, 8), (6, 2, 48, 96), (2, 1, 64, 130)])
def test_attention_inputs_unit_length_temperature_and_value_blend(dtype, H, G, dim, vdim):
    """Positions on both sides of the temperature's steps; values written as they are and blended; cache rows of
    other tokens untouched."""
    from scalellm_b200 import kernels
    g = torch.Generator().manual_seed(dim)
    every, coef, bs = 5, 0.7, 4
    cached, n_new = 3, 14                     # positions 3 .. 16: steps at 4, 9, 14
    (_, pos, par), hb = _params([n_new], [cached], block_size=bs)
    width = H * dim + G * dim + G * vdim
    proj = (torch.randn(n_new, width + 3, generator=g) * 2.0).to(dtype)   # a wider matrix: the blocks are column views
    vo = torch.randn(n_new, G * vdim, generator=g).to(dtype)
    pd = proj.to(DEV)
    qi, ki, vi = pd[:, : H * dim], pd[:, H * dim: (H + G) * dim], pd[:, (H + G) * dim: width]
    for lam, other in ((0.0, None), (0.35, vo.to(DEV))):
        kc = torch.full((256 * bs, G, dim), 7.0, dtype=dtype, device=DEV)
        vc = torch.full((256 * bs, G, vdim), 7.0, dtype=dtype, device=DEV)
        q = kernels.sink_attn_prepare(qi, ki, vi, other, lam, kc, vc, pos, par.new_cache_slots, H, G, dim, vdim, 1e-5,
                                      coef, every)
        p = torch.arange(cached, cached + n_new)
        temp = oz.query_temperature(p, {"coef": coef, "every": every})
        assert len(set(temp.tolist())) == 4
        want_q = oz.unit(proj[:, : H * dim].double().reshape(n_new, H, dim), 1e-5) * temp[:, None, None]
        want_k = oz.unit(proj[:, H * dim: (H + G) * dim].double().reshape(n_new, G, dim), 1e-5)
        want_v = proj[:, (H + G) * dim: width].double().reshape(n_new, G, vdim)
        if other is not None:
            want_v = (1.0 - lam) * want_v + lam * vo.double().reshape(n_new, G, vdim)
        tol = 1e-5 if dtype == torch.float32 else 0.02
        assert float((q.cpu().double() - want_q).abs().max()) < 1e-5 * float(want_q.abs().max())
        slots = _slots(hb, 0, cached + n_new, bs)[cached:]
        assert float((kc[slots].cpu().double() - want_k).abs().max()) < tol
        assert float((vc[slots].cpu().double() - want_v).abs().max()) < tol * float(want_v.abs().max())
        untouched = torch.ones(256 * bs, dtype=torch.bool)
        untouched[slots] = False
        assert bool((kc.cpu()[untouched] == 7.0).all()) and bool((vc.cpu()[untouched] == 7.0).all())
    # no temperature
    q = kernels.sink_attn_prepare(qi, ki, vi, None, 0.0, kc, vc, pos, par.new_cache_slots, H, G, dim, vdim, 1e-5)
    want_q = oz.unit(proj[:, : H * dim].double().reshape(n_new, H, dim), 1e-5)
    assert float((q.cpu().double() - want_q).abs().max()) < 1e-5 * float(want_q.abs().max())


def _attend_case(dtype, H, G, dim, vdim, block_size, cached, n_new, loud, bias=True, sink=True, seed=0, gain=6.0,
                 n_splits=0):
    """The attention kernel alone over a hand-made cache: the query of row i points along key `loud[i]` with a length
    that lets this key take most of the row's weight.  Returns (got, want)."""
    from scalellm_b200 import kernels
    g = torch.Generator().manual_seed(seed)
    n = cached + n_new
    K = oz.unit(torch.randn(n, G, dim, generator=g), 0.0)
    V = torch.randn(n, G, vdim, generator=g)
    q = oz.unit(torch.randn(n_new, H, dim, generator=g), 0.0)
    pos = torch.arange(cached, n)
    for i, j in enumerate(loud):
        if j is None:
            continue
        for hh in range(H):
            q[i, hh] = gain * K[j, hh // (H // G)]
    K, V = K.to(dtype), V.to(dtype)
    r1 = (0.1 + 0.5 * torch.rand(H, generator=g)) if bias else None
    r2 = (0.05 + 0.5 * torch.rand(H, generator=g)) if bias else None
    sk = (2.0 + torch.randn(H, generator=g)) if sink else None
    (_, _, par), hb = _params([n_new], [cached], block_size=block_size)
    slots = _slots(hb, 0, n, block_size)
    kc = torch.zeros(256 * block_size, G, dim, dtype=dtype)
    vc = torch.zeros(256 * block_size, G, vdim, dtype=dtype)
    kc[slots], vc[slots] = K, V
    scale = 1.3 / math.sqrt(dim)            # unit keys have length sqrt(dim): the loud score is 1.3 gain sqrt(dim)
    dv = lambda t: None if t is None else t.to(DEV)
    got = kernels.sink_attn(q.to(DEV), kc.to(DEV), vc.to(DEV), dv(r1), dv(r2), dv(sk), par.q_cu_seq_lens,
                            par.kv_cu_seq_lens, par.block_tables, par.cu_block_lens, par.token_seq, block_size, scale,
                            1, n_new, n, n_splits)   # bf16 cases of fitting sizes take the tensor-core kernels
    f64 = lambda t: None if t is None else t.double()
    # the tensor-core kernel rounds the queries to bf16 as the keys are
    tensor_core = (dtype == torch.bfloat16 and dim % 16 == 0 and vdim % 16 == 0 and dim <= 128 and vdim <= 128
                   and (n_new >= kernels.SINK_ATTN_PREFILL_MIN_ROWS or H // G >= kernels.SINK_ATTN_DECODE_TC_MIN_GROUP))
    qr = q.to(torch.bfloat16).double() if tensor_core else q.double()
    want = oz.sink_attend(qr, K.double(), V.double(), pos, scale, f64(r1), f64(r2), f64(sk))
    return got.float().cpu().reshape(n_new, H, vdim).double(), want


SIZES = [(4, 2, 16, 24), (3, 3, 20, 8), (2, 1, 64, 130), (8, 4, 48, 80), (2, 2, 64, 64), (3, 1, 32, 16), (6, 2, 128, 64),
         (16, 2, 16, 32), (5, 1, 8, 16), (34, 1, 16, 16), (4, 2, 128, 128), (4, 4, 32, 64), (12, 3, 48, 80)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,dim,vdim", SIZES)
def test_attention_far_keys_bias_and_sink(dtype, H, G, dim, vdim):
    tol = 1e-4 if dtype == torch.float32 else 0.05
    # one decoded token over 300 cached: key 1 decides although it is far; then prompt rows whose key is far back
    for bias, sink in ((True, True), (False, True), (True, False), (False, False)):
        for n_splits in (0, 1, 2, 3, 9):      # the row's key tiles shared out over several CTAs, some left empty
            got, want = _attend_case(dtype, H, G, dim, vdim, 8, 300, 1, [1], bias, sink, seed=7, gain=9.0, n_splits=n_splits)
            assert float((got - want).abs().max()) < tol, (bias, sink, n_splits)
    # three single tokens' worth of rows among many keys that all matter (no loud key), split and not
    for n_splits in (0, 1, 4):
        got, want = _attend_case(dtype, H, G, dim, vdim, 16, 700, 3, [None] * 3, seed=11, n_splits=n_splits)
        assert float((got - want).abs().max()) < tol, n_splits
    got, want = _attend_case(dtype, H, G, dim, vdim, 16, 150, 70, [3 * i for i in range(70)], seed=dim, gain=9.0)
    assert float((got - want).abs().max()) < tol
    # the sink really takes weight: with it the rows are shorter than without
    a, _ = _attend_case(dtype, H, G, dim, vdim, 8, 40, 5, [None] * 5, True, True, seed=3)
    b, _ = _attend_case(dtype, H, G, dim, vdim, 8, 40, 5, [None] * 5, True, False, seed=3)
    assert float((a - b).abs().max()) > 0.05
    # and so does the bias: a far key that is loud enough to compete with the near ones loses against it
    a, wa = _attend_case(dtype, H, G, dim, vdim, 8, 300, 1, [1], True, False, seed=7, gain=5.0 / math.sqrt(dim))
    b, wb = _attend_case(dtype, H, G, dim, vdim, 8, 300, 1, [1], False, False, seed=7, gain=5.0 / math.sqrt(dim))
    assert float((wa - wb).abs().max()) > 0.03 and float((a - wa).abs().max()) < tol and float((b - wb).abs().max()) < tol


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_first_tokens_and_block_borders(dtype):
    tol = 1e-4 if dtype == torch.float32 else 0.05
    # a prompt from position 0, block sizes 1 / 3 / 16, both kernels
    for bs in (1, 3, 16):
        for vdim in (24, 32):
            got, want = _attend_case(dtype, 4, 2, 16, vdim, bs, 0, 19,
                                     [0, 0, 1, 2, 3, 1, 2, 2, None, 4, 6, 7, 1, 9, 9, None, 0, 13, 18], seed=bs)
            assert float((got - want).abs().max()) < tol
    # long portions on top of a long cache: tile borders of the keys and of the rows
    for cached, n_new in ((100, 70), (31, 97), (64, 64), (200, 33), (5, 130), (0, 1), (0, 2), (0, 33)):
        loud = [None] * n_new
        loud[0], loud[-1], loud[n_new // 2] = 0, cached, max(0, cached - 1)
        got, want = _attend_case(dtype, 4, 2, 32, 48, 16, cached, n_new, loud, seed=cached + n_new)
        assert float((got - want).abs().max()) < tol, (cached, n_new)
    # two new tokens (the single-token path) on caches that end just before, at and just after a 32- and 64-key border
    for cached in (0, 1, 30, 31, 32, 33, 62, 63, 64, 65, 127, 128, 200):
        for H, G in ((8, 2), (3, 3)):
            got, want = _attend_case(dtype, H, G, 32, 48, 16, cached, 2, [min(cached, 4), None], seed=cached)
            assert float((got - want).abs().max()) < tol, (cached, H, G)


def _latent_case(dtype, H, dim, rd, vd, rank, window, block_size, cached, n_new, loud, seed=0):
    """The latent-attention kernel alone over hand-made cache rows: the unrotated query of row i points along the
    key that head h makes of latent `loud[i]`.  Returns (got, want) as [rows, H, vd]."""
    from scalellm_b200 import kernels
    g = torch.Generator().manual_seed(seed)
    n = cached + n_new
    C = torch.randn(n, rank, generator=g).to(dtype)
    KR = torch.randn(n, rd, generator=g).to(dtype)
    uk = (torch.randn(H, dim, rank, generator=g) / math.sqrt(rank)).to(dtype)
    uv = (torch.randn(H, vd, rank, generator=g) / math.sqrt(rank)).to(dtype)
    q = torch.randn(n_new, H, dim + rd, generator=g)
    for i, j in enumerate(loud):
        if j is None:
            continue
        for hh in range(H):
            kj = uk[hh].double() @ C[j].double()
            q[i, hh, :dim] = (10.0 * math.sqrt(dim) * kj / kj.norm() ** 2).float()      # a score of 10 on key j
    q = q.to(dtype)
    pos = torch.arange(cached, n)
    scale = 1.0 / math.sqrt(dim)
    (_, _, par), hb = _params([n_new], [cached], block_size=block_size)
    slots = _slots(hb, 0, n, block_size)
    cache = torch.zeros(256 * block_size, rank + rd, dtype=dtype)
    cache[slots] = torch.cat([C, KR], dim=1)
    qd = q.reshape(n_new, H * (dim + rd)).to(DEV)
    qa = torch.bmm(q.to(DEV)[:, :, :dim].transpose(0, 1).float(), uk.to(DEV).float())       # [H, rows, rank] fp32
    lat = kernels.latent_attn(qa, qd, cache.to(DEV), par.q_cu_seq_lens, par.kv_cu_seq_lens, par.block_tables,
                              par.cu_block_lens, par.token_seq, H, dim, rd, rank, block_size, scale, n, window)
    got = torch.einsum("htr,hvr->thv", lat.float().cpu().double(), uv.double())
    want = oz.latent_attend(q.double(), C.double(), KR.double(), uk.double(), uv.double(), pos, scale, window)
    return got, want


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dim,rd,vd,rank", [(4, 16, 8, 16, 24), (3, 10, 6, 12, 14), (8, 64, 32, 48, 80), (17, 32, 16, 48, 40)])
def test_latent_attention_window_edges(dtype, H, dim, rd, vd, rank):
    """Decoded rows and prompt rows whose loud key lies just inside / just outside the window; windows shorter and
    longer than a key tile, as long as and longer than the sequence; no window."""
    tol = 1e-4 if dtype == torch.float32 else 0.06
    for window, cached in ((10, 41), (33, 70), (70, 200), (1, 9), (64, 64)):
        # rows at positions cached .. cached + 5; the window of row i covers i - window + 1 .. i
        first = lambda row: cached + row - window + 1
        loud = [first(0), first(1) - 1, first(2), first(3) - 1, cached + 4, first(5)]
        loud = [j if j >= 0 else None for j in loud]
        got, want = _latent_case(dtype, H, dim, rd, vd, rank, window, 4, cached, 6, loud, seed=window)
        assert float((got - want).abs().max()) < tol * max(1.0, float(want.abs().max())), (window, cached)
        for row, j in ((1, first(1) - 1), (3, first(3) - 1)):
            assert j < 0 or not oz.window_visible(cached + row, j, window)
        assert oz.window_visible(cached, first(0), window)
        # and one decoded token alone: just inside, just outside
        for j in (cached - window + 1, cached - window):
            if j >= 0:
                got, want = _latent_case(dtype, H, dim, rd, vd, rank, window, 8, cached, 1, [j], seed=j)
                assert float((got - want).abs().max()) < tol * max(1.0, float(want.abs().max())), (window, cached, j)
    # the loud key outside the window is really unseen: with and without the window the rows differ
    a, wa = _latent_case(dtype, H, dim, rd, vd, rank, 10, 8, 300, 1, [1], seed=5)
    b, wb = _latent_case(dtype, H, dim, rd, vd, rank, 0, 8, 300, 1, [1], seed=5)
    assert float((wa - wb).abs().max()) > 0.05
    assert float((a - wa).abs().max()) < tol * max(1.0, float(wa.abs().max()))
    assert float((b - wb).abs().max()) < tol * max(1.0, float(wb.abs().max()))
    # prompts from position 0 (rows shorter than the window), long portions over tile borders, window > sequence
    for window, cached, n_new in ((5, 0, 19), (40, 100, 70), (33, 31, 97), (500, 0, 60), (0, 64, 64)):
        loud = [None] * n_new
        loud[0], loud[-1] = max(0, cached - window + 1) if window else 0, max(0, cached + n_new - window) if window else 2
        got, want = _latent_case(dtype, H, dim, rd, vd, rank, window, 16, cached, n_new, loud, seed=window + n_new)
        assert float((got - want).abs().max()) < tol * max(1.0, float(want.abs().max())), (window, cached, n_new)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dims,rd", [(8, 8), (16, 16), (4, 12), (64, 64)])
def test_rotary_turn_over_half_pairs(dtype, dims, rd):
    from scalellm_b200 import kernels
    from scalellm_b200.zomurax import rotary_table
    g = torch.Generator().manual_seed(dims)
    H, dim, rank, bs, cached, n_new = 3, 10, 14, 4, 37, 9
    rot = {"dims": dims, "base": 777.0}
    (_, pos, par), hb = _params([n_new], [cached], block_size=bs)
    q = torch.randn(n_new, H * (dim + rd), generator=g).to(dtype)
    dkv = torch.randn(n_new, rank + rd, generator=g).to(dtype)
    cw = (0.5 + torch.rand(rank, generator=g))
    cache = torch.zeros(256 * bs, rank + rd, dtype=dtype, device=DEV)
    qd = q.to(DEV).clone()
    kernels.latent_prepare(qd, dkv.to(DEV), cache, cw.to(DEV), rotary_table(rot).to(DEV), 1.0, pos, par.new_cache_slots,
                           H, dim, rd, dims, rank, 1e-5, half_pairs=True)
    p = torch.arange(cached, cached + n_new)
    q3 = q.double().reshape(n_new, H, dim + rd)
    want_q = torch.cat([q3[..., :dim], oz.turn_half(q3[..., dim:], p, rot)], dim=-1).reshape(n_new, -1)
    want_c = oz.unit(dkv[:, :rank].double(), 1e-5) * cw.double()
    want_kr = oz.turn_half(dkv[:, rank:].double(), p, rot)
    tol = 2e-5 if dtype == torch.float32 else 0.04
    rows = cache[_slots(hb, 0, cached + n_new, bs)[cached:]].cpu().double()
    assert float((qd.cpu().double() - want_q).abs().max()) < tol * float(want_q.abs().max())
    assert float((rows[:, :rank] - want_c).abs().max()) < tol * float(want_c.abs().max())
    assert float((rows[:, rank:] - want_kr).abs().max()) < tol * float(want_kr.abs().max())


# ------------------------------------------------------------------ the model
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(zc.CONFIGS))
def test_whole_prompt_layers_and_logits(name, dtype):
    cfg = zc.CONFIGS[name]
    model, oracle = build(cfg, dtype)
    eng = engine_for(model)
    tokens = toks(75, cfg["vocab"], 1)
    lo = []
    want = oracle.forward(tokens, oracle.new_state(), lo)
    from scalellm_b200.decode_step import build_step_batch
    s = eng.open("x")
    eng.pool.reserve(s.seq, len(tokens))
    hb = build_step_batch(eng.pool, [s.seq], [tokens], [0], None)
    tok, pos, par = eng.bufs.upload(hb)
    got_layers = []
    got = model.forward(tok, pos, par, layer_out=got_layers)
    assert len(got_layers) == len(lo) == len(cfg["layers"])
    for a, b in zip(got_layers, lo):
        assert float((a.cpu().double() - b).abs().max()) < (2e-4 if dtype == torch.float32 else 0.05) * float(b.abs().max())
    assert zc.logits_error(got, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(zc.CONFIGS))
def test_prefill_decode_and_portions_agree_with_the_oracle(name, dtype):
    cfg = zc.CONFIGS[name]
    model, oracle = build(cfg, dtype, seed=1)
    tokens = toks(90, cfg["vocab"], 2)
    want = oracle_logits(oracle, tokens)
    for cuts in ([90], [58], [1] * 3, [2, 2, 5, 2, 31, 1, 2, 17, 2], [7] * 13, [33, 4, 4, 4, 40]):
        eng = engine_for(model, block_size=4)
        got = run_schedule(eng, tokens, cuts)
        assert zc.logits_error(got, want) < TOL[dtype], cuts


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_portions_over_many_key_tiles(dtype):
    """Portions cut at places that are no multiple of a tile or a block, against the whole prompt and the oracle."""
    cfg = zc.CONFIGS["mix"]
    model, oracle = build(cfg, dtype, seed=6)
    tokens = toks(333, cfg["vocab"], 7)
    want = oracle_logits(oracle, tokens)
    for cuts in ([333], [150, 2, 181], [129, 130, 71]):
        eng = engine_for(model, max_tokens=400, block_size=16)
        got = run_schedule(eng, tokens, cuts)
        assert zc.logits_error(got, want) < TOL[dtype], cuts


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_batches_with_reused_blocks(dtype):
    """Five unequal requests through a pool with room for three: portions beside single tokens, requests that
    pause, blocks handed on without being cleared."""
    from scalellm_b200.engine import StepEntry
    cfg = zc.CONFIGS["mix"]
    model, oracle = build(cfg, dtype, seed=2, max_seqs=3)
    lens = {"a": 61, "b": 9, "c": 40, "d": 1, "e": 33}
    T = {k: toks(n, cfg["vocab"], 10 + i) for i, (k, n) in enumerate(lens.items())}
    want = {k: oracle_logits(oracle, v) for k, v in T.items()}
    eng = engine_for(model, max_tokens=128, block_size=4, max_seqs=3)
    plan = [[("a", 17), ("b", 2)], [("a", 2), ("b", 1), ("c", 5)], [("b", 6), ("c", 1)], [("a", 30), ("c", 30)],
            [("a", 1), ("c", 2)], [("a", 1), ("c", 2), ("d", 1)], [("a", 10), ("e", 2)], [("e", 29)], [("e", 1)], [("e", 1)]]
    at = {k: 0 for k in T}
    got = {k: [] for k in T}
    for step in plan:
        entries = [StepEntry(k, T[k][at[k]:at[k] + n], list(range(n))) for k, n in step]
        out = eng.step(entries).float().cpu()
        r = 0
        for k, n in step:
            got[k].append(out[r:r + n])
            r += n
            at[k] += n
            if at[k] == lens[k]:
                eng.finish(k)
    for k in T:
        assert at[k] == lens[k]
        assert zc.logits_error(torch.cat(got[k]), want[k]) < TOL[dtype], k
    # each request alone gives the same rows as in the batch, beyond rounding
    for k in ("a", "e"):
        alone = run_schedule(engine_for(model, max_tokens=128, block_size=4, max_seqs=3), T[k], [lens[k]], rid=k)
        assert zc.logits_error(torch.cat(got[k]), alone) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_over_small_blocks(dtype):
    cfg = zc.CONFIGS["attn_first"]
    model, oracle = build(cfg, dtype, seed=3)
    tokens = toks(150, cfg["vocab"], 4)
    want = oracle_logits(oracle, tokens)
    eng = engine_for(model, max_tokens=160, block_size=2)
    got = run_schedule(eng, tokens, [3])
    assert zc.logits_error(got, want) < TOL[dtype]


def test_graph_replay_of_single_token_steps():
    cfg = zc.CONFIGS["mix"]
    model, oracle = build(cfg, torch.bfloat16, seed=4)
    tokens = toks(40, cfg["vocab"], 5)
    want = oracle_logits(oracle, tokens)
    eng = engine_for(model, block_size=4, use_graphs=True)
    got = run_schedule(eng, tokens, [6])
    assert eng._graphs, "no graph was captured"
    assert zc.logits_error(got, want) < TOL[torch.bfloat16]


def test_greedy_generation_through_the_scheduler():
    """More requests than places; the ids must be those of greedy decoding with the oracle wherever its two
    best logits are not a near tie."""
    from scalellm_b200.engine import SamplingParams
    cfg = zc.CONFIGS["plain"]
    model, oracle = build(cfg, torch.float32, seed=5, max_seqs=2)
    eng = engine_for(model, max_tokens=96, block_size=4, max_seqs=2)
    prompts = [toks(n, cfg["vocab"], 20 + n) for n in (5, 17, 1, 9)]
    outs = eng.generate(prompts, [SamplingParams(max_new_tokens=6) for _ in prompts], max_step_tokens=8)
    for p, o in zip(prompts, outs):
        assert len(o) == 6
        st = oracle.new_state()
        lg = oracle.forward(p, st)[-1]
        for tok in o:
            top = torch.topk(lg, 2).values
            if float(top[0] - top[1]) > 1e-3:
                assert int(lg.argmax()) == tok
            lg = oracle.forward([tok], st)[-1]


def test_model_folder_through_the_registry(tmp_path):
    """config.json + model.safetensors -> registry -> engine: the way the commands load a model."""
    import json
    from scalellm_b200 import checkpoint, registry
    cfg = zc.CONFIGS["attn_first"]
    w = zc.weights(cfg, 8)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    checkpoint.write_safetensors(str(tmp_path / "model.safetensors"), w)
    model = registry.load_model(str(tmp_path), torch.float32, DEV, max_seqs=2)
    tokens = toks(30, cfg["vocab"], 9)
    got = run_schedule(engine_for(model, max_tokens=64, block_size=16, max_seqs=2), tokens, [11, 2])
    assert zc.logits_error(got, oracle_logits(oz.Zomurax(cfg, w), tokens)) < TOL[torch.float32]
