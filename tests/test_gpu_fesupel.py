"""GPU: the Fesupel decoder through the serving engine against the plain CPU restatement (oracle/fesupel.py, float64):
every mechanism alone, whole prompts, token-by-token decoding, portions, mixed batches, reuse of blocks and state
slots, keys far away, at cache-block borders and on both sides of the edge of a block of positions, the first tokens,
filter and matrix state carried over steps, generation through the scheduler."""
import math

import numpy as np
import pytest
import torch

from oracle import fesupel as of
from tests import fesupel_case as fc

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None
TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}
DTYPES = [torch.float32, torch.bfloat16]


def build(cfg, dtype, seed=0, max_seqs=4):
    from scalellm_b200 import registry
    w = fc.weights(cfg, seed)
    model = registry.create_model(fc.public(cfg), dtype, DEV, max_seqs=max_seqs)
    model.load_weights({k: v.to(DEV) for k, v in w.items()})
    return model, of.Fesupel(cfg, w)


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


def _params(n_tokens_per_seq, cached, block_size=4, n_blocks=256, pool_seed=3, slots=None):
    from scalellm_b200.decode_step import BlockPool, StepBuffers, build_step_batch
    pool = BlockPool(n_blocks, block_size, seed=pool_seed)
    seqs = []
    for n, c in zip(n_tokens_per_seq, cached):
        s = pool.open_sequence()
        pool.reserve(s, n + c)
        seqs.append(s)
    hb = build_step_batch(pool, seqs, [[0] * n for n in n_tokens_per_seq], list(cached), slots)
    bufs = StepBuffers(DEV, sum(n_tokens_per_seq) + 8, len(seqs) + 1, n_blocks + 8)
    return bufs.upload(hb), hb


def _slots(hb, seq_index, n, block_size):
    lo = int(hb.cu_block_lens[seq_index])
    return [int(hb.block_tables[lo + j // block_size]) + j % block_size for j in range(n)]


def row_errors(got, want):
    got, want = got.double().cpu(), want.double().cpu()
    got = got - got.mean(dim=-1, keepdim=True)
    want = want - want.mean(dim=-1, keepdim=True)
    return (got - want).pow(2).mean(dim=-1).sqrt() / want.pow(2).mean(dim=-1).sqrt()


def assert_logits(got, want, dtype, what=""):
    """float32: every row within the tolerance.  bfloat16: the router reads rows rounded to 16 bits, so now and then
    a token's last expert is another one than with exact rows, and that row (and, through the cache and the state,
    faintly the ones after it) differs by more than rounding: there the typical row is held to the tolerance and at
    most a tenth of the rows may exceed it.  Faults of logic show in float32, which runs the same kernels."""
    e = row_errors(got, want)
    if dtype == torch.float32:
        assert float(e.max()) < TOL[dtype], f"{what}: {float(e.max())}"
        return
    over = int((e > TOL[dtype]).sum())
    assert float(e.median()) < TOL[dtype] / 3 and over <= max(2, e.numel() // 10), \
        f"{what}: median {float(e.median())}, {over} of {e.numel()} rows over"


def close(got, want, dtype, what=""):
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    err = float((got.double().cpu() - want.double()).abs().max())
    assert err <= tol * max(1.0, float(want.abs().max())), f"{what}: {err}"


# ------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("W", [1, 40, 200, 1030])
@pytest.mark.parametrize("dtype", DTYPES)
def test_branch_norms_into_the_residual(W, dtype):
    """Two branches, one branch with and without its own weight; handed on under the next norm or plain; in place and
    into another buffer."""
    from scalellm_b200 import kernels
    g = torch.Generator().manual_seed(W)
    eps = 1e-5
    for rows, two, own, nxt in ((5, True, True, True), (3, True, True, False), (4, False, False, True),
                                (2, False, True, False), (1, False, False, False)):
        x = torch.randn(rows, W, generator=g) * 3.0
        a = (torch.randn(rows, W, generator=g) * 2.0).to(dtype)
        b = torch.randn(rows, W, generator=g).to(dtype) if two else None
        wa, wb, w, wn = (0.5 + torch.rand(W, generator=g) for _ in range(4))
        m = a.double()
        if own:
            m = of.norm(m, wa.double(), eps)
        if two:
            m = 0.5 * (m + of.norm(b.double(), wb.double(), eps))
        want = x.double() + of.norm(m, w.double(), eps)
        want_h = of.norm(want, wn.double(), eps) if nxt else want
        d = lambda t: None if t is None else t.to(DEV)
        xd = x.to(DEV)
        out, h = kernels.branch_norm_residual(xd, d(a), d(b), d(wa) if own else None, d(wb) if two else None, d(w),
                                              d(wn) if nxt else None, eps)
        assert out.data_ptr() == xd.data_ptr() and h.dtype == dtype
        close(out, want, torch.float32, "residual")
        close(h, want_h, dtype, "handed on")
        other = torch.empty_like(xd)
        xd2 = x.to(DEV)
        out2, h2 = kernels.branch_norm_residual(xd2, d(a), d(b), d(wa) if own else None, d(wb) if two else None, d(w),
                                                d(wn) if nxt else None, eps, x_out=other, want_h=False)
        assert h2 is None and out2.data_ptr() == other.data_ptr() and torch.equal(xd2.cpu(), x)
        assert torch.equal(out2.cpu(), out.cpu())


@pytest.mark.parametrize("dtype", DTYPES)
def test_squared_relu(dtype):
    from scalellm_b200 import kernels
    x = torch.randn(7, 50, generator=torch.Generator().manual_seed(1)).to(dtype)
    big = torch.cat([x, x], dim=1).to(DEV)
    got = kernels.relu_squared(big[:, 50:])                 # a strided column block
    close(got, torch.relu(x.double()) ** 2, dtype)


ROUTES = [  # outputs, pass-through, top, groups, keep
    (6, 0, 2, 1, 1), (6, 2, 3, 4, 2), (8, 4, 4, 3, 1), (5, 1, 6, 1, 1), (16, 0, 4, 4, 1), (9, 0, 3, 3, 3)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,P,top,count,keep", ROUTES)
def test_router_softmax_correction_and_group_limit(dtype, E, P, top, count, keep):
    """Choice by p + correction (corrections large and NEGATIVE too: a dropped group must count as minus infinity, not
    zero), weights by p alone over the chosen sum; the gate of the shared expert rides along."""
    from scalellm_b200 import kernels
    g = torch.Generator().manual_seed(E * 10 + top)
    W, rows, n = 24, 40, E + P
    h = torch.randn(rows, W, generator=g).to(dtype)
    R = torch.randn(n, W, generator=g)
    corr = torch.randn(n, generator=g) * 0.5 - 0.6
    sg = torch.randn(W, generator=g)
    r = {"experts": E, "top": top, "identity": P, "groups": {"count": count, "keep": keep}}
    ids, wts = of.route(h.double(), R.double(), corr.double(), r)
    gi, gw, ge = kernels.moe_route_softmax(h.to(DEV), R.to(DEV), corr.to(DEV), top, count, keep, 1e-20, sg.to(DEV))
    assert torch.equal(gi.cpu().long().sort(dim=1).values, ids.sort(dim=1).values)
    order = gi.cpu().long().argsort(dim=1)
    want_w = wts.gather(1, ids.argsort(dim=1))
    assert float((gw.cpu().double().gather(1, order) - want_w).abs().max()) < 1e-5
    assert float((gw.sum(dim=1) - 1.0).abs().max()) < 1e-5
    assert float((ge.cpu().double() - torch.sigmoid(h.double() @ sg.double())).abs().max()) < 1e-5
    gi2, gw2, none = kernels.moe_route_softmax(h.to(DEV), R.to(DEV), None, top, count, keep, 0.0)
    ids2, _ = of.route(h.double(), R.double(), None, r)
    assert none is None and torch.equal(gi2.cpu().long().sort(dim=1).values, ids2.sort(dim=1).values)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [1, 9, 150])
@pytest.mark.parametrize("E,P,top,count,keep,shared", [(6, 2, 3, 4, 2, 24), (4, 0, 2, 1, 1, 0), (3, 3, 4, 2, 2, 8)])
def test_routed_experts_with_pass_through_and_shared(dtype, rows, E, P, top, count, keep, shared):
    """Few rows (weight-streaming products) and many (grouped products); pass-through outputs chosen and not."""
    from scalellm_b200.layers import ClampedGLU, GroupLimitedMoE
    g = torch.Generator().manual_seed(rows + E)
    W, ff = 32, 16
    mlp = fc.moe(E, top, ff, identity=P, groups=(count, keep), shared_ff=shared or None)
    rnd = lambda *s: (torch.randn(*s, generator=g) / math.sqrt(s[-1])).to(torch.bfloat16)
    w = {"router": (rnd(E + P, W) * 4), "correction": rnd(E + P) * 0.3}
    for e in range(E):
        w.update({f"e{e}.gate": rnd(ff, W) * 2, f"e{e}.up": rnd(ff, W) * 2, f"e{e}.down": rnd(W, ff)})
    if shared:
        w.update({"shared.gate": rnd(shared, W) * 2, "shared.up": rnd(shared, W) * 2, "shared.down": rnd(W, shared),
                  "shared.sg": rnd(1, W)})
    h = torch.randn(rows, W, generator=g).to(dtype)
    want = of.moe_ff(h.double(), {k: v.double() for k, v in w.items()}, mlp)
    d = lambda name: w[name].to(DEV).to(dtype)
    stack = lambda leaf: torch.stack([d(f"e{e}.{leaf}") for e in range(E)])
    sh = ClampedGLU(d("shared.gate"), d("shared.up"), d("shared.down"), 1.0, 1.702) if shared else None
    layer = GroupLimitedMoE(w["router"].to(DEV), w["correction"].to(DEV), stack("gate"), stack("up"), stack("down"),
                            top, count, keep, 1.5, 1.702, 1e-20, sh, w["shared.sg"].to(DEV) if shared else None)
    got = layer(h.to(DEV))
    tol = 1e-4 if dtype == torch.float32 else 4e-2
    assert float((got.double().cpu() - want).abs().max()) < tol * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,dim,vdim,rot", [(4, 2, 16, 24, 8), (3, 3, 10, 6, 10), (6, 2, 48, 96, 0), (2, 1, 64, 130, 32)])
def test_attention_inputs_bias_turn_and_cache_rows(dtype, H, G, dim, vdim, rot):
    from scalellm_b200 import kernels
    g = torch.Generator().manual_seed(H * dim)
    bs = 4
    (tok, pos, par), hb = _params([5, 1], [3, 9], block_size=bs)
    rows = 6
    n = H * dim + G * dim + G * vdim
    proj = torch.randn(rows, n + 5, generator=g).to(dtype)
    qb, kb, vb = (torch.randn(m, generator=g) for m in (H * dim, G * dim, G * vdim))
    rot_cfg = {"dims": rot, "base": 100.0, "scaling": dict(zip(("factor", "low", "high", "original"), fc.SCALING))} if rot else None
    f = torch.tensor(of.turn_frequencies(rot_cfg), dtype=torch.float32) if rot else None
    kc = torch.full((256 * bs, G, dim), 7.0, dtype=dtype, device=DEV)
    vc = torch.full((256 * bs, G, vdim), 7.0, dtype=dtype, device=DEV)
    pd = proj.to(DEV)
    q = kernels.sigmoid_attn_prepare(pd[:, :H * dim], pd[:, H * dim:H * dim + G * dim], pd[:, H * dim + G * dim:n],
                                     qb.to(DEV), kb.to(DEV), vb.to(DEV), kc, vc, None if f is None else f.to(DEV), pos,
                                     par.new_cache_slots, H, G, dim, vdim, rot)
    p64 = proj.double()
    positions = torch.tensor([3, 4, 5, 6, 7, 9])
    wq = of.turn_half((p64[:, :H * dim] + qb.double()).reshape(rows, H, dim), positions, rot_cfg)
    wk = of.turn_half((p64[:, H * dim:H * dim + G * dim] + kb.double()).reshape(rows, G, dim), positions, rot_cfg)
    wv = (p64[:, H * dim + G * dim:n] + vb.double()).reshape(rows, G, vdim)
    close(q, wq, torch.float32 if dtype == torch.float32 else dtype, "queries")
    written = [s for s in _slots(hb, 0, 8, bs)[3:]] + [_slots(hb, 1, 10, bs)[9]]
    close(kc[written], wk, dtype, "keys")
    close(vc[written], wv, dtype, "values")
    mask = torch.ones(kc.shape[0], dtype=torch.bool)
    mask[written] = False
    assert bool((kc.cpu()[mask] == 7.0).all()) and bool((vc.cpu()[mask] == 7.0).all())


def _attend_case(dtype, H, G, dim, vdim, size, block_size, cached, n_new, loud, seed=0, mix=True, cap=0.0, simt=False,
                 n_splits=0):
    """A hand-made cache of one sequence: every key is quiet (its weight is sigmoid of a very negative number) but
    the one at position `loud`, whose weight is close to one for head 0 of every group: a row that sees it carries
    its value, a row that does not carries almost nothing."""
    from scalellm_b200 import kernels
    g = torch.Generator().manual_seed(seed)
    n = cached + n_new
    (tok, pos, par), hb = _params([n_new], [cached], block_size=block_size)
    K = torch.randn(n, G, dim, generator=g) * 0.1
    V = torch.randn(n, G, vdim, generator=g)
    q = torch.randn(n_new, H, dim, generator=g) * 0.1
    if loud is not None:
        K[loud] = 0.0
        K[loud, :, 0] = 4.0
        q[:, :, 0] = 4.0
    K, V = K.to(dtype), V.to(dtype)
    hb_ = torch.full((H,), -9.0)
    T = (torch.eye(H) + 0.3 * torch.randn(H, H, generator=g)) if mix else None
    kc = torch.zeros((256 * block_size, G, dim), dtype=dtype, device=DEV)
    vc = torch.zeros((256 * block_size, G, vdim), dtype=dtype, device=DEV)
    sl = _slots(hb, 0, n, block_size)
    kc[sl], vc[sl] = K.to(DEV), V.to(DEV)
    got = kernels.sigmoid_attn(q.to(DEV), kc, vc, hb_.to(DEV), None if T is None else T.to(DEV), par.q_cu_seq_lens,
                               par.kv_cu_seq_lens, par.block_tables, par.cu_block_lens, par.token_seq, block_size,
                               1.0, cap, size, n_new, 0 if simt else 1, n, n_splits)
    positions = torch.arange(cached, n)
    want = of.sigmoid_attend(q.double(), K.double(), V.double(), positions, 1.0, cap, hb_.double(),
                             None if T is None else T.double(), size)
    return got.reshape(n_new, H, vdim), want, V


SIZES = [(4, 2, 16, 24), (3, 3, 10, 6), (8, 1, 32, 32), (6, 2, 48, 96), (2, 2, 64, 130), (16, 4, 64, 64),
         (12, 3, 16, 48), (32, 8, 32, 64), (20, 20, 16, 16)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,dim,vdim", SIZES)
def test_attention_block_edges_in_prompts_and_decoding(dtype, H, G, dim, vdim):
    """The loud key is the first of the row's block (seen), the last of the block before (not seen), the row itself,
    and far back in a walk without blocks; single rows and portions that cross a block's edge."""
    for size, cached, n_new, loud, seen in ((10, 27, 1, 20, True), (10, 27, 1, 19, False), (10, 29, 1, 20, True),
                                            (10, 30, 1, 29, False), (10, 30, 1, 30, True), (0, 299, 1, 1, True),
                                            (64, 130, 1, 127, False), (64, 130, 1, 128, True)):
        got, want, V = _attend_case(dtype, H, G, dim, vdim, size, 4, cached, n_new, loud, seed=cached)
        close(got, want, dtype, f"size {size} cached {cached} loud {loud}")
        assert (float(want.abs().max()) > 0.3) == seen
        for n_splits in (1, 2, 3, 9):          # the row's key tiles shared out over several CTAs
            got, _, _ = _attend_case(dtype, H, G, dim, vdim, size, 4, cached, n_new, loud, seed=cached, n_splits=n_splits)
            close(got, want, dtype, f"size {size} cached {cached} loud {loud}, {n_splits} shares")
    # portions: rows on both sides of an edge in one step, with the loud key on either side of it
    for size, cached, n_new, loud in ((10, 14, 13, 19), (10, 14, 13, 20), (7, 0, 40, 6), (7, 0, 40, 7), (0, 100, 70, 3),
                                      (33, 60, 10, 65), (1, 5, 9, 8)):
        got, want, V = _attend_case(dtype, H, G, dim, vdim, size, 4, cached, n_new, loud, seed=cached + 1)
        close(got, want, dtype, f"portion size {size} cached {cached} loud {loud}")
        got2, _, _ = _attend_case(dtype, H, G, dim, vdim, size, 4, cached, n_new, loud, seed=cached + 1, simt=True)
        close(got2, want, dtype, f"portion on CUDA cores, size {size} cached {cached} loud {loud}")
        pos = torch.arange(cached, cached + n_new)
        sees = (pos >= loud) & ((pos // size == loud // size) if size else torch.ones_like(pos, dtype=torch.bool))
        loudness = want.abs().amax(dim=(1, 2))
        assert bool((loudness[sees] > 0.3).all()) and bool((loudness[~sees] < 0.1).all())


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_first_tokens_cache_block_borders_head_mix_and_cap(dtype):
    for bs in (1, 3, 16):
        for n_new in (1, 2, 17, 40):
            got, want, _ = _attend_case(dtype, 4, 2, 16, 8, 12, bs, 0, n_new, None, seed=bs + n_new)
            close(got, want, dtype, f"from position 0, cache blocks of {bs}, {n_new} rows")
    for cached in (31, 32, 33, 63, 64, 65):          # walks that end on either side of a key tile
        got, want, _ = _attend_case(dtype, 4, 4, 16, 16, 0, 16, cached, 3, 5, seed=cached)
        close(got, want, dtype, f"cached {cached}")
    a, wa, _ = _attend_case(dtype, 4, 2, 16, 8, 0, 4, 20, 2, 3, seed=9, mix=True)
    b, wb, _ = _attend_case(dtype, 4, 2, 16, 8, 0, 4, 20, 2, 3, seed=9, mix=False)
    close(a, wa, dtype)
    close(b, wb, dtype)
    assert float((wa - wb).abs().max()) > 0.05                       # the mix moves the result
    c, wc, _ = _attend_case(dtype, 4, 2, 16, 8, 0, 4, 20, 2, 3, seed=9, cap=3.0)
    close(c, wc, dtype)
    assert float((wc - wa).abs().max()) > 1e-3                       # so does the cap (16 capped at 3)


def _delta_inputs(H, G, dim, vdim, taps, rows, seed, dtype, rank=5):
    g = torch.Generator().manual_seed(seed)
    nqk, nv = G * dim, H * vdim
    proj = torch.randn(rows, 2 * nqk + nv + H + 3, generator=g).to(dtype)
    dec = torch.randn(rows, H * dim, generator=g).to(dtype)
    gate = torch.randn(rows, nv, generator=g).to(dtype)
    w = {"q.conv": torch.randn(nqk, taps, generator=g) * 0.6, "k.conv": torch.randn(nqk, taps, generator=g) * 0.6,
         "v.conv": torch.randn(nv, taps, generator=g) * 0.6, "A_log": torch.log(0.3 + 3 * torch.rand(H, generator=g)),
         "dt_bias": -3 + 3 * torch.rand(H * dim, generator=g), "norm": 0.5 + torch.rand(vdim, generator=g)}
    return proj, dec, gate, w


def _delta_oracle(proj, dec, gate, w, H, G, dim, vdim, st, eps):
    """The right half from its projections on, in the restatement's functions."""
    p = proj.double()
    rows, nqk, nv = p.shape[0], G * dim, H * vdim
    W = {k: v.double() for k, v in w.items()}
    q = of.silu(of.short_filter(p[:, :nqk], W["q.conv"], st, "cq")).reshape(rows, G, dim)
    k = of.silu(of.short_filter(p[:, nqk:2 * nqk], W["k.conv"], st, "ck")).reshape(rows, G, dim)
    v = of.silu(of.short_filter(p[:, 2 * nqk:2 * nqk + nv], W["v.conv"], st, "cv")).reshape(rows, H, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(p[:, 2 * nqk + nv:2 * nqk + nv + H])
    decay = torch.exp(-torch.exp(W["A_log"])[None, :, None]
                      * torch.nn.functional.softplus(dec.double() + W["dt_bias"]).reshape(rows, H, dim))
    if "S" not in st:
        st["S"] = torch.zeros(H, dim, vdim, dtype=torch.float64)
    o = torch.zeros(rows, H, vdim, dtype=torch.float64)
    for hh in range(H):
        gq = hh // (H // G)
        o[:, hh] = of.delta_scan(q[:, gq], k[:, gq], v[:, hh], beta[:, hh], decay[:, hh], st["S"][hh])
    return (of.unit(o, eps) * W["norm"] * torch.sigmoid(gate.double()).reshape(rows, H, vdim)).reshape(rows, nv), q, k, v


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,dim,vdim,taps", [(4, 2, 16, 8, 4), (2, 2, 24, 32, 3), (3, 1, 8, 40, 2), (5, 5, 10, 6, 1),
                                                (2, 1, 128, 64, 4), (1, 1, 33, 130, 5), (6, 3, 64, 64, 4),
                                                (2, 1, 160, 24, 3), (1, 1, 256, 128, 2)])
def test_gated_delta_rule_filters_and_state_over_portions(dtype, H, G, dim, vdim, taps):
    """Two sequences in two state slots fed in portions of unequal sizes (1, 2, fewer and more than the taps), the
    second slot used before by another sequence: filter inputs and matrices must carry over exactly."""
    from scalellm_b200 import kernels
    eps = 1e-5
    nqk, nv = G * dim, H * vdim
    state = torch.full((3, H, dim, vdim), 5.0, dtype=torch.float32, device=DEV)         # stale numbers of an old owner
    fstate = torch.full((3, max(taps - 1, 0), 2 * nqk + nv), 5.0, dtype=torch.float32, device=DEV)
    plans = {0: [1, 2, 1, 7, 3, 1, 1, 12], 1: [9, 1, 1, 2, 2, 5, 1, 7]}
    total = {s: sum(p) for s, p in plans.items()}
    data = {s: _delta_inputs(H, G, dim, vdim, taps, total[s], 100 + s, dtype) for s in plans}
    want = {}
    for s in plans:
        proj, dec, gate, w = data[s]
        want[s] = _delta_oracle(proj, dec, gate, data[0][3], H, G, dim, vdim, {}, eps)[0]
    w = {k: v.to(DEV) for k, v in data[0][3].items()}
    at = {0: 0, 1: 0}
    got = {0: [], 1: []}
    slot_of = {0: 2, 1: 0}
    for step in range(8):
        ns = [plans[0][step], plans[1][step]]
        (tok, pos, par), hb = _params(ns, [at[0], at[1]], slots=[slot_of[0], slot_of[1]])
        cat = lambda i: torch.cat([data[s][i][at[s]:at[s] + ns[s]] for s in (0, 1)]).to(DEV)
        proj, dec, gate = cat(0), cat(1), cat(2)
        q, k, v, decay, beta = kernels.gated_delta_prepare(
            proj[:, :nqk], proj[:, nqk:2 * nqk], proj[:, 2 * nqk:2 * nqk + nv], proj[:, 2 * nqk + nv:2 * nqk + nv + H],
            dec, w["q.conv"], w["k.conv"], w["v.conv"], w["A_log"], w["dt_bias"], fstate, par.q_cu_seq_lens, pos,
            par.token_seq, par.state_slots, H, G, dim, vdim, 1e-6)
        o = kernels.gated_delta_scan(q, k, v, decay, beta, gate, w["norm"], state, par.q_cu_seq_lens, pos,
                                     par.state_slots, eps, 16 if step % 2 else 1)      # both ends of the walk
        got[0].append(o[:ns[0]].cpu())
        got[1].append(o[ns[0]:].cpu())
        at[0] += ns[0]
        at[1] += ns[1]
    assert bool((state[1] == 5.0).all()) and (taps == 1 or bool((fstate[1] == 5.0).all()))   # the unused slot
    tol = 2e-4 if dtype == torch.float32 else 5e-2
    for s in plans:
        g_ = torch.cat(got[s]).double()
        assert float((g_ - want[s]).abs().max()) < tol * max(1.0, float(want[s].abs().max())), s


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_delta_rule_decodes_long(dtype):
    """300 single tokens after a short portion against the same rows in one portion."""
    from scalellm_b200 import kernels
    H, G, dim, vdim, taps, n = 2, 1, 16, 24, 4, 305
    proj, dec, gate, w = _delta_inputs(H, G, dim, vdim, taps, n, 7, dtype)
    want = _delta_oracle(proj, dec, gate, w, H, G, dim, vdim, {}, 1e-5)[0]
    wd = {k: v.to(DEV) for k, v in w.items()}
    nqk, nv = G * dim, H * vdim
    outs = {}
    for name, cuts in (("whole", [n]), ("decoded", [5] + [1] * (n - 5))):
        state = torch.zeros((1, H, dim, vdim), dtype=torch.float32, device=DEV)
        fstate = torch.zeros((1, taps - 1, 2 * nqk + nv), dtype=torch.float32, device=DEV)
        at, out = 0, []
        for c in cuts:
            (tok, pos, par), hb = _params([c], [at], slots=[0])
            p, d_, g_ = (t[at:at + c].to(DEV) for t in (proj, dec, gate))
            q, k, v, decay, beta = kernels.gated_delta_prepare(
                p[:, :nqk], p[:, nqk:2 * nqk], p[:, 2 * nqk:2 * nqk + nv], p[:, 2 * nqk + nv:2 * nqk + nv + H], d_,
                wd["q.conv"], wd["k.conv"], wd["v.conv"], wd["A_log"], wd["dt_bias"], fstate, par.q_cu_seq_lens, pos,
                par.token_seq, par.state_slots, H, G, dim, vdim, 1e-6)
            out.append(kernels.gated_delta_scan(q, k, v, decay, beta, g_, wd["norm"], state, par.q_cu_seq_lens, pos,
                                                par.state_slots, 1e-5, c).cpu())
            at += c
        outs[name] = torch.cat(out).double()
        tol = 3e-4 if dtype == torch.float32 else 5e-2
        assert float((outs[name] - want).abs().max()) < tol * max(1.0, float(want.abs().max())), name


# ------------------------------------------------------------------ the model
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(fc.CONFIGS))
def test_whole_prompt_layers_and_logits(name, dtype):
    cfg = fc.CONFIGS[name]
    model, oracle = build(cfg, dtype)
    eng = engine_for(model)
    tokens = toks(75, cfg["vocab"], 1)
    lo = []
    want = oracle.forward(tokens, oracle.new_state(), lo)
    from scalellm_b200.decode_step import build_step_batch
    s = eng.open("x")
    eng.pool.reserve(s.seq, len(tokens))
    hb = build_step_batch(eng.pool, [s.seq], [tokens], [0], [s.slot])
    tok, pos, par = eng.bufs.upload(hb)
    got_layers = []
    got = model.forward(tok, pos, par, layer_out=got_layers)
    assert len(got_layers) == len(lo) == len(cfg["layers"])
    for a, b in zip(got_layers, lo):
        if dtype == torch.float32:
            assert float((a.cpu().double() - b).abs().max()) < 2e-4 * float(b.abs().max())
        else:                 # per row, as for the logits: a token whose last expert differs may be off
            e = (a.cpu().double() - b).abs().amax(dim=1) / float(b.abs().max())
            assert float(e.median()) < 0.02 and int((e > 0.05).sum()) <= max(2, e.numel() // 10)
    assert_logits(got, want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(fc.CONFIGS))
def test_prefill_decode_and_portions_agree_with_the_oracle(name, dtype):
    cfg = fc.CONFIGS[name]
    model, oracle = build(cfg, dtype, seed=1)
    tokens = toks(90, cfg["vocab"], 2)
    want = oracle_logits(oracle, tokens)
    for cuts in ([90], [58], [1] * 3, [2, 2, 5, 2, 31, 1, 2, 17, 2], [7] * 13, [33, 4, 4, 4, 40]):
        eng = engine_for(model, block_size=4)
        got = run_schedule(eng, tokens, cuts)
        assert_logits(got, want, dtype, cuts)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_portions_over_many_key_tiles_and_blocks(dtype):
    """Portions cut at places that are no multiple of a key tile, a cache block or a block of positions."""
    cfg = fc.CONFIGS["plain"]                 # one layer without a block limit, one with blocks of 64
    model, oracle = build(cfg, dtype, seed=6)
    tokens = toks(333, cfg["vocab"], 7)
    want = oracle_logits(oracle, tokens)
    for cuts in ([333], [150, 2, 181], [129, 130, 71], [63, 1, 1, 64, 100]):
        eng = engine_for(model, max_tokens=400, block_size=16)
        got = run_schedule(eng, tokens, cuts)
        assert_logits(got, want, dtype, cuts)


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixed_batches_with_reused_blocks_and_slots(dtype):
    """Five unequal requests through a pool and state slots for three: portions beside single tokens, requests that
    pause, blocks and slots handed on without being cleared."""
    from scalellm_b200.engine import StepEntry
    cfg = fc.CONFIGS["mix"]
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
        assert_logits(torch.cat(got[k]), want[k], dtype, k)
    for k in ("a", "e"):       # each request alone gives the same rows as in the batch, beyond rounding
        alone = run_schedule(engine_for(model, max_tokens=128, block_size=4, max_seqs=3), T[k], [lens[k]], rid=k)
        assert_logits(torch.cat(got[k]), alone, dtype)
    assert eng.pool.n_free_blocks() == 32 and len(eng.slots.free) == 3 and not eng.seqs


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_over_small_blocks(dtype):
    cfg = fc.CONFIGS["mix"]
    model, oracle = build(cfg, dtype, seed=3)
    tokens = toks(150, cfg["vocab"], 4)
    want = oracle_logits(oracle, tokens)
    eng = engine_for(model, max_tokens=160, block_size=2)
    got = run_schedule(eng, tokens, [3])
    assert_logits(got, want, dtype)


def test_graph_replay_of_single_token_steps():
    cfg = fc.CONFIGS["mix"]
    model, oracle = build(cfg, torch.bfloat16, seed=4)
    tokens = toks(40, cfg["vocab"], 5)
    want = oracle_logits(oracle, tokens)
    eng = engine_for(model, block_size=4, use_graphs=True)
    got = run_schedule(eng, tokens, [6])
    assert eng._graphs, "no graph was captured"
    assert_logits(got, want, torch.bfloat16)


def test_greedy_generation_through_the_scheduler():
    """More requests than places; the ids must be those of greedy decoding with the oracle wherever its two best
    logits are not a near tie."""
    from scalellm_b200.engine import SamplingParams
    cfg = fc.CONFIGS["plain"]
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
    cfg = fc.CONFIGS["odd"]
    w = fc.weights(cfg, 8)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(fc.public(cfg), f)
    checkpoint.write_safetensors(str(tmp_path / "model.safetensors"), w)
    model = registry.load_model(str(tmp_path), torch.float32, DEV, max_seqs=2)
    tokens = toks(30, cfg["vocab"], 9)
    got = run_schedule(engine_for(model, max_tokens=64, block_size=16, max_seqs=2), tokens, [11, 2])
    assert fc.logits_error(got, oracle_logits(of.Fesupel(cfg, w), tokens)) < TOL[torch.float32]
