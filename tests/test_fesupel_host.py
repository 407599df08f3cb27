"""CPU: host-side parts of the Fesupel path — the plain restatement against itself (whole prompt, token by token,
portions) and its mechanisms by hand, the product's shape table and frequency table against the tests' own, the
registry and a model folder's reader."""
import json
import math

import numpy as np
import torch

from oracle import fesupel as of
from tests import fesupel_case as fc


def toks(n, vocab, seed):
    return [int(x) for x in np.random.default_rng(seed).integers(0, vocab, size=n)]


def test_oracle_whole_equals_token_by_token_and_portions():
    for name, cfg in fc.CONFIGS.items():
        m = of.Fesupel(cfg, fc.weights(cfg, 1))
        tokens = toks(40, cfg["vocab"], 3)
        whole = m.forward(tokens, m.new_state())
        st, rows = m.new_state(), []
        for t in tokens:
            rows.append(m.forward([t], st))
        assert float((torch.cat(rows) - whole).abs().max()) < 1e-9, name
        st, rows, at = m.new_state(), [], 0
        for n in (7, 2, 1, 19, 11):
            rows.append(m.forward(tokens[at:at + n], st))
            at += n
        assert float((torch.cat(rows) - whole).abs().max()) < 1e-9, name


def test_oracle_mechanisms_by_hand():
    # blocks of positions are counted from 0: position 12 with blocks of 5 sees 10 .. 12, position 10 only itself
    assert [j for j in range(20) if of.block_visible(12, j, 5)] == [10, 11, 12]
    assert [j for j in range(20) if of.block_visible(10, j, 5)] == [10]
    assert [j for j in range(20) if of.block_visible(9, j, 5)] == [5, 6, 7, 8, 9]
    assert [j for j in range(6) if of.block_visible(3, j, 0)] == [0, 1, 2, 3]
    # the turn keeps the length of every pair (t, t + dims / 2), leaves the rest alone, is the identity at position 0,
    # and makes q . k depend on the distance only
    rot = {"base": 100.0, "dims": 4}
    x = torch.randn(5, 2, 6, dtype=torch.float64)
    r = of.turn_half(x, torch.arange(5), rot)
    for a in range(2):
        assert torch.allclose(r[..., a] ** 2 + r[..., a + 2] ** 2, x[..., a] ** 2 + x[..., a + 2] ** 2)
    assert torch.equal(r[..., 4:], x[..., 4:]) and torch.allclose(r[0], x[0])
    q, k = torch.randn(1, 1, 4, dtype=torch.float64), torch.randn(1, 1, 4, dtype=torch.float64)
    d1 = (of.turn_half(q, torch.tensor([9]), rot) * of.turn_half(k, torch.tensor([4]), rot)).sum()
    d2 = (of.turn_half(q, torch.tensor([25]), rot) * of.turn_half(k, torch.tensor([20]), rot)).sum()
    assert abs(float(d1 - d2)) < 1e-12
    # frequency bands: short wavelengths kept, long ones divided by the factor, a ramp between
    sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}
    plain = of.turn_frequencies({"base": 10000.0, "dims": 16})
    scaled = of.turn_frequencies({"base": 10000.0, "dims": 16, "scaling": sc})
    for f, s in zip(plain, scaled):
        wl = 2 * math.pi / f
        if wl < 16:
            assert s == f
        elif wl > 64:
            assert abs(s - f / 4.0) < 1e-15
        else:
            assert f / 4.0 <= s <= f
    # sigmoid weights are not normalised: two equal keys give twice the value; the head mix is a plain matrix product
    K = torch.ones(2, 1, 2, dtype=torch.float64)
    V = torch.tensor([[[3.0]], [[3.0]]], dtype=torch.float64)
    qq = torch.ones(1, 2, 2, dtype=torch.float64)
    hb = torch.tensor([0.5, -0.5], dtype=torch.float64)
    o = of.sigmoid_attend(qq, K, V, torch.tensor([1]), 0.25, 0.0, hb, None, 0)
    assert abs(float(o[0, 0, 0]) - 6.0 / (1 + math.exp(-1.0))) < 1e-12 and abs(float(o[0, 1, 0]) - 6.0 / (1 + math.exp(0.0))) < 1e-12
    T = torch.tensor([[0.0, 1.0], [2.0, 0.0]], dtype=torch.float64)
    o2 = of.sigmoid_attend(qq, K, V, torch.tensor([1]), 0.25, 0.0, hb, T, 0)
    assert abs(float(o2[0, 0, 0] - o[0, 1, 0])) < 1e-12 and abs(float(o2[0, 1, 0] - 2 * o[0, 0, 0])) < 1e-12
    # the cap bounds the score
    o3 = of.sigmoid_attend(qq * 100, K, V, torch.tensor([0]), 1.0, 2.0, hb * 0, None, 0)
    assert abs(float(o3[0, 0, 0]) - 3.0 / (1 + math.exp(-2.0))) < 1e-9
    # the short filter: last column is the current token's, zeros before the start, state = the last inputs
    st = {}
    x = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)
    y = of.short_filter(x, w, st, "c")
    assert y[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0] and st["c"][:, 0].tolist() == [4.0, 5.0]
    assert of.short_filter(torch.tensor([[6.0]], dtype=torch.float64), w, st, "c")[0, 0] == 456.0
    # the delta rule with beta 1 and no decay stores v under a unit key exactly, and reads it back with q = k
    S = torch.zeros(3, 2, dtype=torch.float64)
    k1 = torch.tensor([[1.0, 0.0, 0.0]], dtype=torch.float64)
    v1 = torch.tensor([[5.0, -2.0]], dtype=torch.float64)
    one = torch.ones(1, dtype=torch.float64)
    o = of.delta_scan(k1, k1, v1, one, torch.ones(1, 3, dtype=torch.float64), S)
    assert torch.equal(o, v1)
    # writing the same key again with another value replaces it; a decay of 1/2 halves what was there first
    o = of.delta_scan(k1, k1, v1 * 3, one, torch.full((1, 3), 0.5, dtype=torch.float64), S)
    assert torch.equal(o, v1 * 3) and torch.equal(S[0], v1[0] * 3)
    # routing: the correction chooses, the probabilities weigh; a group that is dropped cannot be chosen even when all
    # choice scores are negative
    h = torch.eye(4, dtype=torch.float64)[:1]
    R = torch.tensor([[0.0, 0, 0, 0], [1.0, 0, 0, 0], [2.0, 0, 0, 0], [3.0, 0, 0, 0]], dtype=torch.float64)
    p = torch.softmax(torch.tensor([0.0, 1.0, 2.0, 3.0], dtype=torch.float64), 0)
    ids, wts = of.route(h, R, torch.tensor([0.9, 0.0, 0.0, 0.0], dtype=torch.float64), {"experts": 4, "top": 2})
    assert sorted(ids[0].tolist()) == [0, 3]
    assert abs(float(wts[0].sum()) - 1.0) < 1e-12 and abs(float(wts[0].max()) - float(p[3] / (p[3] + p[0]))) < 1e-12
    ids, _ = of.route(h, R, torch.full((4,), -5.0, dtype=torch.float64),
                      {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}})
    assert sorted(ids[0].tolist()) == [2, 3]
    ids, _ = of.route(h, R, torch.tensor([-5.0, -5.0, -9.0, -9.0], dtype=torch.float64),
                      {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}})
    assert sorted(ids[0].tolist()) == [0, 1]
    # a pass-through expert returns its input: with every chosen output pass-through the layer is the identity
    mlp = fc.moe(1, 1, 4, identity=1)
    w = {"router": torch.tensor([[-50.0, 0, 0, 0], [50.0, 0, 0, 0]], dtype=torch.float64),
         "e0.gate": torch.randn(4, 4, dtype=torch.float64), "e0.up": torch.randn(4, 4, dtype=torch.float64),
         "e0.down": torch.randn(4, 4, dtype=torch.float64)}
    hh = torch.tensor([[1.0, 2.0, 3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(of.moe_ff(hh, w, mlp), hh)
    # the expert clamps its gate from above only and its linear part on both sides
    big = of.clamped_expert(torch.tensor([[10.0]], dtype=torch.float64), torch.ones(1, 1, dtype=torch.float64),
                            torch.ones(1, 1, dtype=torch.float64), torch.ones(1, 1, dtype=torch.float64), 2.0)
    assert abs(float(big) - 2.0 / (1 + math.exp(-1.702 * 2.0)) * 3.0) < 1e-12
    neg = of.clamped_expert(torch.tensor([[-10.0]], dtype=torch.float64), torch.ones(1, 1, dtype=torch.float64),
                            torch.ones(1, 1, dtype=torch.float64), torch.ones(1, 1, dtype=torch.float64), 2.0)
    assert abs(float(neg) - (-10.0) / (1 + math.exp(17.02)) * (-1.0)) < 1e-12


def test_product_shape_and_frequency_tables_agree_with_the_tests_own():
    from scalellm_b200 import fesupel
    for name, cfg in fc.CONFIGS.items():
        assert fesupel.tensor_shapes(fc.public(cfg), lowrank=cfg["_lowrank"]) == fc.shapes(cfg), name
        for L in cfg["layers"]:
            rot = L["mixer"]["left"].get("rot")
            f, dims = fesupel.rotary_table(rot)
            if not rot:
                assert f is None and dims == 0
                continue
            want = torch.tensor(of.turn_frequencies(rot), dtype=torch.float64)
            assert dims == rot["dims"] and float((f.double() - want).abs().max() / want.max()) < 1e-7
    w = fesupel.random_tensors(fc.public(fc.CONFIGS["mix"]), seed=1)
    assert all(t.dtype == torch.bfloat16 for t in w.values())
    m = of.Fesupel(fc.CONFIGS["mix"], w)                 # the product's generator makes weights the restatement runs
    assert bool(torch.isfinite(m.forward(toks(12, 97, 0), m.new_state())).all())


def test_registry_and_model_folder(tmp_path):
    from scalellm_b200 import checkpoint, fesupel, registry
    cfg = fc.CONFIGS["plain"]
    assert registry.model_class(fc.public(cfg)) is fesupel.FesupelDecoder
    w = fc.weights(cfg, 2)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(fc.public(cfg), f)
    checkpoint.write_safetensors(str(tmp_path / "model.safetensors"), w)
    back = checkpoint.read_safetensors(str(tmp_path / "model.safetensors"), "cpu")
    assert set(back) == set(w) and all(torch.equal(back[k], w[k]) for k in w)
    assert checkpoint.read_config(str(tmp_path))["architecture"] == "Fesupel"
