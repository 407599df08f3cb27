"""CPU: host-side parts of the Zomurax path — the plain restatement against itself (whole prompt, token by token,
portions) and its mechanisms by hand, the product's shape table and rotary table against the tests' own, the
registry, the checkpoint reader with integer tables."""
import json
import math

import numpy as np
import torch

from oracle import zomurax as oz
from tests import zomurax_case as zc


def toks(n, vocab, seed):
    return [int(x) for x in np.random.default_rng(seed).integers(0, vocab, size=n)]


def test_oracle_whole_equals_token_by_token_and_portions():
    for name, cfg in zc.CONFIGS.items():
        m = oz.Zomurax(cfg, zc.weights(cfg, 1))
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
    # the window: position 12 with size 4 sees 9 .. 12; size 0 is no window
    assert [j for j in range(20) if oz.window_visible(12, j, 4)] == [9, 10, 11, 12]
    assert [j for j in range(5) if oz.window_visible(2, j, 4)] == [0, 1, 2]
    assert [j for j in range(5) if oz.window_visible(3, j, 0)] == [0, 1, 2, 3]
    # the temperature steps when (p + 1) reaches a multiple of `every`
    t = oz.query_temperature(torch.arange(10), {"coef": 0.5, "every": 4})
    assert t[:3].tolist() == [1.0, 1.0, 1.0] and abs(float(t[3]) - (1.0 + 0.5 * math.log(2.0))) < 1e-12
    assert float(t[6]) == float(t[3]) and abs(float(t[7]) - (1.0 + 0.5 * math.log(3.0))) < 1e-12
    assert oz.query_temperature(torch.arange(4), None).tolist() == [1.0] * 4
    # the turn keeps the length of every pair (t, t + dims / 2), leaves the rest alone, and is the identity at 0
    rot = {"base": 100.0, "dims": 4}
    x = torch.randn(5, 2, 6, dtype=torch.float64)
    r = oz.turn_half(x, torch.arange(5), rot)
    for a in range(2):
        assert torch.allclose(r[..., a] ** 2 + r[..., a + 2] ** 2, x[..., a] ** 2 + x[..., a + 2] ** 2)
    assert torch.equal(r[..., 4:], x[..., 4:]) and torch.allclose(r[0], x[0])
    # relative: the product of a turned query and a turned key depends on the distance only
    q, k = torch.randn(1, 4, dtype=torch.float64), torch.randn(1, 4, dtype=torch.float64)
    d1 = oz.turn_half(q, torch.tensor([9]), rot) @ oz.turn_half(k, torch.tensor([4]), rot).T
    d2 = oz.turn_half(q, torch.tensor([25]), rot) @ oz.turn_half(k, torch.tensor([20]), rot).T
    assert abs(float(d1 - d2)) < 1e-12
    # one key, no bias: the weight of the only key is 1 / (1 + exp(sink - s)); without a sink it is 1
    K = torch.ones(1, 1, 2, dtype=torch.float64)
    V = torch.tensor([[[3.0]]], dtype=torch.float64)
    qq = torch.ones(1, 1, 2, dtype=torch.float64)
    o = oz.sink_attend(qq, K, V, torch.tensor([0]), 0.5, None, None, torch.tensor([0.25], dtype=torch.float64))
    assert abs(float(o) - 3.0 / (1.0 + math.exp(0.25 - 1.0))) < 1e-12
    assert abs(float(oz.sink_attend(qq, K, V, torch.tensor([0]), 0.5, None, None, None)) - 3.0) < 1e-12
    # two equal keys one step apart: the bias r1 ln(1 + r2) tilts the weights
    K2, V2 = torch.ones(2, 1, 2, dtype=torch.float64), torch.tensor([[[1.0]], [[0.0]]], dtype=torch.float64)
    o = oz.sink_attend(qq, K2, V2, torch.tensor([1]), 0.5, torch.tensor([2.0], dtype=torch.float64),
                       torch.tensor([3.0], dtype=torch.float64), None)
    far = math.exp(-2.0 * math.log(4.0))
    assert abs(float(o) - far / (1.0 + far)) < 1e-12
    # the table: a token with two experts gets their mean, plus the shared expert
    W = 4
    eye = torch.eye(W, dtype=torch.float64)
    w = {"table": torch.tensor([[0, 1], [1, 0], [1, 1]], dtype=torch.int32)}
    for e, c in ((0, 1.0), (1, 3.0)):
        w.update({f"e{e}.gate": eye * 50.0, f"e{e}.up": eye * c, f"e{e}.down": eye})
    h = torch.full((1, W), 2.0, dtype=torch.float64)
    out = oz.table_moe(h, [0], w, {"router": {"experts": 2, "top": 2}})      # silu(100) = 100
    assert torch.allclose(out, torch.full((1, W), 0.5 * (100.0 * 2.0 + 100.0 * 6.0), dtype=torch.float64))


def test_shape_table_and_random_weights():
    from scalellm_b200 import zomurax
    for name, cfg in zc.CONFIGS.items():
        assert zomurax.tensor_shapes(cfg) == zc.shapes(cfg), name
        w = zomurax.random_tensors(cfg, 0)
        assert {k: tuple(v.shape) for k, v in w.items()} == zc.shapes(cfg)
        for k, v in w.items():
            if k.endswith(".table"):
                assert v.dtype == torch.int32
                E = cfg["layers"][int(k.split(".")[0][1:])]["mlp"]["router"]["experts"]
                assert int(v.min()) >= 0 and int(v.max()) < E
                assert all(len(set(row)) == len(row) for row in v.tolist())


def test_rotary_table_matches_the_restatement():
    from scalellm_b200 import zomurax
    for rot in ({"base": 10000.0, "dims": 8}, {"base": 1e6, "dims": 64}, {"base": 500.0, "dims": 2}):
        f = zomurax.rotary_table(rot)
        want = torch.tensor([rot["base"] ** (-2.0 * t / rot["dims"]) for t in range(rot["dims"] // 2)], dtype=torch.float64)
        assert f.dtype == torch.float32 and float((f.double() - want).abs().max() / want.abs().max()) < 1e-7


def test_registry_and_model_folder(tmp_path):
    from scalellm_b200 import checkpoint, registry
    cfg = zc.CONFIGS["attn_first"]
    assert registry.architecture_of(cfg) == "Zomurax"
    assert registry.model_class(cfg).__name__ == "ZomuraxDecoder"
    assert registry.model_class(cfg).needs_state_slots is False
    w = zc.weights(cfg, 2)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    checkpoint.write_safetensors(str(tmp_path / "model.safetensors"), w)
    back = checkpoint.read_safetensors(str(tmp_path / "model.safetensors"))
    assert set(back) == set(w)
    for k in w:
        assert back[k].dtype == w[k].dtype and back[k].shape == w[k].shape and torch.equal(back[k], w[k]), k
    assert oz.read_safetensors(str(tmp_path / "model.safetensors"))["l0.mlp.table"].dtype == torch.int32
