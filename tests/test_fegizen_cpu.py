"""No device needed: the Fegizen reader in the model registry (a checkpoint directory opens on the host), refused
configurations, and the oracle's own rules on hand-worked cases."""
import numpy as np
import pytest

import fegizen_oracle as O
from yalm_b200 import api


def three_layers():
    return O.make_config([
        ("latent_attention", O.latent_mixer(), O.moe_mlp()),
        ("gla", O.gla_mixer(), O.dense_mlp()),
        ("latent_attention", O.latent_mixer(heads=2, window=5, kv_from=0), None)], width=40, vocab=50)


def test_directory_checkpoint_opens_through_the_registry(tmp_path):
    cfg = three_layers()
    folder = str(tmp_path / "m")
    O.write_checkpoint(folder, cfg, O.make_weights(cfg, 1))
    m = api.Model(folder, 0, api.F32)
    assert m.is_stack() and (m.dim, m.vocab_size, m.n_layers) == (40, 50, 3)
    assert (m.n_experts, m.n_experts_active, m.hidden_dim, m.weight_dtype) == (5, 2, 48, api.F32)
    assert m.n_heads * m.head_dim >= 4 * (24 + 8)     # scratch covers the queries against the cached rows
    assert m.max_seq_len >= 1 << 20                   # nothing but the caller bounds the context
    m.close()
    m = api.Model(folder, 4096)
    assert m.weight_dtype == api.BF16 and m.max_seq_len == 4096
    m.close()


@pytest.mark.parametrize("edit,what", [
    (lambda c: c["layers"][0].update(type="attention"), "a layer type of another design"),
    (lambda c: c["canon"].update(taps=0), "no convolution taps"),
    (lambda c: c["layers"][0]["mixer"].update(q_rank=0), "no query latent"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "odd rotated size"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "more rotated channels than the rotated part has"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(factor=0.0), "scaling without a factor"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "a shared cache that is no latent-attention layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "a shared cache that is not an earlier layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=16), "a shared cache of another size"),
    (lambda c: c["layers"][1]["mixer"].update(tau=0.0), "no decay temperature"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=8), "more selected than router outputs"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "unknown feed-forward kind"),
])
def test_bad_configurations_are_refused(tmp_path, edit, what):
    cfg = three_layers()
    W = O.make_weights(cfg, 2)
    edit(cfg)
    folder = str(tmp_path / "m")
    O.write_checkpoint(folder, cfg, W)
    with pytest.raises(api.YalmError) as e:
        api.Model(folder)
    assert e.value.code == -3, what


def test_rotation_on_worked_cases():
    f, mag = O.rotary_table({"dims": 4, "base": 100.0})
    assert f.tolist() == [1.0, 0.1] and mag == 1.0
    x = np.array([1.0, 0.0, 0.0, 2.0, 7.0])                       # two pairs, one channel that passes unchanged
    y = O.rotate_pairs(x, 3, f, 1.0)
    np.testing.assert_allclose(y, [np.cos(3), np.sin(3), -2 * np.sin(0.3), 2 * np.cos(0.3), 7.0], atol=1e-12)
    np.testing.assert_allclose(O.rotate_pairs(x, 0, f, 0.5), [0.5, 0.0, 0.0, 1.0, 7.0])


def test_convolution_starts_from_zero_and_adds_its_input():
    x = np.arange(12.0).reshape(4, 3)
    w = np.array([[1.0, 10.0, 100.0]] * 3)
    out = O.causal_conv(x, w)
    assert out[0].tolist() == (100 * x[0]).tolist() and out[2].tolist() == (x[0] + 10 * x[1] + 100 * x[2]).tolist()
    assert O.with_conv(x, w)[1].tolist() == (10 * x[0] + 101 * x[1]).tolist()


def test_router_on_a_worked_case():
    f = {"router": {"experts": 2, "identity": 2, "top": 2, "scale": 3.0}}
    w = {"r.router": np.eye(4), "r.correction": np.array([0.0, 0.0, 0.5, 0.0])}
    h = np.log(np.array([[0.4, 0.3, 0.2, 0.1]]))                  # softmax gives these scores back
    ids, ws = O.route(h, f, w, "r.")
    assert ids.tolist() == [[2, 0]]                                # 0.2 + 0.5 beats 0.4; the weights use the scores alone
    np.testing.assert_allclose(ws, [[3.0 * 0.2 / 0.6, 3.0 * 0.4 / 0.6]])
    x = np.array([[1.0, -2.0, 0.5, 4.0]])
    cfgw = dict(w)
    for e in range(2):
        cfgw["r.e%d.gate" % e], cfgw["r.e%d.up" % e], cfgw["r.e%d.down" % e] = np.eye(4), np.eye(4), np.zeros((4, 4))
    out = O.moe(h, f, cfgw, "r.")
    np.testing.assert_allclose(out, 1.0 * h)                        # the identity expert returns its input times its weight; expert 0 returns zero


def test_linear_attention_state_on_a_worked_case():
    q = np.array([[[1.0, 0.0]], [[0.0, 1.0]], [[1.0, 1.0]]])
    k = np.array([[[1.0, 0.0]], [[0.0, 1.0]], [[0.0, 0.0]]])
    v = np.array([[[2.0]], [[3.0]], [[5.0]]])
    a = np.full((3, 1, 2), 0.5)
    o = O.gla_scan(q, k, v, a)
    assert o[:, 0, 0].tolist() == [2.0, 3.0, 0.25 * 2.0 + 0.5 * 3.0]


def test_weighted_sum_over_depth_feeds_the_next_layer():
    cfg = O.make_config([("gla", O.gla_mixer(), None), ("gla", O.gla_mixer(), None)], width=16, vocab=20)
    W = O.make_weights(cfg, 3)
    toks = [1, 5, 7, 2]
    _, after = O.forward(cfg, W, toks)
    W2 = {k: np.array(v) for k, v in W.items()}
    W2["l1.dwa"] = np.array([1.0, 0.0, 0.0], np.float32)           # the last layer hands on the embedding output alone
    lg2, after2 = O.forward(cfg, W2, toks)
    x0 = W["embed"][toks].astype(np.float64) * cfg["embedding"]["scale"]
    np.testing.assert_allclose(after2[1], x0)
    np.testing.assert_allclose(after2[0], after[0])
