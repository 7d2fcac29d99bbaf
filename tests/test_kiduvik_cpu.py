"""No device needed: the Kiduvik reader in the model registry (a checkpoint directory opens on the host), refused
configurations, and the oracle's own rules on hand-worked cases."""
import math

import numpy as np
import pytest

import kiduvik_oracle as O
from yalm_b200 import api


def three_layers():
    return O.make_config([O.latent_mixer(), O.diff_mixer(), dict(O.latent_mixer(heads=2, kv_from=0), mlp=None)], width=40, vocab=50, ff=56, side=4)


def test_directory_checkpoint_opens_through_the_registry(tmp_path):
    cfg = three_layers()
    folder = str(tmp_path / "m")
    O.write_checkpoint(folder, cfg, O.make_weights(cfg, 1))
    m = api.Model(folder, 0, api.F32)
    assert m.is_stack() and (m.dim, m.vocab_size, m.n_layers) == (40, 50, 3)
    assert (m.n_experts, m.hidden_dim, m.weight_dtype) == (0, 56, api.F32)
    assert m.max_seq_len == 512                        # the learned positions bound the context
    m.close()
    m = api.Model(folder, 100)
    assert m.weight_dtype == api.BF16 and m.max_seq_len == 100
    m.close()


@pytest.mark.parametrize("edit,what", [
    (lambda c: c["layers"][0].update(type="gla"), "a layer type of another design"),
    (lambda c: c.update(max_positions=0), "no positions"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "odd rotated size"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10), "more rotated channels than the rotated part has"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "more rotated channels than a head has"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].update(factor=0.0), "scaling without a factor"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "query heads that do not divide over the key heads"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "a shared cache that is no latent-attention layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "a shared cache that is not an earlier layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=16), "a shared cache of another size"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "unknown feed-forward kind"),
    (lambda c: c["layers"][1]["mlp"].update(ff=0), "no hidden size"),
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


def test_half_split_rotation_on_worked_cases():
    f, mag = O.rotary_table({"dims": 4, "base": 100.0})
    assert f.tolist() == [1.0, 0.1] and mag == 1.0
    x = np.array([1.0, 0.0, 0.0, 2.0, 7.0])                       # pairs (0, 2) and (1, 3); the fifth channel passes unchanged
    y = O.rotate_half(x, 3, f, 1.0)
    np.testing.assert_allclose(y, [math.cos(3.0), -2 * math.sin(0.3), math.sin(3.0), 2 * math.cos(0.3), 7.0], atol=1e-12)
    np.testing.assert_allclose(O.rotate_half(x, 0, f, 1.0), x)
    # scaling: slow pairs are divided by the factor, fast ones kept, and the magnitude grows with the factor's logarithm
    f2, mag2 = O.rotary_table({"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}})
    f0, _ = O.rotary_table({"dims": 8, "base": 10000.0})
    assert mag2 == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert f2[0] == f0[0] and f2[-1] == pytest.approx(f0[-1] / 4.0) and all(f0 / 4.0 - 1e-15 <= f2) and all(f2 <= f0)


def test_window_with_kept_first_tokens():
    see = lambda i, size, keep: [j for j in range(i + 3) if O.visible(i, j, size, keep)]
    assert see(2, 4, 0) == [0, 1, 2]
    assert see(9, 4, 0) == [6, 7, 8, 9]
    assert see(9, 4, 2) == [0, 1, 6, 7, 8, 9]
    assert see(4, 4, 2) == [0, 1, 2, 3, 4]                         # kept tokens inside the window count once
    assert see(0, 1, 5) == [0]


def test_sink_and_lambda():
    s = np.array([0.0, math.log(2.0)])
    np.testing.assert_allclose(O.softmax_with_sink(s, None), [1 / 3, 2 / 3])
    np.testing.assert_allclose(O.softmax_with_sink(s, math.log(3.0)), [1 / 6, 2 / 6])      # the sink takes its share and gives nothing back
    np.testing.assert_allclose(O.softmax_with_sink(s + 1000.0, 0.0), [1 / 3, 2 / 3])
    np.testing.assert_allclose(O.softmax_with_sink(s, 1000.0), [0.0, 0.0], atol=1e-300)
    w = {"lq1": np.array([1.0, 2.0]), "lk1": np.array([0.5, 0.0]), "lq2": np.array([0.0, 1.0]), "lk2": np.array([3.0, -1.0])}
    assert O.diff_lambda({"diff": 0.25}, w, "") == pytest.approx(math.exp(0.5) - math.exp(-1.0) + 0.25)


def test_gelu_forms():
    assert O.gelu_erf(np.array([0.0]))[0] == 0.0
    assert O.gelu_erf(np.array([1.0]))[0] == pytest.approx(0.8413447460685429)
    assert O.gelu_tanh(np.array([1.0]))[0] == pytest.approx(0.8411919906082768)
