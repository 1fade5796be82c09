"""Fekulix without a GPU: the configuration and what it maps onto, sizes taken from a checkpoint's
shapes, a mixer's several cache needs in the cache manager, and the oracle's functions against other
statements of the same formulas."""

import json
import math

import pytest
import torch

from miniserve_b200.cache import CacheManager
from miniserve_b200.cache.manager import KVEntryView, StateEntryView, group_needs
from miniserve_b200.config import resolve
from miniserve_b200.config.fekulix import FekulixConfig
from miniserve_b200.config.registry import architecture_of, checkpoint_shapes
from miniserve_b200.parts import DecoderModel, FixedState, PagedKV
from tests import fekulix_util as fx
from tests.plain import fekulix_plain as plain


def test_config_maps_onto_parts_and_run_order():
    raw = fx.config_a()
    arch, cfg, spec = resolve(raw)
    assert arch.name == "Fekulix" and isinstance(cfg, FekulixConfig)
    assert [e.layer for e in spec.run_order] == [0, 1, 0, 1] and len(spec.layers) == 2
    assert spec.layers[0].mixer.kind == "parallel" and spec.layers[1].mixer.kind == "gated_delta_rule"
    assert spec.layers[1].feed_forward is None and set(spec.layers[1].norms) == {"norm1"}
    left = spec.layers[0].mixer["branches"][0][1]
    assert left["sink"] and left["out_gate"] == "head_sigmoid" and left["value_dim"] == 16 and left["head_dim"] == 32
    assert left["position"].kind == "rope_pairs" and left["position"]["rotary_dim"] == 8
    assert spec.head["scale"] == 1.5
    model = DecoderModel(spec, torch.bfloat16, "cpu")
    decls = {k: tuple(v.shape) for k, v in model.weight_decls().items()}
    assert decls == fx.tensor_shapes(raw)  # names and shapes as the checkpoint format states them


def test_a_borrower_of_a_borrower_runs_with_the_owner_s_tensors():
    raw = fx.config([fx.parallel_layer(), fx.parallel_layer(weights_of=0), fx.parallel_layer(weights_of=1), fx.delta_layer(ff=40)])
    _, _, spec = resolve(raw)
    assert [e.layer for e in spec.run_order] == [0, 0, 0, 1] and len(spec.layers) == 2


def test_each_run_entry_has_pages_and_state_of_its_own():
    _, _, spec = resolve(fx.config_a())
    model = DecoderModel(spec, torch.bfloat16, "cpu")
    needs = [ec.need for ec in model.entry_caches]
    assert needs[0] == (PagedKV(2, 32, None), FixedState((2, 40, 24), torch.float32))  # keys padded to the larger of 32 and 16
    assert needs[1] == (FixedState((4, 24, 16), torch.float32), FixedState((2, 2 * 2 * 16 + 4 * 24), torch.bfloat16))
    groups, states = group_needs(model.entry_caches)
    assert groups == [(PagedKV(2, 32, None), 2)] and len(states) == 6
    cache = CacheManager(model.entry_caches, 8, 16, 3, device=None)
    v = cache.entry_views
    assert isinstance(v[0], tuple) and isinstance(v[0][0], KVEntryView) and isinstance(v[0][1], StateEntryView)
    assert isinstance(v[1], tuple) and all(isinstance(x, StateEntryView) for x in v[1])
    a, b = cache.new_request(), cache.new_request()
    cache.reserve([(a, 20), (b, 3)])
    assert cache.num_free() == (8 - 2 - 1,) and {a.state_slot, b.state_slot} == {0, 1}
    freed = a.state_slot
    cache.release(a)
    c = cache.new_request()
    assert c.state_slot == freed  # the slot that was given back is used again
    cache.release(b), cache.release(c)
    assert cache.is_idle()
    cache.check_invariants()


def test_a_single_tap_needs_no_convolution_state():
    _, _, spec = resolve(fx.config_b())
    model = DecoderModel(spec, torch.float32, "cpu")
    assert model.entry_caches[2].need == FixedState((3, 16, 8), torch.float32)
    assert model.entry_caches[1].need[1] == FixedState((1, 2 * 2 * 40 + 2 * 12), torch.float32)


def test_ranks_come_from_the_checkpoint(tmp_path):
    raw = fx.config_b()
    folder = fx.write_model(tmp_path / "m", raw, 3)
    stored = json.loads((folder / "config.json").read_text())
    assert "decay_rank" not in json.dumps(stored)
    with pytest.raises(KeyError):
        resolve(stored)  # nothing says the ranks
    shapes = checkpoint_shapes(folder)
    assert shapes == fx.tensor_shapes(raw)
    _, _, spec = resolve(stored, folder)
    assert spec.layers[0].mixer["branches"][1][1]["decay_rank"] == 5
    assert (spec.layers[1].mixer["decay_rank"], spec.layers[1].mixer["gate_rank"]) == (3, 7)
    del stored["layers"][1]["mixer"]["conv"]  # the taps, too, are a tensor's shape if config.json does not say
    assert resolve(stored, folder)[2].layers[1].mixer["conv"] == 2
    assert architecture_of({"architectures": ["Qwen3ForCausalLM"]}).name == "Qwen3ForCausalLM"


@pytest.mark.parametrize("change, error", [
    (lambda r: r["layers"][0].update(type="windowed"), NotImplementedError),
    (lambda r: r["layers"][0]["mlp"].update(kind="experts"), NotImplementedError),
    (lambda r: r["layers"][2].update(weights_of=1), ValueError),   # another kind of layer
    (lambda r: (r["layers"][1].update(weights_of=3), r["layers"][3].update(weights_of=1)), ValueError),   # borrowers in a circle
    (lambda r: r["layers"][3].update(weights_of=7), ValueError),
    (lambda r: r["layers"][0]["mixer"]["left"].update(kv_heads=3), ValueError),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"].update(dims=34), ValueError),
    (lambda r: r.pop("width"), KeyError),
])
def test_bad_configurations_are_refused(change, error):
    raw = fx.config_a()
    change(raw)
    with pytest.raises(error):
        resolve(raw)


# --------------------------------------------------------------------------- the oracle against other statements
def test_oracle_sink_attention_is_softmax_over_one_more_key():
    torch.manual_seed(0)
    q, k, v = torch.randn(9, 4, 6, dtype=torch.float64), torch.randn(9, 2, 6, dtype=torch.float64), torch.randn(9, 2, 5, dtype=torch.float64)
    got = plain.sink_attention(q, k, v, 0.3)
    for t in (0, 4, 8):
        for h in range(4):
            s = torch.cat((torch.zeros(1, dtype=torch.float64), (k[:t + 1, h // 2] @ q[t, h]) * 0.3))  # the sink first
            p = torch.softmax(s, 0)[1:]
            assert torch.allclose(got[t, h], p @ v[:t + 1, h // 2], atol=1e-12)


def test_oracle_decay_recurrence_is_a_sum_over_the_past():
    torch.manual_seed(1)
    n, H, dk, dv = 7, 2, 3, 4
    q, k, a = (torch.rand(n, H, dk, dtype=torch.float64) for _ in range(3))
    v = torch.randn(n, H, dv, dtype=torch.float64)
    got = plain.decay_recurrence(q, k, v, a)
    for t in range(n):
        want = torch.zeros(H, dv, dtype=torch.float64)
        for s in range(t + 1):
            w = q[t] * k[s] * a[s + 1:t + 1].prod(dim=0)  # [H, dk]
            want += w.sum(-1, keepdim=True) * v[s]
        assert torch.allclose(got[t], want, atol=1e-12)


def test_oracle_delta_recurrence_without_decay_stores_and_recalls():
    # unit keys that are orthogonal, beta = 1, no decay: reading with a stored key returns its value exactly
    H, dk, dv = 1, 4, 3
    k = torch.eye(4, dtype=torch.float64)[:, None, :]
    v = torch.randn(4, H, dv, dtype=torch.float64)
    out = plain.delta_recurrence(k.clone(), k, v, torch.ones(4, H, dtype=torch.float64), torch.ones(4, H, dk, dtype=torch.float64))
    assert torch.allclose(out, v, atol=1e-12)
    # writing the same key again replaces the value instead of adding to it
    k2 = torch.eye(4, dtype=torch.float64)[[0, 0]][:, None, :]
    out = plain.delta_recurrence(k2.clone(), k2, v[:2], torch.ones(2, H, dtype=torch.float64), torch.ones(2, H, dk, dtype=torch.float64))
    assert torch.allclose(out[1], v[1], atol=1e-12)


def test_oracle_convolution_and_rotation():
    torch.manual_seed(2)
    x, w = torch.randn(6, 5, dtype=torch.float64), torch.randn(5, 3, dtype=torch.float64)
    ref = torch.nn.functional.conv1d(torch.nn.functional.pad(x.T[None], (2, 0)), w[:, None, :], groups=5)[0].T
    assert torch.allclose(plain.causal_conv(x, w), ref, atol=1e-12)
    y = torch.randn(3, 2, 8, dtype=torch.float64)
    r = plain.rotate_pairs(y, torch.tensor([0, 5, 11]), 4, 10.0)
    assert torch.equal(r[0], y[0]) and torch.equal(r[..., 4:], y[..., 4:])
    ang = 11 * 10.0 ** (-2 * 1 / 4)
    assert math.isclose(r[2, 1, 2].item(), y[2, 1, 2].item() * math.cos(ang) - y[2, 1, 3].item() * math.sin(ang), abs_tol=1e-12)
    assert torch.allclose(r.pow(2).sum(-1), y.pow(2).sum(-1))
    assert math.isclose(plain.gelu_tanh(torch.tensor(1.0, dtype=torch.float64)).item(), 0.8411919906082768, abs_tol=1e-12)


def test_oracle_is_causal_and_shared_layers_share(tmp_path):
    folder = fx.write_model(tmp_path / "m", fx.config_a(), 5)
    f = fx.oracle(folder)
    ids = [3, 14, 15, 92, 65, 35, 89, 79, 32, 38]
    assert torch.allclose(f(ids)[:6], f(ids[:6]), atol=1e-10)


def test_preset_writes_a_folder_that_loads_back(tmp_path):
    from miniserve_b200.config import preset
    from miniserve_b200.config.registry import load_config_dict
    from miniserve_b200.weights import load_weights
    from miniserve_b200.weights.random_init import write_model_folder

    folder = write_model_folder(tmp_path / "m", preset("fekulix-tiny"), seed=3, std=0.1)
    _, _, spec = resolve(load_config_dict(folder), folder)
    assert [e.layer for e in spec.run_order] == [0, 1, 0, 1]
    model = DecoderModel(spec, torch.float32, "cpu")
    tensors = load_weights(folder, model.weight_decls(), torch.float32, "cpu", rules=spec.checkpoint_rules, stacks=model.weight_stacks())
    model.bind(tensors)
    logits = fx.oracle(folder)([5, 17, 3])
    assert logits.shape == (3, 503) and torch.isfinite(logits).all()
