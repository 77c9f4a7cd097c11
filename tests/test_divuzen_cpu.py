"""Divuzen without a GPU: the configuration and its errors, the model as data, tensor names and shapes,
what the layers ask of the cache (Python and C++ managers), and the plain implementation's own pieces."""
import copy
import math

import pytest
import torch

import divuzen_cases as dc
import plain_divuzen as pd
from divuzen_cases import CASES
from rllm_b200.cache import CacheManager
from rllm_b200.cache.native import NativeCacheManager
from rllm_b200.config import ConfigError, DivuzenConfig, config_from_dict
from rllm_b200.csrc import ops
from rllm_b200.models.model import DecoderModel, expected_tensors
from rllm_b200.parts import PagedKVNeed, Runtime, StateNeed


@pytest.mark.parametrize("name", list(CASES))
def test_configuration_round_trip_and_tensor_list(name):
    cfg = CASES[name]
    c = config_from_dict(cfg)
    assert isinstance(c, DivuzenConfig)
    assert config_from_dict(c.to_dict()) == c
    exp = expected_tensors(c.model_spec())
    want = dc.tensor_shapes(cfg)
    assert set(exp) == set(want)
    for n, (shape, _) in want.items():
        assert tuple(exp[n][0]) == tuple(shape), n


def test_the_model_as_data():
    spec = config_from_dict(CASES["stack"]).model_spec()
    assert [ls.block for ls in spec.layers] == ["sandwich_norm"] * 5
    assert [ls.mixer.kind for ls in spec.layers] == ["retention", "attention", "retention", "attention", "attention"]
    assert [None if ls.ffn is None else ls.ffn.kind for ls in spec.layers] == \
        ["clamped_glu", "routed_experts", "routed_experts", "clamped_glu", None]
    assert [e.cache_of for e in spec.run_order] == [None, None, None, 1, None]
    a = spec.layers[3].mixer.params
    assert a["own_kv"] is False and a["sink"] and a["v_head_dim"] == 16 and a["head_dim"] == 32
    assert spec.layers[1].position.params["layout"] == "pairs" and spec.layers[0].position.params["layout"] == "half"
    r = spec.layers[0].mixer.params
    assert r["key_scale"] == 16 ** -0.5 and r["decay"] == (0.9, 0.95, 0.99, 0.999)
    m = spec.layers[1].ffn.params
    assert (m["num_experts"], m["top_k"], m["n_groups"], m["keep_groups"], m["shared_size"]) == (8, 3, 4, 2, 40)
    assert m["route_scale"] == 2.5 and m["group_best"] == 2 and m["weight_eps"] == 1e-20
    assert spec.layers[2].ffn.params["shared_size"] == 0
    assert spec.lm_head.params["scale"] == 0.4 and spec.lm_head.params["tied_to"] == "embed"
    assert all(n.params["one_plus"] for ls in spec.layers for n in ls.norms.values()) and spec.final_norm.params["one_plus"]
    assert set(spec.layers[4].norms) == {"mixer", "mixer_out"}


def _broken(name, edit):
    cfg = copy.deepcopy(CASES[name])
    edit(cfg)
    return cfg


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0]["mixer"].pop("decay"), "decay"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=64), "dims"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "kv_heads"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=0), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(vdim=8), "reads"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][0]["mlp"].update(kind="gelu"), "kind"),
    (lambda c: c["layers"][0].update(type="mamba"), "type"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configuration_errors_name_the_key(edit, word):
    with pytest.raises(ConfigError) as e:
        config_from_dict(_broken("stack", edit))
    assert word in str(e.value)


@pytest.mark.parametrize("manager", [CacheManager, NativeCacheManager])
def test_what_the_layers_ask_of_the_cache(manager):
    spec = config_from_dict(CASES["stack"]).model_spec()
    model = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32))
    needs, cache_of = model.cache_needs()
    assert needs[1] == needs[3] == PagedKVNeed(2, 32, 0, 0, 16) and needs[4] == PagedKVNeed(1, 8)
    assert needs[0] == StateNeed((ops.retention_state_floats(4, 16, 24),))
    assert needs[2] == StateNeed((ops.retention_state_floats(2, 24, 40),))
    cm = manager(needs, cache_of, block_size=8, max_tokens=64, max_requests=2)
    assert cm.entry_place[3] == cm.entry_place[1] and cm.entry_place[4] != cm.entry_place[1]
    assert len(cm.paged) == 2 and len(cm.stateful) == 2
    cm.append("a", 20)
    cm.append("b", 3)
    assert cm.state_slot("a") != cm.state_slot("b")
    cm.free("a")
    cm.append("c", 9)
    cm.check_invariants()


def test_state_sizes_follow_the_kernel_tiles():
    assert ops.retention_state_floats(1, 8, 12) == 32 * 16
    assert ops.retention_state_floats(3, 48, 40) == 3 * 64 * 40
    assert ops.retention_state_floats(2, 128, 136) == 2 * 128 * 136
    assert ops.retention_state_floats(1, 129, 2) == 256 * 8


# ---------------------------------------------------------------- the plain implementation's own pieces

def test_plain_rotations_keep_lengths_and_differ_in_layout():
    g = torch.Generator().manual_seed(1)
    v = torch.randn(5, 2, 12, generator=g, dtype=torch.float64)
    a, b = pd.rotate_pairs(v, 8, 100.0), pd.rotate_half(v, 8, 100.0)
    assert torch.allclose(a.norm(dim=-1), v.norm(dim=-1)) and torch.allclose(b.norm(dim=-1), v.norm(dim=-1))
    assert torch.equal(a[0], v[0]) and torch.equal(a[..., 8:], v[..., 8:]) and torch.equal(b[..., 8:], v[..., 8:])
    ang = 3 * 100.0 ** (-2 / 8)                  # position 3, pair 1
    c, s = math.cos(ang), math.sin(ang)
    assert torch.allclose(a[3, 0, 2], v[3, 0, 2] * c - v[3, 0, 3] * s) and torch.allclose(a[3, 0, 3], v[3, 0, 3] * c + v[3, 0, 2] * s)
    assert torch.allclose(b[3, 0, 1], v[3, 0, 1] * c - v[3, 0, 5] * s) and torch.allclose(b[3, 0, 5], v[3, 0, 5] * c + v[3, 0, 1] * s)


def test_plain_retention_is_the_decayed_sum():
    """o_t = sum_{j <= t} c^(t-j) (q_t . k_j) v_j, written out, equals the recurrence."""
    cfg = CASES["retention"]
    w = {k: v.double() for k, v in dc.make_weights(cfg, 2).items()}
    mx = cfg["layers"][0]["mixer"]
    g = torch.Generator().manual_seed(3)
    h = torch.randn(9, cfg["width"], generator=g, dtype=torch.float64)
    T, H, dk, dv = 9, mx["heads"], mx["dim"], mx["vdim"]
    q = pd.rotate_half((h @ w["l0.mix.q"].T).view(T, H, dk), 4, mx["rot"]["base"])
    k = pd.rotate_half((h @ w["l0.mix.k"].T).view(T, H, dk), 4, mx["rot"]["base"]) / math.sqrt(dk)
    v = (h @ w["l0.mix.v"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=torch.float64)
    for head in range(H):
        for t in range(T):
            for j in range(t + 1):
                o[t, head] += mx["decay"][head] ** (t - j) * (q[t, head] @ k[j, head]) * v[j, head]
    gate = h @ w["l0.mix.g"].T
    want = (pd.rms_unit(o, 1e-5).reshape(T, -1) * gate * torch.sigmoid(gate)) @ w["l0.mix.o"].T
    assert torch.allclose(pd.retention(h, w, "l0.mix.", mx, 1e-5), want, rtol=1e-10, atol=1e-12)


def test_plain_router_groups_and_weights():
    r = {"experts": 6, "top": 2, "scale": 3.0, "groups": {"count": 3, "keep": 1}}
    W = {"r.router": torch.eye(6, dtype=torch.float64), "r.correction": torch.tensor([0., 0., 0., 0., -1., 3.], dtype=torch.float64)}
    # scores: sigmoid of the logits; group 2 = experts (4, 5) has choice scores (s4 - 1, s5 + 3): its sum
    # beats the others although expert 4's choice score is negative, and both its experts are chosen
    z = torch.tensor([3.0, 2.5, 3.0, 3.0, 0.0, 0.0], dtype=torch.float64)
    chosen, w = pd.route(z, W, "r.", r)
    assert chosen == [5, 4]
    assert torch.allclose(w, torch.tensor([1.5, 1.5], dtype=torch.float64))
    r["groups"] = {"count": 1, "keep": 1}
    chosen, w = pd.route(z, W, "r.", r)
    s = torch.sigmoid(z)
    assert chosen == [5, 0] and torch.allclose(w, 3.0 * torch.stack([s[5], s[0]]) / (s[5] + s[0]))


def test_plain_attention_sink_takes_its_share():
    cfg = CASES["attention"]
    w = {k: v.double() for k, v in dc.make_weights(cfg, 4).items()}
    mx = cfg["layers"][0]["mixer"]
    g = torch.Generator().manual_seed(5)
    h = torch.randn(6, cfg["width"], generator=g, dtype=torch.float64)
    k, v = pd.attention_keys_values(h, w, "l0.mix.", mx, 1e-5)
    a = pd.attention(h, w, "l0.mix.", mx, 1e-5, k, v)
    w2 = dict(w)
    w2["l0.mix.sink"] = torch.full_like(w["l0.mix.sink"], -1e4)      # no sink to speak of
    b = pd.attention(h, w2, "l0.mix.", mx, 1e-5, k, v)
    # the first token sees one key: without a sink its output is that key's value through Wo
    first = (v[0].repeat_interleave(mx["heads"] // mx["kv_heads"], 0).reshape(-1)) @ w["l0.mix.o"].T
    assert torch.allclose(b[0], first)
    assert float((a[0] - b[0]).abs().max()) > 1e-2 * float(b[0].abs().max())
    w2["l0.mix.sink"] = torch.full_like(w["l0.mix.sink"], 50.0)      # the sink takes everything
    assert float(pd.attention(h, w2, "l0.mix.", mx, 1e-5, k, v).abs().max()) < 1e-12
