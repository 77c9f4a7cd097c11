"""Navulorn without a GPU: the configuration and its errors, the model as data, tensor names and shapes,
what the layers and the embedding ask of the cache (Python and C++ managers), state sizes, and the plain
implementation's own pieces."""
import copy
import math

import pytest
import torch

import navulorn_cases as nc
import plain_navulorn as pn
from navulorn_cases import CASES
from rllm_b200.cache import CacheManager
from rllm_b200.cache.native import NativeCacheManager
from rllm_b200.config import ConfigError, NavulornConfig, config_from_dict
from rllm_b200.csrc import ops
from rllm_b200.models.model import DecoderModel, expected_tensors
from rllm_b200.parts import PagedKVNeed, Runtime, StateNeed


@pytest.mark.parametrize("name", list(CASES))
def test_configuration_round_trip_and_tensor_list(name):
    cfg = CASES[name]
    c = config_from_dict(cfg)
    assert isinstance(c, NavulornConfig)
    assert config_from_dict(c.to_dict()) == c
    exp = expected_tensors(c.model_spec())
    want = nc.tensor_shapes(cfg)
    assert set(exp) == set(want)
    for n, (shape, _) in want.items():
        assert tuple(exp[n][0]) == tuple(shape), n


def test_the_model_as_data():
    spec = config_from_dict(CASES["stack"]).model_spec()
    assert [ls.block for ls in spec.layers] == ["sum_norm"] * 6
    assert all(ls.block_params["alpha"] == 2.5 for ls in spec.layers)
    assert [ls.mixer.kind for ls in spec.layers] == ["mlstm", "gated_attention", "latent_attention", "gated_attention",
                                                     "mlstm", "latent_attention"]
    assert [None if ls.ffn is None else ls.ffn.kind for ls in spec.layers] == \
        ["clamped_glu", "routed_experts", "routed_experts", "clamped_glu", "routed_experts", None]
    a = spec.layers[1].mixer.params
    assert (a["qk_norm"], a["gate"], a["gate_per_head"], a["window"], a["v_head_dim"]) == ("row", "sigmoid", True, 13, 16)
    assert spec.layers[1].position.params["layout"] == "half" and spec.layers[2].position.params["layout"] == "pairs"
    assert spec.layers[1].position.params["scaling"] == {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64.0}
    assert spec.layers[0].position is None
    la = spec.layers[2].mixer.params
    assert (la["q_rank"], la["window"], la["kv_rank"], la["rot_dim"]) == (0, 30, 24, 8)
    m = spec.layers[4].mixer.params
    assert m["gate_cap"] == 10.0 and m["q_scale"] == 24 ** -0.5
    f = spec.layers[0].ffn.params
    assert f["activation"] == "gelu_tanh" and f["limit"] == 0.0 and f["shift"] == 0.0
    r = spec.layers[1].ffn.params
    assert (r["num_experts"], r["top_k"], r["score"], r["normalize"], r["router_bias"]) == (8, 3, "softmax", True, True)
    assert spec.embedding.params["scale"] == 4.0 and spec.embedding.params["pair"]["buckets"] == 37
    assert spec.lm_head.params["softcap"] == 20.0 and not spec.lm_head.params.get("tied_to")
    assert set(spec.layers[5].norms) == {"mixer"}
    bare = config_from_dict(CASES["attention_no_window"]).model_spec()
    assert "pair" not in bare.embedding.params and bare.layers[0].mixer.params["window"] == 0


def _broken(name, edit):
    cfg = copy.deepcopy(CASES[name])
    edit(cfg)
    return cfg


@pytest.mark.parametrize("name,edit,word", [
    ("attention", lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    ("attention", lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "dims"),
    ("attention", lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "dims"),
    ("attention", lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "size"),
    ("attention", lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    ("attention_scaled", lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].update(high=1.0), "high"),
    ("attention_scaled", lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("original"), "original"),
    ("latent", lambda c: c["layers"][0]["mixer"].update(rot_dim=6), "rot_dim"),
    ("latent", lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    ("memory", lambda c: c["layers"][0]["mixer"].update(gate_cap=0.0), "gate_cap"),
    ("memory", lambda c: c["layers"][0].update(type="lstm"), "lstm"),
    ("moe", lambda c: c["layers"][0]["mlp"]["router"].update(top=13), "top"),
    ("moe", lambda c: c["layers"][0]["mlp"].update(kind="glu"), "glu"),
    ("moe", lambda c: c["layers"][0]["mlp"].pop("expert"), "expert"),
    ("attention", lambda c: c["embedding"]["bigram"].update(buckets=0), "buckets"),
    ("attention", lambda c: c.pop("norm"), "norm"),
    ("attention", lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
    ("attention", lambda c: c.update(layers=[]), "layers"),
])
def test_configuration_errors_name_the_key(name, edit, word):
    with pytest.raises(ConfigError) as e:
        config_from_dict(_broken(name, edit))
    assert word in str(e.value)


def _needs(name):
    model = DecoderModel(config_from_dict(CASES[name]).model_spec(), Runtime(torch.device("cpu"), torch.float32))
    return model, *model.cache_needs()


def test_what_the_layers_ask_of_the_cache():
    model, needs, owners = _needs("stack")
    assert len(needs) == 7 and owners == [None] * 7                  # six layers and the embedding's last token
    assert needs[6] == StateNeed((1,), torch.int32) and model.embedding_entry == 6
    assert needs[1] == needs[3] == PagedKVNeed(2, 32, 13, 0, 16)
    assert needs[2] == PagedKVNeed(1, 32, window=30, values_in_keys=24)
    assert needs[5] == PagedKVNeed(1, 24, window=11, values_in_keys=16)
    assert needs[0] == StateNeed((ops.mlstm_state_floats(4, 16, 24),), torch.float32)
    assert needs[4] == StateNeed((ops.mlstm_state_floats(2, 24, 40),), torch.float32)
    _, bare, _ = _needs("attention_no_window")
    assert len(bare) == 1 and bare[0] == PagedKVNeed(2, 12, 0, 0, 4)
    _, same, _ = _needs("heads64")
    assert same[0] == PagedKVNeed(2, 64, 21, 0, 0) and same[1] == PagedKVNeed(2, 64, 44, 0, 0)


def test_state_sizes():
    # per head: the key rows rounded up to 32, 64, 128 or 256, times the value columns and the normaliser's
    # column in whole groups of threads, and four scalars
    assert ops.mlstm_state_floats(1, 8, 12) == 32 * 16 + 4
    assert ops.mlstm_state_floats(2, 48, 40) == 2 * (64 * 48 + 4)
    assert ops.mlstm_state_floats(1, 128, 64) == 128 * 72 + 4
    assert ops.mlstm_state_floats(3, 16, 254) == 3 * (32 * 256 + 4)
    assert ops.mlstm_state_floats(2, 16, 255) == 2 * (16 * 256 + 4)          # beyond the fast kernel: as it is
    assert ops.mlstm_state_floats(1, 257, 8) == 257 * 9 + 4
    from rllm_b200.csrc import build
    try:
        lib = build.load("recur")
    except Exception:
        pytest.skip("the recurrent kernels' library cannot be built here")
    lib.rllm_mlstm_state_floats.restype = __import__("ctypes").c_longlong
    for H, dk, dv in ((1, 8, 12), (2, 48, 40), (4, 128, 64), (1, 200, 254), (3, 33, 1), (2, 16, 255), (1, 300, 300)):
        assert lib.rllm_mlstm_state_floats(H, dk, dv) == ops.mlstm_state_floats(H, dk, dv)


@pytest.mark.parametrize("manager", [CacheManager, NativeCacheManager])
def test_both_cache_managers_take_the_model(manager):
    _, needs, owners = _needs("stack")
    cm = manager(needs, owners, 8, 256, 3)
    assert len(cm.paged) == 3 and len(cm.stateful) == 3            # two sizes of memory and the last tokens
    assert [g.need.window for g in cm.paged] == [13, 30, 11]
    slots = cm.append("a", 50)
    assert len(slots) == 3 and all(len(s) == 50 for s in slots)
    before = [cm.n_free_pages(g) for g in range(3)]
    cm.append("a", 150)
    cm.release_passed("a")                                          # the windows have passed most of the 200 tokens
    assert all(cm.n_free_pages(g) > before[g] - 19 for g in range(3))
    cm.append("b", 9)
    assert cm.state_slot("a") != cm.state_slot("b")
    cm.free("a")
    cm.free("b")
    cm.check_invariants()


# ---------------------------------------------------------------- the plain implementation's own pieces

def test_plain_frequencies_follow_the_three_ranges():
    f = pn.frequencies(16, 50.0)
    assert torch.allclose(f, torch.tensor([50.0 ** (-2 * i / 16) for i in range(8)], dtype=torch.float64))
    g = pn.frequencies(16, 50.0, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64})
    wave = 2 * math.pi / f
    for i in range(8):
        if wave[i] < 16:
            assert g[i] == f[i]
        elif wave[i] > 64:
            assert g[i] == f[i] / 8
        else:
            assert f[i] / 8 < g[i] < f[i]
    assert any(16 <= w <= 64 for w in wave) and any(w > 64 for w in wave) and any(w < 16 for w in wave)


def test_plain_rotation_layouts_agree_up_to_the_order_of_entries():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 2, 12, generator=g, dtype=torch.float64)
    pos, f = torch.tensor([0, 1, 2, 30, 31]), pn.frequencies(8, 100.0)
    half = pn.rotate(x, pos, f, 8, "half")
    order = [0, 4, 1, 5, 2, 6, 3, 7, 8, 9, 10, 11]          # entry i of a pair, then its partner
    pairs = pn.rotate(x[..., order], pos, f, 8, "pairs")
    assert torch.allclose(pairs, half[..., order], atol=1e-12)
    assert torch.equal(half[0], x[0]) and torch.equal(half[..., 8:], x[..., 8:])        # position 0 and the rest pass
    assert torch.allclose(half.norm(dim=-1), x.norm(dim=-1), atol=1e-12)


def test_plain_pair_rows():
    assert pn.bigram_rows([3, 4, 3, 3], 7, 5, 2) == [7, (3 * 5 + 4 * 2) % 7, (4 * 5 + 3 * 2) % 7, (3 * 5 + 3 * 2) % 7]


def test_plain_window_counts_the_token_itself():
    q = torch.ones(6, 1, 2, dtype=torch.float64)
    k = torch.ones(6, 1, 2, dtype=torch.float64)
    v = torch.arange(6, dtype=torch.float64).view(6, 1, 1)
    out = pn.window_softmax_attention(q, k, v, 1.0, 3, 1)[:, 0, 0]
    assert torch.allclose(out, torch.tensor([0.0, 0.5, 1.0, 2.0, 3.0, 4.0], dtype=torch.float64))
    assert torch.allclose(pn.window_softmax_attention(q, k, v, 1.0, 1, 1)[:, 0, 0], v[:, 0, 0])
    assert torch.allclose(pn.window_softmax_attention(q, k, v, 1.0, 0, 1)[:, 0, 0],
                          torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 2.5], dtype=torch.float64))


def test_plain_memory_matches_its_closed_form_and_its_first_token():
    """The recurrence against the sum it stands for, o_t = sum_s exp(F_t - F_s + i_s - m_t) (k_s . q) v_s over the
    same denominator, with m_t from the recurrence; and the first token, where m starts at 0."""
    g = torch.Generator().manual_seed(1)
    mx = {"heads": 1, "dim": 4, "vdim": 3, "gate_cap": 5.0}
    d, n = 6, 9
    w = {"m." + k: torch.randn(s, generator=g, dtype=torch.float64) for k, s in
         (("q", (4, d)), ("k", (4, d)), ("v", (3, d)), ("g", (3, d)), ("i", (1, d)), ("f", (1, d)), ("i.b", (1,)), ("f.b", (1,)))}
    w["m.o"], w["m.norm"] = torch.eye(3, dtype=torch.float64), torch.ones(3, dtype=torch.float64)
    h = torch.randn(n, d, generator=g, dtype=torch.float64)
    got = pn.mlstm(h, w, "m.", mx, 1e-6)
    q, k, v = h @ w["m.q"].T / 2.0, h @ w["m.k"].T, h @ w["m.v"].T
    i = 5.0 * torch.tanh((h @ w["m.i"].T + w["m.i.b"]) / 5.0)[:, 0]
    f = torch.nn.functional.logsigmoid(5.0 * torch.tanh((h @ w["m.f"].T + w["m.f.b"]) / 5.0))[:, 0]
    m = 0.0
    for t in range(n):
        m = max(float(f[t]) + m, float(i[t]))
        F = torch.cumsum(f[:t + 1], 0)
        wgt = torch.exp(F[t] - F + i[:t + 1] - m)
        num = ((k[:t + 1] @ q[t]) * wgt) @ v[:t + 1]
        den = max(abs(float(((k[:t + 1] @ q[t]) * wgt).sum())), math.exp(-m)) + 1e-6
        o = num / den
        want = o / torch.sqrt((o * o).mean() + 1e-6) * torch.sigmoid(h[t] @ w["m.g"].T)
        assert torch.allclose(got[t], want, atol=1e-9), t


def test_plain_router_weights_are_a_softmax_over_the_chosen_logits():
    g = torch.Generator().manual_seed(2)
    w = {"r.router": torch.randn(5, 4, generator=g, dtype=torch.float64), "r.router.b": torch.tensor([0., 9., 0., 0., -9.], dtype=torch.float64)}
    h = torch.randn(7, 4, generator=g, dtype=torch.float64)
    margins = []
    idx, wt, z = pn.route(h, w, "r.", 2, margins=margins)
    assert all(1 in row for row in idx.tolist()) and all(4 not in row for row in idx.tolist())     # the bias decides
    assert torch.allclose(wt.sum(-1), torch.ones(7, dtype=torch.float64))
    for t in range(7):
        zs = z[t, idx[t]]
        assert torch.allclose(wt[t], torch.exp(zs) / torch.exp(zs).sum())
        assert margins[0][t] > 0
    # somebody else's choice is taken over only where it is as good
    worst = int(torch.argmin(z[0]))
    idx2, _, _ = pn.route(h, w, "r.", 2, given={0: [1, worst]}, slack=1e-3)
    assert idx2[0].tolist() == idx[0].tolist()
    idx3, _, _ = pn.route(h, w, "r.", 2, given={0: [1, worst]}, slack=100.0)
    assert sorted(idx3[0].tolist()) == sorted([1, worst])
