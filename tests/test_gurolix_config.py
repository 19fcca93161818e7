"""The Gurolix decoder without a GPU: tensor names and shapes against a list written out
independently, what every layer keeps per request, which layer lends its values, configuration
errors by key, the plain implementation's mechanisms against hand-made cases."""

import copy
import math

import pytest
import torch

import gurolix_helpers as U
import plain_gurolix as P
from bare_cuda_4gib_b200 import models  # noqa: F401
from bare_cuda_4gib_b200.config.gurolix import GurolixConfig
from bare_cuda_4gib_b200.config.registry import resolve_architecture
from bare_cuda_4gib_b200.engine.model import expected_weights
from bare_cuda_4gib_b200.errors import ConfigError
from bare_cuda_4gib_b200.parts.base import KVCacheRequest, StateRequest

F64 = torch.float64


def _spec(cfg):
    arch = resolve_architecture(cfg)
    return arch.build_spec(arch.config_class.from_dict(cfg))


@pytest.mark.parametrize("name", ["A", "B"])
def test_tensor_names_and_shapes(name):
    cfg = U.CONFIGS[name][0]
    expected, _ = expected_weights(_spec(cfg))
    assert {k: tuple(v.shape) for k, v in expected.items()} == U.tensor_shapes(cfg)


def test_caches_states_and_value_lenders():
    spec = _spec(U.CFG_A)
    _, model = expected_weights(spec)
    demands = model.cache_demands()
    # a Mamba-2 layer keeps its matrix state and the convolution's last taps - 1 inputs, no pages
    assert [d.kv for d in demands[0]] == [None, None]
    assert demands[0][0].state == StateRequest((4, 16, 8), torch.float32)
    assert demands[0][1].state == StateRequest((4, 32 + 2 * 2 * 16), torch.float32)      # a ring of `taps` entries
    assert demands[4][1].state == StateRequest((2, 32 + 2 * 8), torch.float32)
    # attention layers keep pages with value heads of their own size, and no state
    assert demands[1][0].kv == KVCacheRequest(2, 16, None, v_head_dim=24) and demands[1][0].state is None
    assert demands[5][0].kv == KVCacheRequest(2, 8, None, v_head_dim=24)
    # the first layer that mixes values lends them, the later ones blend, a layer that says no does neither
    assert [l.mixer.params.get("v_mix") for l in spec.layers] == [None, "source", "mix", None, None, "mix"]
    assert [l.mixer.params.get("qk_norm") for l in spec.layers if l.mixer.kind == "general_attention"] == [False, True, False, True]
    assert spec.layers[2].ffn is None and "post2" not in spec.layers[2].extras
    from bare_cuda_4gib_b200.cache.manager import CacheManager
    cache = CacheManager(demands, page_tokens=16, max_seqs=2, max_tokens=64, allocate=False)
    assert sum(len(g.members) for g in cache.groups) == 4


def test_configuration_errors_name_the_key():
    def broken(change, base=U.CFG_A):
        cfg = copy.deepcopy(base)
        change(cfg)
        with pytest.raises(ConfigError) as e:
            GurolixConfig.from_dict(cfg)
        return str(e.value)

    assert "layers[1].mixer.kv_heads" in broken(lambda c: c["layers"][1]["mixer"].update(kv_heads=3))
    assert "layers[1].mixer.softcap" in broken(lambda c: c["layers"][1]["mixer"].update(softcap=-1.0))
    assert "layers[1].mixer.rot.dims" in broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7))
    assert "layers[1].mixer.rot.dims" in broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18))
    assert "layers[1].mixer.rot.scaling.factor" in broken(lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("factor"))
    assert "layers[2].mixer.rot.scaling.low" in broken(lambda c: c["layers"][2]["mixer"]["rot"].update(scaling={"factor": 2.0}))
    assert "layers[0].mixer.groups" in broken(lambda c: c["layers"][0]["mixer"].update(groups=3))
    assert "layers[0].mixer.norm_groups" in broken(lambda c: c["layers"][0]["mixer"].update(norm_groups=5))
    assert "layers[0].mixer.state" in broken(lambda c: c["layers"][0]["mixer"].pop("state"))
    assert "layers[3].type" in broken(lambda c: c["layers"][3].update(type="mlstm"))
    assert "layers[5].mixer" in broken(lambda c: c["layers"][5]["mixer"].update(vdim=16))          # mixes values of another size
    assert "layers[0].mlp.router.top" in broken(lambda c: c["layers"][0]["mlp"]["router"].update(top=5))
    assert "layers[0].mlp.router.groups.count" in broken(lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4))
    assert "layers[0].mlp.router.groups.keep" in broken(lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=4))
    assert "layers[1].mlp.expert.ff" in broken(lambda c: c["layers"][1]["mlp"].pop("expert"))
    assert "layers[3].mlp.kind" in broken(lambda c: c["layers"][3]["mlp"].update(kind="dense"))
    assert "norm.eps" in broken(lambda c: c.pop("norm"))
    assert "width" in broken(lambda c: c.pop("width"))
    for cfg in (U.CFG_A, U.CFG_B):
        assert GurolixConfig.from_dict(cfg).to_dict() == cfg


def test_plain_frequencies_and_turning():
    # wavelengths 2 pi, 20 pi, 200 pi, 2000 pi against original / high = 16 and original / low = 640
    f = P.frequencies({"dims": 8, "base": 10000.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 40.0, "original": 640}})
    plain = [10000.0 ** (-2.0 * i / 8) for i in range(4)]
    assert math.isclose(float(f[0]), plain[0])                       # short: kept
    assert math.isclose(float(f[3]), plain[3] / 4.0)                 # long: divided
    s = (640 / (2 * math.pi / plain[1]) - 1.0) / 39.0
    assert math.isclose(float(f[1]), (1 - s) * plain[1] / 4.0 + s * plain[1])
    assert torch.equal(P.frequencies({"dims": 8, "base": 10000.0}), torch.tensor(plain, dtype=F64))
    # entry 0 pairs with entry dims/2; entries from dims on stay; position 0 turns nothing
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]], [[1.0, 0.0, 0.0, 0.0, 5.0]]], dtype=F64)
    y = P.turn_halves(x, torch.tensor([0, 2]), torch.tensor([1.0, 0.01], dtype=F64), 4)
    assert torch.equal(y[0], x[0])
    assert torch.allclose(y[1, 0], torch.tensor([math.cos(2.0), 0.0, math.sin(2.0), 0.0, 5.0], dtype=F64))


def test_plain_score_cap_and_causality():
    q = torch.tensor([[100.0], [100.0]], dtype=F64)
    k = torch.tensor([[1.0], [-1.0]], dtype=F64)
    v = torch.tensor([[1.0, 0.0], [0.0, 1.0]], dtype=F64)
    out = P.causal_softmax_attention(q, k, v, 1.0, softcap=2.0)
    assert torch.allclose(out[0], v[0])                              # the first token sees itself only
    w = math.exp(2.0 * math.tanh(50.0)) / (math.exp(2.0 * math.tanh(50.0)) + math.exp(-2.0 * math.tanh(50.0)))
    assert torch.allclose(out[1], torch.tensor([w, 1.0 - w], dtype=F64))


def test_plain_router_groups_correction_and_identity():
    eye = torch.eye(6, dtype=F64)
    t = {"r.router": eye, "r.correction": torch.tensor([0.0, 0.0, 0.0, 0.0, 0.5, 0.0], dtype=F64)}
    r = {"experts": 4, "identity": 2, "top": 2, "groups": {"count": 3, "keep": 2}}
    h = torch.tensor([[3.0, 2.9, 2.0, 0.0, 0.0, 0.0]], dtype=F64)
    s = torch.softmax(h[0], 0)
    ids, w = P.route(t, "r.", r, h)
    # groups (0, 1), (2, 3), (4, 5): the correction lifts the last group above the second, which is barred,
    # so expert 2 cannot be chosen although its score beats expert 4's; the weight is the score without correction
    assert sorted(ids[0].tolist()) == [0, 4]
    assert torch.allclose(w[0].sort().values, torch.stack([s[4], s[0]]).sort().values)
    # an identity expert hands the input on, an expert squares its relu
    t.update({f"r.e{e}.up": torch.tensor([[1.0, 0, 0, 0, 0, 0], [-1.0, 0, 0, 0, 0, 0]], dtype=F64) for e in range(4)})
    t.update({f"r.e{e}.down": torch.ones(6, 2, dtype=F64) for e in range(4)})
    out = P.mixture(t, "r.", {"router": r}, h)
    assert torch.allclose(out[0], s[0] * 9.0 * torch.ones(6, dtype=F64) + s[4] * h[0])


def test_plain_mamba2_against_a_hand_made_case():
    # one head, state of one, one channel, one tap of weight one: x = silu(u_x), B = silu(u_B), C = silu(u_C)
    t = {"m.in": torch.eye(5, dtype=F64), "m.conv": torch.ones(3, 1, dtype=F64), "m.conv.b": torch.zeros(3, dtype=F64),
         "m.dt_bias": torch.zeros(1, dtype=F64), "m.A_log": torch.zeros(1, dtype=F64), "m.D": torch.tensor([0.5], dtype=F64),
         "m.norm": torch.ones(1, dtype=F64), "m.o": torch.ones(1, 1, dtype=F64)}
    m = {"heads": 1, "vdim": 1, "state": 1, "groups": 1, "conv": 1, "norm_groups": 1}
    h = torch.tensor([[1.0, 2.0, 1.0, 1.0, 0.0], [1.0, 1.0, 0.5, 2.0, 1.0]], dtype=F64)     # z, x, B, C, dt
    silu = lambda v: v / (1.0 + math.exp(-v))
    dt = [math.log(2.0), math.log1p(math.e)]
    s1 = dt[0] * silu(1.0) * silu(2.0)
    y1 = s1 * silu(1.0) + 0.5 * silu(2.0)
    s2 = math.exp(-dt[1]) * s1 + dt[1] * silu(0.5) * silu(1.0)
    y2 = s2 * silu(2.0) + 0.5 * silu(1.0)
    out = P.mamba2(t, "m.", m, h, 0.0)
    # the unit norm of one channel leaves the sign: compare before it through a second run with two channels
    assert torch.allclose(out[:, 0], torch.tensor([math.copysign(1.0, y1 * silu(1.0)), math.copysign(1.0, y2 * silu(1.0))], dtype=F64))
    # the convolution reads zeros before the start and the last column meets the current token
    u = torch.tensor([[1.0], [2.0], [3.0]], dtype=F64)
    c = P.short_convolution(u, torch.tensor([[100.0, 10.0, 1.0]], dtype=F64), torch.tensor([0.5], dtype=F64))
    assert c[:, 0].tolist() == [1.5, 12.5, 123.5]


def test_random_weights_of_a_preset():
    from bare_cuda_4gib_b200.models.presets import preset_config
    from bare_cuda_4gib_b200.weights.random_init import random_tensors

    config = preset_config("gurolix-tiny")
    expected, _ = expected_weights(resolve_architecture(config.to_dict()).build_spec(config))
    tensors = random_tensors(expected, 5)
    assert set(tensors) == set(expected)
    assert abs(float(tensors["l0.norm1"].float().mean())) < 0.05          # stored around zero
    assert tuple(tensors["l0.mix.vmix"].shape) == ()
    assert abs(float(tensors["l2.mix.q.norm"].float().mean()) - 1.0) < 0.1
