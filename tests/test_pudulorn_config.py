"""The Pudulorn decoder without a GPU: tensor names and shapes against a list written out
independently, which layers read another layer's cached latent and how long that latent is kept,
configuration errors by key, the plain implementation's mechanisms against hand-made cases."""

import copy
import math

import pytest
import torch

import plain_pudulorn as P
import pudulorn_helpers as U
from bare_cuda_4gib_b200 import models  # noqa: F401
from bare_cuda_4gib_b200.config.pudulorn import PudulornConfig
from bare_cuda_4gib_b200.config.registry import resolve_architecture
from bare_cuda_4gib_b200.engine.model import expected_weights
from bare_cuda_4gib_b200.errors import ConfigError
from bare_cuda_4gib_b200.parts.base import KVCacheRequest


def _spec(cfg):
    arch = resolve_architecture(cfg)
    return arch.build_spec(arch.config_class.from_dict(cfg))


@pytest.mark.parametrize("name", ["P", "Q"])
def test_tensor_names_and_shapes(name):
    cfg = U.CONFIGS[name][0]
    expected, _ = expected_weights(_spec(cfg))
    assert {k: tuple(v.shape) for k, v in expected.items()} == U.tensor_shapes(cfg)


def test_caches_and_borrowed_latents():
    spec = _spec(U.CFG_P)
    assert [c.layer for c in spec.order] == [0, 1, 2, 3, 4]
    assert [c.cache_from for c in spec.order] == [None, None, 1, None, 1]
    _, model = expected_weights(spec)
    demands = model.cache_demands()
    # both maps of a key head side by side, values of their own size, a block of 24 positions
    assert demands[0][0].kv == KVCacheRequest(2, 32, 24, v_head_dim=24)
    assert demands[3][0].kv == KVCacheRequest(2, 16, 7, v_head_dim=8)
    # one head of kv_rank + rot_dim entries without values; kept for the widest window among its readers (17, 30, 9)
    assert demands[1][0].kv == KVCacheRequest(1, 32, 30, v_head_dim=0)
    # a layer that reads another one's latent asks for the same cache and names the layer that fills it
    assert [d.cache_from for d in demands[2]] == [1] and [d.cache_from for d in demands[4]] == [1]
    assert demands[2][0].kv == demands[1][0].kv and demands[1][0].cache_from is None
    from bare_cuda_4gib_b200.cache.manager import CacheManager
    cache = CacheManager(demands, page_tokens=16, max_seqs=2, max_tokens=64, allocate=False)
    assert sum(len(g.members) for g in cache.groups) == 3


def test_configuration_errors_name_the_key():
    def broken(change, base=U.CFG_P):
        cfg = copy.deepcopy(base)
        change(cfg)
        with pytest.raises(ConfigError) as e:
            PudulornConfig.from_dict(cfg)
        return str(e.value)

    assert "layers[0].mixer.kv_heads" in broken(lambda c: c["layers"][0]["mixer"].update(kv_heads=3))
    assert "layers[0].mixer.diff" in broken(lambda c: c["layers"][0]["mixer"].pop("diff"))
    assert "layers[0].mixer.rot.dims" in broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7))
    assert "layers[0].mixer.rot.dims" in broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18))
    assert "layers[0].mixer.mask.size" in broken(lambda c: c["layers"][0]["mixer"].update(mask={}))
    assert "layers[1].mixer.q_rank" in broken(lambda c: c["layers"][1]["mixer"].pop("q_rank"))
    assert "layers[1].type" in broken(lambda c: c["layers"][1].update(type="mlstm"))
    assert "layers[2].mixer.kv_from" in broken(lambda c: c["layers"][2]["mixer"].update(kv_from=2))
    assert "layers[2].mixer.kv_from" in broken(lambda c: c["layers"][2]["mixer"].update(kv_from=0))       # not a latent layer
    assert "layers[4].mixer.kv_from" in broken(lambda c: c["layers"][4]["mixer"].update(kv_from=2))       # caches nothing itself
    assert "layers[2].mixer.kv_rank" in broken(lambda c: c["layers"][2]["mixer"].update(kv_rank=16))
    assert "layers[2].mixer.rot" in broken(lambda c: c["layers"][2]["mixer"]["rot"].update(base=7.0))
    assert "layers[0].mlp.limit" in broken(lambda c: c["layers"][0]["mlp"].pop("limit"))
    assert "layers[1].mlp.router.top" in broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=6))
    assert "layers[1].mlp.expert.ff" in broken(lambda c: c["layers"][1]["mlp"].pop("expert"))
    assert "layers[3].mlp.kind" in broken(lambda c: c["layers"][3]["mlp"].update(kind="sparse"))
    assert "norm.eps" in broken(lambda c: c.pop("norm"))
    assert "vocab" in broken(lambda c: c.pop("vocab"))
    for cfg in (U.CFG_P, U.CFG_Q):
        assert PudulornConfig.from_dict(cfg).to_dict() == cfg


def test_plain_masks_and_turning():
    block = P.sees_block(7, 3)
    assert block[4].tolist() == [False, False, False, True, True, False, False]
    assert block[3].tolist() == [False, False, False, True, False, False, False]
    window = P.sees_window(7, 3)
    assert window[4].tolist() == [False, False, True, True, True, False, False]
    assert window[0].tolist() == [True] + [False] * 6
    # entry 0 pairs with entry dims/2; entries from dims on stay; position 0 turns nothing
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0, 5.0], [1.0, 0.0, 0.0, 0.0, 5.0]], dtype=torch.float64)
    y = P.turn_halves(x, torch.tensor([0, 2]), 4, 100.0)
    assert torch.equal(y[0], x[0])
    assert torch.allclose(y[1], torch.tensor([math.cos(2.0), 0.0, math.sin(2.0), 0.0, 5.0], dtype=torch.float64))
    y = P.turn_halves(torch.tensor([[0.0, 1.0, 0.0, 0.0]], dtype=torch.float64), torch.tensor([3]), 4, 100.0)
    assert torch.allclose(y[0], torch.tensor([0.0, math.cos(0.3), 0.0, math.sin(0.3)], dtype=torch.float64))


def test_plain_router_and_feed_forwards():
    t = {"r.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [-1.0, 0.0]], dtype=torch.float64)}
    mlp = {"router": {"experts": 3, "top": 2, "scale": 2.0}}
    h = torch.tensor([[2.0, 0.5]], dtype=torch.float64)
    s = torch.softmax(torch.tensor([2.0, 0.5, -2.0], dtype=torch.float64), 0)
    assert torch.allclose(P.router(t, "r.", mlp, h)[0], torch.stack([2 * s[0], 2 * s[1], s[2] * 0]))   # not renormalised
    one = torch.ones(1, 1, dtype=torch.float64)
    t = {"f.gate": 5.0 * one, "f.up": -7.0 * one, "f.down": one}
    # gate capped from above only, up from both sides: 1.5 * sigmoid(1.702 * 1.5) * (-1.5 + 1)
    want = 1.5 / (1.0 + math.exp(-1.702 * 1.5)) * (-0.5)
    assert math.isclose(float(P.clamped_feed_forward(t, "f.", {"limit": 1.5}, one)), want, rel_tol=1e-12)
    t["f.gate"] = -5.0 * one
    want = -5.0 / (1.0 + math.exp(1.702 * 5.0)) * (-0.5)
    assert math.isclose(float(P.clamped_feed_forward(t, "f.", {"limit": 1.5}, one)), want, rel_tol=1e-12)


def test_random_weights_of_a_preset():
    from bare_cuda_4gib_b200.models.presets import preset_config
    from bare_cuda_4gib_b200.weights.random_init import random_tensors

    config = preset_config("pudulorn-tiny")
    expected, _ = expected_weights(resolve_architecture(config.to_dict()).build_spec(config))
    tensors = random_tensors(expected, 5)
    assert set(tensors) == set(expected)
    assert abs(float(tensors["l0.norm1"].float().mean())) < 0.05          # stored around zero
    assert abs(float(tensors["l0.mix.q.norm"].float().mean()) - 1.0) < 0.1
