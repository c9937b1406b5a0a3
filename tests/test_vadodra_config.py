"""Vadodra without a GPU: the configuration reader and its errors, the tensors the model declares against the plain
list, the schedule and cache requests of layers that read another layer's latent, and the plain restatement's
mechanisms against closed forms."""
import copy
import math

import pytest
import torch

import plain_vadodra
import vadodra_models
from rust_inference_b200.config.model_config import ConfigError
from rust_inference_b200.config.registry import config_from_dict, get_architecture, registered_architectures
from rust_inference_b200.engine.model import DecoderModel, declared_tensors


def _spec(cfg):
    arch = get_architecture("Vadodra")
    return arch.build_spec(arch.parse_config(cfg))


def test_registered_and_round_trip():
    assert "Vadodra" in registered_architectures()
    for cfg in vadodra_models.CONFIGS.values():
        parsed = config_from_dict(cfg)
        assert parsed.to_dict() == cfg
        assert config_from_dict(parsed.to_dict()) == parsed or config_from_dict(parsed.to_dict()).to_dict() == cfg


@pytest.mark.parametrize("name", list(vadodra_models.CONFIGS))
def test_declared_tensors_equal_the_plain_list(name):
    cfg = vadodra_models.CONFIGS[name]
    got = {k: tuple(v.shape) for k, v in declared_tensors(_spec(cfg)).items()}
    assert got == plain_vadodra.tensor_shapes(cfg)


def test_schedule_and_cache_requests_of_shared_latents():
    from rust_inference_b200.cache.sequence_cache import KVRequest
    cfg = vadodra_models.CONFIGS["A"]
    spec = _spec(cfg)
    assert [(e.layer, e.cache) for e in spec.schedule] == [(0, 0), (1, 1), (2, 0), (3, 3), (4, 0)]
    model = DecoderModel(spec, dtype=torch.float32, device="cpu")
    assert [w for _, _, w in model.schedule] == [True, True, False, True, False]
    reqs = model.cache_requests()
    assert reqs[0] == KVRequest(1, 48, None, 40, True) and reqs[2] is None
    assert reqs[1] == KVRequest(2, 32, 20, None) and reqs[3] == KVRequest(1, 16, 150, None)
    # a window of None: all keys
    specB = _spec(vadodra_models.CONFIGS["B"])
    assert DecoderModel(specB, dtype=torch.float32, device="cpu").cache_requests()[2] == KVRequest(3, 8, None, None)


def _broken(path, value=None, drop=False):
    cfg = copy.deepcopy(vadodra_models.CONFIGS["A"])
    at = cfg
    for k in path[:-1]:
        at = at[k]
    if drop:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    return cfg


@pytest.mark.parametrize("path,value,drop,word", [
    (("width",), None, True, "width"),
    (("embedding",), None, True, "embedding"),
    (("norm", "eps"), 0.0, False, "eps"),
    (("layers", 0, "type"), "conv", False, "conv"),
    (("layers", 1, "mixer", "kv_heads"), 3, False, "multiple"),
    (("layers", 1, "mixer", "vdim"), 16, False, "vdim"),
    (("layers", 1, "mixer", "rot", "dims"), 7, False, "even"),
    (("layers", 1, "mixer", "rot", "dims"), 34, False, "exceeds"),
    (("layers", 1, "mixer", "rot", "scaling", "factor"), 0.0, False, "factor"),
    (("layers", 1, "mixer", "scale"), None, True, "scale"),
    (("layers", 0, "mixer", "kv_rank"), None, True, "kv_rank"),
    (("layers", 2, "mixer", "kv_from"), 2, False, "earlier"),
    (("layers", 2, "mixer", "kv_from"), 1, False, "latent"),
    (("layers", 2, "mixer", "kv_rank"), 48, False, "equal"),
    (("layers", 4, "mixer", "kv_from"), 2, False, "latent of its own"),
    (("layers", 0, "mlp", "kind"), "moe", False, "moe"),
    (("layers", 0, "mlp", "limit"), -1.0, False, "limit"),
])
def test_configuration_errors_name_the_key(path, value, drop, word):
    with pytest.raises(ConfigError) as e:
        config_from_dict(_broken(path, value, drop))
    assert word in str(e.value)


def test_plain_mechanisms_against_closed_forms():
    # the centred norm of a row a + b * z (z of zero mean and unit mean square) is w * z, whatever a
    z = torch.tensor([1.0, -1.0, 1.0, -1.0], dtype=torch.float64)
    out = plain_vadodra.centred_norm(1000.0 + 3.0 * z, torch.full((4,), 2.0, dtype=torch.float64), 0.0)
    assert torch.allclose(out, 2.0 * z)
    # rotation keeps every pair's length, is the identity at position 0, and two rotations add up
    x = torch.randn(3, 2, 10, dtype=torch.float64)
    pos = torch.tensor([0, 5, 9])
    for turn, pairs in ((plain_vadodra.rotate_adjacent, lambda t: (t[..., 0:6:2], t[..., 1:6:2])),
                        (plain_vadodra.rotate_halves, lambda t: (t[..., :3], t[..., 3:6]))):
        y = turn(x, pos, 100.0, 6, 2.0)
        assert torch.equal(y[0], x[0]) and torch.equal(y[..., 6:], x[..., 6:])
        (a, b), (c, d) = pairs(x), pairs(y)
        assert torch.allclose(a * a + b * b, c * c + d * d)
        assert torch.allclose(turn(turn(x, pos, 100.0, 6, 2.0), pos, 100.0, 6, 2.0), turn(x, 2 * pos, 100.0, 6, 2.0))
        # scaling the positions by 1 / factor is what the factor does
        assert torch.allclose(turn(x, 4 * pos, 100.0, 6, 4.0), turn(x, pos, 100.0, 6, 1.0))
    # a window of one position returns the position's own value
    v = torch.randn(5, 1, 4, dtype=torch.float64)
    gap = torch.arange(5)[:, None] - torch.arange(5)[None, :]
    o = plain_vadodra.softmax_attention(torch.randn(1, 5, 5, dtype=torch.float64), v, (gap >= 0) & (gap < 1))
    assert torch.allclose(o, v)
    # the bounded gate at its bounds: g = limit, u = -limit
    W = {"gate": torch.full((1, 1), 10.0, dtype=torch.float64), "up": torch.full((1, 1), -10.0, dtype=torch.float64),
         "down": torch.ones(1, 1, dtype=torch.float64)}
    y = plain_vadodra.bounded_glu(torch.ones(1, 1, dtype=torch.float64), W, "", {"limit": 2.0})
    assert math.isclose(float(y), 2.0 / (1.0 + math.exp(-1.702 * 2.0)) * (-2.0 + 1.0), rel_tol=1e-12)


def test_latent_scores_equal_scores_over_expanded_keys():
    """The plain latent attention forms per-head keys; carrying the query into the latent space gives the same scores."""
    g = torch.Generator().manual_seed(0)
    H, d, r = 3, 4, 6
    uk = torch.randn(H * d, r, generator=g, dtype=torch.float64)
    c = torch.randn(7, r, generator=g, dtype=torch.float64)
    q = torch.randn(5, H, d, generator=g, dtype=torch.float64)
    direct = torch.einsum("ihd,jhd->hij", q, (c @ uk.T).view(7, H, d))
    carried = torch.einsum("ihr,jr->hij", torch.einsum("ihd,hdr->ihr", q, uk.view(H, d, r)), c)
    assert torch.allclose(direct, carried)
