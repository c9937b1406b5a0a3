"""Lulisun without a GPU: the configuration reader, the model spec, the declared tensors, the cache
layout, and the plain restatement checked against itself."""
import copy

import pytest
import torch

import lulisun_models
import plain_lulisun
from rust_inference_b200.config.model_config import ConfigError
from rust_inference_b200.config.registry import config_from_dict, get_architecture, registered_architectures


def test_registered_beside_the_dense_decoder():
    assert {"Lulisun", "LlamaForCausalLM", "Qwen2ForCausalLM"} <= set(registered_architectures())


@pytest.mark.parametrize("name", ["A", "B"])
def test_declared_tensors_are_the_design_s(name):
    from rust_inference_b200.engine.model import declared_tensors
    cfg = lulisun_models.CONFIGS[name]
    typed = config_from_dict(cfg)
    spec = get_architecture("Lulisun").build_spec(typed)
    declared = {k: tuple(v.shape) for k, v in declared_tensors(spec).items()}
    assert declared == plain_lulisun.tensor_shapes(cfg)
    # layers that run another layer's tensors: one LayerSpec, several schedule entries, a cache layer each
    owners = [i for i, L in enumerate(cfg["layers"]) if L.get("weights_of") is None]
    assert len(spec.layers) == len(owners)
    assert [e.cache for e in spec.schedule] == list(range(len(cfg["layers"])))
    for i, (e, L) in enumerate(zip(spec.schedule, cfg["layers"])):
        assert spec.layers[e.layer].prefix == f"l{L.get('weights_of', i) if L.get('weights_of') is not None else i}."
    assert config_from_dict(typed.to_dict()).to_dict() == typed.to_dict()


def test_config_errors_name_the_key():
    base = lulisun_models.CONFIGS["A"]

    def broken(edit):
        c = copy.deepcopy(base)
        edit(c)
        return c

    cases = [
        (lambda c: c.pop("width"), "width"),
        (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "scale"),
        (lambda c: c["layers"][0]["mixer"]["left"]["mask"].pop("size"), "size"),
        (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rot.dims"),
        (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv heads"),
        (lambda c: c["layers"][0].update(type="serial"), "type"),
        (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
        (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "choices"),
        (lambda c: c["layers"][2].update(weights_of=2), "weights_of"),
        (lambda c: (c["layers"][0].update(weights_of=2), c["layers"][2].update(weights_of=0)), "weights_of"),
        (lambda c: c["norm"].pop("eps"), "eps"),
    ]
    for edit, word in cases:
        with pytest.raises(ConfigError, match=word):
            config_from_dict(broken(edit))


def test_cache_layers_of_a_parallel_mixer():
    """Every layer run gets keys and values (values with their own head size) and a state, together;
    layers with the same needs share a storage group."""
    from rust_inference_b200.cache.sequence_cache import CompositeLayer, KVRequest, SequenceCache, StateRequest
    from rust_inference_b200.engine.model import DecoderModel
    cfg = lulisun_models.CONFIGS["A"]
    model = DecoderModel(get_architecture("Lulisun").build_spec(config_from_dict(cfg)), dtype=torch.float32, device="cpu")
    reqs = model.cache_requests()
    assert reqs[0] == reqs[2] == (KVRequest(2, 32, None, 16), StateRequest((3, 24, 40), torch.float32))
    assert reqs[1] == (KVRequest(2, 64, None, None), StateRequest((1, 72, 33), torch.float32))
    cache = SequenceCache(reqs, max_tokens=256, max_seq_len=256, dtype=torch.float32, device="cpu", n_slots=3)
    assert len(cache.groups) == 6
    first = cache.layer(0)
    assert isinstance(first, CompositeLayer)
    assert first.parts[0].k.shape == (4, 2, 64, 32) and first.parts[0].v.shape == (4, 2, 64, 16)
    assert first.parts[1].state.shape == (3, 3, 24, 40)
    assert cache.layer(2).parts[1].state.data_ptr() != first.parts[1].state.data_ptr()
    # a slot's state is zero when it is handed out
    first.parts[1].state.fill_(7.0)
    slot = cache.alloc_slot()
    assert float(first.parts[1].state[slot].abs().max()) == 0.0


def test_plain_recurrence_carries_its_state():
    g = torch.Generator().manual_seed(0)
    heads, dim, vdim, width, n = 2, 6, 5, 16, 19
    w = {"q": torch.randn(heads * dim, width, generator=g), "f": torch.randn(heads * dim, width, generator=g),
         "f.b": torch.randn(heads * dim, generator=g), "lower": torch.rand(heads * dim, generator=g),
         "v": torch.randn(heads * vdim, width, generator=g), "norm": torch.ones(vdim), "o": torch.eye(heads * vdim)}
    w = {k: v.double() for k, v in w.items()}
    x = torch.randn(n, width, generator=g).double()
    whole, s_whole = plain_lulisun.gated_recurrence(x, w, "", heads=heads, dim=dim, vdim=vdim, eps=1e-5)
    a, s = plain_lulisun.gated_recurrence(x[:7], w, "", heads=heads, dim=dim, vdim=vdim, eps=1e-5)
    b, s = plain_lulisun.gated_recurrence(x[7:], w, "", heads=heads, dim=dim, vdim=vdim, eps=1e-5, state=s)
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-12) and torch.allclose(s, s_whole, atol=1e-12)
    # the closed form of one channel: S_t = sum_j (prod_{j<k<=t} f_k) (1 - f_j) v_j
    f = torch.sigmoid(x @ w["f"].T + w["f.b"])
    f = w["lower"] + (1 - w["lower"]) * f
    v = x @ w["v"].T
    t = n - 1
    want = sum(torch.prod(f[j + 1:t + 1, 0]) * (1 - f[j, 0]) * v[j, 0] for j in range(n))
    assert abs(float(s_whole[0, 0, 0] - want)) < 1e-12


def test_plain_chunks_and_groups():
    vis = plain_lulisun.chunk_visible(10, 4)
    assert vis[3, 0] and not vis[4, 3] and vis[4, 4] and vis[7, 4] and not vis[8, 7] and not vis[2, 3]
    # all choice scores negative: the experts of a group that is shut out must not win over kept ones
    w = {"router": torch.zeros(4, 3, dtype=torch.float64), "correction": torch.tensor([-3.0, -2.9, -1.0, -5.0]).double()}
    ids, weights, s = plain_lulisun.route(torch.ones(1, 3).double(), w, "", experts=4, top=2, groups=2, keep=1)
    assert sorted(ids[0].tolist()) == [0, 1]            # group 0: -5.9 beats group 1: -6.0, though expert 2 is the best
    assert torch.allclose(weights, torch.full((1, 2), 0.5).double())


def test_shared_weights_may_be_named_through_another_sharer():
    cfg = copy.deepcopy(lulisun_models.CONFIGS["B"])
    cfg["layers"][0]["weights_of"] = 2             # 0 -> 2 -> 1: the owner is layer 1
    typed = config_from_dict(cfg)
    assert [L.weights_of for L in typed.layers] == [1, None, 1]
    spec = get_architecture("Lulisun").build_spec(typed)
    assert [e.layer for e in spec.schedule] == [0, 0, 0] and [e.cache for e in spec.schedule] == [0, 1, 2]
