"""The Rugesun configuration, its model description and what the cache manager
makes of it; no GPU needed."""
import copy

import pytest
import torch

from rugesun_cases import CASES


def build(cfg):
    from infernum_b200.registry import resolve_config
    arch, typed = resolve_config(cfg)
    return arch, typed, arch.build_spec(typed)


def test_the_architecture_is_found_by_its_name():
    arch, typed, spec = build(CASES["A"])
    assert arch.name == "Rugesun"
    assert typed.width == 96 and typed.vocab == 211 and len(typed.layers) == 3
    assert spec.hidden_size == 96 and spec.vocab_size == 211
    from infernum_b200.registry import supported_architectures
    assert {"llama", "Rugesun"} <= set(supported_architectures())


def test_every_size_and_constant_reaches_the_parts():
    _, typed, spec = build(CASES["A"])
    m0 = spec.layers[0].parts["mixer"].params
    assert (m0["num_heads"], m0["dim"], m0["rot_dim"], m0["vdim"], m0["q_rank"], m0["kv_rank"]) == (3, 16, 8, 24, 24, 40)
    assert m0["scale"] == 0.2 and m0["eps"] == 1e-5 and m0["theta"] == 10000.0
    assert spec.layers[2].parts["mixer"].params["theta"] == 500.0
    assert spec.layers[0].params["alpha"] == 1.5
    assert spec.lm_head.params["softcap"] == 12.0
    e = spec.embedding.params
    assert (e["buckets"], e["mul_prev"], e["mul_cur"]) == (97, 7, 13)
    f0, f1 = spec.layers[0].parts["ffn"], spec.layers[1].parts["ffn"]
    assert f0.kind == "moe" and (f0.params["experts"], f0.params["top"], f0.params["expert_size"]) == (6, 2, 24)
    assert f1.kind == "swiglu" and f1.params["activation"] == "gelu_tanh" and f1.params["intermediate_size"] == 136
    assert "ffn" not in spec.layers[2].parts


def test_a_reader_shares_its_owners_cache_and_widens_its_window():
    _, _, spec = build(CASES["A"])
    assert [s.cache_of for s in spec.schedule] == [None, 0, None]
    # the reader's window (28) is wider than the owner's (20): pages are given back by the wider one
    assert spec.layers[0].parts["mixer"].params["cache_window"] == 28
    assert spec.layers[0].parts["mixer"].params["window"] == 20
    assert spec.layers[1].parts["mixer"].params["kv_shared"] is True
    _, _, spec_b = build(CASES["B"])
    # one reader of layer 0 sees every earlier token: the owner's pages are never given back early
    assert spec_b.layers[0].parts["mixer"].params["cache_window"] == 0


def test_cache_groups_and_latent_pools_without_values():
    from infernum_b200.cache import CacheManager
    from infernum_b200.models.model import Model
    from infernum_b200.parts import Runtime
    _, _, spec = build(CASES["A"])
    model = Model(spec, Runtime(torch.device("cpu"), torch.bfloat16))
    needs = model.cache_needs()
    assert len(needs) == 4  # three layers and the embedding's previous token
    assert needs[0].paged.v_head_dim == 0 and needs[0].paged.head_dim == 48 and needs[0].paged.window == 28
    assert needs[3].state is not None and needs[3].paged is None
    cache = CacheManager(needs, page_size=4, num_pages=16, max_requests=2, device=None)
    assert len(cache.groups) == 2
    assert cache.layer_caches[1].owner is False and cache.layer_caches[1].group == cache.layer_caches[0].group
    assert cache.bytes_per_token() == (48 + 32) * 2
    rc = cache.admit("r")
    cache.extend(rc, 60)
    cache.commit(rc, 60)
    # window 28 / 9: pages wholly below position 60 - w + 1 have been given back
    assert rc.tables[0][:8] == [-1] * 8 and rc.tables[0][8] >= 0
    assert rc.tables[1][:13] == [-1] * 13 and rc.tables[1][13] >= 0
    cache.release(rc)
    cache.check_invariants()


def test_optional_tensors_may_be_missing_from_the_files():
    from infernum_b200.models.model import Model
    from infernum_b200.parts import Runtime
    from infernum_b200.weights.loader import check_against_specs
    from infernum_b200.weights.safetensors_io import TensorEntry
    _, _, spec = build(CASES["A"])
    specs = Model(spec, Runtime(torch.device("cpu"), torch.bfloat16)).weight_specs()
    assert specs["l2.norm2"].optional and not specs["l1.norm2"].optional
    table = {n: TensorEntry(n, torch.bfloat16, tuple(s.shape), 0, 0, None) for n, s in specs.items() if not n.startswith("l2.norm2")}
    assert "l2.norm2" not in check_against_specs(specs, table)


@pytest.mark.parametrize("edit,message", [
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_from", 1), "earlier layer"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_from", 1), "keeps no cache"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("kv_rank", 32), "differs"),
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "not supported"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "sparse"), "not supported"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "exceeds"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "even"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["embedding"].pop("bigram"), "bigram"),
])
def test_bad_configurations_are_refused_with_the_key_named(edit, message):
    from infernum_b200.errors import ConfigError
    cfg = copy.deepcopy(CASES["A"])
    edit(cfg)
    with pytest.raises(ConfigError, match=message):
        build(cfg)
