"""The Nadozen configuration, its model description and the weights it declares (no GPU)."""
import copy

import pytest
import torch

from nadozen_cases import CASES, DENSE, left, parallel, right, wkv


def parse(cfg):
    from infernum_b200.registry import resolve_config
    arch, typed = resolve_config(cfg)
    return arch, typed, arch.build_spec(typed)


def test_every_size_and_constant_is_read_from_the_configuration():
    arch, cfg, spec = parse(CASES["A"])
    assert arch.name == "Nadozen"
    assert (cfg.vocab, cfg.width, cfg.streams, cfg.logit_scale, cfg.norm_eps) == (173, 80, 3, 0.7, 1e-5)
    assert spec.embedding.kind == "sinusoidal_embedding" and spec.embedding.params["streams"] == 3
    assert spec.lm_head.params["scale"] == 0.7
    par = spec.layers[1].parts["mixer"]
    assert par.kind == "parallel" and (par.params["left_scale"], par.params["right_scale"]) == (0.7, 1.3)
    att = par.params["left"]["params"]
    assert (att["num_heads"], att["num_kv_heads"], att["head_dim"], att["window"], att["scale"]) == (6, 2, 16, 21, 0.3)
    assert att["value_from_key"] and att["sink"] == "sink" and att["gate"] == "g" and att["position"] is None
    ssd = par.params["right"]["params"]
    assert (ssd["num_heads"], ssd["vdim"], ssd["state"], ssd["groups"], ssd["conv"], ssd["norm_groups"]) == \
        (4, 12, 20, 2, 3, 2)
    assert spec.layers[0].block == "hyper_prenorm" and "ffn" in spec.layers[0].parts
    assert "ffn" not in spec.layers[1].parts and "norm2" not in spec.layers[1].parts


def test_a_layer_with_anothers_tensors_is_a_further_run_of_it():
    _, _, spec = parse(CASES["A"])
    assert len(spec.layers) == 2
    assert [(s.layer, s.cache_of) for s in spec.schedule] == [(0, None), (1, None), (0, None), (1, None)]
    _, _, spec_c = parse(CASES["C"])
    assert [s.layer for s in spec_c.schedule] == [0, 1, 2, 1]
    from infernum_b200.weights.random_init import model_specs_for
    names = set(model_specs_for(CASES["C"])[2])
    assert not any(n.startswith("l3.") for n in names) and "l1.mix.w1" in names


def test_every_run_gets_a_cache_and_a_state_of_its_own():
    from infernum_b200.cache import CacheManager
    from infernum_b200.models.model import Model
    from infernum_b200.parts.base import Runtime
    _, _, spec = parse(CASES["A"])
    model = Model(spec, Runtime(torch.device("cpu"), torch.float32))
    needs = model.cache_needs()
    assert [n.paged is not None for n in needs] == [False, True, False, True]
    assert all(n.state is not None and n.cache_of is None for n in needs)
    assert needs[1].paged.window == 21 and needs[1].paged.kv_heads == 2 and needs[1].paged.head_dim == 16
    # wkv: heads x dim x dim and the token before; parallel: heads x state x vdim and the convolution's inputs
    assert needs[0].state.shape == (3 * 16 * 16 + 80,)
    assert needs[1].state.shape == (4 * 20 * 12 + 2 * (48 + 2 * 2 * 20),)
    cache = CacheManager(needs, page_size=4, num_pages=12, max_requests=2, device=None)
    assert len(cache.groups) == 1 and cache.groups[0].positions == [1, 3]


def test_without_streams_the_layers_are_plain_pre_norm_layers():
    _, cfg, spec = parse(CASES["B"])
    assert cfg.streams is None
    assert all(l.block == "prenorm" for l in spec.layers)
    from infernum_b200.weights.random_init import model_specs_for
    names = set(model_specs_for(CASES["B"])[2])
    assert not any(".hc" in n for n in names)
    names_d = set(model_specs_for(CASES["D"])[2])
    assert {"l0.hc1.in", "l0.hc1.out", "l0.hc1.mix", "l0.hc2.mix", "l1.hc2.in"} <= names_d


def test_declared_tensors_and_the_rank_that_only_the_checkpoint_knows():
    from infernum_b200.weights.random_init import model_specs_for
    cfg = copy.deepcopy(CASES["A"])
    specs = model_specs_for(cfg)[2]
    assert specs["l0.mix.w1"].shape == (12, 80) and specs["l0.mix.w2"].shape == (48, 12)
    assert specs["l1.mix.left.q"].shape == (96, 80) and specs["l1.mix.left.k"].shape == (32, 80)
    assert specs["l1.mix.left.g"].shape == (96, 80) and specs["l1.mix.left.sink"].shape == (6,)
    assert specs["l1.mix.left.q.norm"].shape == (16,) and "l1.mix.left.v" not in specs
    assert specs["l1.mix.right.in"].shape == (2 * 48 + 2 * 2 * 20 + 4, 80)
    assert specs["l1.mix.right.conv"].shape == (48 + 80, 3) and specs["l1.mix.right.conv.b"].shape == (128,)
    assert specs["l1.hc1.mix"].shape == (3, 3) and specs["l0.hc2.out"].shape == (3,)
    for layer in cfg["layers"]:
        layer["mixer"].pop("decay_rank", None)
    specs = model_specs_for(cfg)[2]
    w1, w2 = specs["l0.mix.w1"], specs["l0.mix.w2"]
    assert w1.shape == (-1, 80) and w2.shape == (48, -1)
    assert w1.matches((16, 80)) and w1.matches((3, 80)) and not w1.matches((16, 81))
    assert w1.concrete_shape[1] == 80 and w2.concrete_shape[1] == w1.concrete_shape[0]


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "not supported"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=4), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(groups=3), "multiple"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][2].update(weights_of=3), "tensors of its own"),
    (lambda c: c["layers"][2].update(weights_of=1), "differs"),
    (lambda c: c["layers"][2].update(weights_of=9), "must name a layer"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c.update(streams=9), "streams"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "not supported"),
])
def test_configurations_that_are_refused(change, message):
    from infernum_b200.errors import ConfigError
    cfg = copy.deepcopy(CASES["A"])
    change(cfg)
    with pytest.raises(ConfigError) as err:
        parse(cfg)
    assert message in str(err.value)


def test_slicing_of_a_scans_columns():
    from infernum_b200.ops.scan import choose_col_slices
    # one long prompt of few heads is cut over more CTAs; a full batch is not
    assert choose_col_slices(1, 4, 64, 4, 148) > 1
    assert choose_col_slices(64, 32, 64, 4, 148) == 1
    # never more than 512 threads, always a divisor
    for cols, split in ((256, 4), (192, 8), (48, 4), (7, 1), (250, 4), (509, 1), (384, 1)):
        s = choose_col_slices(1000, 64, cols, split, 148)
        assert cols % s == 0 and (cols // s) * split <= 512 and cols // s <= 128
