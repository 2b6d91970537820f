"""The Vepitar configuration without a GPU: reading config.json, the registry, the declared tensors, what a
file may leave out, random weights, and the cache's storage for a mixer that keeps keys and values and a
state of fixed size beside them."""
import copy
import json

import numpy as np
import pytest
import torch

from tests.plain import vepitar_plain as P
from tests.test_gpu_vepitar import CONFIGS


def test_the_registry_finds_the_design_by_its_name(tmp_path):
    from gophonic_b200 import registry
    from gophonic_b200.config import VepitarConfig
    cfg = CONFIGS["mix"]
    assert registry.architecture_of(cfg) == "Vepitar"
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    read = registry.read_config(str(tmp_path))
    assert isinstance(read, VepitarConfig) and read.num_layers == len(cfg["layers"])
    assert read.to_dict() == cfg                                       # nothing lost, nothing added
    assert VepitarConfig.from_dict(read.to_dict()) == read
    assert read.with_layers(2).to_dict()["layers"] == cfg["layers"][:2]


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    from gophonic_b200.config import VepitarConfig
    from gophonic_b200.weights import declare_model
    cfg = CONFIGS[name]
    want = P.tensor_shapes(cfg, rank=7)
    decls = declare_model(VepitarConfig.from_dict(cfg).model_spec())
    got = {d.name: d.shape for d in decls if not d.optional}          # the head is the embedding table: no tensor of its own
    assert set(got) == set(want)
    for n, shape in got.items():            # a size the file does not give (the decay's rank) is left open
        assert len(shape) == len(want[n]) and all(a is None or a == b for a, b in zip(shape, want[n])), n
    assert [d.name for d in decls if d.optional] == ["head"]


def test_the_spec_carries_the_designs_constants():
    from gophonic_b200.config import VepitarConfig
    spec = VepitarConfig.from_dict(CONFIGS["mix"]).model_spec()
    assert spec.streams == 3 and spec.head.tied_to == "embed" and spec.final_norm.offset == 1.0
    first, second = spec.layers[0], spec.layers[1]
    assert first.block == "hyper" and first.streams == 3 and first.residual_mult == 0.5
    assert first.mixer.kind == "delta_rule" and abs(first.mixer.decay_scale - np.exp(-0.5)) < 1e-12 and first.mixer.key_eps == 1e-6
    assert first.feed_forward.kind == "swiglu" and first.mixer_norm.offset == 1.0
    assert second.mixer.kind == "sigmoid_attention" and second.mixer.window == 24 and second.mixer.conv_taps == 3
    assert second.feed_forward.kind == "moe" and (second.feed_forward.experts, second.feed_forward.top) == (5, 2)
    assert spec.layers[3].feed_forward is None
    plain = VepitarConfig.from_dict(CONFIGS["plain"]).model_spec()
    assert plain.streams == 1 and plain.layers[0].streams == 0 and plain.layers[0].residual_mult == 0.7


def test_what_a_file_leaves_out_is_not_there():
    from gophonic_b200.config import VepitarConfig
    from gophonic_b200.parts import SigmoidAttention
    from gophonic_b200.parts.base import KVRequest, KVStateRequest
    spec = VepitarConfig.from_dict(CONFIGS["odd"]).model_spec()
    bare = spec.layers[0].mixer
    assert (bare.kv_heads, bare.value_dim, bare.window, bare.conv_taps) == (3, 24, 0, 0)
    assert isinstance(SigmoidAttention.cache_request(bare), KVRequest)                  # no convolution: no state
    assert isinstance(SigmoidAttention.cache_request(spec.layers[2].mixer), KVRequest)  # one tap reaches no earlier row
    both = SigmoidAttention.cache_request(spec.layers[4].mixer)
    assert isinstance(both, KVStateRequest) and both.state.shape == (6 * (6 * 8 + 8 + 40),)
    cfg = copy.deepcopy(CONFIGS["delta"])
    del cfg["residual_mult"]
    assert VepitarConfig.from_dict(cfg).residual_mult == 1.0


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="gla"), "type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c.update(streams=64), "streams"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
])
def test_a_wrong_file_is_refused(change, message):
    from gophonic_b200.config import ConfigError, VepitarConfig
    cfg = copy.deepcopy(CONFIGS["mix"])
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        VepitarConfig.from_dict(cfg)


def test_random_weights_need_the_rank_and_write_a_model_the_plain_reader_takes(tmp_path):
    from gophonic_b200.config import VepitarConfig
    from gophonic_b200.weights import write_random_model
    cfg = copy.deepcopy(CONFIGS["mix"])
    with pytest.raises(ValueError, match="size"):
        write_random_model(VepitarConfig.from_dict(cfg), seed=1, out_dir=str(tmp_path / "a"))
    for layer in cfg["layers"]:
        if layer["type"] == "general_delta":
            layer["mixer"]["rank"] = 4
    d = write_random_model(VepitarConfig.from_dict(cfg), seed=1, out_dir=str(tmp_path / "b"))
    read, w = P.read_model(d)
    assert {n: tuple(a.shape) for n, a in w.items()} == P.tensor_shapes(cfg)
    assert abs(w["l0.norm1"]).max() < 0.2 and abs(w["l0.mix.norm"] - 1).max() < 0.2          # differences from one near 0, plain weights near 1
    assert abs(w["l1.hc2.mix"] - np.eye(3)).max() < 0.2 and abs(w["l1.hc1.in"] - 1).max() < 0.2
    assert np.isfinite(P.forward(read, w, [1, 2, 3])).all()


def test_the_cache_gives_keys_and_state_to_one_run():
    from gophonic_b200.cache import Cache
    from gophonic_b200.parts.base import KVRequest, KVStateRequest, StateRequest
    kv = KVRequest(kv_heads=2, head_dim=8, window=0, value_dim=4)
    reqs = [(StateRequest(shape=(2, 64)), None), (KVStateRequest(kv, StateRequest(shape=(30,))), None), (kv, None),
            (KVStateRequest(kv, StateRequest(shape=(30,))), None)]
    cache = Cache(reqs, max_tokens=256, device="cpu", dtype=torch.float32, max_slots=3)
    views = [cache.view(i) for i in range(4)]
    assert views[0].state.shape == (4, 2, 64)
    assert views[1].k.shape == (5, 2, 64, 8) and views[1].v.shape == (5, 2, 64, 4) and views[1].state.shape == (4, 30)
    assert views[2].state is None and views[2].k.data_ptr() != views[1].k.data_ptr()
    assert views[3].state.data_ptr() != views[1].state.data_ptr()                      # a plane of its own for each run
    a = cache.alloc_slot()
    cache.reserve([(a, 70)])
    cache.commit([(a, 70)])
    views[1].state[a] = 3.0
    views[0].state[a] = 2.0
    with pytest.raises(Exception, match="state"):
        cache.truncate(a, 10)
    mark = cache.snapshot(a)
    views[1].state[a] = 5.0
    cache.restore(a, mark)
    assert float(views[1].state[a].min()) == 3.0
    cache.free_slot(a)
    b = cache.alloc_slot()
    assert b == a and float(views[1].state[b].abs().max()) == 0.0 and float(views[0].state[b].abs().max()) == 0.0
    cache.check()
