"""The Pugalix configuration without a GPU: reading config.json, the registry, the declared tensors,
the schedule and the cache's storage for values of another size and for per-sequence state."""
import copy
import json

import pytest
import torch

from tests.plain import pugalix_plain as P
from tests.test_gpu_pugalix import CONFIGS


def test_the_registry_finds_the_design_by_its_name(tmp_path):
    from gophonic_b200 import registry
    from gophonic_b200.config import PugalixConfig
    cfg = CONFIGS["mix"]
    assert registry.architecture_of(cfg) == "Pugalix"
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    read = registry.read_config(str(tmp_path))
    assert isinstance(read, PugalixConfig) and read.num_layers == len(cfg["layers"])
    assert read.to_dict() == cfg                                       # nothing lost, nothing added
    assert PugalixConfig.from_dict(read.to_dict()) == read
    assert read.with_layers(2).to_dict()["layers"] == cfg["layers"][:2]


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    from gophonic_b200.config import PugalixConfig
    from gophonic_b200.weights import declare_model
    cfg = CONFIGS[name]
    want = P.tensor_shapes(cfg, rank=7)
    got = {d.name: d.shape for d in declare_model(PugalixConfig.from_dict(cfg).model_spec())}
    assert set(got) == set(want)
    for n, shape in got.items():            # a size the file does not give (the decay's rank) is left open
        assert len(shape) == len(want[n]) and all(a is None or a == b for a, b in zip(shape, want[n])), n
    assert any(None in s for s in got.values()) == any(l["type"] == "gla" for l in cfg["layers"])


def test_a_rank_in_the_file_is_taken_and_random_weights_need_it(tmp_path):
    from gophonic_b200.config import PugalixConfig
    from gophonic_b200.weights import declare_model, write_random_model
    cfg = copy.deepcopy(CONFIGS["gla"])
    with pytest.raises(ValueError, match="size"):
        write_random_model(PugalixConfig.from_dict(cfg), seed=1, out_dir=str(tmp_path / "a"))
    cfg["layers"][0]["mixer"]["rank"] = 4
    conf = PugalixConfig.from_dict(cfg)
    shapes = {d.name: d.shape for d in declare_model(conf.model_spec())}
    assert shapes["l0.mix.a1"] == (4, cfg["width"]) and shapes["l0.mix.a2"][1] == 4
    d = write_random_model(conf, seed=1, out_dir=str(tmp_path / "b"))
    _, w = P.read_model(d)
    assert {n: tuple(a.shape) for n, a in w.items()} == P.tensor_shapes(cfg)


def test_what_a_file_leaves_out_of_an_attention_mixer_is_not_there():
    from gophonic_b200.config import PugalixConfig
    cfg = copy.deepcopy(CONFIGS["attention"])
    m = cfg["layers"][0]["mixer"]
    for key in ("kv_heads", "rot", "mask", "vdim"):
        m.pop(key)
    cfg.pop("embedding")
    spec = PugalixConfig.from_dict(cfg).model_spec()
    a = spec.layers[0].mixer
    assert a.kv_heads == a.heads and a.value_dim == a.head_dim and a.position.rotary_dim == 0 and a.keep_first == 0
    assert a.window >= 1 << 20 and spec.embedding.scale == 1.0          # a window no sequence reaches


def test_the_schedule_shares_a_cache_plane_and_layers_may_lack_a_feed_forward():
    from gophonic_b200.config import PugalixConfig
    spec = PugalixConfig.from_dict(CONFIGS["mix"]).model_spec()
    assert [e.cache_of for e in spec.schedule] == [None, None, None, 1, None]
    assert [l.feed_forward is None for l in spec.layers] == [False, True, True, False, True]
    assert spec.layers[3].mixer.own_kv is False and spec.layers[1].mixer.own_kv is True
    assert spec.layers[3].mixer.window == 9 and spec.layers[3].mixer.keep_first == 0
    assert spec.embedding.scale == 3.0 and spec.head.tied_to is None


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=15), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(dim=16), "kv_from"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "mlp.kind"),
    (lambda c: c["layers"][2]["mixer"].update(gate_cap=0), "gate_cap"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c.pop("width"), "width"),
])
def test_a_file_the_design_cannot_run_is_refused_by_key(change, message):
    from gophonic_b200.config import ConfigError, PugalixConfig
    cfg = copy.deepcopy(CONFIGS["mix"])
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        PugalixConfig.from_dict(cfg)


def test_the_cache_stores_values_of_their_own_size_and_state_per_sequence():
    from gophonic_b200.cache import Cache
    from gophonic_b200.config import PugalixConfig
    from gophonic_b200 import parts, registry  # noqa: F401
    spec = PugalixConfig.from_dict(CONFIGS["mix"]).model_spec()
    reqs = [(registry.part_class("block", spec.layers[e.layer].block).cache_request(spec.layers[e.layer]), e.cache_of)
            for e in spec.schedule]
    cache = Cache(reqs, max_tokens=256, device="cpu", dtype=torch.float32)
    kv = cache.view(1)
    assert tuple(kv.k.shape[1:]) == (2, 64, 32) and tuple(kv.v.shape[1:]) == (2, 64, 16) and kv.writable
    shared = cache.view(3)
    assert shared.k.data_ptr() == kv.k.data_ptr() and not shared.writable
    gla0, ml, gla4 = cache.view(0), cache.view(2), cache.view(4)
    assert tuple(gla0.state.shape[1:]) == (2, 16 * 24) and tuple(gla4.state.shape[1:]) == (4, 8 * 8)
    assert tuple(ml.state.shape[1:]) == (3, 8 * 40 + 12)               # the matrix, the normaliser, the maximum (and padding to 16 bytes)
    s = cache.alloc_slot()
    ml.state[s].fill_(3.0)
    saved = cache.copy_state(s)
    ml.state[s].fill_(5.0)
    cache.put_state(s, saved)
    assert float(ml.state[s].min()) == 3.0
    cache.free_slot(s)
    assert cache.alloc_slot() == s and float(ml.state[s].abs().max()) == 0.0      # a slot used again starts from zero
