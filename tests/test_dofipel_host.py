"""Dofipel without a GPU: the configuration reader and its errors, the spec and checkpoint names, which layer reads
whose cache, the bucketed distances, the latent cache rows, and the plain restatement's own mechanisms."""
import copy
import math

import pytest
import torch

import plain_dofipel as plain

CFG = {"architecture": "Dofipel", "vocab": 50, "width": 40, "logit_scale": 2.0, "norm": {"eps": 1e-5}, "layers": [
    {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 12, "kv_rank": 16, "scale": 0.3,
                                           "rot": {"base": 1000.0, "dims": 4}},
     "mlp": {"kind": "moe", "router": {"experts": 5, "top": 2}, "expert": {"ff": 12}, "shared": {"ff": 20}}},
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "mask": {"size": 9}, "scale": 0.3,
                                    "softcap": 10.0, "bias_max": 40}, "mlp": {"kind": "dense", "ff": 24}},
    {"type": "latent_attention", "mixer": {"heads": 3, "dim": 4, "rot_dim": 4, "vdim": 8, "kv_rank": 16, "scale": 0.4,
                                           "rot": {"base": 1000.0, "dims": 4}, "kv_from": 0}, "mlp": None}]}


def test_configuration_spec_and_names():
    from llm_infer_engine_b200.config import load_config
    from llm_infer_engine_b200.models.decoder import DecoderModel
    from llm_infer_engine_b200.parts import Runtime
    arch, cfg = load_config(CFG)
    assert arch.name == "Dofipel" and cfg.layers[2].mixer.kv_from == 0 and cfg.layers[1].mixer.window == 9
    spec = arch.to_spec(cfg)
    assert [l.block for l in spec.layers] == ["parallel", "parallel", "parallel_mixer"]
    assert [(c.layer, c.cache_of) for c in spec.schedule] == [(0, None), (1, None), (2, 0)]
    model = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32, 64))
    names = model.param_specs()
    for n, shape in {"embed": (50, 40), "l0.norm1": (40,), "l0.norm1.alpha": (), "l0.norm1.b": (40,),
                     "l0.mix.q": (24, 40), "l0.mix.dkv": (20, 40), "l0.mix.dkv.norm": (16,), "l0.mix.uk": (16, 16),
                     "l0.mix.uv": (24, 16), "l0.mix.g": (24, 40), "l0.mix.o": (40, 24), "l0.mlp.router": (5, 40),
                     "l0.mlp.router.b": (5,), "l0.mlp.e4.gate": (12, 40), "l0.mlp.e0.down": (40, 12),
                     "l0.mlp.shared.up": (20, 40), "l1.mix.k": (16, 40), "l1.mix.v": (12, 40), "l1.mix.o": (40, 24),
                     "l1.mix.sink": (4,), "l1.mlp.gate": (24, 40), "l2.mix.uk": (12, 16), "final.norm.alpha": ()}.items():
        assert tuple(names[n].shape) == shape, n
    assert names["l1.mix.rel"].shape[1] == 4 and names["l1.mix.rel"].shape[0] < 0       # the checkpoint decides its height
    assert "l2.mix.dkv" not in names and "l2.mlp.gate" not in names and "head" not in names
    assert model.unit_of_entry == [0, 1, 0]
    latent = model.unit_requests[0][0]
    assert (latent.n_kv_heads, latent.head_dim, latent.values_in_keys, latent.window) == (1, 20, 16, 0)
    assert model.unit_requests[1][0].window == 9 and model.unit_requests[1][0].value_dim == 6


@pytest.mark.parametrize("path,value,key", [
    (("layers", 1, "mixer", "softcap"), None, "softcap"), (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "rot", "dims"), 3, "dims"), (("layers", 2, "mixer", "kv_from"), 1, "kv_from"),
    (("layers", 2, "mixer", "kv_from"), 2, "kv_from"), (("layers", 2, "mixer", "kv_rank"), 8, "kv_rank"),
    (("layers", 0, "mlp", "router", "top"), 6, "top"), (("layers", 0, "mlp", "kind"), "sparse", "kind"),
    (("logit_scale",), None, "logit_scale"), (("layers", 1, "type"), "conv", "type"),
    (("layers", 0, "mlp", "expert"), None, "expert")])
def test_configuration_errors_name_the_key(path, value, key):
    from llm_infer_engine_b200.config import ConfigError, load_config
    cfg = copy.deepcopy(CFG)
    at = cfg
    for p in path[:-1]:
        at = at[p]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        load_config(cfg)
    assert key in str(e.value)


def test_random_model_loads_names_and_a_free_table_height(tmp_path):
    """The random-weights mode writes every tensor the model reads; the loader takes a distance table of any height
    and refuses one whose other size is wrong."""
    from llm_infer_engine_b200.weights.loader import compare
    from llm_infer_engine_b200.weights.random_init import random_tensors
    tensors, _ = random_tensors(CFG, seed=3)
    assert tensors["l1.mix.rel"].shape == (16, 4) and tensors["l0.norm1.alpha"].shape == ()
    compare({"t": (-16, 4)}, {"t": (9, 4)}, [], "x")
    with pytest.raises(ValueError):
        compare({"t": (-16, 4)}, {"t": (9, 5)}, [], "x")


def test_latent_rows_serve_as_keys_and_values():
    from llm_infer_engine_b200.cache import Cache, KVRequest
    cache = Cache([[KVRequest(1, 20, 0, values_in_keys=16)], [KVRequest(2, 8, 9, v_head_dim=6)]], 2, 128, 128,
                  torch.float32, "cpu")
    kv = cache.unit(0).kv
    assert kv.v.shape[-1] == 16 and kv.v.data_ptr() == kv.k.data_ptr() and kv.v.stride(-2) == 20
    assert cache.bytes() == (3 * 64 * 20 + 3 * 2 * 64 * (8 + 6)) * 4
    with pytest.raises(ValueError):
        Cache([[KVRequest(1, 20, 0, values_in_keys=21)]], 2, 128, 128, torch.float32, "cpu")


def test_plain_mechanisms():
    """The restatement against hand-made numbers: the buckets, the sink's share, the rotation, the router's weights."""
    assert [plain.distance_bucket(n, 16, 120) for n in (0, 7, 8, 9, 11, 12, 119, 120, 5000)] == [0, 7, 8, 8, 8, 9, 15, 15, 15]
    assert plain.distance_bucket(8 * 15 ** 0.5 + 1, 16, 120) == 12
    ok = torch.ones(1, 2, dtype=torch.bool)
    p = plain.softmax_with_sink(torch.tensor([[0.0, 0.0]]), ok, torch.tensor(math.log(2.0)))
    assert torch.allclose(p, torch.tensor([[0.25, 0.25]]))
    x = torch.tensor([[1.0, 0.0, 5.0, 7.0]]).repeat(3, 1)
    r = plain.rotate_pairs(x, torch.arange(3), 100.0, 2)
    assert torch.allclose(r[1, :2], torch.tensor([math.cos(1.0), math.sin(1.0)])) and torch.equal(r[:, 2:], x[:, 2:])
    w = {"router": torch.eye(3), "router.b": torch.tensor([0.0, 0.0, 1.0])}
    ids, wt = plain.route(torch.tensor([[2.0, 0.0, 0.5]]), w, "", 2)
    assert ids.tolist() == [[0, 2]] and torch.allclose(wt, torch.softmax(torch.tensor([[2.0, 1.5]]), -1))
    assert torch.equal(plain.window_visible(4, 2), torch.tensor([[1, 0, 0, 0], [1, 1, 0, 0], [0, 1, 1, 0], [0, 0, 1, 1]]).bool())
