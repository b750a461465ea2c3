"""Zemivik without a GPU: its configuration and the errors it names, its spec, the checkpoint names it reads,
the cache bookkeeping of a window that keeps the first positions, and the plain restatement's own mechanisms."""
import copy
import math

import pytest
import torch

import plain_zemivik as plain
from llm_infer_engine_b200.cache import CacheError, KVRequest, PageTableHost
from llm_infer_engine_b200.config import ConfigError, load_config


def test_config_reads_every_layer_on_its_own():
    arch, cfg = load_config(plain.TINY_B)
    assert arch.name == "Zemivik" and len(cfg.layers) == 5
    assert cfg.layers[0].mixer.mask is None and cfg.layers[0].mixer.v_mix is False
    assert cfg.layers[1].mlp is None and cfg.layers[1].mixer.mask.size == 33 and cfg.layers[1].mixer.mask.keep_first == 1
    assert (cfg.layers[3].mixer.dim, cfg.layers[3].mixer.vdim, cfg.layers[3].mlp.ff) == (40, 24, 52)
    assert cfg.embedding_scale == 0.7 and cfg.norm_eps == 3e-6 and cfg.vocab == 157 and cfg.max_positions == 400


@pytest.mark.parametrize("path,value,word", [
    (("vocab",), None, "vocab"), (("width",), -3, "width"), (("norm", "eps"), "x", "eps"),
    (("embedding",), None, "embedding"), (("layers",), [], "layers"),
    (("layers", 0, "type"), "recurrent", "type"), (("layers", 0, "mixer", "heads"), 4, "kv_heads"),
    (("layers", 1, "mixer", "mask", "size"), 0, "size"), (("layers", 1, "mixer", "mask", "keep_first"), -1, "keep_first"),
    (("layers", 0, "mlp", "kind"), "routed", "kind"), (("layers", 2, "mixer", "vdim"), 16, "v_mix"),
    (("layers", 0, "mixer", "scale"), None, "scale"), (("layers", 0, "mixer", "v_mix"), "yes", "v_mix")])
def test_config_errors_name_the_key(path, value, word):
    bad = copy.deepcopy(plain.TINY_B)
    bad["layers"][0]["mixer"]["kv_heads"] = 3 if path[-1] == "heads" else bad["layers"][0]["mixer"]["kv_heads"]
    node = bad
    for key in path[:-1]:
        node = node[key]
    node[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        load_config(bad)
    assert word in str(e.value)


def test_both_spellings_of_the_architecture_key():
    from llm_infer_engine_b200.config import architecture_of
    assert architecture_of({"architecture": "Zemivik"}).name == "Zemivik"
    assert architecture_of({"architectures": ["Zemivik"]}).name == "Zemivik"
    with pytest.raises(ConfigError):
        architecture_of({"architecture": "Nobody"})


def test_spec_and_checkpoint_names():
    from llm_infer_engine_b200.models.decoder import DecoderModel
    from llm_infer_engine_b200.parts.base import Runtime
    arch, cfg = load_config(plain.TINY_B)
    spec = arch.to_spec(cfg)
    assert [l.block for l in spec.layers] == ["branch_norm", "branch_norm_mixer", "branch_norm", "branch_norm",
                                              "branch_norm_mixer"]
    assert [l.mixer.get("value_blend") for l in spec.layers] == [None, "first", "blend", None, "blend"]
    model = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32, 1))
    names = model.param_specs()
    assert names["l2.mix.vmix"].shape == () and not names["l2.mix.vmix"].optional and names["l1.mix.vmix"].optional
    assert "l0.mix.vmix" not in names and "l1.mlp.up" not in names and "l1.norm2" not in names
    assert names["l3.mix.g"].shape == (24, 72) and names["l3.mix.o"].shape == (72, 24) and names["l3.mix.q"].shape == (40, 72)
    assert names["l3.mix.q.norm"].shape == (40,) and names["l4.mix.k.norm"].shape == (32,)
    assert names["l0.mlp.up.b"].shape == (100,) and names["l0.mlp.down.b"].shape == (72,)
    for top in ("embed", "pos", "embed.norm", "final.norm", "head", "l0.norm1", "l0.norm2"):
        assert top in names
    assert names["pos"].shape == (400, 72)
    # the cache: one group per distinct (key heads, head sizes, window, kept first positions)
    reqs = [r[0] for r in model.unit_requests]
    assert reqs[1] == KVRequest(2, 20, 33, v_head_dim=12, keep_first=1)
    assert reqs[0].window == 0 and reqs[0].keep_first == 0
    assert len({r.geometry() for r in reqs}) == 5


def test_window_pages_are_given_back_but_the_kept_first_ones_stay():
    t = PageTableHost(n_pages=12, page_size=64, max_pages_per_seq=12, window=100, keep_first=70)   # two kept pages
    t.open_slot(0)
    t.grow(0, 0, 500)
    assert t.pages.n_held == 8
    t.trim(0, 500)                                # the next token (position 500) reads 401.. and 0..69
    assert sorted(t.held_pages(0)) == [0, 1, 6, 7]
    t.grow(0, 500, 520)
    t.trim(0, 520)
    assert sorted(t.held_pages(0)) == [0, 1, 6, 7, 8]
    t.check()
    t.close_slot(0)
    assert t.pages.n_free == 12
    plain_window = PageTableHost(12, 64, 12, window=100)
    plain_window.open_slot(3)
    plain_window.grow(3, 0, 500)
    plain_window.trim(3, 500)
    assert sorted(plain_window.held_pages(3)) == [6, 7]
    none = PageTableHost(12, 64, 12, window=0, keep_first=5)      # no window: nothing is ever given back
    none.open_slot(1)
    none.grow(1, 0, 300)
    assert none.trim(1, 300) == [] and len(none.held_pages(1)) == 5
    with pytest.raises(CacheError):
        none.close_slot(2)


def test_trimmed_pages_are_exactly_those_no_later_token_reads():
    """Against the plain mask: after a sequence has n tokens, a page is kept iff some later query could see a
    position of it."""
    for window, keep, n in [(40, 3, 300), (64, 0, 200), (7, 9, 130), (100, 64, 470), (150, 70, 640)]:
        t = PageTableHost(16, 64, 16, window, keep)
        t.open_slot(0)
        t.grow(0, 0, n)
        t.trim(0, n)
        ok = plain.visible(n + 200, window, keep)[n:, :n]                   # later queries against held positions
        seen = ok.any(0)
        needed = sorted({j // 64 for j in range(n) if seen[j]} | {(n - 1) // 64})
        held = sorted(t.held_pages(0))
        assert set(needed) <= set(held), (window, keep, n, needed, held)
        assert len(held) <= len(needed) + 1


def test_plain_mechanisms():
    ok = plain.visible(10, 3, 2)
    assert ok[9].tolist() == [True, True, False, False, False, False, False, True, True, True]
    assert ok[2].tolist() == [True, True, True] + [False] * 7
    assert plain.visible(4, 0, 0).tolist() == torch.ones(4, 4).tril().bool().tolist()
    s = torch.tensor([[0.0, math.log(3.0)]])
    p = plain.softmax_with_sink(s, torch.tensor([[True, True]]))
    assert torch.allclose(p, torch.tensor([[0.2, 0.6]]))                    # 1 / (1 + 1 + 3), 3 / 5
    p = plain.softmax_with_sink(torch.tensor([[-50.0, 7.0]]), torch.tensor([[True, False]]))
    assert float(p[0, 1]) == 0.0 and float(p[0, 0]) < 1e-20                 # nearly everything goes to the sink
    x = torch.tensor([[3.0, 4.0]])
    assert torch.allclose(plain.rms_norm(x, torch.tensor([1.0, 2.0]), 0.0), torch.tensor([[3.0, 8.0]]) / math.sqrt(12.5))
    assert torch.allclose(plain.blend_values(torch.tensor(2.0), torch.tensor(10.0), torch.tensor(0.25)), torch.tensor(4.0))


def test_checkpoint_tensors_that_nothing_reads(tmp_path):
    """The blend scalar of a layer that does not blend may be in the file or not; any other stray tensor, a missing
    one or a wrong shape is one error that lists them."""
    from safetensors.torch import load_file, save_file
    from llm_infer_engine_b200 import WeightsError, write_random_model
    from llm_infer_engine_b200.weights.loader import build_model
    folder = str(tmp_path / "m")
    write_random_model(plain.TINY_B, folder, seed=5, std=0.05)
    path = folder + "/model.safetensors"
    t = load_file(path)
    assert "l1.mix.vmix" in t and "l0.mix.vmix" not in t          # the random mode writes the first blending layer's
    model, _ = build_model(folder, torch.float32, "cpu")
    assert model.blocks[2].mixer.lam is not None and model.blocks[1].mixer.lam is None
    del t["l1.mix.vmix"]                                             # unused: may be absent
    t["l0.mix.vmix"] = torch.tensor(0.5, dtype=torch.bfloat16)       # and a layer that does not blend may hold one
    save_file(t, path)
    build_model(folder, torch.float32, "cpu")
    del t["l2.mix.vmix"]                                             # this one is read
    t["l0.mix.extra"] = torch.zeros(3)
    t["l0.mix.q.norm"] = torch.ones(5)
    save_file(t, path)
    with pytest.raises(WeightsError) as e:
        build_model(folder, torch.float32, "cpu")
    assert e.value.missing == ["l2.mix.vmix"] and e.value.unexpected == ["l0.mix.extra"]
    assert [w[0] for w in e.value.wrong_shape] == ["l0.mix.q.norm"]
