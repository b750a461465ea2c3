"""Dofipel on the GPU against its plain restatement (tests/plain_dofipel.py): each new kernel and part alone, the
attention's edges with one score made to stand out, and the engine in float32 and bfloat16 over whole prompts,
token-by-token decoding, prompts in pieces down to two tokens, unequal batches with slots and pages used again, long
decoding and greedy generation through the library's own entry point."""
import json
import math
import os

import pytest
import torch

import helpers
import plain_dofipel as plain
from test_parts_gpu import DEV, DTYPES, build, kernel_plan, make_ctx

pytestmark = pytest.mark.gpu

ROT = {"base": 10000.0, "dims": 8}
# Every layer of A differs: a latent layer with routed experts and a shared one, a windowed layer whose value heads
# are narrower than its key heads, a layer that borrows the first layer's latent and has no feed-forward, an unmasked
# layer with head sizes that are no multiples of 8, one expert per token and no shared expert.
TINY_A = {"architecture": "Dofipel", "vocab": 211, "width": 96, "logit_scale": 0.5, "norm": {"eps": 1e-5}, "layers": [
    {"type": "latent_attention", "mixer": {"heads": 3, "dim": 24, "rot_dim": 8, "vdim": 40, "kv_rank": 48, "scale": 0.2,
                                           "rot": ROT},
     "mlp": {"kind": "moe", "router": {"experts": 6, "top": 3}, "expert": {"ff": 40}, "shared": {"ff": 56}}},
    {"type": "attention", "mixer": {"heads": 6, "kv_heads": 3, "dim": 32, "vdim": 16, "mask": {"size": 24}, "scale": 0.2,
                                    "softcap": 20.0, "bias_max": 64},
     "mlp": {"kind": "dense", "ff": 136}},
    {"type": "latent_attention", "mixer": {"heads": 2, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 48, "scale": 0.3,
                                           "rot": ROT, "kv_from": 0}, "mlp": None},
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 4, "dim": 20, "vdim": 28, "mask": None, "scale": 0.3,
                                    "softcap": 5.0, "bias_max": 300},
     "mlp": {"kind": "moe", "router": {"experts": 4, "top": 1}, "expert": {"ff": 24}, "shared": None}}]}
# B: a width that is no multiple of 8, one key head, a window longer than a page, a rotation over a part of the
# rotated entries only, a single-head latent layer.
TINY_B = {"architecture": "Dofipel", "vocab": 97, "width": 100, "logit_scale": 1.5, "norm": {"eps": 1e-6}, "layers": [
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 1, "dim": 16, "vdim": 16, "mask": {"size": 70}, "scale": 0.25,
                                    "softcap": 6.0, "bias_max": 90},
     "mlp": {"kind": "moe", "router": {"experts": 9, "top": 4}, "expert": {"ff": 20}, "shared": {"ff": 12}}},
    {"type": "latent_attention", "mixer": {"heads": 1, "dim": 12, "rot_dim": 4, "vdim": 20, "kv_rank": 40, "scale": 0.25,
                                           "rot": {"base": 500.0, "dims": 2}}, "mlp": {"kind": "dense", "ff": 60}},
    {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 8, "mask": {"size": 3}, "scale": 0.2,
                                    "softcap": 2.5, "bias_max": 20}, "mlp": None}]}
# C: head sizes 64 and 128 with equal value sizes (what the tensor-core attention kernels take) and a wider latent.
TINY_C = {"architecture": "Dofipel", "vocab": 160, "width": 128, "logit_scale": 0.25, "norm": {"eps": 1e-6}, "layers": [
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "mask": {"size": 100}, "scale": 0.125,
                                    "softcap": 5.0, "bias_max": 200}, "mlp": {"kind": "dense", "ff": 256}},
    {"type": "latent_attention", "mixer": {"heads": 4, "dim": 32, "rot_dim": 16, "vdim": 32, "kv_rank": 64, "scale": 0.15,
                                           "rot": {"base": 100000.0, "dims": 16}},
     "mlp": {"kind": "moe", "router": {"experts": 8, "top": 2}, "expert": {"ff": 64}, "shared": {"ff": 64}}},
    {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 128, "vdim": 128, "mask": {"size": 65}, "scale": 0.09,
                                    "softcap": 3.0, "bias_max": 100}, "mlp": {"kind": "dense", "ff": 128}},
    {"type": "latent_attention", "mixer": {"heads": 2, "dim": 64, "rot_dim": 16, "vdim": 64, "kv_rank": 64, "scale": 0.1,
                                           "rot": {"base": 100000.0, "dims": 16}, "kv_from": 1},
     "mlp": {"kind": "dense", "ff": 64}}]}
CFGS = {"a": TINY_A, "b": TINY_B, "c": TINY_C}
BIAS_ROWS = {"a": {1: 12, 3: 20}, "b": {0: 6, 2: 9}, "c": {0: 32, 2: 10}}       # rows of each layer's distance table
LENGTHS = {"a": [1, 5, 64, 65, 130, 300], "b": [3, 77, 200, 257], "c": [40, 129, 260]}
SHARPEN = {"a": 4.0, "b": 4.0, "c": 2.5}        # factor on the query and key projections
_folders, _engines = {}, {}


def folder_for(tag):
    """A model folder of random weights; the distance tables get heights of their own (the loader reads them from
    the tensors), sinks and tables are drawn wide enough to matter."""
    from llm_infer_engine_b200.weights.random_init import random_tensors
    from llm_infer_engine_b200.weights.safetensors_io import save_file
    if tag not in _folders:
        d = helpers.scratch_folder(f"llmie_dofipel_{tag}_")
        tensors, _ = random_tensors(CFGS[tag], seed=21 + len(_folders), std=0.09, norm_range=(0.7, 1.3))
        g = torch.Generator().manual_seed(5)
        for name in tensors:                   # wide embeddings and sharp scores: a key lost or added must show
            if name == "embed" or name.endswith((".mix.q", ".mix.k", ".mix.dkv", ".mix.uk")):
                tensors[name] = (tensors[name].float() * (8.0 if name == "embed" else SHARPEN[tag])).to(torch.bfloat16)
            elif name.endswith((".mix.o", ".mix.v", ".mix.uv", ".down")):
                tensors[name] = (tensors[name].float() * 2.0).to(torch.bfloat16)
        for layer, rows in BIAS_ROWS[tag].items():
            heads = CFGS[tag]["layers"][layer]["mixer"]["heads"]
            tensors[f"l{layer}.mix.rel"] = (torch.randn(rows, heads, generator=g) * 1.5).to(torch.bfloat16)
            tensors[f"l{layer}.mix.sink"] = (torch.randn(heads, generator=g) * 2).to(torch.bfloat16)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(CFGS[tag], f)
        save_file(tensors, os.path.join(d, "model.safetensors"))
        _folders[tag] = d
    return _folders[tag]


def plain_weights(tag):
    from safetensors.torch import load_file
    return {k: v.double() for k, v in load_file(os.path.join(folder_for(tag), "model.safetensors")).items()}


def engine_for(tag, dtype, **kw):
    from llm_infer_engine_b200 import Engine
    key = (tag, dtype, tuple(sorted(kw.items())))
    if key not in _engines:
        _engines[key] = Engine(folder_for(tag), dtype=dtype, max_batch=kw.pop("max_batch", 8),
                               max_tokens=kw.pop("max_tokens", 64 * 48), cuda_graph=kw.pop("cuda_graph", False), **kw)
    return _engines[key]


def bound(dtype, want):
    return (3e-5 if dtype == "float32" else 0.05) * max(1.0, float(want.abs().max()))


def oracle(tag, requests):
    w = plain_weights(tag)
    return {rid: plain.forward(w, CFGS[tag], toks).float() for rid, toks in requests.items()}


def compare(got, want, dtype, what):
    for rid in want:
        assert got[rid].shape == want[rid].shape, (what, rid)
        diff = (got[rid] - want[rid]).abs().max(dim=1).values
        tol = bound(dtype, want[rid])
        over = int((diff > tol).sum())
        allowed = 0 if dtype == "float32" else max(1, len(diff) // 25)
        assert over <= allowed and float(diff.max()) <= (tol if dtype == "float32" else 3 * tol), (
            f"{what}: request {rid}: {over} of {len(diff)} positions over the bound {tol:.3e}, worst "
            f"{float(diff.max()):.3e}, first at token {int((diff > tol).nonzero()[0])}")


def requests_for(tag):
    return {f"r{i}": helpers.random_tokens(CFGS[tag]["vocab"], n, seed=40 + i) for i, n in enumerate(LENGTHS[tag])}


def tol(dtype, scale):
    return (2e-5 if dtype == "float32" else 2e-2) * max(1.0, scale)


# ------------------------------------------------------------------------------------------ kernels and parts alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", [200, 204, 2048])           # 16-byte accesses, element by element, a wide row
@pytest.mark.parametrize("n_delta,delta_dtype", [(0, None), (1, "float32"), (2, "float32"), (2, "bfloat16"), (2, "mixed")])
def test_dynamic_tanh_norm_adds_both_branches(dtype, size, n_delta, delta_dtype):
    norm, w = build("norm", "dynamic_tanh", {"size": size}, dtype, seed=1)
    w["alpha"] = torch.tensor(0.37)
    norm.load({n: t.to(DEV, torch.float32) for n, t in w.items()})
    g = torch.Generator().manual_seed(size + n_delta)
    h = torch.randn(9, size, generator=g) * 3
    kinds = {"float32": ["float32"] * 2, "bfloat16": ["bfloat16"] * 2, "mixed": ["bfloat16", "float32"], None: []}[delta_dtype]
    deltas = [torch.randn(9, size, generator=g).to(DTYPES[k]) for k in kinds[:n_delta]]
    hd = h.clone().to(DEV)
    pending = tuple(d.to(DEV) for d in deltas) if n_delta != 1 else deltas[0].to(DEV)
    y = norm.forward(hd, pending if n_delta else None)
    want_h = h.double() + sum(d.double() for d in deltas)
    assert float((hd.cpu().double() - want_h).abs().max()) < 1e-5         # the stream stays float32 and holds the sum
    want = plain.dyt(want_h, w["alpha"].double(), w["weight"].double(), w["b"].double())
    assert y.dtype == DTYPES[dtype]
    assert float((y.cpu().double() - want).abs().max()) <= tol(dtype, float(want.abs().max()))
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV)
    before = hd.clone()
    some = norm.forward(hd, pending if n_delta else None, rows=rows)        # wanted rows only; the stream is left alone
    want2 = plain.dyt(want_h + sum(d.double() for d in deltas), w["alpha"].double(), w["weight"].double(), w["b"].double())
    assert float((some.cpu().double() - want2[[7, 0, 3]]).abs().max()) <= tol(dtype, float(want2.abs().max()))
    assert torch.equal(hd, before)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows,inner,activation", [(3, 100, "gelu_tanh"), (40, 128, "gelu_tanh"), (5, 96, "silu"),
                                                  (33, 52, "gelu_tanh")])
def test_gated_feed_forward_with_a_choice_of_activation(dtype, rows, inner, activation):
    names = {"gate": "gate", "up": "up", "down": "down"}
    ff, w = build("feed_forward", "swiglu", {"hidden": 72, "intermediate": inner, "activation": activation, "names": names,
                                             "out_float32": True}, dtype, seed=3)
    g = torch.Generator().manual_seed(4)
    x = torch.randn(rows, 72, generator=g).to(DTYPES[dtype])
    y = ff.forward(x.to(DEV), make_ctx([rows], [0], [0], dtype))
    act = plain.gelu_tanh if activation == "gelu_tanh" else plain.silu
    want = plain.gated_ff(x.double(), {k: v.double() for k, v in w.items()}, "", act)
    assert y.dtype == torch.float32
    assert float((y.cpu().double() - want).abs().max()) <= tol(dtype, float(want.abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top,ff,shared,rows", [(6, 3, 40, 56, 37), (4, 1, 24, None, 5), (5, 5, 16, 8, 1),
                                                       (40, 35, 8, None, 3), (16, 2, 72, 24, 300), (3, 2, 10, 10, 64)])
def test_routed_experts(dtype, experts, top, ff, shared, rows):
    """The router's choice and weights, then the whole feed-forward; tokens of 1 to 300 (both tile sizes of the
    routed product), one expert per token, all experts per token, more choices than a warp has lanes."""
    from llm_infer_engine_b200.kernels import ops
    d = 52
    part, w = build("feed_forward", "routed_experts", {"hidden": d, "n_experts": experts, "top": top, "expert_ff": ff,
                                                       "shared_ff": shared}, dtype, seed=experts + top, std=0.3)
    if experts >= 16:                     # three experts that no token chooses: groups without rows
        w["router.b"][:3] = -60.0
        part.load({n: t.to(DEV, DTYPES[dtype]) for n, t in w.items()})
    w64 = {k: v.double() for k, v in w.items()}
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, d, generator=g).to(DTYPES[dtype])
    ids = torch.empty((rows, top), dtype=torch.int32, device=DEV)
    wt = torch.empty((rows, top), dtype=torch.float32, device=DEV)
    ops.moe_route(x.to(DEV), part.w_router, part.b_router, ids, wt)
    want_ids, want_wt = plain.route(x.double(), w64, "", top)
    z = x.double() @ w64["router"].T + w64["router.b"]
    for t in range(rows):                                   # equal unless two logits nearly tie
        if ids[t].tolist() != want_ids[t].tolist():
            gap = z[t].sort(descending=True).values
            assert float((gap[:-1] - gap[1:]).min()) < 1e-4, t
        else:
            assert float((wt[t].cpu().double() - want_wt[t]).abs().max()) < 1e-5
    y = part.forward(x.to(DEV), make_ctx([rows], [0], [0], dtype))
    want = plain.moe(x.double(), w64, "", {"router": {"top": top}, "shared": {"ff": shared} if shared else None})
    assert y.dtype == torch.float32
    assert float((y.cpu().double() - want).abs().max()) <= tol(dtype, float(want.abs().max()))


def test_distance_buckets_follow_the_formula():
    from llm_infer_engine_b200.parts.gated_attention import distance_buckets
    for rows, far in ((16, 120), (12, 64), (20, 300), (6, 90), (9, 20), (32, 128), (2, 5), (10, 100)):
        got = distance_buckets(rows, far, 5000)
        assert got[-1] == rows - 1 and got == [plain.distance_bucket(n, rows, far) for n in range(len(got))]
        assert all(plain.distance_bucket(n, rows, far) == rows - 1 for n in (len(got), len(got) + 1, 4000))
        assert distance_buckets(rows, far, 7) == [plain.distance_bucket(n, rows, far) for n in range(min(7, len(got)))]


def _attention_layer(tag, layer):
    cfg = CFGS[tag]
    m = cfg["layers"][layer]["mixer"]
    params = {"hidden": cfg["width"], "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
              "v_head_dim": m["vdim"], "scale": m["scale"], "window": m["mask"]["size"] if m["mask"] else 0,
              "sink": "learned", "softcap": m["softcap"], "distance_bias": {"rows": BIAS_ROWS[tag][layer], "far": m["bias_max"]}}
    return m, params


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag,layer", [("a", 1), ("a", 3), ("b", 0), ("c", 0), ("c", 2)])
def test_window_attention_part(dtype, tag, layer):
    """The mixer alone over two sequences of unequal lengths: a prompt step, a second piece of the prompts at a
    start position above zero, then one token each."""
    from llm_infer_engine_b200.cache import Cache
    m, params = _attention_layer(tag, layer)
    mixer, w = build("mixer", "gated_attention", params, dtype, seed=layer, std=0.25)
    d = params["hidden"]
    cache = Cache([mixer.cache_requests()], 3, 64 * 12, 512, DTYPES[dtype], DEV)
    slots = [cache.take_slot() for _ in range(2)]
    lens = [150, 71]
    g = torch.Generator().manual_seed(7)
    xs = [torch.randn(n, d, generator=g).to(DTYPES[dtype]) for n in lens]
    want = [plain.window_attention(x.double(), {k: v.double() for k, v in w.items()}, "", m) for x in xs]
    held = [0, 0]
    for pieces in ([100, 40], [49, 30], [1, 1]):
        for s, h0, p in zip(slots, held, pieces):
            cache.reserve(s, h0 + p)
        ctx = make_ctx(pieces, held, slots, dtype, kernels=kernel_plan(dtype))
        x = torch.cat([xs[i][held[i]:held[i] + pieces[i]] for i in range(2)])
        y = mixer.forward(x.to(DEV), ctx, cache.unit(0), True).float().cpu().double()
        ref = torch.cat([want[i][held[i]:held[i] + pieces[i]] for i in range(2)])
        assert float((y - ref).abs().max()) <= tol(dtype, float(ref.abs().max())) * 2, (pieces, held)
        for i, s in enumerate(slots):
            held[i] += pieces[i]
            cache.note_appended(s, held[i], device_updated=False)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag,layer,reader", [("a", 0, 2), ("b", 1, None), ("c", 1, 3)])
def test_latent_attention_part_and_a_layer_that_reads_its_latent(dtype, tag, layer, reader):
    """The layer that makes the latent, the cache rows it leaves ([normed latent | rotated key part]), and a second
    layer with other head sizes that only reads them; prompts in two pieces, then one token each."""
    from llm_infer_engine_b200.cache import Cache
    cfg = CFGS[tag]

    def make(index, owns):
        m = cfg["layers"][index]["mixer"]
        p = {"hidden": cfg["width"], "n_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
             "v_head_dim": m["vdim"], "kv_rank": m["kv_rank"], "scale": m["scale"], "rot_base": m["rot"]["base"],
             "rot_dims": m["rot"]["dims"], "norm_eps": cfg["norm"]["eps"], "gate": True, "owns_latent": owns,
             "out_float32": True}
        part, w = build("mixer", "latent_attention", p, dtype, seed=index + 3, std=0.25)
        return m, part, {k: v.double() for k, v in w.items()}

    m0, owner, w0 = make(layer, True)
    others = [make(reader, False)] if reader is not None else []
    d = cfg["width"]
    cache = Cache([owner.cache_requests()], 3, 64 * 12, 512, DTYPES[dtype], DEV)
    cache.take_slot()
    slots = [cache.take_slot() for _ in range(2)]
    lens = [140, 67]
    g = torch.Generator().manual_seed(9)
    xs = [torch.randn(n, d, generator=g).to(DTYPES[dtype]) for n in lens]
    latents = [plain.latent_keys(x.double(), w0, "", m0, cfg["norm"]["eps"]) for x in xs]
    held = [0, 0]
    for pieces in ([90, 30], [49, 36], [1, 1]):
        for s, h0, p in zip(slots, held, pieces):
            cache.reserve(s, h0 + p)
        ctx = make_ctx(pieces, held, slots, dtype, kernels=kernel_plan(dtype))
        x = torch.cat([xs[i][held[i]:held[i] + pieces[i]] for i in range(2)]).to(DEV)
        for (m, part, w), owns in [((m0, owner, w0), True)] + [(o, False) for o in others]:
            y = part.forward(x, ctx, cache.unit(0), owns).float().cpu().double()
            ref = torch.cat([plain.latent_attention(xs[i].double(), w, "", m, *latents[i])[held[i]:held[i] + pieces[i]]
                             for i in range(2)])
            assert float((y - ref).abs().max()) <= tol(dtype, float(ref.abs().max())) * 2, (pieces, held, owns)
        for i, s in enumerate(slots):
            held[i] += pieces[i]
            cache.note_appended(s, held[i], device_updated=False)
    kv = cache.unit(0).kv
    for i, s in enumerate(slots):                      # the cache rows themselves
        table = kv.block_table[s].cpu()
        for pos in (0, 63, 64, lens[i] - 1):
            row = kv.k[int(table[pos // 64]), 0, pos % 64].float().cpu().double()
            ref = torch.cat([latents[i][0][pos], latents[i][1][pos]])
            assert float((row - ref).abs().max()) <= tol(dtype, float(ref.abs().max()))
    assert kv.v.data_ptr() == kv.k.data_ptr() and kv.v.shape[-1] == m0["kv_rank"]     # the latent is its own value


# ------------------------------------------------------------------------------------------ the attention's edges
def _edge_case(dtype, hd, hdv, n_q, n_kv, window, n, q_len, probe, cap, bias_rows, sink_value, latent=0):
    """A sequence of n keys of which the last q_len are this step's queries; the LAST query points straight at key
    `probe`, whose value is a marker (50 in every entry), while every other value is small. Slots and pages were
    given back and taken again before, so the sequence's pages are out of order. Returns the last query's output
    and the plain result."""
    from llm_infer_engine_b200.cache import Cache, KVRequest
    from llm_infer_engine_b200.parts import AttentionOptions
    req = KVRequest(1, hd, 0, values_in_keys=latent) if latent else KVRequest(n_kv, hd, window, v_head_dim=hdv)
    cache = Cache([[req]], 4, 64 * 24, 1024, DTYPES[dtype], DEV)
    cache.take_slot()
    other = cache.take_slot()
    cache.reserve(other, 130)
    slot = cache.take_slot()
    cache.reserve(slot, 70)
    cache.give_back_slot(other)
    cache.reserve(slot, n)
    g = torch.Generator().manual_seed(n * 7 + probe)
    k = torch.randn(n, n_kv, hd, generator=g) * 0.3
    v = torch.randn(n, n_kv, hdv, generator=g) * 0.1
    q = torch.randn(q_len, n_q, hd, generator=g) * 0.3
    direction = torch.nn.functional.normalize(torch.randn(hd, generator=g), dim=0)
    if latent:
        direction[:latent] = 0                       # the score stands out through the entries that are not values
        direction = torch.nn.functional.normalize(direction, dim=0)
        k[:, :, :latent] *= 0.3
    k[probe] += direction * 8.0
    q[-1] = direction * 8.0
    if latent:
        k[probe, :, :latent] = 50.0
        v = k[:, :, :latent].clone()
    else:
        v[probe] = 50.0
    k, v, q = (t.to(DTYPES[dtype]) for t in (k, v, q))
    kv = cache.unit(0).kv
    table = kv.block_table[slot].cpu()
    for j in range(n):
        kv.k[int(table[j // 64]), :, j % 64] = k[j].to(DEV)
        if not latent:
            kv.v[int(table[j // 64]), :, j % 64] = v[j].to(DEV)
    rel = torch.randn(bias_rows, n_q, generator=g).to(torch.bfloat16).double() if bias_rows else None
    far = 3.0 * bias_rows
    dist_bias = None
    if bias_rows:
        from llm_infer_engine_b200.parts.gated_attention import distance_buckets
        idx = torch.tensor(distance_buckets(bias_rows, far, window or 1024))
        dist_bias = rel[idx].t().contiguous().float().to(DEV)
    sinks = torch.full((n_q,), float(sink_value)).to(DEV) if sink_value is not None else None
    scale = 0.5
    ctx = make_ctx([q_len], [n - q_len], [slot], dtype, kernels=kernel_plan(dtype))
    out = torch.empty(q_len, n_q * hdv, dtype=DTYPES[dtype], device=DEV)
    ctx.attention(q.reshape(q_len, -1).to(DEV), kv, out, n_q, n_kv, hd,
                  AttentionOptions(scale=scale, window=window, softcap=cap, distance_bias=dist_bias, sink_values=sinks))
    ok = plain.window_visible(n, window)[n - 1:]
    want = []
    for h in range(n_q):
        kh = k[:, h // (n_q // n_kv)].double()
        s = (q[-1, h].double() @ kh.T)[None] * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        if bias_rows:
            s = s + rel[:, h][torch.tensor([[plain.distance_bucket(n - 1 - j, bias_rows, far) for j in range(n)]])]
        p = plain.softmax_with_sink(s, ok, torch.tensor(float(sink_value)).double() if sink_value is not None else None)
        want.append(p @ v[:, h // (n_q // n_kv)].double())
    return out[-1].float().cpu(), torch.cat(want, -1).float().reshape(-1), bool(ok[0, probe])


EDGES = [  # window, keys, probe, may the last query (position keys - 1) see it
    (80, 300, 220, True), (80, 300, 219, False),          # just inside and just outside the window
    (64, 257, 193, True), (64, 257, 192, False),          # the window's edge on a page's edge
    (65, 257, 192, True), (65, 257, 191, False),
    (0, 500, 3, True), (0, 500, 255, True), (0, 700, 0, True),      # no window: keys far back, the first token
    (1, 40, 39, True), (1, 40, 38, False), (2, 130, 128, True), (2, 130, 127, False),
    (300, 90, 0, True), (128, 129, 1, True), (128, 129, 0, False)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(24, 40, 4, 2), (64, 64, 6, 1), (128, 128, 2, 2)])
@pytest.mark.parametrize("q_len", [1, 2, 37])
def test_keys_at_every_edge_stand_out(dtype, shape, q_len):
    """With the cap at 30, a distance table and a learned sink at work: a probe key that the query may see takes
    nearly all the weight (the output is about 50), one that it may not see leaves the output small."""
    hd, hdv, n_q, n_kv = shape
    for window, n, probe, visible in EDGES:
        if q_len > n:
            continue
        got, want, ok = _edge_case(dtype, hd, hdv, n_q, n_kv, window, n, q_len, probe, 30.0, 10, -1.0)
        assert ok == visible
        assert float((got - want).abs().max()) <= (1e-3 if dtype == "float32" else 0.6), (window, n, probe)
        assert (float(got.abs().max()) > 25) == visible, (window, n, probe, float(got.abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rank,rot,heads", [(48, 8, 3), (128, 16, 4), (512, 64, 2)])
@pytest.mark.parametrize("q_len", [1, 30])
def test_a_far_key_stands_out_in_latent_rows(dtype, rank, rot, heads, q_len):
    """One key head whose rows are key and value at once (the values are the first `rank` entries of the rows),
    causal: a key hundreds of positions back, at a page's first and last place, the first token."""
    for n, probe in ((700, 0), (700, 63), (700, 64), (700, 699 - 400), (65, 64), (1 + q_len, 0)):
        got, want, ok = _edge_case(dtype, rank + rot, rank, heads, 1, 0, max(n, q_len), q_len, probe, 0.0, 0, None,
                                   latent=rank)
        assert ok
        assert float((got - want).abs().max()) <= (1e-3 if dtype == "float32" else 0.6), (n, probe)
        assert float(got.abs().max()) > 25, (n, probe)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sink_and_the_cap_take_their_share(dtype):
    """A sink of score 4 against one visible key of capped score: the weight of the key is exp(s) / (exp(s) + exp(4)),
    so leaving the sink out, scaling it, or leaving the cap out each moves the output by a large factor."""
    for cap, sink in ((2.0, 4.0), (30.0, 4.0), (2.0, -3.0), (0.0, 9.0)):
        got, want, _ = _edge_case(dtype, 32, 24, 2, 1, 1, 70, 1, 69, cap, 0, sink)
        assert float((got - want).abs().max()) <= (1e-3 if dtype == "float32" else 0.3), (cap, sink)
    capped, _, _ = _edge_case(dtype, 32, 24, 2, 1, 1, 70, 1, 69, 2.0, 0, 4.0)
    uncapped, _, _ = _edge_case(dtype, 32, 24, 2, 1, 1, 70, 1, 69, 0.0, 0, 4.0)
    assert float(capped.abs().max()) < 0.3 * float(uncapped.abs().max())


# ------------------------------------------------------------------------------------------ the engine
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_every_schedule_matches_plain(tag, dtype):
    """Whole prompts; the last tokens one by one (more of them than the longest window); unequal batches in which
    shorter requests end early and the next batch takes their slots and pages; prompts in pieces of 2, 7, 64 and
    100 tokens; a prompt in pieces beside sequences that go on by one token."""
    requests = requests_for(tag)
    want = oracle(tag, requests)
    engine = engine_for(tag, dtype)
    plans = {"whole": helpers.plan_whole(requests), "tail": helpers.plan_tail(requests, 120),
             "batched": helpers.plan_batched(requests, 3, 0.6), "mixed": helpers.plan_mixed(requests, 9)}
    some = {rid: toks for rid, toks in requests.items() if len(toks) <= 200}
    for chunk in (2, 7, 64, 100):
        plans[f"pieces of {chunk}"] = helpers.plan_chunked(some if chunk == 2 else requests, chunk)
    for name, steps in plans.items():
        got = helpers.run_plan_engine(engine, steps)
        compare(got, {rid: want[rid] for rid in got}, dtype, f"{tag}/{dtype}/{name}")
        assert engine.cache.free_slots() == engine.cache.n_slots and engine.cache.free_pages() == engine.cache.n_pages
    if dtype == "bfloat16":
        from llm_infer_engine_b200.kernels import ops
        ops.check_tc_status("cuda")


def test_the_models_are_sharp_enough_to_show_what_a_fault_would_change():
    """The bounds above mean something only if a fault moves the logits by more than they allow. In the plain
    implementation: a window one token off, the sink left out, the distance table shifted by one row and the cap left
    out each differ by several bfloat16 bounds."""
    for tag in ("a", "b", "c"):
        w, cfg = plain_weights(tag), CFGS[tag]
        toks = helpers.random_tokens(cfg["vocab"], max(LENGTHS[tag]), seed=47)
        right = plain.forward(w, cfg, toks)

        def gap(cfg2, w2, factor):
            """The fault must move more positions than `compare` forgives, and the worst by `factor` bounds."""
            diff = (plain.forward(w2, cfg2, toks) - right).abs().max(dim=1).values
            tol = bound("bfloat16", right)
            assert int((diff > tol).sum()) > max(1, len(diff) // 25) and float(diff.max()) > factor * tol, (
                tag, int((diff > tol).sum()), float(diff.max()), tol)

        off = json.loads(json.dumps(cfg))
        for layer in off["layers"]:
            if layer["type"] == "attention" and layer["mixer"]["mask"]:
                layer["mixer"]["mask"]["size"] += 1
        gap(off, w, 2)
        gap(cfg, {k: (v - 30.0 if k.endswith(".sink") else v) for k, v in w.items()}, 2)
        gap(cfg, {k: (torch.roll(v, 1, 0) if k.endswith(".rel") else v) for k, v in w.items()}, 3)
        no_cap = json.loads(json.dumps(cfg))
        for layer in no_cap["layers"]:
            if layer["type"] == "attention":
                layer["mixer"]["softcap"] = 1e6
        gap(no_cap, w, 1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_and_cutting_do_not_change_a_row(dtype):
    """The logits of a position do not depend on what else is in the batch or how the prompt was cut: float32
    kernels sum in a fixed order, so there the rows are equal bit for bit."""
    tag = "a"
    requests = requests_for(tag)
    engine = engine_for(tag, dtype)
    alone = helpers.run_plan_engine(engine, helpers.plan_whole(requests))
    together = helpers.run_plan_engine(engine, helpers.plan_batched(requests, 8, 1.0))
    for rid in requests:
        if dtype == "float32":
            assert torch.equal(alone[rid], together[rid]), rid
        else:
            assert float((alone[rid] - together[rid]).abs().max()) <= bound(dtype, alone[rid])


def test_trace_run_program_and_other_sizes_at_once(tmp_path):
    """bin/trace_run as a subprocess on the configuration with the odd sizes."""
    tag = "b"
    requests = {k: v for k, v in requests_for(tag).items() if len(v) <= 200}
    want = oracle(tag, requests)
    steps = helpers.plan_batched(requests, 4, 0.5)
    peak = max(sum(len(v) for v in requests.values()), 64)
    for dtype in ("float32", "bfloat16"):
        got = helpers.run_plan_trace_run(folder_for(tag), dtype, steps, peak, CFGS[tag]["vocab"])
        compare(got, want, dtype, f"trace_run/{dtype}")


@pytest.mark.parametrize("dtype,gap", [("float32", 1e-4), ("bfloat16", 0.3)])
@pytest.mark.parametrize("graph", [True, False])
def test_greedy_generation_through_the_library(dtype, gap, graph):
    """generate(): admission, ragged prompts, captured one-token steps (the routed feed-forward's sort included),
    slots used again. Greedy tokens equal the plain implementation's; where they part the two candidates are a
    near-tie in the plain logits."""
    from llm_infer_engine_b200 import GenerationStats, generate
    tag = "a"
    w, cfg = plain_weights(tag), CFGS[tag]
    prompts = [helpers.random_tokens(cfg["vocab"], n, seed=60 + i) for i, n in enumerate([1, 5, 42, 64, 3, 90, 2])]
    engine = engine_for(tag, dtype, max_batch=3, max_tokens=64 * 12, cuda_graph=graph)
    stats = GenerationStats()
    out = generate(engine, prompts, max_new_tokens=40, stop_ids=[], stats=stats)          # decoding crosses the window
    assert stats.batches >= 3 and [len(o) for o in out] == [40] * len(prompts)
    for p, o in zip(prompts, out):
        seq = list(p)
        for tok in o:
            row = plain.forward(w, cfg, seq)[-1]
            best = int(row.argmax())
            if tok != best:
                assert float(row[best] - row[tok]) < gap, (len(seq), tok, best)
            seq.append(tok)
    engine.cache.check()
    assert engine.cache.free_slots() == 3 and engine.cache.free_pages() == engine.cache.n_pages


def test_long_decoding_in_float32():
    """A few hundred captured one-token steps against one whole-sequence pass; the window passes over decoded
    tokens many times and the latent layers read keys hundreds of positions back."""
    from llm_infer_engine_b200 import generate
    tag = "b"
    w, cfg = plain_weights(tag), CFGS[tag]
    prompt = helpers.random_tokens(cfg["vocab"], 4, seed=70)
    engine = engine_for(tag, "float32", max_batch=2, max_tokens=64 * 12, cuda_graph=True)
    out = generate(engine, [prompt, prompt[:1]], max_new_tokens=260, stop_ids=[])
    for p, o in zip([prompt, prompt[:1]], out):
        seq = p + o
        ref = plain.forward(w, cfg, seq[:-1])
        picks = ref[len(p) - 1:].argmax(-1).tolist()
        for i, (a, b) in enumerate(zip(o, picks)):
            if a != b:
                row = ref[len(p) - 1 + i]
                assert float(row[b] - row[a]) < 1e-4, (i, a, b)
                break


def test_command_line_generates_with_this_design(tmp_path):
    import subprocess
    import sys
    tag = "c"
    w, cfg = plain_weights(tag), CFGS[tag]
    prompt = helpers.random_tokens(cfg["vocab"], 9, seed=80)
    proc = subprocess.run([sys.executable, os.path.join(helpers.ROOT, "main.py"), "--model", folder_for(tag),
                           "--prompt-ids", ",".join(map(str, prompt)), "--dtype", "float32", "--max-new-tokens", "6",
                           "--temperature", "0", "--env-file", str(tmp_path / "none")],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    ids = [int(x) for x in proc.stdout.split("OUTPUT")[1].split("=" * 70)[1].split()]
    seq = list(prompt)
    for tok in ids:
        row = plain.forward(w, cfg, seq)[-1]
        assert tok == int(row.argmax()) or float(row.max() - row[tok]) < 1e-4
        seq.append(tok)
    assert len(ids) == 6
