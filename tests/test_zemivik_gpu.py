"""Zemivik on the GPU against its plain restatement (tests/plain_zemivik.py): each kernel and part alone, the
attention's edges with scores made to stand out, and the engine in float32 and bfloat16 over whole prompts,
token-by-token decoding, prompts in pieces down to two tokens, unequal batches with slots and pages used again,
long decoding and greedy generation through the library's own entry point."""
import json
import math
import os

import pytest
import torch

import helpers
import plain_zemivik as plain
from test_parts_gpu import DEV, DTYPES, build, kernel_plan, make_ctx

pytestmark = pytest.mark.gpu

CFGS = {"a": plain.TINY_A, "b": plain.TINY_B, "c": plain.TINY_C}
_folders, _engines = {}, {}


def folder_for(tag):
    from llm_infer_engine_b200 import write_random_model
    if tag not in _folders:
        d = helpers.scratch_folder(f"llmie_zemivik_{tag}_")
        write_random_model(CFGS[tag], d, seed=11 + len(_folders), std=0.08, norm_range=(0.7, 1.3))
        _folders[tag] = d
    return _folders[tag]


def engine_for(tag, dtype, **kw):
    from llm_infer_engine_b200 import Engine
    key = (tag, dtype, tuple(sorted(kw.items())))
    if key not in _engines:
        _engines[key] = Engine(folder_for(tag), dtype=dtype, max_batch=kw.pop("max_batch", 8),
                               max_tokens=kw.pop("max_tokens", 64 * 48), cuda_graph=kw.pop("cuda_graph", False), **kw)
    return _engines[key]


def bound(dtype, want):
    """float32 agrees to rounding. bfloat16 rounds every activation between kernels; its bound is a share of the
    request's largest logit (scores this sharp carry the rounding of q and k into the weights), several times below
    what a lost or added key changes on these models."""
    return (3e-5 if dtype == "float32" else 0.1) * max(1.0, float(want.abs().max()))


def oracle(tag, requests):
    w, cfg = helpers.plain_weights(folder_for(tag)), CFGS[tag]
    return {rid: plain.logits(w, cfg, toks) for rid, toks in requests.items()}


def compare(got, want, dtype, what):
    """float32: every position within the bound. bfloat16: sharp scores amplify the rounding of q and k where two
    keys nearly tie, so a few positions stray: at most one in fifty may exceed the bound, none two and a half
    times it (a mask that is one token off moves hundreds of positions by ten bounds)."""
    for rid in want:
        assert got[rid].shape == want[rid].shape, (what, rid)
        diff = (got[rid] - want[rid]).abs().max(dim=1).values
        tol = bound(dtype, want[rid])
        over = int((diff > tol).sum())
        allowed = 0 if dtype == "float32" else max(1, len(diff) // 50)
        worst_ok = tol if dtype == "float32" else 2.5 * tol
        assert over <= allowed and float(diff.max()) <= worst_ok, (
            f"{what}: request {rid}: {over} of {len(diff)} positions over the bound {tol:.3e}, worst "
            f"{float(diff.max()):.3e}, first at token {int((diff > tol).nonzero()[0])}")


# ------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_stage_part(dtype):
    stage, w = build("pointwise", "embedding_stage", {"size": 72, "scale": 1.7, "positions": 50, "norm_eps": 2e-6,
                                                      "names": {"positions": "p", "norm": "n"}}, dtype, seed=4)
    ctx = make_ctx([5, 3], [40, 0], [0, 1], dtype)
    g = torch.Generator().manual_seed(5)
    h = torch.randn(8, 72, generator=g)
    hd = h.clone().to(DEV)
    stage.forward(hd, ctx)
    pos = torch.tensor([40, 41, 42, 43, 44, 0, 1, 2])
    want = plain.rms_norm(h * 1.7 + w["p"][pos], w["n"], 2e-6)
    assert float((hd.cpu() - want).abs().max()) < 1e-5
    if dtype == "bfloat16":
        assert torch.equal(ctx.carry["h_act"].cpu(), hd.cpu().to(torch.bfloat16))
    # each stage alone: no table, no norm
    bare, _ = build("pointwise", "embedding_stage", {"size": 72, "scale": 0.5}, dtype)
    hd = h.clone().to(DEV)
    bare.forward(hd, make_ctx([8], [0], [0], dtype))
    assert float((hd.cpu() - h * 0.5).abs().max()) < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("y_dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", [200, 204, 2048])           # 16-byte accesses, element by element, a wide row
def test_norm_on_a_branch_output(dtype, y_dtype, size):
    norm, w = build("norm", "rmsnorm", {"size": size, "eps": 1e-4, "weight_name": ""}, dtype, seed=6)
    assert list(w) == [""]
    g = torch.Generator().manual_seed(7)
    h, y, bias = torch.randn(9, size, generator=g), torch.randn(9, size, generator=g) * 5, torch.randn(size, generator=g)
    y = y.to(DTYPES[y_dtype])
    for b in (None, bias):
        hd = h.clone().to(DEV)
        act = torch.empty(9, size, dtype=DTYPES[dtype], device=DEV)
        norm.add_normed(hd, y.to(DEV), None if b is None else b.to(DEV), act)
        want = h + plain.rms_norm(y.float() + (0 if b is None else b), w[""], 1e-4)
        assert float((hd.cpu() - want).abs().max()) < 2e-5
        assert torch.equal(act.cpu(), hd.cpu().to(DTYPES[dtype]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("activation,inner", [("relu2", 100), ("relu2", 128), ("relu", 104), ("gelu_tanh", 100), ("silu", 96)])
def test_dense_mlp_part(dtype, activation, inner):
    """Widths that take the one-kernel product with bias and activation (one-token steps of a bfloat16 engine), the
    16-byte kernels and the element-by-element ones."""
    ff, w = build("feed_forward", "dense_mlp", {"hidden": 96 if inner == 128 else 72, "intermediate": inner,
                                                "activation": activation}, dtype, seed=8)
    hidden = ff.hidden
    g = torch.Generator().manual_seed(9)
    for rows in (3, 40):
        x = torch.randn(rows, hidden, generator=g).to(DTYPES[dtype])
        z = x.float() @ w["up"].T + w["up.b"]
        a = {"relu2": torch.relu(z) ** 2, "relu": torch.relu(z), "silu": z * torch.sigmoid(z),
             "gelu_tanh": 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))}[activation]
        want = a @ w["down"].T + w["down.b"]
        got = ff.forward(x.to(DEV), make_ctx([rows], [0], [0], dtype))
        assert got.dtype == torch.float32
        assert float((got.cpu() - want).abs().max()) <= (2e-5 if dtype == "float32" else 3e-2) * max(1.0, float(want.abs().max()))
        bare = ff.forward(x.to(DEV), make_ctx([rows], [0], [0], dtype), defer_bias=True)
        assert float((bare.cpu() + w["down.b"] - got.cpu()).abs().max()) < 1e-5
    if activation == "relu2":
        same, _ = build("feed_forward", "dense_mlp", {"hidden": hidden, "intermediate": inner}, dtype, seed=8)   # the default
        assert same.activation == ff.activation


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("blend", [False, True])
@pytest.mark.parametrize("shape,extra", [((6, 2, 20, 12), 9), ((4, 2, 64, 32), 8), ((5, 5, 16, 40), 16)])
def test_query_key_norm_blend_and_cache_write(dtype, blend, shape, extra):
    from llm_infer_engine_b200.cache import Cache, KVRequest
    from llm_infer_engine_b200.kernels import ops
    n_q, n_kv, hd, hdv = shape
    cache = Cache([[KVRequest(n_kv, hd, v_head_dim=hdv)]], 3, 64 * 6, 512, DTYPES[dtype], DEV)
    slots = [cache.take_slot() for _ in range(2)]
    lens, starts = [70, 3], [0, 0]
    for s, l in zip(slots, lens):
        cache.reserve(s, l)
    ctx = make_ctx(lens, starts, slots, dtype)
    g = torch.Generator().manual_seed(10)
    T, width = sum(lens), n_q * hd + n_kv * hd + n_kv * hdv + extra               # more columns follow v
    proj = (torch.randn(T, width, generator=g) * 3).to(DTYPES[dtype])
    first = torch.randn(T, n_kv * hdv + (5 if extra == 9 else 8), generator=g).to(DTYPES[dtype])
    qw, kw = torch.rand(n_q * hd, generator=g) + 0.5, torch.rand(n_kv * hd, generator=g) + 0.5
    lam = torch.tensor([0.3])
    kv = cache.unit(0).kv
    q = torch.empty(T, n_q * hd, dtype=DTYPES[dtype], device=DEV)
    ops.qk_norm_store(proj.to(DEV), q, kv.k, kv.v, qw.to(DEV), kw.to(DEV), 1e-5, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot,
                      kv.block_table, kv.page_size, n_q, n_kv, hd, hdv, True, lam=lam.to(DEV) if blend else None,
                      v_first=first.to(DEV)[:, :n_kv * hdv] if blend else None)
    p = proj.float()
    q_want = plain.rms_norm(p[:, :n_q * hd], qw, 1e-5)
    k_want = plain.rms_norm(p[:, n_q * hd:(n_q + n_kv) * hd], kw, 1e-5)
    v_want = p[:, (n_q + n_kv) * hd:(n_q + n_kv) * hd + n_kv * hdv]
    if blend:
        v_want = plain.blend_values(v_want, first.float()[:, :n_kv * hdv], lam)
    t = 2e-5 if dtype == "float32" else 3e-2
    assert float((q.float().cpu() - q_want).abs().max()) <= t * float(q_want.abs().max())
    row = 0
    for i, l in enumerate(lens):
        table = kv.block_table[slots[i]].cpu()
        for pos in (0, 63, 64, l - 1):
            if pos >= l:
                continue
            page = int(table[pos // 64])
            k_got = kv.k[page, :, pos % 64].float().cpu().reshape(-1)
            v_got = kv.v[page, :, pos % 64].float().cpu().reshape(-1)
            assert float((k_got - k_want[row + pos]).abs().max()) <= t * float(k_want.abs().max())
            assert float((v_got - v_want[row + pos]).abs().max()) <= t * float(v_want.abs().max())
        row += l


@pytest.mark.parametrize("batch", [1, 5, 8])
@pytest.mark.parametrize("K,N", [(96, 48), (2048, 160)])
def test_branch_add_folded_into_the_next_product(batch, K, N):
    """h_out = h + norm(y + bias) * w and out = h_out W^T (or relu(h_out W^T + b)^2) in one kernel, against the two
    steps done apart in float64."""
    from llm_infer_engine_b200.kernels import ops
    g = torch.Generator().manual_seed(batch + K)
    h, y = torch.randn(batch, K, generator=g) * 2, torch.randn(batch, K, generator=g) * 7
    y_bias, norm_w = torch.randn(K, generator=g), torch.rand(K, generator=g) + 0.5
    W = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    out_bias = torch.randn(N, generator=g)
    for yb in (None, y_bias):
        want_h = h.double() + plain.rms_norm(y.double() + (0 if yb is None else yb.double()), norm_w.double(), 1e-5)
        z = want_h.to(torch.bfloat16).double() @ W.double().T
        for act, want in ((None, z), (ops.ACT_RELU2, torch.relu(z + out_bias.double()) ** 2)):
            h_dev = h.to(DEV)
            h_out = torch.empty_like(h_dev)
            out = torch.empty(batch, N, dtype=torch.bfloat16, device=DEV)
            ops.branch_norm_gemm(h_dev, y.to(DEV), None if yb is None else yb.to(DEV), norm_w.to(DEV), 1e-5, h_out,
                                 W.to(DEV), out, out_bias.to(DEV) if act is not None else None, act)
            assert torch.equal(h_dev.cpu(), h)                                      # the stream that was read is untouched
            assert float((h_out.cpu().double() - want_h).abs().max()) < 1e-5
            assert float((out.float().cpu().double() - want).abs().max()) <= 2e-2 * max(1.0, float(want.abs().max()))


# ------------------------------------------------------------------------------------------ the attention's edges
def _edge_case(dtype, hd, hdv, n_q, n_kv, window, keep, n, q_len, probe, sink):
    """A sequence of n keys of which the last q_len are this step's queries; the LAST query points straight at key
    `probe`, whose value is a marker. Returns (got, want) rows of the last query and whether it may see the probe."""
    from llm_infer_engine_b200.cache import Cache, KVRequest
    from llm_infer_engine_b200.parts import AttentionOptions
    cache = Cache([[KVRequest(n_kv, hd, window, v_head_dim=hdv, keep_first=keep)]], 4, 64 * 24, 1024, DTYPES[dtype], DEV)
    cache.take_slot()                                     # slot 0 stays empty: the sequence below does not start at page 0
    other = cache.take_slot()
    cache.reserve(other, 130)
    slot = cache.take_slot()
    cache.reserve(slot, 70)
    cache.give_back_slot(other)                           # its pages come back and are used again, out of order
    cache.reserve(slot, n)
    g = torch.Generator().manual_seed(n * 7 + probe)
    k = torch.randn(n, n_kv, hd, generator=g) * 0.3
    v = torch.randn(n, n_kv, hdv, generator=g)
    q = torch.randn(q_len, n_q, hd, generator=g) * 0.3
    direction = torch.nn.functional.normalize(torch.randn(hd, generator=g), dim=0)
    k[probe] = direction * 6.0
    q[-1] = direction * 6.0                               # score 36 * scale against the probe, about 0 elsewhere
    v[probe] = 50.0
    k, v, q = (t.to(DTYPES[dtype]) for t in (k, v, q))
    kv = cache.unit(0).kv
    table = kv.block_table[slot].cpu()
    for j in range(n):
        kv.k[int(table[j // 64]), :, j % 64] = k[j].to(DEV)
        kv.v[int(table[j // 64]), :, j % 64] = v[j].to(DEV)
    ctx = make_ctx([q_len], [n - q_len], [slot], dtype, kernels=kernel_plan(dtype))
    out = torch.empty(q_len, n_q * hdv, dtype=DTYPES[dtype], device=DEV)
    scale = 0.5
    ctx.attention(q.reshape(q_len, -1).to(DEV), kv, out, n_q, n_kv, hd,
                  AttentionOptions(scale=scale, window=window, keep_first=keep, sink=sink))
    ok = plain.visible(n, window, keep)[n - 1:]
    want = []
    for h in range(n_q):
        s = (q[-1, h].double() @ k[:, h // (n_q // n_kv)].double().T)[None] * scale
        if sink:
            p = plain.softmax_with_sink(s, ok)
        else:
            p = torch.softmax(s.masked_fill(~ok, -math.inf), -1)
        want.append(p @ v[:, h // (n_q // n_kv)].double())
    return out[-1].float().cpu(), torch.cat(want, -1).float().reshape(-1), bool(ok[0, probe])


EDGES = [  # window, kept first, keys, probe, may the last query (position keys - 1) see it
    (80, 5, 300, 220, True), (80, 5, 300, 219, False),          # just inside and just outside the window
    (80, 5, 300, 4, True), (80, 5, 300, 5, False),              # the last kept token and the first that is not
    (80, 5, 300, 0, True), (64, 0, 300, 0, False),              # the very first token, kept or not
    (64, 0, 257, 193, True), (64, 0, 257, 192, False),          # the window's edge on a page's edge
    (65, 64, 257, 63, True), (65, 64, 257, 64, False),          # a whole page kept
    (100, 70, 640, 69, True), (100, 70, 640, 70, False),        # kept tokens on the second page, far from the query
    (0, 0, 500, 3, True), (0, 0, 500, 255, True),               # no window: a key far back
    (7, 9, 40, 8, True), (7, 9, 40, 32, False), (7, 9, 40, 33, True), (500, 3, 90, 10, True)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(24, 40, 4, 2), (64, 64, 6, 1), (128, 128, 2, 2)])
@pytest.mark.parametrize("q_len", [1, 2, 37])
def test_keys_at_every_edge_stand_out(dtype, shape, q_len):
    """One score is made to tower over the rest, so a key wrongly seen or wrongly hidden changes the output from
    about 0 to about 50. Decoding (one query) and prompt portions (2 and 37 queries, the probing query last)."""
    hd, hdv, n_q, n_kv = shape
    for window, keep, n, probe, visible in EDGES:
        for sink in (True, False):
            got, want, seen = _edge_case(dtype, hd, hdv, n_q, n_kv, window, keep, n, q_len, probe, sink)
            assert seen == visible
            assert (float(want.abs().max()) > 40) == visible, (window, keep, n, probe)
            tol = 1e-4 if dtype == "float32" else 0.5
            assert float((got - want).abs().max()) <= tol, (shape, q_len, window, keep, n, probe, sink,
                                                             float((got - want).abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sink_takes_its_share_and_gate_scales_the_output(dtype):
    """With every score far below zero nearly all the weight goes to the sink and the output is about zero; the
    gate multiplies the heads by its sigmoid inside the same call."""
    from llm_infer_engine_b200.cache import Cache, KVRequest
    from llm_infer_engine_b200.parts import AttentionOptions
    n_q, n_kv, hd, hdv, n = 4, 2, 16, 24, 90
    cache = Cache([[KVRequest(n_kv, hd, v_head_dim=hdv)]], 2, 64 * 4, 256, DTYPES[dtype], DEV)
    slot = cache.take_slot()
    cache.reserve(slot, n)
    kv = cache.unit(0).kv
    g = torch.Generator().manual_seed(12)
    k = torch.nn.functional.normalize(torch.randn(hd, generator=g), dim=0).repeat(n, n_kv, 1)
    v = torch.randn(n, n_kv, hdv, generator=g)
    table = kv.block_table[slot].cpu()
    for j in range(n):
        kv.k[int(table[j // 64]), :, j % 64] = k[j].to(DEV, DTYPES[dtype])
        kv.v[int(table[j // 64]), :, j % 64] = v[j].to(DEV, DTYPES[dtype])
    ctx = make_ctx([n], [0], [slot], dtype, kernels=kernel_plan(dtype))
    q = (-20.0 * k[:, :1]).repeat(1, n_q, 1).reshape(n, -1).to(DEV, DTYPES[dtype])       # every score is -20
    out = torch.empty(n, n_q * hdv, dtype=DTYPES[dtype], device=DEV)
    ctx.attention(q, kv, out, n_q, n_kv, hd, AttentionOptions(scale=1.0, sink=True))
    assert float(out.float().abs().max()) < 1e-5
    ctx.attention(q, kv, out, n_q, n_kv, hd, AttentionOptions(scale=1.0, sink=False))
    assert float(out.float().abs().max()) > 0.1                                          # without the sink: a mean of values
    ungated = out.clone()
    gate = torch.randn(n, n_q * hdv + 6, generator=g).to(DEV, DTYPES[dtype])
    ctx.attention(q, kv, out, n_q, n_kv, hd, AttentionOptions(scale=1.0, sink=False), gate=gate[:, 3:3 + n_q * hdv])
    want = ungated.float() * torch.sigmoid(gate[:, 3:3 + n_q * hdv].float())
    assert float((out.float() - want).abs().max()) <= (1e-5 if dtype == "float32" else 2e-2)


@pytest.mark.parametrize("hd", [64, 128])
def test_decode_attention_in_runs_with_kept_keys_sink_and_gate(hd):
    """The tensor-core decode kernel cut into runs of 1, 2, 3 and 5 pages (runs below the window hold only the
    kept first keys, runs in between hold nothing and are skipped) against the plain kernel, for sequences of
    unequal lengths, some shorter than the window or than the kept prefix."""
    from llm_infer_engine_b200.cache import Cache, KVRequest
    from llm_infer_engine_b200.kernels import ops
    n_q, n_kv = 8, 2
    lens = [700, 64, 65, 130, 3, 391]
    cache = Cache([[KVRequest(n_kv, hd, 150, keep_first=70)]], len(lens), 64 * 40, 1024, torch.bfloat16, DEV)
    slots = [cache.take_slot() for _ in lens]
    for s_, l in zip(slots, lens):
        cache.reserve(s_, l)
    kv = cache.unit(0).kv
    g = torch.Generator().manual_seed(21)
    kv.k.copy_((torch.randn(kv.k.shape, generator=g) * 0.5).to(DEV, torch.bfloat16))
    kv.v.copy_(torch.randn(kv.v.shape, generator=g).to(DEV, torch.bfloat16))
    q = torch.randn(len(lens), n_q * hd, generator=g).to(DEV, torch.bfloat16)
    gate = torch.randn(len(lens), n_q * hd + 16, generator=g).to(DEV, torch.bfloat16)
    ctx = make_ctx([1] * len(lens), [l - 1 for l in lens], slots, "bfloat16")
    for window, keep, sink, gated in [(150, 70, True, True), (150, 70, False, False), (64, 130, True, False),
                                      (0, 0, True, True), (300, 1, False, True)]:
        gt = gate[:, 8:8 + n_q * hd] if gated else None
        want = torch.empty_like(q)
        ops.attention_paged(q, kv.k, kv.v, want, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, kv.block_table, 64, n_q, n_kv,
                            hd, 0.2, window, keep, sink, gt)
        for pages in (1, 2, 3, 5, 16):
            n_runs = (max(lens) + 64 * pages - 1) // (64 * pages)
            out = torch.empty_like(q)
            counters = torch.zeros(ops.decode_counter_ints(len(lens), n_q, n_kv), dtype=torch.int32, device=DEV)
            ops.attention_decode_mma(q, kv.k, kv.v, out, ctx.seq_slot, ctx.seq_kvlen, kv.block_table, 64, n_q, n_kv, hd,
                                     0.2, window, pages, n_runs, counters=counters, keep_first=keep, sink=sink, gate=gt)
            assert float((out.float() - want.float()).abs().max()) < 2e-2, (window, keep, sink, gated, pages)
            assert int(counters.abs().sum()) == 0


# ------------------------------------------------------------------------------------------ the engine
LENGTHS = {"a": [1, 2, 43, 44, 64, 65, 130, 300], "b": [3, 8, 33, 34, 100, 128, 129, 380], "c": [5, 71, 151, 215, 64, 700]}


def requests_for(tag):
    return {f"r{i}": helpers.random_tokens(CFGS[tag]["vocab"], n, seed=40 + i) for i, n in enumerate(LENGTHS[tag])}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_every_schedule_matches_plain(tag, dtype):
    """Whole prompts; the last tokens one by one (more of them than the longest window); unequal batches in which
    shorter requests end early and the next batch takes their slots and pages; prompts in pieces of 2, 7, 64 and
    100 tokens; a prompt in pieces beside sequences that go on by one token."""
    requests = requests_for(tag)
    want = oracle(tag, requests)
    engine = engine_for(tag, dtype)
    plans = {"whole": helpers.plan_whole(requests), "tail": helpers.plan_tail(requests, 210),
             "batched": helpers.plan_batched(requests, 3, 0.6), "mixed": helpers.plan_mixed(requests, 9)}
    some = {rid: toks for rid, toks in requests.items() if len(toks) <= 300}
    for chunk in (2, 7, 64, 100):
        plans[f"pieces of {chunk}"] = helpers.plan_chunked(some if chunk == 2 else requests, chunk)
    for name, steps in plans.items():
        got = helpers.run_plan_engine(engine, steps)
        compare(got, {rid: want[rid] for rid in got}, dtype, f"{tag}/{dtype}/{name}")
        assert engine.cache.free_slots() == engine.cache.n_slots and engine.cache.free_pages() == engine.cache.n_pages
    if dtype == "bfloat16":
        from llm_infer_engine_b200.kernels import ops
        ops.check_tc_status("cuda")


def test_the_models_are_sharp_enough_to_show_a_mask_that_is_one_off():
    """The bounds above mean something only if a window or a kept prefix that is one token off moves the logits
    by more than they allow: the plain implementation with such a mask must differ by several bounds (here:
    at least three of the bfloat16 bound, which is thousands of the float32 bound)."""
    for tag in ("a", "b", "c"):
        w, cfg = helpers.plain_weights(folder_for(tag)), CFGS[tag]
        toks = helpers.random_tokens(cfg["vocab"], max(LENGTHS[tag]), seed=47)
        right = plain.logits(w, cfg, toks)
        for what, change in (("window", ("size", 1)), ("window", ("size", -1)), ("kept", ("keep_first", 1))):
            off = json.loads(json.dumps(cfg))
            for layer in off["layers"]:
                if layer["mixer"]["mask"]:
                    layer["mixer"]["mask"][change[0]] = max(0, layer["mixer"]["mask"][change[0]] + change[1])
            wrong = plain.logits(w, off, toks)
            gap = float((wrong - right).abs().max())
            assert gap > 3 * bound("bfloat16", right), (tag, what, gap, bound("bfloat16", right))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_and_cutting_do_not_change_a_row(dtype):
    """The logits of a position do not depend on what else is in the batch or how the prompt was cut: float32
    kernels sum in a fixed order, so there the rows are equal bit for bit."""
    tag = "b"
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
    """bin/trace_run as a subprocess on the configuration whose layers all differ."""
    tag = "b"
    requests = {k: v for k, v in requests_for(tag).items() if len(v) < 200}
    want = oracle(tag, requests)
    steps = helpers.plan_batched(requests, 4, 0.5)
    peak = max(sum(len(v) for v in requests.values()), 64)
    for dtype in ("float32", "bfloat16"):
        got = helpers.run_plan_trace_run(folder_for(tag), dtype, steps, peak, CFGS[tag]["vocab"])
        compare(got, want, dtype, f"trace_run/{dtype}")


@pytest.mark.parametrize("dtype,gap", [("float32", 1e-4), ("bfloat16", 0.3)])
@pytest.mark.parametrize("graph", [True, False])
def test_greedy_generation_through_the_library(dtype, gap, graph):
    """generate(): admission, ragged prompts, captured one-token steps, slots used again. Greedy tokens equal the
    plain implementation's; where they part the two candidates are a near-tie in the plain logits."""
    from llm_infer_engine_b200 import GenerationStats, generate
    tag = "a"
    w, cfg = helpers.plain_weights(folder_for(tag)), CFGS[tag]
    prompts = [helpers.random_tokens(cfg["vocab"], n, seed=60 + i) for i, n in enumerate([1, 5, 42, 64, 3, 90, 2])]
    engine = engine_for(tag, dtype, max_batch=3, max_tokens=64 * 12, cuda_graph=graph)
    stats = GenerationStats()
    out = generate(engine, prompts, max_new_tokens=50, stop_ids=[], stats=stats)          # decoding crosses the window
    assert stats.batches >= 3 and [len(o) for o in out] == [50] * len(prompts)
    for p, o in zip(prompts, out):
        seq = list(p)
        for tok in o:
            row = plain.logits(w, cfg, seq)[-1]
            best = plain.greedy(row)
            if tok != best:
                assert float(row[best] - row[tok]) < gap, (len(seq), tok, best)
            seq.append(tok)
    engine.cache.check()
    assert engine.cache.free_slots() == 3 and engine.cache.free_pages() == engine.cache.n_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_captured_lone_prompt_equals_the_eager_one(dtype):
    """A lone prompt whose length comes again is replayed as one captured step (any slot, any start position);
    its logits must be those of the eager step: bit for bit in float32."""
    tag = "c"
    eager = engine_for(tag, dtype)
    captured = engine_for(tag, dtype, max_batch=4, max_tokens=64 * 24, cuda_graph=True)
    prompts = [helpers.random_tokens(CFGS[tag]["vocab"], 150, seed=90 + i) for i in range(4)]
    taken = captured.open()                                   # the replays use another slot than the first run
    for i, p in enumerate(prompts):
        want_slot, got_slot = eager.open(), captured.open()
        want = eager.step([want_slot], [p[:100]], "last")
        got = captured.step([got_slot], [p[:100]], "last")
        want2 = eager.step([want_slot], [p[100:]], "last")     # 50 more tokens at start position 100
        got2 = captured.step([got_slot], [p[100:]], "last")
        for w_, g_ in ((want, got), (want2, got2)):
            if dtype == "float32":
                assert torch.equal(w_, g_), i
            else:
                assert float((w_ - g_).abs().max()) <= bound(dtype, w_)
        eager.close(want_slot)
        captured.close(got_slot)
    captured.close(taken)
    assert any(g and g.graph is not None for g in captured._prefill_graphs.values())


def test_long_decoding_in_float32():
    """Several hundred captured one-token steps against one whole-sequence pass; the window and the kept first
    tokens pass over decoded tokens many times."""
    from llm_infer_engine_b200 import generate
    tag = "a"
    w, cfg = helpers.plain_weights(folder_for(tag)), CFGS[tag]
    prompt = helpers.random_tokens(cfg["vocab"], 4, seed=70)
    engine = engine_for(tag, "float32", max_batch=2, max_tokens=64 * 12, cuda_graph=True)
    out = generate(engine, [prompt, prompt[:1]], max_new_tokens=290, stop_ids=[])
    for p, o in zip([prompt, prompt[:1]], out):
        seq = p + o
        ref = plain.logits(w, cfg, seq[:-1])
        picks = ref[len(p) - 1:].argmax(-1).tolist()
        for i, (a, b) in enumerate(zip(o, picks)):
            if a != b:
                row = ref[len(p) - 1 + i]
                assert float(row[b] - row[a]) < 1e-4, (i, a, b)
                break


def test_command_line_generates_with_this_design(tmp_path):
    import subprocess
    import sys
    tag = "a"
    w, cfg = helpers.plain_weights(folder_for(tag)), CFGS[tag]
    prompt = helpers.random_tokens(cfg["vocab"], 9, seed=80)
    proc = subprocess.run([sys.executable, os.path.join(helpers.ROOT, "main.py"), "--model", folder_for(tag),
                           "--prompt-ids", ",".join(map(str, prompt)), "--dtype", "float32", "--max-new-tokens", "6",
                           "--temperature", "0", "--env-file", str(tmp_path / "none")],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    ids = [int(x) for x in proc.stdout.split("OUTPUT")[1].split("=" * 70)[1].split()]
    seq = list(prompt)
    for tok in ids:
        row = plain.logits(w, cfg, seq)[-1]
        assert tok == plain.greedy(row) or float(row.max() - row[tok]) < 1e-4
        seq.append(tok)
    assert len(ids) == 6
