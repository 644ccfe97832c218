"""Zefenex on the layer-list decoder against the float64 restatement (tests/zefenex_oracle.py): every mechanism alone, prefill against
token-by-token decoding, portions, mixed batches, pages and slots used again, window and page edges in prompts and in decoding, other
sizes, greedy generation through the scheduler, the command line.  All configurations are made here, small, with random weights whose
values are exact in bfloat16."""
import importlib
import json
import os
import struct
import subprocess
import sys

import numpy as np
import pytest
import torch

import zefenex_oracle as ref
from util import b200

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _models():
    return importlib.import_module("llm-inference-engine_b200.models.zefenex")


def _serving():
    return importlib.import_module("llm-inference-engine_b200.serving")


def session(config, packed, dtype="float32", pool_tokens=512, max_seqs=4, max_batch_tokens=512):
    model = _models().ZefenexModel(config, packed, dtype=dtype, device=DEV, max_tokens=max_batch_tokens, max_seqs=max_seqs,
                                   max_pages_per_seq=(pool_tokens + 63) // 64)
    return _serving().Session(model, pool_tokens, max_seqs=max_seqs, max_batch_tokens=max_batch_tokens, poison=True)


def tokens_of(config, n, seed):
    return np.random.default_rng(seed).integers(0, config["vocab"], n).tolist()


def replay(sess, requests, schedule):
    """schedule: list of steps, each a list of (name, n) -- the next n tokens of that request, all positions wanted.
    Returns name -> logits [len(tokens), vocab] (numpy)."""
    fed = {k: 0 for k in requests}
    rid, got = {}, {k: [] for k in requests}
    for step in schedule:
        entries, names = [], []
        for name, n in step:
            if name not in rid:
                rid[name] = sess.open()
            toks = requests[name][fed[name]:fed[name] + n]
            assert len(toks) == n
            entries.append((rid[name], toks, list(range(n))))
            names.append((name, n))
            fed[name] += n
        out = sess.feed(entries).cpu().numpy()
        at = 0
        for name, n in names:
            got[name].append(out[at:at + n])
            at += n
        for name, _ in step:
            if fed[name] == len(requests[name]) and name in rid:
                sess.close(rid.pop(name))
    return {k: np.concatenate(v) for k, v in got.items() if v}


def want_logits(config, W, tokens):
    return ref.forward(config, W, tokens).numpy()


def check_all(got, config, W, requests, tol):
    for name, lg in got.items():
        want = want_logits(config, W, requests[name])
        assert not np.isnan(lg).any(), name
        per_pos = np.linalg.norm(lg - want, axis=-1) / np.linalg.norm(want, axis=-1)
        assert per_pos.max() < tol, (name, int(per_pos.argmax()), float(per_pos.max()))


# windows of 24, 70 and 9 positions over pages of 64; rows shared between layers; dense, routed and no feed-forward; odd sizes
MIXED = [ref.latent_layer(mlp=ref.dense()), ref.latent_layer(heads=2, dim=24, vdim=16, window=70, kv_from=0, mlp=ref.moe()),
         ref.latent_layer(heads=2, dim=12, rot_dim=12, rot_dims=8, vdim=20, kv_rank=20, window=9, scale=0.4, base=50.0),
         ref.latent_layer(heads=5, dim=8, rot_dim=12, rot_dims=8, vdim=8, kv_rank=20, window=100, base=50.0, kv_from=2, mlp=ref.moe(experts=3, identity=0, top=1, ff=16, shared_ff=0))]


# ------------------------------------------------------------------ each mechanism alone (one-layer models, residual stream compared)
@pytest.mark.parametrize("layer", [
    ref.latent_layer(),                                              # window shorter than a page
    ref.latent_layer(heads=1, dim=40, rot_dim=16, vdim=33, kv_rank=24, window=100),  # one head, window across pages
    ref.latent_layer(heads=2, dim=20, rot_dim=12, rot_dims=8, vdim=10, kv_rank=20, window=64),  # part of the rotated dimensions pass unchanged; a cache row of 32 with 20 latent columns
    ref.latent_layer(heads=4, dim=6, rot_dim=2, vdim=5, kv_rank=7, window=1000),  # nothing a multiple of 4; the window never binds
    ref.latent_layer(window=1),                                       # a token sees itself only (and the sink)
    ref.latent_layer(heads=6, dim=64, rot_dim=32, vdim=64, kv_rank=96, window=33, base=500000.0),
    ref.latent_layer(mlp=ref.dense()),
    ref.latent_layer(mlp=ref.dense(ff=7)),
    ref.latent_layer(mlp=ref.moe()),
    ref.latent_layer(mlp=ref.moe(experts=2, identity=0, top=2, ff=8, shared_ff=8)),   # every expert chosen, no identity
    ref.latent_layer(mlp=ref.moe(experts=2, identity=3, top=2, ff=8, shared_ff=0)),   # identity experts chosen often, no shared expert
    ref.latent_layer(mlp=ref.moe(experts=3, identity=1, top=1, ff=16)),               # one choice: its weight is 1
    ref.latent_layer(mlp=ref.moe(experts=70, identity=5, top=4, ff=8, shared_ff=16)),  # more router outputs than a warp
    ref.latent_layer(mlp=ref.moe(experts=1, identity=1, top=2, ff=24)),
], ids=["latent", "one_head", "partial_rotation", "odd_sizes", "window_1", "wide", "dense", "dense_ff7", "moe", "moe_all", "moe_identity",
        "moe_top1", "moe_many", "moe_one_expert"])
def test_one_layer_residual_stream(layer):
    config = ref.make_config([layer])
    W, packed = ref.make_weights(config, seed=3)
    toks = tokens_of(config, 150, 1)
    sess = session(config, packed)
    r = sess.open()
    logits, trace = sess.feed([(r, toks, [0, 1, 149])], trace=True)
    res = []
    want = ref.forward(config, W, toks, res).numpy()
    assert ref.rel_err(trace[0].cpu().numpy(), res[0].numpy()) < 2e-5
    assert ref.rel_err(logits.cpu().numpy(), want[[0, 1, 149]]) < 2e-5


def test_rows_shared_between_layers_and_constants_that_differ_from_one():
    """Two layers read the first layer's rows with their own up-projections, heads, windows and scales; no soft cap, embedding scale 1."""
    layers = [ref.latent_layer(), ref.latent_layer(heads=2, dim=8, vdim=40, window=5, scale=0.7, kv_from=0, mlp=ref.dense()),
              ref.latent_layer(heads=4, dim=12, vdim=4, window=80, kv_from=0)]
    config = ref.make_config(layers, width=40, vocab=33, embed_scale=1.0, softcap=None)
    W, packed = ref.make_weights(config, seed=4)
    toks = tokens_of(config, 130, 2)
    res = []
    want = ref.forward(config, W, toks, res).numpy()
    sess = session(config, packed)
    logits, trace = sess.feed([(sess.open(), toks, list(range(130)))], trace=True)
    for i in range(3):
        assert ref.rel_err(trace[i].cpu().numpy(), res[i].numpy()) < 3e-5, i
    assert ref.rel_err(logits.cpu().numpy(), want) < 3e-5
    other = ref.make_config(layers, width=40, vocab=33, embed_scale=2.5, softcap=2.0)   # both constants do something
    assert ref.rel_err(ref.forward(other, W, toks).numpy(), want) > 1e-2
    sess2 = session(other, packed)
    assert ref.rel_err(sess2.feed([(sess2.open(), toks, list(range(130)))]).cpu().numpy(), ref.forward(other, W, toks).numpy()) < 3e-5


def test_whole_model_every_layer_fp32_and_bf16():
    # every router output is chosen in this configuration, so that 16-bit rounding cannot flip a close expert choice
    layers = [ref.latent_layer(mlp=ref.dense()), ref.latent_layer(heads=2, dim=24, vdim=16, window=70, kv_from=0, mlp=ref.moe(experts=2, identity=1, top=3)),
              ref.latent_layer(heads=2, dim=16, rot_dim=16, rot_dims=8, vdim=24, kv_rank=40, window=9, scale=0.4),
              ref.latent_layer(heads=5, dim=8, rot_dim=16, rot_dims=8, vdim=8, kv_rank=40, window=100, kv_from=2, mlp=ref.moe(experts=3, identity=0, top=3, ff=16, shared_ff=0))]
    config = ref.make_config(layers)
    W, packed = ref.make_weights(config, seed=5)
    toks = tokens_of(config, 200, 2)
    res = []
    want = ref.forward(config, W, toks, res).numpy()
    for dtype, tol in (("float32", 5e-5), ("bfloat16", 3e-2), ("float16", 1e-2)):
        sess = session(config, packed, dtype=dtype)
        r = sess.open()
        logits, trace = sess.feed([(r, toks, list(range(200)))], trace=True)
        for i, got in enumerate(list(trace.cpu().numpy()) + [logits.cpu().numpy()]):
            want_i = res[i].numpy() if i < len(layers) else want
            per_token = np.linalg.norm(got - want_i, axis=-1) / np.linalg.norm(want_i, axis=-1)
            assert np.median(per_token) < tol and per_token.max() < 5 * tol, (dtype, i, float(np.median(per_token)), float(per_token.max()))


# ------------------------------------------------------------------ schedules
def test_prefill_equals_token_by_token_decoding_and_first_tokens():
    config = ref.make_config(MIXED)
    W, packed = ref.make_weights(config, seed=7)
    req = {"a": tokens_of(config, 90, 3)}
    whole = replay(session(config, packed), req, [[("a", 90)]])
    single = replay(session(config, packed), req, [[("a", 1)] for _ in range(90)])
    check_all(whole, config, W, req, 5e-5)
    check_all(single, config, W, req, 5e-5)  # includes positions 0, 1, 2 decoded one by one
    assert ref.rel_err(single["a"], whole["a"]) < 2e-5


@pytest.mark.parametrize("cuts", [[2] * 60, [1, 2, 3, 5, 8, 13, 21, 34, 33], [63, 1, 1, 55], [64, 6, 50], [69, 2, 49], [7, 113], [23, 1, 24, 2, 70]],
                         ids=["twos", "growing", "page_edge", "page_then_window_edge", "window_edge", "long_tail", "window_sized"])
def test_portions(cuts):
    config = ref.make_config(MIXED)
    W, packed = ref.make_weights(config, seed=8)
    req = {"a": tokens_of(config, sum(cuts), 4)}
    got = replay(session(config, packed), req, [[("a", n)] for n in cuts])
    check_all(got, config, W, req, 5e-5)


def test_long_decoding_lets_windows_pass_over_decoded_tokens_and_pages():
    config = ref.make_config([ref.latent_layer(window=50, mlp=ref.moe()), ref.latent_layer(window=130, kv_from=0, mlp=ref.dense())])
    W, packed = ref.make_weights(config, seed=9)
    req = {"a": tokens_of(config, 330, 5)}
    got = replay(session(config, packed), req, [[("a", 10)]] + [[("a", 1)] for _ in range(320)])
    check_all(got, config, W, req, 1e-4)


def test_mixed_batches_equal_each_request_alone_and_reuse_pages_and_slots():
    config = ref.make_config(MIXED)
    W, packed = ref.make_weights(config, seed=10)
    req = {"a": tokens_of(config, 130, 11), "b": tokens_of(config, 3, 12), "c": tokens_of(config, 75, 13), "d": tokens_of(config, 64, 14),
           "e": tokens_of(config, 100, 15), "f": tokens_of(config, 1, 16), "g": tokens_of(config, 66, 17)}
    # at most 4 alive and 6 pages held at any time, 12 pages and 7 slots asked for over the run: pages and slots come back and go out again
    schedule = [
        [("a", 60), ("b", 1), ("c", 2)],
        [("a", 1), ("b", 2), ("c", 70), ("d", 5)],          # b ends: its slot and page return
        [("a", 4), ("c", 1), ("d", 58), ("f", 1)],          # f takes b's slot, lives for one step
        [("a", 1), ("c", 1), ("d", 1)],                     # d ends at a page's last position
        [("a", 64), ("c", 1), ("e", 30)],                   # a ends (3 pages back); e took d's page, skipped below
        [("g", 2)],                                         # e is left out of this step
        [("e", 70), ("g", 62)],
        [("g", 1)], [("g", 1)],
    ]
    sess = session(config, packed, pool_tokens=6 * 64, max_seqs=4)
    got = replay(sess, req, schedule)
    check_all(got, config, W, req, 5e-5)
    assert sess.batcher.free_pages() == 6 and sess.batcher.free_slots() == 4
    for name in req:  # and each alone, on a fresh engine: the same numbers up to summation order
        alone = replay(session(config, packed), {name: req[name]}, [[(name, len(req[name]))]])
        assert ref.rel_err(got[name], alone[name]) < 2e-5, name


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_sixteen_bit_logits_do_not_depend_on_the_schedule(dtype):
    """The same form of the computation serves every portion size: whole prompt, portions and single tokens agree to summation order."""
    layers = [ref.latent_layer(mlp=ref.dense()), ref.latent_layer(heads=2, dim=24, vdim=16, window=70, kv_from=0, mlp=ref.moe(experts=2, identity=1, top=3))]
    config = ref.make_config(layers)
    W, packed = ref.make_weights(config, seed=12)
    req = {"a": tokens_of(config, 140, 6)}
    whole = replay(session(config, packed, dtype=dtype), req, [[("a", 140)]])
    cut = replay(session(config, packed, dtype=dtype), req, [[("a", 3)], [("a", 70)], [("a", 2)]] + [[("a", 1)]] * 65)
    assert ref.rel_err(cut["a"], whole["a"]) < 2e-3


# ------------------------------------------------------------------ edges made visible: one key that takes the whole softmax
KEY_TOKEN, QUERY_TOKEN = 7, 11


def _spiked_model(window, seed, heads=2, dim=16, rot_dim=8, kv_rank=24):
    """One layer whose query projection is bent so that QUERY_TOKEN's query points at KEY_TOKEN's key in every head: where that key is
    visible it takes (nearly) the whole softmax, whatever else the window holds; where it is not, nothing of it shows."""
    config = ref.make_config([ref.latent_layer(heads=heads, dim=dim, rot_dim=rot_dim, vdim=16, kv_rank=kv_rank, window=window, scale=0.25)], softcap=None)
    mx = config["layers"][0]["mixer"]
    if not window:
        del mx["mask"]
    W, packed = ref.make_weights(config, seed=seed)
    H, d, dr = mx["heads"], mx["dim"], mx["rot_dim"]
    h = ref.dyt(W["embed"][[KEY_TOKEN, QUERY_TOKEN]] * config["embedding"]["scale"], W, "l0.norm1")
    c, _ = ref.latent_rows(h[:1], W, "l0.mix.", mx, config["norm"]["eps"])
    key = (c @ W["l0.mix.uk"].T).view(H, d)
    wq = W["l0.mix.q"].clone().view(H, d + dr, -1)
    gain = 30.0 / mx["scale"]   # 30 on top of the score the random weights give
    wq[:, :d, :] += gain * (key / (key * key).sum(-1, keepdim=True))[:, :, None] * (h[1] / (h[1] @ h[1]))[None, None, :]
    packed["l0.mix.q"] = wq.reshape(H * (d + dr), -1).to(torch.bfloat16)
    W["l0.mix.q"] = packed["l0.mix.q"].double()
    return config, W, packed


@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
@pytest.mark.parametrize("window,query_pos,key_pos,seen", [
    (40, 100, 61, True),      # the last key the window keeps: 39 back
    (40, 100, 60, False),     # the first one it has dropped: 40 back
    (40, 39, 0, True),        # the first token of the sequence, just inside
    (40, 40, 0, False),       # ... and just outside
    (40, 41, 1, False), (40, 41, 2, True),
    (64, 127, 64, True), (64, 127, 63, False),     # a window edge that is a page edge
    (64, 128, 64, False), (64, 128, 65, True),
    (100, 150, 63, True), (100, 150, 64, True),    # a page edge inside the window
    (300, 299, 0, True),      # far: hundreds of keys and four pages back
    (300, 310, 11, True), (300, 310, 10, False),
    (1, 50, 49, False), (1, 50, 50, True),
    (0, 310, 0, True),        # no window at all
], ids=lambda v: str(v))
def test_window_edges_with_a_dominant_key(window, query_pos, key_pos, seen, decode):
    config, W, packed = _spiked_model(window, seed=window + 1)
    plain = [t for t in tokens_of(config, 3 * (query_pos + 1), query_pos * 1000 + key_pos) if t not in (KEY_TOKEN, QUERY_TOKEN)][:query_pos + 1]
    with_key, without = list(plain), list(plain)
    with_key[query_pos] = without[query_pos] = QUERY_TOKEN
    if key_pos != query_pos:
        with_key[key_pos] = KEY_TOKEN
    else:   # the query's own position: its own key is always visible; compare with another token's query
        without[query_pos] = plain[query_pos]
    want, want_without = want_logits(config, W, with_key)[query_pos], want_logits(config, W, without)[query_pos]
    changed = ref.rel_err(want_without, want)
    assert changed > 1e-2 if seen else changed == 0.0, changed
    for sequence, expect in ((with_key, want), (without, want_without)):
        sess = session(config, packed)
        r = sess.open()
        if decode and query_pos > 0:   # everything before the query is in the pool already; it arrives alone
            sess.feed([(r, sequence[:query_pos], [])])
            got = sess.feed([(r, sequence[query_pos:], [0])]).cpu().numpy()[0]
        else:
            got = sess.feed([(r, sequence, [query_pos])]).cpu().numpy()[0]
        assert ref.rel_err(got, expect) < 3e-5


# ------------------------------------------------------------------ the tensor-core kernels of 16-bit engines
EDGES = [(40, 100, 61, True), (40, 100, 60, False), (40, 39, 0, True), (40, 40, 0, False), (64, 127, 64, True), (64, 127, 63, False),
         (64, 128, 64, False), (64, 128, 65, True), (100, 150, 63, True), (100, 150, 64, True), (300, 299, 0, True), (300, 310, 11, True),
         (300, 310, 10, False), (1, 50, 49, False), (1, 50, 50, True), (0, 310, 0, True), (70, 200, 131, True), (70, 200, 130, False)]


@pytest.mark.parametrize("shape", [dict(heads=2, dim=16, rot_dim=16, kv_rank=32), dict(heads=20, dim=16, rot_dim=16, kv_rank=48),
                                   dict(heads=3, dim=8, rot_dim=0, kv_rank=256)], ids=["few_heads", "many_heads", "rank_256_no_rotation"])
@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
@pytest.mark.parametrize("window,query_pos,key_pos,seen", EDGES, ids=lambda v: str(v))
def test_tensor_core_attention_edges_with_a_dominant_key(window, query_pos, key_pos, seen, decode, shape):
    """bfloat16 engines: prompt portions run as tiles of 64 tokens x one head, decoded tokens of many-headed layers as one token x 64 heads
    (fewer heads: the per-token kernel); a latent rank above 128 is accumulated in blocks of 128 value columns."""
    config, W, packed = _spiked_model(window, seed=window + 1, **shape)
    plain = [t for t in tokens_of(config, 3 * (query_pos + 1), query_pos * 1000 + key_pos) if t not in (KEY_TOKEN, QUERY_TOKEN)][:query_pos + 1]
    with_key, without = list(plain), list(plain)
    with_key[query_pos] = without[query_pos] = QUERY_TOKEN
    if key_pos != query_pos:
        with_key[key_pos] = KEY_TOKEN
    else:
        without[query_pos] = plain[query_pos]
    want, want_without = want_logits(config, W, with_key)[query_pos], want_logits(config, W, without)[query_pos]
    changed = ref.rel_err(want_without, want)
    assert changed > 2.5e-2 if seen else changed == 0.0, changed
    for sequence, expect in ((with_key, want), (without, want_without)):
        sess = session(config, packed, dtype="bfloat16")
        r = sess.open()
        if decode and query_pos > 0:
            sess.feed([(r, sequence[:query_pos], [])])
            got = sess.feed([(r, sequence[query_pos:], [0])]).cpu().numpy()[0]
        else:
            got = sess.feed([(r, sequence, [query_pos])]).cpu().numpy()[0]
        assert ref.rel_err(got, expect) < 2e-2, ref.rel_err(got, expect)


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_tensor_core_paths_against_the_oracle_and_against_single_tokens(dtype):
    """Sizes every tensor-core path takes: tiles of prompt tokens, one-token tiles over 20 heads, a rank of 256 in two value blocks, and --
    with a prompt of 300 tokens -- the head products on 128-row tiles.  Portions that start in the middle of a page and of a window."""
    layers = [ref.latent_layer(heads=6, dim=64, rot_dim=16, vdim=48, kv_rank=80, window=36, mlp=ref.dense()),
              ref.latent_layer(heads=20, dim=64, rot_dim=16, vdim=64, kv_rank=80, window=150, kv_from=0, mlp=ref.moe(experts=2, identity=1, top=3)),
              ref.latent_layer(heads=2, dim=64, rot_dim=16, vdim=24, kv_rank=256, window=70, scale=0.1)]
    config = ref.make_config(layers, width=64)
    W, packed = ref.make_weights(config, seed=41)
    req = {"a": tokens_of(config, 420, 9)}
    want = want_logits(config, W, req["a"])
    tol = 3e-2 if dtype == "bfloat16" else 1e-2
    runs = {}
    for name, schedule in (("whole", [[("a", 420)]]), ("cut", [[("a", 300)], [("a", 37)], [("a", 70)], [("a", 3)]] + [[("a", 1)]] * 10)):
        runs[name] = replay(session(config, packed, dtype=dtype, pool_tokens=448, max_batch_tokens=448), req, schedule)["a"]
        per_pos = np.linalg.norm(runs[name] - want, axis=-1) / np.linalg.norm(want, axis=-1)
        assert np.median(per_pos) < tol and per_pos.max() < 5 * tol, (name, float(np.median(per_pos)), float(per_pos.max()))
    assert ref.rel_err(runs["cut"], runs["whole"]) < tol / 3


def test_sink_takes_its_share():
    """A large sink logit must shrink the head's output: with it the head's weights sum to much less than one."""
    config = ref.make_config([ref.latent_layer(heads=2, window=32)])
    W, packed = ref.make_weights(config, seed=21)
    packed["l0.mix.sink"] = torch.tensor([6.0, -6.0]).to(torch.bfloat16)
    W["l0.mix.sink"] = packed["l0.mix.sink"].double()
    toks = tokens_of(config, 40, 6)
    sess = session(config, packed)
    _, trace = sess.feed([(sess.open(), toks, [])], trace=True)
    res = []
    ref.forward(config, W, toks, res)
    assert ref.rel_err(trace[0].cpu().numpy(), res[0].numpy()) < 2e-5
    packed2 = dict(packed)
    packed2["l0.mix.sink"] = torch.tensor([-30.0, -30.0]).to(torch.bfloat16)
    sess2 = session(config, packed2)
    _, trace2 = sess2.feed([(sess2.open(), toks, [])], trace=True)
    assert ref.rel_err(trace2[0].cpu().numpy(), res[0].numpy()) > 1e-3  # the sink is not a no-op


def test_correction_changes_the_choice_but_not_the_weights():
    """A large correction on one expert makes every token choose it; its weight is still its (small) softmax score's share."""
    config = ref.make_config([ref.latent_layer(mlp=ref.moe(experts=6, identity=2, top=2, shared_ff=0))])
    W, packed = ref.make_weights(config, seed=23)
    corr = torch.zeros(8)
    corr[4] = 5.0
    packed["l0.mlp.correction"] = corr.to(torch.bfloat16)
    W["l0.mlp.correction"] = corr.double()
    toks = tokens_of(config, 60, 8)
    x = torch.randn(60, config["width"], dtype=torch.float64)
    chosen, weight = ref.route(x, W, "l0.mlp.", config["layers"][0]["mlp"])
    assert (chosen == 4).any(-1).all() and float(weight[chosen == 4].mean()) < 0.5
    res = []
    ref.forward(config, W, toks, res)
    sess = session(config, packed)
    _, trace = sess.feed([(sess.open(), toks, [])], trace=True)
    assert ref.rel_err(trace[0].cpu().numpy(), res[0].numpy()) < 2e-5


def test_pool_exhaustion_is_refused_not_overwritten():
    config = ref.make_config([ref.latent_layer()])
    W, packed = ref.make_weights(config, seed=1)
    sess = session(config, packed, pool_tokens=128, max_seqs=2)
    a, b = sess.open(), sess.open()
    sess.feed([(a, tokens_of(config, 100, 1), [])])
    with pytest.raises(b200().B200Error):
        sess.feed([(b, tokens_of(config, 10, 2), [])])   # both pages are a's
    sess.close(a)
    got = sess.feed([(b, tokens_of(config, 10, 2), [9])]).cpu().numpy()
    assert ref.rel_err(got, want_logits(config, W, tokens_of(config, 10, 2))[[9]]) < 5e-5


# ------------------------------------------------------------------ the mechanisms' own launchers
def test_softmax_router_picks_and_weights():
    m = b200()
    g = torch.Generator().manual_seed(0)
    z = (2.0 * torch.randn(37, 11, generator=g)).to(DEV)
    bias = (0.1 * torch.randn(11, generator=g)).to(DEV)
    for b in (bias, None):
        sel, w = m.moe_route_softmax(z, b, 3)
        s = torch.softmax(z.double(), -1)
        _, ti = torch.topk(s + (b.double() if b is not None else 0.0), 3, dim=-1)
        tv = torch.gather(s, 1, ti)
        assert torch.equal(sel.long().cpu(), ti.cpu())
        assert torch.allclose(w.double().cpu(), (tv / tv.sum(-1, keepdim=True)).cpu(), rtol=1e-5)


def test_latent_prep_against_the_plain_computation():
    m = b200()
    H, d, dr, dims, r, base, eps = 3, 12, 10, 6, 20, 300.0, 1e-5
    g = torch.Generator().manual_seed(2)
    T = 70
    proj = torch.randn(T, H * (d + dr) + r + dr, generator=g).to(DEV)
    w = (1.0 + 0.3 * torch.randn(r, generator=g)).to(DEV)
    pool = torch.full((4, 64, r + dr), float("nan"), device=DEV)
    bt = torch.tensor([[2, 0, -1], [3, -1, -1]], dtype=torch.int32, device=DEV)
    seq = torch.tensor([0] * 60 + [1] * 10, dtype=torch.int32, device=DEV)
    pos = torch.tensor(list(range(30, 90)) + list(range(10)), dtype=torch.int32, device=DEV)   # sequence 0 crosses from page 2 to page 0
    qn, qr = m.latent_prep_paged(proj, H, d, dr, r, dims, base, w, eps, seq, pos, bt, pool, 128)
    torch.cuda.synchronize()
    p64, q = proj.cpu().double(), proj.cpu().double()[:, :H * (d + dr)].view(T, H, d + dr)
    assert torch.equal(qn[:, :T].cpu().double(), q[..., :d].transpose(0, 1))
    assert torch.allclose(qr.cpu().double(), ref.rotate(q[..., d:], pos.cpu(), base, dims), rtol=1e-5, atol=1e-6)
    down = p64[:, H * (d + dr):]
    rows = torch.cat([ref.rms_unit(down[:, :r], eps) * w.cpu().double(), ref.rotate(down[:, r:], pos.cpu(), base, dims)], -1)
    for t in range(T):
        page = int(bt[int(seq[t]), int(pos[t]) // 64])
        assert torch.allclose(pool[page, int(pos[t]) % 64].cpu().double(), rows[t], rtol=1e-5, atol=1e-6), t
    assert torch.isnan(pool[1]).all() and torch.isnan(pool[3, 10:]).all()   # nothing else was written


def _latent_tiles(portions):
    out = []
    for s, row0, n, pos0 in portions:
        for a in range(0, n, 64):
            out.append([s, row0 + a, min(64, n - a), pos0 + a])
    return torch.tensor(out, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("heads,rank,rot,window", [(4, 32, 16, 48), (3, 96, 32, 100), (20, 48, 16, 1000), (2, 256, 0, 70), (70, 16, 16, 130),
                                                   (2, 384, 64, 0), (5, 192, 64, 64)])
def test_latent_tensor_core_kernels_match_the_per_token_kernel(heads, rank, rot, window, dtype):
    m = b200()
    pages, t_pad = 12, 448
    g = torch.Generator().manual_seed(heads + rank + window)
    # sequence 0: 37 cached positions, then a portion of 203; sequence 1: a portion of 130 from position 0; then one more token of each
    bt = torch.tensor([[7, 1, 10, 4, -1, -1], [3, 9, 0, -1, -1, -1]], dtype=torch.int32, device=DEV)
    pool = torch.full((pages, 64, rank + rot), float("nan"), dtype=dtype, device=DEV)
    rows = {0: torch.randn(241, rank + rot, generator=g).to(dtype).to(DEV), 1: torch.randn(131, rank + rot, generator=g).to(dtype).to(DEV)}
    for s_, n in ((0, 240), (1, 130)):
        for p_ in range(n):
            pool[int(bt[s_, p_ // 64]), p_ % 64] = rows[s_][p_]
    seq = torch.tensor([0] * 203 + [1] * 130, dtype=torch.int32, device=DEV)
    pos = torch.tensor(list(range(37, 240)) + list(range(130)), dtype=torch.int32, device=DEV)
    T = 333
    ql = (0.3 * torch.randn(heads, t_pad, rank, generator=g)).to(dtype).to(DEV)
    qr = (0.3 * torch.randn(T, heads, max(rot, 1), generator=g)).to(dtype).to(DEV)
    sink = torch.linspace(-2.0, 3.0, heads).to(DEV)
    want = m.latent_attention_paged(ql, qr, pool, sink, seq, pos, bt, rot, 0.2, window)
    got = m.latent_attention_tiles_paged(ql, qr, pool, sink, _latent_tiles([(0, 0, 203, 37), (1, 203, 130, 0)]), bt, rot, 0.2, window)
    torch.cuda.synchronize()
    assert not torch.isnan(got[:, :T]).any() and not torch.isnan(want[:, :T]).any()
    scale_ = want[:, :T].float().abs().max().item()
    assert (got[:, :T].float() - want[:, :T].float()).abs().max().item() < 1.5e-2 * scale_
    # decoded tokens: the next position of each sequence, as one-token tiles over the heads, alone and with their keys shared out
    pool[int(bt[0, 240 // 64]), 240 % 64] = rows[0][240]
    pool[int(bt[1, 130 // 64]), 130 % 64] = rows[1][130]
    seq2 = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    pos2 = torch.tensor([240, 130], dtype=torch.int32, device=DEV)
    want2 = m.latent_attention_paged(ql, qr, pool, sink, seq2, pos2, bt, rot, 0.2, window)
    tiles2 = torch.tensor([[0, 0, 1, 240], [1, 1, 1, 130]], dtype=torch.int32, device=DEV)
    for part_tiles in (0, 2, 16):   # no shares; scratch for one share each; eight shares each
        got2 = m.latent_attention_tiles_paged(ql, qr, pool, sink, tiles2, bt, rot, 0.2, window, by_head=True, part_tiles=part_tiles)
        torch.cuda.synchronize()
        assert not torch.isnan(got2[:, :2]).any()
        assert (got2[:, :2].float() - want2[:, :2].float()).abs().max().item() < 1.5e-2 * want2[:, :2].float().abs().max().item(), part_tiles


# ------------------------------------------------------------------ the scheduler's own entry point, the registry, the command line
@pytest.mark.parametrize("chunk", [0, 5])
def test_greedy_generation_through_the_scheduler(chunk):
    config = ref.make_config(MIXED)
    W, packed = ref.make_weights(config, seed=30)
    prompts = [tokens_of(config, n, 40 + n) for n in (1, 9, 70, 23, 2, 65)]   # six requests over four slots
    sess = session(config, packed, pool_tokens=6 * 64, max_seqs=4, max_batch_tokens=128)
    out = sess.generate(prompts, 12, chunk=chunk)
    for p, ids in zip(prompts, out):
        assert ids == ref.greedy(config, W, p, 12)
    assert sess.batcher.free_pages() == 6 and sess.batcher.free_slots() == 4


def _write_checkpoint(folder, config, packed):
    header, blob = {}, b""
    for k, v in packed.items():
        raw = v.contiguous().view(torch.int16).numpy().tobytes()
        header[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    hj = json.dumps(header).encode()
    (folder / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + blob)
    (folder / "config.json").write_text(json.dumps(config))


def test_registry_loads_a_checkpoint_folder(tmp_path):
    config = ref.make_config(MIXED[:2])
    W, packed = ref.make_weights(config, seed=33)
    _write_checkpoint(tmp_path, config, packed)
    model = importlib.import_module("llm-inference-engine_b200.models").load_model(str(tmp_path), dtype="float32", device=DEV, max_tokens=128, max_seqs=2)
    sess = _serving().Session(model, 128, max_seqs=2)
    toks = tokens_of(config, 20, 1)
    got = sess.feed([(sess.open(), toks, [19])]).cpu().numpy()
    assert ref.rel_err(got, want_logits(config, W, toks)[[19]]) < 5e-5


def test_trace_command_line_replays_a_schedule(tmp_path):
    config = ref.make_config(MIXED)
    W, packed = ref.make_weights(config, seed=34)
    _write_checkpoint(tmp_path, config, packed)
    a, b = tokens_of(config, 80, 1), tokens_of(config, 5, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[70:72], "want": []}, {"id": "b", "tokens": b[:4], "want": [3]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[4:], "want": [0]}, {"id": "a", "tokens": a[72:], "want": [7]}], "end": ["a", "b"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "192"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb = want_logits(config, W, a), want_logits(config, W, b)
    got0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    got1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)
    got2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(2, -1)
    assert ref.rel_err(got0, wa[[0, 69]]) < 5e-5 and ref.rel_err(got1, wb[[3]]) < 5e-5 and ref.rel_err(got2, np.stack([wb[4], wa[79]])) < 5e-5
