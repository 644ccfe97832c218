"""Vasolix on the layer-list decoder against the float64 restatement (tests/vasolix_oracle.py): every mechanism alone, prefill against
token-by-token decoding, portions, mixed batches, pages and slots used again, chunk and page edges, other sizes, greedy generation through
the scheduler.  All configurations are made here, small, with random weights whose values are exact in bfloat16."""
import importlib
import math

import numpy as np
import pytest
import torch

import vasolix_oracle as ref
from util import b200

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _models():
    return importlib.import_module("llm-inference-engine_b200.models.vasolix")


def _serving():
    return importlib.import_module("llm-inference-engine_b200.serving")


def session(config, packed, dtype="float32", pool_tokens=512, max_seqs=4, max_batch_tokens=512):
    model = _models().VasolixModel(config, packed, dtype=dtype, device=DEV, max_tokens=max_batch_tokens, max_seqs=max_seqs,
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


MIXED = [ref.gla_layer(mlp=ref.moe()), ref.attention_layer(mlp=ref.moe(experts=4, top=1, ff=16, shared_ff=24)),
         ref.attention_layer(heads=3, kv_heads=3, dim=12, size=70, scale=0.2), ref.gla_layer(heads=3, dim=8, vdim=20, tau=2.5, mlp=ref.moe(experts=3, top=3))]


# ------------------------------------------------------------------ each mechanism alone (one-layer models, residual stream compared)
@pytest.mark.parametrize("layer", [
    ref.attention_layer(),                                   # grouped kv heads, chunk smaller than a page
    ref.attention_layer(heads=2, kv_heads=2, dim=20, size=100, scale=0.11),  # kv_heads == heads, dim not a multiple of 8, chunk across pages
    ref.attention_layer(heads=6, kv_heads=2, dim=8, size=64),  # three query heads per kv head, chunk == page
    ref.gla_layer(),
    ref.gla_layer(heads=1, dim=40, vdim=33, tau=1.0),        # one head, vdim that is not a multiple of the column tile
    ref.gla_layer(heads=3, dim=8, vdim=72, tau=30.0),
    ref.gla_layer(mlp=ref.moe(experts=5, top=2)),
    ref.gla_layer(mlp=ref.moe(experts=2, top=2, ff=8, shared_ff=8)),  # every expert chosen
    ref.gla_layer(mlp=ref.moe(experts=70, top=4, ff=8, shared_ff=16)),  # more experts than a warp, most of them unused
], ids=["attn", "attn_mha_d20", "attn_gqa3", "gla", "gla_1head", "gla_wide_v", "moe_top2", "moe_all", "moe_many"])
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


def test_whole_model_every_layer_fp32_and_bf16():
    # every expert is chosen in this configuration, so that 16-bit rounding cannot flip a close expert choice (a flip is a legitimate,
    # but large and lasting, difference: the recurrent state carries it on)
    layers = [ref.gla_layer(mlp=ref.moe(experts=3, top=3)), ref.attention_layer(mlp=ref.moe(experts=2, top=2, ff=16, shared_ff=24)),
              ref.attention_layer(heads=3, kv_heads=3, dim=12, size=70, scale=0.2), ref.gla_layer(heads=3, dim=8, vdim=20, tau=2.5, mlp=ref.moe(experts=3, top=3))]
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


@pytest.mark.parametrize("cuts", [[2] * 60, [1, 2, 3, 5, 8, 13, 21, 34, 33], [63, 1, 1, 55], [64, 6, 50], [69, 2, 49], [7, 113]],
                         ids=["twos", "growing", "page_edge", "page_then_chunk_edge", "chunk_edge", "long_tail"])
def test_portions(cuts):
    config = ref.make_config(MIXED)   # chunks of 24 and 70 positions, pages of 64
    W, packed = ref.make_weights(config, seed=8)
    req = {"a": tokens_of(config, sum(cuts), 4)}
    got = replay(session(config, packed), req, [[("a", n)] for n in cuts])
    check_all(got, config, W, req, 5e-5)


def test_long_decoding_through_chunks_and_pages():
    config = ref.make_config([ref.gla_layer(mlp=ref.moe()), ref.attention_layer(size=50, mlp=ref.moe(top=1))])
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


def test_pool_exhaustion_is_refused_not_overwritten():
    config = ref.make_config([ref.attention_layer()])
    W, packed = ref.make_weights(config, seed=1)
    sess = session(config, packed, pool_tokens=128, max_seqs=2)
    a, b = sess.open(), sess.open()
    sess.feed([(a, tokens_of(config, 100, 1), [])])
    with pytest.raises(b200().B200Error):
        sess.feed([(b, tokens_of(config, 10, 2), [])])   # both pages are a's
    with pytest.raises(b200().B200Error):
        sess.open()                                      # both slots are taken
    sess.close(a)
    got = sess.feed([(b, tokens_of(config, 10, 2), [9])]).cpu().numpy()
    assert ref.rel_err(got, want_logits(config, W, tokens_of(config, 10, 2))[[9]]) < 5e-5


# ------------------------------------------------------------------ edges made visible: one key that takes the whole softmax
def _spike_case(chunk, T, query_pos, key_pos, decode):
    """One sequence, 2 heads over 1 kv head, scattered pages in a NaN pool.  Key `key_pos` is large and the query at `query_pos` points at
    it: if that key is visible the output is (nearly) that key, else nothing of it shows."""
    m = b200()
    H, G, d, pages = 2, 1, 16, 8
    g = torch.Generator().manual_seed(query_pos * 1000 + key_pos)
    k = 0.1 * torch.randn(T, G * d, generator=g)
    q = 0.1 * torch.randn(T, H * d, generator=g)
    k[key_pos] = 3.0 * torch.sign(torch.randn(G * d, generator=g))
    q[query_pos] = torch.cat([k[key_pos], k[key_pos]]) * 4.0
    proj = torch.cat([q, k], 1).to(DEV)
    k_pool = torch.full((pages, G, 64, d), float("nan"), device=DEV)
    v_pool = torch.full((pages, G, 64, d), float("nan"), device=DEV)
    bt = torch.tensor([[5, 2, 7, 0, 3, -1, -1, -1]], dtype=torch.int32, device=DEV)
    seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    sink = torch.tensor([0.3, -1.0], device=DEV)
    if decode:  # everything before the query is already in the pool; the query arrives alone
        n0 = query_pos
        m.attn_qk_norm_cache_paged(proj[:n0].contiguous(), H, G, d, None, None, 1e-6, seq[:n0].contiguous(), pos[:n0].contiguous(), bt, k_pool, v_pool)
        rows = slice(query_pos, query_pos + 1)
    else:
        rows = slice(0, T)
    pr, sq, ps = proj[rows].contiguous(), seq[rows].contiguous(), pos[rows].contiguous()
    qn = m.attn_qk_norm_cache_paged(pr, H, G, d, None, None, 1e-6, sq, ps, bt, k_pool, v_pool)
    out = m.chunked_attention_paged(qn, k_pool, v_pool, sink, None, sq, ps, bt, H, G, d, 0.25, chunk)
    torch.cuda.synchronize()
    got = out[0 if decode else query_pos].cpu().double()
    # the plain computation for this one query
    lo = (query_pos // chunk) * chunk
    kk, qq = k[lo:query_pos + 1].double(), q[query_pos].double().view(H, d)
    want = []
    for h in range(H):
        e = torch.exp(kk @ qq[h] * 0.25)
        want.append((e / (e.sum() + math.exp(float(sink[h])))) @ kk)
    return got.view(H, d), torch.stack(want), k[key_pos].double()


@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
@pytest.mark.parametrize("chunk,query_pos,key_pos,visible", [
    (100, 150, 100, True),    # the first key of the query's chunk
    (100, 150, 99, False),    # the last key of the chunk before
    (100, 199, 100, True),    # the chunk's last query still sees its first key, 99 back
    (100, 200, 199, False),   # the next chunk's first query sees only itself
    (100, 100, 100, True),
    (300, 290, 3, True),      # far: hundreds of keys and four pages back
    (300, 299, 0, True),      # the first token of the sequence
    (128, 130, 127, False),   # a chunk edge that is a page edge
    (128, 190, 128, True),
    (48, 70, 63, True),       # a page edge inside a chunk
    (48, 70, 64, True),
    (48, 70, 47, False),
], ids=lambda v: str(v))
def test_attention_edges_with_a_dominant_key(chunk, query_pos, key_pos, visible, decode):
    got, want, key = _spike_case(chunk, 300, query_pos, key_pos, decode)
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-5)
    shows = bool(((got - key).norm(dim=-1) < 0.1 * key.norm()).all())
    assert shows == visible


def test_sink_takes_its_share():
    """A large sink logit must shrink the output: with it the head's weights sum to much less than one."""
    config = ref.make_config([ref.attention_layer(heads=2, kv_heads=1, dim=16, size=32)])
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


def test_gla_state_is_carried_far():
    """Decay close to one: what the first token wrote into the state still decides the output 250 tokens later, across portions."""
    config = ref.make_config([ref.gla_layer(heads=2, dim=8, vdim=16, tau=64.0)])
    W, packed = ref.make_weights(config, seed=22)
    packed["l0.mix.a2.b"] = torch.full_like(packed["l0.mix.a2.b"], 9.0)   # sigmoid(9)^(1/64): decay 0.999998 per step
    W["l0.mix.a2.b"] = packed["l0.mix.a2.b"].double()
    toks = tokens_of(config, 260, 7)
    other = list(toks)
    other[0] = (toks[0] + 1) % config["vocab"]
    want, want_other = want_logits(config, W, toks), want_logits(config, W, other)
    assert ref.rel_err(want[255:], want_other[255:]) > 1e-2   # the first token matters at the end
    got = replay(session(config, packed), {"a": toks}, [[("a", 3)], [("a", 100)], [("a", 150)]] + [[("a", 1)]] * 7)
    assert ref.rel_err(got["a"], want) < 5e-5


def test_router_picks_and_weights():
    m = b200()
    g = torch.Generator().manual_seed(0)
    z = torch.randn(37, 9 + 1, generator=g).to(DEV)
    sel, w, gate = m.moe_route_sigmoid(z, 9, 3)
    tv, ti = torch.topk(torch.sigmoid(z[:, :9]), 3, dim=-1)
    assert torch.equal(sel.long().cpu(), ti.cpu())
    assert torch.allclose(w.cpu(), tv.cpu(), rtol=1e-6) and torch.allclose(gate.cpu(), torch.sigmoid(z[:, 9]).cpu(), rtol=1e-6)


def test_gla_recurrence_op_against_the_loop():
    m = b200()
    H, d, dv = 2, 12, 40
    g = torch.Generator().manual_seed(1)
    T = 50
    proj = torch.randn(T, 2 * H * d + H * dv, generator=g).to(DEV)
    decay = torch.rand(T, H * d, generator=g).to(DEV)
    state = torch.full((3, H, d, dv), float("nan"), device=DEV)
    # two sequences (30 and 20 tokens) in slots 2 and 0, each in two calls
    cuts = [((0, 17), (30, 39)), ((17, 30), (39, 50))]
    outs = torch.zeros(T, H * dv)
    for call, ((a0, a1), (b0, b1)) in enumerate(cuts):
        rows = list(range(a0, a1)) + list(range(b0, b1))
        o = m.gla_recurrent(proj[rows].contiguous(), decay[rows].contiguous(), state,
                            torch.tensor([0, a1 - a0, a1 - a0 + b1 - b0], dtype=torch.int32, device=DEV),
                            torch.tensor([a0, b0 - 30], dtype=torch.int32, device=DEV), torch.tensor([2, 0], dtype=torch.int32, device=DEV), H, d, dv)
        outs[rows] = o.cpu()
    for lo, hi in ((0, 30), (30, 50)):
        S = torch.zeros(H, d, dv, dtype=torch.float64)
        for t in range(lo, hi):
            r = proj[t].cpu().double()
            q, k, v = r[:H * d].view(H, d) / math.sqrt(d), r[H * d:2 * H * d].view(H, d), r[2 * H * d:].view(H, dv)
            S = decay[t].cpu().double().view(H, d, 1) * S + k.unsqueeze(-1) * v.unsqueeze(1)
            assert torch.allclose(outs[t].double().view(H, dv), (S * q.unsqueeze(-1)).sum(1), rtol=1e-4, atol=1e-5), t


# ------------------------------------------------------------------ the scheduler's own entry point
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


def test_generation_survives_preemption():
    config = ref.make_config([ref.gla_layer(mlp=ref.moe()), ref.attention_layer(size=40)])
    W, packed = ref.make_weights(config, seed=31)
    prompts = [tokens_of(config, 60, 50), tokens_of(config, 62, 51), tokens_of(config, 50, 52)]
    sess = session(config, packed, pool_tokens=4 * 64, max_seqs=3, max_batch_tokens=192)   # three sequences that each grow into a second page
    out = sess.generate(prompts, 10)
    assert sum(sess.batcher.preemptions(r) for r in range(3)) >= 1
    for p, ids in zip(prompts, out):
        assert ids == ref.greedy(config, W, p, 10)


def test_registry_loads_a_checkpoint_folder(tmp_path):
    import json
    import struct

    config = ref.make_config([ref.gla_layer(mlp=ref.moe(top=1)), ref.attention_layer()])
    W, packed = ref.make_weights(config, seed=33)
    header, blob = {}, b""
    for k, v in packed.items():
        raw = v.contiguous().view(torch.int16).numpy().tobytes()
        header[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    hj = json.dumps(header).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + blob)
    (tmp_path / "config.json").write_text(json.dumps(config))
    model = importlib.import_module("llm-inference-engine_b200.models").load_model(str(tmp_path), dtype="float32", device=DEV, max_tokens=128, max_seqs=2)
    sess = _serving().Session(model, 128, max_seqs=2)
    toks = tokens_of(config, 20, 1)
    got = sess.feed([(sess.open(), toks, [19])]).cpu().numpy()
    assert ref.rel_err(got, want_logits(config, W, toks)[[19]]) < 5e-5


# ------------------------------------------------------------------ the tensor-core kernel for prompt portions (16-bit, dim 64 / 128)
def _tiles(portions):
    """portions: [(sequence, first packed row, rows, first position)] -> int32 [n, 4] device tensor of tiles of <= 64 rows."""
    out = []
    for s, row0, n, pos0 in portions:
        for a in range(0, n, 64):
            out.append([s, row0 + a, min(64, n - a), pos0 + a])
    return torch.tensor(out, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("dim,chunk", [(64, 48), (64, 100), (128, 128), (64, 1000), (128, 70)])
def test_tensor_core_attention_matches_the_per_token_kernel(dim, chunk, dtype):
    m = b200()
    H, G, pages = 4, 2, 12
    g = torch.Generator().manual_seed(dim + chunk)
    # sequence 0: 37 cached positions, then a portion of 203; sequence 1: a portion of 130 from position 0
    lens = [(0, 37), (0, 203), (1, 130)]
    T = sum(n for _, n in lens)
    proj = torch.randn(T, (H + G + H) * dim, generator=g).to(dtype).to(DEV)   # q | k | gate
    qn_w = (1.0 + 0.3 * torch.randn(H * dim, generator=g)).to(DEV)
    kn_w = (1.0 + 0.3 * torch.randn(G * dim, generator=g)).to(DEV)
    sink = torch.tensor([0.5, -2.0, 3.0, 0.0], device=DEV)
    bt = torch.tensor([[7, 1, 10, 4, -1, -1], [3, 9, 0, -1, -1, -1]], dtype=torch.int32, device=DEV)
    k_pool = torch.full((pages, G, 64, dim), float("nan"), dtype=dtype, device=DEV)
    v_pool = torch.full((pages, G, 64, dim), float("nan"), dtype=dtype, device=DEV)
    seq = torch.tensor([0] * 240 + [1] * 130, dtype=torch.int32, device=DEV)
    pos = torch.tensor(list(range(240)) + list(range(130)), dtype=torch.int32, device=DEV)
    # the cached part first, then the two portions as one batch
    m.attn_qk_norm_cache_paged(proj[:37].contiguous(), H, G, dim, qn_w, kn_w, 1e-5, seq[:37].contiguous(), pos[:37].contiguous(), bt, k_pool, v_pool)
    pr, sq, ps = proj[37:].contiguous(), seq[37:].contiguous(), pos[37:].contiguous()
    qn = m.attn_qk_norm_cache_paged(pr, H, G, dim, qn_w, kn_w, 1e-5, sq, ps, bt, k_pool, v_pool)
    gate = pr[:, (H + G) * dim:]
    # gate is a strided view of the projection: the launchers take a row stride, so hand over the projection's pointer arithmetic
    gate_c = gate.contiguous()
    want = m.chunked_attention_paged(qn, k_pool, v_pool, sink, gate_c, sq, ps, bt, H, G, dim, 0.11, chunk)
    got = m.chunked_attention_prefill_paged(qn, k_pool, v_pool, sink, gate_c, _tiles([(0, 0, 203, 37), (1, 203, 130, 0)]), bt, H, G, dim, 0.11, chunk)
    torch.cuda.synchronize()
    assert not torch.isnan(got).any() and not torch.isnan(want).any()
    err = (got.float() - want.float()).abs().max().item()
    assert err < 1.5e-2 * want.float().abs().max().item(), err


@pytest.mark.parametrize("chunk,query_pos,key_pos,visible", [
    (100, 150, 100, True), (100, 150, 99, False), (100, 199, 100, True), (100, 200, 199, False), (300, 290, 3, True), (300, 299, 0, True),
    (128, 130, 127, False), (128, 190, 128, True), (48, 70, 63, True), (48, 70, 64, True), (48, 70, 47, False),
], ids=lambda v: str(v))
def test_tensor_core_attention_edges_with_a_dominant_key(chunk, query_pos, key_pos, visible):
    m = b200()
    H, G, d, T = 2, 1, 64, 300
    g = torch.Generator().manual_seed(query_pos * 1000 + key_pos)
    k = 0.1 * torch.randn(T, G * d, generator=g)
    q = 0.1 * torch.randn(T, H * d, generator=g)
    k[key_pos] = 2.0 * torch.sign(torch.randn(G * d, generator=g))
    q[query_pos] = torch.cat([k[key_pos], k[key_pos]])
    proj = torch.cat([q, k], 1).to(torch.bfloat16).to(DEV)
    k_pool = torch.full((8, G, 64, d), float("nan"), dtype=torch.bfloat16, device=DEV)
    v_pool = torch.full_like(k_pool, float("nan"))
    bt = torch.tensor([[5, 2, 7, 0, 3, -1]], dtype=torch.int32, device=DEV)
    seq = torch.zeros(T, dtype=torch.int32, device=DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    qn = m.attn_qk_norm_cache_paged(proj, H, G, d, None, None, 1e-6, seq, pos, bt, k_pool, v_pool)
    out = m.chunked_attention_prefill_paged(qn, k_pool, v_pool, torch.tensor([0.3, -1.0], device=DEV), None, _tiles([(0, 0, T, 0)]), bt, H, G, d, 0.25, chunk)
    torch.cuda.synchronize()
    got, key = out[query_pos].float().cpu().view(H, d), k[key_pos].to(torch.bfloat16).float()
    assert not torch.isnan(out).any()
    shows = bool(((got - key).norm(dim=-1) < 0.1 * key.norm()).all())
    assert shows == visible


def test_bf16_engine_with_tensor_core_attention_in_portions():
    """dim 64 attention in a bf16 engine: long portions take the tensor-core kernel, short ones and decoded tokens the per-token kernel;
    both must tell the same story as the float64 model."""
    layers = [ref.attention_layer(heads=4, kv_heads=2, dim=64, size=90, scale=0.125, mlp=ref.moe(experts=2, top=2)), ref.gla_layer(),
              ref.attention_layer(heads=2, kv_heads=1, dim=64, size=40, scale=0.1)]
    config = ref.make_config(layers, width=64)
    W, packed = ref.make_weights(config, seed=44)
    req = {"a": tokens_of(config, 260, 1), "b": tokens_of(config, 100, 2)}
    want = {k: want_logits(config, W, v) for k, v in req.items()}
    schedule = [[("a", 150), ("b", 3)], [("a", 1), ("b", 90)], [("a", 100), ("b", 1)]] + [[("a", 1), ("b", 1)]] * 6 + [[("a", 3)]]
    got = replay(session(config, packed, dtype="bfloat16"), req, schedule)
    for name in req:
        per_pos = np.linalg.norm(got[name] - want[name], axis=-1) / np.linalg.norm(want[name], axis=-1)
        assert np.median(per_pos) < 3e-2 and per_pos.max() < 0.15, (name, float(np.median(per_pos)), float(per_pos.max()))


def test_prompt_sized_expert_batches_take_the_tcgen05_grouped_gemm():
    """More than a thousand (token, expert) pairs in a 16-bit engine: the experts run as 128-row tiles on the tcgen05 grouped GEMM.  Every
    expert is chosen for every token here (no close routing calls), so the result must agree with the float64 model to 16-bit rounding and
    with the same prompt fed in portions small enough to take the 64-row mma.sync kernel."""
    layers = [ref.gla_layer(heads=2, dim=16, vdim=32, mlp=ref.moe(experts=4, top=4, ff=64, shared_ff=72)),
              ref.attention_layer(heads=2, kv_heads=1, dim=64, size=300, scale=0.125, mlp=ref.moe(experts=3, top=3, ff=136, shared_ff=64))]
    config = ref.make_config(layers, width=64)
    W, packed = ref.make_weights(config, seed=71)
    req = {"a": tokens_of(config, 700, 9)}
    want = want_logits(config, W, req["a"])
    for dtype in ("bfloat16", "float16"):
        whole = replay(session(config, packed, dtype=dtype, pool_tokens=768, max_batch_tokens=768), req, [[("a", 700)]])["a"]
        parts = replay(session(config, packed, dtype=dtype, pool_tokens=768, max_batch_tokens=768), req, [[("a", 100)]] * 7)["a"]
        per_pos = np.linalg.norm(whole - want, axis=-1) / np.linalg.norm(want, axis=-1)
        assert np.median(per_pos) < 3e-2 and per_pos.max() < 0.15, (dtype, float(np.median(per_pos)), float(per_pos.max()))
        same = np.linalg.norm(whole - parts, axis=-1) / np.linalg.norm(want, axis=-1)
        assert np.median(same) < 1.5e-2 and same.max() < 0.1, (dtype, float(np.median(same)), float(same.max()))


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 4e-2)])
def test_sizes_that_fit_no_vector_or_tile(dtype, tol):
    """Width, head sizes, expert sizes and ranks that are multiples of nothing convenient (not of 8, some not of 4, a chunk of 7, one kv
    head, one gla head, three experts): every kernel's scalar / bounds path."""
    layers = [ref.attention_layer(heads=3, kv_heads=1, dim=12, size=7, scale=0.4, mlp=ref.moe(experts=3, top=3, ff=10, shared_ff=6)),
              ref.gla_layer(heads=1, dim=20, vdim=12, tau=3.0, mlp=ref.moe(experts=2, top=2, ff=9, shared_ff=5)),
              ref.gla_layer(heads=5, dim=4, vdim=9, tau=1.5)]
    config = ref.make_config(layers, width=52, vocab=37)
    W, packed = ref.make_weights(config, seed=81, decay_rank=5)
    req = {"a": tokens_of(config, 75, 1), "b": tokens_of(config, 20, 2)}
    got = replay(session(config, packed, dtype=dtype), req, [[("a", 30), ("b", 2)], [("a", 1), ("b", 17)], [("a", 44), ("b", 1)]])
    for name in req:
        want = want_logits(config, W, req[name])
        per_pos = np.linalg.norm(got[name] - want, axis=-1) / np.linalg.norm(want, axis=-1)
        assert np.median(per_pos) < tol and per_pos.max() < 5 * tol, (name, float(np.median(per_pos)), float(per_pos.max()))


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 4e-2)])
def test_sizes_that_fit_every_vector(dtype, tol):
    """The opposite corner: every row starts on a 16-byte boundary, so the 16-byte paths of the norm, gather, activation, output and
    append kernels run; a chunk long enough for the per-token attention's widest block with decoded tokens on both sides of its edge;
    a decay rank read in whole vectors; one-token portions on the recurrence's step kernel with a partial last column tile (vdim 72),
    beside longer portions of another sequence in the same call.  Every expert is chosen (no close routing calls)."""
    layers = [ref.gla_layer(heads=2, dim=24, vdim=72, tau=5.0, mlp=ref.moe(experts=4, top=4, ff=32, shared_ff=48)),
              ref.attention_layer(heads=4, kv_heads=2, dim=32, size=520, scale=0.2, mlp=ref.moe(experts=3, top=3, ff=40, shared_ff=16)),
              ref.gla_layer(heads=3, dim=40, vdim=16, tau=12.0)]
    config = ref.make_config(layers, width=64)
    W, packed = ref.make_weights(config, seed=91, decay_rank=16)
    req = {"a": tokens_of(config, 530, 3), "b": tokens_of(config, 40, 4)}
    schedule = [[("a", 500)]] + [[("a", 1)]] * 10 + [[("a", 1), ("b", 25)]] * 1 + [[("a", 1), ("b", 1)]] * 15 + [[("a", 4)]]
    got = replay(session(config, packed, dtype=dtype, pool_tokens=704, max_batch_tokens=512), req, schedule)
    for name in req:
        want = want_logits(config, W, req[name])
        per_pos = np.linalg.norm(got[name] - want, axis=-1) / np.linalg.norm(want, axis=-1)
        assert np.median(per_pos) < tol and per_pos.max() < 5 * tol, (name, float(np.median(per_pos)), float(per_pos.max()))
