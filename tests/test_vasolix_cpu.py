"""Host-side parts of serving Vasolix, no GPU: the scheduler's state slots, portions and caller-driven sequences, the configuration
reader, the checkpoint reader, the registry -- and the oracle's own masks."""
import importlib
import json
import struct

import numpy as np
import pytest
import torch

import vasolix_oracle as ref
from util import b200


def test_registry_knows_the_architectures():
    models = importlib.import_module("llm-inference-engine_b200.models")
    assert {"vasolix", "llama"} <= set(models.architectures())
    assert models.architecture_of({"architecture": "Vasolix"}) == "Vasolix"
    with pytest.raises(ValueError):
        models.architecture_of({})


def test_layer_specs_follow_the_configuration():
    m = b200()
    v = importlib.import_module("llm-inference-engine_b200.models.vasolix")
    config = ref.make_config([ref.attention_layer(heads=6, kv_heads=3, dim=20, size=77, scale=0.07, mlp=ref.moe(experts=9, top=4, ff=30, shared_ff=50)),
                              ref.gla_layer(heads=5, dim=12, vdim=28, tau=3.5)])
    a, g = v.layer_specs(config)
    assert (a["mixer"], a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["chunk"]) == (m.MIXER_ATTN_CHUNKED, 6, 3, 20, 20, 77)
    assert a["scale"] == pytest.approx(0.07) and (a["mlp"], a["experts"], a["top"], a["expert_ff"], a["shared_ff"]) == (m.MLP_MOE, 9, 4, 30, 50)
    assert (g["mixer"], g["heads"], g["dim"], g["vdim"], g["mlp"]) == (m.MIXER_GLA, 5, 12, 28, m.MLP_NONE) and g["tau"] == pytest.approx(3.5)
    with pytest.raises(ValueError):
        v.layer_specs(ref.make_config([{"type": "conv", "mixer": {"heads": 1, "dim": 4}, "mlp": None}]))


def test_safetensors_reader(tmp_path):
    w = importlib.import_module("llm-inference-engine_b200.weights")
    a = torch.randn(3, 5).to(torch.bfloat16)
    b = torch.arange(7, dtype=torch.int32)
    c = torch.randn(4)
    header, blob = {"__metadata__": {"k": "v"}}, b""
    for name, t, dt in (("a.b", a, "BF16"), ("idx", b, "I32"), ("c", c, "F32")):
        raw = (t.view(torch.int16) if dt == "BF16" else t).numpy().tobytes()
        header[name] = {"dtype": dt, "shape": list(t.shape), "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    hj = json.dumps(header).encode()
    (tmp_path / "m.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + blob)
    got = w.read_safetensors(str(tmp_path / "m.safetensors"))
    assert set(got) == {"a.b", "idx", "c"}
    assert got["a.b"].dtype == torch.bfloat16 and torch.equal(got["a.b"], a) and torch.equal(got["idx"], b) and torch.equal(got["c"], c)


def test_caller_driven_sequences_share_pages_and_slots():
    m = b200()
    b = m.Batcher(3, 4, 3, 256)
    b.set_state_slots(2)
    r0, r1 = b.attach(), b.attach()
    with pytest.raises(m.B200Error):
        b.attach()                                   # two slots only
    assert b.extend(r0, list(range(70))) == 0        # two pages
    assert b.extend(r0, [1]) == 70
    assert b.extend(r1, list(range(64))) == 0        # exactly one page
    row0, s0 = b.seq_pages(r0)
    row1, s1 = b.seq_pages(r1)
    assert sorted(row0[:2].tolist() + row1[:1].tolist()) == [0, 1, 2] and row0[2] == -1 and {s0, s1} == {0, 1}
    assert b.extend(r1, [5]) == 64 and b.free_pages() == 0   # the 65th position takes the last page
    with pytest.raises(m.B200Error):
        b.extend(r0, list(range(60)))                # would need a third page for r0: none left -- and nothing is half-taken
    assert b.extend(r0, list(range(57))) == 71       # up to the end of its second page is fine
    with pytest.raises(m.B200Error):
        b.extend(r1, list(range(200)))               # beyond a block-table row
    b.release(r0)
    assert b.free_pages() == 2 and b.free_slots() == 1
    r2 = b.attach()
    assert b.seq_pages(r2)[1] == s0                  # the slot goes out again
    assert b.extend(r2, list(range(128))) == 0 and sorted(b.seq_pages(r2)[0][:2].tolist()) == sorted(row0[:2].tolist())
    b.release(r1), b.release(r2), b.release(r2)
    assert b.free_pages() == 4 and b.free_slots() == 2


def _drain(b, sampler, end_id=-1, check=None):
    """Runs mixed iterations with a sampler that sees the whole sequence so far (prompt + generated)."""
    seqs, it = {}, 0
    while b.pending():
        p, v = b.plan_mixed()
        n = p.n_prefill + p.n_decode
        assert n == len(v["requests"]) and v["starts"][-1] == p.prefill_tokens == len(v["ids"])
        if check:
            check(p, v)
        sampled = []
        for i in range(n):
            r = int(v["requests"][i])
            got = v["ids"][v["starts"][i]:v["starts"][i + 1]].tolist()
            if v["pos0"][i] == 0:
                seqs[r] = []                          # (re)computed from the start
            assert len(seqs[r]) == v["pos0"][i]
            seqs[r] += got
            pages = v["block_table"][i]
            assert (pages[:(len(seqs[r]) + 63) // 64] >= 0).all()
            sampled.append(sampler(seqs[r]) if v["sample_rows"][i] >= 0 else -1)
            if v["sample_rows"][i] >= 0:
                assert v["sample_rows"][i] == v["starts"][i + 1] - 1
        b.commit_mixed(sampled, end_id)
        it += 1
        assert it < 10000
    return it


def _sampler(seq):
    return (sum(seq) * 31 + len(seq)) % 97


def _alone(prompt, n):
    s, out = list(prompt), []
    for _ in range(n):
        out.append(_sampler(s))
        s.append(out[-1])
    return out


@pytest.mark.parametrize("chunk", [0, 2, 7, 64])
def test_mixed_plan_portions_slots_and_results(chunk):
    m = b200()
    b = m.Batcher(3, 6, 3, 100)
    b.set_state_slots(3)
    b.set_chunk(chunk)
    rng = np.random.default_rng(chunk)
    prompts = [rng.integers(0, 97, n).tolist() for n in (1, 70, 33, 2, 64, 65, 90)]
    rids = [b.submit(p, 9) for p in prompts]

    def check(p, v):
        assert p.prefill_tokens <= 100 and len(set(v["requests"].tolist())) == len(v["requests"]) <= 3
        assert len(set(v["slots"].tolist())) == len(v["slots"]) and all(0 <= s < 3 for s in v["slots"])
        if chunk:
            assert all(v["starts"][i + 1] - v["starts"][i] <= chunk for i in range(len(v["requests"])))
        held = [pg for row in v["block_table"] for pg in row if pg >= 0]
        assert len(held) == len(set(held))            # no page in two rows

    _drain(b, _sampler, check=check)
    for r, p in zip(rids, prompts):
        ids, state = b.result(r)
        assert state == m.REQ_FINISHED and ids.tolist() == _alone(p, 9)
    assert b.free_pages() == 6 and b.free_slots() == 3


def test_mixed_plan_preempts_and_recomputes():
    m = b200()
    b = m.Batcher(3, 3, 2, 128)
    b.set_state_slots(3)
    prompts = [list(range(60)), list(range(10, 71)), list(range(5, 50))]
    rids = [b.submit(p, 12) for p in prompts]
    _drain(b, _sampler)
    assert sum(b.preemptions(r) for r in rids) >= 1
    for r, p in zip(rids, prompts):
        assert b.result(r)[0].tolist() == _alone(p, 12)
    assert b.free_pages() == 3 and b.free_slots() == 3


def test_end_id_finishes_a_sequence_in_the_mixed_plan():
    m = b200()
    b = m.Batcher(2, 4, 2, 64)
    b.set_state_slots(2)
    r = b.submit([1, 2, 3], 50)
    _drain(b, lambda seq: 7 if len(seq) >= 6 else 11, end_id=7)
    ids, state = b.result(r)
    assert state == m.REQ_FINISHED and ids.tolist() == [11, 11, 11, 7]


def test_oracle_masks_and_sink():
    """The oracle itself: a key outside the query's block must not matter, the block's first key must, and the sink only scales."""
    config = ref.make_config([ref.attention_layer(heads=2, kv_heads=1, dim=8, size=10)])
    W, _ = ref.make_weights(config, seed=2)
    toks = np.random.default_rng(0).integers(0, 61, 25).tolist()
    base = ref.forward(config, W, toks)
    other = list(toks)
    other[9] = (toks[9] + 1) % 61            # last key of block 0
    moved = ref.forward(config, W, other)
    assert torch.equal(base[10:], moved[10:]) and not torch.equal(base[9], moved[9])
    other = list(toks)
    other[10] = (toks[10] + 1) % 61          # first key of block 1
    moved = ref.forward(config, W, other)
    assert not torch.allclose(base[19], moved[19]) and torch.equal(base[20:], moved[20:])
