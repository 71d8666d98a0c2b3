"""The package's decode loops against the token streams recorded from the reference's own
loops (tests/golden/streams.json), both driven over the CPU oracle forward.  Pins the host
logic: draft/verify input rows, width selection, KV promotion, segment migration,
acceptance accounting and the statistics dictionary."""
import json
import os

import pytest
import torch

from bitmtp_b200 import fast_generate as FG, generate, synthetic
from oracle import oracle as O
from tests.cpu_atlas import CpuAtlas, OracleModel, patched_host_ops

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "streams.json")
RECORDS = json.load(open(GOLDEN))
MODES = {"ar": FG.fast_ar_generate, "spec": FG.fast_speculative_generate,
         "hybrid": FG.fast_hybrid_generate, "conf": FG.fast_confidence_generate}


@pytest.mark.parametrize("rec", RECORDS, ids=lambda r: f"{r['geometry']}-D{r['cfg']['block_size']}-{r['mode']}-"
                                                         f"{r['accept']}" + ("-eos" if r.get("eos_ids") else "") +
                                                         ("-m1verify" if r.get("exact_m1_verify") else ""))
def test_stream_matches_reference_loops(rec):
    cfg = rec["cfg"]
    state = synthetic.make_state(cfg, seed=rec["state_seed"])
    om = O.OracleModel(cfg, state, max_positions=max(rec["ladder"]) + max(rec["m_set"]))
    args = generate.args_from_config(cfg)
    roles = ("ar",) if rec["mode"] == "ar" else ("ar", "draft", "verify")
    atlas = CpuAtlas(om, args, rec["ladder"], rec["m_set"], roles)
    prompt = synthetic.random_prompt(rec["prompt_len"], cfg["vocab_size"], seed=rec["prompt_seed"])
    policy = synthetic.AcceptancePolicy(rec["accept"], cfg["block_size"], seed=rec["accept_seed"])
    with patched_host_ops(cfg["block_size"], policy):
        extra = dict(exact_m1_verify=True) if rec.get("exact_m1_verify") else {}
        out, stats = MODES[rec["mode"]](OracleModel(om, args), atlas, prompt, max_gen_len=rec["new_tokens"],
                                        eos_ids=frozenset(rec.get("eos_ids", ())), **extra)
    assert out.tolist() == rec["tokens"]
    for key, want in rec["stats"].items():
        assert stats[key] == pytest.approx(want), key
    # the run crossed a segment boundary where the record says so
    assert {s for (_, _, s, _, _) in atlas.log} <= set(rec["ladder"])


def test_read_record_single_copy_and_fallback():
    """_read_record returns the same lists whether the parts tile the record (one copy) or
    are separate tensors (one copy each); a count written as int32 into the low half of an
    int64 slot reads back as that count."""
    rec = torch.zeros(12, dtype=torch.long)
    rec[:5] = torch.tensor([7, 8, 9, 10, 11])
    rec[5:6].view(torch.int32)[0] = 3                      # what the kernels write
    rec[6:11] = torch.tensor([1, 2, 3, 4, 5])
    ids, n, more = FG._read_record(rec, rec[:5], rec[5:6], rec[6:11])
    assert (ids, n, more) == ([7, 8, 9, 10, 11], [3], [1, 2, 3, 4, 5])
    # parts that do not start at the record, are out of order, or live elsewhere
    assert FG._read_record(rec, rec[1:5], rec[5:6]) == [[8, 9, 10, 11], [3]]
    assert FG._read_record(rec, rec[5:6], rec[:5]) == [[3], [7, 8, 9, 10, 11]]
    assert FG._read_record(rec, torch.tensor([4, 5]), torch.tensor(6)) == [[4, 5], [6]]


def test_record_read_handles_on_cpu_tensors():
    """_begin_read / _finish_read (the split form of _read_record the draft loops use): on host tensors the
    record is read at once and the handle just carries the lists; parts that do not tile the record fall back to
    one read per part."""
    rec = torch.arange(12, dtype=torch.int64)
    ids, n = rec[:8], rec[8:9]
    h = FG._begin_read(rec, ids, n)
    assert FG._finish_read(h) == [list(range(8)), [8]] == FG._read_record(rec, ids, n)
    other = torch.tensor([5, 6], dtype=torch.int64)
    assert FG._finish_read(FG._begin_read(rec, ids, other)) == [list(range(8)), [5, 6]]
