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
         "hybrid": FG.fast_hybrid_generate}


@pytest.mark.parametrize("rec", RECORDS, ids=lambda r: f"{r['geometry']}-D{r['cfg']['block_size']}-{r['mode']}-"
                                                         f"{'forced' if r['forced'] else 'free'}")
def test_stream_matches_reference_loops(rec):
    cfg = rec["cfg"]
    state = synthetic.make_state(cfg, seed=rec["state_seed"])
    om = O.OracleModel(cfg, state, max_positions=max(rec["ladder"]) + max(rec["m_set"]))
    args = generate.args_from_config(cfg)
    roles = ("ar",) if rec["mode"] == "ar" else ("ar", "draft", "verify")
    atlas = CpuAtlas(om, args, rec["ladder"], rec["m_set"], roles)
    prompt = synthetic.random_prompt(rec["prompt_len"], cfg["vocab_size"], seed=rec["prompt_seed"])
    with patched_host_ops(cfg["block_size"], rec["forced"]):
        out, stats = MODES[rec["mode"]](OracleModel(om, args), atlas, prompt,
                                        max_gen_len=rec["new_tokens"], eos_ids=())
    assert out.tolist() == rec["tokens"]
    for key, want in rec["stats"].items():
        assert stats[key] == pytest.approx(want), key
    # the run crossed a segment boundary where the record says so
    assert {s for (_, _, s, _, _) in atlas.log} <= set(rec["ladder"])
