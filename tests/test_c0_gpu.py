"""The 0.8B-shape Q8_0 configuration end to end on the GPU (prompt 64, 128 generated, MTP k = 3)
against the committed run of the reference CPU engine (tests/golden/reference_greedy.json)."""
import hashlib
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_greedy.json")


def test_c0_spec_ids_match_reference_run(pkg, packs, llb):
    g = json.load(open(GOLD))["c0_0.8b_q8_0"]
    cfg = packs.cfg_c0()
    pack = packs.build_pack(cfg)
    assert hashlib.sha256(pack.data.numpy().tobytes()).hexdigest() == g["pack_sha256"]
    prompt, ids, top2 = np.array(g["prompt"], np.int32), np.array(g["ids"], np.int32), np.array(g["top2"], np.uint32)
    mtp = packs.aux1_bytes(packs.build_mtp(pack))
    eng = pkg.llb.SpecEngine(pack, mtp, k=3, max_ctx=256)
    eng.prefill(prompt)
    got, got2 = eng.generate(len(ids))
    stats = eng.stats()
    eng.close()
    f = lambda u: np.array(u, dtype=np.uint32).view(np.float32)
    n = len(ids)
    for i in range(len(ids)):
        if got[i] != ids[i]:
            gap = float(f(top2[i][1]) - f(top2[i][3]))
            assert gap < 1e-3, f"token {i}: device {got[i]}, reference {ids[i]}, reference top-2 gap {gap}"
            n = i
            break
    assert n >= 32, "the streams should agree well past the first tokens"
    v_dev, v_ref = f(got2[:n, 1]), f(top2[:n, 1])
    assert np.all(np.abs(v_dev - v_ref) <= 2e-2 + 1e-2 * np.abs(v_ref))
    assert stats["served"] >= len(ids) and stats["cycles"] <= len(ids)
