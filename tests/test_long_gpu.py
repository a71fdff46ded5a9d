"""Attention over a context of more than 8192 positions at the long-context configuration's head shape (16 Q / 4 KV
heads of 256 dims: four queries per kv head, 37 context slices per kv head on 148 SMs, 224 positions a slice -- the
slice length is not a divisor of the context), the fp16 hi/lo K/V cache at that depth, 1027 prompt chunks of eight rows,
and k = 1 and k = 5 (two and six verify rows: both plane widths).  Checked against ids, top-2 logit bits, the whole logit
row after the prompt and a K row, all written by the REFERENCE CPU engine (tests/golden/make_golden_long.py: half an
hour of host time on eight cores, which is why the fixture is committed instead of recomputed)."""
import hashlib
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def long_case(packs):
    g = np.load(os.path.join(ROOT, "tests", "golden", "long_context.npz"))
    cfg = packs.cfg_long()
    pack = packs.build_pack(cfg)                       # on the CPU: the same bytes the fixture was made from
    assert hashlib.sha256(pack.data.numpy().tobytes()).hexdigest() == str(g["pack_sha256"])
    prompt = packs.synth_prompt(int(g["prompt_seed"]), int(g["n_prompt"]), cfg.vocab_size)
    return g, cfg, pack, prompt


@pytest.mark.parametrize("k", [1, 5])
def test_context_beyond_8192_positions(pkg, packs, llb, long_case, k):
    g, cfg, pack, prompt = long_case
    f = lambda u: np.array(u, dtype=np.uint32).view(np.float32)
    ref_ids, ref_top2, n = g["ids"], g["top2"], len(prompt)
    steps = len(ref_ids)
    mtp = packs.aux1_bytes(packs.build_mtp(pack))
    eng = pkg.llb.SpecEngine(pack, mtp, k=k, max_ctx=n + steps + 32)
    try:
        eng.prefill(prompt)
        first, t2first = eng.cycle()
        # row 0 of the first cycle is the last prompt position: its logits are the reference's logits after the prompt
        row, ref_row = eng.read_logits(0), g["logits_after_prompt"]
        assert np.all(np.abs(row - ref_row) <= 2e-2 + 1e-2 * np.abs(ref_row)), float(np.abs(row - ref_row).max())
        k_dev = eng.read_state(1, 3, n - 1)
        assert np.allclose(k_dev, g["k_last_prompt_row"], atol=2e-4, rtol=1e-3)
        rest, t2rest = eng.generate(steps - len(first)) if len(first) < steps else (np.zeros(0, np.int32), np.zeros((0, 4), np.uint32))
        ids = np.concatenate([first, rest])[:steps]
        top2 = np.concatenate([t2first, t2rest])[:steps]
    finally:
        eng.close()
    same = steps
    for i in range(steps):
        if ids[i] != ref_ids[i]:
            gap = float(f(ref_top2[i][1]) - f(ref_top2[i][3]))
            assert gap < 1e-3, f"token {i}: device {ids[i]}, reference {ref_ids[i]}, reference top-2 gap {gap}"
            same = i
            break
    assert same >= 1
    v_dev, v_ref = f(top2[:same, 1]), f(ref_top2[:same, 1])
    assert np.all(np.abs(v_dev - v_ref) <= 2e-2 + 1e-2 * np.abs(v_ref))
