"""GPU parity of the speculative cycle (MTP draft -> verify -> accept -> commit) against the CPU
oracle on the same synthetic packs and prompts.

Bars: emitted ids identical to the oracle's greedy ids (a mismatch is tolerated only where the
oracle's own top-2 logit gap is below 1e-3, after which the test stops comparing); logits within
max-abs 2e-2 / rel 1e-2; DeltaNet state within the same tolerance.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _bits_to_f(u):
    return np.array(u, dtype=np.uint32).view(np.float32)


def _compare_ids(got, ref_ids, ref_top2):
    for i, (a, b) in enumerate(zip(got, ref_ids)):
        if a != b:
            gap = float(_bits_to_f(ref_top2[i][1]) - _bits_to_f(ref_top2[i][3]))
            assert gap < 1e-3, f"token {i}: device {a}, oracle {b}, oracle top-2 gap {gap}"
            return i
    return len(ref_ids)


def _run_case(pkg, packs, oracle, cfg, k, n_prompt, steps, layers=0, seed=1):
    pack = packs.build_pack(cfg)
    mtp = packs.aux1_bytes(packs.build_mtp(pack))
    prompt = packs.synth_prompt(seed, n_prompt, cfg.vocab_size)
    orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=n_prompt + steps + 16, layers=layers)
    ref_ids, ref_top2 = orc.greedy(prompt, steps)
    orc.mtp_load(mtp)
    sids, stop2, st = orc.spec_greedy(prompt, steps, k)
    assert np.array_equal(sids, ref_ids)          # the oracle's own losslessness
    eng = pkg.llb.SpecEngine(pack, mtp, k=k, max_ctx=n_prompt + steps + 16, layers=layers)
    try:
        eng.prefill(prompt)
        ids, top2 = eng.generate(steps)
        same = _compare_ids(ids, ref_ids, ref_top2)
        # top-2 logit values of the agreeing prefix within the path's logit tolerance
        v_dev = _bits_to_f(top2[:same, 1]); v_ref = _bits_to_f(ref_top2[:same, 1])
        assert np.all(np.abs(v_dev - v_ref) <= 2e-2 + 1e-2 * np.abs(v_ref)), float(np.abs(v_dev - v_ref).max())
        stats = eng.stats()
        return same, stats, st, eng, orc, ids
    except Exception:
        eng.close()
        raise


@pytest.mark.parametrize("k", [0, 1, 3])
def test_tiny_spec_ids_match_oracle(pkg, packs, oracle, llb, k):
    cfg = packs.cfg_tiny()
    if k == 0:
        pack = packs.build_pack(cfg)
        prompt = packs.synth_prompt(1, 9, cfg.vocab_size)
        orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=64)
        ref_ids, ref_top2 = orc.greedy(prompt, 24)
        eng = pkg.llb.SpecEngine(pack, None, k=0, max_ctx=64)
        eng.prefill(prompt)
        ids, _ = eng.generate(24)
        eng.close()
        assert _compare_ids(ids, ref_ids, ref_top2) == 24
        return
    same, stats, st, eng, orc, ids = _run_case(pkg, packs, oracle, cfg, k, 9, 24)
    eng.close()
    assert same == 24
    # acceptance statistics equal the oracle's cycle by cycle when every id agrees
    assert stats["cycles"] == st.cycles and stats["served"] >= 24
    assert stats["accepted"][1:k + 1] == [int(v) for v in list(st.accepted)[1:k + 1]]


@pytest.mark.parametrize("quant", ["q4_k_m", "q4_k_s"])
def test_tiny_kquant_models(pkg, packs, oracle, llb, quant):
    cfg = packs.cfg_tiny(quant=quant, n_layers=8, tied_head=False, seed=12)
    same, stats, st, eng, orc, ids = _run_case(pkg, packs, oracle, cfg, 3, 6, 20)
    eng.close()
    assert same == 20


def test_spec_equals_plain_on_device(pkg, packs, llb):
    """Lossless by construction: the k = 3 ids equal the k = 0 ids of the same kernels bit for bit
    (the reference's gate R5, reports/unify1-gates.md:42-49)."""
    cfg = packs.cfg_tiny(n_layers=8, seed=5)
    pack = packs.build_pack(cfg)
    mtp = packs.aux1_bytes(packs.build_mtp(pack))
    prompt = packs.synth_prompt(2, 17, cfg.vocab_size)
    out = []
    for k in (0, 2, 3, 5):
        eng = pkg.llb.SpecEngine(pack, mtp if k else None, k=k, max_ctx=128)
        eng.prefill(prompt)
        out.append(eng.generate(40))
        eng.close()
    for ids, t2 in out[1:]:
        assert np.array_equal(ids, out[0][0])
        assert np.array_equal(t2, out[0][1])       # logit bits too: rows are independent of their neighbours


def test_state_and_logits_vs_oracle(pkg, packs, oracle, llb):
    """After the prompt and one cycle: committed DeltaNet state, KV rows and the full logit row
    against the oracle stepped to the same position."""
    cfg = packs.cfg_tiny(n_layers=4, seed=21)
    pack = packs.build_pack(cfg)
    mtp = packs.aux1_bytes(packs.build_mtp(pack))
    prompt = packs.synth_prompt(3, 11, cfg.vocab_size)
    eng = pkg.llb.SpecEngine(pack, mtp, k=3, max_ctx=64)
    eng.prefill(prompt)
    ids, _ = eng.cycle()
    pos = eng.position()                      # positions 0 .. pos-1 are committed
    orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=64)
    seq = list(prompt) + list(ids)
    for t in range(pos):
        orc.forward(seq[t], t)
        if t == len(prompt) - 1:
            lg = orc.logits()
            dev = eng.read_logits(0)
            assert np.all(np.abs(dev - lg) <= 2e-2 + 1e-2 * np.abs(lg)), float(np.abs(dev - lg).max())
            assert float(np.abs(dev - lg).max()) < 1e-3      # in practice far tighter than the bar
    for il in range(cfg.n_layers):
        if cfg.is_full(il):
            for p in (0, pos - 1):
                k_ref, v_ref = orc.state_kv(il, p)
                assert np.allclose(eng.read_state(1, il, p), k_ref, atol=2e-4, rtol=1e-3)
                assert np.allclose(eng.read_state(2, il, p), v_ref, atol=2e-4, rtol=1e-3)
        else:
            s_ref = orc.state_S(il)
            s_dev = eng.read_state(0, il)
            assert np.all(np.abs(s_dev - s_ref) <= 2e-2 + 1e-2 * np.abs(s_ref))
            assert float(np.abs(s_dev - s_ref).max()) < 1e-3
    eng.close()


def test_reference_shaped_pass(pkg, packs, llb):
    """llb_spec_pass serves a cycle's rows in stream order and refuses a step out of order
    (host/llb_host.c:1911, :1929-1930)."""
    cfg = packs.cfg_tiny()
    pack = packs.build_pack(cfg)
    mtp = packs.aux1_bytes(packs.build_mtp(pack))
    prompt = packs.synth_prompt(1, 9, cfg.vocab_size)
    eng = pkg.llb.SpecEngine(pack, mtp, k=3, max_ctx=64)
    eng.prefill(prompt)
    p0 = eng.position()
    ids, t2 = eng.cycle()
    y = np.zeros(4, np.float32)
    tok = int(prompt[-1])
    for r in range(len(ids)):
        assert eng.L.llb_spec_pass(eng.h, p0 + r, tok, y.ctypes.data) == 0
        assert int(y[1]) == ids[r]
        tok = int(ids[r])
    assert eng.L.llb_spec_pass(eng.h, p0 + 7, tok, y.ctypes.data) == -1
    assert b"out of order" in eng.L.llb_b200_last_error()
    eng.close()


@pytest.mark.parametrize("k", [1, 3, 5])
def test_prompt_lookup_drafter(pkg, packs, oracle, llb, k):
    """Without a drafter image the engine drafts by prompt lookup (host/llb_host.c:1655-1676, :1936): ids equal the
    oracle's greedy ids, and cycles, rows and acceptance counts equal those of the oracle's lookup loop."""
    cfg = packs.cfg_tiny(n_layers=8, seed=7)
    pack = packs.build_pack(cfg)
    # a prompt that repeats itself, so that lookups hit from the first cycle on
    base = packs.synth_prompt(4, 12, cfg.vocab_size)
    prompt = np.concatenate([base, base, base[:5]]).astype(np.int32)
    steps = 48
    orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=len(prompt) + steps + 16)
    ref_ids, ref_top2 = orc.greedy(prompt, steps)
    lids, ltop2, st = orc.spec_lookup(prompt, steps, k)
    assert np.array_equal(lids, ref_ids) and np.array_equal(ltop2, ref_top2)     # lossless in the oracle
    eng = pkg.llb.SpecEngine(pack, None, k=k, max_ctx=len(prompt) + steps + 16)
    try:
        eng.prefill(prompt)
        ids, top2 = eng.generate(steps)
        assert _compare_ids(ids, ref_ids, ref_top2) == steps
        stats = eng.stats()
        assert stats["cycles"] == st.cycles and stats["rows"] == st.rows
        assert stats["drafted"][1:k + 1] == [int(v) for v in list(st.drafted)[1:k + 1]]
        assert stats["accepted"][1:k + 1] == [int(v) for v in list(st.accepted)[1:k + 1]]
        assert stats["rows"] < stats["cycles"] * (k + 1) or k == 1   # some cycles found fewer than k drafts
    finally:
        eng.close()


def test_long_context_attention(pkg, packs, oracle, llb):
    """A context of several hundred positions: many 32-position tiles and several context slices per kv head in the
    attention kernel, prefill chunks on a warm cache, and the drafter's own KV at the same length."""
    cfg = packs.cfg_tiny(n_layers=4, seed=33)
    same, stats, st, eng, orc, ids = _run_case(pkg, packs, oracle, cfg, 3, 700, 16, seed=8)
    eng.close()
    assert same == 16


def test_fused_ffn_launch(pkg, packs, oracle, llb):
    """The FFN as one launch with a grid-wide barrier (off by default): same ids as the oracle, no barrier wait ran out,
    fewer kernels in the cycle's graph."""
    L = llb.lib()
    cfg = packs.cfg_tiny(quant="q4_k_m", n_layers=8, tied_head=False, seed=12)
    nodes = {}
    for on in (0, 1):
        was = L.llb_b200_use_fused_ffn(on)
        try:
            same, stats, st, eng, orc, ids = _run_case(pkg, packs, oracle, cfg, 3, 6, 20)
            nodes[on] = eng.graph_nodes(2)
            eng.close()
        finally:
            L.llb_b200_use_fused_ffn(was)
        assert same == 20
    assert L.llb_b200_wait_errors() == 0
    assert nodes[1] < nodes[0]


def test_prompt_chunk_width_does_not_change_the_result(pkg, packs, oracle, llb, monkeypatch):
    """The prompt is fed in chunks of 8 rows by default (LLB_PREFILL_ROWS), whatever k is; chunks of 1, 3 or k + 1 rows
    leave the same emitted ids (the oracle's), the same cycle and acceptance counts, and a DeltaNet state within the
    path's tolerance.  (37 prompt tokens: wide chunks, a ragged one, and the last one held to k + 1 rows.)"""
    cfg = packs.cfg_tiny(n_layers=8, seed=21)
    pack = packs.build_pack(cfg)
    mtp = packs.aux1_bytes(packs.build_mtp(pack))
    prompt = packs.synth_prompt(6, 37, cfg.vocab_size)
    orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=96)
    ref_ids, ref_top2 = orc.greedy(prompt, 20)
    runs = []
    for rows in ("1", "3", "4", "8"):
        monkeypatch.setenv("LLB_PREFILL_ROWS", rows)
        eng = pkg.llb.SpecEngine(pack, mtp, k=3, max_ctx=96)
        try:
            eng.prefill(prompt)
            state = eng.read_state(0, 0)
            ids, top2 = eng.generate(20)
            runs.append((ids, eng.stats(), state))
        finally:
            eng.close()
    for ids, st, state in runs:
        assert _compare_ids(ids, ref_ids, ref_top2) == 20
        assert st == runs[0][1]
        assert np.allclose(state, runs[0][2], rtol=1e-2, atol=2e-2)


@pytest.mark.parametrize("order", ["sorted", "shuffled"])
def test_draft_vocabulary_slice(pkg, packs, oracle, llb, order):
    """The drafter's head is a slice of the vocabulary (tools/mtp27/mtp_pack.py:14-30 keeps 40960 of 151936 rows): its
    argmax is an index into the slice and goes back to a token id through the ids table (host/llb_host.c:1800-1807).
    Half of a 1024-entry vocabulary, in ascending and in shuffled order: emitted ids are still the plain greedy ids, and
    cycles and acceptance counts equal the oracle's loop with the same slice -- a drafter that read the slice index as
    a token id would accept almost nothing."""
    cfg = packs.cfg_tiny(n_layers=8, seed=5)
    pack = packs.build_pack(cfg)
    rng = np.random.default_rng(17)
    ids_tab = rng.permutation(cfg.vocab_size)[:512]
    if order == "sorted":
        ids_tab = np.sort(ids_tab)
    assert not np.array_equal(ids_tab, np.arange(512))
    mtp = packs.aux1_bytes(packs.build_mtp(pack, draft_ids=ids_tab))
    prompt = packs.synth_prompt(2, 17, cfg.vocab_size)
    steps = 48
    orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=len(prompt) + steps + 16)
    ref_ids, ref_top2 = orc.greedy(prompt, steps)
    orc.mtp_load(mtp)
    sids, _, st = orc.spec_greedy(prompt, steps, 3)
    assert np.array_equal(sids, ref_ids)
    eng = pkg.llb.SpecEngine(pack, mtp, k=3, max_ctx=len(prompt) + steps + 16)
    try:
        eng.prefill(prompt)
        ids, _ = eng.generate(steps)
        stats = eng.stats()
    finally:
        eng.close()
        orc.close()
    assert _compare_ids(ids, ref_ids, ref_top2) == steps
    assert stats["cycles"] == st.cycles
    assert stats["accepted"][1:4] == [int(v) for v in list(st.accepted)[1:4]]
    assert stats["accepted"][1] > 0            # tokens inside the slice do get drafted and accepted
