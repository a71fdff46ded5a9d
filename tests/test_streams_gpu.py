"""Several streams per engine sharing one weight read (llb_spec_open_streams): every stream's tokens against the CPU
oracle run on that stream alone, and bit-identity of a stream whatever the other streams do.

Bars as everywhere on this path: ids equal to the oracle's greedy ids unless the oracle's own top-2 gap is below 1e-3;
logits within max-abs 2e-2 / rel 1e-2.  Between two runs of the same engine shape the bar is bit equality.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _f(u):
    return np.array(u, dtype=np.uint32).view(np.float32)


def _prefix(got, ref_ids, ref_top2):
    for i, (a, b) in enumerate(zip(got, ref_ids)):
        if a != b:
            gap = float(_f(ref_top2[i][1]) - _f(ref_top2[i][3]))
            assert gap < 1e-3, f"token {i}: device {a}, oracle {b}, oracle top-2 gap {gap}"
            return i
    return min(len(got), len(ref_ids))


def _drive(eng, steps, live):
    """Cycles until every live stream has `steps` tokens: per stream its ids and top-2 words, in order."""
    ids = {b: [] for b in live}
    t2 = {b: [] for b in live}
    while any(len(ids[b]) < steps for b in live):
        for b, (i, t) in enumerate(eng.cycle_streams()):
            if b in ids:
                ids[b] += [int(v) for v in i]
                t2[b] += [tuple(int(x) for x in row) for row in t]
            else:
                assert len(i) == 0
    return {b: np.array(ids[b][:steps]) for b in live}, {b: np.array(t2[b][:steps], dtype=np.uint32) for b in live}


def _oracle_runs(oracle, pack, mtp, prompts, steps, k, lookup=False):
    out = []
    for p in prompts:
        orc = oracle.Oracle(pack.index_text(), pack.data.cpu().numpy(), cap=len(p) + steps + 24)
        if lookup:
            out.append(orc.spec_lookup(p, steps, k))
        elif k > 0:
            orc.mtp_load(mtp)
            out.append(orc.spec_greedy(p, steps, k))
        else:
            out.append(orc.greedy(p, steps) + (None,))
        orc.close()
    return out


@pytest.mark.parametrize("quant,k,B", [("q8_0", 3, 4), ("q4_k_m", 3, 4), ("q4_k_s", 1, 8), ("q8_0", 0, 8), ("q4_k_m", 7, 2)])
def test_streams_match_the_oracle_per_stream(pkg, packs, oracle, llb, quant, k, B):
    """B streams with prompts of different lengths, the MTP drafter: ids, top-2 logits and acceptance counts of every
    stream equal the oracle's run of that stream alone."""
    cfg = packs.cfg_tiny(quant=quant, n_layers=8, tied_head=False, seed=5) if quant != "q8_0" else packs.cfg_tiny()
    pack = packs.build_pack(cfg)
    mtp = packs.aux1_bytes(packs.build_mtp(pack)) if k > 0 else None
    steps = 20
    prompts = [packs.synth_prompt(10 + b, 5 + 3 * b, cfg.vocab_size) for b in range(B)]
    refs = _oracle_runs(oracle, pack, mtp, prompts, steps, k)
    eng = pkg.llb.SpecEngine(pack, mtp, k=k, max_ctx=96, streams=B)
    try:
        for b, p in enumerate(prompts):
            eng.prefill_stream(b, p)
        ids, t2 = _drive(eng, steps, range(B))
        for b in range(B):
            ref_ids, ref_top2, st = refs[b]
            same = _prefix(ids[b], ref_ids, ref_top2)
            assert same == steps, (b, same)
            v_dev, v_ref = _f(t2[b][:, 1]), _f(np.array(ref_top2)[:steps, 1])
            assert np.all(np.abs(v_dev - v_ref) <= 2e-2 + 1e-2 * np.abs(v_ref)), (b, float(np.abs(v_dev - v_ref).max()))
    finally:
        eng.close()


def test_a_stream_does_not_see_its_neighbours(pkg, packs, oracle, llb):
    """Stream 2 of a four-stream engine alone, then with three other streams running beside it, one of them given its
    prompt only after stream 2 has already run some cycles (the others are parked while a prompt goes in): stream 2's
    ids, top-2 words, DeltaNet state and K rows are bit-identical."""
    cfg = packs.cfg_tiny()
    pack = packs.build_pack(cfg)
    mtp = packs.aux1_bytes(packs.build_mtp(pack))
    prompts = [packs.synth_prompt(20 + b, 6 + 2 * b, cfg.vocab_size) for b in range(4)]
    steps = 24
    runs = []
    for crowd in (False, True):
        eng = pkg.llb.SpecEngine(pack, mtp, k=3, max_ctx=96, streams=4)
        try:
            eng.prefill_stream(2, prompts[2])
            if crowd:
                eng.prefill_stream(0, prompts[0])
            ids, t2 = [], []
            late = False
            while len(ids) < steps:
                out = eng.cycle_streams()
                ids += [int(v) for v in out[2][0]]
                t2 += [tuple(int(x) for x in r) for r in out[2][1]]
                if crowd and not late and len(ids) >= 6:
                    eng.prefill_stream(3, prompts[3])      # a prompt arriving while the others are in flight
                    eng.prefill_stream(1, prompts[1])
                    late = True
            pos = eng.position_stream(2)
            states = [eng.read_state_stream(2, 0, il) for il in range(cfg.n_layers) if not cfg.is_full(il)]
            krows = [eng.read_state_stream(2, 1, il, pos - 1) for il in range(cfg.n_layers) if cfg.is_full(il)]
            runs.append((ids[:steps], t2[:steps], pos, states, krows, eng.stats_stream(2)))
        finally:
            eng.close()
    a, b = runs
    assert a[0] == b[0] and a[1] == b[1] and a[2] == b[2] and a[5] == b[5]
    for x, y in zip(a[3] + a[4], b[3] + b[4]):
        assert np.array_equal(x.view(np.uint32), y.view(np.uint32))
    assert b[5]["accepted"][1] > 0        # and it was speculating


@pytest.mark.parametrize("model,k,B", [("tiny", 3, 4), ("moe", 1, 8), ("moe", 0, 16), ("c2", 3, 4)])
def test_prompts_fed_together_equal_prompts_fed_in_turn(pkg, packs, oracle, llb, model, k, B):
    """llb_spec_prefill_streams on prompts of different lengths (one of a single token, two of equal length; on the 27B
    layer shapes one long enough for the dense prompt path) against llb_spec_prefill_stream stream by stream: every
    stream's ids, top-2 words, position, DeltaNet state and K rows are bit-identical.  A prompt fed later, while the
    others are in flight, joins the same way."""
    if model == "c2":
        cfg = packs.cfg_c2(n_layers=4, vocab_size=2048, mix_gain=0.001)
        pack = packs.build_pack(cfg, device="cuda:0")
        mtp = packs.aux1_bytes(packs.build_mtp(pack, eh="embed"))
        lens = [9, 150, 1, 9]
    else:
        cfg = packs.cfg_tiny_moe() if model == "moe" else packs.cfg_tiny()
        pack = packs.build_pack(cfg)
        mtp = packs.aux1_bytes(packs.build_mtp(pack)) if model == "tiny" else None
        lens = [(1, 7, 23, 7, 12, 4, 30, 2)[b % 8] + b // 8 for b in range(B)]
    prompts = [packs.synth_prompt(70 + b, n, cfg.vocab_size) for b, n in enumerate(lens)]
    late = B - 1
    steps = 12
    runs = []
    for together in (False, True):
        eng = pkg.llb.SpecEngine(pack, mtp, k=k, max_ctx=256, streams=B)
        try:
            eng.set_prefill(True)
            if together:
                eng.prefill_streams({b: prompts[b] for b in range(B) if b != late})
            else:
                for b in range(B):
                    if b != late:
                        eng.prefill_stream(b, prompts[b])
            first = eng.cycle_streams()
            if together:
                eng.prefill_streams({late: prompts[late]})
            else:
                eng.prefill_stream(late, prompts[late])
            ids, t2 = _drive(eng, steps, range(B))
            for b in range(B):
                if b != late:
                    ids[b] = np.concatenate([first[b][0], ids[b]])
            pos = [eng.position_stream(b) for b in range(B)]
            states = [eng.read_state_stream(b, 0, il) for b in range(B) for il in range(cfg.n_layers) if not cfg.is_full(il)]
            krows = [eng.read_state_stream(b, 1, il, pos[b] - 1) for b in range(B) for il in range(cfg.n_layers) if cfg.is_full(il)]
            runs.append((ids, t2, pos, states + krows))
        finally:
            eng.close()
    a, b_ = runs
    assert a[2] == b_[2]
    for b in range(B):
        assert np.array_equal(a[0][b], b_[0][b]) and np.array_equal(a[1][b], b_[1][b]), b
    for x, y in zip(a[3], b_[3]):
        assert np.array_equal(x.view(np.uint32), y.view(np.uint32))


@pytest.mark.parametrize("model", ["tiny", "moe"])
def test_a_sibling_engine_uses_the_first_ones_weights(pkg, packs, oracle, llb, model):
    """llb_spec_open_sibling: a second engine (other k, other streams) on the first one's weights.  Both engines, cycled in
    turn, give the ids, top-2 words and DeltaNet state of engines opened the usual way, bit for bit; the sibling allocates
    no weights; the first engine may be closed while the sibling runs on."""
    moe = model == "moe"
    cfg = packs.cfg_tiny_moe() if moe else packs.cfg_tiny()
    pack = packs.build_pack(cfg)
    mtp = None if moe else packs.aux1_bytes(packs.build_mtp(pack))
    shapes = [(3, 2), (1, 4)]                # (k, streams) of the first engine and of its sibling
    prompts = [packs.synth_prompt(90 + b, 5 + 4 * b, cfg.vocab_size) for b in range(6)]
    if moe:
        prompts = [np.concatenate([p, p, p[:2]]).astype(np.int32) for p in prompts]
    mine = [prompts[:2], prompts[2:]]
    steps = 14

    def one_cycle(eng, out):
        for b, (i, t) in enumerate(eng.cycle_streams()):
            out[b] += [(int(v), tuple(int(x) for x in row)) for v, row in zip(i, t)]

    def snapshot(eng, B):
        pos = [eng.position_stream(b) for b in range(B)]
        return pos, [eng.read_state_stream(b, 0, il).view(np.uint32) for b in range(B) for il in range(cfg.n_layers) if not cfg.is_full(il)]

    alone = []
    for (k, B), ps in zip(shapes, mine):
        eng = pkg.llb.SpecEngine(pack, mtp, k=k, max_ctx=128, streams=B)
        try:
            assert eng.weight_bytes() > 0
            eng.prefill_streams(ps)
            out = {b: [] for b in range(B)}
            for _ in range(steps):
                one_cycle(eng, out)
            alone.append((out,) + snapshot(eng, B))
        finally:
            eng.close()
    first = pkg.llb.SpecEngine(pack, mtp, k=shapes[0][0], max_ctx=128, streams=shapes[0][1])
    sib = first.sibling(k=shapes[1][0], max_ctx=128, streams=shapes[1][1])
    try:
        assert sib.weight_bytes() == 0 and first.weight_bytes() > 0
        engs = [first, sib]
        got = [{b: [] for b in range(B)} for _, B in shapes]
        for e, ps in zip(engs, mine):
            e.prefill_streams(ps)
        for _ in range(steps):                # the two engines' cycles in turn
            for e, out in zip(engs, got):
                one_cycle(e, out)
        for e, out, ref, (_, B) in zip(engs, got, alone, shapes):
            assert out == ref[0]
            pos, states = snapshot(e, B)
            assert pos == ref[1]
            for x, y in zip(states, ref[2]):
                assert np.array_equal(x, y)
        # the first engine closed under the sibling: the weights stay until the sibling closes
        first.close()
        more = sib.cycle_streams()
        assert all(len(i) >= 1 for i, _ in more)
    finally:
        first.close()
        sib.close()
    # and the device still opens and runs an engine of its own afterwards
    eng = pkg.llb.SpecEngine(pack, mtp, k=1, max_ctx=64)
    try:
        eng.prefill(prompts[0])
        assert len(eng.generate(4)[0]) == 4
    finally:
        eng.close()


def test_streams_with_the_prompt_lookup_drafter(pkg, packs, oracle, llb):
    """No drafter image: every stream drafts from its own token history (a separate history per stream)."""
    cfg = packs.cfg_tiny()
    pack = packs.build_pack(cfg)
    base = [packs.synth_prompt(30 + b, 7, cfg.vocab_size) for b in range(3)]
    prompts = [np.concatenate([p, p, p[:3]]).astype(np.int32) for p in base]
    steps = 24
    refs = _oracle_runs(oracle, pack, None, prompts, steps, 3, lookup=True)
    eng = pkg.llb.SpecEngine(pack, None, k=3, max_ctx=128, streams=3)
    try:
        for b, p in enumerate(prompts):
            eng.prefill_stream(b, p)
        ids, _ = _drive(eng, steps, range(3))
        for b in range(3):
            ref_ids, ref_top2, st = refs[b]
            assert _prefix(ids[b], ref_ids, ref_top2) == steps, b
    finally:
        eng.close()


@pytest.mark.parametrize("k,B", [(3, 2), (1, 4), (0, 8), (3, 4), (1, 8), (0, 16)])
def test_streams_of_a_routed_expert_model(pkg, packs, oracle, llb, k, B):
    """Routed experts: the router runs over every row of the pass and the expert launches take each row's own experts;
    up to sixteen rows a pass.  Plain decoding of eight and sixteen streams, and the prompt-lookup drafter on two, four
    and eight."""
    cfg = packs.cfg_tiny_moe()
    pack = packs.build_pack(cfg)
    base = [packs.synth_prompt(50 + b, 6, cfg.vocab_size) for b in range(B)]
    prompts = [np.concatenate([p, p, p[:2]]).astype(np.int32) for p in base]
    steps = 16
    refs = _oracle_runs(oracle, pack, None, prompts, steps, k, lookup=k > 0)
    eng = pkg.llb.SpecEngine(pack, None, k=k, max_ctx=96, streams=B)
    try:
        for b, p in enumerate(prompts):
            eng.prefill_stream(b, p)
        ids, t2 = _drive(eng, steps, range(B))
        for b in range(B):
            ref_ids, ref_top2, st = refs[b]
            assert _prefix(ids[b], ref_ids, ref_top2) == steps, b
    finally:
        eng.close()


def test_streams_at_the_27b_layer_shapes(pkg, packs, oracle, llb):
    """Four streams of k + 1 = 4 rows (16 rows, 32 plane columns) on config 2's own layer shapes, truncated to four
    layers and a small vocabulary: Q4_K and Q6_K in one layer, K = 17408 split 12 to 14 ways, 48 value heads over 16
    groups, 6 queries per kv head.  One stream takes a prompt long enough for the dense prompt path."""
    cfg = packs.cfg_c2(n_layers=4, vocab_size=2048, mix_gain=0.001)
    pack = packs.build_pack(cfg, device="cuda:0")
    mtp = packs.aux1_bytes(packs.build_mtp(pack, eh="embed"))
    lens = (9, 150, 21, 4)
    prompts = [packs.synth_prompt(40 + b, n, cfg.vocab_size) for b, n in enumerate(lens)]
    steps = 16
    refs = _oracle_runs(oracle, pack, mtp, prompts, steps, 3)
    eng = pkg.llb.SpecEngine(pack, mtp, k=3, max_ctx=256, streams=4)
    try:
        eng.set_prefill(True)
        for b, p in enumerate(prompts):
            eng.prefill_stream(b, p)
        assert eng.fast_rows() >= 128                       # stream 1's prompt did take the dense path
        ids, t2 = _drive(eng, steps, range(4))
        for b in range(4):
            ref_ids, ref_top2, st = refs[b]
            same = _prefix(ids[b], ref_ids, ref_top2)
            assert same >= 8, (b, same)
            v_dev, v_ref = _f(t2[b][:same, 1]), _f(np.array(ref_top2)[:same, 1])
            assert np.all(np.abs(v_dev - v_ref) <= 2e-2 + 1e-2 * np.abs(v_ref)), (b, float(np.abs(v_dev - v_ref).max()))
    finally:
        eng.close()


def test_stream_limits_are_refused_by_name(pkg, packs, llb):
    cfg = packs.cfg_tiny()
    pack = packs.build_pack(cfg)
    mtp = packs.aux1_bytes(packs.build_mtp(pack))
    with pytest.raises(pkg.llb.LlbError, match="rows a pass"):
        pkg.llb.SpecEngine(pack, mtp, k=3, max_ctx=64, streams=5)          # 20 rows
    with pytest.raises(pkg.llb.LlbError, match="max_ctx = 0"):
        pkg.llb.SpecEngine(pack, mtp, k=3, max_ctx=0)
    eng = pkg.llb.SpecEngine(pack, mtp, k=1, max_ctx=64, streams=2)
    try:
        with pytest.raises(pkg.llb.LlbError, match="no stream has a prompt"):
            eng.cycle_streams()
        with pytest.raises(pkg.llb.LlbError, match="llb_spec_cycle_streams"):
            eng.cycle()
        with pytest.raises(pkg.llb.LlbError, match="stream 2 of 2"):
            eng.prefill_stream(2, [1, 2, 3])
        with pytest.raises(pkg.llb.LlbError, match="given twice"):
            eng.prefill_streams([[1, 2, 3], [4, 5]], streams=[1, 1])
    finally:
        eng.close()
