"""The 27B-shape Q4_K_M configuration (the one the headline number is quoted on) against the CPU oracle.

Layer shapes are the configuration's own -- d 5120, FFN 17408, 24 Q / 4 KV heads of 256 (six queries per kv head, so
8-row prompt chunks sit exactly on the attention kernel's 48-query limit), 48 DeltaNet value heads over 16 q/k groups
(value head hh reads group hh % 16: every group serves three heads, tools/qwen35_engine.c:621-626), the Q4_K_M mix of
Q4_K and Q6_K inside one layer -- truncated to four layers and a small vocabulary so the oracle finishes in about a
minute.  With N(0, 0.02) weights at this width a drafter is right about once in a vocabulary, so two of the cases
weaken the residual mixing (packs.ModelCfg.mix_gain) to get cycles that accept some drafts and reject others; the
arithmetic under test is unchanged.  The last case is the full 64-layer pack on eight tokens.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _f(u):
    return np.array(u, dtype=np.uint32).view(np.float32)


def _same_prefix(got, ref_ids, ref_top2):
    """Length of the agreeing prefix; a mismatch is tolerated only where the oracle's own top-2 gap is below 1e-3."""
    for i, (a, b) in enumerate(zip(got, ref_ids)):
        if a != b:
            gap = float(_f(ref_top2[i][1]) - _f(ref_top2[i][3]))
            assert gap < 1e-3, f"token {i}: device {a}, oracle {b}, oracle top-2 gap {gap}"
            return i
    return len(ref_ids)


def test_c2_mtp_partial_acceptance(pkg, packs, oracle, llb):
    """MTP k = 3 over a 45-token prompt (five 8-row chunks, a ragged one, the last held to k + 1 rows), then 40 tokens:
    ids, top-2 logits, acceptance counts by position, a full logit row, DeltaNet state and K/V rows."""
    cfg = packs.cfg_c2(n_layers=4, vocab_size=2048, mix_gain=0.001)
    pack = packs.build_pack(cfg, device="cuda:0")
    mtp = packs.aux1_bytes(packs.build_mtp(pack, eh="embed"))
    prompt = packs.synth_prompt(3, 45, cfg.vocab_size)
    steps = 40
    host = pack.data.cpu().numpy()
    types = {e.name.split(".")[-2]: e.ty for e in pack.entries if e.name.startswith("blk.") and e.rows > 1}
    assert {pack.by_name[f"blk.{i}.ffn_down.weight"].ty for i in range(4)} == {"Q4_K", "Q6_K"} and types["ffn_gate"] == "Q4_K"
    orc = oracle.Oracle(pack.index_text(), host, cap=len(prompt) + steps + 16)
    orc.mtp_load(mtp)
    ref_ids, ref_top2, st = orc.spec_greedy(prompt, steps, 3)
    eng = pkg.llb.SpecEngine(pack, mtp, k=3, max_ctx=len(prompt) + steps + 16)
    try:
        eng.prefill(prompt)
        ids, top2 = eng.generate(steps)
        same = _same_prefix(ids, ref_ids, ref_top2)
        v_dev, v_ref = _f(top2[:same, 1]), _f(ref_top2[:same, 1])
        assert np.all(np.abs(v_dev - v_ref) <= 2e-2 + 1e-2 * np.abs(v_ref)), float(np.abs(v_dev - v_ref).max())
        stats = eng.stats()
        if same == steps:
            # cycle by cycle the device accepted what the oracle's loop accepted
            assert stats["cycles"] == st.cycles
            assert stats["accepted"][1:4] == [int(v) for v in list(st.accepted)[1:4]]
        # the point of this pack: some drafts accepted, some rejected, and a rejection after a partial accept
        acc = stats["accepted"][1:4]
        assert acc[0] > 0 and acc[0] < stats["drafted"][1] and acc[2] < acc[0], stats
        assert stats["served"] > stats["cycles"]
        # state after the run: stop the oracle at the device's committed position
        pos = eng.position()
        seq = list(prompt) + [int(t) for t in ids]
        orc2 = oracle.Oracle(pack.index_text(), host, cap=pos + 8)
        for t in range(pos):
            orc2.forward(seq[t], t)
        for il in range(cfg.n_layers):
            if cfg.is_full(il):
                for p in (0, 7, 44, pos - 1):
                    k_ref, v_ref2 = orc2.state_kv(il, p)
                    assert np.allclose(eng.read_state(1, il, p), k_ref, atol=2e-4, rtol=1e-3), (il, p)
                    assert np.allclose(eng.read_state(2, il, p), v_ref2, atol=2e-4, rtol=1e-3), (il, p)
            else:
                s_ref, s_dev = orc2.state_S(il), eng.read_state(0, il)
                assert np.all(np.abs(s_dev - s_ref) <= 2e-2 + 1e-2 * np.abs(s_ref)), (il, float(np.abs(s_dev - s_ref).max()))
                # every q/k group serves three value heads (hh % 16): they must differ from one another
                S = s_dev.reshape(cfg.ssm_heads, 128, 128)
                assert not np.allclose(S[0], S[16]) and not np.allclose(S[16], S[32])
        # one more cycle: row 0 of its verify pass is the oracle's next position
        orc2.forward(seq[pos], pos)
        lg = orc2.logits()
        eng.cycle()
        dev = eng.read_logits(0)
        assert np.all(np.abs(dev - lg) <= 2e-2 + 1e-2 * np.abs(lg)), float(np.abs(dev - lg).max())
        orc2.close()
    finally:
        eng.close()
        orc.close()


def test_c2_prompt_lookup_with_qkv_in_its_own_format(pkg, packs, oracle, llb):
    """The prompt-lookup drafter on a model that soon repeats itself (256-entry vocabulary): cycles serve one to four rows
    and some reject midway.  ids, cycles, rows, drafted and accepted equal the oracle's lookup loop, and the ids and
    logit bits equal the k = 0 engine's.  The DeltaNet input matrices (attn_qkv, attn_gate, ssm_beta, ssm_alpha) are Q5_K
    here: their one launch then wants 2 K-slices at four rows and 4 at eight, and the conv ring, which keeps attn_qkv rows
    as partial sums across both kinds of pass, needs the one split fixed at open."""
    q5 = tuple((leaf, "Q5_K") for leaf in ("attn_qkv", "attn_gate", "ssm_beta", "ssm_alpha"))
    cfg = packs.cfg_c2(n_layers=4, vocab_size=256, mix_gain=0.001, type_overrides=q5)
    pack = packs.build_pack(cfg, device="cuda:0")
    assert pack.by_name["blk.0.attn_qkv.weight"].ty == "Q5_K" and pack.by_name["blk.0.ffn_gate.weight"].ty == "Q4_K"
    L = llb.lib()
    sms = L.llb_b200_sm_count()
    group = (cfg.convd + cfg.vdc + 2 * cfg.ssm_heads + 15) // 16
    k8, k16 = L.llb_b200_gemm_ksplit(9, 8, group, 20, sms), L.llb_b200_gemm_ksplit(9, 16, group, 20, sms)
    assert k8 != k16                                   # the free choice would differ between the two widths
    base = packs.synth_prompt(4, 14, cfg.vocab_size)
    prompt = np.concatenate([base, base, base[:6]]).astype(np.int32)
    steps = 64
    host = pack.data.cpu().numpy()
    orc = oracle.Oracle(pack.index_text(), host, cap=len(prompt) + steps + 16)
    ref_ids, ref_top2, st = orc.spec_lookup(prompt, steps, 3)
    orc.close()
    out = {}
    for k in (0, 3):
        eng = pkg.llb.SpecEngine(pack, None, k=k, max_ctx=len(prompt) + steps + 16)
        try:
            eng.prefill(prompt)
            out[k] = eng.generate(steps) + (eng.stats(),)
        finally:
            eng.close()
    ids, top2, stats = out[3]
    assert _same_prefix(ids, ref_ids, ref_top2) == steps
    assert np.array_equal(ids, out[0][0]) and np.array_equal(top2, out[0][1])      # lossless, bit for bit
    assert stats["cycles"] == st.cycles and stats["rows"] == st.rows
    assert stats["drafted"][1:4] == [int(v) for v in list(st.drafted)[1:4]]
    assert stats["accepted"][1:4] == [int(v) for v in list(st.accepted)[1:4]]
    assert stats["accepted"][1] > 0 and stats["served"] > stats["cycles"]          # the lookups did hit
    assert stats["rows"] < 4 * stats["cycles"]                                     # and some cycles found fewer than k drafts


def test_c2_full_depth_eight_tokens(pkg, packs, oracle, llb):
    """All 64 layers and the 151936-row head, as the benchmark builds them: four prompt tokens and four generated ones
    against the oracle (about half a minute of host time), then the top-2 logits of the generated rows."""
    cfg = packs.cfg_c2()
    pack = packs.build_pack(cfg, device="cuda:0")
    mtp = packs.aux1_bytes(packs.build_mtp(pack))
    prompt = packs.synth_prompt(3, 4, cfg.vocab_size)
    import torch
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    orc = oracle.Oracle(pack.index_text(), pack.data.cpu().numpy(), cap=16)
    ref_ids, ref_top2 = orc.greedy(prompt, 4)
    orc.close()
    eng = pkg.llb.SpecEngine(pack, mtp, k=3, max_ctx=64)
    try:
        eng.prefill(prompt)
        ids, top2 = eng.generate(4)
    finally:
        eng.close()
    same = _same_prefix(ids, ref_ids, ref_top2)
    v_dev, v_ref = _f(top2[:same, 1]), _f(ref_top2[:same, 1])
    assert same >= 1 and np.all(np.abs(v_dev - v_ref) <= 2e-2 + 1e-2 * np.abs(v_ref))
