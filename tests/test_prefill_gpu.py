"""The dense prompt path (llb_spec_set_prefill(1): chunks of 128 rows through tcgen05 GEMMs, two fp16 planes per operand) against
the T-row pass on the same engine build, prompt and weights: after the prompt the DeltaNet states, K/V rows, conv history
and the drafter's K rows agree within the path's bars (max-abs 2e-2 / rel 1e-2), and the first generated ids are the
same (a difference is tolerated only where the T-row pass's own top-2 gap is below 1e-3).  The ids of the T-row pass are
checked against the oracle elsewhere; here one case also runs the oracle so the dense path is compared with it directly.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
STEPS = 16


def _f(u):
    return np.array(u, dtype=np.uint32).view(np.float32)


def _close(a, b):
    return np.all(np.abs(a - b) <= 2e-2 + 1e-2 * np.abs(b))


def _run(pkg, pack, mtp, k, prompt, fast):
    eng = pkg.llb.SpecEngine(pack, mtp, k=k, max_ctx=len(prompt) + STEPS + 32)
    try:
        eng.set_prefill(fast)
        eng.prefill(prompt)
        cfg = pack.cfg
        st = {"fast_rows": eng.fast_rows()}
        n = len(prompt)
        for il in range(cfg.n_layers):
            if cfg.is_full(il):
                st[f"k{il}"] = np.stack([eng.read_state(1, il, p) for p in (0, 1, n // 2, n - 6, n - 2)])
                st[f"v{il}"] = np.stack([eng.read_state(2, il, p) for p in (0, 1, n // 2, n - 6, n - 2)])
            else:
                st[f"S{il}"] = eng.read_state(0, il)
                st[f"c{il}"] = np.stack([eng.read_state(3, il, p) for p in (n - 4, n - 3, n - 2)])
        if mtp is not None:
            st["mk"] = np.stack([eng.read_state(5, 0, p) for p in (0, 1, n // 2, n - 6, n - 2)])
        ids, top2 = eng.generate(STEPS)
        assert pkg.llb.lib().llb_b200_wait_errors() == 0
        return st, ids, top2
    finally:
        eng.close()


def _compare(pkg, pack, mtp, k, prompt):
    ref_st, ref_ids, ref_top2 = _run(pkg, pack, mtp, k, prompt, False)
    st, ids, top2 = _run(pkg, pack, mtp, k, prompt, True)
    assert ref_st.pop("fast_rows") == 0
    assert st.pop("fast_rows") == len(prompt) - 1 - (k + 1)          # all but the last k + 1 rows went through the dense path
    for key, ref in ref_st.items():
        assert _close(st[key], ref), (key, float(np.abs(st[key] - ref).max()), float(np.abs(ref).max()))
    same = STEPS
    for i in range(STEPS):
        if ids[i] != ref_ids[i]:
            gap = float(_f(ref_top2[i][1]) - _f(ref_top2[i][3]))
            assert gap < 1e-3, f"token {i}: dense path {ids[i]}, T-row pass {ref_ids[i]}, top-2 gap {gap}"
            same = i
            break
    assert _close(_f(top2[:same, 1]), _f(ref_top2[:same, 1]))
    return ids, ref_ids


@pytest.mark.parametrize("quant", ["q8_0", "q4_k_m", "q4_k_s"])
def test_tiny_models(pkg, packs, llb, quant):
    """Two full chunks, a ragged one and the k + 1 rows left to the T-row pass; Q8_0, Q4_K + Q6_K, Q4_K + Q5_K + Q6_K."""
    cfg = packs.cfg_tiny(quant=quant, n_layers=8, tied_head=(quant == "q8_0"), seed=12)
    pack = packs.build_pack(cfg)
    mtp = packs.aux1_bytes(packs.build_mtp(pack))
    _compare(pkg, pack, mtp, 3, packs.synth_prompt(7, 300, cfg.vocab_size))


def test_prompt_lookup_engine_and_k0(pkg, packs, llb):
    """No drafter image: nothing of the drafter to fill; k = 0 leaves one row to the T-row pass."""
    cfg = packs.cfg_tiny(n_layers=8, seed=7)
    pack = packs.build_pack(cfg)
    prompt = packs.synth_prompt(8, 530, cfg.vocab_size)
    _compare(pkg, pack, None, 3, prompt)
    _compare(pkg, pack, None, 0, prompt)


def test_c0_shape_against_the_oracle(pkg, packs, oracle, llb):
    """The 0.8B shape (d 1024, FFN 3584 = 14 super-blocks, 8 + 2 heads of 128) on eight layers, Q8_0: the dense path's ids
    also against the CPU oracle's greedy ids."""
    pack = packs.build_pack(packs.cfg_c0(), layers=8)
    cfg = pack.cfg
    mtp = packs.aux1_bytes(packs.build_mtp(pack))
    prompt = packs.synth_prompt(1, 290, cfg.vocab_size)
    ids, _ = _compare(pkg, pack, mtp, 3, prompt)
    orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=len(prompt) + STEPS + 8)
    ref_ids, ref_top2 = orc.greedy(prompt, STEPS)
    orc.close()
    for i in range(STEPS):
        if ids[i] != ref_ids[i]:
            assert float(_f(ref_top2[i][1]) - _f(ref_top2[i][3])) < 1e-3, i
            break


def test_c2_shape_truncated(pkg, packs, llb):
    """The 27B layer shapes (d 5120, FFN 17408, six queries per kv head, 48 DeltaNet heads over 16 groups, Q4_K and Q6_K),
    four layers, 600 prompt tokens: four full chunks, a ragged one."""
    cfg = packs.cfg_c2(n_layers=4, vocab_size=2048)
    pack = packs.build_pack(cfg, device="cuda:0")
    mtp = packs.aux1_bytes(packs.build_mtp(pack))
    _compare(pkg, pack, mtp, 3, packs.synth_prompt(3, 600, cfg.vocab_size))
