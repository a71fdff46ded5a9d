"""GPU parity of the routed-expert FFN (host/llb_host.c:622-724, tools/payload-moeany.patch) through the C ABI:
the expert FFN alone against the known answers of the reference's float64 checker (tests/golden/moe_ffn.npz)
and against the CPU oracle, and whole MoE models (plain greedy and the prompt-lookup speculative loop)
against the oracle's ids and top-2 logits.

Bars: chosen experts identical and in the same ranks; weights and the shared gate within 1e-6; FFN output
within 2e-5 of its norm (measured 1e-6 .. 5e-6 against float64: fp32 sums of a few thousand cancelling terms in
tensor-core order.  Before the K-quant "min" term took the 32-column activation means with their lo half scaled
by 2048, that half was an fp16 subnormal for activations as small as silu(g) * u * weight and the error was
3e-5 .. 1.2e-4); ids as in
test_spec_gpu.py (a mismatch only where the oracle's own top-2 gap is below 1e-3); top-2 logits within
max-abs 2e-2 / rel 1e-2.
"""
import hashlib
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _bits_to_f(u):
    return np.array(u, dtype=np.uint32).view(np.float32)


def _compare_ids(got, ref_ids, ref_top2):
    for i, (a, b) in enumerate(zip(got, ref_ids)):
        if a != b:
            gap = float(_bits_to_f(ref_top2[i][1]) - _bits_to_f(ref_top2[i][3]))
            assert gap < 1e-3, f"token {i}: device {a}, oracle {b}, oracle top-2 gap {gap}"
            return i
    return len(ref_ids)


def test_moe_ffn_matches_reference_checker(pkg, packs, llb):
    z = np.load(os.path.join(GOLD, "moe_ffn.npz"))
    cfg = packs.cfg_tiny_moe(n_layers=8, d_expert=512, d_shared=512)
    pack = packs.build_pack(cfg)
    assert hashlib.sha256(pack.data.numpy().tobytes()).hexdigest() == str(z["pack_sha256"])
    eng = pkg.llb.SpecEngine(pack, None, k=3, max_ctx=64)
    try:
        k = cfg.n_experts_used
        for i in range(len(z["layer"])):
            out, ids, wt = eng.moe_ffn(int(z["layer"][i]), z["h2"][i][None, :])
            assert list(ids[0, :k]) == list(z["rid"][i]) and ids[0, k] == cfg.n_experts
            assert np.abs(wt[0, :k] - z["rw"][i]).max() < 1e-6 and abs(wt[0, k] - z["gs"][i]) < 1e-6
            ref = z["ref"][i]
            assert np.linalg.norm(out[0] - ref) / np.linalg.norm(ref) < 2e-5
    finally:
        eng.close()


@pytest.mark.parametrize("T,k", [(1, 0), (2, 1), (4, 3), (6, 5), (8, 7)])
def test_moe_ffn_rows_vs_oracle_and_row_independence(pkg, packs, oracle, llb, T, k):
    """T rows at once (different experts per row, every plane width): each row equals the oracle's answer for it,
    and equals bit for bit the same row run alone -- the property that keeps greedy speculation lossless."""
    cfg = packs.cfg_tiny_moe(n_layers=8, d_expert=512, d_shared=512)
    pack = packs.build_pack(cfg)
    orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=8)
    eng = pkg.llb.SpecEngine(pack, None, k=k, max_ctx=64)
    try:
        rng = np.random.default_rng(100 + T)
        h2 = rng.standard_normal((T, cfg.d_model)).astype(np.float32)
        for il in (0, 2):      # Q5_K and Q4_K down stacks
            out, ids, wt = eng.moe_ffn(il, h2)
            for t in range(T):
                ro, rid, rw = orc.moe_ffn(il, h2[t])
                assert list(ids[t, :-1]) == list(rid)
                assert np.abs(wt[t] - rw).max() < 1e-6
                assert np.linalg.norm(out[t] - ro) / np.linalg.norm(ro) < 2e-5
            assert len({tuple(r) for r in ids[:, :-1]}) > 1 or T == 1     # the rows do not all share their experts
            alone, _, _ = eng.moe_ffn(il, h2[T - 1:T])
            assert np.array_equal(alone[0].view(np.uint32), out[T - 1].view(np.uint32))
    finally:
        eng.close()
        orc.close()


@pytest.mark.parametrize("T,k,B", [(16, 3, 4), (16, 0, 16), (11, 1, 8)])
def test_moe_ffn_sixteen_rows_of_several_streams(pkg, packs, oracle, llb, T, k, B):
    """The pass of a several-stream engine (32 plane columns staged, an expert tile multiplied with its own row group's
    two n-tiles): every row against the oracle, and bit for bit the same row alone in the pass, where it is row 0 of the
    first row group (between engines of different widths the K-slices of the down launch differ, and with them the order
    of the fp32 sums)."""
    cfg = packs.cfg_tiny_moe(n_layers=8, d_expert=512, d_shared=512)
    pack = packs.build_pack(cfg)
    orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=8)
    eng = pkg.llb.SpecEngine(pack, None, k=k, max_ctx=64, streams=B)
    try:
        rng = np.random.default_rng(300 + T + B)
        h2 = rng.standard_normal((T, cfg.d_model)).astype(np.float32)
        for il in (0, 2):      # Q5_K and Q4_K down stacks
            out, ids, wt = eng.moe_ffn(il, h2)
            for t in range(T):
                ro, rid, rw = orc.moe_ffn(il, h2[t])
                assert list(ids[t, :-1]) == list(rid)
                assert np.abs(wt[t] - rw).max() < 1e-6
                assert np.linalg.norm(out[t] - ro) / np.linalg.norm(ro) < 2e-5
            for t in (0, 7, 8, T - 1):
                alone, _, _ = eng.moe_ffn(il, h2[t:t + 1])
                assert np.array_equal(alone[0].view(np.uint32), out[t].view(np.uint32)), t
    finally:
        eng.close()
        orc.close()


@pytest.mark.parametrize("k", [0, 3])
def test_tiny_moe_model_ids_match_oracle(pkg, packs, oracle, llb, k):
    """A hybrid model whose every FFN is routed: plain greedy (k = 0) and the prompt-lookup speculative loop."""
    cfg = packs.cfg_tiny_moe(n_layers=8, d_expert=512, d_shared=512)
    pack = packs.build_pack(cfg)
    base = packs.synth_prompt(4, 10, cfg.vocab_size)
    prompt = np.concatenate([base, base, base[:4]]).astype(np.int32)
    steps = 32
    orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=len(prompt) + steps + 16)
    ref_ids, ref_top2 = orc.greedy(prompt, steps)
    eng = pkg.llb.SpecEngine(pack, None, k=k, max_ctx=len(prompt) + steps + 16)
    try:
        eng.prefill(prompt)
        ids, top2 = eng.generate(steps)
        same = _compare_ids(ids, ref_ids, ref_top2)
        assert same == steps
        v_dev = _bits_to_f(top2[:same, 1]); v_ref = _bits_to_f(ref_top2[:same, 1])
        assert np.all(np.abs(v_dev - v_ref) <= 2e-2 + 1e-2 * np.abs(v_ref)), float(np.abs(v_dev - v_ref).max())
        if k:
            lids, ltop2, st = orc.spec_lookup(prompt, steps, k)
            assert np.array_equal(lids, ref_ids)
            stats = eng.stats()
            assert stats["cycles"] == st.cycles and stats["rows"] == st.rows
    finally:
        eng.close()
        orc.close()


def test_moe_config3_shape_layers(pkg, packs, oracle, llb):
    """The MoE configuration's own widths (d 2048, 256 experts, top 8 + shared, 512 columns each, Q4_K_S) on four
    layers and a small vocabulary: ids and logits against the oracle."""
    cfg = packs.cfg_c3(n_layers=4, vocab_size=4096, tied_head=True)
    pack = packs.build_pack(cfg)
    prompt = packs.synth_prompt(2, 7, cfg.vocab_size)
    steps = 8
    orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=len(prompt) + steps + 16)
    ref_ids, ref_top2 = orc.greedy(prompt, steps)
    eng = pkg.llb.SpecEngine(pack, None, k=3, max_ctx=len(prompt) + steps + 16)
    try:
        eng.prefill(prompt)
        ids, top2 = eng.generate(steps)
        same = _compare_ids(ids, ref_ids, ref_top2)
        assert same >= steps // 2
        v_dev = _bits_to_f(top2[:same, 1]); v_ref = _bits_to_f(ref_top2[:same, 1])
        assert np.all(np.abs(v_dev - v_ref) <= 2e-2 + 1e-2 * np.abs(v_ref)), float(np.abs(v_dev - v_ref).max())
    finally:
        eng.close()
        orc.close()


def test_moe_router_ties_and_all_experts(pkg, packs, oracle, llb):
    """Edge cases of the routing rule (llb_moe_topk): two experts with bit-identical router rows tie in
    probability and the LOWER id takes the earlier rank; with k = expert count every expert is chosen, in
    descending order of probability, and the weights sum to one."""
    cfg = packs.cfg_tiny_moe(n_layers=4, d_expert=256, d_shared=256, n_experts_used=8)
    pack = packs.build_pack(cfg)
    e = pack.by_name["blk.1.ffn_gate_inp.weight"]
    r = pack.raw(e.name).view(-1, cfg.d_model * 4)
    r[2] = r[5]                                  # experts 2 and 5 of layer 1 get the same router row
    orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=8)
    eng = pkg.llb.SpecEngine(pack, None, k=3, max_ctx=64)
    try:
        h2 = np.random.default_rng(9).standard_normal((4, cfg.d_model)).astype(np.float32)
        out, ids, wt = eng.moe_ffn(1, h2)
        for t in range(4):
            ro, rid, rw = orc.moe_ffn(1, h2[t])
            assert list(ids[t, :-1]) == list(rid) and sorted(rid) == list(range(8))
            pos = list(rid)
            assert pos.index(2) + 1 == pos.index(5) and wt[t, pos.index(2)] == wt[t, pos.index(5)]
            assert np.all(np.diff(wt[t, :-1]) <= 0) and abs(float(wt[t, :-1].sum()) - 1.0) < 1e-5
            assert np.abs(wt[t] - rw).max() < 1e-6
            assert np.linalg.norm(out[t] - ro) / np.linalg.norm(ro) < 2e-5
    finally:
        eng.close()
        orc.close()
