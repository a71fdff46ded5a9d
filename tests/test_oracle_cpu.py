"""CPU tests: the oracle (oracle/q35_oracle.c) against the golden vectors produced from the reference
itself (tests/golden/make_golden.py), and its own invariants.  No GPU."""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = os.path.join(HERE, "golden")


@pytest.fixture(scope="module")
def greedy_gold():
    return json.load(open(os.path.join(GOLD, "reference_greedy.json")))


@pytest.mark.parametrize("ty", ["Q8_0", "Q4_K", "Q5_K", "Q6_K"])
def test_dequant_matches_reference_vectors(packs, oracle, ty):
    """Bit-exact against the reference's numpy decoders (tools/q4k.py, q5k.py, q6k.py) on random blocks."""
    z = np.load(os.path.join(GOLD, "dequant_vectors.npz"))
    raw, want = z[f"{ty}_raw"], z[f"{ty}_deq"]
    rows, cols = want.shape
    got = oracle.Oracle.deq_rows(packs.FMT[ty], raw, rows, cols)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # the torch decoder used to check GPU-written packs agrees too
    t = packs.dequant(ty, torch.from_numpy(raw.copy()), rows, cols).numpy()
    assert np.array_equal(t.view(np.uint32), want.view(np.uint32))
    # the dot is the serial sum of dequantised weight times x (tools/qwen35_engine.c:74-216)
    x = np.random.default_rng(0).standard_normal(cols).astype(np.float32)
    y = oracle.Oracle.gemv(packs.FMT[ty], raw, rows, cols, x)
    for r in range(rows):
        acc = np.float32(0)
        for c in range(cols):
            acc = np.float32(acc + np.float32(want[r, c] * x[c]))
        assert y[r] == acc


def _case(packs, gold, name):
    g = gold[name]
    cfg = packs.ModelCfg(**{k: g["cfg"][k] for k in ("n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim", "d_ff", "vocab_size",
                                                     "ssm_heads", "ssm_groups", "tied_head", "quant", "seed")})
    pack = packs.build_pack(cfg)
    assert hashlib.sha256(pack.data.numpy().tobytes()).hexdigest() == g["pack_sha256"], "the pack writer no longer reproduces the golden pack"
    return cfg, pack, np.array(g["prompt"], np.int32), np.array(g["ids"], np.int32), np.array(g["top2"], np.uint32)


@pytest.mark.parametrize("name", ["tiny_q8_0", "tiny_q4_k_m", "tiny_q4_k_s"])
def test_greedy_matches_reference_engine(packs, oracle, greedy_gold, name):
    """Token ids and top-2 logit bits equal those of the reference CPU engine built from its own sources."""
    cfg, pack, prompt, ids, top2 = _case(packs, greedy_gold, name)
    orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=len(prompt) + len(ids) + 8)
    got_ids, got_top2 = orc.greedy(prompt, len(ids))
    assert np.array_equal(got_ids, ids)
    assert np.array_equal(got_top2, top2)


def test_c0_shape_matches_reference_engine(packs, oracle, greedy_gold):
    """The 0.8B-shape Q8_0 configuration: first generated tokens against the reference engine's run."""
    cfg, pack, prompt, ids, top2 = _case(packs, greedy_gold, "c0_0.8b_q8_0")
    n = 6
    orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=len(prompt) + n + 8)
    got_ids, got_top2 = orc.greedy(prompt, n)
    assert np.array_equal(got_ids, ids[:n])
    assert np.array_equal(got_top2, top2[:n])


@pytest.mark.parametrize("k", [1, 3, 7])
def test_spec_cycle_is_lossless(packs, oracle, greedy_gold, k):
    """Greedy speculative decoding emits exactly the plain greedy stream (host/llb_sampler.h:20-26), for
    both drafter containers, and its statistics add up."""
    cfg, pack, prompt, ids, top2 = _case(packs, greedy_gold, "tiny_q8_0")
    mtp = packs.build_mtp(pack)
    for img in (packs.aux1_bytes(mtp),):
        orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=128)
        orc.mtp_load(img)
        sids, stop2, st = orc.spec_greedy(prompt, len(ids), k)
        assert np.array_equal(sids, ids) and np.array_equal(stop2, top2)
        assert st.served >= len(ids) and st.rows == st.cycles * (k + 1)
        acc = list(st.accepted)[1:k + 1]
        assert all(a >= b for a, b in zip(acc, acc[1:]))          # position j+1 is accepted only if j was
        assert st.served == st.cycles + sum(acc)


def test_mtp1_container_rejects_wrong_formats(packs, oracle, greedy_gold):
    """The positional container fixes Q4_K / Q6_K formats (host/llb_host.c:1574-1577): a Q8_0 drafter in it
    fails the size check instead of being misread."""
    cfg, pack, prompt, ids, top2 = _case(packs, greedy_gold, "tiny_q8_0")
    orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=64)
    with pytest.raises(RuntimeError):
        orc.mtp_load(packs.mtp1_bytes(packs.build_mtp(pack)))
    cfg2, pack2, *_ = _case(packs, greedy_gold, "tiny_q4_k_m")
    # Q4_K_M: attention matrices are Q4_K in this synthetic map, the container wants Q6_K: still refused
    orc2 = oracle.Oracle(pack2.index_text(), pack2.data.numpy(), cap=64)
    with pytest.raises(RuntimeError):
        orc2.mtp_load(packs.mtp1_bytes(packs.build_mtp(pack2)))


def test_oracle_equals_reference_build_when_present(packs, oracle, greedy_gold, tmp_path):
    """Where the reference build exists (this container), step both and compare logits and state bits."""
    if not os.path.exists(oracle.REF_SO):
        pytest.skip("oracle/_ref is not built here")
    import subprocess
    import sys
    cfg, pack, prompt, ids, top2 = _case(packs, greedy_gold, "tiny_q4_k_m")
    pack.write(str(tmp_path))
    code = ("import sys, json; sys.path.insert(0, %r); from oracle.bindings import RefTwin, Oracle; import numpy as np;"
            "r = RefTwin(%r, cap=64); idx = open(%r).read(); pk = np.fromfile(%r, dtype=np.uint8); o = Oracle(idx, pk, cap=64); ok = True\n"
            "for t, tok in enumerate(%r):\n"
            "    r.forward(tok, t); o.forward(tok, t)\n"
            "    ok &= bool((r.logits().view(np.uint32) == o.logits().view(np.uint32)).all())\n"
            "    ok &= bool((r.state_S(0).view(np.uint32) == o.state_S(0).view(np.uint32)).all())\n"
            "print(json.dumps(ok))"
            % (os.path.dirname(HERE), str(tmp_path), str(tmp_path / "index.tsv"), str(tmp_path / "pack.bin"), [int(v) for v in prompt]))
    out = subprocess.run([sys.executable, "-c", code], check=True, capture_output=True, text=True).stdout
    assert json.loads(out.strip().splitlines()[-1]) is True


def _lookup_py(hist, pos, k):
    """host/llb_host.c:1658-1676 once more, in Python."""
    for L in (3, 2, 1):
        for j in range(pos - 1, L - 2, -1):
            if all(hist[j - m] == hist[pos - m] for m in range(L)):
                return [hist[j + 1 + n] for n in range(k) if j + 1 + n <= pos]
    return []


def test_prompt_lookup_drafter(packs, oracle, greedy_gold):
    rng = np.random.default_rng(11)
    for vocab in (3, 7, 40):
        hist = rng.integers(0, vocab, 200).astype(np.int32)
        for pos in (0, 1, 2, 3, 17, 199):
            for k in (1, 3, 7):
                assert list(oracle.lookup_draft(hist, pos, k)) == _lookup_py(list(hist), pos, k)
    # the loop built on it emits the plain greedy stream
    cfg, pack, prompt, ids, top2 = _case(packs, greedy_gold, "tiny_q8_0")
    rep = np.concatenate([prompt, prompt]).astype(np.int32)
    orc = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=len(rep) + 40)
    g_ids, g_top2 = orc.greedy(rep, 24)
    l_ids, l_top2, st = orc.spec_lookup(rep, 24, 3)
    assert np.array_equal(l_ids, g_ids) and np.array_equal(l_top2, g_top2)
    assert st.served >= 24 and st.rows >= st.cycles
    assert st.served == st.cycles + sum(list(st.accepted)[1:4])


def _moe_gold_model(packs, oracle):
    """The tiny MoE pack the fixture was made from (tests/golden/make_golden_moe.py) and its known answers."""
    z = np.load(os.path.join(GOLD, "moe_ffn.npz"))
    cfg = packs.cfg_tiny_moe(n_layers=8, d_expert=512, d_shared=512)
    pack = packs.build_pack(cfg)
    assert hashlib.sha256(pack.data.numpy().tobytes()).hexdigest() == str(z["pack_sha256"])
    return z, cfg, pack


def test_moe_ffn_matches_reference_checker(packs, oracle):
    """The routed-expert FFN of the restatement against the float64 answers of the reference's own checker
    (reports/metal-catchup/tools/mx_ref.py): same experts in the same ranks, weights and shared gate to
    1e-6, output to 5e-6 relative (f32 sums of 256..512 terms against float64)."""
    z, cfg, pack = _moe_gold_model(packs, oracle)
    o = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=8)
    assert bool(np.all(z["oracle_ids_equal"])) and float(z["oracle_rel"].max()) < 5e-6
    for i in range(len(z["layer"])):
        out, ids, wts = o.moe_ffn(int(z["layer"][i]), z["h2"][i])
        assert list(ids) == list(z["rid"][i])
        assert np.abs(wts[:-1] - z["rw"][i]).max() < 1e-6 and abs(wts[-1] - z["gs"][i]) < 1e-6
        ref = z["ref"][i]
        assert np.linalg.norm(out - ref) / np.linalg.norm(ref) < 5e-6
    o.close()


def test_moe_greedy_runs_and_is_deterministic(packs, oracle):
    cfg = packs.cfg_tiny_moe()
    pack = packs.build_pack(cfg)
    prompt = packs.synth_prompt(1, 6, cfg.vocab_size)
    a = oracle.Oracle(pack.index_text(), pack.data.numpy(), cap=32)
    ids1, _ = a.greedy(prompt, 8)
    a.reset()
    ids2, _ = a.greedy(prompt, 8)
    assert list(ids1) == list(ids2) and len(ids1) == 8
    a.close()


def _sampler_cases():
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sampler_vectors.npz"))
    from oracle import bindings
    for name in z["names"]:
        name = str(name)
        p = bindings.SmpParams.from_buffer_copy(z[name + ".params"].tobytes())
        hl = z[name + ".hist_len"]
        off = np.concatenate([[0], np.cumsum(hl)])
        for r in range(len(hl)):
            yield name, r, p, z[name + ".logits"][r], z[name + ".hist"][off[r]:off[r + 1]], int(z[name + ".draft"][r]), int(z[name + ".pos"][r]), \
                int(z[name + ".tok"][r]), int(z[name + ".acc"][r])


def test_sampler_oracle_equals_the_reference_vectors():
    """The oracle's restatement of the sampler chain and of the speculative verify step (oracle/q35_sampler.c) returns, on
    every golden row, the token and the accept flag the reference's own sampler pack returned (host/llb_sampler.c, run by
    tests/golden/make_golden_sampler.py): every stage of the chain, alone and combined."""
    from oracle import bindings
    n = acc = 0
    for name, r, p, lg, hist, draft, pos, tok, a in _sampler_cases():
        t, ac, _ = bindings.smp_row(p, lg, hist, draft, pos)
        assert (t, ac) == (tok, a), (name, r, t, ac, tok, a)
        n += 1
        acc += a
    assert n >= 200 and acc > 10


def test_sampler_oracle_equals_the_reference_build_when_present():
    """On fresh random rows, against the reference's sampler compiled from its own sources (when it is on this machine)."""
    from oracle import bindings
    if not os.path.exists(bindings.REF_SMP_SO):
        pytest.skip("oracle/_ref/libllbsmp.so is not built")
    rng = np.random.default_rng(77)
    for it in range(150):
        V = int(rng.integers(8, 700))
        p = bindings.SmpParams.make(temp=float(rng.choice([0.0, 0.5, 1.0, 1.4])), top_k=int(rng.choice([0, 1, 5, 40, 300])),
                                    top_p=float(rng.choice([1.0, 0.95, 0.5])), min_p=float(rng.choice([0.0, 0.05, 0.3])),
                                    repeat_penalty=float(rng.choice([1.0, 1.2])), presence=float(rng.choice([0.0, 1.5])),
                                    frequency=float(rng.choice([0.0, 0.1])), repeat_last_n=int(rng.choice([0, 4, 64])),
                                    seed=int(rng.integers(0, 1 << 40)), min_keep=int(rng.choice([0, 1, 3])),
                                    bias=((int(rng.integers(0, V)), float(rng.normal() * 5)),) if it % 3 == 0 else ())
        lg = (rng.standard_normal(V) * float(rng.choice([0.3, 2.0, 8.0]))).astype(np.float32)
        hist = rng.integers(0, V, int(rng.integers(0, 90))).astype(np.int32)
        draft = int(np.argsort(-lg)[rng.integers(0, 3)]) if it % 4 else -1
        pos = int(rng.integers(1, 1 << 20))
        assert bindings.smp_row(p, lg, hist, draft, pos)[:2] == bindings.ref_smp_row(p, lg, hist, draft, pos), (it, V)
