"""Sampling-mode verify on the device against the reference's sampler: the golden rows drawn from the reference's own
sampler pack (tests/golden/sampler_vectors.npz), vocabulary-sized rows against the oracle's restatement, and the engine's
sampled cycles replayed row by row through the oracle on the device's own logits.

Bars: the emitted token and the accept flag equal the reference's.  A difference is excused only where the oracle's own
decision was within 1e-6 of flipping (its margin): exp is taken in double and rounded on the device, by libm's expf on the
host, and block-wide double sums replace sequential ones where the whole vocabulary is summed.
"""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sampler_vectors.npz")


def _dev_params(llb, op):
    """oracle.bindings.SmpParams -> the library's llb_smp_params"""
    return llb.SmpParams.make(temp=op.temp, top_p=op.top_p, min_p=op.min_p, top_k=op.top_k, repeat_penalty=op.repeat_penalty,
                              repeat_last_n=op.repeat_last_n, presence=op.presence, frequency=op.frequency, seed=op.seed,
                              min_keep=op.min_keep, bias=[(op.bias_ids[j], op.bias_vals[j]) for j in range(op.n_bias)])


def test_golden_rows_of_the_reference_sampler(llb, oracle, dev):
    from oracle import bindings
    z = np.load(GOLD)
    total = 0
    for name in z["names"]:
        name = str(name)
        op = bindings.SmpParams.from_buffer_copy(z[name + ".params"].tobytes())
        lg = np.ascontiguousarray(z[name + ".logits"])
        T, V = lg.shape
        hl = z[name + ".hist_len"]
        off = np.concatenate([[0], np.cumsum(hl)])
        n = op.repeat_last_n
        wins = [z[name + ".hist"][off[r]:off[r + 1]][-n:] if n > 0 else [] for r in range(T)]
        buf = dev(lg.nbytes).write(lg)
        tok, acc, val = llb.smp_rows(_dev_params(llb, op), buf.ptr, T, V, z[name + ".draft"], z[name + ".pos"], wins)
        for r in range(T):
            if (tok[r], acc[r]) != (z[name + ".tok"][r], z[name + ".acc"][r]):
                _, _, margin = bindings.smp_row(op, lg[r], z[name + ".hist"][off[r]:off[r + 1]], int(z[name + ".draft"][r]), int(z[name + ".pos"][r]))
                assert margin < 1e-6, (name, r, int(tok[r]), int(acc[r]), int(z[name + ".tok"][r]), int(z[name + ".acc"][r]), margin)
            else:
                assert val[r] == lg[r, tok[r]]          # the emitted token's raw logit
                total += 1
    assert total >= 200


@pytest.mark.parametrize("case", ["temp", "top_k", "preset", "min_p", "penalties"])
def test_vocabulary_sized_rows_against_the_oracle(llb, oracle, dev, case):
    from oracle import bindings
    P = bindings.SmpParams.make
    op = {"temp": P(temp=0.9, seed=21), "top_k": P(temp=0.8, top_k=40, seed=22), "preset": P(temp=0.7, top_k=20, top_p=0.8, presence=1.5, seed=23),
          "min_p": P(temp=1.2, min_p=0.02, seed=24), "penalties": P(temp=1.0, top_k=256, top_p=0.98, repeat_penalty=1.1, frequency=0.3, repeat_last_n=200, seed=25)}[case]
    rng = np.random.default_rng(hash(case) % 1000)
    T, V = 8, 151936
    lg = (rng.standard_normal((T, V)) * 2.5).astype(np.float32)
    lg[0, rng.integers(0, V, 5)] = lg[0].max()                   # ties at the top
    hists = [rng.integers(0, V, 300).astype(np.int32) for _ in range(T)]
    for r in range(T):
        hists[r][-5:] = np.argsort(-lg[r])[:5]                  # likely tokens inside the window
    order = [np.argsort(-lg[r]) for r in range(T)]
    drafts = [int(order[r][0]) if r % 3 == 0 else int(order[r][r % 4]) if r % 3 == 1 else -1 for r in range(T)]
    pos = [int(rng.integers(1, 1 << 24)) for _ in range(T)]
    n = op.repeat_last_n
    buf = dev(lg.nbytes).write(lg)
    tok, acc, val = llb.smp_rows(_dev_params(llb, op), buf.ptr, T, V, drafts, pos, [h[-n:] for h in hists])
    hits = 0
    for r in range(T):
        t, a, margin = bindings.smp_row(op, lg[r], hists[r], drafts[r], pos[r])
        if (tok[r], acc[r]) != (t, a):
            assert margin < 1e-6, (case, r, int(tok[r]), int(acc[r]), t, a, margin)
        else:
            hits += 1
    assert hits >= T - 1


def test_what_has_no_device_path_is_refused_by_name(llb, dev):
    lg = np.zeros((1, 64), np.float32)
    buf = dev(lg.nbytes).write(lg)
    for kw, word in ((dict(temp=1.0, top_p=0.9), "top_p < 1 needs top_k"), (dict(temp=1.0, top_k=300), "top_k 300"),
                     (dict(temp=1.0, presence=1.0, repeat_last_n=1000), "penalty window")):
        with pytest.raises(llb.LlbError, match=word):
            llb.smp_rows(llb.SmpParams.make(**kw), buf.ptr, 1, 64, [-1], [1], [[]])


@pytest.mark.parametrize("streams", [1, 2])
def test_sampled_cycles_replayed_on_the_devices_own_logits(pkg, packs, oracle, llb, streams):
    """The engine with top_k 20, top_p 0.9, a presence penalty and the MTP drafter (a low temperature: the tiny model's
    logits are nearly flat, and some drafts should be accepted): after every cycle the rows' logits are read back and the oracle's sampler, given the same logits, history,
    drafts and positions, must emit the tokens the device emitted and stop serving where the device stopped.  Over the run
    some drafts are accepted and some rejected."""
    from oracle import bindings
    cfg = packs.cfg_tiny()
    pack = packs.build_pack(cfg)
    mtp = packs.aux1_bytes(packs.build_mtp(pack))
    op = bindings.SmpParams.make(temp=0.03, top_k=20, top_p=0.9, presence=0.05, seed=99)
    k = 3
    eng = pkg.llb.SpecEngine(pack, mtp, k=k, max_ctx=160, streams=streams)
    try:
        eng.set_sampler(_dev_params(pkg.llb, op))
        prompts = [packs.synth_prompt(60 + b, 8 + 3 * b, cfg.vocab_size) for b in range(streams)]
        hist = [list(int(t) for t in p) for p in prompts]
        for b, p in enumerate(prompts):
            (eng.prefill_stream(b, p) if streams > 1 else eng.prefill(p))
        acc = rej = 0
        for cyc in range(24):
            p0 = [eng.position_stream(b) for b in range(streams)]
            outs = eng.cycle_streams() if streams > 1 else [eng.cycle()]
            for b in range(streams):
                ids, top2 = outs[b]
                # the cycle's inputs: the committed token, then the drafts the device verified (the result record has them)
                rec = eng.last_record(b)
                T, tin = rec["T"], rec["tin"]
                assert rec["p0"] == p0[b] and tin[0] == hist[b][-1] and len(ids) == rec["served"]
                h = list(hist[b])
                for r in range(T):
                    lg = eng.read_logits(b * (k + 1) + r)
                    draft = tin[r + 1] if r + 1 < T else -1
                    t, a, margin = bindings.smp_row(op, lg, h, draft, p0[b] + r + 1)
                    assert t == rec["ids"][r] or margin < 1e-6, (cyc, b, r, t, rec["ids"][r], margin)
                    assert np.float32(lg[rec["ids"][r]]).view(np.uint32) == rec["top2"][r][1]
                    if r + 1 < T and rec["ids"][r] != tin[r + 1]:
                        assert rec["served"] == r + 1
                        rej += 1
                        break
                    acc += r + 1 < T
                    if r + 1 < T:
                        h.append(tin[r + 1])
                hist[b] += [int(t) for t in ids]
        assert eng.sampler_errors() == 0
        assert acc > 0 and rej > 0, (acc, rej)
    finally:
        eng.close()


def test_greedy_parameters_leave_the_cycle_greedy(pkg, packs, oracle, llb):
    cfg = packs.cfg_tiny()
    pack = packs.build_pack(cfg)
    mtp = packs.aux1_bytes(packs.build_mtp(pack))
    prompt = packs.synth_prompt(1, 9, cfg.vocab_size)
    out = []
    for setit in (False, True):
        eng = pkg.llb.SpecEngine(pack, mtp, k=3, max_ctx=96)
        try:
            if setit:
                eng.set_sampler(pkg.llb.SmpParams.make(temp=0.0, top_k=40, top_p=0.5))   # stages that never move the argmax
            eng.prefill(prompt)
            out.append(eng.generate(24))
        finally:
            eng.close()
    assert np.array_equal(out[0][0], out[1][0]) and np.array_equal(out[0][1], out[1][1])
