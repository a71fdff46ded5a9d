#!/usr/bin/env python
"""Writes tests/golden/long_context.npz from the REFERENCE CPU engine (tools/qwen35_engine.c built as oracle/_ref by
`make -C oracle ref REF=<reference tree>`): greedy ids, top-2 logit bits and the logit row after the prompt for a
model with the long-context configuration's attention shape (16 Q / 4 KV heads of 256, Q8_0) at a context beyond 8192
positions.  The reference's own command line stops at 8192 prompt ids (tools/qwen35_engine.c:820,940); the engine's
forward_token has no such limit and is driven directly here, as oracle/bindings.RefTwin does for every fixture.

    python tests/golden/make_golden_long.py [--threads N]

The pack is rebuilt by the test from its seed on the CPU (packs.cfg_long()); the fixture records the sha256 of the
bytes it was made from and how long the reference took.
"""
import argparse
import hashlib
import os
import sys
import tempfile
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

N_PROMPT, STEPS = 8219, 16     # (8219 + 6) / 37 context slices: 223 positions a slice, rounded up to 224


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--threads", type=int, default=0)
    args = ap.parse_args()
    import __graft_entry__ as graft
    packs = graft.load_package().packs
    from oracle.bindings import RefTwin
    cfg = packs.cfg_long()
    pack = packs.build_pack(cfg)
    host = pack.data.numpy()
    prompt = packs.synth_prompt(9, N_PROMPT, cfg.vocab_size)
    t0 = time.time()
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "index.tsv"), "w") as f:
            f.write(pack.index_text())
        ref = RefTwin(d, cap=N_PROMPT + STEPS + 8, pack=host, threads=args.threads)
        for t, tok in enumerate(prompt):
            ref.forward(int(tok), t)
        row = ref.logits()
        ids = np.zeros(STEPS, np.int32)
        t2 = np.zeros((STEPS, 4), np.uint32)
        for s in range(STEPS):
            lg = ref.logits()
            (i1, i2), (v1, v2) = ref.top2()
            ids[s] = i1
            t2[s] = [i1, np.float32(v1).view(np.uint32), i2, np.float32(v2).view(np.uint32)]
            ref.forward(i1, N_PROMPT + s)
        k_last = np.ctypeslib.as_array(ref.L.q35ref_state_k(3, N_PROMPT - 1), shape=(cfg.n_kv_heads * cfg.head_dim,)).copy()
    secs = time.time() - t0
    np.savez_compressed(os.path.join(HERE, "long_context.npz"), ids=ids, top2=t2, logits_after_prompt=row, k_last_prompt_row=k_last,
                        n_prompt=N_PROMPT, prompt_seed=9, pack_sha256=hashlib.sha256(host.tobytes()).hexdigest(),
                        reference_seconds=secs, threads=args.threads or os.cpu_count())
    print(f"long_context.npz: {STEPS} ids after {N_PROMPT} prompt tokens, reference took {secs:.0f} s")


if __name__ == "__main__":
    main()
