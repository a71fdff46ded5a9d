#!/usr/bin/env python
"""Writes the golden fixtures of tests/golden/ from the REFERENCE itself.

Run in a checkout that has the reference tree (--ref REFERENCE_DIR) and after
`make -C oracle ref REF=<reference>`:

    python tests/golden/make_golden.py [--ref REFERENCE_DIR] [--skip-c0]

Sources of truth used here (nothing from this repository's CUDA path or C restatement):
  * the reference's numpy dequantisers tools/q4k.py, tools/q5k.py, tools/q6k.py (dequant_rows) and the
    Q8_0 rule of tools/q8_pack.py:13-18, imported from the reference tree;
  * the reference CPU engine tools/qwen35_engine.c compiled from its own sources (oracle/_ref), stepped
    through oracle/bindings.RefTwin: greedy ids and top-2 logit bits of synthetic packs.
The packs themselves are rebuilt by the tests from their seeds (eureka-engine_b200/packs.py); each
fixture records the sha256 of the pack bytes it was made from.
"""
import argparse
import hashlib
import json
import os
import sys
import tempfile
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def random_blocks(fmt, rows, cols, seed):
    """Random but valid blocks: random bytes everywhere, f16 scale fields forced finite."""
    rng = np.random.default_rng(seed)
    bb = {"Q4_K": 144, "Q5_K": 176, "Q6_K": 210}[fmt]
    raw = rng.integers(0, 256, (rows, cols // 256, bb), dtype=np.uint8)
    d = (rng.standard_normal((rows, cols // 256, 2)) * 0.01).astype(np.float16)
    if fmt == "Q6_K":
        raw[:, :, 208:210] = d[:, :, :1].view(np.uint8)
    else:
        raw[:, :, 0:4] = d.view(np.uint8).reshape(rows, cols // 256, 4)
    return raw.reshape(rows, -1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("LLB_REFERENCE_ROOT"), required=not os.environ.get("LLB_REFERENCE_ROOT"),
                    help="the reference tree (or LLB_REFERENCE_ROOT)")
    ap.add_argument("--skip-c0", action="store_true")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.ref, "tools"))
    import q4k, q5k, q6k  # the reference's own numpy decoders
    import __graft_entry__ as graft
    packs = graft.load_package().packs
    from oracle.bindings import RefTwin

    # ---- dequantisation vectors from the reference's numpy modules ----------------------------
    rows, cols = 4, 512
    deq = {}
    for name, mod in (("Q4_K", q4k), ("Q5_K", q5k), ("Q6_K", q6k)):
        raw = random_blocks(name, rows, cols, seed=100 + packs.FMT[name])
        out = np.asarray(mod.dequant_rows(raw.reshape(-1), rows, cols), dtype=np.float32).reshape(rows, cols)
        deq[name] = {"raw": raw, "deq": out}
    rng = np.random.default_rng(101)
    q = rng.integers(-128, 128, (rows, cols), dtype=np.int8)
    d = (rng.standard_normal((rows, cols // 32)) * 0.01).astype(np.float16)
    raw8 = np.concatenate([q.view(np.uint8), d.view(np.uint8).reshape(rows, cols // 16)], axis=1)
    deq["Q8_0"] = {"raw": raw8, "deq": (q.astype(np.float32) * np.repeat(d.astype(np.float32), 32, axis=1))}
    np.savez_compressed(os.path.join(HERE, "dequant_vectors.npz"), **{f"{k}_{f}": v[f] for k, v in deq.items() for f in ("raw", "deq")})

    # ---- greedy ids / top-2 bits from the reference CPU engine ---------------------------------
    cases = {
        "tiny_q8_0": (packs.cfg_tiny(), 9, 24, 1),
        "tiny_q4_k_m": (packs.cfg_tiny(quant="q4_k_m", n_layers=8, tied_head=False, seed=12), 6, 20, 1),
        "tiny_q4_k_s": (packs.cfg_tiny(quant="q4_k_s", n_layers=8, tied_head=False, seed=12), 6, 20, 1),
    }
    if not args.skip_c0:
        cases["c0_0.8b_q8_0"] = (packs.cfg_c0(), 64, 128, 1)
    out = {}
    for name, (cfg, n_prompt, steps, pseed) in cases.items():
        t0 = time.time()
        pack = packs.build_pack(cfg)
        prompt = packs.synth_prompt(pseed, n_prompt, cfg.vocab_size)
        with tempfile.TemporaryDirectory() as dd:
            with open(os.path.join(dd, "index.tsv"), "w") as f:
                f.write(pack.index_text())
            # one reference model per process: the engine keeps its state in globals
            import subprocess
            pack.data.numpy().tofile(os.path.join(dd, "pack.bin"))
            code = ("import sys, json; sys.path.insert(0, %r); from oracle.bindings import RefTwin; import numpy as np;"
                    "r = RefTwin(%r, cap=%d); ids, t2 = r.greedy(%r, %d); print(json.dumps({'ids': ids.tolist(), 'top2': t2.tolist()}))"
                    % (ROOT, dd, n_prompt + steps + 4, [int(v) for v in prompt], steps))
            res = json.loads(subprocess.run([sys.executable, "-c", code], check=True, capture_output=True, text=True).stdout)
        out[name] = {"cfg": {k: getattr(cfg, k) for k in ("n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim", "d_ff", "vocab_size",
                                                          "ssm_heads", "ssm_groups", "tied_head", "quant", "seed")},
                     "prompt_seed": pseed, "n_prompt": n_prompt, "prompt": [int(v) for v in prompt],
                     "pack_sha256": hashlib.sha256(pack.data.numpy().tobytes()).hexdigest(),
                     "ids": res["ids"], "top2": res["top2"]}
        print(name, "done in %.1f s" % (time.time() - t0), flush=True)
    with open(os.path.join(HERE, "reference_greedy.json"), "w") as f:
        json.dump(out, f)


if __name__ == "__main__":
    main()
