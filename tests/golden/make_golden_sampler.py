"""Golden vectors of the sampler: rows of logits, parameters, penalty windows, drafts and positions with the tokens the
REFERENCE's own sampler pack returns for them (host/llb_sampler.c, compiled where it lies into oracle/_ref/libllbsmp.so by
`make -C oracle ref REF=<reference tree>`): llb_smp_verify for rows with a draft, llb_smp_sample for rows without.

    python tests/golden/make_golden_sampler.py        ->  tests/golden/sampler_vectors.npz

The cases cover every stage of the chain alone and combined (temperature, top_k, top_p, min_p, repeat / presence / frequency
penalties over a window, logit bias, greedy with bias), drafts that are likely and unlikely, and logits with exact ties.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import bindings  # noqa: E402


def cases():
    P = bindings.SmpParams.make
    yield "temp", P(temp=0.8, seed=1)
    yield "temp_hot", P(temp=1.7, seed=2)
    yield "top_k", P(temp=0.9, top_k=20, seed=3)
    yield "top_k_1", P(temp=1.0, top_k=1, seed=4)
    yield "top_k_p", P(temp=0.7, top_k=20, top_p=0.8, seed=5)
    yield "preset_thinking", P(temp=1.0, top_k=20, top_p=0.95, presence=1.5, seed=6)
    yield "top_k_p_minp", P(temp=0.6, top_k=40, top_p=0.9, min_p=0.05, min_keep=2, seed=7)
    yield "min_p", P(temp=1.1, min_p=0.1, seed=8)
    yield "penalties", P(temp=0.9, top_k=50, repeat_penalty=1.3, frequency=0.2, presence=0.4, repeat_last_n=16, seed=9)
    yield "bias", P(temp=0.8, top_k=10, seed=10, bias=((3, 4.0), (17, -100.0), (3, 1.0)))
    yield "greedy_bias", P(temp=0.0, seed=11, bias=((5, 50.0),))
    yield "greedy_pen", P(temp=0.0, repeat_penalty=2.0, presence=5.0, repeat_last_n=8, seed=12)
    yield "top_k_256", P(temp=1.0, top_k=256, top_p=0.99, seed=13)


def main():
    rng = np.random.default_rng(2024)
    V = 512
    out = {}
    names = []
    for name, p in cases():
        rows = []
        for r in range(16):
            scale = (0.5, 2.0, 6.0)[r % 3]
            lg = (rng.standard_normal(V) * scale).astype(np.float32)
            if r % 5 == 0:
                lg[rng.integers(0, V, 8)] = lg.max()          # exact ties at the top
            hist = rng.integers(0, V, int(rng.integers(0, 40))).astype(np.int32)
            if r % 4 == 0 and len(hist):
                hist[-3:] = int(np.argmax(lg))                  # the likely token repeated in the window
            order = np.argsort(-lg)
            draft = int(order[0]) if r % 3 == 0 else int(order[rng.integers(0, 6)]) if r % 3 == 1 else -1
            pos = int(rng.integers(1, 5000))
            tok, acc = bindings.ref_smp_row(p, lg, hist, draft, pos)
            rows.append((lg, hist, draft, pos, tok, acc))
        names.append(name)
        out[name + ".params"] = np.frombuffer(bytes(p), dtype=np.uint8).copy()
        out[name + ".logits"] = np.stack([r[0] for r in rows])
        out[name + ".hist_len"] = np.array([len(r[1]) for r in rows], np.int32)
        out[name + ".hist"] = np.concatenate([r[1] for r in rows]) if any(len(r[1]) for r in rows) else np.zeros(0, np.int32)
        out[name + ".draft"] = np.array([r[2] for r in rows], np.int32)
        out[name + ".pos"] = np.array([r[3] for r in rows], np.int64)
        out[name + ".tok"] = np.array([r[4] for r in rows], np.int32)
        out[name + ".acc"] = np.array([r[5] for r in rows], np.int32)
    out["names"] = np.array(names)
    path = os.path.join(ROOT, "tests", "golden", "sampler_vectors.npz")
    np.savez_compressed(path, **out)
    acc = sum(int(out[n + ".acc"].sum()) for n in names)
    print(f"sampler_vectors.npz: {len(names)} parameter sets x 16 rows, {acc} accepted drafts, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
