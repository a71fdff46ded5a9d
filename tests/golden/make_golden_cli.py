#!/usr/bin/env python
"""Writes tests/golden/engine_cli_tiny.json: what the REFERENCE's own engine process prints for a tiny synthetic pack --
its command line, stdout and stderr -- so that the protocol of eureka-engine_b200/llb-engine-b200 is pinned against the
real thing.  The process is oracle/_ref/qwen35_ref: the reference's tools/qwen35_engine.c with its own main(), compiled
where it lies by `make -C oracle ref REF=<reference tree>`.

    python tests/golden/make_golden_cli.py
"""
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def main():
    import __graft_entry__ as graft
    packs = graft.load_package().packs
    exe = os.path.join(ROOT, "oracle", "_ref", "qwen35_ref")
    cfg = packs.cfg_tiny()
    pack = packs.build_pack(cfg)
    prompt = [int(t) for t in packs.synth_prompt(1, 9, cfg.vocab_size)]
    steps = 12
    with tempfile.TemporaryDirectory() as d:
        pack.write(d)
        args = [str(t) for t in prompt] + ["--steps", str(steps)]
        r = subprocess.run([exe, d] + args, capture_output=True, text=True, check=True)
    out = {"args": args, "stdout": r.stdout.splitlines(), "stderr": r.stderr.splitlines(), "cfg": "packs.cfg_tiny()", "prompt_seed": 1}
    with open(os.path.join(HERE, "engine_cli_tiny.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("\n".join(out["stdout"][:4]), "...", "\n".join(out["stderr"][:4]))


if __name__ == "__main__":
    main()
