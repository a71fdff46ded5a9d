"""The engine process (eureka-engine_b200/llb-engine-b200) speaks the protocol of the reference's engines: argv ids and
--steps, LLB_SPEC / LLB_MTP in the environment, stdout one id per line then wall_ms and tok_s, stderr `logits`, `step`
and `spec:` lines (tools/qwen35_engine.c:15-17,975-1013; host/llb_host.c:1513-1523).  The golden is what the reference's
own process printed for the same tiny pack (tests/golden/make_golden_cli.py)."""
import json
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "eureka-engine_b200", "llb-engine-b200")
GOLD = json.load(open(os.path.join(ROOT, "tests", "golden", "engine_cli_tiny.json")))
RE_LOGITS = re.compile(r"^logits (\d+) (\d+) (\d+) (\d+) (\d+)$")
RE_STEP = re.compile(r"^step (\d+) (\d+)$")
RE_SPEC = re.compile(r"^spec: (mtp|lookup) k (\d+) cycles (\d+) rows (\d+) served (\d+) \((\d+\.\d{3}) a cycle\); accepted/drafted by position:((?: \d+/\d+)+)$")


def _parse(stdout, stderr):
    ids = [int(l) for l in stdout if re.fullmatch(r"-?\d+", l)]
    tail = [l for l in stdout if not re.fullmatch(r"-?\d+", l)]
    logits = [tuple(int(g) for g in RE_LOGITS.match(l).groups()) for l in stderr if l.startswith("logits ")]
    steps = [tuple(int(g) for g in RE_STEP.match(l).groups()) for l in stderr if l.startswith("step ")]
    return ids, tail, logits, steps


def test_golden_is_the_reference_protocol():
    """CPU: the committed golden parses with the expressions the GPU test applies to our process."""
    ids, tail, logits, steps = _parse(GOLD["stdout"], GOLD["stderr"])
    n_prompt = len(GOLD["args"]) - 2
    assert len(ids) == 12 and re.fullmatch(r"wall_ms \d+", tail[0]) and re.fullmatch(r"tok_s \d+\.\d{4}", tail[1])
    assert [l[0] for l in logits] == list(range(n_prompt - 1, n_prompt + 11))      # one row per position from the last prompt token
    assert [l[1] for l in logits] == ids                                            # id1 of a row is the id printed next
    assert [s[0] for s in steps] == list(range(n_prompt, n_prompt + 11))


def test_usage_and_refusals_need_no_gpu():
    if not os.path.exists(EXE):
        import __graft_entry__ as graft
        graft.load_package().llb.build()
    r = subprocess.run([EXE], capture_output=True, text=True)
    assert r.returncode == 2 and "usage:" in r.stderr and "LLB_SPEC" in r.stderr
    env = dict(os.environ, LLB_SAMPLE="temp=0.7,logprobs=3")
    r = subprocess.run([EXE, "/nonexistent", "1"], capture_output=True, text=True, env=env)
    assert r.returncode == 2 and "no key 'logprobs'" in r.stderr
    env = dict(os.environ, LLB_SAMPLE="preset=nonsense")
    r = subprocess.run([EXE, "/nonexistent", "1"], capture_output=True, text=True, env=env)
    assert r.returncode == 2 and "unknown preset" in r.stderr
    r = subprocess.run([EXE, "/nonexistent", "1", "--bogus"], capture_output=True, text=True)
    assert r.returncode == 2 and "unknown option" in r.stderr
    env = dict(os.environ, LLB_SPEC="9")
    r = subprocess.run([EXE, "/nonexistent", "1"], capture_output=True, text=True, env=env)
    assert r.returncode == 2 and "0..7" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["plain", "mtp", "lookup"])
def test_engine_process_matches_the_reference_process(packs, llb, tmp_path, mode):
    """The same pack, prompt and --steps as the golden, launched the way `llb run [--spec]` launches its engine
    (tools/llb/golden/dryrun-27b-fast-spec.txt): ids equal, logits lines at the same positions with the same ids and
    logit values within the path's tolerance, step lines at the same positions, and the spec: summary when LLB_SPEC is set."""
    cfg = packs.cfg_tiny()
    pack = packs.build_pack(cfg)
    pack.write(str(tmp_path))
    env = dict(os.environ)
    if mode != "plain":
        env["LLB_SPEC"] = "3"
    if mode == "mtp":
        (tmp_path / "mtp.bin").write_bytes(packs.aux1_bytes(packs.build_mtp(pack)))
        env["LLB_MTP"] = str(tmp_path / "mtp.bin")
    r = subprocess.run([EXE, "--gpu", "40GB", "--threads", "4", "--", str(tmp_path)] + GOLD["args"], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr
    ids, tail, logits, steps = _parse(r.stdout.splitlines(), r.stderr.splitlines())
    gids, gtail, glogits, gsteps = _parse(GOLD["stdout"], GOLD["stderr"])
    assert ids == gids
    assert [re.sub(r"[\d.]+", "N", t) for t in tail] == [re.sub(r"[\d.]+", "N", t) for t in gtail]
    assert [(l[0], l[1], l[3]) for l in logits] == [(l[0], l[1], l[3]) for l in glogits]
    f = lambda u: np.array(u, dtype=np.uint32).view(np.float32)
    for col in (2, 4):
        a, b = f([l[col] for l in logits]), f([l[col] for l in glogits])
        assert np.all(np.abs(a - b) <= 2e-2 + 1e-2 * np.abs(b))
    assert [s[0] for s in steps] == [s[0] for s in gsteps]
    spec = [l for l in r.stderr.splitlines() if l.startswith("spec:")]
    if mode == "plain":
        assert not spec
    else:
        m = RE_SPEC.match(spec[0])
        assert m and m.group(1) == mode and int(m.group(2)) == 3 and len(m.group(7).split()) == 3
        assert int(m.group(5)) >= len(ids) - 1 and int(m.group(3)) >= 1


@pytest.mark.gpu
def test_engine_process_samples_reproducibly(packs, llb, tmp_path):
    """LLB_SAMPLE as the reference takes it (host/llb_host.c:1376-1380): the same seed gives the same stream, with or
    without speculation (the verify rule is lossless per draw only in distribution, so the two need not be equal to each
    other), another seed gives another stream, and a greedy spec leaves the greedy ids."""
    cfg = packs.cfg_tiny()
    pack = packs.build_pack(cfg)
    pack.write(str(tmp_path))
    (tmp_path / "mtp.bin").write_bytes(packs.aux1_bytes(packs.build_mtp(pack)))

    def run(sample, spec):
        env = dict(os.environ)
        if sample:
            env["LLB_SAMPLE"] = sample
        if spec:
            env["LLB_SPEC"], env["LLB_MTP"] = "3", str(tmp_path / "mtp.bin")
        r = subprocess.run([EXE, str(tmp_path)] + GOLD["args"][:-2] + ["--steps", "24"], capture_output=True, text=True, env=env, timeout=300)
        assert r.returncode == 0, r.stderr
        return _parse(r.stdout.splitlines(), r.stderr.splitlines())[0]

    greedy = run(None, True)
    assert run("temp=0,top_k=5", True) == greedy
    a = run("temp=1.0,top_k=40,top_p=0.95,seed=7", True)
    assert a == run("temp=1.0,top_k=40,top_p=0.95,seed=7", True) and a != greedy
    assert a != run("temp=1.0,top_k=40,top_p=0.95,seed=8", True)
    b = run("preset=qwen_non_thinking,seed=7", False)
    assert b == run("preset=qwen_non_thinking,seed=7", False) and len(b) == 24
