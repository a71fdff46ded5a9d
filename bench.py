#!/usr/bin/env python
"""Benchmark of the speculative-decoding path on the 27B-shape Q4_K_M model, MTP k = 3.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is one speculative cycle (MTP drafts -> 4-row verify -> accept -> commit) of one request
stream on one GPU.  The synthetic 27B-shape pack (seed 3) is drawn and quantised on the GPU, the
3011-token prompt is fed through the engine, then W warm-up and K timed cycles run.

  value     emitted tokens / s over all GPUs, cycles enqueued back to back, timed with CUDA events
            on the library's stream (inputs resident in HBM)
  e2e       the same through the reference-shaped per-token call llb_spec_pass(pos, tok) -> y with
            host buffers: (pos, tok) crosses to the device and the result record comes back every cycle
  roofline  the largest launch (FFN gate|up GEMM), event-timed over cold weights, against the
            measured HBM copy peak; verify_step = weight + KV bytes of one verify pass / its time
  cpu_baseline  the reference CPU engine (oracle/_ref, built from the reference's own sources) on the
            same pack on this box's host cores, a bounded sample

With N > 1 (torchrun) every rank runs its own stream on its own replica: no collective on the data
path, weak scaling.  `--impl reference` times the reference CPU engine alone (rank 0 only).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# DRAM bytes one gate|up launch moved under ncu (102.1 MB read + 4.3 MB written; algorithmic 100.9 MB)
GEMM_DRAM_TRAFFIC = 106.4e6
METRIC = "spec-decode tok/s per B200, 27B-shape Q4_K_M MTP k=3; verify-step HBM GB/s"
WORKLOAD = "config 2: 27B-shape hybrid (d 5120, 64 layers, f 17408, V 151936), Q4_K_M, batch 1, MTP k=3 greedy, prompt 3011"
PROMPT, GEN_CAP, K_DRAFT = 3011, 1200, 3
DRAFT_VOCAB = 40960


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s)"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
        sm = [float(r[1]) for r in self.rows if len(r) >= 8 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 8 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 8 and r[4 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def verify_bytes(pack, pos: int, T: int) -> float:
    """Algorithmic bytes of one verify pass: every trunk matrix and the head once, T embedding rows,
    and the K/V rows of positions 0 .. pos+T-1 of every full-attention layer (f32)."""
    from __graft_entry__ import load_package
    packs = load_package().packs
    c = pack.cfg
    b = 0.0
    for e in pack.entries:
        if e.name == "token_embd.weight":
            b += T * packs.row_bytes(e.ty, e.cols)
        elif e.name == "output.weight" or (e.name.startswith("blk.") and e.rows > 1 and e.ty != "F32"):
            b += e.nbytes
    n_full = sum(1 for i in range(c.n_layers) if c.is_full(i))
    b += n_full * 2.0 * (pos + T) * c.n_kv_heads * c.head_dim * 4
    return b


def build_model(device, layers=None):
    from __graft_entry__ import load_package
    packs = load_package().packs
    cfg = packs.cfg_c2()
    pack = packs.build_pack(cfg, device=device, layers=layers)
    # the drafter's head is the 40960-row draft-vocabulary slice of the reference's 27B drafter pack (tools/mtp27/mtp_pack.py:14-30:
    # 172 MB a drafter pass instead of the whole head's 638 MB); on this synthetic model the slice is the first 40960 ids
    mtp = packs.aux1_bytes(packs.build_mtp(pack, draft_vocab=DRAFT_VOCAB))
    prompt = packs.synth_prompt(3, PROMPT, cfg.vocab_size)
    return packs, pack, mtp, prompt


def cpu_reference_run(pack, prompt, n_prompt: int, n_gen: int, threads: int):
    """The reference CPU engine on the same pack: teacher-forces `n_prompt` prompt tokens, then decodes
    `n_gen` tokens greedily.  Returns (tok/s over the generated tokens, ids, seconds)."""
    from oracle.bindings import RefTwin
    host = pack.data.cpu().numpy()
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "index.tsv"), "w") as f:
            f.write(pack.index_text())
        ref = RefTwin(d, cap=n_prompt + n_gen + 4, pack=host, threads=threads)
        for t in range(n_prompt):
            ref.forward(int(prompt[t]), t)
        ids = []
        t0 = time.perf_counter()
        for s in range(n_gen):
            ref.logits()
            (i1, _), _ = ref.top2()
            ids.append(i1)
            ref.forward(i1, n_prompt + s)
        dt = time.perf_counter() - t0
    return n_gen / dt, ids, dt


def run_reference(args, rank):
    if rank != 0:
        return
    import torch
    cores = os.cpu_count() or 1
    dev = "cuda:0" if torch.cuda.is_available() else "cpu"
    packs, pack, mtp, prompt = build_model(dev)
    n_prompt = 4
    tps, ids, dt = cpu_reference_run(pack, prompt, n_prompt, args.steps + args.warmup, cores)
    # warm-up tokens are part of the loop above; report the rate over all of them
    line = {"metric": METRIC, "value": tps, "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1000.0 / tps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "impl": "reference",
            "config": {"workload": WORKLOAD, "note": "reference CPU engine (tools/qwen35_engine.c), plain greedy: it has no speculative path; "
                       "a step is one decoded token at a context of %d" % n_prompt},
            "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": cores, "kind": "reference",
                             "sample": f"full-depth pack, {n_prompt} prompt tokens then {args.steps + args.warmup} greedy tokens"},
            "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_tp(args, rank, world, local):
    """One request stream over all N GPUs, tensor parallel (strong scaling): every rank holds its share of the
    projections and the passes exchange two all-reduces a layer.  The line's value is that one stream's tok/s."""
    import torch
    import torch.distributed as dist
    import __graft_entry__ as graft
    pkg = graft.load_package()
    llb = pkg.llb
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    llb.init(local)
    llb.tp_init(device=f"cuda:{local}", peer=not args.nccl_allreduce)
    packs, pack, mtp, prompt = build_model(f"cuda:{local}", layers=args.layers or None)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    eng = llb.SpecEngine(pack, mtp, k=K_DRAFT, max_ctx=PROMPT + GEN_CAP + 64, tp=world)
    del pack
    torch.cuda.empty_cache()
    t_pre = time.time()
    eng.prefill(prompt)
    torch.cuda.synchronize()
    t_pre = time.time() - t_pre
    steps, warm = args.steps, max(args.warmup, 3)
    st = torch.cuda.ExternalStream(llb.lib().llb_b200_stream())
    sampler = ClockSampler(local)
    sampler.start()
    eng.run_cycles(warm)
    dist.barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(st)
    _, toks = eng.run_cycles(steps)
    e1.record(st)
    dist.barrier(); torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    ver_ms = eng.time_verify(10)
    prof = eng.profile_verify()
    t = torch.tensor([ms, ver_ms], dtype=torch.float64, device=f"cuda:{local}")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ver_ms = t.tolist()
    if rank == 0:
        total = sum(v[1] for v in prof.values())
        ar = prof.get("all-reduce", (0, 0.0))
        line = {"metric": METRIC, "value": toks / (ms / 1000.0), "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warm,
                "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": WORKLOAD, "streams": 1, "parallelism": f"tp{world}", "layers": args.layers or 64,
                           "l2": "inputs larger than L2", "tokens_per_cycle": toks / steps, "prefill_s": round(t_pre, 2)},
                "clocks": clocks, "gpu_launches": eng.graph_nodes(0) * steps,
                "verify_step": {"ms": ver_ms, "kernels": eng.graph_nodes(2)},
                "all_reduce": {"per_pass": ar[0], "eager_us_per_pass": ar[1], "share_of_eager_pass": ar[1] / total if total else None,
                               "kind": "NCCL" if args.nccl_allreduce else "one-shot kernel over peer memory (K-slice sum, peer stores, flag wait, rank-order sum)",
                               "what": "all-reduce of a [4, 5120] f32 tile after attn_output / ssm_out and after ffn_down; eager per-op event timing"},
                "wait_errors": llb.lib().llb_b200_wait_errors()}
        print(json.dumps(line), flush=True)
    eng.close()
    dist.destroy_process_group()


STREAM_CASES = {
    # config: (builder, workload words, prompt, default k, default streams per GPU, metric)
    2: ("cfg_c2", "config 2: 27B-shape hybrid (d 5120, 64 layers, f 17408, V 151936), Q4_K_M, MTP k=%d greedy, prompt %d, %d streams per GPU",
        3011, 3, 4),
    3: ("cfg_c3", "config 3: 35B-A3B-shape MoE hybrid (d 2048, 40 layers, 256 experts top 8 + shared, V 151936), Q4_K_S, prompt-lookup k=%d "
        "greedy, prompt %d, %d streams per GPU", 512, 3, 8),
    4: ("cfg_c4", "config 4: 9B-shape hybrid (d 4096, 32 layers, f 12288, V 151936), Q8_0, MTP k=%d greedy, prompt %d, %d streams per GPU",
        32768, 3, 4),
}


def streams_bytes(packs, pack, positions, rows: int) -> float:
    """Algorithmic bytes of one verify pass over several streams: every dense matrix and the head ONCE, one embedding row
    per row of the pass, the K/V rows of every stream's context, and for routed experts one expert block per (row, slot)."""
    c = pack.cfg
    b = 0.0
    ne = getattr(c, "n_experts", 0) or 0
    for e in pack.entries:
        if e.name == "token_embd.weight":
            b += rows * packs.row_bytes(e.ty, e.cols)
        elif "_exps." in e.name:
            b += e.nbytes / ne * rows * c.n_experts_used
        elif e.name == "output.weight" or (e.name.startswith("blk.") and e.rows > 1 and e.ty != "F32"):
            b += e.nbytes
    n_full = sum(1 for i in range(c.n_layers) if c.is_full(i))
    for p in positions:
        b += n_full * 2.0 * p * c.n_kv_heads * c.head_dim * 4
    return b


def run_streams(args, rank, world, local):
    """Several streams per GPU sharing one weight read (llb_spec_open_streams), every GPU its own replica and streams
    (weak scaling, no collective).  A step is one cycle of all the GPU's streams; value = tokens of all streams / s."""
    import numpy as np
    import torch
    import __graft_entry__ as graft
    pkg = graft.load_package()
    llb, packs = pkg.llb, pkg.packs
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    llb.init(local)
    builder, words, prompt_len, k_def, b_def = STREAM_CASES[args.config]
    k = args.k if args.k >= 0 else k_def
    B = args.streams if args.streams > 0 else b_def
    n_prompt = args.prompt if args.prompt > 0 else prompt_len
    cfg = getattr(packs, builder)()
    pack = packs.build_pack(cfg, device=f"cuda:{local}", layers=args.layers or None)
    moe = bool(getattr(cfg, "n_experts", 0))
    mtp = None if (moe or k == 0) else packs.aux1_bytes(packs.build_mtp(pack, draft_vocab=DRAFT_VOCAB))   # the drafter's head: the draft-vocabulary slice
    steps, warm = args.steps, max(args.warmup, 3)
    max_ctx = n_prompt + (steps + warm + 8) * (k + 1) + 64
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    # a pass takes 16 rows: more streams than that go into sibling engines on the same weights, whose passes run in turn
    per_eng = max(1, 16 // (k + 1))
    E = -(-B // per_eng)
    if B % E:
        raise SystemExit(f"--streams {B} at k = {k}: {E} engines of at most {per_eng} streams need a stream count they divide")
    Be = B // E
    eng = llb.SpecEngine(pack, mtp, k=k, max_ctx=max_ctx, streams=Be)
    engs = [eng] + [eng.sibling(k=k, max_ctx=max_ctx, streams=Be) for _ in range(E - 1)]
    for e in engs:
        e.set_prefill(True)
    prompts = [packs.synth_prompt(100 * rank + b + 3, n_prompt, cfg.vocab_size) for b in range(B)]
    torch.cuda.synchronize()
    t_pre = time.time()
    for i, e in enumerate(engs):
        e.prefill_streams(prompts[i * Be:(i + 1) * Be])          # the prompts' rows share the prompt passes
    torch.cuda.synchronize()
    t_pre = time.time() - t_pre
    st = torch.cuda.ExternalStream(llb.lib().llb_b200_stream())
    sampler = ClockSampler(local)
    sampler.start()
    for e in engs:
        e.run_cycles_streams(warm)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(st)
    toks = sum(int(e.run_cycles_streams(steps).sum()) for e in engs)
    e1.record(st)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    # end to end: one graph launch and a result record per stream per cycle, the host reading every stream's tokens
    t0 = time.perf_counter()
    n_e2e = 0
    for _ in range(steps):
        for e in engs:
            n_e2e += sum(len(i) for i, _ in e.cycle_streams())
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop()
    ver_ms = sum(e.time_verify(10) for e in engs)          # every engine's pass streams the weights once
    vbytes = sum(streams_bytes(packs, pack, [e.position_stream(b) + k + 1 for b in range(Be)], Be * (k + 1)) for e in engs)
    peak, peak_src = peaks()
    (ms, e2e_s), (toks, n_e2e) = pkg.dp.aggregate([ms, e2e_s], [float(toks), float(n_e2e)], device=f"cuda:{local}")
    if rank == 0:
        acc = [e.stats_stream(b) for e in engs for b in range(Be)]
        line = {
            "metric": "spec-decode tok/s per B200 over all of its streams; verify-step HBM GB/s", "value": toks / (ms / 1000.0), "unit": "tok/s",
            "n_gpus": world, "steps": steps, "warmup": warm, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": words % (k, n_prompt, B), "streams_per_gpu": B, "rows_per_pass": Be * (k + 1), "engines_per_gpu": E, "parallelism": f"stream-dp{world}",
                       "layers": args.layers or cfg.n_layers, "l2": "inputs larger than L2: a cycle streams the whole model",
                       "drafter": "prompt lookup" if mtp is None and k > 0 else ("MTP" if k > 0 else "none"),
                       "tokens_per_cycle_per_stream": toks / (steps * world * B),
                       "accepted_by_position": [round(sum(a["accepted"][j] for a in acc) / max(1, sum(a["drafted"][j] for a in acc)), 4) for j in range(1, k + 1)],
                       "prefill_s": round(t_pre, 3), "prefill_tok_s": round(B * n_prompt / t_pre, 1)},
            "cycle_ms": ms / steps, "tok_s_per_stream": toks / (ms / 1000.0) / (B * world),
            "wait_errors": llb.lib().llb_b200_wait_errors(), "clocks": clocks,
            "e2e": {"value": n_e2e / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 216 * B,
                    "api": "llb_spec_cycle_streams: one graph launch, one result record per stream read back per cycle"},
            "gpu_launches": eng.graph_nodes(0) * steps * E,
            "verify_step": {"bytes": vbytes, "ms": ver_ms, "GBs": vbytes / ver_ms / 1e6, "frac": vbytes / ver_ms / 1e6 / peak, "peak": peak,
                            "peak_source": peak_src, "kernels": eng.graph_nodes(2),
                            "what": "dense weights and head once, KV of every stream, one expert block per (row, slot)"},
        }
        print(json.dumps(line), flush=True)
    for e in engs:
        e.close()
    if world > 1:
        dist.destroy_process_group()


def run_gemm_case(args, local):
    """The isolated verify-step GEMM (configuration 1: the 27B shapes with no model): `--rows` matrices of `--cols` columns in
    format `--fmt` sharing T activation rows, launched over enough copies of the weights that every launch streams from HBM,
    timed with CUDA events on the library's stream.  One JSON line; also the command the ncu summaries under profiles/ run."""
    import numpy as np
    import torch
    import __graft_entry__ as graft
    pkg = graft.load_package()
    llb, packs = pkg.llb, pkg.packs
    torch.cuda.set_device(local)
    llb.init(local)
    L = llb.lib()
    ty, K, T = args.fmt, args.cols, args.t
    fmt = packs.FMT[ty]
    rows = [int(r) for r in args.rows.split(",")]
    g = torch.Generator(device=f"cuda:{local}").manual_seed(2)
    per_copy = sum(r * packs.row_bytes(ty, K) for r in rows)
    copies = max(2, int(400e6 // per_copy) + 1)              # more than the 126 MB L2 between two uses of a copy
    sets = []
    for c in range(copies):
        ws = []
        for r in rows:
            w = torch.randn(r, K, device=f"cuda:{local}", generator=g) * 0.02
            raw = packs.QUANT[ty](w).contiguous()
            p = llb.alloc(L.llb_b200_weight_bytes(fmt, r, K))
            llb.check(L.llb_b200_weight_upload(fmt, r, K, raw.data_ptr(), 1, p), "weight_upload")
            ws.append(p)
            del w, raw
        sets.append(ws)
    x = torch.randn(T, K, device=f"cuda:{local}", generator=g)
    xp = llb.handle(L.llb_b200_xp_new(K, T, 2), "xp_new")
    llb.check(L.llb_b200_xp_set_f32(xp, x.data_ptr()), "xp_set")
    outs = [llb.alloc(T * r * 4 * 16) for r in rows]
    st = torch.cuda.ExternalStream(L.llb_b200_stream())
    for i in range(max(3, args.warmup)):
        llb.gemm(fmt, sets[i % copies], rows, outs, K, xp, args.ksplit)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(st)
    for i in range(args.steps):
        llb.gemm(fmt, sets[i % copies], rows, outs, K, xp, args.ksplit)
    e1.record(st)
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1000.0 / args.steps
    peak, peak_src = peaks()
    nc = 8 if T <= 4 else 16 if T <= 8 else 32
    nbytes = per_copy + nc * K * 2 + sum(T * r * 4 for r in rows)
    print(json.dumps({"case": "gemm", "kernel": f"k_gemm2<{ty}>", "rows": rows, "cols": K, "T": T, "plane_columns": nc, "launches": args.steps,
                      "weight_copies": copies, "us_per_launch": us, "bytes_per_launch": nbytes, "GBs": nbytes / us / 1e3, "frac": nbytes / us / 1e3 / peak,
                      "peak": peak, "peak_source": peak_src, "ksplit": L.llb_b200_gemm_ksplit(fmt, nc, sum((r + 15) // 16 for r in rows), K // 256, L.llb_b200_sm_count()) if args.ksplit == 0 else args.ksplit,
                      "wait_errors": L.llb_b200_wait_errors()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--layers", type=int, default=0, help="truncate the model (debugging only; the number is then not the headline)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--tp", action="store_true", help="one stream over all GPUs, tensor parallel with an NCCL all-reduce per row-split projection (strong scaling)")
    ap.add_argument("--nccl-allreduce", action="store_true", help="with --tp: NCCL all-reduces instead of the library's one-shot kernel over peer memory")
    ap.add_argument("--no-plain", action="store_true", help="skip the plain-decoding (k = 0) leg")
    ap.add_argument("--exact-prefill", action="store_true", help="feed the prompt through the 8-row verify pass instead of the dense tcgen05 path")
    ap.add_argument("--streams", type=int, default=0, help="several streams per GPU sharing one weight read (with --config; 0: the configuration's default)")
    ap.add_argument("--config", type=int, default=0, choices=[0, 2, 3, 4], help="a multi-stream line for configuration 2, 3 or 4 (extra lines; the default run is the headline)")
    ap.add_argument("--k", type=int, default=-1, help="drafts per cycle of a --config line")
    ap.add_argument("--prompt", type=int, default=0, help="prompt length (of a --config line; of the default run: profiling only)")
    ap.add_argument("--case", default="", choices=["", "gemm"], help="gemm: the isolated verify-step GEMM of configuration 1 (no model)")
    ap.add_argument("--fmt", default="Q4_K", help="--case gemm: weight format (Q4_K, Q5_K, Q6_K, Q8_0)")
    ap.add_argument("--rows", default="17408,17408", help="--case gemm: rows of the matrices that share the launch")
    ap.add_argument("--cols", type=int, default=5120, help="--case gemm: columns (K)")
    ap.add_argument("--t", type=int, default=4, help="--case gemm: activation rows (1..16)")
    ap.add_argument("--ksplit", type=int, default=0, help="--case gemm: K-slices (0: the library's choice)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if args.steps > 24:
            args.steps = 24        # a 27B-shape token costs seconds on the host cores
        run_reference(args, rank)
        return

    if args.case == "gemm":
        if rank == 0:
            run_gemm_case(args, local)
        return
    if args.tp and world > 1:
        run_tp(args, rank, world, local)
        return
    if args.config:
        run_streams(args, rank, world, local)
        return
    import numpy as np
    import torch
    import __graft_entry__ as graft
    pkg = graft.load_package()
    llb = pkg.llb
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    llb.init(local)
    t_build = time.time()
    packs, pack, mtp, prompt = build_model(f"cuda:{local}", layers=args.layers or None)
    if args.prompt > 0:
        prompt = prompt[:args.prompt]      # a shorter prompt (profiling only; the number is then not the headline)
    max_ctx = PROMPT + GEN_CAP + 64
    torch.cuda.synchronize()
    torch.cuda.empty_cache()   # the quantisers' temporaries go back to the driver before the engine allocates
    eng = llb.SpecEngine(pack, mtp, k=K_DRAFT, max_ctx=max_ctx)
    t_build = time.time() - t_build
    eng.set_prefill(not args.exact_prefill)     # the dense tcgen05 prompt path (LLB_PREFILL=fast) unless asked otherwise
    torch.cuda.synchronize()
    t_pre = time.time()
    eng.prefill(prompt)
    torch.cuda.synchronize()
    t_pre = time.time() - t_pre

    steps, warm = args.steps, max(args.warmup, 3)
    if (steps + warm) * 2 * (K_DRAFT + 1) + 16 > GEN_CAP:
        raise SystemExit("--steps too large for the context this benchmark allocates")
    st = torch.cuda.ExternalStream(llb.lib().llb_b200_stream())
    sampler = ClockSampler(local)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident arm: K cycles enqueued back to back ------------------------------------
    sampler.start()          # nvidia-smi needs a second to come up: started before the warm-up
    eng.run_cycles(warm)
    t_w = time.time()
    while not sampler.rows and time.time() - t_w < 5.0:
        eng.run_cycles(1)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(st)
    _, toks = eng.run_cycles(steps)
    e1.record(st)
    barrier()
    ms = e0.elapsed_time(e1)
    pos_mid = eng.position()

    # ---- end to end: the per-token operator with host buffers -----------------------------------
    barrier()
    # continue from the engine's committed token: the last id of one more cycle's record
    ids_w, _ = eng.cycle()
    pos, tok = eng.position(), int(ids_w[-1])
    t0 = time.perf_counter()
    n_e2e, c0 = 0, eng.stats()["cycles"]
    while eng.stats()["cycles"] - c0 < steps:
        y = eng.step(pos, tok)
        tok, pos, n_e2e = int(y[1]), pos + 1, n_e2e + 1
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()
    clocks = sampler.stop()

    # ---- roofline legs ---------------------------------------------------------------------------
    ver_ms = eng.time_verify(10)
    gemm_us, gemm_bytes = eng.time_gemm(48)
    vbytes = verify_bytes(pack, pos_mid, K_DRAFT + 1)
    peak, peak_src = peaks()
    stats = eng.stats()
    launches = eng.graph_nodes(0)

    (ms, e2e_s), (toks, n_e2e) = pkg.dp.aggregate([ms, e2e_s], [float(toks), float(n_e2e)], device=f"cuda:{local}")

    # ---- plain greedy decoding (k = 0) on the same weights, prompt and position --------------------
    # What speculation buys or costs on this model: one row per pass, no drafter, same kernels.
    plain = None
    if rank == 0 and not args.no_plain:
        try:
            eng0 = llb.SpecEngine(pack, None, k=0, max_ctx=max_ctx)
            eng0.set_prefill(not args.exact_prefill)
            eng0.prefill(prompt)
            eng0.run_cycles(warm)
            torch.cuda.synchronize()
            p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            p0.record(st)
            _, ptoks = eng0.run_cycles(steps)
            p1.record(st)
            torch.cuda.synchronize()
            pms = p0.elapsed_time(p1)
            plain = {"value": ptoks / (pms / 1000.0), "unit": "tok/s", "ms_per_step": pms / steps, "rows_per_pass": 1,
                     "verify_ms": eng0.time_verify(10), "kernels": eng0.graph_nodes(0)}
            eng0.close()
        except Exception as ex:
            plain = {"value": None, "error": str(ex)}

    # ---- a model on which drafts ARE accepted: config 0's shape (0.8B, Q8_0, the drafter a copy of the last attention block
    # and the tied head) with every sublayer's output scaled by 0.001 (packs.ModelCfg.mix_gain), so that the next token
    # depends mostly on the current one and a one-block drafter that sees the token (eh_proj = [I | 0]) predicts some of
    # them: speculative cycles with partial acceptance, rollback and commit, timed, and plain decoding of the same model
    accept_leg = None
    if rank == 0 and not args.no_plain:
        try:
            cfg0 = packs.cfg_c0(mix_gain=0.001)
            pack0 = packs.build_pack(cfg0, device=f"cuda:{local}")
            mtp0 = packs.aux1_bytes(packs.build_mtp(pack0, eh="embed"))
            prompt0 = packs.synth_prompt(1, 64, cfg0.vocab_size)
            res = {}
            for kk in (K_DRAFT, 0):
                e0 = llb.SpecEngine(pack0, mtp0 if kk else None, k=kk, max_ctx=64 + 128 * (kk + 1) + 64)
                e0.prefill(prompt0)
                e0.run_cycles(3)
                torch.cuda.synchronize()
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record(st)
                _, tk = e0.run_cycles(96)
                a1.record(st)
                torch.cuda.synchronize()
                res[kk] = (tk / (a0.elapsed_time(a1) / 1000.0), tk / 96.0, a0.elapsed_time(a1) / 96.0, e0.stats())
                e0.close()
            sst = res[K_DRAFT][3]
            accept_leg = {"workload": "config 0's shape (0.8B: d 1024, 24 layers, V 32768, Q8_0) with sublayer outputs scaled by 0.001 so that drafts are accepted; "
                                      "MTP k=3 greedy, prompt 64, 96 timed cycles",
                          "spec_tok_s": res[K_DRAFT][0], "tokens_per_cycle": res[K_DRAFT][1], "cycle_ms": res[K_DRAFT][2],
                          "accepted_by_position": [round(a / d, 4) if d else None for a, d in zip(sst["accepted"][1:4], sst["drafted"][1:4])],
                          "plain_tok_s": res[0][0], "plain_ms_per_step": res[0][2], "speedup_over_plain": res[K_DRAFT][0] / res[0][0]}
            del pack0
            torch.cuda.empty_cache()
        except Exception as ex:
            accept_leg = {"error": str(ex)}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        try:
            cores = os.cpu_count() or 1
            tps, cids, dt = cpu_reference_run(pack, prompt, 4, 4, cores)
            # the same 4 + 4 tokens on the device (k = 0 engine on the same weights would be another
            # load; the speculative engine is lossless, so its ids are the plain greedy ids)
            eng2 = llb.SpecEngine(pack, mtp, k=K_DRAFT, max_ctx=128)
            eng2.prefill(prompt[:4])
            gids, _ = eng2.generate(4)
            eng2.close()
            cpu = {"value": tps, "unit": "tok/s", "cores": cores, "kind": "reference",
                   "sample": "full-depth pack, 4 prompt tokens then 4 greedy tokens (context 8, not 3011); plain greedy, "
                             "the reference CPU engine has no speculative path",
                   "ids_equal_device": bool(list(gids) == list(cids))}
            # the single-thread figure on a smaller sample (a 27B-shape token takes one core most of a minute)
            tps1, _, dt1 = cpu_reference_run(pack, prompt, 1, 1, 1)
            cpu["one_thread"] = {"value": tps1, "unit": "tok/s", "cores": 1, "sample": "1 prompt token then 1 greedy token"}
        except Exception as ex:  # the checker must not take the measurement down
            cpu = {"value": None, "unit": "tok/s", "cores": os.cpu_count(), "kind": "reference", "sample": f"failed: {ex}"}

    if rank == 0:
        value = toks / (ms / 1000.0)
        line = {
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": steps, "warmup": warm,
            "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "streams_per_gpu": 1, "parallelism": f"stream-dp{world}", "draft_vocabulary": DRAFT_VOCAB,
                       "layers": args.layers or 64, "l2": "inputs larger than L2: a cycle streams >14 GB of weights",
                       "tokens_per_cycle": toks / (steps * world),
                       "accepted_by_position": [round(a / d, 4) if d else None for a, d in zip(stats["accepted"][1:4], stats["drafted"][1:4])],
                       "acceptance_note": "0 on this model by construction: with N(0, 0.02) weights at d 5120 every sublayer rewrites the residual "
                                          "stream, so no one-block drafter (whatever eh_proj) predicts the trunk; value is the cycle rate. "
                                          "plain_decode is k = 0 on the same engine, prompt and position",
                       "prompt": len(prompt), "prefill_s": round(t_pre, 3), "prefill_tok_s": round(len(prompt) / t_pre, 1),
                       "prefill": "8-row verify passes" if args.exact_prefill else "dense tcgen05 path, chunks of 128 rows (all but the last k + 1 rows)", "build_s": round(t_build, 2)},
            "cycle_ms": ms / steps, "tokens_per_cycle": toks / (steps * world), "plain_decode": plain, "with_acceptance": accept_leg,
            "wait_errors": llb.lib().llb_b200_wait_errors(),   # 1 if a bounded device-side wait ever ran out (results then invalid)
            "clocks": clocks,
            "e2e": {"value": n_e2e / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 12, "d2h_bytes_per_step": 216,
                    "api": "llb_spec_pass(pos, tok) -> y[4], one call per token"},
            "gpu_launches": launches * steps,
            "roofline": {"bound": "hbm", "kernel": "k_gemm2<Q4_K> ffn_gate|ffn_up [2 x 17408 x 5120], T=4", "achieved": gemm_bytes / gemm_us / 1e3,
                         "peak": peak, "unit": "GB/s", "frac": gemm_bytes / gemm_us / 1e3 / peak, "traffic": GEMM_DRAM_TRAFFIC,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one captured launch of this shape",
                         "peak_source": peak_src,
                         "us_per_launch": gemm_us, "bytes_per_launch": gemm_bytes},
            "verify_step": {"bytes": vbytes, "ms": ver_ms, "GBs": vbytes / ver_ms / 1e6, "frac": vbytes / ver_ms / 1e6 / peak,
                            "kernels": eng.graph_nodes(2)},
            "cpu_baseline": cpu,
        }
        print(json.dumps(line), flush=True)
    eng.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
