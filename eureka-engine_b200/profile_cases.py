#!/usr/bin/env python
"""Small, self-ending cases to run under ncu (one GPU).

    python eureka-engine_b200/profile_cases.py gemm FMT ROWS[,ROWS..] K     three launches of one GEMM site
    python eureka-engine_b200/profile_cases.py gemm3 ROWS[,ROWS..] K        the same for Q4_K on the tcgen05 kernel
    python eureka-engine_b200/profile_cases.py verify LAYERS [PROMPT]       two replays of the verify pass of the
                                                                            27B-shape model truncated to LAYERS,
                                                                            bracketed by cudaProfilerStart/Stop
    python eureka-engine_b200/profile_cases.py moe LAYERS [K] [PROMPT]      the MoE configuration (256 experts, top 8 +
                                                                            shared, Q4_K_S) truncated to LAYERS: verify-pass
                                                                            time, bytes and per-op times, prompt-lookup drafter
    python eureka-engine_b200/profile_cases.py c4 CTX [K] [LAYERS]          the 9B-shape Q8_0 configuration at a context of
                                                                            CTX positions (prompt fed through the T-row pass):
                                                                            prefill time, verify-pass time and bytes, per-op times
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import torch  # noqa: E402

import __graft_entry__ as graft  # noqa: E402


def case_gemm(fmt_name, rows_list, K, T=4, tcgen05=False):
    pkg = graft.load_package()
    llb, packs = pkg.llb, pkg.packs
    llb.init(0)
    L = llb.lib()
    L.llb_b200_use_tcgen05(1 if tcgen05 else 0)
    dev = torch.device("cuda:0")
    fmt = packs.FMT[fmt_name]
    raws = [packs.q4k_random_blocks(r, K, seed=2, device=dev) if fmt_name == "Q4_K"
            else packs.QUANT[fmt_name](torch.randn(r, K, device=dev) * 0.02) for r in rows_list]
    sets = []
    for _ in range(3):
        ws = []
        for r, raw in zip(rows_list, raws):
            p = llb.alloc(L.llb_b200_weight_bytes(fmt, r, K))
            llb.check(L.llb_b200_weight_upload(fmt, r, K, raw.data_ptr(), 1, p), "weight_upload")
            ws.append(p)
        sets.append(ws)
    x = torch.randn(T, K, device=dev)
    xp = llb.handle(L.llb_b200_xp_new(K, T, 2), "xp_new")
    llb.check(L.llb_b200_xp_set_f32(xp, x.data_ptr()), "xp_set")
    ys = [torch.zeros(T, r, device=dev) for r in rows_list]
    for ws in sets:
        llb.gemm(fmt, ws, rows_list, [y.data_ptr() for y in ys], K, xp, 0)
    L.llb_sync()
    print("ok", float(ys[0].abs().max()), "wait errors", L.llb_b200_wait_errors())


def case_verify(layers, nprompt=3011):
    import bench
    pkg = graft.load_package()
    llb = pkg.llb
    llb.init(0)
    packs, pack, mtp, prompt = bench.build_model("cuda:0", layers=layers if layers < 64 else None)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    eng = llb.SpecEngine(pack, mtp, k=3, max_ctx=4300)
    eng.prefill(prompt[:nprompt])
    eng.run_cycles(2)
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    ms = eng.time_verify(1)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print("verify ms", ms, "kernels", eng.graph_nodes(2))
    for n, (c, t) in sorted(eng.profile_verify().items(), key=lambda kv: -kv[1][1]):
        print(f"{n:18s} n={c:4d} total_us={t:9.1f}")
    eng.close()


def moe_verify_bytes(pack, packs, T):
    """Algorithmic bytes of one verify pass of an MoE model at context 0: every dense matrix, the routers, the head
    and the shared experts once; each of the T x k (row, rank) slots reads its expert's three matrices once."""
    c = pack.cfg
    dense = sum(e.nbytes for e in pack.entries
                if e.name == "output.weight" or "ffn_gate_inp" in e.name
                or (e.name.startswith("blk.") and e.rows > 1 and e.ty != "F32" and "_exps" not in e.name))
    routed = T * c.n_experts_used * sum(e.nbytes / c.n_experts for e in pack.entries if "_exps" in e.name)
    return dense, routed


def case_moe(layers, k=3, nprompt=512):
    pkg = graft.load_package()
    llb, packs = pkg.llb, pkg.packs
    llb.init(0)
    cfg = packs.cfg_c3()
    pack = packs.build_pack(cfg, device="cuda:0", layers=layers if layers < cfg.n_layers else None)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    eng = llb.SpecEngine(pack, None, k=k, max_ctx=nprompt + 512)
    eng.prefill(packs.synth_prompt(4, nprompt, cfg.vocab_size))
    ids, got = eng.run_cycles(8)
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    ms1 = eng.time_verify(1)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    # the prompt-lookup drafter finds no drafts in random text, so the pass in the control block has one row:
    # time it at every row count (rows beyond the drafter's repeat the first token)
    for rows in range(1, k + 2):
        ms = eng.time_verify_rows(20, rows)
        dense, routed = moe_verify_bytes(pack, packs, rows)
        print(f"moe verify: layers {pack.cfg.n_layers} rows {rows}: {ms:.3f} ms/pass; dense+shared {dense / 1e9:.3f} GB, "
              f"routed slots {routed / 1e9:.3f} GB -> {(dense + routed) / ms / 1e6:.1f} GB/s; kernels {eng.graph_nodes(2)}")
    for n, (c, t) in sorted(eng.profile_verify().items(), key=lambda kv: -kv[1][1]):
        print(f"{n:18s} n={c:4d} total_us={t:9.1f}")
    eng.close()


def case_c4(ctx, k=3, layers=0):
    import time
    import bench
    pkg = graft.load_package()
    llb, packs = pkg.llb, pkg.packs
    llb.init(0)
    cfg = packs.cfg_c4()
    pack = packs.build_pack(cfg, device="cuda:0", layers=layers if 0 < layers < cfg.n_layers else None)
    mtp = packs.aux1_bytes(packs.build_mtp(pack))
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    eng = llb.SpecEngine(pack, mtp, k=k, max_ctx=ctx + 640)
    prompt = packs.synth_prompt(5, ctx, cfg.vocab_size)
    t0 = time.time()
    eng.prefill(prompt)
    torch.cuda.synchronize()
    t_pf = time.time() - t0
    ids, got = eng.run_cycles(8)
    ms = eng.time_verify(10)
    nb = bench.verify_bytes(pack, ctx, k + 1)
    print(f"c4: layers {pack.cfg.n_layers} ctx {ctx} T {k + 1}: prefill {t_pf:.1f} s ({ctx / t_pf:.0f} tok/s), verify {ms:.3f} ms/pass, "
          f"{nb / 1e9:.3f} GB -> {nb / ms / 1e6:.1f} GB/s; kernels {eng.graph_nodes(2)}")
    for n, (c, t) in sorted(eng.profile_verify().items(), key=lambda kv: -kv[1][1]):
        print(f"{n:18s} n={c:4d} total_us={t:9.1f}")
    eng.close()


if __name__ == "__main__":
    if sys.argv[1] == "gemm":
        case_gemm(sys.argv[2], [int(v) for v in sys.argv[3].split(",")], int(sys.argv[4]))
    elif sys.argv[1] == "gemm3":
        case_gemm("Q4_K", [int(v) for v in sys.argv[2].split(",")], int(sys.argv[3]), tcgen05=True)
    elif sys.argv[1] == "verify":
        case_verify(int(sys.argv[2]), int(sys.argv[3]) if len(sys.argv) > 3 else 3011)
    elif sys.argv[1] == "c4":
        case_c4(int(sys.argv[2]), int(sys.argv[3]) if len(sys.argv) > 3 else 3, int(sys.argv[4]) if len(sys.argv) > 4 else 0)
    elif sys.argv[1] == "moe":
        case_moe(int(sys.argv[2]), int(sys.argv[3]) if len(sys.argv) > 3 else 3, int(sys.argv[4]) if len(sys.argv) > 4 else 512)
    else:
        raise SystemExit(__doc__)
