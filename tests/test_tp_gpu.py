"""Tensor parallelism over two GPUs against the one-GPU engine: the same pack, prompt and drafter, each rank holding its
share of the projections and exchanging an NCCL all-reduce after every row-split projection.  Emitted ids must equal the
one-GPU engine's (a difference only where that engine's own top-2 gap is below 1e-3: the sum over ranks adds the partial
products in another order), top-2 logits within the path's bars, cycle and acceptance counts equal.  Runs as two child
processes, one per GPU; skipped on a box with fewer than two."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STEPS = 24


def _cases(packs):
    yield "tiny_q8", packs.cfg_tiny(n_layers=8, n_heads=4, n_kv_heads=2, ssm_heads=8, ssm_groups=4, seed=31), "cpu", 21
    yield "tiny_q4km", packs.cfg_tiny(quant="q4_k_m", n_layers=8, tied_head=False, n_heads=4, n_kv_heads=2, ssm_heads=8, ssm_groups=4, seed=32), "cpu", 13
    yield "c2_4layers", packs.cfg_c2(n_layers=4, vocab_size=2048), "cuda", 45


def _rank(rank, world, port, q, peer):
    import sys
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import __graft_entry__ as graft
    pkg = graft.load_package()
    llb, packs = pkg.llb, pkg.packs
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
        llb.init(rank)
        llb.tp_init(peer=peer)
        assert llb.lib().llb_b200_tp_peer_active() == int(peer)
        out = {}
        for name, cfg, where, n_prompt in _cases(packs):
            pack = packs.build_pack(cfg, device=f"cuda:{rank}" if where == "cuda" else "cpu")
            mtp = packs.aux1_bytes(packs.build_mtp(pack))
            prompt = packs.synth_prompt(5, n_prompt, cfg.vocab_size)
            res = {}
            for tp in ((world, 1) if rank == 0 else (world,)):
                eng = llb.SpecEngine(pack, mtp, k=3, max_ctx=n_prompt + STEPS + 16, tp=tp)
                eng.prefill(prompt)
                ids, top2 = eng.generate(STEPS)
                res[tp] = (ids, top2, eng.stats())
                eng.close()
            out[name] = res
            dist.barrier()
        assert llb.lib().llb_b200_wait_errors() == 0
        q.put((rank, out, None))
        dist.destroy_process_group()
    except Exception as ex:  # the parent must hear about it instead of waiting for the queue
        import traceback
        q.put((rank, None, traceback.format_exc()))


@pytest.mark.parametrize("peer", [False, True], ids=["nccl", "peer-stores"])
def test_two_ranks_equal_one_gpu(peer):
    """peer: the all-reduces are the library's one-shot kernel over peer memory (plain stores into the other rank's buffer,
    bounded flag waits) instead of NCCL calls."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_rank, args=(r, 2, port, q, peer)) for r in range(2)]
    for p in ps:
        p.start()
    got = {}
    for _ in ps:
        rank, out, err = q.get(timeout=900)
        assert err is None, err
        got[rank] = out
    for p in ps:
        p.join(120)
    f = lambda u: np.array(u, dtype=np.uint32).view(np.float32)
    for name, res0 in got[0].items():
        ids_tp, top2_tp, st_tp = res0[2]
        ids_1, top2_1, st_1 = res0[1]
        ids_r1, top2_r1, st_r1 = got[1][name][2]
        assert np.array_equal(ids_tp, ids_r1) and np.array_equal(top2_tp, top2_r1) and st_tp == st_r1, name   # the ranks agree bit for bit
        same = STEPS
        for i in range(STEPS):
            if ids_tp[i] != ids_1[i]:
                gap = float(f(top2_1[i][1]) - f(top2_1[i][3]))
                assert gap < 1e-3, f"{name} token {i}: two ranks {ids_tp[i]}, one GPU {ids_1[i]}, top-2 gap {gap}"
                same = i
                break
        a, b = f(top2_tp[:same, 1]), f(top2_1[:same, 1])
        assert np.all(np.abs(a - b) <= 2e-2 + 1e-2 * np.abs(b)), name
        if same == STEPS:
            assert st_tp["cycles"] == st_1["cycles"] and st_tp["accepted"] == st_1["accepted"], name
