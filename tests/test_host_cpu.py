"""CPU tests of the host-side logic: the C ABI's symbol table, pack and container writers, stream
sharding (2 gloo ranks).  No compute call is made: there is no GPU here."""
import ctypes
import os
import re
import struct

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(pkg):
    """Every LLB_API function of include/llb_b200.h is exported by the built library."""
    hdr = open(os.path.join(ROOT, "include", "llb_b200.h")).read()
    names = re.findall(r"LLB_API\s+[A-Za-z_ \*]+?\b(llb_[a-z0-9_]+)\s*\(", hdr)
    assert len(names) >= 30
    if not os.path.exists(pkg.llb.SO_PATH):
        pkg.llb.build()
    lib = ctypes.CDLL(pkg.llb.SO_PATH)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_calls_fail_loudly_without_a_device(pkg):
    """No CPU fallback: initialisation reports the missing device, and calls before it say so."""
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    L = pkg.llb.lib()
    assert L.llb_b200_alloc_zero(16) == 0
    assert b"llb_b200_init" in L.llb_b200_last_error()
    with pytest.raises(pkg.llb.LlbError):
        pkg.llb.init(0)


def test_index_text_round_trip(packs, tmp_path):
    cfg = packs.cfg_tiny(quant="q4_k_m", n_layers=8, tied_head=False)
    pack = packs.build_pack(cfg)
    pack.write(str(tmp_path))
    back = packs.Pack.read(str(tmp_path), cfg)
    assert [(e.name, e.off, e.nbytes, e.rows, e.cols, e.ty) for e in back.entries] == \
           [(e.name, e.off, e.nbytes, e.rows, e.cols, e.ty) for e in pack.entries]
    assert torch.equal(back.data, pack.data)
    for e in pack.entries:
        assert e.off % 64 == 0                                   # tools/q8_pack.py:32
        want = e.rows * (e.cols * 4 if e.ty == "F32" else packs.row_bytes(e.ty, e.cols))
        assert e.nbytes == want
    types = {e.name.split(".")[-2]: e.ty for e in pack.entries if e.name.startswith("blk.0.") and e.rows > 1}
    assert types["ffn_down"] == "Q6_K" and types["ffn_gate"] == "Q4_K"     # layer 0 is in the "more bits" eighth


def test_tied_head_aliases_the_embedding(packs):
    pack = packs.build_pack(packs.cfg_tiny())
    a, b = pack.by_name["token_embd.weight"], pack.by_name["output.weight"]
    assert (a.off, a.nbytes, a.ty) == (b.off, b.nbytes, b.ty)


def test_truncated_pack_keeps_the_draws(packs):
    """--layers L must see the same bytes for the layers it keeps (the generator is advanced in full pack order)."""
    cfg = packs.cfg_tiny(n_layers=8)
    full, cut = packs.build_pack(cfg), packs.build_pack(cfg, layers=4)
    for e in cut.entries:
        assert torch.equal(cut.raw(e.name), full.raw(e.name)), e.name


def test_aux1_layout(packs):
    """AUX1: 16-byte header, 72-byte named entries, 256-aligned payloads (tools/auxpack/auxpack.py:10-22)."""
    pack = packs.build_pack(packs.cfg_tiny())
    ent = packs.build_mtp(pack)
    img = packs.aux1_bytes(ent)
    assert img[:4] == b"AUX1" and struct.unpack_from("<III", img, 4) == (1, 17, 0)
    for i, (name, ty, shape, raw) in enumerate(ent):
        rec = struct.unpack_from("<32sII4IQQ", img, 16 + 72 * i)
        assert rec[0].rstrip(b"\0").decode() == name and rec[1] == packs.AUX_DT[ty]
        off, nb = rec[-2], rec[-1]
        assert off % 256 == 0 and nb == raw.numel()
        assert img[off:off + nb] == raw.numpy().tobytes()
    assert [e[0] for e in ent] == packs.MTP_ORDER
    d = pack.cfg.d_model
    eh = packs.dequant(ent[2][1], ent[2][3], d, 2 * d)
    assert float(eh[:, :d].abs().max()) == 0.0                    # eh_proj = [0 | I] up to quantisation
    assert float((eh[:, d:] - torch.eye(d)).abs().max()) < 0.02


def test_plane_permutation_is_an_involution():
    perm = lambda c: (c & ~7) | ((c & 4) | ((c & 1) << 1) | ((c & 2) >> 1))
    assert [perm(c) for c in range(8)] == [0, 2, 1, 3, 4, 6, 5, 7]
    assert all(perm(perm(c)) == c for c in range(64))


def test_stream_sharding(pkg):
    dp = pkg.dp
    for n, w in ((8, 1), (8, 2), (32, 8), (5, 4)):
        got = sorted(s for r in range(w) for s in dp.shard_streams(n, r, w))
        assert got == list(range(n))
        sizes = [len(dp.shard_streams(n, r, w)) for r in range(w)]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        dp.shard_streams(4, 2, 2)
    assert dp.aggregate([1.0], [2.0]) == ([1.0], [2.0])           # no process group: one rank


def _gloo_rank(rank, world, port, q):
    import sys
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import __graft_entry__ as graft
    dp = graft.load_package().dp
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    t, c = dp.aggregate([10.0 + rank, 5.0 - rank], [100.0 * (rank + 1), float(len(dp.shard_streams(7, rank, world)))])
    q.put((rank, t, c))
    dist.destroy_process_group()


def test_aggregate_two_gloo_ranks():
    """The N > 1 bench path: MAX of the ranks' times, SUM of what they emitted."""
    import socket
    import torch.multiprocessing as mp
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_gloo_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    out = sorted(q.get(timeout=120) for _ in ps)
    for p in ps:
        p.join(60)
    for rank, t, c in out:
        assert t == [11.0, 5.0] and c == [300.0, 7.0]


# ---- GGUF reader (no GPU: the header only) -------------------------------------------------------
def _index_fields(text):
    cfg, tens = {}, {}
    for line in text.splitlines():
        if line.startswith("#cfg\t"):
            _, k, v = line.split("\t")
            cfg[k] = v
        elif line and not line.startswith("#"):
            n, off, nb, rows, cols, ty = line.split("\t")[:6]
            tens[n] = (int(off), int(nb), int(rows), int(cols), ty)
    return cfg, tens


@pytest.mark.parametrize("case", ["q8_tied", "q4_k_m_nextn", "moe_fused", "moe_split"])
def test_gguf_header_gives_the_packs_index(pkg, packs, tmp_path, case):
    """A pack written as GGUF and read back by the library: same configuration keys, same tensors with the same
    shapes and types (Q8_0 marked as GGUF-blocked), bytes at the recorded file offsets equal the pack's
    (tools/gguf2pack.c:541-600 for the keys; block_count counts nextn blocks, which are left out)."""
    kw = {}
    if case == "q8_tied":
        cfg = packs.cfg_tiny()
    elif case == "q4_k_m_nextn":
        cfg, kw = packs.cfg_tiny(quant="q4_k_m", n_layers=8, tied_head=False, seed=12), {"nextn": 1}
    else:
        cfg, kw = packs.cfg_tiny_moe(n_layers=8, d_expert=512, d_shared=512), {"fused_gate_up": case == "moe_fused"}
    pack = packs.build_pack(cfg)
    path = packs.write_gguf(pack, str(tmp_path / "m.gguf"), **kw)
    gcfg, gt = _index_fields(pkg.llb.gguf_index(path))
    pcfg, pt = _index_fields(pack.index_text())
    for k, v in pcfg.items():
        if k in ("rope_freq_base", "rms_norm_eps"):
            assert float(gcfg[k]) == pytest.approx(float(v), rel=1e-6)
        elif k == "d_ff" and cfg.n_experts:
            assert int(gcfg[k]) == max(cfg.d_expert, cfg.d_shared)    # the reference's rule for qwen35moe
        else:
            assert gcfg[k] == v, k
    blob = open(path, "rb").read()
    for name, (off, nb, rows, cols, ty) in pt.items():
        if case == "moe_fused" and ("ffn_gate_exps" in name or "ffn_up_exps" in name):
            fused = gt[name.replace("ffn_gate_exps", "ffn_gate_up_exps").replace("ffn_up_exps", "ffn_gate_up_exps")]
            assert fused[2] == 2 * rows and fused[3] == cols and fused[4] == ty
            continue
        goff, gnb, grows, gcols, gty = gt[name]
        assert (grows, gcols, gnb) == (rows, cols, nb), name
        assert gty == ("Q8_0G" if ty == "Q8_0" else ty)
        if ty != "Q8_0":
            assert blob[goff:goff + gnb] == pack.raw(name).numpy().tobytes(), name
    if cfg.tied_head:
        assert gt["output.weight"] == gt["token_embd.weight"]


def test_gguf_reader_refuses_bad_files(pkg, tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"GGUF" + b"\x03\x00\x00\x00" + b"\xff" * 40)
    with pytest.raises(pkg.llb.LlbError):
        pkg.llb.gguf_index(str(p))
    p.write_bytes(b"not a gguf file at all, just some text that is long enough")
    with pytest.raises(pkg.llb.LlbError):
        pkg.llb.gguf_index(str(p))
    with pytest.raises(pkg.llb.LlbError):
        pkg.llb.gguf_index(str(tmp_path / "missing.gguf"))


# ---- the drop-in boundary compiles next to the interface it replaces --------------------------------
REF_HOST = os.environ.get("LLB_REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")


def _gcc(src: str, tmp_path, *inc):
    import subprocess
    c = tmp_path / "tu.c"
    c.write_text(src)
    cmd = ["gcc", "-std=gnu11", "-Wall", "-Werror", "-Wno-unused-function", "-Wno-unused-variable", "-c", str(c), "-o", str(tmp_path / "tu.o"),
           "-I", os.path.join(ROOT, "include")]
    for i in inc:
        cmd += ["-I", i]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_backend_header_defines_the_reference_surface(tmp_path):
    """include/llb_backend_b200.h gives the names host/llb_backend.h:7-34 asks of a backend, with the reference's truth
    sense (bool, true = success), so a chain written in the reference's idiom compiles unchanged."""
    _gcc(r'''
#include "llb_backend_b200.h"
static void err_fail(const char *m) { (void)m; }
typedef unsigned int u32;
int chain(void) {
  llb_dptr p = llb_alloc_zero(1024);
  if (p == 0) { err_fail("alloc"); return 1; }
  if (!llb_zero(p + 16, 64)) err_fail("device launch failed");
  float host[4] = {0};
  if (!llb_write(p, host, sizeof host) || !llb_copy(p + 64, p, 16) || !llb_read(host, p + 64, 16) || !llb_sync()) err_fail("io");
  llb_kernel k = llb_kernel_by_name("llb_spec_gu3");      /* a reference kernel name: not exported, NULL */
  u32 n = 4; llb_dptr q = p; float *o = 0; int z = 0; long long st = 0;
  llb_graph_begin();
  bool ok = LLB_LAUNCH(k, 1, 1, 256, &q, &z, &st, &n, &o);
  ok = LLB_LAUNCH_SM(k, 1, 1, 256, 1024, &q, &z, &st, &n, &o) && ok;
  llb_graph_end();
  llb_graph_bail();
  q = llb_dev(host);
  return ok ? 0 : 2;
}
''', tmp_path)


def test_backend_header_compiles_before_the_reference_contract(tmp_path):
    """The reference's contract header refuses to compile unless a backend header came first and defined LLB_LAUNCH
    (host/llb_backend.h:46-49); with ours in front it compiles."""
    root = REF_HOST
    if not os.path.exists(os.path.join(root, "host", "llb_backend.h")):
        pytest.skip("the reference tree is not on this machine (set LLB_REFERENCE_ROOT)")
    _gcc('#include "llb_backend_b200.h"\n#include "llb_backend.h"\nint f(void) { return llb_sync() ? 0 : 1; }\n', tmp_path,
         os.path.join(root, "host"))


def test_integration_snippets_compile(tmp_path):
    """Every C block of INTEGRATION.md compiles as written against include/ (helpers the text calls "any file reader"
    are declared, not defined)."""
    md = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    blocks = re.findall(r"```c\n(.*?)```", md, flags=re.S)
    assert blocks
    pre = r'''
#include <string.h>
#include <stddef.h>
typedef unsigned int u32; typedef unsigned long long u64;
void err_fail(const char *m);
char *slurp(const char *dir, const char *name, size_t *n);
void *map_file(const char *dir, const char *name, size_t *n);
void *map_path(const char *path, size_t *n);
static const char *spec_mtp;
'''
    for b in blocks:
        _gcc(pre + b, tmp_path)


# ---- llb_spec_open's host-side checks --------------------------------------------------------------
def test_check_index_refuses_truncated_packs_and_bad_configurations(pkg, packs):
    L = pkg.llb.lib()
    pack = packs.build_pack(packs.cfg_tiny(quant="q4_k_m", n_layers=8, tied_head=False))
    text = pack.index_text()
    nbytes = pack.data.numel()
    assert L.llb_spec_check_index(text.encode(), nbytes) == 0, L.llb_b200_last_error()
    # a pack cut short: the error names a tensor and says where the pack ends
    assert L.llb_spec_check_index(text.encode(), nbytes - 4096) == -1
    msg = L.llb_b200_last_error().decode()
    assert "past the end of the pack" in msg and "blk." in msg or "output" in msg, msg
    assert L.llb_spec_check_index(text.encode(), 0) == -1
    # an offset near 2^64 must not wrap around the range check
    last = pack.entries[-1]
    bad = text.replace(f"{last.name}\t{last.off}\t", f"{last.name}\t{2**64 - 64}\t")
    assert bad != text and L.llb_spec_check_index(bad.encode(), nbytes) == -1
    # zeroed or missing configuration values: an error message, not a division by zero
    for key in ("n_kv_heads", "n_heads", "full_attention_interval", "ssm_group_count", "ssm_time_step_rank", "n_layers", "head_dim"):
        line = next(l for l in text.splitlines() if l.startswith(f"#cfg\t{key}\t"))
        assert L.llb_spec_check_index(text.replace(line, f"#cfg\t{key}\t0").encode(), nbytes) == -1, key
        assert key.encode() in L.llb_b200_last_error()
        if key != "full_attention_interval":     # a missing interval takes the engine's default of 4
            assert L.llb_spec_check_index(text.replace(line + "\n", "").encode(), nbytes) == -1, key
    # a tensor whose byte count does not match its shape
    e = pack.by_name["blk.0.ffn_gate.weight"]
    bad = text.replace(f"{e.name}\t{e.off}\t{e.nbytes}\t", f"{e.name}\t{e.off}\t{e.nbytes - 144}\t")
    assert L.llb_spec_check_index(bad.encode(), nbytes) == -1 and b"ffn_gate" in L.llb_b200_last_error()


def test_ring_ksplit_is_one_value_for_both_pass_widths(pkg):
    """The conv ring keeps attn_qkv rows as K-slice partial sums across passes of both widths (prompt chunks of 8 rows on
    16 plane columns, speculative passes of k + 1 rows on 8), so the split must not depend on the width.  Replays the
    choice at d = 5120 on 148 SMs for the formats a Q4_K_M / Q4_K_S / Q8_0 file puts attn_qkv in: the free choice differs
    between the widths for Q5_K and Q6_K, the fixed one is valid at both."""
    L = pkg.llb.lib()
    Q8_0, Q4_K, Q6_K, Q5_K = 1, 3, 4, 9
    nsb, sms = 5120 // 256, 148
    group = (10240 + 6144 + 48 + 48 + 15) // 16          # qkv | z | beta | alpha of the 27B shape in one launch
    alone = 10240 // 16                                   # attn_qkv alone in its format
    differs = 0
    for fmt in (Q4_K, Q5_K, Q6_K, Q8_0):
        for ntiles in (group, alone, 97):
            k8, k16 = L.llb_b200_gemm_ksplit(fmt, 8, ntiles, nsb, sms), L.llb_b200_gemm_ksplit(fmt, 16, ntiles, nsb, sms)
            differs += k8 != k16
            ring = L.llb_b200_ring_ksplit(fmt, nsb, ntiles, 8, 16, sms)
            assert 1 <= ring <= 8
            # valid at both widths: asking for it gives it back (the launch refuses anything else)
            for nc in (8, 16):
                lo = L.llb_b200_ring_ksplit(fmt, nsb, ntiles, nc, nc, sms)
                assert lo >= 1
            assert ring >= max(L.llb_b200_ring_ksplit(fmt, nsb, 1 << 20, 8, 8, sms) and 1, 1)
    assert differs > 0            # the case the fixed split exists for does occur
    # a width no split up to 8 can serve is reported as 0 (the engine then refuses the model by name)
    assert L.llb_b200_ring_ksplit(Q6_K, 64, 1000, 8, 16, sms) == 0


# ---- tensor-parallel partition (no GPU) ----------------------------------------------------------------
def test_tp_plan_partitions_the_27b_shape(pkg):
    """Every rank's share of the 27B shape at 2, 4 and 8 ranks: query heads, FFN super-blocks and DeltaNet groups are
    disjoint and cover the model; FFN shares are whole super-blocks, uneven at 8 (68 = 4 x 9 + 4 x 8); kv heads are split
    up to 4 ranks and replicated above (each rank holds the one head its queries read); a rank's value heads are exactly
    the heads hh with hh % 16 in its groups (the tiling of tools/qwen35_engine.c:621-626)."""
    llb = pkg.llb
    H, KV, f, GK, TR = 24, 4, 17408, 16, 48
    for n in (1, 2, 4, 8):
        plans = [llb.tp_plan(r, n, H, KV, f, GK, TR) for r in range(n)]
        heads = sorted(h for p in plans for h in range(p["h0"], p["h0"] + p["H_l"]))
        assert heads == list(range(H))
        cols = sorted(c for p in plans for c in range(p["f0"], p["f0"] + p["f_l"], 256))
        assert cols == list(range(0, f, 256)) and all(p["f_l"] % 256 == 0 for p in plans)
        assert max(p["f_l"] for p in plans) - min(p["f_l"] for p in plans) <= 256
        groups = sorted(g for p in plans for g in range(p["g0"], p["g0"] + p["GK_l"]))
        assert groups == list(range(GK))
        for p in plans:
            assert p["reps"] == TR // GK and p["TR_l"] == p["reps"] * p["GK_l"]
            G = H // KV
            used = {h // G for h in range(p["h0"], p["h0"] + p["H_l"])}
            assert used <= set(range(p["kv0"], p["kv0"] + p["KV_l"]))        # every query head finds its kv head on its rank
            if n <= KV:
                assert p["KV_l"] == KV // n
            else:
                assert p["KV_l"] == 1
    assert [llb.tp_plan(r, 8, H, KV, f, GK, TR)["f_l"] // 256 for r in range(8)] == [9, 9, 9, 9, 8, 8, 8, 8]
    for bad in ((0, 5, H, KV, f, GK, TR), (0, 2, 3, 1, 512, 2, 4), (0, 4, 8, 2, 512, 2, 4), (3, 2, H, KV, f, GK, TR)):
        with pytest.raises(llb.LlbError):
            llb.tp_plan(*bad)


def _gloo_id_rank(rank, world, port, q):
    import sys
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import __graft_entry__ as graft
    llb = graft.load_package().llb
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    uid = llb.exchange_unique_id(lambda: bytes(range(128)), rank)
    q.put((rank, uid))
    dist.destroy_process_group()


def test_unique_id_reaches_every_rank():
    """The N > 1 tensor-parallel set-up on CPU: what rank 0 makes is what rank 1 passes to llb_b200_tp_init."""
    import socket
    import torch.multiprocessing as mp
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_gloo_id_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    out = dict(q.get(timeout=120) for _ in ps)
    for p in ps:
        p.join(60)
    assert out[0] == out[1] == bytes(range(128))
