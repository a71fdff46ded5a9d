#!/usr/bin/env python
"""Writes tests/golden/moe_ffn.npz: the routed-expert FFN's known answers, made by the REFERENCE's own
float64 checker reports/metal-catchup/tools/mx_ref.py (run unmodified, through runpy) on a synthetic
tiny MoE model.

    python tests/golden/make_golden_moe.py [--ref REFERENCE_DIR]

What happens: the tiny MoE pack of eureka-engine_b200/packs.py (seeded) is written as a GGUF holding the
MoE tensors under their GGUF names with the pack's quantised bytes; for a few seeded FFN inputs h2 the C
restatement (oracle/q35_oracle.c: q35_moe_ffn) produces the record the reference engine would dump
(layer, d, k, h2, out, ids, weights + shared gate); mx_ref.py recomputes each record from the GGUF bytes
(gguf-py's dequantize, float64) and reports the relative error of `out`, whether the chosen experts are
equal, and the weight errors.  The fixture keeps, per record: h2, the checker's float64 answer `ref`, its
expert ids `rid`, weights `rw` and shared gate `gs`, and what it said about the restatement's record.
tests/test_oracle_cpu.py compares the restatement against these on every run; the GPU tests compare the
CUDA path against the same vectors.
"""
import argparse
import hashlib
import io
import contextlib
import os
import runpy
import struct
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

LAYERS = (0, 1, 5)          # layer 0: Q5_K down stacks (q4_k_s rule), the others Q4_K
RECORDS_PER_LAYER = 3


def golden_cfg(packs):
    return packs.cfg_tiny_moe(n_layers=8, d_expert=512, d_shared=512)


def write_gguf(path, pack, cfg):
    from gguf import GGUFWriter, GGMLQuantizationType as Q
    qt = {"Q4_K": Q.Q4_K, "Q5_K": Q.Q5_K, "Q6_K": Q.Q6_K, "Q8_0": Q.Q8_0}
    w = GGUFWriter(path, "qwen35moe")
    ne, ef, sf, d = cfg.n_experts, cfg.d_expert, cfg.d_shared, cfg.d_model
    shapes = {"ffn_gate_inp": (ne, d), "ffn_gate_inp_shexp": (d,), "ffn_gate_exps": (ne, ef, d), "ffn_up_exps": (ne, ef, d),
              "ffn_down_exps": (ne, d, ef), "ffn_gate_shexp": (sf, d), "ffn_up_shexp": (sf, d), "ffn_down_shexp": (d, sf)}
    todo = []
    for il in LAYERS:
        for leaf, shp in shapes.items():
            name = f"blk.{il}.{leaf}.weight"
            e = pack.by_name[name]
            raw = pack.raw(name).numpy()
            if e.ty == "F32":
                arr = raw.view(np.float32).reshape(shp)
                w.add_tensor_info(name, shp, np.dtype(np.float32), arr.nbytes)
            else:
                bs = tuple(shp[:-1]) + (e.row_bytes,)
                arr = raw.reshape(bs)
                w.add_tensor_info(name, bs, np.dtype(np.uint8), arr.nbytes, raw_dtype=qt[e.ty])
            todo.append(arr)
    w.write_header_to_file(); w.write_kv_data_to_file(); w.write_ti_data_to_file()
    for arr in todo:
        w.write_tensor_data(np.ascontiguousarray(arr))
    w.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("LLB_REFERENCE_ROOT"), required=not os.environ.get("LLB_REFERENCE_ROOT"),
                    help="the reference tree (or LLB_REFERENCE_ROOT)")
    args = ap.parse_args()
    import __graft_entry__ as graft
    packs = graft.load_package().packs
    from oracle.bindings import Oracle
    cfg = golden_cfg(packs)
    pack = packs.build_pack(cfg)
    sha = hashlib.sha256(pack.data.numpy().tobytes()).hexdigest()
    orc = Oracle(pack.index_text(), pack.data.numpy(), cap=8)
    checker = os.path.join(args.ref, "reports/metal-catchup/tools/mx_ref.py")
    d, k = cfg.d_model, cfg.n_experts_used
    rng = np.random.default_rng(77)
    out = {k_: [] for k_ in ("layer", "h2", "ref", "rid", "rw", "gs", "oracle_rel", "oracle_ids_equal")}
    with tempfile.TemporaryDirectory() as tmp:
        gg = os.path.join(tmp, "tiny_moe.gguf")
        write_gguf(gg, pack, cfg)
        for il in LAYERS:
            for r in range(RECORDS_PER_LAYER):
                # normed hidden rows have unit mean square; scale some to exercise the softmax's range
                h2 = (rng.standard_normal(d) * (1.0, 0.3, 2.5)[r]).astype(np.float32)
                o, ids, wts = orc.moe_ffn(il, h2)
                dump = os.path.join(tmp, f"rec_{il}_{r}.bin")
                with open(dump, "wb") as f:
                    f.write(struct.pack("<3I", il, d, k) + h2.tobytes() + o.tobytes() + ids.astype(np.uint32).tobytes() + wts.tobytes())
                argv, sys.argv = sys.argv, [checker, gg, dump, "1"]
                try:
                    with contextlib.redirect_stdout(io.StringIO()):
                        g = runpy.run_path(checker, run_name="__main__")
                finally:
                    sys.argv = argv
                res = g["res"][0]
                out["layer"].append(il); out["h2"].append(h2); out["ref"].append(np.asarray(g["ref"], np.float64))
                out["rid"].append(np.asarray(g["rid"], np.int32)); out["rw"].append(np.asarray(g["rw"], np.float64))
                out["gs"].append(float(g["gs"])); out["oracle_rel"].append(res["rel"]); out["oracle_ids_equal"].append(bool(res["ids_equal"]))
                print(f"layer {il} record {r}: checker says rel {res['rel']:.3e} ids_equal {res['ids_equal']} w_err {res['w_err']} gs_err {res['gs_err']:.2e}")
    np.savez(os.path.join(HERE, "moe_ffn.npz"), pack_sha256=sha, **{k_: np.asarray(v) for k_, v in out.items()})
    print("wrote moe_ffn.npz; pack sha256", sha)


if __name__ == "__main__":
    main()
