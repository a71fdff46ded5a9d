"""GPU: the engine opened straight from a GGUF file (llb_spec_open_gguf) behaves exactly as the engine opened
from the pack the file was written from -- same emitted ids and the same top-2 logit bits -- for a Q8_0 model
with a tied head (GGUF-blocked Q8_0 re-sliced at upload), a Q4_K_M model whose block_count includes a nextn
block, and MoE models with split and with fused gate/up expert stacks."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", ["q8_tied", "q4_k_m_nextn", "moe_split", "moe_fused"])
def test_gguf_engine_equals_pack_engine(pkg, packs, llb, tmp_path, case):
    kw = {}
    if case == "q8_tied":
        cfg = packs.cfg_tiny()
    elif case == "q4_k_m_nextn":
        cfg, kw = packs.cfg_tiny(quant="q4_k_m", n_layers=8, tied_head=False, seed=12), {"nextn": 1}
    else:
        cfg, kw = packs.cfg_tiny_moe(n_layers=8, d_expert=512, d_shared=512), {"fused_gate_up": case == "moe_fused"}
    pack = packs.build_pack(cfg)
    path = packs.write_gguf(pack, str(tmp_path / "m.gguf"), **kw)
    base = packs.synth_prompt(4, 10, cfg.vocab_size)
    prompt = np.concatenate([base, base, base[:4]]).astype(np.int32)
    out = []
    for opener in ("pack", "gguf"):
        eng = (pkg.llb.SpecEngine(pack, None, k=3, max_ctx=96) if opener == "pack"
               else pkg.llb.SpecEngine.from_gguf(path, cfg, None, k=3, max_ctx=96))
        try:
            eng.prefill(prompt)
            out.append(eng.generate(24))
        finally:
            eng.close()
    assert np.array_equal(out[0][0], out[1][0])
    assert np.array_equal(out[0][1], out[1][1])


def test_gguf_open_fails_loudly(pkg, llb, tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"GGUF" + b"\x03\x00\x00\x00" + b"\x00" * 64)
    with pytest.raises(pkg.llb.LlbError):
        pkg.llb.SpecEngine.from_gguf(str(p), None, None)


def test_gguf_nextn_block_is_the_drafter(pkg, packs, llb, tmp_path):
    """A file that carries its MTP block (nextn_predict_layers = 1, blk.<L>.nextn.* and the block's attention / FFN
    tensors): the engine opened from it drafts with that block and the file's own head, and behaves exactly as the
    pack-opened engine given the same drafter as an AUX1 image: same ids, same top-2 bits, same acceptance counts."""
    cfg = packs.cfg_tiny(quant="q4_k_m", n_layers=8, tied_head=False, seed=12)
    pack = packs.build_pack(cfg)
    entries = packs.build_mtp(pack)
    path = packs.write_gguf(pack, str(tmp_path / "m.gguf"), mtp_entries=entries)
    prompt = packs.synth_prompt(1, 9, cfg.vocab_size)
    out = []
    for opener in ("pack", "gguf"):
        eng = (pkg.llb.SpecEngine(pack, packs.aux1_bytes(entries), k=3, max_ctx=96) if opener == "pack"
               else pkg.llb.SpecEngine.from_gguf(path, cfg, None, k=3, max_ctx=96))
        try:
            eng.prefill(prompt)
            ids, top2 = eng.generate(24)
            out.append((ids, top2, eng.stats()))
        finally:
            eng.close()
    assert np.array_equal(out[0][0], out[1][0]) and np.array_equal(out[0][1], out[1][1])
    assert out[0][2] == out[1][2] and sum(out[1][2]["drafted"]) > 0
