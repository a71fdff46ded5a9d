"""Synthetic weight packs in the reference's on-disk formats.

A pack directory is what the reference CPU engine reads (tools/qwen35_engine.c:379-433):
``pack.bin`` (tensors, each 64-byte aligned) and ``index.tsv`` (``#cfg`` lines, then one line per
tensor ``name off bytes rows cols TYPE row_bytes fmt``).  The MTP drafter travels in the
reference's named ``AUX1`` container (tools/auxpack/auxpack.py:10-22; loader
host/llb_host.c:1543-1570) or the positional ``MTP1`` one (tools/mtp27/mtp_pack.py:51-62).

Block layouts written here are the ones the reference *de*quantises
(tools/qwen35_engine.c:233-327):
  Q8_0  row-split  [cols x int8][cols/32 x f16 scale]            (tools/q8_pack.py:7-10)
  Q4_K  144 B / 256: f16 d, f16 dmin, 12 B of 6-bit scale/min, 128 B nibbles
  Q5_K  176 B / 256: Q4_K plus 32 B of fifth bits before the nibbles
  Q6_K  210 B / 256: 128 B low nibbles, 64 B high pairs, 16 int8 scales, f16 d
The *encoders* are this repository's own (round-to-nearest on a min/max grid); only the decoding
is fixed by the reference, so any encoder that emits valid blocks is admissible.

Everything is written with torch ops so the same code quantises a 0.8B-shape pack on the CPU and
a 27B-shape pack on the GPU (where the bytes then stay resident).
"""
from __future__ import annotations

import dataclasses
import os
import struct
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np
import torch

FMT = {"F32": 0, "Q8_0": 1, "F16": 2, "Q4_K": 3, "Q6_K": 4, "Q5_K": 9}  # host/llb_formats.h:4-15
AUX_DT = {"F32": 0, "BF16": 1, "Q8_0": 2, "Q4_K": 3, "Q6_K": 4, "U32": 5, "BLOB": 6, "Q5_K": 7}
_BLOCK = {"F32": (4, 1), "Q8_0": (34, 32), "F16": (2, 1), "Q4_K": (144, 256), "Q6_K": (210, 256), "Q5_K": (176, 256)}


def row_bytes(ty: str, cols: int) -> int:
    """Stored bytes of one matrix row (host/llb_formats.h:17 LLB_FM_RB)."""
    bb, be = _BLOCK[ty]
    return cols // be * bb


# --------------------------------------------------------------------------------------------
# encoders
# --------------------------------------------------------------------------------------------

def _f16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16)


def _bytes_of(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(torch.uint8)


def quant_q8_0(w: torch.Tensor) -> torch.Tensor:
    """[rows, cols] f32 -> row-split Q8_0 bytes [rows, cols*34/32]."""
    rows, cols = w.shape
    b = w.reshape(rows, cols // 32, 32).float()
    d16 = _f16(b.abs().amax(-1) / 127.0)
    d = d16.float().unsqueeze(-1)
    q = torch.where(d > 0, torch.round(b / torch.where(d > 0, d, torch.ones_like(d))), torch.zeros_like(b))
    q = q.clamp_(-127, 127).to(torch.int8)
    return torch.cat([_bytes_of(q.reshape(rows, cols)), _bytes_of(d16).reshape(rows, cols // 16)], dim=1)


def _pack_scale_min(sc: torch.Tensor, mn: torch.Tensor) -> torch.Tensor:
    """8 six-bit scales + 8 six-bit mins -> the 12 bytes get_scale_min_k4 reads
    (tools/qwen35_engine.c:66-72)."""
    sc = sc.to(torch.int32)
    mn = mn.to(torch.int32)
    b0 = (sc[..., 0:4] & 63) | ((sc[..., 4:8] >> 4) << 6)
    b1 = (mn[..., 0:4] & 63) | ((mn[..., 4:8] >> 4) << 6)
    b2 = (sc[..., 4:8] & 15) | ((mn[..., 4:8] & 15) << 4)
    return torch.cat([b0, b1, b2], dim=-1).to(torch.uint8)


def _kquant_minmax(w: torch.Tensor, levels: int):
    """Shared front end of Q4_K / Q5_K: per 32-value sub-block an affine grid
    value = d*sc*q - dmin*m, q in [0, levels], sc and m six-bit."""
    rows, cols = w.shape
    b = w.reshape(rows, cols // 256, 8, 32).float()
    lo = b.amin(-1).clamp(max=0.0)
    hi = b.amax(-1).clamp(min=0.0)
    scale = (hi - lo) / float(levels)
    mval = -lo
    d16 = _f16(scale.amax(-1) / 63.0)
    m16 = _f16(mval.amax(-1) / 63.0)
    d = d16.float().unsqueeze(-1)
    dm = m16.float().unsqueeze(-1)
    one = torch.ones_like(d)
    sc = torch.where(d > 0, torch.round(scale / torch.where(d > 0, d, one)), torch.zeros_like(scale)).clamp_(0, 63)
    mn = torch.where(dm > 0, torch.round(mval / torch.where(dm > 0, dm, one)), torch.zeros_like(mval)).clamp_(0, 63)
    eff = (d * sc).unsqueeze(-1)
    off = (dm * mn).unsqueeze(-1)
    q = torch.where(eff > 0, torch.round((b + off) / torch.where(eff > 0, eff, torch.ones_like(eff))), torch.zeros_like(b))
    q = q.clamp_(0, levels).to(torch.uint8)
    return d16, m16, sc, mn, q


def quant_q4_k(w: torch.Tensor) -> torch.Tensor:
    """[rows, cols] f32 -> Q4_K bytes [rows, cols/256*144]."""
    rows, cols = w.shape
    d16, m16, sc, mn, q = _kquant_minmax(w, 15)
    nsb = cols // 256
    q = q.reshape(rows, nsb, 4, 2, 32)
    qs = (q[..., 0, :] | (q[..., 1, :] << 4)).reshape(rows, nsb, 128)
    blk = torch.cat([_bytes_of(d16).reshape(rows, nsb, 2), _bytes_of(m16).reshape(rows, nsb, 2),
                     _pack_scale_min(sc, mn), qs], dim=-1)
    return blk.reshape(rows, nsb * 144)


def quant_q5_k(w: torch.Tensor) -> torch.Tensor:
    """[rows, cols] f32 -> Q5_K bytes [rows, cols/256*176]."""
    rows, cols = w.shape
    d16, m16, sc, mn, q = _kquant_minmax(w, 31)
    nsb = cols // 256
    q = q.reshape(rows, nsb, 4, 2, 32)
    nib = q & 15
    hb = (q >> 4).to(torch.int32)
    qs = (nib[..., 0, :] | (nib[..., 1, :] << 4)).reshape(rows, nsb, 128)
    qh = torch.zeros(rows, nsb, 32, dtype=torch.int32, device=w.device)
    for g in range(4):
        qh |= hb[:, :, g, 0, :] << (2 * g)
        qh |= hb[:, :, g, 1, :] << (2 * g + 1)
    blk = torch.cat([_bytes_of(d16).reshape(rows, nsb, 2), _bytes_of(m16).reshape(rows, nsb, 2),
                     _pack_scale_min(sc, mn), qh.to(torch.uint8), qs], dim=-1)
    return blk.reshape(rows, nsb * 176)


def quant_q6_k(w: torch.Tensor) -> torch.Tensor:
    """[rows, cols] f32 -> Q6_K bytes [rows, cols/256*210]."""
    rows, cols = w.shape
    nsb = cols // 256
    b = w.reshape(rows, nsb, 16, 16).float()
    amax = b.abs().amax(-1)
    scale = amax / 31.0
    d16 = _f16(scale.amax(-1) / 127.0)
    d = d16.float().unsqueeze(-1)
    sc = torch.where(d > 0, torch.round(scale / torch.where(d > 0, d, torch.ones_like(d))), torch.zeros_like(scale)).clamp_(0, 127)
    eff = (d * sc).unsqueeze(-1)
    q = torch.where(eff > 0, torch.round(b / torch.where(eff > 0, eff, torch.ones_like(eff))), torch.zeros_like(b))
    code = (q.clamp_(-32, 31) + 32).to(torch.uint8).reshape(rows, nsb, 2, 4, 32)  # [half][quarter][l]
    nib = code & 15
    hi2 = (code >> 4).to(torch.int32)
    ql = torch.empty(rows, nsb, 2, 2, 32, dtype=torch.uint8, device=w.device)
    ql[:, :, :, 0, :] = nib[:, :, :, 0, :] | (nib[:, :, :, 2, :] << 4)
    ql[:, :, :, 1, :] = nib[:, :, :, 1, :] | (nib[:, :, :, 3, :] << 4)
    qh = hi2[:, :, :, 0, :] | (hi2[:, :, :, 1, :] << 2) | (hi2[:, :, :, 2, :] << 4) | (hi2[:, :, :, 3, :] << 6)
    blk = torch.cat([ql.reshape(rows, nsb, 128), qh.to(torch.uint8).reshape(rows, nsb, 64),
                     _bytes_of(sc.to(torch.int8)).reshape(rows, nsb, 16), _bytes_of(d16).reshape(rows, nsb, 2)], dim=-1)
    return blk.reshape(rows, nsb * 210)


QUANT: Dict[str, Callable[[torch.Tensor], torch.Tensor]] = {
    "Q8_0": quant_q8_0, "Q4_K": quant_q4_k, "Q5_K": quant_q5_k, "Q6_K": quant_q6_k,
    "F32": lambda w: _bytes_of(w.float()).reshape(w.shape[0], -1),
}


# --------------------------------------------------------------------------------------------
# plain torch decoders (host logic for tests; NOT the oracle, which is C)
# --------------------------------------------------------------------------------------------

def _scale_min_unpack(sc12: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    q = sc12.to(torch.int32)
    sc = torch.cat([q[..., 0:4] & 63, (q[..., 8:12] & 15) | ((q[..., 0:4] >> 6) << 4)], dim=-1)
    mn = torch.cat([q[..., 4:8] & 63, (q[..., 8:12] >> 4) | ((q[..., 4:8] >> 6) << 4)], dim=-1)
    return sc, mn


def dequant(ty: str, raw: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """Stored bytes -> f32 [rows, cols], op for op as tools/qwen35_engine.c:233-307 (one rounding
    per product, one per subtraction; torch f32 arithmetic is IEEE so the bits agree)."""
    raw = raw.reshape(rows, -1)
    if ty == "F32":
        return raw.view(torch.float32).reshape(rows, cols).clone()
    if ty == "Q8_0":
        q = raw[:, :cols].view(torch.int8).float().reshape(rows, cols // 32, 32)
        d = raw[:, cols:].contiguous().view(torch.float16).float().reshape(rows, cols // 32, 1)
        return (q * d).reshape(rows, cols)
    nsb = cols // 256
    if ty in ("Q4_K", "Q5_K"):
        bb = 144 if ty == "Q4_K" else 176
        blk = raw.reshape(rows, nsb, bb)
        d = blk[..., 0:2].contiguous().view(torch.float16).float()
        dm = blk[..., 2:4].contiguous().view(torch.float16).float()
        sc, mn = _scale_min_unpack(blk[..., 4:16])
        qs = blk[..., bb - 128:].reshape(rows, nsb, 4, 32)
        q = torch.stack([qs & 15, qs >> 4], dim=3).to(torch.int32)  # [r, sb, g, parity, l]
        if ty == "Q5_K":
            qh = blk[..., 16:48].to(torch.int32)
            for g in range(4):
                q[:, :, g, 0, :] += ((qh >> (2 * g)) & 1) * 16
                q[:, :, g, 1, :] += ((qh >> (2 * g + 1)) & 1) * 16
        d1 = (d * sc.float()).reshape(rows, nsb, 4, 2, 1)
        m1 = (dm * mn.float()).reshape(rows, nsb, 4, 2, 1)
        return (d1 * q.float() - m1).reshape(rows, cols)
    if ty == "Q6_K":
        blk = raw.reshape(rows, nsb, 210)
        ql = blk[..., 0:128].reshape(rows, nsb, 2, 2, 32).to(torch.int32)
        qh = blk[..., 128:192].reshape(rows, nsb, 2, 32).to(torch.int32)
        sc = blk[..., 192:208].contiguous().view(torch.int8).float().reshape(rows, nsb, 2, 4, 2, 1)
        d = blk[..., 208:210].contiguous().view(torch.float16).float().reshape(rows, nsb, 1, 1, 1, 1)
        code = torch.empty(rows, nsb, 2, 4, 32, dtype=torch.int32, device=raw.device)
        for qd in range(4):
            nib = (ql[:, :, :, qd & 1, :] & 15) if qd < 2 else (ql[:, :, :, qd & 1, :] >> 4)
            code[:, :, :, qd, :] = (nib | (((qh >> (2 * qd)) & 3) << 4)) - 32
        return ((d * sc) * code.reshape(rows, nsb, 2, 4, 2, 16).float()).reshape(rows, cols)
    raise ValueError(ty)


# --------------------------------------------------------------------------------------------
# model configs
# --------------------------------------------------------------------------------------------

@dataclasses.dataclass
class ModelCfg:
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    d_ff: int
    vocab_size: int
    ssm_heads: int            # value heads (ssm_time_step_rank, TR)
    ssm_groups: int           # q/k groups (ssm_group_count, GK)
    ssm_state: int = 128
    conv_kernel: int = 4
    interval: int = 4
    rope_dim: int = 64
    rope_base: float = 1.0e7
    eps: float = 1.0e-6
    tied_head: bool = True
    quant: str = "q8_0"       # q8_0 | q4_k_m | q4_k_s
    seed: int = 0
    name: str = "synthetic"
    # routed-expert FFN (qwen35moe; host/llb_host.c:622-724): 0 experts = the dense FFN of d_ff columns
    n_experts: int = 0
    n_experts_used: int = 0
    d_expert: int = 0         # expert_feed_forward_length
    d_shared: int = 0         # expert_shared_feed_forward_length
    # (leaf, type) pairs that overrule the quantisation scheme for one kind of matrix, e.g. (("attn_qkv", "Q5_K"),):
    # llama.cpp's Q4_K_M files keep some matrices in a format of their own, which changes how launches group
    type_overrides: tuple = ()
    # multiplies the draws of the matrices that write into the residual stream (attn_output, ssm_out, ffn_down).  1.0 is
    # what the benchmark configurations specify.  A small gain leaves a model whose next token depends mostly on the
    # current one, so greedy output soon repeats and both drafters get some drafts right: test packs use it to reach
    # partial acceptance at real layer shapes (with N(0, 0.02) weights at d = 5120 a drafter is right about once in V)
    mix_gain: float = 1.0

    @property
    def kdc(self): return self.ssm_groups * self.ssm_state

    @property
    def vdc(self): return self.ssm_heads * self.ssm_state

    @property
    def convd(self): return 2 * self.kdc + self.vdc

    def is_full(self, il: int) -> bool:
        return (il + 1) % self.interval == 0


def cfg_c0(**kw) -> ModelCfg:
    """0.8B-shape hybrid, Q8_0, tied head (the reference-CPU-runnable configuration)."""
    return ModelCfg(n_layers=24, d_model=1024, n_heads=8, n_kv_heads=2, head_dim=128, d_ff=3584,
                    vocab_size=32768, ssm_heads=8, ssm_groups=8, tied_head=True, quant="q8_0", seed=0,
                    name="c0-0.8b-q8_0", **kw)


def cfg_c2(**kw) -> ModelCfg:
    """27B-shape hybrid, Q4_K_M."""
    a = dict(n_layers=64, d_model=5120, n_heads=24, n_kv_heads=4, head_dim=256, d_ff=17408,
             vocab_size=151936, ssm_heads=48, ssm_groups=16, tied_head=False, quant="q4_k_m", seed=3,
             name="c2-27b-q4_k_m")
    a.update(kw)
    return ModelCfg(**a)


def cfg_c4(**kw) -> ModelCfg:
    """9B-shape hybrid, Q8_0 (long-context configuration)."""
    a = dict(n_layers=32, d_model=4096, n_heads=16, n_kv_heads=4, head_dim=256, d_ff=12288,
             vocab_size=151936, ssm_heads=32, ssm_groups=16, tied_head=False, quant="q8_0", seed=5,
             name="c4-9b-q8_0")
    a.update(kw)
    return ModelCfg(**a)


def cfg_long(**kw) -> ModelCfg:
    """The long-context configuration's attention shape (16 Q / 4 KV heads of 256, 32 DeltaNet heads over 16 groups,
    Q8_0) on a narrow residual (d 1024, FFN 1024, four layers, 2048-entry vocabulary), so that the reference CPU engine
    gets through a context of more than 8192 positions in minutes."""
    a = dict(n_layers=4, d_model=1024, n_heads=16, n_kv_heads=4, head_dim=256, d_ff=1024, vocab_size=2048, ssm_heads=32,
             ssm_groups=16, tied_head=False, quant="q8_0", seed=6, name="long-context-q8_0")
    a.update(kw)
    return ModelCfg(**a)


def cfg_c3(**kw) -> ModelCfg:
    """MoE hybrid (35B-A3B shape): 256 experts, top 8 plus a shared expert, Q4_K_S."""
    a = dict(n_layers=40, d_model=2048, n_heads=16, n_kv_heads=2, head_dim=256, d_ff=512,
             vocab_size=151936, ssm_heads=32, ssm_groups=16, tied_head=False, quant="q4_k_s", seed=4,
             name="c3-moe-q4_k_s", n_experts=256, n_experts_used=8, d_expert=512, d_shared=512)
    a.update(kw)
    return ModelCfg(**a)


def cfg_tiny_moe(**kw) -> ModelCfg:
    """cfg_tiny with a routed-expert FFN: 8 experts, top 2, plus the shared expert."""
    a = dict(quant="q4_k_s", seed=13, name="tiny-moe", d_ff=256, n_experts=8, n_experts_used=2, d_expert=256,
             d_shared=256)
    a.update(kw)
    return cfg_tiny(**a)


def cfg_tiny(**kw) -> ModelCfg:
    """A few-MB model with every structural feature (GQA, head tiling hh % GK with rep 2,
    partial rope, both layer kinds); used by the fast parity tests."""
    a = dict(n_layers=4, d_model=256, n_heads=4, n_kv_heads=2, head_dim=128, d_ff=512,
             vocab_size=1024, ssm_heads=4, ssm_groups=2, tied_head=True, quant="q8_0", seed=11, name="tiny")
    a.update(kw)
    return ModelCfg(**a)


def _more_bits(il: int, n: int) -> bool:
    return il < n // 8 or il >= 7 * n // 8 or (il - n // 8) % 3 == 2


def tensor_type(cfg: ModelCfg, name: str) -> str:
    """Per-tensor storage type of the synthetic packs.
    q8_0   : every matrix Q8_0.
    q4_k_m : Q4_K, except Q6_K for output.weight and for attn_v / ffn_down in the
             first and last eighth of the layers and every third layer between.
    q4_k_s : Q4_K, except Q6_K for output.weight and Q5_K for attn_v / ffn_down in the first
             eighth of the layers."""
    if name.endswith("norm.weight") or name.endswith("ssm_a") or name.endswith("ssm_dt.bias") \
            or name.endswith("ssm_conv1d.weight") or "ffn_gate_inp" in name:
        return "F32"
    if cfg.quant == "q8_0":
        return "Q8_0"
    il = int(name.split(".")[1]) if name.startswith("blk.") else -1
    leaf = name.split(".")[-2] if name.endswith(".weight") else name
    if leaf.endswith("_exps") or leaf.endswith("_shexp"):   # ffn_down_exps / ffn_down_shexp follow ffn_down's rule
        leaf = leaf.rsplit("_", 1)[0]
    for lf, ty in cfg.type_overrides:
        if lf == leaf:
            return ty
    if name == "output.weight":
        return "Q6_K"
    if cfg.quant == "q4_k_m":
        if leaf in ("attn_v", "ffn_down") and _more_bits(il, cfg.n_layers):
            return "Q6_K"
        return "Q4_K"
    if cfg.quant == "q4_k_s":
        if leaf in ("attn_v", "ffn_down") and il < cfg.n_layers // 8:
            return "Q5_K"
        return "Q4_K"
    raise ValueError(cfg.quant)


def tensor_plan(cfg: ModelCfg) -> List[Tuple[str, int, int]]:
    """(name, rows, cols) in pack order; vectors have rows == 1.  Names and shapes are the ones
    tools/qwen35_engine.c:581-761 looks up."""
    d, hd = cfg.d_model, cfg.head_dim
    qa, kv = cfg.n_heads * hd, cfg.n_kv_heads * hd
    plan = [("token_embd.weight", cfg.vocab_size, d)]
    for il in range(cfg.n_layers):
        p = f"blk.{il}."
        plan.append((p + "attn_norm.weight", 1, d))
        if cfg.is_full(il):
            plan += [(p + "attn_q.weight", 2 * qa, d), (p + "attn_k.weight", kv, d), (p + "attn_v.weight", kv, d),
                     (p + "attn_q_norm.weight", 1, hd), (p + "attn_k_norm.weight", 1, hd),
                     (p + "attn_output.weight", d, qa)]
        else:
            plan += [(p + "attn_qkv.weight", cfg.convd, d), (p + "attn_gate.weight", cfg.vdc, d),
                     (p + "ssm_beta.weight", cfg.ssm_heads, d), (p + "ssm_alpha.weight", cfg.ssm_heads, d),
                     (p + "ssm_dt.bias", 1, cfg.ssm_heads), (p + "ssm_a", 1, cfg.ssm_heads),
                     (p + "ssm_conv1d.weight", cfg.convd, cfg.conv_kernel), (p + "ssm_norm.weight", 1, cfg.ssm_state),
                     (p + "ssm_out.weight", d, cfg.vdc)]
        plan.append((p + "post_attention_norm.weight", 1, d))
        if cfg.n_experts:
            # the expert stacks are [expert][row] flattened over their first two dimensions (GGUF names,
            # reports/cuda-moe/scripts/gen_moe.py:104-113)
            ne, ef, sf = cfg.n_experts, cfg.d_expert, cfg.d_shared
            plan += [(p + "ffn_gate_inp.weight", ne, d), (p + "ffn_gate_inp_shexp.weight", 1, d),
                     (p + "ffn_gate_exps.weight", ne * ef, d), (p + "ffn_up_exps.weight", ne * ef, d),
                     (p + "ffn_down_exps.weight", ne * d, ef), (p + "ffn_gate_shexp.weight", sf, d),
                     (p + "ffn_up_shexp.weight", sf, d), (p + "ffn_down_shexp.weight", d, sf)]
        else:
            plan += [(p + "ffn_gate.weight", cfg.d_ff, d), (p + "ffn_up.weight", cfg.d_ff, d),
                     (p + "ffn_down.weight", d, cfg.d_ff)]
    plan.append(("output_norm.weight", 1, d))
    if not cfg.tied_head:
        plan.append(("output.weight", cfg.vocab_size, d))
    return plan


class _Rng:
    """numpy Generator on the CPU (platform-stable bits for the committed goldens), torch's CUDA
    generator on the GPU (27B-shape packs are drawn and quantised where they stay)."""

    def __init__(self, seed: int, device: torch.device):
        self.device = device
        if device.type == "cuda":
            self.g = torch.Generator(device=device)
            self.g.manual_seed(seed)
        else:
            self.g = np.random.default_rng(seed)

    def normal(self, rows: int, cols: int, std: float) -> torch.Tensor:
        if self.device.type == "cuda":
            return torch.randn(rows, cols, generator=self.g, device=self.device, dtype=torch.float32) * std
        return torch.from_numpy(self.g.standard_normal((rows, cols), dtype=np.float32) * np.float32(std))


def draw_tensor(cfg: ModelCfg, name: str, rows: int, cols: int, rng: _Rng) -> torch.Tensor:
    """Synthetic values: matrices N(0, 0.02); norm weights 1; ssm_a = -exp(0.5 z) (negative, as the
    reference's synthetic models draw it, reports/cuda-moe/scripts/gen_moe.py:131-132);
    ssm_dt.bias N(0, 0.5); conv taps N(0, 0.5)."""
    if name.endswith("norm.weight"):
        return torch.ones(rows, cols, device=rng.device)
    if name.endswith("ssm_a"):
        return -torch.exp(rng.normal(rows, cols, 0.5))
    if name.endswith("ssm_dt.bias") or name.endswith("ssm_conv1d.weight"):
        return rng.normal(rows, cols, 0.5)
    w = rng.normal(rows, cols, 0.02)
    if cfg.mix_gain != 1.0 and name.split(".")[-2] in ("attn_output", "ssm_out", "ffn_down", "ffn_down_exps", "ffn_down_shexp"):
        w = w * cfg.mix_gain
    return w


@dataclasses.dataclass
class TensorEntry:
    name: str
    off: int
    nbytes: int
    rows: int
    cols: int
    ty: str

    @property
    def row_bytes(self): return 0 if self.ty == "F32" else row_bytes(self.ty, self.cols)


class Pack:
    """A model pack held in one uint8 tensor (CPU or CUDA) plus its index."""

    def __init__(self, cfg: ModelCfg, data: torch.Tensor, entries: List[TensorEntry]):
        self.cfg, self.data, self.entries = cfg, data, entries
        self.by_name = {e.name: e for e in entries}

    def raw(self, name: str) -> torch.Tensor:
        e = self.by_name[name]
        return self.data[e.off:e.off + e.nbytes]

    def dequant(self, name: str) -> torch.Tensor:
        e = self.by_name[name]
        return dequant(e.ty, self.raw(name), e.rows, e.cols)

    def index_text(self) -> str:
        c = self.cfg
        kv = [("n_layers", c.n_layers), ("n_heads", c.n_heads), ("n_kv_heads", c.n_kv_heads), ("d_model", c.d_model),
              ("head_dim", c.head_dim), ("d_ff", c.d_ff), ("vocab_size", c.vocab_size),
              ("full_attention_interval", c.interval), ("ssm_conv_kernel", c.conv_kernel),
              ("ssm_state_size", c.ssm_state), ("ssm_group_count", c.ssm_groups), ("ssm_time_step_rank", c.ssm_heads),
              ("ssm_inner_size", c.vdc), ("linear_key_dim", c.kdc), ("linear_value_head_dim", c.ssm_state),
              ("linear_conv_dim", c.convd), ("rope_dim", c.rope_dim), ("rope_freq_base", repr(float(c.rope_base))),
              ("rms_norm_eps", repr(float(c.eps)))]
        if c.n_experts:
            kv += [("expert_count", c.n_experts), ("expert_used_count", c.n_experts_used),
                   ("expert_feed_forward_length", c.d_expert), ("expert_shared_feed_forward_length", c.d_shared)]
        lines = [f"#cfg\t{k}\t{v}" for k, v in kv]
        lines.append(f"# pack_bytes\t{self.data.numel()}")
        lines.append("# name\toffset\tbytes\trows\tcols\tsrc_type\trow_bytes\tfmt")
        for e in self.entries:
            lines.append(f"{e.name}\t{e.off}\t{e.nbytes}\t{e.rows}\t{e.cols}\t{e.ty}\t{e.row_bytes}\t{FMT[e.ty]}")
        return "\n".join(lines) + "\n"

    def write(self, out_dir: str) -> str:
        os.makedirs(out_dir, exist_ok=True)
        self.data.cpu().numpy().tofile(os.path.join(out_dir, "pack.bin"))
        with open(os.path.join(out_dir, "index.tsv"), "w") as f:
            f.write(self.index_text())
        return out_dir

    @staticmethod
    def read(out_dir: str, cfg: ModelCfg, device="cpu") -> "Pack":
        entries = []
        for line in open(os.path.join(out_dir, "index.tsv")):
            if line.startswith("#") or not line.strip():
                continue
            n, off, nb, rows, cols, ty = line.rstrip("\n").split("\t")[:6]
            entries.append(TensorEntry(n, int(off), int(nb), int(rows), int(cols), ty))
        data = torch.from_numpy(np.fromfile(os.path.join(out_dir, "pack.bin"), dtype=np.uint8)).to(device)
        return Pack(cfg, data, entries)


def build_pack(cfg: ModelCfg, device: str | torch.device = "cpu", layers: Optional[int] = None) -> Pack:
    """Draw and quantise every tensor of `cfg` in pack order.  `layers` truncates the model (the
    draws of the kept tensors do not change: the generator is advanced in full pack order only on the
    CPU path when the truncated tensors come last, so truncation is by dropping trailing layers)."""
    device = torch.device(device)
    rng = _Rng(cfg.seed, device)
    plan = tensor_plan(cfg)
    full = cfg
    if layers is not None and layers < cfg.n_layers:
        keep = lambda n: (not n.startswith("blk.")) or int(n.split(".")[1]) < layers
        cfg = dataclasses.replace(cfg, n_layers=layers)
    else:
        keep = lambda n: True
    sizes, off = [], 0
    for name, rows, cols in plan:
        ty = tensor_type(full, name)
        nb = rows * (cols * 4 if ty == "F32" else row_bytes(ty, cols))
        if keep(name):
            sizes.append((name, rows, cols, ty, off, nb))
            off = (off + nb + 63) // 64 * 64
    data = torch.zeros(off, dtype=torch.uint8, device=device)
    entries = []
    kept = {s[0]: s for s in sizes}
    for name, rows, cols in plan:
        w = draw_tensor(cfg, name, rows, cols, rng)   # always drawn: keeps the stream position
        if name not in kept:
            continue
        _, _, _, ty, o, nb = kept[name]
        data[o:o + nb] = QUANT[ty](w).reshape(-1)
        entries.append(TensorEntry(name, o, nb, rows, cols, ty))
        del w
    if cfg.tied_head:
        e = entries[0]
        entries.append(TensorEntry("output.weight", e.off, e.nbytes, e.rows, e.cols, e.ty))
    return Pack(cfg, data, entries)


# --------------------------------------------------------------------------------------------
# MTP drafter container
# --------------------------------------------------------------------------------------------

MTP_ORDER = ["nextn.enorm", "nextn.hnorm", "nextn.eh_proj", "attn_norm", "attn_q", "attn_k", "attn_v",
             "attn_q_norm", "attn_k_norm", "attn_output", "post_attention_norm", "ffn_gate", "ffn_up",
             "ffn_down", "nextn.shared_head_norm", "mtp.head_slice", "mtp.ids"]  # tools/mtp27/mtp_pack.py:14-30


def build_mtp(pack: Pack, draft_vocab: Optional[int] = None, eh: str = "hidden",
              draft_ids: Optional[np.ndarray] = None) -> List[Tuple[str, str, Tuple[int, int], torch.Tensor]]:
    """The synthetic drafter BASELINE config 0 describes: one NextN layer whose attention + FFN block is
    a byte copy of the trunk's last full-attention layer, norms 1, and the trunk head.  eh_proj is not
    specified by the configuration; it is fixed here to [0 | I] (x = rms(h)*hnorm; eh = "hidden"), stored in the
    block's matrix format; eh = "embed" gives [I | 0] (x = rms(e)*enorm: the drafter then sees the token it follows,
    which is what predicts the next one in a model built with a small mix_gain).
    Head slice: the first `draft_vocab` rows of output.weight (all rows by default) with ids 0..n-1, or, with
    `draft_ids` (sorted or not, a multiple of 16 of them), the rows of exactly those vocabulary entries in that order
    -- the draft-vocabulary slice of tools/mtp27/mtp_pack.py:14-30, whose argmax is mapped back through the ids."""
    cfg = pack.cfg
    il = max(i for i in range(cfg.n_layers) if cfg.is_full(i))
    d = cfg.d_model
    dev = pack.data.device
    ones = lambda n: _bytes_of(torch.ones(n, device=dev))
    mat_ty = pack.by_name[f"blk.{il}.ffn_gate.weight"].ty
    assert eh in ("hidden", "embed")
    halves = [torch.zeros(d, d, device=dev), torch.eye(d, device=dev)]
    eh = torch.cat(halves if eh == "hidden" else halves[::-1], dim=1)
    out: List[Tuple[str, str, Tuple[int, int], torch.Tensor]] = []
    for n in MTP_ORDER[:15]:
        if n in ("nextn.enorm", "nextn.hnorm", "nextn.shared_head_norm"):
            out.append((n, "F32", (1, d), ones(d)))
        elif n == "nextn.eh_proj":
            out.append((n, mat_ty, (d, 2 * d), QUANT[mat_ty](eh).reshape(-1)))
        else:
            e = pack.by_name[f"blk.{il}.{n}.weight"]
            out.append((n, e.ty, (e.rows, e.cols), pack.raw(e.name).clone()))
    h = pack.by_name["output.weight"]
    if draft_ids is not None:
        ids = torch.as_tensor(np.asarray(draft_ids, dtype=np.int64), device=dev)
        nv = int(ids.numel())
        assert nv % 16 == 0 and int(ids.min()) >= 0 and int(ids.max()) < h.rows
        rows = pack.raw("output.weight").reshape(h.rows, h.row_bytes)[ids].reshape(-1).clone()
        out.append(("mtp.head_slice", h.ty, (nv, h.cols), rows))
        out.append(("mtp.ids", "U32", (1, nv), _bytes_of(ids.to(torch.int32))))
        return out
    nv = h.rows if draft_vocab is None else draft_vocab
    assert nv % 16 == 0
    out.append(("mtp.head_slice", h.ty, (nv, h.cols), pack.raw("output.weight")[: nv * h.row_bytes].clone()))
    out.append(("mtp.ids", "U32", (1, nv), _bytes_of(torch.arange(nv, dtype=torch.int32, device=dev))))
    return out


def aux1_bytes(entries) -> bytes:
    """Serialise named entries as the reference's AUX1 container (tools/auxpack/auxpack.py:10-22)."""
    a256 = lambda x: (x + 255) // 256 * 256
    off = a256(16 + 72 * len(entries))
    head = b"AUX1" + struct.pack("<III", 1, len(entries), 0)
    tab, blobs = b"", []
    for name, ty, (rows, cols), raw in entries:
        nb = raw.numel()
        rank = 1 if rows == 1 else 2
        ne = [cols, rows if rank == 2 else 0, 0, 0]
        tab += struct.pack("<32sII4IQQ", name.encode(), AUX_DT[ty], rank, *ne, off, nb)
        blobs.append((off, raw))
        off = a256(off + nb)
    buf = bytearray(off)
    buf[: 16] = head
    buf[16: 16 + len(tab)] = tab
    for o, raw in blobs:
        buf[o: o + raw.numel()] = raw.cpu().numpy().tobytes()
    return bytes(buf)


def mtp1_bytes(entries) -> bytes:
    """Positional MTP1 container (tools/mtp27/mtp_pack.py:51-62): "MTP1", u32 N, N x (u64 off, u64 bytes)."""
    a256 = lambda x: (x + 255) // 256 * 256
    off = a256(8 + 16 * len(entries))
    tab, blobs = b"", []
    for _, _, _, raw in entries:
        tab += struct.pack("<QQ", off, raw.numel())
        blobs.append((off, raw))
        off = a256(off + raw.numel())
    buf = bytearray(off)
    buf[:8] = b"MTP1" + struct.pack("<I", len(entries))
    buf[8: 8 + len(tab)] = tab
    for o, raw in blobs:
        buf[o: o + raw.numel()] = raw.cpu().numpy().tobytes()
    return bytes(buf)


def synth_prompt(seed: int, n: int, vocab: int) -> np.ndarray:
    """Prompt ids uniform in [0, vocab) from numpy's default_rng(seed)."""
    return np.random.default_rng(seed).integers(0, vocab, size=n, dtype=np.int64).astype(np.int32)


def q4k_random_blocks(rows: int, cols: int, seed: int = 2, device="cpu") -> torch.Tensor:
    """The isolated GEMM sweep's weights: Q4_K super-blocks built directly -- nibbles uniform 0..15,
    six-bit scales and mins uniform 0..63, f16 d and dmin ~ |N(0, 0.01)|."""
    device = torch.device(device)
    nsb = cols // 256
    if device.type == "cuda":
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        qs = torch.randint(0, 256, (rows, nsb, 128), generator=g, device=device, dtype=torch.uint8)
        sc = torch.randint(0, 64, (rows, nsb, 8), generator=g, device=device)
        mn = torch.randint(0, 64, (rows, nsb, 8), generator=g, device=device)
        dd = (torch.randn(rows, nsb, 2, generator=g, device=device) * 0.01).abs()
    else:
        g = np.random.default_rng(seed)
        qs = torch.from_numpy(g.integers(0, 256, (rows, nsb, 128), dtype=np.uint8))
        sc = torch.from_numpy(g.integers(0, 64, (rows, nsb, 8)))
        mn = torch.from_numpy(g.integers(0, 64, (rows, nsb, 8)))
        dd = torch.from_numpy(np.abs(g.standard_normal((rows, nsb, 2), dtype=np.float32) * np.float32(0.01)))
    blk = torch.cat([_bytes_of(_f16(dd)).reshape(rows, nsb, 4), _pack_scale_min(sc, mn), qs], dim=-1)
    return blk.reshape(rows, nsb * 144)


# --------------------------------------------------------------------------------------------
# a pack written as a GGUF file (what llb_spec_open_gguf reads)
# --------------------------------------------------------------------------------------------

def write_gguf(pack: Pack, path: str, fused_gate_up: bool = False, nextn: int = 0, mtp_entries=None) -> str:
    """Write `pack` as a GGUF file of architecture qwen35 / qwen35moe with the metadata keys the reference reads
    (tools/gguf2pack.c:541-600) and the pack's quantised bytes: K-quants and F32 verbatim, Q8_0 re-sliced from the
    pack's row-split rows to GGUF's [f16 d][32 x int8] blocks, expert stacks as 3-D tensors (optionally gate and
    up fused into ffn_gate_up_exps, [expert][gate rows | up rows]).  A tied head is written as no output.weight.
    `nextn` only adds the key nextn_predict_layers and that many to block_count (no tensors), to exercise the
    reader's trunk-length rule; `mtp_entries` (build_mtp's list) writes the drafter as the file's nextn block
    blk.<n_layers>.* (its 15 block tensors; the head is the file's own output.weight) and sets nextn = 1.
    Needs the gguf Python package."""
    from gguf import GGUFWriter, GGMLQuantizationType as Q
    c = pack.cfg
    if mtp_entries is not None:
        nextn = 1
    arch = "qwen35moe" if c.n_experts else "qwen35"
    w = GGUFWriter(path, arch)
    w.add_uint32(f"{arch}.block_count", c.n_layers + nextn)
    if nextn:
        w.add_uint32(f"{arch}.nextn_predict_layers", nextn)
    w.add_uint32(f"{arch}.embedding_length", c.d_model)
    w.add_uint32(f"{arch}.feed_forward_length", c.d_ff)
    w.add_uint32(f"{arch}.attention.head_count", c.n_heads)
    w.add_uint32(f"{arch}.attention.head_count_kv", c.n_kv_heads)
    w.add_uint32(f"{arch}.attention.key_length", c.head_dim)
    w.add_uint32(f"{arch}.attention.value_length", c.head_dim)
    w.add_float32(f"{arch}.attention.layer_norm_rms_epsilon", c.eps)
    w.add_uint32(f"{arch}.rope.dimension_count", c.rope_dim)
    w.add_float32(f"{arch}.rope.freq_base", c.rope_base)
    w.add_uint32(f"{arch}.ssm.conv_kernel", c.conv_kernel)
    w.add_uint32(f"{arch}.ssm.state_size", c.ssm_state)
    w.add_uint32(f"{arch}.ssm.group_count", c.ssm_groups)
    w.add_uint32(f"{arch}.ssm.time_step_rank", c.ssm_heads)
    w.add_uint32(f"{arch}.ssm.inner_size", c.vdc)
    w.add_uint32(f"{arch}.full_attention_interval", c.interval)
    w.add_uint32(f"{arch}.vocab_size", c.vocab_size)
    if c.n_experts:
        w.add_uint32(f"{arch}.expert_count", c.n_experts)
        w.add_uint32(f"{arch}.expert_used_count", c.n_experts_used)
        w.add_uint32(f"{arch}.expert_feed_forward_length", c.d_expert)
        w.add_uint32(f"{arch}.expert_shared_feed_forward_length", c.d_shared)
    qt = {"Q4_K": Q.Q4_K, "Q5_K": Q.Q5_K, "Q6_K": Q.Q6_K, "Q8_0": Q.Q8_0}
    tied = c.tied_head
    todo = []

    def blocked_q8(raw: np.ndarray, rows: int, cols: int) -> np.ndarray:
        nb = cols // 32
        a = raw.reshape(rows, cols + 2 * nb)
        out = np.empty((rows, nb, 34), np.uint8)
        out[:, :, 0:2] = a[:, cols:].reshape(rows, nb, 2)
        out[:, :, 2:] = a[:, :cols].reshape(rows, nb, 32)
        return out.reshape(rows, nb * 34)

    def add(name, e, raw, lead=None):
        """lead: leading dimensions replacing e.rows (expert stacks)."""
        shape_rows = lead if lead is not None else (e.rows,)
        if e.ty == "F32":
            arr = raw.view(np.float32).reshape(*(shape_rows if e.rows > 1 else ()), e.cols)
            w.add_tensor_info(name, arr.shape, np.dtype(np.float32), arr.nbytes)
        else:
            rows = int(np.prod(shape_rows))
            if e.ty == "Q8_0":
                raw = blocked_q8(raw, rows, e.cols)
            arr = raw.reshape(*shape_rows, -1)
            w.add_tensor_info(name, arr.shape, np.dtype(np.uint8), arr.nbytes, raw_dtype=qt[e.ty])
        todo.append(np.ascontiguousarray(arr))

    skip = set()
    for e in pack.entries:
        if e.name in skip or (e.name == "output.weight" and tied):
            continue
        raw = pack.raw(e.name).cpu().numpy()
        if e.name.endswith("ffn_gate_exps.weight") and fused_gate_up:
            up = pack.by_name[e.name.replace("ffn_gate_exps", "ffn_up_exps")]
            ne, ef = c.n_experts, c.d_expert
            g3 = raw.reshape(ne, ef, -1)
            u3 = pack.raw(up.name).cpu().numpy().reshape(ne, ef, -1)
            both = np.concatenate([g3, u3], axis=1).reshape(-1)
            add(e.name.replace("ffn_gate_exps", "ffn_gate_up_exps"), e, both, lead=(ne, 2 * ef))
            skip.add(up.name)
            continue
        if e.name.endswith("_exps.weight"):
            ne = c.n_experts
            add(e.name, e, raw, lead=(ne, e.rows // ne))
            continue
        add(e.name, e, raw)
    for name, ty, (rows, cols), raw in (mtp_entries or [])[:15]:
        add(f"blk.{c.n_layers}.{name}.weight", TensorEntry(name, 0, raw.numel(), rows, cols, ty), raw.cpu().numpy())
    w.write_header_to_file(); w.write_kv_data_to_file(); w.write_ti_data_to_file()
    for arr in todo:
        w.write_tensor_data(arr)
    w.close()
    return path
