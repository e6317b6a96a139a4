"""Number-format codecs (CPU/torch, bit exact): E2M1, E4M3, UE8M0, NVFP4, MXFP8, block FP8.

These are the oracles of the packed formats.  Conventions follow the checkpoint layout
the reference reads (engine/crates/model/src/flash/nvfp4.rs:96-128, mxfp8.rs:4-16,
engine/docs/flash-fp8-math.md:9-45):

* NVFP4: ``weight`` uint8 [out, in/2] (low nibble = even column), ``weight_scale``
  e4m3 [out, in/16], ``weight_scale_2`` fp32 scalar.  value = (e2m1 * e4m3) * global,
  block scale first, tensor scale second.
* block FP8: ``weight`` e4m3 [out, in], ``weight_scale_inv`` fp32 [out/128, in/128];
  activations per token per 128 columns, scale = max|x| / 448.
"""
from __future__ import annotations

import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
E4M3_MAX = 448.0
E2M1_MAX = 6.0


# ------------------------------------------------------------------ E2M1
def e2m1_decode(codes: torch.Tensor) -> torch.Tensor:
    """uint8 codes (0..15, bit 3 = sign) -> fp32."""
    table = torch.tensor(E2M1_VALUES + tuple(-v for v in E2M1_VALUES), dtype=torch.float32,
                         device=codes.device)
    return table[codes.long()]


def e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> nearest E2M1 code, ties to the even code, saturating at 6."""
    mag = x.abs().to(torch.float32)
    # thresholds between neighbours; a tie goes to the code with an even mantissa bit
    # codes: 0:0 1:.5 2:1 3:1.5 4:2 5:3 6:4 7:6 ; even codes are 0,2,4,6
    code = torch.zeros_like(mag, dtype=torch.uint8)
    bounds = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
    for i, b in enumerate(bounds):
        lower_even = (i % 2 == 0)      # lower neighbour code i is even -> tie stays low
        step = (mag > b) if lower_even else (mag >= b)
        code = code + step.to(torch.uint8)
    sign = (torch.signbit(x)).to(torch.uint8) << 3
    return code | sign


# ------------------------------------------------------------------ E4M3 / UE8M0
def e4m3_encode(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> e4m3fn bytes (RNE, saturating to +-448)."""
    return x.to(torch.float32).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)


def e4m3_decode(b: torch.Tensor) -> torch.Tensor:
    return b.view(torch.float8_e4m3fn).to(torch.float32)


def ue8m0_decode(b: torch.Tensor) -> torch.Tensor:
    """uint8 exponent -> 2^(b-127); 255 is NaN."""
    out = torch.pow(torch.tensor(2.0, dtype=torch.float64), b.to(torch.float64) - 127.0).to(torch.float32)
    return torch.where(b == 255, torch.full_like(out, float("nan")), out)


# ------------------------------------------------------------------ NVFP4
def nvfp4_quantize(w: torch.Tensor, group: int = 16):
    """fp32 [out, in] -> (packed uint8 [out, in/2], scale e4m3 bytes [out, in/group], global fp32).

    global = amax / (6 * 448); block scale = e4m3(block_amax / 6 / global);
    code = e2m1(x / (decoded_scale * global)).
    """
    w = w.to(torch.float32)
    out, k = w.shape
    assert k % group == 0 and group % 2 == 0
    amax = w.abs().max().clamp_min(1e-30)
    glob = (amax / (E2M1_MAX * E4M3_MAX)).to(torch.float32)
    blocks = w.view(out, k // group, group)
    bmax = blocks.abs().amax(-1)
    scale_b = e4m3_encode(bmax / E2M1_MAX / glob)
    scale = e4m3_decode(scale_b)
    denom = (scale * glob).unsqueeze(-1)
    q = torch.where(denom > 0, blocks / denom, torch.zeros_like(blocks))
    codes = e2m1_encode(q).view(out, k)
    packed = codes[:, 0::2] | (codes[:, 1::2] << 4)
    return packed.contiguous(), scale_b.contiguous(), glob.reshape(())


def nvfp4_block_values(packed: torch.Tensor, scale_b: torch.Tensor, group: int = 16) -> torch.Tensor:
    """(e2m1 * e4m3) without the tensor scale; exact in bf16 (<= 6 significant bits)."""
    out, half = packed.shape
    codes = torch.empty(out, half * 2, dtype=torch.uint8, device=packed.device)
    codes[:, 0::2] = packed & 0xF
    codes[:, 1::2] = packed >> 4
    vals = e2m1_decode(codes).view(out, -1, group)
    return (vals * e4m3_decode(scale_b).unsqueeze(-1)).view(out, half * 2)


def nvfp4_dequantize(packed, scale_b, glob, group: int = 16) -> torch.Tensor:
    return nvfp4_block_values(packed, scale_b, group) * glob.to(torch.float32)


def nvfp4_quantize_activation(x: torch.Tensor, glob: torch.Tensor, group: int = 16):
    """W4A4 activation quantizer: block max / 6 -> nearest e4m3 scale -> nearest-even codes
    (engine/crates/model/src/flash/activation_nvfp4.rs:5-63)."""
    x = x.to(torch.float32)
    rows, k = x.shape
    blocks = x.view(rows, k // group, group)
    scale_b = e4m3_encode(blocks.abs().amax(-1) / E2M1_MAX / glob)
    scale = e4m3_decode(scale_b)
    denom = (scale * glob).unsqueeze(-1)
    q = torch.where(denom > 0, blocks / denom, torch.zeros_like(blocks))
    codes = e2m1_encode(q).view(rows, k)
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous(), scale_b


# ------------------------------------------------------------------ MXFP8
def mxfp8_dequantize(vals: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """e4m3 bytes [out, in] with a UE8M0 byte per 32 values -> fp32."""
    out, k = vals.shape
    v = e4m3_decode(vals).view(out, k // 32, 32)
    return (v * ue8m0_decode(scales).unsqueeze(-1)).view(out, k)


# ------------------------------------------------------------------ block FP8
def fp8_block_quantize_weight(w: torch.Tensor, block: int = 128):
    """fp32 [out, in] -> (e4m3 bytes [out, in], fp32 scale_inv [ceil(out/b), ceil(in/b)])."""
    w = w.to(torch.float32)
    out, k = w.shape
    ob, kb = -(-out // block), -(-k // block)
    pad = torch.zeros(ob * block, kb * block, dtype=torch.float32)
    pad[:out, :k] = w
    tiles = pad.view(ob, block, kb, block)
    amax = tiles.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (tiles / scale[:, None, :, None]).reshape(ob * block, kb * block)[:out, :k]
    return e4m3_encode(q).contiguous(), scale.contiguous()


def fp8_block_dequantize_weight(q: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    out, k = q.shape
    s = scale.repeat_interleave(block, 0)[:out].repeat_interleave(block, 1)[:, :k]
    return e4m3_decode(q) * s


def fp8_quantize_activation(x: torch.Tensor, group: int = 128):
    """Dynamic per-token 1 x group quantisation: scale = max|x|/448, q = RNE_satfinite(x / max(scale, 1e-12));
    an all-zero group has scale 0 (engine/docs/flash-fp8-math.md:36-45)."""
    x = x.to(torch.float32)
    rows, k = x.shape
    g = x.view(rows, k // group, group)
    scale = g.abs().amax(-1) / E4M3_MAX
    q = g / scale.clamp_min(1e-12).unsqueeze(-1)
    return e4m3_encode(q).view(rows, k), scale


def fp8_dequantize_activation(q: torch.Tensor, scale: torch.Tensor, group: int = 128) -> torch.Tensor:
    rows, k = q.shape
    return (e4m3_decode(q).view(rows, k // group, group) * scale.unsqueeze(-1)).view(rows, k)


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> nearest-even bf16 -> fp32."""
    return x.to(torch.bfloat16).to(torch.float32)
