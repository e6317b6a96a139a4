"""Random-init checkpoints in the served layout (no network, no real weights).

``synth_state_dict`` draws every tensor from N(0, 0.02) with a seeded generator under the
tensor names of the HF Qwen3-Next layout that the reference validates
(engine/crates/model/src/flash/mod.rs:494-612), then quantises the linear layers that the
config's ``quantization_config`` does not ignore.  ``write_checkpoint`` stores it as a
sharded safetensors directory with config, generation config, a byte-level tokenizer and a
sha256 manifest, i.e. everything a real checkpoint directory carries.
"""
from __future__ import annotations

import fnmatch
import json
import os

import torch

from ..config import ModelConfig
from ..quant import codecs
from . import safetensors as st

PREFIX = "model.language_model."


def _layer_names(cfg: ModelConfig, base: str, attention: bool) -> dict:
    """name -> (shape, kind) for one decoder layer; kind 'linear' tensors may be quantised."""
    H, hd = cfg.hidden_size, cfg.head_dim
    out = {
        base + "input_layernorm.weight": ((H,), "norm"),
        base + "post_attention_layernorm.weight": ((H,), "norm"),
    }
    if attention:
        nh, kvh = cfg.num_attention_heads, cfg.num_key_value_heads
        out.update({
            base + "self_attn.q_proj.weight": ((nh * hd * 2, H), "linear"),
            base + "self_attn.k_proj.weight": ((kvh * hd, H), "linear"),
            base + "self_attn.v_proj.weight": ((kvh * hd, H), "linear"),
            base + "self_attn.o_proj.weight": ((H, nh * hd), "linear"),
            base + "self_attn.q_norm.weight": ((hd,), "norm"),
            base + "self_attn.k_norm.weight": ((hd,), "norm"),
        })
    else:
        vh = cfg.linear_num_value_heads
        out.update({
            base + "linear_attn.in_proj_qkv.weight": ((cfg.gdn_conv_dim, H), "linear"),
            base + "linear_attn.in_proj_z.weight": ((cfg.gdn_value_dim, H), "linear"),
            base + "linear_attn.in_proj_a.weight": ((vh, H), "linear"),
            base + "linear_attn.in_proj_b.weight": ((vh, H), "linear"),
            base + "linear_attn.conv1d.weight": ((cfg.gdn_conv_dim, 1, cfg.linear_conv_kernel_dim), "conv"),
            base + "linear_attn.out_proj.weight": ((H, cfg.gdn_value_dim), "linear"),
            base + "linear_attn.A_log": ((vh,), "alog"),
            base + "linear_attn.dt_bias": ((vh,), "bias"),
            base + "linear_attn.norm.weight": ((cfg.linear_value_head_dim,), "norm1"),
        })
    I, S = cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size
    out[base + "mlp.gate.weight"] = ((cfg.num_experts, H), "linear")
    out[base + "mlp.shared_expert_gate.weight"] = ((1, H), "linear")
    for e in range(cfg.num_experts):
        out[base + f"mlp.experts.{e}.gate_proj.weight"] = ((I, H), "linear")
        out[base + f"mlp.experts.{e}.up_proj.weight"] = ((I, H), "linear")
        out[base + f"mlp.experts.{e}.down_proj.weight"] = ((H, I), "linear")
    out[base + "mlp.shared_expert.gate_proj.weight"] = ((S, H), "linear")
    out[base + "mlp.shared_expert.up_proj.weight"] = ((S, H), "linear")
    out[base + "mlp.shared_expert.down_proj.weight"] = ((H, S), "linear")
    return out


def tensor_inventory(cfg: ModelConfig) -> dict:
    """Every tensor of an unquantised checkpoint: name -> (shape, kind)."""
    H = cfg.hidden_size
    inv = {PREFIX + "embed_tokens.weight": ((cfg.vocab_size, H), "embed"),
           PREFIX + "norm.weight": ((H,), "norm"),
           "lm_head.weight": ((cfg.vocab_size, H), "linear")}
    for i in range(cfg.num_hidden_layers):
        inv.update(_layer_names(cfg, f"{PREFIX}layers.{i}.", cfg.is_attention_layer(i)))
    for i in range(cfg.mtp_num_hidden_layers):
        inv.update(_layer_names(cfg, f"mtp.layers.{i}.", True))
    if cfg.mtp_num_hidden_layers:
        inv.update({"mtp.fc_embedding.weight": ((H, H), "linear"), "mtp.fc_hidden.weight": ((H, H), "linear"),
                    "mtp.pre_fc_norm_embedding.weight": ((H,), "norm"), "mtp.pre_fc_norm_hidden.weight": ((H,), "norm"),
                    "mtp.norm.weight": ((H,), "norm")})
    return inv


def is_quantized(cfg: ModelConfig, name: str, kind: str) -> bool:
    if cfg.quant.method == "none" or kind != "linear":
        return False
    module = name[:-len(".weight")] if name.endswith(".weight") else name
    return not any(fnmatch.fnmatch(module, pat) or fnmatch.fnmatch(module, "*" + pat) for pat in cfg.quant.ignore)


def synth_state_dict(cfg: ModelConfig, seed: int = 0, dtype: torch.dtype = torch.float32) -> dict:
    """Seeded N(0, 0.02) weights (norm weights N(0,0.02) around their neutral value, A_log/dt_bias
    in the usual GDN ranges), quantised per cfg.quant."""
    gen = torch.Generator().manual_seed(seed)
    sd = {}
    for name, (shape, kind) in tensor_inventory(cfg).items():
        if kind == "norm":          # (1 + w) norms: w near zero
            t = torch.randn(shape, generator=gen) * 0.02
        elif kind == "norm1":       # plain-weight norm: w near one
            t = 1.0 + torch.randn(shape, generator=gen) * 0.02
        elif kind == "alog":        # A in [1, 16] as in GDN initialisation
            t = torch.log(1.0 + 15.0 * torch.rand(shape, generator=gen))
        elif kind == "bias":
            t = torch.randn(shape, generator=gen) * 0.5
        elif kind == "conv":
            t = torch.randn(shape, generator=gen) * 0.3
        else:
            t = torch.randn(shape, generator=gen) * 0.02
        if is_quantized(cfg, name, kind):
            if cfg.quant.method == "nvfp4":
                p, s, g = codecs.nvfp4_quantize(t)
                sd[name] = p
                sd[name + "_scale"] = s.view(torch.float8_e4m3fn)
                sd[name + "_scale_2"] = g.reshape(())
            elif cfg.quant.method == "fp8_block":
                q, s = codecs.fp8_block_quantize_weight(t)
                sd[name] = q.view(torch.float8_e4m3fn)
                sd[name + "_scale_inv"] = s
            else:
                raise ValueError(cfg.quant.method)
        else:
            sd[name] = t.to(dtype if kind in ("linear", "embed") else torch.float32)
    return sd


class DictSource:
    """In-memory tensor source with the same read interface as a checkpoint Index."""

    def __init__(self, tensors: dict):
        self.tensors = tensors

    def has(self, name: str) -> bool:
        return name in self.tensors

    def read(self, name: str, row0: int = 0, row1: int | None = None) -> torch.Tensor:
        t = self.tensors[name]
        return t if t.dim() == 0 else t[row0:row1]

    def shape(self, name: str) -> tuple:
        return tuple(self.tensors[name].shape)


class IndexSource:
    """Checkpoint-directory tensor source (bounded row-range reads, header-first)."""

    def __init__(self, index: st.Index):
        self.index = index

    def has(self, name: str) -> bool:
        return self.index.has(name)

    def read(self, name: str, row0: int = 0, row1: int | None = None) -> torch.Tensor:
        return self.index.read(name, row0, row1)

    def shape(self, name: str) -> tuple:
        return tuple(self.index.info(name).shape)


def byte_tokenizer_json(vocab_size: int) -> dict:
    """A minimal byte-level tokenizer description: ids 0..255 are bytes, the rest unused
    placeholders, plus chat special tokens at the top of the vocabulary."""
    return {"type": "vade-bytes", "vocab_size": vocab_size,
            "special_tokens": {"<|im_start|>": vocab_size - 4, "<|im_end|>": vocab_size - 3,
                               "<|endoftext|>": vocab_size - 2, "<think>": vocab_size - 1}}


def write_checkpoint(cfg: ModelConfig, root: str, seed: int = 0, max_shard_bytes: int = 1 << 30,
                     dtype: torch.dtype = torch.bfloat16) -> str:
    from .manifest import write_manifest
    os.makedirs(root, exist_ok=True)
    sd = synth_state_dict(cfg, seed, dtype)
    st.write_sharded(sd, root, max_shard_bytes, metadata={"format": "pt", "generator": "vade_b200.synth"})
    with open(os.path.join(root, "config.json"), "w") as f:
        json.dump(cfg.to_json(), f, indent=1)
    with open(os.path.join(root, "generation_config.json"), "w") as f:
        json.dump({"do_sample": False, "temperature": 1.0, "top_p": 1.0, "top_k": 0,
                   "eos_token_id": cfg.vocab_size - 3}, f)
    with open(os.path.join(root, "tokenizer.json"), "w") as f:
        json.dump(byte_tokenizer_json(cfg.vocab_size), f)
    write_manifest(root)
    return root
