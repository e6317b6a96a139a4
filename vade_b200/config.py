"""Model configuration for hybrid Gated-DeltaNet + gated-attention MoE models.

Everything is derived from a HuggingFace-style ``config.json`` (``text_config`` plus an
optional ``quantization_config``); no dimension is hard-coded anywhere in the engine.
The reference pins its architecture to one exact shape
(engine/crates/model/src/flash/mod.rs:260-340); this build keeps the same field names
but accepts any consistent set of dimensions.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from typing import Any

#: number of canonical K ranges of every row-parallel ("second") matrix. A rank of a
#: TP group owns RANGES / tp consecutive ranges, so TP must divide it.
RANGES = 8


@dataclass
class QuantConfig:
    """Storage class of the linear weights.

    method: "none" (plain bf16/fp32), "nvfp4" (e2m1 + e4m3 scale per 16 + fp32 tensor
    scale, W4A16) or "fp8_block" (e4m3 weights with 128x128 fp32 scales, activations
    e4m3 with 1x128 scales).  ``ignore`` lists module-name globs kept in plain storage
    (router, lm_head, embeddings, norms by default), like ModelOpt's ignore list
    (engine/crates/model/src/flash/mixed.rs:52-94).
    """
    method: str = "none"
    group_size: int = 16
    ignore: list = field(default_factory=lambda: ["lm_head", "*.mlp.gate", "*embed_tokens",
                                                  "*shared_expert_gate", "*norm*", "*conv1d"])

    def to_json(self) -> dict:
        if self.method == "none":
            return {}
        if self.method == "nvfp4":
            return {"quant_method": "modelopt", "quant_algo": "NVFP4",
                    "group_size": self.group_size, "ignore": list(self.ignore)}
        if self.method == "fp8_block":
            return {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [128, 128],
                    "activation_scheme": "dynamic", "ignore": list(self.ignore)}
        raise ValueError(f"unknown quantization method {self.method!r}")

    @staticmethod
    def from_json(obj: dict | None) -> "QuantConfig":
        if not obj:
            return QuantConfig()
        method = obj.get("quant_method")
        ignore = obj.get("ignore", QuantConfig().ignore)
        if method == "modelopt":
            algo = obj.get("quant_algo", "NVFP4")
            if algo != "NVFP4":
                raise ValueError(f"unsupported modelopt algorithm {algo!r}")
            return QuantConfig("nvfp4", int(obj.get("group_size", 16)), list(ignore))
        if method == "fp8":
            if list(obj.get("weight_block_size", [128, 128])) != [128, 128]:
                raise ValueError("fp8 checkpoints must use 128x128 weight blocks")
            return QuantConfig("fp8_block", 128, list(ignore))
        raise ValueError(f"unknown quant_method {method!r}")


@dataclass
class ModelConfig:
    vocab_size: int = 4096
    hidden_size: int = 256
    num_hidden_layers: int = 4
    full_attention_interval: int = 4        # layer i is full attention when (i+1) % interval == 0
    # gated attention
    num_attention_heads: int = 4
    num_key_value_heads: int = 1
    head_dim: int = 64
    partial_rotary_factor: float = 0.25
    rope_theta: float = 1e7
    # gated delta net
    linear_num_key_heads: int = 4
    linear_num_value_heads: int = 8
    linear_key_head_dim: int = 64
    linear_value_head_dim: int = 64
    linear_conv_kernel_dim: int = 4
    # MoE
    num_experts: int = 16
    num_experts_per_tok: int = 2
    moe_intermediate_size: int = 128
    shared_expert_intermediate_size: int = 256
    norm_topk_prob: bool = True
    # misc
    rms_norm_eps: float = 1e-6
    mtp_num_hidden_layers: int = 1
    max_position_embeddings: int = 262144
    tie_word_embeddings: bool = False
    model_type: str = "qwen3_next"
    # optional reference-model extras (hyper-connections, n-gram embeddings, sparse
    # indexer) are config-gated and off for every target configuration.
    hyper_connections: int = 0
    quant: QuantConfig = field(default_factory=QuantConfig)

    # ---- derived ----
    def is_attention_layer(self, i: int) -> bool:
        return (i + 1) % self.full_attention_interval == 0

    @property
    def layer_types(self) -> list:
        return ["full_attention" if self.is_attention_layer(i) else "linear_attention"
                for i in range(self.num_hidden_layers)]

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def gdn_key_dim(self) -> int:
        return self.linear_num_key_heads * self.linear_key_head_dim

    @property
    def gdn_value_dim(self) -> int:
        return self.linear_num_value_heads * self.linear_value_head_dim

    @property
    def gdn_conv_dim(self) -> int:
        return 2 * self.gdn_key_dim + self.gdn_value_dim

    def validate(self) -> None:
        def need(ok: bool, msg: str) -> None:
            if not ok:
                raise ValueError(f"invalid model config: {msg}")
        need(self.num_hidden_layers > 0 and self.hidden_size > 0, "empty model")
        need(self.num_attention_heads % self.num_key_value_heads == 0, "GQA group must be whole")
        need(self.linear_num_value_heads % self.linear_num_key_heads == 0, "GDN value heads per key head")
        need(self.rotary_dim % 2 == 0 and 0 < self.rotary_dim <= self.head_dim, "rotary dim")
        need(self.num_experts_per_tok <= self.num_experts, "top-k larger than expert count")
        need((self.num_attention_heads * self.head_dim) % RANGES == 0, "o_proj K not divisible by ranges")
        need(self.gdn_value_dim % RANGES == 0, "out_proj K not divisible by ranges")
        need(self.linear_conv_kernel_dim == 4, "only conv kernel 4 is implemented")

    # ---- (de)serialisation in the HF layout ----
    def to_json(self) -> dict:
        text = {k: v for k, v in asdict(self).items() if k not in ("quant", "model_type")}
        text["layer_types"] = self.layer_types
        out: dict[str, Any] = {"model_type": self.model_type, "architectures": ["Qwen3NextForCausalLM"],
                               "text_config": text}
        q = self.quant.to_json()
        if q:
            out["quantization_config"] = q
        return out

    @staticmethod
    def from_json(obj: dict) -> "ModelConfig":
        text = obj.get("text_config", obj)
        known = {f for f in ModelConfig.__dataclass_fields__ if f not in ("quant", "model_type")}
        kwargs = {k: v for k, v in text.items() if k in known}
        cfg = ModelConfig(**kwargs)
        cfg.model_type = obj.get("model_type", cfg.model_type)
        cfg.quant = QuantConfig.from_json(obj.get("quantization_config"))
        if "layer_types" in text and list(text["layer_types"]) != cfg.layer_types:
            raise ValueError("layer_types does not follow full_attention_interval")
        cfg.validate()
        return cfg

    @staticmethod
    def load(path: str) -> "ModelConfig":
        with open(path, "rb") as f:
            return ModelConfig.from_json(json.loads(f.read()))


# ---------------------------------------------------------------------------------
# Named configurations used by tests and benchmarks.
# ---------------------------------------------------------------------------------

def tiny_config(**over) -> ModelConfig:
    """4-layer plumbing/determinism model (fp32 on CPU)."""
    cfg = ModelConfig(**over)
    cfg.validate()
    return cfg


def small_gpu_config(quant: str = "nvfp4", **over) -> ModelConfig:
    """Small GPU-shaped model: every dimension satisfies the tile rules of the sm_100a
    kernels (K multiples of 64 per range, head dims 128/256) while staying a few MB."""
    kw = dict(vocab_size=8192, hidden_size=1024, num_hidden_layers=4,
              num_attention_heads=8, num_key_value_heads=2, head_dim=256,
              linear_num_key_heads=8, linear_num_value_heads=16,
              linear_key_head_dim=128, linear_value_head_dim=128,
              num_experts=32, num_experts_per_tok=4, moe_intermediate_size=256,
              shared_expert_intermediate_size=256)
    kw.update(over)
    cfg = ModelConfig(**kw)
    cfg.quant = QuantConfig(quant) if quant != "none" else QuantConfig()
    cfg.validate()
    return cfg


def qwen3_next_80b_config(quant: str = "nvfp4", **over) -> ModelConfig:
    """Qwen3-Next-80B-A3B shape: 48 layers = 12 x [3 GDN + 1 gated attention], hidden 2048,
    512 experts top-10 + shared expert (intermediate 512), vocab 151936."""
    kw = dict(vocab_size=151936, hidden_size=2048, num_hidden_layers=48,
              num_attention_heads=16, num_key_value_heads=2, head_dim=256,
              linear_num_key_heads=16, linear_num_value_heads=32,
              linear_key_head_dim=128, linear_value_head_dim=128,
              num_experts=512, num_experts_per_tok=10, moe_intermediate_size=512,
              shared_expert_intermediate_size=512)
    kw.update(over)
    cfg = ModelConfig(**kw)
    cfg.quant = QuantConfig(quant) if quant != "none" else QuantConfig()
    cfg.validate()
    return cfg


def hybrid_200b_config(quant: str = "nvfp4", **over) -> ModelConfig:
    """~200B-class shape: 60 layers = 15 x [3 GDN + 1 attention], hidden 4096."""
    kw = dict(vocab_size=151936, hidden_size=4096, num_hidden_layers=60,
              num_attention_heads=32, num_key_value_heads=4, head_dim=256,
              linear_num_key_heads=32, linear_num_value_heads=64,
              linear_key_head_dim=128, linear_value_head_dim=128,
              num_experts=512, num_experts_per_tok=10, moe_intermediate_size=512,
              shared_expert_intermediate_size=512)
    kw.update(over)
    cfg = ModelConfig(**kw)
    cfg.quant = QuantConfig(quant) if quant != "none" else QuantConfig()
    cfg.validate()
    return cfg


NAMED_CONFIGS = {
    "tiny": tiny_config,
    "small": small_gpu_config,
    "qwen3-next-80b-a3b": qwen3_next_80b_config,
    "hybrid-200b": hybrid_200b_config,
}
