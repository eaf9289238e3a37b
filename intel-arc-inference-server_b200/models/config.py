"""Model descriptors: per-model shapes as data.

Plays the role of the reference's ``ModelDesc`` (src/model/model_desc.h:67-195):
every shape the loader, the memory planner and the kernels need is derived
from one frozen dataclass, and the table of fused linears (qkv, gate‖up, ...)
is generated from it rather than written per model.
"""
from __future__ import annotations

from dataclasses import dataclass, field, asdict, replace
from typing import Optional


@dataclass(frozen=True)
class LinearDesc:
    """One fused linear: ``out[n] = sum_k x[k] w[n][k]``."""
    name: str
    n: int
    k: int
    parts: tuple          # checkpoint tensors fused along N, in order
    parallel: str         # "column" | "row" | "none": how tensor parallel slices it


@dataclass(frozen=True)
class ModelConfig:
    name: str
    n_layers: int
    hidden: int
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    rope_theta: float = 1e6
    rms_eps: float = 1e-6
    group_size: int = 64
    # mixture of experts (n_experts == 0: dense SwiGLU FFN)
    n_experts: int = 0
    top_k: int = 0
    expert_ffn: int = 0
    shared_ffn: int = 0           # 0: no shared expert
    # multi-token-prediction head: extra decoder layers sharing embed / lm_head
    mtp_layers: int = 0
    architecture: str = "B200DenseForCausalLM"
    page_size: int = 16
    # sliding-window attention: a row attends to its last ``sliding_window`` positions (0: the whole context);
    # with ``full_attn_every`` = n > 0 every n-th layer (li % n == n - 1) keeps full attention, as in the
    # reference's windowed families (src/kernels/kolibri/kol_attn.cl: sliding ring 4096 / full layers)
    sliding_window: int = 0
    full_attn_every: int = 0
    # hybrid family: gated delta-net (linear attention) layers with n_k key heads and n_v value heads of 128;
    # with ``gdn_v_heads`` > 0 every layer is a GDN layer except each ``full_attn_every``-th one, which keeps
    # softmax attention (the reference's hybrid checkpoints: src/kernels/gdn_step.cl, three GDN layers per
    # attention layer)
    gdn_k_heads: int = 0
    gdn_v_heads: int = 0
    gdn_head_dim: int = 128

    @property
    def q_dim(self) -> int:
        return self.n_q_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    @property
    def gqa(self) -> int:
        return self.n_q_heads // self.n_kv_heads

    @property
    def is_moe(self) -> bool:
        return self.n_experts > 0

    def is_gdn_layer(self, li: int) -> bool:
        if self.gdn_v_heads <= 0 or li >= self.n_layers:
            return False
        return not (self.full_attn_every > 0 and li % self.full_attn_every == self.full_attn_every - 1)

    def gdn_index(self, li: int) -> int:
        """Index of GDN layer ``li`` among the GDN layers (its slice of the recurrent-state buffers)."""
        return sum(1 for i in range(li) if self.is_gdn_layer(i))

    @property
    def n_gdn_layers(self) -> int:
        return sum(1 for i in range(self.n_layers) if self.is_gdn_layer(i))

    @property
    def gdn_key_dim(self) -> int:
        return self.gdn_k_heads * self.gdn_head_dim

    @property
    def gdn_value_dim(self) -> int:
        return self.gdn_v_heads * self.gdn_head_dim

    @property
    def gdn_conv_channels(self) -> int:
        return 2 * self.gdn_key_dim + self.gdn_value_dim

    @property
    def gdn_proj_dim(self) -> int:
        """Columns of the fused input projection [ q | k | v | z | b | a ]."""
        return 2 * self.gdn_key_dim + 2 * self.gdn_value_dim + 2 * self.gdn_v_heads

    def window_of(self, li: int) -> int:
        """Attention window of layer ``li`` in positions (0: full attention)."""
        if self.sliding_window <= 0 or self.gdn_v_heads > 0:
            return 0
        if self.full_attn_every > 0 and li % self.full_attn_every == self.full_attn_every - 1:
            return 0
        return self.sliding_window

    def tp_shard(self, world: int) -> "ModelConfig":
        """The shapes one rank of a ``world``-way tensor-parallel group holds: whole attention heads,
        whole FFN interleave runs; hidden size and vocabulary stay (the lm_head is split by rows outside).
        The reference's ``tp_card_desc`` does this for its two cards (src/model/model_desc.cc:252-285)."""
        if world == 1:
            return self
        if self.n_q_heads % world or self.n_kv_heads % world:
            raise ValueError(f"tensor parallel {world} does not divide {self.n_q_heads} q / {self.n_kv_heads} kv heads")
        if self.ffn % (64 * world) or (self.shared_ffn and self.shared_ffn % (64 * world)):
            raise ValueError(f"tensor parallel {world} does not divide FFN {self.ffn} into whole groups of 64")
        import dataclasses
        return dataclasses.replace(self, name=f"{self.name}/tp{world}", n_q_heads=self.n_q_heads // world,
                                   n_kv_heads=self.n_kv_heads // world, ffn=self.ffn // world,
                                   shared_ffn=self.shared_ffn // world)

    def linears(self):
        """Fused linear table of one decoder layer (attention + dense FFN part)."""
        h = self.hidden
        out = [
            LinearDesc("qkv", self.qkv_dim, h, ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"), "column"),
            LinearDesc("o", h, self.q_dim, ("self_attn.o_proj",), "row"),
        ]
        if not self.is_moe:
            out += [
                LinearDesc("gate_up", 2 * self.ffn, h, ("mlp.gate_proj", "mlp.up_proj"), "column"),
                LinearDesc("down", h, self.ffn, ("mlp.down_proj",), "row"),
            ]
        return out

    def _mixer_params(self) -> float:
        """Mean weights per layer of the token mixer (attention projections, or a gated delta-net layer's)."""
        h = self.hidden
        attn = self.qkv_dim * h + h * self.q_dim
        g = self.n_gdn_layers
        if not g:
            return attn
        gdn = self.gdn_proj_dim * h + h * self.gdn_value_dim
        return (g * gdn + (self.n_layers - g) * attn) / self.n_layers

    def param_count(self) -> int:
        h = self.hidden
        per = self._mixer_params()
        if self.is_moe:
            per += self.n_experts * 3 * self.expert_ffn * h + self.n_experts * h
            if self.shared_ffn:
                per += 3 * self.shared_ffn * h + h
        else:
            per += 3 * self.ffn * h
        return int(self.n_layers * per + 2 * self.vocab * h)

    def weight_bytes_per_token(self, lm_head_bytes_per_weight: float = 2.0) -> float:
        """Bytes of weights one decode step must read ("W" in the reference's
        perf model, docs/05-perf-model.md:35-39): int4 nibbles + fp16 group scales
        for every linear that is touched, plus the head."""
        h = self.hidden
        int4 = 0.5 + 2.0 / self.group_size
        per = self._mixer_params() * int4
        if self.is_moe:
            per += self.top_k * 3 * self.expert_ffn * h * int4 + self.n_experts * h * 2
            if self.shared_ffn:
                per += 3 * self.shared_ffn * h * int4
        else:
            per += 3 * self.ffn * h * int4
        return self.n_layers * per + self.vocab * h * lm_head_bytes_per_weight

    def kv_bytes_per_token(self, kv_dtype: str = "bf16") -> int:
        per_head = self.head_dim * (2 if kv_dtype == "bf16" else 1) + (4 if kv_dtype == "int8" else 0)
        return (self.n_layers - self.n_gdn_layers) * 2 * self.n_kv_heads * per_head

    def to_hf_config(self) -> dict:
        d = {
            "architectures": [self.architecture],
            "model_type": "b200_moe" if self.is_moe else "b200_dense",
            "num_hidden_layers": self.n_layers,
            "hidden_size": self.hidden,
            "num_attention_heads": self.n_q_heads,
            "num_key_value_heads": self.n_kv_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.ffn,
            "vocab_size": self.vocab,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_eps,
            "num_experts": self.n_experts,
            "num_experts_per_tok": self.top_k,
            "moe_intermediate_size": self.expert_ffn,
            "shared_expert_intermediate_size": self.shared_ffn,
            "mtp_num_hidden_layers": self.mtp_layers,
            "sliding_window": self.sliding_window or None,
            "full_attention_interval": self.full_attn_every,
            "linear_num_key_heads": self.gdn_k_heads,
            "linear_num_value_heads": self.gdn_v_heads,
            "linear_key_head_dim": self.gdn_head_dim,
            "torch_dtype": "bfloat16",
            "quantization_config": {
                "bits": 4, "group_size": self.group_size, "sym": True, "desc_act": False,
                "quant_method": "gptq", "packing_format": "auto_round:auto_gptq",
            },
            "name": self.name,
        }
        return d

    @staticmethod
    def from_hf_config(d: dict) -> "ModelConfig":
        return ModelConfig(
            name=d.get("name", d.get("_name_or_path", "model")),
            n_layers=d["num_hidden_layers"], hidden=d["hidden_size"],
            n_q_heads=d["num_attention_heads"], n_kv_heads=d.get("num_key_value_heads", d["num_attention_heads"]),
            head_dim=d.get("head_dim", d["hidden_size"] // d["num_attention_heads"]),
            ffn=d.get("intermediate_size", 0), vocab=d["vocab_size"],
            rope_theta=float(d.get("rope_theta", 1e6)), rms_eps=float(d.get("rms_norm_eps", 1e-6)),
            group_size=64,
            n_experts=d.get("num_experts", 0) or 0, top_k=d.get("num_experts_per_tok", 0) or 0,
            expert_ffn=d.get("moe_intermediate_size", 0) or 0,
            shared_ffn=d.get("shared_expert_intermediate_size", 0) or 0,
            mtp_layers=d.get("mtp_num_hidden_layers", 0) or 0,
            sliding_window=d.get("sliding_window", 0) or 0, full_attn_every=d.get("full_attention_interval", 0) or 0,
            gdn_k_heads=d.get("linear_num_key_heads", 0) or 0, gdn_v_heads=d.get("linear_num_value_heads", 0) or 0,
            gdn_head_dim=d.get("linear_key_head_dim", 128) or 128,
            architecture=(d.get("architectures") or ["B200DenseForCausalLM"])[0],
        )


def tiny_dense() -> ModelConfig:
    """The CPU-oracle configuration: 2 layers, hidden 256, 4 q / 2 kv heads of 64."""
    return ModelConfig("tiny-dense", 2, 256, 4, 2, 64, 704, 1024)


def small_dense() -> ModelConfig:
    """Small dense model with the production head size (128), for the tensor-core prefill path."""
    return ModelConfig("small-dense", 2, 512, 8, 2, 128, 1408, 2048)


def small_windowed() -> ModelConfig:
    """Four layers of the small dense shape; layers 0 and 2 attend to the last 48 positions, 1 and 3 to all."""
    return ModelConfig("small-windowed", 4, 512, 8, 2, 128, 1408, 2048, sliding_window=48, full_attn_every=2)


def small_hybrid() -> ModelConfig:
    """Four layers of the small dense shape: layers 0 and 2 are gated delta-net layers (2 key / 4 value heads of
    128), layers 1 and 3 softmax attention."""
    return ModelConfig("small-hybrid", 4, 512, 8, 2, 128, 1408, 2048, full_attn_every=2, gdn_k_heads=2, gdn_v_heads=4,
                       architecture="B200HybridForCausalLM")


def tiny_moe() -> ModelConfig:
    return ModelConfig("tiny-moe", 2, 256, 4, 2, 64, 0, 1024, n_experts=8, top_k=2,
                       expert_ffn=128, shared_ffn=128, architecture="B200MoeForCausalLM")


def small_moe() -> ModelConfig:
    """Small MoE with the production head size, for the grouped tensor-core path."""
    return ModelConfig("small-moe", 2, 512, 8, 2, 128, 0, 2048, n_experts=16, top_k=4, expert_ffn=256,
                       shared_ffn=256, architecture="B200MoeForCausalLM")


def dense_27b() -> ModelConfig:
    """27B-shape dense decoder: 64 layers, hidden 5120, 40 q / 8 kv heads of 128, FFN 17408."""
    return ModelConfig("dense-27b", 64, 5120, 40, 8, 128, 17408, 151936)


def hybrid_27b() -> ModelConfig:
    """27B-shape hybrid decoder: the dense 27B shape with three gated delta-net layers (16 key / 48 value heads of
    128) before every softmax-attention layer."""
    return ModelConfig("hybrid-27b", 64, 5120, 40, 8, 128, 17408, 151936, full_attn_every=4, gdn_k_heads=16,
                       gdn_v_heads=48, architecture="B200HybridForCausalLM")


def moe_35b_a3b() -> ModelConfig:
    """35B-A3B-shape MoE: 40 layers, hidden 2048, 16 q / 4 kv heads, 256 experts top-8 + shared."""
    return ModelConfig("moe-35b-a3b", 40, 2048, 16, 4, 128, 0, 151936, n_experts=256, top_k=8,
                       expert_ffn=512, shared_ffn=512, architecture="B200MoeForCausalLM")


def dflash_drafter(target: ModelConfig) -> ModelConfig:
    """DFlash-style block drafter: a 2-layer W4A16 decoder at the target's width."""
    return replace(target, name=target.name + "-dflash", n_layers=2, n_experts=0, top_k=0, expert_ffn=0,
                   shared_ffn=0, ffn=target.ffn if target.ffn else 4 * target.hidden, mtp_layers=0,
                   architecture="B200DFlashDrafter")


PRESETS = {
    "tiny-dense": tiny_dense, "tiny-moe": tiny_moe, "small-dense": small_dense, "small-windowed": small_windowed, "small-hybrid": small_hybrid, "small-moe": small_moe, "dense-27b": dense_27b, "hybrid-27b": hybrid_27b, "moe-35b-a3b": moe_35b_a3b,
}


def preset(name: str) -> ModelConfig:
    if name not in PRESETS:
        raise KeyError(f"unknown model preset {name!r}; known: {sorted(PRESETS)}")
    return PRESETS[name]()
