"""Model configuration shared by every decoder family, plus the named shapes used by the benchmarks.

The reference hard-codes its model shapes in per-family graph builders
(crates/sllm-core/src/qwen_graph.rs:44-110, gemma4_graph.rs:27-31, native/hip/src/moe_expert_kernel_internal.hpp:10-13);
here one dataclass describes all of them and the graph code branches on its fields.
"""
from __future__ import annotations

from dataclasses import dataclass, field, asdict
from typing import Optional


@dataclass
class ModelConfig:
    name: str = "tiny-llama"
    family: str = "llama"            # llama | moe | qwen35 | gemma4
    n_layers: int = 2
    d_model: int = 256
    n_heads: int = 4
    n_kv_heads: int = 2
    head_dim: int = 64
    ffn: int = 688
    vocab: int = 1024
    rope_theta: float = 10000.0
    rotary_dim: Optional[int] = None  # None = head_dim
    rms_eps: float = 1e-5
    norm_offset_one: bool = False     # scale = 1 + w (Qwen3.5) instead of w
    act: str = "silu"                 # silu | gelu_tanh
    tie_embeddings: bool = False
    embedding_scale: float = 1.0
    logit_softcap: float = 0.0
    weight_format: str = "bf16"       # fp32 | bf16 | fp8 | nvfp4 | mxfp4
    kv_format: str = "bf16"           # fp32 | bf16 | fp8 | fp8-static
    kv_static_scales: Optional[list] = None   # fp8-static: [[k, v]] decode scales per layer (from a quantised checkpoint)
    page_size: int = 16
    max_context: int = 8192
    # sliding-window attention: window size and per-layer flags (True = windowed layer)
    sliding_window: int = 0
    window_layers: Optional[list] = None
    attention_sinks: bool = False
    qk_norm: bool = False
    # mixture of experts
    n_experts: int = 0
    top_k: int = 0
    expert_ffn: int = 0
    shared_expert_ffn: int = 0
    expert_format: str = "mxfp4"
    # linear-attention (gated delta net) hybrid: every `full_attention_interval`-th layer is full attention
    full_attention_interval: int = 0
    gdn_heads: int = 0               # value heads of a gated-delta-net layer
    gdn_qk_heads: int = 0            # query / key heads (value heads are a multiple)
    gdn_head_dim: int = 0
    gdn_conv_kernel: int = 4
    attn_output_gate: bool = False
    post_norms: bool = False         # Gemma-style norms after attention and after the MLP (before the residual add)
    # Gemma-4 attention details (reference: crates/sllm-core/src/gemma4_graph.rs:690-915)
    rope_theta_local: float = 0.0    # rotary base of the sliding-window layers (0: rope_theta)
    rope_proportional: bool = False  # full-attention layers: channel i < rotary_dim_full / 2 pairs with i + head_dim / 2,
    rotary_dim_full: Optional[int] = None  # frequencies theta^(-2 i / head_dim); the channels between are not rotated
    v_norm: bool = False             # unweighted RMS norm of every value head
    attn_scale: Optional[float] = None     # softmax scale (None: 1 / sqrt(head_dim)); 1.0 where q / k norms set the scale
    layer_scalar: bool = False       # the residual stream is multiplied by a learned scalar at the end of every layer
    k_equals_v_full: bool = False    # full-attention layers have no value projection: v = the (un-normed) key projection
    # vision-language models: rotary pairs [0, t) follow the temporal index, [t, t + h) the height index and the rest
    # the width index of a token's 3-axis position (text tokens carry the same value on all three)
    mrope_sections: Optional[list] = None
    image_token_id: Optional[int] = None     # placeholder id of visual tokens (None: vocab - 1)
    vision: Optional[dict] = None            # fields of models.vision_tower.VisionConfig when the file carries a tower

    def to_dict(self) -> dict:
        return asdict(self)

    def layer_window(self, layer: int) -> int:
        if self.sliding_window <= 0:
            return 0
        if self.window_layers is None:
            return self.sliding_window
        return self.sliding_window if self.window_layers[layer] else 0

    def layer_rope(self, layer: int) -> tuple:
        """(theta, rotary_dim, pair_offset) of a layer; pair_offset 0 is the plain split-half layout."""
        windowed = self.layer_window(layer) > 0
        if windowed:
            return (self.rope_theta_local or self.rope_theta), (self.rotary_dim or self.head_dim), 0
        if self.rope_proportional:
            return self.rope_theta, (self.rotary_dim_full or self.rotary_dim or self.head_dim), self.head_dim // 2
        return self.rope_theta, (self.rotary_dim or self.head_dim), 0

    @property
    def q_size(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.n_kv_heads * self.head_dim


def tiny_llama() -> ModelConfig:
    """2-layer CPU check model: fp32 weights, exact greedy comparison."""
    return ModelConfig(name="tiny-llama", n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=688,
                       vocab=1024, rope_theta=10000.0, rms_eps=1e-5, weight_format="fp32", kv_format="fp32")


def llama3_8b(weight_format: str = "fp8", kv_format: str = "fp8") -> ModelConfig:
    return ModelConfig(name="llama3-8b", n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128,
                       ffn=14336, vocab=128256, rope_theta=500000.0, weight_format=weight_format,
                       kv_format=kv_format)


def llama3_70b(weight_format: str = "nvfp4", kv_format: str = "fp8") -> ModelConfig:
    return ModelConfig(name="llama3-70b", n_layers=80, d_model=8192, n_heads=64, n_kv_heads=8, head_dim=128,
                       ffn=28672, vocab=128256, rope_theta=500000.0, weight_format=weight_format,
                       kv_format=kv_format)


def llama_draft_1b() -> ModelConfig:
    """Speculative-decoding draft: 16 layers, d=2048, 32/8 heads (head_dim 64), ffn 8192, shared vocab."""
    return ModelConfig(name="llama-draft", n_layers=16, d_model=2048, n_heads=32, n_kv_heads=8, head_dim=64,
                       ffn=8192, vocab=128256, rope_theta=500000.0, weight_format="bf16", kv_format="bf16")


def gpt_oss_120b_shape() -> ModelConfig:
    """36-layer MoE: d=2880, 64/8 heads of 64, alternating 128-token window / full attention,
    128 experts top-4 (expert ffn 2880) in MXFP4; router and attention in bf16."""
    return ModelConfig(name="moe-120b", family="moe", n_layers=36, d_model=2880, n_heads=64, n_kv_heads=8,
                       head_dim=64, ffn=2880, vocab=201088, rope_theta=150000.0, weight_format="bf16",
                       kv_format="bf16", sliding_window=128, window_layers=[i % 2 == 0 for i in range(36)],
                       attention_sinks=True, n_experts=128, top_k=4, expert_ffn=2880, expert_format="mxfp4")


def qwen35_hybrid_shape(layers: int = 32) -> ModelConfig:
    """Qwen3.5-class hybrid: three gated-delta-net layers then one full-attention layer, repeated; full layers use
    q/k RMSNorm (1 + w), rotary on the first 64 of 256 channels (theta 1e7) and a sigmoid output gate."""
    return ModelConfig(name="qwen35-hybrid", family="qwen35", n_layers=layers, d_model=2560, n_heads=16, n_kv_heads=4, head_dim=256,
                       ffn=9216, vocab=151936, rope_theta=1e7, rotary_dim=64, rms_eps=1e-6, norm_offset_one=True,
                       weight_format="bf16", kv_format="bf16", qk_norm=True, full_attention_interval=4, gdn_heads=32,
                       gdn_qk_heads=16, gdn_head_dim=128, gdn_conv_kernel=4, attn_output_gate=True, max_context=8192)


def gemma4_shape(layers: int = 48) -> ModelConfig:
    """Gemma-4-class dense decoder: five 1024-token sliding-window layers per full layer, q/k norm, sandwich norms,
    gelu-tanh gated MLP, embeddings scaled by sqrt(d), final logit soft-cap 30, tied embeddings; value heads get an
    unweighted RMS norm, the softmax scale is 1, every layer ends in a learned scalar, sliding layers rotate with base
    1e4, full layers with base 1e6 in the proportional layout (a quarter of the head) and reuse the key projection as
    value.  One head geometry (256 wide, 8 kv heads) serves every layer here; the reference's full layers are 512 wide
    with one kv head (gemma4_graph.rs:754-775)."""
    return ModelConfig(rope_theta_local=1e4, rope_proportional=True, rotary_dim_full=64, v_norm=True, attn_scale=1.0,
                       layer_scalar=True, k_equals_v_full=True, name="gemma4", family="gemma4", n_layers=layers, d_model=3840, n_heads=16, n_kv_heads=8, head_dim=256,
                       ffn=15360, vocab=262144, rope_theta=1e6, rms_eps=1e-6, act="gelu_tanh", tie_embeddings=True,
                       embedding_scale=3840 ** 0.5, logit_softcap=30.0, weight_format="bf16", kv_format="bf16",
                       sliding_window=1024, window_layers=[(i + 1) % 6 != 0 for i in range(layers)], qk_norm=True,
                       post_norms=True, max_context=8192)


def _qwen35_moe():
    from .moe import qwen35_moe_shape
    return qwen35_moe_shape()


def _qwen35_moe_hybrid():
    from .qwen35 import qwen35_moe_hybrid_shape
    return qwen35_moe_hybrid_shape()


NAMED = {
    "qwen35-moe": _qwen35_moe,
    "qwen35-moe-hybrid": _qwen35_moe_hybrid,
    "tiny-llama": tiny_llama,
    "llama3-8b": llama3_8b,
    "llama3-70b": llama3_70b,
    "llama-draft": llama_draft_1b,
    "moe-120b": gpt_oss_120b_shape,
    "qwen35-hybrid": qwen35_hybrid_shape,
    "gemma4": gemma4_shape,
}
