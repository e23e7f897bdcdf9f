"""Model configuration.

``TransformerConfig`` mirrors the reference struct field for field
(include/quant/transformer.h:12-43) and serialises to the same raw 128-byte little-endian image
the reference writes into the ``.quant`` header (src/model/model.cpp:219-220), so checkpoints are
interchangeable.  Byte offsets (x86-64): vocab_size@0 i64, hidden_size@8, num_layers@16,
num_heads@24, head_dim@32, ffn_hidden_size@40, norm_eps@48 f32, rope_theta@52 f32, max_seq_len@56
i64, activation@64 u8, num_kv_heads@72 i64, use_parallel_residual@80 bool, mtp_num_heads@84 i32,
mtp_loss_weight@88 f32, rope_scaling_mode@92 u8, rope_scaling_factor@96 f32,
rope_original_max_seq_len@104 i64, yarn_attn_factor@112 f32, yarn_beta_fast@116 f32,
yarn_beta_slow@120 f32, use_fp8@124 bool, fp8_use_e4m3@125 bool.
"""
from __future__ import annotations

import struct
from dataclasses import asdict, dataclass, field

ACTIVATIONS = ["none", "relu", "gelu", "silu", "swiglu", "geglu"]
ROPE_SCALING = ["none", "linear", "ntk", "yarn"]
CONFIG_BYTES = 128


@dataclass
class TransformerConfig:
    vocab_size: int = 32000
    hidden_size: int = 512
    num_layers: int = 8
    num_heads: int = 8
    head_dim: int = 0            # 0 -> hidden_size // num_heads
    ffn_hidden_size: int = 0     # 0 -> 4 * hidden_size
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_seq_len: int = 2048
    activation: str = "swiglu"
    num_kv_heads: int = 0        # 0 -> num_heads
    use_parallel_residual: bool = False
    mtp_num_heads: int = 0
    mtp_loss_weight: float = 0.0
    rope_scaling_mode: str = "none"
    rope_scaling_factor: float = 1.0
    rope_original_max_seq_len: int = 0
    yarn_attn_factor: float = 1.0
    yarn_beta_fast: float = 32.0
    yarn_beta_slow: float = 1.0
    use_fp8: bool = False
    fp8_use_e4m3: bool = True
    # ---- not part of the 128-byte image (kept in the JSON side-car / constructor only) ----
    tie_embeddings: bool = False
    norm_type: str = "rmsnorm"   # "layernorm" for the GPT-2-shaped variant
    position_type: str = "rope"  # "learned" for the GPT-2-shaped variant
    attention_bias: bool = False
    init_std: float = 0.02

    def __post_init__(self):
        if not self.head_dim:
            self.head_dim = self.hidden_size // self.num_heads
        if not self.ffn_hidden_size:
            self.ffn_hidden_size = 4 * self.hidden_size
        if not self.num_kv_heads:
            self.num_kv_heads = self.num_heads
        assert self.num_heads % self.num_kv_heads == 0
        self.activation = self.activation.lower()
        assert self.activation in ACTIVATIONS

    @property
    def gated(self) -> bool:
        return self.activation in ("swiglu", "geglu")

    @property
    def act_kernel(self) -> str:
        return {"swiglu": "silu", "geglu": "gelu"}.get(self.activation, self.activation)

    def num_params(self) -> int:
        H, F, D = self.hidden_size, self.ffn_hidden_size, self.head_dim
        per_layer = H * (self.num_heads + 2 * self.num_kv_heads) * D + self.num_heads * D * H
        per_layer += (3 if self.gated else 2) * H * F + 2 * H
        n = self.num_layers * per_layer + self.vocab_size * H + H
        if not self.tie_embeddings:
            n += self.vocab_size * H
        return n

    def flops_per_token(self, seq_len: int, causal: bool = True) -> float:
        """Training FLOPs per token (forward + backward = 3x forward matmul FLOPs)."""
        H, F, D = self.hidden_size, self.ffn_hidden_size, self.head_dim
        lin = H * (self.num_heads + 2 * self.num_kv_heads) * D + self.num_heads * D * H
        lin += (3 if self.gated else 2) * H * F
        attn = 2 * self.num_heads * D * seq_len * (0.5 if causal else 1.0)
        return 6.0 * (self.num_layers * (lin + attn) + self.vocab_size * H)

    # ------------------------------------------------------------------ binary image
    def to_bytes(self) -> bytes:
        b = bytearray(CONFIG_BYTES)
        struct.pack_into("<6q", b, 0, self.vocab_size, self.hidden_size, self.num_layers, self.num_heads,
                         self.head_dim, self.ffn_hidden_size)
        struct.pack_into("<ffq", b, 48, self.norm_eps, self.rope_theta, self.max_seq_len)
        b[64] = ACTIVATIONS.index(self.activation)
        struct.pack_into("<q", b, 72, self.num_kv_heads)
        b[80] = int(self.use_parallel_residual)
        struct.pack_into("<if", b, 84, self.mtp_num_heads, self.mtp_loss_weight)
        b[92] = ROPE_SCALING.index(self.rope_scaling_mode)
        struct.pack_into("<f", b, 96, self.rope_scaling_factor)
        struct.pack_into("<q", b, 104, self.rope_original_max_seq_len)
        struct.pack_into("<fff", b, 112, self.yarn_attn_factor, self.yarn_beta_fast, self.yarn_beta_slow)
        b[124] = int(self.use_fp8)
        b[125] = int(self.fp8_use_e4m3)
        return bytes(b)

    @classmethod
    def from_bytes(cls, raw: bytes, **extra) -> "TransformerConfig":
        if len(raw) < CONFIG_BYTES:
            raw = raw + bytes(CONFIG_BYTES - len(raw))
        v, h, nl, nh, hd, ff = struct.unpack_from("<6q", raw, 0)
        eps, theta, msl = struct.unpack_from("<ffq", raw, 48)
        (nkv,) = struct.unpack_from("<q", raw, 72)
        mtp_n, mtp_w = struct.unpack_from("<if", raw, 84)
        (rsf,) = struct.unpack_from("<f", raw, 96)
        (romsl,) = struct.unpack_from("<q", raw, 104)
        yaf, ybf, ybs = struct.unpack_from("<fff", raw, 112)
        act = raw[64] if raw[64] < len(ACTIVATIONS) else 0
        rsm = raw[92] if raw[92] < len(ROPE_SCALING) else 0
        return cls(vocab_size=v, hidden_size=h, num_layers=nl, num_heads=nh, head_dim=hd, ffn_hidden_size=ff,
                   norm_eps=eps, rope_theta=theta, max_seq_len=msl, activation=ACTIVATIONS[act], num_kv_heads=nkv,
                   use_parallel_residual=bool(raw[80]), mtp_num_heads=mtp_n, mtp_loss_weight=mtp_w,
                   rope_scaling_mode=ROPE_SCALING[rsm], rope_scaling_factor=rsf or 1.0,
                   rope_original_max_seq_len=romsl, yarn_attn_factor=yaf or 1.0, yarn_beta_fast=ybf or 32.0,
                   yarn_beta_slow=ybs or 1.0, use_fp8=bool(raw[124]), fp8_use_e4m3=bool(raw[125]), **extra)

    def to_dict(self):
        return asdict(self)


@dataclass
class MoEConfig(TransformerConfig):
    """Sparse mixture-of-experts decoder (reference: include/quant/moe_model.h, moe_variants.h:61-123)."""
    num_experts: int = 8
    top_k: int = 2
    expert_hidden_size: int = 0          # 0 -> ffn_hidden_size
    num_shared_experts: int = 0
    load_balance_weight: float = 0.01
    router_z_weight: float = 0.001
    capacity_factor: float = 2.0
    capacity_policy: str = "none"        # none | fixed | token_drop | token_pass
    renormalize_topk: bool = True        # softmax over the selected k (Mixtral); False = reference SparseMoE
    variant: str = "sparse_topk"
    expert_fp8: bool = False             # block-scaled E4M3 expert GEMMs

    def __post_init__(self):
        super().__post_init__()
        if not self.expert_hidden_size:
            self.expert_hidden_size = self.ffn_hidden_size


# Named shapes used by the benchmarks and tests (BASELINE configs).
def preset(name: str) -> TransformerConfig:
    name = name.lower()
    if name in ("llama-50m", "cfg2"):
        return TransformerConfig(vocab_size=32000, hidden_size=512, num_layers=8, num_heads=8, ffn_hidden_size=1408,
                                 rope_theta=10000.0, max_seq_len=1024, activation="swiglu", tie_embeddings=True)
    if name in ("llama-3-8b", "cfg3"):
        return TransformerConfig(vocab_size=128256, hidden_size=4096, num_layers=32, num_heads=32, num_kv_heads=8,
                                 ffn_hidden_size=14336, rope_theta=500000.0, max_seq_len=4096, activation="swiglu")
    if name in ("mixtral-8x7b", "cfg4"):
        return MoEConfig(vocab_size=32000, hidden_size=4096, num_layers=32, num_heads=32, num_kv_heads=8,
                         ffn_hidden_size=14336, rope_theta=1000000.0, max_seq_len=4096, activation="swiglu",
                         num_experts=8, top_k=2, load_balance_weight=0.01, expert_fp8=True)
    if name in ("gpt2-small", "cfg1"):
        return TransformerConfig(vocab_size=50257, hidden_size=768, num_layers=12, num_heads=12, ffn_hidden_size=3072,
                                 max_seq_len=1024, activation="gelu", norm_type="layernorm", position_type="learned",
                                 attention_bias=True, tie_embeddings=True)
    if name == "tiny":
        return TransformerConfig(vocab_size=256, hidden_size=128, num_layers=2, num_heads=2, ffn_hidden_size=256,
                                 max_seq_len=128)
    raise KeyError(name)
