"""Model configuration.

``TransformerConfig`` carries the fields of the reference's ``TransformerConfig``
(include/oil/transformer.h:14-27) and serialises them into the same raw 88-byte little-endian
struct that ``DenseModel::save`` memcpy's into the ``.oil`` header (src/model.cpp:150-158):

    offset  0 i64 vocab_size      8 i64 hidden_size    16 i64 num_layers    24 i64 num_heads
           32 i64 head_dim        40 i64 ffn_hidden    48 f32 norm_eps      52 f32 rope_theta
           56 i64 max_seq_len     64 i32 activation (+4 pad)  72 i64 num_kv_heads
           80 u8  parallel_residual (+7 pad)

Padding is written as zeros and ignored on read. Everything the reference struct cannot express
(weight formats, quantisation block size, MoE, tensor shapes) is appended after those 88 bytes as
UTF-8 JSON; the reference reader copies only the first 88 bytes of the config area and skips the
rest through ``config_size``, so extended files stay readable by it.
"""
from __future__ import annotations

import dataclasses
import json
import struct
from dataclasses import dataclass, field

_STRUCT = struct.Struct("<qqqqqqffqi4xqB7x")
assert _STRUCT.size == 88

ACTIVATIONS = {"relu": 0, "gelu": 1, "silu": 2}  # reference enum Activation { ReLU, GELU, SiLU }
_ACT_NAMES = {v: k for k, v in ACTIVATIONS.items()}


@dataclass
class TransformerConfig:
    vocab_size: int = 32000
    hidden_size: int = 768
    num_layers: int = 12
    num_heads: int = 12
    head_dim: int = 64
    ffn_hidden_size: int = 3072
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    max_seq_len: int = 2048
    activation: str = "silu"          # "silu" (SwiGLU), "gelu", "relu"; extension: "relu2" (gated off)
    num_kv_heads: int = 0             # 0 = same as num_heads
    use_parallel_residual: bool = False
    # ---- extensions (stored in the JSON tail)
    gated_ffn: bool = True            # SwiGLU-style gate/up/down; False = up/down with `activation`
    tie_embeddings: bool = False
    weight_format: str = "oil8"       # format of linear weights: oil8 | oil4 | i2s | fp32 | fp16 | mixed
    attn_format: str = ""             # override for attention projections ("" = weight_format)
    ffn_format: str = ""              # override for FFN projections
    embed_format: str = "fp32"        # embedding table (and tied head)
    oil_block_size: int = 256         # weights per quantisation block (one codebook / scale per block)
    codebook_group: int = 1           # blocks that share one codebook (1 = codebook per block)
    # MoE
    num_experts: int = 0
    moe_top_k: int = 2
    moe_aux_coef: float = 0.01
    moe_z_coef: float = 0.0
    moe_shared_experts: int = 0
    moe_ffn_hidden_size: int = 0
    extras: dict = field(default_factory=dict)

    # -------------------------------------------------------------- derived
    @property
    def kv_heads(self) -> int:
        return self.num_kv_heads if self.num_kv_heads > 0 else self.num_heads

    @property
    def q_dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim

    def format_for(self, role: str) -> str:
        if role == "attn" and self.attn_format:
            return self.attn_format
        if role == "ffn" and self.ffn_format:
            return self.ffn_format
        if role == "embed":
            return self.embed_format
        return self.weight_format

    def param_count(self) -> int:
        d, f, L, V = self.hidden_size, self.ffn_hidden_size, self.num_layers, self.vocab_size
        attn = d * (self.q_dim + 2 * self.kv_dim) + self.q_dim * d
        ffn_f = self.moe_ffn_hidden_size or f
        ffn = (3 if self.gated_ffn else 2) * d * ffn_f
        if self.num_experts > 0:
            ffn = ffn * (self.num_experts + self.moe_shared_experts) + d * self.num_experts
        head = 0 if self.tie_embeddings else V * d
        return V * d + L * (attn + ffn + 2 * d) + d + head

    # -------------------------------------------------------------- 88-byte blob + JSON tail
    def to_bytes(self, extended: bool = True) -> bytes:
        act = ACTIVATIONS.get("relu" if self.activation == "relu2" else self.activation, 2)
        head = _STRUCT.pack(self.vocab_size, self.hidden_size, self.num_layers, self.num_heads, self.head_dim,
                            self.ffn_hidden_size, self.norm_eps, self.rope_theta, self.max_seq_len, act,
                            self.num_kv_heads, 1 if self.use_parallel_residual else 0)
        if not extended:
            return head
        base = {f.name for f in dataclasses.fields(self)} - {
            "vocab_size", "hidden_size", "num_layers", "num_heads", "head_dim", "ffn_hidden_size", "norm_eps",
            "rope_theta", "max_seq_len", "num_kv_heads", "use_parallel_residual"}
        tail = {k: getattr(self, k) for k in sorted(base)}
        return head + json.dumps(tail, sort_keys=True, separators=(",", ":")).encode("utf-8")

    @classmethod
    def from_bytes(cls, blob: bytes) -> "TransformerConfig":
        if len(blob) < _STRUCT.size:
            raise ValueError(f"config blob has {len(blob)} bytes, need at least {_STRUCT.size}")
        (vocab, hidden, layers, heads, head_dim, ffn, eps, theta, max_seq, act, kv, par) = _STRUCT.unpack(
            blob[:_STRUCT.size])
        cfg = cls(vocab_size=vocab, hidden_size=hidden, num_layers=layers, num_heads=heads, head_dim=head_dim,
                  ffn_hidden_size=ffn, norm_eps=eps, rope_theta=theta, max_seq_len=max_seq,
                  activation=_ACT_NAMES.get(act, "silu"), num_kv_heads=kv, use_parallel_residual=bool(par))
        tail = blob[_STRUCT.size:]
        if tail:
            try:
                extra = json.loads(tail.decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError):
                extra = {}
            names = {f.name for f in dataclasses.fields(cls)}
            for k, v in extra.items():
                if k in names:
                    setattr(cfg, k, v)
        else:
            # A file written by the reference: FP32 weights, SwiGLU when SiLU, plain MLP otherwise.
            cfg.weight_format = "fp32"
            cfg.gated_ffn = True
        return cfg

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self), indent=2, sort_keys=True)

    @classmethod
    def from_dict(cls, d: dict) -> "TransformerConfig":
        names = {f.name for f in dataclasses.fields(cls)}
        alias = {"dim": "hidden_size", "n_layers": "num_layers", "n_heads": "num_heads", "n_kv_heads": "num_kv_heads"}
        out = {}
        for k, v in d.items():
            k = alias.get(k, k)
            if k in names:
                out[k] = v
        cfg = cls(**out)
        if "head_dim" not in out and cfg.num_heads > 0:
            cfg.head_dim = cfg.hidden_size // cfg.num_heads
        return cfg


# ---------------------------------------------------------------------------- named configurations
def tiny_byte_config() -> TransformerConfig:
    """Byte-level decoder: 4 layers, d 256, 4 heads x 64, SwiGLU 1024, vocab 256, ctx 128,
    OIL8 with a 256-entry codebook per 64-weight block."""
    return TransformerConfig(vocab_size=256, hidden_size=256, num_layers=4, num_heads=4, head_dim=64,
                             ffn_hidden_size=1024, max_seq_len=128, weight_format="oil8", oil_block_size=64)


def llama_1p3b_config() -> TransformerConfig:
    """Dense 1.3B: 24 layers, d 2048, 16 heads x 128, SwiGLU 5504, vocab 32000, seq 2048, OIL8 STE."""
    return TransformerConfig(vocab_size=32000, hidden_size=2048, num_layers=24, num_heads=16, head_dim=128,
                             ffn_hidden_size=5504, max_seq_len=2048, rope_theta=10000.0, weight_format="oil8",
                             oil_block_size=256, codebook_group=128)


def moe_8x_config() -> TransformerConfig:
    """MoE: 16 layers, d 2048, 16 heads, 8 experts top-2, expert SwiGLU 5632, aux 0.01, OIL8 on experts."""
    return TransformerConfig(vocab_size=32000, hidden_size=2048, num_layers=16, num_heads=16, head_dim=128,
                             ffn_hidden_size=5632, moe_ffn_hidden_size=5632, max_seq_len=2048, num_experts=8,
                             moe_top_k=2, moe_aux_coef=0.01, weight_format="oil8", attn_format="fp32",
                             oil_block_size=256, codebook_group=128)


def llama3_8b_config() -> TransformerConfig:
    """Llama-3-8B shape, mixed OIL4 (attention) / OIL8 (FFN, embeddings)."""
    return TransformerConfig(vocab_size=128256, hidden_size=4096, num_layers=32, num_heads=32, head_dim=128,
                             num_kv_heads=8, ffn_hidden_size=14336, max_seq_len=8192, rope_theta=500000.0,
                             weight_format="oil8", attn_format="oil4", ffn_format="oil8", embed_format="oil8",
                             oil_block_size=256, codebook_group=128)


def bitnet_2p4b_config() -> TransformerConfig:
    """BitNet-style 2.4B: 30 layers, d 2560, 20 heads x 128, FFN 6912 squared-ReLU (gated), I2_S ternary."""
    return TransformerConfig(vocab_size=128256, hidden_size=2560, num_layers=30, num_heads=20, head_dim=128,
                             ffn_hidden_size=6912, max_seq_len=32768 + 512, activation="relu2", gated_ffn=True,
                             weight_format="i2s", embed_format="fp16", oil_block_size=256)


NAMED_CONFIGS = {
    "tiny-byte": tiny_byte_config,
    "llama-1.3b": llama_1p3b_config,
    "moe-8x": moe_8x_config,
    "llama3-8b": llama3_8b_config,
    "bitnet-2.4b": bitnet_2p4b_config,
}
