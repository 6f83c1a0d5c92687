"""Head geometry of the full-attention layers, the only part of the reference's ModelConfig
(tokenrush/config.py:8-29) that the attention / KV path reads."""
from dataclasses import dataclass, field


@dataclass(frozen=True)
class AttnConfig:
    n_heads: int = 24
    n_kv_heads: int = 4
    head_dim: int = 256
    rotary_dim: int = 64
    rope_theta: float = 1e7
    eps: float = 1e-6
    n_attn: int = 16                      # full-attention layers that own a KV cache
    attn_layers: tuple = field(default=None)

    def __post_init__(self):
        if self.attn_layers is None:
            # layer i of every group of four is full attention (tokenrush/config.py:63-64)
            object.__setattr__(self, "attn_layers", tuple(4 * i + 3 for i in range(self.n_attn)))
