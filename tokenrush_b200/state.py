"""Preallocated KV state, the attention half of the reference's `State`
(tokenrush/state.py:13-75): one contiguous cache `[layer, kv_head, position, head_dim]` in
bf16 or e4m3 with fp32 per-(head, position) scales, and the position as a device tensor with
a host mirror.  The GDN fields of the reference's State belong to other layers and are not
kept here."""
from __future__ import annotations

import torch


class State:
    def __init__(self, cfg, max_len: int, device="cuda", kv_dtype=torch.bfloat16, n_slots: int = 1,
                 shard_lo=None, pos_dtype=torch.long):
        """cfg: anything with n_kv_heads, head_dim and attn_layers (the reference's ModelConfig
        or tokenrush_b200.config.AttnConfig).  shard_lo: first position held by this cache
        when the sequence is sharded over several GPUs (None: a whole cache)."""
        layers = list(cfg.attn_layers)
        n_attn = len(layers)
        self.max_len = max_len
        self.kv_dtype = kv_dtype
        self.fp8 = kv_dtype == torch.float8_e4m3fn
        self.shard_lo = shard_lo
        self.k = torch.zeros(n_attn, cfg.n_kv_heads, max_len, cfg.head_dim, device=device, dtype=kv_dtype)
        self.v = torch.zeros_like(self.k)
        if self.fp8:
            self.k_scale = torch.ones(n_attn, cfg.n_kv_heads, max_len, device=device, dtype=torch.float32)
            self.v_scale = torch.ones_like(self.k_scale)
        else:
            self.k_scale = self.v_scale = None
        self.n_slots = n_slots
        self.pos = 0
        self.pos_t = torch.zeros(1, device=device, dtype=pos_dtype)
        self.attn_slot = {l: i for i, l in enumerate(layers)}

    def reset(self):
        self.pos = 0
        self.pos_t.zero_()

    def advance(self, T: int):
        self.pos += T
        self.pos_t += T

    def set_pos(self, pos: int):
        """Rewind / resume at `pos`: rows beyond it stay in the cache as dead data and are
        overwritten by the next append (tokenrush/mtp.py:84-87, tokenrush/session.py:94-95)."""
        self.pos = pos
        self.pos_t.fill_(pos)

    @property
    def nbytes(self):
        ts = [self.k, self.v] + ([self.k_scale, self.v_scale] if self.fp8 else [])
        return sum(t.numel() * t.element_size() for t in ts)

    @property
    def kv_bytes_per_token(self):
        n_attn = self.k.shape[0]
        b = 2 * n_attn * self.k.shape[1] * self.k.shape[3] * self.k.element_size()
        if self.fp8:
            b += 2 * n_attn * self.k.shape[1] * 4
        return b
