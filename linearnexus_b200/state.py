"""Decode caches: the recurrent state ``S [B, H, d_k, d_v]`` (float32) plus the short-conv caches.

Mirrors ``DeltaNetState`` (modules/linear_attn/delta_net.py:81-118), ``GatedDeltaNetState``
(modules/linear_attn/gated_deltanet.py:72-128) and ``KDAState`` (modules/linear_attn/kda.py:57-113):
same field names, same ``zeros`` factory arguments, float32 contents.  ``S`` is the buffer the
decode kernel updates in place (``*_step(..., inplace=True)``); ``device`` is the one extra
argument (torch needs to know where the cache lives).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class DeltaNetState:
    S: torch.Tensor                            # [batch, heads, key_dim, value_dim]
    conv_state: Optional[torch.Tensor] = None  # [batch, kernel-1, channels]

    @classmethod
    def zeros(cls, batch_size: int, num_heads: int, key_dim: int, value_dim: int,
              conv_channels: Optional[int] = None, conv_size: int = 4, device="cuda") -> "DeltaNetState":
        S = torch.zeros(batch_size, num_heads, key_dim, value_dim, dtype=torch.float32, device=device)
        conv_state = None
        if conv_channels is not None:
            conv_state = torch.zeros(batch_size, conv_size - 1, conv_channels, dtype=torch.float32, device=device)
        return cls(S=S, conv_state=conv_state)


@dataclass
class GatedDeltaNetState:
    S: torch.Tensor  # [batch, num_v_heads, key_dim_per_head, value_dim_per_head]
    conv_state_q: Optional[torch.Tensor] = None
    conv_state_k: Optional[torch.Tensor] = None
    conv_state_v: Optional[torch.Tensor] = None

    @classmethod
    def zeros(cls, batch_size: int, num_v_heads: int, key_dim_per_head: int, value_dim_per_head: int,
              key_dim_total: Optional[int] = None, value_dim: Optional[int] = None, conv_size: int = 4,
              use_conv: bool = True, device="cuda"):
        z = lambda *s: torch.zeros(*s, dtype=torch.float32, device=device)
        S = z(batch_size, num_v_heads, key_dim_per_head, value_dim_per_head)
        cq = ck = cv = None
        if use_conv and key_dim_total is not None and value_dim is not None:
            cq = z(batch_size, conv_size - 1, key_dim_total)
            ck = z(batch_size, conv_size - 1, key_dim_total)
            cv = z(batch_size, conv_size - 1, value_dim)
        return cls(S=S, conv_state_q=cq, conv_state_k=ck, conv_state_v=cv)


@dataclass
class KDAState(GatedDeltaNetState):
    """Same fields and factory as GatedDeltaNetState (kda.py:57-113)."""
