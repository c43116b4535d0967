"""Token embedding plus a hashed embedding of the (previous token, token) pair.

    x_t = embed[id_t] + pair[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets]

A sequence's first token takes the pair table's extra last row (index `buckets`).  The previous token of a portion's
first token is the last token of the sequence's previous step: it lives in a slot of the state pool (`prev_token`
int32 [slots, 1]), so steps of any cut - also CUDA-graph replays - need nothing from the host.  The sum is fp32 (the
start of a 32-bit residual stream).  Kernel: `cvllm_pair_hash_embed` (csrc/blocks.cu).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from compactor_vllm import _native as N
from compactor_vllm.config.constants import RESERVED_BATCH
from compactor_vllm.utils.context import get_context


class HashedPairEmbedding(nn.Module):
    def __init__(self, vocab: int, width: int, buckets: int, mul_prev: int, mul_cur: int):
        super().__init__()
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        self.tokens = nn.Embedding(vocab, width)
        self.pairs = nn.Embedding(self.buckets + 1, width)
        self.prev_token: Optional[torch.Tensor] = None    # injected by the state pool: int32 [slots, 1]

    def state_specs(self, dtype: torch.dtype):
        return {"prev_token": ((1,), torch.int32)}

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        """ids int64 [T] of the step -> fp32 [T, width]; positions and slots come from the step's context."""
        ctx = get_context()
        assert self.prev_token is not None, "state pool must be initialized"
        assert input_ids.dtype == torch.int64 and input_ids.is_contiguous()
        T, W = input_ids.numel(), self.tokens.weight.shape[1]
        w = self.tokens.weight
        out = torch.empty((T, W), dtype=torch.float32, device=w.device)
        N.check(N.lib().cvllm_pair_hash_embed(
            N.ptr(input_ids), N.ptr(ctx.positions_i32), N.ptr(ctx.token_slot), N.ptr(w), N.ptr(self.pairs.weight),
            self.buckets, self.mul_prev, self.mul_cur, N.ptr(self.prev_token), N.ptr(out), out.stride(0), T, W,
            RESERVED_BATCH, N.block_dtype_code(w.dtype), N.stream(w.device)), "cvllm_pair_hash_embed")
        return out
