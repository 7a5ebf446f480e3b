"""Token embedding (row gather into the float32 residual, src/model.c:566-571), its form with a scale and a hashed
pair term, and the output head
(final norm rows times the head matrix, float32 logits, src/model.c:629-637; tied head = the
embedding matrix, src/model.c:156-158)."""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import TensorSpec
from .base import Part, StateSpec, register_part


class Embedding(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, tensor: str, **_):
        self.vocab_size, self.hidden_size, self.tensor = int(vocab_size), int(hidden_size), tensor
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.tensor, (self.vocab_size, self.hidden_size))]

    def bind(self, tensors, run_dtype, device):
        self.table = tensors[self.tensor].contiguous()

    def state_spec(self):
        """Per-request state the embedding keeps between steps (none here)."""
        return None

    def forward(self, token_ids: torch.Tensor, out: torch.Tensor, ctx=None, state=None) -> torch.Tensor:
        with kernels.phase("embed"):
            kernels.embed(token_ids, self.table, out)
        return out


class HashedPairEmbedding(Embedding):
    """``x = table[token] * scale + pair[row]``: ``row`` hashes the token with the one before it in its request,
    ``(previous * mul_prev + token * mul_cur) mod buckets``; a request's first token takes row ``buckets``, the last of
    the pair table.  The previous token is per-request state (one int32: token + 1, 0 while the request has none), since
    a step may bring only the next token of a request; the kernel keeps it up to date on the device, so that steps
    whose tokens the host has not seen (ids fed from the sampling kernel) find it too.  ``buckets`` = 0: no pair term."""
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, tensor: str, scale: float = 1.0, pair_tensor=None, buckets: int = 0,
                 mul_prev: int = 0, mul_cur: int = 0, **_):
        super().__init__(vocab_size, hidden_size, tensor)
        self.scale, self.pair_tensor = float(scale), pair_tensor
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        if (self.buckets > 0) != bool(pair_tensor):
            raise ValueError("the pair term needs both its table and its number of buckets")
        self.pair = None

    def tensor_specs(self):
        specs = super().tensor_specs()
        if self.pair_tensor:
            specs.append(TensorSpec(self.pair_tensor, (self.buckets + 1, self.hidden_size)))
        return specs

    def bind(self, tensors, run_dtype, device):
        super().bind(tensors, run_dtype, device)
        if self.pair_tensor:
            self.pair = tensors[self.pair_tensor].contiguous()

    def state_spec(self):
        return StateSpec((), torch.int32) if self.pair_tensor else None

    def forward(self, token_ids, out, ctx=None, state=None):
        if self.pair is not None and (ctx is None or state is None):
            raise ValueError("this embedding needs the step's context and its per-request state")
        with kernels.phase("embed"):
            kernels.embed_pair(token_ids, self.table, self.scale, self.pair, self.buckets, self.mul_prev, self.mul_cur, ctx,
                               state, out)
        return out


class LinearHead(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, hidden_size: int, tensor: str, tied_to=None, scale: float = 1.0, **_):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.tensor, self.tied_to = tensor, tied_to
        self.scale = float(scale)               # logits = (head . x) * scale
        self.weight = None

    def tensor_specs(self):
        # a tied head reads the embedding; a checkpoint that carries a copy of the head anyway is accepted
        shape = (self.vocab_size, self.hidden_size)
        specs = [TensorSpec(self.tensor, shape, optional=bool(self.tied_to))]
        if self.tied_to:
            specs.append(TensorSpec(self.tied_to, shape))       # declared by both: the loader makes it once
        return specs

    def bind(self, tensors, run_dtype, device):
        self.weight = tensors[self.tied_to if self.tied_to else self.tensor].contiguous()

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def flops(self, rows):
        return 2.0 * rows * self.weight.numel()

    def forward(self, xn: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        with kernels.phase("head"):
            kernels.linear(xn, self.weight, None, logits, accumulate=False)
            if self.scale != 1.0:
                kernels.scale_(logits, self.scale)
        return logits


register_part("embedding", "embedding", Embedding)
register_part("embedding", "hashed_pair_embedding", HashedPairEmbedding)
register_part("head", "linear_head", LinearHead)
