"""Mixture-of-experts feed-forward: a router picks ``top`` of ``experts`` small feed-forwards per token.

Router: ``z = x Wr^T + br`` in float32; the ``top`` largest logits choose the experts and their weights are the
softmax over the chosen logits only.  Expert: ``Wd act(Wu x)`` (not gated, no biases).  Output: the weighted sum of the
chosen experts, plus, when the layer has one, a shared expert of the same form (with a width of its own) that every
token runs.  (The reference has dense layers only.)

Nothing comes back to the host: the router's choices are grouped by expert on the device, the experts run as one
grouped product over the groups' tiles (launch sizes are upper bounds), and each token's choices are summed in
the router's order, so a token's output does not depend on what else is in the step, and steps of single tokens
replay as a graph.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.base import UnsupportedError
from ..weights.loader import TensorSpec, fused_rows
from .base import FeedForward, register_part


class MoeFfn(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, experts: int, top: int, expert_size: int, prefix: str, activation: str = "relu2",
                 router_bias: bool = True, shared_size: int = 0, names=None, **_):
        self.E, self.n, self.top, self.F, self.FS = int(hidden_size), int(experts), int(top), int(expert_size), int(shared_size or 0)
        if not 1 <= self.top <= self.n:
            raise UnsupportedError(f"mixture of experts: top {self.top} of {self.n} experts")
        if activation not in kernels.ACTIVATIONS:
            raise UnsupportedError(f"mixture of experts: activation '{activation}' is not supported")
        self.activation, self.router_bias = activation, bool(router_bias)
        n = {"router": "router", "router_bias": "router.b", "expert": "e{}", "shared": "shared", "up": "up", "down": "down"}
        n.update(names or {})
        self.prefix, self.nm = prefix, n
        self.w_router = self.b_router = self.w_up = self.w_down = self.ws_up = self.ws_down = None

    def _expert(self, i, which):
        return f"{self.prefix}.{self.nm['expert'].format(i)}.{self.nm[which]}"

    def tensor_specs(self):
        s = [TensorSpec(f"{self.prefix}.{self.nm['router']}", (self.n, self.E))]
        if self.router_bias:
            s.append(TensorSpec(f"{self.prefix}.{self.nm['router_bias']}", (self.n,)))
        for i in range(self.n):
            s += [TensorSpec(self._expert(i, "up"), (self.F, self.E)), TensorSpec(self._expert(i, "down"), (self.E, self.F))]
        if self.FS:
            p = f"{self.prefix}.{self.nm['shared']}"
            s += [TensorSpec(f"{p}.{self.nm['up']}", (self.FS, self.E)), TensorSpec(f"{p}.{self.nm['down']}", (self.E, self.FS))]
        return s

    def bind(self, tensors, run_dtype, device):
        self.w_router = tensors[f"{self.prefix}.{self.nm['router']}"].contiguous()
        if self.router_bias:
            self.b_router = tensors[f"{self.prefix}.{self.nm['router_bias']}"].to(self.w_router.dtype).contiguous()
        # all experts' matrices in one array each, [experts, out, in], filled a tensor at a time
        self.w_up = fused_rows(tensors, [self._expert(i, "up") for i in range(self.n)], device).view(self.n, self.F, self.E)
        self.w_down = fused_rows(tensors, [self._expert(i, "down") for i in range(self.n)], device).view(self.n, self.E, self.F)
        if self.FS:
            p = f"{self.prefix}.{self.nm['shared']}"
            self.ws_up = tensors[f"{p}.{self.nm['up']}"].contiguous()
            self.ws_down = tensors[f"{p}.{self.nm['down']}"].contiguous()

    def weight_bytes(self):
        """What a step of one token reads: the router, ``top`` experts and the shared expert."""
        per = lambda w: w.numel() * w.element_size()
        b = per(self.w_router) + (per(self.w_up) + per(self.w_down)) * self.top // self.n
        return b + (per(self.ws_up) + per(self.ws_down) if self.FS else 0)

    def flops(self, rows):
        return 2.0 * rows * (self.n * self.E + 2 * self.top * self.E * self.F + 2 * self.E * self.FS)

    def _experts(self, ctx, xn):
        """Router, grouping and the routed experts: (outputs of every (token, choice) [T * top, E] float32, weights [T, top])."""
        T, P = xn.shape[0], xn.shape[0] * self.top
        i32 = torch.int32
        ids = ctx.buf("moe_ids", (T, self.top), i32)
        wts = ctx.buf("moe_weights", (T, self.top), torch.float32)
        z = ctx.buf("moe_logits", (T, self.n), torch.float32)
        with kernels.phase("glue"):
            kernels.moe_route(xn, self.w_router, self.b_router, self.top, ids, wts, z)
            mt = kernels.moe_max_tiles(P, self.n)
            order = ctx.buf("moe_order", (P,), i32)
            tiles = [ctx.buf(f"moe_tile{k}", (mt,), i32) for k in range(3)]
            n_tiles = ctx.buf("moe_n_tiles", (1,), i32)
            kernels.moe_group(ids, self.n, order, *tiles, n_tiles)
        h = ctx.buf("moe_h", (P, self.F), xn.dtype)
        y = ctx.buf("moe_y", (P, self.E), xn.dtype if xn.dtype == torch.float32 else torch.float32)
        with kernels.phase("gate_up"):
            kernels.moe_gemm(xn, self.w_up, h, self.activation, order, self.top, False, *tiles, n_tiles, P)
        with kernels.phase("down"):
            kernels.moe_gemm(h, self.w_down, y, "none", order, 0, True, *tiles, n_tiles, P)
        return y, wts

    def _shared_hidden(self, ctx, xn):
        hs = ctx.buf("moe_hs", (xn.shape[0], self.FS), xn.dtype)
        with kernels.phase("gate_up"):
            kernels.linear_act(xn, self.ws_up, hs, self.activation)
        return hs

    def forward_into_norm(self, ctx, xn, y_buf, residual, post, next_norm, out):
        """residual += post(feed-forward output): the weighted sum of the chosen experts, the shared expert's down
        product and its partial sums are all summed by the norm's own pass."""
        mix = self._experts(ctx, xn)
        if not self.FS:
            return post.add_into(None, residual, next_norm, out, mix=mix)
        hs = self._shared_hidden(ctx, xn)
        with kernels.phase("down"):
            return post.add_product_into(hs, self.ws_down, None, y_buf, residual, next_norm, out, mix=mix)

    def forward(self, ctx, xn, residual, accumulate=True):
        T = xn.shape[0]
        y, wts = self._experts(ctx, xn)
        out = residual
        if accumulate:
            out = ctx.buf("moe_out", residual.shape, torch.float32)
        with kernels.phase("glue"):
            kernels.moe_combine(y, wts, out)
        if self.FS:
            hs = self._shared_hidden(ctx, xn)
            with kernels.phase("down"):
                kernels.linear(hs, self.ws_down, None, out, accumulate=True)
        if accumulate:
            residual.add_(out)


register_part("ffn", "moe", MoeFfn)
