"""Mixture-of-experts feed-forward: a float32 router picks, per token, the ``top`` experts with the largest
softmax scores; their outputs are weighted by those scores over their sum; optionally a shared expert runs for
every token. An expert is down(act(up h)), act(v) = max(v, 0)^2, no biases.

A step's (token, choice) pairs are put in expert order on the device and the experts run as two grouped
products over row tiles; nothing is read back to the host and no token is ever dropped, so a token's result
does not depend on what else is in the batch. The part sits in blocks whose norm follows the sublayer
(``forward_stream``): the weighted sum, the shared expert's term, the norm and the float32 residual sum are
one kernel.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorSpec, register_feed_forward


class Experts(FeedForward):
    graph_safe = True

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.activation != "relu_squared":
            raise ValueError(f"activation {spec.activation!r} is not supported (relu_squared only)")
        self.w_router = self.w_up = self.w_down = self.w_shared_up = self.w_shared_down = None

    def tensors(self):
        s = self.spec
        t = {}
        for e in range(s.num_experts):
            t[f"e{e}.up"] = TensorSpec((s.expert_size, s.hidden_size))
            t[f"e{e}.down"] = TensorSpec((s.hidden_size, s.expert_size))
        t["router"] = TensorSpec((s.num_experts, s.hidden_size))
        if s.shared_size:
            t["shared.up"] = TensorSpec((s.shared_size, s.hidden_size))
            t["shared.down"] = TensorSpec((s.hidden_size, s.shared_size))
        return t

    def load(self, tensors):
        s = self.spec
        self.w_up = torch.stack([tensors[f"e{e}.up"] for e in range(s.num_experts)]).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(s.num_experts)]).contiguous()
        self.w_router = tensors["router"].contiguous()
        if s.shared_size:
            self.w_shared_up = tensors["shared.up"].contiguous()
            self.w_shared_down = tensors["shared.down"].contiguous()

    def _experts(self, x32, x):
        """(routing, float32 sorted rows of the experts' outputs, the shared expert's output or None)."""
        s = self.spec
        # the more rows an expert gets, the taller the row tiles its grouped products are planned with
        routing = ops.route_experts(x32, self.w_router, s.top, s.weight_eps,
                                    tile_rows=ops.expert_tile_rows(x, s.num_experts, s.top, s.expert_size))
        hidden = ops.expert_linear(x, self.w_up, routing, up=True)
        down = ops.expert_linear(hidden, self.w_down, routing, up=False)
        shared = None
        if s.shared_size:
            shared = ops.linear(ops.relu_squared(ops.linear(x, self.w_shared_up)), self.w_shared_down)
        return routing, down, shared

    def forward_stream(self, x32, x, norm, step):
        """x32 += norm(feed_forward(x)) for a float32 stream ``x32`` with its copy ``x`` in the compute dtype;
        returns the new (x32, copy). The router reads the float32 rows."""
        rms = norm.as_rms()
        if rms is None:
            raise ValueError("the experts' fused output needs an RMSNorm behind them")
        routing, down, shared = self._experts(x32, x)
        return ops.experts_combine_norm_add(x32, down, shared, routing, rms[0], rms[1], self.dtype)

    def forward(self, x, step=None):
        """The plain sum, for arrangements that keep the stream in the compute dtype."""
        x32 = x if x.dtype == torch.float32 else x.float()
        routing, down, shared = self._experts(x32, x)
        rows = down[routing.slot_of.long().view(-1)].view(x.shape[0], self.spec.top, -1)
        out = (rows * routing.weight[:, :, None]).sum(dim=1)
        if shared is not None:
            out = out + shared.float()
        return out.to(x.dtype)


register_feed_forward("experts", Experts)
