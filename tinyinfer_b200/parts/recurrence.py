"""Recurrent mixer with a real-gated diagonal linear recurrence (the recurrent block of Griffin, De, Smith et al.
2024): two branches of ``width`` channels, y = gelu_tanh(W_y h + b_y) and u = conv(W_x h + b_x), a causal
per-channel convolution; gates r = sigmoid(A_r[b] u_b + b_r), i = sigmoid(A_i[b] u_b + b_i) per block b of
channels; a = exp(-decay * r * softplus(lam)); S <- a S + sqrt(1 - a^2) * i * u; out = W_o (S * y).

Per request the mixer keeps, in its state slot, S and the convolution's last taps - 1 inputs (float32
[taps, width]: row 0 is S); a slot is zero when a request starts, which is both "S = 0" and "zeros before the
start". Gates, decays and the state are float32; the projections and the convolution run in the compute dtype.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, StateNeed, TensorSpec, register_mixer


class GatedRecurrence(Mixer):
    graph_safe = True

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.width % spec.blocks:
            raise ValueError(f"{spec.width} channels do not split into {spec.blocks} equal blocks")
        self.w_yx = self.b_yx = self.conv_w = self.conv_b = self.w_gates = self.b_gates = self.lam = self.w_o = None

    def state_need(self):
        return StateNeed((self.spec.conv_taps, self.spec.width), torch.float32)

    def tensors(self):
        s = self.spec
        bw = s.width // s.blocks
        return {
            "y": TensorSpec((s.width, s.hidden_size)), "y.b": TensorSpec((s.width,), role="vector32"),
            "x": TensorSpec((s.width, s.hidden_size)), "x.b": TensorSpec((s.width,), role="vector32"),
            "conv": TensorSpec((s.width, s.conv_taps), role="vector32"),
            "conv.b": TensorSpec((s.width,), role="vector32"),
            "ra": TensorSpec((s.blocks, bw, bw)), "ra.b": TensorSpec((s.blocks, bw), role="vector32"),
            "ri": TensorSpec((s.blocks, bw, bw)), "ri.b": TensorSpec((s.blocks, bw), role="vector32"),
            "lam": TensorSpec((s.width,), role="vector32"),
            "o": TensorSpec((s.hidden_size, s.width)),
        }

    def load(self, tensors):
        self.w_yx = torch.cat([tensors["y"], tensors["x"]], dim=0).contiguous()
        self.b_yx = torch.cat([tensors["y.b"], tensors["x.b"]]).contiguous()
        self.conv_w = tensors["conv"].contiguous()
        self.conv_b = tensors["conv.b"]
        # per block [r rows ; i rows]: one batched product gives both gates
        self.w_gates = torch.cat([tensors["ra"], tensors["ri"]], dim=1).contiguous()
        self.b_gates = torch.cat([tensors["ra.b"], tensors["ri.b"]], dim=1).contiguous()
        self.lam = tensors["lam"]
        self.w_o = tensors["o"].contiguous()

    def forward(self, x, step, cache):
        s = self.spec
        bw = s.width // s.blocks
        yx = ops.linear(x, self.w_yx, bias=self.b_yx)                  # [T, y | x]
        u = ops.causal_conv(yx, offset=s.width, width=s.width, state=cache.state, weight=self.conv_w,
                            bias=self.conv_b, token_seq=step.token_seq, cu_seqlens=step.cu_seqlens,
                            state_slots=step.state_slots)
        gates = ops.batched_linear(u, self.w_gates, x_batch_stride=bw, k=bw, bias=self.b_gates, sigmoid=True,
                                   out_float32=True)                   # float32 [T, blocks * (r | i)]
        mixed = ops.gated_scan(u, gates, yx, y_offset=0, x_offset=s.width, state=cache.state, lam=self.lam,
                               block_width=bw, decay=s.decay, cu_seqlens=step.cu_seqlens,
                               state_slots=step.state_slots, num_seqs=step.num_seqs)
        return ops.linear(mixed, self.w_o)


register_mixer("gated_recurrence", GatedRecurrence)
