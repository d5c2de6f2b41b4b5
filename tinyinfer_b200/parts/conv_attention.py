"""Grouped-query softmax attention whose q, k and v pass a short causal convolution over time, without a rotation:
packed projection [q | k | v] with biases, the convolution per channel (its last taps - 1 inputs per request live
in the request's state slot), a query temperature that grows with the logarithm of the position, scores
(q . k) * scale over the request's cached keys and values (which may differ in size), a softmax whose
denominator may hold one more term exp(sink) without a value, and the output projection.

Convolution, temperature, scores and softmax are float32; q and the cached rows are rounded once.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, Mixer, StateNeed, TensorSpec, register_mixer


class ConvAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if spec.conv_taps < 0:
            raise ValueError("conv_taps must not be negative")
        self.w_qkv = self.b_qkv = self.conv_w = self.w_o = self.b_o = None

    # packed channels: [q | k | v]
    @property
    def _sizes(self):
        s = self.spec
        return s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim, s.num_kv_heads * s.v_dim

    def cache_need(self):
        """Keys and values of one size lie in two planes, which is what the tensor-core attention kernels read;
        of different sizes, side by side in one row per token."""
        s = self.spec
        if s.head_dim == s.v_dim:
            return CacheNeed(s.num_kv_heads, s.head_dim, s.window, planes=2)
        return CacheNeed(s.num_kv_heads, s.head_dim + s.v_dim, s.window, planes=1)

    def state_need(self):
        taps = self.spec.conv_taps
        return StateNeed(((taps - 1) * sum(self._sizes),), torch.float32) if taps > 1 else None

    def tensors(self):
        s = self.spec
        nq, nk, nv = self._sizes
        t = {"q": TensorSpec((nq, s.hidden_size)), "k": TensorSpec((nk, s.hidden_size)),
             "v": TensorSpec((nv, s.hidden_size)), "o": TensorSpec((s.hidden_size, s.num_heads * s.v_dim))}
        if s.bias:
            t.update({"q.b": TensorSpec((nq,), role="vector32"), "k.b": TensorSpec((nk,), role="vector32"),
                      "v.b": TensorSpec((nv,), role="vector32"), "o.b": TensorSpec((s.hidden_size,), role="vector32")})
        if s.conv_taps >= 1:
            t.update({"q.conv": TensorSpec((nq, s.conv_taps), role="vector32", init="ones_noise"),
                      "k.conv": TensorSpec((nk, s.conv_taps), role="vector32", init="ones_noise"),
                      "v.conv": TensorSpec((nv, s.conv_taps), role="vector32", init="ones_noise")})
        return t

    def load(self, tensors):
        s = self.spec
        self.w_qkv = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0).contiguous()
        self.w_o = tensors["o"].contiguous()
        if s.bias:
            self.b_qkv = torch.cat([tensors["q.b"], tensors["k.b"], tensors["v.b"]]).contiguous()
            self.b_o = tensors["o.b"]
        if s.conv_taps >= 1:
            # tap by tap, [taps, channels]: neighbouring channels are neighbours in memory, as the kernel reads them
            self.conv_w = torch.cat([tensors["q.conv"], tensors["k.conv"], tensors["v.conv"]], dim=0).t().contiguous()

    def input_rows(self):
        return self.w_qkv, self.b_qkv

    def drop_input_rows(self):
        self.w_qkv = self.b_qkv = None

    def forward_projected(self, projected, offset, x, scale, residual, step, cache):
        bias = self.b_o if self.b_o is None or scale == 1.0 else self._scaled_bias(scale)
        attended = self._attend(x, step, cache, out_scale=scale, qkv=projected, offset=offset)
        return ops.linear(attended, self.w_o, bias=bias, residual=residual)

    def _attend(self, x, step, cache, out_scale=1.0, qkv=None, offset=0):
        s = self.spec
        width = sum(self._sizes)
        if qkv is None:
            qkv = ops.linear(x, self.w_qkv, bias=self.b_qkv)
        history = cache.state.unflatten(1, (s.conv_taps - 1, width)) if s.conv_taps > 1 else None
        single = step.num_tokens == step.num_seqs          # every request brings one token: the kernel keeps the history itself
        q = ops.conv_qkv_append(
            qkv, num_heads=s.num_heads, num_kv_heads=s.num_kv_heads, head_dim=s.head_dim, v_dim=s.v_dim,
            conv_weight=self.conv_w, history=history, temperature=s.query_temperature, positions=step.positions,
            token_seq=step.token_seq, cu_seqlens=step.cu_seqlens, state_slots=step.state_slots,
            cache=cache.kv if cache.writes else None, block_table=cache.block_table, status=step.status,
            shift_history=single and cache.writes, offset=offset)
        if history is not None and cache.writes and not single:
            ops.conv_state_update(history, qkv, offset=offset, width=width, taps=s.conv_taps, cu_seqlens=step.cu_seqlens,
                                  state_slots=step.state_slots, num_seqs=step.num_seqs)
        if cache.kv.shape[0] == 2:          # the paged attention of the plain decoder, tensor cores where the sizes allow
            return ops.paged_attention(q, cache.kv, positions=step.positions, token_seq=step.token_seq,
                                       block_table=cache.block_table, scale=s.scale, window=s.window, step=step,
                                       status=step.status, sink=s.sink, out_scale=out_scale)
        return ops.attention_rows(q, cache.kv, v_dim=s.v_dim, positions=step.positions, token_seq=step.token_seq,
                                  block_table=cache.block_table, scale=s.scale, sink=s.sink, window=s.window,
                                  out_scale=out_scale, step=step, status=step.status)

    def forward(self, x, step, cache):
        return ops.linear(self._attend(x, step, cache), self.w_o, bias=self.b_o)

    def forward_residual(self, x, residual, step, cache):
        return ops.linear(self._attend(x, step, cache), self.w_o, bias=self.b_o, residual=residual)

    def forward_scaled(self, x, scale, residual, step, cache):
        # the factor goes into the attention's output before its rounding, and into the bias
        bias = self.b_o if self.b_o is None or scale == 1.0 else self._scaled_bias(scale)
        return ops.linear(self._attend(x, step, cache, out_scale=scale), self.w_o, bias=bias, residual=residual)

    def _scaled_bias(self, scale):
        kept = getattr(self, "_bias_for", None)
        if kept is None or kept[0] != scale:
            self._bias_for = kept = (scale, (self.b_o * scale).contiguous())
        return kept[1]


register_mixer("conv_attention", ConvAttention)
