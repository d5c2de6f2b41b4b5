"""Several mixers side by side on the same input: sum_i scale_i * branch_i(h). Each branch is a mixer of the
registry with its own tensors under its own prefix. The branches' per-request states lie one after the other in
one state slot, and at most one branch may want pages, so that the cache entry of the layer serves them all.
The sum costs no kernel: a branch folds its factor into a kernel it launches anyway (``Mixer.forward_scaled``)
and its output projection adds what the branches before it gave. Branches that say which rows their input
product has (``Mixer.input_rows``) share ONE product of all those rows, and each reads its columns of the result.
"""
from __future__ import annotations

import torch

from .base import Mixer, StateNeed, build_mixer, register_mixer


class ParallelMixer(Mixer):
    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        if not spec.branches or not len(spec.branches) == len(spec.scales) == len(spec.prefixes):
            raise ValueError("a parallel mixer needs branches, each with a scale and a prefix")
        self.branches = [build_mixer(b, dtype, device) for b in spec.branches]
        if sum(1 for b in self.branches if b.cache_need() is not None) > 1:
            raise ValueError("at most one branch of a parallel mixer may keep pages")
        for b in self.branches:
            need = b.state_need()
            if need is not None and (need.dtype != torch.float32 or len(need.shape) != 1):
                raise ValueError("the branches of a parallel mixer keep their state as one row of float32")
        self.graph_safe = all(b.graph_safe for b in self.branches)

    def parts(self):
        return list(self.branches)

    def cache_need(self):
        for b in self.branches:
            if b.cache_need() is not None:
                return b.cache_need()
        return None

    def _state_sizes(self):
        return [b.state_need().shape[0] if b.state_need() is not None else 0 for b in self.branches]

    def state_need(self):
        total = sum(self._state_sizes())
        return StateNeed((total,), torch.float32) if total else None

    def tensors(self):
        return {prefix + local: ts for b, prefix in zip(self.branches, self.spec.prefixes)
                for local, ts in b.tensors().items()}

    def load(self, tensors):
        for b, prefix in zip(self.branches, self.spec.prefixes):
            b.load({local: tensors[prefix + local] for local in b.tensors()})
        # one product for the input rows of all branches that can take its result (at least two of them)
        self.w_in = self.b_in = None
        self.offsets = [None] * len(self.branches)
        rows = [b.input_rows() for b in self.branches]
        if sum(r is not None for r in rows) >= 2:
            weights, biases, at = [], [], 0
            for i, r in enumerate(rows):
                if r is None:
                    continue
                self.offsets[i] = at
                weights.append(r[0])
                biases.append(r[1] if r[1] is not None else torch.zeros(r[0].shape[0], dtype=torch.float32, device=r[0].device))
                at += r[0].shape[0]
            self.w_in = torch.cat(weights, dim=0).contiguous()
            if any(r is not None and r[1] is not None for r in rows):
                self.b_in = torch.cat(biases).contiguous()
            for b, r in zip(self.branches, rows):
                if r is not None:
                    b.drop_input_rows()

    def _views(self, cache):
        from ..engine.batch import CacheView
        views, at = [], 0
        for b, n in zip(self.branches, self._state_sizes()):
            state = cache.state[:, at:at + n] if n else None
            at += n
            keeps_pages = b.cache_need() is not None
            views.append(CacheView(cache.kv if keeps_pages else None, cache.block_table if keeps_pages else None,
                                   cache.page_size, cache.writes, state))
        return views

    def forward(self, x, step, cache):
        return self.forward_residual(x, None, step, cache)

    def forward_residual(self, x, residual, step, cache):
        return self.forward_scaled(x, 1.0, residual, step, cache)

    def forward_scaled(self, x, scale, residual, step, cache):
        from .. import ops
        projected = ops.linear(x, self.w_in, bias=self.b_in) if getattr(self, "w_in", None) is not None else None
        out = residual
        for i, (b, own, view) in enumerate(zip(self.branches, self.spec.scales, self._views(cache))):
            factor = float(scale) * float(own)
            if projected is not None and self.offsets[i] is not None:
                out = b.forward_projected(projected, self.offsets[i], x, factor, out, step, view)
            else:
                out = b.forward_scaled(x, factor, out, step, view)
        return out


register_mixer("parallel", ParallelMixer)
