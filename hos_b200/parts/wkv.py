"""A linear-recurrence mixer with a matrix state per head (time mixing in the manner of RWKV).

With h' the previous token's input row (zeros for a sequence's first token), each of r, k, v, g, w
reads its own mix h + (h' - h) * mu_s.  r, k, v = W_r, W_k, W_v of their mixes ([heads x dim]),
gate = silu(W_g mix_g), decay w = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0)) per head and key channel.
Per head, with S [dim keys x dim values] starting at zero:
    o_t = (S_{t-1} + diag(u) k_t v_t^T)^T r_t          (u: a bonus for the current token only)
    S_t = diag(w_t) S_{t-1} + k_t v_t^T
Each head's o is divided by its root mean square (eps inside the root), then times `norm`, times
the gate, then W_o.  State per sequence: S (32-bit) and the last input row (for the next step's
h').  The mixes, the decay, the recurrence and the head norm are 32-bit; r, k, v, g and the decay's
low-rank projection come out of the products in 32-bit.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from .. import ops
from ..errors import SpecError
from ..registry import register_part
from . import linear
from .base import CallStore, Mixer, StateNeed, StepInfo, WeightSpec

MIXES = ("r", "k", "v", "g", "w")


class MatrixStateRecurrence(Mixer):
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = spec.params
        self.width, self.n_heads, self.dim = int(p["width"]), int(p["n_heads"]), int(p["dim"])
        self.decay_rank = int(p["decay_rank"]) if p.get("decay_rank") else -1     # -1: the w1 tensor's shape gives it
        self.eps = float(p["eps"])
        if min(self.width, self.n_heads, self.dim) <= 0:
            raise SpecError("arch spec error: the recurrence needs positive sizes")
        self.cols = self.n_heads * self.dim

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        out = [WeightSpec(w["mu_" + s], (self.width,), "vector", 0.3) for s in MIXES]
        out += [WeightSpec(w[s], (self.cols, self.width), "matrix", 0.05) for s in ("r", "k", "v", "g")]
        out += [WeightSpec(w["w1"], (self.decay_rank, self.width), "matrix", 0.05),
                WeightSpec(w["w2"], (self.cols, self.decay_rank), "matrix", 0.1),
                WeightSpec(w["w0"], (self.cols,), "vector", 0.5),
                WeightSpec(w["u"], (self.n_heads, self.dim), "vector", 0.3),
                WeightSpec(w["norm"], (self.cols,), "vector", 0.1),
                WeightSpec(w["o"], (self.width, self.cols), "matrix", 0.02)]
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        w = self.spec.weights
        self.mu = torch.stack([self._vector32(tensors[w["mu_" + s]]) for s in MIXES]).contiguous()     # [5, width]
        self.w_proj = [self._matrix(tensors[w[s]]) for s in ("r", "k", "v", "g")]
        self.w1, self.w2 = self._matrix(tensors[w["w1"]]), self._matrix(tensors[w["w2"]])
        if self.w1.shape[0] != self.w2.shape[1]:
            raise SpecError(f"arch spec error: the decay's two projections do not fit ({tuple(self.w1.shape)}, "
                            f"{tuple(self.w2.shape)})")
        self.w0 = self._vector32(tensors[w["w0"]])
        self.u = self._vector32(tensors[w["u"]]).reshape(-1).contiguous()
        self.norm_w = self._vector32(tensors[w["norm"]])
        self.w_o = self._matrix(tensors[w["o"]])

    def state_needs(self) -> List[StateNeed]:
        return [StateNeed("S", (self.n_heads, self.dim, self.dim), torch.float32),
                StateNeed("last_row", (self.width,), torch.float32)]

    def forward(self, h: torch.Tensor, step: StepInfo, store: CallStore) -> torch.Tensor:
        n = h.shape[0]
        S, kept = store.state["S"], store.state["last_row"]
        mixes = ops.token_shift(h, kept, self.mu, step)
        r, k, v, g = (linear.matmul(mixes[i], self.w_proj[i], out_dtype=torch.float32) for i in range(4))
        low = linear.matmul(mixes[4], self.w1, out_dtype=torch.float32)
        t = torch.empty(low.shape, dtype=h.dtype, device=h.device)
        ops.tanh_rows(low, t)
        wx = linear.matmul(t, self.w2, out_dtype=torch.float32)
        y = torch.empty((n, self.cols), dtype=h.dtype, device=h.device)
        ops.wkv_scan(r, k, v, wx, g, self.w0, self.u, self.norm_w, self.eps, S, kept, h, step, y, self.n_heads, self.dim)
        return linear.matmul(y, self.w_o)


register_part("mixer", "matrix_state_recurrence", MatrixStateRecurrence)
