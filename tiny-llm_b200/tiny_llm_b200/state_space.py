"""A selective state-space mixer in its dual, attention-like form (Mamba-2): a recurrent mixer whose state lives in fp32 slots.

The input projection of the layer gives, side by side, a gate ``z [inner]``, the values ``x [inner]``, input and output
maps ``B, C [groups * state]`` and a step size per head ``dt [heads]`` (``inner = heads * vdim``).  ``x | B | C`` pass
ONE short causal convolution per channel (with bias) and ``silu``.  Per head (head h reads group ``h // (heads // groups)``)

    dt_t = softplus(dt_t + dt_bias)        S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T        y_t = S_t^T C_t + D x_t

with ``S [state, vdim]``.  The output is multiplied by ``silu(z)`` FIRST and then RMS-normed in ``norm_groups`` equal parts,
each by its own root mean square, times ``norm_weight [inner]``; then the output projection.  Seen as linear attention,
``C`` is the query, ``dt B`` the key and ``x`` the value, so the recurrence runs on ``blocks.decay_scan`` (one decay per
head and token, a skip term ``D x``); long portions run as parallel segments like those of the other mixers on that kernel.
The caller makes the projections (gate and ``x | B | C`` as views of one fused product, ``dt`` with its fp32 accumulator);
step size, decay, recurrence and norm are fp32 whatever the compute dtype.  A request's state is two blocks of its slot:
``state [slots, heads, state, vdim]`` and the convolution's last ``K - 1`` inputs ``conv_state [slots, channels, K - 1]``.
"""

from __future__ import annotations

import torch

from .basics import linear_wide


class StateSpaceMixer:
    def __init__(self, *, heads: int, vdim: int, state: int, groups: int, norm_groups: int, taps, conv_bias, dt_bias, a_log, skip, norm_weight, w_o,
                 eps: float = 1e-6):
        self.heads, self.vdim, self.state, self.groups, self.norm_groups, self.eps = int(heads), int(vdim), int(state), int(groups), int(norm_groups), float(eps)
        self.inner = self.heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.state
        if self.heads % self.groups or self.inner % self.norm_groups:
            raise ValueError(f"state space: {heads} heads x {vdim} do not divide into {groups} groups / {norm_groups} norm parts")
        if tuple(taps.shape)[0] != self.channels or (conv_bias is not None and conv_bias.numel() != self.channels):
            raise ValueError("state space: the convolution does not match x | B | C")
        if dt_bias.numel() != heads or a_log.numel() != heads or (skip is not None and skip.numel() != heads) or norm_weight.numel() != self.inner or tuple(w_o.shape)[1] != self.inner:
            raise ValueError("state space: tensor shapes do not match the head sizes")
        self.taps, self.conv_bias = taps.contiguous(), None if conv_bias is None else conv_bias.contiguous()
        self.dt_bias, self.a_log, self.skip = dt_bias.contiguous(), a_log.contiguous(), None if skip is None else skip.contiguous()
        self.norm_weight, self.w_o = norm_weight.contiguous(), w_o.contiguous()

    @property
    def state_shape(self) -> tuple:
        return (self.heads, self.state, self.vdim)

    @property
    def conv_shape(self) -> tuple:
        return (self.channels, self.taps.shape[1] - 1)

    def __call__(self, z, xbc, dt, plan, state: torch.Tensor, conv_state: torch.Tensor | None) -> torch.Tensor:
        """``z [T, inner]`` and ``xbc [T, channels]``: views of the fused projection; ``dt [T, heads]`` fp32."""
        from extensions_b200.tiny_llm_ext_b200 import blocks

        H, P, N, G = self.heads, self.vdim, self.state, self.groups
        y = blocks.short_conv(xbc, self.taps, seq_info=plan.seq_info, state=conv_state, max_tokens=plan.max_tokens, act=1, bias=self.conv_bias)
        x, B, C = y[:, : self.inner], y[:, self.inner : self.inner + G * N], y[:, self.inner + G * N :]
        o = blocks.decay_scan(C.unflatten(1, (G, N)), B.unflatten(1, (G, N)), x.unflatten(1, (H, P)), dt, self.dt_bias, q_scale=1.0,
                              seq_info=plan.seq_info, state=state, max_tokens=plan.max_tokens, decay_kind=blocks.DECAY_STEP, a_log=self.a_log,
                              skip=self.skip)
        parts = self.norm_groups
        n = blocks.head_norm_gate(o.view(o.shape[0], parts, self.inner // parts), self.norm_weight, self.eps, z, act=1, gate_first=True)
        return linear_wide(n, self.w_o)
