"""The gated delta rule: a recurrent mixer that writes into its state only what the state does not yet say.

Per head a matrix ``S [dim, vdim]`` is carried along the sequence,

    S <- diag(g_t) S        u_t = beta_t (v_t - S^T k_t)        S <- S + k_t u_t^T        o_t = S^T q_t

(the read-out sees the token's own write), with ``g_t = exp(-exp(A_log) softplus(a_t + dt_bias))`` and
``beta_t = sigmoid(b_t)``.  ``g`` is one number per head, or, ``channel_decay``, one per head and key channel; then the
decay input comes from a low-rank pair of projections (the second one, ``w_a2``, is applied here and hands its fp32
accumulator on), and so does the output gate (``w_g2``).  q, k and v first pass a short causal convolution per channel
over time (``taps [channels, K]``, the last column the current token's) and ``silu``; q and k are then made unit
vectors per head, q times ``dim^-1/2``.  Query/key heads may be fewer than value heads (``key_heads``).  Each head's
output is RMS-normed over ``vdim`` (plain weight shared by the heads), multiplied by ``gate_act(gate)`` and projected.

The projections of the layer's input are made by the caller in one product, q | k | v side by side so that the
convolution reads them as one ``[T, channels]`` view.  The decay, beta, unit vectors, recurrence and norm are fp32
whatever the compute dtype.  A request's state is two blocks of its state slot: ``state [slots, heads, dim, vdim]`` and
the convolution's last ``K - 1`` inputs ``conv_state [slots, channels, K - 1]``.
"""

from __future__ import annotations

import torch

from .basics import linear, linear_wide

GATE_ACTS = {"none": 0, "silu": 1, "sigmoid": 2}


class GatedDeltaRule:
    def __init__(self, *, heads: int, key_heads: int, dim: int, vdim: int, taps: torch.Tensor, a_log, dt_bias, norm_weight, w_o, eps: float = 1e-6,
                 channel_decay: bool = False, w_a2=None, w_g2=None, gate_act: str = "silu"):
        self.heads, self.key_heads, self.dim, self.vdim, self.eps = int(heads), int(key_heads), int(dim), int(vdim), float(eps)
        self.channels = 2 * self.key_heads * self.dim + self.heads * self.vdim
        if self.heads % self.key_heads:
            raise ValueError(f"delta rule: {heads} heads do not divide into {key_heads} query/key heads")
        if tuple(taps.shape)[0] != self.channels or tuple(w_o.shape)[1] != heads * vdim or tuple(norm_weight.shape) != (vdim,) or a_log.numel() != heads:
            raise ValueError("delta rule: tensor shapes do not match the head sizes")
        self.channel_decay = bool(channel_decay)
        if dt_bias.numel() != (heads * dim if channel_decay else heads):
            raise ValueError("delta rule: dt_bias does not match the decay's layout")
        if w_a2 is not None and tuple(w_a2.shape)[0] != (heads * dim if channel_decay else heads):
            raise ValueError("delta rule: the second decay projection does not match the decay's layout")
        self.taps, self.a_log, self.dt_bias = taps.contiguous(), a_log.contiguous(), dt_bias.contiguous()
        self.norm_weight, self.w_o = norm_weight.contiguous(), w_o.contiguous()
        self.w_a2 = None if w_a2 is None else w_a2.contiguous()
        self.w_g2 = None if w_g2 is None else w_g2.contiguous()
        self.gate_act = GATE_ACTS[gate_act]

    @property
    def state_shape(self) -> tuple:
        return (self.heads, self.dim, self.vdim)

    @property
    def conv_shape(self) -> tuple:
        return (self.channels, self.taps.shape[1] - 1)

    def __call__(self, qkv, beta, a, gate, plan, state: torch.Tensor, conv_state: torch.Tensor | None) -> torch.Tensor:
        """``qkv [T, channels]`` (q | k | v), ``beta [T, heads]``, ``a`` the decay input (its low-rank first step when the
        module has ``w_a2``), ``gate`` likewise: views of the fused projection."""
        from extensions_b200.tiny_llm_ext_b200 import blocks

        H, G, dk, dv = self.heads, self.key_heads, self.dim, self.vdim
        y = blocks.short_conv(qkv, self.taps, seq_info=plan.seq_info, state=conv_state, max_tokens=plan.max_tokens, act=1)
        q, k, v = y[:, : G * dk], y[:, G * dk : 2 * G * dk], y[:, 2 * G * dk :]
        if self.w_a2 is not None:
            a = linear_wide(a.contiguous(), self.w_a2)  # fp32 decay input
        if self.w_g2 is not None:
            gate = linear(gate.contiguous(), self.w_g2)
        o = blocks.delta_scan(q.unflatten(1, (G, dk)), k.unflatten(1, (G, dk)), v.unflatten(1, (H, dv)), beta, a, self.a_log, self.dt_bias,
                              per_channel=self.channel_decay, q_scale=dk ** -0.5, unit_eps=1e-6, seq_info=plan.seq_info, state=state,
                              max_tokens=plan.max_tokens)
        return linear_wide(blocks.head_norm_gate(o, self.norm_weight, self.eps, gate, act=self.gate_act), self.w_o)
