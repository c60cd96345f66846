"""Linear attention with a decay: recurrent mixers whose state lives in fp32 slots.  ``DecayedLinearAttention`` has one
input-dependent decay per key channel, ``RetainedLinearAttention`` (at the end of the file) one fixed decay per head.

Per head a matrix ``S [dim, vdim]`` is carried along the sequence,

    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T        o_t = S_t^T (dim^-1/2 q_t)        alpha_t = sigmoid(z_t)^(1 / tau)

with the decay logits ``z = W_a2 (W_a1 h) + b`` from a low-rank projection.  Each head's output is RMS-normed over
``vdim`` (plain weight shared by the heads), multiplied by ``silu(W_g h)`` and projected.  The projections of ``h``
(q, k, v, gate, the low-rank decay input) are made by the caller in one product; this module takes their views.  The
second decay projection hands its fp32 accumulator over, and the decay, the recurrence and the norm are fp32 whatever
the compute dtype.  ``state`` is the layer's view ``[slots, heads, dim, vdim]`` of the model's ``StateSlotPool``; the
plan's ``seq_info`` says which slot a sequence owns and whether it starts at position 0 (then from zero).
"""

from __future__ import annotations

import torch

from .basics import linear_wide


class DecayedLinearAttention:
    def __init__(self, *, heads: int, dim: int, vdim: int, tau: float, w_a2, a2_bias, norm_weight, w_o, eps: float = 1e-6):
        if tuple(w_a2.shape)[0] != heads * dim or tuple(w_o.shape)[1] != heads * vdim or tuple(norm_weight.shape) != (vdim,):
            raise ValueError("linear attention: tensor shapes do not match the head sizes")
        if not tau > 0:
            raise ValueError("linear attention: tau must be positive")
        self.heads, self.dim, self.vdim, self.tau, self.eps = int(heads), int(dim), int(vdim), float(tau), float(eps)
        self.w_a2, self.a2_bias = w_a2.contiguous(), None if a2_bias is None else a2_bias.contiguous()
        self.norm_weight, self.w_o = norm_weight.contiguous(), w_o.contiguous()

    @property
    def state_shape(self) -> tuple:
        return (self.heads, self.dim, self.vdim)

    def __call__(self, q, k, v, gate, a1, plan, state: torch.Tensor) -> torch.Tensor:
        from extensions_b200.tiny_llm_ext_b200 import blocks

        H = self.heads
        z = linear_wide(a1.contiguous(), self.w_a2)  # fp32 decay logits
        o = blocks.decay_scan(q.unflatten(1, (H, self.dim)), k.unflatten(1, (H, self.dim)), v.unflatten(1, (H, self.vdim)), z, self.a2_bias,
                              tau=self.tau, q_scale=self.dim ** -0.5, seq_info=plan.seq_info, state=state, max_tokens=plan.max_tokens)
        return linear_wide(blocks.head_norm_gate(o, self.norm_weight, self.eps, gate, act=1), self.w_o)


class RetainedLinearAttention:
    """Retention: linear attention with ONE fixed decay per head and no denominator,

        S_t = decay_h S_(t-1) + k_t v_t^T        o_t = S_t^T q_t        (dim^-1/2 folded into q)

    with q and k optionally rotated by the token's position first (``rot`` = ``{"dims", "base", "factor"}``, pairs
    ``(i, i + dims/2)``; in fp32, inside the scan, from the step's tabulated angles).  Each head's output is divided by its
    root mean square (no weight), multiplied by ``silu(gate)`` and projected.  The scan is ``blocks.decay_scan`` with a
    constant decay, so long portions run as parallel segments like those of ``DecayedLinearAttention``."""

    def __init__(self, *, heads: int, dim: int, vdim: int, decay, w_o, eps: float = 1e-6, rot: dict | None = None):
        if len(decay) != heads or tuple(w_o.shape)[1] != heads * vdim:
            raise ValueError("retention: one decay per head and an output projection of heads x vdim wanted")
        self.heads, self.dim, self.vdim, self.eps = int(heads), int(dim), int(vdim), float(eps)
        self.decay = torch.tensor([float(d) for d in decay], dtype=torch.float32, device=w_o.device)
        self.w_o = w_o.contiguous()
        self.rot = None
        if rot and int(rot.get("dims", 0)) > 0:
            self.rot = {"dims": int(rot["dims"]), "base": float(rot["base"]), "factor": float(rot.get("factor", 1.0))}
            if self.rot["dims"] % 2 or self.rot["dims"] > self.dim:
                raise ValueError(f"retention: cannot rotate {self.rot['dims']} of {self.dim} entries")

    @property
    def state_shape(self) -> tuple:
        return (self.heads, self.dim, self.vdim)

    def __call__(self, q, k, v, gate, plan, state: torch.Tensor) -> torch.Tensor:
        from extensions_b200.tiny_llm_ext_b200 import blocks

        H, r = self.heads, self.rot
        tables = plan.rope_tables(r["dims"], r["base"], r["factor"]) if r else None
        o = blocks.decay_scan(q.unflatten(1, (H, self.dim)), k.unflatten(1, (H, self.dim)), v.unflatten(1, (H, self.vdim)), None, None,
                              q_scale=self.dim ** -0.5, seq_info=plan.seq_info, state=state, max_tokens=plan.max_tokens, head_decay=self.decay,
                              rope=tables, rope_dims=r["dims"] if r else 0, rope_interleaved=False)
        return linear_wide(blocks.head_norm_gate(o, None, self.eps, gate, act=1), self.w_o)


class ShiftedBonusLinearAttention:
    """Linear attention in the manner of RWKV's time mixing: every projection reads its own blend of the token and the
    token before it, the decay is a double exponential of a low-rank projection, and the read-out comes BEFORE the update
    with a learned bonus for the token's own contribution,

        m_s = h_t + (h_(t-1) - h_t) * mu_s                     s in r, k, v, g, w   (h_(-1) = 0)
        w_t = exp(-exp(W_w2 tanh(W_w1 m_w) + w0))              per head and key channel
        o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t              S_t = diag(w_t) S_(t-1) + k_t v_t^T

    Each head's output is divided by its root mean square, multiplied by ``norm_weight`` (one entry per head and channel)
    and by ``silu(W_g m_g)``, and projected.  ``mu [5, width]`` in the order r, k, v, g, w; ``w_rkvg [4, heads * dim, width]``.
    The blends are bf16 / fp32 operands of the projections; the second decay projection hands its fp32 accumulator on and
    the decay, the bonus, the recurrence and the norm are fp32 whatever the compute dtype.  A request's state is two blocks
    of its slot: ``state [slots, heads, dim, dim]`` and the previous token's input ``shift [slots, width]``; both start from
    zero at position 0 whatever the slot held."""

    def __init__(self, *, heads: int, dim: int, mu, w_rkvg, w_w1, w_w2, w0, bonus, norm_weight, w_o, eps: float = 1e-6):
        self.heads, self.dim, self.eps = int(heads), int(dim), float(eps)
        hd = self.heads * self.dim
        width = int(mu.shape[1])
        if tuple(mu.shape) != (5, width) or tuple(w_rkvg.shape) != (4, hd, width) or tuple(w_w2.shape)[0] != hd or w0.numel() != hd:
            raise ValueError("time-mix attention: projections do not match heads x dim")
        if bonus.numel() != hd or norm_weight.numel() != hd or tuple(w_o.shape)[1] != hd or tuple(w_w1.shape) != (w_w2.shape[1], width):
            raise ValueError("time-mix attention: bonus, norm and output projection do not match heads x dim")
        self.mu, self.w_rkvg_t = mu.contiguous(), w_rkvg.transpose(1, 2).contiguous()  # [4, width, heads * dim]
        self.w_w1, self.w_w2, self.w0 = w_w1.contiguous(), w_w2.contiguous(), w0.reshape(-1).contiguous()
        self.bonus, self.norm_weight, self.w_o = bonus.reshape(self.heads, self.dim).contiguous(), norm_weight.reshape(-1).contiguous(), w_o.contiguous()
        self.width = width

    @property
    def state_shape(self) -> tuple:
        return (self.heads, self.dim, self.dim)

    @property
    def shift_shape(self) -> tuple:
        return (self.width,)

    def __call__(self, h, plan, state: torch.Tensor, shift: torch.Tensor) -> torch.Tensor:
        from extensions_b200.tiny_llm_ext_b200 import blocks

        from .basics import linear

        H, d = self.heads, self.dim
        m = blocks.shift_mix(h, self.mu, seq_info=plan.seq_info, state=shift, max_tokens=plan.max_tokens)  # [5, T, width]
        rkvg = torch.bmm(m[:4], self.w_rkvg_t)                                                             # [4, T, H * d]
        low = blocks.act_rows(linear(m[4], self.w_w1), blocks.ACT_TANH)
        z = linear_wide(low, self.w_w2)  # fp32 decay logits
        o = blocks.decay_scan(rkvg[0].unflatten(1, (H, d)), rkvg[1].unflatten(1, (H, d)), rkvg[2].unflatten(1, (H, d)), z, self.w0, q_scale=1.0,
                              seq_info=plan.seq_info, state=state, max_tokens=plan.max_tokens, decay_kind=blocks.DECAY_DOUBLE_EXP, bonus=self.bonus)
        return linear_wide(blocks.head_norm_gate(o, self.norm_weight, self.eps, rkvg[3], act=1), self.w_o)
