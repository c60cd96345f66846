"""Latent attention: keys and values of all heads are up-projections of one cached low-rank latent per token.

Per token the layer caches ``c = rms_norm(W_dkv h)[:rank]`` and one rotated key part shared by all heads.  Head ``h``
scores ``q_plain_h . (W_uk_h c_j) + q_rot_h . k_rot_j`` and mixes values ``W_uv_h c_j``.  Both up-projections are
folded into the query and the output ("absorbed" form), so attention runs directly on the cache as multi-query
attention with key width ``rank + rot`` and value width ``rank``:

    q_lat_h = W_uk_h^T q_plain_h        o_h = W_uv_h (sum_j p_hj c_j)

which is what makes decoding cheap (no per-head keys are ever rebuilt) and is exact up to rounding.  Parameters:
``heads, dim`` (un-rotated), ``rot_dim`` (rotated), ``vdim``, ``kv_rank``, the rotary layout (``interleaved`` pairs
(2i, 2i+1) or half pairs (i, i + dims/2)), its ``base`` and ``dims``, an optional sliding ``window`` (a token sees
itself and the window-1 tokens before it) and ``scale``.  A layer built without ``w_dkv`` reads the cache of another
layer (its slab is handed in by the model) with its own up-projections, queries and mask.

Two more choices a design may make.  Queries through a latent of their own: with ``w_q_down`` (and ``q_down_norm``)
``q = W_q rms_norm(W_q_down h)``; the down projection is then the one fused with ``w_dkv``.  A learned ``sink`` per head:
the softmax's denominator holds one more term ``exp(sink[h])``, which stands for no token: it has neither key nor value.
"""

from __future__ import annotations

import torch

from .basics import linear, linear_wide


class LatentAttention:
    def __init__(self, *, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, scale: float, rot_dims: int, rot_base: float,
                 interleaved: bool, window: int | None, w_q, w_uk, w_uv, w_o, w_dkv=None, dkv_norm=None, eps: float = 1e-5,
                 w_q_down=None, q_down_norm=None, sink=None):
        self.heads, self.dim, self.rot_dim, self.vdim, self.rank = heads, dim, rot_dim, vdim, kv_rank
        self.scale, self.rot_dims, self.rot_base, self.interleaved = float(scale), int(rot_dims), float(rot_base), bool(interleaved)
        self.window = int(window) if window else 0
        self.eps = float(eps)
        if tuple(w_q.shape)[0] != heads * (dim + rot_dim) or tuple(w_uk.shape) != (heads * dim, kv_rank) or tuple(w_uv.shape) != (heads * vdim, kv_rank):
            raise ValueError("latent attention: projection shapes do not match the head sizes")
        if rot_dims > rot_dim or rot_dims % 2:
            raise ValueError("latent attention: rotary dims must be even and fit the rotated part")
        self.q_rank = 0 if w_q_down is None else int(w_q_down.shape[0])
        if self.q_rank and (tuple(w_q.shape)[1] != self.q_rank or q_down_norm is None or q_down_norm.numel() != self.q_rank):
            raise ValueError("latent attention: the query up projection and norm must match the query latent")
        self.q_down_norm = None if q_down_norm is None else q_down_norm.contiguous()
        self.sink = None if sink is None else sink.detach().float().contiguous()  # the softmax runs in fp32
        if self.sink is not None and self.sink.numel() != heads:
            raise ValueError("latent attention: one sink per head")
        first = w_q_down if self.q_rank else w_q  # what is projected from the layer's input beside the latent
        self.w_q, self.w_o = (None if (w_dkv is not None and not self.q_rank) else w_q.contiguous()), w_o.contiguous()
        self.w_first = first.contiguous() if w_dkv is None and self.q_rank else None
        self.w_uk = w_uk.reshape(heads, dim, kv_rank).contiguous()                    # q_lat_h = q_plain_h @ w_uk[h]
        self.w_uv_t = w_uv.reshape(heads, vdim, kv_rank).transpose(1, 2).contiguous()  # o_h = o_lat_h @ w_uv_t[h]
        self.dkv_norm = None if dkv_norm is None else dkv_norm.contiguous()
        if w_dkv is not None and tuple(w_dkv.shape)[0] != kv_rank + rot_dim:
            raise ValueError("latent attention: the down projection must have kv_rank + rot_dim rows")
        # a caching layer projects q and the latent in ONE product (rows of w_q, then rows of w_dkv)
        self.caches = w_dkv is not None
        self.w_qd = torch.cat([first, w_dkv], dim=0).contiguous() if self.caches else None

    @property
    def cache_width(self) -> int:
        return self.rank + self.rot_dim

    def attention_kernel(self, slab: torch.Tensor) -> tuple[str, int]:
        """(kernel name, tokens per work-list entry) for this layer on ``slab [P, page_size, rank + rot]``."""
        from extensions_b200.tiny_llm_ext_b200 import blocks

        return blocks.attention_kernel(slab.dtype, self.heads, self.rank, self.rot_dim, slab.shape[1])

    def __call__(self, h: torch.Tensor, plan, slab: torch.Tensor) -> torch.Tensor:
        from extensions_b200.tiny_llm_ext_b200 import blocks

        T, H, dn, dr = h.shape[0], self.heads, self.dim, self.rot_dim
        if self.q_rank:
            if self.caches:
                y = linear(h, self.w_qd)  # [T, q_rank | rank + dr]
                cq = y[:, : self.q_rank]
            else:
                cq = linear(h, self.w_first)
            blocks.kv_prepare(cq.unflatten(1, (1, self.q_rank)), None, None, q_norm=self.q_down_norm, eps=self.eps)  # the row's norm, in place
            q = linear(cq, self.w_q)
            if self.caches:
                blocks.latent_prepare_parts(q, y[:, self.q_rank :], self.dkv_norm, self.eps, heads=H, dim=dn, rot_dim=dr, rank=self.rank,
                                            rot_dims=self.rot_dims, interleaved=self.interleaved, base=self.rot_base, tok_pos=plan.tok_pos,
                                            tok_seq=plan.tok_seq, block_table=plan.block_table, slab=slab)
            else:
                blocks.rope_rows(q, plan.tok_pos, heads=H, head_stride=dn + dr, first=dn, dims=self.rot_dims, base=self.rot_base, interleaved=self.interleaved)
            q3 = q.view(T, H, dn + dr)
        elif self.caches:
            qd = linear(h, self.w_qd)  # [T, H (dn + dr) | rank + dr]
            blocks.latent_prepare(qd, self.dkv_norm, self.eps, heads=H, dim=dn, rot_dim=dr, rank=self.rank, rot_dims=self.rot_dims,
                                  interleaved=self.interleaved, base=self.rot_base, tok_pos=plan.tok_pos, tok_seq=plan.tok_seq,
                                  block_table=plan.block_table, slab=slab)
            q3 = qd[:, : H * (dn + dr)].unflatten(1, (H, dn + dr))
        else:
            q = linear(h, self.w_q)
            blocks.rope_rows(q, plan.tok_pos, heads=H, head_stride=dn + dr, first=dn, dims=self.rot_dims, base=self.rot_base, interleaved=self.interleaved)
            q3 = q.view(T, H, dn + dr)
        kernel, tile_tokens = self.attention_kernel(slab)
        q_lat = torch.bmm(q3[:, :, :dn].transpose(0, 1), self.w_uk)          # [H, T, rank]
        o_lat = torch.empty_like(q_lat)
        blocks.latent_attention(q_lat.transpose(0, 1), q3[:, :, dn:], slab, plan.block_table, plan.tiles_for(tile_tokens), plan.tok_pos,
                                window=self.window, scale=self.scale, out=o_lat.transpose(0, 1), kernel=kernel,
                                max_context=getattr(plan, "max_context", 0), sink=self.sink)
        o = torch.bmm(o_lat, self.w_uv_t)                                     # [H, T, vdim]
        return linear_wide(o.transpose(0, 1).reshape(T, H * self.vdim), self.w_o)  # fp32: the layer's norm reads it unrounded
