"""Grouped-query softmax attention over the paged cache of a ragged batch, with the choices a design may make as
parameters: what a position sees (``mask`` = ``"causal"``, ``"window"``: itself and the ``mask_size - 1`` positions
before it, ``"chunk"``: the earlier positions of its own block of ``mask_size`` positions counted from 0), a tanh
``softcap`` on the scaled scores, a ``sink`` (one more term ``exp(0)`` in the softmax's denominator), per-head RMS
norms of queries and keys (plain weights of size ``dim``, shared by the heads) and a sigmoid output gate per head
(``gate`` None = no gate).  With ``rot`` = ``{"dims", "base", "factor", "interleaved"}`` the first ``dims`` entries of every
query and key head are rotated by the token's position (pairs ``(2i, 2i+1)`` or ``(i, i + dims/2)``, every frequency
divided by ``factor``) before the keys are stored; without it the scores carry no positional term.
``qk_norm="whole"``: each norm takes a token's whole query (key) projection as one vector, ahead of the split into heads and
before any rotation, with weights of that size.  ``head_bias`` (one learned number per head): with ``sink`` the sink's term is
``exp(head_bias[h])``; with ``weights="sigmoid"`` there is no softmax at all, a visible key weighs
``sigmoid(score + head_bias[h])`` and nothing is normalised over the keys.

The layer's input projections are made by the caller in one product (``FusedProjection``); the module takes the views
``q [T, H * dim]``, ``k [T, G * dim]``, ``v [T, G * vdim]`` and ``gate [T, H]`` (logits), stores keys and values in the
layer's slab ``[pages, page_size, G * (dim + vdim)]`` (or, built with ``caches=False``, reads another layer's slab and
gets no k / v), runs the attention kernel over the plan's work list and returns the output projection in fp32.
"""

from __future__ import annotations

import torch

from .basics import linear, linear_wide

MASKS = {"causal": 0, "window": 1, "chunk": 2}
WEIGHTS = {"softmax": 0, "sigmoid": 1}


class FusedProjection:
    """Several projections of one input as ONE product: the weights stacked by rows (padded to a multiple of 8 rows), the
    biases, where any part has one, stacked likewise; ``proj(h)[name]`` is that part's columns of the result."""

    def __init__(self, parts: list, dtype, device):
        self.spans, rows, biases, at = {}, [], [], 0
        for name, weight, bias in parts:
            n = weight.shape[0]
            self.spans[name] = (at, n)
            rows.append(weight)
            biases.append(bias if bias is not None else torch.zeros(n, dtype=weight.dtype, device=weight.device))
            at += n
        pad = -at % 8
        if pad:
            rows.append(torch.zeros((pad, rows[0].shape[1]), dtype=rows[0].dtype, device=rows[0].device))
            biases.append(torch.zeros(pad, dtype=rows[0].dtype, device=rows[0].device))
        self.weight = torch.cat(rows, dim=0).to(device=device, dtype=dtype).contiguous()
        self.bias = torch.cat(biases).to(device=device, dtype=dtype).contiguous() if any(b is not None for _, _, b in parts) else None

    def __call__(self, h: torch.Tensor) -> dict:
        y = linear(h, self.weight) if self.bias is None else torch.addmm(self.bias, h, self.weight.t())
        return {name: y[:, at : at + n] for name, (at, n) in self.spans.items()}


class PagedGroupedAttention:
    def __init__(self, *, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, mask: str, mask_size: int, w_o, softcap: float | None = None,
                 sink: bool = False, q_norm=None, k_norm=None, eps: float = 1e-6, caches: bool = True, page_size: int = 64, rot: dict | None = None,
                 qk_norm: str = "head", head_bias=None, weights: str = "softmax"):
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads do not divide into {kv_heads} key/value heads")
        if mask not in MASKS or (mask != "causal" and int(mask_size) <= 0):
            raise ValueError(f"mask {mask!r} of size {mask_size}")
        if tuple(w_o.shape)[1] != heads * vdim:
            raise ValueError("attention: the output projection does not match heads x vdim")
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        self.scale, self.mask, self.mask_size = float(scale), MASKS[mask], int(mask_size or 0)
        self.softcap, self.sink, self.eps, self.caches = float(softcap or 0.0), bool(sink), float(eps), bool(caches)
        self.q_norm = None if q_norm is None else q_norm.contiguous()
        self.k_norm = None if k_norm is None else k_norm.contiguous()
        self.w_o = w_o.contiguous()
        if qk_norm not in ("head", "whole") or weights not in WEIGHTS:
            raise ValueError(f"attention: qk_norm={qk_norm!r}, weights={weights!r}")
        self.whole_norm, self.weights = qk_norm == "whole", WEIGHTS[weights]
        if self.whole_norm and (q_norm is None or q_norm.numel() != heads * dim or (k_norm is not None and k_norm.numel() != kv_heads * dim)):
            raise ValueError("attention: norms over the whole projection take weights of heads x dim")
        self.head_bias = None if head_bias is None else head_bias.detach().float().contiguous()  # scores and weights are fp32
        if self.head_bias is not None and self.head_bias.numel() != heads:
            raise ValueError("attention: one head_bias per head")
        if self.weights == WEIGHTS["sigmoid"] and (sink or softcap):
            raise ValueError("attention: sigmoid weights take no sink and no cap")
        self.rot = None
        if rot and int(rot.get("dims", 0)) > 0:
            if (q_norm is not None or k_norm is not None) and not self.whole_norm:
                raise ValueError("attention: rotation together with query / key norms is not built")
            self.rot = {"dims": int(rot["dims"]), "base": float(rot["base"]), "factor": float(rot.get("factor", 1.0)), "interleaved": bool(rot.get("interleaved", False))}
            if self.rot["dims"] % 2 or self.rot["dims"] > self.dim:
                raise ValueError(f"attention: cannot rotate {self.rot['dims']} of {self.dim} entries")
        from extensions_b200.tiny_llm_ext_b200 import blocks

        # the kernel (tensor cores for a bf16 cache of fitting sizes, else the general one) and its work-list granularity
        self.kernel, self.tile_tokens = blocks.paged_attention_kernel(self.w_o.dtype, self.heads, self.kv_heads, self.dim, self.vdim, int(page_size))

    @property
    def cache_width(self) -> int:
        return self.kv_heads * (self.dim + self.vdim)

    def __call__(self, q, k, v, gate, plan, slab: torch.Tensor) -> torch.Tensor:
        from extensions_b200.tiny_llm_ext_b200 import blocks

        T, H, G = q.shape[0], self.heads, self.kv_heads
        q3 = q.unflatten(1, (H, self.dim))
        q_norm, k_norm = self.q_norm, self.k_norm
        if self.whole_norm and (self.rot is None or self.rot["factor"] == 1.0):
            # each projection as ONE row: norm, rotation and the store into the cache in one launch
            r = self.rot or {"dims": 0, "base": 1.0, "interleaved": False}
            tables = plan.rope_tables(r["dims"], r["base"]) if r["dims"] and hasattr(plan, "rope_tables") else None  # shared by the step's layers
            blocks.qk_whole_prepare(q, k if self.caches else None, v if self.caches else None, heads=H, kv_heads=G, q_norm=q_norm,
                                    k_norm=k_norm if self.caches else None, eps=self.eps, rot_dims=r["dims"], base=r["base"], interleaved=r["interleaved"],
                                    tok_pos=plan.tok_pos, tok_seq=plan.tok_seq, block_table=plan.block_table, slab=slab if self.caches else None, rope=tables)
        else:
            if self.whole_norm:  # scaled positions: the row norms alone, then the framework's rotation and store
                blocks.kv_prepare(q.unflatten(1, (1, H * self.dim)), None, None, q_norm=q_norm, eps=self.eps)
                if self.caches and k_norm is not None:
                    blocks.kv_prepare(k.unflatten(1, (1, G * self.dim)), None, None, q_norm=k_norm, eps=self.eps)
                q_norm = k_norm = None
            if self.rot is not None:
                r = self.rot
                blocks.rope_rows(q, plan.tok_pos, heads=H, head_stride=self.dim, first=0, dims=r["dims"], base=r["base"], interleaved=r["interleaved"], factor=r["factor"])
                if self.caches:
                    blocks.rope_rows(k, plan.tok_pos, heads=G, head_stride=self.dim, first=0, dims=r["dims"], base=r["base"], interleaved=r["interleaved"], factor=r["factor"])
            if self.caches:
                blocks.kv_prepare(q3, k.unflatten(1, (G, self.dim)), v.unflatten(1, (G, self.vdim)), q_norm=q_norm, k_norm=k_norm, eps=self.eps,
                                  tok_pos=plan.tok_pos, tok_seq=plan.tok_seq, block_table=plan.block_table, slab=slab)
            elif q_norm is not None:
                blocks.kv_prepare(q3, None, None, q_norm=q_norm, eps=self.eps)
        o = blocks.paged_attention(q3, slab, plan.block_table, plan.tiles_for(self.tile_tokens), plan.tok_pos, kv_heads=G, dv=self.vdim, mask=self.mask,
                                   mask_size=self.mask_size, scale=self.scale, softcap=self.softcap, sink=self.sink, gate=gate, kernel=self.kernel,
                                   max_context=getattr(plan, "max_context", 0), head_bias=self.head_bias, weights=self.weights)
        return linear_wide(o.view(T, H * self.vdim), self.w_o)  # fp32: a norm or the residual sum reads it unrounded
