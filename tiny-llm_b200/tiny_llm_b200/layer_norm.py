"""Readable RMSNorm (``/root/reference/src/tiny_llm_ref/layer_norm.py:4-15``)."""

from __future__ import annotations

import torch


class RMSNorm:
    def __init__(self, dim: int, weight: torch.Tensor, eps: float = 1e-5):
        self.dim = dim
        self.eps = eps
        self.weight = weight

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        # fp32 statistics, storage-dtype product with the weight (two roundings;
        # the fused kernel rounds once - week2_kernels.metal:41-47).
        h = x.to(torch.float32)
        h = h * torch.rsqrt(h.square().mean(dim=-1, keepdim=True) + self.eps)
        return h.to(x.dtype) * self.weight.to(x.dtype)


class ResidualRMSNorm:
    """RMS norm on a sublayer's OUTPUT, accumulated into a residual stream that is kept in fp32:

        residual <- residual + y / sqrt(mean(y^2) + eps) * (weight + weight_offset) * scale

    ``weight_offset`` = 1 for weights stored around zero, 0 for plain weights; ``scale`` is an optional per-channel
    layer scale.  One launch of the blocks library does the norm, the scale, the sum and the rounding of the new
    residual to the compute dtype (the next sublayer's input).  Without ``residual`` it is a plain row norm."""

    def __init__(self, weight: torch.Tensor, eps: float, weight_offset: float = 0.0, scale: torch.Tensor | None = None):
        self.weight, self.eps, self.weight_offset, self.scale = weight.contiguous(), float(eps), float(weight_offset), scale
        if scale is not None:
            self.scale = scale.contiguous()

    def __call__(self, y: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        from extensions_b200.tiny_llm_ext_b200 import blocks

        return blocks.norm_residual(y, self.weight, self.eps, weight_offset=self.weight_offset, scale=self.scale, residual=residual)


class ResidualStreams:
    """Several residual streams around the sublayers of a pre-norm decoder, and the sublayers' norms with ONE number as
    their weight.  Instead of one ``x`` the model carries ``n`` copies ``x_1 .. x_n`` (all equal to the embedding at the
    start).  A sublayer with learned ``w_in [n]``, ``w_mix [n, n]`` (indexed [from, to]) and ``w_out [n]`` reads and writes

        h = rms_norm(sum_s w_in[s] x_s) * g            x_t <- sum_s w_mix[s, t] x_s + w_out[t] * sublayer(h)

    and the model's output norm reads the plain sum of the streams.  ``n = 1`` with all weights 1 is the ordinary residual
    sum.  ``site(...)`` packs one sublayer's numbers for the kernel; ``step`` does the write of the sublayer that ended and
    the read of the one that follows in ONE launch over ``xs [rows, n, dim]`` (fp32, in place)."""

    def __init__(self, streams: int, eps: float, dtype, device):
        self.n, self.eps, self.dtype, self.device = int(streams), float(eps), dtype, torch.device(device)
        if not 1 <= self.n <= 8:
            raise ValueError(f"{streams} residual streams (1 to 8 are built)")

    def read_site(self, norm_weight, w_in=None) -> torch.Tensor:
        """fp32 ``[n + 1]``: the input weights (ones without ``w_in``), then the norm's weight."""
        w = torch.ones(self.n) if w_in is None else w_in.detach().float().cpu().reshape(-1)
        if w.numel() != self.n or norm_weight.numel() != 1:
            raise ValueError("residual streams: one input weight per stream and one number as the norm's weight")
        return torch.cat([w, norm_weight.detach().float().cpu().reshape(1)]).to(self.device)

    def write_site(self, w_mix=None, w_out=None) -> torch.Tensor:
        """fp32 ``[n * n + n]``: the mixing matrix [from, to] (identity without ``w_mix``), then the output weights (ones)."""
        mix = torch.eye(self.n) if w_mix is None else w_mix.detach().float().cpu()
        out = torch.ones(self.n) if w_out is None else w_out.detach().float().cpu().reshape(-1)
        if tuple(mix.shape) != (self.n, self.n) or out.numel() != self.n:
            raise ValueError("residual streams: the mixing matrix must be [n, n] and the output weights [n]")
        return torch.cat([mix.reshape(-1), out]).to(self.device)

    def start(self, x0: torch.Tensor, read: torch.Tensor | None):
        """Streams that all equal ``x0 [rows, dim]`` (fp32) -> (xs, the first sublayer's input)."""
        from extensions_b200.tiny_llm_ext_b200 import blocks

        xs = torch.empty((x0.shape[0], self.n, x0.shape[1]), dtype=torch.float32, device=x0.device)
        return xs, blocks.streams_step(xs, x0=x0, read=read, eps=self.eps, dtype=self.dtype)

    def step(self, xs: torch.Tensor, y: torch.Tensor | None, write: torch.Tensor | None, read: torch.Tensor | None, y_bias=None):
        from extensions_b200.tiny_llm_ext_b200 import blocks

        return blocks.streams_step(xs, y=y, y_bias=y_bias, write=write, read=read, eps=self.eps, dtype=self.dtype)
