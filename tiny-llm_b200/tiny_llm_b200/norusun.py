"""Norusun: a pre-norm decoder over several residual streams whose layers pick one of three mixers.

The residual is ``streams`` copies of the stream mixed by small learned matrices around every sublayer
(``l<i>.hc<q>.{in,mix,out}``, ``layer_norm.ResidualStreams``; a checkpoint without them has the plain sum), every norm of
the stack has ONE number as its weight, and the mixer's input first passes ``h + conv(h)``, a causal convolution over time
on each channel (``l<i>.canon1 [width, canon.taps]``, without bias; a checkpoint without it has none).

Mixers (``layers[i].type``):

- ``wkv``: linear attention with token shift, a double-exponential decay per head and key channel from a low-rank
  projection, and a bonus for the current token in a read-out that comes before the update
  (``linear_attention.ShiftedBonusLinearAttention``).
- ``latent_attention``: keys and values as up-projections of a cached latent, queries through a latent of their own, one
  rotated key part shared by the heads (pairs ``(2i, 2i+1)``), a sliding window of ``mask.size`` and a learned sink per head
  in the softmax (``latent_attention.LatentAttention``).
- ``parallel``: two mixers on the same input.  ``mixer.left`` = grouped-query attention within chunks of ``mask.size``
  positions counted from 0, queries and keys RMS-normed over the whole projection and then rotated (pairs ``(i, i + dims/2)``),
  every visible key weighing ``sigmoid(score + pb[h])`` without any normalisation over the keys; ``mixer.right`` = a
  selective state-space mixer (``state_space.StateSpaceMixer``).  Each output is RMS-normed over the width
  (``left.out`` / ``right.out``) and the layer takes half their sum.

Feed-forward (``mlp``, null = none; ``kind`` ``dense``): ``g = min(W_gate h + b, limit)``, ``u = clamp(W_up h + b, -limit,
limit)``, ``W_down (g sigmoid(1.702 g) (u + 1)) + b``.  Everything that can differ between models of the design is read
from ``config.json`` (``vocab``, ``width``, ``norm.eps``, ``streams``, ``canon.taps``, the layers' sizes, scales, rotations,
masks and limits) or from a tensor's shape (the low ranks, the convolutions' taps).

The model is the framework's usual object (``RaggedDecoderModel``).  A request holds one page list for all attention
layers (``LatentPagedPool``: one slab per latent layer and per parallel layer) and one slot of the ``StateSlotPool`` with a
block per layer: the input convolution's last inputs, and for the recurrent mixers their matrix state, the token shift's
previous input or the state-space convolution's last inputs.  Compute dtype bf16 (serving) or fp32 (every product in true
fp32); the streams and their mixing, norms, scores and weights of both attentions, step sizes, decays, recurrent states and
rotation angles are fp32 in both.
"""

from __future__ import annotations

import torch

from extensions_b200.tiny_llm_ext_b200 import blocks

from .basics import linear_wide
from .latent_attention import LatentAttention
from .latent_kv_cache import LatentCacheView, LatentPagedPool
from .layer_norm import ResidualStreams
from .linear_attention import ShiftedBonusLinearAttention
from .mlp import GatedMLP
from .paged_attention import FusedProjection, PagedGroupedAttention
from .ragged import RaggedPlan
from .ragged_model import RaggedDecoderModel
from .state_cache import HybridPagedCache, StateSlotPool
from .state_space import StateSpaceMixer

MIXERS = ("wkv", "latent_attention", "parallel")
SWISH_SLOPE = 1.702  # the design's sigmoid approximation of GELU inside the feed-forward's gate


class NorusunLayer:
    def __init__(self, kind: str):
        self.kind = kind
        self.canon = self.mixer = self.attention = self.recurrent = self.proj = self.w_dt = self.out_weights = self.mlp = None
        self.prefix = ""
        self.slab_index = -1
        self.canon_offset = self.state_offset = self.extra_offset = 0
        self.read1 = self.write1 = self.read2 = self.write2 = None


class NorusunModel(RaggedDecoderModel):
    architecture = "Norusun"
    graph_env = "TL_NORUSUN_GRAPH"

    def __init__(self, config: dict, tensors: dict, dtype=torch.bfloat16, device="cuda", page_size: int = 64, max_tokens: int | None = None,
                 max_requests: int | None = None):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Norusun runs in bfloat16 or float32")
        self.config, self.precision, self.device = config, dtype, torch.device(device)
        self.vocab_size, self.hidden_size = int(config["vocab"]), int(config["width"])
        self.eps = float(config["norm"]["eps"])
        self.num_hidden_layers = len(config["layers"])
        self.page_size = page_size
        self.stream_tap: list | None = None  # a list here receives the sum of the streams after every layer
        self._init_step()

        def take(name: str) -> torch.Tensor:
            if name not in tensors:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            t = tensors[name]
            return t.to(device=self.device, dtype=dtype if t.is_floating_point() else t.dtype).contiguous()

        D = self.hidden_size
        self.embed = take("embed")
        if tuple(self.embed.shape) != (self.vocab_size, D):
            raise ValueError("embed does not match vocab x width")
        self.streams = ResidualStreams(int(config.get("streams") or 1), self.eps, dtype, self.device)
        taps = int((config.get("canon") or {}).get("taps") or 0)
        self.layers: list[NorusunLayer] = []
        widths: list[int] = []
        state_floats = 0
        for i, spec in enumerate(config["layers"]):
            kind, m, p = spec["type"], spec["mixer"], f"l{i}.mix."
            if kind not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            layer = NorusunLayer(kind)
            layer.prefix = p
            if f"l{i}.canon1" in tensors:
                layer.canon = take(f"l{i}.canon1")
                if tuple(layer.canon.shape) != (D, taps):
                    raise ValueError(f"layer {i}: the input convolution must be [width, canon.taps]")
                layer.canon_offset = state_floats
                state_floats += D * (taps - 1)
            if kind == "wkv":
                layer.recurrent = ShiftedBonusLinearAttention(
                    heads=m["heads"], dim=m["dim"], mu=torch.stack([take(p + "mu." + n) for n in "rkvgw"]),
                    w_rkvg=torch.stack([take(p + n) for n in "rkvg"]), w_w1=take(p + "w1"), w_w2=take(p + "w2"), w0=take(p + "w0"),
                    bonus=take(p + "u"), norm_weight=take(p + "norm"), w_o=take(p + "o"), eps=self.eps)
                layer.state_offset = state_floats
                state_floats += layer.recurrent.heads * layer.recurrent.dim ** 2
                layer.extra_offset = state_floats  # the previous token's input
                state_floats += D
            elif kind == "latent_attention":
                rot = m["rot"]
                if int(rot["dims"]) != int(m["rot_dim"]):
                    raise ValueError(f"layer {i}: the rotated key part is rotated whole (rot.dims = rot_dim)")
                layer.mixer = LatentAttention(
                    heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"], kv_rank=m["kv_rank"], scale=m["scale"], rot_dims=rot["dims"],
                    rot_base=rot["base"], interleaved=True, window=m["mask"]["size"], eps=self.eps, w_q=take(p + "uq"), w_uk=take(p + "uk"),
                    w_uv=take(p + "uv"), w_o=take(p + "o"), w_dkv=take(p + "dkv"), dkv_norm=take(p + "dkv.norm"), w_q_down=take(p + "dq"),
                    q_down_norm=take(p + "dq.norm"), sink=take(p + "sink"))
                if layer.mixer.q_rank != int(m["q_rank"]):
                    raise ValueError(f"layer {i}: the query latent does not have q_rank rows")
                layer.slab_index = len(widths)
                widths.append(layer.mixer.cache_width)
            else:
                a, r, lp, rp = m["left"], m["right"], p + "left.", p + "right."
                layer.attention = PagedGroupedAttention(
                    heads=a["heads"], kv_heads=a["kv_heads"], dim=a["dim"], vdim=a["vdim"], scale=a["scale"], mask="chunk", mask_size=a["mask"]["size"],
                    w_o=take(lp + "o"), q_norm=take(lp + "q.norm"), k_norm=take(lp + "k.norm"), eps=self.eps, page_size=page_size, qk_norm="whole",
                    rot=None if not (a.get("rot") or {}).get("dims") else {"dims": int(a["rot"]["dims"]), "base": float(a["rot"]["base"]), "interleaved": False},
                    head_bias=take(lp + "pb"), weights="sigmoid")
                layer.slab_index = len(widths)
                widths.append(layer.attention.cache_width)
                w_in = take(rp + "in")
                heads = int(r["heads"])
                layer.recurrent = StateSpaceMixer(
                    heads=heads, vdim=r["vdim"], state=r["state"], groups=r["groups"], norm_groups=r["norm_groups"], taps=take(rp + "conv"),
                    conv_bias=take(rp + "conv.b"), dt_bias=take(rp + "dt_bias"), a_log=take(rp + "A_log"), skip=take(rp + "D"),
                    norm_weight=take(rp + "norm"), w_o=take(rp + "o"), eps=self.eps)
                s = layer.recurrent
                if w_in.shape[0] != s.inner + s.channels + heads or ("conv" in r and int(r["conv"]) != s.taps.shape[1]):
                    raise ValueError(f"layer {i}: the state-space input projection or convolution does not match its sizes")
                # z | x | B | C join the attention's projections in one product; the step sizes keep their fp32 accumulator
                parts = [(lp + n, take(lp + n), None) for n in ("q", "k", "v")] + [(rp + "z", w_in[: s.inner], None), (rp + "xbc", w_in[s.inner : s.inner + s.channels], None)]
                layer.proj = FusedProjection(parts, dtype, self.device)
                layer.w_dt = w_in[s.inner + s.channels :].contiguous()
                layer.out_weights = (take(lp + "out"), take(rp + "out"))
                layer.state_offset = state_floats
                state_floats += s.heads * s.state * s.vdim
                layer.extra_offset = state_floats  # the convolution's last inputs
                state_floats += s.conv_shape[0] * s.conv_shape[1]
            hc = lambda q, n: take(f"l{i}.hc{q}.{n}") if f"l{i}.hc{q}.{n}" in tensors else None
            layer.read1 = self.streams.read_site(take(f"l{i}.norm1"), hc(1, "in"))
            layer.write1 = self.streams.write_site(hc(1, "mix"), hc(1, "out"))
            ff = spec.get("mlp")
            if ff:
                if ff["kind"] != "dense":
                    raise ValueError(f"unknown feed-forward kind {ff['kind']!r}")
                fp = f"l{i}.mlp."
                layer.mlp = GatedMLP(take(fp + "gate"), take(fp + "up"), take(fp + "down"), "clamped_swish", b_gate=take(fp + "gate.b"),
                                     b_up=take(fp + "up.b"), b_down=take(fp + "down.b"), limit=float(ff["limit"]), slope=SWISH_SLOPE)
                layer.read2 = self.streams.read_site(take(f"l{i}.norm2"), hc(2, "in"))
                layer.write2 = self.streams.write_site(hc(2, "mix"), hc(2, "out"))
            self.layers.append(layer)
        self.final_read = self.streams.read_site(take("final.norm"))
        self.head = take("head")
        max_pages = None if max_tokens is None else -(-int(max_tokens) // page_size)
        self.page_pool = LatentPagedPool(widths, page_size=page_size, dtype=dtype, device=self.device, max_pages=max_pages)
        self.state_pool = StateSlotPool(state_floats, device=self.device, max_slots=max_requests)
        sizes = set()
        for layer in self.layers:
            if layer.attention is not None:
                sizes.add(layer.attention.tile_tokens)
            if layer.mixer is not None:
                sizes.add(blocks.attention_kernel(dtype, layer.mixer.heads, layer.mixer.rank, layer.mixer.rot_dim, page_size)[1])
        self.tile_sizes = sorted(sizes) or [blocks.ATTENTION_TILE_TOKENS]

    @classmethod
    def from_checkpoint(cls, config: dict, tensors: dict, **kwargs) -> "NorusunModel":
        return cls(config, tensors, **kwargs)

    # ---- cache ---------------------------------------------------------------------
    def create_kv_cache(self) -> list:
        """One entry per layer (what the schedulers expect); all are faces of ONE page list + state slot, held by entry 0."""
        owner = HybridPagedCache(self.page_pool, self.state_pool)
        return [owner] + [LatentCacheView(owner, max(layer.slab_index, 0)) for layer in self.layers[1:]]

    def _storage_version(self):
        return (self.page_pool.slab_version, self.state_pool.version)

    # ---- the layers over one plan ------------------------------------------------------
    def _mixer(self, layer: NorusunLayer, h: torch.Tensor, plan: RaggedPlan) -> torch.Tensor:
        view = self.state_pool.layer_view
        if layer.kind == "wkv":
            r = layer.recurrent
            return r(h, plan, view(layer.state_offset, r.state_shape), view(layer.extra_offset, r.shift_shape))
        if layer.kind == "latent_attention":
            return layer.mixer(h, plan, self.page_pool.slabs[layer.slab_index])
        y, lp, rp, s = layer.proj(h), layer.prefix + "left.", layer.prefix + "right.", layer.recurrent
        left = layer.attention(y[lp + "q"], y[lp + "k"], y[lp + "v"], None, plan, self.page_pool.slabs[layer.slab_index])
        conv = view(layer.extra_offset, s.conv_shape) if s.conv_shape[1] > 0 else None
        right = s(y[rp + "z"], y[rp + "xbc"], linear_wide(h, layer.w_dt), plan, view(layer.state_offset, s.state_shape), conv)
        return blocks.norm_mix2(left, layer.out_weights[0], right, layer.out_weights[1], 0.5, self.eps)

    def _forward_plan(self, plan: RaggedPlan) -> torch.Tensor:
        exact = self.precision == torch.float32
        tf32 = torch.backends.cuda.matmul.allow_tf32
        if exact:
            torch.backends.cuda.matmul.allow_tf32 = False  # fp32 means fp32
        try:
            x0, _ = blocks.embed_rows(plan.ids, self.embed)
            xs, h = self.streams.start(x0, self.layers[0].read1)
            for i, layer in enumerate(self.layers):
                if layer.canon is not None:  # h + conv(h), the last taps - 1 inputs kept in the request's slot
                    taps = layer.canon.shape[1]
                    hist = self.state_pool.layer_view(layer.canon_offset, (self.hidden_size, taps - 1)) if taps > 1 else None
                    h = blocks.short_conv(h, layer.canon, seq_info=plan.seq_info, state=hist, max_tokens=plan.max_tokens, act=0, add_input=True)
                mixed = self._mixer(layer, h, plan)
                following = self.layers[i + 1].read1 if i + 1 < len(self.layers) else None
                # the sublayer's write into the streams, fused with the read and norm of the sublayer that follows
                h = self.streams.step(xs, mixed, layer.write1, layer.read2 if layer.mlp is not None else following)
                if layer.mlp is not None:
                    h = self.streams.step(xs, layer.mlp(h, wide=True), layer.write2, following, y_bias=layer.mlp.down_bias)
                if self.stream_tap is not None:
                    self.stream_tap.append(xs.sum(dim=1))
            if plan.num_want == 0:  # a portion whose logits nobody asked for: caches and states are filled, that is all
                return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
            rows = xs.index_select(0, plan.want_rows.long())
            return linear_wide(self.streams.step(rows, None, None, self.final_read), self.head)  # the model's norm reads the streams' sum
        finally:
            if exact:
                torch.backends.cuda.matmul.allow_tf32 = tf32
