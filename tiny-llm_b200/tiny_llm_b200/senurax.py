"""Senurax: a pre-norm decoder (``x <- x + mixer(norm1(x))``, ``x <- x + ff(norm2(x))``, stream in fp32) whose layers
pick one of three mixers, whose middle layers may run several times with shared weights, and whose logits are soft-capped.

Mixers (``layers[i].type``):

- ``retention``: linear attention with one fixed decay per head (``mixer.decay``), queries and keys rotated by position
  (``rot``: pairs ``(i, i + dims/2)``), per-head RMS norm without weight, ``silu`` gate.
- ``channel_delta``: the gated delta rule with one decay per head and key channel (low-rank decay and gate projections
  ``a1 -> a2``, ``g1 -> g2``, sigmoid output gate), short convolutions on q, k, v.
- ``parallel``: two mixers on the same input.  ``mixer.left`` = causal grouped-query softmax attention over the paged
  cache, queries and keys rotated on their first ``rot.dims`` entries (pairs ``(2i, 2i+1)``, frequencies divided by
  ``rot.scaling.factor``); ``mixer.right`` = the gated delta rule with one decay per head and a ``silu`` gate.  Each
  output is RMS-normed over the width (``left.out`` / ``right.out``) and the layer takes half their sum.

Feed-forward (``mlp.kind``; ``mlp`` null = none): ``dense`` = ``down(relu(up x)^2)``; ``moe`` = ``router.top`` of
``router.experts`` gated experts ``down(silu(gate x) * up x)`` plus ``router.identity`` identity experts (no weights,
output = input), scores a softmax over all router outputs, chosen by score + ``correction``, weights the chosen scores
renormalised times ``router.scale``.

``loop`` = ``{start, stop, times}``: layers ``start .. stop-1`` run ``times`` times in a row with the same weights and a
cache / state of their own per pass; every pass is entered by ``x <- loop.in [x; x0] + loop.step[pass]`` with ``x0`` the
embedding.  ``logit_softcap`` c: ``logits <- c tanh(logits / c)``.  Everything that can differ between models of the
design is read from ``config.json`` (``vocab``, ``width``, ``norm.eps``, the layers' ``heads kv_heads dim vdim scale
rot decay``) or from a tensor's shape (taps of the convolutions, low ranks).

The model is the framework's usual object (``RaggedDecoderModel``).  A request holds one page list for all attention
layer runs (``LatentPagedPool``: one slab per run) and one slot of the ``StateSlotPool`` with a block per recurrent run
(matrix state and the convolution's last inputs).  Compute dtype bf16 (serving) or fp32 (every product in true fp32);
norms, softmax, router, decays, unit vectors, recurrent state, rotations that feed a recurrence and the residual sum
are fp32 in both.
"""

from __future__ import annotations

import torch

from extensions_b200.tiny_llm_ext_b200 import blocks

from .basics import linear_wide
from .delta_rule import GatedDeltaRule
from .latent_kv_cache import LatentCacheView, LatentPagedPool
from .linear_attention import RetainedLinearAttention
from .mlp import DenseMLP, MixtureOfExperts, TopKRouter
from .paged_attention import FusedProjection, PagedGroupedAttention
from .ragged import RaggedPlan
from .ragged_model import RaggedDecoderModel
from .state_cache import HybridPagedCache, StateSlotPool

MIXERS = ("retention", "channel_delta", "parallel")


class SenuraxLayer:
    """One layer's weights and modules (shared by all its runs)."""

    def __init__(self, kind: str, norm1, norm2, proj: FusedProjection, prefix: str, mlp, attention=None, recurrent=None, out_weights=None):
        self.kind, self.norm1, self.norm2, self.proj, self.prefix, self.mlp = kind, norm1, norm2, proj, prefix, mlp
        self.attention, self.recurrent, self.out_weights = attention, recurrent, out_weights


class SenuraxRun:
    """One execution of a layer: which pass of the loop it belongs to and where its cache and state live."""

    def __init__(self, layer: int, loop_pass: int | None, enters_pass: bool, slab_index: int = -1, state_offset: int = 0, conv_offset: int = 0):
        self.layer, self.loop_pass, self.enters_pass = layer, loop_pass, enters_pass
        self.slab_index, self.state_offset, self.conv_offset = slab_index, state_offset, conv_offset


def layer_runs(num_layers: int, loop: dict | None) -> list:
    """[(layer, pass or None, first of its pass)] in execution order."""
    if not loop:
        return [(i, None, False) for i in range(num_layers)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    if not (0 <= start < stop <= num_layers) or times < 1:
        raise ValueError(f"loop {loop} does not fit {num_layers} layers")
    runs = [(i, None, False) for i in range(start)]
    for t in range(times):
        runs += [(i, t, i == start) for i in range(start, stop)]
    return runs + [(i, None, False) for i in range(stop, num_layers)]


class SenuraxModel(RaggedDecoderModel):
    architecture = "Senurax"
    graph_env = "TL_SENURAX_GRAPH"

    def __init__(self, config: dict, tensors: dict, dtype=torch.bfloat16, device="cuda", page_size: int = 64, max_tokens: int | None = None,
                 max_requests: int | None = None):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("Senurax runs in bfloat16 or float32")
        self.config, self.precision, self.device = config, dtype, torch.device(device)
        self.vocab_size, self.hidden_size = int(config["vocab"]), int(config["width"])
        self.eps = float(config["norm"]["eps"])
        self.num_hidden_layers = len(config["layers"])
        self.page_size = page_size
        self.softcap = float(config.get("logit_softcap") or 0.0)
        self.stream_tap: list | None = None  # a list here receives a copy of the residual stream after every layer run
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
        self.layers: list[SenuraxLayer] = []
        for i, spec in enumerate(config["layers"]):
            kind, m, p = spec["type"], spec["mixer"], f"l{i}.mix."
            if kind not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            attention = recurrent = outs = None
            if kind == "retention":
                recurrent = RetainedLinearAttention(heads=m["heads"], dim=m["dim"], vdim=m["vdim"], decay=m["decay"], w_o=take(p + "o"), eps=self.eps,
                                                    rot=self._rot(m.get("rot")))
                parts = [(p + n, take(p + n), None) for n in ("q", "k", "v", "g")]
            elif kind == "channel_delta":
                recurrent = self._delta(m, p, take, channel=True)
                parts = [(p + n, take(p + n), None) for n in ("q", "k", "v", "g1", "a1", "b")]
            else:
                a, lp, rp = m["left"], p + "left.", p + "right."
                rot = self._rot(a.get("rot"))
                attention = PagedGroupedAttention(heads=a["heads"], kv_heads=a["kv_heads"], dim=a["dim"], vdim=a["vdim"], scale=a["scale"], mask="causal",
                                                  mask_size=0, w_o=take(lp + "o"), eps=self.eps, page_size=page_size,
                                                  rot=None if rot is None else dict(rot, interleaved=True))
                recurrent = self._delta(m["right"], rp, take, channel=False)
                parts = [(lp + n, take(lp + n), None) for n in ("q", "k", "v")] + [(rp + n, take(rp + n), None) for n in ("q", "k", "v", "g", "a", "b")]
                outs = (take(lp + "out"), take(rp + "out"))
            mlp = self._feed_forward(spec.get("mlp"), f"l{i}.mlp.", take, tensors)
            self.layers.append(SenuraxLayer(kind, take(f"l{i}.norm1"), take(f"l{i}.norm2") if mlp is not None else None,
                                            FusedProjection(parts, dtype, self.device), p, mlp, attention, recurrent, outs))

        loop = config.get("loop") or None
        self.loop_in = self.loop_step = None
        if loop:
            self.loop_in = take("loop.in")
            self.loop_step = take("loop.step").float().contiguous()  # added to the fp32 stream
            if tuple(self.loop_in.shape) != (D, 2 * D) or tuple(self.loop_step.shape) != (int(loop["times"]), D):
                raise ValueError("loop.in must be [width, 2 width] and loop.step [times, width]")
        # every run of a layer has a cache slab (attention) and a block of the state slot (recurrent mixers) of its own
        self.runs: list[SenuraxRun] = []
        widths: list[int] = []
        state_floats = 0
        for i, t, first in layer_runs(self.num_hidden_layers, loop):
            layer, run = self.layers[i], SenuraxRun(i, t, first)
            if layer.attention is not None:
                run.slab_index = len(widths)
                widths.append(layer.attention.cache_width)
            r = layer.recurrent
            run.state_offset = state_floats
            state_floats += r.heads * r.dim * r.vdim
            if isinstance(r, GatedDeltaRule):
                run.conv_offset = state_floats
                state_floats += r.conv_shape[0] * r.conv_shape[1]
            self.runs.append(run)
        self.final_norm = take("final.norm")
        self.head = take("head")
        max_pages = None if max_tokens is None else -(-int(max_tokens) // page_size)
        self.page_pool = LatentPagedPool(widths, page_size=page_size, dtype=dtype, device=self.device, max_pages=max_pages)
        self.state_pool = StateSlotPool(state_floats, device=self.device, max_slots=max_requests)
        self.tile_sizes = sorted({layer.attention.tile_tokens for layer in self.layers if layer.attention is not None}) or [blocks.ATTENTION_TILE_TOKENS]

    @staticmethod
    def _rot(spec):
        if not spec or not int(spec.get("dims", 0)):
            return None
        return {"dims": int(spec["dims"]), "base": float(spec["base"]), "factor": float((spec.get("scaling") or {}).get("factor", 1.0))}

    def _delta(self, m: dict, p: str, take, channel: bool) -> GatedDeltaRule:
        taps = torch.cat([take(p + "q.conv"), take(p + "k.conv"), take(p + "v.conv")], dim=0)
        return GatedDeltaRule(heads=m["heads"], key_heads=m.get("kv_heads", m["heads"]), dim=m["dim"], vdim=m["vdim"], taps=taps, a_log=take(p + "A_log"),
                              dt_bias=take(p + "dt_bias"), norm_weight=take(p + "norm"), w_o=take(p + "o"), eps=self.eps, channel_decay=channel,
                              w_a2=take(p + "a2") if channel else None, w_g2=take(p + "g2") if channel else None,
                              gate_act="sigmoid" if channel else "silu")

    @staticmethod
    def _feed_forward(spec, prefix: str, take, tensors):
        if not spec:
            return None
        if spec["kind"] == "dense":
            return DenseMLP(take(prefix + "up"), take(prefix + "down"), "relu_squared")
        if spec["kind"] != "moe":
            raise ValueError(f"unknown feed-forward kind {spec['kind']!r}")
        r = spec["router"]
        experts, top, identity = int(r["experts"]), int(r["top"]), int(r.get("identity", 0))
        router = TopKRouter(take(prefix + "router"), None, top, scoring="softmax_all", choice_bias=take(prefix + "correction") if prefix + "correction" in tensors else None,
                            weight_scale=float(r.get("scale", 1.0)))
        stack = lambda part: torch.stack([take(f"{prefix}e{k}.{part}") for k in range(experts)]).contiguous()
        return MixtureOfExperts(router, stack("gate"), stack("up"), stack("down"), "silu", identity=identity)

    @classmethod
    def from_checkpoint(cls, config: dict, tensors: dict, **kwargs) -> "SenuraxModel":
        return cls(config, tensors, **kwargs)

    # ---- cache ---------------------------------------------------------------------
    def create_kv_cache(self) -> list:
        """One entry per layer (what the schedulers expect); all are faces of ONE page list + state slot, held by entry 0."""
        owner = HybridPagedCache(self.page_pool, self.state_pool)
        return [owner] + [LatentCacheView(owner, 0) for _ in self.layers[1:]]

    def _storage_version(self):
        return (self.page_pool.slab_version, self.state_pool.version)

    # ---- the layers over one plan ------------------------------------------------------
    def _mixer(self, layer: SenuraxLayer, run: SenuraxRun, h: torch.Tensor, plan: RaggedPlan) -> torch.Tensor:
        y, p, r = layer.proj(h), layer.prefix, layer.recurrent
        state = self.state_pool.layer_view(run.state_offset, r.state_shape)
        if layer.kind == "retention":
            return r(y[p + "q"], y[p + "k"], y[p + "v"], y[p + "g"], plan, state)
        rp = p if layer.kind == "channel_delta" else p + "right."
        qkv = self._span(y[rp + "q"], r.channels)  # q | k | v are adjacent parts of the fused product
        conv = self.state_pool.layer_view(run.conv_offset, r.conv_shape) if r.conv_shape[1] > 0 else None
        if layer.kind == "channel_delta":
            return r(qkv, y[rp + "b"], y[rp + "a1"], y[rp + "g1"], plan, state, conv)
        right = r(qkv, y[rp + "b"], y[rp + "a"], y[rp + "g"], plan, state, conv)
        lp = p + "left."
        left = layer.attention(y[lp + "q"], y[lp + "k"], y[lp + "v"], None, plan, self.page_pool.slabs[run.slab_index])
        return blocks.norm_mix2(left, layer.out_weights[0], right, layer.out_weights[1], 0.5, self.eps)

    @staticmethod
    def _span(part: torch.Tensor, width: int) -> torch.Tensor:
        """``width`` columns of the fused product starting where ``part`` starts (several adjacent parts as one view)."""
        return part.as_strided((part.shape[0], width), part.stride(), part.storage_offset())

    def _forward_plan(self, plan: RaggedPlan) -> torch.Tensor:
        exact = self.precision == torch.float32
        tf32 = torch.backends.cuda.matmul.allow_tf32
        if exact:
            torch.backends.cuda.matmul.allow_tf32 = False  # fp32 means fp32
        try:
            D = self.hidden_size
            x32, _ = blocks.embed_rows(plan.ids, self.embed)
            both = None
            if self.loop_in is not None:  # [x | x0] in the compute dtype: the right half is written once
                both = torch.empty((x32.shape[0], 2 * D), dtype=self.precision, device=self.device)
                blocks.cast_rows(x32, both[:, D:])
            h = None
            for n, run in enumerate(self.runs):
                layer = self.layers[run.layer]
                if run.enters_pass:
                    blocks.cast_rows(x32, both[:, :D])
                    x32 = linear_wide(both, self.loop_in)
                    h = blocks.add_norm(x32, self.loop_step[run.loop_pass], None, layer.norm1, self.eps)
                elif h is None:
                    h = blocks.norm_residual(x32, layer.norm1, self.eps)
                mixed = self._mixer(layer, run, h, plan)
                following = None
                if n + 1 < len(self.runs) and not self.runs[n + 1].enters_pass:
                    following = self.layers[self.runs[n + 1].layer].norm1
                if layer.mlp is not None:
                    h = blocks.add_norm(x32, mixed, None, layer.norm2, self.eps)
                    mixed = layer.mlp(h)
                # the sublayer's sum, fused with the norm that reads the stream next (the model's norm runs on the wanted rows only)
                h = blocks.add_norm(x32, mixed, None, following, self.eps)
                if self.stream_tap is not None:
                    self.stream_tap.append(x32.clone())
            if plan.num_want == 0:  # a portion whose logits nobody asked for: caches and states are filled, that is all
                return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
            rows = x32.index_select(0, plan.want_rows.long())
            logits = linear_wide(blocks.norm_residual(rows, self.final_norm, self.eps), self.head)
            return blocks.softcap_rows(logits, self.softcap) if self.softcap > 0 else logits
        finally:
            if exact:
                torch.backends.cuda.matmul.allow_tf32 = tf32
