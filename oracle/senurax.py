"""Plain, slow restatement of the Senurax design on CPU tensors, one function per mechanism.

Written from the design's equations only; shares no code with the product path.  Every function
works on one whole sequence in the dtype of its inputs (float64 or float32), without a cache or a
carried state: recurrences are explicit loops over the tokens from the first one.  Notation: ``T``
tokens, ``D`` model width, ``H`` heads, ``G`` key heads (query/key heads of a delta mixer, key/value
heads of softmax attention), ``dk`` query/key and ``dv`` value entries per head.

``weights`` maps tensor names (``l<i>.mix.q`` ...) to tensors; ``config`` is the parsed
``config.json``.  The stack: ``layers[i]`` has ``type`` in ``retention`` / ``channel_delta`` /
``parallel``, the mixer's sizes, and a feed-forward (``dense``, ``moe`` or none); the layers
``loop.start .. loop.stop - 1`` run ``loop.times`` times in a row with shared weights, every pass
entered through a mixing product with the embedding.
"""

from __future__ import annotations

import math

import torch


# ---- small pieces ---------------------------------------------------------------------------
def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def relu_squared(z):
    return torch.relu(z).pow(2)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate(x: torch.Tensor, *, dims: int, base: float, factor: float = 1.0, layout: str) -> torch.Tensor:
    """x [T, heads, d]: the first ``dims`` entries of every head turn by position * base^(-2i/dims) / factor; the
    partner of entry 2i is 2i+1 (``interleaved``) or that of entry i is i + dims/2 (``half``)."""
    T = x.shape[0]
    half = dims // 2
    out = x.clone()
    for t in range(T):
        for i in range(half):
            a = t * (base ** (-2.0 * i / dims)) / factor
            c, s = math.cos(a), math.sin(a)
            lo, hi = (2 * i, 2 * i + 1) if layout == "interleaved" else (i, i + half)
            u, v = x[t, :, lo], x[t, :, hi]
            out[t, :, lo] = u * c - v * s
            out[t, :, hi] = v * c + u * s
    return out


def short_conv_silu(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K]: y[t, c] = silu(sum_j taps[c, K-1-j] * x[t-j, c]), inputs before the sequence are zero."""
    T, C = x.shape
    K = taps.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        acc = torch.zeros(C, dtype=x.dtype)
        for j in range(K):
            if t - j >= 0:
                acc = acc + taps[:, K - 1 - j] * x[t - j]
        y[t] = silu(acc)
    return y


# ---- mixers -----------------------------------------------------------------------------------
def causal_attention(q, k, v, scale: float) -> torch.Tensor:
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] -> [T, H, dv]; head h reads key/value head h // (H / G); position i sees
    0..i; plain softmax."""
    T, H, _ = q.shape
    per = H // k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for i in range(T):
        for h in range(H):
            g = h // per
            s = (k[: i + 1, g] @ q[i, h]) * scale
            p = torch.softmax(s, dim=0)
            out[i, h] = p @ v[: i + 1, g]
    return out


def delta_rule(q, k, v, beta, decay) -> torch.Tensor:
    """q, k [T, H, dk] (already per value head), v [T, H, dv], beta [T, H], decay [T, H] or [T, H, dk] -> [T, H, dv].
    Per head, with S [dk, dv] from zero:  S = decay * S (rows);  u = beta (v - S^T k);  S = S + k u^T;  o = S^T q."""
    T, H, dk = q.shape
    dv = v.shape[2]
    S = torch.zeros((H, dk, dv), dtype=q.dtype)
    out = torch.zeros((T, H, dv), dtype=q.dtype)
    for t in range(T):
        g = decay[t]
        g = g[:, None, None] if g.dim() == 1 else g[:, :, None]
        S = g * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + torch.einsum("hk,hv->hkv", k[t], u)
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def retained_sum(q, k, v, decay) -> torch.Tensor:
    """Linear attention with one fixed decay per head: S = decay_h S + k v^T, o = S^T q.  q, k [T, H, dk], v [T, H, dv]."""
    T, H, dk = q.shape
    S = torch.zeros((H, dk, v.shape[2]), dtype=q.dtype)
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    d = torch.as_tensor(decay, dtype=q.dtype)[:, None, None]
    for t in range(T):
        S = d * S + torch.einsum("hk,hv->hkv", k[t], v[t])
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def delta_mixer(h, weights, prefix, spec, *, eps, channel_decay: bool) -> torch.Tensor:
    """The gated delta-rule mixer.  ``channel_decay``: the decay has one value per head and key channel, from a two-step
    projection, and the output gate is a sigmoid of a two-step projection; else one decay per head and a silu gate."""
    H, G, dk, dv = spec["heads"], spec["kv_heads"], spec["dim"], spec["vdim"]
    T = h.shape[0]
    w = lambda name: weights[prefix + name].to(h.dtype)
    q = short_conv_silu(h @ w("q").T, w("q.conv")).view(T, G, dk)
    k = short_conv_silu(h @ w("k").T, w("k.conv")).view(T, G, dk)
    v = short_conv_silu(h @ w("v").T, w("v.conv")).view(T, H, dv)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    per = H // G
    q = q.repeat_interleave(per, dim=1)
    k = k.repeat_interleave(per, dim=1)
    beta = torch.sigmoid(h @ w("b").T)
    rate = torch.exp(w("A_log"))
    if channel_decay:
        step = softplus((h @ w("a1").T) @ w("a2").T + w("dt_bias")).view(T, H, dk)
        decay = torch.exp(-rate[None, :, None] * step)
        gate = torch.sigmoid((h @ w("g1").T) @ w("g2").T)
    else:
        decay = torch.exp(-rate[None, :] * softplus(h @ w("a").T + w("dt_bias")))
        gate = silu(h @ w("g").T)
    o = delta_rule(q, k, v, beta, decay)
    o = rms_unit(o, eps) * w("norm")
    return (o.reshape(T, H * dv) * gate) @ w("o").T


def softmax_mixer(h, weights, prefix, spec) -> torch.Tensor:
    H, G, dk, dv = spec["heads"], spec["kv_heads"], spec["dim"], spec["vdim"]
    T = h.shape[0]
    w = lambda name: weights[prefix + name].to(h.dtype)
    rot = spec.get("rot")
    q = (h @ w("q").T).view(T, H, dk)
    k = (h @ w("k").T).view(T, G, dk)
    v = (h @ w("v").T).view(T, G, dv)
    if rot:
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        q = rotate(q, dims=rot["dims"], base=rot["base"], factor=factor, layout="interleaved")
        k = rotate(k, dims=rot["dims"], base=rot["base"], factor=factor, layout="interleaved")
    o = causal_attention(q, k, v, spec["scale"])
    return o.reshape(T, H * dv) @ w("o").T


def retention_mixer(h, weights, prefix, spec, *, eps) -> torch.Tensor:
    H, dk, dv = spec["heads"], spec["dim"], spec["vdim"]
    T = h.shape[0]
    w = lambda name: weights[prefix + name].to(h.dtype)
    rot = spec.get("rot")
    q = (h @ w("q").T).view(T, H, dk)
    k = (h @ w("k").T).view(T, H, dk)
    v = (h @ w("v").T).view(T, H, dv)
    if rot:
        factor = float((rot.get("scaling") or {}).get("factor", 1.0))
        q = rotate(q, dims=rot["dims"], base=rot["base"], factor=factor, layout="half")
        k = rotate(k, dims=rot["dims"], base=rot["base"], factor=factor, layout="half")
    k = k * dk ** -0.5
    o = rms_unit(retained_sum(q, k, v, spec["decay"]), eps)
    return (o.reshape(T, H * dv) * silu(h @ w("g").T)) @ w("o").T


def parallel_mixer(h, weights, prefix, spec, *, eps) -> torch.Tensor:
    left = softmax_mixer(h, weights, prefix + "left.", spec["left"])
    right = delta_mixer(h, weights, prefix + "right.", spec["right"], eps=eps, channel_decay=False)
    w = lambda name: weights[prefix + name].to(h.dtype)
    return 0.5 * (rms_unit(left, eps) * w("left.out") + rms_unit(right, eps) * w("right.out"))


# ---- feed-forward -------------------------------------------------------------------------------
def dense_ff(h, weights, prefix) -> torch.Tensor:
    w = lambda name: weights[prefix + name].to(h.dtype)
    return relu_squared(h @ w("up").T) @ w("down").T


def route(h, weights, prefix, router):
    """-> (chosen [T, top] indices into experts + identity, weights [T, top]).  Softmax over all router outputs; the choice
    adds the correction to the scores, the weights do not; chosen scores are renormalised and scaled."""
    w = lambda name: weights[prefix + name].to(h.dtype)
    s = torch.softmax(h @ w("router").T, dim=-1)
    chosen = torch.topk(s + w("correction"), int(router["top"]), dim=-1).indices
    picked = torch.gather(s, 1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20) * float(router.get("scale", 1.0))


def expert_mixture(h, weights, prefix, spec) -> torch.Tensor:
    router = spec["router"]
    E = int(router["experts"])
    chosen, weight = route(h, weights, prefix, router)
    w = lambda name: weights[prefix + name].to(h.dtype)
    y = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            if e >= E:  # an identity expert: the token itself
                y[t] += g * h[t]
            else:
                y[t] += g * ((silu(h[t] @ w(f"e{e}.gate").T) * (h[t] @ w(f"e{e}.up").T)) @ w(f"e{e}.down").T)
    return y


# ---- the stack ----------------------------------------------------------------------------------
def layer_runs(config: dict) -> list:
    """The order in which layers run: [(layer index, pass number or None, first of its pass)]."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None, False) for i in range(start)]
    for t in range(times):
        runs += [(i, t, i == start) for i in range(start, stop)]
    return runs + [(i, None, False) for i in range(stop, n)]


def layer_forward(x, weights, config, i: int) -> torch.Tensor:
    spec = config["layers"][i]
    eps = float(config["norm"]["eps"])
    p = f"l{i}."
    h = rms_unit(x, eps) * weights[p + "norm1"].to(x.dtype)
    kind = spec["type"]
    if kind == "retention":
        m = retention_mixer(h, weights, p + "mix.", spec["mixer"], eps=eps)
    elif kind == "channel_delta":
        m = delta_mixer(h, weights, p + "mix.", spec["mixer"], eps=eps, channel_decay=True)
    elif kind == "parallel":
        m = parallel_mixer(h, weights, p + "mix.", spec["mixer"], eps=eps)
    else:
        raise ValueError(kind)
    x = x + m
    ff = spec.get("mlp")
    if ff:
        h = rms_unit(x, eps) * weights[p + "norm2"].to(x.dtype)
        x = x + (dense_ff(h, weights, p + "mlp.") if ff["kind"] == "dense" else expert_mixture(h, weights, p + "mlp.", ff))
    return x


def forward(ids, weights, config, dtype=torch.float64, tap: list | None = None) -> torch.Tensor:
    """Token ids of ONE sequence -> logits [T, vocab]; ``tap`` receives the stream after every layer run."""
    eps = float(config["norm"]["eps"])
    x0 = weights["embed"].to(dtype)[torch.as_tensor(ids, dtype=torch.long)]
    x = x0
    for i, t, first in layer_runs(config):
        if first:
            x = torch.cat([x, x0], dim=-1) @ weights["loop.in"].to(dtype).T + weights["loop.step"].to(dtype)[t]
        x = layer_forward(x, weights, config, i)
        if tap is not None:
            tap.append(x.clone())
    logits = (rms_unit(x, eps) * weights["final.norm"].to(dtype)) @ weights["head"].to(dtype).T
    cap = config.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits


def greedy(ids, weights, config, new_tokens: int, dtype=torch.float64) -> list:
    """``new_tokens`` greedy tokens after the prompt, by recomputing the whole sequence for each."""
    ids, out = list(ids), []
    for _ in range(new_tokens):
        out.append(int(forward(ids, weights, config, dtype)[-1].argmax()))
        ids.append(out[-1])
    return out
