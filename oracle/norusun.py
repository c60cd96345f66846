"""Plain, slow restatement of the Norusun design on CPU tensors, one function per mechanism.

Written from the design's equations only; shares no code with the product path.  Every function
works on one whole sequence in the dtype of its inputs (float64 or float32), without a cache or a
carried state: recurrences and convolutions are explicit loops over the tokens from the first one.
Notation: ``T`` tokens, ``D`` model width, ``H`` heads, ``G`` key/value heads or state groups,
``dk`` query/key and ``dv`` value entries per head, ``n`` parallel residual streams.

``weights`` maps tensor names (``l<i>.mix.o`` ...) to tensors; ``config`` is the parsed
``config.json``.  A layer is ``type`` in ``wkv`` / ``latent_attention`` / ``parallel`` with the
mixer's sizes and a feed-forward (``dense`` or none).  The residual is ``streams`` copies mixed by
small learned matrices around every sublayer; every norm of the stack has ONE number as its weight;
the mixer's input first passes ``h + conv(h)``, a short causal convolution per channel.
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


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate(x: torch.Tensor, *, dims: int, base: float, layout: str, first: int = 0) -> torch.Tensor:
    """x [T, heads, d]: entries ``first .. first + dims - 1`` of every head turn by position * base^(-2i/dims); the
    partner of entry 2i is 2i+1 (``interleaved``) or that of entry i is i + dims/2 (``half``)."""
    T = x.shape[0]
    half = dims // 2
    out = x.clone()
    for t in range(T):
        for i in range(half):
            a = t * (base ** (-2.0 * i / dims))
            c, s = math.cos(a), math.sin(a)
            lo, hi = (2 * i, 2 * i + 1) if layout == "interleaved" else (i, i + half)
            u, v = x[t, :, first + lo], x[t, :, first + hi]
            out[t, :, first + lo] = u * c - v * s
            out[t, :, first + hi] = v * c + u * s
    return out


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """x [T, C], taps [C, K]: y[t, c] = bias[c] + sum_j taps[c, j] * x[t - (K-1) + j, c]; inputs before the sequence are zero."""
    T, C = x.shape
    K = taps.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(K):
            src = t - (K - 1) + j
            if src >= 0:
                y[t] += taps[:, j] * x[src]
        if bias is not None:
            y[t] += bias
    return y


def visible(i: int, j: int, kind: str, size: int) -> bool:
    """May position i read position j?  ``window``: itself and the size-1 before it; ``chunk``: the earlier ones of its own
    block of ``size`` positions counted from 0."""
    if j > i or j < 0:
        return False
    if kind == "window":
        return i - j < size
    if kind == "chunk":
        return i // size == j // size
    return True


# ---- the residual streams ---------------------------------------------------------------------
def streams_read(xs: torch.Tensor, w_in: torch.Tensor) -> torch.Tensor:
    """xs [n, T, D] -> the sublayer's input sum_s w_in[s] xs[s]."""
    return torch.einsum("s,std->td", w_in, xs)


def streams_write(xs: torch.Tensor, y: torch.Tensor, w_mix: torch.Tensor, w_out: torch.Tensor) -> torch.Tensor:
    """new[t] = sum_s w_mix[s, t] xs[s] + w_out[t] y; the right-hand side sees only the streams as they were."""
    return torch.einsum("sr,std->rtd", w_mix, xs) + w_out[:, None, None] * y[None]


# ---- mixers ---------------------------------------------------------------------------------------
def wkv_sum(r, k, v, w, u) -> torch.Tensor:
    """r, k, w [T, H, dk], v [T, H, dv], u [H, dk]: o_t = (S + diag(u) k_t v_t^T)^T r_t with S the state BEFORE token t,
    then S <- diag(w_t) S + k_t v_t^T."""
    T, H, dk = r.shape
    dv = v.shape[2]
    out = torch.zeros((T, H, dv), dtype=r.dtype)
    for h in range(H):
        S = torch.zeros((dk, dv), dtype=r.dtype)
        for t in range(T):
            kv = torch.outer(k[t, h], v[t, h])
            out[t, h] = (S + u[h][:, None] * kv).t() @ r[t, h]
            S = w[t, h][:, None] * S + kv
    return out


def wkv_mixer(h, weights, prefix, spec, *, eps) -> torch.Tensor:
    T, D = h.shape
    H, d = spec["heads"], spec["dim"]
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    shifted = lambda name: h + (before - h) * weights[prefix + "mu." + name]
    r = (shifted("r") @ weights[prefix + "r"].t()).view(T, H, d)
    k = (shifted("k") @ weights[prefix + "k"].t()).view(T, H, d)
    v = (shifted("v") @ weights[prefix + "v"].t()).view(T, H, d)
    gate = silu(shifted("g") @ weights[prefix + "g"].t())
    low = torch.tanh(shifted("w") @ weights[prefix + "w1"].t())
    w = torch.exp(-torch.exp(low @ weights[prefix + "w2"].t() + weights[prefix + "w0"])).view(T, H, d)
    o = rms_unit(wkv_sum(r, k, v, w, weights[prefix + "u"]), eps).reshape(T, H * d)
    return (o * weights[prefix + "norm"] * gate) @ weights[prefix + "o"].t()


def sink_softmax_attention(q, k, v, sink, *, scale, kind, size) -> torch.Tensor:
    """q, k [T, H, dk], v [T, H, dv], sink [H]: softmax over the visible keys whose denominator also holds exp(sink)."""
    T, H, _ = q.shape
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for h in range(H):
        for i in range(T):
            js = [j for j in range(T) if visible(i, j, kind, size)]
            s = (k[js, h] @ q[i, h]) * scale
            m = torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            p = e / (e.sum() + torch.exp(sink[h] - m))
            out[i, h] = p @ v[js, h]
    return out


def latent_mixer(h, weights, prefix, spec, *, eps) -> torch.Tensor:
    T = h.shape[0]
    H, dn, dr, dv, rank = spec["heads"], spec["dim"], spec["rot_dim"], spec["vdim"], spec["kv_rank"]
    cq = rms_unit(h @ weights[prefix + "dq"].t(), eps) * weights[prefix + "dq.norm"]
    q = (cq @ weights[prefix + "uq"].t()).view(T, H, dn + dr)
    down = h @ weights[prefix + "dkv"].t()
    c = rms_unit(down[:, :rank], eps) * weights[prefix + "dkv.norm"]
    rot = dict(dims=spec["rot"]["dims"], base=spec["rot"]["base"], layout="interleaved")
    k_rot = rotate(down[:, rank:].reshape(T, 1, dr), **rot)
    q = rotate(q, first=dn, **rot)
    k = torch.cat([(c @ weights[prefix + "uk"].t()).view(T, H, dn), k_rot.expand(T, H, dr)], dim=2)
    v = (c @ weights[prefix + "uv"].t()).view(T, H, dv)
    o = sink_softmax_attention(q, k, v, weights[prefix + "sink"], scale=spec["scale"], kind="window", size=spec["mask"]["size"])
    return o.reshape(T, H * dv) @ weights[prefix + "o"].t()


def sigmoid_attention(q, k, v, bias, *, scale, kind, size) -> torch.Tensor:
    """Every visible key weighs sigmoid(score + bias[h]); nothing is normalised over the keys."""
    T, H, _ = q.shape
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    for h in range(H):
        for i in range(T):
            js = [j for j in range(T) if visible(i, j, kind, size)]
            out[i, h] = torch.sigmoid((k[js, h] @ q[i, h]) * scale + bias[h]) @ v[js, h]
    return out


def chunk_mixer(h, weights, prefix, spec, *, eps) -> torch.Tensor:
    T = h.shape[0]
    H, G, dk, dv = spec["heads"], spec["kv_heads"], spec["dim"], spec["vdim"]
    q = rms_unit(h @ weights[prefix + "q"].t(), eps) * weights[prefix + "q.norm"]   # over the whole projection
    k = rms_unit(h @ weights[prefix + "k"].t(), eps) * weights[prefix + "k.norm"]
    v = (h @ weights[prefix + "v"].t()).view(T, G, dv)
    rot = dict(dims=spec["rot"]["dims"], base=spec["rot"]["base"], layout="half")
    q, k = rotate(q.view(T, H, dk), **rot), rotate(k.view(T, G, dk), **rot)
    k, v = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    o = sigmoid_attention(q, k, v, weights[prefix + "pb"], scale=spec["scale"], kind="chunk", size=spec["mask"]["size"])
    return o.reshape(T, H * dv) @ weights[prefix + "o"].t()


def state_space_sum(x, B, C, dt, a, skip) -> torch.Tensor:
    """x [T, H, P], B, C [T, G, N], dt [T, H] (already positive), a [H] (positive rate), skip [H]:
    S <- exp(-a dt_t) S + dt_t B_t x_t^T (S is N x P), y_t = S^T C_t + skip x_t."""
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    out = torch.zeros_like(x)
    for h in range(H):
        g = h // (H // G)
        S = torch.zeros((N, P), dtype=x.dtype)
        for t in range(T):
            S = torch.exp(-a[h] * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, g], x[t, h])
            out[t, h] = S.t() @ C[t, g] + skip[h] * x[t, h]
    return out


def state_space_mixer(h, weights, prefix, spec, *, eps) -> torch.Tensor:
    T = h.shape[0]
    H, P, N, G, parts = spec["heads"], spec["vdim"], spec["state"], spec["groups"], spec["norm_groups"]
    inner = H * P
    y = h @ weights[prefix + "in"].t()
    z, xbc, dt = y[:, :inner], y[:, inner : 2 * inner + 2 * G * N], y[:, 2 * inner + 2 * G * N :]
    xbc = silu(causal_conv(xbc, weights[prefix + "conv"], weights[prefix + "conv.b"]))
    x, B, C = xbc[:, :inner].reshape(T, H, P), xbc[:, inner : inner + G * N].reshape(T, G, N), xbc[:, inner + G * N :].reshape(T, G, N)
    dt = softplus(dt + weights[prefix + "dt_bias"])
    o = state_space_sum(x, B, C, dt, torch.exp(weights[prefix + "A_log"]), weights[prefix + "D"]).reshape(T, inner)
    o = o * silu(z)                                              # gated first, normed second
    o = rms_unit(o.view(T, parts, inner // parts), eps).reshape(T, inner) * weights[prefix + "norm"]
    return o @ weights[prefix + "o"].t()


def parallel_mixer(h, weights, prefix, spec, *, eps) -> torch.Tensor:
    left = chunk_mixer(h, weights, prefix + "left.", spec["left"], eps=eps)
    right = state_space_mixer(h, weights, prefix + "right.", spec["right"], eps=eps)
    return 0.5 * (rms_unit(left, eps) * weights[prefix + "left.out"] + rms_unit(right, eps) * weights[prefix + "right.out"])


# ---- feed-forward -------------------------------------------------------------------------------
def clamped_ff(h, weights, prefix, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ weights[prefix + "gate"].t() + weights[prefix + "gate.b"], max=limit)
    u = torch.clamp(h @ weights[prefix + "up"].t() + weights[prefix + "up.b"], min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ weights[prefix + "down"].t() + weights[prefix + "down.b"]


# ---- the stack ------------------------------------------------------------------------------------
MIXERS = {"wkv": wkv_mixer, "latent_attention": latent_mixer, "parallel": parallel_mixer}


def sublayer(xs, weights, config, i: int, q: int, fn):
    """One sublayer around the streams (or around the single stream of a model without ``streams``)."""
    eps = config["norm"]["eps"]
    hc = f"l{i}.hc{q}."
    many = hc + "in" in weights
    u = streams_read(xs, weights[hc + "in"]) if many else xs[0]
    y = fn(rms_unit(u, eps) * weights[f"l{i}.norm{q}"])
    if many:
        return streams_write(xs, y, weights[hc + "mix"], weights[hc + "out"])
    return (xs[0] + y)[None]


def layer_forward(xs, weights, config, i: int):
    spec, eps = config["layers"][i], config["norm"]["eps"]

    def mixer(h):
        if f"l{i}.canon1" in weights:
            h = h + causal_conv(h, weights[f"l{i}.canon1"])
        return MIXERS[spec["type"]](h, weights, f"l{i}.mix.", spec["mixer"], eps=eps)

    xs = sublayer(xs, weights, config, i, 1, mixer)
    if spec.get("mlp"):
        if spec["mlp"]["kind"] != "dense":
            raise ValueError(spec["mlp"]["kind"])
        xs = sublayer(xs, weights, config, i, 2, lambda h: clamped_ff(h, weights, f"l{i}.mlp.", float(spec["mlp"]["limit"])))
    return xs


def forward(ids, weights, config, dtype=torch.float64, tap: list | None = None) -> torch.Tensor:
    """ids: list of token ids -> logits [T, vocab]; ``tap`` receives the sum of the streams after every layer."""
    weights = {n: (t.to(dtype) if t.is_floating_point() else t) for n, t in weights.items()}
    x = weights["embed"][torch.tensor(list(ids), dtype=torch.long)]
    xs = x[None].repeat(int(config.get("streams") or 1), 1, 1)
    for i in range(len(config["layers"])):
        xs = layer_forward(xs, weights, config, i)
        if tap is not None:
            tap.append(xs.sum(dim=0))
    x = rms_unit(xs.sum(dim=0), config["norm"]["eps"]) * weights["final.norm"]
    return x @ weights["head"].t()


def greedy(ids, weights, config, new_tokens: int, dtype=torch.float64) -> list:
    ids, out = list(ids), []
    for _ in range(new_tokens):
        nxt = int(forward(ids, weights, config, dtype)[-1].argmax())
        out.append(nxt)
        ids.append(nxt)
    return out
