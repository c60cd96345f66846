"""Synthetic Qwen3-shaped W4A16 checkpoints in the ``mlx_model`` duck type.

There is no network here, so benchmarks and tests run on random weights of the
right architecture.  The object mirrors what
``mlx_lm.load`` returns as far as the models look at it
(``/root/reference/src/tiny_llm_ref/qwen3_week3.py:225-313``; minimal fake at
``/root/reference/tests/utils.py:12-69``): ``.args`` plus
``.model.{embed_tokens, layers[i].{self_attn, mlp, *_layernorm}, norm}`` where
every quantised layer carries ``weight`` (packed u32), ``scales``, ``biases``,
``group_size`` and ``bits``.

Tensors are always generated on the CPU from a seeded generator (so the CPU
oracle and every GPU rank see identical bytes) and then moved to ``device``.
"""

from __future__ import annotations

from types import SimpleNamespace

import torch

GROUP_SIZE = 128
BITS = 4

# Published Qwen3 dense configs (hidden, layers, heads, kv heads, head dim, mlp).
CONFIGS = {
    "qwen3-4b": dict(hidden_size=2560, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=9728, vocab_size=151936),
    "qwen3-1.7b": dict(hidden_size=2048, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=6144, vocab_size=151936),
    "qwen3-0.6b": dict(hidden_size=1024, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8, head_dim=128, intermediate_size=3072, vocab_size=151936),
    # small shapes for tests (same structure, every kernel family exercised)
    "tiny": dict(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32, intermediate_size=256, vocab_size=128),
    "tiny-d128": dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128, intermediate_size=384, vocab_size=512),
}


def make_args(name_or_dims, **overrides) -> SimpleNamespace:
    dims = dict(CONFIGS[name_or_dims]) if isinstance(name_or_dims, str) else dict(name_or_dims)
    dims.setdefault("rms_norm_eps", 1e-6)
    dims.setdefault("max_position_embeddings", 40960)
    dims.setdefault("rope_theta", 1000000)
    dims.setdefault("tie_word_embeddings", True)
    dims.update(overrides)
    return SimpleNamespace(**dims)


def quantize_w4(weight: torch.Tensor, group_size: int = GROUP_SIZE):
    """Plain affine min/max 4-bit quantiser (our own; ``mx.quantize`` is not in
    the reference tree).  Returns (packed uint32 [K, N/8], scales, biases) in
    the layout ``dequantize_weights`` decodes."""
    K, N = weight.shape
    assert N % group_size == 0
    groups = weight.to(torch.float32).reshape(K, N // group_size, group_size)
    lo = groups.amin(dim=-1, keepdim=True)
    hi = groups.amax(dim=-1, keepdim=True)
    scale = ((hi - lo) / 15.0).clamp_min(1e-8)
    scale_b = scale.to(torch.bfloat16)
    bias_b = lo.to(torch.bfloat16)
    codes = torch.round((groups - bias_b.to(torch.float32)) / scale_b.to(torch.float32)).clamp_(0, 15).to(torch.int64)
    codes = codes.reshape(K, N // 8, 8)
    shifts = torch.arange(0, 32, 4, dtype=torch.int64)
    words = (codes << shifts).sum(dim=-1)  # < 2^32
    words = torch.where(words >= 2**31, words - 2**32, words).to(torch.int32)
    return words.view(torch.uint32), scale_b.squeeze(-1).contiguous(), bias_b.squeeze(-1).contiguous()


def _random_layer(out_dim: int, in_dim: int, gen: torch.Generator) -> SimpleNamespace:
    """Random codes + signed scales; dequantised weights ~ N(0, 1/in_dim)
    (value = (q-7.5)*s + e with q uniform: var = 22.25*sigma^2)."""
    sigma = 1.0 / (4.717 * in_dim**0.5)
    words = torch.randint(-(2**31), 2**31, (out_dim, in_dim // 8), dtype=torch.int64, generator=gen).to(torch.int32)
    scales = (torch.randn(out_dim, in_dim // GROUP_SIZE, generator=gen) * sigma).to(torch.bfloat16)
    biases = (-7.5 * scales.to(torch.float32) + torch.randn(out_dim, in_dim // GROUP_SIZE, generator=gen) * sigma).to(torch.bfloat16)
    return SimpleNamespace(weight=words.view(torch.uint32), scales=scales, biases=biases, group_size=GROUP_SIZE, bits=BITS)


def _quantized_layer(out_dim: int, in_dim: int, gen: torch.Generator, std: float) -> SimpleNamespace:
    dense = torch.randn(out_dim, in_dim, generator=gen) * std
    words, scales, biases = quantize_w4(dense)
    return SimpleNamespace(weight=words, scales=scales, biases=biases, group_size=GROUP_SIZE, bits=BITS)


def _norm_weight(dim: int, gen: torch.Generator) -> SimpleNamespace:
    return SimpleNamespace(weight=(1.0 + 0.1 * torch.randn(dim, generator=gen)).to(torch.bfloat16))


def _empty_norm(dim: int, device) -> SimpleNamespace:
    return SimpleNamespace(weight=torch.empty((dim,), dtype=torch.bfloat16, device=device))


def _empty_layer(out_dim: int, in_dim: int, device) -> SimpleNamespace:
    return SimpleNamespace(
        weight=torch.empty((out_dim, in_dim // 8), dtype=torch.int32, device=device).view(torch.uint32),
        scales=torch.empty((out_dim, in_dim // GROUP_SIZE), dtype=torch.bfloat16, device=device),
        biases=torch.empty((out_dim, in_dim // GROUP_SIZE), dtype=torch.bfloat16, device=device),
        group_size=GROUP_SIZE,
        bits=BITS,
    )


def synthetic_qwen3(name_or_dims="qwen3-4b", seed: int = 0, device="cpu", realistic: bool = False, empty: bool = False,
                    **overrides) -> SimpleNamespace:
    """Random Qwen3-shaped model.  ``realistic=True`` quantises Gaussian dense
    weights with ``quantize_w4`` (slow, for small models); the default draws
    codes/scales directly, which is what the 4B-sized benchmarks use.
    ``empty=True`` only allocates (uninitialised, directly on ``device``): the
    receive side of the data-parallel weight broadcast."""
    args = make_args(name_or_dims, **overrides)
    gen = torch.Generator().manual_seed(seed)

    def layer(out_dim: int, in_dim: int) -> SimpleNamespace:
        if empty:
            return _empty_layer(out_dim, in_dim, device)
        if realistic:
            return _quantized_layer(out_dim, in_dim, gen, std=in_dim**-0.5)
        return _random_layer(out_dim, in_dim, gen)

    def norm(dim: int) -> SimpleNamespace:
        return _empty_norm(dim, device) if empty else _norm_weight(dim, gen)

    q_width = args.num_attention_heads * args.head_dim
    kv_width = args.num_key_value_heads * args.head_dim
    layers = []
    for _ in range(args.num_hidden_layers):
        layers.append(
            SimpleNamespace(
                self_attn=SimpleNamespace(
                    q_proj=layer(q_width, args.hidden_size),
                    k_proj=layer(kv_width, args.hidden_size),
                    v_proj=layer(kv_width, args.hidden_size),
                    o_proj=layer(args.hidden_size, q_width),
                    q_norm=norm(args.head_dim),
                    k_norm=norm(args.head_dim),
                ),
                mlp=SimpleNamespace(
                    gate_proj=layer(args.intermediate_size, args.hidden_size),
                    up_proj=layer(args.intermediate_size, args.hidden_size),
                    down_proj=layer(args.hidden_size, args.intermediate_size),
                ),
                input_layernorm=norm(args.hidden_size),
                post_attention_layernorm=norm(args.hidden_size),
            )
        )
    model = SimpleNamespace(
        args=args,
        model=SimpleNamespace(embed_tokens=layer(args.vocab_size, args.hidden_size), layers=layers, norm=norm(args.hidden_size)),
    )
    if not args.tie_word_embeddings:
        model.lm_head = layer(args.vocab_size, args.hidden_size)
    return model if empty else to_device(model, device)


def to_device(node, device):
    """Move every tensor of the namespace tree to ``device`` (in place)."""
    if isinstance(node, SimpleNamespace):
        for key, value in vars(node).items():
            setattr(node, key, to_device(value, device))
        return node
    if isinstance(node, list):
        return [to_device(item, device) for item in node]
    if isinstance(node, torch.Tensor):
        return node.to(device)
    return node


def named_tensors(node, prefix=""):
    """Depth-first (name, tensor) walk in a deterministic order - the order the
    data-parallel launcher broadcasts weights in."""
    if isinstance(node, SimpleNamespace):
        for key in sorted(vars(node)):
            yield from named_tensors(getattr(node, key), f"{prefix}{key}.")
    elif isinstance(node, list):
        for index, item in enumerate(node):
            yield from named_tensors(item, f"{prefix}{index}.")
    elif isinstance(node, torch.Tensor):
        yield prefix[:-1], node


def weight_stream_bytes(args) -> int:
    """Packed bytes one decode token must stream (projections of every layer +
    tied head): 0.53125 B per weight = N/2 codes + 4 B of scale/bias per 128
    (/root/reference/book/src/week2-03-quantize-model.md:179-181)."""
    q_width = args.num_attention_heads * args.head_dim
    kv_width = args.num_key_value_heads * args.head_dim
    per_layer = args.hidden_size * (q_width + 2 * kv_width) + q_width * args.hidden_size + 3 * args.hidden_size * args.intermediate_size
    weights = args.num_hidden_layers * per_layer + args.vocab_size * args.hidden_size
    return weights * 17 // 32


# ---- Voluzen (latent attention + mixture of experts; voluzen.py) -------------------------------------------
def voluzen_config(*, width=128, vocab=256, pattern="WCSM", heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=32, window=24,
                   ff=96, experts=6, top=2, expert_ff=32, shared_ff=48, eps=1e-5, base=10000.0) -> dict:
    """A config.json for a stack spelled by ``pattern``, one letter a layer: ``W`` sliding-window latent attention
    with a dense feed-forward, ``w`` the same with experts, ``C`` causal latent attention with experts, ``c`` causal
    with a dense feed-forward, ``S`` causal reading the cache of the nearest caching causal layer before it (experts),
    ``M`` causal with experts and no shared expert, ``N`` causal with no feed-forward at all."""
    layers, last_causal = [], None
    for i, letter in enumerate(pattern):
        windowed = letter in "Ww"
        mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": float((dim + rot_dim) ** -0.5),
                 "rot": {"base": float(base) * (2 if windowed else 1), "dims": rot_dim}}
        if windowed:
            mixer["mask"] = {"size": window}
        if letter == "S":
            if last_causal is None:
                raise ValueError("'S' needs a caching causal layer before it")
            mixer["kv_from"] = last_causal
        elif not windowed:
            last_causal = i
        if letter in "Wc":
            mlp = {"kind": "dense", "ff": ff}
        elif letter == "N":
            mlp = None
        else:
            mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": expert_ff}}
            if letter != "M" and shared_ff:
                mlp["shared"] = {"ff": shared_ff}
        layers.append({"type": "latent_attention_2" if windowed else "latent_attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Voluzen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def synthetic_voluzen(config: dict, seed: int = 0, dtype=torch.bfloat16) -> dict:
    """Random tensors for ``config`` under the checkpoint's names (CPU, seeded)."""
    gen = torch.Generator().manual_seed(seed)
    D = config["width"]

    def mat(out_dim, in_dim, gain=1.0):
        return (torch.randn(out_dim, in_dim, generator=gen) * (gain / in_dim**0.5)).to(dtype)

    def vec(n, centre, spread):
        return (centre + spread * torch.randn(n, generator=gen)).to(dtype)

    tensors = {"embed": (torch.randn(config["vocab"], D, generator=gen)).to(dtype), "final.norm": vec(D, 0.0, 0.1), "head": mat(config["vocab"], D)}
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}."
        H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        tensors[p + "mix.q"] = mat(H * (dn + dr), D)
        if m.get("kv_from") is None:
            tensors[p + "mix.dkv"] = mat(R + dr, D, 2.0)
            tensors[p + "mix.dkv.norm"] = vec(R, 1.0, 0.1)
        tensors[p + "mix.uk"] = mat(H * dn, R)
        tensors[p + "mix.uv"] = mat(H * dv, R)
        tensors[p + "mix.o"] = mat(D, H * dv)
        tensors[p + "norm1"], tensors[p + "ls1"] = vec(D, 0.0, 0.1), vec(D, 0.7, 0.2)
        mlp = layer.get("mlp")
        if not mlp:
            continue
        tensors[p + "norm2"], tensors[p + "ls2"] = vec(D, 0.0, 0.1), vec(D, 0.7, 0.2)
        if mlp["kind"] == "dense":
            groups = [("mlp.", mlp["ff"])]
        else:
            tensors[p + "mlp.router"] = mat(mlp["router"]["experts"], D, 2.0)
            tensors[p + "mlp.router.b"] = vec(mlp["router"]["experts"], 0.0, 0.3)
            groups = [(f"mlp.e{k}.", mlp["expert"]["ff"]) for k in range(mlp["router"]["experts"])]
            if mlp.get("shared"):
                groups.append(("mlp.shared.", mlp["shared"]["ff"]))
        for q, ff in groups:
            tensors[p + q + "gate"], tensors[p + q + "up"], tensors[p + q + "down"] = mat(ff, D, 2.0), mat(ff, D), mat(D, ff)
    return tensors


def save_voluzen(config: dict, tensors: dict, path) -> None:
    """Write ``config.json`` + ``model.safetensors`` (a directory ``load_model`` reads)."""
    import json
    from pathlib import Path

    from safetensors.torch import save_file

    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(config, indent=1))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(path / "model.safetensors"))


# ---- Bapovik (windowed / chunked attention beside a recurrent mixer, experts; bapovik.py) ---------------------
def bapovik_config(*, width=96, vocab=200, pattern="APSP", heads=4, kv_heads=2, dim=16, vdim=24, window=20, chunk=28, softcap=30.0,
                   rec_heads=2, rec_dim=16, rec_vdim=32, tau=8.0, experts=6, top=2, expert_ff=40, eps=1e-5) -> dict:
    """A config.json for a stack spelled by ``pattern``, one letter a layer: ``A`` sliding-window attention with experts,
    ``a`` the same without a feed-forward, ``S`` window attention reading the keys and values of the nearest ``A`` / ``a``
    layer before it, ``P`` a parallel layer (chunked attention beside the recurrent mixer) with experts, ``p`` one
    without a feed-forward."""
    layers, last = [], None
    moe = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": expert_ff}}
    for i, letter in enumerate(pattern):
        if letter in "AaS":
            mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(dim ** -0.5), "mask": {"size": window}}
            if letter == "S":
                if last is None:
                    raise ValueError("'S' needs an attention layer with its own keys and values before it")
                mixer["kv_from"] = last
            else:
                last = i
            layers.append({"type": "attention", "mixer": mixer, "mlp": None if letter == "a" else moe})
        elif letter in "Pp":
            left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(dim ** -0.5), "mask": {"size": chunk}, "softcap": softcap}
            right = {"heads": rec_heads, "dim": rec_dim, "vdim": rec_vdim, "tau": tau}
            layers.append({"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": None if letter == "p" else moe})
        else:
            raise ValueError(f"unknown layer letter {letter!r}")
    return {"architecture": "Bapovik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def synthetic_bapovik(config: dict, seed: int = 0, dtype=torch.bfloat16) -> dict:
    """Random tensors for ``config`` under the checkpoint's names (CPU, seeded)."""
    gen = torch.Generator().manual_seed(seed)
    D = config["width"]

    def mat(out_dim, in_dim, gain=1.0):
        return (torch.randn(out_dim, in_dim, generator=gen) * (gain / in_dim**0.5)).to(dtype)

    def vec(n, centre, spread):
        return (centre + spread * torch.randn(n, generator=gen)).to(dtype)

    tensors = {"embed": torch.randn(config["vocab"], D, generator=gen).to(dtype), "final.norm": vec(D, 1.0, 0.1), "head": mat(config["vocab"], D)}

    def attention(p, m):
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        tensors[p + "q"], tensors[p + "q.b"] = mat(H * dk, D, 2.0), vec(H * dk, 0.0, 0.2)
        if m.get("kv_from") is None:
            tensors[p + "k"], tensors[p + "k.b"] = mat(G * dk, D, 2.0), vec(G * dk, 0.0, 0.2)
            tensors[p + "v"], tensors[p + "v.b"] = mat(G * dv, D), vec(G * dv, 0.0, 0.2)
        tensors[p + "g"], tensors[p + "o"] = mat(H, D, 2.0), mat(D, H * dv)

    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}."
        tensors[p + "norm1"] = vec(D, 1.0, 0.1)
        if layer["type"] == "attention":
            attention(p + "mix.", m)
        else:
            attention(p + "mix.left.", m["left"])
            dk = m["left"]["dim"]
            tensors[p + "mix.left.q.norm"], tensors[p + "mix.left.k.norm"] = vec(dk, 1.0, 0.2), vec(dk, 1.0, 0.2)
            r, rp = m["right"], p + "mix.right."
            H, dk, dv = r["heads"], r["dim"], r["vdim"]
            low = max(4, H * dk // 8)
            tensors[rp + "q"], tensors[rp + "k"], tensors[rp + "v"] = mat(H * dk, D, 2.0), mat(H * dk, D, 2.0), mat(H * dv, D)
            tensors[rp + "g"], tensors[rp + "o"], tensors[rp + "norm"] = mat(H * dv, D), mat(D, H * dv), vec(dv, 1.0, 0.2)
            tensors[rp + "a1"], tensors[rp + "a2"], tensors[rp + "a2.b"] = mat(low, D), mat(H * dk, low, 2.0), vec(H * dk, 2.0, 1.0)
            tensors[p + "mix.left.out"], tensors[p + "mix.right.out"] = vec(D, 1.0, 0.2), vec(D, 1.0, 0.2)
        mlp = layer.get("mlp")
        if mlp:
            tensors[p + "mlp.router"] = mat(mlp["router"]["experts"], D, 2.0)
            for k in range(mlp["router"]["experts"]):
                tensors[p + f"mlp.e{k}.up"], tensors[p + f"mlp.e{k}.down"] = mat(mlp["expert"]["ff"], D, 1.5), mat(D, mlp["expert"]["ff"])
    return tensors


save_bapovik = save_voluzen  # the same directory layout: config.json + model.safetensors


# ---- Senurax (retention / gated delta rule / softmax attention beside a delta rule, looped layers; senurax.py) -------
def senurax_config(*, width=96, vocab=200, pattern="CdPmRmCn", loop=(1, 3, 2), heads=4, kv_heads=2, dim=16, vdim=24, rot_dims=8, rot_base=10000.0,
                   rot_factor=2.0, scale=None, rec_heads=4, rec_key_heads=2, rec_dim=16, rec_vdim=32, taps=4, ret_heads=2, ret_dim=16, ret_vdim=32,
                   ret_rot_dims=16, decay=None, ff=160, experts=6, identity=2, top=2, expert_ff=40, router_scale=1.5, softcap=20.0, eps=1e-5) -> dict:
    """A config.json for a stack spelled by ``pattern``, two letters a layer: the mixer (``R`` retention, ``C`` gated delta
    rule with per-channel decay, ``P`` softmax attention beside a gated delta rule) and the feed-forward (``d`` dense,
    ``m`` experts, ``n`` none).  ``loop`` = (start, stop, times) or None."""
    if len(pattern) % 2:
        raise ValueError("the pattern is pairs of letters: mixer, feed-forward")
    layers = []
    for mixer_letter, ff_letter in zip(pattern[0::2], pattern[1::2]):
        if ff_letter == "d":
            mlp = {"kind": "dense", "ff": ff}
        elif ff_letter == "m":
            mlp = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": router_scale}}
        elif ff_letter == "n":
            mlp = None
        else:
            raise ValueError(f"unknown feed-forward letter {ff_letter!r}")
        delta = {"conv": taps, "dim": rec_dim, "heads": rec_heads, "kv_heads": rec_key_heads, "vdim": rec_vdim}
        if mixer_letter == "R":
            d = list(decay) if decay is not None else [1.0 - 2.0 ** (-3 - 1.5 * h) for h in range(ret_heads)]
            mixer = {"heads": ret_heads, "dim": ret_dim, "vdim": ret_vdim, "decay": d}
            if ret_rot_dims:
                mixer["rot"] = {"base": rot_base, "dims": ret_rot_dims}
            layers.append({"type": "retention", "mixer": mixer, "mlp": mlp})
        elif mixer_letter == "C":
            layers.append({"type": "channel_delta", "mixer": delta, "mlp": mlp})
        elif mixer_letter == "P":
            left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale if scale is not None else dim ** -0.5)}
            if rot_dims:
                left["rot"] = {"base": rot_base, "dims": rot_dims}
                if rot_factor and rot_factor != 1.0:
                    left["rot"]["scaling"] = {"factor": rot_factor}
            layers.append({"type": "parallel", "mixer": {"left": left, "right": delta}, "mlp": mlp})
        else:
            raise ValueError(f"unknown mixer letter {mixer_letter!r}")
    config = {"architecture": "Senurax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if softcap:
        config["logit_softcap"] = softcap
    if loop:
        config["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return config


def synthetic_senurax(config: dict, seed: int = 0, dtype=torch.bfloat16) -> dict:
    """Random tensors for ``config`` under the checkpoint's names (CPU, seeded)."""
    gen = torch.Generator().manual_seed(seed)
    D = config["width"]

    def mat(out_dim, in_dim, gain=1.0):
        return (torch.randn(out_dim, in_dim, generator=gen) * (gain / in_dim**0.5)).to(dtype)

    def vec(n, centre, spread):
        return (centre + spread * torch.randn(n, generator=gen)).to(dtype)

    tensors = {"embed": torch.randn(config["vocab"], D, generator=gen).to(dtype), "final.norm": vec(D, 1.0, 0.1), "head": mat(config["vocab"], D)}
    if config.get("loop"):
        times = config["loop"]["times"]
        tensors["loop.in"] = torch.cat([mat(D, D), mat(D, D, 0.5)], dim=1).contiguous()
        tensors["loop.step"] = (0.3 * torch.randn(times, D, generator=gen)).to(dtype)

    def delta(p, m, channel):
        H, G, dk, dv, K = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"], m["conv"]
        for name, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
            tensors[p + name] = mat(rows, D, 2.0)
            tensors[p + name + ".conv"] = (torch.randn(rows, K, generator=gen) * 0.5 + torch.eye(K)[K - 1]).to(dtype)
        tensors[p + "b"], tensors[p + "A_log"], tensors[p + "norm"], tensors[p + "o"] = mat(H, D, 2.0), vec(H, -1.0, 1.0), vec(dv, 1.0, 0.2), mat(D, H * dv)
        if channel:
            low = max(4, D // 12)
            tensors[p + "a1"], tensors[p + "a2"], tensors[p + "dt_bias"] = mat(low, D), mat(H * dk, low, 2.0), vec(H * dk, -1.0, 1.0)
            tensors[p + "g1"], tensors[p + "g2"] = mat(low, D), mat(H * dv, low, 2.0)
        else:
            tensors[p + "a"], tensors[p + "dt_bias"], tensors[p + "g"] = mat(H, D, 2.0), vec(H, -1.0, 1.0), mat(H * dv, D)

    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}."
        tensors[p + "norm1"] = vec(D, 1.0, 0.1)
        if layer["type"] == "retention":
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            tensors[p + "mix.q"], tensors[p + "mix.k"], tensors[p + "mix.v"] = mat(H * dk, D, 2.0), mat(H * dk, D, 2.0), mat(H * dv, D)
            tensors[p + "mix.g"], tensors[p + "mix.o"] = mat(H * dv, D), mat(D, H * dv)
        elif layer["type"] == "channel_delta":
            delta(p + "mix.", m, True)
        else:
            a = m["left"]
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            lp = p + "mix.left."
            tensors[lp + "q"], tensors[lp + "k"], tensors[lp + "v"], tensors[lp + "o"] = mat(H * dk, D, 2.0), mat(G * dk, D, 2.0), mat(G * dv, D), mat(D, H * dv)
            delta(p + "mix.right.", m["right"], False)
            tensors[lp + "out"], tensors[p + "mix.right.out"] = vec(D, 1.0, 0.2), vec(D, 1.0, 0.2)
        mlp = layer.get("mlp")
        if not mlp:
            continue
        tensors[p + "norm2"] = vec(D, 1.0, 0.1)
        if mlp["kind"] == "dense":
            tensors[p + "mlp.up"], tensors[p + "mlp.down"] = mat(mlp["ff"], D, 1.5), mat(D, mlp["ff"])
        else:
            r = mlp["router"]
            outputs = r["experts"] + r.get("identity", 0)
            tensors[p + "mlp.router"], tensors[p + "mlp.correction"] = mat(outputs, D, 2.0), vec(outputs, 0.0, 0.05)
            for k in range(r["experts"]):
                q = p + f"mlp.e{k}."
                tensors[q + "gate"], tensors[q + "up"], tensors[q + "down"] = mat(mlp["expert"]["ff"], D, 2.0), mat(mlp["expert"]["ff"], D), mat(D, mlp["expert"]["ff"])
    return tensors


save_senurax = save_voluzen


# ---- Norusun (time-mix linear attention / latent attention with sinks / sigmoid attention beside a state-space mixer; norusun.py) ----
def norusun_config(*, width=96, vocab=200, pattern="LdPdWnLd", streams=2, canon_taps=4, heads=4, kv_heads=2, dim=16, vdim=24, chunk=24, rot_dims=16,
                   rot_base=20000.0, scale=None, lat_heads=3, lat_dim=16, lat_rot=8, lat_vdim=16, kv_rank=24, q_rank=40, window=20, lat_base=10000.0,
                   lat_scale=None, ss_heads=4, ss_vdim=16, ss_state=16, ss_groups=2, ss_norm_groups=2, ss_taps=4, wkv_heads=3, wkv_dim=32, ff=160,
                   limit=3.0, eps=1e-6) -> dict:
    """A config.json for a stack spelled by ``pattern``, two letters a layer: the mixer (``W`` time-mix linear attention,
    ``L`` latent attention, ``P`` chunked sigmoid attention beside a state-space mixer) and the feed-forward (``d`` dense,
    ``n`` none).  ``streams`` 0 = no residual streams, ``canon_taps`` 0 = no input convolution."""
    if len(pattern) % 2:
        raise ValueError("the pattern is pairs of letters: mixer, feed-forward")
    layers = []
    for mixer_letter, ff_letter in zip(pattern[0::2], pattern[1::2]):
        if ff_letter not in "dn":
            raise ValueError(f"unknown feed-forward letter {ff_letter!r}")
        mlp = {"kind": "dense", "ff": ff, "limit": limit} if ff_letter == "d" else None
        if mixer_letter == "W":
            layers.append({"type": "wkv", "mixer": {"heads": wkv_heads, "dim": wkv_dim}, "mlp": mlp})
        elif mixer_letter == "L":
            mixer = {"heads": lat_heads, "dim": lat_dim, "rot_dim": lat_rot, "vdim": lat_vdim, "kv_rank": kv_rank, "q_rank": q_rank, "mask": {"size": window},
                     "rot": {"base": lat_base, "dims": lat_rot}, "scale": float(lat_scale if lat_scale is not None else (lat_dim + lat_rot) ** -0.5)}
            layers.append({"type": "latent_attention", "mixer": mixer, "mlp": mlp})
        elif mixer_letter == "P":
            left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk}, "rot": {"base": rot_base, "dims": rot_dims},
                    "scale": float(scale if scale is not None else dim ** -0.5)}
            right = {"conv": ss_taps, "groups": ss_groups, "heads": ss_heads, "norm_groups": ss_norm_groups, "state": ss_state, "vdim": ss_vdim}
            layers.append({"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp})
        else:
            raise ValueError(f"unknown mixer letter {mixer_letter!r}")
    config = {"architecture": "Norusun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams:
        config["streams"] = streams
    if canon_taps:
        config["canon"] = {"taps": canon_taps}
    return config


def synthetic_norusun(config: dict, seed: int = 0, dtype=torch.bfloat16) -> dict:
    """Random tensors for ``config`` under the checkpoint's names (CPU, seeded)."""
    gen = torch.Generator().manual_seed(seed)
    D = config["width"]
    n = int(config.get("streams") or 0)
    taps = int((config.get("canon") or {}).get("taps") or 0)

    def mat(out_dim, in_dim, gain=1.0):
        return (torch.randn(out_dim, in_dim, generator=gen) * (gain / in_dim**0.5)).to(dtype)

    def vec(count, centre, spread):
        return (centre + spread * torch.randn(count, generator=gen)).to(dtype)

    def scalar(centre, spread):
        return vec(1, centre, spread).reshape(())

    tensors = {"embed": torch.randn(config["vocab"], D, generator=gen).to(dtype), "final.norm": scalar(1.0, 0.1), "head": mat(config["vocab"], D)}

    def sublayer(p, q):
        tensors[p + f"norm{q}"] = scalar(1.0, 0.1)
        if n:
            tensors[p + f"hc{q}.in"], tensors[p + f"hc{q}.out"] = vec(n, 1.0 / n, 0.2), vec(n, 1.0, 0.3)
            tensors[p + f"hc{q}.mix"] = (torch.eye(n) + 0.2 * torch.randn(n, n, generator=gen)).to(dtype)

    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}."
        sublayer(p, 1)
        if taps:
            tensors[p + "canon1"] = (0.3 * torch.randn(D, taps, generator=gen)).to(dtype)
        x = p + "mix."
        if layer["type"] == "wkv":
            hd = m["heads"] * m["dim"]
            low = max(4, D // 16)
            for name in "rkvgw":
                tensors[x + "mu." + name] = torch.rand(D, generator=gen).to(dtype)
            tensors[x + "r"], tensors[x + "k"], tensors[x + "v"], tensors[x + "g"] = mat(hd, D), mat(hd, D), mat(hd, D), mat(hd, D)
            tensors[x + "w1"], tensors[x + "w2"], tensors[x + "w0"] = mat(low, D), mat(hd, low, 2.0), vec(hd, -1.5, 1.0)
            tensors[x + "u"] = (0.5 * torch.randn(m["heads"], m["dim"], generator=gen)).to(dtype)
            tensors[x + "norm"], tensors[x + "o"] = vec(hd, 1.0, 0.2), mat(D, hd)
        elif layer["type"] == "latent_attention":
            H, dn, dr, dv, rank, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            tensors[x + "dq"], tensors[x + "dq.norm"], tensors[x + "uq"] = mat(qr, D), vec(qr, 1.0, 0.2), mat(H * (dn + dr), qr, 2.0)
            tensors[x + "dkv"], tensors[x + "dkv.norm"] = mat(rank + dr, D, 2.0), vec(rank, 1.0, 0.2)
            tensors[x + "uk"], tensors[x + "uv"], tensors[x + "o"] = mat(H * dn, rank, 2.0), mat(H * dv, rank), mat(D, H * dv)
            tensors[x + "sink"] = vec(H, 0.0, 1.0)
        else:
            a, r, lp, rp = m["left"], m["right"], x + "left.", x + "right."
            H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            tensors[lp + "q"], tensors[lp + "k"], tensors[lp + "v"], tensors[lp + "o"] = mat(H * dk, D, 2.0), mat(G * dk, D, 2.0), mat(G * dv, D), mat(D, H * dv)
            tensors[lp + "q.norm"], tensors[lp + "k.norm"], tensors[lp + "pb"] = vec(H * dk, 1.0, 0.2), vec(G * dk, 1.0, 0.2), vec(H, -2.0, 1.0)
            SH, P, N, SG, K = r["heads"], r["vdim"], r["state"], r["groups"], r["conv"]
            inner, channels = SH * P, SH * P + 2 * SG * N
            tensors[rp + "in"] = mat(2 * inner + 2 * SG * N + SH, D, 1.5)
            tensors[rp + "conv"] = (torch.randn(channels, K, generator=gen) * 0.4 + torch.eye(K)[K - 1]).to(dtype)
            tensors[rp + "conv.b"] = vec(channels, 0.0, 0.1)
            tensors[rp + "dt_bias"], tensors[rp + "A_log"], tensors[rp + "D"] = vec(SH, -1.0, 1.0), vec(SH, -0.5, 0.7), vec(SH, 1.0, 0.3)
            tensors[rp + "norm"], tensors[rp + "o"] = vec(inner, 1.0, 0.2), mat(D, inner)
            tensors[lp + "out"], tensors[rp + "out"] = vec(D, 1.0, 0.2), vec(D, 1.0, 0.2)
        mlp = layer.get("mlp")
        if mlp:
            sublayer(p, 2)
            f = mlp["ff"]
            tensors[p + "mlp.gate"], tensors[p + "mlp.gate.b"] = mat(f, D, 2.0), vec(f, 0.0, 0.5)
            tensors[p + "mlp.up"], tensors[p + "mlp.up.b"] = mat(f, D, 2.0), vec(f, 0.0, 0.5)
            tensors[p + "mlp.down"], tensors[p + "mlp.down.b"] = mat(D, f), vec(D, 0.0, 0.2)
    return tensors


save_norusun = save_voluzen
