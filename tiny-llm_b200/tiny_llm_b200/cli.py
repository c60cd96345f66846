"""Command-line front doors: the equivalents of the reference's ``main.py`` (one prompt,
``/root/reference/main.py:1-190``) and ``batch-main.py`` (continuous batching,
``/root/reference/batch-main.py:1-102``) over a checkpoint DIRECTORY (MLX 4-bit safetensors layout,
see checkpoint.py; there is no hub download here).

    python -m tiny_llm_b200.cli generate --model /path/to/Qwen3-4B-MLX-4bit --prompt "..." [--loader week3]
    python -m tiny_llm_b200.cli batch    --model /path/to/ckpt --prompts-file prompts.txt --batch-size 5
    python -m tiny_llm_b200.cli generate --synthetic tiny-d128 --prompt-ids 5,17,3 --max-new-tokens 8   (no files needed)
    python -m tiny_llm_b200.cli generate --synthetic voluzen:WCSM --prompt-ids 5,17,3 --max-new-tokens 8
    python -m tiny_llm_b200.cli generate --synthetic bapovik:APSP --prompt-ids 5,17,3 --max-new-tokens 8
    python -m tiny_llm_b200.cli generate --synthetic senurax:RdCmPm --prompt-ids 5,17,3 --max-new-tokens 8
    python -m tiny_llm_b200.cli generate --synthetic norusun:LdPdWn --prompt-ids 5,17,3 --max-new-tokens 8
    python -m tiny_llm_b200.cli trace    --model DIR --dtype float32 --out DIR --max-tokens N < steps.jsonl   (trace_runner.py)

A checkpoint whose config.json names its ``architecture`` (Voluzen, Bapovik, Senurax, Norusun) is built by that design's class
(``models.load_model``); such models take ``--dtype`` and batch with mixed prefill + decode steps.
"""

from __future__ import annotations

import argparse
import sys

import torch


def _self_describing(args, device):
    """The model object when --model / --synthetic name a design that config.json describes, else None."""
    import json
    from pathlib import Path

    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype]
    if args.synthetic and args.synthetic.startswith("voluzen"):
        from .models import model_class
        from .synthetic import synthetic_voluzen, voluzen_config

        config = voluzen_config(pattern=args.synthetic.partition(":")[2] or "WCSM")
        return model_class("Voluzen").from_checkpoint(config, synthetic_voluzen(config, seed=0), device=device, dtype=dtype)
    if args.synthetic and args.synthetic.startswith("bapovik"):
        from .models import model_class
        from .synthetic import bapovik_config, synthetic_bapovik

        config = bapovik_config(pattern=args.synthetic.partition(":")[2] or "APSP")
        return model_class("Bapovik").from_checkpoint(config, synthetic_bapovik(config, seed=0), device=device, dtype=dtype)
    if args.synthetic and args.synthetic.startswith("senurax"):
        from .models import model_class
        from .synthetic import senurax_config, synthetic_senurax

        pattern = args.synthetic.partition(":")[2] or "CdPmRmCn"
        count = len(pattern) // 2
        config = senurax_config(pattern=pattern, loop=(min(1, count - 1), count, 2))  # all layers but the first run twice
        return model_class("Senurax").from_checkpoint(config, synthetic_senurax(config, seed=0), device=device, dtype=dtype)
    if args.synthetic and args.synthetic.startswith("norusun"):
        from .models import model_class
        from .synthetic import norusun_config, synthetic_norusun

        config = norusun_config(pattern=args.synthetic.partition(":")[2] or "LdPdWnLd")
        return model_class("Norusun").from_checkpoint(config, synthetic_norusun(config, seed=0), device=device, dtype=dtype)
    if args.model and "architecture" in json.loads((Path(args.model) / "config.json").read_text()):
        from .models import load_model

        return load_model(args.model, device=device, dtype=dtype)
    return None


def _load(args, device):
    from .checkpoint import load_checkpoint, load_tokenizer
    from .synthetic import synthetic_qwen3

    model = _self_describing(args, device)
    if model is not None:
        tokenizer = None
        if args.model:
            try:
                tokenizer = load_tokenizer(args.model)
            except Exception as exc:
                print(f"(no tokenizer loaded from {args.model}: {exc})", file=sys.stderr)
        return model, tokenizer, None
    if args.synthetic:
        return synthetic_qwen3(args.synthetic, seed=0, device=device, realistic=args.synthetic.startswith("tiny")), None, "Qwen/Qwen3-synthetic"
    ns = load_checkpoint(args.model, device=device)
    tokenizer = None
    try:
        tokenizer = load_tokenizer(args.model)
    except Exception as exc:  # token-id mode still works without tokenizer files
        print(f"(no tokenizer loaded from {args.model}: {exc})", file=sys.stderr)
    return ns, tokenizer, "Qwen/Qwen3-" + str(args.model)


def _model(args, ns, name):
    from .models import dispatch_model

    if name is None:  # already a model object
        return ns
    if args.loader == "week2":
        return dispatch_model(name, ns, week=2)
    return dispatch_model(name, ns, week=3, enable_paged_attention=not args.disable_paged_attention)


def _prompt_ids(args, tokenizer, prompt: str | None):
    if args.prompt_ids:
        return [int(t) for t in args.prompt_ids.split(",")]
    if tokenizer is None:
        raise SystemExit("a text prompt needs the checkpoint's tokenizer files; use --prompt-ids")
    messages = [{"role": "system", "content": "You are a helpful assistant."}, {"role": "user", "content": prompt}]
    text = tokenizer.apply_chat_template(messages, tokenize=False, add_generation_prompt=True, enable_thinking=args.enable_thinking)
    return tokenizer.encode(text, add_special_tokens=False)


def cmd_generate(args) -> int:
    from .generate import greedy_generate_ids
    from .sampler import make_sampler

    device = torch.device(args.device)
    ns, tokenizer, name = _load(args, device)
    model = _model(args, ns, name)
    ids = _prompt_ids(args, tokenizer, args.prompt)
    sampler = None if args.sampler_temp == 0 else make_sampler(args.sampler_temp, top_p=args.sampler_top_p, top_k=args.sampler_top_k)
    if tokenizer is not None:
        tokenizer.detokenizer.reset()

    def emit(token: int) -> None:
        if tokenizer is None:
            print(token, end=" ", flush=True)
        else:
            tokenizer.detokenizer.add_token(token)
            print(tokenizer.detokenizer.last_segment, end="", flush=True)

    produced = greedy_generate_ids(model, ids, args.max_new_tokens, eos_token_id=getattr(tokenizer, "eos_token_id", None), device=device,
                                   on_token=emit, sampler=sampler)
    print()
    return 0 if produced is not None else 1


def cmd_batch(args) -> int:
    from .batch import batch_generate

    device = torch.device(args.device)
    ns, tokenizer, name = _load(args, device)
    model = _model(args, ns, name)
    if args.prompts_file:
        prompts = [line.strip() for line in open(args.prompts_file) if line.strip()]
    else:
        prompts = [args.prompt or "Give me a short introduction to large language models."]
    if args.prompt_ids or tokenizer is None:
        queue = [[int(t) for t in p.split(",")] for p in (args.prompt_ids.split(";") if args.prompt_ids else prompts)]
    else:
        queue = [tokenizer.apply_chat_template([{"role": "user", "content": p}], tokenize=False, add_generation_prompt=True,
                                               enable_thinking=args.enable_thinking) for p in prompts]
    results = batch_generate(model, tokenizer, queue, max_seq_len=args.max_seq_len, batch_size=args.batch_size, prefill_step=args.prefill_step,
                             verbose=not args.quiet, device=device, max_new_tokens=[args.max_new_tokens] * len(queue) if args.max_new_tokens else None)
    for idx, text in sorted(results):
        print(f"--- request {idx}\n{text}")
    return 0


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else list(argv)
    if argv and argv[0] == "trace":
        from .trace_runner import main as trace_main

        return trace_main(argv[1:])
    ap = argparse.ArgumentParser(prog="tiny_llm_b200.cli")
    sub = ap.add_subparsers(dest="command", required=True)
    for name, fn in (("generate", cmd_generate), ("batch", cmd_batch)):
        p = sub.add_parser(name)
        p.set_defaults(fn=fn)
        p.add_argument("--model", default=None, help="checkpoint directory (config.json + *.safetensors [+ tokenizer files])")
        p.add_argument("--synthetic", default=None, help="random weights of a named shape (tiny, tiny-d128, qwen3-0.6b, qwen3-4b, voluzen[:LAYERS], bapovik[:LAYERS], senurax[:LAYERS], norusun[:LAYERS]) instead of --model")
        p.add_argument("--prompt", default="Give me a short introduction to large language models.")
        p.add_argument("--prompt-ids", default=None, help="comma-separated token ids (';' between requests for `batch`)")
        p.add_argument("--loader", choices=["week2", "week3"], default="week3")
        p.add_argument("--device", default="cuda:0")
        p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16", help="compute dtype of designs with unquantised weights")
        p.add_argument("--disable-paged-attention", action="store_true")
        p.add_argument("--enable-thinking", action="store_true")
        p.add_argument("--max-new-tokens", type=int, default=128)
    sub.choices["generate"].add_argument("--sampler-temp", type=float, default=0.0)
    sub.choices["generate"].add_argument("--sampler-top-p", type=float, default=None)
    sub.choices["generate"].add_argument("--sampler-top-k", type=int, default=None)
    sub.choices["batch"].add_argument("--prompts-file", default=None)
    sub.choices["batch"].add_argument("--batch-size", type=int, default=5)
    sub.choices["batch"].add_argument("--prefill-step", type=int, default=128)
    sub.choices["batch"].add_argument("--max-seq-len", type=int, default=512)
    sub.choices["batch"].add_argument("--quiet", action="store_true")
    args = ap.parse_args(argv)
    if not args.model and not args.synthetic:
        ap.error("--model or --synthetic is required")
    return args.fn(args)


if __name__ == "__main__":
    raise SystemExit(main())
