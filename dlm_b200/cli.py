"""Command line in the manner of ``dlm generate`` (src/cli.rs:355-415, src/main.rs:249-332):
the same option names with the same meanings and defaults, the same output lines
(``prompt ids   :``, ``generated ids:``).  Options the reference does not have are listed
after its own.  There is no tokenizer: prompts are token ids.

Where the model comes from, in this order: ``--model-path DIR`` (a folder with config.json and
safetensors); ``--random CONFIG.json`` (random weights from ``--seed`` for the architecture and
sizes that config file names, whichever registered architecture that is); else the reference's
demo geometry options.  ``--save-random DIR`` writes the random model as a folder (config.json,
model.safetensors) and generates from that folder.
"""
from __future__ import annotations

import argparse
import sys


def _ids(text: str) -> list[int]:
    try:
        return [int(t) for t in text.split(",") if t.strip() != ""]
    except ValueError as e:
        raise argparse.ArgumentTypeError(f"a prompt is comma-separated token ids: {e}")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="dlm-b200", description="Qwen2-MoE inference on one B200")
    sub = ap.add_subparsers(dest="command", required=True)
    g = sub.add_parser("generate", help="generate token ids from a prompt of token ids")
    # the reference's options
    g.add_argument("--prompt", type=_ids, action="append", default=None,
                   help="prompt as comma-separated token ids (default 1); repeat for several requests")
    g.add_argument("--model-path", metavar="DIR", help="folder with config.json and safetensors; when set, "
                   "the synthetic-model geometry options are ignored")
    g.add_argument("--max-new-tokens", type=int, default=16, help="number of new tokens to generate")
    g.add_argument("--eos-token", type=int, default=None, help="stop when this token id is produced")
    g.add_argument("--vocab-size", type=int, default=32)
    g.add_argument("--hidden-size", type=int, default=64)
    g.add_argument("--num-layers", type=int, default=2)
    g.add_argument("--num-heads", type=int, default=4)
    g.add_argument("--num-kv-heads", type=int, default=2)
    g.add_argument("--intermediate-size", type=int, default=128)
    g.add_argument("--seed", type=int, default=0, help="seed of the synthetic weights")
    g.add_argument("--random", metavar="CONFIG.json", default=None,
                   help="random weights for the architecture and sizes of this config.json (or of the folder "
                        "that holds one); the geometry options are then ignored")
    g.add_argument("--save-random", metavar="DIR", default=None,
                   help="write the random model (config.json, model.safetensors) there and generate from it")
    g.add_argument("--device", choices=["gpu", "cpu"], default="gpu",
                   help="compute device; only gpu exists here (cpu is refused)")
    # synthetic mixture-of-experts geometry (no counterpart in the reference's demo model)
    g.add_argument("--num-experts", type=int, default=8)
    g.add_argument("--num-experts-per-tok", type=int, default=2)
    g.add_argument("--moe-intermediate-size", type=int, default=32)
    g.add_argument("--shared-expert-intermediate-size", type=int, default=64)
    # sampling (the reference's server options, src/generate.rs:61-81)
    g.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--min-p", type=float, default=0.0)
    g.add_argument("--repetition-penalty", type=float, default=1.0)
    g.add_argument("--sample-seed", type=int, default=0)
    # engine
    g.add_argument("--dtype", choices=["bfloat16", "float32", "bf16", "fp32"], default="bfloat16")
    g.add_argument("--page-size", type=int, default=64)
    g.add_argument("--num-pages", type=int, default=None)
    g.add_argument("--max-step-tokens", type=int, default=2048)
    g.add_argument("--max-requests", type=int, default=64)
    g.add_argument("--stats", action="store_true", help="print scheduler and cache statistics")
    return ap


def demo_config(args) -> dict:
    """The config.json of the demo model the geometry options describe (the reference's demo is a
    dense model, src/main.rs:404-470; here it has experts too, since that is what this engine is for)."""
    from .registry import architectures
    return dict(architectures=[architectures()[0]], vocab_size=args.vocab_size, hidden_size=args.hidden_size,
                num_hidden_layers=args.num_layers, num_attention_heads=args.num_heads,
                num_key_value_heads=args.num_kv_heads, intermediate_size=args.intermediate_size,
                num_experts=args.num_experts, num_experts_per_tok=args.num_experts_per_tok,
                moe_intermediate_size=args.moe_intermediate_size,
                shared_expert_intermediate_size=args.shared_expert_intermediate_size, norm_topk_prob=False)


def run_generate(args) -> int:
    from . import __version__
    print(f"dlm-b200 v{__version__}")
    print("  gpu backend  : CUDA (sm_100a)")
    print()
    if args.device == "cpu":
        print("error: this engine has no CPU path; use --device gpu", file=sys.stderr)
        return 2
    prompts = args.prompt if args.prompt else [[1]]
    if any(len(p) == 0 for p in prompts):
        print("error: prompt is empty", file=sys.stderr)
        return 2
    from .engine import Engine
    need = max(len(p) for p in prompts) + args.max_new_tokens
    kw = dict(dtype=args.dtype, page_size=args.page_size, max_step_tokens=args.max_step_tokens,
              max_requests=max(1, min(args.max_requests, max(len(prompts), 1))), max_context=max(need, args.page_size))
    if args.num_pages is not None:
        kw["num_pages"] = args.num_pages
    else:
        kw["max_tokens"] = sum(-(-(len(p) + args.max_new_tokens) // args.page_size) * args.page_size for p in prompts)
    if args.model_path:
        eng = Engine.from_pretrained(args.model_path, **kw)
        print(f"generate     : model {args.model_path}")
    else:
        from .registry import resolve
        if args.random:
            _, cfg, _ = resolve(args.random)
            what = f"random weights for {args.random} (seed {args.seed})"
        else:
            _, cfg, _ = resolve(demo_config(args))
            what = f"demo with randomly-initialized weights (seed {args.seed})"
        if args.save_random:
            from .weights import write_random_model
            write_random_model(cfg, args.seed, args.save_random)
            eng = Engine.from_pretrained(args.save_random, **kw)
            what += f", written to {args.save_random}"
        else:
            eng = Engine.from_random(cfg, args.seed, **kw)
        print(f"generate     : {what}")
    c, spec = eng.config, eng.model.spec
    line = f"model        : vocab {spec.vocab_size}, hidden {spec.hidden_size}, {len(spec.layers)} layers"
    if all(hasattr(c, k) for k in ("num_attention_heads", "num_key_value_heads", "head_dim")):
        line += f", {c.num_attention_heads} q-heads / {c.num_key_value_heads} kv-heads, head_dim {c.head_dim}"
    print(line)
    for p in prompts:
        bad = [t for t in p if t < 0 or t >= spec.vocab_size]
        if bad:
            print(f"error: prompt token {max(bad)} out of vocab range {spec.vocab_size}", file=sys.stderr)
            return 2
    print("device       : Gpu")
    outs = eng.generate(prompts, max_new_tokens=args.max_new_tokens, eos_token=args.eos_token,
                        temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, min_p=args.min_p,
                        repetition_penalty=args.repetition_penalty, seed=args.sample_seed)
    for p, o in zip(prompts, outs):
        print(f"prompt ids   : {p}")
        print(f"generated ids: {o}")
    if args.stats:
        print(f"stats        : {eng.stats()}")
    if not args.model_path:
        print()
        print("note         : weights are untrained random values — output is not")
        print("               meaningful text.")
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.command == "generate":
        return run_generate(args)
    return 2


if __name__ == "__main__":
    sys.exit(main())
