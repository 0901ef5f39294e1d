"""Command line in the manner of sdcb/HyMT2Sharp's HyMT2Sharp.Cli
(src/HyMT2Sharp.Cli/Program.cs:7-28, 41-76): the same option names with the same
meanings where this library has the thing they name.  There is no text layer here,
so prompts are token ids ("12,7,99" or "12 7 99") and replies are printed as ids.

  --model DIR        model folder (config.json + model.safetensors)
  --prompt IDS       one turn, then exit; may be given several times (one batch).
                     Without it: a prompt loop on standard input with /reset /exit /help
  --system IDS       ids that stand before the first prompt of a conversation
  --max-tokens N     limit of decode steps per reply, default 256; as in Program.cs:99
                     the first token comes from the prompt, so a reply has at most N+1 tokens
  --threads N        CPU workers of the reference; accepted, has no meaning on the GPU
  --backend NAME     auto or cuda (cpu, metal and vulkan do not exist here)
  --profile          per-kernel times of the prefill and of the decode steps (the Benchmark program's switch,
                     src/HyMT2Sharp.Benchmark/Program.cs:243-261); kernels then run one after the other
and beyond the reference: --dtype, --temperature, --top-k, --top-p, --min-p,
--repeat-penalty, --penalty-window, --seed, --stop-ids, --max-context, --max-batch,
--random CONFIG.json --weights-seed N --sigma S (write random weights into --model first).
"""
from __future__ import annotations

import argparse
import json
import re
import sys
import time


def parse_ids(text: str) -> list:
    parts = [p for p in re.split(r"[,\s]+", text.strip()) if p]
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit(f"token ids must be integers separated by commas or spaces, got: {text!r}")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="hymt2sharp_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True)
    ap.add_argument("--prompt", action="append")
    ap.add_argument("--system")
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--threads", type=int, default=0)
    ap.add_argument("--backend", default="auto")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--repeat-penalty", type=float, default=1.0)
    ap.add_argument("--penalty-window", type=int, default=64)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--stop-ids", default="")
    ap.add_argument("--max-context", type=int, default=8192, help="tokens that the cache holds")
    ap.add_argument("--max-batch", type=int, default=8)
    ap.add_argument("--random", metavar="CONFIG.json", help="write random weights for this config into --model")
    ap.add_argument("--weights-seed", type=int, default=0)
    ap.add_argument("--sigma", type=float, default=0.02)
    ap.add_argument("--profile", action="store_true")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.backend not in ("auto", "cuda"):
        print(f"backend {args.backend} unavailable (this library runs on CUDA sm_100a only)", file=sys.stderr)
        return 2
    from .sampling.params import SamplingParams

    if args.random:
        from .config.registry import get_architecture
        from .config.base import architecture_name, read_config_json
        from .weights.random_init import write_random_model
        data = read_config_json(args.random)
        cfg = get_architecture(architecture_name(data, args.random)).config_class.from_dict(data, args.random)
        write_random_model(args.model, cfg, args.weights_seed, args.sigma)
        print(f"wrote random weights (seed {args.weights_seed}, sigma {args.sigma}) to {args.model}")

    from .engine.engine import Engine, StepEntry
    print(f"HyMT2Sharp-B200  model={args.model}")
    print(f"threads={'auto' if args.threads <= 0 else args.threads} (unused)  backend=cuda  dtype={args.dtype}")
    t0 = time.perf_counter()
    engine = Engine(args.model, dtype=args.dtype, max_tokens=args.max_context, max_batch=args.max_batch)
    c = engine.config
    print(f"arch={c.architecture} layers={c.num_hidden_layers} hidden={c.hidden_size} "
          f"heads={c.num_attention_heads}/{c.num_key_value_heads} vocab={c.vocab_size}  "
          f"(loaded in {time.perf_counter() - t0:.1f} s)")
    sampling = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p,
                              repeat_penalty=args.repeat_penalty, penalty_window=args.penalty_window, seed=args.seed)
    stop = parse_ids(args.stop_ids) if args.stop_ids else []
    system = parse_ids(args.system) if args.system else []
    max_new = args.max_tokens + 1

    if args.prompt:
        prompts = [system + parse_ids(p) for p in args.prompt]
        out = engine.generate(prompts, max_new_tokens=max_new, sampling=sampling, stop_token_ids=stop,
                              max_batch=args.max_batch, profile=args.profile)
        for i, r in enumerate(out.results):
            label = "Assistant" if len(prompts) == 1 else f"Assistant[{i}]"
            print(f"{label}: {','.join(map(str, r.tokens))}  ({r.finish_reason})")
        print(out.stats.line())
        _print_profile(out.stats)
        return 0

    # prompt loop: each line goes on from the conversation so far (the whole conversation is run again as the
    # next prompt: nothing of a turn's cache is kept once its reply is complete)
    interactive = sys.stdin.isatty()
    if interactive:
        print("\nType token ids.  /reset  /exit")
    history: list = []
    while True:
        if interactive:
            print("\nYou: ", end="", flush=True)
        line = sys.stdin.readline()
        if not line:
            break
        line = line.strip()
        if not line:
            continue
        if line in ("/exit", "/quit"):
            break
        if line in ("/reset", "/clear"):
            history = []
            print("reset")
            continue
        if line == "/help":
            print("/reset  clear conversation\n/exit   quit")
            continue
        turn = (system if not history else []) + parse_ids(line)
        out = engine.generate([history + turn], max_new_tokens=max_new, sampling=sampling, stop_token_ids=stop,
                              profile=args.profile)
        r = out.results[0]
        history = history + turn + r.tokens
        print(f"Assistant: {','.join(map(str, r.tokens))}  ({r.finish_reason})")
        print(out.stats.line())
        _print_profile(out.stats)
    return 0


def _print_profile(stats) -> None:
    from .kernels.ops import profile_line
    for phase, times in stats.profile.items():
        print(profile_line(phase, times))


if __name__ == "__main__":
    sys.exit(main())
