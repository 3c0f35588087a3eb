"""Command line in the manner of the reference's `infer` (examples/infer/main.go:15-114): the same
option names and defaults (-model, -prompt, -tokens 200, -strategy greedy, -temperature 0.8,
-top-k 50, -top-p 0.9, -repeat-penalty 1.1, -repeat-last-n 64, -kernel-info), generated ids on
standard output, the two timing lines on standard error. The prompt is a list of token ids
("1,2,3" or "1 2 3"; several prompts separated by ';' form a batch), since tokenizer and chat
template are not part of this library. Added: -dtype, -seed, -stop, and `-random CONFIG.json
-seed-weights S` which first writes a random-weights model folder to -model.
"""
from __future__ import annotations

import argparse
import json
import sys


def _ids(text: str) -> list[list[int]]:
    out = []
    for part in text.split(";"):
        toks = [int(t) for t in part.replace(",", " ").split()]
        if toks:
            out.append(toks)
    return out


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(
        prog="sllm-b200", description="Run generation on a model folder and print the generated token ids to stdout. "
        "Performance stats are written to stderr.", formatter_class=argparse.RawDescriptionHelpFormatter,
        epilog="Sampling strategies:\n  greedy       pick the highest-probability token every step\n"
               "  temperature  sample with temperature scaling\n  top_k        sample from the top-K most likely tokens\n"
               "  top_p        nucleus sampling up to cumulative probability P\n")
    ap.add_argument("-model", "--model", default="", help="Path to the model folder (required)")
    ap.add_argument("-prompt", "--prompt", default="", help="Input prompt as token ids (required); ';' separates prompts")
    ap.add_argument("-tokens", "--tokens", type=int, default=200, help="Maximum tokens to generate")
    ap.add_argument("-strategy", "--strategy", default="greedy", help="Sampling strategy: greedy, temperature, top_k, top_p")
    ap.add_argument("-temperature", "--temperature", type=float, default=0.8, help="Sampling temperature")
    ap.add_argument("-top-k", "--top-k", dest="top_k", type=int, default=50, help="Top-K candidates (top_k strategy)")
    ap.add_argument("-top-p", "--top-p", dest="top_p", type=float, default=0.9, help="Nucleus probability threshold")
    ap.add_argument("-repeat-penalty", "--repeat-penalty", dest="repeat_penalty", type=float, default=1.1,
                    help="Repetition penalty - 1.0 disables it")
    ap.add_argument("-repeat-last-n", "--repeat-last-n", dest="repeat_last_n", type=int, default=64,
                    help="Token window considered for repeat penalty")
    ap.add_argument("-kernel-info", "--kernel-info", dest="kernel_info", action="store_true",
                    help="Print the device and the kernel libraries of this build and exit")
    ap.add_argument("-dtype", "--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("-seed", "--seed", type=int, default=0, help="Seed of the sampling streams")
    ap.add_argument("-stop", "--stop", default=None, help="Stop token ids (default: config.json's eos ids; '' for none)")
    ap.add_argument("-random", "--random", default=None, metavar="CONFIG.json",
                    help="Write a random-weights model for this config.json into -model first")
    ap.add_argument("-seed-weights", "--seed-weights", dest="seed_weights", type=int, default=0)
    return ap


def kernel_info() -> str:
    import torch
    from .csrc.build import LIBRARIES, library_path
    dev = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "no CUDA device"
    libs = ", ".join(f"{n}={'built' if library_path(n) else 'not built yet'}" for n in sorted(LIBRARIES))
    return f"device: {dev}; kernels: hand-written CUDA for sm_100a ({libs})"


def main(argv=None) -> int:
    ap = build_parser()
    args = ap.parse_args(argv)
    if args.kernel_info:
        print(kernel_info())
        return 0
    if not args.model:
        print("error: -model is required", file=sys.stderr)
        ap.print_usage(sys.stderr)
        return 1
    if args.random:
        import torch
        from . import models  # noqa: F401
        from .config.registry import architecture_for
        from .engine.model import DecoderModel
        from .weights.random_init import write_random_model
        raw = json.loads(open(args.random).read())
        arch = architecture_for(raw["architectures"][0])
        cfg = arch.config_class.from_dict(raw, args.random)
        write_random_model(cfg, DecoderModel(arch.layout(cfg)).tensor_specs(), args.seed_weights, args.model, torch.bfloat16)
    prompts = _ids(args.prompt)
    if not prompts:
        print("error: -prompt is required", file=sys.stderr)
        ap.print_usage(sys.stderr)
        return 1
    from . import llm
    stop = None if args.stop is None else [int(t) for t in args.stop.replace(",", " ").split()]
    try:
        ids, st = llm.generate(args.model, prompts, args.tokens, args.strategy, temperature=args.temperature,
                               top_k=args.top_k, top_p=args.top_p, repeat_penalty=args.repeat_penalty,
                               repeat_last_n=args.repeat_last_n, seed=args.seed, stop_ids=stop, dtype=args.dtype,
                               stats=True)
    except Exception as e:  # the reference prints "error: ..." and exits 1 (examples/infer/main.go:99-102)
        print(f"error: {e}", file=sys.stderr)
        return 1
    for out in ids:
        print(" ".join(str(t) for t in out))
    n_prompt, n_gen = sum(st["prompt_tokens"]), sum(st["generated_tokens"])
    pre_ms, dec_ms = max(st["prefill_ms"]), max(st["decode_ms"])
    tps = lambda n, ms: n / ms * 1000.0 if ms > 0 else 0.0
    print("---", file=sys.stderr)
    print(f"prompt    {n_prompt:4d} tokens   prefill {pre_ms:6.0f} ms   {tps(n_prompt, pre_ms):6.1f} t/s", file=sys.stderr)
    print(f"generated {n_gen:4d} tokens   decode  {dec_ms:6.0f} ms   {tps(n_gen, dec_ms):6.1f} t/s", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
