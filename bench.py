#!/usr/bin/env python3
"""Decode and prefill throughput of the SmolLM2-1.7B-shaped model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 sequences; the K timed steps end at the benchmark
context length (prompts of context - W - K tokens are prefilled first). `value` is decoded tokens
per second, timed on the device with the sampled ids fed to the next step on the device; `e2e` is
the same through the Python entry point (`llm.generate`) with host token ids in and out every step; `prefill` is one 2,048-token prompt; `roofline`
relates the bytes a decode step has to read (every weight once, the cache of the live requests) to
the measured copy bandwidth; `points` holds decoding at batch 1 and 64. One JSON line on stdout.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# the benchmark's primary configuration: the SmolLM2-1.7B layer sizes
SHAPE = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "num_hidden_layers": 24, "hidden_size": 2048,
    "num_attention_heads": 32, "num_key_value_heads": 32, "head_dim": 64, "intermediate_size": 8192,
    "vocab_size": 49152, "rope_theta": 130000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 8192, "hidden_act": "silu",
}
# further sizes of the family (Llama-3.2-1B and Llama-3.1-8B layer sizes); the default run uses SHAPE
OTHER_SHAPES = {
    "llama3.2-1b": dict(SHAPE, num_hidden_layers=16, num_key_value_heads=8, vocab_size=128256, rope_theta=500000.0,
                        rope_scaling={"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                      "original_max_position_embeddings": 8192}),
    "llama3.1-8b": dict(SHAPE, num_hidden_layers=32, hidden_size=4096, num_key_value_heads=8, head_dim=128,
                        intermediate_size=14336, vocab_size=128256, rope_theta=500000.0, tie_word_embeddings=False,
                        rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                      "original_max_position_embeddings": 8192}),
}
CONTEXT = 4096
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]), "source": "measured"}
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self):
        return len(self.rows)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, lo=0, hi=None):
        rows = [r for r in self.rows[lo:hi] if len(r) == 6 and r[0].isdigit()]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": statistics.median(int(r[0]) for r in rows), "sm_max_mhz": int(rows[0][1]), "reasons": reasons,
                "samples": len(rows)}


def model_numbers(cfg, n_layers):
    d, H, G, hd, F, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                         cfg["intermediate_size"], cfg["vocab_size"])
    per_layer = d * (H + 2 * G) * hd + H * hd * d + 3 * d * F          # matrix weights of one layer
    head = V * d
    norms = (2 * n_layers + 1) * d
    return {"layer_params": per_layer, "head_params": head, "norm_params": norms,
            "kv_bytes_per_token": 2 * G * hd * n_layers * 2}


def decode_bytes(nums, n_layers, batch, contexts):
    """Bytes one decode step must read in bfloat16: every matrix once (the tied head is the
    embedding matrix), the norm weights, the embedding rows of the batch, and the cached keys and
    values of every live sequence."""
    weights = 2 * (nums["layer_params"] * n_layers + nums["head_params"] + nums["norm_params"])
    return weights + nums["kv_bytes_per_token"] * sum(contexts)


def prefill_flops(cfg, n_layers, T, logit_rows=1):
    nums = model_numbers(cfg, n_layers)
    linear = 2 * T * nums["layer_params"] * n_layers + 2 * logit_rows * nums["head_params"]
    attn = 2 * T * T * cfg["num_attention_heads"] * cfg["head_dim"] * n_layers     # causal: QK^T and PV, half the square each
    return linear + attn


def flush_l2(torch, buf):
    buf.add_(1)       # 512 MB read + written: more than the 126 MB L2


def write_model(tmp, cfg_raw, seed):
    import torch
    from scriptling_llm_lib_b200 import models  # noqa: F401
    from scriptling_llm_lib_b200.config.registry import architecture_for
    from scriptling_llm_lib_b200.engine.model import DecoderModel
    from scriptling_llm_lib_b200.weights.random_init import random_tensors
    from scriptling_llm_lib_b200.weights.safetensors_io import write_safetensors
    arch = architecture_for(cfg_raw["architectures"][0])
    cfg = arch.config_class.from_dict(cfg_raw, "bench config")
    specs = DecoderModel(arch.layout(cfg)).tensor_specs()
    tensors = random_tensors(specs, seed, torch.bfloat16, "cuda:0")
    os.makedirs(tmp, exist_ok=True)
    open(os.path.join(tmp, "config.json"), "w").write(json.dumps(cfg.to_json_dict()))
    write_safetensors(os.path.join(tmp, "model.safetensors"), {k: v.cpu() for k, v in tensors.items()})
    del tensors
    torch.cuda.empty_cache()
    return cfg


def time_decode(torch, eng, sampler, batch, context, steps, warmup, seed):
    """Prefill `batch` prompts so that warmup + steps decode steps end at `context`; returns
    (ms per step, contexts seen per timed step, launches per step)."""
    import numpy as np
    from scriptling_llm_lib_b200.csrc import bindings
    from scriptling_llm_lib_b200.engine.step import StepEntry
    from scriptling_llm_lib_b200.sampling.sampler import SamplingOptions
    V = eng.layout.vocab_size
    prompt_len = context - steps - warmup
    rng = np.random.default_rng(seed)
    seqs = [eng.open() for _ in range(batch)]
    greedy = SamplingOptions()
    try:
        # prompts go in a few sequences at a time to bound the activations of one step
        group = max(1, 16384 // prompt_len)
        toks = None
        last = []
        for i in range(0, batch, group):
            part = seqs[i:i + group]
            logits = eng.step([StepEntry(s, rng.integers(0, V, prompt_len).tolist()) for s in part])
            last.extend(sampler.sample(logits, greedy, [0] * len(part), [0] * len(part)).tolist())
        toks = last
        # the sampled ids stay on the device and feed the next step there: what is timed is the GPU's
        # work, one replayed step and one sampling kernel after another, with no host round trip between
        ids_dev = torch.tensor(toks, dtype=torch.int32, device=eng.device)

        def one():
            nonlocal ids_dev
            logits = eng.decode_step_device(seqs, ids_dev)
            ids_dev = sampler.sample(logits, greedy, [0] * batch, [0] * batch)
        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        l0 = bindings.LAUNCHES[0]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            one()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        launches = (bindings.LAUNCHES[0] - l0) / steps
        first = prompt_len + warmup + 1               # keys read by the first timed step
        contexts = [first + i for i in range(steps)]
        return ms, contexts, launches
    finally:
        for s in seqs:
            s.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="smollm2-1.7b", choices=["smollm2-1.7b"] + sorted(OTHER_SHAPES),
                    help="layer sizes to run (default: the SmolLM2-1.7B shape of the headline metric)")
    ap.add_argument("--layers", type=int, default=None,
                    help="run fewer layers of the same sizes (named in config as layers_run / layers_full)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--no-points", action="store_true", help="skip decoding at batch 1 and 64")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--only", default="all", choices=["all", "prefill", "decode"],
                    help="run one part only (a small case to profile); the JSON line then holds that part alone")
    args = ap.parse_args()
    shape = SHAPE if args.shape == "smollm2-1.7b" else OTHER_SHAPES[args.shape]
    if args.layers is None:
        args.layers = shape["num_hidden_layers"]

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Go package (go.mod) with CPU-only code; "
                          "pip cannot install it and no Go toolchain is in the image"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": "this library runs on one GPU; bench.py measures N=1 only", "n_gpus": args.gpus}))
        return 2
    args.warmup = max(3, args.warmup)

    import numpy as np
    import torch
    from scriptling_llm_lib_b200 import llm
    from scriptling_llm_lib_b200.csrc import bindings
    from scriptling_llm_lib_b200.engine.step import StepEntry

    pk = peaks()
    cfg_raw = dict(shape, num_hidden_layers=args.layers,
                   max_position_embeddings=max(shape["max_position_embeddings"], args.context + 64))
    nums = model_numbers(cfg_raw, args.layers)
    tmp = tempfile.mkdtemp(prefix="sllm_bench_")
    model_dir = os.path.join(tmp, "model")
    clocks = ClockSampler()
    try:
        write_model(model_dir, cfg_raw, seed=0)
        biggest = 64 if not (args.no_points or args.only != "all") else args.batch
        eng, sampler = llm.load(model_dir, "bfloat16", "cuda:0", max_tokens=biggest * args.context, max_seqs=biggest)
        l2 = torch.zeros(128 * 1024 * 1024, dtype=torch.float32, device="cuda:0")
        rng = np.random.default_rng(1)
        V = cfg_raw["vocab_size"]

        # ---- prefill of 2,048 tokens, L2 flushed between runs
        times = []
        for i in range((3 + 5) if args.only != "decode" else 0):
            flush_l2(torch, l2)
            s = eng.open()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ids = rng.integers(0, V, PREFILL_TOKENS).tolist()
            torch.cuda.synchronize()
            e0.record()
            eng.step([StepEntry(s, ids)])
            e1.record()
            torch.cuda.synchronize()
            s.close()
            if i >= 3:
                times.append(e0.elapsed_time(e1))
        pre_ms = statistics.median(times) if times else float("nan")
        pre_flops = prefill_flops(cfg_raw, args.layers, PREFILL_TOKENS)
        prefill = {"value": round(PREFILL_TOKENS / pre_ms * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
                   "frac": round(pre_flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

        if args.only == "prefill":
            print(json.dumps({"only": "prefill", "layers_run": args.layers, "prefill": prefill}))
            return 0
        # ---- the decode step at the headline batch, clocks sampled meanwhile
        clocks.start()
        time.sleep(0.5)
        c0 = clocks.mark()
        ms, contexts, launches = time_decode(torch, eng, sampler, args.batch, args.context, args.steps, args.warmup, 2)
        c1 = clocks.mark()
        value = args.batch / ms * 1e3
        step_bytes = decode_bytes(nums, args.layers, args.batch, [statistics.mean(contexts)] * args.batch)
        achieved = step_bytes / (ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]}

        points = {}
        if args.only == "decode":
            print(json.dumps({"only": "decode", "layers_run": args.layers, "batch": args.batch, "ms_per_step": round(ms, 4),
                              "value": round(value, 1), "roofline": roofline}))
            return 0
        # ---- end to end through the Python entry point: host ids in, host ids out, every step
        e2e = None
        if not args.no_e2e:
            prompt_len = args.context - args.steps - 1
            prompts = [rng.integers(0, V, prompt_len).tolist() for _ in range(args.batch)]
            marks = {}

            def on_step(i, toks):
                if i == 0:
                    torch.cuda.synchronize()
                    marks["t0"] = time.perf_counter()
                return False
            # warm-up with the same lengths: the cache is sized and the step's graph captured before the timed call
            llm.generate(model_dir, prompts, args.steps + 1, "greedy", temperature=0.0, stop_ids=[])
            out = llm.generate(model_dir, prompts, args.steps + 1, "greedy", temperature=0.0, stop_ids=[], on_step=on_step)
            torch.cuda.synchronize()
            dt = time.perf_counter() - marks["t0"]
            assert all(len(o) == args.steps + 1 for o in out)
            n_pages = -(-args.context // 64)
            e2e = {"value": round(args.batch * args.steps / dt, 1), "unit": "tokens/s",
                   "h2d_bytes_per_step": 4 * (args.batch * (5 + n_pages) + 1), "d2h_bytes_per_step": 4 * args.batch}
        c1 = clocks.mark()          # the clock samples cover the device-timed steps and the end-to-end run
        if not args.no_points:
            for b in (1, 64):
                k = max(8, args.steps // 4) if b == 64 else args.steps
                pms, _, _ = time_decode(torch, eng, sampler, b, args.context, k, args.warmup, 3 + b)
                points[f"decode_b{b}"] = round(b / pms * 1e3, 1)

        clk = clocks.summary(c0, c1)
    finally:
        clocks.stop()
        try:
            llm.unload()
            import shutil
            shutil.rmtree(tmp, ignore_errors=True)
        except Exception:
            pass

    line = {
        "metric": f"decode tokens/s ({args.shape} shape, random weights, batch {args.batch}, context {args.context})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform random token ids, random-init weights N(0,0.02)",
        "impl": "ours",
        "config": {"model": f"{args.shape} shape", "layers_run": args.layers, "layers_full": shape["num_hidden_layers"],
                   "hidden": shape["hidden_size"], "heads": shape["num_attention_heads"],
                   "kv_heads": shape["num_key_value_heads"], "head_dim": shape["head_dim"],
                   "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
                   "rope_theta": shape["rope_theta"], "rms_eps": shape["rms_norm_eps"], "tied": shape["tie_word_embeddings"],
                   "global_batch": args.batch, "seq_len": args.context, "prompt_len": args.context - args.steps - args.warmup,
                   "parallelism": "1gpu", "l2": "step inputs (weights+cache) exceed L2; prefill flushes L2",
                   "sampling": "greedy"},
        "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e,
        "gpu_launches": int(round(launches * args.steps)), "clocks": clk,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
