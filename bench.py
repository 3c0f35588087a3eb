#!/usr/bin/env python3
"""Decode and prefill throughput of the family's three benchmark shapes with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--shape smollm2-1.7b|llama3.2-1b|llama3.1-8b] [--dtype bfloat16|float32]
                    [--batch B] [--context C] [--prompts uniform:LO-HI] [--layers L]

A step is one decode step of a batch of 8 sequences; the K timed steps end at the benchmark
context length (prompts of context - W - K tokens are prefilled first). `value` is decoded tokens
per second, timed on the device with the sampled ids fed to the next step on the device; `e2e` is
the same through the Python entry point (`llm.generate`) with host token ids in and out every
step; `prefill` is one 2,048-token prompt; `roofline` relates the bytes a decode step has to read
(every weight once, the cache of the live requests) to the measured copy bandwidth; `points` holds
decoding at batch 1 and 64. The default run adds `f32`, the same measurements on the true 32-bit
path (its prompt step against a float fused-multiply-add rate measured here), and `shapes`: the
Llama-3.2-1B sizes on a batch of unequal prompts (lengths uniform in 128..2048, seeded; one packed
prompt step, then decoding) and the Llama-3.1-8B sizes at batch 1, 8 and 64. One JSON line on stdout.
`--kernel attn_decode|gemm_small_m` times one decode kernel alone instead (a line per case).

Weights are drawn on the device (`random:<config.json>:seed`), nothing is written but a config.json.
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
# further sizes of the family (Llama-3.2-1B and Llama-3.1-8B layer sizes); the default run's headline uses SHAPE
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
UNEQUAL = "uniform:128-2048"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
WIDTH = {"bfloat16": 2, "float32": 4}


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
    return {"layer_params": per_layer, "head_params": head, "norm_params": norms}


def decode_bytes(eng, contexts, width):
    """Bytes one decode step must read at `width` bytes an element, as the engine's own parts and
    cache state them: every weight a step uses once (the output head once, tied or not; of the
    embedding only rows), and the cached keys and values of every live sequence."""
    weights = eng.model.elements_read_per_step()
    kv_per_token = sum(2 * len(g.units) * g.need.kv_heads * g.need.head_dim for g in eng.cache.groups)
    return width * (weights + kv_per_token * sum(contexts))


def prefill_flops(cfg, n_layers, lengths, logit_rows=None):
    """Products of a prompt step over sequences of `lengths` tokens: 2 per weight and token, the head
    on `logit_rows` rows (default one per sequence), and causal attention (Q K^T and P V, half the
    square each) within each sequence."""
    nums = model_numbers(cfg, n_layers)
    T = sum(lengths)
    rows = len(lengths) if logit_rows is None else logit_rows
    linear = 2 * T * nums["layer_params"] * n_layers + 2 * rows * nums["head_params"]
    attn = sum(2 * n * n * cfg["num_attention_heads"] * cfg["head_dim"] * n_layers for n in lengths)
    return linear + attn


def flush_l2(buf):
    buf.add_(1)       # 512 MB read + written: more than the 126 MB L2


def parse_prompts(text):
    """'uniform:LO-HI' -> (LO, HI)."""
    kind, _, rng = text.partition(":")
    lo, _, hi = rng.partition("-")
    if kind != "uniform" or not lo.isdigit() or not hi.isdigit() or int(lo) < 1 or int(hi) < int(lo):
        raise SystemExit(f"--prompts {text!r}: expected uniform:LO-HI with 1 <= LO <= HI")
    return int(lo), int(hi)


class Bench:
    def __init__(self, args, pk, tmp):
        import numpy as np
        import torch
        from scriptling_llm_lib_b200 import llm
        from scriptling_llm_lib_b200.csrc import bindings
        self.np, self.torch, self.llm, self.bindings = np, torch, llm, bindings
        self.args, self.pk, self.tmp = args, pk, tmp
        self.l2 = None
        self._fma = None

    # ------------------------------------------------------------------ models
    def config(self, shape_name, layers=None):
        shape = SHAPE if shape_name == "smollm2-1.7b" else OTHER_SHAPES[shape_name]
        n_layers = layers or shape["num_hidden_layers"]
        raw = dict(shape, num_hidden_layers=n_layers,
                   max_position_embeddings=max(shape["max_position_embeddings"], self.args.context + 64,
                                               self.args.prefill_tokens))
        path = os.path.join(self.tmp, f"{shape_name}-{n_layers}.json")
        if not os.path.isfile(path):
            with open(path, "w") as f:
                json.dump(raw, f)
        return raw, n_layers, f"random:{path}:0"

    def load(self, spec, dtype, max_tokens, max_seqs):
        import gc
        self.llm.unload()
        self.l2 = None
        gc.collect()                 # an engine and its captured steps refer to each other
        self.torch.cuda.empty_cache()
        eng, sampler = self.llm.load(spec, dtype, "cuda:0", max_tokens=max_tokens, max_seqs=max_seqs)
        self.l2 = self.torch.zeros(128 * 1024 * 1024, dtype=self.torch.float32, device="cuda:0")
        return eng, sampler

    def fma_peak(self):
        if self._fma is None:
            self._fma = self.bindings.ProbeKernels().fma_tflops()
        return self._fma

    # ------------------------------------------------------------------ prompt steps
    def time_prompt_step(self, eng, lengths, seed, repeats=5, warm=3):
        """Median device time of one packed prompt step over sequences of `lengths` tokens, L2 flushed
        between runs; the logits of each sequence's last place are computed."""
        from scriptling_llm_lib_b200.engine.step import StepEntry
        torch = self.torch
        rng = self.np.random.default_rng(seed)
        V = eng.layout.vocab_size
        times = []
        for i in range(warm + repeats):
            flush_l2(self.l2)
            seqs = [eng.open() for _ in lengths]
            ids = [rng.integers(0, V, n).tolist() for n in lengths]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            eng.step([StepEntry(s, t) for s, t in zip(seqs, ids)])
            e1.record()
            torch.cuda.synchronize()
            for s in seqs:
                s.close()
            if i >= warm:
                times.append(e0.elapsed_time(e1))
        return statistics.median(times)

    def prefill_record(self, eng, cfg, n_layers, lengths, dtype, seed=1):
        ms = self.time_prompt_step(eng, lengths, seed)
        flops = prefill_flops(cfg, n_layers, lengths)
        T = sum(lengths)
        if dtype == "bfloat16":
            peak, name = self.pk["bf16_tflops"], f"bf16 tensor ({self.pk['source']})"
        else:
            peak, name = self.fma_peak(), "float FMA (measured here)"
        return {"value": round(T / ms * 1e3, 1), "tokens": T, "ms": round(ms, 3),
                "frac": round(flops / (ms * 1e-3) / (peak * 1e12), 4), "tflops": round(flops / (ms * 1e-3) / 1e12, 1),
                "peak_tflops": round(peak, 1), "peak": name}

    # ------------------------------------------------------------------ decode steps
    def time_decode(self, eng, sampler, prompt_lens, steps, warmup, seed):
        """Prefill one prompt per entry of `prompt_lens`, then warmup + steps decode steps with the
        sampled ids fed back on the device; returns (ms per step, mean keys read per sequence and
        timed step, launches per step)."""
        from scriptling_llm_lib_b200.engine.step import StepEntry
        from scriptling_llm_lib_b200.sampling.sampler import SamplingOptions
        torch, np = self.torch, self.np
        V = eng.layout.vocab_size
        batch = len(prompt_lens)
        rng = np.random.default_rng(seed)
        seqs = [eng.open() for _ in range(batch)]
        greedy = SamplingOptions()
        try:
            # prompts go in a few sequences at a time to bound the activations of one step
            last, i = [], 0
            while i < batch:
                j, tok = i, 0
                while j < batch and (j == i or tok + prompt_lens[j] <= 16384):
                    tok += prompt_lens[j]
                    j += 1
                logits = eng.step([StepEntry(s, rng.integers(0, V, n).tolist()) for s, n in zip(seqs[i:j], prompt_lens[i:j])])
                last.extend(sampler.sample(logits, greedy, [0] * (j - i), [0] * (j - i)).tolist())
                i = j
            ids_dev = torch.tensor(last, dtype=torch.int32, device=eng.device)

            def one():
                nonlocal ids_dev
                logits = eng.decode_step_device(seqs, ids_dev)
                ids_dev = sampler.sample(logits, greedy, [0] * batch, [0] * batch)
            for _ in range(warmup):
                one()
            torch.cuda.synchronize()
            l0 = self.bindings.LAUNCHES[0]
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                one()
            e1.record()
            torch.cuda.synchronize()
            eng.check_errors()
            ms = e0.elapsed_time(e1) / steps
            launches = (self.bindings.LAUNCHES[0] - l0) / steps
            # the first timed step reads prompt + warmup + 1 keys of each sequence, each later step one more
            contexts = [n + warmup + 1 + (steps - 1) / 2 for n in prompt_lens]
            return ms, contexts, launches
        finally:
            for s in seqs:
                s.close()

    def decode_record(self, eng, sampler, cfg, n_layers, prompt_lens, steps, warmup, seed, dtype):
        ms, contexts, launches = self.time_decode(eng, sampler, prompt_lens, steps, warmup, seed)
        achieved = decode_bytes(eng, contexts, WIDTH[dtype]) / (ms * 1e-3) / 1e9
        return {"value": round(len(prompt_lens) / ms * 1e3, 1), "ms": round(ms, 4), "gbs": round(achieved, 1),
                "frac": round(achieved / self.pk["hbm_gbs"], 4)}, launches

    def equal_prompts(self, batch, steps, warmup):
        return [self.args.context - steps - warmup] * batch


def run(args):
    import numpy as np
    import torch
    pk = peaks()
    tmp = tempfile.mkdtemp(prefix="sllm_bench_")
    clocks = ClockSampler()
    b = Bench(args, pk, tmp)
    llm = b.llm
    dtype = args.dtype
    line = None
    try:
        cfg, n_layers, spec = b.config(args.shape, args.layers)
        full_layers = (SHAPE if args.shape == "smollm2-1.7b" else OTHER_SHAPES[args.shape])["num_hidden_layers"]
        want_points = not args.no_points and args.only == "all" and args.prompts is None
        # the batch-64 point needs 64 contexts of cache: at long contexts that is more than the GPU has
        kv_token = 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * n_layers * WIDTH[dtype]
        weights = WIDTH[dtype] * (model_numbers(cfg, n_layers)["layer_params"] * n_layers + 2 * model_numbers(cfg, n_layers)["head_params"])
        free = torch.cuda.mem_get_info()[0]
        point_batches = [bb for bb in (1, 64) if weights + bb * args.context * kv_token < 0.85 * free] if want_points else []
        biggest = max(point_batches + [args.batch])
        eng, sampler = b.load(spec, dtype, max(biggest * args.context, args.prefill_tokens + 64), biggest)
        V = cfg["vocab_size"]

        # ---- the prompt step: 2,048 tokens, or a batch of unequal prompts in one packed step
        if args.prompts is not None:
            lo, hi = parse_prompts(args.prompts)
            lengths = np.random.default_rng(7).integers(lo, hi + 1, args.batch).tolist()
        else:
            lengths = [args.prefill_tokens]
        prefill = b.prefill_record(eng, cfg, n_layers, lengths, dtype) if args.only != "decode" else None
        if args.prompts is not None and prefill is not None:
            prefill["prompts"] = {"dist": args.prompts, "seed": 7, "n": len(lengths), "min": min(lengths), "max": max(lengths)}
        if args.only == "prefill":
            print(json.dumps({"only": "prefill", "shape": args.shape, "dtype": dtype, "layers_run": n_layers, "prefill": prefill}))
            return 0

        # ---- the decode step at the headline batch, clocks sampled meanwhile
        clocks.start()
        time.sleep(0.5)
        c0 = clocks.mark()
        prompt_lens = lengths if args.prompts is not None else b.equal_prompts(args.batch, args.steps, args.warmup)
        head, launches = b.decode_record(eng, sampler, cfg, n_layers, prompt_lens, args.steps, args.warmup, 2, dtype)
        c1 = clocks.mark()
        ms, value = head["ms"], head["value"]
        roofline = {"bound": "hbm", "achieved": head["gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": head["frac"],
                    "peaks": pk["source"]}
        if args.only == "decode":
            print(json.dumps({"only": "decode", "shape": args.shape, "dtype": dtype, "layers_run": n_layers, "batch": args.batch,
                              "ms_per_step": ms, "value": value, "roofline": roofline}))
            return 0

        # ---- end to end through the Python entry point: host ids in, host ids out, every step
        e2e = None
        if not args.no_e2e:
            rng = np.random.default_rng(1)
            n_gen = args.steps + args.warmup + 2          # the prompt's token, warm-up + 1 untimed decode steps, the timed ones
            e2e_lens = prompt_lens if args.prompts is not None else [args.context - n_gen] * args.batch
            prompts = [rng.integers(0, V, n).tolist() for n in e2e_lens]
            marks = {}

            def on_step(i, toks):
                # called when token i of every sequence has reached the host; the loop has already queued
                # decode step i + 1 by then, and the synchronize lets it finish before the clock starts
                if i == args.warmup:
                    torch.cuda.synchronize()
                    marks["t0"] = time.perf_counter()
                return False
            # a first call with the same lengths: the cache is sized and the step's graph captured before the timed call
            llm.generate(spec, prompts, n_gen, "greedy", temperature=0.0, stop_ids=[], dtype=dtype)
            out = llm.generate(spec, prompts, n_gen, "greedy", temperature=0.0, stop_ids=[], dtype=dtype, on_step=on_step)
            torch.cuda.synchronize()
            dt = time.perf_counter() - marks["t0"]
            assert all(len(o) == n_gen for o in out)
            graph = llm.load(spec, dtype)[0].decode_graphs.last_graph      # the captured step the run ended on
            e2e = {"value": round(args.batch * args.steps / dt, 1), "unit": "tokens/s",
                   "h2d_bytes_per_step": graph.h2d_bytes, "d2h_bytes_per_step": 4 * args.batch,
                   "window": f"decode steps {args.warmup + 2}..{n_gen - 1} of a generation of {n_gen} tokens: {args.steps} steps "
                             f"after {args.warmup + 1} untimed ones, wall clock, to the last token on the host"}
        c1 = clocks.mark()          # the clock samples cover the device-timed steps and the end-to-end run

        points = {}
        if want_points:
            for bb in point_batches:
                k = max(8, args.steps // 4) if bb == 64 else args.steps
                rec, _ = b.decode_record(eng, sampler, cfg, n_layers, b.equal_prompts(bb, k, args.warmup), k, args.warmup, 3 + bb, dtype)
                points[f"decode_b{bb}"] = rec["value"]
                points[f"decode_b{bb}_frac"] = rec["frac"]
        clk = clocks.summary(c0, c1)

        line = {
            "metric": f"decode tokens/s ({args.shape} shape, random weights, batch {args.batch}, context {args.context})",
            "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16" if dtype == "bfloat16" else "f32",
            "data": "synthetic: uniform random token ids, random-init weights N(0,0.02) drawn on the device",
            "impl": "ours",
            "config": {"model": f"{args.shape} shape", "layers_run": n_layers, "layers_full": full_layers,
                       "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                       "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                       "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                       "rope_theta": cfg["rope_theta"], "rms_eps": cfg["rms_norm_eps"], "tied": cfg["tie_word_embeddings"],
                       "global_batch": args.batch, "seq_len": args.context,
                       "prompt_len": args.prompts or (args.context - args.steps - args.warmup),
                       "parallelism": "1gpu", "l2": "step inputs (weights+cache) exceed L2; prefill flushes L2",
                       "sampling": "greedy"},
            "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e,
            "gpu_launches": int(round(launches * args.steps)), "clocks": clk,
        }

        # ---- the same model on the true 32-bit path
        if args.f32 and dtype == "bfloat16" and args.prompts is None:
            eng = sampler = None     # the bfloat16 engine's weights and cache go before the next one comes
            eng, sampler = b.load(spec, "float32", 64 * args.context, 64)
            f32 = {"prefill": b.prefill_record(eng, cfg, n_layers, [PREFILL_TOKENS], "float32"), "fma_peak_tflops": round(b.fma_peak(), 1)}
            for bb in (1, 8, 64):
                k = max(8, args.steps // 4) if bb == 64 else args.steps
                rec, _ = b.decode_record(eng, sampler, cfg, n_layers, b.equal_prompts(bb, k, args.warmup), k, args.warmup, 40 + bb, "float32")
                f32[f"decode_b{bb}"] = rec
            line["f32"] = f32

        # ---- the two further shapes of the family
        if args.shapes and dtype == "bfloat16" and args.prompts is None and args.shape == "smollm2-1.7b" and args.layers is None:
            shapes = {}
            lo, hi = parse_prompts(UNEQUAL)
            cfg2, L2, spec2 = b.config("llama3.2-1b")
            lengths = np.random.default_rng(7).integers(lo, hi + 1, 8).tolist()
            eng = sampler = None
            eng, sampler = b.load(spec2, "bfloat16", 8 * args.context, 8)
            rec = {"prompts": UNEQUAL, "batch": 8, "prefill": b.prefill_record(eng, cfg2, L2, lengths, "bfloat16")}
            rec["decode"], _ = b.decode_record(eng, sampler, cfg2, L2, lengths, args.steps, args.warmup, 50, "bfloat16")
            shapes["llama3.2-1b"] = rec
            cfg3, L3, spec3 = b.config("llama3.1-8b")
            eng = sampler = None
            eng, sampler = b.load(spec3, "bfloat16", 64 * args.context, 64)
            rec = {"context": args.context, "prefill": b.prefill_record(eng, cfg3, L3, [PREFILL_TOKENS], "bfloat16")}
            for bb in (1, 8, 64):
                k = max(8, args.steps // 4) if bb == 64 else args.steps
                rec[f"decode_b{bb}"], _ = b.decode_record(eng, sampler, cfg3, L3, b.equal_prompts(bb, k, args.warmup), k,
                                                          args.warmup, 60 + bb, "bfloat16")
            shapes["llama3.1-8b"] = rec
            line["shapes"] = shapes
    finally:
        clocks.stop()
        try:
            llm.unload()
            import shutil
            shutil.rmtree(tmp, ignore_errors=True)
        except Exception:
            pass
    print(json.dumps(line))
    return 0


def kernel_alone(args):
    """One decode kernel by itself, as profiles/ quotes it: launched back to back in a CUDA graph over
    inputs that rotate through more bytes than L2 holds, timed with CUDA events; one JSON line per case.
    attn_decode: the decode attention of --shape for --batch sequences of --context keys, once per split
    count. gemm_small_m: the four products of a layer of --shape (and the head) with --batch rows."""
    import math
    import torch
    from scriptling_llm_lib_b200.csrc.bindings import DecodeKernels
    dk = DecodeKernels()
    cfg = dict(SHAPE if args.shape == "smollm2-1.7b" else OTHER_SHAPES[args.shape])
    H, G = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // H
    D, F, V, B = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], args.batch
    sms = torch.cuda.get_device_properties(0).multi_processor_count

    def timed(launch, n_sets, reps=24):
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            for i in range(3):
                launch(i % n_sets)
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=side):
                for i in range(reps):
                    launch(i % n_sets)
        for _ in range(3):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(5):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (5 * reps) * 1e3

    if args.kernel == "attn_decode":
        pages = -(-args.context // 64)
        layer_bytes = B * pages * G * 64 * hd * 4
        n_sets = max(2, min(16, int(1.5e9 // layer_bytes)))
        ks = [torch.randn(B * pages, G, 64, hd, device="cuda").bfloat16() for _ in range(n_sets)]
        vs = [torch.randn(B * pages, G, 64, hd, device="cuda").bfloat16() for _ in range(n_sets)]
        table = torch.randperm(B * pages, device="cuda").int().view(B, pages).contiguous()
        pos0 = torch.full((B,), args.context - 1, dtype=torch.int32, device="cuda")
        q = torch.randn(B, H * hd, device="cuda").bfloat16()
        out = torch.empty(B, H * hd, dtype=torch.bfloat16, device="cuda")
        tickets = torch.zeros(B * G, dtype=torch.int32, device="cuda")
        chosen = dk.attention_splits(B, H, G, hd, pages, sms)
        for n in sorted({1, 2, 3, 4, 5, 6, 8, 12, 16, chosen}):
            if n > pages:
                continue
            scratch = torch.empty(B * H * n * (hd + 2), dtype=torch.float32, device="cuda")
            us = timed(lambda i: dk.attn_decode(q, out, pos0, table, ks[i], vs[i], scratch, B, H, G, hd, None,
                                                1.0 / math.sqrt(hd), n, tickets=tickets), n_sets)
            print(json.dumps({"kernel": "attn_decode", "shape": args.shape, "batch": B, "context": args.context, "splits": n,
                              "chosen": n == chosen, "blocks": n * G * B, "us": round(us, 1),
                              "tb_per_s": round(B * args.context * G * hd * 4 / us / 1e6, 2)}))
        return 0
    products = [("qkv", (H + 2 * G) * hd, D, False), ("o", D, H * hd, False), ("gate_up", 2 * F, D, True), ("down", D, F, False),
                ("head", V, D, False)]
    for name, N, K, gated in products:
        n_sets = max(2, int(600e6 // (N * K * 2)) + 1)
        ws = [torch.randn(N, K, device="cuda").bfloat16() for _ in range(n_sets)]
        x = torch.randn(B, K, device="cuda").bfloat16()
        if name in ("o", "down") and B <= dk.FOLD_MAX_M:
            # as the step runs them: the product adds to the residual stream and prepares the next norm
            resid = torch.zeros(B, N, dtype=torch.float32, device="cuda")
            fold = (torch.ones(N, dtype=torch.float32, device="cuda"), torch.empty(B, N, dtype=torch.bfloat16, device="cuda"),
                    torch.empty(-(-N // 16), B, dtype=torch.float32, device="cuda"))
            us = timed(lambda i: dk.gemm_small_m(x, ws[i], resid, fold=fold), n_sets)
            name += " (residual epilogue)"
        else:
            y = torch.empty(B, N // 2 if gated else N, dtype=torch.bfloat16, device="cuda")
            us = timed(lambda i: dk.gemm_small_m(x, ws[i], y, swiglu=gated), n_sets)
        print(json.dumps({"kernel": "gemm_small_m", "shape": args.shape, "product": name, "rows": B, "n": N, "k": K,
                          "blocks": -(-N // 16), "us": round(us, 1), "tb_per_s": round(N * K * 2 / us / 1e6, 2)}))
        del ws
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="smollm2-1.7b", choices=["smollm2-1.7b"] + sorted(OTHER_SHAPES),
                    help="layer sizes of the headline run (default: the SmolLM2-1.7B shape of the headline metric)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="precision of the headline run; float32 is the true 32-bit path")
    ap.add_argument("--layers", type=int, default=None,
                    help="run fewer layers of the same sizes (named in config as layers_run / layers_full)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--prefill-tokens", dest="prefill_tokens", type=int, default=PREFILL_TOKENS,
                    help="length of the one prompt of the prompt step (the headline metric's is 2,048)")
    ap.add_argument("--prompts", default=None, metavar="uniform:LO-HI",
                    help="a batch of unequal prompts, lengths uniform in LO..HI (seeded): one packed prompt step, then "
                         "decoding from there (instead of equal prompts that end at --context)")
    ap.add_argument("--no-points", action="store_true", help="skip decoding at batch 1 and 64")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-f32", dest="f32", action="store_false", help="skip the 32-bit path's measurements")
    ap.add_argument("--no-shapes", dest="shapes", action="store_false", help="skip the Llama-3.2-1B and Llama-3.1-8B sizes")
    ap.add_argument("--only", default="all", choices=["all", "prefill", "decode"],
                    help="run one part only (a small case to profile); the JSON line then holds that part alone")
    ap.add_argument("--kernel", default=None, choices=["attn_decode", "gemm_small_m"],
                    help="time one decode kernel alone at --shape, --batch (and --context) instead of the model")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Go package (go.mod) with CPU-only code; "
                          "pip cannot install it and no Go toolchain is in the image"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": "this library runs on one GPU; bench.py measures N=1 only", "n_gpus": args.gpus}))
        return 2
    args.warmup = max(3, args.warmup)
    if args.kernel is not None:
        return kernel_alone(args)
    return run(args)


if __name__ == "__main__":
    sys.exit(main())
