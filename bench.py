#!/usr/bin/env python3
"""Benchmark of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]
                    [--impl ours|reference] [--points LIST | --no-points] [--design tobovik|gubidra|komazen|vugedra [--sizes LIST]]

Headline (`value`): decode tokens/s of `batch` requests whose context ends at 4,096 tokens, on a
model with the layer sizes of Qwen3-8B (36 layers unless --layers says fewer; the JSON names both
numbers), random bfloat16 weights drawn on the device, uniform-random token ids, page size 16.  A
"step" is one decode step.  Before the line is printed, the logits of the last timed step are
compared with the same positions recomputed as whole prompts (`checked`); a mismatch exits 1, and a
mismatch of the float32 path exits 1 as well.

Beside it, on the same line: the prefill of 2,048 tokens, the decode step's share of the memory
roofline, the same decode through the Python entry point (`e2e`: host ids in, host ids out), and
`points`: decode at batch 1 and 64 with their roofline fractions, generation of 256 tokens after
2,048-token prompts, the float32 path at batch 8, the Qwen3-0.6B shape with 32 mixed requests, and
the Qwen3-32B shape at batch 16 (each sub-record names its sizes).

`--design tobovik [--sizes w1024,w2048,w4096]` measures something else and prints a line of its own:
prefill and decode of the Tobovik design beside Qwen3 at equal width, heads, feed-forward, depth and
vocabulary, and the design's own kernels beside the like kernels of the Qwen3 path with their roofline
fractions.  `--design gubidra` does the same for the Gubidra design beside Tobovik, its closest model, and
`--design komazen` for the Komazen design beside Qwen3, `--design vugedra` for the Vugedra design beside Gubidra.
Without it the workload and the line above are what they always were.

`--impl reference` times the unmodified reference engine (float32, its only precision) on the same
shape, batch, context and steps through baseline/reference_arm.py and prints the same keys with
`"impl": "reference"`.  For --gpus > 1 one line says that the engine runs on one GPU; exit code 2.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288,
    vocab_size=151936, rope_theta=1000000.0, rms_norm_eps=1e-6, max_position_embeddings=40960,
    tie_word_embeddings=False, torch_dtype="bfloat16")
QWEN3_0P6B = dict(QWEN3_8B, num_hidden_layers=28, hidden_size=1024, num_attention_heads=16,
                  intermediate_size=3072, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
                 intermediate_size=25600)
CONTEXT = 4096
LONG_CONTEXT = 32768                 # the further context length of the "long" points (Qwen3-8B allows 40,960)
PAGE = 16
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
ALL_POINTS = ("decode", "generate", "long", "fp32", "0p6b", "32b")
# The check before the line is printed: decode steps against whole prompts, same model, same positions.
# Two bfloat16 ways of computing one position are two roundings of the same exact value; their
# difference grows with depth like a random walk.  Measured on this shape against the float32 path
# (same weights, context 4,096, batch 8): root-mean-square difference of the logits, as a fraction of
# the largest |logit|, 0.0018 / 0.0030 / 0.0075 at 2 / 8 / 36 layers = 0.00125 * sqrt(layers), for
# decode-vs-float32, whole-vs-float32 and decode-vs-whole alike.  A wrong page, row or split moves
# logits by their own size (0.2 of the largest).  Allowed: 0.002 * sqrt(layers).  The float32 path
# differs between the two ways by 2e-5 of the largest logit at 36 layers (summation order in the
# library products); allowed there: 1e-5 * sqrt(layers).
CHECK_RMS_PER_SQRT_LAYER = 2e-3
CHECK_FP32_MAX_PER_SQRT_LAYER = 1e-5


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                v = d.get(k)
                if isinstance(v, dict):
                    v = v.get("value")
                if isinstance(v, (int, float)) and v > 0:
                    out[k] = float(v)
            out["source"] = "measured"
            return out
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.proc, self.lines, self.index = None, [], index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def shape_config(shape: dict, layers: int, batch: int, context: int, **more) -> dict:
    """The flat `config` record of a measurement (every size by name, at most 20 keys)."""
    c = {"layers": layers, "layers_full": shape["num_hidden_layers"], "hidden": shape["hidden_size"],
         "heads": shape["num_attention_heads"], "kv_heads": shape["num_key_value_heads"],
         "head_dim": shape["head_dim"], "intermediate": shape["intermediate_size"], "vocab": shape["vocab_size"],
         "tied_head": bool(shape["tie_word_embeddings"]), "global_batch": batch, "seq_len": context,
         "page_size": PAGE, "parallelism": "single GPU"}
    c.update(more)
    return c


# ---- the reference arm -----------------------------------------------------------------------------
def reference_arm(args) -> int:
    """The unmodified reference through its own PagedGenerateEngine: prefill each request, then
    `decode_batch` (src/engine/paged_generate_engine.cpp:99-149,182-341), on random float32 weights
    of the same shape.  Its API takes host token ids and returns host token ids, so its wall-clock
    figure is the end-to-end one."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_arm as ra
        shape = dict(QWEN3_8B, num_hidden_layers=args.layers)
        clocks = ClockSampler()
        clocks.start()
        try:
            r = ra.run(shape, batch=args.batch, context=CONTEXT, steps=args.steps, warmup=args.warmup,
                       page_size=PAGE, seed=2)
        finally:
            ck = clocks.stop()
    except Exception as e:                      # ReferenceUnavailable, a missing compiler, a time-out
        print(json.dumps({"impl": "reference", "unavailable": " ".join(str(e).split())[:400]}))
        return 0
    points = {}
    if not args.no_points and "0p6b" in args.points.split(","):
        # the workload the reference publishes a figure for (readme.md:66: 32 requests, 64 new tokens each,
        # paged batch decode), with the prompts of the 0.6B benchmark configuration: the whole job timed,
        # prefill and engine construction included, as its own benchmark does
        try:
            j = ra.run(QWEN3_0P6B, batch=32, context=512 + 64, steps=0, warmup=1, page_size=PAGE, seed=3,
                       job={"prompt_min": 64, "prompt_max": 512, "new_tokens": 64})
            points["qwen3_0p6b_mixed"] = {"tok_s": round(j["tokens"] / j["wall_s"], 2), "new_tokens": j["tokens"],
                                          "seconds": round(j["wall_s"], 3), "dtype": "fp32",
                                          "config": shape_config(QWEN3_0P6B, QWEN3_0P6B["num_hidden_layers"], 32, 576,
                                                                 prompt_min=64, prompt_max=512, new_tokens=64)}
        except Exception as e:
            points["qwen3_0p6b_mixed"] = {"unavailable": " ".join(str(e).split())[:300]}
    ms = r["device_ms"] / r["steps"]
    out = {
        "impl": "reference",
        "metric": "decode tokens/s (Qwen3-8B shape, batch %d, context %d)" % (args.batch, CONTEXT),
        "value": round(r["tokens"] / (r["device_ms"] * 1e-3), 2), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic (random weights, uniform-random token ids)",
        "config": shape_config(QWEN3_8B, args.layers, args.batch, CONTEXT, model="Qwen3-8B shape",
                               note="the reference computes in float32 only"),
        "e2e": {"value": round(r["tokens"] / r["wall_s"], 2), "unit": "tokens/s",
                "h2d_bytes_per_step": r["h2d_bytes_per_step"], "d2h_bytes_per_step": r["d2h_bytes_per_step"]},
        "prefill": {"value": round(args.batch * r["longest_prompt"] / r["prefill_s"], 1),
                    "tokens": r["longest_prompt"], "ms": round(r["prefill_s"] * 1e3 / args.batch, 1)},
        "points": points, "clocks": ck,
    }
    print(json.dumps(out))
    return 0


# ---- our arm -------------------------------------------------------------------------------------
class Bench:
    """The measurements of this engine.  Each model lives inside one method, so that its memory
    is free again when the next one is built."""

    def __init__(self, args, pk):
        import torch
        from litellmengine_b200.csrc import ops
        from litellmengine_b200.engine import ModelRunner, PagedGenerateEngine, StepEntry
        self.torch, self.ops = torch, ops
        self.ModelRunner, self.Engine, self.Entry = ModelRunner, PagedGenerateEngine, StepEntry
        self.args, self.pk = args, pk
        self.gen = torch.Generator().manual_seed(2)
        torch.cuda.set_device(0)

    # ---- helpers -----------------------------------------------------------------------------------
    def ev(self):
        return self.torch.cuda.Event(enable_timing=True)

    def tokens(self, n, vocab=QWEN3_8B["vocab_size"]):
        return self.torch.randint(0, vocab, (n,), generator=self.gen).tolist()

    def build(self, shape, layers, dtype, max_batch, context, seed, step_tokens=None):
        from litellmengine_b200.config import config_from_dict
        config = config_from_dict(dict(shape, num_hidden_layers=layers))
        return self.ModelRunner.from_config(config, seed=seed, dtype=dtype, device="cuda:0", page_size=PAGE,
                                            max_total_tokens=max_batch * context + 64, max_requests=max_batch,
                                            max_tokens_per_step=step_tokens or context)

    def free_memory(self):
        gc.collect()
        self.torch.cuda.synchronize()
        self.torch.cuda.empty_cache()

    @staticmethod
    def prefill_flops(p, layers, T, prompts=1):
        per_layer = 2 * T * p.hidden_size * ((p.num_attention_heads + 2 * p.num_key_value_heads) * p.head_dim
                                              + p.num_attention_heads * p.head_dim + 3 * p.intermediate_size)
        attn = 2 * 2 * p.num_attention_heads * p.head_dim * (T * (T + 1) // 2)
        return prompts * (layers * (per_layer + attn) + 2 * p.hidden_size * p.vocab_size)

    def settle(self):
        """Between the prompts (seconds at the power cap) and the decode steps that are timed: wait until
        the device is idle, and a moment longer.  Right after a burst at the cap the SM clock is still
        low, and the first dozen decode steps run 10 % slower (4.0 ms falling to 3.6 over 16 steps when
        measured without this pause); whether a measurement saw that depended on whether the host
        happened to stall first (a graph capture does), not on the engine."""
        self.torch.cuda.synchronize()
        time.sleep(0.3)

    def fill(self, runner, batch, prompt_len):
        slots, prompts = [], []
        for _ in range(batch):
            s = runner.admit()
            prompts.append(self.tokens(prompt_len))
            runner.step([self.Entry(s, prompts[-1], [])])
            slots.append(s)
        return slots, prompts

    def decode_device_timed(self, runner, batch, steps, warmup, context=CONTEXT, sample_clocks=False, keep=False):
        """`batch` requests prefilled so that warmup + steps decode steps end at `context`; the steps
        are timed with CUDA events around the launches.  Returns a record; with `keep` also what a
        check needs (prompts, fed tokens, the last step's logits)."""
        torch, ops, Entry = self.torch, self.ops, self.Entry
        slots, prompts = self.fill(runner, batch, context - (steps + warmup))
        feed = [self.tokens(batch) for _ in range(steps + warmup)]
        self.settle()
        for i in range(warmup):
            lg = runner.step([Entry(s, [feed[i][j]], [0]) for j, s in enumerate(slots)])
            ops.argmax_rows(lg)
        torch.cuda.synchronize()
        clocks = ClockSampler() if sample_clocks else None
        if clocks:
            clocks.start()
        launches0 = ops.launch_count
        a, b = self.ev(), self.ev()
        a.record()
        for i in range(warmup, warmup + steps):
            lg = runner.step([Entry(s, [feed[i][j]], [0]) for j, s in enumerate(slots)])
            ops.argmax_rows(lg)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
        ctx_mid = context - steps // 2
        step_bytes = runner.model.weight_bytes() + runner.cache.bytes_per_token() * ctx_mid * batch
        gbs = step_bytes / (ms * 1e-3) / 1e9
        rec = {"ms": ms, "tok_s": batch / (ms * 1e-3), "gbs": gbs, "frac": gbs / self.pk["hbm_gbs"],
               "launches": ops.launch_count - launches0, "clocks": clocks.stop() if clocks else None}
        if keep:
            rec.update(prompts=prompts, feed=feed, logits=lg.clone())
        for s in slots:
            runner.release(s)
        return rec

    def check_last_step(self, runner, rec):
        """The logits of the last timed decode step (a replayed graph over the pages) against the same
        positions as the last token of whole prompts, each run alone in one step without a graph.
        Returns the largest and the root-mean-square difference and the largest |logit|."""
        worst, scale, sq, n = 0.0, 1.0, 0.0, 0
        for j, prompt in enumerate(rec["prompts"]):
            seq = prompt + [f[j] for f in rec["feed"]]
            s = runner.admit()
            whole = runner.step([self.Entry(s, seq, [len(seq) - 1])])
            runner.release(s)
            diff = (whole[0] - rec["logits"][j]).double()
            worst = max(worst, float(diff.abs().max()))
            sq, n = sq + float((diff * diff).sum()), n + diff.numel()
            scale = max(scale, float(whole.abs().max()))
        runner.check_status()
        return {"max": worst, "rms": (sq / n) ** 0.5, "scale": scale}

    def e2e_decode(self, runner, batch, prompt_len, new_tokens, steps, warmup):
        """Through `PagedGenerateEngine`: host token ids in, host token ids out, every step."""
        engine = self.Engine(runner)
        ids = [engine.add_request(self.tokens(prompt_len), new_tokens) for _ in range(batch)]
        while any(engine.request(i).cached_len < engine.request(i).prompt_len for i in ids):
            engine.step()                                    # prompts (and the first sampled tokens)
        self.settle()
        for _ in range(warmup):
            engine.step()
        self.torch.cuda.synchronize()
        t0 = time.perf_counter()
        produced = 0
        for _ in range(steps):
            produced += len(engine.step())
        self.torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        assert produced == steps * batch, "a request left the batch inside the timed steps"
        for i in ids:
            engine.release_request(i)
        while engine.has_work():
            engine.step()
        return produced / e2e_s

    # ---- Qwen3-8B shape, bfloat16: the headline ------------------------------------------------------
    def qwen3_8b(self, want_points, points):
        args, pk, torch = self.args, self.pk, self.torch
        many = bool({"decode", "generate"} & want_points)
        runner = self.build(QWEN3_8B, args.layers, "bfloat16", max(args.batch, 64) if many else args.batch, CONTEXT,
                            seed=2, step_tokens=max(CONTEXT, PREFILL_TOKENS))
        T = PREFILL_TOKENS

        def prefill_once():
            s = runner.admit()
            runner.step([self.Entry(s, self.tokens(T), [T - 1])])
            runner.release(s)
        for _ in range(3):
            prefill_once()
        torch.cuda.synchronize()
        reps = 5
        e0, e1 = self.ev(), self.ev()
        e0.record()
        for _ in range(reps):
            prefill_once()
        e1.record()
        torch.cuda.synchronize()
        prefill_ms = e0.elapsed_time(e1) / reps
        flops = self.prefill_flops(runner.config, args.layers, T)
        prefill = {"value": round(T / (prefill_ms * 1e-3), 1), "tokens": T, "ms": round(prefill_ms, 3),
                   "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

        head = self.decode_device_timed(runner, args.batch, args.steps, args.warmup, sample_clocks=True, keep=True)
        check = self.check_last_step(runner, head)
        check["allowed_rms"] = CHECK_RMS_PER_SQRT_LAYER * args.layers ** 0.5 * check["scale"]
        check["ok"] = check["rms"] <= check["allowed_rms"]
        out = {"prefill": prefill, "head": head, "check": check}
        if not check["ok"]:
            return out
        # Prompts are prefilled one per step, so the first request decodes a few tokens before the last
        # one starts: leave room for that, so that all of them still decode in the timed steps.
        n_new = args.steps + args.warmup + args.batch
        value = self.e2e_decode(runner, args.batch, CONTEXT - n_new, n_new + 8, args.steps, args.warmup)
        out["e2e"] = {"value": round(value, 1), "unit": "tokens/s",
                      "h2d_bytes_per_step": runner.buffers.last.size * 4, "d2h_bytes_per_step": args.batch * 4}
        if "decode" in want_points:
            for b in (1, 64):
                r = self.decode_device_timed(runner, b, max(8, min(args.steps, 32)), 3, keep=True)
                c = self.check_last_step(runner, r)
                allowed = CHECK_RMS_PER_SQRT_LAYER * args.layers ** 0.5 * c["scale"]
                points[f"decode_b{b}"] = round(r["tok_s"], 1)
                points[f"decode_b{b}_ms"] = round(r["ms"], 3)
                points[f"decode_b{b}_frac"] = round(r["frac"], 4)
                points[f"decode_b{b}_check"] = {"ok": c["rms"] <= allowed, "rms_err": float("%.3g" % c["rms"]),
                                                "allowed_rms": float("%.3g" % allowed)}
            # end to end at batch 64 too (beside `decode_b64`: the host's share of a step grows with the batch)
            n64 = max(8, min(args.steps, 32)) + 3 + 64
            points["e2e_b64"] = round(self.e2e_decode(runner, 64, CONTEXT - n64, n64 + 8, max(8, min(args.steps, 32)), 3), 1)
        if "generate" in want_points:
            # the workload the baseline states: 2,048-token prompts, then 256 new tokens, end to end
            for b in (1, 8, 64):
                points[f"generate_p2048_n256_b{b}"] = round(self.e2e_decode(runner, b, 2048, 256 + b, 200, 8), 1)
        return out

    # ---- the same shape at a context of 32,768 ----------------------------------------------------------
    def qwen3_8b_long(self, points):
        """One 32,768-token prompt in one step (the attention's share of the work grows with the length),
        then decode steps at batch 8 and batch 1 that end at that context: a step reads 39 GB of keys
        and values beside the weights, so the attention kernel is most of it."""
        args, pk, torch = self.args, self.pk, self.torch
        C = LONG_CONTEXT
        try:
            runner = self.build(QWEN3_8B, args.layers, "bfloat16", 8, C, seed=2)
            s = runner.admit()
            runner.step([self.Entry(s, self.tokens(C), [C - 1])])
            runner.release(s)
            torch.cuda.synchronize()
            a, b = self.ev(), self.ev()
            a.record()
            s = runner.admit()
            runner.step([self.Entry(s, self.tokens(C), [C - 1])])
            b.record()
            torch.cuda.synchronize()
            runner.release(s)
            pms = a.elapsed_time(b)
            flops = self.prefill_flops(runner.config, args.layers, C)
            rec = {"context": C, "prefill_tok_s": round(C / (pms * 1e-3), 1), "prefill_ms": round(pms, 1),
                   "prefill_frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
                   "prefill_peak": "sustained"}
            for bsz in (8, 1):
                r = self.decode_device_timed(runner, bsz, 16, 4, context=C, keep=True)
                c = self.check_last_step(runner, r)
                allowed = CHECK_RMS_PER_SQRT_LAYER * args.layers ** 0.5 * c["scale"]
                rec[f"decode_b{bsz}"] = round(r["tok_s"], 1)
                rec[f"decode_b{bsz}_ms"] = round(r["ms"], 3)
                rec[f"decode_b{bsz}_frac"] = round(r["frac"], 4)
                rec[f"decode_b{bsz}_check"] = {"ok": c["rms"] <= allowed, "rms_err": float("%.3g" % c["rms"]),
                                               "allowed_rms": float("%.3g" % allowed)}
            rec["ok"] = all(rec[f"decode_b{bsz}_check"]["ok"] for bsz in (8, 1))
            points["context_32768"] = rec
        except torch.cuda.OutOfMemoryError as e:
            points["context_32768"] = {"skipped": "out of device memory: " + str(e)[:80]}

    # ---- the same shape in true float32 -------------------------------------------------------------
    def qwen3_8b_fp32(self, points):
        args = self.args
        key = "decode_b%d_fp32" % args.batch
        try:
            runner = self.build(QWEN3_8B, args.layers, "float32", args.batch, CONTEXT, seed=2)
            r = self.decode_device_timed(runner, args.batch, max(4, min(args.steps, 16)), 3, keep=True)
            check = self.check_last_step(runner, r)
            allowed = CHECK_FP32_MAX_PER_SQRT_LAYER * args.layers ** 0.5 * check["scale"]
            points[key] = round(r["tok_s"], 1)
            points[key + "_ms"] = round(r["ms"], 3)
            points[key + "_frac"] = round(r["frac"], 4)
            points[key + "_check"] = {"ok": check["max"] <= allowed, "max_err": float("%.3g" % check["max"]),
                                      "allowed": float("%.3g" % allowed)}
        except self.torch.cuda.OutOfMemoryError as e:
            points[key] = {"skipped": "out of device memory: " + str(e)[:80]}

    # ---- Qwen3-0.6B shape: 32 requests, prompts of 64..512 tokens, 64 new tokens each, mixed steps ----
    def qwen3_0p6b(self, points):
        torch = self.torch
        L = QWEN3_0P6B["num_hidden_layers"]
        runner = self.build(QWEN3_0P6B, L, "bfloat16", 32, 512 + 64 + 16, seed=3, step_tokens=512)
        lens = torch.randint(64, 513, (32,), generator=self.gen).tolist()
        prompts = [self.tokens(n) for n in lens]

        def job():
            engine = self.Engine(runner, chunk=256)
            steps0 = runner.steps_run
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = engine.generate(prompts, max_new_tokens=64)
            torch.cuda.synchronize()
            return sum(len(o) for o in out), time.perf_counter() - t0, runner.steps_run - steps0
        # Warm-up, twice: a decode step of a batch size is captured as a graph the second time that size is
        # seen, and the sizes of the tail (requests finishing one by one) occur once a job.
        job()
        job()
        made, secs, nsteps = job()
        d32 = self.decode_device_timed(runner, 32, 32, 8, context=384)
        points["qwen3_0p6b_mixed"] = {
            "tok_s": round(made / secs, 1), "new_tokens": made, "seconds": round(secs, 4), "steps": nsteps,
            "ms_per_step": round(secs * 1e3 / nsteps, 3), "decode_b32_tok_s": round(d32["tok_s"], 1),
            "decode_b32_ms": round(d32["ms"], 4), "decode_b32_frac": round(d32["frac"], 4), "dtype": "bf16",
            "config": shape_config(QWEN3_0P6B, L, 32, 384, prompt_min=64, prompt_max=512, new_tokens=64, chunk=256,
                                   step_tokens=512)}

    # ---- Qwen3-32B shape: 16 prompts of 4,096 tokens, then 128 decode steps -----------------------------
    def qwen3_32b(self, points):
        torch, pk = self.torch, self.pk
        free, _ = torch.cuda.mem_get_info()
        free += torch.cuda.memory_reserved() - torch.cuda.memory_allocated()
        need = 100e9
        if free < need:
            points["qwen3_32b"] = {"skipped": f"{free / 1e9:.0f} GB of device memory free, {need / 1e9:.0f} needed"}
            return
        try:
            L = QWEN3_32B["num_hidden_layers"]
            runner = self.build(QWEN3_32B, L, "bfloat16", 16, 4096 + 128, seed=4, step_tokens=4096)
            warm = runner.admit()
            runner.step([self.Entry(warm, self.tokens(4096), [4095])])
            runner.release(warm)
            torch.cuda.synchronize()
            slots = []
            a, b = self.ev(), self.ev()
            a.record()
            for _ in range(16):
                s = runner.admit()
                runner.step([self.Entry(s, self.tokens(4096), [4095])])
                slots.append(s)
            b.record()
            torch.cuda.synchronize()
            pms = a.elapsed_time(b)
            for s in slots:
                runner.release(s)
            d = self.decode_device_timed(runner, 16, 120, 8, context=4096 + 128)
            flops = self.prefill_flops(runner.config, L, 4096, 16)
            points["qwen3_32b"] = {
                "decode_tok_s": round(d["tok_s"], 1), "decode_ms": round(d["ms"], 3), "decode_frac": round(d["frac"], 4),
                "prefill_tok_s": round(16 * 4096 / (pms * 1e-3), 1), "prefill_ms": round(pms, 1),
                "prefill_frac": round(flops / (pms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
                "prefill_peak": "sustained", "weight_gb": round(runner.model.weight_bytes() / 1e9, 2), "dtype": "bf16",
                "config": shape_config(QWEN3_32B, L, 16, 4096 + 128, prompt=4096, decode_steps=128)}
        except torch.cuda.OutOfMemoryError as e:
            points["qwen3_32b"] = {"skipped": "out of device memory: " + str(e)[:80]}


# ---- another design beside its closest model ----------------------------------------------------------
# `--design tobovik`: prefill and decode of the Tobovik design at a few sizes that resemble a real model's
# layers (random weights), beside Qwen3 at equal width, heads, feed-forward, depth and vocabulary, and the
# design's own kernels one by one beside the like kernels of the Qwen3 path with their roofline
# fractions.  The default workload and its JSON line do not change.
DESIGN_VOCAB = 32768
DESIGN_SIZES = {            # width, feed-forward, query heads, kv heads, layers
    "w1024": (1024, 3072, 8, 4, 8),
    "w2048": (2048, 6144, 16, 8, 8),
    "w4096": (4096, 12288, 32, 8, 4),
}
DESIGN_HEAD = 128


def tobovik_dict(width, ff, heads, kv, layers):
    """Three parallel layers, then a gla layer, and so on; key and value heads of 128 so that the softmax side
    takes the same tuned attention kernels as Qwen3; the linear-attention side a quarter of the heads."""
    mlp = {"kind": "dense", "ff": ff}
    par = {"type": "parallel", "mlp": mlp, "mixer": {
        "left": {"heads": heads, "kv_heads": kv, "dim": DESIGN_HEAD, "vdim": DESIGN_HEAD, "scale": DESIGN_HEAD ** -0.5,
                 "q_temp": {"coef": 0.25, "every": 256}},
        "right": {"heads": max(1, heads // 4), "dim": DESIGN_HEAD, "vdim": DESIGN_HEAD, "tau": 8.0, "rank": 64},
        "left_scale": 1.0, "right_scale": 0.5}}
    gla = {"type": "gla", "mlp": mlp,
           "mixer": {"heads": max(1, heads // 2), "dim": DESIGN_HEAD, "vdim": DESIGN_HEAD, "tau": 8.0, "rank": 64}}
    return {"architecture": "Tobovik", "vocab": DESIGN_VOCAB, "width": width, "norm": {"eps": 1e-5},
            "layers": [gla if i % 4 == 3 else par for i in range(layers)]}


def gubidra_dict(width, ff, heads, kv, layers):
    """Retention, retention, attention, matrix memory, and so on; every layer with eight experts of half the
    feed-forward size of which two are chosen (as many active weights as the dense feed-forward of equal size,
    four times as many stored); two residual streams; the attention windowed at the decode context."""
    mlp = {"kind": "moe", "expert": {"ff": ff // 2, "limit": 7.0},
           "router": {"experts": 8, "top": 2, "scale": 1.0, "groups": {"count": 4, "keep": 2}}}
    half = max(1, heads // 2)
    ret = {"type": "retention", "mlp": mlp, "mixer": {
        "heads": half, "dim": DESIGN_HEAD, "vdim": DESIGN_HEAD, "rot": {"dims": DESIGN_HEAD, "base": 10000.0},
        "decay": [1.0 - 2.0 ** (-5 - 3 * i / max(1, half - 1)) for i in range(half)]}}
    att = {"type": "attention", "mlp": mlp, "mixer": {
        "heads": heads, "kv_heads": kv, "dim": DESIGN_HEAD, "vdim": DESIGN_HEAD, "scale": DESIGN_HEAD ** -0.5,
        "mask": {"size": 1024}, "bias_max": 2048, "bias_rows": 32}}
    mem = {"type": "mlstm", "mlp": mlp, "mixer": {"heads": half, "dim": DESIGN_HEAD // 2, "vdim": DESIGN_HEAD, "gate_cap": 15.0}}
    return {"architecture": "Gubidra", "vocab": DESIGN_VOCAB, "width": width, "norm": {"eps": 1e-5},
            "embedding": {"scale": 1.0}, "streams": 2, "layers": [(ret, ret, att, mem)[i % 4] for i in range(layers)]}


def komazen_dict(width, ff, heads, kv, layers):
    """Attention (head temperature, logarithmic distance bias), latent attention that keeps its own rows, attention,
    latent attention that reads the rows of the latent layer before it, and so on; heads of 128; latents of 512 with a
    rotated part of 64 (one cached row of 576 per token), a query latent of three eighths of the width, a window of
    1,024 keys; three convolution taps; the dense gated feed-forward of equal size."""
    mlp = {"kind": "dense", "ff": ff}
    att = {"type": "attention", "mlp": mlp, "mixer": {"heads": heads, "kv_heads": kv, "dim": DESIGN_HEAD, "vdim": DESIGN_HEAD,
                                                      "scale": DESIGN_HEAD ** -0.5}}

    def lat(src):
        m = {"heads": heads, "dim": DESIGN_HEAD, "rot_dim": 64, "vdim": DESIGN_HEAD, "q_rank": 3 * width // 8, "kv_rank": 512,
             "scale": (DESIGN_HEAD + 64) ** -0.5, "rot": {"base": 10000.0, "dims": 64}, "mask": {"size": 1024}}
        if src is not None:
            m["kv_from"] = src
        return {"type": "latent_attention", "mlp": mlp, "mixer": m}
    return {"architecture": "Komazen", "vocab": DESIGN_VOCAB, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "postln_alpha": 2.0, "canon": {"taps": 3},
            "layers": [att if i % 2 == 0 else lat(i - 2 if i % 4 == 3 else None) for i in range(layers)]}


def vugedra_dict(width, ff, heads, kv, layers):
    """Attention (a window of 1,024 keys that keeps the first four, neighbouring pairs of half a head rotated with stretched
    frequencies, a sink, a gate per head), gated linear attention, latent attention over one cached row of 576 per token,
    gated linear attention, and so on; heads of 128.  Every layer has eight experts of half the feed-forward size of which
    two of ten router outputs are chosen (two of the ten are no experts), and a shared expert of a quarter."""
    mlp = {"kind": "moe", "expert": {"ff": ff // 2}, "router": {"experts": 8, "identity": 2, "top": 2}, "shared": {"ff": ff // 4}}
    att = {"type": "attention", "mlp": mlp, "mixer": {
        "heads": heads, "kv_heads": kv, "dim": DESIGN_HEAD, "vdim": DESIGN_HEAD, "scale": DESIGN_HEAD ** -0.5,
        "mask": {"size": 1024, "keep_first": 4},
        "rot": {"base": 10000.0, "dims": DESIGN_HEAD // 2, "scaling": {"factor": 4.0, "original": 1024, "fast": 32.0, "slow": 1.0}}}}
    gla = {"type": "gla", "mlp": mlp,
           "mixer": {"heads": max(1, heads // 2), "dim": DESIGN_HEAD, "vdim": DESIGN_HEAD, "tau": 8.0, "rank": 64}}
    lat = {"type": "latent_attention", "mlp": mlp, "mixer": {
        "heads": heads, "dim": DESIGN_HEAD, "rot_dim": 64, "vdim": DESIGN_HEAD, "q_rank": 3 * width // 8, "kv_rank": 512,
        "scale": (DESIGN_HEAD + 64) ** -0.5,
        "rot": {"base": 10000.0, "dims": 64, "scaling": {"factor": 4.0, "original": 1024, "fast": 32.0, "slow": 1.0}}}}
    return {"architecture": "Vugedra", "vocab": DESIGN_VOCAB, "width": width, "norm": {"eps": 1e-5},
            "layers": [(att, gla, lat, gla)[i % 4] for i in range(layers)]}


def vugedra_bench(args, pk, measure) -> int:
    """`--design vugedra`: the design beside Gubidra (the closest model: recurrent layers beside windowed attention, routed
    experts in every layer) at equal width, heads, expert sizes, depth and vocabulary, and its kernels beside their like."""
    import math
    import torch
    import types
    from litellmengine_b200.config import config_from_dict
    from litellmengine_b200.config.specs import PositionSpec
    from litellmengine_b200.csrc import ops
    from litellmengine_b200.csrc.microbench import Flusher, timed
    from litellmengine_b200.parts.registry import lookup
    dev = "cuda:0"
    sizes = {}
    for name, (width, ff, heads, kv, layers) in DESIGN_SIZES.items():
        if args.sizes and name not in args.sizes.split(","):
            continue
        sizes[name] = {"shape": {"width": width, "ff": ff, "heads": heads, "kv_heads": kv, "layers": layers, "vocab": DESIGN_VOCAB}}
        for label, cfg in (("vugedra", vugedra_dict(width, ff, heads, kv, layers)), ("gubidra", gubidra_dict(width, ff, heads, kv, layers))):
            sizes[name][label] = measure(config_from_dict(cfg))
            gc.collect()
            torch.cuda.empty_cache()
        v, g = sizes[name]["vugedra"], sizes[name]["gubidra"]
        sizes[name]["vugedra_over_gubidra"] = {k: round(v[k] / g[k], 3) for k in v if k.endswith("tok_s")}
    flush = Flusher(dev)
    width, ff, heads, kv, _ = DESIGN_SIZES["w4096"]
    T, hbm, d = 2048, pk["hbm_gbs"] * 1e9, DESIGN_HEAD
    tensor_peak = pk.get("bf16_tflops", 1590.0) * 1e12
    kernels = {}

    def add(name, fn, nbytes=None, flops=None):
        sec = timed(fn, 5, 3, flush)
        rec = {"us": round(sec * 1e6, 2)}
        if nbytes is not None:
            rec.update(gbs=round(nbytes / sec / 1e9, 1), frac_of_hbm=round(nbytes / sec / hbm, 4))
        if flops is not None:
            rec.update(tflops=round(flops / sec / 1e12, 2), frac_of_bf16_peak=round(flops / sec / tensor_peak, 4))
        kernels[name] = rec

    i32 = lambda x: torch.as_tensor(x, dtype=torch.int32, device=dev)
    pos = torch.arange(T, device=dev, dtype=torch.int32)
    prompt = types.SimpleNamespace(positions=pos, token_entry=i32([0] * T), entry_slot=i32([0]), entry_q_start=i32([0]),
                                   entry_q_len=i32([T]))
    status = torch.zeros(2, dtype=torch.int32, device=dev)
    # the norm around the residual add
    h, y, w = torch.randn(T, width, device=dev), torch.randn(T, width, device=dev), torch.ones(width, device=dev)
    one = torch.ones(1, device=dev)
    tri = (one, w, w * 0.1)
    add("tanh_norm (new: norm of a sublayer's output + residual add + norm of the next input, bfloat16 copy)",
        lambda: ops.tanh_norm(h, y, tri, tri, torch.bfloat16), nbytes=T * width * (4 + 4 + 4 + 2))
    add("rmsnorm (like: residual add + norm, bfloat16 copy)", lambda: ops.rmsnorm(h, w, 1e-5, torch.bfloat16, delta=y, write_sum=True),
        nbytes=T * width * (4 + 4 + 4 + 2))
    # between the projection and attention: biases, norm over the projection, pair rotation, page write
    pages = T // PAGE
    qkv = torch.randn(T, (heads + 2 * kv) * d + heads, device=dev)
    cache = torch.zeros(pages, 2, kv, PAGE, d, device=dev, dtype=torch.bfloat16)
    tbl = torch.arange(pages, device=dev, dtype=torch.int32).view(1, pages)
    scaling = (4.0, 1024.0, 32.0, 1.0)
    rot = lookup("position", "rope_pairs")(PositionSpec("rope_pairs", 1e4, d // 2, (("scaling", scaling), ("magnitude", 0.1 * math.log(4.0) + 1.0))),
                                           d, dev).kernel_args()
    bq, bk = torch.zeros(heads * d, device=dev), torch.zeros(kv * d, device=dev)
    wq, wk = torch.ones(heads * d, device=dev), torch.ones(kv * d, device=dev)
    prep = lambda r: ops.attention_prepare(qkv, 0, heads * d, (heads + kv) * d, (bq, bk, bk), wq, wk, "projection", 1e-5, None,
                                           cache[:, 0], cache[:, 1], pos, prompt.token_entry, prompt.entry_slot, tbl, heads, kv, d, d,
                                           PAGE, status, torch.bfloat16, rotation=r)
    prep_bytes = T * (heads + 2 * kv) * d * (4 + 2)
    add("attention_prepare with the rotation of pairs (new)", lambda: prep(rot), nbytes=prep_bytes)
    add("attention_prepare without a rotation (like: what Tobovik's attention takes)", lambda: prep(None), nbytes=prep_bytes)
    # prompt attention: window 1,024, four kept keys, a sink, a gate per head
    cache.normal_()
    qa = torch.randn(T, heads * d, device=dev).to(torch.bfloat16)
    oa = torch.empty_like(qa)
    tiles = torch.tensor([(0, r0) for r0 in range(0, T, ops.PREFILL_TILE_ROWS)][::-1], device=dev, dtype=torch.int32)
    e_len = i32([T])
    window = 1024
    walked = sum(min(p + 1, window) for p in range(T))
    attn_flops = 4.0 * heads * d * walked
    common = (cache, tiles, tiles.shape[0], prompt.entry_slot, prompt.entry_q_start, e_len, e_len, tbl, heads, kv, d, PAGE, window,
              d ** -0.5, status)
    add("prompt attention, window 1024 with kept keys, sink and a gate per head (new; mma.sync): 2048 tokens",
        lambda: ops.paged_attention_prefill_biased(qa, oa, 0, *common, head_gate=qkv, gate_off=(heads + 2 * kv) * d, keep_first=4, sink=0.0),
        flops=attn_flops)
    add("prompt attention, the same kernel with the window and the gate alone (like: what Gubidra's prompt portions take)",
        lambda: ops.paged_attention_prefill_biased(qa, oa, 0, *common, head_gate=qkv, gate_off=(heads + 2 * kv) * d), flops=attn_flops)
    Bd, ctx = 64, 2048
    dpages = ctx // PAGE
    dcache = torch.randn(Bd * dpages, 2, kv, PAGE, d, device=dev).to(torch.bfloat16)
    dtbl = torch.arange(Bd * dpages, device=dev, dtype=torch.int32).view(Bd, dpages)
    dpos = torch.full((Bd,), ctx - 1, device=dev, dtype=torch.int32)
    dent = torch.arange(Bd, device=dev, dtype=torch.int32)
    kv_bytes = Bd * window * 2 * kv * d * 2
    add(f"decode attention, split-key kernel with kept keys and sink (new): {Bd} tokens at position {ctx - 1}, window {window}",
        lambda: ops.paged_attention_decode(qa[:Bd], oa[:Bd], dcache, None, Bd, dpos, dent, dent, dtbl, heads, kv, d, PAGE, window, d ** -0.5,
                                           2, status, keep_first=4, sink=0.0), nbytes=kv_bytes)
    add("decode attention, split-key kernel with the window alone (like)",
        lambda: ops.paged_attention_decode(qa[:Bd], oa[:Bd], dcache, None, Bd, dpos, dent, dent, dtbl, heads, kv, d, PAGE, window, d ** -0.5,
                                           2, status), nbytes=kv_bytes)
    ogen = torch.empty(Bd, heads * d, device=dev, dtype=torch.bfloat16)
    add("decode attention, the general kernel with kept keys and sink (new: the 32-bit mode and odd shapes)",
        lambda: ops.paged_attention_generic_kv(qa[:Bd], dcache[:, 0], dcache[:, 1], dpos, dent, dent, dtbl, heads, kv, d, d, PAGE, window,
                                               d ** -0.5, status, ogen, keep_first=4, sink=0.0), nbytes=kv_bytes)
    # the latent layer's small kernels with the rotation of pairs beside the half-split one
    Q, R, P = 3 * width // 8, 512, 64
    proj = torch.randn(T, Q + R + P, device=dev)
    rows = torch.zeros(pages, 1, PAGE, R + P, device=dev, dtype=torch.bfloat16)
    invf, rd, mag, _ = lookup("position", "rope_pairs")(PositionSpec("rope_pairs", 1e4, P, (("scaling", scaling), ("magnitude", 1.14))), P, dev).kernel_args()
    ones_q, ones_r = torch.ones(Q, device=dev), torch.ones(R, device=dev)
    for label, pairs in (("pairs, stretched (new)", True), ("half-split (like)", False)):
        add(f"latent_prepare, rotation of {label}",
            lambda pairs=pairs: ops.latent_prepare(proj, 0, Q, Q, R, P, P, ones_q, ones_r, 1e-5, invf, rows, prompt, tbl, PAGE, status,
                                                   torch.bfloat16, rot_pairs=pairs, rot_mag=mag if pairs else 1.0),
            nbytes=T * (Q + R + P) * (4 + 2))
    q32 = torch.randn(T, heads * (d + P), device=dev)
    for label, pairs in (("pairs, stretched (new)", True), ("half-split (like)", False)):
        add(f"latent_q_split, rotation of {label}",
            lambda pairs=pairs: ops.latent_q_split(q32, pos, invf, heads, d, P, R, P, torch.bfloat16, rot_pairs=pairs, rot_mag=mag if pairs else 1.0),
            nbytes=T * heads * (d + P) * (4 + 2))
    # the router and what joins the experts' sum
    E, top, fe = 8, 2, ff // 2
    x = torch.randn(T, width, device=dev).to(torch.bfloat16)
    wr = torch.randn(E + 2, width, device=dev) * width ** -0.5
    corr = torch.randn(E + 2, device=dev) * 0.1
    add("moe_route, softmax with a correction and two outputs that are no experts (new)",
        lambda: ops.moe_route(x, wr, top, None, 1.0, score="softmax", correction=corr, identity=2), nbytes=T * (width * 2 + E * 4))
    add("moe_route, sigmoid with groups (like)", lambda: ops.moe_route(x, wr[:E].contiguous(), top, (4, 2), 1.0), nbytes=T * (width * 2 + E * 4))
    gu = torch.randn(T, E * 2 * fe, device=dev)
    dense = ops.moe_route(x, wr[:E].contiguous(), top, (4, 2), 1.0)
    add("moe_act, plain silu gate (new)", lambda: ops.moe_act(gu, dense, E, fe, float("inf"), 1.0, torch.bfloat16, shift=0.0),
        nbytes=T * (top * 2 * fe * 4 + E * fe * 2))
    add("moe_act, clamped gate (like)", lambda: ops.moe_act(gu, dense, E, fe, 7.0, 1.702, torch.bfloat16),
        nbytes=T * (top * 2 * fe * 4 + E * fe * 2))
    out32, sh = torch.randn(T, width, device=dev), torch.randn(T, width, device=dev)
    idw = torch.rand(T, device=dev)
    add("moe_finish (new: the token's own share and the shared expert join the experts' sum)",
        lambda: ops.moe_finish(out32, x, idw, sh), nbytes=T * width * (4 + 4 + 4 + 2))
    add("residual_add (like)", lambda: ops.residual_add(out32, sh), nbytes=T * width * 12)
    print(json.dumps({"metric": "tokens/s of the Vugedra design beside Gubidra at equal sizes (bfloat16, random weights)",
                      "design": "vugedra", "prompt_tokens": 2048, "decode_context": 1024, "steps": args.steps,
                      "warmup": args.warmup, "sizes": sizes, "kernels_at_w4096": kernels,
                      "peaks": {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": round(tensor_peak / 1e12, 1), "source": pk["source"]},
                      "l2": "kernel timings: a 256 MB buffer is overwritten between launches; steps read every weight"}))
    return 0


def komazen_bench(args, pk, measure) -> int:
    """`--design komazen`: the design beside Qwen3 (the closest model: softmax attention and a dense gated feed-forward
    in every layer) at equal width, heads, feed-forward, depth and vocabulary, and its kernels beside their like."""
    import torch
    from litellmengine_b200.config import config_from_dict
    from litellmengine_b200.csrc import ops
    from litellmengine_b200.csrc.microbench import Flusher, timed
    import types
    dev = "cuda:0"
    sizes = {}
    for name, (width, ff, heads, kv, layers) in DESIGN_SIZES.items():
        if args.sizes and name not in args.sizes.split(","):
            continue
        qwen = dict(QWEN3_8B, num_hidden_layers=layers, hidden_size=width, num_attention_heads=heads, num_key_value_heads=kv,
                    head_dim=DESIGN_HEAD, intermediate_size=ff, vocab_size=DESIGN_VOCAB)
        sizes[name] = {"shape": {"width": width, "ff": ff, "heads": heads, "kv_heads": kv, "layers": layers, "vocab": DESIGN_VOCAB}}
        for label, cfg in (("komazen", komazen_dict(width, ff, heads, kv, layers)), ("qwen3", qwen)):
            sizes[name][label] = measure(config_from_dict(cfg))
            gc.collect()
            torch.cuda.empty_cache()
        k, q = sizes[name]["komazen"], sizes[name]["qwen3"]
        sizes[name]["komazen_over_qwen3"] = {x: round(k[x] / q[x], 3) for x in k if x.endswith("tok_s")}
    flush = Flusher(dev)
    width, ff, heads, kv, _ = DESIGN_SIZES["w4096"]
    T, hbm, d = 2048, pk["hbm_gbs"] * 1e9, DESIGN_HEAD
    tensor_peak = pk.get("bf16_tflops", 1590.0) * 1e12
    kernels = {}

    def add(name, fn, nbytes=None, flops=None):
        sec = timed(fn, 5, 3, flush)
        rec = {"us": round(sec * 1e6, 2)}
        if nbytes is not None:
            rec.update(gbs=round(nbytes / sec / 1e9, 1), frac_of_hbm=round(nbytes / sec / hbm, 4))
        if flops is not None:
            rec.update(tflops=round(flops / sec / 1e12, 2), frac_of_bf16_peak=round(flops / sec / tensor_peak, 4))
        kernels[name] = rec

    i32 = lambda x: torch.as_tensor(x, dtype=torch.int32, device=dev)
    pos = torch.arange(T, device=dev, dtype=torch.int32)
    prompt = types.SimpleNamespace(positions=pos, token_entry=i32([0] * T), entry_slot=i32([0]), entry_q_start=i32([0]),
                                   entry_q_len=i32([T]))
    h, y, w = torch.randn(T, width, device=dev), torch.randn(T, width, device=dev), torch.ones(width, device=dev)
    taps = torch.randn(width, 3, device=dev) * 0.3
    kept = torch.zeros(1, 2, width, device=dev)
    add("short_conv (new: the stream plus its 3-tap causal convolution, stored in bfloat16)",
        lambda: ops.short_conv(h, taps, kept, prompt, torch.bfloat16), nbytes=T * width * (4 + 2))
    add("scaled_add_norm (new: norm after the sum, keeps the convolution's rows)",
        lambda: ops.scaled_add_norm(h, y, w, 2.0, 1e-5, kept, prompt), nbytes=T * width * (4 + 4 + 4))
    add("rmsnorm (like: residual add + norm, bfloat16 copy)", lambda: ops.rmsnorm(h, w, 1e-5, torch.bfloat16, delta=y, write_sum=True),
        nbytes=T * width * (4 + 4 + 4 + 2))
    gu = torch.randn(T, 2 * ff, device=dev).to(torch.bfloat16)
    add("gelu_tanh gate (new)", lambda: ops.silu_and_mul(gu, activation="gelu_tanh"), nbytes=T * ff * 6)
    add("silu gate (like)", lambda: ops.silu_and_mul(gu), nbytes=T * ff * 6)
    # the latent layer's small kernels
    Q, R, P = 3 * width // 8, 512, 64
    pages = T // PAGE
    status = torch.zeros(2, dtype=torch.int32, device=dev)
    proj = torch.randn(T, Q + R + P, device=dev)
    rows = torch.zeros(pages, 1, PAGE, R + P, device=dev, dtype=torch.bfloat16)
    tbl = torch.arange(pages, device=dev, dtype=torch.int32).view(1, pages)
    invf = torch.pow(torch.tensor(1e4), -torch.arange(0, P, 2, dtype=torch.float32) / P).to(dev)
    ones_q, ones_r = torch.ones(Q, device=dev), torch.ones(R, device=dev)
    add("latent_prepare (new: two latent norms, rotation, page write)",
        lambda: ops.latent_prepare(proj, 0, Q, Q, R, P, P, ones_q, ones_r, 1e-5, invf, rows, prompt, tbl, PAGE, status, torch.bfloat16),
        nbytes=T * (Q + R + P) * (4 + 2))
    q32 = torch.randn(T, heads * (d + P), device=dev)
    add("latent_q_split (new: query rotation, head-major copy)",
        lambda: ops.latent_q_split(q32, pos, invf, heads, d, P, R, P, torch.bfloat16), nbytes=T * heads * (d + P) * (4 + 2))
    qkv = torch.randn(T, (heads + 2 * kv) * d, device=dev)
    cache = torch.zeros(pages, 2, kv, PAGE, d, device=dev, dtype=torch.bfloat16)
    hw = torch.ones(d, device=dev)
    invd = torch.pow(torch.tensor(1e6), -torch.arange(0, d, 2, dtype=torch.float32) / d).to(dev)
    add("qk_norm_rope_kv_write (like: head norm, rotation, page write)",
        lambda: ops.qk_norm_rope_kv_write(qkv, cache, pos, prompt.token_entry, prompt.entry_slot, tbl, hw, hw, 1e-6, invd, d, heads, kv,
                                          d, PAGE, True, status, q_dtype=torch.bfloat16), nbytes=T * (heads + 2 * kv) * d * (4 + 2))
    # attention with temperature and logarithmic bias beside the plain kernels: one 2,048-token prompt, 64 single tokens
    cache.normal_()
    qa = torch.randn(T, heads * d, device=dev).to(torch.bfloat16)
    oa = torch.empty_like(qa)
    three = torch.stack([torch.ones(heads), torch.ones(heads), torch.ones(heads)], dim=1).to(dev).contiguous()
    tiles = torch.tensor([(0, r0) for r0 in range(0, T, ops.PREFILL_TILE_ROWS)][::-1], device=dev, dtype=torch.int32)
    e_len = i32([T])
    attn_flops = 4.0 * heads * d * (T * (T + 1) / 2)
    common = (cache, tiles, tiles.shape[0], prompt.entry_slot, prompt.entry_q_start, e_len, e_len, tbl, heads, kv, d, PAGE, None,
              d ** -0.5, status)
    add("prompt attention with temperature + logarithmic bias (new; mma.sync): 2048 tokens",
        lambda: ops.paged_attention_prefill_biased(qa, oa, 0, *common, dist_bias_t=three, analytic_bias=True), flops=attn_flops)
    if ops.prefill_tcgen05_biased_supported(d, PAGE, heads // kv):
        add("prompt attention with temperature + logarithmic bias (new; tcgen05, what the design's prompt portions take): 2048 tokens",
            lambda: ops.paged_attention_prefill_tcgen05_biased(qa, oa, *common, three), flops=attn_flops)
    add("prompt attention, the same mma.sync kernel without them (like)", lambda: ops.paged_attention_prefill(qa, oa, *common),
        flops=attn_flops)
    if ops.prefill_tcgen05_supported(d, PAGE):
        add("prompt attention, the tcgen05 kernel (like: what the closest model's prompt portions take)",
            lambda: ops.paged_attention_prefill_tcgen05(qa, oa, *common), flops=attn_flops)
    Bd, ctx = 64, 1024
    dpages = ctx // PAGE
    dcache = torch.randn(Bd * dpages, 2, kv, PAGE, d, device=dev).to(torch.bfloat16)
    dtbl = torch.arange(Bd * dpages, device=dev, dtype=torch.int32).view(Bd, dpages)
    dpos = torch.full((Bd,), ctx - 1, device=dev, dtype=torch.int32)
    dent = torch.arange(Bd, device=dev, dtype=torch.int32)
    kv_bytes = Bd * ctx * 2 * kv * d * 2
    add(f"decode attention with temperature + logarithmic bias, split-key kernel (new): {Bd} tokens, {ctx} keys each",
        lambda: ops.paged_attention_decode(qa[:Bd], oa[:Bd], dcache, None, Bd, dpos, dent, dent, dtbl, heads, kv, d, PAGE, None, d ** -0.5,
                                           2, status, dist_bias_t=three, analytic_bias=True), nbytes=kv_bytes)
    add("decode attention, split-key kernel (like)",
        lambda: ops.paged_attention_decode(qa[:Bd], oa[:Bd], dcache, None, Bd, dpos, dent, dent, dtbl, heads, kv, d, PAGE, None, d ** -0.5,
                                           2, status), nbytes=kv_bytes)
    # latent attention over the cached rows: every head of a token reads the same rows
    lrows = torch.randn(Bd * dpages, 1, PAGE, R + P, device=dev).to(torch.bfloat16)
    ql = torch.randn(T, heads * (R + P), device=dev).to(torch.bfloat16)
    ol = torch.empty(T, heads * R, device=dev, dtype=torch.bfloat16)
    lat_bytes = Bd * ctx * (R + P) * 2
    lat_flops = 2.0 * heads * (2 * R + P)

    def latent(n_tok, positions, entries, slots, table, window):
        return lambda: ops.latent_attention(ql[:n_tok], lrows, positions, entries, slots, table, heads, R, P, PAGE, window, 0.07, status,
                                            ol[:n_tok])
    add(f"latent attention, {Bd} single tokens, {ctx} rows each (new)", latent(Bd, dpos, dent, dent, dtbl, 1024),
        nbytes=lat_bytes, flops=lat_flops * Bd * ctx)
    ptbl = torch.arange(pages, device=dev, dtype=torch.int32).view(1, pages)
    walked = sum(min(p + 1, 1024) for p in range(T))
    add("latent attention, one 2048-token prompt, window 1024 (new)",
        latent(T, pos, prompt.token_entry, prompt.entry_slot, ptbl, 1024), flops=lat_flops * walked)
    print(json.dumps({"metric": "tokens/s of the Komazen design beside Qwen3 at equal sizes (bfloat16, random weights)",
                      "design": "komazen", "prompt_tokens": 2048, "decode_context": 1024, "steps": args.steps,
                      "warmup": args.warmup, "sizes": sizes, "kernels_at_w4096": kernels,
                      "peaks": {"hbm_gbs": pk["hbm_gbs"], "bf16_tflops": round(tensor_peak / 1e12, 1), "source": pk["source"]},
                      "l2": "kernel timings: a 256 MB buffer is overwritten between launches; steps read every weight"}))
    return 0


def gubidra_bench(args, pk, measure) -> int:
    """`--design gubidra`: the design beside Tobovik (the closest model: softmax attention beside a linear
    recurrence) at equal width, heads, feed-forward, depth and vocabulary, and its kernels beside their like."""
    import torch
    from litellmengine_b200.config import config_from_dict
    from litellmengine_b200.csrc import ops
    from litellmengine_b200.csrc.microbench import Flusher, timed
    dev = "cuda:0"
    sizes = {}
    for name, (width, ff, heads, kv, layers) in DESIGN_SIZES.items():
        if args.sizes and name not in args.sizes.split(","):
            continue
        sizes[name] = {"shape": {"width": width, "ff": ff, "heads": heads, "kv_heads": kv, "layers": layers, "vocab": DESIGN_VOCAB}}
        for label, cfg in (("gubidra", gubidra_dict(width, ff, heads, kv, layers)), ("tobovik", tobovik_dict(width, ff, heads, kv, layers))):
            sizes[name][label] = measure(config_from_dict(cfg))
            gc.collect()
            torch.cuda.empty_cache()
        g, t = sizes[name]["gubidra"], sizes[name]["tobovik"]
        sizes[name]["gubidra_over_tobovik"] = {k: round(g[k] / t[k], 3) for k in g if k.endswith("tok_s")}
    flush = Flusher(dev)
    width, ff, heads, kv, _ = DESIGN_SIZES["w4096"]
    T, hbm, d = 2048, pk["hbm_gbs"] * 1e9, DESIGN_HEAD
    kernels = {}
    props = torch.cuda.get_device_properties(0)
    fp32_peak = props.multi_processor_count * 128 * 2 * 1.965e9

    def add(name, fn, nbytes=None, flops=None):
        sec = timed(fn, 5, 3, flush)
        rec = {"us": round(sec * 1e6, 2)}
        if nbytes is not None:
            rec.update(gbs=round(nbytes / sec / 1e9, 1), frac_of_hbm=round(nbytes / sec / hbm, 4))
        if flops is not None:
            rec.update(tflops=round(flops / sec / 1e12, 2), frac_of_fp32_peak=round(flops / sec / fp32_peak, 4))
        kernels[name] = rec

    S = 2
    streams = torch.randn(S, T, width, device=dev)
    y = torch.randn(T, width, device=dev)
    w = torch.ones(width, device=dev)
    mix, vec = torch.eye(S, device=dev).contiguous(), torch.ones(S, device=dev)
    add("stream_norm, 2 streams (new: update of the streams + layer norm of their weighted sum)",
        lambda: ops.stream_norm(streams, y, mix, vec, vec, w, 1e-5, True, torch.bfloat16), nbytes=T * width * (8 * S + 4 + 2))
    add("stream_norm, 1 stream (new: residual add + layer norm)",
        lambda: ops.stream_norm(streams[0], y, None, None, None, w, 1e-5, True, torch.bfloat16), nbytes=T * width * (4 + 4 + 4 + 2))
    add("rmsnorm (like: residual add + norm)", lambda: ops.rmsnorm(streams[0], w, 1e-5, torch.bfloat16, delta=y, write_sum=True),
        nbytes=T * width * (4 + 4 + 4 + 2))
    # the recurrences: a 2,048-token portion in chunks of 64, and 64 single tokens
    H, D, V = heads // 4, d, d
    gp = torch.randn(T, 2 * H * D + 2 * H * V + 2 * H, device=dev)
    offs = (0, H * D, 2 * H * D, 2 * H * D + H * V)
    gout = torch.empty(T, H * V, device=dev, dtype=torch.bfloat16)
    B = 64
    slot0 = torch.zeros(1, device=dev, dtype=torch.int32)
    items = torch.tensor([(0, c, 64, i) for i, c in enumerate(range(0, T, 64))], device=dev, dtype=torch.int32)
    chains = torch.tensor([(0, 0, T // 64)], device=dev, dtype=torch.int32)
    q0, qn = torch.zeros(1, device=dev, dtype=torch.int32), torch.full((1,), T, device=dev, dtype=torch.int32)
    pos = torch.arange(T, device=dev, dtype=torch.int32)
    decay = torch.full((H,), 0.99, device=dev)
    invf = torch.pow(torch.tensor(1e4), -torch.arange(0, D, 2, dtype=torch.float32) / D).to(dev)
    slots = torch.arange(B, device=dev, dtype=torch.int32)
    dq0 = torch.arange(B, device=dev, dtype=torch.int32)
    scan_flops = T * H * D * V * 6

    def recurrence(label, head_floats, cols, alpha, a_tok, kscale, nfloor, norm_w, norm_stride, gate, before=None, step=None):
        state = torch.zeros(B, H, head_floats, device=dev)
        ss, sa = torch.empty(T // 64, H, D * cols, device=dev), torch.empty(T // 64, H, D, device=dev)

        def chunked():
            if before is not None:
                before(state)
            a = alpha() if callable(alpha) else alpha
            scan = lambda mode: ops.recur_scan(gp, offs, a[0] if isinstance(a, tuple) else a, a_tok, 1,
                                               a[1] if isinstance(a, tuple) else kscale, a[2] if isinstance(a, tuple) else nfloor,
                                               norm_w, norm_stride, gate, 1e-5, D ** -0.5, 1.0, gout, 0, state, head_floats, slot0,
                                               q0, qn, items, T // 64, mode, ss, sa, H, D, V)
            scan(ops.GLA_LOCAL)
            ops.recur_chain(state, head_floats, ss, sa, chains, 1, slot0, H, D, V, cols > V)
            scan(ops.GLA_OUT)
        add(f"{label}: one 2048-token portion in chunks of 64 (new)", chunked, flops=scan_flops * cols / V)
        add(f"{label}: {B} single tokens (new: the decode kernel)", lambda: step(state), nbytes=2 * B * H * D * cols * 4)

    recurrence("retention", D * V, V, decay, 0, None, None, None, 0, "silu",
               before=lambda st: ops.rotate_qk(gp, offs[0], offs[1], H, H, D, D, invf, pos),
               step=lambda st: ops.recur_step(gp[:B], offs, decay, (0, 1, 0), None, 0, "silu", 1e-5, D ** -0.5, 1.0, gout[:B], 0, st,
                                              D * V, slots, dq0, B, H, D, V, rotation=(invf, D, pos[:B])))
    i_off, f_off = offs[3] + H * V, offs[3] + H * V + H
    bias = torch.zeros(H, device=dev)
    nw = torch.ones(H * V, device=dev)
    hf = D * (V + 1) + 1
    made = {}

    def gates_of(st):
        made["g"] = ops.recur_gates(gp, i_off, f_off, bias, bias, 15.0, st, D * (V + 1), hf, slot0, q0, qn, 1, H)
    recurrence("matrix memory", hf, V + 1, lambda: (made["g"][0], made["g"][1], made["g"][2]), H, None, None, nw, V, "sigmoid",
               before=gates_of,
               step=lambda st: ops.recur_step(gp[:B], offs, None, None, nw, V, "sigmoid", 1e-5, D ** -0.5, 1.0, gout[:B], 0, st, hf,
                                              slots, dq0, B, H, D, V, gates=(i_off, f_off, bias, bias, 15.0)))
    la = torch.exp(-torch.rand(T, H * D, device=dev) * 0.1)
    state = torch.zeros(B, H, D, V, device=dev)
    ss, sa = torch.empty(T // 64, H, D, V, device=dev), torch.empty(T // 64, H, D, device=dev)
    nv = torch.ones(V, device=dev)
    args_c = (gp, offs, la, nv, 1e-5, D ** -0.5, 0.9, gout, 0, state, slot0, q0, qn)

    def gla_chunked():
        ops.gla_scan(*args_c, items, T // 64, ops.GLA_LOCAL, ss, sa, H, D, V)
        ops.gla_chain(state, ss, sa, chains, 1, slot0, H, D, V)
        ops.gla_scan(*args_c, items, T // 64, ops.GLA_OUT, ss, sa, H, D, V)
    add("gla_scan: one 2048-token portion in chunks of 64 (like)", gla_chunked, flops=scan_flops)
    dqn = torch.ones(B, device=dev, dtype=torch.int32)
    add(f"gla_step: {B} single tokens (like)",
        lambda: ops.gla_step(gp[:B], offs, la[:B], nv, 1e-5, D ** -0.5, 0.9, gout[:B], 0, state, slots, dq0, B, H, D, V),
        nbytes=2 * B * H * D * V * 4)
    # attention with the distance table, a gate per head and a window: the tensor-core kernel of prompt portions beside
    # the same kernel without them and beside the tcgen05 kernel (what the closest model's prompt portions take); single
    # tokens in the general kernel beside the split-key decode kernel
    pages = T // PAGE
    cache = torch.randn(pages, 2, kv, PAGE, d, device=dev).to(torch.bfloat16)
    tbl = torch.arange(pages, device=dev, dtype=torch.int32).view(1, pages)
    ent = torch.zeros(T, device=dev, dtype=torch.int32)
    status = torch.zeros(2, dtype=torch.int32, device=dev)
    qa = torch.randn(T, heads * d, device=dev).to(torch.bfloat16)
    oa = torch.empty(T, heads * d, device=dev, dtype=torch.bfloat16)
    gate = torch.randn(T, heads, device=dev)
    window = 1024
    table = torch.randn(window, heads, device=dev)
    table_t = table.t().contiguous()
    tiles = torch.tensor([(0, r) for r in range(0, T, ops.PREFILL_TILE_ROWS)], device=dev, dtype=torch.int32)
    e_start, e_len = torch.zeros(1, device=dev, dtype=torch.int32), torch.full((1,), T, device=dev, dtype=torch.int32)
    walked = sum(min(p + 1, window) for p in range(T))
    attn_flops = 4.0 * heads * d * walked
    tensor_peak = pk.get("bf16_tflops", 1590.0) * 1e12

    def attn(name, fn):
        sec = timed(fn, 5, 3, flush)
        kernels[name] = {"us": round(sec * 1e6, 1), "tflops": round(attn_flops / sec / 1e12, 1),
                         "frac_of_bf16_peak": round(attn_flops / sec / tensor_peak, 4)}
    common = (cache, tiles, tiles.shape[0], slot0, e_start, e_len, e_len, tbl, heads, kv, d, PAGE, window, d ** -0.5, status)
    attn("prompt attention, distance table + head gate (new): 2048 tokens, window 1024",
         lambda: ops.paged_attention_prefill_biased(qa, oa, 0, *common, dist_bias_t=table_t, head_gate=gate))
    attn("prompt attention, the same mma.sync kernel without them (like)", lambda: ops.paged_attention_prefill(qa, oa, *common))
    if ops.prefill_tcgen05_supported(d, PAGE):
        attn("prompt attention, the tcgen05 kernel (like: what the closest model's prompt portions take)",
             lambda: ops.paged_attention_prefill_tcgen05(qa, oa, *common))
    Bd, ctx = 64, 1024
    dpages = ctx // PAGE
    dcache = torch.randn(Bd * dpages, 2, kv, PAGE, d, device=dev).to(torch.bfloat16)
    dtbl = torch.arange(Bd * dpages, device=dev, dtype=torch.int32).view(Bd, dpages)
    dpos = torch.full((Bd,), ctx - 1, device=dev, dtype=torch.int32)
    dent = torch.arange(Bd, device=dev, dtype=torch.int32)
    kv_bytes = Bd * ctx * 2 * kv * d * 2
    table_t2 = (table.t() * 1.4426950408889634).contiguous()
    a_dec = torch.empty(Bd, heads * d, device=dev, dtype=torch.bfloat16)

    def biased_decode():
        ops.paged_attention_decode(qa[:Bd], a_dec, dcache, None, Bd, dpos, dent, dent, dtbl, heads, kv, d, PAGE, window, d ** -0.5, 2,
                                   status, dist_bias_t=table_t2)
        ops.gate_mul(a_dec, gate[:Bd], 0, oa[:Bd], 0, "sigmoid", 1.0, per_head=d)
    add(f"decode attention, split-key kernel with the distance table, then the gate per head (new): {Bd} tokens, {ctx} keys each",
        biased_decode, nbytes=kv_bytes)
    add(f"decode attention, general kernel with distance table + head gate (new; the 32-bit mode and odd shapes): {Bd} tokens, {ctx} keys each",
        lambda: ops.paged_attention_generic_kv(qa[:Bd], dcache[:, 0], dcache[:, 1], dpos, dent, dent, dtbl, heads, kv, d, d, PAGE, window,
                                               d ** -0.5, status, oa[:Bd], 0, gate=gate[:Bd], dist_bias=table, gate_per_head=True),
        nbytes=kv_bytes)
    add("decode attention, split-key kernel (like: what the closest model's single tokens take)",
        lambda: ops.paged_attention_decode(qa[:Bd], oa[:Bd], dcache, None, Bd, dpos, dent, dent, dtbl, heads, kv, d, PAGE, window,
                                           d ** -0.5, 2, status), nbytes=kv_bytes)
    # routed experts: router, activation, and the kernels that read only the chosen experts
    E, top, fe = 8, 2, ff // 2
    x = torch.randn(T, width, device=dev).to(torch.bfloat16)
    wr = torch.randn(E, width, device=dev) * 0.02
    add("moe_route (new)", lambda: ops.moe_route(x, wr, top, (4, 2), 1.0), nbytes=T * (width * 2 + E * 4))
    gu = torch.randn(T, 2 * E * fe, device=dev)
    dense = ops.moe_route(x, wr, top, (4, 2), 1.0)
    add("moe_act (new: activation of the chosen experts' columns)", lambda: ops.moe_act(gu, dense, E, fe, 7.0, 1.702, torch.bfloat16),
        nbytes=T * (top * 2 * fe * 4 + E * fe * 2))
    gub = torch.randn(T, 2 * fe, device=dev).to(torch.bfloat16)
    add("silu_and_mul (like)", lambda: ops.silu_and_mul(gub), nbytes=T * fe * 6)
    wgu = (torch.randn(E * 2 * fe, width, device=dev) * 0.02).to(torch.bfloat16)
    wd = (torch.randn(width, E * fe, device=dev) * 0.02).to(torch.bfloat16)
    _, ids, wts = ops.moe_route(x[:1], wr, top, (4, 2), 1.0, lists=True)
    add("moe_sparse, one token (new: two kernels over the chosen experts' matrices)",
        lambda: ops.moe_sparse(x[:1], wgu, wd, ids, wts, fe, 7.0, 1.702), nbytes=top * 3 * fe * width * 2)
    wl = (torch.randn(3 * top * fe, width, device=dev) * 0.02).to(torch.bfloat16)
    add("streaming product of equal bytes, one token (like)", lambda: ops.linear(x[:1], wl, out_dtype=torch.float32),
        nbytes=top * 3 * fe * width * 2)
    print(json.dumps({"metric": "tokens/s of the Gubidra design beside Tobovik at equal sizes (bfloat16, random weights)",
                      "design": "gubidra", "prompt_tokens": 2048, "decode_context": 1024, "steps": args.steps,
                      "warmup": args.warmup, "sizes": sizes, "kernels_at_w4096": kernels,
                      "peaks": {"hbm_gbs": pk["hbm_gbs"], "fp32_fma_tflops_nominal": round(fp32_peak / 1e12, 1),
                                "source": pk["source"]},
                      "l2": "kernel timings: a 256 MB buffer is overwritten between launches; steps read every weight"}))
    return 0


def design_bench(args, pk) -> int:
    import torch
    from litellmengine_b200.config import config_from_dict
    from litellmengine_b200.csrc import ops
    from litellmengine_b200.csrc.microbench import Flusher, timed
    from litellmengine_b200.engine import ModelRunner, StepEntry
    torch.cuda.set_device(0)
    dev = "cuda:0"
    gen = torch.Generator().manual_seed(3)
    toks = lambda n: torch.randint(0, DESIGN_VOCAB, (n,), generator=gen).tolist()
    prompt_len, context, batches = 2048, 1024, (8, 32)
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def measure(config):
        runner = ModelRunner.from_config(config, seed=1, dtype="bfloat16", device=dev, page_size=PAGE,
                                         max_total_tokens=max(batches) * (context + 64) + prompt_len, max_requests=max(batches),
                                         max_tokens_per_step=prompt_len)
        rec, times = {}, []
        for i in range(args.warmup + 3):                       # one prompt in one step
            s = runner.admit()
            a, b = ev(), ev()
            a.record()
            runner.step([StepEntry(s, toks(prompt_len), [prompt_len - 1])])
            b.record()
            torch.cuda.synchronize()
            runner.release(s)
            if i >= args.warmup:
                times.append(a.elapsed_time(b))
        rec["prefill_2048_ms"] = round(sum(times) / len(times), 3)
        rec["prefill_2048_tok_s"] = round(prompt_len / (rec["prefill_2048_ms"] * 1e-3), 1)
        for B in batches:
            steps = args.steps
            slots = [runner.admit() for _ in range(B)]
            for s in slots:
                runner.step([StepEntry(s, toks(context - steps - args.warmup), [])])
            feed = [toks(B) for _ in range(steps + args.warmup)]
            torch.cuda.synchronize()
            for i in range(args.warmup):
                runner.step([StepEntry(s, [feed[i][j]], [0]) for j, s in enumerate(slots)])
            torch.cuda.synchronize()
            n0 = ops.launch_count
            a, b = ev(), ev()
            a.record()
            for i in range(args.warmup, args.warmup + steps):
                runner.step([StepEntry(s, [feed[i][j]], [0]) for j, s in enumerate(slots)])
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / steps
            state = sum(t[0].numel() * t.element_size() for k, t in runner.cache.state.items() if not isinstance(k, str))
            step_bytes = runner.model.weight_bytes() + B * (runner.cache.bytes_per_token() * (context - steps // 2) + 2 * state)
            rec[f"decode_b{B}_ms"] = round(ms, 4)
            rec[f"decode_b{B}_tok_s"] = round(B / (ms * 1e-3), 1)
            rec[f"decode_b{B}_hbm_frac"] = round(step_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
            rec[f"decode_b{B}_launches_per_step"] = (ops.launch_count - n0) // steps
            for s in slots:
                runner.release(s)
        runner.check_status()
        return rec

    if args.design == "gubidra":
        return gubidra_bench(args, pk, measure)
    if args.design == "komazen":
        return komazen_bench(args, pk, measure)
    if args.design == "vugedra":
        return vugedra_bench(args, pk, measure)
    sizes = {}
    for name, (width, ff, heads, kv, layers) in DESIGN_SIZES.items():
        if args.sizes and name not in args.sizes.split(","):
            continue
        qwen = dict(QWEN3_8B, num_hidden_layers=layers, hidden_size=width, num_attention_heads=heads, num_key_value_heads=kv,
                    head_dim=DESIGN_HEAD, intermediate_size=ff, vocab_size=DESIGN_VOCAB)
        sizes[name] = {"shape": {"width": width, "ff": ff, "heads": heads, "kv_heads": kv, "layers": layers, "vocab": DESIGN_VOCAB}}
        for label, cfg in (("tobovik", tobovik_dict(width, ff, heads, kv, layers)), ("qwen3", qwen)):
            sizes[name][label] = measure(config_from_dict(cfg))
            gc.collect()
            torch.cuda.empty_cache()
        t, q = sizes[name]["tobovik"], sizes[name]["qwen3"]
        sizes[name]["tobovik_over_qwen3"] = {k: round(t[k] / q[k], 3) for k in t if k.endswith("tok_s")}

    # the design's own kernels beside the like kernels of the Qwen3 path, at the largest size's widths
    flush = Flusher(dev)
    width, _, heads, kv, _ = DESIGN_SIZES["w4096"]
    T, hbm = prompt_len, pk["hbm_gbs"] * 1e9
    kernels = {}

    def add(name, fn, nbytes=None, flops=None, peak_flops=None):
        sec = timed(fn, 5, 3, flush)
        rec = {"us": round(sec * 1e6, 2)}
        if nbytes is not None:
            rec.update(gbs=round(nbytes / sec / 1e9, 1), frac_of_hbm=round(nbytes / sec / hbm, 4))
        if flops is not None:
            rec.update(tflops=round(flops / sec / 1e12, 2), frac_of_fp32_peak=round(flops / sec / peak_flops, 4))
        kernels[name] = rec

    h = torch.randn(T, width, device=dev)
    y = torch.randn(T, width, device=dev)
    w = torch.ones(width, device=dev)
    add("rmsnorm_add (new: norm of a branch output + residual add + copy)", lambda: ops.rmsnorm_add(h, y, w, 1e-5, torch.bfloat16),
        nbytes=T * width * (4 + 4 + 4 + 2))
    add("rmsnorm (like: residual add + norm)", lambda: ops.rmsnorm(h, w, 1e-5, torch.bfloat16, delta=y, write_sum=True),
        nbytes=T * width * (4 + 4 + 4 + 2))
    ids = torch.randint(0, DESIGN_VOCAB, (T,), device=dev, dtype=torch.int32)
    table = torch.randn(DESIGN_VOCAB, width, device=dev).to(torch.bfloat16)
    pos = torch.arange(T, device=dev, dtype=torch.int32)
    status = torch.zeros(2, dtype=torch.int32, device=dev)
    inv = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * torch.arange(width // 2, dtype=torch.float64) / width).to(dev)
    add("embedding_sinusoid (new)", lambda: ops.embedding_sinusoid(ids, table, pos, inv, status, copy_dtype=torch.bfloat16),
        nbytes=T * width * (2 + 4 + 2))
    add("embedding (like)", lambda: ops.embedding(ids, table, status), nbytes=T * width * (2 + 4))
    d = DESIGN_HEAD
    pages = T // PAGE
    proj = torch.randn(T, (heads + 2 * kv) * d + heads * d, device=dev)
    cache = torch.zeros(pages, 2, kv, PAGE, d, device=dev, dtype=torch.bfloat16)
    tbl = torch.arange(pages, device=dev, dtype=torch.int32).view(1, pages)
    ent, slot0 = torch.zeros(T, device=dev, dtype=torch.int32), torch.zeros(1, device=dev, dtype=torch.int32)
    bq, bk, bv = (torch.zeros(n * d, device=dev) for n in (heads, kv, kv))
    qw, kw = torch.ones(heads * d, device=dev), torch.ones(kv * d, device=dev)
    prep_bytes = T * ((heads + 2 * kv) * d * 4 + (heads + 2 * kv) * d * 2)
    add("attention_prepare (new: bias, projection norm, temperature, page write)",
        lambda: ops.attention_prepare(proj, 0, heads * d, (heads + kv) * d, (bq, bk, bv), qw, kw, "projection", 1e-5, (0.25, 256),
                                      cache[:, 0], cache[:, 1], pos, ent, slot0, tbl, heads, kv, d, d, PAGE, status, torch.bfloat16),
        nbytes=prep_bytes)
    qkv = proj[:, :(heads + 2 * kv) * d].contiguous()
    hw = torch.ones(d, device=dev)
    invf = torch.pow(torch.tensor(1e6), -torch.arange(0, d, 2, dtype=torch.float32) / d).to(dev)
    add("qk_norm_rope_kv_write (like: head norm, rotation, page write)",
        lambda: ops.qk_norm_rope_kv_write(qkv, cache, pos, ent, slot0, tbl, hw, hw, 1e-6, invf, d, heads, kv, d, PAGE, True, status,
                                          q_dtype=torch.bfloat16), nbytes=prep_bytes)
    a_out = torch.randn(T, heads * d, device=dev).to(torch.bfloat16)
    gate = torch.randn(T, heads * d, device=dev)
    out = torch.empty(T, heads * d, device=dev, dtype=torch.bfloat16)
    add("gate_mul (new: output gate)", lambda: ops.gate_mul(a_out, gate, 0, out, 0, "sigmoid", 0.8), nbytes=T * heads * d * (2 + 4 + 2))
    gu = torch.randn(T, 2 * heads * d, device=dev).to(torch.bfloat16)
    add("silu_and_mul (like)", lambda: ops.silu_and_mul(gu), nbytes=T * heads * d * (2 + 2 + 2))
    # the recurrence: prompt portion (chunks side by side) and single decoded tokens
    H, D, V = heads // 4, d, d
    gp = torch.randn(T, 2 * H * D + 2 * H * V, device=dev)
    la = torch.exp(-torch.rand(T, H * D, device=dev) * 0.1)          # the decays
    nw = torch.ones(V, device=dev)
    offs = (0, H * D, 2 * H * D, 2 * H * D + H * V)
    gout = torch.empty(T, H * V, device=dev, dtype=torch.bfloat16)
    B = 64
    state = torch.zeros(B, H, D, V, device=dev)
    items = torch.tensor([(0, c, 64, i) for i, c in enumerate(range(0, T, 64))], device=dev, dtype=torch.int32)
    chains = torch.tensor([(0, 0, T // 64)], device=dev, dtype=torch.int32)
    ss, sa = torch.empty(T // 64, H, D, V, device=dev), torch.empty(T // 64, H, D, device=dev)
    q0, qn = torch.zeros(1, device=dev, dtype=torch.int32), torch.full((1,), T, device=dev, dtype=torch.int32)
    args_c = (gp, offs, la, nw, 1e-5, D ** -0.5, 0.9, gout, 0, state, slot0, q0, qn)

    def chunked():
        ops.gla_scan(*args_c, items, T // 64, ops.GLA_LOCAL, ss, sa, H, D, V)
        ops.gla_chain(state, ss, sa, chains, 1, slot0, H, D, V)
        ops.gla_scan(*args_c, items, T // 64, ops.GLA_OUT, ss, sa, H, D, V)
    props = torch.cuda.get_device_properties(0)
    fp32_peak = props.multi_processor_count * 128 * 2 * 1.965e9
    add("gla_scan, one 2048-token portion in chunks of 64 (new; 32-bit recurrence on CUDA cores)", chunked,
        flops=T * H * D * V * (2 + 2 + 2), peak_flops=fp32_peak)
    slots = torch.arange(B, device=dev, dtype=torch.int32)
    dq0, dqn = torch.arange(B, device=dev, dtype=torch.int32), torch.ones(B, device=dev, dtype=torch.int32)
    args_d = (gp[:B], offs, la[:B], nw, 1e-5, D ** -0.5, 0.9, gout[:B], 0, state, slots, dq0, dqn)
    add(f"gla_step, {B} single tokens (new: the decode kernel; reads and writes each state once)",
        lambda: ops.gla_step(*args_d[:-1], B, H, D, V), nbytes=2 * B * H * D * V * 4)
    add(f"gla_scan, {B} single tokens (new: the general kernel on the same work)",
        lambda: ops.gla_scan(*args_d, None, B, ops.GLA_FULL, None, None, H, D, V), nbytes=2 * B * H * D * V * 4)
    print(json.dumps({"metric": "tokens/s of the Tobovik design beside Qwen3 at equal sizes (bfloat16, random weights)",
                      "design": "tobovik", "prompt_tokens": prompt_len, "decode_context": context, "steps": args.steps,
                      "warmup": args.warmup, "sizes": sizes, "kernels_at_w4096": kernels,
                      "peaks": {"hbm_gbs": pk["hbm_gbs"], "fp32_fma_tflops_nominal": round(fp32_peak / 1e12, 1),
                                "source": pk["source"]},
                      "l2": "kernel timings: a 256 MB buffer is overwritten between launches; steps read every weight"}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--points", default=",".join(ALL_POINTS),
                    help="which extra measurements to take: " + ",".join(ALL_POINTS))
    ap.add_argument("--no-points", action="store_true", help="the headline, prefill and e2e only")
    ap.add_argument("--design", choices=["tobovik", "gubidra", "komazen", "vugedra"],
                    help="instead of the default workload: this design beside its closest model (tobovik and komazen beside "
                         "Qwen3, gubidra beside tobovik, vugedra beside gubidra) at equal sizes, and its kernels")
    ap.add_argument("--sizes", default="", help="with --design: which of " + ",".join(DESIGN_SIZES) + " (default: all)")
    args = ap.parse_args()

    if args.gpus != 1:
        print(json.dumps({"error": f"this engine runs on one GPU; --gpus {args.gpus} is not built", "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return reference_arm(args)
    want_points = set() if args.no_points else {p for p in args.points.split(",") if p}
    unknown = want_points - set(ALL_POINTS)
    if unknown:
        ap.error(f"unknown points {sorted(unknown)}; choose from {ALL_POINTS}")

    pk = peaks()
    if args.design:
        return design_bench(args, pk)
    bench = Bench(args, pk)
    points = {}
    main_rec = bench.qwen3_8b(want_points, points)
    head, check = main_rec["head"], main_rec["check"]
    if not check["ok"]:
        print(json.dumps({"error": "the last timed decode step's logits differ from the same positions run as "
                                   "whole prompts", "rms_error": check["rms"], "allowed_rms": check["allowed_rms"],
                          "max_error": check["max"], "largest_logit": check["scale"]}))
        return 1
    bench.free_memory()
    for name, fn in (("long", bench.qwen3_8b_long), ("fp32", bench.qwen3_8b_fp32), ("0p6b", bench.qwen3_0p6b), ("32b", bench.qwen3_32b)):
        if name in want_points:
            fn(points)
            bench.free_memory()

    bad = [k for k, v in points.items() if isinstance(v, dict) and v.get("ok") is False]
    if bad:
        print(json.dumps({"error": "decode steps differ from the same positions run as whole prompts",
                          **{k: points[k] for k in bad}}))
        return 1

    out = {
        "metric": "decode tokens/s (Qwen3-8B shape, batch %d, context %d)" % (args.batch, CONTEXT),
        "value": round(head["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(head["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights, uniform-random token ids)",
        "config": shape_config(QWEN3_8B, args.layers, args.batch, CONTEXT, model="Qwen3-8B shape",
                               l2="inputs larger than L2 (the step reads every weight)"),
        "prefill": main_rec["prefill"],
        "roofline": {"bound": "hbm", "achieved": round(head["gbs"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(head["frac"], 4), "peak_source": pk["source"]},
        "points": points, "e2e": main_rec["e2e"], "gpu_launches": head["launches"],
        "checked": True, "check": {"rms_err": round(check["rms"], 5), "allowed_rms": round(check["allowed_rms"], 5),
                                   "max_err": round(check["max"], 5), "largest_logit": round(check["scale"], 3)},
        "clocks": head["clocks"],
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
