#!/usr/bin/env python3
"""Measures generation of the Qwen2.5 shapes with random bf16 weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--model-size 7b|14b|32b] [--layers L] [--impl ours|reference]

One JSON line on stdout.  With the default --model-size 7b, `value` is decoded tokens per
second at batch 8 (prompts of 1,024 random token ids, slots of 8,192 tokens), timed on
the device with CUDA events around exactly K decode steps after W warm-up steps, every
step between events of its own (`latency_ms`: p50 and p95 of a step).  `e2e` is the same
through the public entry point (Engine.generate: host token ids in, host token ids out,
every step with its host-to-device copy of inputs from pinned memory and its
device-to-host read of the chosen tokens), from the first decoded token on, with the
figure after the clock has settled beside it.  `prefill` is one prompt of 2,048 tokens;
`points` holds decoding at batch 1 and 64, 256 steps at batch 8, and batch 64 with
contexts of 8,000 tokens (the attention-bound end); `roofline` relates the bytes a decode
step must read (every weight once, the cache of the live requests) to its time.
--model-size 14b runs that shape's workload (16 prompts of lengths uniform in [64, 2048],
seed 3, 128 greedy steps, slots of 4,096 tokens), 32b its own (a 2,048-token prompt;
decoding at batch 1 and 32, slots of 4,096 tokens, seed 4); each line has its own roofline.
The generated tokens of two runs of the same requests are compared; a difference ends the
program with status 1 (the reference's bench tool does the same: friday_bench.cpp:237-310).

Every decode step reads all weights (15 GB at the 7B shape), far more than the 126 MB
L2, so consecutive timed steps cannot be served from L2.

The model is the library's own architecture built from a config.json dictionary with
random weights drawn on the device; nothing is loaded from disk.  --layers runs fewer
layers of the same sizes (both numbers are reported).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN25_7B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 28, "hidden_size": 3584,
    "num_attention_heads": 28, "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 18944,
    "vocab_size": 152064, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "use_sliding_window": False, "max_position_embeddings": 32768, "torch_dtype": "bfloat16",
}
QWEN25_14B = dict(QWEN25_7B, num_hidden_layers=48, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                  intermediate_size=13824, rms_norm_eps=1e-5)
QWEN25_32B = dict(QWEN25_14B, num_hidden_layers=64, intermediate_size=27648)
SHAPES = {"7b": QWEN25_7B, "14b": QWEN25_14B, "32b": QWEN25_32B}
CONTEXT, PROMPT, PREFILL_TOKENS = 8192, 1024, 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        flat = {}

        def walk(x):
            if isinstance(x, dict):
                for k, v in x.items():
                    if isinstance(v, (int, float)):
                        flat.setdefault(k, float(v))
                    else:
                        walk(v)
        walk(d)
        return {"hbm_gbs": flat["hbm_gbs"], "bf16_tflops": flat["bf16_tflops"],
                "bf16_tflops_sustained": flat.get("bf16_tflops_sustained"), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return dict(FALLBACK_PEAKS)


class Clocks:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows for n, v in zip(names, r[2:6]) if v.lower() == "active"})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def model_numbers(cfg, layers):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    qd = cfg["num_attention_heads"] * cfg["head_dim"]
    kvd = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (qd + 2 * kvd) * h + (qd + 2 * kvd) + h * qd + 2 * i * h + h * i + 2 * h
    weights = layers * per_layer + v * h + h                 # parameters a decode step reads (head, not the table)
    return {"step_weight_bytes": 2 * weights, "kv_bytes_per_token": 2 * 2 * kvd * layers,
            "matmul_params": layers * ((qd + 2 * kvd) * h + h * qd + 3 * i * h), "head_params": v * h}


def random_prompts(n, length, vocab, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]


def fill(eng, prompts, group=8):
    """Slots holding the prompts (prompts in groups: bounds the working memory of a pass)."""
    slots = [eng.alloc_slot() for _ in prompts]
    for lo in range(0, len(prompts), group):
        eng.step(slots[lo:lo + group], prompts[lo:lo + group], [[]] * len(slots[lo:lo + group]))
    return slots


def percentile(values, q):
    v = sorted(values)
    return v[min(len(v) - 1, int(round(q * (len(v) - 1))))]


E2E_SETTLE_STEPS = SETTLE_STEPS = 32


def time_decode(eng, prompts, steps, warmup):
    """Device time of `steps` decode steps after the prompts; tokens stay on the device.  Every step lies between two
    events on the engine's stream.  Returns (ms per step, launches, mean context, per-step ms)."""
    import torch
    slots = fill(eng, prompts)
    dec = eng.decoder(slots, [p[-1] for p in prompts])       # decoding that stays on the device
    # The prompts drive the GPU into its power cap; the SM clock needs some 15 of the much lighter decode steps to come
    # back.  SETTLE_STEPS untimed steps come before the warm-up steps, so that the timed ones are decoding as it runs
    # from then on (generation from the first token on, slow start included, is the e2e figure).
    for _ in range(SETTLE_STEPS + warmup):
        dec.step()
    stream = eng.stream
    stream.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    launches0 = eng.launches
    with torch.cuda.stream(stream):
        marks[0].record()
        for i in range(steps):
            dec.step()
            marks[i + 1].record()
    stream.synchronize()
    ms = marks[0].elapsed_time(marks[-1])
    per_step = [marks[i].elapsed_time(marks[i + 1]) for i in range(steps)]
    launches = eng.launches - launches0
    mean_len = sum(len(p) for p in prompts) / len(prompts) + SETTLE_STEPS + warmup + steps / 2.0
    dec.close()
    for s in slots:
        eng.free_slot(s)
    eng.check()
    return ms / steps, launches, mean_len, per_step


def time_e2e(eng, prompts, steps):
    """Engine.generate with host tokens in and out: every decode step copies its token ids in from pinned memory and
    the chosen ids out.  Returns tokens/s over the first `steps` decode steps, over the last `steps` ones, and whether
    two runs of the same requests chose the same tokens.

    The first decode steps after the prompts run slower than the rest: 8 x 1,024 prompt tokens drive the GPU into its
    power cap, and the SM clock needs some 15 steps of the much lighter decoding to come back.  The device-timed value
    does not see this (graph capture sits between its prompts and its timed steps); here the figure from the first
    token on leads, and the one after E2E_SETTLE_STEPS steps stands beside it."""
    marks = []

    def on_step(live, drawn):
        marks.append(time.perf_counter())

    batch = len(prompts)
    eng.generate(prompts, max_new_tokens=4, temperature=0.0, ignore_eos=True)       # warm-up: captures the step
    total = E2E_SETTLE_STEPS + steps
    runs = []
    for _ in range(2):
        marks.clear()
        out = eng.generate(prompts, max_new_tokens=total + 1, temperature=0.0, ignore_eos=True, on_step=on_step)
        assert all(len(g.tokens) == total + 1 for g in out)
        runs.append(([g.tokens for g in out], batch * steps / (marks[steps] - marks[0]),
                     batch * steps / (marks[-1] - marks[-1 - steps])))
    same = runs[0][0] == runs[1][0]
    return max(r[1] for r in runs), max(r[2] for r in runs), same


def time_prefill(eng, tokens, warmup, reps, seed=99):
    """Median device time of one prompt of `tokens` tokens through Engine.step, and the host's share: the wall time
    of the call until its launches are queued is what the host costs when the device is the faster of the two."""
    import torch
    (p,) = random_prompts(1, tokens, eng.vocab_size, seed)
    times = []
    stream = eng.stream
    for r in range(warmup + reps):
        s = eng.alloc_slot()
        stream.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            a.record()
            eng.step([s], [p], [[tokens - 1]])
            b.record()
        stream.synchronize()
        if r >= warmup:
            times.append(a.elapsed_time(b))
        eng.free_slot(s)
    return sorted(times)[len(times) // 2]


def host_ms_per_pass(eng, tokens=512):
    """Host time of one pass over all layers: from the call of the step function to the moment its last launch is
    queued (read from the engine), for a prompt long enough that the device is the slower of the two."""
    (p,) = random_prompts(1, tokens, eng.vocab_size, 98)
    best = 1e9
    for _ in range(4):
        s = eng.alloc_slot()
        eng.step([s], [p], [[tokens - 1]])
        best = min(best, eng.stats()["last_queue_ms"])
        eng.free_slot(s)
    return best


def timeline(eng, batch):
    """Kernels of the last of three profiled decode steps: name, start, duration, and `real`, the time from the end
    of the kernel before to the end of this one (kernels overlap under programmatic dependent launch)."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    prompts = random_prompts(batch, PROMPT, eng.vocab_size, 1)
    slots = fill(eng, prompts)
    dec = eng.decoder(slots, [p[-1] for p in prompts])
    for _ in range(5):
        dec.step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            dec.step()
        torch.cuda.synchronize()
    evs = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                 key=lambda e: e.time_range.start)
    last = evs[-(len(evs) // 3):]
    t0 = prev_end = last[0].time_range.start
    for e in last:
        st, en = e.time_range.start, e.time_range.end
        print("%-64s start %8.1f us  duration %7.1f us  real %7.1f us" % (e.name[:64], st - t0, en - st, en - max(prev_end, st) if st < prev_end else en - st))
        prev_end = max(prev_end, en)
    print("step: %.1f us, %d kernels" % (prev_end - t0, len(last)))
    return 0


def cta_trace(eng, batch):
    """Where the CTAs of a decode step's products and attention kernels spend their time: %globaltimer stamps that
    the kernels write when given a trace buffer (csrc/gemm_tc_fusion.h part 4, attention_mma_set_trace), read after
    one replay of the captured step.  Times in us from the step's first stamp; min / median / max over CTAs."""
    import numpy as np
    import torch
    from friday_inference_engine_b200.ops import lib
    info = eng.info()
    layers, sms = info["n_layers"], info["sm_count"]
    prompts = random_prompts(batch, PROMPT, eng.vocab_size, 1)
    slots = fill(eng, prompts)
    dec = eng.decoder(slots, [p[-1] for p in prompts])
    dec.step()                                                # eager: sizes the working memory, loads the libraries
    n_gemm = 4 * layers + 1
    trace = torch.zeros((n_gemm, sms, 16), dtype=torch.int64, device="cuda:0")
    eng.set_trace(trace)
    attn = torch.zeros((8192, 8), dtype=torch.int64, device="cuda:0")
    set_trace = lib.family("attention_mma").declare("attention_mma_set_trace", [lib.P])
    set_trace(attn.data_ptr())
    dec.step()                                                # captured with the trace pointers in place
    for _ in range(5):
        dec.step()
    torch.cuda.synchronize()
    trace.zero_()
    attn.zero_()
    dec.step()
    torch.cuda.synchronize()
    set_trace(None)
    eng.set_trace(None)
    g = trace.cpu().numpy().astype(np.float64)
    a = attn.cpu().numpy().astype(np.float64)
    g[g == 0] = np.nan
    a[a == 0] = np.nan
    t0 = np.nanmin(g)

    def stats(col):
        col = (col - t0) / 1000.0
        return "%6.1f %6.1f %6.1f" % (np.nanmin(col), np.nanmedian(col), np.nanmax(col))

    names = ["qkv", "o", "gate_up", "down"]
    print("products: CTAs | set-up done | predecessor finished | first operands landed | last accumulator complete | "
          "last tile done   (min median max, us)")
    for i in range(n_gemm):
        name = names[i % 4] + " %d" % (i // 4) if i < 4 * layers else "head"
        print("%-10s %4d | %s | %s | %s | %s | %s" % (name, int(np.sum(~np.isnan(g[i, :, 0]))), stats(g[i, :, 1]),
                                                      stats(g[i, :, 3]), stats(g[i, :, 4]), stats(g[i, :, 6]), stats(g[i, :, 7])))
    print("CTAs that sum a tile's split-k partial tiles, us after their own last accumulator: knows it is last | "
          "partial tiles summed | tile transposed | tile written   (median, max)")
    for i in range(n_gemm):
        sel = ~np.isnan(g[i, :, 8])
        if sel.any():
            rel = (g[i, sel][:, [8, 10, 11, 12]] - g[i, sel][:, [6]]) / 1000.0
            print("%-10s %4d | " % (names[i % 4] + " %d" % (i // 4), sel.sum())
                  + " | ".join("%5.2f %5.2f" % (np.nanmedian(rel[:, j]), np.nanmax(rel[:, j])) for j in range(4)))
    # the attention launch that wrote last is the last layer's; its predecessor is that layer's qkv product
    done = np.nanmax(g[4 * (layers - 1), :, 7])
    live = ~np.isnan(a[:, 0])
    print("attention of the last layer: %d CTAs; us after the qkv product's last tile (min median max); the o product's "
          "predecessor finished at %.1f" % (live.sum(), (np.nanmin(g[4 * (layers - 1) + 1, :, 3]) - done) / 1000.0))
    for j, what in enumerate(["kernel entry", "predecessor finished", "loads issued", "first block landed", "blocks done",
                              "warps merged", "cluster barrier passed", "splits merged"]):
        col = (a[live, j] - done) / 1000.0
        print("  %-24s %6.1f %6.1f %6.1f" % (what, np.nanmin(col), np.nanmedian(col), np.nanmax(col)))
    dec.close()
    for s in slots:
        eng.free_slot(s)

    # the prompt attention of the last layer: where the thread of a CTA's first row and the thread that issues the
    # products spend the time of a block of keys
    (p,) = random_prompts(1, PREFILL_TOKENS, eng.vocab_size, 99)
    for _ in range(2):
        s = eng.alloc_slot()
        eng.step([s], [p], [[PREFILL_TOKENS - 1]])
        eng.free_slot(s)
    tc = torch.zeros((4096, 16), dtype=torch.int64, device="cuda:0")
    set_tc = lib.family("attention_tc").declare("attention_tc_set_trace", [lib.P])
    set_tc(tc.data_ptr())
    s = eng.alloc_slot()
    eng.step([s], [p], [[PREFILL_TOKENS - 1]])
    torch.cuda.synchronize()
    set_tc(None)
    eng.free_slot(s)
    t = tc.cpu().numpy().astype(np.float64)
    t = t[t[:, 5] > 0]
    blocks = t[:, 5].sum()
    # (with two row tiles per CTA a block is 128 keys, the rows' figures are the first tile's, the issuer's both tiles')
    print("prompt attention, %d tokens: %d CTAs, %d blocks; us per block: " % (PREFILL_TOKENS, len(t), blocks)
          + ", ".join("%s %.2f" % (what, t[:, k].sum() / blocks / 1000.0) for k, what in
                      ((0, "row waits for S"), (1, "reads S, maximum"), (2, "exponentials and P"), (3, "rescales O"),
                       (4, "waits for the last product"), (8, "issuer waits for K"), (9, "issues Q K^T"),
                       (10, "waits for V"), (11, "waits for P"), (12, "issues P V")))
          + "; kernel %.1f us" % (((t[:, 7] + t[:, 6]).max() - t[:, 7].min()) / 1000.0))
    return 0


def reference_arm():
    why = ("the reference runs one sequence at a time with GGUF k-quant weights and int8 activations (engine.h:46-54: "
           "step(token, pos) and prefill(tokens, n, pos) have no batch dimension; no bf16 or fp16 weight path), so the "
           "metric's configuration (bf16 weights, batch 8) cannot be run through its stock code path; its CPU library "
           "builds here with CMake and anchors the tests under tests/golden/, its CUDA path was not run")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def roofline(step_bytes, ms_step, pk):
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
            "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]}


def prefill_record(cfg, layers, nums, tokens, ms, pk):
    flops = 2.0 * tokens * nums["matmul_params"] + 2.0 * nums["head_params"]
    qd = cfg["num_attention_heads"] * cfg["head_dim"]
    flops += layers * 4.0 * qd * tokens * tokens / 2.0
    return {"value": round(tokens * 1000.0 / ms, 1), "tokens": tokens, "ms": round(ms, 3),
            "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}


def base_line(metric, value, args, ms_step, launches, clk, roof, cfg, layers, full_layers, batch, context, prompt, pk, per_step):
    return {
        "metric": metric, "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "impl": "ours", "gpu_launches": int(launches), "clocks": clk, "roofline": roof,
        "latency_ms": {"p50": round(percentile(per_step, 0.5), 4), "p95": round(percentile(per_step, 0.95), 4)},
        "config": {"model": "Qwen2.5-%s shape, random weights" % args.model_size.upper(), "global_batch": batch,
                   "seq_len": context, "prompt_len": prompt, "parallelism": "none", "layers_run": layers,
                   "layers_full": full_layers, "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "l2": "every step reads all weights (>> 126 MB L2)", "peaks": pk["source"],
                   "settle_steps": SETTLE_STEPS},
    }


def run_7b(eng, args, cfg, layers, full_layers, nums, pk):
    clocks = Clocks()
    clocks.start()
    prompts = random_prompts(args.batch, PROMPT, eng.vocab_size, 1)
    ms_step, launches, mean_len, per_step = time_decode(eng, prompts, args.steps, args.warmup)
    clk = clocks.stop()
    step_bytes = nums["step_weight_bytes"] + args.batch * mean_len * nums["kv_bytes_per_token"]
    line = base_line("Qwen2.5-7B bf16 decode tok/s at batch %d" % args.batch, args.batch * 1000.0 / ms_step, args, ms_step,
                     launches, clk, roofline(step_bytes, ms_step, pk), cfg, layers, full_layers, args.batch, CONTEXT,
                     PROMPT, pk, per_step)
    same = True
    if not args.skip_points:
        # The prompt and the end-to-end figure come first, after a pause: both run at the power cap, and what the GPU
        # has just been doing decides the clock they meet (the long-context point below leaves it hot).
        time.sleep(2.0)
        line["prefill"] = prefill_record(cfg, layers, nums, PREFILL_TOKENS, time_prefill(eng, PREFILL_TOKENS, 2, 5), pk)
        line["host"] = {"ms_per_pass": round(host_ms_per_pass(eng), 3),
                        "prefill_512_ms": round(time_prefill(eng, 512, 2, 3, seed=97), 3)}
        time.sleep(1.0)
        first, settled, same = time_e2e(eng, prompts, min(args.steps, 64))
        # every decode step of generate() copies the step's token ids in from pinned memory and the chosen ids out
        line["e2e"] = {"value": round(first, 1), "unit": "tokens/s", "h2d_bytes_per_step": 4 * args.batch,
                       "d2h_bytes_per_step": 4 * args.batch, "from": "first decoded token",
                       "after_settle_steps": E2E_SETTLE_STEPS, "settled": round(settled, 1),
                       "two_runs_same_tokens": same}
        steps_pt = max(8, args.steps // 2)
        points = {}
        for b in (1, 64):
            ms_b, _, _, _ = time_decode(eng, random_prompts(b, PROMPT, eng.vocab_size, 2 + b), steps_pt, args.warmup)
            points["decode_b%d" % b] = round(b * 1000.0 / ms_b, 1)
        ms_b, _, _, _ = time_decode(eng, prompts, 256, args.warmup)          # the 256 steps the workload names
        points["decode_b8_256_steps"] = round(args.batch * 1000.0 / ms_b, 1)
        if args.slots >= 64:
            # the attention-bound end: 64 sequences of 8,000 tokens (30 GB of keys and values per step)
            long_prompts = random_prompts(64, CONTEXT - 192, eng.vocab_size, 70)
            ms_b, _, mean_b, _ = time_decode(eng, long_prompts, steps_pt, args.warmup)
            points["decode_b64_ctx8000"] = round(64 * 1000.0 / ms_b, 1)
            points["decode_b64_ctx8000_hbm_frac"] = roofline(
                nums["step_weight_bytes"] + 64 * mean_b * nums["kv_bytes_per_token"], ms_b, pk)["frac"]
        line["points"] = points
    print(json.dumps(line))
    return 0 if same else 1


def run_14b(eng, args, cfg, layers, full_layers, nums, pk):
    """16 prompts of lengths uniform in [64, 2048] (seed 3), 128 greedy decode steps, slots of 4,096 tokens."""
    import torch
    g = torch.Generator().manual_seed(3)
    lens = torch.randint(64, 2049, (16,), generator=g).tolist()
    prompts = [torch.randint(0, eng.vocab_size, (n,), generator=g).tolist() for n in lens]
    steps = args.steps if args.steps_given else 128
    args.steps = steps
    clocks = Clocks()
    clocks.start()
    ms_step, launches, mean_len, per_step = time_decode(eng, prompts, steps, args.warmup)
    clk = clocks.stop()
    step_bytes = nums["step_weight_bytes"] + 16 * mean_len * nums["kv_bytes_per_token"]
    line = base_line("Qwen2.5-14B bf16 decode tok/s, 16 unequal prompts", 16 * 1000.0 / ms_step, args, ms_step, launches, clk,
                     roofline(step_bytes, ms_step, pk), cfg, layers, full_layers, 16, 4096, int(sum(lens) / 16), pk, per_step)
    line["config"]["prompt_lens"] = "uniform in [64, 2048], seed 3: %d..%d" % (min(lens), max(lens))
    # the prompts themselves, as one batch of unequal lengths, through the step function
    stream = eng.stream
    times = []
    for _ in range(3):
        slots = [eng.alloc_slot() for _ in prompts]
        stream.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            a.record()
            eng.step(slots, prompts, [[n - 1] for n in lens])
            b.record()
        stream.synchronize()
        times.append(a.elapsed_time(b))
        for s in slots:
            eng.free_slot(s)
    ms = sorted(times)[1]
    line["prefill"] = {"value": round(sum(lens) * 1000.0 / ms, 1), "tokens": sum(lens), "ms": round(ms, 3),
                       "frac": round(2.0 * sum(lens) * nums["matmul_params"] / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                       "note": "16 unequal prompts in one step; products only in the flops"}
    runs = []
    for _ in range(2):
        t0 = time.perf_counter()
        out = eng.generate(prompts, max_new_tokens=steps, temperature=0.0, ignore_eos=True)
        runs.append(([g.tokens for g in out], time.perf_counter() - t0))
    same = runs[0][0] == runs[1][0]
    line["e2e"] = {"value": round(16 * steps / min(r[1] for r in runs), 1), "unit": "tokens/s",
                   "h2d_bytes_per_step": 64, "d2h_bytes_per_step": 64, "from": "request in to last token out, prompts included",
                   "two_runs_same_tokens": same}
    print(json.dumps(line))
    return 0 if same else 1


def run_32b(eng, args, cfg, layers, full_layers, nums, pk):
    """A 2,048-token prompt at batch 1, then decoding at batch 1 and 32 with slots of 4,096 tokens (seed 4)."""
    clocks = Clocks()
    clocks.start()
    prompts = random_prompts(32, PROMPT, eng.vocab_size, 4)
    ms_step, launches, mean_len, per_step = time_decode(eng, prompts, args.steps, args.warmup)
    clk = clocks.stop()
    step_bytes = nums["step_weight_bytes"] + 32 * mean_len * nums["kv_bytes_per_token"]
    line = base_line("Qwen2.5-32B bf16 decode tok/s at batch 32", 32 * 1000.0 / ms_step, args, ms_step, launches, clk,
                     roofline(step_bytes, ms_step, pk), cfg, layers, full_layers, 32, 4096, PROMPT, pk, per_step)
    ms1, _, mean1, _ = time_decode(eng, prompts[:1], max(8, args.steps // 2), args.warmup)
    line["points"] = {"decode_b1": round(1000.0 / ms1, 1),
                      "decode_b1_hbm_frac": roofline(nums["step_weight_bytes"] + mean1 * nums["kv_bytes_per_token"], ms1, pk)["frac"]}
    line["prefill"] = prefill_record(cfg, layers, nums, PREFILL_TOKENS, time_prefill(eng, PREFILL_TOKENS, 1, 3, seed=4), pk)
    runs = []
    for _ in range(2):
        out = eng.generate(prompts[:4], max_new_tokens=24, temperature=0.0, ignore_eos=True)
        runs.append([g.tokens for g in out])
    same = runs[0] == runs[1]
    line["two_runs_same_tokens"] = same
    print(json.dumps(line))
    return 0 if same else 1


def sweeps(Engine, args):
    """Decode steps and prompts away from the headline's sizes (same timing functions), one line of text each."""
    cfg = dict(SHAPES[args.model_size])
    layers = args.layers or cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers
    cases = [tuple(int(v) for v in c.split("x")) for c in args.decode_sweep.split(",") if c]
    lengths = [int(v) for v in args.prompt_sweep.split(",") if v]
    longest = max([c + 64 + SETTLE_STEPS for _, c in cases] + lengths + [1024])
    context = (longest + 1023) // 1024 * 1024
    tokens = max([b * (c + 128) for b, c in cases] + lengths + [1024]) + 4096
    batch = max([b for b, _ in cases] + [1])
    options = {"prefill_chunk": args.prefill_chunk} if args.prefill_chunk else {}
    eng = Engine(config=cfg, seed=0, dtype="bfloat16", max_ctx=context, max_batch=batch, max_tokens=tokens, **options)
    print("[bench] %s" % eng.summary(), file=sys.stderr, flush=True)
    pk = peaks()
    nums = model_numbers(cfg, layers)
    for length in lengths:
        ms = time_prefill(eng, length, 1, 3)
        rec = prefill_record(cfg, layers, nums, length, ms, pk)
        print("prompt of %6d tokens: %8.1f ms, %8.1f tok/s, %.3f of the %s bf16 peak" % (length, ms, rec["value"], rec["frac"], pk["source"]),
              flush=True)
    for b, c in cases:
        prompts = random_prompts(b, c, eng.vocab_size, 3)
        ms, _, mean_len, _ = time_decode(eng, prompts, min(args.steps, 32), args.warmup)
        step_bytes = nums["step_weight_bytes"] + nums["kv_bytes_per_token"] * mean_len * b
        print("decode, %2d sequences of %5d tokens: %.3f ms per step, %8.1f tok/s, %.3f of the %s HBM roofline" % (
            b, c, ms, b * 1000.0 / ms, step_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], pk["source"]), flush=True)
    eng.check()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--model-size", default="7b", choices=sorted(SHAPES), dest="model_size",
                    help="which shape and workload: 7b (the headline line), 14b, 32b")
    ap.add_argument("--layers", type=int, default=0, help="run this many layers of the same sizes (0: all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true", help="leave out the points, prefill and e2e")
    ap.add_argument("--prefill-only", action="store_true", help="time the 2,048-token prompt only (for profiling)")
    ap.add_argument("--slots", type=int, default=0, help="sequences the cache is sized for (smaller for profiling)")
    ap.add_argument("--cta-trace", action="store_true",
                    help="print when the CTAs of a decode step's products and attention reach the points they stamp")
    ap.add_argument("--decode-sweep", default="", dest="decode_sweep",
                    help="decode steps at other batch sizes and context lengths, e.g. 1x32000,8x8000,32x4000: one line each")
    ap.add_argument("--prompt-sweep", default="", dest="prompt_sweep",
                    help="one prompt of each of these lengths, e.g. 2048,8192,32000: one line each")
    ap.add_argument("--prefill-chunk", type=int, default=0, dest="prefill_chunk",
                    help="most tokens of a sequence per pass in the sweeps (0: the engine's own)")
    ap.add_argument("--timeline", action="store_true",
                    help="print the kernels of one decode step as they run inside the captured graph (torch profiler)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print("bench.py: this library runs on one GPU; --gpus %d is not supported" % args.gpus)
        return 2
    args.warmup = max(args.warmup, 3)
    args.steps_given = args.steps is not None
    if args.steps is None:
        args.steps = 64

    from friday_inference_engine_b200 import Engine

    if args.decode_sweep or args.prompt_sweep:
        return sweeps(Engine, args)
    cfg = dict(SHAPES[args.model_size])
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    pk = peaks()
    t0 = time.time()
    context = CONTEXT if args.model_size == "7b" else 4096
    slots = args.slots or {"7b": 64, "14b": 16, "32b": 32}[args.model_size]
    args.slots = slots
    eng = Engine(config=cfg, seed={"7b": 0, "14b": 3, "32b": 4}[args.model_size], dtype="bfloat16", max_ctx=context,
                 max_batch=max(slots, args.batch if args.model_size == "7b" else 1), prefill_chunk=PREFILL_TOKENS)
    print("[bench] %s (%.0f s)" % (eng.summary(), time.time() - t0), file=sys.stderr, flush=True)
    nums = model_numbers(cfg, layers)

    if args.timeline:
        return timeline(eng, args.batch)
    if args.cta_trace:
        return cta_trace(eng, args.batch)
    if args.prefill_only:
        ms_pre = time_prefill(eng, PREFILL_TOKENS, max(1, args.warmup - 2), max(1, args.steps))
        print(json.dumps({"prefill_ms": round(ms_pre, 3), "layers_run": layers}))
        return 0
    run = {"7b": run_7b, "14b": run_14b, "32b": run_32b}[args.model_size]
    return run(eng, args, cfg, layers, full_layers, nums, pk)


if __name__ == "__main__":
    sys.exit(main())
