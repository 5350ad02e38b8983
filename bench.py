#!/usr/bin/env python3
"""Measures generation of the Qwen2.5-7B shape with random bf16 weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]

One JSON line on stdout.  `value` is decoded tokens per second at batch 8 (prompts of
1,024 random token ids, slots of 8,192 tokens), timed on the device with CUDA events
around exactly K decode steps after W warm-up steps.  `e2e` is the same through the
public Python entry point (Engine.generate: host token ids in, host token ids out,
every step with its host-to-device copy of inputs from pinned memory and its
device-to-host read of the chosen tokens).  `prefill` is one prompt of 2,048 tokens;
`points` holds decoding at batch 1 and 64; `roofline` relates the bytes a decode step
must read (every weight once, the cache of the live requests) to its time.

Every decode step reads all weights (15 GB at the full shape), far more than the
126 MB L2, so consecutive timed steps cannot be served from L2.

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


def time_decode(eng, batch, steps, warmup, seed):
    """Device time of `steps` decode steps at `batch` after 1,024-token prompts; tokens stay on the device."""
    import torch
    from friday_inference_engine_b200.ops import lib
    prompts = random_prompts(batch, PROMPT, eng.vocab_size, seed)
    slots = [eng.alloc_slot() for _ in prompts]
    for lo in range(0, batch, 8):                             # prompts in groups: bounds the scratch of a pass
        eng.step(slots[lo:lo + 8], prompts[lo:lo + 8], [[]] * len(slots[lo:lo + 8]))
    dec = eng.decoder(slots, [p[-1] for p in prompts])       # decoding that stays on the device
    for _ in range(warmup):
        dec.step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = lib.launch_count()
    a.record()
    for _ in range(steps):
        dec.step()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b)
    launches = lib.launch_count() - launches0
    mean_len = PROMPT + warmup + steps / 2.0
    dec.close()
    for s in slots:
        eng.free_slot(s)
    return ms / steps, launches, mean_len


E2E_SETTLE_STEPS = 32


def time_e2e(eng, batch, steps, seed):
    """Engine.generate with host tokens in and out: every decode step copies its token ids in from pinned memory and
    the chosen ids out.  Returns tokens/s over the last `steps` decode steps and over the first `steps` ones.

    The first decode steps after the prompts run slower than the rest: 8 x 1,024 prompt tokens drive the GPU into its
    power cap, and the SM clock needs some 15 steps of the much lighter decoding to come back (4.1 ms a step, then
    3.16 ms).  The device-timed value does not see this (graph capture sits between its prompts and its timed steps),
    so the headline figure skips E2E_SETTLE_STEPS steps; the figure from the first token on is reported beside it."""
    import torch
    prompts = random_prompts(batch, PROMPT, eng.vocab_size, seed)
    marks = []

    def on_step(live, drawn):
        marks.append(time.perf_counter())

    eng.generate(prompts, max_new_tokens=4, temperature=0.0, ignore_eos=True)       # warm-up: captures the step
    marks.clear()
    torch.cuda.synchronize()
    total = E2E_SETTLE_STEPS + steps
    out = eng.generate(prompts, max_new_tokens=total + 1, temperature=0.0, ignore_eos=True, on_step=on_step)
    assert all(len(g.tokens) == total + 1 for g in out)
    return batch * steps / (marks[-1] - marks[-1 - steps]), batch * steps / (marks[steps] - marks[0])


def time_prefill(eng, warmup, reps):
    import torch
    (p,) = random_prompts(1, PREFILL_TOKENS, eng.vocab_size, 99)
    times = []
    for r in range(warmup + reps):
        s = eng.alloc_slot()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.step([s], [p], [[PREFILL_TOKENS - 1]])
        b.record()
        torch.cuda.synchronize()
        if r >= warmup:
            times.append(a.elapsed_time(b))
        eng.free_slot(s)
    return sorted(times)[len(times) // 2]


def timeline(eng, batch):
    """Kernels of the last of three profiled decode steps: name, start, duration, and `real`, the time from the end
    of the kernel before to the end of this one (kernels overlap under programmatic dependent launch)."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    prompts = random_prompts(batch, PROMPT, eng.vocab_size, 1)
    slots = [eng.alloc_slot() for _ in prompts]
    for lo in range(0, batch, 8):
        eng.step(slots[lo:lo + 8], prompts[lo:lo + 8], [[]] * len(slots[lo:lo + 8]))
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
    from friday_inference_engine_b200 import ops
    from friday_inference_engine_b200.ops import lib
    layers = len(eng.model.layers)
    prompts = random_prompts(batch, PROMPT, eng.vocab_size, 1)
    slots = [eng.alloc_slot() for _ in prompts]
    for lo in range(0, batch, 8):
        eng.step(slots[lo:lo + 8], prompts[lo:lo + 8], [[]] * len(slots[lo:lo + 8]))
    dec = eng.decoder(slots, [p[-1] for p in prompts])
    dec.step()                                                # eager: sizes scratch, builds libraries
    be = ops.backend()
    n_gemm = 4 * layers + 1
    be.trace = torch.zeros((n_gemm, 148, 16), dtype=torch.int64, device="cuda:0")
    be.trace_next = 0
    attn = torch.zeros((8192, 8), dtype=torch.int64, device="cuda:0")
    set_trace = lib.family("attention_mma").declare("attention_mma_set_trace", [lib.P])
    set_trace(attn.data_ptr())
    dec.step()                                                # captured with the trace pointers in place
    for _ in range(5):
        dec.step()
    torch.cuda.synchronize()
    be.trace.zero_()
    attn.zero_()
    dec.step()
    torch.cuda.synchronize()
    set_trace(None)
    g = be.trace.cpu().numpy().astype(np.float64)
    a = attn.cpu().numpy().astype(np.float64)
    be.trace = None
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
    # products spend the time of a block of 64 keys
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
    print("prompt attention, %d tokens: %d CTAs, %d blocks of 64 keys; us per block: " % (PREFILL_TOKENS, len(t), blocks)
          + ", ".join("%s %.2f" % (what, t[:, k].sum() / blocks / 1000.0) for k, what in
                      ((0, "row waits for S"), (1, "reads S, maximum"), (2, "exponentials and P"), (3, "rescales O"),
                       (4, "waits for the last product"), (8, "issuer waits for K"), (9, "issues Q K^T"),
                       (10, "waits for V"), (11, "waits for P"), (12, "issues P V")))
          + "; kernel %.1f us" % (((t[:, 7] + t[:, 6]).max() - t[:, 7].min()) / 1000.0))
    return 0


def reference_arm():
    why = ("the reference is a C++/CMake program with no Python packaging (pip install of its tree fails: "
           "no setup.py or pyproject.toml), has no bf16 or batched path and targets sm_86 with GGUF k-quant weights")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0, help="run this many layers of the same sizes (0: all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 / 64, prefill and e2e")
    ap.add_argument("--prefill-only", action="store_true", help="time the 2,048-token prompt only (for profiling)")
    ap.add_argument("--slots", type=int, default=64, help="sequences the cache is sized for (smaller for profiling)")
    ap.add_argument("--cta-trace", action="store_true",
                    help="print when the CTAs of a decode step's products and attention reach the points they stamp")
    ap.add_argument("--timeline", action="store_true",
                    help="print the kernels of one decode step as they run inside the captured graph (torch profiler)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.gpus != 1:
        print("bench.py: this library runs on one GPU; --gpus %d is not supported" % args.gpus)
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    from friday_inference_engine_b200 import Engine

    cfg = dict(QWEN25_7B)
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    pk = peaks()
    t0 = time.time()
    eng = Engine(config=cfg, seed=0, dtype="bfloat16", max_ctx=CONTEXT, max_batch=max(args.slots, args.batch),
                 prefill_chunk=PREFILL_TOKENS)
    print("[bench] %s (%.0f s)" % (eng.summary(), time.time() - t0), file=sys.stderr, flush=True)
    nums = model_numbers(cfg, layers)

    if args.timeline:
        return timeline(eng, args.batch)
    if args.cta_trace:
        return cta_trace(eng, args.batch)
    if args.prefill_only:
        ms_pre = time_prefill(eng, max(1, args.warmup - 2), max(1, args.steps))
        print(json.dumps({"prefill_ms": round(ms_pre, 3), "layers_run": layers}))
        return 0
    clocks = Clocks()
    clocks.start()
    ms_step, launches, mean_len = time_decode(eng, args.batch, args.steps, args.warmup, seed=1)
    clk = clocks.stop()
    value = args.batch * 1000.0 / ms_step
    step_bytes = nums["step_weight_bytes"] + args.batch * mean_len * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms_step * 1e-3) / 1e9

    line = {
        "metric": "Qwen2.5-7B bf16 decode tok/s at batch %d" % args.batch, "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "impl": "ours", "gpu_launches": int(launches), "clocks": clk,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"]},
        "config": {"model": "Qwen2.5-7B shape, random weights", "global_batch": args.batch, "seq_len": CONTEXT,
                   "prompt_len": PROMPT, "parallelism": "none", "layers_run": layers, "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "l2": "every step reads all weights (>> 126 MB L2)", "peaks": pk["source"]},
    }
    if not args.skip_points:
        steps_pt = max(8, args.steps // 2)
        points = {}
        for b in (1, 64):
            ms_b, _, _ = time_decode(eng, b, steps_pt, args.warmup, seed=2 + b)
            points["decode_b%d" % b] = round(b * 1000.0 / ms_b, 1)
        line["points"] = points
        ms_pre = time_prefill(eng, 2, 3)
        flops = 2.0 * PREFILL_TOKENS * nums["matmul_params"] + 2.0 * nums["head_params"]
        qd = cfg["num_attention_heads"] * cfg["head_dim"]
        flops += layers * 4.0 * qd * PREFILL_TOKENS * PREFILL_TOKENS / 2.0
        line["prefill"] = {"value": round(PREFILL_TOKENS * 1000.0 / ms_pre, 1), "tokens": PREFILL_TOKENS,
                           "ms": round(ms_pre, 3), "frac": round(flops / (ms_pre * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        e2e, e2e_from_first = time_e2e(eng, args.batch, min(args.steps, 64), seed=1)
        # every decode step of generate() copies the step's token ids in from pinned memory and the chosen ids out
        line["e2e"] = {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": 4 * args.batch,
                       "d2h_bytes_per_step": 4 * args.batch, "settle_steps": E2E_SETTLE_STEPS,
                       "from_first_token": round(e2e_from_first, 1)}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
