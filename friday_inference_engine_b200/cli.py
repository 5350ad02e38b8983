"""Command line, in the manner of the reference's main.cpp (:140-355): a model path,
`--ctx N`, `--backend`, `--kv`, `--info`, then prompts from standard input until
`exit` or `quit`, each answered by up to 100 new tokens (main.cpp:328), greedy unless a
temperature is given.  The library has no tokenizer: a prompt is a line of token ids
(separated by spaces or commas) and the answer is printed as ids.

Kept from the reference with their meaning: the positional model path; `--ctx N`, the
tokens one sequence can hold (default 2048, main.cpp:178); `--backend auto|cuda` (`cpu`
is refused: there is no CPU path); `--kv auto|bf16|f32` (`q8` is refused: no quantized
cache); `--info` (main.cpp:145-164).  `--vram` and `--threads` steer the reference's
CPU offload, which does not exist here; they are accepted and ignored with a note.
Added: `--batch`, `--dtype`, `--random`, `--seed`, `--prompt-ids`, `--prompt-file`,
`--max-new-tokens`, `--temperature`, `--sample-seed`, `--stop-ids`, `--ignore-eos`, and
`--profile`, which prints per request batch where the time went (host time per step,
device time of products, attention and the rest between CUDA events), as the reference
prints its per-token phases under FRIDAY_PROFILE (transformer.cpp:603-613, 1162-1183).

The program is a binding: everything it runs is friday::Engine of libfriday_engine.so.
"""
import argparse
import json
import re
import sys


def _ids(text):
    return [int(t) for t in re.split(r"[\s,]+", text.strip()) if t]


def info():
    import torch
    from . import registered_architectures, registered_parts
    print("FRIDAY Engine (B200) capability report")
    print("  CUDA     : %s" % ("available" if torch.cuda.is_available() else "no device visible"))
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        free, total = torch.cuda.mem_get_info(i)
        print("  GPU      : %s, compute %d.%d, %d SMs, %.1f GB memory (%.1f GB free)"
              % (p.name, p.major, p.minor, p.multi_processor_count, total / 1e9, free / 1e9))
    print("  Backend  : CUDA kernels for sm_100a only; there is no CPU path")
    print("  Models   : %s" % ", ".join(registered_architectures()))
    print("  Parts    : %s" % "; ".join("%s: %s" % (c, ", ".join(registered_parts(c)))
                                        for c in ("norm", "position", "mixer", "feed_forward", "block")))
    return 0


def build_parser():
    ap = argparse.ArgumentParser(prog="friday", description="Qwen2.5 generation on one B200, token ids in and out")
    ap.add_argument("model", nargs="?", help="model folder (config.json + model.safetensors)")
    ap.add_argument("--ctx", type=int, default=2048, help="tokens one sequence can hold (default 2048)")
    ap.add_argument("--batch", type=int, default=8, help="sequences alive at once (default 8)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "bf16", "float32", "fp32"])
    ap.add_argument("--backend", default="auto", help="auto | cuda  (cpu is refused)")
    ap.add_argument("--kv", default="auto", help="auto | bf16 | f32: the cache follows --dtype (q8 is refused)")
    ap.add_argument("--vram", type=float, default=0.0, help="ignored: nothing is offloaded")
    ap.add_argument("--threads", type=int, default=0, help="ignored: no layer runs on the CPU")
    ap.add_argument("--info", action="store_true", help="print the devices and exit")
    ap.add_argument("--random", metavar="CONFIG_JSON", help="random weights for this config.json instead of a model")
    ap.add_argument("--seed", type=int, default=0, help="seed of the random weights")
    ap.add_argument("--prompt-ids", action="append", default=[], help='a prompt as token ids, "1,2,3"; may repeat')
    ap.add_argument("--prompt-file", help="file with one prompt (token ids) per line: run them as batches")
    ap.add_argument("--max-new-tokens", type=int, default=100)
    ap.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    ap.add_argument("--sample-seed", type=int, default=42, help="seed of the sampler")
    ap.add_argument("--stop-ids", default="", help='token ids that end a sequence, "151643,151645"')
    ap.add_argument("--ignore-eos", action="store_true", help="never stop on a stop id")
    ap.add_argument("--json", action="store_true", help="print results as JSON lines")
    ap.add_argument("--profile", action="store_true",
                    help="print where each batch's time went: host time per step; products, attention, other on the device")
    return ap


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] in ("--info", "info"):
        return info()
    args = build_parser().parse_args(argv)
    if args.info:
        return info()
    if args.backend not in ("auto", "cuda"):
        print("unknown --backend '%s' (auto, cuda); this library has no CPU path" % args.backend, file=sys.stderr)
        return 2
    if args.kv not in ("auto", "bf16", "f32"):
        print("unknown --kv '%s' (auto, bf16, f32); quantized caches are not built" % args.kv, file=sys.stderr)
        return 2
    if args.vram or args.threads:
        print("[Init] --vram/--threads are ignored: every layer runs on the GPU", file=sys.stderr)
    if (args.model is None) == (args.random is None):
        print("give a model folder or --random CONFIG_JSON", file=sys.stderr)
        return 2
    from .engine import Engine
    try:
        kw = dict(dtype=args.dtype, max_ctx=args.ctx, max_batch=args.batch, profile=args.profile)
        if args.random:
            with open(args.random) as f:
                eng = Engine(config=json.load(f), seed=args.seed, **kw)
        else:
            eng = Engine(model_path=args.model, **kw)
    except Exception as e:  # noqa: BLE001 - reported to the user as the reference does
        print("[FATAL ERROR] %s" % e, file=sys.stderr)
        return 1
    print("[Init] %s" % eng.summary(), file=sys.stderr)
    gen = dict(max_new_tokens=args.max_new_tokens, temperature=args.temperature, seed=args.sample_seed,
               stop_token_ids=_ids(args.stop_ids), ignore_eos=args.ignore_eos)

    def run(prompts):
        try:
            results = eng.generate(prompts, **gen)
        except Exception as e:  # noqa: BLE001
            print("[Hata] %s" % e, file=sys.stderr)
            return 1
        if args.profile:
            pr = eng.profile()
            total = pr["product_ms"] + pr["attention_ms"] + pr["other_ms"]
            print("[Profile] %d step calls, host %.2f ms in all; device %.2f ms between events: products %.2f ms (%d), "
                  "attention %.2f ms (%d), other %.2f ms (%d)"
                  % (pr["steps"], pr["host_ms"], total, pr["product_ms"], pr["product_calls"], pr["attention_ms"],
                     pr["attention_calls"], pr["other_ms"], pr["other_calls"]), file=sys.stderr)
        for p, g in zip(prompts, results):
            if args.json:
                print(json.dumps({"prompt_tokens": len(p), "tokens": g.tokens, "finish_reason": g.finish_reason}))
            else:
                print("FRIDAY: %s  [%s]" % (" ".join(str(t) for t in g.tokens), g.finish_reason))
        sys.stdout.flush()
        return 0

    prompts = [_ids(p) for p in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [_ids(line) for line in f if line.strip()]
    if prompts:
        return run(prompts)
    print("[Init] FRIDAY Engine ready. Enter token ids ('exit' or 'quit' to leave):", file=sys.stderr)
    while True:
        sys.stderr.write("\nUser> ")
        sys.stderr.flush()
        line = sys.stdin.readline()
        if not line or line.strip() in ("exit", "quit"):
            break
        if not line.strip():
            continue
        try:
            ids = _ids(line)
        except ValueError:
            print("[Hata] a prompt is a line of token ids", file=sys.stderr)
            continue
        run([ids])
    return 0


if __name__ == "__main__":
    sys.exit(main())
