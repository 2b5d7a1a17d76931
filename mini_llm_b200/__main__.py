"""Command line: ``python -m mini_llm_b200`` (also ``bin/mini_llm``).

The reference's program takes no arguments and serves lines of token ids over
TCP (src/main.cpp:3-10; one line of decimal ids in, one id per line out, the last
with " [DONE]": src/runtime/server.cpp:289-305, 344-350); its sizes are constants.
Here the same line format is read from --prompt-ids, --prompts-file or standard
input, and the constants are options named after them: --max-new-tokens
(DEFAULT_MAX_NEW_TOKENS 8), --kv-block-size (DEFAULT_KV_BLOCK_SIZE 16),
--total-kv-blocks (DEFAULT_TOTAL_KV_BLOCKS 4096), --max-batch-num (MAX_BATCH_NUM 16)
(include/constants.h:14-26).  --metrics prints the serving figures of the reference's offline bench
(benchmarks/serving/offline_gpt2_wmma_bench.cu:624-640: TTFT, TPOT and end-to-end latency with
percentiles), --profile writes a per-kernel CSV in the manner of its stage timer
(include/profiling/stage_timer.cuh:40-101).
"""
from __future__ import annotations

import argparse
import json
import sys
import tempfile
from typing import List


def parse_request(line: str) -> List[int]:
    """A line of decimal token ids separated by blanks or commas (the reference's
    parseRequest, src/runtime/server.cpp:271-306)."""
    out = []
    for part in line.replace(",", " ").split():
        out.append(int(part))
    return out


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="mini_llm", description="GPT-2 generation on one B200 from token ids")
    src = ap.add_mutually_exclusive_group(required=True)
    src.add_argument("--model", help="folder with config.json and model.safetensors")
    src.add_argument("--random-config", help="a config.json; weights are drawn from --seed (random-weights mode)")
    ap.add_argument("--seed", type=int, default=0, help="seed of the random weights")
    ap.add_argument("--write-model", help="with --random-config: write the model folder here and keep it")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--kv-block-size", "--page-size", dest="page_size", type=int, default=16)
    ap.add_argument("--total-kv-blocks", "--num-pages", dest="num_pages", type=int, default=None)
    ap.add_argument("--max-batch-num", "--max-num-seqs", dest="max_num_seqs", type=int, default=16)
    ap.add_argument("--max-num-batched-tokens", type=int, default=2048)
    ap.add_argument("--prefill-chunk", type=int, default=2048)
    ap.add_argument("--admission", choices=["lazy", "reserve"], default="lazy")
    ap.add_argument("--max-new-tokens", type=int, default=8)
    ap.add_argument("--temperature", type=float, default=0.0, help="0 = greedy argmax")
    ap.add_argument("--sample-seed", type=int, default=0)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--prompt-ids", action="append", default=[], help='one request, e.g. "15496 11 616 1438 318"')
    ap.add_argument("--prompts-file", help="one request per line of token ids ('-' = standard input)")
    ap.add_argument("--stream", action="store_true", help="print every token as it is produced: '<request> <id>'")
    ap.add_argument("--stats", action="store_true", help="print scheduler counters to standard error")
    ap.add_argument("--metrics", action="store_true",
                    help="print serving metrics to standard error as 'name,value' lines: requests, tokens per second, "
                         "time to first token, time per output token and end-to-end latency (mean, p50, p90, p95, p99)")
    ap.add_argument("--profile", metavar="CSV",
                    help="time every kernel launch with CUDA events (CUDA graphs off) and write "
                         "'step,kind,batch_size,total_tokens,stage,launches,ms' rows, one per kernel entry point and step")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    prompts: List[List[int]] = [parse_request(p) for p in args.prompt_ids]
    if args.prompts_file:
        f = sys.stdin if args.prompts_file == "-" else open(args.prompts_file)
        prompts += [parse_request(l) for l in f if l.strip()]
    if not prompts and not args.write_model:
        prompts = [parse_request(l) for l in sys.stdin if l.strip()]
    if any(not p for p in prompts):
        print("invalid request", file=sys.stderr)
        return 1

    from . import write_random_model
    from .engine.llm import LLM
    from .sampling.params import SamplingParams

    model_dir = args.model
    tmp = None
    if args.random_config:
        with open(args.random_config) as f:
            cfg = json.load(f)
        if args.write_model:
            model_dir = args.write_model
        else:
            tmp = tempfile.TemporaryDirectory(prefix="mini_llm_random_")
            model_dir = tmp.name
        write_random_model(cfg, args.seed, model_dir)
        if not prompts:
            print(model_dir)
            return 0
    llm = LLM(model_dir, dtype=args.dtype, page_size=args.page_size, num_pages=args.num_pages,
              max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens,
              prefill_chunk=args.prefill_chunk, admission=args.admission,
              **({"use_cuda_graphs": False, "async_scheduling": False} if args.profile else {}))
    if args.profile:
        llm.profile = []
    sp = SamplingParams(temperature=args.temperature, seed=args.sample_seed, max_new_tokens=args.max_new_tokens,
                        ignore_eos=args.ignore_eos)
    ids = [llm.add_request(p, sp) for p in prompts]
    outs = {i: [] for i in ids}
    while llm.has_unfinished():
        for r in llm.step():
            outs[r.request_id].append(r.token)
            if args.stream:
                print(f"{r.request_id} {r.token}{' [DONE]' if r.finished else ''}", flush=True)
    if not args.stream:
        for i in ids:
            print(" ".join(str(t) for t in outs[i]) + " [DONE]")
    if args.stats:
        print(json.dumps(vars(llm.scheduler.stats)), file=sys.stderr)
    if args.metrics:
        for k, v in llm.metrics.summary().items():
            print(f"{k},{v:.6f}" if isinstance(v, float) else f"{k},{v}", file=sys.stderr)
    if args.profile:
        with open(args.profile, "w") as f:
            f.write("step,kind,batch_size,total_tokens,stage,launches,ms\n")
            for step, kind, reqs, toks, stage, n, ms in llm.profile:
                f.write(f"{step},{kind},{reqs},{toks},{stage},{n},{ms:.4f}\n")
    if tmp is not None:
        tmp.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
