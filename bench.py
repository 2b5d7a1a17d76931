"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--dtype float32|bfloat16]

A "step" is one decode step: every live request gets one more token.  The default
run is GPT-2 small (n_layer 12, n_embd 768, n_head 12, n_inner 3072, vocab 50257,
n_positions 1024) with seeded random weights, a batch of 8 requests with 512-token
random prompts, page size 16.  The headline numbers are those of the float32 path (true
32-bit: the reference's only precision, so the two arms compare like with like); the
bfloat16 path of the same model is measured in the same run and reported under ``points``
with ``bf16_`` in every key.  ``--dtype bfloat16`` swaps the two.  It prints ONE JSON line:

  value       decoded tokens per second over exactly K steps, timed on the device
              with CUDA events (forward pass + on-device argmax per step).  The default
              K = 512 is the benchmark's whole generation: contexts grow from 512 to
              1,023.  The warm-up is the same generation by other requests, max(W, K)
              steps and never fewer than 3 (``warmup`` in the line is that number, which
              can exceed the W asked for), so the timed steps replay captured graphs; a K
              beyond the 512 positions a request has left is cut to 512;
  e2e         the same through the Python entry point (LLM.step): host token ids in,
              sampled ids back on the host every step (wall clock around K steps, the
              median of three such runs, since K steps may be only a millisecond);
  prefill     2,048 prompt tokens (2 x 1024) in one step: tokens/s, ms, and the share of
              the peak for its dtype that its flops reach (bfloat16: the measured cuBLAS
              rate; float32: the CUDA cores' nominal FFMA rate, SMs x 128 x 2 x clock);
  roofline    bytes the decode step has to read (every weight once + the cache of the
              live requests) / its time, against the HBM copy bandwidth;
  points      decode tokens/s at batch 1 and 64 with their share of the HBM rate, the
              entry point's tokens/s at batch 1, and the other precision's decode at batch
              1 / 8 / 64, entry-point and prefill figures.

Peaks come from MEASURED_PEAKS.json beside this file when present, else from the
fallback figures 6.65 TB/s and 1.59 PFLOP/s ("peaks": "fallback").

``--impl reference`` runs taejuk/mini-llm itself: its unmodified sources from baseline/_ref,
compiled with nvcc for sm_100a together with baseline/reference_arm.cu (a main() that calls its
GPT2Model::prefill / decode only), on the same weights and prompts, and prints the same line
with "impl": "reference" and "dtype": "fp32".  The reference holds at most 16 requests and
4096 cache blocks per process, so a batch of 8 can decode 159 steps after 512-token prompts
(more are cut) and there is no batch-64 point.  Where it cannot be built or run the line is
{"impl": "reference", "unavailable": "<why>"}.

``--profile-step prefill|decode [--kernel-times]`` runs one small eager step (for a profiler, or to
print each kernel's share of the step from CUDA events); ``--workload medium|xl`` runs the
continuous-batching workloads of the larger GPT-2 sizes.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SMALL = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=12, n_embd=768, n_head=12, n_inner=3072,
             vocab_size=50257, n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new",
             eos_token_id=50256)
PROMPT_LEN = 512
PREFILL_TOKENS = 2048
PAGE = 16


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            d = json.load(open(p))
            hbm = float(d.get("hbm_gbs") or d.get("hbm_gb_s") or 0)
            bf = float(d.get("bf16_tflops") or 0)
            sus = float(d.get("bf16_tflops_sustained") or bf)
            if hbm > 0 and bf > 0:
                return dict(hbm_gbs=hbm, bf16_tflops=bf, bf16_tflops_sustained=sus, source="measured")
        except Exception:
            pass
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.p = None

    def _read(self):
        for line in self.p.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            pass
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = max((int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()), default=None)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": reasons,
                "samples": len(mhz)}


def weight_bytes(runner) -> int:
    seen, total = set(), 0
    for label, _ in runner.spec.all_part_specs():
        part = runner.model.part(label)
        for name in part.param_specs():
            t = getattr(part, name)
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
    return total


def decode_bytes(runner, cfg, batch, mean_ctx) -> float:
    """What one decode step must read: every weight once (of the position table only the
    rows used) and the keys and values of the live requests."""
    es = 2 if runner.engine.dtype == "bfloat16" else 4
    w = weight_bytes(runner) - cfg["n_positions"] * cfg["n_embd"] * es + batch * cfg["n_embd"] * es
    kv = batch * mean_ctx * cfg["n_layer"] * 2 * cfg["n_embd"] * es
    return float(w + kv)


def prefill_flops(cfg, lens, rows) -> float:
    L, D, F, V = cfg["n_layer"], cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"]
    T = sum(lens)
    linear = 2.0 * T * L * (3 * D * D + D * D + 2 * D * F) + 2.0 * rows * D * V
    attn = sum(4.0 * (n * (n + 1) / 2) * D * L for n in lens)
    return linear + attn


def decode_steps(cfg, steps: int) -> int:
    """A request starts at a PROMPT_LEN-token prompt and may be fed a token at every further position."""
    return max(1, min(int(steps), int(cfg["n_positions"]) - PROMPT_LEN))


def run_decode(model_dir, dtype, batch, steps, warmup, sample_clocks=False):
    """Device-timed decode: K steps of (forward + argmax) on ``batch`` live requests whose contexts grow from
    PROMPT_LEN.  The warm-up is a generation of max(W, K) steps by other requests of the same shape (every step
    shape of the timed run has then been seen and captured); the timed K steps start right after the prompts of
    the timed requests are in, so that K = 512 covers the contexts 512 .. 1023 of the benchmark."""
    import torch
    import mini_llm_b200 as m
    from mini_llm_b200 import ops
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner, StepEntry

    cfg = json.load(open(os.path.join(model_dir, "config.json")))
    steps = decode_steps(cfg, steps)
    warm_steps = decode_steps(cfg, max(steps, warmup))
    eng = EngineConfig(dtype=dtype, page_size=PAGE, max_tokens=batch * cfg["n_positions"], max_num_seqs=max(batch, 1),
                       max_num_batched_tokens=max(2048, batch))
    runner = ModelRunner(model_dir, eng)
    prompts = bench_prompts(cfg["vocab_size"], batch)
    out = torch.empty(batch, dtype=torch.int32, device=runner.device)
    toks = [int(p[-1]) for p in prompts]

    def start(tag):
        ids = [(tag, i) for i in range(batch)]
        for r in ids:
            runner.add_request(r)
        for lo in range(0, batch, 4):                       # prompts, 2,048 tokens per step
            runner.step([StepEntry(ids[i], prompts[i], []) for i in range(lo, min(batch, lo + 4))])
        return ids

    def one(ids):
        logits = runner.step([StepEntry(ids[i], [toks[i]], [0]) for i in range(batch)])
        ops.argmax(logits, out)

    ids = start("warm")
    for _ in range(warm_steps):
        one(ids)
    for r in ids:
        runner.finish_request(r)
    ids = start("timed")
    torch.cuda.synchronize()
    clocks = ClockSampler()
    if sample_clocks:
        clocks.start()
    ctx0 = runner.computed(ids[0])
    n0 = ops.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        one(ids)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    launches = ops.launches - n0
    mean_ctx = ctx0 + (steps + 1) / 2.0
    res = dict(ms_per_step=ms / steps, tok_s=batch * steps / (ms / 1e3), launches=launches, steps=steps,
               warmup=warm_steps, bytes=decode_bytes(runner, cfg, batch, mean_ctx), mean_ctx=mean_ctx,
               clocks=clocks.stop() if sample_clocks else None)
    del runner
    torch.cuda.empty_cache()
    return res


def run_e2e(model_dir, dtype, batch, steps, warmup):
    """The same decode steps through LLM.step(): host token lists in, sampled ids out.  One generation by other
    requests warms up; then the timed requests' prompts go in and the clock runs from their first decode step
    until the last of their K decoded tokens has been handed back to the host."""
    import torch
    import mini_llm_b200 as m

    cfg = json.load(open(os.path.join(model_dir, "config.json")))
    steps = decode_steps(cfg, steps)
    # all prompts go in with one step, so that the requests decode side by side from the first timed step to the last
    llm = m.LLM(model_dir, dtype=dtype, page_size=PAGE, max_tokens=batch * cfg["n_positions"], max_num_seqs=batch,
                max_num_batched_tokens=batch * PROMPT_LEN, prefill_chunk=PROMPT_LEN)
    prompts = bench_prompts(cfg["vocab_size"], batch)
    sp = m.SamplingParams(max_new_tokens=steps + 1, ignore_eos=True)     # one token from the prompt's step, K decoded

    def prompts_in():
        for p in prompts:
            llm.add_request(p, sp)
        first = 0
        while llm.scheduler.waiting or llm.scheduler.prefill or llm.scheduler.deferred_prefill:
            first += len(llm.step())
        return first

    prompts_in()
    while llm.has_unfinished():
        llm.step()
    rates = []
    for _ in range(3):                         # K steps are a millisecond or so of wall clock: the median of three runs
        first = prompts_in()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        produced = 0
        while llm.has_unfinished():
            produced += len(llm.step())
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        produced -= batch - first              # tokens of the prompts' step that were only handed back inside the clock
        rates.append(produced / dt)
    lay = llm.runner._last_layout_total if hasattr(llm.runner, "_last_layout_total") else None
    res = dict(tok_s=sorted(rates)[1], h2d=(lay or 0) * 4, d2h=batch * 4, tokens=produced)
    del llm
    torch.cuda.empty_cache()
    return res


def run_prefill(model_dir, dtype, iters=5, warmup=3):
    import torch
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner, StepEntry

    cfg = json.load(open(os.path.join(model_dir, "config.json")))
    n = cfg["n_positions"]
    lens = [n] * (PREFILL_TOKENS // n)
    eng = EngineConfig(dtype=dtype, page_size=PAGE, max_tokens=PREFILL_TOKENS, max_num_seqs=len(lens),
                       max_num_batched_tokens=PREFILL_TOKENS)
    runner = ModelRunner(model_dir, eng)
    g = torch.Generator().manual_seed(99)
    # the prompts are host arrays of token ids (int32), as a tokenizer hands them over
    prompts = [torch.randint(0, cfg["vocab_size"], (l,), generator=g).to(torch.int32).numpy() for l in lens]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=runner.device)
    times = []
    for it in range(warmup + iters):
        for i in range(len(lens)):
            runner.add_request(i)
        flush.zero_()                                    # larger than L2: the step starts cold
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        runner.step([StepEntry(i, prompts[i], [l - 1]) for i, l in enumerate(lens)])
        e1.record()
        torch.cuda.synchronize()
        if it >= warmup:
            times.append(e0.elapsed_time(e1))
        for i in range(len(lens)):
            runner.finish_request(i)
    ms = sorted(times)[len(times) // 2]
    fl = prefill_flops(cfg, lens, len(lens))
    del runner
    torch.cuda.empty_cache()
    return dict(ms=ms, tok_s=PREFILL_TOKENS / (ms / 1e3), flops=fl)


def profile_step(kind: str, dtype: str, layers: int, batch: int, kernel_times: bool = False) -> int:
    """One eager prefill step (2 x 1024 tokens) or a few eager decode steps at GPT-2 small's
    layer sizes with ``layers`` layers: a small, bounded workload to put under ncu, e.g.
    ncu --set full --clock-control none -k regex:attention_flash -c 1 python bench.py --profile-step prefill --layers 2
    With ``kernel_times`` the last step's launches are timed one by one with CUDA events and the line carries,
    per entry point of the kernel library, its launches, microseconds and share of the step (eager launches,
    so the gaps between kernels are larger than in the replayed graphs that generation uses)."""
    import torch
    import mini_llm_b200 as m
    from mini_llm_b200 import ops
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner, StepEntry

    cfg = dict(SMALL, n_layer=layers)
    times = None
    with tempfile.TemporaryDirectory(prefix="mini_llm_prof_") as d:
        m.write_random_model(cfg, 0, d, dtype=dtype)
        n = cfg["n_positions"]
        B = 2 if kind == "prefill" else batch
        runner = ModelRunner(d, EngineConfig(dtype=dtype, page_size=PAGE, max_tokens=B * n, max_num_seqs=B,
                                             max_num_batched_tokens=2048, use_cuda_graphs=False))
        g = torch.Generator().manual_seed(7)
        plen = n if kind == "prefill" else PROMPT_LEN
        prompts = torch.randint(0, cfg["vocab_size"], (B, plen), generator=g).tolist()
        out = torch.empty(B, dtype=torch.int32, device=runner.device)

        def prompts_in():
            for i in range(B):
                runner.add_request(i)
            for lo in range(0, B, 2):
                ops.argmax(runner.step([StepEntry(i, prompts[i], [plen - 1]) for i in range(lo, min(B, lo + 2))]),
                           out[lo:min(B, lo + 2)])

        def decode_once():
            ops.argmax(runner.step([StepEntry(i, [11], [0]) for i in range(B)]), out)

        prompts_in()
        if kind == "decode":
            for _ in range(3):
                decode_once()
        if kernel_times:
            if kind == "prefill":
                for i in range(B):
                    runner.finish_request(i)
            torch.cuda.synchronize()
            with ops.time_launches() as tl:
                prompts_in() if kind == "prefill" else decode_once()
            rows = tl.rows()
            total = sum(ms for _, _, ms in rows) or 1.0
            times = {name.replace("mllm_", ""): {"launches": k, "us": round(ms * 1e3, 1), "share": round(ms / total, 3)}
                     for name, k, ms in rows}
        torch.cuda.synchronize()
        ops.check_device_errors()
    line = {"profile_step": kind, "layers": layers, "batch": B, "dtype": dtype, "launches": ops.launches}
    if times is not None:
        line["kernel_times"] = times
        line["kernel_us_total"] = round(sum(v["us"] for v in times.values()), 1)
    print(json.dumps(line))
    return 0


MEDIUM = dict(SMALL, n_layer=24, n_embd=1024, n_head=16, n_inner=4096)
XL = dict(SMALL, n_layer=48, n_embd=1600, n_head=25, n_inner=6400)


def run_workload(kind: str, dtype: str, layers: int) -> int:
    """The two serving workloads of the larger GPT-2 sizes, through the Python entry point.

    medium: 64 requests, prompt lengths uniform in [32, 1024), output lengths uniform in [16, 256),
            continuous batching with prompts cut into portions of 512 tokens.
    xl:     64 requests with 128-token prompts generating 896 tokens each; the cache pool holds 24
            full contexts, so admission defers requests and running ones are preempted by recompute.
    Prints one JSON line with tokens per second and the scheduler's counters."""
    import torch
    import mini_llm_b200 as m

    cfg = dict(MEDIUM if kind == "medium" else XL)
    full_layers = cfg["n_layer"]
    if layers and layers < full_layers:
        cfg["n_layer"] = layers
    g = torch.Generator().manual_seed(2024)
    n = cfg["n_positions"]
    if kind == "medium":
        plens = torch.randint(32, 1024, (64,), generator=g).tolist()
        olens = [min(o, n - p + 1) for p, o in zip(plens, torch.randint(16, 256, (64,), generator=g).tolist())]
        eng = dict(max_tokens=64 * n, max_num_seqs=64, max_num_batched_tokens=1024, prefill_chunk=512)
    else:
        plens, olens = [128] * 64, [896] * 64
        eng = dict(max_tokens=24 * n, max_num_seqs=64, max_num_batched_tokens=2048, prefill_chunk=512)
    prompts = [torch.randint(0, cfg["vocab_size"], (p,), generator=g).tolist() for p in plens]
    with tempfile.TemporaryDirectory(prefix="mini_llm_work_") as d:
        m.write_random_model(cfg, 0, d, dtype=dtype)
        llm = m.LLM(d, dtype=dtype, page_size=PAGE, **eng)
        params = [m.SamplingParams(max_new_tokens=o, ignore_eos=True) for o in olens]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate(prompts, params)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        st = llm.scheduler.stats
        assert [len(o) for o in outs] == olens, "a request produced the wrong number of tokens"
        llm.runner.cache.check()
        print(json.dumps({"workload": kind, "dtype": dtype, "n_layer": cfg["n_layer"], "n_layer_full": full_layers,
                          "n_embd": cfg["n_embd"], "n_head": cfg["n_head"], "requests": 64,
                          "prompt_tokens": sum(plens), "output_tokens": sum(olens), "seconds": round(dt, 3),
                          "output_tok_s": round(sum(olens) / dt, 1), "total_tok_s": round((sum(plens) + sum(olens)) / dt, 1),
                          "steps": st.steps, "deferred_decode": st.deferred_decode,
                          "deferred_prefill": st.deferred_prefill, "preempted": st.preempted,
                          "peak_pages": st.peak_pages, "num_pages": llm.runner.num_pages,
                          "graph_replays": llm.runner.graph_replays}))
    return 0


def fp32_peak_flops() -> float:
    """CUDA-core peak of the float32 path (no tensor-core mode exists for true 32-bit products):
    SMs x 128 lanes x 2 flops x the highest SM clock; nominal, nothing measures it on this pool."""
    import torch
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    mhz = 1965.0
    try:
        mhz = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("sm_max_mhz") or mhz)
    except Exception:
        pass
    return sms * 128 * 2 * mhz * 1e6


def bench_prompts(vocab: int, batch: int, n: int = PROMPT_LEN):
    """The prompts of the decode benchmark: the same ids for this engine and for the reference arm."""
    import torch
    g = torch.Generator().manual_seed(1234)
    return torch.randint(0, vocab, (batch, n), generator=g).tolist()


def base_config(cfg, batch, mean_ctx, pk):
    return {"model": "gpt2-small", "n_layer": cfg["n_layer"], "n_layer_full": SMALL["n_layer"],
            "n_embd": cfg["n_embd"], "n_head": cfg["n_head"], "n_inner": cfg["n_inner"],
            "vocab_size": cfg["vocab_size"], "n_positions": cfg["n_positions"], "global_batch": batch,
            "prompt_len": PROMPT_LEN, "seq_len": cfg["n_positions"], "page_size": PAGE,
            "mean_context": mean_ctx, "parallelism": "single GPU",
            "l2": "inputs exceed L2 (weights + cache > 126 MB)", "peaks": pk["source"],
            "baseline": "854.41 tok/s, FP32, batch 8, on a TITAN V: other hardware (gpt2_decode_batch_sweep_512.csv:5)"}


def run_reference(args) -> int:
    """The reference arm: taejuk/mini-llm itself, unmodified, built from baseline/_ref and driven through its own
    GPT2Model::prefill / decode on the same seeded weights and prompts (float32, its only precision).  Its limits
    (batch <= 16, a pool of 4096 blocks of 16 tokens per layer, include/constants.h:16-26) cap the steps a batch of
    8 can run after 512-token prompts at 159; more are cut and ``config`` says so."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ra

    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": str(why).replace("\n", " ")[:400]}))
        return 0

    if args.gpus != 1:
        return unavailable("the reference runs on one GPU only")
    import torch
    if not torch.cuda.is_available():
        return unavailable("no CUDA device: the reference has no CPU path")
    if args.layers != SMALL["n_layer"] or args.batch > ra.MAX_BATCH:
        return unavailable("the reference is compiled for GPT-2 small with 12 layers and at most 16 requests")
    try:
        if not ra.have_sources() and os.path.isdir("/root/reference/src"):
            ra.fetch_sources("/root/reference")
        exe = ra.build()
    except ra.ReferenceUnavailable as e:
        return unavailable(e)
    import mini_llm_b200 as m
    pk = peaks()
    cfg = dict(SMALL)
    warmup = max(args.warmup, 3)
    most = ra.most_decode_steps(args.batch, PROMPT_LEN)
    steps = max(1, min(decode_steps(cfg, args.steps), most))
    warmup = min(warmup, most)
    try:
        with tempfile.TemporaryDirectory(prefix="mini_llm_ref_") as d:
            m.write_random_model(cfg, 0, os.path.join(d, "model"), dtype="float32")
            ra.prepare_weights(os.path.join(d, "model"), d)
            ra.write_prompts(os.path.join(d, "p8.txt"), bench_prompts(cfg["vocab_size"], args.batch))
            ra.write_prompts(os.path.join(d, "p1.txt"), bench_prompts(cfg["vocab_size"], 1))
            import torch
            g = torch.Generator().manual_seed(99)
            n = cfg["n_positions"]
            ra.write_prompts(os.path.join(d, "pf.txt"),
                             [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for _ in range(PREFILL_TOKENS // n)])
            clocks = ClockSampler()
            clocks.start()
            dec = ra.run(exe, d, ["decode", "p8.txt", str(steps), str(warmup)])
            clk = clocks.stop()
            b1 = ra.run(exe, d, ["decode", "p1.txt", str(steps), str(warmup)]) if not args.no_points else None
            pf = ra.run(exe, d, ["prefill", "pf.txt", "5", "3"]) if not args.no_points else None
    except (ra.ReferenceUnavailable, subprocess.TimeoutExpired, ValueError) as e:
        return unavailable(e)
    B = args.batch
    ms = dec["device_ms_per_step"]
    mean_ctx = dec["first_context"] + (steps + 1) / 2.0
    # what the reference's step has to read: its float32 weights once (wte through the transposed copy its head
    # uses, and the rows of wte/wpe the embedding gathers) and the float32 cache of the live requests
    D, L, F, V = cfg["n_embd"], cfg["n_layer"], cfg["n_inner"], cfg["vocab_size"]
    wbytes = 4.0 * (V * D + L * (3 * D * D + D * D + 2 * D * F + 9 * D + F) + 2 * D + 2 * B * D)
    nbytes = wbytes + B * mean_ctx * L * 2 * D * 4.0
    achieved = nbytes / (ms / 1e3) / 1e9
    blocks = sum(-(-(PROMPT_LEN + steps + 1) // ra.KV_BLOCK) for _ in range(B))
    # host -> device per step (src/model/gpt2_model.cu:474-475, 521-533, 569-588): ids and positions, then per layer
    # two slot words per request, the flat block table, offsets and lengths; device -> host: the sampled ids (:670-675)
    h2d = 4 * (2 * B + L * (4 * B + blocks))
    conf = base_config(cfg, B, round(mean_ctx, 1), pk)
    line = {
        "impl": "reference",
        "note": f"the reference's pool (4096 blocks) and batch limit (16) allow {most} decode steps at batch {B}; no batch 64",
        "metric": "decode tok/s at batch 8 (GPT-2 small, 512-token prompts, greedy)",
        "value": round(B * 1e3 / ms, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(B * 1e3 / ms / 854.41, 2) if B == 8 else None,
        "dtype": "fp32", "data": "synthetic (seeded random weights and token ids)", "config": conf,
        "e2e": {"value": round(B * 1e3 / dec["wall_ms_per_step"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * B},
        "gpu_launches": steps * (L * 7 + 4),
        "clocks": clk,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if pf is not None:
        fl = prefill_flops(cfg, [cfg["n_positions"]] * (PREFILL_TOKENS // cfg["n_positions"]), PREFILL_TOKENS // cfg["n_positions"])
        line["prefill"] = {"value": round(PREFILL_TOKENS / (pf["median_ms"] / 1e3), 1), "tokens": PREFILL_TOKENS,
                           "ms": round(pf["median_ms"], 3),
                           "frac": round(fl / (pf["median_ms"] / 1e3) / fp32_peak_flops(), 4)}
    if b1 is not None:
        line["points"] = {"decode_b1": round(1e3 / b1["device_ms_per_step"], 1), "decode_b64": None,
                          "e2e_decode_b1": round(1e3 / b1["wall_ms_per_step"], 1)}
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="float32", choices=["bfloat16", "float32"],
                    help="precision of the headline numbers; the other precision goes into 'points'")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=SMALL["n_layer"], help="fewer layers than GPT-2 small's 12, if needed")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64, prefill and other-precision measurements")
    ap.add_argument("--profile-step", choices=["prefill", "decode"],
                    help="run one small eager step for a profiler instead of the benchmark")
    ap.add_argument("--kernel-times", action="store_true",
                    help="with --profile-step: time every launch of one eager step with CUDA events and print the shares")
    ap.add_argument("--attention", choices=["auto", "mma_sync"], default="auto",
                    help="mma_sync: prompt portions stay on the mma.sync attention kernel (to compare or profile it)")
    ap.add_argument("--workload", choices=["medium", "xl"],
                    help="run a continuous-batching workload of GPT-2 medium or XL instead of the benchmark")
    args = ap.parse_args()
    if args.attention == "mma_sync":
        from mini_llm_b200 import ops
        ops.use_tcgen05_attention = False
    if args.profile_step:
        return profile_step(args.profile_step, args.dtype, args.layers, args.batch, args.kernel_times)
    if args.workload:
        return run_workload(args.workload, args.dtype, args.layers if args.layers != SMALL["n_layer"] else 0)
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    args.steps = decode_steps(SMALL, args.steps)        # a request has 512 positions left after its prompt
    import torch
    import mini_llm_b200 as m

    pk = peaks()
    cfg = dict(SMALL, n_layer=args.layers)
    other = "bfloat16" if args.dtype == "float32" else "float32"
    short = {"bfloat16": "bf16", "float32": "fp32"}

    def prefill_entry(d, dtype):
        pf = run_prefill(d, dtype)
        peak_fl = pk["bf16_tflops"] * 1e12 if dtype == "bfloat16" else fp32_peak_flops()
        return {"value": round(pf["tok_s"], 1), "tokens": PREFILL_TOKENS, "ms": round(pf["ms"], 3),
                "frac": round(pf["flops"] / (pf["ms"] / 1e3) / peak_fl, 4)}

    points, prefill = {}, None
    with tempfile.TemporaryDirectory(prefix="mini_llm_bench_") as d:
        m.write_random_model(cfg, 0, d, dtype=args.dtype)
        main_run = run_decode(d, args.dtype, args.batch, args.steps, args.warmup, sample_clocks=True)
        e2e = run_e2e(d, args.dtype, args.batch, args.steps, args.warmup)
        if not args.no_points:
            for b in (1, 64):
                r = run_decode(d, args.dtype, b, args.steps, args.warmup)
                points[f"decode_b{b}"] = round(r["tok_s"], 1)
                points[f"decode_b{b}_hbm_frac"] = round(r["bytes"] / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"], 4)
            points["e2e_decode_b1"] = round(run_e2e(d, args.dtype, 1, args.steps, args.warmup)["tok_s"], 1)
            prefill = prefill_entry(d, args.dtype)
    if not args.no_points:
        # the other precision of the same model: every figure carries its dtype in its name
        o = short[other]
        with tempfile.TemporaryDirectory(prefix="mini_llm_bench_") as d:
            m.write_random_model(cfg, 0, d, dtype=other)
            for b in (1, args.batch, 64):
                r = run_decode(d, other, b, args.steps, args.warmup)
                points[f"{o}_decode_b{b}"] = round(r["tok_s"], 1)
                points[f"{o}_decode_b{b}_hbm_frac"] = round(r["bytes"] / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"], 4)
            points[f"{o}_e2e_decode_b{args.batch}"] = round(run_e2e(d, other, args.batch, args.steps, args.warmup)["tok_s"], 1)
            pe = prefill_entry(d, other)
            points[f"{o}_prefill_tok_s"], points[f"{o}_prefill_ms"], points[f"{o}_prefill_frac"] = pe["value"], pe["ms"], pe["frac"]
    achieved = main_run["bytes"] / (main_run["ms_per_step"] / 1e3) / 1e9
    line = {
        "metric": "decode tok/s at batch 8 (GPT-2 small, 512-token prompts, greedy)",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": main_run["steps"],
        "warmup": main_run["warmup"], "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": round(main_run["tok_s"] / 854.41, 2) if args.batch == 8 else None,
        "dtype": short[args.dtype], "data": "synthetic (seeded random weights and token ids)",
        "config": base_config(cfg, args.batch, round(main_run["mean_ctx"], 1), pk),
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d"],
                "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": main_run["launches"],
        "clocks": main_run["clocks"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if prefill is not None:
        line["prefill"] = prefill
    if points:
        line["points"] = points
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
