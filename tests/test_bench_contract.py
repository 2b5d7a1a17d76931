"""bench.py's answers that need no GPU: more than one GPU is refused with one line and exit
code 2, the reference arm answers with one line of its own where it cannot run, and the helpers
that turn a run into bytes and flops count what they say.  (That the reference arm runs where it
can is the GPU box's business: tests/test_reference_anchor_gpu.py builds and runs the reference.)"""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          cwd=ROOT, timeout=120)


def test_more_than_one_gpu_is_refused_with_one_line():
    p = _run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert p.returncode == 2
    lines = [ln for ln in p.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_answers_with_one_line():
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("with a GPU the arm runs the reference: covered by the GPU tests")
    p = _run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert p.returncode == 0
    lines = [ln for ln in p.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and "no CUDA device" in line["unavailable"]


def test_reference_limits_are_the_ones_of_its_constants():
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ra
    # 4096 blocks / 12 layers / 8 requests = 42 blocks = 672 tokens: 512 prompt + 1 + 159 steps
    assert ra.most_decode_steps(8, 512) == 159
    assert ra.most_decode_steps(1, 512) == 1024 - 512 - 1
    assert ra.most_decode_steps(16, 512) == 0
    assert ra.blocks_needed([512] * 8, 21) == 8 * 34 * 12


def test_decode_steps_leave_room_for_the_prompt():
    sys.path.insert(0, ROOT)
    import bench
    n = bench.SMALL["n_positions"]
    assert bench.decode_steps(bench.SMALL, 10 ** 6) == n - bench.PROMPT_LEN
    assert bench.decode_steps(bench.SMALL, 5) == 5


def test_prefill_flops_count_products_and_attention():
    sys.path.insert(0, ROOT)
    import bench
    cfg = dict(bench.SMALL, n_layer=1, n_embd=8, n_inner=32, n_head=2, vocab_size=10)
    # one request of 4 tokens, logits for 1 row: products 2*T*(3d*d + d*d + 2*d*inner) + head 2*rows*V*d,
    # attention 2 * 2 * d * sum over tokens of the keys they see
    d, inner, T = 8, 32, 4
    want = 2 * T * (3 * d * d + d * d + 2 * d * inner) + 2 * 1 * 10 * d + 4 * d * (1 + 2 + 3 + 4)
    assert bench.prefill_flops(cfg, [T], 1) == want
