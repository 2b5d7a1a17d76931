"""bench.py's answers that need no GPU: more than one GPU is refused with one line and exit
code 2, the reference arm says why it is unavailable, and the helpers that turn a run into
bytes and flops count what they say."""
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


def test_reference_arm_reports_unavailable():
    p = _run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert p.returncode == 0
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and "\n" not in line["unavailable"]


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
