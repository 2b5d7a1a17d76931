"""Builds and runs the unmodified reference (taejuk/mini-llm) beside this engine.

The reference is a CMake C++/CUDA project without Python packaging, so there is nothing for pip
to install.  Its sources are copied, unchanged, into ``baseline/_ref`` (kept out of the history);
this module compiles the translation units its CMakeLists.txt lists for ``mini_llm_kernels`` and
``mini_llm_model`` (CMakeLists.txt:40-75) together with ``baseline/reference_arm.cu``, a main()
that calls only ``GPT2Model::prefill / decode`` and the two logits hooks, with nvcc for sm_100a.
The reference reads its weights from a folder fixed at compile time (``WEIGHTS_DIR``,
CMakeLists.txt:37-39): here the relative folder ``weights``, so the program is started in a
folder that holds ``weights/*.bin`` written by ``mini_llm_b200.weights.reference_bins``.

Nothing of this engine is on the reference's path: the program links the CUDA runtime and cuBLAS
(which the reference links but uses only when MINI_LLM_USE_CUBLAS is set; it is not set here).
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
from typing import Dict, List, Optional, Sequence

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
MAIN_CU = os.path.join(HERE, "reference_arm.cu")

# the translation units of the reference's two libraries, as its CMakeLists.txt lists them
KERNEL_SOURCES = ["src/kernels/gemm.cu", "src/kernels/linear.cu", "src/kernels/embedding.cu", "src/kernels/layernorm.cu",
                  "src/kernels/residual.cu", "src/kernels/gelu.cu", "src/kernels/prefill/append_kv.cu",
                  "src/kernels/prefill/flashattention.cu", "src/kernels/decode/paged_attention.cu",
                  "src/kernels/decode_gemm.cu", "src/kernels/argmax.cu"]
MODEL_SOURCES = ["src/model/gpt2_model.cu", "src/model/gpt2_test_api.cu"]

# limits of the reference (include/constants.h:16-26)
MAX_BATCH = 16
MAX_SEQ = 1024
KV_BLOCK = 16
TOTAL_KV_BLOCKS = 4096
N_LAYERS = 12


class ReferenceUnavailable(RuntimeError):
    """The reference cannot be built or run here; the message is one line."""


def _nvcc() -> str:
    for cand in (os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise ReferenceUnavailable("nvcc not found, the reference cannot be compiled")


def have_sources(ref_dir: str = REF_DIR) -> bool:
    return all(os.path.isfile(os.path.join(ref_dir, s)) for s in KERNEL_SOURCES + MODEL_SOURCES)


def fetch_sources(origin: str, ref_dir: str = REF_DIR) -> None:
    """Copy the reference's product sources, unchanged and in its own layout, from ``origin``."""
    for sub in ("include", "src", "scripts"):
        shutil.copytree(os.path.join(origin, sub), os.path.join(ref_dir, sub), dirs_exist_ok=True)
    for sub in ("benchmarks/gpt2", "tests/cpp"):
        shutil.copytree(os.path.join(origin, sub), os.path.join(ref_dir, sub), dirs_exist_ok=True)
    for f in ("CMakeLists.txt", "README.md"):
        shutil.copy2(os.path.join(origin, f), os.path.join(ref_dir, f))


def _digest(ref_dir: str) -> str:
    h = hashlib.sha256()
    paths = [os.path.join(ref_dir, s) for s in KERNEL_SOURCES + MODEL_SOURCES] + [MAIN_CU]
    for root, _, files in os.walk(os.path.join(ref_dir, "include")):
        paths += [os.path.join(root, f) for f in files]
    for p in sorted(paths):
        h.update(p.encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def build(ref_dir: str = REF_DIR, verbose: bool = True) -> str:
    """Compile the reference with reference_arm.cu; returns the program's path.  Built once per source state."""
    if not have_sources(ref_dir):
        raise ReferenceUnavailable(f"the reference's sources are not in {os.path.relpath(ref_dir, os.path.dirname(HERE))} "
                                   "(it is kept out of the history; copy taejuk/mini-llm there unchanged)")
    bdir = os.path.join(ref_dir, "_build")
    try:
        os.makedirs(bdir, exist_ok=True)
        with open(os.path.join(bdir, ".w"), "w"):
            pass
    except OSError:
        bdir = os.path.join(tempfile.gettempdir(), f"mini_llm_reference_build_{os.getuid()}")
        os.makedirs(bdir, exist_ok=True)
    exe = os.path.join(bdir, "reference_arm")
    stamp = os.path.join(bdir, "reference_arm.stamp")
    want = _digest(ref_dir)
    if os.path.isfile(exe) and os.path.isfile(stamp) and open(stamp).read().strip() == want:
        return exe
    cmd = [_nvcc(), "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I", os.path.join(ref_dir, "include"),
           '-DWEIGHTS_DIR="weights"', *[os.path.join(ref_dir, s) for s in KERNEL_SOURCES + MODEL_SOURCES], MAIN_CU,
           "-lcublas", "-o", exe + ".tmp"]
    if verbose:
        print("[reference arm] compiling the reference for sm_100a (once, about half a minute)", file=sys.stderr, flush=True)
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise ReferenceUnavailable("nvcc failed on the reference: " + " ".join(p.stdout.strip().splitlines()[-3:])[:300])
    os.replace(exe + ".tmp", exe)
    with open(stamp, "w") as f:
        f.write(want)
    return exe


def blocks_needed(prompt_lens: Sequence[int], new_tokens: int) -> int:
    """KV blocks the reference needs: one table per layer and request (src/runtime/real_kv_allocator.cu:112-139)."""
    return sum(-(-(n + new_tokens) // KV_BLOCK) for n in prompt_lens) * N_LAYERS


def most_decode_steps(batch: int, prompt_len: int) -> int:
    """How many decode steps (timed + warm-up) ``batch`` requests of ``prompt_len`` tokens can run inside the
    reference's pool of 4096 blocks and its 1024 positions."""
    per_request = (TOTAL_KV_BLOCKS // N_LAYERS // batch) * KV_BLOCK
    return max(0, min(per_request, MAX_SEQ) - prompt_len - 1)


def write_prompts(path: str, prompts: Sequence[Sequence[int]]) -> None:
    with open(path, "w") as f:
        for p in prompts:
            f.write(" ".join(str(int(t)) for t in p) + "\n")


def run(exe: str, work_dir: str, args: List[str], timeout: float = 900.0) -> Dict:
    """Start the program in ``work_dir`` (which holds ``weights/``) and parse its one JSON line."""
    p = subprocess.run([exe, *args], cwd=work_dir, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=timeout)
    if p.returncode != 0:
        raise ReferenceUnavailable(f"the reference exited with {p.returncode}: " + " ".join(p.stderr.strip().splitlines()[-2:])[:300])
    for line in reversed(p.stdout.strip().splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    raise ReferenceUnavailable("the reference printed no result line")


def prepare_weights(model_dir: str, work_dir: str) -> str:
    """``work_dir/weights/*.bin`` from a GPT-2 small model folder."""
    root = os.path.dirname(HERE)
    if root not in sys.path:
        sys.path.insert(0, root)
    from mini_llm_b200.weights.reference_bins import write_reference_bins
    out = os.path.join(work_dir, "weights")
    write_reference_bins(model_dir, out)
    return out
