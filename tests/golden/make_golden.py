"""Makes tests/golden/reference_kernels.npz from the reference's own NumPy oracles.

    python tests/golden/make_golden.py --reference <checkout of taejuk/mini-llm>

The reference's model code is CUDA-only with compile-time sizes and cannot run on a
CPU, but its kernel oracles can: tests/kernels/{layernorm,gelu,embedding,linear}/gen.py
are NumPy scripts that write their inputs and expected outputs as raw float32 files
next to themselves.  This script runs them unchanged in a temporary copy and keeps
what the comparison in tests/test_plain.py needs: the inputs where they are small,
and the expected outputs (the linear case's inputs are re-drawn in the test from the
same NumPy seed).
"""
import argparse
import json
import os
import shutil
import subprocess
import sys
import tempfile

import numpy as np


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    here = os.path.dirname(os.path.abspath(__file__))
    with tempfile.TemporaryDirectory() as tmp:
        work = os.path.join(tmp, "kernels")
        shutil.copytree(os.path.join(args.reference, "tests", "kernels"), work)
        out = {}
        for name in ("layernorm", "gelu", "embedding", "linear"):
            d = os.path.join(work, name)
            subprocess.run([sys.executable, "gen.py"], cwd=d, check=True)
            meta = json.load(open(os.path.join(d, "meta.json")))

            def rd(f, dt=np.float32):
                return np.fromfile(os.path.join(d, f), dtype=dt)

            if name == "layernorm":
                r, c = meta["rows"], meta["cols"]
                out["layernorm_x"] = rd("input_x.bin").reshape(r, c)[:3]
                out["layernorm_gamma"] = rd("input_gamma.bin")
                out["layernorm_beta"] = rd("input_beta.bin")
                out["layernorm_eps"] = np.float64(meta["eps"])
                out["layernorm_y"] = rd("expected.bin").reshape(r, c)[:3]
            elif name == "gelu":
                out["gelu_x"] = rd("input_x.bin")
                out["gelu_y"] = rd("expected.bin")
            elif name == "embedding":
                out["embedding_tokens"] = rd("tokens.bin", np.int32)
                out["embedding_y"] = rd("expected.bin").reshape(meta["seq"], meta["D"])
                out["embedding_dims"] = np.array([meta["vocab"], meta["max_seq"], meta["D"]])
            elif name == "linear":
                out["linear_dims"] = np.array([meta["M"], meta["K"], meta["N"]])
                out["linear_y"] = rd("expected.bin").reshape(meta["M"], meta["N"])
        np.savez_compressed(os.path.join(here, "reference_kernels.npz"), **out)
    print("wrote", os.path.join(here, "reference_kernels.npz"))


if __name__ == "__main__":
    main()
