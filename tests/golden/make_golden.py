"""Regenerates tests/golden/*.npz from the CPU oracle and the numpy generator.

    python tests/golden/make_golden.py

The reference (CUDAnative.jl) has no stored vectors for this path and cannot be run without Julia, so
these fixtures pin the three statements of the same arithmetic against each other instead: the C
oracle (oracle/oracle.c), its numpy front end (oracle/oracle.py) and the library's generator
(cudanative.jl_b200/rng.py; csrc/rng.cuh on the device).  Inputs are the benchmark configurations'
own seeds and distributions, cut down to sizes a CPU test handles in milliseconds.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

HERE = Path(__file__).resolve().parent


def main():
    pkg = entry.load_package()
    oracle = entry.load_oracle()
    rng = pkg.rng
    # 1. generator known answers: first values of each distribution for a few (seed, matrix) pairs
    kat = {}
    for seed in (0, 1, 4):
        for mid in (0, 1, 2):
            for dist, name in ((rng.UNIFORM, "u"), (rng.NORMAL, "n")):
                kat[f"s{seed}_m{mid}_{name}"] = rng.synth_values(seed, mid, np.arange(16, dtype=np.uint64) * np.uint64(1000003), dist)
    np.savez(HERE / "rng_kat.npz", **kat)
    # 2. benchmark config 1: 16x16x16, uniform[-1,1), seed 0, D = A*B + C
    a = rng.matrix(0, 0, 16, 16, rng.UNIFORM, 1.0, np.float16)
    b = rng.matrix(0, 1, 16, 16, rng.UNIFORM, 1.0, np.float16)
    c = rng.matrix(0, 2, 16, 16, rng.UNIFORM, 1.0, np.float32)
    np.savez(HERE / "config1_unit.npz", a=a, b=b, c=c, d=oracle.wmma_unit_ref(a, b, c),
             d_half_c=oracle.wmma_unit_ref(a, b, c, beta=0.5),
             d_rowmajor_f16=oracle.wmma_unit_ref(a, b, c.astype(np.float16), a_layout=1, b_layout=1, c_layout=1, d_layout=1,
                                                 d_type=np.float16, alpha=np.float16(0.75), beta=np.float16(0.25)))
    # 3. a cut-down config 3 (A row-major, B column-major, alpha=2, beta=0.5, seed 2): 96 x 80 x 200
    M, N, K = 96, 80, 200
    a = rng.matrix(2, 0, K, M, rng.NORMAL, K ** -0.5, np.float16)  # stored K x M
    b = rng.matrix(2, 1, K, N, rng.NORMAL, K ** -0.5, np.float16)
    c = rng.matrix(2, 2, M, N, rng.UNIFORM, 1.0, np.float32)
    np.savez(HERE / "config3_small.npz", a=a, b=b, c=c, d=oracle.gemm_ref(True, False, 2.0, a, b, 0.5, c),
             d64=oracle.gemm_c(True, False, 2.0, a.astype(np.float32), b.astype(np.float32), 0.5, c, True))
    # 4. bfloat16 operands (bit patterns in uint16), two matrices of a batch: 72 x 40 x 136, alpha=1.25, beta=0.5, seed 6;
    #    outputs in binary32 and, rounded once more, in bfloat16
    M, N, K = 72, 40, 136
    fix = {}
    for i in range(2):
        a = oracle.bf16_round(rng.matrix(6 + i, 0, M, K, rng.NORMAL, K ** -0.5, np.float32))
        b = oracle.bf16_round(rng.matrix(6 + i, 1, K, N, rng.NORMAL, 1.0, np.float32))
        c = rng.matrix(6 + i, 2, M, N, rng.UNIFORM, 1.0, np.float32)
        d = oracle.gemm_c(False, False, 1.25, oracle.bf16_widen(a), oracle.bf16_widen(b), 0.5, c, True)
        fix.update({f"a{i}": a, f"b{i}": b, f"c{i}": c, f"d{i}": d, f"d{i}_bf16": oracle.bf16_round(d)})
    np.savez(HERE / "bf16_batch_small.npz", **fix)
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    main()
