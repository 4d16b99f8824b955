"""Generates tests/golden/reference_vectors.npz from the REFERENCE'S OWN code.

Run where the reference tree is available and oracle/_ref has been built
(`make -C oracle ref`):   python tests/golden/make_golden.py

Every output array in the file was produced by reference source code, not by
the oracle:
  * gemm_k1_*/gemm_k2_*  cu_GEMM_fp32_spec / cu_GEMM_fp32_ABC_spec
                         (srcs/GEMM/CUDA/large_squares/GEMM.cuh:31-100, :206-280) on host threads
  * pack_*               cu_sIm2Col_r8_within (srcs/convolution/CUDA/im2col/im2col.cuh:86-178)
  * conv_*               the whole Conv2_MK_im2col driver (conv2_mk_im2col.h:57-274) incl. cu_conv_eq_mm
  * cpu_gemm_1024_*      decx::sgemm_caller<4,2> (srcs/GEMM/CPU/sgemm_callers.h:1227-1249),
                         BASELINE config 1 (1024^3): SHA-256 of the result bytes + a strided sample
Arrays above 32 KiB are stored as SHA-256 of their bytes (in `cases["sha256"]`) plus every
97th element (`<name>__sample`).  Inputs are not stored: they are seeded (oracle.fill_uniform / make_tensor /
make_filters with the seeds recorded in `cases`), so the file stays small.
"""
import hashlib
import json
import os
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle as o  # noqa: E402

GEMM_CASES = [  # name, M, N, K, with_C
    ("gemm_k1_128x128x64", 128, 128, 64, False),
    ("gemm_k2_128x128x64", 128, 128, 64, True),
    ("gemm_k1_100x70x50", 100, 70, 50, False),      # padded to 128/128/64 by the host driver
    ("gemm_k1_256x128x160", 256, 128, 160, False),
]
CONV_CASES = [  # name, W, H, depth, kW, kH, N, flag
    ("bc_12x20x6_k5x3_n5", 12, 20, 6, 5, 3, 5, 1),
    ("nb_22x19x6_k3x5_n5", 22, 19, 6, 3, 5, 5, 0),
    ("bc_9x7x3_k3x3_n2", 9, 7, 3, 3, 3, 2, 1),
    ("bc_70x18x4_k3x3_n33", 70, 18, 4, 3, 3, 33, 1),
    ("nb_17x33x8_k7x5_n4", 17, 33, 8, 7, 5, 4, 0),
    ("bc_28x28x64_k3x3_n64", 28, 28, 64, 3, 3, 64, 1),  # config 3 at 1/8 scale
    ("bc_8x8x16_k17x17_n3", 8, 8, 16, 17, 17, 3, 1),     # largest kernel the fixed apron allows
]


BIG = 32768  # arrays above this many bytes are stored as SHA-256 + a strided sample


def main():
    assert o.ref_kernels() is not None and o.ref_cpu_available(), "build oracle/_ref first"
    raw = {}
    cases = {"gemm": [], "conv": [], "sha256": {}}

    class Out(dict):
        def __setitem__(self, k, v):
            if isinstance(v, np.ndarray) and v.nbytes > BIG:
                cases["sha256"][k] = hashlib.sha256(np.ascontiguousarray(v).tobytes()).hexdigest()
                dict.__setitem__(self, k + "__sample", v.reshape(-1)[::97].copy())
            else:
                dict.__setitem__(self, k, v)

    out = Out()
    for name, M, N, K, with_c in GEMM_CASES:
        A = o.fill_uniform(M * K, 1).reshape(M, K)
        B = o.fill_uniform(K * N, 2).reshape(K, N)
        Cin = o.fill_uniform(M * N, 3).reshape(M, N) if with_c else None
        out[name] = o.ref_gemm_spec(A, B, Cin)
        cases["gemm"].append(dict(name=name, M=M, N=N, K=K, with_c=with_c, seeds=[1, 2, 3]))
    for name, W, H, C, kW, kH, N, flag in CONV_CASES:
        src = o.make_tensor(W, H, C, 4)
        flt = o.make_filters(kW, kH, C, N, 5)
        out["pack_" + name] = o.ref_im2col_pack(src, W, C, kW, kH, flag)
        out["conv_" + name] = o.ref_conv2_im2col(src, W, C, flt, kW, flag)
        cases["conv"].append(dict(name=name, W=W, H=H, depth=C, kW=kW, kH=kH, N=N, flag=flag, seeds=[4, 5]))
    with tempfile.TemporaryDirectory() as td:
        f = os.path.join(td, "c.bin")
        o.ref_cpu_gemm(1024, 1024, 1024, "seed:1", "seed:2", reps=1, out=f, split=(4, 2))
        Cref = np.fromfile(f, dtype=np.float32).reshape(1024, 1024)
    out["cpu_gemm_1024_sample"] = Cref[::64, ::64].copy()
    cases["cpu_gemm_1024_sha256"] = hashlib.sha256(Cref.tobytes()).hexdigest()
    out["cases_json"] = np.frombuffer(json.dumps(cases).encode(), dtype=np.uint8)
    dst = Path(__file__).with_name("reference_vectors.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, dst.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
