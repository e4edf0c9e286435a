"""Regenerates the fixtures in this folder from the REFERENCE implementation.

Run where a checkout of the reference (usyd-fsalab/fp6_llm) is available; pass its path, or set FP6_LLM_REFERENCE:
    python tests/golden/make_golden.py [reference_root]

* prepack_dequant_e{E}m{M}.npz : seeded random unpacked weights and scales, with the outputs of the reference's
  own CPU functions weight_matrix_prepacking_fp_eXmY / dequant_matrix_fp_eXmY_to_fp16 (compiled from the
  reference sources by oracle/Makefile into oracle/_ref).
* all_codes_e{E}m{M}.npz       : a matrix that holds every code value in every position class, same outputs.
* splitk_heuristic.json        : values of the reference's pure-Python Num_Wave / HeuristicFuntion_SplitK
  (fp6_llm/__init__.py:6-23), obtained by executing those two function definitions.
"""
import json
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle  # noqa: E402


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else None   # a checkout of usyd-fsalab/fp6_llm; default: see oracle.build
    oracle.build(ref_root)
    assert oracle.have_ref(), "oracle/_ref was not built: reference tree missing?"
    rng = np.random.default_rng(20240607)
    # the two formats the reference dispatches, then three more instantiations of its templates (same generator, appended)
    for e, m in ((3, 2), (2, 2), (2, 1), (3, 1), (2, 3)):
        bw = 1 + e + m
        rows, cols = 256, 192
        w = rng.integers(-2**31, 2**31, size=(rows, cols * bw // 32), dtype=np.int64).astype(np.int32)
        scale = rng.uniform(1e-3, 2.0, size=rows).astype(np.float16)
        np.savez_compressed(os.path.join(HERE, f"prepack_dequant_e{e}m{m}.npz"), unpacked=w, scale=scale,
                            packed=oracle.ref_prepack(w, e, m), dequant=oracle.ref_dequant(w, scale, e, m))
        # every code at every column-in-block position and several rows: code = (r*7 + c*3 + r//16) mod 2^bw
        rows, cols = 256, 64
        r = np.arange(rows)[:, None]
        c = np.arange(cols)[None, :]
        codes = ((r * 7 + c * 3 + r // 16) % (1 << bw)).astype(np.int64)
        bits = ((codes[:, :, None] >> (bw - 1 - np.arange(bw, dtype=np.int64))[None, None, :]) & 1).astype(np.uint8)
        w = np.packbits(bits.reshape(rows, -1), axis=1).view(np.int32).copy()
        scale = np.ones(rows, dtype=np.float16)
        np.savez_compressed(os.path.join(HERE, f"all_codes_e{e}m{m}.npz"), unpacked=w, scale=scale, codes=codes.astype(np.uint8),
                            packed=oracle.ref_prepack(w, e, m), dequant=oracle.ref_dequant(w, scale, e, m))

    ref_root = ref_root or oracle._find_reference()
    src = open(os.path.join(ref_root, "fp6_llm", "__init__.py")).read()
    src = "\n".join(line for line in src.splitlines() if not re.match(r"\s*from fp6_llm_cuda import", line))
    ns = {}
    exec(compile(src, "reference_fp6_llm_init", "exec"), ns)
    cases = []
    for M in (256, 4096, 5120, 8192, 10240, 12288, 15360, 22016, 27648, 57344):
        for N in (1, 8, 16, 32, 64, 128, 512, 1024, 2048):
            for sms in (108, 132, 148):
                cases.append({"M": M, "N": N, "SMs": sms, "split_k": ns["HeuristicFuntion_SplitK"](M, N, sms),
                              "num_wave_k3": ns["Num_Wave"](M, N, 3, sms)})
    json.dump(cases, open(os.path.join(HERE, "splitk_heuristic.json"), "w"), indent=0)
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()
