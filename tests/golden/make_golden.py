"""Generates the golden vectors under tests/golden/ from the REFERENCE's own host
functions (attn_ref_forward / attn_ref_backward / rand_vec of
kernels/tests/kernels_test.cu), reached through oracle/_ref/libhkref.so, which
`make -C oracle` builds from the reference sources where they are mounted.

Run in a container that has the reference mounted:   python tests/golden/make_golden.py

Outputs
  attn_ref_T256.npz   B=1,H=1,T=256,Hd=64, inputs = first 16384 values of the
                      reference test's seeds 101..104 (kernels_test.cu:499,545),
                      scale 1/8, causal and non-causal: O, LSE, D, dQ, dK, dV.
  attn_ref_T77.npz    B=1,H=2,T=77 (ragged), seeds 11..14, same outputs.
  checksums.json      sha256 of every output at the reference test's full shape
                      B=2,H=6,T=256 (kernels_test.cu:491) and of rand_vec heads.
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as ol  # noqa: E402


def run(B, H, T, seeds, causal):
    n = B * H * T * 64
    Q, K, V, dO = (ol.ref_rand_vec(n, s).reshape(B, H, T, 64) for s in seeds)
    O, LSE = ol.ref_attn_forward(Q, K, V, 0.125, causal)
    D, dQ, dK, dV = ol.ref_attn_backward(Q, K, V, O, dO, LSE, 0.125, causal)
    return dict(O=O, LSE=LSE, D=D, dQ=dQ, dK=dK, dV=dV)


def main():
    assert ol.reference() is not None, "build oracle/_ref first (make -C oracle)"
    for name, (B, H, T, seeds) in {"attn_ref_T256": (1, 1, 256, (101, 102, 103, 104)),
                                   "attn_ref_T77": (1, 2, 77, (11, 12, 13, 14))}.items():
        out = {}
        for causal in (0, 1):
            for k, v in run(B, H, T, seeds, causal).items():
                out[f"{k}_causal{causal}"] = v
        out["meta"] = np.array([B, H, T, 64] + list(seeds), dtype=np.int64)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    sums = {"rand_vec_head": {str(s): ol.ref_rand_vec(8, s).tolist() for s in (101, 102, 103, 104, 17, 18)}}
    for causal in (0, 1):
        for k, v in run(2, 6, 256, (101, 102, 103, 104), causal).items():
            sums[f"B2H6T256_{k}_causal{causal}"] = hashlib.sha256(np.ascontiguousarray(v).tobytes()).hexdigest()
    json.dump(sums, open(os.path.join(HERE, "checksums.json"), "w"), indent=1)


if __name__ == "__main__":
    main()
