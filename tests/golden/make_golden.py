"""Generates the committed golden fixtures in this folder from the CPU oracle.

Run from the repository root: ``python tests/golden/make_golden.py``.  Each .npz holds the
seeded inputs (packed weights, scale, activations) and the oracle's outputs (int8
activations, per-token scales, int32 accumulators, fp32 outputs) of one small case, so a
test can check any implementation without regenerating anything.
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))
import oracle  # noqa: E402

# name, seed, M, K, N
CASES = [
    ("decode_m1_k256_n48", 11, 1, 256, 48),
    ("decode_m8_k640_n100", 12, 8, 640, 100),
    ("decode_m13_k1024_n72", 13, 13, 1024, 72),
    ("ragged_m3_k37_n29", 14, 3, 37, 29),
    ("prefill_m256_k256_n128", 15, 256, 256, 128),
]


def main():
    for name, seed, M, K, N in CASES:
        wp = oracle.gen_ternary_packed(seed, 1, N * K)
        x = oracle.gen_activations(seed, 2, (M, K))
        ws = np.float32(oracle.gen_weight_scale(seed, 1, K))
        ref = oracle.bitlinear_forward(wp, float(ws), x, N)
        np.savez_compressed(HERE / f"{name}.npz", wp=wp, w_scale=ws, x=x, M=M, K=K, N=N, **ref)
    # FFN block
    seed, M, H, F = 21, 4, 128, 320
    g, u, d = (oracle.gen_ternary_packed(seed, i, F * H) for i in (1, 2, 3))
    sg, su, sd = (np.float32(oracle.gen_weight_scale(seed, i, k)) for i, k in ((1, H), (2, H), (3, F)))
    x = oracle.gen_activations(seed, 4, (M, H))
    y, h = oracle.ffn_forward(g, float(sg), u, float(su), d, float(sd), x, F)
    np.savez_compressed(HERE / "ffn_m4_h128_f320.npz", gate=g, up=u, down=d, s_gate=sg, s_up=su, s_down=sd,
                        x=x, y=y, h=h, M=M, hidden=H, ffn=F)
    print("wrote", len(CASES) + 1, "fixtures to", HERE)


if __name__ == "__main__":
    main()
