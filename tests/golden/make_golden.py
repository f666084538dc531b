"""Generates tests/golden/ref_vectors.npz by IMPORTING the reference's own CPU code
(ref/prefill_ref.py and the checkpoint-free helpers of ref/oracle.py) and recording its outputs on
seeded inputs.  Run where the reference tree is mounted:

    python tests/golden/make_golden.py /path/to/reference

The vectors pin oracle/attn_oracle.py (tests/test_oracle_golden.py); the GPU box never needs the
reference tree, only the committed .npz.
"""
import os
import sys
import numpy as np


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "ref"))
    import prefill_ref as pr          # ref/prefill_ref.py
    out = {}

    # (1) ref/test_prefill.py:7-19 — chunk == serial, rows {1,3,64,65,130}, seed 12, 8-wide heads.
    for rows in (1, 3, 64, 65, 130):
        rng = np.random.default_rng(12)
        q, k, v = [rng.normal(size=(rows, 8)) for _ in range(3)]
        q /= np.linalg.norm(q, axis=-1, keepdims=True) * np.sqrt(8)
        k /= np.linalg.norm(k, axis=-1, keepdims=True)
        g = -rng.uniform(0, 2, rows)
        beta = rng.uniform(0, 1, rows)
        init = rng.normal(size=(8, 8))
        ys, ss = pr.serial_gdn(q, k, v, g, beta, init)
        yc, sc = pr.chunk_gdn(q, k, v, g, beta, init)
        for name, val in dict(q=q, k=k, v=v, g=g, beta=beta, init=init, ys=ys, ss=ss, yc=yc, sc=sc).items():
            out[f"gdn8_{rows}_{name}"] = val

    # (2) a full-size head (128x128 state), 200 rows, decays like the engine's.
    rng = np.random.default_rng(7)
    rows = 200
    q, k, v = [rng.normal(size=(rows, 128)) for _ in range(3)]
    q /= np.linalg.norm(q, axis=-1, keepdims=True) * np.sqrt(128)
    k /= np.linalg.norm(k, axis=-1, keepdims=True)
    g = -np.exp(rng.normal(-1, 1.5, rows).clip(-5, 1.5)) * np.log1p(np.exp(rng.normal(size=rows)))
    beta = 1 / (1 + np.exp(-rng.normal(size=rows)))
    init = rng.normal(size=(128, 128)) * 0.05
    ys, ss = pr.serial_gdn(q, k, v, g, beta, init)
    yc, sc = pr.chunk_gdn(q, k, v, g, beta, init)
    for name, val in dict(q=q, k=k, v=v, g=g, beta=beta, init=init, ys=ys, ss=ss, yc=yc, sc=sc).items():
        out[f"gdn128_{name}"] = val

    # (3) ref/test_prefill.py:22-28 — decay underflow stays finite.
    q = k = v = np.ones((64, 2)) / np.sqrt(2)
    yu, su = pr.chunk_gdn(q, k, v, np.full(64, -100.), np.ones(64), np.ones((2, 2)))
    out["underflow_y"], out["underflow_s"] = yu, su

    # (4) ref/test_prefill.py:41-53 — visibility rule; plus seeded random scores with ties.
    for n in (2047, 2048, 2049, 2051, 2052, 2055, 2060):
        scores = np.zeros(n // 4)
        if n // 4 > 512:
            scores[512] = 1
        out[f"vis_{n}"] = pr.selected_tokens(scores, n)
    rng = np.random.default_rng(3)
    for n in (2100, 4099, 9001):
        scores = np.round(rng.uniform(0, 4, n // 4), 1).astype(np.float32)   # many exact ties
        out[f"sel_scores_{n}"] = scores
        out[f"sel_tokens_{n}"] = pr.selected_tokens(scores, n)

    # (5) checkpoint-free helpers of ref/oracle.py (rope, rms, sigmoid, silu, had).
    try:
        import oracle as ro               # ref/oracle.py
        rng = np.random.default_rng(5)
        x = rng.normal(size=(6, 3, 256))
        pos = np.array([0., 1., 5., 1000., 65537., 262143.])
        out["rope_x"], out["rope_pos"], out["rope_y"] = x, pos, ro.rope(x, pos)
        w1 = 1 + 0.1 * rng.normal(size=256)
        out["rms_w1"], out["rms_y"] = w1, ro.rms(x, w1)
        out["sigmoid_y"], out["silu_y"] = ro.sigmoid(x), ro.silu(x)
        ro.H128 = None
        out["had_y"] = ro.had(x)
        out["helpers"] = np.array(1)
    except Exception as e:  # torch/safetensors missing: helpers stay unpinned, recurrences are pinned
        print("ref/oracle.py helpers not recorded:", e)
        out["helpers"] = np.array(0)

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_vectors.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of the reference repository>")
    main(sys.argv[1])
