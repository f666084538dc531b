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


class _Prescribed:
    """Stands in for a decoded weight matrix: `lhs @ self` returns had(want), so that the reference's
    linear() = had(had(x * suh) @ what) * svh yields `want` (its Hadamard transform is an involution)."""
    __array_ufunc__ = None

    def __init__(self, had_want):
        self.had_want = had_want

    def __rmatmul__(self, lhs):
        assert lhs.shape[0] == self.had_want.shape[0]
        return self.had_want


class _StubCkpt:
    """The two methods ref/oracle.py::gdn and ::qsa use (ref/oracle.py:47-55)."""

    def __init__(self, arrays, lins):
        self.arrays, self.lins = arrays, lins

    def f64(self, name):
        return np.asarray(self.arrays[name], np.float64)

    def lin(self, prefix):
        return self.lins[prefix]


def layer_vectors(ro):
    out = {}
    f16 = lambda a: np.asarray(a, np.float16).astype(np.float64)          # exactly representable inputs
    ident = lambda want: (_Prescribed(ro.had(want)), np.ones(1), np.ones(1))

    class _Identity:
        __array_ufunc__ = None

        def __rmatmul__(self, lhs):
            return lhs

    # ---- GDN: 20 rows, 48 value / 16 key heads
    rng = np.random.default_rng(21)
    n, hid = 20, 128
    x = f16(rng.normal(size=(n, hid)))
    qkv, z = f16(rng.normal(size=(n, 10240))), f16(rng.normal(size=(n, 6144)))
    wa, wb = f16(rng.normal(size=(48, hid)) * 0.1), f16(rng.normal(size=(48, hid)) * 0.1)
    conv = f16(rng.normal(size=(10240, 4)) * 0.5)
    A_log, dtb = f16(np.clip(rng.normal(-1, 1.5, 48), -5, 1.5)), f16(rng.normal(size=48) * 0.5)
    gamma = f16(1 + 0.1 * rng.normal(size=128))
    p = "g."
    ck = _StubCkpt({p + "in_proj_a.weight": wa, p + "in_proj_b.weight": wb, p + "conv1d.weight": conv[:, None, :],
                    p + "A_log": A_log, p + "dt_bias": dtb, p + "norm.weight": gamma},
                   {p + "in_proj_qkv": ident(qkv), p + "in_proj_z": ident(z), p + "out_proj": (_Identity(), np.ones(1), np.ones(1))})
    o = ro.gdn(ck, p, x)                                   # = had(had(core output)) = core output
    for name, val in dict(x=x, qkv=qkv, z=z, wa=wa, wb=wb, conv=conv, A_log=A_log, dt_bias=dtb, gamma=gamma).items():
        out["layer_gdn_" + name] = val.astype(np.float16)
    out["layer_gdn_out"] = o
    # ---- QSA: 24 rows, dense causal, 24 query / 2 KV heads
    rng = np.random.default_rng(22)
    n = 24
    x = np.zeros((n, hid))
    q, k, v = f16(rng.normal(size=(n, 24 * 512))), f16(rng.normal(size=(n, 512))), f16(rng.normal(size=(n, 512)))
    qn, kn = f16(0.1 * rng.normal(size=256)), f16(0.1 * rng.normal(size=256))
    p = "a."
    ck = _StubCkpt({p + "q_norm.weight": qn, p + "k_norm.weight": kn},
                   {p + "q_proj": ident(q), p + "k_proj": ident(k), p + "v_proj": ident(v), p + "o_proj": (_Identity(), np.ones(1), np.ones(1))})
    o = ro.qsa(ck, p, x)
    for name, val in dict(q=q, k=k, v=v, q_norm=qn, k_norm=kn).items():
        out["layer_qsa_" + name] = val.astype(np.float16)
    out["layer_qsa_out"] = o
    return out


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

    # (6) the reference's own layer functions ref/oracle.py::gdn (:101-130) and ::qsa (:147-165), run at the
    # reference geometry (48/16 GDN heads, 24/2 QSA heads) on a duck-typed checkpoint: they only call ck.f64(name)
    # and ck.lin(prefix).  Projection outputs are prescribed (fp16-exact values, so the stored inputs are exact),
    # the output projection is the identity, so what comes back is the layer core's gated output.
    try:
        import oracle as ro
        out.update(layer_vectors(ro))
        out["layers"] = np.array(1)
    except Exception as e:
        print("ref/oracle.py layer functions not recorded:", e)
        out["layers"] = np.array(0)

    # (7) the YaRN rows of engine/layers/rope_tables.h (generated constants: 32 inverse frequencies + multiplier per mode)
    import re
    text = open(os.path.join(ref_root, "engine", "layers", "rope_tables.h")).read()
    rows = re.findall(r"\{\s*//\s*factor\s+(\d+).*?\n(.*?)\},", text, re.S)
    for factor, body in rows:
        vals = [float.fromhex(v.rstrip("f")) for v in re.findall(r"0x[0-9a-fA-F.]+p[+-]\d+f", body)]
        assert len(vals) == 33
        out["yarn_table_%s" % factor] = np.array(vals, np.float32)

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_vectors.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of the reference repository>")
    main(sys.argv[1])
