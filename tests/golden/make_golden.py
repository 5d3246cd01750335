"""Generates tests/golden/reference_numpy_vectors.npz from the reference itself.

Run in a container that has the reference checkout mounted:

    python tests/golden/make_golden.py <path of the reference checkout>

(default: the directory ``reference`` beside this repository).

It imports ``rope``, ``softmax`` and ``rms_norm`` from the reference's
``bench/reference_numpy.py`` (the file cannot travel with this repository, so
its outputs are committed as small fixtures instead) and evaluates the
reference's attention statements (``bench/reference_numpy.py:170-181``: rotate
q and k, repeat K/V for GQA, scores / sqrt(hd), additive causal mask, softmax,
weighted sum) on seeded inputs.  ``tests/test_oracle_golden.py`` then requires
``oracle/attention_oracle.py`` to reproduce every stored output.
"""

from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np


def load_reference(root: Path):
    spec = importlib.util.spec_from_file_location(
        "reference_numpy", root / "bench" / "reference_numpy.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def reference_prefill(ref, q, k, v, n_q, n_kv, hd, theta):
    """The reference's attention block for one prompt, as its forward() does it."""
    seq = q.shape[0]
    pos = np.arange(seq)
    mask = np.triu(np.full((seq, seq), -np.inf), k=1)
    gqa = n_q // n_kv
    qr = ref.rope(q.reshape(seq, n_q, hd), pos, theta)
    kr = ref.rope(k.reshape(seq, n_kv, hd), pos, theta)
    vr = v.reshape(seq, n_kv, hd)
    kk = np.repeat(kr, gqa, axis=1)
    vv = np.repeat(vr, gqa, axis=1)
    scores = np.einsum("qhd,khd->hqk", qr, kk) / np.sqrt(hd)
    attn = ref.softmax(scores + mask[None, :, :], axis=-1)
    ctx = np.einsum("hqk,khd->qhd", attn, vv).reshape(seq, n_q * hd)
    return qr, kr, ctx


def main() -> None:
    root = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).resolve().parents[3] / "reference"
    ref = load_reference(root)
    out: dict[str, np.ndarray] = {}
    rng = np.random.default_rng(20250)

    # rope: small head counts, both head widths, far positions (long context).
    for tag, (seq, heads, hd, theta) in {
        "rope_a": (6, 3, 64, 1e6),
        "rope_b": (5, 2, 128, 1e4),
    }.items():
        x = rng.standard_normal((seq, heads, hd))
        pos = np.array([0, 1, 7, 513, 32767, 131071][:seq])
        out[f"{tag}_x"] = x
        out[f"{tag}_pos"] = pos
        out[f"{tag}_theta"] = np.float64(theta)
        out[f"{tag}_y"] = ref.rope(x, pos, theta)

    # rms_norm per head, as QK-norm applies it.
    x = rng.standard_normal((4, 5, 128))
    w = 1.0 + 0.02 * rng.standard_normal(128)
    out["norm_x"], out["norm_w"] = x, w
    out["norm_eps"] = np.float64(1e-6)
    out["norm_y"] = ref.rms_norm(x, w, 1e-6)

    # softmax including a -inf masked tail.
    s = rng.standard_normal((3, 4, 9)) * 4.0
    s[:, :, 6:] = -np.inf
    out["softmax_x"] = s
    out["softmax_y"] = ref.softmax(s, axis=-1)

    # the reference's causal attention block on two GQA shapes.
    for tag, (seq, n_q, n_kv, hd, theta) in {
        "attn_q14": (9, 14, 2, 64, 1e6),      # Qwen2.5-0.5B heads
        "attn_q8": (12, 8, 2, 128, 1e6),       # GQA-4, head_dim 128
    }.items():
        q = rng.standard_normal((seq, n_q * hd)).astype(np.float16).astype(np.float64)
        k = rng.standard_normal((seq, n_kv * hd)).astype(np.float16).astype(np.float64)
        v = rng.standard_normal((seq, n_kv * hd)).astype(np.float16).astype(np.float64)
        qr, kr, ctx = reference_prefill(ref, q, k, v, n_q, n_kv, hd, theta)
        out[f"{tag}_shape"] = np.array([seq, n_q, n_kv, hd])
        out[f"{tag}_theta"] = np.float64(theta)
        # inputs are fp16-representable by construction: store them as fp16
        out[f"{tag}_q"], out[f"{tag}_k"], out[f"{tag}_v"] = (
            q.astype(np.float16), k.astype(np.float16), v.astype(np.float16))
        out[f"{tag}_qrot"], out[f"{tag}_krot"], out[f"{tag}_ctx"] = qr, kr, ctx

    dst = Path(__file__).with_name("reference_numpy_vectors.npz")
    np.savez_compressed(dst, **out)
    print(f"wrote {dst} ({dst.stat().st_size} bytes, {len(out)} arrays)")


if __name__ == "__main__":
    main()
