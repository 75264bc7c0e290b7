"""Generate the golden fixtures under tests/golden/ from the reference itself.

Run in a container where the reference project is mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's NumPy-only host case and host oracle
(rocm/probe_w8a8_lora_forward.py: `_construct_host_case` :1193-1261 and
`_host_oracle` :1080-1113), which need neither JAX nor a GPU, and writes

* w8a8_host_case.npz ......... the reference's own known-answer case
  (M=3, K=64, N=17 padded to 32, group 64, rank 8, scaling 0.75) with the
  reference-computed expected output, and the SHA-256 digests the reference
  pins for every tensor (:210-218);
* w8a8_ref_oracle_cases.npz .. further seeded cases pushed through the SAME
  reference function (its module constants are rebound per case), covering a
  second row count, zero rows and the extreme code values.

The fixtures are small (a few KB) and are committed; the reference itself is
not needed to run the test-suite.
"""

from __future__ import annotations

import hashlib
import importlib.util
import json
import sys
from pathlib import Path

import ml_dtypes
import numpy as np

HERE = Path(__file__).resolve().parent


def _load_probe(reference_root: Path):
    path = reference_root / "rocm" / "probe_w8a8_lora_forward.py"
    spec = importlib.util.spec_from_file_location("ref_probe_w8a8", path)
    module = importlib.util.module_from_spec(spec)
    sys.modules["ref_probe_w8a8"] = module
    spec.loader.exec_module(module)
    return module


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes(order="C")).hexdigest()


def _u16(a):
    return np.asarray(a).view(np.uint16)


def main(reference_root: str) -> None:
    probe = _load_probe(Path(reference_root))
    args, _manifests, expected = probe._construct_host_case()
    x, codes, scales, lora_a, lora_b, scaling = args
    digests = dict(probe._EXPECTED_HOST_SHA256)
    observed = {
        "x": _sha(x), "weight_codes": _sha(codes), "weight_scales": _sha(scales),
        "lora_a": _sha(lora_a), "lora_b": _sha(lora_b), "lora_scaling": _sha(scaling),
        "expected": _sha(expected),
    }
    assert observed == digests, "reference host case does not reproduce its own pins"
    np.savez(
        HERE / "w8a8_host_case.npz",
        x_bf16=_u16(x), weight_codes=codes, weight_scales_bf16=_u16(scales),
        lora_a_bf16=_u16(lora_a), lora_b_bf16=_u16(lora_b), lora_scaling=scaling,
        expected_bf16=_u16(expected),
        out_features=np.int32(probe._OUT_FEATURES), group_size=np.int32(probe._GROUP_SIZE),
    )
    (HERE / "w8a8_host_case_sha256.json").write_text(json.dumps(digests, indent=1, sort_keys=True) + "\n")

    # More cases through the reference's own _host_oracle.  The function reads
    # the module constants _ROWS/_GROUP_SIZE/_PADDED_OUT_FEATURES/_OUT_FEATURES,
    # so they are rebound for each case and restored afterwards.
    saved = {k: getattr(probe, k) for k in ("_ROWS", "_GROUP_SIZE", "_PADDED_OUT_FEATURES", "_OUT_FEATURES")}
    out = {}
    specs = [
        # name, rows, K, group, N, rank, seed
        ("pertoken_k256", 5, 256, 256, 24, 8, 11),
        ("group64_k128", 7, 128, 64, 19, 8, 12),
        ("pertoken_k512_r16", 4, 512, 512, 40, 16, 13),
        ("zero_rows", 4, 128, 128, 16, 8, 14),
    ]
    try:
        for name, rows, k, g, n, r, seed in specs:
            rng = np.random.default_rng(seed)
            xx = rng.standard_normal((rows, k)).astype(np.float32)
            if name == "zero_rows":
                xx[1] = 0.0
                xx[3, : k // 2] = 0.0
            xx = xx.astype(ml_dtypes.bfloat16)
            w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
            grouped = w.reshape((-1, g, n))
            amax = np.max(np.abs(grouped), axis=1)
            sw32 = np.where(amax > 0, amax / 127.0, 1.0).astype(np.float32)
            wq = np.clip(np.rint(grouped / sw32[:, None, :]), -127, 127).astype(np.int8).reshape((k, n))
            sw = sw32.astype(ml_dtypes.bfloat16)
            la = (rng.standard_normal((k, r)) / np.sqrt(k)).astype(ml_dtypes.bfloat16)
            lb = (rng.standard_normal((r, n)) * 0.02).astype(ml_dtypes.bfloat16)
            sc = np.asarray(2.0, dtype=np.float32)
            probe._ROWS, probe._GROUP_SIZE = rows, g
            probe._PADDED_OUT_FEATURES, probe._OUT_FEATURES = n, n
            exp = probe._host_oracle((xx, wq, sw, la, lb, sc))
            out[f"{name}.x_bf16"] = _u16(xx)
            out[f"{name}.weight_codes"] = wq
            out[f"{name}.weight_scales_bf16"] = _u16(sw)
            out[f"{name}.lora_a_bf16"] = _u16(la)
            out[f"{name}.lora_b_bf16"] = _u16(lb)
            out[f"{name}.lora_scaling"] = sc
            out[f"{name}.group_size"] = np.int32(g)
            out[f"{name}.expected_bf16"] = _u16(exp)
    finally:
        for key, value in saved.items():
            setattr(probe, key, value)
    np.savez(HERE / "w8a8_ref_oracle_cases.npz", **out)
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path to the reference project>")
    main(sys.argv[1])
