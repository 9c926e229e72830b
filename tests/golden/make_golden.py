"""Generate tests/golden/ref_func_cases.npz from the reference's own test oracle.

Run where a checkout of xytpai/flydsl-examples is at hand (it does not travel to the GPU box), passing its path:

    python tests/golden/make_golden.py <path to the flydsl-examples checkout>

The reference's test module (test_gemm_a16w16_gfx950.py) is loaded by file path; its `from kernels... import`
lines resolve to this repository's drop-in `kernels` package, so the module imports without FlyDSL. Its
`ref_func` (test_gemm_a16w16_gfx950.py:82-94, plain torch.mm / torch.addmm) is then called on seeded CPU inputs
and the inputs (raw 16-bit patterns) and outputs are stored. Shapes follow the reference's small cases:
64x64x768 (fp32-output test :530-533), M=3 N=32 (small-M test :573-579), ragged 65x96 / 129x136 (split-K test
:327-385), padded strides (:696-713).
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

REPO = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(REPO))

CASES = [
    # name, dtype, layout, m, n, k, bias, fp32_out
    ("fp32out_64x64x768", "bf16", "nt", 64, 64, 768, True, True),
    ("fp32out_64x64x768_fp16_nn", "fp16", "nn", 64, 64, 768, False, True),
    ("small_m3", "bf16", "nt", 3, 32, 256, True, False),
    ("small_m3_fp16_nn", "fp16", "nn", 3, 32, 256, False, False),
    ("ragged_65x96", "bf16", "tn", 65, 96, 192, True, False),
    ("ragged_129x136_fp16", "fp16", "tt", 129, 136, 128, True, True),
    ("ktail_40x48x100", "fp16", "nt", 40, 48, 100, False, True),
    ("ktail_40x48x100_bf16_tn", "bf16", "tn", 40, 48, 100, True, False),
]


def load_reference_test_module(ref_root: Path):
    spec = importlib.util.spec_from_file_location("reference_test_module", ref_root / "test_gemm_a16w16_gfx950.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main() -> None:
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path to the flydsl-examples checkout>")
    ref_root = Path(sys.argv[1])
    mod = load_reference_test_module(ref_root)
    dts = {"bf16": torch.bfloat16, "fp16": torch.float16}
    blob = {}
    names = []
    for i, (name, dt, layout, m, n, k, has_bias, fp32_out) in enumerate(CASES):
        g = torch.Generator("cpu").manual_seed(1000 + i)
        dtype = dts[dt]
        # The reference draws U(-1,1) operands and U(10,20) bias (test_gemm_a16w16_gfx950.py:53-73).
        a = (torch.rand(m, k, generator=g) * 2 - 1).to(dtype)
        b = (torch.rand(k, n, generator=g) * 2 - 1).to(dtype)
        bias = (torch.rand(n, generator=g) * 10 + 10).to(dtype) if has_bias else None
        a_l = a.t().contiguous().t() if layout[0] == "t" else a
        b_l = b.t().contiguous().t() if layout[1] == "t" else b
        c = torch.empty(m, n, dtype=torch.float32 if fp32_out else dtype)
        mod.ref_func(a_l, b_l, bias, c, layout)
        names.append(name)
        blob[f"{name}.a"] = a.view(torch.int16).numpy()
        blob[f"{name}.b"] = b.view(torch.int16).numpy()
        if bias is not None:
            blob[f"{name}.bias"] = bias.view(torch.int16).numpy()
        blob[f"{name}.c"] = c.numpy() if fp32_out else c.view(torch.int16).numpy()
        blob[f"{name}.meta"] = np.array([dt, layout, str(int(fp32_out))])
    blob["names"] = np.array(names)
    out = Path(__file__).resolve().parent / "ref_func_cases.npz"
    np.savez_compressed(out, **blob)
    print(f"wrote {out} ({out.stat().st_size} bytes, {len(names)} cases, torch {torch.__version__})")


if __name__ == "__main__":
    main()
