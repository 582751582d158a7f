"""Generate `reference_scale_encoders.npz` from the reference project's own fp4 / fp8 scale encoders.

    REFERENCE_ROOT=/path/to/reference python tests/golden/make_golden_scale_encoders.py

The encoders live in modules that import the reference's compiled extension at import time
(vllm/model_executor/layers/quantization/utils/marlin_utils_fp4.py, marlin_utils_fp8.py), which a
machine without a GPU driver cannot load.  The functions themselves are plain torch code, so this
script reads the two files, compiles only the named function definitions (unchanged) and runs them on
seeded inputs for fp16 and bf16 activations.  The oracle is pinned against the stored outputs by
tests/test_oracle_golden.py; nothing at test time needs the reference."""
from __future__ import annotations

import ast
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
UTILS = "vllm/model_executor/layers/quantization/utils"


class _Logger:
    def warning_once(self, *a, **k):
        pass


def load_functions(path: str, names: tuple[str, ...]) -> dict:
    tree = ast.parse(open(path).read(), filename=path)
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    missing = set(names) - {n.name for n in body}
    if missing:
        raise SystemExit(f"{path}: functions not found: {sorted(missing)}")
    ns = {"torch": torch, "logger": _Logger()}
    exec(compile(ast.Module(body=body, type_ignores=[]), path, "exec"), ns)
    return ns


def _np(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e8m0fnu):
        return t.contiguous().view(torch.uint8).numpy()
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy()
    return t.contiguous().numpy()


def main() -> None:
    root = os.environ.get("REFERENCE_ROOT")
    if not root or not os.path.isdir(root):
        raise SystemExit("set REFERENCE_ROOT to a checkout of the reference project")
    f4 = load_functions(os.path.join(root, UTILS, "marlin_utils_fp4.py"),
                        ("_nvfp4_compute_scale_factor", "nvfp4_marlin_process_scales",
                         "mxfp4_marlin_process_scales", "nvfp4_marlin_process_global_scale"))
    f8 = load_functions(os.path.join(root, UTILS, "marlin_utils_fp8.py"), ("fp8_fused_exponent_bias_into_scales",))
    out: dict[str, np.ndarray] = {}
    g = torch.Generator().manual_seed(11)
    # e4m3 block scales the way an nvfp4 checkpoint holds them: a wide range (small ones force the
    # power-of-two rescale of the bf16 path) and a narrow one (no rescale), plus exact zeros
    wide = (torch.rand(6, 64, generator=g) * 0.5 + 2.0 ** -8).to(torch.float8_e4m3fn)
    wide[0, 3] = 0
    wide[5, 60] = 0
    narrow = (torch.rand(6, 64, generator=g) * 200.0 + 4.0).to(torch.float8_e4m3fn)
    for tag, s in (("wide", wide), ("narrow", narrow)):
        out[f"nvfp4_{tag}_in"] = _np(s)
        for dt, dn in ((torch.float16, "f16"), (torch.bfloat16, "bf16")):
            enc, sf = f4["nvfp4_marlin_process_scales"](s.to(dt), None, dt)
            out[f"nvfp4_{tag}_{dn}_enc"] = _np(enc)
            out[f"nvfp4_{tag}_{dn}_sf"] = np.array([sf], dtype=np.float64)
    gs = torch.tensor([0.0123, 1.0, 3.5e-4], dtype=torch.float32)
    out["nvfp4_global_in"] = _np(gs)
    for dt, dn in ((torch.float16, "f16"), (torch.bfloat16, "bf16")):
        out[f"nvfp4_global_{dn}"] = _np(f4["nvfp4_marlin_process_global_scale"](gs, dt))
    e8 = torch.pow(2.0, torch.randint(-12, 3, (4, 64), generator=g).float())
    out["mxfp4_in"] = _np(e8)
    out["mxfp4_enc"] = _np(f4["mxfp4_marlin_process_scales"](e8.to(torch.bfloat16), torch.bfloat16))
    sc = torch.rand(3, 32, generator=g) * 1e-3 + 1e-5
    for dt, dn in ((torch.float16, "f16"), (torch.bfloat16, "bf16")):
        out[f"fp8_scale_{dn}_in"] = _np(sc.to(dt))
        out[f"fp8_scale_{dn}_out"] = _np(f8["fp8_fused_exponent_bias_into_scales"](sc.to(dt)))
    np.savez_compressed(os.path.join(HERE, "reference_scale_encoders.npz"), **out)
    print(f"wrote {len(out)} arrays")


if __name__ == "__main__":
    main()
