"""Generate the golden fixtures in this folder.

    python tests/golden/make_golden.py --reference <checkout of the reference project>

Two kinds of vectors are written to `quant_golden.npz`:

* `ref_*`  -- produced by the REFERENCE's own PyTorch code, taken from the checkout given on the
  command line: the checkers `ref_quant_row_i8` and `ref_quant_row_fp8`
  (sageattention/sk1_backend/quant_triton.py:1128-1156, imported as a module) pin the row
  quantisers of the oracle; `fold_v_scale` (sageattention/sk1_backend/__init__.py:561-579) and
  `n_pad_for` (sageattention/sk1_backend/hip_prologue.py:93-95) are plain PyTorch / Python
  functions inside modules that cannot be imported here (they load GPU objects at import), so
  their source is cut out of the file and executed on its own; they pin the fold S, the folded
  V scales and the reference's padded length.
* `ora_*`  -- produced by the oracle (oracle/ref_numerics.py) on the same stored inputs: the whole
  prologue and the attention output.  They pin the CUDA path against a committed answer, so a GPU
  test needs neither the reference checkout nor a re-run of the oracle.

Inputs are stored in the file (not re-drawn from a seed) so the fixtures do not depend on a
random-number generator's version.
"""
import argparse
import ast
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import ref_numerics as R  # noqa: E402

CASES = [
    # name, B, H, N, dtype, causal, smooth_k
    ("f16_n1", 1, 2, 1, torch.float16, False, True),
    ("f16_n65", 1, 2, 65, torch.float16, True, True),
    ("f16_n136", 1, 2, 136, torch.float16, False, True),
    ("f16_n70_nosmooth", 1, 1, 70, torch.float16, True, False),
    ("bf16_n40", 1, 1, 40, torch.bfloat16, False, True),
    ("bf16_n136", 1, 2, 136, torch.bfloat16, True, True),
]


def bits(t: torch.Tensor) -> np.ndarray:
    """Byte-exact numpy view of a tensor (fp8/bf16 have no numpy dtype)."""
    t = t.contiguous()
    if t.dtype in (torch.float8_e4m3fn,):
        return t.view(torch.uint8).numpy()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy()
    return t.numpy()


def function_from_source(path: str, name: str):
    """Compile one top-level function of a Python file without importing the file."""
    src = open(path).read()
    body = ast.parse(src).body
    ns = {}
    for node in body:                  # module-level literal constants the function may read (e.g. BN = 64)
        if isinstance(node, ast.Assign) and isinstance(node.value, ast.Constant):
            exec(compile(ast.get_source_segment(src, node), path, "exec"), ns)
    for node in body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            exec(compile(ast.get_source_segment(src, node), path, "exec"), ns)
            return ns[name]
    raise KeyError(name)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    args = ap.parse_args()
    path = os.path.join(args.reference, "sageattention", "sk1_backend", "quant_triton.py")
    spec = importlib.util.spec_from_file_location("reference_quant_triton", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)

    backend = os.path.join(args.reference, "sageattention", "sk1_backend")
    ref_fold = function_from_source(os.path.join(backend, "__init__.py"), "fold_v_scale")
    ref_n_pad = function_from_source(os.path.join(backend, "hip_prologue.py"), "n_pad_for")

    out = {}
    lengths = [1, 15, 63, 64, 65, 127, 128, 129, 300, 1000, 8771, 47520]
    out["n_pad/N"] = np.array(lengths)
    out["n_pad/ref"] = np.array([ref_n_pad(n) for n in lengths])
    for name, b, h, n, dtype, causal, smooth in CASES:
        q, k, v = R.make_inputs(b, h, n, 128, dtype, seed=1234 + n, k_bias_std=0.75)
        if n >= 65 and h >= 2:   # one |V| > 448 token so that S > 1, one all-zero K row, one large Q row
            v[:, 0, 3] = v[:, 0, 3] * 700.0
            k[:, 1, 5] = 0
            q[:, 0, 7] = q[:, 0, 7] * 100.0
        int8 = dtype == torch.float16
        pq = R.prologue(q, k, v, smooth_k=smooth, int8=int8, pad_multiple=128)
        o = R.sageattn_oracle(q, k, v, is_causal=causal, smooth_k=smooth, tile=128)
        o64 = R.sageattn_oracle(q, k, v, is_causal=causal, smooth_k=smooth, tile=64)
        # the reference's own checkers, on the mean-subtracted K and on V
        kc = k.float() - pq["mean"][:, :, None, :] if smooth else k.float()
        if int8:
            rk8, rsk = ref.ref_quant_row_i8(kc)
        else:
            rk8, rsk = ref.ref_quant_row_fp8(kc)
        rv8, rsv = ref.ref_quant_row_fp8(v)
        p = name + "/"
        out[p + "q"], out[p + "k"], out[p + "v"] = bits(q), bits(k), bits(v)
        out[p + "meta"] = np.array([b, h, n, int(dtype == torch.bfloat16), int(causal), int(smooth)])
        out[p + "ref_k8"], out[p + "ref_sk"] = bits(rk8), bits(rsk.float())
        out[p + "ref_v8"], out[p + "ref_sv"] = bits(rv8), bits(rsv.float())
        folded = pq["sv"].reshape(b * h, -1).clone()          # the reference folds in place, (B*H, N_pad)
        out[p + "ref_S"] = bits(ref_fold(folded).float())
        out[p + "ref_svfold"] = bits(folded)
        for key in ("q8", "sq", "k8", "sk", "v8", "sv", "svp", "S"):
            out[p + "ora_" + key] = bits(pq[key])
        if smooth:
            out[p + "ora_mean"] = bits(pq["mean"])
        out[p + "ora_out128"], out[p + "ora_out64"] = bits(o), bits(o64)
    dst = os.path.join(HERE, "quant_golden.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes,", len(out), "arrays")
    return 0


if __name__ == "__main__":
    sys.exit(main())
