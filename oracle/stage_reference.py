"""Stages the reference's own hot-path Python under oracle/_ref/ (git-ignored) so that the
benchmark's reference arm can import the UNMODIFIED reference modules on a machine that has no
reference checkout.  TEST / BENCHMARK INFRASTRUCTURE, NOT PRODUCT CODE: nothing in dualquant_b200/
imports oracle/_ref.

    python oracle/stage_reference.py <path of the reference checkout>

Copied verbatim (files stay byte-identical; oracle/_ref/MANIFEST.txt lists them with sizes):
  activations/        PermLinear, install_perm_linear                (the runtime wrapper)
  formats/            FormatSpec, make_format, rtn_int / mx / nvfp4
  blockfmt/           the indirection module that resolves the external block-format backend
  quarot/             online_had_install, the pure-torch Hadamard transform, vendored QuaRot utils
  legacy_vendor/torch_quant.py, scale_formats.py, _legacy_path.py
  layer_wrapper_dualquant.py                                         (the offline scale search, CPU)
  vendor/dualscale_kernel_benchmark/fused_dual_scale_kernel.py      (Triton A16W4 kernel)
  ablation/real_int4_kernel/fused_w4a4_kernel.py                     (Triton W4A4 kernel)
`import_reference()` installs the same three import shims tests/golden/make_golden.py uses
(a stub for the external `blockfmt` package, stub `accelerate` modules) and returns the modules.
"""
from __future__ import annotations

import os
import shutil
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")

_TREES = ("activations", "formats", "quarot", "blockfmt")
_FILES = (
    "_legacy_path.py",
    "scale_formats.py",
    "layer_wrapper_dualquant.py",
    os.path.join("legacy_vendor", "torch_quant.py"),
    os.path.join("vendor", "dualscale_kernel_benchmark", "fused_dual_scale_kernel.py"),
    os.path.join("ablation", "real_int4_kernel", "fused_w4a4_kernel.py"),
)


def stage(ref_root: str) -> str:
    """Copies the files listed above from `ref_root` into oracle/_ref/; returns that directory."""
    if os.path.isdir(REF_DIR):
        shutil.rmtree(REF_DIR)
    os.makedirs(REF_DIR)
    manifest = []
    for tree in _TREES:
        src = os.path.join(ref_root, tree)
        for dirpath, _dirs, files in os.walk(src):
            for name in files:
                if not name.endswith(".py"):
                    continue
                rel = os.path.relpath(os.path.join(dirpath, name), ref_root)
                manifest.append(rel)
    manifest.extend(_FILES)
    for rel in manifest:
        dst = os.path.join(REF_DIR, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(ref_root, rel), dst)
    with open(os.path.join(REF_DIR, "MANIFEST.txt"), "w") as f:
        for rel in sorted(manifest):
            f.write(f"{os.path.getsize(os.path.join(REF_DIR, rel)):8d}  {rel}\n")
    return REF_DIR


def available() -> bool:
    return os.path.exists(os.path.join(REF_DIR, "activations", "perm_linear.py"))


def import_reference():
    """Imports the staged reference; returns a namespace with PermLinear, make_format,
    hadamard_utils and the paths of the two Triton kernel files."""
    if not available():
        raise RuntimeError("oracle/_ref is not staged: run python oracle/stage_reference.py <reference checkout>")
    stub = types.ModuleType("_dq_blockfmt_stub")

    class Format:  # the external block-format package is absent; its casts are never called here
        @classmethod
        def from_shorthand(cls, s):
            return cls()

        def cast(self, t, axis=-1):
            raise RuntimeError("blockfmt stub: block casts are not available")

    stub.Format = Format
    sys.modules["_dq_blockfmt_stub"] = stub
    os.environ["BLOCKFMT_BACKEND"] = "_dq_blockfmt_stub"
    import transformers  # noqa: F401  (must precede the accelerate stubs)

    if "accelerate" not in sys.modules:
        acc = types.ModuleType("accelerate")
        acc_utils = types.ModuleType("accelerate.utils")
        for name in ("dispatch_model", "infer_auto_device_map"):
            setattr(acc, name, lambda *a, **k: None)
        acc_utils.get_balanced_memory = lambda *a, **k: None
        acc.utils = acc_utils
        sys.modules["accelerate"] = acc
        sys.modules["accelerate.utils"] = acc_utils
    for p in (REF_DIR, os.path.join(REF_DIR, "vendor", "dualscale_kernel_benchmark"),
              os.path.join(REF_DIR, "ablation", "real_int4_kernel")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from activations.perm_linear import PermLinear
    from formats import make_format
    import hadamard_utils

    ns = types.SimpleNamespace()
    ns.PermLinear, ns.make_format, ns.hadamard_utils = PermLinear, make_format, hadamard_utils
    return ns


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python oracle/stage_reference.py <path of the reference checkout>")
    print(stage(sys.argv[1]))
