"""Writes tests/golden/reference_cuda_signatures.json: the argument list of every `keydnn_*` function the reference's
CUDA library declares or defines, reduced to ABI classes (what a caller's registers hold):

    ptr  any pointer          u64  uintptr_t / uint64_t / size_t      i64  int64_t / long long
    i32  int                  f32  float                               f64  double

Read from the `.hpp` and `.cu` files of a checkout of the reference
(src/keydnn/infrastructure/native_cuda/keydnn_v2_cuda_native/KeyDNNV2CudaNative); run where one exists:

    KEYDNN_REFERENCE_ROOT=/path/to/keydnn_v2 python tests/golden/make_signatures.py

tests/test_abi_cpu.py compares include/keydnn_b200.h and include/keydnn_b200_dnn.h against the result."""
from __future__ import annotations

import json
import os
import re
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REF = Path(os.environ.get("KEYDNN_REFERENCE_ROOT") or HERE.parents[2] / "reference")
NC = REF / "src/keydnn/infrastructure/native_cuda/keydnn_v2_cuda_native/KeyDNNV2CudaNative"

DECL = re.compile(r"\b(?:int|void)\s+(keydnn_\w+)\s*\(([^()]*)\)\s*[;{]", re.S)


def abi_class(arg: str) -> str:
    a = " ".join(arg.replace("std::", "").split())
    if "*" in a:
        return "ptr"
    toks = [t for t in a.split(" ") if t not in ("const", "unsigned", "signed")]
    base = " ".join(toks[:-1]) if len(toks) > 1 else toks[0]
    table = {"uintptr_t": "u64", "uint64_t": "u64", "size_t": "u64", "int64_t": "i64", "long long": "i64", "int": "i32",
             "float": "f32", "double": "f64", "T": "T"}
    if base not in table:
        raise ValueError(f"unknown type in {arg!r}")
    return table[base]


def scan(text: str) -> dict[str, list[str]]:
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)
    text = re.sub(r"//[^\n]*", " ", text)
    out = {}
    for m in DECL.finditer(text):
        name, args = m.group(1), m.group(2).strip()
        if "##" in name:
            continue
        try:
            sig = [] if args in ("", "void") else [abi_class(a) for a in args.split(",")]
        except ValueError:
            continue
        if "T" in sig:
            continue
        out[name] = sig
    return out


def main() -> None:
    if not NC.exists():
        sys.exit(f"no checkout of the reference at {REF}")
    sigs: dict[str, list[str]] = {}
    for path in sorted(NC.glob("*.hpp")) + sorted(NC.glob("*.cu")):
        for name, sig in scan(path.read_text(errors="replace")).items():
            if name in sigs and sigs[name] != sig:
                raise SystemExit(f"{name}: {sigs[name]} in an earlier file, {sig} in {path.name}")
            sigs.setdefault(name, sig)
    out = HERE / "reference_cuda_signatures.json"
    out.write_text(json.dumps(dict(sorted(sigs.items())), indent=0) + "\n")
    print(f"{len(sigs)} signatures -> {out}")


if __name__ == "__main__":
    main()
