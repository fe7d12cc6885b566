"""The ctypes signatures in zinfer_b200/kernels.py must match the C prototypes in csrc/*.cu:
a mismatch would pass garbage to a kernel launcher."""
import re
from pathlib import Path

from zinfer_b200 import kernels

CSRC = Path(kernels.__file__).parent / "csrc"


def c_kinds(params: str) -> str:
    out = ""
    for p in [x.strip() for x in params.split(",") if x.strip()]:
        if "*" in p or p.startswith("cudaStream_t"):
            out += "p"
        elif p.startswith("long long"):
            out += "l"
        elif p.startswith("float"):
            out += "f"
        elif p.startswith("int"):
            out += "i"
        else:
            raise AssertionError(f"unknown parameter type: {p}")
    return out


def test_every_signature_matches_its_prototype():
    checked = 0
    for lib, funcs in kernels._SIGNATURES.items():
        text = (CSRC / f"{lib}.cu").read_text()
        for name, sig in funcs.items():
            m = re.search(r"\b(?:int|long long)\s+" + name + r"\s*\(([^)]*)\)\s*\{", text)
            assert m, f"{name} not found in {lib}.cu"
            assert c_kinds(m.group(1)) == sig, f"{name}: C has {c_kinds(m.group(1))}, Python has {sig}"
            checked += 1
    assert checked >= 10


def test_every_exported_launcher_has_a_signature():
    for cu in CSRC.glob("*.cu"):
        exported = set(re.findall(r"\b(?:int|long long)\s+(zk_\w+)\s*\(", cu.read_text()))
        known = set(kernels._SIGNATURES.get(cu.stem, {}))
        assert exported <= known, f"{cu.name}: {sorted(exported - known)} have no ctypes signature"
