"""Stage the reference's own CPU implementation of the path as compiled modules under oracle/_ref/. TEST INFRASTRUCTURE.

    python oracle/build_ref.py [--ref <reference checkout>]

The reference is pure Python / PyTorch: its implementation B (kvq/int8_ref.py), the quantization primitives
(kvq/quant.py) and the paging / bf16 golden code (kvq/ref_attn.py) run on CPU unchanged. This recipe byte-compiles
those modules from the checkout where it lies into one file of marshalled code objects, oracle/_ref/kvq_ref.bin
(nothing of the reference's source text is copied, and oracle/_ref/ is kept out of version control). The result is used only as a
checker and as the timed CPU baseline:
  * tests/test_oracle_golden.py compares the numpy restatement (oracle/kvq_oracle.py) with it on seeded cases;
  * bench.py --impl reference and the cpu_baseline leg time it on the host cores (kind "reference").
Where oracle/_ref/ is absent (no checkout was available at build time) both fall back to the numpy restatement.
"""
import argparse
import marshal
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
MODULES = ("__init__", "quant", "ref_attn", "int8_ref")
DEFAULT_REF = os.environ.get("KVQ_REF", "/root/reference")


BLOB = os.path.join(OUT, "kvq_ref.bin")


def build(ref=DEFAULT_REF, quiet=True):
    """Returns the output directory, or None when the checkout is not there."""
    src_dir = os.path.join(ref, "kvq")
    if not all(os.path.exists(os.path.join(src_dir, m + ".py")) for m in MODULES):
        return None
    os.makedirs(OUT, exist_ok=True)
    code = {}
    for m in MODULES:
        with open(os.path.join(src_dir, m + ".py")) as f:
            # the file name recorded in tracebacks names the module, not a path of the build machine
            code[m] = marshal.dumps(compile(f.read(), f"kvq/{m}.py", "exec"))
    with open(BLOB, "wb") as f:
        marshal.dump({"python": list(sys.version_info[:2]), "modules": code}, f)
    with open(os.path.join(OUT, "BUILT_FROM"), "w") as f:
        f.write(f"compiled by oracle/build_ref.py with python {sys.version.split()[0]}; modules: {', '.join(MODULES)}\n")
    if not quiet:
        print(BLOB)
    return OUT


_LOADED = None


def load():
    """Import the staged modules as the package `kvq`: returns (quant, ref_attn, int8_ref), or None when
    oracle/_ref/ is absent, was compiled by another Python version, or another package named kvq is already
    imported in this process."""
    global _LOADED
    if _LOADED is not None:
        return _LOADED
    if not os.path.exists(BLOB) or "kvq" in sys.modules:
        return None
    with open(BLOB, "rb") as f:
        blob = marshal.load(f)
    if blob["python"] != list(sys.version_info[:2]):
        return None
    pkg = types.ModuleType("kvq")
    pkg.__path__ = []          # a package, so that "from kvq import quant" resolves through sys.modules
    pkg.__file__ = BLOB
    sys.modules["kvq"] = pkg
    mods = {}
    for m in MODULES:
        if m == "__init__":
            exec(marshal.loads(blob["modules"][m]), pkg.__dict__)
            continue
        mod = types.ModuleType(f"kvq.{m}")
        mod.__file__ = BLOB
        sys.modules[f"kvq.{m}"] = mod
        setattr(pkg, m, mod)
        exec(marshal.loads(blob["modules"][m]), mod.__dict__)
        mods[m] = mod
    _LOADED = (mods["quant"], mods["ref_attn"], mods["int8_ref"])
    return _LOADED


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=DEFAULT_REF)
    args = ap.parse_args()
    if build(args.ref, quiet=False) is None:
        raise SystemExit(f"no reference checkout at {args.ref}")
