"""Stage the reference's own CPU implementation of the path as compiled modules under oracle/_ref/. TEST INFRASTRUCTURE.

    python oracle/build_ref.py [--ref <reference checkout>]

The reference is pure Python / PyTorch: its implementation B (kvq/int8_ref.py), the quantization primitives
(kvq/quant.py) and the paging / bf16 golden code (kvq/ref_attn.py) run on CPU unchanged. This recipe byte-compiles
those modules from the checkout where it lies into oracle/_ref/kvq/*.pyc (sourceless modules; nothing of the
reference's source text is copied, and oracle/_ref/ is kept out of version control). The result is used only as a
checker and as the timed CPU baseline:
  * tests/test_oracle_golden.py compares the numpy restatement (oracle/kvq_oracle.py) with it on seeded cases;
  * bench.py --impl reference and the cpu_baseline leg time it on the host cores (kind "reference").
Where oracle/_ref/ is absent (no checkout was available at build time) both fall back to the numpy restatement.
"""
import argparse
import os
import py_compile
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
MODULES = ("__init__", "quant", "ref_attn", "int8_ref")
DEFAULT_REF = os.environ.get("KVQ_REF", "/root/reference")


def build(ref=DEFAULT_REF, quiet=True):
    """Returns the output directory, or None when the checkout is not there."""
    src_dir = os.path.join(ref, "kvq")
    if not all(os.path.exists(os.path.join(src_dir, m + ".py")) for m in MODULES):
        return None
    dst_dir = os.path.join(OUT, "kvq")
    os.makedirs(dst_dir, exist_ok=True)
    for m in MODULES:
        # dfile: the file name recorded in tracebacks; it names the module, not a path of the build machine
        py_compile.compile(os.path.join(src_dir, m + ".py"), cfile=os.path.join(dst_dir, m + ".pyc"),
                           dfile=f"kvq/{m}.py", doraise=True)
    with open(os.path.join(OUT, "BUILT_FROM"), "w") as f:
        f.write(f"byte-compiled by oracle/build_ref.py with python {sys.version.split()[0]}; modules: {', '.join(MODULES)}\n")
    if not quiet:
        print(dst_dir)
    return OUT


def load():
    """Import the staged modules: returns (quant, ref_attn, int8_ref) or None when oracle/_ref/ is absent or was
    compiled by another Python version."""
    if not os.path.exists(os.path.join(OUT, "kvq", "int8_ref.pyc")):
        return None
    if "kvq" in sys.modules and not getattr(sys.modules["kvq"], "__file__", "").startswith(OUT):
        return None   # another package of that name is already imported in this process
    sys.path.insert(0, OUT)
    try:
        from kvq import int8_ref, quant, ref_attn
    except ImportError:
        return None
    finally:
        sys.path.remove(OUT)
    return quant, ref_attn, int8_ref


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=DEFAULT_REF)
    args = ap.parse_args()
    if build(args.ref, quiet=False) is None:
        raise SystemExit(f"no reference checkout at {args.ref}")
