"""Build recipe for the CPU checker (TEST INFRASTRUCTURE ONLY; see tc_oracle.c).

    python oracle/build.py            -> oracle/libtc_oracle.so  (loop-nest restatement)
    python oracle/build.py --ref      -> also oracle/_ref/tc_lang_ref, the reference's OWN
                                         tc/lang front-end compiled from its sources where
                                         they lie (needs the reference checkout; the binary
                                         is never committed and nothing of it is copied)

The shared object is compiled with -ffp-contract=off so the float flavour does one
rounded multiply and one rounded add per step, like the textual loop nest.
"""
import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def _cc(names):
    for n in names:
        p = n if os.path.isabs(n) else shutil.which(n)
        if p and os.path.exists(p):
            return p
    raise RuntimeError("no C compiler found among %r" % (names,))


def build_oracle(verbose=False):
    src = os.path.join(HERE, "tc_oracle.c")
    out = os.path.join(HERE, "libtc_oracle.so")
    if os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(src):
        return out
    cc = _cc(["/usr/bin/gcc", "gcc", "cc"])
    base = [cc, "-O2", "-fPIC", "-shared", "-ffp-contract=off", "-o", out, src]
    # OpenMP spreads the outer loops over the host cores; fall back to one thread
    # when the compiler has no libgomp.
    for extra in (["-fopenmp"], []):
        r = subprocess.run(base + extra, capture_output=True, text=True)
        if r.returncode == 0:
            if verbose:
                print("built", out, "with", extra or "no OpenMP")
            return out
    raise RuntimeError("oracle build failed:\n" + r.stderr)


def build_reference_lang(reference, verbose=False):
    """Compile the reference's tc/lang (lexer, parser, printer) around ref_lang_driver.cc."""
    lang = os.path.join(reference, "tc", "lang")
    if not os.path.isdir(lang):
        return None
    outdir = os.path.join(HERE, "_ref")
    os.makedirs(outdir, exist_ok=True)
    out = os.path.join(outdir, "tc_lang_ref")
    drv = os.path.join(HERE, "ref_lang_driver.cc")
    if os.path.exists(out) and os.path.getmtime(out) >= os.path.getmtime(drv):
        return out
    cxx = _cc(["/usr/bin/g++", "g++", "c++"])
    cmd = [cxx, "-std=c++14", "-O1", "-w", "-I" + reference, "-o", out, drv] + [
        os.path.join(lang, f) for f in ("lexer.cc", "parser.cc", "tc_format.cc")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("reference tc/lang build failed:\n" + r.stderr)
    if verbose:
        print("built", out)
    return out


def reference_checkout():
    """Where the reference's sources lie: $TC_REFERENCE, else a directory `reference` next to this repository.
    None when neither exists (then only the golden files pin the front-end)."""
    for cand in (os.environ.get("TC_REFERENCE"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "tc", "lang")):
            return cand
    return None


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", action="store_true")
    ap.add_argument("--reference", default=reference_checkout() or "")
    a = ap.parse_args()
    build_oracle(verbose=True)
    if a.ref:
        if build_reference_lang(a.reference, verbose=True) is None:
            print("reference checkout not found at", a.reference, file=sys.stderr)
            sys.exit(1)
