"""Generates tests/golden/lang/*.golden from the reference's OWN front-end.

Run in a container that has the reference checkout:
    python oracle/build.py --ref && python tests/golden/make_lang_golden.py

For every *.tc file: the reference's printed tree after parsing, after semantic analysis (with the
environment dump) and after canonicalisation.  For errors.txt: whether the reference rejects each
block and the first line of its message.  The outputs are small text fixtures that travel with
the repository; the reference binary does not.
"""
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.path.join(ROOT, "oracle", "_ref", "tc_lang_ref")
LANG = os.path.join(HERE, "lang")


def split_blocks(text):
    blocks, cur = [], []
    for line in text.splitlines():
        if line.startswith("#"):
            continue
        if line.strip() == "----":
            blocks.append("\n".join(cur).strip() + "\n")
            cur = []
        else:
            cur.append(line)
    if "".join(cur).strip():
        blocks.append("\n".join(cur).strip() + "\n")
    return blocks


def run(mode, path):
    r = subprocess.run([REF, mode, path], capture_output=True, text=True)
    return r.returncode, r.stdout


def main():
    if not os.path.exists(REF):
        sys.exit("build the reference front-end first: python oracle/build.py --ref")
    for name in sorted(os.listdir(LANG)):
        path = os.path.join(LANG, name)
        if name.endswith(".tc"):
            for mode in ("parse", "sema", "canon"):
                rc, out = run(mode, path)
                assert rc == 0, (name, mode, out)
                with open(path[:-3] + "." + mode + ".golden", "w") as f:
                    f.write(out)
    lines = []
    for i, block in enumerate(split_blocks(open(os.path.join(LANG, "errors.txt")).read())):
        with tempfile.NamedTemporaryFile("w", suffix=".tc", delete=False) as t:
            t.write(block)
        rc, out = run("sema", t.name)
        os.unlink(t.name)
        assert rc == 3, "the reference accepts block %d:\n%s" % (i, block)
        msg = [l for l in out.splitlines() if l.strip() and not l.startswith("ERROR:")][0]
        lines.append("%d\t%s" % (i, msg.rstrip(":")))
    with open(os.path.join(LANG, "errors.golden"), "w") as f:
        f.write("\n".join(lines) + "\n")
    print("wrote goldens for", sorted(n for n in os.listdir(LANG) if n.endswith(".golden")))


if __name__ == "__main__":
    main()
