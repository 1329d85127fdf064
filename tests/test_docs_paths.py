"""The documentation names many files; every such name must exist. Names are the back-quoted tokens of the
Markdown files that look like paths into this repository (the reference's own paths, ``picotron/...``, and
wildcards are left alone). A short name such as ``ops/fused_tp.py`` may be given relative to the package, the
kernel tree, the profiles or the file's own folder."""
import glob
import os
import re

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DOCS = ["README.md", "DESIGN.md", "picotron_b200/parallel/README.md", "profiles/README.md"] + \
    sorted(os.path.relpath(p, REPO) for p in glob.glob(os.path.join(REPO, "docs", "*.md")))
EXTS = (".py", ".cu", ".cuh", ".h", ".cpp", ".md", ".txt", ".json", ".toml", ".slurm")
ROOTS = ["", "picotron_b200", "picotron_b200/parallel", "picotron_b200/ops", "picotron_b200/runtime", "picotron_b200/models",
         "csrc", "csrc/fused", "csrc/elementwise", "csrc/runtime", "csrc/common", "csrc/gemm", "csrc/attention", "profiles",
         "benchmarks", "tests", "docs", "template", "baseline"]
IGNORED = ("picotron/", "/root/", "runs/", "hf_model", "baseline/_ref")
NOT_IN_TREE = {"MEASURED_PEAKS.json", "BASELINE.json", "SURVEY.md", "VERDICT.md", "ADVICE.md", "BASELINE.md", "config.json",
               "manifest.json", "metrics.csv", "global_metrics.csv", "status.txt"}


def _candidates(text):
    """(path, symbol or None) for every back-quoted ``path`` or ``path::symbol``."""
    for token in re.findall(r"`([^`\n]+)`", text):
        path, _, symbol = token.partition("::")
        path = path.split(" ")[0].strip("(),.;:")
        if not path.endswith(EXTS) or any(c in path for c in "*{}<>|$=") or path.startswith(IGNORED):
            continue
        if os.path.basename(path) in NOT_IN_TREE:
            continue
        name = re.match(r"[A-Za-z_][A-Za-z0-9_]*", symbol)
        yield path, (name.group(0) if name else None)


def _resolve(path, here):
    for root in ROOTS + [here]:
        full = os.path.join(REPO, root, path)
        if os.path.exists(full):
            return full
    return None


def test_every_file_and_symbol_named_in_the_documentation_exists():
    missing = []
    for doc in DOCS:
        text = open(os.path.join(REPO, doc)).read()
        here = os.path.dirname(doc)
        for path, symbol in set(_candidates(text)):
            if doc == "docs/reference_tests.md" and "/" not in path and path.endswith(".py") and path != "train.py":
                continue                                  # that file lists the reference's own scripts by bare name
            full = _resolve(path, here)
            if full is None:
                missing.append(f"{doc}: {path}")
            elif symbol and not re.search(r"\b" + re.escape(symbol) + r"\b", open(full, errors="replace").read()):
                missing.append(f"{doc}: {path}::{symbol}")
    assert not missing, "\n".join(sorted(missing))
