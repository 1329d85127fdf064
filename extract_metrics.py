"""Collect throughput numbers from training logs.

``python extract_metrics.py <folder>`` walks ``<folder>`` for run directories that contain a
``*.out`` / ``*.log`` file with the trainer's step lines, averages ``Tokens/s/GPU`` and ``MFU``
over the steps after the first three (warm-up), writes ``metrics.csv`` into each run directory and
``global_metrics.csv`` (columns ``run_name,status,dp,tp,pp,micro_batch_size,grad_acc,seq_len,
avg_tokens_s_gpu,avg_mfu``) at the top — the tool of the same name in the reference
(extract_metrics.py:10-234). Run parameters are read from directory names of the form
``dp2_tp4_pp1_mbs4_ga8_sl2048``; ``cp`` and ``ep`` are picked up too when present.
"""
import argparse
import csv
import glob
import os
import re

SUFFIX = {"K": 1e3, "M": 1e6, "B": 1e9, "T": 1e12}
STEP_RE = re.compile(r"Step:\s*(\d+).*?Tokens/s/GPU:\s*([\d.]+)([KMBT]?).*?MFU:\s*([\d.]+)%")
NAME_RE = {k: re.compile(rf"(?:^|_){k}(\d+)") for k in ("dp", "tp", "pp", "cp", "ep", "mbs", "ga", "sl")}
WARMUP_STEPS = 3


def parse_folder_name(name: str) -> dict:
    out = {}
    for k, rx in NAME_RE.items():
        m = rx.search(name)
        out[k] = int(m.group(1)) if m else None
    return out


def parse_log(path: str):
    rows = []
    with open(path, errors="ignore") as fh:
        for line in fh:
            m = STEP_RE.search(line)
            if m:
                rows.append((int(m.group(1)), float(m.group(2)) * SUFFIX.get(m.group(3), 1.0), float(m.group(4))))
    return rows


def summarise(rows):
    rows = [r for r in rows if r[0] > WARMUP_STEPS] or rows
    if not rows:
        return None, None
    return sum(r[1] for r in rows) / len(rows), sum(r[2] for r in rows) / len(rows)


def process_run(run_dir: str):
    logs = sorted(glob.glob(os.path.join(run_dir, "*.out")) + glob.glob(os.path.join(run_dir, "*.log")))
    rows = []
    for lg in logs:
        rows += parse_log(lg)
    tok, mfu = summarise(rows)
    status = "unknown"
    sp = os.path.join(run_dir, "status.txt")
    if os.path.exists(sp):
        status = open(sp).read().strip()
    elif rows:
        status = "completed"
    if tok is not None:
        with open(os.path.join(run_dir, "metrics.csv"), "w", newline="") as fh:
            w = csv.writer(fh)
            w.writerow(["step", "tokens_s_gpu", "mfu"])
            w.writerows(rows)
    return status, tok, mfu


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("folder")
    args = ap.parse_args()
    out_rows = []
    for root, dirs, files in os.walk(args.folder):
        if any(f.endswith((".out", ".log")) for f in files):
            status, tok, mfu = process_run(root)
            p = parse_folder_name(os.path.basename(root))
            out_rows.append([os.path.basename(root), status, p["dp"], p["tp"], p["pp"], p["mbs"], p["ga"], p["sl"],
                             f"{tok:.1f}" if tok is not None else "", f"{mfu:.2f}" if mfu is not None else ""])
    out_rows.sort(key=lambda r: r[0])
    path = os.path.join(args.folder, "global_metrics.csv")
    with open(path, "w", newline="") as fh:
        w = csv.writer(fh)
        w.writerow(["run_name", "status", "dp", "tp", "pp", "micro_batch_size", "grad_acc", "seq_len",
                    "avg_tokens_s_gpu", "avg_mfu"])
        w.writerows(out_rows)
    print(f"wrote {path} ({len(out_rows)} runs)")


if __name__ == "__main__":
    main()
