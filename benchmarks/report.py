#!/usr/bin/env python
"""Turn benchmark JSON lines into Markdown tables.

    OUT=results.jsonl bash benchmarks/sweep.sh
    python benchmarks/report.py results.jsonl            # per-op tables and strong-scaling efficiency
    python benchmarks/report.py a.jsonl b.jsonl --csv    # the same rows as CSV

Reads the lines written by ``bench.py`` (one per run: ``metric``, ``ms_per_step``, ``n_gpus``, ``config``)
and by ``benchmarks/bench_ops.py`` (one per op: ``op``, ``backend``, ``ms``, ``n_gpus``, ``pdims``,
``global_shape``); anything that is not a JSON object is skipped.  The reference plots its CSV output with
an external plotting package (``benchmarks/slurm*.sh`` there, ``README.md`` of its benchmark folder); this
is the text counterpart, with the scaling efficiency computed the way the strong-scaling figure is read:
``t(1 GPU) / (N * t(N GPUs))`` per op, backend, size and dtype, with the fastest process grid at each N.
"""
from __future__ import annotations

import argparse
import json
import sys
from collections import defaultdict
from typing import Dict, Iterable, List, Optional, Tuple


def read_records(paths: Iterable[str]) -> List[dict]:
    """One normalised record per measurement: op, backend, n_gpus, pdims, shape, dtype, ms, extra."""
    out = []
    for path in paths:
        with (sys.stdin if path == "-" else open(path)) as f:
            for line in f:
                line = line.strip()
                if not line.startswith("{"):
                    continue
                try:
                    d = json.loads(line)
                except json.JSONDecodeError:
                    continue
                rec = normalise(d)
                if rec is not None:
                    out.append(rec)
    return out


def normalise(d: dict) -> Optional[dict]:
    if "unavailable" in d:
        return None
    if "op" in d and "ms" in d:  # bench_ops.py
        op = d["op"]
        if "halo" in d:
            op = f"{op} h={d['halo']}"
        extra = {k: d[k] for k in ("gflops", "egress_gbs", "local_gbs", "frac_of_roofline", "frac_of_link") if d.get(k) is not None}
        return {"op": op, "backend": d.get("backend", "?"), "n_gpus": int(d.get("n_gpus", 1)),
                "pdims": tuple(d.get("pdims", (1, 1))), "shape": tuple(d.get("global_shape", ())),
                "dtype": d.get("dtype", "?"), "ms": float(d["ms"]), "extra": extra}
    if "metric" in d and "ms_per_step" in d:  # bench.py
        cfg = d.get("config", {})
        extra = {"value": d.get("value"), "unit": d.get("unit")}
        if isinstance(d.get("e2e"), dict) and d["e2e"].get("ms_per_step") is not None:
            extra["e2e_ms"] = d["e2e"]["ms_per_step"]
        return {"op": "pfft3d+pifft3d", "backend": d.get("impl", cfg.get("backend", "?")), "n_gpus": int(d.get("n_gpus", 1)),
                "pdims": tuple(cfg.get("pdims", (1, 1))), "shape": tuple(cfg.get("global_shape", ())),
                "dtype": str(d.get("dtype", "?")).split()[0], "ms": float(d["ms_per_step"]), "extra": extra}
    return None


def best_per_gpu_count(records: List[dict]) -> Dict[Tuple, Dict[int, dict]]:
    """For every (op, backend, shape, dtype): the fastest record at each GPU count."""
    groups: Dict[Tuple, Dict[int, dict]] = defaultdict(dict)
    for r in records:
        key = (r["op"], r["backend"], r["shape"], r["dtype"])
        cur = groups[key].get(r["n_gpus"])
        if cur is None or r["ms"] < cur["ms"]:
            groups[key][r["n_gpus"]] = r
    return groups


def scaling_rows(records: List[dict]) -> List[dict]:
    rows = []
    for (op, backend, shape, dtype), by_n in sorted(best_per_gpu_count(records).items(), key=lambda kv: str(kv[0])):
        if len(by_n) < 2:
            continue  # a single GPU count says nothing about scaling
        base = by_n.get(1)
        for n in sorted(by_n):
            r = by_n[n]
            eff = base["ms"] / (n * r["ms"]) if base is not None and r["ms"] > 0 else None
            rows.append({"op": op, "backend": backend, "shape": "x".join(map(str, shape)), "dtype": dtype, "n_gpus": n,
                         "pdims": "x".join(map(str, r["pdims"])), "ms": r["ms"],
                         "speedup": (base["ms"] / r["ms"]) if base is not None else None, "efficiency": eff})
    return rows


def _fmt(v) -> str:
    if v is None:
        return "—"
    if isinstance(v, float):
        return f"{v:.3f}" if v < 100 else f"{v:.1f}"
    return str(v)


def markdown_table(rows: List[dict], columns: List[str]) -> str:
    lines = ["| " + " | ".join(columns) + " |", "|" + "---|" * len(columns)]
    for r in rows:
        lines.append("| " + " | ".join(_fmt(r.get(c)) for c in columns) + " |")
    return "\n".join(lines)


def per_op_rows(records: List[dict]) -> List[dict]:
    rows = []
    for r in sorted(records, key=lambda r: (r["op"], r["shape"], r["dtype"], r["n_gpus"], r["pdims"], r["backend"])):
        row = {"op": r["op"], "backend": r["backend"], "shape": "x".join(map(str, r["shape"])), "dtype": r["dtype"],
               "n_gpus": r["n_gpus"], "pdims": "x".join(map(str, r["pdims"])), "ms": r["ms"]}
        row.update({k: v for k, v in r["extra"].items() if isinstance(v, (int, float))})
        rows.append(row)
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("files", nargs="+", help="JSON-lines files ('-' for standard input)")
    ap.add_argument("--csv", action="store_true", help="comma-separated values instead of Markdown")
    args = ap.parse_args(argv)
    records = read_records(args.files)
    if not records:
        print("no measurements found", file=sys.stderr)
        return 1
    ops = per_op_rows(records)
    op_cols = ["op", "backend", "shape", "dtype", "n_gpus", "pdims", "ms"]
    for extra in ("gflops", "egress_gbs", "local_gbs", "frac_of_roofline", "frac_of_link", "e2e_ms"):
        if any(extra in r for r in ops):
            op_cols.append(extra)
    scal = scaling_rows(records)
    scal_cols = ["op", "backend", "shape", "dtype", "n_gpus", "pdims", "ms", "speedup", "efficiency"]
    if args.csv:
        for cols, rows in ((op_cols, ops), (scal_cols, scal)):
            print(",".join(cols))
            for r in rows:
                print(",".join("" if r.get(c) is None else str(r.get(c)) for c in cols))
            print()
        return 0
    print("## Measurements\n")
    print(markdown_table(ops, op_cols))
    print("\n## Strong scaling (fastest process grid at each GPU count)\n")
    print(markdown_table(scal, scal_cols))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
