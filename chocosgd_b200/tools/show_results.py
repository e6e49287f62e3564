"""Load experiment folders and reorganise their JSON records into curves and summaries
(``dl_code/pcode/tools/show_results.py:68-380``).

An experiment folder holds ``arguments.pickle`` and one sub-folder per rank with
``log-*.json``.  Records are split into train / test-local / test-averaged series, can be
filtered by argument conditions, and summarised (mean / std / max / min / count) with pandas."""
from __future__ import annotations

import functools
import json
import os
from typing import Dict, List

from ..utils.op_files import load_pickle


def get_pickle_info(root, folders):
    return [load_pickle(os.path.join(root, f, "arguments.pickle")) for f in folders]


def _load_rank_records(rank_dir):
    recs = []
    files = sorted((f for f in os.listdir(rank_dir) if f.startswith("log-") and f.endswith(".json")),
                   key=lambda s: int(s[4:-5]))
    for f in files:
        with open(os.path.join(rank_dir, f)) as fh:
            recs += json.load(fh)
    return recs


def load_experiment(path) -> dict:
    """{'arguments': dict, 'records': {rank: [record, ...]}}"""
    args_path = os.path.join(path, "arguments.pickle")
    arguments = load_pickle(args_path) if os.path.exists(args_path) else {}
    if not isinstance(arguments, dict):
        arguments = dict(vars(arguments))
    records = {}
    for d in sorted(os.listdir(path)):
        full = os.path.join(path, d)
        if os.path.isdir(full) and d.isdigit():
            records[int(d)] = _load_rank_records(full)
    return {"arguments": arguments, "records": records, "path": path}


def split_records(records: List[dict]) -> Dict[str, List[dict]]:
    out = {"train": [], "test_local": [], "test_averaged": [], "test_best": [], "timer": [], "stat": []}
    for r in records:
        m = r.get("measurement")
        if m == "timer":
            out["timer"].append(r)
        elif m == "stat":
            out["stat"].append(r)
        elif r.get("split") == "train":
            out["train"].append(r)
        elif r.get("split") == "test":
            t = r.get("type")
            if t == "local_model":
                out["test_local"].append(r)
            elif t == "averaged_model":
                out["test_averaged"].append(r)
            elif t == "local_model_avg":
                out["test_best"].append(r)
    return out


def _match(arguments, conditions):
    return all(str(arguments.get(k)) in [str(x) for x in (v if isinstance(v, (list, tuple)) else [v])]
               for k, v in (conditions or {}).items())


def find_experiments(root, conditions=None):
    """Every folder below ``root`` that contains ``arguments.pickle`` and matches ``conditions``."""
    found = []
    for dirpath, _, files in os.walk(root):
        if "arguments.pickle" in files:
            exp = load_experiment(dirpath)
            if _match(exp["arguments"], conditions):
                found.append(exp)
    return found


def curve(exp, split="test_local", metric="top1", x="epoch", reduce_ranks="mean"):
    """(xs, ys) of one metric, averaged over ranks at equal x."""
    acc = {}
    for recs in exp["records"].values():
        for r in split_records(recs)[split]:
            if metric in r and x in r:
                acc.setdefault(round(float(r[x]), 6), []).append(float(r[metric]))
    xs = sorted(acc)
    red = {"mean": lambda v: sum(v) / len(v), "max": max, "min": min}[reduce_ranks]
    return xs, [red(acc[k]) for k in xs]


def summarize(exps, metric="top1", split="test_local", keys=("optimizer", "comm_op", "graph_topology", "lr")):
    """pandas DataFrame: best value of ``metric`` per experiment, grouped over repetitions."""
    import pandas as pd

    rows = []
    for e in exps:
        _, ys = curve(e, split, metric)
        if not ys:
            continue
        row = {k: e["arguments"].get(k) for k in keys}
        row[metric] = min(ys) if metric in ("loss", "ppl") else max(ys)
        rows.append(row)
    df = pd.DataFrame(rows)
    if df.empty:
        return df
    for k in keys:
        df[k] = df[k].astype(str)
    return df.groupby(list(keys))[metric].agg(["mean", "std", "max", "min", "count"]).reset_index()


def extract_list_of_records(list_of_records, conditions):
    return [r for r in list_of_records if _match(r["arguments"], conditions)]
