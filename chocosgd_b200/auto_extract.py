"""``python -m chocosgd_b200.auto_extract --in_dir <experiment root>`` walks the folder and
writes ``summary.pickle`` with every run's arguments and curves (``dl_code/auto_extract.py:37-41``)."""
from __future__ import annotations

import argparse
import os

from .tools.show_results import curve, find_experiments, split_records
from .utils.op_files import write_pickle


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--in_dir", required=True)
    p.add_argument("--out_name", default="summary.pickle")
    a = p.parse_args(argv)
    out = []
    for e in find_experiments(a.in_dir):
        item = {"arguments": e["arguments"], "path": e["path"], "curves": {}}
        for split in ("train", "test_local", "test_averaged"):
            names = set()
            for recs in e["records"].values():
                for r in split_records(recs)[split]:
                    names |= {k for k, v in r.items() if isinstance(v, (int, float)) and k not in ("rank", "epoch")}
            for m in names:
                item["curves"][f"{split}/{m}"] = curve(e, split, m)
        out.append(item)
    path = os.path.join(a.in_dir, a.out_name)
    write_pickle(out, path)
    print(f"wrote {len(out)} runs to {path}")
    return path


if __name__ == "__main__":
    main()
