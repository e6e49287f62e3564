"""JSON-record logger with the reference's record schema.

Records are ``{"measurement": name, **values, **tags}``; ``save_json`` writes ``log-1.json``
and rotates to ``log-K.json`` after more than 1000 records; ``log`` timestamps to stdout and
``log.txt`` (``dl_code/pcode/utils/logging.py:10-154``).  The result tools consume exactly
these files."""
from __future__ import annotations

import json
import os
import platform
import time


class Logger:
    def __init__(self, file_folder):
        self.file_folder = file_folder
        os.makedirs(file_folder, exist_ok=True)
        self.file_json = os.path.join(file_folder, "log-1.json")
        self.file_txt = os.path.join(file_folder, "log.txt")
        self.values = []

    def log_metric(self, name, values, tags, display=False):
        self.values.append({"measurement": name, **values, **tags})
        if display:
            print("{name}: {values} ({tags})".format(name=name, values=values, tags=tags))

    def log(self, value):
        content = time.strftime("%Y-%m-%d %H:%M:%S") + "\t" + value
        print(content)
        self.save_txt(content)

    def save_json(self):
        with open(self.file_json, "w") as fp:
            json.dump(self.values, fp, indent=" ")
        if len(self.values) > 1e3:
            self.values = []
            self.redirect_new_json()

    def save_txt(self, value):
        with open(self.file_txt, "a") as fp:
            fp.write(value + "\n")

    def redirect_new_json(self):
        existing = [f for f in os.listdir(self.file_folder) if "json" in f]
        self.file_json = os.path.join(self.file_folder, "log-{}.json".format(len(existing) + 1))


def _now():
    return time.strftime("%Y-%m-%d %H:%M:%S")


def display_args(conf, graph):
    if graph.rank != 0:
        return
    print("\n\nparameters: ")
    for arg, val in sorted(vars(conf).items()):
        print("\t" + str(arg) + "\t" + str(val))
    print(
        "\n\nexperiment platform: rank {} on {} {}-{}".format(
            graph.rank, platform.node(), "GPU" if graph.on_cuda else "CPU", graph.device
        )
    )
    for name in ("n_nodes", "world", "rank", "device", "on_cuda"):
        print("\t{}: {}".format(name, getattr(graph, name)))
    print("\tget_neighborhood: {}\n\n".format(graph.get_neighborhood()))


def display_training_stat(logger, graph, scheduler, tracker, n_bits_to_transmit, display=True, extra=None):
    values = {
        "time": _now(),
        "rank": graph.rank,
        "epoch": scheduler.epoch_,
        "local_index": scheduler.local_index,
        "n_bits_to_transmit": n_bits_to_transmit / 8 / (2 ** 20),
        **tracker(),
    }
    if extra:
        values.update(extra)
    logger.log_metric(name="runtime", values=values, tags={"split": "train"}, display=display)


def display_test_stat(logger, graph, scheduler, tracker, label="local"):
    logger.log_metric(
        name="runtime",
        values={"time": _now(), "rank": graph.rank, "epoch": scheduler.epoch_, **tracker()},
        tags={"split": "test", "type": label},
        display=True,
    )
    logger.save_json()


def display_best_test_stat(logger, graph, scheduler):
    logger.log_metric(
        name="runtime",
        values={
            "time": _now(),
            "rank": graph.rank,
            "epoch": scheduler.epoch_,
            "best_perf": scheduler.best_tracker.best_perf,
        },
        tags={"split": "test", "type": "local_model_avg"},
        display=False,
    )
    logger.log(
        "best performance at local index {} (best epoch {}, current epoch {:.3f}): {}.".format(
            scheduler.local_index,
            scheduler.best_tracker.get_best_perf_loc(),
            scheduler.epoch_,
            scheduler.best_tracker.best_perf,
        )
    )
