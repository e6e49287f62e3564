"""Remote execution helper: one tmux window per command line, optionally through ssh
(``dl_code/tmux_cluster/tmux.py:10-136``, ``utils.py:9-44``).  ``dry_run`` prints the shell
lines instead of executing them."""
from __future__ import annotations

import os
import shlex
import subprocess
import time


def ossystem(cmd, dry_run=False):
    print(cmd)
    return 0 if dry_run else os.system(cmd)


def wait_for_file(path, timeout_s=60.0, poll_s=0.2):
    t0 = time.time()
    while not os.path.exists(path):
        if time.time() - t0 > timeout_s:
            return False
        time.sleep(poll_s)
    return True


def load_yaml(path):
    import yaml

    with open(path) as f:
        return yaml.safe_load(f)


class Task:
    def __init__(self, host, command):
        self.host, self.command = host, command

    def shell_line(self, session, window):
        inner = self.command
        if self.host not in ("localhost", "127.0.0.1"):
            inner = "ssh {} -t {}".format(self.host, shlex.quote(inner))
        return "tmux send-keys -t {}:{} {} Enter".format(session, window, shlex.quote(inner))


class Job:
    def __init__(self, name, master="localhost"):
        self.name, self.master, self.tasks = name, master, []

    def add(self, host, command):
        self.tasks.append(Task(host, command))

    def lines(self):
        out = ["tmux kill-session -t {} 2>/dev/null; tmux new-session -d -s {} -n w0".format(self.name, self.name)]
        for i, t in enumerate(self.tasks):
            if i > 0:
                out.append("tmux new-window -t {} -n w{}".format(self.name, i))
            out.append(t.shell_line(self.name, "w%d" % i))
        return out

    def run(self, dry_run=True):
        for line in self.lines():
            ossystem(line, dry_run=dry_run)


Run = Job
