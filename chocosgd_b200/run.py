"""Launcher: ``python -m chocosgd_b200.run <all main.py flags>`` starts one rank per graph node.

The reference builds an ``mpirun`` command from a hostfile, or one ``python main.py
--local_rank r`` command per rank, and runs it locally or inside tmux over ssh
(``dl_code/run.py:10-174``, ``dl_code/tmux_cluster/``).  Here ranks are plain child
processes of one node (the 8-GPU NVSwitch box is the unit this framework targets); every
non-None flag is forwarded as ``--k v`` like the reference does, and the rendezvous is given
through ``RANK`` / ``WORLD_SIZE`` / ``MASTER_ADDR`` / ``MASTER_PORT``.  A hostfile
(``host slots=N`` lines) is parsed for slot counts; entries for other hosts produce the
ssh/tmux command lines (``--remote_exec True`` prints / runs them through ``tmux_cluster``)."""
from __future__ import annotations

import os
import re
import signal
import socket
import subprocess
import sys
import time

from . import config as cfg


def read_hostfile(file_path):
    """[{'host': ..., 'slots': int}] from ``host slots=N`` lines."""
    hosts = []
    pattern = re.compile(r"^(\S+)\s+slots=(\d+)")
    with open(file_path) as f:
        for line in f:
            m = pattern.match(line.strip())
            if m:
                hosts.append({"host": m.group(1), "slots": int(m.group(2))})
    return hosts


def map_slot(hosts):
    """One host name per rank, in hostfile order."""
    out = []
    for h in hosts:
        out += [h["host"]] * h["slots"]
    return out


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def build_rank_command(conf, rank, python=None):
    python = python or (conf.python_path if conf.python_path not in (None, "python") else sys.executable)
    args = conf.to_cli(skip=("local_rank", "hostfile", "clean_python", "remote_exec", "work_dir"))
    return [python, "-m", "chocosgd_b200.main"] + args + ["--local_rank", str(rank)]


def rank_env(conf, rank, world, port, base=None):
    env = dict(base if base is not None else os.environ)
    env.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR=conf.master_addr,
               MASTER_PORT=str(port))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    if conf.mpi_env:
        for kv in conf.mpi_env.split(","):
            if "=" in kv:
                k, v = kv.split("=", 1)
                env[k] = v
    return env


def launch_local(conf, timeout=None):
    """Start ``n_mpi_process`` ranks on this machine; returns the list of exit codes."""
    world = conf.n_mpi_process
    port = conf.master_port or free_port()
    procs = []
    for r in range(world):
        procs.append(subprocess.Popen(build_rank_command(conf, r), env=rank_env(conf, r, world, port),
                                      cwd=conf.work_dir or None, start_new_session=True))
    codes, t0 = [None] * world, time.time()
    try:
        while any(c is None for c in codes):
            for i, p in enumerate(procs):
                if codes[i] is None:
                    codes[i] = p.poll()
            if any(c not in (None, 0) for c in codes) or (timeout and time.time() - t0 > timeout):
                break  # one rank failed: stop the others (exact process groups, never by pattern)
            time.sleep(0.2)
    finally:
        for i, p in enumerate(procs):
            if p.poll() is None:
                try:
                    os.killpg(p.pid, signal.SIGTERM)
                except ProcessLookupError:
                    pass
                codes[i] = p.wait()
    return codes


def main(argv=None):
    conf = cfg.get_args(argv)
    if conf.hostfile and os.path.exists(conf.hostfile):
        hosts = map_slot(read_hostfile(conf.hostfile))
        if len(hosts) < conf.n_mpi_process:
            raise SystemExit("the hostfile offers fewer slots than --n_mpi_process")
        remote = [h for h in hosts[: conf.n_mpi_process] if h not in ("localhost", "127.0.0.1", socket.gethostname())]
        if remote:
            from .tmux_cluster import Job

            port = conf.master_port or 29500
            job = Job(conf.experiment or "choco", conf.master_addr)
            for r, h in enumerate(hosts[: conf.n_mpi_process]):
                env = " ".join(f"{k}={v}" for k, v in (("RANK", r), ("WORLD_SIZE", conf.n_mpi_process),
                                                       ("MASTER_ADDR", conf.master_addr), ("MASTER_PORT", port)))
                job.add(h, env + " " + " ".join(build_rank_command(conf, r, conf.python_path)))
            job.run(dry_run=not conf.remote_exec)
            return 0
    codes = launch_local(conf)
    return 0 if all(c == 0 for c in codes) else 1


if __name__ == "__main__":
    sys.exit(main())
