"""``bfrun``: start N ranks of a program on this machine.

Command-line surface of the reference launcher (bluefog/run/run.py:58-118): ``-np``,
``-H/--hosts``, ``--hostfile``, ``-p/--ssh-port``, ``--network-interface``, ``--use-infiniband``,
``--extra-mpi-flags``, ``--prefix``, ``--verbose``, ``--timeline-filename``, ``-v``.  The reference
builds an ``mpirun`` line; here the launcher itself forks one process per rank, hands every
rank its identity through the environment (RANK, WORLD_SIZE, LOCAL_RANK, LOCAL_WORLD_SIZE,
MASTER_ADDR, MASTER_PORT, the same variables ``torchrun`` sets), forwards signals, and
returns the first non-zero exit code.  Remote hosts are recognised and refused: the target is
one NVSwitch box.
"""
import argparse
import os
import signal
import socket
import subprocess
import sys
import time

from bluefog_b200 import __version__
from bluefog_b200.run import env_util, network_util


def parse_args(argv=None):
    p = argparse.ArgumentParser(description="BlueFog-B200 launcher", prog="bfrun")
    p.add_argument("-v", "--version", action="store_true", dest="version", help="Shows the version.")
    p.add_argument("-np", "--num-proc", action="store", dest="np", type=int,
                   help="Total number of training processes.")
    p.add_argument("-p", "--ssh-port", action="store", dest="ssh_port", type=int,
                   help="SSH port on all the hosts (accepted for compatibility).")
    p.add_argument("--network-interface", action="store", dest="nic",
                   help="Network interface the ranks bind their control sockets to (default: loopback).")
    p.add_argument("--use-infiniband", action="store_true", dest="use_infiniband",
                   help="Accepted for compatibility; the data path of one box is NVLink.")
    p.add_argument("--extra-mpi-flags", action="store", dest="extra_flags",
                   help="Accepted for compatibility and ignored: there is no mpirun underneath.")
    p.add_argument("--prefix", action="store", dest="prefix", help="Accepted for compatibility and ignored.")
    p.add_argument("--verbose", action="store_true", dest="verbose", help="Debug logging in every rank.")
    p.add_argument("--timeline-filename", action="store", dest="timeline_filename",
                   help="Prefix of the per-rank timeline files (<prefix><rank>.json).")
    p.add_argument("--master-port", action="store", dest="master_port", type=int, default=None,
                   help="Port of the rendezvous store (default: a free port).")
    g = p.add_mutually_exclusive_group()
    g.add_argument("-H", "--hosts", action="store", dest="hosts",
                   help="Host names and slots, e.g. localhost:8.")
    g.add_argument("-hostfile", "--hostfile", action="store", dest="hostfile",
                   help="File with one 'hostname slots=N' line per host.")
    p.add_argument("command", nargs=argparse.REMAINDER, help="Command to be executed.")
    return p.parse_args(argv)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _check_hosts(args):
    hosts = None
    if args.hostfile:
        hosts = network_util.parse_hostfile(args.hostfile)
    elif args.hosts:
        hosts = network_util.parse_hosts(args.hosts)
    if hosts is None:
        return
    remote = [h for h, _ in hosts if not network_util.is_local_host(h)]
    if remote:
        raise SystemExit("bfrun: remote hosts (%s) are not supported: this build targets a single "
                         "NVSwitch machine; run one bfrun per machine is not meaningful either, because "
                         "the data path is peer-mapped GPU memory." % ", ".join(remote))
    slots = sum(s for _, s in hosts)
    if args.np and args.np > slots:
        raise SystemExit(f"bfrun: -np {args.np} exceeds the {slots} slots given by the host list.")


def main(argv=None):
    args = parse_args(argv)
    if args.version:
        print(__version__)
        return 0
    if not args.np:
        raise SystemExit("bfrun: -np is required.")
    if not args.command:
        raise SystemExit("bfrun: no command given.")
    _check_hosts(args)
    command = args.command[1:] if args.command[0] == "--" else args.command
    bind = "127.0.0.1"
    if args.nic:
        bind = network_util.interface_address(args.nic)
    port = args.master_port or _free_port()
    base_env = env_util.rank_environment(os.environ, timeline=args.timeline_filename, verbose=args.verbose)
    # Every rank is a PyTorch process whose CPU kernels start an OpenMP team as large as the machine; N ranks
    # doing that at once oversubscribe the cores and spin against each other (a 400 KB clone took 25 ms with
    # 4 ranks on 8 cores).  Unless the user chose a thread count, the cores are shared out among the ranks.
    base_env.setdefault("OMP_NUM_THREADS", str(max(1, (os.cpu_count() or 1) // args.np)))
    procs = []
    for r in range(args.np):
        env = dict(base_env)
        env.update({"RANK": str(r), "WORLD_SIZE": str(args.np), "LOCAL_RANK": str(r),
                    "LOCAL_WORLD_SIZE": str(args.np), "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port),
                    "BLUEFOG_BIND_ADDR": bind})
        procs.append(subprocess.Popen(command, env=env))

    def forward(signum, _frame):
        for p in procs:
            if p.poll() is None:
                p.send_signal(signum)

    signal.signal(signal.SIGINT, forward)
    signal.signal(signal.SIGTERM, forward)
    exit_code = 0
    alive = set(range(args.np))
    while alive:
        for r in list(alive):
            code = procs[r].poll()
            if code is None:
                continue
            alive.discard(r)
            if code != 0 and exit_code == 0:
                exit_code = code
                # one rank failed: give the others a moment to notice, then stop them
                deadline = time.time() + 10
                while time.time() < deadline and any(procs[q].poll() is None for q in alive):
                    time.sleep(0.1)
                for q in alive:
                    if procs[q].poll() is None:
                        procs[q].terminate()
        time.sleep(0.05)
    return exit_code


if __name__ == "__main__":
    sys.exit(main())
