"""``ibfrun``: interactive cluster for notebooks (role of bluefog/run/interactive_run.py).

``ibfrun start -np N`` starts an ipyparallel controller and N engines, each engine being one
rank launched through ``bfrun``; ``ibfrun stop`` shuts them down.  Notebooks then attach with
``ipyparallel.Client(profile="bluefog")`` and run ``%%px`` cells that ``import
bluefog_b200.torch as bf; bf.init()``.  ipyparallel is an optional dependency: without it the
command explains what is missing instead of failing obscurely.
"""
import argparse
import json
import os
import signal
import subprocess
import sys
import time

PROFILE = "bluefog"
STATE_DIR = os.path.join(os.path.expanduser("~"), ".bluefog_b200")
STATE_FILE = os.path.join(STATE_DIR, "ibfrun.json")


def _require_ipyparallel():
    try:
        import ipyparallel  # noqa: F401
    except ImportError:
        raise SystemExit("ibfrun needs the optional package 'ipyparallel' (pip install ipyparallel).")


def _version():
    from bluefog_b200 import __version__
    return __version__


def _refuse_remote_hosts(args):
    """The same rule as bfrun: every listed host must be this machine."""
    from bluefog_b200.run import network_util
    hosts = []
    if args.hosts:
        hosts += [h for h, _ in network_util.parse_hosts(args.hosts)]
    if args.hostfile:
        hosts += [h for h, _ in network_util.parse_hostfile(args.hostfile)]
    remote = [h for h in hosts if not network_util.is_local_host(h)]
    if remote:
        raise SystemExit("ibfrun: only this machine is supported (CUDA IPC data plane); remote hosts: " + ", ".join(remote))


def parse_args(argv=None):
    p = argparse.ArgumentParser(prog="ibfrun", description="Interactive BlueFog-B200 cluster")
    p.add_argument("action", choices=["start", "stop", "status"])
    p.add_argument("-np", "--num-proc", dest="np", type=int, default=None)
    p.add_argument("--ipython-profile", dest="profile", default=PROFILE)
    p.add_argument("--enable-heartbeat", action="store_true",
                   help="Keep the heartbeat check between controller and engines (off by default: an engine inside a "
                        "long collective otherwise looks dead).")
    p.add_argument("--disable-heartbeat", action="store_true", help="Accepted; this is the default.")
    p.add_argument("--verbose", action="store_true")
    p.add_argument("-v", "--version", action="version", version=_version())
    p.add_argument("-H", "--hosts", dest="hosts", default=None,
                   help="host:slots list; only this machine is supported (the data plane is CUDA IPC).")
    p.add_argument("-hostfile", "--hostfile", dest="hostfile", default=None, help="As --hosts, one 'host slots=N' per line.")
    p.add_argument("-p", "--ssh-port", dest="ssh_port", type=int, default=None, help="Accepted; no remote hosts.")
    p.add_argument("--network-interface", dest="nic", default=None, help="Accepted; ranks talk over loopback.")
    p.add_argument("--use-infiniband", action="store_true", help="Accepted; no effect inside one machine.")
    p.add_argument("--extra-mpi-flags", dest="extra_flags", default=None, help="Accepted; there is no MPI.")
    return p.parse_args(argv)


def _load_state():
    try:
        with open(STATE_FILE) as f:
            return json.load(f)
    except (OSError, ValueError):
        return None


def _alive(pid):
    try:
        os.kill(pid, 0)
        return True
    except OSError:
        return False


def start(args):
    if not args.np:
        raise SystemExit("ibfrun start: -np is required.")
    _refuse_remote_hosts(args)
    _require_ipyparallel()
    state = _load_state()
    if state and any(_alive(p) for p in state.get("pids", [])):
        raise SystemExit("ibfrun: a cluster is already running; use 'ibfrun stop' first.")
    os.makedirs(STATE_DIR, exist_ok=True)
    out = None if args.verbose else subprocess.DEVNULL
    controller = subprocess.Popen([sys.executable, "-m", "ipyparallel.controller", f"--profile={args.profile}",
                                   "--ip=127.0.0.1"], stdout=out, stderr=out, start_new_session=True)
    time.sleep(3.0)   # connection files must exist before the engines start
    engine_cmd = [sys.executable, "-m", "ipyparallel.engine", f"--profile={args.profile}"]
    if not args.enable_heartbeat:
        engine_cmd.append("--IPEngine.max_heartbeat_misses=0")
    engines = subprocess.Popen([sys.executable, "-m", "bluefog_b200.run.run", "-np", str(args.np), "--"] + engine_cmd,
                               stdout=out, stderr=out, start_new_session=True)
    with open(STATE_FILE, "w") as f:
        json.dump({"pids": [controller.pid, engines.pid], "np": args.np, "profile": args.profile}, f)
    print(f"ibfrun: controller pid {controller.pid}, {args.np} engines under pid {engines.pid}; "
          f"attach with ipyparallel.Client(profile='{args.profile}')")
    return 0


def stop(_args):
    state = _load_state()
    if not state:
        print("ibfrun: nothing to stop.")
        return 0
    for pid in state.get("pids", []):
        if _alive(pid):
            try:
                os.killpg(pid, signal.SIGINT)   # exactly the process groups this tool started
            except OSError:
                pass
    deadline = time.time() + 10
    while time.time() < deadline and any(_alive(p) for p in state.get("pids", [])):
        time.sleep(0.2)
    for pid in state.get("pids", []):
        if _alive(pid):
            try:
                os.killpg(pid, signal.SIGKILL)
            except OSError:
                pass
    os.remove(STATE_FILE)
    print("ibfrun: stopped.")
    return 0


def status(_args):
    state = _load_state()
    if not state:
        print("ibfrun: no cluster.")
        return 1
    alive = [p for p in state["pids"] if _alive(p)]
    print(f"ibfrun: {len(alive)}/{len(state['pids'])} launcher processes alive, np={state['np']}")
    return 0 if alive else 1


def interrupt_hanged_processes(client, timeout=0.2):
    """Sends SIGINT to engines that do not answer a ping within ``timeout`` seconds
    (the engines of an interactive session that are stuck in a collective)."""
    pids = client[:].apply_async(os.getpid).get_dict()
    probes = {eid: client[eid].apply_async(lambda: 0) for eid in client.ids}
    time.sleep(timeout)
    for eid, res in probes.items():
        if not res.ready():
            os.kill(pids[eid], signal.SIGINT)


def main(argv=None):
    args = parse_args(argv)
    return {"start": start, "stop": stop, "status": status}[args.action](args)


if __name__ == "__main__":
    sys.exit(main())
