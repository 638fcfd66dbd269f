"""bfrun: argument surface, environment of the ranks, exit codes, refusal of remote hosts."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENV = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), BLUEFOG_B200_FORCE_CPU="1")


def bfrun(*args, timeout=120):
    return subprocess.run([sys.executable, "-m", "bluefog_b200.run.run", *args], env=ENV, capture_output=True,
                          text=True, timeout=timeout)


def test_version_and_required_arguments():
    assert bfrun("-v").stdout.strip() == "0.1.0"
    assert bfrun("python", "-c", "pass").returncode != 0          # -np missing
    assert bfrun("-np", "2").returncode != 0                       # command missing


def test_ranks_get_identity_and_flags(tmp_path):
    # one os.write per rank: a short write to a pipe is atomic, so the ranks' lines cannot interleave
    code = ("import os;e=os.environ;os.write(1,(' '.join(['R',e['RANK'],e['WORLD_SIZE'],e['LOCAL_RANK'],"
            "str(e.get('BLUEFOG_TIMELINE')),str(e.get('BLUEFOG_LOG_LEVEL'))])+chr(10)).encode())")
    out = bfrun("-np", "3", "--timeline-filename", str(tmp_path / "t_"), "--verbose", sys.executable, "-c", code)
    assert out.returncode == 0, out.stderr
    lines = sorted(l for l in out.stdout.splitlines() if l.startswith("R "))
    assert [l.split()[1] for l in lines] == ["0", "1", "2"]
    assert all(l.split()[2] == "3" and l.split()[4].endswith("t_") and l.split()[5] == "debug" for l in lines)


def test_exit_code_of_a_failing_rank_is_returned():
    code = "import os,sys;sys.exit(7 if os.environ['RANK']=='1' else 0)"
    assert bfrun("-np", "2", sys.executable, "-c", code).returncode == 7


def test_remote_hosts_are_refused():
    out = bfrun("-np", "2", "-H", "some-other-machine.invalid:2", sys.executable, "-c", "pass")
    assert out.returncode != 0 and "not supported" in (out.stderr + out.stdout)
    assert bfrun("-np", "2", "-H", "localhost:2", sys.executable, "-c", "pass").returncode == 0


def test_end_to_end_allreduce_under_bfrun():
    code = ("import torch, bluefog_b200.torch as bf; bf.init(); "
            "x = bf.allreduce(torch.full((3,), float(bf.rank()))); "
            "assert x.tolist() == [1.5] * 3, x; bf.barrier(); bf.shutdown()")
    out = bfrun("-np", "4", sys.executable, "-c", code)
    assert out.returncode == 0, out.stderr[-2000:]


@pytest.mark.parametrize("mode", ["normal", "compute-only", "sleep-and-communicate"])
def test_linear_speedup_study_runs_in_every_mode(mode):
    import json
    script = os.path.join(ROOT, "benchmarks", "linear_speedup_study.py")
    out = bfrun("-np", "2", sys.executable, script, "--no-cuda", "--mode", mode, "--rounds", "2", "--steps-per-round", "3",
                "--warmup-steps", "1", "--samples", "64", "--dim", "16", "--sleep-seconds", "0.01", "--topology", "ring")
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert line["mode"] == mode and line["n_ranks"] == 2 and line["job_total"] > line["per_rank"] > 0


def test_resource_allocation_example_converges_towards_the_admm_solution(tmp_path):
    script = os.path.join(ROOT, "examples", "resource_allocation.py")
    out = bfrun("-np", "3", sys.executable, script, "--no-cuda", "--iterations", "400", "--plot", str(tmp_path / "c.png"),
                timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = {l.split("relative error")[0].strip(): l for l in out.stdout.splitlines() if "relative error" in l}
    assert set(lines) == {"EXTRA", "exact diffusion", "gradient tracking"}
    for l in lines.values():     # "... relative error E after N iterations (E100 after 100)"
        final, early = float(l.split("relative error")[1].split()[0]), float(l.split("(")[1].split()[0])
        assert final < 0.5 * early, l
    assert (tmp_path / "c.png").exists() or (tmp_path / "c.csv").exists()


def test_ibfrun_accepts_the_reference_flags_and_refuses_remote_hosts(tmp_path):
    from bluefog_b200.run import interactive_run
    args = interactive_run.parse_args(["start", "-np", "4", "--ipython-profile", "p", "--enable-heartbeat", "-H", "localhost:4",
                                       "-p", "22", "--network-interface", "lo", "--use-infiniband", "--extra-mpi-flags", "x"])
    assert args.np == 4 and args.profile == "p" and args.enable_heartbeat
    with pytest.raises(SystemExit, match="remote hosts: elsewhere"):
        interactive_run.start(interactive_run.parse_args(["start", "-np", "2", "-H", "elsewhere:2"]))
    hostfile = tmp_path / "hosts"
    hostfile.write_text("localhost slots=2\nfar.away slots=2\n")
    with pytest.raises(SystemExit, match="far.away"):
        interactive_run.start(interactive_run.parse_args(["start", "-np", "4", "-hostfile", str(hostfile)]))
    with pytest.raises(SystemExit, match="-np is required"):
        interactive_run.start(interactive_run.parse_args(["start"]))


def test_cores_are_shared_among_ranks_unless_the_user_set_a_thread_count():
    code = "import os; os.write(1, ('T ' + os.environ['OMP_NUM_THREADS'] + chr(10)).encode())"
    env = {k: v for k, v in ENV.items() if k != "OMP_NUM_THREADS"}
    cmd = [sys.executable, "-m", "bluefog_b200.run.run", "-np", "2", sys.executable, "-c", code]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=120)
    assert out.stdout.split().count(str(max(1, (os.cpu_count() or 1) // 2))) == 2, out.stdout + out.stderr[-500:]
    out = subprocess.run(cmd, env=dict(env, OMP_NUM_THREADS="3"), capture_output=True, text=True, timeout=120)
    assert out.stdout.split().count("3") == 2, out.stdout


def test_host_parsing(tmp_path):
    from bluefog_b200.run import network_util, env_util
    assert network_util.parse_hosts("a:2, b:4,c") == [("a", 2), ("b", 4), ("c", 1)]
    f = tmp_path / "hosts"
    f.write_text("# comment\nlocalhost slots=8\nnode2 slots=4 max_slots=4\n")
    assert network_util.parse_hostfile(str(f)) == [("localhost", 8), ("node2", 4)]
    assert network_util.is_local_host("localhost") and network_util.is_local_host("127.0.0.1")
    env = env_util.rank_environment({"A": "1", "RANK": "5", "BASH_FUNC_x%%": "y"}, timeline="p", verbose=True)
    assert env == {"A": "1", "BLUEFOG_TIMELINE": "p", "BLUEFOG_LOG_LEVEL": "debug"}


_FAKE_CONTROLLER = """
import os, signal, sys, time
out = os.environ["IBF_TEST_OUT"]
with open(os.path.join(out, "controller"), "w") as f:
    f.write(" ".join(sys.argv[1:]))
signal.signal(signal.SIGINT, lambda *_: sys.exit(0))
signal.signal(signal.SIGTERM, lambda *_: sys.exit(0))
while True:
    time.sleep(0.1)
"""

_FAKE_ENGINE = """
import os, signal, sys, time
e, out = os.environ, os.environ["IBF_TEST_OUT"]
with open(os.path.join(out, "engine_" + e["RANK"]), "w") as f:
    f.write("%s %s %s %d %s" % (e["RANK"], e["WORLD_SIZE"], e["LOCAL_RANK"], os.getpid(), " ".join(sys.argv[1:])))
signal.signal(signal.SIGINT, lambda *_: sys.exit(0))
signal.signal(signal.SIGTERM, lambda *_: sys.exit(0))
while True:
    time.sleep(0.1)
"""


def _alive(pid):
    try:
        os.kill(pid, 0)
        return True
    except OSError:
        return False


def test_ibfrun_starts_a_controller_and_engines_as_ranks_and_stops_them(tmp_path):
    """The whole start / status / stop cycle of the interactive launcher against a stand-in for the optional
    ipyparallel package (a controller and engines that only record how they were started): the engines come up as ranks
    of one job, a second start is refused while the cluster lives, stop ends exactly the processes that were started."""
    import time
    fake = tmp_path / "fake" / "ipyparallel"
    fake.mkdir(parents=True)
    (fake / "__init__.py").write_text("")
    (fake / "controller.py").write_text(_FAKE_CONTROLLER)
    (fake / "engine.py").write_text(_FAKE_ENGINE)
    out = tmp_path / "out"
    out.mkdir()
    env = dict(ENV, PYTHONPATH=str(tmp_path / "fake") + os.pathsep + ENV["PYTHONPATH"], HOME=str(tmp_path),
               IBF_TEST_OUT=str(out))

    def ibfrun(*args):
        return subprocess.run([sys.executable, "-m", "bluefog_b200.run.interactive_run", *args], env=env,
                              capture_output=True, text=True, timeout=120)

    assert ibfrun("status").returncode == 1                         # nothing yet
    started = ibfrun("start", "-np", "2", "--ipython-profile", "t")
    assert started.returncode == 0, started.stderr
    try:
        deadline = time.time() + 30
        while time.time() < deadline and not ((out / "engine_0").exists() and (out / "engine_1").exists()):
            time.sleep(0.2)
        engines = [(out / f"engine_{r}").read_text().split() for r in range(2)]
        assert [e[:3] for e in engines] == [["0", "2", "0"], ["1", "2", "1"]]
        assert all("--profile=t" in e and "--IPEngine.max_heartbeat_misses=0" in e for e in engines)
        assert "--profile=t" in (out / "controller").read_text()
        pids = [int(e[3]) for e in engines]
        assert all(_alive(p) for p in pids)
        assert ibfrun("status").returncode == 0
        again = ibfrun("start", "-np", "2", "--ipython-profile", "t")
        assert again.returncode != 0 and "already running" in again.stderr
    finally:
        stopped = ibfrun("stop")
    assert stopped.returncode == 0 and "stopped" in stopped.stdout
    deadline = time.time() + 10
    while time.time() < deadline and any(_alive(p) for p in pids):
        time.sleep(0.2)
    assert not any(_alive(p) for p in pids)
    assert ibfrun("status").returncode == 1
    assert "nothing to stop" in ibfrun("stop").stdout


def test_interrupt_hanged_processes_signals_only_the_engines_that_do_not_answer(tmp_path):
    """Engines stuck in a collective do not answer a ping: they, and only they, get SIGINT."""
    import time
    from bluefog_b200.run import interactive_run
    code = ("import os, signal, sys, time\n"
            "signal.signal(signal.SIGINT, lambda *_: (open(sys.argv[1], 'w').write('interrupted'), sys.exit(0)))\n"
            "open(sys.argv[1] + '.up', 'w').write('up')\n"
            "while True: time.sleep(0.05)\n")
    procs = [subprocess.Popen([sys.executable, "-c", code, str(tmp_path / f"e{k}")]) for k in range(2)]
    try:
        deadline = time.time() + 20
        while time.time() < deadline and not all((tmp_path / f"e{k}.up").exists() for k in range(2)):
            time.sleep(0.05)

        class Result:
            def __init__(self, value, ready=True):
                self.value, self._ready = value, ready

            def get_dict(self):
                return self.value

            def ready(self):
                return self._ready

        class View:
            def __init__(self, client, eid=None):
                self.client, self.eid = client, eid

            def apply_async(self, fn):
                if self.eid is None:
                    return Result({k: p.pid for k, p in enumerate(procs)})
                return Result(0, ready=self.client.answers[self.eid])

        class Client:
            ids = [0, 1]
            answers = {0: True, 1: False}        # engine 1 hangs

            def __getitem__(self, key):
                return View(self, None if isinstance(key, slice) else key)

        interactive_run.interrupt_hanged_processes(Client(), timeout=0.05)
        procs[1].wait(timeout=10)
        assert (tmp_path / "e1").read_text() == "interrupted"
        assert procs[0].poll() is None and not (tmp_path / "e0").exists()
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
