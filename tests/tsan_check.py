"""Runs multi-process CPU cases of tests/_worker.py against a ThreadSanitizer build of the host runtime.

The reference has no sanitizer job (its setup.py builds with `-O2 -Wall` only, setup.py:103).  Here the C++ runtime
(background loop, negotiation, handles, fast path, control plane, windows on shared memory, timeline) can be built with
`-fsanitize=thread` beside the regular library and loaded through ``BLUEFOG_B200_NATIVE``; device code is not
instrumented, so the cases run as CPU ranks.

    make tsan                                   # builds build/tsan/... and runs the default cases
    python tests/tsan_check.py --cases collectives,windows --ranks 4

Exit status 1 when the sanitizer reported anything that ``tests/tsan.supp`` does not cover.
"""
import argparse
import glob
import os
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEFAULT_CASES = "collectives,neighbor_ops,windows,errors,skip_negotiate,optimizers,runtime_stats,win_guard"


def find_libtsan():
    for cc in (os.environ.get("CXX"), "/usr/bin/g++", "g++"):
        if not cc:
            continue
        try:
            path = subprocess.run([cc, "-print-file-name=libtsan.so"], capture_output=True, text=True).stdout.strip()
        except OSError:
            continue
        if os.path.isabs(path) and os.path.exists(path):
            return path
    return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", default=DEFAULT_CASES)
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--native", default="", help="the instrumented _C*.so (default: build/tsan/bluefog_b200/_C*.so)")
    ap.add_argument("--timeout", type=int, default=1800)
    args = ap.parse_args()
    native = args.native or next(iter(glob.glob(os.path.join(ROOT, "build", "tsan", "bluefog_b200", "_C*.so"))), "")
    if not native or not os.path.exists(native):
        print("no ThreadSanitizer build found; build one with `make tsan-build`", file=sys.stderr)
        return 2
    libtsan = find_libtsan()
    if libtsan is None:
        print("libtsan.so not found for the host compiler", file=sys.stderr)
        return 2
    failed = []
    with tempfile.TemporaryDirectory(prefix="bfb_tsan_") as logdir:
        for case in [c for c in args.cases.split(",") if c]:
            env = dict(os.environ)
            env.update({
                "PYTHONPATH": ROOT + os.pathsep + env.get("PYTHONPATH", ""),
                "BLUEFOG_B200_NATIVE": native,
                "LD_PRELOAD": libtsan,
                "CUDA_VISIBLE_DEVICES": "",
                "TSAN_OPTIONS": "log_path=%s exitcode=0 report_signal_unsafe=0 history_size=4 suppressions=%s" % (
                    os.path.join(logdir, case), os.path.join(ROOT, "tests", "tsan.supp")),
            })
            cmd = [sys.executable, "-m", "bluefog_b200.run.run", "-np", str(args.ranks), sys.executable,
                   os.path.join(ROOT, "tests", "_worker.py"), case]
            proc = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=args.timeout)
            reports = []
            for path in sorted(glob.glob(os.path.join(logdir, case + ".*"))):
                with open(path) as f:
                    text = f.read()
                if "WARNING: ThreadSanitizer" in text:
                    reports.append(text)
            status = "ok" if proc.returncode == 0 and not reports else "FAILED"
            print("%-20s ranks=%d exit=%d sanitizer reports=%d  %s" % (case, args.ranks, proc.returncode, len(reports), status),
                  flush=True)
            if status != "ok":
                failed.append(case)
                if proc.returncode != 0:
                    print(proc.stdout[-2000:] + proc.stderr[-2000:])
                for text in reports[:2]:
                    print(text[:6000])
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
