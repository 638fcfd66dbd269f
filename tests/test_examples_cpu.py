"""The example scripts as end-to-end tests on CPU ranks (the reference's examples double as its e2e tests)."""
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ENV = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""), BLUEFOG_B200_FORCE_CPU="1")


def run_example(np_, script, *args, timeout=300):
    cmd = [sys.executable, "-m", "bluefog_b200.run.run", "-np", str(np_), sys.executable,
           os.path.join(ROOT, "examples", script), *args]
    out = subprocess.run(cmd, env=ENV, capture_output=True, text=True, timeout=timeout, cwd=ROOT)
    assert out.returncode == 0, out.stdout[-1500:] + out.stderr[-2500:]
    return out.stdout


@pytest.mark.parametrize("extra", [["--enable-dynamic-topology"], ["--asynchronous-mode"], ["--virtual-topology", "ring"]])
def test_average_consensus_reaches_the_mean(extra, tmp_path):
    out = run_example(4, "pytorch_average_consensus.py", "--no-cuda", "--data-size", "64", "--max-iters", "120",
                      "--save-plot-file", str(tmp_path / "c.png"), *extra)
    errors = [float(m) for m in re.findall(r"relative error after[^:]*:\s*([0-9.]+(?:e[+-]?[0-9]+)?)", out)]
    assert errors and max(errors) < 1e-3, out[-800:]      # ranks share one stdout: lines can merge
    assert (tmp_path / "c.png").exists() or (tmp_path / "c.csv").exists()


@pytest.mark.parametrize("method", ["diffusion", "exact_diffusion", "gradient_tracking", "push_diging"])
def test_decentralized_optimization_methods_converge(method):
    out = run_example(4, "pytorch_optimization.py", "--method", method, "--max-iter", "400")
    norms = [float(l.split("|global gradient| =")[1].split(",")[0]) for l in out.splitlines() if "|global gradient|" in l]
    # plain diffusion keeps a bias of the order of the step size; the corrected methods do not
    assert norms and max(norms) < (0.2 if method == "diffusion" else 1e-2), out[-800:]


@pytest.mark.parametrize("optimizer,extra", [("neighbor_allreduce", ["--atc-style"]), ("win_put", []),
                                             ("push_sum", ["--disable-dynamic-topology"])])
def test_synthetic_benchmark_runs_with_every_optimizer(optimizer, extra):
    out = run_example(2, "pytorch_benchmark.py", "--model", "lenet", "--no-cuda", "--dist-optimizer", optimizer,
                      "--batch-size", "8", "--num-iters", "2", "--num-batches-per-iter", "2", "--num-warmup-batches", "1", *extra)
    assert "Total img/sec on 2 rank(s)" in out, out[-800:]


def test_mnist_example_learns_its_shard():
    out = run_example(2, "pytorch_mnist.py", "--no-cuda", "--log-interval", "25", "--test-batch-size", "256")
    acc = float([l for l in out.splitlines() if "accuracy on the training shard" in l][-1].split()[-1])
    assert acc > 0.5, out[-800:]


def test_resnet_example_trains_checkpoints_and_resumes(tmp_path):
    fmt = str(tmp_path / "ck-{epoch}.pth.tar")
    common = ["--no-cuda", "--batches-per-epoch", "2", "--batch-size", "4", "--image-size", "32", "--num-classes", "10",
              "--val-batch-size", "8", "--checkpoint-format", fmt]
    out = run_example(2, "pytorch_resnet.py", "--epochs", "1", "--batches-per-allreduce", "2", "--log-dir",
                      str(tmp_path / "logs"), *common, timeout=600)
    assert "epoch 0:" in out and (tmp_path / "ck-0.pth.tar").exists() and os.listdir(tmp_path / "logs")
    out = run_example(2, "pytorch_resnet.py", "--epochs", "2", "--resume-from", fmt.format(epoch=0), *common, timeout=600)
    assert "epoch 1:" in out and "epoch 0:" not in out


def test_interactive_notebook_is_valid_and_its_cells_parse():
    import ast
    import json
    with open(os.path.join(ROOT, "examples", "interactive_helloworld.ipynb")) as f:
        nb = json.load(f)
    assert nb["nbformat"] == 4 and nb["cells"]
    import bluefog_b200.torch as bf
    for cell in nb["cells"]:
        if cell["cell_type"] != "code":
            continue
        src = "".join(l for l in cell["source"] if not l.startswith("%%"))
        tree = ast.parse(src)
        # every bf.<name> the notebook teaches exists
        for node in ast.walk(tree):
            if isinstance(node, ast.Attribute) and isinstance(node.value, ast.Name) and node.value.id == "bf":
                assert hasattr(bf, node.attr), node.attr
