"""bin/trace_run as a user runs it: a subprocess fed JSON steps on standard input."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest

import traces
from plain_qwen3 import PlainModel
from tiny_configs import CONFIGS

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16"), ("D", "bfloat16")])
def test_trace_run_program(model_dirs, tmp_path, name, dtype):
    vocab = CONFIGS[name]["config"]["vocab_size"]
    reqs = {r: traces.prompt(500 + i, n, vocab) for i, (r, n) in enumerate({"a": 70, "b": 9, "c": 33, "d": 64, "e": 2, "f": 90}.items())}
    steps = traces.mixed(reqs, seed=3)
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(model_dirs[name]), "--dtype", dtype,
                           "--out", str(out), "--max-tokens", str(traces.max_live_tokens(steps))],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    plain = PlainModel(model_dirs[name])
    want = {r: plain.logits(t).numpy() for r, t in reqs.items()}
    tol = {"float32": 1e-4, "bfloat16": 3e-2}[dtype]
    at = {r: 0 for r in reqs}
    for s in steps:
        rows = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab)
        k = 0
        for e in s["entries"]:
            for w in e["want"]:
                ref = want[e["id"]][at[e["id"]] + w]
                assert np.abs(rows[k] - ref).max() <= tol * np.abs(want[e["id"]]).max()
                k += 1
            at[e["id"]] += len(e["tokens"])
        assert k == rows.shape[0]


def test_cli_run_and_spec(model_dirs):
    env = dict(os.environ, PYTHONPATH=ROOT)
    p = subprocess.run([sys.executable, "-m", "inference_bench_b200", "run", "--model", str(model_dirs["A"]), "--prompt-len", "12", "--max-tokens", "5",
                        "--json", "--dtype", "float32", "--max-ctx", "64"], capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    r = json.loads(p.stdout)
    prompt = [(1000 + i * 7 % 5000) % 256 for i in range(12)]
    assert r["prompt_tokens"] == 12 and r["completion_tokens"] == 5 and r["tokens"] == PlainModel(model_dirs["A"]).greedy(prompt, 5)
    p = subprocess.run([sys.executable, "-m", "inference_bench_b200", "spec", "--model", str(model_dirs["C"])], capture_output=True, text=True, env=env)
    assert p.returncode == 0 and json.loads(p.stdout)["derived"]["qkv_rows"] == (5 + 2) * 32
