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
    assert p.returncode == 0 and json.loads(p.stdout)["derived"]["qkv_rows"] == (5 + 2) * 32 and json.loads(p.stdout)["derived"]["q_dim"] == 160


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_layers_follow_the_plain_model_layer_by_layer(model_dirs, tmp_path, name, dtype):
    """--trace-layers: the residual stream at the wanted places after the embedding and after every layer, against the plain
    model's hidden states up to that layer; a prompt cut in portions with decoded tokens after it. --hashes: one line a step."""
    import plain_qwen3 as P
    from inference_bench_b200.trace import logit_hash
    cfg = CONFIGS[name]["config"]
    vocab, hidden, layers = cfg["vocab_size"], cfg["hidden_size"], cfg["num_hidden_layers"]
    toks = traces.prompt(77, 41, vocab)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:19], "want": [0, 7, 18]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[19:38], "want": list(range(19))}], "end": []}]
    steps += [{"step": 2 + i, "entries": [{"id": "a", "tokens": [toks[38 + i]], "want": [0]}], "end": ["a"] if i == 2 else []} for i in range(3)]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(model_dirs[name]), "--dtype", dtype, "--out", str(out),
                           "--max-tokens", "64", "--page-size", str(CONFIGS[name]["page_size"]), "--trace-layers", "--hashes"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    plain = PlainModel(model_dirs[name])
    want = [P.hidden_states(plain.w, plain.cfg, toks, upto_layers=k).numpy() for k in range(layers + 1)]      # [layers + 1][n, hidden]
    tol = {"float32": 1e-4, "bfloat16": 3e-2}[dtype]
    at = 0
    hashes = dict(line.split() for line in (out / "hashes.txt").read_text().splitlines())
    for s in steps:
        e = s["entries"][0]
        got = np.fromfile(out / f"{s['step']}.layers.f32", dtype="<f4").reshape(layers + 1, len(e["want"]), hidden)
        for k in range(layers + 1):
            for j, w in enumerate(e["want"]):
                ref = want[k][at + w]
                err = np.abs(got[k, j] - ref).max() / np.abs(want[k]).max()
                assert err <= tol, f"step {s['step']}: after {'the embedding' if k == 0 else f'layer {k - 1}'}, position {at + w}: {err:.3e}"
        at += len(e["tokens"])
        logits = np.fromfile(out / f"{s['step']}.f32", dtype="<f4")
        assert hashes[str(s["step"])] == f"{logit_hash(logits):016x}"
    assert logit_hash(np.asarray([1.0, -2.5], dtype="<f4")) == ((((0xcbf29ce484222325 ^ 0x3f800000) * 0x100000001b3) & (2**64 - 1)) ^ 0xc0200000) * 0x100000001b3 & (2**64 - 1)


def test_model_spec_runs_through_the_command_line(model_dirs, tmp_path):
    """A TOML model spec as --model: the folder it names, its [runtime] table, and --runtime laid over that."""
    env = dict(os.environ, PYTHONPATH=ROOT)
    spec = tmp_path / "tiny-b.toml"
    spec.write_text(f'name = "tiny-b"\nrepo = "{model_dirs["B"]}"\n[runtime]\ndtype = "float32"\npage_size = 8\nprefill_chunk = 5\ngraphs = false\n')
    prompt = [(1000 + i * 7 % 5000) % 384 for i in range(12)]
    want = PlainModel(model_dirs["B"]).greedy(prompt, 5)
    for extra in ([], ["--runtime", "graphs=true", "--runtime", "pipeline=false"]):
        p = subprocess.run([sys.executable, "-m", "inference_bench_b200", "run", "--model", str(spec), "--prompt-len", "12", "--max-tokens", "5", "--json",
                            "--max-ctx", "64", *extra], capture_output=True, text=True, env=env, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert json.loads(p.stdout)["tokens"] == want
    p = subprocess.run([sys.executable, "-m", "inference_bench_b200", "spec", "--model", str(spec), "--runtime", "pdl=false"], capture_output=True, text=True, env=env)
    shown = json.loads(p.stdout)
    assert p.returncode == 0 and shown["name"] == "tiny-b" and shown["runtime"]["page_size"] == 8 and shown["runtime"]["pdl"] is False
    assert shown["runtime"]["dtype"] == "float32" and shown["derived"]["layers"] == 3
    p = subprocess.run([sys.executable, "-m", "inference_bench_b200", "run", "--model", str(spec), "--runtime", "tile=big"], capture_output=True, text=True, env=env)
    assert p.returncode != 0 and "unknown option 'tile'" in p.stderr


def test_cli_logit_diff_and_batch(model_dirs, tmp_path):
    """logit-diff against a reference pair written from the plain model (NAME.ref.json + NAME.ref.bin, the layout of the
    reference's scripts: crates/core/src/logitdiff.rs:76-93): exit 0 within tolerance, 2 once one logit is moved. batch: one
    result per size with the reference's field names (crates/core/src/batch.rs:52-57)."""
    env = dict(os.environ, PYTHONPATH=ROOT)
    name = "A"
    vocab = CONFIGS[name]["config"]["vocab_size"]
    toks = traces.prompt(31, 37, vocab)
    ref = PlainModel(model_dirs[name]).logits(toks).numpy().astype("<f4")
    (tmp_path / "a.ref.json").write_text(json.dumps({"tokens": toks, "vocab": vocab}))
    ref.tofile(tmp_path / "a.ref.bin")
    cmd = [sys.executable, "-m", "inference_bench_b200", "logit-diff", "--model", str(model_dirs[name]), "--dtype", "float32", "--max-ctx", "64",
           "--reference", str(tmp_path / "a.ref.json")]
    p = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stdout + p.stderr[-2000:]
    rep = json.loads(p.stdout)
    assert rep["within_tolerance"] and rep["top1_agreement"] == 1.0 and rep["positions"] == 37 and rep["max_abs"] <= 1e-3
    ref[20, 5] += 0.5
    ref.tofile(tmp_path / "a.ref.bin")
    p = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 2 and not json.loads(p.stdout)["within_tolerance"]
    p = subprocess.run([sys.executable, "-m", "inference_bench_b200", "batch", "--model", str(model_dirs[name]), "--dtype", "bfloat16", "--max-ctx", "64",
                        "--prompt-len", "9", "--max-tokens", "6", "--sizes", "1,4", "--json"], capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    rows = json.loads(p.stdout)
    assert [r["batch"] for r in rows] == [1, 4] and [r["completion_tokens"] for r in rows] == [6, 24] and [r["prompt_tokens"] for r in rows] == [9, 36]
    assert all(r["decode_tok_s"] > 0 and r["throughput_tok_s"] > 0 and r["median_ttft_secs"] > 0 for r in rows)
