"""The command line on the GPU: verify against the reference's own fixture, generate, random-weights mode."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden", "tiny-qwen3")
RUN = [sys.executable, os.path.join(ROOT, "bin", "marin-run")]


def test_verify_against_the_reference_fixture_in_float32():
    """The reference's tiny Qwen3 and reference.json (float32 logits of the reference's oracle), under the
    reference's own gate: the engine's float32 path must pass; a tampered reference must be caught
    (crates/cli/src/verify_tests.rs:12-50,66-116)."""
    from marin_b200.cli import verify

    assert verify(GOLDEN, os.path.join(GOLDEN, "reference.json"), "float32") == []


def test_verify_catches_a_tampered_reference(tmp_path):
    from marin_b200.cli import verify

    ref = json.load(open(os.path.join(GOLDEN, "reference.json")))
    ref["cases"][1]["steps"][2]["top"][0][1] += 0.01
    ref["cases"][0]["layer_norms"][1] *= 1.001
    bad = tmp_path / "bad.json"
    bad.write_text(json.dumps(ref))
    problems = verify(GOLDEN, str(bad), "float32")
    assert len(problems) == 2 and "norm" in problems[0] and "logit" in problems[1]


def test_run_random_and_bench_commands(tmp_path):
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps({"model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
                               "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128, "vocab_size": 256,
                               "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
                               "max_position_embeddings": 128}))
    model = str(tmp_path / "model")
    out = subprocess.run(RUN + ["random", "--config", str(cfg), "--seed", "3", "--out", model], capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    assert sorted(os.listdir(model)) == ["config.json", "model.safetensors"]
    a = subprocess.run(RUN + [model, "--prompt-ids", "5,6,7", "--temp", "0", "--max-tokens", "6", "--metrics"], capture_output=True, text=True)
    b = subprocess.run(RUN + [model, "--prompt-ids", "5 6 7", "--temp", "0", "--max-tokens", "6"], capture_output=True, text=True)
    assert a.returncode == 0 and b.returncode == 0, a.stderr + b.stderr
    assert a.stdout == b.stdout and len(a.stdout.split()) == 6          # greedy is deterministic; ids on stdout only
    assert "tok/s" in a.stderr
    c = subprocess.run(RUN + [model, "--prompt-ids", "5,6,7", "--temp", "0.9", "--seed", "1", "--max-tokens", "6"], capture_output=True, text=True)
    d = subprocess.run(RUN + [model, "--prompt-ids", "5,6,7", "--temp", "0.9", "--seed", "1", "--max-tokens", "6"], capture_output=True, text=True)
    assert c.stdout == d.stdout
    j = str(tmp_path / "bench.json")
    e = subprocess.run(RUN + ["bench", model, "--prompt-tokens", "16", "--tokens", "8", "--runs", "2", "--warmup", "1", "--json", j,
                              "--profile"], capture_output=True, text=True)
    assert e.returncode == 0, e.stderr
    # --profile: the stages of the prompt step and of a decode step, each with its time inside the step
    assert "prompt of 16 tokens in one step" in e.stdout and "decode step, one sequence" in e.stdout
    for stage in ("embedding", "q|k|v", "attention", "gate|up", "down", "head", "sampling", "(between steps)"):
        assert stage in e.stdout, stage
    rec = json.load(open(j))
    assert rec["prompt_tokens"] == 16 and rec["decode_tokens_per_s"] > 0 and rec["batch_size"] == 1
    f = subprocess.run(RUN + [model, "--max-tokens", "6"], capture_output=True, text=True)
    assert f.returncode != 0 and "prompt" in f.stderr


def test_the_measuring_aids_run(tmp_path):
    """``python -m marin_b200.kernels.probe`` (the many-token product built with -DTC_PROBE: where its producer and its MMA
    thread wait) prints its table, and ``kernels.trace.Marks`` hands its pinned buffer to the loaded libraries: none of
    the normal build takes it, so no mark is left."""
    import torch

    out = subprocess.run([sys.executable, "-m", "marin_b200.kernels.probe", "--tokens", "512", "--rows", "1024", "--width", "512", "--tile", "256"],
                         capture_output=True, text=True, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = out.stdout.strip().splitlines()
    assert "TFLOP/s" in lines[0] and lines[1].startswith("CTA")
    first = lines[2].split()
    assert int(first[0]) == 0 and int(first[1]) > 0 and all(float(v) >= 0 for v in first[2:])
    assert float(first[-1]) > 0                                 # the MMA thread's loop took some cycles per k-block

    from marin_b200.kernels import ops, trace

    x = torch.zeros(4, 64, device="cuda:0", dtype=torch.bfloat16)
    w = torch.zeros(128, 64, device="cuda:0", dtype=torch.bfloat16)
    ops.gemm(x, w, torch.empty(4, 128, device="cuda:0"))        # a library is loaded
    marks = trace.Marks()
    assert marks.arm() == 0 and marks.count() == 0 and marks.last() == []
