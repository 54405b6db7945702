"""bin/trace_run as a user runs it: a subprocess fed steps on standard input, logits read back from
files, compared with the plain implementation — whole, with the last 32 tokens one by one, in
portions of changing size, and mixed with so few pages that they are used again."""
import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import MATRIX_STD, CONFIGS, make_model_dir, mixed_schedule, portions, random_prompt
from test_engine_gpu import close, plain_forward

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def replay(model_dir, dtype, out_dir, max_tokens, steps, vocab):
    """steps: [(entries [(id, tokens, want)], ends)] → {step: logits [wanted, vocab]}"""
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
                             "--out", out_dir, "--max-tokens", str(max_tokens)],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    results = {}
    for i, (entries, ends) in enumerate(steps):
        line = {"step": i, "entries": [{"id": rid, "tokens": toks, "want": want} for rid, toks, want in entries], "end": ends}
        proc.stdin.write(json.dumps(line) + "\n")
        proc.stdin.flush()
        answer = proc.stdout.readline().strip()
        assert answer == f"done {i}", answer
        wanted = sum(len(w) for _, _, w in entries)
        path = os.path.join(out_dir, f"{i}.f32")
        if wanted:
            results[i] = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(wanted, vocab).copy())
        else:
            assert not os.path.exists(path)
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0
    return results


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_trace_replay_modes(tmp_path, name, dtype):
    raw = CONFIGS[name]
    vocab = raw["vocab_size"]
    d = make_model_dir(str(tmp_path / "model"), raw, seed=21, dtype=torch.float32 if dtype == "float32" else torch.bfloat16, matrix_std=MATRIX_STD[name])
    cfg, w = plain.read_config(d), plain.read_weights(d)
    rng = random.Random(2)
    cap = raw["max_position_embeddings"]
    lengths = {"a": 70, "b": min(cap, 130), "c": 41, "d": 64, "e": 100, "f": 2}
    tokens = {rid: random_prompt(rng, vocab, n) for rid, n in lengths.items()}
    want = {rid: plain_forward(cfg, w, t, dtype) for rid, t in tokens.items()}

    # alone and whole; then most in one step and the last 32 one by one; then changing portions
    steps, expect = [], []
    for rid in ("a", "b"):
        n = lengths[rid]
        steps.append(([(rid + "w", tokens[rid], list(range(n)))], [rid + "w"]))
        expect.append(want[rid])
        steps.append(([(rid + "t", tokens[rid][: n - 32], [n - 33])], []))
        expect.append(want[rid][n - 33:n - 32])
        for j in range(n - 32, n):
            steps.append(([(rid + "t", [tokens[rid][j]], [0])], [rid + "t"] if j == n - 1 else []))
            expect.append(want[rid][j:j + 1])
        at = 0
        sizes = portions(n, [7, 2, 13, 3, 2, 5])
        for k, m in enumerate(sizes):
            wanted = [0, m - 1] if m > 1 else [0]
            steps.append(([(rid + "p", tokens[rid][at:at + m], wanted)], [rid + "p"] if k == len(sizes) - 1 else []))
            expect.append(want[rid][[at + i for i in wanted]])
            at += m
    got = replay(d, dtype, str(tmp_path / "out1"), 192, steps, vocab)
    for i, e in enumerate(expect):
        close(got[i], e, dtype, f"step {i}")

    # mixed: up to four live, the pool sized for the four largest rounded up to 64
    sched = mixed_schedule(rng, lengths, max_live=4, decode_tail=5)
    pool = sum(sorted((-(-n // 64) * 64 for n in lengths.values()), reverse=True)[:4])
    fed = {rid: 0 for rid in tokens}
    steps, expect = [], []
    for entries, ends in sched:
        line = []
        rows = []
        for rid, n in entries:
            wanted = [n - 1] if n > 2 else list(range(n))
            line.append((rid, tokens[rid][fed[rid]:fed[rid] + n], wanted))
            rows.append(want[rid][[fed[rid] + i for i in wanted]])
            fed[rid] += n
        steps.append((line, ends))
        expect.append(torch.cat(rows))
    got = replay(d, dtype, str(tmp_path / "out2"), pool, steps, vocab)
    for i, e in enumerate(expect):
        close(got[i], e, dtype, f"mixed step {i}")
