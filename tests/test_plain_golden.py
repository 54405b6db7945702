"""The plain implementation against the reference's own fixture and gate
(crates/cli/src/verify.rs:15-19: logits |ours - ref| <= 5e-4 + 1e-4 |ref|, layer norms 1e-4
relative, greedy token equal), teacher-forced as `marin-run verify` does (verify.rs:156-262)."""
import json
import os

import torch

import plain_qwen3 as plain

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "tiny-qwen3")


def test_plain_reproduces_reference_fixture():
    cfg = plain.read_config(GOLDEN)
    w = plain.read_weights(GOLDEN)
    ref = json.load(open(os.path.join(GOLDEN, "reference.json")))
    assert ref["math"] == "float32"
    worst = 0.0
    for case in ref["cases"]:
        ids = list(case["prompt_ids"])
        logits, states = plain.forward(cfg, w, ids, return_hidden=True)
        for n, want in enumerate(case["layer_norms"]):
            got = float(torch.linalg.vector_norm(states[n][-1]))
            assert abs(got - want) <= 1e-4 * abs(want), (n, got, want)
        for step in case["steps"]:
            row = plain.forward(cfg, w, ids)[-1]
            for tok, val in step["top"]:
                diff = abs(float(row[tok]) - val)
                worst = max(worst, diff)
                assert diff <= 5e-4 + 1e-4 * abs(val), (tok, float(row[tok]), val)
            assert int(torch.argmax(row)) == step["token"]
            ids.append(step["token"])
    assert worst < 5e-4


def test_plain_parts_by_hand():
    # RMSNorm of [3, 4] with unit weight: mean square 12.5 (crates/tensor/src/norm.rs tests)
    y = plain.rms_norm(torch.tensor([[3.0, 4.0]]), torch.ones(2), 0.0)
    assert torch.allclose(y, torch.tensor([[3.0, 4.0]]) / 12.5 ** 0.5)
    # rotation of [1, 0] at position 1 gives [cos 1, sin 1]; position 0 is the identity
    x = torch.tensor([[[1.0, 0.0]], [[1.0, 0.0]]])
    r = plain.rope(x, torch.tensor([0, 1]), 10000.0)
    assert torch.allclose(r[0, 0], torch.tensor([1.0, 0.0]))
    assert torch.allclose(r[1, 0], torch.tensor([0.5403023, 0.8414710]), atol=1e-6)
    s = plain.softmax(torch.tensor([1.0, 2.0, 3.0]))
    assert torch.allclose(s, torch.tensor([0.09003057, 0.24472847, 0.66524096]), atol=1e-7)
    # one key: attention returns its value whatever the score
    q = torch.randn(1, 2, 4)
    k, v = torch.randn(1, 1, 4), torch.randn(1, 1, 4)
    assert torch.allclose(plain.attention(q, k, v)[0, 1], v[0, 0])
