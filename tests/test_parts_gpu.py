"""Each part alone against the plain implementation's function for it, and a toy mixer with state
of its own — defined here, registered here — built and stepped without a change to the package."""
import json
import math
import os
import random
from dataclasses import dataclass
from types import SimpleNamespace

import pytest
import torch

import plain_qwen3 as plain
from helpers import portions, random_prompt, run_mixed, run_portions, run_whole, mixed_schedule

pytestmark = pytest.mark.gpu
DEV = torch.device(os.environ.get("MARIN_B200_TEST_DEVICE", "cuda:0"))


def runtime(dtype=torch.float32):
    from marin_b200.parts import Runtime
    return Runtime(DEV, dtype)


def harness(mixer, rt, page=8, pages=32, ctx_len=256):
    """A cache and a step-context builder around one mixer (no model)."""
    from marin_b200.cache import CacheManager
    from marin_b200.engine import Runner

    cache = CacheManager([mixer.cache_need()], [None], page, pages, 4)
    cache.allocate(rt.device, rt.dtype)
    fake_model = SimpleNamespace(spec=SimpleNamespace(vocab_size=1 << 30))
    return Runner(fake_model, cache, rt, ctx_len)


def test_rmsnorm_part():
    from marin_b200.parts import lookup

    rt = runtime()
    norm = lookup("norm", "rmsnorm")(dim=72, eps=3e-6, name="n")
    assert [(s.name, s.shape, s.role) for s in norm.tensor_specs()] == [("n.weight", (72,), "norm")]
    w = 1 + 0.1 * torch.randn(72)
    norm.load({"n.weight": w.to(torch.bfloat16)}, rt)
    assert norm.weight.dtype == torch.float32
    x = torch.randn(9, 72)
    out = torch.empty(9, 72, device=DEV)
    norm.forward(x.to(DEV), out)
    torch.testing.assert_close(out.cpu(), plain.rms_norm(x, w.to(torch.bfloat16).float(), 3e-6), rtol=1e-5, atol=1e-6)


def test_rotary_part_through_the_fused_kernel():
    from marin_b200.kernels import ops
    from marin_b200.parts import lookup

    rt = runtime()
    H, K, d, T, page = 3, 1, 48, 11, 8
    pos = lookup("position", "rope")(head_dim=d, theta=5e5)
    pos.load({}, rt)
    i = torch.arange(d // 2, dtype=torch.float32)
    torch.testing.assert_close(pos.inv_freq.cpu(), torch.pow(torch.tensor(5e5), -(i * 2.0 / d)), rtol=1e-6, atol=0)
    qkv = torch.randn(T, (H + 2 * K) * d)
    positions = torch.tensor([0, 1, 2, 3, 100, 101, 1000, 2047, 4095, 17, 5], dtype=torch.int32)
    kc, vc = torch.zeros(4, K, page, d, device=DEV), torch.zeros(4, K, page, d, device=DEV)
    q_out = torch.empty(T, H * d, device=DEV)
    slots = torch.arange(T, dtype=torch.int32, device=DEV)
    ops.qk_norm_rope_write(qkv.to(DEV), q_out, None, None, 0.0, positions.to(DEV), pos.inv_freq, pos.rotary_dim,
                           pos.interleaved, slots, kc, vc, H, K, d, True)
    want_q = plain.rope(qkv[:, : H * d].view(T, H, d), positions, 5e5)
    torch.testing.assert_close(q_out.cpu().view(T, H, d), want_q, rtol=1e-4, atol=2e-4)
    want_k = plain.rope(qkv[:, H * d:(H + K) * d].view(T, K, d), positions, 5e5)
    got_k = torch.stack([kc[t // page, :, t % page] for t in range(T)]).cpu()
    torch.testing.assert_close(got_k, want_k, rtol=1e-4, atol=2e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_mixer_alone(dtype):
    from marin_b200.engine import StepEntry
    from marin_b200.parts import PartSpec, lookup

    rt = runtime(dtype)
    hidden, H, K, d = 72, 6, 3, 48
    mixer = lookup("mixer", "gqa_attention")(hidden=hidden, heads=H, kv_heads=K, head_dim=d, name="att", qk_norm=True,
                                             norm_eps=1e-5, position=PartSpec("rope", {"head_dim": d, "theta": 1e4}))
    g = torch.Generator().manual_seed(1)
    w = {s.name: (torch.randn(s.shape, generator=g) * (0.1 if s.role == "matrix" else 0.05) + (1.0 if s.role == "norm" else 0.0)).to(dtype)
         for s in mixer.tensor_specs()}
    wf = {k: v.float() for k, v in w.items()}
    mixer.load(dict(w), rt)
    runner = harness(mixer, rt)
    T = 29
    x = torch.randn(T, hidden, generator=g).to(dtype)
    runner.begin("r")
    got = []
    at = 0
    for n in (13, 1, 1, 14):     # a prompt portion, two single tokens, another portion: all from the cache
        runner.cache.reserve("r", at + n)
        ctx = runner.build_context([StepEntry("r", [0] * n, [])])
        residual = torch.zeros(n, hidden, device=DEV)
        mixer.forward(x[at:at + n].to(DEV), ctx, runner.views.view(0, ctx), residual)
        runner.cache.commit("r", at + n)
        got.append(residual.cpu())
        at += n
    got = torch.cat(got)
    xf = x.float()
    pos = torch.arange(T)
    q = plain.rope(plain.rms_norm(plain.linear(xf, wf["att.q_proj.weight"]).view(T, H, d), wf["att.q_norm.weight"], 1e-5), pos, 1e4)
    k = plain.rope(plain.rms_norm(plain.linear(xf, wf["att.k_proj.weight"]).view(T, K, d), wf["att.k_norm.weight"], 1e-5), pos, 1e4)
    v = plain.linear(xf, wf["att.v_proj.weight"]).view(T, K, d)
    want = plain.linear(plain.attention(q, k, v).reshape(T, H * d), wf["att.o_proj.weight"])
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=5e-2, atol=5e-2)
    torch.testing.assert_close(got, want, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part_alone(dtype):
    from marin_b200.engine.context import Workspace
    from marin_b200.parts import lookup

    rt = runtime(dtype)
    ffn = lookup("feedforward", "swiglu")(hidden=72, intermediate=136, name="mlp")
    g = torch.Generator().manual_seed(2)
    w = {s.name: (torch.randn(s.shape, generator=g) * 0.1).to(dtype) for s in ffn.tensor_specs()}
    ffn.load(dict(w), rt)
    x = torch.randn(7, 72, generator=g).to(dtype)
    base = torch.randn(7, 72, generator=g)
    residual = base.clone().to(DEV)
    ffn.forward(x.to(DEV), SimpleNamespace(workspace=Workspace(DEV)), residual)
    want = base + plain.swiglu_mlp(x.float(), w["mlp.gate_proj.weight"].float(), w["mlp.up_proj.weight"].float(), w["mlp.down_proj.weight"].float())
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(residual.cpu(), want, **tol)


# ---- a toy architecture whose first layer's mixer keeps a state of its own ---------------------------------

def define_toy():
    from marin_b200.config.base import ModelConfig
    from marin_b200.models import register_architecture
    from marin_b200.parts import (LayerSpec, Mixer, ModelSpec, PartSpec, ScheduleEntry, StateNeed, TensorSpec,
                                  register_mixer)

    @register_mixer("toy_decay")
    class DecayMixer(Mixer):
        """s_t = decay * s_{t-1} + W_in x_t ;  y_t = W_out s_t  — a state per request, no pages."""

        def __init__(self, hidden, decay, name):
            self.hidden, self.decay, self.name = hidden, decay, name

        def cache_need(self):
            return StateNeed((self.hidden,), torch.float32)

        def tensor_specs(self):
            return [TensorSpec(f"{self.name}.in_proj.weight", (self.hidden, self.hidden)),
                    TensorSpec(f"{self.name}.out_proj.weight", (self.hidden, self.hidden))]

        def load(self, tensors, rt):
            self.w_in = tensors.pop(f"{self.name}.in_proj.weight").to(rt.device, torch.float32)
            self.w_out = tensors.pop(f"{self.name}.out_proj.weight").to(rt.device, torch.float32)

        # single-token steps do the same work whatever the batch holds, all of it on the device and addressed through
        # ctx's device tensors: such steps may be captured in a graph (rows that pad a batch use the spare slot)
        capturable = True

        def forward(self, x, ctx, cache, residual):
            u = x.float() @ self.w_in.t()
            if ctx.num_decode == ctx.num_requests:
                slots = ctx.state_slots.long()
                s = self.decay * cache.state.index_select(0, slots) + u
                cache.state.index_copy_(0, slots, s)
                residual += s @ self.w_out.t()
                return
            y = torch.empty_like(u)
            for span in ctx.spans:
                s = cache.state[span.slot].clone()
                for j in range(span.start, span.start + span.count):
                    s = self.decay * s + u[j]
                    y[j] = s
                cache.state[span.slot] = s
            residual += y @ self.w_out.t()

    @dataclass
    class ToyConfig(ModelConfig):
        decay: float = 0.5
        heads: int = 2
        head_dim: int = 16
        intermediate: int = 48
        eps: float = 1e-6

        @classmethod
        def from_dict(cls, raw, generation=None):
            return cls(architecture="ToyStateLM", model_type="toy_state", vocab_size=raw["vocab_size"],
                       hidden_size=raw["hidden_size"], max_position_embeddings=raw["max_position_embeddings"], raw=dict(raw),
                       decay=raw["decay"], heads=raw["heads"], head_dim=raw["head_dim"], intermediate=raw["intermediate"])

        def to_json_dict(self):
            return {"architectures": ["ToyStateLM"], "model_type": "toy_state", "vocab_size": self.vocab_size,
                    "hidden_size": self.hidden_size, "max_position_embeddings": self.max_position_embeddings,
                    "decay": self.decay, "heads": self.heads, "head_dim": self.head_dim, "intermediate": self.intermediate}

    def build_spec(cfg):
        h = cfg.hidden_size
        norm = PartSpec("rmsnorm", {"dim": h, "eps": cfg.eps})
        ffn = PartSpec("swiglu", {"hidden": h, "intermediate": cfg.intermediate})
        names = {"norm1": "norm1", "mixer": "mixer", "norm2": "norm2", "feedforward": "mlp"}
        att = PartSpec("gqa_attention", {"hidden": h, "heads": cfg.heads, "kv_heads": 1, "head_dim": cfg.head_dim,
                                         "qk_norm": False, "position": PartSpec("rope", {"head_dim": cfg.head_dim, "theta": 100.0})})
        layers = [LayerSpec("prenorm", norm, PartSpec("toy_decay", {"hidden": h, "decay": cfg.decay}), ffn, "toy.layers.0", names),
                  LayerSpec("prenorm", norm, att, ffn, "toy.layers.1", names)]
        return ModelSpec(hidden_size=h, vocab_size=cfg.vocab_size,
                         embedding=PartSpec("token_table", {"vocab": cfg.vocab_size, "hidden": h, "name": "toy.embed"}),
                         final_norm=PartSpec("rmsnorm", {"dim": h, "eps": cfg.eps, "name": "toy.norm"}),
                         head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": h, "name": "toy.head"}),
                         layers=layers, schedule=[ScheduleEntry(0), ScheduleEntry(1)])

    register_architecture("ToyStateLM", "toy_state", ToyConfig, build_spec)
    return ToyConfig


def toy_plain(raw, w, ids):
    """The toy model on a whole sequence, from plain functions."""
    h, H, d = raw["hidden_size"], raw["heads"], raw["head_dim"]
    T = len(ids)
    x = plain.embed(ids, w["toy.embed.weight"])
    # layer 0: decay mixer
    n = plain.rms_norm(x, w["toy.layers.0.norm1.weight"], 1e-6)
    u = plain.linear(n, w["toy.layers.0.mixer.in_proj.weight"])
    s, ys = torch.zeros(h), []
    for t in range(T):
        s = raw["decay"] * s + u[t]
        ys.append(s)
    x = x + plain.linear(torch.stack(ys), w["toy.layers.0.mixer.out_proj.weight"])
    n = plain.rms_norm(x, w["toy.layers.0.norm2.weight"], 1e-6)
    x = x + plain.swiglu_mlp(n, w["toy.layers.0.mlp.gate_proj.weight"], w["toy.layers.0.mlp.up_proj.weight"], w["toy.layers.0.mlp.down_proj.weight"])
    # layer 1: attention without q/k norm, one kv head
    p = "toy.layers.1."
    n = plain.rms_norm(x, w[p + "norm1.weight"], 1e-6)
    pos = torch.arange(T)
    q = plain.rope(plain.linear(n, w[p + "mixer.q_proj.weight"]).view(T, H, d), pos, 100.0)
    k = plain.rope(plain.linear(n, w[p + "mixer.k_proj.weight"]).view(T, 1, d), pos, 100.0)
    v = plain.linear(n, w[p + "mixer.v_proj.weight"]).view(T, 1, d)
    x = x + plain.linear(plain.attention(q, k, v).reshape(T, H * d), w[p + "mixer.o_proj.weight"])
    n = plain.rms_norm(x, w[p + "norm2.weight"], 1e-6)
    x = x + plain.swiglu_mlp(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return plain.linear(plain.rms_norm(x, w["toy.norm.weight"], 1e-6), w["toy.head.weight"])


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    from marin_b200.cache import CacheManager
    from marin_b200.engine import Runner, load_model
    from marin_b200.weights import write_random_model

    ToyConfig = define_toy()
    raw = {"architectures": ["ToyStateLM"], "model_type": "toy_state", "vocab_size": 97, "hidden_size": 40,
           "max_position_embeddings": 96, "decay": 0.7, "heads": 2, "head_dim": 16, "intermediate": 48}
    d = write_random_model(str(tmp_path / "toy"), ToyConfig.from_dict(raw), seed=4, dtype=torch.float32, matrix_std=0.15)
    rt = runtime()
    config, model = load_model(d, rt)          # config.json chooses the toy architecture
    assert type(config).__name__ == "ToyConfig"
    cache = CacheManager(model.cache_needs(), [e.cache_of for e in model.spec.schedule], 8, 24, 4)
    cache.allocate(rt.device, rt.dtype)
    assert len(cache.groups) == 1 and list(cache.state) == [0]      # pages for layer 1, state slots for layer 0
    runner = Runner(model, cache, rt, 96)
    w = plain.read_weights(d)
    rng = random.Random(3)
    lengths = {"a": 40, "b": 7, "c": 61, "d": 25, "e": 33, "f": 12}
    tokens = {rid: random_prompt(rng, 97, n) for rid, n in lengths.items()}
    want = {rid: toy_plain(raw, w, t) for rid, t in tokens.items()}
    for rid in ("a", "c"):
        torch.testing.assert_close(run_whole(runner, rid, tokens[rid]).cpu(), want[rid], rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(run_portions(runner, rid, tokens[rid], portions(lengths[rid], [5, 1, 2, 11])).cpu(),
                                   want[rid], rtol=1e-4, atol=1e-4)
    got = run_mixed(runner, tokens, mixed_schedule(rng, lengths, max_live=4))     # state slots are used again too
    for rid in tokens:
        torch.testing.assert_close(got[rid].cpu(), want[rid], rtol=1e-4, atol=1e-4)
    cache.check()
    # the same from captured graphs: whether a hybrid model's single-token steps can be captured is its mixers' answer
    assert model.capturable()
    runner.enable_graphs((1, 2, 4))
    got = run_mixed(runner, tokens, mixed_schedule(random.Random(5), lengths, max_live=3, decode_tail=12))
    assert any(g["graph"] is not None for g in runner.graphs.values()) and {b for b, _ in runner.graphs} >= {1, 2, 4}
    for rid in tokens:
        torch.testing.assert_close(got[rid].cpu(), want[rid], rtol=1e-4, atol=1e-4)
    cache.check()
    # a mixer that says it cannot be captured turns graphs off for its model, and only for its model
    model.blocks[0].mixer.capturable = False
    try:
        plain_runner = Runner(model, cache, rt, 96)
        plain_runner.enable_graphs((1, 2, 4))
        assert not getattr(plain_runner, "graph_sizes", None)
    finally:
        del model.blocks[0].mixer.capturable


def test_block_embedding_and_head_parts_alone():
    """A whole pre-norm block, the embedding and the head, each built from the registries with its own parameters."""
    from marin_b200.engine import StepEntry
    from marin_b200.parts import LayerSpec, PartSpec, lookup

    rt = runtime()
    h, H, K, d, I, V = 72, 6, 3, 48, 136, 333
    spec = LayerSpec(block="prenorm", norm=PartSpec("rmsnorm", {"dim": h, "eps": 3e-6}),
                     mixer=PartSpec("gqa_attention", {"hidden": h, "heads": H, "kv_heads": K, "head_dim": d, "norm_eps": 3e-6,
                                                      "position": PartSpec("rope", {"head_dim": d, "theta": 5e5})}),
                     feedforward=PartSpec("swiglu", {"hidden": h, "intermediate": I}), prefix="model.layers.0",
                     names={"norm1": "input_layernorm", "mixer": "self_attn", "norm2": "post_attention_layernorm", "feedforward": "mlp"})
    block = lookup("block", "prenorm")(spec)
    g = torch.Generator().manual_seed(5)
    w = {s.name: torch.randn(s.shape, generator=g) * (0.1 if s.role != "norm" else 0.05) + (1.0 if s.role == "norm" else 0.0)
         for s in block.tensor_specs()}
    block.load({k: v.clone() for k, v in w.items()}, rt)
    runner = harness(block.mixer, rt, page=16, pages=8)
    T = 21
    x = torch.randn(T, h, generator=g)
    runner.begin("r")
    runner.cache.reserve("r", T)
    ctx = runner.build_context([StepEntry("r", [0] * T, [])])
    hidden = x.clone().to(DEV)
    block.forward(hidden, ctx, runner.views.view(0, ctx))
    cfg = {"heads": H, "kv_heads": K, "head_dim": d, "eps": 3e-6, "theta": 5e5}
    want, _ = plain.layer_forward(cfg, w, 0, x)
    torch.testing.assert_close(hidden.cpu(), want, rtol=1e-4, atol=1e-4)

    emb = lookup("embedding", "token_table")(vocab=V, hidden=h, name="model.embed_tokens")
    table = torch.randn(V, h, generator=g)
    emb.load({"model.embed_tokens.weight": table.clone()}, rt)
    ids = torch.tensor([0, 332, 7, 7], dtype=torch.int32)
    out = torch.empty(4, h, device=DEV)
    emb.forward(ids.to(DEV), out)
    assert torch.equal(out.cpu(), plain.embed(ids.tolist(), table))

    head = lookup("head", "linear")(vocab=V, hidden=h, name="lm_head", tied=True)
    assert head.tensor_specs() == []
    head.load({}, rt)
    head.tie(emb.table)
    logits = torch.empty(4, V, device=DEV)
    rows = torch.randn(4, h, generator=g)
    head.forward(rows.to(DEV), logits)
    torch.testing.assert_close(logits.cpu(), plain.linear(rows, table), rtol=1e-4, atol=1e-4)


def test_other_position_encodings_and_a_routed_feedforward_fit_the_interfaces(tmp_path):
    """Generality of the parts, shown with toys defined here: partial rotary with interleaved pairs (through the
    fused kernel's parameters), no position encoding at all, and a feed-forward that routes each token to one of
    two experts.  None of them is a model of anyone's; each is checked against plain torch written here."""
    from marin_b200.cache import CacheManager
    from marin_b200.config.base import ModelConfig
    from marin_b200.engine import Runner, load_model
    from marin_b200.models import register_architecture
    from marin_b200.parts import FeedForward, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSpec, register_feedforward
    from marin_b200.weights import write_random_model

    @register_feedforward("toy_top1")
    class Top1Experts(FeedForward):
        """y = W2[e] relu(W1[e] x) with e = argmax(router x): routing and experts are the part's own business."""

        def __init__(self, hidden, inner, experts, name):
            self.hidden, self.inner, self.experts, self.name = hidden, inner, experts, name

        def tensor_specs(self):
            n = self.name
            specs = [TensorSpec(f"{n}.router.weight", (self.experts, self.hidden))]
            for e in range(self.experts):
                specs.append(TensorSpec(f"{n}.experts.{e}.w1.weight", (self.inner, self.hidden)))
                specs.append(TensorSpec(f"{n}.experts.{e}.w2.weight", (self.hidden, self.inner)))
            return specs

        def load(self, tensors, rt):
            n = self.name
            self.router = tensors.pop(f"{n}.router.weight").to(rt.device, torch.float32)
            self.w1 = [tensors.pop(f"{n}.experts.{e}.w1.weight").to(rt.device, torch.float32) for e in range(self.experts)]
            self.w2 = [tensors.pop(f"{n}.experts.{e}.w2.weight").to(rt.device, torch.float32) for e in range(self.experts)]

        def forward(self, x, ctx, residual):
            xf = x.float()
            choice = torch.argmax(xf @ self.router.t(), dim=-1)
            for e in range(self.experts):
                rows = torch.nonzero(choice == e).flatten()
                if rows.numel():
                    residual[rows] += torch.relu(xf[rows] @ self.w1[e].t()) @ self.w2[e].t()

    @dataclass
    class Toy2Config(ModelConfig):
        @classmethod
        def from_dict(cls, raw, generation=None):
            return cls(architecture="ToyRoutedLM", model_type="toy_routed", vocab_size=raw["vocab_size"], hidden_size=raw["hidden_size"],
                       max_position_embeddings=raw["max_position_embeddings"], raw=dict(raw))

        def to_json_dict(self):
            return dict(self.raw)

    def build_spec(cfg):
        h = cfg.hidden_size
        norm = PartSpec("rmsnorm", {"dim": h, "eps": 1e-6})
        names = {"norm1": "n1", "mixer": "att", "norm2": "n2", "feedforward": "ff"}

        def att(position):
            return PartSpec("gqa_attention", {"hidden": h, "heads": 2, "kv_heads": 2, "head_dim": 32, "qk_norm": False, "position": position})
        layers = [
            LayerSpec("prenorm", norm, att(PartSpec("rope", {"head_dim": 32, "theta": 50.0, "rotary_dim": 16, "interleaved": True})),
                      PartSpec("toy_top1", {"hidden": h, "inner": 24, "experts": 2}), "t.l0", names),
            LayerSpec("prenorm", norm, att(PartSpec("none", {})), PartSpec("swiglu", {"hidden": h, "intermediate": 48}), "t.l1", names),
        ]
        return ModelSpec(hidden_size=h, vocab_size=cfg.vocab_size,
                         embedding=PartSpec("token_table", {"vocab": cfg.vocab_size, "hidden": h, "name": "t.embed"}),
                         final_norm=PartSpec("rmsnorm", {"dim": h, "eps": 1e-6, "name": "t.norm"}),
                         head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": h, "name": "t.head"}),
                         layers=layers, schedule=[ScheduleEntry(0), ScheduleEntry(1)])

    register_architecture("ToyRoutedLM", "toy_routed", Toy2Config, build_spec)
    raw = {"architectures": ["ToyRoutedLM"], "model_type": "toy_routed", "vocab_size": 61, "hidden_size": 64, "max_position_embeddings": 80}
    d = write_random_model(str(tmp_path / "toy2"), Toy2Config.from_dict(raw), seed=9, dtype=torch.float32, matrix_std=0.2)
    rt = runtime()
    config, model = load_model(d, rt)
    cache = CacheManager(model.cache_needs(), [e.cache_of for e in model.spec.schedule], 8, 20, 4)
    cache.allocate(rt.device, rt.dtype)
    runner = Runner(model, cache, rt, 80)
    w = plain.read_weights(d)

    def toy2_plain(ids):
        T = len(ids)
        x = plain.embed(ids, w["t.embed.weight"])
        pos = torch.arange(T)
        for li in (0, 1):
            p = f"t.l{li}."
            n = plain.rms_norm(x, w[p + "n1.weight"], 1e-6)
            q = plain.linear(n, w[p + "att.q_proj.weight"]).view(T, 2, 32)
            k = plain.linear(n, w[p + "att.k_proj.weight"]).view(T, 2, 32)
            v = plain.linear(n, w[p + "att.v_proj.weight"]).view(T, 2, 32)
            if li == 0:      # partial rotary over the first 16 dims, pairs (2i, 2i+1)
                ang = pos.float()[:, None] * torch.pow(torch.tensor(50.0), -(torch.arange(8, dtype=torch.float32) * 2.0 / 16))[None, :]
                cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
                for t_ in (q, k):
                    a, b = t_[..., 0:16:2].clone(), t_[..., 1:16:2].clone()
                    t_[..., 0:16:2] = a * cos - b * sin
                    t_[..., 1:16:2] = b * cos + a * sin
            x = x + plain.linear(plain.attention(q, k, v).reshape(T, 64), w[p + "att.o_proj.weight"])
            n = plain.rms_norm(x, w[p + "n2.weight"], 1e-6)
            if li == 0:
                choice = torch.argmax(n @ w[p + "ff.router.weight"].t(), dim=-1)
                y = torch.zeros_like(x)
                for e in range(2):
                    rows = torch.nonzero(choice == e).flatten()
                    y[rows] = torch.relu(n[rows] @ w[p + f"ff.experts.{e}.w1.weight"].t()) @ w[p + f"ff.experts.{e}.w2.weight"].t()
                x = x + y
            else:
                x = x + plain.swiglu_mlp(n, w[p + "ff.gate_proj.weight"], w[p + "ff.up_proj.weight"], w[p + "ff.down_proj.weight"])
        return plain.linear(plain.rms_norm(x, w["t.norm.weight"], 1e-6), w["t.head.weight"])

    rng = random.Random(2)
    toks = random_prompt(rng, 61, 70)
    want = toy2_plain(toks)
    torch.testing.assert_close(run_whole(runner, "w", toks).cpu(), want, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(run_portions(runner, "p", toks, portions(70, [9, 1, 2, 17])).cpu(), want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_attention_layouts_in_one_model_decode_from_graphs(tmp_path, dtype):
    """A toy model whose two layers attend with different head counts, kv-head counts and head sizes: two cache groups,
    and for captured single-token steps one decode plan per layout (its own split of the keys, its own scratch and
    counters), asked of the mixers.  Several requests decode together from graphs against plain torch written here."""
    from marin_b200.cache import CacheManager
    from marin_b200.config.base import ModelConfig
    from marin_b200.engine import Runner, load_model
    from marin_b200.models import register_architecture
    from marin_b200.parts import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from marin_b200.weights import write_random_model

    layouts = [(8, 4, 64), (2, 1, 128)]            # (heads, kv heads, head size) of layer 0 and layer 1

    @dataclass
    class Toy3Config(ModelConfig):
        @classmethod
        def from_dict(cls, raw, generation=None):
            return cls(architecture="ToyTwoLayoutsLM", model_type="toy_two_layouts", vocab_size=raw["vocab_size"],
                       hidden_size=raw["hidden_size"], max_position_embeddings=raw["max_position_embeddings"], raw=dict(raw))

        def to_json_dict(self):
            return dict(self.raw)

    def build_spec(cfg):
        h = cfg.hidden_size
        norm = PartSpec("rmsnorm", {"dim": h, "eps": 1e-6})
        names = {"norm1": "n1", "mixer": "att", "norm2": "n2", "feedforward": "ff"}
        layers = [LayerSpec("prenorm", norm,
                            PartSpec("gqa_attention", {"hidden": h, "heads": H, "kv_heads": K, "head_dim": d, "qk_norm": True, "norm_eps": 1e-6,
                                                       "position": PartSpec("rope", {"head_dim": d, "theta": 1e4})}),
                            PartSpec("swiglu", {"hidden": h, "intermediate": 384}), f"t.l{i}", names)
                  for i, (H, K, d) in enumerate(layouts)]
        return ModelSpec(hidden_size=h, vocab_size=cfg.vocab_size,
                         embedding=PartSpec("token_table", {"vocab": cfg.vocab_size, "hidden": h, "name": "t.embed"}),
                         final_norm=PartSpec("rmsnorm", {"dim": h, "eps": 1e-6, "name": "t.norm"}),
                         head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": h, "name": "t.head"}),
                         layers=layers, schedule=[ScheduleEntry(0), ScheduleEntry(1)])

    register_architecture("ToyTwoLayoutsLM", "toy_two_layouts", Toy3Config, build_spec)
    raw = {"architectures": ["ToyTwoLayoutsLM"], "model_type": "toy_two_layouts", "vocab_size": 211, "hidden_size": 256,
           "max_position_embeddings": 512}
    d = write_random_model(str(tmp_path / "toy3"), Toy3Config.from_dict(raw), seed=3, dtype=dtype, matrix_std=0.06)
    rt = runtime(dtype)
    config, model = load_model(d, rt)
    cache = CacheManager(model.cache_needs(), [e.cache_of for e in model.spec.schedule], 16, 80, 4)
    cache.allocate(rt.device, rt.dtype)
    assert len(cache.groups) == 2
    runner = Runner(model, cache, rt, 512)
    runner.GRAPH_MIN_SPAN = 64
    runner.enable_graphs((1, 2, 4))
    w = plain.read_weights(d)

    def twin(ids):
        T = len(ids)
        x = plain.embed(ids, w["t.embed.weight"])
        pos = torch.arange(T)
        for i, (H, K, hd) in enumerate(layouts):
            p = f"t.l{i}."
            n = plain.rms_norm(x, w[p + "n1.weight"], 1e-6)
            q = plain.rope(plain.rms_norm(plain.linear(n, w[p + "att.q_proj.weight"]).view(T, H, hd), w[p + "att.q_norm.weight"], 1e-6), pos, 1e4)
            k = plain.rope(plain.rms_norm(plain.linear(n, w[p + "att.k_proj.weight"]).view(T, K, hd), w[p + "att.k_norm.weight"], 1e-6), pos, 1e4)
            v = plain.linear(n, w[p + "att.v_proj.weight"]).view(T, K, hd)
            x = x + plain.linear(plain.attention(q, k, v).reshape(T, H * hd), w[p + "att.o_proj.weight"])
            n = plain.rms_norm(x, w[p + "n2.weight"], 1e-6)
            x = x + plain.swiglu_mlp(n, w[p + "ff.gate_proj.weight"], w[p + "ff.up_proj.weight"], w[p + "ff.down_proj.weight"])
        return plain.linear(plain.rms_norm(x, w["t.norm.weight"], 1e-6), w["t.head.weight"])

    rng = random.Random(6)
    lengths = {"a": 300, "b": 90, "c": 170, "d": 41}
    tokens = {rid: random_prompt(rng, 211, n) for rid, n in lengths.items()}
    # short prompts, then long decoding side by side: the sequences grow through several spans, each with its own graphs
    steps = mixed_schedule(rng, lengths, max_live=4, decode_tail=150, sizes=(23, 2, 9))
    got = run_mixed(runner, tokens, steps)
    keys = {key for g in runner.graphs.values() for key in g["plans"]}
    if dtype == torch.bfloat16:
        assert len(keys) == 2, keys                  # one plan per layout, each with counters for its own kv heads
        for g in runner.graphs.values():
            bucket = g["key"][0]
            for (_, H, K, hd), plan in g["plans"].items():
                assert plan.buffers[2].numel() == bucket * K and plan.buffers[0].numel() == bucket * H * plan.chunks * hd
    assert len({span for _, span in runner.graphs}) >= 2
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=0.0, atol=0.08)
    for rid in tokens:
        torch.testing.assert_close(got[rid].cpu().float(), twin(tokens[rid]), **tol)
    cache.check()
    runner.scratch.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_that_keep_a_window_of_keys_beside_layers_that_keep_all(tmp_path, dtype):
    """A toy model of three attention layers: one keeps all keys, two keep a window (24 and 40 positions, one of them
    with other head sizes).  Three cache groups with pools of their own; a windowed group gives a page back as soon as
    the window has passed it, so its pool can be far smaller than the sequences are long, and the pages come round
    again within one request.  Whole, in portions, decoded from graphs and mixed with other requests, against the
    plain implementation's layer function with each layer's own window."""
    from test_engine_gpu import close

    from marin_b200.cache import CacheManager
    from marin_b200.config.base import ModelConfig
    from marin_b200.engine import Runner, StepEntry, load_model, parse_dtype
    from marin_b200.models import register_architecture
    from marin_b200.parts import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from marin_b200.weights import write_random_model

    layers = [(4, 2, 32, None), (4, 2, 32, 24), (2, 1, 64, 40)]          # (heads, kv heads, head size, window)

    @dataclass
    class Toy4Config(ModelConfig):
        @classmethod
        def from_dict(cls, raw, generation=None):
            return cls(architecture="ToyWindowLM", model_type="toy_window", vocab_size=raw["vocab_size"], hidden_size=raw["hidden_size"],
                       max_position_embeddings=raw["max_position_embeddings"], raw=dict(raw))

        def to_json_dict(self):
            return dict(self.raw)

    def build_spec(cfg):
        h = cfg.hidden_size
        norm = PartSpec("rmsnorm", {"dim": h, "eps": 1e-6})
        names = {"norm1": "input_layernorm", "mixer": "self_attn", "norm2": "post_attention_layernorm", "feedforward": "mlp"}
        specs = [LayerSpec("prenorm", norm,
                           PartSpec("gqa_attention", {"hidden": h, "heads": H, "kv_heads": K, "head_dim": d, "qk_norm": True, "norm_eps": 1e-6,
                                                      "window": w, "position": PartSpec("rope", {"head_dim": d, "theta": 1e4})}),
                           PartSpec("swiglu", {"hidden": h, "intermediate": 160}), f"model.layers.{i}", names)
                 for i, (H, K, d, w) in enumerate(layers)]
        return ModelSpec(hidden_size=h, vocab_size=cfg.vocab_size,
                         embedding=PartSpec("token_table", {"vocab": cfg.vocab_size, "hidden": h, "name": "model.embed_tokens"}),
                         final_norm=PartSpec("rmsnorm", {"dim": h, "eps": 1e-6, "name": "model.norm"}),
                         head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": h, "name": "lm_head"}),
                         layers=specs, schedule=[ScheduleEntry(i) for i in range(len(layers))])

    register_architecture("ToyWindowLM", "toy_window", Toy4Config, build_spec)
    raw = {"architectures": ["ToyWindowLM"], "model_type": "toy_window", "vocab_size": 173, "hidden_size": 128, "max_position_embeddings": 400}
    d = write_random_model(str(tmp_path / "toy4"), Toy4Config.from_dict(raw), seed=8, dtype=parse_dtype(dtype), matrix_std=0.09)
    rt = runtime(parse_dtype(dtype))
    config, model = load_model(d, rt)
    w = plain.read_weights(d)
    stored = plain.as_bf16 if dtype == "bfloat16" else plain.same

    def twin(ids):
        x = plain.embed(ids, w["model.embed_tokens.weight"])
        for i, (H, K, hd, window) in enumerate(layers):
            cfg = {"heads": H, "kv_heads": K, "head_dim": hd, "eps": 1e-6, "theta": 1e4}
            x, _ = plain.layer_forward(cfg, w, i, x, window=window, stored=stored)
        return plain.linear(stored(plain.rms_norm(x, w["model.norm.weight"], 1e-6)), w["lm_head.weight"])

    page = 8
    # every group gets the same number of pages: enough for three requests side by side where all keys are kept; the
    # windowed groups prove below that they live on a handful of them
    cache = CacheManager(model.cache_needs(), [e.cache_of for e in model.spec.schedule], page, 96, 4)
    cache.allocate(rt.device, rt.dtype)
    assert [g.need.window for g in cache.groups] == [None, 24, 40]
    runner = Runner(model, cache, rt, 400)
    runner.GRAPH_MIN_SPAN = 64
    runner.enable_graphs((1, 2, 4))
    rng = random.Random(12)
    lengths = {"a": 370, "b": 30, "c": 121, "d": 64, "e": 200}
    tokens = {rid: random_prompt(rng, 173, n) for rid, n in lengths.items()}
    want = {rid: twin(t) for rid, t in tokens.items()}
    close(run_whole(runner, "w", tokens["a"]), want["a"], dtype, "whole")
    close(run_portions(runner, "p", tokens["a"], portions(370, [23, 2, 57, 9, 1, 1, 1, 30])), want["a"], dtype, "portions")
    # a long decode: the windowed groups never hold more than the window's pages (+1 for the page being filled, +1 for alignment)
    runner.begin("long")
    runner.step([StepEntry("long", tokens["a"][:10], [])])
    most = [0, 0, 0]
    rows = []
    for t in range(10, 370):
        rows.append(runner.step([StepEntry("long", [tokens["a"][t]], [0])]).clone())
        for g, group in enumerate(cache.groups):
            most[g] = max(most[g], group.pool.num_held)
    close(torch.cat(rows), want["a"][10:], dtype, "decoded one by one")
    assert most[0] == -(-370 // page) and most[1] <= 24 // page + 2 and most[2] <= 40 // page + 2, most
    runner.end("long")
    got = run_mixed(runner, tokens, mixed_schedule(rng, lengths, max_live=3, decode_tail=40, sizes=(31, 2, 70, 5)))
    for rid in tokens:
        close(got[rid], want[rid], dtype, f"mixed {rid}")
    cache.check()
    assert all(g.pool.num_held == 0 for g in cache.groups)
    runner.scratch.check()
