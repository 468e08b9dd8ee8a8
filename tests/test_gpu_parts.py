"""Each part alone against the plain implementation's function for it, and a model made
of other parts: a toy mixer with state of its own, defined here, registered, built from a
config.json and stepped without touching the package's files; its layers differ in their
mixer, its schedule names a layer several times and lets one run read another's cache.  A
second toy model has a feed-forward with routing and positions learned as a table that is
added to the embeddings."""

from __future__ import annotations

import json
import os

import numpy as np
import pytest

import plain_llama
from conftest import TINY_B, round_bf16, seeded_tokens

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def f64(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def runtime(dtype):
    from borrowed_compute_b200.parts import Runtime

    return Runtime(torch.device("cuda:0"), dtype, max_positions=512)


def context(entries, starts):
    """A StepContext on the device for parts run outside an engine."""
    from borrowed_compute_b200.engine.batch import plan_step
    from borrowed_compute_b200.parts import StepContext

    p = plan_step(entries, starts)
    return StepContext(rows=p.rows, seqs=p.seqs, tokens=dev(p.tokens), row_pos=dev(p.row_pos), row_slot=dev(p.row_slot),
                       seq_rows=dev(p.seq_rows), seq_slot=dev(p.seq_slot), seq_start=dev(p.seq_start), max_new=p.max_new,
                       max_total=p.max_total, decode=p.decode, host_seq_rows=tuple(int(x) for x in p.seq_rows),
                       host_seq_slot=tuple(int(x) for x in p.seq_slot), host_seq_start=tuple(int(x) for x in p.seq_start))


DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, ref):
    return (2e-5 if dtype == torch.float32 else 2.0 ** -6) * (1 + np.abs(ref).max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    from borrowed_compute_b200.parts import NORMS

    norm = NORMS.get("rmsnorm")(size=72, eps=1e-6)
    assert norm.tensors()["weight"].shape == (72,)
    w = (1 + 0.2 * np.random.default_rng(0).standard_normal(72)).astype(np.float32)
    norm.load({"weight": dev(w)}, runtime(dtype))
    x = np.random.default_rng(1).standard_normal((9, 72)).astype(np.float32)
    out = torch.empty((9, 72), dtype=dtype, device="cuda")
    norm.forward(dev(x), out)
    ref = plain_llama.rms_norm(x.astype(np.float64), w.astype(np.float64), 1e-6)
    assert np.abs(f64(out) - ref).max() <= tol(dtype, ref)


def test_rotary_part_tables():
    from borrowed_compute_b200.parts import POSITION_ENCODINGS

    scaling = TINY_B["rope_scaling"]
    enc = POSITION_ENCODINGS.get("rotary")(head_dim=32, theta=500000.0, pairing="adjacent", scaling=scaling, max_positions=256)
    enc.load({}, runtime(torch.float32))
    table = enc.rotary()
    inv = plain_llama.rope_inv_freq(32, 500000.0, scaling)
    assert table.pairing == 1 and tuple(table.cos_sin.shape) == (256, 16, 2)
    for pos in (0, 1, 63, 64, 65, 255):     # past the original 64 positions the scaled frequencies matter
        ang = (np.float32(pos) * inv).astype(np.float64)
        got = f64(table.cos_sin[pos])
        assert np.abs(got[:, 0] - np.cos(ang)).max() <= 6e-8 and np.abs(got[:, 1] - np.sin(ang)).max() <= 6e-8
    assert POSITION_ENCODINGS.get("none")().rotary() is None


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part(dtype):
    from borrowed_compute_b200.parts import FEED_FORWARDS

    r = np.random.default_rng(2)
    ff = FEED_FORWARDS.get("swiglu")(hidden_size=40, intermediate_size=88)
    w = {k: (r.standard_normal(s.shape) * 0.2).astype(np.float32) for k, s in ff.tensors().items()}
    ff.load({k: dev(v, dtype) for k, v in w.items()}, runtime(dtype))
    x = r.standard_normal((11, 40)).astype(np.float32)
    base = r.standard_normal((11, 40)).astype(np.float32)
    residual = dev(base)
    ff.forward(dev(x, dtype), residual, None)
    ws = {k: f64(dev(v, dtype)) for k, v in w.items()}
    ref = base + plain_llama.swiglu(f64(dev(x, dtype)), ws["gate_proj.weight"], ws["up_proj.weight"], ws["down_proj.weight"])
    assert np.abs(f64(residual) - ref).max() <= tol(dtype, ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tied", [False, True])
def test_embedding_and_head_parts(dtype, tied):
    from borrowed_compute_b200.parts import EMBEDDINGS, HEADS

    r = np.random.default_rng(3)
    emb = EMBEDDINGS.get("token_embedding")(vocab_size=50, hidden_size=24)
    head = HEADS.get("linear_head")(vocab_size=50, hidden_size=24, tied=tied)
    table, hw = r.standard_normal((50, 24)).astype(np.float32), r.standard_normal((50, 24)).astype(np.float32)
    emb.load({"weight": dev(table, dtype)}, runtime(dtype))
    head.load({} if tied else {"weight": dev(hw, dtype)}, runtime(dtype))
    ctx = context([__import__("borrowed_compute_b200").StepEntry(0, [3, 49, 0])], [0])
    residual = torch.empty((3, 24), dtype=torch.float32, device="cuda")
    emb.forward(ctx, residual)
    assert np.array_equal(f64(residual), f64(dev(table, dtype))[[3, 49, 0]])
    x = r.standard_normal((3, 24)).astype(np.float32)
    scores = torch.empty((3, 50), dtype=torch.float32, device="cuda")
    head.forward(dev(x, dtype), scores, emb.table())
    ref = f64(dev(x, dtype)) @ f64(dev(table if tied else hw, dtype)).T
    assert np.abs(f64(scores) - ref).max() <= 2e-5 * (1 + np.abs(ref).max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_part_alone(dtype):
    """The mixer with a cache of its own: two sequences' prompts in one step, then a token
    each, against the plain attention of the same projections."""
    from borrowed_compute_b200 import StepEntry
    from borrowed_compute_b200.cache import PagedCache
    from borrowed_compute_b200.parts import MIXERS

    r = np.random.default_rng(4)
    H, G, D, E = 6, 2, 16, 40
    att = MIXERS.get("gqa_attention")(hidden_size=E, heads=H, kv_heads=G, head_dim=D,
                                      position={"kind": "rotary", "head_dim": D, "theta": 10000.0, "pairing": "half", "max_positions": 512})
    w = {k: (r.standard_normal(s.shape) * 0.3).astype(np.float32) for k, s in att.tensors().items()}
    rt = runtime(dtype)
    att.load({k: dev(v, dtype) for k, v in w.items()}, rt)
    cache = PagedCache(rt, [att.cache_need()], [att.state_need()], [None], max_tokens=512, n_slots=3, max_seq=256)
    ws = {k: f64(dev(v, dtype)) for k, v in w.items()}
    inv = plain_llama.rope_inv_freq(D, 10000.0, None)
    xs = {0: r.standard_normal((70, E)).astype(np.float32), 1: r.standard_normal((5, E)).astype(np.float32)}

    def reference(x):
        n = x.shape[0]
        x = f64(dev(x, dtype))
        q = plain_llama.rope((x @ ws["q_proj.weight"].T).reshape(n, H, D), range(n), inv, "half")
        k = plain_llama.rope((x @ ws["k_proj.weight"].T).reshape(n, G, D), range(n), inv, "half")
        v = (x @ ws["v_proj.weight"].T).reshape(n, G, D)
        return plain_llama.attention(q, k, v).reshape(n, H * D) @ ws["o_proj.weight"].T

    slots = {0: cache.acquire(), 1: cache.acquire()}
    got = {0: [], 1: []}
    # all but the last token of each in one step, then the last token of each in one step
    for part in (lambda x: x[:-1], lambda x: x[-1:]):
        entries = [StepEntry(slots[i], [0] * len(part(xs[i]))) for i in (0, 1)]
        starts = [cache.slots.length(slots[i]) for i in (0, 1)]
        for e, s in zip(entries, starts):
            cache.slots.reserve(e.slot, s + len(e.tokens), rows=len(e.tokens))
        cache.sync_tables()
        ctx = context(entries, starts)
        x = np.concatenate([part(xs[0]), part(xs[1])])
        residual = torch.zeros((x.shape[0], E), dtype=torch.float32, device="cuda")
        att.forward(dev(x, dtype), residual, ctx, cache.memory(0))
        for e, s in zip(entries, starts):
            cache.slots.commit(e.slot, s + len(e.tokens))
        out = f64(residual)
        n0 = len(part(xs[0]))
        got[0].append(out[:n0]), got[1].append(out[n0:])
    for i in (0, 1):
        ref = reference(xs[i])
        assert np.abs(np.concatenate(got[i]) - ref).max() <= tol(dtype, ref) * 2


@pytest.mark.parametrize("dtype", DTYPES)
def test_windowed_attention_keeps_only_its_window(dtype):
    """A mixer that reads only the last 70 positions gets a storage group of its own whose
    pages behind the window go back to the pool; what it computes is attention over exactly
    those positions, through a prompt, across page edges, and long after pages were dropped."""
    from borrowed_compute_b200 import StepEntry
    from borrowed_compute_b200.cache import PagedCache
    from borrowed_compute_b200.parts import MIXERS

    r = np.random.default_rng(5)
    H, G, D, E, window, n = 4, 2, 16, 32, 70, 330
    position = {"kind": "rotary", "head_dim": D, "theta": 10000.0, "pairing": "half", "max_positions": 512}
    full = MIXERS.get("gqa_attention")(hidden_size=E, heads=H, kv_heads=G, head_dim=D, position=position)
    windowed = MIXERS.get("gqa_attention")(hidden_size=E, heads=H, kv_heads=G, head_dim=D, position=position, window=window)
    w = {k: (r.standard_normal(s.shape) * 0.4).astype(np.float32) for k, s in full.tensors().items()}
    rt = runtime(dtype)
    for m in (full, windowed):
        m.load({k: dev(v, dtype) for k, v in w.items()}, rt)
    cache = PagedCache(rt, [full.cache_need(), windowed.cache_need()], [None, None], [None, None], max_tokens=512, n_slots=2, max_seq=512)
    assert len(cache.groups) == 2, "different needs, different storage"
    ws = {k: f64(dev(v, dtype)) for k, v in w.items()}
    inv = plain_llama.rope_inv_freq(D, 10000.0, None)
    x = r.standard_normal((n, E)).astype(np.float32)
    xs = f64(dev(x, dtype))
    q = plain_llama.rope((xs @ ws["q_proj.weight"].T).reshape(n, H, D), range(n), inv, "half")
    k = plain_llama.rope((xs @ ws["k_proj.weight"].T).reshape(n, G, D), range(n), inv, "half")
    v = (xs @ ws["v_proj.weight"].T).reshape(n, G, D)
    ref = np.zeros((n, H * D))
    for i in range(n):                                      # row i sees positions max(0, i - window + 1) .. i
        lo = max(0, i - window + 1)
        for h in range(H):
            g = h // (H // G)
            sc = k[lo:i + 1, g] @ q[i, h] / np.sqrt(D)
            pr = np.exp(sc - sc.max())
            ref[i, h * D:(h + 1) * D] = (pr / pr.sum()) @ v[lo:i + 1, g]
    ref = ref @ ws["o_proj.weight"].T
    slot = cache.acquire()
    got = []
    # a prompt of 150 rows, then one row a step
    for rows in [list(range(150))] + [[i] for i in range(150, n)]:
        entry = StepEntry(slot, [0] * len(rows))
        start = cache.slots.length(slot)
        cache.slots.reserve(slot, start + len(rows), rows=len(rows))
        cache.sync_tables()
        ctx = context([entry], [start])
        residual = torch.zeros((len(rows), E), dtype=torch.float32, device="cuda")
        windowed.forward(dev(x[rows], dtype), residual, ctx, cache.memory(1))
        scratch = torch.zeros_like(residual)
        full.forward(dev(x[rows], dtype), scratch, ctx, cache.memory(0))
        cache.slots.commit(slot, start + len(rows))
        got.append(f64(residual))
    got = np.concatenate(got)
    assert np.abs(got - ref).max() <= tol(dtype, ref) * 2
    held_full = sum(p >= 0 for p in cache.slots.tables[0][slot])
    held_win = sum(p >= 0 for p in cache.slots.tables[1][slot])
    assert held_full == 6 and held_win == 2, "the windowed group gave the pages behind its window back"
    cache.release(slot)
    cache.slots.check()


# --------------------------------------------------------------------------- the toy model

def register_toy():
    from borrowed_compute_b200.architectures import register_architecture
    from borrowed_compute_b200.config import LlamaConfig
    from borrowed_compute_b200.parts import MIXERS, LayerSpec, Mixer, ModelSpec, PartSpec, RunSpec, StateNeed, TensorSpec

    if "toy_running_mean" not in MIXERS.names():
        @MIXERS.register("toy_running_mean")
        class RunningMean(Mixer):
            """out[row] = mean of this sequence's inputs up to and including row, times W^T.
            The running sum is per-sequence state of fixed size."""

            graph_safe = False    # loops over this step's sequences on the host

            def __init__(self, hidden_size):
                super().__init__(hidden_size=hidden_size)
                self.hidden_size = hidden_size

            def tensors(self):
                return {"mix.weight": TensorSpec((self.hidden_size, self.hidden_size))}

            def state_need(self):
                return StateNeed((self.hidden_size,), torch.float32)

            def load(self, tensors, rt):
                super().load(tensors, rt)
                self.w = tensors["mix.weight"].float()

            def forward(self, x, residual, ctx, mem):
                xf = x.float()
                for s in range(ctx.seqs):
                    a, b, slot = ctx.host_seq_rows[s], ctx.host_seq_rows[s + 1], ctx.host_seq_slot[s]
                    if slot < 0 or a == b:
                        continue
                    run = mem.state[slot][None, :] + torch.cumsum(xf[a:b], dim=0)
                    if mem.writes:
                        mem.state[slot] = run[-1]
                    count = (ctx.row_pos[a:b].float() + 1.0)[:, None]
                    residual[a:b] += (run / count) @ self.w.T

    def toy_spec(cfg):
        position = {"kind": "rotary", "head_dim": cfg.head_dim, "theta": cfg.rope_theta, "pairing": cfg.rope_pairing,
                    "scaling": None, "max_positions": cfg.max_position_embeddings}
        norm = lambda p: PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, p)
        ff = lambda p: PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size}, p)
        layers = (
            LayerSpec("prenorm", norm1=norm("l0.n1."), mixer=PartSpec("gqa_attention", {
                "hidden_size": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim, "position": position}, "l0.attn."), norm2=norm("l0.n2."), feed_forward=ff("l0.ff.")),
            LayerSpec("prenorm", norm1=norm("l1.n1."), mixer=PartSpec("toy_running_mean", {"hidden_size": cfg.hidden_size}, "l1."),
                      norm2=norm("l1.n2."), feed_forward=ff("l1.ff.")),
        )
        # Layer 0 runs three times: twice with a cache of its own, once reading the first run's.
        schedule = (RunSpec(0), RunSpec(1), RunSpec(0), RunSpec(0, memory_of=0), RunSpec(1))
        return ModelSpec(hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
                         embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size}, "emb."),
                         layers=layers, schedule=schedule, final_norm=norm("out_norm."),
                         head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "tied": True}, "head."))

    register_architecture("ToyMixForCausalLM", LlamaConfig.from_dict, toy_spec)


TOY = {"architectures": ["ToyMixForCausalLM"], "num_hidden_layers": 2, "hidden_size": 48, "num_attention_heads": 3,
       "num_key_value_heads": 1, "head_dim": 16, "intermediate_size": 80, "vocab_size": 90, "rope_theta": 10000.0,
       "rms_norm_eps": 1e-5, "max_position_embeddings": 256}


def toy_reference(w, tokens):
    """The toy model in plain NumPy, whole sequence at once."""
    c = plain_llama.read_config(TOY)
    n = len(tokens)
    inv = plain_llama.rope_inv_freq(c["head_dim"], c["theta"], None)
    x = plain_llama.embed(w["emb.weight"], tokens)
    kept = {}

    def attention_layer(x, run, memory_of=None):
        h = plain_llama.rms_norm(x, w["l0.n1.weight"], c["eps"])
        q = plain_llama.rope((h @ w["l0.attn.q_proj.weight"].T).reshape(n, 3, 16), range(n), inv, "half")
        if memory_of is None:
            k = plain_llama.rope((h @ w["l0.attn.k_proj.weight"].T).reshape(n, 1, 16), range(n), inv, "half")
            v = (h @ w["l0.attn.v_proj.weight"].T).reshape(n, 1, 16)
            kept[run] = (k, v)
        else:
            k, v = kept[memory_of]
        x = x + plain_llama.attention(q, k, v).reshape(n, 48) @ w["l0.attn.o_proj.weight"].T
        h = plain_llama.rms_norm(x, w["l0.n2.weight"], c["eps"])
        return x + plain_llama.swiglu(h, w["l0.ff.gate_proj.weight"], w["l0.ff.up_proj.weight"], w["l0.ff.down_proj.weight"])

    def mean_layer(x):
        h = plain_llama.rms_norm(x, w["l1.n1.weight"], c["eps"])
        run = np.cumsum(h, axis=0) / np.arange(1, n + 1)[:, None]
        x = x + run @ w["l1.mix.weight"].T
        h = plain_llama.rms_norm(x, w["l1.n2.weight"], c["eps"])
        return x + plain_llama.swiglu(h, w["l1.ff.gate_proj.weight"], w["l1.ff.up_proj.weight"], w["l1.ff.down_proj.weight"])

    x = attention_layer(x, 0)
    x = mean_layer(x)
    x = attention_layer(x, 2)
    x = attention_layer(x, 3, memory_of=0)
    x = mean_layer(x)
    return plain_llama.rms_norm(x, w["out_norm.weight"], c["eps"]) @ w["emb.weight"].T


def test_toy_model_with_a_stateful_mixer(tmp_path):
    from borrowed_compute_b200 import Engine, StepEntry
    from borrowed_compute_b200.weights import TensorSource, write_safetensors

    register_toy()
    from borrowed_compute_b200.engine.model import expected_tensors_for_config

    expected = expected_tensors_for_config(TOY)
    assert "l1.mix.weight" in expected and "l0.attn.q_proj.weight" in expected and len(expected) == 1 + (2 + 4 + 3) + (2 + 1 + 3) + 1 + 1
    r = np.random.default_rng(9)
    w = {k: ((1 + 0.1 * r.standard_normal(s.shape)) if s.role == "vector" else r.standard_normal(s.shape) * (1.0 if k == "emb.weight" else 0.2))
         .astype(np.float32) for k, s in expected.items() if not s.optional}
    folder = str(tmp_path / "toy")
    os.makedirs(folder)
    json.dump(TOY, open(os.path.join(folder, "config.json"), "w"))
    write_safetensors(os.path.join(folder, "model.safetensors"), {k: torch.from_numpy(v) for k, v in w.items()})
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=1024, max_slots=3)
    assert not eng.use_graphs                                     # the toy mixer plans on the host
    assert len(eng.cache.groups) == 1 and len(eng.cache.groups[0].runs) == 2 and sorted(eng.cache.state) == [1, 4]
    w64 = {k: v.astype(np.float64) for k, v in w.items()}
    a, b = seeded_tokens(1, 70, 90), seeded_tokens(2, 9, 90)
    ref_a, ref_b = toy_reference(w64, a), toy_reference(w64, b)
    tol_a = 1e-4 * (1 + np.abs(ref_a).max())
    # whole
    s = eng.acquire()
    whole = eng.step([StepEntry(s, a, want=tuple(range(len(a))))]).cpu().numpy()
    eng.release(s)
    assert np.abs(whole - ref_a).max() <= tol_a
    # the other request through the slot that was just given back: its state must start from zero
    s2 = eng.acquire()
    assert s2 == s
    other = eng.step([StepEntry(s2, b, want=tuple(range(len(b))))]).cpu().numpy()
    eng.release(s2)
    assert np.abs(other - ref_b).max() <= 1e-4 * (1 + np.abs(ref_b).max())
    # a batch of both: prompts in one step, then one token each; the shorter one ends earlier
    sa, sb = eng.acquire(), eng.acquire()
    first = eng.step([StepEntry(sa, a[:40], want=tuple(range(40))), StepEntry(sb, b[:4], want=tuple(range(4)))]).cpu().numpy()
    got_a, got_b = [first[:40]], [first[40:]]
    for i in range(30):
        entries = [StepEntry(sa, [a[40 + i]], want=(0,))] + ([StepEntry(sb, [b[4 + i]], want=(0,))] if 4 + i < len(b) else [])
        out = eng.step(entries).cpu().numpy()
        got_a.append(out[:1])
        if len(entries) == 2:
            got_b.append(out[1:])
        if 4 + i == len(b) - 1:
            eng.release(sb)
    eng.release(sa)
    assert np.abs(np.concatenate(got_a) - ref_a).max() <= tol_a
    assert np.abs(np.concatenate(got_b) - ref_b).max() <= 1e-4 * (1 + np.abs(ref_b).max())
    eng.cache.slots.check()
    assert eng.cache.slots.live() == []


# -------------------------------------------- toy parts: a routed feed-forward, learned positions

def register_routed_toy():
    """A second toy architecture: attention without rotation, positions learned as a table
    added to the stream after the embedding, and a feed-forward that routes every row to
    one of three small experts.  All of it defined here, none of it in the framework."""
    from borrowed_compute_b200.architectures import register_architecture
    from borrowed_compute_b200.config.llama import LlamaConfig
    from borrowed_compute_b200.parts.base import (FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, LayerSpec, ModelSpec, PartSpec,
                                                  PositionEncoding, RunSpec, TensorSpec)

    if "toy_top1_experts" not in FEED_FORWARDS.names():
        @FEED_FORWARDS.register("toy_top1_experts")
        class Top1Experts(FeedForward):
            """Each row goes to the expert whose router score is largest (float32 scores, the
            first of equals): out = down_e(relu(up_e(x))).  Runs on the device without a
            look at the host, so decode steps can be captured."""

            def __init__(self, hidden_size, inner, experts):
                super().__init__(hidden_size=hidden_size, inner=inner, experts=experts)
                self.hidden_size, self.inner, self.experts = hidden_size, inner, experts

            def tensors(self):
                return {"router.weight": TensorSpec((self.experts, self.hidden_size)),
                        "up.weight": TensorSpec((self.experts * self.inner, self.hidden_size)),
                        "down.weight": TensorSpec((self.experts * self.hidden_size, self.inner))}

            def load(self, tensors, rt):
                super().load(tensors, rt)
                self.router = tensors["router.weight"].float()
                self.up = tensors["up.weight"].float().reshape(self.experts, self.inner, self.hidden_size)
                self.down = tensors["down.weight"].float().reshape(self.experts, self.hidden_size, self.inner)

            def forward(self, x, residual, ctx):
                xf = x.float()
                choice = torch.argmax(xf @ self.router.T, dim=1)                      # [rows]
                hidden = torch.relu(torch.einsum("rh,eih->rei", xf, self.up))         # every expert, then pick: a toy
                out = torch.einsum("rei,ehi->reh", hidden, self.down)
                residual[: x.shape[0]] += out[torch.arange(x.shape[0], device=x.device), choice]

    if "toy_learned_positions" not in POSITION_ENCODINGS.names():
        @POSITION_ENCODINGS.register("toy_learned_positions")
        class LearnedPositions(PositionEncoding):
            """A table [positions, hidden] added to the stream after the embedding."""

            def __init__(self, hidden_size, max_positions):
                super().__init__(hidden_size=hidden_size, max_positions=max_positions)
                self.hidden_size, self.max_positions = hidden_size, max_positions

            def tensors(self):
                return {"table": TensorSpec((self.max_positions, self.hidden_size))}

            def load(self, tensors, rt):
                super().load(tensors, rt)
                self.table = tensors["table"].float()

            def on_embeddings(self, residual, ctx):
                residual[: ctx.rows] += self.table[ctx.row_pos.long()] * (ctx.row_slot >= 0)[:, None]

    def routed_spec(cfg):
        norm = lambda p: PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, p)
        layers = tuple(
            LayerSpec("prenorm", norm1=norm(f"l{i}.n1."), mixer=PartSpec("gqa_attention", {
                "hidden_size": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim, "position": {"kind": "none"}}, f"l{i}.attn."), norm2=norm(f"l{i}.n2."),
                feed_forward=PartSpec("toy_top1_experts", {"hidden_size": cfg.hidden_size, "inner": cfg.intermediate_size, "experts": 3}, f"l{i}.moe."))
            for i in range(cfg.num_hidden_layers))
        return ModelSpec(hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
                         embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size}, "emb."),
                         position=PartSpec("toy_learned_positions", {"hidden_size": cfg.hidden_size, "max_positions": cfg.max_position_embeddings}, "pos."),
                         layers=layers, schedule=tuple(RunSpec(i) for i in range(cfg.num_hidden_layers)), final_norm=norm("out_norm."),
                         head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "tied": True}, "head."))

    register_architecture("ToyRoutedForCausalLM", LlamaConfig.from_dict, routed_spec)


ROUTED = {"architectures": ["ToyRoutedForCausalLM"], "num_hidden_layers": 2, "hidden_size": 40, "num_attention_heads": 2,
          "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 24, "vocab_size": 70, "rope_theta": 10000.0,
          "rms_norm_eps": 1e-5, "max_position_embeddings": 160}


def routed_reference(w, tokens):
    """The routed toy in plain NumPy, whole sequence at once; also which expert each row took."""
    c = plain_llama.read_config(ROUTED)
    n, hid, inner = len(tokens), 40, 24
    x = plain_llama.embed(w["emb.weight"], tokens) + w["pos.table"][:n]
    taken = []
    for i in range(2):
        h = plain_llama.rms_norm(x, w[f"l{i}.n1.weight"], c["eps"])
        q = (h @ w[f"l{i}.attn.q_proj.weight"].T).reshape(n, 2, 16)
        k = (h @ w[f"l{i}.attn.k_proj.weight"].T).reshape(n, 2, 16)
        v = (h @ w[f"l{i}.attn.v_proj.weight"].T).reshape(n, 2, 16)
        x = x + plain_llama.attention(q, k, v).reshape(n, 32) @ w[f"l{i}.attn.o_proj.weight"].T
        h = plain_llama.rms_norm(x, w[f"l{i}.n2.weight"], c["eps"])
        choice = np.argmax(h @ w[f"l{i}.moe.router.weight"].T, axis=1)
        up = w[f"l{i}.moe.up.weight"].reshape(3, inner, hid)
        down = w[f"l{i}.moe.down.weight"].reshape(3, hid, inner)
        x = x + np.stack([down[e] @ np.maximum(up[e] @ h[r], 0.0) for r, e in enumerate(choice)])
        taken.append(choice)
    return plain_llama.rms_norm(x, w["out_norm.weight"], c["eps"]) @ w["emb.weight"].T, taken


def test_toy_model_with_a_routed_feed_forward_and_learned_positions(tmp_path):
    """A feed-forward with routing and a position encoding that acts on the embeddings,
    registered from here, run through the ordinary engine (captured decode steps included)
    in float32, against their plain NumPy twin: whole, prompt then single tokens, and two
    requests in a batch."""
    from borrowed_compute_b200 import Engine, StepEntry
    from borrowed_compute_b200.engine.model import expected_tensors_for_config
    from borrowed_compute_b200.weights import write_safetensors

    register_routed_toy()
    expected = expected_tensors_for_config(ROUTED)
    assert "pos.table" in expected and "l1.moe.router.weight" in expected and "l0.attn.q_proj.weight" in expected
    r = np.random.default_rng(11)
    w = {k: ((1 + 0.1 * r.standard_normal(s.shape)) if s.role == "vector" else r.standard_normal(s.shape) * (1.0 if k == "emb.weight" else 0.3))
         .astype(np.float32) for k, s in expected.items() if not s.optional}
    folder = str(tmp_path / "routed")
    os.makedirs(folder)
    json.dump(ROUTED, open(os.path.join(folder, "config.json"), "w"))
    write_safetensors(os.path.join(folder, "model.safetensors"), {k: torch.from_numpy(v) for k, v in w.items()})
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, max_slots=3)
    assert eng.use_graphs                                          # nothing here plans on the host
    w64 = {k: v.astype(np.float64) for k, v in w.items()}
    a, b = seeded_tokens(5, 90, 70), seeded_tokens(6, 13, 70)
    (ref_a, taken_a), (ref_b, _) = routed_reference(w64, a), routed_reference(w64, b)
    assert all(len(set(t.tolist())) == 3 for t in taken_a), "the routing must reach every expert, or the test shows little"
    tol_a, tol_b = 2e-4 * (1 + np.abs(ref_a).max()), 2e-4 * (1 + np.abs(ref_b).max())
    s = eng.acquire()
    whole = eng.step([StepEntry(s, a, want=tuple(range(len(a))))]).cpu().numpy()
    eng.release(s)
    assert np.abs(whole - ref_a).max() <= tol_a, "whole"
    s = eng.acquire()
    head = eng.step([StepEntry(s, a[:50], want=tuple(range(50)))]).cpu().numpy()
    tail = np.concatenate([eng.step([StepEntry(s, [t], want=(0,))]).cpu().numpy() for t in a[50:]])
    eng.release(s)
    assert np.abs(np.concatenate([head, tail]) - ref_a).max() <= tol_a, "prompt, then single tokens through the captured step"
    sa, sb = eng.acquire(), eng.acquire()
    first = eng.step([StepEntry(sa, a[:60], want=tuple(range(60))), StepEntry(sb, b[:5], want=tuple(range(5)))]).cpu().numpy()
    got_a, got_b = [first[:60]], [first[60:]]
    for i in range(30):
        entries = [StepEntry(sa, [a[60 + i]], want=(0,))] + ([StepEntry(sb, [b[5 + i]], want=(0,))] if 5 + i < len(b) else [])
        out = eng.step(entries).cpu().numpy()
        got_a.append(out[:1])
        if len(entries) == 2:
            got_b.append(out[1:])
        if 5 + i == len(b) - 1:
            eng.release(sb)
    eng.release(sa)
    assert np.abs(np.concatenate(got_a) - ref_a).max() <= tol_a and np.abs(np.concatenate(got_b) - ref_b).max() <= tol_b, "batch"
    eng.cache.slots.check()
