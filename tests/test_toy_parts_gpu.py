"""A toy architecture defined here, in the test: a mixer with a state of its own (a running
mean of its inputs, kept per request in a state slot) beside an attention layer that borrows
nothing from GPT-2's description.  It is registered, its random weights are written and
loaded, and it is stepped whole, in portions and mixed with other requests through the same
ModelRunner as GPT-2, without any change to the package's files."""
import json
import os
from dataclasses import dataclass

import pytest
import torch

pytestmark = pytest.mark.gpu


def _register():
    import mini_llm_b200 as m
    from mini_llm_b200.cache.manager import StateNeed
    from mini_llm_b200.config.base import ModelConfig
    from mini_llm_b200.parts.base import Mixer, ParamSpec
    from mini_llm_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, WeightRef

    class RunningMean(Mixer):
        """out[t] = W . mean(h[0..t]) of the request; the state is (sum of h, count)."""
        graph_safe = False                      # reads the batch's slot ids on the host

        def __init__(self, hidden_size):
            self.hidden_size = hidden_size

        def param_specs(self):
            return {"w": ParamSpec((self.hidden_size, self.hidden_size), "matrix")}

        def cache_need(self):
            return StateNeed((self.hidden_size + 1,), "float32")

        def forward(self, h, ctx, cache, out_accum):
            D = self.hidden_size
            slots = ctx.state_slots.tolist()
            base = 0
            for s, n in enumerate(ctx.q_lens):
                st = cache.state[slots[s]]
                x = h[base:base + n].float()
                csum = torch.cumsum(x, 0) + st[:D]
                cnt = st[D] + torch.arange(1, n + 1, device=x.device, dtype=torch.float32)
                mean = csum / cnt[:, None]
                out_accum[base:base + n] += mean @ self.w.float().t()
                if cache.write:
                    st[:D] = csum[-1]
                    st[D] = cnt[-1]
                base += n

    @dataclass
    class ToyConfig(ModelConfig):
        hidden: int = 0
        vocab: int = 0
        heads: int = 0
        inner: int = 0
        eps: float = 1e-5

        @classmethod
        def from_dict(cls, d):
            return cls(hidden=d["hidden"], vocab=d["vocab"], heads=d["heads"], inner=d["inner"], eps=d["eps"])

        def to_dict(self):
            return dict(architectures=["ToyStateLM"], hidden=self.hidden, vocab=self.vocab, heads=self.heads,
                        inner=self.inner, eps=self.eps)

    def build(cfg):
        D = cfg.hidden

        def norm(name):
            return PartSpec("layernorm", dict(hidden_size=D, eps=cfg.eps),
                            {"weight": WeightRef((name + ".g",), init=("ones",)), "bias": WeightRef((name + ".b",), init=("zeros",))})

        def ff(i):
            return PartSpec("mlp", dict(hidden_size=D, inner_size=cfg.inner, activation="gelu_erf", bias=False),
                            {"fc_weight": WeightRef((f"l{i}.up",), init=("normal", 0.2)),
                             "proj_weight": WeightRef((f"l{i}.down",), init=("normal", 0.2))})

        l0 = LayerSpec(mixer=PartSpec("toy_running_mean", dict(hidden_size=D), {"w": WeightRef(("l0.mix",), init=("normal", 0.3))}),
                       ff=ff(0), mixer_norm=norm("l0.n1"), ff_norm=norm("l0.n2"))
        l1 = LayerSpec(mixer=PartSpec("attention", dict(hidden_size=D, num_heads=cfg.heads, head_dim=D // cfg.heads,
                                                        scale=(D // cfg.heads) ** -0.5, bias=False),
                                      {"qkv_weight": WeightRef(("l1.qkv",), init=("normal", 0.3)),
                                       "out_weight": WeightRef(("l1.o",), init=("normal", 0.3))}),
                       ff=ff(1), mixer_norm=norm("l1.n1"), ff_norm=norm("l1.n2"))
        # the order of layers is data: state mixer, attention, the state mixer's layer again
        # (second run borrows layer 1's ... no: it names layer 0 twice; the second run must not write)
        return ModelSpec(hidden_size=D, vocab_size=cfg.vocab,
                         embedding=PartSpec("token", dict(hidden_size=D, vocab_size=cfg.vocab),
                                            {"table": WeightRef(("emb",), init=("normal", 1.0))}),
                         positions=PartSpec("none", {}), layers=[l0, l1], final_norm=norm("nf"),
                         head=PartSpec("tied", dict(hidden_size=D, vocab_size=cfg.vocab)),
                         schedule=[ScheduleEntry(0), ScheduleEntry(1)], max_positions=None)

    m.register_part("mixer", "toy_running_mean", RunningMean, replace=True)
    m.register_architecture("ToyStateLM", ToyConfig, build, replace=True)
    return dict(architectures=["ToyStateLM"], hidden=48, vocab=97, heads=3, inner=80, eps=1e-5)


def _reference(folder, ids):
    """Whole-sequence float64 statement of the toy model."""
    from safetensors.torch import load_file
    w = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    cfg = json.load(open(os.path.join(folder, "config.json")))
    D, H = cfg["hidden"], cfg["heads"]
    dh = D // H

    def ln(x, n):
        return torch.nn.functional.layer_norm(x, (D,), w[n + ".g"], w[n + ".b"], cfg["eps"])

    x = w["emb"][torch.tensor(ids)]
    T = len(ids)
    h = ln(x, "l0.n1")
    mean = torch.cumsum(h, 0) / torch.arange(1, T + 1, dtype=torch.float64)[:, None]
    x = x + mean @ w["l0.mix"].t()
    x = x + torch.nn.functional.gelu(ln(x, "l0.n2") @ w["l0.up"].t()) @ w["l0.down"].t()
    qkv = ln(x, "l1.n1") @ w["l1.qkv"].t()
    att = torch.zeros(T, D, dtype=torch.float64)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for hh in range(H):
        q, k, v = (qkv[:, i * D + hh * dh:i * D + (hh + 1) * dh] for i in range(3))
        s = (q @ k.t()) * dh ** -0.5
        att[:, hh * dh:(hh + 1) * dh] = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ v
    x = x + att @ w["l1.o"].t()
    x = x + torch.nn.functional.gelu(ln(x, "l1.n2") @ w["l1.up"].t()) @ w["l1.down"].t()
    return ln(x, "nf") @ w["emb"].t()


def test_toy_architecture_with_a_state_mixer(tmp_path):
    import mini_llm_b200 as m
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner, StepEntry

    cfg = _register()
    folder = m.write_random_model(cfg, 3, str(tmp_path / "toy"))
    runner = ModelRunner(folder, EngineConfig(dtype="float32", page_size=8, num_pages=40, max_num_seqs=3))
    assert runner.cache.state_layers and list(runner.cache.state_layers) == [0]
    assert runner.cache.group_of_layer == {1: 0}
    g = torch.Generator().manual_seed(0)
    reqs = {r: torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for r, n in (("a", 37), ("b", 9), ("c", 64))}
    want = {r: _reference(folder, ids) for r, ids in reqs.items()}
    # whole
    for r, ids in reqs.items():
        runner.add_request(r)
        got = runner.step([StepEntry(r, ids, list(range(len(ids))))])
        assert (got.double().cpu() - want[r]).abs().max() < 2e-4 * want[r].abs().max(), r
        runner.finish_request(r)
    # in portions, mixed with the others, slots reused: the state carries over from step to step
    plan = {"a": [5, 2, 13, 1, 1, 15], "b": [2, 7], "c": [30, 1, 1, 32]}
    pos = {r: 0 for r in reqs}
    got = {r: [] for r in reqs}
    for r in ("a", "b"):
        runner.add_request(r)
    live = ["a", "b"]
    while live:
        entries = []
        for r in list(live):
            n = plan[r].pop(0)
            entries.append(StepEntry(r, reqs[r][pos[r]:pos[r] + n], list(range(n))))
            pos[r] += n
        out = runner.step(entries)
        k = 0
        for e in entries:
            got[e.req].append(out[k:k + len(e.tokens)].double().cpu())
            k += len(e.tokens)
        for r in list(live):
            if not plan[r]:
                runner.finish_request(r)
                live.remove(r)
                if r == "b":                 # c takes b's slot: its state must start from zero
                    runner.add_request("c")
                    live.append("c")
    for r in reqs:
        assert (torch.cat(got[r]) - want[r]).abs().max() < 2e-4 * want[r].abs().max(), r
    runner.cache.check()
    assert runner.cache.num_live == 0


def _register_window():
    import mini_llm_b200 as m
    from mini_llm_b200.config.base import ModelConfig
    from mini_llm_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, WeightRef

    @dataclass
    class WinConfig(ModelConfig):
        hidden: int = 0
        vocab: int = 0
        heads: int = 0
        kv_heads: int = 0
        window: int = 0

        @classmethod
        def from_dict(cls, d):
            return cls(hidden=d["hidden"], vocab=d["vocab"], heads=d["heads"], kv_heads=d["kv_heads"], window=d["window"])

        def to_dict(self):
            return dict(architectures=["ToyWindowLM"], hidden=self.hidden, vocab=self.vocab, heads=self.heads,
                        kv_heads=self.kv_heads, window=self.window)

    def build(cfg):
        D, H, Hkv = cfg.hidden, cfg.heads, cfg.kv_heads
        dh = D // H

        def norm(name):
            return PartSpec("layernorm", dict(hidden_size=D, eps=1e-5),
                            {"weight": WeightRef((name + ".g",), init=("ones",)), "bias": WeightRef((name + ".b",), init=("zeros",))})

        def layer(i, window, kvh):
            att = PartSpec("attention", dict(hidden_size=D, num_heads=H, num_kv_heads=kvh, head_dim=dh, scale=dh ** -0.5,
                                             window=window, bias=True),
                           {"qkv_weight": WeightRef((f"l{i}.qkv",), init=("normal", 0.4)),
                            "qkv_bias": WeightRef((f"l{i}.qkv_b",), init=("normal", 0.1)),
                            "out_weight": WeightRef((f"l{i}.o",), init=("normal", 0.3)),
                            "out_bias": WeightRef((f"l{i}.o_b",), init=("normal", 0.1))})
            ff = PartSpec("mlp", dict(hidden_size=D, inner_size=2 * D, activation="gelu_tanh", bias=True),
                          {"fc_weight": WeightRef((f"l{i}.up",), init=("normal", 0.2)), "fc_bias": WeightRef((f"l{i}.up_b",), init=("zeros",)),
                           "proj_weight": WeightRef((f"l{i}.down",), init=("normal", 0.2)), "proj_bias": WeightRef((f"l{i}.down_b",), init=("zeros",))})
            return LayerSpec(mixer=att, ff=ff, mixer_norm=norm(f"l{i}.n1"), ff_norm=norm(f"l{i}.n2"))

        # layer 0: a window of `window` keys and grouped key/value heads; layer 1: all keys, one k/v head per head
        return ModelSpec(hidden_size=D, vocab_size=cfg.vocab,
                         embedding=PartSpec("token", dict(hidden_size=D, vocab_size=cfg.vocab), {"table": WeightRef(("emb",), init=("normal", 1.0))}),
                         positions=PartSpec("learned", dict(hidden_size=D, max_positions=512), {"table": WeightRef(("pos",), init=("normal", 0.5))}),
                         layers=[layer(0, cfg.window, Hkv), layer(1, None, H)], final_norm=norm("nf"),
                         head=PartSpec("tied", dict(hidden_size=D, vocab_size=cfg.vocab)), max_positions=512)

    m.register_architecture("ToyWindowLM", WinConfig, build, replace=True)
    return dict(architectures=["ToyWindowLM"], hidden=64, vocab=120, heads=4, kv_heads=2, window=20)


def _window_reference(folder, ids, store=lambda t: t):
    """Whole-sequence float64 statement; ``store`` rounds the values an engine keeps in bfloat16
    between kernels (normed rows, Q|K|V, attention output, the MLP's hidden row)."""
    from safetensors.torch import load_file
    w = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    cfg = json.load(open(os.path.join(folder, "config.json")))
    D, H, T = cfg["hidden"], cfg["heads"], len(ids)
    dh = D // H

    def ln(x, n):
        return torch.nn.functional.layer_norm(x, (D,), w[n + ".g"], w[n + ".b"], 1e-5)

    x = w["emb"][torch.tensor(ids)] + w["pos"][:T]
    idx = torch.arange(T)
    for i, (window, kvh) in enumerate(((cfg["window"], cfg["kv_heads"]), (None, H))):
        qkv = store(store(ln(x, f"l{i}.n1")) @ w[f"l{i}.qkv"].t() + w[f"l{i}.qkv_b"])
        q, k, v = qkv[:, :D], qkv[:, D:D + kvh * dh], qkv[:, D + kvh * dh:]
        vis = idx[None, :] <= idx[:, None]
        if window:
            vis &= idx[None, :] > idx[:, None] - window
        att = torch.zeros(T, D, dtype=torch.float64)
        for hh in range(H):
            hk = hh // (H // kvh)
            s = (q[:, hh * dh:(hh + 1) * dh] @ k[:, hk * dh:(hk + 1) * dh].t()) * dh ** -0.5
            att[:, hh * dh:(hh + 1) * dh] = torch.softmax(s.masked_fill(~vis, float("-inf")), -1) @ v[:, hk * dh:(hk + 1) * dh]
        x = x + store(att) @ w[f"l{i}.o"].t() + w[f"l{i}.o_b"]
        h = store(torch.nn.functional.gelu(store(ln(x, f"l{i}.n2")) @ w[f"l{i}.up"].t() + w[f"l{i}.up_b"], approximate="tanh"))
        x = x + h @ w[f"l{i}.down"].t() + w[f"l{i}.down_b"]
    return store(ln(x, "nf")) @ w["emb"].t()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_a_window_and_grouped_heads(tmp_path, dtype):
    """Two cache groups in one model: a layer with a 20-key window and 2 key/value heads beside a
    layer that sees everything.  Whole, in portions and token by token; the windowed group gives
    pages back while the request runs, and the logits stay right."""
    import mini_llm_b200 as m
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner, StepEntry

    cfg = _register_window()
    folder = m.write_random_model(cfg, 5, str(tmp_path / "win"), dtype=dtype)
    runner = ModelRunner(folder, EngineConfig(dtype=dtype, page_size=8, num_pages=40, max_num_seqs=2))
    assert len(runner.cache.groups) == 2
    windowed = next(g for g in runner.cache.groups if g.need.window == 20)
    assert windowed.need.kv_heads == 2
    from helpers import assert_close, oracle_store
    ids = torch.randint(0, cfg["vocab"], (150,), generator=torch.Generator().manual_seed(3)).tolist()
    want = _window_reference(folder, ids, oracle_store(dtype))
    for plan in ([150], [70, 1, 1, 1, 40, 37], [3] + [1] * 40 + [107]):
        runner.add_request("r")
        got, pos = [], 0
        for n in plan:
            got.append(runner.step([StepEntry("r", ids[pos:pos + n], list(range(n)))]).double().cpu())
            pos += n
            held = sum(p >= 0 for p in runner.cache.table("r", windowed.index))
            assert held <= (20 + 8 - 2) // 8 + 2 + (n + 7) // 8       # only the window's pages (and this step's) are kept
        assert_close(torch.cat(got).numpy(), want.numpy(), dtype, f"window model, portions {plan[:3]}")
        runner.finish_request("r")
    runner.cache.check()
    assert all(g.allocator.num_free == 40 for g in runner.cache.groups)


# ---------------------------------------------------------------------------------- rotary positions, routed experts
def _register_rotary_routed():
    """A position encoding that acts on queries and keys (a rotation by the absolute position) and a
    feed-forward that routes every token to one of several experts, both defined here."""
    import mini_llm_b200 as m
    from mini_llm_b200.config.base import ModelConfig
    from mini_llm_b200.parts.base import FeedForward, ParamSpec, Positions
    from mini_llm_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, WeightRef

    class ToyRotary(Positions):
        acts_on_qk = True
        graph_safe = False

        def __init__(self, head_dim, base):
            self.head_dim, self.base = int(head_dim), float(base)
            self.max_positions = None

        def apply_qk(self, q, k, ctx):
            dh = self.head_dim
            pos = ctx.positions.float()
            inv = self.base ** (-torch.arange(0, dh, 2, device=q.device, dtype=torch.float32) / dh)
            ang = pos[:, None] * inv[None, :]                       # 32-bit angles
            cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
            for x in (q, k):
                v = x.view(x.shape[0], -1, dh // 2, 2)
                a, b = v[..., 0].float().clone(), v[..., 1].float().clone()     # copies: .float() of float32 is a view
                v[..., 0] = (a * cos - b * sin).to(x.dtype)
                v[..., 1] = (a * sin + b * cos).to(x.dtype)

    class ToyRouted(FeedForward):
        """Top-1 routing: y = p_e(h) * down_e . gelu(up_e . h) for the expert e with the largest router logit."""
        graph_safe = False

        def __init__(self, hidden_size, inner_size, num_experts):
            self.D, self.I, self.E = int(hidden_size), int(inner_size), int(num_experts)

        def param_specs(self):
            return {"router": ParamSpec((self.E, self.D), "matrix"), "up": ParamSpec((self.E * self.I, self.D), "matrix"),
                    "down": ParamSpec((self.E * self.D, self.I), "matrix")}

        def forward(self, h, ctx, out_accum):
            x = h.float()
            probs = torch.softmax(x @ self.router.float().t(), -1)      # router logits and softmax in 32-bit
            top = probs.argmax(-1)
            for e in range(self.E):
                rows = (top == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                up = self.up[e * self.I:(e + 1) * self.I].float()
                down = self.down[e * self.D:(e + 1) * self.D].float()
                y = torch.nn.functional.gelu(x[rows] @ up.t()) @ down.t()
                out_accum[rows] += y * probs[rows, e][:, None]

    @dataclass
    class RRConfig(ModelConfig):
        hidden: int = 0
        vocab: int = 0
        heads: int = 0
        inner: int = 0
        experts: int = 0
        base: float = 10000.0

        @classmethod
        def from_dict(cls, d):
            return cls(hidden=d["hidden"], vocab=d["vocab"], heads=d["heads"], inner=d["inner"], experts=d["experts"],
                       base=d["base"])

        def to_dict(self):
            return dict(architectures=["ToyRotaryRoutedLM"], hidden=self.hidden, vocab=self.vocab, heads=self.heads,
                        inner=self.inner, experts=self.experts, base=self.base)

    def build(cfg):
        D, H = cfg.hidden, cfg.heads
        dh = D // H

        def norm(name):
            return PartSpec("layernorm", dict(hidden_size=D, eps=1e-5),
                            {"weight": WeightRef((name + ".g",), init=("ones",)), "bias": WeightRef((name + ".b",), init=("zeros",))})

        def layer(i):
            att = PartSpec("attention", dict(hidden_size=D, num_heads=H, head_dim=dh, scale=dh ** -0.5, bias=False),
                           {"qkv_weight": WeightRef((f"l{i}.qkv",), init=("normal", 0.4)),
                            "out_weight": WeightRef((f"l{i}.o",), init=("normal", 0.3))})
            ff = PartSpec("toy_routed", dict(hidden_size=D, inner_size=cfg.inner, num_experts=cfg.experts),
                          {"router": WeightRef((f"l{i}.router",), init=("normal", 1.0)),
                           "up": WeightRef((f"l{i}.up",), init=("normal", 0.2)),
                           "down": WeightRef((f"l{i}.down",), init=("normal", 0.2))})
            return LayerSpec(mixer=att, ff=ff, mixer_norm=norm(f"l{i}.n1"), ff_norm=norm(f"l{i}.n2"))

        return ModelSpec(hidden_size=D, vocab_size=cfg.vocab,
                         embedding=PartSpec("token", dict(hidden_size=D, vocab_size=cfg.vocab), {"table": WeightRef(("emb",), init=("normal", 1.0))}),
                         positions=PartSpec("toy_rotary", dict(head_dim=dh, base=cfg.base), {}),
                         layers=[layer(0), layer(1)], final_norm=norm("nf"),
                         head=PartSpec("tied", dict(hidden_size=D, vocab_size=cfg.vocab)), max_positions=None)

    m.register_part("positions", "toy_rotary", ToyRotary, replace=True)
    m.register_part("feed_forward", "toy_routed", ToyRouted, replace=True)
    m.register_architecture("ToyRotaryRoutedLM", RRConfig, build, replace=True)
    return dict(architectures=["ToyRotaryRoutedLM"], hidden=64, vocab=150, heads=2, inner=48, experts=3, base=100.0)


def _rotary_routed_reference(folder, ids):
    from safetensors.torch import load_file
    w = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    cfg = json.load(open(os.path.join(folder, "config.json")))
    D, H, E, I, T = cfg["hidden"], cfg["heads"], cfg["experts"], cfg["inner"], len(ids)
    dh = D // H

    def ln(x, n):
        return torch.nn.functional.layer_norm(x, (D,), w[n + ".g"], w[n + ".b"], 1e-5)

    def rotate(x):                                           # [T, heads*dh]
        pos = torch.arange(T, dtype=torch.float64)
        inv = cfg["base"] ** (-torch.arange(0, dh, 2, dtype=torch.float64) / dh)
        ang = pos[:, None] * inv[None, :]
        v = x.reshape(T, -1, dh // 2, 2)
        a, b = v[..., 0], v[..., 1]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        return torch.stack([a * c - b * s, a * s + b * c], -1).reshape(T, -1)

    x = w["emb"][torch.tensor(ids)]
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    margins = []
    for i in range(2):
        qkv = ln(x, f"l{i}.n1") @ w[f"l{i}.qkv"].t()
        q, k, v = rotate(qkv[:, :D]), rotate(qkv[:, D:2 * D]), qkv[:, 2 * D:]
        att = torch.zeros(T, D, dtype=torch.float64)
        for hh in range(H):
            sl = slice(hh * dh, (hh + 1) * dh)
            s = (q[:, sl] @ k[:, sl].t()) * dh ** -0.5
            att[:, sl] = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ v[:, sl]
        x = x + att @ w[f"l{i}.o"].t()
        h = ln(x, f"l{i}.n2")
        probs = torch.softmax(h @ w[f"l{i}.router"].t(), -1)
        top2 = torch.topk(probs, 2, -1).values
        margins.append((top2[:, 0] - top2[:, 1]).min().item())
        top = probs.argmax(-1)
        y = torch.zeros_like(x)
        for e in range(E):
            rows = (top == e).nonzero().flatten()
            up, down = w[f"l{i}.up"][e * I:(e + 1) * I], w[f"l{i}.down"][e * D:(e + 1) * D]
            y[rows] = (torch.nn.functional.gelu(h[rows] @ up.t()) @ down.t()) * probs[rows, e][:, None]
        x = x + y
    return ln(x, "nf") @ w["emb"].t(), min(margins)


def test_toy_architecture_with_rotary_positions_and_routed_experts(tmp_path):
    """Another position encoding (it rotates queries and keys before the keys are cached, so decoded tokens
    must meet keys rotated at their own positions) and a feed-forward with routing, registered from here and
    run whole, in portions and token by token through the package's step function and attention kernels."""
    import mini_llm_b200 as m
    from mini_llm_b200.config.base import EngineConfig
    from mini_llm_b200.engine.runner import ModelRunner, StepEntry

    cfg = _register_rotary_routed()
    folder = m.write_random_model(cfg, 9, str(tmp_path / "rr"))
    runner = ModelRunner(folder, EngineConfig(dtype="float32", page_size=8, num_pages=64, max_num_seqs=2))
    ids = torch.randint(0, cfg["vocab"], (140,), generator=torch.Generator().manual_seed(4)).tolist()
    want, margin = _rotary_routed_reference(folder, ids)
    assert margin > 1e-4                                    # no routing decision of the oracle hangs on rounding
    for plan in ([140], [60, 1, 1, 1, 33, 44], [2] + [1] * 30 + [108]):
        runner.add_request("r")
        got, pos = [], 0
        for n in plan:
            got.append(runner.step([StepEntry("r", ids[pos:pos + n], list(range(n)))]).double().cpu())
            pos += n
        err = (torch.cat(got) - want).abs().max() / want.abs().max()
        assert err < 2e-4, (plan[:3], float(err))
        runner.finish_request("r")
    # two requests side by side at different positions: every token is rotated by its own position
    other = ids[50:90]
    want2, _ = _rotary_routed_reference(folder, other)
    runner.add_request("a")
    runner.add_request("b")
    runner.step([StepEntry("a", ids[:100], [])])
    out = runner.step([StepEntry("a", ids[100:103], [2]), StepEntry("b", other, [39])]).double().cpu()
    assert (out[0] - want[102]).abs().max() < 2e-4 * want.abs().max()
    assert (out[1] - want2[39]).abs().max() < 2e-4 * want2.abs().max()
    runner.finish_request("a")
    runner.finish_request("b")
    runner.cache.check()
