"""Toy parts defined outside the package, to show that a new mixer, feed-forward, position
encoding or whole architecture is added by registering it - without touching the
framework's files.  They are not models of anything; each comes with a plain reference.

``decay_sum`` mixer: per-request state of its own (a running, decayed sum per channel),
``s_t = sigmoid(a) * s_{t-1} + x_t``, output ``W s_t``.
``routed_ff`` feed-forward: a router picks one of E small linear experts per token.
``rope_linear`` position encoding: a partial rotation with a linear frequency ladder, over
pairs of neighbouring elements (2i, 2i + 1) instead of the half-split pairs LFM2 uses.
``narrow_value_attention`` mixer: one head whose values are narrower than its keys, cached in
an element type of its own (what a latent-KV mixer asks of the cache manager).
``decay_sum`` with ``grid``: the state is float64 and the mixer insists that every portion
starts on a grid, as a recurrence evaluated in chunks of fixed length would.
"""

from __future__ import annotations

import torch

from shiso_llm_b200.parts import (
    FEED_FORWARDS, MIXERS, POSITION_ENCODINGS, FeedForward, FixedState, LayerSpec, Mixer, ModelPlan,
    PagedKV, PartSpec, PositionEncoding, RunEntry,
)
from shiso_llm_b200.weights import VECTOR, TensorSpec


class DecaySum(Mixer):
    graph_safe = False  # loops over the step's sequences on the host

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = spec.params["hidden_size"]
        self.prefix = spec.params["prefix"]

    def tensor_specs(self):
        return [TensorSpec(f"{self.prefix}.decay", (self.hidden,), VECTOR),
                TensorSpec(f"{self.prefix}.out.weight", (self.hidden, self.hidden))]

    def bind(self, tensors):
        self.decay = tensors[f"{self.prefix}.decay"]
        self.out = tensors[f"{self.prefix}.out.weight"]

    def cache_spec(self):
        grid = self.spec.params.get("grid")
        return FixedState((self.hidden,), torch.float64) if grid else FixedState((self.hidden,))

    def forward(self, x, step, cache):
        grid = self.spec.params.get("grid")
        if grid:
            assert cache.state.dtype == torch.float64
            lens = [b - a for a, b in zip(step.h_q_start[:-1], step.h_q_start[1:])]
            # single tokens take the recurrent form anywhere; a portion must start on the grid
            assert all(p % grid == 0 for p, n in zip(step.h_start_pos, lens) if n > 1), \
                f"a portion starts off the grid of {grid}: {step.h_start_pos}"
        a = torch.sigmoid(self.decay.float() * 50.0).to(cache.state.dtype)
        rows = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        for i in range(step.num_seqs):
            s = cache.state[step.h_state_slots[i]].clone()
            for t in range(step.h_q_start[i], step.h_q_start[i + 1]):
                s = a * s + x[t].to(s.dtype)
                rows[t] = s
            cache.state[step.h_state_slots[i]] = s
        return self.env.ops.linear(rows.to(x.dtype), self.out, self.env.dtype)


class NarrowValueAttention(Mixer):
    """One attention head with keys of ``k_dim`` and values of ``v_dim`` columns, cached in
    float32 whatever the compute type: plain tensor code over the step's block table."""

    graph_safe = False

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.k_dim, self.v_dim, self.prefix = p["hidden_size"], p["k_dim"], p["v_dim"], p["prefix"]

    def tensor_specs(self):
        return [TensorSpec(f"{self.prefix}.q.weight", (self.k_dim, self.hidden)), TensorSpec(f"{self.prefix}.k.weight", (self.k_dim, self.hidden)),
                TensorSpec(f"{self.prefix}.v.weight", (self.v_dim, self.hidden)), TensorSpec(f"{self.prefix}.o.weight", (self.hidden, self.v_dim))]

    def bind(self, tensors):
        self.w = {n: tensors[f"{self.prefix}.{n}.weight"] for n in "qkvo"}

    def cache_spec(self):
        return PagedKV(1, self.k_dim, v_head_dim=self.v_dim, dtype=torch.float32)

    def forward(self, x, step, cache):
        ops, page = self.env.ops, cache.page_size
        assert cache.k.shape[-1] == self.k_dim and cache.v.shape[-1] == self.v_dim and cache.k.dtype == torch.float32
        q, k, v = (ops.linear(x, self.w[n], torch.float32) for n in "qkv")
        table = step.block_tables[cache.group].long()
        pos, seq = step.positions.long(), step.seq_of_token.long()
        rows = table[seq, pos // page] * page + pos % page
        keys, values = cache.k.view(-1, self.k_dim), cache.v.view(-1, self.v_dim)
        keys[rows], values[rows] = k, v
        out = torch.empty((x.shape[0], self.v_dim), dtype=torch.float32, device=x.device)
        for t in range(x.shape[0]):
            span = torch.arange(int(pos[t]) + 1, device=x.device)
            seen = table[seq[t], span // page] * page + span % page
            weights = torch.softmax(keys[seen].double() @ q[t].double() * 0.5, 0)
            out[t] = (weights @ values[seen].double()).float()
        return ops.linear(out.to(x.dtype), self.w["o"], self.env.dtype)


class SegmentBias(Mixer):
    """A mixer that reads a further per-row input of the step: ``W x + table[segment]`` with the
    row's ``segment`` taken from ``step.extras["segment"]`` (modulo the table's rows)."""

    graph_safe = False

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden, self.rows, self.prefix = spec.params["hidden_size"], spec.params["rows"], spec.params["prefix"]

    def tensor_specs(self):
        return [TensorSpec(f"{self.prefix}.w.weight", (self.hidden, self.hidden)), TensorSpec(f"{self.prefix}.table.weight", (self.rows, self.hidden))]

    def bind(self, tensors):
        self.w, self.table = tensors[f"{self.prefix}.w.weight"], tensors[f"{self.prefix}.table.weight"]

    def forward(self, x, step, cache):
        segment = step.extras["segment"].long() % self.rows
        return (self.env.ops.linear(x, self.w, torch.float32) + self.table[segment].float()).to(x.dtype)


class RoutedFF(FeedForward):
    graph_safe = False

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden, self.experts, self.prefix = spec.params["hidden_size"], spec.params["experts"], spec.params["prefix"]

    def tensor_specs(self):
        specs = [TensorSpec(f"{self.prefix}.router.weight", (self.experts, self.hidden))]
        specs += [TensorSpec(f"{self.prefix}.expert{e}.weight", (self.hidden, self.hidden)) for e in range(self.experts)]
        return specs

    def bind(self, tensors):
        self.router = tensors[f"{self.prefix}.router.weight"]
        self.expert = [tensors[f"{self.prefix}.expert{e}.weight"] for e in range(self.experts)]

    def forward(self, x, step):
        ops = self.env.ops
        choice = ops.linear(x, self.router, torch.float32).argmax(-1)  # router logits in 32-bit
        out = torch.zeros_like(x)
        for e in range(self.experts):
            rows = torch.nonzero(choice == e).flatten()
            if rows.numel():
                out[rows] = ops.linear(x[rows].contiguous(), self.expert[e], self.env.dtype)
        return out


class RopeLinear(PositionEncoding):
    def __init__(self, spec, env, head_dim):
        super().__init__(spec, env)
        self.interleaved = bool(spec.params.get("interleaved", False))
        self.rotary_dim = spec.params["rotary_dim"]
        n = self.rotary_dim // 2
        self.inv_freq = (spec.params["top"] * (1.0 - torch.arange(n, dtype=torch.float64) / n)).float().to(env.device)

    def rotary(self):
        return self.inv_freq, self.rotary_dim


def register():
    MIXERS.register("decay_sum", DecaySum)
    MIXERS.register("narrow_value_attention", NarrowValueAttention)
    MIXERS.register("segment_bias", SegmentBias)
    FEED_FORWARDS.register("routed_ff", RoutedFF)
    POSITION_ENCODINGS.register("rope_linear", RopeLinear)


def unregister():
    MIXERS.unregister("decay_sum")
    MIXERS.unregister("narrow_value_attention")
    MIXERS.unregister("segment_bias")
    FEED_FORWARDS.unregister("routed_ff")
    POSITION_ENCODINGS.unregister("rope_linear")


HIDDEN, VOCAB, HEADS, KV_HEADS, HEAD_DIM, ROT, EPS, WINDOW = 48, 80, 3, 1, 16, 8, 1e-5, 6


def toy_plan() -> ModelPlan:
    """Layer 0: decay_sum + SwiGLU.  Layer 1: attention (partial linear-ladder rotation, a
    window) + routed_ff.  Layer 2: attention that borrows a cache.  Run order: 0, 1, 0 again
    (same weights, a second state of its own), 2 reading the cache that entry 1 wrote."""

    def norm(name, size=HIDDEN):
        return PartSpec("rmsnorm", {"tensor": name, "size": size, "eps": EPS})

    def attention(prefix, borrows):
        return PartSpec("gqa_attention", {
            "hidden_size": HIDDEN, "num_heads": HEADS, "num_kv_heads": KV_HEADS, "head_dim": HEAD_DIM,
            "scale": 0.3, "window": WINDOW, "borrows_cache": borrows,
            "q_proj": f"{prefix}.q.weight", "k_proj": f"{prefix}.k.weight", "v_proj": f"{prefix}.v.weight",
            "out_proj": f"{prefix}.o.weight",
            "q_norm": norm(f"{prefix}.qn.weight", HEAD_DIM), "k_norm": None if borrows else norm(f"{prefix}.kn.weight", HEAD_DIM),
            "position": PartSpec("rope_linear", {"rotary_dim": ROT, "top": 0.7, "interleaved": True}),
        })

    layers = (
        LayerSpec("l0", PartSpec("pre_norm"), PartSpec("decay_sum", {"hidden_size": HIDDEN, "prefix": "l0.mix"}), norm("l0.n1.weight"),
                  PartSpec("swiglu", {"hidden_size": HIDDEN, "intermediate_size": 40, "gate": "l0.g.weight", "up": "l0.u.weight", "down": "l0.d.weight"}),
                  norm("l0.n2.weight")),
        LayerSpec("l1", PartSpec("pre_norm"), attention("l1.attn", False), norm("l1.n1.weight"),
                  PartSpec("routed_ff", {"hidden_size": HIDDEN, "experts": 3, "prefix": "l1.ff"}), norm("l1.n2.weight")),
        LayerSpec("l2", PartSpec("pre_norm"), attention("l2.attn", True), norm("l2.n1.weight"), None, None),
    )
    return ModelPlan(
        architecture="ToyForCausalLM", hidden_size=HIDDEN, vocab_size=VOCAB,
        embedding=PartSpec("token_embedding", {"tensor": "emb.weight", "vocab_size": VOCAB, "hidden_size": HIDDEN}),
        layers=layers,
        order=(RunEntry(0), RunEntry(1), RunEntry(0), RunEntry(2, cache_of=1)),
        final_norm=norm("final.weight"),
        head=PartSpec("linear_head", {"vocab_size": VOCAB, "hidden_size": HIDDEN, "tied_to": "emb.weight", "tensor": None}),
    )


def toy_reference(w, ids):
    """The toy model over one whole sequence in float64, no cache."""
    w = {k: v.double() for k, v in w.items()}
    T = len(ids)
    pos = torch.arange(T)

    def rms(x, name):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + EPS) * w[name]

    def rotate(v):
        n = ROT // 2
        inv = (0.7 * (1.0 - torch.arange(n, dtype=torch.float64) / n)).float()
        angle = (pos.float()[:, None] * inv[None, :]).double()
        c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        out = v.clone()
        a, b = v[..., 0:ROT:2], v[..., 1:ROT:2]  # neighbours form a pair
        out[..., 0:ROT:2], out[..., 1:ROT:2] = a * c - b * s, a * s + b * c
        return out

    def decay_sum(n):
        a = torch.sigmoid(w["l0.mix.decay"].float() * 50.0).double()
        s, rows = torch.zeros(HIDDEN, dtype=torch.float64), []
        for t in range(T):
            s = a * s + n[t]
            rows.append(s)
        return torch.stack(rows) @ w["l0.mix.out.weight"].T

    kv = {}

    def attention(n, p, borrows):
        q = rotate(rms((n @ w[f"{p}.q.weight"].T).reshape(T, HEADS, HEAD_DIM), f"{p}.qn.weight"))
        if not borrows:
            k = rotate(rms((n @ w[f"{p}.k.weight"].T).reshape(T, KV_HEADS, HEAD_DIM), f"{p}.kn.weight"))
            kv["k"], kv["v"] = k, (n @ w[f"{p}.v.weight"].T).reshape(T, KV_HEADS, HEAD_DIM)
        k, v = kv["k"], kv["v"]
        out = torch.zeros(T, HEADS, HEAD_DIM, dtype=torch.float64)
        ok = (pos[None, :] <= pos[:, None]) & (pos[None, :] > pos[:, None] - WINDOW)
        for h in range(HEADS):
            s = (q[:, h] @ k[:, 0].T * 0.3).masked_fill(~ok, float("-inf"))
            out[:, h] = torch.softmax(s, -1) @ v[:, 0]
        return out.reshape(T, -1) @ w[f"{p}.o.weight"].T

    def swiglu(n):
        g, u = n @ w["l0.g.weight"].T, n @ w["l0.u.weight"].T
        return (g / (1 + torch.exp(-g)) * u) @ w["l0.d.weight"].T

    def routed(n):
        choice = (n @ w["l1.ff.router.weight"].T).argmax(-1)
        return torch.stack([n[t] @ w[f"l1.ff.expert{int(choice[t])}.weight"].T for t in range(T)])

    x = w["emb.weight"][torch.as_tensor(ids)]
    for layer in (0, 1, 0):
        if layer == 0:
            h = x + decay_sum(rms(x, "l0.n1.weight"))
            x = h + swiglu(rms(h, "l0.n2.weight"))
        else:
            h = x + attention(rms(x, "l1.n1.weight"), "l1.attn", False)
            x = h + routed(rms(h, "l1.n2.weight"))
    x = x + attention(rms(x, "l2.n1.weight"), "l2.attn", True)
    return rms(x, "final.weight") @ w["emb.weight"].T


GRID, K_DIM, V_DIM = 4, 12, 5


def grid_plan() -> ModelPlan:
    """Layer 0: decay_sum that insists on portions starting on a grid of 4 and keeps float64
    state + SwiGLU.  Layer 1: an attention head with values narrower than keys in a float32
    cache, no feed-forward.  The plan names the grid; the scheduler cuts prompts on it."""

    def norm(name, size=HIDDEN):
        return PartSpec("rmsnorm", {"tensor": name, "size": size, "eps": EPS})

    layers = (
        LayerSpec("l0", PartSpec("pre_norm"), PartSpec("decay_sum", {"hidden_size": HIDDEN, "prefix": "l0.mix", "grid": GRID}),
                  norm("l0.n1.weight"),
                  PartSpec("swiglu", {"hidden_size": HIDDEN, "intermediate_size": 40, "gate": "l0.g.weight", "up": "l0.u.weight", "down": "l0.d.weight"}),
                  norm("l0.n2.weight")),
        LayerSpec("l1", PartSpec("pre_norm"),
                  PartSpec("narrow_value_attention", {"hidden_size": HIDDEN, "k_dim": K_DIM, "v_dim": V_DIM, "prefix": "l1.attn"}),
                  norm("l1.n1.weight"), None, None),
    )
    return ModelPlan(
        architecture="ToyGridForCausalLM", hidden_size=HIDDEN, vocab_size=VOCAB,
        embedding=PartSpec("token_embedding", {"tensor": "emb.weight", "vocab_size": VOCAB, "hidden_size": HIDDEN}),
        layers=layers, order=(RunEntry(0), RunEntry(1)), final_norm=norm("final.weight"),
        head=PartSpec("linear_head", {"vocab_size": VOCAB, "hidden_size": HIDDEN, "tied_to": "emb.weight", "tensor": None}),
        portion_multiple=GRID,
    )


def grid_reference(w, ids):
    """The grid model over one whole sequence in float64, no cache."""
    w = {k: v.double() for k, v in w.items()}
    T = len(ids)

    def rms(x, name):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + EPS) * w[name]

    x = w["emb.weight"][torch.as_tensor(ids)]
    n = rms(x, "l0.n1.weight")
    a = torch.sigmoid(w["l0.mix.decay"].float() * 50.0).double()
    s, rows = torch.zeros(HIDDEN, dtype=torch.float64), []
    for t in range(T):
        s = a * s + n[t]
        rows.append(s)
    h = x + torch.stack(rows) @ w["l0.mix.out.weight"].T
    n = rms(h, "l0.n2.weight")
    g, u = n @ w["l0.g.weight"].T, n @ w["l0.u.weight"].T
    x = h + (g / (1 + torch.exp(-g)) * u) @ w["l0.d.weight"].T
    n = rms(x, "l1.n1.weight")
    q, k, v = (n @ w[f"l1.attn.{m}.weight"].T for m in "qkv")
    scores = (q @ k.T * 0.5).masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
    x = x + (torch.softmax(scores, -1) @ v) @ w["l1.attn.o.weight"].T
    return rms(x, "final.weight") @ w["emb.weight"].T


SEGMENTS = 5


def segment_plan() -> ModelPlan:
    """One layer whose mixer reads a further per-row input, ``segment``, that the plan names."""

    def norm(name):
        return PartSpec("rmsnorm", {"tensor": name, "size": HIDDEN, "eps": EPS})

    layers = (LayerSpec("l0", PartSpec("pre_norm"), PartSpec("segment_bias", {"hidden_size": HIDDEN, "rows": SEGMENTS, "prefix": "l0.mix"}),
                        norm("l0.n1.weight"), None, None),)
    return ModelPlan(
        architecture="ToySegmentForCausalLM", hidden_size=HIDDEN, vocab_size=VOCAB,
        embedding=PartSpec("token_embedding", {"tensor": "emb.weight", "vocab_size": VOCAB, "hidden_size": HIDDEN}),
        layers=layers, order=(RunEntry(0),), final_norm=norm("final.weight"),
        head=PartSpec("linear_head", {"vocab_size": VOCAB, "hidden_size": HIDDEN, "tied_to": "emb.weight", "tensor": None}),
        row_inputs=("segment",),
    )


def segment_reference(w, ids, segments):
    w = {k: v.double() for k, v in w.items()}

    def rms(x, name):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + EPS) * w[name]

    x = w["emb.weight"][torch.as_tensor(ids)]
    x = x + rms(x, "l0.n1.weight") @ w["l0.mix.w.weight"].T + w["l0.mix.table.weight"][torch.as_tensor(segments) % SEGMENTS]
    return rms(x, "final.weight") @ w["emb.weight"].T
