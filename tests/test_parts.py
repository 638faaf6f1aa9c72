"""Each part of a layer alone against the plain function of the same name, at sizes other than the
engine tests use; and toy parts defined here (a mixer with state of its own, a feed-forward with
routing, another position encoding) that are registered, built into models and stepped without any
change to the package."""
import math

import pytest
import torch

import plain_model as pm
from llmengine_b200.config import ARCHITECTURES, EngineConfig, register_architecture
from llmengine_b200.config.spec import LayerRun, LayerSpec, ModelSpec, PartSpec
from llmengine_b200.engine.engine import Engine, StepEntry
from llmengine_b200.parts import Part, Runtime, StateSpec, WeightSpec, build_part, register_part, registered
from llmengine_b200.weights import random_tensor

DEV = "cuda:0"


def _ops():
    from llmengine_b200.kernels.ops import CudaOps
    return CudaOps(torch.device(DEV))


def _load_random(part, seed, dtype):
    tensors = {}
    for n, s in part.weight_specs().items():
        t = random_tensor(n, s, seed)
        tensors[n] = t.to(dtype if s.role == "matrix" else torch.float32).to(DEV)
    part.load_weights(tensors)
    return {n: t.float().cpu() for n, t in tensors.items()}


# ----------------------------------------------------------------------------- parts alone (GPU)
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    rt = Runtime(_ops(), torch.device(DEV), dtype, 64)
    norm = build_part("norm", PartSpec("rmsnorm", {"size": 200, "eps": 2e-5}), rt, "n")
    w = _load_random(norm, 1, dtype)
    x = torch.randn(11, 200, device=DEV)
    delta = torch.randn(11, 200, device=DEV)
    want = pm.rms_norm((x + delta).cpu(), w["n.weight"], 2e-5)
    got = norm.forward(x, delta=delta)
    assert got.dtype == dtype
    assert (got.float().cpu() - want).abs().max() < (1e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.gpu
def test_position_part_table_matches_the_plain_rotation():
    rt = Runtime(_ops(), torch.device(DEV), torch.float32, 64)
    pe = build_part("position", PartSpec("rope", {"head_dim": 48, "theta": 77777.0, "max_positions": 300}), rt, "p")
    q = torch.randn(9, 5 * 48, device=DEV)
    k = torch.randn(9, 2 * 48, device=DEV)
    pos = torch.tensor([0, 1, 2, 50, 51, 120, 250, 298, 299], dtype=torch.int32, device=DEV)
    want_q = pm.rope(q.cpu().view(9, 5, 48), pos.cpu(), 77777.0).reshape(9, -1)
    want_k = pm.rope(k.cpu().view(9, 2, 48), pos.cpu(), 77777.0).reshape(9, -1)
    pe.apply(q, k, pos, 5, 2)                      # the unfused form, in place
    assert (q.cpu() - want_q).abs().max() < 2e-5 and (k.cpu() - want_k).abs().max() < 2e-5
    none = build_part("position", PartSpec("none"), rt, "p")
    assert none.rotary_table() is None


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    rt = Runtime(_ops(), torch.device(DEV), dtype, 64)
    ffn = build_part("feed_forward", PartSpec("swiglu", {"hidden_size": 72, "intermediate_size": 200}), rt, "f")
    w = _load_random(ffn, 2, dtype)
    h = torch.randn(13, 72, device=DEV).to(dtype)
    hf = h.float().cpu()
    want = pm.linear(pm.swiglu(pm.linear(hf, w["f.gate_proj.weight"]), pm.linear(hf, w["f.up_proj.weight"])),
                     w["f.down_proj.weight"])
    got = ffn.forward(h, None)
    assert got.dtype == torch.float32
    assert (got.cpu() - want).abs().max() < (1e-6 if dtype == torch.float32 else 2e-4)


@pytest.mark.gpu
def test_embedding_and_head_parts():
    rt = Runtime(_ops(), torch.device(DEV), torch.float32, 64)
    emb = build_part("embedding", PartSpec("token_embedding", {"vocab_size": 333, "hidden_size": 40}), rt, "e")
    w = _load_random(emb, 3, torch.float32)
    ids = torch.tensor([0, 332, 17, 17], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(ids).cpu(), pm.embedding(w["e.weight"], ids.tolist()))
    head = build_part("head", PartSpec("lm_head", {"vocab_size": 333, "hidden_size": 40, "tied": True}), rt, "h")
    assert head.weight_specs() == {}
    head.tie(emb.table)
    h = torch.randn(3, 40, device=DEV)
    assert (head.forward(h).cpu() - pm.linear(h.cpu(), w["e.weight"])).abs().max() < 1e-5


def _one_layer_engine(tmp_path, dtype, **mixer_over):
    from helpers import make_model_dir
    cfg = {"architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 1, "hidden_size": 56, "num_attention_heads": 6,
           "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 88, "vocab_size": 301, "rope_theta": 3000.0,
           "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 128, "hidden_act": "silu"}
    d = make_model_dir(str(tmp_path / "one"), cfg, 4, dtype="bfloat16", sharpen=2.0)
    ec = EngineConfig(dtype=dtype, page_size=4, max_cached_tokens=128, max_num_seqs=4, max_num_batched_tokens=128,
                      use_cuda_graphs=False)
    return Engine(d, engine_config=ec), pm.PlainQwen3(d, round_to=torch.bfloat16 if dtype == "bfloat16" else None), cfg


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixer_part_alone_over_two_steps(tmp_path, dtype):
    """The attention part's forward on hand-made inputs: a first portion, then a second one that must
    find the first one's keys in the cache."""
    eng, plain, cfg = _one_layer_engine(tmp_path, dtype)
    mixer = eng.model.blocks[0].mixer
    T1, T2, H = 21, 10, cfg["hidden_size"]
    h_all = torch.randn(T1 + T2, H).to(eng.dtype)
    hf = h_all.float()
    w = plain.w
    p = "model.layers.0.self_attn."
    rt = plain.round_to
    r = (lambda x: x.to(rt).float()) if rt else (lambda x: x)
    nh, nkv, hd = 6, 2, 32
    pos = torch.arange(T1 + T2)
    q = r(pm.rope(pm.qk_norm(r(pm.linear(hf, w[p + "q_proj.weight"])).view(-1, nh, hd), w[p + "q_norm.weight"], 1e-5), pos, 3000.0))
    k = r(pm.rope(pm.qk_norm(r(pm.linear(hf, w[p + "k_proj.weight"])).view(-1, nkv, hd), w[p + "k_norm.weight"], 1e-5), pos, 3000.0))
    v = r(pm.linear(hf, w[p + "v_proj.weight"])).view(-1, nkv, hd)
    want = pm.linear(r(pm.attention(q, k, v).reshape(-1, nh * hd)), w[p + "o_proj.weight"])
    got = []
    for start, n in ((0, T1), (T1, T2)):
        eng.cache.has("x") or eng.cache.add_request("x")
        eng.cache.reserve("x", start + n)
        batch = eng._build_batch([StepEntry("x", [0] * n, [])], [start])
        eng.cache.flush()
        got.append(mixer.forward(h_all[start:start + n].to(DEV).contiguous(), batch, eng._caches[0]).cpu().clone())
        eng.cache.advance("x", start + n)
        eng.steps += 1
    got = torch.cat(got)
    assert (got - want).abs().max() < (2e-5 if dtype == "float32" else 2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_part_alone(tmp_path, dtype):
    eng, plain, cfg = _one_layer_engine(tmp_path, dtype)
    block = eng.model.blocks[0]
    T, H = 17, cfg["hidden_size"]
    x0 = torch.randn(T, H)
    d0 = torch.randn(T, H) * 0.1
    # plain: one layer body on x = x0 + d0
    rt = plain.round_to
    r = (lambda t: t.to(rt).float()) if rt else (lambda t: t)
    w, p = plain.w, "model.layers.0."
    x = x0 + d0
    h = r(pm.rms_norm(x, w[p + "input_layernorm.weight"], 1e-5))
    pos = torch.arange(T)
    q = r(pm.rope(pm.qk_norm(r(pm.linear(h, w[p + "self_attn.q_proj.weight"])).view(T, 6, 32), w[p + "self_attn.q_norm.weight"], 1e-5), pos, 3000.0))
    k = r(pm.rope(pm.qk_norm(r(pm.linear(h, w[p + "self_attn.k_proj.weight"])).view(T, 2, 32), w[p + "self_attn.k_norm.weight"], 1e-5), pos, 3000.0))
    v = r(pm.linear(h, w[p + "self_attn.v_proj.weight"])).view(T, 2, 32)
    x = pm.linear(r(pm.attention(q, k, v).reshape(T, -1)), w[p + "self_attn.o_proj.weight"]) + x
    h = r(pm.rms_norm(x, w[p + "post_attention_layernorm.weight"], 1e-5))
    f = pm.linear(r(pm.swiglu(r(pm.linear(h, w[p + "mlp.gate_proj.weight"])), r(pm.linear(h, w[p + "mlp.up_proj.weight"])))),
                  w[p + "mlp.down_proj.weight"])
    eng.cache.add_request("x")
    eng.cache.reserve("x", T)
    batch = eng._build_batch([StepEntry("x", [0] * T, [])], [0])
    eng.cache.flush()
    xg, dg = block.forward(x0.to(DEV), d0.to(DEV), batch, eng._caches[0])
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert (xg.cpu() - x).abs().max() < tol, "the residual stream after the mixer"
    assert (dg.cpu() - f).abs().max() < tol, "the feed-forward's contribution, not yet added"


# ----------------------------------------------------------------------------- a toy mixer with state
@register_part("mixer", "toy_decaying_sum")
class ToyDecayingSum(Part):
    """y_t = W s_t with s_t = decay * s_{t-1} + h_t: a state of fixed size per request, carried from
    one portion to the next through the request's state slot.  Written with plain tensor operations;
    it exists only to show that a mixer of another kind plugs in."""

    capture_safe = False          # reads slot numbers on the host

    def __init__(self, rt, prefix, hidden_size, decay):
        super().__init__(rt, prefix)
        self.hidden, self.decay = hidden_size, decay
        self.w = None

    def weight_specs(self):
        return {self.name("mix.weight"): WeightSpec((self.hidden, self.hidden))}

    def load_weights(self, t):
        self.w = t[self.name("mix.weight")].float()

    def cache_spec(self):
        return StateSpec((self.hidden,), torch.float32)

    def forward(self, h, batch, cache):
        out = torch.empty(h.shape[0], self.hidden, dtype=torch.float32, device=h.device)
        slots = batch.state_slots.tolist()
        a = 0
        for r, n in enumerate(batch.q_lens):                 # a request's portion is processed in order
            s = cache.state[slots[r]]
            if batch.start_positions[r] == 0:
                assert float(s.abs().max()) == 0.0, "a new request must find a zeroed state"
            for t in range(a, a + n):
                s = self.decay * s + h[t].float()
                out[t] = self.w @ s
            cache.state[slots[r]] = s
            a += n
        return out


class ToyConfig:
    """An architecture made of the toy mixer and the package's other parts."""

    ARCHITECTURE = "ToyStateForCausalLM"

    def __init__(self, d):
        self.d = dict(d)
        self.vocab_size, self.hidden_size = d["vocab_size"], d["hidden_size"]
        self.tie_word_embeddings = False
        self.eos_token_id = None

    @classmethod
    def from_dict(cls, d):
        return cls(d)

    def to_dict(self):
        return dict(self.d)

    @staticmethod
    def canonical_tensor_name(n):
        return n

    def model_spec(self):
        H, d = self.hidden_size, self.d
        norm = PartSpec("rmsnorm", {"size": H, "eps": d["eps"]})
        attn = PartSpec("gqa_attention", {"hidden_size": H, "num_heads": 4, "num_kv_heads": 1, "head_dim": 16,
                                          "qk_norm_eps": None, "window": 0, "position_encoding": PartSpec("none")})
        toy = PartSpec("toy_decaying_sum", {"hidden_size": H, "decay": d["decay"]})
        ffn = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": d["inter"]})
        layers = tuple(LayerSpec(f"layers.{i}", PartSpec("prenorm_residual"), m, norm, ffn, norm)
                       for i, m in enumerate((toy, attn, toy)))
        return ModelSpec(self.ARCHITECTURE, H, self.vocab_size, d["max_positions"],
                         PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": H}), layers,
                         tuple(LayerRun(i) for i in range(3)), norm,
                         PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": H}))


if ToyConfig.ARCHITECTURE not in ARCHITECTURES:
    register_architecture(ToyConfig.ARCHITECTURE, ToyConfig)

TOY = {"architectures": [ToyConfig.ARCHITECTURE], "vocab_size": 97, "hidden_size": 40, "inter": 72, "eps": 1e-5,
       "decay": 0.9, "max_positions": 256}


def _plain_toy(eng, ids):
    """Whole-sequence evaluation of the toy model from the engine's loaded tensors, with plain functions."""
    m = eng.model
    f = lambda t: t.float().cpu()
    x = pm.embedding(f(m.embedding.table), ids)
    T = len(ids)
    for blk in m.blocks:
        h = pm.rms_norm(x, f(blk.mixer_norm.gain), blk.mixer_norm.eps)
        if isinstance(blk.mixer, ToyDecayingSum):
            s = torch.zeros(h.shape[1])
            rows = []
            for t in range(T):
                s = 0.9 * s + h[t]
                rows.append(f(blk.mixer.w) @ s)
            a = torch.stack(rows)
        else:
            mx = blk.mixer
            qkv = pm.linear(h, f(mx.w_qkv))
            q = qkv[:, :mx.q_size].view(T, mx.nh, mx.hd)
            k = qkv[:, mx.q_size:mx.q_size + mx.kv_size].view(T, mx.nkv, mx.hd)
            v = qkv[:, mx.q_size + mx.kv_size:].view(T, mx.nkv, mx.hd)
            a = pm.linear(pm.attention(q, k, v).reshape(T, -1), f(mx.w_o))
        x = x + a
        h = pm.rms_norm(x, f(blk.ffn_norm.gain), blk.ffn_norm.eps)
        gu = pm.linear(h, f(blk.ffn.w_gate_up))
        x = x + pm.linear(pm.swiglu(gu[:, :blk.ffn.inter], gu[:, blk.ffn.inter:]), f(blk.ffn.w_down))
    return pm.linear(pm.rms_norm(x, f(m.final_norm.gain), m.final_norm.eps), f(m.head.weight))


def _toy_roundtrip(ops, device):
    assert "toy_decaying_sum" in registered("mixer")
    ec = EngineConfig(dtype="float32", page_size=8, max_cached_tokens=256, max_num_seqs=3, max_num_batched_tokens=128,
                      device=device, use_cuda_graphs=False)
    eng = Engine(config=TOY, random_seed=5, engine_config=ec, ops=ops)
    assert [type(s).__name__ for s, _ in eng.model.cache_specs()] == ["StateSpec", "PagedKVSpec", "StateSpec"]
    from helpers import random_ids
    a, b = random_ids(50, 97, 1), random_ids(31, 97, 2)
    want_a, want_b = _plain_toy(eng, a), _plain_toy(eng, b)
    # whole
    got = eng.step([StepEntry("a", a, range(50))], end=["a"]).cpu()
    assert (got - want_a).abs().max() < 1e-4
    # portions of a beside b, b starting later and decoding one by one at the end; then a slot is used again
    rows_a, rows_b = [], []
    sched = [(("a", 0, 20),), (("a", 20, 2), ("b", 0, 17)), (("b", 17, 13), ("a", 22, 27)), (("a", 49, 1), ("b", 30, 1))]
    for step in sched:
        entries = [StepEntry(r, (a if r == "a" else b)[s:s + n], range(n)) for r, s, n in step]
        out = eng.step(entries).cpu()
        o = 0
        for r, s, n in step:
            (rows_a if r == "a" else rows_b).append(out[o:o + n].clone())
            o += n
    assert (torch.cat(rows_a) - want_a).abs().max() < 1e-4
    assert (torch.cat(rows_b) - want_b).abs().max() < 1e-4
    eng.free("a"), eng.free("b")
    got = eng.step([StepEntry("c", b, range(31))], end=["c"]).cpu()      # finds its slot's state zeroed again
    assert (got - want_b).abs().max() < 1e-4
    eng.cache.check_invariants()


def test_toy_stateful_mixer_on_the_host():
    from host_ops import HostOps
    _toy_roundtrip(HostOps(), "cpu")


@pytest.mark.gpu
def test_toy_stateful_mixer_registers_builds_and_steps():
    _toy_roundtrip(None, DEV)


# ----------------------------------------------------------------------------- a toy feed-forward with routing, a toy position encoding
@register_part("feed_forward", "toy_top1_experts")
class ToyTop1Experts(Part):
    """r = softmax(Wr h) (32-bit), e = argmax r, y = r_e * W2_e relu(W1_e h): every token goes to one of
    several small two-layer experts.  Plain tensor operations; it exists only to show that a feed-forward
    with routing plugs in (and that its result does not depend on which other tokens share the step)."""

    capture_safe = False          # gathers rows by expert on the host

    def __init__(self, rt, prefix, hidden_size, inter, experts):
        super().__init__(rt, prefix)
        self.hidden, self.inter, self.experts = hidden_size, inter, experts
        self.router = self.w1 = self.w2 = None

    def weight_specs(self):
        s = {self.name("router.weight"): WeightSpec((self.experts, self.hidden))}
        for e in range(self.experts):
            s[self.name(f"experts.{e}.w1.weight")] = WeightSpec((self.inter, self.hidden))
            s[self.name(f"experts.{e}.w2.weight")] = WeightSpec((self.hidden, self.inter))
        return s

    def load_weights(self, t):
        self.router = t[self.name("router.weight")].float() * 40.0      # (N(0, 0.02) weights: make the choice decisive)
        self.w1 = [t[self.name(f"experts.{e}.w1.weight")].float() for e in range(self.experts)]
        self.w2 = [t[self.name(f"experts.{e}.w2.weight")].float() for e in range(self.experts)]

    @staticmethod
    def route(h, router, w1, w2):
        r = torch.softmax(h.float() @ router.t(), dim=-1)
        choice = r.argmax(dim=-1)
        out = torch.zeros(h.shape[0], w2[0].shape[0], dtype=torch.float32, device=h.device)
        for e in range(len(w1)):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                y = torch.relu(h[rows].float() @ w1[e].t()) @ w2[e].t()
                out[rows] = r[rows, e, None] * y
        return out, choice

    def forward(self, h, batch):
        return self.route(h, self.router, self.w1, self.w2)[0]


@register_part("position", "toy_interleaved_rotation")
class ToyInterleavedRotation(Part):
    """Rotates the pairs (2d, 2d+1) of every head by pos * base^(-d): another pairing and another angle than
    the package's rotary part, applied through the unfused path (no table for the fused kernel)."""

    def __init__(self, rt, prefix, head_dim, base):
        super().__init__(rt, prefix)
        self.head_dim, self.base = head_dim, base

    def rotary_table(self):
        return None

    @staticmethod
    def rotate(x, positions, head_dim, base):
        T = x.shape[0]
        v = x.float().view(T, -1, head_dim // 2, 2)
        d = torch.arange(head_dim // 2, dtype=torch.float32, device=x.device)
        ang = positions.to(x.device).float()[:, None] * torch.pow(torch.tensor(float(base), device=x.device), -d)[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        out = torch.stack([v[..., 0] * c - v[..., 1] * s, v[..., 0] * s + v[..., 1] * c], dim=-1)
        return out.view(T, -1)

    def apply(self, q, k, positions, num_heads, num_kv_heads):
        q.copy_(self.rotate(q, positions, self.head_dim, self.base).to(q.dtype))
        if k is not None:
            k.copy_(self.rotate(k, positions, self.head_dim, self.base).to(k.dtype))


class ToyRoutedConfig(ToyConfig):
    """Attention with the toy position encoding, and the routed feed-forward in every second layer."""

    ARCHITECTURE = "ToyRoutedForCausalLM"

    def model_spec(self):
        H, d = self.hidden_size, self.d
        norm = PartSpec("rmsnorm", {"size": H, "eps": d["eps"]})
        pos = PartSpec("toy_interleaved_rotation", {"head_dim": d["head_dim"], "base": d["base"]})
        attn = PartSpec("gqa_attention", {"hidden_size": H, "num_heads": d["heads"], "num_kv_heads": d["kv_heads"],
                                          "head_dim": d["head_dim"], "qk_norm_eps": d["eps"], "window": 0,
                                          "position_encoding": pos})
        dense = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": d["inter"]})
        routed = PartSpec("toy_top1_experts", {"hidden_size": H, "inter": d["expert_inter"], "experts": d["experts"]})
        layers = tuple(LayerSpec(f"layers.{i}", PartSpec("prenorm_residual"), attn, norm, f, norm)
                       for i, f in enumerate((routed, dense, routed)))
        return ModelSpec(self.ARCHITECTURE, H, self.vocab_size, d["max_positions"],
                         PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": H}), layers,
                         tuple(LayerRun(i) for i in range(3)), norm,
                         PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": H}))


if ToyRoutedConfig.ARCHITECTURE not in ARCHITECTURES:
    register_architecture(ToyRoutedConfig.ARCHITECTURE, ToyRoutedConfig)

TOY_ROUTED = {"architectures": [ToyRoutedConfig.ARCHITECTURE], "vocab_size": 113, "hidden_size": 48, "inter": 56,
              "eps": 1e-5, "heads": 6, "kv_heads": 2, "head_dim": 16, "base": 50.0, "experts": 3, "expert_inter": 40,
              "max_positions": 256}


def _plain_toy_routed(eng, ids):
    """Whole-sequence evaluation from the engine's loaded tensors with plain functions; also returns how many
    tokens every expert of the first layer got."""
    m = eng.model
    f = lambda t: t.float().cpu()
    x = pm.embedding(f(m.embedding.table), ids)
    T = len(ids)
    pos = torch.arange(T)
    counts = None
    for blk in m.blocks:
        mx = blk.mixer
        h = pm.rms_norm(x, f(blk.mixer_norm.gain), blk.mixer_norm.eps)
        qkv = pm.linear(h, f(mx.w_qkv))
        q = pm.rms_norm(qkv[:, :mx.q_size].reshape(T * mx.nh, mx.hd), f(mx.q_gain), mx.eps).view(T, -1)
        k = pm.rms_norm(qkv[:, mx.q_size:mx.q_size + mx.kv_size].reshape(T * mx.nkv, mx.hd), f(mx.k_gain), mx.eps).view(T, -1)
        v = qkv[:, mx.q_size + mx.kv_size:].view(T, mx.nkv, mx.hd)
        q = ToyInterleavedRotation.rotate(q, pos, mx.hd, mx.position.base).view(T, mx.nh, mx.hd)
        k = ToyInterleavedRotation.rotate(k, pos, mx.hd, mx.position.base).view(T, mx.nkv, mx.hd)
        x = x + pm.linear(pm.attention(q, k, v).reshape(T, -1), f(mx.w_o))
        h = pm.rms_norm(x, f(blk.ffn_norm.gain), blk.ffn_norm.eps)
        if isinstance(blk.ffn, ToyTop1Experts):
            y, choice = ToyTop1Experts.route(h, f(blk.ffn.router), [f(w) for w in blk.ffn.w1], [f(w) for w in blk.ffn.w2])
            if counts is None:
                counts = torch.bincount(choice, minlength=blk.ffn.experts)
            x = x + y
        else:
            gu = pm.linear(h, f(blk.ffn.w_gate_up))
            x = x + pm.linear(pm.swiglu(gu[:, :blk.ffn.inter], gu[:, blk.ffn.inter:]), f(blk.ffn.w_down))
    return pm.linear(pm.rms_norm(x, f(m.final_norm.gain), m.final_norm.eps), f(m.head.weight)), counts


def _toy_routed_roundtrip(ops, device):
    assert "toy_top1_experts" in registered("feed_forward") and "toy_interleaved_rotation" in registered("position")
    ec = EngineConfig(dtype="float32", page_size=8, max_cached_tokens=192, max_num_seqs=3, max_num_batched_tokens=128,
                      device=device, use_cuda_graphs=False)
    eng = Engine(config=TOY_ROUTED, random_seed=11, engine_config=ec, ops=ops)
    from helpers import random_ids
    a, b = random_ids(61, 113, 3), random_ids(40, 113, 4)
    (want_a, counts), (want_b, _) = _plain_toy_routed(eng, a), _plain_toy_routed(eng, b)
    assert int((counts > 0).sum()) >= 2, "the routing must use more than one expert for the test to mean anything"
    got = eng.step([StepEntry("a", a, range(61))], end=["a"]).cpu()
    assert (got - want_a).abs().max() < 2e-4
    # portions of a beside b and single tokens: a token's expert and result must not depend on its companions
    rows_a, rows_b = [], []
    sched = [(("a", 0, 23),), (("a", 23, 2), ("b", 0, 19)), (("b", 19, 20), ("a", 25, 35)), (("a", 60, 1), ("b", 39, 1))]
    for step in sched:
        entries = [StepEntry(r, (a if r == "a" else b)[s:s + n], range(n)) for r, s, n in step]
        out = eng.step(entries).cpu()
        o = 0
        for r, s, n in step:
            (rows_a if r == "a" else rows_b).append(out[o:o + n].clone())
            o += n
    assert (torch.cat(rows_a) - want_a).abs().max() < 2e-4
    assert (torch.cat(rows_b) - want_b).abs().max() < 2e-4
    eng.free("a"), eng.free("b")
    eng.cache.check_invariants()


def test_toy_routed_feed_forward_and_position_encoding_on_the_host():
    from host_ops import HostOps
    _toy_routed_roundtrip(HostOps(), "cpu")


@pytest.mark.gpu
def test_toy_routed_feed_forward_and_position_encoding_register_build_and_step():
    _toy_routed_roundtrip(None, DEV)


# ----------------------------------------------------------------------------- a cache kind and a block shape of their own
class SplitKVSpec:
    """A paged cache whose keys and values have different widths: one row [key | value] per position.  Defined
    here, outside the package: the cache manager and the engine only use the protocol (paged, window, allocate,
    bytes_per_token, view)."""

    paged, window = True, 0

    def __init__(self, key_dim, value_dim):
        self.key_dim, self.value_dim = key_dim, value_dim

    def __eq__(self, other):
        return isinstance(other, SplitKVSpec) and (self.key_dim, self.value_dim) == (other.key_dim, other.value_dim)

    def allocate(self, count, page_size, dtype, device):
        return torch.zeros(count, page_size, self.key_dim + self.value_dim, dtype=torch.float32, device=device)

    def bytes_per_token(self, dtype):
        return 4 * (self.key_dim + self.value_dim)

    def view(self, tensor, group, writes):
        return {"rows": tensor, "group": group}


@register_part("mixer", "toy_split_kv_attention")
class ToySplitKVAttention(Part):
    """One-head causal attention with keys of width `key_dim` and values of another width `value_dim`, kept in
    a cache of its own layout.  Plain tensor operations; it exists only to show that a mixer with another kind
    of cache plugs in."""

    capture_safe = False

    def __init__(self, rt, prefix, hidden_size, key_dim, value_dim):
        super().__init__(rt, prefix)
        self.hidden, self.dk, self.dv = hidden_size, key_dim, value_dim

    def weight_specs(self):
        return {self.name("q.weight"): WeightSpec((self.dk, self.hidden)), self.name("k.weight"): WeightSpec((self.dk, self.hidden)),
                self.name("v.weight"): WeightSpec((self.dv, self.hidden)), self.name("o.weight"): WeightSpec((self.hidden, self.dv))}

    def load_weights(self, t):
        self.wq, self.wk, self.wv, self.wo = (t[self.name(n + ".weight")].float() * 8.0 for n in "qkvo")

    def cache_spec(self):
        return SplitKVSpec(self.dk, self.dv)

    @staticmethod
    def attend(q, k, v):
        T = q.shape[0]
        s = (q @ k.t()) / math.sqrt(q.shape[1])
        n = k.shape[0]
        mask = torch.arange(n, device=q.device)[None, :] > (torch.arange(T, device=q.device)[:, None] + (n - T))
        return torch.softmax(s.masked_fill(mask, float("-inf")), -1) @ v

    def forward(self, h, batch, cache):
        g = batch.groups[cache["group"]]
        rows = cache["rows"].view(-1, self.dk + self.dv)
        hf = h.float()
        q, k, v = hf @ self.wq.t(), hf @ self.wk.t(), hf @ self.wv.t()
        rows[g.slot_mapping.long()] = torch.cat([k, v], dim=1)
        out = torch.empty(h.shape[0], self.dv, device=h.device)
        tables, slots = g.block_tables.cpu(), batch.state_slots.tolist()
        a = 0
        for r, n in enumerate(batch.q_lens):
            ctx = batch.start_positions[r] + n
            pos = torch.arange(ctx)
            where = (tables[slots[r]][pos // g.page_size].long() * g.page_size + pos % g.page_size).to(h.device)
            kv = rows[where]
            out[a:a + n] = self.attend(q[a:a + n], kv[:, :self.dk], kv[:, self.dk:])
            a += n
        return out @ self.wo.t()


@register_part("block", "toy_postnorm")
class ToyPostNormBlock(Part):
    """x = norm(x + mixer(x)): a norm after the residual sum, no feed-forward.  It reads the parts "mixer" and
    "post_norm" of its layer: another set of roles than the package's block has."""

    capture_safe = False

    def __init__(self, rt, prefix, layer):
        super().__init__(rt, prefix)
        self.mixer = build_part("mixer", layer.parts["mixer"], rt, self.name("mixer"))
        self.post_norm = build_part("norm", layer.parts["post_norm"], rt, self.name("post_norm"))

    def weight_specs(self):
        return {**self.mixer.weight_specs(), **self.post_norm.weight_specs()}

    def load_weights(self, t):
        for p in (self.mixer, self.post_norm):
            p.load_weights({n: t[n] for n in p.weight_specs()})

    def cache_spec(self):
        return self.mixer.cache_spec()

    def forward(self, x, delta, batch, cache):
        if delta is not None:
            x += delta.float()
        y = x + self.mixer.forward(x.to(self.rt.dtype), batch, cache)
        x.copy_(self.post_norm.forward(y).float())        # the package's norm part, run by itself
        return x, None


class ToySplitConfig(ToyConfig):
    ARCHITECTURE = "ToySplitKVForCausalLM"

    def model_spec(self):
        H, d = self.hidden_size, self.d
        norm = PartSpec("rmsnorm", {"size": H, "eps": d["eps"]})
        split = PartSpec("toy_split_kv_attention", {"hidden_size": H, "key_dim": d["key_dim"], "value_dim": d["value_dim"]})
        attn = PartSpec("gqa_attention", {"hidden_size": H, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16,
                                          "qk_norm_eps": d["eps"], "window": 0,
                                          "position_encoding": PartSpec("rope", {"head_dim": 16, "theta": 100.0,
                                                                                  "max_positions": d["max_positions"]})})
        ffn = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": d["inter"]})
        layers = (LayerSpec("layers.0", PartSpec("toy_postnorm"), parts={"mixer": split, "post_norm": norm}),
                  LayerSpec("layers.1", PartSpec("prenorm_residual"), attn, norm, ffn, norm),
                  LayerSpec("layers.2", PartSpec("toy_postnorm"), parts={"mixer": split, "post_norm": norm}))
        return ModelSpec(self.ARCHITECTURE, H, self.vocab_size, d["max_positions"],
                         PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": H}), layers,
                         tuple(LayerRun(i) for i in range(3)), norm,
                         PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": H,
                                              "tied_to": "embedding.weight"}))


if ToySplitConfig.ARCHITECTURE not in ARCHITECTURES:
    register_architecture(ToySplitConfig.ARCHITECTURE, ToySplitConfig)

TOY_SPLIT = {"architectures": [ToySplitConfig.ARCHITECTURE], "vocab_size": 101, "hidden_size": 32, "inter": 48, "eps": 1e-5,
             "key_dim": 24, "value_dim": 8, "max_positions": 256}


def _plain_toy_split(eng, ids):
    m = eng.model
    f = lambda t: t.float().cpu()
    x = pm.embedding(f(m.embedding.table), ids)
    T = len(ids)
    for blk in m.blocks:
        if isinstance(blk, ToyPostNormBlock):
            mx = blk.mixer
            q, k, v = x @ f(mx.wq).t(), x @ f(mx.wk).t(), x @ f(mx.wv).t()
            x = pm.rms_norm(x + ToySplitKVAttention.attend(q, k, v) @ f(mx.wo).t(), f(blk.post_norm.gain), blk.post_norm.eps)
        else:
            mx = blk.mixer
            h = pm.rms_norm(x, f(blk.mixer_norm.gain), blk.mixer_norm.eps)
            qkv = pm.linear(h, f(mx.w_qkv))
            pos = torch.arange(T)
            q = pm.rope(pm.qk_norm(qkv[:, :mx.q_size].view(T, mx.nh, mx.hd), f(mx.q_gain), mx.eps), pos, 100.0)
            k = pm.rope(pm.qk_norm(qkv[:, mx.q_size:mx.q_size + mx.kv_size].view(T, mx.nkv, mx.hd), f(mx.k_gain), mx.eps), pos, 100.0)
            v = qkv[:, mx.q_size + mx.kv_size:].view(T, mx.nkv, mx.hd)
            x = x + pm.linear(pm.attention(q, k, v).reshape(T, -1), f(mx.w_o))
            h = pm.rms_norm(x, f(blk.ffn_norm.gain), blk.ffn_norm.eps)
            gu = pm.linear(h, f(blk.ffn.w_gate_up))
            x = x + pm.linear(pm.swiglu(gu[:, :blk.ffn.inter], gu[:, blk.ffn.inter:]), f(blk.ffn.w_down))
    return pm.linear(pm.rms_norm(x, f(m.final_norm.gain), m.final_norm.eps), f(m.head.weight))


def _toy_split_roundtrip(ops, device):
    from helpers import random_ids, replay, trace_mixed, trace_portions, trace_whole, max_live_tokens
    reqs = {f"r{i}": random_ids(n, 101, 20 + i) for i, n in enumerate([40, 9, 66, 23])}
    steps_by = {"whole": trace_whole(reqs), "portions": trace_portions(reqs, sizes=(16, 3, 2, 9, 1)),
                "mixed": trace_mixed(reqs, {r: max(1, len(v) - 6) for r, v in reqs.items()}, max_live=3, seed=2)}
    want = None
    for what, steps in steps_by.items():
        pool = max_live_tokens(steps, 8)
        ec = EngineConfig(dtype="float32", page_size=8, max_cached_tokens=pool, max_num_seqs=4, max_num_batched_tokens=pool,
                          device=device, use_cuda_graphs=False)
        eng = Engine(config=TOY_SPLIT, random_seed=31, engine_config=ec, ops=ops)
        assert eng.model.head.weight.data_ptr() == eng.model.embedding.table.data_ptr()      # tied through the spec
        assert [type(s).__name__ for s, _ in eng.model.cache_specs()] == ["SplitKVSpec", "PagedKVSpec", "SplitKVSpec"]
        assert eng.cache.kv[0].shape[1:] == (8, 32) and eng.cache.kv[1].shape[1:] == (2, 2, 8, 16)
        if want is None:
            want = {r: _plain_toy_split(eng, ids) for r, ids in reqs.items()}
        got = replay(eng, steps)
        for r in reqs:
            assert (got[r].cpu() - want[r]).abs().max() < 2e-4, (what, r)
        eng.cache.check_invariants()
        assert not eng.cache.requests


def test_toy_cache_kind_and_block_shape_on_the_host():
    from host_ops import HostOps
    _toy_split_roundtrip(HostOps(), "cpu")


@pytest.mark.gpu
def test_toy_cache_kind_and_block_shape_register_build_and_replay():
    _toy_split_roundtrip(None, DEV)
