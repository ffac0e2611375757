"""Each part alone against the plain implementation, the schedule as data (a layer run twice, a
run that reads another run's cache), and a toy mixer with state of its own that is registered,
built from a model folder and stepped without any change to the library's files."""
import json
import math
import os
from dataclasses import dataclass, replace

import numpy as np
import pytest
import torch

from tests.conftest import TEST_SCALES, tiny_configs
from tests.plain import qwen3_plain as P

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {torch.float32: 2e-5, torch.bfloat16: 2e-2}


def rel(got, ref):
    got = got.double().cpu().numpy() if isinstance(got, torch.Tensor) else got
    return float(np.max(np.abs(got - ref)) / np.max(np.abs(ref)))


@pytest.fixture(scope="module")
def rt():
    from gophonic_b200.engine.model import make_runtime
    return {torch.float32: make_runtime("float32", DEV), torch.bfloat16: make_runtime("bfloat16", DEV)}


def layer_tensors(model_dirs, name, dtype):
    from gophonic_b200.weights import declare_model, load_tensors
    cfg = tiny_configs()[name]
    mode = "float32" if dtype == torch.float32 else "bfloat16"
    return cfg, load_tensors(model_dirs[name], declare_model(cfg.model_spec()), mode, DEV)


def one_plane_cache(spec_mixer, dtype, max_tokens=512):
    from gophonic_b200 import registry
    from gophonic_b200.cache import Cache
    req = registry.part_class("mixer", spec_mixer.kind).cache_request(spec_mixer)
    return Cache([(req, None)], max_tokens, DEV, dtype)


def whole_batch(cache, lens):
    from gophonic_b200.engine import build_batch
    slots = [cache.alloc_slot() for _ in lens]
    cache.reserve([(s, n) for s, n in zip(slots, lens)])
    batch, _ = build_batch([(s, [0] * n, 0) for s, n in zip(slots, lens)], DEV)
    return batch, slots


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(rt, dtype):
    from gophonic_b200.config import RMSNormSpec
    from gophonic_b200.parts import RMSNorm
    w = (1 + 0.1 * torch.randn(72)).to(DEV)
    part = RMSNorm(RMSNormSpec(72, 1e-5), "n.", {"n.weight": w.to(torch.bfloat16 if dtype == torch.bfloat16 else dtype)}, rt[dtype])
    wv = part.weight.double().cpu().numpy()
    h, d = torch.randn(5, 72, device=DEV), torch.randn(5, 72, device=DEV)
    out = torch.empty((5, 72), dtype=dtype, device=DEV)
    h0 = h.clone()
    part.forward(h, out, d)
    ref_h = h0.double().cpu().numpy() + d.double().cpu().numpy()
    assert rel(h, ref_h) < 1e-6
    assert rel(out, P.rms_norm(ref_h, wv, 1e-5)) < (1e-5 if dtype == torch.float32 else 1e-2)
    assert [t.name for t in RMSNorm.declare(RMSNormSpec(72, 1e-5), "n.")] == ["n.weight"]


def test_rotary_tables(rt):
    from gophonic_b200.config import RotarySpec
    from gophonic_b200.parts import RotaryEmbedding
    part = RotaryEmbedding(RotarySpec(48, 32, 50000.0), "", {}, rt[torch.float32])
    part.prepare(300)
    cos, sin, rot = part.kernel_args()
    c, s = P.rope_tables(np.arange(300), 32, 50000.0)
    assert rot == 32 and cos.shape == (300, 16)
    assert np.array_equal(cos.cpu().numpy(), c.astype(np.float32)) and np.array_equal(sin.cpu().numpy(), s.astype(np.float32))
    with pytest.raises(ValueError):
        RotaryEmbedding(RotarySpec(48, 50, 1e4), "", {}, rt[torch.float32])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_attention_part(rt, model_dirs, plain_models, name, dtype):
    from gophonic_b200.parts import Attention
    cfg, tensors = layer_tensors(model_dirs, name, dtype)
    pcfg, pw = plain_models[name]
    spec = cfg.model_spec().layers[0].mixer
    part = Attention(spec, "model.layers.0.self_attn.", tensors, rt[dtype])
    cache = one_plane_cache(spec, dtype)
    part.prepare(512)
    lens = [70, 3, 131]
    batch, slots = whole_batch(cache, lens)
    x = torch.randn(sum(lens), cfg.hidden_size, device=DEV).to(dtype)
    out = torch.empty((sum(lens), cfg.hidden_size), dtype=torch.float32, device=DEV)
    part.forward(batch, x, out, cache.view(0))
    r = 0
    for n in lens:
        ref = P.attention_block(x[r:r + n].double().cpu().numpy(), pw, "model.layers.0.self_attn.", pcfg, np.arange(n))
        assert rel(out[r:r + n], ref) < TOL[dtype]
        r += n
    names = [t.name for t in Attention.declare(spec, "p.")]
    assert names == ["p.q_proj.weight", "p.k_proj.weight", "p.v_proj.weight", "p.o_proj.weight", "p.q_norm.weight",
                     "p.k_norm.weight"]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_part_with_a_window_and_partial_rotation(rt, model_dirs, plain_models, dtype):
    """The same part with other constants: a window of 40 and rotation of half of each head."""
    from gophonic_b200.config import RotarySpec
    from gophonic_b200.parts import Attention
    cfg, tensors = layer_tensors(model_dirs, "B", dtype)
    pcfg, pw = plain_models["B"]
    base = cfg.model_spec().layers[0].mixer
    spec = replace(base, window=40, position=RotarySpec(base.head_dim, base.head_dim // 2, 777.0))
    part = Attention(spec, "model.layers.0.self_attn.", tensors, rt[dtype])
    cache = one_plane_cache(spec, dtype)
    assert cache.groups()[0]["window"] == 40
    part.prepare(512)
    n = 150
    batch, _ = whole_batch(cache, [n])
    x = torch.randn(n, cfg.hidden_size, device=DEV).to(dtype)
    out = torch.empty((n, cfg.hidden_size), dtype=torch.float32, device=DEV)
    part.forward(batch, x, out, cache.view(0))
    # plain: the same formulas with the other constants
    p = "model.layers.0.self_attn."
    xs = x.double().cpu().numpy()
    d, nh, nkv = base.head_dim, base.heads, base.kv_heads
    q = P.rms_norm((xs @ pw[p + "q_proj.weight"].T).reshape(n, nh, d), pw[p + "q_norm.weight"], pcfg["rms_norm_eps"])
    k = P.rms_norm((xs @ pw[p + "k_proj.weight"].T).reshape(n, nkv, d), pw[p + "k_norm.weight"], pcfg["rms_norm_eps"])
    v = (xs @ pw[p + "v_proj.weight"].T).reshape(n, nkv, d)
    c, s = P.rope_tables(np.arange(n), d // 2, 777.0)
    ctx = P.causal_attention(P.apply_rope(q, c, s), P.apply_rope(k, c, s), v, 1 / math.sqrt(d), window=40)
    ref = ctx.reshape(n, -1) @ pw[p + "o_proj.weight"].T
    assert rel(out, ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_swiglu_part(rt, model_dirs, plain_models, name, dtype):
    from gophonic_b200.parts import SwiGLU
    cfg, tensors = layer_tensors(model_dirs, name, dtype)
    _, pw = plain_models[name]
    part = SwiGLU(cfg.model_spec().layers[0].feed_forward, "model.layers.0.mlp.", tensors, rt[dtype])
    x = torch.randn(37, cfg.hidden_size, device=DEV).to(dtype)
    out = torch.empty((37, cfg.hidden_size), dtype=torch.float32, device=DEV)
    part.forward(None, x, out)
    assert rel(out, P.swiglu_ffn(x.double().cpu().numpy(), pw, "model.layers.0.mlp.")) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prenorm_block(rt, model_dirs, plain_models, dtype):
    from gophonic_b200.parts import PreNormBlock
    cfg, tensors = layer_tensors(model_dirs, "B", dtype)
    pcfg, pw = plain_models["B"]
    layer = cfg.model_spec().layers[1]
    block = PreNormBlock(layer, layer.prefix, tensors, rt[dtype])
    cache = one_plane_cache(layer.mixer, dtype)
    block.mixer.prepare(512)
    n = 45
    batch, _ = whole_batch(cache, [n])
    h = torch.randn(n, cfg.hidden_size, device=DEV)
    pending = torch.randn(n, cfg.hidden_size, device=DEV)
    h0 = h.double().cpu().numpy() + pending.double().cpu().numpy()
    delta = block.forward(batch, h, pending, cache.view(0))
    ref = P.decoder_layer(h0, pw, 1, pcfg, np.arange(n))
    assert rel(h + delta, ref) < TOL[dtype]  # the block hands its feed-forward output on as the pending addend


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_schedule_runs_a_layer_twice_and_shares_a_cache(model_dirs, plain_models, dtype):
    """Order of layers is data: [0, 1, 1, 0 reading the keys and values of its first run]."""
    from gophonic_b200.config import ScheduleEntry
    from gophonic_b200.engine import Engine, Model
    from gophonic_b200.engine.model import make_runtime
    from gophonic_b200.weights import declare_model, load_tensors
    cfg = tiny_configs()["A"]
    pcfg, pw = plain_models["A"]
    mode = "float32" if dtype == torch.float32 else "bfloat16"
    spec = replace(cfg.model_spec(), schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1), ScheduleEntry(0, cache_of=0)))
    rt = make_runtime(mode, DEV)
    model = Model(spec, load_tensors(model_dirs["A"], declare_model(spec), mode, DEV), rt, cfg)
    eng = Engine(model, max_tokens=512)
    groups = eng.cache.groups()
    assert len(groups) == 1 and groups[0]["planes"] == [0, 1, 2]  # three planes: the fourth run borrows the first
    toks = np.random.default_rng(3).integers(0, cfg.vocab_size, size=80).tolist()
    slot = eng.new_sequence()
    got = [eng.step([(slot, toks[:50])], [list(range(50))]).cpu().numpy()]
    for t in toks[50:]:
        got.append(eng.step([(slot, [t])], [[0]]).cpu().numpy())
    got = np.concatenate(got, 0)
    # plain
    n, eps = len(toks), pcfg["rms_norm_eps"]
    d, nh, nkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    pos = np.arange(n)
    h = P.embed(toks, pw["model.embed_tokens.weight"])
    p0 = "model.layers.0."
    x0 = P.rms_norm(h, pw[p0 + "input_layernorm.weight"], eps)
    c, s = P.rope_tables(pos, d, pcfg["rope_theta"])
    k0 = P.apply_rope(P.rms_norm((x0 @ pw[p0 + "self_attn.k_proj.weight"].T).reshape(n, nkv, d), pw[p0 + "self_attn.k_norm.weight"], eps), c, s)
    v0 = (x0 @ pw[p0 + "self_attn.v_proj.weight"].T).reshape(n, nkv, d)
    h = P.decoder_layer(h, pw, 0, pcfg, pos)
    h = P.decoder_layer(h, pw, 1, pcfg, pos)
    h = P.decoder_layer(h, pw, 1, pcfg, pos)
    x = P.rms_norm(h, pw[p0 + "input_layernorm.weight"], eps)
    q = P.apply_rope(P.rms_norm((x @ pw[p0 + "self_attn.q_proj.weight"].T).reshape(n, nh, d), pw[p0 + "self_attn.q_norm.weight"], eps), c, s)
    ctx = P.causal_attention(q, k0, v0, 1 / math.sqrt(d))
    h = h + ctx.reshape(n, -1) @ pw[p0 + "self_attn.o_proj.weight"].T
    h = h + P.swiglu_ffn(P.rms_norm(h, pw[p0 + "post_attention_layernorm.weight"], eps), pw, p0 + "mlp.")
    ref = P.rms_norm(h, pw["model.norm.weight"], eps) @ P.head_weight(pw).T
    assert rel(got, ref) < TOL[dtype]


# ---- a toy mixer with state of its own, defined here and nowhere else ----------------------------
@dataclass(frozen=True)
class EmaSpec:
    hidden: int
    decay: float
    kind: str = "toy-ema"


def _toy_parts():
    from gophonic_b200.parts.base import Mixer, StateRequest, TensorDecl

    class EmaMixer(Mixer):
        """s_t = decay * s_{t-1} + (1 - decay) * (x_t W^T); out_t = s_t.  Its per-sequence state is
        the running s (fixed size), carried across steps in the cache's state area."""

        @classmethod
        def declare(cls, spec, prefix):
            return [TensorDecl(prefix + "mix.weight", (spec.hidden, spec.hidden))]

        @classmethod
        def cache_request(cls, spec):
            return StateRequest((spec.hidden,), torch.float32)

        def __init__(self, spec, prefix, tensors, runtime):
            self.spec, self.rt = spec, runtime
            self.w = tensors[prefix + "mix.weight"].float()

        def forward(self, batch, x, out, cache):
            y = x.float() @ self.w.T
            a = self.spec.decay
            for slot, start, n in zip(batch.seq_slot.tolist(), batch.seq_q_start.tolist(), batch.seq_q_len.tolist()):
                s = cache.state[slot].clone()
                for r in range(start, start + n):
                    s = a * s + (1 - a) * y[r]
                    out[r] = s
                cache.state[slot] = s
    return EmaMixer


@dataclass(frozen=True)
class ToyConfig:
    hidden_size: int
    num_hidden_layers: int
    intermediate_size: int
    vocab_size: int
    decay: float
    rms_norm_eps: float
    max_position_embeddings: int = 4096
    tie_word_embeddings: bool = True

    @classmethod
    def from_dict(cls, d):
        return cls(d["hidden_size"], d["num_hidden_layers"], d["intermediate_size"], d["vocab_size"], d["decay"],
                   d["rms_norm_eps"])

    def to_dict(self):
        return {"architectures": ["ToyEmaForCausalLM"], "model_type": "toy_ema", "hidden_size": self.hidden_size,
                "num_hidden_layers": self.num_hidden_layers, "intermediate_size": self.intermediate_size,
                "vocab_size": self.vocab_size, "decay": self.decay, "rms_norm_eps": self.rms_norm_eps,
                "tie_word_embeddings": True}

    def model_spec(self):
        from gophonic_b200.config import (EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, RMSNormSpec, SwiGLUSpec,
                                          default_schedule)
        layers = tuple(LayerSpec(prefix=f"toy.layers.{i}.", mixer=EmaSpec(self.hidden_size, self.decay),
                                 feed_forward=SwiGLUSpec(self.hidden_size, self.intermediate_size),
                                 mixer_norm=RMSNormSpec(self.hidden_size, self.rms_norm_eps),
                                 feed_forward_norm=RMSNormSpec(self.hidden_size, self.rms_norm_eps),
                                 mixer_prefix="ema.", feed_forward_prefix="ffn.", mixer_norm_prefix="norm1.",
                                 feed_forward_norm_prefix="norm2.")
                       for i in range(self.num_hidden_layers))
        return ModelSpec("ToyEmaForCausalLM", self.hidden_size, self.vocab_size, self.max_position_embeddings,
                         EmbeddingSpec("toy.embed.weight", self.vocab_size, self.hidden_size), layers,
                         default_schedule(self.num_hidden_layers), RMSNormSpec(self.hidden_size, self.rms_norm_eps),
                         "toy.norm.weight", HeadSpec("toy.head.weight", self.vocab_size, self.hidden_size,
                                                     tied_to="toy.embed.weight"))


def toy_plain(toks, cfg: ToyConfig, w):
    h = P.embed(toks, w["toy.embed.weight"])
    for i in range(cfg.num_hidden_layers):
        p = f"toy.layers.{i}."
        y = P.rms_norm(h, w[p + "norm1.weight"], cfg.rms_norm_eps) @ w[p + "ema.mix.weight"].T
        s = np.zeros(cfg.hidden_size)
        mixed = np.zeros_like(y)
        for t in range(len(toks)):
            s = cfg.decay * s + (1 - cfg.decay) * y[t]
            mixed[t] = s
        h = h + mixed
        h = h + P.swiglu_ffn(P.rms_norm(h, w[p + "norm2.weight"], cfg.rms_norm_eps), w, p + "ffn.")
    return P.rms_norm(h, w["toy.norm.weight"], cfg.rms_norm_eps) @ w["toy.embed.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path, dtype):
    from gophonic_b200 import registry
    from gophonic_b200.engine import Engine, Model
    from gophonic_b200.weights import InitScales, write_random_model
    registry.register_mixer("toy-ema", _toy_parts())
    registry.register_architecture("ToyEmaForCausalLM", ToyConfig, model_type="toy_ema")
    cfg = ToyConfig(hidden_size=48, num_hidden_layers=2, intermediate_size=72, vocab_size=97, decay=0.8, rms_norm_eps=1e-5)
    d = str(tmp_path / "toy")
    write_random_model(cfg, 3, d, scales=InitScales(**TEST_SCALES))
    assert registry.read_config(d) == cfg
    model = Model.from_dir(d, dtype=dtype)
    eng = Engine(model, max_tokens=1024)
    kinds = [g["kind"] for g in eng.cache.groups()]
    assert kinds == ["state"] and eng.cache.groups()[0]["planes"] == [0, 1]
    _, w = P.read_model(d)
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, 97, size=n).tolist() for n in (30, 7, 19)]
    refs = [toy_plain(s, cfg, w) for s in seqs]
    tol = TOL[torch.float32 if dtype == "float32" else torch.bfloat16]
    for round_ in range(2):  # the second round reuses the slots: the state must start at zero again
        slots = [eng.new_sequence() for _ in seqs]
        cut = [10, 7, 1]
        first = eng.step([(sl, s[:c]) for sl, s, c in zip(slots, seqs, cut)], [list(range(c)) for c in cut]).cpu().numpy()
        got = [[first[sum(cut[:i]):sum(cut[:i + 1])]] for i in range(3)]
        step = 0
        while True:
            live = [i for i in range(3) if cut[i] + step < len(seqs[i])]
            if not live:
                break
            out = eng.step([(slots[i], [seqs[i][cut[i] + step]]) for i in live], [[0]] * len(live)).cpu().numpy()
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
            step += 1
        for i in range(3):
            assert rel(np.concatenate(got[i], 0), refs[i]) < tol, (round_, i)
            eng.end_sequence(slots[i])


# ---- a toy feed-forward with routing and a toy position encoding ----------------------------------
# Both are defined here, registered through the registry and used beside the built-in parts, layer
# by layer, without a change to the package.
@dataclass(frozen=True)
class Top1Spec:
    hidden: int
    experts: int
    inner: int
    kind: str = "toy-top1"


@dataclass(frozen=True)
class SlowRotarySpec:
    """Rotary angles of position / slowdown: another position encoding for the built-in attention."""
    head_dim: int
    rotary_dim: int
    theta: float
    slowdown: float
    kind: str = "toy-slow-rope"


def _routed_ffn():
    from gophonic_b200.parts.base import FeedForward, TensorDecl

    class Top1Experts(FeedForward):
        """Router logits in fp32, the single best expert per row (lowest index on ties), output =
        softmax weight of that expert times relu(x W1_e^T) W2_e^T.  Rows are grouped by expert
        inside forward."""

        @classmethod
        def declare(cls, spec, prefix):
            d = [TensorDecl(prefix + "router.weight", (spec.experts, spec.hidden))]
            for e in range(spec.experts):
                d += [TensorDecl(prefix + f"experts.{e}.w1.weight", (spec.inner, spec.hidden)),
                      TensorDecl(prefix + f"experts.{e}.w2.weight", (spec.hidden, spec.inner))]
            return d

        def __init__(self, spec, prefix, tensors, runtime):
            self.spec = spec
            self.router = tensors[prefix + "router.weight"].float()
            self.w1 = [tensors[prefix + f"experts.{e}.w1.weight"].float() for e in range(spec.experts)]
            self.w2 = [tensors[prefix + f"experts.{e}.w2.weight"].float() for e in range(spec.experts)]

        def forward(self, batch, x, out):
            xf = x.float()
            logits = xf @ self.router.T
            prob = torch.softmax(logits, dim=-1)
            best = torch.argmax(logits, dim=-1)
            out.zero_()
            for e in range(self.spec.experts):
                rows = torch.nonzero(best == e).flatten()
                if rows.numel():
                    y = torch.relu(xf[rows] @ self.w1[e].T) @ self.w2[e].T
                    out[rows] = y * prob[rows, e:e + 1]
    return Top1Experts


def _slow_rope():
    from gophonic_b200.parts.base import PositionEncoding

    class SlowRotary(PositionEncoding):
        def __init__(self, spec, prefix, tensors, runtime):
            self.spec, self.rt, self.capacity = spec, runtime, 0
            self.cos = self.sin = None

        def prepare(self, capacity):
            if capacity <= self.capacity:
                return
            rot = self.spec.rotary_dim
            inv = 1.0 / np.power(float(self.spec.theta), 2.0 * np.arange(rot // 2, dtype=np.float64) / rot)
            ang = (np.arange(capacity, dtype=np.float64) / self.spec.slowdown)[:, None] * inv[None, :]
            self.cos = torch.from_numpy(np.cos(ang).astype(np.float32)).to(self.rt.device)
            self.sin = torch.from_numpy(np.sin(ang).astype(np.float32)).to(self.rt.device)
            self.capacity = capacity

        def kernel_args(self):
            return self.cos, self.sin, self.spec.rotary_dim
    return SlowRotary


@dataclass(frozen=True)
class MixedConfig:
    """Layer 0: built-in attention with the toy position encoding and the built-in SwiGLU.
    Layer 1: built-in attention with the built-in rotary embedding and the toy routed feed-forward."""
    hidden_size: int
    heads: int
    kv_heads: int
    head_dim: int
    intermediate_size: int
    experts: int
    inner: int
    vocab_size: int
    theta: float
    slowdown: float
    rms_norm_eps: float
    max_position_embeddings: int = 2048

    @classmethod
    def from_dict(cls, d):
        return cls(*[d[k] for k in ("hidden_size", "heads", "kv_heads", "head_dim", "intermediate_size", "experts", "inner",
                                    "vocab_size", "theta", "slowdown", "rms_norm_eps")])

    def to_dict(self):
        d = {k: getattr(self, k) for k in ("hidden_size", "heads", "kv_heads", "head_dim", "intermediate_size", "experts", "inner",
                                           "vocab_size", "theta", "slowdown", "rms_norm_eps")}
        d.update(architectures=["ToyMixedForCausalLM"], model_type="toy_mixed")
        return d

    def model_spec(self):
        from gophonic_b200.config import (AttentionSpec, EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, RMSNormSpec, RotarySpec,
                                          SwiGLUSpec, default_schedule)
        norm = RMSNormSpec(self.hidden_size, self.rms_norm_eps)
        positions = [SlowRotarySpec(self.head_dim, self.head_dim, self.theta, self.slowdown), RotarySpec(self.head_dim, self.head_dim, self.theta)]
        ffns = [SwiGLUSpec(self.hidden_size, self.intermediate_size), Top1Spec(self.hidden_size, self.experts, self.inner)]
        layers = tuple(LayerSpec(prefix=f"m.layers.{i}.",
                                 mixer=AttentionSpec(self.hidden_size, self.heads, self.kv_heads, self.head_dim, self.head_dim ** -0.5,
                                                     positions[i], qk_norm=None),
                                 feed_forward=ffns[i], mixer_norm=norm, feed_forward_norm=norm, mixer_prefix="attn.",
                                 feed_forward_prefix="ffn.", mixer_norm_prefix="n1.", feed_forward_norm_prefix="n2.")
                       for i in range(2))
        return ModelSpec("ToyMixedForCausalLM", self.hidden_size, self.vocab_size, self.max_position_embeddings,
                         EmbeddingSpec("m.embed.weight", self.vocab_size, self.hidden_size), layers, default_schedule(2), norm,
                         "m.norm.weight", HeadSpec("m.head.weight", self.vocab_size, self.hidden_size, tied_to=None))


def mixed_plain(toks, cfg: MixedConfig, w):
    def attn(x, p, slowdown):
        T = len(toks)
        q = (x @ w[p + "q_proj.weight"].T).reshape(T, cfg.heads, cfg.head_dim)
        k = (x @ w[p + "k_proj.weight"].T).reshape(T, cfg.kv_heads, cfg.head_dim)
        v = (x @ w[p + "v_proj.weight"].T).reshape(T, cfg.kv_heads, cfg.head_dim)
        half = cfg.head_dim // 2
        inv = 1.0 / np.power(cfg.theta, 2.0 * np.arange(half) / cfg.head_dim)
        ang = (np.arange(T) / slowdown)[:, None] * inv[None, :]
        c, s = np.cos(ang).astype(np.float32).astype(np.float64)[:, None, :], np.sin(ang).astype(np.float32).astype(np.float64)[:, None, :]
        rot = lambda y: np.concatenate([y[..., :half] * c - y[..., half:] * s, y[..., half:] * c + y[..., :half] * s], -1)
        q, k = rot(q), rot(k)
        out = np.zeros((T, cfg.heads, cfg.head_dim))
        g = cfg.heads // cfg.kv_heads
        for h in range(cfg.heads):
            sc = (q[:, h] @ k[:, h // g].T) * cfg.head_dim ** -0.5
            sc = np.where(np.tril(np.ones((T, T), bool)), sc, -np.inf)
            pr = np.exp(sc - sc.max(-1, keepdims=True))
            out[:, h] = (pr / pr.sum(-1, keepdims=True)) @ v[:, h // g]
        return out.reshape(T, -1) @ w[p + "o_proj.weight"].T

    h = P.embed(toks, w["m.embed.weight"])
    for i in range(2):
        p = f"m.layers.{i}."
        h = h + attn(P.rms_norm(h, w[p + "n1.weight"], cfg.rms_norm_eps), p + "attn.", cfg.slowdown if i == 0 else 1.0)
        x = P.rms_norm(h, w[p + "n2.weight"], cfg.rms_norm_eps)
        if i == 0:
            h = h + P.swiglu_ffn(x, w, p + "ffn.")
        else:
            logits = x @ w[p + "ffn.router.weight"].T
            prob = np.exp(logits - logits.max(-1, keepdims=True))
            prob /= prob.sum(-1, keepdims=True)
            best = logits.argmax(-1)
            y = np.zeros_like(x)
            for t in range(len(toks)):
                e = best[t]
                y[t] = (np.maximum(x[t] @ w[p + f"ffn.experts.{e}.w1.weight"].T, 0) @ w[p + f"ffn.experts.{e}.w2.weight"].T) * prob[t, e]
            h = h + y
    return P.rms_norm(h, w["m.norm.weight"], cfg.rms_norm_eps) @ w["m.head.weight"].T


@pytest.mark.parametrize("dtype,experts", [("float32", 3), ("bfloat16", 1)])
def test_a_toy_routed_feed_forward_and_a_toy_position_encoding_layer_by_layer(tmp_path, dtype, experts):
    """Two layers whose parts differ: the registry builds each from its spec's kind, the loader and
    the random-weights writer work from the parts' declarations, the engine steps prompts and
    single tokens, and the logits are those of a plain restatement.  In 32-bit with three experts;
    in bfloat16 with one, where no choice can flip on rounding: there the built-in parts fold their
    norms into their products in single-token steps and the toy part, which does not, sits between
    them, and the attention kernel rotates by the toy encoding's tables itself."""
    from gophonic_b200 import registry
    from gophonic_b200.engine import Engine, Model
    from gophonic_b200.weights import InitScales, write_random_model
    registry.register_feed_forward("toy-top1", _routed_ffn())
    registry.register_position("toy-slow-rope", _slow_rope())
    registry.register_architecture("ToyMixedForCausalLM", MixedConfig, model_type="toy_mixed")
    cfg = MixedConfig(hidden_size=64, heads=4, kv_heads=2, head_dim=16, intermediate_size=96, experts=experts, inner=40, vocab_size=211,
                      theta=10000.0, slowdown=4.0, rms_norm_eps=1e-5)
    d = str(tmp_path / "mixed")
    write_random_model(cfg, 5, d, scales=InitScales(**TEST_SCALES))
    assert registry.read_config(d) == cfg
    model = Model.from_dir(d, dtype=dtype)
    assert not model.capturable  # the routed part reads device values on the host: steps run eagerly
    eng = Engine(model, max_tokens=1024)
    _, w = P.read_model(d)
    rng = np.random.default_rng(2)
    seqs = [rng.integers(0, 211, size=n).tolist() for n in (40, 9, 70)]
    refs = [mixed_plain(s, cfg, w) for s in seqs]
    slots = [eng.new_sequence() for _ in seqs]
    cut = [30, 9, 5]
    first = eng.step([(sl, s[:c]) for sl, s, c in zip(slots, seqs, cut)], [list(range(c)) for c in cut]).cpu().numpy()
    got = [[first[sum(cut[:i]):sum(cut[:i + 1])]] for i in range(3)]
    step = 0
    while True:
        live = [i for i in range(3) if cut[i] + step < len(seqs[i])]
        if not live:
            break
        out = eng.step([(slots[i], [seqs[i][cut[i] + step]]) for i in live], [[0]] * len(live)).cpu().numpy()
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1])
        step += 1
    for i in range(3):
        assert rel(np.concatenate(got[i], 0), refs[i]) < TOL[torch.float32 if dtype == "float32" else torch.bfloat16], i
        eng.end_sequence(slots[i])
    eng.cache.check()
