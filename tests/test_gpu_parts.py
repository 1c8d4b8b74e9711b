"""Each part alone on the GPU against the plain function for it, and a toy
mixer with state of its own that is registered, built and stepped without a
change to the package's files."""

import dataclasses
from dataclasses import dataclass

import pytest
import torch

import plain_llama
from helpers import assert_close, random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=3e-6, rtol=1e-5) if dtype is torch.float32 else dict(atol=3e-2, rtol=3e-2)


def close(got, want, dtype):
    """float32: element by element.  bfloat16: an output is a sum of many rounded terms, so its
    error is measured against the largest value of the tensor, as for the logits."""
    got, want = got.float().cpu(), want.float().cpu()
    if dtype is torch.float32:
        return torch.allclose(got, want, atol=3e-6, rtol=1e-5)
    return float((got - want).abs().max()) <= 2e-2 * max(1.0, float(want.abs().max()))


class Harness:
    """A runtime, a cache manager for the given mixers, and contexts for given cuts."""

    def __init__(self, dtype, requirements, page_size=8, n_pages=64, max_requests=4):
        from inf_engine_b200.cache import CacheManager
        from inf_engine_b200.parts import Runtime
        self.rt = Runtime(DEV, dtype)
        self.cache = CacheManager(requirements, page_size, n_pages, max_requests)
        self.cache.allocate_storage(DEV)

    def context(self, entries):
        """entries: [(rid, n_tokens)] — opens unknown requests, reserves, returns the StepContext."""
        from inf_engine_b200.engine import StepEntry, build_context
        es = []
        for rid, n in entries:
            if rid not in self.cache.slots:
                self.cache.open(rid)
            assert self.cache.reserve(rid, self.cache.lengths[rid] + n)
            es.append(StepEntry(rid, [0] * n, []))
        ctx = build_context(self.rt, self.cache, es)
        return ctx

    def advance(self, entries):
        for rid, n in entries:
            self.cache.advance(rid, self.cache.lengths[rid] + n)

    def view(self, entry=0, write=True):
        from inf_engine_b200.parts import CacheView
        b = self.cache.bindings[entry]
        if b.kind == "kv":
            g = self.cache.kv_groups[b.group]
            return CacheView("kv", b.group, g.k[b.row], g.v[b.row], None, write)
        g = self.cache.state_groups[b.group]
        return CacheView("state", b.group, None, None, g.data[b.row], write)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from inf_engine_b200.config import NormSpec
    from inf_engine_b200.parts import RMSNorm, Runtime
    torch.manual_seed(0)
    rt = Runtime(DEV, dtype)
    gain = (1 + 0.1 * torch.randn(200)).to(dtype)
    part = RMSNorm(NormSpec("rmsnorm", 200, 2e-6, "g"), {"g": gain.to(DEV)}, rt)
    assert RMSNorm.expected_tensors(part.spec)["g"].shape == (200,)
    res = torch.randn(11, 200, device=DEV)
    delta = torch.randn(11, 200, device=DEV).to(dtype)
    before = res.clone()
    out = part.add_norm(res, delta)
    want = plain_llama.rms_norm((before + delta.float()).cpu(), gain.float(), 2e-6)
    assert out.dtype is dtype and torch.allclose(out.float().cpu(), want, **tol(dtype))
    assert torch.equal(res, before + delta.float())


def test_rotary_part_shares_its_tables():
    from inf_engine_b200.config import PositionSpec, RopeScaling
    from inf_engine_b200.parts import Rotary, Runtime
    rt = Runtime(DEV, torch.float32)
    spec = PositionSpec("rotary", 48, 30000.0, 300, RopeScaling("llama3", 4.0, 1.0, 4.0, 32))
    a, b = Rotary(spec, {}, rt), Rotary(spec, {}, rt)
    assert a.cos.data_ptr() == b.cos.data_ptr() and a.cos.shape == (300, 24)
    cfg = dict(head_dim=48, hidden_size=48, num_attention_heads=1, rope_theta=30000.0,
               rope_scaling=dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                 original_max_position_embeddings=32))
    cos, sin = plain_llama.rope_tables(cfg, 300)
    assert torch.equal(a.cos.cpu(), cos[:, :24]) and torch.equal(a.sin.cpu(), sin[:, :24])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 10])
def test_attention_part_under_cuts(dtype, window):
    from inf_engine_b200.config import AttentionSpec, PositionSpec
    from inf_engine_b200.parts import PagedAttention
    torch.manual_seed(1)
    hidden, H, Hk, hd, T = 72, 6, 3, 16, 45
    spec = AttentionSpec(kind="attention", hidden=hidden, n_heads=H, n_kv_heads=Hk, head_dim=hd, window=window,
                         position=PositionSpec("rotary", hd, 10000.0, 128, None), q_proj="q", k_proj="k",
                         v_proj="v", o_proj="o")
    w = {"q": torch.randn(H * hd, hidden) * 0.2, "k": torch.randn(Hk * hd, hidden) * 0.2,
         "v": torch.randn(Hk * hd, hidden) * 0.2, "o": torch.randn(hidden, H * hd) * 0.2}
    w = {n: t.to(dtype) for n, t in w.items()}
    assert PagedAttention.expected_tensors(spec)["k"].shape == (Hk * hd, hidden)
    x = torch.randn(T, hidden).to(dtype)
    cfg = dict(hidden_size=hidden, num_attention_heads=H, num_key_value_heads=Hk, head_dim=hd, rope_theta=10000.0)
    cos, sin = plain_llama.rope_tables(cfg, T)
    want = plain_llama.attention(x.float(), *(w[n].float() for n in "qkvo"), cfg, cos, sin, window=window)
    for cuts in ([T], [7, 2, 1, 1, 20, 14]):
        from inf_engine_b200.cache import CacheRequirement
        h = Harness(dtype, [CacheRequirement(kind="kv", n_kv_heads=Hk, head_dim=hd, window=window, dtype=dtype)])
        part = PagedAttention(spec, {n: t.to(DEV) for n, t in w.items()}, h.rt)
        assert part.cache_requirement() == h.cache.kv_groups[0] and False or part.cache_requirement().window == window
        outs, p = [], 0
        for n in cuts:
            ctx = h.context([("r", n)])
            outs.append(part.forward(x[p:p + n].to(DEV), ctx, h.view()).float().cpu().clone())
            h.advance([("r", n)])
            p += n
        assert close(torch.cat(outs), want, dtype), f"cuts {cuts}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_mlp_part(dtype):
    from inf_engine_b200.config import GatedMLPSpec
    from inf_engine_b200.parts import GatedMLP, Runtime
    torch.manual_seed(2)
    rt = Runtime(DEV, dtype)
    spec = GatedMLPSpec(kind="gated_mlp", hidden=72, intermediate=200, gate_proj="g", up_proj="u", down_proj="d")
    w = {"g": torch.randn(200, 72) * 0.2, "u": torch.randn(200, 72) * 0.2, "d": torch.randn(72, 200) * 0.2}
    w = {n: t.to(dtype) for n, t in w.items()}
    part = GatedMLP(spec, {n: t.to(DEV) for n, t in w.items()}, rt)
    x = torch.randn(9, 72).to(dtype)
    want = plain_llama.swiglu(x.float(), w["g"].float(), w["u"].float(), w["d"].float())
    assert close(part.forward(x.to(DEV), None), want, dtype)


def test_gated_mlp_keeps_a_32bit_weight_in_32bit():
    """A tensor stored in 32-bit stays so on the bfloat16 path: the product with it runs in float32."""
    from inf_engine_b200.config import GatedMLPSpec
    from inf_engine_b200.parts import GatedMLP, Runtime
    torch.manual_seed(3)
    rt = Runtime(DEV, torch.bfloat16)
    spec = GatedMLPSpec(kind="gated_mlp", hidden=64, intermediate=96, gate_proj="g", up_proj="u", down_proj="d")
    w = {"g": (torch.randn(96, 64) * 0.2).bfloat16(), "u": (torch.randn(96, 64) * 0.2).bfloat16(),
         "d": torch.randn(64, 96) * 0.2}                                  # the down projection is float32
    part = GatedMLP(spec, {n: t.to(DEV) for n, t in w.items()}, rt)
    assert part.down.weight.dtype is torch.float32
    x = torch.randn(5, 64).bfloat16()
    want = plain_llama.swiglu(x.float(), w["g"].float(), w["u"].float(), w["d"])
    assert torch.allclose(part.forward(x.to(DEV), None).float().cpu(), want, atol=2e-2, rtol=2e-2)


def test_a_product_the_ring_kernel_cannot_keep_goes_to_the_library():
    """Few rows of a weight of real size are streamed only by the kernel with the shared-memory ring; where that one
    does not take the product (a normed input of 9 to 16 rows that does not fit beside the ring, a K that is no multiple
    of 256) the part says so and the library product stands in: the ring-less kernel is for the widths of tiny models."""
    from inf_engine_b200.parts import Runtime
    from inf_engine_b200.parts.linear import Linear
    rt = Runtime(DEV, torch.bfloat16)
    mk = lambda n, k: Linear(torch.zeros(n, k, device=DEV, dtype=torch.bfloat16), rt)
    wide, wider, odd, tiny = mk(2048, 3072), mk(1024, 4096), mk(4096, 1160), mk(96, 120)
    assert wide.streams(8, normed=True) and wide.streams(16, normed=True)        # 16 rows x 3,072 fit: 99 KB
    assert wider.streams(8, normed=True) and not wider.streams(9, normed=True)     # 16 rows x 4,096 do not
    assert wider.streams(16)                                                       # plain rows are read from L2
    assert not odd.streams(4) and not odd.streams(4, normed=True)                  # K % 256 != 0 at real size
    assert tiny.streams(4) and tiny.streams(16, normed=True) and not tiny.streams(17)
    # and the library's answer is the product
    torch.manual_seed(5)
    lin = Linear((torch.randn(4096, 1160, device=DEV) * 0.05).bfloat16(), rt)
    x = torch.randn(4, 1160, device=DEV).bfloat16()
    out = torch.empty(4, 4096, device=DEV, dtype=torch.bfloat16)
    lin(x, out)
    want = x.float().cpu() @ lin.weight.float().cpu().T
    assert float((out.float().cpu() - want).abs().max()) <= 1e-2 * float(want.abs().max())


# ------------------------------------------------------------------ a toy mixer
@dataclass(frozen=True)
class ToyDecaySpec:
    """out[t] = W (state[t]),  state[t] = decay * state[t-1] + x[t]: a mixer whose cache is
    one vector per request instead of pages."""

    kind: str
    hidden: int
    decay: float
    weight: str


class ToyDecayMixer:
    graph_safe = False

    @staticmethod
    def expected_tensors(spec):
        from inf_engine_b200.weights import ExpectedTensor
        return {spec.weight: ExpectedTensor((spec.hidden, spec.hidden))}

    def __init__(self, spec, tensors, rt):
        self.spec, self.rt, self.w = spec, rt, tensors[spec.weight]

    def cache_requirement(self):
        from inf_engine_b200.cache import CacheRequirement
        return CacheRequirement(kind="state", state_shape=(self.spec.hidden,), state_dtype=torch.float32)

    def forward(self, x, ctx, cache):
        out = torch.empty_like(x)
        q_start, slots = ctx.host["q_start"], ctx.host["slots"]
        for r in range(ctx.n_requests):
            s = cache.state[slots[r]]
            for t in range(q_start[r], q_start[r + 1]):
                s.mul_(self.spec.decay).add_(x[t].float())
                out[t] = (self.w.float() @ s).to(x.dtype)
        return out


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_toy_mixer_with_its_own_state_is_registered_built_and_stepped(dtype):
    from inf_engine_b200 import ModelRunner, StepEntry
    from inf_engine_b200.config import ScheduleEntry, parse_config_dict
    from inf_engine_b200.parts import MIXERS, expected_tensors, register_mixer
    from inf_engine_b200.weights import kept_dtype, random_tensors
    from helpers import TINY_A

    register_mixer("toy_decay", ToyDecayMixer)
    try:
        cfg = parse_config_dict(TINY_A)
        base = cfg.model_spec()
        toy_block = dataclasses.replace(base.layers[1], mixer=ToyDecaySpec("toy_decay", 64, 0.8, "toy.mix.weight"))
        spec = dataclasses.replace(base, layers=(base.layers[0], toy_block),
                                   schedule=(ScheduleEntry(0), ScheduleEntry(1)))
        exp = expected_tensors(spec)
        assert "toy.mix.weight" in exp and "model.layers.1.self_attn.q_proj.weight" not in exp
        cpu = random_tensors(exp, seed=4, std=0.05)
        tensors = {n: t.to(DEV, kept_dtype(t.dtype, dtype)) for n, t in cpu.items()}
        r = ModelRunner(cfg, tensors, dtype, page_size=16, n_pages=16, max_requests=3, spec=spec)
        assert len(r.cache.state_groups) == 1 and len(r.cache.kv_groups) == 1 and not r.model.graph_safe

        def plain(toks):
            w = {n: t.float() for n, t in cpu.items()}
            x = w["model.embed_tokens.weight"][torch.tensor(toks)]
            x = plain_llama.block(x, w, "model.layers.0.", TINY_A, *plain_llama.rope_tables(TINY_A, len(toks)))
            h = plain_llama.rms_norm(x, w["model.layers.1.input_layernorm.weight"], 1e-5)
            s, mixed = torch.zeros(64), []
            for t in range(len(toks)):
                s = 0.8 * s + h[t]
                mixed.append(w["toy.mix.weight"] @ s)
            x = x + torch.stack(mixed)
            h = plain_llama.rms_norm(x, w["model.layers.1.post_attention_layernorm.weight"], 1e-5)
            x = x + plain_llama.swiglu(h, w["model.layers.1.mlp.gate_proj.weight"], w["model.layers.1.mlp.up_proj.weight"],
                                       w["model.layers.1.mlp.down_proj.weight"])
            return plain_llama.rms_norm(x, w["model.norm.weight"], 1e-5) @ w["model.embed_tokens.weight"].T

        a, b = random_tokens(256, 40, 1), random_tokens(256, 23, 2)
        ref_a, ref_b = plain(a), plain(b)
        got_a, got_b = [], []
        r.open("a"); r.open("b")
        plan = [(7, 23), (2, 0), (30, 0), (1, 0)]                        # a in portions, b whole beside the first
        pa = pb = 0
        for na, nb in plan:
            es = [StepEntry("a", a[pa:pa + na], list(range(na)))]
            if nb:
                es.append(StepEntry("b", b[pb:pb + nb], list(range(nb))))
            lg = r.step(es).cpu()
            got_a.append(lg[:na].clone()); got_b.append(lg[na:].clone())
            pa += na; pb += nb
        name = "float32" if dtype is torch.float32 else "bfloat16"
        assert_close(torch.cat(got_a), ref_a, name, "toy mixer, request a")
        assert_close(torch.cat(got_b), ref_b, name, "toy mixer, request b")
        # the slot of a finished request is zeroed for the next one
        r.close("a")
        r.open("c")
        lg = r.step([StepEntry("c", a, list(range(len(a))))]).cpu()
        assert_close(lg, ref_a, name, "toy mixer, a slot used again")
    finally:
        MIXERS.pop("toy_decay")


# ------------------------------------------------------- more toy parts
def _two_layer_model(dtype, toy_block_of, seed, fix=None):
    """TINY_A with its second layer replaced by ``toy_block_of(base layer)``: (runner, float32 weights)."""
    from inf_engine_b200 import ModelRunner
    from inf_engine_b200.config import ScheduleEntry, parse_config_dict
    from inf_engine_b200.parts import expected_tensors
    from inf_engine_b200.weights import kept_dtype, random_tensors
    from helpers import TINY_A

    cfg = parse_config_dict(TINY_A)
    base = cfg.model_spec()
    spec = dataclasses.replace(base, layers=(base.layers[0], toy_block_of(base.layers[1])),
                               schedule=(ScheduleEntry(0), ScheduleEntry(1)))
    cpu = random_tensors(expected_tensors(spec), seed=seed, std=0.05)
    if fix is not None:
        fix(cpu)
    tensors = {n: t.to(DEV, kept_dtype(t.dtype, dtype)) for n, t in cpu.items()}
    r = ModelRunner(cfg, tensors, dtype, page_size=16, n_pages=16, max_requests=3, spec=spec)
    return r, {n: t.float() for n, t in cpu.items()}


def _stepped_in_cuts(r, a, b):
    """Request a in portions (then token by token), b whole beside a's first portion: every logit of both."""
    from inf_engine_b200 import StepEntry
    got_a, got_b = [], []
    r.open("a"); r.open("b")
    pa = pb = 0
    for na, nb in [(7, len(b)), (2, 0), (len(a) - 12, 0), (1, 0), (1, 0), (1, 0)]:
        es = [StepEntry("a", a[pa:pa + na], list(range(na)))]
        if nb:
            es.append(StepEntry("b", b[pb:pb + nb], list(range(nb))))
        lg = r.step(es).cpu()
        got_a.append(lg[:na].clone()); got_b.append(lg[na:].clone())
        pa += na; pb += nb
    assert pa == len(a) and pb == len(b)
    return torch.cat(got_a), torch.cat(got_b)


def _check(got, ref, dtype, what):
    assert_close(got, ref, "float32" if dtype is torch.float32 else "bfloat16", what)


@dataclass(frozen=True)
class ToyRoutedSpec:
    """Each token goes to the one expert its router logit is largest for: out = p * W_out[e] relu(W_in[e] x),
    p the softmax weight of that expert."""

    kind: str
    hidden: int
    inner: int
    n_experts: int
    router: str
    w_in: str
    w_out: str


class ToyRoutedFeedForward:
    @staticmethod
    def expected_tensors(spec):
        from inf_engine_b200.weights import ExpectedTensor
        return {spec.router: ExpectedTensor((spec.n_experts, spec.hidden)),
                spec.w_in: ExpectedTensor((spec.n_experts, spec.inner, spec.hidden)),
                spec.w_out: ExpectedTensor((spec.n_experts, spec.hidden, spec.inner))}

    def __init__(self, spec, tensors, rt):
        self.spec = spec
        self.router, self.w_in, self.w_out = tensors[spec.router], tensors[spec.w_in], tensors[spec.w_out]

    def forward(self, x, ctx):
        logits = x.float() @ self.router.float().T                      # router logits in 32-bit
        p, e = torch.softmax(logits, dim=-1).max(dim=-1)
        out = torch.zeros_like(x)
        for i in range(self.spec.n_experts):
            rows = (e == i).nonzero().flatten()
            h = torch.relu(x[rows] @ self.w_in[i].to(x.dtype).T)
            out[rows] = (p[rows, None] * (h @ self.w_out[i].to(x.dtype).T).float()).to(x.dtype)
        return out


def _plain_routed(h, w):
    logits = h @ w["toy.router"].T
    p, e = torch.softmax(logits, dim=-1).max(dim=-1)
    out = torch.stack([p[t] * (w["toy.w_out"][e[t]] @ torch.relu(w["toy.w_in"][e[t]] @ h[t])) for t in range(len(h))])
    top2 = logits.topk(2, dim=-1).values
    return out, float((top2[:, 0] - top2[:, 1]).min())


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_toy_feedforward_with_routing_beside_the_dense_one(dtype):
    """Layer 0 keeps the dense feed-forward (and fuses its norm on short steps), layer 1 routes: the block takes
    either, and the hand-over of a prepared norm stops where a part does not take part in it."""
    from inf_engine_b200.parts import FEEDFORWARDS, register_feedforward
    from helpers import TINY_A

    register_feedforward("toy_routed", ToyRoutedFeedForward)
    try:
        toy = ToyRoutedSpec("toy_routed", 64, 40, 3, "toy.router", "toy.w_in", "toy.w_out")

        def sharpen(cpu):               # router rows far apart, so that rounding does not move a token to another expert
            cpu["toy.router"] = (cpu["toy.router"].float() * 40).to(cpu["toy.router"].dtype)

        r, w = _two_layer_model(dtype, lambda blk: dataclasses.replace(blk, feedforward=toy), seed=6, fix=sharpen)
        assert "model.layers.1.mlp.gate_proj.weight" not in w and w["toy.w_in"].shape == (3, 40, 64)
        assert not r.model.graph_safe                  # the toy part does not say that it is: no captured decode steps

        margins = []

        def plain(toks):
            x = w["model.embed_tokens.weight"][torch.tensor(toks)]
            x = plain_llama.block(x, w, "model.layers.0.", TINY_A, *plain_llama.rope_tables(TINY_A, len(toks)))
            h = plain_llama.rms_norm(x, w["model.layers.1.input_layernorm.weight"], 1e-5)
            x = x + plain_llama.attention(h, *(w[f"model.layers.1.self_attn.{p}_proj.weight"] for p in "qkvo"),
                                          TINY_A, *plain_llama.rope_tables(TINY_A, len(toks)))
            h = plain_llama.rms_norm(x, w["model.layers.1.post_attention_layernorm.weight"], 1e-5)
            routed, margin = _plain_routed(h, w)
            margins.append(margin)
            x = x + routed
            return plain_llama.rms_norm(x, w["model.norm.weight"], 1e-5) @ w["model.embed_tokens.weight"].T

        a, b = random_tokens(256, 40, 1), random_tokens(256, 23, 2)
        ref_a, ref_b = plain(a), plain(b)
        assert min(margins) > 0.25, "the test's tokens must not sit on the edge between two experts"
        got_a, got_b = _stepped_in_cuts(r, a, b)
        _check(got_a, ref_a, dtype, "toy routed feed-forward, a")
        _check(got_b, ref_b, dtype, "toy routed feed-forward, b")
    finally:
        FEEDFORWARDS.pop("toy_routed")


@dataclass(frozen=True)
class ToyDecayPositionSpec:
    """Not a table rotation: q of a head is scaled by exp(-rate * position) and k by exp(+rate * position), so a
    score carries exp(-rate * distance).  One learned rate per kv head."""

    kind: str
    n_kv_heads: int
    head_dim: int
    rates: str


class ToyDecayPosition:
    @staticmethod
    def expected_tensors(spec):
        from inf_engine_b200.weights import ExpectedTensor
        return {spec.rates: ExpectedTensor((spec.n_kv_heads,))}

    def __init__(self, spec, tensors, rt):
        self.spec, self.rates = spec, tensors[spec.rates].float()

    def rotary_tables(self):
        return None

    def rotate(self, q, k, ctx):
        n, c, hd = q.shape[0], self.spec.n_kv_heads, self.spec.head_dim
        f = torch.exp(self.rates[None, :] * ctx.positions[:n, None].float())            # [n, kv heads]
        kk = k.view(n, c, hd)
        kk.copy_((kk.float() * f[:, :, None]).to(k.dtype))
        qq = q.view(n, c, -1, hd)                                                       # heads of a group together
        qq.copy_((qq.float() / f[:, :, None, None]).to(q.dtype))


def _plain_decay_attention(h, w, prefix, config, rates):
    T = h.shape[0]
    H, C, hd = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    q = (h @ w[prefix + "q_proj.weight"].T).view(T, H, hd).transpose(0, 1)
    k = (h @ w[prefix + "k_proj.weight"].T).view(T, C, hd).transpose(0, 1).repeat_interleave(H // C, dim=0)
    v = (h @ w[prefix + "v_proj.weight"].T).view(T, C, hd).transpose(0, 1).repeat_interleave(H // C, dim=0)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    decay = torch.exp(-rates.repeat_interleave(H // C)[:, None, None] * (i - j)[None].float())
    scores = (q @ k.transpose(1, 2)) * decay * hd ** -0.5
    scores = scores.masked_fill(~(j <= i)[None], float("-inf"))
    out = (torch.softmax(scores, dim=-1) @ v).transpose(0, 1).reshape(T, H * hd)
    return out @ w[prefix + "o_proj.weight"].T


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_toy_position_encoding_with_a_learned_tensor(dtype):
    """Layer 0 rotates by tables, layer 1 uses an encoding that is no rotation and owns a tensor of the
    checkpoint: the attention part takes either, chosen by the layer's spec."""
    from inf_engine_b200.parts import POSITIONS, register_position
    from helpers import TINY_A

    register_position("toy_decay_position", ToyDecayPosition)
    try:
        pos = ToyDecayPositionSpec("toy_decay_position", 2, 16, "toy.pos.rates")
        rates = torch.tensor([0.03, 0.008])

        def set_rates(cpu):
            cpu["toy.pos.rates"] = rates.clone()                     # stored in 32-bit: stays so

        r, w = _two_layer_model(
            dtype, lambda blk: dataclasses.replace(blk, mixer=dataclasses.replace(blk.mixer, position=pos)),
            seed=8, fix=set_rates)
        assert r.model.graph_safe                      # the encoding works on the device only: decode steps are graphs

        def plain(toks):
            x = w["model.embed_tokens.weight"][torch.tensor(toks)]
            x = plain_llama.block(x, w, "model.layers.0.", TINY_A, *plain_llama.rope_tables(TINY_A, len(toks)))
            h = plain_llama.rms_norm(x, w["model.layers.1.input_layernorm.weight"], 1e-5)
            x = x + _plain_decay_attention(h, w, "model.layers.1.self_attn.", TINY_A, rates)
            h = plain_llama.rms_norm(x, w["model.layers.1.post_attention_layernorm.weight"], 1e-5)
            x = x + plain_llama.swiglu(h, *(w[f"model.layers.1.mlp.{p}_proj.weight"] for p in ("gate", "up", "down")))
            return plain_llama.rms_norm(x, w["model.norm.weight"], 1e-5) @ w["model.embed_tokens.weight"].T

        a, b = random_tokens(256, 40, 3), random_tokens(256, 23, 4)
        ref_a, ref_b = plain(a), plain(b)
        got_a, got_b = _stepped_in_cuts(r, a, b)
        _check(got_a, ref_a, dtype, "toy position encoding, a")
        _check(got_b, ref_b, dtype, "toy position encoding, b")
    finally:
        POSITIONS.pop("toy_decay_position")


@dataclass(frozen=True)
class ToySlopePositionSpec:
    """No rotation at all: a key that lies d positions back loses slope[head] * d from its score (a linear bias by
    distance, one slope per query head, stated in the spec)."""

    kind: str
    slopes: tuple
    max_positions: int


class ToySlopePosition:
    @staticmethod
    def expected_tensors(spec):
        return {}

    def __init__(self, spec, tensors, rt):
        d = torch.arange(spec.max_positions, dtype=torch.float32)
        self.table = (-torch.tensor(spec.slopes, dtype=torch.float32)[:, None] * d[None, :]).contiguous().to(rt.device)

    def rotary_tables(self):
        return None

    def rotate(self, q, k, ctx):
        return None

    def score_bias(self):
        return self.table


def _plain_slope_attention(h, w, prefix, config, slopes):
    T = h.shape[0]
    H, C, hd = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    q = (h @ w[prefix + "q_proj.weight"].T).view(T, H, hd).transpose(0, 1)
    k = (h @ w[prefix + "k_proj.weight"].T).view(T, C, hd).transpose(0, 1).repeat_interleave(H // C, dim=0)
    v = (h @ w[prefix + "v_proj.weight"].T).view(T, C, hd).transpose(0, 1).repeat_interleave(H // C, dim=0)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    scores = (q @ k.transpose(1, 2)) * hd ** -0.5 - torch.tensor(slopes)[:, None, None] * (i - j)[None].float()
    scores = scores.masked_fill(~(j <= i)[None], float("-inf"))
    out = (torch.softmax(scores, dim=-1) @ v).transpose(0, 1).reshape(T, H * hd)
    return out @ w[prefix + "o_proj.weight"].T


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_toy_position_encoding_that_biases_scores_by_distance(dtype):
    """Layer 0 rotates by tables, layer 1 has no rotation and biases every score by how far back its key lies:
    the attention part hands the bias table to its general kernel (the tensor-core kernels step aside)."""
    from inf_engine_b200.parts import POSITIONS, register_position
    from helpers import TINY_A

    register_position("toy_slope_position", ToySlopePosition)
    try:
        slopes = (0.5, 0.125, 0.03125, 0.0)                     # the last head sees no bias at all
        pos = ToySlopePositionSpec("toy_slope_position", slopes, 512)
        r, w = _two_layer_model(
            dtype, lambda blk: dataclasses.replace(blk, mixer=dataclasses.replace(blk.mixer, position=pos)), seed=12)
        assert r.model.graph_safe

        def plain(toks, slopes=slopes):
            x = w["model.embed_tokens.weight"][torch.tensor(toks)]
            x = plain_llama.block(x, w, "model.layers.0.", TINY_A, *plain_llama.rope_tables(TINY_A, len(toks)))
            h = plain_llama.rms_norm(x, w["model.layers.1.input_layernorm.weight"], 1e-5)
            x = x + _plain_slope_attention(h, w, "model.layers.1.self_attn.", TINY_A, slopes)
            h = plain_llama.rms_norm(x, w["model.layers.1.post_attention_layernorm.weight"], 1e-5)
            x = x + plain_llama.swiglu(h, *(w[f"model.layers.1.mlp.{p}_proj.weight"] for p in ("gate", "up", "down")))
            return plain_llama.rms_norm(x, w["model.norm.weight"], 1e-5) @ w["model.embed_tokens.weight"].T

        a, b = random_tokens(256, 70, 5), random_tokens(256, 23, 6)
        ref_a, ref_b = plain(a), plain(b)
        # the bias matters: without it the logits differ by far more than any tolerance
        assert float((plain(a, (0.0, 0.0, 0.0, 0.0)) - ref_a).abs().max()) > 1e-2
        got_a, got_b = _stepped_in_cuts(r, a, b)
        _check(got_a, ref_a, dtype, "toy score bias, a")
        _check(got_b, ref_b, dtype, "toy score bias, b")
    finally:
        POSITIONS.pop("toy_slope_position")


def _toy_top_level():
    """Another top level, put together from the same blocks: the embedding is scaled by sqrt(hidden) and the logits
    are capped smoothly, cap * tanh(logits / cap).  Registered under a ``kind`` of its own; the runner builds it
    because the spec names it."""
    from inf_engine_b200.parts import DecoderModel

    class ToyTopLevel(DecoderModel):
        CAP = 0.8

        def embed(self, ctx):
            residual = super().embed(ctx)
            residual.mul_(float(self.spec.hidden) ** 0.5)
            return residual

        def finish_logits(self, logits, ctx):
            return logits.div_(self.CAP).tanh_().mul_(self.CAP)

    return ToyTopLevel


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_toy_top_level_with_a_scaled_embedding_and_capped_logits(dtype):
    from inf_engine_b200 import ModelRunner, StepEntry
    from inf_engine_b200.config import parse_config_dict
    from inf_engine_b200.parts import MODELS, expected_tensors, register_model
    from inf_engine_b200.weights import kept_dtype, random_tensors
    from helpers import TINY_A

    ToyTopLevel = _toy_top_level()
    register_model("toy_scaled_capped", ToyTopLevel)
    try:
        cfg = parse_config_dict(TINY_A)
        spec = dataclasses.replace(cfg.model_spec(), kind="toy_scaled_capped")
        cpu = random_tensors(expected_tensors(spec), seed=13, std=0.05)
        tensors = {n: t.to(DEV, kept_dtype(t.dtype, dtype)) for n, t in cpu.items()}
        r = ModelRunner(cfg, tensors, dtype, page_size=16, n_pages=16, max_requests=3, spec=spec)
        assert type(r.model) is ToyTopLevel and r.model.graph_safe
        w = {n: t.float() for n, t in cpu.items()}

        def plain(toks):
            x = w["model.embed_tokens.weight"][torch.tensor(toks)] * 64 ** 0.5
            cos, sin = plain_llama.rope_tables(TINY_A, len(toks))
            for i in range(2):
                x = plain_llama.block(x, w, f"model.layers.{i}.", TINY_A, cos, sin)
            logits = plain_llama.rms_norm(x, w["model.norm.weight"], 1e-5) @ w["model.embed_tokens.weight"].T
            return ToyTopLevel.CAP * torch.tanh(logits / ToyTopLevel.CAP)

        a, b = random_tokens(256, 40, 7), random_tokens(256, 23, 8)
        ref_a, ref_b = plain(a), plain(b)
        assert float(ref_a.abs().max()) > 0.8 * ToyTopLevel.CAP       # the cap bites
        got_a, got_b = _stepped_in_cuts(r, a, b)
        _check(got_a, ref_a, dtype, "toy top level, a")
        _check(got_b, ref_b, dtype, "toy top level, b")
    finally:
        MODELS.pop("toy_scaled_capped")
