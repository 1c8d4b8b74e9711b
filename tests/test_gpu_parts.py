"""Each part alone on the GPU against the plain function for it, and a toy
mixer with state of its own that is registered, built and stepped without a
change to the package's files."""

import dataclasses
from dataclasses import dataclass

import pytest
import torch

import plain_llama
from helpers import random_tokens

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
        t = dict(atol=2e-5, rtol=1e-5) if dtype is torch.float32 else dict(atol=4e-2, rtol=4e-2)
        assert torch.allclose(torch.cat(got_a), ref_a, **t) and torch.allclose(torch.cat(got_b), ref_b, **t)
        # the slot of a finished request is zeroed for the next one
        r.close("a")
        r.open("c")
        lg = r.step([StepEntry("c", a, list(range(len(a))))]).cpu()
        assert torch.allclose(lg, ref_a, **t)
    finally:
        MIXERS.pop("toy_decay")
