"""Each part alone against its plain formula, and the generality of the assembly: a toy mixer with
state of its own, a windowed attention layer, a layer that runs twice and a layer that reads another
layer's cache are registered and built here, in the test, and stepped through the unchanged engine."""
import random

import pytest
import torch

import helpers as H
import plain_model as P

pytestmark = pytest.mark.gpu


def env(h, dt, maxpos=512):
    from dinfer_b200.parts.base import BuildEnv
    return BuildEnv(torch.device("cuda"), dt, h, maxpos)


def make_ctx(reqs, bs, groups=None, num_blocks=64):
    """reqs = [(history, new)]: a context and manager as the step function would build them."""
    from dinfer_b200.cache.manager import CacheManager, GroupSpec
    from dinfer_b200.engine.batch import PlanBuilder, StepEntry
    m = CacheManager(groups or [GroupSpec()], bs, num_blocks, 8)
    entries, starts = [], []
    for i, (hist, new) in enumerate(reqs):
        assert m.allocate(i, hist + new)
        m.advance(i, hist)
        entries.append(StepEntry(i, [0] * new, []))
        starts.append(hist)
    pb = PlanBuilder(m, "cuda", 4096, 8, 64)
    ids, rows, ctx = pb.build(entries, starts)
    return ctx, m


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_norm_and_feed_forward_parts(dt):
    from dinfer_b200.parts.base import FEED_FORWARDS, NORMS
    import dinfer_b200.models.decoder  # noqa: F401  registers the parts
    h, I, T = 88, 136, 13
    g = torch.Generator().manual_seed(1)
    w = (1 + 0.1 * torch.randn(h, generator=g)).to(dt)
    norm = NORMS.get("rmsnorm")({"size": h, "eps": 2e-6, "weight": "n.weight"}, env(h, dt), "p.")
    assert [d.name for d in norm.declare()] == ["p.n.weight"]
    norm.bind({"p.n.weight": w.cuda()})
    x = torch.randn(T, h, generator=g)
    got = norm.forward(x.cuda())
    t = dict(atol=1e-5, rtol=1e-5) if dt == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    assert got.dtype == dt and torch.allclose(got.double().cpu(), P.rms_norm(x.double(), w.double(), 2e-6), **t)
    ffn = FEED_FORWARDS.get("swiglu")({"intermediate_size": I}, env(h, dt), "m.")
    W = {d.name: (torch.randn(d.shape, generator=g) * 0.1).to(dt) for d in ffn.declare()}
    assert {d.name: d.shape for d in ffn.declare()} == {"m.gate_proj.weight": (I, h), "m.up_proj.weight": (I, h),
                                                         "m.down_proj.weight": (h, I)}
    ffn.bind({k: v.cuda() for k, v in W.items()})
    xin = (torch.randn(T, h, generator=g)).to(dt)
    y = ffn.forward(xin.cuda())
    want = P.swiglu_mlp(xin.double(), W["m.gate_proj.weight"].double(), W["m.up_proj.weight"].double(),
                        W["m.down_proj.weight"].double())
    t = dict(atol=1e-5, rtol=1e-4) if dt == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    assert torch.allclose(y.double().cpu(), want, **t)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 6])
def test_attention_part_in_two_portions(dt, window):
    """The mixer alone: a sequence given as 11 + 9 tokens equals the plain whole-sequence block."""
    from dinfer_b200.parts.base import MIXERS, CacheBinding
    from dinfer_b200.parts.spec import PartSpec
    from dinfer_b200.cache.manager import GroupSpec
    import dinfer_b200.models.decoder  # noqa: F401
    h, Hq, Hkv, D, bs = 72, 6, 3, 16, 4
    cfg = dict(num_attention_heads=Hq, num_key_value_heads=Hkv, head_dim=D, rms_norm_eps=1e-5, rope_theta=777.0)
    g = torch.Generator().manual_seed(2)
    mixer = MIXERS.get("gqa_attention")(
        {"num_heads": Hq, "num_kv_heads": Hkv, "head_dim": D, "qk_norm": True, "eps": 1e-5, "window": window,
         "position": PartSpec("rope_neox", {"head_dim": D, "theta": 777.0, "max_positions": 64})}, env(h, dt, 64), "a.")
    W = {}
    for d in mixer.declare():
        W[d.name] = ((1 + 0.1 * torch.randn(d.shape, generator=g)) if d.init == "ones"
                     else torch.randn(d.shape, generator=g) * 0.15).to(dt)
    mixer.bind({k: v.cuda() for k, v in W.items()})
    x = torch.randn(20, h, generator=g).to(dt)
    kv = torch.zeros(16, 2, Hkv, bs, D, dtype=dt, device="cuda")
    from dinfer_b200.cache.manager import CacheManager
    from dinfer_b200.engine.batch import PlanBuilder, StepEntry
    m = CacheManager([GroupSpec(window)], bs, 16, 2)
    pb = PlanBuilder(m, "cuda", 64, 2, 16)
    outs = []
    for lo, hi in ((0, 11), (11, 20)):
        assert m.allocate("r", hi)
        _, _, ctx = pb.build([StepEntry("r", [0] * (hi - lo), [])], [lo])
        outs.append(mixer.forward(x[lo:hi].cuda(), ctx, CacheBinding(kv=kv, group=0, write=True)))
        m.advance("r", hi)
    got = torch.cat(outs).double().cpu()
    want = P.attention_block(x.double(), {k: v.double() for k, v in W.items()}, "a.", cfg, torch.arange(20), window)
    t = dict(atol=2e-5, rtol=1e-4) if dt == torch.float32 else dict(atol=4e-2, rtol=4e-2)
    assert torch.allclose(got, want, **t)


def plain_attention_general(x, W, p, Hq, Hkv, D, eps, theta, rot, style, factor, bias, qk_norm):
    """The attention block of plain_model with the options Qwen3 does not use: biases on the four projections, a
    rotation of the first ``rot`` elements only, in (2i, 2i + 1) pairs, at positions divided by ``factor``."""
    T = x.shape[0]
    lin = lambda name, v: v @ W[p + name + ".weight"].T + (W[p + name + ".bias"] if bias else 0.0)
    q, k, v = lin("q_proj", x).reshape(T, Hq, D), lin("k_proj", x).reshape(T, Hkv, D), lin("v_proj", x).reshape(T, Hkv, D)
    if qk_norm:
        q, k = P.rms_norm(q, W[p + "q_norm.weight"], eps), P.rms_norm(k, W[p + "k_norm.weight"], eps)
    cos, sin = P.rope_cos_sin(torch.arange(T, dtype=torch.float64) / factor, rot, theta)

    def turn(t):
        head, rest = t[..., :rot], t[..., rot:]
        if style == "neox":
            return torch.cat([P.rope_neox(head, cos, sin), rest], -1)
        a, b = head[..., 0::2], head[..., 1::2]
        c, s_ = cos[:, None, :], sin[:, None, :]
        out = torch.stack([a * c - b * s_, b * c + a * s_], -1).flatten(-2)
        return torch.cat([out, rest], -1)

    o = P.causal_gqa_attention(turn(q), turn(k), v, D ** -0.5)
    return lin("o_proj", o.reshape(T, Hq * D))


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D,rot,style,factor,bias,qk_norm", [(16, 16, "interleaved", 1.0, False, True),
                                                             (32, 16, "neox", 4.0, True, False),
                                                             (64, 32, "interleaved", 2.0, True, True),
                                                             (128, 128, "neox", 1.0, True, True)])
def test_attention_part_with_biases_and_other_rotations(dt, D, rot, style, factor, bias, qk_norm):
    """What the attention part takes beyond the Qwen3 dense model's use of it, all as parameters: a bias on the four
    projections, no head norm, a rotation of a part of the head, in interleaved pairs, at scaled positions.  A
    sequence in portions of 9 + 1 + 7 tokens against the plain formula over the whole of it."""
    from dinfer_b200.cache.manager import CacheManager, GroupSpec
    from dinfer_b200.engine.batch import PlanBuilder, StepEntry
    from dinfer_b200.parts.base import MIXERS, CacheBinding
    from dinfer_b200.parts.spec import PartSpec
    import dinfer_b200.models.decoder  # noqa: F401
    h, Hq, Hkv, bs = 80, 4, 2, 8
    g = torch.Generator().manual_seed(D + rot)
    pos = PartSpec("rope", {"head_dim": D, "rotary_dim": rot, "theta": 3000.0, "max_positions": 64, "style": style,
                            "scaling_factor": factor})
    mixer = MIXERS.get("gqa_attention")({"num_heads": Hq, "num_kv_heads": Hkv, "head_dim": D, "qk_norm": qk_norm,
                                         "eps": 1e-5, "bias": bias, "position": pos}, env(h, dt, 64), "a.")
    names = [d.name for d in mixer.declare()]
    assert ("a.q_proj.bias" in names) == bias and ("a.o_proj.bias" in names) == bias and ("a.q_norm.weight" in names) == qk_norm
    W = {}
    for d in mixer.declare():
        W[d.name] = ((1 + 0.1 * torch.randn(d.shape, generator=g)) if d.init == "ones"
                     else torch.randn(d.shape, generator=g) * (0.3 if d.name.endswith(".bias") else 0.12)).to(dt)
    mixer.bind({k: v.cuda() for k, v in W.items()})
    x = torch.randn(17, h, generator=g).to(dt)
    kv = torch.zeros(8, 2, Hkv, bs, D, dtype=dt, device="cuda")
    m = CacheManager([GroupSpec()], bs, 8, 2)
    pb = PlanBuilder(m, "cuda", 64, 2, 8)
    outs = []
    for lo, hi in ((0, 9), (9, 10), (10, 17)):
        assert m.allocate("r", hi)
        _, _, ctx = pb.build([StepEntry("r", [0] * (hi - lo), [])], [lo])
        outs.append(mixer.forward(x[lo:hi].cuda(), ctx, CacheBinding(kv=kv, group=0, write=True)))
        m.advance("r", hi)
    got = torch.cat(outs).double().cpu()
    want = plain_attention_general(x.double(), {k: v.double() for k, v in W.items()}, "a.", Hq, Hkv, D, 1e-5, 3000.0,
                                   rot, style, factor, bias, qk_norm)
    t = dict(atol=2e-5, rtol=1e-4) if dt == torch.float32 else dict(atol=5e-2, rtol=5e-2)
    assert torch.allclose(got, want, **t), float((got - want).abs().max())


# ---------------------------------------------------------------- a toy architecture, defined here

def register_toy():
    from dinfer_b200.config.registry import register_architecture
    from dinfer_b200.parts.base import MIXERS, Mixer, StateNeed
    from dinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorDecl

    class RunningMean(Mixer):
        """y_t = Wo mean_{j<=t}(Wi x_j): the state is the running sum and the count."""

        def __init__(self, params, env, prefix=""):
            super().__init__(params, env, prefix)
            self.d = int(params["state_size"])
            self.h = env.hidden_size

        def declare(self):
            return [TensorDecl(self.prefix + "mix.in.weight", (self.d, self.h)),
                    TensorDecl(self.prefix + "mix.out.weight", (self.h, self.d))]

        def bind(self, tensors):
            self.wi = tensors[self.prefix + "mix.in.weight"].float()
            self.wo = tensors[self.prefix + "mix.out.weight"].float()

        def cache_need(self):
            return StateNeed((self.d + 1,), torch.float32)

        def forward(self, x, ctx, cache):
            out = torch.empty_like(x)
            for b in range(ctx.num_reqs):
                lo, hi = ctx.cu_seqlens_host[b], ctx.cu_seqlens_host[b + 1]
                st = cache.state[ctx.state_slots_host[b]]
                if ctx.state_fresh_host[b]:
                    st.zero_()
                v = x[lo:hi].float() @ self.wi.T
                sums = torch.cumsum(v, 0) + st[:self.d]
                counts = st[self.d] + torch.arange(1, hi - lo + 1, device=x.device)
                out[lo:hi] = ((sums / counts[:, None]) @ self.wo.T).to(x.dtype)
                st[:self.d] = sums[-1]
                st[self.d] = counts[-1]
            return out

    MIXERS.register("toy_running_mean", RunningMean, replace=True)

    def parse(d):
        return dict(d)

    def spec(c):
        h, Hq, Hkv, D = c["hidden_size"], c["heads"], c["kv_heads"], c["head_dim"]
        pos = PartSpec("rope_neox", {"head_dim": D, "theta": c["theta"], "max_positions": c["max_positions"]})
        norm = lambda name: PartSpec("rmsnorm", {"size": h, "eps": c["eps"], "weight": name})
        ffn = PartSpec("swiglu", {"intermediate_size": c["inter"]})

        def attn(window):
            # the windowed layer keeps its keys in pages of its own size, smaller than the engine's
            return PartSpec("gqa_attention", {"num_heads": Hq, "num_kv_heads": Hkv, "head_dim": D, "qk_norm": True,
                                              "eps": c["eps"], "position": pos, "window": window,
                                              "cache_block_size": c["window_page"] if window else None})
        layers = (
            LayerSpec("layers.0.", "prenorm_residual", PartSpec("toy_running_mean", {"state_size": c["state_size"]}),
                      norm("n1.weight"), ffn, norm("n2.weight")),
            LayerSpec("layers.1.", "prenorm_residual", attn(c["window"]), norm("n1.weight"), ffn, norm("n2.weight")),
            LayerSpec("layers.2.", "prenorm_residual", attn(None), norm("n1.weight"), ffn, norm("n2.weight")),
        )
        schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(1), ScheduleEntry(0),
                    ScheduleEntry(2, cache_from=2))
        return ModelSpec("ToyMixedForTest", h, c["vocab_size"], c["max_positions"], "embed.weight", layers, schedule,
                         norm("final.weight"), "head.weight", False)

    register_architecture("ToyMixedForTest", parse, spec, replace=True)


TOY = dict(architectures=["ToyMixedForTest"], vocab_size=203, hidden_size=56, heads=4, kv_heads=2, head_dim=16,
           inter=72, state_size=24, window=9, window_page=4, theta=5000.0, eps=1e-5, max_positions=128)


def toy_plain_logits(W, c, ids):
    W = {k: v.double() for k, v in W.items()}
    T = len(ids)
    pos = torch.arange(T)
    x = W["embed.weight"][torch.tensor(ids)]
    acfg = dict(num_attention_heads=c["heads"], num_key_value_heads=c["kv_heads"], head_dim=c["head_dim"],
                rms_norm_eps=c["eps"], rope_theta=c["theta"])
    kept = {}

    def ffn(x, p):
        return P.swiglu_mlp(x, W[p + "gate_proj.weight"], W[p + "up_proj.weight"], W[p + "down_proj.weight"])

    for entry, (layer, reuse) in enumerate([(0, None), (1, None), (2, None), (1, None), (0, None), (2, 2)]):
        p = f"layers.{layer}."
        hdn = P.rms_norm(x, W[p + "n1.weight"], c["eps"])
        if layer == 0:
            v = hdn @ W[p + "mix.in.weight"].T
            a = (torch.cumsum(v, 0) / torch.arange(1, T + 1)[:, None]) @ W[p + "mix.out.weight"].T
        else:
            H_, Hkv, D = c["heads"], c["kv_heads"], c["head_dim"]
            q = P.rms_norm((hdn @ W[p + "q_proj.weight"].T).reshape(T, H_, D), W[p + "q_norm.weight"], c["eps"])
            cos, sin = P.rope_cos_sin(pos, D, c["theta"])
            q = P.rope_neox(q, cos, sin)
            if reuse is None:
                k = P.rms_norm((hdn @ W[p + "k_proj.weight"].T).reshape(T, Hkv, D), W[p + "k_norm.weight"], c["eps"])
                k = P.rope_neox(k, cos, sin)
                v = (hdn @ W[p + "v_proj.weight"].T).reshape(T, Hkv, D)
                kept[entry] = (k, v)
            else:
                k, v = kept[reuse]                      # this run reads the cache another run wrote
            o = P.causal_gqa_attention(q, k, v, D ** -0.5, c["window"] if layer == 1 else None)
            a = o.reshape(T, H_ * D) @ W[p + "o_proj.weight"].T
        x = x + a
        x = x + ffn(P.rms_norm(x, W[p + "n2.weight"], c["eps"]), p)
    return (P.rms_norm(x, W["final.weight"], c["eps"]) @ W["head.weight"].T).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_registered_in_the_test(tmp_path, dtype):
    register_toy()
    try:
        d = H.make_model_dir(str(tmp_path / "toy"), TOY, 4, 0.08, 0.1,
                             torch.float32 if dtype == "float32" else torch.bfloat16)
        W = H.load_plain_weights(d)
        rng = random.Random(8)
        tokens = {r: H.random_tokens(rng, n, TOY["vocab_size"]) for r, n in {"a": 50, "b": 7, "c": 90, "d": 31}.items()}
        want = {r: toy_plain_logits(W, TOY, t) for r, t in tokens.items()}
        lengths = {r: len(t) for r, t in tokens.items()}
        rp = H.LocalReplay(d, dtype, 256, block_size=8)
        assert rp.runner.manager.block_sizes == [4, 8]             # the windowed group's own page size, the engine's
        worst = {}
        try:
            for name, steps in (("whole", H.schedule_whole(lengths)), ("chunks", H.schedule_chunks(lengths, rng)),
                                ("mixed", H.schedule_mixed(lengths, rng, max_live=3, decode_tail=10))):
                got = H.run_schedule(rp, steps, tokens, tag=name + "/")
                worst[name] = max(H.rel_err(got[r], want[r]) for r in tokens)
        finally:
            assert rp.close() == 0
        print(dtype, worst)
        assert all(v <= H.TOLERANCE[dtype] for v in worst.values()), worst
    finally:
        from dinfer_b200.config.registry import unregister_architecture
        from dinfer_b200.parts.base import MIXERS
        unregister_architecture("ToyMixedForTest")
        MIXERS.unregister("toy_running_mean")


# ------------------------------------------- a second toy: routed feed-forward, another position encoding

def register_toy_routed():
    from dinfer_b200.config.registry import register_architecture
    from dinfer_b200.parts.base import FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, PositionEncoding
    from dinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorDecl

    class Decay(PositionEncoding):
        """q_d <- q_d e^(-lambda_d p), k_d <- k_d e^(+lambda_d p): the score of (i, j) is weighted per
        dimension by e^(-lambda_d (i - j)).  Not a table rotation, so the mixer calls apply()."""
        fused = False

        def __init__(self, params, env, prefix=""):
            super().__init__(params, env, prefix)
            D = int(params["head_dim"])
            self.lam = (float(params["rate"]) * torch.arange(D, dtype=torch.float32) / D).to(env.device)

        def apply(self, q, k, ctx):
            f = torch.exp(ctx.positions.float()[:, None, None] * self.lam[None, None, :])
            q.copy_((q.float() / f).to(q.dtype))
            k.copy_((k.float() * f).to(k.dtype))

    class Routed(FeedForward):
        """Router logits in 32-bit -> the top_k experts -> softmax over the chosen -> weighted sum of
        their gated feed-forwards."""

        def __init__(self, params, env, prefix=""):
            super().__init__(params, env, prefix)
            self.E, self.k, self.I, self.h = int(params["experts"]), int(params["top_k"]), int(params["inter"]), env.hidden_size

        def declare(self):
            d = [TensorDecl(self.prefix + "router.weight", (self.E, self.h))]
            for e in range(self.E):
                d += [TensorDecl(self.prefix + f"experts.{e}.gate.weight", (self.I, self.h)),
                      TensorDecl(self.prefix + f"experts.{e}.up.weight", (self.I, self.h)),
                      TensorDecl(self.prefix + f"experts.{e}.down.weight", (self.h, self.I))]
            return d

        def bind(self, tensors):
            self.t = {k[len(self.prefix):]: v for k, v in tensors.items() if k.startswith(self.prefix)}

        def forward(self, x, ctx):
            xf = x.float()
            logits = xf @ self.t["router.weight"].float().T
            top, idx = torch.topk(logits, self.k, dim=-1)
            w = torch.softmax(top, dim=-1)
            out = torch.zeros_like(xf)
            for e in range(self.E):
                g = xf @ self.t[f"experts.{e}.gate.weight"].float().T
                u = xf @ self.t[f"experts.{e}.up.weight"].float().T
                y = (torch.nn.functional.silu(g) * u) @ self.t[f"experts.{e}.down.weight"].float().T
                out += y * (w * (idx == e)).sum(-1, keepdim=True)
            return out.to(x.dtype)

    POSITION_ENCODINGS.register("toy_decay", Decay, replace=True)
    FEED_FORWARDS.register("toy_routed", Routed, replace=True)

    def spec(c):
        h, Hq, Hkv, D = c["hidden_size"], c["heads"], c["kv_heads"], c["head_dim"]
        norm = lambda name: PartSpec("rmsnorm", {"size": h, "eps": c["eps"], "weight": name})

        def attn(pos):
            return PartSpec("gqa_attention", {"num_heads": Hq, "num_kv_heads": Hkv, "head_dim": D, "qk_norm": True,
                                              "eps": c["eps"], "position": pos})
        decay = PartSpec("toy_decay", {"head_dim": D, "rate": c["rate"]})
        rope = PartSpec("rope_neox", {"head_dim": D, "theta": c["theta"], "max_positions": c["max_positions"]})
        layers = (
            LayerSpec("layers.0.", "prenorm_residual", attn(decay), norm("n1.weight"),
                      PartSpec("toy_routed", {"experts": c["experts"], "top_k": c["top_k"], "inter": c["inter"]}),
                      norm("n2.weight")),
            LayerSpec("layers.1.", "prenorm_residual", attn(rope), norm("n1.weight"),
                      PartSpec("swiglu", {"intermediate_size": c["inter"]}), norm("n2.weight")),
        )
        return ModelSpec("ToyRoutedForTest", h, c["vocab_size"], c["max_positions"], "embed.weight", layers,
                         (ScheduleEntry(0), ScheduleEntry(1)), norm("final.weight"), "head.weight", False,
                         embedding_scale=c["embedding_scale"], logit_softcap=c["logit_softcap"])

    register_architecture("ToyRoutedForTest", lambda d: dict(d), spec, replace=True)


TOY_ROUTED = dict(architectures=["ToyRoutedForTest"], vocab_size=157, hidden_size=40, heads=6, kv_heads=3, head_dim=16,
                  inter=48, experts=4, top_k=2, rate=0.03, theta=20000.0, eps=1e-6, max_positions=128,
                  embedding_scale=6.3, logit_softcap=0.8)


def toy_routed_plain_logits(W, c, ids):
    W = {k: v.double() for k, v in W.items()}
    T, H_, Hkv, D = len(ids), c["heads"], c["kv_heads"], c["head_dim"]
    pos = torch.arange(T)
    x = W["embed.weight"][torch.tensor(ids)] * float(torch.tensor(c["embedding_scale"], dtype=torch.float32))
    for layer in (0, 1):
        p = f"layers.{layer}."
        hdn = P.rms_norm(x, W[p + "n1.weight"], c["eps"])
        q = P.rms_norm((hdn @ W[p + "q_proj.weight"].T).reshape(T, H_, D), W[p + "q_norm.weight"], c["eps"])
        k = P.rms_norm((hdn @ W[p + "k_proj.weight"].T).reshape(T, Hkv, D), W[p + "k_norm.weight"], c["eps"])
        v = (hdn @ W[p + "v_proj.weight"].T).reshape(T, Hkv, D)
        if layer == 0:
            lam = (torch.tensor(c["rate"], dtype=torch.float32) * torch.arange(D, dtype=torch.float32) / D).double()
            f = torch.exp(pos.double()[:, None, None] * lam[None, None, :])
            q, k = q / f, k * f
        else:
            cos, sin = P.rope_cos_sin(pos, D, c["theta"])
            q, k = P.rope_neox(q, cos, sin), P.rope_neox(k, cos, sin)
        o = P.causal_gqa_attention(q, k, v, D ** -0.5, None)
        x = x + o.reshape(T, H_ * D) @ W[p + "o_proj.weight"].T
        hdn = P.rms_norm(x, W[p + "n2.weight"], c["eps"])
        if layer == 0:
            logits = hdn @ W[p + "router.weight"].T
            top, idx = torch.topk(logits, c["top_k"], dim=-1)
            w = torch.softmax(top, dim=-1)
            y = torch.zeros_like(hdn)
            for e in range(c["experts"]):
                ye = P.swiglu_mlp(hdn, W[p + f"experts.{e}.gate.weight"], W[p + f"experts.{e}.up.weight"],
                                  W[p + f"experts.{e}.down.weight"])
                y += ye * (w * (idx == e)).sum(-1, keepdim=True)
        else:
            y = P.swiglu_mlp(hdn, W[p + "gate_proj.weight"], W[p + "up_proj.weight"], W[p + "down_proj.weight"])
        x = x + y
    logits = P.rms_norm(x, W["final.weight"], c["eps"]) @ W["head.weight"].T
    return (c["logit_softcap"] * torch.tanh(logits / c["logit_softcap"])).numpy()


def test_toy_routed_feed_forward_and_other_position_encoding(tmp_path):
    """A feed-forward with routing and a position encoding that is no table rotation, both defined here, in a model
    that scales its embedding and caps its logits softly; registered, built from a model folder and stepped whole /
    in portions / mixed (32-bit: the routing must pick the same experts as the plain implementation)."""
    register_toy_routed()
    try:
        d = H.make_model_dir(str(tmp_path / "toyr"), TOY_ROUTED, 5, 0.1, 0.1, torch.float32)
        W = H.load_plain_weights(d)
        rng = random.Random(9)
        tokens = {r: H.random_tokens(rng, n, TOY_ROUTED["vocab_size"]) for r, n in {"a": 40, "b": 3, "c": 77}.items()}
        want = {r: toy_routed_plain_logits(W, TOY_ROUTED, t) for r, t in tokens.items()}
        lengths = {r: len(t) for r, t in tokens.items()}
        rp = H.LocalReplay(d, "float32", 192, block_size=8)
        worst = {}
        try:
            for name, steps in (("whole", H.schedule_whole(lengths)), ("chunks", H.schedule_chunks(lengths, rng)),
                                ("mixed", H.schedule_mixed(lengths, rng, max_live=3, decode_tail=10))):
                got = H.run_schedule(rp, steps, tokens, tag=name + "/")
                worst[name] = max(H.rel_err(got[r], want[r]) for r in tokens)
        finally:
            assert rp.close() == 0
        print(worst)
        assert all(v <= H.TOLERANCE["float32"] for v in worst.values()), worst
    finally:
        from dinfer_b200.config.registry import unregister_architecture
        from dinfer_b200.parts.base import FEED_FORWARDS, POSITION_ENCODINGS
        unregister_architecture("ToyRoutedForTest")
        FEED_FORWARDS.unregister("toy_routed")
        POSITION_ENCODINGS.unregister("toy_decay")


# ------------------------------------------- a third toy: a mixer with state whose steps replay CUDA graphs

def register_toy_state_graph():
    from dinfer_b200.config.registry import register_architecture
    from dinfer_b200.parts.base import MIXERS, Mixer, StateNeed
    from dinfer_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorDecl

    class RunningMeanOnDevice(Mixer):
        """y_t = Wo mean_{j<=t}(Wi x_j) again, but driven by the context's DEVICE tensors only (request offsets, state
        slots, fresh flags), so that a step can be captured once and replayed with other requests in its rows; rows
        without a request carry the spare slot, which is read and written like any other and never looked at."""
        graph_capturable = True

        def __init__(self, params, env, prefix=""):
            super().__init__(params, env, prefix)
            self.d, self.h = int(params["state_size"]), env.hidden_size

        def declare(self):
            return [TensorDecl(self.prefix + "mix.in.weight", (self.d, self.h)),
                    TensorDecl(self.prefix + "mix.out.weight", (self.h, self.d))]

        def bind(self, tensors):
            self.wi = tensors[self.prefix + "mix.in.weight"].float()
            self.wo = tensors[self.prefix + "mix.out.weight"].float()

        def cache_need(self):
            return StateNeed((self.d + 1,), torch.float32)

        def forward(self, x, ctx, cache):
            T, B, d = x.shape[0], ctx.num_reqs, self.d
            cu = ctx.cu_seqlens.long()
            start, end = cu[:B], cu[1:B + 1]
            slots = ctx.state_slots.long()
            v = x.float() @ self.wi.T
            tok = torch.arange(T, device=x.device)
            req = torch.bucketize(tok, end, right=True).clamp(max=B - 1)         # the request of every token
            c = torch.cumsum(v, 0)
            before = torch.where((start > 0)[:, None], c[(start - 1).clamp(min=0)], torch.zeros_like(c[:1]))
            st = cache.state.index_select(0, slots) * (1.0 - ctx.state_fresh.float())[:, None]
            sums = c - before[req] + st[req, :d]
            counts = st[req, d] + (tok - start[req] + 1).float()
            out = ((sums / counts[:, None]) @ self.wo.T).to(x.dtype)
            last = (end - 1).clamp(min=0)
            new = torch.cat([sums[last], counts[last, None]], 1)
            new = torch.where((end > start)[:, None], new, st)                      # a place without tokens keeps its state
            cache.state.index_copy_(0, slots, new)
            return out

    MIXERS.register("toy_running_mean_device", RunningMeanOnDevice, replace=True)

    def spec(c):
        h, Hq, Hkv, D = c["hidden_size"], c["heads"], c["kv_heads"], c["head_dim"]
        pos = PartSpec("rope", {"head_dim": D, "theta": c["theta"], "max_positions": c["max_positions"], "style": "interleaved"})
        norm = lambda name: PartSpec("rmsnorm", {"size": h, "eps": c["eps"], "weight": name})
        ffn = PartSpec("swiglu", {"intermediate_size": c["inter"]})
        layers = (
            LayerSpec("layers.0.", "prenorm_residual", PartSpec("toy_running_mean_device", {"state_size": c["state_size"]}),
                      norm("n1.weight"), ffn, norm("n2.weight")),
            LayerSpec("layers.1.", "prenorm_residual",
                      PartSpec("gqa_attention", {"num_heads": Hq, "num_kv_heads": Hkv, "head_dim": D, "qk_norm": True,
                                                 "eps": c["eps"], "position": pos, "bias": True}),
                      norm("n1.weight"), ffn, norm("n2.weight")),
        )
        return ModelSpec("ToyStateGraphForTest", h, c["vocab_size"], c["max_positions"], "embed.weight", layers,
                         (ScheduleEntry(0), ScheduleEntry(1)), norm("final.weight"), "head.weight", False)

    register_architecture("ToyStateGraphForTest", lambda d: dict(d), spec, replace=True)


TOY_STATE = dict(architectures=["ToyStateGraphForTest"], vocab_size=111, hidden_size=48, heads=4, kv_heads=2, head_dim=16,
                 inter=64, state_size=20, theta=9000.0, eps=1e-5, max_positions=128)


def toy_state_plain_logits(W, c, ids):
    W = {k: v.double() for k, v in W.items()}
    T, Hq, Hkv, D = len(ids), c["heads"], c["kv_heads"], c["head_dim"]
    x = W["embed.weight"][torch.tensor(ids)]
    p = "layers.0."
    hdn = P.rms_norm(x, W[p + "n1.weight"], c["eps"])
    a = (torch.cumsum(hdn @ W[p + "mix.in.weight"].T, 0) / torch.arange(1, T + 1)[:, None]) @ W[p + "mix.out.weight"].T
    x = x + a
    x = x + P.swiglu_mlp(P.rms_norm(x, W[p + "n2.weight"], c["eps"]), W[p + "gate_proj.weight"], W[p + "up_proj.weight"],
                         W[p + "down_proj.weight"])
    p = "layers.1."
    hdn = P.rms_norm(x, W[p + "n1.weight"], c["eps"])
    x = x + plain_attention_general(hdn, W, p, Hq, Hkv, D, c["eps"], c["theta"], D, "interleaved", 1.0, True, True)
    x = x + P.swiglu_mlp(P.rms_norm(x, W[p + "n2.weight"], c["eps"]), W[p + "gate_proj.weight"], W[p + "up_proj.weight"],
                         W[p + "down_proj.weight"])
    return P.rms_norm(x, W["final.weight"], c["eps"]) @ W["head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_replays_cuda_graphs(tmp_path, dtype):
    """A model whose first mixer keeps per-request state (and says its forward can be captured), whose attention has
    biases and an interleaved rotation: registered here, run with CUDA graphs ON.  Decode-only steps replay a graph
    per bucket (dummy rows on the spare state slot), steps with prompt portions replay theirs; requests join, finish
    and hand their state slots on; every last-token logit against the plain formula."""
    from dinfer_b200.config.engine_config import EngineConfig
    from dinfer_b200.engine.batch import StepEntry
    from dinfer_b200.engine.runner import ModelRunner
    register_toy_state_graph()
    try:
        tdt = torch.float32 if dtype == "float32" else torch.bfloat16
        d = H.make_model_dir(str(tmp_path / "toy"), TOY_STATE, 7, 0.08, 0.1, tdt)
        W = H.load_plain_weights(d)
        rng = random.Random(12)
        names = [f"r{i}" for i in range(9)]
        steps, lengths = H.schedule_rolling(names, [9, 6], 5)
        tokens = {r: H.random_tokens(rng, n, TOY_STATE["vocab_size"]) for r, n in lengths.items()}
        want = {r: toy_state_plain_logits(W, TOY_STATE, t).numpy() for r, t in tokens.items()}
        r = ModelRunner.from_dir(d, EngineConfig(max_model_len=64, max_num_seqs=8, max_num_batched_tokens=16, num_blocks=40,
                                                 block_size=4, dtype=dtype, enable_cuda_graph=True, mixed_cuda_graph=True))
        assert r._graph_ok                                    # state, and still graphs
        worst = 0.0
        # after the rolling part: the survivors decode alone (decode-only buckets), with a newcomer now and then
        for entries, end in steps:
            out = r.step([StepEntry(q, tokens[q][lo:hi], [hi - lo - 1]) for q, lo, hi in entries]).cpu().numpy()
            for i, (q, lo, hi) in enumerate(entries):
                worst = max(worst, H.rel_err(out[i], want[q][hi - 1]))
            for q in end:
                r.finish(q)
        assert any(isinstance(k, int) for k in r._graphs) and any(isinstance(k, tuple) for k in r._graphs), list(r._graphs)
        r.manager.check_invariants()
        assert r.manager.num_free_blocks() == 40
        print("toy with state and graphs", dtype, worst, sorted(map(str, r._graphs)))
        assert worst <= H.TOLERANCE[dtype], worst
    finally:
        from dinfer_b200.config.registry import unregister_architecture
        from dinfer_b200.parts.base import MIXERS
        unregister_architecture("ToyStateGraphForTest")
        MIXERS.unregister("toy_running_mean_device")
