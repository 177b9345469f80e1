"""Each part alone against the plain functions; a schedule that runs a layer twice and lets
a layer read another layer's cache; and toy parts defined here (a mixer with state of its own,
a feed-forward that routes tokens to experts, a position encoding that does not rotate),
registered, built, loaded and stepped through the public interfaces only."""
from dataclasses import dataclass

import pytest
import torch

import plain_llama as pl
import tiny
import traces

pytestmark = pytest.mark.gpu
DEV = "cuda"


def runtime(dtype):
    from fastmlx_b200.engine.loading import make_runtime
    return make_runtime(dtype)


def rnd(*shape, seed=0, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale).to(dtype)


def close(got, ref, dtype, scale=None):
    got, ref = got.double().cpu(), ref.double().cpu()
    s = scale or ref.abs().max().item()
    tol = 1e-5 if dtype == "float32" else 2e-2
    err = (got - ref).abs().max().item() / s
    assert err < tol, err


def step_context(manager, rows, rt):
    """rows: [(request cache, tokens)] -> a reserved step context."""
    from fastmlx_b200.engine.batch import StepEntry, build_context
    entries = [StepEntry(rc, toks, []) for rc, toks in rows]
    for e in entries:
        manager.reserve(e.request, len(e.tokens))
    ctx = build_context(entries, manager, rt.device, torch.zeros(4, dtype=torch.int32, device=rt.device))
    return ctx, entries


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_linear_mlp_embedding_head_alone(dtype):
    from fastmlx_b200.parts import Embedding, Linear, LMHead, RMSNorm, SwiGLU
    rt = runtime(dtype)
    rto = torch.bfloat16 if dtype == "bfloat16" else None
    d, I, V, T = 72, 136, 50, 9
    W = {"n.weight": 1 + rnd(d, seed=1, scale=0.1), "m.g.weight": rnd(I, d, seed=2, scale=0.1),
         "m.u.weight": rnd(I, d, seed=3, scale=0.1), "m.dn.weight": rnd(d, I, seed=4, scale=0.1),
         "m.g.bias": rnd(I, seed=5, scale=0.1), "m.u.bias": rnd(I, seed=6, scale=0.1), "m.dn.bias": rnd(d, seed=7, scale=0.1),
         "e.weight": rnd(V, d, seed=8), "h.weight": rnd(V, d, seed=9, scale=0.1)}
    x = rnd(T, d, seed=10).to(rt.dtype)
    res = rnd(T, d, seed=11).to(rt.dtype)

    norm = RMSNorm(d, 1e-4, "n")
    norm.bind(W, rt)
    out, r2 = norm.forward(x.to(DEV), res.clone().to(DEV))
    h = pl._rnd(x.double() + res.double(), rto)
    close(r2, h, dtype)
    close(out, pl._rnd(pl.rms_norm(h, W["n.weight"], 1e-4), rto), dtype)

    mlp = SwiGLU(d, I, "m", bias=True, proj_names=("g", "u", "dn"))
    mlp.bind(W, rt)
    close(mlp.forward(x.to(DEV), None), pl.swiglu(x, W["m.g.weight"], W["m.u.weight"], W["m.dn.weight"], W["m.g.bias"],
                                                  W["m.u.bias"], W["m.dn.bias"], rto), dtype)

    lin = Linear(d, [("m.g", I)], bias=False)
    lin.bind(W, rt)
    close(lin.forward(x.to(DEV)), pl.linear(x, W["m.g.weight"]), dtype)

    emb = Embedding(V, d, "e")
    emb.bind(W, rt)
    ids = torch.tensor([3, 0, 49, 3], dtype=torch.int32, device=DEV)
    ctx = type("C", (), {"status": torch.zeros(4, dtype=torch.int32, device=DEV)})()
    assert torch.equal(emb.forward(ids, ctx).cpu(), W["e.weight"].to(rt.dtype)[ids.cpu().long()])
    for head in (LMHead(V, d, "h"), LMHead(V, d, None, tied=emb)):
        head.bind(W, rt)
        logits = head.forward(x.to(DEV))
        assert logits.dtype == torch.float32
        close(logits, pl.linear(x, W["h.weight"] if head.tied is None else W["e.weight"]), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,window,trad,rot", [(4, 2, 16, 0, False, None), (6, 2, 32, 0, True, None),
                                                       (3, 1, 64, 9, False, None), (4, 4, 48, 0, False, 24)])
def test_attention_part_alone_with_rotary(dtype, nh, nkv, hd, window, trad, rot):
    """One attention mixer over its own small cache, a sequence fed in three portions, with
    a window and with a partial rotary dimension, against plain attention on the whole."""
    from fastmlx_b200.cache import CacheManager
    from fastmlx_b200.parts import GQAAttention, RotaryEmbedding
    rt = runtime(dtype)
    rto = torch.bfloat16 if dtype == "bfloat16" else None
    d, T = 40, 37
    mixer = GQAAttention(d, nh, nkv, hd, RotaryEmbedding(hd, 777.0, None, trad, rot), "a", window=window)
    W = {s.name: rnd(*s.shape, seed=i, scale=0.3) for i, s in enumerate(mixer.weight_specs())}
    mixer.bind(W, rt)
    x = rnd(T, d, seed=99).to(rt.dtype)
    manager = CacheManager([(mixer.cache_spec(), None, None)], page_size=8, num_pages=8, max_requests=1,
                           dtype=rt.dtype, device=DEV)
    rc = manager.add_request("r")
    outs, at = [], 0
    for n in (20, 2, 15):
        ctx, _ = step_context(manager, [(rc, [0] * n)], rt)
        outs.append(mixer.forward(x[at:at + n].to(DEV), ctx, manager.entries[0]))
        assert ctx.status.tolist()[0] == 0
        manager.commit(rc)
        at += n
    got = torch.cat(outs)
    # plain: the same weights through the plain attention block, with this part's options
    cfg = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "attention_bias": False,
           "rope_traditional": trad}
    inv = pl.rope_inv_freq(rot or hd, 777.0, None)
    Wp = {"self_attn." + k[2:]: v for k, v in W.items()}
    ref = pl.attention_block(x, Wp, "", cfg, torch.arange(T), inv, rto, window or None)
    close(got, ref, dtype)


def test_llama3_frequency_table_matches_plain():
    from fastmlx_b200.config import RopeScaling
    from fastmlx_b200.parts import inverse_frequencies
    sc = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    got = inverse_frequencies(32, 500000.0, RopeScaling.from_dict(sc))
    want = pl.rope_inv_freq(32, 500000.0, sc)
    assert torch.allclose(got, want, rtol=1e-14, atol=0)
    plain = pl.rope_inv_freq(32, 500000.0, None)
    ratio = (got / plain)
    assert (ratio == 1).any() and (ratio == 1 / 8).any() and ((ratio > 1 / 8) & (ratio < 1)).any()   # all three bands


# ----------------------------------------------------------------------------- schedules
@dataclass(frozen=True)
class LoopCfg:
    vocab_size: int = 90
    width: int = 48
    eos_token_id: int = -1

    @staticmethod
    def from_dict(d):
        return LoopCfg(int(d.get("vocab_size", 90)), int(d.get("width", 48)))


def build_loop(cfg):
    """Two blocks run as 0, 1, 0: the second reads the first one's cache and has no k/v
    projections; the first runs twice, with a cache for each run."""
    from fastmlx_b200.parts import (Embedding, GQAAttention, LMHead, Model, PreNormBlock, RMSNorm, RotaryEmbedding,
                                    Run, SwiGLU)
    d = cfg.width
    emb = Embedding(cfg.vocab_size, d, "emb")

    def block(i, share):
        return PreNormBlock(GQAAttention(d, 4, 2, 16, RotaryEmbedding(16, 10000.0), f"l{i}.attn", share_kv=share),
                            SwiGLU(d, 64, f"l{i}.mlp"), RMSNorm(d, 1e-5, f"l{i}.n1"), RMSNorm(d, 1e-5, f"l{i}.n2"))
    return Model(emb, [block(0, False), block(1, True)], RMSNorm(d, 1e-5, "norm"), LMHead(cfg.vocab_size, d, None, tied=emb),
                 schedule=[Run(0), Run(1, cache_from=0), Run(0)], vocab_size=cfg.vocab_size, max_positions=256)


def plain_loop(W, toks):
    T = len(toks)
    pos = torch.arange(T)
    inv = pl.rope_inv_freq(16, 10000.0, None)
    h = pl.embedding(torch.tensor(toks), W["emb.weight"])
    first_kv = None
    for run, share in ((0, False), (1, True), (0, False)):
        p = f"l{run}."
        x = pl.rms_norm(h, W[p + "n1.weight"], 1e-5)
        q = pl.apply_rope(pl.linear(x, W[p + "attn.q_proj.weight"]).view(T, 4, 16), pos, inv)
        if share:
            k, v = first_kv
        else:
            k = pl.apply_rope(pl.linear(x, W[p + "attn.k_proj.weight"]).view(T, 2, 16), pos, inv)
            v = pl.linear(x, W[p + "attn.v_proj.weight"]).view(T, 2, 16)
            if first_kv is None:
                first_kv = (k, v)
        a = pl.attention(q, k, v, 16 ** -0.5).reshape(T, 64)
        h = h + pl.linear(a, W[p + "attn.o_proj.weight"])
        y = pl.rms_norm(h, W[p + "n2.weight"], 1e-5)
        h = h + pl.swiglu(y, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"], W[p + "mlp.down_proj.weight"])
    return pl.linear(pl.rms_norm(h, W["norm.weight"], 1e-5), W["emb.weight"])


def test_schedule_runs_a_layer_twice_and_shares_a_cache(tmp_path):
    from fastmlx_b200 import registry, write_random_model
    from fastmlx_b200.engine.replay import Replayer
    registry.register("toy_loop", LoopCfg.from_dict, build_loop, replace=True)
    try:
        d = write_random_model(str(tmp_path / "loop"), {"model_type": "toy_loop", "vocab_size": 90, "width": 48}, seed=2)
        W = tiny.load_plain_weights(d)
        assert "l1.attn.k_proj.weight" not in W and "l0.attn.k_proj.weight" in W
        prompts = {f"r{i}": tiny.rand_tokens(n, 90, i) for i, n in enumerate([21, 40, 5, 33])}
        ref = {r: plain_loop(W, t) for r, t in prompts.items()}
        rp = Replayer(d, "float32", 256, page_size=8)
        assert len(rp.manager.groups) == 1 and rp.manager.groups[0].entries == [0, 2]
        for cut in (traces.whole, traces.portions, traces.mixed):
            steps = cut(prompts)
            rows = traces.collect(steps, [rp.step(s) for s in steps])
            for r, t in prompts.items():
                got = torch.tensor([rows[r][i].tolist() for i in range(len(t))], dtype=torch.float64)
                assert (got - ref[r]).abs().max().item() / ref[r].abs().max().item() < 1e-5, (cut.__name__, r)
            rp.manager.check()
    finally:
        registry.unregister("toy_loop")


# ----------------------------------------------------------------------------- a toy mixer with state
def make_toy():
    """Defined with the public interfaces only: a mixer whose per-request state is a decaying
    sum of its projected inputs (s_t = decay * s_{t-1} + x_t P^T, y_t = s_t)."""
    from fastmlx_b200.parts import (Embedding, GQAAttention, Linear, LMHead, Mixer, Model, PreNormBlock, RMSNorm,
                                    RotaryEmbedding, StateSpec, SwiGLU)

    class DecayingSum(Mixer):
        def __init__(self, width, decay, name):
            self.width, self.decay = width, decay
            self.proj = Linear(width, [(name + ".proj", width)])

        def children(self):
            return (self.proj,)

        def state_spec(self):
            return StateSpec((self.width,), torch.float32)

        def forward(self, x, ctx, cache):
            u = self.proj.forward(x).float()
            out = torch.empty_like(u)
            for r in range(ctx.R):
                a, b, slot = ctx.h_row_start[r], ctx.h_row_start[r + 1], ctx.h_row_slot[r]
                s = cache.state[slot]
                for t in range(a, b):
                    s = self.decay * s + u[t]
                    out[t] = s
                cache.state[slot] = s
            return out.to(x.dtype)

    @dataclass(frozen=True)
    class ToyCfg:
        vocab_size: int
        width: int
        decay: float
        eos_token_id: int = -1

        @staticmethod
        def from_dict(d):
            return ToyCfg(int(d["vocab_size"]), int(d["width"]), float(d["decay"]))

    def build(cfg):
        d = cfg.width
        emb = Embedding(cfg.vocab_size, d, "emb")
        blocks = [
            PreNormBlock(DecayingSum(d, cfg.decay, "l0.mix"), SwiGLU(d, 56, "l0.mlp"), RMSNorm(d, 1e-5, "l0.n1"),
                         RMSNorm(d, 1e-5, "l0.n2")),
            PreNormBlock(GQAAttention(d, 2, 1, 16, RotaryEmbedding(16, 100.0), "l1.attn"), SwiGLU(d, 56, "l1.mlp"),
                         RMSNorm(d, 1e-5, "l1.n1"), RMSNorm(d, 1e-5, "l1.n2")),
        ]
        return Model(emb, blocks, RMSNorm(d, 1e-5, "norm"), LMHead(cfg.vocab_size, d, "head"),
                     vocab_size=cfg.vocab_size, max_positions=512)

    return ToyCfg, build


def plain_toy(W, toks, decay):
    T = len(toks)
    pos = torch.arange(T)
    h = pl.embedding(torch.tensor(toks), W["emb.weight"])
    x = pl.rms_norm(h, W["l0.n1.weight"], 1e-5)
    u = pl.linear(x, W["l0.mix.proj.weight"])
    s = torch.zeros(u.shape[1], dtype=torch.float64)
    y = torch.empty_like(u)
    for t in range(T):
        s = decay * s + u[t]
        y[t] = s
    h = h + y
    h = h + pl.swiglu(pl.rms_norm(h, W["l0.n2.weight"], 1e-5), W["l0.mlp.gate_proj.weight"], W["l0.mlp.up_proj.weight"],
                      W["l0.mlp.down_proj.weight"])
    x = pl.rms_norm(h, W["l1.n1.weight"], 1e-5)
    inv = pl.rope_inv_freq(16, 100.0, None)
    q = pl.apply_rope(pl.linear(x, W["l1.attn.q_proj.weight"]).view(T, 2, 16), pos, inv)
    k = pl.apply_rope(pl.linear(x, W["l1.attn.k_proj.weight"]).view(T, 1, 16), pos, inv)
    v = pl.linear(x, W["l1.attn.v_proj.weight"]).view(T, 1, 16)
    h = h + pl.linear(pl.attention(q, k, v, 0.25).reshape(T, 32), W["l1.attn.o_proj.weight"])
    h = h + pl.swiglu(pl.rms_norm(h, W["l1.n2.weight"], 1e-5), W["l1.mlp.gate_proj.weight"], W["l1.mlp.up_proj.weight"],
                      W["l1.mlp.down_proj.weight"])
    return pl.linear(pl.rms_norm(h, W["norm.weight"], 1e-5), W["head.weight"])


def test_a_toy_mixer_with_its_own_state_registers_builds_and_steps(tmp_path):
    from fastmlx_b200 import Engine, SamplingParams, registry, write_random_model
    from fastmlx_b200.engine.replay import Replayer
    ToyCfg, build = make_toy()
    registry.register(["toy_decay", "ToyDecayForCausalLM"], ToyCfg.from_dict, build, replace=True)
    try:
        config = {"architectures": ["ToyDecayForCausalLM"], "vocab_size": 77, "width": 40, "decay": 0.9}
        d = write_random_model(str(tmp_path / "toy"), config, seed=4)
        W = tiny.load_plain_weights(d)
        prompts = {f"r{i}": tiny.rand_tokens(n, 77, 10 + i) for i, n in enumerate([19, 34, 3, 50, 27, 41])}
        ref = {r: plain_toy(W, t, 0.9) for r, t in prompts.items()}
        rp = Replayer(d, "float32", 256, page_size=8)
        assert rp.manager.entries[0].state is not None and rp.manager.entries[0].kv is None
        assert rp.manager.entries[1].state is None and rp.manager.entries[1].kv is not None
        for cut in (traces.whole, traces.tail_decoded, traces.portions, traces.mixed):
            steps = cut(prompts)
            rows = traces.collect(steps, [rp.step(s) for s in steps])
            for r, t in prompts.items():
                got = torch.tensor([rows[r][i].tolist() for i in range(len(t))], dtype=torch.float64)
                assert (got - ref[r]).abs().max().item() / ref[r].abs().max().item() < 1e-5, (cut.__name__, r)
            rp.manager.check()
        # and it generates through the entry point, slots being reused by later requests
        eng = Engine(d, dtype="float32", block_size=8, max_cache_tokens=512, max_concurrent_requests=2)
        ps = [prompts["r0"], prompts["r2"], prompts["r4"]]
        outs = eng.generate(ps, SamplingParams(max_tokens=6, temperature=0.0))
        for p, o in zip(ps, outs):
            seq = list(p)
            for _ in range(6):
                seq.append(int(torch.argmax(plain_toy(W, seq, 0.9)[-1])))
            assert o.output_token_ids == seq[len(p):]
    finally:
        registry.unregister(["toy_decay", "ToyDecayForCausalLM"])


# ----------------------------------------------------------------------------- a toy routed feed-forward, a toy position encoding
def make_routed():
    """Public interfaces only: a feed-forward that sends each token to the one expert its router
    prefers (router logits in 32-bit, the expert's output scaled by the router's probability),
    and a position encoding that, instead of rotating, adds a position-dependent sinusoid to q
    and k before k and v are stored."""
    from fastmlx_b200.parts import (Embedding, FeedForward, GQAAttention, Linear, LMHead, Model, PositionEncoding,
                                    PreNormBlock, RMSNorm, SwiGLU)

    class TopOneExperts(FeedForward):
        supports_cuda_graph = False                      # it sorts tokens by expert on the host

        def __init__(self, width, hidden, n_experts, name):
            self.router = Linear(width, [(name + ".router", n_experts)])
            self.experts = [SwiGLU(width, hidden, f"{name}.experts.{e}") for e in range(n_experts)]

        def children(self):
            return (self.router, *self.experts)

        def forward(self, x, ctx):
            logits = self.router.forward(x).float()
            prob = torch.softmax(logits, dim=-1)
            choice = torch.argmax(logits, dim=-1)
            out = torch.zeros_like(x)
            for e, expert in enumerate(self.experts):
                idx = torch.nonzero(choice == e).flatten()
                if idx.numel():
                    y = expert.forward(x.index_select(0, idx).contiguous(), None)
                    out.index_copy_(0, idx, (y.float() * prob[idx, e:e + 1]).to(x.dtype))
            return out

    class AddedSinusoid(PositionEncoding):
        def __init__(self, head_dim, period):
            self.head_dim, self.period = head_dim, period

        def apply_and_store(self, qkv, ctx, cache, nh, nkv, hd):
            ang = ctx.positions.to(torch.float32)[:, None] * (2 * torch.pi / self.period) + \
                torch.arange(hd, device=qkv.device, dtype=torch.float32)[None, :]
            bump = (0.5 * torch.sin(ang)).to(qkv.dtype)                              # [T, hd]
            heads = qkv[:, :(nh + nkv) * hd].view(qkv.shape[0], nh + nkv, hd)
            heads += bump[:, None, :]
            g = ctx.groups[cache.group]
            self.rt.k.rope_kv_write(qkv, ctx.positions, None, 0, False, g.slot_mapping if cache.writable else None,
                                    cache.kv if cache.writable else None, nh, nkv, hd, ctx.status)

    @dataclass(frozen=True)
    class RoutedCfg:
        vocab_size: int
        width: int
        experts: int
        period: float
        eos_token_id: int = -1

        @staticmethod
        def from_dict(d):
            return RoutedCfg(int(d["vocab_size"]), int(d["width"]), int(d["experts"]), float(d["period"]))

    def build(cfg):
        d = cfg.width
        blocks = [PreNormBlock(GQAAttention(d, 3, 1, 16, AddedSinusoid(16, cfg.period), f"l{i}.attn"),
                               TopOneExperts(d, 40, cfg.experts, f"l{i}.moe"), RMSNorm(d, 1e-5, f"l{i}.n1"),
                               RMSNorm(d, 1e-5, f"l{i}.n2")) for i in range(2)]
        return Model(Embedding(cfg.vocab_size, d, "emb"), blocks, RMSNorm(d, 1e-5, "norm"),
                     LMHead(cfg.vocab_size, d, "head"), vocab_size=cfg.vocab_size, max_positions=512)

    return RoutedCfg, build


def plain_routed(W, toks, experts, period):
    T = len(toks)
    pos = torch.arange(T, dtype=torch.float64)
    h = pl.embedding(torch.tensor(toks), W["emb.weight"])
    bump = 0.5 * torch.sin((pos[:, None] * (2 * torch.pi / period)).float() + torch.arange(16, dtype=torch.float32)[None, :]).double()
    for i in range(2):
        x = pl.rms_norm(h, W[f"l{i}.n1.weight"], 1e-5)
        q = pl.linear(x, W[f"l{i}.attn.q_proj.weight"]).view(T, 3, 16) + bump[:, None, :]
        k = pl.linear(x, W[f"l{i}.attn.k_proj.weight"]).view(T, 1, 16) + bump[:, None, :]
        v = pl.linear(x, W[f"l{i}.attn.v_proj.weight"]).view(T, 1, 16)
        h = h + pl.linear(pl.attention(q, k, v, 0.25).reshape(T, 48), W[f"l{i}.attn.o_proj.weight"])
        x = pl.rms_norm(h, W[f"l{i}.n2.weight"], 1e-5)
        logits = pl.linear(x, W[f"l{i}.moe.router.weight"])
        prob = torch.softmax(logits, dim=-1)
        choice = torch.argmax(logits, dim=-1)
        y = torch.zeros_like(h)
        for t in range(T):
            e = int(choice[t])
            y[t] = prob[t, e] * pl.swiglu(x[t:t + 1], W[f"l{i}.moe.experts.{e}.gate_proj.weight"],
                                          W[f"l{i}.moe.experts.{e}.up_proj.weight"],
                                          W[f"l{i}.moe.experts.{e}.down_proj.weight"])[0]
        h = h + y
    return pl.linear(pl.rms_norm(h, W["norm.weight"], 1e-5), W["head.weight"]), choice


def test_a_toy_routed_feed_forward_and_a_toy_position_encoding(tmp_path):
    """Neither part exists in the package: both are defined above, registered as an architecture
    of their own, loaded from a written model folder and replayed under every cut."""
    from fastmlx_b200 import Engine, SamplingParams, registry, write_random_model
    from fastmlx_b200.engine.replay import Replayer
    RoutedCfg, build = make_routed()
    registry.register(["toy_routed"], RoutedCfg.from_dict, build, replace=True)
    try:
        config = {"model_type": "toy_routed", "vocab_size": 61, "width": 48, "experts": 3, "period": 37.0}
        d = write_random_model(str(tmp_path / "routed"), config, seed=9)
        W = tiny.load_plain_weights(d)
        prompts = {f"r{i}": tiny.rand_tokens(n, 61, 20 + i) for i, n in enumerate([23, 40, 5, 33])}
        ref, used = {}, set()
        for r, t in prompts.items():
            ref[r], choice = plain_routed(W, t, 3, 37.0)
            used |= set(choice.tolist())
        assert used == {0, 1, 2}, "the test should exercise every expert"
        rp = Replayer(d, "float32", 256, page_size=8)
        assert not rp.model.graph_safe
        for cut in (traces.whole, traces.tail_decoded, traces.portions, traces.mixed):
            steps = cut(prompts)
            rows = traces.collect(steps, [rp.step(s) for s in steps])
            for r, t in prompts.items():
                got = torch.tensor([rows[r][i].tolist() for i in range(len(t))], dtype=torch.float64)
                assert (got - ref[r]).abs().max().item() / ref[r].abs().max().item() < 1e-5, (cut.__name__, r)
            rp.manager.check()
        eng = Engine(d, dtype="float32", block_size=8, max_cache_tokens=512, max_concurrent_requests=2)
        outs = eng.generate([prompts["r0"], prompts["r2"]], SamplingParams(max_tokens=5, temperature=0.0))
        for p, o in zip([prompts["r0"], prompts["r2"]], outs):
            seq = list(p)
            for _ in range(5):
                seq.append(int(torch.argmax(plain_routed(W, seq, 3, 37.0)[0][-1])))
            assert o.output_token_ids == seq[len(p):]
    finally:
        registry.unregister(["toy_routed"])


# ----------------------------------------------------------------------------- a toy mixer with state, captured in graphs
def make_toy_on_device():
    """The decaying sum again, with its decode step written as dense tensor operations over
    the step's device arrays (no loop over rows on the host), so that a decode step of the
    model may be captured in a CUDA graph.  Rows whose slot is -1 (the padding rows of a
    captured step) match no slot and touch no state."""
    from fastmlx_b200.parts import (Embedding, GQAAttention, Linear, LMHead, Mixer, Model, PreNormBlock, RMSNorm,
                                    RotaryEmbedding, StateSpec, SwiGLU)

    class DecayingSumOnDevice(Mixer):
        supports_cuda_graph = True

        def __init__(self, width, decay, name):
            self.width, self.decay = width, decay
            self.proj = Linear(width, [(name + ".proj", width)])

        def children(self):
            return (self.proj,)

        def state_spec(self):
            return StateSpec((self.width,), torch.float32)

        def forward(self, x, ctx, cache):
            u = self.proj.forward(x).float()
            if ctx.all_decode:
                state = cache.state                                         # [slots, width]
                hit = (ctx.row_slot[:, None] == torch.arange(state.shape[0], device=u.device)[None, :]).float()   # [rows, slots]
                s_new = self.decay * (hit @ state) + u                       # a padding row: 0 + u, written nowhere
                state.mul_(1.0 - hit.sum(0)[:, None]).add_(hit.t() @ s_new)
                return s_new.to(x.dtype)
            out = torch.empty_like(u)
            for r in range(ctx.R):
                a, b, slot = ctx.h_row_start[r], ctx.h_row_start[r + 1], ctx.h_row_slot[r]
                s = cache.state[slot]
                for t in range(a, b):
                    s = self.decay * s + u[t]
                    out[t] = s
                cache.state[slot] = s
            return out.to(x.dtype)

    ToyCfg, _ = make_toy()

    def build(cfg):
        d = cfg.width
        blocks = [
            PreNormBlock(DecayingSumOnDevice(d, cfg.decay, "l0.mix"), SwiGLU(d, 56, "l0.mlp"), RMSNorm(d, 1e-5, "l0.n1"),
                         RMSNorm(d, 1e-5, "l0.n2")),
            PreNormBlock(GQAAttention(d, 2, 1, 16, RotaryEmbedding(16, 100.0), "l1.attn"), SwiGLU(d, 56, "l1.mlp"),
                         RMSNorm(d, 1e-5, "l1.n1"), RMSNorm(d, 1e-5, "l1.n2")),
        ]
        return Model(Embedding(cfg.vocab_size, d, "emb"), blocks, RMSNorm(d, 1e-5, "norm"),
                     LMHead(cfg.vocab_size, d, "head"), vocab_size=cfg.vocab_size, max_positions=512)

    return ToyCfg, build


def test_a_mixer_with_state_runs_in_captured_decode_steps(tmp_path):
    """Three live requests in a graph of four rows, one step ahead of the host: the padding row
    must touch no request's state, and the run that warms a graph up before its capture must
    not count as a step.  Token-equal to the plain statement."""
    from fastmlx_b200 import Engine, SamplingParams, registry, write_random_model
    ToyCfg, build = make_toy_on_device()
    registry.register(["toy_decay_dev"], ToyCfg.from_dict, build, replace=True)
    try:
        config = {"model_type": "toy_decay_dev", "vocab_size": 77, "width": 40, "decay": 0.9}
        d = write_random_model(str(tmp_path / "toydev"), config, seed=4)
        W = tiny.load_plain_weights(d)
        prompts = [tiny.rand_tokens(n, 77, 30 + n) for n in (19, 3, 27)]
        eng = Engine(d, dtype="float32", block_size=8, max_cache_tokens=1024, max_concurrent_requests=4)
        assert eng.model.graph_safe and eng.manager.has_state
        outs = eng.generate(prompts, [SamplingParams(max_tokens=m, temperature=0.0) for m in (14, 9, 20)])
        assert any(k[:2] == (4, 16) for k in eng.step_fn.graphs) and eng.stats()["graph_replays"] > 10
        for p, o in zip(prompts, outs):
            seq = list(p)
            for _ in range(len(o.output_token_ids)):
                seq.append(int(torch.argmax(plain_toy(W, seq, 0.9)[-1])))
            assert o.output_token_ids == seq[len(p):]
        # a failed step leaves the state as it was: a token outside the vocabulary in the second step
        from fastmlx_b200.engine.replay import Replayer
        from fastmlx_b200.engine.step import StepError
        rp = Replayer(d, "float32", 256, page_size=8)
        toks = prompts[0]
        rp.step({"step": 0, "entries": [{"id": "a", "tokens": toks[:10], "want": []}], "end": []})
        before = rp.manager.entries[0].state.clone()
        with pytest.raises(StepError):
            rp.step({"step": 1, "entries": [{"id": "a", "tokens": [5, 99999, 7], "want": []}], "end": []})
        assert torch.equal(rp.manager.entries[0].state, before) and rp.manager.requests["a"].length == 10
        got = rp.step({"step": 2, "entries": [{"id": "a", "tokens": toks[10:], "want": [len(toks) - 11]}], "end": ["a"]})
        ref = plain_toy(W, toks, 0.9)[-1]
        assert (torch.from_numpy(got[0]).double() - ref).abs().max().item() / ref.abs().max().item() < 1e-5
    finally:
        registry.unregister(["toy_decay_dev"])


# ----------------------------------------------------------------------------- a window through the engine's loop
def make_windowed():
    """Two attention layers, the first with a window of 9 keys: two cache groups with pools of
    their own, the first of which gives pages back while a request runs."""
    from fastmlx_b200.parts import Embedding, GQAAttention, LMHead, Model, PreNormBlock, RMSNorm, RotaryEmbedding, SwiGLU

    @dataclass(frozen=True)
    class WinCfg:
        vocab_size: int
        width: int
        window: int
        eos_token_id: int = -1

        @staticmethod
        def from_dict(d):
            return WinCfg(int(d["vocab_size"]), int(d["width"]), int(d["window"]))

    def build(cfg):
        d = cfg.width
        blocks = [PreNormBlock(GQAAttention(d, 4, 2, 16, RotaryEmbedding(16, 100.0), f"l{i}.attn", window=w),
                               SwiGLU(d, 64, f"l{i}.mlp"), RMSNorm(d, 1e-5, f"l{i}.n1"), RMSNorm(d, 1e-5, f"l{i}.n2"))
                  for i, w in enumerate((cfg.window, 0))]
        return Model(Embedding(cfg.vocab_size, d, "emb"), blocks, RMSNorm(d, 1e-5, "norm"),
                     LMHead(cfg.vocab_size, d, "head"), vocab_size=cfg.vocab_size, max_positions=512)

    return WinCfg, build


def plain_windowed(W, toks, window, round_to=None):
    T = len(toks)
    cfg = {"num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "attention_bias": False, "rope_traditional": False}
    inv = pl.rope_inv_freq(16, 100.0, None)
    h = pl.embedding(torch.tensor(toks), W["emb.weight"])
    for i, w in enumerate((window, None)):
        Wp = {k.replace(f"l{i}.attn.", "self_attn."): v for k, v in W.items() if k.startswith(f"l{i}.attn.")}
        x = pl._rnd(pl.rms_norm(h, W[f"l{i}.n1.weight"], 1e-5), round_to)
        h = h + pl.attention_block(x, Wp, "", cfg, torch.arange(T), inv, round_to, w)
        y = pl._rnd(pl.rms_norm(h, W[f"l{i}.n2.weight"], 1e-5), round_to)
        h = h + pl.swiglu(y, W[f"l{i}.mlp.gate_proj.weight"], W[f"l{i}.mlp.up_proj.weight"], W[f"l{i}.mlp.down_proj.weight"],
                          round_to=round_to)
    return pl.linear(pl._rnd(pl.rms_norm(h, W["norm.weight"], 1e-5), round_to), W["head.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_window_gives_pages_back_inside_the_engine_loop(tmp_path, dtype):
    """Prompts in portions, then more than three windows of decode steps under graphs and one
    step ahead, in a tight pool: the windowed group's pages go back at every commit, the graph's
    block tables come from the mirror with -1 holes, and the step launched ahead builds its
    tables after the earlier step's pages were returned.  Tokens against the plain model."""
    from fastmlx_b200 import Engine, SamplingParams, registry, write_random_model
    WinCfg, build = make_windowed()
    registry.register(["toy_window"], WinCfg.from_dict, build, replace=True)
    try:
        config = {"model_type": "toy_window", "vocab_size": 83, "width": 48, "window": 9}
        d = write_random_model(str(tmp_path / "win"), config, seed=6)
        W = tiny.load_plain_weights(d)
        prompts = [tiny.rand_tokens(n, 83, 50 + n) for n in (20, 35, 11)]
        eng = Engine(d, dtype=dtype, block_size=8, initial_cache_blocks=40, max_concurrent_requests=4, prefill_chunk=7,
                     max_num_batched_tokens=16)
        groups = eng.manager.groups
        assert [g.spec.window for g in groups] == [9, 0]
        assert groups[0].pool.num_pages < groups[1].pool.num_pages            # the window's pool is its own size
        ids = [eng.submit(p, SamplingParams(max_tokens=32, temperature=0.0)) for p in prompts]
        final, most = {}, 0
        while eng.has_unfinished():
            for o in eng.step():
                if o.finished:
                    final[o.request_id] = o
            eng.manager.check()
            most = max(most, groups[0].pool.used_pages)
        # per request the window holds at most 9 + 7 keys: which lie on three pages at most
        assert most <= 3 * 3 and eng.stats()["pages_used"] == 0 and eng.stats()["graph_replays"] > 20
        rt, slack = (torch.bfloat16, 2e-2) if dtype == "bfloat16" else (None, 1e-5)
        for p, rid in zip(prompts, ids):
            got = final[rid].output_token_ids
            assert len(got) == 32
            logits = plain_windowed(W, list(p) + got, 9, rt)[len(p) - 1: -1]
            for i, tok in enumerate(got):
                best = int(torch.argmax(logits[i]))
                if best != tok:
                    gap = float(logits[i][best] - logits[i][tok]) / float(logits[i].abs().max())
                    assert gap < slack, (i, tok, best, gap)
    finally:
        registry.unregister(["toy_window"])


# ----------------------------------------------------------------------------- positions in the embedding stream
def make_learned_positions():
    """Learned absolute positions added to the token embeddings (no rotation of q and k): a
    `StreamEncoding` defined here, with a table of its own in the checkpoint."""
    from fastmlx_b200.parts import (Embedding, GQAAttention, LMHead, Model, NoPositionEncoding, PreNormBlock, RMSNorm,
                                    StreamEncoding, SwiGLU, WeightSpec)
    from fastmlx_b200.parts.base import to_compute

    class LearnedPositions(StreamEncoding):
        def __init__(self, max_positions, width, name):
            self.max_positions, self.width, self.name = max_positions, width, name

        def own_weight_specs(self):
            return [WeightSpec(self.name + ".weight", (self.max_positions, self.width), "embedding")]

        def bind_own(self, tensors, rt):
            self.table = to_compute(tensors[self.name + ".weight"], rt)

        def forward(self, h, ctx):
            pos = ctx.positions.long().clamp(min=0)              # a padding row's position is -1: any row will do
            return (h.float() + self.table[pos].float()).to(h.dtype)

    @dataclass(frozen=True)
    class PosCfg:
        vocab_size: int
        width: int
        max_positions: int
        eos_token_id: int = -1

        @staticmethod
        def from_dict(d):
            return PosCfg(int(d["vocab_size"]), int(d["width"]), int(d["max_positions"]))

    def build(cfg):
        d = cfg.width
        blocks = [PreNormBlock(GQAAttention(d, 4, 2, 16, NoPositionEncoding(), f"l{i}.attn"), SwiGLU(d, 64, f"l{i}.mlp"),
                               RMSNorm(d, 1e-5, f"l{i}.n1"), RMSNorm(d, 1e-5, f"l{i}.n2")) for i in range(2)]
        return Model(Embedding(cfg.vocab_size, d, "emb"), blocks, RMSNorm(d, 1e-5, "norm"), LMHead(cfg.vocab_size, d, "head"),
                     vocab_size=cfg.vocab_size, max_positions=cfg.max_positions,
                     stream_encoding=LearnedPositions(cfg.max_positions, d, "pos"))

    return PosCfg, build


def plain_learned_positions(W, toks):
    T = len(toks)
    h = pl.embedding(torch.tensor(toks), W["emb.weight"]) + W["pos.weight"].double()[:T]
    for i in range(2):
        x = pl.rms_norm(h, W[f"l{i}.n1.weight"], 1e-5)
        q = pl.linear(x, W[f"l{i}.attn.q_proj.weight"]).view(T, 4, 16)
        k = pl.linear(x, W[f"l{i}.attn.k_proj.weight"]).view(T, 2, 16)
        v = pl.linear(x, W[f"l{i}.attn.v_proj.weight"]).view(T, 2, 16)
        h = h + pl.linear(pl.attention(q, k, v, 0.25).reshape(T, 64), W[f"l{i}.attn.o_proj.weight"])
        h = h + pl.swiglu(pl.rms_norm(h, W[f"l{i}.n2.weight"], 1e-5), W[f"l{i}.mlp.gate_proj.weight"],
                          W[f"l{i}.mlp.up_proj.weight"], W[f"l{i}.mlp.down_proj.weight"])
    return pl.linear(pl.rms_norm(h, W["norm.weight"], 1e-5), W["head.weight"])


def test_positions_in_the_embedding_stream(tmp_path):
    """An encoding that is added to the embedding stream instead of applied to q and k: a part of
    its own kind (`StreamEncoding`), registered from here, replayed under every cut and generated
    from under graphs."""
    from fastmlx_b200 import Engine, SamplingParams, registry, write_random_model
    from fastmlx_b200.engine.replay import Replayer
    PosCfg, build = make_learned_positions()
    registry.register(["toy_learned_pos"], PosCfg.from_dict, build, replace=True)
    try:
        config = {"model_type": "toy_learned_pos", "vocab_size": 71, "width": 64, "max_positions": 128}
        d = write_random_model(str(tmp_path / "pos"), config, seed=8)
        W = tiny.load_plain_weights(d)
        assert W["pos.weight"].shape == (128, 64)
        prompts = {f"r{i}": tiny.rand_tokens(n, 71, 60 + i) for i, n in enumerate([23, 40, 5, 33])}
        ref = {r: plain_learned_positions(W, t) for r, t in prompts.items()}
        rp = Replayer(d, "float32", 256, page_size=8)
        assert rp.step_fn.native is None                     # a part defined here: the Python path
        for cut in (traces.whole, traces.tail_decoded, traces.portions, traces.mixed):
            steps = cut(prompts)
            rows = traces.collect(steps, [rp.step(s) for s in steps])
            for r, t in prompts.items():
                got = torch.tensor([rows[r][i].tolist() for i in range(len(t))], dtype=torch.float64)
                assert (got - ref[r]).abs().max().item() / ref[r].abs().max().item() < 1e-5, (cut.__name__, r)
        eng = Engine(d, dtype="float32", block_size=8, max_cache_tokens=512, max_concurrent_requests=4)
        outs = eng.generate([prompts["r0"], prompts["r2"], prompts["r3"]], SamplingParams(max_tokens=6, temperature=0.0))
        assert eng.stats()["graph_replays"] > 0
        for p, o in zip([prompts["r0"], prompts["r2"], prompts["r3"]], outs):
            seq = list(p)
            for _ in range(6):
                seq.append(int(torch.argmax(plain_learned_positions(W, seq)[-1])))
            assert o.output_token_ids == seq[len(p):]
    finally:
        registry.unregister(["toy_learned_pos"])
