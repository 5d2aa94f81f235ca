"""Parts of (c) alone, and the proof that the framework is open: a toy mixer with
state of its own and a toy architecture that mixes it with attention, both
defined here, are registered, built and stepped without a change to any file of
the package.  (Toy parts only: they are no model of anyone's.)"""
from dataclasses import dataclass

import pytest
import torch

import plain_qwen3 as P
from cpu_kernels import PlainKernels

pytestmark = pytest.mark.gpu


def _register_toys():
    from zlm_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from zlm_b200.parts.base import Mixer, ParamSpec, StateRequest
    from zlm_b200.registry import ARCHITECTURES, MIXERS, register_architecture, register_mixer

    if "toy_running_mean" not in MIXERS:
        @register_mixer("toy_running_mean")
        class RunningMean(Mixer):
            """y_t = W . mean(x_0 .. x_t); the running sum is the sequence's state."""
            graph_safe = False

            def __init__(self, hidden_size, gain=1.0):
                self.h, self.gain = hidden_size, gain

            def param_specs(self):
                return {"mix.weight": ParamSpec((self.h, self.h))}

            def state_request(self):
                return StateRequest((self.h,), torch.float32)

            def bind(self, params):
                self.w = params["mix.weight"].float()

            def forward(self, x, residual, ctx, io):
                t = 0
                for slot, start, n in zip(ctx.h_seq_slot, ctx.h_seq_start, ctx.h_seq_new):
                    sums = io.state[slot][None, :] + torch.cumsum(x[t:t + n].float(), 0)
                    count = torch.arange(start + 1, start + n + 1, device=x.device, dtype=torch.float32)[:, None]
                    residual[t:t + n] += self.gain * ((sums / count) @ self.w.t())
                    io.state[slot] = sums[-1]
                    t += n

    if "ToyForCausalLM" not in ARCHITECTURES:
        @register_architecture("ToyForCausalLM")
        @dataclass(frozen=True)
        class ToyConfig:
            hidden: int = 48
            vocab: int = 90
            eos_token_ids: tuple = ()

            @classmethod
            def from_dict(cls, d):
                return cls(d.get("hidden", 48), d.get("vocab", 90))

            def to_dict(self):
                return {"architectures": ["ToyForCausalLM"], "hidden": self.hidden, "vocab": self.vocab}

            def to_model_spec(self):
                H = self.hidden
                norm = lambda p: PartSpec("rms_norm", {"eps": 1e-5}, prefix=p)
                toy = LayerSpec("pre_norm", PartSpec("toy_running_mean", {"gain": 0.5}, prefix="l0.toy."),
                                PartSpec("swiglu", {"intermediate_size": 64}, prefix="l0.ffn."),
                                norm("l0.n1."), norm("l0.n2."))
                att = LayerSpec("pre_norm", PartSpec("gqa_attention", {
                    "num_heads": 3, "num_kv_heads": 1, "head_dim": 16, "qk_norm": False,
                    "position": {"kind": "rope_half_split", "theta": 100.0, "head_dim": 16, "n_rot": 8}},
                    prefix="l1.att."), PartSpec("swiglu", {"intermediate_size": 32}, prefix="l1.ffn."),
                    norm("l1.n1."), norm("l1.n2."))
                return ModelSpec("ToyForCausalLM", H, self.vocab, 512, (toy, att),
                                 (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)),
                                 PartSpec("token_embedding", {}, prefix="emb."), norm("out_norm."),
                                 PartSpec("lm_head", {"tied": True}, prefix="head."))
    return ARCHITECTURES["ToyForCausalLM"]


def toy_reference(t, ids, H):
    """Whole-sequence plain forward of the toy model (float32, CPU)."""
    T = len(ids)
    h = P.embed(t["emb.weight"], ids)
    pos = torch.arange(T)

    def toy_layer(h):
        x = P.rms_norm(h, t["l0.n1.weight"], 1e-5)
        mean = torch.cumsum(x, 0) / torch.arange(1, T + 1)[:, None]
        h = h + 0.5 * (mean @ t["l0.toy.mix.weight"].t())
        x = P.rms_norm(h, t["l0.n2.weight"], 1e-5)
        return h + P.linear(P.swiglu(P.linear(x, t["l0.ffn.gate_proj.weight"]), P.linear(x, t["l0.ffn.up_proj.weight"])),
                            t["l0.ffn.down_proj.weight"])

    def att_layer(h):
        x = P.rms_norm(h, t["l1.n1.weight"], 1e-5)
        q = P.linear(x, t["l1.att.q_proj.weight"]).reshape(T, 3, 16)
        k = P.linear(x, t["l1.att.k_proj.weight"]).reshape(T, 1, 16)
        v = P.linear(x, t["l1.att.v_proj.weight"]).reshape(T, 1, 16)
        q, k = P.rope_half_split(q, pos, 100.0, 8), P.rope_half_split(k, pos, 100.0, 8)
        h = h + P.linear(P.causal_attention(q, k, v).reshape(T, 48), t["l1.att.o_proj.weight"])
        x = P.rms_norm(h, t["l1.n2.weight"], 1e-5)
        return h + P.linear(P.swiglu(P.linear(x, t["l1.ffn.gate_proj.weight"]), P.linear(x, t["l1.ffn.up_proj.weight"])),
                            t["l1.ffn.down_proj.weight"])

    h = toy_layer(att_layer(toy_layer(h)))
    return P.linear(P.rms_norm(h, t["out_norm.weight"], 1e-5), t["emb.weight"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_toy_mixer_with_state_is_registered_built_and_stepped(dtype):
    from zlm_b200 import Engine, StepEntry
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import config_from_dict
    from zlm_b200.weights import random_tensors
    _register_toys()
    cfg = config_from_dict({"architectures": ["ToyForCausalLM"], "hidden": 48, "vocab": 90})
    t = random_tensors(DecoderModel(cfg.to_model_spec()).param_specs(), 3)
    for n in t:
        if "toy.mix" in n:
            t[n] = t[n] * 10        # make the state matter
    dev = {n: (v.to(dtype) if v.dim() == 2 else v).cuda() for n, v in t.items()}
    ref = {n: (v.to(dtype).float() if v.dim() == 2 else v) for n, v in t.items()}
    eng = Engine(cfg, dev, dtype, "cuda:0", max_tokens=1024, max_batch=4)
    assert not eng.decoder.use_graphs                       # the toy branches on the host
    assert sum(io.state is not None for io in eng.cache.ios) == 2
    g = torch.Generator().manual_seed(4)
    seqs = [torch.randint(0, 90, (n,), generator=g).tolist() for n in (70, 9)]
    want = [toy_reference(ref, s, 48) for s in seqs]
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    for round_ in range(2):                                 # the second round reuses slots: state starts at zero again
        slots = [eng.new_sequence() for _ in seqs]
        got = eng.step([StepEntry(sl, s[:5], list(range(5))) for sl, s in zip(slots, seqs)]).float().cpu()
        torch.testing.assert_close(got[:5], want[0][:5], **tol)
        torch.testing.assert_close(got[5:], want[1][:5], **tol)
        for i in range(5, 70):
            ents = [StepEntry(slots[0], [seqs[0][i]], [0])]
            if i < 9:
                ents.append(StepEntry(slots[1], [seqs[1][i]], [0]))
            got = eng.step(ents).float().cpu()
            torch.testing.assert_close(got[0], want[0][i], **tol)
            if i < 9:
                torch.testing.assert_close(got[1], want[1][i], **tol)
        toks = eng.generate([seqs[1][:4]], max_tokens=3).tokens     # the loop runs the toy too, without graphs
        assert len(toks[0]) == 3
        for sl in slots:
            eng.release(sl)
    eng.cache.check()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_parts_alone(dtype):
    """Norm, feed-forward, embedding and head built from the registries at sizes of
    their own and run outside any model."""
    from zlm_b200.kernels import get_kernels
    from zlm_b200.parts.base import Runtime, StepContext
    from zlm_b200.registry import EMBEDDINGS, FEED_FORWARDS, HEADS, NORMS
    rt = Runtime(torch.device("cuda:0"), dtype, get_kernels())
    pk = PlainKernels()
    g = torch.Generator().manual_seed(5)
    H, I, V, T = 88, 136, 203, 11
    x32 = torch.randn(T, H, generator=g)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)

    norm = NORMS["rms_norm"](size=H, eps=1e-4)
    norm.attach(rt)
    w = 1 + 0.1 * torch.randn(H, generator=g)
    norm.bind({"weight": w.cuda()})
    out = torch.empty(T, H, dtype=dtype, device="cuda")
    norm.forward(out, x32.cuda())
    torch.testing.assert_close(out.float().cpu(), P.rms_norm(x32, w, 1e-4), **tol)

    ffn = FEED_FORWARDS["swiglu"](hidden_size=H, intermediate_size=I)
    ffn.attach(rt)
    wg, wu, wd = (torch.randn(s, generator=g).mul(0.1).to(dtype) for s in ((I, H), (I, H), (H, I)))
    ffn.bind({"gate_proj.weight": wg.cuda(), "up_proj.weight": wu.cuda(), "down_proj.weight": wd.cuda()})
    xin = x32.to(dtype)
    res = torch.ones(T, H, device="cuda")
    ffn.forward(xin.cuda(), res, None)
    mid = P.swiglu(P.linear(xin.float(), wg.float()), P.linear(xin.float(), wu.float()))
    if dtype == torch.bfloat16:
        mid = mid.to(dtype).float()
    torch.testing.assert_close(res.cpu(), 1 + P.linear(mid, wd.float()), **tol)

    emb = EMBEDDINGS["token_embedding"](vocab_size=V, hidden_size=H)
    emb.attach(rt)
    table = torch.randn(V, H, generator=g).to(dtype)
    emb.bind({"weight": table.cuda()})
    ids = torch.tensor([0, V - 1, 17], dtype=torch.int32).cuda()
    e = torch.empty(3, H, device="cuda")
    emb.forward(e, ids)
    assert torch.equal(e.cpu(), table[[0, V - 1, 17]].float())

    head = HEADS["lm_head"](vocab_size=V, hidden_size=H, tied=True)
    head.attach(rt)
    head.tie(table.cuda())
    logits = torch.empty(T, V, device="cuda")
    head.forward(logits, xin.cuda())
    torch.testing.assert_close(logits.cpu(), P.linear(xin.float(), table.float()), atol=1e-4 if dtype == torch.float32 else 5e-2, rtol=1e-2)


def test_attention_part_alone_with_another_position_encoding():
    """The attention mixer with a position encoding that is not fused: a toy one
    that scales q and k by a position-dependent factor, applied between the norm
    and the cache write."""
    from zlm_b200.kernels import get_kernels
    from zlm_b200.cache import KVCache
    from zlm_b200.config import ScheduleEntry
    from zlm_b200.engine.batch import MetaLayout, MetaStager, StepEntry, make_context, plan_step
    from zlm_b200.parts.base import PositionEncoding, Runtime
    from zlm_b200.registry import MIXERS, POSITION_ENCODINGS, register_position_encoding

    if "toy_scale" not in POSITION_ENCODINGS:
        @register_position_encoding("toy_scale")
        class ToyScale(PositionEncoding):
            fused = False

            def __init__(self, rate):
                self.rate = rate

            def apply(self, q, k, ctx):
                f = (1.0 + self.rate * ctx.token_pos.float())[:, None]
                q.copy_((q.float() * f).to(q.dtype))
                if k is not None:
                    k.copy_((k.float() / f).to(k.dtype))

    H, nq, nkv, hd = 40, 4, 2, 16
    rt = Runtime(torch.device("cuda:0"), torch.float32, get_kernels())
    att = MIXERS["gqa_attention"](hidden_size=H, num_heads=nq, num_kv_heads=nkv, head_dim=hd, qk_norm=True,
                                  qk_norm_eps=1e-6, position={"kind": "toy_scale", "rate": 0.01})
    att.attach(rt)
    g = torch.Generator().manual_seed(6)
    w = {n: torch.randn(s.shape, generator=g) * (0.2 if len(s.shape) == 2 else 1.0) for n, s in att.param_specs().items()}
    att.bind({n: v.cuda() for n, v in w.items()})
    cache = KVCache([ScheduleEntry(0)], [att.cache_request()], [None], 256, 2, 256, torch.float32, "cuda:0")
    slot = cache.alloc_slot()
    layout = MetaLayout(256, 2)
    stager = MetaStager(layout, "cuda:0")
    T = 70
    x = torch.randn(T, H, generator=g)
    res = torch.zeros(T, H, device="cuda")
    for a, b in ((0, 50), (50, 70)):                       # two steps: the second reads what the first cached
        arrays, t, r, _ = plan_step([StepEntry(slot, [0] * (b - a), [])], cache.lengths, 10, layout)
        cache.reserve([(slot, b - a)])
        stager.upload(arrays, t, r)
        ctx = make_context(stager, arrays, t, r, rt.ws)
        att.forward(x[a:b].cuda(), res[a:b], ctx, cache.ios[0])
        cache.commit([(slot, b - a)])
    pos = torch.arange(T)
    q = P.head_rms_norm(P.linear(x, w["q_proj.weight"]).reshape(T, nq, hd), w["q_norm.weight"], 1e-6)
    k = P.head_rms_norm(P.linear(x, w["k_proj.weight"]).reshape(T, nkv, hd), w["k_norm.weight"], 1e-6)
    v = P.linear(x, w["v_proj.weight"]).reshape(T, nkv, hd)
    f = (1.0 + 0.01 * pos.float())[:, None, None]
    want = P.linear(P.causal_attention(q * f, k / f, v).reshape(T, nq * hd), w["o_proj.weight"])
    torch.testing.assert_close(res.cpu(), want, atol=2e-5, rtol=1e-4)


def test_toy_routed_feed_forward_in_one_layer_of_two():
    """A feed-forward with routing of its own (two experts, the router's argmax picks one
    per token), defined here, sits in the first layer of a two-layer model whose second
    layer keeps the dense SwiGLU: feed-forwards are chosen layer by layer, and the
    framework's files do not change.  (A toy: it is no model of anyone's.)"""
    from zlm_b200 import Engine, StepEntry
    from zlm_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from zlm_b200.parts.base import FeedForward, ParamSpec
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import ARCHITECTURES, FEED_FORWARDS, register_architecture, register_feed_forward
    from zlm_b200.weights import random_tensors

    if "toy_two_experts" not in FEED_FORWARDS:
        @register_feed_forward("toy_two_experts")
        class TwoExperts(FeedForward):
            graph_safe = False

            def __init__(self, hidden_size, width):
                self.h, self.w = hidden_size, width

            def param_specs(self):
                return {"router.weight": ParamSpec((2, self.h)), "up.weight": ParamSpec((2 * self.w, self.h)),
                        "down.weight": ParamSpec((2 * self.h, self.w))}

            def bind(self, params):
                self.router = params["router.weight"].float()
                self.up = params["up.weight"].float().view(2, self.w, self.h)
                self.down = params["down.weight"].float().view(2, self.h, self.w)

            def forward(self, x, residual, ctx):
                xf = x.float()
                pick = (xf @ self.router.t()).argmax(-1)                       # router logits in fp32
                for e in range(2):
                    rows = (pick == e).nonzero()[:, 0]
                    if rows.numel():
                        residual[rows] += torch.relu(xf[rows] @ self.up[e].t()) @ self.down[e].t()

    if "ToyRoutedForCausalLM" not in ARCHITECTURES:
        @register_architecture("ToyRoutedForCausalLM")
        @dataclass(frozen=True)
        class ToyRoutedConfig:
            eos_token_ids: tuple = ()

            @classmethod
            def from_dict(cls, d):
                return cls()

            def to_dict(self):
                return {"architectures": ["ToyRoutedForCausalLM"]}

            def to_model_spec(self):
                norm = lambda p: PartSpec("rms_norm", {"eps": 1e-5}, prefix=p)
                att = lambda p: PartSpec("gqa_attention", {
                    "num_heads": 2, "num_kv_heads": 1, "head_dim": 16, "qk_norm": True,
                    "position": {"kind": "rope_half_split", "theta": 1000.0, "head_dim": 16, "n_rot": 16}}, prefix=p)
                l0 = LayerSpec("pre_norm", att("l0.att."), PartSpec("toy_two_experts", {"width": 24}, prefix="l0.moe."),
                               norm("l0.n1."), norm("l0.n2."))
                l1 = LayerSpec("pre_norm", att("l1.att."), PartSpec("swiglu", {"intermediate_size": 40}, prefix="l1.ffn."),
                               norm("l1.n1."), norm("l1.n2."))
                return ModelSpec("ToyRoutedForCausalLM", 32, 70, 256, (l0, l1), (ScheduleEntry(0), ScheduleEntry(1)),
                                 PartSpec("token_embedding", {}, prefix="emb."), norm("out_norm."),
                                 PartSpec("lm_head", {"tied": False}, prefix="head."))

    cfg = ARCHITECTURES["ToyRoutedForCausalLM"]()
    t = random_tensors(DecoderModel(cfg.to_model_spec()).param_specs(), 7)
    for n in t:
        if "router" in n:
            t[n] = t[n] * 50            # clear decisions: no token sits on the fence
    eng = Engine(cfg, {n: v.cuda() for n, v in t.items()}, torch.float32, "cuda:0", max_tokens=512, max_batch=4)

    def reference(ids):
        T = len(ids)
        h = P.embed(t["emb.weight"], ids)
        pos = torch.arange(T)
        for l in ("l0", "l1"):
            x = P.rms_norm(h, t[f"{l}.n1.weight"], 1e-5)
            q = P.head_rms_norm(P.linear(x, t[f"{l}.att.q_proj.weight"]).reshape(T, 2, 16), t[f"{l}.att.q_norm.weight"], 1e-6)
            k = P.head_rms_norm(P.linear(x, t[f"{l}.att.k_proj.weight"]).reshape(T, 1, 16), t[f"{l}.att.k_norm.weight"], 1e-6)
            v = P.linear(x, t[f"{l}.att.v_proj.weight"]).reshape(T, 1, 16)
            q, k = P.rope_half_split(q, pos, 1000.0, 16), P.rope_half_split(k, pos, 1000.0, 16)
            h = h + P.linear(P.causal_attention(q, k, v).reshape(T, 32), t[f"{l}.att.o_proj.weight"])
            x = P.rms_norm(h, t[f"{l}.n2.weight"], 1e-5)
            if l == "l0":
                pick = (x @ t["l0.moe.router.weight"].t()).argmax(-1)
                up = t["l0.moe.up.weight"].view(2, 24, 32)
                down = t["l0.moe.down.weight"].view(2, 32, 24)
                y = torch.stack([torch.relu(x[i] @ up[pick[i]].t()) @ down[pick[i]].t() for i in range(T)])
                assert 0 < int(pick.sum()) < T, "both experts should be used"
                h = h + y
            else:
                h = h + P.linear(P.swiglu(P.linear(x, t["l1.ffn.gate_proj.weight"]), P.linear(x, t["l1.ffn.up_proj.weight"])),
                                 t["l1.ffn.down_proj.weight"])
        return P.linear(P.rms_norm(h, t["out_norm.weight"], 1e-5), t["head.weight"])

    g = torch.Generator().manual_seed(8)
    seqs = [torch.randint(0, 70, (n,), generator=g).tolist() for n in (40, 13)]
    slots = [eng.new_sequence() for _ in seqs]
    got = eng.step([StepEntry(sl, s[:10], list(range(10))) for sl, s in zip(slots, seqs)]).cpu()
    want = [reference(s) for s in seqs]
    torch.testing.assert_close(got[:10], want[0][:10], atol=2e-5, rtol=1e-4)
    torch.testing.assert_close(got[10:], want[1][:10], atol=2e-5, rtol=1e-4)
    for i in range(10, 13):                                    # then token by token, from the cache
        got = eng.step([StepEntry(sl, [s[i]], [0]) for sl, s in zip(slots, seqs)]).cpu()
        torch.testing.assert_close(got[0], want[0][i], atol=2e-5, rtol=1e-4)
        torch.testing.assert_close(got[1], want[1][i], atol=2e-5, rtol=1e-4)


def test_toy_mixer_with_a_cache_record_of_its_own_and_a_step_key():
    """A mixer that caches a small fp32 latent per token instead of keys and values (its pool
    has the record's shape and element type, whatever the compute dtype), attends over the
    latents of its sequence through the block table, and contributes a step key of its own
    to what a captured decode step is keyed by.  Defined here; no file of the package
    changes.  (A toy: it is no model of anyone's.)"""
    from zlm_b200 import Engine, StepEntry
    from zlm_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from zlm_b200.kernels import PAGE_TOKENS
    from zlm_b200.parts.base import CacheRequest, Mixer, ParamSpec
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import ARCHITECTURES, MIXERS, register_architecture, register_mixer
    from zlm_b200.weights import random_tensors

    D = 12
    if "toy_latent" not in MIXERS:
        @register_mixer("toy_latent")
        class LatentMixer(Mixer):
            """c_t = Wc x_t is cached; y_t = Wo sum_s softmax_s(c_t . c_s) c_s over s <= t."""
            graph_safe = False

            def __init__(self, hidden_size, latent):
                self.h, self.d = hidden_size, latent

            def param_specs(self):
                return {"down.weight": ParamSpec((self.d, self.h)), "up.weight": ParamSpec((self.h, self.d))}

            def cache_request(self):
                return CacheRequest(1, self.d, token_shape=(self.d,), dtype=torch.float32)

            def step_key(self, ctx):
                return ("toy_latent", ctx.max_len // 16)

            def bind(self, params):
                self.wc, self.wo = params["down.weight"].float(), params["up.weight"].float()

            def forward(self, x, residual, ctx, io):
                pool, table = io.cache.pool, io.cache.block_table
                assert pool.dtype == torch.float32 and tuple(pool.shape[1:]) == (PAGE_TOKENS, self.d)
                c = x.float() @ self.wc.t()
                t = 0
                for slot, start, n in zip(ctx.h_seq_slot, ctx.h_seq_start, ctx.h_seq_new):
                    pos = torch.arange(start, start + n, device=x.device)
                    pages = table[slot, (pos // PAGE_TOKENS).long()].long()
                    pool[pages, pos % PAGE_TOKENS] = c[t:t + n]
                    allpos = torch.arange(0, start + n, device=x.device)
                    hist = pool[table[slot, (allpos // PAGE_TOKENS).long()].long(), allpos % PAGE_TOKENS]   # [start+n, d]
                    s = c[t:t + n] @ hist.t()
                    s = s.masked_fill(allpos[None, :] > pos[:, None], float("-inf"))
                    residual[t:t + n] += (torch.softmax(s, -1) @ hist) @ self.wo.t()
                    t += n

    if "ToyLatentForCausalLM" not in ARCHITECTURES:
        @register_architecture("ToyLatentForCausalLM")
        @dataclass(frozen=True)
        class ToyLatentConfig:
            eos_token_ids: tuple = ()

            @classmethod
            def from_dict(cls, d):
                return cls()

            def to_dict(self):
                return {"architectures": ["ToyLatentForCausalLM"]}

            def to_model_spec(self):
                norm = lambda p: PartSpec("rms_norm", {"eps": 1e-5}, prefix=p)
                l0 = LayerSpec("pre_norm", PartSpec("toy_latent", {"latent": D}, prefix="l0.mix."),
                               PartSpec("swiglu", {"intermediate_size": 40}, prefix="l0.ffn."), norm("l0.n1."), norm("l0.n2."))
                l1 = LayerSpec("pre_norm", PartSpec("gqa_attention", {
                    "num_heads": 2, "num_kv_heads": 1, "head_dim": 16, "qk_norm": True,
                    "position": {"kind": "rope_half_split", "theta": 1000.0, "head_dim": 16, "n_rot": 16}}, prefix="l1.att."),
                    PartSpec("swiglu", {"intermediate_size": 40}, prefix="l1.ffn."), norm("l1.n1."), norm("l1.n2."))
                return ModelSpec("ToyLatentForCausalLM", 32, 70, 512, (l0, l1), (ScheduleEntry(0), ScheduleEntry(1)),
                                 PartSpec("token_embedding", {}, prefix="emb."), norm("out_norm."),
                                 PartSpec("lm_head", {"tied": False}, prefix="head."))

    cfg = ARCHITECTURES["ToyLatentForCausalLM"]()
    t = random_tensors(DecoderModel(cfg.to_model_spec()).param_specs(), 9)
    for n in t:
        if "l0.mix" in n:
            t[n] = t[n] * 20            # the latents matter, and their softmax is peaked
    dtype = torch.bfloat16
    dev = {n: (v.to(dtype) if v.dim() == 2 else v).cuda() for n, v in t.items()}
    ref = {n: (v.to(dtype).float() if v.dim() == 2 else v) for n, v in t.items()}
    eng = Engine(cfg, dev, dtype, "cuda:0", max_tokens=512, max_batch=2)
    assert len(eng.cache.groups) == 2 and {g.pool.dtype for g in eng.cache.groups} == {torch.float32, torch.bfloat16}

    def reference(ids):
        T = len(ids)
        h = P.embed(ref["emb.weight"], ids)
        pos = torch.arange(T)
        x = P.rms_norm(h, ref["l0.n1.weight"], 1e-5).to(dtype).float()
        c = x @ ref["l0.mix.down.weight"].t()
        s = (c @ c.t()).masked_fill(pos[None, :] > pos[:, None], float("-inf"))
        h = h + (torch.softmax(s, -1) @ c) @ ref["l0.mix.up.weight"].t()
        for l, mix in (("l0", False), ("l1", True)):
            if mix:
                x = P.rms_norm(h, ref["l1.n1.weight"], 1e-5)
                q = P.head_rms_norm(P.linear(x, ref["l1.att.q_proj.weight"]).reshape(T, 2, 16), ref["l1.att.q_norm.weight"], 1e-6)
                k = P.head_rms_norm(P.linear(x, ref["l1.att.k_proj.weight"]).reshape(T, 1, 16), ref["l1.att.k_norm.weight"], 1e-6)
                v = P.linear(x, ref["l1.att.v_proj.weight"]).reshape(T, 1, 16)
                q, k = P.rope_half_split(q, pos, 1000.0, 16), P.rope_half_split(k, pos, 1000.0, 16)
                h = h + P.linear(P.causal_attention(q, k, v).reshape(T, 32), ref["l1.att.o_proj.weight"])
            x = P.rms_norm(h, ref[f"{l}.n2.weight"], 1e-5)
            h = h + P.linear(P.swiglu(P.linear(x, ref[f"{l}.ffn.gate_proj.weight"]), P.linear(x, ref[f"{l}.ffn.up_proj.weight"])),
                             ref[f"{l}.ffn.down_proj.weight"])
        return P.linear(P.rms_norm(h, ref["out_norm.weight"], 1e-5), ref["head.weight"])

    g = torch.Generator().manual_seed(10)
    seqs = [torch.randint(0, 70, (n,), generator=g).tolist() for n in (80, 21)]
    want = [reference(s) for s in seqs]
    tol = dict(atol=4e-2, rtol=4e-2)
    for round_ in range(2):                                    # the second round takes the slots and pages of the first
        slots = [eng.new_sequence() for _ in seqs]
        got = eng.step([StepEntry(sl, s[:15], list(range(15))) for sl, s in zip(slots, seqs)]).float().cpu()
        torch.testing.assert_close(got[:15], want[0][:15], **tol)
        torch.testing.assert_close(got[15:], want[1][:15], **tol)
        keys = set()
        for i in range(15, 80):
            ents = [StepEntry(slots[0], [seqs[0][i]], [0])]
            if i < 21:
                ents.append(StepEntry(slots[1], [seqs[1][i]], [0]))
            got = eng.step(ents).float().cpu()
            torch.testing.assert_close(got[0], want[0][i], **tol)
            if i < 21:
                torch.testing.assert_close(got[1], want[1][i], **tol)
        for sl in slots:
            eng.release(sl)
        eng.cache.check()
    # the toy's key is part of what a captured decode step would be keyed by, beside the attention's
    from zlm_b200.engine.batch import make_context, plan_step
    s = eng.new_sequence()
    arrays, T_, R_, _ = plan_step([StepEntry(s, [1], [0])], eng.cache.lengths, 70, eng.layout)
    key = eng.model.step_key(make_context(eng.stager, arrays, T_, R_, eng.rt.ws))
    assert ("toy_latent", 0) in key and any(k[0] == "gqa_attention" for k in key)
    eng.release(s)


def test_a_norm_that_reads_the_stream_by_itself_sees_finished_products():
    """At layer widths where a few-token product is cut into shares of K, the parts leave their
    last product into the stream to the norm kernel that follows.  A norm defined here, which
    reads the stream with torch operations, is not that kernel: the arrangement has the product
    finished before it, so a model with this norm gives what the same model gives with the
    library's norm (the same weights by name), and the shares are in fact pending in between.
    (A toy: it is no model of anyone's.)"""
    from zlm_b200 import Engine, StepEntry
    from zlm_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from zlm_b200.parts.base import Norm, ParamSpec
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import ARCHITECTURES, NORMS, register_architecture, register_norm
    from zlm_b200.weights import random_tensors

    seen = {"pending": 0}
    if "toy_torch_rms" not in NORMS:
        @register_norm("toy_torch_rms")
        class TorchRms(Norm):
            graph_safe = False

            def __init__(self, size, eps):
                self.size, self.eps = size, eps

            def param_specs(self):
                return {"weight": ParamSpec((self.size,), kind="vector", init="one_plus_normal")}

            def bind(self, params):
                self.weight = params["weight"]

            def forward(self, out, x, rows=None):
                assert getattr(self.rt.k, "_shares", None) is None, "a product was still in shares when this norm read the stream"
                src = x if rows is None else x[rows.long()[: out.shape[0]]]
                y = src * torch.rsqrt(src.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()
                out.copy_(y.to(out.dtype))

    def spec(kind):
        norm = lambda p: PartSpec(kind, {"eps": 1e-6}, prefix=p)
        att = lambda p: PartSpec("gqa_attention", {
            "num_heads": 8, "num_kv_heads": 2, "head_dim": 128, "qk_norm": True,
            "position": {"kind": "rope_half_split", "theta": 10000.0, "head_dim": 128, "n_rot": 128}}, prefix=p)
        layers = tuple(LayerSpec("pre_norm", att(f"l{i}.att."), PartSpec("swiglu", {"intermediate_size": 2048}, prefix=f"l{i}.ffn."),
                                 norm(f"l{i}.n1."), norm(f"l{i}.n2.")) for i in range(2))
        return ModelSpec("ToyWide", 1024, 300, 512, layers, (ScheduleEntry(0), ScheduleEntry(1)),
                         PartSpec("token_embedding", {}, prefix="emb."), norm("out_norm."),
                         PartSpec("lm_head", {"tied": False}, prefix="head."))

    for name, kind in (("ToyWideTorchNormForCausalLM", "toy_torch_rms"), ("ToyWideForCausalLM", "rms_norm")):
        if name not in ARCHITECTURES:
            @register_architecture(name)
            @dataclass(frozen=True)
            class Cfg:
                eos_token_ids: tuple = ()
                _kind = kind
                _name = name

                @classmethod
                def from_dict(cls, d):
                    return cls()

                def to_dict(self):
                    return {"architectures": [self._name]}

                def to_model_spec(self):
                    return spec(self._kind)

    t = random_tensors(DecoderModel(spec("rms_norm")).param_specs(), 11)
    weights = {n: v.to(torch.bfloat16).cuda() if v.dim() > 1 else v.cuda() for n, v in t.items()}
    ids = torch.randint(0, 300, (40,), generator=torch.Generator().manual_seed(12)).tolist()
    logits = {}
    for name in ("ToyWideForCausalLM", "ToyWideTorchNormForCausalLM"):
        eng = Engine(ARCHITECTURES[name](), dict(weights), torch.bfloat16, "cuda:0", max_tokens=512, max_batch=2)
        k = eng.rt.k
        if name == "ToyWideForCausalLM":
            # the hint is taken at this width: watch one product being left in shares
            inner = k.rmsnorm
            def watched(out, x, w, eps, rows=None, _inner=inner, _k=k):
                seen["pending"] += _k._shares is not None
                return _inner(out, x, w, eps, rows)
            k.rmsnorm = watched
        sl = eng.new_sequence()
        logits[name] = eng.step([StepEntry(sl, ids, list(range(40)))]).float().cpu()
        eng.check(sync=True)
    assert seen["pending"] > 0, "no product was left in shares: this test would prove nothing"
    a, b = logits["ToyWideForCausalLM"], logits["ToyWideTorchNormForCausalLM"]
    assert float((a - b).norm() / a.norm()) < 2e-2
    assert (a.argmax(-1) == b.argmax(-1)).float().mean() > 0.9


def test_toy_block_arrangement_in_one_layer_of_two():
    """Another way of putting a mixer and a feed-forward on the stream, defined here: both read
    the same normed input and add into the stream side by side (h += mixer(n(h)) + ffn(n(h))).
    It sits in the first layer of a model whose second layer keeps the pre-norm arrangement;
    the framework's files do not change.  (A toy: it is no model of anyone's.)"""
    from zlm_b200 import Engine, StepEntry
    from zlm_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from zlm_b200.parts.base import Part
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import ARCHITECTURES, ARRANGEMENTS, register_architecture, register_arrangement
    from zlm_b200.weights import random_tensors

    if "toy_side_by_side" not in ARRANGEMENTS:
        @register_arrangement("toy_side_by_side")
        class SideBySide(Part):
            def __init__(self, hidden_size, mixer, feed_forward, mixer_norm, feed_forward_norm):
                self.mixer, self.ffn, self.norm, self.unused_norm = mixer, feed_forward, mixer_norm, feed_forward_norm

            def children(self):
                return {"mixer": self.mixer, "feed_forward": self.ffn, "mixer_norm": self.norm,
                        "feed_forward_norm": self.unused_norm}

            @property
            def graph_safe(self):
                return all(c.graph_safe for c in self.children().values())

            def step_key(self, ctx):
                return tuple(k for k in (c.step_key(ctx) for c in self.children().values()) if k is not None) or None

            def forward(self, hidden, ctx, io):
                x = self.rt.ws.get("toy.normed", hidden.shape, self.rt.dtype)
                self.norm.forward(x, hidden)
                self.mixer.forward(x, hidden, ctx, io)
                self.ffn.forward(x, hidden, ctx)          # the same normed input, the stream already holds the mixer's part

    if "ToySideBySideForCausalLM" not in ARCHITECTURES:
        @register_architecture("ToySideBySideForCausalLM")
        @dataclass(frozen=True)
        class ToySideBySideConfig:
            eos_token_ids: tuple = ()

            @classmethod
            def from_dict(cls, d):
                return cls()

            def to_dict(self):
                return {"architectures": ["ToySideBySideForCausalLM"]}

            def to_model_spec(self):
                norm = lambda p: PartSpec("rms_norm", {"eps": 1e-5}, prefix=p)
                att = lambda p: PartSpec("gqa_attention", {
                    "num_heads": 3, "num_kv_heads": 1, "head_dim": 16, "qk_norm": True,
                    "position": {"kind": "rope_half_split", "theta": 1000.0, "head_dim": 16, "n_rot": 16}}, prefix=p)
                ffn = lambda p: PartSpec("swiglu", {"intermediate_size": 56}, prefix=p)
                l0 = LayerSpec("toy_side_by_side", att("l0.att."), ffn("l0.ffn."), norm("l0.n1."), norm("l0.n2."))
                l1 = LayerSpec("pre_norm", att("l1.att."), ffn("l1.ffn."), norm("l1.n1."), norm("l1.n2."))
                return ModelSpec("ToySideBySideForCausalLM", 40, 77, 256, (l0, l1), (ScheduleEntry(0), ScheduleEntry(1)),
                                 PartSpec("token_embedding", {}, prefix="emb."), norm("out_norm."),
                                 PartSpec("lm_head", {"tied": False}, prefix="head."))

    cfg = ARCHITECTURES["ToySideBySideForCausalLM"]()
    t = random_tensors(DecoderModel(cfg.to_model_spec()).param_specs(), 21)
    eng = Engine(cfg, {n: v.cuda() for n, v in t.items()}, torch.float32, "cuda:0", max_tokens=512, max_batch=4)

    def attention(x, l, T):
        pos = torch.arange(T)
        q = P.head_rms_norm(P.linear(x, t[f"{l}.att.q_proj.weight"]).reshape(T, 3, 16), t[f"{l}.att.q_norm.weight"], 1e-6)
        k = P.head_rms_norm(P.linear(x, t[f"{l}.att.k_proj.weight"]).reshape(T, 1, 16), t[f"{l}.att.k_norm.weight"], 1e-6)
        v = P.linear(x, t[f"{l}.att.v_proj.weight"]).reshape(T, 1, 16)
        q, k = P.rope_half_split(q, pos, 1000.0, 16), P.rope_half_split(k, pos, 1000.0, 16)
        return P.linear(P.causal_attention(q, k, v).reshape(T, 48), t[f"{l}.att.o_proj.weight"])

    def mlp(x, l):
        return P.linear(P.swiglu(P.linear(x, t[f"{l}.ffn.gate_proj.weight"]), P.linear(x, t[f"{l}.ffn.up_proj.weight"])),
                        t[f"{l}.ffn.down_proj.weight"])

    def reference(ids):
        T = len(ids)
        h = P.embed(t["emb.weight"], ids)
        x = P.rms_norm(h, t["l0.n1.weight"], 1e-5)
        h = h + attention(x, "l0", T) + mlp(x, "l0")                       # side by side
        h = h + attention(P.rms_norm(h, t["l1.n1.weight"], 1e-5), "l1", T)   # then the usual order
        h = h + mlp(P.rms_norm(h, t["l1.n2.weight"], 1e-5), "l1")
        return P.linear(P.rms_norm(h, t["out_norm.weight"], 1e-5), t["head.weight"])

    g = torch.Generator().manual_seed(22)
    seqs = [torch.randint(0, 77, (n,), generator=g).tolist() for n in (30, 11)]
    slots = [eng.new_sequence() for _ in seqs]
    got = eng.step([StepEntry(sl, s[:9], list(range(9))) for sl, s in zip(slots, seqs)]).cpu()
    want = [reference(s) for s in seqs]
    torch.testing.assert_close(got[:9], want[0][:9], atol=2e-5, rtol=1e-4)
    torch.testing.assert_close(got[9:], want[1][:9], atol=2e-5, rtol=1e-4)
    for i in range(9, 11):                                     # then token by token, from the cache
        got = eng.step([StepEntry(sl, [s[i]], [0]) for sl, s in zip(slots, seqs)]).cpu()
        torch.testing.assert_close(got[0], want[0][i], atol=2e-5, rtol=1e-4)
        torch.testing.assert_close(got[1], want[1][i], atol=2e-5, rtol=1e-4)
    # and through the generation loop (graphs where the parts allow them)
    out = eng.generate([s[:5] for s in seqs], max_tokens=4)
    assert [len(x) for x in out.tokens] == [4, 4]


def test_toy_mixer_that_reads_its_input_by_products_has_its_norms_left_to_them():
    """A mixer defined here (no cache, no state: y = ((x A^T) * (x B^T)) C^T) says that it reads its
    input through the kernel object's products alone (``reads_input_by_products``) and adds into the
    stream with ``linear(accumulate=True, defer=True)``.  In steps of a few tokens the norms before
    it and after it then launch nothing: its two products take the norm's scale from the sums of
    squares that the product before left, and its last product leaves them for the feed-forward's
    norm.  Compared with a plain forward written here, and with the same engine when the norms run
    as kernels.  (A toy: it is no model of anyone's.)"""
    from zlm_b200 import Engine, StepEntry
    from zlm_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from zlm_b200.parts.base import Mixer, ParamSpec
    from zlm_b200.parts.model import DecoderModel
    from zlm_b200.registry import ARCHITECTURES, MIXERS, register_architecture, register_mixer
    from zlm_b200.weights import random_tensors
    H, I, V, L = 64, 96, 120, 3

    if "toy_two_products" not in MIXERS:
        @register_mixer("toy_two_products")
        class TwoProducts(Mixer):
            reads_input_by_products = True

            def __init__(self, hidden_size, inner):
                self.h, self.inner = hidden_size, inner

            def param_specs(self):
                return {n: ParamSpec(s) for n, s in (("a.weight", (self.inner, self.h)), ("b.weight", (self.inner, self.h)),
                                                     ("c.weight", (self.h, self.inner)))}

            def bind(self, params):
                self.a, self.b, self.c = params["a.weight"], params["b.weight"], params["c.weight"]

            def forward(self, x, residual, ctx, io):
                k, T = self.rt.k, x.shape[0]
                pa = ctx.scratch("toy2.a", (T, self.inner), x.dtype)
                pb = ctx.scratch("toy2.b", (T, self.inner), x.dtype)
                k.linear(pa, x, self.a)
                k.linear(pb, x, self.b)
                pa.mul_(pb)                                     # its own buffers: torch may have them
                k.linear(residual, pa, self.c, accumulate=True, defer=True)

    if "ToyTwoProductsForCausalLM" not in ARCHITECTURES:
        @register_architecture("ToyTwoProductsForCausalLM")
        @dataclass(frozen=True)
        class Cfg:
            eos_token_ids: tuple = ()

            @classmethod
            def from_dict(cls, d):
                return cls()

            def to_dict(self):
                return {"architectures": ["ToyTwoProductsForCausalLM"]}

            def to_model_spec(self):
                norm = lambda p: PartSpec("rms_norm", {"eps": 1e-5}, prefix=p)
                layers = tuple(LayerSpec("pre_norm", PartSpec("toy_two_products", {"inner": I}, prefix=f"l{i}.mix."),
                                         PartSpec("swiglu", {"intermediate_size": I}, prefix=f"l{i}.ffn."),
                                         norm(f"l{i}.n1."), norm(f"l{i}.n2.")) for i in range(L))
                return ModelSpec("ToyTwoProductsForCausalLM", H, V, 512, layers, tuple(ScheduleEntry(i) for i in range(L)),
                                 PartSpec("token_embedding", {}, prefix="emb."), norm("out_norm."),
                                 PartSpec("lm_head", {"tied": True}, prefix="head."))

    cfg = ARCHITECTURES["ToyTwoProductsForCausalLM"]()
    t = random_tensors(DecoderModel(cfg.to_model_spec()).param_specs(), 17)
    for n in t:
        if ".mix." in n:
            t[n] = t[n] * 20                # so that the mixer's share of the stream is not lost in rounding
    ref = {n: (v.to(torch.bfloat16).float() if v.dim() == 2 else v) for n, v in t.items()}
    dev = {n: (v.to(torch.bfloat16) if v.dim() == 2 else v).cuda() for n, v in t.items()}

    def plain(ids):
        h = P.embed(ref["emb.weight"], ids)
        for i in range(L):
            x = P.rms_norm(h, ref[f"l{i}.n1.weight"], 1e-5)
            h = h + P.linear(P.linear(x, ref[f"l{i}.mix.a.weight"]) * P.linear(x, ref[f"l{i}.mix.b.weight"]),
                             ref[f"l{i}.mix.c.weight"])
            x = P.rms_norm(h, ref[f"l{i}.n2.weight"], 1e-5)
            h = h + P.linear(P.swiglu(P.linear(x, ref[f"l{i}.ffn.gate_proj.weight"]), P.linear(x, ref[f"l{i}.ffn.up_proj.weight"])),
                             ref[f"l{i}.ffn.down_proj.weight"])
        return P.linear(P.rms_norm(h, ref["out_norm.weight"], 1e-5), ref["emb.weight"])

    eng = Engine(cfg, dev, torch.bfloat16, "cuda:0", max_tokens=256, max_batch=2)
    k = eng.rt.k
    ids = torch.randint(0, V, (30,), generator=torch.Generator().manual_seed(18)).tolist()
    want = plain(ids)
    got, launches = {}, {}
    for lazy in (True, False):
        k.lazy_norms = lazy
        sl = eng.new_sequence()
        eng.step([StepEntry(sl, ids[:21], [])])                 # 21 tokens: the other products, every norm a kernel
        before = k._launches
        got[lazy] = eng.step([StepEntry(sl, ids[21:], list(range(9)))]).float().cpu()      # 9 tokens: streaming products
        launches[lazy] = k._launches - before
        eng.release(sl)
    k.lazy_norms = True
    assert launches[False] - launches[True] == 2 * L - 1, launches        # every norm but the first and the last
    for lazy in (True, False):
        rel = (got[lazy] - want[21:]).norm(dim=-1) / want[21:].norm(dim=-1)
        assert float(rel.max()) < 2e-2, (lazy, rel)
    eng.check(sync=True)
