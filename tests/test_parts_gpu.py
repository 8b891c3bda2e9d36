"""Each part alone against its plain formula, and the generality of the composition: a toy mixer with
state of its own, a layer run twice and a layer that reads another layer's cache, all defined here and
run through the unchanged step function."""
import json
import math

import pytest
import torch

import plain_llama as P
import util

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_rmsnorm_part_keeps_a_32bit_weight():
    from lmsf_b200.parts.norm import RMSNorm
    n = RMSNorm(hidden_size=100, eps=1e-6)
    assert n.weight_specs()["weight"].keep_fp32
    g = torch.Generator().manual_seed(0)
    w = 1 + 0.2 * torch.randn(100, generator=g)
    x = torch.randn(5, 100, generator=g).bfloat16()
    n.set_weights({"weight": w.to(DEV)})                       # float32 weight under bfloat16 activations
    h, res = n.forward_residual(x.to(DEV), None)
    assert res.dtype == torch.float32 and torch.equal(res.cpu(), x.float())
    assert torch.allclose(h.float().cpu(), P.rms_norm(x.float(), w, 1e-6), rtol=1e-2, atol=1e-2)
    h2, res2 = n.forward_residual(x.to(DEV), res)
    assert res2 is res and torch.equal(res.cpu(), x.float() * 2)
    # the (1 + w) form of other architectures: the offset is folded into the weight when it is set
    n1 = RMSNorm(hidden_size=100, eps=1e-6, weight_offset=1.0)
    n1.set_weights({"weight": (w - 1).to(DEV)})
    assert torch.allclose(n1.forward(x.to(DEV)).float().cpu(), P.rms_norm(x.float(), w, 1e-6), rtol=1e-2, atol=1e-2)


def test_rotary_part_frequencies_match_the_plain_rule():
    from lmsf_b200.parts.rope import RotaryEmbedding
    for cfg in (util.TINY_A, util.TINY_B):
        hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
        sc = cfg.get("rope_scaling") or {}
        r = RotaryEmbedding(rot_dim=hd, theta=cfg["rope_theta"], scaling_type=sc.get("rope_type", "default"),
                            factor=sc.get("factor", 1.0), low_freq_factor=sc.get("low_freq_factor", 1.0),
                            high_freq_factor=sc.get("high_freq_factor", 4.0),
                            original_max_position_embeddings=sc.get("original_max_position_embeddings", 8192))
        r.prepare(torch.float32, torch.device(DEV))
        inv, rot, neox = r.fused_rotary()
        assert rot == hd and neox and torch.equal(inv.cpu(), P.rope_inv_freq(cfg).float())


def test_linear_and_mlp_parts():
    from lmsf_b200.parts.linear import Linear
    from lmsf_b200.parts.mlp import GatedMLP
    g = torch.Generator().manual_seed(1)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
        lin = Linear(in_features=72, out_features=[40, 24])
        assert lin.weight_specs()["weight"].shapes == [(40, 72), (24, 72)]
        w = (torch.randn(64, 72, generator=g) * 0.2).to(dtype)
        x = torch.randn(9, 72, generator=g).to(dtype)
        lin.set_weights({"weight": w.to(DEV)})
        assert torch.allclose(lin.forward(x.to(DEV)).float().cpu(), x.float() @ w.float().T, rtol=tol, atol=tol)
        head = Linear(in_features=72, out_features=64, out_dtype="float32")
        head.set_weights({"weight": w.to(DEV)})
        y = head.forward(x.to(DEV))
        assert y.dtype == torch.float32 and torch.allclose(y.cpu(), x.float() @ w.float().T, rtol=1e-4, atol=1e-4)
        mlp = GatedMLP(hidden_size=72, intermediate_size=100)
        gu = (torch.randn(200, 72, generator=g) * 0.2).to(dtype)
        dn = (torch.randn(72, 100, generator=g) * 0.2).to(dtype)
        mlp.set_weights({"gate_up": gu.to(DEV), "down": dn.to(DEV)})
        ref = P.silu_gated_mlp(x.float(), gu[:100].float(), gu[100:].float(), dn.float())
        assert torch.allclose(mlp.forward(None, x.to(DEV)).float().cpu(), ref, rtol=tol, atol=tol)


# ----------------------------------------------------------------------------- a toy architecture, defined here

def _register_toy():
    from lmsf_b200.config.registry import register_architecture
    from lmsf_b200.parts.base import (LayerCall, LayerSpec, Mixer, ModelSpec, PartSpec, StateSpec, WeightSpec,
                                      register_part)
    from lmsf_b200.parts.linear import matmul_tn

    @register_part("mixer", "toy_decay")
    class ToyDecayMixer(Mixer):
        """s_t = decay * s_{t-1} + h_t W_in^T ; out_t = s_t W_out^T.  Its state is one vector per request."""

        def __init__(self, hidden_size, state_size, decay):
            self.hidden_size, self.state_size, self.decay = hidden_size, state_size, decay

        def weight_specs(self):
            return {"w_in": WeightSpec([(self.state_size, self.hidden_size)]),
                    "w_out": WeightSpec([(self.hidden_size, self.state_size)])}

        def state_spec(self):
            return StateSpec((self.state_size,))

        def forward(self, ctx, h, cache):
            u = matmul_tn(h, self.w_in).float()
            out = torch.empty_like(u)
            off = 0
            for n, slot in zip(ctx.q_lens, ctx.state_slots):
                s = cache.state[slot]
                for t in range(off, off + n):
                    s = self.decay * s + u[t]
                    out[t] = s
                cache.state[slot] = s
                off += n
            return matmul_tn(out.to(h.dtype), self.w_out)

    def parse(d):
        return dict(d)

    def spec(c):
        H = c["hidden_size"]
        norm = lambda name: PartSpec("rmsnorm", dict(hidden_size=H, eps=c["eps"]), {"weight": name})
        rope = PartSpec("rotary", dict(rot_dim=c["head_dim"] // 2, theta=100.0, is_neox=False))   # partial, interleaved
        def attn(i, window=None):
            p = f"l{i}."
            return PartSpec("paged_attention", dict(hidden_size=H, num_heads=c["heads"], num_kv_heads=c["kv_heads"],
                                                    head_dim=c["head_dim"], position_encoding=rope, window=window),
                            {"qkv": [p + "q", p + "k", p + "v"], "o": p + "o"})
        def mlp(i):
            return PartSpec("gated_mlp", dict(hidden_size=H, intermediate_size=c["inter"], activation="gelu_tanh"),
                            {"gate_up": [f"l{i}.g", f"l{i}.u"], "down": f"l{i}.d"})
        def layer(i, mixer):
            return LayerSpec("pre_norm", {"mixer_norm": norm(f"l{i}.n1"), "mixer": mixer, "ffn_norm": norm(f"l{i}.n2"),
                                          "feed_forward": mlp(i)})
        layers = [layer(0, attn(0)),
                  layer(1, PartSpec("toy_decay", dict(hidden_size=H, state_size=c["state"], decay=c["decay"]),
                                    {"w_in": "l1.in", "w_out": "l1.out"})),
                  layer(2, attn(2, window=c["window"])),
                  layer(3, attn(3))]
        # layer 0 runs twice (each run has a cache of its own); the last call reads the first call's cache
        order = [LayerCall(0), LayerCall(1), LayerCall(2), LayerCall(0), LayerCall(3, cache_of=0)]
        return ModelSpec(hidden_size=H, vocab_size=c["vocab"], max_model_len=c["max_len"],
                         embedding=PartSpec("token_embedding", dict(vocab_size=c["vocab"], hidden_size=H), {"weight": "emb"}),
                         layers=layers, order=order, final_norm=norm("nf"),
                         lm_head=PartSpec("dense", dict(in_features=H, out_features=c["vocab"], out_dtype="float32"),
                                          {"weight": "emb"}))

    register_architecture("ToyMixedForTests", parse, spec)


TOY = dict(architectures=["ToyMixedForTests"], hidden_size=48, heads=3, kv_heads=1, head_dim=32, inter=56, vocab=97,
           state=20, decay=0.8, eps=1e-5, window=9, max_len=256)


def _toy_reference(model, ids):
    """The toy model on whole sequences with the plain functions."""
    c = TOY
    W = lambda t: t.float().cpu()
    x = P.embedding(W(model.embedding.weight), torch.tensor(ids))
    T = len(ids)
    pos = torch.arange(T)
    kv_of_call = {}

    def attn(m, h, j, read_from=None):
        nh, nkv, hd = m.num_heads, m.num_kv_heads, m.head_dim
        qkv = h @ W(m.qkv).T
        q = qkv[:, :nh * hd].reshape(T, nh, hd)
        k = qkv[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd)
        v = qkv[:, (nh + nkv) * hd:].reshape(T, nkv, hd)
        rot = hd // 2
        inv = torch.tensor([100.0 ** (-(2.0 * i) / rot) for i in range(rot // 2)], dtype=torch.float64)
        ang = pos.float()[:, None] * inv.float()[None, :]
        cs, sn = ang.cos()[:, None, :], ang.sin()[:, None, :]

        def rotate(z):
            a, b = z[..., 0:rot:2], z[..., 1:rot:2]
            y = torch.stack([a * cs - b * sn, b * cs + a * sn], dim=-1).reshape(*z.shape[:-1], rot)
            return torch.cat([y, z[..., rot:]], dim=-1)
        q = rotate(q)
        if read_from is None:
            kv_of_call[j] = (rotate(k), v)
            k, v = kv_of_call[j]
        else:
            k, v = kv_of_call[read_from]
        o = P.causal_attention(q, k, v, 1.0 / math.sqrt(hd), m.window)
        return o.reshape(T, nh * hd) @ W(m.o).T

    def decay(m, h):
        u = h @ W(m.w_in).T
        s, out = torch.zeros(m.state_size), []
        for t in range(T):
            s = m.decay * s + u[t]
            out.append(s)
        return torch.stack(out) @ W(m.w_out).T

    for j, call in enumerate(model.calls):
        blk = model.blocks[call.layer]
        h = P.rms_norm(x, W(blk.mixer_norm.weight), c["eps"])
        m = blk.mixer
        a = decay(m, h) if hasattr(m, "decay") else attn(m, h, j, call.cache_of)
        x = x + a
        h = P.rms_norm(x, W(blk.ffn_norm.weight), c["eps"])
        ff = blk.feed_forward
        gu = h @ W(ff.gate_up).T
        I = ff.intermediate_size
        x = x + (torch.nn.functional.gelu(gu[:, :I], approximate="tanh") * gu[:, I:]) @ W(ff.down).T
    return P.rms_norm(x, W(model.final_norm.weight), c["eps"]) @ W(model.lm_head.weight).T


@pytest.mark.parametrize("dtype,rel", [("float32", 2e-5), ("bfloat16", 6e-2)])
def test_toy_architecture_is_registered_built_and_stepped(tmp_path, dtype, rel):
    import traces
    from lmsf_b200.cache.storage import plan_groups
    from lmsf_b200.engine.factory import build_model
    _register_toy()
    (tmp_path / "config.json").write_text(json.dumps(TOY))
    model, _, tdt = build_model(str(tmp_path), dtype, DEV, load_format="dummy", seed=3)
    for part, _ in model.parts_with_specs():                      # larger weights: attention must matter
        for name in part.weight_specs():
            if not part.weight_specs()[name].keep_fp32:
                getattr(part, name).mul_(6.0)
    groups, where = plan_groups(model)
    assert [(g.spec.window, g.calls) for g in groups] == [(None, [0, 3]), (9, [2])]    # two page pools
    assert where[4] == where[0]                                                        # the shared cache
    reqs = {f"t{i}": util.random_ids(n, TOY["vocab"], 40 + i) for i, n in enumerate([37, 5, 61, 18, 44])}
    ref = {rid: _toy_reference(model, toks).numpy() for rid, toks in reqs.items()}
    traces._runners[(str(tmp_path), dtype)] = (model, None, tdt)
    results = {}
    for mode, steps in {"whole": traces.whole(reqs), "portions": traces.portions(reqs, [5, 2, 11, 3]),
                        "mixed": traces.mixed(reqs, seed=2, max_live=3, tail=8)}.items():
        out = traces.run_inprocess(str(tmp_path), dtype, steps, 8, traces.max_live_tokens(steps, 8), max_live=3)
        results[mode] = traces.collect(steps, out)
        scale = max(1.0, max(float(abs(r).max()) for r in ref.values()))
        worst = max(float(abs(row - ref[rid][pos]).max()) for (rid, pos), row in results[mode].items())
        assert worst <= rel * scale, (mode, worst, scale)


# ----------------------------------------------------------------------------- a toy with state whose decode steps are replayed from a graph

def _register_toy_graph_state():
    from lmsf_b200.config.registry import register_architecture
    from lmsf_b200.parts.base import LayerCall, LayerSpec, Mixer, ModelSpec, PartSpec, StateSpec, WeightSpec, register_part
    from lmsf_b200.parts.linear import matmul_tn

    @register_part("mixer", "toy_decay_on_device")
    class ToyDecayOnDevice(Mixer):
        """The recurrence of toy_decay with every index taken from device tensors, so that a step of single tokens
        does the same work whatever the requests are and may be replayed from a CUDA graph."""
        graph_safe = True

        def __init__(self, hidden_size, state_size, decay):
            self.hidden_size, self.state_size, self.decay = hidden_size, state_size, decay

        def weight_specs(self):
            return {"w_in": WeightSpec([(self.state_size, self.hidden_size)]),
                    "w_out": WeightSpec([(self.hidden_size, self.state_size)])}

        def state_spec(self):
            return StateSpec((self.state_size,))

        def forward(self, ctx, h, cache):
            u = matmul_tn(h, self.w_in).float()
            if ctx.n_tokens == ctx.n_seqs:                       # one token per request: all on the device
                slots = ctx.state_slot.long()
                s = self.decay * cache.state.index_select(0, slots) + u
                cache.state.index_copy_(0, slots, s)
                return matmul_tn(s.to(h.dtype), self.w_out)
            out, off = torch.empty_like(u), 0
            for n, slot in zip(ctx.q_lens, ctx.state_slots):
                s = cache.state[slot]
                for t in range(off, off + n):
                    s = self.decay * s + u[t]
                    out[t] = s
                cache.state[slot] = s
                off += n
            return matmul_tn(out.to(h.dtype), self.w_out)

    def spec(c):
        H = c["hidden_size"]
        norm = lambda name: PartSpec("rmsnorm", dict(hidden_size=H, eps=c["eps"]), {"weight": name})
        layer = LayerSpec("pre_norm", {
            "mixer_norm": norm("n1"),
            "mixer": PartSpec("toy_decay_on_device", dict(hidden_size=H, state_size=c["state"], decay=c["decay"]),
                              {"w_in": "in", "w_out": "out"}),
            "ffn_norm": norm("n2"),
            "feed_forward": PartSpec("gated_mlp", dict(hidden_size=H, intermediate_size=c["inter"]),
                                     {"gate_up": ["g", "u"], "down": "d"})})
        return ModelSpec(hidden_size=H, vocab_size=c["vocab"], max_model_len=c["max_len"],
                         embedding=PartSpec("token_embedding", dict(vocab_size=c["vocab"], hidden_size=H), {"weight": "emb"}),
                         layers=[layer], order=[LayerCall(0)], final_norm=norm("nf"),
                         lm_head=PartSpec("dense", dict(in_features=H, out_features=c["vocab"], out_dtype="float32"),
                                          {"weight": "emb"}))

    register_architecture("ToyGraphStateForTests", dict, spec)


def test_a_stateful_mixer_in_replayed_decode_steps_keeps_every_request_state(tmp_path):
    """Three requests decode together; the batch is padded to four with a stand-in request and replayed from a
    CUDA graph.  The stand-in's state must go to a slot of its own: each request's logits must equal those it
    gets when it runs alone, step by step, without a graph."""
    from lmsf_b200.engine.factory import build_model
    from lmsf_b200.engine.model_runner import ModelRunner, StepEntry
    _register_toy_graph_state()
    cfg = dict(architectures=["ToyGraphStateForTests"], hidden_size=40, state=24, decay=0.9, inter=56, vocab=61,
               eps=1e-5, max_len=64)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    model, _, tdt = build_model(str(tmp_path), "float32", DEV, load_format="dummy", seed=5)
    reqs = {f"s{i}": util.random_ids(14, cfg["vocab"], 70 + i) for i in range(3)}

    def run(group, enforce_eager):
        runner = ModelRunner(model, tdt, torch.device(DEV), 8, num_blocks=8, max_num_seqs=4, enforce_eager=enforce_eager)
        mgr = runner.make_cache_manager()
        for rid in group:
            mgr.add(rid)
        rows = {rid: [] for rid in group}
        lg = runner.step([StepEntry(rid, reqs[rid][:4], [3]) for rid in group], mgr)        # a prompt portion each
        for j, rid in enumerate(group):
            rows[rid].append(lg[j].cpu())
        for t in range(4, 14):                                                               # then one token a step
            lg = runner.step([StepEntry(rid, [reqs[rid][t]], [0]) for rid in group], mgr)
            for j, rid in enumerate(group):
                rows[rid].append(lg[j].cpu())
        replayed = len(runner._graphs)
        for rid in group:
            mgr.free(rid)
        return rows, replayed

    together, replayed = run(list(reqs), enforce_eager=False)
    assert replayed > 0                           # the steps of three requests ran from a graph of four
    for rid in reqs:
        alone, _ = run([rid], enforce_eager=True)
        for a, b in zip(together[rid], alone[rid]):
            assert torch.allclose(a, b, rtol=1e-5, atol=1e-6), rid


# ----------------------------------------------------------------------------- a second toy: routing and another position encoding

def _register_toy_routed():
    from lmsf_b200.config.registry import register_architecture
    from lmsf_b200.parts.base import (FeedForward, LayerCall, LayerSpec, ModelSpec, PartSpec, PositionEncoding, WeightSpec,
                                      register_part)
    from lmsf_b200.parts.linear import matmul_tn

    @register_part("position_encoding", "toy_learned_shift")
    class ToyLearnedShift(PositionEncoding):
        """q and k of every head get a learned vector of their position added (no rotation: the cache-write
        kernel cannot apply it, so the attention part calls apply() before it writes k)."""

        def __init__(self, max_positions, head_dim):
            self.max_positions, self.head_dim = max_positions, head_dim

        def weight_specs(self):
            return {"table": WeightSpec([(self.max_positions, self.head_dim)])}

        def apply(self, ctx, q, k, n_q_heads, n_kv_heads, head_dim):
            shift = self.table[ctx.positions.long()]                       # [n, head_dim]
            q.view(-1, n_q_heads, head_dim).add_(shift[:, None, :])
            if k is not None:
                k.view(-1, n_kv_heads, head_dim).add_(shift[:, None, :])

    @register_part("feed_forward", "toy_top1_experts")
    class ToyTop1Experts(FeedForward):
        """Router logits in float32; every token goes through the one expert with the largest logit, scaled by
        its softmax weight."""

        def __init__(self, hidden_size, inter, n_experts):
            self.hidden_size, self.inter, self.n_experts = hidden_size, inter, n_experts

        def weight_specs(self):
            return {"router": WeightSpec([(self.n_experts, self.hidden_size)]),
                    "up": WeightSpec([(self.n_experts * self.inter, self.hidden_size)]),
                    "down": WeightSpec([(self.n_experts * self.hidden_size, self.inter)])}

        def forward(self, ctx, h):
            logits = h.float() @ self.router.float().T
            weight, expert = torch.softmax(logits, dim=-1).max(dim=-1)
            out = torch.zeros_like(h)
            for e in range(self.n_experts):
                rows = (expert == e).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                up = self.up[e * self.inter:(e + 1) * self.inter]
                down = self.down[e * self.hidden_size:(e + 1) * self.hidden_size]
                m = torch.relu(matmul_tn(h[rows].contiguous(), up))
                out[rows] = (matmul_tn(m, down).float() * weight[rows, None]).to(h.dtype)
            return out

    def spec(c):
        H = c["hidden_size"]
        norm = lambda name: PartSpec("rmsnorm", dict(hidden_size=H, eps=c["eps"]), {"weight": name})
        def layer(i):
            shift = PartSpec("toy_learned_shift", dict(max_positions=c["max_len"], head_dim=c["head_dim"]), {"table": f"l{i}.pos"})
            attn = PartSpec("paged_attention", dict(hidden_size=H, num_heads=c["heads"], num_kv_heads=c["kv_heads"],
                                                    head_dim=c["head_dim"], position_encoding=shift),
                            {"qkv": [f"l{i}.q", f"l{i}.k", f"l{i}.v"], "o": f"l{i}.o"})
            ffn = PartSpec("toy_top1_experts", dict(hidden_size=H, inter=c["inter"], n_experts=c["experts"]),
                           {"router": f"l{i}.r", "up": f"l{i}.u", "down": f"l{i}.d"})
            return LayerSpec("pre_norm", {"mixer_norm": norm(f"l{i}.n1"), "mixer": attn, "ffn_norm": norm(f"l{i}.n2"),
                                          "feed_forward": ffn})
        n = c["layers"]
        return ModelSpec(hidden_size=H, vocab_size=c["vocab"], max_model_len=c["max_len"],
                         embedding=PartSpec("token_embedding", dict(vocab_size=c["vocab"], hidden_size=H), {"weight": "emb"}),
                         layers=[layer(i) for i in range(n)], order=[LayerCall(i) for i in range(n)], final_norm=norm("nf"),
                         lm_head=PartSpec("dense", dict(in_features=H, out_features=c["vocab"], out_dtype="float32"),
                                          {"weight": "head"}))

    register_architecture("ToyRoutedForTests", dict, spec)


TOY_ROUTED = dict(architectures=["ToyRoutedForTests"], hidden_size=40, heads=4, kv_heads=2, head_dim=16, inter=24, experts=3,
                  layers=2, vocab=83, eps=1e-6, max_len=128)


def _toy_routed_reference(model, ids):
    c = TOY_ROUTED
    W = lambda t: t.float().cpu()
    x = P.embedding(W(model.embedding.weight), torch.tensor(ids))
    T = len(ids)
    for blk in model.blocks:
        m, ff = blk.mixer, blk.feed_forward
        h = P.rms_norm(x, W(blk.mixer_norm.weight), c["eps"])
        nh, nkv, hd = m.num_heads, m.num_kv_heads, m.head_dim
        qkv = h @ W(m.qkv).T
        shift = W(m.position_encoding.table)[:T]
        q = qkv[:, :nh * hd].reshape(T, nh, hd) + shift[:, None, :]
        k = qkv[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd) + shift[:, None, :]
        v = qkv[:, (nh + nkv) * hd:].reshape(T, nkv, hd)
        x = x + P.causal_attention(q, k, v, 1.0 / math.sqrt(hd), None).reshape(T, nh * hd) @ W(m.o).T
        h = P.rms_norm(x, W(blk.ffn_norm.weight), c["eps"])
        weight, expert = torch.softmax(h @ W(ff.router).T, dim=-1).max(dim=-1)
        out = torch.zeros_like(h)
        for t in range(T):
            e = int(expert[t])
            up, down = W(ff.up)[e * ff.inter:(e + 1) * ff.inter], W(ff.down)[e * ff.hidden_size:(e + 1) * ff.hidden_size]
            out[t] = (torch.relu(h[t] @ up.T) @ down.T) * weight[t]
        x = x + out
    return P.rms_norm(x, W(model.final_norm.weight), c["eps"]) @ W(model.lm_head.weight).T


def test_toy_routing_and_another_position_encoding_need_no_change_to_the_package(tmp_path):
    """A feed-forward that routes tokens to experts and a position encoding that is no rotation, both defined here."""
    import traces
    from lmsf_b200.engine.factory import build_model
    _register_toy_routed()
    (tmp_path / "config.json").write_text(json.dumps(TOY_ROUTED))
    model, _, tdt = build_model(str(tmp_path), "float32", DEV, load_format="dummy", seed=5)
    for part, _ in model.parts_with_specs():
        for name, ws in part.weight_specs().items():
            getattr(part, name).mul_(8.0 if name != "router" else 40.0)        # attention and the routing must matter
    reqs = {f"t{i}": util.random_ids(n, TOY_ROUTED["vocab"], 70 + i) for i, n in enumerate([29, 3, 50, 17])}
    ref = {rid: _toy_routed_reference(model, toks).numpy() for rid, toks in reqs.items()}
    experts_used = set()
    for blk in model.blocks:      # the routing is not trivial: more than one expert is chosen
        experts_used |= set(torch.randn(64, TOY_ROUTED["hidden_size"], device=DEV).matmul(blk.feed_forward.router.float().T).argmax(-1).tolist())
    assert len(experts_used) > 1
    traces._runners[(str(tmp_path), "float32")] = (model, None, tdt)
    for mode, steps in {"whole": traces.whole(reqs), "portions": traces.portions(reqs, [4, 2, 9]),
                        "mixed": traces.mixed(reqs, seed=4, max_live=3, tail=6)}.items():
        out = traces.run_inprocess(str(tmp_path), "float32", steps, 8, traces.max_live_tokens(steps, 8), max_live=3)
        rows = traces.collect(steps, out)
        scale = max(1.0, max(float(abs(r).max()) for r in ref.values()))
        worst = max(float(abs(row - ref[rid][pos]).max()) for (rid, pos), row in rows.items())
        assert worst <= 5e-5 * scale, (mode, worst, scale)


def _hand_context(q_lens, ctx_lens, block_size, n_pages, seed=0):
    """A StepContext and block table made by hand, the way ModelRunner lays a batch out."""
    from lmsf_b200.parts.base import CacheGroupView, StepContext
    g = torch.Generator().manual_seed(seed)
    S, N = len(q_lens), sum(q_lens)
    max_blocks = max((c + block_size - 1) // block_size for c in ctx_lens)
    perm = torch.randperm(n_pages, generator=g).tolist()
    bt = torch.full((S, max_blocks), -1, dtype=torch.int32)
    for s, c in enumerate(ctx_lens):
        for i in range((c + block_size - 1) // block_size):
            bt[s, i] = perm.pop()
    dev = torch.device(DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    positions = [p for c, n in zip(ctx_lens, q_lens) for p in range(c - n, c)]
    token_seq = [s for s, n in enumerate(q_lens) for _ in range(n)]
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    tiles = [(s, q0) for s, n in enumerate(q_lens) if n > 1 for q0 in range(0, n, 64)]
    tiles128 = [(s, q0) for s, n in enumerate(q_lens) if n > 1 for q0 in range(0, n, 128)]
    dec = [s for s, n in enumerate(q_lens) if n == 1]
    ctx = StepContext(n_tokens=N, n_seqs=S, dtype=torch.float32, device=dev, token_ids=i32([0] * N), positions=i32(positions),
                      token_seq=i32(token_seq), cu_q=i32(cu), ctx_len=i32(ctx_lens), state_slot=i32(list(range(S))),
                      groups=[CacheGroupView(bt.to(dev), block_size)], q_lens=list(q_lens), ctx_lens=list(ctx_lens),
                      state_slots=list(range(S)), error_flag=torch.zeros(1, dtype=torch.int32, device=dev),
                      decode_seq_ids=i32(dec), n_decode_seqs=len(dec), q_tile_seq=i32([t[0] for t in tiles]),
                      q_tile_q0=i32([t[1] for t in tiles]), n_q_tiles=len(tiles), q_tile128_seq=i32([t[0] for t in tiles128]),
                      q_tile128_q0=i32([t[1] for t in tiles128]), n_q_tiles128=len(tiles128))
    return ctx, bt


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.parametrize("nh,nkv,hd,window,softcap", [(4, 2, 16, None, None), (3, 1, 64, None, None), (2, 2, 48, 7, None),
                                                      (4, 2, 64, None, 2.5)])
@pytest.mark.filterwarnings("ignore:a cap on the attention scores")
def test_attention_mixer_alone_over_two_steps(dtype, tol, nh, nkv, hd, window, softcap, monkeypatch):
    """The mixer part by itself: a whole prompt in step one, then a portion and a decoded token of two requests in
    step two, against the plain attention block on whole sequences.  One case caps the scores (a constant of the
    part that Llama leaves unset): the plain block then caps them too."""
    from lmsf_b200.parts.attention import PagedAttention
    if softcap:
        def capped(q, k, v, scale, window=None):
            T, n_heads, _ = q.shape
            rep = n_heads // k.shape[1]
            out = torch.empty_like(q)
            dead = torch.arange(T)[None, :] > torch.arange(T)[:, None]
            for h in range(n_heads):
                sc = (q[:, h, :] @ k[:, h // rep, :].T) * scale
                sc = (softcap * torch.tanh(sc / softcap)).masked_fill(dead, float("-inf"))
                out[:, h, :] = torch.softmax(sc, dim=-1) @ v[:, h // rep, :]
            return out
        monkeypatch.setattr(P, "causal_attention", capped)
    from lmsf_b200.parts.base import LayerCache
    from lmsf_b200.parts.rope import RotaryEmbedding
    H, bs = 40, 8
    g = torch.Generator().manual_seed(5)
    rope = RotaryEmbedding(rot_dim=hd, theta=1000.0)
    att = PagedAttention(hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd, position_encoding=rope, window=window,
                         softcap=softcap)
    wq, wk, wv = (torch.randn(nh * hd, H, generator=g) * 0.3, torch.randn(nkv * hd, H, generator=g) * 0.3,
                  torch.randn(nkv * hd, H, generator=g) * 0.3)
    wo = torch.randn(H, nh * hd, generator=g) * 0.3
    r = lambda t: t.to(dtype).float()
    att.set_weights({"qkv": torch.cat([wq, wk, wv]).to(dtype).to(DEV), "o": wo.to(dtype).to(DEV)})
    att.prepare(dtype, torch.device(DEV))
    assert att.cache_spec().window == window and att.weight_specs()["qkv"].shapes[1] == (nkv * hd, H)
    lens = [21, 13]
    hs = [torch.randn(n, H, generator=g).to(dtype) for n in lens]
    cfg = dict(hidden_size=H, num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, rope_theta=1000.0, sliding_window=window)
    w = {"q_proj.weight": r(wq), "k_proj.weight": r(wk), "v_proj.weight": r(wv), "o_proj.weight": r(wo)}
    refs = [P.attention_block(cfg, w, "", h.float(), torch.arange(n), P.rope_inv_freq(cfg)) for h, n in zip(hs, lens)]
    kv = torch.zeros(12, 2, nkv, bs, hd, dtype=dtype, device=DEV)
    cache = LayerCache(kv=kv, group=0, owner=True)
    # step one: request 0 up to token 15, request 1 up to token 12
    ctx, bt = _hand_context([15, 12], [21, 13], bs, 12)        # tables sized for the final lengths
    ctx.ctx_len.copy_(torch.tensor([15, 12], dtype=torch.int32))
    ctx.positions.copy_(torch.tensor(list(range(15)) + list(range(12)), dtype=torch.int32))
    ctx.ctx_lens[:] = [15, 12]
    out1 = att.forward(ctx, torch.cat([hs[0][:15], hs[1][:12]]).to(DEV), cache).float().cpu()
    # step two: 6 more tokens of request 0 (a portion), 1 token of request 1 (a decode), same pages
    ctx2, _ = _hand_context([6, 1], [21, 13], bs, 12)
    ctx2.groups[0].block_table.copy_(bt)
    out2 = att.forward(ctx2, torch.cat([hs[0][15:], hs[1][12:]]).to(DEV), cache).float().cpu()
    got = [torch.cat([out1[:15], out2[:6]]), torch.cat([out1[15:], out2[6:]])]
    for a, b in zip(got, refs):
        assert (a - b).abs().max() <= tol * max(1.0, b.abs().max()), (a - b).abs().max()
    assert ctx.error_flag.item() == 0 and ctx2.error_flag.item() == 0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 4e-2)])
@pytest.mark.filterwarnings("ignore:a cap on the attention scores")
def test_attention_mixer_with_a_position_encoding_on_the_scores(dtype, tol):
    """Another position encoding of the package: nothing is done to q and k, a bias slope[head] * (key - query) goes on
    the scores.  The mixer over two steps (a whole prompt; then a portion beside a decoded token) against plain
    attention with that bias on whole sequences."""
    from lmsf_b200.parts.attention import PagedAttention
    from lmsf_b200.parts.base import LayerCache, build_part, PartSpec
    H, nh, nkv, hd, bs = 40, 4, 2, 32, 8
    slopes = [0.5, 0.25, 0.125, 0.0625]
    g = torch.Generator().manual_seed(9)
    enc = build_part("position_encoding", PartSpec("distance_bias", {"slopes": slopes}))
    att = PagedAttention(hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd, position_encoding=enc)
    wq, wk, wv = (torch.randn(nh * hd, H, generator=g) * 0.3, torch.randn(nkv * hd, H, generator=g) * 0.3,
                  torch.randn(nkv * hd, H, generator=g) * 0.3)
    wo = torch.randn(H, nh * hd, generator=g) * 0.3
    r = lambda t: t.to(dtype).float()
    att.set_weights({"qkv": torch.cat([wq, wk, wv]).to(dtype).to(DEV), "o": wo.to(dtype).to(DEV)})
    att.prepare(dtype, torch.device(DEV))
    with pytest.raises(ValueError):
        bad = PagedAttention(hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                             position_encoding=build_part("position_encoding", PartSpec("distance_bias", {"slopes": slopes[:3]})))
        bad.prepare(dtype, torch.device(DEV))
    lens = [21, 13]
    hs = [torch.randn(n, H, generator=g).to(dtype) for n in lens]

    def plain(h):
        T = h.shape[0]
        q, k, v = (h @ r(wq).T).view(T, nh, hd), (h @ r(wk).T).view(T, nkv, hd), (h @ r(wv).T).view(T, nkv, hd)
        out = torch.empty(T, nh, hd)
        dist = (torch.arange(T)[None, :] - torch.arange(T)[:, None]).float()          # key - query
        for hh in range(nh):
            sc = (q[:, hh] @ k[:, hh // (nh // nkv)].T) / math.sqrt(hd) + slopes[hh] * dist
            sc = sc.masked_fill(dist > 0, float("-inf"))
            out[:, hh] = torch.softmax(sc, dim=-1) @ v[:, hh // (nh // nkv)]
        return out.reshape(T, nh * hd) @ r(wo).T

    refs = [plain(h.float()) for h in hs]
    kv = torch.zeros(12, 2, nkv, bs, hd, dtype=dtype, device=DEV)
    cache = LayerCache(kv=kv, group=0, owner=True)
    ctx, bt = _hand_context([15, 12], [21, 13], bs, 12)
    ctx.dtype = dtype
    ctx.ctx_len.copy_(torch.tensor([15, 12], dtype=torch.int32))
    ctx.positions.copy_(torch.tensor(list(range(15)) + list(range(12)), dtype=torch.int32))
    ctx.ctx_lens[:] = [15, 12]
    out1 = att.forward(ctx, torch.cat([hs[0][:15], hs[1][:12]]).to(DEV), cache).float().cpu()
    ctx2, _ = _hand_context([6, 1], [21, 13], bs, 12)
    ctx2.dtype = dtype
    ctx2.groups[0].block_table.copy_(bt)
    out2 = att.forward(ctx2, torch.cat([hs[0][15:], hs[1][12:]]).to(DEV), cache).float().cpu()
    got = [torch.cat([out1[:15], out2[:6]]), torch.cat([out1[15:], out2[6:]])]
    for a, b in zip(got, refs):
        assert (a - b).abs().max() <= tol * max(1.0, b.abs().max()), (a - b).abs().max()
    assert ctx.error_flag.item() == 0 and ctx2.error_flag.item() == 0


def test_a_decode_step_splits_its_norms_between_the_products_around_them(monkeypatch):
    """Two blocks of the package's parts on a step of five single tokens in bfloat16: the norm between the output
    projection and the gated product, and the one between the down product and the next block's q/k/v product, are
    done by those products (a `Prenormed` travels instead of a tensor) and four launches fewer run; the result is the
    one of whole norms within rounding.  A next block whose mixer does not say `takes_prenormed` (a toy, defined
    here) is handed a plain tensor."""
    from lmsf_b200 import kernels
    from lmsf_b200.parts import block as block_mod
    from lmsf_b200.parts.attention import PagedAttention
    from lmsf_b200.parts.base import LayerCache, Mixer, Prenormed
    from lmsf_b200.parts.block import PreNormBlock
    from lmsf_b200.parts.mlp import GatedMLP
    from lmsf_b200.parts.norm import RMSNorm
    from lmsf_b200.parts.rope import RotaryEmbedding
    H, nh, nkv, hd, inter, bs, n = 72, 4, 2, 16, 104, 8, 5
    g = torch.Generator().manual_seed(3)
    dt = torch.bfloat16

    def make_block(mixer=None):
        n1, n2 = RMSNorm(H, 1e-5), RMSNorm(H, 1e-6)
        n1.set_weights({"weight": (1 + 0.2 * torch.randn(H, generator=g)).to(DEV)})          # a 32-bit weight
        n2.set_weights({"weight": (1 + 0.2 * torch.randn(H, generator=g)).to(dt).to(DEV)})   # a bfloat16 one
        if mixer is None:
            mixer = PagedAttention(hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                                   position_encoding=RotaryEmbedding(rot_dim=hd, theta=1000.0))
            mixer.set_weights({"qkv": (torch.randn((nh + 2 * nkv) * hd, H, generator=g) * 0.2).to(dt).to(DEV),
                               "o": (torch.randn(H, nh * hd, generator=g) * 0.2).to(dt).to(DEV)})
            mixer.prepare(dt, torch.device(DEV))
        ff = GatedMLP(hidden_size=H, intermediate_size=inter)
        ff.set_weights({"gate_up": (torch.randn(2 * inter, H, generator=g) * 0.2).to(dt).to(DEV),
                        "down": (torch.randn(H, inter, generator=g) * 0.2).to(dt).to(DEV)})
        return PreNormBlock({"mixer_norm": n1, "mixer": mixer, "ffn_norm": n2, "feed_forward": ff})

    b1, b2 = make_block(), make_block()
    x0 = torch.randn(n, H, generator=g).to(dt).to(DEV)
    ctx_lens = [9, 3, 17, 1, 8]

    def run(split):
        monkeypatch.setattr(block_mod, "FUSE_NORMS", split)
        ctx, _ = _hand_context([1] * n, ctx_lens, bs, 16, seed=2)
        ctx.dtype = dt
        caches = [LayerCache(kv=torch.zeros(16, 2, nkv, bs, hd, dtype=dt, device=DEV), group=0, owner=True) for _ in range(2)]
        before = kernels.launch_count()
        x1, res = b1.forward(ctx, x0, None, caches[0], next_entry=b2.entry())
        launches = kernels.launch_count() - before
        # what the next block's first norm gives: from the Prenormed, or by the whole norm
        h_mid = (b2.mixer_norm.finish(x1) if isinstance(x1, Prenormed) else b2.mixer_norm.forward_residual(x1, res.clone())[0]).float()
        before = kernels.launch_count()
        x2, res2 = b2.forward(ctx, x1, res, caches[1])
        assert ctx.error_flag.item() == 0 and res2 is res
        return x1, h_mid, x2.float(), res.clone(), launches + kernels.launch_count() - before

    mid_s, h_s, x_s, res_s, launches_s = run(True)
    mid_w, h_w, x_w, res_w, launches_w = run(False)
    assert isinstance(mid_s, Prenormed) and isinstance(mid_w, torch.Tensor)
    assert launches_w - launches_s == 3              # the norms after the two output projections and after one down product
    tol = 2e-2 * res_w.abs().max().item()
    assert (res_s - res_w).abs().max().item() <= tol and (x_s - x_w).abs().max().item() <= tol
    assert (h_s - h_w).abs().max().item() <= 2e-2 * h_w.abs().max().item()     # the normed tensor that the Prenormed stands for

    # a product that cannot take a Prenormed itself has the norm finished first (`matmul_tn`)
    from lmsf_b200.parts import linear as linear_mod
    w2 = (torch.randn(24, H, generator=g) * 0.2).to(dt).to(DEV)
    monkeypatch.setattr(block_mod, "FUSE_NORMS", True)
    ctx, _ = _hand_context([1] * n, ctx_lens, bs, 16, seed=2)
    ctx.dtype = dt
    cache = LayerCache(kv=torch.zeros(16, 2, nkv, bs, hd, dtype=dt, device=DEV), group=0, owner=True)
    p, _ = b1.forward(ctx, x0, None, cache, next_entry=b2.entry())
    y_split = linear_mod.matmul_tn(p, w2, torch.float32)
    monkeypatch.setattr(linear_mod, "USE_SKINNY", False)
    y_whole = linear_mod.matmul_tn(p, w2, torch.float32)
    monkeypatch.setattr(linear_mod, "USE_SKINNY", True)
    assert (y_split - y_whole).abs().max().item() <= 2e-2 * y_whole.abs().max().item()

    class Toy(Mixer):
        def forward(self, ctx, h, cache):
            assert isinstance(h, torch.Tensor)
            return h

    b3 = make_block(Toy())
    monkeypatch.setattr(block_mod, "FUSE_NORMS", True)
    ctx, _ = _hand_context([1] * n, ctx_lens, bs, 16, seed=2)
    ctx.dtype = dt
    cache = LayerCache(kv=torch.zeros(16, 2, nkv, bs, hd, dtype=dt, device=DEV), group=0, owner=True)
    x1, res = b1.forward(ctx, x0, None, cache, next_entry=b3.entry())
    assert isinstance(x1, torch.Tensor)
    x3, _ = b3.forward(ctx, x1, res, LayerCache())
    assert isinstance(x3, torch.Tensor)


def test_embedding_rotary_apply_and_block_arrangement():
    from lmsf_b200.parts.base import FeedForward, LayerCache, Mixer, Norm, PartSpec
    from lmsf_b200.parts.block import PreNormBlock
    from lmsf_b200.parts.embedding import TokenEmbedding
    from lmsf_b200.parts.rope import RotaryEmbedding
    dev = torch.device(DEV)
    g = torch.Generator().manual_seed(2)
    # embedding
    emb = TokenEmbedding(vocab_size=37, hidden_size=24)
    table = torch.randn(37, 24, generator=g)
    emb.set_weights({"weight": table.to(dev)})
    ctx, _ = _hand_context([5], [5], 4, 4)
    ids = torch.tensor([3, 36, 0, 7, 7], dtype=torch.int32, device=dev)
    ctx.token_ids.copy_(ids)
    assert torch.equal(emb.forward(ctx).cpu(), table[ids.cpu().long()])
    scaled = TokenEmbedding(vocab_size=37, hidden_size=24, scale=24 ** 0.5)      # a constant that Llama leaves at 1
    scaled.set_weights({"weight": table.to(dev)})
    assert torch.equal(scaled.forward(ctx).cpu(), table[ids.cpu().long()] * torch.tensor(24 ** 0.5, dtype=torch.float32))
    # rotary applied on its own (the path of a mixer that cannot fuse it): partial width, interleaved pairs
    rope = RotaryEmbedding(rot_dim=8, theta=50.0, is_neox=False)
    rope.prepare(torch.float32, dev)
    q = torch.randn(5, 2 * 16, generator=g)
    qd = q.to(dev).clone()
    rope.apply(ctx, qd, None, 2, 0, 16)
    inv = torch.tensor([50.0 ** (-(2.0 * i) / 8) for i in range(4)])
    ang = torch.arange(5).float()[:, None] * inv[None, :]
    x = q.reshape(5, 2, 16)
    a, b = x[..., 0:8:2], x[..., 1:8:2]
    rot = torch.stack([a * ang.cos()[:, None] - b * ang.sin()[:, None], b * ang.cos()[:, None] + a * ang.sin()[:, None]], -1).reshape(5, 2, 8)
    assert torch.allclose(qd.cpu().reshape(5, 2, 16), torch.cat([rot, x[..., 8:]], -1), atol=1e-5)
    # the pre-norm arrangement with stand-in parts: h = n1(x + res); a = mix(h); h2 = n2(a + res'); out = ff(h2)
    calls = []

    class N(Norm):
        def __init__(self, k): self.k = k
        def forward_residual(self, x, res):
            res = x.float() if res is None else res + x.float()
            calls.append(("norm", self.k))
            return (res * self.k).to(x.dtype), res

    class M(Mixer):
        def forward(self, ctx, h, cache): calls.append("mixer"); return h + 1

    class F(FeedForward):
        def forward(self, ctx, h): calls.append("ffn"); return h * 2

    blk = PreNormBlock({"mixer_norm": N(2.0), "mixer": M(), "ffn_norm": N(3.0), "feed_forward": F()})
    x0 = torch.ones(2, 3)
    y, res = blk.forward(None, x0, None, LayerCache())
    assert calls == [("norm", 2.0), "mixer", ("norm", 3.0), "ffn"]
    assert torch.equal(res, x0 + (x0 * 2 + 1)) and torch.equal(y, (res * 3.0) * 2)
    assert PreNormBlock.ROLES == {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "feed_forward": "feed_forward"}
