"""The Niletar design on the GPU against its plain restatement (tests/plain_niletar.py): every mechanism alone, then
whole models of several shapes through the engine — prompts, token-by-token decoding (graphs included), prompts cut
into portions down to two tokens, unequal batches, slots, blocks and states that are used again, long decoding over
the edges of cache blocks and of the decode kernel's key splits, greedy generation and the trace program."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import niletar_models as nm
import plain_niletar as pn

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16}


def _weights(which, mild):
    """Sharp weights for the float32 comparisons (peaked attention rows, saturated gates), mild ones for bfloat16,
    where 16-bit rounding of large scores would itself move the softmax by several percent."""
    i = list(nm.CONFIGS).index(which)
    if mild:
        return nm.tensors(nm.CONFIGS[which], nm.RANKS[which], seed=31 + i, std=0.03, sink_std=0.5)
    return nm.tensors(nm.CONFIGS[which], nm.RANKS[which], seed=11 + i)


def K(which, dtype):
    return which + ("_mild" if dtype == "bf16" else "")


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("niletar")
    out = {}
    for which, cfg in nm.CONFIGS.items():
        out[which] = nm.write_folder(str(root / which), cfg, _weights(which, False))
        out[which + "_mild"] = nm.write_folder(str(root / (which + "_mild")), cfg, _weights(which, True))
    return out


class Oracle:
    def __init__(self, cfg, weights):
        self.cfg, self.weights, self._memo = cfg, weights, {}

    def logits(self, ids):
        key = tuple(ids)
        if key not in self._memo:
            self._memo[key] = pn.logits(self.cfg, self.weights, ids)
        return self._memo[key]


@pytest.fixture(scope="module")
def oracles():
    out = {}
    for which, cfg in nm.CONFIGS.items():
        out[which] = Oracle(cfg, _weights(which, False))
        out[which + "_mild"] = Oracle(cfg, _weights(which, True))
    return out


_models = {}


def model_of(folders, which, dtype):
    from fms_b200.models import get_model

    key = (which, dtype)
    if key not in _models:
        _models[key] = get_model("hf_pretrained", model_path=folders[K(which, dtype)], device_type="cuda", data_type=dtype)
    return _models[key]


def close(got, want, dtype, loose=1.0):
    want = want.to(torch.float64)
    got = got.detach().cpu().to(torch.float64)
    assert got.shape == want.shape and torch.isfinite(got).all()
    top = want.abs().max().item()
    if dtype == "fp32":
        torch.testing.assert_close(got, want, atol=3e-5 * loose * max(1.0, top), rtol=1e-4 * loose)
    else:
        torch.testing.assert_close(got, want, atol=0.03 * loose * top, rtol=0.03 * loose)


def part_with(part, tensors, dtype):
    for q, owner, local, decl in part.named_decls():
        owner.set_tensor(local, tensors[q].to(device="cuda", dtype=dtype).contiguous())
    part.finalize(torch.device("cuda"), dtype)
    return part


def step_through(mixer, x, cuts, dtype, lanes=1):
    """Runs x [n, dim] through a mixer as ``lanes`` equal sequences side by side, each cut into steps of the given sizes;
    returns the first sequence's rows (the others must equal them)."""
    from fms_b200.cache import Cache
    from fms_b200.engine.batch import Batch

    cache = Cache([mixer.cache_request()], max_tokens=1024 * lanes, max_positions=1024, dtype=dtype, device="cuda")
    slots = cache.begin(lanes)
    out, at = [], 0
    for n in cuts:
        before = cache.prepare(slots, [n] * lanes)
        batch = Batch.from_lists(slots, before, [[0] * n] * lanes, [[]] * lanes, "cuda")
        piece = x[at:at + n].contiguous()
        y = mixer.forward(piece.repeat(lanes, 1) if lanes > 1 else piece, batch, cache.layer_view(0), True)
        if hasattr(y, "parts"):
            y = sum(f * t.float() for t, f in y.parts).to(y.parts[0][0].dtype)
        for lane in range(1, lanes):
            assert torch.equal(y[:n], y[lane * n:(lane + 1) * n])
        out.append(y[:n])
        cache.commit(slots, [n] * lanes)
        at += n
    assert at == x.shape[0]
    return torch.cat(out)


# ---- mechanisms alone ---------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("dim", [36, 256, 1000, 5000])
def test_norm_after_the_sum(dtype, dim):
    from fms_b200.kernels import ops

    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(dim)
    res = torch.randn(7, dim, generator=g) * 3
    a, b = ((torch.randn(7, dim, generator=g) * 5).to(dt) for _ in range(2))
    gain = 1 + 0.5 * torch.randn(dim, generator=g)
    for alpha, parts in ((3.0, [(a, 1.0)]), (1.0, [(a, 0.6), (b, 0.5)]), (0.25, [(a, -2.0), (b, 1.0)])):
        x = alpha * res.double() + sum(f * t.double() for t, f in parts)
        want = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * gain.double()
        r = res.clone().cuda()
        copy = ops.scaled_add_rmsnorm(r, alpha, [(t.cuda(), f) for t, f in parts], gain.cuda(), 1e-5, dt)
        close(r, want, "fp32")
        if dtype == "fp32":
            assert copy is None
        else:
            assert torch.equal(copy.cpu(), r.cpu().to(dt))


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_causal_convolution_with_tails(dtype, taps):
    """Several sequences with unequal portions in one step, portions shorter than the taps, a bias or none, the
    convolved channels a run of columns in the middle of wider rows."""
    from fms_b200.cache import Cache
    from fms_b200.cache.requests import StateRequest
    from fms_b200.engine.batch import Batch
    from fms_b200.kernels import ops

    dt, channels, before, after = DTYPES[dtype], 37, 5, 3
    g = torch.Generator().manual_seed(taps)
    lengths = (23, 1, 9)
    xs = [torch.randn(n, before + channels + after, generator=g).to(dt) for n in lengths]
    w, bias = torch.randn(channels, taps, generator=g), torch.randn(channels, generator=g)
    for use_bias in (True, False):
        want = [pn.silu(pn.causal_conv(x[:, before:before + channels].double(), w.double(), bias.double() if use_bias else None))
                for x in xs]
        cache = Cache([StateRequest((taps - 1, channels), torch.float32, "tail")], 256, 256, dt, "cuda")
        slots = cache.begin(3)
        got = [[] for _ in lengths]
        for cuts in ((1, 1, 2), (1, 0, 1), (2, 0, 3), (5, 0, 3), (14, 0, 0)):
            live = [i for i, c in enumerate(cuts) if c]
            at = [sum(len(p) for p in got[i]) for i in live]
            lens = cache.prepare([slots[i] for i in live], [cuts[i] for i in live])
            batch = Batch.from_lists([slots[i] for i in live], lens, [[0] * cuts[i] for i in live], [[] for _ in live], "cuda")
            x = torch.cat([xs[i][a:a + cuts[i]] for i, a in zip(live, at)]).cuda()
            y = ops.causal_conv(x, before, channels, w.cuda(), bias.cuda() if use_bias else None,
                                cache.layer_view(0).state, batch)
            for i, piece in zip(live, torch.split(y, [cuts[i] for i in live])):
                got[i].append(piece)
            cache.commit([slots[i] for i in live], [cuts[i] for i in live])
        for i in range(3):
            close(torch.cat(got[i]), want[i], "fp32", loose=1 if dtype == "fp32" else 3)


def attention_tensors(g, dim_in, m, std=0.3):
    h, kv, k, v = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    mk = lambda *s, sd=std: (torch.randn(*s, generator=g) * sd).to(torch.bfloat16)
    return {"q": mk(h * k, dim_in), "q.b": mk(h * k), "k": mk(kv * k, dim_in), "k.b": mk(kv * k), "v": mk(kv * v, dim_in),
            "v.b": mk(kv * v), "sink": mk(h, sd=1.0), "g": mk(h * v, dim_in), "o": mk(dim_in, h * v)}


def attention_mixer(m, dim_in, w, eps, dt):
    from fms_b200.config import MixerSpec, PositionSpec
    from fms_b200.parts import build_mixer

    rot = m["rot"]
    sc = rot.get("scaling")
    position = PositionSpec("rope", head_dim=rot["dims"], theta=rot["base"], scaling=() if sc is None else (
        ("rope_type", "llama3"), ("factor", sc["factor"]), ("low_freq_factor", sc["low"]), ("high_freq_factor", sc["high"]),
        ("original_max_position_embeddings", sc["original"]))) if rot["dims"] else PositionSpec("none")
    spec = MixerSpec("sink_attention", dim=dim_in, nheads=m["heads"], kvheads=m["kv_heads"], head_dim=m["dim"], bias=True,
                     scale=m["scale"], position=position,
                     options=(("vdim", m["vdim"]), ("rot_dims", rot["dims"]), ("qk_norm", True), ("eps", eps), ("sink", True),
                              ("gate", True)))
    zeros = torch.zeros(m["heads"] * m["vdim"], dtype=torch.bfloat16)
    return part_with(build_mixer(spec), {
        "in_proj.weight": torch.cat([w["q"], w["k"], w["v"], w["g"]]), "in_proj.bias": torch.cat([w["q.b"], w["k.b"], w["v.b"], zeros]),
        "sink": w["sink"], "dense.weight": w["o"]}, dt)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("shape", [(4, 2, 16, 16, 8, None), (6, 1, 24, 8, 24, 1), (2, 2, 10, 40, 0, None), (3, 3, 64, 64, 32, 1),
                                   (8, 2, 128, 64, 64, None), (5, 5, 6, 10, 2, None), (9, 3, 48, 33, 48, 1), (2, 1, 200, 256, 100, None)])
def test_sink_attention_alone(dtype, shape):
    heads, kv, dim, vdim, rot, scaled = shape
    m = nm.left(heads, kv, dim, vdim, rot, 300.0, 0.7 * dim ** -0.5 * (1 if dtype == "bf16" else 3),
                {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 96} if scaled else None)
    dt, dim_in, n = DTYPES[dtype], 40, 331
    g = torch.Generator().manual_seed(sum(x or 0 for x in shape))
    w = attention_tensors(g, dim_in, m)
    mixer = attention_mixer(m, dim_in, w, 1e-5, dt)
    x = torch.randn(n, dim_in, generator=g).to(dt)
    want = pn.sink_attention(x.double(), m, 1e-5, {k: v.double() for k, v in w.items()}, "")
    # whole; portions whose edges fall on and beside the cache's blocks of 64; the last rows one by one (the decode
    # kernels, over the edge of their first split of 256 keys)
    for cuts in ([n], [63, 1, 1, 63, 2, 128, 73], [250] + [1] * 81):
        close(step_through(mixer, x.cuda(), cuts, dt), want, dtype)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_sinks_that_take_all_or_nothing_and_keys_far_back(dtype):
    """Weights and inputs made so that a fault shows.  Head 0's sink is so large that it takes all of the softmax, head
    1's so small that it takes nothing.  Queries read the first half of the input and keys the second half through the
    same matrix, without biases, and every seventh row's first half is the second half of ONE row far back (hundreds of
    positions: another cache block and, when decoding, another split), so that this key's score stands out among
    hundreds."""
    m = nm.left(2, 1, 64, 16, 8, 50.0, 0.5)
    dt = DTYPES[dtype]
    g = torch.Generator().manual_seed(77)
    dim_in, n = 32, 600
    w = attention_tensors(g, dim_in, m)
    w["sink"] = torch.tensor([200.0, -200.0]).to(torch.bfloat16)
    for b in ("q.b", "k.b"):
        w[b] = torch.zeros_like(w[b])
    a = w["k"][:, :16].clone()
    w["k"] = torch.cat([torch.zeros_like(a), a], 1)
    w["q"] = torch.cat([torch.cat([a, torch.zeros_like(a)], 1)] * 2)
    x = torch.randn(n, dim_in, generator=g)
    for t in range(300, n, 7):
        x[t, :16] = x[t - 290 + (t % 50), 16:]
    x = x.to(dt)
    d = {k: v.double() for k, v in w.items()}
    want = pn.sink_attention(x.double(), m, 1e-5, d, "")
    # the oracle itself says that the far keys matter: without the first 200 keys the result is another
    near = pn.sink_attention(x.double()[200:], m, 1e-5, d, "", first_position=200)
    assert (want[300:] - near[100:]).abs().max() > 0.5 * want.abs().max()
    mixer = attention_mixer(m, dim_in, w, 1e-5, dt)
    for cuts in ([n], [520] + [1] * 80, [2] * 300):
        close(step_through(mixer, x.cuda(), cuts, dt), want, dtype)
    # head 0 alone (its sink takes everything): the mixer's output without head 1 is the zero vector
    w0 = dict(w)
    w0["o"] = w["o"].clone()
    w0["o"][:, 16:] = 0
    for cuts in ([n], [590] + [1] * 10):
        assert step_through(attention_mixer(m, dim_in, w0, 1e-5, dt), x.cuda(), cuts, dt).float().abs().max() < 1e-6


def delta_tensors(g, dim_in, m, ranks, std=0.3):
    h, kv, k, v, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    mk = lambda *s, sd=std: (torch.randn(*s, generator=g) * sd).to(torch.bfloat16)
    out = {"b": mk(h, dim_in), "A_log": mk(h, sd=1.0) - 1, "norm": 1 + mk(v), "a1": mk(ranks[0], dim_in), "a2": mk(h * k, ranks[0], sd=0.5),
           "dt_bias": mk(h * k, sd=1.0), "g1": mk(ranks[1], dim_in), "g2": mk(h * v, ranks[1], sd=0.5), "o": mk(dim_in, h * v)}
    for n, rows in (("q", kv * k), ("k", kv * k), ("v", h * v)):
        out[n], out[n + ".conv"] = mk(rows, dim_in), mk(rows, taps, sd=0.6)
    return out


def delta_mixer(m, dim_in, w, ranks, eps, dt):
    from fms_b200.config import MixerSpec
    from fms_b200.parts import build_mixer

    spec = MixerSpec("gated_delta_rule", dim=dim_in, nheads=m["heads"], kvheads=m["kv_heads"], head_dim=m["dim"],
                     options=(("vdim", m["vdim"]), ("conv", m["conv"]), ("eps", eps), ("decay_rank", ranks[0]),
                              ("gate_rank", ranks[1])))
    return part_with(build_mixer(spec), {
        "in_proj.weight": torch.cat([w["q"], w["k"], w["v"], w["b"]]), "conv": torch.cat([w["q.conv"], w["k.conv"], w["v.conv"]]),
        "decay_in.weight": w["a1"], "decay_out.weight": w["a2"], "gate_in.weight": w["g1"], "gate_out.weight": w["g2"],
        "dt_bias": w["dt_bias"], "A_log": w["A_log"], "norm": w["norm"], "dense.weight": w["o"]}, dt)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("shape", [(2, 2, 32, 32, 4, 8, 8), (4, 1, 12, 20, 2, 5, 3), (3, 3, 5, 3, 1, 3, 7), (2, 1, 96, 40, 4, 16, 8),
                                   (1, 1, 256, 33, 3, 8, 8), (6, 2, 64, 128, 4, 24, 24)])
def test_gated_delta_rule_alone(dtype, shape):
    heads, kv, dim, vdim, taps, ra, rg = shape
    m = nm.right(heads, kv, dim, vdim, taps)
    dt, dim_in, n = DTYPES[dtype], 40, 150
    g = torch.Generator().manual_seed(sum(shape))
    w = delta_tensors(g, dim_in, m, (ra, rg))
    mixer = delta_mixer(m, dim_in, w, (ra, rg), 1e-5, dt)
    x = torch.randn(n, dim_in, generator=g).to(dt)
    want = pn.gated_delta_rule(x.double(), m, 1e-5, {k: v.double() for k, v in w.items()}, "")
    for cuts, lanes in (([n], 1), ([15, 1, 1, 17, 2, 16, 98], 3), ([100] + [1] * 50, 2), ([2] * 75, 1)):
        close(step_through(mixer, x.cuda(), cuts, dt, lanes), want, dtype, loose=2)


def ssm_tensors(g, dim_in, m, std=0.3):
    h, v, n, gr, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner, ch = h * v, h * v + 2 * gr * n
    mk = lambda *s, sd=std: (torch.randn(*s, generator=g) * sd).to(torch.bfloat16)
    return {"in": mk(inner + ch + h, dim_in), "conv": mk(ch, taps, sd=0.6), "conv.b": mk(ch), "dt_bias": mk(h, sd=1.0),
            "A_log": mk(h, sd=1.0) - 0.5, "D": 1 + mk(h), "norm": 1 + mk(inner), "o": mk(dim_in, inner)}


def ssm_mixer(m, dim_in, w, eps, dt):
    from fms_b200.config import MixerSpec
    from fms_b200.parts import build_mixer

    spec = MixerSpec("selective_state_space", dim=dim_in, nheads=m["heads"],
                     options=(("vdim", m["vdim"]), ("state", m["state"]), ("groups", m["groups"]), ("conv", m["conv"]),
                              ("norm_groups", m["norm_groups"]), ("eps", eps)))
    return part_with(build_mixer(spec), {"in_proj.weight": w["in"], "conv": w["conv"], "conv_bias": w["conv.b"],
                                         "dt_bias": w["dt_bias"], "A_log": w["A_log"], "D": w["D"], "norm": w["norm"],
                                         "dense.weight": w["o"]}, dt)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("shape", [(4, 32, 48, 2, 2, 4), (3, 8, 5, 1, 3, 3), (4, 16, 33, 4, 1, 5), (5, 6, 7, 1, 5, 2), (2, 48, 128, 2, 2, 4),
                                   (2, 70, 256, 1, 1, 4), (6, 4, 16, 3, 6, 1)])
def test_selective_state_space_alone(dtype, shape):
    heads, vdim, state, groups, norm_groups, taps = shape
    m = nm.mamba2(heads, vdim, state, groups, norm_groups, taps, None)["mixer"]
    dt, dim_in, n = DTYPES[dtype], 40, 150
    g = torch.Generator().manual_seed(sum(shape))
    w = ssm_tensors(g, dim_in, m)
    mixer = ssm_mixer(m, dim_in, w, 1e-5, dt)
    x = torch.randn(n, dim_in, generator=g).to(dt)
    want = pn.mamba2(x.double(), m, 1e-5, {k: v.double() for k, v in w.items()}, "")
    for cuts, lanes in (([n], 1), ([15, 1, 1, 17, 2, 16, 98], 3), ([100] + [1] * 50, 2), ([2] * 75, 1)):
        close(step_through(mixer, x.cuda(), cuts, dt, lanes), want, dtype, loose=2)


def test_state_that_decays_slowly_keeps_the_first_tokens():
    """A scan whose decay is close to 1 (A_log very negative) and whose later inputs are nearly switched off (a very
    negative step-size bias after the first rows cannot be had, so the FIRST token's row is made large): the output
    hundreds of tokens later still carries the first token; a state that was lost or reset on the way shows."""
    m = nm.mamba2(2, 8, 16, 1, 1, 2, None)["mixer"]
    g = torch.Generator().manual_seed(5)
    w = ssm_tensors(g, 24, m)
    w["A_log"] = torch.full_like(w["A_log"], -9.0)
    x = torch.randn(400, 24, generator=g) * 0.2
    x[0] *= 40
    d = {k: v.double() for k, v in w.items()}
    want = pn.mamba2(x.double(), m, 1e-5, d, "")
    lost = pn.mamba2(x.double()[1:], m, 1e-5, d, "")
    assert (want[300:] - lost[299:]).abs().max() > 0.05 * want.abs().max()
    mixer = ssm_mixer(m, 24, w, 1e-5, torch.float32)
    for cuts in ([400], [1] + [3] * 133, [330] + [1] * 70):
        close(step_through(mixer, x.cuda(), cuts, torch.float32), want, "fp32", loose=2)


# ---- whole models -------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("which", ["p", "q", "r", "s"])
def test_whole_prompts_alone(folders, oracles, which, dtype):
    model = model_of(folders, which, dtype)
    engine = model.new_engine(max_tokens=1024, sampling=False)
    for i, n in enumerate((1, 2, 63, 64, 65, 300)):
        ids = nm.prompt(nm.CONFIGS[which], n, i)
        (slot,) = engine.begin(1)
        got = engine.step([slot], [ids], [list(range(n))])
        engine.release([slot])
        close(got, oracles[K(which, dtype)].logits(ids), dtype)
    engine.check()
    assert engine.cache.slots.n_held == 0 and all(g.pool.n_held == 0 for g in engine.cache.groups if hasattr(g, "pool"))


@pytest.mark.parametrize("which,dtype", [("p", "fp32"), ("q", "fp32"), ("r", "bf16"), ("s", "fp32")])
def test_token_by_token_from_the_first_token(folders, oracles, which, dtype):
    """Decode steps from a sequence's very first token (the first plain, the second captured, the rest replayed), over
    the edge of a cache block, twice in the same slot."""
    engine = model_of(folders, which, dtype).new_engine(max_tokens=256, sampling=False)
    for rep in range(2):
        ids = nm.prompt(nm.CONFIGS[which], 70, 20 + rep)
        (slot,) = engine.begin(1)
        got = torch.cat([engine.step([slot], [[t]], [[0]]) for t in ids])
        engine.release([slot])
        close(got, oracles[K(which, dtype)].logits(ids), dtype)
    assert engine.graphs_captured >= 1
    engine.check()


@pytest.mark.parametrize("which,dtype", [("p", "fp32"), ("q", "bf16"), ("r", "fp32"), ("s", "bf16")])
def test_prompt_then_long_decoding_over_split_edges(folders, oracles, which, dtype):
    """A prompt of 250 tokens, then 290 tokens one by one: the decode kernel goes from one split of 256 keys to two and
    to three, the cache from its fourth block to its ninth."""
    engine = model_of(folders, which, dtype).new_engine(max_tokens=1024, sampling=False)
    ids = nm.prompt(nm.CONFIGS[which], 540, 31)
    (slot,) = engine.begin(1)
    got = [engine.step([slot], [ids[:250]], [list(range(250))])]
    got += [engine.step([slot], [[t]], [[0]]) for t in ids[250:]]
    engine.release([slot])
    close(torch.cat(got), oracles[K(which, dtype)].logits(ids), dtype)
    engine.check()


@pytest.mark.parametrize("which,dtype", [("p", "fp32"), ("q", "fp32"), ("r", "fp32"), ("s", "fp32"), ("p", "bf16"), ("s", "bf16")])
def test_prompts_cut_into_portions(folders, oracles, which, dtype):
    engine = model_of(folders, which, dtype).new_engine(max_tokens=1024, sampling=False)
    ids = nm.prompt(nm.CONFIGS[which], 420, 41)
    want = oracles[K(which, dtype)].logits(ids)
    for cuts in ([2, 3, 59, 1, 64, 65, 6, 220], [193, 2, 225], [1, 1, 2, 416], [2] * 40 + [340]):
        (slot,) = engine.begin(1)
        got, at = [], 0
        for n in cuts:
            got.append(engine.step([slot], [ids[at:at + n]], [list(range(n))]))
            at += n
        engine.release([slot])
        close(torch.cat(got), want, dtype)
    engine.check()


@pytest.mark.parametrize("which,dtype", [("p", "fp32"), ("q", "fp32"), ("r", "fp32"), ("s", "fp32"), ("q", "bf16"), ("s", "bf16")])
def test_unequal_batches_freed_slots_and_poisoned_blocks(folders, oracles, which, dtype):
    """Requests of unequal lengths start together and go on one token at a time while the shorter ones end; then
    everything the cache holds is filled with NaN (keys, values, state matrices, the convolutions' tails) and new
    requests take the freed slots and blocks.  Every request against the oracle, alone."""
    cfg = nm.CONFIGS[which]
    engine = model_of(folders, which, dtype).new_engine(max_tokens=64 * 12, max_slots=5, sampling=False)
    for round_ in range(2):
        lengths, extra = ((1, 70, 5, 131, 64), (3, 9, 0, 12, 12)) if round_ == 0 else ((210, 2, 33), (5, 5, 1))
        full = [nm.prompt(cfg, n + e, 50 + 10 * round_ + i) for i, (n, e) in enumerate(zip(lengths, extra))]
        slots = engine.begin(len(lengths))
        got = [[] for _ in lengths]
        first = engine.step(slots, [f[:n] for f, n in zip(full, lengths)], [list(range(n)) for n in lengths])
        for i, piece in enumerate(torch.split(first, list(lengths))):
            got[i].append(piece)
        for t in range(max(extra)):
            live = [i for i in range(len(lengths)) if t < extra[i]]
            out = engine.step([slots[i] for i in live], [[full[i][lengths[i] + t]] for i in live])
            for i, row in zip(live, out):
                got[i].append(row[None])
            done = [i for i in live if t + 1 == extra[i]]
            engine.release([slots[i] for i in done])
        engine.release([slots[i] for i in range(len(lengths)) if extra[i] == 0])
        for i, f in enumerate(full):
            close(torch.cat(got[i]), oracles[K(which, dtype)].logits(f), dtype)
        assert engine.cache.slots.n_held == 0
        for g in engine.cache.groups:
            g.storage.fill_(float("nan") if g.storage.is_floating_point() else 12345)
    engine.check()


def test_many_sequences_in_one_decode_step_fill_rows_and_graphs(folders, oracles):
    """Eleven sequences decode together (filled up to twelve rows with rows in the spare slot), then nine of them."""
    which, cfg, dtype = "p", nm.CONFIGS["p"], "fp32"
    engine = model_of(folders, which, "fp32").new_engine(max_tokens=64 * 24, sampling=False)
    full = [nm.prompt(cfg, 3 + 5 * i + 6, 70 + i) for i in range(11)]
    slots = engine.begin(11)
    engine.step(slots, [f[:-6] for f in full], [[] for _ in full])
    got = [[] for _ in full]
    for t in range(6):
        live = list(range(11)) if t < 3 else list(range(2, 11))
        out = engine.step([slots[i] for i in live], [[full[i][len(full[i]) - 6 + t]] for i in live])
        for i, row in zip(live, out):
            got[i].append(row[None])
    engine.release(slots)
    for i, f in enumerate(full):
        want = oracles[K(which, dtype)].logits(f)
        close(torch.cat(got[i]), want[len(f) - 6: len(f) - 6 + len(got[i])], "fp32")
    engine.check()


def test_greedy_generation_through_generate(folders, oracles):
    from fms_b200.utils.generation import generate

    which, cfg, dtype = "q", nm.CONFIGS["q"], "fp32"
    model = model_of(folders, which, "fp32")
    prompts = [nm.prompt(cfg, n, 80 + i) for i, n in enumerate((5, 1, 40))]
    out = generate(model, [torch.tensor(p) for p in prompts], max_new_tokens=10, do_sample=False)
    for p, o in zip(prompts, out):
        o = o.tolist()
        assert o[: len(p)] == p and len(o) == len(p) + 10
        for k in range(len(p), len(o)):  # every new token is the oracle's choice given what came before
            row = oracles[K(which, dtype)].logits(o[:k])[-1]
            best = row.topk(2).values
            if best[0] - best[1] > 1e-3:
                assert o[k] == int(row.argmax())


def test_trace_program_replays_a_batch(folders, oracles, tmp_path):
    which, cfg, dtype = "r", nm.CONFIGS["r"], "fp32"
    a, b = nm.prompt(cfg, 70, 90), nm.prompt(cfg, 9, 91)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []}]
    for t in range(4):
        steps.append({"step": t + 1, "entries": [{"id": "a", "tokens": [a[66 + t]], "want": [0]},
                                                  {"id": "b", "tokens": [b[5 + t]], "want": [0] if t % 2 else []}],
                      "end": ["a", "b"] if t == 3 else []})
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders[which], "--dtype",
                           "float32", "--out", str(tmp_path), "--max-tokens", "256"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(5)]
    wa, wb = oracles[K(which, dtype)].logits(a), oracles[K(which, dtype)].logits(b)
    read = lambda i: torch.from_numpy(np.fromfile(os.path.join(str(tmp_path), f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"]))
    close(read(0), torch.stack([wa[0], wa[65], wb[4]]), "fp32")
    for t in range(4):
        want = [wa[66 + t]] + ([wb[5 + t]] if t % 2 else [])
        close(read(t + 1), torch.stack(want), "fp32")


def test_trace_program_with_many_short_requests_and_no_room_to_spare(folders, oracles, tmp_path):
    """Six requests of three tokens in one batch with --max-tokens 18, the tokens they hold and not one more: the
    cache's blocks of 64 tokens must not make the program run out of room."""
    which, cfg = "q", nm.CONFIGS["q"]
    reqs = [nm.prompt(cfg, 3, 120 + i) for i in range(6)]
    steps = [{"step": 0, "entries": [{"id": str(i), "tokens": r[:2], "want": [1]} for i, r in enumerate(reqs)], "end": []},
             {"step": 1, "entries": [{"id": str(i), "tokens": r[2:], "want": [0]} for i, r in enumerate(reqs)],
              "end": [str(i) for i in range(6)]}]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders[which], "--dtype",
                           "float32", "--out", str(tmp_path), "--max-tokens", "18"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    read = lambda i: torch.from_numpy(np.fromfile(os.path.join(str(tmp_path), f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"]))
    close(read(0), torch.stack([oracles[which].logits(r)[1] for r in reqs]), "fp32")
    close(read(1), torch.stack([oracles[which].logits(r)[2] for r in reqs]), "fp32")


def test_command_line_and_sampling(folders, oracles):
    """The framework's command line finds the design through config.json: greedy tokens equal the oracle's choices; with
    sampling (temperature, top-k) every token is among the oracle's k best given what came before."""
    from fms_b200.utils.generation import generate

    which, cfg = "p", nm.CONFIGS["p"]
    prompts = [nm.prompt(cfg, n, 95 + i) for i, n in enumerate((4, 9))]
    args = [sys.executable, os.path.join(ROOT, "bin", "fms_inference"), "--architecture", "hf_pretrained", "--model_path", folders[which],
            "--default_dtype", "fp32",
            "--batch_input", "--max_new_tokens", "6", "--deterministic"]
    for p in prompts:
        args += ["--prompt_ids", ",".join(str(t) for t in p)]
    proc = subprocess.run(args, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [[int(x) for x in l.split(",")] for l in proc.stdout.splitlines() if l.strip()]
    assert len(lines) == 2
    for p, o in zip(prompts, lines):
        assert o[: len(p)] == p and len(o) == len(p) + 6
        for k in range(len(p), len(o)):
            row = oracles[which].logits(o[:k])[-1]
            best = row.topk(2).values
            if best[0] - best[1] > 1e-3:
                assert o[k] == int(row.argmax())
    out = generate(model_of(folders, which, "fp32"), [torch.tensor(p) for p in prompts], max_new_tokens=8, do_sample=True,
                   temperature=0.8, top_k=3, seed=5)
    for p, o in zip(prompts, out):
        o = o.tolist()
        for k in range(len(p), len(o)):
            row = oracles[which].logits(o[:k])[-1]
            kth = row.topk(4).values
            assert row[o[k]] >= kth[2] - 1e-4 or kth[2] - kth[3] < 1e-3
