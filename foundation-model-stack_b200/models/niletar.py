"""Niletar: a decoder whose layers put the norm after the residual sum, x = norm(alpha x + sublayer(x)), and mix tokens
either with a selective state-space scan ("mamba2") or with two mixers side by side ("parallel": softmax attention with
rotated, normed queries and keys, a sink and an output gate, beside a gated delta rule), each followed by a dense gated
feed-forward (or none).  A layer may run with the weights of an earlier layer and a state of its own.

This file is all that is specific to the architecture: its ``config.json`` (every size and constant is read from it:
``vocab``, ``width``, ``norm.eps``, ``postln_alpha``, and ``layers``, each entry with its ``type``, the sizes of its
``mixer``, its ``mlp`` or null, and ``weights_of`` where it has no tensors of its own), the ``DecoderSpec`` that
configuration means, and the checkpoint's tensor names and layouts:

    embed [vocab, width]    final.norm [width]    head [vocab, width]
    l<i>.norm1, l<i>.norm2 [width]                                 (stored around zero: the gain is 1 + w)
    mamba2:    l<i>.mix.in [2 inner + 2 groups state + heads, width], .conv [channels, taps], .conv.b, .dt_bias, .A_log,
               .D [heads], .norm [inner], .o [width, inner]
    parallel:  l<i>.mix.left.q, .q.b, .k, .k.b, .v, .v.b, .sink [heads], .g, .o
               l<i>.mix.right.q, .q.conv, .k, .k.conv, .v, .v.conv, .b, .A_log [heads], .norm [vdim], .a1, .a2, .dt_bias,
               .g1, .g2, .o
    dense:     l<i>.mlp.gate, .up [ff, width], .down [width, ff]

Linear weights are stored [out, in].  The ranks of the two low-rank pairs (a1/a2, g1/g2) are not in config.json: they
are read from the shapes of a1 and g1.  The adapter fuses [q; k; v; g] (bias [q.b; k.b; v.b; 0]), [q; k; v; b] with
the three convolutions' taps, and [gate; up] into one matrix each.
"""
from __future__ import annotations

import copy
import dataclasses
import re
from typing import Any, Dict, List, Optional

import torch

from ..config.model_config import ModelConfig
from ..config.specs import BlockSpec, DecoderSpec, FeedForwardSpec, LayerCall, MixerSpec, NormSpec, PositionSpec
from ..weights.adapters import register_adapter, register_adapter_step
from ..weights.sources import TensorLayout
from . import register_architecture, register_model
from .base import Model

LAYER_TYPES = ("mamba2", "parallel")


@dataclasses.dataclass
class NiletarConfig(ModelConfig):
    vocab: int = 512
    width: int = 256
    norm_eps: float = 1e-6
    postln_alpha: float = 1.0
    layers: List[Dict[str, Any]] = dataclasses.field(default_factory=list)
    max_positions: int = 131072  # how long a sequence may get; nothing in the model depends on it

    def __post_init__(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ValueError(f"vocab {self.vocab}, width {self.width}")
        for i, layer in enumerate(self.layers):
            if layer.get("type") not in LAYER_TYPES:
                raise ValueError(f"layer {i}: type {layer.get('type')!r}; known: {', '.join(LAYER_TYPES)}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") != "dense":
                raise ValueError(f"layer {i}: feed-forward kind {mlp.get('kind')!r}; known: dense, or null for none")
            j = layer.get("weights_of")
            if j is not None and not (0 <= int(j) < i and self.layers[int(j)]["type"] == layer["type"]):
                raise ValueError(f"layer {i}: weights_of {j} names no earlier layer of its type")

    def owner_of(self, i: int) -> int:
        """The layer whose tensors layer i runs with: itself, or where its chain of ``weights_of`` ends."""
        while self.layers[i].get("weights_of") is not None:
            i = int(self.layers[i]["weights_of"])
        return i


def _config_from_json(values: Dict[str, Any]) -> NiletarConfig:
    if values.get("architecture") != "Niletar":
        raise ValueError(f"config.json is of architecture {values.get('architecture')!r}, not Niletar")
    absent = [k for k in ("vocab", "width", "layers", "norm", "postln_alpha") if k not in values]
    if absent:
        raise ValueError(f"config.json lacks {absent}")
    return NiletarConfig(vocab=int(values["vocab"]), width=int(values["width"]), norm_eps=float(values["norm"]["eps"]),
                         postln_alpha=float(values["postln_alpha"]), layers=copy.deepcopy(values["layers"]),
                         max_positions=int(values.get("max_positions", 131072)))


# ---- layer entries as config.json has them -----------------------------------------------------------
def dense_mlp(ff: int) -> dict:
    return {"kind": "dense", "ff": ff}


def mamba2_layer(heads: int, vdim: int, state: int, groups: int, norm_groups: int, conv: int, mlp: Optional[dict],
                 weights_of: Optional[int] = None) -> dict:
    out = {"type": "mamba2", "mlp": mlp,
           "mixer": {"conv": conv, "groups": groups, "heads": heads, "norm_groups": norm_groups, "state": state, "vdim": vdim}}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def parallel_layer(left: dict, right: dict, left_scale: float, right_scale: float, mlp: Optional[dict],
                   weights_of: Optional[int] = None) -> dict:
    out = {"type": "parallel", "mlp": mlp,
           "mixer": {"left": left, "left_scale": left_scale, "right": right, "right_scale": right_scale}}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def attention_side(heads: int, kv_heads: int, dim: int, vdim: int, rot_dims: int, base: float, scale: float,
                   scaling: Optional[dict] = None) -> dict:
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = dict(scaling)
    return {"dim": dim, "heads": heads, "kv_heads": kv_heads, "rot": rot, "scale": scale, "vdim": vdim}


def delta_side(heads: int, kv_heads: int, dim: int, vdim: int, conv: int, decay_rank: int, gate_rank: int) -> dict:
    return {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim, "decay_rank": decay_rank,
            "gate_rank": gate_rank}


class Niletar(Model):
    architecture = "niletar"
    default_source = "native"

    def __init__(self, config: Optional[NiletarConfig] = None, **kwargs) -> None:
        config = config if config is not None else NiletarConfig()
        super().__init__(config.updated(**kwargs))

    @classmethod
    def config_from_json(cls, values: dict) -> NiletarConfig:
        return _config_from_json(values)

    def config_json(self) -> dict:
        c = self.config
        return {"architecture": "Niletar", "vocab": c.vocab, "width": c.width, "norm": {"eps": c.norm_eps},
                "postln_alpha": c.postln_alpha, "layers": copy.deepcopy(c.layers)}

    def load(self, source, adapter_source, device, dtype):
        # the ranks of the low-rank pairs stand in no config.json: the checkpoint's shapes give them
        names = set(source.keys())
        for i, layer in enumerate(self.config.layers):
            if layer["type"] == "parallel" and layer.get("weights_of") is None:
                right = layer["mixer"]["right"]
                for key, tensor in (("decay_rank", f"l{i}.mix.right.a1"), ("gate_rank", f"l{i}.mix.right.g1")):
                    if key not in right and tensor in names:
                        right[key] = int(source.spec(tensor)[1][0])
        return super().load(source, adapter_source, device, dtype)

    # ---- specs -------------------------------------------------------------------------------
    def _mixer_spec(self, layer: dict) -> MixerSpec:
        c, m = self.config, layer["mixer"]
        eps = float(c.norm_eps)
        if layer["type"] == "mamba2":
            return MixerSpec("selective_state_space", dim=c.width, nheads=int(m["heads"]),
                             options=(("vdim", int(m["vdim"])), ("state", int(m["state"])), ("groups", int(m["groups"])),
                                      ("conv", int(m["conv"])), ("norm_groups", int(m["norm_groups"])), ("eps", eps)))
        left, right = m["left"], m["right"]
        rot = left.get("rot") or {}
        scaling = rot.get("scaling")
        position = PositionSpec("none")
        if int(rot.get("dims", 0)):
            position = PositionSpec(
                "rope", head_dim=int(rot["dims"]), theta=float(rot["base"]),
                scaling=() if not scaling else (("rope_type", "llama3"), ("factor", float(scaling["factor"])),
                                                ("low_freq_factor", float(scaling["low"])),
                                                ("high_freq_factor", float(scaling["high"])),
                                                ("original_max_position_embeddings", float(scaling["original"]))))
        left_spec = MixerSpec("sink_attention", dim=c.width, nheads=int(left["heads"]), kvheads=int(left["kv_heads"]),
                              head_dim=int(left["dim"]), bias=True,
                              scale=float(left["scale"]) if left.get("scale") is not None else None, position=position,
                              options=(("vdim", int(left["vdim"])), ("rot_dims", int(rot.get("dims", 0))), ("qk_norm", True),
                                       ("eps", eps), ("sink", True), ("gate", True)))
        right_spec = MixerSpec("gated_delta_rule", dim=c.width, nheads=int(right["heads"]), kvheads=int(right["kv_heads"]),
                               head_dim=int(right["dim"]),
                               options=(("vdim", int(right["vdim"])), ("conv", int(right["conv"])), ("eps", eps),
                                        ("decay_rank", int(right.get("decay_rank", 0))),
                                        ("gate_rank", int(right.get("gate_rank", 0)))))
        return MixerSpec("parallel", dim=c.width,
                         options=(("left", left_spec), ("right", right_spec), ("left_factor", float(m["left_scale"])),
                                  ("right_factor", float(m["right_scale"]))))

    def decoder_spec(self) -> DecoderSpec:
        c = self.config
        norm = NormSpec("rmsnorm", c.width, float(c.norm_eps), options=(("offset", 1.0),))
        blocks = []
        for layer in c.layers:
            ff = None
            if layer.get("mlp") is not None:
                ff = FeedForwardSpec("glu", dim=c.width, hidden=int(layer["mlp"]["ff"]), activation="silu")
            j = None if layer.get("weights_of") is None else c.owner_of(len(blocks))
            blocks.append(BlockSpec(mixer=self._mixer_spec(layer), feed_forward=ff, mixer_norm=norm,
                                    feed_forward_norm=norm if ff is not None else None, arrangement="post_norm",
                                    names=("norm1", "mix", "norm2", "mlp"), options=(("alpha", float(c.postln_alpha)),),
                                    weights_of=None if j is None else int(j)))
        return DecoderSpec(vocab_size=c.vocab, dim=c.width, layers=tuple(blocks),
                           schedule=tuple(LayerCall(i) for i in range(len(blocks))), final_norm=norm, tie_head=False,
                           max_positions=int(c.max_positions), names=("embedding", "layers", "final_norm", "head"))

    def checkpoint_layout(self) -> List[TensorLayout]:
        c = self.config
        d = c.width
        out = [TensorLayout("embed", (c.vocab, d), "embedding")]
        for i, layer in enumerate(c.layers):
            if layer.get("weights_of") is not None:
                continue
            p, m = f"l{i}.", layer["mixer"]
            out.append(TensorLayout(p + "norm1", (d,), "around_zero"))
            if layer["type"] == "mamba2":
                h, v, n, g, taps = (int(m[k]) for k in ("heads", "vdim", "state", "groups", "conv"))
                inner, ch = h * v, h * v + 2 * g * n
                out += [TensorLayout(p + "mix.in", (inner + ch + h, d), "matrix"), TensorLayout(p + "mix.conv", (ch, taps), "taps"),
                        TensorLayout(p + "mix.conv.b", (ch,), "around_zero"), TensorLayout(p + "mix.dt_bias", (h,), "around_zero"),
                        TensorLayout(p + "mix.A_log", (h,), "around_zero"), TensorLayout(p + "mix.D", (h,), "gain"),
                        TensorLayout(p + "mix.norm", (inner,), "gain"), TensorLayout(p + "mix.o", (d, inner), "matrix")]
            else:
                left, right = m["left"], m["right"]
                h, g, k, v = (int(left[x]) for x in ("heads", "kv_heads", "dim", "vdim"))
                q = p + "mix.left."
                out += [TensorLayout(q + "q", (h * k, d), "matrix"), TensorLayout(q + "q.b", (h * k,), "around_zero"),
                        TensorLayout(q + "k", (g * k, d), "matrix"), TensorLayout(q + "k.b", (g * k,), "around_zero"),
                        TensorLayout(q + "v", (g * v, d), "matrix"), TensorLayout(q + "v.b", (g * v,), "around_zero"),
                        TensorLayout(q + "sink", (h,), "around_zero"), TensorLayout(q + "g", (h * v, d), "matrix"),
                        TensorLayout(q + "o", (d, h * v), "matrix")]
                h, g, k, v, taps = (int(right[x]) for x in ("heads", "kv_heads", "dim", "vdim", "conv"))
                ra, rg = int(right.get("decay_rank", 0)), int(right.get("gate_rank", 0))
                q = p + "mix.right."
                out += [TensorLayout(q + "q", (g * k, d), "matrix"), TensorLayout(q + "q.conv", (g * k, taps), "taps"),
                        TensorLayout(q + "k", (g * k, d), "matrix"), TensorLayout(q + "k.conv", (g * k, taps), "taps"),
                        TensorLayout(q + "v", (h * v, d), "matrix"), TensorLayout(q + "v.conv", (h * v, taps), "taps"),
                        TensorLayout(q + "b", (h, d), "matrix"), TensorLayout(q + "A_log", (h,), "around_zero"),
                        TensorLayout(q + "norm", (v,), "gain"), TensorLayout(q + "a1", (ra, d), "matrix"),
                        TensorLayout(q + "a2", (h * k, ra), "matrix"), TensorLayout(q + "dt_bias", (h * k,), "around_zero"),
                        TensorLayout(q + "g1", (rg, d), "matrix"), TensorLayout(q + "g2", (h * v, rg), "matrix"),
                        TensorLayout(q + "o", (d, h * v), "matrix")]
            if layer.get("mlp") is not None:
                f = int(layer["mlp"]["ff"])
                out += [TensorLayout(p + "norm2", (d,), "around_zero"), TensorLayout(p + "mlp.gate", (f, d), "matrix"),
                        TensorLayout(p + "mlp.up", (f, d), "matrix"), TensorLayout(p + "mlp.down", (d, f), "matrix")]
        out += [TensorLayout("final.norm", (d,), "around_zero"), TensorLayout("head", (c.vocab, d), "head")]
        return out


# ---- checkpoint adapter ------------------------------------------------------------------------------
_LAYER = re.compile(r"^l(\d+)\.(.*)$")
_RENAMED = {  # checkpoint name within a layer -> the engine's
    "norm1": "norm1.weight", "norm2": "norm2.weight", "mlp.down": "mlp.w2.weight",
    "mix.in": "mix.in_proj.weight", "mix.conv": "mix.conv", "mix.conv.b": "mix.conv_bias", "mix.dt_bias": "mix.dt_bias",
    "mix.A_log": "mix.A_log", "mix.D": "mix.D", "mix.norm": "mix.norm", "mix.o": "mix.dense.weight",
    "mix.left.sink": "mix.left.sink", "mix.left.o": "mix.left.dense.weight",
    "mix.right.A_log": "mix.right.A_log", "mix.right.norm": "mix.right.norm", "mix.right.dt_bias": "mix.right.dt_bias",
    "mix.right.a1": "mix.right.decay_in.weight", "mix.right.a2": "mix.right.decay_out.weight",
    "mix.right.g1": "mix.right.gate_in.weight", "mix.right.g2": "mix.right.gate_out.weight",
    "mix.right.o": "mix.right.dense.weight",
}


def _fuse(held: Dict[str, torch.Tensor], names, out: Dict[str, torch.Tensor], target: str) -> bool:
    """Concatenates the tensors ``names`` of ``held`` along their rows into out[target] if all of them are there."""
    if not all(n in held for n in names):
        return False
    out[target] = torch.cat([held.pop(n) for n in names], dim=0)
    return True


def _native_to_engine(tensors: Dict[str, torch.Tensor], config: NiletarConfig = None, **_) -> Dict[str, torch.Tensor]:
    """Names and layouts of the checkpoint -> the engine's.  Incomplete sets (a projection without its partners) are
    passed on under their own names, so that the loader's one error lists them."""
    out: Dict[str, torch.Tensor] = {}
    layers: Dict[int, Dict[str, torch.Tensor]] = {}
    top = {"embed": "embedding.weight", "final.norm": "final_norm.weight", "head": "head.weight"}
    for name, t in tensors.items():
        m = _LAYER.match(name)
        if m:
            layers.setdefault(int(m.group(1)), {})[m.group(2)] = t
        else:
            out[top.get(name, name)] = t
    for i, held in layers.items():
        p = f"layers.{i}."
        left = ["mix.left.q", "mix.left.k", "mix.left.v", "mix.left.g"]
        biases = ["mix.left.q.b", "mix.left.k.b", "mix.left.v.b"]
        if all(n in held for n in left + biases):
            gate_rows = held["mix.left.g"].shape[0]
            b = [held.pop(n) for n in biases]
            out[p + "mix.left.in_proj.bias"] = torch.cat(b + [torch.zeros(gate_rows, dtype=b[0].dtype, device=b[0].device)])
            _fuse(held, left, out, p + "mix.left.in_proj.weight")
        right = ["mix.right.q", "mix.right.k", "mix.right.v"]
        if all(n in held for n in right + ["mix.right.b"] + [n + ".conv" for n in right]):
            _fuse(held, [n + ".conv" for n in right], out, p + "mix.right.conv")
            _fuse(held, right + ["mix.right.b"], out, p + "mix.right.in_proj.weight")
        _fuse(held, ["mlp.gate", "mlp.up"], out, p + "mlp.wg1_fused.weight")
        for k in list(held):
            if k in _RENAMED:
                out[p + _RENAMED[k]] = held.pop(k)
        for k, t in held.items():  # whatever found no place keeps its name and is reported
            out[f"l{i}.{k}"] = t
    return out


register_architecture("niletar", Niletar, config_json_names=("Niletar",))
register_adapter_step("niletar", "native_to_engine", _native_to_engine)
register_adapter("niletar", "native", ["native_to_engine"])


# ---- variants ----------------------------------------------------------------------------------------
def alternating(n_layers: int, width: int, vocab: int, ff: int, heads: int, kv_heads: int, dim: int, rot_dims: int,
                delta_heads: int, delta_kv_heads: int, delta_dim: int, delta_vdim: int, ssm_heads: int, ssm_vdim: int,
                state: int, groups: int, rank: int, alpha: float = 2.0, base: float = 10000.0) -> NiletarConfig:
    """Layers that alternate the parallel mixer and the state-space scan, each with a dense feed-forward."""
    mlp = dense_mlp(ff)
    par = parallel_layer(attention_side(heads, kv_heads, dim, dim, rot_dims, base, dim ** -0.5),
                         delta_side(delta_heads, delta_kv_heads, delta_dim, delta_vdim, 4, rank, rank), 0.5, 0.5, mlp)
    ssm = mamba2_layer(ssm_heads, ssm_vdim, state, groups, groups, 4, mlp)
    return NiletarConfig(vocab=vocab, width=width, postln_alpha=alpha,
                         layers=[copy.deepcopy(par if i % 2 == 0 else ssm) for i in range(n_layers)])


def _factory(config: NiletarConfig):
    def make(**kwargs) -> Niletar:
        return Niletar(copy.deepcopy(config), **kwargs)

    return make


# "tiny": for trying things out.  "8b-shape": layers of the width of the Llama-3-8B benchmark (4,096 wide; 32 heads of
# 128 over 8 beside a delta rule of 16 heads of 128; a scan of 64 heads of 128 with a state of 128; a feed-forward of
# 14,336), with which the two are measured side by side.
register_model("niletar", "tiny", _factory(alternating(4, 64, 256, 96, 4, 2, 16, 8, 2, 1, 16, 24, 4, 16, 16, 2, 8)))
register_model("niletar", "8b-shape", _factory(alternating(32, 4096, 128256, 14336, 32, 8, 128, 64, 16, 16, 128, 128, 64,
                                                           128, 128, 8, 64)))
