"""Goletar: a decoder whose layers alternate freely between a gated recurrence (minGRU) and attention over cached
latents, each followed by a feed-forward of routed experts (or none), with a norm before and after every sublayer and
an embedding that adds a hashed row for the pair (previous token, token).

This file is all that is specific to the architecture: its ``config.json`` (every size and constant is read from it;
``layers`` lists the layers in order, each with its ``type``, the sizes of its ``mixer`` and its ``mlp`` or null), the
``DecoderSpec`` that configuration means, and the checkpoint's tensor names and layouts:

    embed [vocab, width]    bigram [buckets + 1, width]    final.norm []    head [vocab, width]
    l<i>.norm1, norm1b, norm2, norm2b []          (one number each)
    mingru:            l<i>.mix.z, .z.b, .x, .x.b, .g, .o
    latent_attention:  l<i>.mix.q, .dkv, .dkv.norm, .uk, .uv, .sink, .g, .o
    experts:           l<i>.mlp.router, l<i>.mlp.e<j>.gate, .up, .down

Linear weights are stored [out, in].  The adapter fuses [z; x; g] (bias [z.b; x.b; 0]) and [q; dkv; g] into one
projection each and stacks the experts' matrices.
"""
from __future__ import annotations

import copy
import dataclasses
import re
from typing import Any, Dict, List, Optional

import torch

from ..config.model_config import ModelConfig
from ..config.specs import (BlockSpec, DecoderSpec, EmbeddingSpec, FeedForwardSpec, LayerCall, MixerSpec, NormSpec,
                            PositionSpec)
from ..weights.adapters import register_adapter, register_adapter_step
from ..weights.sources import TensorLayout
from . import register_architecture, register_model
from .base import Model

GATE_ALPHA = 1.702  # the experts' gate is v * sigmoid(GATE_ALPHA * v)


@dataclasses.dataclass
class GoletarConfig(ModelConfig):
    vocab: int = 512
    width: int = 256
    norm_eps: float = 1e-6
    buckets: int = 4093
    mul_prev: int = 1009
    mul_cur: int = 271
    layers: List[Dict[str, Any]] = dataclasses.field(default_factory=list)
    max_positions: int = 131072  # how long a sequence may get; nothing in the model depends on it

    def __post_init__(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or self.buckets <= 0:
            raise ValueError(f"vocab {self.vocab}, width {self.width}, buckets {self.buckets}")
        for i, layer in enumerate(self.layers):
            if layer.get("type") not in ("mingru", "latent_attention"):
                raise ValueError(f"layer {i}: type {layer.get('type')!r}; known: mingru, latent_attention")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") != "moe":
                raise ValueError(f"layer {i}: feed-forward kind {mlp.get('kind')!r}; known: moe, or null for none")


def _config_from_json(values: Dict[str, Any]) -> GoletarConfig:
    if values.get("architecture") != "Goletar":
        raise ValueError(f"config.json is of architecture {values.get('architecture')!r}, not Goletar")
    absent = [k for k in ("vocab", "width", "layers", "norm", "embedding") if k not in values]
    if absent:
        raise ValueError(f"config.json lacks {absent}")
    pairs = values["embedding"]["bigram"]
    return GoletarConfig(vocab=int(values["vocab"]), width=int(values["width"]), norm_eps=float(values["norm"]["eps"]),
                         buckets=int(pairs["buckets"]), mul_prev=int(pairs["mul_prev"]), mul_cur=int(pairs["mul_cur"]),
                         layers=copy.deepcopy(values["layers"]),
                         max_positions=int(values.get("max_positions", 131072)))


def mingru_layer(width: int, mlp: Optional[dict]) -> dict:
    return {"type": "mingru", "mixer": {"width": width}, "mlp": mlp}


def latent_layer(heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, base: float, mlp: Optional[dict],
                 scale: Optional[float] = None) -> dict:
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                      "rot": {"base": base, "dims": rot_dim},
                      "scale": (dim + rot_dim) ** -0.5 if scale is None else scale}}


def moe(experts: int, top: int, ff: int, limit: float) -> dict:
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


class Goletar(Model):
    architecture = "goletar"
    default_source = "native"

    def __init__(self, config: Optional[GoletarConfig] = None, **kwargs) -> None:
        config = config if config is not None else GoletarConfig()
        super().__init__(config.updated(**kwargs))

    @classmethod
    def config_from_json(cls, values: dict) -> GoletarConfig:
        return _config_from_json(values)

    def config_json(self) -> dict:
        c = self.config
        return {"architecture": "Goletar", "vocab": c.vocab, "width": c.width, "norm": {"eps": c.norm_eps},
                "embedding": {"bigram": {"buckets": c.buckets, "mul_prev": c.mul_prev, "mul_cur": c.mul_cur}},
                "layers": copy.deepcopy(c.layers)}

    def decoder_spec(self) -> DecoderSpec:
        c = self.config
        norm = NormSpec("rmsnorm_scalar", c.width, float(c.norm_eps))
        blocks = []
        for layer in c.layers:
            m = layer["mixer"]
            if layer["type"] == "mingru":
                mixer = MixerSpec("mingru", dim=c.width, options=(("width", int(m["width"])),))
            else:
                rot = m.get("rot") or {}
                mixer = MixerSpec(
                    "latent_attention", dim=c.width, nheads=int(m["heads"]), kvheads=1, head_dim=int(m["dim"]),
                    scale=float(m["scale"]),
                    position=PositionSpec("rope", head_dim=int(rot.get("dims", m["rot_dim"])),
                                          theta=float(rot.get("base", 10000.0))),
                    options=(("rot", int(m["rot_dim"])), ("vdim", int(m["vdim"])), ("rank", int(m["kv_rank"])),
                             ("rot_dims", int(rot.get("dims", m["rot_dim"]))), ("eps", float(c.norm_eps))))
            ff = None
            if layer.get("mlp") is not None:
                mlp = layer["mlp"]
                ff = FeedForwardSpec("routed_experts", dim=c.width, hidden=int(mlp["expert"]["ff"]),
                                     activation="swish_clamped",
                                     options=(("experts", int(mlp["router"]["experts"])), ("top", int(mlp["router"]["top"])),
                                              ("limit", float(mlp["expert"]["limit"])), ("alpha", GATE_ALPHA)))
            blocks.append(BlockSpec(mixer=mixer, feed_forward=ff, mixer_norm=norm,
                                    feed_forward_norm=norm if ff is not None else None, arrangement="sandwich",
                                    names=("norm1", "mix", "norm2", "mlp"), mixer_post_norm=norm,
                                    feed_forward_post_norm=norm if ff is not None else None,
                                    post_names=("norm1b", "norm2b")))
        return DecoderSpec(
            vocab_size=c.vocab, dim=c.width, layers=tuple(blocks), schedule=tuple(LayerCall(i) for i in range(len(blocks))),
            final_norm=norm, tie_head=False, max_positions=int(c.max_positions),
            names=("embedding", "layers", "final_norm", "head"),
            embedding=EmbeddingSpec("pair_hash", (("buckets", c.buckets), ("mul_prev", c.mul_prev),
                                                  ("mul_cur", c.mul_cur), ("name", "pairs"))))

    def checkpoint_layout(self) -> List[TensorLayout]:
        c = self.config
        d = c.width
        out = [TensorLayout("embed", (c.vocab, d), "embedding"), TensorLayout("bigram", (c.buckets + 1, d), "embedding")]
        for i, layer in enumerate(c.layers):
            p, m = f"l{i}.", layer["mixer"]
            names = ["norm1", "norm1b"] + (["norm2", "norm2b"] if layer.get("mlp") is not None else [])
            out += [TensorLayout(p + n, (), "gain") for n in names]
            if layer["type"] == "mingru":
                w = int(m["width"])
                out += [TensorLayout(p + "mix.z", (w, d), "matrix"), TensorLayout(p + "mix.z.b", (w,), "matrix"),
                        TensorLayout(p + "mix.x", (w, d), "matrix"), TensorLayout(p + "mix.x.b", (w,), "matrix"),
                        TensorLayout(p + "mix.g", (w, d), "matrix"), TensorLayout(p + "mix.o", (d, w), "matrix")]
            else:
                h, dim, rot, v, r = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"))
                out += [TensorLayout(p + "mix.q", (h * (dim + rot), d), "matrix"),
                        TensorLayout(p + "mix.dkv", (r + rot, d), "matrix"), TensorLayout(p + "mix.dkv.norm", (r,), "gain"),
                        TensorLayout(p + "mix.uk", (h * dim, r), "matrix"), TensorLayout(p + "mix.uv", (h * v, r), "matrix"),
                        TensorLayout(p + "mix.sink", (h,), "matrix"), TensorLayout(p + "mix.g", (h, d), "matrix"),
                        TensorLayout(p + "mix.o", (d, h * v), "matrix")]
            if layer.get("mlp") is not None:
                mlp = layer["mlp"]
                f = int(mlp["expert"]["ff"])
                out.append(TensorLayout(p + "mlp.router", (int(mlp["router"]["experts"]), d), "matrix"))
                for j in range(int(mlp["router"]["experts"])):
                    out += [TensorLayout(p + f"mlp.e{j}.gate", (f, d), "matrix"),
                            TensorLayout(p + f"mlp.e{j}.up", (f, d), "matrix"),
                            TensorLayout(p + f"mlp.e{j}.down", (d, f), "matrix")]
        out += [TensorLayout("final.norm", (), "gain"), TensorLayout("head", (c.vocab, d), "head")]
        return out


# ---- checkpoint adapter ------------------------------------------------------------------------------
_LAYER = re.compile(r"^l(\d+)\.(.*)$")
_EXPERT = re.compile(r"^mlp\.e(\d+)\.(gate|up|down)$")


def _native_to_engine(tensors: Dict[str, torch.Tensor], config: GoletarConfig = None, **_) -> Dict[str, torch.Tensor]:
    """Names and layouts of the checkpoint -> the engine's.  Incomplete sets (a projection without its partners, an
    expert that lacks a matrix) are passed on under their own names, so that the loader's one error lists them."""
    out: Dict[str, torch.Tensor] = {}
    layers: Dict[int, Dict[str, torch.Tensor]] = {}
    top = {"embed": "embedding.weight", "bigram": "embedding.pairs", "final.norm": "final_norm.weight", "head": "head.weight"}
    for name, t in tensors.items():
        m = _LAYER.match(name)
        if m:
            layers.setdefault(int(m.group(1)), {})[m.group(2)] = t
        else:
            out[top.get(name, name)] = t
    for i, held in layers.items():
        p = f"layers.{i}."
        kind = config.layers[i]["type"] if config is not None and i < len(config.layers) else None
        for n in ("norm1", "norm1b", "norm2", "norm2b"):
            if n in held:
                out[p + n + ".weight"] = held.pop(n)
        if kind == "mingru" and all(k in held for k in ("mix.z", "mix.z.b", "mix.x", "mix.x.b", "mix.g")):
            z, zb, x, xb, g = (held.pop(k) for k in ("mix.z", "mix.z.b", "mix.x", "mix.x.b", "mix.g"))
            out[p + "mix.zxg_fused.weight"] = torch.cat([z, x, g], dim=0)
            out[p + "mix.zxg_fused.bias"] = torch.cat([zb, xb, torch.zeros(g.shape[0], dtype=zb.dtype, device=zb.device)])
        if kind == "latent_attention" and all(k in held for k in ("mix.q", "mix.dkv", "mix.g")):
            out[p + "mix.in_proj.weight"] = torch.cat([held.pop("mix.q"), held.pop("mix.dkv"), held.pop("mix.g")], dim=0)
            for src, dst in (("mix.dkv.norm", "mix.latent_norm"), ("mix.uk", "mix.uk"), ("mix.uv", "mix.uv"),
                             ("mix.sink", "mix.sink")):
                if src in held:
                    out[p + dst] = held.pop(src)
        if "mix.o" in held:
            out[p + "mix.dense.weight"] = held.pop("mix.o")
        if "mlp.router" in held:
            out[p + "mlp.router.weight"] = held.pop("mlp.router")
        experts: Dict[int, Dict[str, torch.Tensor]] = {}
        for k in list(held):
            m = _EXPERT.match(k)
            if m:
                experts.setdefault(int(m.group(1)), {})[m.group(2)] = held[k]
        n = len(experts)
        if n and sorted(experts) == list(range(n)) and all(len(e) == 3 for e in experts.values()):
            out[p + "mlp.gate_up"] = torch.stack([torch.cat([experts[j]["gate"], experts[j]["up"]], dim=0) for j in range(n)])
            out[p + "mlp.down"] = torch.stack([experts[j]["down"] for j in range(n)])
            for j in range(n):
                for part in ("gate", "up", "down"):
                    held.pop(f"mlp.e{j}.{part}")
        for k, t in held.items():  # whatever found no place keeps its name and is reported
            out[f"l{i}.{k}"] = t
    return out


register_architecture("goletar", Goletar, config_json_names=("Goletar",))
register_adapter_step("goletar", "native_to_engine", _native_to_engine)
register_adapter("goletar", "native", ["native_to_engine"])


# ---- variants ----------------------------------------------------------------------------------------
def alternating(n_layers: int, width: int, recurrent_width: int, heads: int, dim: int, rot_dim: int, vdim: int,
                kv_rank: int, experts: int, top: int, ff: int, vocab: int, limit: float = 7.0,
                base: float = 10000.0) -> GoletarConfig:
    """Layers that alternate minGRU and latent attention, each with routed experts."""
    mlp = moe(experts, top, ff, limit)
    layers = [mingru_layer(recurrent_width, mlp) if i % 2 == 0 else latent_layer(heads, dim, rot_dim, vdim, kv_rank, base, mlp)
              for i in range(n_layers)]
    return GoletarConfig(vocab=vocab, width=width, layers=layers)


def _factory(config: GoletarConfig):
    def make(**kwargs) -> Goletar:
        return Goletar(config, **kwargs)

    return make


# "tiny": for trying things out.  "8b-shape": layers of the width of the Llama-3-8B benchmark (4,096 wide, 32 heads
# of 128 = 96 + 32 values, a latent of 512, 16 experts of 3,584 of which each token takes 4: the same 14,336 hidden
# values a token as the dense feed-forward), with which the two are measured side by side.
register_model("goletar", "tiny", _factory(alternating(4, 64, 80, 4, 16, 8, 16, 32, 4, 2, 48, 256)))
register_model("goletar", "8b-shape", _factory(alternating(32, 4096, 4096, 32, 96, 32, 128, 512, 16, 4, 3584, 128256)))
