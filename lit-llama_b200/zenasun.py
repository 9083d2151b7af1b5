"""Zenasun: a decoder-only language model of parallel layers.  Every layer reads the same residual x through two
norms, one for its sequence mixer and one for its routed-expert feed-forward, and adds both results at once:

    x = embed[token] * embedding.scale
    x <- x + (mixer(norm1(x)) + experts(norm2(x)))                 per layer (a layer may have no feed-forward)
    logits = cap * tanh(embed . norm(x) / cap)                      the embedding table is the output head

with RMS norms whose weights are stored around zero (x / rms(x) * (1 + w)), an f32 residual stream, and two kinds of
mixer: latent attention (`LatentAttention`) and retention (`RetentionMixer`).  A layer entry with "weights_of": j
runs with layer j's tensors (mixer, feed-forward and norms) on a cache or state of its own.

Everything about a model comes from its config.json (`ZenasunConfig`) and from the shapes of its tensors.  Tensor
names: `embed`, `l<i>.norm1|norm2`, `l<i>.mix.*`, `l<i>.mlp.router|correction|e<k>.gate|up|down`, `final.norm`; linear
weights are [out, in].  The layers are built from the mechanisms of `mixers.py`; what a sequence carries between steps
is declared through `state_specs()` and lives in a `SequenceStatePool`, so the `Engine` serves this model like any
other."""
import copy
import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from . import _seqlib as S
from .mixers import LatentAttention, MoEFeedForward, RetentionMixer, StepContext, _p, linear_f32
from .state import StateSpec

MIXERS = ("latent_attention", "retention")
DEFAULT_MAX_POSITIONS = 4096


@dataclass
class ZenasunConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_softcap: Optional[float]
    layers: List[dict] = field(default_factory=list)

    @classmethod
    def from_dict(cls, d: dict) -> "ZenasunConfig":
        if d.get("architecture") not in (None, "Zenasun"):
            raise ValueError(f"not a Zenasun configuration: architecture = {d.get('architecture')!r}")
        layers = list(d["layers"])
        for i, layer in enumerate(layers):
            if layer["type"] not in MIXERS:
                raise ValueError(f"layer {i}: unknown layer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp and mlp.get("kind", "moe") != "moe":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            j = layer.get("weights_of")
            if j is not None and not (0 <= int(j) < len(layers) and layers[int(j)].get("weights_of") is None and
                                      layers[int(j)]["type"] == layer["type"]):
                raise ValueError(f"layer {i}: weights_of = {j!r} does not name a layer of the same type with tensors of its own")
        cap = d.get("logit_softcap")
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]),
                   embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)), logit_softcap=float(cap) if cap else None, layers=layers)

    @classmethod
    def from_json(cls, path: str) -> "ZenasunConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        return {"architecture": "Zenasun", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "embedding": {"scale": self.embedding_scale}, "logit_softcap": self.logit_softcap, "layers": self.layers}


def build_mixer(name: str, kind: str, c: dict, W: Dict[str, torch.Tensor], p: str, eps: float, max_positions: int):
    if kind == "latent_attention":
        return LatentAttention(name, W, p, heads=c["heads"], dim=c["dim"], rot_dim=c.get("rot_dim", 0), vdim=c["vdim"], q_rank=c["q_rank"],
                               kv_rank=c["kv_rank"], scale=c["scale"], eps=eps, rot=c.get("rot"), max_positions=max_positions, interleaved=True)
    if kind == "retention":
        return RetentionMixer(name, W, p, heads=c["heads"], dim=c["dim"], vdim=c["vdim"], decay=c["decay"], eps=eps, rot=c.get("rot"),
                              interleaved=False)
    raise ValueError(kind)


def build_experts(m: dict, W: Dict[str, torch.Tensor], p: str) -> MoEFeedForward:
    r = m["router"]
    g = r.get("groups") or {}
    return MoEFeedForward(W, p, experts=r["experts"], identity=r.get("identity", 0), top=r["top"], groups=g.get("count", 1), keep=g.get("keep", 1),
                          ff=m["expert"]["ff"], act="silu")


class _Layer:
    """A layer's mechanisms.  `share` is the layer whose tensors this one runs with: the mechanisms are shallow copies
    (the same weight tensors) under this layer's own state names."""

    def __init__(self, i: int, spec: dict, W: Dict[str, torch.Tensor], eps: float, max_positions: int, share: Optional["_Layer"]) -> None:
        if share is not None:
            self.mixer = copy.copy(share.mixer)
            self.mixer.name = f"l{i}"
            self.mlp, self.norm1, self.norm2 = share.mlp, share.norm1, share.norm2
            return
        p = f"l{i}."
        self.mixer = build_mixer(f"l{i}", spec["type"], spec["mixer"], W, p + "mix.", eps, max_positions)
        self.norm1 = W[p + "norm1"].contiguous()
        self.mlp: Optional[MoEFeedForward] = None
        self.norm2 = None
        if spec.get("mlp"):
            self.mlp = build_experts(spec["mlp"], W, p + "mlp.")
            self.norm2 = W[p + "norm2"].contiguous()


class Zenasun:
    """The model over a dict of device tensors in the activation dtype (torch.bfloat16, or torch.float32 for true
    32-bit arithmetic throughout).  `max_positions`: the most positions a sequence may reach (the attention layers
    cache every position)."""

    graph_safe = True

    def __init__(self, config: ZenasunConfig, weights: Dict[str, torch.Tensor], max_positions: int = 0) -> None:
        self.config = config
        self.embed = weights["embed"].contiguous()
        self.dtype, self.device = self.embed.dtype, self.embed.device
        if not self.embed.is_cuda:
            raise RuntimeError("Zenasun runs on CUDA only (no CPU fallback)")
        S.act_code(self.dtype)
        if tuple(self.embed.shape) != (config.vocab, config.width):
            raise ValueError(f"embed is {tuple(self.embed.shape)}, the configuration says {(config.vocab, config.width)}")
        self.vocab, self.width, self.eps = config.vocab, config.width, config.eps
        self.max_positions = int(max_positions) if max_positions and max_positions > 0 else DEFAULT_MAX_POSITIONS
        self.layers: List[Optional[_Layer]] = [None] * len(config.layers)
        for i, spec in enumerate(config.layers):
            if spec.get("weights_of") is None:
                self.layers[i] = _Layer(i, spec, weights, config.eps, self.max_positions, None)
        for i, spec in enumerate(config.layers):
            if self.layers[i] is None:
                self.layers[i] = _Layer(i, spec, weights, config.eps, self.max_positions, self.layers[int(spec["weights_of"])])
        self.final_norm = weights["final.norm"].contiguous()
        self.capture_layers: Optional[List[torch.Tensor]] = None     # set to [] to record the residual stream after every layer

    # ------------------------------------------------------------------ framework interface
    def state_specs(self) -> Dict[str, StateSpec]:
        out: Dict[str, StateSpec] = {}
        for layer in self.layers:
            out.update(layer.mixer.state_specs())
        return out

    def n_parameters(self) -> int:
        seen, n = set(), 0
        for layer in self.layers:
            for obj in (layer.mixer, layer.mlp):
                for k, v in vars(obj).items() if obj is not None else []:
                    if k == "w_expand":            # a second arrangement of W_uk and W_uv, not more parameters
                        continue
                    if isinstance(v, torch.Tensor) and v.is_floating_point() and v.dim() >= 2 and v.data_ptr() not in seen:
                        seen.add(v.data_ptr())
                        n += v.numel()
        return n + self.embed.numel()

    def _norms(self, y1, y2, x, layer: Optional[_Layer], h1, h2, T: int, ctx: StepContext) -> None:
        w1 = layer.norm1 if layer is not None else None
        w2 = layer.norm2 if layer is not None else None
        S.check(S.lib().b2l_seq_add_norm2(_p(y1), _p(y2), _p(x), _p(w1), _p(h1) if w1 is not None else None, _p(w2),
                                          _p(h2) if w2 is not None else None, 1.0, self.eps, None, T, self.width, ctx.act, ctx.stream),
                "b2l_seq_add_norm2")

    @torch.no_grad()
    def forward_portion(self, tokens: torch.Tensor, ctx: StepContext, want: Optional[torch.Tensor] = None) -> torch.Tensor:
        """tokens: device int32/int64 [T], the next T tokens of the sequence in ctx's slot.  want: device int32 indices
        into the portion (None = every token).  Returns f32 logits [len(want), vocab]."""
        lib, T, D, dev = S.lib(), ctx.T, self.width, self.device
        if torch.backends.cuda.matmul.allow_tf32:
            raise RuntimeError("32-bit products of this model (router, float32 mode) must be true f32: torch.backends.cuda.matmul.allow_tf32 is on")
        x = torch.empty((T, D), dtype=torch.float32, device=dev)
        S.check(lib.b2l_seq_embed(_p(tokens), int(tokens.dtype == torch.int64), _p(self.embed), ctx.act, self.config.embedding_scale, _p(x), T, D,
                                  self.vocab, ctx.stream), "b2l_seq_embed")
        h1 = torch.empty((T, D), dtype=self.dtype, device=dev)
        h2 = torch.empty((T, D), dtype=self.dtype, device=dev)
        if self.layers:
            self._norms(None, None, x, self.layers[0], h1, h2, T, ctx)
        n = T if want is None else int(want.numel())
        fuse_last = T == 1 and n == 1 and len(self.layers) > 0      # a single token: the last sum and the final norm in one launch
        hn = torch.empty((n, D), dtype=self.dtype, device=dev) if n else None
        for i, layer in enumerate(self.layers):
            y1 = layer.mixer.forward(h1, ctx)
            y2 = layer.mlp.forward(h2, ctx) if layer.mlp is not None else None
            if i + 1 == len(self.layers) and fuse_last:
                S.check(lib.b2l_seq_add_norm2(_p(y1), _p(y2), _p(x), _p(self.final_norm), _p(hn), None, None, 1.0, self.eps, None, 1, D, ctx.act,
                                              ctx.stream), "b2l_seq_add_norm2")
            else:
                self._norms(y1, y2, x, self.layers[i + 1] if i + 1 < len(self.layers) else None, h1, h2, T, ctx)
            if self.capture_layers is not None:
                self.capture_layers.append(x.clone())
        if n == 0:
            return torch.empty((0, self.vocab), dtype=torch.float32, device=dev)
        if not fuse_last:
            S.check(lib.b2l_seq_add_norm2(None, None, _p(x), _p(self.final_norm), _p(hn), None, None, 1.0, self.eps, _p(want), n, D, ctx.act,
                                          ctx.stream), "b2l_seq_add_norm2")
        logits = linear_f32(hn, self.embed)
        if self.config.logit_softcap:
            S.check(lib.b2l_seq_softcap(_p(logits), logits.numel(), self.config.logit_softcap, ctx.stream), "b2l_seq_softcap")
        return logits


def load(model_dir: str, dtype: torch.dtype = torch.bfloat16, device: Optional[torch.device] = None, max_positions: int = 0) -> Zenasun:
    """config.json + model.safetensors of `model_dir` -> a model on `device`."""
    from .checkpoint_io import read_safetensors

    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    config = ZenasunConfig.from_json(os.path.join(model_dir, "config.json"))
    weights = read_safetensors(os.path.join(model_dir, "model.safetensors"), device=device, float_dtype=dtype)
    return Zenasun(config, weights, max_positions=max_positions)


def random_weights(cfg: dict, device, dtype: torch.dtype = torch.bfloat16, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random tensors with the family's names and shapes (projections ~ N(0, 1/in), norm weights around zero), for
    benchmarks and smoke runs."""
    import math

    g = torch.Generator(device="cpu").manual_seed(seed)
    D, W = cfg["width"], {}

    def lin(o, i):
        return (torch.randn(o, i, generator=g) / math.sqrt(i)).to(device, dtype)

    def vec(n, mean=0.0, std=0.1):
        return (mean + std * torch.randn(n, generator=g)).to(device, dtype)

    W["embed"], W["final.norm"] = (torch.randn(cfg["vocab"], D, generator=g) / math.sqrt(D)).to(device, dtype), vec(D)
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p, m, c = f"l{i}.", f"l{i}.mix.", layer["mixer"]
        W[p + "norm1"] = vec(D)
        if layer["type"] == "latent_attention":
            H, dn, dr, dv, rq, rk = c["heads"], c["dim"], c.get("rot_dim", 0), c["vdim"], c["q_rank"], c["kv_rank"]
            W[m + "dq"], W[m + "dq.norm"], W[m + "uq"] = lin(rq, D), vec(rq, 1.0), lin(H * (dn + dr), rq)
            W[m + "dkv"], W[m + "dkv.norm"] = lin(rk + dr, D), vec(rk, 1.0)
            W[m + "uk"], W[m + "uv"], W[m + "sink"], W[m + "o"] = lin(H * dn, rk), lin(H * dv, rk), vec(H, 0.0, 1.0), lin(D, H * dv)
        else:
            H, K, V = c["heads"], c["dim"], c["vdim"]
            W[m + "q"], W[m + "k"], W[m + "v"], W[m + "g"], W[m + "o"] = lin(H * K, D), lin(H * K, D), lin(H * V, D), lin(H * V, D), lin(D, H * V)
        if layer.get("mlp"):
            r, ff = layer["mlp"]["router"], layer["mlp"]["expert"]["ff"]
            n = r["experts"] + r.get("identity", 0)
            W[p + "norm2"], W[p + "mlp.router"], W[p + "mlp.correction"] = vec(D), lin(n, D), vec(n, 0.0, 0.01)
            for e in range(r["experts"]):
                q = f"{p}mlp.e{e}."
                W[q + "gate"], W[q + "up"], W[q + "down"] = lin(ff, D), lin(ff, D), lin(D, ff)
    return W
