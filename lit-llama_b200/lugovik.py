"""Lugovik: a decoder-only language model whose layers mix three kinds of sequence mixer (a channel-wise gated delta
rule, a block-local sink attention side by side with gated linear attention, and state-space duality layers), each
followed by an optional gated feed-forward, with RMS norms before AND after every sublayer and an f32 residual
stream:

    x = embed[token] * embedding.scale
    x <- x + norm1b(mixer(norm1(x)));   x <- x + norm2b(ff(norm2(x)))          per layer
    logits = head(norm(x))

Everything about a model comes from its config.json (`LugovikConfig`) and from the shapes of its tensors: layer
order, head counts, sizes, block size, rotation, scales.  The layers are built from the mechanisms of `mixers.py`;
what a sequence carries between steps is declared through `state_specs()` and lives in a `SequenceStatePool`, so the
`Engine` serves this model like any other.  Tensor names: `embed`, `l<i>.norm1|norm1b|norm2|norm2b`, `l<i>.mix.*`,
`l<i>.mlp.gate|up|down`, `final.norm`, `head`; linear weights are [out, in]."""
import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from . import _seqlib as S
from .mixers import (BlockSinkAttention, ChannelDeltaMixer, GatedLinearAttention, GatedMLP, Mamba2Mixer, ParallelMixer, StepContext, _p,
                     linear)
from .state import StateSpec


@dataclass
class LugovikConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: List[dict] = field(default_factory=list)

    @classmethod
    def from_dict(cls, d: dict) -> "LugovikConfig":
        if d.get("architecture") not in (None, "Lugovik"):
            raise ValueError(f"not a Lugovik configuration: architecture = {d.get('architecture')!r}")
        for layer in d["layers"]:
            if layer["type"] not in ("channel_delta", "parallel", "mamba2"):
                raise ValueError(f"unknown layer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp and mlp.get("kind", "dense") != "dense":
                raise ValueError(f"unknown feed-forward kind {mlp.get('kind')!r}")
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), eps=float(d["norm"]["eps"]),
                   embedding_scale=float(d.get("embedding", {}).get("scale", 1.0)), layers=list(d["layers"]))

    @classmethod
    def from_json(cls, path: str) -> "LugovikConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        return {"architecture": "Lugovik", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "embedding": {"scale": self.embedding_scale}, "layers": self.layers}


class _Layer:
    def __init__(self, i: int, spec: dict, W: Dict[str, torch.Tensor], eps: float, max_positions: int) -> None:
        p, m, c = f"l{i}.", f"l{i}.mix.", spec["mixer"]
        kind = spec["type"]
        if kind == "channel_delta":
            self.mixer = ChannelDeltaMixer(f"l{i}", W, m, heads=c["heads"], kv_heads=c.get("kv_heads", c["heads"]), dim=c["dim"], vdim=c["vdim"],
                                           conv=c["conv"], eps=eps)
        elif kind == "mamba2":
            self.mixer = Mamba2Mixer(f"l{i}", W, m, heads=c["heads"], vdim=c["vdim"], state=c["state"], groups=c.get("groups", 1),
                                     norm_groups=c.get("norm_groups", 1), conv=c["conv"], eps=eps)
        elif kind == "parallel":
            a, b = c["left"], c["right"]
            left = BlockSinkAttention(f"l{i}.left", W, m + "left.", heads=a["heads"], kv_heads=a.get("kv_heads", a["heads"]), dim=a["dim"],
                                      vdim=a["vdim"], scale=a["scale"], eps=eps, softcap=a.get("softcap"),
                                      block=(a.get("mask") or {}).get("size"), rot=a.get("rot"), sink=True, max_positions=max_positions)
            right = GatedLinearAttention(f"l{i}.right", W, m + "right.", heads=b["heads"], dim=b["dim"], vdim=b["vdim"], tau=b["tau"], eps=eps)
            self.mixer = ParallelMixer([(left, c.get("left_scale", 1.0)), (right, c.get("right_scale", 1.0))])
        else:
            raise ValueError(kind)
        self.norm1, self.norm1b = W[p + "norm1"].contiguous(), W[p + "norm1b"].contiguous()
        self.mlp: Optional[GatedMLP] = None
        self.norm2 = self.norm2b = None
        if spec.get("mlp"):
            self.mlp = GatedMLP(W[p + "mlp.gate"], W[p + "mlp.up"], W[p + "mlp.down"], act="gelu_tanh")
            self.norm2, self.norm2b = W[p + "norm2"].contiguous(), W[p + "norm2b"].contiguous()


class Lugovik:
    """The model over a dict of device tensors in the activation dtype (torch.bfloat16, or torch.float32 for true
    32-bit arithmetic throughout)."""

    def __init__(self, config: LugovikConfig, weights: Dict[str, torch.Tensor], max_positions: int = 0) -> None:
        self.config = config
        self.embed = weights["embed"].contiguous()
        self.dtype, self.device = self.embed.dtype, self.embed.device
        if not self.embed.is_cuda:
            raise RuntimeError("Lugovik runs on CUDA only (no CPU fallback)")
        S.act_code(self.dtype)
        if tuple(self.embed.shape) != (config.vocab, config.width):
            raise ValueError(f"embed is {tuple(self.embed.shape)}, the configuration says {(config.vocab, config.width)}")
        self.vocab, self.width, self.eps = config.vocab, config.width, config.eps
        self.layers = [_Layer(i, spec, weights, config.eps, max_positions) for i, spec in enumerate(config.layers)]
        self.final_norm, self.head = weights["final.norm"].contiguous(), weights["head"].contiguous()
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
            for obj in (layer.mixer, layer.mlp, *(getattr(layer.mixer, "branches", []))):
                for v in vars(obj).values() if obj is not None else []:
                    for t in (v if isinstance(v, list) else [v]):
                        if isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
                            seen.add(t.data_ptr())
                            n += t.numel()
        return n + self.embed.numel() + self.head.numel()

    @torch.no_grad()
    def forward_portion(self, tokens: torch.Tensor, ctx: StepContext, want: Optional[torch.Tensor] = None) -> torch.Tensor:
        """tokens: device int32/int64 [T], the next T tokens of the sequence in ctx's slot.  want: device int32 indices
        into the portion (None = every token).  Returns f32 logits [len(want), vocab]."""
        lib, T, D, dev = S.lib(), ctx.T, self.width, self.device
        if self.dtype == torch.float32 and torch.backends.cuda.matmul.allow_tf32:
            raise RuntimeError("float32 models need true 32-bit products: torch.backends.cuda.matmul.allow_tf32 is on")
        x = torch.empty((T, D), dtype=torch.float32, device=dev)
        S.check(lib.b2l_seq_embed(_p(tokens), int(tokens.dtype == torch.int64), _p(self.embed), ctx.act, self.config.embedding_scale, _p(x), T, D,
                                  self.vocab, ctx.stream), "b2l_seq_embed")
        h = torch.empty((T, D), dtype=self.dtype, device=dev)
        if self.layers:
            S.check(lib.b2l_seq_rmsnorm(_p(x), _p(self.layers[0].norm1), self.eps, _p(h), None, T, D, ctx.act, ctx.stream), "b2l_seq_rmsnorm")
        for i, layer in enumerate(self.layers):
            nxt = self.layers[i + 1].norm1 if i + 1 < len(self.layers) else None
            y = layer.mixer.forward(h, ctx)
            after = layer.norm2 if layer.mlp is not None else nxt
            S.check(lib.b2l_seq_norm_add_norm(_p(y), _p(layer.norm1b), self.eps, _p(x), _p(after), _p(h) if after is not None else None, T, D,
                                              ctx.act, ctx.stream), "b2l_seq_norm_add_norm")
            if layer.mlp is not None:
                y = layer.mlp.forward(h, ctx)
                S.check(lib.b2l_seq_norm_add_norm(_p(y), _p(layer.norm2b), self.eps, _p(x), _p(nxt), _p(h) if nxt is not None else None, T, D,
                                                  ctx.act, ctx.stream), "b2l_seq_norm_add_norm")
            if self.capture_layers is not None:
                self.capture_layers.append(x.clone())
        n = T if want is None else int(want.numel())
        if n == 0:
            return torch.empty((0, self.vocab), dtype=torch.float32, device=dev)
        hn = torch.empty((n, D), dtype=self.dtype, device=dev)
        S.check(lib.b2l_seq_rmsnorm(_p(x), _p(self.final_norm), self.eps, _p(hn), _p(want), n, D, ctx.act, ctx.stream), "b2l_seq_rmsnorm")
        if self.dtype == torch.float32:
            return linear(hn, self.head)
        return torch.mm(hn, self.head.t(), out_dtype=torch.float32)     # bf16 product, f32 accumulator kept


def load(model_dir: str, dtype: torch.dtype = torch.bfloat16, device: Optional[torch.device] = None, max_positions: int = 0) -> Lugovik:
    """config.json + model.safetensors of `model_dir` -> a model on `device`."""
    from .checkpoint_io import read_safetensors

    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    config = LugovikConfig.from_json(os.path.join(model_dir, "config.json"))
    weights = read_safetensors(os.path.join(model_dir, "model.safetensors"), device=device, float_dtype=dtype)
    return Lugovik(config, weights, max_positions=max_positions)
