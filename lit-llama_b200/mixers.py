"""Sequence-mixer mechanisms over libb200seq (include/b2l_seq.h), each usable by any model: its sizes and
constants are constructor parameters.

    GatedMLP             act(W_gate h) * (W_up h) -> W_down, both halves from one product
    ChannelDeltaMixer    gated delta rule with one decay per key channel, short convolutions on q / k / v
    BlockSinkAttention   block-local causal softmax attention: q/k norm, partial rotation (YaRN-scaled), soft-capped
                         scores, a sink in the denominator, grouped kv heads, per-head sigmoid output gate, ring cache
    GatedLinearAttention S_t = diag(alpha_t) S_(t-1) + k_t v_t^T with a low-rank decay projection
    ParallelMixer        two mixers on the same input, one output product over their concatenated read-outs
    Mamba2Mixer          state-space duality layer: scalar decay per head, convolution on x | B | C, gated grouped norm

A mixer is built from a dict of weight tensors (`from_weights`) and runs one portion of one sequence:
`forward(h, ctx)` with h [T, width] in the model's activation dtype.  Products go through torch (cuBLAS), as the
dense linears of the package's LLaMA do; everything else is a kernel of libb200seq.  What a mixer carries between
tokens is declared by `state_specs()` and lives in a `SequenceStatePool`.  CUDA only; no CPU fallback."""
import ctypes as C
import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

from . import _seqlib as S
from .state import StateSpec


class StepContext:
    """One portion of one sequence: T tokens, the device pair {slot, first position} and the slot pool's tensors."""

    def __init__(self, T: int, meta: torch.Tensor, state: Dict[str, torch.Tensor], dtype: torch.dtype) -> None:
        self.T, self.meta, self.state, self.dtype = T, meta, state, dtype
        self.act = S.act_code(dtype)

    @property
    def stream(self) -> int:
        """The current CUDA stream at the time of each launch (the capturing stream while a graph is recorded)."""
        return S.stream_ptr()


def _p(t: Optional[torch.Tensor], offset: int = 0) -> Optional[int]:
    """Device address of element `offset` of a tensor's storage view."""
    if t is None:
        return None
    return S.ptr(t) + offset * t.element_size()


def pad8(n: int) -> int:
    return (n + 7) // 8 * 8


def stack_rows(parts: List[torch.Tensor]) -> Tuple[torch.Tensor, List[int]]:
    """Linear weights that read the same input, stacked into one [sum, in] matrix.  Every part starts at a multiple
    of 8 rows (zero rows between), so each part's columns of the product start 16-byte aligned.  Returns the matrix
    and the first row of every part."""
    offs, rows, at = [], [], 0
    for w in parts:
        offs.append(at)
        rows.append(w)
        gap = pad8(w.shape[0]) - w.shape[0]
        if gap:
            rows.append(w.new_zeros((gap,) + tuple(w.shape[1:])))
        at += pad8(w.shape[0])
    return torch.cat(rows, dim=0).contiguous(), offs


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return F.linear(x, w)


# ------------------------------------------------------------------------------------------------ feed-forward
class GatedMLP:
    ACTS = {"gelu_tanh": S.ACT_GELU_TANH, "silu": S.ACT_SILU}

    def __init__(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, act: str = "gelu_tanh") -> None:
        self.ff = gate.shape[0]
        self.w_in = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = down.contiguous()
        self.act = self.ACTS[act]

    def state_specs(self) -> Dict[str, StateSpec]:
        return {}

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        gu = linear(h, self.w_in)
        mid = torch.empty((ctx.T, self.ff), dtype=h.dtype, device=h.device)
        S.check(S.lib().b2l_seq_gated_act(_p(gu), 2 * self.ff, _p(mid), ctx.T, self.ff, self.act, ctx.act, ctx.stream), "b2l_seq_gated_act")
        return linear(mid, self.w_down)


# ------------------------------------------------------------------------------------------------ recurrences
def _scan(ctx: StepContext, *, q, ldq, k, ldk, v, ldv, q_mult, decay, ldd, per_channel, state, out, ldo, heads, qk_heads,
          K, V, beta=None, ldb=0, vscale=None, ldvs=0, skip=None) -> None:
    lib = S.lib()
    n_chunks = lib.b2l_seq_scan_chunks(ctx.T, int(beta is not None))
    ws = wd = None
    if n_chunks > 1:      # long portion, no delta rule: chunks in parallel (local states, combine, outputs)
        ws = torch.empty((n_chunks, heads, V, K), dtype=torch.float32, device=state.device)
        wd = torch.empty((n_chunks, heads, K if per_channel else 1), dtype=torch.float32, device=state.device)
    a = S.ScanArgs(q=q, ldq=ldq, k=k, ldk=ldk, v=v, ldv=ldv, q_mult=float(q_mult), decay=decay, ldd=ldd,
                   decay_per_channel=int(per_channel), beta=beta, ldb=ldb, delta=int(beta is not None), vscale=vscale, ldvs=ldvs,
                   skip=skip, state=_p(state), meta=_p(ctx.meta), out=out, ldo=ldo, T=ctx.T, heads=heads, qk_heads=qk_heads, K=K, V=V,
                   act_dtype=ctx.act, work_state=_p(ws), work_decay=_p(wd), n_chunks=n_chunks)
    S.check(lib.b2l_seq_scan(C.byref(a), ctx.stream), "b2l_seq_scan")


class ChannelDeltaMixer:
    """Gated delta rule, one decay per head and key channel.

        q, k, v = silu(conv(W h)); q, k unit vectors per head (q times dim^-1/2); beta = sigmoid(W_b h)
        g = exp(-exp(A_log) softplus(W_a2 W_a1 h + dt_bias))              [heads x dim]
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
        y = W_o (o / rms(o) * w_norm * sigmoid(W_g2 W_g1 h))
    State per sequence: S (f32, heads x vdim x dim) and the last taps-1 inputs of the convolutions."""

    def __init__(self, name: str, W: Dict[str, torch.Tensor], p: str, *, heads: int, kv_heads: int, dim: int, vdim: int, conv: int,
                 eps: float, unit_eps: float = 1e-6) -> None:
        self.name, self.H, self.G, self.K, self.V, self.taps, self.eps, self.unit_eps = name, heads, kv_heads, dim, vdim, conv, eps, unit_eps
        parts = [W[p + "q"], W[p + "k"], W[p + "v"], W[p + "b"], W[p + "a1"], W[p + "g1"]]
        self.w_in, (self.o_q, self.o_k, self.o_v, self.o_b, self.o_a1, self.o_g1) = stack_rows(parts)
        self.n_in = self.w_in.shape[0]
        self.rank_a, self.rank_g = W[p + "a1"].shape[0], W[p + "g1"].shape[0]
        self.C = self.o_b                                  # conv channels: q | k | v with their alignment gaps
        self.w_conv, _ = stack_rows([W[p + "q.conv"], W[p + "k.conv"], W[p + "v.conv"]])
        assert self.w_conv.shape == (self.C, conv)
        self.w_a2, self.w_g2 = W[p + "a2"].contiguous(), W[p + "g2"].contiguous()
        self.dt_bias, self.A_log, self.w_norm = W[p + "dt_bias"].contiguous(), W[p + "A_log"].contiguous(), W[p + "norm"].contiguous()
        self.w_o = W[p + "o"].contiguous()

    def state_specs(self) -> Dict[str, StateSpec]:
        return {self.name + ".S": StateSpec((self.H, self.V, self.K), torch.float32),
                self.name + ".conv": StateSpec((self.taps - 1, self.C), self.w_in.dtype)}

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        lib, T, dev = S.lib(), ctx.T, h.device
        proj = linear(h, self.w_in)                                         # [T, n_in]
        a = linear(proj[:, self.o_a1:self.o_a1 + self.rank_a], self.w_a2)    # [T, H*K]
        gate = linear(proj[:, self.o_g1:self.o_g1 + self.rank_g], self.w_g2)  # [T, H*V]
        qkv = torch.empty((T, self.C), dtype=torch.float32, device=dev)
        S.check(lib.b2l_seq_conv_silu(_p(proj), self.n_in, _p(self.w_conv), None, _p(ctx.state[self.name + ".conv"]), _p(ctx.meta),
                                      _p(qkv), self.C, T, self.C, self.taps, ctx.act, ctx.stream), "b2l_seq_conv_silu")
        S.check(lib.b2l_seq_unit_norm(_p(qkv, self.o_q), self.C, T, self.G, self.K, self.unit_eps, self.K ** -0.5, ctx.stream), "b2l_seq_unit_norm")
        S.check(lib.b2l_seq_unit_norm(_p(qkv, self.o_k), self.C, T, self.G, self.K, self.unit_eps, 1.0, ctx.stream), "b2l_seq_unit_norm")
        g = torch.empty((T, self.H * self.K), dtype=torch.float32, device=dev)
        S.check(lib.b2l_seq_decay(_p(a), self.H * self.K, _p(self.dt_bias), _p(self.A_log), S.DECAY_EXP_SOFTPLUS, 0.0, _p(g), None, T,
                                  self.H, self.K, ctx.act, ctx.stream), "b2l_seq_decay")
        o = torch.empty((T, self.H * self.V), dtype=torch.float32, device=dev)
        _scan(ctx, q=_p(qkv, self.o_q), ldq=self.C, k=_p(qkv, self.o_k), ldk=self.C, v=_p(qkv, self.o_v), ldv=self.C,
              q_mult=1.0, decay=_p(g), ldd=self.H * self.K, per_channel=True, beta=_p(proj, self.o_b), ldb=self.n_in,
              state=ctx.state[self.name + ".S"], out=_p(o), ldo=self.H * self.V, heads=self.H, qk_heads=self.G, K=self.K, V=self.V)
        y = torch.empty((T, self.H * self.V), dtype=h.dtype, device=dev)
        S.check(lib.b2l_seq_group_norm_gate(_p(o), self.H * self.V, _p(self.w_norm), 1, _p(gate), self.H * self.V, S.ACT_SIGMOID, 0, self.eps,
                                            1.0, _p(y), self.H * self.V, T, self.H * self.V, self.V, ctx.act, ctx.stream), "b2l_seq_group_norm_gate")
        return linear(y, self.w_o)


class Mamba2Mixer:
    """State-space duality layer.  W_in h = [z | x | B | C | dt]; x | B | C pass a causal convolution (+ bias) and silu;
    dt = softplus(dt + dt_bias); per head S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x; then y silu(z),
    RMS norm in `norm_groups` equal parts, W_o.  State: S (f32, heads x vdim x state) and the convolution's inputs."""

    def __init__(self, name: str, W: Dict[str, torch.Tensor], p: str, *, heads: int, vdim: int, state: int, groups: int, norm_groups: int,
                 conv: int, eps: float) -> None:
        self.name, self.H, self.P, self.N, self.G, self.parts, self.taps, self.eps = name, heads, vdim, state, groups, norm_groups, conv, eps
        self.inner = heads * vdim
        self.C = self.inner + 2 * groups * state
        self.w_in = W[p + "in"].contiguous()
        self.n_in = self.w_in.shape[0]
        assert self.n_in == 2 * self.inner + 2 * groups * state + heads, "mamba2: the input projection does not fit z|x|B|C|dt"
        self.w_conv, self.b_conv = W[p + "conv"].contiguous(), W[p + "conv.b"].contiguous()
        self.dt_bias, self.A_log, self.D = W[p + "dt_bias"].contiguous(), W[p + "A_log"].contiguous(), W[p + "D"].contiguous()
        self.w_norm, self.w_o = W[p + "norm"].contiguous(), W[p + "o"].contiguous()

    def state_specs(self) -> Dict[str, StateSpec]:
        return {self.name + ".S": StateSpec((self.H, self.P, self.N), torch.float32),
                self.name + ".conv": StateSpec((self.taps - 1, self.C), self.w_in.dtype)}

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        lib, T, dev = S.lib(), ctx.T, h.device
        u = linear(h, self.w_in)
        xbc = torch.empty((T, self.C), dtype=torch.float32, device=dev)
        S.check(lib.b2l_seq_conv_silu(_p(u, self.inner), self.n_in, _p(self.w_conv), _p(self.b_conv), _p(ctx.state[self.name + ".conv"]),
                                      _p(ctx.meta), _p(xbc), self.C, T, self.C, self.taps, ctx.act, ctx.stream), "b2l_seq_conv_silu")
        decay = torch.empty((T, self.H), dtype=torch.float32, device=dev)
        dt = torch.empty((T, self.H), dtype=torch.float32, device=dev)
        S.check(lib.b2l_seq_decay(_p(u, self.inner + self.C), self.n_in, _p(self.dt_bias), _p(self.A_log), S.DECAY_EXP_SOFTPLUS, 0.0, _p(decay),
                                  _p(dt), T, self.H, 1, ctx.act, ctx.stream), "b2l_seq_decay")
        y = torch.empty((T, self.inner), dtype=torch.float32, device=dev)
        GN = self.G * self.N
        _scan(ctx, q=_p(xbc, self.inner + GN), ldq=self.C, k=_p(xbc, self.inner), ldk=self.C, v=_p(xbc), ldv=self.C, q_mult=1.0,
              decay=_p(decay), ldd=self.H, per_channel=False, vscale=_p(dt), ldvs=self.H, skip=_p(self.D), state=ctx.state[self.name + ".S"],
              out=_p(y), ldo=self.inner, heads=self.H, qk_heads=self.G, K=self.N, V=self.P)
        out = torch.empty((T, self.inner), dtype=h.dtype, device=dev)
        S.check(lib.b2l_seq_group_norm_gate(_p(y), self.inner, _p(self.w_norm), 0, _p(u), self.n_in, S.ACT_SILU, 1, self.eps, 1.0, _p(out),
                                            self.inner, T, self.inner, self.inner // self.parts, ctx.act, ctx.stream), "b2l_seq_group_norm_gate")
        return linear(out, self.w_o)


# ------------------------------------------------------------------------------------------------ rotation
def rope_frequencies(dims: int, base: float, scaling: Optional[dict]) -> Tuple[torch.Tensor, float]:
    """Per-pair rotation frequencies f_i = base^(-2i/dims), i < dims/2, optionally YaRN-scaled: with
    d(t) = dims ln(original / (2 pi t)) / (2 ln base), lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), dims - 1) and
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) the frequency becomes f_i / factor * ramp_i + f_i (1 - ramp_i),
    and cos / sin are multiplied by 0.1 ln(factor) + 1.  Returns (f32 frequencies on the CPU, multiplier)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    mult = 1.0
    if scaling:
        factor, orig = float(scaling["factor"]), float(scaling["original"])

        def d(t: float) -> float:
            return dims * math.log(orig / (2 * math.pi * t)) / (2 * math.log(float(base)))

        lo = max(math.floor(d(float(scaling["fast"]))), 0)
        hi = min(math.ceil(d(float(scaling["slow"]))), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
        f = f / factor * ramp + f * (1 - ramp)
        mult = 0.1 * math.log(factor) + 1.0
    return f.to(torch.float32), mult


# ------------------------------------------------------------------------------------------------ attention
class BlockSinkAttention:
    """Softmax attention inside blocks of `block` positions (query p sees j <= p with j // block == p // block; block
    None: the whole sequence up to `max_positions`), weights exp(s_j) / (1 + sum exp(s_j)) when `sink`.  As a branch of
    a ParallelMixer it shares the input product: `parts()` lists its projection weights, `run()` consumes columns of
    the shared product and writes its gated heads into a slice of the shared read-out buffer."""

    def __init__(self, name: str, W: Dict[str, torch.Tensor], p: str, *, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                 eps: float, softcap: Optional[float] = None, block: Optional[int] = None, rot: Optional[dict] = None, sink: bool = True,
                 max_positions: int = 0) -> None:
        self.name, self.H, self.G, self.K, self.V, self.scale, self.eps = name, heads, kv_heads, dim, vdim, float(scale), eps
        self.softcap = float(softcap) if softcap else 0.0
        self.block = int(block) if block else int(max_positions)
        if self.block <= 0:
            raise ValueError("attention without a block size needs max_positions")
        self.sink = bool(sink)
        self.w = [W[p + "q"], W[p + "k"], W[p + "v"], W[p + "g"]]
        self.q_norm, self.k_norm = W[p + "q.norm"].contiguous(), W[p + "k.norm"].contiguous()
        self.w_o = W[p + "o"]
        self.rot_dims, self.rot_mult, self.freq = 0, 1.0, None
        if rot:
            self.rot_dims = int(rot["dims"])
            f, self.rot_mult = rope_frequencies(self.rot_dims, float(rot["base"]), rot.get("scaling"))
            self.freq = f.to(self.w_o.device)

    def parts(self) -> List[torch.Tensor]:
        return self.w

    def out_width(self) -> int:
        return self.H * self.V

    def state_specs(self) -> Dict[str, StateSpec]:
        dt = self.w_o.dtype
        return {self.name + ".k": StateSpec((self.block, self.G, self.K), dt, zero_on_acquire=False),
                self.name + ".v": StateSpec((self.block, self.G, self.V), dt, zero_on_acquire=False)}

    def run(self, proj: torch.Tensor, offs: List[int], ctx: StepContext, out: torch.Tensor, out_off: int, out_mult: float) -> None:
        lib, T, dev, ld = S.lib(), ctx.T, proj.device, proj.shape[1]
        o_q, o_k, o_v, o_g = offs
        q = torch.empty((T, self.H * self.K), dtype=torch.float32, device=dev)
        kn = torch.empty((T, self.G * self.K), dtype=proj.dtype, device=dev)
        S.check(lib.b2l_seq_headnorm_rope(_p(proj, o_q), ld, _p(self.q_norm), self.eps, _p(self.freq), self.rot_dims, self.rot_mult, _p(ctx.meta),
                                          _p(q), 1, T, self.H, self.K, ctx.act, ctx.stream), "b2l_seq_headnorm_rope")
        S.check(lib.b2l_seq_headnorm_rope(_p(proj, o_k), ld, _p(self.k_norm), self.eps, _p(self.freq), self.rot_dims, self.rot_mult, _p(ctx.meta),
                                          _p(kn), 0, T, self.G, self.K, ctx.act, ctx.stream), "b2l_seq_headnorm_rope")
        a = S.AttnArgs(q=_p(q), k_new=_p(kn), v_new=_p(proj, o_v), ldv=ld, cache_k=_p(ctx.state[self.name + ".k"]),
                       cache_v=_p(ctx.state[self.name + ".v"]), meta=_p(ctx.meta), gate=_p(proj, o_g), ldg=ld, out=_p(out, out_off),
                       ldo=out.shape[1], scale=self.scale, softcap=self.softcap, out_mult=float(out_mult), has_sink=int(self.sink),
                       block=self.block, T=T, heads=self.H, kv_heads=self.G, K=self.K, V=self.V, act_dtype=ctx.act)
        S.check(lib.b2l_seq_block_attention(C.byref(a), ctx.stream), "b2l_seq_block_attention")


class GatedLinearAttention:
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T (q_t dim^-1/2), alpha = sigmoid(W_a2 W_a1 h + b)^(1/tau);
    read-out: per-head RMS norm (shared weight), times silu(W_g h).  A branch like BlockSinkAttention."""

    def __init__(self, name: str, W: Dict[str, torch.Tensor], p: str, *, heads: int, dim: int, vdim: int, tau: float, eps: float) -> None:
        self.name, self.H, self.K, self.V, self.tau, self.eps = name, heads, dim, vdim, float(tau), eps
        self.w = [W[p + "q"], W[p + "k"], W[p + "v"], W[p + "g"], W[p + "a1"]]
        self.rank = W[p + "a1"].shape[0]
        self.w_a2, self.b_a2 = W[p + "a2"].contiguous(), W[p + "a2.b"].contiguous()
        self.w_norm, self.w_o = W[p + "norm"].contiguous(), W[p + "o"]

    def parts(self) -> List[torch.Tensor]:
        return self.w

    def out_width(self) -> int:
        return self.H * self.V

    def state_specs(self) -> Dict[str, StateSpec]:
        return {self.name + ".S": StateSpec((self.H, self.V, self.K), torch.float32)}

    def run(self, proj: torch.Tensor, offs: List[int], ctx: StepContext, out: torch.Tensor, out_off: int, out_mult: float) -> None:
        lib, T, dev, ld = S.lib(), ctx.T, proj.device, proj.shape[1]
        o_q, o_k, o_v, o_g, o_a1 = offs
        a = linear(proj[:, o_a1:o_a1 + self.rank], self.w_a2)
        n = self.H * self.K
        alpha = torch.empty((T, n), dtype=torch.float32, device=dev)
        S.check(lib.b2l_seq_decay(_p(a), n, _p(self.b_a2), None, S.DECAY_SIGMOID_ROOT, self.tau, _p(alpha), None, T, self.H, self.K, ctx.act,
                                  ctx.stream), "b2l_seq_decay")
        o = torch.empty((T, self.H * self.V), dtype=torch.float32, device=dev)
        nq = o_g - o_q                                   # q | k | v are consecutive columns of the product
        qkv = torch.empty((T, nq), dtype=torch.float32, device=dev)
        S.check(lib.b2l_seq_cast_f32(_p(proj, o_q), ld, _p(qkv), nq, T, nq, ctx.act, ctx.stream), "b2l_seq_cast_f32")
        _scan(ctx, q=_p(qkv), ldq=nq, k=_p(qkv, o_k - o_q), ldk=nq, v=_p(qkv, o_v - o_q), ldv=nq, q_mult=self.K ** -0.5, decay=_p(alpha),
              ldd=n, per_channel=True, state=ctx.state[self.name + ".S"], out=_p(o), ldo=self.H * self.V, heads=self.H, qk_heads=self.H,
              K=self.K, V=self.V)
        S.check(lib.b2l_seq_group_norm_gate(_p(o), self.H * self.V, _p(self.w_norm), 1, _p(proj, o_g), ld, S.ACT_SILU, 0, self.eps, float(out_mult),
                                            _p(out, out_off), out.shape[1], T, self.H * self.V, self.V, ctx.act, ctx.stream),
                "b2l_seq_group_norm_gate")


class ParallelMixer:
    """y = sum_b scale_b * W_o,b branch_b(h): the branches' input projections are one product, and so are their
    output projections (the branches write scale_b * read-out into one buffer that meets [W_o,1 | W_o,2 | ...])."""

    def __init__(self, branches: List[Tuple[object, float]]) -> None:
        self.branches = [b for b, _ in branches]
        self.scales = [float(s) for _, s in branches]
        parts, self.counts = [], []
        for b in self.branches:
            parts += b.parts()
            self.counts.append(len(b.parts()))
        self.w_in, self.offs = stack_rows(parts)
        self.widths = [b.out_width() for b in self.branches]
        self.w_o = torch.cat([b.w_o for b in self.branches], dim=1).contiguous()

    def state_specs(self) -> Dict[str, StateSpec]:
        out: Dict[str, StateSpec] = {}
        for b in self.branches:
            out.update(b.state_specs())
        return out

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        proj = linear(h, self.w_in)
        out = torch.empty((ctx.T, sum(self.widths)), dtype=h.dtype, device=h.device)
        at, col = 0, 0
        for b, n, s, w in zip(self.branches, self.counts, self.scales, self.widths):
            b.run(proj, self.offs[at:at + n], ctx, out, col, s)
            at += n
            col += w
        return linear(out, self.w_o)
