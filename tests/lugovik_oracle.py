"""A plain, slow restatement of the Lugovik design on the CPU: one function per mechanism, token by token where
the design is a recurrence, in whatever float type the inputs have (the tests use float64).  Test
infrastructure only: it shares no code with the package and the package never imports it.

Notation: T tokens, H heads, K key size per head, V value size per head.  Linear weights are [out, in]."""
import math

import torch


# ----------------------------------------------------------------------------- small pieces
def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis (w may be None)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def causal_conv(x, w, bias=None):
    """x [T, C], w [C, taps]: y[t, c] = sum_j w[c, taps-1-j] x[t-j, c] (+ bias), zeros before the first token."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            if t - j >= 0:
                y[t] += w[:, taps - 1 - j] * x[t - j]
    if bias is not None:
        y = y + bias
    return y


def unit(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


# ----------------------------------------------------------------------------- recurrences (one head)
def delta_rule_head(q, k, v, beta, g):
    """q, k, g [T, K]; v [T, V]; beta [T].  S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, K = q.shape
    V = v.shape[1]
    S = torch.zeros(K, V, dtype=q.dtype)
    out = []
    for t in range(T):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.t() @ k[t])
        S = S + torch.outer(k[t], u)
        out.append(S.t() @ q[t])
    return torch.stack(out)


def decayed_outer_head(q, k, v, a):
    """S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  a is [T, K] (per key channel) or [T] (one number)."""
    T, K = q.shape
    S = torch.zeros(K, v.shape[1], dtype=q.dtype)
    out = []
    for t in range(T):
        at = a[t][:, None] if a.dim() == 2 else a[t]
        S = at * S + torch.outer(k[t], v[t])
        out.append(S.t() @ q[t])
    return torch.stack(out)


# ----------------------------------------------------------------------------- rotation
def rope_frequencies(rot):
    """Per-pair frequencies [dims/2] and the factor both cos and sin are multiplied by."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def dim_of(t):
        return dims * math.log(orig / (2 * math.pi * t)) / (2 * math.log(base))

    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
    f = f / factor * ramp + f * (1 - ramp)
    return f, 0.1 * math.log(factor) + 1.0


def rotate(x, pos, rot):
    """x [T, heads, dim]; the first rot.dims entries of every head are rotated, entry i with entry i + dims/2."""
    dims = int(rot["dims"])
    f, m = rope_frequencies(rot)
    ang = pos.to(torch.float64)[:, None] * f[None, :]
    cos, sin = (torch.cos(ang) * m).to(x.dtype)[:, None, :], (torch.sin(ang) * m).to(x.dtype)[:, None, :]
    u, v = x[..., : dims // 2], x[..., dims // 2: dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


# ----------------------------------------------------------------------------- mixers
def chunked_sink_attention(q, k, v, pos, scale, softcap, size):
    """q [T, H, K], k [T, G, K], v [T, G, V].  Query i sees key j <= i of the same block of `size` positions; the
    softmax has one more term in its denominator (score 0, no value)."""
    T, H, K = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if size is None or int(pos[j]) // size == int(pos[i]) // size]
            s = (k[js, g] @ q[i, h]) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            m = torch.clamp(s.max(), min=0.0)
            e = torch.exp(s - m)
            p = e / (torch.exp(-m) + e.sum())
            out[i, h] = p @ v[js, g]
    return out


def left_mixer(h, W, p, c, eps, pos):
    H, G, K, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    T = h.shape[0]
    q = (h @ W[p + "q"].t()).view(T, H, K)
    k = (h @ W[p + "k"].t()).view(T, G, K)
    v = (h @ W[p + "v"].t()).view(T, G, V)
    q = rms_norm(q, W[p + "q.norm"], eps)
    k = rms_norm(k, W[p + "k.norm"], eps)
    if c.get("rot"):
        q, k = rotate(q, pos, c["rot"]), rotate(k, pos, c["rot"])
    size = c["mask"]["size"] if c.get("mask") else None
    o = chunked_sink_attention(q, k, v, pos, float(c["scale"]), c.get("softcap"), size)
    gate = torch.sigmoid(h @ W[p + "g"].t())            # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * V) @ W[p + "o"].t()


def right_mixer(h, W, p, c, eps):
    H, K, V = c["heads"], c["dim"], c["vdim"]
    T = h.shape[0]
    q = (h @ W[p + "q"].t()).view(T, H, K) * K ** -0.5
    k = (h @ W[p + "k"].t()).view(T, H, K)
    v = (h @ W[p + "v"].t()).view(T, H, V)
    z = (h @ W[p + "a1"].t()) @ W[p + "a2"].t() + W[p + "a2.b"]
    alpha = (torch.sigmoid(z) ** (1.0 / float(c["tau"]))).view(T, H, K)
    o = torch.stack([decayed_outer_head(q[:, i], k[:, i], v[:, i], alpha[:, i]) for i in range(H)], dim=1)
    o = rms_norm(o, W[p + "norm"], eps).reshape(T, H * V)
    o = o * silu(h @ W[p + "g"].t())
    return o @ W[p + "o"].t()


def parallel_mixer(h, W, p, c, eps, pos):
    return float(c["left_scale"]) * left_mixer(h, W, p + "left.", c["left"], eps, pos) + \
        float(c["right_scale"]) * right_mixer(h, W, p + "right.", c["right"], eps)


def channel_delta_mixer(h, W, p, c, eps):
    H, G, K, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ W[p + "q"].t(), W[p + "q.conv"])).view(T, G, K)
    k = silu(causal_conv(h @ W[p + "k"].t(), W[p + "k.conv"])).view(T, G, K)
    v = silu(causal_conv(h @ W[p + "v"].t(), W[p + "v.conv"])).view(T, H, V)
    q = unit(q) * K ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ W[p + "b"].t())             # [T, H]
    a = ((h @ W[p + "a1"].t()) @ W[p + "a2"].t() + W[p + "dt_bias"]).view(T, H, K)
    g = torch.exp(-torch.exp(W[p + "A_log"])[None, :, None] * softplus(a))
    outs = []
    for i in range(H):
        j = i // (H // G)
        outs.append(delta_rule_head(q[:, j], k[:, j], v[:, i], beta[:, i], g[:, i]))
    o = torch.stack(outs, dim=1)                          # [T, H, V]
    gate = torch.sigmoid((h @ W[p + "g1"].t()) @ W[p + "g2"].t()).view(T, H, V)
    o = rms_norm(o, W[p + "norm"], eps) * gate
    return o.reshape(T, H * V) @ W[p + "o"].t()


def mamba2_mixer(h, W, p, c, eps):
    H, P, N, G = c["heads"], c["vdim"], c["state"], c["groups"]
    inner = H * P
    T = h.shape[0]
    u = h @ W[p + "in"].t()
    z, xbc, dt = u[:, :inner], u[:, inner: 2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner: inner + G * N].view(T, G, N)
    Cm = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + W[p + "dt_bias"])                  # [T, H]
    decay = torch.exp(-torch.exp(W[p + "A_log"])[None, :] * dt)
    ys = []
    for i in range(H):
        g = i // (H // G)
        y = decayed_outer_head(Cm[:, g], B[:, g], dt[:, i, None] * x[:, i], decay[:, i])
        ys.append(y + W[p + "D"][i] * x[:, i])
    y = torch.stack(ys, dim=1).reshape(T, inner) * silu(z)
    parts = int(c["norm_groups"])
    y = rms_norm(y.view(T, parts, inner // parts), None, eps).reshape(T, inner) * W[p + "norm"]
    return y @ W[p + "o"].t()


def feed_forward(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].t()) * (h @ W[p + "up"].t())) @ W[p + "down"].t()


# ----------------------------------------------------------------------------- the model
def forward(config, W, tokens, return_layers=False):
    """tokens: a list of ids for one sequence from position 0.  Returns logits [T, vocab] (and the residual
    stream after every layer)."""
    eps = float(config["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(tokens.numel())
    x = W["embed"][tokens] * float(config["embedding"]["scale"])
    layers = []
    for i, layer in enumerate(config["layers"]):
        p = "l%d." % i
        h = rms_norm(x, W[p + "norm1"], eps)
        kind, c = layer["type"], layer["mixer"]
        if kind == "channel_delta":
            y = channel_delta_mixer(h, W, p + "mix.", c, eps)
        elif kind == "parallel":
            y = parallel_mixer(h, W, p + "mix.", c, eps, pos)
        elif kind == "mamba2":
            y = mamba2_mixer(h, W, p + "mix.", c, eps)
        else:
            raise ValueError(kind)
        x = x + rms_norm(y, W[p + "norm1b"], eps)
        if layer.get("mlp"):
            y = feed_forward(rms_norm(x, W[p + "norm2"], eps), W, p + "mlp.")
            x = x + rms_norm(y, W[p + "norm2b"], eps)
        layers.append(x)
    logits = rms_norm(x, W["final.norm"], eps) @ W["head"].t()
    return (logits, torch.stack(layers)) if return_layers else logits


# ----------------------------------------------------------------------------- random models for the tests
def tensor_shapes(config):
    """Name -> shape of every tensor a model of this configuration has."""
    D, out = int(config["width"]), {}
    out["embed"] = (config["vocab"], D)
    for i, layer in enumerate(config["layers"]):
        p, c = "l%d." % i, layer["mixer"]
        out[p + "norm1"] = out[p + "norm1b"] = (D,)
        m = p + "mix."
        if layer["type"] == "channel_delta":
            H, G, K, V, r = c["heads"], c["kv_heads"], c["dim"], c["vdim"], c.get("rank", 8)
            for n, ch in (("q", G * K), ("k", G * K), ("v", H * V)):
                out[m + n] = (ch, D)
                out[m + n + ".conv"] = (ch, c["conv"])
            out[m + "b"], out[m + "A_log"], out[m + "norm"] = (H, D), (H,), (V,)
            out[m + "a1"], out[m + "a2"], out[m + "dt_bias"] = (r, D), (H * K, r), (H * K,)
            out[m + "g1"], out[m + "g2"], out[m + "o"] = (r, D), (H * V, r), (D, H * V)
        elif layer["type"] == "parallel":
            a, b = c["left"], c["right"]
            H, G, K, V = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            out[m + "left.q"], out[m + "left.k"], out[m + "left.v"] = (H * K, D), (G * K, D), (G * V, D)
            out[m + "left.q.norm"] = out[m + "left.k.norm"] = (K,)
            out[m + "left.g"], out[m + "left.o"] = (H, D), (D, H * V)
            H, K, V, r = b["heads"], b["dim"], b["vdim"], b.get("rank", 8)
            out[m + "right.q"] = out[m + "right.k"] = (H * K, D)
            out[m + "right.v"] = out[m + "right.g"] = (H * V, D)
            out[m + "right.o"], out[m + "right.norm"] = (D, H * V), (V,)
            out[m + "right.a1"], out[m + "right.a2"], out[m + "right.a2.b"] = (r, D), (H * K, r), (H * K,)
        elif layer["type"] == "mamba2":
            H, P, N, G = c["heads"], c["vdim"], c["state"], c["groups"]
            ch = H * P + 2 * G * N
            out[m + "in"], out[m + "conv"], out[m + "conv.b"] = (2 * H * P + 2 * G * N + H, D), (ch, c["conv"]), (ch,)
            out[m + "dt_bias"] = out[m + "A_log"] = out[m + "D"] = (H,)
            out[m + "norm"], out[m + "o"] = (H * P,), (D, H * P)
        if layer.get("mlp"):
            out[p + "norm2"] = out[p + "norm2b"] = (D,)
            F = layer["mlp"]["ff"]
            out[p + "mlp.gate"] = out[p + "mlp.up"] = (F, D)
            out[p + "mlp.down"] = (D, F)
    out["final.norm"], out["head"] = (D,), (config["vocab"], D)
    return out


def random_weights(config, seed=0, dtype=torch.bfloat16):
    """Random tensors of the right shapes, scaled so that activations stay of order one and the recurrences neither
    die nor blow up.  The low-rank sizes come from config['layers'][i]['mixer'].get('rank', 8)."""
    gen = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if name.endswith(".conv"):
            t = torch.randn(shape, generator=gen) * 0.5
        elif leaf in ("norm1", "norm2", "norm1b", "norm2b", "norm") or name == "final.norm":
            t = 1.0 + 0.2 * torch.randn(shape, generator=gen)
            if leaf in ("norm1b", "norm2b"):
                t = t * 0.5
        elif leaf == "A_log":
            t = torch.rand(shape, generator=gen) * 1.5 - 1.0
        elif leaf in ("dt_bias", "D", "b") and len(shape) == 1:
            t = torch.randn(shape, generator=gen) * 0.5
        elif name == "embed":
            t = torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[-1])
        W[name] = t.to(dtype)
    return W
