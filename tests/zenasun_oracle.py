"""A plain float64 restatement of the Zenasun design, one function per mechanism, whole sequences at once where
that is the plainest form and token by token where the mechanism is a recurrence.  It shares no code with the
package: torch on the CPU only.  Weights are a dict name -> tensor; configurations are the dicts of config.json."""
import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    return rms_unit(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def rotate(x, positions, dims, base, interleaved):
    """x [T, n]: the first `dims` entries rotated by positions [T]; pairs (2i, 2i+1) or (i, i + dims/2)."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        f = float(base) ** (-2.0 * i / dims)
        a = positions.to(F64) * f
        c, s = torch.cos(a), torch.sin(a)
        iu, iv = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
        u, v = x[:, iu], x[:, iv]
        out[:, iu] = u * c - v * s
        out[:, iv] = v * c + u * s
    return out


def latent_attention(h, W, p, m, eps, pos0=0):
    """h [T, width] -> [T, width].  Keys and values are expanded from the latent for every position (the plain form)."""
    T = h.shape[0]
    H, dn, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(pos0, pos0 + T)
    cq = rms_unit(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).view(T, H, dn + dr)
    kv = h @ W[p + "dkv"].T
    c = rms_unit(kv[:, :rk], eps) * W[p + "dkv.norm"]
    k_rot = rotate(kv[:, rk:], pos, m["rot"]["dims"], m["rot"]["base"], True)
    k_nope = (c @ W[p + "uk"].T).view(T, H, dn)
    v = (c @ W[p + "uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        q_rot = rotate(q[:, hd, dn:], pos, m["rot"]["dims"], m["rot"]["base"], True)
        s = (q[:, hd, :dn] @ k_nope[:, hd].T + q_rot @ k_rot.T) * m["scale"]
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), -math.inf)
        sink = W[p + "sink"][hd]
        mx = torch.maximum(s.max(dim=-1, keepdim=True).values, sink)
        e = torch.exp(s - mx)
        wgt = e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink - mx))
        out[:, hd] = wgt @ v[:, hd]
    return out.reshape(T, H * dv) @ W[p + "o"].T


def retention(h, W, p, m, eps, state=None, pos0=0):
    """Token by token.  state [H, dim, vdim] (None = zeros); returns (y [T, width], state)."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(pos0, pos0 + T)
    q = (h @ W[p + "q"].T).view(T, H, dk)
    k = (h @ W[p + "k"].T).view(T, H, dk)
    v = (h @ W[p + "v"].T).view(T, H, dv)
    g = silu(h @ W[p + "g"].T)
    S = torch.zeros(H, dk, dv, dtype=F64) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        qh = rotate(q[:, hd], pos, m["rot"]["dims"], m["rot"]["base"], False)
        kh = rotate(k[:, hd], pos, m["rot"]["dims"], m["rot"]["base"], False) * dk ** -0.5
        for t in range(T):
            S[hd] = m["decay"][hd] * S[hd] + torch.outer(kh[t], v[t, hd])
            o[t, hd] = S[hd].T @ qh[t]
    o = rms_unit(o, eps).reshape(T, H * dv)
    return (o * g) @ W[p + "o"].T, S


def route(h, W, p, r):
    """Chosen experts [T, top] and their weights [T, top]; experts >= r['experts'] are identities."""
    n = r["experts"] + r.get("identity", 0)
    s = torch.softmax(h @ W[p + "router"].T, dim=-1)
    choice = s + W[p + "correction"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    per = n // groups["count"]
    gscore = choice.view(-1, groups["count"], per).max(dim=-1).values
    kept = gscore.topk(groups["keep"], dim=-1).indices
    allowed = torch.zeros_like(gscore, dtype=torch.bool).scatter_(1, kept, True).repeat_interleave(per, dim=1)
    idx = choice.masked_fill(~allowed, -math.inf).topk(r["top"], dim=-1).indices
    w = s.gather(1, idx)
    return idx, w / (w.sum(dim=-1, keepdim=True) + 1e-20)


def moe(h, W, p, mlp):
    r = mlp["router"]
    idx, w = route(h, W, p, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), w[t]):
            if e >= r["experts"]:
                out[t] += a * h[t]
            else:
                q = f"{p}e{e}."
                out[t] += a * ((silu(h[t] @ W[q + "gate"].T) * (h[t] @ W[q + "up"].T)) @ W[q + "down"].T)
    return out


def model(tokens, config, weights, capture=None):
    """tokens: list of ints, one whole sequence from position 0.  Returns logits [T, vocab] in float64."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)] * config["embedding"]["scale"]
    for i, layer in enumerate(config["layers"]):
        j = layer.get("weights_of")
        p = "l%d." % (i if j is None else j)
        h1 = norm_around_zero(x, W[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            y = latent_attention(h1, W, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "retention":
            y, _ = retention(h1, W, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp"):
            y = y + moe(norm_around_zero(x, W[p + "norm2"], eps), W, p + "mlp.", layer["mlp"])
        x = x + y
        if capture is not None:
            capture.append(x.clone())
    z = norm_around_zero(x, W["final.norm"], eps) @ W["embed"].T
    cap = config.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z
