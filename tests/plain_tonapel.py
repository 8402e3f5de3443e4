"""A plain, slow implementation of the Tonapel decoder: one function per mechanism.

Everything is a loop or a dense tensor expression over a whole sequence in the
working precision of the weights handed in (the tests use float64); there is no
cache, no state object and no batching, and nothing here is shared with the
engine's code.  Notation: ``x`` the residual stream ``[T, W]``, ``h`` a
sublayer's input, ``rms(v) = v / sqrt(mean(v^2) + eps)``.

* layer:   ``x += m * n1b(mixer(n1(x)))``, then ``x += m * n2b(ff(n2(x)))``;
  every norm is ``rms(v) * (1 + w)``.
* ``parallel`` mixer: ``a_l * window_attention(h) + a_r * ssd(h)``.
* ``delta`` mixer: the gated delta rule.
* feed-forward: gated dense (tanh-GELU), or routed experts with a clamped
  gate/up pair.
"""

import math

import torch


def rms(v, eps):
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def norm(v, w, eps):
    return rms(v, eps) * (1.0 + w)


def silu(v):
    return v * torch.sigmoid(v)


def softplus(v):
    return torch.where(v > 30, v, torch.log1p(torch.exp(torch.clamp(v, max=30.0))))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate(v, base, dims):
    """``v`` ``[T, heads, dim]`` at positions 0..T-1: the first ``dims`` dimensions of each
    head turn, dimension i paired with i + dims/2, by the angle p * base^(-2i/dims)."""
    T = v.shape[0]
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    angle = torch.arange(T, dtype=torch.float64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    cos, sin = angle.cos().to(v.dtype)[:, None, :], angle.sin().to(v.dtype)[:, None, :]
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, v[..., dims:]], dim=-1)


def causal_conv(u, w, bias=None):
    """``u`` ``[T, C]``, ``w`` ``[C, taps]`` whose last column weighs the current token;
    zeros stand before the sequence."""
    T, C = u.shape
    taps = w.shape[1]
    out = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += w[:, j] * u[s]
    if bias is not None:
        out = out + bias
    return out


def window_attention(h, p, W, c):
    """Left half of the parallel mixer: biased projections, partial rotation, a softmax over
    the token itself and the ``mask.size - 1`` tokens before it."""
    T = h.shape[0]
    H, G, D, DV = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, D)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, DV)
    q = rotate(q, c["rot"]["base"], c["rot"]["dims"])
    k = rotate(k, c["rot"]["base"], c["rot"]["dims"])
    size = c["mask"]["size"]
    out = torch.zeros(T, H, DV, dtype=h.dtype)
    for i in range(T):
        lo = max(0, i - size + 1)
        for head in range(H):
            g = head // (H // G)
            s = (k[lo:i + 1, g] @ q[i, head]) * c["scale"]
            w = torch.softmax(s, 0)
            out[i, head] = w @ v[lo:i + 1, g]
    return out.reshape(T, H * DV) @ W[p + "o"].T + W[p + "o.b"]


def ssd_recurrence(x, B, C, dt, dt_bias, A_log, D, S=None):
    """``x`` ``[T, heads, P]``, ``B``/``C`` ``[T, groups, N]``, ``dt`` ``[T, heads]`` (before its bias and
    softplus); the state ``S`` ``[heads, N, P]`` starts at zero and is returned updated in place."""
    T, Hh, P = x.shape
    G, N = B.shape[1], B.shape[2]
    dt = softplus(dt + dt_bias)
    A = -torch.exp(A_log)
    y = torch.zeros(T, Hh, P, dtype=x.dtype)
    S = torch.zeros(Hh, N, P, dtype=x.dtype) if S is None else S
    for t in range(T):
        for head in range(Hh):
            g = head // (Hh // G)
            S[head] = torch.exp(A[head] * dt[t, head]) * S[head] + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S[head].T @ C[t, g] + D[head] * x[t, head]
    return y


def ssd(h, p, W, c, eps):
    """Right half: a selective state space of one decay per head."""
    T = h.shape[0]
    Hh, P, N, G = c["heads"], c["vdim"], c["state"], c["groups"]
    inner = Hh * P
    zxbcdt = h @ W[p + "in"].T
    z, xbc, dt = zxbcdt[:, :inner], zxbcdt[:, inner:2 * inner + 2 * G * N], zxbcdt[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].view(T, Hh, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    y = ssd_recurrence(x, B, C, dt, W[p + "dt_bias"], W[p + "A_log"], W[p + "D"])
    y = y.reshape(T, inner) * silu(z)
    parts = c["norm_groups"]
    y = rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * W[p + "norm"]
    return y @ W[p + "o"].T


def parallel_mixer(h, p, W, c, eps):
    return (c["left_scale"] * window_attention(h, p + "left.", W, c["left"])
            + c["right_scale"] * ssd(h, p + "right.", W, c["right"], eps))


def delta_recurrence(q, k, v, beta, decay, dt_bias, A_log, S=None, unit_eps=1e-6):
    """``q``/``k`` ``[T, key heads, D]`` and ``v`` ``[T, heads, P]`` after their convolutions; ``beta`` and
    ``decay`` ``[T, heads]`` as projected.  The state ``S`` ``[heads, D, P]`` starts at zero."""
    T, Hh, DV = v.shape
    G, D = q.shape[1], q.shape[2]
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + unit_eps) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
    beta = torch.sigmoid(beta)
    g = torch.exp(-torch.exp(A_log) * softplus(decay + dt_bias))
    o = torch.zeros(T, Hh, DV, dtype=v.dtype)
    S = torch.zeros(Hh, D, DV, dtype=v.dtype) if S is None else S
    for t in range(T):
        for head in range(Hh):
            kv = head // (Hh // G)
            S[head] = g[t, head] * S[head]
            u = beta[t, head] * (v[t, head] - S[head].T @ k[t, kv])
            S[head] = S[head] + torch.outer(k[t, kv], u)
            o[t, head] = S[head].T @ q[t, kv]
    return o


def delta_mixer(h, p, W, c, eps):
    """Gated delta rule: the state forgets by g, then is corrected toward v along k."""
    T = h.shape[0]
    Hh, G, D, DV = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).view(T, G, D)
    k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).view(T, G, D)
    v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).view(T, Hh, DV)
    o = delta_recurrence(q, k, v, h @ W[p + "b"].T, h @ W[p + "a"].T, W[p + "dt_bias"], W[p + "A_log"])
    o = rms(o, eps) * W[p + "norm"] * silu(h @ W[p + "g"].T).view(T, Hh, DV)
    return o.reshape(T, Hh * DV) @ W[p + "o"].T


def dense_ff(h, p, W):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def route(h, p, W, c):
    """``(ids [T, top], weights [T, top])``: the largest logits, softmax over those alone."""
    z = (h @ W[p + "router"].T)
    top = torch.topk(z, c["router"]["top"], dim=-1)
    return top.indices, torch.softmax(top.values, -1)


def expert(h, p, W, limit):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def route_margin(h, p, W, c):
    """Per token: how far the last chosen logit lies above the first one not chosen (inf when all
    experts are chosen)."""
    z = h @ W[p + "router"].T
    top = c["router"]["top"]
    if top >= z.shape[1]:
        return torch.full((z.shape[0],), float("inf"), dtype=z.dtype)
    best = torch.topk(z, top + 1, dim=-1).values
    return best[:, top - 1] - best[:, top]


def moe_ff(h, p, W, c, ids=None):
    own_ids, _ = route(h, p, W, c)
    ids = own_ids if ids is None else ids
    z = h @ W[p + "router"].T
    weights = torch.softmax(torch.gather(z, 1, ids), -1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            out[t] += weights[t, j] * expert(h[t:t + 1], f"{p}e{e}.", W, c["expert"]["limit"])[0]
    return out


def forward(cfg, W, tokens, layer_dump=None, expert_ids=None, margins=None):
    """Logits ``[T, vocab]`` of one sequence; ``layer_dump`` collects the residual stream after
    every layer; ``expert_ids`` (per routed layer, ``[T, top]``) replaces the router's own choice;
    ``margins`` collects every routed layer's :func:`route_margin`."""
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    routed = 0
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm(x, W[p + "norm1"], eps)
        if layer["type"] == "parallel":
            a = parallel_mixer(h, p + "mix.", W, layer["mixer"], eps)
        elif layer["type"] == "delta":
            a = delta_mixer(h, p + "mix.", W, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + m * norm(a, W[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp:
            h = norm(x, W[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                f = dense_ff(h, p + "mlp.", W)
            else:
                ids = None if expert_ids is None else expert_ids[routed]
                routed += 1
                if margins is not None:
                    margins.append(route_margin(h, p + "mlp.", W, mlp))
                f = moe_ff(h, p + "mlp.", W, mlp, ids)
            x = x + m * norm(f, W[p + "norm2b"], eps)
        if layer_dump is not None:
            layer_dump.append(x.clone())
    return norm(x, W["final.norm"], eps) @ W["head"].T
