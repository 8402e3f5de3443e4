"""A plain, slow implementation of the Fazinex decoder, for comparison only.

Whole sequences, no cache, no batching, one function per mechanism, PyTorch on
the CPU in float64 (or float32).  It shares no code with ``freetoken_b200``: it
takes a config dictionary and a ``{name: tensor}`` state and is written from the
design's equations.

The design, in this file's notation (``x`` is the residual stream ``[T, W]``):

* ``x0 = rms(E[tokens]) * g_embed``.
* a layer is parallel: ``h = rms(x) * g1;  x <- x + (mix(h) + ff(h))``; a layer
  without feed-forward adds the mixer only.
* ``rms(v) = v / sqrt(mean(v^2) + eps)``.
* mixer ``attention``: ``q = Wq h`` per head, ``k = Wk h`` per key head, the values
  ARE the keys; query at position ``p`` is multiplied by
  ``1 + coef * ln(floor((p + 1) / every) + 1)``; causal softmax of
  ``q.k * scale``; ``Wo`` on the concatenated heads.
* mixer ``latent_attention``: ``c = rms(Wdkv h) * g_c`` (the only thing a cache
  would keep), per head ``k = Wuk c``, ``v = Wuv c``; causal softmax of
  ``q.k * scale``; head ``i`` is multiplied by ``sigmoid(Wg h)_i``; ``Wo``.
* feed-forward: ``Wdown relu(Wup h)^2``.
* layers ``start .. stop-1`` run ``times`` times in a row, then the rest.
* ``logits = cap * tanh((E rms(x) * g_final) / cap)``.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt(v.pow(2).mean(dim=-1, keepdim=True) + eps)


def rms_norm(v: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(v, eps) * g


def query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    """``1 + coef * ln(floor((p + 1) / every) + 1)`` per position."""
    steps = torch.div(positions + 1, every, rounding_mode="floor")
    return 1.0 + coef * torch.log(steps.to(torch.float64) + 1.0)


def causal_softmax(scores: torch.Tensor) -> torch.Tensor:
    """``scores[..., i, j]``: query i sees keys j <= i."""
    T = scores.shape[-1]
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    return torch.softmax(scores.masked_fill(~mask, float("-inf")), dim=-1)


def shared_kv_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict) -> torch.Tensor:
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ w["q"].T).view(T, H, d)
    k = (h @ w["k"].T).view(T, G, d)
    qt = m.get("q_temp")
    if qt:
        temp = query_temperature(torch.arange(T), float(qt["coef"]), int(qt["every"])).to(h.dtype)
        q = q * temp[:, None, None]
    out = torch.empty(T, H, d, dtype=h.dtype)
    for i in range(H):
        kk = k[:, i // (H // G)]
        p = causal_softmax((q[:, i] @ kk.T) * float(m["scale"]))
        out[:, i] = p @ kk                       # the values are the keys
    return out.reshape(T, H * d) @ w["o"].T


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w["q"].T).view(T, H, d)
    c = rms_norm(h @ w["dkv"].T, w["dkv.norm"], eps)
    k = (c @ w["uk"].T).view(T, H, d)
    v = (c @ w["uv"].T).view(T, H, dv)
    gate = torch.sigmoid(h @ w["g"].T)           # [T, H]
    out = torch.empty(T, H, dv, dtype=h.dtype)
    for i in range(H):
        p = causal_softmax((q[:, i] @ k[:, i].T) * float(m["scale"]))
        out[:, i] = (p @ v[:, i]) * gate[:, i:i + 1]
    return out.reshape(T, H * dv) @ w["o"].T


def relu_squared_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    return torch.relu(h @ w["up"].T).pow(2) @ w["down"].T


def layer_order(config: dict) -> List[int]:
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def _sub(state: Dict[str, torch.Tensor], prefix: str, dtype) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(dtype) for k, v in state.items() if k.startswith(prefix)}


def forward(config: dict, state: Dict[str, torch.Tensor], tokens, dtype=torch.float64,
            layer_outputs: Optional[list] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one whole sequence; ``layer_outputs`` (a list) gets
    the residual stream after every layer run."""
    eps = float(config["norm"]["eps"])
    E = state["embed"].to(dtype)
    x = rms_norm(E[torch.as_tensor(tokens, dtype=torch.long)], state["embed.norm"].to(dtype), eps)
    for li in layer_order(config):
        spec = config["layers"][li]
        h = rms_norm(x, state[f"l{li}.norm1"].to(dtype), eps)
        mix = _sub(state, f"l{li}.mix.", dtype)
        if spec["type"] == "attention":
            y = shared_kv_attention(h, mix, spec["mixer"])
        elif spec["type"] == "latent_attention":
            y = latent_attention(h, mix, spec["mixer"], eps)
        else:
            raise ValueError(spec["type"])
        if spec.get("mlp"):
            y = y + relu_squared_mlp(h, _sub(state, f"l{li}.mlp.", dtype))
        x = x + y
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    logits = rms_norm(x, state["final.norm"].to(dtype), eps) @ E.T
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits


# ------------------------------------------------------------ random models
def random_state(config: dict, seed: int, std: float = 0.05) -> Dict[str, torch.Tensor]:
    """bfloat16 weights ~N(0, std^2) (norm weights around 1) for ``config``."""
    g = torch.Generator().manual_seed(seed)
    W = int(config["width"])

    def mat(*shape, s=std):
        return (torch.randn(*shape, generator=g) * s).to(torch.bfloat16)

    def gain(n):
        return (1.0 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16)

    st = {"embed": mat(int(config["vocab"]), W, s=1.0), "embed.norm": gain(W), "final.norm": gain(W)}
    for i, spec in enumerate(config["layers"]):
        m = spec["mixer"]
        p = f"l{i}."
        st[p + "norm1"] = gain(W)
        H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
        s_in = 1.0 / math.sqrt(W)
        st[p + "mix.q"] = mat(H * d, W, s=s_in)
        if spec["type"] == "attention":
            st[p + "mix.k"] = mat(int(m["kv_heads"]) * d, W, s=s_in)
            st[p + "mix.o"] = mat(W, H * d, s=1.0 / math.sqrt(H * d))
        else:
            R = int(m["kv_rank"])
            st[p + "mix.dkv"] = mat(R, W, s=s_in)
            st[p + "mix.dkv.norm"] = gain(R)
            st[p + "mix.uk"] = mat(H * d, R, s=1.0 / math.sqrt(R))
            st[p + "mix.uv"] = mat(H * dv, R, s=1.0 / math.sqrt(R))
            st[p + "mix.g"] = mat(H, W, s=2.0 * s_in)
            st[p + "mix.o"] = mat(W, H * dv, s=1.0 / math.sqrt(H * dv))
        if spec.get("mlp"):
            F = int(spec["mlp"]["ff"])
            st[p + "mlp.up"] = mat(F, W, s=s_in)
            st[p + "mlp.down"] = mat(W, F, s=1.0 / math.sqrt(F))
    return st
