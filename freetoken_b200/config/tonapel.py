"""Typed configuration of the Tonapel decoder, read from ``config.json``.

A Tonapel model is a list of *sandwich* layers: every sublayer is normed before and
after, and its normed output joins the residual stream times ``residual_mult``::

    x <- x + m * n1b(mixer(n1(x)));   x <- x + m * n2b(ff(n2(x)))      (every norm rms(v) * (1 + w))

with one of two mixers per layer:

* ``parallel``: the weighted sum of two mixers that read the same rows - sliding-window
  grouped-query attention (biased projections, rotation of the first ``rot.dims`` dimensions of
  each head in halves, value heads of a size of their own) and a selective state space with
  one decay per head (Mamba-2's recurrence behind a short convolution, gated, then RMS-normed
  in ``norm_groups`` parts);
* ``delta``: the gated delta rule behind short convolutions on q, k and v, unit-norm q and k,
  a per-head RMS norm and a SiLU gate on the read-out;

and a feed-forward that is dense and gated (tanh-GELU), a set of routed experts (the ``top``
largest router logits, softmax over those alone; gate and up clamped by ``limit``) or absent.

config.json keys: ``architecture`` (``"Tonapel"``), ``vocab``, ``width``, ``norm.eps``,
``residual_mult`` and ``layers[i]`` with ``type``, ``mixer`` and ``mlp`` (``null``: none).
Mixer keys - parallel: ``left.{heads, kv_heads, dim, vdim, scale, mask.size, rot.{base, dims}}``,
``right.{heads, vdim, state, groups, conv, norm_groups}``, ``left_scale``, ``right_scale``;
delta: ``heads, kv_heads, dim, vdim, conv``.  mlp keys: ``kind`` (``dense``: ``ff``; ``moe``:
``expert.{ff, limit}``, ``router.{experts, top}``).  Tensors: ``embed``, ``final.norm``, ``head``
and ``l<i>.{norm1, norm1b, norm2, norm2b, mix.*, mlp.*}``.  Every size and constant is handed
to a part as a parameter by :func:`build_plan`.  The reference has no model of this design;
the module follows the shape of python/freetoken/models/minimax_m3/args.py:135-254.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .model_plan import ConfigError, LayerSpec, ModelPlan, PartSpec, RunEntry

ARCHITECTURE = "Tonapel"
MIXER_TYPES = ("parallel", "delta")
MLP_KINDS = ("dense", "moe")
# constants the design fixes
EXPERT_GATE_ALPHA = 1.702        # g * sigmoid(alpha * g) in an expert
UNIT_NORM_EPS = 1e-6             # under the root of the delta rule's unit norms
NO_POSITION_LIMIT = 1 << 30      # rotation angles are computed, not tabulated by the design


@dataclass(frozen=True)
class WindowAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class StateSpace:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class ParallelMixer:
    left: WindowAttention
    right: StateSpace
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class TonapelMLP:
    kind: str
    ff: int
    experts: int = 0
    top: int = 0
    limit: float = 0.0


@dataclass(frozen=True)
class TonapelLayer:
    type: str
    mixer: Any                      # ParallelMixer | DeltaMixer
    mlp: Optional[TonapelMLP]


def _need(d: Any, key: str, where: str) -> Any:
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key '{where}{key}' is missing")
    return d[key]


def _positive(where: str, **values: int) -> None:
    for name, v in values.items():
        if v <= 0:
            raise ConfigError(f"config.json: '{where}{name}' must be positive")


def _divides(where: str, part: str, p: int, whole: str, w: int) -> None:
    if w % p:
        raise ConfigError(f"config.json: '{where}{part}' = {p} does not divide {whole} = {w}")


def _read_left(m: Any, where: str) -> WindowAttention:
    rot, mask = _need(m, "rot", where), _need(m, "mask", where)
    a = WindowAttention(
        heads=int(_need(m, "heads", where)), kv_heads=int(m.get("kv_heads") or m["heads"]),
        dim=int(_need(m, "dim", where)), vdim=int(m.get("vdim") or m["dim"]),
        scale=float(_need(m, "scale", where)), window=int(_need(mask, "size", where + "mask.")),
        rot_base=float(_need(rot, "base", where + "rot.")), rot_dims=int(_need(rot, "dims", where + "rot.")))
    _positive(where, heads=a.heads, kv_heads=a.kv_heads, dim=a.dim, vdim=a.vdim)
    _positive(where + "mask.", size=a.window)
    _divides(where, "kv_heads", a.kv_heads, "heads", a.heads)
    if a.rot_dims < 0 or a.rot_dims % 2 or a.rot_dims > a.dim:
        raise ConfigError(f"config.json: '{where}rot.dims' = {a.rot_dims} must be even and at most dim = {a.dim}")
    if a.rot_dims and a.rot_base <= 0:
        raise ConfigError(f"config.json: '{where}rot.base' must be positive")
    if max(a.dim, a.vdim) > 512:
        raise ConfigError(f"config.json: '{where}dim' / 'vdim' above 512 are not supported")
    return a


def _read_right(m: Any, where: str) -> StateSpace:
    s = StateSpace(heads=int(_need(m, "heads", where)), vdim=int(_need(m, "vdim", where)),
                   state=int(_need(m, "state", where)), groups=int(m.get("groups") or 1),
                   conv=int(_need(m, "conv", where)), norm_groups=int(m.get("norm_groups") or 1))
    _positive(where, heads=s.heads, vdim=s.vdim, state=s.state, groups=s.groups, conv=s.conv,
              norm_groups=s.norm_groups)
    _divides(where, "groups", s.groups, "heads", s.heads)
    _divides(where, "norm_groups", s.norm_groups, "heads * vdim", s.heads * s.vdim)
    if s.state > 256:
        raise ConfigError(f"config.json: '{where}state' above 256 is not supported")
    return s


def _read_delta(m: Any, where: str) -> DeltaMixer:
    d = DeltaMixer(heads=int(_need(m, "heads", where)), kv_heads=int(m.get("kv_heads") or m["heads"]),
                   dim=int(_need(m, "dim", where)), vdim=int(m.get("vdim") or m["dim"]),
                   conv=int(_need(m, "conv", where)))
    _positive(where, heads=d.heads, kv_heads=d.kv_heads, dim=d.dim, vdim=d.vdim, conv=d.conv)
    _divides(where, "kv_heads", d.kv_heads, "heads", d.heads)
    if d.dim > 256:
        raise ConfigError(f"config.json: '{where}dim' above 256 is not supported")
    return d


def _read_mlp(mlp: Any, where: str) -> Optional[TonapelMLP]:
    if not mlp:
        return None
    kind = str(mlp.get("kind", "dense"))
    if kind not in MLP_KINDS:
        raise ConfigError(f"config.json: '{where}kind' = {kind!r} is not one of {list(MLP_KINDS)}")
    if kind == "dense":
        out = TonapelMLP("dense", int(_need(mlp, "ff", where)))
        _positive(where, ff=out.ff)
        return out
    expert, router = _need(mlp, "expert", where), _need(mlp, "router", where)
    out = TonapelMLP("moe", int(_need(expert, "ff", where + "expert.")),
                     experts=int(_need(router, "experts", where + "router.")),
                     top=int(_need(router, "top", where + "router.")),
                     limit=float(_need(expert, "limit", where + "expert.")))
    _positive(where, ff=out.ff, experts=out.experts, top=out.top)
    if out.top > out.experts:
        raise ConfigError(f"config.json: '{where}router.top' = {out.top} exceeds experts = {out.experts}")
    if not out.limit > 0:
        raise ConfigError(f"config.json: '{where}expert.limit' must be positive")
    return out


@dataclass(frozen=True)
class TonapelConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: Tuple[TonapelLayer, ...]
    raw: Mapping[str, Any]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "TonapelConfig":
        listed = _need(raw, "layers", "")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers: List[TonapelLayer] = []
        for i, entry in enumerate(listed):
            where = f"layers[{i}]."
            kind = str(_need(entry, "type", where))
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{where}type' = {kind!r} is not one of {list(MIXER_TYPES)}")
            m = _need(entry, "mixer", where)
            mw = where + "mixer."
            if kind == "parallel":
                mixer = ParallelMixer(_read_left(_need(m, "left", mw), mw + "left."),
                                      _read_right(_need(m, "right", mw), mw + "right."),
                                      float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0)))
            else:
                mixer = _read_delta(m, mw)
            layers.append(TonapelLayer(kind, mixer, _read_mlp(entry.get("mlp"), where + "mlp.")))
        cfg = cls(vocab=int(_need(raw, "vocab", "")), width=int(_need(raw, "width", "")),
                  norm_eps=float(_need(_need(raw, "norm", ""), "eps", "norm.")),
                  residual_mult=float(raw.get("residual_mult", 1.0)), layers=tuple(layers), raw=dict(raw))
        if cfg.vocab <= 0 or cfg.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if cfg.norm_eps < 0:
            raise ConfigError("config.json: 'norm.eps' must not be negative")
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)


def _mixer_spec(cfg: TonapelConfig, layer: TonapelLayer) -> PartSpec:
    W = cfg.width
    if layer.type == "delta":
        d: DeltaMixer = layer.mixer
        return PartSpec("gated_delta", {
            "hidden_size": W, "heads": d.heads, "key_heads": d.kv_heads, "key_dim": d.dim, "head_dim": d.vdim,
            "conv_taps": d.conv, "norm_eps": cfg.norm_eps, "unit_eps": UNIT_NORM_EPS, "scope": "mix",
            "names": {"q": "q", "k": "k", "v": "v", "gate": "g", "beta": "b", "decay": "a",
                      "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "a_log": "A_log",
                      "dt_bias": "dt_bias", "norm": "norm", "o": "o", "in": "qkvgba", "conv": "qkv.conv"}})
    p: ParallelMixer = layer.mixer
    a, s = p.left, p.right
    left = PartSpec("paged_attention", {
        "hidden_size": W, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
        "value_dim": a.vdim, "sm_scale": a.scale, "qk_norm": "none", "sliding_window": a.window, "bias": True,
        "position": PartSpec("rotary_neox", {"head_dim": a.dim, "rotary_dim": a.rot_dims, "theta": a.rot_base,
                                             "max_position": NO_POSITION_LIMIT, "exact_angles": True}),
        "scope": "mix.left",
        "checkpoint_names": {"qkv": "qkv", "q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm",
                             "k_norm": "k.norm", "qkv_bias": "qkv.b", "q_bias": "q.b", "k_bias": "k.b",
                             "v_bias": "v.b", "o_bias": "o.b"}})
    right = PartSpec("ssd", {
        "hidden_size": W, "heads": s.heads, "head_dim": s.vdim, "state_dim": s.state, "groups": s.groups,
        "conv_taps": s.conv, "norm_groups": s.norm_groups, "norm_eps": cfg.norm_eps, "scope": "mix.right",
        "names": {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log",
                  "d": "D", "norm": "norm", "o": "o"}})
    return PartSpec("mixer_sum", {"hidden_size": W, "members": (left, right),
                                  "scales": (p.left_scale, p.right_scale)})


def _mlp_spec(cfg: TonapelConfig, mlp: TonapelMLP) -> PartSpec:
    if mlp.kind == "dense":
        return PartSpec("dense_mlp", {"hidden_size": cfg.width, "intermediate_size": mlp.ff,
                                      "activation": "gelu_tanh", "gated": True, "scope": "mlp",
                                      "names": {"gate": "gate", "up": "up", "down": "down", "gate_up": "gate_up"}})
    return PartSpec("routed_experts", {
        "hidden_size": cfg.width, "intermediate_size": mlp.ff, "num_experts": mlp.experts, "top_k": mlp.top,
        # the largest logits are the largest softmax scores; renormalising those is the softmax over them alone
        "scoring": "softmax", "use_bias": False, "renormalize": True, "scale": 1.0,
        "activation": "swigluoai", "act_alpha": EXPERT_GATE_ALPHA, "act_limit": mlp.limit, "scope": "mlp",
        "checkpoint_names": {"router": "router", "bias": "router.bias", "gate_up": "experts.gate_up",
                             "down": "experts.down", "gate": "e{e}.gate", "up": "e{e}.up",
                             "down_each": "e{e}.down"}})


def build_plan(cfg: TonapelConfig) -> ModelPlan:
    W = cfg.width

    def norm(tensor: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": W, "eps": cfg.norm_eps, "plus_one": True, "tensor": tensor})

    layers: List[LayerSpec] = []
    for i, layer in enumerate(cfg.layers):
        ffn = _mlp_spec(cfg, layer.mlp) if layer.mlp is not None else None
        layers.append(LayerSpec(
            prefix=f"l{i}", block=PartSpec("sandwich", {"residual_mult": cfg.residual_mult}),
            mixer=_mixer_spec(cfg, layer), feed_forward=ffn, mixer_norm=norm("norm1"),
            feed_forward_norm=norm("norm2") if ffn is not None else None,
            norms={"mixer_out": norm("norm1b"), **({"feed_forward_out": norm("norm2b")} if ffn is not None else {})}))
    plan = ModelPlan(
        architecture=ARCHITECTURE, hidden_size=W, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "prefix": "",
                                               "tensor": "embed"}),
        layers=tuple(layers), schedule=tuple(RunEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", {**norm("final.norm").params, "prefix": ""}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": W, "prefix": "", "tensor": "head",
                                  "tied_to": None}),
        max_position=NO_POSITION_LIMIT)
    plan.validate()
    return plan
