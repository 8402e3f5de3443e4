"""Typed configuration of the Fazinex decoder, read from ``config.json``.

A Fazinex model is a list of layers, each a *parallel* block (one RMS norm whose
output feeds a mixer and, if the layer has one, a feed-forward; the layer adds
the sum of both) with one of two mixers:

* ``attention``: grouped-query attention whose values are its keys, no rotation,
  a query temperature that grows with the logarithm of the position;
* ``latent_attention``: keys and values made from one cached, RMS-normed latent
  vector per token, a sigmoid gate per head on the output.

The embedded tokens are RMS-normed before the first layer; layers ``start ..
stop-1`` of ``loop`` run ``times`` times in a row with the same weights, every
pass with a cache of its own; the head is the embedding table, and the logits
are capped by ``cap * tanh(logits / cap)``.

config.json keys: ``architecture`` (``"Fazinex"``), ``vocab``, ``width``,
``norm.eps``, ``logit_softcap``, ``loop.{start, stop, times}`` and ``layers[i]``
with ``type``, ``mixer`` (``heads``, ``dim``, ``vdim``, ``scale`` and ``kv_heads``,
``q_temp.{coef, every}`` or ``kv_rank``) and ``mlp`` (``kind``, ``ff``; ``null``:
no feed-forward).  Every size and constant is handed to a part as a parameter
by :func:`build_plan`; tensors are ``embed``, ``embed.norm``, ``final.norm`` and
``l<i>.{norm1, mix.*, mlp.*}``.  The reference has no model of this design; the
module follows the shape of python/freetoken/models/minimax_m3/args.py:135-254.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple

from .model_plan import ConfigError, LayerSpec, ModelPlan, PartSpec, RunEntry

ARCHITECTURE = "Fazinex"
MIXER_TYPES = ("attention", "latent_attention")
# the design has no position table and no longest sequence of its own
NO_POSITION_LIMIT = 1 << 30


@dataclass(frozen=True)
class FazinexMixer:
    type: str
    heads: int
    dim: int
    vdim: int
    scale: float
    kv_heads: int = 1            # attention
    q_temp_coef: float = 0.0     # attention
    q_temp_every: int = 1        # attention
    kv_rank: int = 0             # latent_attention


@dataclass(frozen=True)
class FazinexLayer:
    mixer: FazinexMixer
    mlp_kind: Optional[str]      # None: the layer has no feed-forward
    ff: int = 0


@dataclass(frozen=True)
class FazinexConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_softcap: float         # 0: the logits are not capped
    layers: Tuple[FazinexLayer, ...]
    loop_start: int
    loop_stop: int
    loop_times: int
    raw: Mapping[str, Any]

    # ---- reading -------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "FazinexConfig":
        def need(d: Mapping[str, Any], key: str, where: str) -> Any:
            if not isinstance(d, Mapping) or key not in d or d[key] is None:
                raise ConfigError(f"config.json: required key '{where}{key}' is missing")
            return d[key]

        layers: List[FazinexLayer] = []
        listed = need(raw, "layers", "")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        for i, entry in enumerate(listed):
            where = f"layers[{i}]."
            kind = str(need(entry, "type", where))
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{where}type' = {kind!r} is not one of {list(MIXER_TYPES)}")
            m = need(entry, "mixer", where)
            mw = where + "mixer."
            heads, dim = int(need(m, "heads", mw)), int(need(m, "dim", mw))
            fields: Dict[str, Any] = dict(type=kind, heads=heads, dim=dim, vdim=int(m.get("vdim") or dim),
                                          scale=float(need(m, "scale", mw)))
            if kind == "attention":
                fields["vdim"] = dim          # the values are the keys: they have the keys' size
                fields["kv_heads"] = int(m.get("kv_heads") or heads)
                temp = m.get("q_temp")
                if temp:
                    fields["q_temp_coef"] = float(need(temp, "coef", mw + "q_temp."))
                    fields["q_temp_every"] = int(need(temp, "every", mw + "q_temp."))
            else:
                fields["kv_rank"] = int(need(m, "kv_rank", mw))
            mlp = entry.get("mlp")
            if mlp:
                mlp_kind = str(mlp.get("kind", "dense"))
                if mlp_kind != "dense":
                    raise ConfigError(f"config.json: '{where}mlp.kind' = {mlp_kind!r} is not supported (dense only)")
                layers.append(FazinexLayer(FazinexMixer(**fields), mlp_kind, int(need(mlp, "ff", where + "mlp."))))
            else:
                layers.append(FazinexLayer(FazinexMixer(**fields), None))
        loop = raw.get("loop") or {}
        start = int(loop.get("start", 0))
        cfg = cls(
            vocab=int(need(raw, "vocab", "")),
            width=int(need(raw, "width", "")),
            norm_eps=float(need(need(raw, "norm", ""), "eps", "norm.")),
            logit_softcap=float(raw.get("logit_softcap") or 0.0),
            layers=tuple(layers),
            loop_start=start,
            loop_stop=int(loop.get("stop", start)),
            loop_times=int(loop.get("times", 1)),
            raw=dict(raw),
        )
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)

    # ---- validation ------------------------------------------------------------
    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if self.norm_eps < 0:
            raise ConfigError("config.json: 'norm.eps' must not be negative")
        if self.logit_softcap < 0:
            raise ConfigError("config.json: 'logit_softcap' must not be negative")
        n = len(self.layers)
        if not (0 <= self.loop_start <= self.loop_stop <= n) or self.loop_times < 1:
            raise ConfigError(f"config.json: 'loop' {self.loop_start}..{self.loop_stop} x {self.loop_times} "
                              f"does not fit {n} layers")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            where = f"layers[{i}].mixer"
            if min(m.heads, m.dim, m.vdim) <= 0:
                raise ConfigError(f"config.json: '{where}' sizes must be positive")
            if m.type == "attention":
                if m.kv_heads <= 0 or m.heads % m.kv_heads:
                    raise ConfigError(f"config.json: '{where}.kv_heads' = {m.kv_heads} does not divide "
                                      f"heads = {m.heads}")
                if m.q_temp_coef != 0.0 and m.q_temp_every <= 0:
                    raise ConfigError(f"config.json: '{where}.q_temp.every' must be positive")
            elif m.kv_rank <= 0:
                raise ConfigError(f"config.json: '{where}.kv_rank' must be positive")
            if layer.mlp_kind is not None and layer.ff <= 0:
                raise ConfigError(f"config.json: 'layers[{i}].mlp.ff' must be positive")

    def run_order(self) -> List[int]:
        """Layer indices in the order they run: the looped span ``times`` times in a row."""
        n = len(self.layers)
        span = list(range(self.loop_start, self.loop_stop))
        return list(range(self.loop_start)) + span * self.loop_times + list(range(self.loop_stop, n))


def build_plan(cfg: FazinexConfig) -> ModelPlan:
    """Every layer: RMS norm -> (mixer + feed-forward) in parallel; every run of a layer is a
    stop of the schedule with a cache of its own."""
    W = cfg.width

    def norm(tensor: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": W, "eps": cfg.norm_eps, "plus_one": False, "tensor": tensor})

    layers: List[LayerSpec] = []
    for layer in cfg.layers:
        m = layer.mixer
        if m.type == "attention":
            mixer = PartSpec("shared_kv_attention", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "sm_scale": m.scale, "q_temp_coef": m.q_temp_coef, "q_temp_every": m.q_temp_every,
                "sliding_window": None, "scope": "mix",
                "names": {"q": "q", "k": "k", "o": "o", "qk": "qk"},
            })
        else:
            mixer = PartSpec("latent_attention", {
                "hidden_size": W, "num_heads": m.heads, "qk_dim": m.dim, "v_dim": m.vdim, "rank": m.kv_rank,
                "sm_scale": m.scale, "norm_eps": cfg.norm_eps, "output_gate": True, "scope": "mix",
                "names": {"q": "q", "down": "dkv", "gate": "g", "latent_norm": "dkv.norm", "up_k": "uk",
                          "up_v": "uv", "o": "o", "in": "q_dkv_g"},
            })
        ffn = None
        if layer.mlp_kind is not None:
            ffn = PartSpec("dense_mlp", {"hidden_size": W, "intermediate_size": layer.ff, "activation": "relu2",
                                         "scope": "mlp", "names": {"up": "up", "down": "down"}})
        layers.append(LayerSpec(prefix=f"l{len(layers)}", block=PartSpec("parallel", {}), mixer=mixer,
                                feed_forward=ffn, mixer_norm=norm("norm1")))
    plan = ModelPlan(
        architecture=ARCHITECTURE,
        hidden_size=W,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": W, "prefix": "",
                                               "tensor": "embed", "norm_tensor": "embed.norm",
                                               "norm_eps": cfg.norm_eps}),
        layers=tuple(layers),
        schedule=tuple(RunEntry(i) for i in cfg.run_order()),
        final_norm=PartSpec("rmsnorm", {**norm("final.norm").params, "prefix": ""}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": W, "prefix": "", "scope": None,
                                  "tied_to": "embed", "softcap": cfg.logit_softcap}),
        max_position=NO_POSITION_LIMIT,
    )
    plan.validate()
    return plan
