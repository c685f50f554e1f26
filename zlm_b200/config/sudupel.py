"""Typed configuration of the Sudupel architecture, read from its own ``config.json`` keys, and its lowering to a
``ModelSpec``.

A Sudupel config.json names the design with a string and lists its layers one by one; layers of one model may differ
in kind and in every size:

    {"architecture": "Sudupel", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "logit_softcap": c,
     "layers": [{"type": "parallel", "mixer": {"left": {...attention...}, "right": {...recurrent block...},
                                               "left_scale": a, "right_scale": b}, "mlp": ...},
                {"type": "parallel_2", "mixer": {"left": {...attention...}, "right": {...gated linear attention...},
                                                 "left_scale": a, "right_scale": b}, "mlp": ...},
                {"type": "lightning", "mixer": {"heads", "dim", "vdim", "decay": [one per head]}, "mlp": ...}]}

The design.  Every layer norms what a sublayer reads and what it gives: x += norm1b(mixer(norm1(x))), then
x += norm2b(ff(norm2(x))), RMS norms whose stored weight w stands for 1 + w.  A ``parallel`` mixer is softmax attention
(grouped heads, q and k normed over the whole projection with a weight per channel, rotary positions with an optional
long-context blend of the frequencies, every earlier token visible, one more term of score 0 in the denominator) beside
a recurrent block (two branches, a short convolution, block-diagonal gates, a real-gated linear recurrence), their
outputs summed with a scale each.  A ``parallel_2`` mixer is attention over a sliding window whose q, k, v pass through
short convolutions, with a per-head norm of q and k that has one weight for all heads and rotary positions, beside
gated linear attention whose decay per key channel comes from a low-rank projection.  A ``lightning`` mixer is linear
attention with a fixed decay per head on silu(q), silu(k), silu(v), the heads normed together, a sigmoid gate.  The
feed-forward is dense (gate and up clamped by ``limit``, g sigmoid(1.702 g) (u + 1)) or a mixture of gated silu
experts routed by sigmoid scores plus a correction inside the best groups (a group's mark is the sum of its two best
choice scores), weights not renormalised.  The embedding is scaled; a last norm, an untied head and a tanh cap give
the logits.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, coerce, require

ARCHITECTURE = "Sudupel"
NO_POSITION_LIMIT = 1 << 24          # the design sets no longest sequence; the cache an engine is built with does
DECAY_SCALE = 8.0                    # log a = -8 r softplus(lam)
SWISH_ALPHA = 1.702                  # g sigmoid(1.702 g)


def _mapping(d: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return v


def _req(m: Mapping[str, Any], key: str, typ, where: str):
    if key not in m or m[key] is None:
        raise ConfigError(f"config.json: {where}missing key '{key}'")
    return coerce(m[key], where + key, typ)


def _opt(m: Mapping[str, Any], key: str, typ, where: str, default):
    return default if m.get(key) is None else coerce(m[key], where + key, typ)


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]] = None      # factor, original, fast, slow

    @classmethod
    def from_dict(cls, d: Optional[Mapping[str, Any]], where: str, dim: int) -> Optional["RotaryConfig"]:
        if d is None:
            return None
        if not isinstance(d, Mapping):
            raise ConfigError(f"config.json: {where[:-1]} must be an object")
        sc = d.get("scaling")
        scaling = None
        if sc is not None:
            sc = _mapping(d, "scaling", where)
            scaling = tuple(_req(sc, k, float, where + "scaling.") for k in ("factor", "original", "fast", "slow"))
            if scaling[0] <= 0 or scaling[1] <= 0 or scaling[2] <= 0 or scaling[3] <= 0:
                raise ConfigError(f"config.json: {where}scaling: factor, original, fast and slow must be positive")
        c = cls(_req(d, "base", float, where), _req(d, "dims", int, where), scaling)
        if c.dims % 2 or not 0 <= c.dims <= dim:
            raise ConfigError(f"config.json: {where}dims={c.dims} must be even and at most dim={dim}")
        if c.base <= 0 or (scaling is not None and c.base == 1.0):
            raise ConfigError(f"config.json: {where}base={c.base}")
        return c if c.dims else None

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            d["scaling"] = dict(zip(("factor", "original", "fast", "slow"), self.scaling))
        return d

    def position(self) -> Dict[str, Any]:
        p: Dict[str, Any] = {"kind": "rope_half_split", "theta": self.base, "head_dim": self.dims, "n_rot": self.dims}
        if self.scaling is not None:
            p["scaling"] = dict(zip(("factor", "original", "fast", "slow"), self.scaling))
        return p


@dataclass(frozen=True)
class AttentionConfig:
    """The left side of both parallel mixers; ``conv`` 0: no convolution, ``window`` 0: every earlier token."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotaryConfig]
    conv: int = 0
    window: int = 0

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "AttentionConfig":
        heads, dim = _req(d, "heads", int, where), _req(d, "dim", int, where)
        if dim <= 0:
            raise ConfigError(f"config.json: {where}dim must be positive")
        mask = d.get("mask")
        window = 0 if mask is None else _req(_mapping(d, "mask", where), "size", int, where + "mask.")
        c = cls(heads, _opt(d, "kv_heads", int, where, heads), dim, _req(d, "vdim", int, where),
                _req(d, "scale", float, where), RotaryConfig.from_dict(d.get("rot"), where + "rot.", dim),
                _opt(d, "conv", int, where, 0), window)
        if min(c.heads, c.kv_heads, c.vdim) <= 0 or c.window < 0 or c.conv < 0:
            raise ConfigError(f"config.json: {where}sizes must be positive")
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}heads={c.heads} is not a multiple of kv_heads={c.kv_heads}")
        if c.conv > 8:
            raise ConfigError(f"config.json: {where}conv={c.conv}: at most 8 taps are built")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        if self.conv:
            d["conv"] = self.conv
        if self.window:
            d["mask"] = {"size": self.window}
        return d


@dataclass(frozen=True)
class RecurrentConfig:
    width: int
    blocks: int
    conv: int

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "RecurrentConfig":
        c = cls(_req(d, "width", int, where), _req(d, "blocks", int, where), _req(d, "conv", int, where))
        if c.width <= 0 or c.blocks <= 0 or c.width % c.blocks:
            raise ConfigError(f"config.json: {where}width={c.width} in blocks={c.blocks}")
        if not 1 <= c.conv <= 8:
            raise ConfigError(f"config.json: {where}conv={c.conv}: 1 to 8 taps are built")
        return c

    def to_dict(self) -> Dict[str, Any]:
        return {"width": self.width, "blocks": self.blocks, "conv": self.conv}


@dataclass(frozen=True)
class GatedLinearConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: Optional[int] = None       # not a key of the design: a checkpoint's tensors give it; random models may name it

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "GatedLinearConfig":
        c = cls(_req(d, "heads", int, where), _req(d, "dim", int, where), _req(d, "vdim", int, where),
                _req(d, "tau", float, where), _opt(d, "rank", int, where, None))
        if min(c.heads, c.dim, c.vdim) <= 0 or c.tau <= 0 or (c.rank is not None and c.rank <= 0):
            raise ConfigError(f"config.json: {where}sizes and tau must be positive")
        if c.dim > 128:
            raise ConfigError(f"config.json: {where}dim={c.dim}: keys of up to 128 columns are built")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}
        if self.rank is not None:
            d["rank"] = self.rank
        return d


@dataclass(frozen=True)
class ParallelConfig:
    left: AttentionConfig
    right: Union[RecurrentConfig, GatedLinearConfig]
    left_scale: float
    right_scale: float

    def to_dict(self) -> Dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class LightningConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "LightningConfig":
        decay = d.get("decay")
        if not isinstance(decay, (list, tuple)):
            raise ConfigError(f"config.json: {where}'decay' must be a list with one number per head")
        c = cls(_req(d, "heads", int, where), _req(d, "dim", int, where), _req(d, "vdim", int, where),
                tuple(coerce(x, where + "decay", float) for x in decay))
        if min(c.heads, c.dim, c.vdim) <= 0:
            raise ConfigError(f"config.json: {where}sizes must be positive")
        if len(c.decay) != c.heads:
            raise ConfigError(f"config.json: {where}decay lists {len(c.decay)} numbers for {c.heads} heads")
        return c

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class DenseConfig:
    ff: int
    limit: float

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": "dense", "ff": self.ff, "limit": self.limit}


@dataclass(frozen=True)
class ExpertsConfig:
    ff: int
    experts: int
    top: int
    groups: int
    keep: int

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": "moe", "expert": {"ff": self.ff},
                "router": {"experts": self.experts, "top": self.top, "groups": {"count": self.groups, "keep": self.keep}}}


def _feed_forward(d: Optional[Mapping[str, Any]], where: str) -> Union[None, DenseConfig, ExpertsConfig]:
    if d is None:
        return None
    if not isinstance(d, Mapping):
        raise ConfigError(f"config.json: {where[:-1]} must be an object or null")
    kind = d.get("kind")
    if kind == "dense":
        c = DenseConfig(_req(d, "ff", int, where), _req(d, "limit", float, where))
        if c.ff <= 0 or c.limit <= 0:
            raise ConfigError(f"config.json: {where}ff and limit must be positive")
        return c
    if kind == "moe":
        router, expert = _mapping(d, "router", where), _mapping(d, "expert", where)
        groups = router.get("groups")
        if groups is None:
            count, keep = 1, 1
        else:
            groups = _mapping(router, "groups", where + "router.")
            count, keep = _req(groups, "count", int, where + "router.groups."), _req(groups, "keep", int, where + "router.groups.")
        e = ExpertsConfig(_req(expert, "ff", int, where + "expert."), _req(router, "experts", int, where + "router."),
                          _req(router, "top", int, where + "router."), count, keep)
        if e.ff <= 0 or e.experts <= 0 or not 0 < e.top <= e.experts:
            raise ConfigError(f"config.json: {where}router.top={e.top} of {e.experts} experts of ff={e.ff}")
        if not 1 <= e.keep <= e.groups or e.experts % e.groups or e.keep * (e.experts // e.groups) < e.top:
            raise ConfigError(f"config.json: {where}router.groups: {e.groups} groups (keep {e.keep}) over {e.experts} experts "
                              f"cannot give {e.top} choices")
        return e
    raise ConfigError(f"config.json: {where}kind={kind!r} is not known (dense, moe)")


@dataclass(frozen=True)
class SudupelLayer:
    type: str
    mixer: Union[ParallelConfig, LightningConfig]
    mlp: Union[None, DenseConfig, ExpertsConfig]


@dataclass(frozen=True)
class SudupelConfig:
    vocab_size: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_softcap: float             # 0: none
    layers: Tuple[SudupelLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    # ---- reading -----------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "SudupelConfig":
        vocab, width = require(d, "vocab", int), require(d, "width", int)
        eps = require(_mapping(d, "norm", ""), "eps", float)
        if vocab <= 0 or width <= 0 or eps <= 0:
            raise ConfigError("config.json: vocab, width and norm.eps must be positive")
        emb = d.get("embedding")
        scale = 1.0 if emb is None else _opt(_mapping(d, "embedding", ""), "scale", float, "embedding.", 1.0)
        cap = _opt(d, "logit_softcap", float, "", 0.0)
        if cap < 0:
            raise ConfigError("config.json: logit_softcap must be positive")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, l in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(l, Mapping):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = l.get("type")
            m = _mapping(l, "mixer", where)
            mw = where + "mixer."
            if kind in ("parallel", "parallel_2"):
                left = AttentionConfig.from_dict(_mapping(m, "left", mw), mw + "left.")
                rd = _mapping(m, "right", mw)
                right = (RecurrentConfig if kind == "parallel" else GatedLinearConfig).from_dict(rd, mw + "right.")
                mixer: Any = ParallelConfig(left, right, _opt(m, "left_scale", float, mw, 1.0), _opt(m, "right_scale", float, mw, 1.0))
            elif kind == "lightning":
                mixer = LightningConfig.from_dict(m, mw)
            else:
                raise ConfigError(f"config.json: {where}type={kind!r} is not known (parallel, parallel_2, lightning)")
            layers.append(SudupelLayer(kind, mixer, _feed_forward(l.get("mlp"), where + "mlp.")))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab, width, eps, scale, cap, tuple(layers), eos_ids)

    # ---- writing -----------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.width, "norm": {"eps": self.norm_eps},
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                       for l in self.layers],
        }
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- lowering ----------------------------------------------------------
    def _attention(self, a: AttentionConfig, row_norm: bool, sink: bool) -> Tuple[Dict[str, Any], Dict[str, str]]:
        params = {"kind": "conv_attention", "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
                  "v_dim": a.vdim, "conv_taps": max(a.conv, 1), "conv": a.conv > 0, "scale": a.scale,
                  "norm_eps": self.norm_eps, "window": a.window, "qk_norm": "row" if row_norm else "head", "sink": sink,
                  "gate": "none", "position": a.rot.position() if a.rot is not None else {"kind": "none"}}
        names = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                 "q_norm.weight": "q.norm", "k_norm.weight": "k.norm", "q_conv.weight": "q.conv",
                 "k_conv.weight": "k.conv", "v_conv.weight": "v.conv"}
        return params, names

    def to_model_spec(self) -> ModelSpec:
        def norm(prefix: str, name: str) -> PartSpec:
            return PartSpec("rms_norm", {"eps": self.norm_eps, "one_plus": True}, prefix=prefix, rename={"weight": name})
        layers = []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}.", l.mixer
            if isinstance(m, ParallelConfig):
                left, lnames = self._attention(m.left, row_norm=l.type == "parallel", sink=l.type == "parallel")
                if isinstance(m.right, RecurrentConfig):
                    right = {"kind": "rglru", "width": m.right.width, "blocks": m.right.blocks, "conv_taps": m.right.conv,
                             "decay_scale": DECAY_SCALE}
                    rnames = {"y_proj.weight": "y", "y_proj.bias": "y.b", "x_proj.weight": "x", "x_proj.bias": "x.b",
                              "conv.weight": "conv", "conv.bias": "conv.b", "a_gate.weight": "ra", "a_gate.bias": "ra.b",
                              "i_gate.weight": "ri", "i_gate.bias": "ri.b", "lam": "lam", "o_proj.weight": "o"}
                else:
                    right = {"kind": "gated_linear_attention", "num_heads": m.right.heads, "head_dim": m.right.dim,
                             "v_dim": m.right.vdim, "tau": m.right.tau, "norm_eps": self.norm_eps, "rank": m.right.rank,
                             "gate": "silu"}
                    rnames = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "g_proj.weight": "g",
                              "o_proj.weight": "o", "a_down.weight": "a1", "a_up.weight": "a2", "a_up.bias": "a2.b",
                              "norm.weight": "norm"}
                rename = {**{"left." + a: "left." + b for a, b in lnames.items()},
                          **{"right." + a: "right." + b for a, b in rnames.items()}}
                mixer = PartSpec("parallel", {"left": left, "right": right, "left_scale": m.left_scale,
                                              "right_scale": m.right_scale}, prefix=p + "mix.", rename=rename)
            else:
                mixer = PartSpec("retention", {
                    "num_heads": m.heads, "head_dim": m.dim, "v_dim": m.vdim, "decay": tuple(m.decay),
                    "norm_eps": self.norm_eps, "position": {"kind": "none"}, "gate": "sigmoid", "k_scale": 1.0,
                    "qkv_act": "silu", "out_norm": "row"}, prefix=p + "mix.",
                    rename={"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "g_proj.weight": "g",
                            "o_proj.weight": "o", "norm.weight": "norm"})
            f = l.mlp
            if f is None:
                ffn, norm_f, post_f = PartSpec("none", {}), PartSpec("none", {}), None
            else:
                if isinstance(f, DenseConfig):
                    ffn = PartSpec("swiglu", {"intermediate_size": f.ff, "activation": "swish_limit", "limit": f.limit,
                                              "alpha": SWISH_ALPHA}, prefix=p + "mlp.",
                                   rename={"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"})
                else:
                    ffn = PartSpec("routed_experts", {
                        "num_experts": f.experts, "top_k": f.top, "expert_ff": f.ff, "shared_ff": 0, "score": "sigmoid",
                        "renormalize": False, "weight_on": "output", "activation": "swiglu", "correction": True,
                        "groups": f.groups, "keep": f.keep, "group_mark": "top2_sum"}, prefix=p + "mlp.")
                norm_f, post_f = norm(p, "norm2"), norm(p, "norm2b")
            layers.append(LayerSpec("sandwich_norm", mixer, ffn, norm(p, "norm1"), norm_f,
                                    mixer_post_norm=norm(p, "norm1b"), feed_forward_post_norm=post_f))
        spec = ModelSpec(
            architecture=ARCHITECTURE, hidden_size=self.width, vocab_size=self.vocab_size,
            max_position=NO_POSITION_LIMIT, layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
            embedding=PartSpec("token_embedding", {"scale": self.embedding_scale}, rename={"weight": "embed"}),
            final_norm=norm("final.", "norm"),
            head=PartSpec("lm_head", {"tied": False, "softcap": self.logit_softcap}, rename={"weight": "head"}),
        )
        spec.validate()
        return spec
