"""Typed configuration of the Lodevik architecture, read from its own ``config.json`` keys, and its lowering to a
``ModelSpec``.

A Lodevik config.json names the design with a string and lists its layers one by one; layers of one model may differ
in kind and in every size:

    {"architecture": "Lodevik", "vocab": V, "width": W, "norm": {"eps": e}, "logit_scale": s,
     "embedding": {"scale": a, "bigram": {"buckets": B, "mul_prev": p, "mul_cur": c}},
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot": {"base", "dims"}},
                 "mlp": null | {"kind": "dense", "ff": F}},
                {"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "diff", "mask": {"size": chunk},
                           "rot": {"base", "dims"}},
                 "mlp": ...}, ...]}

The design: the stream starts as the token's row of ``embed`` times ``embedding.scale`` plus a row of ``bigram`` that
the token and the token before it choose.  Every layer norms its sublayers' *outputs*: x += ls1 * norm1(mixer(x)),
x += ls2 * norm2(ff(x)) (``l<i>.norm1``, ``l<i>.ls1`` ...: RMS norms and a scale per coordinate); the sublayers read x
itself.  A ``latent_attention`` mixer keeps one small normed latent and one rotated key part per token, has a learned
sink per head in its softmax and a sigmoid gate per head on its output.  An ``attention`` mixer is differential
attention: two maps per head over the same values, normed q and k, rotation on part of a head, a tanh cap on the
scores, keys visible only inside the query's own chunk of positions.  The feed-forward is gated with the tanh form of
gelu.  A last norm (``final.norm``) and the embedding table itself give the logits, times ``logit_scale``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, coerce, require

ARCHITECTURE = "Lodevik"
# the design sets no longest sequence; the cache an engine is built with does
NO_POSITION_LIMIT = 1 << 24


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


def _rot(d: Mapping[str, Any], where: str, limit: int, what: str) -> Tuple[float, int]:
    """(base, dims) of the mixer's ``rot`` object; no object: no rotation."""
    if d.get("rot") is None:
        return 10000.0, 0
    rot = _mapping(d, "rot", where)
    base, dims = _req(rot, "base", float, where + "rot."), _req(rot, "dims", int, where + "rot.")
    if dims % 2 or not 0 <= dims <= limit:
        raise ConfigError(f"config.json: {where}rot.dims={dims} must be even and at most {what}={limit}")
    if base <= 0:
        raise ConfigError(f"config.json: {where}rot.base must be positive")
    return base, dims


def _chunk(d: Mapping[str, Any], where: str) -> int:
    """The size of the mixer's ``mask`` object (keys of the query's own chunk only); no object: every earlier key."""
    if d.get("mask") is None:
        return 0
    size = _req(_mapping(d, "mask", where), "size", int, where + "mask.")
    if size <= 0:
        raise ConfigError(f"config.json: {where}mask.size must be positive")
    return size


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    chunk: int = 0

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "LatentMixerConfig":
        rot_dim = _req(d, "rot_dim", int, where)
        base, dims = _rot(d, where, rot_dim, "rot_dim")
        c = cls(_req(d, "heads", int, where), _req(d, "dim", int, where), rot_dim, _req(d, "vdim", int, where),
                _req(d, "kv_rank", int, where), _req(d, "scale", float, where), base, dims, _chunk(d, where))
        if min(c.heads, c.vdim, c.kv_rank) <= 0 or c.dim < 0 or c.rot_dim < 0 or c.dim + c.rot_dim <= 0:
            raise ConfigError(f"config.json: {where}sizes must be positive")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                             "kv_rank": self.kv_rank, "scale": self.scale}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.chunk:
            d["mask"] = {"size": self.chunk}
        return d


@dataclass(frozen=True)
class DiffMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float
    diff: float
    rot_base: float
    rot_dims: int
    chunk: int = 0

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str) -> "DiffMixerConfig":
        heads, dim = _req(d, "heads", int, where), _req(d, "dim", int, where)
        base, dims = _rot(d, where, dim, "dim")
        c = cls(heads, _opt(d, "kv_heads", int, where, heads), dim, _req(d, "vdim", int, where),
                _req(d, "scale", float, where), _opt(d, "softcap", float, where, 0.0), _req(d, "diff", float, where),
                base, dims, _chunk(d, where))
        if min(c.heads, c.kv_heads, c.dim, c.vdim) <= 0 or c.softcap < 0:
            raise ConfigError(f"config.json: {where}sizes must be positive")
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: {where}heads={c.heads} is not a multiple of kv_heads={c.kv_heads}")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale, "diff": self.diff}
        if self.softcap:
            d["softcap"] = self.softcap
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        if self.chunk:
            d["mask"] = {"size": self.chunk}
        return d


@dataclass(frozen=True)
class LodevikLayer:
    mixer: Union[LatentMixerConfig, DiffMixerConfig]
    ff: int                  # 0: no feed-forward

    @property
    def type(self) -> str:
        return "latent_attention" if isinstance(self.mixer, LatentMixerConfig) else "attention"


@dataclass(frozen=True)
class LodevikConfig:
    vocab_size: int
    width: int
    norm_eps: float
    layers: Tuple[LodevikLayer, ...]
    embedding_scale: float = 1.0
    bigram: Optional[Tuple[int, int, int]] = None         # (buckets, mul_prev, mul_cur)
    logit_scale: float = 1.0
    eos_token_ids: Tuple[int, ...] = ()

    # ---- reading -----------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LodevikConfig":
        vocab, width = require(d, "vocab", int), require(d, "width", int)
        eps = require(_mapping(d, "norm", ""), "eps", float)
        if vocab <= 0 or width <= 0 or eps <= 0:
            raise ConfigError("config.json: vocab, width and norm.eps must be positive")
        scale, bigram = 1.0, None
        if d.get("embedding") is not None:
            e = _mapping(d, "embedding", "")
            scale = _opt(e, "scale", float, "embedding.", 1.0)
            if e.get("bigram") is not None:
                b = _mapping(e, "bigram", "embedding.")
                bigram = tuple(_req(b, key, int, "embedding.bigram.") for key in ("buckets", "mul_prev", "mul_cur"))
                if bigram[0] <= 0 or min(bigram[1:]) < 0:
                    raise ConfigError("config.json: embedding.bigram: buckets must be positive, the multipliers not negative")
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
            if kind == "latent_attention":
                mixer = LatentMixerConfig.from_dict(m, where + "mixer.")
            elif kind == "attention":
                mixer = DiffMixerConfig.from_dict(m, where + "mixer.")
            else:
                raise ConfigError(f"config.json: {where}type={kind!r} is not known (latent_attention, attention)")
            mlp, ff = l.get("mlp"), 0
            if mlp is not None:
                if not isinstance(mlp, Mapping):
                    raise ConfigError(f"config.json: {where}mlp must be an object or null")
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind={mlp.get('kind')!r} is not known (dense)")
                ff = _req(mlp, "ff", int, where + "mlp.")
                if ff <= 0:
                    raise ConfigError(f"config.json: {where}mlp.ff must be positive")
            layers.append(LodevikLayer(mixer, ff))
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab, width, eps, tuple(layers), scale, bigram, optional_float(d, "logit_scale", 1.0), eos_ids)

    # ---- writing -----------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        emb: Dict[str, Any] = {"scale": self.embedding_scale}
        if self.bigram is not None:
            emb["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), self.bigram))
        d: Dict[str, Any] = {
            "architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.width,
            "norm": {"eps": self.norm_eps}, "embedding": emb, "logit_scale": self.logit_scale,
            "layers": [{"type": l.type, "mixer": l.mixer.to_dict(),
                        "mlp": {"kind": "dense", "ff": l.ff} if l.ff else None} for l in self.layers],
        }
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- lowering ----------------------------------------------------------
    def to_model_spec(self) -> ModelSpec:
        def norm(prefix: str, name: str, scale: Optional[str] = None) -> PartSpec:
            if scale is None:
                return PartSpec("rms_norm", {"eps": self.norm_eps}, prefix=prefix, rename={"weight": name})
            return PartSpec("rms_norm", {"eps": self.norm_eps, "layer_scale": True}, prefix=prefix,
                            rename={"weight": name, "scale": scale})
        layers = []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}.", l.mixer
            position = ({"kind": "rope_interleaved", "base": m.rot_base, "dims": m.rot_dims} if m.rot_dims
                        else {"kind": "none"})
            if isinstance(m, LatentMixerConfig):
                mixer = PartSpec("latent_attention", {
                    "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_dim": m.vdim, "kv_rank": m.kv_rank,
                    "scale": m.scale, "norm_eps": self.norm_eps, "position": position, "sink": True, "gate": True,
                    "chunk": m.chunk}, prefix=p + "mix.")
            else:
                mixer = PartSpec("diff_attention", {
                    "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim, "scale": m.scale,
                    "diff": m.diff, "norm_eps": self.norm_eps, "softcap": m.softcap, "chunk": m.chunk,
                    "position": position}, prefix=p + "mix.")
            if l.ff:
                ffn = PartSpec("swiglu", {"intermediate_size": l.ff, "activation": "gelu_tanh"}, prefix=p + "mlp.",
                               rename={"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"})
                norm_f = norm(p, "norm2", "ls2")
            else:
                ffn, norm_f = PartSpec("none", {}), PartSpec("none", {})
            layers.append(LayerSpec("sublayer_norm", mixer, ffn, norm(p, "norm1", "ls1"), norm_f))
        emb: Dict[str, Any] = {"scale": self.embedding_scale}
        rename = {"weight": "embed"}
        if self.bigram is not None:
            emb["pair"] = dict(zip(("buckets", "mul_prev", "mul_cur"), self.bigram))
            rename["pair"] = "bigram"
        spec = ModelSpec(
            architecture=ARCHITECTURE, hidden_size=self.width, vocab_size=self.vocab_size,
            max_position=NO_POSITION_LIMIT, layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
            embedding=PartSpec("token_embedding", emb, rename=rename),
            final_norm=norm("final.", "norm"),
            head=PartSpec("lm_head", {"tied": True, "logit_scale": self.logit_scale}, rename={"weight": "head"}),
        )
        spec.validate()
        return spec


def optional_float(d: Mapping[str, Any], key: str, default: float) -> float:
    return default if d.get(key) is None else coerce(d[key], key, float)
