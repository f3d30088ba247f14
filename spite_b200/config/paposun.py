"""Typed configuration of the Paposun decoder, read from its config.json.

The file lists the layers one by one: `layers[i]` gives the layer's `type` (which mixer it has), the mixer's sizes
and constants (`mixer`) and its feed-forward (`mlp`, or null for none).  `vocab`, `width`, `norm.eps`,
`residual_mult` and `logit_scale` are the model's own; `max_positions` and `eos_token_id` are optional.  Every size
and every constant that the file gives is read from it; what the design fixes is stated in `plan()`:

  * every sublayer is normed before and behind, and a factor stands on what joins the residual stream:
    x += residual_mult * norm_b(sublayer(norm_a(x)));
  * mixer `attention`: grouped-query attention with biases on its four projections, a rotation of the first
    `rot.dims` elements of every q and k head (element i with element i + dims/2, frequencies rescaled by wavelength
    from `rot.scaling`), scores times `scale`, sight limited to the query's chunk of `mask.size` positions, the
    concatenated heads times sigmoid(W_g x) element by element; a layer with `kv_from: j` has no key and value
    projections and reads layer j's cache (keys as cached, after rotation) with its own queries and chunk;
  * mixer `mlstm`: the matrix memory of `parts/mlstm.py` with q scaled by dim^-1/2, gates capped at `gate_cap`, the
    heads' norm with the layer's eps;
  * feed-forward `dense`: down(gelu_tanh(up x)); RMS norms; the output head is the embedding table, logits times
    `logit_scale`.

Tensor names: `embed`, `final.norm`, and per layer `l<i>.norm1`, `l<i>.norm1b`, `l<i>.norm2`, `l<i>.norm2b`,
`l<i>.mix.{q,k,v,g,o}` (attention: with `.b` biases on q, k, v, o; mlstm: also `norm`, `i`, `i.b`, `f`, `f.b`),
`l<i>.mlp.{up,down}`; linear weights `[out, in]`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .registry import register_architecture
from .specs import BlockSpec, ConfigError, LayerCall, ModelPlan, PartSpec, WeightBinding

DEFAULT_MAX_POSITIONS = 1 << 20


def _need(d, key, where):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key `{where}{key}` is missing")
    return d[key]


@dataclass(frozen=True)
class RotScaling:
    factor: float
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class GatedAttention:
    heads: int
    kv_heads: int
    dim: int                       # size of a query and a key head
    vdim: int                      # size of a value head
    scale: float                   # scores are (q . k) * scale
    chunk: Optional[int]           # mask.size; None: every earlier position is visible
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[RotScaling] = None
    kv_from: Optional[int] = None  # the layer whose cached keys and values this one reads


@dataclass(frozen=True)
class MatrixMemory:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class DenseMlp:
    ff: int


@dataclass(frozen=True)
class PaposunLayer:
    type: str
    mixer: object                  # GatedAttention | MatrixMemory
    mlp: Optional[DenseMlp]


@register_architecture("Paposun")
@dataclass(frozen=True)
class PaposunConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    logit_scale: float
    layers: tuple
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Optional[tuple] = None

    MIXERS = ("attention", "mlstm")

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "PaposunConfig":
        layers = []
        for i, L in enumerate(_need(raw, "layers", "")):
            at = f"layers[{i}]."
            kind = _need(L, "type", at)
            m = _need(L, "mixer", at)
            mat = at + "mixer."
            if kind == "attention":
                rot = _need(m, "rot", mat)
                sc = rot.get("scaling")
                scaling = None
                if sc:
                    scaling = RotScaling(*(float(_need(sc, k, mat + "rot.scaling.")) for k in ("factor", "low", "high", "original")))
                kv_from = m.get("kv_from")
                mixer = GatedAttention(
                    heads=int(_need(m, "heads", mat)), kv_heads=int(_need(m, "kv_heads", mat)), dim=int(_need(m, "dim", mat)),
                    vdim=int(_need(m, "vdim", mat)), scale=float(_need(m, "scale", mat)),
                    chunk=int(_need(m["mask"], "size", mat + "mask.")) if m.get("mask") else None,
                    rot_dims=int(_need(rot, "dims", mat + "rot.")), rot_base=float(_need(rot, "base", mat + "rot.")),
                    rot_scaling=scaling, kv_from=None if kv_from is None else int(kv_from))
            elif kind == "mlstm":
                mixer = MatrixMemory(heads=int(_need(m, "heads", mat)), dim=int(_need(m, "dim", mat)),
                                     vdim=int(_need(m, "vdim", mat)), gate_cap=float(_need(m, "gate_cap", mat)))
            else:
                raise ConfigError(f"config.json: {at}type {kind!r} is not a mixer of this design (known: {', '.join(cls.MIXERS)})")
            f = L.get("mlp")
            mlp = None
            if f is not None:
                fk = _need(f, "kind", at + "mlp.")
                if fk != "dense":
                    raise ConfigError(f"config.json: {at}mlp.kind {fk!r} is unknown (dense)")
                mlp = DenseMlp(ff=int(_need(f, "ff", at + "mlp.")))
            layers.append(PaposunLayer(kind, mixer, mlp))
        eos = raw.get("eos_token_id")
        if isinstance(eos, int):
            eos = (eos,)
        elif eos is not None:
            eos = tuple(int(x) for x in eos)
        cfg = cls(vocab=int(_need(raw, "vocab", "")), width=int(_need(raw, "width", "")),
                  norm_eps=float(_need(_need(raw, "norm", ""), "eps", "norm.")),
                  residual_mult=float(_need(raw, "residual_mult", "")), logit_scale=float(_need(raw, "logit_scale", "")),
                  layers=tuple(layers), max_positions=int(raw.get("max_positions") or DEFAULT_MAX_POSITIONS), eos_token_id=eos)
        cfg.validate()
        return cfg

    def validate(self):
        c = self
        for k, v in {"vocab": c.vocab, "width": c.width, "max_positions": c.max_positions}.items():
            if v <= 0:
                raise ConfigError(f"`{k}` must be positive, got {v}")
        if not c.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if not c.layers:
            raise ConfigError("a model needs at least one layer")
        for i, L in enumerate(c.layers):
            m = L.mixer
            at = f"layers[{i}].mixer"
            if isinstance(m, GatedAttention):
                if min(m.heads, m.kv_heads, m.dim, m.vdim, m.chunk if m.chunk is not None else 1) < 1:
                    raise ConfigError(f"{at}: heads, kv_heads, dim, vdim and mask.size must be positive")
                if m.heads % m.kv_heads:
                    raise ConfigError(f"{at}: {m.heads} heads are no multiple of {m.kv_heads} kv_heads")
                if not m.scale > 0:
                    raise ConfigError(f"{at}: scale must be positive")
                if m.rot_dims < 2 or m.rot_dims % 2 or m.rot_dims > m.dim:
                    raise ConfigError(f"{at}: rot.dims {m.rot_dims} must be even and lie in 2..dim ({m.dim})")
                if not m.rot_base > 0:
                    raise ConfigError(f"{at}: rot.base must be positive")
                if m.rot_scaling is not None and (m.rot_scaling.high <= m.rot_scaling.low or m.rot_scaling.factor <= 0):
                    raise ConfigError(f"{at}: rot.scaling needs high > low and a positive factor")
                if m.kv_from is not None:
                    j = m.kv_from
                    if not 0 <= j < i or not isinstance(c.layers[j].mixer, GatedAttention) or c.layers[j].mixer.kv_from is not None:
                        raise ConfigError(f"{at}.kv_from {j}: not an earlier attention layer with keys and values of its own")
                    o = c.layers[j].mixer
                    if (o.kv_heads, o.dim, o.vdim) != (m.kv_heads, m.dim, m.vdim):
                        raise ConfigError(f"{at}.kv_from {j}: that layer's keys and values have other sizes")
            else:
                if min(m.heads, m.dim, m.vdim) < 1 or not m.gate_cap > 0:
                    raise ConfigError(f"{at}: heads, dim, vdim and gate_cap must be positive")
            if L.mlp is not None and L.mlp.ff < 1:
                raise ConfigError(f"layers[{i}].mlp.ff must be positive")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        layers = []
        for L in self.layers:
            m = L.mixer
            if isinstance(m, GatedAttention):
                rot = {"base": m.rot_base, "dims": m.rot_dims}
                if m.rot_scaling is not None:
                    s = m.rot_scaling
                    rot["scaling"] = {"factor": s.factor, "low": s.low, "high": s.high, "original": s.original}
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale, "rot": rot}
                if m.chunk is not None:
                    mixer["mask"] = {"size": m.chunk}
                if m.kv_from is not None:
                    mixer["kv_from"] = m.kv_from
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "gate_cap": m.gate_cap}
            layers.append({"type": L.type, "mixer": mixer, "mlp": None if L.mlp is None else {"kind": "dense", "ff": L.mlp.ff}})
        d = {"architecture": "Paposun", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "residual_mult": self.residual_mult, "logit_scale": self.logit_scale, "layers": layers}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    # ------------------------------------------------------------------ the plan
    def plan(self) -> ModelPlan:
        c = self
        norm = PartSpec("rms_norm", {"size": c.width, "eps": c.norm_eps})
        blocks, order = [], []
        for i, L in enumerate(c.layers):
            m = L.mixer
            if isinstance(m, GatedAttention):
                scaling = None
                if m.rot_scaling is not None:
                    s = m.rot_scaling
                    scaling = {"factor": s.factor, "low": s.low, "high": s.high, "original": s.original}
                mixer = PartSpec("paged_attention", {
                    "hidden_size": c.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                    "value_dim": m.vdim, "softmax_scale": m.scale, "window": ("chunk", m.chunk) if m.chunk is not None else ("full", 0),
                    "position": PartSpec("rotary_halves", {"rotary_dim": m.rot_dims, "theta": m.rot_base, "scaling": scaling}),
                    "bias": True, "output_gate": True, "kv_shared": m.kv_from is not None})
                order.append(LayerCall(i, i if m.kv_from is None else m.kv_from, m.kv_from is None))
            else:
                mixer = PartSpec("mlstm", {"hidden_size": c.width, "num_heads": m.heads, "head_dim": m.dim,
                                           "value_dim": m.vdim, "gate_cap": m.gate_cap, "norm_eps": c.norm_eps})
                order.append(LayerCall(i, i, True))
            parts = {"mixer_norm": norm, "mixer": mixer, "mixer_out_norm": norm}
            if L.mlp is not None:
                parts.update(ffn_norm=norm, ffn_out_norm=norm, ffn=PartSpec("dense_activation", {
                    "hidden_size": c.width, "intermediate_size": L.mlp.ff, "activation": "gelu_tanh"}))
            blocks.append(BlockSpec("sandwich_residual", parts, {"residual_mult": c.residual_mult}))
        return ModelPlan(hidden_size=c.width, vocab_size=c.vocab, blocks=tuple(blocks), order=tuple(order),
                         final_norm=norm, tie_word_embeddings=True, max_positions=c.max_positions,
                         logit_scale=c.logit_scale).validate()

    # ------------------------------------------------------------------ tensor names
    def weight_bindings(self) -> list:
        c = self
        d = c.width
        B = WeightBinding
        out = [B("embed.weight", "embed", (c.vocab, d))]
        for i, L in enumerate(c.layers):
            s, t, m = f"l{i}.", f"layers.{i}.", L.mixer
            out += [B(t + "mixer_norm.weight", s + "norm1", (d,), init="ones"),
                    B(t + "mixer_out_norm.weight", s + "norm1b", (d,), init="ones")]
            if isinstance(m, GatedAttention):
                out += [B(t + "mixer.q_proj", s + "mix.q", (m.heads * m.dim, d)), B(t + "mixer.q_bias", s + "mix.q.b", (m.heads * m.dim,)),
                        B(t + "mixer.out_gate_proj", s + "mix.g", (m.heads * m.vdim, d)),
                        B(t + "mixer.o_proj", s + "mix.o", (d, m.heads * m.vdim)), B(t + "mixer.o_bias", s + "mix.o.b", (d,))]
                if m.kv_from is None:
                    out += [B(t + "mixer.k_proj", s + "mix.k", (m.kv_heads * m.dim, d)), B(t + "mixer.k_bias", s + "mix.k.b", (m.kv_heads * m.dim,)),
                            B(t + "mixer.v_proj", s + "mix.v", (m.kv_heads * m.vdim, d)), B(t + "mixer.v_bias", s + "mix.v.b", (m.kv_heads * m.vdim,))]
            else:
                H = m.heads
                out += [B(t + "mixer.q_proj", s + "mix.q", (H * m.dim, d)), B(t + "mixer.k_proj", s + "mix.k", (H * m.dim, d)),
                        B(t + "mixer.v_proj", s + "mix.v", (H * m.vdim, d)), B(t + "mixer.gate_proj", s + "mix.g", (H * m.vdim, d)),
                        B(t + "mixer.o_proj", s + "mix.o", (d, H * m.vdim)), B(t + "mixer.norm", s + "mix.norm", (H * m.vdim,), init="ones"),
                        B(t + "mixer.igate_proj", s + "mix.i", (H, d)), B(t + "mixer.igate_bias", s + "mix.i.b", (H,)),
                        B(t + "mixer.fgate_proj", s + "mix.f", (H, d)), B(t + "mixer.fgate_bias", s + "mix.f.b", (H,))]
            if L.mlp is not None:
                f = L.mlp.ff
                out += [B(t + "ffn_norm.weight", s + "norm2", (d,), init="ones"),
                        B(t + "ffn_out_norm.weight", s + "norm2b", (d,), init="ones"),
                        B(t + "ffn.up_proj", s + "mlp.up", (f, d)), B(t + "ffn.down_proj", s + "mlp.down", (d, f))]
        out.append(B("final_norm.weight", "final.norm", (d,), init="ones"))
        return out

    def unused_tensor_names(self) -> set:
        """What a file may carry for parts this configuration switches off: the feed-forward's norms of a layer without one."""
        names = set()
        for i, L in enumerate(self.layers):
            if L.mlp is None:
                names |= {f"l{i}.norm2", f"l{i}.norm2b"}
        return names

    checkpoint_prefixes = ("",)
    ignored_prefixes = ()
