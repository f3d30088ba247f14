"""Typed configuration of the Gapevik decoder, read from its config.json.

The file lists the layers one by one: `layers[i]` gives the layer's `type` (which mixer it has), the mixer's sizes
and constants (`mixer`) and its feed-forward (`mlp`, or null for none).  A layer with `weights_of: j` has no tensors
of its own: it runs layer j's mixer, feed-forward and norms (with j's sizes and constants) on a cache and state of
its own.  `vocab`, `width`, `norm.eps`, `residual_mult` and `embedding.scale` are the model's own; `max_positions` and
`eos_token_id` are optional.  Every size and every constant that the file gives is read from it; what the design fixes
is stated in `plan()`:

  * a sublayer reads the residual stream itself and is normed behind: x += residual_mult * norm(sublayer(x));
  * mixer `attention`: grouped-query attention; q, k and v pass a causal convolution over time of `conv` taps right
    behind their projections; q and k heads are RMS-normed with a gain before the rotation of neighbouring pairs of
    their first `rot.dims` elements; scores times `scale`, squashed to softcap * tanh(s / softcap); sight limited to
    the query's chunk of `mask.size` positions; head h's output times sigmoid(w_h . x);
  * mixer `latent_attention`: queries through a normed latent of `q_rank`, keys and values of all heads from one normed
    latent of `kv_rank` per position plus one rotated key part of `rot_dim` elements that the heads share (element i
    paired with element i + rot_dim / 2); sight limited to the last `mask.size` positions; a learned sink per head in
    the softmax's sum; the same gate per head;
  * mixer `delta`: the gated delta rule of `parts/delta.py` with a convolution of `conv` taps, q scaled by dim^-1/2;
  * feed-forward `moe`: gated SiLU experts chosen by softmax share plus a learned correction, weighted by the share
    alone; the router's last `router.identity` outputs stand for experts that return their input;
  * RMS norms; the output head is the embedding table (without the embedding's scale).

Tensor names: `embed`, `final.norm`, and per layer with weights of its own `l<i>.norm1`, `l<i>.norm2`,
`l<i>.mix.*` (attention: q, k, v, their `.conv` and q/k `.norm`, g, o; latent_attention: dq, dq.norm, uq, dkv, dkv.norm,
uk, uv, sink, g, o; delta: q, k, v, their `.conv`, b, a, A_log, dt_bias, norm, g, o), `l<i>.mlp.e<j>.{gate,up,down}`,
`l<i>.mlp.router`, `l<i>.mlp.correction`; linear weights `[out, in]`.
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
class ConvAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float
    chunk: Optional[int]           # mask.size; None: every earlier position is visible
    softcap: Optional[float]
    conv: Optional[int]            # taps; None: no convolution


@dataclass(frozen=True)
class WindowedLatentAttention:
    heads: int
    dim: int                       # unrotated part of a query/key head
    rot_dim: int                   # rotated part, shared by the heads on the key's side
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    window: Optional[int]          # mask.size; None: every earlier position is visible


@dataclass(frozen=True)
class DeltaRule:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class ExpertMixture:
    ff: int
    experts: int
    identity: int
    top: int


@dataclass(frozen=True)
class GapevikLayer:
    type: str
    mixer: object                  # ConvAttention | WindowedLatentAttention | DeltaRule
    mlp: Optional[ExpertMixture]
    weights_of: Optional[int] = None


@register_architecture("Gapevik")
@dataclass(frozen=True)
class GapevikConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    embedding_scale: float
    layers: tuple
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Optional[tuple] = None

    MIXERS = ("attention", "latent_attention", "delta")

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "GapevikConfig":
        layers = []
        for i, L in enumerate(_need(raw, "layers", "")):
            at = f"layers[{i}]."
            kind = _need(L, "type", at)
            m = _need(L, "mixer", at)
            mat = at + "mixer."
            size = int(_need(m["mask"], "size", mat + "mask.")) if m.get("mask") else None
            if kind == "attention":
                rot = _need(m, "rot", mat)
                mixer = ConvAttention(
                    heads=int(_need(m, "heads", mat)), kv_heads=int(_need(m, "kv_heads", mat)), dim=int(_need(m, "dim", mat)),
                    vdim=int(_need(m, "vdim", mat)), scale=float(_need(m, "scale", mat)),
                    rot_dims=int(_need(rot, "dims", mat + "rot.")), rot_base=float(_need(rot, "base", mat + "rot.")),
                    chunk=size, softcap=None if m.get("softcap") is None else float(m["softcap"]),
                    conv=None if m.get("conv") is None else int(m["conv"]))
            elif kind == "latent_attention":
                rot = _need(m, "rot", mat)
                mixer = WindowedLatentAttention(
                    heads=int(_need(m, "heads", mat)), dim=int(_need(m, "dim", mat)), rot_dim=int(_need(m, "rot_dim", mat)),
                    vdim=int(_need(m, "vdim", mat)), q_rank=int(_need(m, "q_rank", mat)), kv_rank=int(_need(m, "kv_rank", mat)),
                    scale=float(_need(m, "scale", mat)), rot_base=float(_need(rot, "base", mat + "rot.")), window=size)
                if int(_need(rot, "dims", mat + "rot.")) != mixer.rot_dim:
                    raise ConfigError(f"{mat}rot.dims must equal rot_dim ({mixer.rot_dim}): the rotated part rotates as a whole")
            elif kind == "delta":
                mixer = DeltaRule(heads=int(_need(m, "heads", mat)), kv_heads=int(_need(m, "kv_heads", mat)),
                                  dim=int(_need(m, "dim", mat)), vdim=int(_need(m, "vdim", mat)), conv=int(_need(m, "conv", mat)))
            else:
                raise ConfigError(f"config.json: {at}type {kind!r} is not a mixer of this design (known: {', '.join(cls.MIXERS)})")
            f = L.get("mlp")
            mlp = None
            if f is not None:
                fk = _need(f, "kind", at + "mlp.")
                if fk != "moe":
                    raise ConfigError(f"config.json: {at}mlp.kind {fk!r} is unknown (moe)")
                r = _need(f, "router", at + "mlp.")
                mlp = ExpertMixture(ff=int(_need(_need(f, "expert", at + "mlp."), "ff", at + "mlp.expert.")),
                                    experts=int(_need(r, "experts", at + "mlp.router.")), identity=int(r.get("identity") or 0),
                                    top=int(_need(r, "top", at + "mlp.router.")))
            src = L.get("weights_of")
            layers.append(GapevikLayer(kind, mixer, mlp, None if src is None else int(src)))
        eos = raw.get("eos_token_id")
        if isinstance(eos, int):
            eos = (eos,)
        elif eos is not None:
            eos = tuple(int(x) for x in eos)
        emb = raw.get("embedding") or {}
        cfg = cls(vocab=int(_need(raw, "vocab", "")), width=int(_need(raw, "width", "")),
                  norm_eps=float(_need(_need(raw, "norm", ""), "eps", "norm.")),
                  residual_mult=float(_need(raw, "residual_mult", "")), embedding_scale=float(emb.get("scale", 1.0)),
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
            if isinstance(m, ConvAttention):
                if min(m.heads, m.kv_heads, m.dim, m.vdim, m.chunk if m.chunk is not None else 1) < 1:
                    raise ConfigError(f"{at}: heads, kv_heads, dim, vdim and mask.size must be positive")
                if m.heads % m.kv_heads:
                    raise ConfigError(f"{at}: {m.heads} heads are no multiple of {m.kv_heads} kv_heads")
                if not m.scale > 0 or not m.rot_base > 0:
                    raise ConfigError(f"{at}: scale and rot.base must be positive")
                if m.rot_dims < 2 or m.rot_dims % 2 or m.rot_dims > m.dim:
                    raise ConfigError(f"{at}: rot.dims {m.rot_dims} must be even and lie in 2..dim ({m.dim})")
                if m.softcap is not None and not m.softcap > 0:
                    raise ConfigError(f"{at}: softcap must be positive")
                if m.conv is not None and not 1 <= m.conv <= 8:
                    raise ConfigError(f"{at}: conv {m.conv} must lie in 1..8")
            elif isinstance(m, WindowedLatentAttention):
                if min(m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, m.window if m.window is not None else 1) < 1:
                    raise ConfigError(f"{at}: sizes and mask.size must be positive")
                if m.rot_dim % 2:
                    raise ConfigError(f"{at}: rot_dim {m.rot_dim} must be even")
                if not m.scale > 0 or not m.rot_base > 0:
                    raise ConfigError(f"{at}: scale and rot.base must be positive")
            else:
                if min(m.heads, m.kv_heads, m.dim, m.vdim) < 1 or m.heads % m.kv_heads:
                    raise ConfigError(f"{at}: heads, kv_heads, dim and vdim must be positive, heads a multiple of kv_heads")
                if not 1 <= m.conv <= 8:
                    raise ConfigError(f"{at}: conv {m.conv} must lie in 1..8")
            f = L.mlp
            if f is not None:
                if f.ff < 1 or f.experts < 0 or f.identity < 0 or f.experts + f.identity < 1:
                    raise ConfigError(f"layers[{i}].mlp: sizes must be positive")
                if not 1 <= f.top <= f.experts + f.identity:
                    raise ConfigError(f"layers[{i}].mlp.router.top {f.top} must lie in 1..{f.experts + f.identity}")
            if L.weights_of is not None:
                j = L.weights_of
                if not 0 <= j < len(c.layers) or j == i or c.layers[j].weights_of is not None:
                    raise ConfigError(f"layers[{i}].weights_of {j}: not another layer with weights of its own")
                if c.layers[j].type != L.type:
                    raise ConfigError(f"layers[{i}].weights_of {j}: that layer is a {c.layers[j].type} layer, this one {L.type}")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        layers = []
        for L in self.layers:
            m = L.mixer
            if isinstance(m, ConvAttention):
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                         "rot": {"base": m.rot_base, "dims": m.rot_dims}}
                if m.chunk is not None:
                    mixer["mask"] = {"size": m.chunk}
                if m.softcap is not None:
                    mixer["softcap"] = m.softcap
                if m.conv is not None:
                    mixer["conv"] = m.conv
            elif isinstance(m, WindowedLatentAttention):
                mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "q_rank": m.q_rank,
                         "kv_rank": m.kv_rank, "scale": m.scale, "rot": {"base": m.rot_base, "dims": m.rot_dim}}
                if m.window is not None:
                    mixer["mask"] = {"size": m.window}
            else:
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv}
            f = L.mlp
            entry = {"type": L.type, "mixer": mixer,
                     "mlp": None if f is None else {"kind": "moe", "expert": {"ff": f.ff},
                                                    "router": {"experts": f.experts, "identity": f.identity, "top": f.top}}}
            if L.weights_of is not None:
                entry["weights_of"] = L.weights_of
            layers.append(entry)
        d = {"architecture": "Gapevik", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "residual_mult": self.residual_mult, "embedding": {"scale": self.embedding_scale}, "layers": layers}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    # ------------------------------------------------------------------ the plan
    def owners(self) -> list:
        """The layers that have weights of their own, in order; `block_of()[i]` is the place of layer i's weights there."""
        return [i for i, L in enumerate(self.layers) if L.weights_of is None]

    def block_of(self) -> list:
        own = {i: b for b, i in enumerate(self.owners())}
        return [own[i if L.weights_of is None else L.weights_of] for i, L in enumerate(self.layers)]

    def plan(self) -> ModelPlan:
        c = self
        norm = PartSpec("rms_norm", {"size": c.width, "eps": c.norm_eps})
        blocks = []
        for i in c.owners():
            L = c.layers[i]
            m = L.mixer
            if isinstance(m, ConvAttention):
                mixer = PartSpec("paged_attention", {
                    "hidden_size": c.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                    "value_dim": m.vdim, "softmax_scale": m.scale,
                    "window": ("chunk", m.chunk) if m.chunk is not None else ("full", 0),
                    "position": PartSpec("rotary_yarn", {"rotary_dim": m.rot_dims, "theta": m.rot_base}),
                    "qk_norm_eps": c.norm_eps, "qk_norm_gain": True, "qk_norm_before_rotation": True, "head_gate": True,
                    "conv_taps": m.conv, "score_softcap": m.softcap})
            elif isinstance(m, WindowedLatentAttention):
                mixer = PartSpec("latent_attention", {
                    "hidden_size": c.width, "num_heads": m.heads, "head_dim": m.dim, "rotary_dim": m.rot_dim,
                    "value_dim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank, "softmax_scale": m.scale,
                    "norm_eps": c.norm_eps, "head_gate": True, "head_sinks": True,
                    "window": ("sliding", m.window) if m.window is not None else ("full", 0),
                    "position": PartSpec("rotary_halves", {"rotary_dim": m.rot_dim, "theta": m.rot_base})})
            else:
                mixer = PartSpec("gated_delta", {
                    "hidden_size": c.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                    "value_dim": m.vdim, "conv_taps": m.conv, "norm_eps": c.norm_eps})
            parts = {"mixer": mixer, "mixer_out_norm": norm}
            if L.mlp is not None:
                f = L.mlp
                parts.update(ffn_out_norm=norm, ffn=PartSpec("moe_softmax_topk", {
                    "hidden_size": c.width, "num_experts": f.experts, "top_k": f.top, "expert_size": f.ff,
                    "renormalize": False, "choice_bias": True, "identity_experts": f.identity}))
            blocks.append(BlockSpec("postnorm_residual", parts, {"residual_mult": c.residual_mult}))
        # a layer that borrows weights runs the lender's block on a cache and state of its own
        order = tuple(LayerCall(b, i, True) for i, b in enumerate(c.block_of()))
        return ModelPlan(hidden_size=c.width, vocab_size=c.vocab, blocks=tuple(blocks), order=order,
                         final_norm=norm, tie_word_embeddings=True, max_positions=c.max_positions,
                         embedding_scale=c.embedding_scale).validate()

    # ------------------------------------------------------------------ tensor names
    def weight_bindings(self) -> list:
        c = self
        d = c.width
        B = WeightBinding
        out = [B("embed.weight", "embed", (c.vocab, d))]
        for b, i in enumerate(c.owners()):
            L = c.layers[i]
            s, t, m = f"l{i}.", f"layers.{b}.", L.mixer
            out.append(B(t + "mixer_out_norm.weight", s + "norm1", (d,), init="ones"))
            x, y = t + "mixer.", s + "mix."
            if isinstance(m, ConvAttention):
                out += [B(x + "q_proj", y + "q", (m.heads * m.dim, d)), B(x + "k_proj", y + "k", (m.kv_heads * m.dim, d)),
                        B(x + "v_proj", y + "v", (m.kv_heads * m.vdim, d)),
                        B(x + "q_norm", y + "q.norm", (m.dim,), init="ones"), B(x + "k_norm", y + "k.norm", (m.dim,), init="ones"),
                        B(x + "gate_proj", y + "g", (m.heads, d)), B(x + "o_proj", y + "o", (d, m.heads * m.vdim))]
                if m.conv is not None:
                    out += [B(x + "q_conv", y + "q.conv", (m.heads * m.dim, m.conv)),
                            B(x + "k_conv", y + "k.conv", (m.kv_heads * m.dim, m.conv)),
                            B(x + "v_conv", y + "v.conv", (m.kv_heads * m.vdim, m.conv))]
            elif isinstance(m, WindowedLatentAttention):
                out += [B(x + "q_down", y + "dq", (m.q_rank, d)), B(x + "q_latent_norm", y + "dq.norm", (m.q_rank,), init="ones"),
                        B(x + "q_up", y + "uq", (m.heads * (m.dim + m.rot_dim), m.q_rank)),
                        B(x + "kv_down", y + "dkv", (m.kv_rank + m.rot_dim, d)),
                        B(x + "kv_latent_norm", y + "dkv.norm", (m.kv_rank,), init="ones"),
                        B(x + "k_up", y + "uk", (m.heads * m.dim, m.kv_rank)), B(x + "v_up", y + "uv", (m.heads * m.vdim, m.kv_rank)),
                        B(x + "sinks", y + "sink", (m.heads,)), B(x + "gate_proj", y + "g", (m.heads, d)),
                        B(x + "o_proj", y + "o", (d, m.heads * m.vdim))]
            else:
                G, H = m.kv_heads, m.heads
                out += [B(x + "q_proj", y + "q", (G * m.dim, d)), B(x + "k_proj", y + "k", (G * m.dim, d)),
                        B(x + "v_proj", y + "v", (H * m.vdim, d)), B(x + "q_conv", y + "q.conv", (G * m.dim, m.conv)),
                        B(x + "k_conv", y + "k.conv", (G * m.dim, m.conv)), B(x + "v_conv", y + "v.conv", (H * m.vdim, m.conv)),
                        B(x + "beta_proj", y + "b", (H, d)), B(x + "decay_proj", y + "a", (H, d)),
                        B(x + "a_log", y + "A_log", (H,)), B(x + "dt_bias", y + "dt_bias", (H,)),
                        B(x + "gate_proj", y + "g", (H * m.vdim, d)), B(x + "norm", y + "norm", (m.vdim,), init="ones"),
                        B(x + "o_proj", y + "o", (d, H * m.vdim))]
            if L.mlp is not None:
                f = L.mlp
                n = f.experts + f.identity
                out += [B(t + "ffn_out_norm.weight", s + "norm2", (d,), init="ones"),
                        B(t + "ffn.router", s + "mlp.router", (n, d)), B(t + "ffn.choice_bias", s + "mlp.correction", (n,)),
                        B(t + "ffn.experts_gate", tuple(f"{s}mlp.e{e}.gate" for e in range(f.experts)), (f.ff, d)),
                        B(t + "ffn.experts_up", tuple(f"{s}mlp.e{e}.up" for e in range(f.experts)), (f.ff, d)),
                        B(t + "ffn.experts_down", tuple(f"{s}mlp.e{e}.down" for e in range(f.experts)), (d, f.ff))]
        out.append(B("final_norm.weight", "final.norm", (d,), init="ones"))
        return out

    def unused_tensor_names(self) -> set:
        """What a file may carry for parts this configuration switches off: the feed-forward's norm of a layer without one."""
        return {f"l{i}.norm2" for i in self.owners() if self.layers[i].mlp is None}

    checkpoint_prefixes = ("",)
    ignored_prefixes = ()
