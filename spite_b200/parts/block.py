"""How the parts of one layer are arranged.

`prenorm_residual` (crates/spite-models/src/llama/llama4.rs:126-127,202-211,272-274):
    h += mixer(norm_a(h));  h += feed_forward(norm_b(h))      (the second half may be left out)
The residual stream h stays float32; the sums are done by the epilogues of the
mixer's and the feed-forward's last products.

`sandwich_residual`: a norm before and a norm behind every sublayer, and a factor on what joins the stream:
    h += mult * norm_c(mixer(norm_a(h)));  h += mult * norm_d(feed_forward(norm_b(h)))
The sublayer's output goes to a float32 buffer of its own; one kernel norms it, adds it to the stream and, where
a feed-forward follows, writes the norm that the feed-forward reads.

`postnorm_residual`: no norm in front of a sublayer, one behind it, and a factor on what joins the stream:
    h += mult * norm_c(mixer(h));  h += mult * norm_d(feed_forward(h))
The sublayers read the stream itself (in the activation type: a copy for bfloat16 products, the stream in place for
float32 ones); the kernel that norms the mixer's output and adds it to the stream also writes the copy that the
feed-forward reads.
"""
from __future__ import annotations

import torch

from ..config.specs import ConfigError
from .base import Block, register_block


@register_block("prenorm_residual")
class PreNormResidual(Block):
    graph_safe = True
    places = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "feed_forward"}
    optional = ("ffn_norm", "ffn")           # a layer may be a mixer alone

    def forward(self, h, batch, cache):
        x = torch.empty(h.shape, dtype=self.ctx.dtype, device=h.device)
        self.mixer_norm.forward(h, x)
        self.mixer.forward(x, h, batch, cache)
        if self.ffn is not None:
            self.ffn_norm.forward(h, x)
            self.ffn.forward(x, h, batch)


@register_block("sandwich_residual")
class SandwichResidual(Block):
    graph_safe = True
    places = {"mixer_norm": "norm", "mixer": "mixer", "mixer_out_norm": "norm",
              "ffn_norm": "norm", "ffn": "feed_forward", "ffn_out_norm": "norm"}
    optional = ("ffn_norm", "ffn", "ffn_out_norm")

    def __init__(self, ctx, spec, residual_mult: float = 1.0):
        super().__init__(ctx, spec)
        self.mult = float(residual_mult)
        if self.ffn is not None and (self.ffn_norm is None or self.ffn_out_norm is None):
            raise ConfigError("sandwich_residual: a feed-forward needs the norm before it and the norm behind it")
        for n in (self.mixer_norm, self.mixer_out_norm, self.ffn_norm, self.ffn_out_norm):
            if n is not None and (n.kind != "rms_norm" or n.eps != self.mixer_norm.eps):
                raise ConfigError("sandwich_residual fuses its norms into one kernel: RMS norms with one epsilon")

    def _run(self, part, x, y, *args):
        if part.can_store:
            part.forward(x, y, *args, accumulate=False)
        else:
            y.zero_()
            part.forward(x, y, *args)

    def forward(self, h, batch, cache):
        k = self.k
        x = torch.empty(h.shape, dtype=self.ctx.dtype, device=h.device)
        y = torch.empty_like(h)
        self.mixer_norm.forward(h, x)
        self._run(self.mixer, x, y, batch, cache)
        eps = self.mixer_norm.eps
        if self.ffn is None:
            k.rms_norm_residual(y, self.mixer_out_norm.weight, eps, self.mult, h)
            return
        k.rms_norm_residual(y, self.mixer_out_norm.weight, eps, self.mult, h, next_gain=self.ffn_norm.weight, next_out=x)
        self._run(self.ffn, x, y, batch)
        k.rms_norm_residual(y, self.ffn_out_norm.weight, eps, self.mult, h)


@register_block("postnorm_residual")
class PostNormResidual(Block):
    graph_safe = True
    places = {"mixer": "mixer", "mixer_out_norm": "norm", "ffn": "feed_forward", "ffn_out_norm": "norm"}
    optional = ("ffn", "ffn_out_norm")

    def __init__(self, ctx, spec, residual_mult: float = 1.0):
        super().__init__(ctx, spec)
        self.mult = float(residual_mult)
        if self.ffn is not None and self.ffn_out_norm is None:
            raise ConfigError("postnorm_residual: a feed-forward needs the norm behind it")
        for n in (self.mixer_out_norm, self.ffn_out_norm):
            if n is not None and (n.kind != "rms_norm" or n.eps != self.mixer_out_norm.eps):
                raise ConfigError("postnorm_residual fuses its norms into one kernel: RMS norms with one epsilon")

    _run = SandwichResidual._run

    def forward(self, h, batch, cache):
        k = self.k
        same = self.ctx.dtype == torch.float32        # float32 products read the stream in place
        x = h if same else torch.empty(h.shape, dtype=self.ctx.dtype, device=h.device)
        y = torch.empty_like(h)
        if not same:
            k.cast_rows(h, x)
        self._run(self.mixer, x, y, batch, cache)
        eps = self.mixer_out_norm.eps
        if self.ffn is None:
            k.rms_norm_residual(y, self.mixer_out_norm.weight, eps, self.mult, h)
            return
        k.rms_norm_residual(y, self.mixer_out_norm.weight, eps, self.mult, h, next_out=None if same else x)
        self._run(self.ffn, x, y, batch)
        k.rms_norm_residual(y, self.ffn_out_norm.weight, eps, self.mult, h)
