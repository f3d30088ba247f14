"""Feed-forward parts: a dense SwiGLU and a mixture of experts whose router
weights the token before the expert, with an always-on shared expert.

Formulas: crates/spite-models/src/llama/llama4.rs:209-274 (dense, shared expert,
residual add) and crates/spite-models/src/moe.rs:53-194 (router, pre-scaled
input, SwiGLU experts, unweighted sum).
"""
from __future__ import annotations

import torch

from ..config.specs import ConfigError
from .base import FeedForward, ParamSpec, register_feed_forward


_SIDE_STREAMS: dict = {}      # one side stream per device, shared by the layers


@register_feed_forward("dense_swiglu")
class DenseSwiGLU(FeedForward):
    """h += down( silu(gate x) * (up x) )          (llama4.rs:257-271)"""
    graph_safe = True
    kernel_libraries = ("gemm_simt",)

    def __init__(self, ctx, hidden_size: int, intermediate_size: int):
        super().__init__(ctx)
        self.d, self.f = int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    def param_specs(self):
        return {"gate_proj": ParamSpec((self.f, self.d)), "up_proj": ParamSpec((self.f, self.d)),
                "down_proj": ParamSpec((self.d, self.f))}

    def bind(self, params):
        dt = self.ctx.dtype
        self.w_gate_up = torch.cat([params["gate_proj"].to(dt), params["up_proj"].to(dt)], 0).contiguous()
        self.w_down = params["down_proj"].to(dt).contiguous()

    def weight_bytes(self):
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def forward(self, x, h, batch):
        a = torch.empty((x.shape[0], self.f), dtype=x.dtype, device=x.device)
        self.k.linear_swiglu(x, self.w_gate_up, a)
        self.k.linear(a, self.w_down, h, accumulate=True)


@register_feed_forward("moe_sigmoid_prescaled")
class MoESigmoidPrescaled(FeedForward):
    """Top-k experts by raw router logit; the token is multiplied by sigmoid(logit)
    before its expert (moe.rs:172-176) and the experts' outputs are summed
    unweighted (moe.rs:188-191); a shared expert runs on the unscaled token
    (llama4.rs:231-256).

    `activation` says what an expert is: "swiglu", down(silu(gate x) * (up x)), or
    "relu2", down(relu(up x)^2) without a gate.  The shared expert has the same form
    and a size of its own (`shared_size`; 0: none).

    Because the expert's two input products are linear in the token, the factor
    is applied to their float32 sums in the epilogue: silu(s g) * (s u) with
    g, u the products of the unscaled token (relu(s u)^2 without a gate).  That equals
    the pre-scaled form and spares rounding the scaled token to the activation type.
    """
    graph_safe = True
    kernel_libraries = ("gemm_simt", "moe")

    ACTIVATIONS = ("swiglu", "relu2")

    def __init__(self, ctx, hidden_size: int, num_experts: int, top_k: int, expert_size: int,
                 shared_size: int = 0, activation: str = "swiglu"):
        super().__init__(ctx)
        if not 1 <= top_k <= num_experts:
            raise ConfigError(f"top_k {top_k} must lie in 1..{num_experts}")
        if activation not in self.ACTIVATIONS:
            raise ConfigError(f"unknown expert activation {activation!r}; known: {', '.join(self.ACTIVATIONS)}")
        self.activation = activation
        self.gated = activation == "swiglu"
        self.d, self.E, self.top_k = int(hidden_size), int(num_experts), int(top_k)
        self.f, self.fs = int(expert_size), int(shared_size)
        self.router = self.w_gate_up = self.w_down = self.ws_gate_up = self.ws_down = None
        self.router_beside_shared = True     # the router's two short kernels on a side stream beside the shared expert
        self.keep_router_logits = False      # `last_routing.logits` [tokens, experts] stays readable after a forward

    def param_specs(self):
        d, E, f, fs = self.d, self.E, self.f, self.fs
        specs = {"router": ParamSpec((E, d)), "experts_down": ParamSpec((E, d, f))}
        if self.gated:
            specs["experts_gate_up"] = ParamSpec((E, 2 * f, d))
        else:
            specs["experts_up"] = ParamSpec((E, f, d))
        if fs:
            if self.gated:
                specs["shared_gate_proj"] = ParamSpec((fs, d))
            specs.update({"shared_up_proj": ParamSpec((fs, d)), "shared_down_proj": ParamSpec((d, fs))})
        return specs

    def bind(self, params):
        dt = self.ctx.dtype
        # router logits are float32 sums of float32 weights in both kernel sets
        self.router = params["router"].to(torch.float32).contiguous()
        # (without a gate `w_gate_up` holds the up rows alone)
        self.w_gate_up = params["experts_gate_up" if self.gated else "experts_up"].to(dt).contiguous()
        self.w_down = params["experts_down"].to(dt).contiguous()
        if self.fs:
            first = [params["shared_gate_proj"].to(dt)] if self.gated else []
            self.ws_gate_up = torch.cat(first + [params["shared_up_proj"].to(dt)], 0).contiguous()
            self.ws_down = params["shared_down_proj"].to(dt).contiguous()

    def weight_bytes(self):
        n = self.w_gate_up.numel() + self.w_down.numel()
        if self.fs:
            n += self.ws_gate_up.numel() + self.ws_down.numel()
        return n * self.w_down.element_size() + self.router.numel() * 4

    def active_weight_bytes(self, n_distinct_experts: float) -> int:
        """Bytes a step reads when its tokens use `n_distinct_experts` experts (a mean over steps may be fractional)."""
        per = (self.w_gate_up.shape[1] * self.d + self.d * self.f) * self.w_down.element_size()
        n = int(per * n_distinct_experts) + self.router.numel() * 4
        if self.fs:
            n += (self.ws_gate_up.numel() + self.ws_down.numel()) * self.w_down.element_size()
        return n

    def forward(self, x, h, batch):
        k = self.k
        M = x.shape[0]
        # The shared expert needs only x, the routed experts need the router's answer first.  On a GPU
        # the router (two short kernels that leave the memory system idle) runs on a side stream beside
        # the shared expert's products; both streams meet before the routed experts.  The residual
        # stream gets the shared expert's output first, then the routed experts', on every path.
        side = self._side_stream(x) if self.fs else None
        if side is not None:
            main = torch.cuda.current_stream(x.device)
            forked = torch.cuda.Event()
            forked.record(main)
            with torch.cuda.stream(side):
                side.wait_event(forked)
                routing = k.moe_route(x, self.router, self.top_k, want_logits=self.keep_router_logits)
                routed = torch.cuda.Event()
                routed.record(side)
        else:
            routing = k.moe_route(x, self.router, self.top_k, want_logits=self.keep_router_logits)
        self.last_routing = routing
        if self.fs:
            a = torch.empty((M, self.fs), dtype=x.dtype, device=x.device)
            if self.gated:
                k.linear_swiglu(x, self.ws_gate_up, a)
            else:
                k.linear(x, self.ws_gate_up, a, activation=self.activation)
            k.linear(a, self.ws_down, h, accumulate=True)
        if side is not None:
            main.wait_event(routed)
            for t in (routing.expert_ids, routing.weights, routing.offsets, routing.sorted_rows, routing.logits):
                if t is not None:
                    t.record_stream(main)                        # made on the side stream, read on this one
        for slot in range(self.top_k):
            a = torch.empty((M, self.f), dtype=x.dtype, device=x.device)
            if self.gated:
                k.grouped_linear_swiglu(x, self.w_gate_up, routing.sorted_rows[slot], routing.offsets[slot],
                                        routing.weights[slot], a)
            else:
                k.grouped_linear_act(x, self.w_gate_up, routing.sorted_rows[slot], routing.offsets[slot],
                                     routing.weights[slot], a, activation=self.activation)
            k.grouped_linear_accumulate(a, self.w_down, routing.sorted_rows[slot], routing.offsets[slot], h)

    def _side_stream(self, x):
        if not x.is_cuda or not self.router_beside_shared:
            return None
        side = _SIDE_STREAMS.get(x.device)
        if side is None:
            side = _SIDE_STREAMS[x.device] = torch.cuda.Stream(device=x.device)
        return side


@register_feed_forward("dense_activation")
class DenseActivation(FeedForward):
    """h += down( act(up x) ) without a gate; `activation` "relu2": act(z) = relu(z)^2; "gelu_tanh":
    act(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))); applied to the float32 sums of the first product
    before they are rounded."""
    graph_safe = True
    can_store = True
    kernel_libraries = ("gemm_simt",)

    ACTIVATIONS = ("relu2", "gelu_tanh")

    def __init__(self, ctx, hidden_size: int, intermediate_size: int, activation: str = "relu2"):
        super().__init__(ctx)
        if activation not in self.ACTIVATIONS:
            raise ConfigError(f"unknown activation {activation!r}; known: {', '.join(self.ACTIVATIONS)}")
        self.d, self.f, self.activation = int(hidden_size), int(intermediate_size), activation
        self.w_up = self.w_down = None

    def param_specs(self):
        return {"up_proj": ParamSpec((self.f, self.d)), "down_proj": ParamSpec((self.d, self.f))}

    def bind(self, params):
        dt = self.ctx.dtype
        self.w_up = params["up_proj"].to(dt).contiguous()
        self.w_down = params["down_proj"].to(dt).contiguous()

    def weight_bytes(self):
        return (self.w_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def forward(self, x, h, batch, accumulate=True):
        a = torch.empty((x.shape[0], self.f), dtype=x.dtype, device=x.device)
        self.k.linear(x, self.w_up, a, activation=self.activation)
        self.k.linear(a, self.w_down, h, accumulate=accumulate)


@register_feed_forward("moe_softmax_topk")
class MoESoftmaxTopK(FeedForward):
    """Mixture of gated experts whose router weights the experts' outputs:

        s = softmax(W_r x) over all experts (float32);  the `top_k` largest are chosen;
        w_e = s_e / (sum of the chosen s + 1e-20);  h += sum_e w_e * down_e( silu(gate_e x) * (up_e x) )

    The weight multiplies the float32 sums of the expert's last product as they are added to the residual
    stream, so no rounded intermediate carries it.

    Variants, all parameters: `renormalize` False leaves the chosen shares as they are (w_e = s_e); `choice_bias` adds a
    learned constant per expert (`choice_bias` [experts]) to the shares for the choice alone, the weights stay the
    shares; `identity_experts` n: the router has n outputs more than there are experts, and a token that draws one of
    those gets its own input back, times the weight (such an expert has no tensors)."""
    graph_safe = True
    can_store = True
    kernel_libraries = ("gemm_simt", "moe")

    def __init__(self, ctx, hidden_size: int, num_experts: int, top_k: int, expert_size: int, renormalize: bool = True,
                 choice_bias: bool = False, identity_experts: int = 0):
        super().__init__(ctx)
        self.identity = int(identity_experts)
        if self.identity < 0 or num_experts < 0 or num_experts + self.identity < 1:
            raise ConfigError("a mixture needs at least one expert")
        if not 1 <= top_k <= num_experts + self.identity:
            raise ConfigError(f"top_k {top_k} must lie in 1..{num_experts + self.identity}")
        self.renormalize, self.has_choice_bias = bool(renormalize), bool(choice_bias)
        if self.renormalize and (self.has_choice_bias or self.identity):
            raise ConfigError("a choice bias and identity experts go with weights that are not renormalised")
        self.d, self.E, self.top_k, self.f = int(hidden_size), int(num_experts), int(top_k), int(expert_size)
        self.router = self.w_gate_up = self.w_down = self.choice_bias = None
        self.keep_router_logits = False      # `last_routing.logits` [tokens, experts] stays readable after a forward

    def param_specs(self):
        d, E, f = self.d, self.E, self.f
        specs = {"router": ParamSpec((E + self.identity, d)), "experts_gate": ParamSpec((E, f, d)),
                 "experts_up": ParamSpec((E, f, d)), "experts_down": ParamSpec((E, d, f))}
        if self.has_choice_bias:
            specs["choice_bias"] = ParamSpec((E + self.identity,))
        return specs

    def bind(self, params):
        dt = self.ctx.dtype
        self.router = params["router"].to(torch.float32).contiguous()        # float32 sums of float32 weights
        if self.renormalize:
            self.choice_bias = None
        elif self.has_choice_bias:
            self.choice_bias = params["choice_bias"].to(torch.float32).contiguous()
        else:
            self.choice_bias = torch.zeros((self.E + self.identity,), dtype=torch.float32, device=self.router.device)
        self.w_gate_up = torch.cat([params["experts_gate"].to(dt), params["experts_up"].to(dt)], 1).contiguous()
        self.w_down = params["experts_down"].to(dt).contiguous()

    def weight_bytes(self):
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size() + self.router.numel() * 4

    def active_weight_bytes(self, n_distinct_experts: float) -> int:
        """Bytes a step reads when its tokens use `n_distinct_experts` experts (a mean over steps may be fractional)."""
        per = 3 * self.f * self.d * self.w_down.element_size()
        return int(per * n_distinct_experts) + self.router.numel() * 4

    def forward(self, x, h, batch, accumulate=True):
        k = self.k
        M = x.shape[0]
        if self.renormalize:
            routing = k.moe_route(x, self.router, self.top_k, want_logits=self.keep_router_logits, scoring="softmax_renorm")
        else:
            routing = k.moe_route(x, self.router, self.top_k, want_logits=self.keep_router_logits, scoring="softmax_biased",
                                  choice_bias=self.choice_bias)
        self.last_routing = routing
        if self.identity:
            # the tokens that drew an identity expert get their input back, times the weight; without `accumulate` this
            # also starts every row of the sum that the experts then add to
            k.moe_identity(x, routing, self.E, h, accumulate=accumulate)
        elif not accumulate:
            h.zero_()
        if not self.E:
            return
        for slot in range(self.top_k):
            a = torch.empty((M, self.f), dtype=x.dtype, device=x.device)
            # (the experts' ranges of the sorted order come first; the places behind them belong to identity experts)
            offsets = routing.offsets[slot][:self.E + 1]
            k.grouped_linear_swiglu(x, self.w_gate_up, routing.sorted_rows[slot], offsets, None, a)
            k.grouped_linear_accumulate(a, self.w_down, routing.sorted_rows[slot], offsets, h,
                                        row_scale=routing.sorted_weights[slot])
