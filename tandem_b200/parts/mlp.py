"""Gated feed-forward (SwiGLU): down(act(gate(x)) * up(x)) with gate and up as one product
(12vivi/tandem python/tandem/layers/mlp.py:23-44; rows [gate | up] as python/tandem/models/loader.py:52-53
stacks them), and the plain two-layer feed-forward down(act(up(x) + b) ) + b with optional biases."""

from __future__ import annotations

import torch

from tandem_b200.config.model_config import ConfigError
from tandem_b200.config.plan import DenseMLPSpec, GatedMLPSpec, ParamSpec, RoutedMLPSpec, WeightSource
from tandem_b200.kernels import deferred, ops
from tandem_b200.parts.base import FeedForward, StepContext


class GatedMLP(FeedForward):
    takes_deferred = True  # x may be a norm whose scale is pending; with ``defer`` the last product may stay pending

    _SUFFIX = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}

    @classmethod
    def params(cls, spec: GatedMLPSpec) -> dict:
        H, I, p = spec.hidden_size, spec.intermediate_size, spec.prefix
        name = {local: f"{p}.{dict(spec.names).get(local, suffix)}" for local, suffix in cls._SUFFIX.items()}
        return {
            "gate_up": ParamSpec((2 * I, H), (WeightSource(name["gate"], 0, I), WeightSource(name["up"], I, I))),
            "down": ParamSpec((H, I), (WeightSource(name["down"]),)),
        }

    def __init__(self, spec: GatedMLPSpec, weights: dict, dtype: torch.dtype, device) -> None:
        if spec.activation != "silu":
            raise ConfigError(f"gated_mlp has no activation {spec.activation!r} (only silu)")
        self.gate_up = weights["gate_up"]
        self.down = weights["down"]
        self.float32_output = spec.float32_output

    def forward(self, x, ctx: StepContext, defer: bool = False):
        if self.float32_output:
            return ops.linear(ops.gated_linear(x, self.gate_up), self.down, out_dtype=torch.float32)
        return ops.linear(ops.gated_linear(x, self.gate_up), self.down, defer=defer)


class DenseMLP(FeedForward):
    """down(act(up(x) + up_bias)) + down_bias.  The first product comes back in float32, bias and
    activation are one kernel that rounds once; the second may come back with its bias not yet added."""

    takes_deferred = True
    _SUFFIX = {"up": "up", "down": "down", "up_bias": "up.b", "down_bias": "down.b"}

    @classmethod
    def _name(cls, spec, local: str) -> str:
        return f"{spec.prefix}.{dict(spec.names).get(local, cls._SUFFIX[local])}"

    @classmethod
    def params(cls, spec: DenseMLPSpec) -> dict:
        H, I = spec.hidden_size, spec.intermediate_size
        out = {"up": ParamSpec((I, H), (WeightSource(cls._name(spec, "up")),)),
               "down": ParamSpec((H, I), (WeightSource(cls._name(spec, "down")),))}
        if spec.bias:
            out["up_bias"] = ParamSpec((I,), (WeightSource(cls._name(spec, "up_bias")),), role="vector")
            out["down_bias"] = ParamSpec((H,), (WeightSource(cls._name(spec, "down_bias")),), role="vector")
        return out

    def __init__(self, spec: DenseMLPSpec, weights: dict, dtype: torch.dtype, device) -> None:
        if spec.activation not in ("gelu_tanh", "silu", "relu2", "none"):
            raise ConfigError(f"dense_mlp has no activation {spec.activation!r} (gelu_tanh, silu, relu2 or none)")
        self.activation = spec.activation
        self.up, self.down = weights["up"], weights["down"]
        self.up_bias, self.down_bias = weights.get("up_bias"), weights.get("down_bias")

    def forward(self, x, ctx: StepContext, defer: bool = False):
        x = deferred.tensor(x)
        a = ops.bias_act(ops.linear(x, self.up, out_dtype=torch.float32), self.up_bias, self.activation, ctx.dtype)
        y = ops.linear(a, self.down, out_dtype=torch.float32)
        if defer:
            return deferred.Unsummed(y, self.down_bias, ctx.dtype)
        return ops.bias_act(y, self.down_bias, "none", ctx.dtype)


class RoutedMLP(FeedForward):
    """Experts chosen by a router (see :class:`~tandem_b200.config.plan.RoutedMLPSpec`).  The router's logits
    come from the package's product in float32; one kernel scores and chooses; the experts' weights are held
    stacked ([E, 2 F, H] with an expert's gate rows in front of its up rows, or [E, F, H] for experts without a
    gate; [E, H, F]) and run by the kernels of ``csrc/moe.cu``.  Router outputs behind the experts' stand for
    identity experts, which have no tensors.  With ``router`` "token_table" there is no router: a table names every
    token id's experts and all weights are 1 / top_k.  A shared expert (``shared_intermediate_size``) is a dense
    feed-forward of the same activation that every token passes; its output is added.  Returns float32."""

    @staticmethod
    def params(spec: RoutedMLPSpec) -> dict:
        H, F, E, p = spec.hidden_size, spec.intermediate_size, spec.num_experts, spec.prefix
        outputs = E + spec.identity_experts
        rows = 2 * F if spec.gated else F
        first, down = [], []
        for e in range(E):
            if spec.gated:
                first.append(WeightSource(f"{p}.e{e}.gate", rows * e, F))
            first.append(WeightSource(f"{p}.e{e}.up", rows * e + (F if spec.gated else 0), F))
            down.append(WeightSource(f"{p}.e{e}.down", H * e, H))
        out = {"gate_up": ParamSpec((rows * E, H), tuple(first)), "down": ParamSpec((H * E, F), tuple(down))}
        if spec.router == "token_table":
            out["table"] = ParamSpec((spec.vocab_size, spec.top_k), (WeightSource(f"{p}.{spec.table}"),), role="table_int")
        else:
            out["router"] = ParamSpec((outputs, H), (WeightSource(f"{p}.router"),))
        if spec.choice_bias is not None:
            out["choice_bias"] = ParamSpec((outputs,), (WeightSource(f"{p}.{spec.choice_bias}"),), role="vector")
        S = spec.shared_intermediate_size
        if S:
            if spec.gated:
                out["shared_up"] = ParamSpec((2 * S, H), (WeightSource(f"{p}.shared.gate", 0, S), WeightSource(f"{p}.shared.up", S, S)))
            else:
                out["shared_up"] = ParamSpec((S, H), (WeightSource(f"{p}.shared.up"),))
            out["shared_down"] = ParamSpec((H, S), (WeightSource(f"{p}.shared.down"),))
        return out

    def __init__(self, spec: RoutedMLPSpec, weights: dict, dtype: torch.dtype, device) -> None:
        if (spec.gated, spec.activation) not in ((True, "silu"), (False, "gelu"), (False, "relu2")):
            raise ConfigError(f"routed_mlp has gated experts with silu and plain experts with gelu (the exact one) or relu2, not "
                              f"gated={spec.gated} with {spec.activation!r}")
        if spec.score not in ("sigmoid", "softmax"):
            raise ConfigError(f"routed_mlp has no score {spec.score!r} (sigmoid or softmax)")
        if spec.shared_intermediate_size and not spec.gated and spec.activation != "relu2":
            raise ConfigError("a shared expert without a gate is built for the relu2 activation only")
        if spec.router not in ("learned", "token_table"):
            raise ConfigError(f"routed_mlp has no router {spec.router!r} (learned or token_table)")
        if spec.router == "token_table" and (spec.identity_experts or spec.choice_bias is not None or spec.vocab_size <= 0):
            raise ConfigError("experts named by a table of token ids: the table's rows are the vocabulary, and there are no "
                              "identity experts and no bias on the choice")
        self.outputs = spec.num_experts + spec.identity_experts
        if spec.identity_experts < 0 or not 1 <= spec.top_k <= min(32, self.outputs):
            raise ConfigError(f"{spec.top_k} of {self.outputs} experts: a token uses 1 to 32 of them")
        self.spec = spec
        H, F, E = spec.hidden_size, spec.intermediate_size, spec.num_experts
        self.router, self.table = weights.get("router"), weights.get("table")
        self.choice_bias = weights.get("choice_bias")
        self.shared_up, self.shared_down = weights.get("shared_up"), weights.get("shared_down")
        self.gate_up = weights["gate_up"].view(E, 2 * F if spec.gated else F, H)
        self.down = weights["down"].view(E, H, F)

    def forward(self, x, ctx: StepContext, defer: bool = False):
        from tandem_b200.kernels import moe

        s = self.spec
        x = deferred.tensor(x)
        if self.table is not None:
            ids, weights = moe.route_table(ctx.token_ids, self.table, s.num_experts)
        else:
            logits = ops.linear(x, self.router, out_dtype=torch.float32)
            ids, weights = moe.route(logits, s.top_k, s.score, s.normalize, s.route_scale, self.choice_bias)
        y = moe.experts(x, self.gate_up, self.down, ids, weights, gated=s.gated, num_router_outputs=self.outputs,
                        activation=s.activation if not s.gated else "gelu")
        if self.shared_up is not None:
            if s.gated:
                a = ops.gated_linear(x, self.shared_up)
            else:
                a = ops.bias_act(ops.linear(x, self.shared_up, out_dtype=torch.float32), None, "relu2", ctx.dtype)
            ops.add_pair(y, ops.linear(a, self.shared_down, out_dtype=torch.float32))
        return y
