"""Feed-forward parts: dense SwiGLU, and sigmoid-routed top-k experts with a shared expert."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .basic import Part
from .context import Pending
from .linear import linear
from .registry import register
from .spec import TensorSpec


class _SwiGLU:
    """(silu(x Wg^T) * x Wu^T) Wd^T with gate and up fused into one product
    (Mlp::forward, crates/hi-mlx/src/models.rs:2307-2312)."""

    def __init__(self, prefix: str, hidden: int, inter: int, short_names: bool = False):
        self.prefix, self.hidden, self.inter = prefix, hidden, inter
        self.suffix = "" if short_names else "_proj.weight"
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def _name(self, which: str) -> str:
        return f"{self.prefix}.{which}{self.suffix}"

    def tensor_specs(self):
        return [TensorSpec(self._name("gate"), (self.inter, self.hidden)),
                TensorSpec(self._name("up"), (self.inter, self.hidden)),
                TensorSpec(self._name("down"), (self.hidden, self.inter))]

    def load(self, fetch):
        g, u = fetch(self._name("gate")), fetch(self._name("up"))
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()
        self.w_down = fetch(self._name("down")).contiguous()

    def forward(self, x):
        return linear(ops.swiglu(linear(x, self.w_gate_up)), self.w_down)


@register("feed_forward", "dense_swiglu")
class DenseSwiGLU(Part):
    """W_down (silu(W_gate x) * (W_up x)).
    params: ``hidden_size``, ``intermediate_size``, ``names`` ("proj", the default: tensors
    ``<prefix>.{gate,up,down}_proj.weight``; "short": ``<prefix>.{gate,up,down}``)."""

    graph_safe = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.mlp = _SwiGLU(prefix, int(params["hidden_size"]), int(params["intermediate_size"]),
                           short_names=params.get("names", "proj") == "short")

    def tensor_specs(self):
        return self.mlp.tensor_specs()

    def load(self, fetch):
        self.mlp.load(fetch)

    def forward(self, normed, ctx):
        return self.mlp.forward(normed)


@register("feed_forward", "dense_mlp")
class DenseMLP(Part):
    """W_down act(W_up x): two products with an activation between them, no gate branch.

    params: ``hidden_size``, ``intermediate_size``, ``activation``:
      "xielu"  z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z/2, with the
               two learned numbers (p, q) of ``<prefix>.act``; the coefficients are worked out once, in float32.
      "relu2"  max(z, 0)^2; no tensor of its own
    tensors: ``<prefix>.up`` [I, H], ``<prefix>.down`` [H, I], ``<prefix>.act`` [2] (xielu)."""

    graph_safe = True
    ACTIVATIONS = ("xielu", "relu2")

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        self.activation = params.get("activation", "xielu")
        if self.activation not in self.ACTIVATIONS:
            raise ValueError(f"{prefix}: activation {self.activation!r} is not supported; known: {self.ACTIVATIONS}")
        self.w_up = self.w_down = self.coef = None

    def tensor_specs(self):
        specs = [TensorSpec(f"{self.prefix}.up", (self.inter, self.hidden)),
                 TensorSpec(f"{self.prefix}.down", (self.hidden, self.inter))]
        return specs + ([TensorSpec(f"{self.prefix}.act", (2,))] if self.activation == "xielu" else [])

    def load(self, fetch):
        self.w_up = fetch(f"{self.prefix}.up").contiguous()
        self.w_down = fetch(f"{self.prefix}.down").contiguous()
        if self.activation != "xielu":
            return
        pq = fetch(f"{self.prefix}.act").to(torch.float64)
        soft = torch.nn.functional.softplus(pq)
        self.coef = torch.stack([soft[0], 0.5 + soft[1]]).to(torch.float32).contiguous()

    def forward(self, normed, ctx):
        z = linear(normed, self.w_up)
        return linear(ops.relu2(z) if self.activation == "relu2" else ops.xielu(z, self.coef), self.w_down)


@register("feed_forward", "routed_experts")
@register("feed_forward", "moe_sigmoid")
class SigmoidRoutedExperts(Part):
    """Router logits in float32, the k largest (ties to the lower id); by default score =
    sigmoid(logit) without renormalisation and the score scales the expert input; an always-on
    shared expert sees the unscaled input; outputs are summed (Llama4Moe::forward,
    crates/hi-mlx/src/models.rs:6055-6103; the reference is top-1 only). The other routing rules of
    the reference's donor kernel (crates/hi-cuda/src/kernels.cu:536-546) are parameters too.

    params: ``hidden_size``, ``num_experts``, ``top_k``, ``intermediate_size``, ``shared_expert``,
      ``shared_intermediate_size`` (the shared expert's inner size; default ``intermediate_size``);
      ``score``        "sigmoid" (default) | "softmax" (over all experts)
      ``renormalize``  the chosen scores are divided by their sum (default False)
      ``scale``        "input" (default: the score multiplies what the expert reads) | "output"
                       (it multiplies what the expert returns, in the sum the next norm takes)
      ``activation``   "swiglu" (default: gate and up stacks) | "relu2" (W_down max(W_up x, 0)^2: no gate stack;
                       the score then has to scale the output)
      ``groups``       None | (count, keep): the experts lie in ``count`` equal groups of neighbours, a group
                       counts as the sum of its two largest scores, and only experts of the ``keep`` best
                       groups can be chosen
      ``score_scale``  a constant factor on every chosen score (default 1)
      ``names``        "stacked" (default, the tensors below) | "per_expert": ``<prefix>.router`` [E, H] and for
                       every expert i ``<prefix>.e<i>.up`` [I, H], ``<prefix>.e<i>.down`` [H, I] (and ``.gate``
                       with swiglu), stacked at load; the shared expert is then ``<prefix>.shared.{gate,up,down}``
    tensors: ``<prefix>.router.weight`` [E, H]; ``<prefix>.experts.{gate,up}_proj.weight`` [E, I, H];
    ``<prefix>.experts.down_proj.weight`` [E, H, I]; ``<prefix>.shared_expert.{gate,up,down}_proj.weight``.
    """

    graph_safe = True

    FEW_ROWS = 10    # up to this many routed rows the weight-streaming kernel is used (measured: from 12
                     # rows the tcgen05 kernel streams the expert weights faster, even with nearly empty tiles)
    wants_f32_input = True   # the router reads the norm's float32 output
    OVERLAP_SHARED = True    # run the shared expert on a second stream beside the routed path

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.hidden, self.experts = int(params["hidden_size"]), int(params["num_experts"])
        self.top_k, self.inter = int(params["top_k"]), int(params["intermediate_size"])
        if not 1 <= self.top_k <= self.experts:
            raise ValueError(f"{prefix}: top_k {self.top_k} outside 1..{self.experts}")
        self.per_expert_names = params.get("names", "stacked") == "per_expert"
        self.shared = None
        if params.get("shared_expert", True):
            shared_inter = int(params.get("shared_intermediate_size") or self.inter)
            self.shared = _SwiGLU(f"{prefix}.shared", self.hidden, shared_inter, short_names=True) \
                if self.per_expert_names else _SwiGLU(f"{prefix}.shared_expert", self.hidden, shared_inter)
        score, scale = params.get("score", "sigmoid"), params.get("scale", "input")
        if score not in ("sigmoid", "softmax") or scale not in ("input", "output"):
            raise ValueError(f"{prefix}: score {score!r} / scale {scale!r} are not known (sigmoid | softmax; input | output)")
        self.router_mode = (ops.ROUTER_SOFTMAX if score == "softmax" else 0) | \
            (ops.ROUTER_RENORMALIZE if params.get("renormalize", False) else 0)
        self.scale_output = scale == "output"
        self.activation = params.get("activation", "swiglu")
        if self.activation not in ("swiglu", "relu2") or (self.activation == "relu2" and not self.scale_output):
            raise ValueError(f"{prefix}: activation {self.activation!r} is not known (swiglu | relu2), or relu2 "
                             f"without scale 'output' (a score on the input would be squared)")
        self.groups = tuple(int(g) for g in params["groups"]) if params.get("groups") else None
        if self.groups:
            count, keep = self.groups
            if score != "sigmoid" or self.experts % count or not 0 < keep <= count or self.top_k > keep * (self.experts // count):
                raise ValueError(f"{prefix}: {self.experts} sigmoid-scored experts do not form {count} equal groups of "
                                 f"which {keep} hold {self.top_k} choices")
            self.router_mode |= ops.router_groups(count, keep)
        self.score_scale = float(params.get("score_scale", 1.0))
        self._ones: Optional[torch.Tensor] = None
        self.w_router = self.w_gate = self.w_up = self.w_down = None
        self._side_stream = None

    def tensor_specs(self):
        e, i, h, p = self.experts, self.inter, self.hidden, self.prefix
        gated = self.activation == "swiglu"
        if self.per_expert_names:
            specs = [TensorSpec(f"{p}.router", (e, h))]
            for j in range(e):
                specs += ([TensorSpec(f"{p}.e{j}.gate", (i, h))] if gated else []) + \
                    [TensorSpec(f"{p}.e{j}.up", (i, h)), TensorSpec(f"{p}.e{j}.down", (h, i))]
        else:
            specs = [TensorSpec(f"{p}.router.weight", (e, h))] + \
                ([TensorSpec(f"{p}.experts.gate_proj.weight", (e, i, h))] if gated else []) + \
                [TensorSpec(f"{p}.experts.up_proj.weight", (e, i, h)),
                 TensorSpec(f"{p}.experts.down_proj.weight", (e, h, i))]
        return specs + (self.shared.tensor_specs() if self.shared else [])

    def load(self, fetch):
        p = self.prefix

        def expert_tensor(name):
            t = fetch(name)
            if t.dtype != self.env.dtype:
                raise ValueError(
                    f"tensor '{name}' is stored in {t.dtype} and stays so; the expert kernels of the "
                    f"{self.env.dtype} path cannot take it (run with --dtype float32)")
            return t.contiguous()

        gated = self.activation == "swiglu"
        if self.per_expert_names:
            stack = lambda part: torch.stack([expert_tensor(f"{p}.e{j}.{part}") for j in range(self.experts)]).contiguous()
            self.w_router = expert_tensor(f"{p}.router")
            self.w_gate = stack("gate") if gated else None
            self.w_up, self.w_down = stack("up"), stack("down")
        else:
            self.w_router = expert_tensor(f"{p}.router.weight")
            self.w_gate = expert_tensor(f"{p}.experts.gate_proj.weight") if gated else None
            self.w_up = expert_tensor(f"{p}.experts.up_proj.weight")
            self.w_down = expert_tensor(f"{p}.experts.down_proj.weight")
        if self.shared:
            self.shared.load(fetch)

    def _shared_on_side_stream(self, normed):
        """The shared expert has no dependency on the routing: it runs on a second stream beside
        the router, the plan and the routed experts (in a captured step: a parallel branch), and
        joins before the sum. Both paths stream weights; together they keep HBM busier than in turn."""
        cur = torch.cuda.current_stream()
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=normed.device)
        side = self._side_stream
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            shared = self.shared.forward(normed)
        normed.record_stream(side)
        shared.record_stream(cur)
        return shared, side

    def forward(self, normed, ctx, normed_f32=None):
        n = normed.shape[0]
        side = None
        if self.shared and self.OVERLAP_SHARED:
            shared, side = self._shared_on_side_stream(normed)
        router_in = normed if normed_f32 is None else normed_f32
        forced = ctx.forced.get(f"{self.prefix}.router_ids") if ctx.forced else None
        if forced is None:
            ids, scores, plan = ops.router_plan(router_in, self.w_router, self.top_k, self.router_mode, self.score_scale)
        else:
            # debug: another run's expert choices, scored with this run's own logits (two runs in
            # different precisions can then be compared token by token)
            _own, _s, logits = ops.router_topk(router_in, self.w_router, self.top_k, want_logits=True)
            ids = forced.to(device=logits.device, dtype=torch.int32).reshape(n, self.top_k).contiguous()
            chosen = torch.gather(logits, 1, ids.long())
            scores = torch.sigmoid(chosen) if not self.router_mode & ops.ROUTER_SOFTMAX else \
                torch.exp(chosen - torch.logsumexp(logits, dim=1, keepdim=True))
            if self.router_mode & ops.ROUTER_RENORMALIZE:
                scores = scores / scores.sum(dim=1, keepdim=True)
            scores = (scores * self.score_scale).contiguous()
            plan = ops.moe_plan(ids, self.experts)
        if ctx.tap is not None:
            ctx.tap(f"{self.prefix}.router_ids", ids)
        entry_weights = None
        if self.scale_output:
            # the experts read the unscaled rows (a factor of one); their outputs take the score in the sum
            if self._ones is None or self._ones.numel() < scores.numel():
                self._ones = torch.ones(max(scores.numel(), 65536), dtype=torch.float32, device=scores.device)
            entry_weights, scores = scores.view(-1), self._ones[: scores.numel()].view_as(scores)
        tc = ops.moe_tc_supported(normed, self.w_up)
        few = n * self.top_k <= (self.FEW_ROWS if tc else 128)
        if not few and tc and self.activation == "relu2":
            # the up stack alone is a plain grouped product with the squared relu as its epilogue
            y = ops.moe_down_tc(ops.moe_up_relu2_tc(normed, plan, self.top_k, self.w_up), self.w_down, plan)
        elif not few and tc:
            # many rows per expert: the grouped products run on tcgen05
            act = ops.moe_gate_up_tc(normed, plan, self.top_k, self.w_gate, self.w_up, scores)
            y = ops.moe_down_tc(act, self.w_down, plan)
        else:
            act = ops.moe_gate_up(normed, plan, self.top_k, self.w_gate, self.w_up, scores, few, self.activation)
            y = ops.moe_down(act, self.w_down, plan, few)
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
        else:
            shared = self.shared.forward(normed) if self.shared else None
        # the sum shared + routed rows is taken inside the next norm's residual add
        return Pending(dense=shared, routed=y, slot_of_entry=plan.slot_of_entry, top_k=self.top_k,
                       entry_weights=entry_weights)
