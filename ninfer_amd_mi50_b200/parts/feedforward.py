"""Feed-forward parts: a dense SwiGLU MLP, and routed SwiGLU experts with a gated
shared expert.

Dense (src/models/model.hip:334-336, gate and up fused to ``[2I, H]`` at load,
model.hip:586-605): ``ffn = Wdown (silu(Wgate x) * Wup x)``, ``silu(g) = g / (1 + exp(-g))``
(src/ops/kernels.hip:131-140).

Sparse (model.hip:338-433; routing in ``moe_route_cpu``, src/ops/moe.hip:49-106):
router logits in float32, softmax over all experts, the k largest probabilities
(ties to the lower index), weights ``p_e`` or, with ``norm_topk_prob``, ``p_e / sum(selected)``
(the reference always renormalises, moe.hip:77-82); every selected expert is a SwiGLU
MLP; ``moe = sum_i w_i y_i`` in selection order.  The shared expert and its sigmoid gate
(``ffn = moe + sigmoid(w_sg x) * shared(x)``) are Qwen2-MoE's and absent from the
reference.  Unlike the reference, routing never leaves the device.
"""

from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..registry import register_part
from .base import FeedForward, Fetch, RoutedSum, StepContext, TensorSpec


_SIDE_STREAMS = {}


def _side_stream(device: torch.device, urgent: bool = False) -> "torch.cuda.Stream":
    """The second stream of a device; `urgent`: the one whose CTAs are placed before others'."""
    key = (str(device), urgent)
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device=device, priority=-1 if urgent else 0)
    return _SIDE_STREAMS[key]


@register_part("feed_forward", "dense_swiglu")
class DenseSwiglu(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.prefix = prefix
        self.w_gate_up = self.w_down = None

    def tensor_specs(self) -> List[TensorSpec]:
        p, H, I = self.prefix, self.hidden_size, self.intermediate_size
        return [TensorSpec(p + "gate_proj.weight", (I, H)),
                TensorSpec(p + "up_proj.weight", (I, H)),
                TensorSpec(p + "down_proj.weight", (H, I))]

    def load(self, fetch: Fetch) -> None:
        p = self.prefix
        self.w_gate_up = torch.cat([fetch(p + "gate_proj.weight"), fetch(p + "up_proj.weight")],
                                   dim=0).contiguous()
        self.w_down = fetch(p + "down_proj.weight")

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * self.w_down.element_size()

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return kernels.linear(kernels.linear_swiglu(x, self.w_gate_up), self.w_down)


@register_part("feed_forward", "sparse_moe_swiglu")
class SparseMoeSwiglu(FeedForward):
    graph_safe = True

    # set to a list to collect each call's selected experts (measurement only)
    record_routing = None

    def __init__(self, hidden_size: int, num_experts: int, top_k: int, norm_topk_prob: bool,
                 moe_intermediate_size: int, shared_intermediate_size: int, prefix: str):
        if not 1 <= top_k <= num_experts:
            raise ValueError(f"top_k={top_k} must lie in [1, num_experts={num_experts}]")
        kernels.check_router_sizes(num_experts, top_k)
        self.hidden_size, self.num_experts, self.top_k = int(hidden_size), int(num_experts), int(top_k)
        self.norm_topk_prob = bool(norm_topk_prob)
        self.moe_intermediate_size = int(moe_intermediate_size)
        self.shared_intermediate_size = int(shared_intermediate_size)
        self.prefix = prefix
        self.w_router = self.w13 = self.w2 = self.ws13 = self.ws2 = self.ws_packed = None
        self.w_router_split = None

    @property
    def has_shared(self) -> bool:
        return self.shared_intermediate_size > 0

    def tensor_specs(self) -> List[TensorSpec]:
        p, H, I, Is = self.prefix, self.hidden_size, self.moe_intermediate_size, self.shared_intermediate_size
        specs = [TensorSpec(p + "gate.weight", (self.num_experts, H), role="router")]
        for e in range(self.num_experts):
            q = f"{p}experts.{e}."
            specs += [TensorSpec(q + "gate_proj.weight", (I, H)),
                      TensorSpec(q + "up_proj.weight", (I, H)),
                      TensorSpec(q + "down_proj.weight", (H, I))]
        if self.has_shared:
            q = p + "shared_expert."
            specs += [TensorSpec(q + "gate_proj.weight", (Is, H)),
                      TensorSpec(q + "up_proj.weight", (Is, H)),
                      TensorSpec(q + "down_proj.weight", (H, Is)),
                      TensorSpec(p + "shared_expert_gate.weight", (1, H), role="router")]
        return specs

    def load(self, fetch: Fetch) -> None:
        p, H, I, E = self.prefix, self.hidden_size, self.moe_intermediate_size, self.num_experts
        router = fetch(p + "gate.weight")
        if self.has_shared:
            # one matrix yields the router logits and the shared expert's gate logit
            router = torch.cat([router, fetch(p + "shared_expert_gate.weight")], dim=0)
        self.w_router = router.contiguous()
        self.w_router_split = kernels.split_router(self.w_router) if self.w_router.is_cuda else None
        first = fetch(f"{p}experts.0.gate_proj.weight")
        self.w13 = torch.empty((E, 2 * I, H), dtype=first.dtype, device=first.device)
        self.w2 = torch.empty((E, H, I), dtype=first.dtype, device=first.device)
        for e in range(E):
            q = f"{p}experts.{e}."
            self.w13[e, :I].copy_(first if e == 0 else fetch(q + "gate_proj.weight"))
            self.w13[e, I:].copy_(fetch(q + "up_proj.weight"))
            self.w2[e].copy_(fetch(q + "down_proj.weight"))
        del first
        if (self.w13.is_cuda and self.w13.dtype == torch.bfloat16 and kernels.can_pack(I, H)
                and kernels.can_pack(H, I)):
            # the bfloat16 kernels stream the experts from a tile layout; the row-major form goes
            self.w13 = kernels.pack_weights(self.w13, swiglu=True)
            self.w2 = kernels.pack_weights(self.w2, swiglu=False)
        if self.has_shared:
            q = p + "shared_expert."
            self.ws13 = torch.cat([fetch(q + "gate_proj.weight"), fetch(q + "up_proj.weight")],
                                  dim=0).contiguous()
            self.ws2 = fetch(q + "down_proj.weight")
            # a second copy in the experts' tile layout, cut into chunks of the experts' width: decode
            # steps then serve the shared expert inside the experts' persistent launch (prompt steps
            # keep the row-major form for the library's products)
            self.ws_packed = None
            if (isinstance(self.w13, kernels.PackedWeights) and kernels.TUNING["moe_stream_shared"]
                    and self.ws13.dtype == torch.bfloat16):
                self.ws_packed = kernels.pack_shared_expert(self.ws13, self.ws2.contiguous(), I)

    def weight_bytes(self) -> int:
        n = self.w_router.numel() * 4 + self._expert_total_bytes()
        if self.has_shared:
            n += (self.ws13.numel() + self.ws2.numel()) * self.ws2.element_size()
        return n

    def _expert_total_bytes(self) -> int:
        if isinstance(self.w13, kernels.PackedWeights):
            return self.w13.nbytes() + self.w2.nbytes()
        return (self.w13.numel() + self.w2.numel()) * self.w2.element_size()

    def expert_bytes(self) -> int:
        """Bytes of one routed expert's matrices."""
        return self._expert_total_bytes() // self.num_experts

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        """The same arithmetic in four arrangements, chosen by the number of rows (thresholds in
        `kernels.TUNING`, each with the measurement behind it):
        6 to 16 rows - routing, experts and shared expert in one persistent launch;
        up to 64 rows - the shared expert on a second stream beside the router and the experts
        (which are one persistent launch from 6 rows on);
        more rows - the routing on a second stream beside the shared expert's products.
        (Without a shared expert, or with the thresholds moved: one kernel after the other.)"""
        E, k = self.num_experts, self.top_k
        if (self.ws_packed is not None and x.is_cuda
                and kernels.can_route_and_run_experts(x, self.w_router, self.w13, self.w2, E, k, shared=self.ws_packed)):
            # a decode step: routing, the experts' products and the shared expert's are one persistent launch
            idx, wts, gate, plan, y, sum_wts, sum_plan = kernels.route_and_run_experts(
                x, self.w_router, E, k, self.norm_topk_prob, self.w13, self.w2, shared=self.ws_packed)
            if SparseMoeSwiglu.record_routing is not None:
                SparseMoeSwiglu.record_routing.append(idx.clone())
            return RoutedSum(y, sum_plan, sum_wts, None, None, x.dtype)
        # The shared expert needs nothing from the router, so on small steps (where kernels are
        # too short to fill the device) it runs beside the routed path on a second stream;
        # inside a captured graph that becomes a parallel branch.
        fork = self.has_shared and x.is_cuda and x.shape[0] <= kernels.TUNING["shared_fork_max_rows"]
        shared = None

        def start_shared():
            main, side = torch.cuda.current_stream(x.device), _side_stream(x.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                kernels.chain_break()       # its input comes from the other stream
                return main, side, kernels.linear(kernels.linear_swiglu(x, self.ws13), self.ws2)

        # The shared expert starts beside the router (whose kernels leave the memory idle) up to
        # `shared_fork_late_rows` rows, beyond that after it, beside the experts' products.
        late = x.shape[0] > kernels.TUNING["shared_fork_late_rows"]
        # In large steps it is the other way round: the shared expert's products fill the device,
        # and the routing - a chain of short kernels of a few CTAs - runs beside them.
        beside = kernels.TUNING["route_beside_shared_min_rows"]
        beside = self.has_shared and x.is_cuda and not fork and 0 < beside <= x.shape[0]
        # A decode step without a shared expert beside it: routing and both products of the experts
        # are one persistent launch.  (With a shared expert on the second stream the router's own
        # kernels are the better choice: they leave the memory idle, and the shared expert's first
        # product fills exactly that gap.  Measured at 8 tokens and A2.7B sizes: 3.45 ms a step with
        # the router's kernels, 3.61 ms with the routing inside the launch; without the second
        # stream 3.74 against 3.61.)
        fused = (x.is_cuda and not beside and not fork
                 and kernels.can_route_and_run_experts(x, self.w_router, self.w13, self.w2, E, k))
        if fork and not late:
            main, side, shared = start_shared()
        gathered = None
        y = None
        if beside:
            main, side = torch.cuda.current_stream(x.device), _side_stream(x.device, urgent=True)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                kernels.chain_break()
                idx, wts, gate, plan = kernels.route(x, self.w_router, E, k, self.norm_topk_prob,
                                                     split=self.w_router_split)
                if kernels.moe_uses_gathered_rows(x, self.w13):
                    gathered = kernels.moe_gather(x, plan, k)
            shared = kernels.linear(kernels.linear_swiglu(x, self.ws13), self.ws2)
            main.wait_stream(side)
            kernels.chain_break()
        elif fused:
            idx, wts, gate, plan, y = kernels.route_and_run_experts(x, self.w_router, E, k, self.norm_topk_prob,
                                                                    self.w13, self.w2)
        else:
            idx, wts, gate, plan = kernels.route(x, self.w_router, E, k, self.norm_topk_prob,
                                                 split=self.w_router_split)
            if fork and late:
                main, side, shared = start_shared()
        if SparseMoeSwiglu.record_routing is not None:
            SparseMoeSwiglu.record_routing.append(idx.clone())
        if y is None:
            y = kernels.moe_experts(x, self.w13, self.w2, plan, k, gathered=gathered)
        if fork:
            main.wait_stream(side)
            kernels.chain_break()           # the kernel that adds up also reads what the other stream produced
        elif self.has_shared and not beside:
            shared = kernels.linear(kernels.linear_swiglu(x, self.ws13), self.ws2)
        # not added up here: the next norm does it inside its own kernel (`RoutedSum`); whoever
        # cannot calls `materialize()`, which is `kernels.moe_combine`
        return RoutedSum(y, plan, wts, shared, gate, x.dtype)
