"""A routed feed-forward (mixture of experts) with an optional shared expert.

With u [T, d] the branch input, E experts of width f, each down_e(act(gate_e u) * (up_e u)) without biases:

    z      = W_r u + b_r                       float32, whatever the engine's precision
    S_t    = the `top` experts with the largest z_t (ties: the lower index)
    a_t,e  = exp(z_t,e) / sum over e' in S_t of exp(z_t,e')        softmax over the chosen logits alone
    y_t    = sum over e in S_t of a_t,e * expert_e(u_t)  (+ shared(u_t), an expert every token uses)

The (token, choice) pairs are sorted by expert on the device into tiles (no host round trip: array sizes are upper
bounds, so a captured step replays it), the experts' two products run as ONE routed launch each over stacked weights
[E, 2 f, d] and [E, d, f] (gate and up fused with the activation), and the pairs are combined per token in the order
of the choices, in float32. A token's result does not depend on what else is in the batch. Prompts of a bfloat16 engine
hand the two products to the vendor library's grouped GEMM instead (as the dense layers hand theirs to its plain one):
the tokens are gathered into the order of their experts first, the offsets stay on the device.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops, trace
from .base import FeedForward, ParamSpec, build_part, register_feed_forward
from ..config.spec import PartSpec


class RoutedExperts(FeedForward):
    """params: hidden, n_experts, top, expert_ff, activation (default "silu"), router_bias (bool, default True),
    shared_ff (width of the shared expert, None = none), shared_activation (default: `activation`), names
    (checkpoint sub-names: router, router_bias, expert (a pattern with {e}), gate, up, down, shared)."""

    def __init__(self, params, runtime):
        super().__init__(params, runtime)
        p = params
        self.hidden, self.n_experts, self.top = int(p["hidden"]), int(p["n_experts"]), int(p["top"])
        self.expert_ff = int(p["expert_ff"])
        if not 0 < self.top <= self.n_experts:
            raise ValueError(f"top ({self.top}) must be between 1 and n_experts ({self.n_experts})")
        name = str(p.get("activation", "silu"))
        if name not in ops.ACTIVATIONS or name == "none":
            raise ValueError(f"activation {name!r} is not known ({sorted(ops.ACTIVATIONS)})")
        self.activation = ops.ACTIVATIONS[name]
        self.router_bias = bool(p.get("router_bias", True))
        self.names = dict({"router": "router", "router_bias": "router.b", "expert": "e{e}", "gate": "gate", "up": "up",
                           "down": "down", "shared": "shared"}, **(p.get("names") or {}))
        self.shared = None
        if p.get("shared_ff"):
            n = self.names
            self.shared = build_part("feed_forward", PartSpec("swiglu", {
                "hidden": self.hidden, "intermediate": int(p["shared_ff"]),
                "activation": str(p.get("shared_activation", name)), "out_float32": True,
                "names": {"gate": n["gate"], "up": n["up"], "down": n["down"]}}), runtime)
        self.w_router = self.b_router = self.w_gate_up = self.w_down = None
        self._library = True          # prompts may use the vendor's grouped GEMM until it refuses a shape

    def _expert_name(self, e: int, which: str) -> str:
        return f"{self.names['expert'].format(e=e)}.{self.names[which]}"

    def param_specs(self) -> Dict[str, ParamSpec]:
        n, d, f = self.names, self.hidden, self.expert_ff
        specs = {n["router"]: ParamSpec((self.n_experts, d))}
        if self.router_bias:
            specs[n["router_bias"]] = ParamSpec((self.n_experts,), role="vector", init=("normal",))
        for e in range(self.n_experts):
            specs[self._expert_name(e, "gate")] = ParamSpec((f, d))
            specs[self._expert_name(e, "up")] = ParamSpec((f, d))
            specs[self._expert_name(e, "down")] = ParamSpec((d, f))
        if self.shared is not None:
            for local, ps in self.shared.param_specs().items():
                specs[f"{n['shared']}.{local}"] = ps
        return specs

    def load(self, tensors):
        n = self.names
        self.w_router = tensors[n["router"]].to(torch.float32).contiguous()
        self.b_router = tensors[n["router_bias"]].to(torch.float32).contiguous() if self.router_bias else None
        gu, dn = [], []
        for e in range(self.n_experts):
            gu.append(torch.cat([tensors[self._expert_name(e, "gate")], tensors[self._expert_name(e, "up")]], dim=0))
            dn.append(tensors[self._expert_name(e, "down")])
        dtype = torch.float32 if any(t.dtype == torch.float32 for t in gu + dn) else gu[0].dtype
        self.w_gate_up = torch.stack([t.to(dtype) for t in gu]).contiguous()       # [E, 2 f, d]
        self.w_down = torch.stack([t.to(dtype) for t in dn]).contiguous()          # [E, d, f]
        if self.shared is not None:
            cut = len(n["shared"]) + 1
            self.shared.load({k[cut:]: v for k, v in tensors.items() if k.startswith(n["shared"] + ".")})

    def weight_bytes(self) -> int:
        """What a one-token step of one sequence reads: the router, `top` experts and the shared expert."""
        per_expert = 3 * self.expert_ff * self.hidden * self.w_down.element_size()
        return self.w_router.numel() * 4 + self.top * per_expert + (self.shared.weight_bytes() if self.shared else 0)

    def forward(self, x, ctx, residual=None):
        trace.push("FFN")
        try:
            T, dev = x.shape[0], x.device
            top, E = self.top, self.n_experts
            w = self.w_gate_up
            xin = x if x.dtype == w.dtype else x.to(w.dtype)
            ids = torch.empty((T, top), dtype=torch.int32, device=dev)
            weights = torch.empty((T, top), dtype=torch.float32, device=dev)
            ops.moe_route(x, self.w_router, self.b_router, ids, weights)
            n_pairs = T * top
            small = n_pairs <= ops.GROUPED_SMALL_ROWS
            tile = ops.grouped_tile_rows(small)
            n_tiles = ops.moe_max_tiles(n_pairs, E, tile)
            index = torch.empty(2 * n_tiles * tile + n_tiles, dtype=torch.int32, device=dev)
            sorted_token, sorted_pair = index[:n_tiles * tile], index[n_tiles * tile:2 * n_tiles * tile]
            tile_group = index[2 * n_tiles * tile:]
            shared = None
            if self._library and ops.library_grouped_mm_ok(n_pairs, w, self.w_down):
                # prompts: each expert's rows side by side, the two products by the library's grouped GEMM
                extra = torch.empty(E + n_pairs, dtype=torch.int32, device=dev)
                group_end, pair_pos = extra[:E], extra[E:]
                ops.moe_sort(ids, E, tile, sorted_token, sorted_pair, tile_group, group_end, pair_pos)
                xs = ops.moe_gather_rows(xin, sorted_token, torch.empty((n_tiles * tile, self.hidden), dtype=w.dtype,
                                                                         device=dev))
                try:
                    gu = ops.library_grouped_mm(xs, w, group_end)
                except RuntimeError as exc:
                    # the library refuses these sizes (it checks before it launches): this library's own routed
                    # products take them, from now on without asking again
                    if "CUDA error" in str(exc):
                        raise
                    self._library = False
                    gu = None
                if gu is not None:
                    act = torch.empty((n_tiles * tile, self.expert_ff), dtype=w.dtype, device=dev)
                    ops.gated_act(gu, act, self.activation)
                    y = ops.library_grouped_mm(act, self.w_down, group_end)
                    if self.shared is not None:
                        shared = self.shared.forward(x, ctx)
                    out = torch.empty((T, self.hidden), dtype=torch.float32, device=dev)
                    return ops.moe_combine(y, weights, shared, out, pair_pos)
            ops.moe_sort(ids, E, tile, sorted_token, sorted_pair, tile_group)
            # gate and up of every pair's expert with the activation; rows stay in sorted order
            act = torch.empty((n_tiles * tile, self.expert_ff), dtype=w.dtype, device=dev)
            ops.routed_gemm_nt(xin, sorted_token, w, act, None, tile_group, n_tiles * tile, small, dual=True,
                               act=self.activation)
            # down: back to the order of the pairs, float32
            y = torch.empty((n_pairs, self.hidden), dtype=torch.float32, device=dev)
            ops.routed_gemm_nt(act, None, self.w_down, y, sorted_pair, tile_group, n_tiles * tile, small)
            shared = self.shared.forward(x, ctx) if self.shared is not None else None
            out = torch.empty((T, self.hidden), dtype=torch.float32, device=dev)
            return ops.moe_combine(y, weights, shared, out)
        finally:
            trace.pop()


register_feed_forward("routed_experts", RoutedExperts)
