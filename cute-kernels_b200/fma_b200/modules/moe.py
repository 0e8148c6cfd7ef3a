"""`MoE` and `Experts` with the reference's constructor, forward signature, parameter names and
state_dict keys (fma/modules/moe/__init__.py:17-124, :127-298), running on hand-written sm_100a
kernels only.

Data flow of `MoE.forward` (T tokens, R = T*k routed rows):
    logits = gate(x)                                  nn.Linear, kept as a replaceable module
    w, sel = top-k + softmax kernel                   [T,k]
    maps   = stable counting sort of sel              expert segments padded to 256-row tiles
    xg     = scatter(x)                               [rows_cap, H], padding rows zero
    pre, a = up-projection GEMM (+ SwiGLU epilogue)   tcgen05 for bf16, FFMA for f32
    out    = down-projection GEMM
    y      = sum_j w[t,j] * out[row(t,j)]             weighted combine
Backward mirrors it with dgrad / wgrad GEMMs (SwiGLU backward in the dgrad epilogue).
"""

from __future__ import annotations

import functools
from typing import Callable

import torch
import torch.nn as nn

from .. import _native
from ..kernel_backend import KernelBackend
from ..ops.grouped_gemm import grouped_gemm
from ..ops.swiglu import swiglu_packed
from . import _kernels as K


class _RouterTopK(torch.autograd.Function):
    """(weights, selected, sort workspace) = softmax(topk(logits)); backward scatters into d_logits.
    The workspace holds the first pass of the expert sort (and the router's probability sums when asked
    for), produced by the same kernel."""

    @staticmethod
    def forward(ctx, logits: torch.Tensor, k: int, want_probs: bool):
        weights, selected, workspace = K.router_topk_softmax_routed(logits, k, want_probs)
        ctx.save_for_backward(weights, selected)
        ctx.num_experts = logits.size(1)
        ctx.mark_non_differentiable(selected, workspace)
        return weights, selected, workspace

    @staticmethod
    def backward(ctx, d_weights, _d_selected, _d_workspace):
        weights, selected = ctx.saved_tensors
        return K.router_topk_softmax_backward(weights, d_weights, selected, ctx.num_experts), None, None


class _RouterMeanProb(torch.autograd.Function):
    """mean_prob[e] = mean over tokens of softmax(router_logits)[t, e].  The value comes from the router
    kernel (passed in); this node only supplies its gradient with respect to the logits."""

    @staticmethod
    def forward(ctx, logits: torch.Tensor, mean_prob: torch.Tensor):
        ctx.save_for_backward(logits)
        return mean_prob.clone()

    @staticmethod
    def backward(ctx, d_mean_prob):
        (logits,) = ctx.saved_tensors
        return K.router_mean_prob_backward(logits, d_mean_prob), None


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, maps: K.RowMaps):
        ctx.maps = maps
        ctx.T = x.size(0)
        return K.scatter(x.contiguous(), maps)

    @staticmethod
    def backward(ctx, d_grouped):
        return K.scatter_backward(d_grouped.contiguous(), ctx.maps, ctx.T), None


class _ExpertLinear(torch.autograd.Function):
    """Y[p] = X[p] . W[e(p)]^T over the grouped layout (Experts.cuda_forward of the reference)."""

    @staticmethod
    def forward(ctx, x, weight, bias, maps: K.RowMaps):
        x = x.contiguous()
        weight = weight.contiguous()
        ctx.save_for_backward(x, weight)
        ctx.maps = maps
        y = K.gemm_forward(x, weight, maps.mtile_expert, maps.row_align)
        if bias is not None:
            K.bias_add_(y, bias.contiguous(), maps)
        return y

    @staticmethod
    def backward(ctx, d_y):
        x, weight = ctx.saved_tensors
        maps = ctx.maps
        d_y = d_y.contiguous()
        d_x = K.gemm_dgrad(d_y, weight, maps.mtile_expert, maps.row_align) if ctx.needs_input_grad[0] else None
        d_w = K.gemm_wgrad(d_y, x, weight.size(0), maps.pad_offsets) if ctx.needs_input_grad[1] else None
        d_b = K.bias_grad(d_y, maps) if ctx.needs_input_grad[2] else None
        return d_x, d_w, d_b, None


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, expert_out, weights, maps: K.RowMaps, T: int):
        expert_out = expert_out.contiguous()
        weights = weights.contiguous()
        ctx.save_for_backward(expert_out, weights)
        ctx.maps = maps
        return K.combine(expert_out, weights, maps, T)

    @staticmethod
    def backward(ctx, dy):
        expert_out, weights = ctx.saved_tensors
        d_out, d_w = K.combine_backward(dy.contiguous(), expert_out, weights, ctx.maps, ctx.needs_input_grad[1])
        return d_out, d_w, None, None


class _FusedSwigluExperts(torch.autograd.Function):
    """scatter -> up projection with SwiGLU epilogue -> down projection -> weighted combine, and the
    matching backward, as one autograd node (no intermediate autograd bookkeeping, `pre` and `act`
    are produced by one kernel, d_pre by one kernel)."""

    @staticmethod
    def forward(ctx, x, weights, w_fc, w_proj, maps: K.RowMaps):
        x = x.contiguous()
        weights = weights.contiguous()
        w_fc = w_fc.contiguous()
        w_proj = w_proj.contiguous()
        T = x.size(0)
        xg = K.scatter(x, maps)
        pre, act = K.gemm_forward_swiglu(xg, w_fc, maps.mtile_expert, keep_pre=True, row_align=maps.row_align)
        out = K.gemm_forward(act, w_proj, maps.mtile_expert, maps.row_align)
        y = K.combine(out, weights, maps, T)
        ctx.save_for_backward(xg, pre, act, out, weights, w_fc, w_proj)
        ctx.maps = maps
        ctx.T = T
        return y

    @staticmethod
    def backward(ctx, dy):
        xg, pre, act, out, weights, w_fc, w_proj = ctx.saved_tensors
        maps = ctx.maps
        E = w_fc.size(0)
        need_x, need_w, need_fc, need_proj = ctx.needs_input_grad[:4]
        d_out, d_w = K.combine_backward(dy.contiguous(), out, weights, maps, need_w)
        d_w_proj = K.gemm_wgrad(d_out, act, E, maps.pad_offsets) if need_proj else None
        d_x = d_w_fc = None
        if need_x or need_fc:
            d_pre = K.gemm_dgrad_swiglu(d_out, w_proj, pre, maps.mtile_expert, maps.row_align)
            if need_fc:
                d_w_fc = K.gemm_wgrad(d_pre, xg, E, maps.pad_offsets)
            if need_x:
                d_xg = K.gemm_dgrad(d_pre, w_fc, maps.mtile_expert, maps.row_align)
                d_x = K.scatter_backward(d_xg, maps, ctx.T)
        return d_x, d_w, d_w_fc, d_w_proj, None


class _GroupedGemmExperts(torch.autograd.Function):
    """The reference's expert linear on its own layout (fma/modules/moe/cuda_implementation/__init__.py:15-80):
    x holds the rows of expert e in M_array[e] consecutive rows (no alignment requirement), weight is
    [E, N, K]; forward and both gradients are calls of the general grouped GEMM."""

    @staticmethod
    def forward(ctx, x, weight, M_array, N_array, K_array):
        x, weight = x.contiguous(), weight.contiguous()
        _, N, K = weight.size()
        assert N % 8 == 0 and K % 8 == 0
        output = grouped_gemm(A=x, B=weight, C=None, M_array=M_array, N_array=N_array, K_array=K_array,
                              output_shape=(x.size(0), N), is_A_transposed=False, is_B_transposed=True)  # fmt: skip
        ctx.save_for_backward(x, weight, M_array, K_array, N_array)
        return output

    @staticmethod
    def backward(ctx, output_grad):
        x, weight, M_array, K_array, N_array = ctx.saved_tensors
        output_grad = output_grad.contiguous()
        x_grad = weight_grad = None
        if ctx.needs_input_grad[0]:
            x_grad = grouped_gemm(A=output_grad, B=weight, C=None, M_array=M_array, N_array=K_array, K_array=N_array,
                                  output_shape=x.size(), is_A_transposed=False, is_B_transposed=False)  # fmt: skip
        if ctx.needs_input_grad[1]:
            weight_grad = grouped_gemm(A=output_grad, B=x, C=None, M_array=N_array, N_array=K_array, K_array=M_array,
                                       output_shape=weight.size(), is_A_transposed=True, is_B_transposed=False)  # fmt: skip
        return x_grad, weight_grad, None, None, None


def grouped_gemm_experts(x: torch.Tensor, weight: torch.Tensor, M_array: torch.Tensor, N_array: torch.Tensor,
                         K_array: torch.Tensor) -> torch.Tensor:
    """y[rows of expert e] = x[rows of expert e] @ weight[e].T with the reference's signature
    (fma/modules/moe/cuda_implementation/__init__.py: grouped_gemm_experts); bf16, differentiable in x and weight."""
    return _GroupedGemmExperts.apply(x, weight, M_array, N_array, K_array)


def _is_swiglu_packed(fn: Callable) -> bool:
    """True if `fn` is this package's swiglu_packed (possibly wrapped in functools.partial with
    backend keywords only), so that it can run inside the GEMM epilogue."""
    if fn is swiglu_packed:
        return True
    if isinstance(fn, functools.partial) and fn.func is swiglu_packed and not fn.args:
        return set(fn.keywords) <= {"kernel_backend_forward", "kernel_backend_backward"}
    return bool(getattr(fn, "_fma_b200_is_swiglu_packed", False))


class Experts(nn.Module):
    def __init__(
        self, num_experts: int, in_features: int, out_features: int, add_bias: bool = True, std: float | None = None
    ) -> None:
        super().__init__()

        self.weight = nn.Parameter(torch.empty(num_experts, out_features, in_features))

        self.bias = None
        if add_bias:
            self.bias = nn.Parameter(torch.empty(num_experts, out_features))

        self.std = std

        self.num_experts = num_experts
        self.in_features = in_features
        self.out_features = out_features

        self.register_buffer("N_array", torch.empty((num_experts,), dtype=torch.uint32))
        self.register_buffer("K_array", torch.empty((num_experts,), dtype=torch.uint32))

        self.reset_parameters()

    def cuda_forward(self, input: torch.Tensor, expert_frequency: torch.Tensor) -> torch.Tensor:
        """The reference's entry point (fma/modules/moe/__init__.py:89-92): `input` holds expert_frequency[e]
        consecutive rows for expert e.  Like the reference it applies no bias."""
        return grouped_gemm_experts(x=input, weight=self.weight, M_array=expert_frequency, N_array=self.N_array,
                                    K_array=self.K_array)  # fmt: skip

    def grouped_forward(self, input: torch.Tensor, maps: K.RowMaps) -> torch.Tensor:
        """Y = X . W[e]^T over the grouped layout (rows of expert e in maps.pad_offsets[e:e+2])."""
        return _ExpertLinear.apply(input, self.weight, self.bias, maps)

    def extra_repr(self):
        return "num_experts={}, in_features={}, out_features={}".format(
            self.num_experts, self.in_features, self.out_features
        )

    @torch.no_grad()
    def reset_parameters(self) -> None:
        nn.init.normal_(self.weight, mean=0, std=self.std)
        if hasattr(self, "bias") and self.bias is not None:
            self.bias.zero_()

        self.N_array.fill_(self.out_features)
        self.K_array.fill_(self.in_features)


class MoE(nn.Module):
    def __init__(
        self,
        num_experts: int,
        num_experts_per_tok: int,
        hidden_size: int,
        intermediate_size: int,
        activation_function: Callable,
        is_glu: bool,
        add_bias: bool,
        std: float,
    ) -> None:
        super().__init__()

        self.num_experts = num_experts
        self.top_k = num_experts_per_tok

        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.is_glu = is_glu

        self.gate = nn.Linear(in_features=self.hidden_size, out_features=num_experts, bias=False)

        self.c_fc = Experts(
            num_experts=num_experts,
            in_features=self.hidden_size,
            out_features=2 * self.intermediate_size if is_glu else self.intermediate_size,
            add_bias=add_bias,
            std=std,
        )

        # Set to True to make every forward also produce the router statistics of a load-balancing loss
        # (see load_balancing_loss); they come out of the routing kernels at no extra pass over the logits.
        self.collect_router_stats = False

        self.act = activation_function
        # decided once, outside any compiled region: can the activation run inside the GEMM epilogue?
        self._act_is_swiglu_packed = _is_swiglu_packed(activation_function)

        self.c_proj = Experts(
            num_experts=num_experts,
            in_features=self.intermediate_size,
            out_features=self.hidden_size,
            add_bias=add_bias,
            std=std,
        )

    def forward(
        self, hidden_states: torch.Tensor, kernel_backend: KernelBackend = KernelBackend.triton
    ) -> tuple[torch.Tensor, torch.Tensor]:
        """Returns (output with the shape of `hidden_states`, router_logits [T, num_experts]).
        `kernel_backend` is accepted for compatibility; every value runs the same CUDA kernels."""
        if not isinstance(kernel_backend, KernelBackend):
            raise ValueError(f"unexpected kernel_backend ({kernel_backend})")
        _native.require_cuda(hidden_states)
        original_shape = hidden_states.shape
        hidden_states = hidden_states.reshape(-1, self.hidden_size)
        if torch.compiler.is_compiling():
            return self._forward_traced(hidden_states, original_shape)

        with torch.cuda.device(hidden_states.device):
            router_logits, router_weights, selected_experts = self._compute_routing_weights(hidden_states)
            hidden_states = self._compute_experts(hidden_states, router_weights, selected_experts)

        return hidden_states.view(original_shape), router_logits

    def _forward_traced(self, hidden_states: torch.Tensor, original_shape) -> tuple[torch.Tensor, torch.Tensor]:
        """The same layer through torch.library custom ops (`_moe_ops`), for torch.compile(fullgraph=True):
        no Python object crosses an op boundary and nothing is stored on the module."""
        from . import _moe_ops

        router_logits = self.gate(hidden_states)
        router_weights, selected_experts, route_workspace = _moe_ops.moe_route(router_logits, self.top_k)
        if self.is_glu and self._act_is_swiglu_packed and self.c_fc.bias is None and self.c_proj.bias is None:
            outputs = _moe_ops.moe_swiglu_experts(hidden_states, router_weights, selected_experts, route_workspace,
                                                  self.c_fc.weight, self.c_proj.weight, K.ROW_ALIGN)  # fmt: skip
            return outputs[0].view(original_shape), router_logits
        # any other activation / experts with bias: the activation is traced as ordinary code between two
        # expert-linear ops (the reference compiles its MoE with GLU and GELU activations,
        # tests/modules/moe_test.py:97-98)
        _count, pad_offsets, row_of_slot, slot_of_row, mtile_expert = _moe_ops.moe_sort_maps(
            selected_experts, route_workspace, self.num_experts, K.ROW_ALIGN)  # fmt: skip
        maps = (pad_offsets, row_of_slot, slot_of_row, mtile_expert)
        grouped = _moe_ops.moe_scatter_rows(hidden_states, *maps, self.top_k, K.ROW_ALIGN)
        grouped = _moe_ops.moe_expert_linear(grouped, self.c_fc.weight, self.c_fc.bias, *maps, self.top_k, K.ROW_ALIGN)
        grouped = self.act(grouped)
        grouped = _moe_ops.moe_expert_linear(grouped, self.c_proj.weight, self.c_proj.bias, *maps, self.top_k, K.ROW_ALIGN)
        y = _moe_ops.moe_combine_rows(grouped, router_weights, *maps, K.ROW_ALIGN)
        return y.view(original_shape), router_logits

    def _compute_routing_weights(self, hidden_states: torch.Tensor):
        router_logits = self.gate(hidden_states)
        router_weights, selected_experts, workspace = _RouterTopK.apply(
            router_logits, self.top_k, bool(getattr(self, "collect_router_stats", False)))  # fmt: skip
        # by-products of the routing kernel for the sort of exactly these ids (see _sort_selected)
        self._routed = (selected_experts, workspace, router_logits)
        return router_logits, router_weights, selected_experts

    def _sort_selected(self, selected_experts: torch.Tensor) -> K.RowMaps:
        """Row maps for `selected_experts`; reuses what the routing kernel prepared when these are the ids
        it produced in this forward."""
        routed = getattr(self, "_routed", None)
        self._routed = None
        self.last_router_stats = None
        with torch.no_grad():
            if routed is None or routed[0] is not selected_experts:
                return K.moe_sort(selected_experts, self.num_experts)
            want = bool(getattr(self, "collect_router_stats", False))
            maps = K.moe_sort(selected_experts, self.num_experts, routed_workspace=routed[1], want_mean_prob=want)
        if maps.router_mean_prob is not None:
            logits = routed[2]
            mean_prob = maps.router_mean_prob
            if logits.requires_grad and torch.is_grad_enabled():
                mean_prob = _RouterMeanProb.apply(logits, mean_prob)
            self.last_router_stats = {"tokens_per_expert": maps.expert_count, "mean_router_prob": mean_prob,
                                      "num_tokens": selected_experts.size(0)}  # fmt: skip
        return maps

    def load_balancing_loss(self) -> torch.Tensor:
        """num_experts * sum_e f_e * P_e for the most recent forward (needs collect_router_stats = True):
        f_e = tokens routed to expert e / tokens, P_e = mean over tokens of softmax(router_logits)[t, e].
        This is the auxiliary loss a caller of the reference builds from the returned router_logits
        (fma/modules/moe/__init__.py:189); here both factors come from the routing kernels.  Differentiable
        with respect to the router logits through P_e (f_e is a count)."""
        stats = getattr(self, "last_router_stats", None)
        if stats is None:
            raise RuntimeError("set collect_router_stats = True before the forward pass")
        f = stats["tokens_per_expert"].to(torch.float32) / float(max(stats["num_tokens"], 1))
        return self.num_experts * torch.sum(f * stats["mean_router_prob"])

    def _compute_experts(
        self, hidden_states: torch.Tensor, router_weights: torch.Tensor, selected_experts: torch.Tensor
    ) -> torch.Tensor:
        T = hidden_states.size(0)
        maps = self._sort_selected(selected_experts)
        self.last_row_maps = maps  # expert_count etc. for callers that log load balance

        fused = (
            self.is_glu and _is_swiglu_packed(self.act) and self.c_fc.bias is None and self.c_proj.bias is None
        )
        if fused:
            return _FusedSwigluExperts.apply(hidden_states, router_weights, self.c_fc.weight, self.c_proj.weight, maps)

        grouped = _Scatter.apply(hidden_states, maps)
        grouped = self.c_fc.grouped_forward(grouped, maps)
        grouped = self.act(grouped)
        grouped = self.c_proj.grouped_forward(grouped, maps)
        return _Combine.apply(grouped, router_weights, maps, T)
