"""The vLLM config and MoE method of this backend, at module level so vLLM can pickle the config into its engine-core process
(the reason the reference keeps them in their own module, sm120fp4/vllm_classes.py:1-7).

Same surface as the reference: `ModelOptNvFp4FusedMoESM120` (alias `SM120Fp4MoEMethod`) with `fits`,
`process_weights_after_loading`, `apply`; `SM120Fp4Config.get_quant_method`. Differences, all widening: any hidden size
that is a multiple of 128 and intermediate size that is a multiple of 64 fit (the reference: 2048 x {768, 1024},
vllm_classes.py:41-45); batches above 16 tokens run the layer's own W4A4 kernels when the checkpoint carries activation
input scales; and expert parallelism is taken (the reference declines it, vllm_classes.py:46-47,95-96). With an expert map
on the layer, `apply` runs this rank's shard with the slots of other ranks' experts masked and returns the PARTIAL rows the
engine then reduces over the expert-parallel group (vLLM hands every rank of the group the same tokens and reduces the
outputs). SM120FP4_EP=own is for an engine that hands each rank its own tokens and expects complete rows: the call then goes
through `ep.ExpertParallelMoE` (dispatch -> local shard -> combine over the expert-parallel group).
"""
from __future__ import annotations

import torch

try:  # vLLM moved RoutedExperts between releases: try the reference's import path first, then the package-level one
    from vllm.model_executor.layers.fused_moe.routed_experts import RoutedExperts
except ImportError:  # pragma: no cover - depends on the installed vLLM
    from vllm.model_executor.layers.fused_moe import RoutedExperts
from vllm.model_executor.layers.fused_moe.activation import MoEActivation
from vllm.model_executor.layers.fused_moe.fused_moe_method_base import FusedMoEMethodBase
from vllm.model_executor.layers.quantization.modelopt import ModelOptNvFp4Config, ModelOptNvFp4FusedMoE

import os

from ._lib import B200MoEError
from .vllm_backend import Weights, _log, map_expert_ids, prefill_explicit, prefill_mode, shared_workspace, weights_from_vllm_layout

RELEASE_ENV = "SM120FP4_RELEASE_CHECKPOINT"   # "1": free the checkpoint-layout weights after the load-time re-layout
EP_ENV = "SM120FP4_EP"     # "own": this backend does the expert-parallel exchange itself (default: the engine reduces partial rows)


class ModelOptNvFp4FusedMoESM120(ModelOptNvFp4FusedMoE):
    """vLLM's NVFP4 MoE method with this package's layer in place of the Marlin repack and kernel. The class name keeps
    "ModelOpt" in it: vLLM's weight loader branches on the method's class name (sm120fp4/vllm_classes.py:22-26)."""

    def __init__(self, quant_config, moe_config) -> None:
        FusedMoEMethodBase.__init__(self, moe_config)   # not the parent's: it would select a vLLM backend that never runs
        self.quant_config = quant_config
        self.use_a16 = True
        self.use_global_sf = False
        self.nvfp4_backend, self.experts_cls = None, None
        self.weights: Weights | None = None
        self._ep = None

    @staticmethod
    def fits(moe_config) -> tuple[bool, str]:
        """Whether the layer described by a FusedMoEConfig can run on the kernels; (False, reason) otherwise."""
        if not getattr(moe_config, "is_act_and_mul", False) or moe_config.activation != MoEActivation.SILU:
            return False, f"activation {moe_config.activation!r} is not gated SiLU"
        if moe_config.hidden_dim % 128:
            return False, f"hidden size {moe_config.hidden_dim} (kernels take multiples of 128)"
        if moe_config.intermediate_size_per_partition % 64:
            return False, f"intermediate size {moe_config.intermediate_size_per_partition} (kernels take multiples of 64)"
        if moe_config.in_dtype != torch.bfloat16:
            return False, f"activations {moe_config.in_dtype} (kernels take bf16)"
        n_local = getattr(moe_config, "num_local_experts", None) or getattr(moe_config, "num_experts", 0) or 0
        if n_local > 256:
            return False, f"{n_local} experts on one rank (kernels take at most 256)"
        top_k = getattr(moe_config, "experts_per_token", None) or getattr(moe_config, "top_k", 0) or 0
        if top_k > 16:
            return False, f"top_k {top_k} (kernels take at most 16)"
        return True, ""

    @property
    def is_monolithic(self) -> bool:
        return False

    @property
    def supports_eplb(self) -> bool:
        return False

    def get_fused_moe_quant_config(self, layer):
        return None

    def process_weights_after_loading(self, layer) -> None:
        self.weights = weights_from_vllm_layout(layer.w13_weight.data, layer.w13_weight_scale.data, layer.w13_weight_scale_2.data,
                                                layer.w2_weight.data, layer.w2_weight_scale.data, layer.w2_weight_scale_2.data,
                                                int(layer.top_k))
        w = self.weights
        if prefill_mode() != "slices":
            if getattr(layer, "w13_input_scale", None) is None or getattr(layer, "w2_input_scale", None) is None:
                if prefill_explicit():
                    raise ValueError("SM120FP4_PREFILL=cutlass needs the checkpoint's w13_input_scale and w2_input_scale")
                _log("no activation input scales in this checkpoint: batches above 16 tokens run as slices")
            else:   # one workspace for all layers of the model: it only holds transient data of one layer call
                w.enable_prefill(layer.w13_input_scale.data, layer.w2_input_scale.data,
                                 workspace=shared_workspace("prefill", w.device, w.prefill_workspace_bytes(8192)))
        try:        # 33 .. 256 tokens in one W4A16 call instead of slices of 16; shapes it does not take keep the slices
            w.enable_mid(256, workspace=shared_workspace("mid", w.device, w.mid_workspace_bytes(256)))
        except B200MoEError:
            pass
        if os.environ.get(RELEASE_ENV, "") == "1":
            # every path of this method reads the kernel-native tile records only: drop the checkpoint-layout copy (half of
            # the layer's memory) and leave empty parameters behind for code that only looks the names up
            w.release_checkpoint_layout()
            empty = torch.empty(0, dtype=torch.uint8, device=w.device)
            params = (("w13_weight", empty), ("w13_weight_scale", empty.view(torch.float8_e4m3fn)), ("w13_weight_scale_2", w.alpha1),
                      ("w2_weight", empty), ("w2_weight_scale", empty.view(torch.float8_e4m3fn)), ("w2_weight_scale_2", w.alpha2))
        else:
            params = (("w13_weight", w.q1), ("w13_weight_scale", w.s1_linear.view(torch.float8_e4m3fn)), ("w13_weight_scale_2", w.alpha1),
                      ("w2_weight", w.q2), ("w2_weight_scale", w.s2_linear.view(torch.float8_e4m3fn)), ("w2_weight_scale_2", w.alpha2))
        for name, t in params:
            layer.register_parameter(name, torch.nn.Parameter(t, requires_grad=False))
        for name in ("w13_input_scale", "w2_input_scale"):
            if hasattr(layer, name):
                layer.register_parameter(name, None)

    def apply(self, layer, x, topk_weights, topk_ids, shared_experts, shared_experts_input):
        assert self.weights is not None, "process_weights_after_loading has not run"
        if shared_experts is not None:
            raise NotImplementedError("shared experts are not run by this backend")
        if getattr(layer, "apply_router_weight_on_input", False):
            raise NotImplementedError("apply_router_weight_on_input")
        emap = getattr(layer, "expert_map", None)
        if emap is None:
            return self.weights.forward(x, topk_ids, topk_weights)
        if os.environ.get(EP_ENV, "") == "own":
            return self._expert_parallel(layer).forward(x, topk_ids, topk_weights)
        ids, wts = map_expert_ids(topk_ids, topk_weights, emap)   # partial rows: the engine reduces them over the EP group
        return self.weights.forward(x, ids, wts)

    def _expert_parallel(self, layer):
        """`ep.ExpertParallelMoE` over the engine's expert-parallel group (even contiguous shards, as vLLM's linear expert
        placement makes them)."""
        if getattr(self, "_ep", None) is None:
            from .ep import ExpertParallelMoE
            group = None
            try:
                from vllm.distributed import get_ep_group
                group = get_ep_group().device_group
            except Exception:  # noqa: BLE001 - outside an engine: the default process group
                pass
            emap = layer.expert_map
            n_global = int(emap.numel())
            ep = ExpertParallelMoE(self.weights.forward, n_global, self.weights.k, group=group)
            lo, hi = ep.lo, ep.hi
            own = torch.nonzero(emap >= 0).flatten().cpu()
            if own.numel() != hi - lo or int(own[0]) != lo or int(own[-1]) != hi - 1 or not torch.equal(emap[lo:hi].cpu().long(), torch.arange(hi - lo)):
                raise NotImplementedError("expert map that is not an even contiguous split (round-robin or redundant-expert placement)")
            self._ep = ep
        return self._ep


class SM120Fp4Config(ModelOptNvFp4Config):
    """vLLM's ModelOpt NVFP4 config, routing the routed-experts layers the kernels fit to the method above."""

    def get_quant_method(self, layer, prefix: str):
        if isinstance(layer, RoutedExperts) and not self.is_layer_excluded(prefix):
            ok, why = ModelOptNvFp4FusedMoESM120.fits(layer.moe_config)
            if ok:
                return ModelOptNvFp4FusedMoESM120(quant_config=self, moe_config=layer.moe_config)
            _log(f"layer {prefix} stays on vLLM's path: {why}")
        return super().get_quant_method(layer, prefix)


SM120Fp4MoEMethod = ModelOptNvFp4FusedMoESM120  # the short name the reference's tests and docs use
